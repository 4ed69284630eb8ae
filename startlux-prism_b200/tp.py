"""Tensor-parallel sharded linears: the reference's tp.py sharding rules and the two exchange steps of a row-parallel
projection, one process per GPU over torch.distributed (NCCL over NVLink; gloo on CPU for tests of the host logic).

    shard_config(cfg, n), shard_index(cfg, n, r)     which rows / columns a rank holds          (tp.py:83-125)
    Group(rank, world, ...)                          process group: sum_, max_                   (tp.py:333-357, :435-439)
                                                     setup, symmetric, begin, sync, words: the in-kernel exchanges of
                                                     short passes (tp.py:358-432)
                                                     scatter_sum_, gather_: the two halves of an all-reduce, for passes
                                                     that keep the residual stream split by rows between them
    PeerBuffer(g, nbytes)                            device memory the other ranks' kernels store into  (tp.py:381-403)
    quantize_rows(g, fn, rows, amax, *args)          global row maximum before quantizing        (tp.py:143-156)
    out_proj(g, a, a_s, w, w_s, flat, rows, n_rows)  int32 partial sums -> all-reduce -> Deferred (tp.py:159-180)

Exactness (tp.py:24-31): weights are quantized whole and then sliced; a column-parallel output is a whole-K dot
product; a row-parallel projection all-reduces int32 partial sums (exact in any order, so NCCL's algorithm choice
cannot change a bit) and the residual's next reader scales the total once; a row-parallel input's per-token scale is
the max over all ranks (exact).  Outputs are therefore bit-identical at every GPU count, 8 included: unlike the
reference's in-kernel protocols (4 ranks at most) nothing here depends on the group size.

Short passes (a few rows: decode) exchange inside the kernels, as the reference does (tp.py:129-180): up to
`fast_rows` rows the producers exchange row maxima as 64-bit words (quant mode 3), up to `pull_rows` rows the kernel that
folds a row-parallel projection reads every rank's int32 slots itself after a flag handshake (quant.Sync) - no
collective call between the kernels.  The buffers are peer-mapped device memory (PeerBuffer); every device-side wait
is bounded.  Many-row passes use w8a8.gemm_scatter (linear_stack) or NCCL.

Not built (engine orchestration, outside the linear-layer path): the shared-memory channel to follower processes and
the mirrored-object RPC.
"""
from __future__ import annotations

import dataclasses
import os

import torch
import torch.distributed as dist

SPLIT_ROWS = 512      # output projections split K into several int32 slots only up to this many rows
MAX_SPLIT = 4
FAST_ROWS = int(os.environ.get("PRISM_B200_TP_FAST_ROWS", "255"))   # row maxima exchanged inside the producers up to here
PULL_ROWS = {2: 128, 4: 64, 8: 64}    # int32 sums read by their consumer up to here, per group size (PRISM_B200_TP_PULL_ROWS)
CHANNELS = 1024                       # flag handshakes per pass at most


def shard_config(cfg, n):
    """What one of n ranks holds, as a config: 1 / n of the attention heads, kv heads, linear-attention key and value
    heads and FFN columns.  `v_heads_full` remembers the whole model's value-head count (the gated norm keeps the whole
    model's head block) and `tp` the group size.  Raises when n does not divide one of them."""
    split = {"n_head": "attention heads", "n_kv_head": "kv heads", "k_heads": "linear-attention key heads", "ffn": "FFN width"}
    for field, what in split.items():
        whole = getattr(cfg, field)
        if whole % n:
            raise ValueError(f"--tp {n} does not divide the model's {whole} {what}")
    if cfg.v_heads % cfg.k_heads:
        raise ValueError("value heads must be a multiple of key heads")
    shard = dataclasses.replace(cfg, v_heads=cfg.v_heads // n, **{f: getattr(cfg, f) // n for f in split})
    shard.v_heads_full, shard.tp = cfg.v_heads, n
    return shard


def shard_index(cfg, n, r):
    """Rank r's rows of the column-parallel projections and columns of the row-parallel ones, as int64 indices over the
    whole model's tensors, in the order the rank's kernels read them:
      qkv   attention: the q|gate rows of its heads (2 * head_dim rows per head), then its kv heads' k rows, then v rows
      o     its heads' input columns
      inp   linear attention: q and k channels of its key heads, the v channels of the value heads that read them (value
            head m * k_heads + k reads key head k), their z rows, then their beta and alpha rows
      conv  its conv channels;  vh its value heads;  out their input columns
      gu    its gate columns then its up columns;  down their input columns."""
    H, KV, HD = cfg.n_head, cfg.n_kv_head, cfg.head_dim
    HK, HV, D, FF = cfg.k_heads, cfg.v_heads, cfg.gdn_dim, cfg.ffn
    Hl, KVl, HKl, FFl = H // n, KV // n, HK // n, FF // n
    span = lambda a, b: torch.arange(a, b, dtype=torch.int64)                        # noqa: E731
    channels = lambda heads: (heads[:, None] * D + span(0, D)[None, :]).reshape(-1)  # noqa: E731
    kh = span(r * HKl, (r + 1) * HKl)
    vh = torch.cat([m * HK + kh for m in range(HV // HK)])
    q_rows, conv_dim = H * 2 * HD, 2 * HK * D + HV * D
    conv = torch.cat([channels(kh), HK * D + channels(kh), 2 * HK * D + channels(vh)])
    return dict(
        qkv=torch.cat([span(r * Hl * 2 * HD, (r + 1) * Hl * 2 * HD), q_rows + span(r * KVl * HD, (r + 1) * KVl * HD),
                       q_rows + KV * HD + span(r * KVl * HD, (r + 1) * KVl * HD)]),
        o=span(r * Hl * HD, (r + 1) * Hl * HD),
        inp=torch.cat([conv, conv_dim + channels(vh), conv_dim + HV * D + vh, conv_dim + HV * D + HV + vh]),
        conv=conv, vh=vh, out=channels(vh),
        gu=torch.cat([span(r * FFl, (r + 1) * FFl), FF + span(r * FFl, (r + 1) * FFl)]),
        down=span(r * FFl, (r + 1) * FFl))


def linear_shards(q_cols, kv_cols, ffn, n, r):
    """Index sets of the plain decoder-layer linear set (q | k | v fused, o, gate | up fused, down) for rank r of n:
    qkv rows (its q columns, then its k, then its v columns; a rank holds 1 / n of each, so with n above the kv head
    count a kv head's rows are split, which is exact: output rows are independent), o input columns (its q columns),
    gu rows, down input columns."""
    span = lambda a, b: torch.arange(a, b, dtype=torch.int64)                        # noqa: E731
    for what, v in (("q columns", q_cols), ("kv columns", kv_cols), ("FFN width", ffn)):
        if v % n:
            raise ValueError(f"{n} ranks do not divide the {v} {what}")
    ql, kl, fl = q_cols // n, kv_cols // n, ffn // n
    return dict(qkv=torch.cat([span(r * ql, (r + 1) * ql), q_cols + span(r * kl, (r + 1) * kl),
                               q_cols + kv_cols + span(r * kl, (r + 1) * kl)]),
                o=span(r * ql, (r + 1) * ql),
                gu=torch.cat([span(r * fl, (r + 1) * fl), ffn + span(r * fl, (r + 1) * fl)]),
                down=span(r * fl, (r + 1) * fl))


class Group:
    """One rank of a tensor-parallel group.  backend "nccl": its GPU is cuda:local_rank, collectives run on the current
    CUDA stream (capturable); backend "gloo": CPU tensors (tests).  Joins an already initialised default process group
    (torchrun) or initialises one at 127.0.0.1:port."""

    def __init__(self, rank, world, port=None, backend="nccl", local_rank=None, timeout_s=600):
        self.rank, self.world, self.backend = rank, world, backend
        if backend == "nccl":
            self.device = torch.device("cuda", rank if local_rank is None else local_rank)
            torch.cuda.set_device(self.device)
        else:
            self.device = torch.device("cpu")
        if not dist.is_initialized():
            import datetime
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            if port is not None:
                os.environ["MASTER_PORT"] = str(port)
            kw = dict(device_id=self.device) if backend == "nccl" else {}
            dist.init_process_group(backend, rank=rank, world_size=world,
                                    timeout=datetime.timedelta(seconds=timeout_s), **kw)
        self.pg = dist.group.WORLD
        self._coalesce = None                    # gather2_: does this torch build coalesce all-gathers? (None: not tried)
        # in-kernel exchanges (setup): every rank's buffers as mapped here, and the per-pass bookkeeping
        self.xs = self.ws = self.fs = None
        self.fast = self.pull = False
        self.fast_rows = self.pull_rows = self.parity = self.hidden = self.word_steps = 0
        self.nsum = self.step = self.mstep = 0
        self._peers = []

    # ------------------------------------------------------------ in-kernel exchanges (quant.Sync)
    def setup(self, hidden, words, fast_rows=None, pull_rows=None):
        """Allocates, on every rank, the peer-mapped buffers of the in-kernel exchanges (the reference's Group.setup,
        tp.py:358-379): the flag words of the handshakes (CHANNELS x ranks), two parities of int32 slots for the output
        projections of passes up to pull_rows rows (MAX_SPLIT slots of `hidden` sums each), the row maxima's words
        (`words` exchanges per pass at most, fast_rows rows, one word per rank) and this rank's pass counter.  A
        collective: every rank calls it at the same point, once.  Without peer memory (gloo, or CUDA IPC refused) the
        group keeps exchanging through collectives."""
        if self.xs is not None:
            if hidden != self.hidden:
                raise ValueError("one tensor-parallel group serves one model")
            return
        if self.world == 1 or self.backend != "nccl":
            return
        fast_rows = FAST_ROWS if fast_rows is None else fast_rows
        if pull_rows is None:
            env = os.environ.get("PRISM_B200_TP_PULL_ROWS")
            pull_rows = int(env) if env else PULL_ROWS.get(self.world, 1)
        fast_rows = max(0, min(fast_rows, 255))              # the exchange lives in the one-CTA-per-row producers
        self.hidden, self.fast_rows, self.pull_rows = hidden, fast_rows, max(0, min(pull_rows, fast_rows))
        self.word_steps = words
        if fast_rows <= 0:
            return
        self.parity = MAX_SPLIT * max(self.pull_rows, 1) * hidden
        fs = self.symmetric(CHANNELS * self.world, torch.int64)
        xs = self.symmetric(2 * self.parity, torch.int32)
        ws = self.symmetric(words * fast_rows * self.world, torch.int64)
        if fs is None or xs is None or ws is None:
            self.fast_rows = self.pull_rows = 0
            return
        self.fs, self.xs, self.ws = fs, xs, ws
        self.epoch = torch.zeros(1, dtype=torch.int64, device=self.device)

    def setup_many(self, rows, words):
        """Word buffers for the row-maximum exchanges of passes with MANY rows (linear_stack's row-split pass): `words`
        exchanges per pass of `rows` rows, one 64-bit word per row and rank, peer-mapped like setup()'s.  The producers
        then quantize a row-parallel projection's input in ONE launch (mode 3: the row stays in registers while the
        other ranks' maxima arrive) instead of a maxima pass, a max-all-reduce and a quantizing pass.  Needs the flag
        words of setup() (their pass counter tags the words).  A collective; False when peer memory is unavailable."""
        if self.world == 1 or self.backend != "nccl" or self.fs is None:
            return False
        wm = self.symmetric(words * rows * self.world, torch.int64)
        if wm is None:
            return False
        self.wm, self.wm_rows, self.wm_steps = wm, rows, words
        return True

    def words_many(self):
        """The next many-rows row-maximum exchange's quant.Sync (begin_handshakes started the pass)."""
        from . import quant as KQ
        if self.mstep >= self.wm_steps:
            raise RuntimeError(f"more than {self.wm_steps} row-maximum exchanges in one pass")
        self.mstep += 1
        return KQ.Sync(self.epoch, tuple(self.wm), (self.mstep - 1) * self.wm_rows, (), self.rank, self.world)

    def symmetric(self, n, dtype):
        """n zeroed elements on every rank, each rank's buffer mapped on every other (CUDA IPC over NVLink): returns
        the ranks' buffers as tensors on this device, in rank order (this rank's own at self.rank), or None when peer
        memory is unavailable.  The peer tensors are views of another GPU's memory: pass them to this package's
        kernels only.  A collective."""
        nbytes = n * torch.empty(0, dtype=dtype).element_size()
        peer = PeerBuffer(self, nbytes)
        if not peer.ok:
            return None
        self._peers.append(peer)
        return [torch.as_tensor(_Raw(p, nbytes), device=self.device).view(dtype) for p in peer.ptrs]

    def begin(self, rows):
        """At the start of a pass, on every rank alike (it is recorded in the pass's graph): up to fast_rows rows the
        producers exchange the maxima themselves - a new pass number for their words and the flags - and up to
        pull_rows rows the consumers read the sums (tp.py:405-416)."""
        from . import quant as KQ
        assert self.nsum % 2 == 0, "a pass's fused sums must alternate buffers evenly"
        self.fast = self.xs is not None and 0 < rows <= self.fast_rows
        self.pull = self.fast and rows <= self.pull_rows
        self.nsum = self.step = self.mstep = 0
        if self.fast:
            KQ.bump(self.epoch)

    def sync(self, buffers):
        """The next flag handshake's quant.Sync over `buffers` (every rank's slots, as mapped here)."""
        from . import quant as KQ
        if self.step >= CHANNELS:
            raise RuntimeError(f"more than {CHANNELS} fused sums in one pass")
        self.step += 1
        return KQ.Sync(self.epoch, tuple(self.fs), self.step - 1,
                       tuple(b for r, b in enumerate(buffers) if r != self.rank), self.rank, self.world)

    def begin_handshakes(self):
        """At the start of a many-rows pass whose folds use flag handshakes instead of barrier collectives
        (linear_stack's row-split pass): a new pass number, the channels counted from zero.  False when the group has
        no peer-mapped flags (then the caller keeps its collectives)."""
        from . import quant as KQ
        if self.fs is None:
            return False
        self.step = self.mstep = 0
        KQ.bump(self.epoch)
        return True

    def handshake(self):
        """The next flag handshake alone (no slots to pull): a quant.Sync with no `others`."""
        return self.sync(())

    def words(self):
        """The next row-maximum exchange's quant.Sync (mode 3): every rank's word buffer and the step's first word row."""
        from . import quant as KQ
        if self.mstep >= self.word_steps:
            raise RuntimeError(f"more than {self.word_steps} row-maximum exchanges in one pass")
        self.mstep += 1
        return KQ.Sync(self.epoch, tuple(self.ws), (self.mstep - 1) * self.fast_rows, (), self.rank, self.world)

    # ------------------------------------------------------------ collectives (on the current stream; capturable)
    def sum_(self, x):
        if self.world > 1:
            dist.all_reduce(x, op=dist.ReduceOp.SUM, group=self.pg)

    def max_(self, x):
        if self.world > 1:
            dist.all_reduce(x, op=dist.ReduceOp.MAX, group=self.pg)

    def scatter_sum_(self, own, x):
        """own [rows / world, ...] = this rank's row block of the sum of x [rows, ...] over the ranks (reduce-scatter:
        half an all-reduce's traffic).  gloo has no reduce-scatter: all-reduce a copy and slice."""
        if self.world == 1:
            own.copy_(x)
        elif self.backend == "nccl":
            dist.reduce_scatter_tensor(own, x, op=dist.ReduceOp.SUM, group=self.pg)
        else:
            t = x.clone()
            dist.all_reduce(t, op=dist.ReduceOp.SUM, group=self.pg)
            rows = x.shape[0] // self.world
            own.copy_(t[self.rank * rows:(self.rank + 1) * rows])

    def gather2_(self, full1, own1, full2, own2):
        """Two gathers in one NCCL launch (a row block's int8 values and its scales travel together): the group call
        of the two all-gathers; elsewhere, or where this torch build has no coalescing of all-gathers, two calls."""
        if self.world > 1 and self.backend == "nccl" and self._coalesce is not False:
            try:
                from torch.distributed.distributed_c10d import _coalescing_manager
                with _coalescing_manager(group=self.pg, device=own1.device, async_ops=False):
                    dist.all_gather_into_tensor(full1, own1, group=self.pg)
                    dist.all_gather_into_tensor(full2, own2, group=self.pg)
                self._coalesce = True
                return
            except Exception:                                      # noqa: BLE001
                if self._coalesce:                                 # it worked before: a real failure
                    raise
                self._coalesce = False
        self.gather_(full1, own1)
        self.gather_(full2, own2)

    def gather_(self, full, own):
        """full [rows, ...] = the ranks' row blocks own [rows / world, ...] in rank order; `own` may be full's own
        block (in place)."""
        if self.world == 1:
            if own.data_ptr() != full.data_ptr():
                full.copy_(own)
        elif self.backend == "nccl":
            dist.all_gather_into_tensor(full, own, group=self.pg)
        else:
            rows = full.shape[0] // self.world
            parts = [torch.empty_like(own) for _ in range(self.world)]
            dist.all_gather(parts, own.clone(), group=self.pg)
            for r, t in enumerate(parts):
                full[r * rows:(r + 1) * rows].copy_(t)

    def barrier(self):
        if self.world > 1:
            dist.barrier(group=self.pg)

    def close(self):
        for peer in self._peers:
            peer.close()
        self._peers = []
        self.xs = self.ws = self.fs = None
        if dist.is_initialized():
            dist.destroy_process_group()


class _Raw:
    """A device address as a CUDA-array-interface object (torch.as_tensor wraps it without a copy)."""

    def __init__(self, ptr, nbytes):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


class PeerBuffer:
    """nbytes of this rank's device memory (zeroed) that every rank of the group can store into from its own kernels:
    ptrs[r] is rank r's buffer as an address valid on this rank's GPU (peer access over NVLink), ptrs[rank] the own
    one.  The role of the reference's symmetric-memory buffers (tp.py:381-403), through CUDA IPC handles exchanged over
    the process group.  Collective: every rank of the group constructs it at the same point."""

    def __init__(self, g, nbytes):
        import ctypes
        from . import _lib
        L = _lib.lib()
        self.g, self.nbytes, self.ptrs, self._open = g, nbytes, [], []
        own, handle = ctypes.c_void_p(), ctypes.create_string_buffer(64)
        _lib.check(L.pb_peer_alloc(nbytes, ctypes.byref(own), handle), f"peer buffer of {nbytes} bytes")
        self.ptr = own.value
        handles = [None] * g.world
        dist.all_gather_object(handles, bytes(handle.raw), group=g.pg)
        err = None
        for r, h in enumerate(handles):
            if r == g.rank:
                self.ptrs.append(self.ptr)
                continue
            p = ctypes.c_void_p()
            rc = L.pb_peer_open(ctypes.create_string_buffer(h, 64), ctypes.byref(p))
            if rc:
                err = err or _lib.PrismError(rc, f"mapping rank {r}'s buffer")
                self.ptrs.append(None)
            else:
                self.ptrs.append(p.value)
                self._open.append(p.value)
        # every rank must agree that the mapping worked before any kernel uses it
        ok = torch.tensor([0 if err else 1], dtype=torch.int32, device=g.device)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=g.pg)
        self.ok = bool(ok.item())
        self.error = err
        if not self.ok:
            self.close()

    def tensor(self, dtype, shape):
        """The own buffer as a tensor."""
        return torch.as_tensor(_Raw(self.ptr, self.nbytes), device=self.g.device).view(dtype).view(*shape)

    def close(self):
        from . import _lib
        L = _lib.lib()
        if self.ptr is None:
            return
        torch.cuda.synchronize(self.g.device)
        for p in self._open:
            L.pb_peer_close(p)
        self._open = []
        if dist.is_initialized():
            self.g.barrier()                       # nobody still maps this rank's memory
        L.pb_peer_free(self.ptr)
        self.ptr = None


def quantize_rows(g, fn, rows, amax, *args):
    """The input of a row-parallel projection, quantized by fn (quant.rows_q8 / swiglu_q8 / gated_norm_q8) with the
    row's maximum over all ranks.  On a short pass (Group.begin decided: g.fast) in one launch, the maxima exchanged
    inside the kernel (mode 3); otherwise this rank's maxima stored (mode 1), max-all-reduced in `amax`, then the rows
    quantized (mode 2).  One rank: the plain kernel."""
    if g is None or g.world == 1:
        fn(*args)
        return
    if g.fast:
        fn(*args, mode=3, sync=g.words())                # one launch: the maxima travel as words between the kernels
        return
    fn(*args, mode=1, amax=amax)
    g.max_(amax[:rows])
    fn(*args, mode=2, amax=amax)


def out_proj(g, a, a_s, w, w_s, flat, rows, n_rows, pdl=0):
    """A row-parallel output projection: this rank's int32 partial sums (w8a8.gemm_i32) into `flat` (int32 room for
    parts_elems(rows, N) values), summed over the ranks, returned as the residual add the next quant.fold finishes."""
    from . import w8a8 as KW
    N = w.shape[0]
    S_max = MAX_SPLIT if rows <= SPLIT_ROWS else 1
    if g is not None and g.pull:
        # a short pass: the sums stay in this rank's peer-mapped slots (two parities: the next projection writes the
        # other one while slow ranks may still read this one) and the fold reads every rank's (tp.py:168-174)
        lo = (g.nsum % 2) * g.parity
        g.nsum += 1
        views = [x[lo:lo + S_max * rows * N].view(S_max, rows, N) for x in g.xs]
        S = KW.gemm_i32(a, a_s, w, w_s, views[g.rank], n_rows, max_split=S_max, pdl=pdl)
        return KW.Deferred(S, a_s, w_s, views[g.rank][:S], g.sync([v[:S] for v in views]))
    slots = flat[:S_max * rows * N].view(S_max, rows, N)
    S = KW.gemm_i32(a, a_s, w, w_s, slots, n_rows, max_split=S_max, pdl=pdl)
    if g is not None:
        g.sum_(slots[:S])
    return KW.Deferred(S, a_s, w_s, slots[:S])


def parts_elems(rows, hidden):
    """int32 elements out_proj needs for passes of up to `rows` rows."""
    return max(MAX_SPLIT * min(rows, SPLIT_ROWS), rows) * hidden
