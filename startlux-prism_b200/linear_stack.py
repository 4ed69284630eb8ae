"""The decoder-layer linear set of the 27B-class model as one callable pass: the workload of the benchmark and of the
tensor-parallel identity tests.  Per layer, on an fp32 residual stream h [M, hidden]:

    rows_q8(h)                        -> int8 input of q|k|v                (stand-in for norm_q8: no RMSNorm weight)
    q|k|v  GEMM, column-parallel      -> bf16 [M, 7168 / n]
    mixer stand-in                    -> this rank's q columns of that output (attention itself is not on the path)
    quantize_rows(rows_q8)            -> int8, scale from the row maximum over all ranks
    o      GEMM, row-parallel         -> h += ...   (one rank: fused residual epilogue; more: int32 sums, all-reduce, fold;
                                                     more ranks and many rows: reduce-scatter, the residual stream split
                                                     by rows until the next projection's int8 input is all-gathered)
    rows_q8(h)                        -> int8 input of gate|up
    gate|up GEMM, column-parallel     -> bf16 [M, 34816 / n]
    quantize_rows(swiglu_q8)          -> int8 [M, 17408 / n]
    down   GEMM, row-parallel         -> h += ...

Weights are quantized whole (Q8_0 -> one scale per output row) and sliced afterwards, so every rank count computes the
single-GPU bits.  All buffers are allocated at construction; a pass allocates nothing and can be graph-captured.
"""
import os

import torch

from . import _lib, quant, synth, tp, w8a8

HIDDEN, Q_COLS, KV_COLS, FFN = 5120, 5120, 1024, 17408
OPS_PER_ROW_LAYER = 2 * (HIDDEN * (Q_COLS + 2 * KV_COLS) + Q_COLS * HIDDEN + HIDDEN * 2 * FFN + FFN * HIDDEN)


def make_layer_weights(layer, device, hidden=HIDDEN, q_cols=Q_COLS, kv_cols=KV_COLS, ffn=FFN, seed_cfg=1):
    """Whole-matrix W8A8 weights of one layer: dict name -> (int8 [N, K], fp32 [N]).  N(0, 0.02^2) values drawn on
    `device` from a seeded generator, quantized to Q8_0 (ggml's rule) and requantized to one scale per output row
    (w8a8.weight_from_q8 with gk == K, the engine's mode)."""
    shapes = {"qkv": (q_cols + 2 * kv_cols, hidden), "o": (hidden, q_cols), "gate_up": (2 * ffn, hidden),
              "down": (hidden, ffn)}
    out = {}
    for i, (name, (n, k)) in enumerate(shapes.items()):
        g = torch.Generator(device=device).manual_seed(synth.seed_w(seed_cfg, i) + 97 * layer)
        wq = torch.empty(n, k, dtype=torch.int8, device=device)
        ws = torch.empty(n, dtype=torch.float32, device=device)
        for r0 in range(0, n, 4096):                                   # in row chunks: bounded temporary memory
            w = torch.randn(min(4096, n - r0), k, generator=g, device=device) * 0.02
            q, s = w8a8.weight_from_q8(synth.q8_0(w), k)
            wq[r0:r0 + w.shape[0]], ws[r0:r0 + w.shape[0]] = q, s.view(-1)
        out[name] = (wq, ws)
    return out


def shard_layer(whole, n, r, hidden=HIDDEN, q_cols=Q_COLS, kv_cols=KV_COLS, ffn=FFN):
    """Rank r's slices of a layer's whole weights (rows of the column-parallel ones, input columns of the others)."""
    if n == 1:
        return whole
    idx = tp.linear_shards(q_cols, kv_cols, ffn, n, r)
    dev = whole["qkv"][0].device
    ix = {k: v.to(dev) for k, v in idx.items()}
    return {"qkv": (whole["qkv"][0][ix["qkv"]].contiguous(), whole["qkv"][1][ix["qkv"]].contiguous()),
            "o": (whole["o"][0][:, ix["o"]].contiguous(), whole["o"][1]),
            "gate_up": (whole["gate_up"][0][ix["gu"]].contiguous(), whole["gate_up"][1][ix["gu"]].contiguous()),
            "down": (whole["down"][0][:, ix["down"]].contiguous(), whole["down"][1])}


class LinearStack:
    def __init__(self, layers, M, device, group=None, hidden=HIDDEN, q_cols=Q_COLS, kv_cols=KV_COLS, ffn=FFN):
        """layers: list of per-rank weight dicts (shard_layer).  group: tp.Group or None."""
        self.layers, self.M, self.g = layers, M, group
        n = group.world if group is not None else 1
        self.n, self.hidden = n, hidden
        self.ql, self.kvl, self.fl = q_cols // n, kv_cols // n, ffn // n
        i8, f32, bf = torch.int8, torch.float32, torch.bfloat16
        e = lambda *s, dtype: torch.empty(*s, dtype=dtype, device=device)             # noqa: E731
        self.h = e(M, hidden, dtype=f32)
        self.xq, self.xs = e(M, hidden, dtype=i8), e(M, dtype=f32)
        self.qkv = e(M, self.ql + 2 * self.kvl, dtype=bf)
        self.aq, self.as_ = e(M, self.ql, dtype=i8), e(M, dtype=f32)
        self.gu = e(M, 2 * self.fl, dtype=bf)
        self.dq, self.ds = e(M, self.fl, dtype=i8), e(M, dtype=f32)
        self.amax = e(M, dtype=f32)
        self.parts = torch.zeros(tp.parts_elems(M, hidden), dtype=torch.int32, device=device)
        self.s_max = tp.MAX_SPLIT if M <= tp.SPLIT_ROWS else 1
        self.slots = self.parts[:self.s_max * M * hidden].view(self.s_max, M, hidden)
        self.n_rows = torch.tensor([M], dtype=torch.int32, device=device)
        # few rows on one GPU: every kernel of the pass is launched as a programmatic dependent of the one before it
        # (pb_set_pdl): a GEMM's set-up and first weight reads run while the quantizer before it still works, a
        # quantizer's launch hides behind the GEMM's tail: 0.364 -> 0.332 ms per four-layer pass at 16 rows, 0.428 ->
        # 0.402 at 64, as a replayed graph.  One row runs on the CUDA-core GEMM, which stays a plain launch: off there.
        # PRISM_B200_PDL=0 keeps plain launches, =all chains the one-row pass too (its GEMMs stay plain launches).
        mode = os.environ.get("PRISM_B200_PDL", "1")                  # "0": never; "all": at one row too
        self.pdl = n == 1 and (1 if mode == "all" else 2) <= M <= w8a8.FEW_ROWS and mode != "0"
        # several ranks and many rows: the residual stream stays split by rows between the projections (each rank
        # folds, normalises and quantizes M / n rows), a row-parallel projection's int32 sums are reduce-scattered and
        # the int8 rows of the next projection's input all-gathered: 5/8 of an all-reduce's bytes, and 1 / n of the
        # quantizer work per rank.  PRISM_B200_TP_ALLREDUCE=1 keeps the all-reduce path at every size.
        self.by_rows = (n > 1 and M % n == 0 and M // n >= 64 and os.environ.get("PRISM_B200_TP_ALLREDUCE", "0") != "1")
        if self.by_rows:
            self.Ml = M // n
            self.r0 = group.rank * self.Ml
            self.own = e(1, self.Ml, hidden, dtype=torch.int32)
            self.nr_own = torch.tensor([self.Ml], dtype=torch.int32, device=device)
        # ... and the reduce-scatter itself disappears into the GEMM: every rank's tile kernel stores the rows another
        # rank will fold straight into that rank's memory (peer stores over NVLink, tile by tile), the fold adds the n
        # ranks' blocks.  Needs own-row blocks of whole tiles and CUDA IPC between the ranks; otherwise (or with
        # PRISM_B200_TP_FUSED=0) NCCL's reduce-scatter.
        self.peer = None
        if (self.by_rows and self.Ml % 128 == 0 and n <= 8 and group.backend == "nccl"
                and os.environ.get("PRISM_B200_TP_FUSED", "1") != "0"):
            peer = tp.PeerBuffer(group, n * self.Ml * hidden * 4)
            if peer.ok:
                self.peer = peer
                self.sym = peer.tensor(torch.int32, (n, self.Ml, hidden))
                mine = group.rank * self.Ml * hidden * 4               # this rank's block inside every rank's buffer
                self.blocks = [p + mine for p in peer.ptrs]
                self.token = torch.zeros(1, dtype=torch.int32, device=device)
            elif group.rank == 0:
                print(f"prism_b200: peer memory unavailable ({peer.error}); NCCL reduce-scatter instead", flush=True)
        # few rows on several ranks: the exchanges move into the kernels (row maxima as words between the producers, the
        # int32 sums read by the fold itself); PRISM_B200_TP_FUSED=0 keeps NCCL's all-reduces
        if (n > 1 and group.backend == "nccl" and os.environ.get("PRISM_B200_TP_FUSED", "1") != "0"):
            group.setup(hidden, words=2 * len(layers))
        # the row-split pass with the scatter fused into the GEMM: flag handshakes inside the folds take the place of
        # the barrier collectives (PRISM_B200_TP_FLAGS=0 keeps the one-element all-reduce)
        self.flags = (self.peer is not None and group.fs is not None and os.environ.get("PRISM_B200_TP_FLAGS", "1") != "0")
        # ... and the row maxima of a row-parallel projection's input travel as words between the producers, which then
        # quantize in one launch instead of two passes around a max-all-reduce (PRISM_B200_TP_WORDS=0 keeps those)
        self.words = (self.flags and os.environ.get("PRISM_B200_TP_WORDS", "1") != "0"
                      and group.setup_many(M, 2 * len(layers)))
        # ... and the all-gather of a column-parallel projection's int8 input: every rank stores its own rows straight
        # into the other ranks' input buffers (peer-mapped), a flag handshake tells the readers
        # (PRISM_B200_TP_PUSH=0 keeps NCCL's all-gather)
        self.push = False
        if self.flags and os.environ.get("PRISM_B200_TP_PUSH", "1") != "0":
            xq_all = group.symmetric(M * hidden, i8)
            xs_all = group.symmetric(M, f32)
            if xq_all is not None and xs_all is not None:
                self.push = True
                self.xq, self.xs = xq_all[group.rank].view(M, hidden), xs_all[group.rank]
                lo, hi = self.r0, self.r0 + self.Ml
                self.xq_peers = [t.view(M, hidden)[lo:hi] for r, t in enumerate(xq_all) if r != group.rank]
                self.xs_peers = [t[lo:hi] for r, t in enumerate(xs_all) if r != group.rank]

    def __call__(self, h_in, own_rows=False):
        """One pass: h_in fp32 [M, hidden] is copied into the working residual, which is returned (a view of an
        internal buffer, overwritten by the next pass).  own_rows (several ranks, row-split pass only): h_in is this
        rank's block of M / n rows and the rank's block of the result is returned - what a caller that feeds and
        reads each rank's rows separately needs; the other rows' residual never has to exist on this rank."""
        M, nr, g = self.M, self.n_rows, self.g
        if own_rows:
            if not self.by_rows:
                raise RuntimeError("own_rows needs the row-split pass (several ranks, M / ranks >= 64 rows)")
            self.h[self.r0:self.r0 + self.Ml].copy_(h_in, non_blocking=True)
            return self._pass_by_rows(gather=False)
        self.h.copy_(h_in, non_blocking=True)
        if self.by_rows:
            return self._pass_by_rows()
        if g is not None and self.n > 1:
            g.begin(M)                            # short pass: a new pass number, exchanges inside the kernels
        if self.pdl:
            before = _lib.lib().pb_set_pdl(1)
            try:
                return self._pass()
            finally:
                _lib.lib().pb_set_pdl(before)
        return self._pass()

    def _pass(self):
        M, nr, g = self.M, self.n_rows, self.g
        pend = None
        for lw in self.layers:
            quant.fold(self.h, self.slots, pend, nr, M)
            quant.rows_q8(self.h, None, self.xq, self.xs, nr, M)
            w8a8.gemm(self.xq, self.xs, *lw["qkv"], self.qkv, nr, self.hidden, pdl=self.pdl)
            tp.quantize_rows(g if self.n > 1 else None, quant.rows_q8, M, self.amax, self.qkv[:, :self.ql], None,
                             self.aq, self.as_, nr, M)
            pend = self._out(self.aq, self.as_, lw["o"])
            quant.fold(self.h, self.slots, pend, nr, M)
            quant.rows_q8(self.h, None, self.xq, self.xs, nr, M)
            w8a8.gemm(self.xq, self.xs, *lw["gate_up"], self.gu, nr, self.hidden, pdl=self.pdl)
            tp.quantize_rows(g if self.n > 1 else None, quant.swiglu_q8, M, self.amax, self.gu, None, self.dq,
                             self.ds, nr, M)
            pend = self._out(self.dq, self.ds, lw["down"])
        quant.fold(self.h, self.slots, pend, nr, M)
        return self.h

    def close(self):
        if self.peer is not None:
            self.peer.close()
            self.peer = None

    def _out(self, a, a_s, wt):
        """A row-parallel projection into the residual: one rank adds in the GEMM's epilogue (or defers a K split to
        the fold); several ranks all-reduce int32 sums and fold."""
        w, w_s = wt
        if self.n > 1:
            return tp.out_proj(self.g, a, a_s, w, w_s, self.parts, self.M, self.n_rows, pdl=self.pdl)
        return w8a8.gemm(a, a_s, w, w_s, self.h, self.n_rows, a.shape[1], epi=1, slots=self.slots, pdl=self.pdl)

    def _pass_by_rows(self, gather=True):
        """Several ranks, many rows.  Between a row-parallel projection and the next column-parallel one every rank
        works on its own M / n rows of the residual stream: int32 partial sums -> reduce-scatter -> fold into the own
        rows -> quantize them -> all-gather the int8 rows and their scales.  Every element sees the operations of the
        one-GPU pass in the same order (exact integer sums, the same fold and quantizer roundings): the same bits."""
        M, nr, g, Ml, r0 = self.M, self.n_rows, self.g, self.Ml, self.r0
        h_own, xq_own, xs_own = self.h[r0:r0 + Ml], self.xq[r0:r0 + Ml], self.xs[r0:r0 + Ml]
        pend = None
        if self.flags:
            g.begin_handshakes()

        def gathered_input():
            quant.fold(h_own, None, pend, self.nr_own, Ml)
            quant.rows_q8(h_own, None, xq_own, xs_own, self.nr_own, Ml)
            if self.push:
                quant.push(xq_own, self.xq_peers)
                quant.push(xs_own, self.xs_peers)
                quant.handshake(g.handshake())
            else:
                g.gather2_(self.xq, xq_own, self.xs, xs_own)

        def out(a, a_s, wt):
            w, w_s = wt
            if self.peer is not None:
                w8a8.gemm_scatter(a, w, self.blocks, Ml, self.hidden, nr)
                if self.flags:
                    # the fold itself waits until every rank has signalled that its scatter kernel ended
                    return w8a8.Deferred(self.n, a_s[r0:r0 + Ml], w_s, self.sym, g.handshake())
                g.sum_(self.token)                 # a barrier: every rank's stores have landed before anyone folds
                return w8a8.Deferred(self.n, a_s[r0:r0 + Ml], w_s, self.sym)
            w8a8.gemm_i32(a, a_s, w, w_s, self.slots[:1], nr, max_split=1)
            g.scatter_sum_(self.own[0], self.slots[0])
            return w8a8.Deferred(1, a_s[r0:r0 + Ml], w_s, self.own)

        def quantize(fn, *args):
            if self.words:
                fn(*args, mode=3, sync=g.words_many())
            else:
                tp.quantize_rows(g, fn, M, self.amax, *args)

        for lw in self.layers:
            gathered_input()
            w8a8.gemm(self.xq, self.xs, *lw["qkv"], self.qkv, nr, self.hidden)
            quantize(quant.rows_q8, self.qkv[:, :self.ql], None, self.aq, self.as_, nr, M)
            pend = out(self.aq, self.as_, lw["o"])
            gathered_input()
            w8a8.gemm(self.xq, self.xs, *lw["gate_up"], self.gu, nr, self.hidden)
            quantize(quant.swiglu_q8, self.gu, None, self.dq, self.ds, nr, M)
            pend = out(self.dq, self.ds, lw["down"])
        quant.fold(h_own, None, pend, self.nr_own, Ml)
        if not gather:
            return h_own
        g.gather_(self.h, h_own)
        return self.h
