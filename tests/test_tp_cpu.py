"""The tensor-parallel host logic on CPU ranks (gloo, world size 2): the process group's exact int32 SUM / fp32 MAX,
tp.out_proj and tp.quantize_rows plumbing, the reduce-scatter / all-gather pair of the row-split pass.  The GPU kernels are replaced by the CPU oracle inside this test only
(monkeypatched in the child processes): what is checked is that the two exchange steps compose to the one-rank bits."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _rank(rank, world, port):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle
    from prism_b200 import tp, w8a8
    g = tp.Group(rank, world, port=port, backend="gloo")
    try:
        gen = torch.Generator().manual_seed(0)
        M, N, K = 6, 32, 256
        a = torch.randint(-127, 128, (M, K), generator=gen, dtype=torch.int8)
        w = torch.randint(-127, 128, (N, K), generator=gen, dtype=torch.int8)
        x = torch.randn(M, K, generator=gen)
        sw = torch.rand(N, generator=gen) * 1e-3
        k = K // world
        # --- quantize_rows: modes 1 / 2 around the MAX all-reduce
        def rows_q8(xs, q, s, mode=0, amax=None):
            qq, ss, am = oracle.quant_rows(xs.numpy(), amax_in=None if mode != 2 else amax.numpy()[:, None].copy(),
                                           want_amax=True)
            q.copy_(torch.from_numpy(qq))
            s.copy_(torch.from_numpy(ss[:, 0]))
            if mode == 1:
                amax.copy_(torch.from_numpy(am[:, 0]))
        shard = x[:, rank * k:(rank + 1) * k].contiguous()
        q = torch.zeros(M, k, dtype=torch.int8)
        s = torch.zeros(M)
        amax = torch.zeros(M)
        tp.quantize_rows(g, rows_q8, M, amax, shard, q, s)
        wq, ws = oracle.quant_rows(x.numpy())
        ok_quant = np.array_equal(q.numpy(), wq[:, rank * k:(rank + 1) * k]) and np.array_equal(s.numpy(), ws[:, 0])
        # --- out_proj: int32 partial sums -> SUM all-reduce -> Deferred
        def gemm_i32(aa, a_s, ww, w_s, slots, n_rows, max_split=4, pdl=False):
            slots[0].copy_(torch.from_numpy(oracle.w8a8_gemm(aa.numpy(), np.ones((M, 1), np.float32), ww.numpy(),
                                                              np.ones((N, 1), np.float32), aa.shape[1], 3)))
            return 1
        w8a8.gemm_i32 = gemm_i32
        flat = torch.zeros(tp.parts_elems(M, N), dtype=torch.int32)
        sa = torch.from_numpy(ws[:, 0].copy())
        d = tp.out_proj(g, torch.from_numpy(wq[:, rank * k:(rank + 1) * k].copy()), sa,
                        w[:, rank * k:(rank + 1) * k].contiguous(), sw, flat, M, None)
        exact = oracle.w8a8_gemm(wq, ws, w.numpy(), sw.numpy()[:, None], K, 3)
        ok_sum = d.n == 1 and np.array_equal(d.parts[0].numpy(), exact)
        h = torch.randn(M, N, generator=torch.Generator().manual_seed(1))
        folded = oracle.fold(h.numpy(), d.parts.numpy(), sa.numpy(), sw.numpy())
        ok_fold = np.array_equal(folded, oracle.w8a8_gemm(wq, ws, w.numpy(), sw.numpy()[:, None], K, 1, out=h.numpy()))
        # --- the row-split exchange: reduce-scatter the sums, fold this rank's rows, gather them
        part = torch.from_numpy(oracle.w8a8_gemm(wq[:, rank * k:(rank + 1) * k].copy(), np.ones((M, 1), np.float32),
                                                 w[:, rank * k:(rank + 1) * k].contiguous().numpy(),
                                                 np.ones((N, 1), np.float32), k, 3))
        rows = M // world
        own = torch.zeros(rows, N, dtype=torch.int32)
        g.scatter_sum_(own, part)
        ok_rs = np.array_equal(own.numpy(), exact[rank * rows:(rank + 1) * rows])
        mine = oracle.fold(h.numpy()[rank * rows:(rank + 1) * rows].copy(), own.numpy()[None],
                           sa.numpy()[rank * rows:(rank + 1) * rows].copy(), sw.numpy())
        full = torch.zeros(M, N)
        full[rank * rows:(rank + 1) * rows] = torch.from_numpy(mine)
        g.gather_(full, full[rank * rows:(rank + 1) * rows])
        ok_rows = ok_rs and np.array_equal(full.numpy(), folded)
        res = (rank, bool(ok_quant), bool(ok_sum), bool(ok_fold and ok_rows))
    finally:
        g.barrier()
        g.close()
    return res


def _entry(rank, world, port, ret):
    ret[rank] = _rank(rank, world, port)


def test_two_cpu_ranks_compose_to_one_rank_bits():
    import oracle
    oracle.build()
    world, port = 2, 29731
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_entry, args=(world, port, ret), nprocs=world, join=True)
    assert len(ret) == world
    for r in range(world):
        assert ret[r] == (r, True, True, True), ret[r]


def test_group_single_rank_is_a_no_op():
    sys.path.insert(0, ROOT)
    from prism_b200 import tp
    calls = []
    tp.quantize_rows(None, lambda *a, **k: calls.append((a, k)), 4, None, 1, 2)
    assert calls == [((1, 2), {})]


def test_exchange_bookkeeping(monkeypatch):
    """Group.begin / words / sync and out_proj's pull path on stand-in buffers (no process group, no GPU): which
    passes exchange inside the kernels, the pass counter, the word rows and flag channels handed out, the two slot
    parities alternating."""
    sys.path.insert(0, ROOT)
    from prism_b200 import quant, tp, w8a8
    hidden, world = 64, 2
    g = tp.Group.__new__(tp.Group)
    g.rank, g.world, g.backend, g.device = 1, world, "nccl", torch.device("cpu")
    g.fast_rows, g.pull_rows, g.word_steps, g.hidden = 255, 128, 4, hidden
    g.parity = tp.MAX_SPLIT * g.pull_rows * hidden
    g.fs = [torch.zeros(tp.CHANNELS * world, dtype=torch.int64) for _ in range(world)]
    g.xs = [torch.zeros(2 * g.parity, dtype=torch.int32) for _ in range(world)]
    g.ws = [torch.zeros(g.word_steps * g.fast_rows * world, dtype=torch.int64) for _ in range(world)]
    g.epoch = torch.zeros(1, dtype=torch.int64)
    g.fast = g.pull = False
    g.nsum = g.step = g.mstep = 0
    g.begin(64)
    assert g.fast and g.pull and int(g.epoch) == 1
    s0, s1 = g.words(), g.words()
    assert isinstance(s0, quant.Sync) and (s0.chan, s1.chan) == (0, 255) and s0.rank == 1 and s0.world == 2 and s0.others == ()
    assert s0.flags[0].data_ptr() == g.ws[0].data_ptr()
    calls = []

    def gemm_i32(a, a_s, w, w_s, slots, n_rows, max_split=4, pdl=False):
        calls.append(slots.data_ptr())
        return 2
    monkeypatch.setattr(w8a8, "gemm_i32", gemm_i32)
    a, w = torch.zeros(64, 32, dtype=torch.int8), torch.zeros(hidden, 32, dtype=torch.int8)
    d0 = tp.out_proj(g, a, None, w, None, None, 64, None)
    d1 = tp.out_proj(g, a, None, w, None, None, 64, None)
    assert d0.n == 2 and d0.sync.chan == 0 and d1.sync.chan == 1
    assert calls[0] == g.xs[1].data_ptr() and calls[1] == g.xs[1].data_ptr() + 4 * g.parity      # own buffer, two parities
    assert d0.sync.others[0].data_ptr() == g.xs[0].data_ptr() and d1.sync.others[0].data_ptr() == g.xs[0].data_ptr() + 4 * g.parity
    assert d0.parts.shape == (2, 64, hidden) and d0.sync.flags[1].data_ptr() == g.fs[1].data_ptr()
    g.begin(200)
    assert g.fast and not g.pull and int(g.epoch) == 2 and g.step == 0 and g.mstep == 0
    for _ in range(4):
        g.words()
    with pytest.raises(RuntimeError, match="row-maximum exchanges"):
        g.words()
    g.begin(300)
    assert not g.fast and not g.pull and int(g.epoch) == 2          # long pass: collectives, no new pass number
    seen = []
    monkeypatch.setattr(g, "max_", lambda x: None, raising=False)
    tp.quantize_rows(g, lambda *a, **k: seen.append(k), 300, torch.zeros(300), "x")
    assert [k.get("mode") for k in seen] == [1, 2]
    g.begin(8)
    seen.clear()
    tp.quantize_rows(g, lambda *a, **k: seen.append(k), 8, None, "x")
    assert len(seen) == 1 and seen[0]["mode"] == 3 and seen[0]["sync"].chan == 0
    # many rows (the row-split pass): a pass number from begin_handshakes, word rows of wm_rows per exchange
    g.wm = [torch.zeros(3 * 1024 * world, dtype=torch.int64) for _ in range(world)]
    g.wm_rows, g.wm_steps = 1024, 3
    assert g.begin_handshakes() and int(g.epoch) == 4 and g.step == 0 and g.mstep == 0
    m0, m1 = g.words_many(), g.words_many()
    assert (m0.chan, m1.chan) == (0, 1024) and m0.flags[1].data_ptr() == g.wm[1].data_ptr() and m0.world == 2
    assert quant._mode_args(3, None, m1, 1024) is None
    with pytest.raises(RuntimeError, match="too small"):
        quant._mode_args(3, None, g.words_many(), 1025)           # third exchange, one row more than its buffer holds
    with pytest.raises(RuntimeError, match="row-maximum exchanges"):
        g.words_many()
    h = g.handshake()
    assert h.chan == 0 and h.others == () and h.flags[0].data_ptr() == g.fs[0].data_ptr()
