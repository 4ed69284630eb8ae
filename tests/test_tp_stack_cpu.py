"""The row-split tensor-parallel pass of linear_stack.LinearStack on CPU ranks (gloo, world sizes 4 and 8 against 1):
its orchestration - which rows a rank folds and quantizes, the reduce-scatter of the int32 sums, the all-gathers of the
int8 inputs, the global row maxima - must compose to the one-rank bits.  The GPU kernels are replaced inside the child
processes by CPU stand-ins with the same argument meaning (the oracle's GEMM and fold; plain numpy row quantizers; the
gated product without the sigmoid, which is elementwise and so independent of how columns are sharded)."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HID, QC, KVC, FFN, ROWS = 256, 256, 64, 512, 512


def _patch():
    import oracle
    from prism_b200 import quant, w8a8

    def bits(x):
        return x.view(torch.int16).numpy().view(np.uint16) if x.dtype == torch.bfloat16 else x.numpy()

    def as_f32(x):
        return oracle.bf16_to_f32(bits(x)) if x.dtype == torch.bfloat16 else x.numpy()

    def quantize(v, q, s, mode, amax):
        """v fp32 [T, K]: the row maximum (mode 1: also stored; mode 2: taken from amax), scale = max / 127."""
        am = np.abs(v).max(axis=1)
        if mode == 1:
            amax[:len(am)] = torch.from_numpy(am)
        if mode == 2:
            am = amax[:len(am)].numpy()
        sc = np.where(am > 0, am / np.float32(127), np.float32(1)).astype(np.float32)
        q.copy_(torch.from_numpy(np.clip(np.rint(v / sc[:, None]), -127, 127).astype(np.int8)))
        s.copy_(torch.from_numpy(sc))

    def rows_q8(x, inv, q, s, n, T, mode=0, amax=None):
        quantize(as_f32(x.contiguous()), q, s, mode, amax)

    def swiglu_q8(gu, inv, q, s, n, T, mode=0, amax=None):
        v = as_f32(gu.contiguous())
        ff = v.shape[1] // 2
        quantize((v[:, :ff] * v[:, ff:]).astype(np.float32), q, s, mode, amax)

    def gemm(a, a_s, w, w_s, out, n_rows, gk, epi=0, slots=None, **kw):
        K = a.shape[1]
        r = oracle.w8a8_gemm(a.numpy(), a_s.numpy()[:, None], w.numpy(), w_s.numpy()[:, None], K, epi,
                             out=out.numpy() if epi == 1 else None)
        if epi == 0:
            out.copy_(torch.from_numpy(r.view(np.int16)).view(torch.bfloat16))
        else:
            out.copy_(torch.from_numpy(r))
        return None

    def gemm_i32(a, a_s, w, w_s, slots, n_rows, max_split=4, **kw):
        K = a.shape[1]
        M, N = a.shape[0], w.shape[0]
        slots[0].copy_(torch.from_numpy(oracle.w8a8_gemm(a.numpy(), np.ones((M, 1), np.float32), w.numpy(),
                                                         np.ones((N, 1), np.float32), K, 3)))
        return 1

    def fold(h, parts, pending, n, T):
        if not pending:
            return
        p = pending.parts if pending.parts is not None else parts
        h.copy_(torch.from_numpy(oracle.fold(h.numpy(), p[:pending.n].numpy(), pending.a_s.numpy(), pending.w_s.numpy())))

    quant.rows_q8, quant.swiglu_q8, quant.fold = rows_q8, swiglu_q8, fold
    w8a8.gemm, w8a8.gemm_i32 = gemm, gemm_i32


def _rank(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    torch.set_num_threads(1)
    from prism_b200 import linear_stack as LS, tp
    _patch()
    dev = torch.device("cpu")
    g = tp.Group(rank, world, port=port, backend="gloo") if world > 1 else None
    try:
        layers = [LS.shard_layer(LS.make_layer_weights(i, dev, HID, QC, KVC, FFN), world, rank, HID, QC, KVC, FFN)
                  for i in range(2)]
        stack = LS.LinearStack(layers, ROWS, dev, g, HID, QC, KVC, FFN)
        assert stack.by_rows == (world > 1) and stack.peer is None
        h0 = torch.randn(ROWS, HID, generator=torch.Generator().manual_seed(3))
        for _ in range(2):
            h = stack(h0).clone()
        ret[(world, rank)] = h.numpy().tobytes()
    finally:
        if g is not None:
            g.barrier()
            g.close()


@pytest.mark.parametrize("world", [4, 8])
def test_row_split_pass_composes_to_one_rank_bits(world):
    import oracle
    oracle.build()
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_rank, args=(1, None, ret), nprocs=1, join=True)          # child processes: the stand-ins stay there
    mp.spawn(_rank, args=(world, 29740 + world, ret), nprocs=world, join=True)
    want = ret[(1, 0)]
    assert np.isfinite(np.frombuffer(want, np.float32)).all() and np.abs(np.frombuffer(want, np.float32)).max() > 0
    for r in range(world):
        assert ret[(world, r)] == want, f"rank {r} of {world}"
