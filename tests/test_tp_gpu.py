"""Tensor-parallel identity on GPUs.  (1) On one GPU, every rank count is emulated arithmetically: K split / N split
per projection, int32 slots summed, folded - the method of the reference's tests/test_cuda_gemm.py:175-225.  (2) With
two or more GPUs, the linear stack runs as real NCCL ranks (child processes) and rank 0's result must be bit-identical
to the one-GPU run (tests/test_tp.py:184-194 compares with torch.equal the same way)."""
import os
import subprocess
import sys

import pytest
import torch

import oracle
from prism_b200 import quant, tp, w8a8
from util import n_rows, rand_w8a8, same

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.parametrize("M,N,K,live", [(64, 5120, 5120, 64), (8, 5120, 17408, 3), (300, 2560, 5120, 280)])
@pytest.mark.parametrize("ranks", [2, 4, 8])
def test_row_parallel_emulated(dev, M, N, K, live, ranks):
    """Each rank's int32 sums over its K shard (every split the kernel offers), added over the ranks and folded,
    equal the one-GPU residual add bit for bit; the sums are the exact integer product."""
    a, w, sa, sw = rand_w8a8(M, N, K, seed=ranks + N)
    exact = oracle.w8a8_gemm(a.numpy(), sa.numpy(), w.numpy(), sw.numpy(), K, 3, live)
    base = torch.randn(M, N, generator=torch.Generator().manual_seed(7))
    ref = oracle.w8a8_gemm(a.numpy(), sa.numpy(), w.numpy(), sw.numpy(), K, 1, live, out=base.numpy())
    nr = n_rows(live, dev)
    sad, swd = sa.to(dev).view(-1), sw.to(dev).view(-1)
    k = K // ranks
    tot = torch.zeros(M, N, dtype=torch.int32, device=dev)
    flat = torch.zeros(tp.parts_elems(M, N), dtype=torch.int32, device=dev)
    for r in range(ranks):
        xa = a[:, r * k:(r + 1) * k].contiguous().to(dev)
        xw = w[:, r * k:(r + 1) * k].contiguous().to(dev)
        flat.fill_(-(1 << 30))
        d = tp.out_proj(None, xa, sad, xw, swd, flat, M, nr)
        tot[:live] += d.parts[:, :live].sum(0, dtype=torch.int32)
    assert same(tot[:live], exact[:live])
    res = base.to(dev)
    quant.fold(res, tot[None], w8a8.Deferred(1, sad, swd), nr, M)
    assert same(res, ref)


@pytest.mark.parametrize("ranks", [2, 8])
def test_column_parallel_emulated(dev, ranks):
    """A column-parallel shard's outputs are the whole matrix's columns: same bits, no communication."""
    M, N, K = 40, 7168, 5120
    a, w, sa, sw = rand_w8a8(M, N, K, seed=ranks)
    nr = n_rows(M, dev)
    ad, sad = a.to(dev), sa.to(dev).view(-1)
    whole = torch.zeros(M, N, dtype=torch.bfloat16, device=dev)
    w8a8.gemm(ad, sad, w.to(dev), sw.to(dev).view(-1), whole, nr, K)
    for r in range(ranks):
        idx = tp.linear_shards(5120, 1024, 17408, ranks, r)["qkv"]
        part = torch.zeros(M, len(idx), dtype=torch.bfloat16, device=dev)
        w8a8.gemm(ad, sad, w[idx].contiguous().to(dev), sw.view(-1)[idx].contiguous().to(dev), part, nr, K)
        assert same(part, whole[:, idx.to(dev)].contiguous())


@pytest.mark.parametrize("M,N,K,blocks,live", [(512, 1024, 1024, 2, 512), (1024, 5120, 640, 8, 1024), (768, 384, 2176, 3, 700),
                                               (512, 100, 512, 4, 300)])
def test_scatter_blocks_emulated(dev, M, N, K, blocks, live):
    """gemm_scatter's row blocks (on one GPU: separate local buffers standing in for the ranks' memory) hold the rows
    of the exact integer product; rows past the live count are not written."""
    a, w, sa, sw = rand_w8a8(M, N, K, seed=blocks + N)
    exact = oracle.w8a8_gemm(a.numpy(), sa.numpy(), w.numpy(), sw.numpy(), K, 3, live)
    rows = M // blocks
    assert rows % 128 == 0
    nr = n_rows(live, dev)
    bufs = [torch.full((rows + 1, N), -7, dtype=torch.int32, device=dev) for _ in range(blocks)]
    w8a8.gemm_scatter(a.to(dev), w.to(dev), [b.data_ptr() for b in bufs], rows, N, nr)
    torch.cuda.synchronize()
    for o, b in enumerate(bufs):
        lo, hi = o * rows, min((o + 1) * rows, live)
        if hi > lo:
            assert same(b[:hi - lo], exact[lo:hi]), o
        assert bool((b[max(hi - lo, 0):] == -7).all()), o


def _run(cmd, env=None):
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]


# rows, extra worker arguments, environment: 1 / 64 rows run the in-kernel exchanges (row maxima as words, sums pulled by
# the fold), eagerly and as a replayed graph, and once more through NCCL's all-reduces; 700 rows NCCL's reduce-scatter;
# 2048 the scatter fused into the GEMM; the last case is the benchmark's own configuration
CASES = [(1, [], {}), (64, [], {}), (64, ["graph"], {}), (1, ["graph"], {}), (64, [], {"PRISM_B200_TP_FUSED": "0"}),
         (200, [], {}), (700, [], {}), (2048, [], {}), (8192, ["full"], {})]


@pytest.mark.parametrize("rows,extra,env_extra", CASES)
def test_real_ranks_bit_identical(dev, tmp_path, rows, extra, env_extra):
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs 2 or more GPUs")
    one = str(tmp_path / "one.pt")
    _run([sys.executable, os.path.join(HERE, "tp_worker.py"), one, str(rows)] + [e for e in extra if e == "full"])
    want = torch.load(one)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", **env_extra)
    for world in [w for w in (2, 4, 8) if w <= n]:
        out = str(tmp_path / f"tp{world}.pt")
        _run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
              "--master-addr", "127.0.0.1", "--master-port", str(29500 + world), os.path.join(HERE, "tp_worker.py"),
              out, str(rows)] + extra, env)
        got = torch.load(out)
        assert torch.equal(got.view(torch.int32), want.view(torch.int32)), f"{world} ranks differ from one GPU"


def test_two_devices_in_one_process(dev):
    """One process driving two GPUs: kernels that need more than 48 KB of shared memory must be opted in on EACH
    device (the opt-in, the SM count and the occupancy answers are kept per device ordinal), and the static-scratch
    entry point must look its array up on each device.  Same inputs on cuda:0 and cuda:1: the same bits."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 or more GPUs")
    from prism_b200 import _lib
    outs = []
    for d in (0, 1, 0):
        device = torch.device("cuda", d)
        with torch.cuda.device(device):
            for (M, N, K) in ((300, 1024, 2560), (16, 5120, 5120)):          # tile kernel, few-rows kernel with K split
                a, w, sa, sw = rand_w8a8(M, N, K, seed=M)
                out = torch.zeros(M, N, dtype=torch.bfloat16, device=device)
                w8a8.gemm(a.to(device), sa.to(device).view(-1), w.to(device), sw.to(device).view(-1), out,
                          n_rows(M, device), K)
                res = torch.randn(M, N, generator=torch.Generator().manual_seed(1)).to(device)
                w8a8.gemm(a.to(device), sa.to(device).view(-1), w.to(device), sw.to(device).view(-1), res,
                          n_rows(M, device), K, epi=1)
                torch.cuda.synchronize(device)
                assert _lib.device_status()[0] == 0
                outs.append((d, M, out.cpu(), res.cpu()))
    ref = {(M): (o, r) for d, M, o, r in outs if d == 0}
    for d, M, o, r in outs:
        assert torch.equal(o.view(torch.int16), ref[M][0].view(torch.int16)) and torch.equal(r, ref[M][1]), (d, M)
