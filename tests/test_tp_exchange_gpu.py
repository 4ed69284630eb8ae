"""The in-kernel tensor-parallel exchanges on ONE GPU: the other ranks are emulated by what they would have written
before this rank's kernel looks - their row-maximum words, their arrival flags, their int32 slots - in local buffers
standing in for their peer-mapped memory.  (Kernels that wait on one another never run as separate launches on one
GPU: nothing guarantees that they run at the same time.  Real ranks on real GPUs: test_tp_gpu.py.)

Checked: a producer in mode 3 quantizes with the maximum over every rank's word and publishes its own word, tagged
with the pass number, into every other rank's buffer; fold / norm_q8 with a Sync add every rank's slots and give the
bits of the same fold over all the slots at once; a wait for a rank that never arrives runs out, reports status 4
and leaves the context usable."""
import types

import numpy as np
import pytest
import torch

import oracle
from prism_b200 import _lib, quant, synth, w8a8
from util import n_rows, np_bits, same

pytestmark = pytest.mark.gpu


def words_setup(dev, world, rank, rows, off, epoch_value, peer_amax):
    """Every rank's word buffer (local stand-ins), this rank's pre-filled with the others' words of this pass."""
    bufs = [torch.zeros((off + rows) * world, dtype=torch.int64, device=dev) for _ in range(world)]
    mine = bufs[rank].view(-1, world)
    for q in range(world):
        if q == rank:
            continue
        bits = torch.from_numpy(peer_amax[q].view(np.int32).astype(np.int64) & 0xFFFFFFFF)
        mine[off:off + rows, q] = ((epoch_value & 0xFFFFFFFF) << 32 | bits).to(dev)
    epoch = torch.tensor([epoch_value], dtype=torch.int64, device=dev)
    return bufs, epoch


@pytest.mark.parametrize("world,rank", [(2, 0), (4, 1), (8, 7)])
def test_row_maximum_exchange(dev, world, rank):
    T, K, live, off, e = 9, 5120, 8, 18, 41
    x = synth.activations(T, K, seed=world)
    rng = np.random.default_rng(world)
    peer = {q: (rng.random(T).astype(np.float32) * 30).astype(np.float32) for q in range(world) if q != rank}
    others_max = np.max(np.stack(list(peer.values())), 0)
    rq, rs = oracle.quant_rows(np_bits(x), live=live, amax_in=others_max.reshape(T, 1))
    _, _, own = oracle.quant_rows(np_bits(x), live=live, want_amax=True)
    bufs, epoch = words_setup(dev, world, rank, T, off, e, peer)
    q = torch.zeros(T, K, dtype=torch.int8, device=dev)
    s = torch.zeros(T, device=dev)
    sync = quant.Sync(epoch, tuple(bufs), off, (), rank, world)
    quant.rows_q8(x.to(dev), None, q, s, n_rows(live, dev), T, mode=3, sync=sync)
    torch.cuda.synchronize()
    assert same(q[:live], rq[:live]) and same(s[:live], rs[:live, 0])
    want_word = (np.int64(e) << 32) | (own[:live, 0].view(np.int32).astype(np.int64) & 0xFFFFFFFF)
    for p in range(world):
        if p != rank:
            got = bufs[p].view(-1, world)[off:off + live, rank].cpu().numpy()
            assert np.array_equal(got, want_word), p                    # published to every other rank, tagged
            assert not bool(bufs[p].view(-1, world)[off + live:, rank].any())


def test_swiglu_and_gated_norm_exchange_match_mode_2(dev):
    """Mode 3 against mode 2 with the same maxima: the same kernel code around a different source of the maximum."""
    world, rank, e = 4, 2, 7
    T, FF = 6, 4352
    rng = np.random.default_rng(1)
    peer = {q: rng.random(T).astype(np.float32) * 200 for q in range(world) if q != rank}
    amax = torch.from_numpy(np.max(np.stack(list(peer.values())), 0)).to(dev)
    gu = (torch.randn(T, 2 * FF, generator=torch.Generator().manual_seed(3)) * 2).to(torch.bfloat16).to(dev)
    nr = n_rows(T, dev)
    q2, s2 = torch.zeros(T, FF, dtype=torch.int8, device=dev), torch.zeros(T, device=dev)
    quant.swiglu_q8(gu, None, q2, s2, nr, T, mode=2, amax=amax.clone())
    bufs, epoch = words_setup(dev, world, rank, T, 0, e, peer)
    q3, s3 = torch.zeros_like(q2), torch.zeros_like(s2)
    quant.swiglu_q8(gu, None, q3, s3, nr, T, mode=3, sync=quant.Sync(epoch, tuple(bufs), 0, (), rank, world))
    assert torch.equal(q2, q3) and torch.equal(s2, s3)
    HV, D = 12, 128
    cfg = types.SimpleNamespace(eps=1e-6, v_heads=HV, gdn_dim=D)
    g = torch.Generator().manual_seed(5)
    o = torch.randn(T, HV * D, generator=g).to(dev)
    proj = torch.randn(T, 2 * HV * D, generator=g).to(torch.bfloat16).to(dev)
    w, inv = (torch.rand(D, generator=g) + 0.5).to(dev), (torch.rand(HV * D, generator=g) + 0.5).to(dev)
    q2, s2 = torch.zeros(T, HV * D, dtype=torch.int8, device=dev), torch.zeros(T, device=dev)
    quant.gated_norm_q8(o, proj, HV * D, w, inv, q2, s2, nr, T, cfg, mode=2, amax=amax.clone())
    bufs, epoch = words_setup(dev, world, rank, T, 0, e, peer)
    q3, s3 = torch.zeros_like(q2), torch.zeros_like(s2)
    quant.gated_norm_q8(o, proj, HV * D, w, inv, q3, s3, nr, T, cfg, mode=3, sync=quant.Sync(epoch, tuple(bufs), 0, (), rank, world))
    assert torch.equal(q2, q3) and torch.equal(s2, s3)


def flags_setup(dev, world, rank, chan, epoch_value, arrived=True):
    flags = [torch.zeros(64 * world, dtype=torch.int64, device=dev) for _ in range(world)]
    if arrived:
        for q in range(world):
            if q != rank:
                flags[rank][chan * world + q] = epoch_value
    return flags, torch.tensor([epoch_value], dtype=torch.int64, device=dev)


@pytest.mark.parametrize("world,rank,S", [(2, 1, 1), (4, 0, 3), (8, 5, 2)])
def test_fold_over_every_ranks_slots(dev, world, rank, S):
    rows, N, live, chan, e = 20, 5120, 17, 5, 9
    g = torch.Generator().manual_seed(world + S)
    h = torch.randn(rows, N, generator=g)
    slots = [torch.randint(-(1 << 22), 1 << 22, (S, rows, N), generator=g, dtype=torch.int32) for _ in range(world)]
    sa, sw = torch.rand(rows, generator=g) * 1e-2, torch.rand(N, generator=g) * 1e-3
    want = oracle.fold(h.numpy(), torch.cat(slots).numpy(), sa.numpy(), sw.numpy(), live)
    flags, epoch = flags_setup(dev, world, rank, chan, e)
    dslots = [t.to(dev) for t in slots]
    sync = quant.Sync(epoch, tuple(flags), chan, tuple(t for r, t in enumerate(dslots) if r != rank), rank, world)
    hd = h.to(dev)
    quant.fold(hd, None, w8a8.Deferred(S, sa.to(dev), sw.to(dev), dslots[rank], sync), n_rows(live, dev), rows)
    torch.cuda.synchronize()
    assert same(hd, want)
    for p in range(world):                                   # this rank's arrival reached every other rank's flags
        if p != rank:
            assert int(flags[p][chan * world + rank]) == e
    # the same through norm_q8: the deferred add over every rank's slots, then the norm of the updated row
    w = (torch.rand(N, generator=g) + 0.5)
    flags, epoch = flags_setup(dev, world, rank, chan, e)
    sync = quant.Sync(epoch, tuple(flags), chan, tuple(t for r, t in enumerate(dslots) if r != rank), rank, world)
    hd = h.to(dev)
    q = torch.zeros(rows, N, dtype=torch.int8, device=dev)
    s = torch.zeros(rows, device=dev)
    quant.norm_q8(hd, w.to(dev), q, s, n_rows(live, dev), rows, 1e-6,
                  pending=w8a8.Deferred(S, sa.to(dev), sw.to(dev), dslots[rank], sync))
    h2 = h.to(dev)
    q2, s2 = torch.zeros_like(q), torch.zeros_like(s)
    quant.norm_q8(h2, w.to(dev), q2, s2, n_rows(live, dev), rows, 1e-6,
                  pending=w8a8.Deferred(S * world, sa.to(dev), sw.to(dev), torch.cat(dslots)))
    assert same(hd, want) and torch.equal(hd, h2) and torch.equal(q, q2) and torch.equal(s, s2)


def test_wait_for_a_rank_that_never_arrives(dev, lib):
    """The flags stay unset (as if the other rank had died between steps): the fold's wait runs out after the bound,
    the status word says where, and the next launch on the context is correct."""
    world, rank, rows, N, chan, e = 2, 0, 4, 1024, 3, 5
    g = torch.Generator().manual_seed(1)
    h = torch.randn(rows, N, generator=g)
    slots = [torch.randint(-1000, 1000, (1, rows, N), generator=g, dtype=torch.int32).to(dev) for _ in range(world)]
    sa, sw = (torch.rand(rows, generator=g) * 1e-2).to(dev), (torch.rand(N, generator=g) * 1e-3).to(dev)
    flags, epoch = flags_setup(dev, world, rank, chan, e, arrived=False)
    sync = quant.Sync(epoch, tuple(flags), chan, (slots[1],), rank, world)
    assert lib.pb_set_wait_limit_ns(2_000_000) == 0
    try:
        hd = h.to(dev)
        quant.fold(hd, None, w8a8.Deferred(1, sa, sw, slots[0], sync), n_rows(rows, dev), rows)
        torch.cuda.synchronize()                              # returns: the wait was bounded
        code, where = _lib.device_status(reset=True)
    finally:
        lib.pb_set_wait_limit_ns(0)
    assert code == 4 and where == 0x2100 + 1, (code, hex(where))
    # a row-maximum word that never comes, likewise
    x = synth.activations(2, 1024, seed=2).to(dev)
    bufs = [torch.zeros(2 * world, dtype=torch.int64, device=dev) for _ in range(world)]
    q, s = torch.zeros(2, 1024, dtype=torch.int8, device=dev), torch.zeros(2, device=dev)
    assert lib.pb_set_wait_limit_ns(2_000_000) == 0
    try:
        quant.rows_q8(x, None, q, s, n_rows(2, dev), 2, mode=3, sync=quant.Sync(epoch, tuple(bufs), 0, (), rank, world))
        torch.cuda.synchronize()
        code, where = _lib.device_status(reset=True)
    finally:
        lib.pb_set_wait_limit_ns(0)
    assert code == 4 and where == 0x2000 + 1, (code, hex(where))
    # the context is intact: the ordinary fold right after
    hd = h.to(dev)
    want = oracle.fold(h.numpy(), torch.cat(slots).cpu().numpy(), sa.cpu().numpy(), sw.cpu().numpy())
    quant.fold(hd, None, w8a8.Deferred(2, sa, sw, torch.cat(slots)), n_rows(rows, dev), rows)
    assert same(hd, want)
