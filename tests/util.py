"""Helpers shared by the GPU parity tests: seeded operands, numpy <-> torch views, exact comparisons."""
import numpy as np
import torch


def np_bits(t):
    """torch bf16 tensor -> uint16 bit patterns (numpy)."""
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def bf16_from_bits(bits):
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).view(torch.bfloat16)


def rand_w8a8(M, N, K, seed, groups=1):
    g = torch.Generator().manual_seed(seed)
    a = torch.randint(-127, 128, (M, K), generator=g, dtype=torch.int8)
    w = torch.randint(-127, 128, (N, K), generator=g, dtype=torch.int8)
    sa = torch.rand(M, groups, generator=g) * 1e-2
    sw = torch.rand(N, groups, generator=g) * 1e-3
    return a, w, sa.contiguous(), sw.contiguous()


def n_rows(live, dev):
    return torch.tensor([live], dtype=torch.int32, device=dev)


def same(x, y):
    """Bit equality of two arrays / tensors (NaN-safe for floats: compares bit patterns)."""
    x = x.detach().cpu().numpy() if isinstance(x, torch.Tensor) and x.dtype != torch.bfloat16 else x
    y = y.detach().cpu().numpy() if isinstance(y, torch.Tensor) and y.dtype != torch.bfloat16 else y
    if isinstance(x, torch.Tensor):
        x = np_bits(x)
    if isinstance(y, torch.Tensor):
        y = np_bits(y)
    x, y = np.ascontiguousarray(x), np.ascontiguousarray(y)
    if x.shape != y.shape:
        return False
    if x.dtype == np.float32:
        x, y = x.view(np.uint32), y.view(np.uint32)
    return bool(np.array_equal(x, y))


def first_diff(x, y):
    x, y = np.asarray(x), np.asarray(y)
    idx = np.argwhere(x != y)
    return None if len(idx) == 0 else (tuple(idx[0]), x[tuple(idx[0])], y[tuple(idx[0])], len(idx))
