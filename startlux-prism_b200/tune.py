"""Tuning-table generator for the decode-shape (few rows) W8A8 GEMMs: measures every K-split count on this GPU and
writes the fastest per projection shape and row count.  The counterpart of the reference's table generators
(bench/cuda_gemm_micro.py --table, bench/w4a8_table.py; tables kernels/gemm_table_<gpu>.json read by
kernels/w8a8.py:151-168): without a table w8a8.pick_split falls back to its rule, with one it takes the measured choice
of the nearest measured row count.

    python -m prism_b200.tune [--out PATH] [--shapes 7168x5120,5120x5120,...] [--rows 1,8,16,64]

Method (the reference's, bench/gemm_micro.py:48-69, bench/cuda_gemm_micro.py:117): a CUDA graph of back-to-back calls
that cycle over weight copies totalling more than three L2 sizes, best of five replays, CUDA events around each replay.
The table is read from PRISM_B200_GEMM_TABLE or gemm_table_b200.json beside this file.
"""
import argparse
import json
import os
import sys

DEFAULT_SHAPES = [(7168, 5120), (5120, 5120), (34816, 5120), (5120, 17408)]
DEFAULT_ROWS = [1, 2, 4, 8, 16, 32, 64]
TABLE = os.path.join(os.path.dirname(os.path.abspath(__file__)), "gemm_table_b200.json")
L2_BYTES = 126 << 20


def graph_us(fn_of_copy, copies, iters=None, reps=5):
    import torch
    iters = iters or max(copies, 8)
    for c in range(copies):
        fn_of_copy(c)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(iters):
            fn_of_copy(i % copies)
    best = 1e30
    for _ in range(reps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1) * 1e3 / iters)
    return best


def measure(shapes, rows, log=print, chained=True):
    """chained: rows from 2 up are timed as LinearStack launches them at few rows - every launch a programmatic
    dependent of the one before it (pb_set_pdl) - so that the choice fits that pass; one row (the CUDA-core kernel,
    a plain launch) is timed alone."""
    import torch

    from . import _lib, quant, w8a8
    dev = torch.device("cuda", torch.cuda.current_device())
    gen = torch.Generator(device=dev).manual_seed(4)
    table = {}
    for N, K in shapes:
        copies = max(4, -(-3 * L2_BYTES // (N * K)))
        ws = [torch.randint(-127, 128, (N, K), dtype=torch.int8, device=dev, generator=gen) for _ in range(copies)]
        sw = torch.rand(N, device=dev, generator=gen) * 1e-3
        for residual in (False, True):
            key = f"{N}x{K}" + ("r" if residual else "")
            table[key] = {}
            for M in rows:
                a = torch.randint(-127, 128, (M, K), dtype=torch.int8, device=dev, generator=gen)
                sa = torch.rand(M, device=dev, generator=gen) * 1e-2
                nr = torch.tensor([M], dtype=torch.int32, device=dev)
                out = torch.zeros(M, N, dtype=torch.float32 if residual else torch.bfloat16, device=dev)
                slots = torch.zeros(w8a8.MAX_SPLIT, M, N, dtype=torch.int32, device=dev) if residual else None
                best = None
                for split in range(1, w8a8.MAX_SPLIT + 1):
                    if w8a8.effective_split(K, split) != split:
                        continue
                    for defer in ((False, True) if residual and split > 1 else (False,)):
                        pend = {}

                        def call(c):
                            pend[0] = w8a8.gemm(a, sa, ws[c], sw, out, nr, K, epi=int(residual), cfg=split,
                                                slots=slots if defer else None)
                            if chained and M > 1 and pend[0] is not None:
                                quant.fold(out, slots, pend[0], nr, M)        # the fold is part of the chain
                        if chained and M > 1:
                            before = _lib.lib().pb_set_pdl(1)
                            try:
                                us = graph_us(call, copies)
                            finally:
                                _lib.lib().pb_set_pdl(before)
                        else:
                            us = graph_us(call, copies)
                            if pend[0] is not None:       # the deferred add is finished by a fold: its time counts
                                us += graph_us(lambda c: quant.fold(out, slots, pend[0], nr, M), 1, iters=8)
                        if best is None or us < best["us"]:
                            best = {"split": split, "defer": bool(defer), "us": round(us, 2)}
                table[key][str(M)] = best
                log(f"{key} M={M}: {best}")
        del ws
        torch.cuda.empty_cache()
    return table


def load_table(path=None):
    """{(N, K, residual): {M: {"split", "defer", "us"}}} from the table file, or {} when there is none."""
    path = path or os.environ.get("PRISM_B200_GEMM_TABLE") or TABLE
    if not os.path.exists(path):
        return {}
    raw = json.load(open(path))["table"]
    out = {}
    for key, by_m in raw.items():
        n, k = key.rstrip("r").split("x")
        out[(int(n), int(k), key.endswith("r"))] = {int(m): v for m, v in by_m.items()}
    return out


def main(argv=None):
    import torch
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=TABLE)
    ap.add_argument("--shapes", default=None)
    ap.add_argument("--rows", default=None)
    ap.add_argument("--plain", action="store_true", help="time every product alone (no chain of dependent launches)")
    args = ap.parse_args(argv)
    shapes = [tuple(int(v) for v in s.split("x")) for s in args.shapes.split(",")] if args.shapes else DEFAULT_SHAPES
    rows = [int(v) for v in args.rows.split(",")] if args.rows else DEFAULT_ROWS
    table = measure(shapes, rows, chained=not args.plain)
    doc = {"gpu": torch.cuda.get_device_name(0), "sms": torch.cuda.get_device_properties(0).multi_processor_count,
           "method": "CUDA graph of calls over rotating weight copies (> 3 x L2), best of 5 replays"
           + ("" if args.plain else "; 2 rows and up as a chain of programmatic dependent launches"), "table": table}
    with open(args.out, "w") as f:
        json.dump(doc, f, indent=1)
    print(f"wrote {args.out}")


if __name__ == "__main__":
    sys.exit(main())
