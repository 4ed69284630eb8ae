"""Worker of the tensor-parallel identity test: runs the decoder-layer linear stack on this process's rank (1 rank, or
N ranks under torch.distributed.run) and saves rank 0's final residual.  Sizes are reduced (hidden 1024) so the 1-rank
and N-rank runs take seconds.

    python tests/tp_worker.py OUT.pt ROWS [graph] [full]            (1 rank)
    python -m torch.distributed.run --nproc-per-node N ... tests/tp_worker.py OUT.pt ROWS [graph] [full]

graph: the pass is captured once in a CUDA graph and replayed (what a decode loop does: the in-kernel exchanges and
the pass counter's increment are part of the graph).  full: the benchmark's own sizes (hidden 5120, FFN 17408, 4 layers).
"""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from prism_b200 import _lib, linear_stack as LS, tp  # noqa: E402

HID, QC, KVC, FFN, LAYERS = 1024, 1024, 256, 2048, 2


def main():
    global HID, QC, KVC, FFN, LAYERS
    out, rows = sys.argv[1], int(sys.argv[2])
    if "full" in sys.argv[3:]:
        HID, QC, KVC, FFN, LAYERS = LS.HIDDEN, LS.Q_COLS, LS.KV_COLS, LS.FFN, 4
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    group = tp.Group(rank, world, backend="nccl", local_rank=local) if world > 1 else None
    layers = [LS.shard_layer(LS.make_layer_weights(i, dev, HID, QC, KVC, FFN), world, rank, HID, QC, KVC, FFN)
              for i in range(LAYERS)]
    stack = LS.LinearStack(layers, rows, dev, group, HID, QC, KVC, FFN)
    h0 = torch.randn(rows, HID, generator=torch.Generator(device=dev).manual_seed(3), device=dev)
    for _ in range(2):                       # twice: the second pass must give the same bits (no state between passes)
        h = stack(h0).clone()
    torch.cuda.synchronize()
    if "graph" in sys.argv[3:]:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            res = stack(h0)
        for _ in range(3):
            res.zero_()
            graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(res, h), "a replayed pass differs from the eager one"
        h = res.clone()
        del graph
    code, where = _lib.device_status()
    assert code == 0, (code, where)
    if rank == 0:
        torch.save(h.cpu(), out)
    if group is not None:
        group.barrier()
        stack.close()
        group.close()


if __name__ == "__main__":
    main()
