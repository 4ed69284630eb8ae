"""The few-row pass with every kernel launched as a programmatic dependent of the one before it (pb_set_pdl) against
the same pass with plain launches: the same bits, eagerly and as a replayed CUDA graph.  The chain's kernels begin
before their predecessor has ended; each reads its predecessor's output only after it has (griddepcontrol.wait)."""
import pytest
import torch

pytestmark = pytest.mark.gpu

HID, QC, KVC, FFN = 1024, 1024, 256, 2816


def build(M, dev, pdl):
    from prism_b200 import linear_stack as LS
    layers = [LS.shard_layer(LS.make_layer_weights(i, dev, HID, QC, KVC, FFN), 1, 0, HID, QC, KVC, FFN)
              for i in range(3)]
    stack = LS.LinearStack(layers, M, dev, None, HID, QC, KVC, FFN)
    stack.pdl = pdl
    return stack


@pytest.mark.parametrize("M", [1, 5, 16, 64])
def test_chain_of_programmatic_dependents(M):
    from prism_b200 import _lib
    dev = torch.device("cuda:0")
    h0 = (torch.randn(M, HID, generator=torch.Generator().manual_seed(M)) * 0.5).to(dev)
    plain, chained = build(M, dev, False), build(M, dev, True)
    want = plain(h0).clone()
    for _ in range(3):
        got = chained(h0).clone()
        assert torch.equal(got.view(torch.int32), want.view(torch.int32))
    assert _lib.lib().pb_set_pdl(0) == 0                   # the switch was put back after each pass
    # as a replayed graph: capture keeps the programmatic edges
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        chained(h0)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            out = chained(h0)
        for _ in range(5):
            out.zero_()
            graph.replay()
        side.synchronize()
        assert torch.equal(out.view(torch.int32), want.view(torch.int32))
    code, where = _lib.device_status()
    assert code == 0, (code, hex(where))
