"""CUDA-graph capture of the fused operator (the reference registers and IPC-maps captured inputs,
src/ops/all_reduce_fusion.cpp:105-137,168-233; here a captured call needs nothing of the kind).

The operator is captured once on a side stream and replayed on new data written into the same
buffers; results must follow the data.  The kernels are programmatic dependent launches, which
stream capture records as such.  Collected late on purpose (new launch attributes are involved).
"""
import pytest
import torch

pytestmark = pytest.mark.gpu

from oracle import epilogue_oracle as eo   # noqa: E402
from tests import util                     # noqa: E402


@pytest.mark.parametrize("tokens,hidden,quant", [(8, 8192, 3), (2400, 1024, 3), (64, 4096, 0)])
def test_replayed_graph_follows_new_data_on_one_gpu(tokens, hidden, quant):
    import gpuk_b200
    parts, res, w = util.random_case(1, tokens, hidden, torch.bfloat16, seed=tokens)
    x, r, g = parts[0].cuda(), res.cuda(), w.cuda()
    res_out, norm_out, scale = util.alloc_outputs(x, quant)

    def call():
        gpuk_b200.allreduce_rms(0, x, r, g, res_out, norm_out, scale, 1e-6, quant)

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        call()
        call()      # two calls in the graph: the second depends on the first programmatically
        torch.cuda.synchronize()
        with torch.cuda.graph(graph, stream=side):
            call()
            call()
    torch.cuda.current_stream().wait_stream(side)
    for rep in range(3):
        parts, res, _ = util.random_case(1, tokens, hidden, torch.bfloat16, seed=1000 + rep)
        x.copy_(parts[0])
        r.copy_(res)
        graph.replay()
        torch.cuda.synchronize()
        want = eo.add_rms_quant(parts[0], res, w, 1e-6, quant)
        util.check_against_oracle((res_out.cpu(), norm_out.cpu(), scale.cpu() if quant else None), want, quant)
