"""The registered op in the situations MagiCompiler puts a split-point op in: eager dispatch, dynamo with a
dynamic row count, a side stream, CUDA-graph capture and replay, and the tensor-parallel MLP wrapper."""
import pytest
import torch

import magicompiler_b200 as mb
from magicompiler_b200.sharding import reference_mlp
from oracle import make_inputs

pytestmark = pytest.mark.gpu


def _inputs(M=256, K=512, N=384, seed=0):
    x, w = make_inputs(M, K, N, seed=seed)
    return x.cuda(), w.cuda()


def test_dispatcher_entry_equals_python_entry():
    x, w = _inputs()
    assert torch.equal(torch.ops.magi_swiglu.gemm_swiglu(x, w), mb.gemm_swiglu_out(x, w))


def test_torch_compile_dynamic_rows():
    torch._dynamo.reset()
    w = _inputs()[1]

    def f(x, w):
        return mb.gemm_swiglu(x * 1.0, w) + 0.0

    cf = torch.compile(f, backend="eager", fullgraph=True, dynamic=True)
    for rows in (64, 200, 129):
        x = _inputs(M=rows, seed=rows)[0]
        assert torch.equal(cf(x, w), f(x, w))


def test_side_stream_and_graph_capture():
    """Warm-up on a side stream, capture, replay with new contents in the static input
    (the sequence of magi_compiler/magi_backend/cuda_graph_mgr.py:465-473 and 548-581)."""
    x, w = _inputs(M=300)
    static_x = x.clone()
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        warm = mb.gemm_swiglu(static_x, w)
    torch.cuda.current_stream().wait_stream(s)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        static_y = mb.gemm_swiglu(static_x, w)
    g.replay()
    torch.cuda.synchronize()
    assert torch.equal(static_y, warm)
    x2 = _inputs(M=300, seed=9)[0]
    static_x.copy_(x2)
    g.replay()
    torch.cuda.synchronize()
    assert torch.equal(static_y, mb.gemm_swiglu(x2, w))


def test_tensor_parallel_mlp_single_rank():
    x, w, wd = make_inputs(512, 256, 384, seed=2, with_down=True)
    x, w, wd = x.cuda(), w.cuda(), wd.cuda()
    mlp = mb.TensorParallelSwiGLUMLP(w, wd, chunks=2)
    got = mlp(x)
    ref = reference_mlp(x, w, wd)
    assert torch.allclose(got.float(), ref.float(), rtol=2e-2, atol=2e-2 * ref.float().abs().max().item())


def test_rewrite_pass_on_gpu_matches_eager_module():
    """An unmodified gate/up/down MLP (the reference's TransformerMLP structure) compiled with the rewrite pass runs
    the fused kernel and matches its own eager execution; the packed weight is built once."""
    import torch.nn.functional as F

    from magicompiler_b200.passes import FuseSwiGLUPass, _pack_cache, clear_pack_cache

    class MLP(torch.nn.Module):
        def __init__(self, k=512, n=1024):
            super().__init__()
            self.gate_proj = torch.nn.Linear(k, n, bias=False, dtype=torch.bfloat16, device="cuda")
            self.up_proj = torch.nn.Linear(k, n, bias=False, dtype=torch.bfloat16, device="cuda")
            self.down_proj = torch.nn.Linear(n, k, bias=False, dtype=torch.bfloat16, device="cuda")

        def forward(self, x):
            return self.down_proj(F.silu(self.gate_proj(x)) * self.up_proj(x))

    counts = []

    def backend(gm, example_inputs):
        counts.append(FuseSwiGLUPass()(gm.graph))
        gm.recompile()
        return gm.forward

    torch.manual_seed(0)
    clear_pack_cache()
    torch._dynamo.reset()
    m = MLP().requires_grad_(False)
    cm = torch.compile(m, backend=backend, fullgraph=True, dynamic=True)
    for rows in (300, 77):
        x = torch.randn(rows, 512, device="cuda").to(torch.bfloat16)
        got, ref = cm(x), m(x)
        assert torch.allclose(got.float(), ref.float(), rtol=2e-2, atol=2e-2 * ref.float().abs().max().item())
    assert counts == [1] and len(_pack_cache) == 1
