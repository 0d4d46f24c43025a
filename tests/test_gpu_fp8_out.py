"""The fp8 (e4m3) output epilogue against the oracle: the kernel rounds the fp32 accumulators ONCE to fp8, so its
bytes must equal ``(gold / scale).to(float8_e4m3fn)`` except where the fp32 values themselves differ in the last
bits right at a rounding boundary.  Mirrors the contract of vLLM's ``silu_and_mul_quant(result, input, scale)``,
the op MagiCompiler's de-functionalisation pass handles
(magi_compiler/passes/piecewise_graph/fix_functionalization.py:110-112): static per-tensor scale, saturating."""
import pytest
import torch

import magicompiler_b200 as mb
from oracle import make_inputs, swiglu_gold

pytestmark = pytest.mark.gpu

FP8_MAX = 448.0


def _quant_ref(gold: torch.Tensor, scale: float) -> torch.Tensor:
    return (gold.float() * (1.0 / scale)).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)


def _step(v: torch.Tensor) -> torch.Tensor:
    """Spacing of e4m3 around |v| (3 mantissa bits; subnormal spacing 2^-9 below 2^-6)."""
    e = torch.floor(torch.log2(v.abs().clamp_min(2.0 ** -6)))
    return torch.exp2(e - 3)


def _compare(y8: torch.Tensor, ref8: torch.Tensor, min_equal: float):
    assert y8.dtype == torch.float8_e4m3fn and y8.shape == ref8.shape
    a, b = y8.float().cpu(), ref8.float().cpu()
    assert torch.isfinite(a).all()
    equal = (y8.cpu().view(torch.uint8) == ref8.cpu().view(torch.uint8)) | ((a == 0) & (b == 0))
    assert equal.float().mean().item() >= min_equal, equal.float().mean().item()
    assert ((a - b).abs() <= _step(torch.maximum(a.abs(), b.abs())) * 1.001).all()


@pytest.mark.parametrize("M,K,N", [(256, 1024, 2816), (64, 1024, 2816), (130, 264, 208), (1, 64, 16), (300, 512, 400),
                                   (1024, 512, 4096)])
def test_fp8_output_matches_single_rounded_gold(M, K, N):
    x, w = make_inputs(M, K, N, seed=M + N)
    gold = swiglu_gold(x, w, want_eager=False)["gold"]
    scale = gold.abs().max().item() / 200.0  # the data uses about half of the e4m3 range
    s = torch.tensor([scale], dtype=torch.float32, device="cuda")
    y8 = mb.gemm_swiglu_fp8(x.cuda(), w.cuda(), s)
    assert y8.shape == (M, N)
    _compare(y8, _quant_ref(gold, scale), min_equal=0.995)


def test_fp8_output_saturates_without_nan():
    x, w = make_inputs(192, 512, 256, seed=5)
    gold = swiglu_gold(x, w, want_eager=False)["gold"]
    scale = gold.abs().max().item() / 4000.0  # the largest values land near 9x the e4m3 maximum
    s = torch.tensor([scale], dtype=torch.float32, device="cuda")
    y8 = mb.gemm_swiglu_fp8(x.cuda(), w.cuda(), s)
    ref = _quant_ref(gold, scale)
    assert (ref.float().abs() == FP8_MAX).any()
    _compare(y8, ref, min_equal=0.995)
    assert y8.float().abs().max().item() == FP8_MAX


def test_fp8_output_full_size_against_the_bf16_path():
    """Llama-3-8B FFN shape: the bf16 output of the same kernels, quantised by torch, differs from the fused fp8
    output only by double rounding (bf16 then fp8): never more than one fp8 step, and on a few percent of elements."""
    M, K, N = 8192, 4096, 14336
    g = torch.Generator(device="cuda")
    g.manual_seed(11)
    x = torch.randn(M, K, generator=g, device="cuda", dtype=torch.float32).to(torch.bfloat16)
    w = (torch.randn(2 * N, K, generator=g, device="cuda", dtype=torch.float32) * 0.02).to(torch.bfloat16)
    y = mb.gemm_swiglu(x, w)
    scale = y.float().abs().max().item() / 300.0
    s = torch.tensor([scale], dtype=torch.float32, device="cuda")
    y8 = mb.gemm_swiglu_fp8(x, w, s)
    ref = (y.float() * (1.0 / scale)).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)
    a, b = y8.float(), ref.float()
    same = (y8.view(torch.uint8) == ref.view(torch.uint8)) | ((a == 0) & (b == 0))
    assert same.float().mean().item() >= 0.93
    assert ((a - b).abs() <= _step(torch.maximum(a.abs(), b.abs())) * 1.001).all()


def test_fp8_leading_dimensions_graph_capture_and_errors():
    x, w = make_inputs(6 * 50, 256, 192, seed=3)
    x, w = x.cuda().view(6, 50, 256), w.cuda()
    s = torch.tensor([0.01], dtype=torch.float32, device="cuda")
    y8 = torch.ops.magi_swiglu.gemm_swiglu_fp8(x, w, s)
    assert y8.shape == (6, 50, 192)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        y_graph = mb.gemm_swiglu_fp8(x, w, s)
    s.fill_(0.02)  # the scale is read on the device at run time: a replay sees the new value
    g.replay()
    torch.cuda.synchronize()
    assert torch.equal(y_graph.view(torch.uint8), mb.gemm_swiglu_fp8(x, w, s).view(torch.uint8))
    assert not torch.equal(y_graph.view(torch.uint8), y8.view(torch.uint8))
    with pytest.raises(ValueError):
        mb.gemm_swiglu_fp8(x, w[: 2 * 184], s)  # N = 184 is not a multiple of 16
    with pytest.raises(TypeError):
        mb.gemm_swiglu_fp8(x, w, s.double())
    with pytest.raises(ValueError):
        mb.gemm_swiglu_fp8(x, w, s.cpu())


def test_fp8_output_against_vllm_silu_and_mul_quant():
    """The op the reference's pass names, run for real when vLLM's compiled ops are present: it quantises the
    bf16-rounded projections (and rounds the activation to bf16 before scaling), the fused kernel rounds once from
    fp32, so a few percent of the bytes differ by one fp8 step and none by more."""
    try:
        import vllm._C  # noqa: F401
    except Exception as exc:  # not installed, or built without this device
        pytest.skip(f"vLLM compiled ops unavailable: {exc}")
    if not hasattr(torch.ops._C, "silu_and_mul_quant"):
        pytest.skip("this vLLM build has no silu_and_mul_quant")
    for M, K, N in ((256, 512, 384), (1000, 1024, 2816)):
        x, w = make_inputs(M, K, N, seed=N)
        x, w = x.cuda(), w.cuda()
        h = mb.gemm_nt(x, w)  # [M, 2N] bf16 = the merged gate/up linear's output
        scale = torch.tensor([mb.gemm_swiglu(x, w).float().abs().max().item() / 300.0], dtype=torch.float32,
                             device="cuda")
        ref = torch.empty(M, N, dtype=torch.float8_e4m3fn, device="cuda")
        torch.ops._C.silu_and_mul_quant(ref, h, scale)
        y8 = mb.gemm_swiglu_fp8(x, w, scale)
        a, b = y8.float(), ref.float()
        same = (y8.view(torch.uint8) == ref.view(torch.uint8)) | ((a == 0) & (b == 0))
        assert same.float().mean().item() >= 0.93, same.float().mean().item()
        assert ((a - b).abs() <= _step(torch.maximum(a.abs(), b.abs())) * 1.001).all()
