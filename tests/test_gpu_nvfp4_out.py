"""The nvfp4 output epilogue against the oracle's restatement of the block-scaled quantisation
(``oracle.nvfp4_quantize_gold`` on the fp32 gold): scale bytes and 4-bit codes must agree except where fp32 noise in
the accumulators sits right on a rounding boundary; the dequantised output approximates the gold as well as the
format allows.  Contract of vLLM's ``silu_and_mul_nvfp4_quant`` as MagiCompiler's de-functionalisation pass sees it
(magi_compiler/passes/piecewise_graph/fix_functionalization.py:113-120)."""
import pytest
import torch

import magicompiler_b200 as mb
from oracle import make_inputs, nvfp4_quantize_gold, nvfp4_swizzled_offsets, swiglu_gold

pytestmark = pytest.mark.gpu


def _unpack(codes_packed: torch.Tensor) -> torch.Tensor:
    p = codes_packed.cpu()
    return torch.stack([p & 0xF, p >> 4], dim=-1).reshape(p.shape[0], -1)  # even column in the low nibble


def _same_code(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    return (a == b) | (((a & 7) == 0) & ((b & 7) == 0))  # +0 and -0 are the same value


@pytest.mark.parametrize("M,K,N", [(256, 1024, 2816), (64, 1024, 2816), (130, 264, 208), (1, 64, 16), (300, 512, 400),
                                   (1000, 512, 4096)])
@pytest.mark.parametrize("swizzled", [False, True])
def test_nvfp4_output_matches_the_gold_quantisation(M, K, N, swizzled):
    x, w = make_inputs(M, K, N, seed=M + N)
    gold = swiglu_gold(x, w, want_eager=False)["gold"]
    gs = 448.0 * 6.0 / gold.abs().max().item()
    ref_codes, ref_sf, ref_deq = nvfp4_quantize_gold(gold, gs)
    gsd = torch.tensor([gs], dtype=torch.float32, device="cuda")
    codes, sf = mb.gemm_swiglu_nvfp4(x.cuda(), w.cuda(), gsd, swizzled)
    assert codes.shape == (M, N // 2) and codes.dtype == torch.uint8 and sf.dtype == torch.float8_e4m3fn
    assert tuple(sf.shape) == mb.nvfp4_scale_shape(M, N, swizzled)
    sf_bytes = sf.cpu().view(torch.uint8)
    if swizzled:
        off = nvfp4_swizzled_offsets(M, N)
        untouched = torch.ones(sf_bytes.numel(), dtype=torch.bool)
        untouched[off.reshape(-1)] = False
        assert (sf_bytes[untouched] == 0).all()  # padding of the tiled layout stays zero
        sf_bytes = sf_bytes[off]
    ref_sf_bytes = ref_sf.view(torch.uint8)
    same_sf = sf_bytes == ref_sf_bytes
    assert same_sf.float().mean().item() >= 0.999
    # a scale byte that differs is a neighbouring e4m3 value
    assert ((sf_bytes.int() - ref_sf_bytes.int()).abs() <= 1).all()
    got = _unpack(codes)
    in_same_block = same_sf.repeat_interleave(16, dim=1)
    agree = _same_code(got, ref_codes)[in_same_block]
    assert agree.float().mean().item() >= 0.995, agree.float().mean().item()
    # dequantised output against the fp32 gold: as close as the reference quantisation of the gold itself
    mag = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])[(got & 7).long()]
    val = torch.where((got & 8) != 0, -mag, mag)
    deq = val * (sf_bytes.view(torch.float8_e4m3fn).float() / gs).repeat_interleave(16, dim=1)
    err = ((deq - gold).norm() / gold.norm()).item()
    ref_err = ((ref_deq - gold).norm() / gold.norm()).item()
    assert err <= ref_err * 1.01 + 1e-6, (err, ref_err)


def test_nvfp4_zero_rows_saturation_and_errors():
    x, w = make_inputs(64, 128, 64, seed=2)
    x[:8] = 0  # all-zero blocks: scale 0, codes 0
    gold = swiglu_gold(x, w, want_eager=False)["gold"]
    gs = 448.0 * 6.0 / gold.abs().max().item() * 8.0  # scale factors above the e4m3 range saturate at 448
    gsd = torch.tensor([gs], dtype=torch.float32, device="cuda")
    codes, sf = mb.gemm_swiglu_nvfp4(x.cuda(), w.cuda(), gsd, False)
    assert (codes[:8] == 0).all() and (sf[:8].view(torch.uint8) == 0).all()
    assert sf.float().max().item() == 448.0 and torch.isfinite(sf.float()).all()
    ref_codes, ref_sf, _ = nvfp4_quantize_gold(gold, gs)
    assert (_same_code(_unpack(codes), ref_codes).float().mean().item()) >= 0.99
    with pytest.raises(ValueError):
        mb.gemm_swiglu_nvfp4(x.cuda(), w.cuda()[: 2 * 56], gsd, False)  # N = 56
    with pytest.raises(TypeError):
        mb.gemm_swiglu_nvfp4(x.cuda(), w.cuda(), gsd.double(), False)


def test_nvfp4_full_size_runs_in_every_tile_and_matches_the_bf16_path():
    """Llama-3-8B FFN shape: dequantised nvfp4 output against the bf16 output of the same kernels."""
    M, K, N = 8192, 4096, 14336
    g = torch.Generator(device="cuda")
    g.manual_seed(5)
    x = torch.randn(M, K, generator=g, device="cuda", dtype=torch.float32).to(torch.bfloat16)
    w = (torch.randn(2 * N, K, generator=g, device="cuda", dtype=torch.float32) * 0.02).to(torch.bfloat16)
    y = mb.gemm_swiglu(x, w).float()
    gs = 448.0 * 6.0 / y.abs().max().item()
    codes, sf = mb.gemm_swiglu_nvfp4(x, w, torch.tensor([gs], dtype=torch.float32, device="cuda"), False)
    lut = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0],
                       device="cuda")
    val = torch.stack([lut[(codes & 0xF).long()], lut[(codes >> 4).long()]], dim=-1).reshape(M, N)
    deq = val * (sf.float() / gs).repeat_interleave(16, dim=1)
    rel = ((deq - y).norm() / y.norm()).item()
    assert rel <= 0.12, rel
    # every block's largest magnitude maps to a code of at least 4 (|q| in (3.5, 6]) unless the block is all zero
    blk = (val.abs().reshape(M, N // 16, 16).amax(dim=-1))
    assert ((blk >= 4.0) | (sf.float() == 0)).float().mean().item() >= 0.999


def test_nvfp4_output_against_vllm_silu_and_mul_nvfp4_quant():
    """The op the reference's pass names (fix_functionalization.py:113-120), run for real when vLLM's compiled ops are
    present: vLLM quantises the bf16-rounded projections and rounds the activation to bf16 before scaling, the fused
    kernel quantises its fp32 accumulators directly, so most scale bytes and codes are identical and the rest are
    neighbours.  Scales are compared in vLLM's own layout (128 x 4 tiles, int32-packed)."""
    try:
        import vllm._custom_ops  # noqa: F401  (loads every compiled extension vLLM ships, the nvfp4 ops among them)
    except Exception as exc:  # not installed, or built without this device
        pytest.skip(f"vLLM compiled ops unavailable: {exc}")
    if not hasattr(torch.ops._C, "silu_and_mul_nvfp4_quant"):
        pytest.skip("this vLLM build has no silu_and_mul_nvfp4_quant")
    for M, K, N in ((256, 512, 384), (1000, 1024, 2816), (128, 256, 64)):
        x, w = make_inputs(M, K, N, seed=N + 1)
        x, w = x.cuda(), w.cuda()
        h = mb.gemm_nt(x, w)  # [M, 2N] bf16 = the merged gate/up linear's output
        gs = torch.tensor([448.0 * 6.0 / mb.gemm_swiglu(x, w).float().abs().max().item()], dtype=torch.float32,
                          device="cuda")
        rows_pad, blocks_pad = -(-M // 128) * 128, -(-(N // 16) // 4) * 4
        ref_codes = torch.empty(M, N // 2, dtype=torch.uint8, device="cuda")
        ref_sf = torch.zeros(rows_pad, blocks_pad // 4, dtype=torch.int32, device="cuda")
        torch.ops._C.silu_and_mul_nvfp4_quant(ref_codes, ref_sf, h, gs)
        codes, sf = mb.gemm_swiglu_nvfp4(x, w, gs, True)
        torch.cuda.synchronize()
        off = nvfp4_swizzled_offsets(M, N)  # where the scale of (row, block) sits in the tiled layout
        ours = sf.cpu().view(torch.uint8)[off]
        theirs = ref_sf.cpu().view(torch.uint8).reshape(-1)[off]
        same_sf = ours == theirs
        assert same_sf.float().mean().item() >= 0.97, same_sf.float().mean().item()
        assert ((ours.int() - theirs.int()).abs() <= 1).all()  # a differing scale is the neighbouring e4m3 value
        got, ref = _unpack(codes), _unpack(ref_codes)
        in_same_block = same_sf.repeat_interleave(16, dim=1)
        agree = _same_code(got, ref)[in_same_block]
        assert agree.float().mean().item() >= 0.93, agree.float().mean().item()
        # codes that differ are neighbours on the e2m1 grid
        lut = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])
        va = torch.where((got & 8) != 0, -lut[(got & 7).long()], lut[(got & 7).long()])
        vb = torch.where((ref & 8) != 0, -lut[(ref & 7).long()], lut[(ref & 7).long()])
        idx_a = torch.bucketize(va, torch.tensor([-6.0, -4.0, -3.0, -2.0, -1.5, -1.0, -0.5, 0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]))
        idx_b = torch.bucketize(vb, torch.tensor([-6.0, -4.0, -3.0, -2.0, -1.5, -1.0, -0.5, 0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]))
        assert ((idx_a - idx_b).abs()[in_same_block] <= 1).all()
