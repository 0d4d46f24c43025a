"""The CPU oracle against (a) fixtures produced by the reference's own TransformerMLP and (b) itself in numpy."""
import zlib

import numpy as np
import pytest
import torch

from oracle import (TOL_FROB, TOL_MAX_NORM, error_metrics, from_bits, make_inputs, swiglu_gold, swiglu_gold_numpy,
                    swiglu_ref_eager, to_bits)
from oracle.swiglu_oracle import _load

CASES = ["tiny_48x128x96", "ragged_37x200x72", "mid_130x512x264", "cfg1_256x1024x2816"]


def _inputs(golden, name):
    M, K, N, seed, step = (int(v) for v in golden[name + "/shape"])
    if name + "/x" in golden.files:
        x, w = from_bits(golden[name + "/x"]), from_bits(golden[name + "/w"])
    else:
        x, w = make_inputs(M, K, N, seed=seed)
    crc = [zlib.crc32(to_bits(x).tobytes()), zlib.crc32(to_bits(w).tobytes())]
    assert crc == [int(v) for v in golden[name + "/crc"]], "seeded inputs differ from the ones the fixture was made with"
    return x, w, step


def test_bf16_conversion_known_answers():
    lib = _load()
    # value -> bf16 bits (round to nearest even, ties, carries into the exponent, specials)
    kat = [(0.0, 0x0000), (1.0, 0x3F80), (-2.0, 0xC000), (1.00390625, 0x3F80), (1.01171875, 0x3F82),
           (1.005859375, 0x3F81), (3.3895313892515355e38, 0x7F7F), (float("inf"), 0x7F80), (65504.0, 0x4780)]
    for v, bits in kat:
        assert lib.oracle_f32_to_bf16(v) == bits, (v, hex(lib.oracle_f32_to_bf16(v)))
        assert lib.oracle_f32_to_bf16(v) == int(to_bits(torch.tensor([v], dtype=torch.float32).to(torch.bfloat16))[0])
    r = torch.randn(4096, dtype=torch.float32) * 37.0
    got = np.array([lib.oracle_f32_to_bf16(float(v)) for v in r], dtype=np.uint16)
    assert np.array_equal(got, to_bits(r.to(torch.bfloat16)))
    assert lib.oracle_bf16_to_f32(0x3FC0) == 1.5


@pytest.mark.parametrize("name", CASES)
def test_oracle_eager_chain_matches_reference_fixture(golden, name):
    """The oracle's restatement of the reference's rounding chain reproduces what the reference itself printed:
    bit-exact except where the fp32 summation order of the two GEMM back-ends flips a bf16 rounding."""
    x, w, step = _inputs(golden, name)
    ref = from_bits(golden[name + "/y_eager"])
    got = swiglu_gold(x, w)["eager"][::step]
    mismatch = float((to_bits(got) != to_bits(ref)).mean())
    assert mismatch <= 1e-3, mismatch
    m = error_metrics(got, ref.float())
    assert m["max_norm"] <= 4e-3 and m["frob"] <= 1e-4, m  # differing elements are one bf16 step apart


@pytest.mark.parametrize("name", CASES)
def test_reference_fixture_within_tolerance_of_gold(golden, name):
    """The tolerance of the path is wide enough for the reference's own eager result and tight enough to
    separate a single-rounded result from it."""
    x, w, step = _inputs(golden, name)
    o = swiglu_gold(x, w)
    ref = from_bits(golden[name + "/y_eager"])
    m_ref = error_metrics(ref, o["gold"][::step])
    m_one = error_metrics(o["gold_bf16"], o["gold"])
    assert m_ref["max_norm"] <= TOL_MAX_NORM and m_ref["frob"] <= TOL_FROB, m_ref
    assert m_one["max_norm"] <= 4e-3 and m_one["frob"] <= 2.5e-3, m_one
    assert m_one["frob"] < m_ref["frob"]


@pytest.mark.parametrize("shape", [(1, 8, 8), (5, 24, 16), (33, 136, 40), (64, 1024, 64)])
def test_c_oracle_matches_numpy_restatement(shape):
    M, K, N = shape
    x, w = make_inputs(M, K, N, seed=11)
    o = swiglu_gold(x, w, threads=3)
    m = error_metrics(swiglu_gold_numpy(x, w), o["gold"])
    assert m["max_norm"] < 5e-6 and m["frob"] < 5e-6, m
    # threading must not change a single bit
    o1 = swiglu_gold(x, w, threads=1)
    assert torch.equal(o1["gold"], o["gold"]) and torch.equal(o1["eager"], o["eager"])


def test_eager_port_is_the_reference_expression():
    """swiglu_ref_eager (timed as the CPU baseline) agrees with the oracle's eager chain on the same inputs."""
    x, w = make_inputs(96, 256, 128, seed=5)
    got = swiglu_ref_eager(x, w)
    exp = swiglu_gold(x, w)["eager"]
    assert got.dtype == torch.bfloat16
    assert float((to_bits(got) != to_bits(exp)).mean()) <= 1e-3


def test_oracle_edge_cases():
    # empty M is a no-op, zero inputs give zero, huge negative gate gives -0/0 without NaN
    x, w = make_inputs(4, 16, 8, seed=1)
    assert swiglu_gold(x[:0], w)["gold"].shape == (0, 8)
    z = swiglu_gold(torch.zeros_like(x), w)
    assert torch.count_nonzero(z["gold"]) == 0 and torch.count_nonzero(z["eager"].float()) == 0
    xb = torch.full((2, 16), 300.0, dtype=torch.bfloat16)
    wb = torch.cat([torch.full((8, 16), -100.0), torch.ones(8, 16)]).to(torch.bfloat16)
    o = swiglu_gold(xb, wb)
    assert torch.isfinite(o["gold"]).all() and (o["gold"].abs() == 0).all()


def test_rmsnorm_oracle_matches_reference_fixture(golden):
    """RMSNorm -> gate/up SwiGLU: the oracle's restatement of the reference's eager chain reproduces what the
    reference's RMSNorm and TransformerMLP modules produced, and the fp32 gold sits within the path's tolerance."""
    from oracle import rmsnorm_swiglu_gold, rmsnorm_swiglu_ref_eager

    name = "rms_96x256x136"
    x, w = from_bits(golden[name + "/x"]), from_bits(golden[name + "/w"])
    gamma = torch.from_numpy(golden[name + "/gamma"])
    eps = float(golden[name + "/eps"][0])
    ref = from_bits(golden[name + "/y_eager"])
    got = rmsnorm_swiglu_ref_eager(x, gamma, w, eps)
    assert float((to_bits(got) != to_bits(ref)).mean()) <= 1e-3
    m = error_metrics(ref, rmsnorm_swiglu_gold(x, gamma, w, eps))
    assert m["max_norm"] <= TOL_MAX_NORM and m["frob"] <= TOL_FROB, m


def test_nvfp4_gold_rounding_table_and_layout():
    """Known answers of the e2m1 grid (round to nearest, ties to the even code, saturation at 6) and the 128 x 4
    tiled scale layout (a bijection onto a buffer of padded size)."""
    from oracle import e2m1_round, nvfp4_quantize_gold, nvfp4_swizzled_offsets

    q = torch.tensor([0.0, 0.25, 0.26, 0.5, 0.75, 1.0, 1.25, 1.26, 1.75, 2.5, 2.6, 3.5, 5.0, 5.1, 100.0, -0.3, -7.0])
    assert e2m1_round(q).tolist() == [0, 0, 1, 1, 2, 2, 2, 3, 4, 4, 5, 6, 6, 7, 7, 9, 15]
    y = torch.zeros(4, 32)
    y[0, :16] = torch.linspace(-6, 6, 16)
    y[1, 16:] = 3.0
    codes, sf, deq = nvfp4_quantize_gold(y, 1.0)
    assert sf.float().tolist() == [[1.0, 0.0], [0.0, 0.5], [0.0, 0.0], [0.0, 0.0]]
    assert (codes[2:] == 0).all() and (codes[1, 16:] == 7).all() and torch.equal(deq[1, 16:], torch.full((16,), 3.0))
    assert codes[0, 0] == 15 and codes[0, 15] == 7
    for M, N in ((1, 16), (130, 208), (256, 2816)):
        off = nvfp4_swizzled_offsets(M, N)
        size = -(-M // 128) * 128 * -(-(N // 16) // 4) * 4
        assert off.unique().numel() == off.numel() and 0 <= off.min() and off.max() < size
    assert nvfp4_swizzled_offsets(256, 128)[33, 5].item() == (0 * 2 + 1) * 512 + 1 * 16 + 1 * 4 + 1
