"""The C-ABI library loads without a GPU, exports every symbol the header declares, plans schedules and
rejects bad arguments on the host (no launch)."""
import ctypes
import re
from pathlib import Path

import pytest

from magicompiler_b200 import _loader

ROOT = Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "magi_swiglu.h"


@pytest.fixture(scope="module")
def lib():
    _loader.build_library()
    return _loader.load_library()


def _declared_functions():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(magi_swiglu_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported(lib):
    names = _declared_functions()
    assert {"magi_swiglu_version", "magi_swiglu_supported", "magi_swiglu_forward_bf16", "magi_swiglu_forward_bf16_ex",
            "magi_swiglu_plan", "magi_swiglu_device_status", "magi_swiglu_kernel_clock", "magi_swiglu_last_error",
            "magi_swiglu_forward_bf16_ws", "magi_swiglu_workspace_bytes"} <= set(names)
    for n in names:
        assert hasattr(lib, n), n


def test_every_declaration_cites_what_it_replaces():
    text = HEADER.read_text()
    for n in _declared_functions():
        decl = re.search(r"^(?:int|int64_t|const char\*)\s+" + n + r"\(", text, re.M).start()
        comment = text[:decl].rsplit("/*", 1)[1]
        assert "Replaces:" in comment or "no counterpart in the reference" in comment, n


def test_version_matches_header(lib):
    v = int(re.search(r"#define MAGI_SWIGLU_ABI_VERSION (\d+)", HEADER.read_text()).group(1))
    assert lib.magi_swiglu_version() == v == _loader.ABI_VERSION


def test_supported_is_false_without_a_b200(lib):
    import torch

    if not torch.cuda.is_available():
        assert lib.magi_swiglu_supported(0) == 0
    assert lib.magi_swiglu_supported(-1) == 0 and lib.magi_swiglu_supported(1000) == 0


def test_plan_for_the_benchmark_configs():
    p = _loader.plan(8192, 14336, 4096, sm_count=148)  # Llama-3-8B FFN: CTA pairs, 256-row tiles
    assert p["variant"] == _loader.VARIANT_MMA2 and p["ctas"] == 2 and p["grid"] == 148 and p["block_n"] % 16 == 0
    assert p["tiles"] == -(-8192 // 256) * -(-14336 // p["block_n"])
    assert p["smem_bytes"] <= 232448 and p["stages"] >= 3
    p = _loader.plan(32760, 13824, 5120, sm_count=148)  # video-DiT FFN, ragged M
    assert p["variant"] == _loader.VARIANT_MMA2 and p["tiles"] == 128 * -(-13824 // p["block_n"])
    p = _loader.plan(32760, 1728, 5120, sm_count=148)  # its 8-GPU column shard: little padding, whole waves
    padded = -(-1728 // p["block_n"]) * p["block_n"]
    assert padded <= 1728 * 1.05 and p["tiles"] == 128 * (padded // p["block_n"])
    for M in (16, 64, 128):  # decode shapes: one slab of W per SM, a single wave
        p = _loader.plan(M, 28672, 8192, sm_count=148)
        assert p["variant"] == _loader.VARIANT_STREAM
        assert p["tiles"] == p["grid"] <= 148 and p["tiles"] * p["block_n"] >= 28672
        assert 2 * p["block_n"] <= 512
    p = _loader.plan(129, 2816, 1024, sm_count=148)
    assert p["variant"] == _loader.VARIANT_MMA2
    for shard in (14336, 7168, 3584):  # column shards of the decode weight at 2/4/8 GPUs
        p = _loader.plan(64, shard, 8192, sm_count=148)
        assert p["tiles"] <= 148 * 2


def test_plan_for_cta_pairs():
    p = _loader.plan(8192, 14336, 4096, variant="mma2", block_n=128, sm_count=148)
    assert p["ctas"] == 2 and p["grid"] == 148 and p["tiles"] == 32 * 112 and p["n_mma"] == 1 and p["acc_bufs"] == 2
    assert p["stages"] >= 6, "half the weight tile per CTA leaves room for a deeper ring"
    p1 = _loader.plan(8192, 14336, 4096, variant="mma", sm_count=148)
    assert p1["ctas"] == 1 and p["stages"] > p1["stages"]
    p = _loader.plan(32760, 13824, 5120, variant="mma2", block_n=128, sm_count=147)  # odd SM count: whole pairs only
    assert p["grid"] == 146 and p["tiles"] == 128 * 108
    p = _loader.plan(300, 528, 320, variant="mma2", block_n=256, sm_count=148)
    assert (p["n_mma"], p["acc_bufs"], p["tiles"]) == (2, 1, 2 * 3)
    with pytest.raises(ValueError):
        _loader.plan(300, 528, 320, variant="mma2", max_ctas=1, sm_count=148)


def test_plan_uses_single_cta_tiles_when_the_last_row_pair_is_half_empty():
    # M = 384 is three 128-row granules: CTA pairs would run four (two 256-row units), single CTAs run three.
    # That holds for whole-tile schedules (no scratch, or stream-K switched off) ...
    prev = _loader.set_tuning("stream_k", 0)
    try:
        for M in (288, 320, 384):
            p = _loader.plan(M, 28672, 8192, sm_count=148)
            assert p["variant"] == _loader.VARIANT_MMA and p["ctas"] == 1 and p["block_n"] <= 224 and p["stages"] >= 3
            assert p["tiles"] == 3 * -(-28672 // p["block_n"])
        # full units, or many of them: pairs stay
        for M in (256, 512, 640, 1024, 8192 + 128):
            assert _loader.plan(M, 28672, 8192, sm_count=148)["variant"] == _loader.VARIANT_MMA2
    finally:
        _loader.set_tuning("stream_k", prev)
    # ... with scratch the pairs' 224 tiles are balanced over the 74 pairs by K ranges, which beats both
    p = _loader.plan(384, 28672, 8192, sm_count=148)
    assert p["variant"] == _loader.VARIANT_MMA2 and p["sk_tiles"] > 0
    # an explicit width or variant is never overridden
    assert _loader.plan(384, 28672, 8192, block_n=256, sm_count=148)["variant"] == _loader.VARIANT_MMA2
    assert _loader.plan(384, 28672, 8192, variant="mma2", sm_count=148)["variant"] == _loader.VARIANT_MMA2


def test_plan_respects_explicit_knobs_and_rejects_bad_ones():
    p = _loader.plan(4096, 4096, 4096, variant="mma", block_n=64, stages=3, max_ctas=10, sm_count=148)
    assert (p["block_n"], p["stages"], p["grid"], p["acc_bufs"], p["n_mma"]) == (64, 3, 10, 2, 1)
    p = _loader.plan(4096, 4096, 4096, variant="mma", block_n=256, sm_count=148)
    assert (p["acc_bufs"], p["n_mma"]) == (1, 2)
    for bad in (dict(block_n=24), dict(block_n=272), dict(stages=1), dict(stages=13), dict(variant=9)):
        with pytest.raises(ValueError):
            _loader.plan(4096, 4096, 4096, sm_count=148, **{"variant": "mma", **bad})
    with pytest.raises(ValueError):
        _loader.plan(256, 4096, 4096, variant="stream", sm_count=148)  # STREAM is for M <= 128
    with pytest.raises(ValueError):
        _loader.plan(16, 100, 64, sm_count=148)  # N % 8
    with pytest.raises(ValueError):
        _loader.plan(16, 64, 100, sm_count=148)  # K % 8


def test_forward_rejects_bad_arguments_before_touching_a_device(lib):
    buf = (ctypes.c_char * 4096)()
    base = ctypes.addressof(buf)
    base += (-base) % 16
    fwd = lib.magi_swiglu_forward_bf16

    def call(x=base, w=base, y=base, M=8, N=8, K=8, ldx=8, ldw=8, ldy=8, dev=0, variant=0):
        return fwd(x, w, y, M, N, K, ldx, ldw, ldy, dev, None, variant)

    assert call(x=None) == -1 and "null" in _loader.last_error()
    assert call(ldx=4) == -2          # row stride shorter than K
    assert call(ldy=12) == -3         # stride not a multiple of 8 elements
    assert call(x=base + 2) == -3     # misaligned pointer
    assert call(M=0) == 0             # empty batch: successful no-op, nothing launched
    assert call(dev=1000) == -5 and "device" in _loader.last_error()
    import torch

    if not torch.cuda.is_available():
        assert call() == -5           # valid arguments, but no sm_100 device: refused, never a CPU fallback


def test_other_entry_points_reject_bad_arguments_on_the_host(lib):
    """fp8 / nvfp4 outputs, the training forward and the fused backward validate before any device is touched."""
    buf = (ctypes.c_char * 8192)()
    b = ctypes.addressof(buf)
    b += (-b) % 16
    fp8, fp4 = lib.magi_swiglu_forward_fp8_e4m3, lib.magi_swiglu_forward_nvfp4
    pre, bwd = lib.magi_swiglu_forward_bf16_preact, lib.magi_swiglu_backward_dh_bf16
    # fp8: scale pointer, N % 16, ldy % 16
    assert fp8(b, b, b, None, 8, 16, 8, 8, 8, 16, 0, None) == -1
    assert fp8(b, b, b, b, 8, 8, 8, 8, 8, 16, 0, None) == -2 and "multiples of 16" in _loader.last_error()
    assert fp8(b, b, b, b, 8, 16, 8, 8, 8, 24, 0, None) == -2
    assert fp8(b, b, b, b, 0, 16, 8, 8, 8, 16, 0, None) == 0  # empty batch
    # nvfp4: pointers, N % 16, row bytes, layout id, linear scale stride
    assert fp4(b, b, b, None, b, 8, 16, 8, 8, 8, 8, 1, 0, 0, None) == -1
    assert fp4(b, b, b, b, None, 8, 16, 8, 8, 8, 8, 1, 0, 0, None) == -1
    assert fp4(b, b, b, b, b, 8, 24, 8, 8, 8, 16, 2, 0, 0, None) == -2
    assert fp4(b, b, b, b, b, 8, 32, 8, 8, 8, 8, 2, 0, 0, None) == -2   # a row of 32 codes is 16 bytes
    assert fp4(b, b, b, b, b, 8, 32, 8, 8, 8, 16, 2, 7, 0, None) == -4 and "layout" in _loader.last_error()
    assert fp4(b, b, b, b, b, 8, 32, 8, 8, 8, 16, 1, 0, 0, None) == -2  # two blocks per row need ld_scale >= 2
    assert fp4(b, b, b, b, b, 8, 32, 8, 8, 8, 16, 2, 0, 1000, None) == -5
    # training forward: h pointer, width and alignment
    assert pre(b, b, b, None, 8, 8, 8, 8, 8, 8, 16, 0, None) == -1
    assert pre(b, b, b, b, 8, 8, 8, 8, 8, 8, 8, 0, None) == -2          # ldh < 2N
    assert pre(b, b, b, b + 8, 8, 8, 8, 8, 8, 8, 16, 0, None) == -3
    # fused backward: dy pointer, strides
    assert bwd(b, b, None, b, 8, 8, 8, 8, 8, 8, 16, 0, None) == -1
    assert bwd(b, b, b, b, 8, 8, 8, 8, 8, 4, 16, 0, None) == -2         # lddy < N
    assert bwd(b, b, b, b, 8, 8, 8, 8, 8, 8, 8, 0, None) == -2          # lddh < 2N
    assert bwd(b, b, b, b, 8, 8, 8, 8, 8, 12, 16, 0, None) == -3        # lddy % 8
    assert bwd(b, b, b, b, 8, 8, 8, 8, 8, 8, 16, 1000, None) == -5


def test_scatter_entry_points_reject_bad_arguments_on_the_host(lib):
    """The scattered down projection and the slot sum validate before any device is touched."""
    buf = (ctypes.c_char * 8192)()
    b = ctypes.addressof(buf)
    b += (-b) % 16
    setup, gemm, sums = lib.magi_swiglu_scatter_setup, lib.magi_swiglu_gemm_nt_bf16_scatter, lib.magi_swiglu_sum_slots_bf16
    dst = (ctypes.c_void_p * 9)(*([b] * 9))
    assert setup(0, 2, dst, 2, 64, 128, 128) == -4 and "set" in _loader.last_error()
    assert setup(0, 0, dst, 0, 64, 128, 128) == -2
    assert setup(0, 0, dst, 9, 64, 128, 128) == -2 and "owners" in _loader.last_error()
    assert setup(0, 0, None, 2, 64, 128, 128) == -1
    assert setup(0, 0, dst, 2, 48, 128, 128) == -2 and "multiple of 32" in _loader.last_error()
    assert setup(0, 0, dst, 2, 64, 96, 96) == -2       # N % 64
    assert setup(0, 0, dst, 2, 64, 128, 64) == -2      # ldc < N
    assert setup(1000, 0, dst, 2, 64, 128, 128) == -5
    assert gemm(b, b, 3, 128, 128, 64, 64, 64, 0, None, None, 0) == -4
    assert gemm(b, b, 0, 128, 128, 64, 64, 64, 1000, None, None, 0) == -5
    assert gemm(b, b, 0, 128, 128, 64, 64, 64, 0, None, None, 0) == -4 and "not been set up" in _loader.last_error()
    assert sums(None, b, 2, 64, 64, 0, None) == -1
    assert sums(b, b, 0, 64, 64, 0, None) == -2
    assert sums(b, b, 2, 64, 60, 0, None) == -2        # n % 8
    assert sums(b, b, 2, 32, 64, 0, None) == -2        # slots overlap
    assert sums(b + 8, b, 2, 64, 64, 0, None) == -3
    assert sums(b, b, 2, 64, 0, 0, None) == 0          # nothing to add
    assert sums(b, b, 2, 64, 64, 1000, None) == -5
    bcast = lib.magi_swiglu_sum_slots_bf16_bcast
    assert bcast(b, dst, 9, 2, 64, 64, 0, None) == -2 and "destinations" in _loader.last_error()
    assert bcast(b, dst, 0, 2, 64, 64, 0, None) == -2
    assert bcast(b, None, 2, 2, 64, 64, 0, None) == -1
    assert bcast(b, dst, 2, 2, 64, 60, 0, None) == -2
    assert bcast(b, dst, 8, 2, 64, 64, 1000, None) == -5


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(_loader, "_lib", None)
    monkeypatch.setattr(_loader, "LIB_PATH", tmp_path / "libmagi_swiglu.so")
    monkeypatch.delenv("MAGI_SWIGLU_AUTOBUILD", raising=False)
    with pytest.raises(_loader.MagiSwigluLibraryError):
        _loader.load_library()


def test_split_k_plans_and_workspace_sizes():
    # the full decode weight keeps one slab per SM and needs no scratch ...
    assert _loader.plan(64, 28672, 8192, sm_count=148)["k_splits"] == 1
    assert _loader.workspace_bytes(64, 28672, 8192, sm_count=148) == 0
    # ... its 8-GPU column shard is too narrow for that: CTAs share slabs and split K
    p = _loader.plan(64, 3584, 8192, sm_count=148)
    assert p["k_splits"] >= 2 and p["tiles"] * p["k_splits"] <= 148 and p["grid"] == p["tiles"] * p["k_splits"]
    need = _loader.workspace_bytes(64, 3584, 8192, sm_count=148)
    assert need == p["tiles"] * p["k_splits"] * 64 * 2 * p["block_n"] * 4  # fp32 partial sums, nothing else
    assert need <= 64 << 20
    # large-M schedules ask for scratch only to balance a last wave that would be at most a quarter full (stream-K):
    # one flag and one 256 KiB slab per CTA; a problem that fills its waves asks for none
    assert _loader.workspace_bytes(8192, 14336, 4096, sm_count=148) == 256 * 3 + 148 * (256 << 10)
    assert _loader.workspace_bytes(32760, 13824, 5120, sm_count=148) == 0      # 93.4 waves: the last one is 40 % full
    assert _loader.workspace_bytes(8192, 4736 * 2, 4096, sm_count=148) == 0    # 37 x 32 tiles: whole waves
    assert _loader.workspace_bytes(0, 64, 64, sm_count=148) == 0
    with pytest.raises(ValueError):
        _loader.workspace_bytes(16, 100, 64, sm_count=148)
