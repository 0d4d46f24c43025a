"""Parity of the CUDA path against the CPU oracle, the reference fixtures and size-independent properties.
Every case goes through the C-ABI library (directly with ctypes, or through the registered op, which is one
ctypes call).  Tolerance of the path (bf16 output, fp32 accumulation), against the fp32-accumulated gold:
    max|y-gold|/max|gold| <= 1e-2,  ||y-gold||_F/||gold||_F <= 5e-3,  allclose(rtol=1e-2, atol=1e-2*max|gold|)."""
import contextlib
import ctypes

import numpy as np
import pytest
import torch

import magicompiler_b200 as mb
from magicompiler_b200 import _loader
from oracle import TOL_FROB, TOL_MAX_NORM, error_metrics, from_bits, make_inputs, swiglu_gold, to_bits

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", autouse=True)
def _require_b200():
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    lib = _loader.load_library()  # raises if the CUDA library was not built: there is no fallback to pass on
    assert lib.magi_swiglu_supported(0) == 1, "device 0 is not sm_100"
    yield
    st = mb.device_status(0)
    assert st["code"] == 0, f"a kernel wait timed out during the tests: {st}"


@contextlib.contextmanager
def whole_tile_schedules():
    """Stream-K off: every output is accumulated over K in one piece, whatever the schedule, so results can be
    compared bit for bit across schedules, tile widths and column shards.  (With stream-K on, the tiles whose K range
    is shared between two workers add two fp32 partial sums instead: same tolerance, not the same bits.)"""
    prev = _loader.set_tuning("stream_k", 0)
    try:
        yield
    finally:
        _loader.set_tuning("stream_k", prev)


def assert_parity(y, gold, what=""):
    m = error_metrics(y, gold)
    assert m["max_norm"] <= TOL_MAX_NORM and m["frob"] <= TOL_FROB, (what, m)
    assert torch.allclose(y.float().cpu(), gold.float().cpu(), rtol=1e-2, atol=1e-2 * m["gold_absmax"]), (what, m)
    return m


def gold_fp32_gpu(x, w):
    """fp32 gold on the GPU for sizes the CPU oracle would take minutes for (TF32 off)."""
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        n = w.shape[0] // 2
        h = x.float() @ w.float().t()
        return torch.nn.functional.silu(h[:, :n]) * h[:, n:]
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev


# ---------------------------------------------------------------- small cases against the CPU oracle
def test_c_abi_direct_call_cfg1():
    """Reference-sized case (256 x 1024 x 2816, seed 0) through the bare C entry point."""
    lib = _loader.load_library()
    x, w = make_inputs(256, 1024, 2816, seed=0)
    xd, wd = x.cuda(), w.cuda()
    y = torch.empty(256, 2816, dtype=torch.bfloat16, device="cuda")
    rc = lib.magi_swiglu_forward_bf16(xd.data_ptr(), wd.data_ptr(), y.data_ptr(), 256, 2816, 1024, 1024, 1024, 2816,
                                      0, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream), 0)
    assert rc == 0, _loader.last_error()
    torch.cuda.synchronize()
    o = swiglu_gold(x, w)
    m = assert_parity(y, o["gold"], "cfg1")
    # a single-rounded result must be at least as close to the gold as the reference's own eager chain
    assert m["frob"] <= error_metrics(o["eager"], o["gold"])["frob"] * 1.05


@pytest.mark.parametrize("name", ["tiny_48x128x96", "ragged_37x200x72", "mid_130x512x264", "cfg1_256x1024x2816"])
@pytest.mark.parametrize("variant", ["auto", "mma", "mma2", "simt"])
def test_against_reference_fixture(golden, name, variant):
    M, K, N, seed, step = (int(v) for v in golden[name + "/shape"])
    if name + "/x" in golden.files:
        x, w = from_bits(golden[name + "/x"]), from_bits(golden[name + "/w"])
    else:
        x, w = make_inputs(M, K, N, seed=seed)
    y = mb.gemm_swiglu_out(x.cuda(), w.cuda(), variant=variant).cpu()
    ref = from_bits(golden[name + "/y_eager"]).float()  # what MagiCompiler's TransformerMLP produced
    m = error_metrics(y[::step], ref)
    assert m["max_norm"] <= TOL_MAX_NORM and m["frob"] <= TOL_FROB, m
    assert_parity(y, swiglu_gold(x, w, want_eager=False)["gold"], name)


SHAPES = [  # (M, N, K): tails in every dimension, single-tile and multi-tile
    (1, 8, 8), (1, 64, 64), (16, 128, 64), (17, 72, 200), (64, 264, 128), (120, 136, 72), (128, 128, 1024),
    (129, 128, 64), (255, 192, 136), (256, 8, 64), (300, 520, 328), (515, 1000, 96), (33, 2816, 64),
    (384, 28672, 72), (300, 14336, 128),  # three 128-row granules and several waves: AUTO picks single-CTA tiles
]


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("variant", ["auto", "mma", "mma2", "stream"])
def test_ragged_shapes(shape, variant):
    M, N, K = shape
    if variant == "stream" and M > 128:
        pytest.skip("STREAM schedule is for M <= 128")
    x, w = make_inputs(M, K, N, seed=M + N + K)
    y = mb.gemm_swiglu_out(x.cuda(), w.cuda(), variant=variant)
    assert_parity(y, swiglu_gold(x, w, want_eager=False)["gold"], f"{shape} {variant}")


@pytest.mark.parametrize("block_n", [16, 32, 48, 64, 96, 112, 128, 144, 160, 192, 208, 224, 256])
@pytest.mark.parametrize("stages,max_ctas,group_m", [(0, 0, 0), (2, 2, 1), (3, 6, 2)])
@pytest.mark.parametrize("variant", ["mma", "mma2"])
def test_schedule_knobs(variant, block_n, stages, max_ctas, group_m):
    """Every tile width (one or two MMAs per step, one or two accumulator buffers), shallow pipelines and a
    single persistent CTA (or CTA pair) walking all tiles (many barrier phase wraps) give the same answer."""
    M, N, K = 600, 528, 320
    if stages:
        stages = min(stages, mb.plan(M, N, K, variant=variant, block_n=block_n)["stages"])  # wide tiles fit fewer
    if variant == "mma":
        max_ctas //= 2
    x, w = make_inputs(M, K, N, seed=block_n)
    y = mb.gemm_swiglu_out(x.cuda(), w.cuda(), variant=variant, block_n=block_n, stages=stages, max_ctas=max_ctas,
                           group_m=group_m)
    base = mb.gemm_swiglu_out(x.cuda(), w.cuda(), variant="mma")
    assert_parity(y, swiglu_gold(x, w, want_eager=False)["gold"], f"bn={block_n}")
    # the K loop order per output is the same for every schedule, so the bits are too
    assert torch.equal(y, base)


def test_guard_bands_strides_and_determinism():
    M, N, K = 200, 264, 136
    x, w = make_inputs(M, K, N, seed=77)
    ldx, ldw, ldy = K + 8, K + 16, N + 24
    xb = torch.full((M + 2, ldx), float("nan"), dtype=torch.bfloat16, device="cuda")
    wb = torch.full((2 * N + 2, ldw), float("nan"), dtype=torch.bfloat16, device="cuda")
    yb = torch.full((M + 4, ldy), 123.0, dtype=torch.bfloat16, device="cuda")
    xv, wv, yv = xb[1:M + 1, :K], wb[1:2 * N + 1, :K], yb[2:M + 2, :N]
    xv.copy_(x)
    wv.copy_(w)
    lib = _loader.load_library()
    runs = []
    for variant in (1, 1, 3):
        rc = lib.magi_swiglu_forward_bf16(xv.data_ptr(), wv.data_ptr(), yv.data_ptr(), M, N, K, ldx, ldw, ldy, 0,
                                          ctypes.c_void_p(torch.cuda.current_stream().cuda_stream), variant)
        assert rc == 0, _loader.last_error()
        torch.cuda.synchronize()
        got = yv.clone()
        assert_parity(got, swiglu_gold(x, w, want_eager=False)["gold"], "strided")
        # nothing outside [M,N] was written: NaN padding of the inputs never leaked in, guard values intact
        assert (yb[:2] == 123.0).all() and (yb[M + 2:] == 123.0).all() and (yb[:, N:] == 123.0).all()
        runs.append(got)
    assert torch.equal(runs[0], runs[1]), "two runs of the same launch differ"


def test_empty_and_noncontiguous_inputs():
    x, w = make_inputs(64, 128, 96, seed=5)
    xd, wd = x.cuda(), w.cuda()
    assert mb.gemm_swiglu(xd[:0], wd).shape == (0, 96)
    y = mb.gemm_swiglu(xd.view(4, 16, 128), wd)
    assert y.shape == (4, 16, 96)
    base = mb.gemm_swiglu(xd, wd)
    assert torch.equal(y.view(64, 96), base)
    xt = xd.t().contiguous().t()  # column-major view: the wrapper must copy, not mis-read
    assert torch.equal(mb.gemm_swiglu(xt, wd), base)
    with pytest.raises(ValueError):
        mb.gemm_swiglu(xd, wd.t().contiguous().t())  # the weight is never silently copied
    with pytest.raises(TypeError):
        mb.gemm_swiglu(xd.half(), wd.half())


def test_special_values():
    M, N, K = 32, 64, 64
    x = torch.zeros(M, K, dtype=torch.bfloat16)
    w = torch.zeros(2 * N, K, dtype=torch.bfloat16)
    x[:, 0] = 1.0
    w[:N, 0] = torch.linspace(-120, 120, N).to(torch.bfloat16)  # gate pre-activations from -120 to 120
    w[N:, 0] = 3.0
    y = mb.gemm_swiglu(x.cuda(), w.cuda()).cpu()
    g = w[:N, 0].float()
    exp = (torch.nn.functional.silu(g) * 3.0).expand(M, N)
    assert torch.isfinite(y.float()).all()
    assert torch.allclose(y.float(), exp, rtol=1e-2, atol=1e-6)


def test_non_finite_values():
    """NaN and +inf pre-activations behave like the eager expression; -inf stays non-finite (eager: NaN)."""
    M, N, K = 32, 64, 64
    inf, nan = float("inf"), float("nan")
    x = torch.zeros(M, K, dtype=torch.bfloat16)
    w = torch.zeros(2 * N, K, dtype=torch.bfloat16)
    x[:, 0] = 1.0
    w[:N, 0] = 1.0
    w[N:, 0] = 3.0
    w[0, 0], w[1, 0], w[2, 0] = inf, -inf, nan   # gate columns 0, 1, 2
    w[N + 3, 0], w[N + 4, 0] = inf, nan          # up columns 3, 4
    w[5, 0], w[N + 5, 0] = 0.0, inf              # 0 * inf
    y = mb.gemm_swiglu(x.cuda(), w.cuda()).cpu().float()
    ref = (torch.nn.functional.silu(w[:N, 0].float()) * w[N:, 0].float()).expand(M, N)
    same = [c for c in range(N) if c != 1]
    assert torch.equal(torch.isnan(y[:, same]), torch.isnan(ref[:, same]))
    assert torch.allclose(y[:, same], ref[:, same], rtol=1e-2, atol=1e-6, equal_nan=True)
    assert not torch.isfinite(y[:, 1]).any()


# ---------------------------------------------------------------- benchmark sizes: properties + sampled gold
@pytest.mark.parametrize("M", [16, 64, 128])
def test_decode_shapes_full_size(M):
    """Decode-shaped weight streaming at full size (K=8192, N=28672) against the fp32 gold on the GPU."""
    x, w = make_inputs(M, 8192, 28672, seed=0)
    xd, wd = x.cuda(), w.cuda()
    y = mb.gemm_swiglu(xd, wd)
    assert_parity(y, gold_fp32_gpu(xd, wd), f"decode M={M}")
    with whole_tile_schedules():
        assert torch.equal(y, mb.gemm_swiglu_out(xd, wd, variant="mma")), "both schedules accumulate in the same order"
        assert torch.equal(y, mb.gemm_swiglu_out(xd, wd, variant="mma2"))


def test_llama_ffn_full_size_properties():
    """8192 x 4096 x 14336: sampled rows against fp32 gold; exact scaling, permutation and shard properties."""
    M, K, N = 8192, 4096, 14336
    x, w = make_inputs(M, K, N, seed=0)
    xd, wd = x.cuda(), w.cuda()
    rows = torch.randperm(M, generator=torch.Generator().manual_seed(1))[:384].cuda()
    gold = gold_fp32_gpu(xd[rows], wd)
    y_auto = mb.gemm_swiglu(xd, wd)  # the schedule a caller gets (stream-K balances its last waves)
    assert_parity(y_auto[rows], gold, "llama ffn sample")
    with whole_tile_schedules():
        y = mb.gemm_swiglu(xd, wd)
        assert_parity(y[rows], gold, "llama ffn sample, whole tiles")
        for variant in ("mma", "mma2"):  # one CTA per tile and CTA pairs: same K order per output, same bits
            assert torch.equal(mb.gemm_swiglu_out(xd, wd, variant=variant), y), variant
        # (1) doubling the up weights doubles every output exactly (power-of-two scaling commutes with rounding)
        w2 = wd.clone()
        w2[N:] *= 2
        assert torch.equal(mb.gemm_swiglu(xd, w2), y * 2)
        # (2) permuting the rows of X permutes the rows of Y bit for bit (no dependence on tile position)
        perm = torch.randperm(M, generator=torch.Generator().manual_seed(2)).cuda()
        assert torch.equal(mb.gemm_swiglu(xd[perm].contiguous(), wd), y[perm])
        # (3) column shards are independent units: 8 shards side by side are the unsharded result bit for bit
        parts = [mb.gemm_swiglu(xd, mb.shard_gate_up(wd, r, 8)) for r in range(8)]
        assert torch.equal(torch.cat(parts, dim=1), y)
    # the balanced schedule differs from the whole-tile one only where a tile's K range was shared, and there by a
    # rounding of the fp32 sum: at most one bf16 step
    assert_close_to_whole_tiles(y_auto, y)
    w2 = wd.clone()
    w2[N:] *= 2
    assert torch.equal(mb.gemm_swiglu(xd, w2), y_auto * 2)  # exact scaling holds in every schedule


def assert_close_to_whole_tiles(y_sk, y_wt):
    """Two schedules that add the same fp32 products in a different order: few outputs change, none by more than one
    bf16 step at the scale of the data, and the change as a whole is far below the rounding noise of the output."""
    a, b = y_sk.float(), y_wt.float()
    diff = (a - b).abs()
    assert (diff > 0).float().mean().item() < 0.05
    assert diff.max().item() <= 2.0 ** -7 * b.abs().max().item()
    assert (diff.norm() / b.norm()).item() <= 5e-4


def test_video_dit_ffn_sampled():
    """32760 x 5120 x 13824 (ragged M): sampled rows incl. the last partial tile against fp32 gold."""
    M, K, N = 32760, 5120, 13824
    x, w = make_inputs(M, K, N, seed=0)
    xd, wd = x.cuda(), w.cuda()
    y = mb.gemm_swiglu(xd, wd)
    rows = torch.cat([torch.arange(M - 130, M), torch.randperm(M - 130, generator=torch.Generator().manual_seed(3))[:254]]).cuda()
    assert_parity(y[rows], gold_fp32_gpu(xd[rows], wd), "video dit sample")
    shard = mb.shard_gate_up(wd, 7, 8)  # 1728 columns: 13.5 tiles of 128
    with whole_tile_schedules():
        y_wt = mb.gemm_swiglu(xd, wd)
        for variant in ("mma", "mma2"):
            assert torch.equal(mb.gemm_swiglu_out(xd, shard, variant=variant), y_wt[:, 7 * 1728:]), variant
    assert_close_to_whole_tiles(y, y_wt)
    y_shard = mb.gemm_swiglu(xd, shard)  # the shard under its own balanced schedule
    assert_parity(y_shard[rows], gold_fp32_gpu(xd[rows], shard), "video dit shard sample")
    assert_close_to_whole_tiles(y_shard, y_wt[:, 7 * 1728:])


# ---------------------------------------------------------------- stream-K (tile schedules, balanced last waves)
@pytest.mark.parametrize("shape,knobs", [
    ((8192, 1792, 4096), {}),                       # 1/8 column shard of the Llama FFN: 224 tiles on 74 CTA pairs
    ((8192, 1792, 4096), dict(block_n=224)),        # 256 tiles
    ((4096, 1792, 1024), {}),                       # short K: pieces of a dozen K-steps
    ((4096, 3584, 1024), {}),
    ((32760, 1728, 5120), {}),                      # ragged rows, 6.75 column tiles
    ((640, 4096, 2048), dict(variant="mma")),       # one CTA per tile
    ((2560, 2816, 1024), dict(max_ctas=24)),        # twelve workers
])
def test_stream_k_matches_whole_tiles_and_gold(shape, knobs):
    """The last waves of a tile schedule are dealt to the workers as equal K ranges; a tile shared by two workers is
    finished by the one that holds its first K-steps, from fp32 partial sums parked in scratch.  Against the fp32 gold,
    against the whole-tile schedule (at most one bf16 step apart), and run to run (bit-identical)."""
    M, N, K = shape
    prev = _loader.set_tuning("stream_k", 1)
    try:
        plan = mb.plan(M, N, K, **knobs)
        assert plan["sk_tiles"] > 0 and mb.workspace_bytes(M, N, K, **knobs) > 0, plan
        x, w = make_inputs(M, K, N, seed=M + N)
        xd, wd = x.cuda(), w.cuda()
        y = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
        mb.gemm_swiglu_out(xd, wd, out=y, **knobs)
        again = mb.gemm_swiglu_out(xd, wd, **knobs)
    finally:
        _loader.set_tuning("stream_k", prev)
    assert torch.equal(y, again), "two launches of the same stream-K schedule differ"
    rows = torch.randperm(M, generator=torch.Generator().manual_seed(4))[:512].cuda()
    assert_parity(y[rows], gold_fp32_gpu(xd[rows], wd), f"stream-K {shape}")
    with whole_tile_schedules():
        assert mb.plan(M, N, K, **knobs)["sk_tiles"] == 0
        y_wt = mb.gemm_swiglu_out(xd, wd, **knobs)
    assert_close_to_whole_tiles(y, y_wt)


def test_stream_k_needs_scratch_and_is_refused_nothing_without_it():
    """Through the C entry point without a workspace the same problem runs whole tiles (no scratch, no flags)."""
    lib = _loader.load_library()
    M, N, K = 2048, 1792, 512
    x, w = make_inputs(M, K, N, seed=9)
    xd, wd = x.cuda(), w.cuda()
    y0 = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    rc = lib.magi_swiglu_forward_bf16(xd.data_ptr(), wd.data_ptr(), y0.data_ptr(), M, N, K, K, K, N, 0,
                                      ctypes.c_void_p(torch.cuda.current_stream().cuda_stream), 0)
    assert rc == 0, _loader.last_error()
    with whole_tile_schedules():
        assert torch.equal(y0, mb.gemm_swiglu(xd, wd))


# ---------------------------------------------------------------- split-K (narrow weights, M <= 128)
@pytest.mark.parametrize("M", [16, 64, 128])
@pytest.mark.parametrize("n_shard", [3584, 7168])
def test_decode_column_shards_split_k(M, n_shard):
    """A 1/8 or 1/4 column shard of the decode weight: several CTAs share a slab and split K through scratch memory.
    Checked against the fp32 gold; repeated launches reuse the scratch and agree bit for bit."""
    plan = mb.plan(M, n_shard, 8192)
    assert plan["k_splits"] > 1 and mb.workspace_bytes(M, n_shard, 8192) > 0
    x, w = make_inputs(M, 8192, n_shard, seed=n_shard + M)
    xd, wd = x.cuda(), w.cuda()
    y1 = mb.gemm_swiglu(xd, wd)
    assert_parity(y1, gold_fp32_gpu(xd, wd), f"shard M={M} N={n_shard}")
    for _ in range(3):
        assert torch.equal(mb.gemm_swiglu(xd, wd), y1)
    # the same problem without scratch (plain C entry point) runs unsplit and agrees within rounding of the sums
    lib = _loader.load_library()
    y0 = torch.empty_like(y1)
    rc = lib.magi_swiglu_forward_bf16(xd.data_ptr(), wd.data_ptr(), y0.data_ptr(), M, n_shard, 8192, 8192, 8192, n_shard,
                                      0, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream), 0)
    assert rc == 0, _loader.last_error()
    assert_parity(y0, gold_fp32_gpu(xd, wd), "unsplit")
    assert error_metrics(y1, y0.float())["max_norm"] < 8e-3  # at most one bf16 step apart


@pytest.mark.parametrize("splits", [2, 3, 5, 8])
@pytest.mark.parametrize("shape", [(1, 264, 2048), (37, 72, 4096), (128, 528, 2304), (100, 2816, 1024)])
def test_forced_k_splits_ragged(splits, shape):
    M, N, K = shape
    prev = _loader.set_tuning("k_splits", splits)
    try:
        # the forced count is used unless it would leave a split without K-steps (then the planner chooses)
        assert mb.plan(M, N, K, variant="stream")["k_splits"] in ({splits} if (-(-K // 64) // splits) >= 4 else {1, 2, 3, 4, 5, 6, 7, 8})
        x, w = make_inputs(M, K, N, seed=splits + M)
        y = mb.gemm_swiglu_out(x.cuda(), w.cuda(), variant="stream")
        y2 = mb.gemm_swiglu_out(x.cuda(), w.cuda(), variant="stream")
    finally:
        _loader.set_tuning("k_splits", prev)
    assert_parity(y, swiglu_gold(x, w, want_eager=False)["gold"], f"{shape} z={splits}")
    assert torch.equal(y, y2)


def test_workspace_entry_point_contract():
    """Through the C ABI with a caller-owned workspace: too small a workspace falls back to an unsplit schedule,
    a misaligned one is rejected on the host, and the workspace needs no initialisation (it starts as NaNs here)."""
    lib = _loader.load_library()
    M, N, K = 64, 3584, 4096
    x, w = make_inputs(M, K, N, seed=3)
    xd, wd = x.cuda(), w.cuda()
    need = mb.workspace_bytes(M, N, K)
    assert need > 0
    ws = torch.full(((need + 256) // 2,), float("nan"), dtype=torch.bfloat16, device="cuda").view(torch.uint8)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    gold = gold_fp32_gpu(xd, wd)

    def call(ws_ptr, ws_len):
        y = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
        rc = lib.magi_swiglu_forward_bf16_ws(xd.data_ptr(), wd.data_ptr(), y.data_ptr(), M, N, K, K, K, N, 0, stream, 0,
                                             0, 0, 0, 0, ws_ptr, ws_len)
        return rc, y

    rc, y = call(ws.data_ptr(), need)
    assert rc == 0, _loader.last_error()
    assert_parity(y, gold, "full workspace")
    rc, y_small = call(ws.data_ptr(), 4096)  # cannot hold the partial sums: unsplit schedule, still correct
    assert rc == 0 and assert_parity(y_small, gold, "small workspace")
    rc, _ = call(ws.data_ptr() + 16, need)
    assert rc == -3 and "aligned" in _loader.last_error()
    rc, y_null = call(None, 0)
    assert rc == 0 and torch.equal(y_null, y_small)


def test_random_shapes_all_schedules():
    """Seeded sweep of irregular shapes (any M, N and K multiples of 8) through every schedule that accepts them."""
    import random

    rng = random.Random(1234)
    checked = 0
    for _ in range(48):
        M = rng.choice([1, 2, 7, 31, 100, 128, 129, 200, 257, 511, 640, 1000])
        N = 8 * rng.randint(1, 180)
        K = 8 * rng.randint(1, 160)
        x, w = make_inputs(M, K, N, seed=checked)
        xd, wd = x.cuda(), w.cuda()
        gold = gold_fp32_gpu(xd, wd)
        variants = ["auto", "mma", "mma2"] + (["stream"] if M <= 128 else [])
        outs = {}
        for v in variants:
            outs[v] = mb.gemm_swiglu_out(xd, wd, variant=v)
            assert_parity(outs[v], gold, f"M={M} N={N} K={K} {v}")
            checked += 1
        assert torch.equal(outs["mma"], outs["mma2"]), (M, N, K)
    assert checked >= 150


@pytest.mark.parametrize("shape", [(262144, 1024, 256), (256, 65536, 64), (100000, 264, 72), (3, 131072, 128)])
def test_extreme_aspect_ratios(shape):
    """Very tall, very wide and very thin problems: index arithmetic, raster bands and tails at their limits."""
    M, N, K = shape
    g = torch.Generator(device="cuda").manual_seed(M % 1000)
    xd = torch.randn(M, K, generator=g, device="cuda").to(torch.bfloat16)
    wd = (torch.randn(2 * N, K, generator=g, device="cuda") * 0.05).to(torch.bfloat16)
    y = mb.gemm_swiglu(xd, wd)
    rows = torch.unique(torch.cat([torch.arange(0, min(M, 64)), torch.arange(max(0, M - 300), M),
                                   torch.randint(0, M, (256,))])).cuda()
    assert_parity(y[rows], gold_fp32_gpu(xd[rows], wd), f"{shape}")
    assert mb.device_status(0)["code"] == 0
