"""Property tests of the schedule selection (pure host arithmetic behind ``magi_swiglu_plan``): whatever the shape,
the chosen schedule fits the SM (shared memory, tensor-memory columns), covers every output exactly once and asks
for scratch only where it may split K."""
import pytest
from hypothesis import given, settings, strategies as st

from magicompiler_b200 import _loader

SMEM_OPT_IN = 232448
TMEM_COLS = 512

dims8 = st.integers(min_value=1, max_value=8192).map(lambda v: v * 8)


@settings(max_examples=300, deadline=None)
@given(M=st.integers(min_value=1, max_value=70000), N=dims8, K=dims8,
       sm_count=st.sampled_from([148, 147, 132, 74, 16, 2]))
def test_auto_plan_invariants(M, N, K, sm_count):
    p = _loader.plan(M, N, K, sm_count=sm_count)
    bn, pair = p["block_n"], p["ctas"]
    assert p["variant"] in (_loader.VARIANT_MMA, _loader.VARIANT_MMA2, _loader.VARIANT_STREAM)
    assert (p["variant"] == _loader.VARIANT_STREAM) == (M <= 128)
    assert 16 <= bn <= 256 and bn % 16 == 0
    assert 2 <= p["stages"] <= 12 and p["smem_bytes"] <= SMEM_OPT_IN - 1024
    assert 2 * bn * p["acc_bufs"] <= TMEM_COLS and p["n_mma"] == (1 if 2 * bn <= 256 else 2)
    n_tiles = -(-N // bn)
    m_units = -(-M // (128 * pair))
    assert p["tiles"] == n_tiles * m_units and (n_tiles - 1) * bn < N <= n_tiles * bn
    assert 1 <= p["grid"] <= sm_count and p["grid"] % pair == 0
    assert p["grid"] <= p["tiles"] * pair * p["k_splits"]
    assert p["group_m"] >= 1
    if p["split"]:
        assert pair == 2 and p["n_mma"] == 2 and bn % 32 == 0
    if p["k_splits"] > 1:  # only the small-M streaming schedule splits K, and only within the scratch it may use
        assert p["variant"] == _loader.VARIANT_STREAM
        k_blocks = -(-K // 64)
        per = -(-k_blocks // p["k_splits"])
        assert per >= 4 and per * (p["k_splits"] - 1) < k_blocks          # every split has work
        need = _loader.workspace_bytes(M, N, K, sm_count=sm_count)
        assert need == p["tiles"] * p["k_splits"] * M * 2 * bn * 4 and need <= 64 << 20
    else:
        assert _loader.workspace_bytes(M, N, K, sm_count=sm_count) in (0,) or M <= 128


@settings(max_examples=150, deadline=None)
@given(M=st.integers(min_value=129, max_value=40000), N=dims8, K=dims8,
       variant=st.sampled_from(["mma", "mma2"]), bn=st.sampled_from(list(range(16, 257, 16))))
def test_explicit_tile_schedules_fit(M, N, K, variant, bn):
    p = _loader.plan(M, N, K, variant=variant, block_n=bn, sm_count=148)
    assert p["block_n"] == bn and p["ctas"] == (2 if variant == "mma2" else 1)
    assert p["smem_bytes"] <= SMEM_OPT_IN - 1024 and p["stages"] >= 2
    stage = 128 * 64 * 2 + 2 * bn * 128 // p["ctas"]
    assert p["stages"] * stage + 1024 <= SMEM_OPT_IN - 1024
    assert p["k_splits"] == 1 and p["tiles"] == -(-N // bn) * -(-M // (128 * p["ctas"]))


def test_without_scratch_nothing_is_split():
    for M in (1, 16, 64, 128):
        for N in (3584, 1792, 7168, 448):
            lib = _loader.load_library()
            # ws_limit 0 is what the entry points without a workspace argument pass
            assert lib.magi_swiglu_workspace_bytes(M, N, 8192, 0, 0, 0, 0, 0, 0, 148) >= 0
            p = _loader.plan(M, N, 8192, sm_count=148)
            assert p["tiles"] * p["k_splits"] <= 2 * 148
