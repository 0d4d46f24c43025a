"""Property tests of the schedule selection (pure host arithmetic behind ``magi_swiglu_plan`` and
``magi_swiglu_schedule``): whatever the shape, the chosen schedule fits the SM (shared memory, tensor-memory columns),
covers every (tile, K-step) exactly once, asks for scratch only where it splits K, and every K range that parks
partial sums has exactly one owner waiting for it."""
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
        rows = -(-M // 32) * 32  # partial sums are parked by whole warps of 32 rows
        assert need == p["tiles"] * p["k_splits"] * rows * 2 * bn * 4 and need <= 64 << 20
    else:
        need = _loader.workspace_bytes(M, N, K, sm_count=sm_count)
        assert 0 <= need <= 64 << 20
        # scratch without split-K means stream-K: a tile schedule whose last waves are dealt out as K ranges
        assert (need > 0) == (p["sk_tiles"] > 0)
        if p["sk_tiles"]:
            assert p["variant"] in (_loader.VARIANT_MMA, _loader.VARIANT_MMA2) and p["sk_tiles"] <= p["tiles"]
            units = p["grid"] // pair
            rem = p["tiles"] % units
            assert 0 < rem * 4 <= units, "stream-K only where the last wave would be at most a quarter full"


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


def _walk(M, N, K, sm_count, **knobs):
    p = _loader.plan(M, N, K, sm_count=sm_count, **knobs)
    units = p["grid"] // p["ctas"]
    return p, [_loader.schedule(M, N, K, u, sm_count=sm_count, **knobs) for u in range(units)]


@settings(max_examples=60, deadline=None)
@given(M=st.integers(min_value=129, max_value=16384), N=st.integers(min_value=8, max_value=1024).map(lambda v: v * 8),
       K=st.integers(min_value=1, max_value=512).map(lambda v: v * 8),
       sm_count=st.sampled_from([148, 132, 74, 16, 6]), variant=st.sampled_from(["auto", "mma", "mma2"]))
def test_every_tile_and_k_step_is_covered_exactly_once(M, N, K, sm_count, variant):
    """Whole tiles and stream-K ranges together: each (tile, K-step) belongs to exactly one worker, each shared tile
    has one owner (the worker with its first K-steps) whose peers are exactly the workers that park a piece of it."""
    p, items = _walk(M, N, K, sm_count, variant=variant)
    nk = -(-K // 64)
    seen, owners, parked = set(), {}, {}
    for u, work in enumerate(items):
        for i, w in enumerate(work):
            assert 0 <= w["kb0"] < w["kb1"] <= nk and 0 <= w["tile"] < p["tiles"]
            for kb in range(w["kb0"], w["kb1"]):
                assert (w["tile"], kb) not in seen
                seen.add((w["tile"], kb))
            if w["role"] == 1:
                assert w["kb0"] == 0 and w["kb1"] < nk and w["first_peer"] == u + 1 and w["peers"] >= 1
                assert w["kb1"] - w["kb0"] >= min(8, nk) and i == len(work) - 1  # the head piece ends a worker's list
                owners[w["tile"]] = (w["first_peer"], w["peers"])
            elif w["role"] == 2:
                assert w["kb0"] > 0 and w["kb1"] - w["kb0"] >= min(8, nk)
                parked.setdefault(w["tile"], []).append(u)
                # a worker parks at most once, before any other stream-K piece of its range
                assert all(v["role"] == 0 and v["tile"] < w["tile"] for v in work[:i])
            else:
                assert (w["kb0"], w["kb1"]) == (0, nk)
    assert len(seen) == p["tiles"] * nk
    assert set(owners) == set(parked)
    for t, (first, n) in owners.items():
        assert parked[t] == list(range(first, first + n))


def test_stream_k_balances_the_column_shards_of_the_llama_ffn():
    """The 1/8 column shard of the Llama FFN: 224 tiles of 256 columns on 74 CTA pairs would run 4 waves with the last
    one 3 % full; stream-K gives every pair the same number of K-steps (to within one short piece)."""
    p, items = _walk(8192, 1792, 4096, 148)
    assert p["variant"] == _loader.VARIANT_MMA2 and p["block_n"] == 256 and p["tiles"] == 224 and p["sk_tiles"] == 76
    steps = [sum(w["kb1"] - w["kb0"] for w in work) for work in items]
    assert sum(steps) == 224 * 64 and max(steps) - min(steps) <= 2 * 16
    assert _loader.workspace_bytes(8192, 1792, 4096, sm_count=148) == 256 * 3 + 148 * 256 * 1024
    # without scratch, or with the aid switched off, the same problem runs whole tiles
    lib = _loader.load_library()
    assert lib.magi_swiglu_schedule(8192, 1792, 4096, 0, 0, 0, 0, 0, 148, 0, 0, None, 0) == -1  # out is required
    prev = _loader.set_tuning("stream_k", 0)
    try:
        assert _loader.plan(8192, 1792, 4096, sm_count=148)["sk_tiles"] == 0
        assert _loader.workspace_bytes(8192, 1792, 4096, sm_count=148) == 0
    finally:
        _loader.set_tuning("stream_k", prev)
