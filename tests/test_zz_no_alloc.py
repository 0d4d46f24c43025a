"""The entry point that brings its own scratch memory, ``magi_swiglu_forward_bf16_static``.

Some callers cannot hand the library a workspace because they cannot obtain device memory where the call happens:
a plain C / ctypes user without an allocator, or a serving process whose pool already owns all of the GPU.  For them
the split-K schedule of the small-M kernel keeps its fp32 partial sums in an 8 MiB array compiled into the library.
This file checks, through the C ABI, that the entry point gives what the workspace-taking entry point gives, twice in
a row (the array is reused and keeps old contents), and that it refuses a problem whose scratch would not fit.
It is collected last so that a failure here cannot hide a failure anywhere else.
"""
import ctypes

import pytest
import torch

from magicompiler_b200 import _loader
from oracle import TOL_FROB, TOL_MAX_NORM, error_metrics, make_inputs

pytestmark = pytest.mark.gpu

STATIC_SCRATCH_BYTES = 8 << 20


def _fp32_gold(x, w):
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        n = w.shape[0] // 2
        h = x.float() @ w.float().t()
        return torch.nn.functional.silu(h[:, :n]) * h[:, n:]
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev


def test_static_scratch_entry_matches_workspace_entry_twice_in_a_row():
    assert torch.cuda.is_available()
    lib = _loader.load_library()
    assert lib.magi_swiglu_supported(0) == 1
    M, N, K = 64, 3584, 4096  # a 1/8 column shard of a decode GEMM: the schedule splits K and needs scratch
    need = _loader.workspace_bytes(M, N, K)
    assert 0 < need <= STATIC_SCRATCH_BYTES and _loader.plan(M, N, K)["k_splits"] > 1
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    results = []
    for seed in (11, 12):  # two calls in a row, different data: the second one finds the first one's partial sums
        x, w = make_inputs(M, K, N, seed=seed)
        xd, wd = x.cuda(), w.cuda()
        ws = torch.empty(need, dtype=torch.uint8, device="cuda")
        y_ws = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
        rc = lib.magi_swiglu_forward_bf16_ws(xd.data_ptr(), wd.data_ptr(), y_ws.data_ptr(), M, N, K, K, K, N, 0, stream,
                                             0, 0, 0, 0, 0, ws.data_ptr(), need)
        assert rc == 0, _loader.last_error()
        y_static = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
        rc = lib.magi_swiglu_forward_bf16_static(xd.data_ptr(), wd.data_ptr(), y_static.data_ptr(), M, N, K, K, K, N,
                                                 0, stream)
        assert rc == 0, _loader.last_error()
        torch.cuda.synchronize()
        # same schedule, same summation order: the two entry points agree to the bit ...
        assert torch.equal(y_static, y_ws)
        # ... and both are within the tolerance of the path against the fp32 gold
        m = error_metrics(y_static, _fp32_gold(xd, wd))
        assert m["max_norm"] <= TOL_MAX_NORM and m["frob"] <= TOL_FROB, m
        results.append(y_static)
    assert not torch.equal(results[0], results[1])
    st = (ctypes.c_int32 * 4)()
    assert lib.magi_swiglu_device_status(0, st) == 0 and st[0] == 0


def test_static_scratch_entry_rejects_what_does_not_fit_and_runs_what_needs_none():
    lib = _loader.load_library()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    # a problem whose preferred schedule wants more scratch than the built-in array holds: refused, nothing launched
    M, N, K = 128, 7168, 8192
    assert _loader.workspace_bytes(M, N, K) > STATIC_SCRATCH_BYTES
    x = torch.zeros(M, K, dtype=torch.bfloat16, device="cuda")
    w = torch.zeros(2 * N, K, dtype=torch.bfloat16, device="cuda")
    y = torch.full((M, N), 7.0, dtype=torch.bfloat16, device="cuda")
    rc = lib.magi_swiglu_forward_bf16_static(x.data_ptr(), w.data_ptr(), y.data_ptr(), M, N, K, K, K, N, 0, stream)
    assert rc == -2 and "scratch" in _loader.last_error()
    torch.cuda.synchronize()
    assert (y == 7.0).all()
    # a large-M problem needs no scratch at all and simply runs
    M, N, K = 384, 512, 256
    xc, wc = make_inputs(M, K, N, seed=5)
    xd, wd = xc.cuda(), wc.cuda()
    y = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    rc = lib.magi_swiglu_forward_bf16_static(xd.data_ptr(), wd.data_ptr(), y.data_ptr(), M, N, K, K, K, N, 0, stream)
    assert rc == 0, _loader.last_error()
    m = error_metrics(y, _fp32_gold(xd, wd))
    assert m["max_norm"] <= TOL_MAX_NORM and m["frob"] <= TOL_FROB, m
