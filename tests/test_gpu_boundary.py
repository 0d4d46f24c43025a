"""The registered op in the situations MagiCompiler puts a split-point op in: eager dispatch, dynamo with a
dynamic row count, a side stream, CUDA-graph capture and replay, and the tensor-parallel MLP wrapper."""
import pytest
import torch

import magicompiler_b200 as mb
from magicompiler_b200 import _loader
from magicompiler_b200.sharding import reference_mlp
from oracle import TOL_FROB, TOL_MAX_NORM, error_metrics, make_inputs, swiglu_gold

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


def test_scratch_of_a_captured_graph_survives_later_larger_calls():
    """A split-K call captured into a CUDA graph keeps its scratch for the life of the graph: a later eager call that
    needs more scratch, and allocations over whatever was freed, must not disturb the graph's replay."""
    M1, M2, N, K = 16, 128, 3584, 8192  # 1/8 decode shards: both split K; the second wants more scratch
    assert 0 < mb.workspace_bytes(M1, N, K) < mb.workspace_bytes(M2, N, K)
    x1, w = make_inputs(M1, K, N, seed=31)
    x2, _ = make_inputs(M2, K, N, seed=32)
    x1, x2, w = x1.cuda(), x2.cuda(), w.cuda()
    expect1 = mb.gemm_swiglu(x1, w)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        mb.gemm_swiglu(x1, w)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        y_graph = mb.gemm_swiglu(x1, w)
    expect2 = mb.gemm_swiglu(x2, w)                      # larger scratch, eager
    junk = [torch.full((1 << 20,), float("nan"), device="cuda") for _ in range(64)]  # lands on freed blocks
    y_graph.zero_()
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(y_graph, expect1)
    assert torch.equal(mb.gemm_swiglu(x2, w), expect2)
    del junk


def test_bounded_wait_gives_up_reports_and_clears():
    """The kernels' bounded wait by itself: a one-block kernel waits on a barrier nothing signals, gives up after about
    a millisecond, returns normally and leaves {role, block, index} for device_status; the status clears on read and
    the next launch of the real kernel on the same context is correct."""
    import ctypes

    lib = _loader.load_library()
    assert mb.device_status(0)["code"] == 0
    rc = lib.magi_swiglu_watchdog_selftest(0, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream), 2_000_000)
    assert rc == 0, _loader.last_error()
    st = mb.device_status(0)  # synchronises
    assert st == {"code": 7, "block": 0, "index": 42, "parity": 0}, st
    assert mb.device_status(0)["code"] == 0, "reading the status clears it"
    assert lib.magi_swiglu_watchdog_selftest(0, None, 10) < 0  # limit out of range: rejected on the host
    x, w = make_inputs(256, 1024, 2816, seed=0)
    y = mb.gemm_swiglu(x.cuda(), w.cuda())
    m = error_metrics(y, swiglu_gold(x, w, want_eager=False)["gold"])
    assert m["max_norm"] <= TOL_MAX_NORM and m["frob"] <= TOL_FROB and mb.device_status(0)["code"] == 0


# ---------------------------------------------------------------- backward (training)
def _grad_errors(got, gold):
    from oracle import error_metrics

    return error_metrics(got, gold)


@pytest.fixture(params=["library", "own"])
def gradient_gemms(request):
    prev = mb.set_gradient_gemms(request.param)
    yield request.param
    mb.set_gradient_gemms(prev)


@pytest.mark.parametrize("shape", [(256, 512, 384), (304, 328, 520), (64, 1024, 2816), (4096, 1024, 2048)])
def test_backward_against_fp32_gold_and_reference_autograd(shape, gradient_gemms):
    """dX and dW of the op against the fp32 gradient of the reference's expression.  Tolerance (bf16 gradients, one
    recomputed bf16 intermediate): max|d-gold|/max|gold| <= 2e-2 and Frobenius-relative <= 1e-2; and the op's error
    stays within 1.5x of what PyTorch's own bf16 autograd of the eager expression makes on the same inputs."""
    import torch.nn.functional as F

    from oracle import swiglu_backward_gold

    M, K, N = shape
    x, w = make_inputs(M, K, N, seed=M)
    dy = torch.randn(M, N, generator=torch.Generator().manual_seed(7)).to(torch.bfloat16)
    xd = x.cuda().requires_grad_(True)
    wd = w.cuda().requires_grad_(True)
    y = mb.gemm_swiglu(xd, wd)
    y.backward(dy.cuda())
    dx_gold, dw_gold = swiglu_backward_gold(x.cuda(), w.cuda(), dy.cuda())
    xe = x.cuda().requires_grad_(True)
    we = w.cuda().requires_grad_(True)
    (F.silu(F.linear(xe, we[:N])) * F.linear(xe, we[N:])).backward(dy.cuda())  # the reference's eager path, bf16
    for name, got, ref, gold in (("dx", xd.grad, xe.grad, dx_gold), ("dw", wd.grad, we.grad, dw_gold)):
        assert got.dtype == torch.bfloat16 and got.shape == gold.shape
        m, mref = _grad_errors(got, gold), _grad_errors(ref, gold)
        assert m["max_norm"] <= 2e-2 and m["frob"] <= 1e-2, (name, m)
        assert m["frob"] <= 1.5 * mref["frob"] + 1e-4, (name, m, mref)


def test_backward_act_kernel_special_cases():
    h = torch.zeros(16, 32, dtype=torch.bfloat16, device="cuda")
    h[:, :16] = torch.linspace(-60, 60, 16).to(torch.bfloat16)  # gate pre-activations
    h[:, 16:] = 2.0
    dy = torch.ones(16, 16, dtype=torch.bfloat16, device="cuda")
    dh = mb.swiglu_backward_act(h, dy).float()
    g = h[:, :16].float()
    s = torch.sigmoid(g)
    assert torch.isfinite(dh).all()
    assert torch.allclose(dh[:, :16], 2.0 * s * (1 + g * (1 - s)), rtol=1e-2, atol=1e-3)
    assert torch.allclose(dh[:, 16:], g * s, rtol=1e-2, atol=1e-3)
    assert mb.swiglu_backward_act(h[:0], dy[:0]).shape == (0, 32)
    with pytest.raises(ValueError):
        mb.swiglu_backward_act(h, dy[:, :8])


@pytest.mark.parametrize("shape", [(1, 64, 8), (64, 1024, 2816), (128, 264, 200), (300, 328, 520), (384, 72, 28672),
                                   (1000, 512, 2048)])
def test_fused_backward_dh_kernel(shape):
    """swiglu_backward_dh (recompute in tensor memory + derivative in the epilogue) against the fp32 formula, in every
    schedule AUTO picks (streaming, CTA pairs, single-CTA tiles); it is at least as close to it as the two-kernel
    route through a bf16 H."""
    M, K, N = shape
    x, w = make_inputs(M, K, N, seed=N)
    dy = torch.randn(M, N, generator=torch.Generator().manual_seed(3)).to(torch.bfloat16)
    xd, wd, dyd = x.cuda(), w.cuda(), dy.cuda()
    dh = mb.swiglu_backward_dh(xd, wd, dyd)
    assert dh.shape == (M, 2 * N) and dh.dtype == torch.bfloat16
    h = xd.float() @ wd.float().t()
    g, u = h[:, :N], h[:, N:]
    s = torch.sigmoid(g)
    gold = torch.cat([dyd.float() * u * s * (1 + g * (1 - s)), dyd.float() * g * s], dim=1)
    m = _grad_errors(dh, gold)
    assert m["max_norm"] <= 1e-2 and m["frob"] <= 5e-3, m
    two_step = mb.swiglu_backward_act(mb.gemm_nt(xd, wd), dyd) if N % 8 == 0 and (2 * N) % 16 == 0 else None
    if two_step is not None:
        assert m["frob"] <= _grad_errors(two_step, gold)["frob"] * 1.02 + 1e-6
    # a strided dY (a column slice of a wider gradient) is read in place
    wide = torch.zeros(M, N + 8, dtype=torch.bfloat16, device="cuda")
    wide[:, :N] = dyd
    assert torch.equal(mb.swiglu_backward_dh(xd, wd, wide[:, :N]), dh)
    with pytest.raises(ValueError):
        mb.swiglu_backward_dh(xd, wd, dyd[:, : N - 8] if N > 8 else dyd[:0])


@pytest.mark.parametrize("shape", [(64, 1024, 2816), (300, 328, 520), (384, 72, 28672), (4096, 1024, 2048)])
def test_training_forward_keeps_preactivations_and_backward_uses_them(shape):
    """gemm_swiglu_preact: y is bit-identical to the inference op (same schedule), h is the single-rounded X·W^T, and the gradients
    from the kept h meet the same bounds as the recomputing backward."""
    from oracle import swiglu_backward_gold

    M, K, N = shape
    x, w = make_inputs(M, K, N, seed=M + 1)
    dy = torch.randn(M, N, generator=torch.Generator().manual_seed(8)).to(torch.bfloat16).cuda()
    xd = x.cuda().requires_grad_(True)
    wd = w.cuda().requires_grad_(True)
    y, h = mb.gemm_swiglu_preact(xd, wd)
    y_inf = mb.gemm_swiglu(x.cuda(), w.cuda())
    if mb.plan(M, N, K)["k_splits"] == 1 or mb.workspace_bytes(M, N, K) == 0:
        assert torch.equal(y, y_inf)
    else:  # the inference op splits K through scratch for this shape (another summation order); this op does not
        assert _grad_errors(y, y_inf.float())["max_norm"] <= 8e-3
    h_gold = x.cuda().float() @ w.cuda().float().t()
    m = _grad_errors(h, h_gold)
    assert m["max_norm"] <= 4e-3 and m["frob"] <= 3e-3, m  # one bf16 rounding of an fp32-accumulated product
    if (2 * N) % 16 == 0:
        assert torch.equal(h, mb.gemm_nt(x.cuda(), w.cuda()))
    mb.gemm_swiglu_train(xd, wd).backward(dy)
    dx_gold, dw_gold = swiglu_backward_gold(x.cuda(), w.cuda(), dy)
    for name, got, gold in (("dx", xd.grad, dx_gold), ("dw", wd.grad, dw_gold)):
        m = _grad_errors(got, gold)
        assert m["max_norm"] <= 2e-2 and m["frob"] <= 1e-2, (name, m)


def test_training_step_through_torch_compile():
    """The op inside a compiled training step (AOTAutograd traces its backward formula): gradients match eager."""
    torch._dynamo.reset()
    x, w = make_inputs(192, 256, 384, seed=4)
    xd = x.cuda()
    w1 = w.cuda().requires_grad_(True)
    w2 = w.cuda().requires_grad_(True)

    def loss_fn(x, w):
        return (mb.gemm_swiglu(x, w).float() ** 2).mean()

    loss_fn(xd, w1).backward()
    torch.compile(loss_fn, backend="aot_eager", fullgraph=True)(xd, w2).backward()
    assert torch.allclose(w1.grad.float(), w2.grad.float(), rtol=1e-2, atol=1e-6)


@pytest.mark.parametrize("shape", [(256, 512, 512), (300, 1056, 328), (64, 2048, 1024), (4096, 4096, 2048), (1, 16, 8)])
def test_plain_gemm_on_the_tile_kernels(shape):
    """gemm_nt = F.linear on the same kernels (identity epilogue) against an fp32 gold."""
    M, N, K = shape
    g = torch.Generator().manual_seed(M + N)
    a = torch.randn(M, K, generator=g).to(torch.bfloat16).cuda()
    b = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16).cuda()
    c = mb.gemm_nt(a, b)
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    gold = a.float() @ b.float().t()
    torch.backends.cuda.matmul.allow_tf32 = prev
    from oracle import error_metrics

    m = error_metrics(c, gold)
    assert c.shape == (M, N) and m["max_norm"] <= 1e-2 and m["frob"] <= 5e-3, m
    lib = torch.nn.functional.linear(a, b)
    assert error_metrics(c, lib.float())["max_norm"] <= 8e-3  # at most a bf16 step from the library GEMM
    with pytest.raises(ValueError):
        mb.gemm_nt(a, b[: N - 8] if N > 8 else b[:, :4])
    # written in place into a row slice of a larger, wider buffer: same bytes, nothing outside the slice touched
    big = torch.full((M + 5, N + 8), 7.0, dtype=torch.bfloat16, device="cuda")
    dst = big[2:2 + M, :N]
    assert mb.gemm_nt_out(a, b, out=dst) is dst
    assert torch.equal(dst, c)
    big[2:2 + M, :N] = 7.0
    assert (big == 7.0).all()
    with pytest.raises(ValueError):
        mb.gemm_nt_out(a, b, out=torch.empty(M, N, dtype=torch.float32, device="cuda"))


@pytest.mark.parametrize("shape", [(256, 512, 512), (64, 256, 128), (304, 1056, 328), (1000, 4096, 2048), (8, 16, 8),
                                   (520, 176, 72)])
@pytest.mark.parametrize("a_is_km,b_is_kn", [(False, True), (True, False), (True, True), (False, False)])
def test_gemm_with_operands_stored_either_way_round(shape, a_is_km, b_is_kn):
    """gemm_bf16: an operand stored [K, rows] is read as an MN-major tile (no transpose in memory); all four
    combinations against an fp32 gold and, bit for bit, against the same product with pre-transposed copies."""
    from oracle import error_metrics

    M, N, K = shape
    g = torch.Generator().manual_seed(M + N + K)
    A = torch.randn(M, K, generator=g).to(torch.bfloat16).cuda()
    B = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16).cuda()
    a = A.t().contiguous() if a_is_km else A
    b = B.t().contiguous() if b_is_kn else B
    c = mb.gemm_bf16(a, b, a_is_km, b_is_kn)
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    gold = A.float() @ B.float().t()
    torch.backends.cuda.matmul.allow_tf32 = prev
    m = error_metrics(c, gold)
    assert c.shape == (M, N) and m["max_norm"] <= 1e-2 and m["frob"] <= 5e-3, m
    assert error_metrics(c, torch.nn.functional.linear(A, B).float())["max_norm"] <= 8e-3
    assert mb.device_status(0)["code"] == 0


def test_mlp_with_own_down_projection():
    x, w, wd = make_inputs(512, 256, 384, seed=2, with_down=True)
    x, w, wd = x.cuda(), w.cuda(), wd.cuda()
    got = mb.TensorParallelSwiGLUMLP(w, wd, chunks=2, down_fn=mb.gemm_nt)(x)
    ref = reference_mlp(x, w, wd)
    assert torch.allclose(got.float(), ref.float(), rtol=2e-2, atol=2e-2 * ref.float().abs().max().item())


def test_call_from_a_fresh_thread():
    """A thread that has never touched CUDA (like an autograd worker) can call the op: the library binds the
    device's context itself before encoding tensor maps."""
    import threading

    x, w = _inputs(M=200)
    expect = mb.gemm_swiglu(x, w)
    out = {}

    def work():
        try:
            out["y"] = mb.gemm_swiglu_out(x, w)
        except Exception as exc:  # surfaced in the main thread below
            out["err"] = exc

    t = threading.Thread(target=work)
    t.start()
    t.join()
    torch.cuda.synchronize()
    assert "err" not in out, out.get("err")
    assert torch.equal(out["y"], expect)


# ---------------------------------------------------------------- RMSNorm fused in front of the op
def test_rmsnorm_fused_against_reference_fixture(golden):
    from oracle import error_metrics, from_bits, rmsnorm_swiglu_gold

    name = "rms_96x256x136"
    x, w = from_bits(golden[name + "/x"]), from_bits(golden[name + "/w"])
    gamma = torch.from_numpy(golden[name + "/gamma"])
    eps = float(golden[name + "/eps"][0])
    wf = mb.fold_rmsnorm_weight(w.cuda(), gamma)
    y = mb.rmsnorm_gemm_swiglu(x.cuda(), wf, eps)
    ref = from_bits(golden[name + "/y_eager"]).float()  # what the reference's RMSNorm + TransformerMLP produced
    m = error_metrics(y, ref)
    assert m["max_norm"] <= 1e-2 and m["frob"] <= 5e-3, m
    m = error_metrics(y, rmsnorm_swiglu_gold(x, gamma, w, eps))
    assert m["max_norm"] <= 1e-2 and m["frob"] <= 5e-3, m


@pytest.mark.parametrize("shape", [(16, 3584, 2048), (128, 264, 520), (300, 528, 328), (4096, 2048, 1024)])
def test_rmsnorm_fused_shapes(shape):
    """Every schedule (split-K reduce, streaming, CTA pairs) applies the row scale; compared with the fp32 gold and
    with the reference's eager chain on the GPU."""
    from oracle import error_metrics, rmsnorm_swiglu_gold, rmsnorm_swiglu_ref_eager

    M, N, K = shape
    x, w = make_inputs(M, K, N, seed=N)
    x = (x.float() * 3.0 + 0.5).to(torch.bfloat16)  # rows whose rms is far from 1
    gamma = 1.0 + 0.2 * torch.randn(K, generator=torch.Generator().manual_seed(1))
    eps = 1e-6
    xd, wd = x.cuda(), w.cuda()
    y = mb.rmsnorm_gemm_swiglu(xd, mb.fold_rmsnorm_weight(wd, gamma), eps)
    gold = rmsnorm_swiglu_gold(xd, gamma.cuda(), wd, eps)
    m = error_metrics(y, gold)
    assert y.shape == (M, N) and m["max_norm"] <= 1e-2 and m["frob"] <= 5e-3, m
    mref = error_metrics(rmsnorm_swiglu_ref_eager(xd, gamma.cuda(), wd, eps), gold)
    assert m["frob"] <= mref["frob"] * 1.2 + 1e-4, (m, mref)
    # the plain op on pre-normalised activations is the same computation up to the rounding of x_norm
    with pytest.raises(ValueError):
        mb.fold_rmsnorm_weight(wd, gamma[:-8])
