"""Backward of the op without a GPU: the oracle's written-out gradient equals PyTorch autograd of the reference's
eager expression, the backward ops are registered with working fake impls, and the mirror wires autograd up."""
import torch
import torch.nn.functional as F
from torch._subclasses.fake_tensor import FakeTensorMode

import magicompiler_b200 as mb
from oracle import make_inputs, swiglu_backward_gold


def test_oracle_backward_equals_autograd_of_reference_expression():
    x, w = make_inputs(24, 64, 40, seed=3)
    dy = torch.randn(24, 40, generator=torch.Generator().manual_seed(1)).to(torch.bfloat16)
    xf = x.float().requires_grad_(True)
    wf = w.float().requires_grad_(True)
    y = F.silu(F.linear(xf, wf[:40])) * F.linear(xf, wf[40:])  # the reference's expression, in fp32
    y.backward(dy.float())
    dx, dw = swiglu_backward_gold(x, w, dy)
    assert torch.allclose(dx, xf.grad, rtol=1e-4, atol=1e-5)
    assert torch.allclose(dw, wf.grad, rtol=1e-4, atol=1e-5)


def test_backward_op_schema_and_fake_impl():
    op = torch.ops.magi_swiglu.swiglu_backward_act.default
    assert str(op._schema) == "magi_swiglu::swiglu_backward_act(Tensor h, Tensor dy) -> Tensor"
    with FakeTensorMode():
        h = torch.empty(10, 96, dtype=torch.bfloat16, device="cuda")
        dy = torch.empty(10, 48, dtype=torch.bfloat16, device="cuda")
        dh = mb.swiglu_backward_act(h, dy)
        assert dh.shape == (10, 96) and dh.dtype == torch.bfloat16
    op = torch.ops.magi_swiglu.swiglu_backward_dh.default
    assert str(op._schema) == "magi_swiglu::swiglu_backward_dh(Tensor x, Tensor w_gate_up, Tensor dy) -> Tensor"
    with FakeTensorMode():
        x = torch.empty(10, 64, dtype=torch.bfloat16, device="cuda")
        w = torch.empty(96, 64, dtype=torch.bfloat16, device="cuda")
        dh = mb.swiglu_backward_dh(x, w, torch.empty(10, 48, dtype=torch.bfloat16, device="cuda"))
        assert dh.shape == (10, 96) and dh.dtype == torch.bfloat16


def test_transposed_gemm_op_schema_and_fake_impl():
    op = torch.ops.magi_swiglu.gemm_bf16.default
    assert str(op._schema) == "magi_swiglu::gemm_bf16(Tensor a, Tensor b, bool a_is_km, bool b_is_kn) -> Tensor"
    with FakeTensorMode():
        dh = torch.empty(40, 96, dtype=torch.bfloat16, device="cuda")
        w = torch.empty(96, 64, dtype=torch.bfloat16, device="cuda")
        x = torch.empty(40, 64, dtype=torch.bfloat16, device="cuda")
        assert mb.gemm_bf16(dh, w, False, True).shape == (40, 64)      # dX = dH · W
        assert mb.gemm_bf16(dh, x, True, True).shape == (96, 64)       # dW = dH^T · X
        assert mb.gemm_bf16(x, w, False, False).shape == (40, 96)      # X · W^T


def test_autograd_graph_through_fake_tensors():
    """The forward op carries an autograd formula built from library GEMMs and the backward op: gradients of the
    right shapes come back for x and for the packed weight (meta tensors: nothing runs on a device)."""
    x = torch.empty(4, 6, 64, dtype=torch.bfloat16, device="meta", requires_grad=True)
    w = torch.empty(80, 64, dtype=torch.bfloat16, device="meta", requires_grad=True)
    y = mb.gemm_swiglu(x, w)
    assert y.requires_grad and y.shape == (4, 6, 40)
    gx, gw = torch.autograd.grad(y, (x, w), torch.empty_like(y))
    assert gx.shape == x.shape and gw.shape == w.shape and gx.dtype == torch.bfloat16
    (gx_only,) = torch.autograd.grad(mb.gemm_swiglu(x, w.detach()), (x,), torch.empty_like(y))
    assert gx_only.shape == x.shape


def test_training_op_keeps_the_preactivations_and_differentiates():
    op = torch.ops.magi_swiglu.gemm_swiglu_preact.default
    assert str(op._schema) == "magi_swiglu::gemm_swiglu_preact(Tensor x, Tensor w_gate_up) -> (Tensor, Tensor)"
    assert "magi_swiglu::gemm_swiglu_preact" in mb.SPLITTING_OPS
    x = torch.empty(4, 6, 64, dtype=torch.bfloat16, device="meta", requires_grad=True)
    w = torch.empty(80, 64, dtype=torch.bfloat16, device="meta", requires_grad=True)
    y, h = mb.gemm_swiglu_preact(x, w)
    assert y.shape == (4, 6, 40) and h.shape == (24, 80) and h.dtype == torch.bfloat16
    y = mb.gemm_swiglu_train(x, w)
    gx, gw = torch.autograd.grad(y, (x, w), torch.empty_like(y))
    assert gx.shape == x.shape and gw.shape == w.shape and gw.dtype == torch.bfloat16


def test_auto_entry_picks_by_grad_mode_and_requires_grad():
    x = torch.empty(4, 64, dtype=torch.bfloat16, device="meta")
    w = torch.empty(80, 64, dtype=torch.bfloat16, device="meta")
    assert mb.gemm_swiglu_auto(x, w).grad_fn is None
    y = mb.gemm_swiglu_auto(x, w.clone().requires_grad_(True))
    assert "gemm_swiglu_preact" in type(y.grad_fn).__name__ or "getitem" in type(y.grad_fn).__name__.lower() \
        or y.requires_grad
    assert y.shape == (4, 40) and y.requires_grad
    with torch.no_grad():
        assert not mb.gemm_swiglu_auto(x, w.clone().requires_grad_(True)).requires_grad
