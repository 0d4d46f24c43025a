"""The drop-in boundary without a GPU: registration, schema, fake impl, dtype rules, graph capture of the op,
and (when a MagiCompiler checkout is importable) placement of the op in MagiCompiler's split graph.

Modelled on the reference's tests/api_tests/test_register_custom_op.py (forward-only ops, meta-function
variants, auto names, ``torch.compile(backend="eager")`` integration)."""
import os
import subprocess
import sys
import textwrap
from pathlib import Path

import pytest
import torch
from torch._subclasses.fake_tensor import FakeTensorMode

import magicompiler_b200 as mb
from magicompiler_b200.register import magi_register_custom_op

ROOT = Path(__file__).resolve().parent.parent


def test_op_is_registered_with_the_expected_schema():
    op = torch.ops.magi_swiglu.gemm_swiglu.default
    assert str(op._schema) == "magi_swiglu::gemm_swiglu(Tensor x, Tensor w_gate_up) -> Tensor"
    assert not op._schema.is_mutable
    assert mb.OP_NAME in mb.SPLITTING_OPS and mb.OP_NAME in mb.COMPUTE_SENSITIVE_OPS


@pytest.mark.parametrize("lead", [(5,), (2, 3), (1, 1, 7)])
def test_fake_impl_shape_dtype_device(lead):
    with FakeTensorMode():
        x = torch.empty(*lead, 64, dtype=torch.bfloat16, device="cuda")
        w = torch.empty(2 * 40, 64, dtype=torch.bfloat16, device="cuda")
        y = mb.gemm_swiglu(x, w)
        assert tuple(y.shape) == (*lead, 40) and y.dtype == torch.bfloat16 and y.device == x.device


def test_fp8_output_op_schema_and_fake_impl():
    op = torch.ops.magi_swiglu.gemm_swiglu_fp8.default
    assert str(op._schema) == "magi_swiglu::gemm_swiglu_fp8(Tensor x, Tensor w_gate_up, Tensor scale) -> Tensor"
    assert not op._schema.is_mutable
    with FakeTensorMode():
        x = torch.empty(3, 5, 64, dtype=torch.bfloat16, device="cuda")
        w = torch.empty(2 * 48, 64, dtype=torch.bfloat16, device="cuda")
        y = mb.gemm_swiglu_fp8(x, w, torch.empty(1, dtype=torch.float32, device="cuda"))
        assert tuple(y.shape) == (3, 5, 48) and y.dtype == torch.float8_e4m3fn and y.device == x.device
    with pytest.raises(TypeError):  # CPU tensors: no CPU path
        mb.gemm_swiglu_fp8(torch.zeros(4, 64, dtype=torch.bfloat16), torch.zeros(32, 64, dtype=torch.bfloat16),
                           torch.ones(1))


def test_nvfp4_output_op_schema_and_fake_impl():
    op = torch.ops.magi_swiglu.gemm_swiglu_nvfp4.default
    assert str(op._schema) == ("magi_swiglu::gemm_swiglu_nvfp4(Tensor x, Tensor w_gate_up, Tensor global_scale, "
                               "bool swizzled_scales) -> (Tensor, Tensor)")
    with FakeTensorMode():
        x = torch.empty(3, 50, 64, dtype=torch.bfloat16, device="cuda")
        w = torch.empty(2 * 48, 64, dtype=torch.bfloat16, device="cuda")
        gs = torch.empty(1, dtype=torch.float32, device="cuda")
        codes, sf = mb.gemm_swiglu_nvfp4(x, w, gs, False)
        assert tuple(codes.shape) == (3, 50, 24) and codes.dtype == torch.uint8
        assert tuple(sf.shape) == (150, 3) and sf.dtype == torch.float8_e4m3fn
        codes, sf = mb.gemm_swiglu_nvfp4(x, w, gs, True)
        assert tuple(sf.shape) == mb.nvfp4_scale_shape(150, 48, True) == (256 * 4,)


def test_fake_impl_with_symbolic_rows():
    from torch.fx.experimental.proxy_tensor import make_fx

    def f(x, w):
        return mb.gemm_swiglu(x * 1.0, w)

    gm = make_fx(f, tracing_mode="symbolic")(torch.empty(6, 64, dtype=torch.bfloat16, device="meta"),
                                             torch.empty(48, 64, dtype=torch.bfloat16, device="meta"))
    targets = [n.target for n in gm.graph.nodes if n.op == "call_function"]
    assert torch.ops.magi_swiglu.gemm_swiglu.default in targets
    out = [n for n in gm.graph.nodes if n.op == "output"][0].args[0]
    assert isinstance(out.meta["val"].shape[0], torch.SymInt)
    assert out.meta["val"].shape[1] == 24


def test_dtype_and_shape_rules_raise_before_any_launch():
    bf, f32 = torch.bfloat16, torch.float32
    with pytest.raises(TypeError):
        mb.gemm_swiglu(torch.zeros(4, 64, dtype=f32), torch.zeros(16, 64, dtype=bf))
    with pytest.raises(TypeError):
        mb.gemm_swiglu(torch.zeros(4, 64, dtype=bf), torch.zeros(16, 64, dtype=torch.float16))
    with pytest.raises(ValueError):
        mb.gemm_swiglu(torch.zeros(4, 64, dtype=bf), torch.zeros(15, 64, dtype=bf))      # odd row count
    with pytest.raises(ValueError):
        mb.gemm_swiglu(torch.zeros(4, 64, dtype=bf), torch.zeros(16, 32, dtype=bf))      # K mismatch
    with pytest.raises(ValueError):
        mb.gemm_swiglu(torch.zeros(4, 60, dtype=bf), torch.zeros(16, 60, dtype=bf))      # K % 8
    with pytest.raises(ValueError):
        mb.gemm_swiglu(torch.zeros(4, 64, dtype=bf), torch.zeros(2, 8, 64, dtype=bf))    # 3-D weight
    with pytest.raises(TypeError):
        mb.gemm_swiglu(torch.zeros(4, 64, dtype=bf), torch.zeros(16, 64, dtype=bf))      # CPU tensors: no CPU path


def test_dynamo_captures_the_op_as_one_node_with_dynamic_rows():
    """torch.compile traces through the fake impl; meta tensors keep the run itself off any device."""
    seen = []

    def backend(gm, example_inputs):
        seen.append([n.target for n in gm.graph.nodes if n.op == "call_function"])
        return gm.forward

    def f(x, w):
        return mb.gemm_swiglu(x + 1, w) * 2

    torch._dynamo.reset()
    cf = torch.compile(f, backend=backend, fullgraph=True, dynamic=True)
    w = torch.empty(32, 64, dtype=torch.bfloat16, device="meta")
    for rows in (8, 24):
        y = cf(torch.empty(rows, 64, dtype=torch.bfloat16, device="meta"), w)
        assert tuple(y.shape) == (rows, 16) and y.dtype == torch.bfloat16
    assert len(seen) == 1, "a second row count must not recompile"
    assert seen[0].count(torch.ops.magi_swiglu.gemm_swiglu.default) == 1


# ---- the decorator mirror, case by case as the reference tests it --------------------------------------
def test_mirror_default_identity_meta_and_auto_name():
    @magi_register_custom_op()
    def _mirror_relu(x: torch.Tensor) -> torch.Tensor:
        return torch.maximum(x, torch.zeros_like(x))

    x = torch.randn(4, 8)
    assert torch.equal(_mirror_relu(x), torch.relu(x))
    assert hasattr(torch.ops.test_boundary_cpu, "_mirror_relu")  # "{file_stem}::{function}"
    with FakeTensorMode():
        assert _mirror_relu(torch.empty(3, 5)).shape == (3, 5)


def test_mirror_named_params_meta_and_multi_output():
    @magi_register_custom_op(name="mirror_test::two_out", infer_output_meta_fn=["weight", "bias"])
    def two_out(g: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        return g.sum(0).view_as(weight).clone(), g.sum().expand_as(bias).clone()

    with FakeTensorMode():
        a, b = two_out(torch.empty(2, 12), torch.empty(3, 4), torch.empty(7))
        assert a.shape == (3, 4) and b.shape == (7,)


def test_mirror_autograd_and_flags():
    def setup(ctx, inputs, output):
        ctx.save_for_backward(inputs[0])

    def backward(ctx, grad):
        (x,) = ctx.saved_tensors
        return grad * 2 * x

    @magi_register_custom_op(name="mirror_test::square", infer_output_meta_fn=lambda x: torch.empty_like(x),
                             setup_context_fn=setup, backward_fn=backward, is_compute_sensitive=True,
                             is_subgraph_boundary=True)
    def square(x: torch.Tensor) -> torch.Tensor:
        return x * x

    x = torch.randn(5, requires_grad=True)
    square(x).sum().backward()
    assert torch.allclose(x.grad, 2 * x.detach())
    assert "mirror_test::square" in mb.SPLITTING_OPS and "mirror_test::square" in mb.COMPUTE_SENSITIVE_OPS


# ---- integration with a real MagiCompiler checkout (CPU, eager backend) --------------------------------
# a MagiCompiler checkout: $MAGI_COMPILER_ROOT, else a directory "reference" next to this repository
_REF = Path(os.environ.get("MAGI_COMPILER_ROOT", ROOT.parent / "reference"))

_SCRIPT = textwrap.dedent('''
    import json, os, sys, tempfile
    stub = tempfile.mkdtemp(); open(os.path.join(stub, "graphviz.py"), "w").write("class Digraph:\\n    pass\\n")
    sys.path[:0] = [stub, sys.argv[1], sys.argv[2]]
    sys.argv = sys.argv[:1]
    os.environ["MAGI_COMPILE_CACHE_ROOT_DIR"] = tempfile.mkdtemp()
    os.environ["MAGI_LOGGING_LEVEL"] = "WARNING"
    os.environ["MAGI_SWIGLU_USE_MAGI_COMPILER"] = "1"
    import torch
    import magicompiler_b200 as mb                      # registers through magi_compiler.magi_register_custom_op
    from magicompiler_b200.register import registered_through_magi_compiler
    from magi_compiler import magi_compile
    from magi_compiler.config import get_compile_config
    from oracle import swiglu_gold                       # CPU stand-in for the kernel: this is a test
    mb.gemm_swiglu.register_kernel("cpu")(lambda x, w: swiglu_gold(x.reshape(-1, x.shape[-1]), w)["gold_bf16"].view(*x.shape[:-1], -1))
    cfg = get_compile_config()
    res = {"through_ref": registered_through_magi_compiler(),
           "splitting": mb.OP_NAME in cfg.splitting_ops,
           "sensitive": mb.OP_NAME in cfg.recompute_config.custom_compute_sensitive_ops}

    class Block(torch.nn.Module):
        def __init__(self):
            super().__init__()
            g = torch.Generator().manual_seed(0)
            self.w = torch.nn.Parameter((torch.randn(2 * 40, 64, generator=g) * 0.05).to(torch.bfloat16), requires_grad=False)
            self.down = torch.nn.Linear(40, 64, bias=False, dtype=torch.bfloat16)
        def forward(self, x):
            return self.down(mb.gemm_swiglu(x * 1.0, self.w))

    def patch(c):
        c.backend = "eager"
        return c
    try:
        model = magi_compile(Block(), dynamic_arg_dims={"x": 0}, config_patch=patch)
    except TypeError:
        model = magi_compile(Block(), dynamic_arg_dims={"x": 0})
    x = torch.randn(12, 64).to(torch.bfloat16)
    with torch.no_grad():
        y = model(x)
        ref = Block()
        ref.load_state_dict(model.state_dict())
        h = swiglu_gold(x, ref.w)["gold_bf16"]
        exp = ref.down(h)
        y2 = model(torch.randn(20, 64).to(torch.bfloat16))
    res["shape"] = list(y.shape); res["shape2"] = list(y2.shape)
    res["close"] = bool(torch.allclose(y.float(), exp.float(), rtol=2e-2, atol=2e-2))
    print("RESULT " + json.dumps(res))
''')


@pytest.mark.skipif(not (_REF / "magi_compiler" / "__init__.py").exists(), reason="no MagiCompiler checkout here")
def test_registers_through_real_magi_compiler_and_splits_graph(tmp_path):
    script = tmp_path / "probe.py"
    script.write_text(_SCRIPT)
    env = dict(os.environ)
    env.pop("MAGI_SWIGLU_USE_MAGI_COMPILER", None)
    proc = subprocess.run([sys.executable, str(script), str(_REF), str(ROOT)], capture_output=True, text=True,
                          timeout=600, env=env, cwd=str(tmp_path))
    line = [l for l in proc.stdout.splitlines() if l.startswith("RESULT ")]
    assert line, proc.stdout[-2000:] + proc.stderr[-4000:]
    import json

    res = json.loads(line[0][7:])
    assert res["through_ref"] and res["splitting"] and res["sensitive"], res
    assert res["shape"] == [12, 64] and res["shape2"] == [20, 64] and res["close"], res
