"""The full-graph rewrite pass on CPU: pattern matching on Dynamo graphs (meta tensors), the cached weight packer,
and the pass running inside a real MagiCompiler (subprocess, eager backend, oracle standing in for the kernel)."""
import gc
import os
import subprocess
import sys
import textwrap
from pathlib import Path

import pytest
import torch
import torch.nn.functional as F

import magicompiler_b200 as mb
from magicompiler_b200.passes import FuseSwiGLUPass, clear_pack_cache, pack_gate_up_cached

ROOT = Path(__file__).resolve().parent.parent
GEMM = torch.ops.magi_swiglu.gemm_swiglu.default
PACK = torch.ops.magi_swiglu.pack_gate_up_cached.default


class MLP(torch.nn.Module):
    """Same structure as the reference's TransformerMLP (tests/model_definition.py:327-339)."""

    def __init__(self, k=64, n=96, bias=False, dtype=torch.bfloat16, device="meta", swap=False, reuse=False):
        super().__init__()
        self.gate_proj = torch.nn.Linear(k, n, bias=bias, dtype=dtype, device=device)
        self.up_proj = torch.nn.Linear(k, n, bias=False, dtype=dtype, device=device)
        self.down_proj = torch.nn.Linear(n, k, bias=False, dtype=dtype, device=device)
        self.swap, self.reuse = swap, reuse

    def forward(self, x):
        gate = F.silu(self.gate_proj(x))
        up = self.up_proj(x)
        h = up * gate if self.swap else gate * up
        if self.reuse:
            h = h + gate
        return self.down_proj(h)


def run_pass(module, x, **pass_kwargs):
    """Compile with a backend that applies the pass to the Dynamo graph; returns (targets before, after, output).
    Unless a test says otherwise the pass emits the plain op (the choice between it and the training op has its own
    test)."""
    seen = {}
    pass_kwargs.setdefault("save_preactivations", False)

    def backend(gm, example_inputs):
        seen["before"] = [n.target for n in gm.graph.nodes if n.op == "call_function"]
        p = FuseSwiGLUPass(**pass_kwargs)
        seen["applicable"] = p.is_applicable(gm.graph)
        seen["count"] = p(gm.graph) if seen["applicable"] else 0
        gm.recompile()
        seen["after"] = [n.target for n in gm.graph.nodes if n.op == "call_function"]
        return gm.forward

    torch._dynamo.reset()
    y = torch.compile(module, backend=backend, fullgraph=True)(x)
    return seen, y


def test_pattern_is_rewritten_to_the_fused_op():
    seen, y = run_pass(MLP(), torch.empty(10, 64, dtype=torch.bfloat16, device="meta"))
    assert seen["applicable"] and seen["count"] == 1
    assert seen["after"].count(GEMM) == 1 and seen["after"].count(PACK) == 1
    assert F.silu not in seen["after"]
    assert sum(t in (F.linear, torch._C._nn.linear) for t in seen["after"]) == 1  # only down_proj is left
    assert tuple(y.shape) == (10, 64) and y.dtype == torch.bfloat16


def test_pass_memoises_the_packed_weight_only_for_frozen_weights():
    """The pack node carries `frozen`: False when the trace shows trainable weights with grad mode on (the weight is
    concatenated on every call), True under no_grad or when no weight requires grad (packed once)."""
    def frozen_flags(module, ctx):
        flags = []

        def backend(gm, example_inputs):
            FuseSwiGLUPass(allowed_devices=("meta",), save_preactivations=False)(gm.graph)
            flags.extend(n.args[2] for n in gm.graph.nodes if n.op == "call_function" and n.target is PACK)
            gm.recompile()
            return gm.forward

        torch._dynamo.reset()
        with ctx:
            torch.compile(module, backend=backend, fullgraph=True)(torch.empty(4, 64, dtype=torch.bfloat16, device="meta"))
        return flags

    import contextlib

    assert frozen_flags(MLP(), contextlib.nullcontext()) == [False]          # trainable parameters, grad mode on
    assert frozen_flags(MLP(), torch.no_grad()) == [True]                     # inference
    assert frozen_flags(MLP().requires_grad_(False), contextlib.nullcontext()) == [True]


def test_training_variant_emits_the_two_output_op():
    import operator

    seen, y = run_pass(MLP(), torch.empty(3, 10, 64, dtype=torch.bfloat16, device="meta"), save_preactivations=True)
    assert seen["count"] == 1 and GEMM not in seen["after"]
    assert seen["after"].count(torch.ops.magi_swiglu.gemm_swiglu_preact.default) == 1
    assert operator.getitem in seen["after"] and F.silu not in seen["after"]
    assert tuple(y.shape) == (3, 10, 64) and y.dtype == torch.bfloat16


class MergedMLP(torch.nn.Module):
    """One merged gate/up projection followed by SiluAndMul: the layout of vLLM-style models whose activation ops
    the reference handles in magi_compiler/passes/piecewise_graph/fix_functionalization.py:100-125."""

    def __init__(self, form, k=64, n=96):
        super().__init__()
        self.gate_up_proj = torch.nn.Linear(k, 2 * n, bias=False, dtype=torch.bfloat16, device="meta")
        self.form, self.n = form, n

    def forward(self, x):
        h, n = self.gate_up_proj(x), self.n
        if self.form == "chunk":
            a, b = h.chunk(2, dim=-1)
        elif self.form == "torch.chunk":
            a, b = torch.chunk(h, 2, -1)
        elif self.form == "split":
            a, b = h.split(n, dim=-1)
        elif self.form == "slice":
            a, b = h[..., :n], h[..., n:]
        elif self.form == "uneven":
            a, b = h[..., : n - 8], h[..., n - 8: 2 * n - 16]
        elif self.form == "up_first":
            b, a = h.chunk(2, dim=-1)
        elif self.form == "reused":
            a, b = h.chunk(2, dim=-1)
            return F.silu(a) * b + h.sum()
        return F.silu(a) * b


@pytest.mark.parametrize("form", ["chunk", "torch.chunk", "split", "slice"])
def test_merged_projection_form_is_rewritten_without_packing(form):
    seen, y = run_pass(MergedMLP(form), torch.empty(2, 5, 64, dtype=torch.bfloat16, device="meta"))
    assert seen["count"] == 1 and seen["after"].count(GEMM) == 1 and PACK not in seen["after"]
    assert F.silu not in seen["after"] and not any(t in (F.linear, torch._C._nn.linear) for t in seen["after"])
    assert tuple(y.shape) == (2, 5, 96) and y.dtype == torch.bfloat16


@pytest.mark.parametrize("form", ["uneven", "up_first", "reused"])
def test_merged_projection_lookalikes_are_left_alone(form):
    seen, _ = run_pass(MergedMLP(form), torch.empty(10, 64, dtype=torch.bfloat16, device="meta"))
    assert seen["count"] == 0 and GEMM not in seen["after"]


def test_default_picks_the_training_op_only_when_a_gradient_can_be_asked_for():
    PRE = torch.ops.magi_swiglu.gemm_swiglu_preact.default
    x = torch.empty(10, 64, dtype=torch.bfloat16, device="meta")
    seen, _ = run_pass(MLP(), x, save_preactivations=None)          # parameters require grad, grad mode on
    assert seen["after"].count(PRE) == 1 and GEMM not in seen["after"]
    with torch.no_grad():
        seen, _ = run_pass(MLP(), x, save_preactivations=None)      # inference
    assert seen["after"].count(GEMM) == 1 and PRE not in seen["after"]
    frozen = MLP().requires_grad_(False)
    seen, _ = run_pass(frozen, x, save_preactivations=None)         # nothing to differentiate
    assert seen["after"].count(GEMM) == 1 and PRE not in seen["after"]
    seen, _ = run_pass(frozen, x.clone().requires_grad_(True), save_preactivations=None)  # gradient w.r.t. x only
    assert seen["after"].count(PRE) == 1


def test_operand_order_and_leading_dims():
    seen, y = run_pass(MLP(swap=True), torch.empty(2, 5, 64, dtype=torch.bfloat16, device="meta"))
    assert seen["count"] == 1 and tuple(y.shape) == (2, 5, 64)


@pytest.mark.parametrize("kwargs", [dict(bias=True), dict(reuse=True), dict(dtype=torch.float32), dict(k=60, n=96)])
def test_non_matching_graphs_are_left_alone(kwargs):
    k = kwargs.get("k", 64)
    m = MLP(**kwargs)
    seen, y = run_pass(m, torch.empty(7, k, dtype=kwargs.get("dtype", torch.bfloat16), device="meta"))
    assert not seen["applicable"] and seen["count"] == 0 and seen["before"] == seen["after"]
    assert GEMM not in seen["after"]


def test_two_blocks_two_rewrites():
    class Two(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.a, self.b = MLP(), MLP()

        def forward(self, x):
            return self.b(self.a(x))

    seen, _ = run_pass(Two(), torch.empty(4, 64, dtype=torch.bfloat16, device="meta"))
    assert seen["count"] == 2 and seen["after"].count(GEMM) == 2


def test_cached_packer_packs_once_and_tracks_updates():
    clear_pack_cache()
    wg = torch.nn.Parameter(torch.randn(16, 8).to(torch.bfloat16), requires_grad=False)
    wu = torch.nn.Parameter(torch.randn(16, 8).to(torch.bfloat16), requires_grad=False)
    p1 = pack_gate_up_cached(wg, wu)
    assert torch.equal(p1, torch.cat([wg, wu])) and p1.shape == (32, 8)
    p2 = pack_gate_up_cached(wg, wu)
    assert p2.data_ptr() == p1.data_ptr(), "same parameters, unmodified: no second copy"
    with torch.no_grad():
        wu.mul_(2)  # in-place update (an optimizer step) bumps the version counter
    p3 = pack_gate_up_cached(wg, wu)
    assert torch.equal(p3, torch.cat([wg, wu])) and not torch.equal(p3, p1)
    from magicompiler_b200 import passes

    assert len(passes._pack_cache) == 1
    del wg, wu, p1, p2, p3
    gc.collect()
    assert len(passes._pack_cache) == 0, "the cache entry dies with its parameters"
    with pytest.raises(ValueError):
        pack_gate_up_cached(torch.zeros(4, 8), torch.zeros(6, 8))


def test_cached_packer_never_memoises_trainable_weights():
    """Weight updates that autograd's version counter does not see (``param.data.copy_``, ``param.data = new``,
    also at the SAME address, which is what FSDP's re-gathered flat parameter looks like) must reach the next call
    while the weights are trainable: nothing is memoised when a gradient can be asked for."""
    from magicompiler_b200 import passes

    clear_pack_cache()
    wg = torch.nn.Parameter(torch.randn(16, 8))
    wu = torch.nn.Parameter(torch.randn(16, 8))
    p1 = pack_gate_up_cached(wg, wu)
    assert torch.equal(p1, torch.cat([wg, wu])) and len(passes._pack_cache) == 0
    v = (wg._version, wu._version)
    wg.data.copy_(torch.full((16, 8), 3.0))          # counted on .data's own counter, not on the parameter's
    assert (wg._version, wu._version) == v
    assert torch.equal(pack_gate_up_cached(wg, wu)[:16], torch.full((16, 8), 3.0))
    fresh = torch.full((16, 8), 5.0)
    wu.data = fresh                                     # re-pointed: same object, same version
    assert torch.equal(pack_gate_up_cached(wg, wu)[16:], fresh)
    old_ptr = wu.data_ptr()
    wu.data.zero_()                                     # new contents at the SAME address
    assert wu.data_ptr() == old_ptr and float(pack_gate_up_cached(wg, wu)[16:].detach().abs().max()) == 0.0
    # without grad mode the same parameters count as frozen: memoised, and clear_pack_cache() is the explicit reset
    with torch.no_grad():
        q1 = pack_gate_up_cached(wg, wu)
        assert pack_gate_up_cached(wg, wu).data_ptr() == q1.data_ptr() and len(passes._pack_cache) == 1
        wg.data.fill_(7.0)
        clear_pack_cache()
        assert float(pack_gate_up_cached(wg, wu)[:16].min()) == 7.0
    clear_pack_cache()


def test_cached_packer_passes_gradients_to_both_weights():
    clear_pack_cache()
    wg = torch.nn.Parameter(torch.randn(8, 16))
    wu = torch.nn.Parameter(torch.randn(8, 16))
    packed = pack_gate_up_cached(wg, wu)
    (packed * torch.arange(16.0).view(16, 1)).sum().backward()
    assert torch.equal(wg.grad, torch.arange(8.0).view(8, 1).expand(8, 16))
    assert torch.equal(wu.grad, torch.arange(8.0, 16.0).view(8, 1).expand(8, 16))


_REF = Path(os.environ.get("MAGI_COMPILER_ROOT", ROOT.parent / "reference"))
_SCRIPT = textwrap.dedent('''
    import json, os, sys, tempfile
    stub = tempfile.mkdtemp(); open(os.path.join(stub, "graphviz.py"), "w").write("class Digraph:\\n    pass\\n")
    sys.path[:0] = [stub, sys.argv[1], sys.argv[2]]
    sys.argv = sys.argv[:1]
    os.environ["MAGI_COMPILE_CACHE_ROOT_DIR"] = tempfile.mkdtemp()
    os.environ["MAGI_LOGGING_LEVEL"] = "WARNING"
    os.environ["MAGI_SWIGLU_USE_MAGI_COMPILER"] = "1"
    import torch, torch.nn.functional as F
    import magicompiler_b200 as mb
    from magi_compiler import magi_compile
    from oracle import swiglu_gold
    calls = {"n": 0}
    def cpu_kernel(x, w):      # the oracle stands in for the CUDA kernel: this is a CPU test of the graph plumbing
        calls["n"] += 1
        return swiglu_gold(x.reshape(-1, x.shape[-1]).contiguous(), w)["gold_bf16"].view(*x.shape[:-1], -1)
    mb.gemm_swiglu.register_kernel("cpu")(cpu_kernel)
    assert mb.install_into_magi_compiler(allowed_devices=("cpu",))

    class MLP(torch.nn.Module):     # the reference's TransformerMLP, bf16
        def __init__(self):
            super().__init__()
            self.gate_proj = torch.nn.Linear(64, 96, bias=False, dtype=torch.bfloat16)
            self.up_proj = torch.nn.Linear(64, 96, bias=False, dtype=torch.bfloat16)
            self.down_proj = torch.nn.Linear(96, 64, bias=False, dtype=torch.bfloat16)
        def forward(self, x):
            gate = F.silu(self.gate_proj(x)); up = self.up_proj(x)
            return self.down_proj(gate * up)

    torch.manual_seed(0)
    eager = MLP()
    def patch(c):
        c.backend = "eager"
        return c
    model = magi_compile(MLP(), dynamic_arg_dims={"x": 0}, config_patch=patch)
    model.load_state_dict(eager.state_dict())
    res = {}
    with torch.no_grad():
        for rows in (12, 20):
            x = torch.randn(rows, 64).to(torch.bfloat16)
            y, ref = model(x), eager(x)
            res[f"close{rows}"] = bool(torch.allclose(y.float(), ref.float(), rtol=3e-2, atol=3e-2))
    res["fused_calls"] = calls["n"]
    print("RESULT " + json.dumps(res))
''')


@pytest.mark.skipif(not (_REF / "magi_compiler" / "__init__.py").exists(), reason="no MagiCompiler checkout here")
def test_pass_inside_real_magi_compiler(tmp_path):
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
    assert res["close12"] and res["close20"], res
    assert res["fused_calls"] == 2, "the unmodified model's eager SwiGLU was replaced by the fused op"
