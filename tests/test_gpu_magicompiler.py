"""The CUDA kernel under the REAL MagiCompiler on a GPU: registered through its own decorator, dispatched from its
piecewise graph with Inductor-compiled pieces either side, under its CUDA-graph manager (PIECEWISE and FULL) and its
offload executor, plus two of the reference's own test files run with this package loaded first.

MagiCompiler is taken from ``baseline/_ref`` (put there by ``baseline/install_reference.py``), else from
``$MAGI_COMPILER_ROOT`` or a checkout beside this repository.  Every case runs in a child process: registration is
process-wide and these cases want the reference's decorator, not the package's mirror of it.

Reference code paths exercised: registration ``magi_compiler/_magi_register_custom_op.py:168-204``; graph split at
the op ``magi_backend/magi_backend.py:492-547`` with compiled pieces ``piecewise_backend.py:83-116``; CUDA-graph
manager warm-up on a side stream and capture ``cuda_graph_mgr.py:465-473,548-581``; offload executor
``offload/offload_warpper.py:140-210``; full-graph pass manager ``passes/full_graph/full_graph_pass_mgr.py:27-38``.
"""
import json
import os
import subprocess
import sys
import textwrap
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent


def _reference_root():
    for cand in (ROOT / "baseline" / "_ref", os.environ.get("MAGI_COMPILER_ROOT"), ROOT.parent / "reference"):
        if cand and (Path(cand) / "magi_compiler" / "__init__.py").exists():
            return Path(cand)
    return None


_REF = _reference_root()
needs_reference = pytest.mark.skipif(_REF is None, reason="no MagiCompiler installation or checkout here")

# Common start of every child: paths, environment, the package (which registers through the reference's decorator),
# the rewrite pass installed into the reference's full-graph pass manager, and a counter of kernel launches.
_PRELUDE = textwrap.dedent('''
    import json, os, sys, tempfile
    ref, root = sys.argv[1], sys.argv[2]
    tests_parent = os.path.join(ref, "reference_tests") if os.path.isdir(os.path.join(ref, "reference_tests")) else ref
    extra = []
    try:
        import graphviz  # noqa: F401
    except Exception:
        if not os.path.exists(os.path.join(ref, "graphviz.py")):
            stub = tempfile.mkdtemp(); open(os.path.join(stub, "graphviz.py"), "w").write("class Digraph:\\n    pass\\n")
            extra = [stub]
    sys.path[:0] = extra + [ref, tests_parent, root]
    sys.argv = sys.argv[:1]
    os.environ["MAGI_COMPILE_CACHE_ROOT_DIR"] = tempfile.mkdtemp()
    os.environ["MAGI_LOGGING_LEVEL"] = "WARNING"
    os.environ["MAGI_SWIGLU_USE_MAGI_COMPILER"] = "1"
    import torch, torch.nn.functional as F
    on_gpu = torch.cuda.is_available()
    dev = "cuda" if on_gpu else "cpu"
    import magicompiler_b200 as mb                      # registers through magi_compiler.magi_register_custom_op
    from magicompiler_b200 import ops as mb_ops
    from magicompiler_b200.register import registered_through_magi_compiler
    from magi_compiler import magi_compile
    from magi_compiler.config import CudaGraphMode, get_compile_config
    calls = {"n": 0, "weights": []}
    if on_gpu:
        _real = mb_ops.gemm_swiglu_out
        def _counting(*a, **k):
            calls["n"] += 1
            calls["weights"].append(a[1])                # the packed weight the kernel is about to read
            return _real(*a, **k)
        mb_ops.gemm_swiglu_out = _counting              # the op's body looks this name up on every call
    else:  # no GPU here: the CPU oracle stands in for the kernel so the graph plumbing can still be exercised
        from oracle import swiglu_gold
        def _cpu(x, w):
            calls["n"] += 1
            return swiglu_gold(x.reshape(-1, x.shape[-1]).contiguous(), w)["gold_bf16"].view(*x.shape[:-1], -1)
        mb.gemm_swiglu.register_kernel("cpu")(_cpu)
        get_compile_config().backend = "eager"          # CPU Inductor needs a host tool chain this box may lack
    assert mb.install_into_magi_compiler(allowed_devices=("cuda", "meta") if on_gpu else ("cpu",))
    res = {"through_ref": registered_through_magi_compiler(), "on_gpu": on_gpu,
           "splitting": mb.OP_NAME in get_compile_config().splitting_ops}
    def close(a, b, tol=3e-2):
        return bool(torch.allclose(a.float(), b.float(), rtol=tol, atol=tol * max(1e-6, b.float().abs().max().item())))
    def patch_backend(c):
        if not on_gpu:
            c.backend = "eager"
        return c
''')

_BLOCK = _PRELUDE + textwrap.dedent('''
    from tests.model_definition import TransformerBlock, TransformerConfig, TransformerMLP
    cfg = TransformerConfig(vocab_size=128, hidden_size=256, intermediate_size=512, num_hidden_layers=1,
                            num_attention_heads=4, num_key_value_heads=4, max_position_embeddings=128)
    torch.manual_seed(0)
    # (a) an UNMODIFIED TransformerMLP instance compiled by magi_compile: the pass turns its eager SwiGLU into the op
    eager = TransformerMLP(cfg).to(dev)
    model = magi_compile(TransformerMLP(cfg).to(dev), dynamic_arg_dims={"x": 0}, config_patch=patch_backend)
    model.load_state_dict(eager.state_dict())
    ok = []
    with torch.no_grad():
        for rows in (300, 77, 512):                      # three lengths through one dynamic-shape compilation
            x = torch.randn(rows, 256, device=dev).to(torch.bfloat16)
            ok.append(close(model(x), eager(x)))
    res["mlp_close"] = ok
    res["mlp_calls"] = calls["n"]
    # (b) the reference's own TransformerBlock class (decorated with magi_compile in its defining module)
    if on_gpu:
        blk = TransformerBlock(cfg).to(dev)
        def eager_block(b, x):
            r = x; h = b.input_layernorm(x).to(torch.bfloat16); h = b.self_attn(h); x = r + h
            r = x; h = b.post_attention_layernorm(x).to(torch.bfloat16); h = b.mlp(h); return r + h
        ok, before = [], calls["n"]
        with torch.no_grad():
            for bsz in (2, 5, 3):
                x = torch.randn(bsz, 64, 256, device=dev).to(torch.bfloat16)
                ok.append(close(blk(x), eager_block(blk, x)))
        res["block_close"] = ok
        res["block_calls"] = calls["n"] - before
    print("RESULT " + json.dumps(res))
''')

_GRAPHS = _PRELUDE + textwrap.dedent('''
    from tests.model_definition import TransformerConfig, TransformerMLP
    import magi_compiler.magi_backend.cuda_graph_mgr as cgm
    cfg = TransformerConfig(vocab_size=128, hidden_size=256, intermediate_size=512, num_hidden_layers=1,
                            num_attention_heads=4, num_key_value_heads=4, max_position_embeddings=128)
    torch.manual_seed(0)
    eager = TransformerMLP(cfg).to(dev)
    for mode in ("PIECEWISE", "FULL"):
        def patch(c, mode=mode):
            c.cudagraph_mode = getattr(CudaGraphMode, mode)
            return patch_backend(c)
        model = magi_compile(TransformerMLP(cfg).to(dev), dynamic_arg_dims={"x": 0}, config_patch=patch,
                             model_tag="mlp_" + mode.lower())
        model.load_state_dict(eager.state_dict())
        ok, before = [], calls["n"]
        with torch.no_grad():
            for rows, seed in ((256, 1), (256, 2), (96, 3), (256, 4), (96, 5)):   # replays see new contents
                x = torch.randn(rows, 256, device=dev, generator=torch.Generator(device=dev).manual_seed(seed)).to(torch.bfloat16)
                ok.append(close(model(x).clone(), eager(x)))
        res[mode] = {"close": ok, "python_calls_of_the_op": calls["n"] - before,
                     "graphs": cgm.cuda_graph_mgr().graph_count if on_gpu else None}
    res["status"] = mb.device_status(0)["code"] if on_gpu else 0
    print("RESULT " + json.dumps(res))
''')

# Under the offload executor the module is traced with its tensors on the host (the executor brings them to the GPU
# call by call), so the pass is told that host-traced graphs are fine here; a tensor that really reaches the op on the
# host still raises (the op has no CPU path).
_OFFLOAD = _PRELUDE.replace('allowed_devices=("cuda", "meta") if on_gpu', 'allowed_devices=("cuda", "meta", "cpu") if on_gpu') + textwrap.dedent('''
    from tests.model_definition import TransformerConfig, TransformerMLP
    cfg = TransformerConfig(vocab_size=128, hidden_size=256, intermediate_size=512, num_hidden_layers=1,
                            num_attention_heads=4, num_key_value_heads=4, max_position_embeddings=128)
    torch.manual_seed(0)
    eager = TransformerMLP(cfg).to(dev)
    conf = get_compile_config()
    conf.offload_config.model_cpu_offload = True        # the decorator reads the global config when it wraps the class
    conf.offload_config.gpu_resident_weight_ratio = 0.0  # nothing stays resident: every call brings the weights in anew

    class MergedMLP(torch.nn.Module):                   # the op called directly on a merged gate/up weight
        def __init__(self, cfg):
            super().__init__()
            self.w_gate_up = torch.nn.Parameter(torch.empty(2 * cfg.intermediate_size, cfg.hidden_size, dtype=torch.bfloat16))
            self.down_proj = torch.nn.Linear(cfg.intermediate_size, cfg.hidden_size, bias=False, dtype=torch.bfloat16)
        def forward(self, x):
            return self.down_proj(mb.gemm_swiglu(x * 1.0, self.w_gate_up))

    def run(model, packed_now):
        model.cuda() if on_gpu else None
        out = {"weights_stay_on_host": next(model.parameters()).device.type == "cpu"}
        ok, before = [], calls["n"]
        calls["weights"].clear()
        with torch.no_grad():
            for rows, seed in ((192, 1), (192, 2), (64, 3), (192, 4)):
                x = torch.randn(rows, 256, device=dev, generator=torch.Generator(device=dev).manual_seed(seed)).to(torch.bfloat16)
                ok.append(close(model(x), eager(x)))
        # what the kernel was handed on every call is the CURRENT host weight, packed (never a stale copy), even though
        # the executor brings the weights to the GPU as new tensors call after call
        current = packed_now().to(dev)
        out["weight_fed_is_current"] = [bool(torch.equal(w.to(dev), current)) for w in calls["weights"]]
        out["close"] = ok
        out["calls"] = calls["n"] - before
        return out

    Merged = magi_compile(dynamic_arg_dims={"x": 0}, config_patch=patch_backend)(MergedMLP)
    merged = Merged(cfg)
    with torch.no_grad():
        merged.w_gate_up.copy_(torch.cat([eager.gate_proj.weight, eager.up_proj.weight]).cpu())
        merged.down_proj.weight.copy_(eager.down_proj.weight.cpu())
    try:
        res["merged"] = run(merged, lambda: merged.w_gate_up.detach())
    except Exception as exc:
        res["merged"] = {"error": repr(exc)[:600]}
    # the UNMODIFIED reference module under the same executor: its weights are traced on the host and the rewrite
    # pass still turns its SwiGLU into the op (the two weights are packed on every call: they are new tensors each time)
    OffloadMLP = magi_compile(dynamic_arg_dims={"x": 0}, config_patch=patch_backend)(type("OffloadMLP", (TransformerMLP,), {}))
    plain = OffloadMLP(cfg)
    plain.load_state_dict(eager.state_dict())
    try:
        res["rewritten"] = run(plain, lambda: torch.cat([plain.gate_proj.weight, plain.up_proj.weight]).detach())
    except Exception as exc:
        res["rewritten"] = {"error": repr(exc)[:600]}
    print("RESULT " + json.dumps(res))
''')


def _run_child(tmp_path, script, timeout=900):
    path = tmp_path / "child.py"
    path.write_text(script)
    env = dict(os.environ)
    env.pop("MAGI_SWIGLU_USE_MAGI_COMPILER", None)
    proc = subprocess.run([sys.executable, str(path), str(_REF), str(ROOT)], capture_output=True, text=True,
                          timeout=timeout, env=env, cwd=str(tmp_path))
    line = [ln for ln in proc.stdout.splitlines() if ln.startswith("RESULT ")]
    assert line, proc.stdout[-3000:] + proc.stderr[-6000:]
    return json.loads(line[0][7:])


@pytest.mark.gpu
@needs_reference
def test_unmodified_reference_models_dispatch_to_the_kernel(tmp_path):
    res = _run_child(tmp_path, _BLOCK)
    assert res["through_ref"] and res["splitting"] and res["on_gpu"], res
    assert all(res["mlp_close"]) and res["mlp_calls"] == 3, res       # one kernel call per forward, three lengths
    assert all(res["block_close"]) and res["block_calls"] == 3, res


@pytest.mark.gpu
@needs_reference
def test_cuda_graph_manager_piecewise_and_full(tmp_path):
    res = _run_child(tmp_path, _GRAPHS)
    assert res["through_ref"] and res["on_gpu"] and res["status"] == 0, res
    for mode in ("PIECEWISE", "FULL"):
        assert all(res[mode]["close"]) and res[mode]["graphs"] >= 1, (mode, res)
    # PIECEWISE runs the split-point op eagerly between captured pieces: one Python call per forward.
    assert res["PIECEWISE"]["python_calls_of_the_op"] == 5, res
    # FULL captures the op itself: replays of a captured shape do not go through Python again.
    assert res["FULL"]["python_calls_of_the_op"] < 5, res


@pytest.mark.gpu
@needs_reference
def test_offload_executor_brings_new_weight_pointers_every_call(tmp_path):
    res = _run_child(tmp_path, _OFFLOAD)
    assert res["through_ref"] and res["on_gpu"], res
    for form in ("merged", "rewritten"):
        got = res[form]
        assert "error" not in got, (form, got)
        assert got["weights_stay_on_host"] and all(got["close"]) and got["calls"] == 4, (form, got)
        assert got["weight_fed_is_current"] == [True] * 4, (form, got)


@needs_reference
@pytest.mark.skipif(torch.cuda.is_available(), reason="the GPU variant of this case runs instead")
def test_child_scripts_run_without_a_gpu(tmp_path):
    """The same child script on a box without a GPU (eager backend, the CPU oracle standing in for the kernel):
    keeps the scripts themselves from rotting between GPU runs."""
    res = _run_child(tmp_path, _BLOCK)
    assert res["through_ref"] and res["splitting"] and not res["on_gpu"], res
    assert all(res["mlp_close"]) and res["mlp_calls"] == 3, res


def _run_reference_tests(tmp_path, rel, with_package):
    """Runs one of the reference's own test files; returns (passed count, set of failed test ids, output tail)."""
    tests_root = _REF / "reference_tests" if (_REF / "reference_tests").is_dir() else _REF
    tag = "with" if with_package else "without"
    env = dict(os.environ, MAGI_SWIGLU_USE_MAGI_COMPILER="1", MAGI_LOGGING_LEVEL="WARNING",
               MAGI_COMPILE_CACHE_ROOT_DIR=str(tmp_path / f"cache_{tag}"))
    stub = tmp_path / f"stub_{tag}"
    stub.mkdir()
    paths = [str(_REF), str(tests_root), str(ROOT)]
    try:
        import graphviz  # noqa: F401
    except Exception:
        if not (_REF / "graphviz.py").exists():
            (stub / "graphviz.py").write_text("class Digraph:\n    pass\n")
            paths.insert(0, str(stub))
    env["PYTHONPATH"] = os.pathsep.join(paths + [env.get("PYTHONPATH", "")])
    # -p magicompiler_b200: pytest imports this package as a plugin before it collects the reference's tests, so the
    # package's ops sit in the same registry and configuration the reference's tests then use
    plugin = ["-p", "magicompiler_b200"] if with_package else []
    cmd = [sys.executable, "-m", "pytest", "-q", "-rf", "--tb=line", "-p", "no:cacheprovider", *plugin,
           "--rootdir", str(tests_root), str(tests_root / rel)]
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=1500, env=env, cwd=str(tests_root))
    failed = {ln.split()[1] for ln in proc.stdout.splitlines() if ln.startswith("FAILED ")}
    passed = 0
    for ln in proc.stdout.splitlines():
        if " passed" in ln and ("=" in ln or "in " in ln):
            for tok_i, tok in enumerate(ln.split()):
                if tok.startswith("passed") and tok_i > 0 and ln.split()[tok_i - 1].isdigit():
                    passed = int(ln.split()[tok_i - 1])
    return passed, failed, proc.stdout[-3000:] + proc.stderr[-1500:]


def _reference_file_is_unharmed(tmp_path, rel, min_passed):
    """The reference's own tests must do with this package loaded exactly what they do without it: no test may fail
    that passes on its own.  (A few of them need a host compiler set-up for CPU Inductor that some boxes lack; those
    fail either way and are not this package's to fix.)"""
    passed_with, failed_with, tail_with = _run_reference_tests(tmp_path, rel, True)
    passed_without, failed_without, tail_without = _run_reference_tests(tmp_path, rel, False)
    assert failed_with <= failed_without, (sorted(failed_with - failed_without), tail_with)
    assert passed_with >= passed_without and passed_with >= min_passed, (passed_with, passed_without, tail_with)


@pytest.mark.gpu
@needs_reference
def test_reference_register_custom_op_tests_unharmed_by_this_package(tmp_path):
    _reference_file_is_unharmed(tmp_path, "tests/api_tests/test_register_custom_op.py", 17)


@pytest.mark.gpu
@needs_reference
def test_reference_cuda_graph_tests_unharmed_by_this_package(tmp_path):
    _reference_file_is_unharmed(tmp_path, "tests/feature_tests/test_cuda_graph.py", 3)
