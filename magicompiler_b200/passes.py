"""Full-graph rewrite pass: ``silu(linear(x, Wg)) * linear(x, Wu)``  ->  ``gemm_swiglu(x, pack(Wg, Wu))``.

This is the fusion pass MagiCompiler's ``PassConfig`` lists as a TODO (``magi_compiler/config.py:62``).  It has the
shape of the reference's own full-graph passes (``passes/full_graph/replace_sage_atten.py:21-36``: a class with
``is_applicable(graph)`` and ``__call__(graph)`` that retargets ``call_function`` nodes of the Dynamo graph) and is
meant to run where ``ReplaceSageAttentionPass`` runs, before the graph is split
(``passes/full_graph/full_graph_pass_mgr.py:27-38``), so that the new op becomes a split point.

The two ``[N,K]`` weights have to become one ``[2N,K]`` tensor.  Concatenating on every call would copy the whole
weight, so the pass routes them through ``magi_swiglu::pack_gate_up_cached``, a small op that packs once and returns
the same buffer again for as long as the same two parameter objects are passed unmodified.
"""
from __future__ import annotations

import operator
import weakref

import torch
import torch.nn.functional as F

from .register import magi_register_custom_op

try:  # the reference's pass base class (uuid by source hash), when MagiCompiler is installed
    from magi_compiler.passes.pass_base import MagiInductorPass as _PassBase  # type: ignore
except Exception:  # pragma: no cover - depends on the environment
    class _PassBase:  # same duck type: is_applicable(graph) / __call__(graph)
        def is_applicable(self, graph, shape=None) -> bool:
            return True


PACK_OP_NAME = "magi_swiglu::pack_gate_up_cached"
_pack_cache: dict[tuple[int, int], tuple] = {}


def _pack_meta(w_gate: torch.Tensor, w_up: torch.Tensor, frozen: bool = True) -> torch.Tensor:
    return w_gate.new_empty((w_gate.shape[0] + w_up.shape[0], w_gate.shape[1]))


def _pack_setup_context(ctx, inputs, output):
    ctx.gate_rows = inputs[0].shape[0]


def _pack_backward(ctx, grad):
    # the packed weight is cat([gate, up]): its gradient splits back into the two halves (training through the pass)
    return grad[: ctx.gate_rows], grad[ctx.gate_rows:], None


_retired_packs: list[torch.Tensor] = []  # packed buffers a CUDA graph may still read (see pack_gate_up_cached)


def _capturing(t: torch.Tensor) -> bool:
    return bool(t.is_cuda and torch.cuda.is_current_stream_capturing())


@magi_register_custom_op(name=PACK_OP_NAME, mutates_args=(), infer_output_meta_fn=_pack_meta,
                         setup_context_fn=_pack_setup_context, backward_fn=_pack_backward)
def _pack_gate_up_op(w_gate: torch.Tensor, w_up: torch.Tensor, frozen: bool) -> torch.Tensor:
    if w_gate.dim() != 2 or w_gate.shape != w_up.shape or w_gate.dtype != w_up.dtype or w_gate.device != w_up.device:
        raise ValueError(f"gate {tuple(w_gate.shape)}/{w_gate.dtype} and up {tuple(w_up.shape)}/{w_up.dtype} differ")
    if not frozen:
        return torch.cat([w_gate, w_up], dim=0)  # trainable weights: never memoised
    key = (id(w_gate), id(w_up))
    stamp = (w_gate._version, w_up._version, w_gate.data_ptr(), w_up.data_ptr())
    hit = _pack_cache.get(key)
    if hit is not None:
        ref_g, ref_u, old_stamp, packed, in_graph = hit
        if ref_g() is w_gate and ref_u() is w_up and old_stamp == stamp:
            if _capturing(packed) and not in_graph:
                _pack_cache[key] = (ref_g, ref_u, old_stamp, packed, True)
            return packed
        if in_graph:
            _retired_packs.append(packed)  # a captured graph may replay with this address
    packed = torch.cat([w_gate, w_up], dim=0)

    def _drop(_ref, key=key):
        entry = _pack_cache.pop(key, None)
        if entry is not None and entry[4]:
            _retired_packs.append(entry[3])

    try:
        _pack_cache[key] = (weakref.ref(w_gate, _drop), weakref.ref(w_up, _drop), stamp, packed, _capturing(packed))
    except TypeError:  # fake / functional tensors during tracing cannot be weakly referenced: do not cache
        pass
    return packed


def weights_are_frozen(w_gate: torch.Tensor, w_up: torch.Tensor) -> bool:
    """True unless a gradient can be asked for: grad mode on and either weight requiring grad."""
    return not (torch.is_grad_enabled() and (w_gate.requires_grad or w_up.requires_grad))


def pack_gate_up_cached(w_gate: torch.Tensor, w_up: torch.Tensor, frozen: bool | None = None) -> torch.Tensor:
    """``cat([w_gate, w_up])`` through the op ``magi_swiglu::pack_gate_up_cached(w_gate, w_up, frozen)``, memoised for
    FROZEN weights only.

    The memo is keyed on the identity, version counter and address of both arguments and its entry dies with either
    argument (weak references).  That key cannot see every way a training loop changes a weight (``param.data = ...``
    keeps the version counter, ``param.data.copy_()`` counts elsewhere, FSDP re-points ``param.data`` at a freshly
    gathered buffer that the allocator tends to place at the old address), so nothing is memoised while a gradient
    can be asked for: ``frozen`` defaults to ``weights_are_frozen(w_gate, w_up)`` (the rewrite pass decides the same
    way when it traces) and with ``frozen=False`` the concatenation runs on every call — one weight copy beside the
    GEMM.  Frozen weights are taken at their word; code that overwrites them behind autograd's back calls
    ``clear_pack_cache()`` afterwards.  Tensors that are new objects on every call (a weight offloaded to the host and
    brought back per iteration) are packed on every call in either mode.

    A packed buffer that was handed out while a CUDA graph was being captured is never freed by a later re-pack:
    the graph has its address baked in, so the buffer is kept for the life of the process.
    """
    if frozen is None:
        frozen = weights_are_frozen(w_gate, w_up)
    return torch.ops.magi_swiglu.pack_gate_up_cached(w_gate, w_up, bool(frozen))


def clear_pack_cache() -> None:
    """Forget every memoised packed weight (call it after overwriting frozen weights in a way autograd's version
    counter does not see).  Buffers that a captured CUDA graph may still read stay alive."""
    for entry in _pack_cache.values():
        if entry[4]:
            _retired_packs.append(entry[3])
    _pack_cache.clear()


_LINEAR_TARGETS = {F.linear, torch._C._nn.linear}
_SILU_TARGETS = {F.silu, torch.ops.aten.silu.default, torch.ops.aten.silu}
_MUL_TARGETS = {operator.mul, torch.mul, torch.ops.aten.mul.Tensor}


def _is_linear_without_bias(node: torch.fx.Node) -> bool:
    if node.op != "call_function" or node.target not in _LINEAR_TARGETS:
        return False
    bias = node.args[2] if len(node.args) > 2 else node.kwargs.get("bias")
    return bias is None and len(node.args) >= 2


def _example(node: torch.fx.Node):
    return node.meta.get("example_value", node.meta.get("val"))


def _is_bf16_on(devices: tuple[str, ...], *nodes: torch.fx.Node) -> bool:
    """The op computes bf16 on CUDA only; skip a match that is known to be something else."""
    for n in nodes:
        ev = _example(n)
        if isinstance(ev, torch.Tensor):
            if ev.dtype != torch.bfloat16 or ev.device.type not in devices:
                return False
    return True


_CHUNK_FUNCS = {torch.chunk, torch.split, torch.functional.split, torch.Tensor.chunk, torch.Tensor.split}


def _last_dim(node: torch.fx.Node):
    ev = _example(node)
    return int(ev.shape[-1]) if isinstance(ev, torch.Tensor) and isinstance(ev.shape[-1], int) else None


def _half_of(node: torch.fx.Node):
    """If ``node`` is the first or second half of another node's last dimension — ``h.chunk(2, -1)[i]``,
    ``h.split(N, -1)[i]`` or ``h[..., :N]`` / ``h[..., N:]`` with N half the width — returns
    ``(h, i, helper nodes)``; otherwise None."""
    if node.op != "call_function" or node.target is not operator.getitem or len(node.args) != 2:
        return None
    src, idx = node.args
    if not isinstance(src, torch.fx.Node):
        return None
    if isinstance(idx, int) and idx in (0, 1):  # an element of chunk(...) / split(...)
        is_fn = src.op == "call_function" and src.target in _CHUNK_FUNCS
        is_method = src.op == "call_method" and src.target in ("chunk", "split")
        if not (is_fn or is_method) or not src.args or not isinstance(src.args[0], torch.fx.Node):
            return None
        h = src.args[0]
        arg = src.args[1] if len(src.args) > 1 else src.kwargs.get("chunks", src.kwargs.get("split_size_or_sections"))
        dim = src.args[2] if len(src.args) > 2 else src.kwargs.get("dim", 0)
        ev = _example(h)
        rank = ev.dim() if isinstance(ev, torch.Tensor) else None
        if not (dim == -1 or (rank is not None and dim == rank - 1)):
            return None
        name = src.target if isinstance(src.target, str) else getattr(src.target, "__name__", "")
        if name == "chunk":
            if arg != 2:
                return None
        else:  # split: exactly two pieces of half the width
            width = _last_dim(h)
            if width is None or not isinstance(arg, int) or 2 * arg != width:
                return None
        return h, idx, (src,)
    if isinstance(idx, tuple) and idx and isinstance(idx[-1], slice):  # h[..., :N] / h[:, N:]
        lead, last = idx[:-1], idx[-1]
        if not all(e is Ellipsis or (isinstance(e, slice) and e == slice(None)) for e in lead):
            return None
        ev = _example(src)
        if not isinstance(ev, torch.Tensor):
            return None
        if Ellipsis not in lead and len(idx) != ev.dim():
            return None
        width = _last_dim(src)
        if width is None or width % 2 or last.step not in (None, 1):
            return None
        half = width // 2
        if last.start in (None, 0) and last.stop == half:
            return src, 0, ()
        if last.start == half and last.stop in (None, width):
            return src, 1, ()
    return None


class FuseSwiGLUPass(_PassBase):
    """Rewrites every ``silu(linear(x, Wg)) * linear(x, Wu)`` (either operand order, bias-free linears that share
    ``x``) of a Dynamo-level FX graph into ``gemm_swiglu(x, pack_gate_up_cached(Wg, Wu))``, and the merged-projection
    form ``h = linear(x, W); silu(h[..., :N]) * h[..., N:]`` (``chunk``, ``split`` or slices; the SiluAndMul layout of
    the ops magi_compiler/passes/piecewise_graph/fix_functionalization.py:100-125 handles) into ``gemm_swiglu(x, W)``.

    ``allowed_devices``: device types of the traced tensors for which the rewrite is made (the kernel exists for
    CUDA; "meta" lets shape-only traces through; tests that stand a CPU function in for the kernel add "cpu").
    ``save_preactivations``: True emits the two-output training op ``gemm_swiglu_preact`` (its backward reads the kept
    ``[M, 2N]`` pre-activations instead of recomputing them) and uses its first output; False emits ``gemm_swiglu``
    (its backward recomputes); None (default) decides per match: the training op when the graph is traced with grad
    mode on and the activations or a weight require grad, else the plain op."""

    def __init__(self, allowed_devices: tuple[str, ...] = ("cuda", "meta"), save_preactivations: bool | None = None):
        self.allowed_devices = tuple(allowed_devices)
        self.save_preactivations = save_preactivations

    def _keep_preactivations(self, *nodes: torch.fx.Node) -> bool:
        if self.save_preactivations is not None:
            return bool(self.save_preactivations)
        if not torch.is_grad_enabled():
            return False
        return any(isinstance(_example(n), torch.Tensor) and _example(n).requires_grad for n in nodes)

    @staticmethod
    def _frozen(*weights: torch.fx.Node) -> bool:
        """Whether the traced weights may be memoised once packed: only when the trace shows that no gradient can be
        asked for (grad mode off, or every weight known not to require grad); unknown counts as trainable."""
        if not torch.is_grad_enabled():
            return True
        evs = [_example(w) for w in weights]
        return all(isinstance(ev, torch.Tensor) and not ev.requires_grad for ev in evs)

    def _matches(self, graph: torch.fx.Graph):
        found = []
        for mul in graph.nodes:
            is_mul = (mul.op == "call_function" and mul.target in _MUL_TARGETS) or \
                     (mul.op == "call_method" and mul.target == "mul")
            if not is_mul or len(mul.args) != 2 or not all(isinstance(a, torch.fx.Node) for a in mul.args):
                continue
            for act, up in (mul.args, mul.args[::-1]):
                is_silu = (act.op == "call_function" and act.target in _SILU_TARGETS) or \
                          (act.op == "call_method" and act.target == "silu")
                if not is_silu or not act.args or not isinstance(act.args[0], torch.fx.Node):
                    continue
                gate = act.args[0]
                if not (_is_linear_without_bias(gate) and _is_linear_without_bias(up)):
                    continue
                if gate.args[0] is not up.args[0] or gate is up:
                    continue
                if len(act.users) != 1 or len(gate.users) != 1 or len(up.users) != 1:
                    continue  # an intermediate is used elsewhere: it must stay materialised
                wg, wu = gate.args[1], up.args[1]
                if not (isinstance(wg, torch.fx.Node) and isinstance(wu, torch.fx.Node)):
                    continue
                # the activations decide where the op runs; weights may be traced on the host when an offload executor
                # brings them to the GPU call by call (magi_compiler/offload/offload_warpper.py:100-131)
                if not _is_bf16_on(self.allowed_devices, gate.args[0]) or \
                        not _is_bf16_on(self.allowed_devices + ("cpu",), wg, wu):
                    continue
                evg, evu = _example(wg), _example(wu)
                if isinstance(evg, torch.Tensor) and isinstance(evu, torch.Tensor):
                    if evg.dim() != 2 or evg.shape != evu.shape or evg.shape[0] % 8 or evg.shape[1] % 8:
                        continue
                found.append((mul, act, gate, up))
                break
        return found

    def _matches_merged(self, graph: torch.fx.Graph):
        """``h = linear(x, W_gate_up); silu(h[..., :N]) * h[..., N:]`` (chunk, split or slices): the merged-projection
        form, whose weight is already packed gate rows first."""
        found = []
        for mul in graph.nodes:
            is_mul = (mul.op == "call_function" and mul.target in _MUL_TARGETS) or \
                     (mul.op == "call_method" and mul.target == "mul")
            if not is_mul or len(mul.args) != 2 or not all(isinstance(a, torch.fx.Node) for a in mul.args):
                continue
            for act, up in (mul.args, mul.args[::-1]):
                is_silu = (act.op == "call_function" and act.target in _SILU_TARGETS) or \
                          (act.op == "call_method" and act.target == "silu")
                if not is_silu or not act.args or not isinstance(act.args[0], torch.fx.Node):
                    continue
                gate = act.args[0]
                hg, hu = _half_of(gate), _half_of(up)
                if hg is None or hu is None or hg[0] is not hu[0] or (hg[1], hu[1]) != (0, 1):
                    continue
                lin = hg[0]
                helpers = tuple(dict.fromkeys(hg[2] + hu[2]))
                if not _is_linear_without_bias(lin) or not isinstance(lin.args[1], torch.fx.Node):
                    continue
                if len(act.users) != 1 or len(gate.users) != 1 or len(up.users) != 1:
                    continue
                inner = set(helpers) | {gate, up}
                if any(u not in inner for u in lin.users) or any(u not in (gate, up) for hn in helpers for u in hn.users):
                    continue  # the merged projection (or a piece of it) is used elsewhere: it must stay
                if not _is_bf16_on(self.allowed_devices, lin.args[0]) or \
                        not _is_bf16_on(self.allowed_devices + ("cpu",), lin.args[1]):
                    continue
                evw = _example(lin.args[1])
                if isinstance(evw, torch.Tensor) and (evw.dim() != 2 or evw.shape[0] % 16 or evw.shape[1] % 8):
                    continue
                found.append((mul, act, gate, up, helpers, lin))
                break
        return found

    def is_applicable(self, graph: torch.fx.Graph, shape: int | None = None) -> bool:
        return bool(self._matches(graph)) or bool(self._matches_merged(graph))

    def __call__(self, graph: torch.fx.Graph) -> int:
        from .ops import gemm_swiglu  # registers the op

        count = 0
        for mul, act, gate, up in self._matches(graph):
            x, wg, wu = gate.args[0], gate.args[1], up.args[1]
            with graph.inserting_before(mul):
                packed = graph.call_function(torch.ops.magi_swiglu.pack_gate_up_cached.default,
                                             (wg, wu, self._frozen(wg, wu)))
                if self._keep_preactivations(x, wg, wu):
                    both = graph.call_function(torch.ops.magi_swiglu.gemm_swiglu_preact.default, (x, packed))
                    fused = graph.call_function(operator.getitem, (both, 0))
                else:
                    fused = graph.call_function(torch.ops.magi_swiglu.gemm_swiglu.default, (x, packed))
            for new, fn in ((packed, _pack_meta), (fused, None)):
                try:  # carry shape metadata forward when the graph has it (fake tensors from Dynamo)
                    if fn is not None:
                        new.meta["example_value"] = fn(_example(wg), _example(wu))
                    else:
                        ex, ep = _example(x), packed.meta["example_value"]
                        new.meta["example_value"] = ex.new_empty((*ex.shape[:-1], ep.shape[0] // 2))
                except Exception:
                    pass
            mul.replace_all_uses_with(fused)
            for dead in (mul, act, gate, up):
                graph.erase_node(dead)
            count += 1
        for mul, act, gate, up, helpers, lin in self._matches_merged(graph):
            x, packed = lin.args[0], lin.args[1]
            with graph.inserting_before(mul):
                if self._keep_preactivations(x, packed):
                    both = graph.call_function(torch.ops.magi_swiglu.gemm_swiglu_preact.default, (x, packed))
                    fused = graph.call_function(operator.getitem, (both, 0))
                else:
                    fused = graph.call_function(torch.ops.magi_swiglu.gemm_swiglu.default, (x, packed))
            try:
                ex, ep = _example(x), _example(packed)
                fused.meta["example_value"] = ex.new_empty((*ex.shape[:-1], ep.shape[0] // 2))
            except Exception:
                pass
            mul.replace_all_uses_with(fused)
            for dead in (mul, act, gate, up, *helpers, lin):
                graph.erase_node(dead)
            count += 1
        if count:
            graph.lint()
        return count


def install_into_magi_compiler(allowed_devices: tuple[str, ...] = ("cuda", "meta"),
                               save_preactivations: bool | None = None) -> bool:
    """Opt-in: make MagiCompiler's ``FullGraphPassManager`` run ``FuseSwiGLUPass`` first.  Returns False when
    MagiCompiler is not importable.  (Upstream, the same effect is two lines in ``full_graph_pass_mgr.py``.)"""
    try:
        from magi_compiler.passes.full_graph import full_graph_pass_mgr as mgr  # type: ignore
    except Exception:
        return False
    cls = mgr.FullGraphPassManager
    if getattr(cls, "_magi_swiglu_installed", False):
        return True
    original_init = cls.__init__

    def patched_init(self, pass_config):
        original_init(self, pass_config)
        self.passes.insert(0, FuseSwiGLUPass(allowed_devices, save_preactivations))

    cls.__init__ = patched_init
    cls._magi_swiglu_installed = True
    return True
