"""Registration surface of the op: MagiCompiler's ``magi_register_custom_op`` when that package is
installed, otherwise a mirror with the same arguments and behaviour.

Mirrors ``magi_compiler/_magi_register_custom_op.py:168-204`` (public wrapper ``magi_compiler/api.py:197-293``):
one decorator that (1) creates a ``torch.library.custom_op`` whose schema is inferred from the type
hints, (2) registers the fake/meta implementation — ``None`` = outputs look like the first tensor
inputs, ``list[str]`` = outputs look like the named parameters, callable = used as given — (3)
optionally registers autograd, and (4) records the op name as a graph-split point
(``is_subgraph_boundary``) and/or as compute-sensitive for the recompute partitioner
(``is_compute_sensitive``).  With MagiCompiler present those two lists live in its global compile
config (``magi_compiler/config.py:296-313``); without it they are kept here in ``SPLITTING_OPS`` and
``COMPUTE_SENSITIVE_OPS`` so an integration can read them.
"""
from __future__ import annotations

import importlib.util
import inspect
import os
import re
from pathlib import Path
from typing import Callable, get_args, get_origin

import torch

SPLITTING_OPS: list[str] = []
COMPUTE_SENSITIVE_OPS: list[str] = []


def _reference_decorator():
    """MagiCompiler's own decorator, or None when the package is absent or disabled."""
    if os.environ.get("MAGI_SWIGLU_USE_MAGI_COMPILER", "1") == "0":
        return None
    try:
        if importlib.util.find_spec("magi_compiler") is None:
            return None
        from magi_compiler import magi_register_custom_op as ref  # type: ignore

        return ref
    except Exception:  # an unusable installation must not take the op down with it
        return None


def _num_outputs(fn: Callable) -> int:
    ann = inspect.signature(fn).return_annotation
    if ann is inspect.Parameter.empty:
        return 1
    if get_origin(ann) is tuple:
        args = get_args(ann)
        if args and args[-1] is not ...:
            return len(args)
    return 1


def _auto_name(fn: Callable) -> str:
    try:
        ns = re.sub(r"[^a-zA-Z0-9_]", "_", Path(inspect.getfile(fn)).stem)
    except (TypeError, OSError):
        ns = "magi_custom"
    return f"{ns}::{fn.__name__}"


def _meta_like_first_inputs(fn: Callable) -> Callable:
    n_out = _num_outputs(fn)
    sig = inspect.signature(fn)

    def meta(*args, **kwargs):
        bound = sig.bind(*args, **kwargs)
        bound.apply_defaults()
        tensors = [v for k, v in bound.arguments.items() if k != "self" and isinstance(v, torch.Tensor)][:n_out]
        if len(tensors) < n_out:
            raise ValueError(f"the default meta function needs {n_out} tensor inputs for {n_out} outputs, found "
                             f"{len(tensors)}; pass infer_output_meta_fn")
        outs = tuple(torch.empty_like(t) for t in tensors)
        return outs[0] if n_out == 1 else outs

    return meta


def _meta_like_named(fn: Callable, names: list[str]) -> Callable:
    sig = inspect.signature(fn)

    def meta(*args, **kwargs):
        bound = sig.bind(*args, **kwargs)
        bound.apply_defaults()
        outs = []
        for name in names:
            if name not in bound.arguments:
                raise ValueError(f"parameter '{name}' is not in the signature {list(bound.arguments)}")
            if not isinstance(bound.arguments[name], torch.Tensor):
                raise ValueError(f"parameter '{name}' is not a Tensor")
            outs.append(torch.empty_like(bound.arguments[name]))
        return outs[0] if len(outs) == 1 else tuple(outs)

    return meta


def magi_register_custom_op(
    name: str | None = None,
    mutates_args: tuple[str, ...] = (),
    infer_output_meta_fn: Callable | list[str] | None = None,
    setup_context_fn: Callable | None = None,
    backward_fn: Callable | None = None,
    is_compute_sensitive: bool = False,
    is_subgraph_boundary: bool = False,
):
    """Same signature and meaning as ``magi_compiler.magi_register_custom_op``."""
    ref = _reference_decorator()
    if ref is not None:
        return ref(name=name, mutates_args=mutates_args, infer_output_meta_fn=infer_output_meta_fn,
                   setup_context_fn=setup_context_fn, backward_fn=backward_fn,
                   is_compute_sensitive=is_compute_sensitive, is_subgraph_boundary=is_subgraph_boundary)

    def decorator(fn: Callable):
        op_name = name if name is not None else _auto_name(fn)
        if is_compute_sensitive:
            COMPUTE_SENSITIVE_OPS.append(op_name)
        if is_subgraph_boundary:
            SPLITTING_OPS.append(op_name)
        op = torch.library.custom_op(op_name, mutates_args=mutates_args)(fn)
        if infer_output_meta_fn is None:
            meta = _meta_like_first_inputs(fn)
        elif isinstance(infer_output_meta_fn, list):
            meta = _meta_like_named(fn, infer_output_meta_fn)
        else:
            meta = infer_output_meta_fn
        torch.library.register_fake(op_name)(meta)
        if backward_fn is not None:
            op.register_autograd(backward_fn, setup_context=setup_context_fn)
        return op

    return decorator


def registered_through_magi_compiler() -> bool:
    return _reference_decorator() is not None
