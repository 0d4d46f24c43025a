"""``magi_swiglu::gemm_swiglu`` — the fused GEMM-SwiGLU custom op, registered the MagiCompiler way.

    y = gemm_swiglu(x, w_gate_up)      y[..., n] = silu(x · Wg[n]) * (x · Wu[n])

``w_gate_up`` is ``[2N, K]`` = ``cat([gate_proj.weight, up_proj.weight])`` (``nn.Linear`` layout, gate
rows first), replacing ``F.silu(self.gate_proj(x)) * self.up_proj(x)`` of the reference's
``TransformerMLP`` (tests/model_definition.py:332-339) and ``F.silu(self.w1(x)) * self.w3(x)`` of its
Llama example (example/training/llama3.py:168-173).

Registration follows ``magi_compiler/_magi_register_custom_op.py:168-204``: functional
(``mutates_args=()``), callable fake impl that works with a symbolic row count, marked as a graph split
point and as compute-sensitive.  The body validates its arguments on the host, allocates the output
with ``torch.empty`` (capture-aware caching allocator) and makes ONE call into the C-ABI library on
torch's current stream: no synchronisation, no host read, no allocation inside the library — so it can
run on a side stream, under an offload executor and inside CUDA-graph capture
(magi_compiler/magi_backend/cuda_graph_mgr.py:465-473, 548-569).

Dtype rules (enforced before any launch): x and w_gate_up are bf16 CUDA tensors on the same device;
the output is bf16 on that device.  There is no fp16/fp32 path, no CPU path and no fallback.
"""
from __future__ import annotations

import ctypes
import os

import torch

from . import _loader
from .register import magi_register_custom_op

OP_NAME = "magi_swiglu::gemm_swiglu"


def _check(x: torch.Tensor, w: torch.Tensor) -> tuple[int, int, int]:
    if not isinstance(x, torch.Tensor) or not isinstance(w, torch.Tensor):
        raise TypeError("gemm_swiglu expects two tensors")
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise TypeError(f"gemm_swiglu computes in bf16 only; got x {x.dtype}, w_gate_up {w.dtype}")
    if w.dim() != 2:
        raise ValueError(f"w_gate_up must be 2-D [2N, K]; got shape {tuple(w.shape)}")
    if x.dim() < 1:
        raise ValueError("x must have at least one dimension [..., K]")
    if w.shape[0] % 2 != 0:
        raise ValueError(f"w_gate_up has {w.shape[0]} rows; it must hold N gate rows followed by N up rows")
    K = x.shape[-1]
    N = w.shape[0] // 2
    if w.shape[1] != K:
        raise ValueError(f"inner dimensions differ: x[..., {K}] vs w_gate_up[{w.shape[0]}, {w.shape[1]}]")
    if K == 0 or N == 0:
        raise ValueError("K and N must be positive")
    if K % 8 != 0 or N % 8 != 0:
        raise ValueError(f"K ({K}) and N ({N}) must be multiples of 8 (16-byte rows for TMA and vector stores)")
    if not x.is_cuda or not w.is_cuda:
        raise TypeError("gemm_swiglu runs on CUDA tensors only (there is no CPU implementation)")
    if x.device != w.device:
        raise ValueError(f"x is on {x.device} but w_gate_up is on {w.device}")
    M = x.numel() // K
    return M, N, K


def _rows_view(t: torch.Tensor, cols: int) -> torch.Tensor:
    """2-D view with unit inner stride, 8-element-aligned row stride and a 16-byte-aligned base (copy if not)."""
    t2 = t.reshape(-1, cols)
    ok = t2.stride(1) == 1 and (t2.shape[0] <= 1 or (t2.stride(0) >= cols and t2.stride(0) % 8 == 0)) \
        and t2.data_ptr() % 16 == 0
    return t2 if ok else t2.contiguous()


def _workspace(device: torch.device, nbytes: int) -> torch.Tensor:
    """Scratch for one split-K call, taken from torch's caching allocator on the current stream and dropped when the
    call returns.  The allocator orders the block's reuse after this stream's work, keeps it apart from launches on
    other streams, and, under CUDA-graph capture, gives it to the graph's private pool for as long as the graph lives
    — so no captured graph can be left with a dangling scratch address and nothing accumulates per stream.  The
    library itself allocates nothing."""
    return torch.empty(nbytes, dtype=torch.uint8, device=device)


_ws_need: dict[tuple, int] = {}  # (M, N, K, schedule knobs, device) -> scratch bytes the preferred schedule wants


def _raw_stream(device_index: int) -> int:
    return torch._C._cuda_getCurrentRawStream(device_index)


def gemm_swiglu_out(x: torch.Tensor, w_gate_up: torch.Tensor, out: torch.Tensor | None = None, *,
                    variant: str | int = "auto", block_n: int = 0, stages: int = 0, group_m: int = 0,
                    max_ctas: int = 0) -> torch.Tensor:
    """The op's body with the schedule knobs of ``magi_swiglu_forward_bf16_ws`` exposed (tests, tuning).

    The host path is kept short (decode-sized calls finish on the GPU in 20-30 us): contiguous operands skip the
    re-striding helper and the scratch size of a shape is asked from the library once."""
    M, N, K = _check(x, w_gate_up)
    lib = _loader.load_library()
    x2 = x if (x.dim() == 2 and x.is_contiguous() and x.data_ptr() % 16 == 0) else _rows_view(x, K)
    if w_gate_up.is_contiguous() and w_gate_up.data_ptr() % 16 == 0:
        w2 = w_gate_up
    else:
        w2 = _rows_view(w_gate_up, K)
        if w2.data_ptr() != w_gate_up.data_ptr() and w_gate_up.numel() > 0:
            # a copy of the weight on every call would double the op's HBM traffic
            raise ValueError("w_gate_up must have unit inner stride, a row stride that is a multiple of 8 and a "
                             "16-byte-aligned base; pack it once with magicompiler_b200.pack_gate_up")
    if out is None:
        y = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    else:
        out_shape = (*x.shape[:-1], N)
        if out.dtype != torch.bfloat16 or out.device != x.device or tuple(out.shape) != tuple(out_shape):
            raise ValueError("out must be a bf16 tensor of the output shape on x's device")
        y = out.reshape(M, N)
        if y.data_ptr() != out.data_ptr() or y.stride(1) != 1 or y.stride(0) % 8 != 0 or y.data_ptr() % 16 != 0:
            raise ValueError("out must be row-contiguous with a 16-byte-aligned base")
    if M == 0:
        return y.view(*x.shape[:-1], N)
    v = _loader.VARIANTS[variant] if isinstance(variant, str) else int(variant)
    dev = x.device.index if x.device.index is not None else torch.cuda.current_device()
    stream = _raw_stream(dev)
    ldx = x2.stride(0) if M > 1 else K
    # scratch: the small-M schedules split K through it, the tile schedules balance their last waves through it
    ws_ptr, ws_len = None, 0
    key = (M, N, K, v, block_n, stages, group_m, max_ctas, dev, _split_env())
    need = _ws_need.get(key)
    if need is None:
        need = lib.magi_swiglu_workspace_bytes(M, N, K, v, block_n, stages, group_m, max_ctas, dev, 0)
        _ws_need[key] = need
    if need > 0:
        ws = _workspace(x.device, need)
        ws_ptr, ws_len = ws.data_ptr(), ws.numel()
    rc = lib.magi_swiglu_forward_bf16_ws(x2.data_ptr(), w2.data_ptr(), y.data_ptr(), M, N, K, ldx, w2.stride(0),
                                         y.stride(0), dev, stream, v, block_n, stages, group_m, max_ctas,
                                         ws_ptr, ws_len)
    if rc != 0:
        msg = f"magi_swiglu_forward_bf16 failed ({rc}): {_loader.last_error()}"
        raise (ValueError(msg) if rc < 0 else RuntimeError(msg))
    return y if x.dim() == 2 else y.view(*x.shape[:-1], N)


def _split_env() -> int:
    return _loader.tuning_epoch()  # a changed tuning aid of the library changes the scratch a shape wants


RMS_OP_NAME = "magi_swiglu::rmsnorm_gemm_swiglu"


def fold_rmsnorm_weight(w_gate_up: torch.Tensor, norm_weight: torch.Tensor) -> torch.Tensor:
    """Fold an RMSNorm weight (``[K]``) into the packed gate/up weight (``[2N, K]``): ``W'[n, k] = W[n, k] * g[k]``
    (computed in fp32, rounded once).  Do this once at load; ``rmsnorm_gemm_swiglu`` then needs only the row scales."""
    if norm_weight.dim() != 1 or norm_weight.shape[0] != w_gate_up.shape[1]:
        raise ValueError(f"norm weight {tuple(norm_weight.shape)} does not match K={w_gate_up.shape[1]}")
    return (w_gate_up.float() * norm_weight.float().to(w_gate_up.device)).to(w_gate_up.dtype).contiguous()


@magi_register_custom_op(name=RMS_OP_NAME, mutates_args=(),
                         infer_output_meta_fn=lambda x, w_folded, eps: x.new_empty((*x.shape[:-1], w_folded.shape[0] // 2)),
                         is_compute_sensitive=True, is_subgraph_boundary=True)
def rmsnorm_gemm_swiglu(x: torch.Tensor, w_folded: torch.Tensor, eps: float) -> torch.Tensor:
    """``gemm_swiglu(rmsnorm(x), w)`` in two launches and without materialising the normalised activations:
    a row-scale kernel computes ``rsqrt(mean(x^2) + eps)`` and the fused kernel multiplies both accumulators of a
    row by it before the activation.  ``w_folded`` = ``fold_rmsnorm_weight(w_gate_up, norm.weight)``.
    Replaces ``self.mlp(self.post_attention_layernorm(x))`` up to the down projection
    (MagiCompiler tests/model_definition.py:42-56, 360-361)."""
    M, N, K = _check(x, w_folded)
    lib = _loader.load_library()
    x2 = x if (x.dim() == 2 and x.is_contiguous() and x.data_ptr() % 16 == 0) else _rows_view(x, K)
    if not w_folded.is_contiguous() or w_folded.data_ptr() % 16:
        raise ValueError("w_folded must be contiguous and 16-byte aligned")
    y = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    if M == 0:
        return y.view(*x.shape[:-1], N)
    dev = x.device.index if x.device.index is not None else torch.cuda.current_device()
    stream = _raw_stream(dev)
    scale = torch.empty((M,), dtype=torch.float32, device=x.device)
    ldx = x2.stride(0) if M > 1 else K
    rc = lib.magi_swiglu_row_rms_f32(x2.data_ptr(), scale.data_ptr(), M, K, ldx, float(eps), dev, stream)
    if rc == 0:
        ws_ptr, ws_len = None, 0
        if M <= 128:
            need = lib.magi_swiglu_workspace_bytes(M, N, K, 0, 0, 0, 0, 0, dev, 0)
            if need > 0:
                ws = _workspace(x.device, need)
                ws_ptr, ws_len = ws.data_ptr(), ws.numel()
        rc = lib.magi_swiglu_forward_bf16_scaled(x2.data_ptr(), w_folded.data_ptr(), y.data_ptr(), scale.data_ptr(), M, N,
                                                 K, ldx, K, N, dev, stream, ws_ptr, ws_len)
    if rc != 0:
        msg = f"rmsnorm_gemm_swiglu failed ({rc}): {_loader.last_error()}"
        raise (ValueError(msg) if rc < 0 else RuntimeError(msg))
    return y if x.dim() == 2 else y.view(*x.shape[:-1], N)


GEMM_NT_OP_NAME = "magi_swiglu::gemm_nt"


def gemm_nt_out(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """``F.linear(a, b)`` on the tile kernels, written into ``out`` (``[M, N]`` bf16, unit inner stride, row stride a
    multiple of 8, 16-byte-aligned base — e.g. a row slice of a larger result) when given: no copy afterwards."""
    if a.dtype != torch.bfloat16 or b.dtype != torch.bfloat16:
        raise TypeError("gemm_nt computes in bf16 only")
    if not (a.is_cuda and b.is_cuda) or a.device != b.device:
        raise TypeError("gemm_nt runs on CUDA tensors of one device")
    if b.dim() != 2 or a.dim() < 1 or a.shape[-1] != b.shape[1] or b.shape[0] % 16 or b.shape[1] % 8 or b.shape[1] == 0:
        raise ValueError(f"shapes do not fit: a {tuple(a.shape)}, b {tuple(b.shape)} (need [..,K], [N,K], N % 16 == 0, K % 8 == 0)")
    n, k = b.shape
    a2, b2 = _rows_view(a, k), _rows_view(b, k)
    m = a2.shape[0]
    if out is None:
        c = torch.empty((m, n), dtype=torch.bfloat16, device=a.device)
    else:
        c = out
        if c.dtype != torch.bfloat16 or c.device != a.device or tuple(c.shape) != (m, n) or c.stride(1) != 1 \
                or (m > 1 and (c.stride(0) < n or c.stride(0) % 8)) or c.data_ptr() % 16:
            raise ValueError("out must be a bf16 [M, N] tensor on a's device with unit inner stride, a row stride that "
                             "is a multiple of 8 and a 16-byte-aligned base")
    if m > 0:
        dev = a.device.index if a.device.index is not None else torch.cuda.current_device()
        rc = _loader.load_library().magi_swiglu_gemm_nt_bf16(
            a2.data_ptr(), b2.data_ptr(), c.data_ptr(), m, n, k, a2.stride(0) if m > 1 else k, b2.stride(0),
            c.stride(0) if m > 1 else n, dev, torch.cuda.current_stream(a.device).cuda_stream)
        if rc != 0:
            msg = f"magi_swiglu_gemm_nt_bf16 failed ({rc}): {_loader.last_error()}"
            raise (ValueError(msg) if rc < 0 else RuntimeError(msg))
    return c if out is not None else c.view(*a.shape[:-1], n)


gemm_nt_out.supports_out = True  # TensorParallelSwiGLUMLP passes its result slice as out=


def scatter_setup(dest_set: int, dst_ptrs: list[int], rows_per_owner: int, n: int, ldc: int | None = None,
                  device: int | None = None) -> None:
    """Tell the library where block ``o`` of a scattered GEMM's rows goes (``magi_swiglu_scatter_setup``): ``dst_ptrs[o]``
    is the address, valid in this process, of a ``[rows_per_owner, n]`` bf16 matrix that may live on another GPU."""
    dev = torch.cuda.current_device() if device is None else device
    arr = (ctypes.c_void_p * len(dst_ptrs))(*dst_ptrs)
    rc = _loader.load_library().magi_swiglu_scatter_setup(dev, dest_set, arr, len(dst_ptrs), rows_per_owner, n,
                                                           n if ldc is None else ldc)
    if rc != 0:
        msg = f"magi_swiglu_scatter_setup failed ({rc}): {_loader.last_error()}"
        raise (ValueError(msg) if rc < 0 else RuntimeError(msg))


def gemm_nt_scatter(a: torch.Tensor, b: torch.Tensor, dest_set: int) -> None:
    """``F.linear(a, b)`` whose row blocks leave the epilogue straight into the destinations of ``dest_set``
    (``magi_swiglu_gemm_nt_bf16_scatter``); nothing is returned and nothing is ordered between GPUs."""
    if a.dtype != torch.bfloat16 or b.dtype != torch.bfloat16 or not (a.is_cuda and b.is_cuda) or a.device != b.device:
        raise TypeError("gemm_nt_scatter computes in bf16 on CUDA tensors of one device")
    if b.dim() != 2 or a.dim() != 2 or a.shape[1] != b.shape[1]:
        raise ValueError(f"shapes do not fit: a {tuple(a.shape)}, b {tuple(b.shape)} (need [M,K], [N,K])")
    n, k = b.shape
    a2, b2 = _rows_view(a, k), _rows_view(b, k)
    m = a2.shape[0]
    dev = a.device.index if a.device.index is not None else torch.cuda.current_device()
    rc = _loader.load_library().magi_swiglu_gemm_nt_bf16_scatter(
        a2.data_ptr(), b2.data_ptr(), dest_set, m, n, k, a2.stride(0), b2.stride(0), dev,
        torch.cuda.current_stream(a.device).cuda_stream, None, 0)  # whole tiles, like gemm_nt: no scratch
    if rc != 0:
        msg = f"magi_swiglu_gemm_nt_bf16_scatter failed ({rc}): {_loader.last_error()}"
        raise (ValueError(msg) if rc < 0 else RuntimeError(msg))


def sum_slots(src: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """``src[0] + src[1] + ...`` over the first dimension (bf16, contiguous), fp32 sums in slot order, one rounding
    (``magi_swiglu_sum_slots_bf16``)."""
    if src.dtype != torch.bfloat16 or not src.is_cuda or not src.is_contiguous() or src.dim() < 2:
        raise TypeError("sum_slots takes a contiguous bf16 CUDA tensor [slots, ...]")
    slots, n = src.shape[0], src[0].numel()
    if out is None:
        out = torch.empty(src.shape[1:], dtype=torch.bfloat16, device=src.device)
    elif out.dtype != torch.bfloat16 or out.device != src.device or out.numel() != n or not out.is_contiguous():
        raise ValueError("out must be a contiguous bf16 tensor of one slot's size on src's device")
    dev = src.device.index if src.device.index is not None else torch.cuda.current_device()
    rc = _loader.load_library().magi_swiglu_sum_slots_bf16(src.data_ptr(), out.data_ptr(), slots, n, n, dev,
                                                            torch.cuda.current_stream(src.device).cuda_stream)
    if rc != 0:
        msg = f"magi_swiglu_sum_slots_bf16 failed ({rc}): {_loader.last_error()}"
        raise (ValueError(msg) if rc < 0 else RuntimeError(msg))
    return out


def sum_slots_bcast(src: torch.Tensor, dst_ptrs: list[int]) -> None:
    """``sum_slots`` stored to every address in ``dst_ptrs`` (``magi_swiglu_sum_slots_bf16_bcast``): the same block of
    the result in the memory of every GPU of a group, peers' memory mapped into this process."""
    if src.dtype != torch.bfloat16 or not src.is_cuda or not src.is_contiguous() or src.dim() < 2:
        raise TypeError("sum_slots_bcast takes a contiguous bf16 CUDA tensor [slots, ...]")
    slots, n = src.shape[0], src[0].numel()
    arr = (ctypes.c_void_p * len(dst_ptrs))(*dst_ptrs)
    dev = src.device.index if src.device.index is not None else torch.cuda.current_device()
    rc = _loader.load_library().magi_swiglu_sum_slots_bf16_bcast(src.data_ptr(), arr, len(dst_ptrs), slots, n, n, dev,
                                                                  torch.cuda.current_stream(src.device).cuda_stream)
    if rc != 0:
        msg = f"magi_swiglu_sum_slots_bf16_bcast failed ({rc}): {_loader.last_error()}"
        raise (ValueError(msg) if rc < 0 else RuntimeError(msg))


@magi_register_custom_op(name=GEMM_NT_OP_NAME, mutates_args=(),
                         infer_output_meta_fn=lambda a, b: a.new_empty((*a.shape[:-1], b.shape[0])),
                         is_compute_sensitive=True)
def gemm_nt(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """``a @ b.T`` (``F.linear(a, b)``) in bf16 on the tile kernels of the fused op (``magi_swiglu_gemm_nt_bf16``):
    ``a`` is ``[..., K]``, ``b`` is ``[N, K]`` with N a multiple of 16; fp32 accumulation, one rounding."""
    return gemm_nt_out(a, b)


GEMM_OP_NAME = "magi_swiglu::gemm_bf16"


def _gemm_bf16_meta(a: torch.Tensor, b: torch.Tensor, a_is_km: bool, b_is_kn: bool) -> torch.Tensor:
    return a.new_empty((a.shape[1] if a_is_km else a.shape[0], b.shape[1] if b_is_kn else b.shape[0]))


@magi_register_custom_op(name=GEMM_OP_NAME, mutates_args=(), infer_output_meta_fn=_gemm_bf16_meta,
                         is_compute_sensitive=True)
def gemm_bf16(a: torch.Tensor, b: torch.Tensor, a_is_km: bool, b_is_kn: bool) -> torch.Tensor:
    """``(a.T if a_is_km else a) @ (b if b_is_kn else b.T)`` for 2-D bf16 CUDA tensors on the tile kernels
    (``magi_swiglu_gemm_bf16``): ``a`` is ``[M, K]`` or, with ``a_is_km``, ``[K, M]``; ``b`` is ``[N, K]`` or, with
    ``b_is_kn``, ``[K, N]``.  Nothing is transposed in memory: an operand stored the other way round is loaded as an
    MN-major tile.  N % 16 == 0; fp32 accumulation, one rounding.  Used for dX = dH · W and dW = dH^T · X."""
    if a.dtype != torch.bfloat16 or b.dtype != torch.bfloat16:
        raise TypeError("gemm_bf16 computes in bf16 only")
    if not (a.is_cuda and b.is_cuda) or a.device != b.device:
        raise TypeError("gemm_bf16 runs on CUDA tensors of one device")
    if a.dim() != 2 or b.dim() != 2:
        raise ValueError(f"gemm_bf16 takes 2-D operands, got {tuple(a.shape)} and {tuple(b.shape)}")
    m, k = (a.shape[1], a.shape[0]) if a_is_km else (a.shape[0], a.shape[1])
    n, kb = (b.shape[1], b.shape[0]) if b_is_kn else (b.shape[0], b.shape[1])
    if k != kb or k == 0 or n % 16 or (a_is_km and m % 8) or (not (a_is_km and b_is_kn) and k % 8) or k % 8:
        raise ValueError(f"shapes do not fit: a {tuple(a.shape)} (a_is_km={a_is_km}), b {tuple(b.shape)} "
                         f"(b_is_kn={b_is_kn}); need equal K (a multiple of 8), N % 16 == 0, M % 8 == 0 if a_is_km")
    a2, b2 = _rows_view(a, a.shape[1]), _rows_view(b, b.shape[1])
    c = torch.empty((m, n), dtype=torch.bfloat16, device=a.device)
    if m > 0:
        dev = a.device.index if a.device.index is not None else torch.cuda.current_device()
        lib = _loader.load_library()
        key = ("gemm_bf16", m, n, k, bool(b_is_kn), dev, _loader.tuning_epoch())
        need = _ws_need.get(key)
        if need is None:  # scratch lets a nearly empty last wave be balanced by K ranges
            need = _ws_need[key] = max(0, int(lib.magi_swiglu_gemm_bf16_workspace_bytes(m, n, k, 1 if b_is_kn else 0, dev)))
        ws = _workspace(a.device, need) if need else None
        rc = lib.magi_swiglu_gemm_bf16_ws(
            a2.data_ptr(), b2.data_ptr(), c.data_ptr(), m, n, k, a2.stride(0) if a2.shape[0] > 1 else a2.shape[1],
            b2.stride(0) if b2.shape[0] > 1 else b2.shape[1], n, 1 if a_is_km else 0, 1 if b_is_kn else 0, dev,
            torch.cuda.current_stream(a.device).cuda_stream, ws.data_ptr() if ws is not None else None, need)
        if rc != 0:
            msg = f"magi_swiglu_gemm_bf16_ws failed ({rc}): {_loader.last_error()}"
            raise (ValueError(msg) if rc < 0 else RuntimeError(msg))
    return c


BWD_ACT_OP_NAME = "magi_swiglu::swiglu_backward_act"


@magi_register_custom_op(name=BWD_ACT_OP_NAME, mutates_args=(),
                         infer_output_meta_fn=lambda h, dy: torch.empty_like(h))
def swiglu_backward_act(h: torch.Tensor, dy: torch.Tensor) -> torch.Tensor:
    """``dH = [dG | dU]`` from the pre-activations ``H = [G | U]`` (``[M, 2N]`` bf16) and ``dY`` (``[M, N]`` bf16):
    one element-wise CUDA kernel (``magi_swiglu_backward_act_bf16``)."""
    if h.dtype != torch.bfloat16 or dy.dtype != torch.bfloat16:
        raise TypeError("swiglu_backward_act computes in bf16 only")
    if not (h.is_cuda and dy.is_cuda) or h.device != dy.device:
        raise TypeError("swiglu_backward_act runs on CUDA tensors of one device")
    if h.dim() != 2 or dy.dim() != 2 or h.shape[0] != dy.shape[0] or h.shape[1] != 2 * dy.shape[1] or dy.shape[1] % 8:
        raise ValueError(f"shapes do not match: h {tuple(h.shape)}, dy {tuple(dy.shape)} (need [M,2N], [M,N], N % 8 == 0)")
    lib = _loader.load_library()
    h2, dy2 = _rows_view(h, h.shape[1]), _rows_view(dy, dy.shape[1])
    dh = torch.empty((h.shape[0], h.shape[1]), dtype=torch.bfloat16, device=h.device)
    if h.shape[0] == 0:
        return dh
    dev = h.device.index if h.device.index is not None else torch.cuda.current_device()
    rc = lib.magi_swiglu_backward_act_bf16(h2.data_ptr(), dy2.data_ptr(), dh.data_ptr(), h.shape[0], dy.shape[1],
                                           h2.stride(0) if h.shape[0] > 1 else h.shape[1],
                                           dy2.stride(0) if h.shape[0] > 1 else dy.shape[1], dh.stride(0), dev,
                                           torch.cuda.current_stream(h.device).cuda_stream)
    if rc != 0:
        msg = f"magi_swiglu_backward_act_bf16 failed ({rc}): {_loader.last_error()}"
        raise (ValueError(msg) if rc < 0 else RuntimeError(msg))
    return dh


BWD_DH_OP_NAME = "magi_swiglu::swiglu_backward_dh"


@magi_register_custom_op(name=BWD_DH_OP_NAME, mutates_args=(),
                         infer_output_meta_fn=lambda x, w_gate_up, dy: dy.new_empty((dy.shape[0], 2 * dy.shape[1])),
                         is_compute_sensitive=True)
def swiglu_backward_dh(x: torch.Tensor, w_gate_up: torch.Tensor, dy: torch.Tensor) -> torch.Tensor:
    """``dH = [dG | dU]`` (``[M, 2N]`` bf16) from ``x [M, K]``, the packed weight and ``dY [M, N]`` in ONE kernel
    (``magi_swiglu_backward_dh_bf16``): the tile kernels recompute the pre-activations into tensor memory and the
    epilogue applies the activation's derivative to the fp32 accumulators, so ``H`` never reaches HBM."""
    M, N, K = _check(x, w_gate_up)
    if x.dim() != 2 or dy.dim() != 2 or dy.dtype != torch.bfloat16 or dy.device != x.device \
            or tuple(dy.shape) != (M, N):
        raise ValueError(f"shapes do not match: x {tuple(x.shape)}, w_gate_up {tuple(w_gate_up.shape)}, "
                         f"dy {tuple(dy.shape)} {dy.dtype} (need [M,K], [2N,K], bf16 [M,N])")
    x2, w2, dy2 = _rows_view(x, K), _rows_view(w_gate_up, K), _rows_view(dy, N)
    dh = torch.empty((M, 2 * N), dtype=torch.bfloat16, device=x.device)
    if M > 0:
        dev = x.device.index if x.device.index is not None else torch.cuda.current_device()
        rc = _loader.load_library().magi_swiglu_backward_dh_bf16(
            x2.data_ptr(), w2.data_ptr(), dy2.data_ptr(), dh.data_ptr(), M, N, K, x2.stride(0) if M > 1 else K,
            w2.stride(0), dy2.stride(0) if M > 1 else N, 2 * N, dev, torch.cuda.current_stream(x.device).cuda_stream)
        if rc != 0:
            msg = f"magi_swiglu_backward_dh_bf16 failed ({rc}): {_loader.last_error()}"
            raise (ValueError(msg) if rc < 0 else RuntimeError(msg))
    return dh


NVFP4_OP_NAME = "magi_swiglu::gemm_swiglu_nvfp4"


def nvfp4_scale_shape(rows: int, n: int, swizzled: bool) -> tuple[int, ...]:
    """Shape of the scale-factor tensor for ``rows`` x ``n`` outputs: ``[rows, n/16]`` linear, or the padded flat
    buffer of the 128 x 4 tiled layout."""
    blocks = n // 16
    if not swizzled:
        return (rows, blocks)
    return (-(-rows // 128) * 128 * -(-blocks // 4) * 4,)


def _gemm_swiglu_nvfp4_meta(x, w_gate_up, global_scale, swizzled_scales):
    n = w_gate_up.shape[0] // 2
    rows = x.numel() // x.shape[-1] if x.dim() != 2 else x.shape[0]
    blocks = n // 16
    if swizzled_scales:
        sf_shape = (((rows + 127) // 128) * 128 * ((blocks + 3) // 4) * 4,)
    else:
        sf_shape = (rows, blocks)
    return (x.new_empty((*x.shape[:-1], n // 2), dtype=torch.uint8),
            x.new_empty(sf_shape, dtype=torch.float8_e4m3fn))


@magi_register_custom_op(name=NVFP4_OP_NAME, mutates_args=(), infer_output_meta_fn=_gemm_swiglu_nvfp4_meta,
                         is_compute_sensitive=True)
def gemm_swiglu_nvfp4(x: torch.Tensor, w_gate_up: torch.Tensor, global_scale: torch.Tensor,
                      swizzled_scales: bool) -> tuple[torch.Tensor, torch.Tensor]:
    """The fused op with an nvfp4 output (``magi_swiglu_forward_nvfp4``): returns ``(codes, scales)`` —
    ``codes`` uint8 ``[..., N/2]`` (two e2m1 values per byte, even column in the low nibble) and one e4m3 scale per
    16 outputs, ``[M, N/16]`` or, with ``swizzled_scales``, the zero-padded 128 x 4 tiled buffer block-scaled GEMMs
    read.  ``global_scale`` is a one-element fp32 CUDA tensor read by the kernel.  Dequantised value =
    ``e2m1 * scale / global_scale``.  This is the merged gate/up linear followed by vLLM's
    ``silu_and_mul_nvfp4_quant`` (magi_compiler/passes/piecewise_graph/fix_functionalization.py:113-120), rounded
    once from the fp32 accumulators.  N must be a multiple of 16.  Inference only."""
    M, N, K = _check(x, w_gate_up)
    if N % 16 != 0:
        raise ValueError(f"N ({N}) must be a multiple of 16 for the nvfp4 output")
    if not isinstance(global_scale, torch.Tensor) or global_scale.dtype != torch.float32 or global_scale.numel() != 1:
        raise TypeError("global_scale must be a one-element fp32 tensor")
    if global_scale.device != x.device:
        raise ValueError(f"global_scale is on {global_scale.device} but x is on {x.device}")
    x2, w2 = _rows_view(x, K), _rows_view(w_gate_up, K)
    codes = torch.empty((M, N // 2), dtype=torch.uint8, device=x.device)
    shape = nvfp4_scale_shape(M, N, bool(swizzled_scales))
    # the tiled layout has padding entries the kernel does not write: hand out zeros there
    scales = (torch.zeros if swizzled_scales else torch.empty)(shape, dtype=torch.uint8, device=x.device)
    if M > 0:
        dev = x.device.index if x.device.index is not None else torch.cuda.current_device()
        rc = _loader.load_library().magi_swiglu_forward_nvfp4(
            x2.data_ptr(), w2.data_ptr(), codes.data_ptr(), scales.data_ptr(), global_scale.data_ptr(), M, N, K,
            x2.stride(0) if M > 1 else K, w2.stride(0), N // 2, N // 16, 1 if swizzled_scales else 0, dev,
            torch.cuda.current_stream(x.device).cuda_stream)
        if rc != 0:
            msg = f"magi_swiglu_forward_nvfp4 failed ({rc}): {_loader.last_error()}"
            raise (ValueError(msg) if rc < 0 else RuntimeError(msg))
    return codes.view(*x.shape[:-1], N // 2), scales.view(torch.float8_e4m3fn)


PREACT_OP_NAME = "magi_swiglu::gemm_swiglu_preact"


def _gemm_swiglu_preact_meta(x: torch.Tensor, w_gate_up: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    n = w_gate_up.shape[0] // 2
    rows = x.numel() // x.shape[-1] if x.dim() != 2 else x.shape[0]
    return x.new_empty((*x.shape[:-1], n)), x.new_empty((rows, 2 * n))


def _gemm_swiglu_preact_setup_context(ctx, inputs, output):
    x, w_gate_up = inputs
    ctx.set_materialize_grads(False)  # the gradient of the auxiliary output H is normally absent: keep it None
    ctx.save_for_backward(x, w_gate_up, output[1])


def _gemm_swiglu_preact_backward(ctx, grad_y, grad_h):
    """dH from the SAVED pre-activations (one element-wise kernel), then dX = dH · W and dW = dH^T · X (library)."""
    x, w, h = ctx.saved_tensors
    if grad_y is None and grad_h is None:
        return None, None
    k = x.shape[-1]
    x2 = x.reshape(-1, k)
    dh = None
    if grad_y is not None:
        dh = torch.ops.magi_swiglu.swiglu_backward_act(h, grad_y.reshape(-1, grad_y.shape[-1]).contiguous())
    if grad_h is not None:
        dh = grad_h if dh is None else dh + grad_h
    dx, dw = _gradient_gemms(dh, w, x2, ctx.needs_input_grad[0], ctx.needs_input_grad[1])
    return (dx.view(x.shape) if dx is not None else None), dw


@magi_register_custom_op(
    name=PREACT_OP_NAME,
    mutates_args=(),
    infer_output_meta_fn=_gemm_swiglu_preact_meta,
    setup_context_fn=_gemm_swiglu_preact_setup_context,
    backward_fn=_gemm_swiglu_preact_backward,
    is_compute_sensitive=True,
    is_subgraph_boundary=True,
)
def gemm_swiglu_preact(x: torch.Tensor, w_gate_up: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """``(y, h)``: the fused op and, from the same kernel, the pre-activations ``h = [x·Wg^T | x·Wu^T]``
    (``[M, 2N]`` bf16; ``magi_swiglu_forward_bf16_preact``).  Its autograd keeps ``h`` (what PyTorch keeps for the
    reference's eager expression, tests/model_definition.py:337-339) and so runs no GEMM again in the backward; the
    single-output op keeps nothing but its inputs and recomputes.  Use ``gemm_swiglu_train`` for the ``y``-only form."""
    M, N, K = _check(x, w_gate_up)
    x2, w2 = _rows_view(x, K), _rows_view(w_gate_up, K)
    if w2.data_ptr() != w_gate_up.data_ptr() and w_gate_up.numel() > 0:
        raise ValueError("w_gate_up must have unit inner stride, a row stride that is a multiple of 8 and a "
                         "16-byte-aligned base; pack it once with magicompiler_b200.pack_gate_up")
    y = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    h = torch.empty((M, 2 * N), dtype=torch.bfloat16, device=x.device)
    if M > 0:
        dev = x.device.index if x.device.index is not None else torch.cuda.current_device()
        rc = _loader.load_library().magi_swiglu_forward_bf16_preact(
            x2.data_ptr(), w2.data_ptr(), y.data_ptr(), h.data_ptr(), M, N, K, x2.stride(0) if M > 1 else K,
            w2.stride(0), N, 2 * N, dev, torch.cuda.current_stream(x.device).cuda_stream)
        if rc != 0:
            msg = f"magi_swiglu_forward_bf16_preact failed ({rc}): {_loader.last_error()}"
            raise (ValueError(msg) if rc < 0 else RuntimeError(msg))
    return y.view(*x.shape[:-1], N), h


def gemm_swiglu_auto(x: torch.Tensor, w_gate_up: torch.Tensor) -> torch.Tensor:
    """``gemm_swiglu_train`` when a gradient will be asked for (grad mode on and an argument requires grad), else the
    plain ``gemm_swiglu``: training keeps the pre-activations (faster than recomputing them and still one tensor fewer
    than PyTorch keeps for the eager expression), inference writes nothing extra."""
    if torch.is_grad_enabled() and (x.requires_grad or w_gate_up.requires_grad):
        return torch.ops.magi_swiglu.gemm_swiglu_preact(x, w_gate_up)[0]
    return torch.ops.magi_swiglu.gemm_swiglu(x, w_gate_up)


def gemm_swiglu_train(x: torch.Tensor, w_gate_up: torch.Tensor) -> torch.Tensor:
    """``gemm_swiglu`` for training steps where memory allows keeping the ``[M, 2N]`` pre-activations: forward +
    backward run four GEMMs' worth of tensor work instead of five (no recomputation)."""
    return torch.ops.magi_swiglu.gemm_swiglu_preact(x, w_gate_up)[0]


FP8_OP_NAME = "magi_swiglu::gemm_swiglu_fp8"


def _gemm_swiglu_fp8_meta(x: torch.Tensor, w_gate_up: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    return x.new_empty((*x.shape[:-1], w_gate_up.shape[0] // 2), dtype=torch.float8_e4m3fn)


@magi_register_custom_op(name=FP8_OP_NAME, mutates_args=(), infer_output_meta_fn=_gemm_swiglu_fp8_meta,
                         is_compute_sensitive=True)
def gemm_swiglu_fp8(x: torch.Tensor, w_gate_up: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """The fused op with a statically scaled fp8 output: ``(silu(g) * u / scale).to(float8_e4m3fn)``, saturating,
    rounded once from the fp32 accumulators (``magi_swiglu_forward_fp8_e4m3``).  ``scale`` is a one-element fp32
    CUDA tensor; the kernel reads it, the host does not.  This is the merged gate/up linear followed by vLLM's
    ``silu_and_mul_quant(result, input, scale)``, the quantising activation the reference's de-functionalisation
    pass handles (magi_compiler/passes/piecewise_graph/fix_functionalization.py:110-112).  N must be a multiple of
    16.  Inference only: no autograd is registered."""
    M, N, K = _check(x, w_gate_up)
    if N % 16 != 0:
        raise ValueError(f"N ({N}) must be a multiple of 16 for the fp8 output")
    if not isinstance(scale, torch.Tensor) or scale.dtype != torch.float32 or scale.numel() != 1:
        raise TypeError("scale must be a one-element fp32 tensor")
    if scale.device != x.device:
        raise ValueError(f"scale is on {scale.device} but x is on {x.device}")
    x2, w2 = _rows_view(x, K), _rows_view(w_gate_up, K)
    y = torch.empty((M, N), dtype=torch.float8_e4m3fn, device=x.device)
    if M > 0:
        dev = x.device.index if x.device.index is not None else torch.cuda.current_device()
        rc = _loader.load_library().magi_swiglu_forward_fp8_e4m3(
            x2.data_ptr(), w2.data_ptr(), y.data_ptr(), scale.data_ptr(), M, N, K, x2.stride(0) if M > 1 else K,
            w2.stride(0), N, dev, torch.cuda.current_stream(x.device).cuda_stream)
        if rc != 0:
            msg = f"magi_swiglu_forward_fp8_e4m3 failed ({rc}): {_loader.last_error()}"
            raise (ValueError(msg) if rc < 0 else RuntimeError(msg))
    return y.view(*x.shape[:-1], N)


_GRADIENT_GEMMS = os.environ.get("MAGI_SWIGLU_GRADIENT_GEMMS", "library")


def set_gradient_gemms(which: str) -> str:
    """Which kernels compute ``dX = dH · W`` and ``dW = dH^T · X`` in the backward: ``"library"`` (torch.matmul; the
    default, 3-6 % faster on the Llama-3-8B FFN shape) or ``"own"`` (``gemm_bf16`` on the op's tile kernels, operands
    read in place as MN-major tiles).  Returns the previous setting.  Initial value: $MAGI_SWIGLU_GRADIENT_GEMMS."""
    global _GRADIENT_GEMMS
    if which not in ("library", "own"):
        raise ValueError("which must be 'library' or 'own'")
    prev, _GRADIENT_GEMMS = _GRADIENT_GEMMS, which
    return prev


def _gradient_gemms(dh: torch.Tensor, w: torch.Tensor, x2: torch.Tensor, need_dx: bool, need_dw: bool):
    own = _GRADIENT_GEMMS == "own" and x2.shape[1] % 16 == 0 and x2.shape[0] % 8 == 0
    if own:
        dx = torch.ops.magi_swiglu.gemm_bf16(dh, w, False, True) if need_dx else None
        dw = torch.ops.magi_swiglu.gemm_bf16(dh, x2, True, True) if need_dw else None
    else:
        dx = torch.matmul(dh, w) if need_dx else None
        dw = torch.matmul(dh.t(), x2) if need_dw else None
    return dx, dw


def _gemm_swiglu_setup_context(ctx, inputs, output):
    x, w_gate_up = inputs
    ctx.save_for_backward(x, w_gate_up)  # the 2N-wide pre-activations are never stored: backward recomputes them


def _gemm_swiglu_backward(ctx, grad_out):
    """dX = dH · W and dW = dH^T · X with dH = [dG | dU] from one kernel that recomputes H = X · W^T in tensor memory
    and applies the activation's derivative in its epilogue (swiglu_backward_dh); the two gradient GEMMs need
    transposed operands and go to the library."""
    x, w = ctx.saved_tensors
    k = x.shape[-1]
    x2 = x.reshape(-1, k)
    dy2 = grad_out.reshape(-1, grad_out.shape[-1]).contiguous()
    dh = torch.ops.magi_swiglu.swiglu_backward_dh(x2, w, dy2)
    dx, dw = _gradient_gemms(dh, w, x2, ctx.needs_input_grad[0], ctx.needs_input_grad[1])
    return (dx.view(x.shape) if dx is not None else None), dw


def _gemm_swiglu_meta(x: torch.Tensor, w_gate_up: torch.Tensor) -> torch.Tensor:
    # shape/dtype/device only; works with a symbolic leading dimension
    return x.new_empty((*x.shape[:-1], w_gate_up.shape[0] // 2))


@magi_register_custom_op(
    name=OP_NAME,
    mutates_args=(),
    infer_output_meta_fn=_gemm_swiglu_meta,
    setup_context_fn=_gemm_swiglu_setup_context,
    backward_fn=_gemm_swiglu_backward,
    is_compute_sensitive=True,
    is_subgraph_boundary=True,
)
def gemm_swiglu(x: torch.Tensor, w_gate_up: torch.Tensor) -> torch.Tensor:
    return gemm_swiglu_out(x, w_gate_up)
