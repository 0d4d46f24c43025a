"""B200-native fused GEMM-SwiGLU for MagiCompiler: ``Y = silu(X·Wg^T) * (X·Wu^T)`` from one packed weight.

Importing the package registers the custom op ``magi_swiglu::gemm_swiglu`` (process-wide, once).  Import it
before a model is decorated with ``magi_compile`` so the op is a graph split point for that model, and
before ahead-of-time artifacts that mention the op are deserialised.
"""
from ._loader import (MagiSwigluLibraryError, build_library, device_status, kernel_clock, load_library,  # noqa: F401
                      plan, workspace_bytes)
from .ops import (OP_NAME, fold_rmsnorm_weight, gemm_bf16, gemm_nt, gemm_nt_out, gemm_swiglu, gemm_swiglu_fp8, gemm_swiglu_out,  # noqa: F401
                  gemm_swiglu_auto, gemm_swiglu_nvfp4, gemm_swiglu_preact, gemm_swiglu_train, nvfp4_scale_shape,
                  rmsnorm_gemm_swiglu, set_gradient_gemms, swiglu_backward_act, swiglu_backward_dh)
from .passes import FuseSwiGLUPass, install_into_magi_compiler, pack_gate_up_cached  # noqa: F401
from .register import COMPUTE_SENSITIVE_OPS, SPLITTING_OPS, magi_register_custom_op  # noqa: F401
from .sharding import (  # noqa: F401
    ColumnParallelSwiGLU,
    PeerScatterReducer,
    TensorParallelSwiGLUMLP,
    pack_gate_up,
    shard_bounds,
    shard_down,
    shard_gate_up,
)

__all__ = [
    "gemm_swiglu", "gemm_swiglu_auto", "gemm_swiglu_fp8", "gemm_swiglu_nvfp4", "nvfp4_scale_shape", "gemm_swiglu_preact", "gemm_swiglu_train", "gemm_swiglu_out", "gemm_bf16", "gemm_nt", "gemm_nt_out", "swiglu_backward_act", "swiglu_backward_dh", "set_gradient_gemms", "rmsnorm_gemm_swiglu", "fold_rmsnorm_weight", "OP_NAME", "pack_gate_up", "shard_gate_up", "shard_down", "shard_bounds",
    "ColumnParallelSwiGLU", "TensorParallelSwiGLUMLP", "PeerScatterReducer", "FuseSwiGLUPass", "install_into_magi_compiler",
    "pack_gate_up_cached", "magi_register_custom_op", "SPLITTING_OPS",
    "COMPUTE_SENSITIVE_OPS", "build_library", "load_library", "plan", "workspace_bytes", "device_status", "kernel_clock", "MagiSwigluLibraryError",
]
