"""Builds and loads ``libmagi_swiglu.so`` (the C-ABI CUDA library, ``include/magi_swiglu.h``) with ctypes.

The calling style mirrors MagiCompiler's only native binding, ``magi_compiler/cuda/cudart.py:24-62``
(a ``ctypes.CDLL`` plus explicit ``argtypes``).  There is no fallback: if the library cannot be
loaded, every compute entry raises.
"""
from __future__ import annotations

import ctypes
import os
import shutil
import subprocess
from pathlib import Path

_PKG = Path(__file__).resolve().parent
CSRC = _PKG / "csrc"
INCLUDE = _PKG.parent / "include"
LIB_PATH = _PKG / "_lib" / "libmagi_swiglu.so"
SOURCES = [CSRC / "swiglu_sm100.cu"]
HEADERS = [CSRC / "ptx_sm100.cuh", CSRC / "swiglu_kernels.cuh", CSRC / "swiglu_plan.hpp", INCLUDE / "magi_swiglu.h"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC",
]

ABI_VERSION = 8
VARIANT_AUTO, VARIANT_MMA, VARIANT_STREAM, VARIANT_SIMT, VARIANT_MMA2 = 0, 1, 2, 3, 4
VARIANTS = {"auto": VARIANT_AUTO, "mma": VARIANT_MMA, "stream": VARIANT_STREAM, "simt": VARIANT_SIMT,
            "mma2": VARIANT_MMA2}

_lib = None


class MagiSwigluLibraryError(RuntimeError):
    """The CUDA library is missing, stale or refused to load."""


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(exe).exists():
        raise MagiSwigluLibraryError("nvcc not found; cannot build libmagi_swiglu.so")
    return exe


def library_is_stale() -> bool:
    if not LIB_PATH.exists():
        return True
    built = LIB_PATH.stat().st_mtime
    return any(p.stat().st_mtime > built for p in SOURCES + HEADERS)


def build_library(force: bool = False, verbose: bool = False) -> Path:
    """Compile the kernels for sm_100a into ``magicompiler_b200/_lib/`` (in-tree, next to the package)."""
    if not force and not library_is_stale():
        return LIB_PATH
    LIB_PATH.parent.mkdir(parents=True, exist_ok=True)
    cmd = [_nvcc(), *NVCC_FLAGS, *(["-Xptxas", "-v"] if verbose else []), "-o", str(LIB_PATH), *map(str, SOURCES)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise MagiSwigluLibraryError(f"nvcc failed ({proc.returncode}):\n{proc.stdout}\n{proc.stderr}")
    if verbose:
        print(proc.stderr)
    return LIB_PATH


def _declare(lib: ctypes.CDLL) -> None:
    i64, i32, vp = ctypes.c_int64, ctypes.c_int, ctypes.c_void_p
    lib.magi_swiglu_version.restype = i32
    lib.magi_swiglu_version.argtypes = []
    lib.magi_swiglu_supported.restype = i32
    lib.magi_swiglu_supported.argtypes = [i32]
    lib.magi_swiglu_forward_bf16.restype = i32
    lib.magi_swiglu_forward_bf16.argtypes = [vp, vp, vp, i64, i64, i64, i64, i64, i64, i32, vp, i32]
    lib.magi_swiglu_forward_bf16_ex.restype = i32
    lib.magi_swiglu_forward_bf16_ex.argtypes = [vp, vp, vp, i64, i64, i64, i64, i64, i64, i32, vp, i32,
                                                i32, i32, i32, i32]
    lib.magi_swiglu_forward_bf16_ws.restype = i32
    lib.magi_swiglu_forward_bf16_ws.argtypes = [vp, vp, vp, i64, i64, i64, i64, i64, i64, i32, vp, i32,
                                                i32, i32, i32, i32, vp, i64]
    lib.magi_swiglu_forward_bf16_static.restype = i32
    lib.magi_swiglu_forward_bf16_static.argtypes = [vp, vp, vp, i64, i64, i64, i64, i64, i64, i32, vp]
    lib.magi_swiglu_row_rms_f32.restype = i32
    lib.magi_swiglu_row_rms_f32.argtypes = [vp, vp, i64, i64, i64, ctypes.c_float, i32, vp]
    lib.magi_swiglu_forward_bf16_scaled.restype = i32
    lib.magi_swiglu_forward_bf16_scaled.argtypes = [vp, vp, vp, vp, i64, i64, i64, i64, i64, i64, i32, vp, vp, i64]
    lib.magi_swiglu_forward_fp8_e4m3.restype = i32
    lib.magi_swiglu_forward_fp8_e4m3.argtypes = [vp, vp, vp, vp, i64, i64, i64, i64, i64, i64, i32, vp]
    lib.magi_swiglu_forward_nvfp4.restype = i32
    lib.magi_swiglu_forward_nvfp4.argtypes = [vp, vp, vp, vp, vp, i64, i64, i64, i64, i64, i64, i64, i32, i32, vp]
    lib.magi_swiglu_forward_bf16_preact.restype = i32
    lib.magi_swiglu_forward_bf16_preact.argtypes = [vp, vp, vp, vp, i64, i64, i64, i64, i64, i64, i64, i32, vp]
    lib.magi_swiglu_backward_dh_bf16.restype = i32
    lib.magi_swiglu_backward_dh_bf16.argtypes = [vp, vp, vp, vp, i64, i64, i64, i64, i64, i64, i64, i32, vp]
    lib.magi_swiglu_gemm_bf16.restype = i32
    lib.magi_swiglu_gemm_bf16.argtypes = [vp, vp, vp, i64, i64, i64, i64, i64, i64, i32, i32, i32, vp]
    lib.magi_swiglu_gemm_bf16_ws.restype = i32
    lib.magi_swiglu_gemm_bf16_ws.argtypes = [vp, vp, vp, i64, i64, i64, i64, i64, i64, i32, i32, i32, vp, vp, i64]
    lib.magi_swiglu_gemm_bf16_workspace_bytes.restype = i64
    lib.magi_swiglu_gemm_bf16_workspace_bytes.argtypes = [i64, i64, i64, i32, i32]
    lib.magi_swiglu_gemm_nt_bf16.restype = i32
    lib.magi_swiglu_gemm_nt_bf16.argtypes = [vp, vp, vp, i64, i64, i64, i64, i64, i64, i32, vp]
    lib.magi_swiglu_scatter_setup.restype = i32
    lib.magi_swiglu_scatter_setup.argtypes = [i32, i32, ctypes.POINTER(vp), i32, i64, i64, i64]
    lib.magi_swiglu_gemm_nt_bf16_scatter.restype = i32
    lib.magi_swiglu_gemm_nt_bf16_scatter.argtypes = [vp, vp, i32, i64, i64, i64, i64, i64, i32, vp, vp, i64]
    lib.magi_swiglu_sum_slots_bf16.restype = i32
    lib.magi_swiglu_sum_slots_bf16.argtypes = [vp, vp, i32, i64, i64, i32, vp]
    lib.magi_swiglu_sum_slots_bf16_bcast.restype = i32
    lib.magi_swiglu_sum_slots_bf16_bcast.argtypes = [vp, ctypes.POINTER(vp), i32, i32, i64, i64, i32, vp]
    lib.magi_swiglu_backward_act_bf16.restype = i32
    lib.magi_swiglu_backward_act_bf16.argtypes = [vp, vp, vp, i64, i64, i64, i64, i64, i32, vp]
    lib.magi_swiglu_workspace_bytes.restype = i64
    lib.magi_swiglu_workspace_bytes.argtypes = [i64, i64, i64, i32, i32, i32, i32, i32, i32, i32]
    lib.magi_swiglu_plan.restype = i32
    lib.magi_swiglu_plan.argtypes = [i64, i64, i64, i32, i32, i32, i32, i32, i32, i32, ctypes.POINTER(ctypes.c_int32)]
    lib.magi_swiglu_device_status.restype = i32
    lib.magi_swiglu_device_status.argtypes = [i32, ctypes.POINTER(ctypes.c_int32)]
    lib.magi_swiglu_schedule.restype = i32
    lib.magi_swiglu_schedule.argtypes = [i64, i64, i64, i32, i32, i32, i32, i32, i32, i64, i32,
                                         ctypes.POINTER(ctypes.c_int32), i32]
    lib.magi_swiglu_tuning.restype = i32
    lib.magi_swiglu_tuning.argtypes = [i32, i32]
    lib.magi_swiglu_watchdog_selftest.restype = i32
    lib.magi_swiglu_watchdog_selftest.argtypes = [i32, vp, i64]
    lib.magi_swiglu_kernel_clock.restype = i32
    lib.magi_swiglu_kernel_clock.argtypes = [i32, ctypes.POINTER(ctypes.c_double)]
    lib.magi_swiglu_last_error.restype = ctypes.c_char_p
    lib.magi_swiglu_last_error.argtypes = []


def load_library() -> ctypes.CDLL:
    """Load the in-tree library (building it first only if ``MAGI_SWIGLU_AUTOBUILD=1``)."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        if os.environ.get("MAGI_SWIGLU_AUTOBUILD", "0") == "1":
            build_library()
        else:
            raise MagiSwigluLibraryError(
                f"{LIB_PATH} is missing. Build it with `python -c 'import __graft_entry__ as g; g.build()'` "
                "or `python -m magicompiler_b200.build` (needs nvcc). There is no CPU or PyTorch fallback.")
    try:
        lib = ctypes.CDLL(str(LIB_PATH))
    except OSError as exc:  # pragma: no cover - depends on the machine
        raise MagiSwigluLibraryError(f"cannot load {LIB_PATH}: {exc}") from exc
    _declare(lib)
    got = lib.magi_swiglu_version()
    if got != ABI_VERSION:
        raise MagiSwigluLibraryError(f"{LIB_PATH} has ABI version {got}, this package expects {ABI_VERSION}; rebuild")
    _lib = lib
    return lib


TUNING_KNOBS = {"k_splits": 0, "no_split": 1, "y_tma": 2, "l2_hints": 3, "stream_k": 4, "scatter_wide": 5}
_tuning_epoch = 0  # bumped by set_tuning so host-side caches keyed on the schedule notice


def set_tuning(knob: str, value: int) -> int:
    """Set a tuning aid of the library (``magi_swiglu_tuning``: k_splits, no_split, y_tma, l2_hints) and return its
    previous value.  Process-wide; for tests and sweeps."""
    global _tuning_epoch
    lib = load_library()
    prev = lib.magi_swiglu_tuning(TUNING_KNOBS[knob], int(value))
    _tuning_epoch += 1
    return prev


def tuning_epoch() -> int:
    return _tuning_epoch


def last_error() -> str:
    return load_library().magi_swiglu_last_error().decode("utf-8", "replace")


def plan(M: int, N: int, K: int, variant: str | int = "auto", block_n: int = 0, stages: int = 0, group_m: int = 0,
         max_ctas: int = 0, device: int = 0, sm_count: int = 0) -> dict:
    """Schedule the library would use (pure host arithmetic when ``sm_count`` > 0)."""
    lib = load_library()
    out = (ctypes.c_int32 * 16)()
    v = VARIANTS[variant] if isinstance(variant, str) else int(variant)
    rc = lib.magi_swiglu_plan(M, N, K, v, block_n, stages, group_m, max_ctas, device, sm_count, out)
    if rc != 0:
        raise ValueError(f"magi_swiglu_plan failed ({rc}): {last_error()}")
    keys = ["variant", "block_n", "stages", "grid", "tiles", "smem_bytes", "acc_bufs", "n_mma", "ctas", "group_m", "split", "k_splits",
            "y_tma", "sk_tiles"]
    return dict(zip(keys, list(out)[:len(keys)]))


def schedule(M: int, N: int, K: int, unit: int, variant: str | int = "auto", block_n: int = 0, stages: int = 0,
             group_m: int = 0, max_ctas: int = 0, sm_count: int = 148, workspace_bytes: int = 64 << 20) -> list[dict]:
    """The work items worker ``unit`` (a CTA or CTA pair) of the planned schedule walks through, in order
    (``magi_swiglu_schedule``; pure host arithmetic): dicts with tile, K-step range, role and peers."""
    lib = load_library()
    v = VARIANTS[variant] if isinstance(variant, str) else int(variant)
    cap = 1 << 16
    buf = (ctypes.c_int32 * (6 * cap))()
    n = lib.magi_swiglu_schedule(M, N, K, v, block_n, stages, group_m, max_ctas, sm_count, workspace_bytes, unit, buf, cap)
    if n < 0:
        raise ValueError(f"magi_swiglu_schedule failed ({n}): {last_error()}")
    keys = ("tile", "kb0", "kb1", "role", "first_peer", "peers")
    return [dict(zip(keys, buf[6 * i:6 * i + 6])) for i in range(min(n, cap))]


def workspace_bytes(M: int, N: int, K: int, variant: str | int = "auto", block_n: int = 0, stages: int = 0,
                    group_m: int = 0, max_ctas: int = 0, device: int = 0, sm_count: int = 0) -> int:
    """Scratch bytes the preferred schedule wants (0 = none)."""
    lib = load_library()
    v = VARIANTS[variant] if isinstance(variant, str) else int(variant)
    n = lib.magi_swiglu_workspace_bytes(M, N, K, v, block_n, stages, group_m, max_ctas, device, sm_count)
    if n < 0:
        raise ValueError(f"magi_swiglu_workspace_bytes failed ({n}): {last_error()}")
    return int(n)


def device_status(device: int = 0) -> dict:
    """Read and clear the kernels' watchdog word (synchronises the device)."""
    lib = load_library()
    out = (ctypes.c_int32 * 4)()
    rc = lib.magi_swiglu_device_status(device, out)
    if rc != 0:
        raise RuntimeError(f"magi_swiglu_device_status failed ({rc}): {last_error()}")
    return {"code": out[0], "block": out[1], "index": out[2], "parity": out[3]}


def kernel_clock(device: int = 0) -> dict:
    """Average SM clock (MHz) the most recent tile kernel ran at, measured inside the kernel (synchronises)."""
    lib = load_library()
    out = (ctypes.c_double * 2)()
    rc = lib.magi_swiglu_kernel_clock(device, out)
    if rc != 0:
        raise RuntimeError(f"magi_swiglu_kernel_clock failed ({rc}): {last_error()}")
    return {"sm_mhz": out[0], "span_us": out[1]}
