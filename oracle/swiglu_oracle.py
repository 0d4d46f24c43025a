"""TEST INFRASTRUCTURE — Python face of the CPU oracle (see ``oracle/__init__.py``).

The arithmetic follows MagiCompiler's eager SwiGLU, ``F.silu(gate_proj(x)) * up_proj(x)``
(tests/model_definition.py:337-339; same expression in example/training/llama3.py:173), evaluated on
one packed weight ``W[2N,K] = [gate_proj.weight ; up_proj.weight]``.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from pathlib import Path

import numpy as np
import torch
import torch.nn.functional as F

_HERE = Path(__file__).resolve().parent
_SRC = _HERE / "swiglu_oracle.c"
_SO = _HERE / "_build" / "libswiglu_oracle.so"
_lib = None

# Tolerance of the path, stated against the fp32-accumulated gold (bf16 output, K up to 8192):
#   max|y - gold| / max|gold| <= 1e-2   and   ||y - gold||_F / ||gold||_F <= 5e-3.
# Element-wise relative error is not usable: the reference's own eager result reaches 0.2 on tiny outputs.
TOL_MAX_NORM = 1e-2
TOL_FROB = 5e-3


def build(force: bool = False) -> Path:
    """Compile the C oracle with gcc (baseline x86-64 code, no fused multiply-add contraction)."""
    if force or not _SO.exists() or _SO.stat().st_mtime < _SRC.stat().st_mtime:
        _SO.parent.mkdir(parents=True, exist_ok=True)
        cmd = ["gcc", "-O2", "-ffp-contract=off", "-fPIC", "-shared", "-o", str(_SO), str(_SRC), "-lm", "-lpthread"]
        subprocess.run(cmd, check=True)
    return _SO


def _load():
    global _lib
    if _lib is None:
        build()
        lib = ctypes.CDLL(str(_SO))
        lib.oracle_swiglu.restype = ctypes.c_int
        lib.oracle_swiglu.argtypes = [ctypes.c_void_p, ctypes.c_void_p] + [ctypes.c_int64] * 5 + [
            ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int]
        lib.oracle_f32_to_bf16.restype = ctypes.c_uint16
        lib.oracle_f32_to_bf16.argtypes = [ctypes.c_float]
        lib.oracle_bf16_to_f32.restype = ctypes.c_float
        lib.oracle_bf16_to_f32.argtypes = [ctypes.c_uint16]
        _lib = lib
    return _lib


def to_bits(t: torch.Tensor) -> np.ndarray:
    """bf16 tensor -> uint16 numpy array of its bit patterns (CPU copy)."""
    assert t.dtype == torch.bfloat16
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def from_bits(a: np.ndarray) -> torch.Tensor:
    """uint16 bit patterns -> bf16 tensor."""
    return torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).view(torch.bfloat16)


def make_inputs(M: int, K: int, N: int, seed: int = 0, with_down: bool = False):
    """The benchmark's synthetic inputs: CPU generator, X ~ N(0,1), W ~ N(0,0.02), both cast to bf16.

    Returns (x[M,K], w[2N,K]) or (x, w, w_down[K,N]); gate rows first in w.
    """
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(2 * N, K, generator=g) * 0.02).to(torch.bfloat16)
    if with_down:
        wd = (torch.randn(K, N, generator=g) * 0.02).to(torch.bfloat16)
        return x, w, wd
    return x, w


def swiglu_gold(x: torch.Tensor, w: torch.Tensor, threads: int | None = None, want_eager: bool = True):
    """C oracle.  x [M,K] bf16, w [2N,K] bf16 (CPU).  Returns dict with
    ``gold`` (fp32 [M,N]), ``gold_bf16`` (bf16, gold rounded once), ``eager`` (bf16, reference rounding chain)."""
    lib = _load()
    assert x.dim() == 2 and w.dim() == 2 and w.shape[0] % 2 == 0 and x.shape[1] == w.shape[1]
    M, K = x.shape
    N = w.shape[0] // 2
    xb, wb = to_bits(x), to_bits(w)
    gold = np.empty((M, N), dtype=np.float32)
    gold_bf16 = np.empty((M, N), dtype=np.uint16)
    eager = np.empty((M, N), dtype=np.uint16) if want_eager else None
    if threads is None:
        threads = min(os.cpu_count() or 1, 16)
    rc = lib.oracle_swiglu(xb.ctypes.data, wb.ctypes.data, M, N, K, K, K, gold.ctypes.data, gold_bf16.ctypes.data,
                           eager.ctypes.data if want_eager else None, threads)
    assert rc == 0
    out = {"gold": torch.from_numpy(gold), "gold_bf16": from_bits(gold_bf16)}
    if want_eager:
        out["eager"] = from_bits(eager)
    return out


def swiglu_gold_numpy(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """fp32 gold in numpy (bf16 values are exact in fp32; products are summed in fp32 by BLAS)."""
    N = w.shape[0] // 2
    xf = x.float().numpy()
    wf = w.float().numpy()
    h = xf @ wf.T
    g, u = h[:, :N], h[:, N:]
    return torch.from_numpy((g / (1.0 + np.exp(-g))) * u)


def swiglu_ref_eager(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """The reference's eager expression, literally, with gate_proj.weight = w[:N], up_proj.weight = w[N:]."""
    N = w.shape[0] // 2
    return F.silu(F.linear(x, w[:N])) * F.linear(x, w[N:])


def error_metrics(y: torch.Tensor, gold: torch.Tensor) -> dict:
    """Normalised error of y (any dtype) against the fp32 gold."""
    yf = y.detach().float().cpu()
    gf = gold.detach().float().cpu()
    diff = (yf - gf)
    gmax = gf.abs().max().item()
    return {
        "max_norm": (diff.abs().max().item() / gmax) if gmax > 0 else diff.abs().max().item(),
        "frob": (diff.norm().item() / gf.norm().item()) if gmax > 0 else diff.norm().item(),
        "gold_absmax": gmax,
    }


def swiglu_backward_gold(x: torch.Tensor, w: torch.Tensor, dy: torch.Tensor):
    """fp32 gold of the backward of ``silu(x·Wg^T) * (x·Wu^T)`` (the autograd PyTorch derives for the reference's
    expression, tests/model_definition.py:337-339), written out: returns (dx [M,K], dw [2N,K]) in fp32."""
    n = w.shape[0] // 2
    xf, wf, dyf = x.float(), w.float(), dy.float()
    h = xf @ wf.t()
    g, u = h[:, :n], h[:, n:]
    s = torch.sigmoid(g)
    dg = dyf * u * s * (1.0 + g * (1.0 - s))
    du = dyf * g * s
    dh = torch.cat([dg, du], dim=1)
    return dh @ wf, dh.t() @ xf


def rmsnorm_swiglu_gold(x: torch.Tensor, norm_weight: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """fp32 gold of RMSNorm followed by the SwiGLU projection, nothing rounded in between:
    MagiCompiler's RMSNorm.forward (tests/model_definition.py:51-56) feeding TransformerMLP's gate/up part (:337-339)."""
    n = w.shape[0] // 2
    xf = x.float()
    xn = xf * torch.rsqrt(xf.pow(2).mean(dim=-1, keepdim=True) + eps) * norm_weight.float()
    h = xn @ w.float().t()
    return F.silu(h[:, :n]) * h[:, n:]


def rmsnorm_swiglu_ref_eager(x: torch.Tensor, norm_weight: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """The reference's eager chain, literally: RMSNorm.forward (fp32 inside, bf16 out), then the eager SwiGLU."""
    variance = x.to(torch.float32).pow(2).mean(dim=-1, keepdim=True)
    xn = x * torch.rsqrt(variance + eps)
    xn = (xn.to(norm_weight.dtype) * norm_weight).to(x.dtype)
    return swiglu_ref_eager(xn, w)


_E2M1_VALUES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)


def e2m1_round(q: torch.Tensor) -> torch.Tensor:
    """fp32 -> e2m1 codes (0..15, bit 3 = sign), round to nearest with ties to the even code, saturating at 6."""
    a = q.abs()
    code = torch.zeros_like(a, dtype=torch.uint8)
    # (lower bound, inclusive?) of each magnitude code; a tie goes to the even code
    for c, (lo, incl) in enumerate([(0.25, False), (0.75, True), (1.25, False), (1.75, True), (2.5, False),
                                    (3.5, True), (5.0, False)], start=1):
        code = torch.where((a >= lo) if incl else (a > lo), torch.full_like(code, c), code)
    return code | ((q < 0) | ((q == 0) & (torch.signbit(q)))).to(torch.uint8) * 8


def nvfp4_quantize_gold(y: torch.Tensor, global_scale: float):
    """NVFP4 quantisation of an fp32 ``[M, N]`` tensor the way vLLM's ``silu_and_mul_nvfp4_quant`` /
    ``scaled_fp4_quant`` kernels do it (vLLM is not a dependency of MagiCompiler and not part of its checkout; the
    reference only names the op, magi_compiler/passes/piecewise_graph/fix_functionalization.py:113-120; this follows
    the published algorithm — parity unpinned: no build of that kernel is available to run beside it):
    per block of 16 columns  sf = e4m3(gs * max|y| / 6),  code = e2m1(y * (1 / (sf / gs))), zeros when sf == 0.
    Returns (codes uint8 [M, N] one code per element, sf float8_e4m3fn [M, N/16], dequantised fp32 [M, N])."""
    M, N = y.shape
    gs = torch.tensor(global_scale, dtype=torch.float32)
    yb = y.float().reshape(M, N // 16, 16)
    vmax = yb.abs().amax(dim=-1)
    sf = gs * (vmax * torch.tensor(1.0 / 6.0, dtype=torch.float32))
    sf8 = sf.clamp(max=448.0).to(torch.float8_e4m3fn)
    sff = sf8.float()
    inv_gs = torch.tensor(1.0, dtype=torch.float32) / gs
    out_scale = torch.where(sff != 0, 1.0 / (sff * inv_gs), torch.zeros_like(sff))
    codes = e2m1_round(yb * out_scale[..., None]).reshape(M, N)
    mag = torch.tensor(_E2M1_VALUES)[(codes & 7).long()] * torch.where((codes & 8) != 0, -1.0, 1.0)
    deq = (mag.reshape(M, N // 16, 16) * (sff * inv_gs)[..., None]).reshape(M, N)
    return codes, sf8, deq


def nvfp4_swizzled_offsets(M: int, N: int) -> torch.Tensor:
    """Byte offset of scale (m, b) in the 128 x 4 tiled layout of block-scale factors: tiles of 128 rows x 4 blocks
    (512 bytes), tile row r at (r % 32) * 16 + (r / 32) * 4.  Returns int64 [M, N/16]."""
    m = torch.arange(M).view(M, 1)
    b = torch.arange(N // 16).view(1, N // 16)
    ktiles = -(-(N // 16) // 4)
    r = m % 128
    return ((m // 128) * ktiles + b // 4) * 512 + (r % 32) * 16 + (r // 32) * 4 + b % 4
