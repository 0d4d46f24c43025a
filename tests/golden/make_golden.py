"""Generate the golden fixtures of the SwiGLU path by running MagiCompiler's own code on CPU.

Usage (only where a MagiCompiler checkout is present; the fixtures themselves are committed):

    python tests/golden/make_golden.py --reference /path/to/MagiCompiler

What runs: ``TransformerMLP`` from the reference's ``tests/model_definition.py`` (lines 327-339) is
instantiated with bf16 parameters, its ``gate_proj.weight`` / ``up_proj.weight`` are set to the two
halves of one packed weight, and the gate/up part of its ``forward`` —
``F.silu(self.gate_proj(x)) * self.up_proj(x)`` — is evaluated through the module's own Linear layers.
The outputs (bf16 bit patterns) are stored together with the inputs (small cases) or a checksum of the
seeded inputs (the 256 x 1024 x 2816 case).

The reference imports ``graphviz`` at package import although it only calls it behind a debug flag;
a stub module with an empty ``Digraph`` class is put on ``sys.path`` when the real one is missing.
"""
from __future__ import annotations

import argparse
import os
import sys
import tempfile
import zlib
from pathlib import Path

import numpy as np
import torch
import torch.nn.functional as F

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))

# (name, M, K, N, seed, store_inputs, row_step)
CASES = [
    ("tiny_48x128x96", 48, 128, 96, 1, True, 1),
    ("ragged_37x200x72", 37, 200, 72, 2, True, 1),
    ("mid_130x512x264", 130, 512, 264, 3, False, 1),
    ("cfg1_256x1024x2816", 256, 1024, 2816, 0, False, 16),
]


def import_reference(ref_root: Path):
    try:
        import graphviz  # noqa: F401
    except ImportError:
        stub = Path(tempfile.mkdtemp(prefix="graphviz_stub_"))
        (stub / "graphviz.py").write_text("class Digraph:\n    pass\n")
        sys.path.insert(0, str(stub))
    os.environ.setdefault("MAGI_COMPILE_CACHE_ROOT_DIR", tempfile.mkdtemp(prefix="magi_cache_"))
    os.environ.setdefault("MAGI_LOGGING_LEVEL", "WARNING")
    sys.path.insert(0, str(ref_root))
    argv, sys.argv = sys.argv, sys.argv[:1]  # the reference's config object parses sys.argv
    try:
        from tests.model_definition import RMSNorm, TransformerConfig, TransformerMLP
    finally:
        sys.argv = argv
    return TransformerConfig, TransformerMLP, RMSNorm


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=str(HERE.parent.parent.parent / "reference"),
                    help="MagiCompiler checkout (default: a directory \"reference\" next to this repository)")
    args = ap.parse_args()
    from oracle import make_inputs, to_bits

    TransformerConfig, TransformerMLP, RMSNorm = import_reference(Path(args.reference))
    torch.set_num_threads(min(os.cpu_count() or 1, 8))
    out = {}
    for name, M, K, N, seed, store_inputs, row_step in CASES:
        x, w = make_inputs(M, K, N, seed=seed)
        cfg = TransformerConfig(vocab_size=8, hidden_size=K, intermediate_size=N, num_hidden_layers=1,
                                num_attention_heads=1, num_key_value_heads=1, max_position_embeddings=8,
                                params_dtype=torch.bfloat16)
        mlp = TransformerMLP(cfg)
        with torch.no_grad():
            mlp.gate_proj.weight.copy_(w[:N])
            mlp.up_proj.weight.copy_(w[N:])
            assert mlp.gate_proj.weight.dtype == torch.bfloat16
            y = F.silu(mlp.gate_proj(x)) * mlp.up_proj(x)  # TransformerMLP.forward before down_proj
        assert y.dtype == torch.bfloat16 and tuple(y.shape) == (M, N)
        out[f"{name}/shape"] = np.array([M, K, N, seed, row_step], dtype=np.int64)
        out[f"{name}/y_eager"] = to_bits(y)[::row_step].copy()
        out[f"{name}/crc"] = np.array([zlib.crc32(to_bits(x).tobytes()), zlib.crc32(to_bits(w).tobytes())], dtype=np.int64)
        if store_inputs:
            out[f"{name}/x"] = to_bits(x)
            out[f"{name}/w"] = to_bits(w)
        print(name, "ok", y.float().abs().max().item())
    # RMSNorm feeding the MLP's gate/up part, as in the reference's TransformerBlock.forward (lines 360-361)
    name, M, K, N, seed, eps = "rms_96x256x136", 96, 256, 136, 4, 1e-6
    x, w = make_inputs(M, K, N, seed=seed)
    gamma = 1.0 + 0.1 * torch.randn(K, generator=torch.Generator().manual_seed(seed))
    norm = RMSNorm(K, eps=eps)
    cfg = TransformerConfig(vocab_size=8, hidden_size=K, intermediate_size=N, num_hidden_layers=1,
                            num_attention_heads=1, num_key_value_heads=1, max_position_embeddings=8,
                            params_dtype=torch.bfloat16)
    mlp = TransformerMLP(cfg)
    with torch.no_grad():
        norm.weight.copy_(gamma)
        mlp.gate_proj.weight.copy_(w[:N])
        mlp.up_proj.weight.copy_(w[N:])
        xn = norm(x).to(torch.bfloat16)
        y = F.silu(mlp.gate_proj(xn)) * mlp.up_proj(xn)
    out[f"{name}/shape"] = np.array([M, K, N, seed, 1], dtype=np.int64)
    out[f"{name}/y_eager"] = to_bits(y)
    out[f"{name}/x"] = to_bits(x)
    out[f"{name}/w"] = to_bits(w)
    out[f"{name}/gamma"] = gamma.numpy()
    out[f"{name}/eps"] = np.array([eps])
    print(name, "ok", y.float().abs().max().item())
    np.savez_compressed(HERE / "swiglu_reference_eager.npz", **out)
    print("wrote", HERE / "swiglu_reference_eager.npz", (HERE / "swiglu_reference_eager.npz").stat().st_size, "bytes")


if __name__ == "__main__":
    main()
