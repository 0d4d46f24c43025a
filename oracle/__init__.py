"""TEST INFRASTRUCTURE — CPU oracle for the fused GEMM-SwiGLU path (not part of the product).

Only the test-suite, the smoke check and the CPU-baseline legs of the benchmark may import this
package.  The product (``magicompiler_b200``) never does, and fails loudly without its CUDA library.

Contents
--------
``swiglu_oracle.c``   plain-C restatement on bf16 bit patterns (built into ``oracle/_build/``)
``swiglu_gold``       fp32-accumulated gold + single-rounded bf16 + the reference's eager rounding chain
``swiglu_gold_numpy`` the same gold in numpy (small cases; cross-checks the C code)
``swiglu_ref_eager``  the reference's eager PyTorch expression on the packed weight
                      (MagiCompiler tests/model_definition.py:337-339, example/training/llama3.py:173)

Parity pin: MagiCompiler's tests hold no golden vector for this path; the oracle is pinned by
fixtures produced by running the reference's own ``TransformerMLP`` (``tests/golden/make_golden.py``).
"""
from .swiglu_oracle import (  # noqa: F401
    build,
    error_metrics,
    e2m1_round,
    make_inputs,
    nvfp4_quantize_gold,
    nvfp4_swizzled_offsets,
    rmsnorm_swiglu_gold,
    rmsnorm_swiglu_ref_eager,
    swiglu_backward_gold,
    swiglu_gold,
    swiglu_gold_numpy,
    swiglu_ref_eager,
    to_bits,
    from_bits,
    TOL_MAX_NORM,
    TOL_FROB,
)
