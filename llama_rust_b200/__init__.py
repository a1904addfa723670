"""B200-native (sm_100a) executor for the quantized matrix-product path of llama-rust.

The product is ``libllama_rust_b200.so`` (C ABI in ``include/llama_rust_b200.h``);
this package is its Python host side: ``executor`` mirrors the reference's
``CudaGemv``/``CudaMatrix``, ``quant`` its ``gemv_*``/``gemm_*`` entry points,
``synth`` the seeded synthetic-weight recipe shared with the device generator.
"""
from .executor import (BF16, DTYPES, F16, F32, Q4_0, Q4_1, Q4_K, Q5_0, Q5_1, Q5_K, Q6_K, Q8_0, Executor, Matrix,
                       NativeCudaError, Session, XOP_NONE, XOP_RMSNORM, XOP_SWIGLU, row_bytes, plan_placement,
                       MOVE_WEIGHTS, DISPATCH_ACTIVATIONS)

from .engine import Engine, EngineCfg

__all__ = ["Engine", "EngineCfg", "Executor", "Matrix", "Session", "NativeCudaError", "row_bytes", "DTYPES", "F16", "BF16", "F32",
           "Q5_0", "Q5_1", "Q4_0", "Q4_1", "Q5_K", "Q8_0", "Q4_K", "Q6_K", "XOP_NONE", "XOP_RMSNORM", "XOP_SWIGLU", "plan_placement",
           "MOVE_WEIGHTS", "DISPATCH_ACTIVATIONS"]
