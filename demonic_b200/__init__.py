"""demonic_b200 -- B200 (sm_100a) backend for demoniC's matmul operator `@`.

The product is ``libdmc_cuda.so`` (C ABI in ``include/dmc_cuda.h``); this
package is the thin host-side mirror used by the tests and the benchmark to
play the role of JIT-emitted code: it passes raw host pointers to the same
entry points the reference JIT would bind.
"""
from ._lib import DmcCudaError, check, load  # noqa: F401
from .backend import (  # noqa: F401
    DeviceBuffer,
    LAYOUT_KN,
    LAYOUT_NK,
    W_BF16,
    W_F32,
    matmul_bf16_gpu,
    matmul_bf16_gpu_batched,
    matmul_bf16_gpu_batched_deferred,
    matmul_bf16_gpu_flush,
    matmul_bf16_gpu_nt,
    matmul_f32_gpu,
    matmul_selected,
)
