"""Python faces of the CUDA kernels.  Every function checks what it is given
(device, dtype, shape, contiguity), launches on the current CUDA stream and
raises `KernelError` if the kernel library refuses or fails.  There is no CPU
path: a tensor that is not on a CUDA device is an error.
"""
from ._lib import (PAGE_TOKENS, SM_COUNT, KernelError, check_status, count_launches, launch_count,  # noqa: F401
                   status_word, stream_scope, trace_report)
from .attention import (DECODE_CLUSTER_SPLITS, Rotation, attention, attention_decode,  # noqa: F401
                        attention_decode_rope, attention_decode_rope_supported, attention_mma_supported,
                        attention_prefill, attention_prefill_tc, attention_rows, attention_tc_supported, decode_splits)
from .chain import Chain, LazyRows  # noqa: F401
from .elementwise import GATE_ACTIVATIONS, embed, gather_rows, rmsnorm, rope_store, swiglu  # noqa: F401
from .gemm import (PendingLinear, ScaledRows, gemm_simt, gemm_tc_skinny, gemm_tc_supported,  # noqa: F401
                   gemm_tc_wide, interleave_gate_up, linear, linear_residual_norm, linear_swiglu, pair_pays,
                   residual_norm_supported)
from .sampling import argmax, sample  # noqa: F401
