"""B200-native (sm_100a) KernelIR backend for StatefulLLM-Compiler's serving path.

Compute lives in libb200serve.so (hand-written CUDA behind a C ABI, include/b200_serve.h);
this package is the host side: ctypes binding, kernel wrappers with the reference's
signatures, the preallocated KV state, the KernelIR executor, and the CUDA-graph serving
engine. There is no Triton, no backend dispatch and no CPU fallback.
"""

from . import _lib
from .kernels import (
    KernelStatusError,
    b200_add,
    b200_advance_lengths,
    b200_argmax,
    b200_contiguous,
    b200_decode_attention,
    b200_decode_attention_no_alloc,
    b200_embedding,
    b200_kv_store,
    b200_linear,
    b200_paged_decode_attention,
    b200_paged_kv_store,
    b200_prefill_attention,
    b200_rms_norm,
    b200_rope,
    b200_rope_kv_store,
    b200_rope_table,
    b200_swiglu,
)
from .kv_state import ExecutionError, PagedKVCacheState, PreallocatedKVCacheState
from .qwen2 import QWEN2_0_5B, QWEN2_7B, TINY_FP32, Qwen2Config, make_prompt_ids, make_weights

__all__ = [
    "ExecutionError", "KernelStatusError", "PagedKVCacheState", "PreallocatedKVCacheState", "Qwen2Config",
    "QWEN2_0_5B", "QWEN2_7B", "TINY_FP32", "make_prompt_ids", "make_weights",
    "b200_add", "b200_advance_lengths", "b200_argmax", "b200_contiguous",
    "b200_decode_attention", "b200_decode_attention_no_alloc", "b200_embedding", "b200_kv_store", "b200_linear",
    "b200_paged_decode_attention", "b200_paged_kv_store", "b200_prefill_attention", "b200_rms_norm", "b200_rope", "b200_rope_kv_store",
    "b200_rope_table", "b200_swiglu",
]
