"""ctypes view of libhipgpt_attn.so (the C ABI declared in include/hipgpt_attn.h).

There is no fallback: if the library is missing and cannot be built, or a call fails, an
exception is raised.
"""
from __future__ import annotations

import ctypes as C
import os

from . import build as _build

OK = 0
ERR_BAD_ARG, ERR_NULL, ERR_UNSUPPORTED, ERR_CUDA, ERR_SCRATCH = -1, -2, -3, -4, -5
ALGO_AUTO, ALGO_GENERIC, ALGO_ROWS, ALGO_TENSOR = 0, 1, 2, 3
TENSOR_DEFAULT, TENSOR_SPLIT_TF32, TENSOR_TILED, TENSOR_WHOLE_HEAD = 0, 1, 5, 6

_vp, _i, _sz = C.c_void_p, C.c_int, C.c_size_t

# name -> (restype, argtypes); one entry per declaration in include/hipgpt_attn.h
SIGNATURES = {
    "hipgpt_mha_forward": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp]),
    "hipgpt_mha_forward_ex": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp]),
    "hipgpt_mha_forward_planes": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _i, _vp]),
    "hipgpt_mha_forward_bf16": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp]),
    "hipgpt_mha_forward_bf16_ex": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp]),
    "hipgpt_mha_forward_host": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _i]),
    "hipgpt_mha_forward_bf16_host": (_i, [_vp, _vp, _i, _i, _i, _i, _i]),
    "hipgpt_release_workspace": (None, []),
    "hipgpt_scaled_dot_product": (_i, [_vp, _vp, _vp, _i, _i, _i, _vp]),
    "hipgpt_softmax": (_i, [_vp, _vp, _i, _i, _vp]),
    "hipgpt_attention_weighted_sum": (_i, [_vp, _vp, _vp, _i, _i, _i, _vp]),
    "hipgpt_mha_backward_scratch_bytes": (_sz, [_i, _i, _i]),
    "hipgpt_mha_backward": (_i, [_vp] * 9 + [_sz, _i, _i, _i, _i, _i, _vp]),
    "hipgpt_mha_backward_planes": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp]),
    "hipgpt_matmul": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _vp]),
    "hipgpt_matmul_tc": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _vp]),
    "hipgpt_matmul_tc_prepare": (_i, [_vp, _i, _i, C.POINTER(_vp), _vp]),
    "hipgpt_matmul_tc_prepared": (_i, [_vp, _vp, _vp, _vp, _i, _vp]),
    "hipgpt_matmul_tc_release": (None, [_vp]),
    "hipgpt_ln_matmul_tc": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp]),
    "hipgpt_ln_matmul_tc_prepared": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _vp]),
    "hipgpt_layer_norm": (_i, [_vp, _vp, _vp, _vp, _i, _i, _vp]),
    "hipgpt_dropout": (_i, [_vp, _vp, _vp, C.c_float, _i, _i, _vp]),
    "hipgpt_dropout_residual": (_i, [_vp, _vp, _vp, _vp, C.c_float, _i, _i, _vp]),
    "hipgpt_add_inplace": (_i, [_vp, _vp, C.c_longlong, _vp]),
    "hipgpt_relu": (_i, [_vp, C.c_longlong, _vp]),
    "hipgpt_embedding_lookup": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp]),
    "hipgpt_mha_decode_scratch_bytes": (_sz, [_i, _i, _i, _i]),
    "hipgpt_mha_decode": (_i, [_vp, _vp, _vp, _vp, _vp, _sz, _i, _i, _i, _i, _i, _vp]),
    "hipgpt_mha_decode_noalloc": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp]),
    "hipgpt_gpt_weight_count": (C.c_longlong, [_i, _i, _i, _i, _i, _i]),
    "hipgpt_gpt_create": (_i, [C.POINTER(_vp), _vp, _i, _i, _i, _i, _i, _i, _i]),
    "hipgpt_gpt_generate": (_i, [_vp, _vp, _i, _i, _i, _vp, _vp, C.POINTER(C.c_float), C.POINTER(C.c_float)]),
    "hipgpt_gpt_destroy": (None, [_vp]),
    "hipgpt_checkpoint_header": (_i, [C.c_char_p] + [C.POINTER(_i)] * 6),
    "hipgpt_checkpoint_weights": (_i, [C.c_char_p, _vp, C.c_longlong]),
    "hipgpt_run_config": (_i, [C.c_char_p] + [C.POINTER(_i)] * 6 + [C.c_char_p, _sz, C.c_char_p, _sz]),
    "hipgpt_gpt_create_from_checkpoint": (_i, [C.POINTER(_vp), C.c_char_p, _i]),
    "hipgpt_gpt_create_from_run": (_i, [C.POINTER(_vp), C.c_char_p, _i]),
    "hipgpt_gpt_set_mode": (_i, [_vp, _i]),
    "hipgpt_shard_range": (_i, [_i, _i, _i, C.POINTER(_i), C.POINTER(_i)]),
    "hipgpt_shard_chunk_range": (_i, [_i, _i, _i, _i, _i, C.POINTER(_i), C.POINTER(_i)]),
    "hipgpt_shard_unique_id": (_i, [_vp]),
    "hipgpt_shard_create": (_i, [C.POINTER(_vp), _vp, _i, _i]),
    "hipgpt_shard_destroy": (None, [_vp]),
    "hipgpt_mha_forward_sharded": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _vp]),
    "hipgpt_shard_output_buffer": (_i, [_vp, _sz, C.POINTER(_vp)]),
    "hipgpt_shard_nccl_version": (_i, []),
    "hipgpt_probe_fma": (_i, [_vp, _i, _i, C.POINTER(C.c_double), _vp]),
    "hipgpt_kernel_status": (_i, [C.POINTER(_i)]),
    "hipgpt_accuracy_notice": (_i, [C.POINTER(_i)]),
    "hipgpt_set_full_range": (_i, [_i]),
    "hipgpt_debug_wait_expiry": (_i, [_vp, _i, C.c_longlong, _vp]),
    "hipgpt_gpt_debug_stall_barrier": (_i, [_vp, C.c_longlong]),
    "hipgpt_last_error": (C.c_char_p, []),
    "hipgpt_version": (_i, []),
}
# the reference-named C++ launchers (include/hipgpt_launchers.hpp), by mangled name
CXX_LAUNCHERS = {
    "launch_multihead_attention": "_Z26launch_multihead_attentionPKfPfS1_iiii",
    "launch_scaled_dot_product": "_Z25launch_scaled_dot_productPKfS0_Pfiii",
    "launch_softmax": "_Z14launch_softmaxPKfPfii",
    "launch_attention_weighted_sum": "_Z29launch_attention_weighted_sumPKfS0_Pfiii",
    "launch_multihead_attention_backward": "_Z35launch_multihead_attention_backwardPKfS0_S0_Pfiiii",
    "launch_matmul": "_Z13launch_matmulPKfS0_Pfiii",
    "launch_matmul_add_bias": "_Z22launch_matmul_add_biasPKfS0_S0_Pfiii",
    "launch_layer_norm_forward": "_Z25launch_layer_norm_forwardPKfPfS0_S0_ii",
    "launch_dropout_forward": "_Z22launch_dropout_forwardPKfPfS1_fii",
    "launch_add_inplace": "_Z18launch_add_inplacePfPKfi",
    "launch_relu": "_Z11launch_reluPfi",
    "launch_embedding_lookup": "_Z23launch_embedding_lookupPKiPKfS2_Pfiiii",
}

_lib = None


class HipGPTError(RuntimeError):
    def __init__(self, code: int, text: str):
        super().__init__(f"hipgpt error {code}: {text}")
        self.code = code


def lib_path() -> str:
    return _build.LIB


def lib() -> C.CDLL:
    """Loads the library, building it first if the .so is absent (needs nvcc)."""
    global _lib
    if _lib is None:
        if not os.path.exists(_build.LIB):
            _build.build()
        handle = C.CDLL(_build.LIB)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype, fn.argtypes = res, args
        _lib = handle
    return _lib


def check(rc: int) -> None:
    if rc != OK:
        raise HipGPTError(rc, lib().hipgpt_last_error().decode("utf-8", "replace"))
