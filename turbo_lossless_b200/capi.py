"""ctypes bindings of libsplit12_b200.so -- the C ABI declared in include/split12_b200.h.

The library is the product; there is no Python or CPU fallback.  Importing this
module on a machine where the shared library has not been built raises.
"""
from __future__ import annotations

import ctypes as C
import os

from . import _build

_vp, _i = C.c_void_p, C.c_int


class S12Tensor(C.Structure):
    """Mirror of the C struct S12Tensor (device pointers of one packed tensor)."""
    _fields_ = [("sm", _vp), ("gr", _vp), ("row_off", _vp), ("cols", _vp), ("correct", _vp),
                ("wrong", _vp), ("M", _i), ("K", _i), ("base_exp", _i), ("num_patches", _i)]


class S12PatchBatchDesc(C.Structure):
    """Mirror of PatchBatchDesc (decompress_v2.hip:36-44 of the reference): 56 bytes."""
    _fields_ = [("row_offsets", _vp), ("patch_cols", _vp), ("patch_correct", _vp),
                ("patch_wrong", _vp), ("activations", _vp), ("output", _vp), ("M", _i)]


# name -> (restype, argtypes); every symbol include/split12_b200.h declares
SIGNATURES = {
    "nv_launch_split12_v2_async": (_i, [_vp, _vp, _i, _vp, _vp, _i, _i, _vp]),
    "nv_launch_split12_v2_dual_async": (_i, [_vp, _vp, _i, _vp, _vp, _i, _vp, _vp, _vp, _i, _i, _vp]),
    "nv_launch_patches_async": (_i, [_vp] * 6 + [_i, _vp]),
    "nv_launch_patches_batch_async": (_i, [_vp] * 5 + [_i, _vp, _i, _vp, _i, _i, _vp]),
    "nv_launch_split12_fused_gemm_async": (_i, [_vp, _vp, _i, _vp, _i, _vp, _i, _i, _i, _i, _vp] + [_vp] * 4),
    "nv_launch_split12_fused_gemm_v3_async": (_i, [_vp, _vp, _i, _vp, _i, _vp, _i, _i, _i, _i, _vp] + [_vp] * 4),
    "nv_launch_split12_cublas_batch_async": (_i, [_vp, _vp, _i, _vp, _i, _vp, _i, _vp, _i, _i, _i, _i, _vp]),
    "launch_split12_v2_async": (_i, [_vp, _vp, _i, _vp, _vp, _i, _i, _vp]),
    "launch_split12_v2_dual_async": (_i, [_vp, _vp, _i, _vp, _vp, _i, _vp, _vp, _vp, _i, _i, _vp]),
    "launch_patches_v2": (_i, [_vp] * 6 + [_i]),
    "launch_patches_v2_async": (_i, [_vp] * 6 + [_i, _vp]),
    "launch_patches_b1_batched_async": (_i, [_vp, _vp, _i, _i, _vp]),
    "launch_split12_batch4_async": (_i, [_vp, _vp, _i] + [_vp] * 4 + [_vp] * 3 + [_vp] * 4 + [_i, _i, _vp]),
    "launch_split12_batch8_async": (_i, [_vp, _vp, _i] + [_vp] * 8 + [_vp] * 3 + [_vp] * 8 + [_i, _i, _vp]),
    "s12_decompress_async": (_i, [C.POINTER(S12Tensor), _vp, _vp]),
    "s12_gemv_async": (_i, [C.POINTER(S12Tensor), _i, _vp, C.POINTER(_vp), _vp]),
    "s12_gemv_batched_async": (_i, [C.POINTER(S12Tensor), _vp, _i, _vp, _i, _i, _vp]),
    "s12_gemm_async": (_i, [C.POINTER(S12Tensor), _vp, _i, _vp, _i, _i, _vp]),
    "s12_gemm_multi_async": (_i, [C.POINTER(S12Tensor), _i, _vp, _i, C.POINTER(_vp), C.POINTER(_i), _i, _vp]),
    "s12_gemm_noalloc_async": (_i, [C.POINTER(S12Tensor), _vp, _i, _vp, _i, _i, _vp]),
    "s12_init": (_i, []),
    "s12_set_dependent_launch": (_i, [_i]),
    "s12_last_error": (C.c_char_p, []),
    "s12_version": (_i, []),
    "s12_device_status": (_i, []),
    "s12_host_build_escape_table": (_i, [_vp, _vp, _vp, _i, _vp, _vp, _vp, _vp]),
    "s12_gemm_grouped_async": (_i, [C.POINTER(S12Tensor), _i, _vp, _i, C.POINTER(_i), C.POINTER(_vp), C.POINTER(_i), _i, _vp]),
    "s12_moe_route_async": (_i, [_vp, _i, _i] + [_vp] * 6),
    "s12_moe_gather_async": (_i, [_vp, _i, _i, _i, _i, _vp, _vp, _vp, _vp]),
    "s12_moe_combine_async": (_i, [_vp, _i, _i, _i, _vp, _vp, _vp, _vp, _i, _vp]),
    "s12_build_escape_table_async": (_i, [_vp] * 3 + [_i] + [_vp] * 6),
    "s12_tensor_dims": (_i, [C.c_char_p, C.c_char_p, C.POINTER(_i), C.POINTER(_i), C.POINTER(C.c_int64), C.POINTER(_i)]),
    "s12_load_tensor": (C.c_int64, [C.c_char_p, C.c_char_p] + [_vp] * 10 + [C.POINTER(_i), _vp]),
    "s12_host_shard_rows": (C.c_int64, [C.POINTER(S12Tensor), _i, _i] + [_vp] * 6),
    "s12_host_shard_cols": (C.c_int64, [C.POINTER(S12Tensor), _i, _i] + [_vp] * 6),
    "s12_pack_histogram_async": (_i, [_vp, C.c_int64, _vp, _vp]),
    "s12_pack_find_base_exp_host": (_i, [_vp]),
    "s12_pack_async": (_i, [_vp, _i, _i, _i, _vp, _vp, _vp, _vp]),
    "s12_pack_fill_async": (_i, [_vp, _i, _i, _i, _vp, _vp, _vp, _vp, _vp]),
    "launch_embed_lookup": (_i, [_vp, _vp, _vp, _i, _i, _i, _vp]),
    "launch_argmax": (_i, [_vp, _vp, _i, _vp]),
    "launch_argmax_batch": (_i, [_vp, _vp, _i, _i, _vp]),
    "launch_rms_norm_bf16_batch": (_i, [_vp, _vp, _vp, _i, C.c_float, _i, _vp]),
    "launch_add_rms_norm_bf16_batch": (_i, [_vp, _vp, _vp, _vp, _i, C.c_float, _i, _vp]),
    "launch_silu_mul_bf16_batch": (_i, [_vp, _vp, _vp, _i, _i, _vp]),
    "launch_add_batch": (_i, [_vp, _vp, _i, _i, _vp]),
    "launch_rope_store_kv": (_i, [_vp] * 7 + [_i, _i, _i, _i, _i, C.c_float, _vp]),
    "launch_rope_batch": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _i, C.c_float, _i, _vp]),
    "launch_store_kv_batch": (_i, [_vp] * 7 + [_i, _i, _i, _i, _i, _vp]),
    "launch_attention_all_heads": (_i, [_vp] * 6 + [_i, _i, _i, _i, _i, C.c_float, _vp]),
    "launch_attention_all_heads_batch": (_i, [_vp] * 7 + [_i, _i, _i, _i, C.c_float, _i, _i, _vp]),
    "launch_flash_attention": (_i, [_vp] * 6 + [_i, _i, _i, _i, _i, C.c_float, _vp]),
    "launch_flash_attention_batch": (_i, [_vp] * 7 + [_i, _i, _i, _i, C.c_float, _i, _i, _vp]),
    "s12_store_kv_batch": (_i, [_vp] * 7 + [_i, _i, C.c_longlong, _i, _vp]),
    "s12_rope_store_kv_batch": (_i, [_vp] * 8 + [_i, _i, _i, C.c_longlong, C.c_float, _i, _vp]),
    "s12_comm_handle_bytes": (_i, []),
    "s12_comm_create": (_i, [_i, _i, C.c_longlong, C.POINTER(_vp), _vp]),
    "s12_comm_connect": (_i, [_vp, _vp]),
    "s12_comm_connect_local": (_i, [C.POINTER(_vp), _i]),
    "s12_allreduce_f32_async": (_i, [_vp, _vp, _vp, _i, _vp]),
    "s12_allreduce_f32_emulated_async": (_i, [C.POINTER(_vp), _i, C.POINTER(_vp), C.POINTER(_vp), _i, _vp]),
    "s12_gemv_allreduce_async": (_i, [_vp, C.POINTER(S12Tensor), _vp, _vp, _vp]),
    "s12_comm_set_wait_limit_ms": (_i, [_vp, _i]),
    "s12_comm_reset": (_i, [_vp]),
    "s12_comm_destroy": (_i, [_vp]),
    "s12_tp_argmax_async": (_i, [_vp, _vp, _i, _i, _i, _vp, _vp]),
    "s12_tp_argmax_partial_async": (_i, [_vp, _i, _i, _i, _i, _i, _vp, _vp]),
    "s12_tp_argmax_merge_async": (_i, [_vp, _i, _i, _vp, _vp]),
}

_lib = None


def load(build_if_missing: bool = True) -> C.CDLL:
    """Loads the shared library (building it in-tree first when nvcc is available)."""
    global _lib
    if _lib is not None:
        return _lib
    path = _build.LIB_PATH
    if build_if_missing and not os.path.exists(path):
        _build.build()
    if not os.path.exists(path):
        raise RuntimeError(f"{path} is missing: run `python -m turbo_lossless_b200._build` (needs nvcc)")
    lib = C.CDLL(path)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)          # AttributeError if the library lacks a declared symbol
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


class S12Error(RuntimeError):
    pass


def check(rc: int, what: str = "") -> None:
    if rc != 0:
        msg = load().s12_last_error().decode(errors="replace")
        raise S12Error(f"{what} failed with {rc}: {msg}")
