"""ctypes binding of libb2a.so.  There is no fallback: a missing library is an error."""
from __future__ import annotations

import ctypes as C
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libb2a.so")

F32, F16, BF16, U8 = 0, 1, 2, 3
MASK_NONE, MASK_BOOL, MASK_ADD = 0, 1, 2
DEV_TIMEOUT, DEV_BAD_BLOCK, DEV_BAD_LEN = 1, 2, 4
BUILTIN_SCRATCH_BYTES = 16 << 20


class SdpaDesc(C.Structure):
    _fields_ = [
        ("dtype", C.c_int32), ("B", C.c_int32), ("Hq", C.c_int32), ("Hkv", C.c_int32), ("Sq", C.c_int32),
        ("Skv", C.c_int32), ("D", C.c_int32), ("Dv", C.c_int32), ("causal", C.c_int32), ("scale", C.c_float),
        ("q_strides", C.c_int64 * 4), ("k_strides", C.c_int64 * 4), ("v_strides", C.c_int64 * 4),
        ("o_strides", C.c_int64 * 4), ("mask_kind", C.c_int32), ("reserved", C.c_int32),
        ("mask_strides", C.c_int64 * 4),
    ]


class PagedDesc(C.Structure):
    _fields_ = [
        ("q_dtype", C.c_int32), ("kv_dtype", C.c_int32), ("Hq", C.c_int32), ("Hkv", C.c_int32), ("D", C.c_int32),
        ("Dv", C.c_int32), ("block_size", C.c_int32), ("num_seqs", C.c_int32), ("num_tokens", C.c_int32),
        ("num_blocks_total", C.c_int32), ("max_context_len", C.c_int32), ("max_q_len", C.c_int32),
        ("scale", C.c_float), ("sliding_window", C.c_int32), ("prefill_row_blocks", C.c_int32),
        ("prefill_kv_tokens", C.c_int32),
        ("cache_rows_settled", C.c_int32),
    ]


# name -> (restype, argtypes); the single list of what include/b2a.h declares
SIGNATURES = {
    "b2a_version": (C.c_int, []),
    "b2a_status_string": (C.c_char_p, [C.c_int]),
    "b2a_sdpa_workspace_bytes": (C.c_int, [C.POINTER(SdpaDesc), C.c_int, C.POINTER(C.c_size_t)]),
    "b2a_sdpa_forward": (C.c_int, [C.POINTER(SdpaDesc), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                   C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p]),
    "b2a_paged_chunk_bytes": (C.c_size_t, [C.c_int32, C.c_int32, C.c_int32]),
    "b2a_paged_workspace_bytes": (C.c_int, [C.POINTER(PagedDesc), C.c_int, C.POINTER(C.c_size_t)]),
    "b2a_paged_kv_store": (C.c_int, [C.POINTER(PagedDesc), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                     C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "b2a_paged_kv_store_rope": (C.c_int, [C.POINTER(PagedDesc), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                          C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                          C.c_int32, C.c_int32, C.c_void_p, C.c_void_p]),
    "b2a_paged_attention": (C.c_int, [C.POINTER(PagedDesc), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                      C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t,
                                      C.c_void_p, C.c_void_p]),
    "b2a_paged_attention_noalloc": (C.c_int, [C.POINTER(PagedDesc), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                              C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "b2a_paged_scores_workspace_bytes": (C.c_int, [C.POINTER(PagedDesc), C.c_int, C.POINTER(C.c_size_t)]),
    "b2a_paged_last_token_scores": (C.c_int, [C.POINTER(PagedDesc), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                              C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p,
                                              C.c_size_t, C.c_void_p, C.c_void_p]),
    "b2a_shard_group_create": (C.c_int, [C.c_int, C.c_int, C.c_size_t, C.POINTER(C.c_void_p)]),
    "b2a_shard_group_handle": (C.c_int, [C.c_void_p, C.c_char_p]),
    "b2a_shard_group_connect": (C.c_int, [C.c_void_p, C.c_char_p]),
    "b2a_shard_group_connect_pointers": (C.c_int, [C.c_void_p, C.POINTER(C.c_void_p)]),
    "b2a_shard_group_set_wait_ms": (C.c_int, [C.c_void_p, C.c_int]),
    "b2a_shard_group_reset": (C.c_int, [C.c_void_p]),
    "b2a_shard_group_destroy": (None, [C.c_void_p]),
    "b2a_shard_group_output": (C.c_int, [C.c_void_p, C.POINTER(C.c_void_p)]),
    "b2a_paged_attention_sharded": (C.c_int, [C.c_void_p, C.POINTER(PagedDesc), C.c_void_p, C.c_void_p, C.c_void_p,
                                              C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                              C.c_size_t, C.c_void_p, C.c_void_p]),
    "b2a_sdpa_forward_sharded": (C.c_int, [C.c_void_p, C.POINTER(SdpaDesc), C.c_void_p, C.c_void_p, C.c_void_p,
                                           C.POINTER(C.c_void_p), C.c_void_p, C.c_void_p]),
    "b2a_host_sdpa_create": (C.c_int, [C.c_int32] * 9 + [C.POINTER(C.c_void_p)]),
    "b2a_host_sdpa_run": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "b2a_host_sdpa_pieces": (C.c_int, [C.c_void_p]),
    "b2a_host_sdpa_destroy": (None, [C.c_void_p]),
    "b2a_kvstate_create": (C.c_int, [C.c_int32] * 8 + [C.POINTER(C.c_void_p)]),
    "b2a_kvstate_destroy": (None, [C.c_void_p]),
    "b2a_kvstate_length": (C.c_int32, [C.c_void_p]),
    "b2a_kvstate_reset": (C.c_int, [C.c_void_p]),
    "b2a_kvstate_set_state": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p]),
    "b2a_kvstate_get_state": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p]),
    "b2a_kvstate_append": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p]),
    "b2a_kvstate_read_dense": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p]),
    "b2a_kvstate_last_step": (C.c_int, [C.c_void_p, C.c_void_p]),
    "b2a_kvstate_export_bytes": (C.c_size_t, [C.c_void_p]),
    "b2a_kvstate_export": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    "b2a_kvstate_import": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    "b2a_kvmgr_create": (C.c_int, [C.c_int32, C.c_int32, C.c_uint64, C.POINTER(C.c_void_p)]),
    "b2a_kvmgr_destroy": (None, [C.c_void_p]),
    "b2a_kvmgr_add_sequence": (C.c_int, [C.c_void_p, C.c_int64]),
    "b2a_kvmgr_free_sequence": (C.c_int, [C.c_void_p, C.c_int64]),
    "b2a_kvmgr_free_blocks": (C.c_int32, [C.c_void_p]),
    "b2a_kvmgr_sequence_len": (C.c_int32, [C.c_void_p, C.c_int64]),
    "b2a_kvmgr_last_prefill_row_blocks": (C.c_int32, [C.c_void_p]),
    "b2a_kvmgr_last_prefill_kv_tokens": (C.c_int32, [C.c_void_p]),
    "b2a_kvmgr_schedule_step": (C.c_int, [C.c_void_p, C.POINTER(C.c_int64), C.POINTER(C.c_int32), C.c_int32,
                                          C.POINTER(C.c_int32), C.POINTER(C.c_int32), C.POINTER(C.c_int32),
                                          C.c_int32, C.POINTER(C.c_int32), C.POINTER(C.c_int32),
                                          C.POINTER(C.c_int32)]),
}

_lib = None


def load() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m openvino_contrib_b200.build` "
                "(there is no CPU or PyTorch fallback for the attention path)")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)  # AttributeError if the library does not export it
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib


class B2AError(RuntimeError):
    def __init__(self, code: int, where: str):
        self.code = code
        super().__init__(f"{where}: {load().b2a_status_string(code).decode()} (b2a_status {code})")


def check(code: int, where: str) -> None:
    if code != 0:
        raise B2AError(code, where)
