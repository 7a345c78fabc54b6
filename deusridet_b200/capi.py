"""ctypes view of the C ABI in include/drkv.h.  Loading fails loudly when libdrkv.so has not
been built: there is no fallback implementation."""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libdrkv.so")

OK, ERR_INVALID, ERR_EXHAUSTED, ERR_NO_DEVICE, ERR_CUDA, ERR_STATE, ERR_CAPACITY = 0, -1, -2, -3, -4, -5, -6
F16, BF16 = 0, 1


class DrkvError(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"drkv status {code}: {msg}")
        self.code = code


class Geometry(C.Structure):
    _fields_ = [("num_layers", C.c_int32), ("num_q_heads", C.c_int32), ("num_kv_heads", C.c_int32),
                ("head_dim", C.c_int32), ("page_size", C.c_int32), ("dtype", C.c_int32),
                ("rotary_dim", C.c_int32), ("rope_theta", C.c_float)]


class Config(C.Structure):
    _fields_ = [("budget_bytes", C.c_size_t), ("max_pages", C.c_int32), ("max_seqs", C.c_int32),
                ("max_pages_per_seq", C.c_int32), ("device", C.c_int32), ("stream_evict", C.c_int32)]


class Stats(C.Structure):
    _fields_ = [(n, C.c_int64) for n in (
        "pages_total", "pages_free", "pages_cached", "pages_active", "evictions_cached", "evictions_stream",
        "cow_copies", "cow_bytes", "table_sync_bytes", "table_syncs", "live_seqs")]


class PlanInfo(C.Structure):
    _fields_ = [("n_seq", C.c_int32), ("n_families", C.c_int32), ("n_blocks", C.c_int32),
                ("chunk_tokens", C.c_int32), ("keys_per_sequence_pass", C.c_int64),
                ("keys_planned_pass", C.c_int64)]


class TierStats(C.Structure):
    _fields_ = [(n, C.c_int64) for n in (
        "pages_stored", "swap_outs", "swap_ins", "bytes_out", "bytes_in", "prefetch_hits", "page_file_bytes",
        "writes_deferred", "write_failures")]


class EvictRecord(C.Structure):
    _fields_ = [("kind", C.c_int32), ("seq", C.c_int32), ("logical", C.c_int32), ("page", C.c_int32)]


_vp, _i, _sz, _f = C.c_void_p, C.c_int, C.c_size_t, C.c_float
_pi32 = C.POINTER(C.c_int32)

# name -> (restype, argtypes); every symbol include/drkv.h declares
SIGNATURES = {
    "drkv_create": (_i, [C.POINTER(Geometry), C.POINTER(Config), C.POINTER(_vp)]),
    "drkv_destroy": (None, [_vp]),
    "drkv_last_error": (C.c_char_p, []),
    "drkv_get_geometry": (_i, [_vp, C.POINTER(Geometry)]),
    "drkv_get_stats": (_i, [_vp, C.POINTER(Stats)]),
    "drkv_pool_alloc": (_i, [_vp]),
    "drkv_pool_free": (_i, [_vp, _i]),
    "drkv_pool_free_count": (_i, [_vp]),
    "drkv_pool_max_pages": (_i, [_vp]),
    "drkv_pool_page_size": (_i, [_vp]),
    "drkv_pool_ptr": (_vp, [_vp]),
    "drkv_pool_total_bytes": (_sz, [_vp]),
    "drkv_pool_k_offset": (_sz, [_vp, _i, _i]),
    "drkv_pool_v_offset": (_sz, [_vp, _i, _i]),
    "drkv_seq_create": (_i, [_vp]),
    "drkv_seq_release": (_i, [_vp, _i, _i]),
    "drkv_seq_fork": (_i, [_vp, _i]),
    "drkv_seq_ensure_pos": (_i, [_vp, _i, _i, _vp]),
    "drkv_seq_ensure_range": (_i, [_vp, _i, _i, _i, _vp]),
    "drkv_seq_reserve": (_i, [_vp, _i, _i, _vp]),
    "drkv_seq_reserve_batch": (_i, [_vp, _i, _pi32, _i, _vp]),
    "drkv_seq_advance_batch": (_i, [_vp, _i, _pi32, _i]),
    "drkv_seq_set_len": (_i, [_vp, _i, _i]),
    "drkv_seq_len": (_i, [_vp, _i]),
    "drkv_seq_num_pages": (_i, [_vp, _i]),
    "drkv_seq_table": (_i, [_vp, _i, _pi32, _i]),
    "drkv_seq_adopt": (_i, [_vp, _i, _pi32, _i, _i]),
    "drkv_seq_evict": (_i, [_vp, _i, _i]),
    "drkv_evict_cached": (_i, [_vp, _i]),
    "drkv_ensure_free": (_i, [_vp, _i, _i]),
    "drkv_refcounts": (_i, [_vp, _pi32, _i]),
    "drkv_free_stack": (_i, [_vp, _pi32, _i]),
    "drkv_cached_lru": (_i, [_vp, _pi32, _i]),
    "drkv_evict_log": (_i, [_vp, C.POINTER(EvictRecord), _i, _i]),
    "drkv_sync_tables": (_i, [_vp, _vp]),
    "drkv_device_tables": (_vp, [_vp]),
    "drkv_table_stride": (_i, [_vp]),
    "drkv_kernel_error": (_i, [_vp]),
    "drkv_set_tail_split": (_i, [_vp, _i]),
    "drkv_set_prefill_on_decode_kernel": (_i, [_vp, _i]),
    "drkv_set_chunk_tokens": (_i, [_vp, _i]),
    "drkv_kernel_timing": (_i, [_vp, _i, C.POINTER(C.c_double), C.POINTER(C.c_int)]),
    "drkv_append_rope": (_i, [_vp, _i, _i, _vp, _vp, _vp, _vp, _vp]),
    "drkv_append_rope_chunk": (_i, [_vp, _i, _i, _i, _i, _vp, _vp, _vp]),
    "drkv_attend_decode": (_i, [_vp, _i, _i, _vp, _vp, _i, _vp, _vp, _f, _vp]),
    "drkv_append_attend_decode": (_i, [_vp, _i, _i, _vp, _vp, _i, _vp, _vp, _vp, _vp, _f, _vp]),
    "drkv_plan_decode": (_i, [_vp, _i, _pi32, _pi32, _vp]),
    "drkv_plan_get_info": (_i, [_vp, C.POINTER(PlanInfo)]),
    "drkv_plan_dump": (_i, [_vp, _pi32, _i]),
    "drkv_attend_decode_planned": (_i, [_vp, _i, _vp, _vp, _f, _vp]),
    "drkv_append_attend_decode_planned": (_i, [_vp, _i, _vp, _vp, _vp, _vp, _f, _vp]),
    "drkv_tier_enable": (_i, [_vp, C.c_char_p]),
    "drkv_tier_disable": (_i, [_vp]),
    "drkv_tier_prefetch": (_i, [_vp, _i, _i]),
    "drkv_tier_drain": (_i, [_vp]),
    "drkv_tier_set_write_behind": (_i, [_vp, _i]),
    "drkv_tier_is_prefetched": (_i, [_vp, _i, _i]),
    "drkv_tier_drop_prefetch": (_i, [_vp, _i, _i]),
    "drkv_tier_page_to_file": (_i, [_vp, _i, C.c_char_p]),
    "drkv_tier_file_to_page": (_i, [_vp, C.c_char_p, _i]),
    "drkv_tier_get_stats": (_i, [_vp, C.POINTER(TierStats)]),
    "drkv_seq_locations": (_i, [_vp, _i, C.POINTER(C.c_int8), _i]),
    "drkv_scorer_enable": (_i, [_vp, _f]),
    "drkv_scorer_update": (_i, [_vp, _i, _vp, _i, _vp]),
    "drkv_scorer_step": (_i, [_vp, _vp]),
    "drkv_scorer_sync": (_i, [_vp, _vp]),
    "drkv_scorer_scores": (_i, [_vp, _i, C.POINTER(C.c_float), _i]),
    "drkv_attend_prefill_chunk": (_i, [_vp, _i, _i, _i, _i, _vp, _vp, _f, _vp]),
    "drkv_attend_prefill_batch": (_i, [_vp, _i, _i, _pi32, _pi32, _pi32, C.POINTER(_vp), C.POINTER(_vp), _f, _vp]),
    "drkv_exchange_create": (_i, [_vp, _i, _i, C.POINTER(C.c_uint8)]),
    "drkv_exchange_connect": (_i, [_vp, C.POINTER(C.c_uint8)]),
    "drkv_exchange_destroy": (_i, [_vp]),
    "drkv_exchange_connect_local": (_i, [_vp, C.POINTER(C.c_void_p)]),
    "drkv_exchange_area": (_vp, [_vp]),
    "drkv_exchange_set_wait_ms": (_i, [_vp, _i]),
    "drkv_attend_exchange": (_i, [_vp, _i, _i, _i, _i, _vp, _vp, _f, _vp]),
    "drkv_append_attend_exchange": (_i, [_vp, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _f, _vp]),
    "drkv_attend_partial": (_i, [_vp, _i, _i, _i, _i, _vp, _vp, _f, _vp]),
    "drkv_combine_partials": (_i, [_vp, _i, _vp, _vp, _vp]),
    "drkv_partial_floats": (_sz, [_vp]),
    "drkv_k_cache_write": (_i, [C.POINTER(Geometry), _vp, _vp, _vp, _vp, _i, _vp, _i, _vp]),
    "drkv_k_cache_write_batch": (_i, [C.POINTER(Geometry), _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp]),
    "drkv_k_decode_attention": (_i, [C.POINTER(Geometry), _vp, _vp, _vp, _vp, _i, _i, _i, _f, _vp, _sz, _vp]),
    "drkv_seq_extract": (_i, [_vp, _i, _i, _i, _vp, _vp]),
    "drkv_seq_inject": (_i, [_vp, _i, _i, _i, _vp, _vp]),
    "drkv_k_extract_kv": (_i, [C.POINTER(Geometry), _vp, _vp, _vp, _i, _i, _i, _vp]),
    "drkv_k_inject_kv": (_i, [C.POINTER(Geometry), _vp, _vp, _vp, _i, _i, _i, _vp]),
    "drkv_shard_page_range": (_i, [_i, _i, _i, C.POINTER(C.c_int), C.POINTER(C.c_int)]),
    "drkv_shard_key_range": (_i, [_i, _i, _i, _i, C.POINTER(C.c_int), C.POINTER(C.c_int)]),
    "drkv_shard_owner_of_position": (_i, [_i, _i, _i, _i]),
    "drkv_shard_sequences": (_i, [_i, C.POINTER(C.c_int64), _pi32, _i, _pi32]),
    "drkv_k_decode_scratch_bytes": (_sz, [C.POINTER(Geometry), _i]),
    "drkv_k_decode_kernel_error": (_i, [_vp, _vp]),
    "drkv_k_decode_attention_noalloc": (_i, [C.POINTER(Geometry), _vp, _vp, _vp, _vp, _i, _i, _i, _f, _vp]),
}
NOALLOC_SCRATCH_BYTES = 4 << 20

_lib = None


def load_library() -> C.CDLL:
    """Loads libdrkv.so and types every entry point; raises if the library is missing."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build the CUDA extension first (python -m deusridet_b200.build). "
            "There is no CPU fallback.")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the library does not export it
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def last_error() -> str:
    return (load_library().drkv_last_error() or b"").decode()


def check(rc: int) -> int:
    if rc < 0:
        raise DrkvError(rc, last_error())
    return rc
