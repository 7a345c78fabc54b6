"""PagedKVEngine: Python host over the C ABI, mirroring the reference's call surface
(BlockPool / CacheManager methods, src/memoria/block_pool.h:69-107 and
src/memoria/cache_manager.h:67-125, plus the paged_* free functions,
src/machina/paged_attention.h:27-71).  Device buffers are passed as raw pointers; torch
tensors are accepted wherever a pointer is (their data_ptr() is used)."""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import numpy as np

from . import capi
from .capi import Config, Geometry, check


def _ptr(x) -> Optional[int]:
    if x is None:
        return None
    if isinstance(x, int):
        return x
    return x.data_ptr()  # torch tensor


def _stream(stream) -> Optional[int]:
    if stream is None:
        return None
    if isinstance(stream, int):
        return stream
    return stream.cuda_stream  # torch.cuda.Stream


class PagedKVEngine:
    def __init__(self, *, num_layers: int, num_q_heads: int, num_kv_heads: int, head_dim: int, page_size: int,
                 dtype: str = "bf16", rotary_dim: Optional[int] = None, rope_theta: float = 10000.0,
                 max_pages: int = 0, budget_bytes: int = 0, max_seqs: int = 1, max_pages_per_seq: int = 0,
                 device: int = 0, stream_evict: bool = False):
        self.lib = capi.load_library()
        self.geom = Geometry(num_layers, num_q_heads, num_kv_heads, head_dim, page_size,
                             capi.F16 if dtype in ("f16", "fp16") else capi.BF16,
                             head_dim if rotary_dim is None else rotary_dim, rope_theta)
        cfg = Config(budget_bytes, max_pages, max_seqs, max_pages_per_seq, device, 1 if stream_evict else 0)
        h = C.c_void_p()
        check(self.lib.drkv_create(C.byref(self.geom), C.byref(cfg), C.byref(h)))
        self.h = h
        self.device = device

    def close(self):
        if getattr(self, "h", None):
            self.lib.drkv_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ---- BlockPool -------------------------------------------------------------------
    def alloc_block(self) -> int: return self.lib.drkv_pool_alloc(self.h)
    def free_block(self, page: int) -> None: check(self.lib.drkv_pool_free(self.h, page))
    def free_count(self) -> int: return self.lib.drkv_pool_free_count(self.h)
    def max_blocks(self) -> int: return self.lib.drkv_pool_max_pages(self.h)
    def block_size(self) -> int: return self.lib.drkv_pool_page_size(self.h)
    def pool_ptr(self) -> int: return self.lib.drkv_pool_ptr(self.h) or 0
    def total_bytes(self) -> int: return self.lib.drkv_pool_total_bytes(self.h)
    def k_offset(self, layer: int, page: int) -> int: return self.lib.drkv_pool_k_offset(self.h, layer, page)
    def v_offset(self, layer: int, page: int) -> int: return self.lib.drkv_pool_v_offset(self.h, layer, page)

    def pool_tensor(self):
        """The pool slab as a flat int16 torch tensor aliasing the engine's device memory."""
        import torch

        class _Raw:
            pass

        raw = _Raw()
        raw.__cuda_array_interface__ = {"shape": (self.total_bytes() // 2,), "typestr": "<i2",
                                        "data": (self.pool_ptr(), False), "version": 2}
        return torch.as_tensor(raw, device=f"cuda:{self.device}")

    # ---- sequences (CacheManager, one row per sequence) ---------------------------------
    def seq_create(self) -> int: return check(self.lib.drkv_seq_create(self.h))
    def seq_release(self, seq: int, discard: bool = False) -> None:
        check(self.lib.drkv_seq_release(self.h, seq, 1 if discard else 0))
    def seq_fork(self, parent: int) -> int: return check(self.lib.drkv_seq_fork(self.h, parent))
    def ensure_blocks_for(self, seq: int, pos: int, stream=None) -> bool:
        return self.lib.drkv_seq_ensure_pos(self.h, seq, pos, _stream(stream)) == 0
    def ensure_blocks_for_range(self, seq: int, pos_start: int, m: int, stream=None) -> bool:
        return self.lib.drkv_seq_ensure_range(self.h, seq, pos_start, m, _stream(stream)) == 0
    def reserve(self, seq: int, n_tokens: int, stream=None) -> None:
        check(self.lib.drkv_seq_reserve(self.h, seq, n_tokens, _stream(stream)))
    def reserve_batch(self, seqs, n_tokens: int, stream=None) -> None:
        arr = np.ascontiguousarray(seqs, dtype=np.int32)
        check(self.lib.drkv_seq_reserve_batch(self.h, len(arr), arr.ctypes.data_as(C.POINTER(C.c_int32)), n_tokens,
                                              _stream(stream)))
    def advance_batch(self, seqs, n_tokens: int) -> None:
        arr = np.ascontiguousarray(seqs, dtype=np.int32)
        check(self.lib.drkv_seq_advance_batch(self.h, len(arr), arr.ctypes.data_as(C.POINTER(C.c_int32)), n_tokens))
    def set_seq_len(self, seq: int, n: int) -> None: check(self.lib.drkv_seq_set_len(self.h, seq, n))
    def seq_len(self, seq: int) -> int: return check(self.lib.drkv_seq_len(self.h, seq))
    def num_logical_blocks(self, seq: int) -> int: return check(self.lib.drkv_seq_num_pages(self.h, seq))
    def adopt(self, seq: int, pages: Sequence[int], n_tokens: int) -> None:
        arr = (C.c_int32 * len(pages))(*pages)
        check(self.lib.drkv_seq_adopt(self.h, seq, arr, len(pages), n_tokens))
    def table(self, seq: int, n: Optional[int] = None) -> np.ndarray:
        n = self.table_stride() if n is None else n
        out = np.empty(n, dtype=np.int32)
        got = check(self.lib.drkv_seq_table(self.h, seq, out.ctypes.data_as(C.POINTER(C.c_int32)), n))
        return out[:got]

    # ---- eviction ----------------------------------------------------------------------
    def evict_blocks(self, seq: int, n: int) -> int: return check(self.lib.drkv_seq_evict(self.h, seq, n))
    def evict_cached(self, n: int) -> int: return check(self.lib.drkv_evict_cached(self.h, n))
    def ensure_free_blocks(self, seq: int, n_free: int) -> bool:
        return self.lib.drkv_ensure_free(self.h, seq, n_free) == 1

    # ---- inspection ----------------------------------------------------------------------
    def _ints(self, fn, cap: int) -> np.ndarray:
        out = np.empty(max(cap, 1), dtype=np.int32)
        n = check(fn(self.h, out.ctypes.data_as(C.POINTER(C.c_int32)), cap))
        return out[:n].copy()
    def refcounts(self) -> np.ndarray: return self._ints(self.lib.drkv_refcounts, self.max_blocks())
    def free_stack(self) -> np.ndarray: return self._ints(self.lib.drkv_free_stack, self.max_blocks())
    def cached_lru(self) -> np.ndarray: return self._ints(self.lib.drkv_cached_lru, self.max_blocks())
    def evict_log(self, clear: bool = True):
        cap = 1 << 16
        buf = (capi.EvictRecord * cap)()
        n = check(self.lib.drkv_evict_log(self.h, buf, cap, 1 if clear else 0))
        return [(buf[i].kind, buf[i].seq, buf[i].logical, buf[i].page) for i in range(n)]
    def stats(self) -> dict:
        s = capi.Stats()
        check(self.lib.drkv_get_stats(self.h, C.byref(s)))
        return {n: getattr(s, n) for n, _ in capi.Stats._fields_}

    # ---- device tables --------------------------------------------------------------------
    def sync_block_table(self, stream=None) -> None: check(self.lib.drkv_sync_tables(self.h, _stream(stream)))
    def d_block_table(self) -> int: return self.lib.drkv_device_tables(self.h) or 0
    def table_stride(self) -> int: return self.lib.drkv_table_stride(self.h)
    def check_kernels(self) -> None: check(self.lib.drkv_kernel_error(self.h))
    def set_tail_split(self, mode: int) -> None: check(self.lib.drkv_set_tail_split(self.h, mode))
    def set_prefill_on_decode_kernel(self, on: bool) -> None:
        check(self.lib.drkv_set_prefill_on_decode_kernel(self.h, 1 if on else 0))
    def set_chunk_tokens(self, n: int) -> None: check(self.lib.drkv_set_chunk_tokens(self.h, n))

    def kernel_timing(self, enable: bool, read: bool = False):
        """Switches per-launch event timing of the decode kernel; with read=True returns
        (total_ms, launches) accumulated since the previous call."""
        if read:
            ms, n = C.c_double(), C.c_int()
            check(self.lib.drkv_kernel_timing(self.h, 1 if enable else 0, C.byref(ms), C.byref(n)))
            return ms.value, n.value
        check(self.lib.drkv_kernel_timing(self.h, 1 if enable else 0, None, None))
        return None

    # ---- kernels ----------------------------------------------------------------------------
    def append_rope(self, layer, n_seq, d_rows, d_pos, k_src, v_src, stream=None) -> None:
        check(self.lib.drkv_append_rope(self.h, layer, n_seq, _ptr(d_rows), _ptr(d_pos), _ptr(k_src), _ptr(v_src),
                                        _stream(stream)))
    def append_rope_chunk(self, layer, seq, pos_start, m, k_src, v_src, stream=None) -> None:
        check(self.lib.drkv_append_rope_chunk(self.h, layer, seq, pos_start, m, _ptr(k_src), _ptr(v_src),
                                              _stream(stream)))
    def attend_decode(self, layer, n_seq, d_rows, d_kv_len, max_kv_len, q, out, scale, stream=None) -> None:
        check(self.lib.drkv_attend_decode(self.h, layer, n_seq, _ptr(d_rows), _ptr(d_kv_len), max_kv_len, _ptr(q),
                                          _ptr(out), scale, _stream(stream)))
    def append_attend_decode(self, layer, n_seq, d_rows, d_kv_len, max_kv_len, k_src, v_src, q, out, scale, stream=None) -> None:
        """Append of each entry's new token (at kv_len - 1) and decode attention over kv_len keys, one call."""
        check(self.lib.drkv_append_attend_decode(self.h, layer, n_seq, _ptr(d_rows), _ptr(d_kv_len), max_kv_len,
                                                 _ptr(k_src), _ptr(v_src), _ptr(q), _ptr(out), scale, _stream(stream)))
    def plan_decode(self, seqs, kv_len, stream=None) -> dict:
        """Shared-prefix plan for a decode batch (host lists); returns the plan's summary."""
        n = len(seqs)
        i32 = lambda v: (C.c_int32 * n)(*[int(x) for x in v])
        check(self.lib.drkv_plan_decode(self.h, n, i32(seqs), i32(kv_len), _stream(stream)))
        info = capi.PlanInfo()
        check(self.lib.drkv_plan_get_info(self.h, C.byref(info)))
        return {f: getattr(info, f) for f, _ in capi.PlanInfo._fields_}
    def plan_dump(self) -> dict:
        """The current plan's arrays (see drkv_plan_dump)."""
        n = check(self.lib.drkv_plan_dump(self.h, None, 0))
        buf = np.empty(n, dtype=np.int32)
        check(self.lib.drkv_plan_dump(self.h, buf.ctypes.data_as(C.POINTER(C.c_int32)), n))
        info = capi.PlanInfo()
        check(self.lib.drkv_plan_get_info(self.h, C.byref(info)))
        ns, nb = info.n_seq, info.n_blocks
        return {"rows": buf[:ns], "kv_len": buf[ns:2 * ns], "first_chunk": buf[2 * ns:3 * ns],
                "fb_row": buf[3 * ns:3 * ns + nb], "fb_chunks": buf[3 * ns + nb:3 * ns + 2 * nb],
                "fb_members": buf[3 * ns + 2 * nb:].reshape(nb, 16)}
    def attend_decode_planned(self, layer, q, out, scale, stream=None) -> None:
        check(self.lib.drkv_attend_decode_planned(self.h, layer, _ptr(q), _ptr(out), scale, _stream(stream)))
    def append_attend_decode_planned(self, layer, k_src, v_src, q, out, scale, stream=None) -> None:
        """The planned pass with each entry's new token (position kv_len - 1 of the plan) appended in the same call."""
        check(self.lib.drkv_append_attend_decode_planned(self.h, layer, _ptr(k_src), _ptr(v_src), _ptr(q), _ptr(out),
                                                         scale, _stream(stream)))
    # ---- storage tier (KVSwapper + CacheManager swap paths) -----------------------------------
    def tier_enable(self, directory: str) -> None: check(self.lib.drkv_tier_enable(self.h, directory.encode()))
    def tier_disable(self) -> None: check(self.lib.drkv_tier_disable(self.h))
    def prefetch_block(self, seq: int, logical: int) -> int: return check(self.lib.drkv_tier_prefetch(self.h, seq, logical))
    def tier_drain(self) -> None: check(self.lib.drkv_tier_drain(self.h))
    def tier_set_write_behind(self, on: bool) -> None: check(self.lib.drkv_tier_set_write_behind(self.h, 1 if on else 0))
    def is_prefetched(self, seq: int, logical: int) -> bool: return check(self.lib.drkv_tier_is_prefetched(self.h, seq, logical)) == 1
    def drop_prefetch(self, seq: int, logical: int) -> None: check(self.lib.drkv_tier_drop_prefetch(self.h, seq, logical))
    def page_to_file(self, page: int, path: str) -> None: check(self.lib.drkv_tier_page_to_file(self.h, page, path.encode()))
    def file_to_page(self, path: str, page: int) -> None: check(self.lib.drkv_tier_file_to_page(self.h, path.encode(), page))
    def tier_stats(self) -> dict:
        st = capi.TierStats()
        check(self.lib.drkv_tier_get_stats(self.h, C.byref(st)))
        return {f: getattr(st, f) for f, _ in capi.TierStats._fields_}
    def locations(self, seq: int) -> np.ndarray:
        out = np.empty(self.table_stride(), dtype=np.int8)
        n = check(self.lib.drkv_seq_locations(self.h, seq, out.ctypes.data_as(C.POINTER(C.c_int8)), len(out)))
        return out[:n]

    # ---- importance scorer (ImportanceScorer + CacheManager::pick_eviction_candidate) ----------
    def scorer_enable(self, decay: float = 0.95) -> None: check(self.lib.drkv_scorer_enable(self.h, decay))
    def scorer_disable(self) -> None: check(self.lib.drkv_scorer_enable(self.h, -1.0))
    def scorer_update(self, seq: int, new_scores, stream=None) -> None:
        """ImportanceScorer::update: a device tensor on a device engine, a float32 array on one without."""
        if isinstance(new_scores, np.ndarray):
            arr = np.ascontiguousarray(new_scores, dtype=np.float32)
            check(self.lib.drkv_scorer_update(self.h, seq, arr.ctypes.data, len(arr), _stream(stream)))
        else:
            check(self.lib.drkv_scorer_update(self.h, seq, _ptr(new_scores), new_scores.numel(), _stream(stream)))
    def scorer_step(self, stream=None) -> None: check(self.lib.drkv_scorer_step(self.h, _stream(stream)))
    def scorer_sync(self, stream=None) -> None: check(self.lib.drkv_scorer_sync(self.h, _stream(stream)))
    def scorer_scores(self, seq: int) -> np.ndarray:
        out = np.empty(self.table_stride(), dtype=np.float32)
        n = check(self.lib.drkv_scorer_scores(self.h, seq, out.ctypes.data_as(C.POINTER(C.c_float)), len(out)))
        return out[:n]
    def attend_prefill_chunk(self, layer, seq, pos_start, m, q, out, scale, stream=None) -> None:
        check(self.lib.drkv_attend_prefill_chunk(self.h, layer, seq, pos_start, m, _ptr(q), _ptr(out), scale,
                                                 _stream(stream)))
    def attend_prefill_batch(self, layer, seqs, pos_start, m, qs, outs, scale, stream=None) -> None:
        n = len(seqs)
        i32 = lambda v: (C.c_int32 * n)(*[int(x) for x in v])
        ptrs = lambda v: (C.c_void_p * n)(*[_ptr(x) for x in v])
        check(self.lib.drkv_attend_prefill_batch(self.h, layer, n, i32(seqs), i32(pos_start), i32(m), ptrs(qs),
                                                 ptrs(outs), scale, _stream(stream)))

    def extract(self, seq, start_token, num_tokens, dst, stream=None) -> None:
        check(self.lib.drkv_seq_extract(self.h, seq, start_token, num_tokens, _ptr(dst), _stream(stream)))
    def inject(self, seq, start_token, num_tokens, src, stream=None) -> None:
        check(self.lib.drkv_seq_inject(self.h, seq, start_token, num_tokens, _ptr(src), _stream(stream)))

    # ---- cross-GPU exchange of split-KV partials by peer stores --------------------------------
    def exchange_create(self, world: int, rank: int) -> bytes:
        """Allocates this rank's exchange area; returns its 64-byte CUDA IPC handle."""
        buf = (C.c_uint8 * 64)()
        check(self.lib.drkv_exchange_create(self.h, world, rank, buf))
        return bytes(buf)
    def exchange_connect(self, handles: Sequence[bytes]) -> None:
        blob = b"".join(handles)
        arr = (C.c_uint8 * len(blob)).from_buffer_copy(blob)
        check(self.lib.drkv_exchange_connect(self.h, arr))
    def exchange_connect_local(self, areas: Sequence[int]) -> None:
        """Ranks in one process: every rank's exchange_area() as a device pointer."""
        arr = (C.c_void_p * len(areas))(*[int(a) for a in areas])
        check(self.lib.drkv_exchange_connect_local(self.h, arr))
    def exchange_area(self) -> int: return self.lib.drkv_exchange_area(self.h) or 0
    def exchange_set_wait_ms(self, ms: int) -> None: check(self.lib.drkv_exchange_set_wait_ms(self.h, ms))
    def exchange_destroy(self) -> None: check(self.lib.drkv_exchange_destroy(self.h))
    def attend_exchange(self, layer, seq, kv_begin, kv_end, q, out, scale, stream=None) -> None:
        check(self.lib.drkv_attend_exchange(self.h, layer, seq, kv_begin, kv_end, _ptr(q), _ptr(out), scale,
                                            _stream(stream)))

    def append_attend_exchange(self, layer, seq, kv_begin, kv_end, k_src, v_src, q, out, scale, stream=None) -> None:
        check(self.lib.drkv_append_attend_exchange(self.h, layer, seq, kv_begin, kv_end, _ptr(k_src), _ptr(v_src),
                                                   _ptr(q), _ptr(out), scale, _stream(stream)))

    def attend_partial(self, layer, seq, kv_begin, kv_end, q, part, scale, stream=None) -> None:
        check(self.lib.drkv_attend_partial(self.h, layer, seq, kv_begin, kv_end, _ptr(q), _ptr(part), scale,
                                           _stream(stream)))
    def combine_partials(self, n_parts, parts, out, stream=None) -> None:
        check(self.lib.drkv_combine_partials(self.h, n_parts, _ptr(parts), _ptr(out), _stream(stream)))
    def partial_floats(self) -> int: return self.lib.drkv_partial_floats(self.h)
