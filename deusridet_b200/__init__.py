"""B200-native paged KV-cache hot path of DeusRidet: page pool, block tables with fork /
copy-on-write / eviction, fused RoPE + K/V append and paged GQA attention, behind the C ABI
declared in include/drkv.h.  This package is the thin Python host used by the tests and the
benchmark; the product is libdrkv.so."""
from .capi import DrkvError, Geometry, Config, load_library  # noqa: F401
from .engine import PagedKVEngine  # noqa: F401
