"""CPU checker for the paged-KV kernels.  Test infrastructure only: imported by tests/,
the smoke check and the CPU-baseline legs of bench.py, never by the product package."""
