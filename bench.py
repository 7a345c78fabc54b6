#!/usr/bin/env python
"""Benchmark of the paged KV-cache decode step (fused RoPE + K/V append, then paged GQA decode
attention, every layer) on B200, through the C ABI of libdrkv.so.

    python bench.py --gpus N --steps K --warmup W            # this repository's CUDA path
    python bench.py --impl reference --gpus N --steps K ...  # the reference semantics on host cores

Default workload (`c2`): Qwen3-8B-shaped batched decode — 36 layers, 32 query / 8 KV heads,
head_dim 128, bf16, page 16, 64 sequences with context lengths uniform in [1024, 8192], block
tables a seeded shuffle of a pool of 1.1x the pages in use, Q/K/V ~ N(0,1), RoPE base 1e6.
With N > 1 every rank runs its own 64-sequence batch (independent sequences shard with no
collective); the reported value is the tokens all ranks decoded per second.

One JSON line is printed by rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: layers, hq, hkv, d, page, n_seq, ctx_lo, ctx_hi, theta
    "c2": dict(layers=36, hq=32, hkv=8, d=128, page=16, n_seq=64, lo=1024, hi=8192, theta=1e6,
               desc="Qwen3-8B-shaped batched decode: 36 layers, 32/8 heads, head_dim 128, bf16, page 16, "
                    "64 sequences, ctx U[1024,8192]"),
    "c5b": dict(layers=32, hq=32, hkv=8, d=128, page=16, n_seq=128, lo=4096, hi=4096, theta=1e6,
                desc="independent 4096-token sequences, 32 layers, 32/8 heads, 128 per GPU (1024 over 8 GPUs)"),
    # one long sequence split by KV page range over the ranks (strong scaling, NCCL all-gather per layer)
    "c5a": dict(layers=8, hq=64, hkv=8, d=128, page=64, seq_len=524288, theta=1e6,
                desc="one 524288-token sequence, 8 layers, 64/8 heads, head_dim 128, bf16, page 64, KV pages split "
                     "by contiguous range across GPUs, partial (m,l,o) all-gathered and LSE-combined"),
    # decode branches forked from one prompt: the shared pages are read once per 16 query rows of the family
    "c3": dict(layers=32, hq=32, hkv=8, d=128, page=16, n_seq=8, prefix=16384, lo=0, hi=2048, theta=1e6,
               desc="multi-branch prefix sharing: 32 layers, 32/8 heads, head_dim 128, bf16, page 16; 8 decode "
                    "branches forked from one 16384-token prefix, private tails U[0,2048], copy-on-write of the "
                    "shared tail page, shared-prefix decode plan per step"),
    # chunked prefill into the paged cache (tensor-core bound)
    "c4": dict(layers=28, hq=28, hkv=4, d=128, page=16, n_seq=4, seq_len=32768, chunk=2048, theta=1e6,
               desc="chunked prefill: 28 layers, 28/4 heads, head_dim 128, bf16, page 16, 4 sequences x 32768 "
                    "tokens in 2048-token chunks (RoPE + scatter, then causal attention over all prior pages)"),
    # single-stream decode at the reference's own attention shape (src/memoria/block_pool.h:34-40)
    "c2r": dict(layers=16, hq=24, hkv=4, d=256, page=256, n_seq=1, lo=32768, hi=32768, theta=1e7, rot=64,
                desc="single-stream decode at the reference model's attention shape: 16 layers, 24/4 heads, head_dim "
                     "256, bf16, page 256, partial rotary 64, one sequence of 32768 cached tokens"),
    # the same at the reference's own attention shape (src/memoria/block_pool.h:34-40): 24/4 heads, head_dim 256,
    # 256-key pages, partial rotary 64, one sequence, 16 full-attention layers
    "c4r": dict(layers=16, hq=24, hkv=4, d=256, page=256, n_seq=1, seq_len=32768, chunk=2048, theta=1e7, rot=64,
                desc="chunked prefill at the reference model's attention shape: 16 layers, 24/4 heads, head_dim 256, "
                     "bf16, page 256, partial rotary 64, 1 sequence x 32768 tokens in 2048-token chunks"),
}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


READ_STREAM_SRC = os.path.join(ROOT, "bench_read_stream.cu")
READ_STREAM_LIB = os.path.join(ROOT, "libbench_read_stream.so")


def build_read_stream(force: bool = False) -> str:
    """The read-only streaming probe (a measurement helper, kept out of libdrkv.so), built next to this file."""
    import shutil
    if force or not os.path.exists(READ_STREAM_LIB) or os.path.getmtime(READ_STREAM_LIB) < os.path.getmtime(READ_STREAM_SRC):
        nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
        subprocess.run([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-shared", "-Xcompiler",
                        "-fPIC,-fvisibility=hidden", READ_STREAM_SRC, "-o", READ_STREAM_LIB + ".tmp"], check=True)
        os.replace(READ_STREAM_LIB + ".tmp", READ_STREAM_LIB)
    return READ_STREAM_LIB


def read_stream_gbs(eng, stream):
    """Read-only streaming bandwidth of this GPU over the first 8 GiB of the engine's pool (the reference's own
    ceiling method, tools/probe_bw.cu): the second denominator beside the measured copy peak."""
    import ctypes as C
    pool = eng.pool_tensor()
    nbytes = min(pool.numel() * pool.element_size(), 8 << 30)
    if nbytes < (256 << 20):
        return None
    try:
        lib = C.CDLL(build_read_stream())
    except (OSError, subprocess.CalledProcessError):
        return None
    lib.bench_read_stream_gbs.argtypes = [C.c_void_p, C.c_size_t, C.c_int, C.c_void_p, C.POINTER(C.c_double)]
    out = C.c_double()
    rc = lib.bench_read_stream_gbs(pool.data_ptr(), nbytes, 10, stream.cuda_stream, C.byref(out))
    return float(out.value) if rc == 0 else None


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []
        self.t_begin = None

    def mark_begin(self):
        """Only samples that arrive from now on count: call right before the timed region.  (nvidia-smi takes
        longer to start than a short timed region lasts, so it is started well before.)"""
        self.t_begin = time.perf_counter()

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                 "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.perf_counter(), line.strip()))

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        t_end = time.perf_counter()
        for t, ln in self.lines:
            if self.t_begin is not None and not (self.t_begin <= t <= t_end):
                continue
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
            except ValueError:
                continue
            for n, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def make_lens(w, seed, n_seq):
    rng = np.random.default_rng(seed)
    return rng.integers(w["lo"], w["hi"] + 1, size=n_seq).astype(np.int32)


def algorithmic_bytes_per_layer(w, lens):
    """KV read once per sequence and KV head + append write + Q read / O write + table."""
    e = 2
    kv_tok = 2 * w["hkv"] * w["d"] * e
    n = len(lens)
    kv = float((lens.astype(np.int64) + 1).sum()) * kv_tok
    app = n * kv_tok
    qo = n * 2 * w["hq"] * w["d"] * e
    tab = 4 * float(sum((int(x) + 1 + w["page"] - 1) // w["page"] for x in lens))
    return kv, kv + app + qo + tab


# --------------------------------------------------------------------------------------------
# this repository's CUDA path
# --------------------------------------------------------------------------------------------
def run_ours(args):
    import torch
    import torch.distributed as dist

    from deusridet_b200 import PagedKVEngine, build
    build.build()

    world, rank, local = _dist_setup()
    dev = torch.device(f"cuda:{local}")

    w = dict(WORKLOADS[args.workload])
    if args.layers:
        w["layers"] = args.layers
    n_seq = args.seqs or w["n_seq"]
    L, hq, hkv, d, page = w["layers"], w["hq"], w["hkv"], w["d"], w["page"]
    lens = make_lens(w, 1234 + rank, n_seq)
    K, W = args.steps, args.warmup
    max_pages, width = c2_pool_pages(lens, page, K, W)
    eng = PagedKVEngine(num_layers=L, num_q_heads=hq, num_kv_heads=hkv, head_dim=d, page_size=page, dtype="bf16",
                        rotary_dim=w.get("rot", d), rope_theta=w["theta"], max_pages=max_pages, max_seqs=n_seq,
                        max_pages_per_seq=width, device=local)
    rng = np.random.default_rng(99 + rank)
    # seeded shuffle of the pool through the public pool calls
    pages = [eng.alloc_block() for _ in range(max_pages)]
    for p in rng.permutation(max_pages):
        eng.free_block(int(p))
    seqs = [eng.seq_create() for _ in range(n_seq)]
    for s, n in zip(seqs, lens):
        assert eng.ensure_blocks_for_range(s, 0, int(n) + 1)
        eng.set_seq_len(s, int(n))
    stream = torch.cuda.current_stream()
    eng.sync_block_table(stream)
    torch.manual_seed(7 + rank)
    pool = eng.pool_tensor().view(torch.bfloat16)
    step_elems = 1 << 28
    for off in range(0, pool.numel(), step_elems):     # N(0,1) cache contents, in slices to bound temporaries
        pool[off:off + step_elems].normal_()
    if args.chunk:
        eng.set_chunk_tokens(args.chunk)
    if args.scorer:
        eng.scorer_enable(0.95)                         # per-page attention mass + score update ride along

    d_rows = torch.tensor(seqs, dtype=torch.int32, device=dev)
    d_pos = torch.from_numpy(lens).to(dev)
    d_len = d_pos + 1
    q = torch.randn(L, n_seq, hq, d, device=dev, dtype=torch.bfloat16)
    kn = torch.randn(L, n_seq, hkv, d, device=dev, dtype=torch.bfloat16)
    vn = torch.randn(L, n_seq, hkv, d, device=dev, dtype=torch.bfloat16)
    out = torch.empty(L, n_seq, hq, d, device=dev, dtype=torch.bfloat16)
    scale = 1.0 / float(np.sqrt(d))
    max_kv = int(lens.max()) + 1

    fused = not args.separate_append            # one call per layer: the attention kernel appends the new token itself

    def layer_step(l, k_l, v_l, q_l, mk, stream):
        if fused:
            eng.append_attend_decode(l, n_seq, d_rows, d_len, mk, k_l, v_l, q_l, out[l], scale, stream)
        else:
            eng.append_rope(l, n_seq, d_rows, d_pos, k_l, v_l, stream)
            eng.attend_decode(l, n_seq, d_rows, d_len, mk, q_l, out[l], scale, stream)

    def device_step(stream=stream):
        for l in range(L):
            layer_step(l, kn[l], vn[l], q[l], max_kv, stream)
        if args.scorer:
            eng.scorer_step(stream)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing: `value` ----
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    for _ in range(W):
        device_step()
    barrier()
    eng.check_kernels()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    sampler.mark_begin()
    e0.record(stream)
    for _ in range(K):
        device_step()
    e1.record(stream)
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    ms = e0.elapsed_time(e1)
    t = torch.tensor([ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step = float(t.item()) / K
    launches = K * L * (2 if fused else 3)             # (append,) attention, combine per layer
    if args.scorer:
        launches += K * (L + 1)                        # + page mass per layer, score update per step

    # ---- the same step replayed from a CUDA graph (captured once; the launch shapes depend only on max_kv) ----
    graph = None
    if not args.no_graph:
        cg = torch.cuda.CUDAGraph()
        with torch.cuda.graph(cg):
            device_step(torch.cuda.current_stream())
        for _ in range(W):
            cg.replay()
        barrier()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        g0.record(stream)
        for _ in range(K):
            cg.replay()
        g1.record(stream)
        barrier()
        tg = torch.tensor([g0.elapsed_time(g1)], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(tg, op=dist.ReduceOp.MAX)
        gms = float(tg.item()) / K
        graph = {"ms_per_step": gms, "value": world * n_seq / (gms * 1e-3), "unit": "tokens/s",
                 "note": "the timed step replayed from one CUDA graph; `value` above is the stream-launched step (headline)"}
        del cg
        eng.check_kernels()

    # ---- dominant kernel: per-launch duration from events around each launch ----
    eng.kernel_timing(True)
    for _ in range(min(K, 3)):
        device_step()
    kms, kn_launch = eng.kernel_timing(False, read=True)
    kv_bytes, all_bytes = algorithmic_bytes_per_layer(w, lens)
    peak, peak_kind = peaks()
    read_peak = read_stream_gbs(eng, stream)
    achieved = kv_bytes / (kms / kn_launch * 1e-3) / 1e9 if kn_launch else None
    # DRAM bytes per algorithmic K/V byte of attend_decode_kernel, from an ncu capture of a 16-sequence case
    # (DRAM traffic grows in proportion to the keys processed: one gather per 16 keys, one partial per item)
    traffic_ratio = 1.025

    # ---- end to end through the public API with host buffers ----
    e2e = None
    if not args.no_e2e:
        # Host side: one pinned block per layer holding that layer's Q, K and V back to back, so that a
        # layer's inputs travel in one copy; the device mirrors it and the kernels get views.
        nq, nk = n_seq * hq * d, n_seq * hkv * d
        h_in = torch.randn(L, nq + 2 * nk, dtype=torch.bfloat16).pin_memory()
        d_in = torch.empty(L, nq + 2 * nk, dtype=torch.bfloat16, device=dev)
        eq = [d_in[l, :nq].view(n_seq, hq, d) for l in range(L)]
        ek = [d_in[l, nq:nq + nk].view(n_seq, hkv, d) for l in range(L)]
        evv = [d_in[l, nq + nk:].view(n_seq, hkv, d) for l in range(L)]
        h_out = torch.empty(out.shape, dtype=torch.bfloat16).pin_memory()
        h_pos = torch.empty(n_seq, dtype=torch.int32).pin_memory()
        cur = lens.copy()
        seq_arr = np.asarray(seqs, dtype=np.int32)

        # Copies ride their own streams (one per direction) and are chained to the layers by events:
        # layer l starts when its inputs have landed, its output leaves as soon as it is written.  The
        # copies are enqueued two layers ahead of the launches so that the first layer starts at once.
        s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
        ev_in = [torch.cuda.Event() for _ in range(L)]
        ev_out = [torch.cuda.Event() for _ in range(L)]
        ev_done = torch.cuda.Event()
        AHEAD = 2

        def send(l):
            with torch.cuda.stream(s_in):
                d_in[l].copy_(h_in[l], non_blocking=True)
                ev_in[l].record(s_in)

        def prepare_next():
            # Room for the next token of every sequence (copy-on-write aware), the changed table rows and the
            # positions: none of it depends on the token being sampled, so it is issued behind the running step
            # (stream order keeps it after that step's kernels) instead of in front of the next one.
            eng.reserve_batch(seq_arr, 1, stream)
            eng.sync_block_table(stream)
            h_pos.copy_(torch.from_numpy(cur))
            d_pos.copy_(h_pos, non_blocking=True)
            torch.add(d_pos, 1, out=d_len)

        def e2e_step():
            mk = int(cur.max()) + 1
            for l in range(min(AHEAD, L)):
                send(l)
            for l in range(L):
                if l + AHEAD < L:
                    send(l + AHEAD)
                stream.wait_event(ev_in[l])
                layer_step(l, ek[l], evv[l], eq[l], mk, stream)
                ev_out[l].record(stream)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(ev_out[l])
                    h_out[l].copy_(out[l], non_blocking=True)
            ev_done.record(s_out)
            cur[:] = cur + 1
            eng.advance_batch(seq_arr, 1)
            prepare_next()
            ev_done.synchronize()                       # the caller samples from the outputs before the next token
            stream.synchronize()

        prepare_next()
        for _ in range(W):
            e2e_step()
        barrier()
        import gc
        gc.collect()
        gc.disable()                      # a collection inside the timed steps would be charged to the path
        t0 = time.perf_counter()
        e0.record(stream)
        for _ in range(K):
            e2e_step()
        e1.record(stream)
        barrier()
        wall = (time.perf_counter() - t0) * 1e3
        gc.enable()
        t = torch.tensor([max(e0.elapsed_time(e1), wall)], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item()) / K
        h2d = h_in.numel() * 2 + n_seq * 4
        e2e = {"value": world * n_seq / (e2e_ms * 1e-3), "unit": "tokens/s", "ms_per_step": e2e_ms,
               "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(h_out.numel() * 2)}
    eng.check_kernels()
    stats = eng.stats()
    eng.close()

    result = None
    if rank == 0:
        result = {
            "metric": "decode tokens/s/GPU + achieved HBM GB/s (% of peak) for paged attn+append",
            "value": world * n_seq / (ms_step * 1e-3), "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": c2_config(args, w, lens, world, max_pages, kv_bytes),
            "tokens_per_s_per_gpu": n_seq / (ms_step * 1e-3),
            "hbm_gbs_step": all_bytes * L / (ms_step * 1e-3) / 1e9,
            "roofline": {"bound": "hbm", "kernel": "attend_decode_kernel", "achieved": achieved, "peak": peak,
                         "peak_kind": peak_kind, "unit": "GB/s", "frac": achieved / peak if achieved else None,
                         "traffic": kv_bytes * traffic_ratio, "bytes_per_launch": kv_bytes,
                         "read_stream_gbs": read_peak,
                         "frac_of_read_stream": achieved / read_peak if (achieved and read_peak) else None,
                         "us_per_launch": kms / kn_launch * 1e3 if kn_launch else None},
            "gpu_launches": launches, "clocks": clocks, "e2e": e2e,
            "cow_copies": stats["cow_copies"],
        }
        if graph is not None:
            result["cuda_graph"] = graph
    return result, (w, lens)


def _dist_setup():
    """One process per GPU: the process group is created once (first call) and torn down by main()."""
    import torch
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1 and not dist.is_initialized():
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
    torch.cuda.set_device(local)
    return world, rank, local


def _dist_teardown():
    import torch.distributed as dist
    if dist.is_available() and dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()


def run_c5a(args, collectives=None):
    """Single long sequence, KV pages split by contiguous range across the ranks.  Returns one result per
    collective in `collectives` ("peer": partials pushed to every rank by peer stores and merged in the same
    kernel; "nccl": all-gather of the partials + merge kernel), measured on one engine."""
    import torch
    import torch.distributed as dist

    from deusridet_b200 import PagedKVEngine, build, sharding
    build.build()
    world, rank, local = _dist_setup()
    dev = torch.device(f"cuda:{local}")
    collectives = list(collectives or [args.collective])
    w = dict(WORKLOADS["c5a"])
    if args.layers:
        w["layers"] = args.layers
    L, hq, hkv, d, page, S = w["layers"], w["hq"], w["hkv"], w["d"], w["page"], w["seq_len"]
    K, W = args.steps, args.warmup
    begin, end = sharding.key_range_for_rank(S, page, rank, world)
    my_pages = (end - begin + page - 1) // page
    width = (S + page - 1) // page + 2
    eng = PagedKVEngine(num_layers=L, num_q_heads=hq, num_kv_heads=hkv, head_dim=d, page_size=page, dtype="bf16",
                        rope_theta=w["theta"], max_pages=max(4, my_pages + 8), max_seqs=1, max_pages_per_seq=width,
                        device=local)
    rng = np.random.default_rng(5 + rank)
    pages = [eng.alloc_block() for _ in range(eng.max_blocks())]
    for p in rng.permutation(eng.max_blocks()):
        eng.free_block(int(p))
    s = eng.seq_create()
    assert eng.ensure_blocks_for_range(s, begin, end - begin)       # only this rank's page range is resident
    eng.set_seq_len(s, S)
    stream = torch.cuda.current_stream()
    eng.sync_block_table(stream)
    torch.manual_seed(11 + rank)
    pool = eng.pool_tensor().view(torch.bfloat16)
    for off in range(0, pool.numel(), 1 << 28):
        pool[off:off + (1 << 28)].normal_()
    if args.chunk:
        eng.set_chunk_tokens(args.chunk)
    torch.manual_seed(3)                                             # the query is replicated
    q = torch.randn(L, hq, d, device=dev, dtype=torch.bfloat16)
    kn = torch.randn(L, 1, hkv, d, device=dev, dtype=torch.bfloat16)
    vn = torch.randn(L, 1, hkv, d, device=dev, dtype=torch.bfloat16)
    out = torch.empty(L, hq, d, device=dev, dtype=torch.bfloat16)
    nf = eng.partial_floats()
    mine = torch.empty(nf, device=dev, dtype=torch.float32)
    gathered = torch.empty(world, nf, device=dev, dtype=torch.float32)
    d_rows = torch.tensor([s], dtype=torch.int32, device=dev)
    d_pos = torch.tensor([S - 1], dtype=torch.int32, device=dev)     # the token being decoded sits at S - 1
    owner = sharding.owner_of_position(S - 1, S, page, world)
    scale = 1.0 / float(np.sqrt(d))
    kv_rank = float(end - begin) * 2 * hkv * d * 2                   # this rank's K/V bytes per layer
    peak, peak_kind = peaks()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    results = {}
    for coll in collectives:
        use_peer = coll == "peer"
        if use_peer:
            # exchange areas: one CUDA IPC handle per rank, passed around once through the process group
            handle = torch.frombuffer(bytearray(eng.exchange_create(world, rank)), dtype=torch.uint8).to(dev)
            handles = torch.empty(world, 64, dtype=torch.uint8, device=dev)
            if world > 1:
                dist.all_gather_into_tensor(handles, handle)
            else:
                handles[0] = handle
            eng.exchange_connect([bytes(h.cpu().numpy().tobytes()) for h in handles])

        def step():
            for l in range(L):
                if use_peer and not args.separate_append:
                    # partial (the owner of the last page appends the new token inside it), peer stores, merge
                    mine_kv = (kn[l], vn[l]) if rank == owner else (None, None)
                    eng.append_attend_exchange(l, s, begin, end, mine_kv[0], mine_kv[1], q[l], out[l], scale, stream)
                    continue
                if rank == owner:
                    eng.append_rope(l, 1, d_rows, d_pos, kn[l], vn[l], stream)
                if use_peer:
                    eng.attend_exchange(l, s, begin, end, q[l], out[l], scale, stream)   # partial, peer stores, merge
                    continue
                eng.attend_partial(l, s, begin, end, q[l], mine, scale, stream)
                if world > 1:
                    dist.all_gather_into_tensor(gathered, mine)
                    eng.combine_partials(world, gathered, out[l], stream)
                else:
                    eng.combine_partials(1, mine, out[l], stream)

        sampler = ClockSampler(local)
        if rank == 0:
            sampler.start()
        for _ in range(W):
            step()
        barrier()
        eng.check_kernels()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        sampler.mark_begin()
        e0.record(stream)
        for _ in range(K):
            step()
        e1.record(stream)
        barrier()
        t = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        clocks = sampler.stop() if rank == 0 else None
        ms_step = float(t.item()) / K
        eng.kernel_timing(True)
        step()
        kms, kn_l = eng.kernel_timing(False, read=True)
        eng.check_kernels()
        if use_peer:
            barrier()                                                # nobody tears down while a peer may still push
            eng.exchange_destroy()
        achieved = kv_rank / (kms / kn_l * 1e-3) / 1e9
        results[coll] = {
            "metric": "decode tokens/s/GPU + achieved HBM GB/s (% of peak) for paged attn+append",
            "value": 1.0 / (ms_step * 1e-3), "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"c5a: {w['desc']}", "layers": L, "keys_per_gpu": end - begin,
                       "parallelism": f"kv-range-split x{world}",
                       "collective": ("partials pushed to every rank by peer stores as {value, call number} words, merged in the same "
                                      "kernel (no library collective)") if use_peer
                       else "nccl all_gather of Hq*(D+2) fp32 per layer",
                       "cold_cache": "inputs larger than L2: %.2f GB of K/V per layer per GPU" % (kv_rank / 1e9)},
            "hbm_gbs_step": world * kv_rank * L / (ms_step * 1e-3) / 1e9,
            "roofline": {"bound": "hbm", "kernel": "attend_decode_kernel", "achieved": achieved, "peak": peak,
                         "peak_kind": peak_kind, "unit": "GB/s", "frac": achieved / peak, "traffic": None,
                         "bytes_per_launch": kv_rank, "us_per_launch": kms / kn_l * 1e3},
            # rank 0's own kernels per layer: attention + merge (the merge is also the exchange with peer stores; with
            # NCCL a second merge follows the all-gather), plus the append kernel where the token is not fused in
            "gpu_launches": K * L * ((2 if use_peer else 3) +
                                     (1 if owner == 0 and (args.separate_append or not use_peer) else 0)),
            "clocks": clocks, "e2e": None}
    eng.close()
    return results if rank == 0 else None


def run_c5b(args):
    """The 1024-sequence workload: 1024 independent 4096-token sequences, data-parallel with no collective.  A rank
    owns 1024 / N of them and streams them through ONE resident pool in waves of at most 128 sequences (all 1024
    together would need 550 GB of K/V): a wave maps the pool's pages to its own sequences through the allocator
    (create, reserve, table sync), decodes one token per sequence on every layer, and releases them.  A step is
    one token for all 1024 sequences; tokens/s = 1024 / (slowest rank's time over its waves).  The K/V contents
    are synthetic and stay resident: no K/V bytes move between waves."""
    import torch
    import torch.distributed as dist

    from deusridet_b200 import PagedKVEngine, build
    build.build()
    world, rank, local = _dist_setup()
    dev = torch.device(f"cuda:{local}")
    w = dict(WORKLOADS["c5b"])
    if args.layers:
        w["layers"] = args.layers
    total = args.seqs or 1024
    L, hq, hkv, d, page, S = w["layers"], w["hq"], w["hkv"], w["d"], w["page"], w["lo"]
    K, W = args.steps, args.warmup
    mine = total // world + (1 if rank < total % world else 0)
    wave = min(128, max(mine, 1))
    n_waves = (mine + wave - 1) // wave
    pages_per_seq = (S + 1 + page - 1) // page
    max_pages = wave * pages_per_seq + 8
    eng = PagedKVEngine(num_layers=L, num_q_heads=hq, num_kv_heads=hkv, head_dim=d, page_size=page, dtype="bf16",
                        rope_theta=w["theta"], max_pages=max_pages, max_seqs=wave, max_pages_per_seq=pages_per_seq + 1,
                        device=local)
    rng = np.random.default_rng(31 + rank)
    pages = [eng.alloc_block() for _ in range(max_pages)]
    for p in rng.permutation(max_pages):
        eng.free_block(int(p))
    stream = torch.cuda.current_stream()
    torch.manual_seed(13 + rank)
    pool = eng.pool_tensor().view(torch.bfloat16)
    for off in range(0, pool.numel(), 1 << 28):
        pool[off:off + (1 << 28)].normal_()
    q = torch.randn(L, wave, hq, d, device=dev, dtype=torch.bfloat16)
    kn = torch.randn(L, wave, hkv, d, device=dev, dtype=torch.bfloat16)
    vn = torch.randn(L, wave, hkv, d, device=dev, dtype=torch.bfloat16)
    out = torch.empty(L, wave, hq, d, device=dev, dtype=torch.bfloat16)
    d_pos = torch.full((wave,), S, dtype=torch.int32, device=dev)
    d_len = d_pos + 1
    d_rows = torch.arange(wave, dtype=torch.int32, device=dev)       # rows are handed out lowest-free-first: 0..n-1
    scale = 1.0 / float(np.sqrt(d))

    def step():
        left = mine
        for _ in range(n_waves):
            n = min(wave, left)
            left -= n
            seqs = [eng.seq_create() for _ in range(n)]
            assert seqs == list(range(n))
            for s_ in seqs:
                assert eng.ensure_blocks_for_range(s_, 0, S + 1)
                eng.set_seq_len(s_, S)
            eng.sync_block_table(stream)
            for l in range(L):
                if args.separate_append:
                    eng.append_rope(l, n, d_rows, d_pos, kn[l], vn[l], stream)
                    eng.attend_decode(l, n, d_rows, d_len, S + 1, q[l], out[l], scale, stream)
                else:
                    eng.append_attend_decode(l, n, d_rows, d_len, S + 1, kn[l], vn[l], q[l], out[l], scale, stream)
            # pages go back to the allocator; the kernels of the next wave are ordered behind these on the stream
            for s_ in seqs:
                eng.seq_release(s_, discard=True)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    for _ in range(W):
        step()
    barrier()
    eng.check_kernels()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    sampler.mark_begin()
    e0.record(stream)
    for _ in range(K):
        step()
    e1.record(stream)
    barrier()
    t = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    clocks = sampler.stop() if rank == 0 else None
    ms_step = float(t.item()) / K
    eng.kernel_timing(True)
    step()
    kms, kn_l = eng.kernel_timing(False, read=True)
    eng.check_kernels()
    eng.close()
    if rank != 0:
        return None
    kv_launch = float(min(wave, mine)) * (S + 1) * 2 * hkv * d * 2      # K/V bytes one full-wave launch reads
    peak, peak_kind = peaks()
    # launches of partial waves are shorter; the per-launch figure is exact when every wave is full
    achieved = kv_launch / (kms / kn_l * 1e-3) / 1e9 if mine % wave == 0 else None
    return {"metric": "decode tokens/s/GPU + achieved HBM GB/s (% of peak) for paged attn+append",
            "value": total / (ms_step * 1e-3), "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"c5b: {total} independent {S}-token sequences, {L} layers, {hq}/{hkv} heads, head_dim "
                                   f"{d}, bf16, page {page}; {mine} per GPU in {n_waves} wave(s) of <= {wave} through one "
                                   f"resident pool (allocator re-maps the pages per wave; K/V contents synthetic and "
                                   f"resident); one step = one token for all {total} sequences",
                       "layers": L, "seqs_total": total, "seqs_per_gpu": mine, "waves_per_gpu": n_waves,
                       "parallelism": f"dp{world}, no collective",
                       "cold_cache": "inputs larger than L2: %.2f GB of K/V per layer per wave" % (kv_launch / 1e9)},
            "tokens_per_s_per_gpu": total / world / (ms_step * 1e-3),
            "hbm_gbs_step": None if achieved is None else float(mine) * (S + 1) * 2 * hkv * d * 2 * L / (ms_step * 1e-3) / 1e9,
            "roofline": {"bound": "hbm", "kernel": "attend_decode_kernel", "achieved": achieved, "peak": peak,
                         "peak_kind": peak_kind, "unit": "GB/s", "frac": achieved / peak if achieved else None,
                         "traffic": None, "bytes_per_launch": kv_launch, "us_per_launch": kms / kn_l * 1e3},
            "gpu_launches": K * n_waves * L * (3 if args.separate_append else 2), "clocks": clocks, "e2e": None}


def run_c4(args, name="c4"):
    """Chunked prefill of the workload's sequences into the paged cache (one GPU)."""
    import torch

    from deusridet_b200 import PagedKVEngine, build
    build.build()
    world, rank, local = _dist_setup()
    dev = torch.device(f"cuda:{local}")
    w = dict(WORKLOADS[name])
    if args.layers:
        w["layers"] = args.layers
    n_seq = args.seqs or w["n_seq"]
    L, hq, hkv, d, page, S, C = w["layers"], w["hq"], w["hkv"], w["d"], w["page"], w["seq_len"], w["chunk"]
    pages_per_seq = S // page
    eng = PagedKVEngine(num_layers=L, num_q_heads=hq, num_kv_heads=hkv, head_dim=d, page_size=page, dtype="bf16",
                        rotary_dim=w.get("rot", d), rope_theta=w["theta"], max_pages=n_seq * pages_per_seq + 16, max_seqs=n_seq,
                        max_pages_per_seq=pages_per_seq + 1, device=local)
    rng = np.random.default_rng(17 + rank)
    pages = [eng.alloc_block() for _ in range(eng.max_blocks())]
    for p in rng.permutation(eng.max_blocks()):
        eng.free_block(int(p))
    stream = torch.cuda.current_stream()
    torch.manual_seed(23 + rank)
    q = torch.randn(C, hq, d, device=dev, dtype=torch.bfloat16)
    kn = torch.randn(C, hkv, d, device=dev, dtype=torch.bfloat16)
    vn = torch.randn(C, hkv, d, device=dev, dtype=torch.bfloat16)
    out = torch.empty(C, hq, d, device=dev, dtype=torch.bfloat16)
    scale = 1.0 / float(np.sqrt(d))

    def full_prefill():
        seqs = [eng.seq_create() for _ in range(n_seq)]
        for pos in range(0, S, C):
            for s in seqs:
                assert eng.ensure_blocks_for_range(s, pos, C)       # C / page new pages per sequence and chunk
            eng.sync_block_table(stream)
            for l in range(L):
                for s in seqs:
                    eng.append_rope_chunk(l, s, pos, C, kn, vn, stream)
                eng.attend_prefill_batch(l, seqs, [pos] * n_seq, [C] * n_seq, [q] * n_seq, [out] * n_seq, scale, stream)
            for s in seqs:
                eng.set_seq_len(s, pos + C)
        return seqs

    def release(seqs):
        torch.cuda.synchronize()
        for s in seqs:
            eng.seq_release(s, discard=True)

    W = max(1, args.warmup)
    for _ in range(W):
        release(full_prefill())
    eng.check_kernels()
    sampler = ClockSampler(local)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    K = max(1, min(args.steps, 3))
    e0.record(stream)
    last = None
    for _ in range(K):
        if last is not None:
            release(last)
        last = full_prefill()
    e1.record(stream)
    torch.cuda.synchronize()
    clocks = sampler.stop()
    ms = e0.elapsed_time(e1) / K
    eng.check_kernels()
    eng.close()
    flop = 4.0 * hq * d * (S * (S + 1) / 2.0) * L * n_seq          # QK^T and PV over the causal pairs
    tfs = flop / (ms * 1e-3) / 1e12
    peak = 1590.0
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    peak_kind = "fallback"
    if os.path.exists(path):
        with open(path) as f:
            peak = float(json.load(f)["bf16_tflops_sustained"])
        peak_kind = "measured (sustained)"
    return {"metric": "prefill tokens/s (chunked prefill into the paged cache) + tensor TFLOP/s",
            "value": n_seq * S / (ms * 1e-3), "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W,
            "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic", "config": {"workload": f"{name}: {w['desc']}", "layers": L, "seqs": n_seq},
            "roofline": {"bound": "tensor", "kernel": "attend_prefill_kernel (incl. append)", "achieved": tfs, "peak": peak,
                         "peak_kind": peak_kind, "unit": "TFLOP/s", "frac": tfs / peak, "traffic": None},
            "gpu_launches": K * n_seq * (S // C) * L * 2, "clocks": clocks, "e2e": None}


def run_c3(args):
    """Decode steps over branches forked from one prompt (one GPU): bookkeeping (reserve with copy-on-write,
    table sync, shared-prefix plan) + append + planned attention; the per-sequence pass is timed beside it."""
    import torch

    from deusridet_b200 import PagedKVEngine, build
    build.build()
    world, rank, local = _dist_setup()
    dev = torch.device(f"cuda:{local}")
    w = dict(WORKLOADS["c3"])
    if args.layers:
        w["layers"] = args.layers
    n_seq = args.seqs or w["n_seq"]
    L, hq, hkv, d, page, prefix = w["layers"], w["hq"], w["hkv"], w["d"], w["page"], w["prefix"]
    K, W = args.steps, args.warmup
    rng = np.random.default_rng(77)
    private = rng.integers(w["lo"], w["hi"] + 1, size=n_seq).astype(np.int64)
    room = 3 * (K + W) + 16
    max_pages = (prefix + page - 1) // page + int(sum((int(x) + room + 2 * page - 1) // page for x in private)) + 8
    width = (prefix + int(private.max()) + room) // page + 2
    eng = PagedKVEngine(num_layers=L, num_q_heads=hq, num_kv_heads=hkv, head_dim=d, page_size=page, dtype="bf16",
                        rope_theta=w["theta"], max_pages=max_pages, max_seqs=n_seq, max_pages_per_seq=width,
                        device=local)
    pages = [eng.alloc_block() for _ in range(max_pages)]
    for p in rng.permutation(max_pages):
        eng.free_block(int(p))
    root = eng.seq_create()
    eng.reserve(root, prefix - 5)                          # the shared tail page is partial: forces copy-on-write
    eng.set_seq_len(root, prefix - 5)
    seqs = [root] + [eng.seq_fork(root) for _ in range(n_seq - 1)]
    stream = torch.cuda.current_stream()
    for s_, x in zip(seqs, private):
        eng.reserve(s_, int(x) + 5, stream)
        eng.set_seq_len(s_, prefix + int(x))
    cur = (prefix + private).astype(np.int32)
    eng.sync_block_table(stream)
    torch.manual_seed(3)
    eng.pool_tensor().view(torch.bfloat16).normal_()
    if args.chunk:
        eng.set_chunk_tokens(args.chunk)
    seq_arr = np.asarray(seqs, dtype=np.int32)
    d_rows = torch.tensor(seqs, dtype=torch.int32, device=dev)
    d_pos = torch.from_numpy(cur.copy()).to(dev)
    d_len = d_pos + 1
    q = torch.randn(L, n_seq, hq, d, device=dev, dtype=torch.bfloat16)
    kn = torch.randn(L, n_seq, hkv, d, device=dev, dtype=torch.bfloat16)
    vn = torch.randn(L, n_seq, hkv, d, device=dev, dtype=torch.bfloat16)
    out = torch.empty(L, n_seq, hq, d, device=dev, dtype=torch.bfloat16)
    scale = 1.0 / float(np.sqrt(d))
    eng.reserve_batch(seq_arr, 1, stream)
    eng.sync_block_table(stream)
    info = eng.plan_decode(seqs, (cur + 1).tolist(), stream)
    max_kv = int(cur.max()) + 1

    fused = not args.separate_append          # the new token is appended by the attention kernel's own item

    def planned_step():
        for l in range(L):
            if fused:
                eng.append_attend_decode_planned(l, kn[l], vn[l], q[l], out[l], scale, stream)
            else:
                eng.append_rope(l, n_seq, d_rows, d_pos, kn[l], vn[l], stream)
                eng.attend_decode_planned(l, q[l], out[l], scale, stream)

    def plain_step():
        for l in range(L):
            if fused:
                eng.append_attend_decode(l, n_seq, d_rows, d_len, max_kv, kn[l], vn[l], q[l], out[l], scale, stream)
            else:
                eng.append_rope(l, n_seq, d_rows, d_pos, kn[l], vn[l], stream)
                eng.attend_decode(l, n_seq, d_rows, d_len, max_kv, q[l], out[l], scale, stream)

    def timed(fn):
        for _ in range(W):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(K):
            fn()
        e1.record(stream)
        torch.cuda.synchronize()
        eng.kernel_timing(True)
        fn()
        kms, kl = eng.kernel_timing(False, read=True)
        return e0.elapsed_time(e1) / K, kms / kl * 1e3

    plain_ms, plain_us = timed(plain_step)
    sampler = ClockSampler(local)
    sampler.start()
    plan_ms, plan_us = timed(planned_step)
    clocks = sampler.stop()
    eng.check_kernels()

    # ---- end to end: host bookkeeping + plan + H2D of the step's Q/K/V + D2H of the outputs ----
    nq, nk = n_seq * hq * d, n_seq * hkv * d
    h_in = torch.randn(L, nq + 2 * nk, dtype=torch.bfloat16).pin_memory()
    d_in = torch.empty(L, nq + 2 * nk, dtype=torch.bfloat16, device=dev)
    h_out = torch.empty(out.shape, dtype=torch.bfloat16).pin_memory()
    h_pos = torch.empty(n_seq, dtype=torch.int32).pin_memory()

    def prepare_next():
        # room for every branch's next token (copy-on-write of a shared tail page), changed table rows, the plan
        # and the positions: independent of the token being sampled, so issued behind the running step
        eng.reserve_batch(seq_arr, 1, stream)
        eng.sync_block_table(stream)
        eng.plan_decode(seqs, (cur + 1).tolist(), stream)
        h_pos.copy_(torch.from_numpy(cur))
        d_pos.copy_(h_pos, non_blocking=True)

    eq = [d_in[l, :nq].view(n_seq, hq, d) for l in range(L)]                 # views made once, not per step
    ek = [d_in[l, nq:nq + nk].view(n_seq, hkv, d) for l in range(L)]
    ev = [d_in[l, nq + nk:].view(n_seq, hkv, d) for l in range(L)]
    eo = [out[l] for l in range(L)]

    def e2e_step():
        d_in.copy_(h_in, non_blocking=True)
        for l in range(L):
            if fused:
                eng.append_attend_decode_planned(l, ek[l], ev[l], eq[l], eo[l], scale, stream)
            else:
                eng.append_rope(l, n_seq, d_rows, d_pos, ek[l], ev[l], stream)
                eng.attend_decode_planned(l, eq[l], eo[l], scale, stream)
        h_out.copy_(out, non_blocking=True)
        cur[:] = cur + 1
        eng.advance_batch(seq_arr, 1)
        prepare_next()
        stream.synchronize()

    prepare_next()
    for _ in range(W):
        e2e_step()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(K):
        e2e_step()
    torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / K
    eng.check_kernels()
    stats = eng.stats()
    eng.close()
    kv_tok = 2 * hkv * d * 2
    unique = float(prefix + private.sum() + n_seq) * kv_tok      # every distinct key/value once
    peak, peak_kind = peaks()
    ach = unique / (plan_us * 1e-6) / 1e9
    return {"metric": "decode tokens/s over forked branches (append + shared-prefix paged attention)",
            "value": n_seq / (plan_ms * 1e-3), "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W,
            "ms_per_step": plan_ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"c3: {w['desc']}", "layers": L, "branches": n_seq, "plan": info,
                       "append": "fused into the attention kernel" if fused else "its own launch",
                       "cold_cache": "the shared prefix (%.0f MB per layer) fits L2; all layers together do not"
                                     % (prefix * kv_tok / 1e6)},
            "per_sequence_pass": {"ms_per_step": plain_ms, "tokens_per_s": n_seq / (plain_ms * 1e-3),
                                  "attend_us_per_launch": plain_us,
                                  "bytes_per_launch": float(info["keys_per_sequence_pass"]) * kv_tok},
            "roofline": {"bound": "hbm", "kernel": "attend_decode_kernel (planned)", "achieved": ach, "peak": peak,
                         "peak_kind": peak_kind, "unit": "GB/s", "frac": ach / peak, "traffic": None,
                         "bytes_per_launch": unique, "bytes_read_per_launch": float(info["keys_planned_pass"]) * kv_tok,
                         "us_per_launch": plan_us},
            "gpu_launches": K * L * (2 if fused else 3), "clocks": clocks,
            "e2e": {"value": n_seq / (e2e_ms * 1e-3), "unit": "tokens/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": int(h_in.numel() * 2 + n_seq * 4), "d2h_bytes_per_step": int(h_out.numel() * 2)},
            "cow_copies": stats["cow_copies"]}


def run_aux(args):
    """The path's other kernels on one GPU, each timed alone with CUDA events on its stream over buffers larger
    than L2: the chunk append (RoPE on K + scatter of K and V into pages), the decode append as its own launch, the
    flat <-> paged copies, and the copy-on-write page copy.  Bytes are the algorithmic ones (read + written)."""
    import torch

    from deusridet_b200 import PagedKVEngine, build
    build.build()
    world, rank, local = _dist_setup()
    dev = torch.device(f"cuda:{local}")
    w = dict(WORKLOADS["c2"])
    if args.layers:
        w["layers"] = args.layers
    L, hq, hkv, d, page = w["layers"], w["hq"], w["hkv"], w["d"], w["page"]
    T = 8192                                                  # tokens of the one long sequence
    n_fork = 32
    K, W = args.steps, max(args.warmup, 1)
    max_pages = T // page + 2 * n_fork + 72
    eng = PagedKVEngine(num_layers=L, num_q_heads=hq, num_kv_heads=hkv, head_dim=d, page_size=page, dtype="bf16",
                        rope_theta=w["theta"], max_pages=max_pages, max_seqs=n_fork + 70,
                        max_pages_per_seq=T // page + 4, device=local)
    stream = torch.cuda.current_stream()
    rng = np.random.default_rng(5)
    for p_ in [eng.alloc_block() for _ in range(max_pages)]:
        pass
    for p_ in rng.permutation(max_pages):
        eng.free_block(int(p_))
    s = eng.seq_create()
    assert eng.ensure_blocks_for_range(s, 0, T)
    eng.set_seq_len(s, T)
    eng.sync_block_table(stream)
    peak, peak_kind = peaks()
    out = {}

    def timed(fn, n_inner):
        for _ in range(W):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(K):
            fn()
        e1.record(stream)
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / (K * n_inner) * 1e3      # us per launch

    def entry(kernel, us, nbytes, note):
        gbs = nbytes / (us * 1e-6) / 1e9
        return {"kernel": kernel, "us_per_launch": us, "bytes_per_launch": nbytes, "achieved": gbs, "unit": "GB/s",
                "peak": peak, "peak_kind": peak_kind, "frac": gbs / peak, "note": note}

    # chunk append: T tokens of one layer per launch, a different layer (source and pages) every launch
    kn = torch.randn(L, T, hkv, d, device=dev, dtype=torch.bfloat16)
    vn = torch.randn(L, T, hkv, d, device=dev, dtype=torch.bfloat16)
    us = timed(lambda: [eng.append_rope_chunk(l, s, 0, T, kn[l], vn[l], stream) for l in range(L)], L)
    out["append_chunk"] = entry("append_rope_kernel", us, 2.0 * 2 * T * hkv * d * 2,
                                f"{T} tokens of one layer per launch: K and V rows read, rotated K and V written")
    # flat <-> paged copies of the whole sequence, all layers in one launch each
    flat = torch.empty(L, 2, T, hkv, d, device=dev, dtype=torch.bfloat16)
    us = timed(lambda: eng.extract(s, 0, T, flat, stream), 1)
    out["extract"] = entry("flat_paged_copy_kernel (pages -> flat)", us, 2.0 * flat.numel() * 2,
                           f"{T} tokens x {L} layers, K and V, one launch")
    us = timed(lambda: eng.inject(s, 0, T, flat, stream), 1)
    out["inject"] = entry("flat_paged_copy_kernel (flat -> pages)", us, 2.0 * flat.numel() * 2,
                          f"{T} tokens x {L} layers, K and V, one launch")
    del flat, kn, vn
    # decode append as its own launch: one token for each of 64 sequences
    seqs = [eng.seq_create() for _ in range(64)]
    for q_ in seqs:
        eng.reserve(q_, 1, stream)
    eng.sync_block_table(stream)
    d_rows = torch.tensor(seqs, dtype=torch.int32, device=dev)
    d_pos = torch.zeros(64, dtype=torch.int32, device=dev)
    k1 = torch.randn(L, 64, hkv, d, device=dev, dtype=torch.bfloat16)
    v1 = torch.randn(L, 64, hkv, d, device=dev, dtype=torch.bfloat16)
    us = timed(lambda: [eng.append_rope(l, 64, d_rows, d_pos, k1[l], v1[l], stream) for l in range(L)], L)
    out["append_decode"] = entry("append_rope_kernel", us, 2.0 * 2 * 64 * hkv * d * 2,
                                 "one token for each of 64 sequences: 0.5 MB, launches issued from Python one after the other: launch-bound")
    # copy-on-write of a shared partial tail page: all layers of one page per copy
    root = eng.seq_create()
    eng.reserve(root, page // 2, stream)
    eng.set_seq_len(root, page // 2)
    page_bytes = float(L * 2 * hkv * page * d * 2)
    cow_us = []
    for _ in range(W + K):
        kids = [eng.seq_fork(root) for _ in range(n_fork)]
        torch.cuda.synchronize()
        c0 = eng.stats()["cow_copies"]
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for k_ in kids:
            eng.reserve(k_, 1, stream)                        # the child's write position is in the shared page
        e1.record(stream)
        torch.cuda.synchronize()
        n_cow = eng.stats()["cow_copies"] - c0
        cow_us.append(e0.elapsed_time(e1) * 1e3 / max(n_cow, 1))
        for k_ in kids:
            eng.seq_release(k_, True)
    us = float(np.median(cow_us[W:]))
    out["cow_copy"] = entry("cow_copy_kernel", us, 2.0 * page_bytes / 2,
                            f"the filled half of one page across {L} layers per copy ({page_bytes / 2e6:.2f} MB), one "
                            "launch per forked sequence, issued from the host one after the other: launch-bound")
    eng.check_kernels()
    eng.close()
    if rank != 0:
        return None
    return {"metric": "achieved HBM GB/s of the secondary kernels (append, flat copies, copy-on-write)",
            "value": out["extract"]["achieved"], "unit": "GB/s", "n_gpus": 1, "steps": K, "warmup": W,
            "ms_per_step": out["extract"]["us_per_launch"] / 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"aux: {L} layers, {hq}/{hkv} heads, head_dim {d}, bf16, page {page}; one "
                                   f"{T}-token sequence, 64 one-token appends, {n_fork} forks of a half-full page",
                       "cold_cache": "buffers larger than L2 except where a note says otherwise"},
            "kernels": out, "gpu_launches": K * (2 * L + 2 + n_fork)}


def eng_bytes(max_pages, w):
    return max_pages * w["layers"] * 2 * w["hkv"] * w["page"] * w["d"] * 2


# --------------------------------------------------------------------------------------------
# the reference semantics on the host cores (CPU restatement in oracle/, OpenMP over (seq, head))
# --------------------------------------------------------------------------------------------
def cpu_pass(w, lens, steps, seed=5):
    """Whole decode steps of the workload on the host: for every layer, append then attention over all
    sequences.  One layer's pool is resident (1.4 GB for the default workload, far beyond the CPU caches) and
    is walked once per layer, so a step does the work and the memory traffic of all layers without holding
    50 GB of synthetic K/V in host memory.  Returns seconds per step (list) and the thread count."""
    from oracle import cbind as ob
    ob.lib()
    ob.use_all_cores()                                   # torchrun exports OMP_NUM_THREADS=1
    hq, hkv, d, page = w["hq"], w["hkv"], w["d"], w["page"]
    n_seq = len(lens)
    g = ob.geom(1, hq, hkv, d, page, ob.BF16, w.get("rot", d), w["theta"])
    rng = np.random.default_rng(seed)
    pages = [(int(n) + 1 + page - 1) // page for n in lens]
    max_pages = int(np.ceil(1.1 * sum(pages)))
    perm = rng.permutation(max_pages).astype(np.int32)
    width = max(pages)
    tables = np.full((n_seq, width), -1, dtype=np.int32)
    off = 0
    for i, n in enumerate(pages):
        tables[i, :n] = perm[off:off + n]
        off += n
    # finite bf16 patterns in +-[0.5, 1): the values do not change the work done
    pool = (rng.integers(0, 1 << 16, ob.pool_elems(g, max_pages), dtype=np.uint16) & np.uint16(0x807F)) | np.uint16(0x3F00)
    mk = lambda shape: ob.from_float(rng.standard_normal(shape, dtype=np.float32), ob.BF16)
    q, k, v = mk((n_seq, hq, d)), mk((n_seq, hkv, d)), mk((n_seq, hkv, d))
    out = np.zeros((n_seq, hq, d), dtype=np.uint16)
    rows = np.arange(n_seq, dtype=np.int32)
    scale = 1.0 / float(np.sqrt(d))
    times = []
    for _ in range(steps):
        t0 = time.perf_counter()
        for _layer in range(w["layers"]):
            for i in range(n_seq):
                ob.append(g, pool, max_pages, tables[i], 0, int(lens[i]), 1, k[i], v[i], rope=True)
            ob.attend_decode(g, pool, max_pages, tables, rows, lens + 1, 0, q, out, scale)
        times.append(time.perf_counter() - t0)
    return times, ob.num_threads()


CPU_SAMPLE = ("whole steps: every layer's append + attention over all {n} sequences ({L} passes over one resident "
              "layer-sized pool per step), median of {k} steps")


def cpu_baseline(w, lens):
    """About 10-30 s of host work: one step to size the sample, then up to 8 more; median."""
    times, threads = cpu_pass(w, lens, steps=1)
    more = int(min(8, max(2, 20.0 / max(times[0], 1e-3))))
    times, _ = cpu_pass(w, lens, steps=more)
    t_step = float(np.median(times))
    return {"value": len(lens) / t_step, "unit": "tokens/s", "cores": threads, "kind": "port",
            "ms_per_step": t_step * 1e3,
            "sample": CPU_SAMPLE.format(n=len(lens), L=w["layers"], k=len(times))}


def c2_config(args, w, lens, world, max_pages, kv_bytes):
    return {"workload": f"{args.workload}: {w['desc']}", "layers": w["layers"], "seqs_per_gpu": len(lens),
            "sum_ctx": int(lens.sum()), "page": w["page"], "pool_pages": max_pages,
            "pool_gb": round(eng_bytes(max_pages, w) / 1e9, 2), "parallelism": f"dp{world}",
            "importance_scorer": bool(args.scorer),
            "append": "own launch" if getattr(args, "separate_append", False) else "fused into the attention kernel",
            "cold_cache": "inputs larger than L2: %.2f GB of K/V per layer" % (kv_bytes / 1e9)}


def c2_pool_pages(lens, page, steps, warmup):
    room = max(64, steps + warmup + 8)                 # tokens each sequence may grow in the end-to-end pass
    pages_needed = int(sum((int(n) + room + page - 1) // page for n in lens))
    width = int(max((int(n) + room + page - 1) // page for n in lens)) + 1
    return int(np.ceil(1.1 * pages_needed)), width


def run_reference(args):
    """The reference arm: the reference's semantics for this path on the host cores (the CPU restatement in
    oracle/: the reference itself has no CPU implementation of its kernels), same workload, same metric."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return None
    w = dict(WORKLOADS[args.workload])
    if args.layers:
        w["layers"] = args.layers
    lens = make_lens(w, 1234, args.seqs or w["n_seq"])
    times, threads = cpu_pass(w, lens, steps=args.warmup + args.steps)
    times = times[args.warmup:]
    t_step = float(np.median(times))
    ms_step = t_step * 1e3
    val = len(lens) / t_step
    sample = CPU_SAMPLE.format(n=len(lens), L=w["layers"], k=len(times))
    max_pages, _ = c2_pool_pages(lens, w["page"], args.steps, args.warmup)
    kv_bytes, _ = algorithmic_bytes_per_layer(w, lens)
    return {
        "impl": "reference",
        "metric": "decode tokens/s/GPU + achieved HBM GB/s (% of peak) for paged attn+append",
        "value": val, "unit": "tokens/s", "n_gpus": int(os.environ.get("WORLD_SIZE", "1")), "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": c2_config(args, w, lens, int(os.environ.get("WORLD_SIZE", "1")), max_pages, kv_bytes),
        "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS) + ["aux"])
    ap.add_argument("--layers", type=int, default=0, help="override the layer count (profiling a small case)")
    ap.add_argument("--seqs", type=int, default=0, help="override sequences per GPU (profiling a small case)")
    ap.add_argument("--chunk", type=int, default=0, help="keys per split-KV chunk (0 = automatic)")
    ap.add_argument("--collective", default="peer", choices=["peer", "nccl"],
                    help="c5a: fused peer-store exchange + merge kernel, or NCCL all-gather + merge")
    ap.add_argument("--scorer", action="store_true", help="c2/c5b: also produce per-page attention mass and scores")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="c2: skip the CUDA-graph replay of the step")
    ap.add_argument("--separate-append", action="store_true",
                    help="append the new token with its own kernel launch instead of inside the attention kernel")
    ap.add_argument("--no-secondary", action="store_true",
                    help="c2: skip the secondary workloads (long split sequence, 1024 sequences, chunked prefill)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    if args.warmup < 3 and not (args.layers or args.seqs):
        args.warmup = 3
    if args.impl == "reference":
        if args.workload not in ("c2", "c5b"):
            args.workload = "c2"
        res = run_reference(args)
        if res is not None:
            print(json.dumps(res), flush=True)
        return
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    try:
        if args.workload == "c5a":
            res = run_c5a(args)
            if res is not None:
                print(json.dumps(res[args.collective]), flush=True)
            return
        if args.workload == "c5b":
            res = run_c5b(args)
            if res is not None:
                print(json.dumps(res), flush=True)
            return
        if args.workload in ("c4", "c4r"):
            res = run_c4(args, args.workload)
            if rank == 0:
                print(json.dumps(res), flush=True)
            return
        if args.workload == "c3":
            res = run_c3(args)
            if rank == 0:
                print(json.dumps(res), flush=True)
            return
        if args.workload == "aux":
            res = run_aux(args)
            if res is not None:
                print(json.dumps(res), flush=True)
            return
        res, (w, lens) = run_ours(args)
        secondary = {}
        if not args.no_secondary and not (args.layers or args.seqs or args.scorer):
            secondary = run_secondary(args, world)
        if res is not None:
            if world == 1 and not args.no_cpu_baseline:
                res["cpu_baseline"] = cpu_baseline(w, lens)
            if secondary:
                res["secondary"] = secondary
            print(json.dumps(res), flush=True)
    finally:
        _dist_teardown()


def run_secondary(args, world):
    """The other workloads of the benchmark list, each on a fresh engine after the headline leg has released its
    own, with fewer steps: the long sequence split by key range over the ranks (strong scaling; both the
    peer-store exchange and the NCCL all-gather), the 1024-sequence workload (strong scaling over the ranks, in
    waves through one pool), and at one GPU the chunked prefill (tensor-core bound).  Every rank takes part;
    rank 0 gets the results."""
    import copy
    import torch

    out = {}

    def leg(name, fn):
        torch.cuda.empty_cache()
        t0 = time.perf_counter()
        try:
            r = fn()
        except Exception as ex:   # a secondary leg never takes the headline line down with it
            r = {"error": f"{type(ex).__name__}: {ex}"}
        if isinstance(r, dict):
            r["leg_wall_s"] = round(time.perf_counter() - t0, 1)
        return r

    a = copy.copy(args)
    a.steps, a.warmup = min(args.steps, 10), 3
    r = leg("c5a", lambda: run_c5a(a, collectives=["peer", "nccl"]))
    if isinstance(r, dict):
        if "error" in r:
            out["c5a"] = r
        else:
            out["c5a_peer_store_exchange"], out["c5a_nccl_all_gather"] = r["peer"], r["nccl"]
    b = copy.copy(args)
    b.steps, b.warmup = min(args.steps, 5), 3
    r = leg("c5b", lambda: run_c5b(b))
    if r is not None:
        out["c5b_1024_sequences"] = r
    if world == 1:
        c = copy.copy(args)
        c.steps, c.warmup = 1, 1
        r = leg("c4", lambda: run_c4(c))
        if r is not None:
            out["c4_chunked_prefill"] = r
    return out


if __name__ == "__main__":
    main()
