#!/usr/bin/env python
"""Benchmark of the decode tick (slow-AR backbone + fast-AR loop + sampler).

    python bench.py --gpus N --steps K --warmup W [--impl reference]
    torchrun ... bench.py --gpus N ...          (one rank per GPU)

A step is one frame of one lockstep tick: `--batch` sessions (default 1) advance
one frame through the public C-ABI call s2p_model_batch_next_frame, i.e. host
staging, the pinned upload, the captured graph, the result download and the
stream sync — that is the end-to-end number (`e2e`).  `value` is the device time
of the same tick (CUDA events on the model's stream around the graph launch).
With N GPUs every rank runs an independent replica on its own sessions (the path
shards by session, there is no data-path collective): weak scaling.

The headline workload is the batch-1 all-INT4 configuration: 36 + 4 layers,
seeded random-init checkpoint (the real one is gated), 512-token uniform random
prompt, temperature 0.8 / top-p 0.8 with a fixed seed.  The same JSON line also
carries the two other parts of the metric: `lockstep_b32` (32 sessions per GPU
with 8192-token contexts, frames/s summed over the GPUs) and, with N >= 2 ranks,
`tp` (one batch-1 session sharded over the N GPUs, with a frame-by-frame check
against the single-GPU run of the same seed).  At N = 1 a `prefill` block times
s2p_session_prefill of the headline prompt through both routes of its linears
(dequantise + cuBLAS, the default; tensor cores from the quantised weights,
S2P_PREFILL_TC=1); the reference arm reports its own.
"""
import argparse
import ctypes as C
import importlib
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# weights one batch-1 frame touches (reference code truth: fast-AR stack 10x, fast head 9x, tied head 4097 rows)
WEIGHTS_PER_LAYER = 6144 * 2560 + 2560 * 4096 + 19456 * 2560 + 2560 * 9728


def algorithmic_bytes_per_frame(mode, n_slow=36):
    """Quantised weight bytes + scales streamed per frame (no KV, no activations)."""
    rows_per_layer = 6144 + 2560 + 19456 + 2560
    if mode == "int4":
        layer = WEIGHTS_PER_LAYER * 0.5625
        fast_head = 4096 * 2560 * 0.5625
    else:
        layer = WEIGHTS_PER_LAYER + 4 * rows_per_layer
        fast_head = 4096 * 2560 + 4 * 4096
    return n_slow * layer + 10 * 4 * layer + 9 * fast_head + 4097 * (2560 + 4)


# dram__bytes_read.sum + dram__bytes_write.sum of one k_tick_mega launch (36+4 layers, all-INT4, batch 1,
# ~540 cached positions) from an ncu capture; the capture is named beside the figure because the figure
# does not follow later kernel changes by itself
NCU_TRAFFIC_TICK_MEGA_INT4 = 4425153280
NCU_TRAFFIC_SOURCE = ("ncu capture of k_tick_mega (dram__bytes_read.sum + dram__bytes_write.sum, fourth of seven launches of "
                      "`bench.py --steps 4 --warmup 3`), kernel source as of commit 09a83d5 (two-group GEMV stages); "
                      "profiles/k_tick_mega_int4_b1.md holds the launch list")


def ncu_traffic_per_launch(mode, layers, batch, stats):
    if mode == "int4" and layers == 36 and batch == 1 and stats.last_tick_persistent:
        return NCU_TRAFFIC_TICK_MEGA_INT4
    return None


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            return json.load(f), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}, "fallback"


class ClockSampler(threading.Thread):
    """nvidia-smi clocks and throttle reasons while the timed region runs."""

    def __init__(self, gpu_index):
        super().__init__(daemon=True)
        self.rows, self.stop_flag, self.idx = [], False, gpu_index

    def run(self):
        q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
        while not self.stop_flag:
            try:
                out = subprocess.run(["nvidia-smi", "-i", str(self.idx), f"--query-gpu={q}", "--format=csv,noheader,nounits"],
                                     capture_output=True, text=True, timeout=5).stdout.strip()
                if out:
                    self.rows.append([c.strip() for c in out.split(",")])
            except Exception:
                pass
            time.sleep(0.2)

    def summary(self):
        sm = [float(r[0]) for r in self.rows if r and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) > 1 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({names[i] for r in self.rows for i in range(4) if len(r) > 2 + i and r[2 + i].lower().startswith("active")})
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(self.rows)}


def set_mode_env(mode):
    os.environ["S2P_INT8"] = "1"
    os.environ["S2P_QCACHE"] = "0"
    if mode == "int4":
        os.environ["S2P_INT4"] = "1"
        os.environ["S2P_INT4_ALL"] = "1"
    else:
        os.environ.pop("S2P_INT4", None)
        os.environ.pop("S2P_INT4_ALL", None)


def checkpoint_dir(n_slow):
    base = os.environ.get("S2P_BENCH_CKPT_DIR") or ("/dev/shm" if os.path.isdir("/dev/shm") else "/tmp")
    return os.path.join(base, f"s2p_synth_l{n_slow}")


class Engine:
    """Sessions of one model behind the C ABI (this library or the rebuilt reference)."""

    def __init__(self, lib, capi, ckpt, ctx_len, max_sessions):
        self.L, self.capi = lib, capi
        opts = capi.ModelOpts(capi.GEMM_INT8, ctx_len, max_sessions)
        self.m = C.c_void_p()
        capi.check(lib.s2p_model_load(ckpt.encode(), C.byref(opts), C.byref(self.m)), "s2p_model_load")
        self.sessions = []
        self.record = None  # a list: tick() appends the first session's ten codes of every frame

    def save_prefix(self, ids):
        """Prefill `ids` in a scratch session and return its KV blob (device memory) for kv_load."""
        import torch
        cfg = self.L.s2p_sampling_defaults()
        s = C.c_void_p()
        self.capi.check(self.L.s2p_session_create(self.m, C.byref(cfg), C.byref(s)), "s2p_session_create")
        for lo in range(0, len(ids), 2048):
            chunk = ids[lo:lo + 2048]
            self.capi.check(self.L.s2p_session_prefill(s, chunk.ctypes.data_as(C.c_void_p), None, len(chunk), None, 0), "s2p_session_prefill")
        blob = torch.empty(int(self.L.s2p_session_kv_bytes(self.m, len(ids))), dtype=torch.uint8, device="cuda")
        self.capi.check(self.L.s2p_session_kv_save(s, len(ids), C.c_void_p(blob.data_ptr())), "s2p_session_kv_save")
        self.L.s2p_session_destroy(s)
        return blob

    def open_sessions(self, prompts, temperature, top_p, seed, prefix=None):
        """prefix = (blob, n_tokens): every session starts from that saved KV prefix (kv_load) and prefills its own prompt after it."""
        for i, ids in enumerate(prompts):
            cfg = self.L.s2p_sampling_defaults()
            cfg.temperature, cfg.top_p, cfg.seed = temperature, top_p, seed + i
            s = C.c_void_p()
            self.capi.check(self.L.s2p_session_create(self.m, C.byref(cfg), C.byref(s)), "s2p_session_create")
            if prefix is not None:
                self.capi.check(self.L.s2p_session_kv_load(s, C.c_void_p(prefix[0].data_ptr()), prefix[1]), "s2p_session_kv_load")
            for lo in range(0, len(ids), 2048):  # prefill scratch holds 2048 rows per pass
                chunk = ids[lo:lo + 2048]
                self.capi.check(self.L.s2p_session_prefill(s, chunk.ctypes.data_as(C.c_void_p), None, len(chunk), None, 0),
                                "s2p_session_prefill")
            self.sessions.append(s)
        n = len(self.sessions)
        self.arr = (C.c_void_p * n)(*[s.value for s in self.sessions])
        self.codes = (C.c_int32 * (10 * n))()
        self.eos = (C.c_int * n)()

    def tick(self):
        self.capi.check(self.L.s2p_model_batch_next_frame(self.m, self.arr, len(self.sessions), self.codes, self.eos),
                        "s2p_model_batch_next_frame")
        if self.record is not None:
            self.record.append(tuple(self.codes[:10]))
        return any(self.eos)

    def close(self):
        for s in self.sessions:
            self.L.s2p_session_destroy(s)
        self.sessions = []
        self.L.s2p_model_free(self.m)


def stage_trace_summary(lib, model, sm_mhz):
    """Per stage kind: microseconds CTA 0 spent staging its input (incl. waiting for it), working, and in the
    stage-end synchronisation, from the SM-clock stamps of the last persistent tick."""
    import numpy as np
    cap = 1024
    stamps = np.zeros((cap, 16), dtype=np.uint64)
    kinds = np.zeros(cap, dtype=np.int32)
    n = C.c_int(0)
    rc = lib.s2p_b200_model_tick_trace(model, stamps.ctypes.data_as(C.c_void_p), kinds.ctypes.data_as(C.c_void_p), cap, C.byref(n))
    if rc != 0:
        return {"unavailable": int(rc)}
    t = stamps[:n.value].astype(np.int64)
    k = kinds[:n.value]
    names = {0: "frame_start", 1: "gemv", 2: "attention_backbone", 3: "attention_fast", 4: "sampler", 5: "frame_end"}
    us = 1.0 / sm_mhz
    out = {"total_us": round(float(t[-1, 3] - t[0, 0]) * us, 1)}
    for kind, name in names.items():
        sel = t[k == kind]
        if not len(sel):
            continue
        staged = np.where(sel[:, 1] > 0, sel[:, 1], sel[:, 0])
        out[name] = {"stages": int(len(sel)), "input_us": round(float((staged - sel[:, 0]).sum()) * us, 1),
                     "work_us": round(float((sel[:, 2] - staged).sum()) * us, 1),
                     "sync_us": round(float((sel[:, 3] - sel[:, 2]).sum()) * us, 1)}
    g = t[k == 1]
    if len(g):
        out["gemv_thread0"] = {"stream_wait_us": round(float(g[:, 4].sum()) * us, 1), "stream_us": round(float(g[:, 5].sum()) * us, 1),
                               "fold_wait_us": round(float(g[:, 6].sum()) * us, 1), "fold_us": round(float(g[:, 7].sum()) * us, 1)}
    return out


def host_threads():
    return len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)


def cpu_baseline(mode, frames=5, layers=36):
    """CPU port of the path (oracle/, exact reference order): whole frames of the full model - backbone
    step, tied head, sampler, ten fast-AR passes - through the oracle's frame function, on all host
    threads (set here, not inherited: a launcher may export OMP_NUM_THREADS=1).  The weights are synthetic
    codes of the right shapes and storage forms (the load-time quantisers are not part of the path)."""
    import numpy as np
    from oracle import oracle_api
    lib = oracle_api.load()
    threads = lib.s2po_set_threads(host_threads())
    int4 = int(mode == "int4")
    m = lib.s2po_model_new(2560, 32, 8, 9728, 155776, layers, 4, 4096, 10, 151678, 151645, 1, int4, int4, 1, 1, 256)
    lib.s2po_model_fill_synthetic(m, 12345)
    times, tries = [], 0
    while len(times) < frames and tries < 4:
        tries += 1
        s = lib.s2po_session_new(m, 0.8, 0.8, 1.1, 16, 42 + tries)
        ids = np.array([151700, 151701], dtype=np.int64)
        lib.s2po_prefill(s, oracle_api.ptr(ids), len(ids), None)
        codes = np.zeros(16, dtype=np.int32)
        lib.s2po_next_frame(s, oracle_api.ptr(codes), None, None)  # first frame: no backbone step, not timed
        while len(times) < frames:
            t0 = time.perf_counter()
            eos = lib.s2po_next_frame(s, oracle_api.ptr(codes), None, None)
            if eos:
                break
            times.append((time.perf_counter() - t0) * 1e3)
        lib.s2po_session_free(s)
    lib.s2po_model_free(m)
    return {"value": round(statistics.median(times), 2), "unit": "ms/frame", "cores": int(threads), "kind": "port",
            "sample": f"{len(times)} whole frames (median) of the {layers}+4-layer model through the CPU port's frame function "
                      f"({'all-INT4 g32' if int4 else 'INT8'} weights + INT8 KV, batch 1, 2-token context, OpenMP over output rows, "
                      f"{threads} threads set explicitly); synthetic codes of the real shapes stand in for quantised weights"}


def isolated_gemv_roofline(lib, torch, mode, peak_gbs):
    """Each GEMV shape of the tick timed alone with CUDA events, weights rotated through
    > L2-sized storage so every launch streams from HBM."""
    out = []
    G = 32
    for name, N, K in (("wqkv", 6144, 2560), ("wo", 2560, 4096), ("gate_up", 19456, 2560), ("w2", 2560, 9728)):
        per = N * K // 2 if mode == "int4" else N * K
        copies = max(3, int(400e6 // per) + 1)
        w = torch.randint(0, 255, (copies, per), dtype=torch.uint8, device="cuda")
        if mode == "int4":
            sc = torch.full((copies, N * (K // G)), 0.001, dtype=torch.float16, device="cuda")
        else:
            sc = torch.full((copies, N), 0.001, dtype=torch.float32, device="cuda")
        x = torch.randn(1, K, device="cuda").to(torch.bfloat16)
        y = torch.empty(1, N, dtype=torch.bfloat16, device="cuda")
        st = torch.cuda.Stream()
        reps = 3 * copies

        def launch(i):
            wp, sp = C.c_void_p(w[i % copies].data_ptr()), C.c_void_p(sc[i % copies].data_ptr())
            if mode == "int4":
                rc = lib.s2p_int4p_gemv(C.c_void_p(y.data_ptr()), C.c_void_p(x.data_ptr()), wp, sp, 1, N, K, G, C.c_void_p(st.cuda_stream))
            else:
                rc = lib.s2p_int8_gemv(C.c_void_p(y.data_ptr()), C.c_void_p(x.data_ptr()), wp, sp, 1, N, K, C.c_void_p(st.cuda_stream))
            assert rc == 0, rc
        torch.cuda.synchronize()
        for i in range(copies):  # warm-up (also sets the kernels' shared-memory attribute before capture)
            launch(i)
        torch.cuda.synchronize()
        # capture `reps` launches into one graph so that launch overhead does not gate the timing
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=st):
            for i in range(reps):
                launch(i)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        g.replay(); torch.cuda.synchronize()
        e0.record(); g.replay(); e1.record(); torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / reps
        byts = per + (N * (K // G) * 2 if mode == "int4" else N * 4)
        out.append({"kernel": f"k_gemv_stage[{name} {N}x{K} {mode}]", "us": round(us, 2), "bytes": byts,
                    "achieved_gbs": round(byts / us / 1e3, 1), "frac": round(byts / us / 1e3 / peak_gbs, 3)})
        del w, sc
    return out


def workload_text(args, seed_used):
    """The one description of the headline workload both arms print."""
    return (f"dual-AR decode, all-{args.mode.upper()} weights + INT8 KV, {args.layers}+4 layers, batch {args.batch} per GPU, " +
            (f"{args.prompt}-token prompt" if args.batch == 1 else f"prompts 256-2048 tokens after a shared {args.shared_prefix}-token KV prefix") +
            f", T=0.8 top-p=0.8 seed {seed_used}")


def config_block(args, seed_used, replicas, tp, ctx_len, eos_in_timed, arm):
    return {"workload": workload_text(args, seed_used), "replicas": replicas, "tensor_parallel": tp, "ctx_len": ctx_len,
            "l2": "weights per frame (4.4-7.8 GB) exceed the 126 MB L2: every frame streams from HBM",
            "eos_in_timed_region": bool(eos_in_timed), "arm": arm}


def tp_attach(lib, capi, eng, rank, world):
    """Exchange the arena handles of all ranks and attach (before any session exists)."""
    import torch
    import torch.distributed as dist
    handle = (C.c_ubyte * 64)()
    capi.check(lib.s2p_b200_model_tp_export(eng.m, handle), "s2p_b200_model_tp_export")
    mine = torch.tensor(list(handle), dtype=torch.uint8, device="cuda")
    allh = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(allh, mine)
    blob = (C.c_ubyte * (64 * world))(*[int(v) for t in allh for v in t.cpu().tolist()])
    capi.check(lib.s2p_b200_model_tp_attach(eng.m, rank, world, blob), "s2p_b200_model_tp_attach")
    dist.barrier()


def max_over_ranks(values, world, device="cuda"):
    """Element-wise maximum of a few floats over the ranks (a multi-GPU time is the slowest rank's)."""
    if world <= 1:
        return [float(v) for v in values]
    import torch
    import torch.distributed as dist
    t = torch.tensor([float(v) for v in values], device=device, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return [float(v) for v in t.tolist()]


def job_frames_per_s(world, sessions_per_gpu, ms_per_tick):
    """Whole-job throughput of `world` GPUs that each advance `sessions_per_gpu` sessions one frame per tick."""
    return world * sessions_per_gpu * 1e3 / ms_per_tick


def timed_ticks(eng, lib, capi, steps, world, device="cuda"):
    """`steps` ticks bracketed by a barrier and a device synchronisation on both sides: (wall ms per tick,
    device ms per tick (mean), per-tick device ms of this rank, EOS seen); wall and device are maxima over the ranks."""
    import torch
    on_gpu = device == "cuda"
    stats = capi.Stats()
    dev_ms = []
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
    if on_gpu:
        torch.cuda.synchronize()
    t0 = time.perf_counter()
    eos = False
    for _ in range(steps):
        eos = eng.tick() or eos
        lib.s2p_b200_model_stats(eng.m, C.byref(stats))
        dev_ms.append(stats.last_tick_device_ms)
    if on_gpu:
        torch.cuda.synchronize()
    wall = (time.perf_counter() - t0) * 1e3 / steps
    dev = sum(dev_ms) / len(dev_ms)
    wall, dev = max_over_ranks([wall, dev], world, device)
    return wall, dev, dev_ms, eos


def lockstep_block(args, lib, capi, synth, ckpt, rank, world, peak):
    """32 lockstep sessions per GPU with 8192-token contexts (data parallel over the ranks, no collective in the
    data path).  One 8192-token context is prefilled in 2048-row slices, saved, and loaded into every session, which
    then prefills a 16-token prompt of its own; every session attends over its own copy of the cache."""
    import numpy as np
    n, ctx_tokens, own = args.lockstep_sessions, args.lockstep_context, 16
    steps = max(3, min(args.steps, args.lockstep_steps))
    ctx_len = ((ctx_tokens + 1 + 3 + steps + 64 + 63) // 64) * 64
    eng = Engine(lib, capi, ckpt, ctx_len, n + 1)
    shared = ctx_tokens - own
    blob = eng.save_prefix(synth.random_prompt(shared, 4242 + rank))
    seed = args.seed + 7919 * rank
    for attempt in range(4):
        eng.open_sessions([synth.random_prompt(own, 1000 * rank + 50 * attempt + i) for i in range(n)], 0.8, 0.8, seed + 100 * attempt,
                          (blob, shared))
        hit = eng.tick()  # first frame: sampled from the prefill state, not captured
        for _ in range(3):
            hit = hit or eng.tick()
        if not hit:
            break
        for sess in eng.sessions:
            lib.s2p_session_destroy(sess)
        eng.sessions = []
    wall, dev, dev_ms, eos = timed_ticks(eng, lib, capi, steps, world)
    stats = capi.Stats()
    lib.s2p_b200_model_stats(eng.m, C.byref(stats))
    kv_tokens = n * (ctx_tokens + 4 + steps // 2)
    byts = algorithmic_bytes_per_frame(args.mode, args.layers) + stats.kv_bytes_per_token * kv_tokens
    out = {"sessions_per_gpu": n, "n_gpus": world, "context_tokens": ctx_tokens, "ctx_len": ctx_len, "steps": steps, "warmup": 3,
           "ms_per_tick": round(dev, 3), "ms_per_tick_e2e": round(wall, 3),
           "frames_per_s": round(job_frames_per_s(world, n, wall), 1), "frames_per_s_device": round(job_frames_per_s(world, n, dev), 1),
           "scaling": "weak", "eos_in_timed_region": bool(eos),
           "tick": {"kernels": int(stats.last_tick_kernels), "graph": int(stats.last_tick_graph)},
           "roofline": {"bound": "hbm", "bytes_per_tick": int(byts), "achieved": round(byts / (dev * 1e-3) / 1e9, 1), "peak": peak,
                        "unit": "GB/s", "frac": round(byts / (dev * 1e-3) / 1e9 / peak, 4),
                        "note": "weights once per tick + every session's INT8 KV at its context length, / device time of the tick"}}
    del blob
    eng.close()
    return out


def prefill_block(lib, capi, synth, ckpt, tokens, routes):
    """Wall time of s2p_session_prefill (it returns after a stream sync) for one `tokens`-token prompt, best of
    three fresh sessions per route.  routes: {"name": value of S2P_PREFILL_TC}."""
    import torch
    eng = Engine(lib, capi, ckpt, 4096, 1)
    ids = synth.random_prompt(tokens, 31)
    out = {"tokens": tokens, "unit": "ms", "note": "host wall time of the call, pageable ids in, KV cache and first-frame state out"}
    for name, tc in routes.items():
        os.environ["S2P_PREFILL_TC"] = tc
        best = None
        for _ in range(3):
            cfg = lib.s2p_sampling_defaults()
            sess = C.c_void_p()
            capi.check(lib.s2p_session_create(eng.m, C.byref(cfg), C.byref(sess)), "s2p_session_create")
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            capi.check(lib.s2p_session_prefill(sess, ids.ctypes.data_as(C.c_void_p), None, tokens, None, 0), "s2p_session_prefill")
            ms = (time.perf_counter() - t0) * 1e3
            lib.s2p_session_destroy(sess)
            best = ms if best is None else min(best, ms)
        out[name] = round(best, 2)
    os.environ["S2P_PREFILL_TC"] = "0"
    eng.close()
    return out


def tp_block(args, lib, capi, synth, ckpt, rank, world, seed_used, ref_frames, n1_value):
    """ONE batch-1 session sharded over the `world` GPUs (tensor parallel, strong scaling): same checkpoint,
    prompt, seed and call sequence as rank 0's single-GPU engine of the headline measurement, whose frames
    (`ref_frames`, rank 0 only) the sharded run must reproduce code for code."""
    import torch.distributed as dist
    ctx_len = max(4096, ((args.prompt + args.steps + args.warmup + 64 + 63) // 64) * 64)
    eng = Engine(lib, capi, ckpt, ctx_len, 1)
    tp_attach(lib, capi, eng, rank, world)
    eng.record = []
    eng.open_sessions([synth.random_prompt(args.prompt, 0)], 0.8, 0.8, seed_used)
    eng.tick()
    for _ in range(args.warmup):
        eng.tick()
    wall, dev, dev_ms, eos = timed_ticks(eng, lib, capi, args.steps, world)
    stats = capi.Stats()
    lib.s2p_b200_model_stats(eng.m, C.byref(stats))
    same = None
    if rank == 0 and ref_frames is not None:
        k = min(len(ref_frames), len(eng.record))
        same = f"{sum(1 for i in range(k) if ref_frames[i] == eng.record[i])}/{k}"
    dist.barrier()  # no rank frees its arena while a peer's kernel may still store into it
    eng.close()
    return {"world": world, "ms_per_frame": round(dev, 4), "ms_per_frame_e2e": round(wall, 4), "steps": args.steps,
            "speedup_vs_one_gpu": round(n1_value / dev, 3) if n1_value else None, "frames_identical": same,
            "persistent": int(stats.last_tick_persistent), "scaling": "strong", "eos_in_timed_region": bool(eos)}


def run_ours(args, rank, world):
    import numpy as np
    import torch
    capi = importlib.import_module("s2pro-native_b200.capi")
    synth = importlib.import_module("s2pro-native_b200.synth")
    set_mode_env(args.mode)
    if args.stage_trace:
        os.environ["S2P_TICK_TRACE"] = "1"
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    os.environ["S2P_DEVICE"] = str(local)
    ckpt = checkpoint_dir(args.layers)
    if local == 0:
        synth.write_checkpoint(ckpt, n_slow=args.layers, seed=1, generator="auto")
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
    lib = capi.load_library()
    longest = args.prompt if args.batch == 1 else 2048 + args.shared_prefix
    ctx_len = max(4096, ((longest + args.steps + args.warmup + 64 + 63) // 64) * 64)
    eng, seed_used = None, args.seed
    tp = bool(args.tp) and world > 1
    if tp and args.batch != 1:
        raise SystemExit("--tp shards the batch-1 tick")
    who = 0 if tp else rank  # tensor-parallel ranks must issue identical calls: same prompt, same seed
    for attempt in range(8):  # a sampled EOS would end a session early: move to the next seed
        eng = Engine(lib, capi, ckpt, ctx_len, max(args.batch, 1))
        if tp:
            tp_attach(lib, capi, eng, rank, world)
        eng.record = []
        rng = np.random.default_rng(1000 * who + attempt)
        lens = [args.prompt] * args.batch if args.batch == 1 else list(rng.integers(256, 2049, size=args.batch))
        prompts = [synth.random_prompt(int(n), 100 * who + i) for i, n in enumerate(lens)]
        prefix = None
        if args.batch > 1 and args.shared_prefix > 0:  # the shared voice-reference prefix: prefilled once, loaded into every session
            prefix = (eng.save_prefix(synth.random_prompt(args.shared_prefix, 4242)), args.shared_prefix)
        eng.open_sessions(prompts, 0.8, 0.8, seed_used + 7919 * who, prefix)
        hit = eng.tick()  # first frame samples from the prefill state (not graph-captured)
        for _ in range(args.warmup):
            hit = hit or eng.tick()
        if not hit:
            break
        if tp:
            dist.barrier()  # no rank frees its arena while a peer's kernel may still store into it
        eng.close()
        seed_used += 1
    stats = capi.Stats()
    sampler = ClockSampler(local)
    sampler.start()
    if args.profile_region:
        torch.cuda.profiler.start()
    step_wall, step_dev, dev_ms, eos_in_timed = timed_ticks(eng, lib, capi, args.steps, world)
    if args.profile_region:
        torch.cuda.profiler.stop()
    sampler.stop_flag = True
    sampler.join(timeout=2)
    lib.s2p_b200_model_stats(eng.m, C.byref(stats))
    if tp:
        dist.barrier()
    frames_rank0 = list(eng.record)
    peaks, peak_kind = measured_peaks()
    peak = float(peaks["hbm_gbs"])
    line = None
    if rank == 0:
        kv_tokens = sum(int(n) for n in lens) + args.batch * (1 + args.warmup + args.steps // 2)
        if args.batch > 1:
            kv_tokens += args.batch * args.shared_prefix
        algo = algorithmic_bytes_per_frame(args.mode, args.layers)
        traffic_model = algo + stats.kv_bytes_per_token * kv_tokens
        achieved = algo / (step_dev * 1e-3) / 1e9
        traffic = ncu_traffic_per_launch(args.mode, args.layers, args.batch, stats)
        line = {
            "metric": "decode ms/frame (B=%d)" % args.batch + (" TP=%d" % world if tp else ""), "value": round(step_dev, 4), "unit": "ms/frame",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(step_wall, 4),
            "higher_is_better": False, "scaling": "strong" if tp else "weak", "vs_baseline": None, "dtype": args.mode,
            "data": "synthetic (seeded random-init checkpoint, uniform random prompt)",
            "config": config_block(args, seed_used, 1 if tp else world, world if tp else 1, ctx_len, eos_in_timed,
                                   "this library (libs2pro_b200.so) through the C ABI"),
            "frames_per_s": round((1 if tp else world) * args.batch * 1e3 / step_wall, 1),
            "e2e": {"value": round(step_wall, 4), "unit": "ms/frame", "h2d_bytes_per_step": int(stats.upload_bytes),
                    "d2h_bytes_per_step": int(stats.download_bytes)},
            "gpu_launches": int(stats.last_tick_kernels) * args.steps,
            "tick": {"kernels": int(stats.last_tick_kernels), "persistent": int(stats.last_tick_persistent),
                     "fused": int(stats.last_tick_fused), "graph": int(stats.last_tick_graph),
                     "device_ms_p50": round(statistics.median(dev_ms), 4), "device_ms_p95": round(sorted(dev_ms)[int(0.95 * (len(dev_ms) - 1))], 4)},
            "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s", "frac": round(achieved / peak, 4),
                         "traffic": traffic, "traffic_source": NCU_TRAFFIC_SOURCE if traffic else None, "peak_source": peak_kind,
                         "kernel": "k_tick_mega (one launch = one frame)" if stats.last_tick_persistent else "whole tick (per-stage launches)",
                         "note": "algorithmic weight bytes per frame / device time of the tick, CUDA events on the model stream; "
                                 "roofline_kernels lists the stand-alone GEMV stage kernels of the non-persistent path",
                         "algorithmic_bytes_per_frame": int(algo), "modelled_bytes_with_kv": int(traffic_model)},
            "clocks": sampler.summary(),
        }
        if args.stage_trace:
            line["stage_trace"] = stage_trace_summary(lib, eng.m, float(line["clocks"].get("sm_mhz") or 1965.0))
    eng.close()
    # the other two parts of the metric, measured in the same run and carried by the same line
    if args.batch == 1 and not tp and not args.no_lockstep:
        blk = lockstep_block(args, lib, capi, synth, ckpt, rank, world, peak)
        if rank == 0:
            line["lockstep_b32"] = blk
    if args.batch == 1 and not tp and world > 1 and not args.no_tp_block:
        blk = tp_block(args, lib, capi, synth, ckpt, rank, world, seed_used, frames_rank0 if rank == 0 else None,
                       line["value"] if rank == 0 else None)
        if rank == 0:
            line["tp"] = blk
    if rank != 0:
        return None
    if world == 1:  # bounded host-side legs only where no other GPU waits for them
        if not args.no_kernel_roofline:
            line["roofline_kernels"] = isolated_gemv_roofline(lib, torch, args.mode, peak)
        if not args.no_prefill_block and args.batch == 1:
            line["prefill"] = prefill_block(lib, capi, synth, ckpt, args.prompt,
                                            {"ms_dequant_cublas": "0", "ms_tensor_core": "1"})
        if not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(args.mode, layers=args.layers)
    return line


def run_reference(args, rank, world):
    """The reference's own implementation of the path.  It has no CPU decode path; its
    CUDA path rebuilt unchanged for sm_100a (oracle/_ref) is timed through the same public
    API calls.  Without that build the CPU port of the hot loop stands in."""
    if rank != 0:
        return None
    ref_path = os.path.join(ROOT, "oracle", "_ref", "libs2pref.so" if args.layers == 36 else "libs2pref_l2.so")
    base = {"impl": "reference", "metric": f"decode ms/frame (B={args.batch})", "unit": "ms/frame", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "higher_is_better": False, "scaling": "weak", "vs_baseline": None, "dtype": args.mode,
            "data": "synthetic (seeded random-init checkpoint, uniform random prompt)"}
    try:
        import torch
        have_gpu = torch.cuda.is_available()
    except Exception:
        have_gpu = False
    if os.path.exists(ref_path) and have_gpu and args.batch <= 16:
        import numpy as np
        capi = importlib.import_module("s2pro-native_b200.capi")
        synth = importlib.import_module("s2pro-native_b200.synth")
        set_mode_env(args.mode)
        ckpt = checkpoint_dir(args.layers)
        synth.write_checkpoint(ckpt, n_slow=args.layers, seed=1, generator="auto")
        ref = C.CDLL(ref_path)
        capi.bind(ref, capi.PROTOTYPES, strict=False)
        seed_used = args.seed
        for attempt in range(8):
            eng = Engine(ref, capi, ckpt, 4096, max(args.batch, 1))
            rng = np.random.default_rng(attempt)
            lens = [args.prompt] * args.batch if args.batch == 1 else list(rng.integers(256, 2049, size=args.batch))
            eng.open_sessions([synth.random_prompt(int(n), i) for i, n in enumerate(lens)], 0.8, 0.8, seed_used)
            hit = eng.tick()
            for _ in range(args.warmup):
                hit = hit or eng.tick()
            if not hit:
                break
            eng.close()
            seed_used += 1
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            eng.tick()
        torch.cuda.synchronize()
        step = (time.perf_counter() - t0) * 1e3 / args.steps
        eng.close()
        if not args.no_prefill_block and args.batch == 1:
            base["prefill"] = prefill_block(ref, capi, synth, ckpt, args.prompt, {"ms_dequant_cublas": "0"})
        base.update({"value": round(step, 4), "ms_per_step": round(step, 4),
                     "config": config_block(args, seed_used, world, 1, 4096, False,
                                            "reference CUDA path rebuilt unchanged for sm_100a (oracle/_ref), same GPU, same API calls"),
                     "cpu_baseline": {"value": round(step, 4), "unit": "ms/frame", "cores": 1, "kind": "reference",
                                      "sample": "the reference has no CPU decode path; this is its CUDA path on the GPU, one host thread issuing"},
                     "e2e": {"value": round(step, 4), "unit": "ms/frame", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0,
                             "note": "the reference's tick uploads its own staging block and downloads its result block inside the "
                                     "timed call; their sizes are private to that library, so none is declared here"}})
        return base
    cb = cpu_baseline(args.mode, layers=args.layers)
    base.update({"value": round(cb["value"], 2), "ms_per_step": round(cb["value"], 2),
                 "config": config_block(args, args.seed, world, 1, 4096, False, "CPU port of the path (oracle/): the reference library is not built here"),
                 "cpu_baseline": cb,
                 "e2e": {"value": round(cb["value"], 2), "unit": "ms/frame", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}})
    return base


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--mode", default="int4", choices=["int4", "int8"])
    ap.add_argument("--batch", type=int, default=1, help="lockstep sessions per GPU")
    ap.add_argument("--prompt", type=int, default=512)
    ap.add_argument("--shared-prefix", type=int, default=1024,
                    help="batch > 1: tokens of a KV prefix prefilled once and loaded into every session (0 = none)")
    ap.add_argument("--layers", type=int, default=36)
    ap.add_argument("--seed", type=int, default=42)
    ap.add_argument("--profile-region", action="store_true",
                    help="bracket the timed steps with the CUDA profiler start/stop calls (for ncu --profile-from-start off)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-kernel-roofline", action="store_true")
    ap.add_argument("--stage-trace", action="store_true",
                    help="batch 1: add the persistent kernel's per-stage clock stamps (CTA 0) of the last frame, summed per stage kind")
    ap.add_argument("--no-lockstep", action="store_true", help="skip the lockstep_b32 block")
    ap.add_argument("--no-prefill-block", action="store_true", help="skip the prefill timing block (N = 1)")
    ap.add_argument("--no-tp-block", action="store_true", help="N > 1: skip the tp block")
    ap.add_argument("--lockstep-sessions", type=int, default=32)
    ap.add_argument("--lockstep-context", type=int, default=8192)
    ap.add_argument("--lockstep-steps", type=int, default=20)
    ap.add_argument("--tp", action="store_true",
                    help="with N > 1 ranks: one batch-1 session sharded over the N GPUs (tensor parallel) instead of N replicas")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1 and args.impl == "ours":
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
        if os.environ.get("NCCL_DEBUG", "").upper() == "VERSION":
            os.environ["NCCL_DEBUG"] = "WARN"  # the version banner goes to stdout, which carries the one JSON line
        dist.init_process_group("nccl")
    line = (run_ours if args.impl == "ours" else run_reference)(args, rank, world)
    if line is not None:
        print(json.dumps(line), flush=True)
    if world > 1 and args.impl == "ours":
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
