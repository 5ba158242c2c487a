"""Benchmark of the packed-contraction hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--dtype bf16] [--impl reference]

One "step" is one nk_dots_packed_<t> call over the metric's configuration: A (8192 x 8192) against a pre-packed B
(8192 x 8192), N(0,1) entries rounded to the storage type, seeded; B is packed outside the timed region exactly as the
reference's own benchmark does (bench/bench.hpp:245). Unit: gso/s = 2*M*N*K / seconds / 1e9 (bench/bench.hpp:257).

N = 1: K steps back to back, operands resident in HBM.

N > 1 (torchrun, one rank per GPU): STRONG scaling of the same problem. The 8192 rows of A are split into N contiguous
blocks, one per rank - the caller-side split the reference documents for its threads (README.md:209-212,
rust/matrix.rs:3016-3026). Packed B exists on rank 0 only when the timed region starts and reaches the other ranks INSIDE
it, once; then every rank runs its K steps. Two ways: rank 0 stores the blob once through the NVSwitch's multicast
mapping with the library's own kernels (multimem.st + a flag barrier: numkong_b200.sharding.SwitchBroadcast), or
ncclBroadcast; by default the set-up times both and the timed region uses the faster (the switch from four GPUs on, NCCL on
two; --broadcast switch / nccl force one), and NCCL is what runs where the GPUs have no multicast mapping. (--broadcast nccl
--broadcast-pieces 2 sends it in two column blocks and multiplies the first while the second is still on its way - the
packed rows of a column block are one contiguous byte range of the blob - which measured no faster: the broadcast kernel
and the persistent GEMM compete for the same SMs.)
The timed region is bracketed by a barrier and a device synchronize; the reported time is the maximum over ranks and
`value` = K * 2 * 8192^3 / that time.

Prints ONE JSON line (rank 0). `value` is measured with operands resident in HBM; `e2e` is the same metric through the
C ABI with HOST buffers (pinned): every step uploads this rank's rows of A and downloads its rows of C inside the timed
region. The default 1-GPU run adds: every other element type at 8192^3, library 8-bit GEMMs as peak probes, a sustained
leg of at least two seconds, the reference's CPU kernels on all host threads and on one, and the two search workloads
(sharded twins, which also run at every N > 1). `--impl reference` times the reference's own CPU kernels (compiled from
its sources into oracle/_ref/) on this host's cores, on a bounded sample of the same workload, without loading this
library.
"""
from __future__ import annotations

import argparse
import ctypes
import importlib.util
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

M = N = K = 8192
METRIC, UNIT = "dots_packed_gso_per_s", "gso/s"
STORE = {1: np.uint8, 2: np.int16}
SEEDS = {"bf16": 1, "f16": 1, "e4m3": 2, "e5m2": 2, "e2m3": 2, "e3m2": 2, "i8": 0, "u8": 0}
ELEMENT_BYTES = {"bf16": 2, "f16": 2, "e4m3": 1, "e5m2": 1, "e2m3": 1, "e3m2": 1, "i8": 1, "u8": 1}

# dram__bytes_read.sum + dram__bytes_write.sum of ONE launch of the dominant kernel, from one ncu capture of this command
# at the full size (1.043e9 read + 2.51e8 written; the algorithmic bytes A + packed B + C are 5.37e8). Keyed by
# (element type, rows of A per launch); other configurations report null.
NCU_DRAM_BYTES_PER_LAUNCH = {("bf16", 8192): 1_294_000_000}


def _synthetic():
    """The input generators, loaded from their file so that the reference arm does not import (and thereby load the shared
    library of) the package it is compared with."""
    spec = importlib.util.spec_from_file_location("_nkb_synthetic", os.path.join(ROOT, "numkong_b200", "synthetic.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"bf16_tflops": float(p["bf16_tflops"]), "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"])),
                "hbm_gbs": float(p["hbm_gbs"]), "source": "measured"}
    return {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


def gen_rows(rows: int, dtype: str, seed: int, first_row: int = 0) -> np.ndarray:
    """Rows [first_row, first_row + rows) of the K-column synthetic matrix of `seed`, in the storage type of `dtype`. The
    matrix is defined in blocks of 1024 rows (block b is drawn from seed * 100003 + 1024 b), so any rank can make its
    own rows without making the others; first_row must be a multiple of 1024 unless the request fits one block."""
    syn = _synthetic()
    out = []
    r = first_row
    while r < first_row + rows:
        block = r // 1024 * 1024
        full = syn.normal_matrix(1024, K, dtype, seed * 100003 + block)
        lo, hi = r - block, min(1024, first_row + rows - block)
        out.append(full[lo:hi])
        r = block + hi
    return np.concatenate(out) if len(out) > 1 else out[0]


class ClockSampler:
    """Samples SM clocks and throttle reasons while a timed region runs: NVML polled in-process (read-only queries, about
    a thousand per second - the timed region of the default run lasts some 15 ms), nvidia-smi as the fall-back."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.device_index, self.proc, self.lines = device_index, None, []
        self.nvml_samples, self.nvml_stop, self.nvml_thread, self.nvml_max = [], threading.Event(), None, None

    def _start_nvml(self) -> bool:
        try:
            import pynvml
            import torch
            pynvml.nvmlInit()
            try:
                uuid = str(torch.cuda.get_device_properties(self.device_index).uuid)
                handle = pynvml.nvmlDeviceGetHandleByUUID(uuid if uuid.startswith("GPU-") else "GPU-" + uuid)
            except Exception:
                handle = pynvml.nvmlDeviceGetHandleByIndex(self.device_index)
            self.nvml_max = float(pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM))
            reasons_fn = getattr(pynvml, "nvmlDeviceGetCurrentClocksEventReasons", None) or pynvml.nvmlDeviceGetCurrentClocksThrottleReasons
            pynvml.nvmlDeviceGetClockInfo(handle, pynvml.NVML_CLOCK_SM)

            def poll():
                while not self.nvml_stop.is_set():
                    try:
                        self.nvml_samples.append((time.time(), float(pynvml.nvmlDeviceGetClockInfo(handle, pynvml.NVML_CLOCK_SM)), int(reasons_fn(handle))))
                    except Exception:
                        break
                    time.sleep(0.0005)

            self.nvml_thread = threading.Thread(target=poll, daemon=True)
            self.nvml_thread.start()
            return True
        except Exception:
            return False

    def _stop_nvml(self, t0: float, t1: float):
        self.nvml_stop.set()
        self.nvml_thread.join(timeout=1.0)
        inside = [(c, r) for (t, c, r) in self.nvml_samples if t0 <= t <= t1] or [(c, r) for (_, c, r) in self.nvml_samples]
        sm = sorted(c for c, _ in inside)
        # NVML reason bits: 0x4 sw_power_cap, 0x8 hw_slowdown, 0x20 sw_thermal_slowdown, 0x40 hw_thermal_slowdown
        names = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown"}
        reasons = sorted({name for _, r in inside for bit, name in names.items() if r & bit})
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_min_mhz": sm[0] if sm else None, "sm_max_mhz": self.nvml_max,
                "reasons": reasons, "samples": len(sm), "source": "nvml polled inside the timed region"}

    def start(self):
        if self._start_nvml():
            return
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.device_index)], stdout=subprocess.PIPE, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def stop(self, t0: float, t1: float):
        if self.nvml_thread is not None:
            return self._stop_nvml(t0, t1)
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        rows = [l.split(", ") for (t, l) in self.lines if t0 - 0.05 <= t <= t1 + 0.15] or [l.split(", ") for (_, l) in self.lines]
        sm = sorted(float(r[1]) for r in rows if len(r) >= 9)
        reasons = set()
        for r in rows:
            if len(r) >= 9:
                for name, col in (("hw_slowdown", 5), ("hw_thermal_slowdown", 6), ("sw_thermal_slowdown", 7), ("sw_power_cap", 8)):
                    if r[col].strip().lower() == "active":
                        reasons.add(name)
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": float(rows[0][2]) if rows and len(rows[0]) >= 9 else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ---------------------------------------------------------------------------------------- reference arm
def _ref_library():
    import oracle
    return oracle.ref()


def _run_threads(ref, threads: int, work) -> float:
    """Seconds `work(t)` takes on `threads` host threads started together (each configures itself once, as the reference
    requires for AMX: include/numkong/capabilities.h:393-410)."""
    barrier = threading.Barrier(threads + 1)

    def body(t):
        ref.configure_thread()
        barrier.wait()
        work(t)
        barrier.wait()

    pool = [threading.Thread(target=body, args=(t,)) for t in range(threads)]
    for th in pool:
        th.start()
    barrier.wait()
    t0 = time.perf_counter()
    barrier.wait()
    dt = time.perf_counter() - t0
    for th in pool:
        th.join()
    return dt


def time_reference(dtype: str, steps: int, warmup: int, threads: int | None = None, seconds_per_step: float = 1.0):
    """Times the reference's dispatched CPU kernel on a bounded sample: `rows_per_step` rows of A against the full packed
    B, rows split evenly over `threads` host threads (default: all this process may run on)."""
    ref = _ref_library()
    if ref is None:
        return None
    import oracle
    threads = threads or max(1, len(os.sched_getaffinity(0)))
    b = gen_rows(N, dtype, SEEDS[dtype] + 1)
    t0 = time.perf_counter()
    blob = ref.pack(b, dtype)
    pack_s = time.perf_counter() - t0
    u64, vp = ctypes.c_uint64, ctypes.c_void_p
    fn = getattr(ref.lib, f"nk_dots_packed_{dtype}")
    fn.restype, fn.argtypes = None, [vp, vp, vp, u64, u64, u64, u64, u64]
    eb = b.itemsize

    def run(a: np.ndarray, c: np.ndarray) -> float:
        rows = a.shape[0]
        per = (rows + threads - 1) // threads

        def work(t):
            lo, hi = t * per, min(rows, (t + 1) * per)
            if hi > lo:
                fn(a[lo:hi].ctypes.data, blob.ctypes.data, c[lo:hi].ctypes.data, hi - lo, N, K, K * eb, N * 4)

        return _run_threads(ref, threads, work)

    # calibrate: about `seconds_per_step` of CPU work per step
    probe_rows = threads * 8
    a = gen_rows(probe_rows, dtype, SEEDS[dtype])
    c = np.zeros((probe_rows, N), dtype=oracle.out_dtype(dtype))
    run(a, c)
    dt = run(a, c)
    rows_per_step = max(threads, int(min(M, max(threads * 8, probe_rows * seconds_per_step / max(dt, 1e-4)))) // threads * threads)
    a = gen_rows(rows_per_step, dtype, SEEDS[dtype])
    c = np.zeros((rows_per_step, N), dtype=oracle.out_dtype(dtype))
    for _ in range(warmup):
        run(a, c)
    total = sum(run(a, c) for _ in range(steps))
    gso = 2.0 * rows_per_step * N * K * steps / total / 1e9
    return {"value": gso, "unit": UNIT, "cores": threads, "kind": "reference",
            "sample": f"{rows_per_step} of {M} rows of A x full packed B per step, {steps} steps, dispatched nk_dots_packed_{dtype}, pack {pack_s:.2f} s outside",
            "ms_per_step": total / steps * 1e3, "rows_per_step": rows_per_step}


def time_reference_search():
    """CPU legs for the two search workloads, on bounded twins: the reference's dispatched nk_angulars_packed_f16 (full
    distance matrix; it has no top-k) and nk_maxsim_packed_bf16 (one call per query/document pair), work split over all
    host threads. Throughput is work-normalised (2 x rows x columns x depth), so it compares with the GPU figures."""
    ref = _ref_library()
    if ref is None:
        return None
    syn = _synthetic()
    threads = max(1, len(os.sched_getaffinity(0)))
    u64, vp = ctypes.c_uint64, ctypes.c_void_p
    out = {}
    # nearest: 1024 queries x 20,000 corpus rows x 768, f16
    q_rows, c_rows, depth = 1024, 20000, 768
    q = syn.normal_matrix(q_rows, depth, "f16", 3, normalize=True)
    c = syn.normal_matrix(c_rows, depth, "f16", 4, normalize=True)
    blob = ref.pack(c, "f16")
    fn = getattr(ref.lib, "nk_angulars_packed_f16")
    fn.restype, fn.argtypes = None, [vp, vp, vp, u64, u64, u64, u64, u64]
    dist_m = np.zeros((q_rows, c_rows), dtype=np.float32)
    per = (q_rows + threads - 1) // threads

    def nearest_work(t):
        lo, hi = t * per, min(q_rows, (t + 1) * per)
        if hi > lo:
            fn(q[lo:hi].ctypes.data, blob.ctypes.data, dist_m[lo:hi].ctypes.data, hi - lo, c_rows, depth, depth * 2, c_rows * 4)

    _run_threads(ref, threads, nearest_work)
    dt = min(_run_threads(ref, threads, nearest_work) for _ in range(2))
    out["nearest"] = {"gso_per_s": 2.0 * q_rows * c_rows * depth / dt / 1e9, "cores": threads, "kind": "reference",
                      "sample": f"nk_angulars_packed_f16, {q_rows} queries x {c_rows} corpus rows x {depth}, distance matrix only (no selection)"}
    # MaxSim: 8 queries x 32 tokens against 256 documents of 64..300 tokens, bf16, depth 128
    rng = np.random.default_rng(5)
    counts = rng.integers(64, 301, size=256)
    queries = [ref.pack(syn.normal_matrix(32, 128, "bf16", 100 + i, normalize=True), "bf16", "maxsim") for i in range(8)]
    docs = [ref.pack(syn.normal_matrix(int(n), 128, "bf16", 200 + i, normalize=True), "bf16", "maxsim") for i, n in enumerate(counts)]
    ms = getattr(ref.lib, "nk_maxsim_packed_bf16")
    ms.restype, ms.argtypes = None, [vp, vp, u64, u64, u64, vp]
    scores = np.zeros((8, 256), dtype=np.float32)

    def maxsim_work(t):
        for j in range(t, 256, threads):
            for i in range(8):
                ms(queries[i].ctypes.data, docs[j].ctypes.data, 32, int(counts[j]), 128, scores[i, j:j + 1].ctypes.data)

    _run_threads(ref, threads, maxsim_work)
    dt = min(_run_threads(ref, threads, maxsim_work) for _ in range(2))
    out["maxsim"] = {"gso_per_s": 2.0 * 8 * 32 * float(counts.sum()) * 128 / dt / 1e9, "cores": threads, "kind": "reference",
                     "sample": f"nk_maxsim_packed_bf16, 8 queries x 32 tokens vs 256 documents ({int(counts.sum())} tokens), one call per pair"}
    return out


def reference_arm(args):
    """The reference's own CPU implementation of the step, on all host threads, one instance whatever --gpus says (rank 0
    runs it under torchrun, the other ranks leave at once)."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    dtype = args.dtype
    res = time_reference(dtype, args.steps, args.warmup)
    if res is None:
        print(json.dumps({"impl": "reference", "unavailable": "oracle/_ref/libnumkong.so has not been built (make -C oracle ref REF=<NumKong tree>)"}))
        return
    line = {
        "impl": "reference", "metric": METRIC, "value": res["value"], "unit": UNIT, "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": res["ms_per_step"], "higher_is_better": True, "scaling": "strong" if args.gpus > 1 else "weak",
        "vs_baseline": None, "dtype": dtype_arith(dtype), "data": "synthetic", "config": workload_config(dtype, args.gpus),
        "cpu_baseline": {k: res[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": res["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0, "sample_rows_per_step": res["rows_per_step"],
        "note": "one CPU instance on this host's cores; --gpus only selects the configuration it is compared with",
    }
    print(json.dumps(line))


# ---------------------------------------------------------------------------------------- our arm
def dtype_arith(dtype: str) -> str:
    return {"i8": "i32", "u8": "u32"}.get(dtype, "f32") + f" accumulate of {dtype}"


def workload_config(dtype: str, n_gpus: int):
    split = "all 8192 rows of A on one GPU" if n_gpus == 1 else \
        f"the 8192 rows of A split into {n_gpus} contiguous blocks of {M // n_gpus}, one per GPU; packed B broadcast from rank 0 inside the timed region"
    return {"workload": f"dots_packed {dtype} M=N=K=8192 (B pre-packed, N(0,1) rounded to {dtype}, seed {SEEDS[dtype]})",
            "global_rows_of_A": M, "rows_of_A_per_gpu": M // n_gpus, "width": N, "depth": K, "parallelism": split,
            "l2": "operands of a step (A block + packed B 128 MiB + C block) exceed the 126 MB L2; no explicit flush"}


def time_device_steps(nk, torch, ta, packed, out, dtype, steps):
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        nk.dots_packed(ta, packed, out=out, dtype=dtype)
    stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop) / 1e3


def library_peak_probes(torch, peaks):
    """Library 8-bit GEMMs at 8192^3 as PEAK PROBES for the 8-bit element types (this pool publishes a measured figure for
    bf16 only): torch._scaled_mm on e4m3 and torch._int_mm on i8, device-resident operands in this GPU's own memory, CUDA
    events, best of three rounds of ten. Not part of any timed region of this library."""
    def best_of(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        best = float("inf")
        for _ in range(3):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(10):
                fn()
            e1.record()
            torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1) / 10 / 1e3)
        return 2.0 * 8192 ** 3 / best / 1e12

    out = {"assumed_8bit_tflops": 2.0 * peaks["bf16_tflops"], "assumed_note": "2 x the measured cuBLAS bf16 burst"}
    try:
        a = torch.randn(8192, 8192, device="cuda").to(torch.float8_e4m3fn)
        b = torch.randn(8192, 8192, device="cuda").to(torch.float8_e4m3fn)
        one = torch.ones((), device="cuda", dtype=torch.float32)
        out["scaled_mm_e4m3_tflops"] = best_of(lambda: torch._scaled_mm(a, b.t(), scale_a=one, scale_b=one, out_dtype=torch.bfloat16))
        del a, b
    except Exception as e:  # a probe that this torch build does not offer is reported, not fatal
        out["scaled_mm_e4m3_error"] = str(e)[:200]
    try:
        a = torch.randint(-128, 128, (8192, 8192), device="cuda", dtype=torch.int8)
        b = torch.randint(-128, 128, (8192, 8192), device="cuda", dtype=torch.int8)
        out["int_mm_i8_tops"] = best_of(lambda: torch._int_mm(a, b.t()))
        del a, b
    except Exception as e:
        out["int_mm_i8_error"] = str(e)[:200]
    try:
        # f64 library GEMM at 4096^3: the denominator for the f32 -> f64 product, which runs on the FP64 CUDA cores
        a = torch.randn(4096, 4096, device="cuda", dtype=torch.float64)
        b = torch.randn(4096, 4096, device="cuda", dtype=torch.float64)
        fn = lambda: torch.matmul(a, b)
        for _ in range(2):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(3):
            fn()
        e1.record()
        torch.cuda.synchronize()
        out["matmul_f64_tflops"] = 2.0 * 4096 ** 3 * 3 / (e0.elapsed_time(e1) / 1e3) / 1e12
        del a, b
    except Exception as e:
        out["matmul_f64_error"] = str(e)[:200]
    torch.cuda.empty_cache()
    return out


def sustained_leg(nk, torch, ta, packed, out, dtype, peaks, device_index, seconds=2.5):
    """Back-to-back launches for at least `seconds`, NVML clocks sampled throughout: the figure to set beside the measured
    SUSTAINED cuBLAS rate (a 20-step burst runs at the full boost clock, a long run settles at the power cap)."""
    sampler = ClockSampler(device_index)
    sampler.start()
    time.sleep(0.2)
    torch.cuda.synchronize()
    wall0 = time.time()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    launches = 0
    while True:
        for _ in range(200):
            nk.dots_packed(ta, packed, out=out, dtype=dtype)
        launches += 200
        torch.cuda.synchronize()
        if time.time() - wall0 >= seconds:
            break
    stop.record()
    torch.cuda.synchronize()
    wall1 = time.time()
    elapsed = start.elapsed_time(stop) / 1e3
    clocks = sampler.stop(wall0, wall1)
    tflops = 2.0 * ta.shape[0] * N * K * launches / elapsed / 1e12
    ms = elapsed / launches * 1e3
    return {"value": tflops * 1e3, "unit": UNIT, "seconds": elapsed, "launches": launches, "ms_per_step": ms,
            "frac_of_sustained_peak": tflops / peaks["bf16_tflops_sustained"],
            "peak": peaks["bf16_tflops_sustained"], "peak_note": f"{peaks['source']} cuBLAS bf16, seconds-long loop under the power cap",
            "clocks": clocks, "ms_x_sm_mhz": ms * clocks["sm_mhz"] if clocks.get("sm_mhz") else None,
            "note": "host synchronises every 200 launches (a few microseconds of idle per 150 ms)"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--dtype", default="bf16")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-extras", action="store_true", help="skip everything but the headline measurement")
    ap.add_argument("--broadcast-pieces", type=int, default=1, choices=[1, 2],
                    help="N > 1: 1 = broadcast the packed matrix whole, then multiply (default); 2 = broadcast it in two column blocks "
                         "and multiply the first while the second is in flight (measured on two B200s: 0.73-0.77 ms for the first step "
                         "against 0.74-0.76 ms whole - the broadcast kernel and the persistent GEMM compete for SMs, so nothing is won)")
    ap.add_argument("--broadcast", default="auto", choices=["auto", "switch", "nccl"],
                    help="N > 1: how packed B reaches the ranks inside the timed region. switch = rank 0 stores it once through the "
                         "NVSwitch multicast mapping with the library's own kernels (numkong_b200.sharding.SwitchBroadcast); nccl = "
                         "ncclBroadcast; auto (default) = whichever of the two delivered the blob faster in the set-up (the switch "
                         "from four GPUs on, NCCL on two). Without a multicast mapping switch falls back to nccl and says so.")
    ap.add_argument("--rows", type=int, default=8192,
                    help="global rows of A; anything but 8192 is a reduced case for profiler captures, not the benchmark")
    args = ap.parse_args()
    global M
    M = args.rows
    args.warmup = max(args.warmup, 3) if M == 8192 else args.warmup
    if args.impl == "reference":
        reference_arm(args)
        return

    import torch
    import torch.distributed as dist
    import numkong_b200 as nk
    from numkong_b200 import sharding, workloads

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    dtype = args.dtype
    eb = ELEMENT_BYTES[dtype]
    compute = torch.cuda.current_stream()
    nk.set_stream(compute.cuda_stream)

    # ---- set-up (untimed): this rank's rows of A on the device; B packed on rank 0
    row0, row1 = sharding.row_shard(M, world, rank)
    rows = row1 - row0
    a_host = gen_rows(rows, dtype, SEEDS[dtype], first_row=row0)
    ta = torch.from_numpy(a_host.view(STORE[eb])).cuda()
    size = nk.PackedMatrix.packed_size(N, K, dtype)
    # `blob` is what every rank multiplies with. Through the switch it is this rank's copy of a symmetric buffer that rank 0's
    # multicast stores fill on all GPUs at once (rank 0's own copy included), and rank 0 packs into a buffer of its own.
    channel, switch_note = None, None
    if world > 1 and args.broadcast in ("switch", "auto"):
        # Every rank must take the same road: one that cannot map the buffer (or has no multicast address) sends all to NCCL.
        try:
            channel = sharding.SwitchBroadcast(size)
            usable = channel.available
        except Exception as exc:  # no symmetric memory in this build of torch, no fabric, ...
            usable, switch_note = False, f"{type(exc).__name__}: {exc}"[:200]
        agreed = torch.tensor([1.0 if usable else 0.0], device="cuda")
        dist.all_reduce(agreed, op=dist.ReduceOp.MIN)
        if agreed.item() == 0.0:
            channel = None
            switch_note = switch_note or "no multicast mapping on these GPUs"
    blob = channel.buffer[:size] if channel is not None else torch.zeros(size, dtype=torch.uint8, device="cuda")
    packed_on_sender = torch.zeros(size, dtype=torch.uint8, device="cuda") if (channel is not None and rank == 0) else blob
    if rank == 0:
        b_host = gen_rows(N, dtype, SEEDS[dtype] + 1)
        tb = torch.from_numpy(b_host.view(STORE[eb])).cuda()
        getattr(nk.lib, f"nk_dots_pack_{dtype}")(tb.data_ptr(), N, K, K * eb, packed_on_sender.data_ptr())
        nk.check("pack")
        del tb
    torch.cuda.synchronize()
    packed = nk.PackedMatrix(blob, dtype, N, K)
    out_dtype = torch.int32 if dtype in ("i8", "u8") else torch.float32
    out = torch.empty((rows, N), dtype=out_dtype, device="cuda")

    # The broadcast of the timed region: two column blocks, each one contiguous byte range of the blob (the first carries
    # the 128-byte header, the second the norms behind the payload). Packed rows come in blocks of 256.
    half_cols = N // 2 // 256 * 256
    depth_padded = (K * eb + 127) // 128 * 128
    cut = 128 + half_cols * depth_padded
    pieces = [(0, cut, 0, half_cols), (cut, size, half_cols, N - half_cols)]
    if args.broadcast_pieces == 1:
        pieces = [(0, size, 0, N)]
    comm = torch.cuda.Stream() if world > 1 else None

    def broadcast_and_first_step():
        """Through the switch: rank 0's multicast stores, a flag barrier, the first product. Over NCCL: rank 0 sends the packed
        matrix piece by piece on the communication stream; every rank multiplies a piece as soon as it has arrived while the
        next one is still in flight."""
        if use_switch:
            channel.send(packed_on_sender if rank == 0 else None, src=0, blocks=128)
            nk.dots_packed(ta, packed, out=out, dtype=dtype)
            return
        comm.wait_stream(compute)
        arrived = []
        with torch.cuda.stream(comm):
            for lo, hi, _, _ in pieces:
                dist.broadcast(blob[lo:hi], src=0)
                ev = torch.cuda.Event()
                ev.record(comm)
                arrived.append(ev)
        # The products of all pieces but the last leave 32 SMs to the broadcast kernel (NCCL runs 32 channels here), which
        # otherwise would not run before they end.
        nk.lib.nkb_set_sm_budget(116)
        for ev, (_, _, first, count) in zip(arrived[:-1], pieces[:-1]):
            compute.wait_event(ev)
            nk.dots_packed(ta, packed, out=out, dtype=dtype, columns=(first, count))
        nk.lib.nkb_set_sm_budget(0)
        compute.wait_event(arrived[-1])
        nk.dots_packed(ta, packed, out=out, dtype=dtype, columns=(pieces[-1][2], pieces[-1][3]))

    collective = None
    use_switch = channel is not None
    if world > 1:
        # untimed: B reaches every rank once so that the warm-up steps have data; also warms NCCL up and times the plain
        # broadcast of the whole blob for the report
        def standalone_ms(send):
            send()
            torch.cuda.synchronize()
            dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            send()
            e1.record()
            torch.cuda.synchronize()
            ms = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device="cuda")
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
            return float(ms.item())

        nccl_scratch = torch.empty(size, dtype=torch.uint8, device="cuda") if channel is not None else blob
        nccl_ms = standalone_ms(lambda: dist.broadcast(nccl_scratch, src=0))
        if channel is not None:
            del nccl_scratch
            switch_ms = standalone_ms(lambda: channel.send(packed_on_sender if rank == 0 else None, src=0, blocks=128))
            # every rank's copy must be rank 0's blob, bit for bit, before anything is timed with it
            digest = blob[: size // 8 * 8].view(torch.int64).sum().reshape(1)
            lowest, highest = digest.clone(), digest.clone()
            dist.all_reduce(lowest, op=dist.ReduceOp.MIN)
            dist.all_reduce(highest, op=dist.ReduceOp.MAX)
            sender = packed_on_sender[: size // 8 * 8].view(torch.int64).sum().reshape(1) if rank == 0 else digest
            assert lowest.item() == highest.item() == sender.item(), "the switch delivered different bytes to different ranks"
            use_switch = args.broadcast == "switch" or switch_ms <= nccl_ms   # the same numbers on every rank (reduced above)
            if use_switch:
                collective = {"op": "packed B stored once by rank 0 through the NVSwitch multicast mapping (multimem.st, the library's "
                                    "nkb_multicast_store) and a flag barrier between the GPUs (nkb_peer_barrier), inside the timed "
                                    "region, once, ahead of the first step",
                              "bytes": int(size), "standalone_ms_whole_blob": switch_ms, "standalone_ms_ncclBroadcast": nccl_ms}
            else:
                # NCCL was faster here (two GPUs): rank 0's copy of the symmetric buffer becomes the sender's blob
                if rank == 0:
                    blob.copy_(packed_on_sender)
                collective = {"op": "ncclBroadcast of packed B from rank 0, inside the timed region, once, ahead of the first step "
                                    "(chosen over the switch delivery by the set-up's timings)",
                              "bytes": int(size), "standalone_ms_whole_blob": nccl_ms, "standalone_ms_switch": switch_ms}
        else:
            collective = {"op": "ncclBroadcast of packed B from rank 0, inside the timed region, once" + (", in 2 column blocks overlapped with the first step" if len(pieces) == 2 else ", ahead of the first step")
                                + (f" (switch delivery not used: {switch_note})" if switch_note else ""),
                          "bytes": int(size), "standalone_ms_whole_blob": nccl_ms}
        broadcast_and_first_step()   # warm-up of the timed path

    # The clock sampler starts ahead of the warm-up, so that nothing idles between the warm-up and the timed region (NVLink
    # and the SM clocks drop to a lower state within a fraction of a second of idling).
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    for _ in range(args.warmup):
        nk.dots_packed(ta, packed, out=out, dtype=dtype)
    torch.cuda.synchronize()
    assert nk.synchronize() == 0, "device error word set during warm-up"
    reference_rows = out[:4].clone()
    if world > 1:
        # the timed region must deliver B itself: every rank but the sender forgets what the warm-up left behind; one
        # more untimed broadcast (of a scratch buffer the size of the blob) is the communication path's own warm-up
        if rank != 0 or use_switch:
            blob.zero_()
        if not use_switch:
            scratch = torch.empty_like(blob)
            dist.broadcast(scratch, src=0)
            del scratch
        else:
            channel.barrier()
        torch.cuda.synchronize()

    # ---- timed region: the broadcast (N > 1) and exactly K steps, barrier + synchronize on both sides, max over ranks
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    launches0, wall0 = nk.launch_count(), time.time()
    start, first_done, stop = (torch.cuda.Event(enable_timing=True) for _ in range(3))
    start.record()
    if world > 1:
        broadcast_and_first_step()
        first_done.record()
        for _ in range(args.steps - 1):
            nk.dots_packed(ta, packed, out=out, dtype=dtype)
    else:
        for _ in range(args.steps):
            nk.dots_packed(ta, packed, out=out, dtype=dtype)
    stop.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    wall1 = time.time()
    launches = nk.launch_count() - launches0
    seconds = start.elapsed_time(stop) / 1e3
    t = torch.tensor([seconds, start.elapsed_time(first_done) / 1e3 if world > 1 else 0.0], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    seconds, first_step_seconds = float(t[0].item()), float(t[1].item())
    clocks = sampler.stop(wall0, wall1) if rank == 0 else None
    assert nk.synchronize() == 0, "device error word set during the timed region"
    assert torch.equal(out[:4], reference_rows), "the timed region's result differs from the warm-up's"
    if collective is not None:
        collective["first_step_ms_with_broadcast"] = first_step_seconds * 1e3
        collective["steady_ms_per_step"] = (seconds - first_step_seconds) / max(1, args.steps - 1) * 1e3

    # ---- end to end through the C ABI with host buffers (pinned): upload this rank's rows of A, multiply, download its C
    a_pin = torch.from_numpy(a_host.view(STORE[eb])).pin_memory()
    c_pin = torch.empty((rows, N), dtype=out_dtype).pin_memory()
    fn = getattr(nk.lib, f"nk_dots_packed_{dtype}")

    def e2e_step():
        fn(a_pin.data_ptr(), blob.data_ptr(), c_pin.data_ptr(), rows, N, K, K * eb, N * 4)

    for _ in range(2):
        e2e_step()
    assert nk.last_error() == "", nk.last_error()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e2e_steps = max(3, min(args.steps, 10))
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    torch.cuda.synchronize()
    e2e_seconds = time.perf_counter() - t0
    te = torch.tensor([e2e_seconds], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(te, op=dist.ReduceOp.MAX)
    e2e_seconds = float(te.item())
    assert torch.equal(c_pin[:4].cuda(), out[:4]), "host-buffer path and device path disagree"
    del a_pin, c_pin

    ops_per_step = 2.0 * M * N * K                     # the whole job's step: all ranks together
    value = ops_per_step * args.steps / seconds / 1e9
    peaks = measured_peaks()
    # roofline of the dominant kernel: one launch = this rank's rows; duration = the steady step (all launches at N = 1)
    launch_seconds = seconds / args.steps if world == 1 else (seconds - first_step_seconds) / max(1, args.steps - 1)
    achieved_tflops = 2.0 * rows * N * K / launch_seconds / 1e12
    bf16_like = dtype in ("bf16", "f16")
    peak = peaks["bf16_tflops"] * (1.0 if bf16_like else 2.0)

    extras, probes, sustained, cpu_baseline, cpu_single, pack_leg = {}, None, None, None, None, None
    if rank == 0 and world == 1 and not args.no_extras:
        # The packer, timed on its own (it runs outside the timed region above, as in the reference's benchmark): payload in the
        # tensor cores' shared-memory layout + one squared norm per row. HBM bound: rows read twice (payload pass, norm pass),
        # payload written once.
        xb = torch.from_numpy(gen_rows(N, dtype, SEEDS[dtype] + 1).view(STORE[eb])).cuda()
        xblob = torch.empty(size, dtype=torch.uint8, device="cuda")
        pack_fn = getattr(nk.lib, f"nk_dots_pack_{dtype}")
        for _ in range(3):
            pack_fn(xb.data_ptr(), N, K, K * eb, xblob.data_ptr())
        torch.cuda.synchronize()
        p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        p0.record()
        for _ in range(20):
            pack_fn(xb.data_ptr(), N, K, K * eb, xblob.data_ptr())
        p1.record()
        torch.cuda.synchronize()
        pack_ms = p0.elapsed_time(p1) / 20
        pack_bytes = 3.0 * N * K * eb + 4.0 * N
        pack_leg = {"ms": pack_ms, "algorithmic_bytes": pack_bytes, "gb_per_s": pack_bytes / pack_ms / 1e6,
                    "frac_of_measured_hbm": pack_bytes / pack_ms / 1e6 / peaks["hbm_gbs"],
                    "note": f"nk_dots_pack_{dtype} of {N} x {K}, device-resident, 20 calls (payload kernel + norm kernel + header)"}
        del xb, xblob
        probes = library_peak_probes(torch, peaks)
        peak8 = max(probes["assumed_8bit_tflops"], probes.get("scaled_mm_e4m3_tflops", 0.0), probes.get("int_mm_i8_tops", 0.0))
        sustained = sustained_leg(nk, torch, ta, packed, out, dtype, peaks, local)
        for dt in ("bf16", "f16", "i8", "u8", "e4m3", "e5m2", "e2m3", "e3m2"):
            pk = peaks["bf16_tflops"] if dt in ("bf16", "f16") else peak8
            if dt == dtype:
                extras[dt] = {"gso_per_s": value, "frac_of_measured_peak": achieved_tflops / pk, "peak_tflops": pk}
                continue
            xa = torch.from_numpy(gen_rows(M, dt, SEEDS[dt]).view(STORE[ELEMENT_BYTES[dt]])).cuda()
            xb = torch.from_numpy(gen_rows(N, dt, SEEDS[dt] + 1).view(STORE[ELEMENT_BYTES[dt]])).cuda()
            xp = nk.dots_pack(xb, dt)
            xo = torch.empty((M, N), dtype=torch.int32 if dt in ("i8", "u8") else torch.float32, device="cuda")
            for _ in range(3):
                nk.dots_packed(xa, xp, out=xo, dtype=dt)
            torch.cuda.synchronize()
            s = time_device_steps(nk, torch, xa, xp, xo, dt, 10)
            extras[dt] = {"gso_per_s": ops_per_step * 10 / s / 1e9, "frac_of_measured_peak": ops_per_step * 10 / s / 1e12 / pk, "peak_tflops": pk}
            del xa, xb, xp, xo
        # f32 inputs: f64 accumulation on the FP64 CUDA cores (the reference's numerics demand it), against the f64 library GEMM
        xa, xb = torch.randn(M, K, device="cuda"), torch.randn(N, K, device="cuda")
        xp = nk.dots_pack(xb, "f32")
        xo = torch.empty((M, N), dtype=torch.float64, device="cuda")
        nk.dots_packed(xa, xp, out=xo, dtype="f32")
        torch.cuda.synchronize()
        s = time_device_steps(nk, torch, xa, xp, xo, "f32", 3)
        pk = probes.get("matmul_f64_tflops")
        extras["f32"] = {"gso_per_s": ops_per_step * 3 / s / 1e9, "frac_of_measured_peak": (ops_per_step * 3 / s / 1e12 / pk) if pk else None,
                         "peak_tflops": pk, "note": "f64 accumulation on CUDA cores; peak = the f64 library GEMM timed in this run"}
        del xa, xb, xp, xo
        res = time_reference(dtype, steps=3, warmup=1)
        if res is not None:
            cpu_baseline = {k: res[k] for k in ("value", "unit", "cores", "kind", "sample")}
            one = time_reference(dtype, steps=2, warmup=1, threads=1, seconds_per_step=2.0)
            cpu_single = {k: one[k] for k in ("value", "unit", "cores", "kind", "sample")}

    # ---- the two search workloads on sharded twins, at every N: corpus rows / documents split over the ranks, every rank
    # searches its shard, the k best per query are merged on rank 0 with one gather and the library's merge kernel; timed
    # from "shards packed and resident" to "merged lists on rank 0", slowest rank.
    search = {}
    if not args.no_extras:
        del ta, out
        torch.cuda.empty_cache()
        near = workloads.run_nearest_sharded(8192, 8_000_000, 768, 10, "f16", steps=2, warmup=1)
        late = workloads.run_maxsim_sharded(256, 200_000, 128, 100, steps=2, warmup=1)
        if rank == 0:
            cpu_search = (time_reference_search() or {}) if world == 1 else {}
            # Steps of 20 - 120 ms run under the power cap, so the tensor peak beside them is the sustained one, per GPU.
            for leg in (near, late):
                leg["frac_of_sustained_bf16_peak"] = leg["gso_per_s"] / 1e3 / (peaks["bf16_tflops_sustained"] * world)
            search = {"nearest_top10_8192x8000000x768_f16": dict(near, cpu=cpu_search.get("nearest")),
                      "maxsim_top100_256x200000_bf16": dict(late, cpu=cpu_search.get("maxsim"))}

    if rank == 0:
        note = f"peak = {peaks['source']} cuBLAS bf16 burst {peaks['bf16_tflops']} TF/s"
        if not bf16_like:
            note += " x 2 for 8-bit operands (see peak_probes for the library 8-bit GEMMs measured in this run)"
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": seconds / args.steps * 1e3, "higher_is_better": True, "scaling": "strong" if world > 1 else "weak",
            "vs_baseline": None, "dtype": dtype_arith(dtype), "data": "synthetic", "config": workload_config(dtype, world),
            "roofline": {"bound": "tensor", "achieved": achieved_tflops, "peak": peak, "unit": "TFLOP/s", "frac": achieved_tflops / peak,
                         "traffic": NCU_DRAM_BYTES_PER_LAUNCH.get((dtype, rows)), "note": note,
                         "launch": f"{rows} x {N} x {K}, mean duration {launch_seconds * 1e3:.4f} ms (CUDA events on the launching stream)"},
            "cpu_baseline": cpu_baseline, "cpu_baseline_single_thread": cpu_single,
            "e2e": {"value": ops_per_step * e2e_steps / e2e_seconds / 1e9, "unit": UNIT,
                    "h2d_bytes_per_step": M * K * eb, "d2h_bytes_per_step": M * N * 4, "steps": e2e_steps,
                    "ms_per_step": e2e_seconds / e2e_steps * 1e3},
            "gpu_launches": int(launches), "clocks": clocks, "collective": collective, "sustained": sustained, "pack": pack_leg,
            "peak_probes": probes, "per_dtype": extras, "search_workloads": search,
        }
        print(json.dumps(line))
    if world > 1:
        if channel is not None:
            del packed, blob
            channel.close()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
