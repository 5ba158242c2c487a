"""Benchmark of the packed-contraction hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--dtype bf16] [--impl reference]

One "step" is one nk_dots_packed_<t> call over one batch: A (8192 x 8192) against a pre-packed B
(8192 x 8192), the configuration the metric is quoted on (M = N = K = 8192, N(0,1) entries rounded to
the storage type, seeded; B is packed once outside the timed region exactly as the reference's own
benchmark does, bench/bench.hpp:245). Unit: gso/s = 2*M*N*K / seconds / 1e9 (bench/bench.hpp:257).

With N > 1 ranks (torchrun) every rank multiplies its own 8192-row block of A against the same packed B
(rows of A partitioned across GPUs: weak scaling, no collective on the data path; B is packed on rank 0
and broadcast over NCCL once during set-up). The timed region is bracketed by a barrier and a device
synchronize; the reported time is the maximum over ranks.

Prints ONE JSON line (rank 0). `value` is measured with operands resident in HBM; `e2e` is the same metric
through the C ABI with HOST buffers (pinned): every step uploads A and downloads C inside the timed region.
`--impl reference` times the reference's own CPU kernels (compiled from its sources into oracle/_ref/) on
this host's cores, on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import ctypes
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


# dram__bytes_read.sum + dram__bytes_write.sum of ONE launch of the dominant kernel, from the ncu capture summarised in
# profiles/gemm_tc_pair_bf16_8192_dram_traffic.md (1.116e9 read + 2.52e8 written; algorithmic bytes A + packed B + C
# are 5.37e8). Keyed by (dtype, rows of A); other configurations report null.
NCU_DRAM_BYTES_PER_LAUNCH = {("bf16", 8192): 1_367_000_000}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"bf16_tflops": float(p["bf16_tflops"]), "hbm_gbs": float(p["hbm_gbs"]), "source": "measured"}
    return {"bf16_tflops": 1590.0, "hbm_gbs": 6650.0, "source": "fallback"}


def gen_rows(rows: int, dtype: str, seed: int) -> np.ndarray:
    """rows x K synthetic matrix in the storage type of `dtype`, generated in blocks to bound host memory."""
    from numkong_b200 import synthetic as syn
    return np.concatenate([syn.normal_matrix(min(1024, rows - r), K, dtype, seed * 100003 + r) for r in range(0, rows, 1024)])


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.device_index, self.proc, self.lines = device_index, None, []
        self.nvml_samples, self.nvml_stop, self.nvml_thread, self.nvml_max = [], threading.Event(), None, None

    def _start_nvml(self) -> bool:
        """In-process NVML polling (read-only queries, about a thousand per second): the timed region of the default run
        lasts some 15 ms, shorter than nvidia-smi's fastest sampling period."""
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


def time_reference(dtype: str, steps: int, warmup: int, rows_per_step: int | None = None):
    """Times the reference's dispatched CPU kernel on a bounded sample: `rows_per_step` rows of A against the
    full packed B, rows split evenly over all host threads (each thread configures itself once, as
    the reference requires for AMX: include/numkong/capabilities.h:393-410)."""
    ref = _ref_library()
    if ref is None:
        return None
    import oracle
    threads = max(1, len(os.sched_getaffinity(0)))
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
        barrier = threading.Barrier(threads + 1)

        def work(t):
            ref.configure_thread()
            lo, hi = t * per, min(rows, (t + 1) * per)
            barrier.wait()
            if hi > lo:
                fn(a[lo:hi].ctypes.data, blob.ctypes.data, c[lo:hi].ctypes.data, hi - lo, N, K, K * eb, N * 4)
            barrier.wait()

        pool = [threading.Thread(target=work, args=(t,)) for t in range(threads)]
        for th in pool:
            th.start()
        barrier.wait()
        t0 = time.perf_counter()
        barrier.wait()
        dt = time.perf_counter() - t0
        for th in pool:
            th.join()
        return dt

    if rows_per_step is None:
        # calibrate: about one second of CPU work per step
        probe_rows = threads * 8
        a = gen_rows(probe_rows, dtype, SEEDS[dtype])
        c = np.zeros((probe_rows, N), dtype=oracle.out_dtype(dtype))
        run(a, c)
        dt = run(a, c)
        rows_per_step = int(min(M, max(threads * 8, probe_rows * 1.0 / max(dt, 1e-4)))) // threads * threads
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
    from numkong_b200 import synthetic as syn
    threads = max(1, len(os.sched_getaffinity(0)))
    u64, vp = ctypes.c_uint64, ctypes.c_void_p

    def run_threads(work):
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

    run_threads(nearest_work)
    dt = min(run_threads(nearest_work) for _ in range(2))
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

    run_threads(maxsim_work)
    dt = min(run_threads(maxsim_work) for _ in range(2))
    out["maxsim"] = {"gso_per_s": 2.0 * 8 * 32 * float(counts.sum()) * 128 / dt / 1e9, "cores": threads, "kind": "reference",
                     "sample": f"nk_maxsim_packed_bf16, 8 queries x 32 tokens vs 256 documents ({int(counts.sum())} tokens), one call per pair"}
    return out


def reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    dtype = args.dtype
    res = time_reference(dtype, args.steps, args.warmup)
    if res is None:
        print(json.dumps({"impl": "reference", "unavailable": "oracle/_ref/libnumkong.so has not been built (make -C oracle ref)"}))
        return
    line = {
        "impl": "reference", "metric": METRIC, "value": res["value"], "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": res["ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": dtype_arith(dtype), "data": "synthetic",
        "config": workload_config(dtype, 1) | {"sample_rows_per_step": res["rows_per_step"]},
        "cpu_baseline": {k: res[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": res["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ---------------------------------------------------------------------------------------- our arm
def dtype_arith(dtype: str) -> str:
    return {"i8": "i32", "u8": "u32"}.get(dtype, "f32") + f" accumulate of {dtype}"


def workload_config(dtype: str, n_gpus: int):
    return {"workload": f"dots_packed {dtype} M=N=K=8192 per GPU (B pre-packed, N(0,1) rounded to {dtype}, seed {SEEDS[dtype]})",
            "rows_of_A_per_gpu": M, "global_rows_of_A": M * n_gpus, "width": N, "depth": K,
            "parallelism": f"rows of A partitioned over {n_gpus} GPU(s), packed B replicated",
            "l2": "operands (A 8192x8192 + packed B + C = 384-512 MiB) exceed the 126 MB L2; no explicit flush"}


def time_device_steps(nk, torch, ta, packed, out, dtype, steps):
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        nk.dots_packed(ta, packed, out=out, dtype=dtype)
    stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop) / 1e3


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--dtype", default="bf16")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-extras", action="store_true", help="skip the per-dtype table and the CPU baseline")
    ap.add_argument("--rows", type=int, default=8192,
                    help="rows of A per GPU; anything but 8192 is a reduced case for profiler captures, not the benchmark")
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
    from numkong_b200 import sharding

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    dtype = args.dtype
    nk.set_stream(torch.cuda.current_stream().cuda_stream)

    # ---- set-up (untimed): this rank's rows of A, B packed on rank 0 and broadcast
    a_host = gen_rows(M, dtype, SEEDS[dtype] + 1000 * rank)
    ta = torch.from_numpy(a_host.view(STORE[a_host.itemsize])).cuda()
    size = nk.PackedMatrix.packed_size(N, K, dtype)
    blob = torch.empty(size, dtype=torch.uint8, device="cuda")
    if rank == 0:
        b_host = gen_rows(N, dtype, SEEDS[dtype] + 1)
        tb = torch.from_numpy(b_host.view(STORE[b_host.itemsize])).cuda()
        packed0 = nk.dots_pack(tb, dtype)
        blob.copy_(packed0.buffer)
        del tb, packed0
    torch.cuda.synchronize()
    sharding.broadcast_bytes(blob, src=0)
    packed = nk.PackedMatrix(blob, dtype, N, K)
    out_dtype = torch.int32 if dtype in ("i8", "u8") else torch.float32
    out = torch.empty((M, N), dtype=out_dtype, device="cuda")

    for _ in range(args.warmup):
        nk.dots_packed(ta, packed, out=out, dtype=dtype)
    torch.cuda.synchronize()
    assert nk.synchronize() == 0, "device error word set during warm-up"

    # ---- timed region: exactly K steps, barrier + synchronize on both sides, max over ranks
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    launches0, wall0 = nk.launch_count(), time.time()
    seconds = time_device_steps(nk, torch, ta, packed, out, dtype, args.steps)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    wall1 = time.time()
    launches = nk.launch_count() - launches0
    t = torch.tensor([seconds], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    seconds = float(t.item())
    clocks = sampler.stop(wall0, wall1) if rank == 0 else None
    assert nk.synchronize() == 0, "device error word set during the timed region"

    # ---- end to end through the C ABI with host buffers (pinned): upload A, multiply, download C every step
    a_pin = torch.from_numpy(a_host.view(STORE[a_host.itemsize])).pin_memory()
    c_pin = torch.empty((M, N), dtype=out_dtype).pin_memory()
    fn = getattr(nk.lib, f"nk_dots_packed_{dtype}")
    eb = a_host.itemsize

    def e2e_step():
        fn(a_pin.data_ptr(), blob.data_ptr(), c_pin.data_ptr(), M, N, K, K * eb, N * 4)

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
    # spot check of the e2e result against the device-resident result
    assert torch.equal(c_pin[:4].cuda(), out[:4]), "host-buffer path and device path disagree"

    ops_per_step = 2.0 * M * N * K
    value = ops_per_step * world * args.steps / seconds / 1e9
    peaks = measured_peaks()
    per_launch_s = seconds / args.steps
    achieved_tflops = ops_per_step / per_launch_s / 1e12
    peak = peaks["bf16_tflops"] * (1.0 if dtype in ("bf16", "f16") else 2.0)

    extras = {}
    search = {}
    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_extras:
        del a_pin, c_pin
        for dt in ("bf16", "f16", "i8", "u8", "e4m3", "e5m2", "e2m3", "e3m2"):
            if dt == dtype:
                extras[dt] = {"gso_per_s": value, "frac_of_peak": achieved_tflops / peak}
                continue
            xa = torch.from_numpy(gen_rows(M, dt, SEEDS[dt]).view(STORE[nk.DTYPE_BYTES[dt]])).cuda()
            xb = torch.from_numpy(gen_rows(N, dt, SEEDS[dt] + 1).view(STORE[nk.DTYPE_BYTES[dt]])).cuda()
            xp = nk.dots_pack(xb, dt)
            xo = torch.empty((M, N), dtype=torch.int32 if dt in ("i8", "u8") else torch.float32, device="cuda")
            for _ in range(3):
                nk.dots_packed(xa, xp, out=xo, dtype=dt)
            torch.cuda.synchronize()
            s = time_device_steps(nk, torch, xa, xp, xo, dt, 10)
            pk = peaks["bf16_tflops"] * (1.0 if dt in ("bf16", "f16") else 2.0)
            extras[dt] = {"gso_per_s": ops_per_step * 10 / s / 1e9, "frac_of_peak": ops_per_step * 10 / s / 1e12 / pk}
            del xa, xb, xp, xo
        res = time_reference(dtype, steps=3, warmup=1)
        if res is not None:
            cpu_baseline = {k: res[k] for k in ("value", "unit", "cores", "kind", "sample")}
        # The two search workloads on their small twins (BASELINE configs 4 and 5 scaled down), GPU and reference CPU.
        from numkong_b200 import workloads
        near = workloads.run_nearest(1024, 200000, 768, 10, "f16", steps=5)
        late = workloads.run_maxsim(64, 20000, steps=3)
        cpu_search = time_reference_search() or {}
        search = {"nearest_top10_1024x200000x768_f16": {"gso_per_s": near["gso_per_s"], "ms": near["ms"], "cpu": cpu_search.get("nearest")},
                  "maxsim_top100_64x20000_bf16": {"gso_per_s": late["gso_per_s"], "ms": late["ms"], "cpu": cpu_search.get("maxsim")}}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": seconds / args.steps * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": dtype_arith(dtype), "data": "synthetic", "config": workload_config(dtype, world),
            "roofline": {"bound": "tensor", "achieved": achieved_tflops, "peak": peak, "unit": "TFLOP/s", "frac": achieved_tflops / peak,
                         "traffic": NCU_DRAM_BYTES_PER_LAUNCH.get((dtype, args.rows)),
                         "note": f"peak = {peaks['source']} cuBLAS bf16 burst {peaks['bf16_tflops']} TF/s"
                                 + ("" if dtype in ("bf16", "f16") else " x 2 for 8-bit operands (no measured 8-bit figure on this pool)")},
            "cpu_baseline": cpu_baseline,
            "e2e": {"value": ops_per_step * world * e2e_steps / e2e_seconds / 1e9, "unit": UNIT,
                    "h2d_bytes_per_step": M * K * eb, "d2h_bytes_per_step": M * N * 4, "steps": e2e_steps,
                    "ms_per_step": e2e_seconds / e2e_steps * 1e3},
            "gpu_launches": int(launches), "clocks": clocks, "per_dtype": extras, "search_workloads": search,
        }
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
