"""Benchmark of the ternary hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload (config 1 of the baseline): the PQ2_0 ternary matvec K=5120 -> N=17408, batch 1, on q8k
activations; synthetic weights (codes uniform over {-1,0,+1}, f16 scales in [0.01,0.05]) and an
N(0,1) activation vector, all seeded.  One step = one sweep of `matvec_t2` over 12 distinct weight
matrices (285 MB, larger than the 126 MB L2, so every launch reads its weights from HBM).

`value` is the algorithmic GB/s of the sweep with everything resident in HBM, timed with CUDA
events on the library's stream.  `e2e` is the same metric through the public call sequence with
host buffers: pinned-host activation -> device, Hadamard + q8k, matvec, result row -> host.
"""
import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

ROWS, COLS = 17408, 5120
N_WEIGHTS = 12
METRIC = "matvec_t2_hbm_gbs"
# dram__bytes_read.sum + dram__bytes_write.sum of one k_matvec_t2 launch on this workload, from the ncu capture
# summarised in profiles/matvec_t2_config1_K5120_N17408.md
NCU_DRAM_BYTES_PER_LAUNCH = 23698944


def algorithmic_bytes(rows, cols, ntok=1, accum=False):
    """rows*cols/128*34 (codes + f16 scales) + ntok*(cols + 4*cols/256) (q8 row + scales) + 4*ntok*rows (output)."""
    return rows * cols // 128 * 34 + ntok * (cols + 4 * cols // 256) + 4 * ntok * rows * (2 if accum else 1)


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed region runs (read only)."""

    def __init__(self, index):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thr = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        names = {"hw_slowdown": nv.nvmlClocksThrottleReasonHwSlowdown, "hw_thermal_slowdown": nv.nvmlClocksThrottleReasonHwThermalSlowdown,
                 "sw_thermal_slowdown": nv.nvmlClocksThrottleReasonSwThermalSlowdown, "sw_power_cap": nv.nvmlClocksThrottleReasonSwPowerCap}
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for k, bit in names.items():
                    if r & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            time.sleep(0.005)

    def __enter__(self):
        if self.nv:
            self._thr = threading.Thread(target=self._run, daemon=True)
            self._thr.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._thr:
            self._thr.join()

    def summary(self):
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(s)}


def measured_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        return json.load(open(p))["hbm_gbs"], "measured"
    return 6650.0, "fallback"


def cpu_arm(steps, warmup, as_reference):
    """The reference's CPU path (cpu::matvec, Numerics::Ggml) restated in C++, all host threads."""
    import numpy as np
    from oracle import orc
    from tests.util import synth_pq2
    raw = synth_pq2(1, ROWS, COLS)
    x = np.random.default_rng(0).standard_normal(COLS).astype(np.float32)
    nthreads = orc.max_threads()
    for _ in range(max(warmup, 1)):
        orc.matvec_ternary(raw, ROWS, COLS, x, nthreads=nthreads)
    t0 = time.perf_counter()
    n = 0
    while n < steps and (as_reference or time.perf_counter() - t0 < 10.0):
        orc.matvec_ternary(raw, ROWS, COLS, x, nthreads=nthreads)
        n += 1
    dt = (time.perf_counter() - t0) / n
    gbs = algorithmic_bytes(ROWS, COLS) / dt / 1e9
    return {"value": gbs, "unit": "GB/s", "cores": nthreads, "kind": "port",
            "sample": f"{n} calls of the {ROWS}x{COLS} matvec incl. q8k quantisation, {dt * 1e3:.2f} ms each"}, dt


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=400)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="b200")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    config = {"workload": f"config1: PQ2_0 ternary matvec K={COLS} N={ROWS} batch 1 on q8k activations", "rows": ROWS, "cols": COLS,
              "l2": f"inputs larger than L2: sweep over {N_WEIGHTS} distinct weight matrices ({N_WEIGHTS * algorithmic_bytes(ROWS, COLS) // 1000000} MB)",
              "launches_per_step": N_WEIGHTS, "sharding": "independent replicas of the sweep per GPU (rows of one matrix are not split at this size)"}

    if args.impl == "reference":
        if rank != 0:
            return
        cb, dt = cpu_arm(max(args.steps, 1), max(args.warmup, 1), True)
        print(json.dumps({"impl": "reference", "metric": METRIC, "value": cb["value"], "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps,
                          "warmup": args.warmup, "ms_per_step": dt * 1e3 * N_WEIGHTS, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                          "dtype": "int8 x 2-bit codes -> int32, f32 epilogue", "data": "synthetic", "config": config, "cpu_baseline": cb,
                          "e2e": {"value": cb["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))
        return

    import numpy as np
    import torch
    from irontimber_b200.backend import CudaBackend

    dist = None
    if world > 1:
        import torch.distributed as dist
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    be = CudaBackend(local_rank, arena_floats=1 << 22)
    stream = torch.cuda.ExternalStream(be.stream, device=f"cuda:{local_rank}")
    mats = [be.mat_synth(1000 + 17 * rank + i, ROWS, COLS) for i in range(N_WEIGHTS)]
    rng = np.random.default_rng(rank)
    x = rng.standard_normal(COLS).astype(np.float32)
    signs = np.where(rng.integers(0, 2, COLS) == 1, 1.0, -1.0).astype(np.float32)
    be.set_signs(signs)
    q = be.q8_rows(COLS, 1)
    XO, YO = 0, 8192
    be.upload(XO, x)
    be.had_q8(COLS, 1, XO, COLS, q)

    def sweep():
        for m in mats:
            be.mv(m, 1, q, YO, ROWS)

    def barrier():
        be.sync()
        torch.cuda.synchronize()
        if dist:
            dist.barrier()
        torch.cuda.synchronize()

    # one step = one replay of a recorded sweep (the launches are queued on the device, so the host
    # launch path is not what is timed)
    be.capture_begin()
    sweep()
    graph = be.capture_end()
    for _ in range(max(args.warmup, 3)):
        be.graph_launch(graph)
    barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as clocks:
        barrier()
        ev0.record(stream)
        for _ in range(args.steps):
            be.graph_launch(graph)
        ev1.record(stream)
        barrier()
    ms = ev0.elapsed_time(ev1)
    if dist:
        t = torch.tensor([ms], device=f"cuda:{local_rank}")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    launches = args.steps * N_WEIGHTS
    per_launch_s = ms / 1e3 / launches
    abytes = algorithmic_bytes(ROWS, COLS)
    achieved = abytes / per_launch_s / 1e9
    peak, peak_kind = measured_peak()

    # end to end through the public calls with host buffers (pinned): H2D x, had_q8, mv, D2H y
    import ctypes as C
    from irontimber_b200 import _lib
    hx = torch.from_numpy(x).pin_memory()
    hy = torch.empty(ROWS, dtype=torch.float32).pin_memory()
    e2e_steps = max(args.steps // 4, 10)

    def e2e_step(m):
        _lib.check(be.L.it_arena_write(be.ctx, XO, C.c_void_p(hx.data_ptr()), COLS))
        be.had_q8(COLS, 1, XO, COLS, q)
        be.mv(m, 1, q, YO, ROWS)
        _lib.check(be.L.it_arena_read(be.ctx, YO, C.c_void_p(hy.data_ptr()), ROWS))
    for i in range(5):
        e2e_step(mats[i % N_WEIGHTS])
    barrier()
    t0 = time.perf_counter()
    for i in range(e2e_steps * N_WEIGHTS):
        e2e_step(mats[i % N_WEIGHTS])
    barrier()
    e2e_s = (time.perf_counter() - t0) / (e2e_steps * N_WEIGHTS)
    if dist:
        t = torch.tensor([e2e_s], device=f"cuda:{local_rank}")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())

    out = {"metric": METRIC, "value": achieved * world, "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
           "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
           "dtype": "int8 x 2-bit codes -> int32, f32 epilogue", "data": "synthetic", "config": config,
           "clocks": clocks.summary(), "gpu_launches": launches,
           "e2e": {"value": abytes / e2e_s / 1e9 * world, "unit": "GB/s", "h2d_bytes_per_step": COLS * 4 * N_WEIGHTS, "d2h_bytes_per_step": ROWS * 4 * N_WEIGHTS,
                   "us_per_call": e2e_s * 1e6},
           "roofline": {"bound": "hbm", "kernel": "k_matvec_t2<1>", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                        "peak_kind": peak_kind, "algorithmic_bytes_per_launch": abytes, "us_per_launch": per_launch_s * 1e6, "traffic": NCU_DRAM_BYTES_PER_LAUNCH}}
    if rank == 0:
        cb, _ = cpu_arm(10 ** 9, 1, False)
        out["cpu_baseline"] = cb
        print(json.dumps(out))
    be.graph_destroy(graph)
    for m in mats:
        m.close()
    q.close()
    be.close()
    if dist:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
