"""Benchmark of the ternary hot path on B200: greedy decode of the 27B-shape ternary decoder.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--prompt P] [--layers L] [--decode-only | --roofline-only | --sweep]

Workload (config 2 of the baseline): the 64-layer random-init ternary decoder with the reference architecture
(48 gated-delta-net + 16 attention layers, n_embd 5120, n_ff 17408, vocab 248320, f16 KV), batch 1, greedy decode
after a prompt of P = 512 uniform-random token ids.  One step = one decoded token = one replay of the engine's
recorded step (`launches_per_step` kernels, counted from the recorded graph; 401 ternary matvecs stream 6.8 GB of
weights - far more than the 126 MB L2, so every step reads its weights from HBM).

`value`: decode tokens/s with everything resident and no read-back between steps, timed with CUDA events on the
library's stream.  `e2e`: the same through the public call `it_engine_generate`, which takes the token ids from
host memory and reads every pick back to the host (4 bytes per token), timed on the host clock.
`roofline`: the dominant kernel, `k_matvec_t2`, timed alone on the baseline's config 1 (K=5120 -> N=17408, batch 1)
as a sweep over 12 distinct weight matrices (285 MB), against the measured HBM copy bandwidth.
`cpu_baseline` / `--impl reference`: the reference's CPU path (C++ port of src/cpu.rs forward_token, reference
order, every host thread the process may use) on a truncated stack, extrapolated to the full depth; the sample is stated.
`prefill_lengths` (config 4): prompts of 64 / 2048 / 4096 / 7168 tokens in 64-row passes.  `mtp` (config 3): 256 tokens
after prompts of 128 and 2048 tokens with draft lengths 1..3, random head and scripted right drafts.
With N > 1 (one process per GPU, torchrun) `value` is ONE sequence on the row-sharded engine (strong scaling): every
trunk matrix and the LM head split by output rows over the ranks, each rank's matvec kernels push their result slices
into every peer's arena over NVLink (8-byte value+epoch slots) and collect the peers' slices at the end of the kernel,
everything else replicated, every rank producing the same tokens; tokens per second from the max over ranks of the
device time.  `sharded.parity` says whether every rank produced the tokens of rank 0's unsharded engine.  `replicas` is
the aggregate of N independent sequences, one full engine per GPU and no collective, for comparison.
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
METRIC = "decode_tok_s"
# dram__bytes_read.sum + dram__bytes_write.sum of one k_matvec_t2 launch on config 1, taken from an ncu capture of
# `bench.py --roofline-only` (a constant of the kernel and shape, not measured by this script)
NCU_DRAM_BYTES_PER_LAUNCH = 23717632
CPU_LAYERS = 4      # layers of the truncated stack the CPU arm runs


def algorithmic_bytes(rows, cols, ntok=1, accum=False):
    """rows*cols/128*34 (codes + f16 scales) + ntok*(cols + 4*cols/256) (q8 row + scales) + 4*ntok*rows (output)."""
    return rows * cols // 128 * 34 + ntok * (cols + 4 * cols // 256) + 4 * ntok * rows * (2 if accum else 1)


def step_weight_bytes(cfg):
    """PQ2_0 bytes of every ternary matrix one decoded token streams (shapes of src/cpu.rs:97-111)."""
    e, ff, hd, nh, nkv = cfg.n_embd, cfg.n_ff, cfg.head_dim, cfg.n_head, cfg.n_head_kv
    cd = 2 * cfg.ssm_state * cfg.ssm_groups + cfg.ssm_inner
    gdn = cd * e + cfg.ssm_inner * e + e * cfg.ssm_inner
    att = 2 * nh * hd * e + 2 * nkv * hd * e + e * nh * hd
    n_att = sum(1 for il in range(cfg.n_layer) if not cfg.is_recurrent(il))
    weights = (cfg.n_layer - n_att) * gdn + n_att * att + cfg.n_layer * 3 * ff * e + cfg.n_vocab * e
    return weights // 128 * 34


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


def cpu_decode_tok_s(n_layer_full, steps):
    """Reference CPU forward_token (oracle, reference order) on a CPU_LAYERS-deep stack of the 27B shapes with
    numpy-random weights; the per-layer time is extrapolated to the full depth, the LM head is timed once."""
    import numpy as np
    from oracle import orc
    from tests.util import make_pq2, tensor_shapes
    from irontimber_b200.engine import config_27b
    cfg = orc.ModelConfig.from_buffer_copy(bytes(config_27b(n_layer=CPU_LAYERS, ctx_len=64)))
    rng = np.random.default_rng(0)
    nthreads = host_threads()
    m = orc.Model(cfg, nthreads=nthreads)
    shapes = tensor_shapes(cfg)
    cache = {}

    def make(name):
        kind, r, c = shapes[name]
        if kind == "pq2":
            if (r, c) not in cache:      # one random matrix per shape is enough for timing
                cache[(r, c)] = make_pq2(rng, r, c)[0]
            return cache[(r, c)]
        lo, hi = {"conv": (-0.5, 0.5), "dt": (-0.5, 0.5), "a": (-1.1, -0.1), "beta": (-0.05, 0.05), "alpha": (-0.05, 0.05)}.get(name, (0.9, 1.1))
        return rng.uniform(lo, hi, r * c).astype(np.float32)
    for il in range(cfg.n_layer):
        names = ("attn_norm", "post_norm", "ffn_gate", "ffn_up", "ffn_down") + (
            ("qkv", "gate", "conv", "dt", "a", "beta", "alpha", "ssm_norm", "ssm_out") if cfg.is_recurrent(il) else ("q", "k", "v", "o", "q_norm", "k_norm"))
        for n in names:
            m.set(n, make(n), il)
    m.set("tok_embd", rng.uniform(-1, 1, 64 * cfg.n_embd).astype(np.float32))          # token ids < 64 only
    m.set("output_norm", make("output_norm")); m.set("output", make("output"))
    for w in {cfg.n_embd, cfg.ssm_inner, cfg.n_head * cfg.head_dim, cfg.n_ff}:
        m.set_signs(np.where(rng.integers(0, 2, w) == 1, 1.0, -1.0).astype(np.float32))
    st = m.new_state()
    m.forward_token(st, 1, True)                                                         # warm-up
    t0 = time.perf_counter(); n = 0
    while n < steps and (n < 2 or time.perf_counter() - t0 < 15.0):
        m.forward_token(st, 2 + n % 60, False); n += 1
    t_layers = (time.perf_counter() - t0) / n
    t0 = time.perf_counter(); m.forward_token(st, 3, True); t_with_head = time.perf_counter() - t0
    t_head = max(t_with_head - t_layers, 0.0)
    t_full = t_layers * n_layer_full / CPU_LAYERS + t_head
    m.close()
    return {"value": 1.0 / t_full, "unit": "tok/s", "cores": nthreads, "kind": "port",
            "sample": f"{n} tokens through a {CPU_LAYERS}-layer stack of the 27B shapes ({t_layers * 1e3:.0f} ms per token) + one LM head ({t_head * 1e3:.0f} ms); "
                      f"extrapolated to {n_layer_full} layers: {t_full:.2f} s per token"}, t_full


def matvec_roofline(torch, local_rank, steps):
    """The dominant kernel alone: replayed sweep of k_matvec_t2 over 12 distinct 17408x5120 matrices."""
    import numpy as np
    from irontimber_b200.backend import CudaBackend
    be = CudaBackend(local_rank, arena_floats=1 << 20)
    stream = torch.cuda.ExternalStream(be.stream, device=f"cuda:{local_rank}")
    mats = [be.mat_synth(1000 + i, ROWS, COLS) for i in range(N_WEIGHTS)]
    rng = np.random.default_rng(0)
    be.set_signs(np.where(rng.integers(0, 2, COLS) == 1, 1.0, -1.0).astype(np.float32))
    q = be.q8_rows(COLS, 1)
    be.upload(0, rng.standard_normal(COLS).astype(np.float32))
    be.had_q8(COLS, 1, 0, COLS, q)
    be.capture_begin()
    for m in mats:
        be.mv(m, 1, q, 8192, ROWS)
    graph = be.capture_end()
    for _ in range(5):
        be.graph_launch(graph)
    be.sync()
    # five timed segments of `steps / 5` replays each; the median segment is reported (and all five listed), so that one
    # disturbed segment (another process waking up, a clock step) does not move the figure
    seg = max(steps // 5, 1)
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(6)]
    evs[0].record(stream)
    for k in range(5):
        for _ in range(seg):
            be.graph_launch(graph)
        evs[k + 1].record(stream)
    be.sync(); torch.cuda.synchronize()
    segs = sorted(evs[k].elapsed_time(evs[k + 1]) / 1e3 / (seg * N_WEIGHTS) for k in range(5))
    per_launch = segs[2]
    be.graph_destroy(graph)
    for m in mats:
        m.close()
    q.close(); be.close()
    abytes = algorithmic_bytes(ROWS, COLS)
    peak, kind = measured_peak()
    ach = abytes / per_launch / 1e9
    return {"bound": "hbm", "kernel": "k_matvec_t2<1> alone on config 1 (K=5120, N=17408, batch 1), sweep of 12 matrices (285 MB > L2)",
            "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak, "peak_kind": kind,
            "algorithmic_bytes_per_launch": abytes, "us_per_launch": per_launch * 1e6, "segments_us_per_launch": [round(x * 1e6, 3) for x in segs],
            "traffic": NCU_DRAM_BYTES_PER_LAUNCH}


def sweep(args, torch, np, rank, world, local_rank, base, emit=True, head_only=False, own_group=True):
    """Config 5 of the baseline: K = 5120, N in {17408, 34816, 69632}, M in {1, 4, 64, 512}, and the Q8_0 LM head
    (N = 248320, M = 1).  With more than one rank every matrix is split by output rows and each launch ends with the
    exchange of the result slices through peer memory; the time is the max over ranks of the device time per launch."""
    from irontimber_b200.backend import CudaBackend
    from irontimber_b200.sharding import shard_range
    dist = None
    if world > 1:
        import torch.distributed as dist
        if own_group:
            torch.cuda.set_device(local_rank)
            dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    be = CudaBackend(local_rank, arena_floats=1 << 26)
    if world > 1:
        be.attach_peers(rank, world)
    stream = torch.cuda.ExternalStream(be.stream, device=f"cuda:{local_rank}")
    rng = np.random.default_rng(0)
    K = COLS
    out = []

    def timed(launch, nmat):
        launch(); be.sync()
        if dist:
            dist.barrier()
        be.capture_begin(); launch(); g = be.capture_end()
        for _ in range(3):
            be.graph_launch(g)
        be.sync()
        if dist:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = max(3, args.steps // 8)
        e0.record(stream)
        for _ in range(reps):
            be.graph_launch(g)
        e1.record(stream)
        be.sync(); torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / (reps * nmat)
        if dist:
            t = torch.tensor([us], device=f"cuda:{local_rank}")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            us = float(t.item())
        be.graph_destroy(g)
        return us

    for N in (() if head_only else (17408, 34816, 69632)):
        row0, n = shard_range(N, rank, world)
        nmat = max(2, min(12, int(300e6 // (n * K * 34 / 128)) + 1))        # distinct matrices: more bytes than L2
        mats = [be.mat_synth_rows(100 + i, N, K, row0, n) if world > 1 else be.mat_synth(100 + i, N, K) for i in range(nmat)]
        for M in (1, 4, 64, 512):
            q = be.q8_rows(K, M)
            be.upload(0, rng.standard_normal((M, K)).astype(np.float32))
            be.had_q8(K, M, 0, K, q, signs=False, rotate=False)
            yo = ((M * K + 63) // 64) * 64
            us = timed(lambda: [be.mv(w, M, q, yo, N) for w in mats], nmat)
            out.append({"op": "matvec_t2" if M <= 8 else "matmul_t2", "N": N, "K": K, "M": M, "us": us,
                        "weights_GBs": N * K * 34 / 128 / us / 1e3, "TOPs": 2 * M * N * K / us / 1e6})
            q.close()
        for w in mats:
            w.close()
    N = 248320
    row0, n = shard_range(N, rank, world)
    heads = [be.qmat_synth_rows(7 + i, N, K, row0, n) if world > 1 else be.qmat_synth(7 + i, N, K) for i in range(2)]
    be.upload(0, rng.standard_normal(K).astype(np.float32))
    us = timed(lambda: [be.mvq(h, 1, 0, K, 1 << 20, N) for h in heads], 2)
    out.append({"op": "matvec_q8 (Q8_0 LM head)", "N": N, "K": K, "M": 1, "us": us, "weights_GBs": N * K * 34 / 32 / us / 1e3})
    for h in heads:
        h.close()
    be.sync()
    if dist:
        dist.barrier()
    be.close()
    if rank == 0 and emit:
        print(json.dumps(dict(base, metric="config5_sweep_us_per_launch", unit="us", higher_is_better=False, scaling="strong", value=out[0]["us"],
                              sweep=out, config={"workload": "config5: ternary product K=5120, N x M grid, and the Q8_0 LM head; rows split evenly over the ranks, result slices exchanged inside the kernels"})))
    if dist and own_group:
        dist.destroy_process_group()
    return out


def host_threads():
    """Host threads this process may run on (torchrun exports OMP_NUM_THREADS=1, which says nothing about the machine)."""
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def prefill_leg(eng, cfg, rng, lengths):
    """Config 4: end-to-end prompt passes (64-row chunks into the f16 KV cache at ctx 8192), host clock, pick read back."""
    out = []
    for n in lengths:
        if n + 1 > cfg.ctx_len:
            continue
        toks = rng.integers(0, cfg.n_vocab, n).tolist()
        eng.reset(); eng.sync()
        t0 = time.perf_counter()
        eng.eval_argmax(toks)
        dt = time.perf_counter() - t0
        out.append({"tokens": n, "seconds": dt, "tok_s": n / dt})
    return out


def mtp_leg(eng, cfg, rng, prompt_len, n_tokens):
    """Config 3 on one prompt length: the library's speculative loop with the random-init NextN head (its drafts are almost
    never right: the reject path) and with the head's draft replaced by the token plain greedy decoding produced (every
    draft accepted: the accept path, as the reference's scripted-draft tests do, tests/mtp_review.rs:23-26), draft length 1..3."""
    from irontimber_b200 import engine as E
    prompt = rng.integers(0, cfg.n_vocab, prompt_len).tolist()
    keep = ("drafted", "accepted", "rejected", "steps", "verify_calls", "single_forwards")

    def timed(fn):
        t0 = time.perf_counter()
        r = fn()
        return time.perf_counter() - t0, r
    eng.generate_mtp_k(prompt[:8], 6, 3); eng.generate_mtp(prompt[:8], 6)       # records the pass graphs of every shape met below
    eng.mtp_prefill(prompt)
    pre_s, _ = timed(lambda: eng.mtp_prefill(prompt))                             # prompt pass with the head's catch-up, common to all runs
    eng.reset()
    plain_s, plain = timed(lambda: eng.generate(prompt, n_tokens))
    res = {"prompt_tokens": prompt_len, "tokens": n_tokens, "prefill_with_head_catch_up_s": pre_s,
           "plain_greedy_tok_s": (n_tokens - 1) / max(plain_s - pre_s, 1e-9)}
    for kd in (1, 2, 3):
        class Scripted:
            def __init__(self, e): self.e, self.i = e, 1
            def __getattr__(self, name): return getattr(self.e, name)
            def mtp_draft_k(self, toks, kk):
                self.e.mtp_draft_k(toks, kk)                 # the head still runs; only its picks are overridden
                return [plain[min(self.i + j, len(plain) - 1)] for j in range(kk)]
            def mtp_rollback(self, keep_rows):
                self.i += keep_rows; return self.e.mtp_rollback(keep_rows)
        k_s, (out_k, st_k) = timed(lambda: E.greedy_mtp_k(Scripted(eng), prompt, n_tokens, kd))
        assert out_k == plain, "speculative decoding must reproduce plain greedy decoding"
        n_s, (out_n, st_n) = timed(lambda: eng.generate_mtp_k(prompt, n_tokens, kd) if kd > 1 else eng.generate_mtp(prompt, n_tokens))
        assert out_n == plain, "speculative decoding must reproduce plain greedy decoding"
        res[f"k{kd}"] = {"scripted_right_drafts": {"tok_s": (n_tokens - 1) / max(k_s - pre_s, 1e-9), **{q: st_k[q] for q in keep if q in st_k}},
                         "random_head": {"tok_s": (n_tokens - 1) / max(n_s - pre_s, 1e-9), **{q: st_n[q] for q in keep if q in st_n}}}
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="b200")
    ap.add_argument("--prompt", type=int, default=512)
    ap.add_argument("--layers", type=int, default=64)
    ap.add_argument("--roofline-only", action="store_true", help="only the k_matvec_t2 sweep on config 1 (the run to put under a profiler for that kernel)")
    ap.add_argument("--sweep", action="store_true", help="config 5: op-level sweep of the ternary product (N x M grid) and the q8 LM head, row-sharded over the ranks when N > 1")
    ap.add_argument("--q8-only", action="store_true", help="only the Q8_0 LM head of config 5 (the run to put under a profiler for k_matvec_q8)")
    ap.add_argument("--decode-only", action="store_true", help="prompt + timed decode steps only (no end-to-end, speculative, roofline or CPU legs): the run to put under a profiler")
    ap.add_argument("--no-extras", action="store_true", help="skip the config 3 / 4 / 5 legs (speculative decoding, prompt lengths, op sweep)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    warmup = max(args.warmup, 3)
    from irontimber_b200.engine import config_27b
    cfg = config_27b(n_layer=args.layers)
    config = {"workload": f"config2: {args.layers}-layer 27B-shape ternary decoder (3 delta-net layers per attention layer), batch 1, greedy decode "
                          f"after a {args.prompt}-token random prompt, f16 KV, ctx 8192",
              "prompt_tokens": args.prompt, "weights_bytes_per_token": step_weight_bytes(cfg),
              "l2": "inputs larger than L2: every step streams its weights (6.8 GB at 64 layers) from HBM; L2 is 126 MB",
              "sharding": "single GPU" if world == 1 else f"one sequence, trunk matrices and LM head split by output rows over {world} GPUs, result slices exchanged over NVLink inside the kernels; "
                                                            f"everything else replicated (side object `replicas`: {world} independent sequences, one engine per GPU, no collective)"}
    base = {"metric": METRIC, "unit": "tok/s", "n_gpus": world if args.impl != "reference" else args.gpus, "steps": args.steps, "warmup": warmup,
            "higher_is_better": True, "scaling": "weak" if world == 1 else "strong", "vs_baseline": None, "dtype": "int8 x 2-bit codes -> int32, f32 epilogue", "data": "synthetic", "config": config}

    if args.impl == "reference":
        if rank != 0:
            return
        base["scaling"] = "weak" if args.gpus == 1 else "strong"      # one CPU whatever N is: the same single sequence
        cb, t_full = cpu_decode_tok_s(args.layers, max(args.steps, 2))
        print(json.dumps(dict(base, impl="reference", value=cb["value"], ms_per_step=t_full * 1e3, cpu_baseline=cb,
                              e2e={"value": cb["value"], "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0})))
        return

    import numpy as np
    import torch
    from irontimber_b200 import _lib
    from irontimber_b200.engine import CudaEngine

    if args.sweep or args.q8_only:
        sweep(args, torch, np, rank, world, local_rank, base, head_only=args.q8_only)
        return
    if args.roofline_only:
        if rank == 0:
            print(json.dumps(dict(base, roofline=matvec_roofline(torch, local_rank, max(args.steps, 3)), roofline_only=True)))
        return

    dist = None
    if world > 1:
        import torch.distributed as dist
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    L = _lib.load()
    dev = f"cuda:{local_rank}"

    def barrier(ctx=None):
        if ctx is not None:
            _lib.check(L.it_sync(ctx))
        torch.cuda.synchronize()
        if dist:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x):
        if not dist:
            return x
        t = torch.tensor([x], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def timed_decode(eng, prompt, steps, sampler=None):
        """Prompt pass, warm-up steps, then `steps` chained greedy steps between CUDA events on the library's stream."""
        ctx = L.it_engine_ctx(eng.h)
        stream = torch.cuda.ExternalStream(L.it_ctx_stream(ctx), device=dev)
        barrier(ctx)
        t0 = time.perf_counter()
        eng.eval_argmax(prompt)
        prefill_s = time.perf_counter() - t0
        eng.decode_steps(warmup)
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

        def region():
            barrier(ctx)
            ev0.record(stream)
            eng.decode_steps(steps, read_last=False)
            ev1.record(stream)
            barrier(ctx)
        if sampler is not None:
            with sampler:
                region()
        else:
            region()
        return max_over_ranks(ev0.elapsed_time(ev1)), prefill_s

    def timed_e2e(eng, prompt, steps):
        """The public generate call: token ids from host memory, every pick read back (4 bytes each way per token), host clock."""
        eng.reset()
        first = eng.eval_argmax(prompt)
        barrier(L.it_engine_ctx(eng.h))
        t0 = time.perf_counter()
        hist = eng.generate([first], steps)
        dt = time.perf_counter() - t0
        assert len(hist) == steps
        return max_over_ranks(dt), [first] + hist

    # the same model and prompt on every rank (seed 7, rng 100): the row-sharded engine must reproduce rank 0's unsharded engine
    prompt = np.random.default_rng(100).integers(0, cfg.n_vocab, args.prompt).tolist()
    clocks = ClockSampler(local_rank)
    sharded = replicas = None
    if world > 1:
        seng = CudaEngine(cfg, seed=7, with_mtp=False, device=local_rank, rank=rank, world=world)
        ms, prefill_s = timed_decode(seng, prompt, args.steps, clocks)
        launches = seng.step_kernels()
        e2e_s, hist = timed_e2e(seng, prompt, args.steps)
        n_par = min(args.steps + 1, 33)
        gathered = [None] * world
        dist.all_gather_object(gathered, hist[:n_par])
        seng.close()
        eng = CudaEngine(cfg, seed=7 + rank, with_mtp=False, device=local_rank)      # rank 0: the same model, unsharded
        rprompt = prompt if rank == 0 else np.random.default_rng(100 + rank).integers(0, cfg.n_vocab, args.prompt).tolist()
        rsteps = min(args.steps, 32)
        rms, _ = timed_decode(eng, rprompt, rsteps)
        parity = None
        if rank == 0:
            eng.reset()
            first = eng.eval_argmax(prompt)
            want = [first] + eng.generate([first], n_par - 1)
            parity = {"tokens_compared": n_par, "ranks_agree": all(g == gathered[0] for g in gathered), "equals_unsharded_engine": gathered[0] == want}
        eng.close()
        replicas = {"value": world * rsteps / (rms / 1e3), "unit": "tok/s", "steps": rsteps, "scaling": "weak",
                    "note": f"{world} independent sequences, one full engine per GPU, no collective"}
        sharded = {"parity": bool(parity and parity["ranks_agree"] and parity["equals_unsharded_engine"]) if rank == 0 else None, "parity_detail": parity,
                   "prefill_tok_s": args.prompt / prefill_s,
                   "exchange": "257 exchanges per token (4 per layer + LM head), each inside the matvec kernel: peer stores of 8-byte value+epoch slots over NVLink, no NCCL call on the data path"}
    else:
        eng = CudaEngine(cfg, seed=7, with_mtp=True, device=local_rank)
        ms, prefill_s = timed_decode(eng, prompt, args.steps, clocks)
        launches = eng.step_kernels()
        if args.decode_only:
            eng.close()
            print(json.dumps(dict(base, value=args.steps / (ms / 1e3), ms_per_step=ms / args.steps, clocks=clocks.summary(), gpu_launches=args.steps * launches,
                                  prefill={"tokens": args.prompt, "seconds": prefill_s, "tok_s": args.prompt / prefill_s, "rows_per_pass": 256}, decode_only=True)))
            return
        e2e_s, step_hist = timed_e2e(eng, prompt, args.steps)
    out = dict(base, value=args.steps / (ms / 1e3), ms_per_step=ms / args.steps, clocks=clocks.summary(), gpu_launches=args.steps * launches, launches_per_step=launches,
               e2e={"value": args.steps / e2e_s, "unit": "tok/s", "h2d_bytes_per_step": 4, "d2h_bytes_per_step": 4, "ms_per_token": e2e_s / args.steps * 1e3},
               prefill={"tokens": args.prompt, "seconds": prefill_s, "tok_s": args.prompt / prefill_s, "rows_per_pass": 256},
               step_weight_gbs=step_weight_bytes(cfg) * args.steps / (ms / 1e3) / 1e9)
    if world == 1 and not args.no_extras:
        rng = np.random.default_rng(300)
        out["prefill_lengths"] = prefill_leg(eng, cfg, rng, (64, 2048, 4096, 7168))                  # config 4
        out["mtp"] = {"note": "decode tok/s = (tokens - 1) / (run time - prefill time); pass graphs recorded beforehand",
                      "prompts": [mtp_leg(eng, cfg, rng, p, 256) for p in (128, 2048)]}               # config 3
    if world == 1:
        eng.close()
        if not args.no_extras:
            # the same workload on the per-op schedule (one launch per op, about 650 launches per token, replayed as a graph):
            # the library reads the switch when an engine is built
            os.environ["IT_STEP_KERNEL"] = "0"
            try:
                peng = CudaEngine(cfg, seed=7, with_mtp=False, device=local_rank)
                psteps = min(args.steps, 64)
                pms, _ = timed_decode(peng, prompt, psteps)
                plaunches = peng.step_kernels()
                pe2e, phist = timed_e2e(peng, prompt, psteps)
                peng.close()
                out["per_op_schedule"] = {"value": psteps / (pms / 1e3), "unit": "tok/s", "steps": psteps, "launches_per_step": plaunches, "e2e": psteps / pe2e,
                                          "same_picks_as_step_kernel": phist == step_hist[:len(phist)], "picks_compared": len(phist),
                                          "note": "the same decode as one kernel launch per op instead of the persistent step kernel (IT_STEP_KERNEL=0)"}
            finally:
                del os.environ["IT_STEP_KERNEL"]
    if sharded:
        out["sharded"] = sharded
        out["replicas"] = replicas
        if not args.no_extras:
            # config 5 on the same ranks: every matrix split by output rows, result slices exchanged inside the kernels
            out["sweep"] = sweep(args, torch, np, rank, world, local_rank, base, emit=False, own_group=False)
    if rank == 0:
        out["roofline"] = matvec_roofline(torch, local_rank, 200)
        out["roofline"]["traffic_source"] = "ncu dram__bytes_read.sum + dram__bytes_write.sum of one launch, from the committed profile summary (not measured in this run)"
        out["cpu_baseline"] = cpu_decode_tok_s(args.layers, 8)[0]
        print(json.dumps(out))
    if dist:
        barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
