"""Worker functions of the multi-process tests (one process per rank; importable so that multiprocessing can spawn them)."""
import os
import traceback

import numpy as np


def _init(rank, world, port, backend="gloo"):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group(backend, rank=rank, world_size=world)
    return dist


def run_ranks(fn, world, *args, timeout=600):
    """Runs fn(rank, world, port, queue, *args) in `world` spawned processes; returns the per-rank results in rank order."""
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() % 2000)
    procs = [ctx.Process(target=fn, args=(r, world, port, q) + args) for r in range(world)]
    for p in procs:
        p.start()
    out = {}
    try:
        for _ in range(world):
            rank, ok, val = q.get(timeout=timeout)
            if not ok:
                raise AssertionError(f"rank {rank} failed:\n{val}")
            out[rank] = val
    finally:
        for p in procs:
            p.join(timeout=60)
            if p.is_alive():
                p.kill()          # the exact processes started above
    return [out[r] for r in range(world)]


def oracle_sharded_matvec(rank, world, port, q, seed, rows, cols):
    """CPU ranks: every rank computes the oracle matvec of its rows (the library's shard rule) and the slices are
    all-gathered over gloo; the result must be the full matvec on every rank."""
    try:
        import torch
        from oracle import orc
        from irontimber_b200.sharding import shard_range
        from tests.util import synth_pq2
        dist = _init(rank, world, port)
        raw = synth_pq2(seed, rows, cols).reshape(rows, cols // 128 * 34)
        x = np.random.default_rng(seed).standard_normal(cols).astype(np.float32)
        row0, n = shard_range(rows, rank, world)
        mine = orc.matvec_ternary(np.ascontiguousarray(raw[row0:row0 + n]).reshape(-1), n, cols, x)
        parts = [torch.empty(n, dtype=torch.float32) for _ in range(world)]
        dist.all_gather(parts, torch.from_numpy(mine))
        full = np.concatenate([p.numpy() for p in parts])
        want = orc.matvec_ternary(raw.reshape(-1), rows, cols, x)
        pick = int(orc.argmax(full))
        dist.barrier()
        dist.destroy_process_group()
        q.put((rank, True, (bool(np.array_equal(full.view(np.uint32), want.view(np.uint32))), pick, int(orc.argmax(want)))))
    except Exception:
        q.put((rank, False, traceback.format_exc()))


def gpu_sharded_engine(rank, world, port, q, n_layer, prompt, n_predict, with_mtp):
    """GPU ranks: a row-sharded engine per GPU; returns the logits of the prompt, the greedy continuation and, with a
    NextN head, the speculative continuation with its counters."""
    try:
        import torch
        from irontimber_b200.engine import CudaEngine, ModelConfig
        from tests.util import tiny_config
        dist = _init(rank, world, port)
        torch.cuda.set_device(rank)
        eng = CudaEngine(tiny_config(ModelConfig, n_layer=n_layer, ctx_len=128), seed=11, with_mtp=with_mtp, device=rank, rank=rank, world=world)
        try:
            lg = eng.eval(prompt)
            eng.reset()
            hist = eng.generate(prompt, n_predict)
            spec = None
            if with_mtp:
                spec = eng.generate_mtp(prompt, n_predict)
            eng.sync()
            dist.barrier()
        finally:
            eng.close()
        dist.destroy_process_group()
        q.put((rank, True, (lg, hist, spec)))
    except Exception:
        q.put((rank, False, traceback.format_exc()))


def gpu_sharded_gguf_engine(rank, world, port, q, path, head_path, prompt, n_predict):
    """GPU ranks: each loads its rows of every trunk matrix from the same model file; logits, greedy and speculative
    continuations as in gpu_sharded_engine."""
    try:
        import torch
        from irontimber_b200.engine import CudaEngine
        dist = _init(rank, world, port)
        torch.cuda.set_device(rank)
        eng = CudaEngine.from_gguf(path, head_path, ctx_len=128, device=rank, rank=rank, world=world)
        try:
            lg = eng.eval(prompt)
            eng.reset()
            hist = eng.generate(prompt, n_predict)
            spec = eng.generate_mtp(prompt, n_predict) if eng.with_mtp else None
            eng.sync()
            dist.barrier()
        finally:
            eng.close()
        dist.destroy_process_group()
        q.put((rank, True, (lg, hist, spec)))
    except Exception:
        q.put((rank, False, traceback.format_exc()))


def gpu_sharded_matvec(rank, world, port, q, seed, rows, cols, ntok, acc):
    """GPU ranks: one sharded ternary matvec (rows split by the library's rule), results pushed to every rank's arena."""
    try:
        import torch
        from irontimber_b200.backend import CudaBackend
        from irontimber_b200.sharding import shard_range
        dist = _init(rank, world, port)
        torch.cuda.set_device(rank)
        be = CudaBackend(rank, arena_floats=1 << 22)
        try:
            be.attach_peers(rank, world)
            row0, n = shard_range(rows, rank, world)
            w = be.mat_synth_rows(seed, rows, cols, row0, n)
            qx = be.q8_rows(cols, ntok)
            rng = np.random.default_rng(seed)
            X = rng.standard_normal((ntok, cols)).astype(np.float32)
            y0 = rng.standard_normal(ntok * rows).astype(np.float32)
            yo = ((ntok * cols + 63) // 64) * 64
            be.upload(0, X); be.upload(yo, y0)
            be.sync(); dist.barrier()
            be.had_q8(cols, ntok, 0, cols, qx, signs=False, rotate=False)
            for _ in range(3 if not acc else 1):          # repeated ops exercise the epoch counter
                be.mv(w, ntok, qx, yo, rows, acc=acc)
            got = be.download(yo, ntok * rows).reshape(ntok, rows)
            be.sync(); dist.barrier()
            w.close(); qx.close()
        finally:
            be.close()
        dist.destroy_process_group()
        q.put((rank, True, (X, y0, got)))
    except Exception:
        q.put((rank, False, traceback.format_exc()))
