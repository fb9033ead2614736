"""Shared helpers for the tests: seeded synthetic inputs in the reference's formats."""
import numpy as np

M64 = (1 << 64) - 1


def make_pq2(rng, rows, cols, ncodes=3, dlo=0.01, dhi=0.05):
    """Random PQ2_0 rows (src/quant.rs:21-29): returns (raw uint8 [rows*cols/128*34], codes, f16 scales)."""
    nb = cols // 128
    codes = rng.integers(0, ncodes, (rows, cols), dtype=np.uint8)
    d16 = rng.uniform(dlo, dhi, (rows, nb)).astype(np.float16)
    raw = np.zeros((rows, nb, 34), np.uint8)
    raw[:, :, 0:2] = d16.view(np.uint8).reshape(rows, nb, 2)
    c4 = codes.reshape(rows, nb, 32, 4)
    raw[:, :, 2:] = c4[..., 0] | (c4[..., 1] << 2) | (c4[..., 2] << 4) | (c4[..., 3] << 6)
    return raw.reshape(-1), codes, d16


def make_q8_0(rng, rows, cols, dlo=0.002, dhi=0.006):
    """Random ggml Q8_0 rows (src/quant.rs:188-191)."""
    nblk = rows * cols // 32
    raw = np.zeros((nblk, 34), np.uint8)
    raw[:, 0:2] = rng.uniform(dlo, dhi, (nblk, 1)).astype(np.float16).view(np.uint8)
    raw[:, 2:] = rng.integers(-127, 128, (nblk, 32)).astype(np.int8).view(np.uint8)
    return raw.reshape(-1)


def bits(a):
    return np.ascontiguousarray(a, np.float32).view(np.uint32)


# ---- numpy mirror of the library's synthetic-data rule (it_matrix_synth / it_qmatrix_synth) -------
def _mix64(z):
    z = (z ^ (z >> np.uint64(30))) * np.uint64(0xbf58476d1ce4e5b9)
    z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94d049bb133111eb)
    return z ^ (z >> np.uint64(31))


def synth_hash(seed, idx):
    """idx-th output of splitmix64 seeded with `seed` (the reference's RNG, src/sampling.rs:43)."""
    with np.errstate(over="ignore"):
        idx = np.asarray(idx, np.uint64)
        return _mix64(np.uint64(seed & M64) + np.uint64(0x9e3779b97f4a7c15) * (idx + np.uint64(1)))


def synth_pq2(seed, rows, cols, four_codes=False):
    nb = cols // 128
    n = rows * cols
    h = synth_hash(seed, np.arange(n // 2, dtype=np.uint64))
    v = np.empty(n, np.uint32)
    v[0::2] = (h & np.uint64(0xffffffff)).astype(np.uint32)
    v[1::2] = (h >> np.uint64(32)).astype(np.uint32)
    codes = ((v & 3) if four_codes else (v % 3)).astype(np.uint8).reshape(rows, cols)
    hb = synth_hash(seed ^ 0x5ca1e5, np.arange(rows * nb, dtype=np.uint64))
    u = (hb >> np.uint64(40)).astype(np.float32) * np.float32(1.0 / 16777216.0)
    d16 = (np.float32(0.01) + np.float32(0.04) * u).astype(np.float16).reshape(rows, nb)
    raw = np.zeros((rows, nb, 34), np.uint8)
    raw[:, :, 0:2] = d16.view(np.uint8).reshape(rows, nb, 2)
    c4 = codes.reshape(rows, nb, 32, 4)
    raw[:, :, 2:] = c4[..., 0] | (c4[..., 1] << 2) | (c4[..., 2] << 4) | (c4[..., 3] << 6)
    return raw.reshape(-1)


def synth_q8_0(seed, rows, cols):
    n = rows * cols
    h = synth_hash(seed, np.arange(n // 2, dtype=np.uint64))
    q = np.empty(n, np.int8)
    q[0::2] = ((h & np.uint64(0xffffffff)) % np.uint64(255)).astype(np.int64) - 127
    q[1::2] = ((h >> np.uint64(32)) % np.uint64(255)).astype(np.int64) - 127
    hb = synth_hash(seed ^ 0x5ca1e5, np.arange(n // 32, dtype=np.uint64))
    u = (hb >> np.uint64(40)).astype(np.float32) * np.float32(1.0 / 16777216.0)
    d16 = (np.float32(0.002) + np.float32(0.004) * u).astype(np.float16)
    raw = np.zeros((n // 32, 34), np.uint8)
    raw[:, 0:2] = d16.view(np.uint8).reshape(-1, 2)
    raw[:, 2:] = q.view(np.uint8).reshape(-1, 32)
    return raw.reshape(-1)


# ---- small decoder models for the oracle ---------------------------------------------------------------
def tiny_config(cls, n_layer=4, ctx_len=64, n_vocab=1000):
    """A 4-layer model with the 27B's structure (3 delta-net layers + 1 attention layer) at small widths."""
    import ctypes as C
    return cls(n_layer=n_layer, n_embd=1024, n_ff=2048, n_vocab=n_vocab, n_head=4, n_head_kv=2, head_dim=256, n_rot=64,
               rope_base=1e7, rope_sections=(C.c_int32 * 4)(11, 11, 10, 0), eps=1e-6, conv_k=4, ssm_state=128, ssm_groups=2,
               ssm_vheads=8, ssm_inner=1024, full_attn_interval=4, gdn_v_grouped=1, ctx_len=ctx_len)


def tensor_shapes(cfg):
    """name -> (kind, rows, cols) with kind in {'pq2', 'q8', 'f32'}; shapes of src/cpu.rs:97-111 and src/mtp.rs:51-52."""
    e, ff, hd, nh, nkv = cfg.n_embd, cfg.n_ff, cfg.head_dim, cfg.n_head, cfg.n_head_kv
    qk = cfg.ssm_state * cfg.ssm_groups
    cd, inner, nv, sd, kvd, qf = 2 * qk + cfg.ssm_inner, cfg.ssm_inner, cfg.ssm_vheads, cfg.ssm_state, nkv * hd, 2 * nh * hd
    return {"attn_norm": ("f32", 1, e), "post_norm": ("f32", 1, e), "ffn_gate": ("pq2", ff, e), "ffn_up": ("pq2", ff, e), "ffn_down": ("pq2", e, ff),
            "qkv": ("pq2", cd, e), "gate": ("pq2", inner, e), "conv": ("f32", cd, cfg.conv_k), "dt": ("f32", 1, nv), "a": ("f32", 1, nv),
            "beta": ("f32", nv, e), "alpha": ("f32", nv, e), "ssm_norm": ("f32", 1, sd), "ssm_out": ("pq2", e, inner),
            "q": ("pq2", qf, e), "k": ("pq2", kvd, e), "v": ("pq2", kvd, e), "o": ("pq2", e, nh * hd), "q_norm": ("f32", 1, hd), "k_norm": ("f32", 1, hd),
            "tok_embd": ("f32", cfg.n_vocab, e), "output_norm": ("f32", 1, e), "output": ("pq2", cfg.n_vocab, e),
            "mtp_eh": ("q8", e, 2 * e), "mtp_q": ("q8", qf, e), "mtp_k": ("q8", kvd, e), "mtp_v": ("q8", kvd, e), "mtp_o": ("q8", e, nh * hd),
            "mtp_gate": ("q8", ff, e), "mtp_up": ("q8", ff, e), "mtp_down": ("q8", e, ff),
            "mtp_enorm": ("f32", 1, e), "mtp_hnorm": ("f32", 1, e), "mtp_attn_norm": ("f32", 1, e), "mtp_post_norm": ("f32", 1, e),
            "mtp_q_norm": ("f32", 1, hd), "mtp_k_norm": ("f32", 1, hd), "mtp_head_norm": ("f32", 1, e)}


def random_oracle_model(orc, cfg, seed=0, with_mtp=True):
    """An oracle model with numpy-random weights in the synthetic model's ranges (no GPU involved)."""
    rng = np.random.default_rng(seed)
    m = orc.Model(cfg)
    shapes = tensor_shapes(cfg)

    def make(name):
        kind, r, c = shapes[name]
        if kind == "pq2":
            return make_pq2(rng, r, c)[0]
        if kind == "q8":
            return make_q8_0(rng, r, c)
        lo, hi = {"conv": (-0.5, 0.5), "dt": (-0.5, 0.5), "a": (-1.1, -0.1), "beta": (-0.05, 0.05), "alpha": (-0.05, 0.05), "tok_embd": (-1, 1)}.get(name, (0.9, 1.1))
        return rng.uniform(lo, hi, r * c).astype(np.float32)
    for il in range(cfg.n_layer):
        names = ("attn_norm", "post_norm", "ffn_gate", "ffn_up", "ffn_down") + (
            ("qkv", "gate", "conv", "dt", "a", "beta", "alpha", "ssm_norm", "ssm_out") if cfg.is_recurrent(il) else ("q", "k", "v", "o", "q_norm", "k_norm"))
        for n in names:
            m.set(n, make(n), il)
    for n in ("tok_embd", "output_norm", "output"):
        m.set(n, make(n))
    if with_mtp:
        for n in shapes:
            if n.startswith("mtp_"):
                m.set(n, make(n))
    for w in {cfg.n_embd, cfg.ssm_inner, cfg.n_head * cfg.head_dim, cfg.n_ff}:
        m.set_signs(np.where(rng.integers(0, 2, w) == 1, 1.0, -1.0).astype(np.float32))
    return m


def oracle_model_from_engine(orc, eng, with_mtp):
    """Builds the oracle's host-memory model from an engine's device weights (read back through the C ABI)."""
    from irontimber_b200 import engine as E
    cfg = orc.ModelConfig.from_buffer_copy(bytes(eng.cfg))
    m = orc.Model(cfg)
    for il in range(cfg.n_layer):
        for n in E.COMMON_TENSORS + (E.GDN_TENSORS if cfg.is_recurrent(il) else E.ATTN_TENSORS):
            m.set(n, eng.tensor(n, il), il)
    for n in E.GLOBAL_TENSORS + (E.MTP_TENSORS if with_mtp else ()):
        m.set(n, eng.tensor(n))
    for w in {cfg.n_embd, cfg.ssm_inner, cfg.n_head * cfg.head_dim, cfg.n_ff}:
        m.set_signs(eng.signs(w))
    return m


def reference_order_walk(orc, eng, model, prompt, n_steps):
    """Walks the REFERENCE_ORDER greedy history of the oracle (the reference CPU arithmetic as written, src/cpu.rs:168-192)
    and feeds the same tokens to the engine.  At every step returns the reference's top-1 margin, the largest logit
    deviation of the engine, and whether the picks agree.  The engine is teacher-forced along the reference history,
    so one low-margin step cannot hide what follows it."""
    st = model.new_state()
    ref = None
    for i, t in enumerate(prompt):
        ref = model.forward_token(st, t, i + 1 == len(prompt), orc.REFERENCE_ORDER)
    eng.reset()
    got = eng.eval(prompt)
    steps = []
    for _ in range(n_steps):
        top2 = np.partition(ref, -2)[-2:]
        margin = float(top2[1] - top2[0])
        dev = float(np.max(np.abs(ref - got)))
        scale = float(np.max(np.abs(ref)))
        pick_ref, pick_got = orc.argmax(ref), int(np.argmax(got))
        steps.append({"margin": margin, "dev": dev, "rel": dev / scale, "same": pick_ref == pick_got, "pick": pick_ref})
        ref = model.forward_token(st, pick_ref, True, orc.REFERENCE_ORDER)
        got = eng.eval([pick_ref])
    model.free_state(st)
    return steps


def assert_reference_order_history(steps, bound=0.1):
    """The engine's pick equals the reference-order pick at every step whose reference top-1 margin exceeds twice the
    largest logit deviation seen on the walk (the rule the reference applies between its own GPU and CPU paths,
    src/bin/bonsai-tools.rs:247, :278); prints the smallest margin and the largest deviation."""
    dev = max(s["dev"] for s in steps)
    rel = max(s["rel"] for s in steps)
    margin = min(s["margin"] for s in steps)
    decided = [s for s in steps if s["margin"] > 2 * dev]
    print(f"reference-order walk: {len(steps)} steps, min top-1 margin {margin:.4g}, max |dlogit| {dev:.4g} "
          f"({rel:.2e} of the largest logit), {len(decided)} steps decided by margin, {sum(s['same'] for s in steps)} picks equal")
    assert dev <= bound
    assert all(s["same"] for s in decided)
    return dev, rel, margin
