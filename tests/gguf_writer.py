"""Writes GGUF v3 files for the loader tests: a container writer, numpy encoders of the ggml block formats the loader
reads, and a small random qwen35 model (trunk, optional NextN head in the same file or in a sidecar) together with
the tensors the oracle needs to run the same model.

Layouts follow the container the reference reads (src/gguf.rs:99-140), the metadata keys of Config::from_gguf
(src/model.rs:16-47) and load_hadamard (:50-62), and the tensor names of Model::load (src/cpu.rs:91-112) and
MtpHead::load (src/mtp.rs:85-101).
"""
import struct

import numpy as np

F32, F16, Q8_0, Q4_K, Q6_K, BF16, PQ2_0, PTQ1_0 = 0, 1, 8, 12, 14, 30, 142, 143
U8, I8, U16, I16, U32, I32, FLT, BOOL, STR, ARR, U64, I64, F64 = range(13)
_FMT = {U8: "<B", I8: "<b", U16: "<H", I16: "<h", U32: "<I", I32: "<i", FLT: "<f", BOOL: "<B", U64: "<Q", I64: "<q", F64: "<d"}


def _s(s):
    b = s.encode()
    return struct.pack("<Q", len(b)) + b


def _scalar(t, v):
    return _s(v) if t == STR else struct.pack(_FMT[t], v)


def kv_bytes(key, t, v, elem=None):
    """One metadata pair; arrays pass t=ARR, elem=<element type>, v=<list>."""
    out = _s(key) + struct.pack("<I", t)
    if t == ARR:
        out += struct.pack("<IQ", elem, len(v)) + b"".join(_scalar(elem, x) for x in v)
    else:
        out += _scalar(t, v)
    return out


def write_gguf(path, kvs, tensors, align=32, version=3):
    """kvs: list of (key, type, value[, elem]); tensors: list of (name, dims (innermost first), ggml type, bytes)."""
    head = b"GGUF" + struct.pack("<IQQ", version, len(tensors), len(kvs))
    for kv in kvs:
        head += kv_bytes(*kv)
    off = 0
    blobs = []
    for name, dims, ty, data in tensors:
        data = bytes(data)
        head += _s(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims) + struct.pack("<IQ", ty, off)
        pad = (-len(data)) % align
        blobs.append(data + b"\0" * pad)
        off += len(data) + pad
    head += b"\0" * ((-len(head)) % align)
    with open(path, "wb") as f:
        f.write(head + b"".join(blobs))


# ---- block encoders ---------------------------------------------------------------------------------------
def encode_pq2(codes, d16):
    """codes [rows, cols] in 0..3, d16 [rows, cols/128] f16 -> PQ2_0 bytes (f16 scale, then 32 bytes of four 2-bit codes)."""
    rows, cols = codes.shape
    c4 = codes.reshape(rows, cols // 128, 32, 4).astype(np.uint8)
    raw = np.zeros((rows, cols // 128, 34), np.uint8)
    raw[:, :, 0:2] = d16.reshape(rows, cols // 128, 1).view(np.uint8)
    raw[:, :, 2:] = c4[..., 0] | (c4[..., 1] << 2) | (c4[..., 2] << 4) | (c4[..., 3] << 6)
    return raw.reshape(-1)


def _trits_to_byte(d):
    """Five base-3 digits (first most significant; pad missing ones with 0) -> the byte whose digit n is
    ((byte * 3^n mod 256) * 3) >> 8."""
    v = np.zeros(d.shape[:-1], np.uint32)
    for n in range(5):
        v = v * 3 + (d[..., n] if n < d.shape[-1] else 0)
    return ((v * 256 + 242) // 243).astype(np.uint8)


def encode_ptq1(codes, d16):
    """codes [rows, cols] in 0..2 -> PTQ1_0 bytes: 24 bytes of five digits (elements 0..79 digit-major over bytes 0..15,
    elements 80..119 over bytes 16..23), 2 bytes of four digits (elements 120..127 digit-major), f16 scale."""
    rows, cols = codes.shape
    nb = rows * cols // 128
    c = codes.reshape(nb, 128).astype(np.uint32)
    raw = np.zeros((nb, 28), np.uint8)
    raw[:, 0:16] = _trits_to_byte(c[:, 0:80].reshape(nb, 5, 16).transpose(0, 2, 1))
    raw[:, 16:24] = _trits_to_byte(c[:, 80:120].reshape(nb, 5, 8).transpose(0, 2, 1))
    raw[:, 24:26] = _trits_to_byte(c[:, 120:128].reshape(nb, 4, 2).transpose(0, 2, 1))
    raw[:, 26:28] = d16.reshape(nb, 1).view(np.uint8)
    return raw.reshape(-1)


def random_q4_k(rng, rows, cols):
    """Random but well-formed Q4_K blocks (any byte pattern decodes; scales kept small so values stay near +-1)."""
    nb = rows * cols // 256
    raw = rng.integers(0, 256, (nb, 144), dtype=np.uint8)
    raw[:, 0:2] = rng.uniform(0.001, 0.004, nb).astype(np.float16).reshape(nb, 1).view(np.uint8)
    raw[:, 2:4] = rng.uniform(0.0005, 0.002, nb).astype(np.float16).reshape(nb, 1).view(np.uint8)
    return raw.reshape(-1)


def random_q8_0(rng, rows, cols, dlo=0.002, dhi=0.006):
    nb = rows * cols // 32
    raw = np.zeros((nb, 34), np.uint8)
    raw[:, 0:2] = rng.uniform(dlo, dhi, nb).astype(np.float16).reshape(nb, 1).view(np.uint8)
    raw[:, 2:] = rng.integers(-127, 128, (nb, 32)).astype(np.int8).view(np.uint8)
    return raw.reshape(-1)


def random_q6_k(rng, rows, cols):
    """Random well-formed Q6_K blocks: 128 low nibbles, 64 bytes of high bit pairs, 16 int8 sub-block scales, f16 d."""
    nb = rows * cols // 256
    raw = rng.integers(0, 256, (nb, 210), dtype=np.uint8)
    raw[:, 192:208] = rng.integers(-40, 41, (nb, 16)).astype(np.int8).view(np.uint8)
    raw[:, 208:210] = rng.uniform(1e-4, 3e-4, nb).astype(np.float16).reshape(nb, 1).view(np.uint8)
    return raw.reshape(-1)


def q6_k_to_g16(raw):
    """Q6_K blocks -> (int8 values q - 32, one f32 scale per 16 weights = d * sub-block scale), the int8-group form of
    Q8G16::from_ggml (src/quant.rs:245-257), as one byte string: values, then scales."""
    b = np.ascontiguousarray(raw, np.uint8).reshape(-1, 210)
    nb = b.shape[0]
    d = b[:, 208:210].copy().view(np.float16).astype(np.float32)                       # [nb, 1]
    scales = d * b[:, 192:208].view(np.int8).astype(np.float32)                        # [nb, 16]
    q = np.zeros((nb, 2, 4, 32), np.int32)
    for h in range(2):
        ql, qh = b[:, h * 64:h * 64 + 64].astype(np.int32), b[:, 128 + h * 32:160 + h * 32].astype(np.int32)
        q[:, h, 0] = ((ql[:, :32] & 0xF) | ((qh & 3) << 4)) - 32
        q[:, h, 1] = ((ql[:, 32:] & 0xF) | (((qh >> 2) & 3) << 4)) - 32
        q[:, h, 2] = ((ql[:, :32] >> 4) | (((qh >> 4) & 3) << 4)) - 32
        q[:, h, 3] = ((ql[:, 32:] >> 4) | (((qh >> 6) & 3) << 4)) - 32
    return q.astype(np.int8).reshape(-1).view(np.uint8).tobytes() + scales.astype(np.float32).reshape(-1).tobytes()


def to_bf16(x):
    """f32 -> bf16 bytes, round to nearest even; returns (bytes, the f32 values they decode to)."""
    u = np.ascontiguousarray(x, np.float32).view(np.uint32)
    r = ((u + (0x7fff + ((u >> 16) & 1))) >> 16).astype(np.uint16)
    return r.view(np.uint8), (r.astype(np.uint32) << 16).view(np.float32)


# ---- a small model ----------------------------------------------------------------------------------------
LAYER_NAMES = {"attn_norm": "attn_norm.weight", "post_norm": "post_attention_norm.weight", "ffn_gate": "ffn_gate.weight", "ffn_up": "ffn_up.weight",
               "ffn_down": "ffn_down.weight", "qkv": "attn_qkv.weight", "gate": "attn_gate.weight", "conv": "ssm_conv1d.weight", "dt": "ssm_dt.bias",
               "a": "ssm_a", "beta": "ssm_beta.weight", "alpha": "ssm_alpha.weight", "ssm_norm": "ssm_norm.weight", "ssm_out": "ssm_out.weight",
               "q": "attn_q.weight", "k": "attn_k.weight", "v": "attn_v.weight", "o": "attn_output.weight", "q_norm": "attn_q_norm.weight", "k_norm": "attn_k_norm.weight"}
HEAD_NAMES = {"mtp_eh": "nextn.eh_proj.weight", "mtp_q": "attn_q.weight", "mtp_k": "attn_k.weight", "mtp_v": "attn_v.weight", "mtp_o": "attn_output.weight",
              "mtp_gate": "ffn_gate.weight", "mtp_up": "ffn_up.weight", "mtp_down": "ffn_down.weight", "mtp_enorm": "nextn.enorm.weight",
              "mtp_hnorm": "nextn.hnorm.weight", "mtp_attn_norm": "attn_norm.weight", "mtp_post_norm": "post_attention_norm.weight",
              "mtp_q_norm": "attn_q_norm.weight", "mtp_k_norm": "attn_k_norm.weight", "mtp_head_norm": "nextn.shared_head_norm.weight"}
F32_RANGE = {"conv": (-0.5, 0.5), "dt": (-0.5, 0.5), "a": (-1.1, -0.1), "beta": (-0.05, 0.05), "alpha": (-0.05, 0.05)}


def config_kvs(cfg, n_blocks, nextn):
    k = "qwen35."
    return [("general.architecture", STR, "qwen35"), ("general.alignment", U32, 32),
            (k + "block_count", U32, n_blocks), (k + "nextn_predict_layers", U32, nextn),
            (k + "embedding_length", U32, cfg.n_embd), (k + "feed_forward_length", U32, cfg.n_ff),
            (k + "attention.head_count", U32, cfg.n_head), (k + "attention.head_count_kv", U32, cfg.n_head_kv),
            (k + "attention.key_length", U32, cfg.head_dim), (k + "rope.dimension_count", U32, cfg.n_rot),
            (k + "rope.freq_base", FLT, float(cfg.rope_base)), (k + "rope.dimension_sections", ARR, list(cfg.rope_sections), I32),
            (k + "attention.layer_norm_rms_epsilon", FLT, float(cfg.eps)),
            (k + "ssm.conv_kernel", U32, cfg.conv_k), (k + "ssm.state_size", U32, cfg.ssm_state), (k + "ssm.group_count", U32, cfg.ssm_groups),
            (k + "ssm.time_step_rank", U32, cfg.ssm_vheads), (k + "ssm.inner_size", U64, cfg.ssm_inner),
            (k + "full_attention_interval", U32, cfg.full_attn_interval),
            ("tokenizer.ggml.model", STR, "gpt2"), ("tokenizer.ggml.tokens", ARR, ["tok%d" % i for i in range(7)], STR),
            ("tokenizer.ggml.token_type", ARR, [1] * 7, I32)]


def build_model(rng, cfg, shapes, dequant, hadamard_inverse, head="same", head_embd=True, explicit_signs=True, tied=False, head_type="q8_0"):
    """Random weights for `cfg` in a mix of the accepted storage types.

    shapes: tests.util.tensor_shapes(cfg); dequant(ggml_type, bytes, n) -> f32 and hadamard_inverse(row, signs) supply
    the arithmetic for the tensors whose expected values are decoded ones.  head: "same", "sidecar" or None;
    head_type: "q8_0", "q6_k" or "mixed" (alternating) storage of the head's matrices.
    Returns (trunk_kvs, trunk_tensors, head_kvs, head_tensors, expect) where expect maps (name, layer) -> what the oracle
    is given (raw PQ2_0 / Q8_0 bytes or f32 arrays) and expect["signs"] maps width -> sign vector.
    """
    e = cfg.n_embd
    expect, tensors, folded = {}, [], []
    widths = sorted({cfg.n_embd, cfg.ssm_inner, cfg.n_head * cfg.head_dim, cfg.n_ff})
    signs = {w: (np.where(rng.integers(0, 2, w) == 1, 1, -1).astype(np.int8) if explicit_signs else np.ones(w, np.int8)) for w in widths}
    expect["signs"] = {w: s.astype(np.float32) for w, s in signs.items()}
    flip = [0]

    def ternary(gname, key, rows, cols):
        codes = rng.integers(0, 3, (rows, cols), dtype=np.uint8)
        d16 = rng.uniform(0.01, 0.05, (rows, cols // 128)).astype(np.float16)
        expect[key] = encode_pq2(codes, d16)
        flip[0] ^= 1                                           # alternate the two ternary storage types
        tensors.append((gname, [cols, rows], PTQ1_0, encode_ptq1(codes, d16)) if flip[0] else (gname, [cols, rows], PQ2_0, expect[key]))
        folded.append(gname)

    def vector(gname, key, n, name, dims=None, into=None):
        lo, hi = F32_RANGE.get(name, (0.9, 1.1))
        x = rng.uniform(lo, hi, n).astype(np.float32)
        dst = tensors if into is None else into
        if name == "beta":
            h = x.astype(np.float16); expect[key] = h.astype(np.float32); dst.append((gname, dims or [n], F16, h.view(np.uint8)))
        elif name == "alpha":
            b, back = to_bf16(x); expect[key] = back; dst.append((gname, dims or [n], BF16, b))
        else:
            expect[key] = x; dst.append((gname, dims or [n], F32, x.view(np.uint8)))

    for il in range(cfg.n_layer):
        names = ("attn_norm", "post_norm", "ffn_gate", "ffn_up", "ffn_down") + (
            ("qkv", "gate", "conv", "dt", "a", "beta", "alpha", "ssm_norm", "ssm_out") if cfg.is_recurrent(il) else ("q", "k", "v", "o", "q_norm", "k_norm"))
        for n in names:
            kind, r, c = shapes[n]
            g = "blk.%d.%s" % (il, LAYER_NAMES[n])
            if kind == "pq2":
                ternary(g, (n, il), r, c)
            else:
                vector(g, (n, il), r * c, n, dims=[c, r] if r > 1 else [c])
    vector("output_norm.weight", ("output_norm", -1), e, "output_norm")
    if tied:                                                   # one ternary table: latent embedding and LM head
        ternary("token_embd.weight", ("output", -1), cfg.n_vocab, e)
        ty, raw = tensors[-1][2], tensors[-1][3]
        z = dequant(ty, raw, cfg.n_vocab * e).reshape(cfg.n_vocab, e)
    else:
        ternary("output.weight", ("output", -1), cfg.n_vocab, e)
        raw = random_q4_k(rng, cfg.n_vocab, e)
        tensors.append(("token_embd.weight", [e, cfg.n_vocab], Q4_K, raw))
        z = dequant(Q4_K, raw, cfg.n_vocab * e).reshape(cfg.n_vocab, e)
    expect[("tok_embd", -1)] = np.stack([hadamard_inverse(row, expect["signs"][e]) for row in z]).reshape(-1)

    had = [("prism.hadamard.version", U32, 1), ("prism.hadamard.transform", STR, "normalized-sylvester-walsh-hadamard"),
           ("prism.hadamard.block_size", U32, 1024), ("prism.hadamard.gdn_v_grouped", BOOL, int(cfg.gdn_v_grouped)),
           ("prism.hadamard.weight_names", ARR, folded, STR), ("prism.hadamard.inverse_weight_names", ARR, ["token_embd.weight"], STR)]
    if explicit_signs:
        had += [("prism.hadamard.sign_mode", STR, "explicit"), ("prism.hadamard.sign_widths", ARR, widths, U32),
                ("prism.hadamard.sign_values", ARR, [int(v) for w in widths for v in signs[w]], I8)]
    else:
        had += [("prism.hadamard.sign_mode", STR, "none")]

    head_tensors = []
    if head:
        il = cfg.n_layer
        for n, gname in HEAD_NAMES.items():
            kind, r, c = shapes[n]
            g = "blk.%d.%s" % (il, gname)
            if kind == "q8":
                flip[0] ^= 1
                if head_type == "q6_k" or (head_type == "mixed" and flip[0]):
                    raw = random_q6_k(rng, r, c)
                    expect[(n, -1)] = np.frombuffer(q6_k_to_g16(raw), np.uint8)
                    head_tensors.append((g, [c, r], Q6_K, raw))
                else:
                    expect[(n, -1)] = random_q8_0(rng, r, c)
                    head_tensors.append((g, [c, r], Q8_0, expect[(n, -1)]))
            else:
                vector(g, (n, -1), r * c, n, into=head_tensors)
        if head_embd:
            raw = random_q4_k(rng, cfg.n_vocab, e)
            head_tensors.append(("blk.%d.nextn.embed_tokens.weight" % il, [e, cfg.n_vocab], Q4_K, raw))
            expect[("mtp_embd", -1)] = dequant(Q4_K, raw, cfg.n_vocab * e)
        else:
            expect[("mtp_embd", -1)] = expect[("tok_embd", -1)]
    if head == "same":
        return config_kvs(cfg, cfg.n_layer + 1, 1) + had, tensors + head_tensors, None, None, expect
    trunk_kvs = config_kvs(cfg, cfg.n_layer, 0) + had
    if head == "sidecar":
        return trunk_kvs, tensors, config_kvs(cfg, cfg.n_layer + 1, 1) + had, head_tensors, expect
    return trunk_kvs, tensors, None, None, expect
