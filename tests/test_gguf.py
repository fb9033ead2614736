"""Model files: the library's GGUF reader, its ggml decoders and the engine it builds from a file.

CPU tests (no device): the decoders against the reference's golden ggml vectors (tests/dequant_vs_ggml.rs), the
PTQ1_0 -> PQ2_0 re-coding, the fail-closed parser cases of tests/gguf_malformed.rs, the configuration read from the
metadata (Config::from_gguf, src/model.rs:16-47) and the models the loader refuses.  GPU tests: a small random model
written to disk, loaded through it_engine_create_gguf, read back tensor by tensor and run against the oracle, which is
given the same tensors; everything must be bit-identical.
"""
import ctypes as C
import os
import struct

import numpy as np
import pytest

from tests import gguf_writer as W
from tests.util import bits, tensor_shapes, tiny_config

DATA = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_data")
EFORMAT, EUNSUPPORTED = -6, -7


def _lib():
    from irontimber_b200 import _lib
    return _lib


def dequant(ty, raw, n):
    raw = np.ascontiguousarray(raw, np.uint8)
    out = np.empty(n, np.float32)
    L = _lib().load()
    _lib().check(L.it_gguf_dequant(ty, raw.ctypes.data_as(C.c_void_p), n, out.ctypes.data_as(C.c_void_p)))
    return out


def ptq1_to_pq2(raw):
    raw = np.ascontiguousarray(raw, np.uint8)
    out = np.empty(raw.size // 28 * 34, np.uint8)
    _lib().check(_lib().load().it_gguf_ptq1_to_pq2(raw.ctypes.data_as(C.c_void_p), raw.size // 28, out.ctypes.data_as(C.c_void_p)))
    return out


# ---- decoders -----------------------------------------------------------------------------------------------
@pytest.mark.parametrize("name,ty", [("mtp_q4k3", W.Q4_K), ("mtp_q6k3", W.Q6_K), ("mtp_q80_3", W.Q8_0), ("attn_k3", W.PQ2_0), ("ssm_out4", W.PQ2_0),
                                     ("attn_k3.ptq1", W.PTQ1_0), ("ssm_out4.ptq1", W.PTQ1_0)])
def test_decoders_match_ggml_vectors_bit_exact(name, ty):
    raw = np.fromfile(os.path.join(DATA, name + ".raw"), np.uint8)
    want = np.fromfile(os.path.join(DATA, name + ".f32"), np.float32)
    assert np.array_equal(bits(dequant(ty, raw, want.size)), bits(want))


def test_q6_k_int8_group_form_decodes_to_ggml_values():
    """The writer's restatement of Q8G16::from_ggml's Q6_K arm: scale * q equals ggml's decode bit for bit
    (tests/dequant_vs_ggml.rs:29-32)."""
    raw = np.fromfile(os.path.join(DATA, "mtp_q6k3.raw"), np.uint8)
    want = np.fromfile(os.path.join(DATA, "mtp_q6k3.f32"), np.float32)
    g = np.frombuffer(W.q6_k_to_g16(raw), np.uint8)
    q = g[:want.size].view(np.int8).astype(np.float32)
    sc = g[want.size:].view(np.float32)
    assert np.array_equal(bits(np.repeat(sc, 16) * q), bits(want))


@pytest.mark.parametrize("name", ["attn_k3", "ssm_out4"])
def test_ptq1_recoded_as_pq2_decodes_to_the_same_values(name):
    raw = np.fromfile(os.path.join(DATA, name + ".ptq1.raw"), np.uint8)
    want = np.fromfile(os.path.join(DATA, name + ".ptq1.f32"), np.float32)
    assert np.array_equal(bits(dequant(W.PQ2_0, ptq1_to_pq2(raw), want.size)), bits(want))


def test_plain_types_and_encoders(orc):
    rng = np.random.default_rng(3)
    x = rng.standard_normal(512).astype(np.float32)
    assert np.array_equal(bits(dequant(W.F32, x.view(np.uint8), 512)), bits(x))
    h = x.astype(np.float16)
    assert np.array_equal(bits(dequant(W.F16, h.view(np.uint8), 512)), bits(h.astype(np.float32)))
    b, back = W.to_bf16(x)
    assert np.array_equal(bits(dequant(W.BF16, b, 512)), bits(back))
    # the test writer's PTQ1_0 encoder agrees with the oracle's decoder (pinned to ggml's vectors elsewhere)
    codes = rng.integers(0, 3, (4, 256), dtype=np.uint8)
    d16 = rng.uniform(0.01, 0.05, (4, 2)).astype(np.float16)
    want = (codes.astype(np.float32) - 1).reshape(4, 2, 128) * d16.astype(np.float32)[..., None]
    assert np.array_equal(bits(orc.dequant_ptq1_0(W.encode_ptq1(codes, d16))), bits(want.reshape(-1)))
    assert np.array_equal(bits(orc.dequant_pq2_0(W.encode_pq2(codes, d16))), bits(want.reshape(-1)))
    assert np.array_equal(ptq1_to_pq2(W.encode_ptq1(codes, d16)), W.encode_pq2(codes, d16))
    with pytest.raises(_lib().IronTimberError):
        dequant(W.Q4_K, np.zeros(144, np.uint8), 255)            # not a whole block
    with pytest.raises(_lib().IronTimberError):
        dequant(99, np.zeros(144, np.uint8), 256)                # unknown type


# ---- the container: fail closed ------------------------------------------------------------------------------
def _inspect(path, head=None, ctx=64):
    from irontimber_b200.engine import inspect_gguf
    return inspect_gguf(path, head, ctx)


def _code(path, head=None):
    with pytest.raises(_lib().IronTimberError) as ei:
        _inspect(path, head)
    return ei.value.code, str(ei.value)


def _header(nt, nkv, version=3):
    return b"GGUF" + struct.pack("<IQQ", version, nt, nkv)


def _tensor(dims, ty, off, name="head"):
    return W._s(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims) + struct.pack("<IQ", ty, off)


MALFORMED = {
    "truncated": b"GGUF",
    "bad-magic": b"GGUX" + b"\0" * 60,
    "version-1": _header(0, 0, version=1) + b"\0" * 40,
    "string-overflow": _header(0, 1) + struct.pack("<Q", 2**64 - 1),
    "duplicate-kv": _header(0, 2) + W.kv_bytes("general.alignment", W.U32, 32) * 2,
    "zero-alignment": _header(0, 1) + W.kv_bytes("general.alignment", W.U32, 0),
    "odd-alignment": _header(0, 1) + W.kv_bytes("general.alignment", W.U32, 48),
    "bad-value-type": _header(0, 1) + W._s("k") + struct.pack("<I", 13) + b"\0" * 16,
    "nested-array": _header(0, 1) + W._s("k") + struct.pack("<IIQ", W.ARR, W.ARR, 1) + b"\0" * 16,
    "array-overflow": _header(0, 1) + W._s("k") + struct.pack("<IIQ", W.ARR, W.U8, 2**40),
    "dims-overflow": _header(1, 0) + _tensor([2**64 - 1, 2], 0, 0),
    "zero-dim": _header(1, 0) + _tensor([0], 0, 0) + b"\0" * 64,
    "rank-5": _header(1, 0) + _tensor([1, 1, 1, 1, 1], 0, 0) + b"\0" * 64,
    "offset-overflow": _header(1, 0) + _tensor([32], 0, 2**64 - 1),
    "tensor-past-eof": (_header(1, 0) + _tensor([1024], 0, 0)).ljust(256, b"\0"),
    "quant-row-misaligned": (_header(1, 0) + _tensor([31], 8, 0)).ljust(256, b"\0"),
    "duplicate-tensor": (_header(2, 0) + _tensor([32], 0, 0) + _tensor([32], 0, 0)).ljust(256, b"\0"),
    "count-overflow": _header(2**60, 0),
}


@pytest.mark.parametrize("name", sorted(MALFORMED))
def test_malformed_files_are_refused(tmp_path, name):
    p = tmp_path / (name + ".gguf")
    p.write_bytes(MALFORMED[name])
    code, msg = _code(p)
    assert code == EFORMAT, msg


def test_missing_file_and_empty_path(tmp_path):
    assert _code(tmp_path / "nope.gguf")[0] == EFORMAT
    with pytest.raises(_lib().IronTimberError):
        _inspect("")


# ---- configuration and what the loader refuses ------------------------------------------------------------------
@pytest.fixture(scope="module")
def model_parts(orc):
    from irontimber_b200.engine import ModelConfig
    cfg = tiny_config(ModelConfig)
    parts = W.build_model(np.random.default_rng(5), cfg, tensor_shapes(cfg), dequant, lambda z, s: orc.hadamard_inverse(z, 1024, s), head="same")
    return cfg, parts


def _write(tmp_path, name, kvs, tensors):
    p = tmp_path / name
    W.write_gguf(p, kvs, tensors)
    return p


def test_config_from_metadata(tmp_path, model_parts):
    cfg, (kvs, tensors, _, _, _) = model_parts
    p = _write(tmp_path, "m.gguf", kvs, tensors)
    got, has_mtp, nt, nbytes = _inspect(p, "", ctx=64)
    assert has_mtp and nt == len(tensors) and nbytes == sum(len(bytes(t[3])) for t in tensors)
    for f, _ in cfg._fields_:
        a, b = getattr(got, f), getattr(cfg, f)
        assert (list(a) == list(b)) if f == "rope_sections" else (a == b), f
    got, has_mtp, _, _ = _inspect(p, None, ctx=32)                  # the NextN block is ignored unless asked for
    assert not has_mtp and got.n_layer == cfg.n_layer and got.ctx_len == 32
    got, has_mtp, _, _ = _inspect(p, str(p))                        # naming the trunk file as the head file = appended block
    assert has_mtp


def _edit(kvs, key, value=None, drop=False):
    out = [kv for kv in kvs if kv[0] != key]
    if not drop:
        old = [kv for kv in kvs if kv[0] == key][0]
        out.append((key, old[1], value) + tuple(old[3:]))
    return out


def test_models_outside_the_supported_set_are_refused(tmp_path, model_parts):
    cfg, (kvs, tensors, _, _, _) = model_parts
    il = cfg.n_layer

    def code(kv=None, ts=None, head=""):
        p = _write(tmp_path, "x.gguf", kv or kvs, ts or tensors)
        return _code(p, head)

    assert code(kv=_edit(kvs, "general.architecture", "llama"))[0] == EUNSUPPORTED
    assert code(kv=_edit(kvs, "prism.hadamard.block_size", 512))[0] == EUNSUPPORTED
    assert code(kv=_edit(kvs, "prism.hadamard.block_size", drop=True))[0] == EUNSUPPORTED
    assert code(kv=_edit(kvs, "prism.hadamard.version", 2))[0] == EUNSUPPORTED
    assert code(kv=_edit(kvs, "prism.hadamard.transform", "other"))[0] == EUNSUPPORTED
    assert code(kv=_edit(kvs, "prism.hadamard.sign_mode", "seeded"))[0] == EUNSUPPORTED
    assert code(kv=_edit(kvs, "qwen35.embedding_length", drop=True))[0] == EFORMAT
    c, msg = code(kv=_edit(kvs, "prism.hadamard.sign_widths", [1024, 1024]))
    assert c == EFORMAT and "sign" in msg
    names = [kv for kv in kvs if kv[0] == "prism.hadamard.weight_names"][0][2]
    c, msg = code(kv=_edit(kvs, "prism.hadamard.weight_names", names[1:]))            # a ternary matrix that is not folded
    assert c == EUNSUPPORTED and names[0] in msg
    assert code(kv=_edit(kvs, "prism.hadamard.weight_names", names + ["blk.0.attn_norm.weight"]))[0] == EUNSUPPORTED
    assert code(kv=_edit(kvs, "prism.hadamard.weight_names", names + ["blk.%d.attn_q.weight" % il]))[0] == EUNSUPPORTED   # folded head
    assert code(ts=[t for t in tensors if t[0] != "blk.1.ffn_up.weight"])[0] == EFORMAT                                  # missing tensor
    bad = [(n, [d[0], d[1] - 32] if n == "blk.0.ffn_gate.weight" else d, ty, (raw[:-32 * (d[0] // 128) * (34 if ty == W.PQ2_0 else 28)] if n == "blk.0.ffn_gate.weight" else raw))
           for n, d, ty, raw in tensors]
    assert code(ts=bad)[0] == EFORMAT                                                                                    # wrong shape
    f16 = [(n, d, W.F16 if n == "blk.%d.ffn_up.weight" % il else ty, (np.zeros(d[0] * d[1], np.float16).view(np.uint8) if n == "blk.%d.ffn_up.weight" % il else raw))
           for n, d, ty, raw in tensors]
    c, msg = code(ts=f16)
    assert c == EUNSUPPORTED and "F16" in msg                                                                            # a dense head matrix
    inf = np.zeros(cfg.n_embd * cfg.n_ff // 256 * 210, np.uint8).reshape(-1, 210)
    inf[3, 208:210] = np.array([np.inf], np.float16).view(np.uint8)
    q6 = [(n, d, W.Q6_K if n == "blk.%d.ffn_up.weight" % il else ty, (inf.reshape(-1) if n == "blk.%d.ffn_up.weight" % il else raw)) for n, d, ty, raw in tensors]
    _inspect(_write(tmp_path, "q6.gguf", kvs, q6), "")                   # a Q6_K head matrix is accepted; its scales are checked at load
    own = tensors + [("blk.%d.nextn.shared_head_head.weight" % il, [32], W.F32, np.zeros(32, np.float32).view(np.uint8))]
    assert code(ts=own)[0] == EUNSUPPORTED
    dense = [(n, d, W.F16 if n == "blk.3.attn_k.weight" else ty, (np.zeros(d[0] * d[1], np.float16).view(np.uint8) if n == "blk.3.attn_k.weight" else raw))
             for n, d, ty, raw in tensors]
    assert code(ts=dense)[0] == EUNSUPPORTED                                                                             # a dense trunk matrix
    nan = np.full(cfg.n_embd, np.nan, np.float32).view(np.uint8)
    assert code(ts=[(n, d, ty, nan if n == "blk.%d.nextn.enorm.weight" % il else raw) for n, d, ty, raw in tensors])[0] == EFORMAT
    # no NextN block in the file, but one was asked for; two NextN blocks
    assert code(kv=_edit(_edit(kvs, "qwen35.nextn_predict_layers", 0), "qwen35.block_count", il))[0] == EFORMAT
    assert code(kv=_edit(_edit(kvs, "qwen35.nextn_predict_layers", 2), "qwen35.block_count", il + 2))[0] == EUNSUPPORTED
    # geometry the kernels do not cover is refused by the engine's own validation
    assert code(kv=_edit(kvs, "qwen35.ssm.conv_kernel", 12), head=None)[0] == -1


def test_sidecar_head_must_describe_the_same_model(tmp_path, orc):
    from irontimber_b200.engine import ModelConfig
    cfg = tiny_config(ModelConfig)
    tk, tt, hk, ht, _ = W.build_model(np.random.default_rng(6), cfg, tensor_shapes(cfg), dequant, lambda z, s: orc.hadamard_inverse(z, 1024, s), head="sidecar")
    trunk, head = _write(tmp_path, "trunk.gguf", tk, tt), _write(tmp_path, "head.gguf", hk, ht)
    got, has_mtp, _, _ = _inspect(trunk, head)
    assert has_mtp and got.n_layer == cfg.n_layer
    assert _code(trunk, "")[0] == EFORMAT                                        # the trunk itself holds no NextN block
    other = _write(tmp_path, "head2.gguf", _edit(hk, "qwen35.rope.freq_base", 5e5), ht)
    c, msg = _code(trunk, other)
    assert c == EFORMAT and "rope.freq_base" in msg
    fewer = _write(tmp_path, "head3.gguf", _edit(hk, "tokenizer.ggml.model", drop=True), ht)
    assert _code(trunk, fewer)[0] == EFORMAT
    deeper = _write(tmp_path, "head4.gguf", _edit(hk, "qwen35.block_count", cfg.n_layer + 2), ht)
    assert _code(trunk, deeper)[0] == EFORMAT


# ---- the engine built from a file ------------------------------------------------------------------------------------
def _oracle_from_expect(orc, cfg, expect, with_mtp):
    m = orc.Model(orc.ModelConfig.from_buffer_copy(bytes(cfg)))
    for (name, il), data in [(k, v) for k, v in expect.items() if k != "signs"]:
        if name.startswith("mtp_") and not with_mtp:
            continue
        m.set(name, data, il)
    for s in expect["signs"].values():
        m.set_signs(s)
    return m


def _check_engine(orc, eng, cfg, expect, with_mtp):
    for (name, il), data in [(k, v) for k, v in expect.items() if k != "signs"]:
        if name.startswith("mtp_") and not with_mtp:
            continue
        got = eng.tensor(name, il)
        want = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
        assert np.array_equal(got, want), f"tensor {name} layer {il}"
    for w, s in expect["signs"].items():
        assert np.array_equal(eng.signs(w), s)
    m = _oracle_from_expect(orc, cfg, expect, with_mtp)
    prompt = [5, 77, 901, 13, 640, 2, 999, 0, 321, 45, 600]
    lg = eng.eval(prompt)
    st = m.new_state()
    for i, t in enumerate(prompt):
        want = m.forward_token(st, t, i + 1 == len(prompt), orc.DEVICE_ORDER)
    assert np.array_equal(bits(lg), bits(want))
    eng.reset()
    plain = orc.generate_greedy(m, prompt, 16, orc.DEVICE_ORDER)
    assert eng.generate(prompt, 16) == plain
    if with_mtp:
        want_out, want_stats = orc.greedy_mtp(orc.CpuMtp(m, orc.DEVICE_ORDER), prompt, 16)
        eng.reset()
        out, stats = eng.generate_mtp(prompt, 16)
        assert out == plain == want_out and stats == want_stats
    m.close()


@pytest.mark.gpu
@pytest.mark.parametrize("head,head_embd,explicit,tied,head_type", [("same", True, True, False, "q8_0"), ("sidecar", False, False, False, "mixed"),
                                                                    ("same", True, True, False, "q6_k"), (None, False, True, True, "q8_0")])
def test_engine_from_file_matches_oracle_bit_exact(tmp_path, orc, head, head_embd, explicit, tied, head_type):
    from irontimber_b200.engine import CudaEngine, ModelConfig
    cfg = tiny_config(ModelConfig)
    tk, tt, hk, ht, expect = W.build_model(np.random.default_rng(17), cfg, tensor_shapes(cfg), dequant, lambda z, s: orc.hadamard_inverse(z, 1024, s),
                                           head=head, head_embd=head_embd, explicit_signs=explicit, tied=tied, head_type=head_type)
    trunk = _write(tmp_path, "trunk.gguf", tk, tt)
    hp = None if head is None else "" if head == "same" else str(_write(tmp_path, "head.gguf", hk, ht))
    eng = CudaEngine.from_gguf(trunk, hp, ctx_len=64)
    try:
        assert eng.with_mtp == (head is not None)
        assert eng.as_engine() is eng and (eng.mtp_backend() is eng) == (head is not None)      # ServeEngine, src/engine.rs:69-78
        _check_engine(orc, eng, eng.cfg, expect, head is not None)
    finally:
        eng.close()


@pytest.mark.gpu
def test_refused_file_leaves_no_engine(tmp_path):
    from irontimber_b200.engine import CudaEngine
    p = tmp_path / "bad.gguf"
    p.write_bytes(MALFORMED["duplicate-kv"])
    with pytest.raises(_lib().IronTimberError):
        CudaEngine.from_gguf(p)
