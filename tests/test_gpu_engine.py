"""GPU parity of the decoder engine against the oracle in device order, through the C ABI.

The engine generates its random-init weights on the device; the oracle's host-memory model is built from those same
weights read back through the ABI.  Logits, recurrent / KV state and token histories must be bit-identical to the
oracle's device-order mode (see oracle/oracle_model.cpp for what that mode is), and the speculative loop must give
plain greedy decoding with the oracle's acceptance counts.
"""
import numpy as np
import pytest

from tests.util import assert_reference_order_history, bits, oracle_model_from_engine, reference_order_walk, tiny_config

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def pair(orc):
    from irontimber_b200.engine import CudaEngine, ModelConfig
    eng = CudaEngine(tiny_config(ModelConfig), seed=11, with_mtp=True)
    model = oracle_model_from_engine(orc, eng, with_mtp=True)
    yield eng, model
    model.close(); eng.close()


PROMPT = [5, 77, 901, 13, 640, 2, 999, 0, 321, 45, 600]     # 11 tokens: one pass of 11 rows through the tile kernel


def test_prompt_logits_and_state_bit_exact(orc, pair):
    eng, m = pair
    eng.reset()
    lg = eng.eval(PROMPT)
    st = m.new_state()
    for i, t in enumerate(PROMPT):
        want = m.forward_token(st, t, i + 1 == len(PROMPT), orc.DEVICE_ORDER)
    assert np.array_equal(bits(lg), bits(want))
    assert eng.pos == m.state_pos(st) == len(PROMPT)
    assert np.array_equal(bits(eng.hidden(len(PROMPT) - 1)), bits(m.state_h(st)))      # last row of the pass = last token
    for il in range(eng.cfg.n_layer):
        if eng.cfg.is_recurrent(il):
            assert np.array_equal(bits(eng.state(il, 0)), bits(m.state_read(st, il, 0))), f"conv state layer {il}"
            assert np.array_equal(bits(eng.state(il, 1)), bits(m.state_read(st, il, 1))), f"ssm state layer {il}"
        else:
            assert np.array_equal(bits(eng.state(il, 2)), bits(m.state_read(st, il, 2))), f"K cache layer {il}"
            assert np.array_equal(bits(eng.state(il, 3)), bits(m.state_read(st, il, 3))), f"V cache layer {il}"
    # token by token gives the same bits as the multi-row pass
    eng.reset()
    for t in PROMPT:
        lg1 = eng.eval([t])
    assert np.array_equal(bits(lg1), bits(lg))
    # and stays within the reference's GPU-vs-CPU bound of the reference-order arithmetic (src/bin/bonsai-tools.rs:247)
    st0 = m.new_state()
    for i, t in enumerate(PROMPT):
        ref = m.forward_token(st0, t, i + 1 == len(PROMPT), orc.REFERENCE_ORDER)
    assert np.max(np.abs(ref - lg)) <= 0.1


def test_greedy_history_identical_and_graph_replay(orc, pair):
    eng, m = pair
    want = orc.generate_greedy(m, PROMPT, 24, orc.DEVICE_ORDER)
    eng.reset()
    assert eng.generate(PROMPT, 24) == want
    eng.reset()                                   # the recorded step is reused by a second request
    assert eng.generate(PROMPT[:5], 9) == orc.generate_greedy(m, PROMPT[:5], 9, orc.DEVICE_ORDER)
    eng.reset()                                   # host-driven loop through eval_argmax gives the same history
    t = eng.eval_argmax(PROMPT); hist = [t]
    for _ in range(7):
        t = eng.eval_argmax([t]); hist.append(t)
    assert hist == want[:8]


def test_history_against_the_reference_summation_order(orc, pair):
    """The oracle's REFERENCE_ORDER mode is the reference CPU arithmetic as written (src/cpu.rs:168-192); the engine's
    greedy pick equals its pick at every step that the top-1 margin decides (tests/util.py states the rule)."""
    eng, m = pair
    assert_reference_order_history(reference_order_walk(orc, eng, m, PROMPT, 24))


def test_speculative_decode_equals_plain_greedy_with_oracle_counts(orc, pair):
    from irontimber_b200 import engine as E
    eng, m = pair
    plain = orc.generate_greedy(m, PROMPT, 20, orc.DEVICE_ORDER)
    want_out, want_stats = orc.greedy_mtp(orc.CpuMtp(m, orc.DEVICE_ORDER), PROMPT, 20)
    assert want_out == plain
    out, stats = eng.generate_mtp(PROMPT, 20)
    assert out == plain
    assert stats == want_stats
    # MTP head state after the run matches the oracle's (f32 KV of confirmed pairs)
    # forced-wrong and always-right drafts exercise rollback and acceptance with known counts (tests/mtp_review.rs:18,23-26)
    class Wrong:
        def __init__(self, e): self.e = e
        def __getattr__(self, n): return getattr(self.e, n)
        def mtp_draft(self, toks): return (self.e.mtp_draft(toks) * 0 + self._next_wrong())
    idx = [1]
    w = Wrong(eng)
    w._next_wrong = lambda: (plain[idx[0]] + 1) % eng.cfg.n_vocab
    orig = eng.mtp_verify
    def verify(x, d):
        r = orig(x, d); idx[0] += 2 if r[0] == d else 1; return r
    w.mtp_verify = verify
    out, st = E.greedy_mtp(w, PROMPT, 12)
    assert out == plain[:12] and st["accepted"] == 0 and st["rejected"] == st["drafted"] > 0
    idx[0] = 1
    w._next_wrong = lambda: plain[idx[0]]
    out, st = E.greedy_mtp(w, PROMPT, 12)
    assert out == plain[:12] and st["rejected"] == 0 and st["accepted"] == st["drafted"] > 0


def test_long_prompt_in_several_passes_bit_exact(orc):
    """A 300-token prompt runs as one pass of 256 rows and one of 44 (prefill_chunks, src/vk/mod.rs:130-134, with a larger
    chunk): logits, the greedy continuation and the speculative loop with its head catch-up across passes equal the
    token-by-token oracle."""
    from irontimber_b200.engine import CudaEngine, ModelConfig
    eng = CudaEngine(tiny_config(ModelConfig, ctx_len=352), seed=23, with_mtp=True)
    m = oracle_model_from_engine(orc, eng, with_mtp=True)
    try:
        prompt = [int(t) for t in np.random.default_rng(9).integers(0, eng.cfg.n_vocab, 300)]
        lg = eng.eval(prompt)
        st = m.new_state()
        for i, t in enumerate(prompt):
            want = m.forward_token(st, t, i + 1 == len(prompt), orc.DEVICE_ORDER)
        assert np.array_equal(bits(lg), bits(want))
        for il in range(eng.cfg.n_layer):
            kinds = (0, 1) if eng.cfg.is_recurrent(il) else (2, 3)
            for kind in kinds:
                assert np.array_equal(bits(eng.state(il, kind)), bits(m.state_read(st, il, kind))), f"state {kind} of layer {il}"
        plain = orc.generate_greedy(m, prompt, 10, orc.DEVICE_ORDER)
        eng.reset()
        assert eng.generate(prompt, 10) == plain
        want_out, want_stats = orc.greedy_mtp(orc.CpuMtp(m, orc.DEVICE_ORDER), prompt, 10)
        out, stats = eng.generate_mtp(prompt, 10)
        assert out == plain == want_out and stats == want_stats
    finally:
        m.close(); eng.close()


@pytest.mark.parametrize("k", [1, 2, 3])
def test_draft_length_k_equals_plain_greedy_with_oracle_counts(orc, pair, k):
    """Draft length k (k > 1: chained head steps, k + 1 verification rows, rollback to the first mismatch): tokens and
    counters identical to the oracle's loop, which is plain greedy decoding; scripted right drafts are all accepted."""
    eng, m = pair
    n = 14
    plain = orc.generate_greedy(m, PROMPT, n, orc.DEVICE_ORDER)
    want_out, want_stats = orc.greedy_mtp_k(orc.CpuMtp(m, orc.DEVICE_ORDER), PROMPT, n, k)
    assert want_out == plain
    out, stats = eng.generate_mtp_k(PROMPT, n, k)
    assert out == plain and stats == want_stats
    if k == 1:
        assert eng.generate_mtp(PROMPT, n) == (out, stats)

    class Right:                                   # the head runs, its drafts are replaced by the true continuation
        def __init__(self, e): self.e, self.i = e, 1
        def __getattr__(self, name): return getattr(self.e, name)
        def mtp_draft_k(self, toks, kk):
            self.e.mtp_draft_k(toks, kk)
            return [plain[min(self.i + j, n - 1)] for j in range(kk)]
        def mtp_rollback(self, keep):
            self.i += keep; return self.e.mtp_rollback(keep)
    out, st = orc.greedy_mtp_k(Right(eng), PROMPT, n, k)
    assert out == plain and st["rejected"] == 0 and st["accepted"] == st["drafted"] > 0


def test_engine_rejects_bad_requests_without_touching_state(pair):
    from irontimber_b200 import _lib
    eng, _ = pair
    eng.reset()
    with pytest.raises(_lib.IronTimberError):
        eng.eval([eng.cfg.n_vocab])                       # out-of-vocabulary id (tests/review_regressions.rs:14)
    with pytest.raises(_lib.IronTimberError):
        eng.eval(list(range(eng.cfg.ctx_len + 1)))        # context overflow is an error, not an abort
    assert eng.pos == 0


def test_bad_geometry_fails_before_device_work():
    import ctypes as C
    from irontimber_b200 import _lib
    from irontimber_b200.engine import ModelConfig
    cfg = tiny_config(ModelConfig); cfg.n_embd = 1000
    h = C.c_void_p()
    assert _lib.load().it_engine_create_synth(0, C.byref(cfg), 1, 0, C.byref(h)) == -1


def test_recorded_and_direct_small_passes_agree(orc, monkeypatch):
    """Passes of up to eight rows replay a recorded graph by default; IT_PASS_GRAPHS=0 issues the same launches one by
    one.  Logits, picks, speculative histories and counters must not depend on the choice."""
    from irontimber_b200.engine import CudaEngine, ModelConfig
    results = []
    for flag in ("1", "0"):
        monkeypatch.setenv("IT_PASS_GRAPHS", flag)
        eng = CudaEngine(tiny_config(ModelConfig), seed=31, with_mtp=True)
        try:
            lg = eng.eval(PROMPT[:3])                       # one recorded 3-row pass / three direct rows
            lg2 = eng.eval([PROMPT[3]])
            eng.reset()
            out1, st1 = eng.generate_mtp(PROMPT, 14)
            out3, st3 = eng.generate_mtp_k(PROMPT, 14, 3)
            eng.reset()
            with pytest.raises(Exception):
                eng.eval([eng.cfg.n_vocab])                 # out-of-vocabulary id: refused before any device work
            assert eng.pos == 0
            results.append((bits(lg).copy(), bits(lg2).copy(), out1, st1, out3, st3))
        finally:
            eng.close()
    a, b = results
    assert np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1])
    assert a[2:] == b[2:]


def test_context_capacity_is_enforced_on_every_path(orc):
    """A full context refuses further tokens before any device work, on the recorded small-pass path, on the direct
    path and in the generation loops (the reference asserts pos + n <= ctx_len, src/vk/mod.rs:765)."""
    from irontimber_b200 import _lib
    from irontimber_b200.engine import CudaEngine, ModelConfig
    eng = CudaEngine(tiny_config(ModelConfig, ctx_len=16), seed=5, with_mtp=True)
    try:
        eng.eval(list(range(16)), want_logits=False)          # fills the context in one 16-row pass
        assert eng.pos == 16
        for toks in ([1], [1, 2, 3], list(range(12))):         # recorded one- and three-row passes, a direct 12-row pass
            with pytest.raises(_lib.IronTimberError):
                eng.eval(toks)
            assert eng.pos == 16
        eng.reset()
        with pytest.raises(_lib.IronTimberError):
            eng.generate(list(range(10)), 8)                   # 10 + 8 - 1 > 16
        eng.reset()
        assert len(eng.generate(list(range(10)), 7)) == 7      # exactly fills it
    finally:
        eng.close()


def test_step_kernel_and_per_op_schedule_agree(orc, monkeypatch):
    """A single-row pass runs as one persistent kernel by default; IT_STEP_KERNEL=0 runs the same pass op by op.  Logits,
    picks, histories and state must not depend on the choice."""
    from irontimber_b200.engine import CudaEngine, ModelConfig
    results = []
    for flag in ("1", "0"):
        monkeypatch.setenv("IT_STEP_KERNEL", flag)
        eng = CudaEngine(tiny_config(ModelConfig), seed=41, with_mtp=True)
        try:
            eng.eval(PROMPT[:7], want_logits=False)
            lgs = [bits(eng.eval([t])).copy() for t in PROMPT[7:]]
            hist = eng.generate(PROMPT[:3], 20)
            n_kernels = eng.step_kernels()
            states = [bits(eng.state(il, k)).copy() for il in range(eng.cfg.n_layer) for k in ((0, 1) if eng.cfg.is_recurrent(il) else (2, 3))]
            out3, st3 = eng.generate_mtp_k(PROMPT, 14, 3)
            results.append((lgs, hist, states, out3, st3, n_kernels))
        finally:
            eng.close()
    a, b = results
    assert a[5] == 1 and b[5] > 10
    assert all(np.array_equal(x, y) for x, y in zip(a[0], b[0]))
    assert a[1] == b[1] and a[3:5] == b[3:5]
    assert all(np.array_equal(x, y) for x, y in zip(a[2], b[2]))


def test_prompt_of_several_full_passes_bit_exact(orc):
    """A 1100-token prompt is four 256-row passes and one of 76 rows, enqueued back to back while the device still works on
    the first: every pass must see its own token ids (the host stages them in a ring of pinned blocks).  Logits, state and
    the continuation (attention over more K / V tiles than the step kernel's ring holds) equal the token-by-token oracle."""
    from irontimber_b200.engine import CudaEngine, ModelConfig
    eng = CudaEngine(tiny_config(ModelConfig, ctx_len=1152), seed=43, with_mtp=False)
    m = oracle_model_from_engine(orc, eng, with_mtp=False)
    try:
        prompt = [int(t) for t in np.random.default_rng(77).integers(0, 1000, 1100)]
        st = m.new_state()
        for i, t in enumerate(prompt):
            want = m.forward_token(st, t, i + 1 == len(prompt), orc.DEVICE_ORDER)
        for _ in range(3):              # the hazard is one of timing: more than one try
            eng.reset()
            lg = eng.eval(prompt)
            assert np.array_equal(bits(lg), bits(want))
            for il in range(eng.cfg.n_layer):
                for kind in ((0, 1) if eng.cfg.is_recurrent(il) else (2, 3)):
                    assert np.array_equal(bits(eng.state(il, kind)), bits(m.state_read(st, il, kind))), f"state {kind} of layer {il}"
        eng.reset()
        assert eng.generate(prompt, 12) == orc.generate_greedy(m, prompt, 12, orc.DEVICE_ORDER)
    finally:
        m.close(); eng.close()


def test_step_kernel_matches_the_per_op_schedule_at_long_positions(monkeypatch):
    """Decode steps after a 330-token prompt: the attention block of the step kernel then walks more K tiles and V chunks
    than its ring holds and crosses a 32-position tile boundary.  Picks, logits and caches equal the per-op schedule's."""
    from irontimber_b200.engine import CudaEngine, ModelConfig
    prompt = [int(t) for t in np.random.default_rng(77).integers(0, 1000, 330)]
    results = []
    for flag in ("1", "0"):
        monkeypatch.setenv("IT_STEP_KERNEL", flag)
        eng = CudaEngine(tiny_config(ModelConfig, ctx_len=448), seed=43, with_mtp=False)
        try:
            first = eng.eval_argmax(prompt)
            hist = [first] + eng.generate([first], 40)
            lg = bits(eng.eval([hist[-1]])).copy()
            states = [bits(eng.state(il, k)).copy() for il in range(eng.cfg.n_layer) for k in ((0, 1) if eng.cfg.is_recurrent(il) else (2, 3))]
            results.append((hist, lg, states))
        finally:
            eng.close()
    a, b = results
    assert a[0] == b[0] and np.array_equal(a[1], b[1])
    assert all(np.array_equal(x, y) for x, y in zip(a[2], b[2]))
