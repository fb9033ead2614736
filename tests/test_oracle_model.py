"""CPU-only checks of the oracle's decoder: the two summation orders stay close, the speculative loop
reproduces plain greedy decoding (the reference's own invariant, tests/mtp_tests.rs), and the library's
greedy_mtp passes the reference's loop scenarios (tests/mtp_loop_regressions.rs)."""
import numpy as np
import pytest

from tests.test_oracle_golden import loop_scenarios
from tests.util import random_oracle_model, tiny_config


@pytest.fixture(scope="module")
def tiny(orc):
    cfg = tiny_config(orc.ModelConfig)
    m = random_oracle_model(orc, cfg, seed=3)
    yield m
    m.close()


def test_reference_and_device_order_agree_within_the_reference_bound(orc, tiny):
    """The two orders differ by a few ulp per op, but q8k rounding amplifies that: one activation that lands on the
    other side of a rounding boundary moves a logit by a quantisation step.  The reference accepts 0.02 (8 layers) and
    0.1 (full model) between its own GPU and CPU paths (src/bin/bonsai-tools.rs:247, :278); the same bound is used here,
    and the greedy pick must agree whenever the reference's top-1 margin exceeds twice the deviation."""
    prompt = [5, 77, 901, 13, 640, 2]
    sa, sb = tiny.new_state(), tiny.new_state()
    for t in prompt:
        la = tiny.forward_token(sa, t, True, orc.REFERENCE_ORDER)
        lb = tiny.forward_token(sb, t, True, orc.DEVICE_ORDER)
        assert np.all(np.isfinite(la)) and np.all(np.isfinite(lb))
        dev = float(np.max(np.abs(la - lb)))
        assert dev <= 0.1
        top = np.sort(la)[-2:]
        if top[1] - top[0] > 2 * dev:
            assert orc.argmax(la) == orc.argmax(lb)


@pytest.mark.parametrize("mode", [0, 1])
def test_speculative_loop_equals_plain_greedy(orc, tiny, mode):
    prompt = [9, 8, 7, 300, 2]
    plain = orc.generate_greedy(tiny, prompt, 10, mode)
    b = orc.CpuMtp(tiny, mode)
    out, st = orc.greedy_mtp(b, prompt, 10)
    assert out == plain
    assert st["drafted"] == st["accepted"] + st["rejected"]

    class TrueNext(orc.CpuMtp):   # a draft that is always right: every step accepts (tests/mtp_review.rs:23-26)
        def mtp_draft(self, toks):
            super().mtp_draft(toks)
            return plain[plain_index[0]]
    plain_index = [1]
    b = TrueNext(tiny, mode)
    orig_verify = b.mtp_verify

    def verify(x, d):
        r = orig_verify(x, d)
        plain_index[0] += 2 if r[0] == d else 1
        return r
    b.mtp_verify = verify
    out, st = orc.greedy_mtp(b, prompt, 10)
    assert out == plain and st["rejected"] == 0 and st["accepted"] == st["drafted"] > 0


def test_library_greedy_mtp_passes_the_reference_loop_scenarios():
    from irontimber_b200 import engine
    loop_scenarios(engine.greedy_mtp)
    with pytest.raises(Exception):
        engine.greedy_mtp(None, [], 3)


class _ScriptedK:
    """Wraps a k-draft backend: the head still runs, but the drafts are replaced by a script (true continuation or wrong ids)."""

    def __init__(self, inner, plain, right, vocab):
        self.b, self.plain, self.right, self.vocab, self.i = inner, plain, right, vocab, 1

    def __getattr__(self, name):
        return getattr(self.b, name)

    def mtp_draft_k(self, toks, k):
        self.b.mtp_draft_k(toks, k)
        nxt = [self.plain[min(self.i + j, len(self.plain) - 1)] for j in range(k)]
        return nxt if self.right else [(t + 1) % self.vocab for t in nxt]

    def mtp_rollback(self, keep_rows):
        self.i += keep_rows
        return self.b.mtp_rollback(keep_rows)


@pytest.mark.parametrize("k", [1, 2, 3])
def test_draft_length_k_reproduces_plain_greedy(orc, tiny, k):
    """Draft length k (k = 1: the reference's loop; k > 1: the chained-head extension): whatever the head drafts, the
    output is plain greedy decoding; scripted right drafts are all accepted, scripted wrong ones all rejected."""
    prompt = [9, 8, 7, 300, 2]
    n = 12
    plain = orc.generate_greedy(tiny, prompt, n, orc.DEVICE_ORDER)
    out, st = orc.greedy_mtp_k(orc.CpuMtp(tiny, orc.DEVICE_ORDER), prompt, n, k)
    assert out == plain
    assert st["drafted"] == st["accepted"] + st["rejected"] and st["verify_calls"] == st["steps"] == st["draft_calls"]
    if k == 1:      # same list and counters as the reference's loop
        out1, st1 = orc.greedy_mtp(orc.CpuMtp(tiny, orc.DEVICE_ORDER), prompt, n)
        assert out1 == out and st1 == st
    vocab = tiny.cfg.n_vocab
    out, st = orc.greedy_mtp_k(_ScriptedK(orc.CpuMtp(tiny, orc.DEVICE_ORDER), plain, True, vocab), prompt, n, k)
    assert out == plain and st["rejected"] == 0 and st["accepted"] == st["drafted"] > 0
    assert st["steps"] <= -(-(n - 1) // (k + 1)) + 1          # k + 1 tokens per step
    out, st = orc.greedy_mtp_k(_ScriptedK(orc.CpuMtp(tiny, orc.DEVICE_ORDER), plain, False, vocab), prompt, n, k)
    assert out == plain and st["accepted"] == 0 and st["rejected"] == st["drafted"] > 0


def test_draft_length_k_stops_on_end_of_generation(orc, tiny):
    prompt = [9, 8, 7, 300, 2]
    plain = orc.generate_greedy(tiny, prompt, 12, orc.DEVICE_ORDER)
    eog = plain[5]
    want = plain[:plain.index(eog) + 1]
    for right in (True, False):
        b = _ScriptedK(orc.CpuMtp(tiny, orc.DEVICE_ORDER), plain, right, tiny.cfg.n_vocab)
        out, _ = orc.greedy_mtp_k(b, prompt, 12, 3, is_eog=lambda t: t == eog)
        assert out == want
        # the trunk state holds exactly the emitted tokens but the last: one more forward gives plain greedy's next token
        nxt = b.mtp_single(out[-1])
        if len(want) < len(plain):
            assert nxt == plain[len(want)]


@pytest.mark.parametrize("k", [1, 2, 3])
def test_library_loop_with_draft_length_k_matches_the_oracle_loop(orc, tiny, k):
    """it_greedy_mtp_k (host code of the library, no GPU) over the oracle's CPU backend: same tokens and counters as the
    oracle's own loop, with the head's drafts and with scripted ones, and with an end-of-generation token in the middle."""
    from irontimber_b200 import engine
    prompt = [9, 8, 7, 300, 2]
    n = 12
    plain = orc.generate_greedy(tiny, prompt, n, orc.DEVICE_ORDER)
    want = orc.greedy_mtp_k(orc.CpuMtp(tiny, orc.DEVICE_ORDER), prompt, n, k)
    assert engine.greedy_mtp_k(orc.CpuMtp(tiny, orc.DEVICE_ORDER), prompt, n, k) == want
    for right in (True, False):
        want = orc.greedy_mtp_k(_ScriptedK(orc.CpuMtp(tiny, orc.DEVICE_ORDER), plain, right, tiny.cfg.n_vocab), prompt, n, k)
        got = engine.greedy_mtp_k(_ScriptedK(orc.CpuMtp(tiny, orc.DEVICE_ORDER), plain, right, tiny.cfg.n_vocab), prompt, n, k)
        assert got == want
    eog = plain[5]
    want = orc.greedy_mtp_k(_ScriptedK(orc.CpuMtp(tiny, orc.DEVICE_ORDER), plain, True, tiny.cfg.n_vocab), prompt, n, k, is_eog=lambda t: t == eog)
    got = engine.greedy_mtp_k(_ScriptedK(orc.CpuMtp(tiny, orc.DEVICE_ORDER), plain, True, tiny.cfg.n_vocab), prompt, n, k, is_eog=lambda t: t == eog)
    assert got == want and got[0] == plain[:plain.index(eog) + 1]
