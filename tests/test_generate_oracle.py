"""The oracle's incremental generation against its own one-shot forward, the
way the reference pins it (src/model.rs:4991-5004 generate_step_logits_match_
one_shot_hidden, 5044-5056 generate_step_rejects_past_context_len): logits of
step t equal the head applied to row t of hidden(), exactly."""
import numpy as np
import pytest

from ullis_b200 import synth


def test_generate_step_logits_match_one_shot(oracle):
    data = synth.heron_checkpoint("tiny", batch_size=1)
    m = oracle.HeronOracle(data)
    T = 40
    tokens = synth.zipf_tokens(3, T, m.vocab)
    one_shot = m.logits(tokens, 1, T).reshape(T, m.vocab)
    state = m.generate_state()
    assert state["time"] == 0
    for t in range(T):
        logits = m.generate_step(state, int(tokens[t]))
        assert np.array_equal(logits.reshape(-1), one_shot[t]), t
        assert state["time"] == t + 1


def test_generate_step_rejects_bad_token_and_context_overflow(oracle):
    data = synth.heron_checkpoint("tiny", batch_size=1, context_len=4)
    m = oracle.HeronOracle(data)
    state = m.generate_state()
    with pytest.raises(ValueError, match="vocabulary"):
        m.generate_step(state, m.vocab)
    for t in range(4):
        m.generate_step(state, 5 + t)
    with pytest.raises(ValueError, match="context_len"):
        m.generate_step(state, 1)
