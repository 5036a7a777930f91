"""Incremental generation on the device (ullis_cuda_generate_*) against the
oracle: the logits of step t are bit-identical to row t of the one-shot
forward (reference test src/model.rs:4991-5004), for one and for several
sequences advancing in lock step, after a reset, and whatever arithmetic mode
the runtime is in; the reference's error cases leave the state untouched."""
import numpy as np
import pytest

from ullis_b200 import cuda, synth

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", params=[("tiny", 1, 64, False), ("tiny", 3, 37, True), ("small", 2, 48, False)],
                ids=["tiny-b1-full-context", "tiny-gain1-b3", "config0-b2"])
def gen_case(request, oracle):
    name, B, T, gain = request.param
    data = synth.heron_checkpoint(name, batch_size=max(B, 2), ln_gain_one=gain)
    m = oracle.HeronOracle(data)
    tokens = synth.zipf_tokens(17, B * T, m.vocab).reshape(B, T)
    one_shot = m.logits(tokens.reshape(-1), B, T).reshape(B, T, m.vocab)
    return dict(data=data, B=B, T=T, tokens=tokens, one_shot=one_shot, vocab=m.vocab)


@pytest.mark.parametrize("mode", [cuda.MODE_FAST, cuda.MODE_EXACT], ids=["runtime-fast", "runtime-exact"])
def test_generate_matches_one_shot_bit_for_bit(cuda_rt, gen_case, mode):
    cuda_rt.set_mode(mode)
    try:
        m = cuda.CudaHeron(cuda_rt, gen_case["data"])
        state = m.generate_state(gen_case["B"])
        assert state.time == 0
        for t in range(gen_case["T"]):
            logits = m.generate_step(state, gen_case["tokens"][:, t])
            assert logits.shape == (gen_case["B"], gen_case["vocab"])
            assert np.array_equal(logits, gen_case["one_shot"][:, t, :]), t
            assert state.time == t + 1
        # a reset state replays the same logits; so does a second state of the same model
        state.reset()
        assert state.time == 0
        other = m.generate_state(gen_case["B"])
        for t in range(min(gen_case["T"], 9)):
            a = m.generate_step(state, gen_case["tokens"][:, t])
            b = m.generate_step(other, gen_case["tokens"][:, t])
            assert np.array_equal(a, gen_case["one_shot"][:, t, :]) and np.array_equal(a, b), t
        other.close()
        state.close()
        m.close()
    finally:
        cuda_rt.set_mode(cuda.MODE_FAST)


def test_generate_equals_device_one_shot_in_exact_mode(cuda_rt, gen_case):
    cuda_rt.set_mode(cuda.MODE_EXACT)
    try:
        m = cuda.CudaHeron(cuda_rt, gen_case["data"])
        B, T = gen_case["B"], gen_case["T"]
        one = m.logits(gen_case["tokens"].reshape(-1), B, T).reshape(B, T, -1)
        state = m.generate_state(B)
        for t in range(T):
            assert np.array_equal(m.generate_step(state, gen_case["tokens"][:, t]), one[:, t, :]), t
        state.close()
        m.close()
    finally:
        cuda_rt.set_mode(cuda.MODE_FAST)


def test_late_context_of_the_benchmark_model(cuda_rt):
    """The whole 2 048-token context of the benchmark model, two sequences: by the end the suffix-link chains of the
    biased channels are as long as the context, which is where the chain stamping (src/rosa.rs:168-173) is done
    by a warp per stream from the chain kept as an array.  Every step against the device's one-shot forward in
    EXACT mode (itself held to the oracle bit for bit in test_gpu_benchmark_shape)."""
    d, layers, vocab, T, ffn = synth.CONFIGS["default"]
    B = 2
    data = synth.heron_checkpoint("default", batch_size=B)
    tokens = synth.zipf_tokens(23, B * T, vocab).reshape(B, T)
    cuda_rt.set_mode(cuda.MODE_EXACT)
    try:
        m = cuda.CudaHeron(cuda_rt, data)
        one = m.logits(tokens.reshape(-1), B, T).reshape(B, T, vocab)
        state = m.generate_state(B)
        for t in range(T):
            assert np.array_equal(m.generate_step(state, tokens[:, t]), one[:, t, :]), t
        state.close()
        m.close()
    finally:
        cuda_rt.set_mode(cuda.MODE_FAST)


def test_fused_and_unfused_steps_give_the_same_logits(cuda_rt, oracle, monkeypatch):
    """A step runs LayerNorm + time-shift mixes as one kernel, Q / K / V as one launch and relu^2 on the key matvec;
    with ULLIS_CUDA_GEN_UNFUSED each is a kernel of its own, as the one-shot exact path has them.  Same sums either
    way: the logits must be identical bit for bit (and equal to the oracle's one-shot rows)."""
    data = synth.heron_checkpoint("small", batch_size=2)
    m_or = oracle.HeronOracle(data)
    B, T = 2, 24
    tokens = synth.zipf_tokens(29, B * T, m_or.vocab).reshape(B, T)
    one_shot = m_or.logits(tokens.reshape(-1), B, T).reshape(B, T, m_or.vocab)
    m = cuda.CudaHeron(cuda_rt, data)
    fused = m.generate_state(B)
    got = [m.generate_step(fused, tokens[:, t]) for t in range(T)]
    fused.close()
    monkeypatch.setenv("ULLIS_CUDA_GEN_UNFUSED", "1")
    plain = m.generate_state(B)
    for t in range(T):
        a = m.generate_step(plain, tokens[:, t])
        assert np.array_equal(a, got[t]) and np.array_equal(a, one_shot[:, t, :]), t
    plain.close()
    m.close()


def test_generate_error_cases_leave_the_state_unchanged(cuda_rt, oracle):  # src/model.rs:2718-2723, 5044-5056
    data = synth.heron_checkpoint("tiny", batch_size=2, context_len=6)
    ref = oracle.HeronOracle(data)
    m = cuda.CudaHeron(cuda_rt, data)
    with pytest.raises(cuda.UllisCudaError) as e:
        m.generate_state(0)
    assert e.value.code == cuda.ERR_SHAPE
    state = m.generate_state(2)
    tokens = synth.zipf_tokens(5, 12, ref.vocab).reshape(2, 6)
    one_shot = ref.logits(tokens.reshape(-1), 2, 6).reshape(2, 6, -1)
    for t in range(3):
        m.generate_step(state, tokens[:, t])
    with pytest.raises(cuda.UllisCudaError) as e:
        m.generate_step(state, np.array([1, ref.vocab], np.uint32))
    assert e.value.code == cuda.ERR_TOKEN and "vocabulary" in str(e.value) and state.time == 3
    with pytest.raises(cuda.UllisCudaError) as e:
        m.generate_step(state, np.array([1], np.uint32))  # one token for two sequences
    assert e.value.code == cuda.ERR_SHAPE and state.time == 3
    for t in range(3, 6):  # the failed calls consumed nothing
        assert np.array_equal(m.generate_step(state, tokens[:, t]), one_shot[:, t, :]), t
    with pytest.raises(cuda.UllisCudaError) as e:
        m.generate_step(state, tokens[:, 0])
    assert e.value.code == cuda.ERR_SHAPE and "context_len" in str(e.value) and state.time == 6
    state.close()
    m.close()


def test_a_step_that_fails_after_its_kernels_ran_poisons_the_state_until_reset(cuda_rt, monkeypatch):
    """The failure is injected on the host (no GPU fault): step 3 raises after its kernels have advanced the
    device-side automata.  `time` has not moved, so a retry would push position 2 twice; the state must refuse
    further steps until it is reset, and after the reset it must generate exactly what a fresh state does."""
    data = synth.heron_checkpoint("tiny", batch_size=1)
    m = cuda.CudaHeron(cuda_rt, data)
    tokens = synth.zipf_tokens(5, 8, 512)
    fresh = m.generate_state(1)
    want = [fresh.step(tokens[t:t + 1]).copy() for t in range(6)]
    fresh.close()
    monkeypatch.setenv("ULLIS_CUDA_INJECT_GENERATE_FAILURE", "3")
    state = m.generate_state(1)
    monkeypatch.delenv("ULLIS_CUDA_INJECT_GENERATE_FAILURE")
    for t in range(2):
        assert np.array_equal(state.step(tokens[t:t + 1]), want[t])
    with pytest.raises(cuda.UllisCudaError) as e:
        state.step(tokens[2:3])
    assert e.value.code == cuda.ERR_CUDA and "injected" in e.value.message
    assert state.time == 2
    with pytest.raises(cuda.UllisCudaError) as e:      # no silent retry on a state that is out of step with itself
        state.step(tokens[2:3])
    assert e.value.code == cuda.ERR_ARG and "reset" in e.value.message
    state.reset()
    assert state.time == 0
    for t in range(6):
        assert np.array_equal(state.step(tokens[t:t + 1]), want[t]), t
    state.close()
    m.close()
