"""Training step on the device (ullis_cuda_model_train_step) against the CPU
restatement of the reference's step (oracle/train.py; reference
src/model.rs:2827-3020, stop_grad_bits mode).

Loss, valid-target count and which tensors move are exact statements.  The
gradients are FP16-operand tensor-core products on the device and f32 numpy
products in the oracle, so stepped tensors are compared through w + carry (the
f32 value the optimiser tracks, src/precision.rs:106-113) with a tolerance of
GRAD_TOL in clipped-gradient units: |d(w + carry)| <= lr * GRAD_TOL."""
import numpy as np
import pytest

from ullis_b200 import checkpoint as ckpt
from ullis_b200 import cuda, synth
from oracle import train as T

pytestmark = pytest.mark.gpu

GRAD_TOL = 5e-3     # absolute, on gradients that are clipped to [-1, 1] before the step
LOSS_TOL = 1e-3     # absolute, mean CE in nats

CASES = {
    # name: (shape (d, layers, vocab, context, ffn), batch, time, lr, steps)
    "tiny-b2": (synth.CONFIGS["tiny"], 2, 64, 0.05, 3),
    "d128-vocab260": ((128, 2, 260, 128, 512), 2, 128, 0.02, 2),
    "ragged-time-37": ((64, 1, 260, 40, 96), 3, 37, 0.05, 2),
    "reference-tiny-d16": ((16, 1, 260, 32, 64), 1, 32, 0.05, 3),
    # the benchmark model itself (D=512, L=12, vocab 8192, T=2048), one sequence, the benchmark's weight distributions
    "benchmark-model-b1": (synth.CONFIGS["default"], 1, 2048, 0.005, 1),
}


def hamming(a, b):
    return int(np.unpackbits((a ^ b).view(np.uint8)).sum())


# both arithmetic modes at the small shapes; the benchmark model in the tensor-core mode it is benchmarked in
RUNS = [(c, mode) for c in CASES for mode in ("fast", "exact") if not (c.startswith("benchmark") and mode == "exact")]


@pytest.mark.parametrize("case,mode_name", RUNS, ids=[f"{c}-{m}" for c, m in RUNS])
def test_steps_match_the_cpu_restatement(cuda_rt, oracle, case, mode_name):
    shape, B, Tn, lr, steps = CASES[case]
    mode = cuda.MODE_FAST if mode_name == "fast" else cuda.MODE_EXACT
    data = synth.heron_checkpoint(shape, batch_size=B, seed=11, ln_gain_one=not case.startswith("benchmark"))
    cuda_rt.set_mode(mode)
    try:
        ref = T.HeronTrainer(data)
        m = cuda.CudaHeron(cuda_rt, data)
        st = m.train_state()
        tokens = synth.zipf_tokens(5, B * Tn, ref.m.vocab)
        for s in range(steps):
            want = ref.train_step(tokens, tokens, oracle.CE_NO_IGNORE, B, Tn, lr)
            got = st.train_step(tokens, tokens, oracle.CE_NO_IGNORE, B, Tn, lr)
            assert got["n_valid"] == want["n_valid"] == B * (Tn - 1)
            assert abs(got["loss"] - want["loss"]) <= LOSS_TOL, (s, got, want)
            for k in ("flips_head", "flips_cmix", "flips_rosa_o"):
                assert abs(got[k] - want[k]) <= max(2, 0.02 * want[k]), (s, k, got, want)
        for name in ref.fp16_names():
            w = ref.m.t[name]
            a = oracle.fp16_to_f32(w) + ref.residual[name]
            b = oracle.fp16_to_f32(st.read(name, np.uint16, w.size)) + st.read(name + ".residual", np.float32, w.size)
            assert np.abs(a - b).max() <= lr * GRAD_TOL, name
        for prefix in ref.packed_names():
            lat = ref.latent[prefix]
            a = oracle.fp16_to_f32(lat) + ref.residual[prefix + ".latent"]
            b = oracle.fp16_to_f32(st.read(prefix + ".latent", np.uint16, lat.size)) + \
                st.read(prefix + ".latent.residual", np.float32, lat.size)
            assert np.abs(a - b).max() <= lr * GRAD_TOL, prefix
            bits = ref.m.t[prefix + ".bits"]
            got_bits = st.read(prefix + ".bits", np.uint32, bits.size)
            assert hamming(bits, got_bits) <= max(1, lat.size // 1000), prefix
            # the packed bits are the signs of the device's own latents (rebinarize, src/model.rs:878-884)
            assert np.array_equal(got_bits, T.pack_signs(st.read(prefix + ".latent", np.uint16, lat.size), lat.size))
    finally:
        cuda_rt.set_mode(cuda.MODE_FAST)


def test_step_freezes_qkv_and_moves_e_o_head(cuda_rt, oracle):
    # the reference's train_step_stop_grad_freezes_qkv_and_updates_e_o_head (src/model.rs:4690-4720)
    data = synth.heron_checkpoint((16, 1, 260, 32, 64), batch_size=2, seed=3, ln_gain_one=True)
    m = cuda.CudaHeron(cuda_rt, data)
    st = m.train_state()
    d = 16
    frozen = {"blocks.0.rosa.q.bits": (np.uint32, d * d // 32), "blocks.0.rosa.k.bits": (np.uint32, d * d // 32),
              "blocks.0.rosa.v.bits": (np.uint32, d * d // 32), "blocks.0.ln3.weight": (np.uint16, d),
              "blocks.0.rosa.x_q": (np.uint16, d)}
    moving = {"blocks.0.rosa.e": (np.uint16, d), "head.scale": (np.uint16, 260), "head.bias": (np.uint16, 260)}
    before = {k: st.read(k, *v) for k, v in {**frozen, **moving}.items()}
    o_before = (st.read("blocks.0.rosa.o.bits", np.uint32, d * d // 32), st.read("blocks.0.rosa.o.scale", np.uint16, d))
    tokens = np.array([4 + i % 8 for i in range(32)], np.uint32)
    r = st.train_step(tokens, tokens, oracle.CE_NO_IGNORE, 1, 32, 0.05)
    assert np.isfinite(r["loss"]) and r["n_valid"] == 31
    for k, v in frozen.items():
        assert np.array_equal(st.read(k, *v), before[k]), k
    for k, v in moving.items():
        assert not np.array_equal(st.read(k, *v), before[k]), k
    o_after = (st.read("blocks.0.rosa.o.bits", np.uint32, d * d // 32), st.read("blocks.0.rosa.o.scale", np.uint16, d))
    assert not (np.array_equal(o_before[0], o_after[0]) and np.array_equal(o_before[1], o_after[1]))


def test_training_lowers_the_loss_and_the_model_handle_sees_the_new_weights(cuda_rt, oracle):
    # train_step_loss_drops_below_ln_v_without_qkv_bit_grad (src/model.rs:4786-4800), on the device
    data = synth.heron_checkpoint((64, 2, 260, 64, 128), batch_size=2, seed=5, ln_gain_one=True)
    m = cuda.CudaHeron(cuda_rt, data)
    tokens = np.array([4 + i % 4 for i in range(128)], np.uint32)
    first, _, _ = m.forward_ce(tokens, tokens, oracle.CE_NO_IGNORE, 2, 64)
    st = m.train_state()
    losses = [st.train_step(tokens, tokens, oracle.CE_NO_IGNORE, 2, 64, 0.08)["loss"] for _ in range(60)]
    assert abs(losses[0] - first) <= LOSS_TOL          # the step reports the loss BEFORE its update
    assert losses[-1] < np.log(260) - 0.2
    after, _, n = m.forward_ce(tokens, tokens, oracle.CE_NO_IGNORE, 2, 64)
    assert n == 126 and after < losses[-1] + 0.05       # the borrowed model was stepped in place


def test_ignored_labels_and_padding(cuda_rt, oracle):
    shape, B, Tn = (64, 1, 260, 40, 96), 2, 40
    data = synth.heron_checkpoint(shape, batch_size=B, seed=2, ln_gain_one=True)
    ref = T.HeronTrainer(data)
    m = cuda.CudaHeron(cuda_rt, data)
    st = m.train_state()
    tokens = synth.zipf_tokens(9, B * Tn, 260)
    labels = tokens.copy()
    labels.reshape(B, Tn)[:, 25:] = 3        # padded tail of every sequence
    want = ref.train_step(tokens, labels, 3, B, Tn, 0.05)
    got = st.train_step(tokens, labels, 3, B, Tn, 0.05)
    lab2 = labels.reshape(B, Tn)
    assert got["n_valid"] == want["n_valid"] == int((lab2[:, 1:] != 3).sum()) <= B * 24   # id 3 also occurs in the text
    assert abs(got["loss"] - want["loss"]) <= LOSS_TOL
    a = oracle.fp16_to_f32(ref.m.t["head.bias"]) + ref.residual["head.bias"]
    b = oracle.fp16_to_f32(st.read("head.bias", np.uint16, 260)) + st.read("head.bias.residual", np.float32, 260)
    assert np.abs(a - b).max() <= 0.05 * T.HEAD_BIAS_LR_MULT * GRAD_TOL
    # nothing valid: the loss is 0 over 0 targets and no tensor moves
    none = np.full_like(tokens, 3)
    emb = st.read("embedding", np.uint16, 260 * 64)
    r = st.train_step(tokens, none, 3, B, Tn, 0.05)
    assert r["n_valid"] == 0 and r["loss"] == 0.0 and r["flips_head"] == 0
    assert np.array_equal(st.read("embedding", np.uint16, 260 * 64), emb)


def test_the_reference_s_rejections(cuda_rt, oracle):
    data = synth.heron_checkpoint((64, 1, 260, 40, 96), batch_size=2, seed=2)
    m = cuda.CudaHeron(cuda_rt, data)
    st = m.train_state()
    tokens = synth.zipf_tokens(9, 80, 260)
    for lr in (0.0, -0.1, float("nan"), float("inf")):
        with pytest.raises(cuda.UllisCudaError) as e:
            st.train_step(tokens, tokens, oracle.CE_NO_IGNORE, 2, 40, lr)
        assert e.value.code == cuda.ERR_ARG and "positive learning rate" in e.value.message
    with pytest.raises(cuda.UllisCudaError) as e:
        st.train_step(tokens[:2], tokens[:2], oracle.CE_NO_IGNORE, 2, 1, 0.1)
    assert e.value.code == cuda.ERR_ARG
    with pytest.raises(cuda.UllisCudaError) as e:       # batch beyond the configured batch_size
        st.train_step(np.zeros(120, np.uint32), np.zeros(120, np.uint32), oracle.CE_NO_IGNORE, 3, 40, 0.1)
    assert e.value.code == cuda.ERR_SHAPE
    bad = tokens.copy()
    bad[7] = 260
    for tk, lab in ((bad, tokens), (tokens, bad)):
        with pytest.raises(cuda.UllisCudaError) as e:
            st.train_step(tk, lab, oracle.CE_NO_IGNORE, 2, 40, 0.1)
        assert e.value.code == cuda.ERR_SHAPE and "token shape or context length is invalid" in e.value.message
    with pytest.raises(cuda.UllisCudaError) as e:
        st.read("no.such.tensor", np.uint16, 4)
    assert e.value.code == cuda.ERR_ARG
    with pytest.raises(cuda.UllisCudaError) as e:
        st.read("embedding", np.uint16, 4)
    assert e.value.code == cuda.ERR_SHAPE
    # the state still steps after the rejected calls
    assert np.isfinite(st.train_step(tokens, tokens, oracle.CE_NO_IGNORE, 2, 40, 0.1)["loss"])


def test_carry_of_a_resumed_run_is_restored(cuda_rt, oracle):
    cfg = synth.train_config(64, 1, 260, 40, 2, 96)
    tensors = synth.heron_tensors(cfg, seed=3, ln_gain_one=True)
    rng = np.random.default_rng(0)
    n = 260 * 64
    tensors["head.latent"] = synth.f16_bits(rng.uniform(-0.5, 0.5, n))
    tensors["head.bits"] = T.pack_signs(tensors["head.latent"], n)
    tensors["head.latent.residual"] = rng.normal(scale=1e-5, size=n).astype(np.float32)
    tensors["embedding.residual"] = rng.normal(scale=1e-5, size=n).astype(np.float32)
    tensors["blocks.0.rosa.q.latent"] = synth.f16_bits(rng.uniform(-0.5, 0.5, 64 * 64))   # frozen: ignored
    data = ckpt.to_safetensors_bytes(tensors, cfg, step=5)
    m = cuda.CudaHeron(cuda_rt, data)
    st = m.train_state(data)
    assert np.array_equal(st.read("head.latent", np.uint16, n), tensors["head.latent"])
    assert np.array_equal(st.read("head.latent.residual", np.float32, n), tensors["head.latent.residual"])
    assert np.array_equal(st.read("embedding.residual", np.float32, n), tensors["embedding.residual"])
    assert not st.read("ln_out.weight.residual", np.float32, 64).any()
    fresh = st.read("blocks.0.rosa.o.latent", np.uint16, 64 * 64)
    assert np.all(np.abs(np.abs(oracle.fp16_to_f32(fresh)) - T.BINARYCONNECT_INIT_ABS) < 1e-4)
    assert np.array_equal(T.pack_signs(fresh, 64 * 64), tensors["blocks.0.rosa.o.bits"])
    # and a step from that carry matches the restatement started from the same file
    ref = T.HeronTrainer(data)
    tokens = synth.zipf_tokens(4, 80, 260)
    want = ref.train_step(tokens, tokens, oracle.CE_NO_IGNORE, 2, 40, 0.05)
    got = st.train_step(tokens, tokens, oracle.CE_NO_IGNORE, 2, 40, 0.05)
    assert abs(got["loss"] - want["loss"]) <= LOSS_TOL
    assert abs(got["flips_head"] - want["flips_head"]) <= max(2, 0.02 * want["flips_head"])
    a = oracle.fp16_to_f32(ref.latent["head"]) + ref.residual["head.latent"]
    b = oracle.fp16_to_f32(st.read("head.latent", np.uint16, n)) + st.read("head.latent.residual", np.float32, n)
    assert np.abs(a - b).max() <= 0.05 * GRAD_TOL
