"""The CPU restatement of the training step (oracle/train.py): the optimiser
steps against hand-derived known answers (the inputs of the reference's
clipped_sgd_fp16_matches_cpu_residual / binaryconnect_sgd_fp16_matches_cpu_magnitude_clip,
src/metal.rs:4006-4042), every backward piece against float64 autograd of the
forward it differentiates, the straight-through vector and the latent-persistence
behaviour the reference holds (tests/binary_linear.rs:13-66), and the behaviours
the reference's own train-step tests assert (src/model.rs:4690-4800)."""
import numpy as np
import pytest
import torch

from ullis_b200 import synth
from oracle import oracle as O
from oracle import train as T


def f16(x):
    return synth.f16_bits(np.asarray(x, np.float32))


def test_clipped_sgd_known_answers():
    # 0.25 - 0.01*0.001 rounds back to 0.25 and the 1e-5 goes to the carry; -1 - 0.005 -> -(1 + 5/1024);
    # 2 + 0.0025 -> 2 + 1/512
    bits, res = T.clipped_sgd(f16([0.25, -1.0, 2.0]), np.zeros(3, np.float32), [0.001, 0.5, -0.25], 0.01)
    assert np.array_equal(bits, f16([0.25, -(1 + 5 / 1024), 2 + 1 / 512]))
    want = np.array([0.25 - np.float32(0.01) * np.float32(0.001) - 0.25,
                     (np.float32(-1.0) - np.float32(0.01) * np.float32(0.5)) + (1 + 5 / 1024),
                     (np.float32(2.0) + np.float32(0.01) * np.float32(0.25)) - (2 + 1 / 512)], np.float32)
    assert np.allclose(res, want, rtol=0, atol=1e-9)
    # the gradient is clipped to [-1, 1] before the learning rate
    bits, _ = T.clipped_sgd(f16([0.0]), np.zeros(1, np.float32), [50.0], 0.5)
    assert np.array_equal(bits, f16([-0.5]))
    # the carry makes sub-ULP steps add up: 2000 steps of 1e-6 move 1.0 (FP16 spacing 2^-11 just below it)
    # by 2e-3, up to the f32 rounding of each step
    bits, res = f16([1.0]), np.zeros(1, np.float32)
    for _ in range(2000):
        bits, res = T.clipped_sgd(bits, res, [1.0], 1e-6)
    assert abs(float(O.fp16_to_f32(bits)[0] + res[0]) - (1.0 - 2e-3)) < 1e-4
    assert O.fp16_to_f32(bits)[0] < 1.0


def test_binaryconnect_sgd_known_answers():
    bits, res = T.binaryconnect_sgd(f16([0.0625, -0.0625, 0.9]), np.zeros(3, np.float32), [1e-5, -1e-6, 2.0], 0.1)
    # tiny steps stay in the carry; the third gradient is clipped to 1: 0.9 - 0.1 = 0.8
    assert np.array_equal(bits, f16([0.0625, -0.0625, 0.8]))
    assert abs(res[0] + 1e-6) < 1e-8 and abs(res[1] - 1e-7) < 1e-8   # f32 rounding next to 0.0625
    # the proxy is clipped to [-1, 1]; zero and non-finite gradients leave the element alone
    bits, res = T.binaryconnect_sgd(f16([0.95, 0.5, 0.5, 0.5]), np.full(4, 0.125, np.float32),
                                    [-1.0, 0.0, np.nan, np.inf], 0.5)
    assert np.array_equal(bits, f16([1.0, 0.5, 0.5, 0.5]))
    assert np.array_equal(res, np.array([0.0, 0.125, 0.125, 0.125], np.float32))


def test_pack_signs_follows_latent_sign_with_minus_zero_as_plus():
    latent = f16([0.01, -0.01, 0.0, -0.0] + [1.0] * 30)
    words = T.pack_signs(latent, 34)
    assert words.size == 2 and words[0] == 0xFFFFFFFD and words[1] == 0x3
    assert np.array_equal(T.unpack_signs(words, 1, 34)[0, :4], [1, -1, 1, 1])


def _t64(a):
    return torch.tensor(np.asarray(a, np.float64), dtype=torch.float64, requires_grad=True)


def test_layer_norm_backward_matches_autograd():
    rng = np.random.default_rng(1)
    rows, c = 7, 24
    x = rng.normal(size=(rows, c)).astype(np.float32)
    gy = rng.normal(size=(rows, c)).astype(np.float32)
    w = f16(rng.normal(size=c))
    gx, gw, gb = T.layer_norm_backward(x.ravel(), gy.ravel(), w, rows, c)
    xt, wt, bt = _t64(x), _t64(O.fp16_to_f32(w)), _t64(np.zeros(c))
    y = torch.nn.functional.layer_norm(xt, (c,), wt, bt, eps=T.LAYER_NORM_EPS)
    y.backward(torch.tensor(gy, dtype=torch.float64))
    assert np.allclose(gx.reshape(rows, c), xt.grad.numpy(), atol=2e-5)
    assert np.allclose(gw, wt.grad.numpy(), atol=2e-5)
    assert np.allclose(gb, bt.grad.numpy(), atol=2e-5)


def test_packed_backward_ste_matches_autograd_of_the_scaled_sign_product():
    rng = np.random.default_rng(2)
    rows, inn, out = 9, 40, 12
    x = rng.normal(size=(rows, inn)).astype(np.float32)
    gy = rng.normal(size=(rows, out)).astype(np.float32)
    bits = synth.bernoulli_words(5, out * inn)
    scale = f16(0.01 + 0.02 * rng.random(out))
    g_w, g_x, g_scale, g_bias = T.packed_backward_ste(x.ravel(), gy.ravel(), bits, scale, rows, inn, out)
    s = T.unpack_signs(bits, out, inn)
    # y = bias + scale * (x . W^T) with W standing in for the signs (straight-through)
    xt, wt, st, bt = _t64(x), _t64(s), _t64(O.fp16_to_f32(scale)), _t64(np.zeros(out))
    y = bt + st * (xt @ wt.T)
    y.backward(torch.tensor(gy, dtype=torch.float64))
    assert np.allclose(g_w, wt.grad.numpy(), atol=1e-5)
    assert np.allclose(g_x, xt.grad.numpy(), atol=1e-5)
    assert np.allclose(g_scale, st.grad.numpy(), atol=1e-4)
    assert np.allclose(g_bias, bt.grad.numpy(), atol=1e-5)


def test_packed_backward_ste_reference_vector():
    """The vector the reference holds for the straight-through gradients
    (tests/binary_linear.rs:13-40): one output over inputs (2, 3), signs (+1, -1), row scale 0.5, gy = 1
    => g_w = (1.0, 1.5), g_x = (0.5, -0.5), g_scale = -1, g_bias = 1."""
    bits = np.array([0b01], np.uint32)                      # weight 0 = +1, weight 1 = -1
    g_w, g_x, g_scale, g_bias = T.packed_backward_ste(np.array([2.0, 3.0], np.float32), np.array([1.0], np.float32),
                                                      bits, f16([0.5]), 1, 2, 1)
    assert np.abs(g_w.ravel() - [1.0, 1.5]).max() < 1e-6
    assert np.abs(g_x.ravel() - [0.5, -0.5]).max() < 1e-6
    assert abs(float(g_scale[0]) + 1.0) < 1e-6 and abs(float(g_bias[0]) - 1.0) < 1e-6
    # the forward of the same layer (tests/binary_linear.rs:3-11): y = 0 + 0.5 * (2 - 3) = -0.5
    y = O.binary_linear(np.array([2.0, 3.0], np.float32), bits, f16([0.5]), f16([0.0]), 1, 2, 1)
    assert abs(float(y[0]) + 0.5) < 1e-6


def test_latent_persists_across_steps_instead_of_reconstructing():
    """tests/binary_linear.rs:42-66: a 1x1 layer, sign +1, scale 0.5, so the latent starts at 0.5; x = 1,
    gy = 1 give g_w = 0.5, and a BinaryConnect step with lr 0.1 moves the latent to 0.45 - it must not snap
    back to scale * sign = 0.5 - and a second step moves it again (to 0.40)."""
    bits = np.array([1], np.uint32)
    latent, residual = f16([0.5]), np.zeros(1, np.float32)
    g_w, _, _, _ = T.packed_backward_ste(np.array([1.0], np.float32), np.array([1.0], np.float32), bits, f16([0.5]),
                                         1, 1, 1)
    assert abs(float(g_w.ravel()[0]) - 0.5) < 1e-6
    latent, residual = T.binaryconnect_sgd(latent, residual, g_w.ravel(), 0.1)
    after_one = float(O.fp16_to_f32(latent)[0])
    assert abs(after_one - 0.5) > 1e-3 and abs(after_one + float(residual[0]) - 0.45) < 1e-6
    latent, residual = T.binaryconnect_sgd(latent, residual, g_w.ravel(), 0.1)
    after_two = float(O.fp16_to_f32(latent)[0])
    assert after_two != after_one and abs(after_two + float(residual[0]) - 0.40) < 1e-6
    assert np.array_equal(T.pack_signs(latent, 1), bits)     # still positive: the packed sign is unchanged


def test_lerp_shift_backward_matches_autograd():
    rng = np.random.default_rng(3)
    b, t, c = 2, 5, 6
    x = rng.normal(size=(b, t, c)).astype(np.float32)
    g = rng.normal(size=(b, t, c)).astype(np.float32)
    mix = f16(rng.random(c))
    xx = O.time_shift_delta(x.ravel(), b, t, c)
    g_x, g_mix = T.lerp_shift_backward(xx, mix, g.ravel(), b, t, c)
    xt, mt = _t64(x), _t64(O.fp16_to_f32(mix))
    prev = torch.cat([torch.zeros(b, 1, c, dtype=torch.float64), xt[:, :-1, :]], 1)
    shifted = xt + (prev - xt) * mt
    shifted.backward(torch.tensor(g, dtype=torch.float64))
    assert np.allclose(g_x.reshape(b, t, c), xt.grad.numpy(), atol=1e-5)
    assert np.allclose(g_mix, mt.grad.numpy(), atol=1e-5)


@pytest.fixture()
def tiny_trainer():
    # the reference's tiny_train_cfg shape: vocab 260, d_model 16, one layer
    return T.HeronTrainer(synth.heron_checkpoint((16, 1, 260, 32, 64), batch_size=2, seed=3, ln_gain_one=True))


def test_fresh_latents_are_plus_minus_the_init_magnitude(tiny_trainer):
    # src/model.rs:4668-4688
    for prefix, latent in tiny_trainer.latent.items():
        v = O.fp16_to_f32(latent)
        assert np.all(np.abs(np.abs(v) - T.BINARYCONNECT_INIT_ABS) < 1e-4)
        assert np.array_equal(T.pack_signs(latent, v.size), tiny_trainer.m.t[prefix + ".bits"])


def test_step_freezes_qkv_and_updates_e_o_head(tiny_trainer):
    # src/model.rs:4690-4720
    t = tiny_trainer.m.t
    frozen = ["blocks.0.rosa.q.bits", "blocks.0.rosa.k.bits", "blocks.0.rosa.v.bits", "blocks.0.ln3.weight",
              "blocks.0.rosa.x_q"]
    before = {k: t[k].copy() for k in frozen + ["blocks.0.rosa.e", "blocks.0.rosa.o.bits", "blocks.0.rosa.o.scale",
                                                "head.scale", "head.bias"]}
    tokens = np.array([4 + i % 8 for i in range(32)], np.uint32)
    r = tiny_trainer.train_step(tokens, tokens, O.CE_NO_IGNORE, 1, 32, 0.05)
    assert np.isfinite(r["loss"]) and r["n_valid"] == 31
    for k in frozen:
        assert np.array_equal(t[k], before[k]), k
    assert not np.array_equal(t["blocks.0.rosa.e"], before["blocks.0.rosa.e"])
    assert (not np.array_equal(t["blocks.0.rosa.o.bits"], before["blocks.0.rosa.o.bits"])
            or not np.array_equal(t["blocks.0.rosa.o.scale"], before["blocks.0.rosa.o.scale"]))
    assert not np.array_equal(t["head.scale"], before["head.scale"])
    assert not np.array_equal(t["head.bias"], before["head.bias"])


def test_head_bias_rises_for_a_repeated_target(tiny_trainer):
    # src/model.rs:4722-4742
    tokens = np.full(32, 7, np.uint32)
    before = O.fp16_to_f32(tiny_trainer.m.t["head.bias"])[7]
    for _ in range(24):
        tiny_trainer.train_step(tokens, tokens, O.CE_NO_IGNORE, 1, 32, 0.05)
    bias = O.fp16_to_f32(tiny_trainer.m.t["head.bias"])
    assert bias[7] > before and bias[7] > bias[20]


def test_loss_drops_below_ln_v(tiny_trainer):
    # src/model.rs:4786-4800
    tokens = np.array([4 + i % 4 for i in range(32)], np.uint32)
    last = np.inf
    for _ in range(80):
        last = tiny_trainer.train_step(tokens, tokens, O.CE_NO_IGNORE, 1, 32, 0.08)["loss"]
    assert last < np.log(260) - 0.2


def test_step_rejects_what_the_reference_rejects(tiny_trainer):
    tokens = np.arange(4, 36, dtype=np.uint32)
    with pytest.raises(ValueError):
        tiny_trainer.train_step(tokens, tokens, O.CE_NO_IGNORE, 1, 32, 0.0)
    with pytest.raises(ValueError):
        tiny_trainer.train_step(tokens[:1], tokens[:1], O.CE_NO_IGNORE, 1, 1, 0.1)


def test_ignored_labels_do_not_train_the_head_on_those_rows(tiny_trainer):
    tokens = np.array([4 + i % 8 for i in range(32)], np.uint32)
    labels = tokens.copy()
    labels[10:] = 3   # ignore id: only the first nine targets count
    r = tiny_trainer.train_step(tokens, labels, 3, 1, 32, 0.05)
    assert r["n_valid"] == 9


def test_carry_tensors_of_a_checkpoint_are_restored():
    cfg = synth.train_config(16, 1, 260, 32, 2, 64)
    tensors = synth.heron_tensors(cfg, seed=3, ln_gain_one=True)
    rng = np.random.default_rng(0)
    tensors["head.latent"] = f16(rng.uniform(-0.5, 0.5, 260 * 16))
    tensors["head.bits"] = T.pack_signs(tensors["head.latent"], 260 * 16)
    tensors["head.latent.residual"] = rng.normal(scale=1e-5, size=260 * 16).astype(np.float32)
    tensors["embedding.residual"] = rng.normal(scale=1e-5, size=260 * 16).astype(np.float32)
    from ullis_b200 import checkpoint as ckpt
    tr = T.HeronTrainer(ckpt.to_safetensors_bytes(tensors, cfg, step=5))
    assert np.array_equal(tr.latent["head"], tensors["head.latent"])
    assert np.array_equal(tr.residual["head.latent"], tensors["head.latent.residual"])
    assert np.array_equal(tr.residual["embedding"], tensors["embedding.residual"])
    assert not tr.residual["ln_out.weight"].any()


def _kaiming_head_checkpoint(d=16, vocab=260):
    """Head as the reference initialises it: zero bias, row scale 1/sqrt(d) (src/model.rs:569-592)."""
    cfg = synth.train_config(d, 1, vocab, 32, 2, 64)
    tensors = synth.heron_tensors(cfg, seed=3, ln_gain_one=True)
    tensors["head.bias"] = np.zeros(vocab, np.uint16)
    tensors["head.scale"] = f16(np.full(vocab, 1.0 / np.sqrt(d)))
    from ullis_b200 import checkpoint as ckpt
    return ckpt.to_safetensors_bytes(tensors, cfg, step=0)


def test_head_unigram_prior_install():
    # unigram_prior_drops_ce_toward_batch_unigram (src/model.rs:4744-4776)
    data = _kaiming_head_checkpoint()
    tokens = np.array([4 + i % 8 for i in range(32)], np.uint32)
    before = T.HeronTrainer(data).train_step(tokens, tokens, O.CE_NO_IGNORE, 1, 32, 1e-8)["loss"]
    tr = T.HeronTrainer(data)
    corpus = np.array([4 + i % 8 for i in range(4096)], np.uint32)
    prior = tr.install_head_unigram_prior(corpus, O.CE_NO_IGNORE)
    assert prior["applied"] and prior["shrunk_kaiming_scale"] and prior["n_targets"] == 4096
    assert prior["bias_rms"] > 0.2
    bias = O.fp16_to_f32(tr.m.t["head.bias"])
    # log((count+1)/(n+V)) minus its mean: seen classes share one value, unseen ones another
    seen, unseen = np.log1p(512.0) - np.log(4096 + 260.0), -np.log(4096 + 260.0)
    mean = (8 * seen + 252 * unseen) / 260
    assert np.allclose(bias[4:12], seen - mean, atol=2e-3) and np.allclose(bias[20:30], unseen - mean, atol=2e-3)
    assert np.allclose(O.fp16_to_f32(tr.m.t["head.scale"]), 0.25 / 4.0, atol=1e-4)
    after = tr.train_step(tokens, tokens, O.CE_NO_IGNORE, 1, 32, 1e-8)["loss"]
    assert after < before - 0.5 and after < np.log(8) + 1.0
    skipped = tr.install_head_unigram_prior(corpus, O.CE_NO_IGNORE)
    assert not skipped["applied"] and skipped["n_targets"] == 0
    with pytest.raises(ValueError):
        T.HeronTrainer(data).install_head_unigram_prior(np.full(8, 3, np.uint32), 3)
