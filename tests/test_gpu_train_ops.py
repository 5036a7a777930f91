"""Op-level training calls of the C ABI (the MetalRuntime methods of the same
names) against the CPU restatement: the optimiser steps bit for bit (as the
reference's clipped_sgd_fp16_matches_cpu_residual and
binaryconnect_sgd_fp16_matches_cpu_magnitude_clip demand of its Metal kernels,
src/metal.rs:4006-4042), the reductions within f32 reordering."""
import numpy as np
import pytest

from ullis_b200 import checkpoint as ckpt
from ullis_b200 import cuda, synth
from oracle import train as T

pytestmark = pytest.mark.gpu


def f16(x):
    return synth.f16_bits(np.asarray(x, np.float32))


def sgd_inputs(n, seed):
    rng = np.random.default_rng(seed)
    w = f16(rng.uniform(-1.2, 1.2, n))
    w[:8] = f16([0.0, -0.0, 1.0, -1.0, 0.999, -0.999, 6e-5, -6e-8])          # zeros, the clip edge, subnormals
    res = (rng.normal(size=n) * 1e-4).astype(np.float32)
    g = (rng.normal(size=n) * rng.choice([1e-6, 1e-3, 0.3, 5.0], n)).astype(np.float32)
    g[8:14] = [0.0, -0.0, np.nan, np.inf, -np.inf, 1e-30]
    return w, res, g


def test_reference_sgd_vectors(cuda_rt):
    # the inputs of the reference's two Metal-vs-CPU tests
    w, r = cuda_rt.clipped_sgd_fp16(f16([0.25, -1.0, 2.0]), np.zeros(3, np.float32), [0.001, 0.5, -0.25], 0.01)
    ww, wr = T.clipped_sgd(f16([0.25, -1.0, 2.0]), np.zeros(3, np.float32), [0.001, 0.5, -0.25], 0.01)
    assert np.array_equal(w, ww) and np.array_equal(r, wr)
    assert np.array_equal(w, f16([0.25, -(1 + 5 / 1024), 2 + 1 / 512]))
    w, r = cuda_rt.binaryconnect_sgd_fp16(f16([0.0625, -0.0625, 0.9]), np.zeros(3, np.float32), [1e-5, -1e-6, 2.0], 0.1)
    ww, wr = T.binaryconnect_sgd(f16([0.0625, -0.0625, 0.9]), np.zeros(3, np.float32), [1e-5, -1e-6, 2.0], 0.1)
    assert np.array_equal(w, ww) and np.array_equal(r, wr)
    assert np.array_equal(w, f16([0.0625, -0.0625, 0.8]))


@pytest.mark.parametrize("n", [1, 31, 32, 33, 1000, 70001])
@pytest.mark.parametrize("lr", [0.005, 0.5])
def test_sgd_ops_are_bit_identical_to_the_cpu_steps(cuda_rt, n, lr):
    w, res, g = sgd_inputs(max(n, 14), n)
    w, res, g = w[:n], res[:n], g[:n]
    finite = np.where(np.isfinite(g), g, 0).astype(np.float32)   # clipped SGD has no non-finite guard: keep it defined
    got = cuda_rt.clipped_sgd_fp16(w, res, finite, lr)
    want = T.clipped_sgd(w, res, finite, lr)
    assert np.array_equal(got[0], want[0]) and np.array_equal(got[1], want[1])
    got = cuda_rt.binaryconnect_sgd_fp16(w, res, g, lr)
    want = T.binaryconnect_sgd(w, res, g, lr)
    assert np.array_equal(got[0], want[0]) and np.array_equal(got[1], want[1])
    for ste in (1.0, 2047.0):
        lat, r2, bits = cuda_rt.apply_latent_sgd(w, res, g, lr, ste)
        with np.errstate(invalid="ignore", over="ignore"):
            wl, wr2 = T.binaryconnect_sgd(w, res, (g * np.float32(ste)).astype(np.float32), lr)
        assert np.array_equal(lat, wl) and np.array_equal(r2, wr2)
        assert np.array_equal(bits, T.pack_signs(wl, n))


def test_empty_and_mismatched_inputs(cuda_rt):
    e16, e32 = np.empty(0, np.uint16), np.empty(0, np.float32)
    assert cuda_rt.clipped_sgd_fp16(e16, e32, e32, 0.1)[0].size == 0
    assert cuda_rt.apply_latent_sgd(e16, e32, e32, 0.1, 1.0)[2].size == 0
    with pytest.raises(cuda.UllisCudaError):
        cuda_rt.clipped_sgd_fp16(f16([1.0, 2.0]), np.zeros(2, np.float32), np.zeros(3, np.float32), 0.1)
    with pytest.raises(cuda.UllisCudaError):
        cuda_rt.rosa_qkv_1bit_bwd_e(np.zeros(5, np.float32), np.zeros(6, np.uint8), 1, 2, 3)
    assert cuda_rt.cmix_relu2_backward(e32, e32).size == 0


@pytest.mark.parametrize("shape", [(1, 1, 1), (2, 37, 48), (3, 300, 64), (1, 2048, 16)])
def test_rosa_e_grad(cuda_rt, shape):
    b, t, c = shape
    rng = np.random.default_rng(b * t + c)
    gy = rng.normal(size=b * t * c).astype(np.float32)
    idx = rng.integers(0, 2, b * t * c).astype(np.uint8)
    got = cuda_rt.rosa_qkv_1bit_bwd_e(gy, idx, b, t, c)
    want = (gy.astype(np.float64) * (2.0 * idx - 1.0)).reshape(b * t, c).sum(0)
    assert np.allclose(got, want, rtol=0, atol=1e-5 * np.sqrt(b * t) * 4)


@pytest.mark.parametrize("n", [1, 3, 4, 1023, 4096 + 5])
def test_relu2_backward_is_exact(cuda_rt, n):
    rng = np.random.default_rng(n)
    x = rng.normal(size=n).astype(np.float32)
    x[: min(n, 2)] = [0.0, -0.0][: min(n, 2)]
    g = rng.normal(size=n).astype(np.float32)
    want = np.where(x > 0, (np.float32(2.0) * x) * g, np.float32(0)).astype(np.float32)   # src/model.rs:1198-1203
    assert np.array_equal(cuda_rt.cmix_relu2_backward(x, g), want)


@pytest.mark.parametrize("rows,c", [(1, 16), (7, 24), (300, 64), (1000, 512)])
def test_layer_norm_backward(cuda_rt, rows, c):
    rng = np.random.default_rng(rows + c)
    x = (rng.normal(size=(rows, c)) * 3 + 1).astype(np.float32)
    gy = rng.normal(size=(rows, c)).astype(np.float32)
    w = f16(1 + 0.1 * rng.normal(size=c))
    gx, gw, gb = cuda_rt.layer_norm_backward(x, gy, w, rows, c)
    wx, ww, wb = T.layer_norm_backward(x.ravel(), gy.ravel(), w, rows, c)
    assert np.allclose(gx, wx, rtol=1e-4, atol=1e-5)
    assert np.allclose(gw, ww, rtol=1e-4, atol=1e-4 * np.sqrt(rows))
    assert np.allclose(gb, wb, rtol=1e-4, atol=1e-4 * np.sqrt(rows))


def test_head_unigram_prior_matches_the_restatement(cuda_rt, oracle):
    d, vocab = 64, 260
    cfg = synth.train_config(d, 1, vocab, 40, 2, 96)
    tensors = synth.heron_tensors(cfg, seed=3, ln_gain_one=True)
    tensors["head.bias"] = np.zeros(vocab, np.uint16)
    tensors["head.scale"] = f16(np.full(vocab, 1.0 / np.sqrt(d)))
    data = ckpt.to_safetensors_bytes(tensors, cfg, step=0)
    ref = T.HeronTrainer(data)
    m = cuda.CudaHeron(cuda_rt, data)
    st = m.train_state()
    corpus = synth.zipf_tokens(3, 5000, vocab)
    corpus[::7] = 3                                   # ignored positions
    want = ref.install_head_unigram_prior(corpus, 3)
    got = st.install_head_unigram_prior(corpus, 3)
    assert got["applied"] and got["shrunk_kaiming_scale"] and got["n_targets"] == want["n_targets"]
    assert abs(got["bias_rms"] - want["bias_rms"]) < 1e-4 and abs(got["scale_rms"] - want["scale_rms"]) < 1e-6
    gb, wb = st.read("head.bias", np.uint16, vocab), ref.m.t["head.bias"]
    # FP16 roundings of the same f32 expression; log1p / log may differ in the last f32 bit between libms
    assert np.abs(gb.astype(np.int32) - wb.astype(np.int32)).max() <= 1
    assert np.array_equal(st.read("head.scale", np.uint16, vocab), ref.m.t["head.scale"])
    assert not st.read("head.bias.residual", np.float32, vocab).any()
    # a fitted prior is left alone; the model's forward now sees it
    again = st.install_head_unigram_prior(corpus, 3)
    assert not again["applied"] and again["n_targets"] == 0
    tokens = corpus[:80].copy()
    tokens[tokens == 3] = 5
    loss_dev, _, _ = m.forward_ce(tokens, tokens, oracle.CE_NO_IGNORE, 2, 40)
    loss_ref, _, _, _ = ref.m.forward_ce(tokens, tokens, oracle.CE_NO_IGNORE, 2, 40)
    assert abs(loss_dev - loss_ref) < 2e-3
    with pytest.raises(cuda.UllisCudaError) as e:
        cuda.CudaHeron(cuda_rt, data).train_state().install_head_unigram_prior(np.full(8, 3, np.uint32), 3)
    assert e.value.code == cuda.ERR_ARG
