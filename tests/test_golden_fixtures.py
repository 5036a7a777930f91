"""Committed golden fixtures (tests/golden/*.npz, written by
tests/golden/make_golden.py): the oracle must still reproduce them on CPU,
and the CUDA path must match them on a GPU without consulting the oracle."""
import os

import numpy as np
import pytest

from conftest import pack_plane
from ullis_b200 import cuda, synth

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def test_oracle_reproduces_sam_fixture(oracle):
    g = np.load(os.path.join(GOLD, "sam_streams.npz"))
    T = int(g["T"])
    for kind in ("iid", "biased", "periodic"):
        q, k, v, idx = (np.unpackbits(g[f"{kind}_{m}"], axis=1)[:, :T] for m in ("q", "k", "v", "idx"))
        for s in range(q.shape[0]):
            assert np.array_equal(oracle.rosa_qkv_ref(q[s], k[s], v[s]), idx[s])


@pytest.mark.parametrize("variant,gain", [("literal", False), ("gain1", True)])
def test_oracle_reproduces_heron_fixture(oracle, variant, gain):
    g = np.load(os.path.join(GOLD, "heron_tiny.npz"))
    m = oracle.HeronOracle(synth.heron_checkpoint("tiny", batch_size=2, seed=7, ln_gain_one=gain))
    taps = {}
    mean, n_valid, row_loss, _ = m.forward_ce(g[f"{variant}_tokens"], g[f"{variant}_labels"], 3, 2, 64, taps=taps)
    assert n_valid == int(g[f"{variant}_n_valid"]) and np.float32(mean) == g[f"{variant}_mean"]
    assert np.array_equal(row_loss, g[f"{variant}_row_loss"])
    assert np.array_equal(taps["hidden"], g[f"{variant}_hidden"])
    for l in range(m.layers):
        assert np.array_equal(np.packbits(taps[f"{l}.idx"]), g[f"{variant}_idx{l}"])


@pytest.mark.gpu
def test_cuda_sam_matches_fixture(cuda_rt):
    g = np.load(os.path.join(GOLD, "sam_streams.npz"))
    T = int(g["T"])
    for kind in ("iid", "biased", "periodic"):
        q, k, v, idx = (np.unpackbits(g[f"{kind}_{m}"], axis=1)[:, :T] for m in ("q", "k", "v", "idx"))
        n = q.shape[0]
        planes = [pack_plane(a.T.reshape(-1)) for a in (q, k, v)]  # streams as channels: [T, C=n]
        e = np.full(n, 0x3400, np.uint16)  # 0.25
        for algo in (cuda.SAM_EULER, cuda.SAM_EAGER):
            cuda_rt.set_sam(algo)
            got, out = cuda_rt.rosa_qkv_1bit_fwd(*planes, e, 1, T, n)
            assert np.array_equal(got.reshape(T, n).T, idx), (kind, algo)
            assert np.array_equal(out, (2.0 * got - 1.0).astype(np.float32) * np.float32(0.25))
    cuda_rt.set_sam(cuda.SAM_EULER)


@pytest.mark.gpu
@pytest.mark.parametrize("variant,gain", [("literal", False), ("gain1", True)])
def test_cuda_heron_matches_fixture(cuda_rt, variant, gain):
    g = np.load(os.path.join(GOLD, "heron_tiny.npz"))
    cuda_rt.set_mode(cuda.MODE_EXACT)
    try:
        m = cuda.CudaHeron(cuda_rt, synth.heron_checkpoint("tiny", batch_size=2, seed=7, ln_gain_one=gain))
        m.set_taps(True)
        mean, loss_sum, n_valid, row_loss = m.forward_ce(g[f"{variant}_tokens"], g[f"{variant}_labels"], 3, 2, 64,
                                                         want_row_loss=True)
        assert n_valid == int(g[f"{variant}_n_valid"])
        assert abs(mean - float(g[f"{variant}_mean"])) <= 1e-3          # mean CE: 1e-3 absolute
        assert np.abs(row_loss - g[f"{variant}_row_loss"]).max() <= 1e-4
        # EXACT mode: everything up to the head is bit-identical to the CPU path
        assert np.array_equal(m.tap(0, "hidden", 128), g[f"{variant}_hidden"])
        for l in range(m.n_layers):
            assert np.array_equal(np.packbits(m.tap(l, "idx", 128)), g[f"{variant}_idx{l}"])
            assert np.array_equal(np.packbits(m.tap(l, "q_bits", 128)), g[f"{variant}_qbits{l}"])
            assert np.array_equal(m.tap(l, "block_out", 128), g[f"{variant}_block_out{l}"])
        lg = m.logits(g[f"{variant}_tokens"], 2, 64)
        assert np.array_equal(lg[:m.vocab_size], g[f"{variant}_logits_row0"])
        m.close()
    finally:
        cuda_rt.set_mode(cuda.MODE_FAST)
