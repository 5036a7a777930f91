"""Seeded random sweeps through the C ABI against the oracle: ROSA streams of
mixed kinds (random, constant, biased, periodic, one flip, one odd bit) at
ragged shapes - every closed form and both automaton schedules must agree with
RosaSam::push bit for bit - and whole models of random shapes in both
arithmetic modes."""
import numpy as np
import pytest

from conftest import pack_plane
from ullis_b200 import cuda, synth

pytestmark = pytest.mark.gpu


def _stream(rng, T, kind):
    if kind == 0:
        return rng.integers(0, 2, T, dtype=np.uint8)
    if kind == 1:
        return np.full(T, rng.integers(0, 2), np.uint8)
    if kind == 2:
        return (rng.random(T) < rng.choice([0.001, 0.01, 0.05, 0.95, 0.99, 0.999])).astype(np.uint8)
    if kind == 3:
        P = int(rng.integers(1, 40))
        s = np.tile(rng.integers(0, 2, P, dtype=np.uint8), T // P + 1)[:T]
        return (s ^ (rng.random(T) < rng.choice([0, 0.01, 0.1]))).astype(np.uint8)
    s = np.full(T, rng.integers(0, 2), np.uint8)
    if kind == 4:
        s[rng.integers(0, T):] ^= 1      # constant with one flip
    else:
        s[rng.integers(0, T)] ^= 1       # one odd bit
    return s


@pytest.mark.parametrize("seed", range(4))
def test_rosa_streams_of_mixed_kinds(cuda_rt, oracle, seed):
    rng = np.random.default_rng(1000 + seed)
    try:
        for _ in range(24):
            B = int(rng.integers(1, 4))
            C = int(rng.choice([1, 3, 16, 33, 64]))
            T = int(rng.choice([1, 2, 7, 31, 32, 33, 64, 100, 257, 512, 1000, 2048, 3000]))
            q, k, v = (np.stack([np.stack([_stream(rng, T, rng.integers(0, 6)) for _ in range(C)], 1) for _ in range(B)])
                       for _ in range(3))
            qp, kp, vp = (pack_plane(a.reshape(-1)) for a in (q, k, v))
            ref = oracle.rosa_qkv_batch_packed(qp, kp, vp, B, T, C)
            e = np.linspace(0.01, 0.5, C).astype(np.float16).view(np.uint16)
            for algo in (cuda.SAM_EULER, cuda.SAM_EAGER):
                if algo == cuda.SAM_EAGER and T > 1000:
                    continue
                cuda_rt.set_sam(algo)
                idx, _ = cuda_rt.rosa_qkv_1bit_fwd(qp, kp, vp, e, B, T, C)
                assert np.array_equal(idx, ref), (B, T, C, algo)
    finally:
        cuda_rt.set_sam(cuda.SAM_EULER)


@pytest.mark.parametrize("seed", range(3))
def test_models_of_random_shapes(cuda_rt, oracle, seed):
    rng = np.random.default_rng(2000 + seed)
    try:
        for case in range(5):
            d = int(rng.choice([64, 128, 192, 256, 320, 448, 512]))
            layers = int(rng.integers(1, 4))
            vocab = int(rng.choice([264, 328, 520, 1000, 2048]))
            ffn = int(rng.choice([64, 128, 192, 320, 1024]))
            T = int(rng.choice([32, 64, 96, 160, 50, 257]))
            B = int(rng.integers(1, 4))
            data = synth.heron_checkpoint((d, layers, vocab, T, ffn), batch_size=B, ln_gain_one=bool(rng.integers(0, 2)))
            ref = oracle.HeronOracle(data)
            tok = synth.zipf_tokens(100 * seed + case, B * T, vocab)
            lab = tok.copy()
            lab[1] = 0
            mean_ref, n_ref, _, lg_ref = ref.forward_ce(tok, lab, 0, B, T, want_logits=True)
            for mode in (cuda.MODE_FAST, cuda.MODE_EXACT):
                cuda_rt.set_mode(mode)
                m = cuda.CudaHeron(cuda_rt, data)
                mean, _, n = m.forward_ce(tok, lab, 0, B, T)
                lg = m.logits(tok, B, T)
                m.close()
                assert n == n_ref and abs(mean - mean_ref) <= 1e-3, (d, layers, vocab, T, ffn, B, mode)   # mean CE: 1e-3
                if mode == cuda.MODE_EXACT:
                    assert np.array_equal(lg, lg_ref.reshape(-1)), (d, layers, vocab, T, ffn, B)
                else:
                    rel = np.linalg.norm(lg.astype(np.float64) - lg_ref.reshape(-1)) / np.linalg.norm(lg_ref.astype(np.float64))
                    assert rel <= 1e-2, (d, layers, vocab, T, ffn, B, rel)                              # logits: 1e-2 relative
    finally:
        cuda_rt.set_mode(cuda.MODE_FAST)


@pytest.mark.parametrize("env", [{"ULLIS_CUDA_SAM_SIDE": "0"}, {"ULLIS_CUDA_SAM_WORDS": "0"},
                                 {"ULLIS_CUDA_SAM_COOP_THREADS": "512"}, {"ULLIS_CUDA_SAM_COOP_THREADS": "1024"},
                                 {"ULLIS_CUDA_SAM_LANES": "4"}],
                         ids=lambda e: "-".join(f"{k[11:].lower()}={v}" for k, v in e.items()))
def test_rosa_streams_under_every_kernel_choice(oracle, monkeypatch, env):
    """The automaton's alternative forms (constant-q closed form on the main stream, field-wise pass 1, more threads
    per stream in tour / pass 2, several streams per warp) give the same idx as the defaults: all equal RosaSam::push."""
    for k, v in env.items():
        monkeypatch.setenv(k, v)
    rt = cuda.CudaRuntime(0)
    try:
        rng = np.random.default_rng(77)
        for B, T, C in ((2, 2048, 48), (1, 1000, 33), (3, 96, 64)):
            q, k, v = (np.stack([np.stack([_stream(rng, T, rng.integers(0, 6)) for _ in range(C)], 1) for _ in range(B)])
                       for _ in range(3))
            qp, kp, vp = (pack_plane(a.reshape(-1)) for a in (q, k, v))
            ref = oracle.rosa_qkv_batch_packed(qp, kp, vp, B, T, C)
            e = np.linspace(0.01, 0.5, C).astype(np.float16).view(np.uint16)
            idx, _ = rt.rosa_qkv_1bit_fwd(qp, kp, vp, e, B, T, C)
            assert np.array_equal(idx, ref), (B, T, C)
    finally:
        rt.close()
