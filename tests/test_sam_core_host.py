"""The device suffix-automaton routines (ullis_b200/csrc/sam_core.cuh), compiled
for the host, against the oracle: exhaustively for short streams and on long
random, constant, biased and periodic streams, for both schedules and both
state-id widths."""
import numpy as np
import pytest

from conftest import pack_streams

ALGOS = {"eager": 0, "euler": 1, "euler_with_constant_k_shortcut": 2, "incremental_pushes_lazy_chain": 6}
PACKED_WORDS = 4   # pass 1 on packed state words: 16-bit state ids only
DEFERRED_CLIMB = 7 # interleaved pass 1 that records (w_t, h_t); the climb to v_t afterwards, links read as of step t
SPLIT = 5          # pass 1 as extend / walk / climb against the final automaton: 16-bit state ids only
SPLIT_PIECES = [100 + p for p in (1, 3, 32, 256)]   # the same with the query walk in pieces of p steps, guessed and put right


@pytest.mark.parametrize("T", [1, 2, 3, 4, 5])
def test_exhaustive_short_streams(oracle, sam_host, T):
    n = 1 << (3 * T)
    a = np.arange(n, dtype=np.uint32)
    m = (1 << T) - 1
    q, k, v = a & m, (a >> T) & m, (a >> (2 * T)) & m
    ref = oracle.rosa_qkv_streams(q, k, v, n, T)
    for algo in ALGOS.values():
        for ix in (16, 32):
            assert np.array_equal(sam_host(algo, ix, q, k, v, n, T), ref)
    assert np.array_equal(sam_host(PACKED_WORDS, 16, q, k, v, n, T), ref)
    assert np.array_equal(sam_host(SPLIT, 16, q, k, v, n, T), ref)
    assert np.array_equal(sam_host(DEFERRED_CLIMB, 16, q, k, v, n, T), ref)
    for algo in SPLIT_PIECES[:2]:
        assert np.array_equal(sam_host(algo, 16, q, k, v, n, T), ref)


@pytest.mark.parametrize("T", [9, 14])
def test_exhaustive_key_sequences_under_a_constant_query(oracle, sam_host, T):
    """Every key sequence of length T with q constant (both values) and several v
    sequences: the closed form for constant q against the reference's pushes."""
    rng = np.random.default_rng(T)
    kk = np.arange(1 << T, dtype=np.uint32)
    m = np.uint32((1 << T) - 1)
    for c in (0, 1):
        q = np.full(kk.size, m if c else 0, np.uint32)
        for v in (kk ^ np.uint32(0x2A5), rng.integers(0, 1 << T, kk.size).astype(np.uint32), np.full(kk.size, 0x1555 & int(m), np.uint32)):
            ref = oracle.rosa_qkv_streams(q, kk, v, kk.size, T)
            assert np.array_equal(sam_host(2, 16, q, kk, v, kk.size, T), ref), c
            assert np.array_equal(sam_host(1, 16, q, kk, v, kk.size, T), ref), c
            assert np.array_equal(sam_host(PACKED_WORDS, 16, q, kk, v, kk.size, T), ref), c
            assert np.array_equal(sam_host(SPLIT, 16, q, kk, v, kk.size, T), ref), c
            assert np.array_equal(sam_host(DEFERRED_CLIMB, 16, q, kk, v, kk.size, T), ref), c


def _streams(kind, n, T, rng):
    if kind == "iid":
        return [rng.integers(0, 2, (n, T), dtype=np.uint8) for _ in range(3)]
    if kind == "const":
        return [np.repeat(rng.integers(0, 2, (n, 1), dtype=np.uint8), T, 1),
                np.repeat(rng.integers(0, 2, (n, 1), dtype=np.uint8), T, 1), rng.integers(0, 2, (n, T), dtype=np.uint8)]
    if kind == "k_const":
        return [rng.integers(0, 2, (n, T), dtype=np.uint8), np.repeat(rng.integers(0, 2, (n, 1), dtype=np.uint8), T, 1),
                rng.integers(0, 2, (n, T), dtype=np.uint8)]
    if kind == "v_const":   # idx = 0 everywhere (v all 0) or "a match exists" (v all 1)
        return [rng.integers(0, 2, (n, T), dtype=np.uint8), rng.integers(0, 2, (n, T), dtype=np.uint8),
                np.repeat(rng.integers(0, 2, (n, 1), dtype=np.uint8), T, 1)]
    if kind == "v_const_biased":
        pr = rng.choice([0.002, 0.02, 0.98], (n, 1))
        return [(rng.random((n, T)) < pr).astype(np.uint8), (rng.random((n, T)) < pr).astype(np.uint8),
                np.repeat(rng.integers(0, 2, (n, 1), dtype=np.uint8), T, 1)]
    if kind == "q_const":   # the query bits all equal: idx follows the runs of that bit among the keys
        pr = rng.choice([0.002, 0.05, 0.3, 0.5, 0.7, 0.95, 0.995, 0.9995], (n, 1))
        return [np.repeat(rng.integers(0, 2, (n, 1), dtype=np.uint8), T, 1), (rng.random((n, T)) < pr).astype(np.uint8),
                rng.integers(0, 2, (n, T), dtype=np.uint8)]
    if kind == "q_const_periodic":
        P = rng.integers(2, 40, n)
        base = rng.integers(0, 2, (n, 64), dtype=np.uint8)
        b = np.take_along_axis(base, np.arange(T)[None, :] % P[:, None], 1)
        return [np.repeat(rng.integers(0, 2, (n, 1), dtype=np.uint8), T, 1), (b ^ (rng.random((n, T)) < 0.03)).astype(np.uint8),
                rng.integers(0, 2, (n, T), dtype=np.uint8)]
    if kind == "biased":
        pr = rng.choice([0.001, 0.01, 0.99, 0.999], (n, 1))
        return [(rng.random((n, T)) < pr).astype(np.uint8), (rng.random((n, T)) < pr).astype(np.uint8),
                rng.integers(0, 2, (n, T), dtype=np.uint8)]
    if kind in ("periodic", "periodic_clean"):
        P = rng.integers(2, 64, n)
        base = rng.integers(0, 2, (n, 64), dtype=np.uint8)
        b = np.take_along_axis(base, np.arange(T)[None, :] % P[:, None], 1)
        fl = 0.0 if kind == "periodic_clean" else 0.05
        return [(b ^ (rng.random((n, T)) < fl)).astype(np.uint8), (b ^ (rng.random((n, T)) < fl)).astype(np.uint8),
                rng.integers(0, 2, (n, T), dtype=np.uint8)]
    if kind == "qk_same":
        q = rng.integers(0, 2, (n, T), dtype=np.uint8)
        return [q, q.copy(), rng.integers(0, 2, (n, T), dtype=np.uint8)]
    raise ValueError(kind)


@pytest.mark.parametrize("kind,T,n", [("q_const", 2048, 48), ("q_const", 333, 64), ("q_const_periodic", 1500, 32), ("v_const", 777, 32), ("v_const_biased", 2048, 16), ("iid", 97, 200), ("iid", 2048, 24), ("const", 1024, 16), ("k_const", 1000, 16), ("k_const", 64, 8), ("biased", 2048, 16),
                                      ("periodic", 1500, 16), ("periodic_clean", 2048, 8), ("qk_same", 777, 32)])
def test_long_streams(oracle, sam_host, kind, T, n):
    rng = np.random.default_rng(hash((kind, T)) & 0xFFFF)
    q, k, v = (pack_streams(b) for b in _streams(kind, n, T, rng))
    ref = oracle.rosa_qkv_streams(q, k, v, n, T)
    for algo in list(ALGOS.values()) + [PACKED_WORDS, SPLIT, DEFERRED_CLIMB] + SPLIT_PIECES:
        assert np.array_equal(sam_host(algo, 16, q, k, v, n, T), ref), (kind, algo)
    assert np.array_equal(sam_host(1, 32, q, k, v, n, T), ref)


def test_wide_state_ids_beyond_16_bits(oracle, sam_host):
    T, n = 33000, 2  # 2T+2 > 65535: the 32-bit state-id instantiation is required
    rng = np.random.default_rng(5)
    q, k, v = (pack_streams(b) for b in _streams("iid", n, T, rng))
    ref = oracle.rosa_qkv_streams(q, k, v, n, T)
    assert np.array_equal(sam_host(1, 32, q, k, v, n, T), ref)
