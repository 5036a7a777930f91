"""RosaSam::push (src/rosa.rs:100-176) for many streams with the automata kept on the device between calls
(ullis_cuda_rosa_pushers_*, the kernel that incremental generation runs per layer) against the oracle's pushes:
idx identical at every position of every stream, on the stream families whose suffix-link chains grow with the
context (biased, periodic, a key that is constant for a long time and then is not)."""
import numpy as np
import pytest

from conftest import pack_streams
from test_sam_core_host import _streams
from ullis_b200 import cuda

pytestmark = pytest.mark.gpu


def _oracle_idx(oracle, q, k, v):
    n, T = q.shape
    words = oracle.rosa_qkv_streams(pack_streams(q), pack_streams(k), pack_streams(v), n, T)
    bits = np.unpackbits(words.view(np.uint8).reshape(n, -1), axis=1, bitorder="little")[:, :T]
    return bits.T.copy()   # [T, n]


def _late_change(n, T, rng):
    """key constant for most of the context (no automaton is written), then arbitrary"""
    q = rng.integers(0, 2, (n, T), dtype=np.uint8)
    k = np.repeat(rng.integers(0, 2, (n, 1), dtype=np.uint8), T, 1)
    v = rng.integers(0, 2, (n, T), dtype=np.uint8)
    for s in range(n):
        at = int(rng.integers(1, T))
        k[s, at:] = rng.integers(0, 2, T - at, dtype=np.uint8) if s % 2 else (rng.random(T - at) < 0.02) ^ k[s, 0]
    return [q, k, v]


@pytest.mark.parametrize("kind,T,n", [("iid", 300, 96), ("biased", 2048, 64), ("periodic", 2048, 32), ("periodic_clean", 1024, 16),
                                      ("k_const", 700, 16), ("q_const", 2048, 32), ("qk_same", 777, 32), ("late_change", 2048, 64),
                                      ("late_change", 33, 40)])
def test_pushes_match_the_reference_at_every_position(cuda_rt, oracle, kind, T, n):
    rng = np.random.default_rng(hash((kind, T)) & 0xFFFF)
    q, k, v = _late_change(n, T, rng) if kind == "late_change" else _streams(kind, n, T, rng)
    ref = _oracle_idx(oracle, q, k, v)
    p = cuda.CudaRosaPushers(cuda_rt, n, T)
    # in one call, and in uneven pieces (the state carries over)
    assert np.array_equal(p.push(q.T, k.T, v.T), ref), kind
    p.reset()
    got, t = [], 0
    for piece in (1, 1, 5, 32, 31, 64, T):
        piece = min(piece, T - t)
        if piece == 0:
            break
        got.append(p.push(q.T[t:t + piece], k.T[t:t + piece], v.T[t:t + piece]))
        t += piece
    assert np.array_equal(np.concatenate(got), ref), kind
    p.close()


def test_wide_state_ids(cuda_rt, oracle):
    T, n = 33000, 2   # 2T + 2 > 65535: 32-bit state ids
    rng = np.random.default_rng(9)
    q, k, v = _streams("iid", n, T, rng)
    ref = _oracle_idx(oracle, q, k, v)
    p = cuda.CudaRosaPushers(cuda_rt, n, T)
    assert np.array_equal(p.push(q.T, k.T, v.T), ref)
    p.close()


def test_capacity_and_arguments(cuda_rt):
    with pytest.raises(cuda.UllisCudaError) as e:
        cuda.CudaRosaPushers(cuda_rt, 0, 8)
    assert e.value.code == cuda.ERR_SHAPE
    p = cuda.CudaRosaPushers(cuda_rt, 3, 4)
    z = np.zeros((3, 3), np.uint8)
    p.push(z, z, z)
    with pytest.raises(cuda.UllisCudaError) as e:   # two more than the capacity: nothing is pushed
        p.push(z, z, z)
    assert e.value.code == cuda.ERR_SHAPE
    assert p.push(z[:1], z[:1], z[:1]).shape == (1, 3)
    p.close()
