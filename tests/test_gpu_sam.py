"""ROSA 1-bit suffix-automaton kernel against the oracle: idx must be
bit-exact for every stream, for both schedules, at ragged sizes, on worst-case
(constant / periodic) streams and at the benchmark's context lengths."""
import numpy as np
import pytest

from conftest import pack_plane
from ullis_b200 import cuda, synth

pytestmark = pytest.mark.gpu


def f16(x):
    return np.asarray(x, np.float32).astype(np.float16).view(np.uint16)


def run_both(cuda_rt, oracle, q, k, v, B, T, C, algos=(cuda.SAM_EULER, cuda.SAM_EAGER)):
    e = f16(np.linspace(0.01, 0.5, C))
    ref = oracle.rosa_qkv_batch_packed(q, k, v, B, T, C)
    for algo in algos:
        cuda_rt.set_sam(algo)
        idx, out = cuda_rt.rosa_qkv_1bit_fwd(q, k, v, e, B, T, C)
        assert np.array_equal(idx, ref), f"algo {algo}"
        assert np.array_equal(out, oracle.rosa_qkv_out_batched(ref, e, B, T, C))
    cuda_rt.set_sam(cuda.SAM_EULER)


@pytest.mark.parametrize("B,T,C", [(1, 1, 1), (1, 5, 3), (3, 31, 5), (2, 33, 32), (1, 64, 70), (2, 100, 33), (1, 1000, 9)])
def test_ragged_sizes_random_bits(cuda_rt, oracle, B, T, C):
    rng = np.random.default_rng(B * 10000 + T * 10 + C)
    q, k, v = (pack_plane(rng.integers(0, 2, B * T * C, dtype=np.uint8)) for _ in range(3))
    run_both(cuda_rt, oracle, q, k, v, B, T, C)


def test_exhaustive_t4_as_one_batch(cuda_rt, oracle):
    T = 4
    n = 1 << (3 * T)  # every (q,k,v) triple of 4-bit streams, one stream per channel
    a = np.arange(n)
    bits = lambda s: ((a[None, :] >> (s * T + np.arange(T)[:, None])) & 1).astype(np.uint8).reshape(-1)  # [T, n]
    run_both(cuda_rt, oracle, pack_plane(bits(0)), pack_plane(bits(1)), pack_plane(bits(2)), 1, T, n)


@pytest.mark.parametrize("kind", ["const", "k_const_mixed", "q_const_mixed", "q_const_biased", "v_const_mixed", "v_const_biased",
                                  "biased", "periodic_clean", "qk_same"])
def test_worst_case_streams(cuda_rt, oracle, kind):
    B, T, C = 1, 2048, 32
    rng = np.random.default_rng(len(kind))
    if kind == "const":
        q = np.repeat(rng.integers(0, 2, (1, C), dtype=np.uint8), T, 0)
        k = np.repeat(rng.integers(0, 2, (1, C), dtype=np.uint8), T, 0)
    elif kind == "k_const_mixed":  # half of the streams have constant k (closed-form path), random q
        q = rng.integers(0, 2, (T, C), dtype=np.uint8)
        k = rng.integers(0, 2, (T, C), dtype=np.uint8)
        k[:, ::2] = rng.integers(0, 2, (1, C // 2), dtype=np.uint8)
    elif kind in ("biased", "v_const_biased", "q_const_biased"):
        pr = rng.choice([0.001, 0.01, 0.99, 0.999], (1, C))
        q, k = (rng.random((T, C)) < pr).astype(np.uint8), (rng.random((T, C)) < pr).astype(np.uint8)
    elif kind == "q_const_mixed":  # three quarters of the streams have constant q (scan over the key runs), keys of several densities
        q = rng.integers(0, 2, (T, C), dtype=np.uint8)
        k = (rng.random((T, C)) < rng.choice([0.1, 0.5, 0.9], (1, C))).astype(np.uint8)
    elif kind == "periodic_clean":
        P = rng.integers(2, 64, C)
        base = rng.integers(0, 2, (64, C), dtype=np.uint8)
        q = np.take_along_axis(base, np.arange(T)[:, None] % P[None, :], 0)
        k = q.copy()
    else:
        q = rng.integers(0, 2, (T, C), dtype=np.uint8)
        k = q.copy()
    v = rng.integers(0, 2, (T, C), dtype=np.uint8)
    if kind.startswith("q_const"):
        q[:, 0::4] = 0
        q[:, 1::4] = 1
        q[:, 2::4] = rng.integers(0, 2, (1, C // 4), dtype=np.uint8)
    if kind.startswith("v_const"):  # three quarters of the streams have constant v: all 0 (idx = 0), all 1 (pass 1 only)
        v[:, 0::4] = 0
        v[:, 1::4] = 1
        v[:, 2::4] = rng.integers(0, 2, (1, C // 4), dtype=np.uint8)
    run_both(cuda_rt, oracle, pack_plane(q), pack_plane(k), pack_plane(v), B, T, C)


def test_model_context_length_batch(cuda_rt, oracle):
    B, T, C = 2, 2048, 256
    q, k, v = synth.rosa_bits_iid(21, B, T, C)
    run_both(cuda_rt, oracle, q, k, v, B, T, C)


def test_standalone_benchmark_context_length(cuda_rt, oracle):
    B, T, C = 1, 8192, 64  # context of the standalone ROSA configuration, fewer streams
    q, k, v = synth.rosa_bits_iid(22, B, T, C)
    run_both(cuda_rt, oracle, q, k, v, B, T, C, algos=(cuda.SAM_EULER,))
    q, k, v = synth.rosa_bits_periodic(23, B, T, C)
    run_both(cuda_rt, oracle, q, k, v, B, T, C)


def test_standalone_benchmark_at_its_full_size(cuda_rt, oracle):
    """The standalone ROSA configuration as stated: 64 sequences x 512 channels x 8192 steps, i.i.d. bits - all
    268 M idx positions against the oracle's pushes (rosa_qkv_batch_packed, src/rosa.rs:459-481) - and a
    4096-stream slice (8 sequences) of the periodic variant, whose streams have long suffix matches."""
    e = f16(np.linspace(0.01, 0.5, 512))
    oracle.set_threads(oracle.max_threads())
    try:
        for gen, seed, B in ((synth.rosa_bits_iid, 21, 64), (synth.rosa_bits_periodic, 23, 8)):
            T, C = 8192, 512
            q, k, v = gen(seed, B, T, C)
            idx, _ = cuda_rt.rosa_qkv_1bit_fwd(q, k, v, e, B, T, C, want_out=False)
            ref = oracle.rosa_qkv_batch_packed(q, k, v, B, T, C)
            assert idx.size == B * T * C and np.array_equal(idx, ref), gen.__name__
            del idx, ref, q, k, v
    finally:
        oracle.set_threads(min(16, oracle.max_threads()))


def test_context_beyond_16_bit_state_ids(cuda_rt, oracle):
    B, T, C = 1, 32768, 4  # MAX_CONTEXT_LEN: needs the 32-bit state-id kernels
    q, k, v = synth.rosa_bits_iid(24, B, T, C)
    run_both(cuda_rt, oracle, q, k, v, B, T, C, algos=(cuda.SAM_EULER,))


@pytest.mark.parametrize("budget_mb", ["4", "5"])
def test_streams_in_waves_when_the_scratch_budget_is_small(oracle, monkeypatch, budget_mb):
    """More streams than the automaton scratch may hold at once run in waves over the same blocks (4 MiB: 56 blocks
    of 74 368 B at T=2048; 5 MiB: 70, not a multiple of the streams a warp or a CTA carries, so the rounded-up grid
    of a wave reaches past it)."""
    monkeypatch.setenv("ULLIS_CUDA_SAM_BUDGET_MB", budget_mb)
    rt = cuda.CudaRuntime(0)
    try:
        B, T, C = 2, 2048, 96                                     # 192 streams: four waves
        q, k, v = synth.rosa_bits_iid(31, B, T, C)
        run_both(rt, oracle, q, k, v, B, T, C)
        q, k, v = synth.rosa_bits_periodic(32, B, T, C)
        run_both(rt, oracle, q, k, v, B, T, C, algos=(cuda.SAM_EULER,))
    finally:
        rt.close()


@pytest.mark.parametrize("chunked", ["0", "1"])
def test_pass_one_in_parts_gives_the_same_idx(oracle, monkeypatch, chunked):
    """The optional form of pass 1 - extend chain and query walk as two kernels against the final automaton read
    as of each step, the climb inside the tour kernel; the walk either serial or in eight guessed pieces per stream -
    is off by default (it measured slower than the interleaved form) but stays bit-exact."""
    monkeypatch.setenv("ULLIS_CUDA_SAM_SPLIT", "1")
    monkeypatch.setenv("ULLIS_CUDA_SAM_WALK_CHUNKED", chunked)
    rt = cuda.CudaRuntime(0)
    try:
        B, T, C = 2, 2048, 64
        q, k, v = synth.rosa_bits_iid(41, B, T, C)
        run_both(rt, oracle, q, k, v, B, T, C, algos=(cuda.SAM_EULER,))
        q, k, v = synth.rosa_bits_periodic(42, B, T, C)
        run_both(rt, oracle, q, k, v, B, T, C, algos=(cuda.SAM_EULER,))
        rng = np.random.default_rng(43)
        T, C = 777, 96                                       # a ragged length, biased streams
        pr = rng.choice([0.01, 0.1, 0.5, 0.9, 0.99], (1, C))
        q, k, v = (pack_plane((rng.random((T, C)) < pr).astype(np.uint8)) for _ in range(3))
        run_both(rt, oracle, q, k, v, 1, T, C, algos=(cuda.SAM_EULER,))
    finally:
        rt.close()


@pytest.mark.parametrize("waves", ["0", "1", "1000"])
def test_both_forms_of_the_serial_pass_give_the_same_idx(oracle, monkeypatch, waves):
    """Pass 1 keeps a stream's state array in shared memory (one one-warp CTA per stream) when it expects few
    enough streams for all of them to be resident at once, and in global memory otherwise.  The expectation is
    the number of streams the same call site sent to the automaton the last time, so a first call takes the
    global-memory kernel and a repeated one may take the other.  Forced here in turn: 0 = never shared memory,
    1000 = always (also when the streams need several rounds of resident CTAs), 1 = the default rule; every input
    runs twice."""
    monkeypatch.setenv("ULLIS_CUDA_SAM_SMEM_WAVES", waves)
    rt = cuda.CudaRuntime(0)
    try:
        rt.kernel_timing(True)
        rng = np.random.default_rng(53)
        cases = []
        B, T, C = 2, 2048, 64
        cases.append((synth.rosa_bits_iid(51, B, T, C), B, T, C))
        B, T, C = 6, 2048, 256      # 1 536 streams, more than one round of resident CTAs at this length
        cases.append((synth.rosa_bits_periodic(52, B, T, C), B, T, C))
        T, C = 333, 96                                       # a ragged length, biased streams
        pr = rng.choice([0.01, 0.1, 0.5, 0.9, 0.99], (1, C))
        cases.append((tuple(pack_plane((rng.random((T, C)) < pr).astype(np.uint8)) for _ in range(3)), 1, T, C))
        T, C = 5000, 40                                      # 80 KB of states per stream: two CTAs per SM
        cases.append((tuple(pack_plane(rng.integers(0, 2, (T, C), dtype=np.uint8)) for _ in range(3)), 1, T, C))
        for (q, k, v), B, T, C in cases:
            for _ in range(2):
                run_both(rt, oracle, q, k, v, B, T, C, algos=(cuda.SAM_EULER,))
        ran = rt.kernel_times()
        assert ("rosa_pass1_smem" in ran) == (waves != "0") and ("rosa_pass1" in ran) == (waves != "1000")
    finally:
        rt.close()
