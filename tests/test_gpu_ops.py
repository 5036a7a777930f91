"""Op-level parity through the C ABI on a real GPU: the reference's golden
vectors, then random shapes against the CPU oracle - bit-exact in EXACT mode,
within the stated tolerance in FAST mode."""
import numpy as np
import pytest

from conftest import pack_plane, unpack_plane
from test_oracle_golden import (QKV_IDX, QKV_K, QKV_Q, QKV_V, ROSA_T5_C3, ROSA_Y, patterned_bits, signs_to_bits,
                                tile_boundary_case)
from ullis_b200 import cuda

pytestmark = pytest.mark.gpu


def f16(x):
    return np.asarray(x, np.float32).astype(np.float16).view(np.uint16)


@pytest.fixture(params=[cuda.MODE_EXACT, cuda.MODE_FAST], ids=["exact", "fast"])
def rt(request, cuda_rt):
    cuda_rt.set_mode(request.param)
    cuda_rt.mode = request.param
    yield cuda_rt
    cuda_rt.set_mode(cuda.MODE_FAST)


def close(rt, got, ref, rel=1e-2):
    """EXACT: bit-identical.  FAST: |got-ref| <= rel * max|ref| (1e-2 relative)."""
    got, ref = np.asarray(got), np.asarray(ref)
    if rt.mode == cuda.MODE_EXACT:
        assert np.array_equal(got.view(np.uint32), ref.view(np.uint32))
    else:
        assert np.abs(got - ref).max() <= rel * max(np.abs(ref).max(), 1e-30)


# ------------------------------------------------------------ golden vectors

def test_qkv_fixture(cuda_rt):  # tests/rosa_metal.rs:92-115
    for algo in (cuda.SAM_EULER, cuda.SAM_EAGER):
        cuda_rt.set_sam(algo)
        idx, out = cuda_rt.rosa_qkv_1bit_fwd(pack_plane(QKV_Q), pack_plane(QKV_K), pack_plane(QKV_V), f16([0.25]), 1, 8, 1)
        assert idx.tolist() == QKV_IDX
        assert out.tolist() == [-0.25, 0.25, -0.25, 0.25, 0.25, -0.25, 0.25, -0.25]
    cuda_rt.set_sam(cuda.SAM_EULER)


def test_t5_c3_collapses_unmatched_to_minus_e(cuda_rt):  # tests/rosa_metal.rs:117-143
    bits = (ROSA_T5_C3.reshape(-1) > 0).astype(np.uint8)
    w = pack_plane(bits)
    idx, out = cuda_rt.rosa_qkv_1bit_fwd(w, w, w, f16([0.5, 0.25, 1.0]), 1, 5, 3)
    for c in range(3):
        assert idx.reshape(5, 3)[:, c].tolist() == [max(y, 0) for y in ROSA_Y[c]]
    assert np.all(np.abs(out) > 0.1)
    assert np.array_equal(out.reshape(5, 3), (2.0 * idx.reshape(5, 3) - 1.0) * np.array([0.5, 0.25, 1.0], np.float32))


@pytest.mark.parametrize("B,T,C,salts", [(2, 32, 8, (1, 2, 3)), (1, 32, 256, (4, 5, 6))])
def test_patterned_bits_bit_exact(cuda_rt, oracle, B, T, C, salts):  # tests/rosa_metal.rs:145-205
    q, k, v = (patterned_bits(B, T, C, s) for s in salts)
    e = f16([0.125 * (c + 1) for c in range(C)])
    idx, out = cuda_rt.rosa_qkv_1bit_fwd(pack_plane(q), pack_plane(k), pack_plane(v), e, B, T, C)
    ref = oracle.rosa_qkv_batch(q, k, v, B, T, C)
    assert np.array_equal(idx, ref)
    assert np.array_equal(out, oracle.rosa_qkv_out_batched(ref, e, B, T, C))


def test_binary_linear_golden(rt, oracle):  # tests/binary_linear.rs:3-11, src/metal.rs:3805-3820
    y = rt.binary_linear([2.0, 3.0], signs_to_bits([1, -1]), f16([0.5]), f16([0.0]), 1, 2, 1)
    assert abs(y[0] + 0.5) < 2e-3
    signs = [1, -1, -1, 1, 1, 1]
    x = np.array([0.5, -1.0, 2.0, 1.0, 0.0, -0.5], np.float32)
    y = rt.binary_linear(x, signs_to_bits(signs), f16([0.5, 0.5]), f16([0, 0]), 2, 3, 2)
    close(rt, y, oracle.binary_linear(x, signs_to_bits(signs), f16([0.5, 0.5]), f16([0, 0]), 2, 3, 2))


def test_linears_past_tile_boundary(rt, oracle):  # src/metal.rs:3907-3974
    rows, inn, out, signs, weight, x = tile_boundary_case()
    bits = signs_to_bits(signs)
    y = rt.binary_linear(x, bits, f16([0.5] * out), f16([0.0] * out), rows, inn, out)
    ref = oracle.binary_linear(x, bits, f16([0.5] * out), f16([0.0] * out), rows, inn, out)
    assert np.abs(y - ref).max() <= 3e-3
    close(rt, y, ref)
    yd = rt.fp16_linear(x, f16(weight), rows, inn, out)
    refd = oracle.fp16_linear(x, f16(weight), rows, inn, out)
    assert np.abs(yd - refd).max() <= 3e-3
    close(rt, yd, refd)


def test_layer_norm_golden(rt, oracle):  # src/metal.rs:3772-3788, tests/cmix.rs:19-31
    w, b = f16([1.25, 0.75, 1.0, 0.5]), f16([0.1, -0.2, 0.0, 0.05])
    x = np.array([1.0, 2.0, 3.0, 4.0, 0.5, -1.0, 0.0, 2.5], np.float32)
    y = rt.layer_norm(x, w, b, 2, 4)
    ref = oracle.layer_norm(x, w, b, 2, 4)
    assert np.abs(y - ref).max() <= 2e-3
    close(rt, y, ref, rel=1e-5)


def test_cmix_golden(rt):  # tests/cmix.rs:33-72
    y = rt.cmix_block_forward([1.0, 0.0, 0.0, 1.0], f16([0, 0]), signs_to_bits([1, -1, -1, 1]), f16([1, 1]),
                              f16([1.0, 0.0, 0.0, 1.0]), 1, 2, 2, 2)
    assert np.allclose(y, [1, 0, 0, 1], atol=1e-5)
    y = rt.cmix_block_forward([2.0, 0.0, 0.0, 0.0], f16([1, 0]), signs_to_bits([1, 1]), f16([1]), f16([1.0, 0.0]),
                              1, 2, 2, 1)
    assert np.allclose(y, [0, 0, 4, 0], atol=1e-4)


def test_streamed_ce_three_row_case(rt, oracle):  # src/metal.rs:4044-4064
    signs = [1, -1, 1, -1, -1, 1, 1, 1]
    hidden = np.array([0.5, -0.25, 1.0, 0.0, -0.5, 0.75], np.float32)
    tokens = np.array([1, 3, 0], np.uint32)
    mean, n_valid, rl = rt.streamed_ce(hidden, signs_to_bits(signs), f16([0.5] * 4), None, tokens, cuda.CE_NO_IGNORE,
                                       3, 3, 2, 4)
    rmean, rn, rrl, _ = oracle.head_ce(hidden, signs_to_bits(signs), f16([0.5] * 4), None, tokens,
                                       oracle.CE_NO_IGNORE, 3, 3, 2, 4)
    assert n_valid == rn == 2 and rl[2] == 0.0
    assert abs(mean - rmean) < 1e-3 and np.abs(rl - rrl).max() < 1e-3  # mean CE: 1e-3 absolute


# -------------------------------------------------------- elementwise, exact

def test_elementwise_ops_are_bit_exact(cuda_rt, oracle):
    rng = np.random.default_rng(0)
    x = rng.standard_normal(3 * 7 * 37).astype(np.float32)
    x[5] = 0.0
    x[6] = -0.0
    assert np.array_equal(cuda_rt.time_shift_delta(x, 21, 7, 37), oracle.time_shift_delta(x, 3, 7, 37))
    assert np.array_equal(cuda_rt.sign_pack_bits(x), oracle.sign_pack_bits(x))
    assert np.array_equal(cuda_rt.sign_pack_bits(x[:1]), oracle.sign_pack_bits(x[:1]))
    m = np.maximum(x, 0)
    assert np.array_equal(cuda_rt.cmix_relu2(x), m * m)
    y = rng.standard_normal(x.size).astype(np.float32)
    assert np.array_equal(cuda_rt.residual_add(x, y), x + y)
    assert cuda_rt.sign_pack_bits(np.array([0.0, -0.0, 1e-8, np.nan], np.float32))[0] == 0b0100


# ------------------------------------------------------- random vs the oracle

@pytest.mark.parametrize("rows,C", [(1, 4), (33, 19), (64, 256), (100, 512), (7, 1024), (5, 1100)])
def test_layer_norm_random(rt, oracle, rows, C):
    rng = np.random.default_rng(rows * 1000 + C)
    x = (rng.standard_normal(rows * C) * rng.uniform(0.01, 5.0)).astype(np.float32) + np.float32(rng.normal())
    w, b = f16(1 + 0.1 * rng.standard_normal(C)), f16(0.1 * rng.standard_normal(C))
    close(rt, rt.layer_norm(x, w, b, rows, C), oracle.layer_norm(x, w, b, rows, C), rel=1e-4)


@pytest.mark.parametrize("rows,K,N,bias", [(1, 32, 1, True), (70, 64, 130, False), (128, 512, 512, True),
                                           (200, 256, 1024, False), (3, 33, 5, True), (256, 512, 2048, False)])
def test_binary_linear_random(rt, oracle, rows, K, N, bias):
    rng = np.random.default_rng(rows + K + N)
    x = rng.standard_normal(rows * K).astype(np.float32)
    bits = rng.integers(0, 2 ** 32, (K * N + 31) // 32, dtype=np.uint32)
    s, b = f16(rng.uniform(0.005, 0.02, N)), (f16(rng.normal(0, 0.01, N)) if bias else None)
    close(rt, rt.binary_linear(x, bits, s, b, rows, K, N), oracle.binary_linear(x, bits, s, b, rows, K, N))


@pytest.mark.parametrize("rows,K,N", [(5, 7, 3), (128, 2048, 512), (77, 1024, 256)])
def test_fp16_linear_random(rt, oracle, rows, K, N):
    rng = np.random.default_rng(K + N)
    x = np.abs(rng.standard_normal(rows * K)).astype(np.float32)
    w = f16(rng.uniform(-1, 1, K * N) / np.sqrt(K))
    close(rt, rt.fp16_linear(x, w, rows, K, N), oracle.fp16_linear(x, w, rows, K, N))


def _rosa_params(rng, d):
    p = {m: f16(rng.uniform(0, 1, d)) for m in ("x_q", "x_k", "x_v")}
    p["e"] = f16(rng.normal(0, 0.02, d))
    for m in "qkvo":
        p[m] = {"bits": rng.integers(0, 2 ** 32, d * d // 32, dtype=np.uint32), "scale": f16(rng.uniform(0.005, 0.02, d)),
                "bias": f16(rng.normal(0, 0.01, d))}
    return p


@pytest.mark.parametrize("B,T,d", [(1, 40, 64), (2, 96, 128), (1, 256, 256)])
def test_rosa_block_forward(rt, oracle, B, T, d):
    """Given the same f32 input, Q/K/V sign bits and idx must be bit-exact in
    both modes; activations bit-exact (EXACT) or within 1e-2 relative (FAST)."""
    rng = np.random.default_rng(B * T + d)
    p = _rosa_params(rng, d)
    x = rng.standard_normal(B * T * d).astype(np.float32)
    ref_out, t = oracle.rosa_block_forward(x, p, B, T, d, taps=True)
    got = rt.rosa_block_forward(x, p, B, T, d)
    n = B * T * d
    for m in "qkv":
        assert np.array_equal(unpack_plane(got[m + "_plane"], n), t[m + "_bits"]), m
    assert np.array_equal(got["idx"], t["idx"])
    assert np.array_equal(got["y"], t["y"])
    close(rt, got["out"], ref_out)


@pytest.mark.parametrize("B,T,d,f", [(1, 33, 64, 128), (2, 64, 256, 1024)])
def test_cmix_block_forward(rt, oracle, B, T, d, f):
    rng = np.random.default_rng(d + f)
    x = rng.standard_normal(B * T * d).astype(np.float32)
    mix = f16(rng.uniform(0, 1, d))
    kb = rng.integers(0, 2 ** 32, d * f // 32, dtype=np.uint32)
    ks = f16(rng.uniform(0.005, 0.02, f))
    val = f16(rng.uniform(-1, 1, d * f) / np.sqrt(f))
    close(rt, rt.cmix_block_forward(x, mix, kb, ks, val, B, T, d, f), oracle.cmix_forward(x, mix, kb, ks, val, B, T, d, f))


@pytest.mark.parametrize("rows,T,D,V,ignore", [(64, 16, 64, 512, None), (96, 32, 256, 8192, 3), (8, 4, 32, 300, 1)])
def test_streamed_ce_random(rt, oracle, rows, T, D, V, ignore):
    rng = np.random.default_rng(V)
    h = rng.standard_normal(rows * D).astype(np.float32)
    bits = rng.integers(0, 2 ** 32, (D * V + 31) // 32, dtype=np.uint32)
    s, b = f16(rng.uniform(0.005, 0.05, V)), f16(rng.normal(0, 0.1, V))
    labels = rng.integers(0, min(V, 8), rows).astype(np.uint32)
    ig = cuda.CE_NO_IGNORE if ignore is None else ignore
    mean, nv, rl = rt.streamed_ce(h, bits, s, b, labels, ig, rows, T, D, V)
    rmean, rnv, rrl, _ = oracle.head_ce(h, bits, s, b, labels, ig, rows, T, D, V)
    assert nv == rnv
    assert abs(mean - rmean) <= 1e-3                      # mean CE within 1e-3 absolute
    assert np.abs(rl - rrl).max() <= 1e-2 * max(np.abs(rrl).max(), 1.0)
    assert np.array_equal(rl == 0, rrl == 0)


# -------------------------------------------------------------- error paths

def test_shape_errors_and_empty_inputs(cuda_rt):
    with pytest.raises(cuda.UllisCudaError) as e:
        cuda_rt.rosa_qkv_1bit_fwd(np.zeros(1, np.uint32), np.zeros(1, np.uint32), np.zeros(1, np.uint32), f16([1.0]), 0, 8, 1)
    assert e.value.code == cuda.ERR_SHAPE
    lib = cuda_rt._lib
    import ctypes as C
    x = np.zeros(4, np.float32)
    rc = lib.ullis_cuda_time_shift_delta(cuda_rt._h, C.c_void_p(x.ctypes.data), C.c_void_p(x.ctypes.data),
                                         C.c_size_t(4), C.c_size_t(3), C.c_size_t(1))
    assert rc == cuda.ERR_SHAPE and b"mismatch" in lib.ullis_cuda_last_error(cuda_rt._h)
    rc = lib.ullis_cuda_layer_norm(cuda_rt._h, None, None, None, None, C.c_size_t(2), C.c_size_t(2))
    assert rc == cuda.ERR_ARG
    assert cuda_rt.layer_norm(np.zeros(0, np.float32), f16([1, 1]), f16([0, 0]), 0, 2).size == 0
    with pytest.raises(cuda.UllisCudaError) as e:  # target id beyond the vocabulary
        cuda_rt.streamed_ce(np.zeros(8, np.float32), np.zeros(4, np.uint32), f16([1] * 32), None,
                            np.array([0, 99], np.uint32), cuda.CE_NO_IGNORE, 2, 2, 4, 32)
    assert e.value.code == cuda.ERR_TOKEN
    assert cuda_rt.launch_count > 0 and cuda_rt.stream != 0


def test_fp16_operand_range_is_reported_not_turned_into_inf(cuda_rt):
    """The tensor-core path takes FP16 operands (65504 at most): a larger activation is an error with the
    row in the message, never an inf in the output; the reference-order mode takes the same input."""
    rows, K, N = 128, 64, 64
    x = np.ones((rows, K), np.float32)
    x[37, 5] = 1.0e5
    w = f16(0.1 * np.random.default_rng(3).standard_normal(N * K))
    with pytest.raises(cuda.UllisCudaError) as e:
        cuda_rt.fp16_linear(x, w, rows, K, N)
    assert e.value.code == cuda.ERR_DEVICE_CHECK and "FP16 range" in e.value.message and "row 37" in e.value.message
    cuda_rt.set_mode(cuda.MODE_EXACT)
    try:
        y = cuda_rt.fp16_linear(x, w, rows, K, N)
        assert np.isfinite(y).all()
    finally:
        cuda_rt.set_mode(cuda.MODE_FAST)
    y = cuda_rt.fp16_linear(np.ones((rows, K), np.float32), w, rows, K, N)   # the runtime is usable afterwards
    assert np.isfinite(y).all()


def test_a_device_wait_that_runs_out_is_reported_and_the_runtime_stays_usable(cuda_rt):
    """Nothing ever arrives on the barrier the self-test kernel waits on: the bounded wait gives up after the
    requested polls, the kernel returns by itself, the status word carries the time-out to the host as
    ERR_TIMEOUT, and the next call on the same runtime works (no fault, no hang, no lost context)."""
    with pytest.raises(cuda.UllisCudaError) as e:
        cuda_rt.wait_selftest(2000)
    assert e.value.code == cuda.ERR_TIMEOUT and "gave up waiting" in e.value.message and "99" in e.value.message
    x = np.arange(8, dtype=np.float32)
    assert np.array_equal(cuda_rt.residual_add(x, x), 2 * x)      # the status words were cleared; the context lives
    with pytest.raises(cuda.UllisCudaError) as e:
        cuda_rt.wait_selftest(0)
    assert e.value.code == cuda.ERR_ARG
