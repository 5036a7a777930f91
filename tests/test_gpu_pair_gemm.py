"""The CTA-pair form of the tensor-core linears (tcgen05 cta_group::2, 256 x 256 tiles) through the C ABI.
The library picks it from 4096 rows upwards; here a runtime of its own lowers that bound to 256 rows so that
every epilogue of the pair kernel (f32 store, residual add, relu^2 -> FP16, sign bits, CE partials) and the
dense-weight variant meet the CPU oracle at sizes the oracle finishes in seconds, ragged row counts included.
Tolerances are those of the tensor-core mode: activations within 1e-2 relative, mean CE within 1e-3 absolute,
Q/K/V sign bits and idx bit-exact given the same f32 input."""
import numpy as np
import pytest

from conftest import unpack_plane
from test_gpu_ops import _rosa_params, f16
from ullis_b200 import cuda

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def pair_rt():
    mp = pytest.MonkeyPatch()
    mp.setenv("ULLIS_CUDA_WS2_MIN_ROWS", "256")
    rt = cuda.CudaRuntime(0)
    rt.set_mode(cuda.MODE_FAST)
    rt.kernel_timing(True)
    yield rt
    rt.close()
    mp.undo()


@pytest.fixture(autouse=True)
def pair_kernel_must_run(pair_rt):
    """While kernel timing is on, the library puts a zero-length "(cta_pair)" entry into its timing table in front
    of every launch of the pair kernel: each test here must have produced at least one."""
    pair_rt.kernel_timing(True)      # restarts the table
    yield
    assert pair_rt.kernel_times().get("(cta_pair)", (0.0, 0))[1] >= 1


def within(got, ref, rel=1e-2):
    got, ref = np.asarray(got), np.asarray(ref)
    assert np.abs(got - ref).max() <= rel * max(np.abs(ref).max(), 1e-30)


@pytest.mark.parametrize("rows,K,N,bias", [(512, 512, 512, True), (300, 256, 1024, False), (257, 64, 256, True),
                                           (1024, 512, 2048, True)])
def test_packed_linear_store(pair_rt, oracle, rows, K, N, bias):
    rng = np.random.default_rng(rows + K + N)
    x = rng.standard_normal(rows * K).astype(np.float32)
    bits = rng.integers(0, 2 ** 32, K * N // 32, dtype=np.uint32)
    s, b = f16(rng.uniform(0.005, 0.02, N)), (f16(rng.normal(0, 0.01, N)) if bias else None)
    within(pair_rt.binary_linear(x, bits, s, b, rows, K, N), oracle.binary_linear(x, bits, s, b, rows, K, N))


def test_dense_linear_store(pair_rt, oracle):
    rows, K, N = 19000, 256, 512      # enough row tiles for the persistent dense kernel; a ragged last tile
    rng = np.random.default_rng(7)
    x = np.abs(rng.standard_normal(rows * K)).astype(np.float32)
    w = f16(rng.uniform(-1, 1, K * N) / np.sqrt(K))
    within(pair_rt.fp16_linear(x, w, rows, K, N), oracle.fp16_linear(x, w, rows, K, N))


@pytest.mark.parametrize("B,T,d", [(2, 256, 256), (3, 160, 512)])
def test_rosa_block_sign_bits_and_residual(pair_rt, oracle, B, T, d):
    rng = np.random.default_rng(B * T + d)
    p = _rosa_params(rng, d)
    x = rng.standard_normal(B * T * d).astype(np.float32)
    ref_out, t = oracle.rosa_block_forward(x, p, B, T, d, taps=True)
    got = pair_rt.rosa_block_forward(x, p, B, T, d)
    n = B * T * d
    for m in "qkv":
        assert np.array_equal(unpack_plane(got[m + "_plane"], n), t[m + "_bits"]), m
    assert np.array_equal(got["idx"], t["idx"])
    within(got["out"], ref_out)


@pytest.mark.parametrize("B,T,d,f", [(2, 256, 256, 1024), (1, 300, 512, 2048)])
def test_cmix_block_relu2(pair_rt, oracle, B, T, d, f):
    rng = np.random.default_rng(d + f)
    x = rng.standard_normal(B * T * d).astype(np.float32)
    mix = f16(rng.uniform(0, 1, d))
    kb = rng.integers(0, 2 ** 32, d * f // 32, dtype=np.uint32)
    ks = f16(rng.uniform(0.005, 0.02, f))
    val = f16(rng.uniform(-1, 1, d * f) / np.sqrt(f))
    within(pair_rt.cmix_block_forward(x, mix, kb, ks, val, B, T, d, f), oracle.cmix_forward(x, mix, kb, ks, val, B, T, d, f))


@pytest.mark.parametrize("rows,T,D,V,ignore", [(512, 32, 256, 8192, 3), (288, 32, 512, 512, None)])
def test_streamed_ce_partials(pair_rt, oracle, rows, T, D, V, ignore):
    rng = np.random.default_rng(V + rows)
    h = rng.standard_normal(rows * D).astype(np.float32)
    bits = rng.integers(0, 2 ** 32, D * V // 32, dtype=np.uint32)
    s, b = f16(rng.uniform(0.005, 0.05, V)), f16(rng.normal(0, 0.1, V))
    labels = rng.integers(0, min(V, 8), rows).astype(np.uint32)
    ig = cuda.CE_NO_IGNORE if ignore is None else ignore
    mean, nv, rl = pair_rt.streamed_ce(h, bits, s, b, labels, ig, rows, T, D, V)
    rmean, rnv, rrl, _ = oracle.head_ce(h, bits, s, b, labels, ig, rows, T, D, V)
    assert nv == rnv
    assert abs(mean - rmean) <= 1e-3
    assert np.abs(rl - rrl).max() <= 1e-2 * max(np.abs(rrl).max(), 1.0)
    assert np.array_equal(rl == 0, rrl == 0)
