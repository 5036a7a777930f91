"""The CPU oracle against every golden vector / known-answer test the
reference holds for the Heron forward path (values transcribed from the
reference's tests/rosa.rs, tests/binary_linear.rs, tests/cmix.rs,
tests/rosa_metal.rs and the test module of src/metal.rs)."""
import numpy as np
import pytest

from conftest import pack_plane

# tests/rosa.rs:8-21
ROSA_T5_C3 = np.array([[-0.1, 2.0, 0.0], [0.4, -4.2, -1.5], [1.1, 1.2, 2.5], [-3.1, -2.2, 1.5], [2.1, -3.2, -2.5]],
                      np.float32)
ROSA_Y = [[-1, -1, 1, 1, 1], [-1, -1, 0, 1, 0], [-1, 0, -1, 1, 1]]
QKV_Q = [0, 1, 1, 0, 1, 1, 0, 0]
QKV_K = [1, 1, 0, 1, 0, 1, 1, 0]
QKV_V = [0, 1, 0, 1, 1, 0, 1, 0]
QKV_IDX = [0, 1, 0, 1, 1, 0, 1, 0]


def f16(x, oracle):
    return oracle.fp16_from_f32(np.asarray(x, np.float32))


def signs_to_bits(signs):
    return pack_plane([1 if s >= 0 else 0 for s in signs])


def test_rosa_matches_t5_c3_fixture(oracle):  # tests/rosa.rs:30-36
    for c in range(3):
        bits = oracle.bits_from_activation(ROSA_T5_C3[:, c])
        assert oracle.rosa(bits).tolist() == ROSA_Y[c]


def test_zero_activation_is_bit_zero(oracle):  # tests/rosa.rs:38-43
    assert oracle.bits_from_activation([0.0, -0.0, 1e-8, np.nan, -1.0]).tolist() == [0, 0, 1, 0, 0]


def test_qkv_matches_python_fixture(oracle):  # tests/rosa.rs:45-48
    assert oracle.rosa_qkv_ref(QKV_Q, QKV_K, QKV_V).tolist() == QKV_IDX


def test_qkv_output_is_plus_or_minus_e(oracle):  # tests/rosa.rs:50-55
    out = oracle.rosa_qkv_out_batched(QKV_IDX, f16([0.25], oracle), 1, 8, 1)
    assert out.tolist() == [-0.25, 0.25, -0.25, 0.25, 0.25, -0.25, 0.25, -0.25]


def test_incremental_push_and_reset(oracle):  # tests/rosa.rs:57-88
    sam = oracle.RosaSam(8)
    first = [sam.push(q, k, v) for q, k, v in zip(QKV_Q, QKV_K, QKV_V)]
    sam.reset()
    second = [sam.push(q, k, v) for q, k, v in zip(QKV_Q, QKV_K, QKV_V)]
    assert first == QKV_IDX and second == QKV_IDX


def test_qkv_same_streams_collapse_unmatched_to_zero(oracle):  # tests/rosa.rs:90-98
    for c in range(3):
        bits = oracle.bits_from_activation(ROSA_T5_C3[:, c])
        assert oracle.rosa_qkv_ref(bits, bits, bits).tolist() == [max(y, 0) for y in ROSA_Y[c]]


def test_pack_bitplane_lsb_layout(oracle):  # tests/rosa.rs:150-157
    assert oracle.pack_bitplane([1, 0, 1, 1, 0, 0, 0, 1]).tolist() == [1 | (1 << 2) | (1 << 3) | (1 << 7)]
    with pytest.raises(ValueError):
        oracle.pack_bitplane([2])


def test_batched_qkv_packed_equals_unpacked(oracle):  # tests/rosa.rs:159-193
    bits = oracle.bits_from_activation(ROSA_T5_C3.reshape(-1))
    idx = oracle.rosa_qkv_batch(bits, bits, bits, 1, 5, 3)
    w = oracle.pack_bitplane(bits)
    assert (oracle.rosa_qkv_batch_packed(w, w, w, 1, 5, 3) == idx).all()
    for c in range(3):
        assert idx.reshape(5, 3)[:, c].tolist() == [max(y, 0) for y in ROSA_Y[c]]
    out = oracle.rosa_qkv_out_batched(idx, f16([0.5, 0.25, 1.0], oracle), 1, 5, 3).reshape(5, 3)
    e = np.array([0.5, 0.25, 1.0], np.float32)
    assert np.array_equal(out, (2.0 * idx.reshape(5, 3) - 1.0) * e)


def patterned_bits(batch, time, channels, salt):  # tests/rosa_metal.rs:41-52
    b, t, c = np.meshgrid(np.arange(batch), np.arange(time), np.arange(channels), indexing="ij")
    return (((t * 13 + c * 7 + b * 3 + salt) >> 2) & 1).astype(np.uint8).reshape(-1)


def test_patterned_bits_batched_equals_per_stream(oracle):  # tests/rosa_metal.rs:145-172
    B, T, C = 2, 32, 8
    q, k, v = (patterned_bits(B, T, C, s) for s in (1, 2, 3))
    idx = oracle.rosa_qkv_batch(q, k, v, B, T, C).reshape(B, T, C)
    for b in range(B):
        for c in range(C):
            sel = lambda a: a.reshape(B, T, C)[b, :, c]
            assert (oracle.rosa_qkv_ref(sel(q), sel(k), sel(v)) == idx[b, :, c]).all()


def test_binary_linear_uses_signs(oracle):  # tests/binary_linear.rs:3-11
    y = oracle.binary_linear([2.0, 3.0], signs_to_bits([1, -1]), f16([0.5], oracle), f16([0.0], oracle), 1, 2, 1)
    assert abs(y[0] + 0.5) < 1e-6
    y2 = oracle.binary_linear([2.0, 3.0], signs_to_bits([1, -1]), f16([0.5], oracle), f16([0.0], oracle), 1, 2, 1,
                              scalar=True)
    assert y2[0] == y[0]


def test_binary_linear_2x3x2(oracle):  # src/metal.rs:3805-3820 (CPU side of the comparison)
    signs = [1, -1, -1, 1, 1, 1]
    x = np.array([0.5, -1.0, 2.0, 1.0, 0.0, -0.5], np.float32)
    y = oracle.binary_linear(x, signs_to_bits(signs), f16([0.5, 0.5], oracle), f16([0, 0], oracle), 2, 3, 2)
    w = np.array(signs, np.float32).reshape(2, 3)
    assert np.allclose(y.reshape(2, 2), 0.5 * x.reshape(2, 3) @ w.T, atol=1e-6)


def tile_boundary_case():  # src/metal.rs:3907-3934
    rows, inn, out = 17, 19, 18
    signs = [1 if (o + i) % 2 == 0 else -1 for o in range(out) for i in range(inn)]
    weight = [((o * 3 + i) % 7) * 0.25 - 0.5 for o in range(out) for i in range(inn)]
    x = [((r * 5 + i) % 11) * 0.125 - 0.5 for r in range(rows) for i in range(inn)]
    return rows, inn, out, signs, np.array(weight, np.float32), np.array(x, np.float32)


def test_linears_past_tile_boundary(oracle):
    rows, inn, out, signs, weight, x = tile_boundary_case()
    bits = signs_to_bits(signs)
    y = oracle.binary_linear(x, bits, f16([0.5] * out, oracle), f16([0.0] * out, oracle), rows, inn, out)
    ys = oracle.binary_linear(x, bits, f16([0.5] * out, oracle), f16([0.0] * out, oracle), rows, inn, out, scalar=True)
    assert np.array_equal(y, ys)
    ref = 0.5 * x.reshape(rows, inn).astype(np.float64) @ np.array(signs, np.float64).reshape(out, inn).T
    assert np.allclose(y.reshape(rows, out), ref, atol=1e-5)
    yd = oracle.fp16_linear(x, f16(weight, oracle), rows, inn, out)
    assert np.array_equal(yd, oracle.fp16_linear(x, f16(weight, oracle), rows, inn, out, scalar=True))
    assert np.allclose(yd.reshape(rows, out), x.reshape(rows, inn) @ weight.reshape(out, inn).T, atol=1e-5)


def test_vectorised_linears_equal_literal_loops_bitwise(oracle):
    rng = np.random.default_rng(3)
    for rows, inn, out in [(5, 64, 37), (9, 100, 70), (4, 512, 64)]:
        x = rng.standard_normal(rows * inn).astype(np.float32)
        bits = rng.integers(0, 2 ** 32, (inn * out + 31) // 32, dtype=np.uint32)
        scale = f16(rng.uniform(0.005, 0.02, out), oracle)
        bias = f16(rng.normal(0, 0.01, out), oracle)
        assert np.array_equal(oracle.binary_linear(x, bits, scale, bias, rows, inn, out),
                              oracle.binary_linear(x, bits, scale, bias, rows, inn, out, scalar=True))
        assert np.array_equal(oracle.binary_linear(x, bits, scale, None, rows, inn, out),
                              oracle.binary_linear(x, bits, scale, None, rows, inn, out, scalar=True))
        w = f16(rng.normal(0, 0.05, inn * out), oracle)
        assert np.array_equal(oracle.fp16_linear(x, w, rows, inn, out),
                              oracle.fp16_linear(x, w, rows, inn, out, scalar=True))


def test_layer_norm_population_moments(oracle):  # tests/cmix.rs:19-31
    y = oracle.layer_norm([1.0, 2.0, 3.0], f16([1, 1, 1], oracle), f16([0, 0, 0], oracle), 1, 3)
    inv = 1.0 / np.sqrt(2.0 / 3.0 + 1e-5)
    assert np.allclose(y, (np.array([1.0, 2.0, 3.0]) - 2.0) * inv, atol=1e-5)


def test_layer_norm_affine(oracle):  # src/metal.rs:3772-3788
    w, b = [1.25, 0.75, 1.0, 0.5], [0.1, -0.2, 0.0, 0.05]
    x = np.array([1.0, 2.0, 3.0, 4.0, 0.5, -1.0, 0.0, 2.5], np.float32).reshape(2, 4)
    y = oracle.layer_norm(x, f16(w, oracle), f16(b, oracle), 2, 4).reshape(2, 4)
    wf, bf = oracle.fp16_to_f32(f16(w, oracle)), oracle.fp16_to_f32(f16(b, oracle))
    ref = (x - x.mean(1, keepdims=True)) / np.sqrt(x.var(1, keepdims=True) + 1e-5) * wf + bf
    assert np.allclose(y, ref, atol=1e-5)


def test_cmix_zero_shift_is_relu2_then_value(oracle):  # tests/cmix.rs:33-54
    y = oracle.cmix_forward([1.0, 0.0, 0.0, 1.0], f16([0, 0], oracle), signs_to_bits([1, -1, -1, 1]),
                            f16([1, 1], oracle), f16([1.0, 0.0, 0.0, 1.0], oracle), 1, 2, 2, 2)
    assert np.allclose(y, [1, 0, 0, 1], atol=1e-5)


def test_cmix_time_shift_uses_previous_token(oracle):  # tests/cmix.rs:56-72
    y = oracle.cmix_forward([2.0, 0.0, 0.0, 0.0], f16([1, 0], oracle), signs_to_bits([1, 1]), f16([1], oracle),
                            f16([1.0, 0.0], oracle), 1, 2, 2, 1)
    assert np.allclose(y, [0, 0, 4, 0], atol=1e-4)


def test_time_shift_delta(oracle):  # src/metal.rs:3628-3640 cpu_time_shift
    x = np.arange(12, dtype=np.float32).reshape(2, 3, 2) * 0.5 - 1
    xx = oracle.time_shift_delta(x, 2, 3, 2).reshape(2, 3, 2)
    assert np.array_equal(xx[:, 0], -x[:, 0])
    assert np.array_equal(xx[:, 1:], x[:, :-1] - x[:, 1:])


def test_streamed_ce_three_row_case(oracle):  # src/metal.rs:4044-4064 with cpu_streamed_ce 3642-3703
    signs = [1, -1, 1, -1, -1, 1, 1, 1]
    hidden = np.array([0.5, -0.25, 1.0, 0.0, -0.5, 0.75], np.float32)
    tokens = np.array([1, 3, 0], np.uint32)
    mean, n_valid, row_loss, logits = oracle.head_ce(hidden, signs_to_bits(signs), f16([0.5] * 4, oracle), None,
                                                     tokens, oracle.CE_NO_IGNORE, 3, 3, 2, 4, want_logits=True)
    w = np.array(signs, np.float64).reshape(4, 2)
    lg = 0.5 * hidden.reshape(3, 2).astype(np.float64) @ w.T
    assert np.allclose(logits.reshape(3, 4), lg, atol=1e-6)
    ref = [np.log(np.exp(lg[r]).sum()) - lg[r, tokens[r + 1]] for r in range(2)]
    assert n_valid == 2 and row_loss[2] == 0.0
    assert np.allclose(row_loss[:2], ref, atol=1e-6)
    assert abs(mean - np.mean(ref)) < 1e-6


def test_ce_ignore_and_sequence_boundaries(oracle):  # src/model.rs:27-39, 4530-4544
    rng = np.random.default_rng(0)
    rows, T, D, V = 8, 4, 8, 16
    hidden = rng.standard_normal(rows * D).astype(np.float32)
    bits = rng.integers(0, 2 ** 32, D * V // 32, dtype=np.uint32)
    scale = f16(np.full(V, 0.1), oracle)
    labels = rng.integers(0, V, rows).astype(np.uint32)
    mean, n_valid, rl, _ = oracle.head_ce(hidden, bits, scale, None, labels, oracle.CE_NO_IGNORE, rows, T, D, V)
    assert n_valid == 2 * (T - 1) and rl[3] == 0 and rl[7] == 0
    pad = 5
    labels[2] = pad
    labels[6] = pad
    mean2, n2, rl2, _ = oracle.head_ce(hidden, bits, scale, None, labels, pad, rows, T, D, V)
    expect_invalid = [r for r in range(rows) if r % T == T - 1 or labels[r + 1] == pad]
    assert n2 == rows - len(expect_invalid)
    assert all(rl2[r] == 0 for r in expect_invalid)
    mean3, n3, _, _ = oracle.head_ce(hidden, bits, scale, None, np.full(rows, pad, np.uint32), pad, rows, T, D, V)
    assert n3 == 0 and mean3 == 0.0


def test_fp16_conversions_match_ieee(oracle):  # src/precision.rs:23-76 vs numpy's binary16
    rng = np.random.default_rng(1)
    x = np.concatenate([rng.standard_normal(20000).astype(np.float32) * np.float32(10.0) ** rng.integers(-9, 6, 20000),
                        np.array([0.0, -0.0, 65504.0, 65520.0, 1e-8, 6e-8, 5.96e-8, 2.98e-8, np.inf, -np.inf],
                                 np.float32)]).astype(np.float32)
    with np.errstate(over="ignore"):
        assert np.array_equal(oracle.fp16_from_f32(x), x.astype(np.float16).view(np.uint16))
    allbits = np.arange(65536, dtype=np.uint16)
    finite = ~np.isnan(allbits.view(np.float16))
    assert np.array_equal(oracle.fp16_to_f32(allbits)[finite], allbits.view(np.float16).astype(np.float32)[finite])
    assert oracle.fp16_from_f32(np.array([np.nan], np.float32))[0] & 0x7fff == 0x7e00
