"""Pins the CPU oracle against every known-answer vector the reference holds for the
quantized-linear path, against its committed torch-derived golden, and against
outputs of the reference's own Python exporter (fixtures under tests/golden/)."""
import os

import numpy as np
import pytest

import oracle
from tests import cases


def bits(a):
    return np.ascontiguousarray(a, np.float32).view(np.uint32)


# ---- decodeI4 known answers (packages/runtime/tests/format_i4_test.ts) -----

def test_i4_even_element_is_the_low_nibble():
    # format_i4_test.ts:10-15 and tools/exporter/tests/test_emit.py:588-593: q=[1,2] <-> 0xA9
    out = oracle.decode_i4([0xA9], (1, 2), [1.0], (1, 1), 2)
    assert out.tolist() == [[1.0, 2.0]]


def test_i4_exporter_byte_kat():
    # test_emit.py:595-604: q=[-7,7,0,-7] <-> bytes [0xF1,0x18]
    out = oracle.decode_i4([0xF1, 0x18], (1, 4), [1.0], (1, 1), 4)
    assert out.tolist() == [[-7.0, 7.0, 0.0, -7.0]]


def test_i4_asymmetric_pattern_positions():
    # format_i4_test.ts:17-28
    q = [((i % 7) + 1) * (1 if i % 2 == 0 else -1) for i in range(16)]
    data = cases.pack_nibbles(np.array(q) + 8)
    out = oracle.decode_i4(data, (1, 16), [0.5], (1, 1), 16)
    assert out.reshape(-1).tolist() == [v * 0.5 for v in q]


def test_i4_scale_is_indexed_row_major_by_group():
    # format_i4_test.ts:30-37
    out = oracle.decode_i4([0x99] * 8, (2, 8), [1, 2, 4, 8], (2, 2), 4)
    assert out.reshape(-1).tolist() == [1] * 4 + [2] * 4 + [4] * 4 + [8] * 4


def test_i4_vocab_table_g32():
    # format_i4_test.ts:39-66
    vocab, hidden, g = 3, 64, 32
    q = np.array([((i // hidden + i) % 15) - 7 for i in range(vocab * hidden)])
    scale = np.array([0.5, 0.25, 1, 2, 4, 8], np.float32)
    out = oracle.decode_i4(cases.pack_nibbles(q + 8), (vocab, hidden), scale, (vocab, 2), g)
    want = [np.float32(q[i] * scale[(i // hidden) * 2 + (i % hidden) // g]) for i in range(q.size)]
    assert out.reshape(-1).tolist() == want


def test_i4_rank3_weight_uses_rank2_scale():
    # format_i4_test.ts:68-96
    q = np.array([(i % 15) - 7 for i in range(32)])
    scale = np.array([0.5, 0.25, 1, 2], np.float32)
    data = cases.pack_nibbles(q + 8)
    out = oracle.decode_i4(data, (2, 4, 4), scale, (2, 2), 8)
    want = [np.float32(q[i] * scale[(i // 16) * 2 + (i % 16) // 8]) for i in range(32)]
    assert out.reshape(-1).tolist() == want
    with pytest.raises(oracle.OracleError):
        oracle.decode_i4(data, (2, 4, 4), np.ones(8, np.float32), (2, 4, 1), 4)


def test_i4_single_f32_rounding():
    # format_i4_test.ts:98-106: 0x1F with s = fround(0.1)
    s = np.float32(0.1)
    out = oracle.decode_i4([0x1F], (1, 2), [s], (1, 1), 2).reshape(-1)
    assert bits(out).tolist() == bits([np.float32(7 * np.float64(s)), np.float32(-7 * np.float64(s))]).tolist()


def test_i4_rejections():
    # format_i4_test.ts:108-141
    data = np.zeros(8, np.uint8)
    with pytest.raises(oracle.OracleError):
        oracle.decode_i4(np.zeros(7, np.uint8), (2, 8), [1, 1], (2, 1), 8)
    with pytest.raises(oracle.OracleError):
        oracle.decode_i4(data, (2, 8), [1, 1], (2, 1), 4)
    with pytest.raises(oracle.OracleError):
        oracle.decode_i4(data, (2, 8), [1, 1], (2, 1), 3)
    with pytest.raises(oracle.OracleError):
        oracle.decode_i4(data, (2, 8), [1], (2, 2), 4)
    with pytest.raises(oracle.OracleError):
        oracle.decode_i4(np.zeros(0, np.uint8), (), [], (), 16)


# ---- decodeI8 known answers (packages/runtime/tests/gpu_i8_weights_test.ts) -

def test_i8_keepdim_broadcast_kats():
    # gpu_i8_weights_test.ts:69-87
    q = np.array([127, -128, 0, 1, -1, 64], np.int8)
    assert oracle.decode_i8(q, (2, 3), [0.5, 0.25], (2, 1)).reshape(-1).tolist() == [63.5, -64, 0, 0.25, -0.25, 16]
    assert oracle.decode_i8(q, (2, 3), [1, 2, 4], (1, 3)).reshape(-1).tolist() == [127, -256, 0, 1, -2, 256]
    assert oracle.decode_i8(q, (2, 3), [2], (1, 1)).reshape(-1).tolist() == [254, -256, 0, 2, -2, 128]


def test_i8_single_f32_rounding():
    # gpu_i8_weights_test.ts:104-113
    s = np.float32(0.1)
    out = oracle.decode_i8(np.array([3, 7, 127], np.int8), (3, 1), [s], (1, 1)).reshape(-1)
    for got, q in zip(out, [3, 7, 127]):
        assert got == np.float32(q * np.float64(s))


def test_i8_rejections():
    # gpu_i8_weights_test.ts:115-133
    q = np.array([1, 2, 3, 4, 5, 6], np.int8)
    with pytest.raises(oracle.OracleError):
        oracle.decode_i8(q, (2, 3), [1, 2], (2,))
    with pytest.raises(oracle.OracleError):
        oracle.decode_i8(q, (2, 3), [1, 2, 3, 4], (2, 2))
    with pytest.raises(oracle.OracleError):
        oracle.decode_i8(q, (2, 4), [1, 2], (2, 1))


def test_i8_all_256_values_times_row_scales():
    # the value grid of gpu_i8_weights_test.ts:612-660 (every byte value in all 4 lanes)
    q = np.repeat(np.arange(256) - 128, 4).astype(np.int8).reshape(256, 4)
    scale = (0.1 + np.arange(256) * 0.003).astype(np.float32)
    out = oracle.decode_i8(q, (256, 4), scale, (256, 1))
    want = (q.astype(np.float64) * scale.astype(np.float64)[:, None]).astype(np.float32)
    assert np.array_equal(bits(out), bits(want))


# ---- f16 ---------------------------------------------------------------------

def test_f16_widening_is_exact_for_all_patterns():
    pat = np.arange(65536, dtype=np.uint16)
    got = oracle.f16_bits_to_f32(pat)
    want = pat.view(np.float16).astype(np.float32)
    nan = np.isnan(want)
    assert np.array_equal(np.isnan(got), nan)
    assert np.array_equal(bits(got[~nan]), bits(want[~nan]))


def test_f16_rounding_matches_ieee():
    rng = np.random.default_rng(1)
    x = np.concatenate([
        rng.standard_normal(20000).astype(np.float32) * np.float32(10.0) ** rng.integers(-9, 6, 20000).astype(np.float32),
        np.array([0.0, -0.0, 65504, 65519.99, 65520, 1e9, -1e9, 2.0 ** -24, 2.0 ** -25, 1.5 * 2.0 ** -25,
                  2.0 ** -14, 2.0 ** -14 - 2.0 ** -26, 1 + 2.0 ** -11, 1 + 3 * 2.0 ** -11], np.float32)])
    with np.errstate(over="ignore"):
        want = x.astype(np.float16).astype(np.float32)
    assert np.array_equal(bits(oracle.round_to_f16(x)), bits(want))


def test_bf16_rounding_is_nearest_even():
    x = np.array([1.0, 1 + 2.0 ** -8, 1 + 3 * 2.0 ** -8, 1 + 2.0 ** -9, -3.14159, 1e-30], np.float32)
    import torch
    want = torch.from_numpy(x).to(torch.bfloat16).to(torch.float32).numpy()
    assert np.array_equal(bits(oracle.round_to_bf16(x)), bits(want))


# ---- golden fixtures made from the reference checkout ------------------------

def test_exporter_int4_vectors_bit_exact(golden_dir):
    z = np.load(os.path.join(golden_dir, "exporter_vectors.npz"))
    for i in range(int(z["i4_count"])):
        n, k, g = (int(v) for v in z[f"i4_{i}_shape"])
        packed, scale, want = z[f"i4_{i}_packed"], z[f"i4_{i}_scale"], z[f"i4_{i}_dequant"]
        # the packer's bytes, restated: even flat element -> low nibble, u = q + 8
        assert np.array_equal(cases.pack_nibbles(z[f"i4_{i}_q"].astype(np.int16) + 8), packed)
        got = oracle.decode_i4(packed, (n, k), scale, (n, k // g), g)
        assert np.array_equal(bits(got), bits(want)), f"case {i}"


def test_exporter_int8_vectors_bit_exact(golden_dir):
    z = np.load(os.path.join(golden_dir, "exporter_vectors.npz"))
    for i in range(int(z["i8_count"])):
        q, scale, want = z[f"i8_{i}_q"], z[f"i8_{i}_scale"], z[f"i8_{i}_dequant"]
        got = oracle.decode_i8(q, q.shape, scale, scale.shape)
        assert np.array_equal(bits(got), bits(want)), f"case {i}"


def test_committed_i8_golden_model(golden_dir):
    """embedding(i8 table) -> linear(i8 dense) of the reference's torch-derived golden;
    tolerance is the one its e2e test uses (atol 1e-6, rtol 1e-5)."""
    z = np.load(os.path.join(golden_dir, "i8_weights_golden.npz"))
    table = oracle.decode_i8(z["table_q"], z["table_q"].shape, z["table_scale"], z["table_scale"].shape)
    dense = oracle.decode_i8(z["dense_q"], z["dense_q"].shape, z["dense_scale"], z["dense_scale"].shape)
    x = table[z["index"]]
    got = oracle.linear_f64(x, dense, z["dense_bias"])
    rep = oracle.allclose(got, z["expected"], atol=1e-6, rtol=1e-5)
    assert rep["pass"], rep
    fused = oracle.linear_i8(x, z["dense_q"], z["dense_scale"], z["dense_bias"], 3, 5)
    assert np.array_equal(bits(fused), bits(got))


# ---- linear + allclose ---------------------------------------------------------

@pytest.mark.parametrize("name,m,n,k,g", cases.REFERENCE_I4_LINEAR_CASES)
def test_reference_i4_linear_cases_agree_across_oracle_variants(name, m, n, k, g):
    x, data, q, scale, bias = cases.reference_i4_case(m, n, k, g)
    w = oracle.decode_i4(data, (n, k), scale, scale.shape, g)
    # the decoder recovers exactly q * scale
    assert np.array_equal(bits(w), bits((q.astype(np.float64) * np.repeat(scale, g, axis=1)).astype(np.float32)))
    ref = oracle.linear_f64(x, w, bias)
    want = (x.astype(np.float64) @ w.astype(np.float64).T + bias).astype(np.float32)
    assert oracle.allclose(ref, want, atol=1e-6, rtol=1e-6)["pass"]
    assert np.array_equal(bits(oracle.linear_i4(x, data, scale, bias, n, k, g)), bits(ref))
    seq = oracle.linear_i4(x, data, scale, bias, n, k, g, f64=False)
    assert np.array_equal(bits(seq), bits(oracle.linear_f32_seq(x, w, bias, fused=True)))
    assert oracle.allclose(seq, ref)["pass"]
    assert oracle.allclose(oracle.linear_f32_seq(x, w, bias, fused=False), ref)["pass"]


@pytest.mark.parametrize("name,m,n,k,gen", cases.REFERENCE_I8_LINEAR_CASES)
def test_reference_i8_linear_cases_agree_across_oracle_variants(name, m, n, k, gen):
    x, q, scale, bias = cases.reference_i8_case(m, n, k, gen)
    if gen == "row_varying":
        assert len(set(scale.tolist())) > 1
    w = oracle.decode_i8(q, (n, k), scale, (n, 1))
    ref = oracle.linear_f64(x, w, bias)
    assert np.array_equal(bits(oracle.linear_i8(x, q, scale, bias, n, k)), bits(ref))
    assert oracle.allclose(oracle.linear_i8(x, q, scale, bias, n, k, f64=False), ref)["pass"]


def test_linear_f64_is_sequential_f64_then_one_rounding():
    x = np.array([[1e8, 1.0, -1e8, 0.5]], np.float32)
    w = np.array([[1.0, 1.0, 1.0, 1.0]], np.float32)
    out = oracle.linear_f64(x, w, np.array([0.25], np.float32))
    assert out.tolist() == [[1.75]]  # an f32 accumulator would lose the 1.0
    assert oracle.linear_f32_seq(x, w, np.array([0.25], np.float32)).tolist() == [[0.75]]


def test_allclose_rule():
    # packages/runtime/src/reference/allclose.ts:47-82
    e = np.array([0.0, 1.0, 100.0, -2.0], np.float32)
    assert oracle.allclose(e + np.float32(9e-6), e)["pass"]
    assert not oracle.allclose(e + np.array([2e-5, 0, 0, 0], np.float32), e)["pass"]
    assert oracle.allclose(e * np.float32(1.0009), e)["pass"]
    assert not oracle.allclose(e * np.float32(1.0012), e)["pass"]
    rep = oracle.allclose(np.array([np.nan, 1.0], np.float32), np.array([np.nan, 1.0], np.float32))
    assert not rep["pass"] and rep["non_finite"] == 1
    with pytest.raises(oracle.OracleError):
        oracle.allclose(np.zeros(2), np.zeros(3))


# ---- integer-dot contracts (packages/runtime/src/reference/i8a8.ts) -----------

def test_quantize_rows_contract():
    x = np.array([[0.5, -1.27, 1.27, 0.005, 0.015, 0.025], [0, 0, 0, 0, 0, 0]], np.float32)
    q, s = oracle.quantize_rows(x, 2, 6)
    assert s[0] == max(np.float32(np.float32(1.27) * np.float32(1 / 127)), oracle.F32_TINY)
    assert s[1] == oracle.F32_TINY
    want = np.clip(np.rint((x[0] / s[0]).astype(np.float32)), -127, 127)
    assert q[0].tolist() == want.tolist() and q[1].tolist() == [0] * 6
    _, s_nan = oracle.quantize_rows(np.array([[1.0, np.nan]], np.float32), 1, 2)
    assert np.isnan(s_nan[0])


def test_w8a8_and_w4a8_against_plain_python_loops():
    rng = np.random.default_rng(3)
    m, n, k, g = 3, 5, 32, 16
    x = rng.standard_normal((m, k)).astype(np.float32)
    bias = rng.standard_normal(n).astype(np.float32)
    w8 = rng.integers(-127, 128, (n, k)).astype(np.int8)
    s8 = (rng.random(n).astype(np.float32) + np.float32(0.1)) * np.float32(0.01)
    xq, xs = oracle.quantize_rows(x, m, k)
    want = np.empty((m, n), np.float32)
    for r in range(m):
        for c in range(n):
            acc = int(np.dot(xq[r].astype(np.int64), w8[c].astype(np.int64)))
            comb = np.float32(xs[r] * s8[c])
            want[r, c] = np.float32(np.float64(np.float32(acc)) * np.float64(comb) + np.float64(bias[c]))
    assert np.array_equal(bits(oracle.linear_w8a8(x, w8, s8, bias)), bits(want))
    w4 = rng.integers(-7, 8, (n, k)).astype(np.int8)
    s4 = (rng.random((n, k // g)).astype(np.float32) + np.float32(0.1)) * np.float32(0.1)
    for r in range(m):
        for c in range(n):
            accf = np.float32(0)
            for gi in range(k // g):
                acci = int(np.dot(xq[r, gi * g:(gi + 1) * g].astype(np.int64), w4[c, gi * g:(gi + 1) * g].astype(np.int64)))
                accf = np.float32(np.float64(np.float32(acci)) * np.float64(s4[c, gi]) + np.float64(accf))
            want[r, c] = np.float32(np.float64(accf) * np.float64(xs[r]) + np.float64(bias[c]))
    assert np.array_equal(bits(oracle.linear_w4a8(x, w4, s4, bias, g)), bits(want))


# ---- the reference's own known-answer tests for the integer-dot contracts -----------------
# packages/runtime/tests/i8a8_reference_test.ts:42-183, restated value for value.  The expected
# numbers are the literals that file holds (written down from the contract, not from the
# implementation), so they pin kqo_quantize_rows / kqo_linear_w8a8 / kqo_linear_w4a8 to
# something the reference itself commits to.

def test_reference_kat_zero_row_scale_is_f32_tiny():
    # i8a8_reference_test.ts:42-48
    q, s = oracle.quantize_rows(np.zeros((1, 4), np.float32), 1, 4)
    assert float(s[0]) == 1.1754943508222875e-38
    assert q.tolist() == [[0, 0, 0, 0]]


def test_reference_kat_non_finite_rows_propagate_and_stay_in_their_row():
    # i8a8_reference_test.ts:54-78
    x = np.array([[1, np.nan, -3], [2, np.inf, 1], [2, -np.inf, 1], [1, 2, 3]], np.float32)
    q, s = oracle.quantize_rows(x, 4, 3)
    assert np.isnan(s[0])
    assert s[1] == np.inf and s[2] == np.inf
    assert float(s[3]) == 0.023622047156095505
    assert q[3].tolist() == [42, 85, 127]


def test_reference_kat_absolute_maximum_lands_on_127():
    # i8a8_reference_test.ts:85-91
    q, s = oracle.quantize_rows(np.array([[127, -127, 3, 0]], np.float32), 1, 4)
    assert float(s[0]) == 1.0
    assert q.tolist() == [[127, -127, 3, 0]]


def test_reference_kat_w8a8_linear_known_values():
    # i8a8_reference_test.ts:98-116
    x = np.array([[8, 3]], np.float32)
    q, s = oracle.quantize_rows(x, 1, 2)
    assert q.tolist() == [[127, 48]] and float(s[0]) == 0.06299212574958801
    out = oracle.linear_w8a8(x, np.array([[1, 2], [-3, 4]], np.int8), np.array([0.5, 0.25], np.float32),
                             np.array([1, -1], np.float32))
    assert [float(v) for v in out[0]] == [8.023621559143066, -3.9763779640197754]


def test_reference_kat_w8a8_folds_the_two_scales_first():
    # i8a8_reference_test.ts:119-133: f32(127 * f32(s * w)), not f32(f32(127 * s) * w)
    out = oracle.linear_w8a8(np.array([[0.001, 0]], np.float32), np.array([[1, 0]], np.int8),
                             np.array([0.001], np.float32), np.array([0], np.float32))
    assert float(out[0, 0]) == 9.999999974752427e-7
    assert float(out[0, 0]) != 1.0000001111620804e-6


def test_reference_kat_w4a8_linear_known_values():
    # i8a8_reference_test.ts:141-162 (group size 2)
    out = oracle.linear_w4a8(np.array([[8, 3, -2, 5]], np.float32), np.array([[1, 2, -3, 4], [7, -7, 5, -6]], np.int8),
                             np.array([[0.5, 0.25], [0.125, 2]], np.float32), np.array([1, -1], np.float32), 2)
    assert [float(v) for v in out[0]] == [14.511811256408691, -76.51968383789062]


def test_reference_kat_w4a8_flushes_every_group_to_f32():
    # i8a8_reference_test.ts:165-183: one rounding per group, not one for the whole row
    scale = np.float32(0.017009999603033066)
    out = oracle.linear_w4a8(np.array([[127, 37, 121, 20]], np.float32), np.array([[-7, -3, -7, -6]], np.int8),
                             np.array([[scale, scale]], np.float32), np.array([0], np.float32), 2)
    assert float(out[0, 0]) == -33.45867156982422
    assert float(out[0, 0]) != -33.45866775512695


# ---- the matmul's neighbours: rms_norm, sigmoid / SiLU gate, residual add ------------------
# Known answers of packages/runtime/tests/reference_ops_test.ts:73-74 (sigmoid) and :646-680
# (rms_norm), restated with the same hand-computed expectations.

def test_reference_kat_sigmoid():
    out = oracle.sigmoid(np.array([0.0, 2.0], np.float32))
    assert float(out[0]) == 0.5
    assert abs(float(out[1]) - 0.8807970779778823) <= 1e-6


def test_reference_kat_rms_norm_does_not_subtract_the_mean():
    x = np.array([[1, 2, 3, 4]], np.float32)
    inv = 1 / np.sqrt(7.5)  # mean(x^2) = 7.5
    out = oracle.rms_norm(x, np.ones(4, np.float32), 1e-12)
    assert abs(out[0, 0] - 1 * inv) <= 1e-6 and abs(out[0, 3] - 4 * inv) <= 1e-6
    assert np.all(out > 0)  # a layer norm would have made the first entries negative
    scaled = oracle.rms_norm(x, np.array([2, 0, -1, 0.5], np.float32), 1e-12)
    assert abs(scaled[0, 0] - 2 * inv) <= 1e-6 and scaled[0, 1] == 0 and abs(scaled[0, 2] + 3 * inv) <= 1e-6
    rows = oracle.rms_norm(np.array([[3, 4], [6, 8]], np.float32), np.ones(2, np.float32), 1e-12)
    assert abs(rows[0, 0] - 3 / np.sqrt(12.5)) <= 1e-6 and abs(rows[1, 0] - 6 / np.sqrt(50)) <= 1e-6


def test_reference_kat_rms_norm_eps_sits_inside_the_root():
    zeros = oracle.rms_norm(np.zeros((1, 3), np.float32), np.full(3, 5, np.float32), 1e-6)
    assert zeros.tolist() == [[0, 0, 0]]
    epsy = oracle.rms_norm(np.array([[1]], np.float32), np.ones(1, np.float32), 0.5)
    assert abs(float(epsy[0, 0]) - 1 / np.sqrt(1.5)) <= 1e-6
    with pytest.raises(oracle.OracleError):
        oracle.rms_norm(np.ones((1, 4), np.float32), np.ones(3, np.float32), 1e-6)


def test_silu_mul_and_add_round_every_node_to_f32():
    g = np.array([-3.0, -0.5, 0.0, 0.25, 4.0], np.float32)
    u = np.array([2.0, -1.5, 7.0, 0.125, -0.75], np.float32)
    s = (1.0 / (1.0 + np.exp(-g.astype(np.float64)))).astype(np.float32)
    want = ((g * s).astype(np.float32) * u).astype(np.float32)
    assert np.array_equal(bits(oracle.silu_mul(g, u)), bits(want))
    assert np.array_equal(bits(oracle.add(g, u)), bits((g + u).astype(np.float32)))
