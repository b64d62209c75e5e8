"""The CPU oracle against the committed golden vectors (no GPU)."""
import json
import os

import numpy as np
import pytest

import blaze_oracle as o

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


@pytest.fixture(scope="module")
def micro():
    with open(os.path.join(GOLDEN, "micro_vectors.json")) as f:
        return json.load(f)


def test_e4m3_hand_vectors(micro):
    x = np.array([v for v, _ in micro["e4m3"]], dtype=np.float32)
    want = np.array([c for _, c in micro["e4m3"]], dtype=np.uint8)
    assert np.array_equal(o.e4m3_encode(x), want)


def test_e2m1_hand_vectors(micro):
    x = np.array([v for v, _ in micro["e2m1"]], dtype=np.float32)
    want = np.array([c for _, c in micro["e2m1"]], dtype=np.uint8)
    assert np.array_equal(o.e2m1_encode(x), want)


def test_e8m0_hand_vectors(micro):
    for case in micro["e8m0_from_amax"]:
        got = o.e8m0_from_amax(np.array([case["amax"]], dtype=np.float32), case["emax"])[0]
        assert got == case["byte"], case


def test_nan_conventions():
    assert o.e4m3_encode(np.array([np.nan], dtype=np.float32))[0] == 0x7F
    assert o.e2m1_encode(np.array([np.nan], dtype=np.float32))[0] == 0x7
    x = np.ones((1, 32), dtype=np.float32)
    x[0, 3] = np.nan
    codes, scales = o.quant_mx(x)
    # the finite elements are still scaled by the exponent of their amax (1.0 -> 2^8 = code 0x78)
    assert scales[0, 0] == 0xFF and codes[0, 3] == 0x7F and codes[0, 0] == 0x78


def test_independent_cast_fixtures():
    d = np.load(os.path.join(GOLDEN, "narrow_float_casts.npz"))
    assert np.array_equal(o.e4m3_encode(d["e4m3_in"]), d["e4m3_codes"])
    assert np.array_equal(o.e2m1_encode(d["e2m1_in"]), d["e2m1_codes"])
    # torch's E8M0 code of 2^e is e+127; the oracle decodes it back exactly
    assert np.array_equal(o.e8m0_decode(d["e8m0_codes"]), d["e8m0_in"].astype(np.float64))


def test_decode_encode_round_trip():
    finite = ~np.isnan(o.E4M3_VALUES)
    codes = np.arange(256, dtype=np.uint8)[finite]
    back = o.e4m3_encode(o.e4m3_decode(codes))
    # +0 and -0 keep their sign bit
    assert np.array_equal(back, codes)
    assert np.array_equal(o.e2m1_encode(o.e2m1_decode(np.arange(16))), np.arange(16, dtype=np.uint8))


def test_mx_group_known_answer(micro):
    case = micro["mx_group_quarter_steps"]
    x = (0.25 * np.arange(32, dtype=np.float32))[None, :]
    codes, scales = o.quant_mx(x)
    assert scales[0, 0] == case["scale_byte"] and scales[0, 1] == 127
    for idx, code in case["codes_at"].items():
        assert codes[0, int(idx)] == code, idx


def test_mx_dot_known_answer(micro):
    c = micro["mx_dot"]
    a = np.full((1, 32), c["a_value"], dtype=np.float32)
    b = np.full((1, 32), c["b_value"], dtype=np.float32)
    qa, sa = o.quant_mx(a)
    qb, sb = o.quant_mx(b)
    assert sa[0, 0] == c["a_byte"] and sb[0, 0] == c["b_byte"]
    assert np.all(qa == c["code"]) and np.all(qb == c["code"])
    y = o.matmul_ref64(o.dequant_mx(qa, sa, 32), o.dequant_mx(qb, sb, 32))
    assert y[0, 0] == c["dot"]


def test_fp8_1x128_known_answer(micro):
    c = micro["fp8_1x128"]
    x = np.full((2, 128), c["fill"], dtype=np.float32)
    x[0, c["special_index"]] = c["special"]
    x[1, :] = 0
    codes, scale = o.quant_fp8_1x128(x)
    assert scale.view(np.uint32)[0, 0] == c["scale_bits"]
    assert scale.view(np.uint32)[1, 0] == c["zero_group_scale_bits"]
    assert codes[0, 0] == c["fill_code"] and codes[0, c["special_index"]] == c["special_code"]
    assert np.all(codes[1] == 0)


def test_fp8_block_scale_is_transpose_invariant():
    rng = np.random.default_rng(3)
    w = (rng.standard_normal((200, 300)) * 0.02).astype(np.float32)
    codes, scale = o.quant_fp8_128x128(w)                    # [N, K] view
    assert scale.shape == (3, 2)
    # the same rule applied to the [K, N] view gives the transposed codes and the transposed scale grid
    codes_t, scale_t = o.quant_fp8_128x128(np.ascontiguousarray(w.T))
    assert np.array_equal(codes_t, codes.T) and np.array_equal(scale_t, scale.T)
    deq = o.dequant_fp8_128x128(codes, scale)
    assert np.max(np.abs(deq - w)) <= np.max(np.abs(w)) * 2.0 ** -4


def test_scale_layout_and_padding(micro):
    for K, cols in micro["mx_scale_cols"]:
        assert o.mx_scale_cols(K) == cols
    x = np.ones((3, 96), dtype=np.float32)
    codes, scales = o.quant_mx(x)
    assert codes.shape == (3, 96) and scales.shape == (3, 4)
    assert np.all(scales[:, 3] == 127)                       # pad byte is 2^0, never NaN
    codes4, scales4 = o.quant_mx(x, "e2m1")
    assert codes4.shape == (3, 48) and np.array_equal(scales4[:, 3], scales[:, 3])


def test_nibble_order_and_w4_rebase(micro):
    p = micro["pack"]
    assert np.array_equal(o.e2m1_pack(np.array(p["codes"], dtype=np.uint8)), np.array(p["bytes"], dtype=np.uint8))
    assert np.array_equal(o.e2m1_unpack(np.array(p["bytes"], dtype=np.uint8)), np.array(p["codes"], dtype=np.uint8))
    r = micro["e2m1_rebase"]
    assert np.array_equal(o.e2m1_to_e4m3_rebased(np.array(r["nibbles"])), np.array(r["bytes"], dtype=np.uint8))
    # every E2M1 value is an E4M3 value; the re-based byte is that value times 2^-6 exactly
    all16 = np.arange(16)
    assert np.array_equal(o.e4m3_decode(o.e2m1_to_e4m3_rebased(all16)) * 64.0, o.e2m1_decode(all16))
    assert np.array_equal(o.e4m3_decode(o.e2m1_to_e4m3_exact(all16)), o.e2m1_decode(all16))


def test_quantisers_round_trip_error_bounds():
    rng = np.random.default_rng(11)
    x = rng.standard_normal((64, 512)).astype(np.float32)
    for elem, bound in (("e4m3", 2.0 ** -3), ("e2m1", 0.5)):
        codes, scales = o.quant_mx(x, elem)
        deq = o.dequant_mx(codes, scales, 512, elem)
        g = np.abs(x).reshape(64, 16, 32).max(axis=2)
        assert np.all(np.abs(deq - x).reshape(64, 16, 32).max(axis=2) <= bound * g + 1e-30)
    codes, scale = o.quant_fp8_1x128(x)
    deq = o.dequant_fp8_1x128(codes, scale)
    g = np.repeat(np.abs(x).reshape(64, 4, 128).max(axis=2), 128, axis=1)
    assert np.all(np.abs(deq - x) <= g * 2.0 ** -4)


def test_reference_generator_goldens():
    """The golden style the oracle adopts reproduces the goldens of the reference's own generators."""
    d = np.load(os.path.join(GOLDEN, "ref_gen_data.npz"))
    got = np.matmul(d["mm_f32_a"], d["mm_f32_b"])
    assert np.allclose(got, d["mm_f32_golden"], rtol=1e-5, atol=1e-5)
    got16 = np.matmul(d["mm_f16_a"].astype(np.float32), d["mm_f16_b"].astype(np.float32)).astype(np.float16)
    assert np.allclose(got16.astype(np.float32), d["mm_f16_golden"].astype(np.float32), rtol=2e-3, atol=2e-3)
    with np.errstate(over="ignore"):
        q = (np.matmul(d["qbmm_a"].astype(np.float32), d["qbmm_b"].astype(np.float32)) * d["qbmm_pertoken"][0]).astype(
            np.float16)
    assert np.array_equal(q, d["qbmm_golden"])               # integer-valued products: exact in float32
    # the oracle's golden path on the same data (B given K-contiguous), before the bf16 cast
    a, b = d["mm_f32_a"], d["mm_f32_b"]
    mine = o.matmul_golden32(a, np.ascontiguousarray(b.T))
    assert np.allclose(mine, o.bf16_round(d["mm_f32_golden"]), rtol=2.0 ** -7, atol=1e-5)


def test_a8w8_oracle_reproduces_the_reference_generator_bit_for_bit():
    """The INT8 path is the one GEMM whose result the reference's own generator fixes exactly (integer products, every
    float32 partial sum below 2^24 for K < 1024): the oracle's int32 sum -> float32 -> scale -> float16 must equal it."""
    d = np.load(os.path.join(GOLDEN, "ref_gen_data.npz"))
    k = np.load(os.path.join(GOLDEN, "ref_gen_kernels.npz"))
    cases = [(d["qbmm_a"], d["qbmm_b"], d["qbmm_golden"]), (k["a8w8_300_a"], k["a8w8_300_b"], k["a8w8_300_golden"]),
             (k["a8w8_136_a"], k["a8w8_136_b"], k["a8w8_136_golden"])]
    for a, b, golden in cases:
        b_nk = np.ascontiguousarray(b.T)                       # the generator stores B as [K][N]
        got = o.a8w8_ref(a, b_nk, scale=np.float32(1.0) * np.float32(1.0))
        assert got.dtype == np.float16 and np.array_equal(got.view(np.uint16), golden.view(np.uint16))
        assert np.array_equal(o.a8w8_ref(a, b_nk).view(np.uint16), golden.view(np.uint16))      # no scale at all
    # the scale loses its low 13 mantissa bits before it is applied (DEQ_SCALE_MUL)
    s = np.float32(0.0123456789)
    assert o.masked_scale(s).view(np.uint32) == (s.view(np.uint32) & 0xFFFFE000)
    a, b = cases[1][0], np.ascontiguousarray(cases[1][1].T)
    sums = o.a8w8_sums(a, b).astype(np.float32)
    assert np.array_equal(o.a8w8_ref(a, b, scale=s), (sums * o.masked_scale(s)).astype(np.float16))
    words = o.per_channel_scale_words(np.full(4, s, dtype=np.float32))
    assert words.dtype == np.uint64 and int(words[0]) == int(s.view(np.uint32))


def test_e5m2_codes_against_an_independent_cast_and_known_answers():
    """E5M2 (IEEE-like: 5 exponent, 2 mantissa bits), the other 8-bit element type of the reference's MX operand pairs:
    round to nearest even, saturating at 57344; checked against ml_dtypes' cast after the clamp that turns its
    overflow-to-infinity into saturation."""
    import ml_dtypes
    rng = np.random.default_rng(11)
    x = np.concatenate([rng.standard_normal(4096).astype(np.float32) * np.float32(s) for s in (1e-5, 1e-3, 1, 300, 3e4)])
    x = np.concatenate([x, np.array([0.0, -0.0, 57344, 57345, 61440, 65535, 1e9, -1e9, 2.0 ** -16, 2.0 ** -17,
                                     3 * 2.0 ** -17, 2.0 ** -14, 1.125, 1.375, 1.625, 1.875], dtype=np.float32)])
    want = np.clip(x, -57344, 57344).astype(ml_dtypes.float8_e5m2).view(np.uint8)
    got = o.e5m2_encode(x)
    assert np.array_equal(got, want)
    finite = np.array([c for c in range(256) if (c >> 2) & 0x1F != 31], dtype=np.uint8)
    assert np.array_equal(o.e5m2_encode(o.e5m2_decode(finite)), finite)
    # ties: 1.125 is halfway between 1.0 and 1.25 -> even mantissa (1.0); 1.375 -> 1.5; NaN -> 0x7F
    assert list(o.e5m2_encode(np.array([1.125, 1.375, np.nan], dtype=np.float32))) == [0x3C, 0x3E, 0x7F]
    # MX groups of E5M2: the shared exponent leaves the largest element in [2^15, 2^16), values above 57344 saturate
    xs = np.zeros((1, 32), dtype=np.float32)
    xs[0, :3] = [60000.0 * 8, 1.0, -3.0]
    codes, scales = o.quant_mx(xs, "e5m2")
    assert scales[0, 0] == 127 + 3 and codes[0, 0] == 0x7B                 # 480000 / 8 = 60000 -> 57344
    assert np.array_equal(o.dequant_mx(codes, scales, 32, "e5m2")[0, 1:3], np.array([1.0, -3.0]))


def test_bf16_rounding_is_nearest_even():
    x = np.array([1.0, 1.00390625, 1.01171875, -1.00390625, 3.0e38], dtype=np.float32)
    # 1 + 2^-8 ties to 1.0 (even), 1 + 3*2^-8 ties up to 1 + 2^-6
    assert np.array_equal(o.bf16_round(x)[:4], np.array([1.0, 1.0, 1.015625, -1.0], dtype=np.float32))
    assert np.array_equal(o.bf16_from_bits(o.bf16_bits(x)), o.bf16_round(x))


def test_gelu_and_epilogue_order(micro):
    for x, y in micro["gelu_tanh"]:
        assert abs(float(o.gelu_tanh(np.float64(x))) - y) < 1e-12
    acc = np.array([[1.0, -2.0]])
    out = o.epilogue(acc, bias=np.array([0.5, 0.5]), act=o.ACT_RELU, residual=np.array([[10.0, 10.0]]))
    assert np.array_equal(out, np.array([[11.5, 10.0]]))     # relu(acc + bias) + residual


def test_tile_order_and_streamk_models(micro):
    assert [list(t) for t in o.serpentine_tile_order(5, 3, 4)] == micro["serpentine_5x3_w4"]
    for m_tiles, n_tiles, w in ((7, 5, 4), (1, 56, 16), (64, 37, 16), (3, 3, 8)):
        order = o.serpentine_tile_order(m_tiles, n_tiles, w)
        assert sorted(order) == [(m, n) for m in range(m_tiles) for n in range(n_tiles)]
    s = micro["streamk_reference_units"]
    assert o.streamk_reference_split(s["m_tiles"], s["n_tiles"], s["sk"], s["cores"]) == s["units"]
    rng = np.random.default_rng(5)
    for _ in range(50):
        tiles, kb, ctas = int(rng.integers(1, 200)), int(rng.integers(1, 150)), int(rng.integers(1, 149))
        ctas = min(ctas, tiles * kb)
        parts = o.streamk_partition(tiles, kb, ctas)
        seen = np.zeros((tiles, kb), dtype=np.int32)
        for segs in parts:
            assert sum(1 for (_, k0, _) in segs if k0 > 0) <= 1          # at most one partial publisher per CTA
            for t, k0, k1 in segs:
                seen[t, k0:k1] += 1
        assert np.all(seen == 1)
        sizes = [sum(k1 - k0 for _, k0, k1 in segs) for segs in parts]
        assert max(sizes) - min(sizes) <= 1


def test_lpt_partition_properties():
    rows = o.moe_group_rows()
    assert rows.sum() == 32768 and len(rows) == 128 and (rows == 0).any()
    members, load = o.lpt_partition(rows, 8)
    assert sorted(i for m in members for i in m) == list(range(128))
    assert max(load) <= rows.sum() / 8 + rows.max()


def test_acceptance_metric():
    y64 = np.array([[1.0, -2.0], [1e-6, 4.0]])
    assert o.maxrel(y64, y64) == 0.0
    ok, e, e_ref = o.tolerance_ok(y64 * (1 + 2.0 ** -9), y64, y64 * (1 + 2.0 ** -9))
    assert ok and abs(e - 2.0 ** -9) < 1e-9
    ok, e, _ = o.tolerance_ok(y64 * 1.02, y64, y64)
    assert not ok
