"""CPU oracle for the Blaze quantized-matmul hot path (TEST INFRASTRUCTURE ONLY).

This module is a numpy restatement of the arithmetic the CUDA kernels must reproduce.  It is imported
only by the tests, by the smoke check and by the CPU-baseline leg of the benchmark; the product path never
calls into it.

PARITY UNPINNED: the reference (Atlas-Ascend-Fork/ops-tensor) keeps the MX multiply-accumulate inside the
un-vendored CANN toolkit (call site: include/tensor_api/impl/tensor_api/arch/cube/mmad/mmad_impl/instruction.h:108,
`asc_mmad_mx`; toolkit dependency pinned ">=8.5" in version.cmake) and ships no golden vector, known-answer test
or host quantiser for FP8 / MX data.  What the reference does fix, and what this file follows, is

* the scale and operand *layouts* in global memory
  (include/blaze/gemm/kernel/kernel_qbmm_mx.h:383-404, include/tensor_api/impl/tensor_api/tensor/layout_pattern.h:180-226),
* the group sizes (`MXFP_DIVISOR_SIZE = 64`, `MXFP_MULTI_BASE_SIZE = 2`, `PER_BLOCK_SIZE = 128`:
  include/blaze/gemm/utils/common_utils.h:59-66),
* the nibble order of packed E2M1 (include/blaze/gemm/tile/arch35/shift_w4_to_w8.h:88-99),
* the "golden style" of its data generators: up-cast to float32, `np.matmul`, scale, cast
  (tests/ut/op_kernel/mat_mul/matmul_data/gen_data.py:30-38,
   tests/ut/op_kernel/quant_batch_matmul/qbmm_data/gen_data.py:30-40),
* bias entering the sum before the activation (include/blaze/gemm/block/block_mmad_qbmm_mx.h:500-506) and the
  activation being applied after the complete K reduction
  (include/blaze/epilogue/block/block_epilogue_matmul_streamk.h:142-182),
* the stream-K work split (include/blaze/gemm/block/block_scheduler_matmul_streamk.h:59-65) and the windowed
  serpentine tile order (include/blaze/gemm/block/block_scheduler_qbmm.h:271-317).

The element formats themselves (E4M3 "fn", E2M1, E8M0) are the public OCP definitions; they are cross-checked
against ml_dtypes / torch in tests/test_oracle.py and against hand-derived vectors in tests/golden/.
"""
from __future__ import annotations

import numpy as np

# ----------------------------------------------------------------------------------------------------------
# Element formats
# ----------------------------------------------------------------------------------------------------------

E4M3_MAX = 448.0
E2M1_MAX = 6.0
E5M2_MAX = 57344.0
E5M2_EMAX = 15         # 57344 = 1.75 * 2**15
E4M3_EMAX = 8          # 448 = 1.75 * 2**8
E2M1_EMAX = 2          # 6   = 1.5  * 2**2
MX_GROUP = 32          # elements sharing one E8M0 scale
FP8_GROUP = 128        # PER_BLOCK_SIZE, include/blaze/gemm/utils/common_utils.h:59


def _e4m3_table() -> np.ndarray:
    """Value of every E4M3 (fn: no infinities, 0x7F/0xFF = NaN) code, as float32."""
    codes = np.arange(256, dtype=np.uint32)
    sign = np.where(codes & 0x80, -1.0, 1.0)
    exp = (codes >> 3) & 0xF
    man = codes & 0x7
    val = np.where(exp == 0, man * 2.0 ** -9, (8 + man) * 2.0 ** (exp.astype(np.float64) - 10))
    val = sign * val
    val[(codes & 0x7F) == 0x7F] = np.nan
    return val.astype(np.float32)


def _e2m1_table() -> np.ndarray:
    mags = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=np.float32)
    return np.concatenate([mags, -mags]).astype(np.float32)


def _e5m2_table() -> np.ndarray:
    """Value of every E5M2 code (IEEE-like: exponent 31 is infinity / NaN), as float32."""
    codes = np.arange(256, dtype=np.uint32)
    sign = np.where(codes & 0x80, -1.0, 1.0)
    exp = (codes >> 2) & 0x1F
    man = codes & 0x3
    val = np.where(exp == 0, man * 2.0 ** -16, (4 + man) * 2.0 ** (exp.astype(np.float64) - 17))
    val = np.where(exp == 31, np.where(man == 0, np.inf, np.nan), val)
    return (sign * val).astype(np.float32)


E5M2_VALUES = _e5m2_table()
E4M3_VALUES = _e4m3_table()
E2M1_VALUES = _e2m1_table()


def e4m3_decode(codes: np.ndarray) -> np.ndarray:
    return E4M3_VALUES[np.asarray(codes, dtype=np.uint8)]


def e2m1_decode(codes: np.ndarray) -> np.ndarray:
    return E2M1_VALUES[np.asarray(codes, dtype=np.uint8) & 0xF]


def e4m3_encode(x: np.ndarray) -> np.ndarray:
    """float32 -> E4M3 code, round-to-nearest-even, saturating to +-448 (infinities saturate too).

    NaN maps to 0x7F.  The sign of zero is kept (-0.0 -> 0x80).
    """
    x = np.asarray(x, dtype=np.float32)
    a = np.abs(x).astype(np.float64)
    nan = np.isnan(x)
    a = np.where(nan, 0.0, np.minimum(a, E4M3_MAX))
    # exponent of the binade, clamped at the subnormal binade (2**-6)
    with np.errstate(divide="ignore"):
        e = np.floor(np.log2(np.where(a > 0, a, 1.0)))
    e = np.maximum(e, -6.0)
    step = np.exp2(e - 3.0)                       # spacing of E4M3 values inside the binade
    r = np.rint(a / step) * step                  # np.rint rounds halves to even
    r = np.minimum(r, E4M3_MAX)
    # r is now exactly representable; turn it into a code
    with np.errstate(divide="ignore"):
        er = np.floor(np.log2(np.where(r > 0, r, 1.0)))
    sub = r < 2.0 ** -6
    exp_field = np.where(sub, 0, er + 7).astype(np.int64)
    man_field = np.where(sub, np.rint(r * 2.0 ** 9), np.rint(r / np.exp2(er) * 8.0) - 8).astype(np.int64)
    code = (exp_field << 3) | man_field
    code = np.where(np.signbit(x), code | 0x80, code)
    code = np.where(nan, 0x7F, code)
    return code.astype(np.uint8)


def e5m2_decode(codes: np.ndarray) -> np.ndarray:
    return E5M2_VALUES[np.asarray(codes, dtype=np.uint8)]


def e5m2_encode(x: np.ndarray) -> np.ndarray:
    """float32 -> E5M2 code, round-to-nearest-even, saturating to +-57344 (infinities saturate too).  NaN maps to
    0x7F.  The sign of zero is kept.  (The second 8-bit element type of the reference's MX operand pairs:
    include/tensor_api/impl/tensor_api/arch/utils/check_data_type.h:41-50.)"""
    x = np.asarray(x, dtype=np.float32)
    a = np.abs(x).astype(np.float64)
    nan = np.isnan(x)
    a = np.where(nan, 0.0, np.minimum(a, E5M2_MAX))
    with np.errstate(divide="ignore"):
        e = np.floor(np.log2(np.where(a > 0, a, 1.0)))
    e = np.maximum(e, -14.0)                      # subnormal binade
    step = np.exp2(e - 2.0)                       # spacing inside the binade (2 mantissa bits)
    r = np.minimum(np.rint(a / step) * step, E5M2_MAX)
    with np.errstate(divide="ignore"):
        er = np.floor(np.log2(np.where(r > 0, r, 1.0)))
    sub = r < 2.0 ** -14
    exp_field = np.where(sub, 0, er + 15).astype(np.int64)
    man_field = np.where(sub, np.rint(r * 2.0 ** 16), np.rint(r / np.exp2(er) * 4.0) - 4).astype(np.int64)
    code = (exp_field << 2) | man_field
    code = np.where(np.signbit(x), code | 0x80, code)
    code = np.where(nan, 0x7F, code)
    return code.astype(np.uint8)


def e2m1_encode(x: np.ndarray) -> np.ndarray:
    """float32 -> E2M1 code (4 bits in a uint8), round-to-nearest-even, saturating to +-6.

    E2M1 has no NaN; NaN maps to +6 (0x7) and is signalled by the group's scale byte (0xFF).
    """
    x = np.asarray(x, dtype=np.float32)
    a = np.abs(x).astype(np.float64)
    nan = np.isnan(x)
    a = np.where(nan, E2M1_MAX, np.minimum(a, E2M1_MAX))
    with np.errstate(divide="ignore"):
        e = np.floor(np.log2(np.where(a > 0, a, 1.0)))
    e = np.maximum(e, 0.0)                        # subnormal binade: spacing 0.5 below 1.0
    step = np.exp2(e - 1.0)
    r = np.minimum(np.rint(a / step) * step, E2M1_MAX)
    mags = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])
    code = np.searchsorted(mags, r).astype(np.int64)
    code = np.where(np.signbit(x) & ~nan, code | 0x8, code)
    return code.astype(np.uint8)


def e2m1_pack(codes: np.ndarray) -> np.ndarray:
    """Pack 4-bit codes two per byte along the last axis: element 2i in bits 0-3, 2i+1 in bits 4-7
    (include/blaze/gemm/tile/arch35/shift_w4_to_w8.h:88-99)."""
    c = np.asarray(codes, dtype=np.uint8)
    assert c.shape[-1] % 2 == 0
    return (c[..., 0::2] & 0xF) | ((c[..., 1::2] & 0xF) << 4)


def e2m1_unpack(packed: np.ndarray) -> np.ndarray:
    p = np.asarray(packed, dtype=np.uint8)
    out = np.empty(p.shape[:-1] + (p.shape[-1] * 2,), dtype=np.uint8)
    out[..., 0::2] = p & 0xF
    out[..., 1::2] = p >> 4
    return out


def e2m1_to_e4m3_rebased(codes: np.ndarray) -> np.ndarray:
    """The reference's W4->W8 expansion: the E2M1 bit pattern `s e1 e0 m` is re-based into an E4M3 byte
    `s 0 0 e1 e0 m 0 0`, which reads as the same value times 2**-6
    (include/blaze/gemm/tile/arch35/shift_w4_to_w8.h:45-108, mask 0x9C)."""
    c = np.asarray(codes, dtype=np.uint8) & 0xF
    return (((c & 0x8) << 4) | ((c & 0x7) << 2)).astype(np.uint8)


def e2m1_to_e4m3_exact(codes: np.ndarray) -> np.ndarray:
    """E4M3 code holding exactly the same value as the E2M1 code (every E2M1 value is an E4M3 value)."""
    return e4m3_encode(e2m1_decode(codes))


def e8m0_decode(b: np.ndarray) -> np.ndarray:
    """E8M0 byte -> float64 scale 2**(b-127); 0xFF is NaN."""
    b = np.asarray(b, dtype=np.uint8)
    v = np.exp2(b.astype(np.float64) - 127.0)
    return np.where(b == 0xFF, np.nan, v)


def bf16_round(x: np.ndarray) -> np.ndarray:
    """float32 -> nearest bfloat16 (ties to even), returned as float32."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    u = x.view(np.uint32).astype(np.uint64)
    rounded = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    out = rounded.astype(np.uint32).view(np.float32)
    return np.where(np.isnan(x), x, out).astype(np.float32)


def bf16_bits(x: np.ndarray) -> np.ndarray:
    """float32 -> bfloat16 bit patterns (uint16), ties to even."""
    return (bf16_round(x).view(np.uint32) >> 16).astype(np.uint16)


def bf16_from_bits(b: np.ndarray) -> np.ndarray:
    return (np.asarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


# ----------------------------------------------------------------------------------------------------------
# Quantisers
# ----------------------------------------------------------------------------------------------------------

def mx_scale_cols(K: int) -> int:
    """Bytes per row of an MX scale array: one per 32 K, padded to an even count
    (`ceil(K/64)*2`, include/blaze/gemm/kernel/kernel_qbmm_mx.h:383-385)."""
    return -(-K // 64) * 2


def e8m0_from_amax(amax: np.ndarray, emax_elem: int) -> np.ndarray:
    """Shared-exponent rule: byte = clamp(biased_exponent(amax) - emax_elem, 0, 254); NaN -> 255.

    biased_exponent is the float32 exponent field, so amax == 0 and float32 denormals give byte 0 ... except
    that an all-zero group is given the neutral byte 127 (scale 1).
    """
    amax = np.asarray(amax, dtype=np.float32)
    field = ((amax.view(np.uint32) >> 23) & 0xFF).astype(np.int64)
    b = np.clip(field - emax_elem, 0, 254)
    b = np.where(amax == 0, 127, b)
    b = np.where(np.isnan(amax), 255, b)
    return b.astype(np.uint8)


def _pow2_f32(e: np.ndarray) -> np.ndarray:
    """Exact float32 2**e for integer e in [-127, 127]."""
    return np.ldexp(np.float32(1.0), np.asarray(e, dtype=np.int32)).astype(np.float32)


def quant_mx(x: np.ndarray, elem: str = "e4m3"):
    """fp32 [rows, K] -> (codes, scales) in the MX format.

    One E8M0 byte per 32 consecutive K elements; scales are `[rows, mx_scale_cols(K)]` row-major, the layout
    the reference calls ScaleA-ND / ScaleB-DN (row = m for A, row = n for a K-contiguous B); pad bytes are
    127.  codes are `[rows, K]` uint8 for E4M3, `[rows, K/2]` packed nibbles for E2M1.
    """
    x = np.asarray(x, dtype=np.float32)
    rows, K = x.shape
    emax = {"e4m3": E4M3_EMAX, "e5m2": E5M2_EMAX, "e2m1": E2M1_EMAX}[elem]
    ng = -(-K // MX_GROUP)
    xp = np.zeros((rows, ng * MX_GROUP), dtype=np.float32)
    xp[:, :K] = x
    g = xp.reshape(rows, ng, MX_GROUP)
    absg = np.abs(g)
    amax = np.max(np.where(np.isnan(absg), 0, absg), axis=2).astype(np.float32)
    anynan = np.isnan(g).any(axis=2)
    eff = e8m0_from_amax(amax, emax).astype(np.int32)            # exponent from the finite elements of the group
    byte = np.where(anynan, 255, eff).astype(np.uint8)           # a NaN anywhere marks the whole group
    inv = _pow2_f32(127 - eff)                                   # 2**(-e)
    q = (g * inv[:, :, None]).astype(np.float32)
    if elem == "e4m3":
        codes = e4m3_encode(q).reshape(rows, ng * MX_GROUP)[:, :K]
    elif elem == "e5m2":
        codes = e5m2_encode(q).reshape(rows, ng * MX_GROUP)[:, :K]
    else:
        assert K % 2 == 0
        codes = e2m1_pack(e2m1_encode(q).reshape(rows, ng * MX_GROUP)[:, :K])
    scales = np.full((rows, mx_scale_cols(K)), 127, dtype=np.uint8)
    scales[:, :ng] = byte
    return np.ascontiguousarray(codes), scales


def dequant_mx(codes: np.ndarray, scales: np.ndarray, K: int, elem: str = "e4m3", dtype=np.float64) -> np.ndarray:
    if elem == "e4m3":
        v = e4m3_decode(codes).astype(dtype)
    elif elem == "e5m2":
        v = e5m2_decode(codes).astype(dtype)
    else:
        v = e2m1_decode(e2m1_unpack(codes)).astype(dtype)
    ng = -(-K // MX_GROUP)
    s = e8m0_decode(scales[:, :ng]).astype(dtype)
    s = np.repeat(s, MX_GROUP, axis=1)[:, :K]
    return v[:, :K] * s


def quant_fp8_1x128(x: np.ndarray):
    """fp32 [rows, K] -> (E4M3 codes [rows, K], fp32 scales [rows, ceil(K/128)]).

    scale = amax / 448 (float32 divide; 1.0 for an all-zero group), q = e4m3(x / scale) (float32 divide).
    """
    x = np.asarray(x, dtype=np.float32)
    rows, K = x.shape
    ng = -(-K // FP8_GROUP)
    xp = np.zeros((rows, ng * FP8_GROUP), dtype=np.float32)
    xp[:, :K] = x
    g = xp.reshape(rows, ng, FP8_GROUP)
    amax = np.max(np.abs(g), axis=2).astype(np.float32)
    scale = (amax / np.float32(E4M3_MAX)).astype(np.float32)
    scale = np.where(amax == 0, np.float32(1.0), scale).astype(np.float32)
    q = (g / scale[:, :, None]).astype(np.float32)
    codes = e4m3_encode(q).reshape(rows, ng * FP8_GROUP)[:, :K]
    return np.ascontiguousarray(codes), scale


def quant_fp8_128x128(w_nk: np.ndarray):
    """fp32 weight stored K-contiguous `[N, K]` -> (E4M3 codes [N, K], fp32 scales [ceil(K/128), ceil(N/128)]).

    One scale per 128(K) x 128(N) block, same rule as quant_fp8_1x128.  The scale array is indexed
    [k_block][n_block], matching B viewed as [K, N]."""
    w = np.asarray(w_nk, dtype=np.float32)
    N, K = w.shape
    nb, kb = -(-N // FP8_GROUP), -(-K // FP8_GROUP)
    wp = np.zeros((nb * FP8_GROUP, kb * FP8_GROUP), dtype=np.float32)
    wp[:N, :K] = w
    blk = wp.reshape(nb, FP8_GROUP, kb, FP8_GROUP)
    amax = np.max(np.abs(blk), axis=(1, 3)).astype(np.float32)          # [nb, kb]
    scale = (amax / np.float32(E4M3_MAX)).astype(np.float32)
    scale = np.where(amax == 0, np.float32(1.0), scale).astype(np.float32)
    q = (blk / scale[:, None, :, None]).astype(np.float32)
    codes = e4m3_encode(q).reshape(nb * FP8_GROUP, kb * FP8_GROUP)[:N, :K]
    return np.ascontiguousarray(codes), np.ascontiguousarray(scale.T)   # [kb, nb]


def dequant_fp8_1x128(codes, scale, dtype=np.float64):
    rows, K = codes.shape
    s = np.repeat(scale.astype(dtype), FP8_GROUP, axis=1)[:, :K]
    return e4m3_decode(codes).astype(dtype) * s


def dequant_fp8_128x128(codes_nk, scale_kn, dtype=np.float64):
    N, K = codes_nk.shape
    s = np.repeat(np.repeat(scale_kn.T.astype(dtype), FP8_GROUP, axis=0), FP8_GROUP, axis=1)[:N, :K]
    return e4m3_decode(codes_nk).astype(dtype) * s


# ----------------------------------------------------------------------------------------------------------
# Epilogues and matmul references
# ----------------------------------------------------------------------------------------------------------

ACT_IDENTITY, ACT_RELU, ACT_GELU_TANH, ACT_SILU, ACT_SIGMOID, ACT_TANH = 0, 1, 2, 3, 4, 5


def gelu_tanh(x):
    x = np.asarray(x)
    c = np.asarray(0.7978845608028654, dtype=x.dtype)          # sqrt(2/pi)
    k = np.asarray(0.044715, dtype=x.dtype)
    return (0.5 * x * (1.0 + np.tanh(c * (x + k * x * x * x)))).astype(x.dtype)


def epilogue(acc, bias=None, act=ACT_IDENTITY, residual=None):
    """y = act(acc + bias) + residual, in the dtype of acc."""
    y = acc
    if bias is not None:
        y = y + np.asarray(bias, dtype=acc.dtype)[None, :]
    if act == ACT_RELU:
        y = np.maximum(y, 0)
    elif act == ACT_GELU_TANH:
        y = gelu_tanh(y)
    elif act == ACT_SILU:
        y = y / (1 + np.exp(-y))
    elif act == ACT_SIGMOID:
        y = 1 / (1 + np.exp(-y))
    elif act == ACT_TANH:
        y = np.tanh(y)
    if residual is not None:
        y = y + np.asarray(residual, dtype=acc.dtype)
    return y


def matmul_ref64(a_deq64, b_deq64_nk, bias=None, act=ACT_IDENTITY, residual=None):
    """fp64 reference on de-quantised operands; B is `[N, K]`.  Not rounded to the output type."""
    return epilogue(a_deq64 @ b_deq64_nk.T, bias, act, residual)


def matmul_golden32(a_deq32, b_deq32_nk, bias=None, act=ACT_IDENTITY, residual=None):
    """Reference-style golden: float32 operands, np.matmul, float32 epilogue, bf16 (nearest-even) output."""
    acc = np.matmul(a_deq32.astype(np.float32), b_deq32_nk.astype(np.float32).T)
    return bf16_round(epilogue(acc, bias, act, residual).astype(np.float32))


def grouped_matmul_ref(a_deq, b_deq_gnk, group_rows, dtype=np.float64):
    """C[rows of group g, :] = A[rows of g, :] @ B[g].T ; group_rows = per-group row counts."""
    M = a_deq.shape[0]
    G, N, _ = b_deq_gnk.shape
    out = np.zeros((M, N), dtype=dtype)
    r0 = 0
    for g in range(G):
        r1 = r0 + int(group_rows[g])
        if r1 > r0:
            out[r0:r1] = a_deq[r0:r1].astype(dtype) @ b_deq_gnk[g].astype(dtype).T
        r0 = r1
    return out


# ------------------------------------------------------------------------------------------------ A8W8 (INT8)

DEQ_SCALE_MASK = 0xFFFFE000     # include/blaze/gemm/kernel/kernel_qbmm_cube.h:68 (DEQ_SCALE_MUL)


def masked_scale(scale) -> np.ndarray:
    """float32 scale(s) with the low 13 mantissa bits cleared, as the reference prepares them for its fix pipe
    (include/blaze/gemm/kernel/kernel_qbmm_cube.h:190-220)."""
    bits = np.asarray(scale, dtype=np.float32).view(np.uint32) & np.uint32(DEQ_SCALE_MASK)
    return bits.view(np.float32)


def per_channel_scale_words(scale_f32: np.ndarray) -> np.ndarray:
    """The per-column scale array the A8W8 kernel takes: one uint64 per column, float32 bits in the low word."""
    return np.asarray(scale_f32, dtype=np.float32).view(np.uint32).astype(np.uint64)


def a8w8_sums(a_i8: np.ndarray, b_i8_nk: np.ndarray, bias_i32=None) -> np.ndarray:
    """Exact int32 sums of an INT8 product (B given [N][K]) plus the optional int32 bias per column: the accumulator
    the reference's cube unit holds before its fix pipe (block_mmad_a8w8_fixpipe_quant.h:309, :227-234)."""
    # float64 holds these integer sums exactly (|sum| <= K * 2^14 < 2^53) and goes through BLAS
    acc = np.rint(a_i8.astype(np.float64) @ b_i8_nk.astype(np.float64).T).astype(np.int64)
    if bias_i32 is not None:
        acc = acc + np.asarray(bias_i32, dtype=np.int64)[None, :]
    assert np.all(np.abs(acc) < 2 ** 31)
    return acc.astype(np.int32)


def a8w8_ref(a_i8, b_i8_nk, scale=None, bias_i32=None, act=ACT_IDENTITY, residual=None, out=np.float16):
    """De-quantisation on store, in the reference's golden style (tests/ut/op_kernel/quant_batch_matmul/qbmm_data/
    gen_data.py:30-40: product in float32, times the scales, cast): float32(int32 sum) * masked scale -> activation ->
    + residual -> cast.  `scale` is a scalar (per tensor: scaleA * scaleB multiplied in float32 by the caller) or one
    float32 per column; None stores the plain conversion."""
    acc = a8w8_sums(a_i8, b_i8_nk, bias_i32).astype(np.float32)          # int32 -> float32, nearest even
    if scale is not None:
        acc = acc * masked_scale(scale).reshape(1, -1)
    y = epilogue(acc.astype(np.float64), None, act, residual).astype(np.float32) if (act != ACT_IDENTITY or residual is not None) else acc
    with np.errstate(over="ignore"):
        return bf16_round(y) if out == "bf16" else y.astype(out)


def maxrel(y, y64, floor_frac=2.0 ** -7):
    """max |y - y64| / max(|y64|, floor_frac * rms(y64))."""
    y = np.asarray(y, dtype=np.float64)
    y64 = np.asarray(y64, dtype=np.float64)
    rms = float(np.sqrt(np.mean(y64 * y64))) if y64.size else 0.0
    den = np.maximum(np.abs(y64), max(floor_frac * rms, 1e-300))
    return float(np.max(np.abs(y - y64) / den)) if y64.size else 0.0


def tolerance_ok(y, y64, y_golden, abs_limit=1e-2):
    """GEMM acceptance: error <= 1e-2 and not above the reference-style golden's own error, where one bf16
    ulp (2**-8 relative) is the smallest error bound asked of a bf16 result."""
    e = maxrel(y, y64)
    e_ref = maxrel(y_golden, y64)
    return (e <= abs_limit) and (e <= max(e_ref, 2.0 ** -8)), e, e_ref


# ----------------------------------------------------------------------------------------------------------
# Scheduler models
# ----------------------------------------------------------------------------------------------------------

def serpentine_tile_order(m_tiles: int, n_tiles: int, window: int = 4):
    """Tile visiting order of the reference's quantized-matmul scheduler: a linear tile id first walks the
    M tiles of a `window`-row band, then steps N; odd bands walk N backwards
    (include/blaze/gemm/block/block_scheduler_qbmm.h:271-317, WINDOW_LEN=4 common_utils.h:42)."""
    order = []
    band = 0
    m0 = 0
    while m0 < m_tiles:
        rows = min(window, m_tiles - m0)
        ns = range(n_tiles) if band % 2 == 0 else range(n_tiles - 1, -1, -1)
        for n in ns:
            for r in range(rows):
                order.append((m0 + r, n))
        m0 += rows
        band += 1
    return order


def streamk_reference_split(m_tiles: int, n_tiles: int, k_blocks_per_slice_count: int, cores: int):
    """Work-unit count of the reference's hybrid scheduler: full tiles in data-parallel rounds, the
    `tiles % cores` tail split into `sk` K slices each
    (include/blaze/gemm/block/block_scheduler_matmul_streamk.h:59-65)."""
    tiles = m_tiles * n_tiles
    tail = tiles % cores
    return (tiles - tail) + tail * k_blocks_per_slice_count


def streamk_partition(num_tiles: int, k_blocks: int, ctas: int):
    """Even stream-K split used by the B200 kernel: the num_tiles*k_blocks (tile, k-block) units are cut
    into `ctas` contiguous ranges whose lengths differ by at most one.  Returns, per CTA, a list of segments
    (tile, k_begin, k_end)."""
    total = num_tiles * k_blocks
    out = []
    for c in range(ctas):
        lo = (total * c) // ctas
        hi = (total * (c + 1)) // ctas
        segs = []
        u = lo
        while u < hi:
            t = u // k_blocks
            kb = u - t * k_blocks
            ke = min(k_blocks, kb + (hi - u))
            segs.append((t, kb, ke))
            u += ke - kb
        out.append(segs)
    return out


def lpt_partition(costs, bins: int):
    """Longest-processing-time-first placement of groups onto `bins` ranks; ties go to the rank holding
    fewer groups.  Returns (assignment list per rank, load per rank)."""
    order = sorted(range(len(costs)), key=lambda i: (-int(costs[i]), i))
    load = [0] * bins
    members = [[] for _ in range(bins)]
    for i in order:
        b = min(range(bins), key=lambda j: (load[j], len(members[j]), j))
        members[b].append(i)
        load[b] += int(costs[i])
    return members, load


# ----------------------------------------------------------------------------------------------------------
# Synthetic inputs of the five benchmark configurations
# ----------------------------------------------------------------------------------------------------------

def rng_for(cfg: int, tensor_id: int) -> np.random.Generator:
    return np.random.default_rng(np.random.SeedSequence([0, cfg, tensor_id]))


def normal_f32(cfg: int, tensor_id: int, shape, sigma: float) -> np.ndarray:
    x = rng_for(cfg, tensor_id).standard_normal(shape, dtype=np.float32)
    if sigma != 1.0:
        x *= np.float32(sigma)
    return x


def moe_group_rows(cfg: int = 4, groups: int = 128, tokens: int = 32768, alpha: float = 0.5) -> np.ndarray:
    r = rng_for(cfg, 4)
    p = r.dirichlet(np.full(groups, alpha))
    return r.multinomial(tokens, p).astype(np.int64)
