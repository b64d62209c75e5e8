"""GPU parity of the unscaled GEMMs (INT8 A8W8 with de-quantisation on store, fp16 / bf16 matmul) through the C ABI.

The INT8 results are bit-exact by construction (int32 accumulation), so they are compared bit for bit: with the goldens of
the reference's own generator (tests/ut/op_kernel/quant_batch_matmul/qbmm_data/gen_data.py, committed as
tests/golden/ref_gen_kernels.npz) and with the oracle's exact integer sums at the sizes the generator's float32 matmul
can no longer pin.  The 16-bit matmuls accumulate in float32 in another order than numpy: tolerance in the tests.
"""
import os

import numpy as np
import pytest

import blaze_oracle as o
from ops_tensor_b200 import native

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def dev(x, device):
    import torch
    return torch.from_numpy(np.ascontiguousarray(x)).to(device)


def test_a8w8_matches_the_reference_generator_goldens(cuda_device):
    import torch
    d = np.load(os.path.join(GOLDEN, "ref_gen_data.npz"))
    k = np.load(os.path.join(GOLDEN, "ref_gen_kernels.npz"))
    one = torch.ones(1, dtype=torch.float32, device=cuda_device)
    for a, b, golden in ((d["qbmm_a"], d["qbmm_b"], d["qbmm_golden"]),
                         (k["a8w8_300_a"], k["a8w8_300_b"], k["a8w8_300_golden"]),
                         (k["a8w8_136_a"], k["a8w8_136_b"], k["a8w8_136_golden"])):
        a_t, b_t = dev(a, cuda_device), dev(b.T, cuda_device)          # the generator stores B as [K][N]
        out = native.dense_gemm(a_t, b_t, scale_a=one, scale_b=one, out_dtype=torch.float16)    # pertoken 1.0 x scale 1.0
        assert np.array_equal(out.cpu().numpy().view(np.uint16), golden.view(np.uint16))
        plain = native.dense_gemm(a_t, b_t, out_dtype=torch.float16)                            # no scale at all
        assert np.array_equal(plain.cpu().numpy().view(np.uint16), golden.view(np.uint16))
    assert native.device_status() == 0


@pytest.mark.parametrize("M,N,K", [(1, 8, 16), (256, 256, 128), (300, 520, 1040), (1000, 1544, 2048), (4096, 4096, 4096)])
def test_a8w8_bit_exact_with_scales_and_bias(cuda_device, M, N, K):
    """Raw int32 sums, per-tensor and per-channel de-quantisation (masked scales), int32 bias, float32 / half / bf16
    outputs, activation and residual: every output bit equals the oracle's."""
    import torch
    rng = np.random.default_rng(np.random.SeedSequence([0, 60, M, N, K]))
    a = rng.integers(-128, 128, size=(M, K), dtype=np.int8)
    b = rng.integers(-128, 128, size=(N, K), dtype=np.int8)
    bias = rng.integers(-(1 << 20), 1 << 20, size=N, dtype=np.int32)
    a_t, b_t, bias_t = dev(a, cuda_device), dev(b, cuda_device), dev(bias, cuda_device)
    sums = o.a8w8_sums(a, b, bias)
    # 1. raw sums with the bias as accumulator init
    raw = native.dense_gemm(a_t, b_t, bias=bias_t, out=torch.empty((M, N), dtype=torch.int32, device=cuda_device))
    assert np.array_equal(raw.cpu().numpy(), sums)
    raw0 = native.dense_gemm(a_t, b_t, out=torch.empty((M, N), dtype=torch.int32, device=cuda_device))
    assert np.array_equal(raw0.cpu().numpy(), o.a8w8_sums(a, b))
    # 2. per tensor: scaleA[0] * scaleB[0], mantissa masked
    sa, sb = np.float32(0.0123456789), np.float32(0.00371)
    want = o.a8w8_ref(a, b, scale=sa * sb, bias_i32=bias, out=np.float32)
    got = native.dense_gemm(a_t, b_t, scale_a=dev(np.array([sa]), cuda_device), scale_b=dev(np.array([sb]), cuda_device),
                            bias=bias_t, out_dtype=torch.float32)
    assert np.array_equal(got.cpu().numpy().view(np.uint32), want.view(np.uint32))
    # 3. per channel: one uint64 per column, float32 bits in the low word; half output as in the reference's test
    scale_n = (rng.random(N, dtype=np.float32) + np.float32(0.5)) * np.float32(2.0 ** -12)
    words = dev(o.per_channel_scale_words(scale_n), cuda_device)
    want = o.a8w8_ref(a, b, scale=scale_n, bias_i32=bias, out=np.float16)
    got = native.dense_gemm(a_t, b_t, scale_n=words, bias=bias_t, out_dtype=torch.float16)
    assert np.array_equal(got.cpu().numpy().view(np.uint16), want.view(np.uint16))
    # 4. fused epilogue: ReLU then a bf16 residual, bf16 output
    residual = o.bf16_round(rng.standard_normal((M, N), dtype=np.float32))
    want = o.a8w8_ref(a, b, scale=scale_n, act=o.ACT_RELU, residual=residual, out="bf16")
    got = native.dense_gemm(a_t, b_t, scale_n=words, residual=dev(residual, cuda_device).to(torch.bfloat16),
                            activation=native.ACT_RELU, out_dtype=torch.bfloat16)
    assert np.array_equal(got.float().cpu().numpy().view(np.uint32), want.view(np.uint32))
    assert native.device_status() == 0


def test_fp16_matmul_matches_the_reference_generator_golden(cuda_device):
    """fp16 x fp16 with float32 accumulation and a half result: the reference generator's golden
    (tests/ut/op_kernel/mat_mul/matmul_data/gen_data.py:30-31) within two half ulps (summation order)."""
    import torch
    k = np.load(os.path.join(GOLDEN, "ref_gen_kernels.npz"))
    a, b, golden = k["mm_f16_136_a"], k["mm_f16_136_b"], k["mm_f16_136_golden"].astype(np.float64)
    out = native.dense_gemm(dev(a, cuda_device), dev(b.T, cuda_device), out_dtype=torch.float16).cpu().numpy().astype(np.float64)
    assert np.all(np.abs(out - golden) <= 2.0 ** -9 * np.maximum(np.abs(golden), 1.0))
    exact = a.astype(np.float64) @ b.astype(np.float64)
    assert np.all(np.abs(out - exact) <= 2.0 ** -10 * np.maximum(np.abs(exact), 1.0) + 1e-3)
    assert native.device_status() == 0


@pytest.mark.parametrize("dtype", ["float16", "bfloat16"])
@pytest.mark.parametrize("M,N,K", [(1, 8, 8), (256, 256, 64), (300, 520, 1048), (1000, 1544, 2048)])
def test_half_and_bf16_matmul_with_epilogue(cuda_device, dtype, M, N, K):
    """16-bit operands, float32 accumulation, bias + GELU + residual in the epilogue, bf16 / float32 outputs; tolerance
    1e-2 relative (floor 2^-7 of the rms) against float64, and not above the float32 golden's own error."""
    import torch
    rng = np.random.default_rng(np.random.SeedSequence([0, 61, M, N, K]))
    t = getattr(torch, dtype)
    a_t = dev(rng.standard_normal((M, K), dtype=np.float32), cuda_device).to(t)
    b_t = dev(rng.standard_normal((N, K), dtype=np.float32) * np.float32(0.05), cuda_device).to(t)
    bias = o.bf16_round(rng.standard_normal(N, dtype=np.float32) * np.float32(0.5))
    residual = o.bf16_round(rng.standard_normal((M, N), dtype=np.float32))
    a64, b64 = a_t.double().cpu().numpy(), b_t.double().cpu().numpy()
    ref = o.matmul_ref64(a64, b64, bias, o.ACT_GELU_TANH, residual)
    gold = o.matmul_golden32(a64.astype(np.float32), b64.astype(np.float32), bias, o.ACT_GELU_TANH, residual)
    for out_dtype in (torch.bfloat16, torch.float32):
        got = native.dense_gemm(a_t, b_t, bias=dev(bias, cuda_device).to(torch.bfloat16),
                                residual=dev(residual, cuda_device).to(torch.bfloat16),
                                activation=native.ACT_GELU_TANH, out_dtype=out_dtype).double().cpu().numpy()
        assert np.all(np.isfinite(got))
        err = o.maxrel(got, ref)
        # (the float32 golden sums in another order: a half ulp of bf16, 2^-8, plus the difference of two float32 sums)
        assert err <= 1e-2 and err <= max(o.maxrel(gold, ref), 2.0 ** -8) + 2.0 ** -10, f"max relative error {err}"
    plain = native.dense_gemm(a_t, b_t, out_dtype=torch.float32).double().cpu().numpy()
    assert o.maxrel(plain, a64 @ b64.T) <= 2.0 ** -10          # float32 accumulation in the tensor core's own order
    assert native.device_status() == 0


def test_dense_gemms_through_the_contraction_api(cuda_device):
    """The same kernels behind acltensorCreateContraction / acltensorContract: INT8 operands with per-tensor scales,
    with a per-channel scale array, with raw int32 sums; bf16 operands with a fused epilogue."""
    import torch
    from ops_tensor_b200 import host as H
    M, N, K = 300, 520, 1040
    rng = np.random.default_rng(np.random.SeedSequence([0, 62]))
    a = rng.integers(-128, 128, size=(M, K), dtype=np.int8)
    b = rng.integers(-128, 128, size=(N, K), dtype=np.int8)
    bias = rng.integers(-(1 << 20), 1 << 20, size=N, dtype=np.int32)
    a_t, b_t = dev(a, cuda_device), dev(b, cuda_device)
    sa, sb = np.float32(0.021), np.float32(0.0047)
    out = torch.empty((M, N), dtype=torch.float16, device=cuda_device)
    with H.Contraction(M, N, K, scale_mode_a=H.SCALE_PER_TENSOR, scale_mode_b=H.SCALE_PER_TENSOR, a_dtype=H.R_8I,
                       b_dtype=H.R_8I, d_dtype=H.R_16F, bias=True, bias_dtype=H.R_32I) as c:
        assert c.workspace_bytes == 0
        c(a_t, dev(np.array([sa]), cuda_device), b_t, dev(np.array([sb]), cuda_device), out, bias=dev(bias, cuda_device))
    want = o.a8w8_ref(a, b, scale=sa * sb, bias_i32=bias, out=np.float16)
    assert np.array_equal(out.cpu().numpy().view(np.uint16), want.view(np.uint16))
    scale_n = (rng.random(N, dtype=np.float32) + np.float32(0.5)) * np.float32(2.0 ** -11)
    with H.Contraction(M, N, K, scale_mode_a=H.SCALE_NONE, scale_mode_b=H.SCALE_PER_CHANNEL, a_dtype=H.R_8I,
                       b_dtype=H.R_8I, d_dtype=H.R_16F) as c:
        c(a_t, None, b_t, dev(o.per_channel_scale_words(scale_n), cuda_device), out)
    want = o.a8w8_ref(a, b, scale=scale_n, out=np.float16)
    assert np.array_equal(out.cpu().numpy().view(np.uint16), want.view(np.uint16))
    sums = torch.empty((M, N), dtype=torch.int32, device=cuda_device)
    with H.Contraction(M, N, K, scale_mode_a=H.SCALE_NONE, scale_mode_b=H.SCALE_NONE, a_dtype=H.R_8I, b_dtype=H.R_8I,
                       d_dtype=H.R_32I) as c:
        c(a_t, None, b_t, None, sums)
    assert np.array_equal(sums.cpu().numpy(), o.a8w8_sums(a, b))
    # bf16 x bf16 with bias + SiLU + residual
    x = dev(rng.standard_normal((M, K), dtype=np.float32), cuda_device).to(torch.bfloat16)
    w = dev(rng.standard_normal((N, K), dtype=np.float32) * np.float32(0.05), cuda_device).to(torch.bfloat16)
    fb = o.bf16_round(rng.standard_normal(N, dtype=np.float32))
    res = o.bf16_round(rng.standard_normal((M, N), dtype=np.float32))
    y = torch.empty((M, N), dtype=torch.bfloat16, device=cuda_device)
    with H.Contraction(M, N, K, scale_mode_a=H.SCALE_NONE, scale_mode_b=H.SCALE_NONE, a_dtype=H.R_16BF, b_dtype=H.R_16BF,
                       activation=H.OP_SILU, bias=True, residual=True) as c:
        c(x, None, w, None, y, bias=dev(fb, cuda_device).to(torch.bfloat16), residual=dev(res, cuda_device).to(torch.bfloat16))
    ref = o.matmul_ref64(x.double().cpu().numpy(), w.double().cpu().numpy(), fb, o.ACT_SILU, res)
    assert o.maxrel(y.double().cpu().numpy(), ref) <= 1e-2
    # pairs the build does not offer are refused when the plan is made
    with pytest.raises(native.BlazeError) as e:
        H.Contraction(M, N, K, scale_mode_a=H.SCALE_NONE, scale_mode_b=H.SCALE_NONE, a_dtype=H.R_8I, b_dtype=H.R_16F)
    assert e.value.status == H.STATUS_NOT_SUPPORTED
    assert H.device_status() == 0
