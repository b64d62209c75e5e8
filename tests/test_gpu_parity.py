"""GPU parity: the CUDA path, called through the C ABI, against the CPU oracle on the same seeded inputs.

Quantiser outputs must be bit-equal.  GEMM outputs must satisfy max relative error <= 1e-2 against the float64
de-quantised reference (floor 2^-7 * rms) and must not exceed the error of the reference-style float32 golden
(or one bf16 ulp, 2^-8, whichever is larger).  At the full benchmark sizes the float64 reference is evaluated on a
strided sample of rows.
"""
import numpy as np
import pytest

import blaze_oracle as o
from ops_tensor_b200 import host as H

pytestmark = pytest.mark.gpu

TOL = 1e-2


def dev_tensor(x, device):
    import torch
    return torch.from_numpy(np.ascontiguousarray(x)).to(device)


def bf16_tensor(x, device):
    import torch
    return dev_tensor(o.bf16_round(x.astype(np.float32)), device).to(torch.bfloat16)


def to_np(t):
    import torch
    if t.dtype == torch.bfloat16:
        return t.float().cpu().numpy()
    return t.cpu().numpy()


def assert_gemm_ok(got, ref64, golden=None):
    got = got.astype(np.float64)
    assert np.all(np.isfinite(got))
    e = o.maxrel(got, ref64)
    assert e <= TOL, f"max relative error {e}"
    if golden is not None:
        e_ref = o.maxrel(golden, ref64)
        assert e <= max(e_ref, 2.0 ** -8), f"error {e} above the float32 golden's {e_ref}"
    assert H.device_status() == 0


# ------------------------------------------------------------------------------------------------ elementwise

@pytest.mark.parametrize("n", [3, 8, 100, 1024, 1000003])
def test_elementwise_add_call_sequence(cuda_device, n):
    """The reference's ADD cases (src/add/tests/add_test.cpp:27-104: sizes 3..1024, tolerance 1e-6) plus a large one."""
    rng = np.random.default_rng(n)
    a = rng.standard_normal(n).astype(np.float32)
    c = rng.standard_normal(n).astype(np.float32)
    d = H.elementwise_add(dev_tensor(a, cuda_device), dev_tensor(c, cuda_device))
    assert np.array_equal(to_np(d), a + c)


def test_abandoned_wait_is_reported_and_context_survives(cuda_device):
    """A kernel wait that runs out of its budget returns an error status to the host; nothing hangs, nothing faults,
    and the next GEMM on the same context is still right."""
    import ctypes as C
    import torch
    from ops_tensor_b200 import native
    assert H.device_status() == 0
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert native.lib().blazeSelfTestWaitTimeout(1 << 20, stream) == H.STATUS_SUCCESS      # ~0.5 ms budget
    code = C.c_int32(0)
    assert H.api.acltensorGetDeviceStatus(None, C.byref(code)) == H.STATUS_EXECUTION_FAILED
    assert code.value == 7
    assert H.api.acltensorGetDeviceStatus(None, C.byref(code)) == H.STATUS_SUCCESS and code.value == 0
    assert native.lib().blazeSelfTestWaitTimeout(-1, stream) == H.STATUS_INVALID_VALUE
    a = np.full((128, 32), 1.0, dtype=np.float32)
    w = np.full((8, 32), 0.5, dtype=np.float32)
    got, *_ = run_mx(cuda_device, a, w)
    assert np.all(got == 16.0) and H.device_status() == 0


def test_empty_and_invalid_calls(cuda_device):
    """Edge cases of the C ABI on a live device: empty problems succeed without touching memory, a problem without K
    or with a missing / misaligned / too-small buffer is refused with the documented status, and nothing is left in
    the device status word."""
    import ctypes as C
    import torch
    from ops_tensor_b200 import native
    dev = cuda_device
    u8 = lambda *shape: torch.zeros(shape, dtype=torch.uint8, device=dev)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    lib = native.lib()
    # MX: M = 0 and N = 0 are no-ops (null pointers are fine), K = 0 is not a GEMM
    for M, N in ((0, 64), (64, 0)):
        args = native.MxGemmArgs()
        args.struct_size = C.sizeof(args)
        args.M, args.N, args.K = M, N, 128
        args.lda = args.ldb = 128
        args.ldd = max(N, 8)
        assert lib.blazeMxGemm(C.byref(args), stream) == native.STATUS_SUCCESS
    a, sa, b, sb = u8(64, 128), u8(64, 4), u8(64, 128), u8(64, 4)
    out = torch.zeros((64, 64), dtype=torch.bfloat16, device=dev)
    good = native.mx_gemm_args(a, sa, b, sb, out)
    ws = u8(native.mx_gemm_workspace_bytes(good) + 256)
    good.workspace, good.workspace_bytes = ws.data_ptr(), ws.numel()
    assert lib.blazeMxGemm(C.byref(good), stream) == native.STATUS_SUCCESS

    def variant(**kw):
        v = native.MxGemmArgs.from_buffer_copy(good)
        for k, val in kw.items():
            setattr(v, k, val)
        return lib.blazeMxGemm(C.byref(v), stream)

    assert variant(K=0) == native.STATUS_NOT_SUPPORTED
    assert variant(A=None) == native.STATUS_INVALID_VALUE
    assert variant(scaleB=None) == native.STATUS_INVALID_VALUE
    assert variant(lda=64) == native.STATUS_INVALID_VALUE                       # shorter than a row
    assert variant(lda=136) == native.STATUS_NOT_SUPPORTED                      # rows not 16-byte aligned
    assert variant(A=a.data_ptr() + 8) == native.STATUS_NOT_SUPPORTED
    assert variant(K=72) == native.STATUS_NOT_SUPPORTED                         # K % 16
    assert variant(N=60, ldd=64) == native.STATUS_NOT_SUPPORTED                 # N % 8
    assert variant(workspace_bytes=16) == native.STATUS_INSUFFICIENT_WORKSPACE
    assert variant(workspace=ws.data_ptr() + 16) == native.STATUS_INVALID_VALUE  # workspace must be 256-byte aligned
    assert variant(activation=17) == native.STATUS_NOT_SUPPORTED
    assert variant(struct_size=8) == native.STATUS_INVALID_VALUE
    # FP8: all groups empty, and a dense problem with no rows
    sa32 = torch.zeros((0, 1), dtype=torch.float32, device=dev)
    sb32 = torch.ones((3, 1, 1), dtype=torch.float32, device=dev)
    empty_rows = torch.zeros(3, dtype=torch.int64, device=dev)
    out0 = torch.zeros((0, 128), dtype=torch.bfloat16, device=dev)
    native.fp8_gemm(u8(0, 128), sa32, u8(3, 128, 128), sb32, out=out0, group_rows=empty_rows)
    native.fp8_gemm(u8(0, 128), sa32, u8(128, 128), sb32[0], out=out0)
    # quantisers: nothing to do for zero rows
    x0 = torch.zeros((0, 64), dtype=torch.float32, device=dev)
    codes, scales = H.quantize(x0, H.SCALE_MX_E8M0_VEC32)
    assert codes.shape == (0, 64) and scales.shape == (0, 2)
    torch.cuda.synchronize()
    assert H.device_status() == 0


# ------------------------------------------------------------------------------------------------ quantisers

@pytest.mark.parametrize("rows,K", [(1, 32), (4, 128), (37, 96), (256, 1024), (130, 4160), (515, 2048)])
def test_quantisers_bit_exact(cuda_device, rows, K):
    rng = np.random.default_rng(rows * 7919 + K)
    x = (rng.standard_normal((rows, K)) * rng.choice([1e-4, 1.0, 37.0, 3e4], size=(rows, 1))).astype(np.float32)
    special = np.array([0, -0.0, 448, 464, 1e9, -1e9, 2 ** -9, 3 * 2 ** -10, 1e-40, np.inf, -np.inf, 6, 5, 0.25, 0.75,
                        1.75], dtype=np.float32)
    x[0, :min(K, special.size)] = special[:min(K, special.size)]
    if rows > 2:
        x[2, :] = 0.0                                     # all-zero groups
        x[1, 5] = np.nan                                  # NaN marks its MX group
    xd = dev_tensor(x, cuda_device)
    for dtype, name in ((H.R_8F_E4M3, "e4m3"), (H.R_4F_E2M1, "e2m1"), (H.R_8F_E5M2, "e5m2")):
        codes, scales = H.quantize(xd, H.SCALE_MX_E8M0_VEC32, dtype)
        want_codes, want_scales = o.quant_mx(x, name)
        assert np.array_equal(to_np(scales), want_scales), name
        assert np.array_equal(to_np(codes), want_codes), name
    finite = np.nan_to_num(x, nan=1.0, posinf=3e38, neginf=-3e38)
    fd = dev_tensor(finite, cuda_device)
    codes, scales = H.quantize(fd, H.SCALE_FP32_1X128)
    want_codes, want_scales = o.quant_fp8_1x128(finite)
    assert np.array_equal(to_np(scales).view(np.uint32), want_scales.view(np.uint32))
    assert np.array_equal(to_np(codes), want_codes)
    codes, scales = H.quantize(fd, H.SCALE_FP32_128X128)
    want_codes, want_scales = o.quant_fp8_128x128(finite)
    assert np.array_equal(to_np(scales).view(np.uint32), want_scales.view(np.uint32))
    assert np.array_equal(to_np(codes), want_codes)
    assert H.device_status() == 0


# ------------------------------------------------------------------------------------------------ FP8, fp32 scales

def fp8_problem(cfg, M, N, K, sigma_b=0.02):
    a = o.normal_f32(cfg, 0, (M, K), 1.0)
    w = o.normal_f32(cfg, 1, (N, K), sigma_b)
    return a, w


def run_fp8(device, a, w, *, split=H.SPLIT_AUTO, act=H.OP_IDENTITY, bias=None, residual=None, sm_limit=0,
            check_quant=True):
    import torch
    M, K = a.shape
    N = w.shape[0]
    qa, sa = H.quantize(dev_tensor(a, device), H.SCALE_FP32_1X128)
    qb, sb = H.quantize(dev_tensor(w, device), H.SCALE_FP32_128X128)
    if check_quant:
        ra, rsa = o.quant_fp8_1x128(a)
        rb, rsb = o.quant_fp8_128x128(w)
        assert np.array_equal(to_np(qa), ra) and np.array_equal(to_np(sa).view(np.uint32), rsa.view(np.uint32))
        assert np.array_equal(to_np(qb), rb) and np.array_equal(to_np(sb).view(np.uint32), rsb.view(np.uint32))
    out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=device)
    bias_t = bf16_tensor(bias, device) if bias is not None else None
    res_t = bf16_tensor(residual, device) if residual is not None else None
    with H.Contraction(M, N, K, scale_mode_a=H.SCALE_FP32_1X128, scale_mode_b=H.SCALE_FP32_128X128, activation=act,
                       bias=bias is not None, residual=residual is not None, split=split, sm_limit=sm_limit) as c:
        ws = None
        if c.workspace_bytes:
            ws = torch.full((c.workspace_bytes // 4,), float("nan"), dtype=torch.float32, device=device).view(torch.uint8)
        c(qa, sa, qb, sb, out, bias=bias_t, residual=res_t, workspace=ws)
        first = to_np(out).copy()
        out.fill_(float("nan"))
        c(qa, sa, qb, sb, out, bias=bias_t, residual=res_t, workspace=ws)
        assert np.array_equal(to_np(out).view(np.uint32), first.view(np.uint32)), "two runs differ"
    return first, to_np(qa), to_np(sa), to_np(qb), to_np(sb)


def fp8_reference(qa, sa, qb, sb, act=o.ACT_IDENTITY, bias=None, residual=None, rows=None):
    da = o.dequant_fp8_1x128(qa, sa)
    db = o.dequant_fp8_128x128(qb, sb)
    if rows is not None:
        da = da[rows]
        residual = residual[rows] if residual is not None else None
    b16 = o.bf16_round(bias.astype(np.float32)) if bias is not None else None
    r16 = o.bf16_round(residual.astype(np.float32)) if residual is not None else None
    ref = o.matmul_ref64(da, db, b16, act, r16)
    gold = o.matmul_golden32(da.astype(np.float32), db.astype(np.float32), b16, act, r16)
    return ref, gold


ACT = {H.OP_IDENTITY: o.ACT_IDENTITY, H.OP_RELU: o.ACT_RELU, H.OP_GELU: o.ACT_GELU_TANH, H.OP_SILU: o.ACT_SILU,
       H.OP_SIGMOID: o.ACT_SIGMOID, H.OP_TANH: o.ACT_TANH}


@pytest.mark.parametrize("split", [H.SPLIT_DATA_PARALLEL, H.SPLIT_STREAM_K, H.SPLIT_AUTO])
def test_config1_fp8_per_group(cuda_device, split):
    """C[256,512] = A[256,1024] x B[1024,512], 1x128 / 128x128 float32 scales, bf16 output, seed 0."""
    a, w = fp8_problem(1, 256, 512, 1024)
    got, qa, sa, qb, sb = run_fp8(cuda_device, a, w, split=split)
    ref, gold = fp8_reference(qa, sa, qb, sb)
    assert_gemm_ok(got, ref, gold)


@pytest.mark.parametrize("M,N,K", [(1, 8, 16), (128, 128, 128), (100, 264, 1040), (129, 136, 144), (300, 1000, 272)])
@pytest.mark.parametrize("split", [H.SPLIT_DATA_PARALLEL, H.SPLIT_STREAM_K])
def test_fp8_ragged_shapes(cuda_device, M, N, K, split):
    a, w = fp8_problem(11, M, N, K)
    got, qa, sa, qb, sb = run_fp8(cuda_device, a, w, split=split)
    ref, gold = fp8_reference(qa, sa, qb, sb)
    assert_gemm_ok(got, ref, gold)


@pytest.mark.parametrize("act", [H.OP_IDENTITY, H.OP_RELU, H.OP_GELU, H.OP_SILU, H.OP_SIGMOID, H.OP_TANH])
def test_fp8_fused_epilogue(cuda_device, act):
    M, N, K = 200, 392, 640
    a, w = fp8_problem(12, M, N, K, sigma_b=0.05)
    bias = o.normal_f32(12, 2, (N,), 0.5)
    residual = o.normal_f32(12, 3, (M, N), 1.0)
    got, qa, sa, qb, sb = run_fp8(cuda_device, a, w, act=act, bias=bias, residual=residual, split=H.SPLIT_STREAM_K,
                                  sm_limit=37)
    ref, gold = fp8_reference(qa, sa, qb, sb, ACT[act], bias, residual)
    assert_gemm_ok(got, ref, gold)


@pytest.mark.parametrize("M", [16, 64, 128])
def test_config5_decode_streamk(cuda_device, M):
    """Stream-K decode shape: N=7168, K=18432, residual add, bf16; checked on every row."""
    N, K = 7168, 18432
    a = o.normal_f32(5, 0, (M, K), 1.0)
    w = o.normal_f32(5, 1, (N, K), 0.02)
    residual = o.normal_f32(5, 3, (M, N), 1.0)
    got, qa, sa, qb, sb = run_fp8(cuda_device, a, w, residual=residual, split=H.SPLIT_AUTO, check_quant=False)
    ref, gold = fp8_reference(qa, sa, qb, sb, residual=residual)
    assert_gemm_ok(got, ref, gold)


def run_grouped(device, cfg, group_rows, N, K, sigma_b=0.02, split=H.SPLIT_AUTO, dirty_workspace=False):
    import torch
    G = len(group_rows)
    M = int(group_rows.sum())
    a = o.normal_f32(cfg, 0, (M, K), 1.0)
    w = o.normal_f32(cfg, 1, (G * N, K), sigma_b)
    qa, sa = H.quantize(dev_tensor(a, device), H.SCALE_FP32_1X128)
    qb = torch.empty((G, N, K), dtype=torch.uint8, device=device)
    sb = torch.empty((G, -(-K // 128), -(-N // 128)), dtype=torch.float32, device=device)
    wd = dev_tensor(w, device)
    for g in range(G):
        c, s = H.quantize(wd[g * N:(g + 1) * N], H.SCALE_FP32_128X128)
        qb[g].copy_(c)
        sb[g].copy_(s)
    out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=device)
    rows_t = dev_tensor(group_rows.astype(np.int64), device)
    with H.Contraction(M, N, K, scale_mode_a=H.SCALE_FP32_1X128, scale_mode_b=H.SCALE_FP32_128X128, groups=G,
                       split=split) as c:
        ws = None
        if dirty_workspace and c.workspace_bytes:
            ws = torch.full((c.workspace_bytes,), 0xFF, dtype=torch.uint8, device=device)
        c(qa, sa, qb, sb, out, group_rows=rows_t, workspace=ws)
        if split != H.SPLIT_DATA_PARALLEL:
            first = to_np(out).copy()
            out.fill_(float("nan"))
            c(qa, sa, qb, sb, out, group_rows=rows_t, workspace=ws)
            assert np.array_equal(to_np(out).view(np.uint32), first.view(np.uint32)), "two runs differ"
    got = to_np(out)
    da = o.dequant_fp8_1x128(to_np(qa), to_np(sa))
    qb_n, sb_n = to_np(qb), to_np(sb)
    db = np.stack([o.dequant_fp8_128x128(qb_n[g], sb_n[g]) for g in range(G)])
    ref = o.grouped_matmul_ref(da, db, group_rows)
    return got, ref


def test_grouped_small_with_empty_groups(cuda_device):
    rows = np.array([0, 5, 128, 0, 129, 1, 300, 0], dtype=np.int64)
    got, ref = run_grouped(cuda_device, 14, rows, 264, 400)
    assert_gemm_ok(got, ref)


@pytest.mark.parametrize("split", [H.SPLIT_STREAM_K, H.SPLIT_AUTO, H.SPLIT_DATA_PARALLEL])
@pytest.mark.parametrize("rows,N,K", [
    ([0, 5, 128, 0, 129, 1, 300, 0], 264, 1040),               # a handful of tiles, far fewer than SMs
    ([700, 0, 64, 1500, 333, 1, 0, 2050, 129, 127], 768, 2048),   # ~1.7 tiles per SM: the case the split is for
    ([100], 128, 20480),                                       # one tile, 160 K blocks: every SM contributes to it, so
                                                               # the owner polls far more than 32 marks
])
def test_grouped_split_along_k(cuda_device, split, rows, N, K):
    """Grouped matmul with the (tile, K block) units dealt evenly over the SMs: partial tiles of ragged groups go
    through the float32 workspace (handed over dirty) and are added in CTA order; forced, chosen by the kernel's own
    cost model once it has counted the tiles, and switched off."""
    got, ref = run_grouped(cuda_device, 15, np.array(rows, dtype=np.int64), N, K, split=split, dirty_workspace=True)
    assert_gemm_ok(got, ref)


def test_config4_moe_grouped(cuda_device):
    """G=128, K=2048, N=768, 32768 tokens split Multinomial(Dirichlet(0.5)): some groups empty, some large."""
    rows = o.moe_group_rows()
    got, ref = run_grouped(cuda_device, 4, rows, 768, 2048)
    assert_gemm_ok(got, ref)


# ------------------------------------------------------------------------------------------------ MX

def run_mx(device, a, w, *, b_dtype=H.R_8F_E4M3, act=H.OP_IDENTITY, bias=None, residual=None, tile_n=0,
           check_quant=True, static_b=False, cta_pair=0, sm_limit=0):
    import torch
    M, K = a.shape
    N = w.shape[0]
    name = "e2m1" if b_dtype == H.R_4F_E2M1 else "e4m3"
    qa, sa = H.quantize(dev_tensor(a, device), H.SCALE_MX_E8M0_VEC32)
    qb, sb = H.quantize(dev_tensor(w, device), H.SCALE_MX_E8M0_VEC32, b_dtype)
    if check_quant:
        ra, rsa = o.quant_mx(a)
        rb, rsb = o.quant_mx(w, name)
        assert np.array_equal(to_np(qa), ra) and np.array_equal(to_np(sa), rsa)
        assert np.array_equal(to_np(qb), rb) and np.array_equal(to_np(sb), rsb)
    out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=device)
    bias_t = bf16_tensor(bias, device) if bias is not None else None
    res_t = bf16_tensor(residual, device) if residual is not None else None
    with H.Contraction(M, N, K, scale_mode_a=H.SCALE_MX_E8M0_VEC32, scale_mode_b=H.SCALE_MX_E8M0_VEC32, b_dtype=b_dtype,
                       activation=act, bias=bias is not None, residual=residual is not None, tile_n=tile_n,
                       b_is_static=static_b, cta_pair=cta_pair, sm_limit=sm_limit) as c:
        c(qa, sa, qb, sb, out, bias=bias_t, residual=res_t)
        first = to_np(out).copy()
        out.fill_(float("nan"))
        c(qa, sa, qb, sb, out, bias=bias_t, residual=res_t)      # second call may reuse the weight pre-pass
        assert np.array_equal(to_np(out).view(np.uint32), first.view(np.uint32)), "two runs differ"
    return first, to_np(qa), to_np(sa), to_np(qb), to_np(sb)


def mx_reference(qa, sa, qb, sb, K, name="e4m3", act=o.ACT_IDENTITY, bias=None, residual=None, rows=None):
    da = o.dequant_mx(qa if rows is None else qa[rows], sa if rows is None else sa[rows], K)
    db = o.dequant_mx(qb, sb, K, name)
    if rows is not None and residual is not None:
        residual = residual[rows]
    b16 = o.bf16_round(bias.astype(np.float32)) if bias is not None else None
    r16 = o.bf16_round(residual.astype(np.float32)) if residual is not None else None
    ref = o.matmul_ref64(da, db, b16, act, r16)
    gold = o.matmul_golden32(da.astype(np.float32), db.astype(np.float32), b16, act, r16)
    return ref, gold


@pytest.mark.parametrize("M,N,K", [(1, 8, 32), (128, 128, 128), (128, 224, 256), (300, 520, 1040), (129, 232, 96),
                                   (256, 512, 1024), (77, 456, 2064)])
@pytest.mark.parametrize("tile_n,cta_pair", [(128, 1), (224, 1), (0, 2), (256, 2)])
def test_mx_shapes_and_tails(cuda_device, M, N, K, tile_n, cta_pair):
    """Single-CTA tiles of both widths and the 2-CTA 256 x 224 / 256 x 256 tiles, on aligned and ragged shapes."""
    a = o.normal_f32(21, 0, (M, K), 1.0)
    w = o.normal_f32(21, 1, (N, K), 1.0)
    got, qa, sa, qb, sb = run_mx(cuda_device, a, w, tile_n=tile_n, cta_pair=cta_pair)
    ref, gold = mx_reference(qa, sa, qb, sb, K)
    assert_gemm_ok(got, ref, gold)


@pytest.mark.parametrize("a_dtype,b_dtype", [(H.R_8F_E5M2, H.R_8F_E5M2), (H.R_8F_E4M3, H.R_8F_E5M2),
                                             (H.R_8F_E5M2, H.R_8F_E4M3), (H.R_8F_E5M2, H.R_4F_E2M1)])
@pytest.mark.parametrize("M,N,K,cta_pair", [(300, 520, 1056, 2), (129, 232, 96, 1), (64, 1000, 4096, 1)])
def test_mx_e5m2_operand_pairs(cuda_device, a_dtype, b_dtype, M, N, K, cta_pair):
    """The 8-bit operand pairs of the reference's MX matmul (E4M3 or E5M2 on either side:
    include/tensor_api/impl/tensor_api/arch/utils/check_data_type.h:41-50), plus E5M2 activations on a 4-bit weight:
    codes and scales bit-equal to the oracle's quantiser, product within tolerance of the float64 reference."""
    import torch
    names = {H.R_8F_E4M3: "e4m3", H.R_8F_E5M2: "e5m2", H.R_4F_E2M1: "e2m1"}
    MX = H.SCALE_MX_E8M0_VEC32
    a = o.normal_f32(26, 0, (M, K), 1.0) * np.exp2(o.rng_for(26, 5).integers(-8, 9, size=(M, 1))).astype(np.float32)
    w = o.normal_f32(26, 1, (N, K), 0.05)
    bias = o.normal_f32(26, 2, (N,), 0.5)
    qa, sa = H.quantize(dev_tensor(a, cuda_device), MX, a_dtype)
    qb, sb = H.quantize(dev_tensor(w, cuda_device), MX, b_dtype)
    ra, rsa = o.quant_mx(a, names[a_dtype])
    rb, rsb = o.quant_mx(w, names[b_dtype])
    assert np.array_equal(to_np(qa), ra) and np.array_equal(to_np(sa), rsa)
    assert np.array_equal(to_np(qb), rb) and np.array_equal(to_np(sb), rsb)
    out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=cuda_device)
    with H.Contraction(M, N, K, scale_mode_a=MX, scale_mode_b=MX, a_dtype=a_dtype, b_dtype=b_dtype, activation=H.OP_RELU,
                       bias=True, cta_pair=cta_pair) as c:
        c(qa, sa, qb, sb, out, bias=bf16_tensor(bias, cuda_device))
    da = o.dequant_mx(ra, rsa, K, names[a_dtype])
    db = o.dequant_mx(rb, rsb, K, names[b_dtype])
    b16 = o.bf16_round(bias)
    ref = o.matmul_ref64(da, db, b16, o.ACT_RELU)
    gold = o.matmul_golden32(da.astype(np.float32), db.astype(np.float32), b16, o.ACT_RELU)
    assert_gemm_ok(to_np(out), ref, gold)


def test_mx_single_group_known_answer(cuda_device):
    """32 x 1.0 times 32 x 0.5 is exactly 16 (tests/golden/micro_vectors.json, mx_dot)."""
    a = np.full((128, 32), 1.0, dtype=np.float32)
    w = np.full((8, 32), 0.5, dtype=np.float32)
    got, *_ = run_mx(cuda_device, a, w)
    assert np.all(got == 16.0)


def test_mx_scale_extremes(cuda_device):
    """Rows whose groups differ by 2^40 in magnitude exercise the per-group exponents, not just one scale."""
    M, N, K = 128, 128, 256
    rng = np.random.default_rng(5)
    a = rng.standard_normal((M, K)).astype(np.float32)
    w = rng.standard_normal((N, K)).astype(np.float32)
    a *= np.exp2(rng.integers(-20, 20, size=(M, K // 32))).repeat(32, axis=1).astype(np.float32)
    w *= np.exp2(rng.integers(-20, 20, size=(N, K // 32))).repeat(32, axis=1).astype(np.float32)
    got, qa, sa, qb, sb = run_mx(cuda_device, a, w)
    ref, gold = mx_reference(qa, sa, qb, sb, K)
    assert_gemm_ok(got, ref, gold)


@pytest.mark.parametrize("cta_pair", [1, 2, 256])
@pytest.mark.parametrize("act", [H.OP_IDENTITY, H.OP_RELU, H.OP_GELU, H.OP_SILU, H.OP_SIGMOID, H.OP_TANH])
def test_mx_fused_epilogue(cuda_device, act, cta_pair):
    M, N, K = 260, 456, 512
    a = o.normal_f32(22, 0, (M, K), 1.0)
    w = o.normal_f32(22, 1, (N, K), 0.05)
    bias = o.normal_f32(22, 2, (N,), 0.5)
    residual = o.normal_f32(22, 3, (M, N), 1.0)
    got, qa, sa, qb, sb = run_mx(cuda_device, a, w, act=act, bias=bias, residual=residual,
                                 cta_pair=min(cta_pair, 2), tile_n=256 if cta_pair == 256 else 0)
    ref, gold = mx_reference(qa, sa, qb, sb, K, "e4m3", ACT[act], bias, residual)
    assert_gemm_ok(got, ref, gold)


def test_w4a8_native_and_expanded_weights_agree(cuda_device):
    """A packed E2M1 weight goes to the tensor core as it is (TMA unpacks the nibbles) when its rows are 32-byte
    aligned, and through the one-time expansion to E4M3 codes otherwise; both must give the same bits."""
    import torch
    from ops_tensor_b200 import native
    M, N, K = 300, 520, 1024
    a = o.normal_f32(26, 0, (M, K), 1.0)
    w = o.normal_f32(26, 1, (N, K), 0.02)
    qa, sa = H.quantize(dev_tensor(a, cuda_device), H.SCALE_MX_E8M0_VEC32)
    qb, sb = H.quantize(dev_tensor(w, cuda_device), H.SCALE_MX_E8M0_VEC32, H.R_4F_E2M1)
    assert qb.data_ptr() % 32 == 0
    direct = native.mx_gemm(qa, sa, qb, sb, b_elem=native.ELEM_E2M1)
    shifted = torch.empty(qb.numel() + 16, dtype=torch.uint8, device=cuda_device)[16:].view(N, K // 2)
    shifted.copy_(qb)
    assert shifted.data_ptr() % 32 == 16
    expanded = native.mx_gemm(qa, sa, shifted, sb, b_elem=native.ELEM_E2M1)
    assert torch.equal(direct.view(torch.int16), expanded.view(torch.int16))
    ref, gold = mx_reference(to_np(qa), to_np(sa), to_np(qb), to_np(sb), K, "e2m1")
    assert_gemm_ok(to_np(direct), ref, gold)


@pytest.mark.parametrize("M,N,K", [(128, 224, 128), (300, 520, 1024), (64, 1000, 4096)])
def test_mxfp4_both_operands(cuda_device, M, N, K):
    """FP4 x FP4 (the reference's other legal operand pair): A and B packed E2M1 with E8M0 scales per 32 K."""
    import torch
    a = o.normal_f32(27, 0, (M, K), 1.0)
    w = o.normal_f32(27, 1, (N, K), 0.05)
    MX = H.SCALE_MX_E8M0_VEC32
    qa, sa = H.quantize(dev_tensor(a, cuda_device), MX, H.R_4F_E2M1)
    qb, sb = H.quantize(dev_tensor(w, cuda_device), MX, H.R_4F_E2M1)
    out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=cuda_device)
    with H.Contraction(M, N, K, scale_mode_a=MX, scale_mode_b=MX, a_dtype=H.R_4F_E2M1, b_dtype=H.R_4F_E2M1) as c:
        c(qa, sa, qb, sb, out)
    da = o.dequant_mx(to_np(qa), to_np(sa), K, "e2m1")
    db = o.dequant_mx(to_np(qb), to_np(sb), K, "e2m1")
    ref = o.matmul_ref64(da, db)
    gold = o.matmul_golden32(da.astype(np.float32), db.astype(np.float32))
    assert_gemm_ok(to_np(out), ref, gold)
    # an FP4 A against an FP8 B is not an operand pair
    with pytest.raises(Exception):
        H.Contraction(M, N, K, scale_mode_a=MX, scale_mode_b=MX, a_dtype=H.R_4F_E2M1)


@pytest.mark.parametrize("M,N,K,sm_limit", [(1000, 1544, 768, 4), (512, 1024, 2048, 0), (300, 520, 256, 0)])
def test_mxfp4_double_rate_kernel(cuda_device, M, N, K, sm_limit):
    """FP4 x FP4 on kind::mxf4 (dense 4-bit tiles, K = 64 per instruction; chosen for 2-CTA tiles when K % 256 == 0)
    against the float64 reference, and against the same product computed through kind::mxf8f6f4 (tile width 224 forces
    that route): products of E2M1 codes and power-of-two scales are exact, so the two may differ only by summation
    order."""
    import torch
    a = o.normal_f32(32, 0, (M, K), 1.0)
    w = o.normal_f32(32, 1, (N, K), 0.05)
    bias = o.normal_f32(32, 2, (N,), 0.5)
    MX = H.SCALE_MX_E8M0_VEC32
    qa, sa = H.quantize(dev_tensor(a, cuda_device), MX, H.R_4F_E2M1)
    qb, sb = H.quantize(dev_tensor(w, cuda_device), MX, H.R_4F_E2M1)
    outs = []
    for tile_n in (0, 224):
        out = torch.full((M, N), float("nan"), dtype=torch.float32, device=cuda_device)
        with H.Contraction(M, N, K, scale_mode_a=MX, scale_mode_b=MX, a_dtype=H.R_4F_E2M1, b_dtype=H.R_4F_E2M1,
                           activation=H.OP_RELU, bias=True, d_dtype=H.R_32F, tile_n=tile_n, cta_pair=2,
                           sm_limit=sm_limit) as c:
            c(qa, sa, qb, sb, out, bias=bf16_tensor(bias, cuda_device))
        outs.append(out.cpu().numpy().astype(np.float64))
    da = o.dequant_mx(to_np(qa), to_np(sa), K, "e2m1")
    db = o.dequant_mx(to_np(qb), to_np(sb), K, "e2m1")
    ref = o.matmul_ref64(da, db, o.bf16_round(bias), o.ACT_RELU)
    for got in outs:
        assert np.all(np.isfinite(got))
        assert o.maxrel(got, ref) <= 2.0 ** -13
    assert o.maxrel(outs[0], outs[1]) <= 2.0 ** -13
    assert H.device_status() == 0


@pytest.mark.parametrize("M,N,K", [(128, 224, 128), (200, 448, 1024), (64, 1000, 4096), (150, 264, 96), (300, 520, 1056)])
def test_w4a8_mx(cuda_device, M, N, K):
    a = o.normal_f32(23, 0, (M, K), 1.0)
    w = o.normal_f32(23, 1, (N, K), 0.02)
    got, qa, sa, qb, sb = run_mx(cuda_device, a, w, b_dtype=H.R_4F_E2M1, static_b=True)
    ref, gold = mx_reference(qa, sa, qb, sb, K, "e2m1")
    assert_gemm_ok(got, ref, gold)


@pytest.mark.parametrize("kind", ["mx", "mx_pair256", "fp8", "fp8_streamk"])
@pytest.mark.parametrize("d_dtype", ["float16", "float32"])
def test_half_and_float32_outputs(cuda_device, kind, d_dtype):
    """The other two cast-on-store modes of the reference (float32 -> half, float32 -> float32:
    include/tensor_api/impl/tensor_api/arch/cube/utils/l0c2out_utils.h:122-132) on ragged shapes, with bias, ReLU and
    a bf16 residual."""
    import torch
    M, N, K = (300, 520, 1040) if kind.startswith("mx") else (200, 392, 640)
    tdt = getattr(torch, d_dtype)
    code = H.R_16F if d_dtype == "float16" else H.R_32F
    a = o.normal_f32(28, 0, (M, K), 1.0)
    w = o.normal_f32(28, 1, (N, K), 1.0 if kind.startswith("mx") else 0.05)
    bias = o.normal_f32(28, 2, (N,), 0.5)
    residual = o.normal_f32(28, 3, (M, N), 1.0)
    out = torch.full((M, N), float("nan"), dtype=tdt, device=cuda_device)
    if kind.startswith("mx"):
        MX = H.SCALE_MX_E8M0_VEC32
        qa, sa = H.quantize(dev_tensor(a, cuda_device), MX)
        qb, sb = H.quantize(dev_tensor(w, cuda_device), MX)
        extra = dict(cta_pair=2, tile_n=256) if kind == "mx_pair256" else dict(cta_pair=1)
        plan = H.Contraction(M, N, K, scale_mode_a=MX, scale_mode_b=MX, activation=H.OP_RELU, bias=True, residual=True,
                             d_dtype=code, **extra)
        da, db = o.dequant_mx(to_np(qa), to_np(sa), K), o.dequant_mx(to_np(qb), to_np(sb), K)
    else:
        qa, sa = H.quantize(dev_tensor(a, cuda_device), H.SCALE_FP32_1X128)
        qb, sb = H.quantize(dev_tensor(w, cuda_device), H.SCALE_FP32_128X128)
        plan = H.Contraction(M, N, K, scale_mode_a=H.SCALE_FP32_1X128, scale_mode_b=H.SCALE_FP32_128X128,
                             activation=H.OP_RELU, bias=True, residual=True, d_dtype=code,
                             split=H.SPLIT_STREAM_K if kind == "fp8_streamk" else H.SPLIT_DATA_PARALLEL)
        da, db = o.dequant_fp8_1x128(to_np(qa), to_np(sa)), o.dequant_fp8_128x128(to_np(qb), to_np(sb))
    with plan as c:
        c(qa, sa, qb, sb, out, bias=bf16_tensor(bias, cuda_device), residual=bf16_tensor(residual, cuda_device))
    got = out.float().cpu().numpy().astype(np.float64)
    ref = o.matmul_ref64(da, db, o.bf16_round(bias), o.ACT_RELU, o.bf16_round(residual))
    assert np.all(np.isfinite(got))
    # half keeps 11 significant bits, float32 24: far tighter than the bf16 bound
    bound = 2.0 ** -10 if d_dtype == "float16" else 2.0 ** -13
    assert o.maxrel(got, ref) <= bound, o.maxrel(got, ref)
    assert H.device_status() == 0


@pytest.mark.parametrize("M,N,K,pair", [(300, 520, 1040, 1), (300, 520, 1040, 2), (136, 96, 256, 1), (512, 1024, 512, 2)])
def test_mx_quantised_output_feeds_the_next_gemm(cuda_device, M, N, K, pair):
    """Fused quantising epilogue: D leaves as E4M3 codes + one E8M0 byte per 32 columns.  The float32-output run of
    the same call holds the very values the epilogue quantises, so the codes and scales must be bit-equal to the
    oracle's quantiser applied to it (including the pad byte of an odd group count); then the pair is used, as it is,
    as the A operand of a second MX GEMM."""
    import torch
    from ops_tensor_b200 import native
    a = o.normal_f32(29, 0, (M, K), 1.0)
    w1 = o.normal_f32(29, 1, (N, K), 1.0)
    bias = bf16_tensor(o.normal_f32(29, 2, (N,), 0.5), cuda_device)
    qa, sa = H.quantize(dev_tensor(a, cuda_device), H.SCALE_MX_E8M0_VEC32)
    qb, sb = H.quantize(dev_tensor(w1, cuda_device), H.SCALE_MX_E8M0_VEC32)
    kw = dict(bias=bias, activation=native.ACT_GELU_TANH, cta_pair=pair)
    f32 = native.mx_gemm(qa, sa, qb, sb, out=torch.empty((M, N), dtype=torch.float32, device=cuda_device), **kw)
    pitch = -(-N // 16) * 16                               # rows of one-byte codes must start 16 bytes apart
    codes = torch.full((M, pitch), 0xAA, dtype=torch.uint8, device=cuda_device)[:, :N]
    scales = torch.full((M, native.mx_scale_cols(N)), 0xAA, dtype=torch.uint8, device=cuda_device)
    native.mx_gemm(qa, sa, qb, sb, out=codes, scale_out=scales, **kw)
    want_codes, want_scales = o.quant_mx(to_np(f32))
    assert np.array_equal(to_np(scales), want_scales)
    assert np.array_equal(to_np(codes.contiguous()), want_codes)
    if N % 16 == 0:
        # the same through the host API: D described as E4M3 with SCALE_MODE_D = MX
        codes2 = torch.zeros((M, N), dtype=torch.uint8, device=cuda_device)
        scales2 = torch.zeros_like(scales)
        with H.Contraction(M, N, K, scale_mode_a=H.SCALE_MX_E8M0_VEC32, scale_mode_b=H.SCALE_MX_E8M0_VEC32,
                           activation=H.OP_GELU, bias=True, cta_pair=pair, d_dtype=H.R_8F_E4M3) as c:
            c(qa, sa, qb, sb, codes2, bias=bias, scale_out=scales2)
            with pytest.raises(Exception):
                c(qa, sa, qb, sb, codes2, bias=bias)                   # nowhere to put the scales
        assert torch.equal(codes2, codes.contiguous()) and torch.equal(scales2, scales)
    # second layer: D (quantised) x W2^T
    N2 = 264
    w2 = o.normal_f32(29, 3, (N2, N), 0.1)
    if N % 16 == 0:
        qb2, sb2 = H.quantize(dev_tensor(w2, cuda_device), H.SCALE_MX_E8M0_VEC32)
        out2 = native.mx_gemm(codes, scales, qb2, sb2)
        ref = o.matmul_ref64(o.dequant_mx(want_codes, want_scales, N), o.dequant_mx(to_np(qb2), to_np(sb2), N))
        assert_gemm_ok(to_np(out2), ref)
    assert H.device_status() == 0


@pytest.mark.parametrize("M,N,K,split", [(200, 392, 640, H.SPLIT_DATA_PARALLEL), (200, 392, 640, H.SPLIT_STREAM_K),
                                         (128, 1024, 2048, H.SPLIT_AUTO)])
def test_fp8_quantised_output_feeds_the_next_gemm(cuda_device, M, N, K, split):
    """FP8 kernel, quantising epilogue: E4M3 codes + one float32 scale per row per 128 columns, bit-equal to the
    oracle's 1x128 quantiser applied to the float32-output run of the same call, then used as the next GEMM's A."""
    import torch
    a = o.normal_f32(30, 0, (M, K), 1.0)
    w1 = o.normal_f32(30, 1, (N, K), 0.05)
    bias = bf16_tensor(o.normal_f32(30, 2, (N,), 0.5), cuda_device)
    A_MODE, B_MODE = H.SCALE_FP32_1X128, H.SCALE_FP32_128X128
    qa, sa = H.quantize(dev_tensor(a, cuda_device), A_MODE)
    qb, sb = H.quantize(dev_tensor(w1, cuda_device), B_MODE)
    kw = dict(scale_mode_a=A_MODE, scale_mode_b=B_MODE, activation=H.OP_RELU, bias=True, split=split)
    f32 = torch.empty((M, N), dtype=torch.float32, device=cuda_device)
    with H.Contraction(M, N, K, d_dtype=H.R_32F, **kw) as c:
        c(qa, sa, qb, sb, f32, bias=bias)
    pitch = -(-N // 16) * 16
    codes = torch.full((M, pitch), 0xAA, dtype=torch.uint8, device=cuda_device)[:, :N]
    scales = torch.full((M, -(-N // 128)), float("nan"), dtype=torch.float32, device=cuda_device)
    with H.Contraction(M, N, K, d_dtype=H.R_8F_E4M3, ldd=pitch, **kw) as c:
        c(qa, sa, qb, sb, codes, bias=bias, scale_out=scales)
    want_codes, want_scales = o.quant_fp8_1x128(to_np(f32))
    assert np.array_equal(to_np(scales).view(np.uint32), want_scales.view(np.uint32))
    assert np.array_equal(to_np(codes.contiguous()), want_codes)
    if N % 16 == 0:
        N2 = 264
        w2 = o.normal_f32(30, 3, (N2, N), 0.1)
        qb2, sb2 = H.quantize(dev_tensor(w2, cuda_device), B_MODE)
        out2 = torch.empty((M, N2), dtype=torch.bfloat16, device=cuda_device)
        with H.Contraction(M, N2, N, scale_mode_a=A_MODE, scale_mode_b=B_MODE, lda=pitch) as c:
            c(codes, scales, qb2, sb2, out2)
        ref = o.matmul_ref64(o.dequant_fp8_1x128(want_codes, want_scales), o.dequant_fp8_128x128(to_np(qb2), to_np(sb2)))
        assert_gemm_ok(to_np(out2), ref)
    assert H.device_status() == 0


@pytest.mark.parametrize("M,N,K", [(300, 520, 1040), (128, 136, 96), (512, 768, 2048)])
def test_mx_n_major_weight(cuda_device, M, N, K):
    """B stored [K][N] (N contiguous) with the scale layout the reference pairs with it, [K/64][N][2]
    (include/tensor_api/impl/tensor_api/tensor/layout_pattern.h:204-215): same bits as the K-major call, through the
    C ABI and through a descriptor whose n stride is 1."""
    import ctypes as C
    import torch
    from ops_tensor_b200 import native
    a = o.normal_f32(31, 0, (M, K), 1.0)
    w = o.normal_f32(31, 1, (N, K), 1.0)
    MX = H.SCALE_MX_E8M0_VEC32
    qa, sa = H.quantize(dev_tensor(a, cuda_device), MX)
    qb, sb = H.quantize(dev_tensor(w, cuda_device), MX)
    want = native.mx_gemm(qa, sa, qb, sb)
    ldb = -(-N // 16) * 16
    qb_t = torch.zeros((K, ldb), dtype=torch.uint8, device=cuda_device)[:, :N]
    qb_t.copy_(qb.t())
    pairs = sb.shape[1] // 2
    sb_pairs = sb.view(N, pairs, 2).permute(1, 0, 2).contiguous()            # [K/64][N][2]
    got = native.mx_gemm(qa, sa, qb_t, sb_pairs, b_n_major=True)
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))
    # host API: B described as [n, k] with strides (1, ldb)
    h = H.create_handle()
    dA = H.create_tensor_descriptor(h, [M, K], [K, 1], H.R_8F_E4M3)
    dB = H.create_tensor_descriptor(h, [N, K], [1, ldb], H.R_8F_E4M3)
    dD = H.create_tensor_descriptor(h, [M, N], [N, 1], H.R_16BF)
    op, pref, plan = C.c_void_p(), C.c_void_p(), C.c_void_p()
    H.check(H.api.acltensorCreateContraction(h, C.byref(op), dA, H.i32([0, 2]), H.OP_IDENTITY, dB, H.i32([1, 2]),
                                             H.OP_IDENTITY, None, None, H.OP_IDENTITY, dD, H.i32([0, 1]),
                                             H.COMPUTE_DESC_32F), "create")
    H.set_attribute(h, op, H.ATTR_SCALE_MODE_A, MX)
    H.set_attribute(h, op, H.ATTR_SCALE_MODE_B, MX)
    H.check(H.api.acltensorCreatePlanPreference(h, C.byref(pref), H.ALGO_DEFAULT), "pref")
    H.check(H.api.acltensorCreatePlan(h, C.byref(plan), op, pref, 2 ** 62), "plan")
    need = C.c_uint64(0)
    H.check(H.api.acltensorPlanGetRequiredWorkspace(plan, C.byref(need)), "ws")
    ws = torch.empty(need.value, dtype=torch.uint8, device=cuda_device)
    out = torch.empty((M, N), dtype=torch.bfloat16, device=cuda_device)
    aux = H.ContractionAux(sa.data_ptr(), sb_pairs.data_ptr(), None, None, None)
    H.check(H.api.acltensorContract(h, plan, None, qa.data_ptr(), qb_t.data_ptr(), None, None, out.data_ptr(),
                                    C.byref(aux), ws.data_ptr(), ws.numel(), torch.cuda.current_stream().cuda_stream),
            "contract")
    assert torch.equal(out.view(torch.int16), want.view(torch.int16))
    for obj, destroy in ((plan, H.api.acltensorDestroyPlan), (pref, H.api.acltensorDestroyPlanPreference),
                         (op, H.api.acltensorDestroyOperationDescriptor)):
        destroy(obj)
    for d in (dA, dB, dD):
        H.api.acltensorDestroyTensorDescriptor(d)
    H.api.acltensorDestroy(h)
    assert H.device_status() == 0


@pytest.mark.parametrize("M,N,K,tile_n,b_dtype", [
    (128, 1024, 8192, 128, H.R_8F_E4M3), (100, 520, 4128, 224, H.R_8F_E4M3), (16, 2048, 6144, 128, H.R_4F_E2M1),
    (128, 264, 512, 128, H.R_8F_E4M3)])
def test_mx_stream_k_decode_shapes(cuda_device, M, N, K, tile_n, b_dtype):
    """Skinny MX GEMMs (one row of 128-row tiles, long K) split along K over the SMs: the CTA that holds K step 0 of a
    tile adds the other CTAs' float32 partial tiles in CTA order and runs the fused epilogue.  Checked against the
    float64 reference, against whole-tile scheduling, and for run-to-run bit equality (run_mx calls twice)."""
    import torch
    from ops_tensor_b200 import native
    name = "e2m1" if b_dtype == H.R_4F_E2M1 else "e4m3"
    a = o.normal_f32(33, 0, (M, K), 1.0)
    w = o.normal_f32(33, 1, (N, K), 0.05)
    bias = o.normal_f32(33, 2, (N,), 0.5)
    residual = o.normal_f32(33, 3, (M, N), 1.0)
    MX = H.SCALE_MX_E8M0_VEC32
    qa, sa = H.quantize(dev_tensor(a, cuda_device), MX)
    qb, sb = H.quantize(dev_tensor(w, cuda_device), MX, b_dtype)
    a2 = o.normal_f32(33, 4, (M, K), 1.0)                # a second activation matrix for the same workspace
    qa2, sa2 = H.quantize(dev_tensor(a2, cuda_device), MX)
    outs = {}
    for split in (H.SPLIT_STREAM_K, H.SPLIT_DATA_PARALLEL):
        out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=cuda_device)
        with H.Contraction(M, N, K, scale_mode_a=MX, scale_mode_b=MX, b_dtype=b_dtype, activation=H.OP_SILU, bias=True,
                           residual=True, tile_n=tile_n, cta_pair=1, split=split) as c:
            if split == H.SPLIT_STREAM_K:
                assert c.workspace_bytes > 128 * tile_n * 4            # room for partial tiles
            # the workspace arrives dirty: every byte 0xFF, so flags read as "set" and partial tiles as NaN unless the
            # call clears and rewrites what it uses
            ws = torch.full((max(c.workspace_bytes, 256),), 0xFF, dtype=torch.uint8, device=cuda_device)
            for qx, sx in ((qa, sa), (qa, sa), (qa2, sa2), (qa, sa)):
                c(qx, sx, qb, sb, out, bias=bf16_tensor(bias, cuda_device), residual=bf16_tensor(residual, cuda_device),
                  workspace=ws)
                outs.setdefault(split, []).append(to_np(out).copy())
    first, second, other, again = outs[H.SPLIT_STREAM_K]
    assert np.array_equal(first.view(np.uint16), second.view(np.uint16)), "stream-K is not deterministic"
    assert np.array_equal(first.view(np.uint16), again.view(np.uint16)), "stale partial tiles leaked into a later call"
    ref, gold = mx_reference(to_np(qa), to_np(sa), to_np(qb), to_np(sb), K, name, o.ACT_SILU, bias, residual)
    assert_gemm_ok(first, ref, gold)
    assert_gemm_ok(outs[H.SPLIT_DATA_PARALLEL][0], ref, gold)
    ref2, gold2 = mx_reference(to_np(qa2), to_np(sa2), to_np(qb), to_np(sb), K, name, o.ACT_SILU, bias, residual)
    assert_gemm_ok(other, ref2, gold2)
    assert_gemm_ok(outs[H.SPLIT_DATA_PARALLEL][2], ref2, gold2)


def test_static_weight_plans_sharing_one_workspace(cuda_device):
    """Two plans that treat their weights as static keep their pre-pass results in the workspace; when they share one
    buffer, each call of the other plan overwrites them, and the next call must rebuild them instead of trusting the
    remembered pointers."""
    import torch
    MX = H.SCALE_MX_E8M0_VEC32
    M, N, K = 256, 520, 544            # K % 128 != 0: the packed 4-bit weight goes through the expansion pre-pass
    a = o.normal_f32(41, 0, (M, K), 1.0)
    qa, sa = H.quantize(dev_tensor(a, cuda_device), MX)
    weights = [H.quantize(dev_tensor(o.normal_f32(41, 1 + i, (N, K), 0.5), cuda_device), MX, dt)
               for i, dt in enumerate((H.R_8F_E4M3, H.R_4F_E2M1))]
    plans = [H.Contraction(M, N, K, scale_mode_a=MX, scale_mode_b=MX, b_dtype=dt, b_is_static=True, tile_n=128, cta_pair=1)
             for dt in (H.R_8F_E4M3, H.R_4F_E2M1)]
    ws = torch.empty(max(p.workspace_bytes for p in plans), dtype=torch.uint8, device=cuda_device)
    outs = []
    for which in (0, 0, 1, 0, 1, 1):
        out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=cuda_device)
        plans[which](qa, sa, *weights[which], out, workspace=ws)
        outs.append((which, to_np(out).copy()))
    for which, got in outs:
        want = next(g for w, g in outs if w == which)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
        name = "e4m3" if which == 0 else "e2m1"
        ref, gold = mx_reference(to_np(qa), to_np(sa), to_np(weights[which][0]), to_np(weights[which][1]), K, name,
                                 o.ACT_IDENTITY, None)
        assert_gemm_ok(got, ref, gold)
    for p in plans:
        p.close()


def test_calls_capture_into_a_cuda_graph(cuda_device):
    """A serving loop records the quantiser, an MX GEMM with its pre-pass and an FP8 stream-K GEMM once and replays
    them: the launch path allocates nothing and never synchronises, and the programmatic launches inside keep their
    order in the graph.  Replays on new input data must equal eager calls on the same data."""
    import torch
    M, N, K = 256, 512, 1024
    MX = H.SCALE_MX_E8M0_VEC32
    x = dev_tensor(o.normal_f32(34, 0, (M, K), 1.0), cuda_device)
    w = dev_tensor(o.normal_f32(34, 1, (N, K), 0.1), cuda_device)
    qb, sb = H.quantize(w, MX)
    qb8, sb8 = H.quantize(w, H.SCALE_FP32_128X128)
    qa = torch.empty((M, K), dtype=torch.uint8, device=cuda_device)
    sa = torch.empty((M, K // 32), dtype=torch.uint8, device=cuda_device)
    qa8 = torch.empty((M, K), dtype=torch.uint8, device=cuda_device)
    sa8 = torch.empty((M, K // 128), dtype=torch.float32, device=cuda_device)
    out_mx = torch.empty((M, N), dtype=torch.bfloat16, device=cuda_device)
    out_f8 = torch.empty((M, N), dtype=torch.bfloat16, device=cuda_device)
    mx = H.Contraction(M, N, K, scale_mode_a=MX, scale_mode_b=MX, activation=H.OP_GELU)
    f8 = H.Contraction(M, N, K, scale_mode_a=H.SCALE_FP32_1X128, scale_mode_b=H.SCALE_FP32_128X128,
                       split=H.SPLIT_STREAM_K)
    ws_mx = torch.empty(mx.workspace_bytes, dtype=torch.uint8, device=cuda_device)
    ws_f8 = torch.empty(f8.workspace_bytes, dtype=torch.uint8, device=cuda_device)

    def step(stream):
        s = stream.cuda_stream
        H.check(H.api.acltensorQuantize(None, x.data_ptr(), K, M, K, MX, H.R_8F_E4M3, qa.data_ptr(), K, sa.data_ptr(), s), "q")
        H.check(H.api.acltensorQuantize(None, x.data_ptr(), K, M, K, H.SCALE_FP32_1X128, H.R_8F_E4M3, qa8.data_ptr(), K,
                                        sa8.data_ptr(), s), "q8")
        mx(qa, sa, qb, sb, out_mx, workspace=ws_mx, stream=s)
        f8(qa8, sa8, qb8, sb8, out_f8, workspace=ws_f8, stream=s)

    side = torch.cuda.Stream(device=cuda_device)
    with torch.cuda.stream(side):
        step(side)                                   # first calls outside the capture (one-time set-up)
    side.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        step(side)
    for seed in (35, 36):
        x.copy_(dev_tensor(o.normal_f32(seed, 0, (M, K), 1.0), cuda_device))
        graph.replay()
        torch.cuda.synchronize()
        got_mx, got_f8 = out_mx.clone(), out_f8.clone()
        with torch.cuda.stream(side):
            step(side)
        side.synchronize()
        assert torch.equal(got_mx.view(torch.int16), out_mx.view(torch.int16))
        assert torch.equal(got_f8.view(torch.int16), out_f8.view(torch.int16))
        assert torch.isfinite(out_mx.float()).all() and torch.isfinite(out_f8.float()).all()
    mx.close()
    f8.close()
    assert H.device_status() == 0


def test_mx_agrees_with_vendor_mxfp8_gemm(cuda_device):
    """An independent implementation of the same format: the vendor library's MXFP8 GEMM (torch._scaled_mm with E8M0
    scales per 32 K) on the same codes and scales.  Both accumulate in float32 and round once to bf16, so they may
    differ by the order of the additions only: at most one bf16 ulp, and bit-equal almost everywhere."""
    import torch
    if not hasattr(torch, "float8_e8m0fnu"):
        pytest.skip("this torch has no E8M0 dtype")
    M, N, K = 512, 768, 1024
    a = o.normal_f32(25, 0, (M, K), 1.0) * np.exp2(o.rng_for(25, 5).integers(-6, 7, size=(M, 1))).astype(np.float32)
    w = o.normal_f32(25, 1, (N, K), 1.0)
    got, qa, sa, qb, sb = run_mx(cuda_device, a, w)

    def library_layout(scales):
        # [rows][K/32] -> 128-row x 4-group blocks of 512 bytes: byte (r % 32) * 16 + (r // 32) * 4 + g
        rows, groups = scales.shape
        t = torch.from_numpy(scales).to(cuda_device).view(rows // 128, 4, 32, groups // 4, 4)
        return t.permute(0, 3, 2, 1, 4).contiguous().view(-1).view(torch.float8_e8m0fnu)

    qa_t = torch.from_numpy(qa).to(cuda_device).view(torch.float8_e4m3fn)
    qb_t = torch.from_numpy(qb).to(cuda_device).view(torch.float8_e4m3fn)
    try:
        lib = torch._scaled_mm(qa_t, qb_t.t(), scale_a=library_layout(sa), scale_b=library_layout(sb),
                               out_dtype=torch.bfloat16)
    except (RuntimeError, ValueError) as exc:
        pytest.skip(f"vendor MXFP8 GEMM unavailable here: {exc}")
    lib = to_np(lib)
    assert np.all(np.isfinite(lib))
    same = np.mean(lib.view(np.uint32) == got.view(np.uint32))
    ulp = np.abs(lib - got) / np.maximum(np.abs(lib), 1e-30)
    assert same > 0.97, f"only {same:.4f} of the outputs are bit-equal"
    assert float(ulp.max()) <= 2.0 ** -7, f"largest relative difference {float(ulp.max())}"


@pytest.mark.parametrize("batch,batch_a,batch_b,per_batch_bias", [
    ((3,), (True,), (False,), False),                      # one weight for all batches: runs as one tall GEMM
    ((2, 3), (False, True), (True, False), True),          # A broadcast over the outer, B over the inner dimension
    ((2, 1, 2, 2), (True, True, True, True), (True, False, False, True), False),
])
@pytest.mark.parametrize("d_dtype", ["bfloat16", "float32"])
def test_mx_batched_broadcast(cuda_device, batch, batch_a, batch_b, per_batch_bias, d_dtype):
    """Batched MX GEMM with numpy-style broadcast of either operand over up to four batch dimensions
    (include/blaze/gemm/kernel/kernel_qbmm_mx.h:282-377)."""
    import torch
    M, N, K = 136, 264, 160
    dims_a = [d if k else 1 for d, k in zip(batch, batch_a)]
    dims_b = [d if k else 1 for d, k in zip(batch, batch_b)]
    na, nb, nc = int(np.prod(dims_a)), int(np.prod(dims_b)), int(np.prod(batch))
    a = o.normal_f32(24, 0, (na * M, K), 1.0)
    w = o.normal_f32(24, 1, (nb * N, K), 1.0)
    bias = o.normal_f32(24, 2, (nc if per_batch_bias else 1, N), 0.5)
    residual = o.normal_f32(24, 3, (nc * M, N), 1.0)
    qa, sa = H.quantize(dev_tensor(a, cuda_device), H.SCALE_MX_E8M0_VEC32)
    qb, sb = H.quantize(dev_tensor(w, cuda_device), H.SCALE_MX_E8M0_VEC32)
    # a float32 D has another batch pitch in bytes than the 16-bit ones: every batch must land in its own rows
    out = torch.full((nc * M, N), float("nan"), dtype=getattr(torch, d_dtype), device=cuda_device)
    with H.Contraction(M, N, K, scale_mode_a=H.SCALE_MX_E8M0_VEC32, scale_mode_b=H.SCALE_MX_E8M0_VEC32,
                       activation=H.OP_RELU, bias=True, residual=True, batch=batch, batch_a=batch_a, batch_b=batch_b,
                       bias_per_batch=per_batch_bias, d_dtype=H.R_32F if d_dtype == "float32" else H.R_16BF) as c:
        c(qa, sa, qb, sb, out, bias=bf16_tensor(bias, cuda_device), residual=bf16_tensor(residual, cuda_device))
    got = to_np(out).reshape(*batch, M, N)
    da = o.dequant_mx(to_np(qa), to_np(sa), K).reshape(*dims_a, M, K)
    db = o.dequant_mx(to_np(qb), to_np(sb), K).reshape(*dims_b, N, K)
    acc = np.matmul(da, np.swapaxes(db, -1, -2))                       # float64, numpy broadcasting over the batch
    b16 = o.bf16_round(bias).astype(np.float64).reshape(*(batch if per_batch_bias else [1] * len(batch)), 1, N)
    r16 = o.bf16_round(residual).astype(np.float64).reshape(*batch, M, N)
    ref = np.maximum(acc + b16, 0.0) + r16
    assert_gemm_ok(got.reshape(-1, N), ref.reshape(-1, N))


@pytest.mark.parametrize("tile_n", [224, 256])
def test_mx_pair_many_tiles_per_pair(cuda_device, tile_n):
    """Two CTA pairs walk 24-28 tiles each, so both accumulators (and, for 256-wide tiles, the columns they share)
    are handed back and forth many times; every element is checked."""
    M, N, K = 1000, 1544, 384
    a = o.normal_f32(23, 0, (M, K), 1.0)
    w = o.normal_f32(23, 1, (N, K), 1.0)
    bias = o.normal_f32(23, 2, (N,), 0.5)
    got, qa, sa, qb, sb = run_mx(cuda_device, a, w, act=H.OP_RELU, bias=bias, tile_n=tile_n, cta_pair=2, sm_limit=4)
    ref, gold = mx_reference(qa, sa, qb, sb, K, "e4m3", o.ACT_RELU, bias)
    assert_gemm_ok(got, ref, gold)


@pytest.mark.parametrize("M,N,K,tile_n,sm_limit,b_dtype", [
    (1000, 1544, 384, 256, 6, H.R_8F_E4M3),      # 28 tiles on 3 pairs: the 28th is cut three ways
    (1000, 1544, 384, 224, 10, H.R_8F_E4M3),     # 224-wide tiles (disjoint accumulators), 5 pairs
    (512, 1024, 2048, 256, 0, H.R_8F_E4M3),      # 8 tiles on 74 pairs: every tile is shared by about nine pairs
    (512, 1024, 2048, 256, 0, H.R_4F_E2M1),      # the same with a packed 4-bit weight
    (300, 520, 4096, 0, 0, H.R_8F_E4M3),         # ragged edges
])
def test_mx_pair_last_round_split_along_k(cuda_device, M, N, K, tile_n, sm_limit, b_dtype):
    """2-CTA tiles: the tiles of the last, partly filled round are cut along K so that every CTA pair gets the same
    share; partial tiles go through the float32 workspace (handed over dirty) and the pair that holds K step 0 adds
    them in pair order.  Checked against the float64 reference and for run-to-run bit equality; a second activation
    matrix on the same workspace must not see the first one's partial tiles."""
    import torch
    name = "e2m1" if b_dtype == H.R_4F_E2M1 else "e4m3"
    MX = H.SCALE_MX_E8M0_VEC32
    a = o.normal_f32(37, 0, (M, K), 1.0)
    a2 = o.normal_f32(37, 4, (M, K), 1.0)
    w = o.normal_f32(37, 1, (N, K), 0.05)
    bias = o.normal_f32(37, 2, (N,), 0.5)
    residual = o.normal_f32(37, 3, (M, N), 1.0)
    qa, sa = H.quantize(dev_tensor(a, cuda_device), MX)
    qa2, sa2 = H.quantize(dev_tensor(a2, cuda_device), MX)
    qb, sb = H.quantize(dev_tensor(w, cuda_device), MX, b_dtype)
    out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=cuda_device)
    outs = []
    with H.Contraction(M, N, K, scale_mode_a=MX, scale_mode_b=MX, b_dtype=b_dtype, activation=H.OP_GELU, bias=True,
                       residual=True, tile_n=tile_n, cta_pair=2, sm_limit=sm_limit, split=H.SPLIT_STREAM_K) as c:
        with H.Contraction(M, N, K, scale_mode_a=MX, scale_mode_b=MX, b_dtype=b_dtype, activation=H.OP_GELU, bias=True,
                           residual=True, tile_n=tile_n, cta_pair=2, sm_limit=sm_limit,
                           split=H.SPLIT_DATA_PARALLEL) as whole:
            assert c.workspace_bytes > whole.workspace_bytes + 128 * 224 * 4          # room for partial tiles
        ws = torch.full((c.workspace_bytes,), 0xFF, dtype=torch.uint8, device=cuda_device)
        for qx, sx in ((qa, sa), (qa, sa), (qa2, sa2), (qa, sa)):
            c(qx, sx, qb, sb, out, bias=bf16_tensor(bias, cuda_device), residual=bf16_tensor(residual, cuda_device),
              workspace=ws)
            outs.append(to_np(out).copy())
    first, second, other, again = outs
    assert np.array_equal(first.view(np.uint32), second.view(np.uint32)), "the split is not deterministic"
    assert np.array_equal(first.view(np.uint32), again.view(np.uint32)), "stale partial tiles leaked into a later call"
    ref, gold = mx_reference(to_np(qa), to_np(sa), to_np(qb), to_np(sb), K, name, o.ACT_GELU_TANH, bias, residual)
    assert_gemm_ok(first, ref, gold)
    ref2, gold2 = mx_reference(to_np(qa2), to_np(sa2), to_np(qb), to_np(sb), K, name, o.ACT_GELU_TANH, bias, residual)
    assert_gemm_ok(other, ref2, gold2)


def test_config2_mxfp8_8192_bias_gelu(cuda_device):
    """M=N=K=8192, bf16 bias ~N(0,0.1), GELU(tanh), bf16 out; float64 reference on every 37th row."""
    M = N = K = 8192
    a = o.normal_f32(2, 0, (M, K), 1.0)
    w = o.normal_f32(2, 1, (N, K), 1.0)
    bias = o.normal_f32(2, 2, (N,), 0.1)
    got, qa, sa, qb, sb = run_mx(cuda_device, a, w, act=H.OP_GELU, bias=bias, check_quant=False)
    rows = np.arange(0, M, 37)
    ref, gold = mx_reference(qa, sa, qb, sb, K, "e4m3", o.ACT_GELU_TANH, bias, rows=rows)
    assert_gemm_ok(got[rows], ref, gold)
    # quantisation of the sampled rows is bit-equal to the oracle's
    ra, rsa = o.quant_mx(a[rows])
    assert np.array_equal(qa[rows], ra) and np.array_equal(sa[rows], rsa)


def test_config3_w4a8_4096x14336x4096(cuda_device):
    M, N, K = 4096, 14336, 4096
    a = o.normal_f32(3, 0, (M, K), 1.0)
    w = o.normal_f32(3, 1, (N, K), 0.02)
    got, qa, sa, qb, sb = run_mx(cuda_device, a, w, b_dtype=H.R_4F_E2M1, check_quant=False, static_b=True)
    rows = np.arange(0, M, 29)
    ref, gold = mx_reference(qa, sa, qb, sb, K, "e2m1", rows=rows)
    assert_gemm_ok(got[rows], ref, gold)
    cols = np.arange(0, N, 61)
    rb, rsb = o.quant_mx(w[cols], "e2m1")
    assert np.array_equal(qb[cols], rb) and np.array_equal(sb[cols], rsb)


# ------------------------------------------------------------------------------------------------ plan cache / PATIENT

def test_patient_plan_times_candidates_and_fills_the_cache(cuda_device, tmp_path):
    """An ALGO_DEFAULT_PATIENT plan times its candidate configurations during its first execution, keeps one, stores it
    in the handle's plan cache; results stay within the acceptance bounds whichever candidate wins, and a default plan
    for the same problem on the same handle then runs with the cached choice and gives the same bits."""
    import torch
    M, N, K = 512, 1024, 1024
    mx = H.SCALE_MX_E8M0_VEC32
    a = o.normal_f32(21, 0, (M, K), 1.0)
    w = o.normal_f32(21, 1, (N, K), 1.0)
    bias = o.normal_f32(21, 2, (N,), 0.1)
    qa, sa = H.quantize(dev_tensor(a, cuda_device), mx)
    qb, sb = H.quantize(dev_tensor(w, cuda_device), mx)
    bias_d = bf16_tensor(bias, cuda_device)
    ref, gold = mx_reference(to_np(qa), to_np(sa), to_np(qb), to_np(sb), K, act=o.ACT_GELU_TANH, bias=bias)
    h = H.create_handle()
    try:
        patient = H.Contraction(M, N, K, scale_mode_a=mx, scale_mode_b=mx, activation=H.OP_GELU, bias=True, handle=h,
                                algo=H.ALGO_DEFAULT_PATIENT, b_is_static=True)
        assert patient.kernel_choice()[3] is True
        out1 = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=cuda_device)
        patient(qa, sa, qb, sb, out1, bias=bias_d)
        torch.cuda.synchronize()
        tile_n, cta_pair, split, pending = patient.kernel_choice()
        assert pending is False and (tile_n, cta_pair) in ((0, 0), (256, 2), (224, 2), (128, 1), (224, 1))
        assert_gemm_ok(to_np(out1), ref, gold)
        out2 = torch.full_like(out1, float("nan"))
        patient(qa, sa, qb, sb, out2, bias=bias_d)                      # second call: no timing, weight pre-pass reused
        torch.cuda.synchronize()
        assert torch.equal(out1.view(torch.int16), out2.view(torch.int16))
        H.write_plan_cache(h, tmp_path / "cache.txt")
        lines = (tmp_path / "cache.txt").read_text().splitlines()
        assert len(lines) == 2 and lines[1].endswith(" %d %d %d" % (tile_n, cta_pair, split))
        quick = H.Contraction(M, N, K, scale_mode_a=mx, scale_mode_b=mx, activation=H.OP_GELU, bias=True, handle=h,
                              b_is_static=True)
        assert quick.kernel_choice() == (tile_n, cta_pair, split, False)
        out3 = torch.full_like(out1, float("nan"))
        quick(qa, sa, qb, sb, out3, bias=bias_d)
        torch.cuda.synchronize()
        assert torch.equal(out1.view(torch.int16), out3.view(torch.int16))
        # the FP8 family has scheduler modes to choose from
        af, wf = fp8_problem(22, 128, 1024, 2048)
        qaf, saf = H.quantize(dev_tensor(af, cuda_device), H.SCALE_FP32_1X128)
        qbf, sbf = H.quantize(dev_tensor(wf, cuda_device), H.SCALE_FP32_128X128)
        p8 = H.Contraction(128, 1024, 2048, scale_mode_a=H.SCALE_FP32_1X128, scale_mode_b=H.SCALE_FP32_128X128, handle=h,
                           algo=H.ALGO_DEFAULT_PATIENT)
        out8 = torch.full((128, 1024), float("nan"), dtype=torch.bfloat16, device=cuda_device)
        p8(qaf, saf, qbf, sbf, out8)
        torch.cuda.synchronize()
        assert p8.kernel_choice()[3] is False
        ref8, gold8 = fp8_reference(to_np(qaf), to_np(saf), to_np(qbf), to_np(sbf))
        assert_gemm_ok(to_np(out8), ref8, gold8)
        for c in (patient, quick, p8):
            c.close()
    finally:
        H.api.acltensorDestroy(h)
