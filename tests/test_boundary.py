"""The C-ABI boundary on a machine without a GPU: exported symbols, object life cycle, every argument check.

The call sequences follow the reference's client helper (tests/test_elementwise.cpp:159-208): handle, tensor
descriptors, operation descriptor, plan preference, plan, execute, destroy in reverse order."""
import ctypes as C
import re
import threading
from pathlib import Path

import pytest

from ops_tensor_b200 import host as H
from ops_tensor_b200 import native

ROOT = Path(__file__).resolve().parents[1]


@pytest.fixture(scope="module")
def api(built_library):
    return H.api


def test_library_exports_every_declared_symbol(built_library):
    lib = C.CDLL(str(built_library))
    declared = []
    for header in sorted((ROOT / "include").glob("*.h")):
        text = header.read_text()
        declared += re.findall(r"(?:ACLTENSOR_API|BLAZE_API)\s+[\w\s\*]+?\b(\w+)\s*\(", text)
    assert len(declared) >= 30, declared
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in include/ but not exported"
    for name in ("acltensorCreate", "acltensorDestroy", "acltensorCreateTensorDescriptor",
                 "acltensorDestroyTensorDescriptor", "acltensorCreateElementwiseBinary",
                 "acltensorDestroyOperationDescriptor", "acltensorCreatePlanPreference",
                 "acltensorDestroyPlanPreference", "acltensorCreatePlan", "acltensorDestroyPlan",
                 "acltensorElementwiseBinaryExecute", "acltensorGetErrorString", "acltensorGetVersion"):
        assert name in declared                      # the reference's thirteen entry points


def test_version_and_error_strings(api):
    assert api.acltensorGetVersion() == 1 << 16
    assert H.error_string(0) == "The operation completed successfully."
    assert H.error_string(7) == "Invalid parameter value."
    assert H.error_string(15) == "Operation not supported."
    assert H.error_string(19) == "Insufficient workspace size."
    assert H.error_string(12345) == "Unknown error."


def test_destroy_accepts_null(api):
    for fn in (api.acltensorDestroy, api.acltensorDestroyTensorDescriptor, api.acltensorDestroyOperationDescriptor,
               api.acltensorDestroyPlanPreference, api.acltensorDestroyPlan):
        assert fn(None) == H.STATUS_SUCCESS


def test_handle_and_tensor_descriptor_checks(api):
    assert api.acltensorCreate(None) == H.STATUS_INVALID_VALUE
    h = H.create_handle()
    d = C.c_void_p()
    lens = H.i64([4, 8])
    assert api.acltensorCreateTensorDescriptor(h, None, 2, lens, None, H.R_32F, 0) == H.STATUS_INVALID_VALUE
    assert api.acltensorCreateTensorDescriptor(h, C.byref(d), 2, None, None, H.R_32F, 0) == H.STATUS_INVALID_VALUE
    assert api.acltensorCreateTensorDescriptor(h, C.byref(d), 0, lens, None, H.R_32F, 0) == H.STATUS_INVALID_VALUE
    for unsupported in (H.R_64F, H.R_32U, H.C_32F, H.C_64F):
        assert api.acltensorCreateTensorDescriptor(h, C.byref(d), 2, lens, None, unsupported, 0) == H.STATUS_NOT_SUPPORTED
    for ok in (H.R_32F, H.R_16BF, H.R_16F, H.R_8F_E4M3, H.R_4F_E2M1, H.R_8F_UE8M0, H.R_64I, H.R_8I, H.R_32I, H.R_8F_E5M2):
        assert api.acltensorCreateTensorDescriptor(h, C.byref(d), 2, lens, None, ok, 0) == H.STATUS_SUCCESS
        assert api.acltensorDestroyTensorDescriptor(d) == H.STATUS_SUCCESS
    assert api.acltensorDestroy(h) == H.STATUS_SUCCESS


def _ew_descs(h, n=16):
    return [H.create_tensor_descriptor(h, [n]) for _ in range(3)]


def test_elementwise_descriptor_checks(api):
    h = H.create_handle()
    da, dc, dd = _ew_descs(h)
    m = H.i32([0])
    op = C.c_void_p()
    f = api.acltensorCreateElementwiseBinary
    ok_args = (da, m, H.OP_IDENTITY, dc, m, H.OP_IDENTITY, dd, m, H.OP_ADD, H.COMPUTE_DESC_32F)
    assert f(h, None, *ok_args) == H.STATUS_INVALID_VALUE
    assert f(h, C.byref(op), None, *ok_args[1:]) == H.STATUS_INVALID_VALUE
    assert f(h, C.byref(op), da, None, *ok_args[2:]) == H.STATUS_INVALID_VALUE
    assert f(h, C.byref(op), da, m, H.OP_SQRT, dc, m, H.OP_IDENTITY, dd, m, H.OP_ADD, H.COMPUTE_DESC_32F) == H.STATUS_NOT_SUPPORTED
    assert f(h, C.byref(op), da, m, H.OP_IDENTITY, dc, m, H.OP_IDENTITY, dd, m, H.OP_MUL, H.COMPUTE_DESC_32F) == H.STATUS_NOT_SUPPORTED
    assert f(h, C.byref(op), *ok_args[:-1], H.COMPUTE_DESC_NONE) == H.STATUS_INVALID_VALUE
    assert f(h, C.byref(op), *ok_args[:-1], H.COMPUTE_DESC_16F) == H.STATUS_NOT_SUPPORTED
    assert f(h, C.byref(op), *ok_args) == H.STATUS_SUCCESS

    pref, plan = C.c_void_p(), C.c_void_p()
    assert api.acltensorCreatePlanPreference(h, None, H.ALGO_DEFAULT) == H.STATUS_INVALID_VALUE
    # the reference accepts ALGO_DEFAULT only (lib/core/plan_preference.cpp:34-36); here the PATIENT value of its enum is
    # accepted too (contraction plans time their candidates), anything else is refused as there
    assert api.acltensorCreatePlanPreference(h, C.byref(pref), -2) == H.STATUS_NOT_SUPPORTED
    assert api.acltensorCreatePlanPreference(h, C.byref(pref), H.ALGO_DEFAULT_PATIENT) == H.STATUS_SUCCESS
    assert api.acltensorDestroyPlanPreference(pref) == H.STATUS_SUCCESS
    assert api.acltensorCreatePlanPreference(h, C.byref(pref), H.ALGO_DEFAULT) == H.STATUS_SUCCESS
    assert api.acltensorCreatePlan(h, None, op, pref, 0) == H.STATUS_INVALID_VALUE
    assert api.acltensorCreatePlan(h, C.byref(plan), None, pref, 0) == H.STATUS_INVALID_VALUE
    assert api.acltensorCreatePlan(h, C.byref(plan), op, None, 0) == H.STATUS_INVALID_VALUE
    assert api.acltensorCreatePlan(h, C.byref(plan), op, pref, 0) == H.STATUS_SUCCESS
    need = C.c_uint64(99)
    assert api.acltensorPlanGetRequiredWorkspace(plan, C.byref(need)) == H.STATUS_SUCCESS and need.value == 0

    ex = api.acltensorElementwiseBinaryExecute
    fake = 4096
    assert ex(h, None, None, fake, None, fake, fake, None) == H.STATUS_INVALID_VALUE
    assert ex(h, plan, None, None, None, fake, fake, None) == H.STATUS_INVALID_VALUE
    assert ex(h, plan, None, fake, None, None, fake, None) == H.STATUS_INVALID_VALUE
    assert ex(h, plan, None, fake, None, fake, None, None) == H.STATUS_INVALID_VALUE
    import torch
    if not torch.cuda.is_available():
        # no fallback: without a device the call reports that instead of computing on the host
        assert ex(h, plan, None, fake, None, fake, fake, None) == H.STATUS_NOT_INITIALIZED

    for fn, obj in ((api.acltensorDestroyPlan, plan), (api.acltensorDestroyPlanPreference, pref),
                    (api.acltensorDestroyOperationDescriptor, op)):
        assert fn(obj) == H.STATUS_SUCCESS
    for t in (da, dc, dd):
        api.acltensorDestroyTensorDescriptor(t)
    api.acltensorDestroy(h)


def _contraction_descs(h, M=256, N=512, K=1024, b_dtype=H.R_8F_E4M3, groups=0):
    dA = H.create_tensor_descriptor(h, [M, K], None, H.R_8F_E4M3)
    dB = H.create_tensor_descriptor(h, [groups, N, K] if groups else [N, K], None, b_dtype)
    dD = H.create_tensor_descriptor(h, [M, N], None, H.R_16BF)
    return dA, dB, dD


def test_contraction_descriptor_checks(api):
    h = H.create_handle()
    dA, dB, dD = _contraction_descs(h)
    op = C.c_void_p()
    f = api.acltensorCreateContraction
    mA, mB, mD = H.i32([0, 2]), H.i32([1, 2]), H.i32([0, 1])
    good = (dA, mA, H.OP_IDENTITY, dB, mB, H.OP_IDENTITY, None, None, H.OP_IDENTITY, dD, mD, H.COMPUTE_DESC_32F)
    assert f(h, None, *good) == H.STATUS_INVALID_VALUE
    assert f(h, C.byref(op), None, *good[1:]) == H.STATUS_INVALID_VALUE
    assert f(h, C.byref(op), dA, None, *good[2:]) == H.STATUS_INVALID_VALUE
    assert f(h, C.byref(op), dA, mA, H.OP_RELU, *good[3:]) == H.STATUS_NOT_SUPPORTED
    assert f(h, C.byref(op), *good[:-1], H.COMPUTE_DESC_NONE) == H.STATUS_INVALID_VALUE
    assert f(h, C.byref(op), *good[:-1], H.COMPUTE_DESC_16BF) == H.STATUS_NOT_SUPPORTED
    # K extents disagree
    dBbad = H.create_tensor_descriptor(h, [512, 512], None, H.R_8F_E4M3)
    assert f(h, C.byref(op), dA, mA, H.OP_IDENTITY, dBbad, mB, H.OP_IDENTITY, None, None, H.OP_IDENTITY, dD, mD,
             H.COMPUTE_DESC_32F) == H.STATUS_INVALID_VALUE
    # output may be bf16, half or float32 (the reference's cast-on-store modes), nothing else
    dD32 = H.create_tensor_descriptor(h, [256, 512], None, H.R_32F)
    assert f(h, C.byref(op), dA, mA, H.OP_IDENTITY, dB, mB, H.OP_IDENTITY, None, None, H.OP_IDENTITY, dD32, mD,
             H.COMPUTE_DESC_32F) == H.STATUS_SUCCESS
    api.acltensorDestroyOperationDescriptor(op)
    dD8 = H.create_tensor_descriptor(h, [256, 512], None, H.R_64I)
    assert f(h, C.byref(op), dA, mA, H.OP_IDENTITY, dB, mB, H.OP_IDENTITY, None, None, H.OP_IDENTITY, dD8, mD,
             H.COMPUTE_DESC_32F) == H.STATUS_NOT_SUPPORTED
    # K must be the contiguous mode of A
    dAt = H.create_tensor_descriptor(h, [256, 1024], [1, 256], H.R_8F_E4M3)
    assert f(h, C.byref(op), dAt, mA, H.OP_IDENTITY, dB, mB, H.OP_IDENTITY, None, None, H.OP_IDENTITY, dD, mD,
             H.COMPUTE_DESC_32F) == H.STATUS_NOT_SUPPORTED
    # B described as [K, N] with K contiguous ("column-major") is the same operand
    dBkn = H.create_tensor_descriptor(h, [1024, 512], [1, 1024], H.R_8F_E4M3)
    assert f(h, C.byref(op), dA, mA, H.OP_IDENTITY, dBkn, H.i32([2, 1]), H.OP_IDENTITY, None, None, H.OP_IDENTITY, dD,
             mD, H.COMPUTE_DESC_32F) == H.STATUS_SUCCESS
    api.acltensorDestroyOperationDescriptor(op)
    assert f(h, C.byref(op), *good) == H.STATUS_SUCCESS

    # attributes
    v = C.c_int32(H.SCALE_MX_E8M0_VEC32)
    sa = api.acltensorOperationDescriptorSetAttribute
    assert sa(h, None, H.ATTR_SCALE_MODE_A, C.byref(v), 4) == H.STATUS_INVALID_VALUE
    assert sa(h, op, H.ATTR_SCALE_MODE_A, None, 4) == H.STATUS_INVALID_VALUE
    assert sa(h, op, H.ATTR_SCALE_MODE_A, C.byref(v), 8) == H.STATUS_INVALID_VALUE
    assert sa(h, op, 77, C.byref(v), 4) == H.STATUS_INVALID_VALUE
    assert sa(h, op, H.ATTR_SCALE_MODE_A, C.byref(C.c_int32(9)), 4) == H.STATUS_INVALID_VALUE
    assert sa(h, op, H.ATTR_EPILOGUE_ACT, C.byref(C.c_int32(H.OP_SQRT)), 4) == H.STATUS_NOT_SUPPORTED
    assert sa(h, op, H.ATTR_TILE_N, C.byref(C.c_int32(96)), 4) == H.STATUS_NOT_SUPPORTED
    assert sa(h, op, H.ATTR_GROUP_COUNT, C.byref(C.c_int32(4)), 4) == H.STATUS_INVALID_VALUE
    H.set_attribute(h, op, H.ATTR_EPILOGUE_ACT, H.OP_GELU)
    assert H.get_attribute(h, op, H.ATTR_EPILOGUE_ACT) == H.OP_GELU
    assert H.get_attribute(h, op, H.ATTR_BIAS_TYPE) == -1

    # no scale modes yet: no registered solution matches
    pref, plan = C.c_void_p(), C.c_void_p()
    H.check(api.acltensorCreatePlanPreference(h, C.byref(pref), H.ALGO_DEFAULT), "pref")
    assert api.acltensorCreatePlan(h, C.byref(plan), op, pref, 1 << 40) == H.STATUS_NOT_SUPPORTED
    est = C.c_uint64(0)
    assert api.acltensorEstimateWorkspaceSize(h, op, pref, H.WORKSPACE_DEFAULT, C.byref(est)) == H.STATUS_NOT_SUPPORTED
    # MX x FP32 is not a registered pairing either
    H.set_attribute(h, op, H.ATTR_SCALE_MODE_A, H.SCALE_MX_E8M0_VEC32)
    H.set_attribute(h, op, H.ATTR_SCALE_MODE_B, H.SCALE_FP32_128X128)
    assert api.acltensorCreatePlan(h, C.byref(plan), op, pref, 1 << 40) == H.STATUS_NOT_SUPPORTED
    H.set_attribute(h, op, H.ATTR_SCALE_MODE_B, H.SCALE_MX_E8M0_VEC32)
    assert api.acltensorEstimateWorkspaceSize(h, op, pref, 0, C.byref(est)) == H.STATUS_INVALID_VALUE
    assert api.acltensorEstimateWorkspaceSize(h, op, pref, H.WORKSPACE_DEFAULT, C.byref(est)) == H.STATUS_SUCCESS
    # re-tiled scale factors of A (2 tiles x 8 k-steps x 512 B) and B live in the workspace
    assert est.value >= 2 * 8 * 512 * 2
    assert api.acltensorCreatePlan(h, C.byref(plan), op, pref, est.value - 1) == H.STATUS_INSUFFICIENT_WORKSPACE
    assert api.acltensorCreatePlan(h, C.byref(plan), op, pref, est.value) == H.STATUS_SUCCESS

    aux = H.ContractionAux(4096, 4096, None, None)
    one, two, zero = C.c_float(1.0), C.c_float(2.0), C.c_float(0.0)
    ct = api.acltensorContract
    fake = 4096
    assert ct(h, None, None, fake, fake, None, None, fake, C.byref(aux), fake, est.value, None) == H.STATUS_INVALID_VALUE
    assert ct(h, plan, None, None, fake, None, None, fake, C.byref(aux), fake, est.value, None) == H.STATUS_INVALID_VALUE
    assert ct(h, plan, None, fake, fake, None, None, fake, None, fake, est.value, None) == H.STATUS_INVALID_VALUE
    assert ct(h, plan, C.byref(two), fake, fake, None, None, fake, C.byref(aux), fake, est.value, None) == H.STATUS_NOT_SUPPORTED
    assert ct(h, plan, C.byref(one), fake, fake, C.byref(two), None, fake, C.byref(aux), fake, est.value, None) == H.STATUS_NOT_SUPPORTED
    # beta = 1 asks for a residual the descriptor does not have
    assert ct(h, plan, None, fake, fake, C.byref(one), fake, fake, C.byref(aux), fake, est.value, None) == H.STATUS_INVALID_VALUE
    assert ct(h, plan, None, fake, fake, C.byref(zero), None, fake, C.byref(aux), fake, est.value - 1, None) == H.STATUS_INSUFFICIENT_WORKSPACE
    no_scales = H.ContractionAux(None, 4096, None, None)
    assert ct(h, plan, None, fake, fake, None, None, fake, C.byref(no_scales), fake, est.value, None) == H.STATUS_INVALID_VALUE
    # GELU epilogue was requested without bias: fine; with BIAS_TYPE set the pointer becomes mandatory
    api.acltensorDestroyPlan(plan)
    H.set_attribute(h, op, H.ATTR_BIAS_TYPE, H.R_16BF)
    assert api.acltensorCreatePlan(h, C.byref(plan), op, pref, est.value) == H.STATUS_SUCCESS
    assert ct(h, plan, None, fake, fake, None, None, fake, C.byref(aux), fake, est.value, None) == H.STATUS_INVALID_VALUE
    # the elementwise entry point refuses a contraction plan
    assert api.acltensorElementwiseBinaryExecute(h, plan, None, fake, None, fake, fake, None) == H.STATUS_NOT_SUPPORTED

    api.acltensorDestroyPlan(plan)
    api.acltensorDestroyPlanPreference(pref)
    api.acltensorDestroyOperationDescriptor(op)
    for t in (dA, dB, dD, dBbad, dD32, dAt, dBkn):
        api.acltensorDestroyTensorDescriptor(t)
    api.acltensorDestroy(h)


def test_streamk_plan_falls_back_without_workspace(api):
    """A plan asked to use stream-K with no workspace allowance degrades to whole tiles per CTA."""
    with H.Contraction(64, 7168, 18432, scale_mode_a=H.SCALE_FP32_1X128, scale_mode_b=H.SCALE_FP32_128X128,
                       split=H.SPLIT_STREAM_K) as c:
        assert c.workspace_bytes > 148 * 128 * 128 * 4 // 2
    with H.Contraction(64, 7168, 18432, scale_mode_a=H.SCALE_FP32_1X128, scale_mode_b=H.SCALE_FP32_128X128,
                       split=H.SPLIT_STREAM_K, workspace_limit=0) as c:
        assert c.workspace_bytes == 0


def test_grouped_and_w4_descriptors(api):
    with H.Contraction(4096, 768, 2048, scale_mode_a=H.SCALE_FP32_1X128, scale_mode_b=H.SCALE_FP32_128X128,
                       groups=16) as c:
        # room for the split along K, which the kernel may choose once it has counted the tiles of the group list
        assert c.workspace_bytes >= 148 * 128 * 128 * 4
        assert H.get_attribute(c.handle, c.op, H.ATTR_GROUP_COUNT) == 16
    with H.Contraction(4096, 768, 2048, scale_mode_a=H.SCALE_FP32_1X128, scale_mode_b=H.SCALE_FP32_128X128,
                       groups=16, split=H.SPLIT_DATA_PARALLEL) as c:
        assert c.workspace_bytes == 0                       # whole tiles per CTA need none
    with H.Contraction(4096, 768, 2048, scale_mode_a=H.SCALE_FP32_1X128, scale_mode_b=H.SCALE_FP32_128X128,
                       groups=16, workspace_limit=0) as c:
        assert c.workspace_bytes == 0                       # and a caller without workspace falls back to them
    with pytest.raises(native.BlazeError) as e:           # grouped MX is not registered
        H.Contraction(4096, 768, 2048, scale_mode_a=H.SCALE_MX_E8M0_VEC32, scale_mode_b=H.SCALE_MX_E8M0_VEC32, groups=4)
    assert e.value.status == H.STATUS_NOT_SUPPORTED
    with H.Contraction(256, 512, 1024, scale_mode_a=H.SCALE_MX_E8M0_VEC32, scale_mode_b=H.SCALE_MX_E8M0_VEC32,
                       b_dtype=H.R_4F_E2M1) as c:
        assert c.workspace_bytes >= 512 * 1024             # room for the expanded weight
    with pytest.raises(native.BlazeError) as e:           # K not a multiple of 16 cannot be staged by TMA
        H.Contraction(256, 512, 1000, scale_mode_a=H.SCALE_MX_E8M0_VEC32, scale_mode_b=H.SCALE_MX_E8M0_VEC32)
    assert e.value.status == H.STATUS_NOT_SUPPORTED


def test_objects_are_independent_across_threads(api):
    errors = []

    def worker():
        try:
            for _ in range(200):
                with H.Contraction(256, 512, 1024, scale_mode_a=H.SCALE_MX_E8M0_VEC32,
                                   scale_mode_b=H.SCALE_MX_E8M0_VEC32, activation=H.OP_GELU, bias=True):
                    pass
        except Exception as exc:                           # pragma: no cover
            errors.append(exc)

    threads = [threading.Thread(target=worker) for _ in range(8)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors


def test_kernel_abi_argument_checks(built_library):
    """The launch layer rejects malformed arguments before touching a device."""
    l = native.lib()
    n = C.c_size_t(0)
    a = native.MxGemmArgs()
    assert l.blazeMxGemmWorkspaceSize(C.byref(a), C.byref(n)) == H.STATUS_INVALID_VALUE        # struct_size unset
    a.struct_size = C.sizeof(a)
    a.M, a.N, a.K = 128, 128, 100
    assert l.blazeMxGemmWorkspaceSize(C.byref(a), C.byref(n)) == H.STATUS_NOT_SUPPORTED        # K % 16
    a.K = 128
    a.tile_n = 64
    assert l.blazeMxGemmWorkspaceSize(C.byref(a), C.byref(n)) == H.STATUS_NOT_SUPPORTED
    a.tile_n = 0
    assert l.blazeMxGemmWorkspaceSize(C.byref(a), None) == H.STATUS_INVALID_VALUE
    assert l.blazeMxGemmWorkspaceSize(C.byref(a), C.byref(n)) == H.STATUS_SUCCESS and n.value == 1024
    f = native.Fp8GemmArgs()
    f.struct_size = C.sizeof(f)
    f.M, f.N, f.K, f.groups = 128, 128, 128, 2000
    assert l.blazeFp8GemmWorkspaceSize(C.byref(f), C.byref(n)) == H.STATUS_NOT_SUPPORTED       # too many groups
    f.M, f.K = 1024, 1024
    f.groups, f.sched = 4, native.SCHED_STREAM_K                                               # grouped, split along K
    assert l.blazeFp8GemmWorkspaceSize(C.byref(f), C.byref(n)) == H.STATUS_SUCCESS and n.value >= 128 * 128 * 4
    f.M, f.K = 128, 128
    f.groups, f.sched = 0, native.SCHED_DATA_PARALLEL
    assert l.blazeFp8GemmWorkspaceSize(C.byref(f), C.byref(n)) == H.STATUS_SUCCESS and n.value == 0
    assert l.blazeQuantizeMx(None, 0, 4, 32, 0, None, 0, None, None) == H.STATUS_INVALID_VALUE
    assert l.blazeAddF32(None, None, None, 0, None) == H.STATUS_SUCCESS
    assert l.blazeAddF32(None, None, None, -1, None) == H.STATUS_INVALID_VALUE
    # the closing signal of a fused gather refuses incomplete arguments before it touches a device
    l.blazePeerSignal.restype = C.c_int
    assert l.blazePeerSignal(None, None) == H.STATUS_INVALID_VALUE
    ps = native.PeerSignalArgs()
    ps.struct_size = C.sizeof(ps)
    ps.n_peers = 0
    assert l.blazePeerSignal(C.byref(ps), None) == H.STATUS_INVALID_VALUE          # no peers
    ps.n_peers, ps.my_rank = native.MAX_PEERS + 1, 0
    assert l.blazePeerSignal(C.byref(ps), None) == H.STATUS_INVALID_VALUE          # too many
    ps.n_peers = 1
    assert l.blazePeerSignal(C.byref(ps), None) == H.STATUS_INVALID_VALUE          # no flag arrays


def test_benchmark_generators_match_the_oracle():
    """bench.py draws its inputs from ops_tensor_b200.synthetic; the parity tests draw theirs from the oracle.  Both
    must produce the same tensors for the same (config, tensor id)."""
    import numpy as np
    import blaze_oracle as o
    from ops_tensor_b200 import synthetic as s
    assert np.array_equal(s.normal_f32(2, 0, (5, 64), 1.0), o.normal_f32(2, 0, (5, 64), 1.0))
    assert np.array_equal(s.normal_f32(5, 1, (3, 128), 0.02), o.normal_f32(5, 1, (3, 128), 0.02))
    assert np.array_equal(s.moe_group_rows(), o.moe_group_rows())


def test_batched_contraction_descriptor_rules(built_library):
    """Batch modes of D with broadcast operands (the loop nest of kernel_qbmm_mx.h:282-338): accepted when every tensor
    is packed batch after batch; a batch mode D does not have, a wrong extent or a gap between batches is refused."""
    MX = H.SCALE_MX_E8M0_VEC32
    # A per batch, B broadcast; A broadcast over the outer batch dim, B batched over the inner one
    for kw in (dict(batch=(3,)), dict(batch=(2, 3), batch_a=(False, True), batch_b=(False, True)),
               dict(batch=(2, 1, 2, 2), batch_a=(True, True, True, True), batch_b=(True, False, False, True))):
        with H.Contraction(64, 72, 128, scale_mode_a=MX, scale_mode_b=MX, **kw) as c:
            assert c.workspace_bytes > 0
    h = H.create_handle()
    dA = H.create_tensor_descriptor(h, [3, 64, 128], [64 * 128, 128, 1], H.R_8F_E4M3)
    dB = H.create_tensor_descriptor(h, [72, 128], [128, 1], H.R_8F_E4M3)
    dD = H.create_tensor_descriptor(h, [3, 64, 72], [64 * 72, 72, 1], H.R_16BF)
    dD_gap = H.create_tensor_descriptor(h, [3, 64, 72], [64 * 72 + 8, 72, 1], H.R_16BF)
    dA_bad = H.create_tensor_descriptor(h, [4, 64, 128], [64 * 128, 128, 1], H.R_8F_E4M3)
    op = C.c_void_p()
    args = lambda a, ma, d, md: (h, C.byref(op), a, H.i32(ma), H.OP_IDENTITY, dB, H.i32([1, 2]), H.OP_IDENTITY, None,
                                 None, H.OP_IDENTITY, d, H.i32(md), H.COMPUTE_DESC_32F)
    assert H.api.acltensorCreateContraction(*args(dA, [10, 0, 2], dD, [10, 0, 1])) == H.STATUS_SUCCESS
    H.api.acltensorDestroyOperationDescriptor(op)
    assert H.api.acltensorCreateContraction(*args(dA, [11, 0, 2], dD, [10, 0, 1])) == H.STATUS_INVALID_VALUE
    assert H.api.acltensorCreateContraction(*args(dA_bad, [10, 0, 2], dD, [10, 0, 1])) == H.STATUS_INVALID_VALUE
    assert H.api.acltensorCreateContraction(*args(dA, [10, 0, 2], dD_gap, [10, 0, 1])) == H.STATUS_NOT_SUPPORTED
    for d in (dA, dB, dD, dD_gap, dA_bad):
        H.api.acltensorDestroyTensorDescriptor(d)
    H.api.acltensorDestroy(h)
    # the C ABI refuses batch extents that are neither the output's nor 1
    bd = native.BatchDims()
    for i in range(4):
        bd.c[i], bd.a[i], bd.b[i] = 1, 1, 1
    bd.c[3], bd.a[3], bd.b[3] = 4, 2, 1
    a = native.MxGemmArgs()
    a.struct_size = C.sizeof(a)
    a.M = a.N = a.K = 128
    n = C.c_size_t(0)
    assert native.lib().blazeMxGemmBatchedWorkspaceSize(C.byref(a), C.byref(bd), C.byref(n)) == H.STATUS_INVALID_VALUE
    bd.a[3] = 4
    assert native.lib().blazeMxGemmBatchedWorkspaceSize(C.byref(a), C.byref(bd), C.byref(n)) == H.STATUS_SUCCESS
    assert n.value > 0


def test_c99_client_compiles_and_runs(built_library, tmp_path):
    """The public headers are plain C and the library links from C: tests/c_client/client.c walks the reference's call
    sequence (handle, descriptors, operation, preference, plan) and the contraction planning flow on the host."""
    import shutil
    import subprocess
    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("no C compiler")
    root = Path(__file__).resolve().parent.parent
    exe = tmp_path / "blaze_c_client"
    libdir = Path(built_library).parent
    cmd = [gcc, "-std=c99", "-Wall", "-Wextra", "-pedantic", "-Werror", f"-I{root / 'include'}",
           str(root / "tests" / "c_client" / "client.c"), f"-L{libdir}", "-lops_tensor_b200", f"-Wl,-rpath,{libdir}",
           "-o", str(exe)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    r = subprocess.run([str(exe)], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "c client ok" in r.stdout


def test_plan_choices_show_in_the_workspace_size(built_library):
    """The planner's decisions for the benchmark shapes, read off the workspace sizes (148 SMs assumed without a device):
    256-wide 2-CTA tiles with four-fold B scale blocks for C2; stream-K for the decode shapes of both kernel families and
    whole tiles for the small and the grouped ones."""
    lib = native.lib()

    def mx_bytes(M, N, K, **kw):
        a = native.MxGemmArgs()
        a.struct_size = C.sizeof(a)
        a.M, a.N, a.K = M, N, K
        for k, v in kw.items():
            setattr(a, k, v)
        n = C.c_size_t(0)
        assert lib.blazeMxGemmWorkspaceSize(C.byref(a), C.byref(n)) == H.STATUS_SUCCESS
        return n.value

    def fp8_bytes(M, N, K, **kw):
        a = native.Fp8GemmArgs()
        a.struct_size = C.sizeof(a)
        a.M, a.N, a.K = M, N, K
        for k, v in kw.items():
            setattr(a, k, v)
        n = C.c_size_t(0)
        assert lib.blazeFp8GemmWorkspaceSize(C.byref(a), C.byref(n)) == H.STATUS_SUCCESS
        return n.value

    sfa = 8192 // 128 * 64 * 512                          # re-tiled scales of A: 64 row tiles x 64 K steps
    sfb_256 = 8192 // 256 * 64 * 2 * 4 * 512              # 32 column tiles x 64 K steps x 2 atoms x 4 copies
    assert mx_bytes(8192, 8192, 8192) == sfa + sfb_256
    assert mx_bytes(8192, 8192, 8192, tile_n=224, cta_pair=2) == sfa + 37 * 64 * 2 * 4 * 512
    # skinny MX problem: stream-K adds flags and 148 partial tiles of 128 x 128 floats; whole tiles when forbidden
    whole = mx_bytes(128, 7168, 18432, sched=native.SCHED_DATA_PARALLEL)
    split = mx_bytes(128, 7168, 18432)
    assert split - whole == 148 * 128 * 128 * 4 + 768
    assert mx_bytes(256, 512, 1024) == mx_bytes(256, 512, 1024, sched=native.SCHED_DATA_PARALLEL)
    # FP8 family: C5 splits along K (148 partial tiles + 148 eight-byte marks, rounded to 256), C1 does not; a grouped
    # problem reserves the room and lets the kernel decide once it has counted the tiles
    assert fp8_bytes(128, 7168, 18432) == 148 * 128 * 128 * 4 + 1280
    assert fp8_bytes(256, 512, 1024) == 0
    assert fp8_bytes(32768, 768, 2048, groups=128) == 148 * 128 * 128 * 4 + 1280
    assert fp8_bytes(32768, 768, 2048, groups=128, sched=native.SCHED_DATA_PARALLEL) == 0
    assert fp8_bytes(256, 512, 1024, sched=native.SCHED_STREAM_K) > 0


def test_peer_outputs_are_validated_at_plan_time(built_library):
    """`n_peers` / `peerD` (the epilogue's extra copies of D): 1 KB more workspace for the tensor maps, only with the 2-CTA
    tiles and a 16-bit D, never through the batched or the allocation-free entry."""
    lib = native.lib()

    def size(M, N, K, **kw):
        a = native.MxGemmArgs()
        a.struct_size = C.sizeof(a)
        a.M, a.N, a.K = M, N, K
        for k, v in kw.items():
            setattr(a, k, v)
        n = C.c_size_t(0)
        return lib.blazeMxGemmWorkspaceSize(C.byref(a), C.byref(n)), n.value

    ok, plain = size(8192, 8192, 8192)
    assert ok == H.STATUS_SUCCESS
    assert size(8192, 8192, 8192, n_peers=1) == (H.STATUS_SUCCESS, plain + 1024)
    assert size(8192, 8192, 8192, n_peers=7) == (H.STATUS_SUCCESS, plain + 1024)
    assert size(8192, 8192, 8192, n_peers=8)[0] == H.STATUS_INVALID_VALUE
    assert size(8192, 8192, 8192, n_peers=-1)[0] == H.STATUS_INVALID_VALUE
    assert size(128, 7168, 18432, n_peers=1)[0] == H.STATUS_NOT_SUPPORTED               # single-CTA tiles
    assert size(8192, 8192, 8192, n_peers=1, d_type=native.OUT_F32)[0] == H.STATUS_NOT_SUPPORTED
    # batched entry
    a = native.MxGemmArgs()
    a.struct_size = C.sizeof(a)
    a.M, a.N, a.K, a.n_peers = 256, 256, 256, 1
    bd = native.BatchDims()
    for i in range(4):
        bd.c[i] = bd.a[i] = bd.b[i] = 1
    n = C.c_size_t(0)
    assert lib.blazeMxGemmBatched(C.byref(a), C.byref(bd), None) == H.STATUS_NOT_SUPPORTED
    # the FP8 GEMM takes the same fields and needs no workspace for them
    f = native.Fp8GemmArgs()
    f.struct_size = C.sizeof(f)
    f.M, f.N, f.K = 256, 512, 1024
    for peers, d_type, want in ((0, native.OUT_BF16, H.STATUS_SUCCESS), (7, native.OUT_F16, H.STATUS_SUCCESS),
                                (8, native.OUT_BF16, H.STATUS_INVALID_VALUE), (1, native.OUT_F32, H.STATUS_NOT_SUPPORTED),
                                (1, native.OUT_FP8_128, H.STATUS_NOT_SUPPORTED)):
        f.n_peers, f.d_type = peers, d_type
        assert lib.blazeFp8GemmWorkspaceSize(C.byref(f), C.byref(n)) == want
        assert want != H.STATUS_SUCCESS or n.value == 0



def test_plan_cache_file_round_trip_and_lookup(built_library, tmp_path):
    """The handle's plan cache (names reserved by the reference, lib/core/handle.cpp:105-108): entries read from a file
    decide the kernel choice of plans that leave it open, survive a write / read round trip, are evicted oldest first,
    and a damaged file changes nothing."""
    mx = H.SCALE_MX_E8M0_VEC32
    h = H.create_handle()
    try:
        base = H.Contraction(8192, 8192, 8192, scale_mode_a=mx, scale_mode_b=mx, handle=h)
        assert base.kernel_choice() == (0, 0, H.SPLIT_AUTO, False)
        default_bytes = base.workspace_bytes
        base.close()
        # learn the signature the library uses for this problem from a PATIENT plan's cache key: write an empty cache,
        # then a hand-made one with the same key format
        H.write_plan_cache(h, tmp_path / "empty.txt")
        assert (tmp_path / "empty.txt").read_text() == "acltensor-plan-cache 1\n"
        key = "c:8192:8192:8192:a%d:b%d:d%d:c0:sa%d:sb%d:sd0:act%d:bias-1:g0:bm0:nm0:st0:sm0" % (
            H.R_8F_E4M3, H.R_8F_E4M3, H.R_16BF, mx, mx, H.OP_IDENTITY)
        (tmp_path / "one.txt").write_text("acltensor-plan-cache 1\n%s 224 2 %d\n" % (key, H.SPLIT_DATA_PARALLEL))
        assert H.read_plan_cache(h, tmp_path / "one.txt") == 1
        tuned = H.Contraction(8192, 8192, 8192, scale_mode_a=mx, scale_mode_b=mx, handle=h)
        assert tuned.kernel_choice() == (224, 2, H.SPLIT_DATA_PARALLEL, False)
        forced = H.Contraction(8192, 8192, 8192, scale_mode_a=mx, scale_mode_b=mx, handle=h, tile_n=224, cta_pair=2)
        assert tuned.workspace_bytes == forced.workspace_bytes != default_bytes
        # a descriptor that fixes its own choice ignores the cache; another problem misses it
        assert forced.kernel_choice()[:2] == (224, 2)
        other = H.Contraction(4096, 8192, 8192, scale_mode_a=mx, scale_mode_b=mx, handle=h)
        assert other.kernel_choice() == (0, 0, H.SPLIT_AUTO, False)
        for c in (tuned, forced, other):
            c.close()
        # round trip into a second handle
        H.write_plan_cache(h, tmp_path / "copy.txt")
        h2 = H.create_handle()
        assert H.read_plan_cache(h2, tmp_path / "copy.txt") == 1
        again = H.Contraction(8192, 8192, 8192, scale_mode_a=mx, scale_mode_b=mx, handle=h2)
        assert again.kernel_choice() == (224, 2, H.SPLIT_DATA_PARALLEL, False)
        again.close()
        # capacity: the oldest entry goes first
        (tmp_path / "two.txt").write_text("acltensor-plan-cache 1\nk1 128 1 0\nk2 256 2 0\n")
        H.resize_plan_cache(h2, 2)
        assert H.read_plan_cache(h2, tmp_path / "two.txt") == 2
        H.write_plan_cache(h2, tmp_path / "after.txt")
        assert (tmp_path / "after.txt").read_text().splitlines()[1:] == ["k1 128 1 0", "k2 256 2 0"]
        # damaged or missing files
        (tmp_path / "bad1.txt").write_text("something else\n")
        (tmp_path / "bad2.txt").write_text("acltensor-plan-cache 1\nk3 100 1 0\n")
        (tmp_path / "bad3.txt").write_text("acltensor-plan-cache 1\nk3 128 1\n")
        for name in ("bad1.txt", "bad2.txt", "bad3.txt"):
            with pytest.raises(native.BlazeError) as e:
                H.read_plan_cache(h2, tmp_path / name)
            assert e.value.status == H.STATUS_INVALID_VALUE
        with pytest.raises(native.BlazeError) as e:
            H.read_plan_cache(h2, tmp_path / "missing.txt")
        assert e.value.status == H.STATUS_IO_ERROR
        H.write_plan_cache(h2, tmp_path / "still.txt")
        assert (tmp_path / "still.txt").read_text().splitlines()[1:] == ["k1 128 1 0", "k2 256 2 0"]
        H.api.acltensorDestroy(h2)
    finally:
        H.api.acltensorDestroy(h)


def test_patient_preference_marks_the_plan_for_tuning(built_library):
    """ALGO_DEFAULT_PATIENT (include/cann_ops_tensor_types.h:113): accepted; a contraction plan with an open choice and
    no cached entry waits to time its candidates at the first execution and asks for the workspace of the hungriest one."""
    mx = H.SCALE_MX_E8M0_VEC32
    h = H.create_handle()
    try:
        quick = H.Contraction(256, 7168, 4096, scale_mode_a=mx, scale_mode_b=mx, handle=h)
        patient = H.Contraction(256, 7168, 4096, scale_mode_a=mx, scale_mode_b=mx, handle=h, algo=H.ALGO_DEFAULT_PATIENT)
        assert quick.kernel_choice()[3] is False and patient.kernel_choice()[3] is True
        assert patient.workspace_bytes >= quick.workspace_bytes
        fixed = H.Contraction(256, 7168, 4096, scale_mode_a=mx, scale_mode_b=mx, handle=h, algo=H.ALGO_DEFAULT_PATIENT,
                              tile_n=128, cta_pair=1)
        assert fixed.kernel_choice() == (128, 1, H.SPLIT_AUTO, False)          # nothing left open, nothing to tune
        for c in (quick, patient, fixed):
            c.close()
    finally:
        H.api.acltensorDestroy(h)
