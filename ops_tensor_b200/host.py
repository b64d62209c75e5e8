"""Python face of the acltensor* host API (cann_ops_tensor.h), bound with ctypes.

`api` exposes the C functions under their own names with their own argument order, so a test written here reads
like a client of the reference (tests/test_elementwise.cpp:159-208 of Atlas-Ascend-Fork/ops-tensor): create handle,
tensor descriptors, operation descriptor, plan preference, plan; execute; destroy.  The `Contraction` helper wraps
that sequence for torch tensors.  All arithmetic runs in libops_tensor_b200.so.
"""
from __future__ import annotations

import ctypes as C

from . import native

# --- enumerations (values of include/cann_ops_tensor_types.h) -----------------------------------------------
R_16F, R_32F, R_64F, R_16BF, R_8I, R_8U, R_32I, R_32U, C_32F, C_64F = range(10)
R_8F_E4M3, R_8F_E5M2, R_4F_E2M1, R_8F_UE8M0, R_64I = 32, 33, 34, 35, 36
COMPUTE_DESC_NONE, COMPUTE_DESC_16F, COMPUTE_DESC_32F, COMPUTE_DESC_64F, COMPUTE_DESC_16BF = 0, 1, 4, 16, 1024
OP_IDENTITY, OP_SQRT, OP_ADD, OP_MUL, OP_RELU, OP_GELU, OP_SILU = 1, 2, 3, 5, 8, 39, 40
OP_SIGMOID, OP_TANH = 11, 12
ALGO_DEFAULT, ALGO_DEFAULT_PATIENT = -1, -6
WORKSPACE_MIN, WORKSPACE_DEFAULT, WORKSPACE_MAX = 1, 2, 3
SCALE_NONE, SCALE_MX_E8M0_VEC32, SCALE_FP32_1X128, SCALE_FP32_128X128 = 0, 1, 2, 3
SCALE_PER_TENSOR, SCALE_PER_CHANNEL = 4, 5
SPLIT_AUTO, SPLIT_DATA_PARALLEL, SPLIT_STREAM_K = 0, 1, 2
(ATTR_SCALE_MODE_A, ATTR_SCALE_MODE_B, ATTR_EPILOGUE_ACT, ATTR_BIAS_TYPE, ATTR_GROUP_COUNT, ATTR_SPLIT_POLICY,
 ATTR_TILE_N, ATTR_SM_LIMIT, ATTR_B_IS_STATIC, ATTR_CTA_PAIR, ATTR_BIAS_PER_BATCH, ATTR_SCALE_MODE_D) = range(1, 13)

STATUS_SUCCESS = 0
STATUS_NOT_INITIALIZED = 1
STATUS_ALLOC_FAILED = 3
STATUS_INVALID_VALUE = 7
STATUS_ARCH_MISMATCH = 8
STATUS_EXECUTION_FAILED = 13
STATUS_INTERNAL_ERROR = 14
STATUS_NOT_SUPPORTED = 15
STATUS_INSUFFICIENT_WORKSPACE = 19
STATUS_IO_ERROR = 21


class ContractionAux(C.Structure):
    _fields_ = [("scaleA", C.c_void_p), ("scaleB", C.c_void_p), ("bias", C.c_void_p), ("groupList", C.c_void_p),
                ("scaleD", C.c_void_p)]


_PROTOTYPES = {
    "acltensorCreate": [C.POINTER(C.c_void_p)],
    "acltensorDestroy": [C.c_void_p],
    "acltensorCreateTensorDescriptor": [C.c_void_p, C.POINTER(C.c_void_p), C.c_uint32, C.POINTER(C.c_int64),
                                        C.POINTER(C.c_int64), C.c_int, C.c_uint32],
    "acltensorDestroyTensorDescriptor": [C.c_void_p],
    "acltensorCreateElementwiseBinary": [C.c_void_p, C.POINTER(C.c_void_p), C.c_void_p, C.POINTER(C.c_int32), C.c_int,
                                         C.c_void_p, C.POINTER(C.c_int32), C.c_int, C.c_void_p, C.POINTER(C.c_int32),
                                         C.c_int, C.c_int],
    "acltensorDestroyOperationDescriptor": [C.c_void_p],
    "acltensorCreatePlanPreference": [C.c_void_p, C.POINTER(C.c_void_p), C.c_int],
    "acltensorDestroyPlanPreference": [C.c_void_p],
    "acltensorCreatePlan": [C.c_void_p, C.POINTER(C.c_void_p), C.c_void_p, C.c_void_p, C.c_uint64],
    "acltensorDestroyPlan": [C.c_void_p],
    "acltensorElementwiseBinaryExecute": [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                          C.c_void_p, C.c_void_p],
    "acltensorCreateContraction": [C.c_void_p, C.POINTER(C.c_void_p), C.c_void_p, C.POINTER(C.c_int32), C.c_int,
                                   C.c_void_p, C.POINTER(C.c_int32), C.c_int, C.c_void_p, C.POINTER(C.c_int32), C.c_int,
                                   C.c_void_p, C.POINTER(C.c_int32), C.c_int],
    "acltensorOperationDescriptorSetAttribute": [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_size_t],
    "acltensorOperationDescriptorGetAttribute": [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_size_t],
    "acltensorEstimateWorkspaceSize": [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.POINTER(C.c_uint64)],
    "acltensorPlanGetRequiredWorkspace": [C.c_void_p, C.POINTER(C.c_uint64)],
    "acltensorHandleResizePlanCache": [C.c_void_p, C.c_uint32],
    "acltensorHandleWritePlanCacheToFile": [C.c_void_p, C.c_char_p],
    "acltensorHandleReadPlanCacheFromFile": [C.c_void_p, C.c_char_p, C.POINTER(C.c_uint32)],
    "acltensorPlanGetKernelChoice": [C.c_void_p, C.POINTER(C.c_int32), C.POINTER(C.c_int32), C.POINTER(C.c_int32),
                                     C.POINTER(C.c_int32)],
    "acltensorContract": [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                          C.c_void_p, C.POINTER(ContractionAux), C.c_void_p, C.c_uint64, C.c_void_p],
    "acltensorQuantize": [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_int, C.c_int, C.c_void_p,
                          C.c_int64, C.c_void_p, C.c_void_p],
    "acltensorGetDeviceStatus": [C.c_void_p, C.POINTER(C.c_int32)],
}


class _Api:
    """The C functions, loaded on first attribute access."""

    def __init__(self):
        self._ready = False

    def _load(self):
        l = native.lib()
        for name, argtypes in _PROTOTYPES.items():
            fn = getattr(l, name)
            fn.argtypes = argtypes
            fn.restype = C.c_int
        l.acltensorGetErrorString.argtypes = [C.c_int]
        l.acltensorGetErrorString.restype = C.c_char_p
        l.acltensorGetVersion.argtypes = []
        l.acltensorGetVersion.restype = C.c_size_t
        self._lib = l
        self._ready = True

    def __getattr__(self, name):
        if name.startswith("_"):
            raise AttributeError(name)
        if not self._ready:
            self._load()
        return getattr(self._lib, name)


api = _Api()


def i64(values):
    return (C.c_int64 * len(values))(*values)


def i32(values):
    return (C.c_int32 * len(values))(*values)


def error_string(status: int) -> str:
    return api.acltensorGetErrorString(status).decode()


def check(status: int, where: str):
    if status != STATUS_SUCCESS:
        raise native.BlazeError(status, f"{where} ({error_string(status)})")


def create_handle() -> C.c_void_p:
    h = C.c_void_p()
    check(api.acltensorCreate(C.byref(h)), "acltensorCreate")
    return h


def resize_plan_cache(handle, entries: int) -> None:
    check(api.acltensorHandleResizePlanCache(handle, entries), "acltensorHandleResizePlanCache")


def write_plan_cache(handle, path: str) -> None:
    check(api.acltensorHandleWritePlanCacheToFile(handle, str(path).encode()), "acltensorHandleWritePlanCacheToFile")


def read_plan_cache(handle, path: str) -> int:
    """Entries read from the file into the handle's plan cache."""
    n = C.c_uint32(0)
    check(api.acltensorHandleReadPlanCacheFromFile(handle, str(path).encode(), C.byref(n)),
          "acltensorHandleReadPlanCacheFromFile")
    return n.value


def create_tensor_descriptor(handle, lens, strides=None, dtype=R_32F, align=256) -> C.c_void_p:
    d = C.c_void_p()
    check(api.acltensorCreateTensorDescriptor(handle, C.byref(d), len(lens), i64(lens),
                                              i64(strides) if strides is not None else None, dtype, align),
          "acltensorCreateTensorDescriptor")
    return d


def set_attribute(handle, desc, attr: int, value: int):
    v = C.c_int32(value)
    check(api.acltensorOperationDescriptorSetAttribute(handle, desc, attr, C.byref(v), 4),
          "acltensorOperationDescriptorSetAttribute")


def get_attribute(handle, desc, attr: int) -> int:
    v = C.c_int32(0)
    check(api.acltensorOperationDescriptorGetAttribute(handle, desc, attr, C.byref(v), 4),
          "acltensorOperationDescriptorGetAttribute")
    return v.value


def elementwise_add(a, c):
    """D = A + C through the full elementwise-binary call sequence of the C API (FP32)."""
    import torch
    d = torch.empty_like(a)
    h = create_handle()
    lens = list(a.shape) if a.dim() > 0 else [1]
    modes = i32(list(range(len(lens))))
    da = create_tensor_descriptor(h, lens)
    dc = create_tensor_descriptor(h, lens)
    dd = create_tensor_descriptor(h, lens)
    op, pref, plan = C.c_void_p(), C.c_void_p(), C.c_void_p()
    try:
        check(api.acltensorCreateElementwiseBinary(h, C.byref(op), da, modes, OP_IDENTITY, dc, modes, OP_IDENTITY, dd,
                                                   modes, OP_ADD, COMPUTE_DESC_32F), "acltensorCreateElementwiseBinary")
        check(api.acltensorCreatePlanPreference(h, C.byref(pref), ALGO_DEFAULT), "acltensorCreatePlanPreference")
        check(api.acltensorCreatePlan(h, C.byref(plan), op, pref, 0), "acltensorCreatePlan")
        one = C.c_float(1.0)
        check(api.acltensorElementwiseBinaryExecute(h, plan, C.byref(one), a.data_ptr(), C.byref(one), c.data_ptr(),
                                                    d.data_ptr(), torch.cuda.current_stream().cuda_stream),
              "acltensorElementwiseBinaryExecute")
    finally:
        api.acltensorDestroyPlan(plan)
        api.acltensorDestroyPlanPreference(pref)
        api.acltensorDestroyOperationDescriptor(op)
        for t in (da, dc, dd):
            api.acltensorDestroyTensorDescriptor(t)
        api.acltensorDestroy(h)
    return d


class Contraction:
    """A planned quantized matmul  D = act(A x B^T + bias) + C  driven through the C API.

    a_shape = (M, K); b_shape = (N, K) or (G, N, K); scale modes choose the kernel family:
    (MX, MX) -> block-scaled MX GEMM; (FP32_1X128, FP32_128X128) -> FP8 GEMM (dense, stream-K or grouped).
    `batch` = extents of up to four leading batch modes of D; `batch_a` / `batch_b` say which of them A and B carry
    (True) or broadcast over (False); all tensors are packed batch after batch (MX only).
    """

    def __init__(self, M, N, K, *, scale_mode_a, scale_mode_b, b_dtype=R_8F_E4M3, groups=0, activation=OP_IDENTITY,
                 bias=False, residual=False, split=SPLIT_AUTO, tile_n=0, sm_limit=0, b_is_static=False, cta_pair=0,
                 lda=None, ldb=None, ldd=None, ldc=None, workspace_limit=2 ** 62, batch=(), batch_a=None, batch_b=None,
                 bias_per_batch=False, a_dtype=R_8F_E4M3, d_dtype=R_16BF, handle=None, algo=ALGO_DEFAULT,
                 bias_dtype=R_16BF):
        self.M, self.N, self.K, self.groups = M, N, K, groups
        # a handle passed in is shared (its plan cache with it) and stays the caller's to destroy
        self._own_handle = handle is None
        self.handle = create_handle() if handle is None else handle
        self._descs = []
        m, n, k, g = 0, 1, 2, 3
        lda = lda or K
        ldb = ldb or K
        ldd = ldd or N
        ldc = ldc or N
        batch = list(batch)
        labels = [10 + i for i in range(len(batch))]
        batch_a = [True] * len(batch) if batch_a is None else list(batch_a)
        batch_b = [False] * len(batch) if batch_b is None else list(batch_b)

        def packed(dims, keep, rows, pitch):
            """lens, strides and modes of [kept batch dims..., rows, cols] packed batch after batch."""
            lens = [d for d, kp in zip(dims, keep) if kp]
            modes = [l for l, kp in zip(labels, keep) if kp]
            strides, step = [], rows * pitch
            for d in reversed(lens):
                strides.insert(0, step)
                step *= d
            return lens, strides, modes

        la, sa, ma = packed(batch, batch_a, M, lda)
        self.dA = create_tensor_descriptor(self.handle, la + [M, K], sa + [lda, 1], a_dtype)
        if groups:
            self.dB = create_tensor_descriptor(self.handle, [groups, N, K], [N * ldb, ldb, 1], b_dtype)
            mode_b = i32([g, n, k])
        else:
            lb, sb, mb = packed(batch, batch_b, N, ldb)
            self.dB = create_tensor_descriptor(self.handle, lb + [N, K], sb + [ldb, 1], b_dtype)
            mode_b = i32(mb + [n, k])
        ld_, sd, md = packed(batch, [True] * len(batch), M, ldd)
        self.dD = create_tensor_descriptor(self.handle, ld_ + [M, N], sd + [ldd, 1], d_dtype)
        self.dC = None
        if residual:
            lc, sc, _ = packed(batch, [True] * len(batch), M, ldc)
            self.dC = create_tensor_descriptor(self.handle, lc + [M, N], sc + [ldc, 1], R_16BF)
        self.op, self.pref, self.plan = C.c_void_p(), C.c_void_p(), C.c_void_p()
        check(api.acltensorCreateContraction(self.handle, C.byref(self.op), self.dA, i32(ma + [m, k]), OP_IDENTITY,
                                             self.dB, mode_b, OP_IDENTITY, self.dC,
                                             i32(md + [m, n]) if residual else None, OP_IDENTITY, self.dD,
                                             i32(md + [m, n]), COMPUTE_DESC_32F),
              "acltensorCreateContraction")
        if bias_per_batch:
            set_attribute(self.handle, self.op, ATTR_BIAS_PER_BATCH, 1)
        if d_dtype == R_8F_E4M3:          # quantising epilogue: D gets the scale mode of A (it is the next layer's A)
            set_attribute(self.handle, self.op, ATTR_SCALE_MODE_D, scale_mode_a)
        set_attribute(self.handle, self.op, ATTR_SCALE_MODE_A, scale_mode_a)
        set_attribute(self.handle, self.op, ATTR_SCALE_MODE_B, scale_mode_b)
        set_attribute(self.handle, self.op, ATTR_EPILOGUE_ACT, activation)
        if bias:
            set_attribute(self.handle, self.op, ATTR_BIAS_TYPE, bias_dtype)
        set_attribute(self.handle, self.op, ATTR_SPLIT_POLICY, split)
        if tile_n:
            set_attribute(self.handle, self.op, ATTR_TILE_N, tile_n)
        if sm_limit:
            set_attribute(self.handle, self.op, ATTR_SM_LIMIT, sm_limit)
        if b_is_static:
            set_attribute(self.handle, self.op, ATTR_B_IS_STATIC, 1)
        if cta_pair:
            set_attribute(self.handle, self.op, ATTR_CTA_PAIR, cta_pair)
        check(api.acltensorCreatePlanPreference(self.handle, C.byref(self.pref), algo),
              "acltensorCreatePlanPreference")
        check(api.acltensorCreatePlan(self.handle, C.byref(self.plan), self.op, self.pref, workspace_limit),
              "acltensorCreatePlan")
        need = C.c_uint64(0)
        check(api.acltensorPlanGetRequiredWorkspace(self.plan, C.byref(need)), "acltensorPlanGetRequiredWorkspace")
        self.workspace_bytes = need.value
        self._workspace = None

    def __call__(self, a, scale_a, b, scale_b, out, *, bias=None, residual=None, group_rows=None, workspace=None,
                 stream=None, scale_out=None):
        import torch
        if workspace is None:
            if self._workspace is None and self.workspace_bytes:
                self._workspace = torch.empty(self.workspace_bytes, dtype=torch.uint8, device=a.device)
            workspace = self._workspace
        aux = ContractionAux(scale_a.data_ptr() if scale_a is not None else None,
                             scale_b.data_ptr() if scale_b is not None else None, bias.data_ptr() if bias is not None else None,
                             group_rows.data_ptr() if group_rows is not None else None,
                             scale_out.data_ptr() if scale_out is not None else None)
        if stream is None:
            stream = torch.cuda.current_stream().cuda_stream
        check(api.acltensorContract(self.handle, self.plan, None, a.data_ptr(), b.data_ptr(), None,
                                    residual.data_ptr() if residual is not None else None, out.data_ptr(),
                                    C.byref(aux), workspace.data_ptr() if workspace is not None else None,
                                    workspace.numel() if workspace is not None else 0, stream), "acltensorContract")
        return out

    def kernel_choice(self):
        """(tile_n, cta_pair, split policy, tuning still pending) of the plan; 0 = left to the launch layer."""
        t, p, s, pend = C.c_int32(0), C.c_int32(0), C.c_int32(0), C.c_int32(0)
        check(api.acltensorPlanGetKernelChoice(self.plan, C.byref(t), C.byref(p), C.byref(s), C.byref(pend)),
              "acltensorPlanGetKernelChoice")
        return t.value, p.value, s.value, bool(pend.value)

    def close(self):
        api.acltensorDestroyPlan(self.plan)
        api.acltensorDestroyPlanPreference(self.pref)
        api.acltensorDestroyOperationDescriptor(self.op)
        for d in (self.dA, self.dB, self.dD, self.dC):
            if d is not None:
                api.acltensorDestroyTensorDescriptor(d)
        if self._own_handle:
            api.acltensorDestroy(self.handle)
        self.plan = self.pref = self.op = self.handle = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
        return False


def quantize(x, scale_mode: int, dtype: int = R_8F_E4M3):
    """fp32 CUDA tensor [rows, cols] -> (codes, scales) through acltensorQuantize."""
    import torch
    rows, cols = x.shape
    dev = x.device
    if scale_mode == SCALE_MX_E8M0_VEC32:
        codes = torch.empty((rows, cols // 2 if dtype == R_4F_E2M1 else cols), dtype=torch.uint8, device=dev)
        scales = torch.empty((rows, native.mx_scale_cols(cols)), dtype=torch.uint8, device=dev)
    elif scale_mode == SCALE_FP32_1X128:
        codes = torch.empty((rows, cols), dtype=torch.uint8, device=dev)
        scales = torch.empty((rows, -(-cols // 128)), dtype=torch.float32, device=dev)
    else:
        codes = torch.empty((rows, cols), dtype=torch.uint8, device=dev)
        scales = torch.empty((-(-cols // 128), -(-rows // 128)), dtype=torch.float32, device=dev)
    check(api.acltensorQuantize(None, x.data_ptr(), x.stride(0), rows, cols, scale_mode, dtype, codes.data_ptr(),
                                codes.stride(0), scales.data_ptr(), torch.cuda.current_stream().cuda_stream),
          "acltensorQuantize")
    return codes, scales


def device_status() -> int:
    """0 when no kernel wait has been abandoned since the last query; synchronises the device."""
    code = C.c_int32(0)
    api.acltensorGetDeviceStatus(None, C.byref(code))
    return code.value
