"""ctypes binding of libops_tensor_b200.so.

Loading fails loudly when the library has not been built: there is no CPU or PyTorch fallback for any operation of
this package.  torch tensors are used only as owners of device memory; every computation happens inside the shared
library.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

_LIB_PATH = Path(__file__).resolve().parent / "libops_tensor_b200.so"

STATUS_SUCCESS = 0
STATUS_NOT_INITIALIZED = 1
STATUS_ALLOC_FAILED = 3
STATUS_INVALID_VALUE = 7
STATUS_ARCH_MISMATCH = 8
STATUS_EXECUTION_FAILED = 13
STATUS_INTERNAL_ERROR = 14
STATUS_NOT_SUPPORTED = 15
STATUS_INSUFFICIENT_WORKSPACE = 19

ELEM_E4M3, ELEM_E2M1, ELEM_E5M2 = 0, 1, 2
ACT_IDENTITY, ACT_RELU, ACT_GELU_TANH, ACT_SILU, ACT_SIGMOID, ACT_TANH = 0, 1, 2, 3, 4, 5
SCHED_AUTO, SCHED_DATA_PARALLEL, SCHED_STREAM_K = 0, 1, 2
OUT_BF16, OUT_F16, OUT_F32, OUT_MX_E4M3, OUT_FP8_128 = 0, 1, 2, 3, 4


def out_type_of(tensor) -> int:
    """blazeOutType_t of a torch output tensor (bf16, half or float32)."""
    import torch
    return {torch.bfloat16: OUT_BF16, torch.float16: OUT_F16, torch.float32: OUT_F32,
            torch.uint8: OUT_MX_E4M3}[tensor.dtype]


class MxGemmArgs(C.Structure):
    _fields_ = [
        ("struct_size", C.c_size_t),
        ("M", C.c_int32), ("N", C.c_int32), ("K", C.c_int32),
        ("b_elem", C.c_int32),
        ("A", C.c_void_p), ("lda", C.c_int64),
        ("B", C.c_void_p), ("ldb", C.c_int64),
        ("scaleA", C.c_void_p), ("scaleB", C.c_void_p),
        ("bias", C.c_void_p),
        ("residual", C.c_void_p), ("ldr", C.c_int64),
        ("D", C.c_void_p), ("ldd", C.c_int64),
        ("activation", C.c_int32),
        ("tile_n", C.c_int32),
        ("reuse_b_prepass", C.c_int32),
        ("sm_limit", C.c_int32),
        ("cta_pair", C.c_int32),
        ("a_elem", C.c_int32),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("d_type", C.c_int32), ("b_layout", C.c_int32),
        ("scaleD", C.c_void_p),
        ("sched", C.c_int32), ("n_peers", C.c_int32),
        ("peerD", C.c_void_p * 7),
    ]


class BatchDims(C.Structure):
    """blazeBatchDims: batch extents of D, A and B (outermost first, 1 = unused or broadcast)."""
    _fields_ = [("c", C.c_int32 * 4), ("a", C.c_int32 * 4), ("b", C.c_int32 * 4), ("bias_per_batch", C.c_int32),
                ("reserved", C.c_int32)]


class Fp8GemmArgs(C.Structure):
    _fields_ = [
        ("struct_size", C.c_size_t),
        ("M", C.c_int32), ("N", C.c_int32), ("K", C.c_int32),
        ("groups", C.c_int32),
        ("group_rows", C.c_void_p),
        ("A", C.c_void_p), ("lda", C.c_int64),
        ("B", C.c_void_p), ("ldb", C.c_int64),
        ("scaleA", C.c_void_p), ("scaleB", C.c_void_p),
        ("bias", C.c_void_p),
        ("residual", C.c_void_p), ("ldr", C.c_int64),
        ("D", C.c_void_p), ("ldd", C.c_int64),
        ("activation", C.c_int32),
        ("sched", C.c_int32),
        ("sm_limit", C.c_int32),
        ("d_type", C.c_int32),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("scaleD", C.c_void_p),
        ("n_peers", C.c_int32), ("b_is_static", C.c_int32),
        ("peerD", C.c_void_p * 7),
    ]


class DenseGemmArgs(C.Structure):
    """blazeDenseGemmArgs: INT8 (A8W8) and fp16 / bf16 GEMMs without block scales."""
    _fields_ = [
        ("struct_size", C.c_size_t),
        ("M", C.c_int32), ("N", C.c_int32), ("K", C.c_int32),
        ("kind", C.c_int32),
        ("A", C.c_void_p), ("lda", C.c_int64),
        ("B", C.c_void_p), ("ldb", C.c_int64),
        ("scale_mode", C.c_int32), ("activation", C.c_int32),
        ("scaleA", C.c_void_p), ("scaleB", C.c_void_p), ("scaleN", C.c_void_p),
        ("bias", C.c_void_p),
        ("residual", C.c_void_p), ("ldr", C.c_int64),
        ("D", C.c_void_p), ("ldd", C.c_int64),
        ("d_type", C.c_int32), ("sm_limit", C.c_int32),
    ]


DENSE_S8, DENSE_F16, DENSE_BF16 = 0, 1, 2
DENSE_SCALE_NONE, DENSE_SCALE_PER_TENSOR, DENSE_SCALE_PER_CHANNEL = 0, 1, 2
OUT_S32 = 5


class BlazeError(RuntimeError):
    def __init__(self, status: int, where: str):
        self.status = status
        super().__init__(f"{where} failed with acltensorStatus_t {status}")


_lib = None


def lib() -> C.CDLL:
    """The loaded shared library; raises if it is missing (build it with `python -m ops_tensor_b200.build`)."""
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            raise RuntimeError(
                f"{_LIB_PATH} is missing: the CUDA library has not been built. Run `python -m ops_tensor_b200.build`. "
                "There is no fallback path.")
        _lib = C.CDLL(str(_LIB_PATH))
        _declare(_lib)
    return _lib


def _declare(l: C.CDLL) -> None:
    l.blazeMxGemmWorkspaceSize.argtypes = [C.POINTER(MxGemmArgs), C.POINTER(C.c_size_t)]
    l.blazeMxGemm.argtypes = [C.POINTER(MxGemmArgs), C.c_void_p]
    l.blazeMxGemmNoAlloc.argtypes = [C.POINTER(MxGemmArgs), C.c_void_p, C.c_void_p]
    l.blazeMxGemmNoAlloc.restype = C.c_int
    l.blazeMxGemmBatchedWorkspaceSize.argtypes = [C.POINTER(MxGemmArgs), C.POINTER(BatchDims), C.POINTER(C.c_size_t)]
    l.blazeMxGemmBatchedWorkspaceSize.restype = C.c_int
    l.blazeMxGemmBatched.argtypes = [C.POINTER(MxGemmArgs), C.POINTER(BatchDims), C.c_void_p]
    l.blazeMxGemmBatched.restype = C.c_int
    l.blazeDenseGemm.argtypes = [C.POINTER(DenseGemmArgs), C.c_void_p]
    l.blazeDenseGemm.restype = C.c_int
    l.blazeFp8GemmWorkspaceSize.argtypes = [C.POINTER(Fp8GemmArgs), C.POINTER(C.c_size_t)]
    l.blazeFp8Gemm.argtypes = [C.POINTER(Fp8GemmArgs), C.c_void_p]
    l.blazeQuantizeMx.argtypes = [C.c_void_p, C.c_int64, C.c_int32, C.c_int32, C.c_int32, C.c_void_p, C.c_int64,
                                  C.c_void_p, C.c_void_p]
    l.blazeQuantizeFp8RowGroups.argtypes = [C.c_void_p, C.c_int64, C.c_int32, C.c_int32, C.c_void_p, C.c_int64,
                                            C.c_void_p, C.c_void_p]
    l.blazeQuantizeFp8Blocks.argtypes = [C.c_void_p, C.c_int64, C.c_int32, C.c_int32, C.c_void_p, C.c_int64,
                                         C.c_void_p, C.c_void_p]
    l.blazeAddF32.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p]
    l.blazeSelfTestWaitTimeout.argtypes = [C.c_int64, C.c_void_p]
    l.blazeSelfTestWaitTimeout.restype = C.c_int
    l.blazeDeviceStatus.argtypes = [C.POINTER(C.c_int32), C.c_int32]
    l.blazeDeviceInfo.argtypes = [C.POINTER(C.c_int32), C.POINTER(C.c_int32), C.POINTER(C.c_int32)]
    for name in ("blazeMxGemmWorkspaceSize", "blazeMxGemm", "blazeFp8GemmWorkspaceSize", "blazeFp8Gemm",
                 "blazeQuantizeMx", "blazeQuantizeFp8RowGroups", "blazeQuantizeFp8Blocks", "blazeAddF32",
                 "blazeDeviceStatus", "blazeDeviceInfo"):
        getattr(l, name).restype = C.c_int


def check(status: int, where: str) -> None:
    if status != STATUS_SUCCESS:
        raise BlazeError(status, where)


def _ptr(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def _stream():
    import torch
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def device_status(reset: bool = True) -> int:
    v = C.c_int32(0)
    check(lib().blazeDeviceStatus(C.byref(v), 1 if reset else 0), "blazeDeviceStatus")
    return v.value


def device_info():
    a, b, c = C.c_int32(), C.c_int32(), C.c_int32()
    check(lib().blazeDeviceInfo(C.byref(a), C.byref(b), C.byref(c)), "blazeDeviceInfo")
    return a.value, b.value, c.value


# ------------------------------------------------------------------------------------------------ quantisers

def mx_scale_cols(K: int) -> int:
    return -(-K // 64) * 2


def quantize_mx(x, elem: int = ELEM_E4M3):
    """x: float32 CUDA tensor [rows, K] -> (codes uint8 [rows, K] or [rows, K/2], scales uint8 [rows, ceil(K/64)*2])."""
    import torch
    assert x.is_cuda and x.dtype == torch.float32 and x.dim() == 2 and x.stride(1) == 1
    rows, K = x.shape
    codes = torch.empty((rows, K // 2 if elem == ELEM_E2M1 else K), dtype=torch.uint8, device=x.device)
    scales = torch.empty((rows, mx_scale_cols(K)), dtype=torch.uint8, device=x.device)
    check(lib().blazeQuantizeMx(_ptr(x), x.stride(0), rows, K, elem, _ptr(codes), codes.stride(0), _ptr(scales),
                                _stream()), "blazeQuantizeMx")
    return codes, scales


def quantize_fp8_row_groups(x):
    import torch
    assert x.is_cuda and x.dtype == torch.float32 and x.dim() == 2 and x.stride(1) == 1
    rows, K = x.shape
    codes = torch.empty((rows, K), dtype=torch.uint8, device=x.device)
    scales = torch.empty((rows, -(-K // 128)), dtype=torch.float32, device=x.device)
    check(lib().blazeQuantizeFp8RowGroups(_ptr(x), x.stride(0), rows, K, _ptr(codes), codes.stride(0), _ptr(scales),
                                          _stream()), "blazeQuantizeFp8RowGroups")
    return codes, scales


def quantize_fp8_blocks(w):
    import torch
    assert w.is_cuda and w.dtype == torch.float32 and w.dim() == 2 and w.stride(1) == 1
    N, K = w.shape
    codes = torch.empty((N, K), dtype=torch.uint8, device=w.device)
    scales = torch.empty((-(-K // 128), -(-N // 128)), dtype=torch.float32, device=w.device)
    check(lib().blazeQuantizeFp8Blocks(_ptr(w), w.stride(0), N, K, _ptr(codes), codes.stride(0), _ptr(scales),
                                       _stream()), "blazeQuantizeFp8Blocks")
    return codes, scales


# ------------------------------------------------------------------------------------------------ GEMMs

def mx_gemm_args(a, sa, b, sb, out, *, b_elem=ELEM_E4M3, bias=None, residual=None, activation=ACT_IDENTITY,
                 tile_n=0, reuse_b_prepass=False, sm_limit=0, cta_pair=0, workspace=None, a_elem=ELEM_E4M3,
                 scale_out=None, b_n_major=False, sched=SCHED_AUTO, peer_outs=None) -> MxGemmArgs:
    M, K = a.shape
    if a_elem == ELEM_E2M1:
        K *= 2                       # two codes per byte
    N = b.shape[1] if b_n_major else b.shape[0]
    args = MxGemmArgs()
    args.struct_size = C.sizeof(MxGemmArgs)
    args.M, args.N, args.K = M, N, K
    args.b_elem = b_elem
    args.A, args.lda = a.data_ptr(), a.stride(0)
    args.B, args.ldb = b.data_ptr(), b.stride(0)
    args.scaleA, args.scaleB = sa.data_ptr(), sb.data_ptr()
    args.bias = bias.data_ptr() if bias is not None else None
    args.residual = residual.data_ptr() if residual is not None else None
    args.ldr = residual.stride(0) if residual is not None else 0
    args.D, args.ldd = out.data_ptr(), out.stride(0)
    args.d_type = out_type_of(out)
    args.activation = activation
    args.tile_n = tile_n
    args.reuse_b_prepass = 1 if reuse_b_prepass else 0
    args.sm_limit = sm_limit
    args.cta_pair = cta_pair
    args.a_elem = a_elem
    args.scaleD = scale_out.data_ptr() if scale_out is not None else None
    args.b_layout = 1 if b_n_major else 0
    args.sched = sched
    if peer_outs:
        # further copies of `out` (same shape, pitch and dtype) that the epilogue stores every tile to as well
        if len(peer_outs) > 7 or any(t.shape != out.shape or t.stride(0) != out.stride(0) or t.dtype != out.dtype
                                     for t in peer_outs):
            raise ValueError("peer outputs must match the output's shape, pitch and dtype (at most 7)")
        args.n_peers = len(peer_outs)
        for i, t in enumerate(peer_outs):
            args.peerD[i] = t.data_ptr()
    if workspace is not None:
        args.workspace, args.workspace_bytes = workspace.data_ptr(), workspace.numel() * workspace.element_size()
    return args


def mx_gemm_workspace_bytes(args: MxGemmArgs) -> int:
    n = C.c_size_t(0)
    check(lib().blazeMxGemmWorkspaceSize(C.byref(args), C.byref(n)), "blazeMxGemmWorkspaceSize")
    return n.value


def mx_gemm(a, sa, b, sb, *, out=None, workspace=None, **kw):
    """D = act(A x B^T + bias) + residual for MX operands; allocates `out` / `workspace` when not given."""
    import torch
    M = a.shape[0]
    N = b.shape[1] if kw.get("b_n_major") else b.shape[0]
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=a.device)
    args = mx_gemm_args(a, sa, b, sb, out, workspace=workspace, **kw)
    if workspace is None:
        need = mx_gemm_workspace_bytes(args)
        workspace = torch.empty(max(need, 256), dtype=torch.uint8, device=a.device)
        args.workspace, args.workspace_bytes = workspace.data_ptr(), workspace.numel()
    check(lib().blazeMxGemm(C.byref(args), _stream()), "blazeMxGemm")
    return out


def fp8_gemm_args(a, sa, b, sb, out, *, group_rows=None, bias=None, residual=None, activation=ACT_IDENTITY,
                  sched=SCHED_AUTO, sm_limit=0, workspace=None, scale_out=None, peer_outs=None,
                  b_is_static=False) -> Fp8GemmArgs:
    M, K = a.shape
    if b.dim() == 3:
        G, N, _ = b.shape
        ldb = b.stride(1)
    else:
        G, (N, _) = 0, b.shape
        ldb = b.stride(0)
    args = Fp8GemmArgs()
    args.struct_size = C.sizeof(Fp8GemmArgs)
    args.M, args.N, args.K = M, N, K
    args.groups = G
    args.group_rows = group_rows.data_ptr() if group_rows is not None else None
    args.A, args.lda = a.data_ptr(), a.stride(0)
    args.B, args.ldb = b.data_ptr(), ldb
    args.scaleA, args.scaleB = sa.data_ptr(), sb.data_ptr()
    args.bias = bias.data_ptr() if bias is not None else None
    args.residual = residual.data_ptr() if residual is not None else None
    args.ldr = residual.stride(0) if residual is not None else 0
    args.D, args.ldd = out.data_ptr(), out.stride(0)
    args.d_type = OUT_FP8_128 if scale_out is not None else out_type_of(out)
    args.scaleD = scale_out.data_ptr() if scale_out is not None else None
    args.activation = activation
    args.sched = sched
    args.sm_limit = sm_limit
    args.b_is_static = 1 if b_is_static else 0
    if peer_outs:
        if len(peer_outs) > 7 or any(t.shape != out.shape or t.stride(0) != out.stride(0) or t.dtype != out.dtype
                                     for t in peer_outs):
            raise ValueError("peer outputs must match the output's shape, pitch and dtype (at most 7)")
        args.n_peers = len(peer_outs)
        for i, t in enumerate(peer_outs):
            args.peerD[i] = t.data_ptr()
    if workspace is not None:
        args.workspace, args.workspace_bytes = workspace.data_ptr(), workspace.numel() * workspace.element_size()
    return args


def fp8_gemm_workspace_bytes(args: Fp8GemmArgs) -> int:
    n = C.c_size_t(0)
    check(lib().blazeFp8GemmWorkspaceSize(C.byref(args), C.byref(n)), "blazeFp8GemmWorkspaceSize")
    return n.value


def fp8_gemm(a, sa, b, sb, *, out=None, workspace=None, **kw):
    import torch
    M = a.shape[0]
    N = b.shape[-2]
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=a.device)
    args = fp8_gemm_args(a, sa, b, sb, out, workspace=workspace, **kw)
    if workspace is None:
        need = fp8_gemm_workspace_bytes(args)
        if need:
            workspace = torch.empty(need, dtype=torch.uint8, device=a.device)
            args.workspace, args.workspace_bytes = workspace.data_ptr(), workspace.numel()
    check(lib().blazeFp8Gemm(C.byref(args), _stream()), "blazeFp8Gemm")
    return out


def dense_gemm(a, b, *, out=None, out_dtype=None, scale_a=None, scale_b=None, scale_n=None, bias=None, residual=None,
               activation=ACT_IDENTITY, sm_limit=0):
    """D = act(A x B^T + bias) + residual for int8, half or bf16 operands (A [M, K], B [N, K], K contiguous).
    int8: `scale_a` and `scale_b` (one float32 each) or `scale_n` (uint64 per column) de-quantise on store, `bias` is
    int32; with no scale and an int32 `out` the raw sums are stored."""
    import torch
    M, K = a.shape
    N = b.shape[0]
    kind = {torch.int8: DENSE_S8, torch.float16: DENSE_F16, torch.bfloat16: DENSE_BF16}[a.dtype]
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype or (torch.float16 if kind != DENSE_BF16 else torch.bfloat16),
                          device=a.device)
    args = DenseGemmArgs()
    args.struct_size = C.sizeof(DenseGemmArgs)
    args.M, args.N, args.K = M, N, K
    args.kind = kind
    args.A, args.lda = a.data_ptr(), a.stride(0)
    args.B, args.ldb = b.data_ptr(), b.stride(0)
    args.scale_mode = DENSE_SCALE_PER_CHANNEL if scale_n is not None else (
        DENSE_SCALE_PER_TENSOR if scale_a is not None else DENSE_SCALE_NONE)
    args.activation = activation
    args.scaleA = scale_a.data_ptr() if scale_a is not None else None
    args.scaleB = scale_b.data_ptr() if scale_b is not None else None
    args.scaleN = scale_n.data_ptr() if scale_n is not None else None
    args.bias = bias.data_ptr() if bias is not None else None
    args.residual = residual.data_ptr() if residual is not None else None
    args.ldr = residual.stride(0) if residual is not None else 0
    args.D, args.ldd = out.data_ptr(), out.stride(0)
    args.d_type = OUT_S32 if out.dtype == torch.int32 else out_type_of(out)
    args.sm_limit = sm_limit
    check(lib().blazeDenseGemm(C.byref(args), _stream()), "blazeDenseGemm")
    return out


MAX_PEERS = 7          # BLAZE_MAX_PEERS


class PeerSignalArgs(C.Structure):
    _fields_ = [
        ("struct_size", C.c_size_t),
        ("my_rank", C.c_int32),
        ("n_peers", C.c_int32),
        ("peer_ranks", C.c_int32 * MAX_PEERS),
        ("local_flags", C.c_void_p),
        ("peer_flags", C.c_void_p * MAX_PEERS),
        ("value", C.c_uint64),
        ("limit_cycles", C.c_int64),
    ]


def peer_signal(local_flags, peer_flags, my_rank: int, peer_ranks, value: int, limit_cycles: int = 0) -> None:
    """Closing signal of a fused gather (`blazePeerSignal`): stores `value` into slot `my_rank` of every peer's flag
    array and waits, bounded, until this GPU's own array shows `value` from every peer.  `local_flags`: this rank's
    int64 tensor [ranks]; `peer_flags`: the peers' arrays as mapped into this process, in the order of `peer_ranks`."""
    args = PeerSignalArgs()
    args.struct_size = C.sizeof(PeerSignalArgs)
    args.my_rank = my_rank
    args.n_peers = len(peer_flags)
    for q, (t, r) in enumerate(zip(peer_flags, peer_ranks)):
        args.peer_flags[q] = t.data_ptr()
        args.peer_ranks[q] = r
    args.local_flags = local_flags.data_ptr()
    args.value = value
    args.limit_cycles = limit_cycles
    l = lib()
    l.blazePeerSignal.restype = C.c_int
    check(l.blazePeerSignal(C.byref(args), _stream()), "blazePeerSignal")


def add_f32(a, c, out=None):
    import torch
    if out is None:
        out = torch.empty_like(a)
    check(lib().blazeAddF32(_ptr(a), _ptr(c), _ptr(out), a.numel(), _stream()), "blazeAddF32")
    return out
