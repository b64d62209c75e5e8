"""blazeMxGemmNoAlloc: the MX GEMM for hosts that cannot hand the library device memory.

Some processes that load this library never let a plugin allocate on the GPU: an inference server that reserved the
whole device for its own pool, or a real-time loop where an allocation would stall the GPU.  For them the GEMM keeps
its scratch (the re-tiled scale factors) in a fixed 8 MiB array inside the library.  This test calls that entry
point through the C ABI twice in a row, on two different problems, so the second call finds the first call's data in
the shared array, and requires the same bits as the regular entry point produces with caller-provided workspace.
tests/conftest.py moves this file's tests to the end of the collection, so that a run stopping at the first failure
has already run every other test.
"""
import ctypes as C

import numpy as np
import pytest

import blaze_oracle as o
from ops_tensor_b200 import native

pytestmark = pytest.mark.gpu


def _problem(device, cfg, M, N, K, with_bias):
    import torch
    a = o.normal_f32(cfg, 0, (M, K), 1.0)
    w = o.normal_f32(cfg, 1, (N, K), 0.5)
    to_dev = lambda x: torch.from_numpy(np.ascontiguousarray(x)).to(device)
    qa, sa = native.quantize_mx(to_dev(a))
    qb, sb = native.quantize_mx(to_dev(w))
    bias = to_dev(o.bf16_round(o.normal_f32(cfg, 2, (N,), 0.3))).to(torch.bfloat16) if with_bias else None
    return qa, sa, qb, sb, bias


def _run_both(device, qa, sa, qb, sb, bias, activation):
    import torch
    M, N = qa.shape[0], qb.shape[0]
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    # (the regular entry may cut a partly filled last round of tiles along K, which needs workspace the other entry does
    # not have; whole tiles on both sides make the two results comparable bit for bit)
    want = native.mx_gemm(qa, sa, qb, sb, bias=bias, activation=activation, sched=native.SCHED_DATA_PARALLEL)
    got = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=device)
    status_word = torch.zeros(1, dtype=torch.int32, device=device)
    args = native.mx_gemm_args(qa, sa, qb, sb, got, bias=bias, activation=activation)      # no workspace given
    rc = native.lib().blazeMxGemmNoAlloc(C.byref(args), C.c_void_p(status_word.data_ptr()), stream)
    assert rc == native.STATUS_SUCCESS
    torch.cuda.synchronize()
    assert int(status_word.item()) == 0
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))
    # a further call leaves the amount of free device memory exactly where it was: nothing was allocated or freed
    free_before = torch.cuda.mem_get_info()[0]
    rc = native.lib().blazeMxGemmNoAlloc(C.byref(args), C.c_void_p(status_word.data_ptr()), stream)
    torch.cuda.synchronize()
    assert rc == native.STATUS_SUCCESS and torch.cuda.mem_get_info()[0] == free_before
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))
    return got


def test_no_alloc_entry_matches_regular_entry_twice(cuda_device):
    import torch
    first = _problem(cuda_device, 31, 300, 520, 1040, with_bias=True)
    second = _problem(cuda_device, 32, 128, 224, 256, with_bias=False)
    allocated = torch.cuda.memory_allocated()
    out1 = _run_both(cuda_device, *first, activation=native.ACT_GELU_TANH)
    out2 = _run_both(cuda_device, *second, activation=native.ACT_IDENTITY)      # finds call one's tiles in the array
    assert torch.isfinite(out1.float()).all() and torch.isfinite(out2.float()).all()
    # and the result is right, not merely equal: compare the second problem with the float64 oracle
    qa, sa, qb, sb, _ = second
    ref = o.matmul_ref64(o.dequant_mx(qa.cpu().numpy(), sa.cpu().numpy(), 256),
                         o.dequant_mx(qb.cpu().numpy(), sb.cpu().numpy(), 256))
    assert o.maxrel(out2.float().cpu().numpy(), ref) <= 1e-2
    del out1, out2
    assert torch.cuda.memory_allocated() <= allocated + (1 << 20)


def test_no_alloc_entry_keeps_one_scale_copy_when_four_do_not_fit(cuda_device):
    """M=256, N=K=8192: four copies of the weight's re-tiled scale blocks (what the regular entry uses on 2-CTA tiles)
    need over 8 MiB, one copy needs 2 MiB; the allocation-free entry takes the second form and returns the same bits."""
    problem = _problem(cuda_device, 33, 256, 8192, 8192, with_bias=True)
    out = _run_both(cuda_device, *problem, activation=native.ACT_RELU)
    assert bool((out.float() >= 0).all())


def test_no_alloc_entry_refuses_what_does_not_fit(cuda_device):
    """Too large for the 8 MiB array, or needing an expansion buffer: refused before any launch.  Every operand pointer
    is NULL, so no ordering of the checks could ever start a kernel: were the size check not first, the NULL check would
    answer INVALID_VALUE instead and this test would fail without touching the GPU."""
    a = native.MxGemmArgs()
    a.struct_size = C.sizeof(a)
    a.M = a.N = a.K = 32768                       # re-tiled scales alone need ~70 MiB
    a.lda = a.ldb = a.ldd = 32768
    assert native.lib().blazeMxGemmNoAlloc(C.byref(a), None, None) == native.STATUS_INSUFFICIENT_WORKSPACE
    a.M = a.N = a.K = 256
    a.lda = a.ldb = a.ldd = 256
    a.b_elem = native.ELEM_E2M1
    assert native.lib().blazeMxGemmNoAlloc(C.byref(a), None, None) == native.STATUS_NOT_SUPPORTED
    a.b_elem = native.ELEM_E4M3
    a.b_layout = 1                                # an N-major B would need a transposed copy
    assert native.lib().blazeMxGemmNoAlloc(C.byref(a), None, None) == native.STATUS_NOT_SUPPORTED
    a.b_layout = 0
    assert native.lib().blazeMxGemmNoAlloc(C.byref(a), None, None) == native.STATUS_INVALID_VALUE     # NULL operands


def test_no_alloc_calls_on_two_streams_ordered_by_an_event(cuda_device):
    """The documented way to use the entry from more than one stream: the calls share one scratch array, so the second
    stream waits for an event recorded behind the first call.  Ordered like that, both calls give the regular bits."""
    import torch
    first = _problem(cuda_device, 35, 384, 520, 512, with_bias=True)
    second = _problem(cuda_device, 36, 200, 264, 1024, with_bias=False)
    want1 = native.mx_gemm(*first[:4], bias=first[4], activation=native.ACT_RELU, sched=native.SCHED_DATA_PARALLEL)
    want2 = native.mx_gemm(*second[:4], bias=None, activation=native.ACT_IDENTITY, sched=native.SCHED_DATA_PARALLEL)
    got1, got2 = torch.empty_like(want1), torch.empty_like(want2)
    args1 = native.mx_gemm_args(*first[:4], got1, bias=first[4], activation=native.ACT_RELU)
    args2 = native.mx_gemm_args(*second[:4], got2, activation=native.ACT_IDENTITY)
    torch.cuda.synchronize()
    s1, s2 = torch.cuda.Stream(device=cuda_device), torch.cuda.Stream(device=cuda_device)
    done = torch.cuda.Event()
    for _ in range(3):
        assert native.lib().blazeMxGemmNoAlloc(C.byref(args1), None, C.c_void_p(s1.cuda_stream)) == native.STATUS_SUCCESS
        done.record(s1)
        s2.wait_event(done)
        assert native.lib().blazeMxGemmNoAlloc(C.byref(args2), None, C.c_void_p(s2.cuda_stream)) == native.STATUS_SUCCESS
        done.record(s2)
        s1.wait_event(done)
    s1.synchronize()
    s2.synchronize()
    assert torch.equal(got1.view(torch.int16), want1.view(torch.int16))
    assert torch.equal(got2.view(torch.int16), want2.view(torch.int16))
    # with no status pointer given, a wait that gave up would show in the device status query: nothing did
    assert native.device_status() == 0
