"""Two GPUs: an N-sharded MXFP8 GEMM computed in column chunks, each chunk all-gathered (NCCL) while the next one
computes, must give the same bits as the same shard computed in one launch and gathered afterwards.

Skipped on a box with fewer than two GPUs.  One process per GPU, rendezvous on 127.0.0.1.
"""
import os
import socket

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, results):
    import torch
    import torch.distributed as dist
    from ops_tensor_b200 import host as H
    from ops_tensor_b200 import shard
    from ops_tensor_b200 import synthetic as syn
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        M, N, K = 512, 2048, 1024                         # N is the global width; every rank owns N / world columns
        n0, n1 = shard.n_shard(N, world, rank, 256)
        width = n1 - n0
        a = torch.from_numpy(syn.normal_f32(7, 0, (M, K), 1.0)).to(dev)
        w = torch.from_numpy(syn.normal_f32(7, 1, (N, K), 1.0)).to(dev)[n0:n1].contiguous()
        bias = torch.from_numpy(syn.normal_f32(7, 2, (N,), 0.1)).to(dev).to(torch.bfloat16)[n0:n1].contiguous()
        mode = H.SCALE_MX_E8M0_VEC32
        qa, sa = H.quantize(a, mode)
        qb, sb = H.quantize(w, mode)

        def plan_for(cols):
            return H.Contraction(M, cols, K, scale_mode_a=mode, scale_mode_b=mode, activation=H.OP_GELU, bias=True)

        local = torch.empty((M, width), dtype=torch.bfloat16, device=dev)
        plan_for(width)(qa, sa, qb, sb, local, bias=bias)
        whole_after = shard.gather_columns(local, world)

        plans = {}

        def run_chunk(c0, c1, out):
            plan = plans.setdefault(c1 - c0, plan_for(c1 - c0))
            plan(qa, sa, qb[c0:c1], sb[c0:c1], out, bias=bias[c0:c1])

        for _ in range(2):                                # the second pass reuses the side stream
            whole = shard.gemm_gather_overlapped(run_chunk, M, width, world, chunks=4, dtype=torch.bfloat16, device=dev,
                                                 multiple=256)
        torch.cuda.synchronize()
        same = bool(torch.equal(whole.view(torch.int16), whole_after.view(torch.int16)))
        # the same again with the chunks pushed into the peers' buffers by device-to-device copies
        peer = shard.PeerGatherBuffers(M, width, world, rank, 4, torch.bfloat16, dev, 256)
        for _ in range(2):
            whole_p = shard.gemm_gather_overlapped(run_chunk, M, width, world, chunks=4, dtype=torch.bfloat16, device=dev,
                                                   multiple=256, peer_buffers=peer)
            torch.cuda.synchronize()
            dist.barrier()                                # nobody overwrites a buffer that a peer still reads
        same = same and bool(torch.equal(whole_p.view(torch.int16), whole_after.view(torch.int16)))
        # and with one full-width GEMM whose epilogue stores every tile to both GPUs' buffers (C ABI: peerD)
        from ops_tensor_b200 import native
        fused = shard.PeerGatherBuffers(M, width, world, rank, 1, torch.bfloat16, dev, 256)

        def run_fused(out, peers):
            native.mx_gemm(qa, sa, qb, sb, out=out, bias=bias, activation=native.ACT_GELU_TANH, peer_outs=peers)

        # closing signal: the step counter in the peers' flag arrays (twice: the counter grows), then the all-reduce
        for sig in ("flag", "flag", "allreduce"):
            fused.gathered[0].zero_()
            torch.cuda.synchronize()
            dist.barrier()                                # nobody's zeroing lands on a peer's fresh tiles
            g = shard.gemm_gather_fused(run_fused, fused, signal=sig)
            torch.cuda.synchronize()                      # this rank's signal kernel has seen every peer's counter
            whole_f = torch.cat([g[r] for r in range(world)], dim=1)
            same = same and bool(torch.equal(whole_f.view(torch.int16), whole_after.view(torch.int16)))
            dist.barrier()
        # the FP8 kernel (stream-K decode shape): output rows go to both GPUs as bulk copies
        Mf, Kf = 128, 2048
        af = torch.from_numpy(syn.normal_f32(8, 0, (Mf, Kf), 1.0)).to(dev)
        wf = (torch.from_numpy(syn.normal_f32(8, 1, (N, Kf), 1.0)).to(dev) * 0.02)[n0:n1].contiguous()
        res = torch.from_numpy(syn.normal_f32(8, 3, (Mf, N), 1.0)).to(dev).to(torch.bfloat16)[:, n0:n1].contiguous()
        qaf, saf = H.quantize(af, H.SCALE_FP32_1X128)
        qbf, sbf = H.quantize(wf, H.SCALE_FP32_128X128)
        for sched in (native.SCHED_STREAM_K, native.SCHED_DATA_PARALLEL):
            plain = native.fp8_gemm(qaf, saf, qbf, sbf, residual=res, sched=sched)
            ref_whole = shard.gather_columns(plain, world)
            fused8 = shard.PeerGatherBuffers(Mf, width, world, rank, 1, torch.bfloat16, dev, 128)
            g8 = shard.gemm_gather_fused(lambda out, peers: native.fp8_gemm(qaf, saf, qbf, sbf, out=out, residual=res,
                                                                            sched=sched, peer_outs=peers), fused8)
            torch.cuda.synchronize()
            dist.barrier()
            whole8 = torch.cat([g8[r] for r in range(world)], dim=1)
            same = same and bool(torch.equal(whole8.view(torch.int16), ref_whole.view(torch.int16)))
        results[rank] = (same, tuple(whole.shape), H.device_status())
    finally:
        dist.destroy_process_group()


def test_chunked_gemm_with_overlapped_gather_matches_gemm_then_gather(cuda_device):
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    ctx = mp.get_context("spawn")
    manager = ctx.Manager()
    results = manager.dict()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, results), daemon=True) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
    for p in procs:
        if p.is_alive():
            p.terminate()
        assert p.exitcode == 0
    for r in range(2):
        same, shape, status = results[r]
        assert same and shape == (512, 2048) and status == 0
