"""Partitioning of the matmul path over the GPUs of one box (host logic only; no collective on the data path).

* Dense GEMMs are split along N: every rank keeps A and its scales, and owns a contiguous range of B's rows
  (= output columns) whose width is a multiple of 128, so that 128x128 scale blocks and tile boundaries never
  straddle two ranks.
* Grouped matmul is split by expert: experts are placed longest-first on the least loaded rank (cost = rows); an
  expert with more rows than the per-rank target is cut into row ranges that may land on different ranks (its weight
  is then needed on each of them).

The reference is single-device (its multi-device line is an unchecked roadmap item, docs/implementation.md:168); this
module is the B200 build's own.  The only collective the path ever needs is an all-gather of output shards when a
consumer wants the whole matrix: `gather_columns` after the GEMM, or `gemm_gather_overlapped`, which computes the
shard in column chunks and gathers each finished chunk while the next one computes.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Sequence, Tuple


def n_shard(N: int, world: int, rank: int, multiple: int = 128) -> Tuple[int, int]:
    """Column range [n0, n1) of `rank`: blocks of `multiple` columns dealt as evenly as possible, in rank order."""
    if world < 1 or not (0 <= rank < world):
        raise ValueError("bad rank/world")
    blocks = -(-N // multiple)
    base, extra = divmod(blocks, world)
    b0 = rank * base + min(rank, extra)
    b1 = b0 + base + (1 if rank < extra else 0)
    return min(b0 * multiple, N), min(b1 * multiple, N)


@dataclass(frozen=True)
class ExpertPiece:
    expert: int
    row_begin: int      # within the expert's rows
    row_end: int

    @property
    def rows(self) -> int:
        return self.row_end - self.row_begin


def plan_experts(group_rows: Sequence[int], world: int, allow_split: bool = True, quantum: int = 128) -> List[List[ExpertPiece]]:
    """Assign experts (or row ranges of oversized experts) to ranks, balancing rows.  Empty experts are dropped.
    Deterministic: every rank computes the same plan from the same group list."""
    total = int(sum(int(r) for r in group_rows))
    target = max(1, -(-total // world))
    pieces: List[ExpertPiece] = []
    for e, r in enumerate(group_rows):
        r = int(r)
        if r <= 0:
            continue
        if allow_split and r > target and world > 1:
            parts = -(-r // target)
            step = -(-(-(-r // parts)) // quantum) * quantum
            b = 0
            while b < r:
                pieces.append(ExpertPiece(e, b, min(r, b + step)))
                b += step
        else:
            pieces.append(ExpertPiece(e, 0, r))
    order = sorted(range(len(pieces)), key=lambda i: (-pieces[i].rows, pieces[i].expert, pieces[i].row_begin))
    load = [0] * world
    plan: List[List[ExpertPiece]] = [[] for _ in range(world)]
    for i in order:
        r = min(range(world), key=lambda j: (load[j], len(plan[j]), j))
        plan[r].append(pieces[i])
        load[r] += pieces[i].rows
    for lst in plan:
        lst.sort(key=lambda p: (p.expert, p.row_begin))
    return plan


def plan_loads(plan: List[List[ExpertPiece]]) -> List[int]:
    return [sum(p.rows for p in lst) for lst in plan]


def gather_columns(local_out, world: int, group=None):
    """All-gather N-shards of equal width into the whole [M, N] matrix (NCCL on GPUs, gloo on CPU tensors)."""
    import torch
    import torch.distributed as dist
    if world == 1:
        return local_out
    parts = [torch.empty_like(local_out) for _ in range(world)]
    dist.all_gather(parts, local_out.contiguous(), group=group)
    return torch.cat(parts, dim=1)


def max_over_ranks(value: float, device=None, group=None) -> float:
    """Largest `value` among the ranks (used for device-timed durations)."""
    import torch
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64, device=device if device is not None else "cpu")
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())


def column_chunks(width: int, chunks: int, multiple: int = 128) -> List[Tuple[int, int]]:
    """Cuts a shard of `width` columns into at most `chunks` ranges of whole `multiple`-column blocks (the last may be ragged)."""
    if width <= 0 or chunks < 1:
        raise ValueError("bad width/chunks")
    blocks = -(-width // multiple)
    chunks = min(chunks, blocks)
    base, extra = divmod(blocks, chunks)
    out, b0 = [], 0
    for c in range(chunks):
        b1 = b0 + base + (1 if c < extra else 0)
        out.append((min(b0 * multiple, width), min(b1 * multiple, width)))
        b0 = b1
    return out


_comm_streams = {}          # one side stream per device for the gathers


def gather_buffers(M: int, width: int, world: int, chunks: int, dtype, device, multiple: int = 128):
    """Chunk outputs [M, wc] and gathered chunks [world, M, wc] for `gemm_gather_overlapped`."""
    import torch
    ranges = column_chunks(width, chunks, multiple)
    outs = [torch.empty((M, c1 - c0), dtype=dtype, device=device) for c0, c1 in ranges]
    gathered = [torch.empty((world, M, c1 - c0), dtype=dtype, device=device) for c0, c1 in ranges] if world > 1 else []
    return outs, gathered


class PeerGatherBuffers:
    """Gathered output chunks in symmetric memory (one process per GPU, one box).

    Every rank maps every peer's copy, so a finished chunk is pushed into the peers' buffers with plain device-to-device
    copies over NVLink: no communication kernel competes with the persistent GEMM for SMs (an NCCL all-gather needs
    ~32 CTAs for its bandwidth and waits for the GEMM's CTAs to retire).  `gathered[c]` is this rank's
    [world, M, chunk width] tensor of chunk c; `peer_slots[c][p]` is the [M, chunk width] slot of this rank inside
    rank p's copy.
    """

    def __init__(self, M: int, width: int, world: int, rank: int, chunks: int, dtype, device, multiple: int = 128,
                 group=None):
        import torch
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm
        self.ranges = column_chunks(width, chunks, multiple)
        self.world, self.rank = world, rank
        self.local = symm.empty(world * M * width, dtype=dtype, device=device)
        self.handle = symm.rendezvous(self.local, group if group is not None else dist.group.WORLD)
        self.gathered, self.peer_slots = [], []
        offset = 0
        for c0, c1 in self.ranges:
            shape = (world, M, c1 - c0)
            count = world * M * (c1 - c0)
            self.gathered.append(self.local[offset:offset + count].view(shape))
            self.peer_slots.append([None if p == rank else self.handle.get_buffer(p, shape, dtype, offset)[rank]
                                    for p in range(world)])
            offset += count
        self.token = torch.zeros(1, dtype=torch.float32, device=device)
        # flag arrays for the closing signal of the fused form (one int64 per rank, in symmetric memory as well)
        self.flags = symm.empty(world, dtype=torch.int64, device=device)
        self.flags.zero_()
        self.flag_handle = symm.rendezvous(self.flags, group if group is not None else dist.group.WORLD)
        self.peer_ranks = [p for p in range(world) if p != rank]
        self.peer_flags = [self.flag_handle.get_buffer(p, (world,), torch.int64, 0) for p in self.peer_ranks]
        self.step = 0
        torch.cuda.synchronize(device)
        dist.barrier(group=group)                      # every rank's flags are zero before anyone signals


def gemm_gather_fused(run_gemm, peer_buffers: "PeerGatherBuffers", group=None, signal: str = "flag"):
    """N-sharded GEMM whose epilogue itself writes every output tile into all ranks' gathered buffers.

    `peer_buffers` must have one chunk.  `run_gemm(out, peer_outs)` launches one GEMM on the current stream that stores
    its result to `out` (this rank's slot of its own buffer) and to each tensor of `peer_outs` (this rank's slot in the
    peers' buffers; `native.mx_gemm(..., peer_outs=...)`).  The stores cross NVLink tile by tile while later tiles
    compute.  Behind the GEMM every rank stores a step counter into its slot of the peers' flag arrays and waits
    (bounded, on the device) for the peers' counters in its own array (`signal="flag"`, `native.peer_signal`: peer
    stores and local loads only), or - `signal="allreduce"` - a one-element all-reduce tells every rank that its peers'
    GEMMs, and with them their stores, have finished.  Returns this rank's [world, M, width] buffer.
    """
    import torch.distributed as dist
    pb = peer_buffers
    if len(pb.ranges) != 1:
        raise ValueError("the fused form writes the whole shard at once: build the buffers with chunks=1")
    run_gemm(pb.gathered[0][pb.rank], [slot for slot in pb.peer_slots[0] if slot is not None])
    if signal == "flag":
        from . import native
        pb.step += 1
        native.peer_signal(pb.flags, pb.peer_flags, pb.rank, pb.peer_ranks, pb.step)
    else:
        dist.all_reduce(pb.token, group=group)
    return pb.gathered[0]


def gemm_gather_overlapped(run_chunk, M: int, width: int, world: int, *, chunks: int = 4, dtype=None, device=None,
                           group=None, multiple: int = 128, assemble: bool = True, buffers=None, peer_buffers=None):
    """N-sharded GEMM whose consumer needs the whole [M, world * width] output on every rank.

    The rank's shard is computed as `chunks` launches, `run_chunk(c0, c1, out)` filling the contiguous [M, c1 - c0]
    tensor `out` with columns [c0, c1) of the shard on the current stream; each finished chunk is all-gathered on a
    second stream while the next one computes, so only the last chunk's gather is exposed.  Every rank must use the
    same `width` and `chunks`.  Returns the whole matrix (columns in rank order), or with `assemble=False` the gathered
    chunks as they arrived, one [world, M, chunk width] tensor per chunk, without the final copy.  On CPU tensors (gloo)
    the gathers are asynchronous work handles instead of a stream.  `buffers` = (chunk outputs, gathered chunks) from
    `gather_buffers` lets a caller that repeats the step reuse its memory.  With `peer_buffers` (a
    `PeerGatherBuffers`, GPUs only) each chunk is computed straight into its slot of the gathered buffer and pushed to
    the peers by device-to-device copies instead of an NCCL all-gather; a one-element all-reduce behind the copies tells
    every rank that its peers' chunks have landed.
    """
    import torch
    import torch.distributed as dist
    if peer_buffers is not None:
        pb = peer_buffers
        compute = torch.cuda.current_stream(pb.local.device)
        comm = _comm_streams.get(pb.local.device)
        if comm is None:
            comm = _comm_streams[pb.local.device] = torch.cuda.Stream(device=pb.local.device)
        for i, (c0, c1) in enumerate(pb.ranges):
            mine = pb.gathered[i][pb.rank]
            run_chunk(c0, c1, mine)
            done = torch.cuda.Event()
            done.record(compute)
            comm.wait_event(done)
            with torch.cuda.stream(comm):
                for slot in pb.peer_slots[i]:
                    if slot is not None:
                        slot.copy_(mine, non_blocking=True)
        with torch.cuda.stream(comm):
            dist.all_reduce(pb.token, group=group)        # behind the copies: when it ends, every peer's copies have too
        compute.wait_stream(comm)
        if not assemble:
            return pb.gathered
        return torch.cat([g[r] for r in range(pb.world) for g in pb.gathered], dim=1)
    ranges = column_chunks(width, chunks, multiple)
    outs, gathered = buffers if buffers is not None else gather_buffers(M, width, world, chunks, dtype, device, multiple)
    if world == 1:
        for (c0, c1), out in zip(ranges, outs):
            run_chunk(c0, c1, out)
        return torch.cat(outs, dim=1) if assemble else [o.unsqueeze(0) for o in outs]
    on_gpu = outs[0].is_cuda
    if on_gpu:
        compute = torch.cuda.current_stream(outs[0].device)
        comm = _comm_streams.get(outs[0].device)
        if comm is None:
            comm = _comm_streams[outs[0].device] = torch.cuda.Stream(device=outs[0].device)
        for (c0, c1), out, g in zip(ranges, outs, gathered):
            run_chunk(c0, c1, out)
            done = torch.cuda.Event()
            done.record(compute)
            comm.wait_event(done)
            with torch.cuda.stream(comm):
                dist.all_gather_into_tensor(g.view(world * M, -1), out, group=group)
            out.record_stream(comm)
            g.record_stream(comm)
        compute.wait_stream(comm)
    else:
        pending = []
        for (c0, c1), out, g in zip(ranges, outs, gathered):
            run_chunk(c0, c1, out)
            pending.append(dist.all_gather_into_tensor(g.view(world * M, -1), out, group=group, async_op=True))
        for w in pending:
            w.wait()
    if not assemble:
        return gathered
    # rank r's shard = its chunks side by side; the whole = the shards side by side
    return torch.cat([g[r] for r in range(world) for g in gathered], dim=1)
