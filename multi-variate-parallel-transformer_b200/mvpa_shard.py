"""Multi-GPU partitioning of the MVPA operator (one process per GPU, `torch.distributed`).

Two ways the path shards (no counterpart in the reference, whose only parallelism is Lightning
DDP, `configs/*.yaml:3-6`):

1. Independent units.  Every (batch element, kv-head group) is independent, so a job splits its
   batch (or its heads) across ranks and calls `attentions.flashmvpa` unchanged; no collective on
   the data path.  `batch_slice` gives a rank its share.

2. One long sample across ranks.  Queries are split by time blocks; each rank projects K/V for its
   own tokens, all ranks all-gather K and V into local HBM (NCCL over NVLink; `gloo` in the CPU
   tests), and each rank runs the kernel on its own query rows against the gathered K/V
   (`q_time_range`).  Causality makes late time blocks more expensive than early ones, so the
   time axis is cut into 2R chunks and rank r owns chunks r and 2R-1-r ("zig-zag"), which
   balances the causal work to within one chunk.

   The gather is split in the same two halves and runs on a communication stream
   (`start_kv_gather`): the early half (chunks 0..R-1) goes straight into its final place in the
   `(B, N, heads, D)` buffer with one `all_gather_into_tensor`; the late half follows.  A rank's
   early chunk is causal, so it needs the early half only: its attention starts as soon as that
   half has landed and runs while the late half is still arriving.  Whatever the caller passes as
   `overlap` (at model level the MLP branch of the parallel block, `models/mvpformer.py:146-147`,
   which does not depend on attention) is enqueued before the first wait and runs during the
   early half.  The kernels read only local HBM, through ordinary per-CTA TMA loads.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist


def batch_slice(n_items: int, world: int, rank: int) -> slice:
    """Contiguous share of `n_items` independent units for `rank` (sizes differ by at most one)."""
    base, extra = divmod(n_items, world)
    start = rank * base + min(rank, extra)
    return slice(start, start + base + (1 if rank < extra else 0))


def tile_time_steps(C: int) -> int:
    """Time steps per 128-row tile of the tensor-core forward: query ranges must start on these."""
    cp = 32 if C <= 32 else (64 if C <= 64 else 128)
    return 128 // cp


def zigzag_chunks(T: int, C: int, world: int) -> List[List[Tuple[int, int]]]:
    """Time ranges `(t0, n)` owned by each rank: 2*world tile-aligned chunks, rank r gets chunks
    r and 2*world-1-r.  Chunks may be empty (n == 0) when T is small; every time step is owned once."""
    step = tile_time_steps(C)
    n_chunks = 2 * world
    tiles = -(-T // step)
    bounds = [min(T, step * ((tiles * i) // n_chunks)) for i in range(n_chunks + 1)]
    chunks = [(bounds[i], bounds[i + 1] - bounds[i]) for i in range(n_chunks)]
    return [[chunks[r], chunks[n_chunks - 1 - r]] for r in range(world)]


def causal_work(T: int, owned: Sequence[Tuple[int, int]]) -> int:
    """Number of (query time step, key time step) pairs a rank evaluates: its share of the work."""
    return sum(t + 1 for t0, n in owned for t in range(t0, t0 + n))


_comm_streams = {}


def _comm_stream(device: torch.device) -> "torch.cuda.Stream":
    key = (device.type, device.index)
    if key not in _comm_streams:
        _comm_streams[key] = torch.cuda.Stream(device=device)
    return _comm_streams[key]


class KVGather:
    """An all-gather of per-token rows in flight.  `full` (B, T*C, heads, D) fills in two halves;
    `wait(i)` makes the current stream wait until halves 0..i have landed (a no-op on CPU, where the
    gather has completed by the time `start_kv_gather` returns)."""

    def __init__(self, full: torch.Tensor, events: list):
        self.full = full
        self._events = events

    def wait(self, half: int = 1) -> torch.Tensor:
        for ev in self._events[:half + 1]:
            if ev is not None:
                torch.cuda.current_stream(self.full.device).wait_event(ev)
        return self.full


def _gather_half(full: torch.Tensor, mine: Optional[torch.Tensor], plan, half: int, C: int, rank: int,
                 world: int, group) -> None:
    """Brings every rank's chunk `half` into its place in `full`.  All ranks call this with the same
    plan, so all of them take the same branch (the collectives match) whether or not they own rows."""
    B, _, Hh, D = full.shape
    spans = [(plan[r][half][0] * C, plan[r][half][1] * C) for r in range(world)]
    sizes = [n for _, n in spans]
    width = max(sizes)
    if width == 0:
        return
    views = [full[:, t0:t0 + n] for t0, n in spans]
    if min(sizes) == width and B == 1:
        if half == 0:
            # chunks 0..R-1 are adjacent and in rank order: NCCL writes them in place, no staging at all
            lo = spans[0][0]
            dist.all_gather_into_tensor(full[0, lo:lo + world * width], mine[0], group=group)
        else:
            # chunks 2R-1-r: rank order is the reverse of memory order; torch gathers into a flat
            # temporary and copies each part to its view (all on the communication stream)
            dist.all_gather(views, mine, group=group)
        return
    # ragged chunks or a batch dimension in the way: pad to the widest chunk, gather, copy the valid rows
    padded = torch.zeros((B, width, Hh, D), dtype=full.dtype, device=full.device)
    if sizes[rank]:
        padded[:, :sizes[rank]] = mine
    parts = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(parts, padded, group=group)
    for r in range(world):
        if sizes[r]:
            views[r].copy_(parts[r][:, :sizes[r]])


def start_kv_gather(local: Sequence[Optional[torch.Tensor]], plan: List[List[Tuple[int, int]]], T: int, C: int,
                    heads: int, dim: int, dtype: torch.dtype, device: torch.device, batch: int = 1,
                    group=None) -> KVGather:
    """Starts the all-gather of one per-token tensor (K, V, or both fused along the head axis).
    `local[i]` holds this rank's rows of its i-th chunk, shaped (batch, n_i*C, heads, dim) (the layout the
    projection produces), or None when that chunk is empty.  Shapes come from the arguments, not from
    `local`, so a rank that owns nothing still takes part in every collective.  On a CUDA device the
    collectives and copies run on a communication stream and the call returns at once."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    full = torch.empty((batch, T * C, heads, dim), dtype=dtype, device=device)
    # Attention on the early chunk may start while the late half is still arriving.  It never uses those
    # rows (they are causally masked), but a kernel whose key tiles are not aligned to time steps may load
    # them next to rows it does use, and 0 x NaN is NaN: start the late half from zeros.
    full[:, plan[world - 1][1][0] * C:].zero_()
    if device.type != "cuda":
        for half in range(2):
            _gather_half(full, local[half], plan, half, C, rank, world, group)
        return KVGather(full, [None, None])
    comm = _comm_stream(device)
    comm.wait_stream(torch.cuda.current_stream(device))      # the local rows were produced on the current stream
    full.record_stream(comm)
    events = []
    with torch.cuda.stream(comm):
        for half in range(2):
            if local[half] is not None:
                local[half].record_stream(comm)
            _gather_half(full, local[half], plan, half, C, rank, world, group)
            ev = torch.cuda.Event()
            ev.record(comm)
            events.append(ev)
    return KVGather(full, events)


def gather_kv(local: Sequence[Optional[torch.Tensor]], plan: List[List[Tuple[int, int]]], T: int, C: int,
              heads: int, dim: int, dtype: torch.dtype, device: torch.device, batch: int = 1,
              group=None) -> torch.Tensor:
    """Blocking form of `start_kv_gather`: the whole sequence as (batch, T*C, heads, dim); the kernels read
    it as a strided (B, heads, N, D) view, no further copy."""
    return start_kv_gather(local, plan, T, C, heads, dim, dtype, device, batch, group).wait(1)


def time_sharded_attention(op: Callable, q_local: Sequence[Optional[torch.Tensor]], u, vt, z,
                           k_local: Sequence[Optional[torch.Tensor]], r_time, r_chan,
                           v_local: Optional[Sequence[Optional[torch.Tensor]]], T: int, C: int, sm_scale: float,
                           window: int = 10, group=None, batch: int = 1,
                           overlap: Optional[Callable[[], None]] = None) -> List[Optional[torch.Tensor]]:
    """Attention of one long sample whose time axis is spread over the ranks of `group`.

    `q_local[i]` (B, n_i*C, H, D), `k_local[i]`, `v_local[i]` (B, n_i*C, Hkv, D) are this rank's
    tokens of its two zig-zag chunks (`zigzag_chunks`), None for an empty chunk; `op` is
    `attentions.flashmvpa`.  With `v_local=None`, `k_local[i]` holds K and V fused along the head axis,
    (B, n_i*C, 2*Hkv, D), the way `c_attn` produces them: one collective per half instead of two.
    `overlap()`, if given, is called after the gathers have been started and before anything waits for
    them.  Returns this rank's outputs, one (B, n_i*C, H, D) tensor per chunk (None for an empty chunk).
    """
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    plan = zigzag_chunks(T, C, world)
    Hkv, D = r_time.shape[-3], r_time.shape[-1]
    common = dict(dim=D, dtype=r_time.dtype, device=r_time.device, batch=batch, group=group)
    if v_local is None:
        gk = gv = start_kv_gather(k_local, plan, T, C, heads=2 * Hkv, **common)
        k_of = lambda full: full[:, :, :Hkv].permute(0, 2, 1, 3)       # (B,Hkv,N,D) strided views
        v_of = lambda full: full[:, :, Hkv:].permute(0, 2, 1, 3)
    else:
        gk = start_kv_gather(k_local, plan, T, C, heads=Hkv, **common)
        gv = start_kv_gather(v_local, plan, T, C, heads=Hkv, **common)
        k_of = v_of = lambda full: full.permute(0, 2, 1, 3)
    if overlap is not None:
        overlap()
    outs: List[Optional[torch.Tensor]] = []
    for i, (t0, n) in enumerate(plan[rank]):
        # chunk 0 lies in the early half and is causal: it reads no key beyond that half
        k_full, v_full = k_of(gk.wait(i)), v_of(gv.wait(i))
        if n == 0:
            outs.append(None)
            continue
        q = q_local[i].permute(0, 2, 1, 3)                               # (B,H,n*C,D) strided view
        o = op(q, u, vt, z, k_full, r_time, r_chan, v_full, causal=True, sm_scale=sm_scale,
               window_size=window, q_time_range=(t0, n))
        outs.append(o.permute(0, 2, 1, 3))
    return outs
