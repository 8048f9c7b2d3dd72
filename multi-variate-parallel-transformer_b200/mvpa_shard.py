"""Multi-GPU partitioning of the MVPA operator (one process per GPU, `torch.distributed`).

Two ways the path shards (no counterpart in the reference, whose only parallelism is Lightning
DDP, `configs/*.yaml:3-6`):

1. Independent units.  Every (batch element, kv-head group) is independent, so a job splits its
   batch (or its heads) across ranks and calls `attentions.flashmvpa` unchanged; no collective on
   the data path.  `batch_slice` gives a rank its share.

2. One long sample across ranks.  Queries are split by time blocks; each rank projects K/V for its
   own tokens, all ranks `all_gather` K and V into local HBM (NCCL over NVLink; `gloo` in the CPU
   tests), and each rank runs the kernel on its own query rows against the whole K/V
   (`q_time_range`).  Causality makes late time blocks more expensive than early ones, so the
   time axis is cut into 2R chunks and rank r owns chunks r and 2R-1-r ("zig-zag"), which
   balances the causal work to within one chunk.
"""
from __future__ import annotations

from typing import Callable, List, Sequence, Tuple

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


def gather_kv(local: Sequence[torch.Tensor], plan: List[List[Tuple[int, int]]], T: int, C: int,
              group=None) -> torch.Tensor:
    """All-gather one of K / V.  `local[i]` holds this rank's tokens of its i-th chunk, shaped
    (B, n_i*C, Hkv, D) (the layout the projection produces).  Returns the whole sequence as
    (B, T*C, Hkv, D); the kernels read it as a strided (B, Hkv, N, D) view, no further copy."""
    world = dist.get_world_size(group)
    ref = next(x for x in local if x is not None)
    B, _, Hkv, D = ref.shape
    full = torch.empty((B, T * C, Hkv, D), dtype=ref.dtype, device=ref.device)
    for i in range(2):
        sizes = [plan[r][i][1] * C for r in range(world)]
        width = max(sizes)
        if width == 0:
            continue
        mine = torch.zeros((B, width, Hkv, D), dtype=ref.dtype, device=ref.device)
        n_mine = plan[dist.get_rank(group)][i][1] * C
        if n_mine:
            mine[:, :n_mine] = local[i]
        parts = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(parts, mine, group=group)
        for r in range(world):
            t0, n = plan[r][i]
            if n:
                full[:, t0 * C:(t0 + n) * C] = parts[r][:, :n * C]
    return full


def time_sharded_attention(op: Callable, q_local: Sequence[torch.Tensor], u, vt, z,
                           k_local: Sequence[torch.Tensor], r_time, r_chan,
                           v_local: Sequence[torch.Tensor], T: int, C: int, sm_scale: float,
                           window: int = 10, group=None) -> List[torch.Tensor]:
    """Attention of one long sample whose time axis is spread over the ranks of `group`.

    `q_local[i]` (B, n_i*C, H, D), `k_local[i]`, `v_local[i]` (B, n_i*C, Hkv, D) are this rank's
    tokens of its two zig-zag chunks (`zigzag_chunks`); `op` is `attentions.flashmvpa`.
    Returns this rank's outputs, one (B, n_i*C, H, D) tensor per chunk (None for an empty chunk).
    """
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    plan = zigzag_chunks(T, C, world)
    k_full = gather_kv(k_local, plan, T, C, group).permute(0, 2, 1, 3)  # (B,Hkv,N,D) strided view
    v_full = gather_kv(v_local, plan, T, C, group).permute(0, 2, 1, 3)
    outs: List[torch.Tensor] = []
    for i, (t0, n) in enumerate(plan[rank]):
        if n == 0:
            outs.append(None)
            continue
        q = q_local[i].permute(0, 2, 1, 3)                               # (B,H,n*C,D) strided view
        o = op(q, u, vt, z, k_full, r_time, r_chan, v_full, causal=True, sm_scale=sm_scale,
               window_size=window, q_time_range=(t0, n))
        outs.append(o.permute(0, 2, 1, 3))
    return outs
