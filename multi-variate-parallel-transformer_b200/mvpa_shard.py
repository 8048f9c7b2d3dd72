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

   Two transports bring the rows over: NCCL collectives (`transport="nccl"`; `gloo` in the CPU tests),
   or this library's own kernels over NVLink (`transport="p2p"`, `PeerKV`): every rank keeps its rows in
   a send buffer that the other ranks of the node have mapped through CUDA IPC handles; a rank stores a
   step counter into every peer's flag area when its rows are written, the gather kernel of a rank starts
   once all counters have arrived (a bounded wait) and pulls all peers' pieces at once with plain peer
   loads, and a second set of counters says "read" before a send buffer may be overwritten.  No
   collective and no host synchronisation on the data path.
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
        # (a third event, where present, marks the end of the communication stream's work for the step; the
        # last wait takes it along so that the stream is joined again, as a CUDA graph capture requires)
        for ev in self._events[:half + 1] + (self._events[2:] if half >= 1 else []):
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


class PeerKV:
    """Send buffer and flags of one per-token tensor (K, V or both fused) for the peer-load transport, one
    per (shape, tag, group).  One device allocation per rank, mapped into every other rank's process through
    a CUDA IPC handle (all ranks on one node): this rank's rows of its two chunks (`send[i]`), then two
    arrays of 32-bit step counters that the PEERS write - `written[r]`: rank r's rows of step n are complete;
    `read[r]`: rank r has copied this rank's rows of step n - and a status word that a bounded wait sets
    when it runs out.  `peer[r][i]` is rank r's `send[i]`.  Built collectively by `PeerKV.get` on first
    use and kept; the mappings stay valid as long as the owners keep their buffers, which they do for the
    life of the process.  No collective runs on the data path: ordering between GPUs comes from the flags."""

    _cache = {}

    def __init__(self, plan, C: int, heads: int, dim: int, dtype, device, batch: int, group):
        from torch.multiprocessing.reductions import reduce_tensor
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        assert world <= 32, "at most 32 ranks (pieces per gather launch)"
        self.world, self.rank, self.group = world, rank, group
        self.rows = [[plan[r][i][1] * C for i in range(2)] for r in range(world)]
        item = torch.empty((), dtype=dtype).element_size()
        row_bytes = heads * dim * item
        nbytes = lambda r: -(-(batch * (self.rows[r][0] + self.rows[r][1]) * row_bytes) // 256) * 256
        self._all = torch.zeros(nbytes(rank) + 1024, dtype=torch.uint8, device=device)   # flags start at zero
        torch.cuda.synchronize(device)
        fn, args = reduce_tensor(self._all)                           # (rebuild function, arguments): picklable
        everyone = [None] * world
        dist.all_gather_object(everyone, (fn, args), group=group)     # (also: nobody signals before every rank has zeroed)

        def opened(r):
            if r == rank:
                return self._all
            fn_r, args_r = everyone[r]
            args_r = list(args_r)
            # The handle is opened with THIS rank's device current (argument 6 is the device the storage is
            # attributed to), which is what makes the driver set up peer access from this GPU to the owner's
            # memory; opened under the owner's index it would be mapped for that device's context instead.
            args_r[6] = device.index
            return fn_r(*args_r)

        # every rank learns whether every mapping worked, so that a failure raises on all of them instead of
        # leaving the others waiting
        try:
            whole, err = [opened(r) for r in range(world)], None
        except Exception as e:
            whole, err = None, repr(e)
        failed = [None] * world
        dist.all_gather_object(failed, err, group=group)
        if any(failed):
            raise RuntimeError(f"peer-load transport unavailable: {[f for f in failed if f][0]}")

        def rows_of(t, r):
            n0, n1 = self.rows[r]
            v = t[:batch * (n0 + n1) * row_bytes].view(dtype).view(batch * (n0 + n1), heads, dim)
            # chunk-major: all batch rows of chunk 0, then of chunk 1 (each piece of a gather is contiguous)
            return [v[:batch * n0].view(batch, n0, heads, dim), v[batch * n0:].view(batch, n1, heads, dim)]

        self._keep = whole
        self.send = rows_of(self._all, rank)
        self.peer = [rows_of(whole[r], r) for r in range(world)]
        base = [whole[r].data_ptr() + nbytes(r) for r in range(world)]           # flag area of rank r
        self._written_here = [base[rank] + 4 * r for r in range(world)]          # slots the peers write, polled locally
        self._read_here = [base[rank] + 256 + 4 * r for r in range(world)]
        self._written_there = [base[r] + 4 * rank for r in range(world)]         # this rank's slot in every rank's area
        self._read_there = [base[r] + 256 + 4 * rank for r in range(world)]
        self._status_ptr = base[rank] + 512
        self._status = self._all[nbytes(rank) + 512:nbytes(rank) + 516].view(torch.int32)
        self._pieces = {}                                             # argument arrays of the gather launches, per receive buffer
        # The step counter lives on the device (the flag kernels add it to the number they are given), so the
        # same launches serve every step and a CUDA graph can replay them.
        self._step = torch.zeros(1, dtype=torch.int32, device=device)
        self.joined, self.joined_capturing = None, False              # event: the communication stream is done with the step

    @classmethod
    def get(cls, plan, C, heads, dim, dtype, device, batch, group, tag=0):
        key = (tuple(tuple(tuple(c) for c in owned) for owned in plan), C, heads, dim, dtype, device.index, batch,
               id(group), tag)
        if key not in cls._cache:
            cls._cache[key] = cls(plan, C, heads, dim, dtype, device, batch, group)
        return cls._cache[key]

    @classmethod
    def forget_events(cls) -> None:
        """Drops the "communication stream is done" events of all buffers.  Called with every stream joined
        (before and after a CUDA graph capture): stream order alone then orders the next step."""
        for px in cls._cache.values():
            px.joined = None

    def _slots(self, ptrs):
        import ctypes
        return (ctypes.c_void_p * len(ptrs))(*ptrs), len(ptrs)

    def next_step(self) -> None:
        """Advances the step counter on the current stream (which has waited for the previous step's `joined`)."""
        self._step.add_(1)

    def signal(self, which: str, device) -> None:
        """Tells every rank (on the current stream, after everything enqueued before) that this rank's rows
        of the current step are written (`which="written"`) or that it has read theirs (`"read"`)."""
        import ctypes
        import mvpa_native as _nat
        arr, n = self._slots(self._written_there if which == "written" else self._read_there)
        _nat.check(_nat.lib().mvpa_peer_signal(arr, n, 0, ctypes.c_void_p(self._step.data_ptr()),
                                               ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)), "mvpa_peer_signal")

    def wait(self, which: str, back: int, device) -> None:
        """Holds the current stream until every rank has signalled `which` for the step `back` steps ago (at
        most two seconds: after that the status word is set and the stream goes on; `check()` reports it)."""
        import ctypes
        import mvpa_native as _nat
        arr, n = self._slots(self._written_here if which == "written" else self._read_here)
        _nat.check(_nat.lib().mvpa_peer_wait(arr, n, (-back) & 0xFFFFFFFF, ctypes.c_void_p(self._step.data_ptr()), 0,
                                             ctypes.c_void_p(self._status_ptr),
                                             ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)), "mvpa_peer_wait")

    def check(self) -> None:
        """Raises if a wait of this buffer has run out (synchronises)."""
        if int(self._status.item()) != 0:
            raise RuntimeError("peer-load transport: a wait for another rank's flag ran out")


def _peer_gather_half(full: torch.Tensor, px: "PeerKV", plan, half: int, C: int) -> None:
    """One launch of the library's gather kernel: every rank's chunk `half` into its place in `full`
    (the other ranks' rows through peer loads, this rank's own through the same kernel)."""
    import ctypes
    import mvpa_native as _nat
    key = (full.data_ptr(), half)
    calls = px._pieces.get(key)
    if calls is None:                                                # (the allocator hands the same buffer back step after step)
        B = full.shape[0]
        dst, src, nbytes = [], [], []
        for r in range(px.world):
            t0, n = plan[r][half][0] * C, px.rows[r][half]
            if n == 0:
                continue
            for b in range(B):                                        # a batch row of `full` is not contiguous with the next
                d, s_ = full[b, t0:t0 + n], px.peer[r][half][b]
                dst.append(d.data_ptr()); src.append(s_.data_ptr()); nbytes.append(d.numel() * d.element_size())
        calls = []
        for lo in range(0, len(dst), 32):
            k = len(dst[lo:lo + 32])
            calls.append(((ctypes.c_void_p * k)(*dst[lo:lo + 32]), (ctypes.c_void_p * k)(*src[lo:lo + 32]),
                          (ctypes.c_int64 * k)(*nbytes[lo:lo + 32]), k))
        if len(px._pieces) > 64:
            px._pieces.clear()
        px._pieces[key] = calls
    stream = ctypes.c_void_p(torch.cuda.current_stream(full.device).cuda_stream)
    for d_arr, s_arr, n_arr, k in calls:
        _nat.check(_nat.lib().mvpa_peer_gather(d_arr, s_arr, n_arr, k, stream), "mvpa_peer_gather")


def start_kv_gather(local: Sequence[Optional[torch.Tensor]], plan: List[List[Tuple[int, int]]], T: int, C: int,
                    heads: int, dim: int, dtype: torch.dtype, device: torch.device, batch: int = 1,
                    group=None, transport: str = "nccl", tag=0) -> KVGather:
    """Starts the all-gather of one per-token tensor (K, V, or both fused along the head axis).
    `local[i]` holds this rank's rows of its i-th chunk, shaped (batch, n_i*C, heads, dim) (the layout the
    projection produces), or None when that chunk is empty.  Shapes come from the arguments, not from
    `local`, so a rank that owns nothing still takes part in every collective.  On a CUDA device the
    collectives and copies run on a communication stream and the call returns at once.
    `transport="p2p"` (CUDA, all ranks on one node) uses the library's peer-load gather kernel instead of
    NCCL for the rows themselves (see `PeerKV`)."""
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
    if transport == "p2p":
        px = PeerKV.get(plan, C, heads, dim, dtype, device, batch, group, tag)   # `tag` keeps K's and V's buffers apart
        cur = torch.cuda.current_stream(device)
        capturing = torch.cuda.is_current_stream_capturing()
        if px.joined is not None and px.joined_capturing == capturing:
            # the communication stream has read the previous step's counter.  (An event recorded outside a graph
            # capture cannot be waited for inside one, nor the other way round; at those two boundaries the
            # previous step has been joined to the current stream already - `KVGather.wait(1)` - and plain stream
            # order does the rest.)
            cur.wait_event(px.joined)
        px.next_step()
        px.wait("read", 1, device)                           # the peers have copied the previous rows (step 0: nothing to wait for)
        for i in range(2):
            if local[i] is not None and local[i].data_ptr() != px.send[i].data_ptr():
                px.send[i].copy_(local[i])                   # (a caller may produce its rows in `send[i]` directly)
        px.signal("written", device)
        comm.wait_stream(cur)
        full.record_stream(comm)
        events = []
        with torch.cuda.stream(comm):
            px.wait("written", 0, device)                    # every rank's rows of this step are complete
            for half in range(2):
                _peer_gather_half(full, px, plan, half, C)
                ev = torch.cuda.Event()
                ev.record(comm)
                events.append(ev)
            px.signal("read", device)
            px.joined = torch.cuda.Event()
            px.joined.record(comm)
            px.joined_capturing = capturing
        events.append(px.joined)
        return KVGather(full, events)
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
              group=None, transport: str = "nccl") -> torch.Tensor:
    """Blocking form of `start_kv_gather`: the whole sequence as (batch, T*C, heads, dim); the kernels read
    it as a strided (B, heads, N, D) view, no further copy."""
    return start_kv_gather(local, plan, T, C, heads, dim, dtype, device, batch, group, transport).wait(1)


def time_sharded_attention(op: Callable, q_local: Sequence[Optional[torch.Tensor]], u, vt, z,
                           k_local: Sequence[Optional[torch.Tensor]], r_time, r_chan,
                           v_local: Optional[Sequence[Optional[torch.Tensor]]], T: int, C: int, sm_scale: float,
                           window: int = 10, group=None, batch: int = 1,
                           overlap: Optional[Callable[[], None]] = None,
                           transport: str = "nccl") -> List[Optional[torch.Tensor]]:
    """Attention of one long sample whose time axis is spread over the ranks of `group`.

    `q_local[i]` (B, n_i*C, H, D), `k_local[i]`, `v_local[i]` (B, n_i*C, Hkv, D) are this rank's
    tokens of its two zig-zag chunks (`zigzag_chunks`), None for an empty chunk; `op` is
    `attentions.flashmvpa`.  With `v_local=None`, `k_local[i]` holds K and V fused along the head axis,
    (B, n_i*C, 2*Hkv, D), the way `c_attn` produces them: one collective per half instead of two.
    `overlap()`, if given, is called after the gathers have been started and before anything waits for
    them.  `transport`: "nccl" (collectives) or "p2p" (this library's peer-load gather kernel, one node).
    Returns this rank's outputs, one (B, n_i*C, H, D) tensor per chunk (None for an empty chunk).
    """
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    plan = zigzag_chunks(T, C, world)
    Hkv, D = r_time.shape[-3], r_time.shape[-1]
    common = dict(dim=D, dtype=r_time.dtype, device=r_time.device, batch=batch, group=group, transport=transport)
    if v_local is None:
        gk = gv = start_kv_gather(k_local, plan, T, C, heads=2 * Hkv, **common)
        k_of = lambda full: full[:, :, :Hkv].permute(0, 2, 1, 3)       # (B,Hkv,N,D) strided views
        v_of = lambda full: full[:, :, Hkv:].permute(0, 2, 1, 3)
    else:
        gk = start_kv_gather(k_local, plan, T, C, heads=Hkv, tag="k", **common)
        gv = start_kv_gather(v_local, plan, T, C, heads=Hkv, tag="v", **common)
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
