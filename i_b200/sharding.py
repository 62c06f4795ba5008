"""Multi-GPU execution of independent attention units: one process per GPU.

The reference has no parallelism at all (single thread, single process).  What
shards here is what its kernel leaves independent: heads are separate
invocations, and within one head every query row touches only its own running
maximum, sum and output row (ilang-python/annotated-flashattn.c:92-127,
240-307), so a row slice of Q with the full K and V reproduces those rows of
the full result.  Each rank therefore computes

  * a contiguous block of heads when there are at least as many heads as ranks,
  * otherwise a contiguous block of query rows of every head, with K and V
    replicated,

and the outputs are assembled with one all-gather per call (NCCL over NVLink on
GPUs, gloo on CPU for the tests).  There is no other exchange on the data path.
"""
from dataclasses import dataclass


@dataclass(frozen=True)
class Shard:
    """What one rank computes: heads [head_lo, head_hi) x rows [row_lo, row_hi)."""
    head_lo: int
    head_hi: int
    row_lo: int
    row_hi: int
    by_heads: bool


def split_even(n, parts, index):
    """[lo, hi) of block `index` when n items are cut into `parts` contiguous blocks."""
    base, extra = divmod(n, parts)
    lo = index * base + min(index, extra)
    return lo, lo + base + (1 if index < extra else 0)


def plan_shard(n_heads, n_rows, world, rank, row_align=256):
    """Partition (heads, query rows) over `world` ranks.

    Heads are split when n_heads >= world.  Otherwise query rows are split in
    multiples of `row_align` (the kernel's query block), so no block straddles
    two ranks.
    """
    if world < 1 or not 0 <= rank < world:
        raise ValueError("bad world/rank")
    if n_heads >= world:
        lo, hi = split_even(n_heads, world, rank)
        return Shard(lo, hi, 0, n_rows, True)
    blocks = (n_rows + row_align - 1) // row_align
    lo, hi = split_even(blocks, world, rank)
    return Shard(0, n_heads, min(lo * row_align, n_rows), min(hi * row_align, n_rows), False)


def all_shards(n_heads, n_rows, world, row_align=256):
    return [plan_shard(n_heads, n_rows, world, r, row_align) for r in range(world)]


def sharded_attention(attend, q, k, v, group=None, out=None):
    """Run `attend(q_part, k_part, v_part) -> o_part` on this rank's shard and
    all-gather the result.

    q, k, v: torch tensors [heads, rows, d] / [heads, keys, d] / [heads, keys, dv]
    holding the *whole* problem on every rank (synthetic benchmarks and tests) —
    only the shard is read.  Returns the full [heads, rows, dv] output on every
    rank.  `attend` is any callable with the component's semantics (the compiled
    component's exec_torch on GPUs).
    """
    import torch
    import torch.distributed as dist

    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    heads, rows = q.shape[0], q.shape[1]
    shard = plan_shard(heads, rows, world, rank)
    qs = q[shard.head_lo:shard.head_hi, shard.row_lo:shard.row_hi]
    ks = k[shard.head_lo:shard.head_hi]
    vs = v[shard.head_lo:shard.head_hi]
    part = attend(qs.contiguous(), ks.contiguous(), vs.contiguous())
    dv = part.shape[-1]
    if out is None:
        out = torch.empty((heads, rows, dv), dtype=part.dtype, device=part.device)
    if world == 1:
        out.copy_(part)
        return out
    shards = all_shards(heads, rows, world)
    sizes = [(s.head_hi - s.head_lo) * (s.row_hi - s.row_lo) * dv for s in shards]
    if shard.by_heads and len(set(sizes)) == 1:
        # Equal contiguous head blocks land in place: one all-gather, no copies.
        dist.all_gather_into_tensor(out.view(-1), part.reshape(-1), group=group)
        return out
    # Uneven shards: pad every contribution to the largest, gather once, unpack.
    widest = max(sizes)
    send = torch.zeros(widest, dtype=part.dtype, device=part.device)
    send[: part.numel()] = part.reshape(-1)
    gathered = torch.empty(world * widest, dtype=part.dtype, device=part.device)
    dist.all_gather_into_tensor(gathered, send, group=group)
    for r, (s, n) in enumerate(zip(shards, sizes)):
        out[s.head_lo:s.head_hi, s.row_lo:s.row_hi] = gathered[r * widest: r * widest + n].view(
            s.head_hi - s.head_lo, s.row_hi - s.row_lo, dv)
    return out


def chunk_bounds(n, chunks):
    """Cuts n units into at most `chunks` contiguous, non-empty [lo, hi) blocks of near-equal size."""
    chunks = max(1, min(chunks, n))
    return [split_even(n, chunks, c) for c in range(chunks) if split_even(n, chunks, c)[1] >
            split_even(n, chunks, c)[0]]


def sharded_attention_chunked(attend_into, q, k, v, out, chunks=4, gather=None, slot=0, group=None,
                              local_inputs=False):
    """The head-sharded path with the assembly of the output overlapped with the computation.

    This rank's heads are computed `chunks` blocks at a time; as soon as a block is done its rows
    of the output travel to the other ranks while the next block is computed, so only the last
    block's transfer is exposed.  `attend_into(o_part, q_part, k_part, v_part)` writes one block.

      * with `gather` (a PeerGather whose shape is [heads per rank, rows, dv]): `out` is ignored,
        the result is `gather.gathered(slot)` viewed as [heads, rows, dv]; copies run on copy
        engines.  The caller ends a sequence of calls with `gather.finish()`.
      * without: every block is all-gathered through torch.distributed (NCCL on GPUs, gloo on CPU)
        into `out` ([heads, rows, dv], on every rank).

    q, k, v hold the whole problem on every rank ([heads, ...]; only this rank's heads are read)
    or, with `local_inputs`, just this rank's heads ([heads / world, ...]).  Heads must divide
    evenly over the ranks (the uneven and the row-sharded cases go through sharded_attention).
    Returns the assembled [heads, rows, dv] tensor.
    """
    import torch.distributed as dist

    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    heads = q.shape[0] * world if local_inputs else q.shape[0]
    if heads % world:
        raise ValueError("sharded_attention_chunked: %d heads do not divide over %d ranks" % (heads, world))
    per = heads // world
    lo = rank * per                  # this rank's first head in the assembled output
    src = 0 if local_inputs else lo  # and in q, k, v
    bounds = chunk_bounds(per, chunks)
    if gather is not None:
        import torch
        mine = gather.local(slot)
        main = torch.cuda.current_stream()
        for a, b in bounds:
            attend_into(mine[a:b], q[src + a:src + b], k[src + a:src + b], v[src + a:src + b])
            done = gather.block_event(slot, a)
            done.record(main)
            gather.publish(slot, done, a, b)
        return gather.gathered(slot).reshape((heads,) + tuple(mine.shape[1:]))
    side = None
    if world > 1 and out.is_cuda:
        import torch
        side = _side_stream(out.device)
        main = torch.cuda.current_stream()
    for a, b in bounds:
        attend_into(out[lo + a:lo + b], q[src + a:src + b], k[src + a:src + b], v[src + a:src + b])
        if world == 1:
            continue
        # Block [a, b) of every rank: gathered into a staging tensor [world, b - a, rows, dv], then
        # placed (the blocks of one rank are not adjacent to the next rank's in `out`).  On GPUs the
        # collective runs on a side stream, under the computation of the next block.
        part = out[lo + a:lo + b]
        if side is not None:
            ready = torch.cuda.Event()
            ready.record(main)
            side.wait_event(ready)
            torch.cuda.set_stream(side)
        try:
            staged = part.new_empty((world,) + tuple(part.shape))
            dist.all_gather_into_tensor(staged.view(-1), part.reshape(-1), group=group)
            for r in range(world):
                if r != rank:
                    out[r * per + a:r * per + b] = staged[r]
        finally:
            if side is not None:
                torch.cuda.set_stream(main)
    if side is not None:
        main.wait_stream(side)
    return out


_SIDE_STREAMS = {}


def _side_stream(device):
    import torch
    key = (device.type, device.index)
    if key not in _SIDE_STREAMS:
        _SIDE_STREAMS[key] = torch.cuda.Stream(device=device)
    return _SIDE_STREAMS[key]


class PeerGather:
    """All-gather of per-rank output shards by copy engines over NVLink.

    Every rank owns a symmetric buffer `[slots][world][*shape]`; rank r computes
    into `local(slot)` (= its own row of its own buffer) and `publish(slot)`
    queues one device-to-device copy per peer into row r of that peer's buffer
    (one call into the library, ib_peer_publish: wait for the producer's event,
    the copies, the completion event).  The copies are DMA transfers: they use no
    SM, so they run entirely under the next kernel, which a collective made of SM
    kernels cannot do while a persistent kernel holds every SM.  `finish()` waits
    for this rank's copies and then for everybody's (host barrier); after it every
    rank holds all rows.

    Needs torch symmetric memory (peer-mapped allocations); `available()` tells.
    """

    @staticmethod
    def available():
        try:
            import torch.distributed._symmetric_memory as symm  # noqa: F401
            return True
        except Exception:
            return False

    def __init__(self, shape, slots=2, group=None, device=None, streams=4):
        import ctypes
        import torch
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm
        from . import ilang
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        full = (slots, self.world) + tuple(shape)
        self.buffer = symm.empty(full, dtype=torch.float32, device=device)
        self.handle = symm.rendezvous(self.buffer, self.group)
        self.peers = [self.buffer if r == self.rank else
                      self.handle.get_buffer(r, full, torch.float32) for r in range(self.world)]
        # Copies to different peers go out on several streams, so that more than one copy engine
        # works on them: on one stream the seven 8 MiB copies of an 8-GPU step ran one after the
        # other at ~350 GB/s, which bound the step.
        self.streams = [torch.cuda.Stream(device=device) for _ in range(max(1, min(streams, self.world - 1)))]
        self.stream = self.streams[0]
        self._done = [None] * slots
        # Byte geometry for the library call: one unit is one rank's row of one slot; a block of
        # it is addressed by its offset along the unit's leading axis.
        self._unit_bytes = 4
        for n in shape:
            self._unit_bytes *= n
        self._lead = shape[0] if shape else 1
        self._lead_bytes = self._unit_bytes // max(1, self._lead)
        self._base = [t.data_ptr() for t in self.peers]
        order = [(self.rank + step) % self.world for step in range(1, self.world)]
        self._groups = [order[g::len(self.streams)] for g in range(len(self.streams))]
        self._dsts = [(ctypes.c_void_p * max(1, len(g)))() for g in self._groups]
        self._lib = ilang.core()
        self._lib.ib_peer_publish.restype = ctypes.c_int
        self._lib.ib_peer_publish.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_void_p), ctypes.c_int,
                                              ctypes.c_size_t, ctypes.c_void_p, ctypes.c_void_p,
                                              ctypes.c_void_p]
        # Completion events, created up front (an event's handle exists once it has been recorded).
        self._events = {}
        self._block_events = {}

    def _event(self, table, key, stream):
        import torch
        ev = table.get(key)
        if ev is None:
            ev = torch.cuda.Event()
            ev.record(stream)
            table[key] = ev
        return ev

    def block_event(self, slot, block):
        """A reusable event for the producer of block `block` of `slot` to record."""
        import torch
        return self._event(self._block_events, (slot, block), torch.cuda.current_stream())

    def local(self, slot):
        return self.buffer[slot, self.rank]

    def gathered(self, slot):
        return self.buffer[slot]

    def publish(self, slot, after, lo=None, hi=None):
        """Queue the copies of `local(slot)` (entries [lo, hi) of its leading axis; all of it when
        omitted) to every peer once event `after` has fired.  Returns the events recorded behind
        them, one per copy stream."""
        lo = 0 if lo is None else lo
        hi = self._lead if hi is None else hi
        offset = (slot * self.world + self.rank) * self._unit_bytes + lo * self._lead_bytes
        done = []
        for g, (peers, dsts, stream) in enumerate(zip(self._groups, self._dsts, self.streams)):
            for n, peer in enumerate(peers):
                dsts[n] = self._base[peer] + offset
            event = self._event(self._events, (slot, lo, g), stream)
            rc = self._lib.ib_peer_publish(self._base[self.rank] + offset, dsts, len(peers),
                                           (hi - lo) * self._lead_bytes, after.cuda_event, event.cuda_event,
                                           stream.cuda_stream)
            if rc != 0:
                err = self._lib.i_error()
                raise RuntimeError(err.decode() if err else "ib_peer_publish failed")
            done.append(event)
        self._done[slot] = done
        return done

    def wait_on(self, stream, events):
        """Make `stream` wait for the events a publish returned (None: nothing to wait for)."""
        for event in events or ():
            stream.wait_event(event)

    def join(self, stream):
        """Make `stream` wait for everything queued on the copy streams so far."""
        for s in self.streams:
            stream.wait_stream(s)

    def reusable(self, slot):
        """Events after which `local(slot)` may be overwritten (its last copies have read it)."""
        return self._done[slot]

    def finish(self):
        import torch.distributed as dist
        for s in self.streams:
            s.synchronize()
        dist.barrier(self.group)
