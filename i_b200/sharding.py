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


class PeerGather:
    """All-gather of per-rank output shards by copy engines over NVLink.

    Every rank owns a symmetric buffer `[slots][world][*shape]`; rank r computes
    into `local(slot)` (= its own row of its own buffer) and `publish(slot)`
    queues one device-to-device copy per peer into row r of that peer's buffer.
    The copies are DMA transfers: they use no SM, so they run entirely under the
    next step's kernel, which a collective made of SM kernels cannot do while a
    persistent kernel holds every SM.  `finish()` waits for this rank's copies
    and then for everybody's (host barrier); after it every rank holds all rows.

    Needs torch symmetric memory (peer-mapped allocations); `available()` tells.
    """

    @staticmethod
    def available():
        try:
            import torch.distributed._symmetric_memory as symm  # noqa: F401
            return True
        except Exception:
            return False

    def __init__(self, shape, slots=2, group=None, device=None):
        import torch
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        full = (slots, self.world) + tuple(shape)
        self.buffer = symm.empty(full, dtype=torch.float32, device=device)
        self.handle = symm.rendezvous(self.buffer, self.group)
        self.peers = [self.buffer if r == self.rank else
                      self.handle.get_buffer(r, full, torch.float32) for r in range(self.world)]
        self.stream = torch.cuda.Stream(device=device)
        self._done = [None] * slots

    def local(self, slot):
        return self.buffer[slot, self.rank]

    def gathered(self, slot):
        return self.buffer[slot]

    def publish(self, slot, after):
        """Queue the copies of `local(slot)` to every peer once event `after` has fired."""
        import torch
        self.stream.wait_event(after)
        with torch.cuda.stream(self.stream):
            src = self.buffer[slot, self.rank]
            for step in range(1, self.world):
                peer = (self.rank + step) % self.world
                self.peers[peer][slot, self.rank].copy_(src, non_blocking=True)
            done = torch.cuda.Event()
            done.record(self.stream)
        self._done[slot] = done
        return done

    def reusable(self, slot):
        """Event after which `local(slot)` may be overwritten (its last copies have read it)."""
        return self._done[slot]

    def finish(self):
        import torch.distributed as dist
        self.stream.synchronize()
        dist.barrier(self.group)
