"""CPU tests of the multi-rank path: partition arithmetic and the all-gather
assembly, run as two gloo ranks.  The per-rank compute is a stand-in (the
float64 NumPy attention of the oracle) because no GPU is involved; what is under
test is that shards tile the problem exactly and land in the right place."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_split_even_tiles_exactly():
    from i_b200.sharding import split_even
    for n in (0, 1, 7, 64, 65):
        for parts in (1, 2, 3, 8):
            cuts = [split_even(n, parts, i) for i in range(parts)]
            assert cuts[0][0] == 0 and cuts[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(cuts, cuts[1:]))
            sizes = [hi - lo for lo, hi in cuts]
            assert max(sizes) - min(sizes) <= 1


@pytest.mark.parametrize("heads,rows,world", [(64, 32768, 8), (64, 32768, 1), (1, 16384, 8),
                                               (3, 1000, 2), (5, 300, 4), (1, 100, 4)])
def test_shards_cover_every_row_once(heads, rows, world):
    from i_b200.sharding import all_shards
    seen = np.zeros((heads, rows), dtype=int)
    for s in all_shards(heads, rows, world):
        seen[s.head_lo:s.head_hi, s.row_lo:s.row_hi] += 1
        if not s.by_heads and s.row_hi < rows:
            assert s.row_hi % 256 == 0
    assert np.all(seen == 1)


def _worker(rank, world, port, heads, rows, result_dir):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist
    import oracle
    from i_b200.sharding import sharded_attention
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    rng = np.random.default_rng(7)
    q = torch.from_numpy(rng.standard_normal((heads, rows, 16), dtype=np.float32))
    k = torch.from_numpy(rng.standard_normal((heads, 40, 16), dtype=np.float32))
    v = torch.from_numpy(rng.standard_normal((heads, 40, 8), dtype=np.float32))

    def attend(qs, ks, vs):
        out = [oracle.numpy_attention(a.numpy(), b.numpy(), c.numpy()) for a, b, c in zip(qs, ks, vs)]
        return torch.from_numpy(np.stack(out).astype(np.float32)) if out else torch.empty(
            (0, qs.shape[1], vs.shape[2]))

    full = sharded_attention(attend, q, k, v)
    ref = attend(q, k, v)
    ok = bool(torch.equal(full, ref))
    with open(os.path.join(result_dir, "rank%d" % rank), "w") as f:
        f.write("ok" if ok else "mismatch")
    dist.destroy_process_group()


@pytest.mark.parametrize("heads,rows", [(4, 64), (3, 64), (1, 600)])
def test_two_ranks_gather_the_full_output(tmp_path, heads, rows):
    import torch.multiprocessing as mp
    port = 29500 + (os.getpid() + heads * 7 + rows) % 2000
    mp.spawn(_worker, args=(2, port, heads, rows, str(tmp_path)), nprocs=2, join=True)
    for r in range(2):
        assert (tmp_path / ("rank%d" % r)).read_text() == "ok"


def test_chunk_bounds_cover_the_units_in_order():
    from i_b200.sharding import chunk_bounds
    for n in (1, 2, 7, 8, 64):
        for chunks in (1, 2, 3, 4, 100):
            cuts = chunk_bounds(n, chunks)
            assert cuts[0][0] == 0 and cuts[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(cuts, cuts[1:]))
            assert all(hi > lo for lo, hi in cuts) and len(cuts) == min(n, chunks)


def _chunked_worker(rank, world, port, heads, chunks, result_dir):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist
    import oracle
    from i_b200.sharding import sharded_attention_chunked
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    rng = np.random.default_rng(11)
    q = torch.from_numpy(rng.standard_normal((heads, 48, 16), dtype=np.float32))
    k = torch.from_numpy(rng.standard_normal((heads, 40, 16), dtype=np.float32))
    v = torch.from_numpy(rng.standard_normal((heads, 40, 8), dtype=np.float32))
    calls = []

    def attend_into(o, qs, ks, vs):
        calls.append(qs.shape[0])
        for h in range(qs.shape[0]):
            o[h] = torch.from_numpy(oracle.numpy_attention(qs[h].numpy(), ks[h].numpy(), vs[h].numpy())
                                    .astype(np.float32))

    out = torch.full((heads, 48, 8), float("nan"))
    full = sharded_attention_chunked(attend_into, q, k, v, out, chunks=chunks)
    ref = torch.empty_like(out)
    attend_into(ref, q, k, v)
    ok = bool(torch.equal(full, ref)) and sum(calls[:-1]) == heads // world
    with open(os.path.join(result_dir, "rank%d" % rank), "w") as f:
        f.write("ok %d" % (len(calls) - 1) if ok else "mismatch")
    dist.destroy_process_group()


@pytest.mark.parametrize("heads,chunks,blocks", [(8, 2, 2), (8, 4, 4), (6, 4, 3), (2, 4, 1)])
def test_two_ranks_assemble_the_output_block_by_block(tmp_path, heads, chunks, blocks):
    import torch.multiprocessing as mp
    port = 31500 + (os.getpid() + heads * 13 + chunks) % 2000
    mp.spawn(_chunked_worker, args=(2, port, heads, chunks, str(tmp_path)), nprocs=2, join=True)
    for r in range(2):
        assert (tmp_path / ("rank%d" % r)).read_text() == "ok %d" % blocks


def test_chunked_path_on_one_rank_needs_no_process_group():
    import torch
    from i_b200.sharding import sharded_attention_chunked
    import torch.distributed as dist
    assert not dist.is_initialized()
    q = torch.zeros(3, 4, 2)
    out = torch.zeros(3, 4, 2)
    sharded_attention_chunked(lambda o, a, b, c: o.zero_(), q, q, q, out, chunks=2)
    assert torch.count_nonzero(out) == 0
