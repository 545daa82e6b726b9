"""Host logic of the multi-GPU path, on CPU: the (batch, head) partition and, with two
gloo ranks, that sharding + all-gather reproduces the unsharded result (the per-slice
operator is stood in for by the CPU oracle; no GPU is involved)."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from llsa_b200 import shard, synth

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("n,world", [(48, 1), (48, 2), (48, 8), (6, 4), (6, 8), (5, 8), (7, 3)])       # (6, 8): two ranks without a slice
def test_slice_ranges_tile_the_axis(n, world):
    ranges = [shard.slice_range(n, world, r) for r in range(world)]
    assert ranges[0][0] == 0 and ranges[-1][1] == n
    assert all(a[1] == b[0] for a, b in zip(ranges, ranges[1:]))
    sizes = [e - b for b, e in ranges]
    assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard.slice_range(n, world, world)


def test_take_slices_is_a_view_of_contiguous_input():
    x = torch.arange(2 * 3 * 4 * 8, dtype=torch.float32).reshape(2, 3, 4, 8)
    parts = [shard.take_slices(x, 4, r) for r in range(4)]
    assert [p.shape[1] for p in parts] == [2, 2, 1, 1]
    assert torch.equal(torch.cat(parts, 1).reshape(2, 3, 4, 8), x)
    assert parts[1].data_ptr() == x.reshape(1, 6, 4, 8)[:, 2:].data_ptr()


def _worker(rank, world, port, out):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import llsa_oracle as O
        torch.set_num_threads(2)
        q, k, v, _ = synth.gaussian_qkv(5, 1, 3, 1024, 64)
        fn = lambda a, b, c: O.llsa_l1_fwd_bwd(a, b, c)["o"]
        full = shard.sharded_call(fn, q, k, v)
        local = shard.sharded_call(fn, q, k, v, gather=False)
        if rank == 0:
            torch.save(dict(full=full, ref=fn(q, k, v), n_local=local.shape[1]), out)
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_reproduce_the_unsharded_result(tmp_path):
    out = str(tmp_path / "r0.pt")
    port = 29500 + os.getpid() % 2000
    mp.spawn(_worker, args=(2, port, out), nprocs=2, join=True)
    r = torch.load(out)
    assert r["n_local"] == 2                       # 3 slices over 2 ranks: 2 + 1
    assert torch.equal(r["full"], r["ref"])
