"""llsa_l2 / llsa_l1 with the SEQUENCE sharded over ranks (long sequences, B*H smaller than the GPU count).

Rank r owns the contiguous token range [r*N/W, (r+1)*N/W) of q, k and v (N/W a multiple of
block_size**2, so pooled blocks never straddle ranks).  Per call:

  forward   1. pool the local q, k, v ranges (the pooled pyramid of a range is the range of the
               pooled pyramid: mean_pool.py:26-31 pools disjoint windows);
            2. all-gather k, v and their pooled levels along the sequence -- the one exchange the
               forward needs: fine blocks and pooled keys may be selected anywhere;
            3. selection, index transpose and attention run on LOCAL query rows against the
               full-length keys (rectangular: Nq = N/W query rows, N keys), all in local memory.
  backward  dq is local.  dk, dv (with the pooling backward folded in) are sums over every rank's
            queries: each rank produces a full-length partial and a reduce-scatter along the
            sequence leaves every rank with the gradient of its own k, v range.

The arithmetic per query row is exactly the unsharded operator's, so o and dq are bit-identical to
it; dk and dv differ only by the summation order of the reduce-scatter.

`backend` supplies the stage functions; the default is this package's CUDA kernels.  Tests on CPU
pass a backend built from their checker to exercise the exchange logic with the gloo backend.
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist

__all__ = ["llsa_l2_seq_parallel", "llsa_l1_seq_parallel", "CudaBackend", "gather_seq", "reduce_scatter_seq", "local_forward",
           "head_groups", "make_head_group"]


_PER_SLICE_MAX = 16     # up to this many (b,h) slices the exchange runs per slice, straight into / out of place


def head_groups(n_slices: int, world: int) -> int:
    """How many groups the ranks are cut into when a problem of n_slices (batch, head) slices is spread over `world`
    ranks: the (b,h) slices are split over the groups first (no communication between groups: every stage of the
    operator is independent per slice), and only inside a group is the SEQUENCE sharded.  The largest divisor of `world`
    that also divides n_slices: 6 slices on 8 ranks -> 2 groups of 4 ranks with 3 slices each, so a rank exchanges k, v
    and dk, dv of three heads with three peers instead of six heads with seven."""
    g = 1
    for d in range(1, world + 1):
        if world % d == 0 and n_slices % d == 0:
            g = d
    return g


def make_head_group(n_slices: int, world: Optional[int] = None, rank: Optional[int] = None):
    """(group index, ranks per group, rank inside its group, process group of this rank's group).  Every rank of the
    default group must call this (torch.distributed.new_group is collective)."""
    world = dist.get_world_size() if world is None else world
    rank = dist.get_rank() if rank is None else rank
    g = head_groups(n_slices, world)
    rpg = world // g
    mine = None
    for i in range(g):
        ranks = list(range(i * rpg, (i + 1) * rpg))
        pg = dist.new_group(ranks) if rpg > 1 else None
        if rank in ranks:
            mine = pg
    return rank // rpg, rpg, rank % rpg, mine


_ALONE = "alone"        # group argument of a rank that shares its slices' sequence with nobody: no exchange at all


def _group_size(group) -> int:
    return 1 if group is _ALONE else dist.get_world_size(group)


def gather_seq_start(x: torch.Tensor, group=None):
    """Starts the all-gather of [B,H,n_local,D] along dim 2 and returns a handle for gather_seq_finish: the collectives run on
    the communicator's own stream, so kernels enqueued before the finish overlap with them."""
    world = _group_size(group)
    if world == 1:
        return x, [], None
    x = x.contiguous()
    B, H, n, D = x.shape
    if B * H <= _PER_SLICE_MAX:
        # a slice's full sequence [W*n, D] is the rank-major concatenation of the ranks' [n, D]: gather in place
        out = x.new_empty((B, H, world * n, D))
        works = [dist.all_gather_into_tensor(out[b, h], x[b, h], group=group, async_op=True) for b in range(B) for h in range(H)]
        return out, works, None
    out = x.new_empty((world * B, H, n, D))           # rank-major concatenation along dim 0, then one transposing copy
    work = dist.all_gather_into_tensor(out, x, group=group, async_op=True)
    return out, [work], (world, B, H, n, D)


def gather_seq_finish(handle) -> torch.Tensor:
    out, works, shape = handle
    for w in works:
        w.wait()
    if shape is None:
        return out
    world, B, H, n, D = shape
    return out.view(world, B, H, n, D).permute(1, 2, 0, 3, 4).reshape(B, H, world * n, D)


def gather_seq(x: torch.Tensor, group=None) -> torch.Tensor:
    """[B,H,n_local,D] on every rank -> [B,H,W*n_local,D], ranks in order along dim 2."""
    return gather_seq_finish(gather_seq_start(x, group))


def reduce_scatter_seq(x: torch.Tensor, group=None) -> torch.Tensor:
    """Full-length partial sums [B,H,W*n_local,D] on every rank -> this rank's [B,H,n_local,D] of the total."""
    world = _group_size(group)
    if world == 1:
        return x
    B, H, N, D = x.shape
    n = N // world
    out = x.new_empty((B, H, n, D))
    gloo = dist.get_backend(group) == "gloo"          # gloo has no reduce_scatter: all-reduce and keep the own part
    if B * H <= _PER_SLICE_MAX and not gloo:
        x = x.contiguous()
        works = [dist.reduce_scatter_tensor(out[b, h], x[b, h], group=group, async_op=True) for b in range(B) for h in range(H)]
        for w in works:
            w.wait()
        return out
    parts = x.reshape(B, H, world, n, D).permute(2, 0, 1, 3, 4).contiguous()
    if gloo:
        dist.all_reduce(parts, group=group)
        out.copy_(parts[dist.get_rank(group)])
    else:
        dist.reduce_scatter_tensor(out, parts, group=group)
    return out


class CudaBackend:
    """The stage functions of llsa_b200.ops (sm_100a kernels through the C ABI)."""

    def pool_pyramid(self, xs: List[torch.Tensor], block_size: int, levels: int):
        from . import ops
        return ops.pool_pyramid(xs, block_size, levels)

    def coarse_topk(self, pq, pk, topk):
        from . import ops
        return ops._coarse_topk(pq, pk, topk)

    def refine_topk(self, pq, pk, p_indices, topk, p_topk, block_size):
        from . import ops
        return ops._refine_topk(pq, pk, p_indices, topk, p_topk, block_size)

    def attn_fwd(self, q, k, v, pk, pv, pk2, pv2, indices, p_indices, topk, topk_p, block_size, w1, w2):
        from . import ops
        return ops._attn_fwd(q, k, v, pk, pv, pk2, pv2, indices, p_indices, topk, topk_p, block_size, w1, w2)

    def attn_bwd_folded(self, do, q, k, v, pk, pv, pk2, pv2, o, lse, indices, p_indices, topk, topk_p, block_size, w1, w2, kvw1, kvw2):
        """dq [like q], dk, dv [like k] with the pooled-key gradients folded through the pooling backward."""
        from . import ops
        dq, dk, dv = ops._attn_bwd(do, q, k, v, pk, pv, pk2, pv2, o, lse, indices, p_indices, topk, topk_p, block_size, w1, w2, kvw1, kvw2, True)[:3]
        return dq, dk, dv


def local_select(backend, pq_levels, pk, pk2, topk1, topk2, block_size):
    """Block selection of LOCAL query rows (pooled levels pq_levels) against the full-length pooled keys.
    Returns (indices, p_indices, w1, w2, topk_p)."""
    bs = block_size
    if pk2 is not None:
        p_indices = backend.coarse_topk(pq_levels[1], pk2, topk2)
        indices = backend.refine_topk(pq_levels[0], pk, p_indices, topk1, p_indices.shape[-1], bs)
        return indices, p_indices, float(bs), float(bs * bs), p_indices.shape[-1]
    return backend.coarse_topk(pq_levels[0], pk, topk1), None, float(bs), 1.0, 0


def local_forward(backend, q, kf, vf, pq_levels, pk, pv, pk2, pv2, topk1, topk2, block_size):
    """Selection and attention of LOCAL query rows q [B,H,Nq,D] (pooled levels pq_levels) against the
    full-length keys kf, vf and their pooled levels.  Returns (o, lse, indices, p_indices, w1, w2)."""
    indices, p_indices, w1, w2, topk_p = local_select(backend, pq_levels, pk, pk2, topk1, topk2, block_size)
    o, lse = backend.attn_fwd(q, kf, vf, pk, pv, pk2, pv2, indices, p_indices, indices.shape[-1], topk_p, block_size, w1, w2)
    return o, lse, indices, p_indices, w1, w2


def _mark(name):
    from . import ops
    ops._mark(name)


class _SeqParallel(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, topk1, topk2, block_size, levels, group, backend):
        bs = block_size
        if q.shape[2] % (bs * bs):
            raise ValueError("the local sequence length %d must be a multiple of block_size**2" % q.shape[2])
        pyr = backend.pool_pyramid([q.detach(), k.detach(), v.detach()], bs, levels)
        _mark("all_gather")
        # the pooled levels go first (the selection needs only them); k and v follow on the communicator's stream while the
        # selection kernels run, and are waited for right before the attention kernel
        small = [gather_seq_start(t, group) for t in ([pyr[0][1], pyr[0][2]] + ([pyr[1][1], pyr[1][2]] if levels == 2 else []))]
        big = [gather_seq_start(k.detach(), group), gather_seq_start(v.detach(), group)]
        pk, pv = gather_seq_finish(small[0]), gather_seq_finish(small[1])
        pk2, pv2 = (gather_seq_finish(small[2]), gather_seq_finish(small[3])) if levels == 2 else (None, None)
        indices, p_indices, w1, w2, topk_p = local_select(backend, [lv[0] for lv in pyr[:levels]], pk, pk2, topk1, topk2, bs)
        _mark("all_gather_wait")
        kf, vf = gather_seq_finish(big[0]), gather_seq_finish(big[1])
        o, lse = backend.attn_fwd(q.detach(), kf, vf, pk, pv, pk2, pv2, indices, p_indices, indices.shape[-1], topk_p, bs, w1, w2)
        ctx.save_for_backward(q, kf, vf, o, lse, indices, pk, pv, *([p_indices, pk2, pv2] if levels == 2 else []))
        ctx.cfg = (bs, w1, w2, levels, group, backend)
        return o

    @staticmethod
    def backward(ctx, do):
        bs, w1, w2, levels, group, backend = ctx.cfg
        q, kf, vf, o, lse, indices, pk, pv = ctx.saved_tensors[:8]
        p_indices, pk2, pv2 = ctx.saved_tensors[8:] if levels == 2 else (None, None, None)
        # one level: the reference's pooled dK/dV omit the token weight (sparse_attention_res_1.py:389)
        from . import ops
        kvw1 = w1 if (levels == 2 or ops._exact_pooled_grad) else 1.0
        topk_p = p_indices.shape[-1] if levels == 2 else 0
        dq, dk, dv = backend.attn_bwd_folded(do, q, kf, vf, pk, pv, pk2, pv2, o, lse, indices, p_indices, indices.shape[-1], topk_p, bs,
                                             w1, w2, kvw1, w2)
        _mark("reduce_scatter")
        dk, dv = reduce_scatter_seq(dk, group), reduce_scatter_seq(dv, group)
        _mark("end")
        return dq, dk, dv, None, None, None, None, None, None


def llsa_l2_seq_parallel(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, topk1: int = 8, topk2: int = 8, block_size: int = 16,
                         group: Optional[dist.ProcessGroup] = None, backend=None) -> torch.Tensor:
    """llsa_l2 (torch_op/flash_sparse_attention_res_2.py:48-59) on this rank's token range of q, k, v
    [B,H,N/W,D]; returns this rank's range of o.  Differentiable in q, k, v."""
    return _SeqParallel.apply(q, k, v, topk1, topk2, block_size, 2, group, backend or CudaBackend())


def llsa_l1_seq_parallel(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, topk: int = 8, block_size: int = 16,
                         group: Optional[dist.ProcessGroup] = None, backend=None) -> torch.Tensor:
    """llsa_l1 (torch_op/flash_sparse_attention_res_1.py:41-47) on this rank's token range."""
    return _SeqParallel.apply(q, k, v, topk, 0, block_size, 1, group, backend or CudaBackend())
