"""CPU oracle for the LLSA hot path -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.

A plain PyTorch-eager (CPU) restatement of the reference algorithm
(SingleZombie/LLSA), one function per reference kernel group.  It is the
checker the CUDA path is compared against and the timed CPU baseline; nothing
in the shipped package imports it.

Parity pin: every function here is checked against the reference's own Triton
kernels executed under the Triton CPU interpreter (fp32) -- see
tests/golden/make_golden.py (generator) and tests/test_oracle_golden.py.  The
reference ships no golden vectors of its own.

All attention math is evaluated in fp32 on the given inputs.  `faithful=True`
additionally reproduces the roundings to the tensor dtype that the reference
kernels perform (q*scale, P before P@V, dS before dS@K, outputs).

Conventions: q, k, v are [B, H, N, D]; block b holds tokens 16b..16b+15; the
pooled pyramid is pk1 = pool16(k) [B,H,N/16,D], pk2 = pool16(pk1).
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

__all__ = [
    "mean_pool1d", "mean_pool1d_bwd", "gen_sparse_indices", "stable_topk",
    "compute_topk_indices_sparse", "transpose_indices",
    "attn_fwd_l1", "attn_bwd_l1", "attn_fwd_l2", "attn_bwd_l2",
    "llsa_l1_fwd_bwd", "llsa_l2_fwd_bwd", "llsa_dense_masked",
    "rope_table_2d", "rope_fwd", "rope_bwd", "morton_perm",
]


# ----------------------------------------------------------------------------
# pooling  (src/llsa/kernel/triton/mean_pool.py:6-58)
# ----------------------------------------------------------------------------
def mean_pool1d(x: torch.Tensor, k: int) -> torch.Tensor:
    """Mean over k consecutive tokens, accumulated SEQUENTIALLY IN x.dtype
    (mean_pool.py:26-30: `acc += load` with acc of the input element type, then
    `acc / K`).  Output is contiguous [B,H,S/k,C] (mean_pool.py:134-135)."""
    B, H, S, C = x.shape
    assert S % k == 0
    xv = x.reshape(B, H, S // k, k, C)
    acc = torch.zeros(B, H, S // k, C, dtype=x.dtype)
    for t in range(k):
        acc = acc + xv[:, :, :, t, :]          # each add rounds to x.dtype
    return (acc / k).contiguous()


def mean_pool1d_bwd(dy: torch.Tensor, k: int) -> torch.Tensor:
    """dx[s*k+t] = dy[s] / k  (mean_pool.py:54-58)."""
    return (dy / k).repeat_interleave(k, dim=2)


# ----------------------------------------------------------------------------
# selection  (src/llsa/kernel/triton/topk.py)
# ----------------------------------------------------------------------------
def stable_topk(score: torch.Tensor, topk: int) -> torch.Tensor:
    """Indices of the top-k along the last dim, descending score, ties broken
    by the SMALLEST index (the repo's own rule, topk.py:60-62 / :159-161;
    torch.topk leaves tie order unspecified)."""
    order = torch.sort(score.float(), dim=-1, descending=True, stable=True).indices
    return order[..., :topk].contiguous()


def gen_sparse_indices(pq: torch.Tensor, pk: torch.Tensor, topk: int) -> torch.Tensor:
    """Coarse selection (topk.py:6-9): score = pq @ pk^T with the OUTPUT IN THE
    INPUT DTYPE (fp32 accumulate, one rounding), top-k sorted descending, int64."""
    score = (pq.float() @ pk.float().transpose(-1, -2)).to(pq.dtype)
    topk = min(topk, score.shape[-1])
    return stable_topk(score, topk)


def compute_topk_indices_sparse(pq: torch.Tensor, pk: torch.Tensor, p_indices: torch.Tensor,
                                topk: int = 8, p_topk: int = 8, block_size: int = 16) -> torch.Tensor:
    """Refine selection (topk.py:102-197).  For level-2 query block P the
    candidates are the children `parent*bs + 0..bs-1` of its p_topk selected
    parents (:131-133); scores pq1[bs rows] . pk1[cand] in fp32, NOT rounded
    (:141-143); top-k per row by repeated arg-max, ties -> smallest block index
    (:155-164).  int32 [B,H,M,topk], sorted by descending score."""
    B, H, M, D = pq.shape
    bs = block_size
    n2 = M // bs
    cand = (p_indices.long()[..., :, None] * bs + torch.arange(bs)).reshape(B, H, n2, p_topk * bs)
    out = torch.empty(B, H, M, topk, dtype=torch.int32)
    pqf = pq.float().reshape(B, H, n2, bs, D)
    pkf = pk.float()
    for b in range(B):
        for h in range(H):
            kc = pkf[b, h][cand[b, h]]                                   # [n2, C, D]
            s = torch.einsum("pid,pcd->pic", pqf[b, h], kc)              # [n2, bs, C]
            c = cand[b, h][:, None, :].expand(n2, bs, -1)                # block index per candidate
            # sort by (score desc, block index asc): stable sort on index first, then on score
            o1 = torch.sort(c, dim=-1, stable=True).indices
            s1 = torch.gather(s, -1, o1)
            c1 = torch.gather(c, -1, o1)
            o2 = torch.sort(s1, dim=-1, descending=True, stable=True).indices[..., :topk]
            out[b, h] = torch.gather(c1, -1, o2).reshape(M, topk).to(torch.int32)
    return out


# ----------------------------------------------------------------------------
# index transpose  (src/llsa/kernel/triton/indices_transpose.py)
# ----------------------------------------------------------------------------
def transpose_indices(indices: torch.Tensor, k_ntx: Optional[int] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Query-major top-k lists -> KV-major CSR (indices_transpose.py:104-109).
    offsets[j] = #{(i,kk): idx[i,kk] < j} (int64, length M+1, :23-27 + cumsum :108);
    flat[offsets[j]:offsets[j+1]] = query blocks that selected j.  The reference
    fills buckets in atomic order (:73-78); the canonical form used for
    comparison -- and emitted here -- is ascending query block."""
    B, H, M, T = indices.shape
    if k_ntx is None:
        k_ntx = M
    idx = indices.long().reshape(B, H, M * T)
    qid = torch.arange(M).repeat_interleave(T)
    offsets = torch.zeros(B, H, k_ntx + 1, dtype=torch.int64)
    flat = torch.empty(B, H, M * T, dtype=torch.int64)
    for b in range(B):
        for h in range(H):
            cnt = torch.bincount(idx[b, h], minlength=k_ntx)
            offsets[b, h, 1:] = torch.cumsum(cnt, 0)
            order = torch.sort(idx[b, h], stable=True).indices        # stable => ascending q inside a bucket
            flat[b, h] = qid[order]
    return offsets, flat


# ----------------------------------------------------------------------------
# attention forward / backward, block-gather evaluation
# ----------------------------------------------------------------------------
def _rnd(x: torch.Tensor, dtype, faithful: bool) -> torch.Tensor:
    return x.to(dtype).float() if faithful and dtype != torch.float32 else x


def _gather_blocks(x: torch.Tensor, idx: torch.Tensor, bs: int) -> torch.Tensor:
    """x [n*bs, D], idx [m, t] block ids -> [m, t*bs, D]."""
    n = x.shape[0] // bs
    return x.reshape(n, bs, -1)[idx.long()].reshape(idx.shape[0], idx.shape[1] * bs, -1)


def _key_sets(q, k, v, pk, pv, pk2, pv2, indices, p_indices, bs, w1, w2):
    """For one (b,h): the attended keys/values grouped per level-2 query block.
    Returns lists of (K [G, nk, D], V [G, nk, D], log-weight, rows-per-group)."""
    N, D = q.shape                      # query rows; k / v / pk may be longer (q a shard of the sequence)
    n1 = pk.shape[0]
    sets = []
    # fine tokens of the selected blocks: per 16-row query block
    sets.append((_gather_blocks(k, indices, bs), _gather_blocks(v, indices, bs), 0.0, bs))
    if p_indices is None:
        # L1: ALL pooled keys (sparse_attention_res_1.py:85-106), dropped when fewer than 64 (:85)
        if n1 >= 64:
            sets.append((pk[None], pv[None], math.log(w1), N))
    else:
        # L2: level-1 pooled children of the PARENT's selected level-2 blocks
        # (sparse_attention_res_2.py:94-125), then all level-2 pooled keys (:127-149)
        sets.append((_gather_blocks(pk, p_indices, bs), _gather_blocks(pv, p_indices, bs), math.log(w1), bs * bs))
        if pk2.shape[0] >= 64:
            sets.append((pk2[None], pv2[None], math.log(w2), N))
    return sets


def _attn_fwd_one(q, sets, scale, dtype, faithful):
    N, D = q.shape
    qs = _rnd(q * scale, dtype, faithful)                     # `q *= scale` in q.dtype (res_1.py:48)
    logits = []
    for K, V, lw, rows in sets:
        s = torch.einsum("grd,gkd->grk", qs.reshape(-1, rows, D), K).reshape(N, -1)
        logits.append(s)
    m = torch.cat(logits, -1).max(-1, keepdim=True).values
    l = torch.zeros(N, 1)
    acc = torch.zeros(N, D)
    for (K, V, lw, rows), s in zip(sets, logits):
        e = torch.exp(s - m)
        w = math.exp(lw)
        l = l + e.sum(-1, keepdim=True) * w                   # l += l_ij * TOKEN_WEIGHT (:100-102)
        pe = _rnd(e, dtype, faithful)                         # exp_scores.to(v.dtype) before the dot (:82, :105)
        acc = acc + torch.einsum("grk,gkd->grd", pe.reshape(-1, rows, pe.shape[-1]), V).reshape(N, D) * w
    o = acc / l
    lse = (m + torch.log(l)).squeeze(-1)                      # M = m_i + log(l_i) (:116)
    return o, lse


def _attn_bwd_one(q, do, o, lse, sets, scale, dtype, faithful, kv_weights):
    """Reference backward (sparse_attention_res_1.py:225-400, res_2.py:287-575).
    k*scale is a separate tensor rounded to dtype (:420-422); p = w*exp(q.(k*scale) - m);
    dp = do.v; ds = p*(dp - delta); dq += ds.to(dtype) @ (k*scale);
    dv += p^T.to(dtype) @ do; dk += (ds^T.to(dtype) @ q) * scale.
    kv_weights[i] is the weight used on the dK/dV side of key set i (the L1
    reference omits TOKEN_WEIGHT there, res_1.py:389)."""
    N, D = q.shape
    delta = (o * do).sum(-1, keepdim=True)                    # _attn_bwd_preprocess
    dq = torch.zeros(N, D)
    grads = []
    for (K, V, lw, rows), wkv in zip(sets, kv_weights):
        G = K.shape[0]
        Ks = _rnd(K * scale, dtype, faithful)
        qg, dog = q.reshape(G, rows, D), do.reshape(G, rows, D)
        s = torch.einsum("grd,gkd->grk", qg, Ks)
        e = torch.exp(s - lse.reshape(G, rows, 1))
        dp = torch.einsum("grd,gkd->grk", dog, V)
        dlt = delta.reshape(G, rows, 1)
        wq = math.exp(lw)
        ds_q = _rnd(e * wq * (dp - dlt), dtype, faithful)
        dq = dq + torch.einsum("grk,gkd->grd", ds_q, Ks).reshape(N, D)
        p_kv = e * wkv
        ds_kv = _rnd(p_kv * (dp - dlt), dtype, faithful)
        dV = torch.einsum("grk,grd->gkd", _rnd(p_kv, dtype, faithful), dog)
        dK = torch.einsum("grk,grd->gkd", ds_kv, qg) * scale
        grads.append((dK, dV))
    return dq, grads


def _scatter_fine(dKg, idx, n1, bs, D):
    """Sum per-(query block, slot) gradients of gathered fine keys into [N, D]
    (what the reference does through the KV-major CSR, res_1.py:283-327)."""
    out = torch.zeros(n1, bs, D)
    m, t = idx.shape
    out.index_add_(0, idx.long().reshape(-1), dKg.reshape(m * t, bs, D))
    return out.reshape(n1 * bs, D)


def attn_fwd_l1(q, k, v, pk, pv, indices, topk=8, token_weight=16, block_size=16, faithful=True):
    """L1 forward (sparse_attention_res_1.py:9-150) -> (o in q.dtype, lse fp32 [B,H,N])."""
    return _attn_fwd(q, k, v, pk, pv, None, None, indices, None, block_size, token_weight, 1, faithful)


def attn_fwd_l2(q, k, v, pk, pv, pk2, pv2, indices, p_indices, topk=8, topk_p=8,
                token_weight=16, token_weight_2=256, block_size=16, faithful=True):
    """L2 forward (sparse_attention_res_2.py:9-199)."""
    return _attn_fwd(q, k, v, pk, pv, pk2, pv2, indices, p_indices, block_size,
                     token_weight, token_weight_2, faithful)


def _attn_fwd(q, k, v, pk, pv, pk2, pv2, indices, p_indices, bs, w1, w2, faithful):
    B, H, N, D = q.shape
    scale = 1.0 / math.sqrt(D)
    o = torch.empty(B, H, N, D, dtype=q.dtype)
    lse = torch.empty(B, H, N, dtype=torch.float32)
    for b in range(B):
        for h in range(H):
            sets = _key_sets(q[b, h].float(), k[b, h].float(), v[b, h].float(), pk[b, h].float(), pv[b, h].float(),
                             None if pk2 is None else pk2[b, h].float(), None if pv2 is None else pv2[b, h].float(),
                             indices[b, h], None if p_indices is None else p_indices[b, h], bs, w1, w2)
            ob, mb = _attn_fwd_one(q[b, h].float(), sets, scale, q.dtype, faithful)
            o[b, h] = ob.to(q.dtype)
            lse[b, h] = mb
    return o, lse


def attn_bwd_l1(do, q, k, v, pk, pv, o, lse, indices, topk=8, block_size=16, token_weight=16,
                exact_pooled_grad=False, faithful=True):
    """L1 backward (sparse_attention_res_1.py:403-471) -> dq, dk, dv, dpk, dpv
    (fp32, before the stores' cast to the tensor dtype).  With
    exact_pooled_grad=False the pooled-key gradients use weight 1 as the
    reference does (:389); True gives the mathematically exact gradient."""
    wkv = float(token_weight) if exact_pooled_grad else 1.0
    return _attn_bwd(do, q, k, v, pk, pv, None, None, o, lse, indices, None, block_size,
                     token_weight, 1, (1.0, wkv), faithful)


def attn_bwd_l2(do, q, k, v, pk, pv, pk2, pv2, o, lse, indices, p_indices, topk=8, topk_p=8,
                block_size=16, token_weight=16, token_weight_2=256, faithful=True):
    """L2 backward (sparse_attention_res_2.py:578-681) -> dq, dk, dv, dpk, dpv, dpk2, dpv2 (fp32)."""
    return _attn_bwd(do, q, k, v, pk, pv, pk2, pv2, o, lse, indices, p_indices, block_size,
                     token_weight, token_weight_2, (1.0, float(token_weight), float(token_weight_2)), faithful)


def _attn_bwd(do, q, k, v, pk, pv, pk2, pv2, o, lse, indices, p_indices, bs, w1, w2, kv_weights, faithful):
    B, H, N, D = q.shape
    nq1, n1 = N // bs, k.shape[2] // bs          # query-side / key-side block counts (equal in the reference)
    scale = 1.0 / math.sqrt(D)
    f = lambda t: torch.zeros(t.shape, dtype=torch.float32)
    dq, dk, dv, dpk, dpv = f(q), f(k), f(v), f(pk), f(pv)
    dpk2 = f(pk2) if pk2 is not None else None
    dpv2 = f(pv2) if pv2 is not None else None
    for b in range(B):
        for h in range(H):
            sets = _key_sets(q[b, h].float(), k[b, h].float(), v[b, h].float(), pk[b, h].float(), pv[b, h].float(),
                             None if pk2 is None else pk2[b, h].float(), None if pv2 is None else pv2[b, h].float(),
                             indices[b, h], None if p_indices is None else p_indices[b, h], bs, w1, w2)
            # the backward loops use 16-key chunks and never drop a short pooled tail
            # (res_1.py:261, res_2.py:348); with N >= 1024 (L1) / 16384 (L2) fwd and bwd agree.
            dqb, grads = _attn_bwd_one(q[b, h].float(), do[b, h].float(), o[b, h].float(), lse[b, h], sets,
                                       scale, q.dtype, faithful, kv_weights[:len(sets)])
            dq[b, h] = dqb
            dKf, dVf = grads[0]
            dk[b, h] = _scatter_fine(dKf.reshape(nq1, -1, bs, D), indices[b, h], n1, bs, D)
            dv[b, h] = _scatter_fine(dVf.reshape(nq1, -1, bs, D), indices[b, h], n1, bs, D)
            if p_indices is None:
                if len(grads) > 1:
                    dpk[b, h], dpv[b, h] = grads[1][0][0], grads[1][1][0]
            else:
                nq2, n2 = nq1 // bs, n1 // bs
                pi = p_indices[b, h]
                dpk[b, h] = _scatter_fine(grads[1][0].reshape(nq2, -1, bs, D), pi, n2, bs, D)
                dpv[b, h] = _scatter_fine(grads[1][1].reshape(nq2, -1, bs, D), pi, n2, bs, D)
                if len(grads) > 2:
                    dpk2[b, h], dpv2[b, h] = grads[2][0][0], grads[2][1][0]
    if p_indices is None:
        return dq, dk, dv, dpk, dpv
    return dq, dk, dv, dpk, dpv, dpk2, dpv2


# ----------------------------------------------------------------------------
# whole operator, forward + backward
# ----------------------------------------------------------------------------
def llsa_l1_fwd_bwd(q, k, v, do=None, topk=8, block_size=16, exact_pooled_grad=False, faithful=True):
    """llsa_l1 (torch_op/flash_sparse_attention_res_1.py:10-47) forward and, if
    `do` is given, the gradients autograd would leave in q/k/v.grad:
    dk_total = dk + up(dpk)/bs (mean_pool.py:150-165).  Returns a dict."""
    bs = block_size
    pq, pk, pv = mean_pool1d(q, bs), mean_pool1d(k, bs), mean_pool1d(v, bs)
    idx = gen_sparse_indices(pq, pk, topk)
    o, lse = attn_fwd_l1(q, k, v, pk, pv, idx, topk, bs, bs, faithful)
    out = dict(o=o, lse=lse, indices=idx, pq=pq, pk=pk, pv=pv)
    if do is not None:
        dq, dk, dv, dpk, dpv = attn_bwd_l1(do, q, k, v, pk, pv, o, lse, idx, topk, bs, bs,
                                           exact_pooled_grad, faithful)
        out.update(dq=dq, dk_fine=dk, dv_fine=dv, dpk=dpk, dpv=dpv,
                   dk=dk + mean_pool1d_bwd(dpk, bs), dv=dv + mean_pool1d_bwd(dpv, bs))
    return out


def llsa_l2_fwd_bwd(q, k, v, do=None, topk1=8, topk2=8, block_size=16, faithful=True):
    """llsa_l2 (torch_op/flash_sparse_attention_res_2.py:10-59), as above with two levels:
    dpk_total = dpk + up(dpk2)/bs, dk_total = dk + up(dpk_total)/bs."""
    bs = block_size
    pq, pk, pv = mean_pool1d(q, bs), mean_pool1d(k, bs), mean_pool1d(v, bs)
    pq2, pk2, pv2 = mean_pool1d(pq, bs), mean_pool1d(pk, bs), mean_pool1d(pv, bs)
    pidx = gen_sparse_indices(pq2, pk2, topk2)
    idx = compute_topk_indices_sparse(pq, pk, pidx, topk1, topk2, bs)
    o, lse = attn_fwd_l2(q, k, v, pk, pv, pk2, pv2, idx, pidx, topk1, topk2, bs, bs * bs, bs, faithful)
    out = dict(o=o, lse=lse, indices=idx, p_indices=pidx, pq=pq, pk=pk, pv=pv, pq2=pq2, pk2=pk2, pv2=pv2)
    if do is not None:
        dq, dk, dv, dpk, dpv, dpk2, dpv2 = attn_bwd_l2(do, q, k, v, pk, pv, pk2, pv2, o, lse, idx, pidx,
                                                       topk1, topk2, bs, bs, bs * bs, faithful)
        dpk_t = dpk + mean_pool1d_bwd(dpk2, bs)
        dpv_t = dpv + mean_pool1d_bwd(dpv2, bs)
        out.update(dq=dq, dk_fine=dk, dv_fine=dv, dpk=dpk, dpv=dpv, dpk2=dpk2, dpv2=dpv2,
                   dk=dk + mean_pool1d_bwd(dpk_t, bs), dv=dv + mean_pool1d_bwd(dpv_t, bs))
    return out


def llsa_dense_masked(q, k, v, indices, p_indices=None, block_size=16):
    """Tiny-N transparent form: a dense softmax over [tokens | pooled-1 | pooled-2]
    with -inf masks and +ln(weight) on pooled logits, differentiable by autograd
    (the mathematically exact gradient).  fp32/fp64 only; O(N^2) memory."""
    B, H, N, D = q.shape
    bs = block_size
    n1 = N // bs
    sc = 1.0 / math.sqrt(D)
    pool = lambda x: x.reshape(B, H, x.shape[2] // bs, bs, D).mean(3)
    pk1, pv1 = pool(k), pool(v)
    m1 = torch.zeros(B, H, n1, n1, dtype=torch.bool).scatter_(-1, indices.long(), True)
    fine = m1.repeat_interleave(bs, 2).repeat_interleave(bs, 3)
    s = (q @ k.transpose(-1, -2) * sc).masked_fill(~fine, float("-inf"))
    sp1 = q @ pk1.transpose(-1, -2) * sc + math.log(bs)
    if p_indices is None:
        if n1 < 64:
            sp1 = sp1[..., :0]
        a = torch.softmax(torch.cat([s, sp1], -1), -1)
        return a[..., :N] @ v + a[..., N:] @ pv1[..., :sp1.shape[-1], :]
    n2 = n1 // bs
    pk2, pv2 = pool(pk1), pool(pv1)
    m2 = torch.zeros(B, H, n2, n2, dtype=torch.bool).scatter_(-1, p_indices.long(), True)
    cand = m2.repeat_interleave(bs * bs, 2).repeat_interleave(bs, 3)       # [N, n1]
    sp1 = sp1.masked_fill(~cand, float("-inf"))
    sp2 = q @ pk2.transpose(-1, -2) * sc + math.log(bs * bs)
    if n2 < 64:
        sp2 = sp2[..., :0]
    a = torch.softmax(torch.cat([s, sp1, sp2], -1), -1)
    return a[..., :N] @ v + a[..., N:N + n1] @ pv1 + a[..., N + n1:] @ pv2[..., :sp2.shape[-1], :]


# ----------------------------------------------------------------------------
# RoPE  (src/llsa/kernel/triton/rope.py; tables: models/rope_dit_transformer_2d.py:71-109,153-173)
# ----------------------------------------------------------------------------
def morton_perm(side: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Quad-tree (Morton) token order of a side x side grid, closed form of
    gen_permuatations (rope_dit_transformer_2d.py:714-732): perm[r*side+c] is the
    bit interleave with column bits in even and row bits in odd positions;
    returns (perm, inv_perm) as the reference does."""
    bits = int(math.log2(side))
    r = torch.arange(side)[:, None].expand(side, side)
    c = torch.arange(side)[None, :].expand(side, side)
    code = torch.zeros(side, side, dtype=torch.long)
    for i in range(bits):
        code |= ((c >> i) & 1) << (2 * i)
        code |= ((r >> i) & 1) << (2 * i + 1)
    perm = code.flatten()
    inv = torch.empty_like(perm)
    inv[perm] = torch.arange(side * side)
    return perm, inv


def rope_table_2d(side: int, axes_dim=(32, 32), theta: float = 10000.0, perm: Optional[torch.Tensor] = None,
                  dtype=torch.float32) -> torch.Tensor:
    """[side*side, sum(axes_dim)] table: per axis, per frequency j the pair
    (sin, cos) of pos * theta^(-2j/dim) (rope :77-89, gen_rope_freq :71-74), row
    axis first then column axis (RopeEmbedding.forward :99-109), positions are
    integer pixel coordinates (register_rope_emb :153-166), optionally permuted
    (:168-170), built in fp64 then cast (:172-173)."""
    ids = torch.zeros(side, side, 2, dtype=torch.float64)
    ar = torch.arange(side, dtype=torch.float64)
    ids[..., 0] += ar[:, None]
    ids[..., 1] += ar[None, :]
    ids = ids.reshape(side * side, 2)
    if perm is not None:
        ids = ids[perm]
    parts = []
    for a, dim in enumerate(axes_dim):
        omega = 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.float64) / dim))
        ang = ids[:, a, None] * omega[None, :]
        parts.append(torch.stack([torch.sin(ang), torch.cos(ang)], -1).reshape(-1, dim))
    return torch.cat(parts, -1).to(dtype)


def rope_fwd(x: torch.Tensor, freq: torch.Tensor) -> torch.Tensor:
    """y_even = cos*x_even - sin*x_odd; y_odd = sin*x_even + cos*x_odd with
    sin = F[s,2c], cos = F[s,2c+1] (rope.py:28-50); each product and the
    subtraction/addition rounded to the tensor dtype."""
    sin, cos = freq[:, 0::2].to(x.dtype), freq[:, 1::2].to(x.dtype)
    xe, xo = x[..., 0::2], x[..., 1::2]
    y = torch.empty_like(x)
    y[..., 0::2] = cos * xe - sin * xo
    y[..., 1::2] = sin * xe + cos * xo
    return y


def rope_bwd(dy: torch.Tensor, freq: torch.Tensor) -> torch.Tensor:
    """dx_even = cos*dy_even + sin*dy_odd; dx_odd = -sin*dy_even + cos*dy_odd (rope.py:75-97)."""
    sin, cos = freq[:, 0::2].to(dy.dtype), freq[:, 1::2].to(dy.dtype)
    de, do_ = dy[..., 0::2], dy[..., 1::2]
    dx = torch.empty_like(dy)
    dx[..., 0::2] = cos * de + sin * do_
    dx[..., 1::2] = -sin * de + cos * do_
    return dx
