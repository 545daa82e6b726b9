"""Sequence-sharded llsa_l1 / llsa_l2 (llsa_b200/seqpar.py).

CPU: two gloo ranks, the stage functions stood in for by the CPU oracle -- checks the exchange
logic (all-gather of k, v and pooled levels; reduce-scatter of dk, dv) against the unsharded oracle.
GPU: the rectangular kernels (Nq query rows, N keys) on one device, rank by rank, against the
unsharded operator; and, where two GPUs are present, the real thing over NCCL.
"""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from llsa_b200 import seqpar, synth

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


class OracleBackend:
    """seqpar backend on the CPU oracle (fp32, faithful=False: plain fp32 evaluation)."""

    def __init__(self):
        from oracle import llsa_oracle as O
        self.O = O

    def pool_pyramid(self, xs, bs, levels):
        l1 = [self.O.mean_pool1d(x, bs) for x in xs]
        l2 = [self.O.mean_pool1d(x, bs) for x in l1] if levels == 2 else None
        return l1, l2

    def coarse_topk(self, pq, pk, topk):
        return self.O.gen_sparse_indices(pq, pk, min(topk, pk.shape[2]))

    def refine_topk(self, pq, pk, p_indices, topk, p_topk, bs):
        return self.O.compute_topk_indices_sparse(pq, pk, p_indices, topk, p_topk, bs)

    def attn_fwd(self, q, k, v, pk, pv, pk2, pv2, indices, p_indices, topk, topk_p, bs, w1, w2):
        return self.O._attn_fwd(q, k, v, pk, pv, pk2, pv2, indices, p_indices, bs, w1, w2, False)

    def attn_bwd_folded(self, do, q, k, v, pk, pv, pk2, pv2, o, lse, indices, p_indices, topk, topk_p, bs, w1, w2, kvw1, kvw2):
        O = self.O
        r = O._attn_bwd(do, q, k, v, pk, pv, pk2, pv2, o, lse, indices, p_indices, bs, w1, w2, [1.0, kvw1, kvw2], False)
        dq, dk, dv, dpk, dpv = r[:5]
        if pk2 is not None:
            dpk, dpv = dpk + O.mean_pool1d_bwd(r[5], bs), dpv + O.mean_pool1d_bwd(r[6], bs)
        return dq, dk + O.mean_pool1d_bwd(dpk, bs), dv + O.mean_pool1d_bwd(dpv, bs)


def _gloo_worker(rank, world, port, out, levels):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import llsa_oracle as O
        torch.set_num_threads(2)
        N = 16384 if levels == 2 else 2048
        q, k, v, do = synth.gaussian_qkv(7, 1, 2, N, 64)
        n = N // world
        sl = slice(rank * n, (rank + 1) * n)
        ql, kl, vl = [t[:, :, sl].clone().requires_grad_(True) for t in (q, k, v)]
        be = OracleBackend()
        if levels == 2:
            o = seqpar.llsa_l2_seq_parallel(ql, kl, vl, 8, 8, 16, backend=be)
        else:
            o = seqpar.llsa_l1_seq_parallel(ql, kl, vl, 8, 16, backend=be)
        o.backward(do[:, :, sl])
        got = [seqpar.gather_seq(t.detach(), None) for t in (o, ql.grad, kl.grad, vl.grad)]
        if rank == 0:
            ref = (O.llsa_l2_fwd_bwd if levels == 2 else O.llsa_l1_fwd_bwd)(q, k, v, do, faithful=False)
            torch.save(dict(got=got, ref=[ref["o"], ref["dq"], ref["dk"], ref["dv"]]), out)
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("levels", [1, 2])
def test_two_gloo_ranks_sequence_sharded_matches_unsharded_oracle(tmp_path, levels):
    out = str(tmp_path / "r0.pt")
    port = 31500 + (os.getpid() + levels) % 2000
    mp.spawn(_gloo_worker, args=(2, port, out, levels), nprocs=2, join=True)
    r = torch.load(out)
    for name, g, w in zip(("o", "dq", "dk", "dv"), r["got"], r["ref"]):
        err = (g.float() - w.float()).abs().max().item()
        assert err < 2e-5, (name, err)


# ------------------------------------------------------------------ GPU
def _rank_by_rank(levels, world, dtype):
    """Every rank's local forward + backward on ONE device, in turn; the exchange is a plain sum."""
    import llsa_b200 as L
    dev = "cuda:0"
    N = 16384 if levels == 2 else 4096
    q, k, v, do = [t.to(dev) for t in synth.correlated_qkv(11, 1, 2, N, 64, dtype=dtype)]
    be = seqpar.CudaBackend()
    pyr = be.pool_pyramid([q, k, v], 16, levels)
    pk, pv = pyr[0][1], pyr[0][2]
    pk2, pv2 = (pyr[1][1], pyr[1][2]) if levels == 2 else (None, None)
    n = N // world
    os_, dqs, dk, dv = [], [], 0, 0
    for r in range(world):
        sl = slice(r * n, (r + 1) * n)
        ql = q[:, :, sl].contiguous()
        pq_levels = [lv[0][:, :, sl.start // (16 ** (i + 1)):sl.stop // (16 ** (i + 1))].contiguous() for i, lv in enumerate(pyr[:levels])]
        o, lse, idx, pidx, w1, w2 = seqpar.local_forward(be, ql, k, v, pq_levels, pk, pv, pk2, pv2, 8, 8, 16)
        dq, dkp, dvp = be.attn_bwd_folded(do[:, :, sl].contiguous(), ql, k, v, pk, pv, pk2, pv2, o, lse, idx, pidx, idx.shape[-1],
                                          pidx.shape[-1] if levels == 2 else 0, 16, w1, w2, w1 if levels == 2 else 1.0, w2)
        os_.append(o); dqs.append(dq)
        dk, dv = dk + dkp.float(), dv + dvp.float()
    qg, kg, vg = [t.clone().requires_grad_(True) for t in (q, k, v)]
    o_ref = L.llsa_l2(qg, kg, vg, 8, 8, 16) if levels == 2 else L.llsa_l1(qg, kg, vg, 8, 16)
    o_ref.backward(do)
    return torch.cat(os_, 2), torch.cat(dqs, 2), dk, dv, o_ref.detach(), qg.grad, kg.grad.float(), vg.grad.float()


@pytest.mark.gpu
@pytest.mark.parametrize("levels,world,dtype", [(2, 2, torch.bfloat16), (2, 8, torch.bfloat16), (1, 4, torch.bfloat16), (2, 4, torch.float32)])
def test_rectangular_kernels_rank_by_rank_match_unsharded(levels, world, dtype):
    from helpers import rel_l2
    o, dq, dk, dv, o_ref, dq_ref, dk_ref, dv_ref = _rank_by_rank(levels, world, dtype)
    assert torch.equal(o, o_ref)                 # per-row arithmetic is the unsharded operator's
    assert torch.equal(dq, dq_ref)
    tol = 4e-3 if dtype == torch.bfloat16 else 1e-5      # W partials, each rounded to the dtype, against one rounding
    assert rel_l2(dk, dk_ref) < tol and rel_l2(dv, dv_ref) < tol


def _nccl_worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        import llsa_b200 as L
        N = 16384
        q, k, v, do = [t.to(dev) for t in synth.correlated_qkv(13, 1, 2, N, 64, dtype=torch.bfloat16)]
        n = N // world
        sl = slice(rank * n, (rank + 1) * n)
        ql, kl, vl = [t[:, :, sl].clone().requires_grad_(True) for t in (q, k, v)]
        o = seqpar.llsa_l2_seq_parallel(ql, kl, vl, 8, 8, 16)
        o.backward(do[:, :, sl].contiguous())
        got = [seqpar.gather_seq(t.detach(), None).cpu() for t in (o, ql.grad, kl.grad, vl.grad)]
        if rank == 0:
            qg, kg, vg = [t.clone().requires_grad_(True) for t in (q, k, v)]
            o_ref = L.llsa_l2(qg, kg, vg, 8, 8, 16)
            o_ref.backward(do)
            torch.save(dict(got=got, ref=[t.cpu() for t in (o_ref.detach(), qg.grad, kg.grad, vg.grad)]), out)
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.gpu
def test_two_gpus_sequence_sharded_over_nccl(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from helpers import rel_l2
    out = str(tmp_path / "r0.pt")
    port = 33500 + os.getpid() % 2000
    mp.spawn(_nccl_worker, args=(2, port, out), nprocs=2, join=True)
    r = torch.load(out)
    assert torch.equal(r["got"][0], r["ref"][0]) and torch.equal(r["got"][1], r["ref"][1])
    assert rel_l2(r["got"][2], r["ref"][2]) < 4e-3 and rel_l2(r["got"][3], r["ref"][3]) < 4e-3


def test_head_groups_split_slices_before_the_sequence():
    """(b,h) slices are split over groups of ranks first, only the rest shards the sequence: 6 heads on 8 GPUs are two
    groups of four ranks with three heads each."""
    from llsa_b200 import seqpar
    assert seqpar.head_groups(6, 8) == 2 and seqpar.head_groups(6, 4) == 2 and seqpar.head_groups(6, 2) == 2
    assert seqpar.head_groups(48, 8) == 8 and seqpar.head_groups(6, 3) == 3 and seqpar.head_groups(5, 4) == 1
    assert seqpar.head_groups(6, 1) == 1
