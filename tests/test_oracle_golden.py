"""The CPU oracle against the golden vectors produced by the reference's own
Triton kernels under the Triton interpreter (tests/golden/make_golden.py).
Selection outputs must match bit for bit; floating-point outputs to ~1e-6
(both sides are fp32; only summation order differs)."""
import numpy as np
import pytest
import torch

from helpers import load_golden, rel_l2, sha
from llsa_b200 import synth
from oracle import llsa_oracle as O

FP_TOL = 5e-6


def test_pool_matches_reference_bits():
    g = load_golden("pool_fp32.npz")
    x, dy = synth.gaussian_qkv(int(g["seed"]), *[int(s) for s in g["shape"]], n_tensors=2)
    assert sha(x, dy) == str(g["input_sha"])
    y = O.mean_pool1d(x, 16)
    assert np.array_equal(y.numpy(), g["y"])
    assert np.array_equal(O.mean_pool1d(y, 16).numpy(), g["y2"])
    assert np.array_equal(O.mean_pool1d_bwd(dy[:, :, :32], 16).numpy(), g["dx"])


def test_rope_matches_reference_bits():
    g = load_golden("rope_fp32.npz")
    B, H, S, D = [int(s) for s in g["shape"]]
    x, dy = synth.gaussian_qkv(int(g["seed"]), B, S, H, D, n_tensors=2)
    assert sha(x, dy) == str(g["input_sha"])
    table = synth.rope_table_2d(16)
    assert torch.equal(table, O.rope_table_2d(16, perm=O.morton_perm(16)[1]))
    assert np.array_equal(O.rope_fwd(x.transpose(1, 2), table).numpy(), g["y"])
    assert np.array_equal(O.rope_bwd(dy.transpose(1, 2), table).numpy(), g["dx"])


def test_morton_perm_is_involution_pair():
    p, ip = O.morton_perm(32)
    assert torch.equal(p[ip], torch.arange(1024))
    p2, ip2 = synth.morton_perm(32)
    assert np.array_equal(p.numpy(), p2) and np.array_equal(ip.numpy(), ip2)
    # first 2x2 quad of the grid occupies the first four tokens
    assert sorted(ip[:4].tolist()) == [0, 1, 32, 33]


def test_l1_cfg1_matches_reference():
    g = load_golden("l1_cfg1_fp32.npz")
    q, k, v, do, _ = synth.make_config_inputs("cfg1")
    assert sha(q, k, v, do) == str(g["input_sha"])
    r = O.llsa_l1_fwd_bwd(q, k, v, do)
    rows = int(g["rows"])
    assert np.array_equal(r["pq"].numpy(), g["pq"]) and np.array_equal(r["pk"].numpy(), g["pk"])
    assert np.array_equal(r["indices"].numpy(), g["indices"].astype(np.int64))
    off, flat = O.transpose_indices(r["indices"])
    assert np.array_equal(off.numpy(), g["offsets"])
    assert rel_l2(r["lse"], g["lse"]) < FP_TOL
    for name in ("o", "dq", "dk", "dv"):
        assert rel_l2(r[name][:, :, ::rows], g[name]) < FP_TOL, name
    # the reference's one-level backward leaves the token weight out of dpk/dpv
    assert rel_l2(r["dpk"], g["dpk"]) < FP_TOL and rel_l2(r["dpv"], g["dpv"]) < FP_TOL
    exact = O.llsa_l1_fwd_bwd(q, k, v, do, exact_pooled_grad=True)
    assert rel_l2(exact["dpk"], 16 * g["dpk"]) < FP_TOL


def test_l2_n16384_matches_reference():
    g = load_golden("l2_n16384_fp32.npz")
    B, H, N, D = [int(s) for s in g["shape"]]
    q, k, v, do = synth.correlated_qkv(int(g["seed"]), B, H, N, D, dtype=torch.float32)
    assert sha(q, k, v, do) == str(g["input_sha"])
    r = O.llsa_l2_fwd_bwd(q, k, v, do)
    rows = int(g["rows"])
    assert np.array_equal(r["pk2"].numpy(), g["pk2"]) and np.array_equal(r["pq2"].numpy(), g["pq2"])
    assert np.array_equal(r["p_indices"].numpy(), g["p_indices"].astype(np.int64))
    assert np.array_equal(r["indices"].numpy(), g["indices"].astype(np.int32))
    off, _ = O.transpose_indices(r["indices"])
    offp, _ = O.transpose_indices(r["p_indices"])
    assert np.array_equal(off.numpy(), g["offsets"]) and np.array_equal(offp.numpy(), g["offsets_p"])
    assert rel_l2(r["lse"], g["lse"]) < FP_TOL
    for name in ("o", "dq", "dk", "dv"):
        assert rel_l2(r[name][:, :, ::rows], g[name]) < FP_TOL, name
    dpk_t = r["dpk"] + O.mean_pool1d_bwd(r["dpk2"], 16)
    dpv_t = r["dpv"] + O.mean_pool1d_bwd(r["dpv2"], 16)
    assert rel_l2(dpk_t[:, :, ::rows], g["dpk_total"]) < FP_TOL
    assert rel_l2(dpv_t[:, :, ::rows], g["dpv_total"]) < FP_TOL
    assert rel_l2(r["dpk2"], g["dpk2"]) < FP_TOL and rel_l2(r["dpv2"], g["dpv2"]) < FP_TOL


def test_block_gather_equals_dense_masked_autograd():
    """The explicit backward formulas equal autograd through the dense masked
    softmax (the mathematically exact gradient) on a small two-level case."""
    torch.manual_seed(0)
    B, H, N, D = 1, 1, 16384, 64
    q, k, v, do = synth.correlated_qkv(21, B, H, N, D, dtype=torch.float32)
    r = O.llsa_l2_fwd_bwd(q, k, v, do, faithful=False)
    rows = slice(0, 2048)    # dense evaluation of the first 2048 query rows only (memory)
    qd = q[:, :, rows].clone().double().requires_grad_(True)
    kd, vd = k.double().requires_grad_(True), v.double().requires_grad_(True)
    bs = 16
    sc = 1.0 / 8.0
    pool = lambda x: x.reshape(B, H, x.shape[2] // bs, bs, D).mean(3)
    pk1, pv1 = pool(kd), pool(vd)
    pk2, pv2 = pool(pk1), pool(pv1)
    idx, pidx = r["indices"][:, :, :128], r["p_indices"][:, :, :8]
    m1 = torch.zeros(B, H, 128, N // bs, dtype=torch.bool).scatter_(-1, idx.long(), True)
    fine = m1.repeat_interleave(bs, 2).repeat_interleave(bs, 3)
    s = (qd @ kd.transpose(-1, -2) * sc).masked_fill(~fine, float("-inf"))
    m2 = torch.zeros(B, H, 8, N // 256, dtype=torch.bool).scatter_(-1, pidx.long(), True)
    cand = m2.repeat_interleave(256, 2).repeat_interleave(bs, 3)
    sp1 = (qd @ pk1.transpose(-1, -2) * sc + np.log(16.0)).masked_fill(~cand, float("-inf"))
    sp2 = qd @ pk2.transpose(-1, -2) * sc + np.log(256.0)
    a = torch.softmax(torch.cat([s, sp1, sp2], -1), -1)
    o = a[..., :N] @ vd + a[..., N:N + N // bs] @ pv1 + a[..., N + N // bs:] @ pv2
    assert rel_l2(r["o"][:, :, rows], o.detach()) < 1e-5
    (dq,) = torch.autograd.grad(o, qd, do[:, :, rows].double())
    assert rel_l2(r["dq"][:, :, rows], dq) < 1e-5
