"""Generate the golden fixtures in this directory by running the REFERENCE's own
Triton kernels under the Triton CPU interpreter (fp32).

Run once, where the reference checkout is available:

    python tests/golden/make_golden.py /path/to/reference [case ...]

It needs `TRITON_INTERPRET=1` before triton is imported (set below) and puts
`<reference>/src` on sys.path; nothing is copied from the reference.  Inputs
come from llsa_b200.synth (numpy PCG64) so tests can rebuild them from the seed;
each fixture stores a SHA-256 of its input bytes.  Large outputs are stored on a
row stride (`rows`) to keep the files small.
"""
import hashlib
import os
import sys
import time

os.environ["TRITON_INTERPRET"] = "1"
HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

import numpy as np
import torch


def sha(*tensors):
    h = hashlib.sha256()
    for t in tensors:
        h.update(t.contiguous().numpy().tobytes())
    return h.hexdigest()


def npy(t):
    return t.detach().cpu().numpy()


def case_pool(ref):
    from llsa.kernel.triton.mean_pool import mean_pool1d
    from llsa_b200.synth import gaussian_qkv
    x, dy_full = gaussian_qkv(11, 1, 2, 512, 64, n_tensors=2)
    x.requires_grad_(True)
    y = mean_pool1d(x, 16)
    y2 = mean_pool1d(y, 16)
    dy = dy_full[:, :, :32].contiguous()
    (dx,) = torch.autograd.grad(y, x, dy)
    np.savez_compressed(os.path.join(HERE, "pool_fp32.npz"), seed=11, shape=[1, 2, 512, 64], input_sha=sha(x.detach(), dy_full),
                        y=npy(y), y2=npy(y2), dx=npy(dx))


def case_rope(ref):
    from llsa.kernel.triton.rope import my_rope_fn
    from llsa_b200.synth import gaussian_qkv, rope_table_2d
    B, H, S, D = 1, 2, 256, 64
    x, dy = gaussian_qkv(12, B, S, H, D, n_tensors=2)            # physical [B,S,H,D]
    table = rope_table_2d(16, dtype=torch.float32)
    xv = x.transpose(1, 2).requires_grad_(True)                   # strided [B,H,S,D] view, as the model passes it
    y = my_rope_fn(xv, table)
    (dx,) = torch.autograd.grad(y, xv, dy.transpose(1, 2))
    np.savez_compressed(os.path.join(HERE, "rope_fp32.npz"), seed=12, shape=[B, H, S, D], input_sha=sha(x, dy),
                        y=npy(y.contiguous()), dx=npy(dx.contiguous()), y_strides=list(y.stride()))


def case_l1(ref):
    """BASELINE config 1: llsa_l1 fp32 B=1,H=2,N=1024,D=64, block 16, topk 8, fwd+bwd."""
    from llsa.kernel.triton.mean_pool import mean_pool1d
    from llsa.kernel.triton.topk import gen_sparse_indices
    from llsa.kernel.triton.indices_transpose import transpose_indices
    from llsa.kernel.torch_op.flash_sparse_attention_res_1 import flash_sparse_residual_attention_l1_op
    from llsa.kernel.triton.sparse_attention_res_1 import sparse_indices_attn_res_fwd
    from llsa_b200.synth import make_config_inputs
    q, k, v, do, _ = make_config_inputs("cfg1")
    insha = sha(q, k, v, do)
    q.requires_grad_(True); k.requires_grad_(True); v.requires_grad_(True)
    pq, pk, pv = mean_pool1d(q, 16), mean_pool1d(k, 16), mean_pool1d(v, 16)
    pk.retain_grad(); pv.retain_grad()
    t = time.time()
    o = flash_sparse_residual_attention_l1_op(q, k, v, pq, pk, pv, 8, 16, 16)
    o.backward(do)
    print("l1 fwd+bwd %.0fs" % (time.time() - t))
    with torch.no_grad():
        idx = gen_sparse_indices(pq, pk, 8)
        _, lse = sparse_indices_attn_res_fwd(q, k, v, pk, pv, idx, 8, 16, 4)
        off, flat = transpose_indices(idx)
    rows = 4
    np.savez_compressed(os.path.join(HERE, "l1_cfg1_fp32.npz"), config="cfg1", input_sha=insha, rows=rows,
                        pq=npy(pq), pk=npy(pk), pv=npy(pv), indices=npy(idx).astype(np.int16), lse=npy(lse),
                        offsets=npy(off).astype(np.int32),
                        o=npy(o)[:, :, ::rows], dq=npy(q.grad)[:, :, ::rows], dk=npy(k.grad)[:, :, ::rows],
                        dv=npy(v.grad)[:, :, ::rows], dpk=npy(pk.grad), dpv=npy(pv.grad))


def case_l2(ref):
    """llsa_l2 fp32 B=1,H=1,N=16384 (the smallest N where every stage of L2 is active), fwd+bwd."""
    from llsa.kernel.triton.mean_pool import mean_pool1d
    from llsa.kernel.triton.topk import gen_sparse_indices, compute_topk_indices_sparse
    from llsa.kernel.triton.indices_transpose import transpose_indices
    from llsa.kernel.torch_op.flash_sparse_attention_res_2 import flash_sparse_residual_attention_l2_op
    from llsa.kernel.triton.sparse_attention_res_2 import sparse_indices_attn_res_2_2_fwd
    from llsa_b200.synth import correlated_qkv
    B, H, N, D = 1, 1, 16384, 64
    q, k, v, do = correlated_qkv(13, B, H, N, D, dtype=torch.float32)
    insha = sha(q, k, v, do)
    q.requires_grad_(True); k.requires_grad_(True); v.requires_grad_(True)
    pq, pk, pv = mean_pool1d(q, 16), mean_pool1d(k, 16), mean_pool1d(v, 16)
    pq2, pk2, pv2 = mean_pool1d(pq, 16), mean_pool1d(pk, 16), mean_pool1d(pv, 16)
    for t_ in (pk, pv, pk2, pv2):
        t_.retain_grad()
    t = time.time()
    o = flash_sparse_residual_attention_l2_op(q, k, v, pq, pk, pv, pq2, pk2, pv2, 8, 8, 16, 256, 16)
    print("l2 fwd %.0fs" % (time.time() - t)); t = time.time()
    o.backward(do)
    print("l2 bwd %.0fs" % (time.time() - t))
    with torch.no_grad():
        pidx = gen_sparse_indices(pq2, pk2, 8)
        idx = compute_topk_indices_sparse(pq, pk, pidx, 8, 8, 16)
        off, flat = transpose_indices(idx)
        off_p, flat_p = transpose_indices(pidx)
        _, lse = sparse_indices_attn_res_2_2_fwd(q, k, v, pk, pv, pk2, pv2, idx, pidx, 8, 8, 16, 256, 4)
    rows = 32
    sub = lambda x: npy(x)[:, :, ::rows]
    np.savez_compressed(os.path.join(HERE, "l2_n16384_fp32.npz"), seed=13, shape=[B, H, N, D], input_sha=insha, rows=rows,
                        pq2=npy(pq2), pk2=npy(pk2), pv2=npy(pv2), pk=sub(pk), pq=sub(pq),
                        p_indices=npy(pidx).astype(np.int16), indices=npy(idx).astype(np.int16),
                        offsets=npy(off).astype(np.int32), offsets_p=npy(off_p).astype(np.int32), lse=npy(lse),
                        o=sub(o), dq=sub(q.grad), dk=sub(k.grad), dv=sub(v.grad),
                        dpk_total=sub(pk.grad), dpv_total=sub(pv.grad), dpk2=npy(pk2.grad), dpv2=npy(pv2.grad))


CASES = dict(pool=case_pool, rope=case_rope, l1=case_l1, l2=case_l2)

if __name__ == "__main__":
    ref = sys.argv[1]
    sys.path.insert(0, os.path.join(ref, "src"))
    torch.set_num_threads(max(1, os.cpu_count() // 2))
    for name in (sys.argv[2:] or list(CASES)):
        t0 = time.time()
        CASES[name](ref)
        print("golden case %s done in %.0fs" % (name, time.time() - t0), flush=True)
