"""Shared comparison helpers for the parity tests."""
import hashlib
import os

import numpy as np
import torch

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def load_golden(name):
    return np.load(os.path.join(GOLDEN, name), allow_pickle=False)


def sha(*tensors):
    h = hashlib.sha256()
    for t in tensors:
        h.update(t.contiguous().numpy().tobytes())
    return h.hexdigest()


def rel_l2(a, b):
    a = torch.as_tensor(a).detach().double().cpu()
    b = torch.as_tensor(b).detach().double().cpu()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))


def max_abs(a, b):
    return float((torch.as_tensor(a).detach().double().cpu() - torch.as_tensor(b).detach().double().cpu()).abs().max())


def topk_mismatch_rows(idx_a, idx_b, scores, margin=1e-6):
    """Tie-aware comparison of two top-k index tensors [..., M, T] against the
    score matrix [..., M, n] both were selected from.  Rows where the ordered
    lists differ are accepted only if the selected SCORES agree position by
    position within `margin` (an exact tie or a last-ulp accumulation
    difference); returns (rows that differ, rows that differ beyond the margin)."""
    idx_a = torch.as_tensor(idx_a).long().cpu()
    idx_b = torch.as_tensor(idx_b).long().cpu()
    scores = torch.as_tensor(scores).double().cpu()
    diff_rows = (idx_a != idx_b).any(-1)
    sa = torch.gather(scores, -1, idx_a)
    sb = torch.gather(scores, -1, idx_b)
    bad = ((sa - sb).abs() > margin * sb.abs().clamp_min(1.0)).any(-1) & diff_rows
    return int(diff_rows.sum()), int(bad.sum())


def csr_canonical(offsets, flat):
    """Sort every bucket of a CSR (offsets [.., n+1], flat [.., E]) ascending."""
    offsets = torch.as_tensor(offsets).long().cpu()
    flat = torch.as_tensor(flat).long().cpu().clone()
    o2 = offsets.reshape(-1, offsets.shape[-1])
    f2 = flat.reshape(-1, flat.shape[-1])
    for r in range(o2.shape[0]):
        for j in range(o2.shape[1] - 1):
            s, e = int(o2[r, j]), int(o2[r, j + 1])
            f2[r, s:e] = f2[r, s:e].sort().values
    return f2.reshape(flat.shape)
