"""The rope-DiT caller (llsa_b200/dit.py): structure on CPU with dense attention, the sparse operators on the GPU."""
import math

import pytest
import torch

from llsa_b200.dit import RopeDiT, timestep_embedding


def test_timestep_embedding_layout():
    e = timestep_embedding(torch.tensor([0.0, 7.0]), 256)
    assert e.shape == (2, 256)
    assert torch.allclose(e[0, :128], torch.ones(128)) and torch.allclose(e[0, 128:], torch.zeros(128))      # cos half first
    assert abs(e[1, 0].item() - math.cos(7.0)) < 1e-6 and abs(e[1, 128].item() - math.sin(7.0)) < 1e-6        # frequency 1 first
    assert abs(e[1, 127].item() - math.cos(7.0 / 10000.0)) < 1e-6                                             # last: 1 / max_period


def _tiny(attn_type="pixel", perm=True, **kw):
    torch.manual_seed(0)
    return RopeDiT(heads=2, head_dim=64, layers=2, sample_size=16, attn_type=attn_type, token_permutation=perm, **kw)


def test_dense_dit_shapes_and_grads_on_cpu():
    m = _tiny()
    x = torch.randn(2, 3, 16, 16)
    y = m(x, torch.tensor([3, 500]))
    assert y.shape == (2, 3, 16, 16) and torch.isfinite(y).all()
    y.square().mean().backward()
    assert all(p.grad is not None and torch.isfinite(p.grad).all() for p in m.parameters())


def test_token_permutation_does_not_change_dense_attention():
    """Dense attention is permutation-equivariant and the RoPE table is permuted with the tokens
    (rope_dit_transformer_2d.py:168-170), so Morton order in and out must leave the output unchanged."""
    a, b = _tiny(perm=True), _tiny(perm=False)
    b.load_state_dict(a.state_dict())
    x = torch.randn(1, 3, 16, 16)
    t = torch.tensor([42])
    assert torch.allclose(a(x, t), b(x, t), atol=2e-5)


@pytest.mark.gpu
@pytest.mark.parametrize("qk_norm", [False, True])
def test_sparse_l2_dit_fused_rope_equals_unfused(qk_norm):
    """The fused q / k preparation inside the model.  Without q/k RMSNorm (RoPE + pooling fused) the fused and the unfused
    model agree bit for bit.  With it, the fused pass sums the squares in its own fixed order while the unfused model runs
    the eager RMSNorm, so the normalised q, k can differ in the last bf16 bit: outputs and gradients agree like two bf16
    evaluations of one model."""
    dev = "cuda:0"
    torch.manual_seed(1)
    a = RopeDiT(layers=2, attn_type="sparse_l2", fused_rope=True, qk_norm=qk_norm).to(dev)
    b = RopeDiT(layers=2, attn_type="sparse_l2", fused_rope=False, qk_norm=qk_norm).to(dev)
    b.load_state_dict(a.state_dict())
    x = torch.randn(1, 3, 128, 128, device=dev)
    t = torch.tensor([321], device=dev)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        ya, yb = a(x, t), b(x, t)
    assert ya.shape == (1, 3, 128, 128) and torch.isfinite(ya).all()
    if qk_norm:
        assert (ya.float() - yb.float()).norm() <= 3e-2 * yb.float().norm()
    else:
        assert torch.equal(ya, yb)
    ya.float().square().mean().backward()
    yb.float().square().mean().backward()
    for (n, p), (_, q) in zip(a.named_parameters(), b.named_parameters()):
        assert torch.isfinite(p.grad).all(), n
        # dk / dv sum fp32 reductions in a run-dependent order and bf16 rounding follows: the two runs differ like two runs of one model
        assert (p.grad - q.grad).norm() <= (1e-1 if qk_norm else 5e-2) * (q.grad.norm() + 1e-12), n


@pytest.mark.gpu
def test_sparse_l1_dit_runs():
    dev = "cuda:0"
    torch.manual_seed(2)
    m = RopeDiT(layers=1, sample_size=64, attn_type="sparse_l1").to(dev)
    x = torch.randn(2, 3, 64, 64, device=dev)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        y = m(x, torch.tensor([1, 999], device=dev))
    y.float().square().mean().backward()
    assert torch.isfinite(y).all() and all(torch.isfinite(p.grad).all() for p in m.parameters())
