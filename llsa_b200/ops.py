"""Host side of the LLSA operators: the reference's Python API over the C ABI.

Function names, argument order and return values mirror the reference
(SingleZombie/LLSA, src/llsa/kernel/...), so callers written against it run
unchanged:

    mean_pool1d, my_rope_fn                    triton/mean_pool.py:209, triton/rope.py:148
    gen_sparse_indices, compute_topk_indices_sparse   triton/topk.py:6, :172
    transpose_indices                          triton/indices_transpose.py:104
    sparse_indices_attn_res_fwd / ..._scatter_bwd_v2          triton/sparse_attention_res_1.py:123, :403
    sparse_indices_attn_res_2_2_fwd / ..._scatter_2_2_bwd_v2  triton/sparse_attention_res_2.py:166, :578
    flash_sparse_residual_attention_l1_op / _l2_op            torch_op/flash_sparse_attention_res_{1,2}.py:38, :45
    llsa_l1, llsa_l2                           torch_op/flash_sparse_attention_res_1.py:41, _res_2.py:48

Every function enqueues CUDA work on the current stream through
libllsa_b200.so; tensors must live on a CUDA device.  The differentiable
entry points are torch.library custom ops with registered autograd.
"""
from __future__ import annotations

import ctypes as C
import math
import os
from typing import List, Optional, Tuple

import torch

from . import _lib
from ._lib import desc, ptr, ref

__all__ = [
    "mean_pool1d", "my_rope_fn", "gen_sparse_indices", "compute_topk_indices_sparse", "transpose_indices",
    "sparse_indices_attn_res_fwd", "sparse_indices_attn_res_scatter_bwd_v2",
    "sparse_indices_attn_res_2_2_fwd", "sparse_indices_attn_res_scatter_2_2_bwd_v2",
    "flash_sparse_residual_attention_l1_op", "flash_sparse_residual_attention_l2_op",
    "llsa_l1", "llsa_l2", "llsa_l1_rope", "llsa_l2_rope", "pool_pyramid", "rope_pool_pyramid", "set_exact_pooled_grad",
    "set_device_checks", "rms_norm", "rms_rope_pool_pyramid", "llsa_l1_rms_rope", "llsa_l2_rms_rope",
]

_FLOAT = (torch.float32, torch.bfloat16)
_force_generic = os.environ.get("LLSA_B200_FORCE_GENERIC", "0") == "1"
# The reference's one-level backward drops the token weight from the pooled-key
# gradients (sparse_attention_res_1.py:389).  False reproduces that; True gives
# the exact gradient.
_exact_pooled_grad = os.environ.get("LLSA_B200_EXACT_POOLED_GRAD", "0") == "1"


_stage_hook = None
_overlap_transpose = os.environ.get("LLSA_B200_OVERLAP_TRANSPOSE", "1") != "0"
_side_streams = {}
# Cross-check switch: keep the pooled-key stages on the mma.sync kernels (the form other shapes use).
_no_tcgen05 = False
# Cross-check switch: False = long pooled key lists take two passes over the keys for every row (no `fwd_redo` scratch).
_one_pass_pooled = True
_last_fwd_redo = None        # the marks of the most recent forward (tests look at how many rows the second launch redid)
# Test hook: polls after which a bounded wait inside the tcgen05 kernels gives up (0 = the kernels' default).
_wait_limit = 0
# Device-side checks.  The kernels OR bits into a status word when they meet an out-of-range block index or when a
# bounded wait runs out.  Reading the word back costs a host synchronisation, which the reference's operators never do,
# so it is off by default; with it on, every operator synchronises and raises (LLSA_ERR_DEVICE_CHECK) on a set bit.
_device_checks = os.environ.get("LLSA_B200_DEVICE_CHECKS", "0") == "1"


def set_device_checks(flag: bool) -> None:
    """Debug mode: read the kernels' device status word back after every operator (a host sync) and raise if a kernel
    met an out-of-range block index or gave up a bounded wait."""
    global _device_checks
    _device_checks = bool(flag)


def _new_status(device):
    return torch.zeros(1, dtype=torch.int32, device=device) if _device_checks else None


def _check_status(status, what: str) -> None:
    if status is not None:
        _lib.check(_lib.lib().llsa_status_check(int(status.item())), what)


def _side_stream(device) -> "torch.cuda.Stream":
    key = (device.type, device.index if device.index is not None else torch.cuda.current_device())
    if key not in _side_streams:
        _side_streams[key] = torch.cuda.Stream(device)
    return _side_streams[key]


def set_stage_hook(fn) -> None:
    """fn(name) is called right before each kernel group is enqueued (and with
    "end" after the last one of an operator); None disables it.  Used by the
    benchmark to bracket kernels with CUDA events."""
    global _stage_hook
    _stage_hook = fn


def _mark(name: str) -> None:
    if _stage_hook is not None:
        _stage_hook(name)


def set_exact_pooled_grad(flag: bool) -> None:
    """Choose between the reference-compatible (False, default) and the
    mathematically exact (True) pooled-key gradient of llsa_l1."""
    global _exact_pooled_grad
    _exact_pooled_grad = bool(flag)


def _need_cuda(*ts: torch.Tensor) -> None:
    for t in ts:
        if t is not None and not t.is_cuda:
            raise RuntimeError("llsa_b200 runs on CUDA tensors only (got a %s tensor); there is no CPU path" % t.device.type)


def _prep(t: torch.Tensor) -> torch.Tensor:
    """Kernels take any batch/head/token strides but need unit channel stride and 16-byte aligned rows."""
    return t if _rows_ok(t) else t.contiguous()


def _check_float(*ts: torch.Tensor) -> None:
    dt = ts[0].dtype
    if dt not in _FLOAT:
        raise TypeError("llsa_b200 supports float32 and bfloat16 tensors, got %s" % dt)
    for t in ts:
        if t.dtype != dt:
            raise TypeError("llsa_b200: all floating-point operands must share one dtype")


def _stream(t: torch.Tensor):
    return _lib.stream_ptr(t.device)


# ----------------------------------------------------------------------------- pooling
def _pool_fwd_impl(x: torch.Tensor, k: int) -> torch.Tensor:
    _need_cuda(x)
    _check_float(x)
    B, H, S, Cc = x.shape
    assert S % k == 0, "sequence length must be divisible by the pooling factor"
    x = x if x.stride(-1) == 1 else x.contiguous()
    y = torch.empty((B, H, S // k, Cc), device=x.device, dtype=x.dtype)
    with torch.cuda.device(x.device):
        dx, dy = desc(x), desc(y)
        _lib.check(_lib.lib().llsa_mean_pool_fwd(ref(dx), ref(dy), k, _stream(x)), "mean_pool_fwd")
    return y


def _pool_bwd_impl(dy: torch.Tensor, k: int) -> torch.Tensor:
    _need_cuda(dy)
    dy = dy if dy.stride(-1) == 1 else dy.contiguous()
    B, H, S, Cc = dy.shape
    dx = torch.empty((B, H, S * k, Cc), device=dy.device, dtype=dy.dtype)
    with torch.cuda.device(dy.device):
        a, b = desc(dy), desc(dx)
        _lib.check(_lib.lib().llsa_mean_pool_bwd(ref(a), ref(b), k, _stream(dy)), "mean_pool_bwd")
    return dx


@torch.library.custom_op("llsa_b200::mean_pool_fwd", mutates_args=())
def _mean_pool_fwd_op(x: torch.Tensor, k: int) -> torch.Tensor:
    return _pool_fwd_impl(x, k)


@_mean_pool_fwd_op.register_fake
def _(x, k):
    return x.new_empty((x.shape[0], x.shape[1], x.shape[2] // k, x.shape[3]))


@torch.library.custom_op("llsa_b200::mean_pool_bwd", mutates_args=())
def _mean_pool_bwd_op(dy: torch.Tensor, k: int) -> torch.Tensor:
    return _pool_bwd_impl(dy, k)


@_mean_pool_bwd_op.register_fake
def _(dy, k):
    return dy.new_empty((dy.shape[0], dy.shape[1], dy.shape[2] * k, dy.shape[3]))


def _pool_setup(ctx, inputs, output):
    ctx.k = inputs[1]


def _pool_backward(ctx, dy):
    return _mean_pool_bwd_op(dy, ctx.k), None


_mean_pool_fwd_op.register_autograd(_pool_backward, setup_context=_pool_setup)


def mean_pool1d(x: torch.Tensor, k: int, format: str = "bhsc") -> torch.Tensor:
    """Mean over k consecutive tokens of a [B,H,S,C] tensor, accumulated in x's
    dtype; differentiable.  Mirrors mean_pool1d (triton/mean_pool.py:209-216);
    only the 'bhsc' layout the attention path uses is provided."""
    if format != "bhsc":
        raise NotImplementedError("format %r is not part of the attention hot path" % (format,))
    return _mean_pool_fwd_op(x, k)


def pool_pyramid(xs: List[torch.Tensor], block_size: int, levels: int):
    """All pyramid levels of up to three [B,H,N,D] tensors in one launch.
    Returns (level-1 list, level-2 list or None).  Not differentiable by itself."""
    _need_cuda(*xs)
    _check_float(*xs)
    xs = [_prep(x) for x in xs]
    B, H, N, D = xs[0].shape
    bs = block_size
    y1 = [torch.empty((B, H, N // bs, D), device=x.device, dtype=x.dtype) for x in xs]
    y2 = [torch.empty((B, H, N // bs // bs, D), device=x.device, dtype=x.dtype) for x in xs] if levels == 2 else None
    n = len(xs)
    XA = (_lib.LlsaTensor * n)(*[desc(x) for x in xs])
    Y1 = (_lib.LlsaTensor * n)(*[desc(y) for y in y1])
    Y2 = (_lib.LlsaTensor * n)(*[desc(y) for y in y2]) if y2 is not None else None
    _mark("pool_pyramid")
    with torch.cuda.device(xs[0].device):
        _lib.check(_lib.lib().llsa_pool_pyramid_fwd(n, XA, Y1, Y2, bs, _stream(xs[0])), "pool_pyramid_fwd")
    return y1, y2


def rope_pool_pyramid(xs: List[torch.Tensor], freq: torch.Tensor, rope: List[bool], block_size: int, levels: int):
    """RoPE on the flagged tensors and all pyramid levels of every tensor in ONE pass over HBM.
    Returns (tensors after RoPE (unflagged ones unchanged), level-1 list, level-2 list or None); the
    rotated tensors and the pooled levels carry the bits of my_rope_fn followed by mean_pool1d.
    Falls back to the two separate kernels when the table's dtype differs from the data's."""
    _need_cuda(*xs, freq)
    _check_float(*xs)
    if freq.dtype != xs[0].dtype or not any(rope):
        out = [my_rope_fn(x, freq) if r else x for x, r in zip(xs, rope)]
        y1, y2 = pool_pyramid(out, block_size, levels)
        return out, y1, y2
    xs = [_prep(x) for x in xs]
    freq = freq if (freq.stride(-1) == 1 and freq.data_ptr() % 16 == 0 and (freq.stride(0) * freq.element_size()) % 16 == 0) else freq.contiguous()
    B, H, N, D = xs[0].shape
    assert freq.shape[0] == N and freq.shape[1] == D, "freq must be [N, D]"
    bs = block_size
    xr = [torch.empty_like(x) if r else x for x, r in zip(xs, rope)]     # empty_like keeps x's strides (rope.py:109)
    y1 = [torch.empty((B, H, N // bs, D), device=x.device, dtype=x.dtype) for x in xs]
    y2 = [torch.empty((B, H, N // bs // bs, D), device=x.device, dtype=x.dtype) for x in xs] if levels == 2 else None
    n = len(xs)
    XA = (_lib.LlsaTensor * n)(*[desc(x) for x in xs])
    XR = (_lib.LlsaTensor * n)(*[desc(x) for x in xr])
    Y1 = (_lib.LlsaTensor * n)(*[desc(y) for y in y1])
    Y2 = (_lib.LlsaTensor * n)(*[desc(y) for y in y2]) if y2 is not None else None
    mask = sum(1 << i for i, r in enumerate(rope) if r)
    _mark("pool_pyramid")
    with torch.cuda.device(xs[0].device):
        f = desc(freq)
        _lib.check(_lib.lib().llsa_rope_pool_pyramid_fwd(n, XA, ref(f), mask, XR, Y1, Y2, bs, _stream(xs[0])), "rope_pool_pyramid_fwd")
    return xr, y1, y2


def rms_rope_pool_pyramid(xs: List[torch.Tensor], weights: List[Optional[torch.Tensor]], eps: float, freq: Optional[torch.Tensor],
                          rope: List[bool], block_size: int, levels: int):
    """RMSNorm (tensors with a weight entry that is not None... or True for an all-ones weight), RoPE (flagged tensors) and
    every pyramid level in ONE pass over HBM: what the attention block does to q and k before llsa_l1 / llsa_l2
    (models/rope_dit_transformer_2d.py:215-238).  Returns (transformed tensors, level-1 list, level-2 list or None); the
    results carry the bits of rms_norm -> my_rope_fn -> mean_pool1d run one after the other."""
    _need_cuda(*xs)
    _check_float(*xs)
    xs = [_prep(x) for x in xs]
    B, H, N, D = xs[0].shape
    bs = block_size
    use_rope = freq is not None and any(rope)
    if use_rope:
        if freq.dtype != xs[0].dtype:
            freq = freq.to(xs[0].dtype)
        freq = freq if (freq.stride(-1) == 1 and freq.data_ptr() % 16 == 0 and (freq.stride(0) * freq.element_size()) % 16 == 0) else freq.contiguous()
    normed = [w is not None for w in weights]
    changed = [(r and use_rope) or nm for r, nm in zip(rope, normed)]
    xr = [torch.empty_like(x) if c else x for x, c in zip(xs, changed)]
    y1 = [torch.empty((B, H, N // bs, D), device=x.device, dtype=x.dtype) for x in xs]
    y2 = [torch.empty((B, H, N // bs // bs, D), device=x.device, dtype=x.dtype) for x in xs] if levels == 2 else None
    n = len(xs)
    TP = C.POINTER(_lib.LlsaTensor)
    XA = (_lib.LlsaTensor * n)(*[desc(x) for x in xs])
    XR = (_lib.LlsaTensor * n)(*[desc(x) for x in xr])
    Y1 = (_lib.LlsaTensor * n)(*[desc(y) for y in y1])
    Y2 = (_lib.LlsaTensor * n)(*[desc(y) for y in y2]) if y2 is not None else None
    keep = [w.detach().float().contiguous() if isinstance(w, torch.Tensor) else None for w in weights]
    wdesc = [desc(k) for k in keep]
    WP = (TP * n)(*[C.pointer(d) if d is not None else TP() for d in wdesc])
    rmask = sum(1 << i for i, r in enumerate(rope) if r) if use_rope else 0
    nmask = sum(1 << i for i, nm in enumerate(normed) if nm)
    _mark("pool_pyramid")
    with torch.cuda.device(xs[0].device):
        f = desc(freq) if use_rope else None
        _lib.check(_lib.lib().llsa_rms_rope_pool_pyramid_fwd(n, XA, WP, nmask, float(eps), ref(f), rmask, XR, Y1, Y2, bs, _stream(xs[0])),
                   "rms_rope_pool_pyramid_fwd")
    return xr, y1, y2


def rms_norm(x: torch.Tensor, weight: Optional[torch.Tensor], eps: float = 1e-5) -> torch.Tensor:
    """RMSNorm over the last dimension of [B,H,S,C] with a fixed summation order (the stand-alone form of the
    normalisation fused into rms_rope_pool_pyramid); not differentiable by itself."""
    _need_cuda(x)
    _check_float(x)
    x = _prep(x)
    y = torch.empty_like(x)
    w = weight.detach().float().contiguous() if weight is not None else None
    with torch.cuda.device(x.device):
        a, b, wd = desc(x), desc(y), desc(w)
        _lib.check(_lib.lib().llsa_rms_norm_fwd(ref(a), ref(wd), float(eps), ref(b), _stream(x)), "rms_norm_fwd")
    return y


def _rms_norm_bwd(x: torch.Tensor, weight: Optional[torch.Tensor], eps: float, dy: torch.Tensor):
    """Gradient of y = (x * rsqrt(mean(x^2) + eps)) * w with respect to x and w (fp32 arithmetic, eager)."""
    xf, g = x.float(), dy.float()
    rstd = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    xh = xf * rstd
    gw = g * weight.float() if weight is not None else g
    dx = rstd * (gw - xh * (gw * xh).mean(-1, keepdim=True))
    dw = (g * xh).reshape(-1, x.shape[-1]).sum(0).to(weight.dtype) if weight is not None else None
    return dx.to(x.dtype), dw


# ----------------------------------------------------------------------------- RoPE
def _rope_impl(x: torch.Tensor, freq: torch.Tensor, bwd: bool) -> torch.Tensor:
    _need_cuda(x, freq)
    assert x.dim() == 4 and freq.dim() == 2, "x:[B,H,S,D], freq:[S,D]"
    assert x.shape[-1] % 2 == 0, "D must be even (pairs of cos/sin)."
    assert freq.shape[0] == x.shape[2] and freq.shape[1] == x.shape[3]
    if freq.dtype == torch.float64 or (x.dtype == torch.float32 and freq.dtype == torch.bfloat16):
        freq = freq.to(torch.float32)
    x = _prep(x)
    freq = freq if (freq.stride(-1) == 1 and freq.data_ptr() % 16 == 0) else freq.contiguous()
    y = torch.empty_like(x)     # keeps x's strides, as the reference does (rope.py:109)
    with torch.cuda.device(x.device):
        a, f, b = desc(x), desc(freq), desc(y)
        fn = _lib.lib().llsa_rope_bwd if bwd else _lib.lib().llsa_rope_fwd
        _lib.check(fn(ref(a), ref(f), ref(b), _stream(x)), "rope")
    return y


@torch.library.custom_op("llsa_b200::rope_fwd", mutates_args=())
def _rope_fwd_op(x: torch.Tensor, freq: torch.Tensor) -> torch.Tensor:
    return _rope_impl(x, freq, False)


@_rope_fwd_op.register_fake
def _(x, freq):
    return torch.empty_like(x)


@torch.library.custom_op("llsa_b200::rope_bwd", mutates_args=())
def _rope_bwd_op(dy: torch.Tensor, freq: torch.Tensor) -> torch.Tensor:
    return _rope_impl(dy, freq, True)


@_rope_bwd_op.register_fake
def _(dy, freq):
    return torch.empty_like(dy)


def _rope_setup(ctx, inputs, output):
    ctx.save_for_backward(inputs[1])


def _rope_backward(ctx, dy):
    (freq,) = ctx.saved_tensors
    return _rope_bwd_op(dy, freq), None


_rope_fwd_op.register_autograd(_rope_backward, setup_context=_rope_setup)


def my_rope_fn(x: torch.Tensor, freq: torch.Tensor) -> torch.Tensor:
    """Interleaved-pair RoPE by a [S,D] (sin, cos) table; differentiable in x.
    Mirrors my_rope_fn = MyRopeFunction.apply (triton/rope.py:100-148)."""
    return _rope_fwd_op(x, freq)


# ----------------------------------------------------------------------------- selection
def _coarse_topk(pq: torch.Tensor, pk: torch.Tensor, topk: int, out_dtype=torch.int32) -> torch.Tensor:
    _need_cuda(pq, pk)
    _check_float(pq, pk)
    pq, pk = pq.contiguous(), pk.contiguous()
    topk = min(topk, pk.shape[2])
    idx = torch.empty((*pq.shape[:3], topk), device=pq.device, dtype=out_dtype)
    _mark("coarse_topk")
    with torch.cuda.device(pq.device):
        a, b, c = desc(pq), desc(pk), desc(idx)
        _lib.check(_lib.lib().llsa_coarse_topk(ref(a), ref(b), ref(c), topk, _stream(pq)), "coarse_topk")
    return idx


def gen_sparse_indices(pq: torch.Tensor, pk: torch.Tensor, topk: int) -> torch.Tensor:
    """Top-k key blocks per query block from pooled scores (scores rounded to the
    input dtype, descending, ties to the smallest index); int64 like
    torch.topk.  Mirrors gen_sparse_indices (triton/topk.py:6-9)."""
    return _coarse_topk(pq.detach(), pk.detach(), topk, torch.int64)


def _refine_topk(pq, pk, p_indices, topk, p_topk, block_size) -> torch.Tensor:
    _need_cuda(pq, pk, p_indices)
    _check_float(pq, pk)
    pq, pk, p_indices = pq.contiguous(), pk.contiguous(), p_indices.contiguous()
    idx = torch.empty((*pq.shape[:3], topk), device=pq.device, dtype=torch.int32)
    _mark("refine_topk")
    with torch.cuda.device(pq.device):
        a, b, c, d = desc(pq), desc(pk), desc(p_indices), desc(idx)
        _lib.check(_lib.lib().llsa_refine_topk(ref(a), ref(b), ref(c), ref(d), topk, p_topk, block_size, _stream(pq)), "refine_topk")
    return idx


def _select_two_level(pq, pk, pq2, pk2, topk, p_topk, block_size):
    """(indices, p_indices) of the two-level operator: gen_sparse_indices on the level-2 pooled tensors followed by
    compute_topk_indices_sparse (torch_op/flash_sparse_attention_res_2.py:14-16), one launch where the shape allows."""
    _need_cuda(pq, pk, pq2, pk2)
    _check_float(pq, pk, pq2, pk2)
    pq, pk, pq2, pk2 = pq.contiguous(), pk.contiguous(), pq2.contiguous(), pk2.contiguous()
    p_topk = min(p_topk, pk2.shape[2])
    p_indices = torch.empty((*pq2.shape[:3], p_topk), device=pq.device, dtype=torch.int32)
    indices = torch.empty((*pq.shape[:3], topk), device=pq.device, dtype=torch.int32)
    _mark("select_two_level")
    with torch.cuda.device(pq.device):
        a, b, c, d, e, f = desc(pq), desc(pk), desc(pq2), desc(pk2), desc(p_indices), desc(indices)
        _lib.check(_lib.lib().llsa_select_two_level(ref(a), ref(b), ref(c), ref(d), ref(e), ref(f), topk, p_topk, block_size, _stream(pq)),
                   "select_two_level")
    return indices, p_indices


def compute_topk_indices_sparse(pq, pk, p_indices, topk=8, p_topk=8, block_size=16) -> torch.Tensor:
    """Fine top-k among the children of the selected parent blocks; int32
    [B,H,M,topk].  Mirrors compute_topk_indices_sparse (triton/topk.py:172-197)."""
    return _refine_topk(pq.detach(), pk.detach(), p_indices, topk, p_topk, block_size)


def _transpose(idx: torch.Tensor, k_ntx: int, offsets_dtype, want_pairs: bool):
    B, H, M, T = idx.shape
    offsets = torch.empty((B, H, k_ntx + 1), device=idx.device, dtype=offsets_dtype)
    lists = torch.empty((2 if want_pairs else 1, B, H, M * T), device=idx.device, dtype=torch.int32)
    flat, pairs = lists[0], (lists[1] if want_pairs else None)
    S = _lib.lib().llsa_transpose_range_entries(B, H, M, T)
    ranges = torch.empty((B, H, (M * T + S - 1) // S, 2), device=idx.device, dtype=torch.int32) if want_pairs else None
    status = _new_status(idx.device)
    _mark("transpose_indices")
    with torch.cuda.device(idx.device):
        L = _lib.lib()
        nbytes = L.llsa_transpose_scratch_bytes(B, H, M, T, k_ntx)
        scratch = torch.empty((nbytes,), device=idx.device, dtype=torch.uint8) if nbytes else None
        sp = C.c_void_p(scratch.data_ptr() if nbytes else 0)
        st = C.c_void_p(status.data_ptr()) if status is not None else None
        a, b, c = desc(idx), desc(offsets), desc(flat)
        if want_pairs:
            d, e = desc(pairs), desc(ranges)
            _lib.check(L.llsa_transpose_indices_pairs(ref(a), ref(b), ref(c), ref(d), ref(e), k_ntx, sp, nbytes, st, _stream(idx)), "transpose_indices")
        else:
            _lib.check(L.llsa_transpose_indices(ref(a), ref(b), ref(c), k_ntx, sp, nbytes, st, _stream(idx)), "transpose_indices")
    return offsets, flat, (pairs, ranges), status


def transpose_indices(q_topk_indices: torch.Tensor, k_ntx: Optional[int] = None, offsets_dtype=torch.int64):
    """Query-major top-k lists -> (offsets [B,H,k_ntx+1], flat [B,H,M*T]) with every
    bucket in ascending query order.  Mirrors transpose_indices
    (triton/indices_transpose.py:104-109); `flat` is int32 (the reference's
    uint32 holds the same values).  Indices outside [0, k_ntx) are left out of the
    lists (offsets[..., -1] is then below M*T); with set_device_checks(True) they raise."""
    _need_cuda(q_topk_indices)
    idx = q_topk_indices.contiguous()
    offsets, flat, _, status = _transpose(idx, idx.shape[2] if k_ntx is None else k_ntx, offsets_dtype, False)
    _check_status(status, "transpose_indices")
    return offsets, flat


# ----------------------------------------------------------------------------- attention core
def _attn_args(q, k, v, pk, pv, pk2, pv2, indices, p_indices, o, lse, topk, topk_p, block_size, w1, w2):
    keep = dict(q=desc(q), k=desc(k), v=desc(v), pk=desc(pk), pv=desc(pv), pk2=desc(pk2), pv2=desc(pv2),
                indices=desc(indices), p_indices=desc(p_indices), o=desc(o), lse=desc(lse))
    a = _lib.LlsaAttnArgs()
    for name, d in keep.items():
        setattr(a, name, ptr(d))
    a.topk, a.topk_p, a.block_size = int(topk), int(topk_p), int(block_size)
    a.token_weight, a.token_weight_2 = float(w1), float(w2)
    a.force_generic = 1 if _force_generic else 0
    a.no_tcgen05 = 1 if _no_tcgen05 else 0
    a.wait_limit = int(_wait_limit)
    return a, keep


def _attn_fwd(q, k, v, pk, pv, pk2, pv2, indices, p_indices, topk, topk_p, block_size, w1, w2):
    _need_cuda(q, k, v)
    _check_float(q, k, v, pk, pv)
    q, k, v = _prep(q), _prep(k), _prep(v)
    pk, pv = pk.contiguous(), pv.contiguous()
    if pk2 is not None:
        pk2, pv2, p_indices = pk2.contiguous(), pv2.contiguous(), p_indices.contiguous()
    indices = indices.contiguous()
    o = torch.empty_like(q)
    lse = torch.empty(q.shape[:-1], device=q.device, dtype=torch.float32)
    a, keep = _attn_args(q, k, v, pk, pv, pk2, pv2, indices, p_indices, o, lse, topk, topk_p, block_size, w1, w2)
    status = _new_status(q.device)
    a.status = status.data_ptr() if status is not None else None
    # one byte per query row for the one-pass form of the long pooled key lists (include/llsa_b200.h: fwd_redo)
    one_pass = q.dtype == torch.bfloat16 and _one_pass_pooled
    redo = torch.empty((q.shape[0] * q.shape[1] * q.shape[2] + 3) // 4, device=q.device, dtype=torch.int32) if one_pass else None
    redo_d = desc(redo)
    a.fwd_redo = ptr(redo_d)
    _mark("attn_fwd")
    with torch.cuda.device(q.device):
        _lib.check(_lib.lib().llsa_attn_fwd(C.byref(a), _stream(q)), "attn_fwd")
    _mark("end")
    _check_status(status, "attn_fwd")
    global _last_fwd_redo
    _last_fwd_redo = redo
    return o, lse


def _rows_ok(t: torch.Tensor) -> bool:
    """Unit channel stride; bf16 rows on 32-byte boundaries (what the tensor-core kernels load with one 256-bit
    instruction per lane), fp32 rows on 16-byte boundaries."""
    align = 32 if t.dtype == torch.bfloat16 else 16
    per = align // t.element_size()
    if t.stride(-1) != 1 or t.data_ptr() % align:
        return False
    return all(t.shape[i] == 1 or t.stride(i) % per == 0 for i in range(t.dim() - 1))


def _carve(buf: torch.Tensor, specs):
    """Views into one byte buffer: specs = [(name, dtype, shape)], every view 256-byte aligned."""
    out, off = {}, 0
    for name, dtype, shape in specs:
        n = int(torch.Size(shape).numel()) * torch.empty((), dtype=dtype).element_size()
        out[name] = buf[off:off + n].view(dtype).view(shape)
        off += (n + 255) // 256 * 256
    return out


def _carve_bytes(specs) -> int:
    return sum((int(torch.Size(shape).numel()) * torch.empty((), dtype=dtype).element_size() + 255) // 256 * 256 for _, dtype, shape in specs)


def _attn_bwd(do, q, k, v, pk, pv, pk2, pv2, o, lse, indices, p_indices, topk, topk_p, block_size, w1, w2, kvw1, kvw2, fold):
    _need_cuda(do, q, k, v)
    q, k, v, o, do = _prep(q), _prep(k), _prep(v), _prep(o), _prep(do)
    pk, pv = pk.contiguous(), pv.contiguous()
    if pk2 is not None:
        pk2, pv2, p_indices = pk2.contiguous(), pv2.contiguous(), p_indices.contiguous()
    indices = indices.contiguous()
    lse = lse.contiguous()
    B, H, Nq, T = q.shape[0], q.shape[1], q.shape[2], indices.shape[3]
    tensor_core = q.dtype == torch.bfloat16 and not _force_generic
    # The index transpose (one CTA per (b,h): a latency-bound kernel that leaves most SMs idle) is needed only by the fine
    # dK/dV stage, so it runs on a side stream next to the dQ and pooled stages.
    cur = torch.cuda.current_stream(q.device)
    side = _side_stream(q.device) if _overlap_transpose and _stage_hook is None else None     # a stage hook times every stage on ONE stream
    n_kv = k.shape[2] // block_size                       # buckets = KEY blocks
    if side is not None:
        side.wait_stream(cur)
        with torch.cuda.stream(side):
            offsets, flat, (pairs, ranges), t_status = _transpose(indices, n_kv, torch.int32, tensor_core)
    else:
        offsets, flat, (pairs, ranges), t_status = _transpose(indices, n_kv, torch.int32, tensor_core)
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    # every scratch tensor of the call comes out of ONE allocation; the fp32 pooled-gradient accumulators sit back to back in
    # it (the library clears them with one memset)
    f32 = torch.float32
    specs = [("delta", f32, lse.shape), ("dpk", f32, pk.shape), ("dpv", f32, pv.shape)]
    if pk2 is not None:
        specs += [("dpk2", f32, pk2.shape), ("dpv2", f32, pv2.shape)]
    if tensor_core:     # window partials of the fine dK/dV kernel and the P / dS hand-over (csrc/attn_bwd_mma.cu)
        L = _lib.lib()
        specs += [("partial", f32, (B, H, L.llsa_attn_bwd_partial_elems(B, H, Nq, T) // (B * H * 4096), 4096)),
                  ("pds", f32, (L.llsa_attn_bwd_pds_elems(B, H, Nq, T),))]
    ws = _carve(torch.empty(_carve_bytes(specs), device=q.device, dtype=torch.uint8), specs)
    delta, dpk, dpv = ws["delta"], ws["dpk"], ws["dpv"]
    dpk2, dpv2 = ws.get("dpk2"), ws.get("dpv2")
    a, keep = _attn_args(q, k, v, pk, pv, pk2, pv2, indices, p_indices, o, lse, topk, topk_p, block_size, w1, w2)
    status = _new_status(q.device)
    a.status = status.data_ptr() if status is not None else None
    extra = dict(d_o=desc(do), dq=desc(dq), dk=desc(dk), dv=desc(dv), offsets=desc(offsets), flat=desc(flat), delta=desc(delta),
                 dpk_acc=desc(dpk), dpv_acc=desc(dpv), dpk2_acc=desc(dpk2), dpv2_acc=desc(dpv2), dkv_partial=desc(ws.get("partial")),
                 fine_pds=desc(ws.get("pds")), flat_pairs=desc(pairs), flat_ranges=desc(ranges))
    for name, d in extra.items():
        setattr(a, name, ptr(d))
    a.fold_pool_bwd = 1 if fold else 0
    a.kv_weight, a.kv_weight_2 = float(kvw1), float(kvw2)

    def join_side():
        cur.wait_stream(side)                 # the CSR is ready; its memory now also belongs to this stream
        for t in (offsets, flat) + ((pairs, ranges) if pairs is not None else ()):
            t.record_stream(cur)

    with torch.cuda.device(q.device):
        if _stage_hook is None and side is None:
            _lib.check(_lib.lib().llsa_attn_bwd(C.byref(a), _stream(q)), "attn_bwd")
        elif _stage_hook is None:             # dQ and pooled stages, then the CSR's stream joins, then dK/dV
            a.stage_mask = 3
            _lib.check(_lib.lib().llsa_attn_bwd(C.byref(a), _stream(q)), "attn_bwd")
            join_side()
            a.stage_mask = 4
            _lib.check(_lib.lib().llsa_attn_bwd(C.byref(a), _stream(q)), "attn_bwd")
        else:
            for mask, name in ((1, "attn_bwd_dq"), (2, "attn_bwd_dkv_pooled"), (4, "attn_bwd_dkv_fine")):
                if mask == 4 and side is not None:
                    join_side()
                _mark(name)
                a.stage_mask = mask
                _lib.check(_lib.lib().llsa_attn_bwd(C.byref(a), _stream(q)), name)
            _mark("end")
    _check_status(t_status, "transpose_indices")
    _check_status(status, "attn_bwd")
    return dq, dk, dv, dpk, dpv, dpk2, dpv2


def sparse_indices_attn_res_fwd(q, k, v, pk, pv, indices, topk, token_weight=1, down_scale=4):
    """One-level forward -> (o, m) with m the fp32 log-sum-exp.  Mirrors
    sparse_indices_attn_res_fwd (triton/sparse_attention_res_1.py:123-150)."""
    return _attn_fwd(q, k, v, pk, pv, None, None, indices, None, topk, 0, down_scale * down_scale, token_weight, 1.0)


def sparse_indices_attn_res_2_2_fwd(q, k, v, pk, pv, pk2, pv2, indices, p_indices, topk, topk_p,
                                    token_weight=1, token_weight_2=1, down_scale=4):
    """Two-level forward -> (o, m).  Mirrors sparse_indices_attn_res_2_2_fwd
    (triton/sparse_attention_res_2.py:166-199)."""
    return _attn_fwd(q, k, v, pk, pv, pk2, pv2, indices, p_indices, topk, topk_p, down_scale * down_scale,
                     token_weight, token_weight_2)


def sparse_indices_attn_res_scatter_bwd_v2(do, q, k, v, pk, pv, o, m, indices, topk, block_size, token_weight):
    """One-level backward -> (dq, dk, dv, None, dpk, dpv) in the tensors' dtype.
    Mirrors sparse_indices_attn_res_scatter_bwd_v2 (triton/sparse_attention_res_1.py:403-471),
    including its unweighted pooled-key gradients unless set_exact_pooled_grad(True)."""
    kvw = token_weight if _exact_pooled_grad else 1.0
    dq, dk, dv, dpk, dpv, _, _ = _attn_bwd(do, q, k, v, pk, pv, None, None, o, m, indices, None, topk, 0, block_size,
                                           token_weight, 1.0, kvw, 1.0, False)
    return dq, dk, dv, None, dpk.to(pk.dtype), dpv.to(pv.dtype)


def sparse_indices_attn_res_scatter_2_2_bwd_v2(do, q, k, v, pk, pv, pk2, pv2, o, m, indices, prev_indices, topk, topk_p,
                                               block_size, token_weight, token_weight_2):
    """Two-level backward -> (dq, dk, dv, None, dpk, dpv, None, dpk2, dpv2).  Mirrors
    sparse_indices_attn_res_scatter_2_2_bwd_v2 (triton/sparse_attention_res_2.py:578-681)."""
    dq, dk, dv, dpk, dpv, dpk2, dpv2 = _attn_bwd(do, q, k, v, pk, pv, pk2, pv2, o, m, indices, prev_indices, topk, topk_p,
                                                 block_size, token_weight, token_weight_2, token_weight, token_weight_2, False)
    return dq, dk, dv, None, dpk.to(pk.dtype), dpv.to(pv.dtype), None, dpk2.to(pk2.dtype), dpv2.to(pv2.dtype)


# ----------------------------------------------------------------------------- operators with explicit pooled inputs
class _FlashSparseResidualAttentionL1(torch.autograd.Function):
    """torch_op/flash_sparse_attention_res_1.py:10-35."""

    @staticmethod
    def forward(ctx, q, k, v, pq, pk, pv, topk, token_weight=1, block_size=16):
        indices = _coarse_topk(pq, pk, topk)
        o, m = _attn_fwd(q, k, v, pk, pv, None, None, indices, None, topk, 0, block_size, token_weight, 1.0)
        ctx.save_for_backward(q, k, v, pk, pv, o, m, indices)
        ctx.topk, ctx.block_size, ctx.token_weight = topk, block_size, token_weight
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, pk, pv, o, m, indices = ctx.saved_tensors
        g = sparse_indices_attn_res_scatter_bwd_v2(do, q, k, v, pk, pv, o, m, indices, ctx.topk, ctx.block_size, ctx.token_weight)
        return (*g, None, None, None)


class _FlashSparseResidualAttentionL2(torch.autograd.Function):
    """torch_op/flash_sparse_attention_res_2.py:10-42."""

    @staticmethod
    def forward(ctx, q, k, v, pq, pk, pv, pq2, pk2, pv2, topk, topk2, token_weight=1, token_weight_2=1, block_size=16):
        indices, p_indices = _select_two_level(pq, pk, pq2, pk2, topk, topk2, block_size)
        o, m = _attn_fwd(q, k, v, pk, pv, pk2, pv2, indices, p_indices, topk, topk2, block_size, token_weight, token_weight_2)
        ctx.save_for_backward(q, k, v, pk, pv, pk2, pv2, o, m, indices, p_indices)
        ctx.cfg = (topk, topk2, block_size, token_weight, token_weight_2)
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, pk, pv, pk2, pv2, o, m, indices, p_indices = ctx.saved_tensors
        topk, topk2, bs, w1, w2 = ctx.cfg
        g = sparse_indices_attn_res_scatter_2_2_bwd_v2(do, q, k, v, pk, pv, pk2, pv2, o, m, indices, p_indices, topk, topk2, bs, w1, w2)
        return (*g, None, None, None, None, None)


flash_sparse_residual_attention_l1_op = _FlashSparseResidualAttentionL1.apply
flash_sparse_residual_attention_l2_op = _FlashSparseResidualAttentionL2.apply


# ----------------------------------------------------------------------------- fused drop-in operators
@torch.library.custom_op("llsa_b200::llsa_l1_fwd", mutates_args=())
def _llsa_l1_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, topk: int, block_size: int) -> List[torch.Tensor]:
    (pq, pk, pv), _ = pool_pyramid([q, k, v], block_size, 1)
    indices = _coarse_topk(pq, pk, topk)
    o, lse = _attn_fwd(q, k, v, pk, pv, None, None, indices, None, indices.shape[-1], 0, block_size, float(block_size), 1.0)
    return [o, lse, indices, pk, pv]


@_llsa_l1_fwd.register_fake
def _(q, k, v, topk, block_size):
    B, H, N, D = q.shape
    n1 = N // block_size
    return [torch.empty_like(q), q.new_empty((B, H, N), dtype=torch.float32), q.new_empty((B, H, n1, min(topk, n1)), dtype=torch.int32),
            k.new_empty((B, H, n1, D)), v.new_empty((B, H, n1, D))]


@torch.library.custom_op("llsa_b200::llsa_l1_bwd", mutates_args=())
def _llsa_l1_bwd(do: torch.Tensor, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, o: torch.Tensor, lse: torch.Tensor,
                 indices: torch.Tensor, pk: torch.Tensor, pv: torch.Tensor, block_size: int, exact: bool) -> List[torch.Tensor]:
    w = float(block_size)
    dq, dk, dv, _, _, _, _ = _attn_bwd(do, q, k, v, pk, pv, None, None, o, lse, indices, None, indices.shape[-1], 0, block_size,
                                       w, 1.0, w if exact else 1.0, 1.0, True)
    return [dq, dk, dv]


@_llsa_l1_bwd.register_fake
def _(do, q, k, v, o, lse, indices, pk, pv, block_size, exact):
    return [torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)]


def _l1_setup(ctx, inputs, output):
    q, k, v, topk, block_size = inputs
    o, lse, indices, pk, pv = output
    ctx.save_for_backward(q, k, v, o, lse, indices, pk, pv)
    ctx.block_size = block_size
    ctx.set_materialize_grads(False)       # only o carries a gradient: no zero-filled stand-ins for the other outputs


def _l1_backward(ctx, grads):
    if grads[0] is None:
        return None, None, None, None, None
    q, k, v, o, lse, indices, pk, pv = ctx.saved_tensors
    dq, dk, dv = _llsa_l1_bwd(grads[0], q, k, v, o, lse, indices, pk, pv, ctx.block_size, _exact_pooled_grad)
    return dq, dk, dv, None, None


_llsa_l1_fwd.register_autograd(_l1_backward, setup_context=_l1_setup)


@torch.library.custom_op("llsa_b200::llsa_l2_fwd", mutates_args=())
def _llsa_l2_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, topk1: int, topk2: int, block_size: int) -> List[torch.Tensor]:
    (pq, pk, pv), (pq2, pk2, pv2) = pool_pyramid([q, k, v], block_size, 2)
    indices, p_indices = _select_two_level(pq, pk, pq2, pk2, topk1, topk2, block_size)
    o, lse = _attn_fwd(q, k, v, pk, pv, pk2, pv2, indices, p_indices, topk1, p_indices.shape[-1], block_size,
                       float(block_size), float(block_size * block_size))
    return [o, lse, indices, p_indices, pk, pv, pk2, pv2]


@_llsa_l2_fwd.register_fake
def _(q, k, v, topk1, topk2, block_size):
    B, H, N, D = q.shape
    n1 = N // block_size
    n2 = n1 // block_size
    return [torch.empty_like(q), q.new_empty((B, H, N), dtype=torch.float32), q.new_empty((B, H, n1, topk1), dtype=torch.int32),
            q.new_empty((B, H, n2, min(topk2, n2)), dtype=torch.int32), k.new_empty((B, H, n1, D)), v.new_empty((B, H, n1, D)),
            k.new_empty((B, H, n2, D)), v.new_empty((B, H, n2, D))]


@torch.library.custom_op("llsa_b200::llsa_l2_bwd", mutates_args=())
def _llsa_l2_bwd(do: torch.Tensor, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, o: torch.Tensor, lse: torch.Tensor,
                 indices: torch.Tensor, p_indices: torch.Tensor, pk: torch.Tensor, pv: torch.Tensor, pk2: torch.Tensor,
                 pv2: torch.Tensor, block_size: int) -> List[torch.Tensor]:
    w1, w2 = float(block_size), float(block_size * block_size)
    dq, dk, dv, _, _, _, _ = _attn_bwd(do, q, k, v, pk, pv, pk2, pv2, o, lse, indices, p_indices, indices.shape[-1],
                                       p_indices.shape[-1], block_size, w1, w2, w1, w2, True)
    return [dq, dk, dv]


@_llsa_l2_bwd.register_fake
def _(do, q, k, v, o, lse, indices, p_indices, pk, pv, pk2, pv2, block_size):
    return [torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)]


def _l2_setup(ctx, inputs, output):
    q, k, v, topk1, topk2, block_size = inputs
    o, lse, indices, p_indices, pk, pv, pk2, pv2 = output
    ctx.save_for_backward(q, k, v, o, lse, indices, p_indices, pk, pv, pk2, pv2)
    ctx.block_size = block_size
    ctx.set_materialize_grads(False)


def _l2_backward(ctx, grads):
    if grads[0] is None:
        return None, None, None, None, None, None
    q, k, v, o, lse, indices, p_indices, pk, pv, pk2, pv2 = ctx.saved_tensors
    dq, dk, dv = _llsa_l2_bwd(grads[0], q, k, v, o, lse, indices, p_indices, pk, pv, pk2, pv2, ctx.block_size)
    return dq, dk, dv, None, None, None


_llsa_l2_fwd.register_autograd(_l2_backward, setup_context=_l2_setup)


# ----------------------------------------------------------------------------- RoPE fused in front of the operators
@torch.library.custom_op("llsa_b200::llsa_rope_fwd", mutates_args=())
def _llsa_rope_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, freq: torch.Tensor, topk1: int, topk2: int, block_size: int,
                   levels: int) -> List[torch.Tensor]:
    (qr, kr, _), l1, l2 = rope_pool_pyramid([q, k, v], freq, [True, True, False], block_size, levels)
    pq, pk, pv = l1
    bs = block_size
    if levels == 2:
        pq2, pk2, pv2 = l2
        indices, p_indices = _select_two_level(pq, pk, pq2, pk2, topk1, topk2, bs)
        o, lse = _attn_fwd(qr, kr, v, pk, pv, pk2, pv2, indices, p_indices, topk1, p_indices.shape[-1], bs, float(bs), float(bs * bs))
        return [o, lse, qr, kr, indices, pk, pv, p_indices, pk2, pv2]
    indices = _coarse_topk(pq, pk, topk1)
    o, lse = _attn_fwd(qr, kr, v, pk, pv, None, None, indices, None, indices.shape[-1], 0, bs, float(bs), 1.0)
    return [o, lse, qr, kr, indices, pk, pv]


@_llsa_rope_fwd.register_fake
def _(q, k, v, freq, topk1, topk2, block_size, levels):
    B, H, N, D = q.shape
    n1 = N // block_size
    n2 = n1 // block_size
    out = [torch.empty_like(q), q.new_empty((B, H, N), dtype=torch.float32), torch.empty_like(q), torch.empty_like(k),
           q.new_empty((B, H, n1, min(topk1, n1) if levels == 1 else topk1), dtype=torch.int32), k.new_empty((B, H, n1, D)), v.new_empty((B, H, n1, D))]
    if levels == 2:
        out += [q.new_empty((B, H, n2, min(topk2, n2)), dtype=torch.int32), k.new_empty((B, H, n2, D)), v.new_empty((B, H, n2, D))]
    return out


def _rope_op_setup(ctx, inputs, output):
    q, k, v, freq, topk1, topk2, block_size, levels = inputs
    ctx.save_for_backward(v, freq, *output)
    ctx.block_size, ctx.levels = block_size, levels
    ctx.set_materialize_grads(False)


def _rope_op_backward(ctx, grads):
    if grads[0] is None:
        return (None,) * 8
    v, freq, o, lse, qr, kr, indices, pk, pv = ctx.saved_tensors[:9]
    if ctx.levels == 2:
        p_indices, pk2, pv2 = ctx.saved_tensors[9:]
        dqr, dkr, dv = _llsa_l2_bwd(grads[0], qr, kr, v, o, lse, indices, p_indices, pk, pv, pk2, pv2, ctx.block_size)
    else:
        dqr, dkr, dv = _llsa_l1_bwd(grads[0], qr, kr, v, o, lse, indices, pk, pv, ctx.block_size, _exact_pooled_grad)
    return _rope_bwd_op(dqr, freq), _rope_bwd_op(dkr, freq), dv, None, None, None, None, None


_llsa_rope_fwd.register_autograd(_rope_op_backward, setup_context=_rope_op_setup)


def llsa_l1_rope(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, freq: torch.Tensor, topk: int = 8, block_size: int = 16) -> torch.Tensor:
    """llsa_l1(my_rope_fn(q, freq), my_rope_fn(k, freq), v, topk, block_size) -- what RopeAttnProcessor computes
    (models/rope_dit_transformer_2d.py:232-241) -- with the rotation fused into the pooling pass."""
    return _llsa_rope_fwd(q, k, v, freq, topk, 0, block_size, 1)[0]


def llsa_l2_rope(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, freq: torch.Tensor, topk1: int = 8, topk2: int = 8,
                 block_size: int = 16) -> torch.Tensor:
    """llsa_l2(my_rope_fn(q, freq), my_rope_fn(k, freq), v, topk1, topk2, block_size)
    (models/rope_dit_transformer_2d.py:232-251) with the rotation fused into the pooling pass."""
    return _llsa_rope_fwd(q, k, v, freq, topk1, topk2, block_size, 2)[0]


class _LlsaRmsRope(torch.autograd.Function):
    """llsa_l1 / llsa_l2 on RMS-normalised, rotated q and k: normalisation, rotation and pooling in one pass forward; the
    backward runs the operator's backward, then the rotation's and the normalisation's."""

    @staticmethod
    def forward(ctx, q, k, v, wq, wk, freq, eps, topk1, topk2, block_size, levels):
        bs = block_size
        (qr, kr, _), l1, l2 = rms_rope_pool_pyramid([q.detach(), k.detach(), v.detach()], [wq, wk, None], eps, freq, [True, True, False], bs, levels)
        pq, pk, pv = l1
        vd = v.detach()
        if levels == 2:
            pq2, pk2, pv2 = l2
            indices, p_indices = _select_two_level(pq, pk, pq2, pk2, topk1, topk2, bs)
            o, lse = _attn_fwd(qr, kr, vd, pk, pv, pk2, pv2, indices, p_indices, topk1, p_indices.shape[-1], bs, float(bs), float(bs * bs))
            extra = [p_indices, pk2, pv2]
        else:
            indices = _coarse_topk(pq, pk, topk1)
            o, lse = _attn_fwd(qr, kr, vd, pk, pv, None, None, indices, None, indices.shape[-1], 0, bs, float(bs), 1.0)
            extra = []
        ctx.save_for_backward(q, k, v, wq, wk, freq, o, lse, qr, kr, indices, pk, pv, *extra)
        ctx.cfg = (float(eps), bs, levels)
        return o

    @staticmethod
    def backward(ctx, do):
        eps, bs, levels = ctx.cfg
        q, k, v, wq, wk, freq, o, lse, qr, kr, indices, pk, pv = ctx.saved_tensors[:13]
        if levels == 2:
            p_indices, pk2, pv2 = ctx.saved_tensors[13:]
            dqr, dkr, dv = _llsa_l2_bwd(do, qr, kr, v, o, lse, indices, p_indices, pk, pv, pk2, pv2, bs)
        else:
            dqr, dkr, dv = _llsa_l1_bwd(do, qr, kr, v, o, lse, indices, pk, pv, bs, _exact_pooled_grad)
        dq, dwq = _rms_norm_bwd(q, wq, eps, _rope_bwd_op(dqr, freq))
        dk, dwk = _rms_norm_bwd(k, wk, eps, _rope_bwd_op(dkr, freq))
        return dq, dk, dv, dwq, dwk, None, None, None, None, None, None


def llsa_l1_rms_rope(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, wq: torch.Tensor, wk: torch.Tensor, freq: torch.Tensor,
                     eps: float = 1e-5, topk: int = 8, block_size: int = 16) -> torch.Tensor:
    """llsa_l1(my_rope_fn(norm_q(q)), my_rope_fn(norm_k(k)), v, topk, block_size): the whole q / k preparation of the attention
    block (models/rope_dit_transformer_2d.py:215-241) fused into the pooling pass.  wq, wk: RMSNorm weights [D]."""
    return _LlsaRmsRope.apply(q, k, v, wq, wk, freq, eps, topk, 0, block_size, 1)


def llsa_l2_rms_rope(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, wq: torch.Tensor, wk: torch.Tensor, freq: torch.Tensor,
                     eps: float = 1e-5, topk1: int = 8, topk2: int = 8, block_size: int = 16) -> torch.Tensor:
    """llsa_l2 on RMS-normalised, rotated q and k (models/rope_dit_transformer_2d.py:215-251), q / k read once."""
    return _LlsaRmsRope.apply(q, k, v, wq, wk, freq, eps, topk1, topk2, block_size, 2)


def llsa_l1(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, topk: int = 8, block_size: int = 16) -> torch.Tensor:
    """One-level log-linear sparse attention; q, k, v [B,H,N,D] (any batch/head/token
    strides), returns o like q; differentiable in q, k, v.  Drop-in for llsa_l1
    (torch_op/flash_sparse_attention_res_1.py:41-47)."""
    return _llsa_l1_fwd(q, k, v, topk, block_size)[0]


def llsa_l2(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, topk1: int = 8, topk2: int = 8, block_size: int = 16) -> torch.Tensor:
    """Two-level log-linear sparse attention.  Drop-in for llsa_l2
    (torch_op/flash_sparse_attention_res_2.py:48-59)."""
    return _llsa_l2_fwd(q, k, v, topk1, topk2, block_size)[0]


def llsa_l1_debug(q, k, v, topk=8, block_size=16):
    """llsa_l1 returning its intermediates: dict(o, lse, indices, pk, pv)."""
    o, lse, indices, pk, pv = _llsa_l1_fwd(q, k, v, topk, block_size)
    return dict(o=o, lse=lse, indices=indices, pk=pk, pv=pv)


def llsa_l2_debug(q, k, v, topk1=8, topk2=8, block_size=16):
    """llsa_l2 returning its intermediates: dict(o, lse, indices, p_indices, pk, pv, pk2, pv2)."""
    o, lse, indices, p_indices, pk, pv, pk2, pv2 = _llsa_l2_fwd(q, k, v, topk1, topk2, block_size)
    return dict(o=o, lse=lse, indices=indices, p_indices=p_indices, pk=pk, pv=pv, pk2=pk2, pv2=pv2)
