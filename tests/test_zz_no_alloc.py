"""GPU test of llsa_transpose_indices_noalloc, the index transpose for hosts that
cannot allocate device memory themselves (a process whose device memory is
owned by its own arena, or a plugin runtime that only hands buffers across).

It is called through the C ABI exactly as such a host would: inputs and outputs
are caller buffers, no scratch pointer is passed.  Its results must equal,
bit for bit, those of llsa_transpose_indices given caller scratch (both run the
same stable counting sort) on two calls in a row: the second call finds the
built-in scratch dirty from the first and must still be right.  The shape is
a long-sequence one (n_kv = 16384 KV blocks) where the regular entry point does
need scratch.  This file sorts last so that a `-x` run has executed every other
test before it.
"""
import ctypes as C

import pytest
import torch

from llsa_b200 import _lib
from oracle import llsa_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _case(seed, B=1, H=2, M=16384, T=8):
    gen = torch.Generator().manual_seed(seed)
    hot = torch.randint(0, M // 64, (B, H, M, T // 2), generator=gen)        # skewed: hot buckets and empty ones
    cold = torch.randint(0, M, (B, H, M, T - T // 2), generator=gen)
    return torch.cat([hot, cold], -1).to(torch.int32)


def _regular(idx, n_kv):
    lib = _lib.lib()
    B, H, M, T = idx.shape
    off = torch.empty((B, H, n_kv + 1), device=idx.device, dtype=torch.int64)
    flat = torch.empty((B, H, M * T), device=idx.device, dtype=torch.int32)
    nbytes = lib.llsa_transpose_scratch_bytes(B, H, M, T, n_kv)
    assert nbytes > 0, "this shape is meant to need scratch in the regular entry point"
    scratch = torch.empty((nbytes,), device=idx.device, dtype=torch.uint8)
    a, b, c = _lib.desc(idx), _lib.desc(off), _lib.desc(flat)
    rc = lib.llsa_transpose_indices(C.byref(a), C.byref(b), C.byref(c), n_kv, C.c_void_p(scratch.data_ptr()), nbytes, None,
                                    _lib.stream_ptr(idx.device))
    _lib.check(rc, "transpose_indices")
    return off, flat


def _noalloc(idx, n_kv, off, flat):
    """off / flat are caller-provided outputs; nothing else is handed over."""
    lib = _lib.lib()
    a, b, c = _lib.desc(idx), _lib.desc(off), _lib.desc(flat)
    return lib.llsa_transpose_indices_noalloc(C.byref(a), C.byref(b), C.byref(c), n_kv, None, _lib.stream_ptr(idx.device))


def test_noalloc_transpose_equals_regular_on_two_calls_in_a_row():
    lib = _lib.lib()
    n_kv = 16384
    cases = [_case(101).to(DEV), _case(202).to(DEV)]
    outs = [(torch.empty((1, 2, n_kv + 1), device=DEV, dtype=torch.int64), torch.empty((1, 2, n_kv * 8), device=DEV, dtype=torch.int32))
            for _ in cases]
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated()
    for idx, (off, flat) in zip(cases, outs):          # back to back on one stream, no allocation in between
        rc = _noalloc(idx, n_kv, off, flat)
        assert rc == 0, lib.llsa_last_error_string().decode()
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == before
    for idx, (off, flat) in zip(cases, outs):
        want_off, want_flat = _regular(idx, n_kv)
        assert torch.equal(off, want_off)
        assert torch.equal(flat, want_flat)
        assert int(off[..., -1].min()) == n_kv * 8
        # ... and the CPU oracle's lists (indices_transpose.py:104-109, buckets ascending), so that the entry point is pinned to the
        # reference's semantics and not only to its sibling
        o_off, o_flat = O.transpose_indices(idx.cpu())
        assert torch.equal(off.cpu(), o_off) and torch.equal(flat.cpu().long(), o_flat)
    # the same input again, after the other case dirtied the scratch: identical bits
    off2, flat2 = torch.empty_like(outs[0][0]), torch.empty_like(outs[0][1])
    assert _noalloc(cases[0], n_kv, off2, flat2) == 0
    torch.cuda.synchronize()
    assert torch.equal(off2, outs[0][0]) and torch.equal(flat2, outs[0][1])


def test_noalloc_transpose_refuses_what_does_not_fit():
    lib = _lib.lib()
    # B*H*32*n_kv*2 = 8 heads * 32 * 32768 * 2 = 16 MiB > the 8 MiB built in
    idx = torch.zeros((1, 8, 32768, 2), device=DEV, dtype=torch.int32)
    off = torch.empty((1, 8, 32769), device=DEV, dtype=torch.int64)
    flat = torch.empty((1, 8, 65536), device=DEV, dtype=torch.int32)
    assert _noalloc(idx, 32768, off, flat) == 6          # LLSA_ERR_WORKSPACE
    assert b"built-in scratch" in lib.llsa_last_error_string()
