"""CPU-side checks of the C ABI: the shared library loads, exports every entry
point include/llsa_b200.h declares, and rejects bad arguments with the
documented status codes before touching the GPU (no kernel is launched here)."""
import ctypes as C
import os
import re

import pytest
import torch

from llsa_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "llsa_b200.h")

OK, ERR_NULL, ERR_DTYPE, ERR_SHAPE, ERR_STRIDE, ERR_ARG, ERR_WORKSPACE = 0, 1, 2, 3, 4, 5, 6


def declared_functions():
    src = open(HEADER).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(llsa_[a-z0-9_]+)\s*\(", src)))


def fake(shape, dtype=torch.bfloat16, strides=None, ptr=0x10000):
    """A tensor descriptor with a non-null fake device pointer (never dereferenced on the host)."""
    t = torch.empty(shape, dtype=dtype) if strides is None else torch.empty_strided(shape, strides, dtype=dtype)
    d = _lib.desc(t)
    d.ptr = ptr
    return d


def test_header_and_binding_agree():
    names = declared_functions()
    assert names, "no declarations found in the header"
    assert sorted(_lib.EXPORTS) == names


def test_library_exports_every_declared_symbol():
    lib = _lib.lib()
    for name in declared_functions():
        assert hasattr(lib, name), "missing export %s" % name
    assert lib.llsa_version() >= 100
    assert isinstance(lib.llsa_last_error_string(), bytes)


def test_struct_layout_matches_header(tmp_path):
    """The ctypes mirrors of LlsaTensor / LlsaAttnArgs against what a C compiler makes of the header itself."""
    import shutil
    import subprocess
    assert C.sizeof(_lib.LlsaTensor) == 8 + 4 + 4 + 32 + 32
    cc = shutil.which("gcc") or shutil.which("cc")
    if cc is None:
        pytest.skip("no C compiler")
    fields = [name for name, _ in _lib.LlsaAttnArgs._fields_]
    src = tmp_path / "layout.c"
    src.write_text('#include <stdio.h>\n#include <stddef.h>\n#include "llsa_b200.h"\nint main(void) {\n'
                   '  printf("%zu %zu\\n", sizeof(LlsaTensor), sizeof(LlsaAttnArgs));\n' +
                   "".join('  printf("%s %%zu\\n", offsetof(LlsaAttnArgs, %s));\n' % (f, f) for f in fields) + "  return 0;\n}\n")
    exe = tmp_path / "layout"
    subprocess.run([cc, "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe)], check=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split("\n")
    st, sa = [int(x) for x in out[0].split()]
    assert st == C.sizeof(_lib.LlsaTensor) and sa == C.sizeof(_lib.LlsaAttnArgs)
    for line in out[1:]:
        if line.strip():
            name, off = line.split()
            assert getattr(_lib.LlsaAttnArgs, name).offset == int(off), name


def test_pool_argument_errors():
    lib = _lib.lib()
    x, y = fake((1, 2, 64, 64)), fake((1, 2, 4, 64))
    assert lib.llsa_mean_pool_fwd(None, C.byref(y), 16, None) == ERR_NULL
    assert b"null" in lib.llsa_last_error_string()
    assert lib.llsa_mean_pool_fwd(C.byref(x), C.byref(y), 7, None) == ERR_ARG           # 64 % 7 != 0
    assert lib.llsa_mean_pool_fwd(C.byref(x), C.byref(fake((1, 2, 4, 64), torch.float32)), 16, None) == ERR_DTYPE
    assert lib.llsa_mean_pool_fwd(C.byref(x), C.byref(fake((1, 2, 5, 64))), 16, None) == ERR_SHAPE
    assert lib.llsa_mean_pool_fwd(C.byref(fake((1, 2, 64, 64), torch.int32)), C.byref(y), 16, None) == ERR_DTYPE
    xs = fake((1, 2, 64, 64), strides=(2 * 64 * 128, 64 * 128, 128, 2))                  # channel stride 2
    assert lib.llsa_mean_pool_fwd(C.byref(xs), C.byref(y), 16, None) == ERR_STRIDE
    arr = (_lib.LlsaTensor * 1)(x)
    y1 = (_lib.LlsaTensor * 1)(y)
    assert lib.llsa_pool_pyramid_fwd(4, arr, y1, None, 16, None) == ERR_ARG
    assert lib.llsa_pool_pyramid_fwd(1, arr, (_lib.LlsaTensor * 1)(fake((1, 2, 8, 64))), None, 16, None) == ERR_SHAPE
    odd = (_lib.LlsaTensor * 1)(fake((1, 2, 64, 64), ptr=0x10008))                       # rows not 16-byte aligned
    assert lib.llsa_pool_pyramid_fwd(1, odd, y1, None, 16, None) == ERR_STRIDE


def test_topk_and_transpose_argument_errors():
    lib = _lib.lib()
    pq, pk = fake((1, 1, 64, 64)), fake((1, 1, 64, 64))
    idx = fake((1, 1, 64, 8), torch.int32)
    assert lib.llsa_coarse_topk(C.byref(pq), C.byref(pk), C.byref(fake((1, 1, 64, 8), torch.float32)), 8, None) == ERR_DTYPE
    assert lib.llsa_coarse_topk(C.byref(pq), C.byref(pk), C.byref(idx), 65, None) == ERR_ARG
    assert lib.llsa_coarse_topk(C.byref(pq), C.byref(fake((1, 1, 64, 64), torch.float32)), C.byref(idx), 8, None) == ERR_DTYPE
    assert lib.llsa_coarse_topk(C.byref(pq), C.byref(pk), C.byref(fake((1, 1, 64, 4), torch.int32)), 8, None) == ERR_SHAPE
    pidx = fake((1, 1, 4, 8), torch.int64)
    assert lib.llsa_refine_topk(C.byref(pq), C.byref(pk), C.byref(pidx), C.byref(idx), 8, 8, 15, None) == ERR_ARG
    assert lib.llsa_refine_topk(C.byref(pq), C.byref(pk), C.byref(pidx), C.byref(idx), 8, 2, 16, None) == ERR_SHAPE   # p_idx shape
    off, flat = fake((1, 1, 65), torch.int64), fake((1, 1, 512), torch.int32)
    assert lib.llsa_transpose_indices(C.byref(idx), C.byref(off), C.byref(fake((1, 1, 512), torch.int64)), 64, None, 0, None, None) == ERR_DTYPE
    assert lib.llsa_transpose_indices(C.byref(idx), C.byref(fake((1, 1, 64), torch.int64)), C.byref(flat), 64, None, 0, None, None) == ERR_SHAPE
    # a key range too large for shared memory needs caller scratch
    big_idx, big_off, big_flat = fake((1, 1, 32768, 8), torch.int32), fake((1, 1, 32769), torch.int64), fake((1, 1, 262144), torch.int32)
    need = lib.llsa_transpose_scratch_bytes(1, 1, 32768, 8, 32768)
    assert need == 32 * 32768 * 2
    assert lib.llsa_transpose_indices(C.byref(big_idx), C.byref(big_off), C.byref(big_flat), 32768, None, 0, None, None) == ERR_WORKSPACE
    assert lib.llsa_transpose_scratch_bytes(8, 6, 1024, 8, 1024) == 0


def test_attention_argument_errors():
    lib = _lib.lib()
    B, H, N, D = 1, 2, 1024, 64
    t = dict(q=fake((B, H, N, D)), k=fake((B, H, N, D)), v=fake((B, H, N, D)), o=fake((B, H, N, D)),
             pk=fake((B, H, N // 16, D)), pv=fake((B, H, N // 16, D)), lse=fake((B, H, N), torch.float32),
             indices=fake((B, H, N // 16, 8), torch.int32))

    def args(**over):
        a = _lib.LlsaAttnArgs()
        d = dict(t)
        d.update(over)
        for name, val in d.items():
            setattr(a, name, _lib.ptr(val))
        a.topk, a.topk_p, a.block_size = 8, 0, 16
        a.token_weight, a.token_weight_2 = 16.0, 1.0
        a._keep = d
        return a

    assert lib.llsa_attn_fwd(None, None) == ERR_NULL
    assert lib.llsa_attn_fwd(C.byref(args(q=None)), None) == ERR_NULL
    assert lib.llsa_attn_fwd(C.byref(args(q=fake((B, H, N, 32)))), None) == ERR_SHAPE            # head dim
    assert lib.llsa_attn_fwd(C.byref(args(k=fake((B, H, N, D), torch.float32))), None) == ERR_DTYPE
    assert lib.llsa_attn_fwd(C.byref(args(lse=fake((B, H, N)))), None) == ERR_DTYPE
    assert lib.llsa_attn_fwd(C.byref(args(pk=fake((B, H, N // 16, D), strides=(2 * 64 * 128, 64 * 128, 128, 1)))), None) == ERR_STRIDE
    a = args()
    a.block_size = 32
    assert lib.llsa_attn_fwd(C.byref(a), None) == ERR_ARG
    a = args()
    a.topk = 7
    assert lib.llsa_attn_fwd(C.byref(a), None) == ERR_ARG
    # the forward's optional one-byte-per-row scratch: one I32 element per four query rows at least
    assert lib.llsa_attn_fwd(C.byref(args(fwd_redo=fake((B * H * N // 4 - 1,), torch.int32))), None) == ERR_WORKSPACE
    assert lib.llsa_attn_fwd(C.byref(args(fwd_redo=fake((B * H * N // 4,), torch.float32))), None) == ERR_WORKSPACE
    # backward without its outputs
    assert lib.llsa_attn_bwd(C.byref(args()), None) == ERR_NULL
    # two-level form without p_indices
    assert lib.llsa_attn_fwd(C.byref(args(pk2=fake((B, H, N // 256, D)))), None) == ERR_NULL


def test_ops_refuse_cpu_tensors():
    import llsa_b200
    x = torch.randn(1, 1, 1024, 64)
    for call in (lambda: llsa_b200.llsa_l1(x, x, x), lambda: llsa_b200.llsa_l2(x, x, x), lambda: llsa_b200.mean_pool1d(x, 16),
                 lambda: llsa_b200.transpose_indices(torch.zeros(1, 1, 4, 2, dtype=torch.int32))):
        with pytest.raises(RuntimeError, match="CUDA"):
            call()


def test_reference_import_paths_resolve_to_this_package():
    import sys
    import llsa_b200
    saved = {k: v for k, v in sys.modules.items() if k == "llsa" or k.startswith("llsa.")}
    try:
        for k in saved:
            del sys.modules[k]
        llsa_b200.install_reference_shims()
        from llsa.kernel.torch_op.flash_sparse_attention_res_1 import llsa_l1
        from llsa.kernel.torch_op.flash_sparse_attention_res_2 import llsa_l2
        from llsa.kernel.triton.mean_pool import mean_pool1d
        from llsa.kernel.triton.rope import my_rope_fn
        assert llsa_l1 is llsa_b200.llsa_l1 and llsa_l2 is llsa_b200.llsa_l2
        assert mean_pool1d is llsa_b200.mean_pool1d and my_rope_fn is llsa_b200.my_rope_fn
    finally:
        for k in [k for k in sys.modules if k == "llsa" or k.startswith("llsa.")]:
            del sys.modules[k]
        sys.modules.update(saved)


def test_bwd_partial_scratch_size():
    L = _lib.lib()
    assert L.llsa_transpose_range_entries(8, 6, 1024, 8) == 32 and L.llsa_transpose_range_entries(1, 6, 1024, 8) == 16
    assert L.llsa_attn_bwd_partial_elems(8, 6, 16384, 8) == 8 * 6 * (8192 // 16 // 4) * 4096     # sized for 16-entry ranges, four per CTA
    assert L.llsa_attn_bwd_partial_elems(1, 1, 256, 8) == 2 * 4096
    assert L.llsa_attn_bwd_pds_elems(1, 1, 256, 8) == 16 * 8 * 256                  # 1 KB per (query block, selected block) pair
    assert L.llsa_attn_bwd_partial_elems(0, 6, 16384, 8) == 0
