"""Makes `import llsa.kernel...` resolve to this package.

The reference's model imports its operators by module path
(models/rope_dit_transformer_2d.py:35-38):

    from llsa.kernel.torch_op.flash_sparse_attention_res_1 import llsa_l1
    from llsa.kernel.torch_op.flash_sparse_attention_res_2 import llsa_l2
    from llsa.kernel.triton.mean_pool import mean_pool1d
    from llsa.kernel.triton.rope import my_rope_fn

install_reference_shims() registers modules of those names in sys.modules whose
attributes are this package's functions, so the model code runs unmodified on
the B200 kernels.  Call it before the model module is imported.
"""
from __future__ import annotations

import sys
import types


def install_reference_shims(force: bool = False) -> None:
    from . import ops

    table = {
        "llsa.kernel.torch_op.flash_sparse_attention_res_1": dict(
            llsa_l1=ops.llsa_l1, flash_sparse_residual_attention_l1_op=ops.flash_sparse_residual_attention_l1_op,
            FlashSparseResidualAttentionL1=ops._FlashSparseResidualAttentionL1),
        "llsa.kernel.torch_op.flash_sparse_attention_res_2": dict(
            llsa_l2=ops.llsa_l2, flash_sparse_residual_attention_l2_op=ops.flash_sparse_residual_attention_l2_op,
            FlashSparseResidualAttentionL2=ops._FlashSparseResidualAttentionL2),
        "llsa.kernel.triton.mean_pool": dict(mean_pool1d=ops.mean_pool1d),
        "llsa.kernel.triton.rope": dict(my_rope_fn=ops.my_rope_fn),
        "llsa.kernel.triton.topk": dict(gen_sparse_indices=ops.gen_sparse_indices,
                                        compute_topk_indices_sparse=ops.compute_topk_indices_sparse),
        "llsa.kernel.triton.indices_transpose": dict(transpose_indices=ops.transpose_indices),
        "llsa.kernel.triton.sparse_attention_res_1": dict(
            sparse_indices_attn_res_fwd=ops.sparse_indices_attn_res_fwd,
            sparse_indices_attn_res_scatter_bwd_v2=ops.sparse_indices_attn_res_scatter_bwd_v2),
        "llsa.kernel.triton.sparse_attention_res_2": dict(
            sparse_indices_attn_res_2_2_fwd=ops.sparse_indices_attn_res_2_2_fwd,
            sparse_indices_attn_res_scatter_2_2_bwd_v2=ops.sparse_indices_attn_res_scatter_2_2_bwd_v2),
    }
    for name in ("llsa", "llsa.kernel", "llsa.kernel.torch_op", "llsa.kernel.triton"):
        if name not in sys.modules:
            m = types.ModuleType(name)
            m.__path__ = []          # a package
            sys.modules[name] = m
    for name, attrs in table.items():
        if name in sys.modules and not force:
            continue
        m = types.ModuleType(name)
        m.__dict__.update(attrs)
        sys.modules[name] = m
        parent, _, leaf = name.rpartition(".")
        setattr(sys.modules[parent], leaf, m)
    for name in ("llsa.kernel", "llsa.kernel.torch_op", "llsa.kernel.triton"):
        parent, _, leaf = name.rpartition(".")
        setattr(sys.modules[parent], leaf, sys.modules[name])
