"""llsa_b200 -- the LLSA (log-linear sparse attention) hot path for NVIDIA B200.

`llsa_l1(q, k, v, topk, block_size)` and `llsa_l2(q, k, v, topk1, topk2, block_size)`
keep the signatures, autograd behaviour and [B,H,N,D] layout of
SingleZombie/LLSA's operators and run hand-written sm_100a CUDA kernels through
the C ABI in include/llsa_b200.h.  There is no CPU or Triton fallback.
"""
from .ops import (compute_topk_indices_sparse, flash_sparse_residual_attention_l1_op,  # noqa: F401
                  flash_sparse_residual_attention_l2_op, gen_sparse_indices, llsa_l1, llsa_l1_debug, llsa_l1_rope, llsa_l2, llsa_l2_rope, rope_pool_pyramid, rms_norm, rms_rope_pool_pyramid, llsa_l1_rms_rope, llsa_l2_rms_rope,
                  llsa_l2_debug, mean_pool1d, my_rope_fn, pool_pyramid, set_device_checks, set_exact_pooled_grad,
                  sparse_indices_attn_res_2_2_fwd, sparse_indices_attn_res_fwd,
                  sparse_indices_attn_res_scatter_2_2_bwd_v2, sparse_indices_attn_res_scatter_bwd_v2,
                  transpose_indices)
from .hostpipe import HostPipeline, capture_fwd_bwd  # noqa: F401
from .shims import install_reference_shims  # noqa: F401

__version__ = "0.1.0"
