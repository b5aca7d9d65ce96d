"""come_b200 -- B200 (sm_100a) kernels for the Co-Me accelerated-inference hot path.

Host side in Python/PyTorch (device memory, streams), compute in ``libcome_b200.so`` behind a C ABI
(``include/come_b200.h``).  The modules mirror the operator surface of the reference project:

* :mod:`come_b200.co_me_cuext`          -- ``co_me_token_merge_cuda`` / ``co_me_token_split_cuda``
* :mod:`come_b200.flash_attn_fwd_cuda`  -- ``varlen_fwd`` / ``varlen_fwd_w_perkey_bias``
* :mod:`come_b200.flash_attn`           -- ``flash_attn_varlen_qkvpacked_func[_w_perkey_bias]``
* :mod:`come_b200.cuda_extension`       -- stands in for the reference's ``src.cuda_extension`` package
* :mod:`come_b200.qkv`                  -- ``prepare_packed_self_attention_qkv`` (q/k LayerNorm + 2-D RoPE + bias in
  one kernel), ``RotaryPositionEmbedding2D``
* :mod:`come_b200.token_merger`         -- ``JaggedTokens``, ``func_token_merge[_2d]``, ``func_token_split``,
  ``MergePlan`` (merge, split, ``merge_layernorm``, ``split_add``, ``split_concat``, ``positions``), ``select_windows``
  and the 2-D merger class
* :mod:`come_b200.bias_attention`       -- ``JaggedAttention_w_Bias`` (the reference's attention wrapper module)
* :mod:`come_b200.plain_attention`      -- ``JaggedAttention`` (the same without the count bias)
* :mod:`come_b200.block`                -- ``JaggedBlock`` / ``JaggedBlock_w_Bias`` and the block with LayerScale + residual
  add + LayerNorm fused (``residual_layernorm``, ``forward_fused``)
* :mod:`come_b200.fused`                -- ``FusedAggregator``: the merged forward pass of the alternating-attention
  stack, ``CapturedForward``: its CUDA-graph replay, ``ShardedFusedAggregator``: one scene sharded by frame over GPUs
* :mod:`come_b200.timer`                -- ``Timer`` (named CUDA-event ranges and their percentile table)
* :mod:`come_b200.vggt_arch`            -- seeded random VGGT-shaped blocks for tests and benchmarks
* :mod:`come_b200.direct`               -- ``DirectAttention``: the per-layer replacement of ``block.attn.forward``
* :mod:`come_b200.chain`                -- the standalone operator chain of a scene, also sharded by frame over GPUs
* :mod:`come_b200.static_scene`         -- the chain as one CUDA graph with no device-to-host read
* :mod:`come_b200.dist`                 -- frame / row sharding helpers, the K/V row all-gather, ``GlobalExchange``
"""
from . import _lib  # noqa: F401

__version__ = "0.1.0"
