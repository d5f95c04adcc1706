"""B200 (sm_100a) implementation of the Qwen3.5 decoder hot path of ax-dsl-kernels: MoE block, paged flash attention
and gated delta net, behind the reference's runtime-weight, tensors-by-name kernel interface.

Host code is a thin Python layer over the C ABI in include/q35b200.h (libq35b200.so, hand-written CUDA).  There is no
CPU path and no fallback: without the built library every call raises.
"""
from . import _lib, layers, packs, speculative  # noqa: F401
from ._lib import Q35Error, device_status, io_table, roles, run, workspace_bytes  # noqa: F401
from .attention import (kv_write, mrope_cos_sin, paged_attention_decode, paged_attention_prefill,  # noqa: F401
                        rope_cos_sin)
from .gdn import gdn_chunk_prefill, gdn_conv1d_silu, gdn_recurrent_step  # noqa: F401
from .moe import (linear, moe_block, moe_combine, moe_experts, moe_permute, moe_pre, moe_slots_px,  # noqa: F401
                  prepare_moe_weights, qwen3_moe, route, tile_scales)

__all__ = ["run", "roles", "io_table", "workspace_bytes", "device_status", "Q35Error", "route", "moe_pre",
           "moe_experts", "moe_slots_px", "moe_combine", "moe_permute", "moe_block", "qwen3_moe", "prepare_moe_weights", "tile_scales", "linear",
           "paged_attention_decode", "paged_attention_prefill", "kv_write", "gdn_recurrent_step", "gdn_conv1d_silu", "gdn_chunk_prefill"]
