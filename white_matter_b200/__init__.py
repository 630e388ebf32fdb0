"""B200 (sm_100a) kernels for the WhiteMatter attention hot path.

Public names match ``white_matter.ops`` of the upstream project; the kernels
live in ``libwm_b200.so`` behind the C ABI of ``include/wm_b200.h``.
"""

from .cyclic import cyclic_attention
from .cyclic_prefill import FeedbackBlock
from .decode_step import DecodeStepGraph, KVPoolCache, document_key_mask
from .metadata import (
    CyclicAttentionMetadata,
    StrictCausalMetadata,
    prepare_cyclic_attention_metadata,
    prepare_feedback_metadata,
    prepare_strict_causal_metadata,
)
from .kv_pool import KVPool
from .layer import cyclic_attention_layer, prepare_queries
from .mixing import mix_kv_sources, mixed_pool_decode
from .strict import strict_causal_attention

__all__ = [
    "prepare_queries",
    "cyclic_attention_layer",
    "StrictCausalMetadata",
    "prepare_strict_causal_metadata",
    "strict_causal_attention",
    "CyclicAttentionMetadata",
    "cyclic_attention",
    "prepare_cyclic_attention_metadata",
    "prepare_feedback_metadata",
    "mix_kv_sources",
    "mixed_pool_decode",
    "FeedbackBlock",
    "KVPool",
    "KVPoolCache",
    "DecodeStepGraph",
    "document_key_mask",
]
