"""B200-native (sm_100a) GQA decode attention: a drop-in for the public API of
alityb/gqa-decode (``gqa_decode``), backed by hand-written CUDA kernels behind a C ABI."""
from .gqa_decode import (
    GQADecodeConfig,
    gqa_decode_attention,
    gqa_decode_attention_batched,
    gqa_decode_attention_fp8,
    gqa_decode_attention_persistent,
    merge_partials,
    plan_decode,
    DecodePlan,
    read_status,
    reduce_partials,
    reference_gqa_decode,
    reset_workspace,
    select_num_splits,
    workspace_bytes,
)

__all__ = [
    "GQADecodeConfig",
    "gqa_decode_attention",
    "gqa_decode_attention_batched",
    "gqa_decode_attention_fp8",
    "gqa_decode_attention_persistent",
    "merge_partials",
    "plan_decode",
    "DecodePlan",
    "read_status",
    "reduce_partials",
    "reference_gqa_decode",
    "reset_workspace",
    "select_num_splits",
    "workspace_bytes",
]
