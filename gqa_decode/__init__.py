"""Import-compatible alias of the reference package name: ``import gqa_decode`` resolves
to the B200 implementation in ``gqa_decode_b200`` (same names as the reference's
``gqa_decode/__init__.py``)."""
from gqa_decode_b200 import (
    GQADecodeConfig,
    gqa_decode_attention,
    gqa_decode_attention_fp8,
    gqa_decode_attention_persistent,
    reduce_partials,
    reference_gqa_decode,
    select_num_splits,
)

__all__ = [
    "GQADecodeConfig",
    "gqa_decode_attention",
    "gqa_decode_attention_fp8",
    "gqa_decode_attention_persistent",
    "reduce_partials",
    "reference_gqa_decode",
    "select_num_splits",
]
