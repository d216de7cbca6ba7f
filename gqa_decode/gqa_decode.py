"""Module-path alias: the reference's tests import ``gqa_decode.gqa_decode``."""
from gqa_decode_b200.gqa_decode import *  # noqa: F401,F403
from gqa_decode_b200.gqa_decode import (  # noqa: F401
    GQADecodeConfig,
    gqa_decode_attention,
    gqa_decode_attention_batched,
    gqa_decode_attention_fp8,
    gqa_decode_attention_persistent,
    merge_partials,
    reduce_partials,
    reference_gqa_decode,
    select_num_splits,
)
