"""Module-path alias of ``gqa_decode_b200.fp8_utils``."""
from gqa_decode_b200.fp8_utils import append_kv_fp8, dequantize_kv_fp8, quantize_kv_fp8  # noqa: F401
