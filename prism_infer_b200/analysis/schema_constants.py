"""Constants shared by the record validators (reference: ``prism_infer/analysis/schema_constants.py:5-12``)."""

LOWERCASE_HEX_DIGITS = frozenset("0123456789abcdef")
RGB_CHANNEL_COUNT = 3
SHA256_HEX_LENGTH = 64
GIT_REVISION_HEX_LENGTH = 40
COMPUTE_CAPABILITY_COMPONENT_COUNT = 2
PERCENTAGE_POINTS_SCALE = 100.0
# names of the fused decode regions recorded in benchmark metadata: here they are kernels, not
# compiler subgraphs
DECODE_FUSED_PROJECTION = "split_k_qkv_projection_qk_norm_mrope_kv_store"
DECODE_FUSED_MLP = "dual_gate_up_swiglu"
DECODE_KV_BOUNDARY = "scaled_fp8_store_and_paged_decode"


def is_lower_hex(text: object, length: int) -> bool:
    return isinstance(text, str) and len(text) == length and all(c in LOWERCASE_HEX_DIGITS for c in text)
