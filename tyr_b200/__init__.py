"""B200-native attention operator behind Tyr's typed attention call.

Host-side mirror of the reference interface (same names, argument meaning and
error behaviour as Tyr/Torch.lean:663-671 and 1058-1082) over the C ABI in
include/tyr_b200_attn.h.  PyTorch is used for device memory and streams only.
"""
from . import nn  # noqa: F401
from .nn import (attentionFwd, flashDecode, scaled_dot_product_attention,  # noqa: F401
                 scaledDotProductAttentionGQA, scaledDotProductAttentionGQAQKV,
                 scaledDotProductAttentionGQAMask, scaledDotProductAttentionGQAWindow)

__all__ = ["nn", "attentionFwd", "flashDecode", "scaled_dot_product_attention",
           "scaledDotProductAttentionGQA", "scaledDotProductAttentionGQAQKV",
           "scaledDotProductAttentionGQAWindow", "scaledDotProductAttentionGQAMask"]
