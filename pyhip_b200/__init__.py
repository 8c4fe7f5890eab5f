"""B200-native fused-MoE operator behind the call surface of tingqli/pyhip's quantised MoE path."""
from .fused_moe import (ActivationType, QuantType, PreparedWeights, fused_moe, fused_topk, moe_sorting,  # noqa: F401
                        prepare_weights, release_prepared)

from .linear import linear_fp8_128x128, linear_mxfp4  # noqa: F401,E402

__all__ = ["ActivationType", "QuantType", "PreparedWeights", "fused_moe", "moe_sorting", "prepare_weights",
           "linear_mxfp4", "linear_fp8_128x128", "fused_topk", "release_prepared"]
