"""B200-native chunked gated-delta-rule (GDN) linear attention.

Same operator interface as FlashQLA's ``flash_qla`` package; the kernels are hand-written
sm_100a CUDA behind the C ABI of ``include/flashqla.h``.
"""
__version__ = "0.1.0"

from .ops import (  # noqa: E402
    chunk_gated_delta_rule,
    chunk_gated_delta_rule_bwd,
    chunk_gated_delta_rule_fwd,
)

from .decode import fused_recurrent_gated_delta_rule  # noqa: E402

__all__ = ["chunk_gated_delta_rule_fwd", "chunk_gated_delta_rule_bwd", "chunk_gated_delta_rule",
           "fused_recurrent_gated_delta_rule"]
