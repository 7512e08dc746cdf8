"""Drop-in import path: ``from flash_qla import chunk_gated_delta_rule, ...`` resolves to the
B200-native implementation in ``flashqla_b200`` (same names as flash_qla/__init__.py:6-16 of
the reference)."""
from flashqla_b200 import (  # noqa: F401
    __version__,
    chunk_gated_delta_rule,
    chunk_gated_delta_rule_bwd,
    chunk_gated_delta_rule_fwd,
)

__all__ = ["chunk_gated_delta_rule_fwd", "chunk_gated_delta_rule_bwd", "chunk_gated_delta_rule"]
