"""B200-native chunked gated-delta-rule (GDN) linear attention.

Same operator interface as FlashQLA's ``flash_qla`` package; the kernels are hand-written
sm_100a CUDA behind the C ABI of ``include/flashqla.h``.
"""
__version__ = "0.1.0"
