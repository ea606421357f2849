"""Drop-in import name of the reference package: ``import prime_moe`` resolves to the B200 build.

Same public names as the reference (prime_moe/__init__.py:117-122) plus ``moe_align``.
"""
from prime_flash_moe_b200 import BLOCK, fused_moe_bf16, fused_moe_mxfp8, moe_align, pack_scales_blocked

__all__ = ["fused_moe_bf16", "fused_moe_mxfp8", "pack_scales_blocked", "BLOCK", "moe_align"]
