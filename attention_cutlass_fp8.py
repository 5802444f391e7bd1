"""Drop-in module name of the reference extension (setup.py:45 names it
``attention_cutlass_fp8``; test.py:3 imports ``flash_attention_v2_cutlass`` from it)."""
from cutlass_flash_atten_fp8_b200.api import flash_attention_v2_cutlass  # noqa: F401

__all__ = ["flash_attention_v2_cutlass"]
