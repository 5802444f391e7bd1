"""B200 (sm_100a) FP8 flash-attention forward behind the operator interface of
weishengying/cutlass_flash_atten_fp8.  See api.py for the operator, shard.py for
the (batch x head) partition used on multi-GPU boxes, synth.py for the seeded
synthetic workloads of the benchmark."""
from .api import HostRunner, check_status, flash_attention_v2_cutlass, quantize_e4m3  # noqa: F401
from .shard import shard_range  # noqa: F401

__all__ = ["flash_attention_v2_cutlass", "check_status", "HostRunner", "quantize_e4m3", "shard_range"]
