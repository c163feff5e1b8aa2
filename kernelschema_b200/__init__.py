"""B200-native NVFP4 mixture-of-experts layer: host-side mirror of the reference operator interface
over the libb200moe C ABI (see include/b200moe.h)."""
from .ops import (MoELayer, nvfp4_quantize, scales_to_tiles, route_topk, router_logits, mm_nvfp4, mm_bf16_nvfp4, combine)  # noqa: F401
from .solution import DenseModel, Model  # noqa: F401
