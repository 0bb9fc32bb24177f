"""B200 (sm_100a) SVDQuant W4A4 linear: fused NVFP4 activation quantizer and
block-scaled tcgen05 GEMM behind the reference's operator API."""
from .ops import (  # noqa: F401
    LinearPlan,
    gemm_w4a4,
    launch_v2,
    quantize_nvfp4_rows,
    quantize_w4a4_act_fuse_lora,
    swizzle_scales,
)

__version__ = "0.1.0"
