"""q35b: B200-native NVFP4 projection engine (Python front-end of the C ABI in include/q35b_nvfp4.h)."""
from .engine import (  # noqa: F401
    GEMV_AUTO,
    GEMV_SIMT,
    GEMV_STREAM,
    Nvfp4Weight,
    Q35bError,
    act_scratch,
    gemm_w4a4,
    gemv_w4a16,
    gemv_w4a16_f32,
    launch_count,
    lib,
    project_prefill,
    quantize_activations,
    quantize_activations_reference_recipe,
    quantize_weight,
    shard_range,
)
