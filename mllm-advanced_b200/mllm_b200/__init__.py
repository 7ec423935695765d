"""Python (ctypes) binding of the mllmb200 C ABI - used by the tests and bench.py.

The product is the C ABI in include/mllmb200.h and the C++ backend under
mllm-advanced_b200/backend/; this module only lets Python drive the same entry points.  torch is
used for device memory and streams, nothing else: every computation goes through libmllm_b200.so,
and importing this module fails loudly when that library has not been built.
"""
from .binding import (  # noqa: F401
    SCALE_BF16_TRUNC, SCALE_BF16_RNE, SCALE_FP16, KERNEL_AUTO, KERNEL_GEMV, KERNEL_SIMT, KERNEL_TC, KERNEL_TC_F16, KERNEL_FASTEST, KERNEL_GEMV_2LAUNCH, KERNEL_STREAM_TC, gemv_plan_check, linear_forward_multi,
    MllmB200Error, lib, lib_path, status_str, prepack_size, quant_prepack, prepack_from_quantized, blob_info,
    blob_sections, tiled_size, workspace_size, W4A32Weights, linear_forward, linear_forward_grouped, quant_activations, check_device_status, conv3d_forward,
)
from .decoder import Qwen2Decoder, Qwen2BatchDecoder, Qwen2Config, QWEN2_1P5B, LINEAR_NAMES, plan_check, DECODE_AUTO, DECODE_GRAPH, DECODE_PERSISTENT  # noqa: F401,E402
