"""B200 (sm_100a) implementation of DeepSeek-V3's FP8 inference GEMM path."""
from .ops import (act_quant, weight_dequant, fp8_gemm, weight_quant, set_gemm_policy, check_device_status,
                  KERNEL_AUTO, KERNEL_CUDA_CORE, KERNEL_TC_TOKEN_MAJOR, KERNEL_TC_WEIGHT_MAJOR)
from ._lib import Dsv3Error, LIB_PATH

__all__ = ["act_quant", "weight_dequant", "fp8_gemm", "weight_quant", "set_gemm_policy", "check_device_status",
           "Dsv3Error", "LIB_PATH", "KERNEL_AUTO", "KERNEL_CUDA_CORE", "KERNEL_TC_TOKEN_MAJOR",
           "KERNEL_TC_WEIGHT_MAJOR"]
