"""B200 (sm_100a) implementation of DeepSeek-V3's FP8 inference GEMM path."""
from .ops import (act_quant, weight_dequant, fp8_gemm, fp8_linear, swiglu_quant, weight_quant, set_gemm_policy, set_num_sms, check_device_status,
                  enable_weight_dequant_cache, disable_weight_dequant_cache,
                  KERNEL_AUTO, KERNEL_CUDA_CORE, KERNEL_TC_TOKEN_MAJOR, KERNEL_TC_WEIGHT_MAJOR, KERNEL_TC_TOKEN_PAIR, KERNEL_DECODE, KERNEL_TC_TOKEN_PAIR_WIDE)
from ._lib import Dsv3Error, LIB_PATH
from .linear_seam import linear, install_linear
from .moe_seam import grouped_moe_forward, install_moe
from .collective import P2PAllReduce, install_all_reduce
from .mlp_seam import mlp_forward, install_mlp

__all__ = ["P2PAllReduce", "install_all_reduce", "mlp_forward", "install_mlp", "linear", "install_linear", "grouped_moe_forward", "install_moe", "act_quant", "weight_dequant", "fp8_gemm", "fp8_linear", "swiglu_quant", "weight_quant", "set_gemm_policy", "set_num_sms", "check_device_status", "enable_weight_dequant_cache", "disable_weight_dequant_cache",
           "Dsv3Error", "LIB_PATH", "KERNEL_AUTO", "KERNEL_CUDA_CORE", "KERNEL_TC_TOKEN_MAJOR",
           "KERNEL_TC_WEIGHT_MAJOR", "KERNEL_TC_TOKEN_PAIR", "KERNEL_DECODE", "KERNEL_TC_TOKEN_PAIR_WIDE"]
