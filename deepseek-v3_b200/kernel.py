"""Drop-in replacement for the reference's ``inference/kernel.py``.

Put this directory ahead of the reference's ``inference/`` on ``sys.path`` and
``model.py:10`` (``from kernel import act_quant, weight_dequant, fp8_gemm``) and
``fp8_cast_bf16.py:10`` bind to the sm_100a CUDA kernels with no source change.
"""
from dsv3_b200.ops import act_quant, weight_dequant, fp8_gemm

__all__ = ["act_quant", "weight_dequant", "fp8_gemm"]
