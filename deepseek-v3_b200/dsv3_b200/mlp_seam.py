"""Seam above the operators: ``MLP.forward`` and ``Expert.forward`` with the SwiGLU folded into the quantisation.

Both compute ``w2(F.silu(w1(x)) * w3(x))`` (model.py:532, 633).  In FP8 mode the product is quantised straight away by
the ``linear()`` call of ``w2`` (model.py:158-159), so silu, multiply and act_quant are three launches and two bf16
round trips through HBM for what is one pass over the data.  ``mlp_forward`` calls ``w1`` and ``w3`` as before (through
whatever ``linear`` is installed), then ``swiglu_quant`` (one launch, same rounding points, bit-identical FP8 codes and
scales) and feeds ``fp8_gemm`` of ``w2`` directly, followed by what ``w2.forward`` would have done after its GEMM: the
all-reduce of a ``RowParallelLinear`` (model.py:263-264) and the bias.

    import model, dsv3_b200
    dsv3_b200.install_mlp(model)        # model.MLP.forward, model.Expert.forward
"""
from __future__ import annotations

import torch

from .ops import fp8_gemm, swiglu_quant


def _fusable(self, x, model_module) -> bool:
    w2 = self.w2
    return (getattr(model_module, "gemm_impl", "fp8") == "fp8" and getattr(model_module, "block_size", 128) == 128
            and w2.weight.element_size() == 1 and self.w1.weight.element_size() == 1 and self.w3.weight.element_size() == 1
            and w2.weight.size(1) % 128 == 0 and x.dtype == torch.bfloat16)


def mlp_forward(self, x: torch.Tensor, *, model_module, original) -> torch.Tensor:
    """Same inputs and outputs as ``MLP.forward`` / ``Expert.forward`` (model.py:520-532, 622-633)."""
    if not _fusable(self, x, model_module):
        return original(self, x)
    w2 = self.w2
    row_parallel = type(w2).__name__ == "RowParallelLinear"
    # only plain Linear hands its scale_fmt to linear() (model.py:205); the parallel Linears do not (model.py:233, 262)
    scale_fmt = None if (row_parallel or type(w2).__name__ == "ColumnParallelLinear") else getattr(w2, "scale_fmt", None)
    hq, hs = swiglu_quant(self.w1(x), self.w3(x), scale_fmt)
    y = fp8_gemm(hq, hs, w2.weight, w2.weight.scale)
    if row_parallel:
        if model_module.world_size > 1:
            model_module.dist.all_reduce(y)
        if w2.bias is not None:
            y += w2.bias
    elif getattr(w2, "bias", None) is not None:
        y += w2.bias
    return y


def install_mlp(model_module) -> None:
    """Replace ``model_module.MLP.forward`` and ``model_module.Expert.forward``; ``gemm_impl``, ``block_size``,
    ``world_size`` and ``dist`` of the module are read at call time."""
    for cls_name in ("MLP", "Expert"):
        cls = getattr(model_module, cls_name)
        original = cls.forward

        def forward(self, x, _original=original):
            return mlp_forward(self, x, model_module=model_module, original=_original)

        forward.__doc__ = mlp_forward.__doc__
        cls.forward = forward
