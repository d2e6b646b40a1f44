"""Seam above the three operators: a replacement for ``linear()`` of the reference's ``model.py``.

``model.py:131-163`` dispatches every projection through the module-level function ``linear``;
``Linear.forward``, ``ColumnParallelLinear.forward``, ``RowParallelLinear.forward`` and
``Gate.forward`` look the name up at call time (model.py:205, 233, 262, 576), so one assignment

    import model, dsv3_b200
    dsv3_b200.install_linear(model)

redirects all of them without touching the file.  The replacement keeps the reference's three
branches and adds one thing: the FP8 quantisation of an activation tensor is remembered while that
tensor is alive and unmodified, so that Linears fed the same input (``wq_a``/``wkv_a`` in MLA,
``w1``/``w3`` in MLP and Expert) quantise it once instead of twice.  Results are bit-identical to
the unfused path because the very same ``act_quant`` output is reused.
"""
from __future__ import annotations

import weakref
from typing import Optional

import torch
import torch.nn.functional as F

from .ops import act_quant, fp8_gemm, weight_dequant

_memo = {"ref": None, "version": -1, "key": None, "value": None}
stats = {"act_quant_calls": 0, "act_quant_reused": 0}


def _version(x: torch.Tensor) -> int:
    """In-place modification counter; tensors created under torch.inference_mode() have none, and there
    the memo relies on object identity alone (model.py does not modify a projection's input in place)."""
    try:
        return x._version
    except RuntimeError:
        return -2


def _quantised(x: torch.Tensor, block_size: int, scale_fmt: Optional[str]):
    ref = _memo["ref"]
    key = (x.data_ptr(), tuple(x.shape), block_size, scale_fmt)
    if ref is not None and ref() is x and _memo["version"] == _version(x) and _memo["key"] == key:
        stats["act_quant_reused"] += 1
        return _memo["value"]
    value = act_quant(x, block_size, scale_fmt)
    stats["act_quant_calls"] += 1
    try:
        _memo.update(ref=weakref.ref(x), version=_version(x), key=key, value=value)
    except TypeError:           # tensor subclasses that cannot be weakly referenced: no memo
        _memo.update(ref=None, value=None)
    return value


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
           scale_fmt: Optional[str] = None, *, gemm_impl: str = "fp8", block_size: int = 128) -> torch.Tensor:
    """``y = x @ weight.T + bias`` with the reference's dispatch (model.py:153-163)."""
    if weight.element_size() > 1:
        return F.linear(x, weight, bias)
    if gemm_impl == "bf16":
        return F.linear(x, weight_dequant(weight, weight.scale), bias)
    xq, xs = _quantised(x, block_size, scale_fmt)
    y = fp8_gemm(xq, xs, weight, weight.scale)
    if bias is not None:
        y += bias
    return y


def install_linear(model_module) -> None:
    """Point ``model_module.linear`` at this implementation; ``model_module.gemm_impl`` and
    ``model_module.block_size`` keep their meaning and are read at call time, as in the reference."""
    def _linear(x, weight, bias=None, scale_fmt=None):
        return linear(x, weight, bias, scale_fmt, gemm_impl=model_module.gemm_impl,
                      block_size=model_module.block_size)
    _linear.__doc__ = linear.__doc__
    model_module.linear = _linear


def reset_memo() -> None:
    _memo.update(ref=None, version=-1, key=None, value=None)
    stats.update(act_quant_calls=0, act_quant_reused=0)
