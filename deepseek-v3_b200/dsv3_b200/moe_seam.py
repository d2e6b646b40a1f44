"""Seam above the operators: the MoE expert loop as grouped GEMMs.

``MoE.forward`` of the reference (model.py:669-693) walks over the local experts in Python; every
expert costs two host synchronisations (``bincount(...).tolist()``, ``torch.where``) and about six
small launches.  ``grouped_moe_forward`` keeps inputs, outputs and arithmetic (same quantisation per
token row, same bf16 rounding points, same ascending-expert accumulation order) but sorts the
(token, expert) pairs on the device (one launch) and runs each of the three projections as one grouped GEMM
over all local experts, followed by one combine kernel.  Nothing is read back to the host.

    import model, dsv3_b200
    dsv3_b200.install_moe(model)        # model.MoE.forward = grouped_moe_forward
"""
from __future__ import annotations

import ctypes
from typing import List

import torch

from . import _lib
from ._lib import lib
from .linear_seam import _quantised
from .ops import swiglu_quant, _stream


class GroupedExperts:
    """Device tables (tensor maps + scale pointers) of the local experts' three projections."""

    def __init__(self, experts: List, start: int):
        self.start = start
        self.n = len(experts)
        e0 = experts[0]
        self.dim = e0.w1.weight.size(1)
        self.inter = e0.w1.weight.size(0)
        self.scale_fmt = getattr(e0.w1, "scale_fmt", None)
        self.device = e0.w1.weight.device
        self._keep = experts                       # the tables point into these parameters
        self.tables = {}
        for name, N, K in (("w1", self.inter, self.dim), ("w3", self.inter, self.dim), ("w2", self.dim, self.inter)):
            ws = [getattr(e, name).weight for e in experts]
            ss = [getattr(e, name).weight.scale for e in experts]
            for w, s in zip(ws, ss):
                assert w.element_size() == 1 and w.is_contiguous() and s.is_contiguous() and s.dtype == torch.float32
                assert tuple(w.shape) == (N, K)
            table = torch.empty(lib.dsv3_group_table_bytes(self.n), dtype=torch.uint8, device=self.device)
            wp = (ctypes.c_void_p * self.n)(*[w.data_ptr() for w in ws])
            sp = (ctypes.c_void_p * self.n)(*[s.data_ptr() for s in ss])
            with torch.cuda.device(self.device):
                _lib.check(lib.dsv3_group_table_build(table.data_ptr(), wp, sp, self.n, N, K, _stream()))
            self.tables[name] = (table, N, K)
        self.signature = tuple(getattr(e, n).weight.data_ptr() for e in experts for n in ("w1", "w2", "w3"))

    def gemm(self, name: str, a: torch.Tensor, a_s: torch.Tensor, seg: torch.Tensor, rows_hint: int = 0) -> torch.Tensor:
        table, N, K = self.tables[name]
        rows = a.size(0)
        c = torch.empty(rows, N, dtype=torch.bfloat16, device=a.device)
        _lib.check(lib.dsv3_fp8_gemm_grouped(table.data_ptr(), self.n, a.data_ptr(), a_s.data_ptr(), seg.data_ptr(),
                                             rows, rows_hint, N, K, c.data_ptr(), _stream()))
        return c

    def routed(self, x: torch.Tensor, weights: torch.Tensor, indices: torch.Tensor, n_routed: int = 0) -> torch.Tensor:
        """Sum over the local experts of ``expert(x[idx]) * weights`` (model.py:683-689).  ``n_routed``: experts of
        the whole layer (this rank owns ``self.n`` of them and, on average, that share of the pairs)."""
        T, topk = indices.shape
        P = T * topk
        n = self.n
        hint = max(1, (P * n + n_routed - 1) // n_routed) if n_routed > n else 0
        with torch.cuda.device(x.device):
            # ---- group the (token, expert) pairs by local expert (pairs of other ranks' experts go last) and
            # order every token's pairs by expert id: one launch, nothing read back
            idx = indices if indices.dtype == torch.int64 else indices.long()
            idx = idx if idx.is_contiguous() else idx.contiguous()
            wf = (weights if weights.dtype == torch.float32 else weights.float()).contiguous()
            seg = torch.empty(n + 1, dtype=torch.int32, device=x.device)
            tok = torch.empty(P, dtype=torch.int32, device=x.device)
            pair_row = torch.empty(P, dtype=torch.int32, device=x.device)
            pos_s = torch.empty(T, topk, dtype=torch.int32, device=x.device)
            w_s = torch.empty(T, topk, dtype=torch.bfloat16, device=x.device)
            _lib.check(lib.dsv3_moe_route(idx.data_ptr(), wf.data_ptr(), T, topk, self.start, n, seg.data_ptr(),
                                          tok.data_ptr(), pair_row.data_ptr(), pos_s.data_ptr(), w_s.data_ptr(), _stream()))
            # ---- quantise every token once, gather the rows in expert order
            xq, xs = _quantised(x, 128, self.scale_fmt)
            xq_p = xq.view(torch.uint8).index_select(0, tok).view(torch.float8_e4m3fn)
            xs_p = xs.index_select(0, tok)
            # ---- w2(silu(w1 x) * w3 x), the bf16 rounding points of Expert.forward (model.py:633)
            hq, hs = swiglu_quant(self.gemm("w1", xq_p, xs_p, seg, hint), self.gemm("w3", xq_p, xs_p, seg, hint), self.scale_fmt)
            o = self.gemm("w2", hq, hs, seg, hint)
            # ---- y[t] = sum over the token's local experts, ascending expert id, bf16 at every step
            y = torch.empty(T, self.dim, dtype=torch.bfloat16, device=x.device)
            _lib.check(lib.dsv3_moe_combine(o.data_ptr(), pos_s.data_ptr(), w_s.data_ptr(), T, topk, self.dim,
                                            y.data_ptr(), _stream()))
        return y


def _grouped(moe) -> GroupedExperts:
    local = [moe.experts[i] for i in range(moe.experts_start_idx, moe.experts_end_idx)]
    sig = tuple(getattr(e, n).weight.data_ptr() for e in local for n in ("w1", "w2", "w3"))
    st = getattr(moe, "_dsv3_grouped", None)
    if st is None or st.signature != sig:
        st = GroupedExperts(local, moe.experts_start_idx)
        object.__setattr__(moe, "_dsv3_grouped", st)      # not a Module/Parameter: keep it out of the registry
    return st


def grouped_moe_forward(self, x: torch.Tensor, *, world_size: int = 1, fallback=None) -> torch.Tensor:
    """Same inputs and outputs as ``MoE.forward`` (model.py:669-693)."""
    e0 = self.experts[self.experts_start_idx]
    if e0.w1.weight.element_size() != 1 or x.dtype != torch.bfloat16 or self.n_local_experts > 256:
        if fallback is None:
            raise NotImplementedError("grouped MoE needs FP8 expert weights, bf16 activations and <= 256 local experts")
        return fallback(self, x)
    shape = x.size()
    x = x.view(-1, self.dim)
    weights, indices = self.gate(x)
    y = _grouped(self).routed(x, weights, indices, getattr(self, "n_routed_experts", 0))
    z = self.shared_experts(x)
    if world_size > 1:
        import torch.distributed as dist
        dist.all_reduce(y)
    return (y + z).view(shape)


def install_moe(model_module) -> None:
    """Replace ``model_module.MoE.forward``; ``model_module.world_size`` is read at call time."""
    original = model_module.MoE.forward

    def forward(self, x):
        if getattr(model_module, "gemm_impl", "fp8") != "fp8":
            return original(self, x)
        return grouped_moe_forward(self, x, world_size=model_module.world_size, fallback=original)

    forward.__doc__ = grouped_moe_forward.__doc__
    model_module.MoE.forward = forward
