"""The three operators of the reference's ``inference/kernel.py`` on sm_100a.

Signatures, argument meaning, allocation behaviour and assertion messages follow
``kernel.py`` (``act_quant`` :38-57, ``weight_dequant`` :89-110, ``fp8_gemm``
:175-196) so that ``model.py`` and ``generate.py`` run unchanged on top of them.
The work is done by hand-written CUDA behind a C ABI; tensors must live on a CUDA
device and nothing here falls back to another implementation.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from . import _lib
from ._lib import lib

KERNEL_AUTO, KERNEL_CUDA_CORE, KERNEL_TC_TOKEN_MAJOR, KERNEL_TC_WEIGHT_MAJOR, KERNEL_TC_TOKEN_PAIR, KERNEL_DECODE = 0, 1, 2, 3, 4, 5
KERNEL_TC_TOKEN_PAIR_WIDE = 6

_workspaces: Dict[Tuple[int, int], torch.Tensor] = {}


def _require_cuda(*tensors: torch.Tensor) -> torch.device:
    dev = tensors[0].device
    for t in tensors:
        if t.device.type != "cuda":
            raise RuntimeError("dsv3_b200 runs on CUDA tensors only (there is no CPU path); got a "
                               f"{t.device.type} tensor")
        if t.device != dev:
            raise RuntimeError("all tensors of one call must be on the same device")
    return dev


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _out_dtype() -> torch.dtype:
    dt = torch.get_default_dtype()
    if dt != torch.bfloat16:
        raise NotImplementedError(
            "the CUDA path writes bfloat16 only; call torch.set_default_dtype(torch.bfloat16) "
            f"as every entry point of the reference does (default dtype is {dt})")
    return dt


def _workspace(dev: torch.device, nbytes: int) -> Optional[torch.Tensor]:
    """Scratch for split-K, one per (device, stream); its header must be zero on first use and
    every call leaves it zero again."""
    if nbytes == 0:
        return None
    key = (dev.index if dev.index is not None else torch.cuda.current_device(), _stream())
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        size = max(nbytes, 8 << 20)
        ws = torch.zeros(size, dtype=torch.uint8, device=dev)
        _workspaces[key] = ws
    return ws


def act_quant(x: torch.Tensor, block_size: int = 128, scale_fmt: Optional[str] = None
              ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Block-wise FP8 quantisation of activations (kernel.py:38-57).

    Returns ``(y, s)``: ``y`` float8_e4m3fn of x's shape, ``s`` float32 of shape
    ``[..., K // block_size]`` with ``s = max(amax, 1e-4) / 448`` per block (rounded up to a
    power of two when ``scale_fmt == "ue8m0"``).
    """
    assert x.is_contiguous(), 'Input tensor must be contiguous'
    assert x.size(-1) % block_size == 0, \
        f'Last dimension size must be divisible by block_size (block_size={block_size})'
    dev = _require_cuda(x)
    if x.dtype != torch.bfloat16:
        raise NotImplementedError(f"act_quant takes bfloat16 activations (got {x.dtype})")
    y = torch.empty_like(x, dtype=torch.float8_e4m3fn)
    s = x.new_empty(*x.size()[:-1], x.size(-1) // block_size, dtype=torch.float32)
    K = x.size(-1)
    rows = x.numel() // K if K else 0
    with torch.cuda.device(dev):
        _lib.check(lib.dsv3_act_quant(x.data_ptr(), rows, K, block_size, 1 if scale_fmt == "ue8m0" else 0,
                                      y.data_ptr(), s.data_ptr(), _stream()))
    return y, s


def swiglu_quant(a: torch.Tensor, b: torch.Tensor, scale_fmt: Optional[str] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """``act_quant(F.silu(a) * b, 128, scale_fmt)`` in one launch (model.py:532 / 633 followed by :158-159), with the
    rounding points of the three-launch form; the bf16 product is never written."""
    assert a.is_contiguous() and b.is_contiguous(), 'Input tensors must be contiguous'
    assert a.shape == b.shape and a.size(-1) % 128 == 0, 'a and b must have the same shape, last dimension divisible by 128'
    dev = _require_cuda(a, b)
    if a.dtype != torch.bfloat16 or b.dtype != torch.bfloat16:
        raise NotImplementedError("swiglu_quant takes bfloat16 tensors")
    K = a.size(-1)
    rows = a.numel() // K if K else 0
    y = torch.empty_like(a, dtype=torch.float8_e4m3fn)
    s = a.new_empty(*a.size()[:-1], K // 128, dtype=torch.float32)
    with torch.cuda.device(dev):
        _lib.check(lib.dsv3_swiglu_quant(a.data_ptr(), b.data_ptr(), rows, K, 1 if scale_fmt == "ue8m0" else 0,
                                         y.data_ptr(), s.data_ptr(), _stream()))
    return y, s


# Cache of de-quantised weights (off by default).  MLA.forward in "absorb" mode de-quantises wkv_b on every call of
# every layer (model.py:481) although the weight never changes; with the cache on, the call after the first returns
# the tensor computed before and launches nothing.  An entry is keyed on the weight's and the scales' storage
# address, shape and in-place modification counter and holds a weak reference to the weight, so loading new values
# into the parameter (copy_, load_model) or freeing it invalidates the entry.
_dequant_cache = None            # OrderedDict when enabled
_dequant_cache_limit = 0
dequant_stats = {"launches": 0, "hits": 0}


def enable_weight_dequant_cache(max_bytes: int = 2 << 30) -> None:
    """Remember the results of ``weight_dequant`` (up to ``max_bytes`` of bf16 copies, oldest dropped first).
    The caller must treat the returned tensors as read-only (model.py:481-495 only views and multiplies them).
    Meant for inference loops; leave it off for one-pass tools such as ``fp8_cast_bf16.py``."""
    global _dequant_cache, _dequant_cache_limit
    import collections
    _dequant_cache = collections.OrderedDict()
    _dequant_cache_limit = int(max_bytes)


def disable_weight_dequant_cache() -> None:
    global _dequant_cache
    _dequant_cache = None


def _version_or_none(t: torch.Tensor):
    try:
        return t._version
    except RuntimeError:          # inference tensors carry no counter: never cached
        return None


def weight_dequant(x: torch.Tensor, s: torch.Tensor, block_size: int = 128) -> torch.Tensor:
    """De-quantise a block-scaled FP8 weight to the default dtype (kernel.py:89-110)."""
    assert x.is_contiguous() and s.is_contiguous(), 'Input tensors must be contiguous'
    assert x.dim() == 2 and s.dim() == 2, 'Input tensors must have 2 dimensions'
    dev = _require_cuda(x, s)
    if x.element_size() != 1 or s.dtype != torch.float32:
        raise NotImplementedError("weight_dequant takes a 1-byte FP8 weight and float32 scales")
    M, N = x.size()
    key = None
    if _dequant_cache is not None:
        vx, vs = _version_or_none(x), _version_or_none(s)
        if vx is not None and vs is not None:
            key = (x.data_ptr(), s.data_ptr(), M, N, block_size, vx, vs, _out_dtype())
            hit = _dequant_cache.get(key)
            if hit is not None and hit[0]() is x:
                _dequant_cache.move_to_end(key)
                dequant_stats["hits"] += 1
                return hit[1]
    y = torch.empty_like(x, dtype=_out_dtype())
    with torch.cuda.device(dev):
        _lib.check(lib.dsv3_weight_dequant(x.data_ptr(), s.data_ptr(), M, N, block_size, y.data_ptr(), _stream()))
    dequant_stats["launches"] += 1
    if key is not None:
        import weakref
        try:
            _dequant_cache[key] = (weakref.ref(x), y)
        except TypeError:
            return y
        total = sum(v[1].numel() * v[1].element_size() for v in _dequant_cache.values())
        while total > _dequant_cache_limit and len(_dequant_cache) > 1:
            _, old = _dequant_cache.popitem(last=False)
            total -= old[1].numel() * old[1].element_size()
    return y


def fp8_gemm(a: torch.Tensor, a_s: torch.Tensor, b: torch.Tensor, b_s: torch.Tensor) -> torch.Tensor:
    """Block-scaled FP8 GEMM ``c = a @ b.T`` with fp32 accumulation (kernel.py:175-196)."""
    assert a.is_contiguous() and b.is_contiguous(), 'Input tensors must be contiguous'
    assert a_s.is_contiguous() and b_s.is_contiguous(), 'Scaling factor tensors must be contiguous'
    dev = _require_cuda(a, a_s, b, b_s)
    if a.element_size() != 1 or b.element_size() != 1 or a_s.dtype != torch.float32 or b_s.dtype != torch.float32:
        raise NotImplementedError("fp8_gemm takes 1-byte FP8 operands and float32 scales")
    K = a.size(-1)
    M = a.numel() // K
    N = b.size(0)
    c = a.new_empty(*a.size()[:-1], N, dtype=_out_dtype())
    with torch.cuda.device(dev):
        ws = _workspace(dev, lib.dsv3_fp8_gemm_workspace_bytes(M, N, K))
        _lib.check(lib.dsv3_fp8_gemm(a.data_ptr(), a_s.data_ptr(), b.data_ptr(), b_s.data_ptr(), M, N, K,
                                     c.data_ptr(), ws.data_ptr() if ws is not None else None,
                                     ws.numel() if ws is not None else 0, _stream()))
    return c


def fp8_linear(x: torch.Tensor, weight: torch.Tensor, scale: torch.Tensor, scale_fmt: Optional[str] = None) -> torch.Tensor:
    """``fp8_gemm(*act_quant(x, 128, scale_fmt), weight, scale)`` (model.py:158-160) in one launch, for at most 16
    rows: the activations are quantised in the GEMM's prologue.  Raises ``Dsv3Error`` (status -2) for other shapes."""
    assert x.is_contiguous() and weight.is_contiguous() and scale.is_contiguous(), 'Input tensors must be contiguous'
    dev = _require_cuda(x, weight, scale)
    if x.dtype != torch.bfloat16 or weight.element_size() != 1 or scale.dtype != torch.float32:
        raise NotImplementedError("fp8_linear takes bfloat16 activations, a 1-byte FP8 weight and float32 scales")
    K = x.size(-1)
    M = x.numel() // K if K else 0
    N = weight.size(0)
    c = x.new_empty(*x.size()[:-1], N, dtype=_out_dtype())
    with torch.cuda.device(dev):
        _lib.check(lib.dsv3_fp8_linear(x.data_ptr(), M, K, weight.data_ptr(), scale.data_ptr(), N,
                                       1 if scale_fmt == "ue8m0" else 0, c.data_ptr(), _stream()))
    return c


# The kernel takes up to 16 rows; the seam uses it up to 4, where quantising the activations inside every CTA is
# cheaper than a separate act_quant launch (measured on B200, K 7168 x N 1536: 1 row 7.7 vs 8.5 us, 8 rows 13.5 vs 8.8 us).
FUSED_LINEAR_MAX_ROWS = 4
FUSED_LINEAR_MAX_WEIGHT_BYTES = 16 << 20


def weight_quant(w: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Harness quantiser: bf16 ``[N, K]`` -> (float8_e4m3fn ``[N, K]``, float32 ``[ceil(N/128), ceil(K/128)]``)
    with ``s = max(amax, 1e-4) / 448`` per 128x128 block; the inverse of ``weight_dequant``."""
    assert w.is_contiguous() and w.dim() == 2
    dev = _require_cuda(w)
    if w.dtype != torch.bfloat16:
        raise NotImplementedError("weight_quant takes a bfloat16 weight")
    N, K = w.shape
    q = torch.empty_like(w, dtype=torch.float8_e4m3fn)
    s = w.new_empty((N + 127) // 128, (K + 127) // 128, dtype=torch.float32)
    with torch.cuda.device(dev):
        _lib.check(lib.dsv3_weight_quant(w.data_ptr(), N, K, q.data_ptr(), s.data_ptr(), _stream()))
    return q, s


def set_gemm_policy(kernel: int = KERNEL_AUTO, split_k: int = 0) -> None:
    """Pin the fp8_gemm kernel / split-K factor (tests and benchmarks); (0, 0) restores automatic choice."""
    _lib.check(lib.dsv3_set_gemm_policy(kernel, split_k))


def set_num_sms(n: int = 0) -> None:
    """SMs the persistent GEMM kernels may occupy from now on (0 = all): leave a concurrent collective its SMs."""
    _lib.check(lib.dsv3_set_num_sms(int(n)))


def check_device_status() -> None:
    """Synchronise the current stream and raise if a kernel's bounded wait gave up."""
    import ctypes
    detail = (ctypes.c_uint32 * 4)()
    rc = lib.dsv3_check_device_status(_stream(), ctypes.byref(detail))
    if rc != _lib.OK:
        for ws in _workspaces.values():   # tickets may be left non-zero by an aborted launch
            ws[: _lib.WORKSPACE_HEADER_BYTES].zero_()
        _lib.check(rc)
