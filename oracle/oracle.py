"""CPU oracle for the FP8 GEMM path of DeepSeek-V3's inference code.

TEST INFRASTRUCTURE ONLY: the checker for the CUDA kernels and the timed CPU
baseline.  Product code must never import this module.

Two independent restatements live here so that they can check each other:

* the C library ``libdsv3_oracle.so`` (``dsv3_oracle.c``; OpenMP, used for
  parity tests and as the CPU baseline), wrapped by ``act_quant``,
  ``weight_dequant``, ``fp8_gemm``, ``weight_quant``, ``linear_fp8``;
* plain torch ops (``*_torch``), which rely on torch's own e4m3 / bf16 casts.

Reference being restated: ``inference/kernel.py`` (``act_quant`` :38-57,
``weight_dequant`` :89-110, ``fp8_gemm`` :175-196) and ``linear()`` in
``inference/model.py:131-163``.

Numerics are those of the reference's kernels compiled for a GPU
(round-to-nearest-even casts); the Triton CPU interpreter deviates from that
in its casts, and ``e4m3_cast_triton_interpreter`` / ``bf16_truncate`` restate
those deviations so that CPU runs of the reference can be matched bit for bit.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from typing import Optional, Tuple

import numpy as np
import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libdsv3_oracle.so")
_lib = None

FP8_MAX = 448.0
BLOCK = 128


def build(force: bool = False) -> str:
    """Compile the C oracle with the Makefile next to this file."""
    src = os.path.join(_HERE, "dsv3_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE], check=True, capture_output=True)
    return _LIB_PATH


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(_LIB_PATH)
        i64, p, ci = ctypes.c_int64, ctypes.c_void_p, ctypes.c_int
        L.orc_act_quant.argtypes = [p, i64, i64, ci, ci, p, p]
        L.orc_weight_dequant.argtypes = [p, p, i64, i64, ci, p]
        L.orc_fp8_gemm.argtypes = [p, p, p, p, i64, i64, i64, p]
        L.orc_weight_quant.argtypes = [p, i64, i64, ci, p, p]
        L.orc_linear_fp8.argtypes = [p, p, p, i64, i64, i64, p, p, p]
        L.orc_f32_to_e4m3_array.argtypes = [p, i64, p]
        L.orc_f32_to_e4m3_array.restype = None
        L.orc_e4m3_to_f32.argtypes = [ctypes.c_uint8]
        L.orc_e4m3_to_f32.restype = ctypes.c_float
        L.orc_f32_to_bf16.argtypes = [ctypes.c_float]
        L.orc_f32_to_bf16.restype = ctypes.c_uint16
        L.orc_num_threads.restype = ci
        L.orc_set_num_threads.argtypes = [ci]
        L.orc_set_num_threads.restype = None
        _lib = L
    return _lib


def num_threads() -> int:
    return int(lib().orc_num_threads())


def set_num_threads(n: int) -> None:
    lib().orc_set_num_threads(int(n))


def _cpu(t: torch.Tensor) -> torch.Tensor:
    return t.detach().to("cpu").contiguous()


def _check(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"oracle {what} failed with status {rc}")


# --------------------------------------------------------------------------
# C-library wrappers (same signatures as the reference's three functions)
# --------------------------------------------------------------------------

def act_quant(x: torch.Tensor, block_size: int = 128, scale_fmt: Optional[str] = None
              ) -> Tuple[torch.Tensor, torch.Tensor]:
    """kernel.py:38-57.  ``x`` is upcast exactly to fp32 as the kernel does (:25);
    only bf16 input is accepted because that is what the model feeds it."""
    assert x.is_contiguous(), "Input tensor must be contiguous"
    assert x.size(-1) % block_size == 0, \
        f"Last dimension size must be divisible by block_size (block_size={block_size})"
    assert x.dtype == torch.bfloat16
    xc = _cpu(x)
    K = xc.size(-1)
    rows = xc.numel() // K if K else 0
    y = torch.empty(xc.shape, dtype=torch.uint8)
    s = torch.empty(*xc.shape[:-1], K // block_size, dtype=torch.float32)
    if xc.numel():
        _check(lib().orc_act_quant(xc.view(torch.int16).data_ptr(), rows, K, block_size,
                                   1 if scale_fmt == "ue8m0" else 0, y.data_ptr(), s.data_ptr()),
               "act_quant")
    return y.view(torch.float8_e4m3fn), s


def weight_dequant(x: torch.Tensor, s: torch.Tensor, block_size: int = 128) -> torch.Tensor:
    """kernel.py:89-110."""
    assert x.is_contiguous() and s.is_contiguous(), "Input tensors must be contiguous"
    assert x.dim() == 2 and s.dim() == 2, "Input tensors must have 2 dimensions"
    xc, sc = _cpu(x).view(torch.uint8), _cpu(s).float()
    N, K = xc.shape
    y = torch.empty(N, K, dtype=torch.int16)
    if xc.numel():
        _check(lib().orc_weight_dequant(xc.data_ptr(), sc.data_ptr(), N, K, block_size, y.data_ptr()),
               "weight_dequant")
    return y.view(torch.bfloat16)


def fp8_gemm(a: torch.Tensor, a_s: torch.Tensor, b: torch.Tensor, b_s: torch.Tensor) -> torch.Tensor:
    """kernel.py:175-196."""
    assert a.is_contiguous() and b.is_contiguous(), "Input tensors must be contiguous"
    assert a_s.is_contiguous() and b_s.is_contiguous(), "Scaling factor tensors must be contiguous"
    ac, bc = _cpu(a).view(torch.uint8), _cpu(b).view(torch.uint8)
    asc, bsc = _cpu(a_s).float(), _cpu(b_s).float()
    K = ac.size(-1)
    M = ac.numel() // K if K else 0
    N = bc.size(0)
    c = torch.empty(*ac.shape[:-1], N, dtype=torch.int16)
    if M and N:
        _check(lib().orc_fp8_gemm(ac.data_ptr(), asc.data_ptr(), bc.data_ptr(), bsc.data_ptr(),
                                  M, N, K, c.data_ptr()), "fp8_gemm")
    return c.view(torch.bfloat16)


def weight_quant(w: torch.Tensor, block_size: int = 128) -> Tuple[torch.Tensor, torch.Tensor]:
    """Harness quantiser (the reference ships none): per 128x128 block
    ``s = max(amax, 1e-4) / 448``, ``q = e4m3(w / s)``; edge blocks are partial
    (equivalent to the zero padding of README_WEIGHTS.md:89)."""
    assert w.dim() == 2 and w.dtype == torch.bfloat16
    wc = _cpu(w)
    N, K = wc.shape
    q = torch.empty(N, K, dtype=torch.uint8)
    s = torch.empty((N + block_size - 1) // block_size, (K + block_size - 1) // block_size,
                    dtype=torch.float32)
    _check(lib().orc_weight_quant(wc.view(torch.int16).data_ptr(), N, K, block_size,
                                  q.data_ptr(), s.data_ptr()), "weight_quant")
    return q.view(torch.float8_e4m3fn), s


def linear_fp8(x: torch.Tensor, w: torch.Tensor, w_s: torch.Tensor) -> torch.Tensor:
    """model.py:158-160: ``fp8_gemm(*act_quant(x), weight, weight.scale)``."""
    xq, xs = act_quant(x)
    return fp8_gemm(xq, xs, w, w_s)


# --------------------------------------------------------------------------
# Independent torch restatements
# --------------------------------------------------------------------------

def act_quant_torch(x: torch.Tensor, block_size: int = 128, scale_fmt: Optional[str] = None):
    xf = x.float().reshape(*x.shape[:-1], x.size(-1) // block_size, block_size)
    amax = xf.abs().amax(dim=-1).clamp_min(1e-4)
    s = amax / FP8_MAX
    if scale_fmt == "ue8m0":
        s = torch.exp2(torch.ceil(torch.log2(s)))
    y = (xf / s.unsqueeze(-1)).reshape(x.shape).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)
    return y, s


def _expand_block_scale(s: torch.Tensor, N: int, K: int, block: int) -> torch.Tensor:
    return s.repeat_interleave(block, 0)[:N].repeat_interleave(block, 1)[:, :K]


def weight_dequant_torch(x: torch.Tensor, s: torch.Tensor, block_size: int = 128) -> torch.Tensor:
    N, K = x.shape
    return (x.float() * _expand_block_scale(s.float(), N, K, block_size)).to(torch.bfloat16)


def fp8_gemm_torch(a, a_s, b, b_s, out_fp32: bool = False) -> torch.Tensor:
    """Per-chunk fp64 dot (exact), rounded to fp32, then the reference's
    ``acc += dot * a_s * b_s`` in fp32 (kernel.py:162)."""
    K = a.size(-1)
    M = a.numel() // K
    N = b.size(0)
    kc = (K + 127) // 128
    af = a.reshape(M, K).double()
    bf = b.double()
    asf = a_s.reshape(M, kc).float()
    bse = b_s.float().repeat_interleave(128, 0)[:N]            # [N, kc]
    acc = torch.zeros(M, N, dtype=torch.float32)
    for i in range(kc):
        sl = slice(i * 128, min((i + 1) * 128, K))
        p = (af[:, sl] @ bf[:, sl].T).float()
        t = p * asf[:, i:i + 1]
        acc = torch.addcmul(acc, t, bse[:, i].unsqueeze(0))     # one rounding less than fma at most
    out = acc if out_fp32 else acc.to(torch.bfloat16)
    return out.reshape(*a.shape[:-1], N)


def weight_quant_torch(w: torch.Tensor, block_size: int = 128):
    N, K = w.shape
    nb, kb = -(-N // block_size), -(-K // block_size)
    wp = torch.zeros(nb * block_size, kb * block_size, dtype=torch.float32)
    wp[:N, :K] = w.float()
    blocks = wp.view(nb, block_size, kb, block_size)
    s = blocks.abs().amax(dim=(1, 3)).clamp_min(1e-4) / FP8_MAX
    q = (blocks / s[:, None, :, None]).reshape(nb * block_size, kb * block_size)[:N, :K]
    return q.contiguous().to(torch.float8_e4m3fn), s.contiguous()


# --------------------------------------------------------------------------
# Casts of the Triton CPU interpreter (needed to match a CPU run of the reference)
# --------------------------------------------------------------------------

def e4m3_cast_triton_interpreter(x: np.ndarray) -> np.ndarray:
    """fp32 -> e4m3 bytes the way Triton 3.6's CPU interpreter does it for normal
    results: truncate to three mantissa bits, add one if the first discarded bit
    is set, and OR the fields together without carrying a mantissa overflow into
    the exponent; results below the e4m3 normal range shift the truncated
    mantissa right and set the implicit-one bit (no rounding there either)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.int64)
    sign = (u >> 31) & 1
    exp = (u >> 23) & 0xFF
    mant = u & 0x7FFFFF
    # fp32 subnormal inputs never reach an e4m3 value other than zero
    e_out = np.clip(exp - 127 + 7, 0, 15)
    sig = ((mant >> 20) & 7) + ((mant & (1 << 19)) > 0)
    sub = (e_out == 0) & (exp != 0)
    shift = np.where(sub, (1 - 7) - (exp - 127), 0)
    shift_c = np.clip(shift, 0, 62)
    sig_sub = (sig >> shift_c) | (1 << np.clip(3 - shift, -62, 62).clip(min=0)) * (3 - shift >= 0)
    sig = np.where(sub, sig_sub, sig)
    out = (sign << 7) | (e_out << 3) | sig
    return (out & 0xFF).astype(np.uint8).reshape(np.shape(x))


def bf16_truncate(x: torch.Tensor) -> torch.Tensor:
    """fp32 -> bf16 by dropping the low 16 bits (the interpreter's store cast)."""
    return (x.float().contiguous().view(torch.int32) >> 16).to(torch.int16).view(torch.bfloat16)


# --------------------------------------------------------------------------
# Seeded inputs (numpy PCG64 streams are stable across machines and versions)
# --------------------------------------------------------------------------

def randn_bf16(shape, seed: int, std: float = 1.0) -> torch.Tensor:
    g = np.random.Generator(np.random.PCG64(seed))
    a = g.standard_normal(size=shape, dtype=np.float32) * np.float32(std)
    return torch.from_numpy(a).to(torch.bfloat16)


def make_case(M: int, N: int, K: int, seed: int = 0):
    """Activations ~ N(0,1) bf16 [M,K]; weights ~ N(0,0.02) bf16 [N,K] block-quantised."""
    x = randn_bf16((M, K), seed * 2 + 1, 1.0)
    w = randn_bf16((N, K), seed * 2 + 2, 0.02)
    wq, ws = weight_quant(w)
    return x, w, wq, ws


def gemm_tolerance_ok(y: torch.Tensor, y_ref: torch.Tensor, rel: float = 1e-2):
    """|y - y_ref| <= rel * (|y_ref| + rms(y_ref)); returns (ok, worst ratio)."""
    yr = y_ref.float()
    err = (y.float().cpu() - yr).abs()
    rms = yr.pow(2).mean().sqrt()
    bound = rel * (yr.abs() + rms)
    ratio = (err / bound.clamp_min(1e-30)).max().item() if err.numel() else 0.0
    return bool((err <= bound).all()), ratio
