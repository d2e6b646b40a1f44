"""CPU-side checks: the C-ABI library loads and exports what the header declares, and the
Python shim keeps the reference's preconditions (kernel.py:51-52, :104-105, :188-189)."""
import ctypes
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_functions():
    text = open(os.path.join(ROOT, "include", "dsv3_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(dsv3_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from dsv3_b200 import _lib
    names = header_functions()
    assert "dsv3_fp8_gemm" in names and "dsv3_act_quant" in names and "dsv3_weight_dequant" in names
    cdll = ctypes.CDLL(_lib.LIB_PATH)
    for n in names:
        assert hasattr(cdll, n), f"{n} is declared in include/dsv3_b200.h but not exported"
    assert set(_lib.EXPORTS) <= set(names)


def test_version_and_strerror():
    from dsv3_b200 import _lib
    assert _lib.lib.dsv3_version() >= 100
    assert _lib.lib.dsv3_strerror(0) == b"ok"
    assert b"workspace" in _lib.lib.dsv3_strerror(_lib.ERR_WORKSPACE)


def test_argument_validation_without_gpu():
    """Checks that run before any CUDA call."""
    from dsv3_b200 import _lib
    L = _lib.lib
    assert L.dsv3_act_quant(None, -1, 128, 128, 0, None, None, None) == _lib.ERR_INVALID_ARGUMENT
    assert L.dsv3_act_quant(None, 4, 100, 128, 0, None, None, None) == _lib.ERR_INVALID_ARGUMENT
    assert b"divisible" in L.dsv3_last_error()
    assert L.dsv3_act_quant(None, 4, 128, 128, 7, None, None, None) == _lib.ERR_INVALID_ARGUMENT
    assert L.dsv3_act_quant(None, 4, 128, 128, 0, None, None, None) == _lib.ERR_INVALID_ARGUMENT   # null
    assert L.dsv3_act_quant(None, 0, 128, 128, 0, None, None, None) == _lib.OK                       # empty
    assert L.dsv3_weight_dequant(None, None, 0, 64, 128, None, None) == _lib.OK
    assert L.dsv3_weight_dequant(None, None, 8, 64, 128, None, None) == _lib.ERR_INVALID_ARGUMENT
    assert L.dsv3_fp8_gemm(None, None, None, None, 0, 16, 128, None, None, 0, None) == _lib.OK
    assert L.dsv3_fp8_gemm(None, None, None, None, 4, 16, 128, None, None, 0, None) == _lib.ERR_INVALID_ARGUMENT
    assert L.dsv3_set_gemm_policy(9, 0) == _lib.ERR_INVALID_ARGUMENT
    assert L.dsv3_set_gemm_policy(0, 0) == _lib.OK


def test_plan_and_setters_without_gpu():
    """Host-side planning: the workspace query is pure arithmetic over the shape, the policy and the SM budget."""
    from dsv3_b200 import _lib
    L = _lib.lib
    ws = L.dsv3_fp8_gemm_workspace_bytes
    try:
        assert L.dsv3_set_num_sms(1) == _lib.ERR_INVALID_ARGUMENT and L.dsv3_set_num_sms(-3) == _lib.ERR_INVALID_ARGUMENT
        assert L.dsv3_set_num_sms(0) == _lib.OK
        # prefill-sized problems with more tiles than SMs never split K: no workspace, whichever pair kernel is chosen
        assert ws(4096, 18432, 7168) == 0 and ws(16384, 7168, 2048) == 0 and ws(4096, 1536, 7168) == 0
        # a decode problem with few weight tiles and long K splits K: ticket header + padded partial tiles
        need = ws(8, 7168, 16384)
        assert need > _lib.WORKSPACE_HEADER_BYTES and (need - _lib.WORKSPACE_HEADER_BYTES) % (128 * 16 * 4) == 0
        # pinned kernels that never split ask for nothing; a pinned split factor is reflected in the size
        for policy in (1, 4, 5, 6):
            assert L.dsv3_set_gemm_policy(policy, 0) == _lib.OK
            assert ws(4096, 7168, 2048) == 0
        assert L.dsv3_set_gemm_policy(3, 4) == _lib.OK
        tiles = -(-7168 // 128)
        assert ws(8, 7168, 16384) == _lib.WORKSPACE_HEADER_BYTES + 4 * tiles * 128 * 16 * 4
        # an SM budget changes the plan of a problem that filled the machine before
        assert L.dsv3_set_gemm_policy(0, 0) == _lib.OK
        full = ws(32, 18432, 7168)
        assert L.dsv3_set_num_sms(32) == _lib.OK
        small = ws(32, 18432, 7168)
        assert small <= full
    finally:
        L.dsv3_set_gemm_policy(0, 0)
        L.dsv3_set_num_sms(0)


def test_shim_signatures_match_reference():
    import inspect
    import kernel
    sig = inspect.signature(kernel.act_quant)
    assert list(sig.parameters) == ["x", "block_size", "scale_fmt"]
    assert sig.parameters["block_size"].default == 128 and sig.parameters["scale_fmt"].default is None
    sig = inspect.signature(kernel.weight_dequant)
    assert list(sig.parameters) == ["x", "s", "block_size"] and sig.parameters["block_size"].default == 128
    assert list(inspect.signature(kernel.fp8_gemm).parameters) == ["a", "a_s", "b", "b_s"]


def test_shim_preconditions_raise_like_reference():
    import kernel
    x = torch.zeros(4, 256, dtype=torch.bfloat16)
    with pytest.raises(AssertionError, match="contiguous"):
        kernel.act_quant(x.t())
    with pytest.raises(AssertionError, match="divisible by block_size"):
        kernel.act_quant(torch.zeros(4, 100, dtype=torch.bfloat16))
    w = torch.zeros(4, 256, dtype=torch.uint8).view(torch.float8_e4m3fn)
    s = torch.zeros(1, 2)
    with pytest.raises(AssertionError, match="2 dimensions"):
        kernel.weight_dequant(w.view(2, 2, 256), s)
    with pytest.raises(AssertionError, match="contiguous"):
        kernel.weight_dequant(w, torch.zeros(2, 3).t())
    with pytest.raises(AssertionError, match="Scaling factor tensors must be contiguous"):
        kernel.fp8_gemm(w, torch.zeros(2, 4).t(), w, s)


def test_no_cpu_fallback():
    import kernel
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        kernel.act_quant(torch.zeros(4, 256, dtype=torch.bfloat16))
    w = torch.zeros(4, 256, dtype=torch.uint8).view(torch.float8_e4m3fn)
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        kernel.weight_dequant(w, torch.zeros(1, 2))
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        kernel.fp8_gemm(w, torch.zeros(4, 2), w, torch.zeros(1, 2))


def test_product_does_not_import_oracle():
    """The oracle is test infrastructure: no file of the package may mention it."""
    pkg = os.path.join(ROOT, "deepseek-v3_b200")
    for base, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(base, f)).read()
                assert "oracle" not in text.lower(), f"{f} refers to the oracle"
