"""The linear() seam (model.py:131-163): same three branches as the reference, identical results to
act_quant + fp8_gemm, and one quantisation for Linears that share an input."""
import types

import numpy as np
import pytest
import torch

from oracle import oracle as O
from gpu_util import bf16_bits, assert_gemm_close

pytestmark = pytest.mark.gpu


def _weight(N, K, seed):
    import dsv3_b200
    w = O.randn_bf16((N, K), seed, 0.02).cuda()
    q, s = dsv3_b200.weight_quant(w)
    q.scale = s                      # the alias model.py:187 creates
    return w, q


def test_linear_seam_matches_unfused_path_and_reuses_quantisation():
    import dsv3_b200
    import kernel
    from dsv3_b200 import linear_seam as L
    torch.set_default_dtype(torch.bfloat16)
    try:
        x = O.randn_bf16((5, 7, 512), 71, 1.0).cuda()
        w1, q1 = _weight(384, 512, 72)
        w3, q3 = _weight(256, 512, 73)
        L.reset_memo()
        y1 = L.linear(x, q1)
        y3 = L.linear(x, q3)                       # same input object: quantised once
        assert L.stats == {"act_quant_calls": 1, "act_quant_reused": 1}
        xq, xs = kernel.act_quant(x)
        assert np.array_equal(bf16_bits(y1), bf16_bits(kernel.fp8_gemm(xq, xs, q1, q1.scale)))
        assert np.array_equal(bf16_bits(y3), bf16_bits(kernel.fp8_gemm(xq, xs, q3, q3.scale)))
        assert_gemm_close(y1.reshape(35, 384), O.fp8_gemm(xq.cpu().reshape(35, 512), xs.cpu().reshape(35, 4),
                                                           q1.cpu(), q1.scale.cpu()))
        # an in-place update of x invalidates the memo
        x.mul_(2)
        L.linear(x, q1)
        assert L.stats["act_quant_calls"] == 2
        # a different tensor does too, even with equal contents
        L.linear(x.clone(), q1)
        assert L.stats["act_quant_calls"] == 3
        # bias, bf16 weights and the bf16 GEMM mode follow model.py:153-157
        b = torch.randn(384, device="cuda")
        assert torch.equal(L.linear(x, q1, b), L.linear(x, q1) + b)
        assert torch.equal(L.linear(x, w1), torch.nn.functional.linear(x, w1))
        ref_bf16 = torch.nn.functional.linear(x, kernel.weight_dequant(q1, q1.scale))
        assert torch.equal(L.linear(x, q1, gemm_impl="bf16"), ref_bf16)
        # install_linear rebinds a module-level `linear` and honours the module's globals at call time
        fake = types.SimpleNamespace(gemm_impl="bf16", block_size=128, linear=None)
        dsv3_b200.install_linear(fake)
        assert torch.equal(fake.linear(x, q1), ref_bf16)
        fake.gemm_impl = "fp8"
        assert np.array_equal(bf16_bits(fake.linear(x, q1)), bf16_bits(L.linear(x, q1)))
        dsv3_b200.check_device_status()
    finally:
        torch.set_default_dtype(torch.float32)
