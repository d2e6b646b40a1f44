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
        assert L.stats == {"act_quant_calls": 1, "act_quant_reused": 1, "fused_linear_calls": 0}
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
        # two inputs used alternately, as wq_a(x), wq_b(q), wkv_a(x) of model.py:464-468: both stay remembered
        L.reset_memo()
        x2 = O.randn_bf16((35, 512), 74, 1.0).cuda()
        L.linear(x, q1); L.linear(x2, q3); L.linear(x, q3); L.linear(x2, q1)
        assert (L.stats["act_quant_calls"], L.stats["act_quant_reused"]) == (2, 2)
        # tensors made under inference_mode carry no modification counter: no memo unless the host vouches for them
        L.reset_memo()
        with torch.inference_mode():
            xi = O.randn_bf16((40, 512), 75, 1.0).cuda()
            a1 = L.linear(xi, q1); L.linear(xi, q3)
            assert (L.stats["act_quant_calls"], L.stats["act_quant_reused"]) == (2, 0)
            fake_i = types.SimpleNamespace(gemm_impl="fp8", block_size=128, linear=None)
            dsv3_b200.install_linear(fake_i, assume_no_inplace=True)
            a2 = fake_i.linear(xi, q1); fake_i.linear(xi, q3)
            assert (L.stats["act_quant_calls"], L.stats["act_quant_reused"]) == (3, 1)
            assert torch.equal(a1, a2)
            dsv3_b200.install_linear(fake_i)
        # a few rows: one fused launch, no separate act_quant; within the GEMM tolerance of the two-operator path
        L.reset_memo()
        xs4 = O.randn_bf16((2, 2, 512), 76, 1.0).cuda()
        yf = L.linear(xs4, q1)
        assert L.stats == {"act_quant_calls": 0, "act_quant_reused": 0, "fused_linear_calls": 1}
        xq4, xs4s = kernel.act_quant(xs4)
        assert_gemm_close(yf.reshape(4, 384), kernel.fp8_gemm(xq4, xs4s, q1, q1.scale).reshape(4, 384).cpu())
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


def test_mlp_seam_matches_the_unfused_forward_bit_for_bit():
    """install_mlp: MLP.forward / Expert.forward with SwiGLU folded into the quantisation, against
    w2(F.silu(w1(x)) * w3(x)) on the same operators (model.py:532, 633)."""
    import dsv3_b200
    import kernel
    import torch.nn.functional as F
    torch.set_default_dtype(torch.bfloat16)
    try:
        class Lin:                                     # model.py's Linear: weight with a .scale attribute, bias, scale_fmt
            def __init__(self, N, K, seed, bias=None):
                _, self.weight = _weight(N, K, seed)
                self.bias, self.scale_fmt = bias, None

            def __call__(self, x):
                xq, xs = kernel.act_quant(x, 128, self.scale_fmt)
                y = kernel.fp8_gemm(xq, xs, self.weight, self.weight.scale)
                return y if self.bias is None else y + self.bias

        class RowParallelLinear(Lin):
            pass

        class MLP:
            def __init__(self, dim, inter, row):
                self.w1, self.w3 = Lin(inter, dim, 81), Lin(inter, dim, 82)
                self.w2 = (RowParallelLinear if row else Lin)(dim, inter, 83, bias=torch.randn(dim, device="cuda").bfloat16())

            def forward(self, x):
                return self.w2(F.silu(self.w1(x)) * self.w3(x))

        class Expert(MLP):
            pass

        calls = []
        fake_dist = types.SimpleNamespace(all_reduce=lambda y: calls.append(tuple(y.shape)))
        mod = types.SimpleNamespace(MLP=MLP, Expert=Expert, gemm_impl="fp8", block_size=128, world_size=2, dist=fake_dist)
        x = O.randn_bf16((24, 512), 84, 1.0).cuda()
        dsv3_b200.install_mlp(mod)
        for cls, row in ((MLP, True), (Expert, False)):
            m = cls(512, 384, row)
            want = m.w2(F.silu(m.w1(x)) * m.w3(x))      # the reference's forward, spelled out
            got = m.forward(x)
            assert np.array_equal(bf16_bits(got), bf16_bits(want))
            mod.gemm_impl = "bf16"                      # other modes fall back to the original forward
            assert np.array_equal(bf16_bits(m.forward(x)), bf16_bits(want))
            mod.gemm_impl = "fp8"
        assert calls == [(24, 512)], "the all_reduce of a RowParallelLinear must follow its GEMM (model.py:263-264)"
        dsv3_b200.check_device_status()
    finally:
        torch.set_default_dtype(torch.float32)
