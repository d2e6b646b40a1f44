"""The decode-sized Linear (`dsv3_fp8_linear`: act_quant folded into the GEMM, at most 16 rows) and the same kernel
fed already quantised activations (`dsv3_fp8_gemm` with kernel policy 5).

What is checked:
  * against the CPU oracle (`oracle.fp8_gemm` on the FP8 codes the device's act_quant produces -- those are held
    bit for bit against the reference's GPU kernel elsewhere) within the stated fp8_gemm tolerance
    |y - y_ref| <= 1e-2 (|y_ref| + rms(y_ref));
  * the fused entry point and the two-step form (act_quant, then the same kernel on quantised activations) give
    the same bf16 bits: the prologue quantises exactly as act_quant does, for both scale formats;
  * determinism, row counts around the 8-token groups, N that is not a multiple of the 16-row tile, a K tail
    (quantised-activation form only: act_quant itself needs K % 128 == 0), both warp layouts (N <= 4096 / above)
    and cluster sizes 1..8;
  * shapes the kernel does not take are refused with DSV3_ERR_UNSUPPORTED.
"""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from gpu_util import bf16_bits, assert_gemm_close

pytestmark = pytest.mark.gpu

DECODE = 5


@pytest.fixture(autouse=True)
def _env():
    import dsv3_b200
    torch.set_default_dtype(torch.bfloat16)
    yield
    torch.set_default_dtype(torch.float32)
    dsv3_b200.set_gemm_policy(0, 0)
    dsv3_b200.check_device_status()


SHAPES = [  # (M, N, K, seed)
    (1, 576, 7168, 2),        # wkv_a: 36 row tiles, cluster of 8
    (8, 1536, 7168, 80),      # wq_a
    (3, 4096, 512, 81),       # wkv_b slice: four chunks, one per warp, no cluster
    (16, 2048, 1024, 0),      # BASELINE config 1
    (9, 3072, 1536, 82),      # wq_b slice, two token groups
    (5, 7168, 2048, 83),      # expert w2: wide layout (four row tiles per CTA)
    (16, 18432, 256, 84),     # wide layout, two chunks
    (2, 1000, 384, 85),       # N not a multiple of 16
    (7, 16, 128, 86),         # one row tile, one chunk
    (1, 24, 2304, 87),        # 18 chunks over a cluster, tile edge
]


@pytest.mark.parametrize("M,N,Kd,seed", SHAPES)
def test_fused_linear_vs_oracle_and_two_step_form(M, N, Kd, seed):
    import dsv3_b200
    import kernel
    x, _, wq, ws = O.make_case(M, N, Kd, seed)
    xd, wqd, wsd = x.cuda(), wq.cuda(), ws.cuda()
    y = dsv3_b200.fp8_linear(xd, wqd, wsd)
    assert y.shape == (M, N) and y.dtype == torch.bfloat16
    xq, xs = kernel.act_quant(xd)
    assert_gemm_close(y, O.fp8_gemm(xq.cpu(), xs.cpu(), wq, ws))
    dsv3_b200.set_gemm_policy(DECODE, 0)
    y2 = kernel.fp8_gemm(xq, xs, wqd, wsd)
    assert np.array_equal(bf16_bits(y), bf16_bits(y2)), "prologue quantisation differs from act_quant"
    assert np.array_equal(bf16_bits(dsv3_b200.fp8_linear(xd, wqd, wsd)), bf16_bits(y)), "not deterministic"
    # and the tcgen05 path on the same quantised activations agrees within the tolerance
    dsv3_b200.set_gemm_policy(0, 0)
    assert_gemm_close(y, kernel.fp8_gemm(xq, xs, wqd, wsd).cpu())


def test_fused_linear_ue8m0_and_leading_dims():
    import dsv3_b200
    import kernel
    x, _, wq, ws = O.make_case(12, 640, 1024, 88)
    xd = x.cuda().view(3, 4, 1024)
    y = dsv3_b200.fp8_linear(xd, wq.cuda(), ws.cuda(), "ue8m0")
    assert y.shape == (3, 4, 640)
    xq, xs = kernel.act_quant(xd, 128, "ue8m0")
    dsv3_b200.set_gemm_policy(DECODE, 0)
    assert np.array_equal(bf16_bits(y), bf16_bits(kernel.fp8_gemm(xq, xs, wq.cuda(), ws.cuda())))
    assert_gemm_close(y.view(12, 640), O.fp8_gemm(xq.cpu().view(12, 1024), xs.cpu().view(12, 8), wq, ws))


def test_decode_kernel_on_quantised_activations_with_k_tail():
    import dsv3_b200
    import kernel
    M, N, Kd = 6, 200, 208                                    # K % 128 = 80, K % 16 == 0
    x, _, wq, ws = O.make_case(M, N, Kd, 89)
    xp = torch.zeros(M, 256, dtype=torch.bfloat16)
    xp[:, :Kd] = x
    xq, xs = O.act_quant(xp)
    xq = xq.view(torch.uint8)[:, :Kd].contiguous().view(torch.float8_e4m3fn)
    dsv3_b200.set_gemm_policy(DECODE, 0)
    y = kernel.fp8_gemm(xq.cuda(), xs.cuda(), wq.cuda(), ws.cuda())
    assert_gemm_close(y, O.fp8_gemm(xq, xs, wq, ws))


def test_fused_linear_refuses_what_it_cannot_take():
    import dsv3_b200
    x, _, wq, ws = O.make_case(17, 64, 256, 90)
    with pytest.raises(dsv3_b200.Dsv3Error) as e:
        dsv3_b200.fp8_linear(x.cuda(), wq.cuda(), ws.cuda())
    assert e.value.status == -2
    x, _, wq, ws = O.make_case(4, 64, 192, 91)               # K % 128 != 0
    with pytest.raises(dsv3_b200.Dsv3Error) as e:
        dsv3_b200.fp8_linear(x.cuda(), wq.cuda(), ws.cuda())
    assert e.value.status == -2
    import kernel
    xq, xs = kernel.act_quant(O.randn_bf16((40, 256), 92).cuda())
    dsv3_b200.set_gemm_policy(DECODE, 0)
    with pytest.raises(dsv3_b200.Dsv3Error, match="M <= 16"):
        kernel.fp8_gemm(xq, xs, O.make_case(1, 64, 256, 93)[2].cuda(), O.make_case(1, 64, 256, 93)[3].cuda())
