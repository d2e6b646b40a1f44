"""GPU parity of act_quant / weight_dequant / weight_quant through the drop-in module.

Bit-exactness is judged against golden vectors produced by the reference's own Triton
kernels compiled for the GPU (tests/golden/ref_gpu_triton.npz); against the CPU oracle the
only admissible differences are those of the approximate division (see gpu_util)."""
import hashlib

import numpy as np
import pytest
import torch

from oracle import oracle as O
from gpu_util import u8, bf16_bits, f32_bits, compare_act_quant_with_oracle

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def K():
    import kernel
    torch.set_default_dtype(torch.bfloat16)
    yield kernel
    torch.set_default_dtype(torch.float32)


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


@pytest.mark.parametrize("shape,seed,std", [((16, 1024), 1, 1.0), ((1, 128), 2, 1.0), ((3, 7168), 3, 1.0),
                                            ((2, 5, 256), 4, 10.0), ((257, 2048), 5, 0.01), ((4096, 7168), 11, 1.0)])
def test_act_quant_vs_oracle(K, shape, seed, std):
    x = O.randn_bf16(shape, seed, std)
    y, s = K.act_quant(x.cuda())
    assert y.shape == x.shape and y.dtype == torch.float8_e4m3fn
    assert s.shape == (*shape[:-1], shape[-1] // 128) and s.dtype == torch.float32
    compare_act_quant_with_oracle(x, y, s)


@pytest.mark.parametrize("block", [8, 32, 64, 256, 1024])
def test_act_quant_other_block_sizes(K, block):
    x = O.randn_bf16((6, 2048), 20 + block, 1.0)
    y, s = K.act_quant(x.cuda(), block)
    assert s.shape == (6, 2048 // block)
    compare_act_quant_with_oracle(x, y, s, block)


def test_act_quant_ue8m0(K):
    x = O.randn_bf16((16, 1024), 1, 1.0)
    y, s = K.act_quant(x.cuda(), 128, "ue8m0")
    compare_act_quant_with_oracle(x, y, s, 128, "ue8m0")   # power-of-two scales must be equal


def test_act_quant_special_values(K, golden_cpu):
    x = torch.from_numpy(golden_cpu["special.in.x"].view(np.int16)).view(torch.bfloat16)
    y, s = K.act_quant(x.cuda())
    s, yb = s.cpu(), u8(y)
    floor = np.float32(1e-4) / np.float32(448.0)
    assert abs(s[0, 0].item() - floor) <= 2 * np.spacing(floor) and (yb[0, :128] == 0).all()  # zero block
    assert s[0, 1].item() == s[0, 0].item()                                                  # below the clamp
    assert s[1, 0].item() == 1.0 and yb[1, 0] == 0x7E and yb[1, 128] == 0xFE                 # +-448
    vals = O.weight_dequant(y[1:2, :128].cpu().contiguous(), torch.ones(1, 1)).float()[0]
    assert vals[1].item() == 0.5 and vals[33].item() == 16.0 and vals[35].item() == 18.0     # ties to even
    assert (yb[3, 0:128:2] == 0x80).all()                                                    # -0 keeps its sign
    rows = [1, 3, 4, 5, 6, 7]
    compare_act_quant_with_oracle(x[rows].contiguous(), y[rows].contiguous(), s[rows].contiguous())


def test_act_quant_empty(K):
    y, s = K.act_quant(torch.empty(0, 256, dtype=torch.bfloat16, device="cuda"))
    assert y.shape == (0, 256) and s.shape == (0, 2)


GOLD_CASES = [("cfg1", 16, 2048, 1024, 0), ("edge", 3, 192, 256, 1), ("wkv_a_m1", 1, 576, 7168, 2),
              ("expert_w13_m256", 256, 2048, 7168, 3), ("expert_w2_m64", 64, 7168, 2048, 4),
              ("wkv_a_m1024", 1024, 576, 7168, 5), ("wq_b_tp8_m4096", 4096, 3072, 1536, 6)]


@pytest.mark.parametrize("name,M,N,Kd,seed", GOLD_CASES)
def test_act_quant_bit_exact_vs_gpu_reference(K, golden_gpu, name, M, N, Kd, seed):
    x = O.randn_bf16((M, Kd), seed * 2 + 1, 1.0)
    y, s = K.act_quant(x.cuda())
    assert sha(f32_bits(s).view(np.float32)) == str(golden_gpu[f"{name}.act_quant.s.sha"])
    assert sha(u8(y)) == str(golden_gpu[f"{name}.act_quant.y.sha"])


def test_act_quant_bit_exact_at_scale_and_special(K, golden_gpu):
    for tag, shape, seed, std in (("big", (4096, 7168), 11, 1.0), ("big30", (2048, 2048), 12, 30.0)):
        x = O.randn_bf16(shape, seed, std)
        y, s = K.act_quant(x.cuda())
        assert sha(f32_bits(s).view(np.float32)) == str(golden_gpu[f"{tag}.act_quant.s.sha"]), tag
        assert sha(u8(y)) == str(golden_gpu[f"{tag}.act_quant.y.sha"]), tag
    x = torch.from_numpy(golden_gpu["special.in.x"].view(np.int16)).view(torch.bfloat16)
    for tag, fmt in (("special", None), ("special_ue8m0", "ue8m0")):
        y, s = K.act_quant(x.cuda(), 128, fmt)
        ref_s, ref_y = golden_gpu[f"{tag}.act_quant.s"], golden_gpu[f"{tag}.act_quant.y"]
        ok = np.isfinite(ref_s) & np.isfinite(s.cpu().numpy())
        assert np.array_equal(np.isfinite(ref_s), np.isfinite(s.cpu().numpy()))
        assert np.array_equal(f32_bits(s)[ok], ref_s.view(np.uint32)[ok]), tag
        okb = np.repeat(ok, 128, axis=1)
        assert np.array_equal(u8(y)[okb], ref_y[okb]), tag
    x = O.randn_bf16((16, 1024), 1, 1.0)
    y, s = K.act_quant(x.cuda(), 128, "ue8m0")
    assert np.array_equal(f32_bits(s), golden_gpu["cfg1_ue8m0.act_quant.s"].view(np.uint32))
    assert np.array_equal(u8(y), golden_gpu["cfg1_ue8m0.act_quant.y"])


@pytest.mark.parametrize("N,Kd,seed", [(2048, 1024, 0), (192, 256, 1), (576, 7168, 2), (4096, 512, 13),
                                       (130, 200, 7), (7, 24, 8), (1, 1, 9)])
def test_weight_dequant_bit_exact_vs_oracle(K, N, Kd, seed):
    w = O.randn_bf16((N, Kd), seed * 2 + 2, 0.02)
    wq, ws = O.weight_quant(w)
    y = K.weight_dequant(wq.cuda(), ws.cuda())
    assert y.dtype == torch.bfloat16 and y.shape == (N, Kd)
    assert np.array_equal(bf16_bits(y), bf16_bits(O.weight_dequant(wq, ws)))


def test_weight_dequant_all_codes(K):
    codes = torch.arange(256, dtype=torch.uint8).repeat(128, 1)            # [128, 256]
    s = torch.tensor([[0.37, 1.0e-3]], dtype=torch.float32)
    y = K.weight_dequant(codes.view(torch.float8_e4m3fn).cuda(), s.cuda())
    ref = O.weight_dequant(codes.view(torch.float8_e4m3fn), s)
    finite = ~torch.isnan(ref.float())
    assert np.array_equal(bf16_bits(y)[finite.numpy()], bf16_bits(ref)[finite.numpy()])
    assert torch.isnan(y.float().cpu()[~finite]).all()


@pytest.mark.parametrize("name,M,N,Kd,seed", [c for c in GOLD_CASES if c[2] * c[3] <= (1 << 23)])
def test_weight_dequant_bit_exact_vs_gpu_reference(K, golden_gpu, name, M, N, Kd, seed):
    _, _, wq, ws = O.make_case(1, N, Kd, seed)
    y = K.weight_dequant(wq.cuda(), ws.cuda())
    assert sha(bf16_bits(y)) == str(golden_gpu[f"{name}.weight_dequant.y.sha"])


def test_weight_dequant_other_block_and_empty(K):
    w = O.randn_bf16((96, 160), 31, 0.02)
    wq, _ = O.weight_quant(w)
    s = torch.rand(3, 5, dtype=torch.float32) + 0.5
    y = K.weight_dequant(wq.cuda(), s.cuda(), 32)
    assert np.array_equal(bf16_bits(y), bf16_bits(O.weight_dequant(wq, s, 32)))
    e = K.weight_dequant(torch.empty(0, 128, dtype=torch.float8_e4m3fn, device="cuda"),
                         torch.empty(0, 1, dtype=torch.float32, device="cuda"))
    assert e.shape == (0, 128)


@pytest.mark.parametrize("N,Kd,seed", [(2048, 1024, 0), (576, 7168, 2), (130, 200, 7), (1, 1, 9)])
def test_weight_quant_bit_exact_vs_oracle(N, Kd, seed):
    import dsv3_b200
    w = O.randn_bf16((N, Kd), seed * 2 + 2, 0.02)
    q, s = dsv3_b200.weight_quant(w.cuda())
    qo, so = O.weight_quant(w)
    assert np.array_equal(f32_bits(s), f32_bits(so)) and np.array_equal(u8(q), u8(qo))


def test_weight_dequant_cache_skips_the_launch_for_an_unchanged_weight():
    """model.py:481 de-quantises wkv_b on every forward of every layer; with the cache on, only the first call launches.
    The cache must notice new values in the parameter and must not outlive it."""
    import dsv3_b200
    import kernel
    from dsv3_b200 import ops
    torch.set_default_dtype(torch.bfloat16)
    try:
        _, _, wq, ws = O.make_case(1, 4096, 512, 13)               # wkv_b at TP=8
        wq, ws = wq.cuda(), ws.cuda()
        ref = O.weight_dequant(wq.cpu(), ws.cpu())
        dsv3_b200.enable_weight_dequant_cache(64 << 20)
        ops.dequant_stats.update(launches=0, hits=0)
        y1 = kernel.weight_dequant(wq, ws)
        y2 = kernel.weight_dequant(wq, ws)
        assert y2 is y1 and ops.dequant_stats == {"launches": 1, "hits": 1}
        assert np.array_equal(bf16_bits(y1), bf16_bits(ref))
        # new values loaded into the same storage (what load_model does): recomputed
        wq.view(torch.uint8).copy_(torch.flip(wq.view(torch.uint8), dims=[0]))
        y3 = kernel.weight_dequant(wq, ws)
        assert ops.dequant_stats["launches"] == 2
        assert np.array_equal(bf16_bits(y3), bf16_bits(O.weight_dequant(wq.cpu(), ws.cpu())))
        # a different weight object is a different entry, even at a recycled address
        wq2 = wq.clone()
        kernel.weight_dequant(wq2, ws)
        assert ops.dequant_stats["launches"] == 3
        # inference-mode tensors have no modification counter: never cached
        with torch.inference_mode():
            wi = wq.clone()
            kernel.weight_dequant(wi, ws); kernel.weight_dequant(wi, ws)
        assert ops.dequant_stats["launches"] == 5
        # off again: every call launches
        dsv3_b200.disable_weight_dequant_cache()
        kernel.weight_dequant(wq, ws); kernel.weight_dequant(wq, ws)
        assert ops.dequant_stats["launches"] == 7
    finally:
        dsv3_b200.disable_weight_dequant_cache()
        torch.set_default_dtype(torch.float32)


@pytest.mark.parametrize("rows,K,fmt", [(1, 128, None), (37, 2048, None), (300, 1408, None), (64, 2304, "ue8m0")])
def test_swiglu_quant_equals_the_three_launch_form_bit_for_bit(rows, K, fmt):
    """`dsv3_swiglu_quant` against `act_quant(F.silu(a) * b)` (model.py:532/633 followed by :158-159): same FP8 codes,
    same scales.  Inputs include magnitudes where exp(-a) overflows or underflows and exact zeros."""
    import dsv3_b200
    import kernel
    import torch.nn.functional as F
    a = O.randn_bf16((rows, K), 700 + rows, 3.0)
    b = O.randn_bf16((rows, K), 701 + rows, 1.0)
    a[0, :8] = torch.tensor([-200.0, 200.0, 0.0, -0.0, 88.0, -88.0, 1e-3, -1e-3]).bfloat16()
    b[0, 8:16] = 0.0
    a, b = a.cuda(), b.cuda()
    y, s = dsv3_b200.swiglu_quant(a, b, fmt)
    y_ref, s_ref = kernel.act_quant(F.silu(a) * b, 128, fmt)
    assert np.array_equal(u8(y), u8(y_ref))
    assert np.array_equal(f32_bits(s), f32_bits(s_ref))
    dsv3_b200.check_device_status()
