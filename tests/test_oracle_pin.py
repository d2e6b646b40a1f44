"""Pins the CPU oracle against outputs of the reference's own kernel.py.

``ref_cpu_interp.npz`` was produced by ``tests/golden/make_golden.py`` from the
reference run under the Triton CPU interpreter.  That interpreter casts
fp32->e4m3 and fp32->bf16 differently from a GPU (no round-to-nearest-even), so
the comparison applies the interpreter's casts to the oracle's fp32 values: then
every FP8 byte, scale and bf16 bit must agree, which pins everything except the
final rounding; the rounding itself is pinned against torch and ml_dtypes.
"""
import hashlib

import numpy as np
import pytest
import torch

from oracle import oracle as O

CASES = [("cfg1", 16, 2048, 1024, 0), ("edge", 3, 192, 256, 1), ("wkv_a_m1", 1, 576, 7168, 2)]


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def u8(t):
    return t.contiguous().view(torch.uint8).numpy()


def bf16_bits(t):
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def get(g, name):
    """Full array if stored, else (digest, head)."""
    if name in g.files:
        return g[name]
    return None


@pytest.mark.parametrize("name,M,N,K,seed", CASES)
def test_inputs_reproduce(golden_cpu, name, M, N, K, seed):
    x, w, wq, ws = O.make_case(M, N, K, seed)
    assert sha(bf16_bits(x)) == str(golden_cpu[f"{name}.in.x.sha"])
    assert sha(u8(wq)) == str(golden_cpu[f"{name}.in.wq.sha"])
    assert sha(ws.numpy()) == str(golden_cpu[f"{name}.in.ws.sha"])


@pytest.mark.parametrize("name,M,N,K,seed", CASES)
def test_act_quant_matches_reference_run(golden_cpu, name, M, N, K, seed):
    x, _, _, _ = O.make_case(M, N, K, seed)
    y, s = O.act_quant(x)
    ref_s = golden_cpu[f"{name}.act_quant.s"]
    assert np.array_equal(s.numpy().view(np.uint32), ref_s.view(np.uint32)), "scales must be bit-equal"
    # bytes: same fp32 quotient, interpreter's cast
    q = (x.float().view(M, K // 128, 128) / s.unsqueeze(-1)).reshape(M, K).numpy()
    assert np.array_equal(O.e4m3_cast_triton_interpreter(q), golden_cpu[f"{name}.act_quant.y"])
    # and the oracle's own bytes are the RNE cast of that same quotient
    assert np.array_equal(u8(y), u8(torch.from_numpy(q).to(torch.float8_e4m3fn)))
    # both restatements agree
    y2, s2 = O.act_quant_torch(x)
    assert torch.equal(s, s2) and np.array_equal(u8(y), u8(y2))


def test_act_quant_special_and_ue8m0(golden_cpu):
    x = torch.from_numpy(golden_cpu["special.in.x"].view(np.int16)).view(torch.bfloat16)
    for tag, fmt in (("special", None), ("special_ue8m0", "ue8m0")):
        y, s = O.act_quant(x, 128, fmt)
        ref_s = golden_cpu[f"{tag}.act_quant.s"]
        fin = np.isfinite(ref_s)
        assert np.array_equal(s.numpy()[fin].view(np.uint32), ref_s[fin].view(np.uint32))
        assert np.array_equal(np.isfinite(s.numpy()), fin)
        q = (x.float().view(8, 4, 128) / s.unsqueeze(-1)).reshape(8, 512).numpy()
        ok = np.isfinite(q)
        got = O.e4m3_cast_triton_interpreter(np.where(ok, q, 0))
        assert np.array_equal(got[ok], golden_cpu[f"{tag}.act_quant.y"][ok])
    # documented corner cases of the oracle itself
    y, s = O.act_quant(x)
    assert s[0, 0].item() == np.float32(1e-4) / np.float32(448.0)         # all-zero block
    assert (u8(y)[0, :128] == 0).all()
    assert s[0, 1].item() == np.float32(1e-4) / np.float32(448.0)         # below the clamp
    assert s[1, 0].item() == 1.0 and u8(y)[1, 0] == 0x7E                  # 448 -> 0x7e
    assert u8(y)[1, 128] == 0xFE                                          # -448
    # ties round to even: 0.5 -> code for 0.5 exactly; 16.5..: spacing 2 at [16,32)
    vals = O.weight_dequant(y[1:2, :128].contiguous(), torch.ones(1, 1)).float()[0]
    assert vals[1].item() == 0.5 and vals[33].item() == 16.0 and vals[35].item() == 18.0  # 16.5->16, 17.5->18
    # ue8m0: power-of-two scales that are >= the fp32 ones
    y8, s8 = O.act_quant(O.randn_bf16((16, 1024), 1), 128, "ue8m0")
    ref = golden_cpu["cfg1_ue8m0.act_quant.s"]
    assert np.array_equal(s8.numpy().view(np.uint32), ref.view(np.uint32))
    assert ((s8.numpy().view(np.uint32) & 0x7FFFFF) == 0).all()


@pytest.mark.parametrize("name,M,N,K,seed", CASES)
def test_weight_dequant_matches_reference_run(golden_cpu, name, M, N, K, seed):
    _, _, wq, ws = O.make_case(M, N, K, seed)
    y = O.weight_dequant(wq, ws)
    assert torch.equal(y, O.weight_dequant_torch(wq, ws))
    # the interpreter truncates the fp32 product to bf16
    prod = wq.float() * O._expand_block_scale(ws, N, K, 128)
    trunc = bf16_bits(O.bf16_truncate(prod))
    assert sha(trunc) == str(golden_cpu[f"{name}.weight_dequant.y.sha"])
    # RNE and truncation differ by at most one bf16 ulp
    d = bf16_bits(y).astype(np.int32) - trunc.astype(np.int32)
    assert set(np.unique(d)).issubset({0, 1})


@pytest.mark.parametrize("name,M,N,K,seed", CASES)
def test_fp8_gemm_matches_reference_run(golden_cpu, name, M, N, K, seed):
    x, _, wq, ws = O.make_case(M, N, K, seed)
    # feed the reference's own FP8 activations so only the GEMM is compared
    xq = torch.from_numpy(golden_cpu[f"{name}.act_quant.y"]).view(torch.float8_e4m3fn)
    xs = torch.from_numpy(golden_cpu[f"{name}.act_quant.s"])
    c = O.fp8_gemm(xq, xs, wq, ws)
    ref = torch.from_numpy(golden_cpu[f"{name}.fp8_gemm.c"].view(np.int16)).view(torch.bfloat16)
    ok, ratio = O.gemm_tolerance_ok(c, ref)          # |y-y_ref| <= 1e-2 (|y_ref| + rms)
    assert ok, ratio
    # far tighter in practice: within 2 bf16 ulp everywhere (truncation + summation order)
    d = np.abs(bf16_bits(c).astype(np.int32) - bf16_bits(ref).astype(np.int32))
    assert d.max() <= 2
    c2 = O.fp8_gemm_torch(xq, xs, wq, ws)
    d2 = np.abs(bf16_bits(c).astype(np.int32) - bf16_bits(c2).astype(np.int32))
    assert d2.max() <= 1 and (d2 != 0).mean() < 1e-2


def test_e4m3_cast_all_bf16_inputs():
    """RNE/saturating cast of the C oracle == torch == ml_dtypes on every bf16 value in range."""
    import ml_dtypes
    bits = np.arange(65536, dtype=np.uint32).astype(np.uint16)
    f = (bits.astype(np.uint32) << 16).view(np.float32)
    f = f[np.isfinite(f) & (np.abs(f) <= 448.0)]
    out = np.empty(f.size, np.uint8)
    O.lib().orc_f32_to_e4m3_array(f.ctypes.data, f.size, out.ctypes.data)
    assert np.array_equal(out, torch.from_numpy(f).to(torch.float8_e4m3fn).view(torch.uint8).numpy())
    assert np.array_equal(out, f.astype(ml_dtypes.float8_e4m3fn).view(np.uint8))
    # saturation beyond 448 and NaN
    sat = np.float32([449.0, 464.0, 1e9, np.inf, -500.0, np.nan])
    o2 = np.empty(6, np.uint8)
    O.lib().orc_f32_to_e4m3_array(sat.ctypes.data, 6, o2.ctypes.data)
    assert list(o2) == [0x7E, 0x7E, 0x7E, 0x7E, 0xFE, 0x7F]


def test_e4m3_decode_table():
    import ml_dtypes
    tab = np.arange(256, dtype=np.uint8).view(ml_dtypes.float8_e4m3fn).astype(np.float32)
    mine = np.float32([O.lib().orc_e4m3_to_f32(int(b)) for b in range(256)])
    assert np.array_equal(np.isnan(tab), np.isnan(mine))
    ok = ~np.isnan(tab)
    assert np.array_equal(tab[ok], mine[ok])


def test_weight_quant_round_trip_and_restatements():
    w = O.randn_bf16((300, 200), 5, 0.02)
    q, s = O.weight_quant(w)
    q2, s2 = O.weight_quant_torch(w)
    assert torch.equal(s, s2) and np.array_equal(u8(q), u8(q2))
    assert s.shape == (3, 2)
    back = O.weight_dequant(q, s).float()
    # e4m3 has 3 mantissa bits: relative error <= 2^-4 of the block amax
    blk = O._expand_block_scale(s, 300, 200, 128) * 448.0
    assert ((back - w.float()).abs() <= blk * 2 ** -4 + 1e-12).all()


# ---------------------------------------------------------------------------------------
# Second pin: outputs of the reference's Triton kernels compiled for and run on a B200
# (tests/golden/ref_gpu_triton.npz, made by tests/golden/make_golden.py --device cuda).
# ---------------------------------------------------------------------------------------
GPU_CASES = CASES + [("expert_w13_m256", 256, 2048, 7168, 3), ("expert_w2_m64", 64, 7168, 2048, 4),
                     ("wkv_a_m1024", 1024, 576, 7168, 5)]


@pytest.mark.parametrize("name,M,N,K,seed", GPU_CASES)
def test_oracle_vs_gpu_reference_act_quant(golden_gpu, name, M, N, K, seed):
    from gpu_util import compare_act_quant_with_oracle
    if f"{name}.act_quant.y" not in golden_gpu.files:
        pytest.skip("only a digest is stored for this case")
    x, _, _, _ = O.make_case(M, N, K, seed)
    y = torch.from_numpy(golden_gpu[f"{name}.act_quant.y"]).view(torch.float8_e4m3fn)
    s = torch.from_numpy(golden_gpu[f"{name}.act_quant.s"])
    frac_s, frac_y = compare_act_quant_with_oracle(x, y, s)
    assert frac_y < 0.01        # differences only at (near-)ties of the quotient


@pytest.mark.parametrize("name,M,N,K,seed", GPU_CASES)
def test_oracle_vs_gpu_reference_weight_dequant(golden_gpu, name, M, N, K, seed):
    if N * K > (1 << 23):
        pytest.skip("not stored")
    _, _, wq, ws = O.make_case(1, N, K, seed)
    assert sha(bf16_bits(O.weight_dequant(wq, ws))) == str(golden_gpu[f"{name}.weight_dequant.y.sha"])


@pytest.mark.parametrize("name,M,N,K,seed", CASES)
def test_oracle_vs_gpu_reference_fp8_gemm(golden_gpu, name, M, N, K, seed):
    _, _, wq, ws = O.make_case(M, N, K, seed)
    xq = torch.from_numpy(golden_gpu[f"{name}.act_quant.y"]).view(torch.float8_e4m3fn)
    xs = torch.from_numpy(golden_gpu[f"{name}.act_quant.s"])
    ref = torch.from_numpy(golden_gpu[f"{name}.fp8_gemm.c"].view(np.int16)).view(torch.bfloat16)
    ok, ratio = O.gemm_tolerance_ok(O.fp8_gemm(xq, xs, wq, ws), ref)
    assert ok, ratio


def test_oracle_vs_gpu_reference_special(golden_gpu):
    from gpu_util import compare_act_quant_with_oracle
    x = torch.from_numpy(golden_gpu["special.in.x"].view(np.int16)).view(torch.bfloat16)
    rows = [0, 1, 3, 4, 5, 6, 7]           # row 2 holds inf / overflow to inf
    for tag, fmt in (("special", None), ("special_ue8m0", "ue8m0")):
        y = torch.from_numpy(golden_gpu[f"{tag}.act_quant.y"]).view(torch.float8_e4m3fn)[rows].contiguous()
        s = torch.from_numpy(golden_gpu[f"{tag}.act_quant.s"])[rows].contiguous()
        compare_act_quant_with_oracle(x[rows].contiguous(), y, s, 128, fmt)
