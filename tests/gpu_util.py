"""Helpers shared by the GPU parity tests."""
import numpy as np
import torch

from oracle import oracle as O


def u8(t):
    return t.detach().cpu().contiguous().view(torch.uint8).numpy()


def bf16_bits(t):
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def f32_bits(t):
    return t.detach().cpu().contiguous().numpy().view(np.uint32)


def ulp_distance_f32(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """Distance in units of the last place between positive fp32 bit patterns."""
    return np.abs(a.astype(np.int64) - b.astype(np.int64))


def compare_act_quant_with_oracle(x, y, s, block=128, scale_fmt=None):
    """Checks (y, s) produced on a GPU against the CPU oracle.

    A GPU divides with the approximate full-range division the reference's compiled kernel uses
    (at most 2 ulp from the IEEE quotient); the oracle divides exactly.  Admissible therefore:
      * every scale within 2 ulp of the oracle's (equal for power-of-two "ue8m0" scales);
      * every byte equal to the round-to-nearest-even e4m3 cast of SOME fp32 value within 3 ulp of
        x / s (s = the scale the GPU produced), i.e. between the casts of the two ends of that interval.
    Returns (fraction of scales that differ, fraction of bytes that differ from the oracle's bytes).
    """
    xc, yc, sc = x.detach().cpu(), y.detach().cpu(), s.detach().cpu()
    yo, so = O.act_quant(xc, block, scale_fmt)
    sd = ulp_distance_f32(f32_bits(sc), f32_bits(so))
    fin = np.isfinite(so.numpy())
    assert np.array_equal(np.isfinite(sc.numpy()), fin)
    assert (sd[fin].max() if fin.any() else 0) <= (0 if scale_fmt == "ue8m0" else 2), f"scale differs by {sd[fin].max()} ulp"
    K = xc.size(-1)
    q = xc.double().reshape(-1, K // block, block) / sc.double().reshape(-1, K // block, 1)
    q = q.reshape(-1)
    ok = torch.isfinite(q)
    eps = 3.0 * 2.0 ** -24
    lo = (q - q.abs() * eps).float().clamp(-448, 448).to(torch.float8_e4m3fn).float()
    hi = (q + q.abs() * eps).float().clamp(-448, 448).to(torch.float8_e4m3fn).float()
    yv = yc.reshape(-1).float()
    good = (yv >= lo) & (yv <= hi)
    # zeros: +0 and -0 compare equal as floats, the sign byte must still follow x
    assert bool(good[ok].all()), f"{int((~good[ok]).sum())} bytes are outside the admissible interval"
    yb, yob = u8(yc).reshape(-1), u8(yo).reshape(-1)
    sign_ok = ((yb & 0x80) == (yob & 0x80)) | ~ok.numpy()
    assert sign_ok.all()
    return float((sd != 0).mean()), float((yb != yob)[ok.numpy()].mean() if ok.any() else 0.0)


def assert_gemm_close(y, y_ref, rel=1e-2):
    """|y - y_ref| <= rel * (|y_ref| + rms(y_ref)), the stated fp8_gemm tolerance."""
    ok, ratio = O.gemm_tolerance_ok(y, y_ref, rel)
    assert ok, f"worst |err| / bound = {ratio:.3f}"
    return ratio
