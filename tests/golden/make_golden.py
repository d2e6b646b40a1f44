"""Generate golden vectors by running the reference's own ``inference/kernel.py``.

Usage (from the repository root)::

    # CPU: the reference's Triton kernels under the Triton interpreter
    python tests/golden/make_golden.py --device cpu  --reference-dir <reference>/inference
    # GPU: the reference's Triton kernels compiled for the GPU in the machine
    python tests/golden/make_golden.py --device cuda --reference-dir <copy of inference/>

The reference directory is only read (imported); nothing of it is written into
the fixtures except the outputs its functions return.  Inputs come from seeded
numpy PCG64 streams (``oracle.oracle.randn_bf16``) so the tests can rebuild them;
their SHA-256 digests are stored to detect drift.

Outputs: ``tests/golden/ref_cpu_interp.npz`` or ``tests/golden/ref_gpu_triton.npz``.
Large outputs are stored as a digest plus a leading slice.
"""
from __future__ import annotations

import argparse
import hashlib
import importlib.util
import os
import sys
import time

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

FULL_LIMIT = 1 << 17  # arrays up to 128 KiB are stored whole


def sha(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def special_act_input():
    """[8, 512] bf16 with the corner cases of act_quant: an all-zero block, a block
    below the 1e-4 clamp, exact ties on the e4m3 grid, a block whose amax element
    maps to exactly 448, huge and tiny magnitudes, negative zero."""
    import torch
    from oracle import oracle as O
    x = O.randn_bf16((8, 512), 77, 1.0).float()
    x[0, 0:128] = 0.0
    x[0, 128:256] = torch.linspace(-9e-5, 9e-5, 128)
    # ties: amax 448 -> s = 1 exactly; values k + 0.5 on the e4m3 grid spacing
    x[1, 0:128] = torch.tensor([448.0] + [float(v) for v in np.arange(0.5, 64.0, 0.5)][:127])
    x[1, 128:256] = torch.tensor([-448.0] + [-(16.0 + 1.0 * i) for i in range(127)])
    x[2, 0:128] = x[2, 0:128] * 3.0e38 / 4.0
    x[2, 128:256] = x[2, 128:256] * 1e-30
    x[3, 0:128] = torch.where(torch.arange(128) % 2 == 0, torch.tensor(-0.0), torch.tensor(1.0))
    x[4, 0:128] = 224.0 * torch.ones(128)
    x[4, 5] = 17.0
    x[4, 6] = 18.0
    x[4, 7] = 19.0
    return x.to(torch.bfloat16)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--device", choices=["cpu", "cuda"], default="cpu")
    ap.add_argument("--reference-dir", required=True, help="the reference's inference/ directory (read only)")
    ap.add_argument("--out", default=None)
    args = ap.parse_args()

    if args.device == "cpu":
        os.environ["TRITON_INTERPRET"] = "1"
    import torch
    import triton
    from oracle import oracle as O

    spec = importlib.util.spec_from_file_location("_reference_kernel", os.path.join(args.reference_dir, "kernel.py"))
    ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref)

    torch.set_default_dtype(torch.bfloat16)
    dev = args.device

    def ref_gemm(a, a_s, b, b_s):
        if dev == "cuda":
            return ref.fp8_gemm(a, a_s, b, b_s)
        # the autotuner needs a GPU driver: call the undecorated kernel with the
        # allocation logic of kernel.py:190-194 (results do not depend on the tile)
        K = a.size(-1)
        M = a.numel() // K
        N = b.size(0)
        c = a.new_empty(*a.size()[:-1], N, dtype=torch.get_default_dtype())
        grid = (triton.cdiv(M, 16), triton.cdiv(N, 32))
        ref.fp8_gemm_kernel.fn[grid](a, b, c, a_s, b_s, M, N, K,
                                     BLOCK_SIZE_M=16, BLOCK_SIZE_N=32, BLOCK_SIZE_K=128)
        return c

    out = {}
    meta = {"device": dev, "torch": torch.__version__, "triton": triton.__version__,
            "gpu": torch.cuda.get_device_name(0) if dev == "cuda" else "none"}

    def put(name, t):
        if t.dtype == torch.bfloat16:
            a = t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)
        elif t.dtype == torch.float8_e4m3fn:
            a = t.detach().cpu().contiguous().view(torch.uint8).numpy()
        else:
            a = t.detach().cpu().contiguous().numpy()
        out[name + ".sha"] = np.array(sha(a))
        out[name + ".shape"] = np.array(a.shape, dtype=np.int64)
        if a.nbytes <= FULL_LIMIT:
            out[name] = a
        else:
            out[name + ".head"] = a.reshape(-1)[:4096].copy()

    # (name, M, N, K, seed); sizes the CPU interpreter finishes in seconds
    cases = [("cfg1", 16, 2048, 1024, 0), ("edge", 3, 192, 256, 1), ("wkv_a_m1", 1, 576, 7168, 2)]
    if dev == "cuda":
        cases += [("expert_w13_m256", 256, 2048, 7168, 3), ("expert_w2_m64", 64, 7168, 2048, 4),
                  ("wkv_a_m1024", 1024, 576, 7168, 5), ("wq_b_tp8_m4096", 4096, 3072, 1536, 6)]
    t0 = time.time()
    for name, M, N, K, seed in cases:
        x, w, wq, ws = O.make_case(M, N, K, seed)
        out[f"{name}.in.x.sha"] = np.array(sha(x.view(torch.int16).numpy()))
        out[f"{name}.in.wq.sha"] = np.array(sha(wq.view(torch.uint8).numpy()))
        out[f"{name}.in.ws.sha"] = np.array(sha(ws.numpy()))
        xd, wqd, wsd = x.to(dev), wq.to(dev), ws.to(dev)
        xq, xs = ref.act_quant(xd)
        put(f"{name}.act_quant.y", xq)
        put(f"{name}.act_quant.s", xs)
        put(f"{name}.fp8_gemm.c", ref_gemm(xq, xs, wqd, wsd))
        if N * K <= (1 << 23):
            put(f"{name}.weight_dequant.y", ref.weight_dequant(wqd, wsd))
        print(f"[{time.time() - t0:6.1f}s] {name} done", flush=True)

    # act_quant corner cases, both scale formats
    xs_in = special_act_input()
    out["special.in.x"] = xs_in.view(torch.int16).numpy().view(np.uint16)
    for fmt in (None, "ue8m0"):
        tag = "special" if fmt is None else "special_ue8m0"
        y, s = ref.act_quant(xs_in.to(dev), 128, fmt)
        put(f"{tag}.act_quant.y", y)
        put(f"{tag}.act_quant.s", s)
    x1 = O.randn_bf16((16, 1024), 1, 1.0).to(dev)
    y, s = ref.act_quant(x1, 128, "ue8m0")
    put("cfg1_ue8m0.act_quant.y", y)
    put("cfg1_ue8m0.act_quant.s", s)

    if dev == "cuda":
        # bit-exactness at scale: digests only
        xb = O.randn_bf16((4096, 7168), 11, 1.0).to(dev)
        y, s = ref.act_quant(xb)
        put("big.act_quant.y", y)
        put("big.act_quant.s", s)
        xb = O.randn_bf16((2048, 2048), 12, 30.0).to(dev)
        y, s = ref.act_quant(xb)
        put("big30.act_quant.y", y)
        put("big30.act_quant.s", s)
        _, _, wq, ws = O.make_case(1, 4096, 512, 13)
        put("wkv_b_tp8.weight_dequant.y", ref.weight_dequant(wq.to(dev), ws.to(dev)))

    out["meta"] = np.array(repr(meta))
    path = args.out or os.path.join(HERE, "ref_cpu_interp.npz" if dev == "cpu" else "ref_gpu_triton.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes", meta)


if __name__ == "__main__":
    main()
