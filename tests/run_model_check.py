#!/usr/bin/env python
"""Runs the reference's unchanged ``model.py`` on top of the drop-in ``kernel`` module and, on the
same GPU and the same random weights, on top of the reference's own ``kernel.py``; compares logits
and greedy tokens.

    python tests/run_model_check.py --reference-dir <DeepSeek-V3>/inference \
        [--config configs/config_16B.json] [--n-layers 27] [--batch 32] [--prompt-len 1024] [--new-tokens 32] [--seams] [--graph]

A tool, not a pytest module: it needs the reference's source tree, which the committed tests must not depend on.

What it checks (the end-to-end parity targets): relative RMS difference of the logits of the prefill
and of every decode step (target <= 2e-2), and the fraction of decode steps whose greedy token is the
same (target >= 99 %), evaluated teacher-forced on the reference's token stream so that one early flip
does not cascade.  Because the reference's own result depends on which of its tile configurations the
autotuner picked, the same comparison is also made between two of the reference's configurations
(16x32 and 64x128 tiles): that is the reference's numerical noise on the model at hand, and on a
random-initialised model (near-uniform logits) it can exceed the targets by itself.

To make the token criterion decidable on such a model, the match is also reported over the DECIDABLE steps only:
those where the reference's margin between its best and second-best logit exceeds four times the RMS difference
between the reference's own two tile configurations at that step.  Where the margin is smaller, the reference's
greedy token is decided by its own rounding noise and no implementation, the reference included, can be expected to
reproduce it.  `pass_decidable` is: token match >= 99 % over the decidable steps, and logits within 2e-2 relative
RMS or within 1.25 x the reference's own noise, whichever is larger.

--graph additionally captures one decode step (seqlen 1 at a fixed position, seams installed: no host
synchronisation is left in the forward) in a CUDA graph and reports eager against replayed time per step.

Notes taken from the reference: ``model.gemm_impl`` must be set to "fp8" or ``linear()`` never reaches
``act_quant``/``fp8_gemm`` (model.py:16,155); weights are written in place because replacing a
``Parameter`` drops the ``weight.scale`` alias (model.py:187); Linears whose in_features is not a
multiple of 128 cannot be FP8 in the reference either (``act_quant`` asserts, kernel.py:52) and are
given bf16 weights for both runs.  Nothing of the reference is copied: it is imported from the
directory given on the command line.
"""
from __future__ import annotations

import argparse
import importlib.util
import json
import os
import sys
import time

HERE = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "deepseek-v3_b200")


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference-dir", required=True, help="the reference's inference/ directory")
    ap.add_argument("--config", default="configs/config_16B.json", help="relative to --reference-dir")
    ap.add_argument("--n-layers", type=int, default=4)
    ap.add_argument("--batch", type=int, default=4)
    ap.add_argument("--prompt-len", type=int, default=128)
    ap.add_argument("--new-tokens", type=int, default=32)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--seams", action="store_true",
                    help="also run with dsv3_b200.install_linear / install_moe (shared quantisation, grouped MoE)")
    ap.add_argument("--graph", action="store_true", help="with --seams: time one decode step eagerly and as a replayed CUDA graph")
    ap.add_argument("--skip-noise", action="store_true", help="skip the two fixed-tile runs of the reference")
    ap.add_argument("--out", default=None, help="write the result as JSON to this file")
    args = ap.parse_args()

    import torch
    from torch import nn

    sys.path.insert(0, HERE)                     # our kernel.py shadows the reference's
    sys.path.append(args.reference_dir)
    import kernel as ours
    import dsv3_b200
    import model as M                            # the reference's model.py, unchanged
    assert M.act_quant is ours.act_quant, "model.py did not bind to the drop-in kernel module"
    spec = importlib.util.spec_from_file_location("_reference_kernel", os.path.join(args.reference_dir, "kernel.py"))
    ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref)

    torch.cuda.set_device(0)
    torch.set_default_dtype(torch.bfloat16)
    torch.manual_seed(args.seed)
    M.gemm_impl = "fp8"
    cfg = json.load(open(os.path.join(args.reference_dir, args.config)))
    cfg.update(dtype="fp8", n_layers=args.n_layers, max_batch_size=args.batch,
               max_seq_len=args.prompt_len + args.new_tokens + 8)
    cfg["n_dense_layers"] = min(cfg.get("n_dense_layers", 1), max(1, args.n_layers - 1))
    margs = M.ModelArgs(**cfg)
    with torch.device("cuda"):
        model = M.Transformer(margs)

    # ---- random initialisation, in place
    n_fp8 = n_bf16_fallback = 0
    with torch.no_grad():
        for name, mod in model.named_modules():
            if isinstance(mod, M.Linear) and mod.weight.element_size() == 1:
                N, K = mod.weight.shape
                w = (torch.randn(N, K, device="cuda", dtype=torch.float32) * 0.02).to(torch.bfloat16)
                if K % 128 != 0:
                    mod.weight = nn.Parameter(w)          # bf16 Linear: linear() takes the F.linear branch
                    mod.scale = None
                    n_bf16_fallback += 1
                else:
                    q, s = dsv3_b200.weight_quant(w)
                    mod.weight.data.copy_(q)
                    mod.scale.data.copy_(s)
                    n_fp8 += 1
        for name, p in model.named_parameters():
            if p.element_size() == 1 or name.endswith("scale"):
                continue
            if "norm" in name:
                p.data.fill_(1.0)
            elif name.endswith("bias"):
                p.data.normal_(0.0, 0.01)
            elif p.dim() >= 2:
                p.data.normal_(0.0, 0.02)     # embedding, gate, head, bf16 Linears
    torch.cuda.synchronize()

    tokens = torch.randint(0, margs.vocab_size, (args.batch, args.prompt_len), device="cuda")

    def use(impl):
        M.act_quant, M.weight_dequant, M.fp8_gemm = impl.act_quant, impl.weight_dequant, impl.fp8_gemm

    @torch.inference_mode()
    def run(impl, forced=None):
        """Prefill + greedy decode; with `forced`, feeds those tokens instead of its own choices."""
        use(impl)
        logits = [model.forward(tokens, 0)]
        chosen = [logits[-1].argmax(dim=-1)]
        t_dec = 0.0
        for i in range(args.new_tokens - 1):
            nxt = (forced[i] if forced is not None else chosen[-1]).view(-1, 1)
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            lg = model.forward(nxt, args.prompt_len + i)
            torch.cuda.synchronize()
            t_dec += time.perf_counter() - t0
            logits.append(lg)
            chosen.append(lg.argmax(dim=-1))
        return torch.stack(logits).float(), torch.stack(chosen), t_dec / max(1, args.new_tokens - 1)

    class FixedTile:
        """The reference's kernels with fp8_gemm pinned to one of its own tile configurations
        (kernel.py:113-116) instead of the autotuned choice: the reference's results depend on that
        choice (different MMA instruction, different summation order), which gives the size of the
        reference's own numerical noise on this model."""
        def __init__(self, bm, bn):
            self.bm, self.bn = bm, bn
            self.act_quant, self.weight_dequant = ref.act_quant, ref.weight_dequant

        def fp8_gemm(self, a, a_s, b, b_s):
            import triton
            K = a.size(-1)
            Mr = a.numel() // K
            N = b.size(0)
            c = a.new_empty(*a.size()[:-1], N, dtype=torch.get_default_dtype())
            grid = (triton.cdiv(Mr, self.bm), triton.cdiv(N, self.bn))
            ref.fp8_gemm_kernel.fn[grid](a, b, c, a_s, b_s, Mr, N, K, BLOCK_SIZE_M=self.bm, BLOCK_SIZE_N=self.bn,
                                         BLOCK_SIZE_K=128, num_warps=8, num_stages=4)
            return c

    run(ref)                                              # warm-up: Triton JIT + autotune
    lg_ref, tok_ref, dt_ref = run(ref)
    run(ours, forced=tok_ref)
    lg_ours, tok_ours, dt_ours = run(ours, forced=tok_ref)
    dsv3_b200.check_device_status()
    if args.skip_noise:
        lg_small = lg_large = lg_ref
        tok_small = tok_large = tok_ref
    else:
        small, large = FixedTile(16, 32), FixedTile(64, 128)
        run(small, forced=tok_ref)
        lg_small, tok_small, _ = run(small, forced=tok_ref)
        run(large, forced=tok_ref)
        lg_large, tok_large, _ = run(large, forced=tok_ref)
    use(ours)
    seam = None
    graph_res = None
    if args.seams:
        orig_linear, orig_moe, orig_mlp, orig_expert = M.linear, M.MoE.forward, M.MLP.forward, M.Expert.forward
        dsv3_b200.install_linear(M, assume_no_inplace=True)      # model.py never modifies a projection's input in place
        dsv3_b200.install_moe(M)
        dsv3_b200.install_mlp(M)
        dsv3_b200.enable_weight_dequant_cache(2 << 30)           # wkv_b of every layer (model.py:481)
        run(ours, forced=tok_ref)
        lg_seam, tok_seam, dt_seam = run(ours, forced=tok_ref)
        dsv3_b200.check_device_status()
        seam = (lg_seam, tok_seam, dt_seam)
        if args.graph:
            # one decode step at a fixed position: with both seams installed the forward has no host synchronisation
            pos = args.prompt_len + args.new_tokens - 2
            nxt = tok_ref[-2].view(-1, 1).clone()
            side = torch.cuda.Stream()
            with torch.cuda.stream(side), torch.inference_mode():
                for _ in range(2):
                    eager_out = model.forward(nxt, pos)
                side.synchronize()
                t0 = time.perf_counter()
                for _ in range(10):
                    eager_out = model.forward(nxt, pos)
                side.synchronize()
                eager_ms = (time.perf_counter() - t0) / 10 * 1e3
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=side):
                    graph_out = model.forward(nxt, pos)
                g.replay()
                side.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(10):
                    g.replay()
                e1.record()
                side.synchronize()
                graph_res = {"position": pos, "eager_ms_per_step": eager_ms, "replayed_ms_per_step": e0.elapsed_time(e1) / 10,
                             "same_logits_as_eager": bool(torch.equal(graph_out, eager_out))}
            dsv3_b200.check_device_status()
        dsv3_b200.disable_weight_dequant_cache()
        M.linear, M.MoE.forward, M.MLP.forward, M.Expert.forward = orig_linear, orig_moe, orig_mlp, orig_expert

    def rel_rms(a, b):
        return ((a - b).pow(2).mean().sqrt() / b.pow(2).mean().sqrt()).item()

    per_step = [rel_rms(lg_ours[i], lg_ref[i]) for i in range(lg_ref.size(0))]
    match = (tok_ours == tok_ref).float().mean().item()
    noise = [rel_rms(lg_small[i], lg_large[i]) for i in range(lg_ref.size(0))]
    noise_match = (tok_small == tok_large).float().mean().item()
    # decidable steps: reference margin (best minus second-best logit) against the reference's own tile-config noise
    top2 = lg_ref.topk(2, dim=-1).values                                     # [steps, batch, 2]
    margin = top2[..., 0] - top2[..., 1]
    sigma = (lg_small - lg_large).pow(2).mean(dim=-1).sqrt()                 # [steps, batch]
    decidable = margin > 4.0 * sigma
    n_dec = int(decidable.sum())
    match_dec = ((tok_ours == tok_ref) & decidable).sum().item() / max(1, n_dec)
    noise_match_dec = ((tok_small == tok_large) & decidable).sum().item() / max(1, n_dec)
    vs_small = max(rel_rms(lg_ours[i], lg_small[i]) for i in range(lg_ref.size(0)))
    vs_large = max(rel_rms(lg_ours[i], lg_large[i]) for i in range(lg_ref.size(0)))
    res = {
        "config": args.config, "n_layers": args.n_layers, "batch": args.batch, "prompt_len": args.prompt_len,
        "new_tokens": args.new_tokens, "fp8_linears": n_fp8, "bf16_linears_k_not_multiple_of_128": n_bf16_fallback,
        "logits_rel_rms_prefill": per_step[0], "logits_rel_rms_max": max(per_step),
        "greedy_token_match": match, "steps_compared": int(tok_ref.numel()),
        "decode_ms_per_step_reference_kernels": dt_ref * 1e3, "decode_ms_per_step_this_library": dt_ours * 1e3,
        "reference_noise_logits_rel_rms_max": max(noise), "reference_noise_greedy_token_match": noise_match,
        "logits_rel_rms_max_vs_reference_tile_16x32": vs_small, "logits_rel_rms_max_vs_reference_tile_64x128": vs_large,
        "seams": None if seam is None else {
            "logits_rel_rms_max_vs_reference": max(rel_rms(seam[0][i], lg_ref[i]) for i in range(lg_ref.size(0))),
            "logits_rel_rms_max_vs_this_library_without_seams": max(rel_rms(seam[0][i], lg_ours[i]) for i in range(lg_ref.size(0))),
            "greedy_token_match_vs_reference": (seam[1] == tok_ref).float().mean().item(),
            "decode_ms_per_step": seam[2] * 1e3},
        "decidable_steps": n_dec, "greedy_token_match_decidable": match_dec,
        "reference_noise_greedy_token_match_decidable": noise_match_dec,
        "graph": graph_res,
        "pass": bool(max(per_step) <= 2e-2 and match >= 0.99),
        "pass_decidable": bool(n_dec > 0 and match_dec >= 0.99 and max(per_step) <= max(2e-2, 1.25 * max(noise))),
        "within_reference_noise": bool(max(per_step) <= 1.5 * max(noise) and match >= noise_match - 0.05),
    }
    print(json.dumps(res), flush=True)
    if args.out:
        json.dump(res, open(args.out, "w"), indent=1)


if __name__ == "__main__":
    main()
