"""Grouped MoE path against the reference's expert loop (model.py:669-693).

The loop is restated here with the drop-in operators (one act_quant + fp8_gemm per Linear and expert,
``y[idx] += expert(x[idx]) * weights[idx, top, None]`` in ascending expert order); the grouped path
must agree within the fp8_gemm tolerance scaled to the layer output, and the combine kernel must
reproduce the bf16 accumulation bit for bit when given the same expert outputs."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

from oracle import oracle as O
from gpu_util import bf16_bits

pytestmark = pytest.mark.gpu


class _Lin:
    scale_fmt = None

    def __init__(self, N, K, seed):
        import dsv3_b200
        w = O.randn_bf16((N, K), seed, 0.02).cuda()
        self.weight, s = dsv3_b200.weight_quant(w)
        self.weight.scale = s

    def __call__(self, x):
        import kernel
        xq, xs = kernel.act_quant(x)
        return kernel.fp8_gemm(xq, xs, self.weight, self.weight.scale)


class _Expert:
    def __init__(self, dim, inter, seed):
        self.w1, self.w2, self.w3 = _Lin(inter, dim, seed), _Lin(dim, inter, seed + 1), _Lin(inter, dim, seed + 2)

    def __call__(self, x):
        return self.w2(F.silu(self.w1(x)) * self.w3(x))


class _MoE:
    """Attribute names of model.py's MoE (model.py:636-666)."""

    def __init__(self, dim, inter, n_routed, topk, start, end, seed):
        self.dim, self.n_routed_experts, self.n_activated_experts = dim, n_routed, topk
        self.n_local_experts = end - start
        self.experts_start_idx, self.experts_end_idx = start, end
        self.experts = [_Expert(dim, inter, seed + 10 * i) if start <= i < end else None for i in range(n_routed)]
        g = torch.Generator(device="cuda").manual_seed(seed)
        self.gate_w = (torch.randn(n_routed, dim, generator=g, device="cuda") * 0.02).bfloat16()
        self.shared = _Expert(dim, inter, seed + 5000)

    def gate(self, x):
        scores = F.linear(x, self.gate_w).softmax(dim=-1, dtype=torch.float32)
        indices = torch.topk(scores, self.n_activated_experts, dim=-1)[1]
        weights = scores.gather(1, indices)
        return weights.type_as(x), indices

    def shared_experts(self, x):
        return self.shared(x)

    def reference_forward(self, x):
        """MoE.forward, model.py:669-693, single rank."""
        shape = x.size()
        x = x.view(-1, self.dim)
        weights, indices = self.gate(x)
        y = torch.zeros_like(x)
        counts = torch.bincount(indices.flatten(), minlength=self.n_routed_experts).tolist()
        for i in range(self.experts_start_idx, self.experts_end_idx):
            if counts[i] == 0:
                continue
            idx, top = torch.where(indices == i)
            y[idx] += self.experts[i](x[idx]) * weights[idx, top, None]
        z = self.shared_experts(x)
        return (y + z).view(shape), y


@pytest.fixture(autouse=True)
def _bf16_default():
    torch.set_default_dtype(torch.bfloat16)
    yield
    torch.set_default_dtype(torch.float32)


@pytest.mark.parametrize("T,dim,inter,n_routed,topk,start,end", [
    (50, 512, 256, 8, 2, 0, 8),        # all experts local, ~12 tokens per expert
    (300, 512, 384, 8, 3, 0, 8),       # ~110 tokens per expert: several 64-token tiles per expert
    (40, 256, 128, 16, 4, 4, 12),      # half of the experts live on other ranks
    (3, 512, 256, 32, 2, 0, 32),       # decode-like: most experts get no token
])
def test_grouped_moe_matches_expert_loop(T, dim, inter, n_routed, topk, start, end):
    import dsv3_b200
    from dsv3_b200 import linear_seam as L
    moe = _MoE(dim, inter, n_routed, topk, start, end, seed=100 + T)
    x = O.randn_bf16((T, dim), 7 + T, 1.0).cuda()
    ref_out, ref_y = moe.reference_forward(x)
    L.reset_memo()
    out = dsv3_b200.grouped_moe_forward(moe, x)
    dsv3_b200.check_device_status()
    assert out.shape == ref_out.shape and out.dtype == torch.bfloat16
    err = (out.float() - ref_out.float()).abs()
    rms = ref_out.float().pow(2).mean().sqrt()
    assert bool((err <= 2e-2 * (ref_out.float().abs() + rms)).all()), float((err / (ref_out.float().abs() + rms)).max())
    # tokens without any local expert get exactly the shared-expert output
    _, indices = moe.gate(x)
    none_local = ~((indices >= start) & (indices < end)).any(dim=1)
    if none_local.any():
        assert torch.equal(out[none_local], moe.shared_experts(x)[none_local])


def test_moe_combine_is_bit_exact():
    from dsv3_b200 import _lib
    T, topk, dim, rows = 37, 4, 256, 200
    g = torch.Generator(device="cuda").manual_seed(3)
    o = torch.randn(rows, dim, generator=g, device="cuda").bfloat16()
    w = torch.rand(T, topk, generator=g, device="cuda").bfloat16()
    pos = torch.randint(-1, rows, (T, topk), generator=g, device="cuda", dtype=torch.int32)
    y = torch.empty(T, dim, dtype=torch.bfloat16, device="cuda")
    _lib.check(_lib.lib.dsv3_moe_combine(o.data_ptr(), pos.data_ptr(), w.data_ptr(), T, topk, dim, y.data_ptr(),
                                         torch.cuda.current_stream().cuda_stream))
    ref = torch.zeros(T, dim, dtype=torch.bfloat16, device="cuda")
    for j in range(topk):                                    # the arithmetic of `y[idx] += out * weights[...]`
        valid = pos[:, j] >= 0
        contrib = o[pos[:, j].clamp_min(0).long()] * w[:, j, None]
        ref = torch.where(valid[:, None], ref + contrib, ref)
    assert np.array_equal(bf16_bits(y), bf16_bits(ref))


def test_install_moe_rebinds_forward():
    import types
    import dsv3_b200

    class FakeMoE(_MoE):
        def forward(self, x):
            return "original"

    mod = types.SimpleNamespace(MoE=FakeMoE, world_size=1, gemm_impl="fp8")
    dsv3_b200.install_moe(mod)
    moe = FakeMoE(256, 128, 4, 2, 0, 4, seed=9)
    x = O.randn_bf16((6, 256), 3, 1.0).cuda()
    out = moe.forward(x)
    assert isinstance(out, torch.Tensor) and out.shape == (6, 256)
    mod.gemm_impl = "bf16"
    assert moe.forward(x) == "original"


@pytest.mark.parametrize("T,topk,E,start,n", [(64, 8, 256, 0, 256), (300, 6, 64, 16, 32), (1, 8, 256, 224, 32), (2048, 8, 256, 0, 256)])
def test_moe_route_groups_pairs_by_expert_and_orders_each_tokens_pairs(T, topk, E, start, n):
    """dsv3_moe_route against the torch operations it replaces (bincount / where / sort of model.py:680-686)."""
    from dsv3_b200 import _lib
    lib = _lib.lib
    g = torch.Generator(device="cpu").manual_seed(T * 31 + topk)
    scores = torch.rand(T, E, generator=g)
    weights, indices = scores.topk(topk, dim=-1)            # distinct experts per token, descending score
    indices, weights = indices.cuda(), weights.float().cuda()
    P = T * topk
    seg = torch.empty(n + 1, dtype=torch.int32, device="cuda")
    tok = torch.empty(P, dtype=torch.int32, device="cuda")
    pair_row = torch.empty(P, dtype=torch.int32, device="cuda")
    pos_s = torch.empty(T, topk, dtype=torch.int32, device="cuda")
    w_s = torch.empty(T, topk, dtype=torch.bfloat16, device="cuda")
    _lib.check(lib.dsv3_moe_route(indices.data_ptr(), weights.data_ptr(), T, topk, start, n, seg.data_ptr(), tok.data_ptr(),
                                  pair_row.data_ptr(), pos_s.data_ptr(), w_s.data_ptr(), torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    key = indices.reshape(-1) - start
    local = (key >= 0) & (key < n)
    counts = torch.bincount(torch.where(local, key, torch.full_like(key, n)), minlength=n + 1)
    want_seg = torch.zeros(n + 1, dtype=torch.int64, device="cuda")
    want_seg[1:] = torch.cumsum(counts[:n], 0)
    assert torch.equal(seg.long(), want_seg)
    # every pair got a distinct row; local pairs sit inside their expert's segment and carry their token
    rows = torch.where(local, pair_row.long(), torch.full_like(key, -1))
    lp = torch.nonzero(local).flatten()
    assert torch.equal(torch.sort(rows[lp]).values, torch.arange(int(want_seg[n]), device="cuda"))
    e = key[lp]
    assert bool(((rows[lp] >= want_seg[e]) & (rows[lp] < want_seg[e + 1])).all())
    assert torch.equal(tok.long()[rows[lp]], lp // topk)
    assert torch.equal(torch.sort(tok.long()).values, torch.arange(P, device="cuda") // topk)
    # per token: ascending expert order
    _, by_expert = indices.sort(dim=1)
    assert torch.equal(pos_s.long(), rows.view(T, topk).gather(1, by_expert))
    assert torch.equal(w_s, weights.gather(1, by_expert).to(torch.bfloat16))
