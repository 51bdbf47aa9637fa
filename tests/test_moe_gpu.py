"""Quantized MoE expert path against the oracle composition (softmax/top-k/renormalise,
silu(gate)*up, down, weighted sum; expert projections are quantized linears).  The
reference has no quantized MoE arithmetic, so this composition is pinned only through
its pieces."""
import pytest
import torch

import polar_oracle as oracle
from helpers import max_rel

pytestmark = pytest.mark.gpu


def build(e, h, i, seed=0):
    from polarengine_vllm_b200.moe_method import PolarQuantMoEMethod
    g = torch.Generator().manual_seed(seed)
    method = PolarQuantMoEMethod(3, 4)
    layer = torch.nn.Module()
    method.create_weights(layer, e, h, i, torch.float16)
    layer = layer.cuda()
    experts = []
    for ex in range(e):
        q = {}
        for name, shape, bits in (("gate", (i, h), 3), ("up", (i, h), 3), ("down", (h, i), 4)):
            q[name] = oracle.quantize_tensor(torch.randn(*shape, generator=g) * 0.02, bits)
        method.load_expert(layer, ex, q["gate"], q["up"], q["down"])
        experts.append({n: (q[n]["codes"], q[n]["norms"], q[n]["ct_scaled"], None) for n in q})
    method.process_weights_after_loading(layer)
    return method, layer, experts


@pytest.mark.parametrize("tokens", [1, 5, 64, 200])
def test_moe_matches_oracle(tokens):
    e, h, i, top_k = 16, 384, 200, 4   # ragged intermediate: down-projection K pads 200 -> 256
    method, layer, experts = build(e, h, i)
    g = torch.Generator().manual_seed(tokens)
    x = torch.randn(tokens, h, generator=g).half()
    gate_w = (torch.randn(e, h, generator=g) * 0.02).half()
    w, ids = oracle.moe_route(x, gate_w, top_k)
    ref = oracle.moe_forward(x, w, ids, experts)
    y = method.apply(layer, x.cuda(), w.cuda(), ids.cuda())
    assert y.shape == (tokens, h) and y.dtype == torch.float16
    assert max_rel(y, ref) <= 1e-2
    # the per-expert path (tensor-core kernel for experts with more than 16 rows) agrees
    y_loop = method._moe_forward_per_expert(layer, x.cuda(), w.cuda(), ids.cuda())
    assert max_rel(y_loop, ref) <= 1e-2
    # older contract: router logits in, routing done inside
    logits = (x.float() @ gate_w.float().T).cuda()
    y2 = method.apply(layer, x.cuda(), logits, top_k, True)
    assert max_rel(y2, ref) <= 1e-2


def test_moe_expert_parallel_partition_sums_to_full():
    e, h, i, top_k = 8, 256, 128, 2
    method, layer, experts = build(e, h, i, seed=3)
    g = torch.Generator().manual_seed(1)
    x = torch.randn(9, h, generator=g).half().cuda()
    w, ids = oracle.moe_route(x.cpu(), (torch.randn(e, h, generator=g) * 0.02).half(), top_k)
    full = method.moe_forward(layer, x, w.cuda(), ids.cuda()).float()
    parts = torch.zeros_like(full)
    for rank in range(2):
        emap = torch.full((e,), -1, dtype=torch.long)
        emap[rank * 4:(rank + 1) * 4] = torch.arange(4)
        sub = torch.nn.Module()
        for name in ("w13_codes", "w13_norms", "w2_codes", "w2_norms"):
            setattr(sub, name, getattr(layer, name)[rank * 4:(rank + 1) * 4])
        for name in ("w13_ct_scaled", "w2_ct_scaled", "moe_hidden", "moe_inter", "moe_hidden_padded", "moe_inter_padded"):
            setattr(sub, name, getattr(layer, name))
        parts += method.moe_forward(sub, x, w.cuda(), ids.cuda(), expert_map=emap.cuda()).float()
    assert max_rel(parts, full) <= 2e-3


def build_random_codes(e, h, i, seed=0):
    """Experts with uniformly random codes and |randn| norms (helpers.rand_layer): no quantizer run, so the
    128-expert layer of the benchmark configuration builds in seconds."""
    from helpers import rand_layer
    from polarengine_vllm_b200.moe_method import PolarQuantMoEMethod
    method = PolarQuantMoEMethod(3, 4)
    layer = torch.nn.Module()
    method.create_weights(layer, e, h, i, torch.float16)
    layer = layer.cuda()
    hp, ip = -(-h // 128) * 128, -(-i // 128) * 128
    experts = []
    for ex in range(e):
        q = {}
        for name, (n, kp, k), bits in (("gate", (i, hp, h), 3), ("up", (i, hp, h), 3), ("down", (h, ip, i), 4)):
            codes, norms, cts = rand_layer(n, kp, bits, seed=seed + 3 * ex + len(q))
            q[name] = {"codes": codes, "norms": norms, "ct_scaled": cts}
        method.load_expert(layer, ex, q["gate"], q["up"], q["down"])
        experts.append({n: (q[n]["codes"], q[n]["norms"], q[n]["ct_scaled"], None) for n in q})
    method.process_weights_after_loading(layer)
    return method, layer, experts


@pytest.mark.parametrize("tokens", [1, 64, 2048])
def test_moe_benchmark_configuration(tokens):
    """128 experts, top-8, hidden 2688, intermediate 1856 (down-projection K pads to 1920): the shapes of the
    expert-layer benchmark.  64 tokens run the decode-size grouped launches (pe_gemv_grouped), 2048 the
    grouped tensor-core launches (pe_gemm_grouped, about 2000 device-built tiles).  The GPU computes every
    token; the CPU oracle (routing, silu(gate)*up, down, weighted sum: nemotron_offload.py:180-226) is
    evaluated on a sample of them."""
    e, h, i, top_k = 128, 2688, 1856, 8
    method, layer, experts = build_random_codes(e, h, i, seed=500)
    g = torch.Generator().manual_seed(tokens)
    x = torch.randn(tokens, h, generator=g).half()
    gate_w = (torch.randn(e, h, generator=g) * 0.02).half()
    w, ids = oracle.moe_route(x, gate_w, top_k)
    y = method.apply(layer, x.cuda(), w.cuda(), ids.cuda())
    assert y.shape == (tokens, h) and y.dtype == torch.float16 and torch.isfinite(y.float()).all()
    sample = torch.arange(tokens) if tokens <= 64 else torch.randperm(tokens, generator=g)[:24].sort().values
    ref = oracle.moe_forward(x[sample], w[sample], ids[sample], experts)
    assert max_rel(y[sample.cuda()], ref) <= 1e-2


@pytest.mark.parametrize("t,e,k", [(1, 128, 8), (64, 128, 8), (300, 60, 4), (7, 1000, 32)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
def test_routing_kernel_matches_softmax_topk(t, e, k, dtype):
    """pe_moe_route = softmax (fp32) -> top-k -> renormalise of nemotron_offload.py:180-189: the same weights as
    torch.topk on the same logits to fp32 rounding (and the same experts in the same order where no two logits are
    equal); with and without renormalisation."""
    from polarengine_vllm_b200.moe_method import route_softmax_topk
    g = torch.Generator().manual_seed(t + e)
    logits = (torch.randn(t, e, generator=g) * 3).to(dtype)
    for renorm in (True, False):
        w, ids = route_softmax_topk(logits.cuda(), k, renorm)
        p = torch.softmax(logits.float(), dim=-1)
        rw, rids = p.topk(k, dim=-1)
        if renorm:
            rw = rw / rw.sum(-1, keepdim=True)
        assert ids.dtype == torch.int64 and w.dtype == torch.float32
        w, ids = w.cpu(), ids.cpu()
        # the k largest probabilities in descending order (equal logits -- common in 16-bit -- may swap places or, at
        # the k-th place, experts: either choice is a valid top-k), each weight being its own expert's probability
        assert torch.allclose(w, rw, rtol=1e-5, atol=1e-7)
        own = p.gather(1, ids)
        if renorm:
            own = own / own.sum(-1, keepdim=True)
        assert torch.allclose(w, own, rtol=1e-5, atol=1e-7)
        assert all(len(set(r.tolist())) == k for r in ids)
        if dtype == torch.float32:
            assert torch.equal(ids, rids)
