"""The decoder-layer glue ops (residual add + RMSNorm, rotary + KV-cache write, SiLU * up)
against their op-by-op torch formulations (decoder.rms_norm / decoder.rope / F.silu)."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("rows,hidden", [(1, 4096), (5, 4096), (3, 512), (2, 12288), (7, 16384), (4, 2688)])
@pytest.mark.parametrize("delta_kind", ["none", "f16", "f32"])
def test_add_rmsnorm(rows, hidden, delta_kind):
    from polarengine_vllm_b200.decode_ops import add_rmsnorm
    from polarengine_vllm_b200.decoder import rms_norm
    g = torch.Generator(device="cuda").manual_seed(rows + hidden)
    x = torch.randn(rows, hidden, device="cuda", generator=g).half()
    w = (1 + 0.1 * torch.randn(hidden, device="cuda", generator=g)).half()
    delta = None
    if delta_kind != "none":
        delta = 0.5 * torch.randn(rows, hidden, device="cuda", generator=g)
        delta = delta.half() if delta_kind == "f16" else delta
    x_ref = x.clone() if delta is None else x + delta.half()
    ref = rms_norm(x_ref, w, 1e-6)
    xs = x.clone()
    out = add_rmsnorm(xs, delta, w, 1e-6)
    assert torch.equal(xs, x_ref)  # the residual stream is updated bit-exactly
    assert out.dtype == torch.float16 and out.shape == x.shape
    # the sum of squares is reduced in another order: results may differ by one fp16 rounding
    assert torch.allclose(out.float(), ref.float(), rtol=2e-3, atol=1e-3)
    assert (out != ref).float().mean() < 0.02


@pytest.mark.parametrize("batch,t,pos0,on_device", [(1, 1, 37, True), (2, 1, 5, True), (2, 20, 0, False), (1, 33, 7, False)])
def test_rope_cache(batch, t, pos0, on_device):
    from polarengine_vllm_b200.decode_ops import rope_cache
    from polarengine_vllm_b200.decoder import rope
    hq, hkv, d, max_len, theta = 4, 2, 128, 64, 1e6
    g = torch.Generator(device="cuda").manual_seed(t + pos0)
    qkv = torch.randn(batch * t, (hq + 2 * hkv) * d, device="cuda", generator=g).half()
    kc = torch.zeros(batch, hkv, max_len, d, dtype=torch.float16, device="cuda")
    vc = torch.zeros_like(kc)
    p = torch.tensor(pos0, device="cuda") if on_device else pos0
    q = rope_cache(qkv, p, kc, vc, batch, t, hq, hkv, d, theta)
    v4 = qkv.view(batch, t, hq + 2 * hkv, d)
    pos = torch.arange(pos0, pos0 + t, device="cuda")
    q_ref = rope(v4[:, :, :hq].transpose(1, 2), pos, theta)
    k_ref = rope(v4[:, :, hq:hq + hkv].transpose(1, 2), pos, theta)
    v_ref = v4[:, :, hq + hkv:].transpose(1, 2)
    assert q.shape == (batch, hq, t, d)
    assert torch.allclose(q.float(), q_ref.float(), rtol=2e-3, atol=2e-3)
    assert torch.allclose(kc[:, :, pos0:pos0 + t].float(), k_ref.float(), rtol=2e-3, atol=2e-3)
    assert torch.equal(vc[:, :, pos0:pos0 + t], v_ref)
    # nothing outside the written positions is touched
    assert float(kc[:, :, :pos0].abs().max() if pos0 else 0) == 0 and float(kc[:, :, pos0 + t:].abs().max()) == 0


@pytest.mark.parametrize("rows,inter", [(1, 12288), (3, 1024), (64, 1856)])
def test_silu_mul(rows, inter):
    from polarengine_vllm_b200.decode_ops import silu_mul
    g = torch.Generator(device="cuda").manual_seed(rows)
    gu = (2 * torch.randn(rows, 2 * inter, device="cuda", generator=g)).half()
    ref = F.silu(gu[:, :inter]) * gu[:, inter:]
    out = silu_mul(gu, inter)
    assert torch.allclose(out.float(), ref.float(), rtol=2e-3, atol=1e-4)
    assert (out != ref).float().mean() < 0.02


@pytest.mark.parametrize("batch,hq,hkv,pos,on_device", [(1, 32, 8, 512, True), (2, 4, 2, 20, True), (3, 8, 8, 0, False),
                                                        (1, 16, 2, 639, False), (8, 32, 8, 100, True)])
def test_decode_attention(batch, hq, hkv, pos, on_device):
    """One-token attention over the cache against torch's SDPA on the first pos + 1 positions."""
    from polarengine_vllm_b200.decode_ops import decode_attention
    d, max_len = 128, 640
    g = torch.Generator(device="cuda").manual_seed(pos + hq)
    q = torch.randn(batch, hq, 1, d, device="cuda", generator=g).half()
    kc = torch.randn(batch, hkv, max_len, d, device="cuda", generator=g).half()
    vc = torch.randn(batch, hkv, max_len, d, device="cuda", generator=g).half()
    p = torch.tensor(pos, device="cuda") if on_device else pos
    out = decode_attention(q, kc, vc, p)
    rep = hq // hkv
    k = kc[:, :, : pos + 1].float().repeat_interleave(rep, dim=1)
    v = vc[:, :, : pos + 1].float().repeat_interleave(rep, dim=1)
    ref = F.scaled_dot_product_attention(q.float(), k, v).transpose(1, 2).reshape(batch, hq * d)
    assert out.shape == (batch, hq * d) and out.dtype == torch.float16
    assert torch.allclose(out.float(), ref, rtol=2e-3, atol=2e-3)


@pytest.mark.parametrize("rows,hidden", [(1, 4096), (4, 4096), (3, 512)])
def test_exchange_with_one_rank_equals_add_rmsnorm(rows, hidden):
    """World size 1: the fused all-reduce + add + norm kernel pushes to, waits for and reads
    its own buffer, so the whole protocol (slots, flags, sequence numbers, both parities)
    runs inside one launch on one GPU and must give the bits of add_rmsnorm."""
    from polarengine_vllm_b200.decode_ops import add_rmsnorm
    from polarengine_vllm_b200.parallel import PeerExchange
    g = torch.Generator(device="cuda").manual_seed(rows)
    xchg = PeerExchange(torch.device("cuda"), 0, 1, 4, hidden)
    w = (1 + 0.1 * torch.randn(hidden, device="cuda", generator=g)).half()
    x = torch.randn(rows, hidden, device="cuda", generator=g).half()
    x_ref = x.clone()
    for _ in range(5):  # consecutive calls alternate the slot parity
        part = torch.randn(rows, hidden, device="cuda", generator=g)
        out = xchg.allreduce_add_rmsnorm(part, x, w, 1e-6)
        ref = add_rmsnorm(x_ref, part, w, 1e-6)
        assert torch.equal(x, x_ref) and torch.equal(out, ref)
    assert not xchg.timed_out()
    assert int(xchg.seq[0]) == 5


def test_exchange_wait_runs_out_and_reports():
    """A peer that never arrives costs a bounded time and a status word, not a hung GPU: a world of two whose
    peer table points at two LOCAL buffers, with only rank 0 ever launched.  Rank 0 pushes its partial into
    both buffers, waits for rank 1's flag (nothing sets it), gives up after the limit (10 ms here), records
    status 1 and finishes with what it has (its own partial; rank 1's slot reads zero).  The next call on a
    healthy exchange works."""
    from polarengine_vllm_b200 import _native as nv
    from polarengine_vllm_b200.decode_ops import add_rmsnorm
    from polarengine_vllm_b200.parallel import PeerExchange
    dev = torch.device("cuda")
    lib = nv.lib()
    rows, hidden, max_rows = 2, 4096, 4
    g = torch.Generator(device="cuda").manual_seed(3)
    nbytes = lib.pe_allreduce_buffer_bytes(2, max_rows, hidden)
    bufs = [torch.zeros(nbytes, dtype=torch.uint8, device=dev) for _ in range(2)]
    peers = torch.tensor([b.data_ptr() for b in bufs], dtype=torch.int64, device=dev)
    seq = torch.zeros(max_rows, dtype=torch.int32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    w = (1 + 0.1 * torch.randn(hidden, device=dev, generator=g)).half()
    x = torch.randn(rows, hidden, device=dev, generator=g).half()
    x_ref = x.clone()
    part = torch.randn(rows, hidden, device=dev, generator=g)
    out = torch.empty_like(x)
    assert lib.pe_set_wait_limit_us(10_000) == 0
    try:
        torch.cuda.synchronize()
        import time
        t0 = time.perf_counter()
        nv.check(lib.pe_allreduce_add_rmsnorm(part.data_ptr(), x.data_ptr(), w.data_ptr(), out.data_ptr(), rows, hidden, 1e-6,
                                              peers.data_ptr(), 0, 2, max_rows, seq.data_ptr(), status.data_ptr(),
                                              nv.stream_ptr(dev)), "pe_allreduce_add_rmsnorm")
        torch.cuda.synchronize()
        assert time.perf_counter() - t0 < 1.0           # the limit, not the default second
    finally:
        assert lib.pe_set_wait_limit_us(1_000_000) == 0
    assert int(status.item()) == 1                      # the wait ran out and said so
    ref = add_rmsnorm(x_ref, part, w, 1e-6)             # rank 1 contributed zeros
    assert torch.equal(x, x_ref) and torch.equal(out, ref)
    # the context is intact: a healthy exchange runs right after
    xchg = PeerExchange(dev, 0, 1, 4, hidden)
    out2 = xchg.allreduce_add_rmsnorm(part, x, w, 1e-6)
    assert torch.equal(out2, add_rmsnorm(x_ref, part, w, 1e-6)) and not xchg.timed_out()
    assert lib.pe_set_wait_limit_us(0) == -1


@pytest.mark.parametrize("bits,n,k", [(5, 6144, 4096), (3, 24576, 4096), (6, 151936 // 8, 4096), (4, 4096, 1024)])
def test_projection_with_folded_add_rmsnorm(bits, n, k):
    """pe_gemv_pro(PE_PRO_ADD_RMSNORM) = pe_add_rmsnorm followed by pe_gemv: same updated residual (bit for bit)
    and the same projection within the fp16 rounding of the norm scale (the two kernels sum the squares in
    different orders)."""
    from helpers import rand_layer
    from polarengine_vllm_b200 import _native as nv, kernels, packing
    from polarengine_vllm_b200.decode_ops import add_rmsnorm
    dev = torch.device("cuda")
    codes, norms, cts = rand_layer(n, k, bits, seed=bits + n)
    packed = bits <= 4
    w = packing.pack_codes_half_block(codes.to(dev)) if packed else codes.to(dev)
    nd, ctd = norms.to(dev), cts.to(dev)
    g = torch.Generator(device="cuda").manual_seed(1)
    x = torch.randn(1, k, device=dev, generator=g).half()
    lnw = (1 + 0.1 * torch.randn(k, device=dev, generator=g)).half()
    for delta in (None, torch.randn(1, k, device=dev, generator=g), torch.randn(1, k, device=dev, generator=g).half()):
        x_ref = x.clone()
        h = add_rmsnorm(x_ref, delta, lnw, 1e-6)
        y_ref = kernels.quant_matmul(w, packed, nd, ctd, h, False, n, k, k, torch.float32)
        resid = torch.full_like(x, float("nan"))
        y = kernels.quant_matmul_pro(w, packed, nd, ctd, nv.PE_PRO_ADD_RMSNORM, x, k, n, k, torch.float32, delta=delta,
                                     norm_weight=lnw, eps=1e-6, resid_out=resid if delta is not None else None)
        assert y is not None and y.shape == (1, n)
        if delta is not None:
            assert torch.equal(resid, x_ref)
        assert float((y - y_ref).abs().max() / y_ref.abs().max()) <= 2e-3


@pytest.mark.parametrize("bits,n,inter", [(4, 4096, 12288), (4, 4096, 1536), (3, 2048, 4096)])
def test_projection_with_folded_silu_mul(bits, n, inter):
    """pe_gemv_pro(PE_PRO_SILU_MUL) = pe_silu_mul followed by pe_gemv (same rounding steps: bit-identical)."""
    from helpers import rand_layer
    from polarengine_vllm_b200 import _native as nv, kernels, packing
    from polarengine_vllm_b200.decode_ops import silu_mul
    dev = torch.device("cuda")
    codes, norms, cts = rand_layer(n, inter, bits, seed=inter)
    w = packing.pack_codes_half_block(codes.to(dev))
    nd, ctd = norms.to(dev), cts.to(dev)
    g = torch.Generator(device="cuda").manual_seed(2)
    gu = torch.randn(1, 2 * inter, device=dev, generator=g).half()
    y_ref = kernels.quant_matmul(w, True, nd, ctd, silu_mul(gu, inter), False, n, inter, inter, torch.float32)
    y = kernels.quant_matmul_pro(w, True, nd, ctd, nv.PE_PRO_SILU_MUL, gu, inter, n, inter, torch.float32)
    assert y is not None
    assert torch.equal(y, y_ref)


def test_folded_prologue_declines_shapes_of_other_kernels():
    from helpers import rand_layer
    from polarengine_vllm_b200 import _native as nv, kernels
    codes, norms, cts = rand_layer(48, 256, 5, seed=1)
    x = torch.randn(1, 256, device="cuda").half()
    y = kernels.quant_matmul_pro(codes.cuda(), False, norms.cuda(), cts.cuda(), nv.PE_PRO_ADD_RMSNORM, x, 256, 48, 256,
                                 norm_weight=torch.ones(256, device="cuda").half(), eps=1e-6)
    assert y is None


@pytest.mark.parametrize("batch,hq,hkv,pos,on_device", [(1, 32, 8, 512, True), (2, 4, 2, 20, True), (3, 8, 8, 0, False),
                                                        (1, 4, 1, 639, True), (8, 32, 8, 100, False)])
def test_rope_attention_equals_the_two_launches(batch, hq, hkv, pos, on_device):
    """pe_rope_attention = pe_rope_cache (one token) followed by pe_decode_attention: same cache rows, and the
    same attention output bit for bit where both run the warp-per-position kernel (with many sequences the
    two-launch form takes the thread-per-position kernel: equal within fp16 rounding)."""
    from polarengine_vllm_b200.decode_ops import decode_attention, rope_attention, rope_cache
    d, max_len, theta = 128, 640, 1e6
    g = torch.Generator(device="cuda").manual_seed(pos + hq + batch)
    qkv = torch.randn(batch, (hq + 2 * hkv) * d, device="cuda", generator=g).half()
    kc = torch.randn(batch, hkv, max_len, d, device="cuda", generator=g).half()
    vc = torch.randn(batch, hkv, max_len, d, device="cuda", generator=g).half()
    kc2, vc2 = kc.clone(), vc.clone()
    p = torch.tensor(pos, device="cuda") if on_device else pos
    q = rope_cache(qkv, p, kc, vc, batch, 1, hq, hkv, d, theta)
    ref = decode_attention(q, kc, vc, p)
    out = rope_attention(qkv, p, kc2, vc2, hq, hkv, d, theta)
    assert torch.equal(kc2, kc) and torch.equal(vc2, vc)
    if batch * hkv * 4 < torch.cuda.get_device_properties(0).multi_processor_count:
        assert torch.equal(out, ref)
    else:
        assert torch.allclose(out.float(), ref.float(), rtol=2e-3, atol=2e-3)
