"""The measurement decoder: graph-captured decode equals eager decode, and one layer's
quantized projections agree with a dense torch layer built from the dequantised weights."""
import pytest
import torch

import polar_oracle as oracle

pytestmark = pytest.mark.gpu


def small_model(batch=2):
    from polarengine_vllm_b200.decoder import DecoderConfig, QuantDecoder
    cfg = DecoderConfig(hidden=512, n_heads=4, n_kv_heads=2, head_dim=128, intermediate=1024, n_layers=2, vocab=1024)
    return cfg, QuantDecoder(cfg, torch.device("cuda"), max_len=64, batch=batch)


def test_graph_decode_equals_eager():
    cfg, m = small_model()
    g = torch.Generator(device="cuda").manual_seed(0)
    prompt = torch.randint(0, cfg.vocab, (2, 20), device="cuda", generator=g)
    nxt = m.forward(prompt, 0)
    assert nxt.shape == (2,) and int(nxt.max()) < cfg.vocab
    ids, pos = nxt.view(2, 1).clone(), torch.tensor(20, device="cuda")
    eager = []
    for _ in range(4):
        out = m.forward(ids, pos)
        eager.append(out.clone()); ids.copy_(out.view(2, 1)); pos.add_(1)
    # same tokens when prefill is replayed position by position with the static-shape path
    m2cfg, m2 = small_model()
    n2 = m2.forward(prompt, 0)
    assert torch.equal(n2, nxt)
    ids2, pos2 = n2.view(2, 1).clone(), torch.tensor(20, device="cuda")
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        def step():
            out = m2.forward(ids2, pos2); ids2.copy_(out.view(2, 1)); pos2.add_(1)
        step(); torch.cuda.synchronize()
        first = ids2.clone()
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr, stream=s):
            step()
        got = [first.view(-1)]      # capture itself runs nothing; three replays give steps 2..4
        for _ in range(3):
            gr.replay(); got.append(ids2.view(-1).clone())
        torch.cuda.synchronize()
    for a, b in zip(eager, got):
        assert torch.equal(a, b)


def test_projection_matches_dense_layer():
    cfg, m = small_model(batch=1)
    L = m.layers[0]
    x = torch.randn(3, cfg.hidden, device="cuda").half()
    from polarengine_vllm_b200.packing import unpack_codes_half_block
    for name in ("qkv", "gate_up", "down", "o"):
        w = L[name]
        codes = (unpack_codes_half_block(w.codes) if w.packed else w.codes).cpu()
        dense = oracle.dequant_fp32(codes, w.norms.cpu(), w.ct.cpu())
        xin = torch.randn(3, w.in_f, device="cuda").half()
        ref = xin.float().cpu() @ dense.T
        y = w(xin, torch.float32).cpu()
        assert float((y - ref).abs().max() / ref.abs().max()) <= 1e-2


def test_folded_glue_ops_give_the_same_tokens():
    """One-token decode with the norm / activation folded into the projections' launches against the same model
    with every glue op as its own launch: same logits within fp16 rounding, same next tokens."""
    from polarengine_vllm_b200.decoder import DecoderConfig, QuantDecoder
    cfg = DecoderConfig(hidden=1024, n_heads=8, n_kv_heads=2, head_dim=128, intermediate=2048, n_layers=3, vocab=4096)
    dev = torch.device("cuda")
    a = QuantDecoder(cfg, dev, max_len=64, batch=1)
    b = QuantDecoder(cfg, dev, max_len=64, batch=1)
    b.fuse_glue = False
    g = torch.Generator(device="cuda").manual_seed(3)
    prompt = torch.randint(0, cfg.vocab, (1, 12), device=dev, generator=g)
    ia, ib = a.forward(prompt, 0), b.forward(prompt, 0)
    assert torch.equal(ia, ib)
    ids = ia.view(1, 1)
    for s in range(4):
        pos = torch.tensor(12 + s, device=dev)
        la, lb = a.forward(ids, pos, return_logits=True), b.forward(ids, pos, return_logits=True)
        assert float((la - lb).abs().max() / lb.abs().max()) <= 5e-3
        assert torch.equal(la.argmax(-1), lb.argmax(-1))
        ids = lb.argmax(-1).view(1, 1)
