"""Checkpoint reader: the on-disk PolarEngine layouts (split codes / norms / centroids,
legacy unscaled centroids, LSB-first packed Q5, nibble-packed codes, the HLWQ 5-bit stream)
come back as the tensors the kernels read, whole or as tensor-parallel shards.  Synthetic
checkpoints are written with the package's own packers, whose bit layouts are pinned by the
golden vectors (test_host_cpu.py)."""
import json
import math

import pytest
import torch
from safetensors.torch import save_file

import polar_oracle as oracle
from polarengine_vllm_b200 import loader, packing
from polarengine_vllm_b200.linear_method import PolarQuantLinearMethod
from polarengine_vllm_b200.utils import get_centroids


def quantized(n, k, bits, seed):
    g = torch.Generator().manual_seed(seed)
    return oracle.quantize_tensor(torch.randn(n, k, generator=g) * 0.02, bits)


@pytest.fixture()
def v5_dir(tmp_path):
    """Two shards, four layers: int8 Q6, nibble-packed Q4, LSB-first packed Q5 with legacy .ct, and a dense layer."""
    q6, q4, q5 = quantized(32, 512, 6, 1), quantized(48, 300, 4, 2), quantized(16, 256, 5, 3)
    a = {"m.o_proj.codes": q6["codes"], "m.o_proj.norms": q6["norms"], "m.o_proj.ct_scaled": q6["ct_scaled"],
         "m.o_proj.bias": torch.arange(32).half(),
         "m.down_proj.codes": packing.pack_codes_half_block(q4["codes"]), "m.down_proj.norms": q4["norms"],
         "m.down_proj.ct_scaled": q4["ct_scaled"]}
    b = {"m.q_proj.codes": packing.pack_codes_q5(q5["codes"]), "m.q_proj.norms": q5["norms"],
         "m.q_proj.ct": q5["ct_scaled"] * math.sqrt(128), "m.norm.weight": torch.ones(64).half()}
    save_file(a, str(tmp_path / "model-00001-of-00002.safetensors"))
    save_file(b, str(tmp_path / "model-00002-of-00002.safetensors"))
    wm = {k: "model-00001-of-00002.safetensors" for k in a}
    wm.update({k: "model-00002-of-00002.safetensors" for k in b})
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": wm}))
    cfg = {"format": "polar_engine_v5", "block_size": 128,
           "layers": {"m.o_proj": {"bits": 6}, "m.down_proj": {"bits": 4, "in_features": 300},
                      "m.q_proj": {"bits": 5, "packed_q5": True}}}
    (tmp_path / "polar_config.json").write_text(json.dumps(cfg))
    return tmp_path, {"o": q6, "down": q4, "q": q5}


def test_split_tensor_formats(v5_dir):
    d, q = v5_dir
    with loader.PolarCheckpoint(str(d)) as ck:
        assert ck.layer_names() == ["m.down_proj", "m.o_proj", "m.q_proj"]
        assert ck.is_quantized_layer("m.o_proj") and not ck.is_quantized_layer("m.norm")
        assert [ck.layer_bits(n) for n in ck.layer_names()] == [4, 6, 5]
        o = ck.load_layer("m.o_proj")
        assert o["codes"].dtype == torch.int8 and torch.equal(o["codes"], q["o"]["codes"]) and not o["packed"]
        assert torch.equal(o["norms"], q["o"]["norms"]) and torch.equal(o["ct_scaled"], q["o"]["ct_scaled"])
        assert torch.equal(o["bias"], torch.arange(32).half())
        dn = ck.load_layer("m.down_proj")   # nibbles stay as stored; K is padded 300 -> 384
        assert dn["packed"] and dn["codes"].dtype == torch.uint8 and dn["codes"].shape == (48, 192) and dn["in_f"] == 300
        assert torch.equal(packing.unpack_codes_half_block(dn["codes"]), q["down"]["codes"])
        qq = ck.load_layer("m.q_proj")      # packed Q5 is unpacked, legacy .ct is scaled
        assert torch.equal(qq["codes"], q["q"]["codes"])
        assert torch.allclose(qq["ct_scaled"], q["q"]["ct_scaled"], rtol=1e-6, atol=0)
        assert torch.equal(ck.load_layer("m.norm")["weight"], torch.ones(64).half())
        with pytest.raises(KeyError):
            ck.load_tensor("m.missing.codes")


def test_tensor_parallel_shards(v5_dir):
    d, q = v5_dir
    with loader.PolarCheckpoint(str(d)) as ck:
        cols = [ck.load_layer("m.o_proj", r, 2, "column") for r in range(2)]
        assert torch.equal(torch.cat([c["codes"] for c in cols]), q["o"]["codes"])
        assert torch.equal(torch.cat([c["bias"] for c in cols]), torch.arange(32).half())
        rows = [ck.load_layer("m.o_proj", r, 4, "row") for r in range(4)]
        assert torch.equal(torch.cat([c["codes"] for c in rows], 1), q["o"]["codes"])
        assert torch.equal(torch.cat([c["norms"] for c in rows], 1), q["o"]["norms"])
        assert "bias" in rows[0] and all("bias" not in c for c in rows[1:])
        # nibble codes are cut on whole blocks (64 bytes); the true width is split with them
        dn = [ck.load_layer("m.down_proj", r, 3, "row") for r in range(3)]
        assert torch.equal(torch.cat([c["codes"] for c in dn], 1), packing.pack_codes_half_block(q["down"]["codes"]))
        assert [c["in_f"] for c in dn] == [128, 128, 44]
        with pytest.raises(ValueError):
            ck.load_layer("m.q_proj", 0, 4, "row")   # 2 blocks over 4 ranks
        # the shards reproduce the layer: partial products of the K slices add up (oracle arithmetic)
        x = torch.randn(3, 512, generator=torch.Generator().manual_seed(9)).half()
        full = oracle.linear_dequant(x, q["o"]["codes"], q["o"]["norms"], q["o"]["ct_scaled"])
        part = sum(oracle.linear_dequant(x[:, 128 * r:128 * (r + 1)], c["codes"], c["norms"], c["ct_scaled"]) for r, c in enumerate(rows))
        assert float((part - full).abs().max() / full.abs().max()) < 1e-5


def test_hlwq_stream_format(tmp_path):
    q5 = quantized(24, 200, 5, 4)   # K padded to 256
    codes = q5["codes"]
    save_file({"l.weight__packed": packing.pack_codes_q5_hlwq(codes.flatten()), "l.weight__norms": q5["norms"].flatten(),
               "l.weight__meta": torch.tensor([24, 2, 128, codes.numel(), 200], dtype=torch.int64)}, str(tmp_path / "model.safetensors"))
    (tmp_path / "polar_config.json").write_text(json.dumps({"format": "hlwq-q5", "block_size": 128}))
    with loader.PolarCheckpoint(str(tmp_path)) as ck:   # no index file: keys are listed from the shard
        assert ck.layer_names() == ["l"] and ck.layer_bits("l") == 5
        t = ck.load_layer("l")
        assert torch.equal(t["codes"], codes) and torch.equal(t["norms"], q5["norms"]) and t["in_f"] == 200
        assert torch.equal(t["ct_scaled"], (get_centroids(5) / math.sqrt(128)).float())
    (tmp_path / "polar_config.json").write_text(json.dumps({"format": "hlwq-q4"}))
    with loader.PolarCheckpoint(str(tmp_path)) as ck, pytest.raises(ValueError):
        ck.load_layer("l")


def test_fill_linear_then_forward_matches_oracle(v5_dir):
    d, q = v5_dir
    with loader.PolarCheckpoint(str(d)) as ck:
        for name, key, bits, in_f in (("m.o_proj", "o", 6, 512), ("m.down_proj", "down", 4, 300)):
            method = PolarQuantLinearMethod(128, bits)
            layer = torch.nn.Module()
            method.create_weights(layer, in_f, [q[key]["codes"].shape[0]], in_f, q[key]["codes"].shape[0], torch.float16)
            loader.fill_linear(layer, ck.load_layer(name))
            assert torch.equal(layer.codes.data, q[key]["codes"]) and torch.equal(layer.norms.data, q[key]["norms"])
            assert torch.equal(layer.ct_scaled, q[key]["ct_scaled"])
        layer = torch.nn.Module()
        PolarQuantLinearMethod(128, 6).create_weights(layer, 512, [16], 512, 16, torch.float16)
        with pytest.raises(ValueError):
            loader.fill_linear(layer, ck.load_layer("m.o_proj"))   # 32 rows into a 16-row layer


def test_golden_checkpoints_match_the_reference_loader():
    """tests/golden/ckpt_v5 and ckpt_hlwq were written with the reference's quantizer and
    packers, and checkpoint_expected.npz holds what the reference's PolarWeightLoader returned
    for them (make_golden_checkpoint.py): this reader returns the same tensors."""
    import os
    import numpy as np
    here = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
    exp = np.load(os.path.join(here, "checkpoint_expected.npz"))
    with loader.PolarCheckpoint(os.path.join(here, "ckpt_v5")) as ck:
        assert ck.layer_names() == list(exp["v5/layer_names"])
        for layer in ("m.o_proj", "m.down_proj", "m.q_proj", "m.norm"):
            got = ck.load_layer(layer)
            keys = [k.split("/")[-1] for k in exp.files if k.startswith(f"v5/{layer}/")]
            assert keys
            for key in keys:
                want = torch.from_numpy(exp[f"v5/{layer}/{key}"])
                assert torch.equal(got[key].to(want.dtype), want), (layer, key)
        assert ck.load_layer("m.down_proj")["packed"] and ck.load_layer("m.down_proj")["in_f"] == 200
    with loader.PolarCheckpoint(os.path.join(here, "ckpt_hlwq")) as ck:
        got = ck.load_layer("l")
        assert torch.equal(got["codes"], torch.from_numpy(exp["hlwq/l/codes"]))
        assert torch.equal(got["norms"].float().flatten(), torch.from_numpy(exp["hlwq/l/norms"]).flatten())
        assert torch.equal(got["ct_scaled"], torch.from_numpy(exp["hlwq/l/ct_scaled"]))
        assert got["in_f"] == int(exp["hlwq/l/_hlwq_in_f"][0])


def test_quantize_save_load_round_trip(tmp_path):
    """quantize_state_dict -> save_checkpoint -> PolarCheckpoint gives back the quantizer's codes,
    norms and tables for every layer, across shard boundaries and for every packing."""
    from polarengine_vllm_b200.quantizer import PolarQuantizer, save_checkpoint
    g = torch.Generator().manual_seed(11)
    state = {"model.layers.0.self_attn.q_proj.weight": torch.randn(32, 256, generator=g) * 0.02,      # Q5 -> packed_q5
             "model.layers.0.self_attn.o_proj.weight": torch.randn(32, 256, generator=g) * 0.02,      # Q6 -> int8
             "model.layers.0.mlp.gate_up_proj.weight": torch.randn(64, 200, generator=g) * 0.02,      # Q3 -> nibbles, padded K
             "model.layers.0.mlp.down_proj.weight": torch.randn(32, 384, generator=g) * 0.02,         # Q4 -> nibbles
             "model.layers.0.input_layernorm.weight": torch.ones(256), "model.layers.0.mlp.down_proj.bias": torch.zeros(32)}
    qz = PolarQuantizer()
    tensors, cfg = qz.quantize_state_dict(state)
    wm = save_checkpoint(tensors, cfg, str(tmp_path), max_shard_bytes=16 * 1024)
    assert len(set(wm.values())) > 1 and cfg["format"] == "polar_engine_v5"
    with loader.PolarCheckpoint(str(tmp_path)) as ck:
        assert ck.layer_names() == sorted(k[:-7] for k in state if k.endswith("proj.weight"))
        for name, w in state.items():
            if not name.endswith("proj.weight"):
                continue
            prefix = name[:-7]
            bits = cfg["layers"][prefix]["bits"]
            q = qz.quantize_tensor(w, bits)
            t = ck.load_layer(prefix)
            codes = packing.unpack_codes_half_block(t["codes"]) if t["packed"] else t["codes"]
            assert t["packed"] == (bits <= 4) and torch.equal(codes, q["codes"]), prefix
            assert torch.equal(t["norms"], q["norms"]) and torch.equal(t["ct_scaled"], q["ct_scaled"])
            assert t["in_f"] == w.shape[1] and ck.layer_bits(prefix) == bits
        assert torch.equal(ck.load_layer("model.layers.0.input_layernorm")["weight"], torch.ones(256).half())
        assert "bias" in ck.load_layer("model.layers.0.mlp.down_proj")


def _vllm_like_layer_loader(sections, tp_rank, tp_size, row_parallel=False):
    """What vLLM's linear layers hand to ``create_weights`` as ``weight_loader`` (linear.py: MergedColumnParallel /
    QKVParallel / RowParallel ``weight_loader``): narrow the loaded tensor to this rank's slice along the
    parameter's ``output_dim`` (or ``input_dim`` for row-parallel layers) and copy it into the section that
    ``loaded_shard_id`` names."""
    def loader(param, loaded_weight, loaded_shard_id=None):
        data = param.data
        if row_parallel:
            dim = param.input_dim
            size = data.shape[dim]
            data.copy_(loaded_weight.narrow(dim, tp_rank * size, size))
            return
        dim = param.output_dim
        names = list(sections)
        if loaded_shard_id is None:
            offset, size = 0, data.shape[dim]
        else:
            i = names.index(loaded_shard_id)
            size = sections[loaded_shard_id] // tp_size
            offset = sum(sections[n] for n in names[:i]) // tp_size
        data.narrow(dim, offset, size).copy_(loaded_weight.narrow(dim, tp_rank * size, size))
    return loader


def test_checkpoint_tensors_through_the_vllm_weight_loader_callbacks():
    """`<prefix>.codes / .norms / .ct_scaled` as vLLM's model loader delivers them (by parameter name, one call per
    checkpoint tensor, fused q/k/v sections by shard id, tensor-parallel narrowing by the layer's own loader) land in
    the parameters `create_weights` registered: nibble-packed and 5-bit-packed codes are unpacked on the way, so the
    result equals the rank's slice of the quantizer's int8 codes."""
    from polarengine_vllm_b200.linear_method import PolarQuantLinearMethod
    from polarengine_vllm_b200.packing import pack_codes_half_block, pack_codes_q5
    g = torch.Generator().manual_seed(5)
    hidden, tp = 512, 2
    # fused q/k/v (Q5, stored 5-bit packed), column parallel
    sections = {"q": 256, "k": 128, "v": 128}
    q5 = {n: oracle.quantize_tensor(torch.randn(rows, hidden, generator=g) * 0.02, 5) for n, rows in sections.items()}
    for rank in range(tp):
        m = PolarQuantLinearMethod(128, 5)
        layer = torch.nn.Module()
        m.create_weights(layer, hidden, [r // tp for r in sections.values()], hidden, sum(sections.values()), torch.float16,
                         weight_loader=_vllm_like_layer_loader(sections, rank, tp))
        params = dict(layer.named_parameters())
        assert set(params) == {"codes", "norms", "ct_scaled"}
        for n in sections:   # three checkpoint layers feed one fused parameter
            params["codes"].weight_loader(params["codes"], pack_codes_q5(q5[n]["codes"]), n)
            params["norms"].weight_loader(params["norms"], q5[n]["norms"], n)
            params["ct_scaled"].weight_loader(params["ct_scaled"], q5[n]["ct_scaled"], n)
        want_c = torch.cat([q5[n]["codes"].chunk(tp, 0)[rank] for n in sections])
        want_n = torch.cat([q5[n]["norms"].chunk(tp, 0)[rank] for n in sections])
        assert torch.equal(layer.codes.data, want_c) and torch.equal(layer.norms.data, want_n)
        assert torch.equal(layer.ct_scaled.data, q5["q"]["ct_scaled"])
    # down projection (Q4, stored nibble-packed), row parallel: whole blocks of K per rank
    q4 = oracle.quantize_tensor(torch.randn(192, hidden, generator=g) * 0.02, 4)
    for rank in range(tp):
        m = PolarQuantLinearMethod(128, 4)
        layer = torch.nn.Module()
        m.create_weights(layer, hidden // tp, [192], hidden, 192, torch.float16,
                         weight_loader=_vllm_like_layer_loader({}, rank, tp, row_parallel=True))
        layer.codes.weight_loader(layer.codes, pack_codes_half_block(q4["codes"]))
        layer.norms.weight_loader(layer.norms, q4["norms"])
        layer.ct_scaled.weight_loader(layer.ct_scaled, q4["ct_scaled"])
        k0 = rank * hidden // tp
        assert torch.equal(layer.codes.data, q4["codes"][:, k0:k0 + hidden // tp])
        assert torch.equal(layer.norms.data, q4["norms"][:, rank * 2:(rank + 1) * 2])
    # a layer without a framework loader (offline use): plain copies, int8 codes as they are
    m = PolarQuantLinearMethod(128, 4)
    layer = torch.nn.Module()
    m.create_weights(layer, hidden, [192], hidden, 192, torch.float16)
    layer.codes.weight_loader(layer.codes, q4["codes"])
    assert torch.equal(layer.codes.data, q4["codes"])
    with pytest.raises(ValueError):
        layer.codes.weight_loader(layer.codes, torch.zeros(192, 100, dtype=torch.uint8))
