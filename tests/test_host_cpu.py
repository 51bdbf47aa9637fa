"""Host-side mirror of the reference's plugin surface, on the CPU: packing, Lloyd-Max
tables, bit table, Hadamard helpers, config parsing, quantizer.  Same assertions as the
reference's tests/test_packing.py, test_utils.py, test_fwht.py and test_config.py,
re-targeted at this package, plus golden vectors produced by the reference."""
import math

import numpy as np
import pytest
import torch

from polarengine_vllm_b200 import packing, utils
from polarengine_vllm_b200.fwht import FWHTCache, build_hadamard, fwht_butterfly, fwht_matmul
from polarengine_vllm_b200.quantizer import PolarQuantizer


# ---- packing (reference tests/test_packing.py) -------------------------------
@pytest.mark.parametrize("shape", [(64, 512), (4096, 4096), (12288, 4096)])
def test_nibble_roundtrip(shape):
    codes = torch.randint(0, 16, shape, dtype=torch.int8)
    packed = packing.pack_codes_half_block(codes)
    assert packed.dtype == torch.uint8 and packed.shape == (shape[0], shape[1] // 2)
    assert torch.equal(packing.unpack_codes_half_block(packed), codes)
    assert packing.verify_packing_roundtrip(codes)


def test_nibble_known_answers():
    for lo, hi, byte in [(3, 12, 0xC3), (15, 0, 0x0F), (0, 15, 0xF0)]:
        c = torch.zeros(8, 512, dtype=torch.int8).view(8, 4, 128)
        c[:, :, :64], c[:, :, 64:] = lo, hi
        assert (packing.pack_codes_half_block(c.reshape(8, 512)) == byte).all()


@pytest.mark.parametrize("bs", [32, 64, 128, 256])
def test_nibble_block_sizes(bs):
    codes = torch.randint(0, 16, (16, bs * 4), dtype=torch.int8)
    assert packing.verify_packing_roundtrip(codes, bs)


def test_nibble_two_implementations_agree():
    codes = torch.randint(0, 16, (32, 1024), dtype=torch.int8)
    assert torch.equal(packing.pack_codes_half_block(codes), utils.pack_codes_half_block(codes))
    lead = torch.randint(0, 16, (3, 5, 256), dtype=torch.int8)  # N-D leading dims (utils.py:211-260)
    assert torch.equal(utils.unpack_codes_half_block(utils.pack_codes_half_block(lead)), lead)
    with pytest.raises(ValueError):
        utils.pack_codes_half_block(torch.zeros(2, 100, dtype=torch.int8))


def test_pack_rejects_out_of_range():
    with pytest.raises(AssertionError):
        packing.pack_codes_half_block(torch.full((2, 128), 16, dtype=torch.int8))


def test_q5_layouts_golden(golden):
    c5 = torch.from_numpy(golden["q5_codes"])
    assert np.array_equal(packing.pack_codes_q5(c5).numpy(), golden["q5_packed"])
    assert np.array_equal(packing.pack_codes_q5_hlwq(c5).numpy(), golden["q5_hlwq_packed"])
    assert torch.equal(packing.unpack_codes_q5(torch.from_numpy(golden["q5_packed"])), c5)
    assert torch.equal(packing.unpack_codes_q5_hlwq(torch.from_numpy(golden["q5_hlwq_packed"])), c5)
    assert packing.unpack_codes_q5_hlwq(torch.from_numpy(golden["q5_hlwq_packed"]), total=250).shape == (4, 250)
    big = torch.randint(0, 32, (64, 4096), dtype=torch.int8)
    assert packing.pack_codes_q5(big).shape == (64, 2560) and packing.verify_q5_roundtrip(big)


def test_pack_model_codes():
    class Fake(torch.nn.Module):
        def __init__(self, bits):
            super().__init__()
            self.bits = bits
            self.register_buffer("codes", torch.randint(0, 1 << min(bits, 4), (64, 256), dtype=torch.int8))

    model = torch.nn.Module()
    model.a, model.b, model.c = Fake(3), Fake(4), Fake(5)
    before = model.a.codes.clone()
    stats = packing.pack_model_codes(model)
    assert stats["layers_packed"] == 2 and stats["layers_skipped"] == 1
    assert model.a.packed and not hasattr(model.a, "codes") and model.a.in_f_half == 128
    assert torch.equal(packing.unpack_codes_half_block(model.a.codes_packed), before)
    assert hasattr(model.c, "codes") and stats["bytes_after"] * 2 == stats["bytes_before"]


# ---- centroids and the bit table (reference tests/test_utils.py) ---------------
@pytest.mark.parametrize("bits", [2, 3, 4, 5, 6])
def test_centroid_properties(bits, golden):
    c = utils.get_centroids(bits)
    assert c.dtype == torch.float32 and c.shape == (1 << bits,)
    assert torch.isfinite(c).all() and (c[1:] > c[:-1]).all()
    assert torch.allclose(c, -c.flip(0), atol=1e-5)
    assert utils.get_centroids(bits) is c
    assert np.array_equal(c.numpy(), golden[f"centroids_{bits}"])


def test_centroid_errors_and_convergence():
    for bad in (1, 9):
        with pytest.raises(ValueError):
            utils.get_centroids(bad)
    a = utils.compute_lloyd_max_centroids(16, 200)
    b = utils.compute_lloyd_max_centroids(16, 300)
    assert torch.allclose(a, b, atol=0.01)
    assert torch.allclose(utils.get_ct_scaled(4), utils.get_centroids(4) / math.sqrt(128))


def test_bit_table_golden(golden):
    big = torch.zeros(64, 64)
    for name, bits in zip(golden["bits_names"], golden["bits_values"]):
        assert utils.get_bits_for_layer(str(name), big) == int(bits), name
    assert dict(zip(map(str, golden["bits_default_keys"]), map(int, golden["bits_default_vals"]))) == utils.DEFAULT_BIT_ASSIGNMENT
    assert utils.get_bits_for_layer("model.layers.0.mlp.down_proj.weight", torch.zeros(8, 8)) == 16
    assert utils.get_bits_for_layer("x.q_proj.bias", torch.zeros(512)) == 16
    assert utils.get_bits_for_layer("x.q_proj.weight", big, {"q_proj": 7}) == 7


# ---- rotation helpers (reference tests/test_fwht.py) --------------------------
def test_hadamard_properties(golden):
    h = build_hadamard(128)
    assert np.array_equal(h.numpy(), golden["hadamard_128"])
    assert torch.allclose(h @ h, torch.eye(128), atol=1e-5) and torch.equal(h, h.T)
    assert torch.allclose(build_hadamard(2), torch.tensor([[1.0, 1.0], [1.0, -1.0]]) / math.sqrt(2))
    assert build_hadamard(128) is h
    with pytest.raises(AssertionError):
        build_hadamard(100)


def test_fwht_cpu_forms(golden):
    x = torch.from_numpy(golden["fwht_in"])
    y = fwht_matmul(x)
    assert np.array_equal(y.numpy(), golden["fwht_out"])
    assert torch.allclose(fwht_butterfly(x.reshape(-1, 128)).reshape(x.shape), y, atol=1e-5)
    assert torch.allclose(fwht_matmul(y), x, atol=1e-5)
    with pytest.raises(AssertionError):
        fwht_matmul(torch.zeros(2, 100))


def test_fwht_cache_semantics():
    cache = FWHTCache()
    a, b = torch.zeros(4, 128), torch.zeros(4, 128)
    assert cache.get(a, 128) is None
    cache.put(a, 128, a)
    assert cache.get(a, 128) is a and cache.get(a, 64) is None and cache.get(b, 128) is None
    cache.put(b, 128, b)  # single entry: the first one is gone
    assert cache.get(a, 128) is None and cache.get(b, 128) is b
    cache.clear()
    assert cache.get(b, 128) is None


# ---- quantizer (reference quantizer.py:178-257; pinned by golden vectors) -------
@pytest.mark.parametrize("bits", [2, 3, 4, 5, 6, 8])
def test_quantizer_matches_reference(golden, bits):
    r = PolarQuantizer().quantize_tensor(torch.from_numpy(golden["quant_w"]), bits)
    assert np.array_equal(r["codes"].numpy(), golden[f"quant_codes_{bits}"])
    assert np.array_equal(r["norms"].numpy(), golden[f"quant_norms_{bits}"])
    assert np.array_equal(r["ct_scaled"].numpy(), golden[f"quant_ct_scaled_{bits}"])


def test_quantize_state_dict_layout():
    g = torch.Generator().manual_seed(0)
    state = {"model.layers.0.self_attn.q_proj.weight": torch.randn(32, 256, generator=g),
             "model.layers.0.mlp.down_proj.weight": torch.randn(32, 200, generator=g),
             "model.layers.0.input_layernorm.weight": torch.ones(256)}
    tensors, cfg = PolarQuantizer().quantize_state_dict(state)
    assert cfg["format"] == "polar_engine_v5" and cfg["quantization"] == "polarengine"
    meta = cfg["layers"]["model.layers.0.mlp.down_proj"]
    assert meta["bits"] == 4 and meta["packed"] and meta["in_features_padded"] == 256 and meta["n_blocks"] == 2
    assert tensors["model.layers.0.mlp.down_proj.codes"].shape == (32, 128)
    assert cfg["layers"]["model.layers.0.self_attn.q_proj"]["packed_q5"]
    assert tensors["model.layers.0.self_attn.q_proj.codes"].shape == (32, 160)
    assert tensors["model.layers.0.input_layernorm.weight"].dtype == torch.float16
