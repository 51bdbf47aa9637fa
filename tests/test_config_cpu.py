"""The vLLM-facing config class (reference tests/test_config.py, minus its stale case:
an unmatched layer now gets vLLM's unquantized method, config.py:208-210)."""
import pytest
import torch

from polarengine_vllm_b200.config import HAVE_VLLM, PolarQuantConfig

CFG = {
    "format": "polar_engine_v4", "quantization": "polarengine", "block_size": 128,
    "bit_assignment": {"q_proj": 5, "k_proj": 5, "v_proj": 5, "o_proj": 6, "gate_up_proj": 3, "gate_proj": 3,
                       "up_proj": 3, "down_proj": 4, "embed": 5, "lm_head": 6},
    "layers": {"model.layers.0.self_attn.q_proj": {"in_features": 4096, "out_features": 4096, "bits": 5},
               "model.layers.0.mlp.special": {"bits": 2}},
}


def test_from_config_and_constants():
    c = PolarQuantConfig.from_config(CFG)
    assert c.block_size == 128 and c.bit_assignment["down_proj"] == 4 and len(c.layers_meta) == 2
    d = PolarQuantConfig.from_config({})
    assert d.block_size == 128 and d.bit_assignment == {} and d.layers_meta == {}
    assert PolarQuantConfig.get_name() == "polarengine"
    assert PolarQuantConfig.get_config_filenames() == ["polar_config.json"]
    assert PolarQuantConfig.get_min_capability() == 70
    assert set(PolarQuantConfig.get_supported_act_dtypes()) == {torch.float16, torch.bfloat16}
    assert "PolarQuantConfig" in repr(c)
    PolarQuantConfig.from_config({"format": "something-else"})  # warns, does not raise


def test_resolve_bits_precedence():
    c = PolarQuantConfig.from_config(CFG)
    assert c._resolve_bits("model.layers.0.self_attn.q_proj") == 5      # exact entry
    assert c._resolve_bits("model.layers.0.mlp.special") == 2           # exact entry beats patterns
    assert c._resolve_bits("model.layers.7.mlp.gate_up_proj") == 3      # longest pattern wins
    assert c._resolve_bits("model.layers.7.mlp.gate_proj") == 3
    assert c._resolve_bits("model.layers.7.self_attn.qkv_proj") == 5    # contains "v_proj"
    assert c._resolve_bits("model.layers.7.mixer.conv") is None


@pytest.mark.skipif(not HAVE_VLLM, reason="vLLM not importable")
def test_method_selection():
    from vllm.model_executor.layers.linear import UnquantizedLinearMethod
    from polarengine_vllm_b200.linear_method import PolarQuantLinearMethod
    c = PolarQuantConfig.from_config(CFG)
    m = c.get_quant_method(torch.nn.Linear(8, 8), "model.layers.3.mlp.down_proj")
    assert isinstance(m, PolarQuantLinearMethod) and m.bits == 4 and m.block_size == 128
    assert isinstance(c.get_quant_method(torch.nn.Linear(8, 8), "model.layers.3.unknown"), UnquantizedLinearMethod)
    assert isinstance(c.get_quant_method(torch.nn.LayerNorm(8), "model.norm"), UnquantizedLinearMethod)
    assert type(c.get_quant_method(torch.nn.Embedding(4, 4), "model.embed_tokens")).__name__ == "UnquantizedEmbeddingMethod"


def test_create_weights_on_cpu():
    from polarengine_vllm_b200.linear_method import PolarQuantLinearMethod, create_fwht_clear_hook
    m = PolarQuantLinearMethod(128, 4)
    layer = torch.nn.Module()
    seen = {}
    m.create_weights(layer, 1856, [1000, 344], 1856, 1344, torch.float16, weight_loader=lambda *a: seen.update(ok=1))
    assert layer.codes.shape == (1344, 1920) and layer.codes.dtype == torch.int8
    assert layer.norms.shape == (1344, 15) and layer.norms.dtype == torch.float16
    assert layer.ct_scaled.shape == (16,) and layer.ct_scaled.dtype == torch.float32
    assert (layer.in_f, layer.out_f, layer.in_f_padded, layer.n_blocks, layer.bits, layer.packed) == (1856, 1344, 1920, 15, 4, False)
    assert layer.codes.input_dim == 1 and layer.codes.output_dim == 0 and callable(layer.codes.weight_loader)
    assert not layer.codes.requires_grad
    with pytest.raises(ValueError):  # a K shard must be whole blocks
        m.create_weights(torch.nn.Module(), 1000, [8], 4000, 8, torch.float16)
    with pytest.raises(ValueError):
        PolarQuantLinearMethod(64, 4)
    assert create_fwht_clear_hook(m)(None, None) is None  # kept for callers written against the reference


@pytest.mark.skipif(not HAVE_VLLM, reason="vLLM not importable")
def test_plugin_entry_point_registers_with_vllm():
    """``vllm.general_plugins`` calls register_polar_quant(); afterwards ``--quantization polarengine``
    resolves to this package's config class (reference: polarengine_vllm/__init__.py:24-38)."""
    import polarengine_vllm_b200
    polarengine_vllm_b200.register_polar_quant()
    from vllm.model_executor.layers.quantization import QUANTIZATION_METHODS, get_quantization_config
    assert "polarengine" in QUANTIZATION_METHODS
    assert get_quantization_config("polarengine") is PolarQuantConfig


def test_packaging_declares_the_vllm_entry_point():
    """The packaging metadata names the entry point vLLM discovers plugins by, with the reference's group and
    name (setup.py:31-34, pyproject.toml:45-46), and the target resolves to the registration function."""
    import importlib
    import os
    import tomllib
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    with open(os.path.join(root, "pyproject.toml"), "rb") as f:
        meta = tomllib.load(f)
    eps = meta["project"]["entry-points"]["vllm.general_plugins"]
    assert list(eps) == ["polarengine"]
    mod_name, _, attr = eps["polarengine"].partition(":")
    fn = getattr(importlib.import_module(mod_name), attr)
    import polarengine_vllm_b200
    assert fn is polarengine_vllm_b200.register_polar_quant
    assert "libpolar_b200.so" in meta["tool"]["setuptools"]["package-data"]["polarengine_vllm_b200"]
