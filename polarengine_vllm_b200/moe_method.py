"""MoE methods behind vLLM's fused-MoE interface.

Reference: polarengine_vllm/moe_method.py:18-107 (``PolarPassthroughMoEMethod``), which
keeps expert weights in bf16 and forwards every call to vLLM's unquantized fused MoE.
That pass-through is kept here under the same name and with the same lazy construction.
"""
from __future__ import annotations

import torch


class PolarPassthroughMoEMethod:
    """Delegates to vLLM's ``UnquantizedFusedMoEMethod``; built lazily because vLLM asks
    for the method before the FusedMoE layer is fully constructed."""

    def __init__(self) -> None:
        self._inner = None

    def _lazy_init(self, layer) -> bool:
        if self._inner is None:
            try:
                from vllm.model_executor.layers.fused_moe.unquantized_fused_moe_method import UnquantizedFusedMoEMethod
                self._inner = UnquantizedFusedMoEMethod(moe=layer)
            except (AttributeError, TypeError, ImportError):
                return False
        return True

    def create_weights(self, layer, num_experts, hidden_size, intermediate_size_per_partition, params_dtype, **kw):
        if self._lazy_init(layer):
            return self._inner.create_weights(layer, num_experts=num_experts, hidden_size=hidden_size,
                                              intermediate_size_per_partition=intermediate_size_per_partition,
                                              params_dtype=params_dtype, **kw)
        for name, shape in (("w13_weight", (num_experts, 2 * intermediate_size_per_partition, hidden_size)),
                            ("w2_weight", (num_experts, hidden_size, intermediate_size_per_partition))):
            layer.register_parameter(name, torch.nn.Parameter(torch.empty(*shape, dtype=params_dtype), requires_grad=False))

    def apply(self, layer, x, *args, **kwargs):
        if not self._lazy_init(layer):
            raise RuntimeError("PolarPassthroughMoEMethod: vLLM's fused MoE method could not be constructed")
        return self._inner.apply(layer, x, *args, **kwargs)

    def get_fused_moe_quant_config(self, *args):
        if self._inner is not None and hasattr(self._inner, "get_fused_moe_quant_config"):
            return self._inner.get_fused_moe_quant_config(*args)
        return None


def make_moe_method(config, layer, prefix):
    return PolarPassthroughMoEMethod()


try:
    from vllm.model_executor.layers.fused_moe.layer import FusedMoEMethodBase
    FusedMoEMethodBase.register(PolarPassthroughMoEMethod)
except Exception:
    pass
