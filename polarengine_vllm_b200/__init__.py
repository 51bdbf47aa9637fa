"""B200-native kernels for the PolarEngine quantized-linear path, behind the vLLM
plugin surface of caiovicentino/polarengine-vllm.

``register_polar_quant`` is the ``vllm.general_plugins`` entry point
(reference: polarengine_vllm/__init__.py:24-38): importing the config module registers
the ``"polarengine"`` quantization method.  Nothing here imports vLLM or loads the
native library until it is needed.
"""
__version__ = "0.1.0"


def register_polar_quant() -> None:
    from . import config  # noqa: F401  (registration happens on import)


__all__ = ["register_polar_quant", "__version__"]
