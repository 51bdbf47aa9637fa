"""Generate the golden vectors under tests/golden/ by importing the reference project.

Run once in a container where the reference checkout is mounted:

    python tests/golden/make_golden.py /path/to/polarengine-vllm

It imports the reference's own CPU code (centroids, Hadamard matrix, quantizer,
packers, dequantiser) and stores small seeded input/output pairs.  The fixtures are
committed; the tests read only the .npz files and never the reference checkout.
"""
import math
import os
import sys

import numpy as np
import torch

if len(sys.argv) < 2:
    sys.exit("usage: make_golden.py /path/to/polarengine-vllm")
ref_root = sys.argv[1]
sys.path.insert(0, ref_root)
here = os.path.dirname(os.path.abspath(__file__))

from polarengine_vllm.utils import get_centroids, get_bits_for_layer, DEFAULT_BIT_ASSIGNMENT  # noqa: E402
from polarengine_vllm.kernels.fwht import build_hadamard, fwht_matmul, fwht_butterfly  # noqa: E402
from polarengine_vllm.quantizer import PolarQuantizer  # noqa: E402
from polarengine_vllm import packing  # noqa: E402
from polarengine_vllm.weight_converter import _dequant_weight  # noqa: E402

out = {}

# Lloyd-Max tables, every supported width, exact fp32 bits.
for b in range(2, 9):
    out[f"centroids_{b}"] = get_centroids(b).numpy()

# Hadamard matrix and a rotated sample.
out["hadamard_128"] = build_hadamard(128).numpy()
g = torch.Generator().manual_seed(3)
xs = torch.randn(5, 384, generator=g)
out["fwht_in"] = xs.clone().numpy()
out["fwht_out"] = fwht_matmul(xs, 128).numpy()
out["fwht_butterfly_out"] = fwht_butterfly(xs.clone().reshape(-1, 128)).reshape(5, 384).numpy()

# Quantizer: ragged K (300 -> 384), several widths, plus a 64-row-chunk boundary (70 rows).
q = PolarQuantizer(block_size=128)
g = torch.Generator().manual_seed(11)
w = torch.randn(70, 300, generator=g) * 0.02
out["quant_w"] = w.numpy()
for b in (2, 3, 4, 5, 6, 8):
    r = q.quantize_tensor(w, b)
    out[f"quant_codes_{b}"] = r["codes"].numpy()
    out[f"quant_norms_{b}"] = r["norms"].numpy()
    out[f"quant_ct_scaled_{b}"] = r["ct_scaled"].numpy()

# Degenerate blocks: an all-zero row exercises the 1e-10 clamp.
wz = w.clone()
wz[3] = 0
rz = q.quantize_tensor(wz, 4)
out["quant_zero_row_codes_4"] = rz["codes"].numpy()
out["quant_zero_row_norms_4"] = rz["norms"].numpy()

# Layouts.
g = torch.Generator().manual_seed(5)
c4 = torch.randint(0, 16, (6, 256), generator=g, dtype=torch.int8)
out["nib_codes"] = c4.numpy()
out["nib_packed"] = packing.pack_codes_half_block(c4, 128).numpy()
c5 = torch.randint(0, 32, (4, 256), generator=g, dtype=torch.int8)
out["q5_codes"] = c5.numpy()
out["q5_packed"] = packing.pack_codes_q5(c5, 128).numpy()
out["q5_hlwq_packed"] = packing.pack_codes_q5_hlwq(c5).numpy()
assert torch.equal(packing.unpack_codes_q5(packing.pack_codes_q5(c5)), c5)
assert torch.equal(packing.unpack_codes_q5_hlwq(packing.pack_codes_q5_hlwq(c5)), c5)

# Forward: the reference's two CPU-runnable forms of one quantized linear
# (4-bit and 5-bit; x fp16; Hadamard-domain einsum, and dequant + matmul).
g = torch.Generator().manual_seed(7)
x = torch.randn(3, 300, generator=g).half()
out["fwd_x"] = x.numpy()
for b in (4, 5):
    codes = torch.from_numpy(out[f"quant_codes_{b}"])
    norms = torch.from_numpy(out[f"quant_norms_{b}"])
    cts = torch.from_numpy(out[f"quant_ct_scaled_{b}"])
    xp = torch.nn.functional.pad(x.float(), (0, 84))
    xt = fwht_matmul(xp, 128).view(3, 3, 128)
    vals = cts[codes.long()].view(70, 3, 128) * norms.float().view(70, 3, 1)
    out[f"fwd_hadamard_{b}"] = torch.einsum("rnk,mnk->mr", vals, xt).numpy()
    # _dequant_weight expects unscaled centroids and returns bf16
    wd = _dequant_weight(codes, norms, cts * math.sqrt(128), 128)
    out[f"fwd_dequant_bf16_{b}"] = wd.float().numpy()

# Bit table as (name, bits) pairs.
names = [
    "model.embed_tokens.weight", "lm_head.weight",
    "model.layers.0.self_attn.q_proj.weight", "model.layers.0.self_attn.k_proj.weight",
    "model.layers.0.self_attn.v_proj.weight", "model.layers.0.self_attn.o_proj.weight",
    "model.layers.0.self_attn.qkv_proj.weight",
    "model.layers.0.mlp.gate_proj.weight", "model.layers.0.mlp.up_proj.weight",
    "model.layers.0.mlp.gate_up_proj.weight", "model.layers.0.mlp.down_proj.weight",
    "model.layers.0.mixer.in_proj.weight", "model.layers.0.mixer.out_proj.weight",
    "model.layers.0.input_layernorm.weight", "model.layers.0.mixer.A_log",
    "model.layers.0.mixer.D", "model.layers.0.mixer.conv1d.weight",
    "model.layers.0.mlp.gate.weight", "model.layers.0.mlp.router.weight",
    "model.layers.0.mlp.experts.3.down_proj.weight", "model.layers.0.something_else.weight",
]
big = torch.zeros(64, 64)
out["bits_names"] = np.array(names)
out["bits_values"] = np.array([get_bits_for_layer(n, big) for n in names], dtype=np.int32)
out["bits_default_keys"] = np.array(sorted(DEFAULT_BIT_ASSIGNMENT))
out["bits_default_vals"] = np.array([DEFAULT_BIT_ASSIGNMENT[k] for k in sorted(DEFAULT_BIT_ASSIGNMENT)], dtype=np.int32)

np.savez_compressed(os.path.join(here, "polar_golden.npz"), **out)
print("wrote", os.path.join(here, "polar_golden.npz"), {k: v.shape for k, v in out.items()})
