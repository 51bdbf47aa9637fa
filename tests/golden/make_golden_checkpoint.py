"""Write two tiny PolarEngine checkpoints under tests/golden/ and what the REFERENCE's loader
returns for every layer of them.

    python tests/golden/make_golden_checkpoint.py /path/to/polarengine-vllm

The checkpoints are produced with the reference's own quantizer and packers
(polarengine_vllm.quantizer / packing) and read back with its PolarWeightLoader
(polarengine_vllm/loader.py); `checkpoint_expected.npz` holds the loader's outputs.  The
tests read only these files.
"""
import json
import math
import os
import sys

import numpy as np
import torch
from safetensors.torch import save_file

if len(sys.argv) < 2:
    sys.exit("usage: make_golden_checkpoint.py /path/to/polarengine-vllm")
sys.path.insert(0, sys.argv[1])
here = os.path.dirname(os.path.abspath(__file__))

from polarengine_vllm import packing  # noqa: E402
from polarengine_vllm.loader import PolarWeightLoader, load_polar_config  # noqa: E402
from polarengine_vllm.quantizer import PolarQuantizer  # noqa: E402


def quantize(n, k, bits, seed):
    g = torch.Generator().manual_seed(seed)
    q = PolarQuantizer(block_size=128)
    r = q.quantize_tensor(torch.randn(n, k, generator=g) * 0.02, bits)
    return r["codes"], r["norms"], r["ct_scaled"]


expected = {}

# --- split-tensor format: int8 codes, nibble-packed codes, LSB-first packed Q5 with unscaled centroids, a dense tensor
d = os.path.join(here, "ckpt_v5")
os.makedirs(d, exist_ok=True)
c6, n6, t6 = quantize(16, 256, 6, 1)
c4, n4, t4 = quantize(24, 200, 4, 2)
c5, n5, t5 = quantize(8, 256, 5, 3)
shard_a = {"m.o_proj.codes": c6, "m.o_proj.norms": n6, "m.o_proj.ct_scaled": t6, "m.o_proj.bias": torch.arange(16).half(),
           "m.down_proj.codes": packing.pack_codes_half_block(c4), "m.down_proj.norms": n4, "m.down_proj.ct_scaled": t4}
shard_b = {"m.q_proj.codes": packing.pack_codes_q5(c5), "m.q_proj.norms": n5, "m.q_proj.ct": t5 * math.sqrt(128),
           "m.norm.weight": torch.linspace(0.5, 1.5, 32).half()}
save_file(shard_a, os.path.join(d, "model-00001-of-00002.safetensors"))
save_file(shard_b, os.path.join(d, "model-00002-of-00002.safetensors"))
wm = {k: "model-00001-of-00002.safetensors" for k in shard_a}
wm.update({k: "model-00002-of-00002.safetensors" for k in shard_b})
json.dump({"weight_map": wm}, open(os.path.join(d, "model.safetensors.index.json"), "w"), indent=1)
json.dump({"format": "polar_engine_v5", "block_size": 128,
           "layers": {"m.o_proj": {"bits": 6}, "m.down_proj": {"bits": 4, "in_features": 200},
                      "m.q_proj": {"bits": 5, "packed_q5": True}}}, open(os.path.join(d, "polar_config.json"), "w"), indent=1)
ref = PolarWeightLoader(d, load_polar_config(d))
for layer in ("m.o_proj", "m.down_proj", "m.q_proj", "m.norm"):
    for key, val in ref.load_layer_weights(layer).items():
        expected[f"v5/{layer}/{key}"] = val.float().numpy() if val.dtype in (torch.float16, torch.bfloat16) else val.numpy()
expected["v5/layer_names"] = np.array(sorted(ref.get_all_layer_names()))
ref.close()

# --- HLWQ 5-bit stream format
d = os.path.join(here, "ckpt_hlwq")
os.makedirs(d, exist_ok=True)
ch, nh, _ = quantize(8, 200, 5, 4)
tensors = {"l.weight__packed": packing.pack_codes_q5_hlwq(ch.flatten()), "l.weight__norms": nh.flatten(),
           "l.weight__meta": torch.tensor([8, 2, 128, ch.numel(), 200], dtype=torch.int64)}
save_file(tensors, os.path.join(d, "model.safetensors"))
json.dump({"weight_map": {k: "model.safetensors" for k in tensors}}, open(os.path.join(d, "model.safetensors.index.json"), "w"), indent=1)
json.dump({"format": "hlwq-q5", "block_size": 128}, open(os.path.join(d, "polar_config.json"), "w"), indent=1)
ref = PolarWeightLoader(d, load_polar_config(d))
for key, val in ref.load_layer_weights("l").items():
    expected[f"hlwq/l/{key}"] = val.float().numpy() if val.dtype in (torch.float16, torch.bfloat16) else val.numpy()
ref.close()

np.savez_compressed(os.path.join(here, "checkpoint_expected.npz"), **expected)
print("wrote", sorted(expected))
