"""The native quantizer (pe_quantize) against the CPU oracle of the reference's quantize_tensor
(quantizer.py:178-257): norms equal to within one fp16 step, codes equal except where a rotated value sits on a
cell boundary to within fp32 rounding (bounded flip rate, every flip to a neighbouring level), and the
dequantised weights equally close to the original."""
import pytest
import torch

import polar_oracle as oracle

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("bits", [2, 3, 4, 5, 6, 8])
def test_gpu_quantizer_matches_the_cpu_order(bits):
    from polarengine_vllm_b200.quantizer import PolarQuantizer
    g = torch.Generator().manual_seed(bits)
    w = torch.randn(512, 1000, generator=g) * 0.02     # ragged K: pads to 1024
    w[7] = 0                                            # an all-zero row: norm clamps at 1e-10
    ref = oracle.quantize_tensor(w, bits)
    q = PolarQuantizer().quantize_tensor_gpu(w.cuda(), bits)
    codes, norms = q["codes"].cpu(), q["norms"].cpu()
    assert codes.shape == ref["codes"].shape and codes.dtype == torch.int8 and norms.dtype == torch.float16
    assert torch.equal(q["ct_scaled"].cpu(), ref["ct_scaled"])
    # norms: the sum of squares is taken in another order
    assert ((norms.float() - ref["norms"].float()).abs() <= ref["norms"].float().abs() * 2 ** -10 + 1e-12).all()
    live = torch.ones(512, dtype=torch.bool); live[7] = False   # codes of a zero block are noise around 0 either way
    diff = (codes[live].view(torch.uint8).int() - ref["codes"][live].view(torch.uint8).int()).abs()
    flips = int((diff != 0).sum())
    assert flips <= max(8, int(2e-5 * diff.numel())), f"{flips} of {diff.numel()} codes differ"
    assert int(diff.max()) <= 1                                  # and only to the neighbouring level
    a = oracle.dequant_fp32(codes, norms, q["ct_scaled"].cpu())[:, :1000]
    b = oracle.dequant_fp32(ref["codes"], ref["norms"], ref["ct_scaled"])[:, :1000]
    ea, eb = float((a - w).norm() / w.norm()), float((b - w).norm() / w.norm())
    assert abs(ea - eb) <= 1e-4 * max(eb, 1e-6) + 1e-6


def test_gpu_quantizer_half_and_bf16_inputs():
    from polarengine_vllm_b200.quantizer import PolarQuantizer
    g = torch.Generator().manual_seed(1)
    w = (torch.randn(64, 384, generator=g) * 0.02)
    for dt in (torch.float16, torch.bfloat16):
        wd = w.to(dt)
        ref = oracle.quantize_tensor(wd.float(), 4)
        q = PolarQuantizer().quantize_tensor_gpu(wd.cuda(), 4)
        assert (q["codes"].cpu() != ref["codes"]).float().mean() < 1e-3
