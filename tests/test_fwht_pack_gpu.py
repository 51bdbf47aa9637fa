"""Native rotation and nibble-packing kernels against the oracle."""
import numpy as np
import pytest
import torch

import polar_oracle as oracle

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("batch,in_f", [(1, 128), (3, 300), (5, 4096), (17, 1856), (64, 12288)])
def test_fwht128_matches_oracle(dtype, batch, in_f):
    from polarengine_vllm_b200.fwht import fwht128
    g = torch.Generator().manual_seed(batch + in_f)
    x = torch.randn(batch, in_f, generator=g).to(dtype)
    kp = (in_f + 127) // 128 * 128
    ref = oracle.fwht(torch.nn.functional.pad(x.float(), (0, kp - in_f)))
    y = fwht128(x.cuda(), kp, torch.float32).cpu()
    assert y.shape == (batch, kp)
    # butterfly order vs one matmul: same value up to fp32 rounding (reference tolerance 1e-5,
    # tests/test_fwht.py:19-40)
    assert (y - ref).abs().max() <= 1e-5 * max(1.0, float(ref.abs().max()))
    y16 = fwht128(x.cuda(), kp, torch.float16).cpu()
    assert (y16.float() - ref).abs().max() <= 2e-3 * max(1.0, float(ref.abs().max()))


def test_fwht_is_involution_on_device():
    from polarengine_vllm_b200.fwht import fwht_matmul
    x = torch.randn(8, 1024, generator=torch.Generator().manual_seed(0)).cuda()
    assert (fwht_matmul(fwht_matmul(x)) - x).abs().max() < 1e-5


@pytest.mark.parametrize("n,k", [(1, 128), (6, 256), (4096, 4096), (1000, 1920)])
def test_pack_nibble_bit_exact(n, k):
    from polarengine_vllm_b200.packing import pack_codes_half_block
    g = torch.Generator().manual_seed(n)
    codes = torch.randint(0, 16, (n, k), generator=g, dtype=torch.int16).to(torch.int8)
    packed = pack_codes_half_block(codes.cuda()).cpu().numpy()
    assert packed.dtype == np.uint8 and packed.shape == (n, k // 2)
    assert np.array_equal(packed, oracle.pack_nibble(codes.numpy()))


def test_pack_golden(golden):
    from polarengine_vllm_b200.packing import pack_codes_half_block
    out = pack_codes_half_block(torch.from_numpy(golden["nib_codes"]).cuda()).cpu().numpy()
    assert np.array_equal(out, golden["nib_packed"])


@pytest.mark.parametrize("bits,hidden", [(5, 4096), (4, 300), (6, 1856)])
def test_quantized_embedding_rows(bits, hidden):
    """Embedding gather = rows of the fp32 dequantised table (weight_converter.py:34-67 math)."""
    from polarengine_vllm_b200 import kernels, packing
    g = torch.Generator().manual_seed(bits)
    w = torch.randn(500, hidden, generator=g) * 0.02
    q = oracle.quantize_tensor(w, bits)
    table = oracle.dequant_fp32(q["codes"], q["norms"], q["ct_scaled"])[:, :hidden]
    ids = torch.randint(0, 500, (3, 7), generator=g)
    packed = bits <= 4
    cd = q["codes"].cuda()
    cw = packing.pack_codes_half_block(cd) if packed else cd
    out = kernels.quant_embedding(cw, packed, q["norms"].cuda(), q["ct_scaled"].cuda(), ids.cuda(), hidden, torch.float32)
    assert out.shape == (3, 7, hidden)
    ref = table[ids]
    assert (out.cpu() - ref).abs().max() <= 1e-5 * ref.abs().max() + 1e-7
    out16 = kernels.quant_embedding(cw, packed, q["norms"].cuda(), q["ct_scaled"].cuda(), ids.cuda(), hidden)
    assert out16.dtype == torch.float16 and (out16.float().cpu() - ref).abs().max() <= 2e-3 * ref.abs().max()
