"""The CPU oracle against vectors produced by the reference itself (tests/golden/)
and against the known-answer values the reference's own tests hold."""
import math

import numpy as np
import pytest
import torch

import polar_oracle as oracle


@pytest.mark.parametrize("bits", range(2, 9))
def test_centroids_bit_exact(golden, bits):
    assert np.array_equal(oracle.centroids(bits), golden[f"centroids_{bits}"])


def test_centroid_range_error():
    for bad in (1, 9):
        with pytest.raises(ValueError):
            oracle.centroids(bad)


def test_hadamard_and_rotation(golden):
    assert np.array_equal(oracle.hadamard(128).numpy(), golden["hadamard_128"])
    x = torch.from_numpy(golden["fwht_in"])
    assert np.array_equal(oracle.fwht(x).numpy(), golden["fwht_out"])
    bf = oracle.fwht_butterfly(x.reshape(-1, 128)).reshape(x.shape).numpy()
    assert np.abs(bf - golden["fwht_butterfly_out"]).max() < 1e-5
    # known answers of the reference's tests/test_fwht.py:57-70, 191-195
    h2 = oracle.hadamard(2)
    assert torch.allclose(h2, torch.tensor([[1.0, 1.0], [1.0, -1.0]]) / math.sqrt(2))
    h = oracle.hadamard(128)
    assert torch.allclose(h @ h, torch.eye(128), atol=1e-5) and torch.equal(h, h.T)


@pytest.mark.parametrize("bits", [2, 3, 4, 5, 6, 8])
def test_quantizer_bit_exact(golden, bits):
    r = oracle.quantize_tensor(torch.from_numpy(golden["quant_w"]), bits)
    assert np.array_equal(r["codes"].numpy(), golden[f"quant_codes_{bits}"])
    assert np.array_equal(r["norms"].numpy(), golden[f"quant_norms_{bits}"])
    assert np.array_equal(r["ct_scaled"].numpy(), golden[f"quant_ct_scaled_{bits}"])


def test_quantizer_zero_row(golden):
    w = torch.from_numpy(golden["quant_w"]).clone()
    w[3] = 0
    r = oracle.quantize_tensor(w, 4)
    assert np.array_equal(r["codes"].numpy(), golden["quant_zero_row_codes_4"])
    assert np.array_equal(r["norms"].numpy(), golden["quant_zero_row_norms_4"])


def test_layouts(golden):
    assert np.array_equal(oracle.pack_nibble(golden["nib_codes"]), golden["nib_packed"])
    assert np.array_equal(oracle.unpack_nibble(golden["nib_packed"]), golden["nib_codes"])
    assert np.array_equal(oracle.pack_q5(golden["q5_codes"]), golden["q5_packed"])
    assert np.array_equal(oracle.unpack_q5(golden["q5_packed"]), golden["q5_codes"])
    assert np.array_equal(oracle.pack_q5_hlwq(golden["q5_codes"]), golden["q5_hlwq_packed"])
    assert np.array_equal(oracle.unpack_q5_hlwq(golden["q5_hlwq_packed"]), golden["q5_codes"])
    # known-answer bytes of the reference's tests/test_packing.py:78-108
    c = np.zeros((2, 256), np.int8).reshape(2, 2, 128)
    c[:, :, :64], c[:, :, 64:] = 3, 12
    assert (oracle.pack_nibble(c.reshape(2, 256)) == 0xC3).all()
    c[:, :, :64], c[:, :, 64:] = 15, 0
    assert (oracle.pack_nibble(c.reshape(2, 256)) == 0x0F).all()
    c[:, :, :64], c[:, :, 64:] = 0, 15
    assert (oracle.pack_nibble(c.reshape(2, 256)) == 0xF0).all()


@pytest.mark.parametrize("bits", [4, 5])
def test_forward_forms(golden, bits):
    codes = torch.from_numpy(golden[f"quant_codes_{bits}"])
    norms = torch.from_numpy(golden[f"quant_norms_{bits}"])
    cts = torch.from_numpy(golden[f"quant_ct_scaled_{bits}"])
    x = torch.from_numpy(golden["fwd_x"])
    yh = oracle.linear_hadamard_domain(x, codes, norms, cts)
    assert np.allclose(yh.numpy(), golden[f"fwd_hadamard_{bits}"], rtol=0, atol=1e-6)
    yd = oracle.linear_dequant(x, codes, norms, cts, in_f=300)
    assert float((yd - yh).abs().max() / yh.abs().max()) < 1e-5
    # the reference's dequantiser rounds to bf16; ours is the same weight before rounding
    w = oracle.dequant_fp32(codes, norms, cts)
    assert np.array_equal(w.bfloat16().float().numpy(), golden[f"fwd_dequant_bf16_{bits}"]) or \
        np.abs(w.numpy() - golden[f"fwd_dequant_bf16_{bits}"]).max() <= np.abs(w.numpy()).max() * 2 ** -7
    y16 = oracle.apply_forward(x, codes, norms, cts, 300, bias=torch.ones(70))
    assert y16.dtype == torch.float16 and y16.shape == (3, 70)
