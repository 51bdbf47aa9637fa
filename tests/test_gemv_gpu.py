"""Parity of the native decode-size matmul (pe_gemv, through the C ABI) with the CPU
oracle on the same seeded inputs.  Tolerance: max |y - ref| / max |ref| <= 1e-2 against
the fp32 dequant reference, plus the reference's own acceptance metrics (cosine >
0.9999, mean relative error < 0.01; tests/test_kernel_correctness.py:128-139)."""
import pytest
import torch

import polar_oracle as oracle
from helpers import max_rel, rand_layer, rand_x, ref_metrics

pytestmark = pytest.mark.gpu
TOL = 1e-2


def run_native(codes, norms, cts, x, bits, rotated, out_dtype=torch.float32, bias=None, in_f=None):
    from polarengine_vllm_b200 import kernels, packing
    dev = "cuda"
    n, kp = codes.shape
    packed = bits <= 4
    cd = codes.to(dev)
    w = packing.pack_codes_half_block(cd) if packed else cd
    return kernels.quant_matmul(w, packed, norms.to(dev), cts.to(dev), x.to(dev), rotated, n,
                                in_f if in_f is not None else kp, kp, out_dtype,
                                bias.to(dev) if bias is not None else None)


SHAPES = [(4096, 4096), (1024, 4096), (12288, 4096), (4096, 12288), (512, 4096), (2048, 8192),
          (16, 128), (48, 256), (130, 384), (1000, 1920), (2688, 1920), (1856, 2688), (257, 2560)]


@pytest.mark.parametrize("bits", [3, 4, 5, 6])
@pytest.mark.parametrize("n,k", SHAPES)
def test_gemv_batch1_rotated_input(n, k, bits):
    codes, norms, cts = rand_layer(n, k, bits, seed=n + k + bits)
    x = rand_x(1, k, seed=7, dtype=torch.float32)
    xt = oracle.fwht(x)
    ref = torch.einsum("rnk,mnk->mr", cts[codes.long() & 0xFF].view(n, -1, 128) * norms.float().view(n, -1, 1),
                       xt.view(1, -1, 128))
    y = run_native(codes, norms, cts, xt, bits, rotated=True)
    assert y.shape == (1, n) and y.dtype == torch.float32
    assert torch.isfinite(y).all()
    assert max_rel(y, ref) <= TOL
    cos, mre = ref_metrics(y, ref)
    assert cos > 0.9999
    if k >= 4096:  # the reference applies its mean-relative-error bound to model-sized K only
        assert mre < 0.01


@pytest.mark.parametrize("batch", [1, 2, 4, 7, 8, 9, 15, 16])
@pytest.mark.parametrize("bits,n,k,in_f", [(3, 12288, 4096, 4096), (4, 4096, 12288, 12288), (5, 6144, 4096, 4096),
                                           (6, 4096, 4096, 4096), (4, 2688, 1920, 1856), (3, 1856, 2688, 2688),
                                           (2, 300, 384, 300), (8, 144, 256, 200)])
def test_gemv_fused_rotation(batch, bits, n, k, in_f):
    """Raw fp16 activations: pad + FWHT happen inside the kernel."""
    codes, norms, cts = rand_layer(n, k, bits, seed=31 * bits + n)
    x = rand_x(batch, in_f, seed=batch)
    ref = oracle.linear_dequant(x, codes, norms, cts, in_f=in_f)
    y = run_native(codes, norms, cts, x, bits, rotated=False, in_f=in_f)
    assert max_rel(y, ref) <= TOL
    cos, mre = ref_metrics(y, ref)
    assert cos > 0.9999


@pytest.mark.parametrize("x_dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("y_dtype", [torch.float16, torch.bfloat16, torch.float32])
def test_gemv_dtypes_and_bias(x_dtype, y_dtype):
    n, k, bits = 1024, 2048, 4
    codes, norms, cts = rand_layer(n, k, bits, seed=5)
    x = rand_x(3, k, seed=9, dtype=x_dtype)
    bias = rand_x(1, n, seed=10).reshape(n)
    ref = oracle.linear_dequant(x, codes, norms, cts) + bias.float()
    y = run_native(codes, norms, cts, x, bits, rotated=False, out_dtype=y_dtype, bias=bias)
    assert y.dtype == y_dtype
    assert max_rel(y, ref) <= TOL


def test_gemv_bitwise_deterministic():
    """Run-to-run reproducibility (the reference asserts atol 1e-6,
    tests/test_kernel_correctness.py:160-186; the native kernel has no float atomics)."""
    n, k, bits = 4096, 12288, 4
    codes, norms, cts = rand_layer(n, k, bits, seed=1)
    x = rand_x(4, k, seed=2)
    a = run_native(codes, norms, cts, x, bits, rotated=False)
    for _ in range(3):
        b = run_native(codes, norms, cts, x, bits, rotated=False)
        assert torch.equal(a, b)


def test_gemv_many_row_tiles_per_cta():
    """A tall layer (vocabulary-sized) makes every CTA walk several activation windows."""
    n, k, bits = 151936, 4096, 6
    g = torch.Generator().manual_seed(3)
    codes = torch.randint(0, 64, (n, k), generator=g, dtype=torch.int16).to(torch.int8)
    norms = (torch.rand(n, k // 128, generator=g) * 0.02 + 0.002).half()
    cts = oracle.ct_scaled(bits)
    x = rand_x(2, k, seed=4)
    xt = oracle.fwht(x.float())
    rows = torch.cat([torch.arange(0, 600), torch.arange(75000, 75600), torch.arange(n - 600, n)])
    ref = torch.einsum("rnk,mnk->mr", cts[codes[rows].long()].view(len(rows), -1, 128) * norms[rows].float().unsqueeze(2),
                       xt.view(2, -1, 128))
    y = run_native(codes, norms, cts, x, bits, rotated=False)
    assert max_rel(y[:, rows.cuda()], ref) <= TOL
    assert torch.isfinite(y).all()


def test_polar_matmul_reference_signature():
    """The reference's dispatcher signature (polar_gemm.py:425-437): 1-D in -> 1-D out,
    packed and unpacked agree (tests/test_kernel_correctness.py:262-302)."""
    from polarengine_vllm_b200 import kernels
    n, k, bits = 512, 4096, 4
    codes, norms, cts = rand_layer(n, k, bits, seed=8)
    xt = oracle.fwht(rand_x(1, k, seed=3, dtype=torch.float32)).reshape(-1)
    cd, nd, ctd, xd = codes.cuda(), norms.cuda(), cts.cuda(), xt.cuda()
    y0 = kernels.polar_matmul(cd, xd, nd.reshape(-1), ctd, n, k, k // 128)
    pk = kernels.pack_codes_int4(cd)
    y1 = kernels.polar_matmul(None, xd, nd, ctd, n, k, k // 128, 128, True, pk, k // 2)
    assert y0.shape == (n,) and y0.dtype == torch.float32
    assert (y0 - y1).abs().max() <= 2e-3 * y0.abs().max()  # batch 1 runs the fp16x2 path: two different code layouts, same values
    y2 = kernels.polar_gemv_packed(pk, xd, nd, ctd, n, k // 2, k // 128)
    assert torch.equal(y1, y2)
    yb = kernels.polar_matmul(cd, xd.reshape(1, -1), nd, ctd, n, k, k // 128)
    assert yb.shape == (1, n)


def test_apply_matches_oracle_forward():
    """linear_method.apply end to end: create_weights -> load -> pack -> apply."""
    from polarengine_vllm_b200.linear_method import PolarQuantLinearMethod
    for bits, n, in_f in [(4, 2688, 1856), (5, 1024, 4096)]:
        g = torch.Generator().manual_seed(bits)
        w = torch.randn(n, in_f, generator=g) * 0.02
        q = oracle.quantize_tensor(w, bits)
        m = PolarQuantLinearMethod(128, bits)
        layer = torch.nn.Module()
        m.create_weights(layer, in_f, [n], in_f, n, torch.float16)
        layer.codes.data.copy_(q["codes"])
        layer.norms.data.copy_(q["norms"])
        layer = layer.cuda()
        m.process_weights_after_loading(layer)
        assert layer.packed == (bits <= 4)
        x = rand_x(6, in_f, seed=1).reshape(2, 3, in_f)
        bias = rand_x(1, n, seed=2).reshape(n)
        y = m.apply(layer, x.cuda(), bias.cuda())
        ref = oracle.apply_forward(x, q["codes"], q["norms"], q["ct_scaled"], in_f, bias)
        assert y.shape == (2, 3, n) and y.dtype == torch.float16
        assert max_rel(y, ref) <= TOL
        # against the un-quantized weight the error is the quantizer's, not the kernel's
        dense = x.float().reshape(-1, in_f) @ w.T + bias.float()
        assert max_rel(y.reshape(-1, n), dense) < 0.25


def _gemv_tiled_direct(tiles, packed, ct, x, n, in_f, k):
    """pe_gemv_tiled through the C ABI for any batch <= 16 (quant_matmul itself keeps one
    and two activation rows on the row-major arrays)."""
    from polarengine_vllm_b200 import _native as nv
    l = nv.lib()
    b = x.shape[0]
    y = torch.empty(b, n, dtype=torch.float32, device=x.device)
    ws = nv.gemv_scratch(x.device, l.pe_gemv_workspace_bytes(b, n, k))
    nv.check(l.pe_gemv_tiled(tiles.data_ptr(), int(packed), ct.data_ptr(), ct.numel(), x.data_ptr(), nv.PE_X_RAW,
                             nv.dtype_code(x), x.stride(0), in_f, y.data_ptr(), nv.PE_F32, y.stride(0), None, b, n, k,
                             ws.data_ptr(), ws.numel(), nv.stream_ptr(x.device)), "pe_gemv_tiled")
    return y


@pytest.mark.parametrize("batch", [1, 2, 3, 8, 16])
@pytest.mark.parametrize("bits,n,k,in_f", [(3, 12288, 4096, 4096), (4, 4096, 12288, 12288), (5, 6144, 4096, 4096),
                                           (6, 1000, 1920, 1856), (4, 130, 384, 300), (8, 144, 256, 200)])
def test_gemv_tiled_layout_matches_row_major(batch, bits, n, k, in_f):
    """The tiled copy of a layer (pe_retile) gives the same bits as the row-major layout
    wherever both go through the tile kernel, and the same values within the packed /
    unpacked tolerance where the row-major call takes a row- or column-owner kernel."""
    from polarengine_vllm_b200 import kernels, packing
    codes, norms, cts = rand_layer(n, k, bits, seed=7 * bits + n)
    x = rand_x(batch, in_f, seed=batch + 1).cuda()
    packed = bits <= 4
    cd = codes.cuda()
    w = packing.pack_codes_half_block(cd) if packed else cd
    nd, ctd = norms.cuda(), cts.cuda()
    tiles = kernels.retile(w, packed, nd)
    y0 = kernels.quant_matmul(w, packed, nd, ctd, x, False, n, in_f, k, torch.float32)
    y1 = _gemv_tiled_direct(tiles, packed, ctd, x, n, in_f, k)
    small = 3 <= batch <= kernels.SMALL_BATCH_MAX and kernels.small_batch_takes(w, packed, nd, n, k)
    if batch > 2 and not small:
        assert torch.equal(y0, y1)
        assert torch.equal(y1, kernels.quant_matmul(w, packed, nd, ctd, x, False, n, in_f, k, torch.float32, tiles=tiles))
    else:  # one or two rows, and 3..8 rows of layers the column-owner kernels take, do not go through the tile kernel
        assert max_rel(y0, y1) <= 2e-3
        if small:  # ... with or without a tiled copy at hand, and with the same bits from run to run
            y2 = kernels.quant_matmul(w, packed, nd, ctd, x, False, n, in_f, k, torch.float32, tiles=tiles)
            assert torch.equal(y0, y2)
    ref = oracle.linear_dequant(x.cpu(), codes, norms, cts, in_f=in_f)
    assert max_rel(y1, ref) <= TOL
    assert max_rel(y0, ref) <= TOL


# Shapes the row-owner kernel takes (whole 512-byte items per weight row, enough items
# per warp): rows that do not divide by the CTA count, rows shared by two and by many
# warps, one item per row, the deepest and the shallower code ring, every table kind.
ROW_SHAPES = [(2, 9500, 1024), (3, 12288, 4096), (3, 24576, 4096), (4, 4096, 12288), (4, 4097, 12288), (4, 2500, 8192),
              (4, 1200, 28672), (5, 6144, 4096), (6, 4096, 4096), (6, 4099, 2048), (8, 9600, 512), (5, 151936, 1024)]


@pytest.mark.parametrize("batch", [1, 2])
@pytest.mark.parametrize("bits,n,k", ROW_SHAPES)
def test_gemv_row_owner_shapes(batch, bits, n, k):
    codes, norms, cts = rand_layer(n, k, bits, seed=11 * bits + n + k)
    in_f = k - 37 if bits in (4, 6) else k  # ragged true width on some
    x = rand_x(batch, in_f, seed=batch + 5)
    bias = rand_x(1, n, seed=3).reshape(n)
    ref = oracle.linear_dequant(x, codes, norms, cts, in_f=in_f) + bias.float()
    y = run_native(codes, norms, cts, x, bits, rotated=False, in_f=in_f, bias=bias)
    y2 = run_native(codes, norms, cts, x, bits, rotated=False, in_f=in_f, bias=bias)
    assert torch.equal(y, y2)  # fixed summation order: bit-identical from run to run
    assert max_rel(y, ref) <= TOL
    cos, mre = ref_metrics(y, ref)
    assert cos > 0.9999
    # already-rotated fp32 input and a bf16 output
    xt = oracle.fwht(torch.nn.functional.pad(x.float(), (0, k - in_f)))
    yb = run_native(codes, norms, cts, xt, bits, rotated=True, out_dtype=torch.bfloat16)
    assert max_rel(yb.float(), ref - bias.float()) <= TOL
