"""Parity of the tcgen05 prefill kernel (pe_gemm, through the C ABI) with the CPU oracle.
bf16 operands, fp32 accumulation: max |y - ref| / max |ref| <= 1e-2 against the fp32
dequant reference (the north-star tolerance), cosine > 0.9999."""
import pytest
import torch

import polar_oracle as oracle
from helpers import max_rel, rand_layer, rand_x, ref_metrics

pytestmark = pytest.mark.gpu
TOL = 1e-2


def run_gemm(codes, norms, cts, x, bits, rotated=False, out_dtype=torch.float16, bias=None, in_f=None):
    from polarengine_vllm_b200 import _native as nv, gemm, packing
    dev = torch.device("cuda")
    nv.ensure_init(dev)
    n, kp = codes.shape
    packed = bits <= 4
    cd = codes.to(dev)
    w = packing.pack_codes_half_block(cd) if packed else cd
    xd = x.to(dev).contiguous()
    y = torch.full((x.shape[0], n), float("nan"), dtype=out_dtype, device=dev)
    gemm.quant_gemm(w, packed, norms.to(dev), cts.to(dev), xd, rotated, n, in_f if in_f is not None else kp, kp, y,
                    bias.to(dev).half() if bias is not None else None, check_status=True)
    return y


@pytest.mark.parametrize("bits", [3, 4, 5, 6])
@pytest.mark.parametrize("m,n,k", [(64, 256, 256), (256, 512, 1024), (128, 256, 128), (300, 1856, 2688),
                                   (100, 2688, 1920), (17, 130, 384), (1024, 4096, 4096),
                                   (64, 40000, 256)])  # the last: more 256-row tiles than SMs, several tiles per CTA
def test_gemm_matches_oracle(m, n, k, bits):
    codes, norms, cts = rand_layer(n, k, bits, seed=m + n + bits)
    x = rand_x(m, k, seed=3, dtype=torch.bfloat16)
    ref = oracle.linear_dequant(x, codes, norms, cts)
    y = run_gemm(codes, norms, cts, x, bits)
    assert y.shape == (m, n) and torch.isfinite(y.float()).all()
    assert max_rel(y, ref) <= TOL
    cos, _ = ref_metrics(y, ref)
    assert cos > 0.9999


@pytest.mark.parametrize("bits,n,k", [(4, 4096, 4096), (4, 12288, 4096), (4, 4096, 12288), (5, 4096, 4096), (6, 4096, 4096),
                                      (3, 12288, 4096)])
def test_gemm_prefill_sweep_shapes_m4096(bits, n, k):
    """The prefill sweep's largest case: 4096 bf16 tokens into the decoder-layer shapes (the reference's own
    self-test list is polar_gemm.py:541-615).  The kernel runs all 4096 tokens; the CPU oracle is evaluated
    on every 16th token (all output columns), which covers every token tile and every weight tile."""
    m = 4096
    codes, norms, cts = rand_layer(n, k, bits, seed=n + k + bits)
    x = rand_x(m, k, seed=12, dtype=torch.bfloat16)
    y = run_gemm(codes, norms, cts, x, bits)
    assert y.shape == (m, n) and torch.isfinite(y.float()).all()
    rows = torch.arange(5, m, 16)
    ref = oracle.linear_dequant(x[rows], codes, norms, cts)
    assert max_rel(y[rows.cuda()], ref) <= TOL
    cos, _ = ref_metrics(y[rows.cuda()], ref)
    assert cos > 0.9999
    # the first and the last token tile in full
    edge = torch.cat([torch.arange(0, 64), torch.arange(m - 64, m)])
    assert max_rel(y[edge.cuda()], oracle.linear_dequant(x[edge], codes, norms, cts)) <= TOL


def test_gemm_ragged_in_features_bias_and_dtypes():
    n, k, in_f, bits, m = 512, 1920, 1856, 4, 200
    codes, norms, cts = rand_layer(n, k, bits, seed=9)
    bias = rand_x(1, n, seed=4).reshape(n)
    for xdt in (torch.float16, torch.bfloat16, torch.float32):
        x = rand_x(m, in_f, seed=5, dtype=xdt)
        ref = oracle.linear_dequant(x, codes, norms, cts, in_f=in_f) + bias.float()
        for ydt in (torch.float16, torch.bfloat16, torch.float32):
            y = run_gemm(codes, norms, cts, x, bits, out_dtype=ydt, bias=bias, in_f=in_f)
            assert y.dtype == ydt and max_rel(y, ref) <= TOL


@pytest.mark.parametrize("m,n", [(257, 256), (700, 1000), (513, 2688), (1100, 130)])
def test_gemm_paired_ctas_ragged_edges_bias_and_dtypes(m, n):
    """More than 256 tokens run on pairs of CTAs (512-token tiles, each CTA decoding half of the weight tile)
    with the output leaving through clipped TMA stores: token and weight-row counts off every tile, box and
    vector boundary, padded K, bias, all output types (fp32 output takes the direct-store path)."""
    k, in_f, bits = 1920, 1856, 4
    codes, norms, cts = rand_layer(n, k, bits, seed=m + n)
    bias = rand_x(1, n, seed=4).reshape(n)
    x = rand_x(m, in_f, seed=5, dtype=torch.bfloat16)
    ref = oracle.linear_dequant(x, codes, norms, cts, in_f=in_f) + bias.float()
    for ydt in (torch.float16, torch.bfloat16, torch.float32):
        y = run_gemm(codes, norms, cts, x, bits, out_dtype=ydt, bias=bias, in_f=in_f)
        assert y.dtype == ydt and y.shape == (m, n) and max_rel(y, ref) <= TOL
    y5 = run_gemm(*rand_layer(n, k, 5, seed=n)[:3], x, 5, in_f=in_f)
    c5, n5, t5 = rand_layer(n, k, 5, seed=n)
    assert max_rel(y5, oracle.linear_dequant(x, c5, n5, t5, in_f=in_f)) <= TOL


def test_gemm_few_tiles_with_and_without_room_for_the_k_split():
    """A launch of up to 256 rows on few 256-row tiles splits K over the SMs when the workspace holds the fp32
    partials (pe_gemm_workspace_bytes_splitk) and runs unsplit in a workspace of pe_gemm_workspace_bytes: same
    values either way (only the order of the fp32 sums differs), bias and output type included."""
    from polarengine_vllm_b200 import _native as nv, packing
    dev = torch.device("cuda")
    nv.ensure_init(dev)
    m, n, k, bits = 96, 1024, 4096, 4
    codes, norms, cts = rand_layer(n, k, bits, seed=31)
    bias = rand_x(1, n, seed=2).reshape(n)
    x = rand_x(m, k, seed=8, dtype=torch.bfloat16)
    ref = oracle.linear_dequant(x, codes, norms, cts) + bias.float()
    w = packing.pack_codes_half_block(codes.to(dev))
    nd, ctd, xd, bd = norms.to(dev), cts.to(dev), x.to(dev), bias.to(dev).half()
    l = nv.lib()
    small, large = l.pe_gemm_workspace_bytes(m, k), l.pe_gemm_workspace_bytes_splitk(m, n, k)
    assert large > small
    out = []
    for size in (small, large):
        ws = torch.zeros(size, dtype=torch.uint8, device=dev)
        y = torch.full((m, n), float("nan"), dtype=torch.float16, device=dev)
        nv.check(l.pe_gemm(w.data_ptr(), 1, w.stride(0), nd.data_ptr(), nd.stride(0), ctd.data_ptr(), ctd.numel(), xd.data_ptr(),
                           nv.PE_X_RAW, nv.dtype_code(xd), xd.stride(0), k, y.data_ptr(), nv.dtype_code(y), y.stride(0),
                           bd.data_ptr(), m, n, k, ws.data_ptr(), ws.numel(), nv.stream_ptr(dev)), "pe_gemm")
        torch.cuda.synchronize()
        assert int(ws[:4].view(torch.int32).item()) == 0
        assert max_rel(y, ref) <= TOL
        out.append(y.float())
    assert max_rel(out[0], out[1]) <= 2e-3


def test_gemm_rotated_input_and_reference_signature():
    """polar_gemm / polar_gemm_packed of the reference take fp32 x_transformed
    (polar_gemm.py:312-418) and agree with the decode kernel (reference self-test
    polar_gemm.py:680-718 bounds the GEMM-vs-GEMV difference)."""
    from polarengine_vllm_b200 import kernels
    n, k, bits, m = 1024, 4096, 4, 64
    codes, norms, cts = rand_layer(n, k, bits, seed=21)
    xt = oracle.fwht(rand_x(m, k, seed=6, dtype=torch.float32))
    cd, nd, ctd, xd = codes.cuda(), norms.cuda(), cts.cuda(), xt.cuda()
    pk = kernels.pack_codes_int4(cd)
    y = kernels.polar_gemm_packed(pk, xd, nd, ctd, n, k // 2, k // 128)
    y_unpacked = kernels.polar_gemm(cd, xd, nd, ctd, n, k, k // 128)
    ref = torch.einsum("rnk,mnk->mr", cts[codes.long()].view(n, -1, 128) * norms.float().view(n, -1, 1), xt.view(m, -1, 128))
    assert y.dtype == torch.float32 and y.shape == (m, n)
    assert max_rel(y, ref) <= TOL and max_rel(y_unpacked, ref) <= TOL
    y_gemv = torch.cat([kernels.polar_matmul(None, xd[i], nd, ctd, n, k, k // 128, 128, True, pk, k // 2).reshape(1, n)
                        for i in range(4)])
    assert max_rel(y[:4], y_gemv) <= TOL


def test_apply_prefill_matches_oracle():
    from polarengine_vllm_b200.linear_method import PolarQuantLinearMethod
    bits, n, in_f = 4, 1024, 1856
    g = torch.Generator().manual_seed(2)
    w = torch.randn(n, in_f, generator=g) * 0.02
    q = oracle.quantize_tensor(w, bits)
    m = PolarQuantLinearMethod(128, bits)
    layer = torch.nn.Module()
    m.create_weights(layer, in_f, [n], in_f, n, torch.float16)
    layer.codes.data.copy_(q["codes"]); layer.norms.data.copy_(q["norms"])
    layer = layer.cuda()
    m.process_weights_after_loading(layer)
    x = rand_x(96, in_f, seed=1).reshape(2, 48, in_f)
    y = m.apply(layer, x.cuda())
    ref = oracle.apply_forward(x, q["codes"], q["norms"], q["ct_scaled"], in_f)
    assert y.shape == (2, 48, n) and y.dtype == torch.float16 and max_rel(y, ref) <= TOL
