#!/usr/bin/env python
"""Benchmark of the quantized-linear decode path: one "step" is one pass of the four
projection launches of a 9B-class decoder layer (fused q/k/v 6144x4096 Q5, o 4096x4096
Q6, fused gate/up 24576x4096 Q3, down 4096x12288 Q4; block 128, fp16 norms) over a
batch of fp16 activations, rotating through a ring of layers larger than L2.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--batch B] [--impl reference]

Prints ONE JSON line.  `value` is algorithmic GB/s of the whole job with everything
resident in HBM; `e2e` goes through linear_method.apply with host buffers; `roofline`
is the dominant kernel (nibble-code GEMV) against the measured HBM copy bandwidth;
`cpu_baseline` is the CPU oracle (the reference's torch math) on a bounded sample.
With N > 1 (torchrun) every rank streams its own ring of layers (independent units, no
collective on the data path): weak scaling.
"""
import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

HIDDEN, INTER, QKV = 4096, 12288, 6144
# (name, out_f, in_f, bits)
PROJ = [("qkv_proj", QKV, HIDDEN, 5), ("o_proj", HIDDEN, HIDDEN, 6),
        ("gate_up_proj", 2 * INTER, HIDDEN, 3), ("down_proj", HIDDEN, INTER, 4)]
NCU_DRAM_BYTES_DOWN_B1 = 26035072  # dram__bytes_read + write of one batch-1 down_proj launch (ncu capture summarised in profiles/)
RING = 8  # layers in the ring: 8 x 120.5 MB = 964 MB >> 126 MB of L2


def alg_bytes(out_f, in_f, bits, batch):
    """Algorithmic bytes of one launch: codes + fp16 norms + activations in/out + table."""
    code = out_f * in_f // 2 if bits <= 4 else out_f * in_f
    return code + out_f * (in_f // 128) * 2 + batch * in_f * 2 + batch * out_f * 2 + (1 << bits) * 4


def step_bytes(batch):
    return sum(alg_bytes(n, k, b, batch) for _, n, k, b in PROJ)


def lloyd_max_boundaries(ct):
    return (ct[1:] + ct[:-1]) / 2


def make_layer(dev, seed):
    """Synthetic quantized layer: codes are the Lloyd-Max cells of N(0,1) draws (the
    distribution the quantizer produces for Gaussian weights), norms ~ 0.02*sqrt(128)."""
    from polarengine_vllm_b200.utils import get_centroids, get_ct_scaled
    from polarengine_vllm_b200.packing import pack_codes_half_block
    from polarengine_vllm_b200.kernels import retile
    g = torch.Generator(device=dev).manual_seed(seed)
    out = {}
    for name, n, k, bits in PROJ:
        ct = get_centroids(bits).to(dev)
        r = torch.randn(n, k, device=dev, generator=g)
        codes = torch.bucketize(r, lloyd_max_boundaries(ct)).to(torch.int8)
        del r
        norms = (0.02 * math.sqrt(128) * (1 + 0.05 * torch.randn(n, k // 128, device=dev, generator=g))).half()
        w = pack_codes_half_block(codes) if bits <= 4 else codes
        # the decode kernel streams the tiled copy (what process_weights_after_loading builds)
        out[name] = (w, bits <= 4, norms, get_ct_scaled(bits).to(dev), n, k, retile(w, bits <= 4, norms))
    return out


class ClockSampler(threading.Thread):
    def __init__(self, index):
        super().__init__(daemon=True)
        self.index, self.rows, self.stop_flag = index, [], False

    def run(self):
        q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
        while not self.stop_flag:
            try:
                o = subprocess.run(["nvidia-smi", "-i", str(self.index), f"--query-gpu={q}", "--format=csv,noheader,nounits"],
                                   capture_output=True, text=True, timeout=5).stdout.strip()
                if o:
                    self.rows.append([c.strip() for c in o.split(",")])
            except Exception:
                pass
            time.sleep(0.02)

    def summary(self):
        sm = sorted(int(r[0]) for r in self.rows if r and r[0].isdigit())
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({names[i] for r in self.rows if len(r) >= 6 for i in range(4) if r[2 + i].lower().startswith("active")})
        mx = max((int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()), default=None)
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "reasons": reasons, "samples": len(sm)}


def cpu_baseline(batch, budget_s=12.0):
    """The reference's CPU-runnable form of the path (rotate, gather centroids, scale by
    norms, contract) timed on the host cores for whole layer passes until ~budget_s."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import polar_oracle as oracle
    g = torch.Generator().manual_seed(0)
    layers = []
    for name, n, k, bits in PROJ:
        codes = torch.randint(0, 1 << bits, (n, k), generator=g, dtype=torch.int16).to(torch.int8)
        norms = (torch.rand(n, k // 128, generator=g) * 0.02 + 0.2).half()
        layers.append((codes, norms, oracle.ct_scaled(bits), k))
    x = {k: torch.randn(batch, k, generator=g).half() for k in (HIDDEN, INTER)}
    def one_pass():
        for codes, norms, cts, k in layers:
            oracle.linear_hadamard_domain(x[k], codes, norms, cts)
    one_pass()
    t0 = time.perf_counter()
    n = 0
    while True:
        one_pass()
        n += 1
        if time.perf_counter() - t0 > budget_s or n >= 50:
            break
    dt = time.perf_counter() - t0
    return {"value": step_bytes(batch) * n / dt / 1e9, "unit": "GB/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"{n} decoder-layer passes (4 projections, batch {batch}) of the CPU oracle in {dt:.1f} s"}, dt / n


def prefill_sweep(a, dev, rank, world):
    """BASELINE configs[2]: M tokens x K into N, bf16 activations, Q4 nibble codes.  One step = the three layer
    shapes once; value = TFLOP/s of 2*M*N*K (rotation and activation preparation included in the time)."""
    from polarengine_vllm_b200 import kernels
    shapes = [(4096, 4096), (12288, 4096), (4096, 12288)]
    m = a.m
    g = torch.Generator(device=dev).manual_seed(3)
    data = []
    for n, k in shapes:
        w = torch.randint(0, 256, (n, k // 2), dtype=torch.uint8, device=dev, generator=g)
        norms = (0.2 + 0.02 * torch.rand(n, k // 128, device=dev, generator=g)).half()
        from polarengine_vllm_b200.utils import get_ct_scaled
        x = torch.randn(m, k, device=dev, generator=g).bfloat16()
        data.append((w, norms, get_ct_scaled(4).to(dev), x, n, k))
    def step():
        for w, norms, ct, x, n, k in data:
            kernels.quant_matmul(w, True, norms, ct, x, False, n, k, k, torch.float16)
    if a.probe:
        step(); torch.cuda.synchronize()
        print(json.dumps({"probe": "prefill", "m": m}))
        return
    steps = max(3, min(a.steps, 50))
    for _ in range(3):
        step()
    torch.cuda.synchronize()
    per = []
    for w, norms, ct, x, n, k in data:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            kernels.quant_matmul(w, True, norms, ct, x, False, n, k, k, torch.float16)
        e1.record(); torch.cuda.synchronize()
        per.append(e0.elapsed_time(e1) / 1e3 / steps)
    flops = [2.0 * m * n * k for n, k in shapes]
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        pass
    peak = float(peaks.get("bf16_tflops", 1590.0))
    best = max(range(3), key=lambda i: flops[i] / per[i])
    if rank == 0:
        print(json.dumps({
            "metric": "prefill quantized GEMM TFLOP/s", "unit": "TFLOP/s", "value": sum(flops) / sum(per) / 1e12,
            "n_gpus": a.gpus, "steps": steps, "warmup": 3, "ms_per_step": sum(per) * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"prefill_gemm (BASELINE configs[2]) M={m}, Q4, (N,K) in {shapes}",
                       "l2_defeat": "operands larger than L2 at M=4096 (x + y + codes > 126 MB for two of three shapes)"},
            "per_shape_tflops": {f"{n}x{k}": flops[i] / per[i] / 1e12 for i, (n, k) in enumerate(shapes)},
            "roofline": {"bound": "tensor", "kernel": "gemm_kernel<packed> N=%d K=%d" % shapes[best],
                         "achieved": flops[best] / per[best] / 1e12, "peak": peak,
                         "peak_source": "measured burst (MEASURED_PEAKS.json)" if peaks else "fallback",
                         "unit": "TFLOP/s", "frac": flops[best] / per[best] / 1e12 / peak, "traffic": None},
            "gpu_launches": 2 * 3 * steps}))


def model_decode(a, dev, rank, world):
    """BASELINE configs[3]: prompt of random ids, then greedy decode; every projection, the embedding and the LM
    head are quantized; tensor parallel over the ranks (column q/k/v/gate/up, row o/down + NCCL all-reduce).
    The decode step is captured in a CUDA graph.  value = batch * new_tokens / time (tok/s), strong scaling."""
    import torch.distributed as dist
    from polarengine_vllm_b200.decoder import DecoderConfig, QuantDecoder
    cfg = DecoderConfig(n_layers=a.layers)
    b = a.batch
    fused = world > 1 and not a.nccl_allreduce
    fused_note = "nccl all-reduce + add/norm kernels"
    try:
        model = QuantDecoder(cfg, dev, rank, world, None, max_len=a.prompt + a.new_tokens + 8, batch=b, fused_allreduce=fused)
        if fused:
            fused_note = "all-reduce + residual add + RMSNorm in one kernel over peer memory (decode steps); nccl in prefill"
    except Exception as exc:  # peer mappings unavailable: the NCCL path still measures the model
        if not fused:
            raise
        fused_note = f"nccl all-reduce (peer exchange unavailable: {type(exc).__name__})"
        model = QuantDecoder(cfg, dev, rank, world, None, max_len=a.prompt + a.new_tokens + 8, batch=b)
    g = torch.Generator(device=dev).manual_seed(17)
    prompt = torch.randint(0, cfg.vocab, (b, a.prompt), device=dev, generator=g)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    nxt = model.forward(prompt, 0)
    torch.cuda.synchronize()
    prefill_s = time.perf_counter() - t0
    ids_buf = nxt.view(b, 1).clone()
    pos = torch.tensor(a.prompt, device=dev, dtype=torch.int64)
    stream = torch.cuda.Stream(dev)
    def step():
        out = model.forward(ids_buf, pos)
        ids_buf.copy_(out.view(b, 1))
        pos.add_(1)
    sampler = ClockSampler(int(os.environ.get("LOCAL_RANK", "0")))
    sampler.start()  # from the warm-up on: a query takes longer than a short timed region on a full box
    with torch.cuda.stream(stream):
        for _ in range(3):
            step()
        torch.cuda.synchronize()
        graph = None
        if not a.no_graph:
            graph = torch.cuda.CUDAGraph()
            # thread_local: the NCCL watchdog thread may query events while this thread captures
            with torch.cuda.graph(graph, stream=stream, capture_error_mode="thread_local"):
                step()
        torch.cuda.synchronize()
        pos.fill_(a.prompt)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(a.new_tokens):
            if graph is not None:
                graph.replay()
            else:
                step()
        e1.record(stream)
        torch.cuda.synchronize()
        sampler.stop_flag = True
        if world > 1:
            dist.barrier()
    el = e0.elapsed_time(e1) / 1e3
    if world > 1:
        t = torch.tensor([el], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        el = float(t)
    if rank == 0:
        peaks = {}
        try:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        except Exception:
            pass
        wb = model.weight_bytes_per_step()
        print(json.dumps({
            "metric": "9B-class decode tok/s", "unit": "tok/s", "value": b * a.new_tokens / el, "n_gpus": a.gpus,
            "steps": a.new_tokens, "warmup": 3, "ms_per_step": el / a.new_tokens * 1e3, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": f"model_decode (BASELINE configs[3]): {a.layers} layers, hidden 4096, vocab 151936, "
                                   f"prompt {a.prompt}, {a.new_tokens} new tokens", "batch": b,
                       "parallelism": f"tp{world}", "l2_defeat": "weights per rank larger than L2",
                       "launch": "eager" if a.no_graph else "cuda graph", "row_parallel_epilogue": fused_note},
            "exchange_timed_out": bool(model.xchg.timed_out()) if model.xchg is not None else None,
            "prefill_s": prefill_s, "weight_bytes_per_step_per_rank": wb,
            "hbm_frac_of_measured": wb / (el / a.new_tokens) / 1e9 / float(peaks.get("hbm_gbs", 6650.0)),
            "clocks": sampler.summary(), "gpu_launches": a.new_tokens * (8 * a.layers + 3)}))
    finish(world)


def moe_layer(a, dev, rank, world):
    """BASELINE configs[4]: 128 experts, top-8 softmax routing from a seeded fp16 gate (2688 -> 128), expert
    intermediate 1856, gate/up Q3 and down Q4 codes; expert parallel over the ranks (tokens replicated, every rank
    runs its local experts, all-reduce of the layer output).  value = tokens / time."""
    import torch.distributed as dist
    from polarengine_vllm_b200.moe_method import PolarQuantMoEMethod, route_softmax_topk
    from polarengine_vllm_b200.parallel import expert_placement
    from polarengine_vllm_b200.utils import get_ct_scaled
    E, H, I, K = 128, 2688, 1856, 8
    T = a.tokens
    e_local = E // world
    method = PolarQuantMoEMethod(3, 4)
    if a.moe_grouped_rows is not None:
        method.GROUPED_MAX_ROWS_PER_EXPERT = a.moe_grouped_rows
    layer = torch.nn.Module()
    g = torch.Generator(device=dev).manual_seed(4242 + rank)
    hp, ip = 2688, 1920
    layer.w13_codes = torch.randint(0, 256, (e_local, 2 * I, hp // 2), dtype=torch.uint8, device=dev, generator=g) & 0x77
    layer.w13_norms = (0.02 * math.sqrt(128) * (1 + 0.05 * torch.randn(e_local, 2 * I, hp // 128, device=dev, generator=g))).half()
    layer.w2_codes = torch.randint(0, 256, (e_local, H, ip // 2), dtype=torch.uint8, device=dev, generator=g)
    layer.w2_norms = (0.02 * math.sqrt(128) * (1 + 0.05 * torch.randn(e_local, H, ip // 128, device=dev, generator=g))).half()
    layer.w13_ct_scaled, layer.w2_ct_scaled = get_ct_scaled(3).to(dev), get_ct_scaled(4).to(dev)
    layer.moe_hidden, layer.moe_inter, layer.moe_hidden_padded, layer.moe_inter_padded = H, I, hp, ip
    gs = torch.Generator(device=dev).manual_seed(7)  # same gate and tokens on every rank
    gate = (0.02 * torch.randn(E, H, device=dev, generator=gs)).half()
    x = torch.randn(T, H, device=dev, generator=gs).half()
    emap = expert_placement(E, rank, world).to(dev) if world > 1 else None

    def step():
        w, ids = route_softmax_topk(x @ gate.T, K, True)
        y = method.moe_forward(layer, x, w, ids, emap)
        if world > 1:
            dist.all_reduce(y)
        return y

    if a.probe:  # one layer pass and out: the case captured under ncu
        step(); step()
        torch.cuda.synchronize()
        print(json.dumps({"probe": "moe", "tokens": T}))
        return
    stream = torch.cuda.Stream(dev)
    local_pairs = method.expected_local_pairs(T * K, e_local, emap)
    grouped = local_pairs <= method.GROUPED_MAX_ROWS_PER_EXPERT * e_local
    steps = a.steps if a.steps != 4000 else (200 if grouped else 10)
    sampler = ClockSampler(int(os.environ.get("LOCAL_RANK", "0")))
    sampler.start()  # from the warm-up on: a query takes longer than a short timed region on a full box
    with torch.cuda.stream(stream):
        for _ in range(3):
            step()
        torch.cuda.synchronize()
        graph = None
        if grouped:  # the grouped path reads nothing back to the host: one graph per step
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream, capture_error_mode="thread_local"):
                step()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(steps):
            graph.replay() if graph is not None else step()
        e1.record(stream)
        torch.cuda.synchronize()
        sampler.stop_flag = True
    el = e0.elapsed_time(e1) / 1e3
    if world > 1:
        t = torch.tensor([el], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        el = float(t)
    # algorithmic bytes: codes + norms of the experts that received a token (all ranks), activations negligible
    _, ids = route_softmax_topk(x @ gate.T, K, True)
    active = int(torch.unique(ids).numel())
    per_expert = 2 * I * (hp // 2 + hp // 128 * 2) + H * (ip // 2 + ip // 128 * 2)
    flops = 2.0 * T * K * (2 * I * H + H * I)
    if rank == 0:
        peaks = {}
        try:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        except Exception:
            pass
        ms = el / steps * 1e3
        print(json.dumps({
            "metric": "MoE layer tokens/s", "unit": "tok/s", "value": T * steps / el, "n_gpus": a.gpus, "steps": steps,
            "warmup": 3, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f16", "data": "synthetic",
            "config": {"workload": f"moe_layer (BASELINE configs[4]): 128 experts top-8, hidden 2688, intermediate 1856, "
                                   f"gate/up Q3 down Q4, {T} tokens", "parallelism": f"ep{world}",
                       "path": ("two grouped tcgen05 launches (pe_gemm_grouped), CUDA graph" if local_pairs >= method.TENSOR_CORE_MIN_ROWS_PER_EXPERT * e_local
                                else "two grouped decode-size launches (pe_gemv_grouped), CUDA graph") if grouped
                               else "per-expert tensor-core matmuls, eager",
                       "l2_defeat": "expert weights 970 MB >> L2"},
            "active_experts": active, "expert_bytes_per_step": active * per_expert,
            "weight_gbs": active * per_expert / (ms / 1e3) / 1e9,
            "hbm_frac_of_measured": active * per_expert / (ms / 1e3) / 1e9 / float(peaks.get("hbm_gbs", 6650.0)) / world,
            "tflops": flops / (ms / 1e3) / 1e12, "clocks": sampler.summary(),
            "gpu_launches": steps * (5 if grouped else 2 * min(active, e_local))}))
    finish(world)


def finish(world):
    """Leave a multi-rank run.  Tearing down the NCCL communicator while captured graphs that contain its kernels are
    alive can block forever; the ranks synchronise and exit without running the destructors instead."""
    if world > 1:
        import torch.distributed as dist
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=4000)
    ap.add_argument("--warmup", type=int, default=40)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--workload", default="decode", choices=["decode", "prefill", "model", "moe"],
                    help="decode: decoder-layer GEMV pass (default, the headline); prefill: Q4 GEMM sweep of BASELINE "
                         "configs[2]; model: 36-layer 9B-class decode tok/s, tensor parallel over --gpus (configs[3])")
    ap.add_argument("--layers", type=int, default=36, help="decoder layers for --workload model")
    ap.add_argument("--prompt", type=int, default=512)
    ap.add_argument("--new-tokens", type=int, default=128)
    ap.add_argument("--no-graph", action="store_true", help="model workload: launch decode steps eagerly")
    ap.add_argument("--nccl-allreduce", action="store_true", help="model workload: NCCL all-reduce instead of the fused peer-memory epilogue")
    ap.add_argument("--m", type=int, default=4096, help="tokens for --workload prefill")
    ap.add_argument("--tokens", type=int, default=64, help="tokens for --workload moe (1 / 64 / 2048)")
    ap.add_argument("--moe-grouped-rows", type=int, default=None,
                    help="moe workload: average rows per expert up to which the grouped launches are used (default: the method's)")
    ap.add_argument("--probe", default=None, metavar="PROJ",
                    help="profiling aid: launch PROJ (e.g. down_proj) once per ring layer and exit, no timing")
    a = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    config = {"workload": "decoder_layer_gemv (BASELINE configs[1]): q/k/v Q5 fused, o Q6, gate/up Q3 fused, down Q4; "
                          "hidden 4096, intermediate 12288", "batch": a.batch, "ring_layers": RING,
              "l2_defeat": "inputs larger than L2 (ring of 8 layers = 964 MB of codes)",
              "parallelism": f"replicas x{a.gpus}: each rank streams its own layers, no collective"}
    base = {"metric": "quantized GEMV HBM GB/s", "unit": "GB/s", "n_gpus": a.gpus, "steps": a.steps, "warmup": a.warmup,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": config}

    if a.impl == "reference":
        if rank != 0:
            return
        # The reference has no CPU implementation of apply() (its Triton wrappers need a GPU);
        # its CPU-runnable path is the torch math its kernels are tested against = the oracle.
        cb, per_step = cpu_baseline(a.batch, budget_s=max(5.0, min(60.0, 0.3 * (a.steps + a.warmup))))
        line = dict(base, impl="reference", value=cb["value"], ms_per_step=per_step * 1e3, cpu_baseline=cb, gpu_launches=0,
                    e2e={"value": cb["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0})
        print(json.dumps(line))
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (the product path has no CPU fallback)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    from polarengine_vllm_b200 import kernels
    from polarengine_vllm_b200.linear_method import PolarQuantLinearMethod
    if a.workload == "prefill":
        prefill_sweep(a, dev, rank, world)
        return finish(world)
    if a.workload == "moe":
        return moe_layer(a, dev, rank, world)
    if a.workload == "model":
        return model_decode(a, dev, rank, world)

    steps = max(RING, a.steps // RING * RING)
    warm = max(3, a.warmup)
    layers = [make_layer(dev, 1000 + 16 * i + 97 * rank) for i in range(RING)]
    g = torch.Generator(device=dev).manual_seed(7)
    xh = torch.randn(a.batch, HIDDEN, device=dev, generator=g).half()
    xi = torch.randn(a.batch, INTER, device=dev, generator=g).half()
    outs = {name: torch.empty(a.batch, n, dtype=torch.float16, device=dev) for name, n, _, _ in PROJ}

    def launch(layer, name):
        w, packed, norms, ct, n, k, tiles = layer[name]
        return kernels.quant_matmul(w, packed, norms, ct, xh if k == HIDDEN else xi, False, n, k, k, torch.float16,
                                    tiles=tiles)

    def ring_pass(names):
        for layer in layers:
            for name in names:
                launch(layer, name)

    all_names = [p[0] for p in PROJ]
    if a.probe:
        ring_pass([a.probe])
        torch.cuda.synchronize()
        print(json.dumps({"probe": a.probe, "launches": RING, "batch": a.batch}))
        return
    stream = torch.cuda.Stream(dev)

    def timed_graph(names, reps, warm_reps):
        """Capture one ring pass (RING steps) as a CUDA graph and time `reps` replays."""
        with torch.cuda.stream(stream):
            ring_pass(names)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                ring_pass(names)
            for _ in range(warm_reps):
                graph.replay()
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
                torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(reps):
                graph.replay()
            e1.record(stream)
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
            return e0.elapsed_time(e1) / 1e3

    sampler = ClockSampler(local)
    sampler.start()
    elapsed = timed_graph(all_names, steps // RING, max(1, math.ceil(warm / RING)))
    # dominant kernel alone: the nibble-code GEMV on the 4096x12288 Q4 layer (down_proj)
    dom = ["down_proj"]
    dom_elapsed = timed_graph(dom, steps // RING, 1)
    sampler.stop_flag = True
    if world > 1:
        t = torch.tensor([elapsed], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed = float(t)
    value = step_bytes(a.batch) * steps * world / elapsed / 1e9

    # ---- end to end through the plugin surface with host buffers
    method = {}
    mods = {}
    for name, n, k, bits in PROJ:
        m = PolarQuantLinearMethod(128, bits)
        mod = torch.nn.Module()
        w, packed, norms, ct, _, _, tiles = layers[0][name]
        mod.in_f, mod.out_f, mod.in_f_padded, mod.n_blocks, mod.bits, mod.block_size = k, n, k, k // 128, bits, 128
        mod.packed, mod.norms, mod.ct_scaled = packed, norms, ct
        if packed:
            mod.codes_packed, mod.in_f_half = w, k // 2
        else:
            mod.codes = w
        method[name], mods[name] = m, mod
    hx = {k: torch.randn(a.batch, k).half().pin_memory() for k in (HIDDEN, INTER)}
    hy = torch.empty(a.batch, HIDDEN, dtype=torch.float16).pin_memory()
    e2e_steps = min(steps, 1000)

    def e2e_body(i, dx):
        layer = layers[i % RING]
        y = None
        for name, n, k, bits in PROJ:
            mod = mods[name]
            w, packed, norms, ct, _, _, tiles = layer[name]
            mod.norms = norms
            mod.codes_tiled = tiles
            if packed:
                mod.codes_packed = w
            else:
                mod.codes = w
            y = method[name].apply(mod, dx[k])
        return y

    def e2e_step_eager(i):
        dx = {k: v.to(dev, non_blocking=True) for k, v in hx.items()}
        hy.copy_(e2e_body(i, dx), non_blocking=True)
        torch.cuda.current_stream().synchronize()

    # The way a serving engine drives decode: the step (host->device copies of the pinned
    # inputs, the four apply() calls, device->host copy of the result) is captured once per
    # ring layer in a CUDA graph and replayed; every replay is followed by a host wait.
    dx_static = {k: torch.empty(a.batch, k, dtype=torch.float16, device=dev) for k in hx}
    graphs = []
    with torch.cuda.stream(stream):
        for i in range(RING):
            for k in hx:
                dx_static[k].copy_(hx[k], non_blocking=True)
            hy.copy_(e2e_body(i, dx_static), non_blocking=True)  # warm the allocator
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream, capture_error_mode="thread_local"):
                for k in hx:
                    dx_static[k].copy_(hx[k], non_blocking=True)
                hy.copy_(e2e_body(i, dx_static), non_blocking=True)
            graphs.append(g)

    def e2e_step_graph(i):
        graphs[i % RING].replay()
        stream.synchronize()

    def time_e2e(step_fn):
        with torch.cuda.stream(stream):
            for i in range(2 * RING):
                step_fn(i)
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
            t0 = time.perf_counter()
            for i in range(e2e_steps):
                step_fn(i)
            torch.cuda.synchronize()
            dt = time.perf_counter() - t0
        if world > 1:
            t = torch.tensor([dt], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dt = float(t)
        return step_bytes(a.batch) * e2e_steps * world / dt / 1e9

    e2e_graph = time_e2e(e2e_step_graph)
    e2e_eager = time_e2e(e2e_step_eager)
    e2e = {"value": e2e_graph, "unit": "GB/s",
           "h2d_bytes_per_step": a.batch * (HIDDEN + INTER) * 2, "d2h_bytes_per_step": a.batch * HIDDEN * 2,
           "steps": e2e_steps, "eager_value": e2e_eager,
           "api": "PolarQuantLinearMethod.apply x4 per step with pinned host in/out copies, the step captured in a "
                  "CUDA graph and waited on by the host after every replay; eager_value = same step without the graph"}

    if rank == 0:
        peaks = {}
        try:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        except Exception:
            pass
        peak = float(peaks.get("hbm_gbs", 6650.0))
        dom_launches = steps
        dom_bytes = sum(alg_bytes(n, k, b, a.batch) for nm, n, k, b in PROJ if nm in dom)
        achieved = dom_bytes / (dom_elapsed / dom_launches) / 1e9
        roofline = {"bound": "hbm", "kernel": "gemv_cols_kernel<packed, table, 3 chunks per warp> on down_proj 4096x12288 Q4", "achieved": achieved,
                    "peak": peak, "peak_source": "measured (MEASURED_PEAKS.json)" if peaks else "fallback",
                    "unit": "GB/s", "frac": achieved / peak, "avg_launch_us": dom_elapsed / dom_launches * 1e6,
                    "alg_bytes_per_launch": dom_bytes,
                    # dram__bytes_read.sum + dram__bytes_write.sum of one batch-1 launch (profiles/)
                    "traffic": NCU_DRAM_BYTES_DOWN_B1 if a.batch == 1 else None}
        line = dict(base, value=value, ms_per_step=elapsed / steps * 1e3, steps=steps, e2e=e2e, gpu_launches=4 * steps,
                    roofline=roofline, clocks=sampler.summary(),
                    frac_of_measured_hbm=value / world / peak)
        if not a.no_cpu_baseline:
            line["cpu_baseline"], _ = cpu_baseline(a.batch)
        print(json.dumps(line))
    finish(world)


if __name__ == "__main__":
    main()
