#!/usr/bin/env python
"""Benchmark of the quantized-linear path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--batch B] [--impl reference]
    torchrun ... bench.py --gpus N ...            (one rank per GPU)

Prints ONE JSON line.  The headline is the decode-size matmul: one "step" is one pass of the four
projection launches of a 9B-class decoder layer (fused q/k/v 6144x4096 Q5, o 4096x4096 Q6, fused
gate/up 24576x4096 Q3, down 4096x12288 Q4; block 128, fp16 norms) over a batch of fp16 activations,
rotating through a ring of layers larger than L2.  `value` is algorithmic GB/s of the whole job with
everything resident in HBM; `e2e` goes through linear_method.apply with host buffers; `roofline` is
the nibble-code launch on the 4096x12288 Q4 layer against the measured HBM copy bandwidth;
`cpu_baseline` is the CPU oracle (the reference's torch math) on a bounded sample.  With N > 1 every
rank streams its own ring of layers (independent units, no collective on that path: weak scaling).

The same run then measures the rest of the metric and reports it as extra keys of the line:
`prefill` (4096 bf16 tokens through the tensor-core kernel on the three layer shapes), `model_decode`
(the 36-layer decoder, tensor parallel over the N ranks, batch 1 and 8, with a numeric check of the
sharded model against the un-sharded one) and `moe` (128-expert layer, expert parallel over the N
ranks, 1, 64 and 2048 tokens).  `--workload prefill|model|moe` runs one of them alone with its own line.
"""
import argparse
import json
import math
import os
import re
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
RING = 8  # layers in the ring: 8 x 120.5 MB = 964 MB >> 126 MB of L2
MIN_TIMED_S = 0.25  # a timed region shorter than this is repeated (more replays, so that the clocks are sampled several times)


def load_peaks():
    try:
        return json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        return {}


def measured_traffic(kernel_tag):
    """dram__bytes_read.sum + dram__bytes_write.sum per launch from the kept ncu summary of that kernel
    (a `traffic_bytes_per_launch[<tag>]: N` line under profiles/), or None when no capture is on record."""
    pat = re.compile(r"traffic_bytes_per_launch\[" + re.escape(kernel_tag) + r"\]\s*:\s*(\d+)")
    pdir = os.path.join(ROOT, "profiles")
    try:
        for name in sorted(os.listdir(pdir)):
            if name.endswith((".md", ".txt")):
                m = pat.search(open(os.path.join(pdir, name)).read())
                if m:
                    return int(m.group(1))
    except OSError:
        pass
    return None


def alg_bytes(out_f, in_f, bits, batch):
    """Algorithmic bytes of one launch: codes + fp16 norms + activations in/out + table."""
    code = out_f * in_f // 2 if bits <= 4 else out_f * in_f
    return code + out_f * (in_f // 128) * 2 + batch * in_f * 2 + batch * out_f * 2 + (1 << bits) * 4


def step_bytes(batch):
    return sum(alg_bytes(n, k, b, batch) for _, n, k, b in PROJ)


def make_layer(dev, seed):
    """Synthetic quantized layer: codes are the Lloyd-Max cells of N(0,1) draws (the distribution the
    quantizer produces for Gaussian weights), norms ~ 0.02*sqrt(128)."""
    from polarengine_vllm_b200.utils import get_centroids, get_ct_scaled
    from polarengine_vllm_b200.packing import pack_codes_half_block
    g = torch.Generator(device=dev).manual_seed(seed)
    out = {}
    for name, n, k, bits in PROJ:
        ct = get_centroids(bits).to(dev)
        r = torch.randn(n, k, device=dev, generator=g)
        codes = torch.bucketize(r, (ct[1:] + ct[:-1]) / 2).to(torch.int8)
        del r
        norms = (0.02 * math.sqrt(128) * (1 + 0.05 * torch.randn(n, k // 128, device=dev, generator=g))).half()
        w = pack_codes_half_block(codes) if bits <= 4 else codes
        out[name] = (w, bits <= 4, norms, get_ct_scaled(bits).to(dev), n, k)
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
                if o and not self.stop_flag:
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
    """The reference's CPU-runnable form of the path (rotate, gather centroids, scale by norms, contract)
    timed on the host cores for whole layer passes until ~budget_s.  Every host core is used: launchers such
    as torch.distributed.run export OMP_NUM_THREADS=1, which would time one core."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import polar_oracle as oracle
    cores = os.cpu_count() or 1
    try:
        cores = len(os.sched_getaffinity(0))
    except Exception:
        pass
    torch.set_num_threads(max(1, cores))
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
            "sample": f"{n} decoder-layer passes (4 projections, batch {batch}) of the CPU oracle in {dt:.1f} s on one host"}, dt / n


# ------------------------------------------------------------------------------------------ prefill
def prefill_record(dev, m=4096, steps=20, bits=4):
    """BASELINE configs[2]: M tokens x K into N, bf16 activations, Q4 nibble codes (other widths with ``bits``).  Per shape: TFLOP/s of
    2*M*N*K (rotation and activation preparation included in the time) and the fraction of the measured
    cuBLAS bf16 peaks (burst and sustained)."""
    from polarengine_vllm_b200 import kernels
    from polarengine_vllm_b200.utils import get_ct_scaled
    shapes = [(4096, 4096), (12288, 4096), (4096, 12288)]
    g = torch.Generator(device=dev).manual_seed(3)
    peaks = load_peaks()
    burst, sustained = float(peaks.get("bf16_tflops", 1590.0)), float(peaks.get("bf16_tflops_sustained", 1400.0))
    rec = {"m": m, "dtype": "bf16", "bits": bits, "steps": steps, "peak_burst_tflops": burst, "peak_sustained_tflops": sustained,
           "peak_source": "measured (MEASURED_PEAKS.json)" if peaks else "fallback", "shapes": {}}
    for n, k in shapes:
        if bits <= 4:  # nibble pairs, every code below 2^bits
            lo = torch.randint(0, 1 << bits, (n, k // 2), dtype=torch.uint8, device=dev, generator=g)
            w = lo | (torch.randint(0, 1 << bits, (n, k // 2), dtype=torch.uint8, device=dev, generator=g) << 4)
            del lo
        else:
            w = torch.randint(0, 1 << bits, (n, k), dtype=torch.uint8, device=dev, generator=g).view(torch.int8)
        norms = (0.2 + 0.02 * torch.rand(n, k // 128, device=dev, generator=g)).half()
        ct = get_ct_scaled(bits).to(dev)
        x = torch.randn(m, k, device=dev, generator=g).bfloat16()
        for _ in range(3):
            kernels.quant_matmul(w, bits <= 4, norms, ct, x, False, n, k, k, torch.float16)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            kernels.quant_matmul(w, bits <= 4, norms, ct, x, False, n, k, k, torch.float16)
        e1.record()
        torch.cuda.synchronize()
        per = e0.elapsed_time(e1) / 1e3 / steps
        tf = 2.0 * m * n * k / per / 1e12
        rec["shapes"][f"{n}x{k}"] = {"tflops": tf, "ms": per * 1e3, "frac_of_burst": tf / burst, "frac_of_sustained": tf / sustained}
        del w, norms, x
    rec["gpu_launches"] = 2 * 3 * steps
    return rec


# ------------------------------------------------------------------------------------------ model decode
def decode_run(model, dev, rank, world, batch, prompt_len, new_tokens, use_graph=True):
    """Prompt of random ids, then greedy decode of `new_tokens` tokens; the decode step is captured in a CUDA
    graph.  Returns the record and the objects that must be released before the process group."""
    import torch.distributed as dist
    cfg = model.cfg
    model.alloc_cache(batch)
    g = torch.Generator(device=dev).manual_seed(17)
    prompt = torch.randint(0, cfg.vocab, (batch, prompt_len), device=dev, generator=g)
    model.forward(prompt, 0)  # first pass: allocations, lazy set-up (untimed)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    nxt = model.forward(prompt, 0)
    torch.cuda.synchronize()
    prefill_s = time.perf_counter() - t0
    ids_buf = nxt.view(batch, 1).clone()
    pos = torch.tensor(prompt_len, device=dev, dtype=torch.int64)
    stream = torch.cuda.Stream(dev)

    def step():
        out = model.forward(ids_buf, pos)
        ids_buf.copy_(out.view(batch, 1))
        pos.add_(1)
    with torch.cuda.stream(stream):
        for _ in range(3):
            step()
        torch.cuda.synchronize()
        graph = None
        if use_graph:
            graph = torch.cuda.CUDAGraph()
            # thread_local: the NCCL watchdog thread may query events while this thread captures
            with torch.cuda.graph(graph, stream=stream, capture_error_mode="thread_local"):
                step()
        torch.cuda.synchronize()
        pos.fill_(prompt_len)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(new_tokens):
            if graph is not None:
                graph.replay()
            else:
                step()
        e1.record(stream)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
    el = e0.elapsed_time(e1) / 1e3
    if world > 1:
        t = torch.tensor([el], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        el = float(t)
    wb = model.weight_bytes_per_step()
    peak = float(load_peaks().get("hbm_gbs", 6650.0))
    rec = {"tok_s": batch * new_tokens / el, "ms_per_step": el / new_tokens * 1e3, "batch": batch, "new_tokens": new_tokens,
           "prompt": prompt_len, "prefill_s": prefill_s, "weight_bytes_per_step_per_rank": wb,
           "hbm_frac_of_measured": wb / (el / new_tokens) / 1e9 / peak,
           "exchange_timed_out": bool(model.xchg.timed_out()) if model.xchg is not None else None,
           "launch": "cuda graph" if graph is not None else "eager"}
    if graph is not None:
        graph.reset()
    return rec


def tp_parity(dev, rank, world, fused):
    """Numeric check of the sharded decoder: a 2-layer model of the full layer shapes, sharded over the ranks
    (same seeded weights, every rank keeps its slice), against the un-sharded model computed on every rank:
    logits of the last prompt position and of three decode steps.  Returns max |a - b| / max |b|."""
    from polarengine_vllm_b200.decoder import DecoderConfig, QuantDecoder
    cfg = DecoderConfig(n_layers=2, vocab=32768)
    sharded = QuantDecoder(cfg, dev, rank, world, None, seed=4321, max_len=64, batch=2, fused_allreduce=fused)
    full = QuantDecoder(cfg, dev, 0, 1, None, seed=4321, max_len=64, batch=2)
    g = torch.Generator(device=dev).manual_seed(5)
    prompt = torch.randint(0, cfg.vocab, (2, 24), device=dev, generator=g)
    worst = 0.0
    a, b = sharded.forward(prompt, 0, return_logits=True), full.forward(prompt, 0, return_logits=True)
    worst = max(worst, float((a - b).abs().max() / b.abs().max()))
    same_tokens = True
    ids = b.argmax(-1).view(2, 1)
    for s in range(3):
        pos = torch.tensor(24 + s, device=dev, dtype=torch.int64)
        a, b = sharded.forward(ids, pos, return_logits=True), full.forward(ids, pos, return_logits=True)
        worst = max(worst, float((a - b).abs().max() / b.abs().max()))
        same_tokens = same_tokens and bool(torch.equal(a.argmax(-1), b.argmax(-1)))
        ids = b.argmax(-1).view(2, 1)
    timed_out = bool(sharded.xchg.timed_out()) if sharded.xchg is not None else None
    del sharded, full
    torch.cuda.empty_cache()
    return {"max_rel": worst, "same_next_tokens": same_tokens, "exchange_timed_out": timed_out,
            "model": "2 layers, hidden 4096, intermediate 12288, vocab 32768, batch 2, prompt 24 + 3 decode steps"}


def model_record(a, dev, rank, world, batches=(1, 8)):
    """BASELINE configs[3]: every projection, the embedding and the LM head quantized; tensor parallel over the
    ranks (column q/k/v/gate/up/head, row o/down).  Strong scaling: the model is fixed, the ranks share it."""
    from polarengine_vllm_b200.decoder import DecoderConfig, QuantDecoder
    fused = world > 1 and not a.nccl_allreduce
    note = "nccl all-reduce + add/norm kernels" if world > 1 else "no exchange (one rank)"
    rec = {"layers": a.layers, "parallelism": f"tp{world}", "scaling": "strong"}
    if world > 1:
        try:
            rec["tp_parity"] = tp_parity(dev, rank, world, fused)
            rec["tp_parity_max_rel"] = rec["tp_parity"]["max_rel"]
        except Exception as exc:
            rec["tp_parity"] = {"error": f"{type(exc).__name__}: {exc}"}
            rec["tp_parity_max_rel"] = None
    else:
        rec["tp_parity_max_rel"] = None
    cfg = DecoderConfig(n_layers=a.layers)
    max_len = a.prompt + a.new_tokens + 8
    try:
        model = QuantDecoder(cfg, dev, rank, world, None, max_len=max_len, batch=1, fused_allreduce=fused)
        if fused:
            note = "all-reduce + residual add + RMSNorm in one kernel over peer memory (decode steps); nccl in prefill"
    except Exception as exc:  # peer mappings unavailable: the NCCL path still measures the model
        if not fused:
            raise
        note = f"nccl all-reduce (peer exchange unavailable: {type(exc).__name__})"
        model = QuantDecoder(cfg, dev, rank, world, None, max_len=max_len, batch=1)
    rec["row_parallel_epilogue"] = note
    for b in batches:
        rec[f"batch{b}"] = decode_run(model, dev, rank, world, b, a.prompt, a.new_tokens, not a.no_graph)
    rec["gpu_launches_per_step"] = 8 * a.layers + 3
    del model
    torch.cuda.empty_cache()
    return rec


# ------------------------------------------------------------------------------------------ MoE
def moe_run(dev, rank, world, tokens, steps=None):
    """BASELINE configs[4]: 128 experts, top-8 softmax routing from a seeded fp16 gate (2688 -> 128), expert
    intermediate 1856, gate/up Q3 and down Q4 codes; expert parallel over the ranks (tokens replicated, every
    rank runs its local experts, all-reduce of the layer output)."""
    import torch.distributed as dist
    from polarengine_vllm_b200.moe_method import PolarQuantMoEMethod, route_softmax_topk
    from polarengine_vllm_b200.parallel import expert_placement
    from polarengine_vllm_b200.utils import get_ct_scaled
    E, H, I, K = 128, 2688, 1856, 8
    T = tokens
    e_local = E // world
    method = PolarQuantMoEMethod(3, 4)
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

    stream = torch.cuda.Stream(dev)
    local_pairs = method.expected_local_pairs(T * K, e_local, emap)
    grouped = local_pairs <= method.GROUPED_MAX_ROWS_PER_EXPERT * e_local
    if steps is None:
        steps = 200 if grouped else 10
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
    peaks = load_peaks()
    ms = el / steps * 1e3
    tensor = local_pairs >= method.TENSOR_CORE_MIN_ROWS_PER_EXPERT * e_local
    rec = {"tokens": T, "tok_s": T * steps / el, "ms_per_layer": ms, "steps": steps, "parallelism": f"ep{world}",
           "path": (("two grouped tcgen05 launches (pe_gemm_grouped), CUDA graph" if tensor
                     else "two grouped decode-size launches (pe_gemv_grouped), CUDA graph") if grouped
                    else "per-expert tensor-core matmuls, eager"),
           "active_experts": active, "expert_bytes_per_step": active * per_expert,
           "weight_gbs": active * per_expert / (ms / 1e3) / 1e9,
           "hbm_frac_of_measured": active * per_expert / (ms / 1e3) / 1e9 / float(peaks.get("hbm_gbs", 6650.0)) / world,
           "tflops": flops / (ms / 1e3) / 1e12,
           "tensor_frac_of_burst": flops / (ms / 1e3) / 1e12 / float(peaks.get("bf16_tflops", 1590.0)) / world,
           "gpu_launches": steps * (5 if grouped else 2 * min(active, e_local))}
    if graph is not None:
        graph.reset()
    return rec


def moe_record(dev, rank, world, token_counts=(1, 64, 2048)):
    rec = {"config": "128 experts top-8, hidden 2688, intermediate 1856, gate/up Q3, down Q4; expert weights 970 MB >> L2"}
    for t in token_counts:
        rec[f"tokens{t}"] = moe_run(dev, rank, world, t)
        torch.cuda.empty_cache()
    return rec


# ------------------------------------------------------------------------------------------ leaving
def finish(world):
    """Leave a multi-rank run in order: captured graphs were reset by their owners, every rank has finished its
    device work, then the process group is destroyed.  (Destroying the communicator while captured graphs that
    hold its kernels were alive blocked a 2-GPU run for good.)  A watchdog ends the process if the teardown
    does not return within 30 s: the result line is already printed."""
    if world > 1:
        import torch.distributed as dist
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        sys.stderr.flush()
        threading.Timer(30.0, lambda: os._exit(0)).start()
        dist.destroy_process_group()
        os._exit(0)  # the timer thread must not keep the interpreter alive


def sub_record(fn, *args, **kw):
    """A secondary measurement must not take the headline down with it."""
    try:
        return fn(*args, **kw)
    except Exception as exc:
        torch.cuda.synchronize()
        return {"error": f"{type(exc).__name__}: {exc}"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=40)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--workload", default="decode", choices=["decode", "prefill", "model", "moe"],
                    help="decode: decoder-layer GEMV pass (default, the headline) followed by the prefill, model and moe "
                         "records; prefill / model / moe: that record alone")
    ap.add_argument("--headline-only", action="store_true", help="decode workload without the prefill / model / moe records")
    ap.add_argument("--secondary-limit", type=float, default=480.0, help="seconds the prefill / model / moe records may take together")
    ap.add_argument("--layers", type=int, default=36, help="decoder layers of the model record")
    ap.add_argument("--prompt", type=int, default=512)
    ap.add_argument("--new-tokens", type=int, default=128)
    ap.add_argument("--no-graph", action="store_true", help="model record: launch decode steps eagerly")
    ap.add_argument("--nccl-allreduce", action="store_true", help="model record: NCCL all-reduce instead of the fused peer-memory epilogue")
    ap.add_argument("--m", type=int, default=4096, help="tokens of the prefill record")
    ap.add_argument("--bits", type=int, default=4, choices=[3, 4, 5, 6], help="prefill workload alone: code width of the layers")
    ap.add_argument("--tokens", type=int, default=None, help="moe workload alone: one token count instead of 1, 64 and 2048")
    a = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    config = {"workload": "decoder_layer_gemv (BASELINE configs[1]): q/k/v Q5 fused, o Q6, gate/up Q3 fused, down Q4; "
                          "hidden 4096, intermediate 12288", "batch": a.batch, "ring_layers": RING,
              "l2_defeat": "inputs larger than L2 (ring of 8 layers = 964 MB of codes)",
              "parallelism": f"replicas x{a.gpus}: each rank streams its own layers, no collective (the model_decode and "
                             f"moe records shard over the ranks)"}
    base = {"metric": "quantized GEMV HBM GB/s", "unit": "GB/s", "n_gpus": a.gpus, "steps": a.steps, "warmup": a.warmup,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": config}

    if a.impl == "reference":
        if rank != 0:
            return
        # The reference has no CPU implementation of apply() (its Triton wrappers need a GPU);
        # its CPU-runnable path is the torch math its kernels are tested against = the oracle.
        cb, per_step = cpu_baseline(a.batch, budget_s=max(5.0, min(60.0, 0.3 * (a.steps + a.warmup))))
        config["parallelism"] = "one host: the CPU arm runs on rank 0 only, whatever --gpus says"
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
    peaks = load_peaks()

    if a.workload != "decode":  # one secondary record alone, as its own line
        common = {"n_gpus": a.gpus, "higher_is_better": True, "vs_baseline": None, "data": "synthetic", "warmup": 3}
        sampler = ClockSampler(local)
        sampler.start()
        if a.workload == "prefill":
            rec = prefill_record(dev, a.m, max(3, min(a.steps, 50)), a.bits)
            best = max(rec["shapes"].values(), key=lambda s: s["tflops"])
            line = dict(common, metric="prefill quantized GEMM TFLOP/s", unit="TFLOP/s", value=best["tflops"], steps=rec["steps"],
                        ms_per_step=best["ms"], scaling="weak", dtype="bf16",
                        config={"workload": f"prefill_gemm (BASELINE configs[2]) M={a.m}, Q{a.bits}"}, prefill=rec, gpu_launches=rec["gpu_launches"])
        elif a.workload == "model":
            rec = model_record(a, dev, rank, world, (a.batch,))
            r = rec[f"batch{a.batch}"]
            line = dict(common, metric="9B-class decode tok/s", unit="tok/s", value=r["tok_s"], steps=a.new_tokens,
                        ms_per_step=r["ms_per_step"], scaling="strong", dtype="f16",
                        config={"workload": f"model_decode (BASELINE configs[3]): {a.layers} layers", "batch": a.batch,
                                "parallelism": f"tp{world}"}, model_decode=rec, gpu_launches=a.new_tokens * rec["gpu_launches_per_step"])
        else:
            rec = moe_record(dev, rank, world, (a.tokens,) if a.tokens else (1, 64, 2048))
            first = next(v for k, v in rec.items() if k.startswith("tokens"))
            line = dict(common, metric="MoE layer tokens/s", unit="tok/s", value=first["tok_s"], steps=first["steps"],
                        ms_per_step=first["ms_per_layer"], scaling="strong", dtype="f16",
                        config={"workload": "moe_layer (BASELINE configs[4])", "parallelism": f"ep{world}"}, moe=rec,
                        gpu_launches=first["gpu_launches"])
        sampler.stop_flag = True
        line["clocks"] = sampler.summary()
        if rank == 0:
            print(json.dumps(line))
        return finish(world)

    # ---- headline: the decoder-layer pass
    ring_passes = max(1, math.ceil(a.steps / RING))  # the graph holds RING steps: the asked-for step count is rounded up
    warm = max(3, a.warmup)
    layers = [make_layer(dev, 1000 + 16 * i + 97 * rank) for i in range(RING)]
    g = torch.Generator(device=dev).manual_seed(7)
    xh = torch.randn(a.batch, HIDDEN, device=dev, generator=g).half()
    xi = torch.randn(a.batch, INTER, device=dev, generator=g).half()

    def launch(layer, name):
        w, packed, norms, ct, n, k = layer[name]
        return kernels.quant_matmul(w, packed, norms, ct, xh if k == HIDDEN else xi, False, n, k, k, torch.float16)

    def ring_pass(names):
        for layer in layers:
            for name in names:
                launch(layer, name)

    all_names = [p[0] for p in PROJ]
    stream = torch.cuda.Stream(dev)

    def timed_graph(names, passes, warm_passes):
        """Capture one ring pass (RING steps) as a CUDA graph and time `passes` replays, repeated until the
        timed region is at least MIN_TIMED_S long.  Returns (seconds, ring passes timed)."""
        with torch.cuda.stream(stream):
            ring_pass(names)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                ring_pass(names)
            for _ in range(warm_passes):
                graph.replay()
            torch.cuda.synchronize()
            total, done = 0.0, 0
            while True:
                if world > 1:
                    dist.barrier()
                    torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(stream)
                for _ in range(passes):
                    graph.replay()
                e1.record(stream)
                torch.cuda.synchronize()
                el = e0.elapsed_time(e1) / 1e3
                if world > 1:
                    dist.barrier()
                    t = torch.tensor([el], device=dev, dtype=torch.float64)
                    dist.all_reduce(t, op=dist.ReduceOp.MAX)
                    el = float(t)
                total += el
                done += passes
                if total >= MIN_TIMED_S or done >= 200000:
                    break
                passes = max(passes, int(passes * (MIN_TIMED_S - total) / max(el, 1e-6)) + 1)  # same on every rank (el is the max)
            graph.reset()
            return total, done

    sampler = ClockSampler(local)
    sampler.start()
    elapsed, passes_done = timed_graph(all_names, ring_passes, max(1, math.ceil(warm / RING)))
    steps = passes_done * RING
    # dominant kernel alone: the nibble-code GEMV on the 4096x12288 Q4 layer (down_proj)
    dom = ["down_proj"]
    dom_elapsed, dom_passes = timed_graph(dom, ring_passes, 1)
    sampler.stop_flag = True
    value = step_bytes(a.batch) * steps * world / elapsed / 1e9

    # ---- end to end through the plugin surface with host buffers
    method = {}
    mods = {}
    for name, n, k, bits in PROJ:
        m = PolarQuantLinearMethod(128, bits)
        mod = torch.nn.Module()
        w, packed, norms, ct, _, _ = layers[0][name]
        mod.in_f, mod.out_f, mod.in_f_padded, mod.n_blocks, mod.bits, mod.block_size = k, n, k, k // 128, bits, 128
        mod.packed, mod.norms, mod.ct_scaled = packed, norms, ct
        if packed:
            mod.codes_packed, mod.in_f_half = w, k // 2
        else:
            mod.codes = w
        method[name], mods[name] = m, mod
    hx = {k: torch.randn(a.batch, k).half().pin_memory() for k in (HIDDEN, INTER)}
    hy = torch.empty(a.batch, HIDDEN, dtype=torch.float16).pin_memory()
    e2e_steps = min(max(steps, 200), 1000)

    def e2e_body(i, dx):
        layer = layers[i % RING]
        y = None
        for name, n, k, bits in PROJ:
            mod = mods[name]
            w, packed, norms, ct, _, _ = layer[name]
            mod.norms = norms
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
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr, stream=stream, capture_error_mode="thread_local"):
                for k in hx:
                    dx_static[k].copy_(hx[k], non_blocking=True)
                hy.copy_(e2e_body(i, dx_static), non_blocking=True)
            graphs.append(gr)

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
    for gr in graphs:
        gr.reset()
    e2e = {"value": e2e_graph, "unit": "GB/s",
           "h2d_bytes_per_step": a.batch * (HIDDEN + INTER) * 2, "d2h_bytes_per_step": a.batch * HIDDEN * 2,
           "steps": e2e_steps, "eager_value": e2e_eager,
           "api": "PolarQuantLinearMethod.apply x4 per step with pinned host in/out copies, the step captured in a "
                  "CUDA graph and waited on by the host after every replay; eager_value = same step without the graph"}

    peak = float(peaks.get("hbm_gbs", 6650.0))
    dom_launches = dom_passes * RING
    dom_bytes = sum(alg_bytes(n, k, b, a.batch) for nm, n, k, b in PROJ if nm in dom)
    achieved = dom_bytes / (dom_elapsed / dom_launches) / 1e9
    dom_kernel = ("gemv_cols_kernel<nibble codes, table, 3 chunks per warp>" if a.batch == 1 else
                  "gemv_rows_kernel<nibble codes, table>" if a.batch == 2 else "gemv_kernel (tile kernel)<nibble codes, table>")
    roofline = {"bound": "hbm", "kernel": dom_kernel + " on down_proj 4096x12288 Q4",
                "achieved": achieved, "peak": peak, "peak_source": "measured (MEASURED_PEAKS.json)" if peaks else "fallback",
                "unit": "GB/s", "frac": achieved / peak, "avg_launch_us": dom_elapsed / dom_launches * 1e6,
                "alg_bytes_per_launch": dom_bytes, "launches_timed": dom_launches,
                "traffic": measured_traffic("down_proj_b1") if a.batch == 1 else None}
    line = dict(base, value=value, ms_per_step=elapsed / steps * 1e3, steps=steps, steps_requested=a.steps, e2e=e2e,
                gpu_launches=4 * steps, roofline=roofline, clocks=sampler.summary(), frac_of_measured_hbm=value / world / peak,
                timed_region_s=elapsed)
    del layers, mods, graphs
    torch.cuda.empty_cache()

    if rank == 0 and not a.no_cpu_baseline and world == 1:
        line["cpu_baseline"], _ = cpu_baseline(a.batch)

    # The secondary records run under a time limit: if one of them stalls (a rank that left a collective), the
    # line is printed with what has been measured and the process ends.
    emitted = threading.Lock()

    def emit():
        if emitted.acquire(blocking=False) and rank == 0:
            print(json.dumps(line))
            sys.stdout.flush()

    def out_of_time():
        line["secondary_records_cut_short_after_s"] = a.secondary_limit
        emit()
        os._exit(0)

    if not a.headline_only:
        limit = threading.Timer(a.secondary_limit, out_of_time)
        limit.daemon = True
        limit.start()
        line["prefill"] = sub_record(prefill_record, dev, a.m)
        line["model_decode"] = sub_record(model_record, a, dev, rank, world)
        line["moe"] = sub_record(moe_record, dev, rank, world)
        limit.cancel()
    emit()
    finish(world)


if __name__ == "__main__":
    main()
