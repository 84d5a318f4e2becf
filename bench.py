#!/usr/bin/env python
"""Headline benchmark: decode throughput of the grouped-expert MoE path on B200.

Workload (N = 1): an OLMoE-shaped MoE stack - 16 distinct layers, each 64 experts, top-8,
hidden 2048, expert intermediate 1024, SwiGLU, shared fp16 backbones of rank 256, compact3
experts with block Golomb-Rice bitmaps - at decode batch 128 (batches 1/8/32 are reported
in `sweep`).  A step pushes one batch through all 16 layers; 16 distinct payloads (~290 MB)
exceed the 126 MB L2, so every step streams the compressed weights from HBM.  All data is
seeded synthetic (no checkpoints or datasets are available offline).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

`value`   : tokens/s with inputs resident in HBM, CUDA-graph replay of the step, CUDA events.
`e2e`     : tokens/s through the public Python API (TrisSparseMoeBlock.forward) with the batch
            copied from pinned host memory and the result copied back inside the timed region.
`roofline`: the dominant kernel (grouped compact3 matmul) timed alone with CUDA events over
            the same 16 payloads: compressed bytes per launch / duration, against the measured
            HBM copy bandwidth of MEASURED_PEAKS.json.
`cpu_baseline` / `--impl reference`: the CPU port of the reference's expert-loop path
            (oracle/cpu_reference_path.py) timed on the host cores on a bounded sample.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (ROOT, os.path.join(ROOT, "oracle")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import numpy as np
import torch

from trismoe_b200.clocks import ClockSampler

LAYERS = 16
HEADLINE_TOKENS = 128
SWEEP_TOKENS = (1, 8, 32, 128)
NOMINAL_HBM_GBS = 8000.0
FALLBACK_HBM_GBS = 6650.0
LAUNCHES_PER_LAYER = 7  # backbone+router GEMM, top-k, route, gate/up, down backbone, down, combine


KERNEL_SOURCES = ("grouped_tiled.cu", "tile_records.cuh", "tile_records.cu")  # what the dominant kernel is built from
TRAFFIC_FILE = os.path.join(ROOT, "profiles", "grouped_tiled_traffic.json")


def kernel_source_hash():
    import hashlib

    h = hashlib.sha256()
    for name in KERNEL_SOURCES:
        with open(os.path.join(ROOT, "neurips26-tris-moe_b200", "csrc", name), "rb") as fh:
            h.update(fh.read())
    return h.hexdigest()[:16]


def measured_traffic(kernel):
    """DRAM bytes per launch of the grouped kernels from the last ncu capture, recorded in
    profiles/grouped_tiled_traffic.json together with a hash of the kernel sources it was taken
    on; None once the sources have changed since (a stale figure is worse than none)."""
    try:
        with open(TRAFFIC_FILE) as fh:
            rec = json.load(fh)
    except Exception:
        return None, "no capture on record"
    if rec.get("source_hash") != kernel_source_hash():
        return None, f"capture {rec.get('source_hash')} is older than the kernel sources"
    return rec.get("dram_bytes_per_launch", {}).get(kernel), rec.get("command", "ncu capture, see profiles/")


def measured_hbm_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as fh:
            return float(json.load(fh)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


def build_stack(device, layers=LAYERS, seed=1234, keep_sparse=False):
    import trismoe_b200 as tm
    from trismoe_b200 import synth

    blocks, infos = [], []
    for l in range(layers):
        layer = synth.synth_layer(synth.OLMOE, seed=seed + l, keep_sparse_gmap=keep_sparse)
        blk = tm.TrisSparseMoeBlock(2048, 1024, 64, 8, True)
        blk.load_grouped_payloads(layer["gate"], layer["up"], layer["down"], layer["shared_gate"], layer["shared_up"],
                                  layer["shared_down"], layer["router_weight"], device=device)
        blocks.append(blk)
        infos.append(layer)
    return blocks, infos


def layer_algorithmic_bytes(info, active_experts, tokens):
    """Compressed weight bytes of the active experts + backbones + router + activations in/out;
    intermediates count zero (the figure an ideally fused layer must move)."""
    from trismoe_b200 import synth

    shape = synth.OLMOE
    per_proj = {n: synth.projection_algorithmic_bytes(info[n], active_experts) for n in ("gate", "up", "down")}
    backbone = 2 * (2 * shape.rank * shape.hidden_size + shape.rank * shape.intermediate_size)
    router = 2 * shape.num_experts * shape.hidden_size
    act = 4 * tokens * shape.hidden_size
    return per_proj, sum(per_proj.values()) + backbone + router + act


REPEATS = 5


def time_replays(graph, steps, warmup, repeats=REPEATS):
    """Median over `repeats` timings of `steps` back-to-back replays (CUDA events), ms per step."""
    for _ in range(warmup):
        graph.replay()
    torch.cuda.synchronize()
    samples = []
    for _ in range(repeats):
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(steps):
            graph.replay()
        stop.record()
        torch.cuda.synchronize()
        samples.append(start.elapsed_time(stop) / steps)
    return statistics.median(samples)


def capture(fn, error_mode="global"):
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(3):
            fn()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, capture_error_mode=error_mode):
        fn()
    return graph


def run_ours(args):
    import trismoe_b200 as tm
    from trismoe_b200 import synth

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        from trismoe_b200 import expert_parallel

        try:
            return expert_parallel.run_bench(args, rank, world, device)
        finally:
            dist.barrier()
            dist.destroy_process_group()

    blocks, infos = build_stack(device)
    peak, peak_kind = measured_hbm_peak()
    sampler = ClockSampler(local)
    results = {}
    sampler.start()
    for T in SWEEP_TOKENS:
        x = synth.synth_activations(T, 2048, seed=T).to(device)
        outs = [None] * LAYERS

        def step():
            for l, blk in enumerate(blocks):
                outs[l] = blk(x.view(1, T, 2048))[0]

        graph = capture(step)
        steps = args.steps if T == HEADLINE_TOKENS else max(10, args.steps // 2)
        ms = time_replays(graph, steps, args.warmup)
        # bytes: which experts each layer activates for this batch
        total_bytes = 0
        for blk, info in zip(blocks, infos):
            logits = torch.nn.functional.linear(x, blk.gate.weight).float()
            sel = torch.topk(torch.softmax(logits, dim=1), 8, dim=-1)[1]
            active = sorted(set(sel.reshape(-1).tolist()))
            total_bytes += layer_algorithmic_bytes(info, active, T)[1]
        results[T] = {"ms_per_step": ms, "tokens_per_s": T / (ms * 1e-3), "us_per_layer": ms * 1e3 / LAYERS,
                      "algorithmic_mb_per_layer": total_bytes / LAYERS / 1e6,
                      "layer_gbs": total_bytes / (ms * 1e-3) / 1e9}
        del graph
    T = HEADLINE_TOKENS
    head = results[T]
    # the same batch through ONE layer 16 times: its ~22 MB payload stays in the 126 MB L2
    x = synth.synth_activations(T, 2048, seed=T).to(device)

    def warm_step():
        for _ in range(LAYERS):
            blocks[0](x.view(1, T, 2048))

    graph = capture(warm_step)
    l2_resident_us = time_replays(graph, max(10, args.steps // 2), args.warmup) * 1e3 / LAYERS
    del graph

    # ---- dominant kernel alone: grouped gate/up (SiLU*mul epilogue) and grouped down ----------
    x = synth.synth_activations(T, 2048, seed=T).to(device)
    kern = {}
    routes, hid, byts = [], [], {"pair": 0, "down": 0}
    for blk, info in zip(blocks, infos):
        logits = torch.nn.functional.linear(x, blk.gate.weight).float()
        sel = torch.topk(torch.softmax(logits, dim=1), 8, dim=-1)[1]
        route = tm.build_grouped_route(sel, 64)
        routes.append(route)
        tok = route["grouped_token_indices"]
        # what the layer path feeds the grouped kernels: backbone outputs in lane order, read through the route's gather
        hg = tm.compute_shared_hidden(x, blk.shared_gate, layout=tm.HIDDEN_LANE_ORDER)
        hu = tm.compute_shared_hidden(x, blk.shared_up, layout=tm.HIDDEN_LANE_ORDER)
        hd = torch.randn((tok.numel(), 256), device=device).half()
        hid.append((hg, hu, hd))
        route["_gather_route"] = dict(route, _row_gather=tok.to(torch.int32), _hidden_layout=tm.HIDDEN_LANE_ORDER)
        route["_lane_route"] = dict(route, _hidden_layout=tm.HIDDEN_LANE_ORDER)
        active = route["expert_ids"].tolist()
        per_proj, _ = layer_algorithmic_bytes(info, active, T)
        byts["pair"] += per_proj["gate"] + per_proj["up"]
        byts["down"] += per_proj["down"]

    def pair_step():
        for blk, route, (hg, hu, hd) in zip(blocks, routes, hid):
            tm.run_grouped_structured_expert_pair_forward(blk._get_grouped_payload("gate"), blk._get_grouped_payload("up"),
                                                          hg, hu, None, route["_gather_route"], fuse_silu_mul=True)

    def down_step():
        for blk, route, (hg, hu, hd) in zip(blocks, routes, hid):
            tm.run_grouped_structured_expert_forward(blk._get_grouped_payload("down"), hd, None, route["_lane_route"])

    for name, fn in (("pair", pair_step), ("down", down_step)):
        graph = capture(fn)
        ms = time_replays(graph, args.steps, args.warmup)
        kern[name] = {"us_per_launch": ms * 1e3 / LAYERS, "bytes_per_launch": byts[name] / LAYERS,
                      "gbs": byts[name] / (ms * 1e-3) / 1e9}
        del graph
    dom = max(kern, key=lambda n: kern[n]["us_per_launch"])
    roofline = {
        "bound": "hbm", "kernel": f"grouped_tiled_kernel ({'gate/up dual + SiLU*mul' if dom == 'pair' else 'down'})",
        "achieved": round(kern[dom]["gbs"], 1), "peak": peak, "peak_kind": peak_kind, "unit": "GB/s",
        "frac": round(kern[dom]["gbs"] / peak, 4), "frac_of_nominal_8TBs": round(kern[dom]["gbs"] / NOMINAL_HBM_GBS, 4),
        # dram__bytes_read.sum + dram__bytes_write.sum of one launch of this kernel on this workload, from the
        # ncu capture on record (not measured in this run); null when the kernel sources changed since
        "traffic": measured_traffic(dom)[0], "traffic_source": measured_traffic(dom)[1],
        "us_per_launch": round(kern[dom]["us_per_launch"], 2),
        "algorithmic_bytes_per_launch": int(kern[dom]["bytes_per_launch"]),
        "other_kernels": {n: {k: round(v, 2) for k, v in d.items()} for n, d in kern.items() if n != dom},
        "whole_layer": {"gbs": round(head["layer_gbs"], 1), "frac": round(head["layer_gbs"] / peak, 4),
                        "frac_of_nominal_8TBs": round(head["layer_gbs"] / NOMINAL_HBM_GBS, 4)},
    }

    # ---- end to end through the public API with host buffers --------------------------------
    x_host = synth.synth_activations(T, 2048, seed=T).pin_memory()
    y_host = torch.empty((T, 2048), dtype=torch.float16).pin_memory()
    x_dev = torch.empty((T, 2048), dtype=torch.float16, device=device)

    def e2e_step():
        x_dev.copy_(x_host, non_blocking=True)
        y = None
        for blk in blocks:
            y = blk(x_dev.view(1, T, 2048))[0]
        y_host.copy_(y.view(T, 2048), non_blocking=True)

    for _ in range(args.warmup):
        e2e_step()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    start.record()
    for _ in range(args.steps):
        e2e_step()
    stop.record()
    torch.cuda.synchronize()
    e2e_ms = max(start.elapsed_time(stop), (time.perf_counter() - t0) * 1e3) / args.steps
    clocks = sampler.stop()
    olmoe_status = max(b.last_kernel_status() for b in blocks)  # sticky status words of every layer: 0 = no bounded wait ran out

    # the Mixtral-shaped stack of the expert-parallel lines (config 3), here on one GPU: 4 of the 32 layers
    del blocks
    torch.cuda.empty_cache()
    mixtral = {"shape": "8 experts, top-2, hidden 4096, intermediate 14336, rank-256 backbones", "layers_timed": 4,
               "of_layers": 32, "experts_per_gpu": 8, "decode": []}
    mblocks = []
    for l in range(4):
        layer = synth.synth_layer(synth.MIXTRAL, seed=600 + l)
        blk = tm.TrisSparseMoeBlock(4096, 14336, 8, 2, True)
        blk.load_grouped_payloads(layer["gate"], layer["up"], layer["down"], layer["shared_gate"], layer["shared_up"],
                                  layer["shared_down"], layer["router_weight"], device=device)
        mblocks.append(blk)
    for TB in (1, 64):
        xm = synth.synth_activations(TB, 4096, seed=2000).to(device)

        def mstep():
            for blk in mblocks:
                blk(xm.view(1, TB, 4096))

        graph = capture(mstep)
        mms = time_replays(graph, max(10, args.steps // 2), args.warmup, repeats=3)
        mixtral["decode"].append({"tokens_per_gpu": TB, "tokens_per_s": round(TB / (mms * 1e-3), 1),
                                  "us_per_layer": round(mms * 1e3 / 4, 2), "launch_mode": "cuda graph"})
        del graph
    mixtral["kernel_status"] = max(b.last_kernel_status() for b in mblocks)
    del mblocks
    torch.cuda.empty_cache()
    cpu = cpu_baseline(sample_tokens=T)
    out = {
        "metric": "decode_tokens_per_s", "value": round(head["tokens_per_s"], 1), "unit": "tokens/s", "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(head["ms_per_step"], 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": WORKLOAD,
                   "tokens_per_step": T, "layers": LAYERS, "cold_cache": "16 distinct layer payloads (~290 MB) > 126 MB L2",
                   "parallelism": "single GPU"},
        "e2e": {"value": round(T / (e2e_ms * 1e-3), 1), "unit": "tokens/s", "h2d_bytes_per_step": T * 2048 * 2,
                "d2h_bytes_per_step": T * 2048 * 2, "ms_per_step": round(e2e_ms, 4)},
        "gpu_launches": args.steps * REPEATS * LAYERS * LAUNCHES_PER_LAYER,
        "timing": f"median of {REPEATS} repeats of {args.steps} graph replays (CUDA events)",
        "roofline": roofline, "cpu_baseline": cpu, "clocks": clocks, "mixtral_ep": mixtral, "kernel_status": olmoe_status,
        "sweep": {str(t): {k: round(v, 3) for k, v in r.items()} for t, r in results.items()},
        "l2_resident": {"tokens": T, "us_per_layer": round(l2_resident_us, 3),
                        "note": "one layer replayed 16 times (payload stays in L2); the headline uses 16 distinct layers"},
    }
    print(json.dumps(out))


WORKLOAD = ("OLMoE-shaped 16-layer MoE stack (64 experts top-8, hidden 2048, intermediate 1024, "
            "rank-256 fp16 backbones, compact3 + block-GR experts), decode batch 128")


def cpu_reference_stack(layers):
    """`layers` distinct CPU layers with the seeds of the GPU arm's stack (sparse g_map planes: the
    reference's CPU path reads q_gmap_sparse, it has no Golomb-Rice decoder on the CPU)."""
    from trismoe_b200 import synth

    return [synth.synth_layer(synth.OLMOE, seed=1234 + l, keep_sparse_gmap=True, use_block_gr=False) for l in range(layers)]


def cpu_reference_pass(stack, x):
    import cpu_reference_path as cpu

    y = None
    for layer in stack:
        y = cpu.moe_block_forward(x, layer, 8, True)
    return y


def cpu_baseline(sample_tokens=HEADLINE_TOKENS, layers=3, iters=2):
    """Times the CPU port of the reference path (oracle/cpu_reference_path.py, pinned to the
    reference by tests/test_oracle_golden.py) on a bounded sample: the first `layers` layers of
    the stack at the headline batch, scaled to the 16-layer step."""
    from trismoe_b200 import synth

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    stack = cpu_reference_stack(layers)
    x = synth.synth_activations(sample_tokens, 2048, seed=sample_tokens)
    cpu_reference_pass(stack, x)  # warm-up
    t0 = time.perf_counter()
    for _ in range(iters):
        cpu_reference_pass(stack, x)
    per_layer = (time.perf_counter() - t0) / iters / layers
    return {"value": round(sample_tokens / (per_layer * LAYERS), 3), "unit": "tokens/s", "cores": cores, "kind": "port",
            "sample": f"{layers} of {LAYERS} distinct layers x {sample_tokens} tokens, {iters} timed passes after 1 warm-up, "
                      f"{per_layer:.3f} s per layer, scaled to the 16-layer step",
            "s_per_layer": round(per_layer, 4)}


def run_reference(args):
    """The CPU arm: the port of the reference's expert-loop path on all host cores, the GPU arm's
    workload.  A step is one batch of 128 tokens through all 16 distinct layers (no scaling) as long
    as warm-up + steps fit a ~4.5 minute budget; otherwise a step covers the first L layers and the
    value is scaled by 16 / L (said in `sample`)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from trismoe_b200 import synth

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    steps, warmup = max(1, args.steps), max(1, args.warmup)
    stack = cpu_reference_stack(LAYERS)
    x = synth.synth_activations(HEADLINE_TOKENS, 2048, seed=HEADLINE_TOKENS)
    t0 = time.perf_counter()
    cpu_reference_pass(stack, x)  # first warm-up step, also the estimate
    t_pass = time.perf_counter() - t0
    budget_s = 270.0
    per_step_layers = LAYERS
    if t_pass * (steps + warmup - 1) > budget_s:
        per_step_layers = max(1, min(LAYERS, int(LAYERS * budget_s / (t_pass * (steps + warmup - 1)))))
    sub = stack[:per_step_layers]
    for _ in range(warmup - 1):
        cpu_reference_pass(sub, x)
    t0 = time.perf_counter()
    for _ in range(steps):
        cpu_reference_pass(sub, x)
    step_s = (time.perf_counter() - t0) / steps
    value = HEADLINE_TOKENS / (step_s * LAYERS / per_step_layers)
    cpu = {"value": round(value, 3), "unit": "tokens/s", "cores": cores, "kind": "port",
           "sample": (f"{per_step_layers} of {LAYERS} distinct layers x {HEADLINE_TOKENS} tokens per step, {steps} timed steps "
                      f"after {warmup} warm-up, {step_s:.3f} s per step"
                      + ("" if per_step_layers == LAYERS else f", scaled by {LAYERS}/{per_step_layers} to the 16-layer step")),
           "s_per_layer": round(step_s / per_step_layers, 4)}
    out = {
        "impl": "reference", "metric": "decode_tokens_per_s", "value": cpu["value"], "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": warmup, "ms_per_step": round(step_s * 1e3, 1),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "tokens_per_step": HEADLINE_TOKENS, "layers": LAYERS,
                   "cold_cache": "16 distinct layer payloads (~290 MB) > 126 MB L2", "parallelism": "single GPU"},
        "cpu_baseline": cpu,
        "e2e": {"value": cpu["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "CPU port of the reference's expert-loop path (the Python reference cannot travel to the GPU box); "
                "pinned to the reference's own outputs by tests/test_oracle_golden.py",
    }
    print(json.dumps(out))


def run_ncu_case(args):
    """Small fixed launch sequence for profiler captures (no timing, no graphs):
    `layer`   - one warm-up pass and one pass of the whole block over `--layers` layers;
    `grouped` - two passes of the grouped gate/up and grouped down kernels alone;
    `packed4` - two passes of the 4-bit GEMM over 80 distinct 2048 x 2048 matrices, `--tokens` rows."""
    import trismoe_b200 as tm
    from trismoe_b200 import synth

    torch.cuda.set_device(0)
    device = torch.device("cuda", 0)
    T = args.tokens
    if args.ncu_case == "packed4":  # 80 distinct 2048 x 2048 4-bit matrices (176 MB > L2), two passes
        rng = np.random.default_rng(0)
        mats = [tm.Packed4Linear(synth.packed4_matrix(rng, 2048, 2048, 128), device) for _ in range(80)]
        x = synth.synth_activations(T, 2048, seed=T).to(device)
        for _ in range(2):
            for m in mats:
                m(x, 3)
            torch.cuda.synchronize()
        return
    blocks, _ = build_stack(device, layers=args.layers)
    x = synth.synth_activations(T, 2048, seed=T).to(device)
    if args.ncu_case == "layer":
        for _ in range(2):
            for blk in blocks:
                blk(x.view(1, T, 2048))
            torch.cuda.synchronize()
        return
    prepared = []
    for blk in blocks:
        logits = torch.nn.functional.linear(x, blk.gate.weight).float()
        sel = torch.topk(torch.softmax(logits, dim=1), 8, dim=-1)[1]
        route = tm.build_grouped_route(sel, 64)
        tok = route["grouped_token_indices"]
        hg = tm.compute_shared_hidden(x, blk.shared_gate).index_select(0, tok)
        hu = tm.compute_shared_hidden(x, blk.shared_up).index_select(0, tok)
        hd = torch.randn((tok.numel(), 256), device=device).half()
        prepared.append((blk, route, hg, hu, hd))
    torch.cuda.synchronize()
    for _ in range(2):
        for blk, route, hg, hu, hd in prepared:
            tm.run_grouped_structured_expert_pair_forward(blk._get_grouped_payload("gate"), blk._get_grouped_payload("up"),
                                                          hg, hu, None, route, fuse_silu_mul=True)
            tm.run_grouped_structured_expert_forward(blk._get_grouped_payload("down"), hd, None, route)
        torch.cuda.synchronize()


def streaming_records(blocks, manager, shape, device):
    """Times `forward_streaming` over the stack at batch 1 and 16: eager (with the pager's copy and stall
    intervals from CUDA events) and as one CUDA graph."""
    from trismoe_b200 import staging, synth

    n_layers, H = len(blocks), shape.hidden_size
    per_expert = [sum(manager.entries[(l, p)].block_bytes[k] for p in staging.PROJECTIONS
                      for k in manager.entries[(l, p)].block_bytes) for l in range(n_layers)]
    recs = []
    for T in (1, 16):
        x = synth.synth_activations(T, H, seed=T).to(device)

        def step():
            for l, blk in enumerate(blocks):
                blk.forward_streaming(x.view(1, T, H), manager, l)

        paged_bytes = 0
        for l, blk in enumerate(blocks):  # bytes one pass pages: distinct routed experts x per-expert block sizes
            _, logits = blk.forward_streaming(x.view(1, T, H), manager, l)
            paged_bytes += torch.unique(torch.topk(logits, shape.top_k, dim=-1).indices).numel() * per_expert[l]
        for _ in range(3):
            step()
        torch.cuda.synchronize()
        manager.overlap_report()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 10
        start.record()
        for _ in range(reps):
            step()
        stop.record()
        torch.cuda.synchronize()
        ms = start.elapsed_time(stop) / reps
        rep = manager.overlap_report()
        # the same step as one CUDA graph (kernels on two streams, ordered by events)
        graph_ms, graph_err = None, None
        try:
            manager.collect_timings = False
            graph = capture(step)
            graph_ms = time_replays(graph, 10, 3)
            del graph
        except Exception as exc:  # noqa: BLE001
            graph_ms, graph_err = None, str(exc)[:160]
            torch.cuda.synchronize()
        finally:
            manager.collect_timings = True
        best_ms = ms if graph_ms is None else min(ms, graph_ms)
        recs.append({"tokens": T, "layers": n_layers,
                     "us_per_layer": round(ms * 1e3 / n_layers, 2), "tokens_per_s": round(T / (ms * 1e-3), 1),
                     "graph_us_per_layer": None if graph_ms is None else round(graph_ms * 1e3 / n_layers, 2),
                     "graph_tokens_per_s": None if graph_ms is None else round(T / (graph_ms * 1e-3), 1),
                     "graph_error": graph_err,
                     "overlapped_fraction": None if rep["overlapped_fraction"] is None else round(rep["overlapped_fraction"], 3),
                     "copy_ms_per_layer": round(rep["copy_ms"] / max(1, rep["layers"]), 4),
                     "paged_mb_per_pass": round(paged_bytes / 1e6, 2),
                     "pager_gbs": round(paged_bytes * reps / (rep["copy_ms"] * 1e-3) / 1e9, 2) if rep["copy_ms"] else None,
                     "paged_gbs_over_step": round(paged_bytes / (best_ms * 1e-3) / 1e9, 2),
                     "staging_buffer_mb": round(manager.buffer_nbytes / 1e6, 1)})
    return recs


def run_extra(args):
    """Secondary workloads (not the contract line): prints one JSON object with
    - prefill of 2048 tokens through OLMoE-shaped layers (tcgen05 grouped path),
    - a Mixtral-shaped layer (8 experts, top-2, hidden 4096, intermediate 14336): prefill 2048, decode 1/64,
    - streaming: OLMoE-shaped layers with the payload paged from pinned host memory, decode 1/16,
      tokens/s and overlapped fraction of the transfer time."""
    import trismoe_b200 as tm
    from trismoe_b200 import staging, synth

    torch.cuda.set_device(0)
    device = torch.device("cuda", 0)
    out = {}

    def stack(shape, layers, seed, **kw):
        blocks = []
        for l in range(layers):
            layer = synth.synth_layer(shape, seed=seed + l, **kw)
            blk = tm.TrisSparseMoeBlock(shape.hidden_size, shape.intermediate_size, shape.num_experts, shape.top_k, True)
            blk.load_grouped_payloads(layer["gate"], layer["up"], layer["down"], layer["shared_gate"], layer["shared_up"],
                                      layer["shared_down"], layer["router_weight"], device=device)
            blocks.append(blk)
        return blocks

    def time_stack(blocks, T, hidden, steps=10):
        x = synth.synth_activations(T, hidden, seed=T).to(device)

        def step():
            for blk in blocks:
                blk(x.view(1, T, hidden))

        graph = capture(step)
        ms = time_replays(graph, steps, 3)
        return {"tokens": T, "us_per_layer": round(ms * 1e3 / len(blocks), 2), "tokens_per_s": round(T / (ms * 1e-3), 1)}

    olmoe = stack(synth.OLMOE, 8, 500)
    out["olmoe_prefill"] = [time_stack(olmoe, T, 2048) for T in (512, 2048)]
    flops = lambda shape, T: 2 * T * shape.top_k * shape.rank * (2 * shape.intermediate_size + shape.hidden_size) + \
        2 * T * shape.hidden_size * 2 * shape.rank + 2 * T * shape.top_k * shape.intermediate_size * shape.rank
    for rec in out["olmoe_prefill"]:
        rec["tflops"] = round(flops(synth.OLMOE, rec["tokens"]) / (rec["us_per_layer"] * 1e-6) / 1e12, 2)
    del olmoe
    torch.cuda.empty_cache()
    mixtral = stack(synth.MIXTRAL, 4, 600)
    out["mixtral_layer"] = [time_stack(mixtral, T, 4096) for T in (1, 64, 2048)]
    for rec in out["mixtral_layer"]:
        rec["tflops"] = round(flops(synth.MIXTRAL, rec["tokens"]) / (rec["us_per_layer"] * 1e-6) / 1e12, 2)
    del mixtral
    torch.cuda.empty_cache()
    # BASELINE config 2: the full 16-layer OLMoE-1B-7B-shaped decoder (fp16 attention, 16 heads of 128, vocab
    # 50304), random prompt of 512 tokens, 256 generated tokens, batch 1 and 32; definitions of
    # tools/benchmark_e2e_grid.py (decode tokens/s = batch * decode steps / decode time)
    from trismoe_b200 import decode_harness as dh

    full = stack(synth.OLMOE, LAYERS, 1234)
    model = dh.TrisDecoder(full, dh.DecoderShape(), max_length=512 + 256, max_batch=32, device=device, seed=0)
    out["e2e_decode_olmoe_16_layers"] = []
    for B in (1, 32):
        ids = torch.randint(0, 50304, (B, 512), generator=torch.Generator().manual_seed(B)).to(device)
        dh.run_exact_generation(model, ids, 8)  # warm-up
        rec = dh.run_exact_generation(model, ids, 256)
        out["e2e_decode_olmoe_16_layers"].append({k: (round(v, 3) if isinstance(v, float) else v) for k, v in rec.items() if k != "tokens"})
    for blk in full:
        blk.raise_on_kernel_status()
    del model, full
    torch.cuda.empty_cache()
    # 4-bit backbones read in place (2048 x 2048, 128-column groups) against their fp16 expansion on the
    # skinny / tcgen05 GEMMs: 80 distinct matrices per pass (160 MB of nibbles, 640 MB of fp16: both beyond L2)
    from trismoe_b200 import Packed4Linear, compute_shared_hidden, dequantize_packed_4bit

    rng = np.random.default_rng(0)
    mats = [synth.packed4_matrix(rng, 2048, 2048, 128) for _ in range(80)]
    packed = [Packed4Linear(m, device) for m in mats]
    dense = [dequantize_packed_4bit(m, device) for m in mats]
    out["packed4_backbone_2048x2048"] = []
    for T in (1, 16, 128):
        x = synth.synth_activations(T, 2048, seed=T).to(device)
        g4 = capture(lambda: [p(x, 3) for p in packed])
        g16 = capture(lambda: [compute_shared_hidden(x, w, layout=3) for w in dense])
        t4, t16 = time_replays(g4, 10, 3) / len(mats), time_replays(g16, 10, 3) / len(mats)
        out["packed4_backbone_2048x2048"].append({
            "tokens": T, "nibbles_us": round(t4 * 1e3, 2), "fp16_us": round(t16 * 1e3, 2),
            "nibbles_gbs": round(packed[0].nbytes / (t4 * 1e-3) / 1e9, 1), "fp16_gbs": round(dense[0].numel() * 2 / (t16 * 1e-3) / 1e9, 1)})
        del g4, g16
    del mats, packed, dense
    torch.cuda.empty_cache()
    # host link peak: one large copy from pinned host memory by the copy engine (what the pager, which reads
    # the same kind of buffer from inside a kernel, is compared with)
    pinned = torch.empty((256 << 20,), dtype=torch.uint8, pin_memory=True)
    pinned.fill_(1)
    landing = torch.empty_like(pinned, device=device)
    h0, h1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    best = 0.0
    for _ in range(4):
        h0.record()
        landing.copy_(pinned, non_blocking=True)
        h1.record()
        torch.cuda.synchronize()
        best = max(best, pinned.numel() / (h0.elapsed_time(h1) * 1e-3) / 1e9)
    out["host_to_device_copy_gbs"] = round(best, 2)
    del pinned, landing

    def stack_cycled(shape, layers, distinct, seed, **kw):
        """`layers` blocks built from `distinct` synthetic layers (each block gets its own pinned host copy)."""
        made = [synth.synth_layer(shape, seed=seed + l, **kw) for l in range(distinct)]
        blocks = []
        for l in range(layers):
            layer = made[l % distinct]
            fresh = lambda p: {k: (v.clone() if isinstance(v, torch.Tensor) else v) for k, v in layer[p].items()}
            blk = tm.TrisSparseMoeBlock(shape.hidden_size, shape.intermediate_size, shape.num_experts, shape.top_k, True)
            blk.load_grouped_payloads(fresh("gate"), fresh("up"), fresh("down"), layer["shared_gate"], layer["shared_up"],
                                      layer["shared_down"], layer["router_weight"], device=device)
            blocks.append(blk)
        return blocks

    # BASELINE config 4 (streaming): a Qwen3.5-35B-A3B-shaped stack of 40 layers (256 experts, top-8, hidden 2048,
    # intermediate 512), batch 1 and 16; and the 8-layer OLMoE-shaped stack
    for prefix, shape, n_layers, distinct in (("streaming_qwen35_40_layers_", synth.QWEN35, 40, 4), ("streaming_", synth.OLMOE, 8, 8)):
        for mode, fmt_gr in (("bitmap", False), ("payload", True)):
            blocks = stack_cycled(shape, n_layers, distinct, 700, keep_sparse_gmap=not fmt_gr, use_block_gr=fmt_gr)
            manager = staging.GroupedQGmapCPUStagingManager(blocks, mode=mode)
            manager.initialize()
            out[prefix + mode] = streaming_records(blocks, manager, shape, device)
            for blk in blocks:
                blk.raise_on_kernel_status()
            del blocks, manager
            torch.cuda.empty_cache()
    print(json.dumps(out))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--ncu-case", default=None, choices=["layer", "grouped", "packed4"],
                    help="run a short untimed launch sequence for a profiler capture and exit")
    ap.add_argument("--extra", action="store_true", help="run the secondary workloads (prefill, Mixtral shape, streaming)")
    ap.add_argument("--layers", type=int, default=LAYERS, help="layers for --ncu-case")
    ap.add_argument("--tokens", type=int, default=HEADLINE_TOKENS, help="decode batch for --ncu-case")
    ap.add_argument("--tc-min-rows", type=int, default=None,
                    help="rows per expert segment above which the tcgen05 grouped kernel is used (library default 2048)")
    args = ap.parse_args()
    if args.tc_min_rows is not None and args.impl == "ours":
        import trismoe_b200 as tm

        tm._native.load().tris_set_grouped_tc_min_rows(int(args.tc_min_rows))
    args.warmup = max(args.warmup, 3)
    if args.ncu_case:
        return run_ncu_case(args)
    if args.extra:
        return run_extra(args)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
