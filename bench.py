#!/usr/bin/env python
"""Benchmark of the Hyena convolution hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload mr|se|li|li_pc|cc1d|decode_mr|decode_se|decode_li|decode_stack]

Default workload: Hyena-MR grouped causal FIR prefill, B=4, L=8192, D=4096, bf16 I/O with fp32
accumulation, 128-tap filters shared by groups of 16 channels, featurizer and gates fused, prefill
caches written (seeded synthetic data).  A step is one pass of the fused block over the whole batch.
With N > 1 the SAME problem is cut into N channel shards (strong scaling: rank r owns the hidden channels
`sharding.channel_range(D, G, N, r)`; decode workloads cut the batch instead).  Channels are independent, so
the block itself needs no exchange and its output stays sharded, as a row-parallel output projection
consumes it; the all-gather over NCCL that a replicated projection would need instead is measured in the
same run and reported under `collective`, alone and behind the kernel.  `--scaling weak` gives every rank a
full-width problem of its own instead.

Prints ONE JSON line (rank 0).  `value` is measured with the inputs resident in HBM; `e2e` goes
through the public API with pinned host buffers, host<->device copies inside the timed region.
`--impl reference` times the reference's CPU path (torch F.conv1d / torch.fft restated in
oracle/torch_port.py) on the host cores.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (B, L, D, G, K, io, description)
    "mr": dict(B=4, L=8192, D=4096, G=256, K=128, io="bf16", seed=1,
               name="hyena_mr_prefill B=4 L=8192 D=4096 bf16 (featurizer3 + gate + 128-tap grouped FIR + gate)"),
    "se": dict(B=4, L=8192, D=4096, G=256, K=7, io="bf16", seed=1,
               name="hyena_se_prefill B=4 L=8192 D=4096 bf16 (featurizer3 + gate + 7-tap grouped FIR + gate)"),
    "li": dict(B=1, L=131072, D=4096, G=256, K=0, io="bf16", seed=2,
               name="hyena_li_prefill B=1 L=131072 D=4096 bf16 (featurizer3 + gate + 16-pole modal filter + gate)"),
    # the same block through the drop-in engine, as the reference's HyenaCascade.parallel_forward calls it
    # (model.py:233-291): parallel_fir(gate=False) -> z [B, 3D, L], then parallel_fir(gate=True) on it -> y [B, D, L].
    # Per hidden channel and token: featurizer 6 bytes in + 6 out, gate-conv-gate 6 in + 2 out.  Plain q | k | v split
    # (a model with config.interleave adds its own interleave() copy between the two calls).
    "mr_dropin": dict(B=4, L=8192, D=4096, G=256, K=128, io="bf16", seed=1, dropin=True,
                      name="hyena_mr_prefill through the drop-in engine B=4 L=8192 D=4096 bf16 (parallel_fir featurizer + "
                           "parallel_fir gate / 128-tap grouped FIR / gate, z [B,3D,L] materialised between them)"),
    # configuration 1: the reference's own CPU-runnable case, fp32, small enough for L2 (25 MB per step): the steps
    # replay from a CUDA graph with a buffer larger than L2 written between them
    "se_cfg1": dict(B=1, L=2048, D=768, G=48, K=7, io="f32", seed=0, layout="split",
                    name="hyena_se_prefill B=1 L=2048 D=768 fp32 (configuration 1: featurizer3 + gate + 7-tap grouped FIR + gate)"),
    # the long-filter layer as Evo 2 has it (configs/evo2-7b-8k.yml: hcl_filter_groups == hidden size): 16 real poles
    # per CHANNEL, at the 7B prefill shape of configuration 2
    "li_pc": dict(B=4, L=8192, D=4096, G=4096, K=0, io="bf16", seed=2, real_poles=True,
                  name="hyena_li_prefill B=4 L=8192 D=4096 bf16 (featurizer3 + gate + modal long conv, 16 real poles per "
                       "channel + skip, state after the last token)"),
    # the featurizer as the conv extension's operator runs it (causal_conv1d_fn on the channel-last view [B,3D,L] of
    # the projection rows, width 3, no activation): 2 bytes in + 2 bytes out per packed channel and token
    # backward of the gate-conv-gate operator at configuration 2's operator-only size: (bs, l, g, dg) = (4, 8192, 256, 16)
    # operands x, B, C (the three thirds of one [B, L, 3D] tensor), dy and the saved filter output y2 in, dx, dB, dC, dh out
    "gcg_bwd": dict(B=4, L=8192, D=4096, G=256, K=128, io="bf16", seed=1, cc1d=True, bwd=True,
                    name="hyena_ops gate-conv-gate BACKWARD (two_pass_bwd_grouped) B=4 L=8192 D=4096 bf16, 128 taps, groups of 16"),
    "cc1d": dict(B=4, L=8192, D=4096, G=256, K=3, io="bf16", seed=1, cc1d=True,
                 name="causal_conv1d_fwd B=4 L=8192 channels=12288 bf16 channel-last (width-3 depthwise causal conv)"),
    # one-token decode of one Hyena layer (one launch): a step = B tokens; fp32 caches as after the first decode step
    "decode_mr": dict(B=64, L=1, D=4096, G=256, K=128, io="bf16", seed=3, decode=True,
                      name="hyena_mr_decode B=64 D=4096 bf16 (one layer, one token: featurizer + 128-tap FIR caches)"),
    "decode_se": dict(B=64, L=1, D=4096, G=256, K=7, io="bf16", seed=3, decode=True,
                      name="hyena_se_decode B=64 D=4096 bf16 (one layer, one token: featurizer + 7-tap FIR caches)"),
    "decode_li": dict(B=64, L=1, D=4096, G=256, K=0, io="bf16", seed=3, decode=True,
                      name="hyena_li_decode B=64 D=4096 bf16 (one layer, one token: featurizer cache + 16 complex modal states)"),
    # one token through the 27 Hyena layers of an Evo 2 7B-shaped stack (9 SE, 9 MR, 9 LI; the 5 attention layers, the
    # projections and the MLPs are not part of the path): 27 launches per step, every layer with caches of its own
    "decode_stack": dict(B=64, L=1, D=4096, G=256, K=-1, io="bf16", seed=3, decode=True, stack=True,
                         name="hyena_decode_stack B=64 D=4096 bf16 (one token through 9 SE + 9 MR + 9 LI layers, "
                              "reference cache layout: fp32 caches, 16 real modal states per channel)"),
    # configuration 4's Hyena share end to end: the 27 Hyena layers of an Evo 2 7B-shaped stack prefill a prompt of 8192
    # tokens for 64 sequences through engine.fused_prefill (which fills the reference's cache containers), then 512
    # decode steps run through engine.fused_decode on those caches (attention, projections and MLPs are not part of
    # the path).  One "step" of this workload is one decode step of the whole batch through the 27 layers.
    "evo2_7b_hyena": dict(B=64, L=8192, D=4096, G=256, K=-1, io="bf16", seed=3, decode=True, stack=True, harness=True,
                          name="Evo 2 7B-shaped Hyena stack (9 SE + 9 MR + 9 LI with 16 real poles per channel): prefill of "
                               "64 x 8192 tokens through engine.fused_prefill, then decode steps through engine.fused_decode "
                               "on the caches the prefill left"),
    # configuration 5's Hyena share: the 42 Hyena layers of an Evo 2 40B-shaped stack (14 SE + 14 MR + 14 LI, hidden size
    # 8192, `configs/evo2-40b-1m.yml`) prefill ONE sequence of 1,048,576 tokens through engine.fused_prefill, the hidden
    # channels cut into N shards of whole filter groups (no collective: projections, attention and MLPs are not part of
    # the path).  One "step" is one prefill of the whole stack.
    "evo2_40b_hyena": dict(B=1, L=1048576, D=8192, G=512, K=-1, io="bf16", seed=4, stack=True, harness=True, n_each=14,
                           prefill_only=True,
                           name="Evo 2 40B-shaped Hyena stack (14 SE + 14 MR + 14 LI with 16 real poles per channel, hidden 8192): "
                                "prefill of one sequence of 1,048,576 tokens through engine.fused_prefill, channel-sharded"),
}


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def make_inputs(w, device, dtype=None):
    dtype = dtype or (torch.float32 if w.get("io") == "f32" else torch.bfloat16)
    g = torch.Generator().manual_seed(w["seed"])
    B, L, D, G, K = w["B"], w["L"], w["D"], w["G"], w["K"]
    p = {}
    if w.get("stack"):
        return make_stack(w, g, dtype)
    # generated in slices to bound host memory; values ~ N(0, 1)
    p["u"] = torch.empty(B, L, 3 * D, dtype=dtype)
    for b in range(B):
        for t0 in range(0, L, 65536):
            t1 = min(L, t0 + 65536)
            p["u"][b, t0:t1] = torch.randn(t1 - t0, 3 * D, generator=g).to(dtype)
    p["w3"] = (torch.randn(3 * D, 1, 3, generator=g) / 3 ** 0.5).to(dtype)
    if K > 0:
        wt = torch.randn(G, 1, K, generator=g) / K ** 0.5
        if K >= 128:
            alpha = 0.01 + 0.09 * torch.rand(G, 1, 1, generator=g)
            wt = wt * torch.exp(-alpha * torch.arange(K)[None, None])
        p["h"] = wt.to(dtype)
        p["Dp"] = torch.zeros(D, dtype=dtype) if K >= 128 else None
    else:
        p["log_poles"] = torch.log(0.9 + 0.099 * torch.rand(G, 16, generator=g))[..., None]
        p["residues"] = torch.randn(G, 16, generator=g)
        p["theta"] = p["res_im"] = None
        if not w.get("real_poles"):
            p["theta"] = torch.pi * torch.rand(G, 16, generator=g)
            p["res_im"] = torch.randn(G, 16, generator=g)
        p["Dp"] = torch.randn(D, generator=g).to(dtype)
    if w.get("decode"):
        # caches as a decode step leaves them (fp32); several sets, used in turn, so that the timed steps stream
        # their caches from HBM instead of finding them in the 126 MB L2
        p["D"] = D
        per_set = B * 3 * D * 2 * 4 + (B * D * (K - 1) * 4 if K > 0 else B * D * 16 * 2 * 4)
        nsets = max(2, min(32, -(-300_000_000 // per_set)))
        p["sets"] = []
        for _ in range(nsets):
            c = {"fir_state": torch.randn(B, 3 * D, 2, generator=g)}
            if K > 0:
                c["inner_state"] = torch.randn(B, D, K - 1, generator=g)
            else:
                c["iir_state"] = torch.randn(B, D, 16, 2, generator=g)
            p["sets"].append(c)
        p["turn"] = [0]
    return p


# layer kinds of the 27 Hyena layers in the order of the 7B block pattern (short, medium, long; attention left out)
STACK_KINDS = ["se", "mr", "li"] * 9


def make_stack(w, g, dtype):
    """Parameters and caches of the Hyena layers of an Evo 2 7B-shaped stack, as a decode step finds them."""
    B, D, G = w["B"], w["D"], w["G"]
    p = {"u": torch.randn(B, 1, 3 * D, generator=g).to(dtype), "D": D, "layers": []}
    for kind in STACK_KINDS:
        c = {"kind": kind, "w3": (torch.randn(3 * D, 1, 3, generator=g) / 3 ** 0.5).to(dtype),
             "fir_state": torch.randn(B, 3 * D, 2, generator=g)}
        if kind == "li":
            # the reference's live form: real poles and residues per channel, state [B, D, 16] fp32
            c["log_poles"] = torch.log(0.9 + 0.099 * torch.rand(D, 16, generator=g))[..., None]
            c["residues"] = torch.randn(D, 16, generator=g)
            c["Dp"] = torch.randn(D, generator=g).to(dtype)
            c["iir_state"] = torch.randn(B, D, 16, generator=g)
        else:
            K = 7 if kind == "se" else 128
            wt = torch.randn(G, 1, K, generator=g) / K ** 0.5
            c["h"] = wt.to(dtype)
            c["Dp"] = torch.zeros(D, dtype=dtype) if kind == "mr" else None
            c["inner_state"] = torch.randn(B, D, K - 1, generator=g)
        p["layers"].append(c)
    return p


def run_harness(a, w, full, dev, rank, world, config, max_over_ranks, barrier):
    """Configuration 4, Hyena share: prefill then cached decode through the engine's fused entry points on the
    reference's cache containers, batch-sharded (every cache is per sequence: no collective)."""
    from vortex_b200 import HyenaInferenceEngine, ops
    from vortex_b200.cache import HyenaCascadeFIRInferenceParams, HyenaCascadeIIRInferenceParams
    B, L, D, G = w["B"], w["L"], w["D"], w["G"]
    g = torch.Generator(device=dev).manual_seed(w["seed"] + 1000 * rank)
    gc = torch.Generator().manual_seed(w["seed"])
    dims = (D, 1, D, 16, G)
    layers = []
    kinds = ["se", "mr", "li"] * w.get("n_each", 9)
    for i, kind in enumerate(kinds):
        c = {"kind": kind, "eng": HyenaInferenceEngine(layer_idx=i),
             "w3": (torch.randn(3 * D, 1, 3, generator=gc) / 3 ** 0.5).bfloat16().to(dev)}
        if kind == "li":
            c["kw"] = dict(log_poles=torch.log(0.9 + 0.099 * torch.rand(D, 16, generator=gc))[..., None].to(dev),
                           residues=torch.randn(D, 16, generator=gc).to(dev), D=torch.randn(D, generator=gc).bfloat16().to(dev))
        else:
            K = 7 if kind == "se" else 128
            c["kw"] = dict(h=(torch.randn(G, 1, K, generator=gc) / K ** 0.5).bfloat16().to(dev),
                           D=torch.zeros(D, dtype=torch.bfloat16, device=dev) if kind == "mr" else None)
        layers.append(c)
    fir_cache, iir_cache = HyenaCascadeFIRInferenceParams(), HyenaCascadeIIRInferenceParams()
    # one projection output stands for every layer's (values do not matter to the kernels' speed)
    u = torch.empty(B, L, 3 * D, device=dev, dtype=torch.bfloat16)
    for b0 in range(B):
        for t0 in range(0, L, 8192):
            u[b0, t0:t0 + 8192] = torch.randn(min(8192, L - t0), 3 * D, device=dev, generator=g).bfloat16()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def prefill():
        for c in layers:
            ip = iir_cache if c["kind"] == "li" else fir_cache
            y = c["eng"].fused_prefill(u, c["w3"], None, dims, inference_params=ip, **c["kw"])
        return y

    prefill()
    ops.device_status()
    n_pre = max(1, min(a.steps, 3))
    c0 = ops.launch_count()
    with ClockSampler(int(os.environ.get("LOCAL_RANK", "0"))) as cs_pre:
        barrier()
        ev0.record()
        for _ in range(n_pre):
            y = prefill()
        ev1.record()
        barrier()
    launches_pre = ops.launch_count() - c0
    ms_prefill = max_over_ranks(ev0.elapsed_time(ev1)) / n_pre
    assert bool(torch.isfinite(y[:, -4096:].float()).all())
    pre_bytes = algorithmic_bytes(dict(w, decode=False, prefill_only=True, n_each=w.get("n_each", 9)))
    del y
    # the share of each kind of layer: its layers alone, timed the same way
    per_kind = {}
    for kind in ("se", "mr", "li"):
        mine = [c for c in layers if c["kind"] == kind]
        barrier()
        ev0.record()
        for c in mine:
            c["eng"].fused_prefill(u, c["w3"], None, dims, inference_params=iir_cache if kind == "li" else fir_cache, **c["kw"])
        ev1.record()
        barrier()
        per_kind[kind] = max_over_ranks(ev0.elapsed_time(ev1)) / len(mine)
    if w.get("prefill_only"):
        if rank != 0:
            return None
        peak, peak_kind = _peaks()
        return {
            "metric": "hyena_prefill_throughput", "value": full["B"] * L / (ms_prefill * 1e-3), "unit": "tok/s", "n_gpus": world,
            "steps": n_pre, "warmup": 1, "ms_per_step": ms_prefill, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": config, "clocks": cs_pre.summary(),
            "gpu_launches": launches_pre,
            "roofline": {"bound": "hbm", "achieved": pre_bytes / (ms_prefill * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
                         "frac": pre_bytes / (ms_prefill * 1e-3) / 1e9 / peak, "traffic": None, "peak_kind": f"of {peak_kind}",
                         "algorithmic_bytes_per_launch": pre_bytes,
                         "note": "per rank and prefill of the whole stack (one fused launch per FIR layer, three per "
                                 "per-channel long-filter layer): 8 bytes per hidden channel and token plus the caches"},
            "ms_per_layer": per_kind, "collective": None, "e2e": None,
        }
    tok = torch.randn(B, 3 * D, device=dev, generator=g).bfloat16()

    def decode_step():
        for c in layers:
            ip = iir_cache if c["kind"] == "li" else fir_cache
            yd = c["eng"].fused_decode(tok, c["w3"], None, dims, ip, **c["kw"])
        return yd


    for _ in range(max(a.warmup, 3)):
        decode_step()                       # (the first step turns the prefill's bf16 caches into fp32 ones)
    ops.device_status()
    # the timed steps replay from one CUDA graph (as a serving loop would run them), so that the device, not the Python
    # caller, sets the pace; the caches the captured steps hand from one to the next live in the graph's pool
    graph, how = None, "replayed from one CUDA graph"
    c0 = ops.launch_count()
    try:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                for _ in range(a.steps):
                    yd = decode_step()
        torch.cuda.current_stream().wait_stream(side)
        launches = ops.launch_count() - c0
        graph.replay()
        torch.cuda.synchronize()
    except Exception as e:      # capture refused: time the eager loop and say so
        graph, how = None, f"launched from Python without a graph ({type(e).__name__}): host launch time is inside the figure"
        torch.cuda.synchronize()
    with ClockSampler(int(os.environ.get("LOCAL_RANK", "0"))) as cs:
        barrier()
        if graph is None:
            c0 = ops.launch_count()
        ev0.record()
        if graph is not None:
            graph.replay()
        else:
            for _ in range(a.steps):
                yd = decode_step()
        ev1.record()
        barrier()
    if graph is None:
        launches = ops.launch_count() - c0
    ms = max_over_ranks(ev0.elapsed_time(ev1))
    assert bool(torch.isfinite(yd.float()).all())
    if rank != 0:
        return None
    peak, peak_kind = _peaks()
    ms_step = ms / a.steps
    step_bytes = decode_bytes(dict(w, stack=True))
    tokens = full["B"]
    kinds = None
    return {
        "metric": "hyena_decode_throughput", "value": tokens / (ms_step * 1e-3), "unit": "tok/s", "n_gpus": world,
        "steps": a.steps, "warmup": max(a.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": config, "clocks": cs.summary(),
        "gpu_launches": launches,
        "roofline": {"bound": "hbm", "achieved": step_bytes / (ms_step * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
                     "frac": step_bytes / (ms_step * 1e-3) / 1e9 / peak, "traffic": None, "peak_kind": f"of {peak_kind}",
                     "algorithmic_bytes_per_launch": step_bytes,
                     "note": f"per rank and decode step (27 launches, {how}): every cache read and written once"},
        "prefill": {"ms": ms_prefill, "ms_per_layer": per_kind, "tokens_per_s": full["B"] * L / (ms_prefill * 1e-3),
                    "frac_of_hbm_peak_per_rank": pre_bytes / (ms_prefill * 1e-3) / 1e9 / peak,
                    "note": "27 layers, one fused launch each (three for the per-channel long filter), caches written"},
        "collective": None, "e2e": None,
    }


def decode_bytes(w):
    """Algorithmic HBM bytes of one decode launch: every cache element read and written once, plus the token."""
    B, D, K = w["B"], w["D"], w["K"]
    if w.get("stack"):
        per = {"se": B * D * 6 * 4, "mr": B * D * 127 * 4, "li": B * D * 16 * 4}
        return sum(2 * (B * 3 * D * 2 * 4 + per[k]) + B * 3 * D * 2 + B * D * 2 for k in STACK_KINDS)
    cache = B * 3 * D * 2 * 4 + (B * D * (K - 1) * 4 if K > 0 else B * D * 16 * 2 * 4)
    return 2 * cache + B * 3 * D * 2 + B * D * 2


def algorithmic_bytes(w):
    """HBM bytes one step has to move.  Prefill: 3 reads + 1 write of 2-byte elements per hidden channel and token, plus
    the caches when they are written (featurizer rows, and the inner FIR samples or the fp32 modal state); the conv
    extension's operator: 2 in + 2 out per packed channel; decode: every cache element read and written once."""
    if w.get("decode"):
        return decode_bytes(w)
    B, L, D, K = w["B"], w["L"], w["D"], w["K"]
    if w.get("prefill_only"):
        return sum(8 * B * D * L + B * 3 * D * 4 + (B * D * 16 * 4 if k == "li" else B * D * ((7 if k == "se" else 128) - 1) * 2)
                   for k in ["se", "mr", "li"] * w["n_each"])
    if w.get("bwd"):
        return 16 * B * D * L            # dy, x, B, C, y2 in; dx, dB, dC out (2 bytes each)
    if w.get("cc1d"):
        return 12 * B * D * L
    if w.get("dropin"):
        return 20 * B * D * L + (B * 3 * D * 2 * 2 + B * D * (K - 1) * 2 if w.get("caches") else 0)
    n = (16 if w.get("io") == "f32" else 8) * B * D * L
    if w.get("caches"):
        n += B * 3 * D * 2 * 2
        n += B * D * (K - 1) * 2 if K > 0 else B * D * 16 * 4 * (1 if w.get("real_poles") else 2)
    return n


def run_block(name, pc, u=None):
    """One step through the public API; returns y [B, L, D]."""
    from vortex_b200 import hyena_ops, ops
    u = pc["u"] if u is None else u
    if name == "decode_stack":
        un = u[:, 0]
        for c in pc["layers"]:
            if c["kind"] == "li":
                y = ops.decode_layer(un, c["w3"], None, c["fir_state"], pc["D"], log_poles=c["log_poles"],
                                     residues=c["residues"], iir_state=c["iir_state"], bias=c["Dp"])[0]
            else:
                y = ops.decode_layer(un, c["w3"], None, c["fir_state"], pc["D"], h=c["h"], inner_state=c["inner_state"],
                                     bias=c["Dp"], flip_filter=c["kind"] == "mr", gated_bias=c["kind"] == "mr")[0]
        return y
    if name.startswith("decode"):
        un = u[:, 0]
        c = pc["sets"][pc["turn"][0] % len(pc["sets"])]
        pc["turn"][0] += 1
        if name == "decode_li":
            return ops.decode_layer(un, pc["w3"], None, c["fir_state"], pc["D"], log_poles=pc["log_poles"],
                                    residues=pc["residues"], iir_state=c["iir_state"], theta=pc["theta"],
                                    res_im=pc["res_im"], bias=pc["Dp"])[0]
        return ops.decode_layer(un, pc["w3"], None, c["fir_state"], pc["D"], h=pc["h"], inner_state=c["inner_state"],
                                bias=pc["Dp"], flip_filter=name == "decode_mr", gated_bias=name == "decode_mr")[0]
    if name == "gcg_bwd":
        B, L, D3 = u.shape
        D, G = D3 // 3, pc["h"].shape[0]
        if "dy" not in pc:
            g = torch.Generator(device=u.device).manual_seed(5)
            pc["dy"] = torch.randn(B, L, D, device=u.device, generator=g).to(u.dtype)
            pc["y2"] = torch.randn(B, L, D, device=u.device, generator=g).to(u.dtype)
        v4 = lambda t: t.unflatten(2, (G, D // G))  # noqa: E731
        return hyena_ops.two_pass_bwd_grouped(v4(pc["dy"]), v4(u[..., :D]), v4(u[..., D:2 * D]), v4(u[..., 2 * D:]), pc["h"],
                                              v4(pc["y2"]))[0].flatten(2)
    if name == "cc1d":
        return hyena_ops.causal_conv1d_fn(u.transpose(1, 2), pc["w3"].reshape(-1, 3))
    caches = bool(pc.get("caches"))
    if name == "mr_dropin":
        import torch.nn.functional as F
        eng, D, G = pc["engine"], pc["u"].shape[-1] // 3, pc["h"].shape[0]
        dims = (D, 1, D, 16, G)
        ip = True if caches else None
        z, _ = eng.parallel_fir(F.conv1d, u, pc["w3"], None, u.shape[1], dims=dims, gate=False, inference_params=ip)
        y, _ = eng.parallel_fir(F.conv1d, z, pc["hx"], pc["Dp"], u.shape[1], dims=dims, gate=True, gated_bias=True,
                                dim_last=False, fir_length=pc["h"].shape[-1], inference_params=ip, groups=G)
        return y
    if name == "se_cfg1":
        return hyena_ops.hyena_se_fwd(u, pc["w3"], None, pc["h"], layout="split", want_state=caches)[0]
    if name == "mr":
        return hyena_ops.hyena_mr_fwd(u, pc["w3"], None, pc["h"], pc["Dp"], want_state=caches)[0]
    if name == "se":
        return hyena_ops.hyena_se_fwd(u, pc["w3"], None, pc["h"], want_state=caches)[0]
    return hyena_ops.hyena_li_fwd(u, pc["w3"], None, pc["log_poles"], pc["residues"], pc["Dp"], theta=pc["theta"],
                                  res_im=pc["res_im"], want_state=caches)[0]


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.index)], stdout=subprocess.PIPE, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *a):
        if self.proc:
            time.sleep(0.25)
            self.proc.terminate()
            self.t.join(timeout=2)

    def summary(self):
        mhz = sorted(int(r[0]) for r in self.rows if r and r[0].isdigit())
        if not mhz:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) > 2 + i and r[2 + i] == "Active" for r in self.rows)]
        mx = [int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()]
        return {"sm_mhz": mhz[len(mhz) // 2], "sm_max_mhz": max(mx) if mx else None, "reasons": reasons,
                "samples": len(mhz)}


def cpu_baseline(name, w, steps=1, warmup=1, cap_s=25.0):
    """The reference's CPU path (oracle/torch_port.py) on a bounded channel slice, scaled to the full width."""
    from oracle import torch_port as TP
    # all the host threads this process may use (a launcher such as torchrun presets OMP_NUM_THREADS=1)
    try:
        torch.set_num_threads(max(torch.get_num_threads(), len(os.sched_getaffinity(0))))
    except (AttributeError, RuntimeError):
        pass
    torch.manual_seed(0)
    Ds = min(w["D"], {"mr": 256, "se": 256, "li": 64, "li_pc": 64, "cc1d": 256, "mr_dropin": 256, "se_cfg1": 768, "gcg_bwd": 256}[name])
    B, L, D, G, K = w["B"], w["L"], w["D"], w["G"], w["K"]
    Gs = max(1, G * Ds // D)
    dt = torch.float32 if w.get("io") == "f32" else torch.bfloat16
    u = torch.randn(B, L, 3 * Ds).to(dt)
    w3 = (torch.randn(3 * Ds, 1, 3) / 3 ** 0.5).to(dt)
    if w.get("bwd"):
        # autograd through the reference's forward math (F.conv1d on the gated product, ref_fwd.py:80-127)
        hb = (torch.randn(Gs, 1, K) / K ** 0.5).to(dt).repeat_interleave(Ds // Gs, 0).float()
        xs, Bs, Cs = (u[..., i * Ds:(i + 1) * Ds].float().transpose(1, 2).contiguous().requires_grad_(True) for i in range(3))
        dy = torch.randn(B, Ds, L)

        def step():
            y = Cs * torch.nn.functional.conv1d(Bs * xs, hb, groups=Ds, padding=K - 1)[..., :L]
            return torch.autograd.grad(y, (xs, Bs, Cs), dy)[0]
    elif w.get("cc1d"):
        def step():
            return TP.featurizer(u, w3)[0]
    elif K > 0:
        h = (torch.randn(Gs, 1, K) / K ** 0.5).to(dt)
        Dp = torch.zeros(Ds, dtype=dt)

        def step():
            z, _ = TP.featurizer(u, w3)
            return TP.gate_conv_gate(z, h, Dp if K >= 128 else None, Ds, K, layout="interleaved", gated_bias=K >= 128)[0]
    else:
        lp = torch.log(0.9 + 0.099 * torch.rand(Ds, 16, 1))
        R = torch.randn(Ds, 16)
        Dp = torch.randn(Ds).to(dt)

        def step():
            z, _ = TP.featurizer(u, w3)
            hh = TP.modal_filter(lp, R, L)
            return TP.long_conv_gate(z, hh, Dp, Ds, layout="interleaved")[0]
    for _ in range(max(1, warmup)):
        step()
    # every step timed; the figure is the mean over the steps (a 25 s cap keeps the default run short)
    times = []
    t_all = time.perf_counter()
    for _ in range(max(1, steps)):
        t0 = time.perf_counter()
        step()
        times.append(time.perf_counter() - t0)
        if cap_s and time.perf_counter() - t_all > cap_s:
            break
    best = sum(times) / len(times)
    full = best * (D / Ds)
    return {"value": B * L / full, "unit": "tok/s", "cores": torch.get_num_threads(), "kind": "port",
            "extrapolated": Ds != D, "slice_ms": best * 1e3, "slice_channels": Ds, "scale": D / Ds,
            "sample": f"{Ds} of {D} channels (B={B}, L={L}) measured ({best * 1e3:.1f} ms, mean of {len(times)} passes) "
                      f"and scaled by {D // Ds}x (channels are independent); "
                      f"torch {torch.__version__} F.conv1d/torch.fft on {os.cpu_count()} host cpus"}, full


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="mr", choices=sorted(WORKLOADS))
    ap.add_argument("--scaling", default="strong", choices=["strong", "weak"],
                    help="N > 1: strong = one problem cut into N channel (prefill) or batch (decode) shards (the all-gather "
                         "of the block output is measured apart); weak = a full-size problem per rank")
    ap.add_argument("--no-caches", action="store_true", help="prefill workloads: do not write the prefill caches")
    ap.add_argument("--batch", type=int, default=0, help="override the batch size (small cases for profiling)")
    ap.add_argument("--seq", type=int, default=0, help="override the sequence length (small cases for profiling)")
    ap.add_argument("--channels", type=int, default=0, help="override the hidden channels (the shard of one GPU)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    a = ap.parse_args()
    a.warmup = max(a.warmup, 3) if a.impl == "ours" else a.warmup
    w = dict(WORKLOADS[a.workload])
    if a.batch > 0:
        w["B"] = a.batch
        w["name"] += f" [batch overridden to {a.batch}]"
    if a.seq > 0:
        w["L"] = a.seq
        w["name"] += f" [sequence length overridden to {a.seq}]"
    if a.channels > 0:
        w["G"] = max(1, w["G"] * a.channels // w["D"])
        w["D"] = a.channels
        w["name"] += f" [hidden channels overridden to {a.channels}]"
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    prefill = not w.get("decode") and not w.get("cc1d")
    w["caches"] = prefill and not a.no_caches
    strong = world > 1 and a.scaling == "strong"
    full = dict(w)                      # the whole problem; w becomes this rank's share of it
    from vortex_b200 import sharding
    if strong:
        if w.get("decode"):
            b0, b1 = sharding.batch_range(full["B"], world, rank)
            w["B"] = b1 - b0
        else:
            d0, d1 = sharding.channel_range(full["D"], full["G"], world, rank)
            w["D"], w["G"] = d1 - d0, (d1 - d0) // (full["D"] // full["G"])
    tokens = full["B"] * full["L"] if strong else world * w["B"] * w["L"]      # whole-job tokens per step
    step_bytes = algorithmic_bytes(w)
    if world == 1:
        how = "one GPU holds the whole problem"
    elif not strong:
        how = f"weak: each of {world} ranks runs a full-size problem of its own, no collective"
    elif w.get("decode"):
        how = (f"strong, batch shards: the {full['B']} sequences are cut into {world} shards of {w['B']}; every cache is "
               "per sequence, so there is no collective on the data path")
    else:
        how = (f"strong, channel shards: the {full['D']} hidden channels are cut into {world} shards of whole filter "
               f"groups ({w['D']} on this rank); the block needs no exchange and y stays sharded for a row-parallel "
               "output projection (the all-gather a replicated projection would need is measured under `collective`)")
    config = {"workload": full["name"], "seed": full["seed"], "qkv_layout": "interleaved", "sharding": how,
              "caches": bool(w["caches"]),
              "l2": (f"{step_bytes / 1e6:.0f} MB of caches and tokens per step and rank" +
                     (", caches rotate over sets larger than L2" if not w.get("stack") else "")
                     if w.get("decode") else
                     f"inputs and outputs of a rank ({step_bytes / 1e6:.0f} MB per step) " +
                     ("are larger than the 126 MB L2" if step_bytes > 2 * 126e6 else
                      "fit the 126 MB L2: a buffer larger than L2 is written between timed steps"))}

    if a.impl == "reference":
        if rank != 0:
            return
        # the reference's CPU path on the host cores: every step is one pass over a bounded channel slice of the
        # whole (un-sharded) workload; throughput is scaled to the full width
        cb, _ = cpu_baseline(a.workload, full, steps=max(1, a.steps), warmup=max(1, a.warmup), cap_s=0)
        line = {"impl": "reference", "metric": "hyena_prefill_throughput", "value": cb["value"], "unit": "tok/s",
                "n_gpus": a.gpus, "steps": a.steps, "warmup": a.warmup, "ms_per_step": cb["slice_ms"],
                "ms_per_step_full_width": cb["slice_ms"] * cb["scale"], "extrapolated": cb["extrapolated"],
                "higher_is_better": True, "scaling": "strong" if strong or world == 1 else "weak", "vs_baseline": None,
                "dtype": "bf16", "data": "synthetic", "config": config, "cpu_baseline": cb,
                "e2e": {"value": cb["value"], "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(line))
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (the product path has no CPU fallback)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        if os.environ.get("NCCL_DEBUG", "").upper() in ("", "VERSION"):
            os.environ["NCCL_DEBUG"] = "WARN"      # keep the version banner off stdout: one JSON line only
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        if dist is None:
            return ms
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    if w.get("harness"):
        p, pc = {}, {}
    elif strong and prefill:
        # every rank builds the same seeded problem and keeps its own channels (contiguous copies of the slices)
        pfull = make_inputs(full, dev)
        p = sharding.shard_block({k: v for k, v in pfull.items() if torch.is_tensor(v) or v is None},
                                 full["D"], full["G"], world, rank, layout="interleaved")
        p = {k: (v.contiguous() if torch.is_tensor(v) else v) for k, v in p.items()}
        del pfull
    else:
        p = make_inputs(dict(w, seed=w["seed"] + (1000 * rank if world > 1 else 0)), dev)
    pc = {k: (v.to(dev) if torch.is_tensor(v) else v) for k, v in p.items()}
    for key in ("sets", "layers"):
        if key in pc:
            pc[key] = [{k: (v.to(dev) if torch.is_tensor(v) else v) for k, v in c.items()} for c in pc[key]]
    if w.get("harness"):
        line = run_harness(a, w, full, dev, rank, world, config, max_over_ranks, barrier)
        if line is not None:
            print(json.dumps(line))
        if dist is not None:
            dist.destroy_process_group()
        return
    pc["caches"] = w["caches"]
    from vortex_b200 import ops
    if w.get("dropin"):
        from vortex_b200 import HyenaInferenceEngine
        pc["engine"] = HyenaInferenceEngine()
        pc["hx"] = pc["h"].repeat_interleave(w["D"] // w["G"], 0)       # what the caller hands over (model.py:261-262)

    gather = None
    if strong and prefill:
        widths = [hi - lo for lo, hi in (sharding.channel_range(full["D"], full["G"], world, r) for r in range(world))]
        recv = torch.empty(world, w["B"], w["L"], max(widths), device=dev, dtype=torch.bfloat16)

        def gather(y):
            return sharding.gather_channels(y, widths=widths, out=recv, concat=False)

    flush = None
    if not w.get("decode") and step_bytes <= 2 * 126e6:
        flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)     # written between steps: evicts the 126 MB L2

    def step():
        return run_block(a.workload, pc)

    def step_gathered():
        return gather(run_block(a.workload, pc))

    for _ in range(a.warmup):
        y = step()
    ops.device_status()
    c0 = ops.launch_count()
    y = step()
    launches_per_step = ops.launch_count() - c0      # the library's own count of the kernels one step launches
    barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    graph = None
    if w.get("decode"):
        # a decode step is one short launch: replay the timed steps from a CUDA graph (as a serving loop would), so
        # that the device, not the Python caller, sets the pace
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                for _ in range(a.steps):
                    y = run_block(a.workload, pc)
        torch.cuda.current_stream().wait_stream(side)
        graph.replay()
        torch.cuda.synchronize()

    def timed(fn, n):
        """n calls of fn between two events on the current stream; with a flush buffer every call is timed on its own
        (the flush in between is not counted)."""
        if flush is None:
            barrier()
            ev0.record()
            for _ in range(n):
                fn()
            ev1.record()
            barrier()
            return max_over_ranks(ev0.elapsed_time(ev1))
        total = 0.0
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(n)]
        barrier()
        for e0, e1 in evs:
            flush.fill_(1)
            e0.record()
            fn()
            e1.record()
        barrier()
        for e0, e1 in evs:
            total += e0.elapsed_time(e1)
        return max_over_ranks(total)

    with ClockSampler(local) as cs:
        if graph is not None:
            ms = timed(graph.replay, 1)
        else:
            ms = timed(step, a.steps)
    ms_step = ms / a.steps
    value = tokens / (ms_step * 1e-3)
    collective = None
    if gather is not None:
        # The block output stays sharded in `value`: a row-parallel output projection consumes its rank's channels as
        # they are, and the exchange that follows (an all-reduce of the projection's result) belongs to that GEMM.  The
        # other boundary -- a replicated projection, which needs y gathered on every rank -- is measured here on the
        # same buffers: the all-gather alone, and the step with the all-gather behind the kernel.
        step_gathered()
        ms_g = timed(step_gathered, a.steps) / a.steps
        y_sh = run_block(a.workload, pc)
        ms_c = timed(lambda: gather(y_sh), a.steps) / a.steps
        nrecv = recv.numel() * 2 * (world - 1) // world
        collective = {"op": "all_gather", "backend": "nccl", "in_value": False, "bytes_received_per_rank": nrecv,
                      "ms": ms_c, "recv_GBps_per_rank": nrecv / (ms_c * 1e-3) / 1e9,
                      "ms_per_step_kernel_then_collective": ms_g, "value_with_collective": tokens / (ms_g * 1e-3),
                      "limiter": "collective" if ms_c > ms_step else "kernel",
                      "note": "every rank has to receive (N-1)/N of y: at 770 GB/s per direction that alone takes "
                              f"{nrecv / 770e9 * 1e3:.3f} ms per step, against {ms_step:.3f} ms of kernel"}

    # ---- end to end: pinned host input -> device -> kernel -> pinned host output, every step
    e2e = None
    if not a.no_e2e and not w.get("decode"):
        hu = p["u"].pin_memory()
        y1 = run_block(a.workload, pc)
        hy = [torch.empty(y1.shape, dtype=y1.dtype).pin_memory() for _ in range(2)]
        du = [torch.empty_like(pc["u"]) for _ in range(2)]
        main_s, s_in, s_out = torch.cuda.current_stream(), torch.cuda.Stream(), torch.cuda.Stream()
        ev_in = [torch.cuda.Event() for _ in range(2)]
        ev_k = [torch.cuda.Event() for _ in range(2)]
        ev_o = [torch.cuda.Event() for _ in range(2)]

        def e2e_steps(n):
            # every step: pinned host input -> device (copy stream), kernel (main stream), output -> pinned host (copy
            # stream); two buffers, so the copies of neighbouring steps overlap the kernel and each other.  With
            # channel shards every rank moves its own columns in and its own slice of y out: the host assembles.
            for i in range(n):
                j = i % 2
                with torch.cuda.stream(s_in):
                    if i >= 2:
                        s_in.wait_event(ev_k[j])            # the kernel that read this input buffer is done
                    du[j].copy_(hu, non_blocking=True)
                    ev_in[j].record(s_in)
                main_s.wait_event(ev_in[j])
                yy = run_block(a.workload, pc, du[j])
                ev_k[j].record(main_s)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(ev_k[j])
                    if i >= 2:
                        s_out.wait_event(ev_o[j])
                    hy[j].copy_(yy, non_blocking=True)
                    yy.record_stream(s_out)
                    ev_o[j].record(s_out)
            main_s.wait_stream(s_out)
            main_s.wait_stream(s_in)

        e2e_steps(2)
        barrier()
        n_e2e = max(3, min(a.steps, 10))
        ev0.record()
        e2e_steps(n_e2e)
        ev1.record()
        barrier()
        ms_e = max_over_ranks(ev0.elapsed_time(ev1))
        e2e = {"value": tokens / (ms_e / n_e2e * 1e-3), "unit": "tok/s",
               "h2d_bytes_per_step": hu.numel() * hu.element_size(), "d2h_bytes_per_step": hy[0].numel() * hy[0].element_size(),
               "bytes_are": "per rank", "steps": n_e2e}

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return
    peak, peak_kind = _peaks()
    achieved = step_bytes / (ms_step * 1e-3) / 1e9
    traffic = NCU_TRAFFIC.get(a.workload)
    if traffic is not None:
        traffic = traffic * step_bytes / algorithmic_bytes(dict(WORKLOADS[a.workload], caches=w["caches"]))
    line = {
        "metric": "hyena_decode_throughput" if w.get("decode") else "hyena_prefill_throughput", "value": value, "unit": "tok/s", "n_gpus": world, "steps": a.steps,
        "warmup": a.warmup, "ms_per_step": ms_step, "higher_is_better": True,
        "scaling": "weak" if (world > 1 and not strong) else "strong", "vs_baseline": None,
        "dtype": "f32" if w.get("io") == "f32" else "bf16", "data": "synthetic", "config": config, "clocks": cs.summary(),
        "gpu_launches": launches_per_step * a.steps,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": traffic, "peak_kind": f"of {peak_kind}",
                     "algorithmic_bytes_per_launch": step_bytes,
                     "note": "per rank: achieved = algorithmic bytes of the rank's share / kernel time per step (the "
                             f"collective, if any, is reported apart); one step = {launches_per_step} kernel launch(es)"},
        "collective": collective,
        "e2e": e2e,
    }
    if not a.no_cpu_baseline and world == 1 and not w.get("decode"):
        line["cpu_baseline"] = cpu_baseline(a.workload, full, steps=3)[0]
    print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


# kernel launches of ours per step of each workload
# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel, from the ncu captures
# summarised under profiles/ (None until captured)
NCU_TRAFFIC = {"mr": 1.026e9, "se": 1.024e9, "mr_dropin": 2.407e9, "li": 4.13e9, "cc1d": 1.44e9}   # small-case captures scaled by the units of a bench launch

if __name__ == "__main__":
    main()
