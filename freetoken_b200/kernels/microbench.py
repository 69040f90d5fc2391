"""Times one kernel at a time at given sizes and reports it against its roofline.

    python -m freetoken_b200.kernels.microbench moe --experts 256 --tokens 8 [--hidden 3072 --inter 1536 --top-k 8]
    python -m freetoken_b200.kernels.microbench attention --batch 8 --context 2048
    python -m freetoken_b200.kernels.microbench attention --prefill 2048
    python -m freetoken_b200.kernels.microbench sample --rows 8 --vocab 200064
    python -m freetoken_b200.kernels.microbench few --tokens 1
    python -m freetoken_b200.kernels.microbench sparse --batch 8 --context 32768
    python -m freetoken_b200.kernels.microbench sparse --prefill 2048 --context 32768
    python -m freetoken_b200.kernels.microbench attention --prefill 2048 --tied --dist-bias 200
    python -m freetoken_b200.kernels.microbench rows --tokens 2048 --hidden 3072
    python -m freetoken_b200.kernels.microbench attention --prefill 2048 --window 1024 --sink
    python -m freetoken_b200.kernels.microbench gla --prefill 2048 [--heads 16 --dim 128 --vdim 128]
    python -m freetoken_b200.kernels.microbench gla --batch 8
    python -m freetoken_b200.kernels.microbench kekopel --tokens 2048 [--batch 8]
    python -m freetoken_b200.kernels.microbench attention --prefill 2048 --tied --kv-heads 1 --window 1024 --head-sinks
    python -m freetoken_b200.kernels.microbench nusudra --tokens 2048 [--batch 8]
    python -m freetoken_b200.kernels.microbench attention --prefill 2048 --dist-bias 2048 --head-sinks

Each case allocates its inputs once (larger than L2 where the real workload is), warms up, then
times ``--iters`` launches with CUDA events and prints one JSON line: time, the bytes the kernel has
to move (or its flops), and the fraction of the HBM or tensor peak that this is.  ``--profile`` brackets
a few launches with cudaProfilerStart/Stop for ``ncu --profile-from-start off`` on a small case.
The reference reports per-kernel bandwidth the same way (python/freetoken/benchmark/perf.py:60-74).
"""

from __future__ import annotations

import argparse
import json
import os
import sys

import torch

from ..engine.attention_plan import TC_ONE_TILE_COSTS, TC_TWO_TILE_COSTS, build_plan, wave_splits
from . import ops

HBM_GBS = 6650.0  # used when no measured peaks are on file
BF16_TFLOPS = 1590.0
_PEAKS = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "..", "MEASURED_PEAKS.json")
if os.path.isfile(_PEAKS):  # the copy rate and library product rate measured on this machine's GPUs
    try:
        with open(_PEAKS) as _f:
            _m = json.load(_f)
        HBM_GBS = float(_m.get("hbm_gbs", HBM_GBS))
        BF16_TFLOPS = float(_m.get("bf16_tflops", BF16_TFLOPS))
    except (OSError, ValueError):
        pass


def _time(fn, iters: int, warmup: int, profile: bool) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if profile:
        torch.cuda.profiler.start()
        for _ in range(min(iters, 3)):
            fn()
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
        return float("nan")
    # the launches are replayed from a CUDA graph so that the figure is device time, not the
    # Python call overhead of issuing them
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(iters):
            fn()
    graph.replay()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    graph.replay()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / iters * 1e3  # microseconds


def bench_moe(a) -> dict:
    dev = "cuda"
    ops.set_moe_pairs(not getattr(a, "no_pairs", False))
    E, H, I, k, T = a.experts, a.hidden, a.inter, a.top_k, a.tokens
    g = torch.Generator(device=dev).manual_seed(0)
    w1 = torch.empty(E, 2 * I, H, dtype=torch.bfloat16, device=dev).normal_(0, 0.02, generator=g)
    w2 = torch.empty(E, H, I, dtype=torch.bfloat16, device=dev).normal_(0, 0.02, generator=g)
    ids = torch.stack([torch.randperm(E, device=dev, generator=g)[:k] for _ in range(T)]).to(torch.int32)
    counts = torch.empty(E, dtype=torch.int32, device=dev)
    off = torch.empty(E + 1, dtype=torch.int32, device=dev)
    routes = torch.empty(T * k, dtype=torch.int32, device=dev)
    pos = torch.empty(T * k, dtype=torch.int32, device=dev)
    ops.moe_permute(ids, E, counts, off, routes, pos)
    h = torch.randn(T, H, device=dev, generator=g).to(torch.bfloat16)
    x = torch.empty(T * k, H, dtype=torch.bfloat16, device=dev)
    ops.moe_gather(h, routes, k, x)
    act = torch.empty(T * k, I, dtype=torch.bfloat16, device=dev)
    y = torch.empty(T * k, H, dtype=torch.bfloat16, device=dev)
    wts = torch.rand(T * k, device=dev)
    distinct = int((counts > 0).sum())
    out = {}
    for name, fn, wbytes, flops in (
            ("gemm1", lambda: ops.moe_gemm1_act(x, w1, off, "silu", 1.702, 7.0, act), distinct * 2 * I * H * 2,
             2 * T * k * 2 * I * H),
            ("gemm1_gather", (lambda: ops.moe_gemm1_act_gather(h, routes, k, w1, off, "silu", 1.702, 7.0, act))
             if ops.moe_gemm1_gather_fits(torch.bfloat16, H, I, E, T * k) else None,
             distinct * 2 * I * H * 2, 2 * T * k * 2 * I * H),
            ("gemm2", lambda: ops.moe_gemm2(act, w2, off, routes, wts, y), distinct * H * I * 2, 2 * T * k * H * I)):
        if (a.only and a.only != name) or fn is None:
            continue
        us = _time(fn, a.iters, a.warmup, a.profile)
        out[name] = {"us": round(us, 2), "weight_bytes": wbytes, "gbs": round(wbytes / us / 1e3, 1),
                     "hbm_frac": round(wbytes / us / 1e3 / HBM_GBS, 3),
                     "tflops": round(flops / us / 1e6, 1), "tensor_frac": round(flops / us / 1e6 / BF16_TFLOPS, 3)}
    out["distinct_experts"] = distinct
    out["status"] = ops.read_status()
    return out


def bench_attention(a) -> dict:
    dev = "cuda"
    Hq, Hkv, D, P = a.q_heads, a.kv_heads, a.head_dim, a.page_size
    G = Hq // Hkv
    if a.prefill:
        segs = [(a.prefill, a.past + a.prefill)]  # a portion of a prompt after --past earlier tokens
    else:
        segs = [(1, a.context)] * a.batch
    n_pages = sum(-(-kv // P) for _, kv in segs) + 1
    g = torch.Generator(device=dev).manual_seed(0)
    ks = torch.empty(n_pages, Hkv, P, D, dtype=torch.bfloat16, device=dev).normal_(0, 1, generator=g)
    tied = bool(getattr(a, "tied", False))  # the values are the keys: one slab, read once where the kernel can
    vs = ks if tied else torch.empty(n_pages, Hkv, P, D, dtype=torch.bfloat16, device=dev).normal_(0, 1, generator=g)
    n_bias = int(getattr(a, "dist_bias", 0) or 0)  # entries per head of a bias by distance
    bias = torch.randn(Hq, n_bias, device=dev, generator=g) if n_bias else None
    width = max(-(-kv // P) for _, kv in segs)
    bt = torch.zeros(len(segs), width, dtype=torch.int32)
    info, q0, page = [], 0, 1
    for row, (ql, kv) in enumerate(segs):
        n = -(-kv // P)
        bt[row, :n] = torch.arange(page, page + n)
        page += n
        info.append([q0, ql, kv, row])
        q0 += ql
    bt = bt.to(dev)
    seg = torch.tensor(info, dtype=torch.int32, device=dev)
    q = torch.randn(q0, Hq, D, device=dev, generator=g).to(torch.bfloat16)
    fixed = None
    window = int(getattr(a, "window", 0) or 0) or None  # a sliding window
    sink = 0.0 if getattr(a, "sink", False) else None  # a sink of logit 0 in the softmax's denominator
    if getattr(a, "head_sinks", False):  # a logit per query head
        sink = torch.randn(Hq, device=dev, generator=g)
    special = window is not None or sink is not None  # of the tcgen05 kernels the one with 128-row tiles takes these
    no_tc = a.no_tc
    tile = 128 if (a.prefill >= 128 and not no_tc and ops.attention_tc_fits(D, P, G)) else 64
    if tile == 128 and a.pair and bias is None and not special:
        tile = 256  # two query tiles per CTA
    few_rows = False
    if not a.prefill:
        few_rows = a.few_rows and not no_tc and not special and ops.attention_tc_few_fits(D, P, G)
        tc = few_rows or (a.tc and not no_tc and not special and ops.attention_tc_fits(D, P, G))
        fixed = wave_splits(len(segs) * Hkv, 148 if tc else 2 * 148, 16, a.context) if a.splits is None else a.splits
        tile = 16 if few_rows else 128 if tc else (16 if G <= 16 else 64)
    tensor_core = few_rows or tile >= 128  # (one CTA per SM: the engine plans these for half as many CTA slots)
    costs = None
    if tile >= 128 and fixed is None:  # as the engine plans these kernels' work lists
        costs = TC_TWO_TILE_COSTS if tile == 256 else TC_ONE_TILE_COSTS
    plan = build_plan(segs, G, tile, window, Hkv, sm_count=74 if tensor_core else 148, fixed_splits=fixed,
                      key_tile=128 if tensor_core else 0, costs=costs)
    items = torch.from_numpy(plan.items).to(dev)
    po = pm = None
    if plan.n_slots:
        po = torch.empty(plan.n_slots, Hkv, tile, D, dtype=torch.float32, device=dev)
        pm = torch.empty(plan.n_slots, Hkv, tile, 2, dtype=torch.float32, device=dev)
    out = torch.empty_like(q)
    us = _time(lambda: ops.paged_attention(q, ks, vs, bt, seg, len(segs), items, plan.n_items, po, pm, out, tile,
                                           D ** -0.5, window, few_rows=few_rows, dist_bias=bias, sink=sink), a.iters,
               a.warmup, a.profile)
    seen = [(ql, kv if window is None else min(kv, window - 1 + ql)) for ql, kv in segs]  # keys a segment's queries can see
    kv_bytes = sum(kv for _, kv in seen) * Hkv * D * 2 * (1 if tied else 2)
    pairs = lambda ql, kv: sum(min(kv - ql + t + 1, window or (1 << 60)) for t in range(ql))  # noqa: E731  (query, key) pairs
    flops = sum(4 * pairs(ql, kv) * Hq * D for ql, kv in segs)
    return {"us": round(us, 2), "tile_rows": tile, "tied": tied, "dist_bias": n_bias, "window": window, "sink": sink is not None,
            "items": plan.n_items,
            "est_us": None if plan.est_us is None else round(plan.est_us, 1), "kv_bytes": kv_bytes, "gbs": round(kv_bytes / us / 1e3, 1),
            "hbm_frac": round(kv_bytes / us / 1e3 / HBM_GBS, 3), "tflops": round(flops / us / 1e6, 1),
            "tensor_frac": round(flops / us / 1e6 / BF16_TFLOPS, 3)}


def bench_rows(a) -> dict:
    """The row-wise kernels around the 32-bit stream: RMSNorm with the residual sum, Dynamic Tanh with two
    addends (a parallel layer's), and the head store with norm + rotation or with bias + position factor."""
    dev = "cuda"
    T, H = a.tokens, a.hidden
    Hq, Hkv, D, P = a.q_heads, a.kv_heads, a.head_dim, 16
    g = torch.Generator(device=dev).manual_seed(0)
    bf = torch.bfloat16
    res = torch.randn(T, H, device=dev, generator=g)
    x1, x2 = (torch.randn(T, H, device=dev, generator=g).to(bf) for _ in range(2))
    out = torch.empty(T, H, dtype=bf, device=dev)
    w, b, alpha = torch.ones(H, device=dev), torch.zeros(H, device=dev), torch.full((1,), 0.5, device=dev)
    results = {}

    def add(name, fn, nbytes):
        us = _time(fn, a.iters, a.warmup, a.profile)
        results[name] = {"us": round(us, 2), "bytes": nbytes, "gbs": round(nbytes / us / 1e3, 1),
                         "hbm_frac": round(nbytes / us / 1e3 / HBM_GBS, 3)}

    add("add_rmsnorm", lambda: ops.add_rmsnorm(x1, res, w, 1e-6, False, out), T * H * (4 + 4 + 2 + 2))
    add("stream_add_norm (dynamic tanh, two addends)",
        lambda: ops.stream_add_norm(res, out, x1=x1, x2=x2, norm=("dynamic_tanh", w, b, alpha)), T * H * (4 + 4 + 2 + 2 + 2))
    rows = (Hq + 2 * Hkv) * D
    qkv = torch.randn(T, rows, device=dev, generator=g).to(bf)
    q = torch.empty(T, Hq, D, dtype=bf, device=dev)
    n_pages = -(-T // P) + 1
    slab_k, slab_v = (torch.zeros(n_pages, Hkv, P, D, dtype=bf, device=dev) for _ in range(2))
    slots = torch.arange(P, P + T, dtype=torch.int32, device=dev)
    positions = torch.arange(T, dtype=torch.int32, device=dev)
    rd = D // 2
    table = torch.randn(T, rd, device=dev, generator=g)
    nw = torch.ones(D, device=dev)
    add("norm_rope_store (norm, rotation, k and v)", lambda: ops.norm_rope_store(qkv, D, rd, positions, table, 1e-6, False, [
        dict(first_head=0, n_heads=Hq, norm_weight=nw, rotate=True, dense_out=q),
        dict(first_head=Hq, n_heads=Hkv, norm_weight=nw, rotate=True, slab=slab_k, slot_map=slots),
        dict(first_head=Hq + Hkv, n_heads=Hkv, norm_weight=None, rotate=False, slab=slab_v, slot_map=slots)]),
        T * (Hq + 2 * Hkv) * D * 2 * 2)
    qb, kb = torch.randn(Hq * D, device=dev, generator=g), torch.randn(Hkv * D, device=dev, generator=g)
    factors = torch.rand(T, device=dev, generator=g) + 1
    add("norm_rope_store (bias, position factor, k only)", lambda: ops.norm_rope_store(qkv, D, 0, positions, None, 0.0, False, [
        dict(first_head=0, n_heads=Hq, norm_weight=None, rotate=False, dense_out=q, bias=qb, pos_scale=factors),
        dict(first_head=Hq, n_heads=Hkv, norm_weight=None, rotate=False, slab=slab_k, slot_map=slots, bias=kb)]),
        T * (Hq + Hkv) * D * 2 * 2)
    o = torch.randn(T, Hq, D, device=dev, generator=g).to(bf)
    gates = torch.randn(T, Hq, device=dev, generator=g).to(bf)
    add("head_gate", lambda: ops.head_gate(o, gates), T * Hq * D * 2 * 2)
    # a sub-layer's output through a norm of its own into the stream, and the stream's norm, in one pass
    add("postnorm_add_norm", lambda: ops.postnorm_add_norm(x1, None, w, 1e-6, True, res, w, 1e-6, True, out),
        T * H * (2 + 4 + 4 + 2))
    wide = torch.randn(T, Hq * D, device=dev, generator=g).to(bf)
    add("gated_heads (sigmoid gate, element by element, in place)", lambda: ops.gated_heads(o, wide, o, D, "sigmoid"),
        T * Hq * D * 2 * 3)
    o32 = torch.randn(T, Hq, D, device=dev, generator=g)
    add("gated_heads (32-bit input, head norm, silu gate)", lambda: ops.gated_heads(o32, wide, o, D, "silu", nw, 1e-6),
        T * Hq * D * (4 + 2 + 2))
    return results


def bench_gla(a) -> dict:
    """The recurrence of gated linear attention: a prompt of --prefill tokens (chunks side by side), or --batch
    requests with one token each (state in, state out).  Everything is 32-bit arithmetic on the CUDA cores: the
    figure beside the time is the recurrence's 5 D Dv operations per token and head against the nominal 32-bit
    rate (148 SMs x 128 lanes x 2 x the SM clock), and the bytes moved against the measured copy rate."""
    from ..parts.gla import chunk_list

    dev = "cuda"
    H, D, Dv = a.heads, a.dim, a.vdim
    segs = [(a.prefill, a.prefill)] if a.prefill else [(1, a.context)] * a.batch
    T = sum(q for q, _ in segs)
    g = torch.Generator(device=dev).manual_seed(0)
    bf = torch.bfloat16
    wide = (torch.randn(T, 2 * H * D + H * Dv, device=dev, generator=g) * 0.3).to(bf)
    q, k, v = wide[:, : H * D], wide[:, H * D: 2 * H * D], wide[:, 2 * H * D:]
    z = torch.randn(T, H * D, device=dev, generator=g) + 2.0
    zb = torch.zeros(H * D, device=dev)
    state = torch.zeros(len(segs) + 1, H, D, Dv, device=dev)
    info, q0 = [], 0
    for ql, kv in segs:
        info.append([q0, ql, kv, 0])
        q0 += ql
    seg = torch.tensor(info, dtype=torch.int32, device=dev)
    slots = torch.arange(1, len(segs) + 1, dtype=torch.int32, device=dev)
    chunks, per_seg, single, multi = chunk_list(segs, a.chunk)
    n = chunks.shape[0]
    carry = torch.empty(n, H, D, Dv, device=dev) if multi else None
    decay = torch.empty(n, H, D, device=dev) if multi else None
    out = torch.empty(T, H, Dv, device=dev)
    cd, pd = torch.from_numpy(chunks).to(dev), torch.from_numpy(per_seg).to(dev)
    us = _time(lambda: ops.gla_scan(q, k, v, z, zb, 16.0, D ** -0.5, state, slots, seg, len(segs), cd, n, pd, single, multi,
                                    carry, decay, out), a.iters, a.warmup, a.profile)
    passes = 2 if multi else 1  # a long portion runs the recurrence twice (contributions, then outputs)
    flops = T * H * D * Dv * (5 if not multi else 8)
    nbytes = T * (2 * H * D + H * Dv) * 2 * passes + T * H * D * 4 * passes + T * H * Dv * 4 + \
        (2 * len(segs) + (2 * n if multi else 0)) * H * D * Dv * 4
    fp32_tflops = 148 * 128 * 2 * 1.965e9 / 1e12
    return {"us": round(us, 2), "chunks": n, "launches": 4 if multi else 1, "flops": flops, "tflops": round(flops / us / 1e6, 2),
            "fp32_frac_nominal": round(flops / us / 1e6 / fp32_tflops, 3), "bytes": nbytes,
            "gbs": round(nbytes / us / 1e3, 1), "hbm_frac": round(nbytes / us / 1e3 / HBM_GBS, 3)}


def bench_kekopel(a) -> dict:
    """The kernels that the Kekopel layers add around the library products: the short convolution in front of a
    sub-layer, the sub-layer's norm into the stream, the mix over all layers' outputs, the latent-attention rows
    (norms, rotation, cache row; the queries' rotated part), the matrix memory's gates, inputs, recurrence (with the
    normaliser as one more value column) and output, the squared ReLU and the scaled expert inputs.  Attention over
    the latent rows is ``attention --tied --kv-heads 1 --window W --head-sinks``."""
    from ..parts.gla import chunk_list

    dev = "cuda"
    T, C, H, D, taps, depth = a.tokens, a.hidden, a.heads, a.head_dim, a.taps, a.depth
    decode = a.batch > 0
    segs = [(1, a.context)] * a.batch if decode else [(T, T)]
    T = sum(q for q, _ in segs)
    g = torch.Generator(device=dev).manual_seed(0)
    bf, f32 = torch.bfloat16, torch.float32
    info, q0 = [], 0
    for ql, kv in segs:
        info.append([q0, ql, kv, 0])
        q0 += ql
    seg = torch.tensor(info, dtype=torch.int32, device=dev)
    slots = torch.arange(1, len(segs) + 1, dtype=torch.int32, device=dev)
    n_slots = len(segs) + 1
    results = {}

    def add(name, fn, nbytes, flops=0):
        us = _time(fn, a.iters, a.warmup, a.profile)
        results[name] = {"us": round(us, 2), "bytes": nbytes, "gbs": round(nbytes / us / 1e3, 1),
                         "hbm_frac": round(nbytes / us / 1e3 / HBM_GBS, 3)}
        if flops:
            fp32_tflops = 148 * 128 * 2 * 1.965e9 / 1e12
            results[name].update(flops=flops, tflops=round(flops / us / 1e6, 2),
                                 fp32_frac_nominal=round(flops / us / 1e6 / fp32_tflops, 3))

    res = torch.randn(T, C, device=dev, generator=g)
    y = torch.randn(T, C, device=dev, generator=g).to(bf)
    out = torch.empty(T, C, dtype=bf, device=dev)
    cw = torch.randn(C, taps, device=dev, generator=g) * 0.3
    cstate = torch.zeros(n_slots, max(taps - 1, 1), C, device=dev)[:, : taps - 1]
    add("short_conv", lambda: ops.short_conv(res, cw, cstate if taps > 1 else None, slots, seg, len(segs), out),
        T * C * (4 + 2) + (2 * len(segs) * (taps - 1) * C * 4 if decode else 0))
    w = torch.ones(C, device=dev)
    add("postnorm_add_norm (a sub-layer's norm into the stream)",
        lambda: ops.postnorm_add_norm(y, None, w, 1e-6, False, res), T * C * (2 + 4 + 4))
    hist = torch.randn(depth + 1, T, C, device=dev, generator=g)
    mix = torch.rand(depth + 1, device=dev, generator=g)
    add(f"depth_mix (over {depth + 1} outputs)", lambda: ops.depth_mix(hist, depth, mix, res), T * C * 4 * (depth + 3))
    inter = a.inter
    act = torch.randn(T, inter, device=dev, generator=g).to(bf)
    add("relu2 (in place)", lambda: ops.relu2_(act), T * inter * 2 * 2)
    k_top = a.top_k
    routes = torch.randperm(T * k_top, device=dev, generator=g).to(torch.int32)
    wts = torch.rand(T * k_top, device=dev, generator=g)
    xin = torch.empty(T * k_top, C, dtype=bf, device=dev)
    add("moe_gather_scaled", lambda: ops.moe_gather_scaled(y, routes, wts, k_top, xin), T * C * 2 + T * k_top * C * 2)
    # latent attention
    qr, kr, rot, P = a.q_rank, a.kv_rank, a.rot_dim, 16
    pad = -(-(kr + rot) // 16) * 16
    proj = torch.randn(T, qr + kr + rot, device=dev, generator=g).to(bf)
    cq = torch.empty(T, qr, dtype=bf, device=dev)
    slab = torch.zeros(-(-T // P) + 1, 1, P, pad, dtype=bf, device=dev)
    slot_map = torch.arange(P, P + T, dtype=torch.int32, device=dev)
    positions = torch.arange(T, dtype=torch.int32, device=dev) if not decode else \
        torch.full((T,), a.context - 1, dtype=torch.int32, device=dev)
    table = torch.randn(max(T, a.context), rot, device=dev, generator=g)
    wq, wkv = torch.ones(qr, device=dev), torch.ones(kr, device=dev)
    add("latent_store", lambda: ops.latent_store(proj, qr, kr, rot, rot, True, wq, wkv, 1e-6, positions, table, cq, slab,
                                                 slot_map), T * ((qr + kr + rot) * 2 + qr * 2 + pad * 2))
    q = torch.randn(T, H, D + rot, device=dev, generator=g).to(bf)
    qa = torch.empty(T, H, pad, dtype=bf, device=dev)
    add("latent_query_rotate", lambda: ops.latent_query_rotate(q, D, rot, rot, True, positions, table, qa, kr),
        T * H * (rot * 2 + (pad - kr) * 2))
    # matrix memory
    Dv = a.vdim
    pre = torch.randn(T, 2 * H, device=dev, generator=g)
    bias = torch.randn(2 * H, device=dev, generator=g)
    m_state = torch.zeros(n_slots, H, device=dev)
    gi, zf, m = (torch.empty(T, H, device=dev) for _ in range(3))
    add("mlstm_gates", lambda: ops.mlstm_gates(pre, bias[:H], bias[H:], 12.0, m_state, slots, seg, len(segs), gi, zf, m),
        T * H * 4 * 5)
    wide = (torch.randn(T, H * (2 * D + 2 * Dv), device=dev, generator=g) * 0.3).to(bf)
    chunks, per_seg, single, multi = chunk_list(segs, a.chunk)
    n = chunks.shape[0]
    state = torch.zeros(n_slots, H, D, Dv + 1, device=dev)
    carry = torch.empty(n, H, D, Dv + 1, device=dev) if multi else None
    decay = torch.empty(n, H, D, device=dev) if multi else None
    o32, nq = torch.empty(T, H, Dv, device=dev), torch.empty(T, H, device=dev)
    cd, pd = torch.from_numpy(chunks).to(dev), torch.from_numpy(per_seg).to(dev)
    passes = 2 if multi else 1
    add("gla_scan (a key factor and a decay per head, the normaliser as a column of ones)",
        lambda: ops.gla_scan(wide[:, :H * D], wide[:, H * D:2 * H * D], wide[:, 2 * H * D:H * (2 * D + Dv)], None, None, 1.0,
                             D ** -0.5, state, slots, seg, len(segs), cd, n, pd, single, multi, carry, decay, o32,
                             k_fac=gi, a_head=zf, ones_col=True, out_ones=nq),
        T * H * ((2 * D + Dv) * 2 + 8) * passes + T * H * (Dv + 1) * 4 + (2 * len(segs) + (2 * n if multi else 0)) * H * D * (Dv + 1) * 4,
        T * H * D * (Dv + 1) * (8 if multi else 5))
    o = torch.empty(T, H * Dv, dtype=bf, device=dev)
    nw = torch.ones(H * Dv, device=dev)
    add("mlstm_output", lambda: ops.mlstm_output(o32, nq, m, wide[:, H * (2 * D + Dv):], nw, 1e-6, o),
        T * H * ((Dv + 1) * 4 + 4 + Dv * 2 * 2))
    results["status"] = ops.read_status()
    return results


def bench_nusudra(a) -> dict:
    """The kernels that the Nusudra layers add around the library products: the pass over the residual streams
    (write a sub-layer's result, read for the next one, norm), the token shift, the mean of the normed branches, the
    convolution of projected rows, the state-space layer's gates, recurrence (queries and keys shared by groups of
    heads) and output, and the delta rule.  Attention with a bias by distance and a sink per head is
    ``attention --dist-bias L --head-sinks``."""
    from ..parts.gla import chunk_list

    dev = "cuda"
    T, C, H, D, Dv, S = a.tokens, a.hidden, a.heads, a.head_dim, a.vdim, a.streams
    decode = a.batch > 0
    segs = [(1, a.context)] * a.batch if decode else [(T, T)]
    T = sum(q for q, _ in segs)
    g = torch.Generator(device=dev).manual_seed(0)
    bf, f32 = torch.bfloat16, torch.float32
    info, q0 = [], 0
    for ql, kv in segs:
        info.append([q0, ql, kv, 0])
        q0 += ql
    seg = torch.tensor(info, dtype=torch.int32, device=dev)
    slots = torch.arange(1, len(segs) + 1, dtype=torch.int32, device=dev)
    n_slots = len(segs) + 1
    results = {}
    fp32_tflops = 148 * 128 * 2 * 1.965e9 / 1e12

    def add(name, fn, nbytes, flops=0):
        us = _time(fn, a.iters, a.warmup, a.profile)
        results[name] = {"us": round(us, 2), "bytes": nbytes, "gbs": round(nbytes / us / 1e3, 1),
                         "hbm_frac": round(nbytes / us / 1e3 / HBM_GBS, 3)}
        if flops:
            results[name].update(flops=flops, tflops=round(flops / us / 1e6, 2),
                                 fp32_frac_nominal=round(flops / us / 1e6 / fp32_tflops, 3))

    streams = torch.randn(S, T, C, device=dev, generator=g)
    y = torch.randn(T, C, device=dev, generator=g).to(bf)
    mix, ow, iw = torch.rand(S, S, device=dev, generator=g), torch.rand(S, device=dev, generator=g), torch.rand(S, device=dev, generator=g)
    nw = torch.ones(C, device=dev)
    h32, h = torch.empty(T, C, device=dev), torch.empty(T, C, dtype=bf, device=dev)
    add(f"hyper_step (write, read and norm over {S} streams; 32-bit out)",
        lambda: ops.hyper_step(streams, y=y, mix=mix, out_w=ow, in_w=iw, norm_w=nw, eps=1e-6, h_out=h32),
        T * C * (2 * S * 4 + 2 + 4))
    add(f"hyper_step (write, read and norm over {S} streams)",
        lambda: ops.hyper_step(streams, y=y, mix=mix, out_w=ow, in_w=iw, norm_w=nw, eps=1e-6, h_out=h),
        T * C * (2 * S * 4 + 2 + 2))
    sw = torch.rand(C, 2, device=dev, generator=g)
    sstate = torch.zeros(n_slots, 1, C, device=dev)
    add("short_conv (token shift: two taps on the normed rows)",
        lambda: ops.short_conv(h32, sw, sstate, slots, seg, len(segs), h), T * C * (4 + 2) + (2 * len(segs) * C * 4 if decode else 0))
    y2 = torch.randn(T, C, device=dev, generator=g).to(bf)
    add("norm_mean (two branches)", lambda: ops.norm_mean([y, y2], [nw, nw], 1e-6, h), T * C * 2 * 3)
    # state space: inner = heads_ssm * 64, state N, groups
    Hs, P, N, G, taps = a.ssm_heads, 64, a.state, a.groups, a.taps
    inner, bc = Hs * P, G * N
    proj = (torch.randn(T, 2 * inner + 2 * bc + Hs, device=dev, generator=g) * 0.5).to(bf)
    cw = torch.randn(inner + 2 * bc, taps, device=dev, generator=g) * 0.3
    cb = torch.zeros(inner + 2 * bc, device=dev)
    cstate = torch.zeros(n_slots, taps - 1, inner + 2 * bc, device=dev)
    xbc = torch.empty(T, inner + 2 * bc, dtype=bf, device=dev)
    add("conv_act (bias, silu, on a view of the projection)",
        lambda: ops.conv_act(proj[:, inner:2 * inner + 2 * bc], cw, cb, "silu", cstate, slots, seg, len(segs), xbc),
        T * (inner + 2 * bc) * 4 + (2 * len(segs) * (taps - 1) * (inner + 2 * bc) * 4 if decode else 0))
    dtb, alog = torch.zeros(Hs, device=dev), torch.zeros(Hs, device=dev)
    step, dec = torch.empty(T, Hs, device=dev), torch.empty(T, Hs, device=dev)
    add("ssm_gates", lambda: ops.ssm_gates(proj[:, 2 * inner + 2 * bc:], dtb, alog, step, dec), T * Hs * (2 + 8))
    chunks, per_seg, single, multi = chunk_list(segs, a.chunk)
    n = chunks.shape[0]
    state = torch.zeros(n_slots, Hs, N, P, device=dev)
    carry = torch.empty(n, Hs, N, P, device=dev) if multi else None
    decay = torch.empty(n, Hs, N, device=dev) if multi else None
    o32 = torch.empty(T, Hs, P, device=dev)
    cd, pd = torch.from_numpy(chunks).to(dev), torch.from_numpy(per_seg).to(dev)
    passes = 2 if multi else 1
    add("gla_scan (state space: keys times a step size, a decay per head, q and k shared by groups of heads)",
        lambda: ops.gla_scan(xbc[:, inner + bc:], xbc[:, inner:inner + bc], xbc[:, :inner], None, None, 1.0, 1.0, state, slots,
                             seg, len(segs), cd, n, pd, single, multi, carry, decay, o32, k_fac=step, a_head=dec,
                             qk_div=Hs // G),
        T * Hs * ((2 * N + P) * 2 + 8) * passes + T * Hs * P * 4 + (2 * len(segs) + (2 * n if multi else 0)) * Hs * N * P * 4,
        T * Hs * N * P * (8 if multi else 5))
    dsk, snw = torch.ones(Hs, device=dev), torch.ones(inner, device=dev)
    yo = torch.empty(T, inner, dtype=bf, device=dev)
    add("ssm_output (skip, gate, norm in groups)",
        lambda: ops.ssm_output(o32, xbc[:, :inner], dsk, proj[:, :inner], snw, G, 1e-6, yo), T * inner * (4 + 2 * 3))
    # delta rule
    Gk = a.kv_heads
    dproj = (torch.randn(T, 2 * Gk * D + 2 * H * Dv + 2 * H, device=dev, generator=g) * 0.5).to(bf)
    dconv = 2 * Gk * D + H * Dv
    dw = torch.randn(dconv, taps, device=dev, generator=g) * 0.3
    dstate_c = torch.zeros(n_slots, taps - 1, dconv, device=dev)
    qkv = torch.empty(T, dconv, dtype=bf, device=dev)
    add("conv_act (no bias, silu: q, k, v of the delta rule)",
        lambda: ops.conv_act(dproj[:, :dconv], dw, None, "silu", dstate_c, slots, seg, len(segs), qkv), T * dconv * 4)
    dstate = torch.zeros(n_slots, H, Dv, D, device=dev)
    do32 = torch.empty(T, H, Dv, device=dev)
    al, db = torch.zeros(H, device=dev), torch.zeros(H, device=dev)
    add("delta_scan",
        lambda: ops.delta_scan(qkv[:, :Gk * D], qkv[:, Gk * D:2 * Gk * D], qkv[:, 2 * Gk * D:], dproj[:, -2 * H:-H], dproj[:, -H:],
                               al, db, D ** -0.5, 1e-6, dstate, slots, seg, len(segs), do32),
        T * H * ((2 * D + Dv) * 2 + 4) + T * H * Dv * 4 + 2 * len(segs) * H * D * Dv * 4, T * H * D * Dv * 6)
    o = torch.empty(T, H, Dv, dtype=bf, device=dev)
    hw = torch.ones(Dv, device=dev)
    add("gated_heads (head norm, silu gate)",
        lambda: ops.gated_heads(do32, dproj[:, dconv:dconv + H * Dv], o, Dv, "silu", hw, 1e-6), T * H * Dv * (4 + 2 + 2))
    results["status"] = ops.read_status()
    return results


def bench_few(a) -> dict:
    """The few-token kernels (``csrc/gemv.cu``) at the headline sizes: the qkv and output projections of
    ``--tokens`` tokens, and the routed gate/up and down products of their routes.  Six copies of the dense
    weights and other experts every launch, so that every launch reads its weights from memory."""
    dev = "cuda"
    H, I, E, k, T = a.hidden, a.inter, a.experts, a.top_k, a.tokens
    q_dim, kv_dim, copies = a.q_heads * a.head_dim, a.kv_heads * a.head_dim, 6
    g = torch.Generator(device=dev).manual_seed(0)
    wq = torch.empty(copies, q_dim + 2 * kv_dim, H, dtype=torch.bfloat16, device=dev).normal_(0, 0.02, generator=g)
    wo = torch.empty(copies, H, q_dim, dtype=torch.bfloat16, device=dev).normal_(0, 0.02, generator=g)
    w1 = torch.empty(E, 2 * I, H, dtype=torch.bfloat16, device=dev).normal_(0, 0.02, generator=g)
    w2 = torch.empty(E, H, I, dtype=torch.bfloat16, device=dev).normal_(0, 0.02, generator=g)
    x = torch.randn(T, H, device=dev, generator=g).to(torch.bfloat16)
    xo = torch.randn(T, q_dim, device=dev, generator=g).to(torch.bfloat16)
    qkv = torch.empty(T, q_dim + 2 * kv_dim, dtype=torch.bfloat16, device=dev)
    o = torch.empty(T, H, dtype=torch.bfloat16, device=dev)
    ids = [torch.stack([(torch.randperm(E, device=dev, generator=g)[:k]) for _ in range(T)]).to(torch.int32)
           for _ in range(copies)]
    wts = torch.rand(T, k, device=dev)
    act = torch.empty(T * k, I, dtype=torch.bfloat16, device=dev)
    y = torch.empty(T * k, H, dtype=torch.bfloat16, device=dev)
    turn = [0]

    def nxt():
        turn[0] = (turn[0] + 1) % copies
        return turn[0]

    cases = (
        ("qkv", lambda: ops.small_linear(x, wq[nxt()], qkv), (q_dim + 2 * kv_dim) * H * 2),
        ("out_proj", lambda: ops.small_linear(xo, wo[nxt()], o), H * q_dim * 2),
        ("gate_up", lambda: ops.moe_small_gate_up(x, ids[nxt()], w1, "silu", 1.702, 7.0, act), T * k * 2 * I * H * 2),
        ("down", lambda: ops.moe_small_down(act, ids[nxt()], wts, w2, y), T * k * H * I * 2))
    out = {}
    for name, fn, nbytes in cases:
        if a.only and a.only != name:
            continue
        us = _time(fn, a.iters, a.warmup, a.profile)
        out[name] = {"us": round(us, 2), "weight_bytes": nbytes, "gbs": round(nbytes / us / 1e3, 1),
                     "hbm_frac": round(nbytes / us / 1e3 / HBM_GBS, 3)}
    return out


def bench_sparse(a) -> dict:
    """The block-sparse layer kind at its real geometry (the reference's M3: blocks of 128 keys, 16 chosen
    blocks, 64 query heads on 4 KV heads of 128, one shared index key of 128 per token): block selection
    (index scores, forced blocks, top-k) and attention over the chosen blocks, for single tokens of
    ``--batch`` requests at ``--context`` tokens, or for a ``--prefill`` portion at the end of one request of
    ``--context`` tokens.  Bytes: the visible index keys once per request and step; the chosen keys and values
    per token and KV head."""
    dev = "cuda"
    Hq, Hkv, D, P, Di = a.q_heads, a.kv_heads, a.head_dim, a.page_size, a.head_dim
    block, topk = a.block, a.topk
    segs = [(a.prefill, a.context)] if a.prefill else [(1, a.context)] * a.batch
    n_pages = sum(-(-kv // P) for _, kv in segs) + 1
    g = torch.Generator(device=dev).manual_seed(0)
    ks = torch.empty(n_pages, Hkv, P, D, dtype=torch.bfloat16, device=dev).normal_(0, 1, generator=g)
    vs = torch.empty(n_pages, Hkv, P, D, dtype=torch.bfloat16, device=dev).normal_(0, 1, generator=g)
    iks = torch.empty(n_pages, 1, P, Di, dtype=torch.bfloat16, device=dev).normal_(0, 1, generator=g)
    width = max(-(-kv // P) for _, kv in segs)
    bt = torch.zeros(len(segs), width, dtype=torch.int32)
    info, q0, page = [], 0, 1
    for row, (ql, kv) in enumerate(segs):
        n = -(-kv // P)
        bt[row, :n] = torch.arange(page, page + n)
        page += n
        info.append([q0, ql, kv, row])
        q0 += ql
    bt, T = bt.to(dev), q0
    seg = torch.tensor(info, dtype=torch.int32, device=dev)
    q = torch.randn(T, Hq, D, device=dev, generator=g).to(torch.bfloat16)
    iq = torch.randn(T, Hkv, Di, device=dev, generator=g).to(torch.bfloat16)
    sel = torch.empty(T, Hkv, topk, dtype=torch.int32, device=dev)
    max_blocks = -(-a.context // block)
    out = {}
    scores = None
    if not a.no_tc and ops.sparse_score_fits(Hkv, Di, block):
        scores = torch.empty(T, Hkv, max_blocks, dtype=torch.float32, device=dev)
    us = _time(lambda: ops.sparse_select(iq, iks, bt, seg, len(segs), block, a.local, a.init, max_blocks, sel, scores,
                                         live_blocks=-(-a.context // block)),
               a.iters, a.warmup, a.profile)
    index_bytes = sum(kv for _, kv in segs) * Di * 2
    flops = sum(2 * (ql * kv - ql * (ql - 1) // 2) * Hkv * Di for ql, kv in segs)
    out["select"] = {"us": round(us, 2), "index_key_bytes": index_bytes, "gbs": round(index_bytes / us / 1e3, 1),
                     "hbm_frac": round(index_bytes / us / 1e3 / HBM_GBS, 3), "tflops": round(flops / us / 1e6, 2)}
    plan = build_plan(segs, Hq // Hkv, 16, None, Hkv, sparse=(block, topk))
    items = torch.from_numpy(plan.items).to(dev)
    po = pm = None
    if plan.n_slots:
        po = torch.empty(plan.n_slots, Hkv, 16, D, dtype=torch.float32, device=dev)
        pm = torch.empty(plan.n_slots, Hkv, 16, 2, dtype=torch.float32, device=dev)
    o = torch.empty_like(q)
    us = _time(lambda: ops.paged_attention(q, ks, vs, bt, seg, len(segs), items, plan.n_items, po, pm, o, 16, D ** -0.5,
                                           None, sel=sel, block_size=block), a.iters, a.warmup, a.profile)
    kv_bytes = sum(min(topk * block, kv - ql + t + 1) for ql, kv in segs for t in range(ql)) * Hkv * D * 2 * 2
    out["attend"] = {"us": round(us, 2), "items": plan.n_items, "kv_bytes": kv_bytes, "gbs": round(kv_bytes / us / 1e3, 1),
                     "hbm_frac": round(kv_bytes / us / 1e3 / HBM_GBS, 3)}
    return out


def bench_sample(a) -> dict:
    dev = "cuda"
    logits = torch.randn(a.rows, a.vocab, device=dev)
    temp = torch.full((a.rows,), a.temperature, device=dev)
    top_k = torch.zeros(a.rows, dtype=torch.int32, device=dev)
    top_p = torch.ones(a.rows, device=dev)
    u = torch.rand(a.rows, device=dev)
    out = torch.empty(a.rows, dtype=torch.int32, device=dev)
    us = _time(lambda: ops.sample(logits, temp, top_k, top_p, u, out), a.iters, a.warmup, a.profile)
    nbytes = a.rows * a.vocab * 4
    return {"us": round(us, 2), "bytes": nbytes, "gbs": round(nbytes / us / 1e3, 1)}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="microbench")
    sub = ap.add_subparsers(dest="case", required=True)
    for name in ("moe", "attention", "sample", "sparse", "few", "rows", "gla", "kekopel", "nusudra"):
        p = sub.add_parser(name)
        p.add_argument("--iters", type=int, default=20)
        p.add_argument("--warmup", type=int, default=5)
        p.add_argument("--profile", action="store_true")
        if name == "moe":
            p.add_argument("--experts", type=int, default=256)
            p.add_argument("--tokens", type=int, default=8)
            p.add_argument("--hidden", type=int, default=3072)
            p.add_argument("--inter", type=int, default=1536)
            p.add_argument("--top-k", type=int, default=8)
            p.add_argument("--only", choices=["gemm1", "gemm2"], default=None)
            p.add_argument("--no-pairs", action="store_true",
                           help="128- and 256-token tiles on the one-CTA form of the tcgen05 kernel instead of pairs of CTAs")
        elif name == "attention":
            p.add_argument("--batch", type=int, default=8)
            p.add_argument("--context", type=int, default=2048)
            p.add_argument("--prefill", type=int, default=0)
            p.add_argument("--past", type=int, default=0, help="tokens of the request before the --prefill portion")
            p.add_argument("--q-heads", type=int, default=48)
            p.add_argument("--kv-heads", type=int, default=8)
            p.add_argument("--head-dim", type=int, default=128)
            p.add_argument("--page-size", type=int, default=16)
            p.add_argument("--splits", type=int, default=None)
            p.add_argument("--no-tc", action="store_true", help="prefill on the mma.sync kernel instead of tcgen05")
            p.add_argument("--tc", action="store_true", help="decode on the tcgen05 kernel with 128-row query tiles")
            p.add_argument("--few-rows", action="store_true",
                           help="decode on the tcgen05 kernel in its form for tiles of at most 16 rows")
            p.add_argument("--pair", action="store_true", help="prefill on the tcgen05 kernel with two query tiles per CTA")
            p.add_argument("--tied", action="store_true", help="the values are the keys (one slab)")
            p.add_argument("--dist-bias", type=int, default=0, help="entries per head of a bias by distance (0 = none)")
            p.add_argument("--window", type=int, default=0, help="a sliding window of this many tokens (0 = none)")
            p.add_argument("--sink", action="store_true", help="a sink of logit 0 in the softmax's denominator")
            p.add_argument("--head-sinks", action="store_true", help="a sink with a logit of its own per query head")
        elif name == "rows":
            p.add_argument("--tokens", type=int, default=2048)
            p.add_argument("--hidden", type=int, default=3072)
            p.add_argument("--q-heads", type=int, default=48)
            p.add_argument("--kv-heads", type=int, default=8)
            p.add_argument("--head-dim", type=int, default=128)
        elif name == "kekopel":
            p.add_argument("--tokens", type=int, default=2048)
            p.add_argument("--batch", type=int, default=0, help="requests with one token each instead of one portion")
            p.add_argument("--context", type=int, default=2048)
            p.add_argument("--hidden", type=int, default=3072)
            p.add_argument("--inter", type=int, default=12288)
            p.add_argument("--top-k", type=int, default=8)
            p.add_argument("--heads", type=int, default=48)
            p.add_argument("--head-dim", type=int, default=128)
            p.add_argument("--vdim", type=int, default=128)
            p.add_argument("--q-rank", type=int, default=1536)
            p.add_argument("--kv-rank", type=int, default=192)
            p.add_argument("--rot-dim", type=int, default=64)
            p.add_argument("--taps", type=int, default=4)
            p.add_argument("--depth", type=int, default=3, help="outputs before this layer's that the mix reads")
            p.add_argument("--chunk", type=int, default=64)
        elif name == "nusudra":
            p.add_argument("--tokens", type=int, default=2048)
            p.add_argument("--batch", type=int, default=0, help="requests with one token each instead of one portion")
            p.add_argument("--context", type=int, default=2048)
            p.add_argument("--hidden", type=int, default=3072)
            p.add_argument("--streams", type=int, default=4)
            p.add_argument("--heads", type=int, default=48)
            p.add_argument("--kv-heads", type=int, default=8)
            p.add_argument("--head-dim", type=int, default=128)
            p.add_argument("--vdim", type=int, default=128)
            p.add_argument("--ssm-heads", type=int, default=48)
            p.add_argument("--state", type=int, default=128)
            p.add_argument("--groups", type=int, default=8)
            p.add_argument("--taps", type=int, default=4)
            p.add_argument("--chunk", type=int, default=64)
        elif name == "few":
            p.add_argument("--tokens", type=int, default=1)
            p.add_argument("--hidden", type=int, default=3072)
            p.add_argument("--inter", type=int, default=1536)
            p.add_argument("--experts", type=int, default=256)
            p.add_argument("--top-k", type=int, default=8)
            p.add_argument("--q-heads", type=int, default=48)
            p.add_argument("--kv-heads", type=int, default=8)
            p.add_argument("--head-dim", type=int, default=128)
            p.add_argument("--only", choices=["qkv", "out_proj", "gate_up", "down"], default=None)
        elif name == "gla":
            p.add_argument("--batch", type=int, default=8)
            p.add_argument("--context", type=int, default=2048)
            p.add_argument("--prefill", type=int, default=0)
            p.add_argument("--heads", type=int, default=16)
            p.add_argument("--dim", type=int, default=128)
            p.add_argument("--vdim", type=int, default=128)
            p.add_argument("--chunk", type=int, default=64)
        elif name == "sparse":
            p.add_argument("--batch", type=int, default=8)
            p.add_argument("--context", type=int, default=32768)
            p.add_argument("--prefill", type=int, default=0)
            p.add_argument("--q-heads", type=int, default=64)
            p.add_argument("--kv-heads", type=int, default=4)
            p.add_argument("--head-dim", type=int, default=128)
            p.add_argument("--page-size", type=int, default=16)
            p.add_argument("--block", type=int, default=128)
            p.add_argument("--topk", type=int, default=16)
            p.add_argument("--local", type=int, default=1)
            p.add_argument("--init", type=int, default=0)
            p.add_argument("--no-tc", action="store_true", help="block scores by a CTA per token and head instead of mma.sync")
        else:
            p.add_argument("--rows", type=int, default=8)
            p.add_argument("--vocab", type=int, default=200064)
            p.add_argument("--temperature", type=float, default=0.0)
    a = ap.parse_args(argv)
    res = {"moe": bench_moe, "attention": bench_attention, "sample": bench_sample, "sparse": bench_sparse, "few": bench_few,
           "rows": bench_rows, "gla": bench_gla, "kekopel": bench_kekopel, "nusudra": bench_nusudra}[a.case](a)
    print(json.dumps({"case": a.case, **{k: v for k, v in vars(a).items() if k != "case"}, "result": res}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
