"""Two larger workloads beside the headline benchmark, on the same layer sizes and random weights.

``long_contexts``: several requests with prompts of very different lengths (thousands to tens of
thousands of tokens) go through the scheduler, the prompts in portions beside the decoding of the
others, then every request decodes a few hundred tokens greedily.  Reported: prefill and decode
tokens a second, the high-water mark of the page pool.

``chunked_prefill``: one very long prompt is read in portions of a few hundred tokens, every step
beside one decoded token of many other requests.  Reported: tokens a second of the mixed steps, the
time of a step at the start and at the end of the prompt.

    python bench.py --workload long_contexts [--layers 16] [--requests 8] [--max-prompt 24576] [--new-tokens 512]
    python bench.py --workload chunked_prefill [--layers 4] [--prompt 131072] [--chunk 512] [--decoders 63]

``designs``: Rumalorn (parallel Dynamic-Tanh layers, key-tied attention with a bias by distance, experts
named by a table over token ids) and Pabavik (layers normed on both sides of every sub-layer; windowed attention
with a sink and an output gate, gated linear attention and attention over an earlier layer's cache in turns) and
Kekopel (a short convolution in front of every sub-layer, norms behind them, a mix over all layers' outputs; latent
attention with a learned sink per head and matrix memory in turns; dense and input-weighted expert feed-forwards)
beside MiniMax-M3 at equal layer sizes, all with random weights: a
2 048-token prompt in one step and decode steps of eight requests at 2 048 tokens of context, at a few
sizes that resemble real models' layers.

    python bench.py --workload designs [--layers 4] [--designs kekopel,pabavik]

Each prints one JSON line.  The reference times whole generations of this kind in
benchmarks/bench_decode_moe.py:8-24 (tokens after the first / time between first and last).
"""

from __future__ import annotations

import json
import time
from typing import Any, Dict, Optional

import numpy as np
import torch

from .config.engine_config import EngineConfig
from .engine.engine import Engine, StepEntry
from .engine.scheduler import Scheduler
from .sampling import Sampler, SamplingParams


def _engine(raw: Dict[str, Any], layers: int, max_seq: int, max_tokens: int, reqs: int, step_tokens: int) -> Engine:
    cfg = dict(raw, num_hidden_layers=layers, max_position_embeddings=max_seq)
    return Engine(EngineConfig(model_path="", dtype="bfloat16", use_dummy_weight=True, seed=0, page_size=16,
                               max_running_req=reqs, num_token_override=max_tokens, max_seq_len_override=max_seq,
                               max_extend_tokens=step_tokens, max_step_tokens=step_tokens), raw_config=cfg)


def long_contexts(raw: Dict[str, Any], layers: int = 16, requests: int = 8, min_prompt: int = 1024,
                  max_prompt: int = 24576, new_tokens: int = 512, seed: int = 0) -> Dict[str, Any]:
    rng = np.random.default_rng(seed)
    lengths = [int(x) for x in rng.integers(min_prompt, max_prompt + 1, requests)]
    max_seq = max_prompt + new_tokens + 16
    pool_tokens = sum(-(-(n + new_tokens) // 16) * 16 for n in lengths) + 16 * requests
    eng = _engine(raw, layers, max_seq, pool_tokens, requests, 8192)
    V = eng.spec.vocab_size
    sched = Scheduler(eng, Sampler(eng.device, V, requests), ())
    for i, n in enumerate(lengths):
        sched.add_request(rng.integers(0, V, n).tolist(), SamplingParams(max_tokens=new_tokens, ignore_eos=True), rid=i)
    pool = eng.cache.paged[0].pool
    high = 0
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    t_prefill_done = None
    decoded_at_prefill_done = 0
    steps = 0
    while not sched.idle:
        sched.step_overlapped()
        steps += 1
        high = max(high, pool.num_pages - pool.free_count)
        if t_prefill_done is None and all(r.decoding for r in sched.running) and not sched.waiting:
            torch.cuda.synchronize()
            t_prefill_done = time.perf_counter()
            decoded_at_prefill_done = sum(len(r.output) + r.in_flight for r in sched.running)
    sched.drain()
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    total_new = sum(len(sched.done[i].output) for i in range(requests))
    assert total_new == requests * new_tokens, (total_new, requests, new_tokens)
    t_mid = t_prefill_done if t_prefill_done is not None else t1
    decode_tokens = total_new - decoded_at_prefill_done
    return {
        "workload": "long_contexts", "layers": layers, "requests": requests, "prompt_lengths": lengths,
        "new_tokens": new_tokens, "steps": steps,
        "prefill_tokens_per_s": round(sum(lengths) / (t_mid - t0), 1), "prefill_s": round(t_mid - t0, 3),
        "decode_tokens_per_s": round(decode_tokens / max(t1 - t_mid, 1e-9), 1), "decode_s": round(t1 - t_mid, 3),
        "pages_high_water": int(high), "pages": int(pool.num_pages), "page_size": 16,
    }


def chunked_prefill(raw: Dict[str, Any], layers: int = 4, prompt: int = 131072, chunk: int = 512, decoders: int = 63,
                    seed: int = 0) -> Dict[str, Any]:
    rng = np.random.default_rng(seed)
    n_steps = -(-prompt // chunk)
    dec_prompts = [int(x) for x in rng.integers(128, 4097, decoders)]
    max_seq = max(prompt, max(dec_prompts) + n_steps) + 16
    pool_tokens = -(-prompt // 16) * 16 + sum(-(-(n + n_steps) // 16) * 16 for n in dec_prompts) + 16 * (decoders + 1)
    eng = _engine(raw, layers, max_seq, pool_tokens, decoders + 1, max(8192, chunk + decoders))
    V = eng.spec.vocab_size
    for i, n in enumerate(dec_prompts):  # the others' prompts first
        eng.step([StepEntry(("d", i), rng.integers(0, V, n).tolist(), [])])
    long_prompt = rng.integers(0, V, prompt).tolist()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(n_steps + 1)]
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    ev[0].record()
    fed = 0
    for s in range(n_steps):
        part = long_prompt[fed:fed + chunk]
        fed += len(part)
        entries = [StepEntry("long", part, [len(part) - 1] if fed == prompt else [])]
        entries += [StepEntry(("d", i), [int(rng.integers(0, V))], [0]) for i in range(decoders)]
        eng.step(entries)
        ev[s + 1].record()
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    ms = [ev[i].elapsed_time(ev[i + 1]) for i in range(n_steps)]
    tokens = prompt + decoders * n_steps
    return {
        "workload": "chunked_prefill", "layers": layers, "prompt": prompt, "chunk": chunk, "decoders": decoders,
        "decoder_prompts": [min(dec_prompts), max(dec_prompts)], "steps": n_steps,
        "tokens_per_s": round(tokens / (t1 - t0), 1), "seconds": round(t1 - t0, 3),
        "ms_first_steps": round(float(np.median(ms[: max(1, n_steps // 16)])), 3),
        "ms_last_steps": round(float(np.median(ms[-max(1, n_steps // 16):])), 3),
    }


DESIGN_SIZES = (
    # name, width, query heads, KV heads, head size, experts, experts per token, expert width, vocabulary
    ("w1024_h64", 1024, 16, 4, 64, 16, 2, 1408, 32768),
    ("w2048_h128", 2048, 16, 4, 128, 32, 4, 1024, 32768),
    ("w3072_h128", 3072, 48, 8, 128, 64, 8, 1536, 65536),
)


def _design_configs(width, heads, kv, dim, experts, top, ff, vocab, layers):
    mixer = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": dim, "scale": dim ** -0.5, "bias_max": 256,
             "q_temp": {"coef": 0.3, "every": 64}, "buckets": 32}
    mlp = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    ruma = {"architecture": "Rumalorn", "vocab": vocab, "width": width, "logit_scale": 1.0, "norm": {"eps": 1e-5},
            "layers": [{"type": "attention", "mixer": mixer, "mlp": mlp} for _ in range(layers)]}
    m3 = {"architectures": ["MiniMaxM3SparseForCausalLM"], "model_type": "minimax_m3", "vocab_size": vocab,
          "hidden_size": width, "num_hidden_layers": layers, "num_attention_heads": heads, "num_key_value_heads": kv,
          "head_dim": dim, "rotary_dim": dim // 2, "rope_theta": 5000000.0, "max_position_embeddings": 8192,
          "rms_norm_eps": 1e-6, "use_qk_norm": True, "use_gemma_norm": True, "tie_word_embeddings": False,
          "hidden_act": "silu", "num_local_experts": experts, "num_experts_per_tok": top, "intermediate_size": ff,
          "scoring_func": "sigmoid", "use_routing_bias": True, "routed_scaling_factor": 1.0, "n_shared_experts": 0,
          "torch_dtype": "bfloat16"}
    # Pabavik: windowed attention with a sink and an output gate, gated linear attention, and attention layers that
    # read an earlier layer's cache, in turns; the same experts (its router takes the softmax over the chosen logits)
    window = 1024
    att = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": dim, "scale": dim ** -0.5, "mask": {"size": window},
           "rot": {"dims": dim // 2, "base": 5000000.0}}
    gla = {"heads": heads, "dim": dim, "vdim": dim, "tau": 16.0, "decay_rank": 16}
    pmlp = {"kind": "moe", "expert": {"ff": ff, "limit": 7.0}, "router": {"experts": experts, "top": top}}
    players = []
    for i in range(layers):
        if i % 4 == 0 or (i % 4 == 3):
            players.append({"type": "attention", "mixer": dict(att), "mlp": pmlp})
        elif i % 4 == 1:
            players.append({"type": "gla", "mixer": dict(gla), "mlp": pmlp})
        else:
            players.append({"type": "attention", "mixer": dict(att, kv_from=i - 2), "mlp": pmlp})
    paba = {"architecture": "Pabavik", "vocab": vocab, "width": width, "embedding": {"scale": 1.0}, "norm": {"eps": 1e-6},
            "logit_softcap": 30.0, "layers": players}
    # Kekopel: latent attention (one cached row of kv_rank + rot_dim per token under all heads, the same window)
    # and matrix memory in turns (two to one), dense and expert feed-forwards in turns, a short convolution in front of
    # every sub-layer and the mix over all layers' outputs behind every layer
    # (a cached row of 128 at the two smaller sizes, which the tcgen05 attention kernel takes, of 256 at the largest)
    rank, rot = (64, 64) if width <= 2048 else (192, 64)
    lat = {"heads": heads, "dim": dim, "rot_dim": rot, "vdim": dim, "q_rank": width // 2, "kv_rank": rank,
           "scale": (dim + rot) ** -0.5, "mask": {"size": window}, "rot": {"dims": rot, "base": 1000000.0}}
    mem = {"heads": heads, "dim": dim, "vdim": dim, "gate_cap": 12.0}
    kmlp = [{"kind": "dense", "ff": top * ff}, {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}]
    keko = {"architecture": "Kekopel", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "canon": {"taps": 4},
            "layers": [{"type": "mlstm" if i % 3 == 2 else "latent_attention", "mixer": dict(mem if i % 3 == 2 else lat),
                        "mlp": kmlp[i % 2]} for i in range(layers)]}
    # Nusudra: latent attention (no query latent, a gate per head; the same cached rows as Kekopel's, no window), softmax
    # attention with biases, a bias by the logarithm of the distance and a sink per head beside a Mamba-2 layer, and the
    # gated delta rule, in turns; four residual streams, token shift, dense feed-forwards as wide as a token's experts
    nlat = {"heads": heads, "dim": dim, "rot_dim": rot, "vdim": dim, "kv_rank": rank, "scale": (dim + rot) ** -0.5,
            "rot": {"dims": rot, "base": 1000000.0}}
    pair = {"left": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": dim, "scale": dim ** -0.5},
            "right": {"heads": width // 64, "vdim": 64, "state": 128, "groups": kv, "conv": 4, "norm_groups": kv}}
    delta = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": dim, "conv": 4}
    kinds = [("latent_attention", nlat), ("parallel", pair), ("delta", delta)]
    nusu = {"architecture": "Nusudra", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0},
            "streams": 4, "layers": [{"type": kinds[i % 3][0], "mixer": kinds[i % 3][1],
                                      "mlp": {"kind": "dense", "ff": top * ff}} for i in range(layers)]}
    return {"rumalorn": ruma, "pabavik": paba, "kekopel": keko, "nusudra": nusu, "minimax_m3": m3}


def _time_design(raw: Dict[str, Any], prompt: int, batch: int, steps: int, warmup: int) -> Dict[str, Any]:
    eng = Engine(EngineConfig(model_path="", dtype="bfloat16", use_dummy_weight=True, seed=0, page_size=16,
                              max_running_req=batch, num_token_override=(batch + 1) * (prompt + 256),
                              max_seq_len_override=prompt + 256, max_extend_tokens=prompt, max_step_tokens=prompt),
                 raw_config=raw)
    V = eng.spec.vocab_size
    rng = np.random.default_rng(0)

    def ev():
        return torch.cuda.Event(enable_timing=True)

    times = []
    for i in range(3 + 3):  # one prompt in one step
        toks = rng.integers(0, V, prompt).tolist()
        a, b = ev(), ev()
        torch.cuda.synchronize()
        a.record()
        eng.step([StepEntry(("p", i), toks, [prompt - 1])])
        b.record()
        torch.cuda.synchronize()
        eng.close(("p", i))
        if i >= 3:
            times.append(a.elapsed_time(b))
    prefill_ms = float(np.median(times))
    rids = [("d", i) for i in range(batch)]
    for r in rids:
        eng.step([StepEntry(r, rng.integers(0, V, prompt).tolist(), [])])

    def one():
        eng.step([StepEntry(r, [int(rng.integers(0, V))], [0]) for r in rids])

    for _ in range(warmup):
        one()
    torch.cuda.synchronize()
    a, b = ev(), ev()
    a.record()
    for _ in range(steps):
        one()
    b.record()
    torch.cuda.synchronize()
    decode_ms = a.elapsed_time(b) / steps
    del eng
    torch.cuda.empty_cache()
    return {"prefill_ms": round(prefill_ms, 3), "prefill_tokens_per_s": round(prompt / (prefill_ms / 1e3), 1),
            "decode_ms_per_step": round(decode_ms, 4), "decode_tokens_per_s": round(batch / (decode_ms / 1e3), 1)}


def designs(raw: Dict[str, Any], layers: int = 4, prompt: int = 2048, batch: int = 8, steps: int = 32,
            warmup: int = 8, only: Optional[str] = None) -> Dict[str, Any]:
    """``raw`` (the headline configuration) is not used: the sizes are this workload's own.  ``only``: designs to time,
    with commas between them (MiniMax-M3 is always timed)."""
    import gc

    out: Dict[str, Any] = {"workload": "designs", "layers": layers, "prompt": prompt, "decode_batch": batch,
                           "decode_context": prompt, "steps": steps, "warmup": warmup, "dtype": "bf16",
                           "data": "synthetic: uniform random token ids, random weights made on the device", "sizes": {}}
    for name, *dims in DESIGN_SIZES:
        width, heads, kv, dim, experts, top, ff, vocab = dims
        row: Dict[str, Any] = {"width": width, "q_heads": heads, "kv_heads": kv, "head_dim": dim, "experts": experts,
                               "top_k": top, "expert_width": ff, "vocab": vocab}
        chosen = set(only.split(",")) | {"minimax_m3"} if only else None
        for design, cfg in _design_configs(*dims, layers).items():
            if chosen is not None and design not in chosen:
                continue
            row[design] = _time_design(cfg, prompt, batch, steps, warmup)
            gc.collect()
            torch.cuda.empty_cache()
        for design in ("rumalorn", "pabavik", "kekopel", "nusudra"):
            if design not in row:
                continue
            row[f"{design}_over_minimax_m3"] = {
                "prefill": round(row[design]["prefill_tokens_per_s"] / row["minimax_m3"]["prefill_tokens_per_s"], 3),
                "decode": round(row[design]["decode_tokens_per_s"] / row["minimax_m3"]["decode_tokens_per_s"], 3)}
        out["sizes"][name] = row
    return out


def run(name: str, raw: Dict[str, Any], **kw: Any) -> int:
    fn = {"long_contexts": long_contexts, "chunked_prefill": chunked_prefill, "designs": designs}[name]
    print(json.dumps(fn(raw, **{k: v for k, v in kw.items() if v is not None})))
    return 0
