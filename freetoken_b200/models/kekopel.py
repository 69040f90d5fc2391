"""Kekopel: from its typed config to a model description, and its checkpoint names.

Layers are ``conv_postnorm_residual`` blocks: every sub-layer reads the stream itself through a short causal
convolution over time, is RMS-normed (one number as weight) and scaled channel by channel on its way out, and
the layer hands on a learned mix of all layers' outputs so far.  The mixer is ``latent_attention`` (low-rank
latents for queries and for keys/values, one rotated key part for all heads with neighbouring dimensions turning
in pairs, a sliding window, a learned sink per head) or ``mlstm`` (matrix memory with capped exponential gates).
The feed-forward is ``dense_mlp`` (squared ReLU, biases), ``moe`` with raw sigmoid scores whose weight scales the
expert's input (``sigmoid_raw``, ``weight_on="input"``), or none.  The final norm has one number as weight.

Checkpoint names: ``embed``, ``head``, ``final.norm`` and, per layer ``l<i>``: ``norm1``, ``norm2``, ``ls1``, ``ls2``,
``canon1``, ``canon2``, ``dwa``; latent attention ``mix.{dq,dq.norm,uq,dkv,dkv.norm,uk,uv,sink,o}``; matrix memory
``mix.{q,k,v,g,o,norm,i,i.b,f,f.b}``; ``mlp.{up,up.b,down,down.b}`` or ``mlp.e<j>.{gate,up,down}`` with
``mlp.router``.  The projections of a mixer's input are concatenated into one matrix; gate/up pairs and experts
are stacked as for every other architecture here.  The reference has no such design.
"""

from __future__ import annotations

from typing import Any, List, Mapping, Optional

from ..config.kekopel import ARCHITECTURES, MAX_POSITION, KekopelConfig
from ..config.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from ..registry import Architecture, register_architecture
from ..weights.binder import FusionRule


def build_spec(cfg: KekopelConfig) -> ModelSpec:
    layers: List[LayerSpec] = []
    schedule: List[ScheduleEntry] = []
    L = len(cfg.layers)
    # random models: spreads that keep every activation of order one, so that a fault anywhere shows in the logits
    w_in = cfg.width ** -0.5
    for i, l in enumerate(cfg.layers):
        a = l.mixer
        if l.type == "latent_attention":
            position = (PartSpec("rope_interleaved", dict(rotary_dim=a.rot_dims, theta=a.rot_base, precise=True))
                        if a.rot_dims else PartSpec("none"))
            mixer = PartSpec("latent_attention", dict(
                hidden=cfg.width, n_heads=a.heads, head_dim=a.dim, rot_dim=a.rot_dim, v_head_dim=a.vdim, q_rank=a.q_rank,
                kv_rank=a.kv_rank, eps=cfg.norm_eps, position=position, window=a.window, scale=a.scale, sink="learned",
                init_std=(w_in, 2.0 * a.q_rank ** -0.5, a.kv_rank ** -0.5, (a.heads * a.vdim) ** -0.5)))
        else:
            mixer = PartSpec("mlstm", dict(hidden=cfg.width, n_heads=a.heads, head_dim=a.dim, v_head_dim=a.vdim,
                                           gate_cap=a.gate_cap, eps=cfg.norm_eps,
                                           init_std=(w_in, (a.heads * a.vdim) ** -0.5)))
        f = l.mlp
        if f is None:
            ffn = PartSpec("none")
        elif f.kind == "dense":
            ffn = PartSpec("dense_mlp", dict(hidden=cfg.width, inter=f.ff, act="relu2", bias=True,
                                             init_std=(w_in, f.ff ** -0.5)))
        else:
            ffn = PartSpec("moe", dict(hidden=cfg.width, inter=f.ff, n_experts=f.experts, top_k=f.top,
                                       scoring="sigmoid_raw", bias=False, scale=1.0, act="silu", weight_on="input",
                                       init_std=(w_in, f.ff ** -0.5)))
        block = PartSpec("conv_postnorm_residual", dict(hidden=cfg.width, taps=cfg.taps, eps=cfg.norm_eps, depth=i,
                                                        n_layers=L, depth_mix=True, init_std=1.0))
        layers.append(LayerSpec(name=f"l{i}", block=block, mixer=mixer, ffn=ffn, mixer_name="mix", ffn_name="mlp"))
        schedule.append(ScheduleEntry(i, None))
    return ModelSpec(
        architecture=cfg.architecture, vocab_size=cfg.vocab, hidden_size=cfg.width, layers=tuple(layers),
        schedule=tuple(schedule),
        embedding=PartSpec("token_embedding", dict(vocab=cfg.vocab, hidden=cfg.width, init_std=1.0)),
        final_norm=PartSpec("rmsnorm", dict(size=cfg.width, eps=cfg.norm_eps, gemma=False, scalar=True, init_std=0.1)),
        head=PartSpec("linear_head", dict(tied=False, init_std=w_in)),
        max_position=MAX_POSITION,
        embedding_name="embed_tokens", final_norm_name="final.norm", head_name="head",
        source=cfg,
    )


def fusion_rules(cfg: KekopelConfig) -> List[FusionRule]:
    """How checkpoint tensors combine into (or are renamed to) the model's tensors."""
    one = lambda target, source: FusionRule(target, [source], "same")  # noqa: E731  (a plain rename)
    rules = [one("embed_tokens.weight", "embed"), one("head.weight", "head"), one("final.norm.weight", "final.norm")]
    for i, l in enumerate(cfg.layers):
        p = f"l{i}"
        a = l.mixer
        if l.type == "latent_attention":
            rules += [FusionRule(f"{p}.mix.in_proj.weight", [f"{p}.mix.dq", f"{p}.mix.dkv"], "cat0",
                                 [a.q_rank, a.kv_rank + a.rot_dim]),
                      one(f"{p}.mix.q_norm.weight", f"{p}.mix.dq.norm"), one(f"{p}.mix.kv_norm.weight", f"{p}.mix.dkv.norm"),
                      one(f"{p}.mix.q_up.weight", f"{p}.mix.uq"), one(f"{p}.mix.k_up.weight", f"{p}.mix.uk"),
                      one(f"{p}.mix.v_up.weight", f"{p}.mix.uv"), one(f"{p}.mix.o_proj.weight", f"{p}.mix.o")]
        else:
            H = a.heads
            rules += [FusionRule(f"{p}.mix.in_proj.weight", [f"{p}.mix.{n}" for n in ("q", "k", "v", "g")], "cat0",
                                 [H * a.dim, H * a.dim, H * a.vdim, H * a.vdim]),
                      FusionRule(f"{p}.mix.gate_proj.weight", [f"{p}.mix.i", f"{p}.mix.f"], "cat0", [H, H]),
                      FusionRule(f"{p}.mix.gate_proj.bias", [f"{p}.mix.i.b", f"{p}.mix.f.b"], "cat0", [H, H]),
                      one(f"{p}.mix.norm.weight", f"{p}.mix.norm"), one(f"{p}.mix.o_proj.weight", f"{p}.mix.o")]
        f = l.mlp
        if f is None:
            continue
        if f.kind == "dense":
            rules += [one(f"{p}.mlp.up_proj.weight", f"{p}.mlp.up"), one(f"{p}.mlp.up_proj.bias", f"{p}.mlp.up.b"),
                      one(f"{p}.mlp.down_proj.weight", f"{p}.mlp.down"), one(f"{p}.mlp.down_proj.bias", f"{p}.mlp.down.b")]
        else:
            E = f.experts
            rules += [FusionRule(f"{p}.mlp.experts.gate_up_proj",
                                 [f"{p}.mlp.e{e}.{w}" for e in range(E) for w in ("gate", "up")], "stack_pairs"),
                      FusionRule(f"{p}.mlp.experts.down_proj", [f"{p}.mlp.e{e}.down" for e in range(E)], "stack"),
                      one(f"{p}.mlp.gate.weight", f"{p}.mlp.router")]
    return rules


def parse(raw: Mapping[str, Any], num_layers: Optional[int] = None) -> KekopelConfig:
    return KekopelConfig.from_dict(raw, num_layers=num_layers)


ARCH = Architecture(names=ARCHITECTURES, parse_config=parse, build_spec=build_spec, fusion_rules=fusion_rules)
register_architecture(ARCH)
