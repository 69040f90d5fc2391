"""Nusudra: from its typed config to a model description, and its checkpoint names.

Layers are ``hyper_residual`` blocks: the residual is carried in several streams that every sub-layer reads as a
weighted sum and writes back to while they are mixed, and the mixer's input is blended with the token before
(token shift).  The mixer is ``latent_attention`` (no query latent, one cached latent and one rotated key part
under all heads, rotate-half pairing, a sigmoid gate per head), ``side_by_side`` of ``gqa_attention`` (projection
biases, a bias by the logarithm of the distance, a learned sink per head) and ``mamba2`` whose normed results are
averaged, or ``gated_delta``.  The feed-forward is ``dense_mlp`` (squared ReLU, no biases) or none.  The embedding
is scaled; final norm and head are plain.

Checkpoint names: ``embed``, ``head``, ``final.norm`` and, per layer ``l<i>``: ``norm1``, ``norm2``, ``shift``,
``hc<q>.{in,out,mix}``; latent attention ``mix.{q,dkv,dkv.norm,uk,uv,g,o}``; the pair ``mix.left.{q,k,v}`` (each with
``.b``), ``mix.left.{r1,r2,sink,o,out}``, ``mix.right.{in,conv,conv.b,dt_bias,A_log,D,norm,o,out}``; the delta rule
``mix.{q,k,v}`` (each with ``.conv``), ``mix.{b,a,g,A_log,dt_bias,norm,o}``; ``mlp.{up,down}``.  The projections of
a mixer's input are concatenated into one matrix.  The reference has no such design.
"""

from __future__ import annotations

from typing import Any, List, Mapping, Optional

from ..config.nusudra import ARCHITECTURES, MAX_POSITION, NusudraConfig
from ..config.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from ..registry import Architecture, register_architecture
from ..weights.binder import FusionRule


def build_spec(cfg: NusudraConfig) -> ModelSpec:
    layers: List[LayerSpec] = []
    schedule: List[ScheduleEntry] = []
    L = len(cfg.layers)
    W = cfg.width
    # random models: spreads that keep every activation of order one, so that a fault anywhere shows in the logits
    w_in = W ** -0.5
    for i, l in enumerate(cfg.layers):
        a = l.mixer
        if l.type == "latent_attention":
            position = (PartSpec("rope_neox", dict(rotary_dim=a.rot_dims, theta=a.rot_base, precise=True))
                        if a.rot_dims else PartSpec("none"))
            mixer = PartSpec("latent_attention", dict(
                hidden=W, n_heads=a.heads, head_dim=a.dim, rot_dim=a.rot_dim, v_head_dim=a.vdim, q_rank=None,
                kv_rank=a.kv_rank, eps=cfg.norm_eps, position=position, window=None, scale=a.scale, sink=None,
                head_gate=True, init_std=(w_in, w_in, a.kv_rank ** -0.5, (a.heads * a.vdim) ** -0.5)))
        elif l.type == "parallel":
            le, ri = a.left, a.right
            left = PartSpec("gqa_attention", dict(
                hidden=W, n_heads=le.heads, n_kv_heads=le.kv_heads, head_dim=le.dim, v_head_dim=le.vdim, qk_norm=False,
                eps=cfg.norm_eps, gemma=False, position=PartSpec("none"), scale=le.scale, sink="learned", proj_bias=True,
                log_dist_bias=True, init_std=(w_in, (le.heads * le.vdim) ** -0.5)))
            right = PartSpec("mamba2", dict(
                hidden=W, n_heads=ri.heads, v_head_dim=ri.vdim, state=ri.state, groups=ri.groups, taps=ri.taps,
                norm_groups=ri.norm_groups, eps=cfg.norm_eps, init_std=(w_in, (ri.heads * ri.vdim) ** -0.5)))
            mixer = PartSpec("side_by_side", dict(hidden=W, eps=cfg.norm_eps, branches=(("left", left), ("right", right)),
                                                  init_std=1.0))
        else:
            mixer = PartSpec("gated_delta", dict(
                hidden=W, n_heads=a.heads, n_kv_heads=a.kv_heads, head_dim=a.dim, v_head_dim=a.vdim, taps=a.taps,
                eps=cfg.norm_eps, init_std=(w_in, (a.heads * a.vdim) ** -0.5)))
        f = l.mlp
        if f is None:
            ffn = PartSpec("none")
        else:
            ffn = PartSpec("dense_mlp", dict(hidden=W, inter=f.ff, act="relu2", bias=False, init_std=(w_in, f.ff ** -0.5)))
        block = PartSpec("hyper_residual", dict(hidden=W, streams=cfg.streams, eps=cfg.norm_eps, token_shift=True,
                                                last=i == L - 1, init_std=1.0))
        layers.append(LayerSpec(name=f"l{i}", block=block, mixer=mixer, ffn=ffn, mixer_name="mix", ffn_name="mlp"))
        schedule.append(ScheduleEntry(i, None))
    return ModelSpec(
        architecture=cfg.architecture, vocab_size=cfg.vocab, hidden_size=W, layers=tuple(layers),
        schedule=tuple(schedule),
        embedding=PartSpec("token_embedding", dict(vocab=cfg.vocab, hidden=W, init_std=1.0, scale=cfg.embedding_scale)),
        final_norm=PartSpec("rmsnorm", dict(size=W, eps=cfg.norm_eps, gemma=False)),
        head=PartSpec("linear_head", dict(tied=False, init_std=w_in)),
        max_position=MAX_POSITION,
        embedding_name="embed_tokens", final_norm_name="final.norm", head_name="head",
        source=cfg,
    )


def fusion_rules(cfg: NusudraConfig) -> List[FusionRule]:
    """How checkpoint tensors combine into (or are renamed to) the model's tensors."""
    one = lambda target, source: FusionRule(target, [source], "same")  # noqa: E731  (a plain rename)
    rules = [one("embed_tokens.weight", "embed"), one("head.weight", "head"), one("final.norm.weight", "final.norm")]
    for i, l in enumerate(cfg.layers):
        p = f"l{i}"
        a = l.mixer
        if l.type == "latent_attention":
            rules += [FusionRule(f"{p}.mix.in_proj.weight", [f"{p}.mix.dkv", f"{p}.mix.g"], "cat0",
                                 [a.kv_rank + a.rot_dim, a.heads]),
                      one(f"{p}.mix.kv_norm.weight", f"{p}.mix.dkv.norm"),
                      one(f"{p}.mix.q_up.weight", f"{p}.mix.q"), one(f"{p}.mix.k_up.weight", f"{p}.mix.uk"),
                      one(f"{p}.mix.v_up.weight", f"{p}.mix.uv"), one(f"{p}.mix.o_proj.weight", f"{p}.mix.o")]
        elif l.type == "parallel":
            le, ri = a.left, a.right
            q = f"{p}.mix.left"
            rules += [FusionRule(f"{q}.qkv_proj.weight", [f"{q}.q", f"{q}.k", f"{q}.v"], "cat0",
                                 [le.heads * le.dim, le.kv_heads * le.dim, le.kv_heads * le.vdim]),
                      one(f"{q}.q_bias", f"{q}.q.b"), one(f"{q}.k_bias", f"{q}.k.b"), one(f"{q}.v_bias", f"{q}.v.b"),
                      one(f"{q}.o_proj.weight", f"{q}.o")]
            r = f"{p}.mix.right"
            rules += [one(f"{r}.in_proj.weight", f"{r}.in"), one(f"{r}.conv.weight", f"{r}.conv"),
                      one(f"{r}.conv.bias", f"{r}.conv.b"), one(f"{r}.norm.weight", f"{r}.norm"),
                      one(f"{r}.o_proj.weight", f"{r}.o")]
        else:
            H, G = a.heads, a.kv_heads
            sizes = [G * a.dim, G * a.dim, H * a.vdim]
            rules += [FusionRule(f"{p}.mix.in_proj.weight", [f"{p}.mix.{n}" for n in ("q", "k", "v", "g", "b", "a")], "cat0",
                                 sizes + [H * a.vdim, H, H]),
                      FusionRule(f"{p}.mix.conv.weight", [f"{p}.mix.{n}.conv" for n in ("q", "k", "v")], "cat0", sizes),
                      one(f"{p}.mix.norm.weight", f"{p}.mix.norm"), one(f"{p}.mix.o_proj.weight", f"{p}.mix.o")]
        if l.mlp is not None:
            rules += [one(f"{p}.mlp.up_proj.weight", f"{p}.mlp.up"), one(f"{p}.mlp.down_proj.weight", f"{p}.mlp.down")]
    return rules


def parse(raw: Mapping[str, Any], num_layers: Optional[int] = None) -> NusudraConfig:
    return NusudraConfig.from_dict(raw, num_layers=num_layers)


ARCH = Architecture(names=ARCHITECTURES, parse_config=parse, build_spec=build_spec, fusion_rules=fusion_rules)
register_architecture(ARCH)
