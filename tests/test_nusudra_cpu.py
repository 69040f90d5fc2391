"""Nusudra without a GPU: its config reader, model description and checkpoint names, the plain statements of its
mechanisms against other ways of writing them, and the engine's step, cache, state and batching logic with the plain
PyTorch statements of the kernels (tests/kernel_refs.py) standing in for the CUDA kernels."""

import copy

import pytest
import torch

import kernel_refs
from helpers import make_engine, mixed_schedule, model_folder, replay_cuts, replay_mixed, replay_whole, tokens_for
from plain import nusudra_plain as plain_model
from plain.nusudra_plain import PlainNusudra
from tiny_nusudra import ALL, NUSU_1, NUSU_2, NUSU_4, PAGE

from freetoken_b200.config.spec import PagedKVNeed, StateNeed
from freetoken_b200.engine.build import describe_model
from freetoken_b200.engine.engine import StepEntry
from freetoken_b200.errors import ConfigError
from freetoken_b200.registry import architecture_of

TOL = dict(rtol=1e-4, atol=5e-5)


@pytest.fixture
def cpu_ops(monkeypatch):
    kernel_refs.install(monkeypatch)


# --------------------------------------------------------------------------- config, description, names
def test_the_description_follows_the_config():
    _, cfg, spec, expected = describe_model(NUSU_1)
    assert [l.mixer.kind for l in spec.layers] == ["gated_delta", "side_by_side", "latent_attention", "gated_delta"]
    assert [l.ffn.kind for l in spec.layers] == ["dense_mlp", "none", "dense_mlp", "dense_mlp"]
    assert all(l.block.kind == "hyper_residual" and l.block["streams"] == 2 and l.block["token_shift"] for l in spec.layers)
    assert [l.block["last"] for l in spec.layers] == [False, False, False, True]
    assert spec.embedding["scale"] == 2.0
    left, right = (s for _, s in spec.layers[1].mixer["branches"])
    assert (left.kind, left["n_kv_heads"], left["v_head_dim"], left["scale"], left["sink"]) == ("gqa_attention", 2, 24, 0.3, "learned")
    assert left["proj_bias"] and left["log_dist_bias"] and not left["qk_norm"]
    assert (right.kind, right["state"], right["groups"], right["taps"], right["norm_groups"]) == ("mamba2", 16, 2, 2, 4)
    a = spec.layers[2].mixer
    assert (a["q_rank"], a["kv_rank"], a["rot_dim"], a["head_gate"], a["sink"], a["window"]) == (None, 20, 8, True, None, None)
    assert a["position"].kind == "rope_neox" and a["position"]["rotary_dim"] == 8 and a["position"]["theta"] == 100.0
    assert expected["l0.mix.in_proj.weight"].shape == (2 * 16 + 2 * 16 + 4 * 24 + 4 * 24 + 4 + 4, 64)
    assert expected["l0.mix.conv.weight"].shape == (2 * 16 + 2 * 16 + 4 * 24, 3)
    assert expected["l1.mix.right.in_proj.weight"].shape == (2 * 32 + 2 * 2 * 16 + 4, 64)
    assert expected["l1.mix.left.qkv_proj.weight"].shape == (4 * 16 + 2 * 16 + 2 * 24, 64)
    assert expected["l1.mix.left.out"].shape == (64,) and expected["l1.mix.left.sink"].shape == (4,)
    assert expected["l2.mix.in_proj.weight"].shape == (20 + 8 + 3, 64) and expected["l2.mix.q_up.weight"].shape == (3 * 16, 64)
    assert expected["l0.hc1.mix"].shape == (2, 2) and expected["l3.hc2.in"].shape == (2,) and expected["l0.shift"].shape == (64,)
    assert "l1.norm2" not in expected and "l1.hc2.in" not in expected
    _, _, spec2, expected2 = describe_model(NUSU_2)
    assert spec2.layers[0].block["streams"] is None and "l0.hc1.in" not in expected2 and "l0.shift" in expected2
    assert spec2.embedding["scale"] == 1.0


def test_the_checkpoint_names_are_the_designs():
    arch, cfg, _, _ = describe_model(NUSU_1)
    sources = {s for r in arch.fusion_rules(cfg) for s in r.sources}
    for name in ("embed", "head", "final.norm", "l0.mix.q.conv", "l0.mix.b", "l0.mix.a", "l0.mix.g", "l1.mix.left.q.b",
                 "l1.mix.left.o", "l1.mix.right.in", "l1.mix.right.conv.b", "l1.mix.right.norm", "l2.mix.dkv", "l2.mix.dkv.norm",
                 "l2.mix.uk", "l2.mix.uv", "l2.mix.g", "l2.mix.q", "l0.mlp.up", "l0.mlp.down"):
        assert name in sources, name


def test_config_errors_name_the_key():
    def broken(path, value, delete=False):
        raw = copy.deepcopy(NUSU_1)
        d = raw
        for k in path[:-1]:
            d = d[k]
        if delete:
            del d[path[-1]]
        else:
            d[path[-1]] = value
        return raw

    for raw, word in [
        (broken(["vocab"], None, True), "vocab"),
        (broken(["norm"], None, True), "eps"),
        (broken(["streams"], 0), "streams"),
        (broken(["streams"], 9), "streams"),
        (broken(["layers", 0, "mixer", "kv_heads"], 3), "kv_heads"),
        (broken(["layers", 0, "mixer", "conv"], None, True), "conv"),
        (broken(["layers", 1, "mixer", "left", "scale"], None, True), "scale"),
        (broken(["layers", 1, "mixer", "right", "groups"], 3), "groups"),
        (broken(["layers", 1, "mixer", "right", "norm_groups"], 5), "norm_groups"),
        (broken(["layers", 2, "mixer", "rot", "dims"], 10), "rot.dims"),
        (broken(["layers", 2, "mixer", "kv_rank"], None, True), "kv_rank"),
        (broken(["layers", 0, "mlp", "kind"], "glu"), "kind"),
        (broken(["layers", 2, "type"], "conv"), "type"),
    ]:
        with pytest.raises(ConfigError, match=word):
            architecture_of(raw).parse_config(raw)


def test_pages_and_states():
    from freetoken_b200.models.model import Model
    from freetoken_b200.parts import BuildEnv, Workspace

    _, _, spec, _ = describe_model(NUSU_1)
    cpu = torch.device("cpu")
    model = Model(spec, BuildEnv(dtype=torch.float32, device=cpu, max_seq_len=8, max_step_tokens=8, workspace=Workspace(cpu)))
    needs = dict(model.cache_needs())
    assert needs[0] == StateNeed((("s", (4, 24, 16), "float32"), ("conv", (2, 2 * 16 + 2 * 16 + 4 * 24), "float32")))
    assert needs[(1, 0)] == PagedKVNeed((("k", 2, 32), ("v", 2, 32)), None)  # keys of 16 and values of 24 on rows of 32
    assert needs[(1, 1)] == StateNeed((("s", (4, 16, 8), "float32"), ("conv", (1, 32 + 2 * 32), "float32")))
    assert needs[2] == PagedKVNeed((("kv", 1, 32),), None)  # one row of latent and rotated part per token, padded to 16s
    blocks = dict(model.block_state_needs())
    assert len(blocks) == 4 and blocks[0] == StateNeed((("shift", (1, 64), "float32"),))
    _, _, spec2, _ = describe_model(NUSU_2)
    model2 = Model(spec2, BuildEnv(dtype=torch.float32, device=cpu, max_seq_len=8, max_step_tokens=8, workspace=Workspace(cpu)))
    assert dict(model2.cache_needs())[1] == StateNeed((("s", (1, 14, 22), "float32"),))  # one tap: no convolution state


# --------------------------------------------------------------------------- the plain mechanisms among themselves
def test_the_plain_token_shift_and_convolution():
    h = torch.arange(8.0).view(4, 2)
    y = plain_model.token_shift(h, torch.tensor([0.25, 1.0]))
    assert y[0].tolist() == [0.0, 0.0] and y[2].tolist() == [4.0 + (2.0 - 4.0) * 0.25, 3.0]
    w = torch.tensor([[1.0, 10.0, 100.0], [0.0, 0.0, 1.0]])
    c = plain_model.causal_conv(h, w, torch.tensor([0.5, 0.0]))
    assert c[0].tolist() == [0.5, 1.0] and c[2].tolist() == [0.5 + 0.0 + 10 * 2.0 + 100 * 4.0, 5.0]


def test_the_plain_delta_rule_is_the_one_with_the_state_written_out_as_a_product():
    """``S_t = g_t (I - beta_t k_t k_t^T) S_(t-1) + beta_t k_t v_t^T`` gives the same outputs as the three steps."""
    torch.manual_seed(1)
    m = dict(heads=2, kv_heads=1, dim=6, vdim=5, conv=3)
    W = 12
    w = {n: torch.randn(r, W).double() / 3 for n, r in (("q", 6), ("k", 6), ("v", 10), ("g", 10), ("b", 2), ("a", 2))}
    w.update({"q.conv": torch.randn(6, 3).double(), "k.conv": torch.randn(6, 3).double(), "v.conv": torch.randn(10, 3).double(),
              "A_log": torch.randn(2).double(), "dt_bias": torch.randn(2).double(), "norm": torch.rand(5).double() + 0.5,
              "o": torch.eye(10, 10).double()[:W].T.contiguous().T if False else torch.randn(W, 10).double()})
    h = torch.randn(9, W).double()
    want = plain_model.delta_rule(h, w, m, 1e-5)
    F = torch.nn.functional
    q = F.silu(plain_model.causal_conv(h @ w["q"].T, w["q.conv"]))
    k = F.silu(plain_model.causal_conv(h @ w["k"].T, w["k.conv"]))
    v = F.silu(plain_model.causal_conv(h @ w["v"].T, w["v.conv"])).view(9, 2, 5)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * 6 ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w["b"].T)
    g = torch.exp(-torch.exp(w["A_log"]) * F.softplus(h @ w["a"].T + w["dt_bias"]))
    o = torch.zeros(9, 2, 5).double()
    for a in range(2):
        S = torch.zeros(6, 5).double()
        for t in range(9):
            S = g[t, a] * (torch.eye(6).double() - beta[t, a] * torch.outer(k[t], k[t])) @ S + beta[t, a] * torch.outer(k[t], v[t, a])
            o[t, a] = S.T @ q[t]
    o = plain_model.unit(o, 1e-5) * w["norm"]
    got = (o.reshape(9, 10) * F.silu(h @ w["g"].T)) @ w["o"].T
    torch.testing.assert_close(got, want, rtol=1e-10, atol=1e-10)


def test_the_plain_state_space_layer_is_its_sum_over_the_past():
    """``y_t = sum_(s <= t) (prod_(s < r <= t) a_r) dt_s (C_t . B_s) x_s + D x_t``, the attention-like form."""
    torch.manual_seed(2)
    m = dict(heads=2, vdim=3, state=4, groups=1, conv=2, norm_groups=1)
    W, inner = 10, 6
    w = {"in": torch.randn(2 * inner + 2 * 4 + 2, W).double() / 3, "conv": torch.randn(inner + 8, 2).double(),
         "conv.b": torch.randn(inner + 8).double() / 3, "dt_bias": torch.randn(2).double(), "A_log": torch.randn(2).double(),
         "D": torch.randn(2).double(), "norm": torch.rand(inner).double() + 0.5, "o": torch.randn(W, inner).double()}
    h = torch.randn(7, W).double()
    want = plain_model.state_space(h, w, m, 1e-5)
    F = torch.nn.functional
    proj = h @ w["in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 8], proj[:, 2 * inner + 8:]
    xbc = F.silu(plain_model.causal_conv(xbc, w["conv"], w["conv.b"]))
    x, B, C = xbc[:, :inner].view(7, 2, 3), xbc[:, inner:inner + 4], xbc[:, inner + 4:]
    dt = F.softplus(dt + w["dt_bias"])
    la = -torch.exp(w["A_log"]) * dt  # log decays
    y = torch.zeros(7, 2, 3).double()
    for a in range(2):
        for t in range(7):
            for s in range(t + 1):
                y[t, a] += torch.exp(la[s + 1:t + 1, a].sum()) * dt[s, a] * (C[t] @ B[s]) * x[s, a]
            y[t, a] += w["D"][a] * x[t, a]
    y = plain_model.unit(y.reshape(7, inner) * F.silu(z), 1e-5) * w["norm"]
    torch.testing.assert_close(y @ w["o"].T, want, rtol=1e-10, atol=1e-10)


def test_one_stream_with_unit_coefficients_is_the_plain_residual(tmp_path_factory):
    """A model without streams, and the same weights with one stream whose coefficients are all 1, say the same."""
    folder = model_folder(tmp_path_factory.getbasetemp(), "N2", NUSU_2)
    plain = PlainNusudra(folder)
    toks = tokens_for(plain.vocab, 12, 3)
    weights = dict(plain.w)
    for i, l in enumerate(NUSU_2["layers"]):
        for q in ("1", "2") if l["mlp"] is not None else ("1",):
            weights[f"l{i}.hc{q}.in"] = torch.ones(1, dtype=torch.float64)
            weights[f"l{i}.hc{q}.out"] = torch.ones(1, dtype=torch.float64)
            weights[f"l{i}.hc{q}.mix"] = torch.ones(1, 1, dtype=torch.float64)
    one = PlainNusudra(raw=dict(NUSU_2, streams=1), weights=weights)
    torch.testing.assert_close(one.logits(toks), plain.logits(toks), rtol=1e-6, atol=1e-6)


# --------------------------------------------------------------------------- the engine on CPU stand-ins
@pytest.mark.parametrize("name", ["N1", "N2", "N3", "N4"])
def test_cuts_agree_with_the_plain_model(name, tmp_path_factory, cpu_ops):
    folder = model_folder(tmp_path_factory.getbasetemp(), name, ALL[name])
    plain = PlainNusudra(folder)
    toks = tokens_for(plain.vocab, 41, 7)
    want = plain.logits(toks)
    eng = make_engine(folder, "float32", "cpu", PAGE, pages=30)
    torch.testing.assert_close(replay_whole(eng, "w", toks), want, **TOL)
    torch.testing.assert_close(replay_cuts(eng, "c", toks, [5, 2, 11, 2, 3, 7]), want, **TOL)
    torch.testing.assert_close(replay_cuts(eng, "o", toks[:12], []), want[:12], **TOL)
    eng.cache.check()
    assert all(g.pool.free_count == g.pool.num_pages for g in eng.cache.paged)


def test_batches_of_unequal_requests_and_slots_used_again(tmp_path_factory, cpu_ops):
    folder = model_folder(tmp_path_factory.getbasetemp(), "N1", NUSU_1)
    plain = PlainNusudra(folder)
    lengths = {"r0": 25, "r1": 33, "r2": 18, "r3": 29, "r4": 21, "r5": 27}
    seqs = {r: tokens_for(plain.vocab, n, i) for i, (r, n) in enumerate(lengths.items())}
    eng = make_engine(folder, "float32", "cpu", PAGE, pages=4 * 10)
    got = replay_mixed(eng, seqs, mixed_schedule(lengths, seed=5))
    for r, toks in seqs.items():
        torch.testing.assert_close(got[r], plain.logits(toks), **TOL, msg=lambda m: f"{r}: {m}")
    assert eng.cache.slots.free_count == 4
    for g in eng.cache.paged:
        assert g.pool.handed_out > g.pool.num_pages


def test_a_slot_used_again_starts_from_nothing(tmp_path_factory, cpu_ops):
    """One request slot: every request gets the slot (and pages) of the one before; the states, the convolutions'
    inputs and the shift's last input of the earlier owner must not leak."""
    folder = model_folder(tmp_path_factory.getbasetemp(), "N4", NUSU_4)
    plain = PlainNusudra(folder)
    eng = make_engine(folder, "float32", "cpu", PAGE, pages=12, reqs=1)
    for i in range(3):
        toks = tokens_for(plain.vocab, 20 + i, 30 + i)
        torch.testing.assert_close(replay_cuts(eng, f"r{i}", toks, [1, 1, 6, 2]), plain.logits(toks), **TOL)


def test_the_streams_sum_after_every_layer_is_the_plain_models(tmp_path_factory, cpu_ops):
    folder = model_folder(tmp_path_factory.getbasetemp(), "N1", NUSU_1)
    plain = PlainNusudra(folder)
    toks = tokens_for(plain.vocab, 19, 2)
    want = plain.layer_sums(toks)
    # (random tensors are drawn by name: a model of the first n layers has the full model's weights, and leaves the
    # sum of its streams after layer n to the final norm)
    for n in range(1, len(NUSU_1["layers"]) + 1):
        cut = model_folder(tmp_path_factory.getbasetemp(), f"N1_first{n}", dict(NUSU_1, layers=NUSU_1["layers"][:n]))
        eng = make_engine(cut, "float32", "cpu", PAGE, pages=30)
        seen = []
        norm = eng.model.final_norm
        orig = norm.add_forward

        def wrapped(x, residual, out, out_f32=None, rows=None, orig=orig):
            seen.append(residual.clone())
            return orig(x, residual, out, out_f32=out_f32, rows=rows)

        norm.add_forward = wrapped
        eng.step([StepEntry("a", toks, [len(toks) - 1])])
        torch.testing.assert_close(seen[0], want[n - 1], **TOL, msg=lambda m: f"after layer {n - 1}: {m}")


def plain_for_the_command_line(folder):
    from types import SimpleNamespace

    plain = PlainNusudra(folder)
    return SimpleNamespace(cfg=SimpleNamespace(vocab=plain.vocab), logits=lambda toks: plain.logits(toks).float())


def test_the_command_line_makes_a_model_generates_and_replays(tmp_path, capsys, cpu_ops):
    from test_cli import generate_and_replay, make_model

    folder = make_model(tmp_path, NUSU_1, capsys)
    generate_and_replay(folder, "cpu", "float32", capsys, tmp_path, plain_for_the_command_line(folder))
