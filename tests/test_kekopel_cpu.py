"""Kekopel without a GPU: its config reader, model description and checkpoint names, the plain statements of its
mechanisms against each other, and the engine's step, cache, state and batching logic with the plain PyTorch
statements of the kernels (tests/kernel_refs.py) standing in for the CUDA kernels."""

import copy

import pytest
import torch

import kernel_refs
from helpers import make_engine, mixed_schedule, model_folder, replay_cuts, replay_mixed, replay_whole, tokens_for
from plain import kekopel_plain as plain_model
from plain.kekopel_plain import PlainKekopel
from tiny_kekopel import ALL, KEKO_1, KEKO_2, PAGE

from freetoken_b200.config.spec import PagedKVNeed, StateNeed
from freetoken_b200.engine.build import describe_model
from freetoken_b200.engine.engine import StepEntry
from freetoken_b200.errors import ConfigError
from freetoken_b200.registry import architecture_of

TOL = dict(rtol=1e-4, atol=2e-5)


@pytest.fixture
def cpu_ops(monkeypatch):
    kernel_refs.install(monkeypatch)


# --------------------------------------------------------------------------- config, description, names
def test_the_description_follows_the_config():
    _, cfg, spec, expected = describe_model(KEKO_1)
    assert [l.mixer.kind for l in spec.layers] == ["latent_attention", "mlstm", "latent_attention", "mlstm"]
    assert [l.ffn.kind for l in spec.layers] == ["dense_mlp", "moe", "moe", "dense_mlp"]
    assert [l.block["depth"] for l in spec.layers] == [0, 1, 2, 3] and all(l.block["taps"] == 3 for l in spec.layers)
    a = spec.layers[0].mixer
    assert (a["window"], a["scale"], a["q_rank"], a["kv_rank"], a["rot_dim"]) == (9, 0.2, 24, 40, 8)
    assert a["position"].kind == "rope_interleaved" and a["position"]["rotary_dim"] == 4
    assert spec.layers[2].ffn["weight_on"] == "input" and spec.layers[2].ffn["scoring"] == "sigmoid_raw"
    assert expected["l0.dwa"].shape == (2,) and expected["l3.dwa"].shape == (5,)
    assert expected["l0.norm1"].shape == () and expected["final.norm.weight"].shape == ()
    assert expected["l0.mix.in_proj.weight"].shape == (24 + 40 + 8, 64)
    assert expected["l1.mix.gate_proj.bias"].shape == (4,)
    _, _, spec2, expected2 = describe_model(KEKO_2)
    assert spec2.layers[2].mixer["window"] is None and spec2.layers[1].ffn.kind == "none"
    assert "l1.norm2" not in expected2 and "l1.canon2" not in expected2 and "l1.dwa" in expected2


def test_config_errors_name_the_key():
    def broken(path, value, delete=False):
        raw = copy.deepcopy(KEKO_1)
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
        (broken(["canon"], None, True), "canon"),
        (broken(["canon", "taps"], 40), "taps"),
        (broken(["layers", 0, "mixer", "kv_rank"], None, True), "kv_rank"),
        (broken(["layers", 0, "mixer", "rot", "dims"], 10), "rot.dims"),
        (broken(["layers", 0, "mixer", "mask", "size"], 0), "mask.size"),
        (broken(["layers", 1, "mixer", "gate_cap"], 0.0), "gate_cap"),
        (broken(["layers", 1, "mlp", "router", "top"], 9), "top"),
        (broken(["layers", 0, "mlp", "kind"], "glu"), "kind"),
        (broken(["layers", 2, "type"], "conv"), "type"),
    ]:
        with pytest.raises(ConfigError, match=word):
            architecture_of(raw).parse_config(raw)


def test_cached_rows_and_states():
    from freetoken_b200.models.model import Model
    from freetoken_b200.parts import BuildEnv, Workspace

    _, _, spec, _ = describe_model(KEKO_1)
    cpu = torch.device("cpu")
    model = Model(spec, BuildEnv(dtype=torch.float32, device=cpu, max_seq_len=8, max_step_tokens=8, workspace=Workspace(cpu)))
    needs = dict(model.cache_needs())
    assert needs[0] == PagedKVNeed((("kv", 1, 48),), 9)  # one row of latent and rotated part per token, padded to 16s
    assert needs[2] == PagedKVNeed((("kv", 1, 48),), 20)
    assert needs[1] == StateNeed((("s", (2, 16, 25), "float32"), ("m", (2,), "float32")))
    blocks = dict(model.block_state_needs())
    assert blocks[0] == StateNeed((("conv1", (2, 64), "float32"), ("conv2", (2, 64), "float32")))
    assert len(blocks) == 4


# --------------------------------------------------------------------------- the plain mechanisms among themselves
def test_the_plain_attention_is_the_one_with_keys_and_values_spelled_out():
    """The latents' up-projections can be moved onto the query and the output without changing the result."""
    torch.manual_seed(0)
    m = KEKO_1["layers"][0]["mixer"]
    H, D, R, Dv, C, Q, W = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"], 64
    w = {"dq": torch.randn(Q, W) / 8, "dq.norm": torch.rand(Q) + 0.5, "uq": torch.randn(H * (D + R), Q) / 5,
         "dkv": torch.randn(C + R, W) / 8, "dkv.norm": torch.rand(C) + 0.5, "uk": torch.randn(H * D, C) / 6,
         "uv": torch.randn(H * Dv, C) / 6, "sink": torch.randn(H), "o": torch.randn(W, H * Dv) / 7}
    w = {k: v.double() for k, v in w.items()}
    h = torch.randn(30, W).double()
    want = plain_model.latent_attention(h, w, m, 1e-5)
    # absorbed: scores against the latent itself
    cq = plain_model.unit(h @ w["dq"].T, 1e-5) * w["dq.norm"]
    q = (cq @ w["uq"].T).view(30, H, D + R)
    kv = h @ w["dkv"].T
    c = plain_model.unit(kv[:, :C], 1e-5) * w["dkv.norm"]
    kr = plain_model.rotate_pairs(kv[:, C:], range(30), m["rot"]["dims"], m["rot"]["base"])
    qr = plain_model.rotate_pairs(q[..., D:], range(30), m["rot"]["dims"], m["rot"]["base"])
    uk, uv = w["uk"].view(H, D, C), w["uv"].view(H, Dv, C)
    out = torch.zeros(30, H, Dv).double()
    for t in range(30):
        lo = max(0, t - m["mask"]["size"] + 1)
        for a in range(H):
            ql = uk[a].T @ q[t, a, :D]
            s = (c[lo:t + 1] @ ql + kr[lo:t + 1] @ qr[t, a]) * m["scale"]
            e = torch.exp(s)
            p = e / (e.sum() + torch.exp(w["sink"][a]))
            out[t, a] = uv[a] @ (p @ c[lo:t + 1])
    torch.testing.assert_close(out.reshape(30, -1) @ w["o"].T, want, rtol=1e-9, atol=1e-9)


def test_the_plain_short_convolution():
    h = torch.arange(12.0).view(6, 2)
    w = torch.tensor([[1.0, 10.0, 100.0], [0.0, 0.0, 1.0]])
    y = plain_model.short_conv(h, w)
    assert y[0].tolist() == [0.0 + 100 * 0.0, 1.0 + 1.0]          # only the last tap sees the first token
    assert y[2].tolist() == [4.0 + 1 * 0.0 + 10 * 2.0 + 100 * 4.0, 5.0 + 5.0]


# --------------------------------------------------------------------------- the engine on CPU stand-ins
@pytest.mark.parametrize("name", ["K1", "K2", "K3", "K4"])
def test_cuts_agree_with_the_plain_model(name, tmp_path_factory, cpu_ops):
    folder = model_folder(tmp_path_factory.getbasetemp(), name, ALL[name])
    plain = PlainKekopel(folder)
    toks = tokens_for(plain.vocab, 41, 7)
    want = plain.logits(toks)
    eng = make_engine(folder, "float32", "cpu", PAGE, pages=30)
    torch.testing.assert_close(replay_whole(eng, "w", toks), want, **TOL)
    torch.testing.assert_close(replay_cuts(eng, "c", toks, [5, 2, 11, 2, 3, 7]), want, **TOL)
    torch.testing.assert_close(replay_cuts(eng, "o", toks[:12], []), want[:12], **TOL)
    eng.cache.check()
    assert all(g.pool.free_count == g.pool.num_pages for g in eng.cache.paged)


def test_batches_of_unequal_requests_and_slots_used_again(tmp_path_factory, cpu_ops):
    folder = model_folder(tmp_path_factory.getbasetemp(), "K1", KEKO_1)
    plain = PlainKekopel(folder)
    lengths = {"r0": 25, "r1": 33, "r2": 18, "r3": 29, "r4": 21, "r5": 27}
    seqs = {r: tokens_for(plain.vocab, n, i) for i, (r, n) in enumerate(lengths.items())}
    eng = make_engine(folder, "float32", "cpu", PAGE, pages=4 * 10)
    got = replay_mixed(eng, seqs, mixed_schedule(lengths, seed=5))
    # (r1's first token has a query nearly at a right angle to its key in one matrix-memory head: the 32-bit sum k . q
    # loses two digits there, in any order of its terms, and nothing later in the sequence is touched by it)
    for r, toks in seqs.items():
        torch.testing.assert_close(got[r], plain.logits(toks), rtol=1e-4, atol=5e-5, msg=lambda m: f"{r}: {m}")
    assert eng.cache.slots.free_count == 4
    for g in eng.cache.paged:
        assert g.pool.handed_out > g.pool.num_pages


def test_a_slot_used_again_starts_from_nothing(tmp_path_factory, cpu_ops):
    """One request slot: every request gets the slot (and pages) of the one before; states and convolution inputs of
    the earlier owner must not leak."""
    folder = model_folder(tmp_path_factory.getbasetemp(), "K1", KEKO_1)
    plain = PlainKekopel(folder)
    eng = make_engine(folder, "float32", "cpu", PAGE, pages=12, reqs=1)
    for i in range(3):
        toks = tokens_for(plain.vocab, 20 + i, 30 + i)
        torch.testing.assert_close(replay_cuts(eng, f"r{i}", toks, [1, 1, 6, 2]), plain.logits(toks), **TOL)


def test_every_layer_hands_on_the_plain_models_stream(tmp_path_factory, cpu_ops):
    folder = model_folder(tmp_path_factory.getbasetemp(), "K1", KEKO_1)
    plain = PlainKekopel(folder)
    toks = tokens_for(plain.vocab, 19, 2)
    want = plain.streams(toks)
    eng = make_engine(folder, "float32", "cpu", PAGE, pages=30)
    seen = []
    blocks = eng.model.blocks
    for b in blocks:
        orig = b.forward

        def wrapped(x, residual, step, cache, writes, orig=orig):
            out = orig(x, residual, step, cache, writes)
            seen.append(residual.clone())
            return out

        b.forward = wrapped
    eng.step([StepEntry("a", toks, [len(toks) - 1])])
    for i in range(len(blocks)):
        torch.testing.assert_close(seen[i], want[i], **TOL, msg=lambda m: f"after layer {i}: {m}")


def plain_for_the_command_line(folder):
    from types import SimpleNamespace

    plain = PlainKekopel(folder)
    return SimpleNamespace(cfg=SimpleNamespace(vocab=plain.vocab), logits=lambda toks: plain.logits(toks).float())


def test_the_command_line_makes_a_model_generates_and_replays(tmp_path, capsys, cpu_ops):
    from test_cli import generate_and_replay, make_model

    folder = make_model(tmp_path, KEKO_1, capsys)
    generate_and_replay(folder, "cpu", "float32", capsys, tmp_path, plain_for_the_command_line(folder))
