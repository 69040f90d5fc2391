"""Nusudra on the GPU: each new kernel against its plain statement (tests/kernel_refs.py), inputs made so that a
sink or a distance bias left out, a key one place off or a lost state shows, and the engine (32-bit and bfloat16)
against the plain model (tests/plain/nusudra_plain.py) under every way of cutting and batching the work."""

import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import kernel_refs as ref
from freetoken_b200.engine.engine import StepEntry
from helpers import make_engine, mixed_schedule, model_folder, replay_cuts, replay_mixed, replay_whole, tokens_for
from plain.nusudra_plain import PlainNusudra
from test_pabavik_gpu import assert_rows, attention_problem, attn_tol
from tiny_nusudra import ALL, NUSU_1, NUSU_3, PAGE

from freetoken_b200.engine.attention_plan import build_plan
from freetoken_b200.kernels import ops
from freetoken_b200.parts.gla import chunk_list

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def rnd(*shape, dtype=torch.float32, scale=1.0, seed=0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


def tol(dtype, f32=1e-5, bf16=2e-2):
    return dict(rtol=f32, atol=f32) if dtype == torch.float32 else dict(rtol=bf16, atol=bf16)


def segs(lens):
    """``lens``: (q_len, kv_len) per request -> seg_info [S, 4] and slots 1..S on the device."""
    rows, q0 = [], 0
    for i, (q, kv) in enumerate(lens):
        rows.append((q0, q, kv, i))
        q0 += q
    return (torch.tensor(rows, dtype=torch.int32, device=DEV),
            torch.arange(1, len(lens) + 1, dtype=torch.int32, device=DEV), q0)


def cpu(t):
    return None if t is None else t.detach().cpu().clone()


# --------------------------------------------------------------------------- streams, branch mean
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("S,T,C", [(1, 5, 64), (2, 9, 90), (3, 33, 320), (4, 3, 1030), (8, 2, 4096), (3, 1, 7)])
def test_hyper_step_every_combination_of_its_steps(dtype, S, T, C):
    cap = T + 3  # the streams lie farther apart than a step's rows
    mix, out_w, in_w = rnd(S, S, seed=1, scale=0.6), rnd(S, seed=2), rnd(S, seed=3)
    norm_w = rnd(C, seed=4) + 1.0
    y = rnd(T, C, dtype=dtype, seed=5)
    init = rnd(T, C, seed=6)
    for kw in (dict(init=True, read=True), dict(write=True, read=True), dict(write=True), dict(write=True, total=True),
               dict(read=True), dict(init=True, write=True, read=True, total=True), dict(write=True, read=True, f32=True)):
        got_s = rnd(S, cap, C, seed=7)
        want_s = got_s.cpu().clone()
        hdt = torch.float32 if kw.get("f32") else dtype
        h = [torch.zeros(T, C, dtype=hdt, device=d) if kw.get("read") else None for d in (DEV, "cpu")]
        tot = [torch.zeros(T, C, device=d) if kw.get("total") else None for d in (DEV, "cpu")]
        for fn, st, hh, tt, mv in ((ops.hyper_step, got_s, h[0], tot[0], lambda t: t), (ref.hyper_step, want_s, h[1], tot[1], cpu)):
            fn(st[:, :T], init_from=mv(init) if kw.get("init") else None, y=mv(y) if kw.get("write") else None,
               mix=mv(mix) if kw.get("write") else None, out_w=mv(out_w) if kw.get("write") else None,
               in_w=mv(in_w) if kw.get("read") else None, norm_w=mv(norm_w) if kw.get("read") else None, eps=1e-5,
               h_out=hh, sum_out=tt)
        torch.testing.assert_close(got_s.cpu(), want_s, rtol=1e-5, atol=1e-5, msg=lambda m: f"{kw}: streams: {m}")
        if kw.get("read"):
            torch.testing.assert_close(h[0].float().cpu(), h[1].float(), **tol(hdt), msg=lambda m: f"{kw}: read: {m}")
        if kw.get("total"):
            torch.testing.assert_close(tot[0].cpu(), tot[1], rtol=1e-5, atol=1e-5)


def test_hyper_step_rows_past_the_step_stay_as_they_are():
    S, T, C = 3, 4, 64
    st = rnd(S, 9, C, seed=1)
    before = st.clone()
    ops.hyper_step(st[:, :T], y=rnd(T, C, seed=2), mix=rnd(S, S, seed=3), out_w=rnd(S, seed=4))
    torch.testing.assert_close(st[:, T:], before[:, T:], rtol=0, atol=0)
    assert not torch.equal(st[:, :T], before[:, :T])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n,T,C", [(1, 3, 64), (2, 17, 320), (3, 5, 90), (4, 2, 2050)])
def test_norm_mean(dtype, n, T, C):
    xs = [rnd(T, C, dtype=dtype, seed=i, scale=1.0 + i) for i in range(n)]
    ws = [rnd(C, seed=10 + i) for i in range(n)]
    got, want = torch.zeros(T, C, dtype=dtype, device=DEV), torch.zeros(T, C, dtype=dtype)
    ops.norm_mean(xs, ws, 1e-5, got)
    ref.norm_mean([cpu(x) for x in xs], [cpu(w) for w in ws], 1e-5, want)
    torch.testing.assert_close(got.float().cpu(), want.float(), **tol(dtype))


# --------------------------------------------------------------------------- convolution of projected rows
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("C,taps,off,bias,act", [(64, 4, 0, True, "silu"), (90, 3, 6, False, "silu"), (7, 2, 1, True, None),
                                               (512, 5, 8, False, "silu"), (1030, 16, 2, True, "silu"), (32, 1, 0, True, "silu"),
                                               (416, 4, 288, True, "silu")])
def test_conv_act_uses_and_advances_the_state(dtype, C, taps, off, bias, act):
    """Requests that start, requests that go on (their first outputs need the slot's rows), single tokens, portions
    shorter than the taps and longer than a tile, on a view of a wider projection's columns."""
    lens = [(37, 37), (1, 9), (2, 30), (taps, taps + 5), (1, 1), (17, 40), (1, 2)]
    info, slots, T = segs(lens)
    wide = rnd(T, off + C + 5, dtype=dtype, seed=1)
    x = wide[:, off:off + C]
    w = rnd(C, taps, seed=2, scale=0.5)
    b = rnd(C, seed=6) if bias else None
    st = rnd(len(lens) + 1, max(taps - 1, 1), C, seed=3) if taps > 1 else None
    for i, (q, kv) in enumerate(lens):  # a request that held fewer tokens than the state has rows: zeros before its start
        if taps > 1 and kv - q < taps - 1:
            st[i + 1, : taps - 1 - (kv - q)] = 0
    st_a, st_b = (st.clone(), st.clone().cpu()) if taps > 1 else (None, None)
    got = torch.zeros(T, C, dtype=dtype, device=DEV)
    want = torch.zeros(T, C, dtype=dtype)
    ops.conv_act(x, w, b, act, st_a, slots, info, len(lens), got)
    ref.conv_act(x.cpu(), w.cpu(), cpu(b), act, st_b, slots.cpu(), info.cpu(), len(lens), want)
    torch.testing.assert_close(got.float().cpu(), want.float(), **tol(dtype))
    if taps > 1:
        torch.testing.assert_close(st_a.cpu(), st_b, rtol=0, atol=0)


@pytest.mark.parametrize("cuts", [[50], [1] * 50, [2, 3, 16, 17, 1, 11], [15, 1, 16, 2, 16]])
def test_conv_act_cut_anywhere_is_the_whole(cuts):
    C, taps, T = 48, 4, 50
    x, w, b = rnd(T, C, seed=4), rnd(C, taps, seed=5), rnd(C, seed=6)
    state = torch.full((2, taps - 1, C), 7.0, device=DEV)  # the slot's earlier owner left something behind
    whole = torch.zeros(T, C, device=DEV)
    info, slots, _ = segs([(T, T)])
    ops.conv_act(x, w, b, "silu", state.clone(), slots, info, 1, whole)
    got, i = [], 0
    for c in cuts:
        c = min(c, T - i)
        if c <= 0:
            break
        info, slots, _ = segs([(c, i + c)])
        out = torch.zeros(c, C, device=DEV)
        ops.conv_act(x[i:i + c].contiguous(), w, b, "silu", state, slots, info, 1, out)
        got.append(out)
        i += c
    torch.testing.assert_close(torch.cat(got), whole[:i], rtol=1e-6, atol=1e-6)


# --------------------------------------------------------------------------- state space
@pytest.mark.parametrize("dtype", DTYPES)
def test_state_space_gates_and_output(dtype):
    T, H, P = 19, 6, 10
    wide = rnd(T, 3 + H + 2, dtype=dtype, seed=1, scale=2.0)
    dt_bias, a_log = rnd(H, seed=2), rnd(H, seed=3)
    got = [torch.zeros(T, H, device=DEV) for _ in range(2)]
    want = [torch.zeros(T, H) for _ in range(2)]
    ops.ssm_gates(wide[:, 3:3 + H], dt_bias, a_log, *got)
    ref.ssm_gates(wide[:, 3:3 + H].cpu(), dt_bias.cpu(), a_log.cpu(), *want)
    for g, w in zip(got, want):
        torch.testing.assert_close(g.cpu(), w, rtol=1e-5, atol=1e-6)
    assert float(got[1].max()) <= 1.0 and float(got[0].min()) > 0.0
    for groups in (1, 2, 3, 6):
        o32 = rnd(T, H, P, seed=4)
        rows = rnd(T, 2 * H * P + 4, dtype=dtype, seed=5)
        x, z = rows[:, 4:4 + H * P], rows[:, 4 + H * P:]
        d, nw = rnd(H, seed=6), rnd(H * P, seed=7) + 1.0
        out, ow = torch.zeros(T, H * P, dtype=dtype, device=DEV), torch.zeros(T, H * P, dtype=dtype)
        ops.ssm_output(o32, x, d, z, nw, groups, 1e-5, out)
        ref.ssm_output(o32.cpu(), x.cpu(), d.cpu(), z.cpu(), nw.cpu(), groups, 1e-5, ow)
        torch.testing.assert_close(out.float().cpu(), ow.float(), **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,N,P", [(6, 2, 32, 48), (4, 1, 16, 8), (3, 3, 24, 6), (8, 2, 128, 64), (2, 1, 6, 30)])
def test_the_recurrence_with_queries_and_keys_shared_by_groups_of_heads(dtype, H, G, N, P):
    """The state-space recurrence on the kernel of gated linear attention: keys times a step size, one decay per
    (token, head), queries and keys of a group under several heads; requests of one chunk and of several, from given states."""
    lens = [(150, 150), (1, 40), (70, 100), (2, 2), (64, 64)]
    info, slots, T = segs(lens)
    rows = rnd(T, P * H + 2 * G * N, dtype=dtype, seed=1)
    v, k, q = rows[:, :H * P], rows[:, H * P:H * P + G * N], rows[:, H * P + G * N:]
    step = torch.rand(T, H, generator=torch.Generator().manual_seed(2)).to(DEV) * 0.5
    dec = torch.exp(-torch.rand(T, H, generator=torch.Generator().manual_seed(3)).to(DEV) * 0.3)
    state = rnd(len(lens) + 1, H, N, P, seed=4)
    chunks, per_seg, single, multi = chunk_list(lens, 64)
    n_chunks = chunks.shape[0]
    ch, ps = torch.from_numpy(chunks).to(DEV), torch.from_numpy(per_seg).to(DEV)
    carry = torch.zeros(n_chunks, H, N, P, device=DEV)
    dprod = torch.zeros(n_chunks, H, N, device=DEV)
    got, want = torch.zeros(T, H, P, device=DEV), torch.zeros(T, H, P)
    st_a, st_b = state.clone(), state.cpu().clone()
    ops.gla_scan(q, k, v, None, None, 1.0, 1.0, st_a, slots, info, len(lens), ch, n_chunks, ps, single, multi, carry, dprod,
                 got, k_fac=step, a_head=dec, qk_div=H // G)
    ref.gla_scan(q.cpu(), k.cpu(), v.cpu(), None, None, 1.0, 1.0, st_b, slots.cpu(), info.cpu(), len(lens), None, 0, None,
                 single, multi, None, None, want, k_fac=step.cpu(), a_head=dec.cpu(), qk_div=H // G)
    torch.testing.assert_close(got.cpu(), want, rtol=2e-4, atol=2e-4)
    torch.testing.assert_close(st_a.cpu()[1:], st_b[1:], rtol=2e-4, atol=2e-4)


# --------------------------------------------------------------------------- delta rule
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,D,Dv", [(4, 4, 32, 64), (4, 2, 16, 24), (3, 1, 40, 10), (2, 2, 8, 33), (1, 1, 128, 128),
                                      (2, 1, 200, 70), (6, 3, 6, 5), (8, 2, 128, 128), (8, 4, 96, 104)])  # (the last two: the form
# with two lanes a column, which steps with thousands of columns take)
def test_delta_rule_against_the_stated_recurrence(dtype, H, G, D, Dv):
    lens = [(45, 45), (1, 40), (17, 100), (2, 2), (1, 1), (33, 64)]
    info, slots, T = segs(lens)
    rows = rnd(T, 2 * G * D + H * Dv + 2 * H + 3, dtype=dtype, seed=1)
    q, k = rows[:, :G * D], rows[:, G * D:2 * G * D]
    v = rows[:, 2 * G * D:2 * G * D + H * Dv]
    b, a = rows[:, -2 * H - 3:-H - 3], rows[:, -H - 3:-3]
    a_log, dt_bias = rnd(H, seed=2, scale=0.5) - 1.0, rnd(H, seed=3)
    state = rnd(len(lens) + 1, H, Dv, D, seed=4, scale=0.3)
    st_a, st_b = state.clone(), state.cpu().clone()
    got, want = torch.zeros(T, H, Dv, device=DEV), torch.zeros(T, H, Dv)
    ops.delta_scan(q, k, v, b, a, a_log, dt_bias, D ** -0.5, 1e-6, st_a, slots, info, len(lens), got)
    ref.delta_scan(q.cpu(), k.cpu(), v.cpu(), b.cpu(), a.cpu(), a_log.cpu(), dt_bias.cpu(), D ** -0.5, 1e-6, st_b, slots.cpu(),
                   info.cpu(), len(lens), want)
    torch.testing.assert_close(got.cpu(), want, rtol=2e-4, atol=2e-5)
    torch.testing.assert_close(st_a.cpu()[1:], st_b[1:], rtol=2e-4, atol=2e-5)
    # requests whose first tokens these are start from zero, whatever the slot held
    for i, (ql, kv) in enumerate(lens):
        if ql == kv and ql == 1:
            t = int(info[i, 0])
            assert torch.isfinite(got[t]).all()


@pytest.mark.parametrize("cuts", [[700], [333, 2, 365], [64, 64, 1, 1, 570], [699, 1], [16, 17, 15, 1, 651]])
def test_a_value_written_once_is_read_hundreds_of_tokens_later(cuts):
    """Token 3 writes a value along a key that no later token touches (the others' keys lie in other channels, decays
    are near one); token 699 asks for it.  A state lost or restarted at any cut loses the value."""
    H, G, D, Dv, T = 2, 1, 16, 8, 700
    g = torch.Generator().manual_seed(5)
    k = torch.zeros(T, D)
    k[:, 1:] = torch.randn(T, D - 1, generator=g)
    k[3] = 0
    k[3, 0] = 5.0
    q = torch.randn(T, D, generator=g) * 0.1
    q[T - 1] = 0
    q[T - 1, 0] = 4.0
    v = torch.randn(T, H * Dv, generator=g)
    v[3] = torch.arange(1, H * Dv + 1).float()
    b = torch.full((T, H), 4.0)   # beta near one
    a = torch.full((T, H), -9.0)  # softplus near zero: decays near one
    a_log, dt_bias = torch.zeros(H), torch.zeros(H)
    dev = lambda t: t.to(DEV).contiguous()  # noqa: E731
    state = torch.full((2, H, Dv, D), 3.0, device=DEV)
    outs, i = [], 0
    for c in cuts:
        info, slots, _ = segs([(c, i + c)])
        o = torch.zeros(c, H, Dv, device=DEV)
        ops.delta_scan(dev(q[i:i + c]), dev(k[i:i + c]), dev(v[i:i + c]), dev(b[i:i + c]), dev(a[i:i + c]), dev(a_log), dev(dt_bias),
                       1.0, 1e-6, state, slots, info, 1, o)
        outs.append(o)
        i += c
    got = torch.cat(outs).cpu()
    want = torch.zeros(T, H, Dv)
    info, slots, _ = segs([(T, T)])
    ref.delta_scan(q, k, v, b, a, a_log, dt_bias, 1.0, 1e-6, torch.zeros(2, H, Dv, D), slots.cpu(), info.cpu(), 1, want)
    torch.testing.assert_close(got, want, rtol=1e-4, atol=1e-4)
    read = got[T - 1].reshape(-1)
    kept = float(torch.sigmoid(torch.tensor(4.0))) * float(torch.exp(-torch.nn.functional.softplus(torch.tensor(-9.0)))) ** (T - 4)
    assert float((read - torch.arange(1, H * Dv + 1).float() * kept).abs().max()) < 0.05, read


# --------------------------------------------------------------------------- attention: bias by distance, sink per head
def run_biased(dtype, Hq, Hkv, D, P, lens, tile, r1, r2, sink, scale, problem=None, force_split=False):
    q, ks, vs, bt, seg = problem or attention_problem(dtype, Hq, Hkv, D, P, lens)
    kw = dict(sm_count=4096, min_split_keys=32) if force_split else dict(sm_count=148)
    if tile == 128:
        kw["key_tile"] = 128  # as the engine plans the tcgen05 kernel's work
    plan = build_plan(lens, Hq // Hkv, tile, None, Hkv, **kw)
    items = torch.from_numpy(plan.items).to(DEV)
    part_o = part_ml = None
    if plan.n_slots:
        part_o = torch.full((plan.n_slots, Hkv, tile, D), float("nan"), dtype=torch.float32, device=DEV)
        part_ml = torch.full((plan.n_slots, Hkv, tile, 2), float("nan"), dtype=torch.float32, device=DEV)
    longest = max(kv for _, kv in lens)
    d = torch.arange(longest, dtype=torch.float64)[None, :]
    table = (-r1.double()[:, None] * torch.log1p(r2.double()[:, None] * d)).float().to(DEV)
    out = torch.full(q.shape, float("nan"), dtype=dtype, device=DEV)
    want = torch.empty_like(out)
    ops.paged_attention(q, ks, vs, bt, seg, len(lens), items, plan.n_items, part_o, part_ml, out, tile, scale, None,
                        dist_bias=table, sink=sink)
    ref.paged_attention(q, ks, vs, bt, seg, len(lens), items, plan.n_items, None, None, want, tile, scale, None,
                        dist_bias=table, sink=sink)
    return out, want, table


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("Hq,Hkv,D,P,split", [(4, 4, 64, 16, False), (4, 2, 16, 4, False), (6, 3, 32, 8, True), (1, 1, 48, 16, False),
                                             (8, 2, 128, 16, True)])
def test_attention_with_a_log_distance_bias_and_a_sink_per_head(dtype, Hq, Hkv, D, P, split):
    lens = [(1, 1), (5, 5), (70, 70), (2, 131), (1, 64), (33, 97), (1, 300)]
    r1 = torch.rand(Hq, generator=torch.Generator().manual_seed(1)) + 0.2
    r2 = torch.rand(Hq, generator=torch.Generator().manual_seed(2)) + 0.05
    sink = rnd(Hq, seed=3)
    for tile in ([16] if dtype == torch.float32 else [16, 64]):
        out, want, _ = run_biased(dtype, Hq, Hkv, D, P, lens, tile, r1, r2, sink, 0.8 * D ** -0.5, force_split=split)
        torch.testing.assert_close(out.float().cpu(), want.float().cpu(), **attn_tol(dtype))


@pytest.mark.parametrize("Hq,Hkv,P,split", [(4, 4, 16, False), (8, 2, 16, True), (16, 1, 32, False), (6, 3, 64, True)])
def test_the_tensor_core_kernel_takes_the_bias_and_the_sink_together(Hq, Hkv, P, split):
    """Heads of 128 in steps of 128 tokens and more: long portions, portions behind hundreds of cached tokens, tiles cut
    along the keys (the sink then joins in the merge), beside single tokens."""
    lens = [(300, 300), (130, 700), (1, 64), (128, 128), (2, 515)]
    r1 = torch.rand(Hq, generator=torch.Generator().manual_seed(1)) + 0.2
    r2 = torch.rand(Hq, generator=torch.Generator().manual_seed(2)) + 0.05
    sink = rnd(Hq, seed=3) + 1.0
    ops.variant_counts(reset=True)
    out, want, _ = run_biased(torch.bfloat16, Hq, Hkv, 128, P, lens, 128, r1, r2, sink, 0.8 * 128 ** -0.5, force_split=split)
    assert ops.variant_counts().get("attention: tcgen05, 128-row query tiles, bias by distance", 0) == 1
    torch.testing.assert_close(out.float().cpu(), want.float().cpu(), **attn_tol(torch.bfloat16))
    no_sink, _, _ = run_biased(torch.bfloat16, Hq, Hkv, 128, P, lens, 128, r1, r2, None, 0.8 * 128 ** -0.5, force_split=split)
    assert float((no_sink.float() - out.float()).abs().max()) > 0.05  # the sink is not lost on the way


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_far_key_that_stands_out_feels_the_distance_bias_and_the_sink(dtype):
    """One key 250 places back is made to match the query (score about 12 above the rest); with the bias by distance
    it wins or loses by ``r1 ln(1 + 250 r2)``, and a large sink takes the weight from a head's keys altogether."""
    Hq, Hkv, D, P = 3, 1, 32, 16
    lens = [(1, 300)]
    q, ks, vs, bt, seg = attention_problem(dtype, Hq, Hkv, D, P, lens, seed=4, scale_k=0.1)
    far = 300 - 1 - 250
    page = int(bt[1, far // P])
    ks[page, 0, far % P] = 0
    ks[page, 0, far % P, 0] = 6.0
    q[:] = 0
    q[:, :, 0] = 2.0
    r1 = torch.tensor([0.0, 4.0, 0.0])   # head 1: the far key is pushed below the others
    r2 = torch.tensor([1.0, 1.0, 1.0])
    sink = torch.tensor([-30.0, -30.0, 30.0], device=DEV)  # head 2: the sink takes everything
    out, want, table = run_biased(dtype, Hq, Hkv, D, P, lens, 16, r1, r2, sink, 1.0, problem=(q, ks, vs, bt, seg))
    torch.testing.assert_close(out.float().cpu(), want.float().cpu(), **attn_tol(dtype))
    v_far = vs[page, 0, far % P].float().cpu()
    o = out[0].float().cpu()
    assert float((o[0] - v_far).abs().max()) < 0.05          # head 0 reads the far key's value alone
    assert float((o[1] - v_far).abs().max()) > 0.3           # head 1 does not: 4 ln(251) = 22 > 12
    assert float(o[2].abs().max()) < 1e-3                    # head 2 reads nothing


# --------------------------------------------------------------------------- the engine against the plain model
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["N1", "N2", "N3", "N4"])
def test_cuts_and_batches_agree_with_the_plain_model(name, dtype, tmp_path_factory):
    folder = model_folder(tmp_path_factory.getbasetemp(), name, ALL[name])
    plain = PlainNusudra(folder)
    eng = make_engine(folder, dtype, DEV, 16 if name == "N3" else PAGE, pages=40)
    toks = tokens_for(plain.vocab, 70, 11)
    want = plain.logits(toks)
    assert_rows(replay_whole(eng, "w", toks), want, dtype, "whole")
    assert_rows(replay_cuts(eng, "d", toks, [38]), want, dtype, "last 32 one by one")
    assert_rows(replay_cuts(eng, "c", toks, [7, 2, 13, 2, 5, 3, 2, 11, 2]), want, dtype, "portions")
    assert_rows(replay_cuts(eng, "one", toks[:24], []), want[:24], dtype, "one by one from the first token")
    eng.cache.check()
    eng.check_kernels()
    assert all(g.pool.free_count == g.pool.num_pages for g in eng.cache.paged)


def test_every_layer_leaves_the_plain_models_streams(tmp_path_factory):
    """Random tensors are drawn by name, so a model of the first n layers has the full model's weights: its logits say
    whether the sum of the streams after layer n is right."""
    for n in (1, 2, 3, 4):
        raw = dict(NUSU_1, layers=NUSU_1["layers"][:n])
        folder = model_folder(tmp_path_factory.getbasetemp(), f"N1_first{n}", raw)
        plain = PlainNusudra(folder)
        toks = tokens_for(plain.vocab, 40, 5)
        eng = make_engine(folder, "float32", DEV, PAGE, pages=40)
        assert_rows(replay_cuts(eng, "c", toks, [9, 2, 20]), plain.logits(toks), "float32", f"{n} layers")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["N1", "N4"])
def test_mixed_steps_with_few_pages_and_slots(name, dtype, tmp_path_factory):
    folder = model_folder(tmp_path_factory.getbasetemp(), name, ALL[name])
    plain = PlainNusudra(folder)
    lengths = {"r0": 45, "r1": 60, "r2": 38, "r3": 52, "r4": 41, "r5": 47}
    seqs = {r: tokens_for(plain.vocab, n, i) for i, (r, n) in enumerate(lengths.items())}
    eng = make_engine(folder, dtype, DEV, PAGE, pages=4 * (-(-64 // PAGE)))
    got = replay_mixed(eng, seqs, mixed_schedule(lengths, seed=3))
    for r, toks in seqs.items():
        assert_rows(got[r], plain.logits(toks), dtype, r)
    for g in eng.cache.paged:
        assert g.pool.handed_out > g.pool.num_pages, "the trace was meant to use pages again"
    assert eng.cache.slots.free_count == 4


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["N1", "N3"])
def test_long_prompt_long_decoding_and_recorded_steps(name, dtype, tmp_path_factory):
    """Hundreds of tokens across many pages and chunks, a hundred tokens one by one (recorded into a CUDA graph at the
    first), and a long step in between."""
    folder = model_folder(tmp_path_factory.getbasetemp(), name, ALL[name])
    plain = PlainNusudra(folder)
    toks = tokens_for(plain.vocab, 300, 3)
    want = plain.logits(toks)
    eng = make_engine(folder, dtype, DEV, 16, pages=64, max_step=512)
    assert_rows(replay_whole(eng, "w", toks), want, dtype, "whole")
    assert_rows(replay_cuts(eng, "d", toks, [200]), want, dtype, "a hundred tokens one by one")
    assert eng.graphs, "the decode steps were meant to be recorded"
    assert_rows(replay_cuts(eng, "c", toks, [63, 2, 64, 65, 17, 2, 33] + [1] * 20 + [30, 2]), want, dtype, "portions")
    other = tokens_for(plain.vocab, 130, 5)
    got = [eng.step([StepEntry("a", toks[:3], [0, 1, 2])]).logits.float().cpu().clone()]
    for i in range(3, 12):
        got.append(eng.step([StepEntry("a", toks[i:i + 1], [0])]).logits.float().cpu().clone())
    long = eng.step([StepEntry("b", other, list(range(len(other))))]).logits.float().cpu().clone()
    for i in range(12, 40):
        got.append(eng.step([StepEntry("a", toks[i:i + 1], [0])]).logits.float().cpu().clone())
    assert_rows(long, plain.logits(other), dtype, "the long step")
    assert_rows(torch.cat(got), want[:40], dtype, "decode steps before and after it")
    eng.check_kernels()


def test_long_steps_of_latent_rows_of_128_run_the_tensor_core_attention(tmp_path_factory):
    folder = model_folder(tmp_path_factory.getbasetemp(), "N3", NUSU_3)
    plain = PlainNusudra(folder)
    toks = tokens_for(plain.vocab, 300, 9)
    want = plain.logits(toks)
    eng = make_engine(folder, "bfloat16", DEV, 16, pages=96, max_step=512)
    ops.variant_counts(reset=True)
    assert_rows(replay_whole(eng, "w", toks), want, "bfloat16", "whole")
    assert any("tcgen05" in k and n for k, n in ops.variant_counts().items() if k.startswith("attention")), ops.variant_counts()
    assert_rows(replay_cuts(eng, "c", toks, [150, 130, 2]), want, "bfloat16", "portions, the rest one by one")
    others = {f"o{i}": tokens_for(plain.vocab, 20 + i, 20 + i) for i in range(3)}
    for r, t in others.items():  # three requests that decode beside a long portion
        eng.step([StepEntry(r, t[:-1], [])])
    out = eng.step([StepEntry("long", toks[:200], list(range(200)))] + [StepEntry(r, t[-1:], [0]) for r, t in others.items()])
    assert_rows(out.logits[:200], want[:200], "bfloat16", "a long portion beside single tokens")
    for i, (r, t) in enumerate(others.items()):
        assert_rows(out.logits[200 + i:201 + i], plain.logits(t)[-1:], "bfloat16", r)
    eng.check_kernels()


REAL_LAYERS = {  # layers of the size of a real model's (no test of the tiny configurations reaches these kernel forms)
    "architecture": "Nusudra", "vocab": 8192, "width": 2048, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0}, "streams": 4,
    "layers": [
        {"type": "parallel", "mixer": {"left": {"heads": 16, "kv_heads": 4, "dim": 128, "vdim": 128, "scale": 128 ** -0.5},
                                       "right": {"heads": 32, "vdim": 64, "state": 128, "groups": 4, "conv": 4, "norm_groups": 4}},
         "mlp": {"kind": "dense", "ff": 4096}},
        {"type": "delta", "mixer": {"heads": 48, "kv_heads": 8, "dim": 128, "vdim": 128, "conv": 4}, "mlp": {"kind": "dense", "ff": 4096}},
        {"type": "latent_attention", "mixer": {"heads": 16, "dim": 128, "rot_dim": 64, "vdim": 128, "kv_rank": 64, "scale": 192 ** -0.5,
                                               "rot": {"dims": 64, "base": 1000000.0}}, "mlp": None},
    ]}


def test_layers_of_real_sizes_agree_across_cuts_and_dtypes():
    """Heads of 128, thousands of state columns, long portions: the pair's attention with bias and sink and the latent
    attention on the tcgen05 kernels, the delta rule in its form for many columns, the recurrences' chunks side by side.
    No plain model at these sizes: the 32-bit engine is compared with itself across cuts, the bfloat16 engine with it."""
    from freetoken_b200.config.engine_config import EngineConfig
    from freetoken_b200.engine.engine import Engine
    from test_pabavik_gpu import row_error

    toks = tokens_for(REAL_LAYERS["vocab"], 600, 4)
    seen = sorted(set(range(0, 600, 7)) | set(range(560, 600)))

    def rows(eng, rid, cuts):
        got, i, cuts = {}, 0, list(cuts)
        while i < len(toks):
            c = min(cuts.pop(0) if cuts else 1, len(toks) - i)
            want = [p - i for p in seen if i <= p < i + c]
            out = eng.step([StepEntry(rid, toks[i:i + c], want)])
            for j, w in enumerate(want):
                got[w + i] = out.logits[j].float().cpu().clone()
            i += c
        eng.close(rid)
        return torch.stack([got[p] for p in seen])

    res = {}
    for dtype in ("float32", "bfloat16"):
        eng = Engine(EngineConfig(model_path="", dtype=dtype, use_dummy_weight=True, seed=3, page_size=16, max_running_req=4,
                                  num_page_override=100, max_seq_len_override=1024, max_extend_tokens=640, max_step_tokens=640,
                                  check_cache=True), raw_config=REAL_LAYERS)
        ops.variant_counts(reset=True)
        res[dtype, "whole"] = rows(eng, "w", [600])
        if dtype == "bfloat16":
            forms = ops.variant_counts()
            assert forms.get("attention: tcgen05, 128-row query tiles, bias by distance", 0) == 1, forms
            assert forms.get("attention: tcgen05, 128-row query tiles", 0) >= 1, forms
        res[dtype, "cuts"] = rows(eng, "c", [300, 256, 2, 7])
        eng.check_kernels()
        del eng
        torch.cuda.empty_cache()
    assert torch.isfinite(res["float32", "whole"]).all()
    assert float(row_error(res["float32", "cuts"], res["float32", "whole"]).max()) < 1e-4
    assert float(row_error(res["bfloat16", "whole"], res["float32", "whole"]).max()) < 0.08
    assert float(row_error(res["bfloat16", "cuts"], res["float32", "whole"]).max()) < 0.08
    assert float(row_error(res["bfloat16", "whole"], res["float32", "whole"]).median()) < 0.03


def test_greedy_generation_through_the_scheduler(tmp_path_factory):
    from freetoken_b200 import LLM, SamplingParams

    folder = model_folder(tmp_path_factory.getbasetemp(), "N1", NUSU_1)
    plain = PlainNusudra(folder)
    prompts = [[5, 17, 3, 150, 41], [9, 8, 7, 6, 5, 4, 3, 2, 1, 0, 11, 12], [199]]
    for dtype in ("float32", "bfloat16"):
        llm = LLM(folder, dtype=dtype, device=DEV, page_size=4, num_page_override=48, max_step_tokens=8,
                  max_extend_tokens=8, max_running_req=2)  # three prompts on two request slots, in portions of eight
        outs = llm.generate(prompts, SamplingParams(max_tokens=10))
        for p, o in zip(prompts, outs):
            toks = list(p)
            assert len(o["token_ids"]) == 10
            for got in o["token_ids"]:
                logits = plain.logits(toks)[-1]
                top2 = torch.topk(logits, 2).values
                if dtype == "float32" or float(top2[0] - top2[1]) > 0.1:
                    assert got == int(torch.argmax(logits)), (dtype, p, o)
                toks.append(got)


def test_the_replay_tool_runs_the_design(tmp_path_factory, tmp_path):
    folder = model_folder(tmp_path_factory.getbasetemp(), "N4", ALL["N4"])
    plain = PlainNusudra(folder)
    a, b = tokens_for(plain.vocab, 30, 1), tokens_for(plain.vocab, 9, 2)
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": a[:20], "want": [0, 19]}, {"id": "b", "tokens": b[:2], "want": []}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": a[20:21], "want": [0]}, {"id": "b", "tokens": b[2:], "want": [6]}], "end": ["b"]},
        {"step": 2, "entries": [{"id": "a", "tokens": a[21:], "want": [8]}], "end": ["a"]},
    ]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for dtype in ("float32", "bfloat16"):
        out = tmp_path / dtype
        p = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", folder, "--dtype", dtype,
                            "--out", str(out), "--max-tokens", "128"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                           capture_output=True, text=True, timeout=600)
        assert p.returncode == 0, p.stderr[-2000:]
        assert [l for l in p.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
        la, lb = plain.logits(a), plain.logits(b)
        got = [np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(-1, plain.vocab) for i in range(3)]
        assert_rows(torch.from_numpy(got[0]), la[[0, 19]], dtype, "step 0")
        assert_rows(torch.from_numpy(got[1]), torch.stack([la[20], lb[8]]), dtype, "step 1")
        assert_rows(torch.from_numpy(got[2]), la[[29]], dtype, "step 2")
