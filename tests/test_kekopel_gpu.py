"""Kekopel on the GPU: each new kernel against its plain statement (tests/kernel_refs.py), inputs made so that a
sink left out, a window one token off or a lost state shows, and the engine (32-bit and bfloat16) against the plain
model (tests/plain/kekopel_plain.py) under every way of cutting and batching the work."""

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
from plain.kekopel_plain import PlainKekopel
from test_pabavik_gpu import assert_rows, attention_problem, attn_tol
from test_pabavik_gpu import run_attention as run_attention_case
from tiny_kekopel import ALL, KEKO_1, PAGE

from freetoken_b200.engine.attention_plan import build_plan
from freetoken_b200.kernels import ops
from freetoken_b200.parts.gla import chunk_list

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]
# K5's attention is sharp on purpose: what bfloat16 adds to a score is multiplied up, and so is what reaches the routers;
# its router margins count as near-ties four times as far out
SHARP = {"K5": 0.25}


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


# --------------------------------------------------------------------------- short convolution, depth mix, small ones
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("C,taps", [(64, 4), (90, 3), (7, 2), (512, 5), (1030, 16), (32, 1)])
def test_short_conv_uses_and_advances_the_state(dtype, C, taps):
    """Requests that start, requests that go on (their first outputs need the slot's rows), single tokens, portions
    shorter than the taps and longer than a tile; the kernel's state after the step is the plain one's."""
    lens = [(37, 37), (1, 9), (2, 30), (taps, taps + 5), (1, 1), (17, 40)]
    info, slots, T = segs(lens)
    x = rnd(T, C, seed=1)
    w = rnd(C, taps, seed=2, scale=0.5)
    st = rnd(len(lens) + 1, max(taps - 1, 1), C, seed=3) if taps > 1 else None
    for i, (q, kv) in enumerate(lens):  # a request that held fewer tokens than the state has rows: zeros before its start
        if taps > 1 and kv - q < taps - 1:
            st[i + 1, : taps - 1 - (kv - q)] = 0
    st_a, st_b = (st.clone(), st.clone().cpu()) if taps > 1 else (None, None)
    got = torch.zeros(T, C, dtype=dtype, device=DEV)
    want = torch.zeros(T, C, dtype=dtype)
    ops.short_conv(x, w, st_a, slots, info, len(lens), got)
    ref.short_conv(x.cpu(), w.cpu(), st_b, slots.cpu(), info.cpu(), len(lens), want)
    torch.testing.assert_close(got.float().cpu(), want.float(), **tol(dtype))
    if taps > 1:
        torch.testing.assert_close(st_a.cpu(), st_b, rtol=0, atol=0)


@pytest.mark.parametrize("cuts", [[50], [1] * 50, [2, 3, 16, 17, 1, 11], [15, 1, 16, 2, 16]])
def test_short_conv_cut_anywhere_is_the_whole(cuts):
    C, taps, T = 48, 4, 50
    x, w = rnd(T, C, seed=4), rnd(C, taps, seed=5)
    whole = torch.zeros(T, C, device=DEV)
    info, slots, _ = segs([(T, T)])
    st = torch.full((2, taps - 1, C), 7.0, device=DEV)  # what an earlier owner of the slot left: never read
    ops.short_conv(x, w, st, slots, info, 1, whole)
    st2 = torch.full((2, taps - 1, C), -3.0, device=DEV)
    got, t0 = torch.zeros(T, C, device=DEV), 0
    for n in cuts:
        info, slots, _ = segs([(n, t0 + n)])
        part = torch.zeros(n, C, device=DEV)
        ops.short_conv(x[t0:t0 + n].contiguous(), w, st2, slots, info, 1, part)
        got[t0:t0 + n] = part
        t0 += n
    torch.testing.assert_close(got, whole, rtol=0, atol=0)
    torch.testing.assert_close(st2[1], st[1], rtol=0, atol=0)


@pytest.mark.parametrize("T,C,n", [(5, 64, 0), (33, 90, 3), (7, 1030, 6)])
def test_depth_mix(T, C, n):
    cap = T + 3
    hist = rnd(n + 2, cap, C, seed=1)
    x, mix = rnd(T, C, seed=2), rnd(n + 1, seed=3)
    ha, hb, xa, xb = hist.clone(), hist.clone().cpu(), x.clone(), x.clone().cpu()
    ops.depth_mix(ha, n, mix, xa)
    ref.depth_mix(hb, n, mix.cpu(), xb)
    torch.testing.assert_close(xa.cpu(), xb, rtol=1e-6, atol=1e-6)
    torch.testing.assert_close(ha.cpu(), hb, rtol=0, atol=0)


@pytest.mark.parametrize("dtype", DTYPES)
def test_scaled_gather_and_squared_relu(dtype):
    T, H, k = 9, 70, 3
    h = rnd(T, H, dtype=dtype, seed=1)
    routes = torch.randperm(T * k, generator=torch.Generator().manual_seed(2)).to(torch.int32).to(DEV)
    w = rnd(T * k, seed=3).abs()
    got, want = torch.zeros(T * k, H, dtype=dtype, device=DEV), torch.zeros(T * k, H, dtype=dtype)
    ops.moe_gather_scaled(h, routes, w, k, got)
    ref.moe_gather_scaled(h.cpu(), routes.cpu(), w.cpu(), k, want)
    torch.testing.assert_close(got.cpu().float(), want.float(), **tol(dtype, bf16=1e-2))
    a = rnd(T, H, dtype=dtype, seed=4)
    b = a.clone().cpu()
    ops.relu2_(a)
    ref.relu2_(b)
    torch.testing.assert_close(a.cpu().float(), b.float(), **tol(dtype, bf16=1e-2))


@pytest.mark.parametrize("E,k,T", [(8, 1, 7), (5, 2, 40), (3, 3, 4), (64, 6, 33)])
def test_router_keeps_the_raw_sigmoid_scores(E, k, T):
    logits = rnd(T, E, seed=1, scale=2.0)
    ids, wts = torch.zeros(T, k, dtype=torch.int32, device=DEV), torch.zeros(T, k, device=DEV)
    ops.router_topk(logits, None, k, "sigmoid_raw", 1.0, ids, wts)
    top = torch.topk(torch.sigmoid(logits), k, dim=-1)
    assert torch.equal(ids.long(), top.indices)
    torch.testing.assert_close(wts, top.values, rtol=1e-6, atol=1e-6)  # not divided by their sum


# --------------------------------------------------------------------------- latent attention
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("Q,C,R,n_rot,inter,pad", [(80, 112, 16, 16, True, 128), (24, 40, 8, 4, True, 48), (18, 22, 6, 6, True, 32),
                                                    (16, 24, 16, 16, False, 48), (12, 16, 8, 0, True, 32), (300, 200, 56, 56, True, 256)])
def test_latent_rows_and_queries(dtype, Q, C, R, n_rot, inter, pad):
    T, H, D, P, pages = 11, 3, 10, 4, 9
    proj = rnd(T, Q + C + R, dtype=dtype, seed=1, scale=2.0)
    wq, wkv = rnd(Q, seed=2) + 1.0, rnd(C, seed=3) + 1.0
    pos = torch.tensor([0, 1, 2, 3, 30, 31, 32, 5, 6, 63, 7], dtype=torch.int32, device=DEV)
    table = None
    if n_rot:
        ang = torch.arange(64, dtype=torch.float64)[:, None] * 100.0 ** (-torch.arange(0, n_rot, 2, dtype=torch.float64) / n_rot)
        table = torch.cat([ang.cos(), ang.sin()], -1).float().to(DEV).contiguous()
    slot_map = torch.tensor([4, 5, 6, 7, 20, 21, -1, 9, 10, 35, 0], dtype=torch.int32, device=DEV)  # one row is not stored
    slabs = [torch.full((pages, 1, P, pad), 5.0, dtype=dtype, device=DEV), torch.full((pages, 1, P, pad), 5.0, dtype=dtype)]
    cqs = [torch.zeros(T, Q, dtype=dtype, device=DEV), torch.zeros(T, Q, dtype=dtype)]
    ops.latent_store(proj, Q, C, R, n_rot, inter, wq, wkv, 1e-5, pos, table, cqs[0], slabs[0], slot_map)
    ref.latent_store(proj.cpu(), Q, C, R, n_rot, inter, wq.cpu(), wkv.cpu(), 1e-5, pos.cpu(),
                     table.cpu() if n_rot else None, cqs[1], slabs[1], slot_map.cpu())
    torch.testing.assert_close(cqs[0].cpu().float(), cqs[1].float(), **tol(dtype))
    torch.testing.assert_close(slabs[0].cpu().float(), slabs[1].float(), **tol(dtype))
    q = rnd(T, H, D + R, dtype=dtype, seed=5)
    outs = [torch.full((T, H, pad), 3.0, dtype=dtype, device=DEV), torch.full((T, H, pad), 3.0, dtype=dtype)]
    ops.latent_query_rotate(q, D, R, n_rot, inter, pos, table, outs[0], C)
    ref.latent_query_rotate(q.cpu(), D, R, n_rot, inter, pos.cpu(), table.cpu() if n_rot else None, outs[1], C)
    torch.testing.assert_close(outs[0].cpu().float(), outs[1].float(), **tol(dtype))
    assert float((outs[0][:, :, :C] - 3.0).abs().max()) == 0  # the latent part of the query rows is another kernel's


@pytest.mark.parametrize("dtype", DTYPES)
def test_products_per_head_on_views_of_wider_heads(dtype):
    T, H, K, N = 13, 5, 24, 40
    x, out = rnd(T, H, K + 8, dtype=dtype, seed=1), torch.full((T, H, N + 16), 2.0, dtype=dtype, device=DEV)
    w = rnd(H, K, N, dtype=dtype, seed=2, scale=0.2)
    ops.heads_linear(x[:, :, :K], w, out[:, :, :N])
    want = torch.einsum("thk,hkn->thn", x[:, :, :K].float(), w.float())
    torch.testing.assert_close(out[:, :, :N].float(), want, **tol(dtype, f32=1e-4, bf16=3e-2))
    assert float((out[:, :, N:] - 2.0).abs().max()) == 0


def paged(keys, P, n_pages, dtype, shuffle_seed=1):
    """``keys [L, D]`` into a slab ``[pages, 1, P, D]`` through a shuffled block table (one request, row 0)."""
    L, D = keys.shape
    n_blocks = -(-L // P)
    order = torch.randperm(n_pages - 1, generator=torch.Generator().manual_seed(shuffle_seed))[:n_blocks] + 1
    slab = torch.zeros(n_pages, 1, P, D, dtype=dtype, device=DEV)
    table = torch.zeros(1, n_blocks + 2, dtype=torch.int32, device=DEV)
    for b in range(n_blocks):
        rows = keys[b * P:(b + 1) * P]
        slab[int(order[b]), 0, : rows.shape[0]] = rows.to(dtype)
        table[0, b] = int(order[b])
    return slab, table


def run_attention(q, slab, table, q_len, kv_len, dtype, window, sink, scale=1.0, split=1):
    Hq, D = q.shape[1], q.shape[2]
    rows = 16 if dtype == torch.float32 or (q_len == 1 and Hq // split <= 16) else 64
    plan = build_plan([(q_len, kv_len)], Hq // split, rows, window, split, sm_count=148)
    items = torch.from_numpy(plan.items).to(DEV)
    part_o = torch.zeros(max(plan.n_slots, 1), split, rows, D, device=DEV) if plan.n_slots else None
    part_ml = torch.zeros(max(plan.n_slots, 1), split, rows, 2, device=DEV) if plan.n_slots else None
    info = torch.tensor([[0, q_len, kv_len, 0]], dtype=torch.int32, device=DEV)
    out = torch.zeros_like(q)
    ops.paged_attention(q, slab, slab, table, info, 1, items, plan.n_items, part_o, part_ml, out, rows, scale, window,
                        kv_split=split, sink=sink)
    return out, info


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("Hq,D,P,window,split", [(6, 128, 16, 72, 1), (8, 32, 4, 13, 1), (32, 16, 4, 300, 2), (2, 48, 8, 17, 1), (1, 32, 16, 1, 1)])
def test_one_cached_row_as_key_and_value_with_a_sink_per_head(dtype, Hq, D, P, window, split):
    L, q_len = 150, 40
    if dtype == torch.bfloat16 and split > 1:
        split = 1  # (tiles of 64 rows take the 32 heads)
    keys = rnd(L, D, seed=1)
    slab, table = paged(keys, P, 60, dtype)
    sink = rnd(Hq, seed=7, scale=2.0)
    for ql in (q_len, 1):
        q = rnd(ql, Hq, D, dtype=dtype, seed=2)
        got, info = run_attention(q, slab, table, ql, L, dtype, window, sink, 0.2, split)
        want = torch.zeros_like(q).cpu()
        ref.paged_attention(q.cpu(), slab.cpu(), slab.cpu(), table.cpu(), info.cpu(), 1, None, 0, None, None, want, 16, 0.2,
                            window, sink=sink.cpu())
        torch.testing.assert_close(got.cpu().float(), want.float(), **tol(dtype, f32=2e-5))


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_large_sink_silences_its_head_only(dtype):
    L, Hq, D = 70, 4, 32
    slab, table = paged(rnd(L, D, seed=1), 8, 20, dtype)
    q = rnd(1, Hq, D, dtype=dtype, seed=2)
    none = torch.full((Hq,), -60.0, device=DEV)
    one = none.clone()
    one[2] = 60.0
    base, _ = run_attention(q, slab, table, 1, L, dtype, 50, none, 0.2)
    got, _ = run_attention(q, slab, table, 1, L, dtype, 50, one, 0.2)
    assert float(got[0, 2].float().abs().max()) < 1e-6
    torch.testing.assert_close(got[0, [0, 1, 3]].float(), base[0, [0, 1, 3]].float(), rtol=0, atol=0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [1, 7, 16, 17, 64, 65, 100])
@pytest.mark.parametrize("q_len", [1, 33])
def test_a_key_at_the_windows_edge(dtype, window, q_len):
    """Among 200 keys one matches the last query (its score stands out): just inside the window the output is that
    row, just outside it is not; the same for the step's first query.  Pages of 16: the edges fall on and beside
    page borders."""
    L, Hq, D = 200, 2, 32
    for inside in (True, False):
        for which in (q_len - 1, 0):
            p_q = L - q_len + which
            p_k = p_q - window + 1 if inside else p_q - window
            if p_k < 0:
                continue
            keys = rnd(L, D, seed=3, scale=0.1)
            star = torch.zeros(D, device=DEV)
            star[5] = 8.0
            keys[p_k] = star
            slab, table = paged(keys, 16, 30, dtype, shuffle_seed=window)
            q = rnd(q_len, Hq, D, dtype=dtype, seed=4, scale=0.1)
            q[which] = (star * 4.0).to(dtype)
            sink = torch.zeros(Hq, device=DEV)
            got, _ = run_attention(q, slab, table, q_len, L, dtype, window, sink, 1.0)
            hit = float(got[which, 0, 5].float())
            if inside:
                assert hit > 7.5, (window, q_len, which, hit)
            else:
                assert hit < 1.0, (window, q_len, which, hit)


@pytest.mark.parametrize("Hq,P,window", [(6, 16, 72), (16, 16, 200), (8, 32, 37), (48, 16, 128), (2, 64, 1), (128, 16, 1000)])
def test_one_slab_with_window_and_sinks_on_the_tensor_core_kernel(Hq, P, window):
    """The tcgen05 kernel with 128-row tiles on cached rows that are key and value at once: pieces that start on a
    key tile before the window's first key, pages before the window that hold NaN (they may have gone back to the
    pool), tiles split along the keys, one sink per head."""
    dtype = torch.bfloat16
    sink = rnd(Hq, seed=8, scale=1.5)
    for segs_, force in (([(300, 300)], False), ([(128, 128), (1, 40), (200, 517), (3, 3)], False), ([(256, 900)], True),
                         ([(130, 1000)], False)):
        q, ks, _, bt, seg = attention_problem(dtype, Hq, 1, 128, P, segs_, seed=6)
        for q_start, q_len, kv_len, row in seg.tolist():
            for j in range(0, max(0, kv_len - q_len - window + 1)):
                ks[int(bt[row, j // P]), :, j % P] = float("nan")
        ops.variant_counts(reset=True)
        out, want, plan = run_attention_case(dtype, Hq, 1, 128, P, segs_, 128, window, sink, force_split=force,
                                             problem=(q, ks, ks, bt, seg))
        assert ops.variant_counts().get("attention: tcgen05, 128-row query tiles, window or sink", 0) == 1
        torch.testing.assert_close(out.float(), want.float(), **attn_tol(dtype))
    assert ops.read_status() == 0


# --------------------------------------------------------------------------- matrix memory
def plain_memory(q, k, v, gi, f, m0, S0, n0):
    """The recurrence as the design states it, with the running maximum, from a given state."""
    outs, S, n, m = [], S0.clone(), n0.clone(), m0.clone()
    for t in range(q.shape[0]):
        new = torch.maximum(f[t] + m, gi[t])
        keep, take = torch.exp(f[t] + m - new), torch.exp(gi[t] - new)
        S = keep[:, None, None] * S + take[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        n = keep[:, None] * n + take[:, None] * k[t]
        m = new
        den = torch.maximum((n * q[t]).sum(-1).abs(), torch.exp(-m)) + 1e-6
        outs.append(torch.einsum("hdv,hd->hv", S, q[t]) / den[:, None])
    return torch.stack(outs), S, n, m


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,D,Dv,cap", [(4, 32, 48, 15.0), (2, 16, 24, 8.0), (1, 40, 12, 5.0), (3, 10, 14, 12.0), (5, 6, 33, 3.0)])
def test_matrix_memory_kernels_against_the_stated_recurrence(dtype, H, D, Dv, cap):
    """Gates, running maximum, the recurrence kernel on prepared inputs and the output step together, for requests that
    start and one that goes on from a state, portions longer than a chunk and single tokens; the state left behind
    (S, n, m) is the stated one's."""
    lens = [(150, 150), (1, 20), (70, 90), (3, 3)]
    info, slots, T = segs(lens)
    proj = rnd(T, H * (2 * D + 2 * Dv), dtype=dtype, seed=1)
    pre = rnd(T, 2 * H, seed=2, scale=4.0)
    bi, bf = rnd(H, seed=3), rnd(H, seed=4) + 2.0
    w = rnd(H * Dv, seed=5) + 1.0
    S0 = rnd(len(lens) + 1, H, D, Dv + 1, seed=6)
    m0 = rnd(len(lens) + 1, H, seed=7)
    state, m_state = S0.clone(), m0.clone()
    f32 = dict(dtype=torch.float32, device=DEV)
    kf, dec, m = torch.zeros(T, H, **f32), torch.zeros(T, H, **f32), torch.zeros(T, H, **f32)
    ops.mlstm_gates(pre, bi, bf, cap, m_state, slots, info, len(lens), kf, dec, m)
    chunks, per_seg, single, multi = chunk_list(lens, 64)
    n_chunks = chunks.shape[0]
    carry = torch.zeros(n_chunks, H, D, Dv + 1, **f32)
    decay = torch.zeros(n_chunks, H, D, **f32)
    o32, nq = torch.zeros(T, H, Dv, **f32), torch.zeros(T, H, **f32)
    ops.gla_scan(proj[:, :H * D], proj[:, H * D:2 * H * D], proj[:, 2 * H * D:H * (2 * D + Dv)], None, None, 1.0, D ** -0.5,
                 state, slots, info, len(lens), torch.from_numpy(chunks).to(DEV), n_chunks,
                 torch.from_numpy(per_seg).to(DEV), single, multi, carry, decay, o32, k_fac=kf, a_head=dec, ones_col=True,
                 out_ones=nq)
    out = torch.zeros(T, H * Dv, dtype=dtype, device=DEV)
    gates = proj[:, H * (2 * D + Dv):]
    ops.mlstm_output(o32, nq, m, gates, w, 1e-5, out)
    # the stated recurrence, request by request
    p = proj.float().cpu().double()
    qq = p[:, :H * D].view(T, H, D) * D ** -0.5
    kk, vv = p[:, H * D:2 * H * D].view(T, H, D), p[:, 2 * H * D:2 * H * D + H * Dv].view(T, H, Dv)
    g_i = cap * torch.tanh((pre.cpu().double()[:, :H] + bi.cpu().double()) / cap)
    g_f = torch.nn.functional.logsigmoid(cap * torch.tanh((pre.cpu().double()[:, H:] + bf.cpu().double()) / cap))
    for i, (q_len, kv_len) in enumerate(lens):
        a, b = int(info[i, 0]), int(info[i, 0]) + q_len
        if kv_len == q_len:
            S, n, mm = torch.zeros(H, D, Dv).double(), torch.zeros(H, D).double(), torch.zeros(H).double()
        else:
            mm = m0[i + 1].cpu().double()
            S, n = S0[i + 1, :, :, :Dv].cpu().double(), S0[i + 1, :, :, Dv].cpu().double()
        o, S, n, mm = plain_memory(qq[a:b], kk[a:b], vv[a:b], g_i[a:b], g_f[a:b], mm, S, n)
        o = o / torch.sqrt((o * o).mean(-1, keepdim=True) + 1e-5)
        want = o.reshape(q_len, H * Dv) * w.cpu().double() * torch.sigmoid(gates[a:b].float().cpu().double())
        torch.testing.assert_close(out[a:b].float().cpu().double(), want, **tol(dtype, f32=1e-4))
        torch.testing.assert_close(m_state[i + 1].cpu().double(), mm, rtol=1e-5, atol=1e-5)
        for got_s, want_s in ((state[i + 1, :, :, :Dv], S), (state[i + 1, :, :, Dv], n)):  # (relative to the largest entry)
            torch.testing.assert_close(got_s.cpu().double() / want_s.abs().max(), want_s / want_s.abs().max(), rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("cuts", [[700], [333, 2, 365], [64, 64, 1, 1, 570], [699, 1]])
def test_a_memory_written_once_is_read_hundreds_of_tokens_later(cuts):
    """One token writes a value under a key that no later token uses, with its input gate open and every later one nearly
    shut, and the forget gate stays open: 700 tokens and many chunks later a query along that key reads that value back,
    however the tokens are cut into steps (the state and the maximum go through the slot).  Without the far token the
    output would be another one altogether."""
    H, D, Dv, cap, T = 2, 16, 24, 15.0, 700
    f32 = dict(dtype=torch.float32, device=DEV)
    g = torch.Generator().manual_seed(5)
    k = torch.randn(T, H, D, generator=g) * 0.3
    k[:, :, 0] = 0.0            # nobody but the first token writes along key channel 0
    k[0] = 0.0
    k[0, :, 0] = 4.0
    v = torch.randn(T, H, Dv, generator=g)
    q = torch.randn(T, H, D, generator=g) * 0.3
    q[-1] = 0.0
    q[-1, :, 0] = 4.0           # the last token asks along channel 0
    gate = torch.zeros(T, H * Dv)
    proj = torch.cat([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1), gate], 1).to(DEV)
    pre = torch.zeros(T, 2 * H)
    pre[:, :H] = -2.0           # input gates: e^-2 for everyone ...
    pre[0, :H] = 6.0            # ... but e^6 for the first token
    pre[:, H:] = 40.0           # forget gates at the cap: logsigmoid(15), a few 1e-7 below 0
    pre = pre.to(DEV)
    zero, w = torch.zeros(H, device=DEV), torch.ones(H * Dv, device=DEV)
    state, m_state = torch.zeros(2, H, D, Dv + 1, **f32), torch.zeros(2, H, **f32)
    rows, t0 = [], 0
    for n in cuts:
        info, slots, _ = segs([(n, t0 + n)])
        kf, dec, m = (torch.zeros(n, H, **f32) for _ in range(3))
        ops.mlstm_gates(pre[t0:t0 + n].contiguous(), zero, zero, cap, m_state, slots, info, 1, kf, dec, m)
        chunks, per_seg, single, multi = chunk_list([(n, t0 + n)], 64)
        nc = chunks.shape[0]
        carry, decay = torch.zeros(nc, H, D, Dv + 1, **f32), torch.zeros(nc, H, D, **f32)
        o32, nq = torch.zeros(n, H, Dv, **f32), torch.zeros(n, H, **f32)
        pr = proj[t0:t0 + n]
        ops.gla_scan(pr[:, :H * D], pr[:, H * D:2 * H * D], pr[:, 2 * H * D:H * (2 * D + Dv)], None, None, 1.0, D ** -0.5,
                     state, slots, info, 1, torch.from_numpy(chunks).to(DEV), nc, torch.from_numpy(per_seg).to(DEV), single,
                     multi, carry, decay, o32, k_fac=kf, a_head=dec, ones_col=True, out_ones=nq)
        out = torch.zeros(n, H * Dv, **f32)
        ops.mlstm_output(o32, nq, m, pr[:, H * (2 * D + Dv):], w, 1e-6, out)
        rows.append(out.cpu())
        t0 += n
    got = torch.cat(rows)[-1].view(H, Dv).double()
    gi = cap * torch.tanh(pre.cpu().double()[:, :H] / cap)
    gf = torch.nn.functional.logsigmoid(cap * torch.tanh(pre.cpu().double()[:, H:] / cap))
    z = torch.zeros
    o, _, _, _ = plain_memory(q.double() * D ** -0.5, k.double(), v.double(), gi, gf, z(H).double(), z(H, D, Dv).double(),
                              z(H, D).double())
    want = o[-1] / torch.sqrt((o[-1] * o[-1]).mean(-1, keepdim=True) + 1e-6) * 0.5
    torch.testing.assert_close(got, want, rtol=1e-4, atol=1e-4)
    far = v[0].double() / torch.sqrt((v[0].double() ** 2).mean(-1, keepdim=True)) * 0.5  # the first token's value, unit norm, half open gate
    torch.testing.assert_close(got, far, rtol=1e-3, atol=1e-3)


def test_the_running_maximum_starts_at_zero_and_is_carried():
    """Input gates far below zero: the maximum stays what the forget gates leave of its start at 0 (it would be the input
    gate had it started at minus infinity); cut into steps, the slot carries it on."""
    H, T = 2, 70
    pre = torch.zeros(T, 2 * H, device=DEV)
    pre[:, :H] = -30.0   # i = -cap
    pre[:, H:] = 30.0    # f = logsigmoid(cap), just below 0
    zero = torch.zeros(H, device=DEV)
    cap = 6.0
    f = float(torch.nn.functional.logsigmoid(cap * torch.tanh(torch.tensor(30.0 / cap))))
    outs = []
    for cuts in ([T], [1] * T, [33, 2, 35]):
        m_state = torch.full((2, H), 9.0, device=DEV)
        got, t0 = [], 0
        for n in cuts:
            info, slots, _ = segs([(n, t0 + n)])
            gi, zf, m = (torch.zeros(n, H, device=DEV) for _ in range(3))
            ops.mlstm_gates(pre[t0:t0 + n].contiguous(), zero, zero, cap, m_state, slots, info, 1, gi, zf, m)
            got.append(m.cpu())
            t0 += n
        outs.append(torch.cat(got))
        want = f * torch.arange(1, T + 1, dtype=torch.float32)[:, None].expand(T, H)
        torch.testing.assert_close(outs[-1], want, rtol=1e-5, atol=1e-5)  # (the input gate, -cap, never gets above it)
    torch.testing.assert_close(outs[1], outs[0], rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(outs[2], outs[0], rtol=1e-5, atol=1e-6)


# --------------------------------------------------------------------------- the engine against the plain model
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["K1", "K2", "K3", "K4", "K5"])
def test_cuts_and_batches_agree_with_the_plain_model(name, dtype, tmp_path_factory):
    folder = model_folder(tmp_path_factory.getbasetemp(), name, ALL[name])
    plain = PlainKekopel(folder)
    eng = make_engine(folder, dtype, DEV, 16 if name == "K5" else PAGE, pages=40)
    toks = tokens_for(plain.vocab, 70, 11)
    want, gaps = plain.logits(toks), plain.router_gaps(toks) * SHARP.get(name, 1.0)
    assert_rows(replay_whole(eng, "w", toks), want, dtype, "whole", gaps)
    assert_rows(replay_cuts(eng, "d", toks, [38]), want, dtype, "last 32 one by one", gaps)
    assert_rows(replay_cuts(eng, "c", toks, [7, 2, 13, 2, 5, 3, 2, 11, 2]), want, dtype, "portions", gaps)
    assert_rows(replay_cuts(eng, "one", toks[:24], []), want[:24], dtype, "one by one from the first token", gaps)
    eng.cache.check()
    eng.check_kernels()
    assert all(g.pool.free_count == g.pool.num_pages for g in eng.cache.paged)


def test_every_layer_hands_on_what_the_plain_model_does(tmp_path_factory):
    """The 32-bit stream after every layer (read from the block's history of layer outputs is not possible: it holds
    the outputs before the mix), so the last layer's mix is checked through models cut after every layer."""
    for n in (1, 2, 3, 4):
        raw = dict(KEKO_1, layers=KEKO_1["layers"][:n])
        folder = model_folder(tmp_path_factory.getbasetemp(), f"K1_first{n}", raw)
        plain = PlainKekopel(folder)
        toks = tokens_for(plain.vocab, 40, 5)
        eng = make_engine(folder, "float32", DEV, PAGE, pages=40)
        assert_rows(replay_cuts(eng, "c", toks, [9, 2, 20]), plain.logits(toks), "float32", f"{n} layers")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["K1", "K3"])
def test_mixed_steps_with_few_pages_and_slots(name, dtype, tmp_path_factory):
    folder = model_folder(tmp_path_factory.getbasetemp(), name, ALL[name])
    plain = PlainKekopel(folder)
    lengths = {"r0": 45, "r1": 60, "r2": 38, "r3": 52, "r4": 41, "r5": 47}
    seqs = {r: tokens_for(plain.vocab, n, i) for i, (r, n) in enumerate(lengths.items())}
    eng = make_engine(folder, dtype, DEV, PAGE, pages=4 * (-(-64 // PAGE)))
    got = replay_mixed(eng, seqs, mixed_schedule(lengths, seed=3))
    for r, toks in seqs.items():
        assert_rows(got[r], plain.logits(toks), dtype, r, plain.router_gaps(toks))
    for g in eng.cache.paged:
        assert g.pool.handed_out > g.pool.num_pages, "the trace was meant to use pages again"
    assert eng.cache.slots.free_count == 4


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["K1", "K5"])
def test_long_prompt_long_decoding_and_recorded_steps(name, dtype, tmp_path_factory):
    """Hundreds of tokens across many pages and chunks, windows that pass over decoded tokens, a hundred tokens one
    by one (recorded into a CUDA graph at the first, replayed afterwards), and a long step in between."""
    folder = model_folder(tmp_path_factory.getbasetemp(), name, ALL[name])
    plain = PlainKekopel(folder)
    toks = tokens_for(plain.vocab, 300, 3)
    want, gaps = plain.logits(toks), plain.router_gaps(toks) * SHARP.get(name, 1.0)
    eng = make_engine(folder, dtype, DEV, 16, pages=64, max_step=512)
    assert_rows(replay_whole(eng, "w", toks), want, dtype, "whole", gaps)
    assert_rows(replay_cuts(eng, "d", toks, [200]), want, dtype, "a hundred tokens one by one", gaps)
    assert eng.graphs, "the decode steps were meant to be replayed from graphs"
    assert_rows(replay_cuts(eng, "c", toks, [63, 2, 64, 65, 17, 2, 33] + [1] * 20 + [30, 2]), want, dtype, "portions", gaps)
    other = tokens_for(plain.vocab, 130, 5)
    got = [eng.step([StepEntry("a", toks[:3], [0, 1, 2])]).logits.float().cpu().clone()]
    for i in range(3, 12):
        got.append(eng.step([StepEntry("a", toks[i:i + 1], [0])]).logits.float().cpu().clone())
    long = eng.step([StepEntry("b", other, list(range(len(other))))]).logits.float().cpu().clone()
    for i in range(12, 40):
        got.append(eng.step([StepEntry("a", toks[i:i + 1], [0])]).logits.float().cpu().clone())
    assert_rows(long, plain.logits(other), dtype, "the long step", plain.router_gaps(other) * SHARP.get(name, 1.0))
    assert_rows(torch.cat(got), want[:40], dtype, "decode steps before and after it", gaps)
    eng.check_kernels()


def test_long_steps_of_rows_of_128_run_the_tensor_core_attention(tmp_path_factory):
    folder = model_folder(tmp_path_factory.getbasetemp(), "K5", ALL["K5"])
    plain = PlainKekopel(folder)
    toks = tokens_for(plain.vocab, 300, 9)
    want, gaps = plain.logits(toks), plain.router_gaps(toks) * SHARP["K5"]
    eng = make_engine(folder, "bfloat16", DEV, 16, pages=96, max_step=512)
    ops.variant_counts(reset=True)
    assert_rows(replay_whole(eng, "w", toks), want, "bfloat16", "whole", gaps)
    assert ops.variant_counts().get("attention: tcgen05, 128-row query tiles, window or sink", 0) == 2
    assert_rows(replay_cuts(eng, "c", toks, [150, 130, 2]), want, "bfloat16", "portions, the rest one by one", gaps)
    others = {f"o{i}": tokens_for(plain.vocab, 20 + i, 20 + i) for i in range(3)}
    for r, t in others.items():  # three requests that decode beside a long portion
        eng.step([StepEntry(r, t[:-1], [])])
    out = eng.step([StepEntry("long", toks[:200], list(range(200)))] + [StepEntry(r, t[-1:], [0]) for r, t in others.items()])
    assert_rows(out.logits[:200], want[:200], "bfloat16", "a long portion beside single tokens", gaps)
    for i, (r, t) in enumerate(others.items()):
        assert_rows(out.logits[200 + i:201 + i], plain.logits(t)[-1:], "bfloat16", r)
    eng.check_kernels()


def test_greedy_generation_through_the_scheduler(tmp_path_factory):
    from freetoken_b200 import LLM, SamplingParams

    folder = model_folder(tmp_path_factory.getbasetemp(), "K1", KEKO_1)
    plain = PlainKekopel(folder)
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
    folder = model_folder(tmp_path_factory.getbasetemp(), "K3", ALL["K3"])
    plain = PlainKekopel(folder)
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
        ga, gb = plain.router_gaps(a), plain.router_gaps(b)
        assert_rows(torch.from_numpy(got[0]), la[[0, 19]], dtype, "step 0", ga[[0, 19]])
        assert_rows(torch.from_numpy(got[1]), torch.stack([la[20], lb[8]]), dtype, "step 1", torch.stack([ga[20], gb[8]]))
        assert_rows(torch.from_numpy(got[2]), la[[29]], dtype, "step 2", ga[[29]])
