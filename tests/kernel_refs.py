"""Plain PyTorch statement of every op in ``freetoken_b200.kernels.ops``, argument for argument.

Two uses: the ``-m gpu`` tests compare each CUDA kernel with its function here (computed in
float32 on the same inputs), and the CPU tests run the engine's step, cache and scheduler
logic with these functions standing in for the kernels (``install``), so that the host-side
code can be checked without a GPU.  Nothing in ``freetoken_b200`` imports this file.

Rounding: a function computes in float32 and rounds once into the dtype of its output.
"""

from __future__ import annotations

from typing import Optional, Sequence

import torch


def embedding_gather(table, ids, out):
    out.copy_(table[ids.long()].float())


def add_rmsnorm(x, residual, weight, eps, gemma, out, out_f32=None, rows=None):
    if rows is not None:
        idx = rows.long()
        z = residual[idx].float() if residual is not None else 0
        if x is not None:
            z = z + x[idx].float()
    else:
        z = residual.float() if residual is not None else 0
        if x is not None:
            z = z + x.float()
        if residual is not None and x is not None:
            residual.copy_(z)
    w = weight.float() + 1.0 if gemma else weight.float()
    inv = torch.rsqrt((z * z).sum(-1, keepdim=True) / z.shape[-1] + eps)
    y = (z * inv * w).to(out.dtype)
    out.view(y.shape).copy_(y)
    if out_f32 is not None:
        out_f32.view(y.shape).copy_(y.float())


def add_rmsnorm_routes(y, route_pos, top_k, shared, residual, weight, eps, gemma, out, out_f32=None, rows=None):
    T = residual.shape[0]
    delta = torch.empty(T, y.shape[1], dtype=y.dtype, device=y.device)
    moe_combine(y, route_pos, T, top_k, shared, delta)
    add_rmsnorm(delta, residual, weight, eps, gemma, out, out_f32=out_f32, rows=rows)


def act_and_mul(gate_up, out, act, alpha, limit):
    I = gate_up.shape[1] // 2
    g, u = gate_up[:, :I].float(), gate_up[:, I:].float()
    if act == "silu":
        y = g * torch.sigmoid(g) * u
    else:
        g = torch.clamp(g, max=limit)
        u = torch.clamp(u, min=-limit, max=limit)
        y = g * torch.sigmoid(alpha * g) * (u + 1.0)
    out.copy_(y.to(out.dtype))


def cast(src, dst):
    dst.view(-1).copy_(src.reshape(-1).to(dst.dtype))


def copy_tokens(dst, pairs, src, n, vocab):
    for d, s_ in pairs.view(-1, 2)[:n].tolist():
        if d >= 0 and s_ >= 0:
            v = int(src[s_])
            dst[d] = v if 0 <= v < vocab else 0


def table_update(table, updates, n_updates):
    u = updates.view(-1, 2)[:n_updates]
    ok = u[:, 0] >= 0
    table.view(-1)[u[ok, 0].long()] = u[ok, 1]


def norm_rope_store(x, head_dim, rotary_dim, positions, rope_table, eps, gemma, sections):
    T = x.shape[0]
    whole = x.shape[1] // head_dim * head_dim  # a row may end in columns that belong to no head
    xs = x[:, :whole].reshape(T, -1, head_dim).float()
    half = rotary_dim // 2
    if rotary_dim:
        cs = rope_table[positions.long()]
        cos, sin = cs[:, None, :half], cs[:, None, half:]
    for s in sections:
        u = xs[:, s["first_head"]: s["first_head"] + s["n_heads"]]
        if s.get("bias") is not None:
            u = u + s["bias"].float().view(1, s["n_heads"], head_dim)
        w = s.get("norm_weight")
        if w is not None:
            scale = w.float() + 1.0 if gemma else w.float()
            u = u * torch.rsqrt((u * u).sum(-1, keepdim=True) / head_dim + eps) * scale
        if s.get("rotate") and rotary_dim:
            a, b, rest = u[..., :half], u[..., half:rotary_dim], u[..., rotary_dim:]
            u = torch.cat([a * cos - b * sin, b * cos + a * sin, rest], dim=-1)
        if s.get("pos_scale") is not None:
            f = s["pos_scale"].float()
            u = u * f[positions.long().clamp(0, f.numel() - 1)][:, None, None]
        dst_dim = int(s.get("dst_head_dim") or head_dim)
        if dst_dim != head_dim:
            u = torch.cat([u, torch.zeros(*u.shape[:-1], dst_dim - head_dim, dtype=u.dtype, device=u.device)], dim=-1)
        if s.get("dense_out") is not None:
            s["dense_out"].view(T, s["n_heads"], dst_dim).copy_(u.to(x.dtype))
        else:
            slab, slots = s["slab"], s["slot_map"][:T].long()
            P = slab.shape[2]
            ok = slots >= 0
            page, off = slots[ok] // P, slots[ok] % P
            slab[page, :, off, :] = u[ok].to(slab.dtype)


def paged_attention(q, k_slab, v_slab, block_table, seg_info, n_segs, items, n_items, part_o, part_ml,
                    out, tile_rows, scale, window, sel=None, block_size=0, few_rows=False, dist_bias=None, kv_split=1,
                    sink=None):
    """Per query token, softmax over the visible keys gathered through the block table; the
    work list and the scratch are ignored (they only steer how the kernel splits the work).
    With ``sel`` a query reads only the keys of its chosen blocks."""
    T, Hq, D = q.shape
    P = k_slab.shape[2]
    Hkv = k_slab.shape[1]
    G = Hq // Hkv
    info = seg_info.view(-1, 4)[:n_segs].tolist()
    for q_start, q_len, kv_len, row in info:
        pos = torch.arange(kv_len, device=q.device)
        pages = block_table[row, (pos // P).long()].long()
        K = k_slab[pages, :, (pos % P).long(), :].float()  # [kv, Hkv, D]
        V = v_slab[pages, :, (pos % P).long(), :].float()
        for t in range(q_len):
            p_q = kv_len - q_len + t
            lo = 0 if not window else max(0, p_q - window + 1)
            qq = q[q_start + t].float().view(-1, G, D)  # [Hkv, G, D]
            if sel is None:
                kk, vv = K[lo:p_q + 1], V[lo:p_q + 1]
                s = torch.einsum("hgd,khd->hgk", qq, kk) * scale
                if dist_bias is not None:  # [Hq, L] by distance, the last entry for everything farther
                    dist = (p_q - torch.arange(lo, p_q + 1, device=q.device)).clamp(max=dist_bias.shape[1] - 1)
                    s = s + dist_bias.float()[:, dist].view(Hkv, G, -1)
                if sink is None:
                    p = torch.softmax(s, dim=-1)
                else:  # a key without a value: it only takes its share of the weights (one logit, or one per head)
                    sk = sink.float().view(Hkv, G, 1) if isinstance(sink, torch.Tensor) else torch.full((1, 1, 1), float(sink), device=q.device)
                    top = torch.maximum(s.max(dim=-1, keepdim=True).values, sk)
                    e = torch.exp(s - top)
                    p = e / (e.sum(-1, keepdim=True) + torch.exp(sk - top))
                o = torch.einsum("hgk,khd->hgd", p, vv)
            else:
                o = torch.zeros(Hkv, G, D, device=q.device)
                for h in range(Hkv):
                    blocks = [int(b) for b in sel[q_start + t, h].tolist() if b >= 0]
                    idx = torch.cat([torch.arange(b * block_size, min((b + 1) * block_size, p_q + 1))
                                     for b in blocks]).to(q.device)
                    s = (qq[h] @ K[idx, h].T) * scale
                    o[h] = torch.softmax(s, dim=-1) @ V[idx, h]
            out[q_start + t] = o.reshape(Hq, D).to(out.dtype)


def sparse_score_fits(n_heads, dim, block_size):
    return False


def sparse_select(iq, ik_slab, block_table, seg_info, n_segs, block_size, local_blocks, init_blocks, max_blocks, sel,
                  scores=None, live_blocks=0):
    T, Hi, Di = iq.shape
    P = ik_slab.shape[2]
    topk = sel.shape[2]
    sel[:T] = -1
    for q_start, q_len, kv_len, row in seg_info.view(-1, 4)[:n_segs].tolist():
        pos = torch.arange(kv_len, device=iq.device)
        pages = block_table[row, (pos // P).long()].long()
        IK = ik_slab[pages, 0, (pos % P).long(), :].float()  # [kv, Di]
        for t in range(q_len):
            p_q = kv_len - q_len + t
            nb = p_q // block_size + 1
            scores = iq[q_start + t].float() @ IK[: p_q + 1].T  # [Hi, p_q + 1]
            pad = nb * block_size - (p_q + 1)
            if pad:
                scores = torch.nn.functional.pad(scores, (0, pad), value=float("-inf"))
            bs = scores.view(Hi, nb, block_size).amax(-1)
            bs = torch.where(torch.isnan(bs), torch.full_like(bs, -1e30), bs)
            if init_blocks:
                bs[:, : min(init_blocks, nb)] = 1e30
            if local_blocks:
                bs[:, max(0, nb - local_blocks):] = 1e29
            order = torch.argsort(bs, dim=-1, descending=True, stable=True)[:, : min(topk, nb)]
            chosen = torch.sort(order, dim=-1).values
            sel[q_start + t, :, : chosen.shape[1]] = chosen.to(torch.int32)


def router_topk(logits, bias, top_k, scoring, scale, ids, weights, n_parts=1):
    l = logits.float()
    if n_parts > 1:
        parts = l.view(l.shape[0], n_parts, -1)
        l = parts[:, 0]
        for q in range(1, n_parts):
            l = l + parts[:, q]
    if scoring == "softmax_of_chosen":  # the bias belongs to the logit; the softmax runs over the chosen logits only
        l = l + bias.float() if bias is not None else l
        idx = torch.argsort(l, dim=-1, descending=True, stable=True)[:, :top_k]
        ids.copy_(idx.to(torch.int32))
        weights.copy_(torch.softmax(l.gather(-1, idx), dim=-1) * scale)
        return
    if scoring == "sigmoid_raw":  # the chosen experts' sigmoid scores as they are
        sg = torch.sigmoid(l)
        idx = torch.argsort(sg, dim=-1, descending=True, stable=True)[:, :top_k]
        ids.copy_(idx.to(torch.int32))
        weights.copy_(sg.gather(-1, idx) * scale)
        return
    s = torch.sigmoid(l) if scoring == "sigmoid" else torch.softmax(l, dim=-1)
    c = s + bias.float() if bias is not None else s
    idx = torch.argsort(c, dim=-1, descending=True, stable=True)[:, :top_k]
    w = s.gather(-1, idx)
    w = w / (w.sum(-1, keepdim=True) + (1e-20 if scoring == "sigmoid" else 0.0))
    ids.copy_(idx.to(torch.int32))
    weights.copy_(w * scale)


def moe_permute(topk_ids, n_experts, expert_counts, expert_offsets, sorted_routes, route_pos):
    flat = topk_ids.reshape(-1).long()
    order = torch.argsort(flat, stable=True)
    counts = torch.bincount(flat, minlength=n_experts)
    expert_counts.copy_(counts.to(torch.int32))
    expert_offsets[0] = 0
    expert_offsets[1:] = torch.cumsum(counts, 0).to(torch.int32)
    sorted_routes.copy_(order.to(torch.int32))
    route_pos[order] = torch.arange(flat.numel(), dtype=torch.int32, device=flat.device)


def moe_gemm1_gather_fits(dtype, hidden, inter, n_experts, n_routes):
    return False  # the CPU tests copy the rows first


def attention_tc_fits(head_dim, page_size, group):
    return False  # the CPU tests plan for the other kernels


def attention_tc_few_fits(head_dim, page_size, group):
    return False


def moe_small_fits(n_tokens, hidden, inter, top_k):
    return False  # the few-token kernels are a second route to the same result; the CPU stand-ins take the general one


def moe_route_fits(n_tokens, hidden, n_experts, top_k):
    return 1 <= n_tokens <= 32 and hidden % 4 == 0


def moe_route(x, gate_w, bias, top_k, scoring, scale, logits, ids, weights, expert_counts, expert_offsets,
              sorted_routes, route_pos):
    logits.copy_(x.float() @ gate_w.float().T)
    router_topk(logits, bias, top_k, scoring, scale, ids, weights)
    moe_permute(ids, gate_w.shape[0], expert_counts, expert_offsets, sorted_routes, route_pos)


def moe_gather(h, sorted_routes, top_k, out):
    out.copy_(h[(sorted_routes.long() // top_k)])


def moe_gemm1_act(x_sorted, w1, expert_offsets, act, alpha, limit, out):
    off = expert_offsets.tolist()
    for e in range(w1.shape[0]):
        a, b = off[e], off[e + 1]
        if b > a:
            gu = x_sorted[a:b].float() @ w1[e].float().T
            gu = gu.to(x_sorted.dtype)  # the serving path stores the product before the activation
            act_and_mul(gu, out[a:b], act, alpha, limit)


def moe_gemm2(a, w2, expert_offsets, sorted_routes, topk_weights, out):
    off = expert_offsets.tolist()
    wr = topk_weights.reshape(-1)[sorted_routes.long()].float()
    for e in range(w2.shape[0]):
        lo, hi = off[e], off[e + 1]
        if hi > lo:
            y = (a[lo:hi].float() @ w2[e].float().T) * wr[lo:hi, None]
            out[lo:hi] = y.to(out.dtype)


def moe_combine(y, route_pos, n_tokens, top_k, shared, out):
    pos = route_pos.view(n_tokens, top_k).long()
    acc = torch.zeros(n_tokens, y.shape[1], dtype=torch.float32, device=y.device)
    for j in range(top_k):
        acc = acc + y[pos[:, j]].float()
    if shared is not None:
        acc = acc + shared.float()
    out.copy_(acc.to(out.dtype))


def sample(logits, temperature, top_k, top_p, u, out):
    R, V = logits.shape
    for r in range(R):
        t = float(temperature[r])
        row = logits[r].float()
        if t <= 0:
            out[r] = int(torch.argmax(row))
            continue
        p = torch.softmax(row / max(t, 1e-6), dim=-1)
        k = int(top_k[r])
        if 0 < k < V:
            kth = torch.topk(p, k).values[-1]
            p = torch.where(p >= kth, p, torch.zeros_like(p))
        tp = float(top_p[r])
        if tp < 1.0:
            vals = torch.sort(p, descending=True).values.double()
            csum = torch.cumsum(vals, 0)
            n = int((csum < tp * float(csum[-1])).sum())
            th = vals[min(n, V - 1)].float()
            p = torch.where(p >= th, p, torch.zeros_like(p))
        csum = torch.cumsum(p.double(), 0)
        target = float(u[r]) * float(csum[-1])
        idx = int((csum <= target).sum())
        nz = torch.nonzero(p > 0).view(-1)
        idx = min(idx, int(nz[-1]))
        out[r] = idx


def stream_add_norm(residual, out, x1=None, x2=None, routed=None, table=None, ids=None, vec=None, norm=None, rows=None):
    src = next(t for t in (residual, x1, x2, out) if t is not None)
    H = src.shape[-1]
    total = (residual if residual is not None else src).numel() // H
    z = residual.float().view(total, H).clone() if residual is not None else torch.zeros(total, H, device=src.device)
    any_addend = False
    for x in (x1, x2):
        if x is not None:
            z = z + x.float().view(total, H)
            any_addend = True
    if routed is not None:
        y, pos, k = routed
        acc = torch.zeros_like(z)
        pos = pos.view(total, k).long()
        for j in range(k):
            acc = acc + y[pos[:, j]].float()
        z = z + acc
        any_addend = True
    if table is not None:
        z = z + table[ids[:total].long()].float()
        any_addend = True
    if vec is not None:
        z = z + vec.float()
        any_addend = True
    if rows is None and residual is not None and any_addend:
        residual.view(total, H).copy_(z)
    if rows is not None:
        z = z[rows.long()]
    if out is not None:
        if norm is not None:
            _, w, b, alpha = norm
            z = torch.tanh(alpha.float() * z) * w.float() + b.float()
        out.view(z.shape).copy_(z.to(out.dtype))


def head_gate(o, gates):
    o.copy_((o.float() * torch.sigmoid(gates.float())[:, :, None]).to(o.dtype))


def table_route(token_ids, table, n_experts, ids, weights):
    T, k = ids.shape
    ids.copy_(table[token_ids[:T].long()].clamp(0, n_experts - 1))
    weights.fill_(1.0 / k)


def scale_(x, s):
    x.mul_(s)


def linear(x, w, out, bias=None):
    y = x.float() @ w.float().T
    if bias is not None:
        y = y + bias.float()
    out.copy_(y.to(out.dtype))


def linear_f32(x, w, out):
    out.copy_(x.float() @ w.float().T)


def softcap_(x, cap):
    x.copy_(cap * torch.tanh(x / cap))


def postnorm_add_norm(x, routed, post_weight, post_eps, post_gemma, residual, pre_weight=None, pre_eps=0.0,
                      pre_gemma=True, out=None, out_f32=None, rows=None):
    T = residual.shape[0]
    if routed is not None:
        pos, top_k, shared = routed
        a = x.float()[pos.view(-1)[: T * top_k].long()].view(T, top_k, -1).sum(1)
        if shared is not None:
            a = a + shared.float()
    else:
        a = x.float()[:T]
    wa = post_weight.float() + 1.0 if post_gemma else post_weight.float()
    z = residual.float() + a * torch.rsqrt((a * a).mean(-1, keepdim=True) + post_eps) * wa
    if rows is None:
        residual.copy_(z)
    else:
        z = z[rows.long()]
    if pre_weight is not None:
        wr = pre_weight.float() + 1.0 if pre_gemma else pre_weight.float()
        y = (z * torch.rsqrt((z * z).mean(-1, keepdim=True) + pre_eps) * wr).to(out.dtype)
        out.view(y.shape).copy_(y)
        if out_f32 is not None:
            out_f32.view(y.shape).copy_(y.float())


def gated_heads(x, gates, out, dim, act="sigmoid", norm_weight=None, eps=0.0):
    T, H, _ = x.shape
    v = x[:, :, :dim].float()
    if norm_weight is not None:
        v = v * torch.rsqrt((v * v).mean(-1, keepdim=True) + eps) * norm_weight.float()
    g = gates.float().view(T, H, dim)
    s = torch.sigmoid(g)
    out[:, :, :dim] = (v * (g * s if act == "silu" else s)).to(out.dtype)


def gla_scan(q, k, v, z, z_bias, tau, q_scale, state, state_slots, seg_info, n_segs, chunks, n_chunks, seg_chunks,
             any_single, any_multi, carry, decay_prod, out, k_fac=None, a_head=None, ones_col=False, out_ones=None,
             qk_div=1):
    """Token by token from each request's slot; the chunk lists only steer how the kernel shares the work."""
    H, D, Dv = state.shape[1:]
    if qk_div > 1:  # queries and keys shared by groups of heads
        q = q.float().view(-1, H // qk_div, D).repeat_interleave(qk_div, dim=1).reshape(-1, H * D)
        k = k.float().view(-1, H // qk_div, D).repeat_interleave(qk_div, dim=1).reshape(-1, H * D)
    if a_head is not None:
        decay = a_head.float()[:, :, None].expand(-1, H, D)
    else:
        zz = z.float() + (z_bias.float().view(1, -1) if z_bias is not None else 0.0)
        decay = torch.exp(-torch.nn.functional.softplus(-zz) / tau).view(-1, H, D)
    qq, kk = q.float().view(-1, H, D) * q_scale, k.float().view(-1, H, D)
    if k_fac is not None:
        kk = kk * k_fac.float()[:, :, None]
    vv = v.float().view(-1, H, Dv - (1 if ones_col else 0))
    if ones_col:
        vv = torch.cat([vv, torch.ones(vv.shape[0], H, 1)], dim=-1)
    for i, (q_start, q_len, kv_len, _) in enumerate(seg_info.view(-1, 4)[:n_segs].tolist()):
        slot = int(state_slots[i])
        S = torch.zeros(H, D, Dv) if kv_len == q_len else state[slot].clone()
        for t in range(q_start, q_start + q_len):
            S = decay[t][:, :, None] * S + kk[t][:, :, None] * vv[t][:, None, :]
            o = torch.einsum("hdv,hd->hv", S, qq[t])
            if out_ones is None:
                out[t] = o
            else:
                out[t], out_ones[t] = o[:, :-1], o[:, -1]
        state[slot] = S


def short_conv(x, w, state, state_slots, seg_info, n_segs, out):
    """Per request: the step's inputs behind the slot's last ones; every output is its input plus the taps' sum."""
    taps = w.shape[1]
    keep = taps - 1
    for i, (q_start, q_len, kv_len, _) in enumerate(seg_info.view(-1, 4)[:n_segs].tolist()):
        slot = int(state_slots[i])
        rows = x[q_start:q_start + q_len].float()
        if keep:
            old = torch.zeros(keep, x.shape[1]) if kv_len == q_len else state[slot].clone().float()
            line = torch.cat([old, rows])
        else:
            line = rows
        y = rows.clone()
        for j in range(taps):
            y = y + w[:, j].float() * line[j:j + q_len]
        out[q_start:q_start + q_len] = y.to(out.dtype)
        if keep:
            state[slot] = line[-keep:]


def depth_mix(hist, n_prev, mix, x):
    T = x.shape[0]
    hist[n_prev, :T] = x
    acc = torch.zeros_like(x)
    for j in range(n_prev + 1):
        acc = acc + mix[j] * hist[j, :T]
    x.copy_(acc)


def moe_gather_scaled(h, sorted_routes, weights, top_k, out):
    r = sorted_routes.long()
    out.copy_((weights.float()[r][:, None] * h.float()[r // top_k]).to(out.dtype))


def relu2_(x):
    x.copy_((torch.relu(x.float()) ** 2).to(x.dtype))


def _turn(v, pos, table, n_rot, interleaved):
    """``v [..., dim]`` at position ``pos``: the first ``n_rot`` columns turn, by the table's row ``cos || sin``."""
    if not n_rot:
        return v
    half = n_rot // 2
    c, s = table[pos, :half].float(), table[pos, half:].float()
    out = v.clone()
    a = v[..., 0:n_rot:2] if interleaved else v[..., :half]
    b = v[..., 1:n_rot:2] if interleaved else v[..., half:n_rot]
    if interleaved:
        out[..., 0:n_rot:2], out[..., 1:n_rot:2] = a * c - b * s, b * c + a * s
    else:
        out[..., :half], out[..., half:n_rot] = a * c - b * s, b * c + a * s
    return out


def latent_store(proj, q_rank, kv_rank, rot_dim, n_rot, interleaved, wq, wkv, eps, positions, rope_table, cq_out, slab,
                 slot_map):
    p = proj.float()
    a, c, kr = p[:, :q_rank], p[:, q_rank:q_rank + kv_rank], p[:, q_rank + kv_rank:]
    if q_rank:
        cq_out.copy_((a * torch.rsqrt((a * a).mean(-1, keepdim=True) + eps) * wq.float()).to(cq_out.dtype))
    c = c * torch.rsqrt((c * c).mean(-1, keepdim=True) + eps) * wkv.float()
    flat = slab.view(-1, slab.shape[3])
    for t in range(p.shape[0]):
        slot = int(slot_map[t])
        if slot < 0:
            continue
        row = torch.zeros(slab.shape[3])
        row[:kv_rank] = c[t]
        row[kv_rank:kv_rank + rot_dim] = _turn(kr[t], int(positions[t]), rope_table, n_rot, interleaved)
        flat[slot] = row.to(slab.dtype)


def latent_query_rotate(q, flat_dim, rot_dim, n_rot, interleaved, positions, rope_table, q_out, kv_rank):
    for t in range(q.shape[0]):
        q_out[t, :, kv_rank:] = 0
        q_out[t, :, kv_rank:kv_rank + rot_dim] = _turn(q[t, :, flat_dim:].float(), int(positions[t]), rope_table, n_rot,
                                                       interleaved).to(q_out.dtype)


def mlstm_gates(pre, bias_i, bias_f, cap, m_state, state_slots, seg_info, n_segs, key_fac, decay, m_out):
    H = pre.shape[1] // 2
    gi = cap * torch.tanh((pre[:, :H].float() + bias_i.float()) / cap)
    zf = cap * torch.tanh((pre[:, H:].float() + bias_f.float()) / cap)
    f = torch.nn.functional.logsigmoid(zf)
    for i, (q_start, q_len, kv_len, _) in enumerate(seg_info.view(-1, 4)[:n_segs].tolist()):
        slot = int(state_slots[i])
        m = torch.zeros(H) if kv_len == q_len else m_state[slot].clone()
        for t in range(q_start, q_start + q_len):
            new = torch.maximum(f[t] + m, gi[t])
            key_fac[t] = torch.exp(gi[t] - new)
            decay[t] = torch.exp(f[t] + m - new)
            m_out[t] = m = new
        m_state[slot] = m


def mlstm_output(o32, nq, m, gates, norm_weight, eps, out):
    T, H, Dv = o32.shape
    o = o32 / (torch.maximum(nq.abs(), torch.exp(-m)) + 1e-6)[:, :, None]
    o = o * torch.rsqrt((o * o).mean(-1, keepdim=True) + eps)
    y = o.reshape(T, H * Dv) * norm_weight.float() * torch.sigmoid(gates.float())
    out.copy_(y.to(out.dtype))


def hyper_step(streams, init_from=None, y=None, mix=None, out_w=None, in_w=None, norm_w=None, eps=0.0, h_out=None,
               sum_out=None):
    S = streams.shape[0]
    x = streams.float().clone()
    if init_from is not None:
        x = init_from.float()[None].expand(S, -1, -1).clone()
    if y is not None:
        x = torch.einsum("st,snc->tnc", mix.float(), x) + out_w.float()[:, None, None] * y.float()[None]
    if init_from is not None or y is not None:
        streams.copy_(x)
    if in_w is not None:
        u = torch.einsum("s,snc->nc", in_w.float(), x)
        h_out.copy_((u * torch.rsqrt((u * u).mean(-1, keepdim=True) + eps) * norm_w.float()).to(h_out.dtype))
    if sum_out is not None:
        sum_out.copy_(x.sum(0))


def norm_mean(xs, ws, eps, out):
    acc = 0
    for x, w in zip(xs, ws):
        v = x.float()
        acc = acc + v * torch.rsqrt((v * v).mean(-1, keepdim=True) + eps) * w.float()
    out.copy_((acc / len(xs)).to(out.dtype))


def conv_act(x, w, bias, act, state, state_slots, seg_info, n_segs, out):
    """Per request: the step's inputs behind the slot's last ones; every output is the taps' sum (+ bias), activated."""
    taps = w.shape[1]
    keep = taps - 1
    for i, (q_start, q_len, kv_len, _) in enumerate(seg_info.view(-1, 4)[:n_segs].tolist()):
        slot = int(state_slots[i])
        rows = x[q_start:q_start + q_len].float()
        if keep:
            old = torch.zeros(keep, x.shape[1]) if kv_len == q_len else state[slot].clone().float()
            line = torch.cat([old, rows])
        else:
            line = rows
        y = torch.zeros_like(rows)
        for j in range(taps):
            y = y + w[:, j].float() * line[j:j + q_len]
        if bias is not None:
            y = y + bias.float()
        if act == "silu":
            y = y * torch.sigmoid(y)
        out[q_start:q_start + q_len] = y.to(out.dtype)
        if keep:
            state[slot] = line[-keep:]


def ssm_gates(dt_raw, dt_bias, a_log, dt_out, decay_out):
    dt = torch.nn.functional.softplus(dt_raw.float() + dt_bias.float(), threshold=1e9)
    dt_out.copy_(dt)
    decay_out.copy_(torch.exp(-torch.exp(a_log.float()) * dt))


def ssm_output(o32, x, d_skip, z, norm_weight, norm_groups, eps, out):
    T, H, P = o32.shape
    zz = z.float()
    y = (o32.float() + d_skip.float()[None, :, None] * x.float().view(T, H, P)).reshape(T, H * P) * (zz * torch.sigmoid(zz))
    y = y.view(T, norm_groups, -1)
    y = (y * torch.rsqrt((y * y).mean(-1, keepdim=True) + eps)).reshape(T, H * P) * norm_weight.float()
    out.copy_(y.to(out.dtype))


def delta_scan(q, k, v, b_raw, a_raw, a_log, dt_bias, q_scale, unit_eps, state, state_slots, seg_info, n_segs, out):
    T, H, Dv = out.shape
    D = state.shape[3]  # the state is kept column by column: [slots, H, Dv, D]
    G = q.shape[1] // D
    qq, kk = q.float().view(T, G, D), k.float().view(T, G, D)
    qq = qq * torch.rsqrt((qq * qq).sum(-1, keepdim=True) + unit_eps) * q_scale
    kk = kk * torch.rsqrt((kk * kk).sum(-1, keepdim=True) + unit_eps)
    qq, kk = qq.repeat_interleave(H // G, dim=1), kk.repeat_interleave(H // G, dim=1)
    vv = v.float().view(T, H, Dv)
    beta = torch.sigmoid(b_raw.float())
    g = torch.exp(-torch.exp(a_log.float()) * torch.nn.functional.softplus(a_raw.float() + dt_bias.float(), threshold=1e9))
    for i, (q_start, q_len, kv_len, _) in enumerate(seg_info.view(-1, 4)[:n_segs].tolist()):
        slot = int(state_slots[i])
        S = torch.zeros(H, D, Dv) if kv_len == q_len else state[slot].transpose(1, 2).clone()
        for t in range(q_start, q_start + q_len):
            S = g[t][:, None, None] * S
            u = beta[t][:, None] * (vv[t] - torch.einsum("hdv,hd->hv", S, kk[t]))
            S = S + kk[t][:, :, None] * u[:, None, :]
            out[t] = torch.einsum("hdv,hd->hv", S, qq[t])
        state[slot] = S.transpose(1, 2)


ALL = ["hyper_step", "norm_mean", "conv_act", "ssm_gates", "ssm_output", "delta_scan", "short_conv", "depth_mix", "moe_gather_scaled", "relu2_", "latent_store", "latent_query_rotate", "mlstm_gates", "mlstm_output", "linear_f32", "softcap_", "postnorm_add_norm", "gated_heads", "gla_scan", "stream_add_norm", "head_gate", "table_route", "scale_", "sparse_score_fits", "moe_small_fits", "copy_tokens", "sparse_select", "embedding_gather", "add_rmsnorm", "add_rmsnorm_routes", "act_and_mul", "cast", "table_update", "norm_rope_store",
       "paged_attention", "router_topk", "moe_permute", "moe_route", "moe_route_fits", "linear", "attention_tc_fits", "attention_tc_few_fits", "moe_gemm1_gather_fits", "moe_gather", "moe_gemm1_act", "moe_gemm2",
       "moe_combine", "sample"]


def install(monkeypatch) -> None:
    """Make ``freetoken_b200.kernels.ops`` run these functions (CPU tests of the host logic)."""
    from freetoken_b200.kernels import ops

    for name in ALL:
        monkeypatch.setattr(ops, name, globals()[name])
