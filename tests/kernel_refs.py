"""Plain PyTorch references of the kernels, one per entry point of
``zinfer_b200.ops`` and with the same signature.  Written from the formulas (cited
in tests/plain_qwen3.py), with 32-bit arithmetic and simple loops; they share no
code with the kernels.  GPU tests compare each kernel with its reference; the
CPU tests of the engine's host logic put these in the kernels' place.
"""
from __future__ import annotations

import numpy as np
import torch


def embed_gather(table, ids, out=None):
    return table[ids.long()].to(torch.float32)


class Scaled:
    def __init__(self, delta, scale):
        self.delta, self.scale = delta, float(scale)


class Several:
    def __init__(self, terms, row_bias=None):
        self.terms, self.row_bias = [], row_bias
        for t in terms:
            if isinstance(t, Several):
                self.terms += t.terms
                if t.row_bias is not None:
                    self.row_bias = t.row_bias if self.row_bias is None else t.row_bias + self.row_bias
            elif t is not None and type(t).__name__ != "Carried":
                self.terms.append(t)


def _terms_sum(delta):
    """The 32-bit sum of what is pending (a tensor, Scaled, Several or nothing), or None."""
    if delta is None or type(delta).__name__ == "Carried":
        return None
    total = None
    for t in (delta.terms if isinstance(delta, Several) else [delta]):
        scale = 1.0
        if isinstance(t, Scaled):
            t, scale = t.delta, t.scale
        v = torch.tensor(scale, dtype=torch.float32) * t.to(torch.float32)
        total = v if total is None else total + v
    return total


def sum_norm(h, delta, w1, eps, out_dtype, w2=None, rows=None, bias=None):
    if isinstance(delta, Several) and delta.row_bias is not None:
        bias = delta.row_bias if bias is None else delta.row_bias + bias
        delta = Several(delta.terms)
    x1 = add_rmsnorm(h, _terms_sum(delta), w1, eps, out_dtype, rows=rows, bias=bias)
    if w2 is None:
        return x1
    return x1, add_rmsnorm(h, None, w2, eps, out_dtype, rows=rows)


def add_rmsnorm_pair(h, delta, w1, w2, eps1, eps2, out_dtype, bias=None):
    x1 = sum_norm(h, delta, w1, eps1, out_dtype, bias=bias)
    return x1, sum_norm(h, None, w2, eps2, out_dtype)


def embed_bigram(table, bigram, ids, step, last_token, scale, buckets, mul_prev, mul_cur):
    out = torch.empty((ids.shape[0], table.shape[1]), dtype=torch.float32)
    for s in range(step.n_seqs):
        a, b = int(step.cu_q[s]), int(step.cu_q[s + 1])
        slot = int(step.state_slots[s])
        for t in range(a, b):
            tok = int(ids[t])
            x = table[tok].to(torch.float32) * torch.tensor(scale, dtype=torch.float32)
            if bigram is not None:
                if int(step.positions[t]) == 0:
                    row = buckets
                else:
                    prev = int(ids[t - 1]) if t > a else int(last_token[slot, 0])
                    row = (prev * mul_prev + tok * mul_cur) % buckets
                x = x + bigram[row].to(torch.float32)
            out[t] = x
        if b > a:
            last_token[slot, 0] = int(ids[b - 1])
    return out


def add_rmsnorm(h, delta, weight, eps, out_dtype, rows=None, out=None, bias=None):
    scale = 1.0
    if type(delta).__name__ == "Carried":      # nothing pending
        delta = None
    if isinstance(delta, Several):
        if delta.row_bias is not None:
            bias = delta.row_bias if bias is None else delta.row_bias + bias
        delta = _terms_sum(delta)
    if isinstance(delta, Scaled):
        delta, scale = delta.delta, delta.scale
    if rows is None:
        if delta is not None:
            h += torch.tensor(scale, dtype=torch.float32) * delta.to(torch.float32)
        if bias is not None:
            h += bias
        x = h
    else:   # picked rows (repeats allowed): h itself stays as it is
        x = h[rows.long()]
        if delta is not None:
            x = x + torch.tensor(scale, dtype=torch.float32) * delta[rows.long()].to(torch.float32)
        if bias is not None:
            x = x + bias
    ms = (x * x).mean(dim=-1, keepdim=True)
    inv = 1.0 / torch.sqrt(ms + torch.tensor(eps, dtype=torch.float32))
    return (x * weight * inv).to(out_dtype)


def residual_add(h, delta):
    if isinstance(delta, Several):
        delta = _terms_sum(delta)
    scale = 1.0
    if isinstance(delta, Scaled):
        delta, scale = delta.delta, delta.scale
    h += torch.tensor(scale, dtype=torch.float32) * delta.to(torch.float32)


def scale_(x, factor):
    x *= factor
    return x


def sigmoid_gate(x, gate, out=None, group=1):
    res = (x.to(torch.float32) * torch.sigmoid(gate.to(torch.float32)).repeat_interleave(group, dim=1)).to(x.dtype)
    if out is not None:
        out.copy_(res)
        return out
    return res


ACTIVATIONS = {"silu": 0, "gelu_tanh": 1}


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(0.7978845608028654 * (z + 0.044715 * z * z * z)))


SWIGLU_INTERLEAVE = 64


def interleave_gate_up(gate, up, block=64):
    I, K = gate.shape
    return torch.stack([gate.view(I // block, block, K), up.view(I // block, block, K)], dim=1).reshape(2 * I, K).contiguous()


def linear_swiglu(x, w_interleaved, out_dtype=None, activation="silu"):
    return swiglu(linear(x, w_interleaved, out_dtype=torch.float32), interleave=64, activation=activation).to(out_dtype or x.dtype)


def swiglu(gate_up, out=None, out_dtype=None, interleave=0, activation="silu"):
    I = gate_up.shape[1] // 2
    if interleave:
        blocks = gate_up.reshape(gate_up.shape[0], I // interleave, 2, interleave)
        gate_up = torch.cat([blocks[:, :, 0].reshape(-1, I), blocks[:, :, 1].reshape(-1, I)], dim=1)
    g, u = gate_up[:, :I].to(torch.float32), gate_up[:, I:].to(torch.float32)
    if activation == "gelu_tanh":
        return (gelu_tanh(g) * u).to(out_dtype or gate_up.dtype)
    return (g / (1.0 + torch.exp(-g)) * u).to(out_dtype or gate_up.dtype)


def rope_table(n_pos, head_dim, theta, device, factor=1.0):
    half = head_dim // 2
    exponent = (np.arange(half, dtype=np.float32) * np.float32(2)) / np.float32(head_dim)
    p = np.power(np.float64(np.float32(theta)), exponent.astype(np.float64)).astype(np.float32)
    inv = ((np.float32(1) / p).astype(np.float32) / np.float32(factor)).astype(np.float32)
    ang = (np.arange(n_pos, dtype=np.float32)[:, None] * inv[None, :]).astype(np.float32)
    cos = torch.from_numpy(np.cos(ang.astype(np.float64)).astype(np.float32)).to(device)
    sin = torch.from_numpy(np.sin(ang.astype(np.float64)).astype(np.float32)).to(device)
    return cos, sin


def qk_norm_rope_store(qkv, num_heads, num_kv_heads, head_dim, q_weight, k_weight, eps, cos, sin, positions,
                       k_cache, v_cache, slots, page_size, write_kv=True, out_dtype=None):
    T = qkv.shape[0]
    nq, nkv, d = num_heads, num_kv_heads, head_dim
    half = d // 2
    pos = positions.long()

    def norm_rope(x, w):  # x [T, heads, d] float32
        if w is not None:
            ms = (x * x).mean(dim=-1, keepdim=True)
            x = x * w * (1.0 / torch.sqrt(ms + torch.tensor(eps, dtype=torch.float32)))
        if cos is not None:
            c, s = cos[pos][:, None, :], sin[pos][:, None, :]
            a, b = x[..., :half], x[..., half:]
            x = torch.cat([a * c - b * s, b * c + a * s], dim=-1)
        return x

    q = norm_rope(qkv[:, :nq * d].to(torch.float32).reshape(T, nq, d), q_weight)
    qkv[:, :nq * d] = q.reshape(T, nq * d).to(qkv.dtype)
    if not write_kv:
        return qkv
    k = norm_rope(qkv[:, nq * d:(nq + nkv) * d].to(torch.float32).reshape(T, nkv, d), k_weight).to(qkv.dtype)
    v = qkv[:, (nq + nkv) * d:(nq + 2 * nkv) * d].reshape(T, nkv, d)
    for t in range(T):
        slot = int(slots[t])
        k_cache[slot // page_size, :, slot % page_size, :] = k[t]
        v_cache[slot // page_size, :, slot % page_size, :] = v[t]
    return qkv


def linear(x, weight, out_dtype=None, out=None, allow_partials=False, fresh_weight=False, relu2=False):
    y = x.to(torch.float32) @ weight.to(torch.float32).T
    if relu2:
        y = torch.relu(y) ** 2
    if out is not None:
        out.copy_(y)
        return out
    return y.to(out_dtype or x.dtype)


def linear_cuda_cores(x, weight, out_dtype=None):
    return linear(x, weight, out_dtype=out_dtype)


def tensor_core_linear_ok(x, weight):
    return False


def linear_heads_ok(x, weight, out):
    return False


def linear_batched(x, weight, out, bias=None, relu2=False):
    y = torch.einsum("bmk,bnk->bmn", x.to(torch.float32), weight.to(torch.float32))
    if bias is not None:
        y = y + bias[:, None, :]
    if relu2:
        y = torch.relu(y) ** 2
    out.copy_(y)
    return out


def linear_grouped(x, weight, out, row_src, tile_group, n_tiles, tile_rows, relu2=False):
    for tile in range(int(n_tiles[0])):
        w = weight[int(tile_group[tile])].to(torch.float32)
        for r in range(tile * tile_rows, (tile + 1) * tile_rows):
            src = int(row_src[r])
            if src < 0:
                continue
            y = w @ x[src].to(torch.float32)
            out[r] = torch.relu(y) ** 2 if relu2 else y
    return out


# ---------------------------------------------------------------- mixture of experts
MOE_TILE_ROWS_SMALL, MOE_TILE_ROWS = 16, 64


def moe_route(logits, correction, top, renormalize=False):
    s = torch.softmax(logits.to(torch.float32), dim=-1)
    pick = s if correction is None else s + correction
    chosen = torch.topk(pick, top, dim=-1).indices
    weight = torch.gather(s, 1, chosen)
    if renormalize:
        weight = weight / weight.sum(dim=-1, keepdim=True)
    return chosen.to(torch.int32), weight


def moe_router(x, w_router, correction, top, renormalize=False):
    return moe_route(linear(x, w_router, out_dtype=torch.float32), correction, top, renormalize)


def linear_few_rows_ok(x, weight):
    return False


def moe_align(chosen, experts, tile_rows):
    T, top = chosen.shape
    flat = chosen.reshape(-1).tolist()
    row_token, row_self, tile_expert = [], [], []
    pair_row = [-1] * len(flat)
    for e in range(experts):
        pairs = [p for p, c in enumerate(flat) if c == e]
        for p in pairs:
            pair_row[p] = len(row_token)
            row_self.append(len(row_token))
            row_token.append(p // top)
        pad = -len(pairs) % tile_rows
        row_token += [-1] * pad
        row_self += [-1] * pad
        tile_expert += [e] * ((len(pairs) + pad) // tile_rows)
    cap = (-(-len(flat) // tile_rows) + experts) * tile_rows
    n_tiles = len(tile_expert)
    row_token += [-1] * (cap - len(row_token))
    row_self += [-1] * (cap - len(row_self))
    i32 = lambda v: torch.tensor(v, dtype=torch.int32)
    return i32(row_token), i32(row_self), i32(pair_row), i32(tile_expert + [0] * (cap // tile_rows - n_tiles)), i32([n_tiles])


MOE_TILE_ROWS_TENSOR = 128


def linear_grouped_tensor_ok(weight):
    return False


def gather_rows(x, row_src):
    out = torch.zeros((row_src.numel(), x.shape[1]), dtype=x.dtype)
    for r, src in enumerate(row_src.tolist()):
        if src >= 0:
            out[r] = x[src]
    return out


def moe_combine(y, x, chosen, weight, pair_row, experts):
    T, H = x.shape
    top = chosen.shape[1]
    out = torch.zeros((T, H), dtype=torch.float32)
    for t in range(T):
        for k in range(top):
            e = int(chosen[t, k])
            v = y[int(pair_row[t * top + k])] if e < experts else x[t].to(torch.float32)
            out[t] += weight[t, k] * v
    return out.to(x.dtype)


# ---------------------------------------------------------------- recurrent mixers
def _conv_inputs(x, x_bias, state_rows, taps):
    """The carried inputs (oldest first) followed by this step's inputs of one request."""
    return torch.cat([state_rows[:taps - 1], x.to(torch.float32) + x_bias], dim=0)


def causal_conv(x, x_bias, kernel, bias, state, step):
    T, C = x.shape
    taps = kernel.shape[1]
    u = torch.empty((T, C), dtype=torch.float32)
    cu, slots = step.cu_q.tolist(), step.state_slots.tolist()
    for s in range(step.n_seqs):
        a, b = cu[s], cu[s + 1]
        seq = _conv_inputs(x[a:b], x_bias, state[slots[s]], taps)
        for t in range(b - a):
            u[a + t] = bias + (kernel * seq[t:t + taps].T).sum(dim=1)
    return u


def rglru_scan(u, gates, block_width, r_bias, i_bias, lam, decay_scale, y, y_bias, x, x_bias, state, step):
    T, C = u.shape
    taps = state.shape[1]
    g = gates.reshape(T, C // block_width, 2, block_width)
    r = torch.sigmoid(g[:, :, 0].reshape(T, C) + r_bias)
    i = torch.sigmoid(g[:, :, 1].reshape(T, C) + i_bias)
    log_a = -decay_scale * r * torch.nn.functional.softplus(lam)
    a = torch.exp(log_a)
    drive = torch.sqrt(-torch.expm1(2.0 * log_a)) * i * u
    out = torch.empty((T, C), dtype=torch.float32)
    cu, slots = step.cu_q.tolist(), step.state_slots.tolist()
    for s in range(step.n_seqs):
        lo, hi = cu[s], cu[s + 1]
        S = state[slots[s], taps - 1].clone()
        for t in range(lo, hi):
            S = a[t] * S + drive[t]
            out[t] = S
        if taps > 1:
            seq = _conv_inputs(x[lo:hi], x_bias, state[slots[s]], taps)
            state[slots[s], :taps - 1] = seq[seq.shape[0] - (taps - 1):]
        state[slots[s], taps - 1] = S
    return (out * gelu_tanh(y.to(torch.float32) + y_bias)).to(y.dtype)


def rglru_decode(yx, y_bias, x_bias, kernel, bias, w_gates, r_bias, i_bias, lam, decay_scale, state, step):
    n, C = yx.shape[0], yx.shape[1] // 2
    B, _, bw = w_gates.shape
    y, x = yx[:, :C], yx[:, C:]
    u = causal_conv(x, x_bias, kernel, bias, state, step)
    gates = torch.einsum("tbi,boi->tbo", u.view(n, B, bw), w_gates.to(torch.float32)).contiguous()
    return rglru_scan(u, gates, bw, r_bias, i_bias, lam, decay_scale, y, y_bias, x, x_bias, state, step)


# ----------------------------------------------------------------- latent attention
def _rotate_first(v, cos, sin, rot_dims):
    half = rot_dims // 2
    a, b = v[..., :half], v[..., half:rot_dims]
    return torch.cat([a * cos - b * sin, b * cos + a * sin, v[..., rot_dims:]], dim=-1)


def latent_prepare(proj, heads, dim, rot_dim, rank, rot_dims, c_weight, eps, cos, sin, positions, q_eff, cache, slots):
    T = proj.shape[0]
    D = rank + rot_dim
    pos = positions.long()
    c, s = cos[pos], sin[pos]
    q = proj[:, :heads * (dim + rot_dim)].to(torch.float32).reshape(T, heads, dim + rot_dim)
    q_eff.view(T, heads, D)[:, :, rank:] = _rotate_first(q[:, :, dim:], c[:, None, :], s[:, None, :], rot_dims).to(q_eff.dtype)
    if cache is None:
        return
    kv = proj[:, heads * (dim + rot_dim):heads * (dim + rot_dim) + D].to(torch.float32)
    lat = kv[:, :rank]
    lat = lat * c_weight * (1.0 / torch.sqrt((lat * lat).mean(dim=-1, keepdim=True) + torch.tensor(eps, dtype=torch.float32)))
    row = torch.cat([lat, _rotate_first(kv[:, rank:], c, s, rot_dims)], dim=-1).to(cache.dtype)
    page_size = cache.shape[2]
    for t in range(T):
        slot = int(slots[t])
        if slot >= 0:
            cache[slot // page_size, 0, slot % page_size] = row[t]


def latent_decode_splits(n_dec, head_groups, sm_count, max_kv_len, fixed=False):
    return 1


def latent_attention(q_eff, cache, block_tables, step, heads, rank, page_size, window, scale, sink_logit=None):
    T = q_eff.shape[0]
    D = cache.shape[-1]
    full = paged_attention(q_eff, cache, cache, block_tables, step.cu_q, step.kv_lens, step.tile_seq, step.tile_q0,
                           heads, 1, D, page_size, window, scale, sink_logit=sink_logit)
    return full.view(T, heads, D)[:, :, :rank].reshape(T, heads * rank).contiguous()


def attention_tile_rows():
    return 16


def attention_prefill_tile_rows():
    return 128


def paged_attention(q, k_cache, v_cache, block_tables, cu_q, kv_lens, tile_seq, tile_q0, num_heads, num_kv_heads,
                    head_dim, page_size, window, scale, out=None, sink=0.0, keep_first=0, value_dim=None, sink_logit=None,
                    softcap=0.0, dist_bias=None):
    T = q.shape[0]
    nq, nkv, d = num_heads, num_kv_heads, head_dim
    dv = int(value_dim or d)
    g = nq // nkv
    o = torch.zeros((T, nq * dv), dtype=torch.float32, device=q.device)
    n = kv_lens.shape[0]
    for s in range(n):
        a, b = int(cu_q[s]), int(cu_q[s + 1])
        kv_len = int(kv_lens[s])
        ctx = kv_len - (b - a)
        for t in range(a, b):
            pos = ctx + (t - a)
            lo = 0 if not window else max(0, pos - window + 1)
            js = torch.arange(lo, pos + 1, device=q.device)
            if window and keep_first and lo > 0:      # the request's first tokens stay visible beside the window
                js = torch.cat([torch.arange(0, min(keep_first, lo), device=q.device), js])
            pages = block_tables[s, (js // page_size)].long()
            offs = js % page_size
            K = k_cache[pages, :, offs, :].to(torch.float32)   # [keys, nkv, d]
            V = v_cache[pages, :, offs, :].to(torch.float32)
            qt = q[t, :nq * d].to(torch.float32).reshape(nq, d)
            for h in range(nq):
                sc = (K[:, h // g, :] @ qt[h]) * scale
                if softcap:
                    sc = softcap * torch.tanh(sc / softcap)
                if dist_bias is not None:
                    sc = sc + dist_bias[h, (pos - js).clamp(max=dist_bias.shape[1] - 1)]
                if sink_logit is not None:       # exp(sink_logit[h]) joins the denominator
                    m = torch.maximum(sc.max(), sink_logit[h])
                    e = torch.exp(sc - m)
                    p = e / (torch.exp(sink_logit[h] - m) + e.sum())
                elif sink:       # `sink` keys of score 0 without a value
                    e = torch.exp(sc - sc.max())
                    p = e / (sink * torch.exp(-sc.max()) + e.sum())
                else:
                    p = torch.softmax(sc, dim=0)
                o[t, h * dv:(h + 1) * dv] = p @ V[:, h // g, :]
    return o.to(q.dtype)


def argmax(logits, out=None):
    return torch.argmax(logits, dim=-1).to(torch.int32)


def linear_argmax(x, weight):
    logits = linear(x, weight, out_dtype=torch.float32)
    return logits, argmax(logits)


def attention(q, k_cache, v_cache, block_tables, step, num_heads, num_kv_heads, head_dim, page_size, window, scale, sink=0.0,
              keep_first=0, value_dim=None, sink_logit=None, softcap=0.0, dist_bias=None):
    return paged_attention(q, k_cache, v_cache, block_tables, step.cu_q, step.kv_lens, step.tile_seq, step.tile_q0,
                           num_heads, num_kv_heads, head_dim, page_size, window, scale, sink=sink, keep_first=keep_first,
                           value_dim=value_dim, sink_logit=sink_logit, softcap=softcap, dist_bias=dist_bias)


def patch_tokens(ids, prev, dst, src):
    for i in range(dst.numel()):
        if int(dst[i]) >= 0:
            ids[int(dst[i])] = prev[int(src[i])]


def decode_fused_ok(dtype, num_heads, num_kv_heads, head_dim, step):
    return False


def count_tokens(counts_row, tokens):
    for t in tokens.tolist():
        counts_row[int(t)] += 1


def sample(logits, temperature, seeds, draw_index, top_k=None, top_p=None, min_p=None, repetition_penalty=None,
           presence_penalty=None, frequency_penalty=None, count_rows=None, counts=None, out=None):
    """The reference's chain per row (penalties, top-k, temperature, min-p, top-p, draw) with the
    host sampler of tests/plain_qwen3.py.  The uniform number of a draw comes from (seed, draw
    index) alone, as on the device, but by another generator: tokens are comparable with the
    kernel's only where the kept set has one member (greedy rows)."""
    import hashlib

    import plain_qwen3 as P

    R, V = logits.shape
    res = torch.empty((R,), dtype=torch.int32)
    get = lambda t, i, default: default if t is None else t[i].item()
    for i in range(R):
        row = logits[i].float().numpy()
        crow = int(get(count_rows, i, -1))
        if counts is not None and crow >= 0:
            hist = np.repeat(np.arange(V), counts[crow].numpy())
            row = P.adjusted_logits(row, hist.tolist(), get(repetition_penalty, i, 1.0), get(presence_penalty, i, 0.0),
                                    get(frequency_penalty, i, 0.0))
        T, k = float(temperature[i]), int(get(top_k, i, 0))
        if T <= 0.0 or k == 1:
            tok = int(np.argmax(row))
        else:
            p = P.kept_distribution(row, T, k, float(get(top_p, i, 1.0)), float(get(min_p, i, 0.0)))
            h = hashlib.sha256(f"{int(seeds[i])}:{int(draw_index[i])}".encode()).digest()
            u = int.from_bytes(h[:8], "little") / 2.0 ** 64
            tok = int(min(np.searchsorted(np.cumsum(p), u, side="right"), V - 1))
            if p[tok] == 0.0:
                tok = int(np.argmax(p))
        if counts is not None and crow >= 0:
            counts[crow, tok] += 1
        res[i] = tok
    return res


# ------------------------------------------------ the parts of the output-norm blocks and linear attention
class Carried:
    def __init__(self, x):
        self.x = x


def _plain(delta):
    if delta is None:
        return None
    scale = 1.0
    if isinstance(delta, Scaled):
        delta, scale = delta.delta, delta.scale
    return delta.to(torch.float32) * scale


def norm_residual(h, a, weight, eps, out_dtype, b=None):
    y = _plain(a)
    if b is not None:
        y = y + _plain(b)
    h += y / torch.sqrt((y * y).mean(-1, keepdim=True) + eps) * weight
    return h if out_dtype == torch.float32 else h.to(out_dtype)


def cast_rows(h, dtype):
    return h if dtype == torch.float32 else h.to(dtype)


def relu2_(x):
    x.copy_(torch.relu(x.to(torch.float32)) ** 2)
    return x


def qk_prepare(qkv, num_heads, num_kv_heads, head_dim, rot_dims, q_weight, k_weight, eps, cos, sin, positions, k_cache,
               v_cache, slots, page_size, values_from_keys=False, write_kv=True, value_dim=None):
    T, nq, nkv, d = qkv.shape[0], num_heads, num_kv_heads, head_dim
    dv = int(value_dim or d)
    pos = positions.long()

    def prep(x, w):                                        # [T, heads, d] float32
        if w is not None:
            x = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w
        if cos is not None:
            x = _rotate_first(x, cos[pos][:, None, :], sin[pos][:, None, :], rot_dims)
        return x

    q = qkv[:, :nq * d].to(torch.float32).reshape(T, nq, d)
    qn = prep(q, q_weight)
    if write_kv:
        k_raw = qkv[:, nq * d:(nq + nkv) * d].to(torch.float32).reshape(T, nkv, d)
        kn = prep(k_raw, k_weight)
        v = k_raw if values_from_keys else \
            qkv[:, (nq + nkv) * d:(nq + nkv) * d + nkv * dv].to(torch.float32).reshape(T, nkv, dv)
        for t in range(T):
            slot = int(slots[t])
            if slot < 0:
                continue
            k_cache[slot // page_size, :, slot % page_size] = kn[t].to(k_cache.dtype)
            v_cache[slot // page_size, :, slot % page_size] = v[t].to(v_cache.dtype)
    qkv[:, :nq * d] = qn.reshape(T, nq * d).to(qkv.dtype).clone()      # (qn is qkv itself where nothing was done to it)
    return qkv


def _requests(step):
    cu = [int(v) for v in step.cu_q[:step.n_seqs + 1]]
    return [(s, cu[s], cu[s + 1], int(step.state_slots[s])) for s in range(step.n_seqs)]


def short_conv(x, kernel, tail, step, activation="silu"):
    T, C = x.shape
    taps = kernel.shape[1]
    y = torch.zeros((T, C), dtype=torch.float32)
    for _, a, b, slot in _requests(step):
        full = torch.cat([tail[slot].to(torch.float32).reshape(taps - 1, C), x[a:b].to(torch.float32)])
        for t in range(b - a):
            y[a + t] = (full[t:t + taps] * kernel.T).sum(0)
    return y * torch.sigmoid(y) if activation == "silu" else y


def short_conv_carry(x, taps, tail, step):
    if taps <= 1:
        return
    C = x.shape[1]
    for _, a, b, slot in _requests(step):
        full = torch.cat([tail[slot].to(torch.float32).reshape(taps - 1, C), x[a:b].to(torch.float32)])
        tail[slot] = full[full.shape[0] - (taps - 1):].reshape(tail[slot].shape)


def decay_sigmoid_root_(z, bias, tau):
    z.copy_(torch.exp(torch.nn.functional.logsigmoid(z + (bias if bias is not None else 0.0)) / tau))
    return z


def decay_exp_softplus_(z, bias, a_log, head_dim):
    x = torch.nn.functional.softplus(z + (bias if bias is not None else 0.0))
    z.copy_(torch.exp(-torch.exp(a_log).repeat_interleave(head_dim) * x))
    return z


def unit_norm_(x, heads, head_dim, eps, scale=1.0):
    v = x[:, :heads * head_dim].reshape(x.shape[0], heads, head_dim)
    x[:, :heads * head_dim] = (scale * v / torch.sqrt((v * v).sum(-1, keepdim=True) + eps)).reshape(x.shape[0], -1)
    return x


def sigmoid_rows(x):
    return torch.sigmoid(x.to(torch.float32)).contiguous()


def linear_recurrence(q, k, v, decay, beta, q_scale, state, heads, key_heads, dim, vdim, step):
    T = q.shape[0]
    out = torch.zeros((T, heads * vdim), dtype=torch.float32)
    rep = heads // key_heads
    qf, kf, vf = (t.to(torch.float32) for t in (q, k, v))
    for _, a, b, slot in _requests(step):
        S = state[slot].reshape(heads, dim, vdim).clone()
        for t in range(a, b):
            for h in range(heads):
                kk = kf[t, (h // rep) * dim:(h // rep + 1) * dim]
                qq = qf[t, (h // rep) * dim:(h // rep + 1) * dim] * q_scale
                Sh = decay[t, h * dim:(h + 1) * dim].unsqueeze(-1) * S[h]
                u = vf[t, h * vdim:(h + 1) * vdim]
                if beta is not None:
                    u = beta[t, h] * (u - Sh.T @ kk)
                S[h] = Sh + kk.unsqueeze(-1) * u.unsqueeze(0)
                out[t, h * vdim:(h + 1) * vdim] = S[h].T @ qq
        state[slot] = S.reshape(state[slot].shape)
    return out


def head_norm_gate(o, weight, eps, gate, gate_kind, heads, vdim, out_dtype):
    T = o.shape[0]
    x = o.reshape(T, heads, vdim)
    g = gate.to(torch.float32).reshape(T, heads, vdim)
    act = g * torch.sigmoid(g) if gate_kind == "silu" else torch.sigmoid(g)
    return (x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * weight * act).reshape(T, heads * vdim).to(out_dtype)


def moe_route_grouped(logits, top, score="sigmoid", groups=1, keep=1, scale=1.0, renormalize=False, correction=None):
    T, NR = logits.shape
    s = torch.sigmoid(logits) if score == "sigmoid" else torch.softmax(logits, dim=-1)
    c = s if correction is None else s + correction          # what is compared; the weights stay uncorrected
    per = NR // groups
    gscore = c.reshape(T, groups, per).topk(min(2, per), dim=-1).values.sum(-1)
    best = gscore.topk(keep, dim=-1).indices
    allowed = torch.zeros((T, groups), dtype=torch.bool).scatter_(1, best, True).repeat_interleave(per, dim=1)
    pick = torch.where(allowed, c, torch.full_like(c, -float("inf")))
    chosen = pick.topk(top, dim=-1).indices
    weight = s.gather(1, chosen)
    if renormalize:
        weight = weight / weight.sum(-1, keepdim=True)
    return chosen.to(torch.int32), (weight * scale).to(torch.float32)


def moe_router_grouped(x, w_router, top, score="sigmoid", groups=1, keep=1, scale=1.0, renormalize=False, correction=None):
    return moe_route_grouped(x.to(torch.float32) @ w_router.to(torch.float32).T, top, score, groups, keep, scale, renormalize,
                             correction)


# ------------------------------------------------ rows of projections, rescaled rotations, clamped gates, logits routers
def clamped_gate(gate_up, limit, alpha, shift, out_dtype, interleave=0):
    gu = gate_up.to(torch.float32)
    I = gu.shape[1] // 2
    g, u = gu[:, :I].clamp(max=limit), gu[:, I:].clamp(min=-limit, max=limit)
    return (g * torch.sigmoid(alpha * g) * (u + shift)).to(out_dtype)


def rmsnorm_rows(x, weight, eps, out_dtype):
    v = x.to(torch.float32)
    return (v * weight * (1.0 / torch.sqrt((v * v).mean(dim=-1, keepdim=True) + torch.tensor(eps, dtype=torch.float32)))).to(out_dtype)


def rope_table_freqs(n_pos, freqs, magnitude=1.0):
    angle = torch.arange(n_pos, dtype=torch.float32, device=freqs.device)[:, None] * freqs[None, :]
    return ((torch.cos(angle.double()) * magnitude).to(torch.float32), (torch.sin(angle.double()) * magnitude).to(torch.float32))


def qkv_rows_prepare(proj, bias, num_heads, num_kv_heads, head_dim, value_dim, n_gate, q_weight, k_weight, eps, rot_dims, cos, sin,
                     positions, k_cache, v_cache, slots, page_size, out_dtype):
    T = proj.shape[0]
    qn, kn, vn = num_heads * head_dim, num_kv_heads * head_dim, num_kv_heads * value_dim
    row = proj.to(torch.float32) + (bias if bias is not None else 0.0)
    q, k, v, gate = row[:, :qn], row[:, qn:qn + kn], row[:, qn + kn:qn + kn + vn], row[:, qn + kn + vn:]

    def finish(x, w, heads):
        if w is not None:
            x = x * w * (1.0 / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + torch.tensor(eps, dtype=torch.float32)))
        x = x.reshape(T, heads, head_dim)
        if cos is not None:
            pos = positions.long()
            x = _rotate_first(x, cos[pos][:, None, :], sin[pos][:, None, :], rot_dims)
        return x

    qo = finish(q, q_weight, num_heads).reshape(T, qn).to(out_dtype)
    ko = finish(k, k_weight, num_kv_heads).to(out_dtype)
    vo = v.reshape(T, num_kv_heads, value_dim).to(out_dtype)
    for t in range(T):
        slot = int(slots[t])
        if slot >= 0:
            k_cache[slot // page_size, :, slot % page_size] = ko[t]
            v_cache[slot // page_size, :, slot % page_size] = vo[t]
    return qo, (gate.to(out_dtype).contiguous() if n_gate else None)


def _rotate_neighbours(v, cos, sin, rot_dims):
    a, b = v[..., 0:rot_dims:2], v[..., 1:rot_dims:2]
    turned = torch.stack([a * cos - b * sin, b * cos + a * sin], dim=-1).flatten(-2)
    return torch.cat([turned, v[..., rot_dims:]], dim=-1)


def latent_prepare_rows(q, kv, heads, dim, rot_dim, rank, rot_dims, neighbours, c_weight, eps, cos, sin, positions, q_eff, cache,
                        slots):
    T = q.shape[0]
    D = rank + rot_dim
    pos = positions.long()
    c, s = cos[pos], sin[pos]
    turn = _rotate_neighbours if neighbours else _rotate_first
    qs = q[:, :heads * (dim + rot_dim)].to(torch.float32).reshape(T, heads, dim + rot_dim)
    q_eff.view(T, heads, D)[:, :, rank:] = turn(qs[:, :, dim:], c[:, None, :], s[:, None, :], rot_dims).to(q_eff.dtype)
    if cache is None:
        return
    rows = kv[:, :D].to(torch.float32)
    lat = rows[:, :rank]
    lat = lat * c_weight * (1.0 / torch.sqrt((lat * lat).mean(dim=-1, keepdim=True) + torch.tensor(eps, dtype=torch.float32)))
    row = torch.cat([lat, turn(rows[:, rank:], c, s, rot_dims)], dim=-1).to(cache.dtype)
    page_size = cache.shape[2]
    for t in range(T):
        slot = int(slots[t])
        if slot >= 0:
            cache[slot // page_size, 0, slot % page_size] = row[t]


def moe_router_top_logits(x, w_router, bias, top):
    z = x.to(torch.float32) @ w_router.to(torch.float32).T
    if bias is not None:
        z = z + bias
    order = torch.sort(z, dim=-1, descending=True, stable=True).indices[:, :top]
    weight = torch.softmax(torch.gather(z, 1, order), dim=-1)
    return order.to(torch.int32), weight
