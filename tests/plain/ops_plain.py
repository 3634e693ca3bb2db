"""Plain PyTorch statements of every kernel entry point, same signatures as the product's ops.

Two uses, both in tests only: (1) the 32-bit reference that each CUDA kernel is compared
with on the GPU, at sizes of the test's choosing; (2) a stand-in for the kernels so that
the engine's host logic (packing, cache, block tables, slots) can be exercised on a
machine without a GPU.  Nothing here is imported by the product.

Formulas: CodeClaper/tinyllama.c cpu_op.c (rms_norm :44-64, rope :637-651, conv :836-889,
scan :924-958, attention :1010-1062) and sampler.c:107-257.
"""
from __future__ import annotations

import math

import torch

PAGE = 64


def _f(t):
    return t.to(torch.float64)


def embed(tokens, table, scale, out):
    out.copy_((_f(table)[tokens.long()] * scale).to(out.dtype))


def rmsnorm(x, weight, eps, out, rows=None):
    xs = _f(x if rows is None else x[rows.long()])
    s = 1.0 / torch.sqrt((xs * xs).sum(-1, keepdim=True) / xs.shape[-1] + eps)
    out.copy_((xs * s * _f(weight)).to(out.dtype))


def gated_rmsnorm(y, z, weight, eps, n_groups, norm_before_gate, out, out_scale=1.0, y_add=None):
    T, Di = y.shape
    y, z = _f(y), _f(z)
    if y_add is not None:
        y = y + _f(y_add)
    gate = z / (1.0 + torch.exp(-z))
    if weight is None:
        res = y * gate
    else:
        gs = Di // n_groups

        def norm(v):
            v = v.reshape(T, n_groups, gs)
            s = 1.0 / torch.sqrt((v * v).sum(-1, keepdim=True) / gs + eps)
            return (v * s).reshape(T, Di) * _f(weight)
        res = norm(y) * gate if norm_before_gate else norm(y * gate)
    out.copy_((res * out_scale).to(out.dtype))


def _gate_up(gate_up, interleaved):
    F = gate_up.shape[1] // 2
    if not interleaved:
        return _f(gate_up[:, :F]), _f(gate_up[:, F:])
    r = _f(gate_up).reshape(gate_up.shape[0], F // 8, 2, 8)
    return r[:, :, 0, :].reshape(-1, F), r[:, :, 1, :].reshape(-1, F)


def linear_swiglu(a, w, out, colscale=None, colbias=None):
    gu = torch.empty((a.shape[0], w.shape[0]), dtype=torch.float64)
    linear(a, w, gu, colscale, colbias)
    swiglu(gu, out, interleaved=True)


def swiglu(gate_up, out, interleaved=False):
    g, u = _gate_up(gate_up, interleaved)
    out.copy_((g / (1.0 + torch.exp(-g)) * u).to(out.dtype))


def gather_rows(x, rows, out):
    out.copy_(x[rows.long()])


def linear(a, w, out, colscale=None, colbias=None, accumulate=False):
    r = _f(a) @ _f(w).T
    if colscale is not None:
        r = r * _f(colscale)
    if colbias is not None:
        r = r + _f(colbias)
    if accumulate:
        r = r + _f(out)
    out.copy_(r.to(out.dtype))


def rope_kv_store(qkv, q_off, k_off, v_off, q_out, k_pages, v_pages, inv_freq, positions, row_seq, slots, block_table,
                  H, KV, hd, write_kv=True):
    T = qkv.shape[0]
    half = inv_freq.numel()
    ang = (positions.to(torch.float32)[:, None] * inv_freq.to(torch.float32)[None, :]).to(torch.float64)
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]

    def rot(x, n):
        x = _f(x).reshape(T, n, hd).clone()
        a, b = x[..., :half].clone(), x[..., half:2 * half].clone()
        x[..., :half] = a * c - b * s
        x[..., half:2 * half] = a * s + b * c
        return x

    q_out.copy_(rot(qkv[:, q_off:q_off + H * hd], H).reshape(T, H * hd).to(q_out.dtype))
    if not write_kv:
        return
    k = rot(qkv[:, k_off:k_off + KV * hd], KV).to(k_pages.dtype)
    v = qkv[:, v_off:v_off + KV * hd].reshape(T, KV, hd).to(v_pages.dtype)
    for t in range(T):
        p = int(positions[t])
        page = int(block_table[int(slots[int(row_seq[t])]), p // PAGE])
        k_pages[page, :, p % PAGE, :] = k[t]
        v_pages[page, :, p % PAGE, :] = v[t]


def attention(q, k_pages, v_pages, block_table, positions, row_seq, slots, out, H, KV, hd, scale, window=0,
              decode_max_keys=0, cu_seqlens=None, start_pos=None, max_keys=0, max_blocks=0, key_ranges=0):
    T = q.shape[0]
    res = torch.zeros((T, H, hd), dtype=torch.float64)
    qf = _f(q).reshape(T, H, hd)
    for t in range(T):
        p = int(positions[t])
        table = block_table[int(slots[int(row_seq[t])])]
        n_keys = p + 1
        start = n_keys - window if (window and n_keys > window) else 0
        idx = torch.arange(start, n_keys)
        pages = table[(idx // PAGE).long()].long()
        K = _f(k_pages[pages, :, (idx % PAGE).long(), :])          # [n, KV, hd]
        V = _f(v_pages[pages, :, (idx % PAGE).long(), :])
        for h in range(H):
            g = h // (H // KV)
            sc = (K[:, g] @ qf[t, h]) * scale
            pr = torch.softmax(sc, dim=0)
            res[t, h] = pr @ V[:, g]
    out.copy_(res.reshape(T, H * hd).to(out.dtype))


def mamba_conv(proj, xbc_off, dt_off, w, bias, dt_bias, A, conv_state, cu_seqlens, row_seq, slots, start_pos,
               xbc_out, dt_out, dA_out, single_rows=False, bf16_run=False, all_fresh=False):
    Cd, K = w.shape
    Hs = dt_bias.numel()
    wf = _f(w)
    for b in range(slots.numel()):
        t0, t1 = int(cu_seqlens[b]), int(cu_seqlens[b + 1])
        if t1 == t0:
            continue
        slot = int(slots[b])
        raw = _f(proj[t0:t1, xbc_off:xbc_off + Cd])
        prev = _f(conv_state[slot]) if int(start_pos[b]) > 0 else torch.zeros((K - 1, Cd), dtype=torch.float64)
        full = torch.cat([prev, raw], dim=0)                        # rows 0..K-2 = window, oldest first
        acc = torch.zeros_like(raw)
        for k in range(K):
            acc += full[k:k + (t1 - t0)] * wf[:, k][None, :]
        if bias is not None:
            acc = acc + _f(bias)
        act = acc / (1.0 + torch.exp(-acc))
        if bf16_run:
            act = act.to(torch.bfloat16).to(torch.float64)
        xbc_out[t0:t1] = act.to(xbc_out.dtype)
        if K > 1:
            conv_state[slot] = full[-(K - 1):].to(conv_state.dtype)
    d = _f(proj[:, dt_off:dt_off + Hs]) + _f(dt_bias)
    dtv = torch.where(d > 20.0, d, torch.log1p(torch.exp(torch.clamp(d, max=20.0))))
    dt_out.copy_(dtv.to(dt_out.dtype))
    dA_out.copy_(torch.exp(dtv * _f(A)).to(dA_out.dtype))


def ssm_scan(xbc, dt, dA, Dskip, state, cu_seqlens, slots, start_pos, y, Hs, P, N, G, chunks=None, A=None, y_part=None):
    # y_part: the engine may leave its outputs as two summands there and in y; the plain scan has one
    if y_part is not None:
        y_part.zero_()
    Di = Hs * P
    for b in range(slots.numel()):
        t0, t1 = int(cu_seqlens[b]), int(cu_seqlens[b + 1])
        if t1 == t0:
            continue
        slot = int(slots[b])
        S = _f(state[slot]).clone() if int(start_pos[b]) > 0 else torch.zeros((Hs, P, N), dtype=torch.float64)
        for t in range(t0, t1):
            x = _f(xbc[t, :Di]).reshape(Hs, P)
            Bm = _f(xbc[t, Di:Di + G * N]).reshape(G, N).repeat_interleave(Hs // G, dim=0)     # [Hs, N]
            Cm = _f(xbc[t, Di + G * N:]).reshape(G, N).repeat_interleave(Hs // G, dim=0)
            S = S * _f(dA[t])[:, None, None] + (x * _f(dt[t])[:, None])[:, :, None] * Bm[:, None, :]
            yt = (S * Cm[:, None, :]).sum(-1) + x * _f(Dskip)[:, None]
            y[t] = yt.reshape(Di).to(y.dtype)
        state[slot] = S.to(state.dtype)


def argmax(logits, out, work=None):
    out.copy_(torch.argmax(logits, dim=1).to(torch.int32))


def sample_row(logits, history, u, temperature, top_k, top_p, min_p, repeat_penalty, frequency_penalty,
               presence_penalty):
    """The reference's sample_token on one row (sampler.c:107-257), with the draw walking the
    survivors in token-id order from the uniform number u."""
    lg = logits.to(torch.float64).clone()
    V = lg.numel()
    if (repeat_penalty != 1.0 or frequency_penalty != 0.0 or presence_penalty != 0.0) and history is not None:
        win = [int(t) for t in history if 0 <= int(t) < V]
        for tid in dict.fromkeys(win):
            cnt = win.count(tid)
            lg[tid] = lg[tid] * repeat_penalty if lg[tid] <= 0 else lg[tid] / repeat_penalty
            lg[tid] -= cnt * frequency_penalty + presence_penalty
    no_filter = top_k == 0 and top_p >= 1.0 and min_p <= 1e-6
    if temperature <= 1e-6 or no_filter:
        return int(torch.argmax(lg))
    z = lg / temperature
    p = torch.exp(z - z.max())
    total = p.sum()
    order = torch.argsort(-p, stable=True)
    if 0 < top_k < V:
        order = order[:top_k]
    probs = p[order]
    cutoff = len(order)
    if min_p > 1e-6:
        keep = probs >= min_p * probs[0]
        nc = int(keep.sum()) if bool(keep.all()) else int(torch.argmin(keep.to(torch.int8)))
        if nc > 0:
            cutoff = nc
    if top_p < 1.0:
        cum = torch.cumsum(probs[:cutoff], 0) / total
        hit = (cum >= top_p).nonzero()
        if hit.numel():
            cutoff = min(cutoff, int(hit[0]) + 1)
    alive = torch.zeros(V, dtype=torch.float64)
    alive[order[:cutoff]] = p[order[:cutoff]]
    cdf = torch.cumsum(alive, 0)
    target = u * cdf[-1]
    idx = int((cdf > target).nonzero()[0]) if bool((cdf > target).any()) else int(alive.nonzero()[-1])
    return idx


def sample(logits, work, history, uniforms, temperature, top_k, top_p, min_p, repeat_penalty, frequency_penalty,
           presence_penalty, out):
    for r in range(logits.shape[0]):
        out[r] = sample_row(logits[r], None if history is None else history[r].tolist(), float(uniforms[r]),
                            temperature, top_k, top_p, min_p, repeat_penalty, frequency_penalty, presence_penalty)


ALL = ["embed", "rmsnorm", "gated_rmsnorm", "swiglu", "gather_rows", "linear", "linear_swiglu", "rope_kv_store", "attention",
       "mamba_conv", "ssm_scan", "argmax", "sample"]


def install(monkeypatch, ops_module):
    """Replaces the product's kernel entry points by the functions above (tests without a GPU)."""
    g = globals()
    for name in ALL:
        monkeypatch.setattr(ops_module, name, g[name])
