"""Plain, slow Falcon-H1 forward pass: whole sequences, no cache, one function per part.

This is the oracle of the test-suite.  It is written from the formulas of
CodeClaper/tinyllama.c (each function cites the file and lines that state the
math) and shares no code with the product package: it takes a plain ``dict``
of configuration values and a ``dict`` of numpy arrays keyed by tensor name.

Everything is computed in float64 unless ``dtype`` says otherwise, with two
deliberate exceptions that follow the reference's 32-bit arithmetic because a
64-bit evaluation would *differ* from every 32-bit engine by more than
rounding: the rotary angle is the float32 product of the float32 position and
the float32 inverse frequency (cpu_op.c:644-646).

Where the reference has no statement (the muP multipliers, the projection
biases, norm-before-gate), the placement used here is the definition that the
product follows; those lines say "not in the reference".
"""
from __future__ import annotations

import numpy as np


# --------------------------------------------------------------------------
# small helpers
# --------------------------------------------------------------------------
def _get(cfg: dict, key: str, default):
    v = cfg.get(key, default)
    return default if v is None else v


def derived(cfg: dict) -> dict:
    """Sizes derived from config.json keys (falcon_h1.c:108-124, core.c:1611-1636)."""
    D = cfg["hidden_size"]
    H = cfg["num_attention_heads"]
    KV = _get(cfg, "num_key_value_heads", H)
    hd = _get(cfg, "head_dim", D // H)
    d_ssm = _get(cfg, "mamba_d_ssm", None)
    if d_ssm is None:
        d_ssm = int(_get(cfg, "mamba_expand", 2) * D)
    Hs = cfg["mamba_n_heads"]
    P = cfg.get("mamba_d_head", "auto")
    if P in (None, "auto"):
        P = d_ssm // Hs
    G = _get(cfg, "mamba_n_groups", 1)
    N = cfg["mamba_d_state"]
    K = _get(cfg, "mamba_d_conv", 4)
    conv_dim = d_ssm + 2 * G * N                       # falcon_h1.c:124
    proj_dim = d_ssm + conv_dim + Hs                   # falcon_h1.c:342
    return dict(D=D, H=H, KV=KV, hd=hd, Di=d_ssm, Hs=Hs, P=P, G=G, N=N, K=K,
                Cd=conv_dim, Pd=proj_dim, F=cfg["intermediate_size"], V=cfg["vocab_size"],
                L=cfg["num_hidden_layers"])


def bf16_round(x):
    """Round to the nearest bfloat16 (ties to even), keeping the array's type.  Passed as
    ``rnd`` to forward() it models a bfloat16 engine that keeps 32-bit accumulators: the
    inputs of every matrix product are rounded -- activations that a projection reads, the
    stored queries, keys and values, the softmax numerators that multiply the values, and
    x|B|C as the convolution hands them to the scan -- nothing else is."""
    x32 = np.ascontiguousarray(x, dtype=np.float32)
    u = x32.view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    return u.astype(np.uint32).view(np.float32).astype(np.asarray(x).dtype).reshape(np.shape(x))


def _same(x):
    return x


def silu(x):
    """x / (1 + exp(-x))  (cpu_op.c:332-335)."""
    return x / (1.0 + np.exp(-x))


def softplus(x):
    """x > 20 ? x : log1p(exp(x))  (cpu_op.c:354-356)."""
    x = np.asarray(x)
    return np.where(x > 20.0, x, np.log1p(np.exp(np.minimum(x, 20.0))))


# --------------------------------------------------------------------------
# parts
# --------------------------------------------------------------------------
def embedding(table, tokens, multiplier=1.0):
    """Row gather x[t] = E[tok[t]] (cpu_op.c:508-524); the multiplier is not in the reference."""
    return table[np.asarray(tokens, dtype=np.int64)] * multiplier


def rms_norm(x, w, eps):
    """ss = sum x^2; s = 1/sqrt(ss/n + eps); o = x*s*w  (cpu_op.c:44-64)."""
    ss = np.sum(x * x, axis=-1, keepdims=True)
    scale = 1.0 / np.sqrt(ss / x.shape[-1] + eps)
    return x * scale * w


def linear(x, w, b=None):
    """y[r] = sum_c W[r,c] x[c] (+ bias)  (cpu_op.c:121-189, 546-556); W is [out, in]."""
    y = x @ w.T
    if b is not None:
        y = y + b
    return y


def rope_neox(x, positions, n_heads, head_dim, rope_dim, theta):
    """Split-half rotary embedding (cpu_op.c:637-651).

    theta_i = 1/base^(2i/r); pairs (i, i+r/2) of the first r dims of each head;
    the angle is float32(pos) * float32(theta_i) as at cpu_op.c:644-646."""
    T = x.shape[0]
    x = x.reshape(T, n_heads, head_dim).copy()
    half = rope_dim // 2
    i = np.arange(half, dtype=np.float64)
    inv_freq = (1.0 / np.power(float(theta), 2.0 * i / rope_dim)).astype(np.float32)
    ang = (np.asarray(positions, dtype=np.float32)[:, None] * inv_freq[None, :]).astype(np.float32)
    ang = ang.astype(x.dtype)
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    a = x[..., :half].copy()
    b = x[..., half:rope_dim].copy()
    x[..., :half] = a * c - b * s
    x[..., half:rope_dim] = a * s + b * c
    return x.reshape(T, n_heads * head_dim)


def causal_attention(q, k, v, n_heads, n_kv, head_dim, window=0, rnd=_same):
    """Causal grouped-query attention of one whole sequence (cpu_op.c:1010-1062).

    kv head = h / (H/KV); keys 0..p inclusive; scale 1/sqrt(head_dim)
    (graph.c:1275); softmax with max subtraction (cpu_op.c:338-349); a window w
    keeps the last w keys including the current one (cpu_op.c:1019-1022).  rnd rounds the
    softmax numerators where they enter the product with the values (their sum is exact)."""
    T = q.shape[0]
    q = q.reshape(T, n_heads, head_dim)
    k = k.reshape(T, n_kv, head_dim)
    v = v.reshape(T, n_kv, head_dim)
    out = np.zeros_like(q)
    gqa = n_heads // n_kv
    scale = 1.0 / np.sqrt(float(head_dim))
    for h in range(n_heads):
        g = h // gqa
        for t in range(T):
            n_keys = t + 1
            start = n_keys - window if (window and n_keys > window) else 0
            s = (k[start:n_keys, g] @ q[t, h]) * scale
            e = np.exp(s - s.max())
            out[t, h] = (rnd(e) @ v[start:n_keys, g]) / e.sum()
    return out.reshape(T, n_heads * head_dim)


def mamba2_conv(xbc, w, b):
    """Causal depthwise convolution + SiLU with a zero initial window (cpu_op.c:836-889).

    w is [Cd, K]; tap K-1 multiplies the newest sample (cpu_op.c:870-874)."""
    T, Cd = xbc.shape
    K = w.shape[1]
    padded = np.concatenate([np.zeros((K - 1, Cd), dtype=xbc.dtype), xbc], axis=0)
    out = np.zeros_like(xbc)
    for k in range(K):
        out += padded[k:k + T] * w[:, k][None, :]
    if b is not None:
        out = out + b
    return silu(out)


def mamba2_scan(x, B, C, dt_raw, A, Dskip, dt_bias, Hs, P, G, N):
    """Sequential selective scan (cpu_op.c:924-951).

    dt = softplus(dt_raw + dt_bias); dA = exp(dt*A); S = S*dA + B*(x*dt);
    y = sum_n S*C (after the update) + x*D.  Returns y [T, Hs*P] before gating."""
    T = x.shape[0]
    x = x.reshape(T, Hs, P)
    B = B.reshape(T, G, N)
    C = C.reshape(T, G, N)
    S = np.zeros((Hs, P, N), dtype=x.dtype)
    y = np.zeros((T, Hs, P), dtype=x.dtype)
    hpg = Hs // G
    for t in range(T):
        dtv = softplus(dt_raw[t] + dt_bias)                    # [Hs]
        dA = np.exp(dtv * A)                                   # [Hs]
        for h in range(Hs):
            g = h // hpg
            xdt = x[t, h] * dtv[h]                             # [P]
            S[h] = S[h] * dA[h] + xdt[:, None] * B[t, g][None, :]
            y[t, h] = S[h] @ C[t, g] + x[t, h] * Dskip[h]
    return y.reshape(T, Hs * P)


def gated_norm(y, z, w, eps, G, rms_norm_on, norm_before_gate):
    """Gate then grouped RMSNorm (cpu_op.c:950-958).  norm-before-gate (norm y, then
    multiply by silu(z)) and the no-norm case are options not in the reference."""
    T, Di = y.shape
    if not rms_norm_on:
        return y * silu(z)
    gs = Di // G

    def grouped(v):
        v = v.reshape(T, G, gs)
        return rms_norm(v, w.reshape(G, gs)[None], eps).reshape(T, Di)

    if norm_before_gate:
        return grouped(y) * silu(z)
    return grouped(y * silu(z))


def attention_mixer(n, W, pre, cfg, d, positions, rnd=_same):
    """q/k/v projection, optional bias, RoPE, attention, output projection
    (falcon_h1.c:315-338).  key_multiplier scales k after its bias (not in the reference)."""
    q = linear(n, W[pre + "self_attn.q_proj.weight"], W.get(pre + "self_attn.q_proj.bias"))
    k = linear(n, W[pre + "self_attn.k_proj.weight"], W.get(pre + "self_attn.k_proj.bias"))
    v = linear(n, W[pre + "self_attn.v_proj.weight"], W.get(pre + "self_attn.v_proj.bias"))
    k = k * _get(cfg, "key_multiplier", 1.0)
    theta = _get(cfg, "rope_theta", 10000.0)                  # falcon_h1.c:126-128
    rope_dim = d["hd"]                                         # falcon_h1.c:265
    q = rnd(rope_neox(q, positions, d["H"], d["hd"], rope_dim, theta))
    k = rnd(rope_neox(k, positions, d["KV"], d["hd"], rope_dim, theta))
    o = causal_attention(q, k, rnd(v), d["H"], d["KV"], d["hd"], int(_get(cfg, "sliding_window", 0) or 0), rnd)
    return linear(rnd(o), W[pre + "self_attn.o_proj.weight"], W.get(pre + "self_attn.o_proj.bias"))


def mamba2_mixer(n, W, pre, cfg, d, rnd=_same, round_at_scale=1.0):
    """in_proj -> conv -> scan -> gate/norm -> out_proj (falcon_h1.c:342-368).

    round_at_scale: where a rounding function models a bfloat16 engine, the input of out_proj is
    rounded after a multiplication by this number, which is divided out again afterwards (the
    engine applies a part of the output multiplier in front of the product); exact arithmetic
    does not see it.

    The in_proj row order is z | x | B | C | dt (cpu_op.c:849, 865, 925-929).  The five
    ssm_multipliers scale those slices after the bias (not in the reference)."""
    Di, Cd, Hs, G, N = d["Di"], d["Cd"], d["Hs"], d["G"], d["N"]
    proj = linear(n, W[pre + "mamba.in_proj.weight"], W.get(pre + "mamba.in_proj.bias"))
    m = _get(cfg, "ssm_multipliers", [1.0] * 5)
    mup = np.concatenate([np.full(Di, m[0]), np.full(Di, m[1]), np.full(G * N, m[2]),
                          np.full(G * N, m[3]), np.full(Hs, m[4])])
    proj = proj * mup
    z, xbc, dt = proj[:, :Di], proj[:, Di:Di + Cd], proj[:, Di + Cd:]
    cw = W[pre + "mamba.conv1d.weight"].reshape(Cd, -1)
    cv = rnd(mamba2_conv(xbc, cw, W.get(pre + "mamba.conv1d.bias")))      # the scan's operands
    x, B, C = cv[:, :Di], cv[:, Di:Di + G * N], cv[:, Di + G * N:]
    A = -np.exp(W[pre + "mamba.A_log"].astype(n.dtype))       # cpu_op.c:806-808, 934
    y = mamba2_scan(x, B, C, dt, A, W[pre + "mamba.D"], W[pre + "mamba.dt_bias"],
                    Hs, d["P"], G, N)
    y = gated_norm(y, z, W.get(pre + "mamba.norm.weight"), cfg["rms_norm_eps"], G,
                   bool(_get(cfg, "mamba_rms_norm", True)) and (pre + "mamba.norm.weight") in W,
                   bool(_get(cfg, "mamba_norm_before_gate", False)))
    if rnd is not _same and round_at_scale != 1.0:
        y = rnd(y * round_at_scale) / round_at_scale
    return linear(rnd(y) if rnd is _same or round_at_scale == 1.0 else y, W[pre + "mamba.out_proj.weight"],
                  W.get(pre + "mamba.out_proj.bias"))


def swiglu_mlp(hn, W, pre, cfg, rnd=_same):
    """down(silu(gate(x)) * up(x)) (falcon_h1.c:382-395); mlp_multipliers = [gate, down]
    scale the gate pre-activation and the down output (not in the reference)."""
    mg, md = _get(cfg, "mlp_multipliers", [1.0, 1.0])
    g = linear(hn, W[pre + "feed_forward.gate_proj.weight"], W.get(pre + "feed_forward.gate_proj.bias"))
    u = linear(hn, W[pre + "feed_forward.up_proj.weight"], W.get(pre + "feed_forward.up_proj.bias"))
    a = rnd(silu(g * mg) * u)
    return linear(a, W[pre + "feed_forward.down_proj.weight"], W.get(pre + "feed_forward.down_proj.bias")) * md


def block(x, W, layer, cfg, d, positions, rnd=_same):
    """x = (x + attn(n)) + ssm(n); x = x + mlp(norm(x))  (falcon_h1.c:311-395)."""
    pre = f"model.layers.{layer}."
    eps = cfg["rms_norm_eps"]
    n = rnd(rms_norm(x, W[pre + "input_layernorm.weight"], eps))
    a = attention_mixer(n * _get(cfg, "attention_in_multiplier", 1.0), W, pre, cfg, d, positions, rnd)
    a = a * _get(cfg, "attention_out_multiplier", 1.0)
    # An engine that runs o_proj and out_proj as one product has one output scale for both, the attention's,
    # and multiplies the Mamba activations by the ratio of the two before they are rounded; it does so where
    # both input widths are multiples of 8.
    a_out, m_out = _get(cfg, "attention_out_multiplier", 1.0), _get(cfg, "ssm_out_multiplier", 1.0)
    ratio = m_out / a_out if a_out != 0 and (d["H"] * d["hd"]) % 8 == 0 and d["Di"] % 8 == 0 else 1.0
    m = mamba2_mixer(n * _get(cfg, "ssm_in_multiplier", 1.0), W, pre, cfg, d, rnd, ratio)
    m = m * m_out
    x = (x + a) + m                                            # falcon_h1.c:372-375
    hn = rnd(rms_norm(x, W[pre + "pre_ff_layernorm.weight"], eps))
    return x + swiglu_mlp(hn, W, pre, cfg, rnd)


def forward(cfg: dict, weights: dict, tokens, dtype=np.float64, rnd=_same) -> np.ndarray:
    """Logits [T, V] of one whole sequence starting at position 0 (falcon_h1.c:256-417).
    rnd: identity, or bf16_round to model a bfloat16 engine (see bf16_round)."""
    W = {k: np.asarray(v).astype(dtype) for k, v in weights.items()}
    d = derived(cfg)
    T = len(tokens)
    positions = np.arange(T)
    x = embedding(W["model.embed_tokens.weight"], tokens, _get(cfg, "embedding_multiplier", 1.0))
    for layer in range(d["L"]):
        x = block(x, W, layer, cfg, d, positions, rnd)
    f = rnd(rms_norm(x, W["model.final_layernorm.weight"], cfg["rms_norm_eps"]))
    head = W["model.embed_tokens.weight"] if _get(cfg, "tie_word_embeddings", False) \
        else W["lm_head.weight"]                               # core.c:1246-1249
    return linear(f, head) * _get(cfg, "lm_head_multiplier", 1.0)


# --------------------------------------------------------------------------
# sampling
# --------------------------------------------------------------------------
def apply_penalties(logits, history, repeat_penalty=1.0, repeat_last_n=64,
                    frequency_penalty=0.0, presence_penalty=0.0):
    """Repeat / frequency / presence penalties, once per unique token of the last
    repeat_last_n history tokens (sampler.c:116-144)."""
    logits = np.array(logits, dtype=np.float64)
    if (repeat_penalty == 1.0 and frequency_penalty == 0.0 and presence_penalty == 0.0) \
            or repeat_last_n <= 0 or len(history) == 0:
        return logits
    win = list(history)[-repeat_last_n:]
    for tid in dict.fromkeys(win):
        if tid >= len(logits):
            continue
        count = win.count(tid)
        logits[tid] = logits[tid] * repeat_penalty if logits[tid] <= 0 else logits[tid] / repeat_penalty
        logits[tid] -= count * frequency_penalty + presence_penalty
    return logits


def greedy(logits) -> int:
    """First maximum (sampler.c:92-102)."""
    return int(np.argmax(logits))


def filtered_distribution(logits, temperature, top_k=0, top_p=1.0, min_p=0.0):
    """softmax(logits/T) then top-k, min-p, top-p, renormalise (sampler.c:156-239).
    Returns (token ids by descending probability, probabilities)."""
    z = np.asarray(logits, dtype=np.float64) / temperature
    p = np.exp(z - z.max())
    p /= p.sum()
    order = np.argsort(-p, kind="stable")
    if top_k > 0:
        order = order[:top_k]
    probs = p[order]
    cutoff = len(order)
    if min_p > 1e-6:
        keep = probs >= min_p * probs[0]
        nc = int(np.argmin(keep)) if not keep.all() else len(keep)
        if nc > 0:
            cutoff = nc
    if top_p < 1.0:
        cum = np.cumsum(probs[:cutoff])
        idx = int(np.searchsorted(cum, top_p, side="left"))
        if idx + 1 < cutoff:
            cutoff = idx + 1
    cutoff = max(cutoff, 1)
    probs = probs[:cutoff] / probs[:cutoff].sum()
    return order[:cutoff], probs
