"""Plain, slow float64 statement of the Bededra design, one function per mechanism (numpy only; test infrastructure,
never imported by the product).  It works on a whole sequence at once and keeps no cache: whatever schedule the product
runs (portions, single tokens, rings, recurrent state handed from step to step), its logits must equal these.

A layer reads the stream x through two norms and adds both branches to the same x:

    x <- x + mixer(h1 + shortconv(h1)) + ff(h2),      h1 = rmsnorm(x) * w1,   h2 = rmsnorm(x) * w2

Mixers: ``mamba2`` (selective state space with a scalar decay per head) and ``parallel`` (softmax attention over a
sliding window plus kept first tokens, beside gated linear attention; their outputs are added with fixed scales).
Feed-forwards: dense (squared relu) or a mixture of gated experts chosen among the best groups of experts.

Checkpoint names: ``embed``, ``head``, ``final.norm``; per layer i ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.canon1``,
``l<i>.mix.*``, ``l<i>.mlp.*``; Linear weights are [out, in].
"""
import numpy as np


def rms(x, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, z)


def short_conv(h, w, bias=None):
    """Causal convolution over time, channel by channel.  h [T, C], w [C, taps]; the LAST tap weighs the current token,
    inputs before the sequence's start are zero."""
    T, C = h.shape
    taps = w.shape[1]
    out = np.zeros((T, C))
    for t in range(T):
        for j in range(taps):
            s = t - (taps - 1) + j
            if s >= 0:
                out[t] += w[:, j] * h[s]
    if bias is not None:
        out += bias
    return out


def mamba2(h, W, p, m, eps):
    """Selective state space mixer.  W_in h = [z | x | B | C | dt]; x, B, C pass a short convolution (with bias) and silu;
    per head S_t = exp(-exp(A_log) dt_t) S_(t-1) + dt_t B_t x_t^T, y_t = S_t^T C_t + D x_t; then y * silu(z), RMS norm in
    ``norm_groups`` equal parts times a weight, and the output projection."""
    T = h.shape[0]
    H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * P
    u = h @ W[p + "in"].T
    z, xbc, dt = u[:, :inner], u[:, inner:2 * inner + 2 * G * N], u[:, 2 * inner + 2 * G * N:]
    xbc = silu(short_conv(xbc, W[p + "conv"], W[p + "conv.b"]))
    x = xbc[:, :inner].reshape(T, H, P)
    Bm = xbc[:, inner:inner + G * N].reshape(T, G, N)
    Cm = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = softplus(dt + W[p + "dt_bias"])
    decay = np.exp(-np.exp(W[p + "A_log"]) * dt)           # [T, H]
    y = np.zeros((T, H, P))
    for hd in range(H):
        g = hd // (H // G)
        S = np.zeros((N, P))
        for t in range(T):
            S = decay[t, hd] * S + dt[t, hd] * np.outer(Bm[t, g], x[t, hd])
            y[t, hd] = S.T @ Cm[t, g] + W[p + "D"][hd] * x[t, hd]
    y = y.reshape(T, inner) * silu(z)
    ng = m["norm_groups"]
    y = rms(y.reshape(T, ng, inner // ng), eps).reshape(T, inner) * W[p + "norm"]
    return y @ W[p + "o"].T


def visible(i, j, window, keep_first):
    return j <= i and (i - j < window or j < keep_first)


def attention_core(q, k, v, gate_logits, r1, r2, talk, scale, cap, window, keep):
    """q [T, H, D], k [T, G, D], v [T, G, V], gate_logits [T, H] (or None) -> [T, H, V].  cap 0: no cap; window None: all."""
    T, H, _ = q.shape
    G, V = k.shape[1], v.shape[2]
    window = T + 1 if window is None else window
    weights = np.zeros((H, T, T))
    for hd in range(H):
        g = hd // (H // G)
        s = q[:, hd] @ k[:, g].T * scale
        if cap:
            s = cap * np.tanh(s / cap)
        for i in range(T):
            js = [j for j in range(i + 1) if visible(i, j, window, keep)]
            row = np.array([s[i, j] - r1[hd] * np.log1p(r2[hd] * (i - j)) for j in js])
            e = np.exp(row - row.max())
            weights[hd, i, js] = e / e.sum()
    mixed = np.einsum("hg,gij->hij", talk, weights)
    out = np.zeros((T, H, V))
    for hd in range(H):
        out[:, hd] = mixed[hd] @ v[:, hd // (H // G)]
    if gate_logits is not None:
        out = out * sigmoid(gate_logits)[:, :, None]
    return out


def window_attention(h, W, p, m):
    """Softmax attention with grouped key/value heads and no rotation: score = softcap * tanh(q.k * scale / softcap)
    - r1 * ln(1 + r2 * (i - j)); sliding window plus the first ``keep_first`` tokens; the heads' softmax weights are mixed
    by a [H, H] matrix before they meet the values; each head's output is gated by sigmoid of one number per head."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ W[p + "q"].T).reshape(T, H, D)
    k = (h @ W[p + "k"].T).reshape(T, G, D)
    v = (h @ W[p + "v"].T).reshape(T, G, V)
    mask = m.get("mask") or {}
    out = attention_core(q, k, v, h @ W[p + "g"].T, W[p + "r1"], W[p + "r2"], W[p + "talk"], m["scale"], m.get("softcap") or 0.0,
                         mask.get("size"), mask.get("keep_first") or 0)
    return out.reshape(T, H * V) @ W[p + "o"].T


def linear_recurrence(q, k, v, a, kscale=None, skip=None, qscale=1.0):
    """S_t = diag(a_t) S_(t-1) + (kscale_t k_t) v_t^T;  y_t = qscale S_t^T q_t + skip * v_t.
    q, k [T, n]; v [T, p]; a [T, n] or [T] (one decay for all rows); kscale [T] or None; skip a number or None."""
    T, n = k.shape
    S = np.zeros((n, v.shape[1]))
    y = np.zeros((T, v.shape[1]))
    for t in range(T):
        at = a[t] if np.ndim(a[t]) else np.full(n, a[t])
        S = at[:, None] * S + np.outer(k[t] * (1.0 if kscale is None else kscale[t]), v[t])
        y[t] = qscale * (S.T @ q[t]) + (0.0 if skip is None else skip * v[t])
    return y


def gated_linear_attention(h, W, p, m, eps):
    """Linear attention with a decay per key channel: alpha = sigmoid(W_a2 W_a1 h + b)^(1/tau);
    S_t = diag(alpha_t) S_(t-1) + k_t v_t^T, o_t = S_t^T q_t with q scaled by dim^-1/2; each head's o is RMS-normed over
    its value size with one shared weight, the heads are gated by silu(W_g h) and projected."""
    T = h.shape[0]
    H, D, V = m["heads"], m["dim"], m["vdim"]
    q = (h @ W[p + "q"].T).reshape(T, H, D) * D ** -0.5
    k = (h @ W[p + "k"].T).reshape(T, H, D)
    v = (h @ W[p + "v"].T).reshape(T, H, V)
    zz = (h @ W[p + "a1"].T) @ W[p + "a2"].T + W[p + "a2.b"]
    alpha = (sigmoid(zz) ** (1.0 / m["tau"])).reshape(T, H, D)
    o = np.zeros((T, H, V))
    for hd in range(H):
        S = np.zeros((D, V))
        for t in range(T):
            S = alpha[t, hd][:, None] * S + np.outer(k[t, hd], v[t, hd])
            o[t, hd] = S.T @ q[t, hd]
    o = rms(o, eps) * W[p + "norm"]
    o = o.reshape(T, H * V) * silu(h @ W[p + "g"].T)
    return o @ W[p + "o"].T


def parallel_mixer(h, W, p, m, eps):
    return m["left_scale"] * window_attention(h, W, p + "left.", m["left"]) \
        + m["right_scale"] * gated_linear_attention(h, W, p + "right.", m["right"], eps)


def dense_ff(h, W, p):
    return np.maximum(h @ W[p + "up"].T, 0.0) ** 2 @ W[p + "down"].T


def route(h, w_router, top, n_groups, keep_groups):
    """Scores = softmax over all experts; experts outside the ``keep_groups`` best groups (a group's score is its largest)
    cannot be chosen; weights = chosen scores / (their sum + 1e-20).  Returns (indices [T, top], weights [T, top])."""
    z = h @ w_router.T
    e = np.exp(z - z.max(axis=-1, keepdims=True))
    s = e / e.sum(axis=-1, keepdims=True)
    T, X = s.shape
    idx = np.zeros((T, top), dtype=np.int64)
    wts = np.zeros((T, top))
    for t in range(T):
        gs = s[t].reshape(n_groups, X // n_groups).max(axis=1)
        best = np.argsort(-gs, kind="stable")[:keep_groups]
        allowed = np.full(X, -np.inf)
        for g in best:
            lo = g * (X // n_groups)
            allowed[lo:lo + X // n_groups] = s[t, lo:lo + X // n_groups]
        chosen = np.argsort(-allowed, kind="stable")[:top]
        idx[t] = chosen
        wts[t] = s[t, chosen] / (s[t, chosen].sum() + 1e-20)
    return idx, wts


def moe_ff(h, W, p, f):
    r = f["router"]
    groups = r.get("groups") or {}
    idx, wts = route(h, W[p + "router"], r["top"], groups.get("count", 1), groups.get("keep", groups.get("count", 1)))
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e, w in zip(idx[t], wts[t]):
            q = f"{p}e{e}."
            out[t] += w * ((silu(W[q + "gate"] @ h[t]) * (W[q + "up"] @ h[t])) @ W[q + "down"].T)
    return out


def forward(cfg, W, tokens, return_layers=False):
    """Logits [T, vocab] of one sequence (and the stream after every layer, [L, T, width])."""
    W = {k: np.asarray(v, dtype=np.float64) for k, v in W.items()}
    eps = cfg["norm"]["eps"]
    x = W["embed"][np.asarray(tokens)]
    streams = []
    for i, lc in enumerate(cfg["layers"]):
        p = f"l{i}."
        n = rms(x, eps)
        h = n * W[p + "norm1"]
        h = h + short_conv(h, W[p + "canon1"])
        if lc["type"] == "mamba2":
            y = mamba2(h, W, p + "mix.", lc["mixer"], eps)
        elif lc["type"] == "parallel":
            y = parallel_mixer(h, W, p + "mix.", lc["mixer"], eps)
        else:
            raise ValueError(lc["type"])
        f = lc.get("mlp")
        if f is not None:
            h2 = n * W[p + "norm2"]
            y = y + (dense_ff(h2, W, p + "mlp.") if f["kind"] == "dense" else moe_ff(h2, W, p + "mlp.", f))
        x = x + y
        streams.append(x)
    logits = (rms(x, eps) * W["final.norm"]) @ W["head"].T
    return (logits, np.stack(streams)) if return_layers else logits
