"""Plain, slow float64 statement of the Lepalorn design, one function per mechanism (numpy only; test infrastructure,
never imported by the product).  It works on a whole sequence at once, without any cache: whatever schedule the
product runs (portions, single tokens, rings), its logits must equal these.

Checkpoint names: ``embed``, ``head``, ``final.norm``, and per layer i ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.dwa``,
``l<i>.mix.{q,g,dkv,dkv.norm,uk,uv,o}``, ``l<i>.mlp.{router,router.b,e<k>.gate,e<k>.up,e<k>.down,shared.gate,shared.up,
shared.down,shared.sg}``; Linear weights are [out, in].
"""
import numpy as np


def rms(x, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def rotate_pairs(x, pos, base, dims):
    """x [..., T, D]; the pair (x[2i], x[2i+1]), i < dims/2, turns by pos * base^(-2i/dims); the rest passes."""
    y = np.array(x, dtype=np.float64, copy=True)
    for i in range(dims // 2):
        a = np.asarray(pos, dtype=np.float64) * float(base) ** (-2.0 * i / dims)
        u, v = x[..., 2 * i], x[..., 2 * i + 1]
        y[..., 2 * i] = u * np.cos(a) - v * np.sin(a)
        y[..., 2 * i + 1] = v * np.cos(a) + u * np.sin(a)
    return y


def latent_rows(h, w_dkv, w_norm, kv_rank, pos, base, dims, eps):
    """The per-token rows a layer would cache: (c [T, kv_rank], k_rot [T, rot_dim])."""
    d = h @ w_dkv.T
    return rms(d[:, :kv_rank], eps) * w_norm, rotate_pairs(d[:, kv_rank:], pos, base, dims)


def window_softmax(scores, window):
    """scores [T, T] (query, key) -> weights; key j is visible to query i when 0 <= i - j < window (None: j <= i)."""
    T = scores.shape[0]
    out = np.zeros_like(scores)
    for i in range(T):
        lo = 0 if window is None else max(0, i - window + 1)
        s = scores[i, lo:i + 1]
        e = np.exp(s - s.max())
        out[i, lo:i + 1] = e / e.sum()
    return out


def latent_attention(h, W, p, m, eps, rows_of):
    """The mixer of one layer.  ``m`` is the layer's mixer config, ``rows_of`` maps a layer index to its (c, k_rot)."""
    T = h.shape[0]
    H, D, R, V = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    pos = np.arange(T)
    base, dims = m["rot"]["base"], m["rot"]["dims"]
    q = (h @ W[p + "q"].T).reshape(T, H, D + R)
    if m.get("kv_from") is not None:
        c, k_rot = rows_of[m["kv_from"]]
    else:
        c, k_rot = latent_rows(h, W[p + "dkv"], W[p + "dkv.norm"], m["kv_rank"], pos, base, dims, eps)
    k = (c @ W[p + "uk"].T).reshape(T, H, D)
    v = (c @ W[p + "uv"].T).reshape(T, H, V)
    gate = 1.0 / (1.0 + np.exp(-(h @ W[p + "g"].T)))
    window = (m.get("mask") or {}).get("size")
    heads = []
    for a in range(H):
        q_rot = rotate_pairs(q[:, a, D:], pos, base, dims)
        s = (q[:, a, :D] @ k[:, a].T + q_rot @ k_rot.T) * m["scale"]
        heads.append(window_softmax(s, window) @ v[:, a] * gate[:, a:a + 1])
    return np.concatenate(heads, axis=-1) @ W[p + "o"].T, (c, k_rot)


def glu_expert(h, gate, up, down, limit, alpha=1.702):
    g = np.minimum(h @ gate.T, limit)
    u = np.clip(h @ up.T, -limit, limit)
    return (g / (1.0 + np.exp(-alpha * g)) * (u + 1.0)) @ down.T


def route(h, w_router, bias, top):
    """(chosen experts [T, top], weights [T, top]): the largest logits, softmax over the chosen ones."""
    z = h @ w_router.T + (bias if bias is not None else 0.0)
    idx = np.argsort(-z, axis=-1, kind="stable")[:, :top]
    zc = np.take_along_axis(z, idx, axis=-1)
    e = np.exp(zc - zc.max(axis=-1, keepdims=True))
    return idx, e / e.sum(axis=-1, keepdims=True)


def moe(h, W, p, f):
    idx, w = route(h, W[p + "router"], W.get(p + "router.b"), f["router"]["top"])
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for k in range(idx.shape[1]):
            e = int(idx[t, k])
            out[t] += w[t, k] * glu_expert(h[t:t + 1], W[p + f"e{e}.gate"], W[p + f"e{e}.up"], W[p + f"e{e}.down"],
                                           f["expert"]["limit"])[0]
    if f.get("shared"):
        y = glu_expert(h, W[p + "shared.gate"], W[p + "shared.up"], W[p + "shared.down"], f["shared"]["limit"])
        if p + "shared.sg" in W:
            y = y / (1.0 + np.exp(-(h @ W[p + "shared.sg"].reshape(1, -1).T)))
        out += y
    return out


def forward(cfg, W, tokens, return_layers=False):
    """Logits [T, vocab] of one sequence (float64), optionally the stream after every layer as the next layer reads it."""
    W = {k: np.asarray(v, dtype=np.float64) for k, v in W.items()}
    eps = cfg["norm"]["eps"]
    x = W["embed"][np.asarray(tokens)] * cfg["embedding"]["scale"]
    outs, rows_of, streams = [x], {}, []
    for i, layer in enumerate(cfg["layers"]):
        y, rows = latent_attention(x, W, f"l{i}.mix.", layer["mixer"], eps, rows_of)
        if layer["mixer"].get("kv_from") is None:
            rows_of[i] = rows
        x = x + rms(y, eps) * W[f"l{i}.norm1"]
        if layer.get("mlp") is not None:
            x = x + rms(moe(x, W, f"l{i}.mlp.", layer["mlp"]), eps) * W[f"l{i}.norm2"]
        outs.append(x)
        x = sum(W[f"l{i}.dwa"][j] * outs[j] for j in range(i + 2))
        streams.append(x)
    logits = (rms(x, eps) * W["final.norm"]) @ W["head"].T
    return (logits, streams) if return_layers else logits


def greedy(cfg, W, tokens, n_new):
    toks = list(tokens)
    for _ in range(n_new):
        toks.append(int(np.argmax(forward(cfg, W, toks)[-1])))
    return toks


# ------------------------------------------------------------------ random models for the tests
def bf16_round(a):
    """Round float32 values to the nearest bfloat16 (ties to even), returned as float32."""
    u = np.asarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    u = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    return u.astype(np.uint32).view(np.float32)


def mixer_cfg(heads, dim, rot_dim, vdim, kv_rank, window, base=10000.0, rot_dims=None, scale=None, kv_from=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "mask": {"size": window},
         "rot": {"base": base, "dims": rot_dim if rot_dims is None else rot_dims},
         "scale": float(scale if scale is not None else (dim + rot_dim) ** -0.5)}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def mlp_cfg(experts, top, ff, limit, shared_ff=None, shared_limit=None):
    f = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff, "limit": limit}}
    if shared_ff:
        f["shared"] = {"ff": shared_ff, "limit": shared_limit if shared_limit is not None else limit}
    return f


def model_cfg(vocab, width, layers, eps=1e-5, embedding_scale=1.0):
    return {"architecture": "Lepalorn", "vocab": vocab, "width": width, "norm": {"eps": eps},
            "embedding": {"scale": embedding_scale},
            "layers": [{"type": "latent_attention", "mixer": m, "mlp": f} for m, f in layers]}


def random_weights(cfg, seed=0, shared_gate=True, gain=1.0):
    """bf16-representable float32 weights with O(1) activations everywhere (so that every branch matters)."""
    r = np.random.RandomState(seed)
    E, W = cfg["width"], {}

    def lin(o, i, g=1.0):
        return bf16_round(r.randn(o, i) * g / np.sqrt(i))

    W["embed"] = bf16_round(r.randn(cfg["vocab"], E))
    W["head"] = lin(cfg["vocab"], E)
    W["final.norm"] = bf16_round(np.array(1.0 + 0.2 * r.randn()))
    for i, layer in enumerate(cfg["layers"]):
        m, p = layer["mixer"], f"l{i}.mix."
        H, D, R, V, K = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
        W[p + "q"] = lin(H * (D + R), E, 2.0 * gain)
        W[p + "g"] = lin(H, E, 2.0)
        if m.get("kv_from") is None:
            W[p + "dkv"] = lin(K + R, E, 2.0 * gain)
            W[p + "dkv.norm"] = bf16_round(1.0 + 0.3 * r.randn(K))
        W[p + "uk"] = lin(H * D, K, 2.0)
        W[p + "uv"] = lin(H * V, K)
        W[p + "o"] = lin(E, H * V)
        W[f"l{i}.norm1"] = bf16_round(np.array(0.7 + 0.2 * r.rand()))
        if layer.get("mlp") is not None:
            f, q = layer["mlp"], f"l{i}.mlp."
            X, F = f["router"]["experts"], f["expert"]["ff"]
            W[q + "router"] = lin(X, E, 3.0)
            W[q + "router.b"] = bf16_round(0.5 * r.randn(X))
            for e in range(X):
                W[q + f"e{e}.gate"] = lin(F, E, 1.5)
                W[q + f"e{e}.up"] = lin(F, E, 1.5)
                W[q + f"e{e}.down"] = lin(E, F)
            if f.get("shared"):
                S = f["shared"]["ff"]
                W[q + "shared.gate"] = lin(S, E, 1.5)
                W[q + "shared.up"] = lin(S, E, 1.5)
                W[q + "shared.down"] = lin(E, S)
                if shared_gate:
                    W[q + "shared.sg"] = lin(1, E, 2.0)
            W[f"l{i}.norm2"] = bf16_round(np.array(0.7 + 0.2 * r.rand()))
        W[f"l{i}.dwa"] = bf16_round(np.concatenate([0.3 * r.randn(i + 1) / (i + 1), [1.0 + 0.1 * r.randn()]]))
    return W
