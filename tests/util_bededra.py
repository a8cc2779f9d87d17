"""Builders shared by the Bededra tests: small random models written as model folders (config.json + safetensors) and
loaded back through the package's registry, and comparisons against the float64 oracle (oracle/bededra.py)."""
import json

import numpy as np
import torch

from oracle import bededra as O


def bf16(a):
    """Round to bfloat16 (what the model folder stores), as float64."""
    return torch.from_numpy(np.asarray(a, dtype=np.float32)).to(torch.bfloat16).double().numpy()


def parallel(heads, kv_heads, dim, vdim, window, keep, r_heads, r_dim, r_vdim, tau=8.0, softcap=30.0, ls=0.7, rs=1.3, rank=6):
    return {"type": "parallel", "_rank": rank, "mixer": {
        "left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": dim ** -0.5, "softcap": softcap,
                 "mask": {"size": window, "keep_first": keep}},
        "right": {"heads": r_heads, "dim": r_dim, "vdim": r_vdim, "tau": tau}, "left_scale": ls, "right_scale": rs}}


def mamba(heads, vdim, state, groups=1, norm_groups=1, conv=4):
    return {"type": "mamba2", "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "norm_groups": norm_groups,
                                        "conv": conv}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, count=1, keep=1):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "groups": {"count": count, "keep": keep}}}


def model_cfg(vocab, width, layers, eps=1e-5, taps=4):
    """``layers``: (mixer entry from parallel() / mamba(), feed-forward entry or None)."""
    return {"architecture": "Bededra", "vocab": vocab, "width": width, "norm": {"eps": eps}, "canon": {"taps": taps},
            "layers": [dict(m, mlp=f) for m, f in layers]}


def random_weights(cfg, seed=0):
    """Every tensor of the design with values that keep activations of order one; already rounded to bfloat16."""
    r = np.random.RandomState(seed)
    E, W = cfg["width"], {}

    def lin(o, i, gain=1.0):
        return r.randn(o, i) * gain / np.sqrt(i)

    W["embed"] = r.randn(cfg["vocab"], E)
    W["head"] = lin(cfg["vocab"], E)
    W["final.norm"] = 1 + 0.1 * r.randn(E)
    for i, lc in enumerate(cfg["layers"]):
        p, m = f"l{i}.", lc["mixer"]
        W[p + "norm1"] = 1 + 0.1 * r.randn(E)
        W[p + "canon1"] = 0.4 * r.randn(E, cfg["canon"]["taps"])
        if lc["type"] == "mamba2":
            H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
            ch = H * P + 2 * G * N
            W[p + "mix.in"] = lin(2 * H * P + 2 * G * N + H, E)
            W[p + "mix.conv"] = 0.5 * r.randn(ch, m["conv"])
            W[p + "mix.conv.b"] = 0.2 * r.randn(ch)
            W[p + "mix.dt_bias"] = r.uniform(-2.0, 0.5, H)
            W[p + "mix.A_log"] = r.uniform(-1.0, 1.0, H)
            W[p + "mix.D"] = r.randn(H)
            W[p + "mix.norm"] = 1 + 0.1 * r.randn(H * P)
            W[p + "mix.o"] = lin(E, H * P)
        else:
            l, rt = m["left"], m["right"]
            H, G, D, V = l["heads"], l["kv_heads"], l["dim"], l["vdim"]
            W[p + "mix.left.q"] = lin(H * D, E, 2.0)
            W[p + "mix.left.k"] = lin(G * D, E, 2.0)
            W[p + "mix.left.v"] = lin(G * V, E)
            W[p + "mix.left.g"] = lin(H, E)
            W[p + "mix.left.r1"] = r.uniform(0.0, 0.6, H)
            W[p + "mix.left.r2"] = r.uniform(0.1, 2.0, H)
            W[p + "mix.left.talk"] = np.eye(H) + 0.3 * r.randn(H, H)
            W[p + "mix.left.o"] = lin(E, H * V)
            H, D, V, rank = rt["heads"], rt["dim"], rt["vdim"], lc.get("_rank", 6)
            W[p + "mix.right.q"] = lin(H * D, E)
            W[p + "mix.right.k"] = lin(H * D, E)
            W[p + "mix.right.v"] = lin(H * V, E)
            W[p + "mix.right.g"] = lin(H * V, E)
            W[p + "mix.right.a1"] = lin(rank, E)
            W[p + "mix.right.a2"] = lin(H * D, rank)
            W[p + "mix.right.a2.b"] = r.uniform(0.0, 3.0, H * D)
            W[p + "mix.right.norm"] = 1 + 0.1 * r.randn(V)
            W[p + "mix.right.o"] = lin(E, H * V)
        f = lc.get("mlp")
        if f is not None:
            W[p + "norm2"] = 1 + 0.1 * r.randn(E)
            if f["kind"] == "dense":
                W[p + "mlp.up"] = lin(f["ff"], E)
                W[p + "mlp.down"] = lin(E, f["ff"])
            else:
                W[p + "mlp.router"] = lin(f["router"]["experts"], E, 3.0)
                for e in range(f["router"]["experts"]):
                    W[p + f"mlp.e{e}.gate"] = lin(f["expert"]["ff"], E)
                    W[p + f"mlp.e{e}.up"] = lin(f["expert"]["ff"], E)
                    W[p + f"mlp.e{e}.down"] = lin(E, f["expert"]["ff"])
    return {k: bf16(v) for k, v in W.items()}


def file_cfg(cfg):
    """The dictionary as a config.json holds it (builder-only keys removed)."""
    out = json.loads(json.dumps(cfg))
    for lc in out["layers"]:
        lc.pop("_rank", None)
    return out


def case_mixed(seed=0):
    """Sizes that share nothing with each other, both mixers in an order of its own, every kind of feed-forward and none."""
    layers = [
        (mamba(3, 8, 10, groups=1, norm_groups=3, conv=3), moe(6, 2, 12, count=3, keep=2)),
        (parallel(6, 2, 12, 20, window=7, keep=3, r_heads=2, r_dim=10, r_vdim=12, tau=5.0, rank=5), dense(40)),
        (parallel(4, 4, 8, 8, window=5, keep=0, r_heads=3, r_dim=20, r_vdim=4, tau=12.0, softcap=8.0, ls=1.2, rs=0.4), None),
        (mamba(4, 6, 20, groups=2, norm_groups=1, conv=2), dense(24)),
        (parallel(2, 1, 16, 12, window=11, keep=2, r_heads=1, r_dim=12, r_vdim=20), moe(8, 3, 10, count=4, keep=2)),
    ]
    cfg = model_cfg(53, 48, layers, eps=1e-4, taps=4)
    return cfg, random_weights(cfg, seed)


def case_ones(seed=1):
    """Sizes that are 1 or equal where a real model's differ: one head, one group, one expert, window 1, one tap in the
    inner convolution, a window longer than any test sequence, no kept tokens and more kept tokens than the window."""
    layers = [
        (parallel(1, 1, 8, 8, window=1, keep=0, r_heads=1, r_dim=8, r_vdim=8, rank=1), moe(1, 1, 8)),
        (mamba(1, 8, 8, conv=1), moe(4, 4, 8, count=2, keep=2)),
        (parallel(2, 2, 4, 4, window=1000, keep=0, r_heads=2, r_dim=4, r_vdim=4, softcap=0.0), moe(4, 2, 8, count=1, keep=1)),
        (parallel(2, 1, 4, 4, window=2, keep=5, r_heads=2, r_dim=4, r_vdim=4), None),
    ]
    cfg = model_cfg(19, 8, layers, eps=1e-6, taps=2)
    return cfg, random_weights(cfg, seed)


def case_odd(seed=2):
    """Nothing is a multiple of 4: every kernel takes its padded / unaligned path."""
    layers = [
        (parallel(3, 3, 5, 7, window=6, keep=1, r_heads=3, r_dim=7, r_vdim=5, rank=3), moe(9, 2, 11, count=3, keep=1)),
        (mamba(5, 3, 7, groups=5, norm_groups=5, conv=5), dense(13)),
    ]
    cfg = model_cfg(37, 30, layers, eps=1e-6, taps=3)
    return cfg, random_weights(cfg, seed)


def case_one_kind(kind, seed=3):
    """Models with a single kind of mixer (no key/value rows at all, or no state-space layer), unbounded window."""
    if kind == "mamba2":
        layers = [(mamba(2, 8, 12, groups=2, norm_groups=2), dense(20)), (mamba(4, 4, 6), None)]
    else:
        p1 = parallel(2, 2, 16, 16, window=9, keep=4, r_heads=2, r_dim=8, r_vdim=8)
        p2 = parallel(4, 1, 8, 8, window=9, keep=0, r_heads=1, r_dim=16, r_vdim=16, softcap=0.0)
        p2["mixer"]["left"]["mask"] = {}                      # no window, nothing kept: every earlier token is visible
        layers = [(p1, moe(4, 2, 8, count=2, keep=1)), (p2, dense(16))]
    cfg = model_cfg(29, 24, layers, eps=1e-5, taps=4)
    return cfg, random_weights(cfg, seed)


def write_model(folder, cfg, W):
    from lit_llama.safetensors_io import save_safetensors

    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(file_cfg(cfg)))
    save_safetensors({k: torch.from_numpy(np.asarray(v, dtype=np.float32)).to(torch.bfloat16) for k, v in W.items()},
                     folder / "model.safetensors")
    return folder


def load(folder, dtype, **attrs):
    from lit_llama.registry import load_model_dir

    m = load_model_dir(folder, dtype=dtype, device="cuda")
    for k, v in attrs.items():
        setattr(m, k, v)
    return m


def run_schedule(model, tokens, portions, max_tokens):
    """Feed ``tokens`` [B, T] (or a list for one sequence) in portions; returns fp32 logits [B, T, vocab] on the host."""
    idx = torch.as_tensor(tokens, dtype=torch.int64, device="cuda")
    if idx.dim() == 1:
        idx = idx[None]
    assert sum(portions) == idx.shape[1]
    model.reset_cache()
    out, at = [], 0
    for n in portions:
        out.append(model(idx[:, at:at + n], max_tokens, torch.arange(at, at + n)))
        at += n
    return torch.cat(out, dim=1).double().cpu().numpy()


def rel_err(got, want):
    return float(np.abs(got - want).max() / np.abs(want).max())


def agrees(got, want, dtype):
    """fp32: summation order only.  bf16: GEMM operands, cache rows and activations are rounded through every layer, and a
    token whose router scores nearly tie may take another expert than the oracle's; the typical token must be close and
    only a few may be far."""
    if dtype == torch.float32:
        return rel_err(got, want) < TOL32
    per_token = np.abs(got - want).reshape(-1, got.shape[-1]).max(-1) / np.abs(want).max()
    return bool(np.median(per_token) < 0.05 and np.mean(per_token > 0.2) <= 0.2)


TOL32 = 2e-4
