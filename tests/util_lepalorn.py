"""Builders shared by the Lepalorn tests: small random models written as model folders (config.json + safetensors) and
loaded back through the package's registry, and the comparison against the float64 oracle."""
import json

import numpy as np
import torch

from oracle import lepalorn as O


def case_mixed(seed=0):
    """Sizes that share nothing with each other: 3 heads, 5 experts of which 3, kv_rank 40, windows 5 / 7 / 9 / 6 / 4, a layer
    without feed-forward, two layers that read other layers' rows, rotation of only part of the rotated dimensions."""
    a = O.mixer_cfg(3, 16, 8, 24, 40, 5, base=1000.0)
    b = O.mixer_cfg(2, 8, 6, 10, 12, 7, base=500.0, rot_dims=4)
    layers = [
        (a, O.mlp_cfg(5, 3, 20, 0.8, 12, 1.2)),
        (b, None),
        (O.mixer_cfg(3, 16, 8, 24, 40, 9, base=1000.0, kv_from=0), O.mlp_cfg(4, 1, 10, 1.0)),
        (O.mixer_cfg(4, 12, 8, 6, 40, 6, base=1000.0), O.mlp_cfg(6, 6, 9, 0.5, 7, 0.6)),
        (O.mixer_cfg(2, 8, 6, 10, 12, 4, base=500.0, rot_dims=4, kv_from=1), O.mlp_cfg(3, 2, 33, 2.0)),
    ]
    cfg = O.model_cfg(61, 96, layers, eps=1e-4, embedding_scale=3.0)
    return cfg, O.random_weights(cfg, seed)


def case_ones(seed=1):
    """Sizes that are 1 or equal where a real model's differ: one head, one expert, top 1, window 1 and a window longer
    than any test sequence, kv_rank = head size = value size."""
    layers = [
        (O.mixer_cfg(1, 8, 8, 8, 8, 1), O.mlp_cfg(1, 1, 8, 1.0)),
        (O.mixer_cfg(1, 8, 8, 8, 8, 1000, kv_from=0), O.mlp_cfg(2, 2, 8, 1.0, 8, 1.0)),
        (O.mixer_cfg(2, 4, 2, 4, 4, 2), None),
    ]
    cfg = O.model_cfg(17, 8, layers, embedding_scale=1.0)
    return cfg, O.random_weights(cfg, seed, shared_gate=False)


def case_odd(seed=2):
    """Nothing is a multiple of 8 (or of 4): every kernel takes its unaligned path."""
    layers = [
        (O.mixer_cfg(5, 5, 6, 7, 13, 11, base=77.0), O.mlp_cfg(3, 2, 11, 0.9, 5, 0.7)),
        (O.mixer_cfg(3, 7, 6, 3, 13, 3, base=77.0, kv_from=0), O.mlp_cfg(7, 3, 9, 1.1)),
    ]
    cfg = O.model_cfg(37, 50, layers, eps=1e-6, embedding_scale=2.5)
    return cfg, O.random_weights(cfg, seed)


def write_model(folder, cfg, W):
    from lit_llama.safetensors_io import save_safetensors

    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(cfg))
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
    """Largest difference relative to the largest value; printed by a failing assert."""
    return float(np.abs(got - want).max() / np.abs(want).max())


def rms_err(got, want):
    return float(np.sqrt(np.mean((got - want) ** 2) / np.mean(want ** 2)))


def agrees(got, want, dtype):
    """fp32: every value within summation-order noise.  bf16: GEMM operands and cache rows are rounded (2^-9 each) through
    five layers, and a token whose two best router logits nearly tie may take another expert than the oracle's - which
    moves that token (and, through attention, its neighbours) by far more than rounding.  So for bf16 the typical token
    must be close and only a few may be far."""
    if dtype == torch.float32:
        return rel_err(got, want) < TOL[dtype] and rms_err(got, want) < RMS_TOL[dtype]
    per_token = np.abs(got - want).reshape(-1, got.shape[-1]).max(-1) / np.abs(want).max()
    return bool(np.median(per_token) < 0.04 and np.mean(per_token > 0.15) <= 0.2)


# fp32: summation order only.  bf16: GEMM operands and the cache rows are rounded (2^-9 each), through five layers
TOL = {torch.float32: 2e-4, torch.bfloat16: 0.15}
RMS_TOL = {torch.float32: 1e-4, torch.bfloat16: 0.04}
