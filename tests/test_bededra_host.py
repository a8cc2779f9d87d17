"""Host-side parts of the Bededra family (no GPU): configuration from a config.json dictionary and tensor shapes, the
kept-tokens + ring arithmetic, the registry entry and per-family kernel lists, and properties of the float64 oracle the
GPU tests compare with."""
import importlib.util
from pathlib import Path

import numpy as np
import pytest

from oracle import bededra as O
from tests.util_bededra import case_mixed, case_ones, file_cfg

ROOT = Path(__file__).resolve().parent.parent


def test_oracle_portions_of_the_recurrence_compose():
    r = np.random.RandomState(0)
    T, n, p = 12, 5, 3
    q, k, v, a = r.randn(T, n), r.randn(T, n), r.randn(T, p), r.uniform(0.5, 1, (T, n))
    y = O.linear_recurrence(q, k, v, a)
    # closed form: y_t = sum_{s <= t} (q_t . (prod_{s < u <= t} a_u) k_s) v_s
    want = np.zeros((T, p))
    for t in range(T):
        for s in range(t + 1):
            want[t] += (q[t] * np.prod(a[s + 1:t + 1], axis=0) * k[s]).sum() * v[s]
    assert np.allclose(y, want)


def test_oracle_visibility():
    assert O.visible(10, 10, 1, 0) and not O.visible(10, 9, 1, 0)
    assert O.visible(100, 85, 16, 3) and not O.visible(100, 84, 16, 3)
    assert O.visible(100, 2, 16, 3) and not O.visible(100, 3, 16, 3)
    assert not O.visible(5, 6, 16, 3)


def test_oracle_router_keeps_to_the_best_groups():
    h = np.eye(8)
    w = np.array([[9, 0, 0, 0, 0, 0, 0, 0], [0, 1, 0, 0, 0, 0, 0, 0], [8, 0, 0, 0, 0, 0, 0, 0], [7, 0, 0, 0, 0, 0, 0, 0]], dtype=float)
    idx, wts = O.route(h[:1], w, 2, 2, 1)          # groups {0, 1}, {2, 3}: the first holds the best expert
    assert sorted(idx[0].tolist()) == [0, 1] and abs(wts.sum() - 1) < 1e-12
    idx, _ = O.route(h[:1], w, 2, 2, 2)
    assert sorted(idx[0].tolist()) == [0, 2]


def test_config_from_file_and_from_shapes():
    pytest.importorskip("torch")
    try:
        from lit_llama.bededra import BededraConfig
    except ImportError as e:          # the kernels' library is not built here
        pytest.skip(str(e))
    cfg, W = case_mixed()
    shapes = {k: tuple(v.shape) for k, v in W.items()}
    c = BededraConfig.from_dict(file_cfg(cfg), shapes)
    assert [l.kind for l in c.layers] == ["mamba2", "parallel", "parallel", "mamba2", "parallel"]
    assert c.layers[0].mixer.taps == 3 and c.layers[0].mixer.norm_groups == 3 and c.canon_taps == 4
    assert c.layers[1].mixer.left.keep_first == 3 and c.layers[1].mixer.right.decay_rank == 5
    assert c.layers[2].mlp is None and c.layers[1].mlp.ff == 40
    assert c.layers[4].mlp.groups == 4 and c.layers[4].mlp.keep_groups == 2 and c.layers[4].mlp.score == "all"
    # sizes the file leaves out come from the tensors
    thin = file_cfg(cfg)
    del thin["vocab"], thin["width"], thin["layers"][1]["mixer"]["left"]["dim"], thin["layers"][0]["mixer"]["conv"]
    c2 = BededraConfig.from_dict(thin, shapes)
    assert (c2.vocab, c2.width, c2.layers[1].mixer.left.dim, c2.layers[0].mixer.taps) == (53, 48, 12, 3)
    bad = file_cfg(cfg)
    bad["layers"][0]["type"] = "other"
    with pytest.raises(ValueError):
        BededraConfig.from_dict(bad, shapes)


def test_kept_tokens_and_ring_arithmetic():
    pytest.importorskip("torch")
    try:
        from lit_llama.window_attention import WindowAttentionSpec
    except ImportError as e:
        pytest.skip(str(e))
    s = WindowAttentionSpec(width=8, heads=2, kv_heads=1, dim=4, vdim=4, scale=0.5, softcap=0.0, window=16, keep_first=3)
    assert s.ring(1000, 20) == 35 and s.portion(35, 1000) == 20
    assert s.ring(30, 4096) == 27 and s.portion(27, 30) == 27          # never more than the sequence needs
    u = WindowAttentionSpec(width=8, heads=2, kv_heads=2, dim=4, vdim=4, scale=0.5, softcap=0.0, window=None, keep_first=0)
    assert u.ring(50, 8) == 50
    # a pass of `portion` tokens never writes a slot one of its own queries reads
    for portion in (1, 2, 7):
        ring = s.ring(1000, portion)
        for p0 in (3, 17, 200):
            written = {3 + (p - 3) % ring for p in range(p0, p0 + portion)}
            read = {3 + (p - 3) % ring for p in range(max(3, p0 - 15), p0)}
            assert not (written & read)


def test_registry_and_family_kernel_lists():
    spec = importlib.util.spec_from_file_location("llb200_build", ROOT / "lit-llama-ja_b200" / "build.py")
    build = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(build)
    assert set(build.FAMILY_SOURCES) >= {"Lepalorn", "Bededra"}
    for stems in build.FAMILY_SOURCES.values():
        for s in stems:
            assert (build.CSRC / f"{s}.cu").is_file(), s
    try:
        from lit_llama.registry import architectures
    except ImportError as e:
        pytest.skip(str(e))
    assert {"Lepalorn", "Bededra"} <= set(architectures())


def test_cases_are_what_they_claim():
    cfg, _ = case_ones()
    assert cfg["layers"][0]["mixer"]["left"]["mask"]["size"] == 1 and cfg["layers"][1]["mixer"]["conv"] == 1
