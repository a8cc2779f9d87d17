"""Host-side pieces of the model-folder path (no GPU): the safetensors container, configuration from config.json and tensor
shapes, ring arithmetic, the registry's choice of class, the oracle's own consistency, and the trace session's bookkeeping."""
import json
import struct

import numpy as np
import pytest
import torch

from oracle import lepalorn as O


def test_safetensors_round_trip_and_layout(tmp_path):
    from lit_llama.safetensors_io import SafetensorsFile, save_safetensors

    t = {"a": torch.randn(3, 5).to(torch.bfloat16), "s": torch.tensor(1.5, dtype=torch.bfloat16),
         "i": torch.arange(7, dtype=torch.int32), "empty": torch.zeros((0, 4)), "f": torch.randn(2, 2, 2)}
    save_safetensors(t, tmp_path / "m.safetensors")
    raw = (tmp_path / "m.safetensors").read_bytes()
    (n,) = struct.unpack("<Q", raw[:8])
    head = json.loads(raw[8:8 + n])
    assert head["a"] == {"dtype": "BF16", "shape": [3, 5], "data_offsets": [0, 30]} and head["s"]["shape"] == []
    with SafetensorsFile(tmp_path / "m.safetensors") as f:
        assert set(f.names()) == set(t) and f.shape("f") == (2, 2, 2) and "a" in f and "zz" not in f
        for k, v in t.items():
            got = f.get(k)
            assert got.dtype == v.dtype and got.shape == v.shape and torch.equal(got, v)


def test_safetensors_rejects_a_broken_file(tmp_path):
    from lit_llama.safetensors_io import SafetensorsFile

    (tmp_path / "short").write_bytes(b"\x01\x02")
    with pytest.raises(ValueError):
        SafetensorsFile(tmp_path / "short")
    js = json.dumps({"a": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}).encode()
    (tmp_path / "cut").write_bytes(struct.pack("<Q", len(js)) + js + b"\0" * 8)
    with pytest.raises(ValueError):
        SafetensorsFile(tmp_path / "cut")


def test_config_from_json_and_shapes():
    from lit_llama.lepalorn import LepalornConfig
    from tests.util_lepalorn import case_mixed

    cfg, W = case_mixed()
    shapes = {k: tuple(np.shape(v)) for k, v in W.items()}
    c = LepalornConfig.from_dict(cfg, shapes)
    assert (c.vocab, c.width, c.n_layer, c.eps, c.embedding_scale) == (61, 96, 5, 1e-4, 3.0)
    m = c.layers[1].mixer
    assert (m.heads, m.nope_dim, m.rot_dim, m.rot_dims, m.v_dim, m.kv_rank, m.window, m.rot_base) == (2, 8, 6, 4, 10, 12, 7, 500.0)
    assert c.layers[1].mlp is None and c.layers[2].mixer.kv_from == 0 and c.layers[4].mixer.kv_from == 1
    f = c.layers[3].mlp
    assert (f.experts, f.top, f.ff, f.limit, f.shared_ff, f.shared_limit, f.shared_gate) == (6, 6, 9, 0.5, 7, 0.6, True)
    assert c.layers[2].mlp.shared_ff is None
    # sizes the file leaves out come from the tensors
    slim = json.loads(json.dumps(cfg))
    del slim["vocab"], slim["width"]
    for l in slim["layers"]:
        for k in ("heads", "dim", "rot_dim", "vdim", "kv_rank"):
            del l["mixer"][k]
        if l["mlp"]:
            del l["mlp"]["router"]["experts"], l["mlp"]["expert"]["ff"]
    assert LepalornConfig.from_dict(slim, shapes) == c


@pytest.mark.parametrize("edit, message", [
    (lambda c: c["layers"][2]["mixer"].update(kv_from=3), "earlier layer"),
    (lambda c: c["layers"][4]["mixer"].update(kv_from=2), "cache of its own"),
    (lambda c: c["layers"][2]["mixer"].update(kv_rank=41), "latent row differs"),
    (lambda c: c["layers"][0].update(type="other"), "unknown mixer"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=5), "even"),
])
def test_config_rejects_what_cannot_run(edit, message):
    from lit_llama.lepalorn import LepalornConfig
    from tests.util_lepalorn import case_mixed

    cfg, _ = case_mixed()
    edit(cfg)
    with pytest.raises(ValueError, match=message):
        LepalornConfig.from_dict(cfg)


def test_ring_arithmetic():
    from lit_llama.cache import max_portion, ring_length

    assert ring_length(1000, 40, 64) == 103 and max_portion(103, 1000, 40) == 64
    assert ring_length(50, 40, 64) == 50 and max_portion(50, 50, 40) == 50      # the ring never wraps: no limit from it
    assert ring_length(1000, None, 64) == 1000 and max_portion(1000, 1000, None) == 1000
    assert ring_length(1000, 1, 1) == 1 and max_portion(1, 1000, 1) == 1
    for window in (1, 2, 7, 40):
        for portion in (1, 2, 5, 64):
            n = ring_length(10 ** 6, window, portion)
            p = max_portion(n, 10 ** 6, window)
            # a step of p tokens starting at any position: the slots it writes and the slots its queries read never collide
            start = 12345
            written = {(start + t) % n for t in range(p)}
            needed_before = {(j) % n for j in range(start - (window - 1), start)}
            assert p == portion and not (written & needed_before) and len(written) == p


def test_tensor_pool_hands_out_the_same_tensors():
    from lit_llama.cache import TensorPool

    dropped = []
    pool = TensorPool(max_sets=2, on_evict=lambda: dropped.append(1))
    a = pool.get([(2, 3), (4,)], torch.float32, "cpu")
    a[0].fill_(7)
    b = pool.get([(2, 3), (4,)], torch.float32, "cpu", zero=False)
    assert b[0].data_ptr() == a[0].data_ptr() and float(b[0].sum()) == 42
    assert float(pool.get([(2, 3), (4,)], torch.float32, "cpu")[0].sum()) == 0
    pool.get([(5,)], torch.float32, "cpu")
    assert not dropped
    pool.get([(6,)], torch.float32, "cpu")
    assert dropped == [1] and len(pool) == 2


def test_registry_picks_the_class_by_architecture(tmp_path):
    from lit_llama import registry

    assert "Lepalorn" in registry.architectures()
    (tmp_path / "config.json").write_text(json.dumps({"architecture": "Nonesuch"}))
    with pytest.raises(ValueError, match="Nonesuch"):
        registry.load_model_dir(tmp_path)
    seen = {}
    registry.register_architecture("Nonesuch", lambda p, dtype, device: seen.setdefault("args", (p, dtype, device)) or "model")
    registry.load_model_dir(tmp_path, dtype=torch.float32, device="cpu")
    assert seen["args"] == (tmp_path, torch.float32, "cpu")
    registry._FROM_DIR.pop("Nonesuch")


def test_oracle_windows_and_shared_rows():
    """The oracle against itself: a window at least as long as the sequence equals no window; logits at a position do not
    depend on later tokens; a layer reading another layer's rows differs from one making its own."""
    from tests.util_lepalorn import case_mixed

    cfg, W = case_mixed()
    toks = list(np.random.RandomState(0).randint(0, 61, size=14))
    base = O.forward(cfg, W, toks)
    assert np.allclose(O.forward(cfg, W, toks[:9]), base[:9], atol=1e-12)
    wide = json.loads(json.dumps(cfg))
    for l in wide["layers"]:
        l["mixer"]["mask"]["size"] = 14
    none = json.loads(json.dumps(wide))
    for l in none["layers"]:
        l["mixer"]["mask"]["size"] = None
    assert np.allclose(O.forward(wide, W, toks), O.forward(none, W, toks), atol=1e-12)
    assert np.abs(O.forward(wide, W, toks) - base).max() > 1e-3          # the windows of the case do cut keys off
    s = np.array([[0.0, 5.0, 1.0], [2.0, 0.0, 9.0], [1.0, 1.0, 1.0]])
    w = O.window_softmax(s, 2)
    assert w[0, 0] == 1 and w[1, 2] == 0 and w[2, 0] == 0 and np.allclose(w.sum(-1), 1) and np.allclose(w[2, 1:], 0.5)


def test_trace_session_bookkeeping():
    from lit_llama.trace import TraceSession

    class Fake:
        def __init__(self):
            self.calls, self.resets = [], 0

        def reset_cache(self):
            self.resets += 1

        def __call__(self, idx, max_seq_length, input_pos, out_rows=None):
            self.calls.append((idx.tolist(), max_seq_length, input_pos.tolist(), list(out_rows)))
            return torch.arange(len(out_rows) * 3, dtype=torch.float32).reshape(1, len(out_rows), 3)

    fake = Fake()
    s = TraceSession(fake, 10, device="cpu")
    assert s.step([{"id": "a", "tokens": [4, 5, 6], "want": []}]) is None
    out = s.step([{"id": "a", "tokens": [7, 8], "want": [1]}], end=["a"])
    assert out.shape == (1, 3) and fake.calls[1] == ([[7, 8]], 10, [3, 4], [1])
    assert fake.resets == 2 and not s.live                              # once at the start, once when the request ended
    s.step([{"id": "b", "tokens": [1], "want": [0]}])
    assert fake.calls[2][2] == [0]
    with pytest.raises(RuntimeError, match="holds"):
        s.step([{"id": "b", "tokens": list(range(10)), "want": []}])
    with pytest.raises(RuntimeError, match="still hold"):
        s.step([{"id": "c", "tokens": [1], "want": []}])


def test_expert_gemm_path_choice():
    """Which steps run their expert GEMMs on the tcgen05 kernels: bfloat16, rows TMA can tile, enough rows per expert."""
    from lit_llama.moe import MoE, MoESpec, TC_MIN_ROWS, TC_MIN_ROWS_PER_EXPERT

    moe = MoE(MoESpec(64, 4, 2, 24, 1.0), torch.bfloat16, "cpu")
    x = torch.zeros((TC_MIN_ROWS, 64), dtype=torch.bfloat16)
    n = max(TC_MIN_ROWS, TC_MIN_ROWS_PER_EXPERT * 4)
    assert moe.takes_tensor_cores(n, x)
    assert not moe.takes_tensor_cores(TC_MIN_ROWS - 1, x)                      # a small step
    assert not moe.takes_tensor_cores(n, x.float())                            # float32 stays on the fp32 kernels
    assert not moe.takes_tensor_cores(n, torch.zeros((8, 72), dtype=torch.bfloat16)[:, :64][:, ::1].as_strided((8, 64), (68, 1)))
    many = MoE(MoESpec(64, 64, 2, 24, 1.0), torch.bfloat16, "cpu")
    assert not many.takes_tensor_cores(TC_MIN_ROWS_PER_EXPERT * 64 - 1, x)     # too few rows per expert for 128-row tiles
    odd = MoE(MoESpec(60, 4, 2, 24, 1.0), torch.bfloat16, "cpu")
    assert not odd.takes_tensor_cores(n, torch.zeros((8, 60), dtype=torch.bfloat16))   # rows that are no 16-byte multiple
    odd_ff = MoE(MoESpec(64, 4, 2, 20, 1.0), torch.bfloat16, "cpu")
    assert not odd_ff.takes_tensor_cores(n, x)
