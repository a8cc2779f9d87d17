"""Lepalorn on the GPU against the float64 oracle (oracle/lepalorn.py): whole prompts, single-token decoding, portions
down to two tokens, rings that wrap and are reused, batches, sizes that are 1, and greedy generation through
``generate()``.  Every comparison is against the oracle run on the WHOLE sequence without any cache."""
import numpy as np
import pytest
import torch

from oracle import lepalorn as O
from tests.util_lepalorn import RMS_TOL, TOL, agrees, case_mixed, case_odd, case_ones, load, rel_err, rms_err, run_schedule, write_model

pytestmark = pytest.mark.gpu

T_LONG = 45


@pytest.fixture(scope="module")
def mixed(tmp_path_factory):
    cfg, W = case_mixed()
    folder = write_model(tmp_path_factory.mktemp("mixed"), cfg, W)
    toks = np.random.RandomState(7).randint(0, cfg["vocab"], size=T_LONG).tolist()
    return cfg, W, folder, toks, O.forward(cfg, W, toks)


@pytest.fixture(scope="module")
def ones(tmp_path_factory):
    cfg, W = case_ones()
    folder = write_model(tmp_path_factory.mktemp("ones"), cfg, W)
    toks = np.random.RandomState(8).randint(0, cfg["vocab"], size=23).tolist()
    return cfg, W, folder, toks, O.forward(cfg, W, toks)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_whole_prompt_and_every_layer(mixed, dtype):
    cfg, W, folder, toks, want = mixed
    m = load(folder, dtype)
    streams = []
    m.layer_probe = lambda i, x: streams.append(x.double().cpu().numpy())
    got = run_schedule(m, toks, [len(toks)], 64)[0]
    _, want_streams = O.forward(cfg, W, toks, return_layers=True)
    for i, (g, w) in enumerate(zip(streams, want_streams)):
        assert agrees(g, w, dtype), f"stream after layer {i}: {rel_err(g, w)} {rms_err(g, w)}"
    assert agrees(got, want, dtype), (rel_err(got, want), rms_err(got, want))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_token_by_token_equals_prefill(mixed, dtype):
    cfg, W, folder, toks, want = mixed
    m = load(folder, dtype)
    got = run_schedule(m, toks, [1] * len(toks), 64)[0]        # the first tokens of a sequence included
    assert agrees(got, want, dtype), rel_err(got, want)
    got = run_schedule(m, toks, [len(toks) - 20] + [1] * 20, 64)[0]
    assert agrees(got, want, dtype), rel_err(got, want)


@pytest.mark.parametrize("portions", [[2] * 22 + [1], [3, 2, 7, 1, 1, 11, 2, 5, 13], [44, 1], [1, 44], [5, 40]])
def test_portions_of_any_size(mixed, portions):
    cfg, W, folder, toks, want = mixed
    m = load(folder, torch.float32)
    assert rel_err(run_schedule(m, toks, portions, 64)[0], want) < TOL[torch.float32]


@pytest.mark.parametrize("portion", [1, 2, 3, 8])
def test_ring_wraps_and_slots_are_reused(mixed, portion):
    """A ring of (longest window - 1 + portion) slots: every slot is overwritten several times within one sequence, in
    prompts (cut into passes by the model itself) and in decoding."""
    cfg, W, folder, toks, want = mixed
    m = load(folder, torch.float32, prefill_portion=portion)
    got = run_schedule(m, toks, [30] + [1] * 15, 64)[0]
    assert m._ring == 9 - 1 + portion and m._ring < len(toks)
    assert rel_err(got, want) < TOL[torch.float32]
    got = run_schedule(m, toks, [7, 2, 21, 15], 64)[0]
    assert rel_err(got, want) < TOL[torch.float32]


def test_a_new_request_reuses_the_rows_of_an_ended_one(mixed):
    cfg, W, folder, toks, want = mixed
    m = load(folder, torch.float32)
    other = np.random.RandomState(9).randint(0, cfg["vocab"], size=40).tolist()
    run_schedule(m, other, [33] + [1] * 7, 64)                       # fills rows and captures the step graph
    ptr = m.kv_caches[0].data_ptr()
    got = run_schedule(m, toks, [len(toks) - 5] + [1] * 5, 64)[0]   # reset_cache() inside: same tensors, from position 0
    assert m.kv_caches[0].data_ptr() == ptr
    assert rel_err(got, want) < TOL[torch.float32]
    short = run_schedule(m, toks[:3], [3], 64)[0]                    # a shorter request over a longer one's leftovers
    assert rel_err(short, want[:3]) < TOL[torch.float32]


def test_batch_rows_are_independent(mixed):
    cfg, W, folder, toks, want = mixed
    m = load(folder, torch.float32)
    other = np.random.RandomState(10).randint(0, cfg["vocab"], size=len(toks)).tolist()
    both = run_schedule(m, [toks, other], [len(toks) - 6] + [1] * 6, 64)
    assert rel_err(both[0], want) < TOL[torch.float32]
    assert rel_err(both[1], O.forward(cfg, W, other)) < TOL[torch.float32]
    alone = run_schedule(m, toks, [len(toks) - 6] + [1] * 6, 64)[0]
    assert np.abs(both[0] - alone).max() < 1e-4 * np.abs(alone).max()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_sizes_that_are_one(ones, dtype):
    cfg, W, folder, toks, want = ones
    m = load(folder, dtype)
    assert agrees(run_schedule(m, toks, [len(toks)], 32)[0], want, dtype)
    assert agrees(run_schedule(m, toks, [2, 1, 1, 9, 1, 1, 1, 7], 32)[0], want, dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_sizes_that_are_multiples_of_nothing(tmp_path, dtype):
    cfg, W = case_odd()
    folder = write_model(tmp_path / "odd", cfg, W)
    toks = np.random.RandomState(12).randint(0, cfg["vocab"], size=31).tolist()
    want = O.forward(cfg, W, toks)
    m = load(folder, dtype, prefill_portion=5)
    assert agrees(run_schedule(m, toks, [len(toks)], 40)[0], want, dtype)
    assert agrees(run_schedule(m, toks, [2, 3, 9, 1, 1, 1, 14], 40)[0], want, dtype)


def test_long_decoding_through_several_ring_lengths(mixed):
    cfg, W, folder, _, _ = mixed
    toks = np.random.RandomState(11).randint(0, cfg["vocab"], size=120).tolist()
    want = O.forward(cfg, W, toks)
    m = load(folder, torch.float32, prefill_portion=4)               # ring of 12 slots: ten trips round it
    got = run_schedule(m, toks, [10] + [1] * 110, 128)[0]
    assert rel_err(got, want) < TOL[torch.float32]


def test_out_rows_and_forward_without_cache(mixed):
    cfg, W, folder, toks, want = mixed
    m = load(folder, torch.float32)
    idx = torch.tensor([toks], device="cuda")
    rows = [0, 7, 44]
    got = m(idx, 64, torch.arange(len(toks)), out_rows=rows)[0].double().cpu().numpy()
    assert rel_err(got, want[rows]) < TOL[torch.float32]
    m.reset_cache()
    run_schedule(m, toks[:10], [10], 64)
    nocache = m(idx)[0].double().cpu().numpy()                       # keeps nothing, disturbs nothing
    assert rel_err(nocache, want) < TOL[torch.float32]
    nxt = m(idx[:, 10:11], 64, torch.arange(10, 11))[0].double().cpu().numpy()
    assert rel_err(nxt, want[10:11]) < TOL[torch.float32]
    assert m(idx, 64, torch.arange(len(toks)), out_rows=[]).shape == (1, 0, cfg["vocab"])


def test_greedy_generation_through_generate(mixed):
    """``generate()`` - the package's own loop and sampler - on a model folder; top_k = 1 makes the draw the argmax."""
    import generate as G

    cfg, W, folder, toks, _ = mixed
    m = G.load_model(folder, None, torch.device("cuda"), torch.float32)
    prompt = torch.tensor(toks[:9], device="cuda")
    out = G.generate(m, prompt, 12, temperature=1.0, top_k=1).tolist()
    want = O.greedy(cfg, W, toks[:9], 12)
    # a near-tie between the two largest logits may legitimately flip under fp32: compare up to the first such place
    for n in range(9, len(want)):
        if out[n] != want[n]:
            lg = np.sort(O.forward(cfg, W, want[:n])[-1])
            assert lg[-1] - lg[-2] < 1e-3, f"token {n}: {out[n]} != {want[n]}"
            break
    assert out[:9] == toks[:9]
    m.reset_cache()
    out2 = G.generate(m, prompt, 12, temperature=1.0, top_k=1).tolist()
    assert out2 == out


def test_trace_session_replays_steps(mixed):
    from lit_llama.trace import TraceSession

    cfg, W, folder, toks, want = mixed
    m = load(folder, torch.float32)
    s = TraceSession(m, 64)
    assert s.step([{"id": "a", "tokens": toks[:20], "want": []}]) is None
    got = s.step([{"id": "a", "tokens": toks[20:31], "want": [0, 10]}]).double().cpu().numpy()
    assert rel_err(got, want[[20, 30]]) < TOL[torch.float32]
    got = s.step([{"id": "a", "tokens": toks[31:32], "want": [0]}], end=["a"]).double().cpu().numpy()
    assert rel_err(got, want[31:32]) < TOL[torch.float32]
    got = s.step([{"id": "b", "tokens": toks[:4], "want": [3]}]).double().cpu().numpy()
    assert rel_err(got, want[3:4]) < TOL[torch.float32]
    with pytest.raises(RuntimeError):
        s.step([{"id": "c", "tokens": [1], "want": []}])


def test_long_prompt_takes_the_tensor_core_expert_path(tmp_path, monkeypatch):
    """A prompt with hundreds of (token, choice) rows per step: with the thresholds lowered the expert GEMMs of the
    prefill run on the tcgen05 kernels inside the model (also in portions, whose row counts differ), and decoding after
    it on the small-step kernels; both against the oracle, and the prefill against the same model kept off that path."""
    import lit_llama.moe as MOE
    from lit_llama import _native as N

    layers = [
        (O.mixer_cfg(4, 16, 8, 16, 24, 33, base=1000.0), O.mlp_cfg(6, 2, 40, 0.8, 24, 1.2)),
        (O.mixer_cfg(2, 8, 8, 24, 24, 150, base=1000.0, kv_from=0), O.mlp_cfg(3, 3, 72, 1.0)),
    ]
    cfg = O.model_cfg(83, 64, layers, eps=1e-5, embedding_scale=2.0)
    W = O.random_weights(cfg, 21)
    folder = write_model(tmp_path / "wide", cfg, W)
    toks = np.random.RandomState(22).randint(0, cfg["vocab"], size=260).tolist()
    want = O.forward(cfg, W, toks)
    m = load(folder, torch.bfloat16)
    monkeypatch.setattr(MOE, "TC_MIN_ROWS", 1 << 30)
    plain = run_schedule(m, toks, [len(toks)], 300)[0]
    monkeypatch.setattr(MOE, "TC_MIN_ROWS", 128)
    monkeypatch.setattr(MOE, "TC_MIN_ROWS_PER_EXPERT", 1)
    x = torch.zeros((250, 64), dtype=torch.bfloat16, device="cuda")
    assert all(b.mlp.takes_tensor_cores(250 * b.mlp.spec.top, x) for b in m.blocks)
    got = run_schedule(m, toks, [250] + [1] * 10, 300)[0]
    assert N.call_ret("ll_moe_tc_error") == 0
    assert agrees(got, want, torch.bfloat16), (rel_err(got, want), rms_err(got, want))
    assert rms_err(got, plain) < RMS_TOL[torch.bfloat16]
    got = run_schedule(m, toks, [130, 70, 60], 300)[0]
    assert agrees(got, want, torch.bfloat16), (rel_err(got, want), rms_err(got, want))
