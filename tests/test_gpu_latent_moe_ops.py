"""The kernels behind latent attention, the mixture of experts and the fp32 residual stream, each alone against the
float64 oracle (oracle/lepalorn.py), on inputs made so that a fault shows: one key that dominates among hundreds, keys just
inside and just outside a window, rings that have wrapped, pre-activations beyond the clamp, experts nobody chose."""
import numpy as np
import pytest
import torch

from oracle import lepalorn as O

pytestmark = pytest.mark.gpu
DT = [torch.float32, torch.bfloat16]
TOL = {torch.float32: 3e-5, torch.bfloat16: 2e-2}


def dev(a, dtype=torch.float32):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to("cuda", dtype)


def host(t):
    return t.double().cpu().numpy()


def close(got, want, tol):
    assert np.abs(got - want).max() <= tol * max(1.0, np.abs(want).max()), np.abs(got - want).max()


@pytest.mark.parametrize("dtype", DT)
def test_gain_norm_add_and_depth_mix(dtype):
    from lit_llama.lepalorn import gain_norm_add_mix

    r = np.random.RandomState(0)
    rows, dim, n = 7, 50, 4
    stack = r.randn(n, rows, dim)
    x, y = r.randn(rows, dim), O.bf16_round(3 * r.randn(rows, dim)).astype(np.float64)
    w = r.randn(n)
    gain, eps = 0.625, 1e-3
    res = x + gain * O.rms(y, eps)
    t_stack = dev(stack)
    out = t_stack[n - 1]
    nxt = torch.empty((rows, dim), device="cuda")
    act = torch.empty((rows, dim), device="cuda", dtype=dtype)
    tx, ty, tg, tw = dev(x), dev(y, dtype), dev([gain]), dev(w)
    gain_norm_add_mix(tx, ty, tg, eps, out=out, stack=t_stack, mix_w=tw, n_mix=n, nxt=nxt, nxt_act=act)
    close(host(out), res, 1e-5)
    mixed = w[n - 1] * res + sum(w[j] * stack[j] for j in range(n - 1))
    close(host(nxt), mixed, 1e-5)
    close(host(act), mixed, TOL[dtype])
    # without a mix, and the norm alone on an fp32 stream
    gain_norm_add_mix(tx, ty, tg, eps, out=nxt, nxt_act=act)
    close(host(nxt), res, 1e-5)
    gain_norm_add_mix(None, tx, tg, eps, nxt_act=act)
    close(host(act), gain * O.rms(x, eps), TOL[dtype])


@pytest.mark.parametrize("dtype", DT)
def test_clamped_glu_beyond_its_limits(dtype):
    from lit_llama.moe import glu_clamp

    r = np.random.RandomState(1)
    ff, limit = 13, 0.75
    gu = O.bf16_round(2 * r.randn(9, 2 * ff + 1)).astype(np.float64)      # many values beyond +-limit; one extra column
    g, u = np.minimum(gu[:, :ff], limit), np.clip(gu[:, ff:2 * ff], -limit, limit)
    want = g / (1 + np.exp(-1.702 * g)) * (u + 1)
    close(host(glu_clamp(dev(gu, dtype), ff, limit, 1.702)), want, TOL[dtype])


def _append(dtype, d, norm_w, pos, S, KR, R, dims, base, eps, cache=None, B=1):
    from lit_llama import _native as N
    from lit_llama.latent_attention import build_rope_table

    T = len(pos)
    rope = build_rope_table(max(pos) + 1, dims, base, "cuda")
    if cache is None:
        cache = torch.zeros((B, S, KR + R), device="cuda", dtype=dtype)
    proj = torch.zeros((B * T, 3 + KR + R), device="cuda", dtype=dtype)    # the rows sit at column 3 of a wider projection
    proj[:, 3:] = dev(d, dtype)
    w, p = dev(norm_w), torch.tensor(pos, dtype=torch.int32, device="cuda")     # named: alive until the launch
    N.call("ll_latent_kv_append", N.ptr(proj), N.dtype_code(dtype), proj.shape[1], 3, N.ptr(w), eps, N.ptr(rope),
           N.ptr(p), N.ptr(cache), B, T, KR, R, dims, S, N.stream())
    return cache, rope


@pytest.mark.parametrize("dtype", DT)
def test_latent_rows_norm_rotation_and_ring_slots(dtype):
    r = np.random.RandomState(2)
    KR, R, dims, S, base, eps = 20, 10, 6, 8, 300.0, 1e-3
    pos = [1013, 1014, 1015]                                  # far positions; slots 5, 6, 7 of the ring
    d = O.bf16_round(r.randn(3, KR + R)).astype(np.float64)
    w = 1 + 0.3 * r.randn(KR)
    cache, _ = _append(dtype, d, w, pos, S, KR, R, dims, base, eps)
    want_c = O.rms(d[:, :KR], eps) * w
    want_k = O.rotate_pairs(d[:, KR:], np.array(pos), base, dims)
    got = host(cache[0])
    for t, p in enumerate(pos):
        close(got[p % S, :KR], want_c[t], TOL[dtype])
        close(got[p % S, KR:], want_k[t], TOL[dtype])
    assert np.abs(got[:5]).max() == 0                          # nothing else was touched
    close(got[[5, 6, 7], KR + dims:], d[:, KR + dims:], 0)     # beyond rot_dims: passed through unchanged


def _attend(dtype, q_lat, q_rot, gate, cache_rows, pos, S, window, scale, dims, base, splits, H, KR, R):
    """Run ll_latent_attn for ONE sequence whose ring holds ``cache_rows`` (already normed / rotated) by position."""
    from lit_llama import _native as N
    from lit_llama.latent_attention import build_rope_table

    T = len(pos)
    rope = build_rope_table(max(pos) + 1, dims, base, "cuda")
    ring = torch.zeros((1, S, KR + R), device="cuda", dtype=dtype)
    for p, row in cache_rows.items():
        ring[0, p % S] = dev(row, dtype)
    stride = H * (3 + R) + H + 2
    proj = torch.zeros((T, stride), device="cuda", dtype=dtype)
    for h in range(H):
        proj[:, h * (3 + R) + 3: (h + 1) * (3 + R)] = dev(q_rot[:, h], dtype)
    proj[:, H * (3 + R): H * (3 + R) + H] = dev(gate, dtype)
    ql = dev(q_lat.transpose(1, 0, 2), dtype).contiguous()                 # [H, T, KR]
    out = torch.empty_like(ql)
    scratch = torch.empty(max(1, N.call_ret("ll_latent_attn_scratch_bytes", T, H, KR, splits) // 4), device="cuda")
    p = torch.tensor(pos, dtype=torch.int32, device="cuda")
    N.call("ll_latent_attn", N.ptr(ql), T * KR, KR, N.ptr(proj), stride, 3, 3 + R, H * (3 + R), N.ptr(rope),
           N.ptr(p), N.ptr(ring), N.ptr(out), T * KR, KR, N.dtype_code(dtype), 1, T,
           H, KR, R, dims, S, window, scale, splits, N.ptr(scratch), N.stream())
    return host(out).transpose(1, 0, 2)                                     # [T, H, KR]


def _attend_oracle(q_lat, q_rot, gate, rows, pos, window, scale, dims, base, KR):
    out = np.zeros_like(q_lat)
    for t, p in enumerate(pos):
        lo = max(0, p - window + 1) if window > 0 else 0
        keys = list(range(lo, p + 1))
        c = np.stack([rows[j][:KR] for j in keys])
        kr = np.stack([rows[j][KR:] for j in keys])
        for h in range(q_lat.shape[1]):
            qr = O.rotate_pairs(q_rot[t:t + 1, h], np.array([p]), base, dims)[0]
            s = (c @ q_lat[t, h] + kr @ qr) * scale
            e = np.exp(s - s.max())
            out[t, h] = (e / e.sum()) @ c / (1 + np.exp(-gate[t, h]))
    return out


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("splits", [1, 3])
@pytest.mark.parametrize("sizes", [(3, 24, 6), (5, 320, 16)])
def test_window_edges_with_a_key_that_dominates(dtype, splits, sizes):
    """Position 100 holds a key whose score dwarfs all others.  With a window of 37, the queries at 100 .. 136 must
    return (almost exactly) its row and the query at 137 must not see it; likewise in the first tokens of a sequence.
    Short rows and rows of hundreds of values (in bfloat16 these take the two block shapes of the tensor-core kernel)."""
    r = np.random.RandomState(3)
    H, KR, R = sizes
    dims, base, window, scale = R, 100.0, 37, 0.5
    S = 80                                                     # the ring has wrapped by position 137: slot of p is p % 80
    rows = {j: O.bf16_round(0.3 * r.randn(KR + R)).astype(np.float64) for j in range(138 - S, 138)}
    probe = np.zeros(KR)
    probe[5] = 1.0
    rows[100][:KR] = O.bf16_round(0.3 * r.randn(KR))
    rows[100][5] = 16.0                                        # a query along `probe` scores 16 * 8 * scale = 64 here
    pos = [100, 101, 135, 136, 137]
    q_lat = np.tile(8.0 * probe, (len(pos), H, 1)) + O.bf16_round(0.1 * r.randn(len(pos), H, KR))
    q_rot = O.bf16_round(r.randn(len(pos), H, R)).astype(np.float64)
    gate = O.bf16_round(r.randn(len(pos), H)).astype(np.float64)
    got = _attend(dtype, q_lat, q_rot, gate, rows, pos, S, window, scale, dims, base, splits, H, KR, R)
    want = _attend_oracle(q_lat, q_rot, gate, rows, pos, window, scale, dims, base, KR)
    close(got, want, TOL[dtype])
    sig = 1 / (1 + np.exp(-gate))
    assert np.abs(want[3, :, 5] / sig[3] - 16.0).max() < 0.1   # 136 - 100 = 36 < 37: seen
    assert np.abs(want[4, :, 5] / sig[4]).max() < 2.0          # 137 - 100 = 37: just outside
    assert np.abs(got[3, :, 5] / sig[3] - 16.0).max() < 0.2 and np.abs(got[4, :, 5] / sig[4]).max() < 2.0


@pytest.mark.parametrize("dtype", DT)
def test_a_far_key_among_hundreds_and_the_first_tokens(dtype):
    r = np.random.RandomState(4)
    H, KR, R, dims, base, window, scale = 2, 16, 4, 2, 50.0, 600, 0.25
    S = 700
    rows = {j: O.bf16_round(0.3 * r.randn(KR + R)).astype(np.float64) for j in range(0, 650)}
    rows[60][KR:KR + 2] = [24.0, 0.0]                          # found through the ROTATED part: only the right angle scores
    pos = [0, 1, 2, 59, 60, 649]
    q_lat = O.bf16_round(0.2 * r.randn(len(pos), H, KR)).astype(np.float64)
    q_rot = np.zeros((len(pos), H, R))
    gate = np.full((len(pos), H), 30.0)                        # gate ~ 1
    # the query at 649 carries, before rotation, the vector that its own rotation turns onto the stored (rotated) key of 60
    ang = 649 * 1.0                                            # frequency of pair 0 is 1
    q_rot[5, :, 0], q_rot[5, :, 1] = 16 * np.cos(-ang), 16 * np.sin(-ang)
    for splits in (1, 4):
        got = _attend(dtype, q_lat, q_rot, gate, rows, pos, S, window, scale, dims, base, splits, H, KR, R)
        want = _attend_oracle(q_lat, q_rot, gate, rows, pos, window, scale, dims, base, KR)
        close(got, want, TOL[dtype] * 2)
        assert np.abs(want[5] - rows[60][:KR]).max() < 0.05    # the far key takes (almost) all the weight
        assert np.abs(got[5] - rows[60][:KR]).max() < 0.08
        assert np.abs(got[0] - rows[0][:KR]).max() < 0.02      # position 0 sees itself only


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("shape", [(11, 40, 7, 3, 12), (64, 33, 1, 1, 12), (5, 24, 4, 4, 16), (300, 96, 16, 2, 24), (700, 64, 3, 2, 72)])
def test_router_permutation_and_grouped_experts(dtype, shape):
    from lit_llama.moe import MoE, MoESpec

    M, width, X, top, ff = shape      # widths / ff that are and are not multiples of 8: tensor-core and plain kernels
    sff = 9
    r = np.random.RandomState(5)
    cfgf = O.mlp_cfg(X, top, ff, 0.6, sff, 0.9)
    mc = O.model_cfg(8, width, [(O.mixer_cfg(1, 2, 2, 2, 2, 2), cfgf)])
    W = O.random_weights(mc, 6)
    if X > 4:
        W["l0.mlp.router.b"][X - 1] = -50.0                    # an expert nobody chooses: an empty segment in the sort
    moe = MoE(MoESpec(width, X, top, ff, 0.6, sff, 0.9), dtype, "cuda")
    moe.load(lambda s: dev(W["l0.mlp." + s], dtype))
    h = O.bf16_round(r.randn(M, width)).astype(np.float64)
    idx, w, offsets, perm = moe.route(dev(h, dtype))
    want_idx, want_w = O.route(h, W["l0.mlp.router"].astype(np.float64), W["l0.mlp.router.b"].astype(np.float64), top)
    assert np.array_equal(host(idx).astype(int), want_idx)
    close(host(w), want_w, 1e-5)
    off, pm = host(offsets).astype(int), host(perm).astype(int)
    assert off[0] == 0 and off[-1] == M * top and sorted(pm.tolist()) == list(range(M * top))
    flat = want_idx.reshape(-1)
    for e in range(X):
        assert all(flat[p] == e for p in pm[off[e]:off[e + 1]])
    close(host(moe(dev(h, dtype))), O.moe(h, {k: np.asarray(v, dtype=np.float64) for k, v in W.items()}, "l0.mlp.", cfgf), TOL[dtype] * 3)


@pytest.mark.parametrize("shape", [(1500, 64, 5, 2, 72), (700, 320, 3, 3, 40), (1100, 200, 7, 2, 136), (2300, 512, 4, 1, 264), (1900, 64, 40, 2, 24)])
def test_grouped_experts_on_the_tcgen05_path(shape, monkeypatch):
    """Many rows per expert: the tensor-core kernels (row tiles of 128 that run past an expert's last row, an output
    width that is no multiple of the tile, a K that is no multiple of 64, an empty expert, more experts than one pass of
    the tile lookup examines) against the float64 oracle
    and against the kernels that small steps take."""
    import lit_llama.moe as MOE
    from lit_llama import _native as N

    M, width, X, top, ff = shape
    r = np.random.RandomState(11)
    cfgf = O.mlp_cfg(X, top, ff, 0.6, 9, 0.9)
    mc = O.model_cfg(8, width, [(O.mixer_cfg(1, 2, 2, 2, 2, 2), cfgf)])
    W = O.random_weights(mc, 12)
    if X > 4:
        W["l0.mlp.router.b"][1] = -50.0                        # an empty segment between two full ones
    moe = MOE.MoE(MOE.MoESpec(width, X, top, ff, 0.6, 9, 0.9), torch.bfloat16, "cuda")
    moe.load(lambda s: dev(W["l0.mlp." + s], torch.bfloat16))
    h = O.bf16_round(r.randn(M, width)).astype(np.float64)
    x = dev(h, torch.bfloat16)
    monkeypatch.setattr(MOE, "TC_MIN_ROWS", 256)
    monkeypatch.setattr(MOE, "TC_MIN_ROWS_PER_EXPERT", 1)
    assert moe.takes_tensor_cores(M * top, x)
    got = host(moe(x))
    assert N.call_ret("ll_moe_tc_error") == 0
    monkeypatch.setattr(MOE, "TC_MIN_ROWS", 1 << 30)
    assert not moe.takes_tensor_cores(M * top, x)
    other = host(moe(x))
    want = O.moe(h, {k: np.asarray(v, dtype=np.float64) for k, v in W.items()}, "l0.mlp.", cfgf)
    close(got, want, TOL[torch.bfloat16] * 3)
    close(got, other, 1e-2)
