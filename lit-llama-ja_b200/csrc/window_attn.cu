// Softmax attention over a sliding window plus a number of kept first tokens, with grouped key/value heads, a soft cap on
// the scores, a logarithmic distance penalty per head, and a mixing of the heads' softmax weights before they meet the
// values ("talking heads", after the softmax):
//
//   s_h(i, j)  = cap * tanh(scale * q_h(i) . k_g(j) / cap)  -  r1_h * ln(1 + r2_h * (i - j))          (cap 0: no cap)
//   visible    : j <= i and (i - j < window  or  j < keep)
//   w_h(i, .)  = softmax over the visible j of s_h(i, .)
//   o_h(i)     = sigmoid(gate_h(i)) * sum_j (sum_h' talk[h][h'] w_h'(i, j)) v_g(h)(j)
//
// Cache: rows [B][keep + R][G * dim] (keys) and [B][keep + R][G * vdim] (values); position j lives in slot j when
// j < keep and in slot keep + (j - keep) % R otherwise, so the kept tokens are never written over and the rest is a ring.
// Scores, softmax, the mix and the weighted sums are fp32 whatever the dtype of the rows.
//
// Because the mix needs the NORMALISED weights of every head at each (i, j), a query's keys are swept twice: once for
// every head's maximum and sum (stats), once for the weights, their mix and the values (out).  Both sweeps split a
// query's keys over `splits` blocks (decoding: one query, a long window); the parts are merged in split order.
#include "common.cuh"

namespace llb {

constexpr int WA_THREADS = 256;
constexpr int WA_ACC = 4;       // float4 accumulators per thread in the value sweep

struct WaParams {
  const void* q;  int q_stride;
  const void* kc; const void* vc;
  const int32_t* pos_ids;
  const float* r1; const float* r2; const float* talk;
  float scale, cap;
  int B, T, H, G, dim, vdim, window, keep, ring, splits, kchunk;
  int dimp, kpitch, vpitch;     // dim rounded up to 4; shared-memory row pitches (floats)
  float* stats;                 // [splits][M][H][2]
  float* part;                  // [splits][M][H * vdim]
};

struct WaRange { int i, ns, w0, u0, u1; };

// visible keys of query position i as one list u -> j (kept tokens first, then the window), and this split's part of it
__device__ __forceinline__ WaRange wa_range(const WaParams& P, int i, int split) {
  WaRange r;
  r.i = i;
  r.ns = min(P.keep, i + 1);
  r.w0 = max(P.keep, i - P.window + 1);
  const int n_vis = r.ns + max(0, i - r.w0 + 1);
  const int per = (n_vis + P.splits - 1) / P.splits;
  r.u0 = split * per;
  r.u1 = min(n_vis, r.u0 + per);
  return r;
}
__device__ __forceinline__ int wa_key(const WaRange& r, int u) { return u < r.ns ? u : r.w0 + (u - r.ns); }
__device__ __forceinline__ int wa_slot(const WaParams& P, int j) { return j < P.keep ? j : P.keep + (j - P.keep) % P.ring; }

// One cache row (G heads of `dim` elements) -> shared memory as fp32 with every head padded to `dimp` (zeros); by one warp.
template <typename T>
__device__ __forceinline__ void wa_row_to_smem(float* __restrict__ dst, const T* __restrict__ src, int G, int dim, int dimp, int lane) {
  const int n = G * dim;
  if (dim == dimp && (n & 7) == 0 && (((uintptr_t)src) & 15) == 0) {
    if (sizeof(T) == 2) {
      for (int c = lane * 8; c < n; c += 256) {
        const uint4 v = *(const uint4*)(src + c);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
        float f[8];
#pragma unroll
        for (int e = 0; e < 4; ++e) { f[2 * e] = bf16_bits_to_f32(w[e] & 0xffffu); f[2 * e + 1] = bf16_bits_to_f32(w[e] >> 16); }
        *(float4*)(dst + c) = make_float4(f[0], f[1], f[2], f[3]);
        *(float4*)(dst + c + 4) = make_float4(f[4], f[5], f[6], f[7]);
      }
    } else {
      for (int c = lane * 4; c < n; c += 128) *(float4*)(dst + c) = *(const float4*)((const float*)src + c);
    }
    return;
  }
  for (int c = lane; c < G * dimp; c += 32) {
    const int g = c / dimp, d = c - g * dimp;
    dst[c] = d < dim ? dt<T>::ld(src, (size_t)g * dim + d) : 0.f;
  }
}

// Scores of all heads against the keys u0 .. u0 + nk of the list -> ss[H][kchunk] (-inf past nk).  ks is scratch.
template <typename T>
__device__ __forceinline__ void wa_scores(const WaParams& P, const WaRange& r, int b, int u0, int nk, const float* qs, float* ks,
                                          float* ss) {
  const int GD = P.G * P.dim;
  const T* kc = (const T*)P.kc;
  const int S = P.keep + P.ring;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int jj = warp; jj < nk; jj += WA_THREADS / 32)       // a warp per key row: one slot computation, wide coalesced loads
    wa_row_to_smem<T>(ks + jj * P.kpitch, kc + ((size_t)b * S + wa_slot(P, wa_key(r, u0 + jj))) * GD, P.G, P.dim, P.dimp, lane);
  __syncthreads();
  const int hg = P.H / P.G;
  for (int idx = threadIdx.x; idx < P.H * P.kchunk; idx += WA_THREADS) {
    const int h = idx / P.kchunk, jj = idx - h * P.kchunk;
    float s = -INFINITY;
    if (jj < nk) {
      const float4* q4 = (const float4*)(qs + h * P.dimp);
      const float4* k4 = (const float4*)(ks + jj * P.kpitch + (h / hg) * P.dimp);
      float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
      for (int d = 0; d < P.dimp / 4; ++d) {
        const float4 qv = q4[d], kv = k4[d];
        a0 += qv.x * kv.x; a1 += qv.y * kv.y; a2 += qv.z * kv.z; a3 += qv.w * kv.w;
      }
      s = ((a0 + a1) + (a2 + a3)) * P.scale;
      if (P.cap > 0.f) s = P.cap * tanhf(s / P.cap);
      const int dist = r.i - wa_key(r, u0 + jj);
      s -= P.r1[h] * log1pf(P.r2[h] * (float)dist);
    }
    ss[h * P.kchunk + jj] = s;
  }
  __syncthreads();
}

template <typename T>
__device__ __forceinline__ void wa_load_q(const WaParams& P, int m, float* qs) {
  const T* q = (const T*)P.q;
  for (int idx = threadIdx.x; idx < P.H * P.dimp; idx += WA_THREADS) {
    const int h = idx / P.dimp, d = idx - h * P.dimp;
    qs[idx] = d < P.dim ? dt<T>::ld(q, (size_t)m * P.q_stride + h * P.dim + d) : 0.f;
  }
}

// shared memory: qs[H * dimp] | ss[H * kchunk] | pm[H * kchunk] | mh[H up to 4] | lh[H up to 4] | kv[kchunk * max(kpitch, vpitch)]
template <typename T>
__global__ void __launch_bounds__(WA_THREADS) window_attn_stats_kernel(WaParams P) {
  extern __shared__ __align__(16) float wa_sm[];
  float* qs = wa_sm;
  float* ss = qs + P.H * P.dimp;
  float* pm = ss + P.H * P.kchunk;
  float* mh = pm + P.H * P.kchunk;
  float* lh = mh + ((P.H + 3) / 4) * 4;     // every region starts on a 16-byte boundary
  float* kv = lh + ((P.H + 3) / 4) * 4;
  const int m = blockIdx.x, split = blockIdx.y;
  const int b = m / P.T, t = m - b * P.T;
  const WaRange r = wa_range(P, P.pos_ids[t], split);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  wa_load_q<T>(P, m, qs);
  for (int h = threadIdx.x; h < P.H; h += WA_THREADS) { mh[h] = -INFINITY; lh[h] = 0.f; }
  __syncthreads();
  for (int u0 = r.u0; u0 < r.u1; u0 += P.kchunk) {
    const int nk = min(P.kchunk, r.u1 - u0);
    wa_scores<T>(P, r, b, u0, nk, qs, kv, ss);
    for (int h = warp; h < P.H; h += WA_THREADS / 32) {
      float mx = -INFINITY;
      for (int jj = lane; jj < nk; jj += 32) mx = fmaxf(mx, ss[h * P.kchunk + jj]);
      mx = warp_max(mx);
      const float mo = mh[h], mn = fmaxf(mo, mx);
      float sum = 0.f;
      for (int jj = lane; jj < nk; jj += 32) sum += expf(ss[h * P.kchunk + jj] - mn);
      sum = warp_sum(sum);
      if (lane == 0) {
        lh[h] = lh[h] * (mo == -INFINITY ? 0.f : expf(mo - mn)) + sum;
        mh[h] = mn;
      }
    }
    __syncthreads();
  }
  float* out = P.stats + (((size_t)split * P.B * P.T + m) * P.H) * 2;
  for (int h = threadIdx.x; h < P.H; h += WA_THREADS) { out[2 * h] = mh[h]; out[2 * h + 1] = lh[h]; }
}

template <typename T>
__global__ void __launch_bounds__(WA_THREADS) window_attn_out_kernel(WaParams P) {
  extern __shared__ __align__(16) float wa_sm[];
  float* qs = wa_sm;
  float* ss = qs + P.H * P.dimp;
  float* pm = ss + P.H * P.kchunk;
  float* mh = pm + P.H * P.kchunk;
  float* lh = mh + ((P.H + 3) / 4) * 4;     // every region starts on a 16-byte boundary
  float* kv = lh + ((P.H + 3) / 4) * 4;
  const int m = blockIdx.x, split = blockIdx.y;
  const int M = P.B * P.T;
  const int b = m / P.T, t = m - b * P.T;
  const WaRange r = wa_range(P, P.pos_ids[t], split);
  const T* vc = (const T*)P.vc;
  const int S = P.keep + P.ring, GV = P.G * P.vdim, hg = P.H / P.G;
  wa_load_q<T>(P, m, qs);
  // every split's maximum and sum -> the query's own (merged in split order)
  for (int h = threadIdx.x; h < P.H; h += WA_THREADS) {
    float mx = -INFINITY;
    for (int s = 0; s < P.splits; ++s) mx = fmaxf(mx, P.stats[(((size_t)s * M + m) * P.H + h) * 2]);
    float l = 0.f;
    for (int s = 0; s < P.splits; ++s) {
      const float* e = P.stats + (((size_t)s * M + m) * P.H + h) * 2;
      if (e[1] > 0.f) l += e[1] * expf(e[0] - mx);
    }
    mh[h] = mx;
    lh[h] = 1.f / l;
  }
  __syncthreads();
  const int vq = (P.vdim + 3) / 4;                    // column quads per head
  const int items = P.H * vq;
  for (int base = 0; base < items; base += WA_THREADS * WA_ACC) {
    float4 acc[WA_ACC];
#pragma unroll
    for (int a = 0; a < WA_ACC; ++a) acc[a] = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int u0 = r.u0; u0 < r.u1; u0 += P.kchunk) {
      const int nk = min(P.kchunk, r.u1 - u0);
      wa_scores<T>(P, r, b, u0, nk, qs, kv, ss);
      for (int idx = threadIdx.x; idx < P.H * P.kchunk; idx += WA_THREADS) {
        const int h = idx / P.kchunk, jj = idx - h * P.kchunk;
        ss[idx] = jj < nk ? expf(ss[idx] - mh[h]) * lh[h] : 0.f;
      }
      // the values of this chunk (the keys are done with)
      for (int jj = (threadIdx.x >> 5); jj < nk; jj += WA_THREADS / 32)
        wa_row_to_smem<T>(kv + jj * P.vpitch, vc + ((size_t)b * S + wa_slot(P, wa_key(r, u0 + jj))) * GV, P.G, P.vdim, vq * 4,
                          threadIdx.x & 31);
      __syncthreads();
      for (int idx = threadIdx.x; idx < P.H * P.kchunk; idx += WA_THREADS) {
        const int h = idx / P.kchunk, jj = idx - h * P.kchunk;
        float v = 0.f;
        for (int g = 0; g < P.H; ++g) v += P.talk[h * P.H + g] * ss[g * P.kchunk + jj];
        pm[idx] = v;
      }
      __syncthreads();
#pragma unroll
      for (int a = 0; a < WA_ACC; ++a) {
        const int it = base + a * WA_THREADS + threadIdx.x;
        if (it < items) {
          const int h = it / vq, c4 = it - h * vq;
          const float* pw = pm + h * P.kchunk;
          const float* vv = kv + (h / hg) * (vq * 4) + c4 * 4;
          float4 s = acc[a];
          for (int jj = 0; jj < nk; ++jj) {
            const float w = pw[jj];
            const float4 x = *(const float4*)(vv + jj * P.vpitch);
            s.x += w * x.x; s.y += w * x.y; s.z += w * x.z; s.w += w * x.w;
          }
          acc[a] = s;
        }
      }
      __syncthreads();
    }
    float* out = P.part + ((size_t)split * M + m) * ((size_t)P.H * P.vdim);
#pragma unroll
    for (int a = 0; a < WA_ACC; ++a) {
      const int it = base + a * WA_THREADS + threadIdx.x;
      if (it < items) {
        const int h = it / vq, c4 = it - h * vq;
        const float vals[4] = {acc[a].x, acc[a].y, acc[a].z, acc[a].w};
        for (int e = 0; e < 4; ++e)
          if (c4 * 4 + e < P.vdim) out[h * P.vdim + c4 * 4 + e] = vals[e];
      }
    }
  }
}

// y[m][h * vdim + c] = sigmoid(gate[m][h]) * sum_s part[s][m][h * vdim + c]   (the parts summed in split order)
template <typename T>
__global__ void window_attn_finish_kernel(const float* __restrict__ part, int splits, const T* __restrict__ gate, int gate_stride,
                                          T* __restrict__ y, int M, int H, int vdim) {
  const int m = blockIdx.x;
  const int HV = H * vdim;
  const int i = blockIdx.y * blockDim.x + threadIdx.x;
  if (i >= HV) return;
  const float* src = part + (size_t)m * HV + i;
  const size_t step = (size_t)M * HV;
  float s = 0.f;
  int k = 0;
  for (; k + 8 <= splits; k += 8) {          // eight independent loads in flight, added in order
    float v[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] = src[(size_t)(k + e) * step];
#pragma unroll
    for (int e = 0; e < 8; ++e) s += v[e];
  }
  for (; k < splits; ++k) s += src[(size_t)k * step];
  if (gate) s *= 1.f / (1.f + expf(-dt<T>::ld(gate, (size_t)m * gate_stride + i / vdim)));
  dt<T>::st(y, (size_t)m * HV + i, s);
}

// Append the step's key and value rows (column slices of projection outputs) to the kept-tokens + ring cache.
template <typename T>
__global__ void sink_ring_append_kernel(const T* __restrict__ k, int k_stride, const T* __restrict__ v, int v_stride,
                                        const int32_t* __restrict__ pos_ids, T* __restrict__ kc, T* __restrict__ vc, int Tn,
                                        int kcols, int vcols, int keep, int ring) {
  const int m = blockIdx.x;
  const int b = m / Tn, t = m - b * Tn;
  const int j = pos_ids[t];
  const int slot = j < keep ? j : keep + (j - keep) % ring;
  const size_t row = (size_t)b * (keep + ring) + slot;
  for (int i = threadIdx.x; i < kcols; i += blockDim.x) kc[row * kcols + i] = k[(size_t)m * k_stride + i];
  for (int i = threadIdx.x; i < vcols; i += blockDim.x) vc[row * vcols + i] = v[(size_t)m * v_stride + i];
}

// ---- tensor-core form for prompts (bf16, mma.sync m16n8k16, fp32 accumulation) ---------------------------------------
// One block = 16 consecutive queries of one sequence x ALL heads, 16 warps.  The keys the tile can see (kept tokens, then
// the window of the whole tile) are walked in chunks of 32 rows staged in shared memory with cp.async, twice:
//   sweep 1: S = Q K^T per head (a warp owns heads w, w + 16, ..), cap / distance penalty / mask, running maximum and sum
//            of every (head, query) in registers;
//   sweep 2: S again, w = exp(S - max) / sum -> Ps[head][query][key] (bf16); the mix over heads as one more product,
//            Pm[h][(q, j)] = sum_g talk[h][g] Ps[g][(q, j)] (A = talk, B = Ps); then O_h += Pm_h V_g(h) per head.
// Heads beyond 16 take sweep 2 in rounds of 16 output heads.  The gate and the store are the epilogue.
constexpr int WM_WARPS = 16, WM_THREADS = WM_WARPS * 32, WM_Q = 16, WM_KC = 32, WM_PP = WM_KC + 8;
constexpr int WM_DK_MAX = 8, WM_VT_MAX = 16;     // dim <= 128, vdim <= 128

__device__ __forceinline__ void wm_cp_async16(void* smem, const void* gmem, bool valid) {
  const int n = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(smem)), "l"(gmem), "r"(n) : "memory");
}
__device__ __forceinline__ void wm_ldmatrix_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void wm_ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ uint32_t wm_pack(float lo, float hi) {
  return (uint32_t)f32_to_bf16_bits(lo) | ((uint32_t)f32_to_bf16_bits(hi) << 16);
}

struct WmTile { int b, t0, rows, i_first, i_last, ns, w0, n_list; };

__device__ __forceinline__ int wm_key(const WmTile& tl, int u) { return u < tl.ns ? u : tl.w0 + (u - tl.ns); }

// A chunk of the window part that lies before every query of a full tile and inside every query's window
__device__ __forceinline__ bool wm_interior(const WaParams& P, const WmTile& tl, int u0, int jf) {
  return tl.rows == WM_Q && tl.i_last - tl.i_first == WM_Q - 1 && u0 >= tl.ns && u0 + WM_KC <= tl.n_list &&
         jf + WM_KC - 1 <= tl.i_first && tl.i_last - jf < P.window;
}

// A fragments of one head's 16 x dim query tile, straight from the projection's rows
__device__ __forceinline__ void wm_load_q(const WaParams& P, const WmTile& tl, int h, int lane, uint32_t (&qf)[WM_DK_MAX][4]) {
  const __nv_bfloat16* q = (const __nv_bfloat16*)P.q;
  const int r0 = lane >> 2, c0 = (lane & 3) * 2;
  const int dk = P.dim / 16;
#pragma unroll
  for (int ks = 0; ks < WM_DK_MAX; ++ks) {
    if (ks < dk) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int row = r0 + (e & 1) * 8, col = ks * 16 + c0 + (e >> 1) * 8;
        uint32_t v = 0u;
        if (row < tl.rows) v = *(const uint32_t*)(q + ((size_t)tl.b * P.T + tl.t0 + row) * P.q_stride + h * P.dim + col);
        qf[ks][e] = v;
      }
    }
  }
}

// K (and V) rows of one chunk of the key list -> shared memory; rows past the list are zero-filled
__device__ __forceinline__ void wm_stage(const WaParams& P, const WmTile& tl, int u0, __nv_bfloat16* Ks, int kpitch,
                                         __nv_bfloat16* Vs, int vpitch, bool with_v) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int S = P.keep + P.ring, GD = P.G * P.dim, GV = P.G * P.vdim;
  const __nv_bfloat16* kc = (const __nv_bfloat16*)P.kc;
  const __nv_bfloat16* vc = (const __nv_bfloat16*)P.vc;
  for (int jj = warp; jj < WM_KC; jj += WM_WARPS) {
    const bool ok = u0 + jj < tl.n_list;
    const size_t row = (size_t)tl.b * S + (ok ? wa_slot(P, wm_key(tl, u0 + jj)) : 0);
    for (int c = lane; c < GD / 8; c += 32) wm_cp_async16(Ks + jj * kpitch + c * 8, kc + row * GD + c * 8, ok);
    if (with_v)
      for (int c = lane; c < GV / 8; c += 32) wm_cp_async16(Vs + jj * vpitch + c * 8, vc + row * GV + c * 8, ok);
  }
  asm volatile("cp.async.commit_group;" ::: "memory");
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncthreads();
}

// S[16 x 32] of head h against the staged chunk, then cap, distance penalty and mask (-inf where not visible)
// interior: every key of the chunk (positions jf .. jf + 31) is visible to every query of the tile - no mask to evaluate
__device__ __forceinline__ void wm_scores(const WaParams& P, const WmTile& tl, int u0, int h, int lane, const uint32_t (&qf)[WM_DK_MAX][4],
                                          const __nv_bfloat16* Ks, int kpitch, const int (&qpos)[2], bool interior, int jf,
                                          float (&s)[4][4]) {
  const int g = h / (P.H / P.G), dk = P.dim / 16;
#pragma unroll
  for (int nt = 0; nt < 4; ++nt)
#pragma unroll
    for (int e = 0; e < 4; ++e) s[nt][e] = 0.f;
#pragma unroll
  for (int ks = 0; ks < WM_DK_MAX; ++ks) {
    if (ks < dk) {
#pragma unroll
      for (int np = 0; np < 2; ++np) {
        uint32_t bf[4];
        wm_ldmatrix_x4(bf, Ks + (np * 16 + (lane & 7) + (lane >> 4) * 8) * kpitch + g * P.dim + ks * 16 + ((lane >> 3) & 1) * 8);
        mma_bf16_16816(s[2 * np], qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], bf[0], bf[1]);
        mma_bf16_16816(s[2 * np + 1], qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], bf[2], bf[3]);
      }
    }
  }
  const float r1 = P.r1[h], r2 = P.r2[h];
  const float inv_cap = P.cap > 0.f ? 1.f / P.cap : 0.f;
#pragma unroll
  for (int nt = 0; nt < 4; ++nt)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int col = nt * 8 + (lane & 3) * 2 + (e & 1);
      const int u = u0 + col;
      const int i = qpos[e >> 1];
      float v = -INFINITY;
      if (interior || (u < tl.n_list && i >= 0)) {
        const int j = interior ? jf + col : wm_key(tl, u);
        if (interior || (j <= i && (i - j < P.window || j < P.keep))) {
          v = s[nt][e] * P.scale;
          if (P.cap > 0.f) {                                        // cap * tanh(v / cap), tanh(x) = 1 - 2 / (exp(2x) + 1)
            const float ex = __expf(2.f * v * inv_cap);
            v = P.cap * (1.f - __fdividef(2.f, ex + 1.f));
          }
          v -= r1 * __logf(1.f + r2 * (float)(i - j));
        }
      }
      s[nt][e] = v;
    }
}

template <int HPW>
__global__ void __launch_bounds__(WM_THREADS, 1) window_attn_mma_kernel(WaParams P, const __nv_bfloat16* __restrict__ gate,
                                                                     int gate_stride, __nv_bfloat16* __restrict__ y) {
  extern __shared__ __align__(16) unsigned char wm_smem[];
  const int Hp = (P.H + 15) / 16 * 16;
  const int kpitch = P.G * P.dim + 8, vpitch = P.G * P.vdim + 8;
  __nv_bfloat16* Ks = (__nv_bfloat16*)wm_smem;                       // [32][kpitch]
  __nv_bfloat16* Vs = Ks + WM_KC * kpitch;                           // [32][vpitch]
  __nv_bfloat16* Ps = Vs + WM_KC * vpitch;                           // [Hp][16][40]
  __nv_bfloat16* Pm = Ps + Hp * WM_Q * WM_PP;                        // [Hp][16][40]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int tiles_per_seq = (P.T + WM_Q - 1) / WM_Q;
  WmTile tl;
  tl.b = blockIdx.x / tiles_per_seq;
  tl.t0 = (blockIdx.x - tl.b * tiles_per_seq) * WM_Q;
  tl.rows = min(WM_Q, P.T - tl.t0);
  tl.i_first = P.pos_ids[tl.t0];
  tl.i_last = P.pos_ids[tl.t0 + tl.rows - 1];
  tl.ns = min(P.keep, tl.i_last + 1);
  tl.w0 = max(P.keep, tl.i_first - P.window + 1);
  tl.n_list = tl.ns + max(0, tl.i_last - tl.w0 + 1);
  int qpos[2];
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    const int row = (lane >> 2) + e * 8;
    qpos[e] = row < tl.rows ? P.pos_ids[tl.t0 + row] : -1;
  }
  for (int idx = threadIdx.x; idx < Hp * WM_Q * WM_PP; idx += WM_THREADS) Ps[idx] = __float2bfloat16_rn(0.f);   // rows of heads past H stay zero

  uint32_t qf[HPW][WM_DK_MAX][4];          // the warp's query fragments stay in registers (spilled where they do not fit)
#pragma unroll
  for (int hs = 0; hs < HPW; ++hs)
    if (warp + hs * WM_WARPS < P.H) wm_load_q(P, tl, warp + hs * WM_WARPS, lane, qf[hs]);
  float mrun[HPW][2], lrun[HPW][2];
#pragma unroll
  for (int hs = 0; hs < HPW; ++hs)
#pragma unroll
    for (int e = 0; e < 2; ++e) { mrun[hs][e] = -INFINITY; lrun[hs][e] = 0.f; }

  // ---- sweep 1: maximum and sum of every (head, query)
  for (int u0 = 0; u0 < tl.n_list; u0 += WM_KC) {
    wm_stage(P, tl, u0, Ks, kpitch, Vs, vpitch, false);
    const int jf = wm_key(tl, u0);
    const bool interior = wm_interior(P, tl, u0, jf);
#pragma unroll
    for (int hs = 0; hs < HPW; ++hs) {
      const int h = warp + hs * WM_WARPS;
      if (h < P.H) {
        float s[4][4];
        wm_scores(P, tl, u0, h, lane, qf[hs], Ks, kpitch, qpos, interior, jf, s);
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          float mx = -INFINITY;
#pragma unroll
          for (int nt = 0; nt < 4; ++nt) mx = fmaxf(mx, fmaxf(s[nt][2 * e], s[nt][2 * e + 1]));
          const float mn = fmaxf(mrun[hs][e], mx);
          if (mn > -INFINITY) {
            float sum = 0.f;
#pragma unroll
            for (int nt = 0; nt < 4; ++nt) sum += __expf(s[nt][2 * e] - mn) + __expf(s[nt][2 * e + 1] - mn);
            lrun[hs][e] = lrun[hs][e] * (mrun[hs][e] == -INFINITY ? 0.f : __expf(mrun[hs][e] - mn)) + sum;
            mrun[hs][e] = mn;
          }
        }
      }
    }
    __syncthreads();
  }
  // the four lanes of a row hold parts of it: merge
#pragma unroll
  for (int hs = 0; hs < HPW; ++hs)
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      float m = mrun[hs][e], l = lrun[hs][e];
#pragma unroll
      for (int o = 1; o <= 2; o <<= 1) {
        const float mo = __shfl_xor_sync(0xffffffffu, m, o), lo = __shfl_xor_sync(0xffffffffu, l, o);
        const float mn = fmaxf(m, mo);
        l = (m == -INFINITY ? 0.f : l * __expf(m - mn)) + (mo == -INFINITY ? 0.f : lo * __expf(mo - mn));
        m = mn;
      }
      mrun[hs][e] = m;
      lrun[hs][e] = l > 0.f ? 1.f / l : 0.f;
    }

  // ---- sweep 2: weights, their mix over heads, values; rounds of 16 output heads
  const int hg = P.H / P.G, vt = P.vdim / 8;
  for (int round = 0; round * WM_WARPS < P.H; ++round) {
    const int ho = round * WM_WARPS + warp;                         // the head whose output this warp accumulates
    float o[WM_VT_MAX][4];
#pragma unroll
    for (int nt = 0; nt < WM_VT_MAX; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) o[nt][e] = 0.f;
    for (int u0 = 0; u0 < tl.n_list; u0 += WM_KC) {
      wm_stage(P, tl, u0, Ks, kpitch, Vs, vpitch, true);
      const int jf = wm_key(tl, u0);
      const bool interior = wm_interior(P, tl, u0, jf);
#pragma unroll
      for (int hs = 0; hs < HPW; ++hs) {
        const int h = warp + hs * WM_WARPS;
        if (h < P.H) {
          float s[4][4];
          wm_scores(P, tl, u0, h, lane, qf[hs], Ks, kpitch, qpos, interior, jf, s);
#pragma unroll
          for (int nt = 0; nt < 4; ++nt)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const float m = mrun[hs][e], il = lrun[hs][e];
              const float p0 = s[nt][2 * e] == -INFINITY ? 0.f : __expf(s[nt][2 * e] - m) * il;
              const float p1 = s[nt][2 * e + 1] == -INFINITY ? 0.f : __expf(s[nt][2 * e + 1] - m) * il;
              *(uint32_t*)(Ps + (h * WM_Q + (lane >> 2) + e * 8) * WM_PP + nt * 8 + (lane & 3) * 2) = wm_pack(p0, p1);
            }
        }
      }
      __syncthreads();
      // mix: this warp takes query row `warp` (32 keys = 4 column tiles) for every output head
      for (int mt = 0; mt < Hp / 16; ++mt) {
        float c[4][4];
#pragma unroll
        for (int nt = 0; nt < 4; ++nt)
#pragma unroll
          for (int e = 0; e < 4; ++e) c[nt][e] = 0.f;
        for (int kt = 0; kt < Hp / 16; ++kt) {
          uint32_t a[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int hr = mt * 16 + (lane >> 2) + (e & 1) * 8, gc = kt * 16 + (lane & 3) * 2 + (e >> 1) * 8;
            const float t0 = (hr < P.H && gc < P.H) ? P.talk[hr * P.H + gc] : 0.f;
            const float t1 = (hr < P.H && gc + 1 < P.H) ? P.talk[hr * P.H + gc + 1] : 0.f;
            a[e] = wm_pack(t0, t1);
          }
#pragma unroll
          for (int np = 0; np < 2; ++np) {
            uint32_t bf[4];
            wm_ldmatrix_x4_trans(bf, Ps + ((kt * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * WM_Q + warp) * WM_PP + np * 16 + (lane >> 4) * 8);
            mma_bf16_16816(c[2 * np], a[0], a[1], a[2], a[3], bf[0], bf[1]);
            mma_bf16_16816(c[2 * np + 1], a[0], a[1], a[2], a[3], bf[2], bf[3]);
          }
        }
#pragma unroll
        for (int nt = 0; nt < 4; ++nt)
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int hr = mt * 16 + (lane >> 2) + e * 8;
            *(uint32_t*)(Pm + (hr * WM_Q + warp) * WM_PP + nt * 8 + (lane & 3) * 2) = wm_pack(c[nt][2 * e], c[nt][2 * e + 1]);
          }
      }
      __syncthreads();
      if (ho < P.H) {
        const int g = ho / hg;
#pragma unroll
        for (int ks = 0; ks < WM_KC / 16; ++ks) {
          uint32_t af[4];
          wm_ldmatrix_x4(af, Pm + (ho * WM_Q + (lane & 15)) * WM_PP + ks * 16 + (lane >> 4) * 8);
#pragma unroll
          for (int jp = 0; jp < WM_VT_MAX / 2; ++jp) {
            if (2 * jp < vt) {
              uint32_t bf[4];
              wm_ldmatrix_x4_trans(bf, Vs + (ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * vpitch + g * P.vdim + jp * 16 + (lane >> 4) * 8);
              mma_bf16_16816(o[2 * jp], af[0], af[1], af[2], af[3], bf[0], bf[1]);
              mma_bf16_16816(o[2 * jp + 1], af[0], af[1], af[2], af[3], bf[2], bf[3]);
            }
          }
        }
      }
      __syncthreads();
    }
    if (ho < P.H) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int row = (lane >> 2) + e * 8;
        if (row < tl.rows) {
          const size_t m = (size_t)tl.b * P.T + tl.t0 + row;
          float gt = 1.f;
          if (gate) gt = 1.f / (1.f + __expf(-__bfloat162float(gate[m * gate_stride + ho])));
#pragma unroll
          for (int nt = 0; nt < WM_VT_MAX; ++nt)
            if (nt < vt)
              *(uint32_t*)(y + m * ((size_t)P.H * P.vdim) + (size_t)ho * P.vdim + nt * 8 + (lane & 3) * 2) =
                  wm_pack(o[nt][2 * e] * gt, o[nt][2 * e + 1] * gt);
        }
      }
    }
  }
}

// whether the tensor-core form takes a step, and its shared memory
static bool wm_takes(const WaParams& P, int dtype, size_t* smem) {
  if (dtype != LL_BF16 || P.T < 8 || P.dim % 16 || P.vdim % 16 || P.dim > 16 * WM_DK_MAX || P.vdim > 8 * WM_VT_MAX || P.H > 4 * WM_WARPS)
    return false;
  if (P.q_stride % 2 || (((uintptr_t)P.q) & 3) || (((uintptr_t)P.kc) & 15) || (((uintptr_t)P.vc) & 15)) return false;
  const int Hp = (P.H + 15) / 16 * 16;
  *smem = sizeof(__nv_bfloat16) * ((size_t)WM_KC * (P.G * P.dim + 8) + (size_t)WM_KC * (P.G * P.vdim + 8) + 2 * (size_t)Hp * WM_Q * WM_PP);
  return *smem <= 220 * 1024;
}

template <int HPW>
static int wm_launch(const WaParams& P, const void* gate, int gate_stride, void* y, size_t smem, cudaStream_t st) {
  static bool once = false;
  if (!once) {
    LL_CUDA(cudaFuncSetAttribute(window_attn_mma_kernel<HPW>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024));
    once = true;
  }
  const int tiles = P.B * ((P.T + WM_Q - 1) / WM_Q);
  window_attn_mma_kernel<HPW><<<tiles, WM_THREADS, smem, st>>>(P, (const __nv_bfloat16*)gate, gate_stride, (__nv_bfloat16*)y);
  LL_LAUNCH_OK("window_attn_mma_kernel");
  return LL_OK;
}

static void wa_layout(WaParams& P, size_t budget, size_t* smem) {
  P.dimp = (P.dim + 3) / 4 * 4;
  int kq = P.G * P.dimp / 4;
  if (kq % 2 == 0) kq += 1;                 // an odd number of 16-byte units per row: conflict-free 128-bit loads
  P.kpitch = kq * 4;
  P.vpitch = P.G * ((P.vdim + 3) / 4 * 4);
  const size_t fixed = (size_t)P.H * P.dimp + 2 * ((P.H + 3) / 4 * 4);
  int kc = 64;
  for (;;) {
    *smem = sizeof(float) * (fixed + 2 * (size_t)P.H * kc + (size_t)kc * (size_t)(P.kpitch > P.vpitch ? P.kpitch : P.vpitch));
    if (*smem <= budget || kc == 4) break;
    kc /= 2;
  }
  P.kchunk = kc;
}

template <typename T>
static int window_attn_run(WaParams& P, const void* gate, int gate_stride, void* y, int dtype, cudaStream_t st) {
  size_t smem = 0;
  if (wm_takes(P, dtype, &smem)) {       // prompts in bfloat16: tensor cores (the splits are for few queries)
    if (P.H <= WM_WARPS) return wm_launch<1>(P, gate, gate_stride, y, smem, st);
    if (P.H <= 2 * WM_WARPS) return wm_launch<2>(P, gate, gate_stride, y, smem, st);
    return wm_launch<4>(P, gate, gate_stride, y, smem, st);
  }
  // many queries: two blocks per SM; few (decoding): one chunk as long as shared memory allows, one per split if possible
  wa_layout(P, (size_t)P.B * P.T * P.splits <= 2 * (size_t)sm_count() ? 200 * 1024 : 96 * 1024, &smem);
  if (smem > 220 * 1024) {
    set_error("window_attn: %d heads of %d do not fit shared memory", P.H, P.dim);
    return LL_ERR_UNSUPPORTED;
  }
  static bool once = false;
  if (!once) {
    LL_CUDA(cudaFuncSetAttribute(window_attn_stats_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024));
    LL_CUDA(cudaFuncSetAttribute(window_attn_out_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024));
    once = true;
  }
  const int M = P.B * P.T;
  dim3 grid(M, P.splits);
  window_attn_stats_kernel<T><<<grid, WA_THREADS, smem, st>>>(P);
  LL_LAUNCH_OK("window_attn_stats_kernel");
  window_attn_out_kernel<T><<<grid, WA_THREADS, smem, st>>>(P);
  LL_LAUNCH_OK("window_attn_out_kernel");
  window_attn_finish_kernel<T><<<dim3(M, (P.H * P.vdim + 127) / 128), 128, 0, st>>>(P.part, P.splits, (const T*)gate, gate_stride, (T*)y, M,
                                                                                     P.H, P.vdim);
  LL_LAUNCH_OK("window_attn_finish_kernel");
  return LL_OK;
}

}  // namespace llb

using namespace llb;

extern "C" {

size_t ll_window_attn_scratch_bytes(int M, int H, int vdim, int splits) {
  return sizeof(float) * (size_t)splits * M * ((size_t)H * 2 + (size_t)H * vdim);
}

int ll_sink_ring_append(const void* k, int k_stride, const void* v, int v_stride, int dtype, const int32_t* pos_ids, void* kc,
                        void* vc, int B, int T, int kcols, int vcols, int keep, int ring, ll_stream stream) {
  LL_CHECK_ARG(k && v && pos_ids && kc && vc, "sink_ring_append: null pointer");
  LL_CHECK_ARG(B >= 0 && T >= 0 && kcols > 0 && vcols > 0 && keep >= 0 && ring > 0 && k_stride >= kcols && v_stride >= vcols,
               "bad sink_ring_append arguments");
  if (B * T == 0) return LL_OK;
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == LL_F32)
    sink_ring_append_kernel<float><<<B * T, 128, 0, st>>>((const float*)k, k_stride, (const float*)v, v_stride, pos_ids, (float*)kc,
                                                         (float*)vc, T, kcols, vcols, keep, ring);
  else if (dtype == LL_BF16)
    sink_ring_append_kernel<__nv_bfloat16><<<B * T, 128, 0, st>>>((const __nv_bfloat16*)k, k_stride, (const __nv_bfloat16*)v, v_stride,
                                                                 pos_ids, (__nv_bfloat16*)kc, (__nv_bfloat16*)vc, T, kcols, vcols, keep,
                                                                 ring);
  else {
    set_error("sink_ring_append: unsupported dtype %d", dtype);
    return LL_ERR_UNSUPPORTED;
  }
  LL_LAUNCH_OK("sink_ring_append_kernel");
  return LL_OK;
}

int ll_window_attn(const void* q, int q_stride, const void* gate, int gate_stride, const void* kc, const void* vc, int dtype,
                   const int32_t* pos_ids, const float* r1, const float* r2, const float* talk, float scale, float softcap, int B,
                   int T, int H, int G, int dim, int vdim, int window, int keep, int ring, int splits, float* scratch, void* y,
                   ll_stream stream) {
  LL_CHECK_ARG(q && kc && vc && pos_ids && r1 && r2 && talk && scratch && y, "window_attn: null pointer");
  LL_CHECK_ARG(B >= 0 && T >= 0 && H > 0 && G > 0 && H % G == 0 && dim > 0 && vdim > 0 && window > 0 && keep >= 0 && ring > 0 &&
                   splits >= 1 && q_stride >= H * dim,
               "bad window_attn arguments");
  if (B * T == 0) return LL_OK;
  WaParams P{};
  P.q = q; P.q_stride = q_stride; P.kc = kc; P.vc = vc; P.pos_ids = pos_ids;
  P.r1 = r1; P.r2 = r2; P.talk = talk; P.scale = scale; P.cap = softcap;
  P.B = B; P.T = T; P.H = H; P.G = G; P.dim = dim; P.vdim = vdim; P.window = window; P.keep = keep; P.ring = ring; P.splits = splits;
  P.stats = scratch;
  P.part = scratch + (size_t)splits * B * T * H * 2;
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == LL_F32) return window_attn_run<float>(P, gate, gate_stride, y, dtype, st);
  if (dtype == LL_BF16) return window_attn_run<__nv_bfloat16>(P, gate, gate_stride, y, dtype, st);
  set_error("window_attn: unsupported dtype %d", dtype);
  return LL_ERR_UNSUPPORTED;
}

}  // extern "C"
