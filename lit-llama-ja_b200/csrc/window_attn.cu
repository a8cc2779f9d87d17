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

// Scores of all heads against the keys u0 .. u0 + nk of the list -> ss[H][kchunk] (-inf past nk).  ks is scratch.
template <typename T>
__device__ __forceinline__ void wa_scores(const WaParams& P, const WaRange& r, int b, int u0, int nk, const float* qs, float* ks,
                                          float* ss) {
  const int GD = P.G * P.dim;
  const T* kc = (const T*)P.kc;
  const int S = P.keep + P.ring;
  for (int idx = threadIdx.x; idx < nk * P.G * P.dimp; idx += WA_THREADS) {
    const int jj = idx / (P.G * P.dimp), rem = idx - jj * (P.G * P.dimp);
    const int g = rem / P.dimp, d = rem - g * P.dimp;
    float v = 0.f;
    if (d < P.dim) v = dt<T>::ld(kc, ((size_t)b * S + wa_slot(P, wa_key(r, u0 + jj))) * GD + g * P.dim + d);
    ks[jj * P.kpitch + rem] = v;
  }
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
      for (int idx = threadIdx.x; idx < nk * P.vpitch; idx += WA_THREADS) {
        const int jj = idx / P.vpitch, col = idx - jj * P.vpitch;
        const int g = col / (vq * 4), c = col - g * (vq * 4);
        kv[idx] = c < P.vdim ? dt<T>::ld(vc, ((size_t)b * S + wa_slot(P, wa_key(r, u0 + jj))) * GV + g * P.vdim + c) : 0.f;
      }
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

// y[m][h * vdim + c] = out_scale * sigmoid(gate[m][h]) * sum_s part[s][m][h * vdim + c]
template <typename T>
__global__ void window_attn_finish_kernel(const float* __restrict__ part, int splits, const T* __restrict__ gate, int gate_stride,
                                          T* __restrict__ y, int M, int H, int vdim) {
  const int m = blockIdx.x;
  const int HV = H * vdim;
  for (int i = threadIdx.x; i < HV; i += blockDim.x) {
    float s = 0.f;
    for (int k = 0; k < splits; ++k) s += part[((size_t)k * M + m) * HV + i];
    if (gate) s *= 1.f / (1.f + expf(-dt<T>::ld(gate, (size_t)m * gate_stride + i / vdim)));
    dt<T>::st(y, (size_t)m * HV + i, s);
  }
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
static int window_attn_run(WaParams& P, const void* gate, int gate_stride, void* y, cudaStream_t st) {
  size_t smem = 0;
  wa_layout(P, 96 * 1024, &smem);
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
  window_attn_finish_kernel<T><<<M, 256, 0, st>>>(P.part, P.splits, (const T*)gate, gate_stride, (T*)y, M, P.H, P.vdim);
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
  if (dtype == LL_F32) return window_attn_run<float>(P, gate, gate_stride, y, st);
  if (dtype == LL_BF16) return window_attn_run<__nv_bfloat16>(P, gate, gate_stride, y, st);
  set_error("window_attn: unsupported dtype %d", dtype);
  return LL_ERR_UNSUPPORTED;
}

}  // extern "C"
