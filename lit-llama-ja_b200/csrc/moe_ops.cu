// Mixture-of-experts feed-forward: fp32 router with top-k selection, the sort of (token, choice)
// pairs by expert entirely on the device (no host synchronisation: the step stays graph-capturable),
// a grouped GEMM over the sorted rows whose blocks find their expert from the device-side counts,
// and the weighted combination with an optional always-on shared expert.
//
//   route    z = W_r x + b (fp32), the `top` largest logits, weights = softmax over the chosen logits; or scores =
//            softmax over ALL experts with weights = chosen scores / (their sum + 1e-20); optionally only experts of the
//            `keep_groups` best of `n_groups` equal groups of neighbouring experts (a group's score: its largest) compete
//   permute  rows sorted by expert: perm[offsets[e] + rank] = token * top + choice
//   grouped  MODE_GLU : h[r][:] = glu(x[token(r)] . Wgu[e]^T)   (stacked [gate; up] weight; g s(alpha g) (u + shift), clamped)
//            MODE_DOWN: y[perm[r]][:] = h[r] . Wd[e]^T
//   combine  out[m] = sum_k w[m][k] * y[m * top + k]  (+ sigmoid(s[m]) * shared[m])
#include "common.cuh"

namespace llb {

constexpr int RT_TOK = 4;        // tokens per routing block
constexpr int RT_THREADS = 256;
constexpr int RT_EG = 4;         // experts a warp accumulates side by side

template <typename T>
__global__ void __launch_bounds__(RT_THREADS) moe_route_kernel(const T* __restrict__ x, const float* __restrict__ w_router,
                                                               const float* __restrict__ bias, int M, int dim, int X, int top,
                                                               int score_all, int n_groups, int keep_groups,
                                                               int32_t* __restrict__ expert_idx, float* __restrict__ expert_w,
                                                               int32_t* __restrict__ counts, int32_t* __restrict__ rank) {
  extern __shared__ float sm[];
  float* xs = sm;                      // [RT_TOK][dim]
  float* zs = xs + RT_TOK * dim;       // [RT_TOK][X]
  float* gms = zs + RT_TOK * X;        // [RT_TOK][n_groups] group maxima, then [RT_TOK][n_groups] "may compete" flags
  const int m0 = blockIdx.x * RT_TOK;
  const int nt = min(RT_TOK, M - m0);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  for (int idx = tid; idx < nt * dim; idx += RT_THREADS) xs[idx] = dt<T>::ld(x, (size_t)m0 * dim + idx);
  for (int idx = nt * dim + tid; idx < RT_TOK * dim; idx += RT_THREADS) xs[idx] = 0.f;
  __syncthreads();
  const bool vec4 = (dim % 4 == 0) && (((uintptr_t)w_router & 15) == 0);
  // RT_EG experts at a time per warp and four columns per step: 16 independent weight loads in flight per lane
  for (int e0 = warp * RT_EG; e0 < X; e0 += (RT_THREADS / 32) * RT_EG) {
    float a[RT_EG][RT_TOK];
#pragma unroll
    for (int g = 0; g < RT_EG; ++g)
#pragma unroll
      for (int t = 0; t < RT_TOK; ++t) a[g][t] = 0.f;
    if (vec4) {          // 16-byte weight loads, four steps unrolled: 16 independent loads in flight per lane
#pragma unroll 4
      for (int i4 = lane; i4 < dim / 4; i4 += 32) {
        float4 w[RT_EG];
#pragma unroll
        for (int g = 0; g < RT_EG; ++g) w[g] = ((const float4*)(w_router + (size_t)min(e0 + g, X - 1) * dim))[i4];
#pragma unroll
        for (int t = 0; t < RT_TOK; ++t) {
          const float4 xv = ((const float4*)(xs + t * dim))[i4];
#pragma unroll
          for (int g = 0; g < RT_EG; ++g) a[g][t] += w[g].x * xv.x + w[g].y * xv.y + w[g].z * xv.z + w[g].w * xv.w;
        }
      }
    } else {
#pragma unroll 4
      for (int i = lane; i < dim; i += 32) {
        float w[RT_EG];
#pragma unroll
        for (int g = 0; g < RT_EG; ++g) w[g] = w_router[(size_t)min(e0 + g, X - 1) * dim + i];
#pragma unroll
        for (int t = 0; t < RT_TOK; ++t) {
          const float xv = xs[t * dim + i];
#pragma unroll
          for (int g = 0; g < RT_EG; ++g) a[g][t] += w[g] * xv;
        }
      }
    }
#pragma unroll
    for (int g = 0; g < RT_EG; ++g)
#pragma unroll
      for (int t = 0; t < RT_TOK; ++t) {
        const float sum = warp_sum(a[g][t]);
        if (lane == 0 && e0 + g < X) zs[t * X + e0 + g] = sum + (bias ? bias[e0 + g] : 0.f);
      }
  }
  __syncthreads();
  if (warp < nt) {
    float* z = zs + warp * X;
    const int m = m0 + warp;
    float v0 = 0.f, denom = 0.f;
    float zmax = -INFINITY, zsum = 1.f;
    if (score_all) {                   // softmax over every expert, also those that cannot be chosen
      for (int e = lane; e < X; e += 32) zmax = fmaxf(zmax, z[e]);
      zmax = warp_max(zmax);
      float acc = 0.f;
      for (int e = lane; e < X; e += 32) acc += expf(z[e] - zmax);
      zsum = warp_sum(acc);
    }
    if (n_groups > 1 && keep_groups < n_groups) {
      float* gm = gms + warp * n_groups;
      float* ga = gms + RT_TOK * n_groups + warp * n_groups;
      const int gs = X / n_groups;
      for (int g = lane; g < n_groups; g += 32) {
        float mx = -INFINITY;
        for (int e = g * gs; e < (g + 1) * gs; ++e) mx = fmaxf(mx, z[e]);
        gm[g] = mx;
      }
      __syncwarp();
      for (int g = lane; g < n_groups; g += 32) {      // a group competes when fewer than keep_groups groups beat it
        int before = 0;
        for (int o = 0; o < n_groups; ++o) before += (gm[o] > gm[g] || (gm[o] == gm[g] && o < g)) ? 1 : 0;
        ga[g] = before < keep_groups ? 1.f : 0.f;
      }
      __syncwarp();
      for (int e = lane; e < X; e += 32)
        if (ga[e / gs] == 0.f) z[e] = -INFINITY;
      __syncwarp();
    }
    for (int k = 0; k < top; ++k) {
      float best = -INFINITY;
      int bi = 0x7fffffff;
      for (int e = lane; e < X; e += 32) {
        const float v = z[e];
        if (v > best || (v == best && e < bi)) { best = v; bi = e; }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
      }
      if (k == 0) v0 = best;
      const float p = score_all ? expf(best - zmax) / zsum : expf(best - v0);
      denom += p;
      if (lane == 0) {
        z[bi] = -INFINITY;
        expert_idx[(size_t)m * top + k] = bi;
        expert_w[(size_t)m * top + k] = p;                       // normalised below
        rank[(size_t)m * top + k] = atomicAdd(&counts[bi], 1);
      }
      __syncwarp();
    }
    __syncwarp();
    if (score_all) denom += 1e-20f;
    for (int k = lane; k < top; k += 32) expert_w[(size_t)m * top + k] /= denom;
  }
}

__global__ void moe_permute_kernel(const int32_t* __restrict__ expert_idx, const int32_t* __restrict__ rank,
                                   const int32_t* __restrict__ counts, int n_pairs, int X, int32_t* __restrict__ offsets,
                                   int32_t* __restrict__ perm) {
  extern __shared__ int32_t off[];   // [X + 1]
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int e = 0; e < X; ++e) { off[e] = acc; acc += counts[e]; }
    off[X] = acc;
  }
  __syncthreads();
  if (blockIdx.x == 0)
    for (int e = threadIdx.x; e <= X; e += blockDim.x) offsets[e] = off[e];
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n_pairs) perm[off[expert_idx[i]] + rank[i]] = i;
}

constexpr int GG_BN = 64, GG_BK = 16, GG_THREADS = 256;
enum { MODE_DOWN = 0, MODE_GLU = 1 };

// One block = a tile of 16*TM sorted rows of ONE expert x 64 output columns.  fp32 FMAs on operands
// converted from T (exact for bf16), fp32 accumulation.
template <typename T, int TM, int MODE>
__global__ void __launch_bounds__(GG_THREADS) moe_grouped_gemm_kernel(const T* __restrict__ a, int lda, const T* __restrict__ w,
                                                                      const int32_t* __restrict__ offsets,
                                                                      const int32_t* __restrict__ perm, int top, int X, int N,
                                                                      int K, float limit, float alpha, float shift, T* __restrict__ c, int ldc) {
  constexpr int BM = 16 * TM;
  constexpr int NB = MODE == MODE_GLU ? 2 : 1;
  __shared__ float As[GG_BK][BM + 1];
  __shared__ float Bs[NB][GG_BK][GG_BN + 1];
  __shared__ int32_t src_row[BM], dst_row[BM];
  __shared__ int s_tile[3];
  const int tid = threadIdx.x;
  if (tid < 32) grouped_tile_lookup(offsets, X, blockIdx.x, BM, s_tile);
  __syncthreads();
  if (s_tile[0] < 0) return;
  const int e = s_tile[0], r0 = s_tile[1], cnt = s_tile[2];
  const int n0 = blockIdx.y * GG_BN;
  if (tid < BM) {
    const int r = r0 + min(tid, cnt - 1);
    const int pr = perm[r];
    src_row[tid] = MODE == MODE_GLU ? pr / top : r;
    dst_row[tid] = MODE == MODE_GLU ? r : pr;
  }
  __syncthreads();
  const size_t rows_w = MODE == MODE_GLU ? 2 * (size_t)N : (size_t)N;   // rows of one expert's weight
  const T* we = w + (size_t)e * rows_w * K;
  const int tx = tid & 15, ty = tid >> 4;   // 16 x 16 threads: columns tx*4.., rows ty*TM..
  float acc[NB][TM][4];
#pragma unroll
  for (int b = 0; b < NB; ++b)
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[b][i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += GG_BK) {
    for (int idx = tid; idx < BM * GG_BK; idx += GG_THREADS) {
      const int r = idx / GG_BK, kk = idx - r * GG_BK;
      As[kk][r] = (k0 + kk < K) ? dt<T>::ld(a, (size_t)src_row[r] * lda + k0 + kk) : 0.f;
    }
    for (int idx = tid; idx < NB * GG_BN * GG_BK; idx += GG_THREADS) {
      const int b = idx / (GG_BN * GG_BK), rem = idx - b * GG_BN * GG_BK;
      const int n = rem / GG_BK, kk = rem - n * GG_BK;
      const int col = n0 + n;
      Bs[b][kk][n] = (col < N && k0 + kk < K) ? dt<T>::ld(we, ((size_t)b * N + col) * K + k0 + kk) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < GG_BK; ++kk) {
      float av[TM];
#pragma unroll
      for (int i = 0; i < TM; ++i) av[i] = As[kk][ty * TM + i];
#pragma unroll
      for (int b = 0; b < NB; ++b) {
        float bv[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) bv[j] = Bs[b][kk][tx * 4 + j];
#pragma unroll
        for (int i = 0; i < TM; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[b][i][j] += av[i] * bv[j];
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int r = ty * TM + i;
    if (r >= cnt) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int col = n0 + tx * 4 + j;
      if (col >= N) continue;
      float v;
      if (MODE == MODE_GLU) {
        const float g = fminf(acc[0][i][j], limit);
        const float u = fminf(fmaxf(acc[NB - 1][i][j], -limit), limit);
        v = g / (1.f + expf(-alpha * g)) * (u + shift);
      } else {
        v = acc[0][i][j];
      }
      dt<T>::st(c, (size_t)dst_row[r] * ldc + col, v);
    }
  }
}

// ---- bf16 tensor-core form of the same grouped GEMM (mma.sync m16n8k16, fp32 accumulation) ----
// 128 threads; a block = BM sorted rows of one expert x 64 output columns (x2 matrices for the GLU), K in steps of 64
// through a cp.async ring (two stages, four for the 16-row tiles of decoding).  Needs 16-byte aligned rows (K, lda multiples of 8); other shapes take the kernel above.
constexpr int GM_BN = 64, GM_BK = 64, GM_PITCH = GM_BK + 8, GM_THREADS = 128;
// stages of the operand ring: narrow row tiles (decoding: a few rows per expert, the weights are the traffic) keep more
// k-steps in flight per block
__host__ __device__ constexpr int gm_stages(int bm) { return bm <= 16 ? 4 : 2; }

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
  const int n = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(smem)), "l"(gmem), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N_>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N_) : "memory"); }
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}

template <int BM, int MODE>
__global__ void __launch_bounds__(GM_THREADS) moe_grouped_gemm_mma_kernel(
    const __nv_bfloat16* __restrict__ a, int lda, const __nv_bfloat16* __restrict__ w, const int32_t* __restrict__ offsets,
    const int32_t* __restrict__ perm, int top, int X, int N, int K, float limit, float alpha, float shift,
    __nv_bfloat16* __restrict__ c, int ldc) {
  constexpr int NB = MODE == MODE_GLU ? 2 : 1;
  constexpr int ST = gm_stages(BM);
  constexpr int WARPS_M = BM >= 32 ? 2 : 1, WARPS_N = 4 / WARPS_M;
  constexpr int WM = BM / WARPS_M, WN = GM_BN / WARPS_N, MT = WM / 16, NT = WN / 8;
  extern __shared__ __align__(16) unsigned char gm_smem[];
  __nv_bfloat16* As = (__nv_bfloat16*)gm_smem;                               // [ST][BM][PITCH]
  __nv_bfloat16* Bs = As + ST * BM * GM_PITCH;                               // [ST][NB][BN][PITCH]
  __shared__ int32_t src_row[BM], dst_row[BM];
  __shared__ int s_tile[3];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (warp == 0) grouped_tile_lookup(offsets, X, blockIdx.x, BM, s_tile);
  __syncthreads();
  if (s_tile[0] < 0) return;
  const int e = s_tile[0], r0 = s_tile[1], cnt = s_tile[2];
  const int n0 = blockIdx.y * GM_BN;
  for (int i = tid; i < BM; i += GM_THREADS) {
    const int r = r0 + min(i, cnt - 1);
    const int pr = perm[r];
    src_row[i] = MODE == MODE_GLU ? pr / top : r;
    dst_row[i] = MODE == MODE_GLU ? r : pr;
  }
  __syncthreads();
  const __nv_bfloat16* we = w + (size_t)e * NB * N * K;

  auto load_stage = [&](int stage, int k0) {
    __nv_bfloat16* as = As + stage * BM * GM_PITCH;
    for (int ch = tid; ch < BM * (GM_BK / 8); ch += GM_THREADS) {
      const int r = ch / (GM_BK / 8), kc = (ch % (GM_BK / 8)) * 8;
      const bool ok = r < cnt && k0 + kc < K;
      cp_async16(as + r * GM_PITCH + kc, a + (size_t)src_row[r] * lda + (ok ? k0 + kc : 0), ok);
    }
    __nv_bfloat16* bs = Bs + stage * NB * GM_BN * GM_PITCH;
    for (int ch = tid; ch < NB * GM_BN * (GM_BK / 8); ch += GM_THREADS) {
      const int b = ch / (GM_BN * (GM_BK / 8)), rem = ch % (GM_BN * (GM_BK / 8));
      const int n = rem / (GM_BK / 8), kc = (rem % (GM_BK / 8)) * 8;
      const bool ok = n0 + n < N && k0 + kc < K;
      cp_async16(bs + (b * GM_BN + n) * GM_PITCH + kc, we + ((size_t)b * N + (ok ? n0 + n : 0)) * K + (ok ? k0 + kc : 0), ok);
    }
    cp_async_commit();
  };

  float acc[NB][MT][NT][4];
#pragma unroll
  for (int b = 0; b < NB; ++b)
#pragma unroll
    for (int i = 0; i < MT; ++i)
#pragma unroll
      for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int q = 0; q < 4; ++q) acc[b][i][j][q] = 0.f;
  const int wm0 = (warp / WARPS_N) * WM, wn0 = (warp % WARPS_N) * WN;
  const int nk = (K + GM_BK - 1) / GM_BK;
  // a ring of ST stages: ST - 1 k-steps are in flight under the math of one (a group is committed every step, empty
  // past the end, so that "all but the newest ST - 1 groups" always means "this step's operands have landed")
#pragma unroll
  for (int s = 0; s < ST - 1; ++s) {
    if (s < nk) load_stage(s, s * GM_BK); else cp_async_commit();
  }
  for (int kt = 0; kt < nk; ++kt) {
    if (kt + ST - 1 < nk) load_stage((kt + ST - 1) % ST, (kt + ST - 1) * GM_BK); else cp_async_commit();
    cp_async_wait<ST - 1>();
    __syncthreads();
    const __nv_bfloat16* as = As + (kt % ST) * BM * GM_PITCH;
    const __nv_bfloat16* bs = Bs + (kt % ST) * NB * GM_BN * GM_PITCH;
#pragma unroll
    for (int ks = 0; ks < GM_BK / 16; ++ks) {
      uint32_t af[MT][4];
#pragma unroll
      for (int i = 0; i < MT; ++i) ldmatrix_x4(af[i], as + (wm0 + i * 16 + (lane & 15)) * GM_PITCH + ks * 16 + (lane >> 4) * 8);
#pragma unroll
      for (int b = 0; b < NB; ++b)
#pragma unroll
        for (int jp = 0; jp < NT / 2; ++jp) {
          uint32_t bf[4];
          ldmatrix_x4(bf, bs + (b * GM_BN + wn0 + jp * 16 + (lane & 7) + (lane >> 4) * 8) * GM_PITCH + ks * 16 + ((lane >> 3) & 1) * 8);
#pragma unroll
          for (int i = 0; i < MT; ++i) {
            mma_bf16_16816(acc[b][i][2 * jp], af[i][0], af[i][1], af[i][2], af[i][3], bf[0], bf[1]);
            mma_bf16_16816(acc[b][i][2 * jp + 1], af[i][0], af[i][1], af[i][2], af[i][3], bf[2], bf[3]);
          }
        }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < MT; ++i)
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int r = wm0 + i * 16 + (lane >> 2) + (q >> 1) * 8;
        const int col = n0 + wn0 + j * 8 + (lane & 3) * 2 + (q & 1);
        if (r >= cnt || col >= N) continue;
        float v;
        if (MODE == MODE_GLU) {
          const float g = fminf(acc[0][i][j][q], limit);
          const float u = fminf(fmaxf(acc[NB - 1][i][j][q], -limit), limit);
          v = g / (1.f + expf(-alpha * g)) * (u + shift);
        } else {
          v = acc[0][i][j][q];
        }
        c[(size_t)dst_row[r] * ldc + col] = __float2bfloat16_rn(v);
      }
}

template <int BM, int MODE>
static int launch_grouped_mma(const void* a, int lda, const void* w, const int32_t* offsets, const int32_t* perm, int top, int X, int N,
                              int K, float limit, float alpha, float shift, void* c, int ldc, int n_rows, cudaStream_t st) {
  constexpr int NB = MODE == MODE_GLU ? 2 : 1;
  const size_t smem = sizeof(__nv_bfloat16) * gm_stages(BM) * (BM + NB * GM_BN) * GM_PITCH;
  static bool once = false;
  if (!once) {
    LL_CUDA(cudaFuncSetAttribute(moe_grouped_gemm_mma_kernel<BM, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    once = true;
  }
  dim3 grid((n_rows + BM - 1) / BM + X, (N + GM_BN - 1) / GM_BN);
  moe_grouped_gemm_mma_kernel<BM, MODE><<<grid, GM_THREADS, smem, st>>>((const __nv_bfloat16*)a, lda, (const __nv_bfloat16*)w, offsets, perm,
                                                                       top, X, N, K, limit, alpha, shift, (__nv_bfloat16*)c, ldc);
  LL_LAUNCH_OK("moe_grouped_gemm_mma_kernel");
  return LL_OK;
}

template <typename T>
__global__ void moe_combine_kernel(const T* __restrict__ y, const float* __restrict__ expert_w, int top,
                                   const T* __restrict__ shared_y, int shared_ld, const T* __restrict__ shared_gate,
                                   int gate_ld, T* __restrict__ out, int dim) {
  const int m = blockIdx.x;
  float sg = 0.f;
  if (shared_y) sg = shared_gate ? 1.f / (1.f + expf(-dt<T>::ld(shared_gate, (size_t)m * gate_ld))) : 1.f;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) {
    float v = 0.f;
    for (int k = 0; k < top; ++k) v += expert_w[(size_t)m * top + k] * dt<T>::ld(y, ((size_t)m * top + k) * dim + i);
    if (shared_y) v += sg * dt<T>::ld(shared_y, (size_t)m * shared_ld + i);
    dt<T>::st(out, (size_t)m * dim + i, v);
  }
}

template <typename T, int TM, int MODE>
static int launch_grouped(const void* a, int lda, const void* w, const int32_t* offsets, const int32_t* perm, int top, int X, int N,
                          int K, float limit, float alpha, float shift, void* c, int ldc, int n_rows, cudaStream_t st) {
  constexpr int BM = 16 * TM;
  dim3 grid((n_rows + BM - 1) / BM + X, (N + GG_BN - 1) / GG_BN);
  moe_grouped_gemm_kernel<T, TM, MODE><<<grid, GG_THREADS, 0, st>>>((const T*)a, lda, (const T*)w, offsets, perm, top, X, N, K, limit,
                                                                   alpha, shift, (T*)c, ldc);
  LL_LAUNCH_OK("moe_grouped_gemm_kernel");
  return LL_OK;
}

}  // namespace llb

using namespace llb;

extern "C" {

int ll_moe_route(const void* x, int dtype, const float* w_router, const float* bias, int M, int dim, int n_experts, int top,
                 int32_t* expert_idx, float* expert_w, int32_t* counts, int32_t* rank, int32_t* offsets, int32_t* perm,
                 ll_stream stream) {
  return ll_moe_route_scored(x, dtype, w_router, bias, M, dim, n_experts, top, 0, 1, 1, expert_idx, expert_w, counts, rank, offsets,
                             perm, stream);
}

int ll_moe_route_scored(const void* x, int dtype, const float* w_router, const float* bias, int M, int dim, int n_experts, int top,
                        int score_all, int n_groups, int keep_groups, int32_t* expert_idx, float* expert_w, int32_t* counts,
                        int32_t* rank, int32_t* offsets, int32_t* perm, ll_stream stream) {
  LL_CHECK_ARG(x && w_router && expert_idx && expert_w && counts && rank && offsets && perm, "moe_route: null pointer");
  LL_CHECK_ARG(M >= 0 && dim > 0 && n_experts > 0 && top > 0 && top <= n_experts, "bad moe_route arguments");
  LL_CHECK_ARG(n_groups >= 1 && keep_groups >= 1 && keep_groups <= n_groups && n_experts % n_groups == 0 &&
                   top <= keep_groups * (n_experts / n_groups),
               "moe_route: %d groups (keep %d) of %d experts cannot give %d choices", n_groups, keep_groups, n_experts, top);
  if (M == 0) return LL_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const size_t smem = sizeof(float) * RT_TOK * ((size_t)dim + n_experts + 2 * (size_t)n_groups);
  if (smem > 200 * 1024) {
    set_error("moe_route: width %d with %d experts does not fit shared memory", dim, n_experts);
    return LL_ERR_UNSUPPORTED;
  }
  LL_CUDA(cudaMemsetAsync(counts, 0, sizeof(int32_t) * n_experts, st));
  const int blocks = (M + RT_TOK - 1) / RT_TOK;
  if (dtype == LL_F32) {
    LL_CUDA(cudaFuncSetAttribute(moe_route_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    moe_route_kernel<float><<<blocks, RT_THREADS, smem, st>>>((const float*)x, w_router, bias, M, dim, n_experts, top, score_all,
                                                             n_groups, keep_groups, expert_idx, expert_w, counts, rank);
  } else if (dtype == LL_BF16) {
    LL_CUDA(cudaFuncSetAttribute(moe_route_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    moe_route_kernel<__nv_bfloat16><<<blocks, RT_THREADS, smem, st>>>((const __nv_bfloat16*)x, w_router, bias, M, dim, n_experts, top,
                                                                     score_all, n_groups, keep_groups, expert_idx, expert_w, counts,
                                                                     rank);
  } else {
    set_error("moe_route: unsupported dtype %d", dtype);
    return LL_ERR_UNSUPPORTED;
  }
  LL_LAUNCH_OK("moe_route_kernel");
  const int n_pairs = M * top;
  moe_permute_kernel<<<(n_pairs + 255) / 256, 256, sizeof(int32_t) * (n_experts + 1), st>>>(expert_idx, rank, counts, n_pairs,
                                                                                          n_experts, offsets, perm);
  LL_LAUNCH_OK("moe_permute_kernel");
  return LL_OK;
}

int ll_moe_grouped_gemm(const void* a, int lda, const void* w, const int32_t* offsets, const int32_t* perm, int mode, int dtype,
                        int n_rows, int top, int n_experts, int N, int K, float limit, float alpha, void* c, int ldc,
                        ll_stream stream) {
  LL_CHECK_ARG(a && w && offsets && perm && c, "moe_grouped_gemm: null pointer");
  LL_CHECK_ARG(n_rows >= 0 && top > 0 && n_experts > 0 && N > 0 && K > 0 && lda >= K && ldc >= N && mode >= 0 && mode <= 2,
               "bad moe_grouped_gemm arguments");
  if (n_rows == 0) return LL_OK;
  const float shift = mode == 2 ? 0.f : 1.f;     // mode 2: the up branch enters as it is
  if (mode == 2) mode = MODE_GLU;
  cudaStream_t st = (cudaStream_t)stream;
  const bool small = n_rows <= 16 * n_experts / 2 + 16;   // few rows per expert: narrow row tiles waste less
#define LL_GG(T)                                                                                                              \
  (mode == MODE_GLU ? (small ? launch_grouped<T, 1, MODE_GLU>(a, lda, w, offsets, perm, top, n_experts, N, K, limit, alpha, shift, c, ldc, n_rows, st)  \
                             : launch_grouped<T, 4, MODE_GLU>(a, lda, w, offsets, perm, top, n_experts, N, K, limit, alpha, shift, c, ldc, n_rows, st)) \
                    : (small ? launch_grouped<T, 1, MODE_DOWN>(a, lda, w, offsets, perm, top, n_experts, N, K, limit, alpha, shift, c, ldc, n_rows, st) \
                             : launch_grouped<T, 4, MODE_DOWN>(a, lda, w, offsets, perm, top, n_experts, N, K, limit, alpha, shift, c, ldc, n_rows, st)))
  if (dtype == LL_F32) return LL_GG(float);
  if (dtype == LL_BF16 && K % 8 == 0 && lda % 8 == 0 && ((uintptr_t)a & 15) == 0 && ((uintptr_t)w & 15) == 0) {
    if (mode == MODE_GLU)
      return small ? launch_grouped_mma<16, MODE_GLU>(a, lda, w, offsets, perm, top, n_experts, N, K, limit, alpha, shift, c, ldc, n_rows, st)
                   : launch_grouped_mma<64, MODE_GLU>(a, lda, w, offsets, perm, top, n_experts, N, K, limit, alpha, shift, c, ldc, n_rows, st);
    return small ? launch_grouped_mma<16, MODE_DOWN>(a, lda, w, offsets, perm, top, n_experts, N, K, limit, alpha, shift, c, ldc, n_rows, st)
                 : launch_grouped_mma<64, MODE_DOWN>(a, lda, w, offsets, perm, top, n_experts, N, K, limit, alpha, shift, c, ldc, n_rows, st);
  }
  if (dtype == LL_BF16) return LL_GG(__nv_bfloat16);
#undef LL_GG
  set_error("moe_grouped_gemm: unsupported dtype %d", dtype);
  return LL_ERR_UNSUPPORTED;
}

int ll_moe_combine(const void* y, const float* expert_w, int top, const void* shared_y, int shared_ld, const void* shared_gate,
                   int gate_ld, void* out, int dtype, int M, int dim, ll_stream stream) {
  LL_CHECK_ARG(y && expert_w && out && top > 0 && M >= 0 && dim > 0, "bad moe_combine arguments");
  if (M == 0) return LL_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const int threads = dim >= 1024 ? 256 : 128;
  if (dtype == LL_F32)
    moe_combine_kernel<float><<<M, threads, 0, st>>>((const float*)y, expert_w, top, (const float*)shared_y, shared_ld,
                                                    (const float*)shared_gate, gate_ld, (float*)out, dim);
  else if (dtype == LL_BF16)
    moe_combine_kernel<__nv_bfloat16><<<M, threads, 0, st>>>((const __nv_bfloat16*)y, expert_w, top, (const __nv_bfloat16*)shared_y,
                                                            shared_ld, (const __nv_bfloat16*)shared_gate, gate_ld,
                                                            (__nv_bfloat16*)out, dim);
  else {
    set_error("moe_combine: unsupported dtype %d", dtype);
    return LL_ERR_UNSUPPORTED;
  }
  LL_LAUNCH_OK("moe_combine_kernel");
  return LL_OK;
}

}  // extern "C"
