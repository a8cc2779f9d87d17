// Latent (low-rank, shared-key) attention over a ring cache of latent rows.
//
// A cache row of one token holds [c (kv_rank) | k_rot (rot_dim)]: the RMS-normed down-projection and
// one rotated key part that every head shares.  With the key up-projection absorbed into the query
// (q_lat[h] = W_uk[h]^T q_nope[h]) and the value up-projection applied after the weighted sum, the
// score of head h against token j is  (q_lat[h] . c_j + q_rot[h] . k_rot_j) * scale  and the head's
// output in latent space is  sum_j w_j c_j : all heads read the same row, once.
//
// Positions are a device array (one per token of the step), the slot of position p is p % cache_len,
// and a query at position p sees the positions p - window + 1 .. p (window <= 0: all of 0 .. p).
// Rotation pairs dimension 2i with 2i+1 (interleaved) on the first rot_dims dimensions of the rotated
// part; the (cos, sin) table is [positions][rot_dims / 2][2] fp32.  Scores, softmax weights and sums
// are fp32; T is the dtype of activations and of the cache.
#include "common.cuh"

namespace llb {

constexpr int LA_THREADS = 256;
constexpr int LA_KC = 32;     // keys per chunk (one per lane in the softmax step)
constexpr int LA_NACC = 16;   // output accumulators per thread: heads-per-block * kv_rank <= 256 * 16

template <typename T>
__global__ void latent_kv_append_kernel(const T* __restrict__ proj, int proj_stride, int col0,
                                        const float* __restrict__ norm_w, float eps, const float* __restrict__ rope,
                                        const int32_t* __restrict__ pos_ids, T* __restrict__ cache, int Tn, int kv_rank,
                                        int rot_dim, int rot_dims, int cache_len) {
  __shared__ float red[32];
  const int m = blockIdx.x, b = m / Tn, t = m - b * Tn;
  const int pos = pos_ids[t];
  const T* src = proj + (size_t)m * proj_stride + col0;
  T* dst = cache + ((size_t)b * cache_len + (pos % cache_len)) * (kv_rank + rot_dim);
  float ss = 0.f;
  for (int i = threadIdx.x; i < kv_rank; i += blockDim.x) {
    const float v = dt<T>::ld(src, i);
    ss += v * v;
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
  for (int w = 0; w < (int)(blockDim.x >> 5); ++w) tot += red[w];
  const float k = 1.f / sqrtf(tot / (float)kv_rank + eps);
  for (int i = threadIdx.x; i < kv_rank; i += blockDim.x) dt<T>::st(dst, i, dt<T>::ld(src, i) * k * norm_w[i]);
  const float* cs = rope + (size_t)pos * rot_dims;   // [rot_dims/2][2]
  for (int i = threadIdx.x; i < rot_dim / 2 + (rot_dim & 1); i += blockDim.x) {
    const int d0 = 2 * i;
    if (d0 + 1 < rot_dims) {   // rot_dims is even and <= rot_dim
      const float u = dt<T>::ld(src, kv_rank + d0), v = dt<T>::ld(src, kv_rank + d0 + 1);
      const float c = cs[2 * i], s = cs[2 * i + 1];
      dt<T>::st(dst, kv_rank + d0, u * c - v * s);
      dt<T>::st(dst, kv_rank + d0 + 1, v * c + u * s);
    } else {
      dst[kv_rank + d0] = src[kv_rank + d0];
      if (d0 + 1 < rot_dim) dst[kv_rank + d0 + 1] = src[kv_rank + d0 + 1];
    }
  }
}

struct LatentAttnParams {
  const void* q_lat;   // (h, m, i) at h * qs_h + m * qs_m + i
  long long qs_h, qs_m;
  const void* proj;    // row m at m * proj_stride; head h's un-rotated rotary part at q_rot_col0 + h * q_head_stride
  int proj_stride, q_rot_col0, q_head_stride;
  int gate_col0;       // head h's gate logit at gate_col0 + h of the same row; < 0: no gate
  const float* rope;
  const int32_t* pos_ids;
  const void* cache;
  void* out;           // (h, m, i) at h * os_h + m * os_m + i
  long long os_h, os_m;
  float* scratch;      // splits > 1: [M][H][splits][kv_rank + 2]
  int Tn, H, HG, kv_rank, rot_dim, rot_dims, cache_len, window, splits;
  float scale;
};

template <typename T>
__global__ void __launch_bounds__(LA_THREADS) latent_attn_kernel(const LatentAttnParams P) {
  extern __shared__ float sm[];
  const int KR = P.kv_rank, R = P.rot_dim, Dk = KR + R;
  const int ldk = Dk + ((33 - (Dk & 31)) & 31);          // row pitch = 1 mod 32: conflict-free column reads
  const int m = blockIdx.x, b = m / P.Tn, t = m - b * P.Tn;
  const int h0 = blockIdx.y * P.HG;
  const int HG = min(P.HG, P.H - h0);
  const int sp = blockIdx.z;
  float* qs = sm;                                   // [P.HG][Dk]
  float* ks = qs + P.HG * Dk;                       // [LA_KC][ldk]
  float* ps = ks + LA_KC * ldk;                     // [P.HG][LA_KC]
  float* m_run = ps + P.HG * LA_KC;                 // [P.HG]
  float* l_run = m_run + P.HG;
  float* corr = l_run + P.HG;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int pos = P.pos_ids[t];
  const T* q_lat = (const T*)P.q_lat;
  const T* prow = (const T*)P.proj + (size_t)m * P.proj_stride;
  const float* cs = P.rope + (size_t)pos * P.rot_dims;

  for (int idx = tid; idx < HG * KR; idx += LA_THREADS) {
    const int h = idx / KR, i = idx - h * KR;
    qs[h * Dk + i] = dt<T>::ld(q_lat, (size_t)((h0 + h) * P.qs_h + (long long)m * P.qs_m + i)) * P.scale;
  }
  const int npair = (R + 1) / 2;
  for (int idx = tid; idx < HG * npair; idx += LA_THREADS) {
    const int h = idx / npair, i = idx - h * npair, d0 = 2 * i;
    const T* qr = prow + P.q_rot_col0 + (size_t)(h0 + h) * P.q_head_stride;
    if (d0 + 1 < R && d0 + 1 < P.rot_dims) {
      const float u = dt<T>::ld(qr, d0), v = dt<T>::ld(qr, d0 + 1);
      const float c = cs[2 * i], s = cs[2 * i + 1];
      qs[h * Dk + KR + d0] = (u * c - v * s) * P.scale;
      qs[h * Dk + KR + d0 + 1] = (v * c + u * s) * P.scale;
    } else {
      qs[h * Dk + KR + d0] = dt<T>::ld(qr, d0) * P.scale;
      if (d0 + 1 < R) qs[h * Dk + KR + d0 + 1] = dt<T>::ld(qr, d0 + 1) * P.scale;
    }
  }
  if (tid < P.HG) { m_run[tid] = -INFINITY; l_run[tid] = 0.f; }

  // this split's share of the visible positions lo .. pos
  const int lo = (P.window > 0 && pos - P.window + 1 > 0) ? pos - P.window + 1 : 0;
  const int n_all = pos - lo + 1;
  const int per = (n_all + P.splits - 1) / P.splits;
  const int j_begin = lo + sp * per;
  const int j_end = min(pos + 1, j_begin + per);

  float acc[LA_NACC];
#pragma unroll
  for (int a = 0; a < LA_NACC; ++a) acc[a] = 0.f;
  const T* cache = (const T*)P.cache + (size_t)b * P.cache_len * Dk;
  __syncthreads();

  for (int j0 = j_begin; j0 < j_end; j0 += LA_KC) {
    const int nk = min(LA_KC, j_end - j0);
    for (int idx = tid; idx < nk * Dk; idx += LA_THREADS) {
      const int jj = idx / Dk, i = idx - jj * Dk;
      ks[jj * ldk + i] = dt<T>::ld(cache, (size_t)((j0 + jj) % P.cache_len) * Dk + i);
    }
    __syncthreads();
    for (int idx = tid; idx < HG * LA_KC; idx += LA_THREADS) {
      const int h = idx / LA_KC, jj = idx - h * LA_KC;
      float s = -INFINITY;
      if (jj < nk) {
        const float* qv = qs + h * Dk;
        const float* kv = ks + jj * ldk;
        float s0 = 0.f, s1 = 0.f;
        int i = 0;
        for (; i + 1 < Dk; i += 2) { s0 += qv[i] * kv[i]; s1 += qv[i + 1] * kv[i + 1]; }
        if (i < Dk) s0 += qv[i] * kv[i];
        s = s0 + s1;
      }
      ps[idx] = s;
    }
    __syncthreads();
    for (int h = warp; h < HG; h += LA_THREADS / 32) {
      const float s = ps[h * LA_KC + lane];
      const float mo = m_run[h];
      const float mn = fmaxf(mo, warp_max(s));
      const float p = (s == -INFINITY) ? 0.f : expf(s - mn);
      const float sum = warp_sum(p);
      ps[h * LA_KC + lane] = p;
      if (lane == 0) {
        const float c = (mo == -INFINITY) ? 0.f : expf(mo - mn);
        corr[h] = c;
        l_run[h] = l_run[h] * c + sum;
        m_run[h] = mn;
      }
    }
    __syncthreads();
#pragma unroll
    for (int a = 0; a < LA_NACC; ++a) {
      const int o = tid + a * LA_THREADS;
      if (o < HG * KR) {
        const int h = o / KR, i = o - h * KR;
        float v = acc[a] * corr[h];
        const float* pv = ps + h * LA_KC;
        for (int jj = 0; jj < nk; ++jj) v += pv[jj] * ks[jj * ldk + i];
        acc[a] = v;
      }
    }
    __syncthreads();
  }

  if (P.splits == 1) {
    T* out = (T*)P.out;
#pragma unroll
    for (int a = 0; a < LA_NACC; ++a) {
      const int o = tid + a * LA_THREADS;
      if (o < HG * KR) {
        const int h = o / KR, i = o - h * KR;
        float g = 1.f;
        if (P.gate_col0 >= 0) g = 1.f / (1.f + expf(-dt<T>::ld(prow, P.gate_col0 + h0 + h)));
        dt<T>::st(out, (size_t)((h0 + h) * P.os_h + (long long)m * P.os_m + i), acc[a] / l_run[h] * g);
      }
    }
  } else {
#pragma unroll
    for (int a = 0; a < LA_NACC; ++a) {
      const int o = tid + a * LA_THREADS;
      if (o < HG * KR) {
        const int h = o / KR, i = o - h * KR;
        P.scratch[(((size_t)m * P.H + h0 + h) * P.splits + sp) * (KR + 2) + i] = acc[a];
      }
    }
    if (tid < HG) {
      float* rec = P.scratch + (((size_t)m * P.H + h0 + tid) * P.splits + sp) * (KR + 2) + KR;
      rec[0] = m_run[tid];
      rec[1] = l_run[tid];
    }
  }
}

// ---- bf16 tensor-core form (mma.sync m16n8k16, fp32 scores / softmax / accumulation) ----
// A block owns 32 query rows = (a few consecutive tokens) x (up to 32 heads) and walks the union of their windows in
// chunks of 64 cache rows: S = Q K^T (all heads against the same rows; a warp takes 16 rows x 16 keys x half of the row's
// dimensions, the two halves meet in shared memory), online softmax in fp32, O += P C with the accumulators of the
// 32 x kv_rank output split by columns over the 16 warps (NTW n-tiles of 8 columns each).  Sixteen warps, four per
// scheduler: every phase is a chain of shared-memory loads and tensor instructions whose latency the other warps cover.
constexpr int LM_ROWS = 32, LM_KC = 64;

__device__ __forceinline__ void la_cp_async16(void* smem, const void* gmem, bool valid) {
  const int n = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(smem)), "l"(gmem), "r"(n) : "memory");
}
__device__ __forceinline__ void la_ldmatrix_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void la_ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void la_ldmatrix_x2_trans(uint32_t (&r)[2], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(smem_u32(p)));
}

struct LatentMmaGeom {
  int HB, TQ, DKP, pitch;   // heads and tokens per block (HB * TQ <= 32), padded row length, shared-memory row pitch (elements)
};

// WARPS = 16: one block per SM, four warps per scheduler, the score product split over halves of the dimensions.
// WARPS = 8: for rows short enough that two blocks share an SM (the same number of warps, two chunks in different phases).
template <int NTW, int WARPS>
__global__ void __launch_bounds__(WARPS * 32, WARPS == 8 ? 2 : 1) latent_attn_mma_kernel(const LatentAttnParams P, const LatentMmaGeom G) {
  constexpr int LM_THREADS = WARPS * 32, LM_WARPS = WARPS;
  extern __shared__ __align__(16) unsigned char la_smem[];
  const int KR = P.kv_rank, R = P.rot_dim, Dk = KR + R;
  const int pitch = G.pitch;
  __nv_bfloat16* Qs = (__nv_bfloat16*)la_smem;                 // [32][pitch]
  __nv_bfloat16* Ks0 = Qs + LM_ROWS * pitch;                   // [2 stages][64][pitch]
  __nv_bfloat16* Ps = Ks0 + 2 * LM_KC * pitch;                 // [32][64 + 8]
  float* Ss = (float*)(Ps + LM_ROWS * (LM_KC + 8));            // [2 halves of the row's dimensions][32][64 + 1]
  float* m_run = Ss + (WARPS == 16 ? 2 : 1) * LM_ROWS * (LM_KC + 1);   // [32]
  float* l_run = m_run + LM_ROWS;
  float* corr = l_run + LM_ROWS;
  int* row_pos = (int*)(corr + LM_ROWS);                       // [32] position of the row's token, -1: padding row

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int tiles_t = (P.Tn + G.TQ - 1) / G.TQ;
  const int b = blockIdx.x / tiles_t, t0 = (blockIdx.x - b * tiles_t) * G.TQ;
  const int ntok = min(G.TQ, P.Tn - t0);
  const int h0 = blockIdx.y * G.HB, HB = min(G.HB, P.H - h0);
  const int sp = blockIdx.z;
  const __nv_bfloat16* q_lat = (const __nv_bfloat16*)P.q_lat;
  const __nv_bfloat16* proj = (const __nv_bfloat16*)P.proj;

  if (tid < LM_ROWS) {
    const int tq = tid / G.HB, hh = tid - tq * G.HB;
    row_pos[tid] = (tq < ntok && hh < HB) ? P.pos_ids[t0 + tq] : -1;
    m_run[tid] = -INFINITY;
    l_run[tid] = 0.f;
  }
  // queries: latent part as it is (16-byte pieces when rows allow), rotary part rotated in fp32, zero padding
  const bool qvec = (KR % 8 == 0) && (P.qs_h % 8 == 0) && (P.qs_m % 8 == 0) && (((uintptr_t)q_lat & 15) == 0);
  for (int r = warp; r < LM_ROWS; r += LM_THREADS / 32) {       // a row per warp pass, lanes along the row
    const int tq = r / G.HB, hh = r - tq * G.HB;
    const bool live = tq < ntok && hh < HB;
    const __nv_bfloat16* src = q_lat + (size_t)((h0 + hh) * P.qs_h + (long long)((size_t)b * P.Tn + t0 + tq) * P.qs_m);
    if (qvec) {
      for (int c = lane; c < KR / 8; c += 32) {
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (live) v = *(const uint4*)(src + c * 8);
        *(uint4*)(Qs + r * pitch + c * 8) = v;
      }
    } else {
      for (int i = lane; i < KR; i += 32) Qs[r * pitch + i] = live ? src[i] : __float2bfloat16_rn(0.f);
    }
  }
  {
    const int npair = (G.DKP - KR + 1) / 2;      // the rotary part and the zero padding behind it, two columns at a time
    for (int r = warp; r < LM_ROWS; r += LM_THREADS / 32) {
      const int tq = r / G.HB, hh = r - tq * G.HB;
      const bool live = tq < ntok && hh < HB;
      const size_t m = (size_t)b * P.Tn + t0 + (live ? tq : 0);
      const __nv_bfloat16* qr = proj + m * P.proj_stride + P.q_rot_col0 + (size_t)(h0 + (live ? hh : 0)) * P.q_head_stride;
      const float* cs_row = P.rope + (size_t)(live ? P.pos_ids[t0 + tq] : 0) * P.rot_dims;
      for (int pi = lane; pi < npair; pi += 32) {
        const int d = 2 * pi;
        float v0 = 0.f, v1 = 0.f;
        if (live && d < R) {
          const float u = __bfloat162float(qr[d]), w = (d + 1 < R) ? __bfloat162float(qr[d + 1]) : 0.f;
          if (d + 1 < P.rot_dims) {
            const float c0 = cs_row[d], s0 = cs_row[d + 1];
            v0 = u * c0 - w * s0;
            v1 = w * c0 + u * s0;
          } else {
            v0 = u;
            v1 = w;
          }
        }
        if (KR + d < G.DKP) Qs[r * pitch + KR + d] = __float2bfloat16_rn(v0);
        if (KR + d + 1 < G.DKP) Qs[r * pitch + KR + d + 1] = __float2bfloat16_rn(v1);
      }
    }
  }
  // zero the padding columns of the key rows once (the loads below never touch them)
  for (int idx = tid; idx < 2 * LM_KC * (G.DKP - Dk); idx += LM_THREADS) {
    const int r = idx / (G.DKP - Dk), i = Dk + idx - r * (G.DKP - Dk);
    Ks0[r * pitch + i] = __float2bfloat16_rn(0.f);
  }

  const int p_first = P.pos_ids[t0], p_last = P.pos_ids[t0 + ntok - 1];
  const int lo = (P.window > 0 && p_first - P.window + 1 > 0) ? p_first - P.window + 1 : 0;
  const int n_all = p_last - lo + 1;
  const int per = (n_all + P.splits - 1) / P.splits;
  const int j_begin = lo + sp * per;
  const int j_end = min(p_last + 1, j_begin + per);
  const __nv_bfloat16* cache = (const __nv_bfloat16*)P.cache + (size_t)b * P.cache_len * Dk;
  const bool vec = (Dk % 8 == 0) && (((uintptr_t)cache & 15) == 0);

  float acc[2][NTW][4];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < NTW; ++j)
#pragma unroll
      for (int q = 0; q < 4; ++q) acc[i][j][q] = 0.f;
  const int wcol0 = warp * NTW * 8;            // this warp's first output column
  __syncthreads();

  // rows j0 .. j0 + 63 of the cache into one of the two stages (16-byte asynchronous copies when rows allow)
  auto load_keys = [&](int stage, int j0) {
    __nv_bfloat16* dst = Ks0 + stage * LM_KC * pitch;
    const int nk = min(LM_KC, j_end - j0);
    if (vec) {
      const int cpr = Dk / 8;
      int slot = (j0 + warp) % P.cache_len;
      for (int jj = warp; jj < LM_KC; jj += LM_THREADS / 32) {
        const bool ok = jj < nk;
        const __nv_bfloat16* src = cache + (size_t)(ok ? slot : 0) * Dk;
        __nv_bfloat16* d = dst + jj * pitch;
        for (int c = lane; c < cpr; c += 32) la_cp_async16(d + c * 8, src + c * 8, ok);
        slot += LM_THREADS / 32;
        while (slot >= P.cache_len) slot -= P.cache_len;
      }
    } else {
      for (int idx = tid; idx < LM_KC * Dk; idx += LM_THREADS) {
        const int jj = idx / Dk, i = idx - jj * Dk;
        dst[jj * pitch + i] = jj < nk ? cache[(size_t)((j0 + jj) % P.cache_len) * Dk + i] : __float2bfloat16_rn(0.f);
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };

  if (j_begin < j_end) load_keys(0, j_begin);
  int stage = 0;
  for (int j0 = j_begin; j0 < j_end; j0 += LM_KC, stage ^= 1) {
    const int nk = min(LM_KC, j_end - j0);
    const __nv_bfloat16* Ks = Ks0 + stage * LM_KC * pitch;
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();            // this chunk has landed; every warp is done with the other stage, with Ss and with Ps
    if (j0 + LM_KC < j_end) load_keys(stage ^ 1, j0 + LM_KC);     // the next chunk travels under this chunk's math
    {   // S = Q K^T: warp -> m-tile (warp & 1), key columns ((warp >> 1) & 3) * 16 .. + 15, half (warp >> 3) of the k-steps
      const int mt = warp & 1, np = (warp >> 1) & 3, kh = WARPS == 16 ? warp >> 3 : 0;
      float part[4][2][4];     // four interleaved slices of the k range: independent accumulation chains, summed below
#pragma unroll
      for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
          for (int q = 0; q < 4; ++q) part[c][j][q] = 0.f;
      const int nks_all = G.DKP / 16, nks_half = WARPS == 16 ? (nks_all + 1) / 2 : nks_all;
      const int ks_begin = kh * nks_half, nks = min(nks_all, ks_begin + nks_half);
      for (int ks0 = ks_begin; ks0 < nks; ks0 += 4) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int ks = ks0 + c;
          if (ks < nks) {
            uint32_t af[4], bf[4];
            la_ldmatrix_x4(af, Qs + (mt * 16 + (lane & 15)) * pitch + ks * 16 + (lane >> 4) * 8);
            la_ldmatrix_x4(bf, Ks + (np * 16 + (lane & 7) + (lane >> 4) * 8) * pitch + ks * 16 + ((lane >> 3) & 1) * 8);
            mma_bf16_16816(part[c][0], af[0], af[1], af[2], af[3], bf[0], bf[1]);
            mma_bf16_16816(part[c][1], af[0], af[1], af[2], af[3], bf[2], bf[3]);
          }
        }
      }
      float sacc[2][4];
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int q = 0; q < 4; ++q) sacc[j][q] = (part[0][j][q] + part[1][j][q]) + (part[2][j][q] + part[3][j][q]);
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int r = mt * 16 + (lane >> 2) + (q >> 1) * 8;
          const int col = np * 16 + j * 8 + (lane & 3) * 2 + (q & 1);
          const int pr = row_pos[r], jpos = j0 + col;
          const bool vis = pr >= 0 && col < nk && jpos <= pr && (P.window <= 0 || jpos > pr - P.window);
          Ss[(kh * LM_ROWS + r) * (LM_KC + 1) + col] = vis ? sacc[j][q] * P.scale : -INFINITY;
        }
    }
    __syncthreads();
    for (int r = warp * (LM_ROWS / LM_WARPS); r < (warp + 1) * (LM_ROWS / LM_WARPS); ++r) {   // online softmax: 2 columns per lane
      const float* sb = Ss + (LM_ROWS + r) * (LM_KC + 1);     // the other half of the dimensions (-inf + -inf stays -inf)
      const float s0 = Ss[r * (LM_KC + 1) + lane] + (WARPS == 16 ? sb[lane] : 0.f);
      const float s1 = Ss[r * (LM_KC + 1) + lane + 32] + (WARPS == 16 ? sb[lane + 32] : 0.f);
      const float mo = m_run[r];
      const float mn = fmaxf(mo, warp_max(fmaxf(s0, s1)));
      const float p0 = (s0 == -INFINITY) ? 0.f : expf(s0 - mn), p1 = (s1 == -INFINITY) ? 0.f : expf(s1 - mn);
      const __nv_bfloat16 b0 = __float2bfloat16_rn(p0), b1 = __float2bfloat16_rn(p1);
      Ps[r * (LM_KC + 8) + lane] = b0;
      Ps[r * (LM_KC + 8) + lane + 32] = b1;
      const float sum = warp_sum(__bfloat162float(b0) + __bfloat162float(b1));   // the weights as the product below sees them
      if (lane == 0) {
        const float c = (mo == -INFINITY) ? 0.f : expf(mo - mn);
        corr[r] = c;
        l_run[r] = l_run[r] * c + sum;
        m_run[r] = mn;
      }
    }
    __syncthreads();
    if (wcol0 < KR) {   // O = O * corr + P C over this warp's columns
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const float c0 = corr[i * 16 + (lane >> 2)], c1 = corr[i * 16 + (lane >> 2) + 8];
#pragma unroll
        for (int j = 0; j < NTW; ++j) { acc[i][j][0] *= c0; acc[i][j][1] *= c0; acc[i][j][2] *= c1; acc[i][j][3] *= c1; }
      }
#pragma unroll
      for (int ks = 0; ks < LM_KC / 16; ++ks) {
        uint32_t af[2][4];
#pragma unroll
        for (int i = 0; i < 2; ++i) la_ldmatrix_x4(af[i], Ps + (i * 16 + (lane & 15)) * (LM_KC + 8) + ks * 16 + (lane >> 4) * 8);
        if (NTW == 1) {
          uint32_t bf[2];
          la_ldmatrix_x2_trans(bf, Ks + (ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * pitch + wcol0);
#pragma unroll
          for (int i = 0; i < 2; ++i) mma_bf16_16816(acc[i][0], af[i][0], af[i][1], af[i][2], af[i][3], bf[0], bf[1]);
        } else {
#pragma unroll
          for (int jp = 0; jp < NTW / 2; ++jp) {
            if (wcol0 + jp * 16 >= KR) break;
            uint32_t bf[4];
            la_ldmatrix_x4_trans(bf, Ks + (ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * pitch + wcol0 + jp * 16 + (lane >> 4) * 8);
#pragma unroll
            for (int i = 0; i < 2; ++i) {
              mma_bf16_16816(acc[i][2 * jp], af[i][0], af[i][1], af[i][2], af[i][3], bf[0], bf[1]);
              mma_bf16_16816(acc[i][2 * jp + 1], af[i][0], af[i][1], af[i][2], af[i][3], bf[2], bf[3]);
            }
          }
        }
      }
    }
  }

  __nv_bfloat16* out = (__nv_bfloat16*)P.out;
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {           // the rows this thread holds: resolved once, columns walked below
      const int r = i * 16 + (lane >> 2) + hf * 8;
      if (row_pos[r] < 0) continue;
      const int tq = r / G.HB, hh = r - tq * G.HB;
      const size_t m = (size_t)b * P.Tn + t0 + tq;
      if (P.splits == 1) {
        float g = 1.f;
        if (P.gate_col0 >= 0) g = 1.f / (1.f + expf(-__bfloat162float(proj[m * P.proj_stride + P.gate_col0 + h0 + hh])));
        const float f = g / l_run[r];
        __nv_bfloat16* orow = out + (size_t)((h0 + hh) * P.os_h + (long long)m * P.os_m);
#pragma unroll
        for (int j = 0; j < NTW; ++j) {
          const int col = wcol0 + j * 8 + (lane & 3) * 2;
          if (col < KR) orow[col] = __float2bfloat16_rn(acc[i][j][hf * 2] * f);
          if (col + 1 < KR) orow[col + 1] = __float2bfloat16_rn(acc[i][j][hf * 2 + 1] * f);
        }
      } else {
        float* srow = P.scratch + ((m * P.H + h0 + hh) * P.splits + sp) * (KR + 2);
#pragma unroll
        for (int j = 0; j < NTW; ++j) {
          const int col = wcol0 + j * 8 + (lane & 3) * 2;
          if (col < KR) srow[col] = acc[i][j][hf * 2];
          if (col + 1 < KR) srow[col + 1] = acc[i][j][hf * 2 + 1];
        }
      }
    }
  if (P.splits > 1 && tid < LM_ROWS && row_pos[tid] >= 0) {
    const int tq = tid / G.HB, hh = tid - tq * G.HB;
    const size_t m = (size_t)b * P.Tn + t0 + tq;
    float* rec = P.scratch + ((m * P.H + h0 + hh) * P.splits + sp) * (KR + 2) + KR;
    rec[0] = m_run[tid];
    rec[1] = l_run[tid];
  }
}

static size_t latent_mma_smem(int pitch, int halves) {
  return sizeof(__nv_bfloat16) * ((size_t)(LM_ROWS + 2 * LM_KC) * pitch + (size_t)LM_ROWS * (LM_KC + 8)) +
         sizeof(float) * ((size_t)halves * LM_ROWS * (LM_KC + 1) + 3 * LM_ROWS) + sizeof(int) * LM_ROWS;
}

template <int NTW, int WARPS>
static int launch_latent_mma(const LatentAttnParams& P, const LatentMmaGeom& G, int B, cudaStream_t st) {
  const size_t smem = latent_mma_smem(G.pitch, WARPS == 16 ? 2 : 1);
  static size_t configured = 0;
  if (smem > configured) {
    LL_CUDA(cudaFuncSetAttribute(latent_attn_mma_kernel<NTW, WARPS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = smem;
  }
  dim3 grid(B * ((P.Tn + G.TQ - 1) / G.TQ), (P.H + G.HB - 1) / G.HB, P.splits);
  latent_attn_mma_kernel<NTW, WARPS><<<grid, WARPS * 32, smem, st>>>(P, G);
  LL_LAUNCH_OK("latent_attn_mma_kernel");
  return LL_OK;
}

// Merge the splits of one (token, head) in split order: out = sum_s e^(m_s - m) acc_s / sum_s e^(m_s - m) l_s, times the gate.
template <typename T>
__global__ void latent_attn_combine_kernel(const LatentAttnParams P) {
  const int m = blockIdx.x, h = blockIdx.y, KR = P.kv_rank;
  const float* base = P.scratch + ((size_t)m * P.H + h) * P.splits * (KR + 2);
  float mx = -INFINITY;
  for (int s = 0; s < P.splits; ++s) mx = fmaxf(mx, base[s * (KR + 2) + KR]);
  float l = 0.f;
  for (int s = 0; s < P.splits; ++s) {
    const float ms = base[s * (KR + 2) + KR];
    if (ms != -INFINITY) l += expf(ms - mx) * base[s * (KR + 2) + KR + 1];
  }
  float g = 1.f;
  if (P.gate_col0 >= 0) g = 1.f / (1.f + expf(-dt<T>::ld((const T*)P.proj + (size_t)m * P.proj_stride, P.gate_col0 + h)));
  T* out = (T*)P.out;
  __shared__ float wsp[64];                      // weight of every split, with 1 / l and the gate folded in
  for (int s0 = 0; s0 < P.splits; s0 += 64) {    // 64 splits at a time (in split order)
    const int ns = min(64, P.splits - s0);
    __syncthreads();
    if ((int)threadIdx.x < ns) {
      const float ms = base[(s0 + threadIdx.x) * (KR + 2) + KR];
      wsp[threadIdx.x] = (ms != -INFINITY) ? expf(ms - mx) / l * g : 0.f;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < KR; i += blockDim.x) {
      float v = 0.f;
#pragma unroll 8
      for (int s = 0; s < ns; ++s) v += wsp[s] * base[(size_t)(s0 + s) * (KR + 2) + i];
      const size_t o = (size_t)(h * P.os_h + (long long)m * P.os_m + i);
      if (s0 > 0) v += dt<T>::ld(out, o);
      dt<T>::st(out, o, v);
    }
  }
}

static size_t latent_attn_smem(int HG, int Dk) {
  const int ldk = Dk + ((33 - (Dk & 31)) & 31);
  return sizeof(float) * ((size_t)HG * Dk + (size_t)LA_KC * ldk + (size_t)HG * LA_KC + 3 * (size_t)HG);
}

// heads per block: bounded by the accumulator budget and by shared memory
static int latent_attn_heads_per_block(int H, int KR, int Dk) {
  int hg = (LA_THREADS * LA_NACC) / KR;
  if (hg > H) hg = H;
  if (hg > 32) hg = 32;
  while (hg > 1 && latent_attn_smem(hg, Dk) > 200 * 1024) --hg;
  return hg;
}

}  // namespace llb

using namespace llb;

extern "C" {

int ll_latent_kv_append(const void* proj, int dtype, int proj_stride, int col0, const float* norm_w, float eps,
                        const float* rope, const int32_t* pos_ids, void* cache, int B, int T, int kv_rank, int rot_dim,
                        int rot_dims, int cache_len, ll_stream stream) {
  LL_CHECK_ARG(proj && norm_w && rope && pos_ids && cache, "latent_kv_append: null pointer");
  LL_CHECK_ARG(B >= 0 && T >= 0 && kv_rank > 0 && rot_dim >= 0 && rot_dims >= 0 && rot_dims <= rot_dim && rot_dims % 2 == 0 &&
                   cache_len > 0 && T <= cache_len && proj_stride >= col0 + kv_rank + rot_dim,
               "bad latent_kv_append arguments");
  if (B * T == 0) return LL_OK;
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == LL_F32)
    latent_kv_append_kernel<float><<<B * T, 128, 0, st>>>((const float*)proj, proj_stride, col0, norm_w, eps, rope, pos_ids,
                                                         (float*)cache, T, kv_rank, rot_dim, rot_dims, cache_len);
  else if (dtype == LL_BF16)
    latent_kv_append_kernel<__nv_bfloat16><<<B * T, 128, 0, st>>>((const __nv_bfloat16*)proj, proj_stride, col0, norm_w, eps, rope,
                                                                 pos_ids, (__nv_bfloat16*)cache, T, kv_rank, rot_dim, rot_dims,
                                                                 cache_len);
  else {
    set_error("latent_kv_append: unsupported dtype %d", dtype);
    return LL_ERR_UNSUPPORTED;
  }
  LL_LAUNCH_OK("latent_kv_append_kernel");
  return LL_OK;
}

size_t ll_latent_attn_scratch_bytes(int M, int n_head, int kv_rank, int splits) {
  return splits > 1 ? sizeof(float) * (size_t)M * n_head * splits * (kv_rank + 2) : 0;
}

int ll_latent_attn(const void* q_lat, long long qs_h, long long qs_m, const void* proj, int proj_stride, int q_rot_col0,
                   int q_head_stride, int gate_col0, const float* rope, const int32_t* pos_ids, const void* cache, void* out,
                   long long os_h, long long os_m, int dtype, int B, int T, int n_head, int kv_rank, int rot_dim, int rot_dims,
                   int cache_len, int window, float scale, int splits, float* scratch, ll_stream stream) {
  LL_CHECK_ARG(q_lat && proj && rope && pos_ids && cache && out, "latent_attn: null pointer");
  LL_CHECK_ARG(B >= 0 && T >= 0 && n_head > 0 && kv_rank > 0 && rot_dim >= 0 && rot_dims >= 0 && rot_dims <= rot_dim &&
                   rot_dims % 2 == 0 && cache_len > 0 && splits >= 1 && (splits == 1 || scratch),
               "bad latent_attn arguments");
  if (B * T == 0) return LL_OK;
  if (kv_rank > LA_THREADS * LA_NACC) {
    set_error("latent_attn: kv_rank %d above %d", kv_rank, LA_THREADS * LA_NACC);
    return LL_ERR_UNSUPPORTED;
  }
  const int Dk = kv_rank + rot_dim;
  LatentAttnParams P;
  P.q_lat = q_lat; P.qs_h = qs_h; P.qs_m = qs_m;
  P.proj = proj; P.proj_stride = proj_stride; P.q_rot_col0 = q_rot_col0; P.q_head_stride = q_head_stride; P.gate_col0 = gate_col0;
  P.rope = rope; P.pos_ids = pos_ids; P.cache = cache; P.out = out; P.os_h = os_h; P.os_m = os_m; P.scratch = scratch;
  P.Tn = T; P.H = n_head; P.kv_rank = kv_rank; P.rot_dim = rot_dim; P.rot_dims = rot_dims; P.cache_len = cache_len;
  P.window = window; P.splits = splits; P.scale = scale;
  P.HG = latent_attn_heads_per_block(n_head, kv_rank, Dk);
  const size_t smem = latent_attn_smem(P.HG, Dk);
  if (smem > 200 * 1024) {
    set_error("latent_attn: a row of %d values does not fit shared memory", Dk);
    return LL_ERR_UNSUPPORTED;
  }
  cudaStream_t st = (cudaStream_t)stream;
  bool done = false;
  if (dtype == LL_BF16 && kv_rank <= 512) {   // tensor-core kernel; the fp32 path and very long rows take the kernel below
    LatentMmaGeom G;
    G.HB = n_head < LM_ROWS ? n_head : LM_ROWS;
    G.TQ = LM_ROWS / G.HB < T ? LM_ROWS / G.HB : T;
    if (G.TQ < 1) G.TQ = 1;
    G.DKP = (Dk + 15) / 16 * 16;
    G.pitch = G.DKP + 8;
    if (latent_mma_smem(G.pitch, 2) <= 220 * 1024) {
      // two 8-warp blocks per SM when two fit (shared memory, and 32 columns of O per warp at most), else one of 16 warps
      const bool pair = 2 * (latent_mma_smem(G.pitch, 1) + 1024) <= 227 * 1024 && kv_rank <= 256;
      const int warps = pair ? 8 : 16;
      const int cols_per_warp = (kv_rank + warps - 1) / warps;
      int rc;
      if (pair) {
        if (cols_per_warp <= 8) rc = launch_latent_mma<1, 8>(P, G, B, st);
        else if (cols_per_warp <= 16) rc = launch_latent_mma<2, 8>(P, G, B, st);
        else rc = launch_latent_mma<4, 8>(P, G, B, st);
      } else {
        if (cols_per_warp <= 8) rc = launch_latent_mma<1, 16>(P, G, B, st);
        else if (cols_per_warp <= 16) rc = launch_latent_mma<2, 16>(P, G, B, st);
        else rc = launch_latent_mma<4, 16>(P, G, B, st);
      }
      if (rc != LL_OK) return rc;
      done = true;
    }
  }
  dim3 grid(B * T, (n_head + P.HG - 1) / P.HG, splits);
  if (done) {
  } else if (dtype == LL_F32) {
    LL_CUDA(cudaFuncSetAttribute(latent_attn_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    latent_attn_kernel<float><<<grid, LA_THREADS, smem, st>>>(P);
  } else if (dtype == LL_BF16) {
    LL_CUDA(cudaFuncSetAttribute(latent_attn_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    latent_attn_kernel<__nv_bfloat16><<<grid, LA_THREADS, smem, st>>>(P);
  } else {
    set_error("latent_attn: unsupported dtype %d", dtype);
    return LL_ERR_UNSUPPORTED;
  }
  if (!done) LL_LAUNCH_OK("latent_attn_kernel");
  if (splits > 1) {
    dim3 g2(B * T, n_head);
    if (dtype == LL_F32) latent_attn_combine_kernel<float><<<g2, 128, 0, st>>>(P);
    else latent_attn_combine_kernel<__nv_bfloat16><<<g2, 128, 0, st>>>(P);
    LL_LAUNCH_OK("latent_attn_combine_kernel");
  }
  return LL_OK;
}

}  // extern "C"
