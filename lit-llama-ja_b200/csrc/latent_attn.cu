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
  for (int i = threadIdx.x; i < KR; i += blockDim.x) {
    float v = 0.f;
    for (int s = 0; s < P.splits; ++s) {
      const float ms = base[s * (KR + 2) + KR];
      if (ms != -INFINITY) v += expf(ms - mx) * base[s * (KR + 2) + i];
    }
    dt<T>::st(out, (size_t)(h * P.os_h + (long long)m * P.os_m + i), v / l * g);
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
  dim3 grid(B * T, (n_head + P.HG - 1) / P.HG, splits);
  if (dtype == LL_F32) {
    LL_CUDA(cudaFuncSetAttribute(latent_attn_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    latent_attn_kernel<float><<<grid, LA_THREADS, smem, st>>>(P);
  } else if (dtype == LL_BF16) {
    LL_CUDA(cudaFuncSetAttribute(latent_attn_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    latent_attn_kernel<__nv_bfloat16><<<grid, LA_THREADS, smem, st>>>(P);
  } else {
    set_error("latent_attn: unsupported dtype %d", dtype);
    return LL_ERR_UNSUPPORTED;
  }
  LL_LAUNCH_OK("latent_attn_kernel");
  if (splits > 1) {
    dim3 g2(B * T, n_head);
    if (dtype == LL_F32) latent_attn_combine_kernel<float><<<g2, 128, 0, st>>>(P);
    else latent_attn_combine_kernel<__nv_bfloat16><<<g2, 128, 0, st>>>(P);
    LL_LAUNCH_OK("latent_attn_combine_kernel");
  }
  return LL_OK;
}

}  // extern "C"
