// Latent attention: the plain kernels.
//
// A latent attention layer caches, per position, one row  [c (rank dims) | k_rot (rot dims)]
// shared by all heads: c is the RMS-normed low-rank projection of the layer's input and k_rot a
// rotated key part.  A head's unrotated key is  W_uk[h] c  and its value  W_uv[h] c.  Both
// matrices are moved to the query side, so attention runs on the cached rows as they are:
//
//   qa[t, h, :rank] = W_uk[h]^T q_nope[t, h]      (gb_heads_gemm, w = W_uk[h] transposed)
//   qa[t, h, rank:] = rotate(q_rot[t, h])
//   s[t, h, j]      = qa[t, h] . row[j]           (q already carries the score scale)
//   p               = softmax_j over j <= pos(t)  (float32)
//   ol[t, h]        = sum_j p[j] row[j, :rank]
//   o[t, h]         = gate[t, h] * W_uv[h] ol[t, h]   (gb_heads_gemm with a row scale)
//
// This unit holds what every precision and size can use: the kernel that norms, rotates and
// writes the cache row (gb_latent_prepare), the per-head products (gb_heads_gemm, FFMA), the
// attention itself one (token, head) per block (gb_latent_attention_ref), and the stand-alone
// rotation of interleaved pairs (gb_rope_pairs).  The arithmetic for one (token, head) depends on
// its position and the cache alone, so prompts, single tokens and any batch give the same bits.
#include "common.cuh"

// Rotation of interleaved pairs: dims (2i, 2i+1), i < rot/2, angle = float(pos) * inv_freq[i]:
// (u, v) -> (u cos - v sin, v cos + u sin), all in float32.
__device__ __forceinline__ void rotate_pair(float u, float v, float angle, float& ou, float& ov) {
  float s, c;
  sincosf(angle, &s, &c);
  ou = u * c - v * s;
  ov = v * c + u * s;
}

// One block per token.  Inputs are the float32 results of the layer's projections.
template <typename T>
__global__ void __launch_bounds__(256) latent_prepare_kernel(
    const float* __restrict__ q_in, long long ldq, const float* __restrict__ kv_in, long long ldkv,
    const float* __restrict__ g_in, long long ldg, const float* __restrict__ norm_w, float eps,
    const float* __restrict__ inv_freq, int rot, float q_scale, T* __restrict__ q_nope, long long ldqn,
    T* __restrict__ q_lat, long long ldql, float* __restrict__ gate, T* __restrict__ cache,
    const int* __restrict__ page_table, int table_width, int page_size, const int* __restrict__ tok_pos,
    const int* __restrict__ tok_seq, const int* __restrict__ seq_slot, int H, int dim, int rd, int rank,
    T* __restrict__ dense, long long ldd) {
  __shared__ float scratch[34];
  pdl_release_next();
  pdl_wait_prior();
  const int t = blockIdx.x, tid = threadIdx.x;
  const int pos = tok_pos[t];
  const float fpos = (float)pos;
  const float* kv = kv_in + (size_t)t * ldkv;
  // the latent: x / sqrt(mean(x^2) + eps) * w
  float ss = 0.f;
  for (int i = tid; i < rank; i += blockDim.x) ss = fmaf(kv[i], kv[i], ss);
  ss = block_sum(ss, scratch);
  const float rstd = 1.0f / sqrtf(ss / (float)rank + eps);
  // the row goes into the paged cache and, when asked for, into a dense copy [ntok, rank + rd] as well
  for (int copy = 0; copy < 2; ++copy) {
    T* row;
    if (copy == 0) {
      if (cache == nullptr) continue;
      const int slot = seq_slot[tok_seq[t]];
      const int page = page_table[(size_t)slot * table_width + (pos / page_size) % table_width];
      row = cache + ((size_t)page * page_size + pos % page_size) * (size_t)(rank + rd);
    } else {
      if (dense == nullptr) continue;
      row = dense + (size_t)t * ldd;
    }
    for (int i = tid; i < rank; i += blockDim.x) row[i] = from_f32<T>(kv[i] * rstd * norm_w[i]);
    // the shared rotated key part: pairs below `rot` turn, the rest passes
    for (int i = tid; i < rd / 2 + (rd & 1); i += blockDim.x) {
      const int a = 2 * i, b = 2 * i + 1;
      if (b < rot) {
        float u, v;
        rotate_pair(kv[rank + a], kv[rank + b], fpos * inv_freq[i], u, v);
        row[rank + a] = from_f32<T>(u);
        row[rank + b] = from_f32<T>(v);
      } else {
        row[rank + a] = from_f32<T>(kv[rank + a]);
        if (b < rd) row[rank + b] = from_f32<T>(kv[rank + b]);
      }
    }
  }
  // queries: the unrotated dims go to the absorbing product, the rotated ones straight into qa
  const float* q = q_in + (size_t)t * ldq;
  const int qd = dim + rd;
  for (int e = tid; e < H * dim; e += blockDim.x) {
    const int h = e / dim, d = e % dim;
    q_nope[(size_t)t * ldqn + e] = from_f32<T>(q[h * qd + d] * q_scale);
  }
  const int halves = rd / 2 + (rd & 1);
  for (int e = tid; e < H * halves; e += blockDim.x) {
    const int h = e / halves, i = e % halves;
    const int a = 2 * i, b = 2 * i + 1;
    const float* src = q + h * qd + dim;
    T* dst = q_lat + (size_t)t * ldql + (size_t)h * (rank + rd) + rank;
    if (b < rot) {
      float u, v;
      rotate_pair(src[a], src[b], fpos * inv_freq[i], u, v);
      dst[a] = from_f32<T>(u * q_scale);
      dst[b] = from_f32<T>(v * q_scale);
    } else {
      dst[a] = from_f32<T>(src[a] * q_scale);
      if (b < rd) dst[b] = from_f32<T>(src[b] * q_scale);
    }
  }
  if (g_in != nullptr)
    for (int h = tid; h < H; h += blockDim.x) gate[(size_t)t * H + h] = 1.0f / (1.0f + expf(-g_in[(size_t)t * ldg + h]));
}

GB_EXPORT int gb_latent_prepare(const float* q_in, long long ldq, const float* kv_in, long long ldkv, const float* g_in,
                                long long ldg, const float* norm_w, float eps, const float* inv_freq, int rot,
                                float q_scale, void* q_nope, long long ldqn, void* q_lat, long long ldql, float* gate,
                                void* cache, int dtype, const int* page_table, int table_width, int page_size,
                                const int* tok_pos, const int* tok_seq, const int* seq_slot, int ntok, int H, int dim,
                                int rd, int rank, void* dense, long long ldd, cudaStream_t stream) {
  if (ntok <= 0) return 0;
  if (H <= 0 || dim < 0 || rd < 0 || rank <= 0 || rot < 0 || rot > rd || (rot & 1)) return GB_ERR_SIZE;
  if (rot > 0 && inv_freq == nullptr) return GB_ERR_ARG;
#define LAUNCH(T)                                                                                                     \
  gb_launch(latent_prepare_kernel<T>, dim3(ntok), dim3(256), 0, stream, q_in, ldq, kv_in, ldkv, g_in, ldg, norm_w, eps, \
            inv_freq, rot, q_scale, (T*)q_nope, ldqn, (T*)q_lat, ldql, gate, (T*)cache, page_table, table_width,       \
            page_size, tok_pos, tok_seq, seq_slot, H, dim, rd, rank, (T*)dense, ldd)
  if (dtype == GB_F32) LAUNCH(float);
  else if (dtype == GB_BF16) LAUNCH(bf16);
  else return GB_ERR_DTYPE;
#undef LAUNCH
  return gb_launch_status();
}

// ---------------------------------------------------------------------------------------------
// y[t, h, n] = scale[t, h] * sum_k x[t, h, k] * w[h, n, k]: one product per head, FFMA with
// float32 accumulation in ascending k (a row's result does not depend on the other rows).
constexpr int HB = 64, HK = 16;

template <typename TI, typename TO>
__global__ void __launch_bounds__(256) heads_gemm_kernel(const TI* __restrict__ x, long long ldx_t, long long ldx_h,
                                                         const TI* __restrict__ w, TO* __restrict__ y, long long ldy_t,
                                                         long long ldy_h, const float* __restrict__ scale, int M, int H,
                                                         int N, int K) {
  pdl_release_next();
  pdl_wait_prior();
  __shared__ float xs[HK][HB + 4];
  __shared__ float ws[HK][HB + 4];
  const int tid = threadIdx.x, h = blockIdx.z;
  const int m0 = blockIdx.y * HB, n0 = blockIdx.x * HB;
  const int tm = (tid / 16) * 4, tn = (tid % 16) * 4;
  const TI* xh = x + (size_t)h * ldx_h;
  const TI* wh = w + (size_t)h * N * K;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < K; k0 += HK) {
    for (int e = tid; e < HB * HK; e += 256) {
      const int r = e / HK, c = e % HK;
      const int gm = m0 + r, gk = k0 + c, gn = n0 + r;
      xs[c][r] = (gm < M && gk < K) ? to_f32(xh[(size_t)gm * ldx_t + gk]) : 0.f;
      ws[c][r] = (gn < N && gk < K) ? to_f32(wh[(size_t)gn * K + gk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < HK; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = xs[kk][tm + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = ws[kk][tn + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int gm = m0 + tm + i;
    if (gm >= M) continue;
    const float s = scale ? scale[(size_t)gm * H + h] : 1.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gn = n0 + tn + j;
      if (gn < N) y[(size_t)gm * ldy_t + (size_t)h * ldy_h + gn] = from_f32<TO>(acc[i][j] * s);
    }
  }
}

GB_EXPORT int gb_heads_gemm(const void* x, long long ldx_t, long long ldx_h, const void* w, void* y, long long ldy_t,
                            long long ldy_h, const float* scale, int dtype, int M, int H, int N, int K,
                            cudaStream_t stream) {
  if (M <= 0 || H <= 0 || N <= 0) return 0;
  if (K <= 0 || H > 65535) return GB_ERR_SIZE;
  dim3 grid((N + HB - 1) / HB, (M + HB - 1) / HB, H);
  if (dtype == GB_F32)
    gb_launch(heads_gemm_kernel<float, float>, grid, dim3(256), 0, stream, (const float*)x, ldx_t, ldx_h, (const float*)w,
              (float*)y, ldy_t, ldy_h, scale, M, H, N, K);
  else if (dtype == GB_BF16)
    gb_launch(heads_gemm_kernel<bf16, bf16>, grid, dim3(256), 0, stream, (const bf16*)x, ldx_t, ldx_h, (const bf16*)w,
              (bf16*)y, ldy_t, ldy_h, scale, M, H, N, K);
  else
    return GB_ERR_DTYPE;
  return gb_launch_status();
}

// ---------------------------------------------------------------------------------------------
// Attention over the cached rows, one block per (token, head); online softmax over chunks of
// 128 keys from the window's first key (key 0 without a window).
constexpr int CHUNK = 128;
constexpr int MAX_U = 8;      // rank <= MAX_U * CHUNK

template <typename T>
__global__ void __launch_bounds__(CHUNK) latent_attention_ref_kernel(
    const T* __restrict__ qa, long long ldq, T* __restrict__ out, long long ldo, const T* __restrict__ cache,
    const int* __restrict__ page_table, int table_width, int page_size, const int* __restrict__ tok_pos,
    const int* __restrict__ tok_seq, const int* __restrict__ seq_slot, int rank, int rd, int window) {
  extern __shared__ float smem[];
  pdl_release_next();
  pdl_wait_prior();
  const int kd = rank + rd;
  float* qs = smem;                    // [kd]
  float* p = qs + kd;                  // [CHUNK]
  float* scratch = p + CHUNK;          // [34]
  size_t* rows = (size_t*)(((uintptr_t)(scratch + 34) + 7) & ~(uintptr_t)7);   // [CHUNK]
  const int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const int pos = tok_pos[t];
  const int slot = seq_slot[tok_seq[t]];
  const int hi = pos + 1;
  const int lo = window > 0 ? max(0, hi - window) : 0;
  const T* qrow = qa + (size_t)t * ldq + (size_t)h * kd;
  for (int i = tid; i < kd; i += CHUNK) qs[i] = to_f32(qrow[i]);
  __syncthreads();
  float m = -INFINITY, l = 0.f, acc[MAX_U];
#pragma unroll
  for (int u = 0; u < MAX_U; ++u) acc[u] = 0.f;
  for (int c0 = lo; c0 < hi; c0 += CHUNK) {
    const int j = c0 + tid;
    float s = -INFINITY;
    if (j < hi) {
      const int page = page_table[(size_t)slot * table_width + (j / page_size) % table_width];
      const size_t r = ((size_t)page * page_size + j % page_size) * (size_t)kd;
      rows[tid] = r;
      const T* kr = cache + r;
      float d = 0.f;
      for (int i = 0; i < kd; ++i) d = fmaf(qs[i], to_f32(kr[i]), d);
      s = d;
    }
    const float m_new = fmaxf(m, block_max(s, scratch));
    const float pj = j < hi ? expf(s - m_new) : 0.f;
    p[tid] = pj;
    const float csum = block_sum(pj, scratch);   // also orders the writes of p and rows
    const float alpha = expf(m - m_new);
    l = l * alpha + csum;
    const int n = min(CHUNK, hi - c0);
#pragma unroll
    for (int u = 0; u < MAX_U; ++u) {
      const int d = tid + u * CHUNK;
      if (d < rank) {
        float a = acc[u] * alpha;
        for (int jj = 0; jj < n; ++jj) a = fmaf(p[jj], to_f32(cache[rows[jj] + d]), a);
        acc[u] = a;
      }
    }
    m = m_new;
    __syncthreads();
  }
  T* orow = out + (size_t)t * ldo + (size_t)h * rank;
#pragma unroll
  for (int u = 0; u < MAX_U; ++u) {
    const int d = tid + u * CHUNK;
    if (d < rank) orow[d] = from_f32<T>(acc[u] / l);
  }
}

// qa: [ntok, H, rank + rd] rows ldq apart; out: [ntok, H, rank] rows ldo apart;
// cache: [pages, page_size, rank + rd].
GB_EXPORT int gb_latent_attention_ref(const void* qa, long long ldq, void* out, long long ldo, int dtype, const void* cache,
                                      const int* page_table, int table_width, int page_size, const int* tok_pos,
                                      const int* tok_seq, const int* seq_slot, int ntok, int H, int rank, int rd,
                                      int window, cudaStream_t stream) {
  if (ntok <= 0) return 0;
  if (rank <= 0 || rank > MAX_U * CHUNK || rd < 0 || H <= 0 || H > 65535) return GB_ERR_SIZE;
  const size_t smem = (size_t)(rank + rd + CHUNK + 34) * sizeof(float) + CHUNK * sizeof(size_t) + 8;
  if (smem > 48 * 1024) return GB_ERR_SIZE;
  dim3 grid(ntok, H);
#define LAUNCH(T)                                                                                                      \
  gb_launch(latent_attention_ref_kernel<T>, grid, dim3(CHUNK), smem, stream, (const T*)qa, ldq, (T*)out, ldo,          \
            (const T*)cache, page_table, table_width, page_size, tok_pos, tok_seq, seq_slot, rank, rd, window)
  if (dtype == GB_F32) LAUNCH(float);
  else if (dtype == GB_BF16) LAUNCH(bf16);
  else return GB_ERR_DTYPE;
#undef LAUNCH
  return gb_launch_status();
}

// ---------------------------------------------------------------------------------------------
// Stand-alone rotation of interleaved pairs, in place: x [ntok, heads, hd], the first `rot` dims
// of every head.
template <typename T>
__global__ void rope_pairs_kernel(T* __restrict__ x, long long ldx, const int* __restrict__ tok_pos,
                                  const float* __restrict__ inv_freq, int heads, int hd, int rot) {
  pdl_release_next();
  pdl_wait_prior();
  const int t = blockIdx.x;
  const float fpos = (float)tok_pos[t];
  const int half = rot / 2;
  for (int e = threadIdx.x; e < heads * half; e += blockDim.x) {
    const int h = e / half, i = e % half;
    T* v = x + (size_t)t * ldx + (size_t)h * hd + 2 * i;
    float a, b;
    rotate_pair(to_f32(v[0]), to_f32(v[1]), fpos * inv_freq[i], a, b);
    v[0] = from_f32<T>(a);
    v[1] = from_f32<T>(b);
  }
}

GB_EXPORT int gb_rope_pairs(void* x, long long ldx, int dtype, const int* tok_pos, const float* inv_freq, int ntok,
                            int heads, int hd, int rot, cudaStream_t stream) {
  if (ntok <= 0 || rot <= 0) return 0;
  if (rot > hd || (rot & 1)) return GB_ERR_SIZE;
  if (dtype == GB_F32)
    gb_launch(rope_pairs_kernel<float>, dim3(ntok), dim3(128), 0, stream, (float*)x, ldx, tok_pos, inv_freq, heads, hd, rot);
  else if (dtype == GB_BF16)
    gb_launch(rope_pairs_kernel<bf16>, dim3(ntok), dim3(128), 0, stream, (bf16*)x, ldx, tok_pos, inv_freq, heads, hd, rot);
  else
    return GB_ERR_DTYPE;
  return gb_launch_status();
}
