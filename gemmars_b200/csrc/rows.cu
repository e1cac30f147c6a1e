// Row-wise kernels around the residual stream that the pre-norm models do not need:
//  * a second table added to the stream by an index per token (learned position vectors);
//  * an RMSNorm applied to a sublayer's OUTPUT and added into the stream (norms on both sides of
//    a sublayer): x[t] += y[t] * (mean(y[t]^2) + eps)^-1/2 * w;
//  * the gated activation act(g) * u for a choice of act;
//  * a scale on float32 rows (logits).
// Statistics, sums and the activation's arithmetic are float32.
#include "common.cuh"

enum { ACT_SILU = 0, ACT_GELU_TANH = 1 };

// x[t, :] += table[idx[t], :]
template <typename W>
__global__ void gather_add_kernel(const W* __restrict__ table, const int* __restrict__ idx, float* __restrict__ x,
                                  int hidden, int rows) {
  pdl_release_next();
  pdl_wait_prior();
  const int t = blockIdx.x;
  int id = idx[t];
  id = id < 0 ? 0 : (id >= rows ? rows - 1 : id);   // the host refuses positions beyond the table; never read outside
  const W* row = table + (size_t)id * hidden;
  float* out = x + (size_t)t * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) out[i] += to_f32(row[i]);
}

GB_EXPORT int gb_gather_add(const void* table, int table_dtype, const int* idx, float* x, int ntok, int hidden, int rows,
                            cudaStream_t stream) {
  if (ntok <= 0) return 0;
  const int threads = hidden >= 1024 ? 256 : 128;
  if (table_dtype == GB_F32)
    gb_launch(gather_add_kernel<float>, ntok, threads, 0, stream, (const float*)table, idx, x, hidden, rows);
  else if (table_dtype == GB_BF16)
    gb_launch(gather_add_kernel<bf16>, ntok, threads, 0, stream, (const bf16*)table, idx, x, hidden, rows);
  else
    return GB_ERR_DTYPE;
  return gb_launch_status();
}

// x[t, :] += y[t, :] * rstd(y[t]) * w, and, when a second weight is given, the norm that reads the
// stream next in the same pass: h[t, :] = x[t, :] * rstd(x[t]) * w2 (x the row after the add).  One
// block a row; the row is kept in registers between the passes where it fits (rows up to 8 floats a
// thread), else read again.  The order of the additions depends on n and the block size alone.
template <typename O>
__global__ void __launch_bounds__(512) rmsnorm_add_kernel(const float* __restrict__ y, const float* __restrict__ w,
                                                          float* __restrict__ x, int n, float eps, const float* __restrict__ w2,
                                                          O* __restrict__ h, float eps2) {
  __shared__ float scratch[33];
  pdl_release_next();
  pdl_wait_prior();
  constexpr int KEEP = 8;
  const float* row = y + (size_t)blockIdx.x * n;
  float* out = x + (size_t)blockIdx.x * n;
  const bool keep = n <= KEEP * (int)blockDim.x;
  float held[KEEP], ss = 0.f;
  if (keep) {
#pragma unroll
    for (int u = 0; u < KEEP; ++u) {
      const int i = threadIdx.x + u * blockDim.x;
      held[u] = i < n ? row[i] : 0.f;
      ss = fmaf(held[u], held[u], ss);
    }
  } else {
    for (int i = threadIdx.x; i < n; i += blockDim.x) ss = fmaf(row[i], row[i], ss);
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)n + eps);
  float ss2 = 0.f;
  if (keep) {
#pragma unroll
    for (int u = 0; u < KEEP; ++u) {
      const int i = threadIdx.x + u * blockDim.x;
      if (i < n) {
        held[u] = out[i] + held[u] * inv * w[i];
        out[i] = held[u];
        ss2 = fmaf(held[u], held[u], ss2);
      }
    }
  } else {
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      const float v = out[i] + row[i] * inv * w[i];
      out[i] = v;
      ss2 = fmaf(v, v, ss2);
    }
  }
  if (!w2) return;
  ss2 = block_sum(ss2, scratch);
  const float inv2 = 1.0f / sqrtf(ss2 / (float)n + eps2);
  O* hrow = h + (size_t)blockIdx.x * n;
  if (keep) {
#pragma unroll
    for (int u = 0; u < KEEP; ++u) {
      const int i = threadIdx.x + u * blockDim.x;
      if (i < n) hrow[i] = from_f32<O>(held[u] * inv2 * w2[i]);
    }
  } else {
    for (int i = threadIdx.x; i < n; i += blockDim.x) hrow[i] = from_f32<O>(out[i] * inv2 * w2[i]);
  }
}

// w2, h (of h_dtype), eps2: the following norm, or null.
GB_EXPORT int gb_rmsnorm_add(const float* y, const float* w, float* x, int rows, int n, float eps, const float* w2, void* h,
                             int h_dtype, float eps2, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (n <= 0) return GB_ERR_SIZE;
  const int threads = n >= 2048 ? 512 : (n >= 512 ? 256 : 128);
  if (w2 && h_dtype == GB_BF16)
    gb_launch(rmsnorm_add_kernel<bf16>, rows, threads, 0, stream, y, w, x, n, eps, w2, (bf16*)h, eps2);
  else if (!w2 || h_dtype == GB_F32)
    gb_launch(rmsnorm_add_kernel<float>, rows, threads, 0, stream, y, w, x, n, eps, w2, (float*)h, eps2);
  else
    return GB_ERR_DTYPE;
  return gb_launch_status();
}

__device__ __forceinline__ float act_apply(float g, int act) {
  if (act == ACT_GELU_TANH) {
    // 0.5 g (1 + tanh(sqrt(2/pi) (g + 0.044715 g^3)))
    const float inner = 0.7978845608028654f * (g + 0.044715f * g * g * g);
    return 0.5f * g * (1.0f + tanhf(inner));
  }
  return g / (1.0f + expf(-g));
}

// out[t, i] = act(gu[t, i]) * gu[t, inter + i]
template <typename T>
__global__ void gated_act_kernel(const T* __restrict__ gu, T* __restrict__ out, long long total, int inter, int act) {
  pdl_release_next();
  pdl_wait_prior();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / inter;
    const int c = (int)(i - t * inter);
    const T* row = gu + t * 2 * inter;
    out[i] = from_f32<T>(act_apply(to_f32(row[c]), act) * to_f32(row[inter + c]));
  }
}

GB_EXPORT int gb_gated_act(const void* gu, void* out, int dtype, int ntok, int inter, int act, cudaStream_t stream) {
  if (ntok <= 0) return 0;
  if (act != ACT_SILU && act != ACT_GELU_TANH) return GB_ERR_ARG;
  const long long total = (long long)ntok * inter;
  const int blocks = (int)((total + 255) / 256 < 4096 ? (total + 255) / 256 : 4096);
  if (dtype == GB_F32)
    gb_launch(gated_act_kernel<float>, blocks, 256, 0, stream, (const float*)gu, (float*)out, total, inter, act);
  else if (dtype == GB_BF16)
    gb_launch(gated_act_kernel<bf16>, blocks, 256, 0, stream, (const bf16*)gu, (bf16*)out, total, inter, act);
  else
    return GB_ERR_DTYPE;
  return gb_launch_status();
}

__global__ void scale_kernel(float* __restrict__ y, long long total, float s) {
  pdl_release_next();
  pdl_wait_prior();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x)
    y[i] *= s;
}

GB_EXPORT int gb_scale_f32(float* y, long long total, float s, cudaStream_t stream) {
  if (total <= 0) return 0;
  const int blocks = (int)((total + 255) / 256 < 2048 ? (total + 255) / 256 : 2048);
  gb_launch(scale_kernel, blocks, 256, 0, stream, y, total, s);
  return gb_launch_status();
}
