// Routed feed-forward (mixture of experts): the router and the token-major expert kernels.
//
//   z[t, e]  = router[e] . h[t] + bias[e]                       (float32)
//   chosen   = the `top` largest z (the lower index wins a tie); weight = softmax over the chosen z
//   expert:    g = min(gate h, limit), u = clamp(up h, -limit, limit)
//              y = g * sigmoid(alpha g) * (u + shift);  out = down y
//   residual[t] += sum over chosen of weight * expert_e(h[t])  +  sigmoid(sg . h[t]) * shared(h[t])
//
// Token-major: a block owns one (token, chosen expert) pair and a run of the expert's features,
// so the kernels need nothing from the host about who chose what and run inside captured steps.
// A token's experts are added in the order of its chosen list, then the shared expert: the same
// bits whatever else is in the batch.  All sums are float32.
#include "common.cuh"

template <typename T> struct Vec;
template <> struct Vec<float> { static constexpr int N = 4; typedef float4 type; };
template <> struct Vec<bf16> { static constexpr int N = 8; typedef uint4 type; };

__device__ __forceinline__ void unpack(const float4& v, float* f) { f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w; }
__device__ __forceinline__ void unpack(const uint4& v, float* f) {
  const __nv_bfloat162* p = (const __nv_bfloat162*)&v;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 a = __bfloat1622float2(p[i]);
    f[2 * i] = a.x;
    f[2 * i + 1] = a.y;
  }
}

// Lane's share of row . xs (xs float32 in shared memory); the caller adds the lanes with warp_sum.
// `vec`: the row starts on a 16-byte boundary and n is a multiple of the vector width.
template <typename T>
__device__ __forceinline__ float lane_dot(const T* __restrict__ row, const float* __restrict__ xs, int n, int lane, bool vec) {
  float acc = 0.f;
  if (vec) {
    constexpr int V = Vec<T>::N;
    const typename Vec<T>::type* r = (const typename Vec<T>::type*)row;
    for (int i = lane; i < n / V; i += 32) {
      float f[V];
      unpack(r[i], f);
#pragma unroll
      for (int k = 0; k < V; ++k) acc = fmaf(f[k], xs[i * V + k], acc);
    }
  } else {
    for (int i = lane; i < n; i += 32) acc = fmaf(to_f32(row[i]), xs[i], acc);
  }
  return acc;
}

template <typename T> __device__ __forceinline__ bool rows_vectorize(const T* base, int n) {
  return n % Vec<T>::N == 0 && ((uintptr_t)base & 15) == 0;
}

// ---- router: one block of 128 threads per token
template <typename T>
__global__ void __launch_bounds__(128) moe_route_kernel(const T* __restrict__ h, long long ldh,
                                                        const float* __restrict__ router, const float* __restrict__ bias,
                                                        const float* __restrict__ sg_w, int* __restrict__ idx,
                                                        float* __restrict__ wts, float* __restrict__ sg, int width, int E,
                                                        int top) {
  extern __shared__ float smem[];
  pdl_release_next();
  pdl_wait_prior();
  float* xs = smem;              // [width]
  float* z = smem + width;       // [E]
  const int t = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  for (int i = tid; i < width; i += 128) xs[i] = to_f32(h[(size_t)t * ldh + i]);
  __syncthreads();
  const bool vec = rows_vectorize(router, width);
  for (int e = warp; e < E + (sg_w ? 1 : 0); e += 4) {
    const float* row = e < E ? router + (size_t)e * width : sg_w;
    const float d = warp_sum(lane_dot(row, xs, width, lane, vec && rows_vectorize(row, width)));
    if (lane == 0) {
      if (e < E) z[e] = d + (bias ? bias[e] : 0.f);
      else sg[t] = 1.0f / (1.0f + expf(-d));
    }
  }
  __syncthreads();
  if (warp != 0) return;
  float mine = 0.f, first = 0.f, sum = 0.f;   // lane k keeps the k-th chosen logit
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY;
    int at = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      const float v = z[e];
      if (v > best || (v == best && e < at)) { best = v; at = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, at, o);
      if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
    }
    if (k == 0) first = best;
    if (lane == k) mine = best;
    if (lane == 0) {
      idx[(size_t)t * top + k] = at < E ? at : 0;
      if (at < E) z[at] = -INFINITY;
    }
    __syncwarp();
  }
  const float e = lane < top ? expf(mine - first) : 0.f;
  sum = warp_sum(e);
  if (lane < top) wts[(size_t)t * top + lane] = e / sum;
}

// ---- gate and up of one (token, slot): FEATS features a block, a warp per feature in turn
constexpr int FEATS = 32;

template <typename T>
__global__ void __launch_bounds__(256) moe_gate_up_kernel(const T* __restrict__ h, long long ldh,
                                                          const int* __restrict__ idx, const T* __restrict__ w_gu,
                                                          const T* __restrict__ ws_gu, T* __restrict__ y, int width,
                                                          int ff, int ffs, int ffmax, int top, int slots, float limit,
                                                          float limit_s, float alpha, float shift) {
  extern __shared__ float xs[];   // [width]
  pdl_release_next();
  pdl_wait_prior();
  const int t = blockIdx.x / slots, s = blockIdx.x % slots;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const bool routed = s < top;
  const int nf = routed ? ff : ffs;
  const int f0 = blockIdx.y * FEATS;
  if (f0 >= nf) return;
  const T* W = routed ? w_gu + (size_t)idx[(size_t)t * top + s] * 2 * ff * width : ws_gu;
  const float lim = routed ? limit : limit_s;
  for (int i = tid; i < width; i += 256) xs[i] = to_f32(h[(size_t)t * ldh + i]);
  __syncthreads();
  const bool vec = rows_vectorize(W, width);
  for (int f = f0 + warp; f < min(nf, f0 + FEATS); f += 8) {
    float g = warp_sum(lane_dot(W + (size_t)f * width, xs, width, lane, vec));
    float u = warp_sum(lane_dot(W + (size_t)(nf + f) * width, xs, width, lane, vec));
    if (lane == 0) {
      g = fminf(g, lim);
      u = fminf(fmaxf(u, -lim), lim);
      const float a = g / (1.0f + expf(-alpha * g)) * (u + shift);
      y[((size_t)t * slots + s) * ffmax + f] = from_f32<T>(a);
    }
  }
}

// ---- down of all of a token's slots, weighted and added into the residual
template <typename T>
__global__ void __launch_bounds__(256) moe_down_kernel(const T* __restrict__ y, const int* __restrict__ idx,
                                                       const float* __restrict__ wts, const float* __restrict__ sg,
                                                       const T* __restrict__ w_d, const T* __restrict__ ws_d,
                                                       float* __restrict__ residual, long long ldr, int width, int ff,
                                                       int ffs, int ffmax, int top, int slots) {
  extern __shared__ float ys[];   // [slots, ffmax]
  pdl_release_next();
  pdl_wait_prior();
  const int t = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  for (int i = tid; i < slots * ffmax; i += 256) ys[i] = to_f32(y[(size_t)t * slots * ffmax + i]);
  __syncthreads();
  const int n0 = blockIdx.y * FEATS;
  for (int n = n0 + warp; n < min(width, n0 + FEATS); n += 8) {
    float total = 0.f;
    for (int s = 0; s < slots; ++s) {
      const bool routed = s < top;
      const int nf = routed ? ff : ffs;
      const T* row = routed ? w_d + ((size_t)idx[(size_t)t * top + s] * width + n) * ff : ws_d + (size_t)n * ffs;
      const float d = warp_sum(lane_dot(row, ys + (size_t)s * ffmax, nf, lane, rows_vectorize(row, nf) && ffmax % 4 == 0));
      total += d * (routed ? wts[(size_t)t * top + s] : sg[t]);
    }
    if (lane == 0) residual[(size_t)t * ldr + n] += total;
  }
}

GB_EXPORT int gb_moe_route(const void* h, long long ldh, int dtype, const float* router, const float* bias,
                           const float* sg_w, int* idx, float* wts, float* sg, int ntok, int width, int E, int top,
                           cudaStream_t stream) {
  if (ntok <= 0) return 0;
  if (E <= 0 || top <= 0 || top > 32 || top > E || width <= 0) return GB_ERR_SIZE;
  const size_t smem = (size_t)(width + E) * sizeof(float);
  if (smem > 48 * 1024) return GB_ERR_SIZE;
  if (dtype == GB_F32)
    gb_launch(moe_route_kernel<float>, dim3(ntok), dim3(128), smem, stream, (const float*)h, ldh, router, bias, sg_w, idx,
              wts, sg, width, E, top);
  else if (dtype == GB_BF16)
    gb_launch(moe_route_kernel<bf16>, dim3(ntok), dim3(128), smem, stream, (const bf16*)h, ldh, router, bias, sg_w, idx,
              wts, sg, width, E, top);
  else
    return GB_ERR_DTYPE;
  return gb_launch_status();
}

// w_gu: [E, 2 ff, width] (an expert's gate rows, then its up rows); ws_gu: [2 ffs, width] or null;
// y: [ntok, slots, ffmax], slots = top (+ 1 with a shared expert), ffmax = max(ff, ffs).
GB_EXPORT int gb_moe_gate_up(const void* h, long long ldh, int dtype, const int* idx, const void* w_gu, const void* ws_gu,
                             void* y, int ntok, int width, int ff, int ffs, int top, float limit, float limit_s,
                             float alpha, float shift, cudaStream_t stream) {
  if (ntok <= 0) return 0;
  const int slots = top + (ws_gu ? 1 : 0), ffmax = ff > ffs ? ff : ffs;
  if (width <= 0 || ffmax <= 0 || slots <= 0) return GB_ERR_SIZE;
  const size_t smem = (size_t)width * sizeof(float);
  if (smem > 48 * 1024) return GB_ERR_SIZE;
  dim3 grid(ntok * slots, (ffmax + FEATS - 1) / FEATS);
  if (dtype == GB_F32)
    gb_launch(moe_gate_up_kernel<float>, grid, dim3(256), smem, stream, (const float*)h, ldh, idx, (const float*)w_gu,
              (const float*)ws_gu, (float*)y, width, ff, ffs, ffmax, top, slots, limit, limit_s, alpha, shift);
  else if (dtype == GB_BF16)
    gb_launch(moe_gate_up_kernel<bf16>, grid, dim3(256), smem, stream, (const bf16*)h, ldh, idx, (const bf16*)w_gu,
              (const bf16*)ws_gu, (bf16*)y, width, ff, ffs, ffmax, top, slots, limit, limit_s, alpha, shift);
  else
    return GB_ERR_DTYPE;
  return gb_launch_status();
}

// w_d: [E, width, ff]; ws_d: [width, ffs] or null; residual: float32 [ntok, width] rows ldr apart.
GB_EXPORT int gb_moe_down(const void* y, int dtype, const int* idx, const float* wts, const float* sg, const void* w_d,
                          const void* ws_d, float* residual, long long ldr, int ntok, int width, int ff, int ffs, int top,
                          cudaStream_t stream) {
  if (ntok <= 0) return 0;
  const int slots = top + (ws_d ? 1 : 0), ffmax = ff > ffs ? ff : ffs;
  if (width <= 0 || ffmax <= 0 || slots <= 0) return GB_ERR_SIZE;
  const size_t smem = (size_t)slots * ffmax * sizeof(float);
  if (smem > 200 * 1024) return GB_ERR_SIZE;
  dim3 grid(ntok, (width + FEATS - 1) / FEATS);
  if (dtype == GB_F32) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(moe_down_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    gb_launch(moe_down_kernel<float>, grid, dim3(256), smem, stream, (const float*)y, idx, wts, sg, (const float*)w_d,
              (const float*)ws_d, residual, ldr, width, ff, ffs, ffmax, top, slots);
  } else if (dtype == GB_BF16) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(moe_down_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    gb_launch(moe_down_kernel<bf16>, grid, dim3(256), smem, stream, (const bf16*)y, idx, wts, sg, (const bf16*)w_d,
              (const bf16*)ws_d, residual, ldr, width, ff, ffs, ffmax, top, slots);
  } else {
    return GB_ERR_DTYPE;
  }
  return gb_launch_status();
}
