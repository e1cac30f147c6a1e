// Kernels of the mixers that carry a fixed-size state from token to token: the short causal
// filter over time, the gated delta rule, the selective state-space recurrence with a scalar
// decay per head, and the gated RMS norm over groups of channels that follows them.
//
// A step's tokens are packed; sequence b owns rows cu[b] .. cu[b+1]-1 and the state row
// seq_slot[b].  Every kernel walks a sequence's rows in order on the device, so a whole prompt, a
// part of one and a single token run the same arithmetic, and a captured step needs no host.
// Rows that pad a captured step carry the spare slot, whose state row nobody reads.
//
// States and everything that enters a recurrence are float32: decays, step sizes, gates of the
// recurrence, unit norms.  Inputs are the float32 results of the projections.
#include "common.cuh"

constexpr int MAX_TAPS = 8;
enum { ACT_NONE = 0, ACT_SILU = 1 };

__device__ __forceinline__ float sigmoid_f(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.0f ? z : log1pf(expf(z)); }

// ------------------------------------------------------------------ short causal filter
// y[t, c] = act(bias[c] + sum_j taps[c, j] * u[t - (K-1) + j, c]); rows before the step's first
// row of the sequence come from the K-1 rows kept in the state (oldest first), which are zero
// for a new sequence.
template <typename T>
__device__ __forceinline__ float filter_input(const T* __restrict__ u, long long ldu, int row0, int local,
                                              const float* __restrict__ hist, int C, int c, int K) {
  return local >= 0 ? to_f32(u[(size_t)(row0 + local) * ldu + c]) : hist[(size_t)(K - 1 + local) * C + c];
}

template <typename T, typename O>
__global__ void __launch_bounds__(256) short_filter_kernel(const T* __restrict__ u, long long ldu, const float* __restrict__ taps,
                                                          const float* __restrict__ bias, const float* __restrict__ state,
                                                          const int* __restrict__ cu, const int* __restrict__ tok_seq,
                                                          const int* __restrict__ seq_slot, O* __restrict__ out, long long ldo,
                                                          int C, int K, int act) {
  pdl_release_next();
  pdl_wait_prior();
  const int t = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int b = tok_seq[t], row0 = cu[b], local = t - row0;
  const float* hist = state + (size_t)seq_slot[b] * (K - 1) * C;
  float acc = bias ? bias[c] : 0.f;
  for (int j = 0; j < K; ++j)
    acc = fmaf(taps[(size_t)c * K + j], filter_input(u, ldu, row0, local - (K - 1) + j, hist, C, c, K), acc);
  if (act == ACT_SILU) acc = silu_f(acc);
  out[(size_t)t * ldo + c] = from_f32<O>(acc);
}

// The state after the step: the last K-1 inputs of the sequence, old rows shifted where the step
// brought fewer than K-1.
template <typename T>
__global__ void __launch_bounds__(256) short_filter_state_kernel(const T* __restrict__ u, long long ldu, float* __restrict__ state,
                                                                const int* __restrict__ cu, const int* __restrict__ seq_slot,
                                                                int C, int K) {
  pdl_release_next();
  pdl_wait_prior();
  const int b = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int row0 = cu[b], n = cu[b + 1] - row0;
  float* hist = state + (size_t)seq_slot[b] * (K - 1) * C;
  float next[MAX_TAPS - 1];
#pragma unroll
  for (int i = 0; i < MAX_TAPS - 1; ++i)
    if (i < K - 1) next[i] = filter_input(u, ldu, row0, n - (K - 1) + i, hist, C, c, K);
#pragma unroll
  for (int i = 0; i < MAX_TAPS - 1; ++i)
    if (i < K - 1) hist[(size_t)i * C + c] = next[i];
}

GB_EXPORT int gb_short_filter(const void* u, int in_dtype, long long ldu, const float* taps, const float* bias, float* state,
                              const int* cu, const int* tok_seq, const int* seq_slot, void* out, int out_dtype, long long ldo,
                              int ntok, int nseq, int C, int K, int act, int update_state, cudaStream_t stream) {
  if (ntok <= 0) return 0;
  if (K < 1 || K > MAX_TAPS || C <= 0) return GB_ERR_SIZE;
  dim3 grid(ntok, (C + 255) / 256), sgrid(nseq, (C + 255) / 256);
#define GB_FILTER(T, O)                                                                                                   \
  gb_launch(short_filter_kernel<T, O>, grid, 256, 0, stream, (const T*)u, ldu, taps, bias, (const float*)state, cu, tok_seq, \
            seq_slot, (O*)out, ldo, C, K, act)
  if (in_dtype == GB_F32 && out_dtype == GB_F32) GB_FILTER(float, float);
  else if (in_dtype == GB_F32 && out_dtype == GB_BF16) GB_FILTER(float, bf16);
  else if (in_dtype == GB_BF16 && out_dtype == GB_BF16) GB_FILTER(bf16, bf16);
  else if (in_dtype == GB_BF16 && out_dtype == GB_F32) GB_FILTER(bf16, float);
  else return GB_ERR_DTYPE;
#undef GB_FILTER
  if (update_state && K > 1) {
    if (in_dtype == GB_F32)
      gb_launch(short_filter_state_kernel<float>, sgrid, 256, 0, stream, (const float*)u, ldu, state, cu, seq_slot, C, K);
    else
      gb_launch(short_filter_state_kernel<bf16>, sgrid, 256, 0, stream, (const bf16*)u, ldu, state, cu, seq_slot, C, K);
  }
  return gb_launch_status();
}

// Only the state update (for a caller whose own kernel has applied the filter).
GB_EXPORT int gb_short_filter_state(const void* u, int in_dtype, long long ldu, float* state, const int* cu,
                                    const int* seq_slot, int nseq, int C, int K, cudaStream_t stream) {
  if (nseq <= 0 || K <= 1) return 0;
  if (K > MAX_TAPS || C <= 0) return GB_ERR_SIZE;
  dim3 sgrid(nseq, (C + 255) / 256);
  if (in_dtype == GB_F32)
    gb_launch(short_filter_state_kernel<float>, sgrid, 256, 0, stream, (const float*)u, ldu, state, cu, seq_slot, C, K);
  else if (in_dtype == GB_BF16)
    gb_launch(short_filter_state_kernel<bf16>, sgrid, 256, 0, stream, (const bf16*)u, ldu, state, cu, seq_slot, C, K);
  else
    return GB_ERR_DTYPE;
  return gb_launch_status();
}

// Sums of up to three values over the block, the same in every thread.  One warp: shuffles alone.
__device__ __forceinline__ void block_sum3(float& a, float& b, float& c, float* red /* 3 * 32 */) {
  a = warp_sum(a); b = warp_sum(b); c = warp_sum(c);
  const int nwarp = (blockDim.x + 31) >> 5;
  if (nwarp == 1) return;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { red[warp * 3] = a; red[warp * 3 + 1] = b; red[warp * 3 + 2] = c; }
  __syncthreads();
  a = b = c = 0.f;
  for (int w = 0; w < nwarp; ++w) { a += red[w * 3]; b += red[w * 3 + 1]; c += red[w * 3 + 2]; }
}

// ------------------------------------------------------------------ gated delta rule
// One block per (sequence, head); thread j owns column j of the head's state S [D, V] in shared
// memory.  Per token, with k^ = k / sqrt(|k|^2 + 1e-6), q^ = q / sqrt(|q|^2 + 1e-6) * qscale,
// beta = sigmoid(bl), g = exp(-exp(A_log) * softplus(al + dt_bias)):
//   S <- g S;  u = beta (v - S^T k^);  S <- S + k^ u^T;  y = S^T q^
// The two products with the old state are taken in one pass (y = g S_old^T q^ + (k^ . q^) u).
// The next token's k, q and v are asked for before the current token is worked.
constexpr int PREFETCH = 8;   // D <= PREFETCH * threads

__global__ void delta_rule_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
                                  long long ld, const float* __restrict__ beta_logit, const float* __restrict__ a_logit,
                                  long long ldg, const float* __restrict__ A_log, const float* __restrict__ dt_bias,
                                  float* __restrict__ state, const int* __restrict__ cu, const int* __restrict__ seq_slot,
                                  float* __restrict__ y, int H, int G, int D, int V, float qscale) {
  extern __shared__ float sm[];
  float* S = sm;                 // [D][V]
  float* kq = S + (size_t)D * V; // two buffers of k[D], q[D]
  float* red = kq + 4 * D;       // 96
  pdl_release_next();
  pdl_wait_prior();
  const int b = blockIdx.x, head = blockIdx.y, g = head / (H / G), tid = threadIdx.x, nthr = blockDim.x;
  const int t0 = cu[b], t1 = cu[b + 1];
  float* Sg = state + ((size_t)seq_slot[b] * H + head) * D * V;
  for (int i = tid; i < D * V; i += nthr) S[i] = Sg[i];
  const float rate = expf(A_log[head]), dtb = dt_bias[head];
  float v_next = 0.f, bl_next = 0.f, al_next = 0.f;
  if (t0 < t1) {
    for (int i = tid; i < D; i += nthr) {
      kq[i] = k[(size_t)t0 * ld + g * D + i];
      kq[D + i] = q[(size_t)t0 * ld + g * D + i];
    }
    if (tid < V) v_next = v[(size_t)t0 * ld + head * V + tid];
    bl_next = beta_logit[(size_t)t0 * ldg + head];
    al_next = a_logit[(size_t)t0 * ldg + head];
  }
  __syncthreads();
  for (int t = t0; t < t1; ++t) {
    const int buf = (t - t0) & 1;
    const float* ks = kq + buf * 2 * D;
    const float* qs = ks + D;
    const float v_cur = v_next, bl = bl_next, al = al_next;
    float pk[PREFETCH], pq[PREFETCH];
    if (t + 1 < t1) {
#pragma unroll
      for (int r = 0; r < PREFETCH; ++r) {
        const int i = tid + r * nthr;
        if (i < D) {
          pk[r] = k[(size_t)(t + 1) * ld + g * D + i];
          pq[r] = q[(size_t)(t + 1) * ld + g * D + i];
        }
      }
      if (tid < V) v_next = v[(size_t)(t + 1) * ld + head * V + tid];
      bl_next = beta_logit[(size_t)(t + 1) * ldg + head];
      al_next = a_logit[(size_t)(t + 1) * ldg + head];
    }
    float kk = 0.f, qq = 0.f, kdq = 0.f;
    for (int i = tid; i < D; i += nthr) {
      kk = fmaf(ks[i], ks[i], kk);
      qq = fmaf(qs[i], qs[i], qq);
      kdq = fmaf(ks[i], qs[i], kdq);
    }
    block_sum3(kk, qq, kdq, red);
    const float inv_k = 1.0f / sqrtf(kk + 1e-6f), inv_q = qscale / sqrtf(qq + 1e-6f);
    const float beta = sigmoid_f(bl), decay = expf(-rate * softplus_f(al + dtb));
    if (tid < V) {
      float sk = 0.f, sq = 0.f;
      for (int d = 0; d < D; ++d) {
        const float s = S[d * V + tid];
        sk = fmaf(s, ks[d], sk);
        sq = fmaf(s, qs[d], sq);
      }
      const float u = beta * (v_cur - decay * inv_k * sk);
      const float ku = inv_k * u;
      for (int d = 0; d < D; ++d) S[d * V + tid] = fmaf(ks[d], ku, decay * S[d * V + tid]);
      y[(size_t)t * H * V + head * V + tid] = fmaf(kdq * inv_k * inv_q, u, decay * inv_q * sq);
    }
    if (t + 1 < t1) {
      float* nb = kq + (buf ^ 1) * 2 * D;
#pragma unroll
      for (int r = 0; r < PREFETCH; ++r) {
        const int i = tid + r * nthr;
        if (i < D) { nb[i] = pk[r]; nb[D + i] = pq[r]; }
      }
    }
    __syncthreads();
  }
  for (int i = tid; i < D * V; i += nthr) Sg[i] = S[i];
}

GB_EXPORT int gb_delta_rule(const float* q, const float* k, const float* v, long long ld, const float* beta_logit,
                            const float* a_logit, long long ldg, const float* A_log, const float* dt_bias, float* state,
                            const int* cu, const int* seq_slot, float* y, int nseq, int H, int G, int D, int V, float qscale,
                            cudaStream_t stream) {
  if (nseq <= 0) return 0;
  int threads = ((V + 31) / 32) * 32;
  if (G <= 0 || H % G || V <= 0 || threads > 1024 || D <= 0 || D > PREFETCH * threads) return GB_ERR_SIZE;
  const size_t smem = ((size_t)D * V + 4 * D + 96) * sizeof(float);
  if (smem > 200 * 1024) return GB_ERR_SIZE;
  static bool raised = false;
  if (!raised) {
    cudaFuncSetAttribute(delta_rule_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    raised = true;
  }
  gb_launch(delta_rule_kernel, dim3(nseq, H), threads, smem, stream, q, k, v, ld, beta_logit, a_logit, ldg, A_log, dt_bias,
            state, cu, seq_slot, y, H, G, D, V, qscale);
  return gb_launch_status();
}

// ------------------------------------------------------------------ selective state space, scalar decay per head
// One block per (sequence, head); thread j owns column j of S [N, V].  Per token, with
// dt = softplus(dt_raw + dt_bias):  S <- exp(-exp(A_log) dt) S + dt B x^T;  y = S^T C + D x.
__global__ void ssd_scan_kernel(const float* __restrict__ x, const float* __restrict__ Bm, const float* __restrict__ Cm,
                                long long ld, const float* __restrict__ dt_raw, long long ldd, const float* __restrict__ A_log,
                                const float* __restrict__ dt_bias, const float* __restrict__ skip, float* __restrict__ state,
                                const int* __restrict__ cu, const int* __restrict__ seq_slot, float* __restrict__ y, int H,
                                int G, int N, int V) {
  extern __shared__ float sm[];
  float* S = sm;                 // [N][V]
  float* bc = S + (size_t)N * V; // two buffers of B[N], C[N]
  pdl_release_next();
  pdl_wait_prior();
  const int b = blockIdx.x, head = blockIdx.y, g = head / (H / G), tid = threadIdx.x, nthr = blockDim.x;
  const int t0 = cu[b], t1 = cu[b + 1];
  float* Sg = state + ((size_t)seq_slot[b] * H + head) * N * V;
  for (int i = tid; i < N * V; i += nthr) S[i] = Sg[i];
  const float rate = expf(A_log[head]), dtb = dt_bias[head], dskip = skip[head];
  float x_next = 0.f, dt_next = 0.f;
  if (t0 < t1) {
    for (int i = tid; i < N; i += nthr) {
      bc[i] = Bm[(size_t)t0 * ld + g * N + i];
      bc[N + i] = Cm[(size_t)t0 * ld + g * N + i];
    }
    if (tid < V) x_next = x[(size_t)t0 * ld + head * V + tid];
    dt_next = dt_raw[(size_t)t0 * ldd + head];
  }
  __syncthreads();
  for (int t = t0; t < t1; ++t) {
    const int buf = (t - t0) & 1;
    const float* Bs = bc + buf * 2 * N;
    const float* Cs = Bs + N;
    const float xv = x_next, dt = softplus_f(dt_next + dtb);
    float pb[PREFETCH], pc[PREFETCH];
    if (t + 1 < t1) {
#pragma unroll
      for (int r = 0; r < PREFETCH; ++r) {
        const int i = tid + r * nthr;
        if (i < N) {
          pb[r] = Bm[(size_t)(t + 1) * ld + g * N + i];
          pc[r] = Cm[(size_t)(t + 1) * ld + g * N + i];
        }
      }
      if (tid < V) x_next = x[(size_t)(t + 1) * ld + head * V + tid];
      dt_next = dt_raw[(size_t)(t + 1) * ldd + head];
    }
    const float decay = expf(-rate * dt);
    if (tid < V) {
      const float dx = dt * xv;
      float acc = 0.f;
      for (int n = 0; n < N; ++n) {
        const float s = fmaf(Bs[n], dx, decay * S[n * V + tid]);
        S[n * V + tid] = s;
        acc = fmaf(s, Cs[n], acc);
      }
      y[(size_t)t * H * V + head * V + tid] = fmaf(dskip, xv, acc);
    }
    if (t + 1 < t1) {
      float* nb = bc + (buf ^ 1) * 2 * N;
#pragma unroll
      for (int r = 0; r < PREFETCH; ++r) {
        const int i = tid + r * nthr;
        if (i < N) { nb[i] = pb[r]; nb[N + i] = pc[r]; }
      }
    }
    __syncthreads();
  }
  for (int i = tid; i < N * V; i += nthr) Sg[i] = S[i];
}

GB_EXPORT int gb_ssd_scan(const float* x, const float* Bm, const float* Cm, long long ld, const float* dt_raw, long long ldd,
                          const float* A_log, const float* dt_bias, const float* skip, float* state, const int* cu,
                          const int* seq_slot, float* y, int nseq, int H, int G, int N, int V, cudaStream_t stream) {
  if (nseq <= 0) return 0;
  int threads = ((V + 31) / 32) * 32;
  if (G <= 0 || H % G || V <= 0 || threads > 1024 || N <= 0 || N > PREFETCH * threads) return GB_ERR_SIZE;
  const size_t smem = ((size_t)N * V + 4 * N) * sizeof(float);
  if (smem > 200 * 1024) return GB_ERR_SIZE;
  static bool raised = false;
  if (!raised) {
    cudaFuncSetAttribute(ssd_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    raised = true;
  }
  gb_launch(ssd_scan_kernel, dim3(nseq, H), threads, smem, stream, x, Bm, Cm, ld, dt_raw, ldd, A_log, dt_bias, skip, state, cu,
            seq_slot, y, H, G, N, V);
  return gb_launch_status();
}

// ------------------------------------------------------------------ gated RMS norm over groups of channels
// Row t of y [T, n] is cut into groups of gs channels, each divided by its own root mean square;
// channel i is weighed by w[i % wn] and gated by silu(gate[t, i]).  gate_first: the gate is
// multiplied in before the statistics are taken (the norm sees the gated values), else after.
template <typename O>
__global__ void __launch_bounds__(128) gated_group_norm_kernel(const float* __restrict__ y, const float* __restrict__ gate,
                                                              long long ldgate, const float* __restrict__ w, int wn,
                                                              O* __restrict__ out, int n, int gs, float eps, int gate_first,
                                                              float out_scale) {
  __shared__ float scratch[33];
  pdl_release_next();
  pdl_wait_prior();
  const int t = blockIdx.x, base = blockIdx.y * gs;
  const float* row = y + (size_t)t * n + base;
  const float* grow = gate + (size_t)t * ldgate + base;
  float ss = 0.f;
  for (int i = threadIdx.x; i < gs; i += blockDim.x) {
    const float val = gate_first ? row[i] * silu_f(grow[i]) : row[i];
    ss = fmaf(val, val, ss);
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)gs + eps);
  for (int i = threadIdx.x; i < gs; i += blockDim.x) {
    const float gt = silu_f(grow[i]);
    const float val = gate_first ? row[i] * gt * inv * w[(base + i) % wn] : row[i] * inv * w[(base + i) % wn] * gt;
    out[(size_t)t * n + base + i] = from_f32<O>(val * out_scale);
  }
}

GB_EXPORT int gb_gated_group_norm(const float* y, const float* gate, long long ldgate, const float* w, int wn, void* out,
                                  int out_dtype, int ntok, int n, int gs, float eps, int gate_first, float out_scale,
                                  cudaStream_t stream) {
  if (ntok <= 0) return 0;
  if (gs <= 0 || n % gs || wn <= 0) return GB_ERR_SIZE;
  dim3 grid(ntok, n / gs);
  const int threads = gs <= 32 ? 32 : (gs <= 64 ? 64 : 128);
  if (out_dtype == GB_F32)
    gb_launch(gated_group_norm_kernel<float>, grid, threads, 0, stream, y, gate, ldgate, w, wn, (float*)out, n, gs, eps,
              gate_first, out_scale);
  else if (out_dtype == GB_BF16)
    gb_launch(gated_group_norm_kernel<bf16>, grid, threads, 0, stream, y, gate, ldgate, w, wn, (bf16*)out, n, gs, eps, gate_first,
              out_scale);
  else
    return GB_ERR_DTYPE;
  return gb_launch_status();
}
