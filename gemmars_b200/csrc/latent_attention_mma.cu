// bfloat16 latent attention on the tensor cores, for prompts and for single positions alike.
// Compiled for one latent size and one width of the rotated part (-DGB_LATENT_RANK, -DGB_LATENT_ROT).
//
// All heads read the same cached rows [c (RANK) | k_rot (ROT)], so the rows of a tile are
// (token, head) pairs: row r of a sequence's step is token r / H, head r % H, and a tile of keys
// that has been brought into shared memory once serves every head of several tokens (a prompt),
// or every head of the one token (decoding).  Per tile of KEYS keys:
//
//   S = Q K^T        mma.sync m16n8k16, Q [rows, RANK + ROT] and the key tile in shared memory
//   P = softmax      online, float32, log2 units, each row masked at its own position (and window)
//   O += P V         V = the first RANK columns of the same key tile (ldmatrix.trans)
//
// A group of 16 rows is worked by NSPLIT warps.  Each keeps its share of the queries' columns in
// registers for the whole kernel and scores every key of a tile over that share alone, so a key
// tile is read from shared memory once per group, not once per warp; the partial scores meet in
// shared memory and are added in warp order.  Each warp then owns RANK / NSPLIT of the output's
// columns, so that a wide latent does not have to fit one warp's registers.  Key tiles arrive by
// cp.async, one tile ahead; the queries pass through the same buffers before the first tile.
// With `ksplits` > 1 (decoding: few rows, many keys) the keys of a tile of rows are dealt to
// ksplits CTAs, which leave (m, l, o) parts that a second kernel adds in split
// order: the same bits every run.
//
// The same kernel serves a prompt step whose keys and values were expanded per head (rows
// [v | k_nope | k_rot] with the value's width in RANK's place): head_stride > 0 gives every head rows
// of its own, contiguous from a sequence's first packed token, one head per grid layer, and
// out_scale (the layer's gate) is multiplied into the output.
#include "mma.cuh"

#ifndef GB_LATENT_RANK
#define GB_LATENT_RANK 128
#endif
#ifndef GB_LATENT_ROT
#define GB_LATENT_ROT 16
#endif

namespace {

constexpr int RANK = GB_LATENT_RANK, ROT = GB_LATENT_ROT, KD = RANK + ROT;
static_assert(RANK % 16 == 0 && ROT % 16 == 0 && RANK >= 16, "latent and rotated widths must be multiples of 16");
constexpr int NSPLIT = RANK <= 128 ? 1 : (RANK <= 256 ? 2 : 4);
static_assert(RANK % (16 * NSPLIT) == 0, "the latent must divide into 16-column blocks per warp");
constexpr int LDS = KD + ((KD / 8) % 2 == 0 ? 8 : 0);   // row pitch in shared memory: an odd number of 16-byte units
constexpr int KSTEPS = KD / 16;                          // 16-column steps of a score
constexpr int KSW = (KSTEPS + NSPLIT - 1) / NSPLIT;      // steps a warp owns
constexpr int DW = RANK / NSPLIT;                        // output columns a warp owns
constexpr int MAX_GROUPS = NSPLIT == 4 ? 2 : 4;          // groups of 16 rows a CTA at most
constexpr int PART = RANK + 4;                           // floats of a split's part: o, then m and l (rows stay 16-byte aligned)
constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void ldsm_x4(uint32_t* r, const void* p) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t* r, const void* p) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}

// grid (row tiles upper bound, ksplits); block groups * NSPLIT * 32.  KEYS: keys a tile (64 for
// prompts; 32 for decoding, where two CTAs then share an SM and hide each other's waits).
template <int KEYS>
__global__ void __launch_bounds__(MAX_GROUPS * NSPLIT * 32)
latent_attention_mma_kernel(const bf16* __restrict__ qa, long long ldq, bf16* __restrict__ out, long long ldo,
                            float* __restrict__ part, const bf16* __restrict__ cache, const int* __restrict__ page_table,
                            int table_width, int page_size, const int* __restrict__ cu_seqlens,
                            const int* __restrict__ seq_start, const int* __restrict__ seq_slot, int n_seqs, int H,
                            int window, int ksplits, long long head_stride, const float* __restrict__ out_scale) {
  constexpr int NB = KEYS / 8;                         // blocks of 8 keys a tile
  constexpr int SXP = KEYS + 4;                        // pitch of the exchanged scores
  static_assert(NB % 2 == 0, "key blocks come in pairs");
  extern __shared__ __align__(16) unsigned char smem_raw[];
  pdl_release_next();
  pdl_wait_prior();
  const int groups = blockDim.x / (32 * NSPLIT);
  const int tile_rows = groups * 16;
  bf16* Ks = (bf16*)smem_raw;                         // [2][KEYS][LDS]
  bf16* Qs = Ks;                                      // [tile_rows][LDS], before the first key tile
  float* Sx = (float*)(Ks + 2 * KEYS * LDS);          // [groups][NSPLIT][16][SXP], only with NSPLIT > 1
  // ---- which sequence and which tile of its rows
  const int heads_all = H;
  if (head_stride > 0) H = 1;                          // see per_head below
  int b = 0, tile = blockIdx.x, rows_b = 0;
  for (; b < n_seqs; ++b) {
    rows_b = (cu_seqlens[b + 1] - cu_seqlens[b]) * H;
    const int tiles = (rows_b + tile_rows - 1) / tile_rows;
    if (tile < tiles) break;
    tile -= tiles;
  }
  if (b >= n_seqs) return;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, c = lane & 3;
  const int rg = warp / NSPLIT, w = warp % NSPLIT;
  const int slot = seq_slot[b], start = seq_start[b], tok_base = cu_seqlens[b];
  const int row_base = tile * tile_rows;
  // head_stride > 0: every head has rows of its own (keys and values expanded per head), head
  // blockIdx.z's at cache + z * head_stride, a sequence's rows contiguous from its first packed token
  // (all sequences start at position 0); the rows of a tile are then tokens of that one head
  const bool per_head = head_stride > 0;
  const int hz = per_head ? (int)blockIdx.z : 0;
  if (per_head) {
    qa += (size_t)hz * KD;
    out += (size_t)hz * RANK;
    cache += (size_t)hz * head_stride;
  }
  // ---- the keys this CTA reads
  const int first_tok = row_base / H;
  const int last_tok = (min(rows_b, row_base + tile_rows) - 1) / H;
  const int hi = start + last_tok;
  const int lo_cta = window > 0 ? max(0, start + first_tok + 1 - window) : 0;
  const int t_begin = lo_cta / KEYS, t_end = hi / KEYS + 1;
  const int per = (t_end - t_begin + ksplits - 1) / ksplits;
  const int my_begin = t_begin + (int)blockIdx.y * per, my_end = min(t_end, my_begin + per);
  // ---- this thread's two rows
  const int r0 = row_base + rg * 16 + g, r1 = r0 + 8;
  const bool v0 = r0 < rows_b, v1 = r1 < rows_b;
  const int pos0 = v0 ? start + r0 / H : -1, pos1 = v1 ? start + r1 / H : -1;
  const int lo0 = window > 0 ? max(0, pos0 + 1 - window) : 0, lo1 = window > 0 ? max(0, pos1 + 1 - window) : 0;

  constexpr int CH = KD / 8;                           // 16-byte pieces of a row
  for (int e = tid; e < tile_rows * CH; e += blockDim.x) {
    const int r = e / CH, ch = e % CH, row = row_base + r;
    bf16* dst = Qs + (size_t)r * LDS + ch * 8;
    if (row < rows_b)
      cp_async16(dst, qa + (size_t)(tok_base + row / H) * ldq + (size_t)(row % H) * KD + ch * 8);
    else
      *(uint4*)dst = make_uint4(0, 0, 0, 0);
  }
  auto load_keys = [&](int t, int stage) {
    const int key0 = t * KEYS;
    const bf16* src;
    if (per_head) {
      src = cache + (size_t)(tok_base + key0) * KD;
    } else {
      const int page = page_table[(size_t)slot * table_width + (key0 / page_size) % table_width];
      src = cache + ((size_t)page * page_size + key0 % page_size) * KD;
    }
    bf16* dst = Ks + (size_t)stage * KEYS * LDS;
    for (int e = tid; e < KEYS * CH; e += blockDim.x) {
      const int r = e / CH, ch = e % CH;
      cp_async16(dst + (size_t)r * LDS + ch * 8, src + (size_t)r * KD + ch * 8);
    }
  };
  // ---- this warp's share of the queries' columns, into registers
  cp_async_commit();
  cp_async_wait_all();
  __syncthreads();
  uint32_t qf[KSW][4];
  {
    const bf16* q_lane = Qs + (size_t)(rg * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * LDS + 8 * (lane >> 4);
#pragma unroll
    for (int i = 0; i < KSW; ++i) {
      const int ks = w * KSW + i;
      if (ks < KSTEPS) ldsm_x4(qf[i], q_lane + ks * 16);
      else qf[i][0] = qf[i][1] = qf[i][2] = qf[i][3] = 0;
    }
  }
  __syncthreads();                                     // the buffers are free for keys
  if (my_begin < my_end) load_keys(my_begin, 0);
  cp_async_commit();

  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  float o[DW / 8][4];
#pragma unroll
  for (int d = 0; d < DW / 8; ++d) o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f;

  for (int t = my_begin; t < my_end; ++t) {
    const int stage = (t - my_begin) & 1;
    cp_async_wait_all();
    __syncthreads();                                   // tile t (and Q) landed; everyone is done with tile t - 1
    if (t + 1 < my_end) load_keys(t + 1, stage ^ 1);
    cp_async_commit();
    const bf16* kt = Ks + (size_t)stage * KEYS * LDS;
    // ---- scores of all the tile's keys over this warp's share of the columns
    float s[NB][4];
#pragma unroll
    for (int j = 0; j < NB; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
    {
      const bf16* k_lane = kt + (size_t)((lane & 7) + 8 * (lane >> 4)) * LDS + 8 * ((lane >> 3) & 1);
#pragma unroll
      for (int i = 0; i < KSW; ++i) {
        const int ks = w * KSW + i;
        if (ks < KSTEPS) {
#pragma unroll
          for (int j = 0; j < NB; j += 2) {
            uint32_t kb[4];                              // keys 8j..8j+7: regs 0, 1; keys 8j+8..8j+15: regs 2, 3
            ldsm_x4(kb, k_lane + (size_t)j * 8 * LDS + ks * 16);
            mma16816(s[j], qf[i][0], qf[i][1], qf[i][2], qf[i][3], kb[0], kb[1]);
            mma16816(s[j + 1], qf[i][0], qf[i][1], qf[i][2], qf[i][3], kb[2], kb[3]);
          }
        }
      }
      if (NSPLIT > 1) {
        float* sx = Sx + (size_t)rg * NSPLIT * 16 * SXP;
        float* mine = sx + (size_t)w * 16 * SXP;
#pragma unroll
        for (int j = 0; j < NB; ++j) {
          *(float2*)(mine + g * SXP + j * 8 + 2 * c) = make_float2(s[j][0], s[j][1]);
          *(float2*)(mine + (g + 8) * SXP + j * 8 + 2 * c) = make_float2(s[j][2], s[j][3]);
        }
        __syncthreads();
#pragma unroll
        for (int j = 0; j < NB; ++j) {
          float2 x = make_float2(0.f, 0.f), y = make_float2(0.f, 0.f);
#pragma unroll
          for (int ww = 0; ww < NSPLIT; ++ww) {
            const float2 a = *(const float2*)(sx + (size_t)ww * 16 * SXP + g * SXP + j * 8 + 2 * c);
            const float2 bb = *(const float2*)(sx + (size_t)ww * 16 * SXP + (g + 8) * SXP + j * 8 + 2 * c);
            x.x += a.x; x.y += a.y; y.x += bb.x; y.y += bb.y;
          }
          s[j][0] = x.x; s[j][1] = x.y; s[j][2] = y.x; s[j][3] = y.y;
        }
      }
    }
    // ---- softmax of the tile, each row masked at its own position
    const int key0 = t * KEYS;
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int j = 0; j < NB; ++j)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int key = key0 + 8 * j + 2 * c + e;
        s[j][e] = (key >= lo0 && key <= pos0) ? s[j][e] * LOG2E : -INFINITY;
        s[j][2 + e] = (key >= lo1 && key <= pos1) ? s[j][2 + e] * LOG2E : -INFINITY;
        mx0 = fmaxf(mx0, s[j][e]);
        mx1 = fmaxf(mx1, s[j][2 + e]);
      }
    const float n0 = fmaxf(m0, quad_max(mx0)), n1 = fmaxf(m1, quad_max(mx1));
    const float u0 = n0 == -INFINITY ? 0.f : n0, u1 = n1 == -INFINITY ? 0.f : n1;
    const float alpha0 = exp2f(m0 - u0), alpha1 = exp2f(m1 - u1);
    m0 = n0;
    m1 = n1;
    uint32_t p[NB][2];
    float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
    for (int j = 0; j < NB; ++j) {
      const float a = exp2f(s[j][0] - u0), bb = exp2f(s[j][1] - u0);
      const float cc = exp2f(s[j][2] - u1), d = exp2f(s[j][3] - u1);
      sum0 += a + bb;
      sum1 += cc + d;
      p[j][0] = pack_bf16(a, bb);
      p[j][1] = pack_bf16(cc, d);
    }
    l0 = l0 * alpha0 + sum0;
    l1 = l1 * alpha1 + sum1;
#pragma unroll
    for (int d = 0; d < DW / 8; ++d) { o[d][0] *= alpha0; o[d][1] *= alpha0; o[d][2] *= alpha1; o[d][3] *= alpha1; }
    // ---- O += P V over this warp's columns of the latent
    const bf16* v_lane = kt + (size_t)((lane & 7) + 8 * ((lane >> 3) & 1)) * LDS + w * DW + 8 * (lane >> 4);
#pragma unroll
    for (int kk = 0; kk < KEYS / 16; ++kk) {
#pragma unroll
      for (int db = 0; db < DW / 16; ++db) {
        uint32_t vb[4];
        ldsm_x4_t(vb, v_lane + (size_t)kk * 16 * LDS + db * 16);
        mma16816(o[2 * db], p[2 * kk][0], p[2 * kk][1], p[2 * kk + 1][0], p[2 * kk + 1][1], vb[0], vb[1]);
        mma16816(o[2 * db + 1], p[2 * kk][0], p[2 * kk][1], p[2 * kk + 1][0], p[2 * kk + 1][1], vb[2], vb[3]);
      }
    }
  }
  cp_async_wait_all();
  l0 = quad_sum(l0);
  l1 = quad_sum(l1);
  if (ksplits == 1) {
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int row = half ? r1 : r0;
      if (!(half ? v1 : v0)) continue;
      float inv = 1.0f / (half ? l1 : l0);
      if (out_scale) inv *= out_scale[(size_t)(tok_base + row / H) * heads_all + (per_head ? hz : row % H)];
      bf16* dst = out + (size_t)(tok_base + row / H) * ldo + (size_t)(row % H) * RANK + w * DW + 2 * c;
#pragma unroll
      for (int d = 0; d < DW / 8; ++d) *(uint32_t*)(dst + d * 8) = pack_bf16(o[d][2 * half] * inv, o[d][2 * half + 1] * inv);
    }
    return;
  }
  // parts: [row of the step][split][PART]: unnormalised o, then m (log2 units) and l
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int row = half ? r1 : r0;
    if (!(half ? v1 : v0)) continue;
    float* dst = part + (((size_t)(tok_base + row / H) * H + row % H) * ksplits + blockIdx.y) * PART;
    if (w == 0 && c == 0) { dst[RANK] = half ? m1 : m0; dst[RANK + 1] = half ? l1 : l0; }
#pragma unroll
    for (int d = 0; d < DW / 8; ++d) *(float2*)(dst + w * DW + d * 8 + 2 * c) = make_float2(o[d][2 * half], o[d][2 * half + 1]);
  }
}

// one block per (token, head): adds the splits' parts in split order, four columns a thread
constexpr int MAX_KSPLITS = 64;

__global__ void __launch_bounds__(128) latent_attention_merge_kernel(const float* __restrict__ part, bf16* __restrict__ out,
                                                                     long long ldo, int H, int ksplits) {
  __shared__ float ms[MAX_KSPLITS], ls[MAX_KSPLITS];
  pdl_release_next();
  pdl_wait_prior();
  const int row = blockIdx.x, t = row / H, h = row % H;
  const float* src = part + (size_t)row * ksplits * PART;
  if (threadIdx.x < ksplits) {
    ms[threadIdx.x] = src[(size_t)threadIdx.x * PART + RANK];
    ls[threadIdx.x] = src[(size_t)threadIdx.x * PART + RANK + 1];
  }
  __syncthreads();
  float M = -INFINITY;
  for (int s = 0; s < ksplits; ++s) M = fmaxf(M, ms[s]);
  float L = 0.f;
  for (int s = 0; s < ksplits; ++s) L += ms[s] > -INFINITY ? ls[s] * exp2f(ms[s] - M) : 0.f;
  const float inv = 1.0f / L;
  for (int d = 4 * threadIdx.x; d < RANK; d += 4 * 128) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 8
    for (int s = 0; s < ksplits; ++s) {
      const float4 v = *(const float4*)(src + (size_t)s * PART + d);     // a split without keys left zeros
      const float wgt = ms[s] > -INFINITY ? exp2f(ms[s] - M) : 0.f;
      acc.x += v.x * wgt; acc.y += v.y * wgt; acc.z += v.z * wgt; acc.w += v.w * wgt;
    }
    bf16* dst = out + (size_t)t * ldo + (size_t)h * RANK + d;
    *(uint32_t*)dst = pack_bf16(acc.x * inv, acc.y * inv);
    *(uint32_t*)(dst + 2) = pack_bf16(acc.z * inv, acc.w * inv);
  }
}

template <int KEYS>
int launch_latent(const bf16* qa, long long ldq, bf16* out, long long ldo, float* part, const bf16* cache, const int* page_table,
                  int table_width, int page_size, const int* cu_seqlens, const int* seq_start, const int* seq_slot, int n_seqs,
                  int ntok, int H, int groups, int window, int ksplits, long long head_stride, const float* out_scale,
                  cudaStream_t stream) {
  const int tile_rows = groups * 16;
  if (tile_rows > 2 * KEYS) return GB_ERR_SIZE;       // the queries are staged in the key buffers
  const size_t smem = 2 * (size_t)KEYS * LDS * sizeof(bf16) +
                      (NSPLIT > 1 ? (size_t)groups * NSPLIT * 16 * (KEYS + 4) * sizeof(float) : 0);
  static size_t allowed = 0;
  if (smem > allowed) {
    if (cudaFuncSetAttribute(latent_attention_mma_kernel<KEYS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return GB_ERR_SIZE;
    allowed = smem;
  }
  const int row_heads = head_stride > 0 ? 1 : H;
  dim3 grid(((long long)ntok * row_heads + tile_rows - 1) / tile_rows + n_seqs, ksplits, head_stride > 0 ? H : 1);
  gb_launch(latent_attention_mma_kernel<KEYS>, grid, dim3(groups * NSPLIT * 32), smem, stream, qa, ldq, out, ldo, part, cache,
            page_table, table_width, page_size, cu_seqlens, seq_start, seq_slot, n_seqs, H, window, ksplits, head_stride,
            out_scale);
  return 0;
}

}  // namespace

GB_EXPORT long long gb_latent_attention_mma_scratch(int ntok, int H, int ksplits) {
  return ksplits > 1 ? (long long)ntok * H * ksplits * PART : 0;
}

// qa: [ntok, H * (RANK + ROT)] bfloat16 rows ldq apart, packed by sequence (cu_seqlens [n_seqs + 1]);
// out: [ntok, H * RANK]; cache: [pages, page_size, RANK + ROT]; seq_start: each sequence's length
// before the step (the cache already holds the step's own rows); part: float32 scratch of
// gb_latent_attention_mma_scratch() floats when ksplits > 1.  max_rows: the most rows (tokens * H)
// one sequence brings, for the size of a CTA.  head_stride > 0: the rows are per head and contiguous
// (cache: [H][all packed tokens + a tile's worth][RANK + ROT], elements head_stride apart; every
// sequence starts at position 0; no page table; ksplits 1).  out_scale: float32 [ntok, H] or null,
// multiplied into the output (ksplits 1 only).
GB_EXPORT int gb_latent_attention_mma(const void* qa, long long ldq, void* out, long long ldo, float* part,
                                      const void* cache, const int* page_table, int table_width, int page_size,
                                      const int* cu_seqlens, const int* seq_start, const int* seq_slot, int n_seqs,
                                      int ntok, int H, int rank, int rot, int max_rows, int window, int ksplits,
                                      long long head_stride, const float* out_scale, cudaStream_t stream) {
  if (ntok <= 0 || n_seqs <= 0) return 0;
  if (rank != RANK || rot != ROT || H <= 0 || page_size % 64 || ksplits < 1 || ksplits > MAX_KSPLITS) return GB_ERR_SIZE;
  if (((uintptr_t)qa & 15) || (ldq % 8) || ((uintptr_t)out & 3) || (ldo % 2) || ((uintptr_t)cache & 15)) return GB_ERR_SIZE;
  if (ksplits > 1 && (part == nullptr || ((uintptr_t)part & 15) || head_stride > 0 || out_scale)) return GB_ERR_ARG;
  if (head_stride > 0 && (H > 65535 || head_stride % 8)) return GB_ERR_SIZE;
  int groups = (max_rows + 15) / 16;
  groups = groups < 1 ? 1 : (groups > MAX_GROUPS ? MAX_GROUPS : groups);
  int rc;
  if (ksplits > 1)
    rc = launch_latent<32>((const bf16*)qa, ldq, (bf16*)out, ldo, part, (const bf16*)cache, page_table, table_width, page_size,
                           cu_seqlens, seq_start, seq_slot, n_seqs, ntok, H, groups, window, ksplits, head_stride, out_scale, stream);
  else
    rc = launch_latent<64>((const bf16*)qa, ldq, (bf16*)out, ldo, part, (const bf16*)cache, page_table, table_width, page_size,
                           cu_seqlens, seq_start, seq_slot, n_seqs, ntok, H, groups, window, ksplits, head_stride, out_scale, stream);
  if (rc) return rc;
  if (ksplits > 1)
    gb_launch(latent_attention_merge_kernel, dim3(ntok * H), dim3(128), 0, stream, (const float*)part, (bf16*)out, ldo, H,
              ksplits);
  return gb_launch_status();
}
