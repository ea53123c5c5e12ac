// Attention whose keys and values are made from one low-rank latent per token.
//
// Per token the cache keeps one row of `rank + rot` elements: the latent c (RMS-normed) and a rotated key part
// r that all heads share.  Head j's key is [W_uk_j c ; r] and its value W_uv_j c, so with the query folded
// through W_uk_j (a_j = W_uk_j^T q_j, done by a batched product before this kernel)
//     score_j(t, s) = (a_j(t) . c(s) + qr_j(t) . r(s)) * scale,      out_j(t) = W_uv_j sum_s p_j(t, s) c(s)
// which is attention with ONE key head of width rank + rot whose value is the first `rank` elements of
// the key.  This file has the two kernels in between the products:
//
//   latent_append     per token: c = rmsnorm(dkv[:rank]) * w, r = rotate(dkv[rank:]), both stored in the token's
//                     page; qr_j = rotate(q_j[dim:]) written behind a_j in the folded query rows.  Rotary pairs
//                     are (2i, 2i+1), or (i, i + n_freq), angle = position * inv_freq[i] in fp32, on the first
//                     2 * n_freq elements.
//   latent_attention  causal softmax attention of the folded queries [tokens, heads, rank + rot] (fp32) over
//                     the paged latent rows; out [tokens, heads, rank] (fp32).  Two kernels:
//                     - CUDA cores, fp32 throughout (the 32-bit path, and every shape): one warp owns one
//                       (token, head) row and walks the keys in blocks of 32 aligned to absolute positions, so a
//                       row's arithmetic does not depend on how the batch was cut;
//                     - tensor cores (mma.sync m16n8k16) for bf16 latent rows with rank a multiple of 64: tiles of
//                       64 keys aligned to absolute positions through two cp.async stages; the four warps of a
//                       block split a tile's keys for the scores and the value columns for the output; scores,
//                       maxima, sums and the accumulator are fp32, and the softmax weights enter the second
//                       product as TWO bf16 terms (p = hi + lo, 16 bits of mantissa), so they are not cut to 8.
#include "mma.cuh"

namespace tib {

struct LatentAppendArgs {
  const int* positions;    // [tokens]
  const int* token_slot;   // [tokens]
  const int* block_table;
  int table_stride;
  const float* norm_weight;   // [rank]
  const float* inv_freq;      // [n_freq]
  int n_freq;
  int rank, rot, heads, dim;  // dim: unrotated query elements per head
  int64_t ld_dkv, ld_q;
  int page_size, num_pages;
  int64_t page_stride;
  float eps;
  int* error_word;
  int half_pairs;             // 0: rotary pairs are (2i, 2i + 1); 1: (i, i + n_freq)
};

template <typename T>
__global__ void latent_append_kernel(const T* __restrict__ dkv, const T* __restrict__ q, T* __restrict__ pool,
                                     float* __restrict__ folded, LatentAppendArgs a) {
  pdl_wait();
  pdl_trigger();
  __shared__ float scratch[33];
  const size_t t = blockIdx.x;
  const int pos = a.positions[t];
  const int width = a.rank + a.rot;
  const T* src = dkv + t * a.ld_dkv;
  T* dst = nullptr;
  if (pool) {
    const int page = a.block_table[(size_t)a.token_slot[t] * a.table_stride + pos / a.page_size];
    if (page >= 0 && page < a.num_pages) {
      dst = pool + (size_t)page * a.page_stride + (size_t)(pos % a.page_size) * width;
    } else if (a.error_word && threadIdx.x == 0) {
      atomicExch(a.error_word, 0x20000 + (int)(t & 0xffff));
    }
  }
  float ss = 0.f;
  for (int c = threadIdx.x; c < a.rank; c += blockDim.x) {
    const float v = to_f32(src[c]);
    ss += v * v;
  }
  const float inv = 1.f / sqrtf(block_sum(ss, scratch) / (float)a.rank + a.eps);
  if (dst)
    for (int c = threadIdx.x; c < a.rank; c += blockDim.x) dst[c] = from_f32<T>(to_f32(src[c]) * inv * a.norm_weight[c]);
  // the shared key part (job 0) and every head's rotated query part (jobs 1 .. heads)
  if (a.half_pairs) {
    // pairs (i, i + n_freq) over the first 2 * n_freq elements; the rest pass unchanged
    for (int e = threadIdx.x; e < (a.heads + 1) * a.rot; e += blockDim.x) {
      const int job = e / a.rot, i = e - job * a.rot;
      if (i >= a.n_freq && i < 2 * a.n_freq) continue;       // (written with its partner)
      const T* from = job == 0 ? src + a.rank : q + t * a.ld_q + (size_t)(job - 1) * (a.dim + a.rot) + a.dim;
      float* f = job == 0 ? nullptr : folded + (t * a.heads + (job - 1)) * (size_t)width + a.rank;
      if (i < a.n_freq) {
        const float lo = to_f32(from[i]), hi = to_f32(from[i + a.n_freq]);
        const float angle = (float)pos * a.inv_freq[i];
        const float c = cosf(angle), sn = sinf(angle);
        const float l2 = rope_lo(lo, hi, c, sn), h2 = rope_hi(lo, hi, c, sn);
        if (f) { f[i] = l2; f[i + a.n_freq] = h2; }
        else if (dst) { dst[a.rank + i] = from_f32<T>(l2); dst[a.rank + i + a.n_freq] = from_f32<T>(h2); }
      } else {
        if (f) f[i] = to_f32(from[i]);
        else if (dst) dst[a.rank + i] = from[i];
      }
    }
    return;
  }
  // pairs (2i, 2i + 1)
  const int half = a.rot / 2;      // an odd last element, if any, passes unchanged below
  for (int e = threadIdx.x; e < (a.heads + 1) * half; e += blockDim.x) {
    const int job = e / half, i = e - job * half;
    const T* from = job == 0 ? src + a.rank : q + t * a.ld_q + (size_t)(job - 1) * (a.dim + a.rot) + a.dim;
    float lo = to_f32(from[2 * i]), hi = to_f32(from[2 * i + 1]);
    if (i < a.n_freq) {
      const float angle = (float)pos * a.inv_freq[i];
      const float c = cosf(angle), s = sinf(angle);
      const float l2 = rope_lo(lo, hi, c, s), h2 = rope_hi(lo, hi, c, s);
      lo = l2; hi = h2;
    }
    if (job == 0) {
      if (dst) { dst[a.rank + 2 * i] = from_f32<T>(lo); dst[a.rank + 2 * i + 1] = from_f32<T>(hi); }
    } else {
      float* f = folded + (t * a.heads + (job - 1)) * (size_t)width + a.rank;
      f[2 * i] = lo; f[2 * i + 1] = hi;
    }
  }
  if ((a.rot & 1) && threadIdx.x == 0) {
    if (dst) dst[width - 1] = src[width - 1];
    for (int h = 0; h < a.heads; ++h)
      folded[(t * a.heads + h) * (size_t)width + width - 1] = to_f32(q[t * a.ld_q + (size_t)h * (a.dim + a.rot) + a.dim + a.rot - 1]);
  }
}

// ---------------------------------------------------------------- attention
constexpr int kLatWarps = 4;
constexpr int kLatRowsPerWarp = 4;
constexpr int kLatRows = kLatWarps * kLatRowsPerWarp;
constexpr int kLatKeys = 32;

struct LatentAttnArgs {
  const int* q_start;
  const int* kv_start;
  const int* slots;
  const int* block_table;
  int table_stride;
  int heads, rank, width;     // width = rank + rot
  int page_size, num_pages;
  int64_t page_stride;
  float scale;
  int head_chunk, q_tile;
  int* error_word;
  // a step of single tokens may cut every context into `n_splits` runs of `blocks_per_split` key blocks, one block
  // each: they leave their running maximum, sum and unnormalised output in `partial` [tokens, heads, n_splits,
  // 2 + rank] and latent_merge_kernel puts them together
  float* partial;
  int n_splits, blocks_per_split;
};

template <typename T, int DPL>
__global__ void __launch_bounds__(kLatWarps * 32)
latent_attention_kernel(const float* __restrict__ folded, const T* __restrict__ pool, float* __restrict__ out,
                        LatentAttnArgs a) {
  extern __shared__ float smem[];
  const int w = a.width, wp = w + 1;
  float* q_s = smem;                       // [kLatRows][w]
  float* k_s = q_s + kLatRows * w;         // [32][w + 1]
  pdl_wait();
  pdl_trigger();
  const int entry = blockIdx.y;
  const int h0 = blockIdx.z * a.head_chunk;
  const int hc = min(a.head_chunk, a.heads - h0);
  const int row0 = a.q_start[entry];
  const int q_len = a.q_start[entry + 1] - row0;
  const int split = a.partial ? blockIdx.x : 0;
  const int t0 = a.partial ? 0 : blockIdx.x * a.q_tile;
  if (t0 >= q_len) return;
  const int nt = min(a.q_tile, q_len - t0);
  const int nrows = nt * hc;
  const int pos0 = a.kv_start[entry] + t0;
  const int last_pos = pos0 + nt - 1;
  const int* table = a.block_table + (size_t)a.slots[entry] * a.table_stride;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

  for (int e = threadIdx.x; e < nrows * w; e += blockDim.x) {
    const int r = e / w, dd = e - r * w;
    const int t = r / hc, g = r - t * hc;
    q_s[r * w + dd] = folded[((size_t)(row0 + t0 + t) * a.heads + h0 + g) * w + dd];
  }
  float m[kLatRowsPerWarp], l[kLatRowsPerWarp], acc[kLatRowsPerWarp][DPL];
#pragma unroll
  for (int i = 0; i < kLatRowsPerWarp; ++i) {
    m[i] = -CUDART_INF_F;
    l[i] = 0.f;
#pragma unroll
    for (int j = 0; j < DPL; ++j) acc[i][j] = 0.f;
  }
  int b_lo = 0, b_hi = last_pos / kLatKeys;
  if (a.partial) {
    b_lo = split * a.blocks_per_split;
    b_hi = min(b_hi, b_lo + a.blocks_per_split - 1);
  }
  for (int b = b_lo; b <= b_hi; ++b) {
    __syncthreads();
    // Latent rows of block b; rows past last_pos are not written yet (or are nobody's): zeros, always masked.
    for (int e = threadIdx.x; e < kLatKeys * w; e += blockDim.x) {
      const int j = e / w, dd = e - j * w;
      const int kp = b * kLatKeys + j;
      float kval = 0.f;
      if (kp <= last_pos) {
        const int page = table[kp / a.page_size];
        if (page >= 0 && page < a.num_pages) {
          kval = to_f32(pool[(size_t)page * a.page_stride + (size_t)(kp % a.page_size) * w + dd]);
        } else if (a.error_word) {
          atomicExch(a.error_word, 0x30000 + entry);
        }
      }
      k_s[j * wp + dd] = kval;
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < kLatRowsPerWarp; ++i) {
      const int r = warp * kLatRowsPerWarp + i;
      if (r >= nrows) continue;                       // uniform in the warp
      const int qpos = pos0 + r / hc;
      if (b * kLatKeys > qpos) continue;
      const int kp = b * kLatKeys + lane;
      const bool allowed = kp <= qpos;
      float s = 0.f;
      const float* qr = q_s + r * w;
      const float* kr = k_s + lane * wp;
      for (int dd = 0; dd < w; ++dd) s = fmaf(qr[dd], kr[dd], s);
      s = allowed ? s * a.scale : -CUDART_INF_F;
      const float m_new = fmaxf(m[i], warp_max(s));
      const float alpha = m[i] == -CUDART_INF_F ? 0.f : expf(m[i] - m_new);
      const float p = allowed ? expf(s - m_new) : 0.f;
      l[i] = l[i] * alpha + warp_sum(p);
      m[i] = m_new;
#pragma unroll
      for (int j = 0; j < DPL; ++j) acc[i][j] *= alpha;
      for (int kk = 0; kk < kLatKeys; ++kk) {
        const float pk = __shfl_sync(0xffffffffu, p, kk);
#pragma unroll
        for (int j = 0; j < DPL; ++j) {
          const int dd = lane + 32 * j;
          if (dd < a.rank) acc[i][j] = fmaf(pk, k_s[kk * wp + dd], acc[i][j]);
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < kLatRowsPerWarp; ++i) {
    const int r = warp * kLatRowsPerWarp + i;
    if (r >= nrows) continue;
    const int t = r / hc, g = r - t * hc;
    if (a.partial) {      // (one token per entry: t = 0)
      float* p = a.partial + (((size_t)row0 * a.heads + h0 + g) * a.n_splits + split) * (2 + a.rank);
      if (lane == 0) { p[0] = m[i]; p[1] = l[i]; }
#pragma unroll
      for (int j = 0; j < DPL; ++j) {
        const int dd = lane + 32 * j;
        if (dd < a.rank) p[2 + dd] = acc[i][j];
      }
      continue;
    }
    float* dst = out + ((size_t)(row0 + t0 + t) * a.heads + h0 + g) * a.rank;
    const float inv = 1.f / l[i];
#pragma unroll
    for (int j = 0; j < DPL; ++j) {
      const int dd = lane + 32 * j;
      if (dd < a.rank) dst[dd] = acc[i][j] * inv;
    }
  }
}

// grid (heads, tokens): out = sum_s w_s acc_s / sum_s w_s l_s with w_s = exp(m_s - max m); a run without keys has m = -inf
__global__ void latent_merge_kernel(const float* __restrict__ partial, float* __restrict__ out, int heads, int n_splits, int rank) {
  pdl_wait();
  pdl_trigger();
  __shared__ float weight[64], sums[64];      // (at most 64 runs)
  __shared__ float inv_total;
  const size_t row = (size_t)blockIdx.y * heads + blockIdx.x;
  const float* p = partial + row * n_splits * (2 + rank);
  if ((int)threadIdx.x < n_splits) {
    weight[threadIdx.x] = p[(size_t)threadIdx.x * (2 + rank)];          // (the maximum for now)
    sums[threadIdx.x] = p[(size_t)threadIdx.x * (2 + rank) + 1];
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float mx = -CUDART_INF_F;
    for (int s = 0; s < n_splits; ++s) mx = fmaxf(mx, weight[s]);
    float total = 0.f;
    for (int s = 0; s < n_splits; ++s) {
      weight[s] = weight[s] == -CUDART_INF_F ? 0.f : expf(weight[s] - mx);
      total = fmaf(weight[s], sums[s], total);
    }
    inv_total = 1.f / total;
  }
  __syncthreads();
  for (int c = threadIdx.x; c < rank; c += blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < n_splits; ++s)
      if (weight[s] != 0.f) acc = fmaf(weight[s], p[(size_t)s * (2 + rank) + 2 + c], acc);
    out[row * rank + c] = acc * inv_total;
  }
}

// ------------------------------------------------------- tensor-core kernel
constexpr int kMmaKeys = 64;        // keys per tile
constexpr int kMmaWarps = 4;

static inline size_t latent_mma_smem(int width, int mt) {
  const size_t wp = width + 8;
  return 2 * ((size_t)mt * 16 * wp + 2 * (size_t)kMmaKeys * wp + 2 * (size_t)mt * 16 * (kMmaKeys + 8))   // bf16: Q, K x 2, P hi / lo
         + 4 * ((size_t)2 * kMmaWarps * mt * 16);                                                          // fp32: maxima and sums per warp
}

// MT: m-tiles of 16 rows a block owns (rows are (token, head) pairs of one entry, heads fastest);
// R64 = rank / 64: every warp owns 16 * R64 value columns.
template <int MT, int R64>
__global__ void __launch_bounds__(kMmaWarps * 32)
latent_attention_mma_kernel(const float* __restrict__ folded, const __nv_bfloat16* __restrict__ pool, float* __restrict__ out,
                            LatentAttnArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  constexpr int RB = MT * 16;
  const int w = a.width, wp = w + 8, pp = kMmaKeys + 8;
  __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(smem_raw);       // [RB][wp]
  __nv_bfloat16* k_s = q_s + RB * wp;                                     // [2][64][wp]
  __nv_bfloat16* p_hi = k_s + 2 * kMmaKeys * wp;                          // [RB][pp]
  __nv_bfloat16* p_lo = p_hi + RB * pp;                                   // [RB][pp]
  float* red_max = reinterpret_cast<float*>(p_lo + RB * pp);              // [4][RB]
  float* red_sum = red_max + kMmaWarps * RB;                              // [4][RB]
  pdl_wait();
  pdl_trigger();
  const int entry = blockIdx.y;
  const int row0 = a.q_start[entry];
  const int q_len = a.q_start[entry + 1] - row0;
  const int total_rows = q_len * a.heads;
  const int split = a.partial ? blockIdx.x : 0;
  const int r0 = a.partial ? blockIdx.z * RB : blockIdx.x * RB;           // first (token, head) row of the block
  if (r0 >= total_rows) return;
  const int nrows = min(RB, total_rows - r0);
  const int kv0 = a.kv_start[entry];
  const int last_pos = kv0 + (r0 + nrows - 1) / a.heads;                  // highest key any row of the block reads
  const int* table = a.block_table + (size_t)a.slots[entry] * a.table_stride;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t4 = lane & 3;

  int tile_lo = 0, tile_hi = last_pos / kMmaKeys;
  if (a.partial) {      // (blocks_per_split counts runs of 32 keys; a tile is two of them)
    const int tiles_per_split = (a.blocks_per_split + 1) / 2;
    tile_lo = split * tiles_per_split;
    tile_hi = min(tile_hi, tile_lo + tiles_per_split - 1);
  }
  const int pieces_per_key = w / 8;
  auto fetch = [&](int stage, int tile) {      // a warp takes every fourth key, its lanes the 16-byte pieces of the row
    __nv_bfloat16* dst = k_s + (size_t)stage * kMmaKeys * wp;
    // the tile's 64 page ids first, two a lane and all in flight together: looked up key by key, every one of a
    // warp's sixteen keys waited a memory latency of its own
    int page_of[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int kp = tile * kMmaKeys + i * 32 + lane;
      page_of[i] = kp <= last_pos ? table[kp / a.page_size] : -1;
    }
    for (int j = warp; j < kMmaKeys; j += kMmaWarps) {
      const int kp = tile * kMmaKeys + j;
      const int page = __shfl_sync(0xffffffffu, j < 32 ? page_of[0] : page_of[1], j & 31);
      const bool valid = page >= 0 && page < a.num_pages;
      if (kp <= last_pos && !valid && a.error_word && lane == 0) atomicExch(a.error_word, 0x30000 + entry);
      const __nv_bfloat16* src = valid ? pool + (size_t)page * a.page_stride + (size_t)(kp % a.page_size) * w : pool;
      for (int c = lane; c < pieces_per_key; c += 32)
        cp_async16(dst + j * wp + c * 8, valid ? src + c * 8 : pool, valid);      // (not valid: zeros; such keys are always masked)
    }
    cp_async_commit();
  };

  float m_run[MT][2], l_run[MT][2], o[MT][2 * R64][4];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
    m_run[mt][0] = m_run[mt][1] = -CUDART_INF_F;
    l_run[mt][0] = l_run[mt][1] = 0.f;
#pragma unroll
    for (int n = 0; n < 2 * R64; ++n)
#pragma unroll
      for (int c = 0; c < 4; ++c) o[mt][n][c] = 0.f;
  }
  int qpos[MT][2];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int r = mt * 16 + g + h * 8;
      qpos[mt][h] = r < nrows ? kv0 + (r0 + r) / a.heads : -1;      // -1: no key is allowed
    }

  if (tile_lo <= tile_hi) fetch(0, tile_lo);      // (the first tile is on its way while the queries are read)
  for (int r = warp; r < RB; r += kMmaWarps) {
    const float* src = folded + ((size_t)row0 * a.heads + r0 + r) * w;
    for (int dd = lane; dd < w; dd += 32) q_s[r * wp + dd] = __float2bfloat16_rn(r < nrows ? src[dd] : 0.f);
  }
  for (int tile = tile_lo; tile <= tile_hi; ++tile) {
    const int stage = (tile - tile_lo) & 1;
    if (tile + 1 <= tile_hi) {
      fetch(stage ^ 1, tile + 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();                                   // the tile (and, the first time, q_s) is in shared memory
    const __nv_bfloat16* kt = k_s + (size_t)stage * kMmaKeys * wp;
    // scores of this warp's 16 keys
    float s[MT][2][4], s2[MT][2][4];      // (two sets of accumulators, for even and odd steps of k: shorter chains of dependent products)
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int n = 0; n < 2; ++n)
#pragma unroll
        for (int c = 0; c < 4; ++c) s[mt][n][c] = s2[mt][n][c] = 0.f;
    for (int kk = 0; kk < w; kk += 32) {
      uint32_t b[4], b2[4];
      const bool second = kk + 16 < w;
      ldmatrix_x4(b, kt + (warp * 16 + ((lane >> 4) << 3) + (lane & 7)) * wp + kk + ((lane >> 3) & 1) * 8);
      if (second) ldmatrix_x4(b2, kt + (warp * 16 + ((lane >> 4) << 3) + (lane & 7)) * wp + kk + 16 + ((lane >> 3) & 1) * 8);
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        uint32_t qa[4], qa2[4];
        ldmatrix_x4(qa, q_s + (mt * 16 + (lane & 15)) * wp + kk + (lane >> 4) * 8);
        if (second) ldmatrix_x4(qa2, q_s + (mt * 16 + (lane & 15)) * wp + kk + 16 + (lane >> 4) * 8);
        mma_bf16(s[mt][0], qa, b[0], b[1]);
        mma_bf16(s[mt][1], qa, b[2], b[3]);
        if (second) {
          mma_bf16(s2[mt][0], qa2, b2[0], b2[1]);
          mma_bf16(s2[mt][1], qa2, b2[2], b2[3]);
        }
      }
    }
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int n = 0; n < 2; ++n)
#pragma unroll
        for (int c = 0; c < 4; ++c) s[mt][n][c] += s2[mt][n][c];
    const int key0 = tile * kMmaKeys + warp * 16;
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        float mx = -CUDART_INF_F;
#pragma unroll
        for (int n = 0; n < 2; ++n)
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            const int key = key0 + n * 8 + 2 * t4 + c;
            float& v = s[mt][n][2 * h + c];
            v = key <= qpos[mt][h] ? v * a.scale : -CUDART_INF_F;
            mx = fmaxf(mx, v);
          }
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        if (t4 == 0) red_max[warp * RB + mt * 16 + g + h * 8] = mx;
      }
    __syncthreads();
    float alpha[MT][2];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int r = mt * 16 + g + h * 8;
        float mx = fmaxf(fmaxf(red_max[r], red_max[RB + r]), fmaxf(red_max[2 * RB + r], red_max[3 * RB + r]));
        const float m_new = fmaxf(m_run[mt][h], mx);
        const float base = m_new == -CUDART_INF_F ? 0.f : m_new;
        alpha[mt][h] = m_run[mt][h] == -CUDART_INF_F ? 0.f : expf(m_run[mt][h] - base);
        m_run[mt][h] = m_new;
        float sum = 0.f;
#pragma unroll
        for (int n = 0; n < 2; ++n) {
          const float p0 = expf(s[mt][n][2 * h] - base), p1 = expf(s[mt][n][2 * h + 1] - base);
          sum += p0 + p1;
          const __nv_bfloat16 h0 = __float2bfloat16_rn(p0), h1 = __float2bfloat16_rn(p1);
          const int col = warp * 16 + n * 8 + 2 * t4;
          *reinterpret_cast<__nv_bfloat162*>(p_hi + r * pp + col) = __halves2bfloat162(h0, h1);
          *reinterpret_cast<__nv_bfloat162*>(p_lo + r * pp + col) =
              __floats2bfloat162_rn(p0 - __bfloat162float(h0), p1 - __bfloat162float(h1));
        }
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        if (t4 == 0) red_sum[warp * RB + r] = sum;
      }
    __syncthreads();
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int r = mt * 16 + g + h * 8;
        l_run[mt][h] = l_run[mt][h] * alpha[mt][h] + (red_sum[r] + red_sum[RB + r]) + (red_sum[2 * RB + r] + red_sum[3 * RB + r]);
#pragma unroll
        for (int n = 0; n < 2 * R64; ++n) {
          o[mt][n][2 * h] *= alpha[mt][h];
          o[mt][n][2 * h + 1] *= alpha[mt][h];
        }
      }
    // output columns of this warp: [warp * 16 * R64, +16 * R64) of the tile's rows read as values
    const int col0 = warp * 16 * R64;
#pragma unroll
    for (int ks = 0; ks < kMmaKeys / 16; ++ks) {
      uint32_t ph[MT][4], pl[MT][4];
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        ldmatrix_x4(ph[mt], p_hi + (mt * 16 + (lane & 15)) * pp + ks * 16 + (lane >> 4) * 8);
        ldmatrix_x4(pl[mt], p_lo + (mt * 16 + (lane & 15)) * pp + ks * 16 + (lane >> 4) * 8);
      }
#pragma unroll
      for (int cg = 0; cg < R64; ++cg) {
        uint32_t v[4];     // (k lo, n 0-7), (k hi, n 0-7), (k lo, n 8-15), (k hi, n 8-15), transposed on the way in
        ldmatrix_x4_trans(v, kt + (ks * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * wp + col0 + cg * 16 + ((lane >> 4) << 3));
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {      // (the low terms after all the high ones: no product waits for the one before it)
          mma_bf16(o[mt][2 * cg], ph[mt], v[0], v[1]);
          mma_bf16(o[mt][2 * cg + 1], ph[mt], v[2], v[3]);
        }
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          mma_bf16(o[mt][2 * cg], pl[mt], v[0], v[1]);
          mma_bf16(o[mt][2 * cg + 1], pl[mt], v[2], v[3]);
        }
      }
    }
    __syncthreads();      // the stage, p_hi / p_lo and the reduction arrays are free again
  }

  const int col0 = warp * 16 * R64;
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int r = mt * 16 + g + h * 8;
      if (r >= nrows) continue;
      if (a.partial) {      // (one token per entry: the block's rows are heads)
        float* p = a.partial + (((size_t)row0 * a.heads + r0 + r) * a.n_splits + split) * (2 + a.rank);
        if (warp == 0 && t4 == 0) { p[0] = m_run[mt][h]; p[1] = l_run[mt][h]; }
#pragma unroll
        for (int n = 0; n < 2 * R64; ++n) {
          p[2 + col0 + n * 8 + 2 * t4] = o[mt][n][2 * h];
          p[2 + col0 + n * 8 + 2 * t4 + 1] = o[mt][n][2 * h + 1];
        }
      } else {
        float* dst = out + ((size_t)row0 * a.heads + r0 + r) * a.rank;
        const float inv = 1.f / l_run[mt][h];
#pragma unroll
        for (int n = 0; n < 2 * R64; ++n) {
          dst[col0 + n * 8 + 2 * t4] = o[mt][n][2 * h] * inv;
          dst[col0 + n * 8 + 2 * t4 + 1] = o[mt][n][2 * h + 1] * inv;
        }
      }
    }
}

template <int MT, int R64>
static int launch_latent_mma(const float* folded, const void* pool, float* out, const LatentAttnArgs& a, int n_entries,
                             int max_q_len, cudaStream_t stream) {
  const size_t smem = latent_mma_smem(a.width, MT);
  if (smem > 227 * 1024) return TIB_E_SMEM;
  auto kern = latent_attention_mma_kernel<MT, R64>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  const int rb = MT * 16;
  dim3 grid(a.partial ? a.n_splits : ceil_div(max_q_len * a.heads, rb), n_entries, a.partial ? ceil_div(a.heads, rb) : 1);
  TIB_LAUNCH_DEPENDENT(kern, grid, kMmaWarps * 32, smem, stream, folded, (const __nv_bfloat16*)pool, out, a);
  if (a.partial)
    TIB_LAUNCH_DEPENDENT(latent_merge_kernel, dim3(a.heads, n_entries), 128, 0, stream, (const float*)a.partial, out, a.heads,
                         a.n_splits, a.rank);
  return TIB_OK;
}

template <typename T, int DPL>
static int launch_latent_attention(const float* folded, const void* pool, float* out, const LatentAttnArgs& a, int n_entries,
                                   int max_q_len, cudaStream_t stream) {
  const size_t smem = sizeof(float) * ((size_t)kLatRows * a.width + (size_t)kLatKeys * (a.width + 1));
  if (smem > 227 * 1024) return TIB_E_SMEM;
  auto kern = latent_attention_kernel<T, DPL>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  dim3 grid(a.partial ? a.n_splits : ceil_div(max_q_len, a.q_tile), n_entries, ceil_div(a.heads, a.head_chunk));
  TIB_LAUNCH_DEPENDENT(kern, grid, kLatWarps * 32, smem, stream, folded, (const T*)pool, out, a);
  if (a.partial)
    TIB_LAUNCH_DEPENDENT(latent_merge_kernel, dim3(a.heads, n_entries), 128, 0, stream, (const float*)a.partial, out, a.heads,
                         a.n_splits, a.rank);
  return TIB_OK;
}

}  // namespace tib

using namespace tib;

// dkv: [tokens, rank + rot] (row stride ld_dkv); q: [tokens, heads * (dim + rot)] (row stride ld_q); pool: this layer's
// pages, each [page_size][rank + rot] (null: nothing is stored); folded: [tokens, heads, rank + rot] fp32, of which
// this call writes the last `rot` elements of every head.  half_pairs: the rotary pairs are (i, i + n_freq) instead of
// (2i, 2i + 1).
TIB_API int tib_latent_append(const void* dkv, int64_t ld_dkv, const void* q, int64_t ld_q, void* pool, float* folded,
                              const int* positions, const int* token_slot, const int* block_table, int table_stride,
                              const float* norm_weight, float eps, const float* inv_freq, int n_freq, int n_tokens, int heads,
                              int dim, int rank, int rot, int page_size, int64_t page_stride, int num_pages,
                              int half_pairs, int* error_word, int dtype, cudaStream_t stream) {
  if (n_tokens == 0) return TIB_OK;
  if (!dkv || !q || !folded || !positions || !norm_weight || (n_freq > 0 && !inv_freq)) return TIB_E_ARG;
  if (pool && (!token_slot || !block_table || page_size < 1)) return TIB_E_ARG;
  if (heads < 1 || dim < 0 || rank < 1 || rot < 0 || 2 * n_freq > rot) return TIB_E_SIZE;
  LatentAppendArgs a;
  a.positions = positions; a.token_slot = token_slot; a.block_table = block_table; a.table_stride = table_stride;
  a.norm_weight = norm_weight; a.inv_freq = inv_freq; a.n_freq = n_freq; a.rank = rank; a.rot = rot; a.heads = heads;
  a.dim = dim; a.ld_dkv = ld_dkv; a.ld_q = ld_q; a.page_size = page_size; a.num_pages = num_pages;
  a.page_stride = page_stride; a.eps = eps; a.error_word = error_word; a.half_pairs = half_pairs;
  if (dtype == TIB_F32)
    TIB_LAUNCH_DEPENDENT(latent_append_kernel<float>, n_tokens, 128, 0, stream, (const float*)dkv, (const float*)q,
                         (float*)pool, folded, a);
  else if (dtype == TIB_BF16)
    TIB_LAUNCH_DEPENDENT(latent_append_kernel<__nv_bfloat16>, n_tokens, 128, 0, stream, (const __nv_bfloat16*)dkv,
                         (const __nv_bfloat16*)q, (__nv_bfloat16*)pool, folded, a);
  else
    return TIB_E_DTYPE;
  return TIB_OK;
}

// How many runs a step of `n_entries` single tokens should cut its contexts of up to `max_kv_len` keys into (1: none).
TIB_API int tib_latent_attention_splits(int n_entries, int heads, int max_kv_len) {
  const int head_chunk = heads < kLatRows ? heads : kLatRows;
  const int blocks = n_entries * ceil_div(heads, head_chunk);
  const int key_blocks = ceil_div(max_kv_len, kLatKeys);
  int splits = 148 / (blocks < 1 ? 1 : blocks);      // (one block per SM: the tensor-core kernel's stages fill its shared memory)
  if (splits > key_blocks) splits = key_blocks;
  if (splits > 64) splits = 64;
  return splits < 1 ? 1 : splits;
}

// folded: [tokens, heads, rank + rot] fp32; pool: pages of [page_size][rank + rot] in `dtype`; out: [tokens, heads, rank] fp32.
// n_splits > 1 (a step of single tokens only, contexts of at most max_kv_len keys): partial [tokens, heads, n_splits, 2 + rank].
// force_simt: the CUDA-core kernel also where the tensor-core one takes the shape.
TIB_API int tib_latent_attention(const float* folded, const void* pool, float* out, const int* q_start, const int* kv_start,
                                 const int* slots, const int* block_table, int table_stride, int n_entries, int max_q_len,
                                 int heads, int rank, int rot, int page_size, int64_t page_stride, int num_pages, float scale,
                                 float* partial, int n_splits, int max_kv_len, int force_simt, int* error_word, int dtype,
                                 cudaStream_t stream) {
  if (n_entries == 0 || max_q_len == 0) return TIB_OK;
  if (!folded || !pool || !out || !q_start || !kv_start || !slots || !block_table) return TIB_E_ARG;
  if (heads < 1 || rank < 1 || rot < 0 || page_size < 1 || rank > 512 || n_entries > 65535) return TIB_E_SIZE;
  LatentAttnArgs a;
  a.q_start = q_start; a.kv_start = kv_start; a.slots = slots; a.block_table = block_table; a.table_stride = table_stride;
  a.heads = heads; a.rank = rank; a.width = rank + rot; a.page_size = page_size; a.num_pages = num_pages;
  a.page_stride = page_stride; a.scale = scale; a.error_word = error_word;
  a.partial = nullptr; a.n_splits = 1; a.blocks_per_split = 0;
  if (n_splits > 1) {
    if (!partial || max_q_len != 1 || max_kv_len < 1) return TIB_E_ARG;
    a.partial = partial; a.n_splits = n_splits;
    a.blocks_per_split = ceil_div(ceil_div(max_kv_len, kLatKeys), n_splits);
  }
  a.head_chunk = heads < kLatRows ? heads : kLatRows;
  a.q_tile = kLatRows / a.head_chunk;
  if (ceil_div(heads, a.head_chunk) > 65535) return TIB_E_SIZE;
  const int width = rank + rot;
  if (dtype == TIB_BF16 && !force_simt && width % 16 == 0 && rank % 64 == 0 && (page_stride % 8) == 0 && ((uintptr_t)pool & 15) == 0) {
    const int r64 = rank / 64;
    const bool single = max_q_len == 1;
    if (latent_mma_smem(width, single ? 1 : 2) <= 227 * 1024 && (r64 <= 4 || r64 == 6 || r64 == 8)) {
#define TIB_LAT_MMA(MT)                                                                                         \
  (r64 == 1 ? launch_latent_mma<MT, 1>(folded, pool, out, a, n_entries, max_q_len, stream)                     \
   : r64 == 2 ? launch_latent_mma<MT, 2>(folded, pool, out, a, n_entries, max_q_len, stream)                   \
   : r64 == 3 ? launch_latent_mma<MT, 3>(folded, pool, out, a, n_entries, max_q_len, stream)                   \
   : r64 == 4 ? launch_latent_mma<MT, 4>(folded, pool, out, a, n_entries, max_q_len, stream)                   \
   : r64 == 6 ? launch_latent_mma<MT, 6>(folded, pool, out, a, n_entries, max_q_len, stream)                   \
              : launch_latent_mma<MT, 8>(folded, pool, out, a, n_entries, max_q_len, stream))
      return single ? TIB_LAT_MMA(1) : TIB_LAT_MMA(2);
#undef TIB_LAT_MMA
    }
  }
  const int dpl = (rank + 31) / 32;
#define TIB_LAT_DISPATCH(T)                                                                             \
  (dpl <= 1 ? launch_latent_attention<T, 1>(folded, pool, out, a, n_entries, max_q_len, stream)        \
   : dpl <= 2 ? launch_latent_attention<T, 2>(folded, pool, out, a, n_entries, max_q_len, stream)      \
   : dpl <= 4 ? launch_latent_attention<T, 4>(folded, pool, out, a, n_entries, max_q_len, stream)      \
   : dpl <= 8 ? launch_latent_attention<T, 8>(folded, pool, out, a, n_entries, max_q_len, stream)      \
              : launch_latent_attention<T, 16>(folded, pool, out, a, n_entries, max_q_len, stream))
  if (dtype == TIB_F32) return TIB_LAT_DISPATCH(float);
  if (dtype == TIB_BF16) return TIB_LAT_DISPATCH(__nv_bfloat16);
#undef TIB_LAT_DISPATCH
  return TIB_E_DTYPE;
}
