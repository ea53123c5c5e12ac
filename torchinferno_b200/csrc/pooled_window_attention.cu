// Attention over a sliding window plus one averaged key and value for every block of tokens that lies wholly behind
// the window, with values that are rotated by their own position.
//
//   rotary_kv_append   q, k (+ bias) get the rotary encoding on the first rot_dim elements of a head (pairs i, i + rot/2;
//                      angle = position * freq[i]; cos and sin times `amplitude`); v (+ bias) is turned over its whole
//                      width (pairs m, m + vdim/2; angle = position * vfreq[m]); q goes to q_out, k and v into the pages
//   pool_blocks        for every token that completes a block of `pool` positions (position % pool == pool - 1): the
//                      mean of the block's cached keys and of its cached values goes into entry position / pool of the
//                      second, strided cache (sums in fp32, in rising order of position)
//   attention          query i sees the tokens j with 0 <= i - j < window, and the blocks b with
//                      b * pool + pool - 1 <= i - window; score = q . k * scale * temp[h]; one softmax over both, with
//                      exp(sink[h]) added to its denominator; the head's sum of values is turned back by -i over the
//                      value pairs and multiplied element by element by sigmoid(gate).  Optionally a learned number per
//                      head and distance, rel_bias[h][min(i - j, span - 1)], is added to a token's score (a design
//                      without window or blocks passes a window beyond every position and pool 0)
//
// Scores, the softmax, the sums over values, the turning back and the gate are fp32.  Two kernels.  On the CUDA cores
// (32-bit, any head size) one warp owns one (query token, query head) row from start to end and walks
// first the blocks, then the tokens, 32 at a time, aligned to absolute block numbers / positions, in rising order: a
// row's arithmetic depends only on its own position, never on how the batch was cut, which rows share the thread
// block, or which pages hold the keys.  On the tensor cores (bf16, head sizes that are multiples of 8) the same
// walk runs in tiles of 64 with mma.sync, see below; a step of single tokens may share each context's tiles out over
// several blocks, whose sums a small second kernel adds in the order of the parts.
#include "mma.cuh"
#include <math_constants.h>

namespace tib {

struct PwaCache {
  void* keys; void* values;          // first key / value of the layer's first page
  const int* block_table; int table_stride;
  int page_size; int64_t page_stride; int num_pages;
};

__device__ __forceinline__ int pwa_page(const PwaCache& c, const int* table, int index, int* error_word, int code) {
  const int page = table[index / c.page_size];
  if (page >= 0 && page < c.num_pages) return page;
  if (error_word) atomicExch(error_word, code);
  return -1;
}

// ---------------------------------------------------------------------------------------------------- append
struct PwaAppendArgs {
  int64_t ld; int q_off, k_off, v_off;
  const float* q_bias; const float* k_bias; const float* v_bias;     // [heads * dim], [kv_heads * dim], [kv_heads * vdim] or null
  const int* positions; const int* token_slot;
  const float* freq; const float* vfreq;                             // [rot_dim / 2], [vdim / 2] (null: values are not turned)
  float amplitude;
  int heads, kv_heads, dim, vdim, rot_dim;
  PwaCache cache;
  int* error_word;
};

// One block per token; a warp per head (q heads, then k heads, then v heads).
template <typename T>
__global__ void __launch_bounds__(512) pwa_append_kernel(const T* __restrict__ proj, T* __restrict__ q_out, PwaAppendArgs a) {
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int pos = a.positions[t];
  const float fpos = (float)pos;
  const T* row = proj + (size_t)t * a.ld;
  int page = -1, in_page = 0;
  if (a.cache.keys) {
    const int* table = a.cache.block_table + (size_t)a.token_slot[t] * a.cache.table_stride;
    page = pwa_page(a.cache, table, pos, a.error_word, 0x30000 + (t & 0xffff));
    in_page = pos % a.cache.page_size;
  }
  const int total = a.heads + 2 * a.kv_heads;
  for (int head = warp; head < total; head += nwarps) {
    if (head < a.heads + a.kv_heads) {       // a query or key head: partial rotary, pairs (i, i + rot/2)
      const bool is_q = head < a.heads;
      const int hh = is_q ? head : head - a.heads;
      const T* src = row + (is_q ? a.q_off : a.k_off) + hh * a.dim;
      const float* bias = is_q ? a.q_bias : a.k_bias;
      T* dst;
      if (is_q) dst = q_out + (size_t)t * a.heads * a.dim + hh * a.dim;
      else {
        if (page < 0) continue;
        dst = reinterpret_cast<T*>(a.cache.keys) + (size_t)page * a.cache.page_stride + ((size_t)hh * a.cache.page_size + in_page) * a.dim;
      }
      const int half = a.rot_dim / 2;
      for (int i = lane; i < half; i += 32) {
        float lo = to_f32(src[i]), hi = to_f32(src[i + half]);
        if (bias) { lo += bias[hh * a.dim + i]; hi += bias[hh * a.dim + i + half]; }
        const float angle = fpos * a.freq[i];
        const float c = cosf(angle) * a.amplitude, s = sinf(angle) * a.amplitude;
        dst[i] = from_f32<T>(rope_lo(lo, hi, c, s));
        dst[i + half] = from_f32<T>(rope_hi(lo, hi, c, s));
      }
      for (int i = a.rot_dim + lane; i < a.dim; i += 32) {
        float v = to_f32(src[i]);
        if (bias) v += bias[hh * a.dim + i];
        dst[i] = from_f32<T>(v);
      }
    } else {                                  // a value head: turned over its whole width
      if (page < 0) continue;
      const int hh = head - a.heads - a.kv_heads;
      const T* src = row + a.v_off + hh * a.vdim;
      T* dst = reinterpret_cast<T*>(a.cache.values) + (size_t)page * a.cache.page_stride + ((size_t)hh * a.cache.page_size + in_page) * a.vdim;
      if (a.vfreq) {
        const int half = a.vdim / 2;
        for (int i = lane; i < half; i += 32) {
          float lo = to_f32(src[i]), hi = to_f32(src[i + half]);
          if (a.v_bias) { lo += a.v_bias[hh * a.vdim + i]; hi += a.v_bias[hh * a.vdim + i + half]; }
          const float angle = fpos * a.vfreq[i];
          const float c = cosf(angle), s = sinf(angle);
          dst[i] = from_f32<T>(rope_lo(lo, hi, c, s));
          dst[i + half] = from_f32<T>(rope_hi(lo, hi, c, s));
        }
      } else {
        for (int i = lane; i < a.vdim; i += 32) {
          float v = to_f32(src[i]);
          if (a.v_bias) v += a.v_bias[hh * a.vdim + i];
          dst[i] = from_f32<T>(v);
        }
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------ block means
struct PwaPoolArgs {
  const int* positions; const int* token_slot;
  int kv_heads, dim, vdim, pool;
  PwaCache tokens, blocks;
  int* error_word;
};

// grid (tokens, kv_heads); a block has work only where its token completes a block of `pool` positions.  The block's
// positions are dealt to kPoolLanes lanes (lane l sums l, l + lanes, ... in rising order, every load of a thread in
// flight at once); then one thread per element adds the lanes' sums in the order of the lanes.  The order is the same
// wherever the block is completed, in a prompt's portion or by a single token.
constexpr int kPoolLanes = 8;
constexpr int kPoolTile = 64;             // elements a lane's threads cover side by side
constexpr int kPoolAhead = 8;             // loads a thread keeps in flight

template <typename T>
__global__ void __launch_bounds__(kPoolLanes * kPoolTile) pwa_pool_kernel(PwaPoolArgs a) {
  pdl_wait();
  pdl_trigger();
  __shared__ float part_s[kPoolLanes][kPoolTile + 1];
  const int t = blockIdx.x, kvh = blockIdx.y;
  const int pos = a.positions[t];
  if (pos % a.pool != a.pool - 1) return;
  const int b = pos / a.pool, first = b * a.pool, slot = a.token_slot[t];
  const int* ttable = a.tokens.block_table + (size_t)slot * a.tokens.table_stride;
  const int* btable = a.blocks.block_table + (size_t)slot * a.blocks.table_stride;
  const int bpage = pwa_page(a.blocks, btable, b, a.error_word, 0x40000 + (t & 0xffff));
  if (bpage < 0) return;
  const int width = a.dim + a.vdim;
  const float inv = 1.f / (float)a.pool;
  const int lane = threadIdx.x / kPoolTile, col = threadIdx.x % kPoolTile;
  bool bad = false;
  for (int e0 = 0; e0 < width; e0 += kPoolTile) {
    const int e = e0 + col;
    const bool live = e < width, is_k = e < a.dim;
    const int dd = is_k ? e : e - a.dim, w = is_k ? a.dim : a.vdim;
    const T* base = reinterpret_cast<const T*>(is_k ? a.tokens.keys : a.tokens.values);
    float sum = 0.f;
    for (int j0 = lane; j0 < a.pool; j0 += kPoolLanes * kPoolAhead) {
      float got[kPoolAhead];
#pragma unroll
      for (int u = 0; u < kPoolAhead; ++u) {
        const int j = j0 + u * kPoolLanes;
        got[u] = 0.f;
        if (!live || j >= a.pool) continue;
        const int page = ttable[(first + j) / a.tokens.page_size];
        if (page < 0 || page >= a.tokens.num_pages) { bad = true; continue; }
        got[u] = to_f32(base[(size_t)page * a.tokens.page_stride + ((size_t)kvh * a.tokens.page_size + (first + j) % a.tokens.page_size) * w + dd]);
      }
#pragma unroll
      for (int u = 0; u < kPoolAhead; ++u) sum += got[u];
    }
    __syncthreads();
    part_s[lane][col] = sum;
    __syncthreads();
    if (lane == 0 && live) {
      float total = 0.f;
#pragma unroll
      for (int l = 0; l < kPoolLanes; ++l) total += part_s[l][col];
      T* out = reinterpret_cast<T*>(is_k ? a.blocks.keys : a.blocks.values);
      out[(size_t)bpage * a.blocks.page_stride + ((size_t)kvh * a.blocks.page_size + b % a.blocks.page_size) * w + dd] = from_f32<T>(total * inv);
    }
  }
  if (bad && a.error_word) atomicExch(a.error_word, 0x50000 + (t & 0xffff));
}

// ------------------------------------------------------------------------------------------------- attention
constexpr int kPwaWarps = 4;
constexpr int kPwaRowsPerWarp = 4;
constexpr int kPwaRows = kPwaWarps * kPwaRowsPerWarp;      // rows (token, head) per block
constexpr int kPwaKeys = 32;                               // keys per step = lanes

struct PwaArgs {
  const int* q_start; const int* kv_start; const int* slots;
  int heads, kv_heads, dim, vdim;
  int window, pool;                  // pool 0: no blocks, only the window
  float scale;
  const float* temp; const float* sink;                    // [heads] or null
  const float* vfreq;                                      // [vdim / 2] or null (values were not turned)
  const void* gate; int gate_dtype; int64_t ld_gate;       // [tokens, heads * vdim] logits or null
  const float* rel_bias; int rel_span;                     // [heads, rel_span] or null: added to a token's score by distance
  PwaCache tokens, blocks;
  int group_chunk, q_tile;
  int* error_word;
  float* partial; int n_splits; int n_tokens;              // a step of single tokens whose contexts are shared out over blocks
};

template <typename T, int DPL>
__global__ void __launch_bounds__(kPwaWarps * 32)
pwa_attention_kernel(const T* __restrict__ q, T* __restrict__ out, PwaArgs a) {
  pdl_wait();
  pdl_trigger();
  extern __shared__ float smem[];
  const int d = a.dim, dv = a.vdim;
  float* q_s = smem;                             // [kPwaRows][d]
  float* k_s = q_s + kPwaRows * d;               // [32][d + 1]
  float* v_s = k_s + kPwaKeys * (d + 1);         // [32][dv]
  float* o_s = v_s + kPwaKeys * dv;              // [kPwaWarps][dv]: a row's sum, for the turning back

  const int entry = blockIdx.y;
  const int group = a.heads / a.kv_heads;
  const int chunks = (group + a.group_chunk - 1) / a.group_chunk;
  const int kvh = blockIdx.z / chunks;
  const int g0 = (blockIdx.z - kvh * chunks) * a.group_chunk;
  const int gc = min(a.group_chunk, group - g0);

  const int row0 = a.q_start[entry];
  const int q_len = a.q_start[entry + 1] - row0;
  const int t0 = blockIdx.x * a.q_tile;
  if (t0 >= q_len) return;
  const int nt = min(a.q_tile, q_len - t0);
  const int nrows = nt * gc;
  const int pos0 = a.kv_start[entry] + t0;       // position of the first query of the tile
  const int last_pos = pos0 + nt - 1;
  const int slot = a.slots[entry];
  const int* ttable = a.tokens.block_table + (size_t)slot * a.tokens.table_stride;
  const int* btable = a.pool > 0 ? a.blocks.block_table + (size_t)slot * a.blocks.table_stride : nullptr;

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int q_width = a.heads * d, o_width = a.heads * dv;

  for (int e = threadIdx.x; e < nrows * d; e += blockDim.x) {
    const int r = e / d, dd = e - r * d;
    const int t = r / gc, g = r - t * gc;
    q_s[r * d + dd] = to_f32(q[(size_t)(row0 + t0 + t) * q_width + (kvh * group + g0 + g) * d + dd]);
  }

  float m[kPwaRowsPerWarp], l[kPwaRowsPerWarp], acc[kPwaRowsPerWarp][DPL], factor[kPwaRowsPerWarp];
#pragma unroll
  for (int i = 0; i < kPwaRowsPerWarp; ++i) {
    m[i] = -CUDART_INF_F;
    l[i] = 0.f;
#pragma unroll
    for (int j = 0; j < DPL; ++j) acc[i][j] = 0.f;
    const int r = warp * kPwaRowsPerWarp + i;
    const int head = kvh * group + g0 + (r < nrows ? r % gc : 0);
    factor[i] = a.scale * (a.temp ? a.temp[head] : 1.f);
  }

  // how many blocks the last query of the tile sees, and the first token any query of the tile sees
  const int n_blocks = a.pool > 0 ? max(0, last_pos - a.window + 1) / a.pool : 0;
  const int first_key = max(0, pos0 - a.window + 1);
  const int steps_b = (n_blocks + kPwaKeys - 1) / kPwaKeys;
  const int s_lo = first_key / kPwaKeys, s_hi = last_pos / kPwaKeys;

  for (int step = 0; step < steps_b + (s_hi - s_lo + 1); ++step) {
    const bool pooled = step < steps_b;
    const int base = pooled ? step * kPwaKeys : (s_lo + step - steps_b) * kPwaKeys;      // first block / position of the step
    const PwaCache& c = pooled ? a.blocks : a.tokens;
    const int* table = pooled ? btable : ttable;
    __syncthreads();      // the tiles of the step before are no longer read (and q_s is written)
    // Keys outside what the tile can see are zeros and always masked (unwritten cache may hold anything).
    for (int e = threadIdx.x; e < kPwaKeys * (d + dv); e += blockDim.x) {
      const int j = e / (d + dv), dd = e - j * (d + dv);
      const int idx = base + j;
      const bool wanted = pooled ? idx < n_blocks : (idx <= last_pos && idx >= first_key);
      float val = 0.f;
      if (wanted) {
        const int page = pwa_page(c, table, idx, a.error_word, 0x10000 + entry);
        if (page >= 0) {
          const size_t at = (size_t)page * c.page_stride + ((size_t)kvh * c.page_size + idx % c.page_size) * (dd < d ? d : dv);
          val = dd < d ? to_f32(reinterpret_cast<const T*>(c.keys)[at + dd]) : to_f32(reinterpret_cast<const T*>(c.values)[at + dd - d]);
        }
      }
      if (dd < d) k_s[j * (d + 1) + dd] = val;
      else v_s[j * dv + dd - d] = val;
    }
    __syncthreads();

#pragma unroll
    for (int i = 0; i < kPwaRowsPerWarp; ++i) {
      const int r = warp * kPwaRowsPerWarp + i;
      if (r >= nrows) continue;                       // uniform in the warp
      const int qpos = pos0 + r / gc;
      const int idx = base + lane;
      bool allowed;
      if (pooled) {
        const int seen = max(0, qpos - a.window + 1) / a.pool;      // blocks 0 .. seen - 1 lie wholly behind the window
        if (base >= seen) continue;
        allowed = idx < seen;
      } else {
        const int lo = max(0, qpos - a.window + 1);
        if (base > qpos || base + kPwaKeys - 1 < lo) continue;
        allowed = idx <= qpos && idx >= lo;
      }
      float s = 0.f;
      const float* qr = q_s + r * d;
      const float* kr = k_s + lane * (d + 1);
      for (int dd = 0; dd < d; ++dd) s = fmaf(qr[dd], kr[dd], s);
      s = allowed ? s * factor[i] : -CUDART_INF_F;
      if (a.rel_bias && allowed && !pooled)           // a learned number per head and distance (the last entry serves all beyond)
        s += a.rel_bias[(size_t)(kvh * group + g0 + r % gc) * a.rel_span + min(qpos - idx, a.rel_span - 1)];
      const float m_new = fmaxf(m[i], warp_max(s));   // finite: the step holds a key the row sees
      const float alpha = m[i] == -CUDART_INF_F ? 0.f : expf(m[i] - m_new);
      const float p = allowed ? expf(s - m_new) : 0.f;
      l[i] = l[i] * alpha + warp_sum(p);
      m[i] = m_new;
#pragma unroll
      for (int j = 0; j < DPL; ++j) acc[i][j] *= alpha;
      for (int kk = 0; kk < kPwaKeys; ++kk) {
        const float pk = __shfl_sync(0xffffffffu, p, kk);
#pragma unroll
        for (int j = 0; j < DPL; ++j) {
          const int dd = lane + 32 * j;
          if (dd < dv) acc[i][j] = fmaf(pk, v_s[kk * dv + dd], acc[i][j]);
        }
      }
    }
  }

  float* o_row = o_s + warp * dv;
#pragma unroll
  for (int i = 0; i < kPwaRowsPerWarp; ++i) {
    const int r = warp * kPwaRowsPerWarp + i;
    if (r >= nrows) continue;
    const int t = r / gc, g = r - t * gc;
    const int head = kvh * group + g0 + g;
    const size_t token = (size_t)(row0 + t0 + t);
    // the number in the denominator has no key: it only takes weight away from the others
    float top = m[i], denom = l[i];
    if (a.sink) {
      const float sink = a.sink[head];
      top = fmaxf(m[i], sink);
      denom = l[i] * expf(m[i] - top) + expf(sink - top);
    }
    const float inv = expf(m[i] - top) / denom;
    __syncwarp();
#pragma unroll
    for (int j = 0; j < DPL; ++j) {
      const int dd = lane + 32 * j;
      if (dd < dv) o_row[dd] = acc[i][j] * inv;
    }
    __syncwarp();
    T* dst = out + token * o_width + head * dv;
    const float fpos = (float)(pos0 + t);
    const int half = dv / 2;
    for (int mm = lane; mm < (a.vfreq ? half : dv); mm += 32) {
      if (a.vfreq) {
        // turn the pair (mm, mm + half) back by the query's position: (u, v) -> (u cos + v sin, v cos - u sin)
        const float angle = fpos * a.vfreq[mm];
        const float c = cosf(angle), s = sinf(angle);
        float u = rope_lo(o_row[mm], o_row[mm + half], c, -s), v = rope_hi(o_row[mm], o_row[mm + half], c, -s);
        if (a.gate) {
          const float gu = a.gate_dtype == TIB_F32 ? reinterpret_cast<const float*>(a.gate)[token * a.ld_gate + head * dv + mm]
                                                   : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(a.gate)[token * a.ld_gate + head * dv + mm]);
          const float gv = a.gate_dtype == TIB_F32 ? reinterpret_cast<const float*>(a.gate)[token * a.ld_gate + head * dv + mm + half]
                                                   : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(a.gate)[token * a.ld_gate + head * dv + mm + half]);
          u *= 1.f / (1.f + expf(-gu));
          v *= 1.f / (1.f + expf(-gv));
        }
        dst[mm] = from_f32<T>(u);
        dst[mm + half] = from_f32<T>(v);
      } else {
        float u = o_row[mm];
        if (a.gate) {
          const float gu = a.gate_dtype == TIB_F32 ? reinterpret_cast<const float*>(a.gate)[token * a.ld_gate + head * dv + mm]
                                                   : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(a.gate)[token * a.ld_gate + head * dv + mm]);
          u *= 1.f / (1.f + expf(-gu));
        }
        dst[mm] = from_f32<T>(u);
      }
    }
  }
}

template <typename T, int DPL>
static int pwa_launch(const void* q, void* out, const PwaArgs& a, int n_entries, int max_q_len, cudaStream_t stream) {
  const size_t smem = sizeof(float) * ((size_t)kPwaRows * a.dim + (size_t)kPwaKeys * (a.dim + 1) + (size_t)kPwaKeys * a.vdim +
                                       (size_t)kPwaWarps * a.vdim);
  if (smem > 227 * 1024) return TIB_E_SMEM;
  auto kern = pwa_attention_kernel<T, DPL>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  const int group = a.heads / a.kv_heads;
  const int chunks = (group + a.group_chunk - 1) / a.group_chunk;
  const dim3 grid(ceil_div(max_q_len, a.q_tile), n_entries, a.kv_heads * chunks);
  TIB_LAUNCH_DEPENDENT(kern, grid, kPwaWarps * 32, smem, stream, (const T*)q, (T*)out, a);
  return TIB_OK;
}

// ------------------------------------------------------------ tensor cores
// 64 rows (tokens x the query heads of one kv head) against tiles of 64 keys, four warps of 16 rows: first the tiles of
// block means (aligned to absolute block numbers), then the tiles of tokens (aligned to absolute positions), both in
// rising order, so a row's sums do not depend on how the prompt was cut or on what else the step holds.  Keys and values
// of a tile come in by cp.async, row by row from their pages, two stages; rows the tile's queries cannot see are
// zero-filled (unwritten cache may hold anything) and masked.  Scores accumulate in fp32; the softmax runs in fp32 on
// scores in units of ln 2; the weights enter the second product as a high bf16 part plus the remainder, so that they
// keep 16 bits.  The rows' sums then pass through shared memory, where pairs (m, m + vdim / 2) meet for the turning back.
constexpr int kPmRows = 64, kPmKeys = 64, kPmThreads = 128;
// Tiles a block of few rows has in flight (a warp each) when the contexts are shared out over blocks.  Two: the stages are
// 87 KB and two blocks share an SM, so that one block's loads run under the other's arithmetic; with four (156 KB, a block
// an SM: the form for contexts that are not shared out) nothing overlaps.
constexpr int kPmFewRowStages = 2;
constexpr float kLog2e = 1.4426950408889634f;

// REL: the kernel knows the table of biases by distance and contexts shared out over blocks (without it, it is the kernel
// as the designs without either have always run it, register for register).
template <int DK, int DV, int ST, bool WT, bool REL>
__global__ void __launch_bounds__(kPmThreads)
pwa_attention_mma_kernel(const __nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ out, PwaArgs a) {
  pdl_wait();
  pdl_trigger();
  constexpr int KP = DK + 8, VP = DV + 8;        // padded rows: ldmatrix rows fall in different banks
  extern __shared__ __align__(16) unsigned char sm_raw[];
  __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(sm_raw);          // [64][KP]
  __nv_bfloat16* k_s = q_s + kPmRows * KP;                                 // [ST][64][KP]
  __nv_bfloat16* v_s = k_s + ST * kPmKeys * KP;                            // [ST][64][VP]
  __shared__ long long page_base[ST][kPmKeys];
  __shared__ int key_row[ST][kPmKeys];

  const int d = a.dim, vd = a.vdim;
  const int entry = blockIdx.y;
  const int group = a.heads / a.kv_heads;
  const int chunks = (group + a.group_chunk - 1) / a.group_chunk;
  const int kvh = blockIdx.z / chunks;
  const int g0 = (blockIdx.z - kvh * chunks) * a.group_chunk;
  const int gc = min(a.group_chunk, group - g0);
  const int row0 = a.q_start[entry];
  const int q_len = a.q_start[entry + 1] - row0;
  // (with the contexts shared out, blockIdx.x counts the parts of a context, and the block's rows are the entry's only ones)
  const bool shared_out = REL && WT && a.n_splits > 1;
  const int t0 = shared_out ? 0 : blockIdx.x * a.q_tile;
  if (t0 >= q_len) return;
  const int nt = min(a.q_tile, q_len - t0);
  const int nrows = nt * gc;
  const int pos0 = a.kv_start[entry] + t0;
  const int last_pos = pos0 + nt - 1;
  const int slot = a.slots[entry];
  const int* ttable = a.tokens.block_table + (size_t)slot * a.tokens.table_stride;
  const int* btable = a.pool > 0 ? a.blocks.block_table + (size_t)slot * a.blocks.table_stride : nullptr;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  // how many blocks the last query of the tile sees, and the first token any query of the tile sees
  const int n_blocks = a.pool > 0 ? max(0, last_pos - a.window + 1) / a.pool : 0;
  const int first_key = max(0, pos0 - a.window + 1);
  const int steps_b = (n_blocks + kPmKeys - 1) / kPmKeys;
  const int s_lo = first_key / kPmKeys, s_hi = last_pos / kPmKeys;
  const int steps = steps_b + (s_hi - s_lo + 1);
  int step_lo = 0, step_hi = steps;                   // this block's share of the tiles
  if (shared_out) {
    const int per = (steps + a.n_splits - 1) / a.n_splits;
    step_lo = min(steps, (int)blockIdx.x * per);
    step_hi = min(steps, step_lo + per);
  }

  // where key j of a tile lives: its page's first element and its row in the page
  auto locate = [&](int stage, int step, int j) {
    const bool pooled = step < steps_b;
    const PwaCache& c = pooled ? a.blocks : a.tokens;
    const int idx = (pooled ? step : s_lo + step - steps_b) * kPmKeys + j;
    long long base = -1;
    int row = 0;
    if (pooled ? idx < n_blocks : (idx <= last_pos && idx >= first_key)) {
      const int page = pwa_page(c, pooled ? btable : ttable, idx, a.error_word, 0x10000 + entry);
      if (page >= 0) {
        base = (long long)page * c.page_stride;
        row = kvh * c.page_size + idx % c.page_size;
      }
    }
    page_base[stage][j] = base;
    key_row[stage][j] = row;
  };
  // the tile's keys and values, row by row from where `locate` found them
  auto copy = [&](int stage, int step) {
    const bool pooled = step < steps_b;
    const PwaCache& c = pooled ? a.blocks : a.tokens;
    const __nv_bfloat16* k_pages = reinterpret_cast<const __nv_bfloat16*>(c.keys);
    const __nv_bfloat16* v_pages = reinterpret_cast<const __nv_bfloat16*>(c.values);
    constexpr int KPIECES = DK / 8, VPIECES = DV / 8;
    for (int e = tid; e < kPmKeys * KPIECES; e += kPmThreads) {
      const int j = e / KPIECES, cc = (e - j * KPIECES) * 8;
      const long long base = page_base[stage][j];
      const bool ok = base >= 0 && cc < d;
      cp_async16(k_s + ((size_t)stage * kPmKeys + j) * KP + cc, k_pages + (ok ? base + (long long)key_row[stage][j] * d + cc : 0), ok);
    }
    for (int e = tid; e < kPmKeys * VPIECES; e += kPmThreads) {
      const int j = e / VPIECES, cc = (e - j * VPIECES) * 8;
      const long long base = page_base[stage][j];
      const bool ok = base >= 0 && cc < vd;
      cp_async16(v_s + ((size_t)stage * kPmKeys + j) * VP + cc, v_pages + (ok ? base + (long long)key_row[stage][j] * vd + cc : 0), ok);
    }
    cp_async_commit();
  };
  auto fetch = [&](int stage, int step) {
    if (tid < kPmKeys) locate(stage, step, tid);
    __syncthreads();
    copy(stage, step);
  };

  // queries: 16-byte pieces, rows past the tile's end and padding columns are zero
  {
    constexpr int QPIECES = DK / 8;
    for (int e = tid; e < kPmRows * QPIECES; e += kPmThreads) {
      const int r = e / QPIECES, cc = (e - r * QPIECES) * 8;
      const bool ok = r < nrows && cc < d;
      const int t = ok ? r / gc : 0, g = ok ? r - t * gc : 0;
      const __nv_bfloat16* src = q + (size_t)(row0 + t0 + t) * a.heads * d + (size_t)(kvh * group + g0 + g) * d + (ok ? cc : 0);
      cp_async16(q_s + (size_t)r * KP + cc, src, ok);
    }
  }
  // ST - 1 tiles ahead (there is always the tile of the query's own position); every step commits one group, an empty
  // one when no tile is left, so that the wait below always leaves the same number pending
  if (!WT) {
#pragma unroll
    for (int s0 = 0; s0 < ST - 1; ++s0) {
      if (s0 < steps) fetch(s0, s0);
      else cp_async_commit();
    }
  }

  // this thread's two rows: g8 and g8 + 8 of the warp's sixteen
  const int g8 = lane >> 2, t4 = lane & 3;
  const int row_base = WT ? 0 : warp * 16;           // (WT: every warp holds the block's only sixteen rows)
  int qpos[2], lo[2], seen[2];
  float factor[2], m[2], l[2];
  bool live[2];
  const float* rel[2];               // the row's head's biases by distance, or null
  float rel_far[2];                  // the bias of every distance from the table's last on, in units of ln 2
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = row_base + g8 + 8 * h;
    live[h] = r < nrows;
    const int t = live[h] ? r / gc : 0, g = live[h] ? r - t * gc : 0;
    qpos[h] = pos0 + t;
    lo[h] = max(0, qpos[h] - a.window + 1);
    seen[h] = a.pool > 0 ? lo[h] / a.pool : 0;       // blocks 0 .. seen - 1 lie wholly behind the window
    factor[h] = a.scale * (a.temp ? a.temp[kvh * group + g0 + g] : 1.f) * kLog2e;
    rel[h] = REL && a.rel_bias ? a.rel_bias + (size_t)(kvh * group + g0 + g) * a.rel_span : nullptr;
    rel_far[h] = REL && rel[h] ? rel[h][a.rel_span - 1] * kLog2e : 0.f;
    m[h] = -CUDART_INF_F;
    l[h] = 0.f;
  }
  constexpr int NT = kPmKeys / 8;
  float o[DV / 8][4];
#pragma unroll
  for (int n = 0; n < DV / 8; ++n)
#pragma unroll
    for (int c = 0; c < 4; ++c) o[n][c] = 0.f;
  // what the warp's rows see, for skipping whole tiles
  const int warp_first = pos0 + row_base / gc, warp_last = pos0 + min(nrows - 1, row_base + 15) / gc;
  const int warp_lo = max(0, warp_first - a.window + 1);
  const int warp_seen = a.pool > 0 ? max(0, warp_last - a.window + 1) / a.pool : 0;

  auto tile = [&](int stage, int step) {
    const bool pooled = step < steps_b;
    const int base = (pooled ? step : s_lo + step - steps_b) * kPmKeys;
    // (a warp whose rows see nothing of this tile still passes the barriers)
    const bool any = row_base < nrows && (pooled ? base < warp_seen : (base <= warp_last && base + kPmKeys - 1 >= warp_lo));
    if (any) {
      const __nv_bfloat16* kt = k_s + (size_t)stage * kPmKeys * KP;
      const __nv_bfloat16* vt = v_s + (size_t)stage * kPmKeys * VP;
      float s[NT][4];
#pragma unroll
      for (int n = 0; n < NT; ++n)
#pragma unroll
        for (int c = 0; c < 4; ++c) s[n][c] = 0.f;
#pragma unroll
      for (int kk = 0; kk < DK; kk += 16) {
        uint32_t af[4];
        ldmatrix_x4(af, q_s + (size_t)(row_base + (lane & 15)) * KP + kk + (lane >> 4) * 8);
#pragma unroll
        for (int j = 0; j < NT / 2; ++j) {
          uint32_t bf[4];
          ldmatrix_x4(bf, kt + (size_t)(j * 16 + ((lane >> 4) << 3) + (lane & 7)) * KP + kk + ((lane >> 3) & 1) * 8);
          mma_bf16(s[2 * j], af, bf[0], bf[1]);
          mma_bf16(s[2 * j + 1], af, bf[2], bf[3]);
        }
      }
      // mask, then the streaming softmax in fp32 (scores in units of ln 2)
#pragma unroll
      for (int n = 0; n < NT; ++n)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int h = c >> 1;
          const int idx = base + n * 8 + 2 * t4 + (c & 1);
          const bool allowed = live[h] && (pooled ? idx < seen[h] : (idx <= qpos[h] && idx >= lo[h]));
          s[n][c] = allowed ? s[n][c] * factor[h] : -CUDART_INF_F;
        }
      if (REL && a.rel_bias && !pooled) {
        // the learned number of every (head, distance), without a branch per score: a masked score stays minus infinity
        // whatever is added, so its distance is clamped into the table; a row whose every key of the tile lies beyond
        // the table's last distance reads nothing
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int d0 = qpos[h] - base - 2 * t4;            // distance to the first of this thread's keys
          if (d0 - (kPmKeys - 1) >= a.rel_span - 1) {
#pragma unroll
            for (int n = 0; n < NT; ++n) {
              s[n][2 * h] += rel_far[h];
              s[n][2 * h + 1] += rel_far[h];
            }
          } else {
#pragma unroll
            for (int n = 0; n < NT; ++n)
#pragma unroll
              for (int b = 0; b < 2; ++b)
                s[n][2 * h + b] = fmaf(rel[h][min(max(d0 - n * 8 - b, 0), a.rel_span - 1)], kLog2e, s[n][2 * h + b]);
          }
        }
      }
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        float mx = -CUDART_INF_F;
#pragma unroll
        for (int n = 0; n < NT; ++n) mx = fmaxf(mx, fmaxf(s[n][2 * h], s[n][2 * h + 1]));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m[h], mx);
        const float top = m_new == -CUDART_INF_F ? 0.f : m_new;
        const float alpha = exp2f(m[h] - top);
        m[h] = m_new;
        float sum = 0.f;
#pragma unroll
        for (int n = 0; n < NT; ++n) {
          s[n][2 * h] = exp2f(s[n][2 * h] - top);
          s[n][2 * h + 1] = exp2f(s[n][2 * h + 1] - top);
          sum += s[n][2 * h] + s[n][2 * h + 1];
        }
        l[h] = l[h] * alpha + sum;
        if (__any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll
          for (int n = 0; n < DV / 8; ++n) {
            o[n][2 * h] *= alpha;
            o[n][2 * h + 1] *= alpha;
          }
        }
      }
      uint32_t p_hi[NT / 2][4], p_lo[NT / 2][4];
#pragma unroll
      for (int n = 0; n < NT; ++n) {
        const int kk = n >> 1, half = (n & 1) * 2;
        const __nv_bfloat162 h01 = __floats2bfloat162_rn(s[n][0], s[n][1]), h23 = __floats2bfloat162_rn(s[n][2], s[n][3]);
        p_hi[kk][half] = *reinterpret_cast<const uint32_t*>(&h01);
        p_hi[kk][half + 1] = *reinterpret_cast<const uint32_t*>(&h23);
        const float2 f01 = bf16x2_floats(h01), f23 = bf16x2_floats(h23);
        p_lo[kk][half] = pack_bf16(s[n][0] - f01.x, s[n][1] - f01.y);
        p_lo[kk][half + 1] = pack_bf16(s[n][2] - f23.x, s[n][3] - f23.y);
      }
#pragma unroll
      for (int kk = 0; kk < NT / 2; ++kk) {
        uint32_t bv[DV / 16][4];
#pragma unroll
        for (int dn = 0; dn < DV / 16; ++dn) {
          ldmatrix_x4_trans(bv[dn], vt + (size_t)(kk * 16 + (lane & 15)) * VP + dn * 16 + ((lane >> 4) << 3));
          mma_bf16(o[2 * dn], p_hi[kk], bv[dn][0], bv[dn][1]);
          mma_bf16(o[2 * dn + 1], p_hi[kk], bv[dn][2], bv[dn][3]);
        }
#pragma unroll
        for (int dn = 0; dn < DV / 16; ++dn) {
          mma_bf16(o[2 * dn], p_lo[kk], bv[dn][0], bv[dn][1]);
          mma_bf16(o[2 * dn + 1], p_lo[kk], bv[dn][2], bv[dn][3]);
        }
      }
    }
  };
  if (WT) {
    // Few rows: only one warp would have work.  So ST of the warps each take one tile of a set of ST (all in flight
    // at once), with sums of their own, which are added in the order of the warps afterwards.
    static_assert(!WT || ST <= kPmThreads / 32, "at most a stage a warp");
    for (int first = step_lo; first < step_hi; first += ST) {
      // (all of the set's page numbers are asked for at once, then all of its tiles)
      for (int e = tid; e < ST * kPmKeys; e += kPmThreads)
        if (first + e / kPmKeys < step_hi) locate(e / kPmKeys, first + e / kPmKeys, e % kPmKeys);
      __syncthreads();
#pragma unroll
      for (int s0 = 0; s0 < ST; ++s0)
        if (first + s0 < step_hi) copy(s0, first + s0);
      cp_async_wait<0>();
      __syncthreads();
      if (warp < ST && first + warp < step_hi) tile(warp, first + warp);
      __syncthreads();    // the stages are free for the next set
    }
  } else {
    for (int step = 0; step < steps; ++step) {
      const int stage = step % ST;
      if (step + ST - 1 < steps) fetch((step + ST - 1) % ST, step + ST - 1);      // (the stage of the step before this one)
      else cp_async_commit();
      cp_async_wait<ST - 1>();
      __syncthreads();
      tile(stage, step);
      __syncthreads();      // the stage is free for the next step's fetch
    }
  }

  if (WT) {
    // every warp leaves its maxima, denominators and sums where warp 0's thread of the same lane finds them
    constexpr int PER = DV / 2 + 4;                      // floats a thread leaves
    float* part_s = reinterpret_cast<float*>(k_s);       // [warps][32][PER] over the stages
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      l[h] += __shfl_xor_sync(0xffffffffu, l[h], 1);
      l[h] += __shfl_xor_sync(0xffffffffu, l[h], 2);
    }
    if (warp > 0) {
      float* mine = part_s + ((size_t)warp * 32 + lane) * PER;
      mine[0] = m[0], mine[1] = m[1], mine[2] = l[0], mine[3] = l[1];
#pragma unroll
      for (int n = 0; n < DV / 8; ++n)
#pragma unroll
        for (int c = 0; c < 4; ++c) mine[4 + n * 4 + c] = o[n][c];
    }
    __syncthreads();
    if (warp == 0) {
      float top[2] = {m[0], m[1]};
      for (int w = 1; w < kPmThreads / 32; ++w) {
        const float* theirs = part_s + ((size_t)w * 32 + lane) * PER;
        top[0] = fmaxf(top[0], theirs[0]);
        top[1] = fmaxf(top[1], theirs[1]);
      }
      float keep[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        keep[h] = m[h] == -CUDART_INF_F ? 0.f : exp2f(m[h] - top[h]);
        l[h] *= keep[h];
        m[h] = top[h];
      }
#pragma unroll
      for (int n = 0; n < DV / 8; ++n)
#pragma unroll
        for (int c = 0; c < 4; ++c) o[n][c] *= keep[c >> 1];
      for (int w = 1; w < kPmThreads / 32; ++w) {
        const float* theirs = part_s + ((size_t)w * 32 + lane) * PER;
        float weight[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          weight[h] = theirs[h] == -CUDART_INF_F ? 0.f : exp2f(theirs[h] - top[h]);
          l[h] = fmaf(theirs[2 + h], weight[h], l[h]);
        }
#pragma unroll
        for (int n = 0; n < DV / 8; ++n)
#pragma unroll
          for (int c = 0; c < 4; ++c) o[n][c] = fmaf(theirs[4 + n * 4 + c], weight[c >> 1], o[n][c]);
      }
    }
    __syncthreads();      // the partial sums are read: the place is free for the rows' sums
    if (shared_out) {
      // this part's maxima, denominators and sums (in units of ln 2, not yet divided) go to the kernel that adds the parts
      if (warp == 0) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int r = g8 + 8 * h;
          if (!live[h]) continue;
          const int t = r / gc, g = r - t * gc;
          float* dst = a.partial + (((size_t)blockIdx.x * a.n_tokens + (row0 + t)) * a.heads + (kvh * group + g0 + g)) * (DV + 2);
          if (t4 == 0) { dst[0] = m[h]; dst[1] = l[h]; }
#pragma unroll
          for (int n = 0; n < DV / 8; ++n) {
            dst[2 + n * 8 + 2 * t4] = o[n][2 * h];
            dst[2 + n * 8 + 2 * t4 + 1] = o[n][2 * h + 1];
          }
        }
      }
      return;
    }
  }
  // the rows' sums, divided by the softmax's denominator (with the number that has no key), into shared memory
  float* o_s = reinterpret_cast<float*>(k_s);           // [64][DV] floats over the key and value stages, which adjoin
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    float sum = l[h];
    if (!WT) {                                           // (WT: already summed over the four lanes of a row)
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    }
    float inv = 0.f;
    if (live[h]) {
      const int r = row_base + g8 + 8 * h;
      float top = m[h], denom = sum;
      if (a.sink) {
        const float sink = a.sink[kvh * group + g0 + (r - (r / gc) * gc)] * kLog2e;
        top = fmaxf(m[h], sink);
        denom = sum * exp2f(m[h] - top) + exp2f(sink - top);
      }
      inv = exp2f(m[h] - top) / denom;
    }
    const int r = row_base + g8 + 8 * h;
    if (WT && warp > 0) continue;                        // (warp 0 holds the rows' whole sums)
#pragma unroll
    for (int n = 0; n < DV / 8; ++n) {
      o_s[(size_t)r * DV + n * 8 + 2 * t4] = o[n][2 * h] * inv;
      o_s[(size_t)r * DV + n * 8 + 2 * t4 + 1] = o[n][2 * h + 1] * inv;
    }
  }
  __syncthreads();
  const int o_width = a.heads * vd;
  const int half = vd / 2;
  const int per_row = a.vfreq ? half : vd;
  const __nv_bfloat16* gate = reinterpret_cast<const __nv_bfloat16*>(a.gate);
  for (int e = tid; e < nrows * per_row; e += kPmThreads) {
    const int r = e / per_row, mm = e - r * per_row;
    const int t = r / gc, g = r - t * gc;
    const int head = kvh * group + g0 + g;
    const size_t token = (size_t)(row0 + t0 + t);
    __nv_bfloat16* dst = out + token * o_width + (size_t)head * vd;
    const float* o_row = o_s + (size_t)r * DV;
    if (a.vfreq) {
      // turn the pair (mm, mm + half) back by the query's position: (u, v) -> (u cos + v sin, v cos - u sin)
      const float angle = (float)(pos0 + t) * a.vfreq[mm];
      const float c = cosf(angle), sn = sinf(angle);
      float u = rope_lo(o_row[mm], o_row[mm + half], c, -sn), v = rope_hi(o_row[mm], o_row[mm + half], c, -sn);
      if (gate) {
        const float gu = a.gate_dtype == TIB_F32 ? reinterpret_cast<const float*>(a.gate)[token * a.ld_gate + head * vd + mm]
                                                 : __bfloat162float(gate[token * a.ld_gate + head * vd + mm]);
        const float gv = a.gate_dtype == TIB_F32 ? reinterpret_cast<const float*>(a.gate)[token * a.ld_gate + head * vd + mm + half]
                                                 : __bfloat162float(gate[token * a.ld_gate + head * vd + mm + half]);
        u *= 1.f / (1.f + expf(-gu));
        v *= 1.f / (1.f + expf(-gv));
      }
      dst[mm] = __float2bfloat16_rn(u);
      dst[mm + half] = __float2bfloat16_rn(v);
    } else {
      float u = o_row[mm];
      if (gate) {
        const float gu = a.gate_dtype == TIB_F32 ? reinterpret_cast<const float*>(a.gate)[token * a.ld_gate + head * vd + mm]
                                                 : __bfloat162float(gate[token * a.ld_gate + head * vd + mm]);
        u *= 1.f / (1.f + expf(-gu));
      }
      dst[mm] = __float2bfloat16_rn(u);
    }
  }
}

// Adds the parts of a context that was shared out over blocks, in the order of the parts: out = sum_s o_s 2^(m_s - top)
// / (sum_s l_s 2^(m_s - top) + 2^(sink - top)).  One block per token, a warp per head.
template <int DV>
__global__ void __launch_bounds__(128) pwa_merge_kernel(__nv_bfloat16* __restrict__ out, PwaArgs a) {
  pdl_wait();
  pdl_trigger();
  const int token = blockIdx.x, lane = threadIdx.x & 31;
  for (int head = threadIdx.x >> 5; head < a.heads; head += blockDim.x >> 5) {
    float top = -CUDART_INF_F;
    for (int s = 0; s < a.n_splits; ++s)
      top = fmaxf(top, a.partial[(((size_t)s * a.n_tokens + token) * a.heads + head) * (DV + 2)]);
    float denom = 0.f, acc[DV / 32];
#pragma unroll
    for (int j = 0; j < DV / 32; ++j) acc[j] = 0.f;
    for (int s = 0; s < a.n_splits; ++s) {
      const float* part = a.partial + (((size_t)s * a.n_tokens + token) * a.heads + head) * (DV + 2);
      if (part[0] == -CUDART_INF_F) continue;
      const float weight = exp2f(part[0] - top);
      denom = fmaf(part[1], weight, denom);
#pragma unroll
      for (int j = 0; j < DV / 32; ++j) acc[j] = fmaf(part[2 + lane + 32 * j], weight, acc[j]);
    }
    float scale = 1.f;
    if (a.sink) {
      const float sink = a.sink[head] * kLog2e, high = fmaxf(top, sink);
      scale = exp2f(top - high);
      denom = denom * scale + exp2f(sink - high);
    }
    const float inv = denom > 0.f ? scale / denom : 0.f;
#pragma unroll
    for (int j = 0; j < DV / 32; ++j)
      if (lane + 32 * j < a.vdim) out[(size_t)token * a.heads * a.vdim + (size_t)head * a.vdim + lane + 32 * j] = __float2bfloat16_rn(acc[j] * inv);
  }
}

template <int DK, int DV, int ST, bool WT, bool REL>
static int pwa_launch_mma_staged(const void* q, void* out, const PwaArgs& a, dim3 grid, cudaStream_t stream) {
  static_assert(kPmRows * DV * sizeof(float) <= ST * kPmKeys * (DK + 8 + DV + 8) * sizeof(__nv_bfloat16), "the rows' sums fit the stages");
  const size_t smem = sizeof(__nv_bfloat16) * ((size_t)kPmRows * (DK + 8) + ST * (size_t)kPmKeys * (DK + 8) + ST * (size_t)kPmKeys * (DV + 8));
  auto kern = pwa_attention_mma_kernel<DK, DV, ST, WT, REL>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  TIB_LAUNCH_DEPENDENT(kern, grid, kPmThreads, smem, stream, (const __nv_bfloat16*)q, (__nv_bfloat16*)out, a);
  return TIB_OK;
}

// In a step whose blocks all have at most sixteen rows (single tokens, say) one warp of four would have work while it
// walks a dozen tiles one after the other: there the warps take a tile each, four tiles in flight at once, and their
// sums are added afterwards in a fixed order.  A row's result then differs from the other form's in the order of fp32
// sums only.
template <int DK, int DV>
static int pwa_launch_mma(const void* q, void* out, PwaArgs a, int n_entries, int max_q_len, cudaStream_t stream) {
  const int group = a.heads / a.kv_heads;
  a.group_chunk = group < kPmRows ? group : kPmRows;
  a.q_tile = kPmRows / a.group_chunk;
  const int chunks = (group + a.group_chunk - 1) / a.group_chunk;
  if ((int64_t)a.kv_heads * chunks > 65535) return TIB_E_SIZE;
  dim3 grid(ceil_div(max_q_len, a.q_tile), n_entries, a.kv_heads * chunks);
  if ((int64_t)max_q_len * a.group_chunk <= 16) {
    if (a.n_splits > 1) {
      // single tokens whose contexts are shared out over n_splits blocks each; a second kernel adds the parts
      if (max_q_len != 1 || !a.partial || a.vfreq || a.gate) return TIB_E_ARG;
      grid.x = a.n_splits;
      const int status = pwa_launch_mma_staged<DK, DV, kPmFewRowStages, true, true>(q, out, a, grid, stream);
      if (status != TIB_OK) return status;
      TIB_LAUNCH_DEPENDENT(pwa_merge_kernel<DV>, a.n_tokens, 128, 0, stream, (__nv_bfloat16*)out, a);
      return TIB_OK;
    }
    a.n_splits = 1;
    if (a.rel_bias) return pwa_launch_mma_staged<DK, DV, kPmFewRowStages, true, true>(q, out, a, grid, stream);
    return pwa_launch_mma_staged<DK, DV, 4, true, false>(q, out, a, grid, stream);
  }
  a.n_splits = 1;
  if (a.rel_bias) return pwa_launch_mma_staged<DK, DV, 2, false, true>(q, out, a, grid, stream);
  return pwa_launch_mma_staged<DK, DV, 2, false, false>(q, out, a, grid, stream);
}

// How many blocks a step of `n_entries` single tokens should share each context of up to `max_kv_len` visible keys out
// over (1: none), and the floats of scratch a part of one (token, head) row takes.
TIB_API int tib_pooled_window_attention_splits(int n_entries, int heads, int kv_heads, int visible) {
  const int group = heads / (kv_heads < 1 ? 1 : kv_heads);
  if (group > 16) return 1;                            // (more than sixteen rows a block: the other form of the kernel)
  const int blocks = n_entries * kv_heads;
  const int sets = ceil_div(ceil_div(visible < 1 ? 1 : visible, kPmKeys) + 1, kPmFewRowStages);      // rounds of tiles
  int splits = 2 * 148 / (blocks < 1 ? 1 : blocks);
  if (splits > sets) splits = sets;
  if (splits > 32) splits = 32;
  return splits < 1 ? 1 : splits;
}
TIB_API int tib_pooled_window_attention_part_floats(int vdim) { return (vdim <= 64 ? 64 : 128) + 2; }

// Whether the tensor-core kernel takes these shapes (bf16; rows of 16-byte pieces in every array it copies from).
static bool pwa_mma_takes(const PwaArgs& a, const void* q) {
  const bool pieces = a.dim % 8 == 0 && a.vdim % 8 == 0 && a.dim <= 128 && a.vdim <= 128;
  uintptr_t bits = (uintptr_t)q | (uintptr_t)a.tokens.keys | (uintptr_t)a.tokens.values;
  bool strides = a.tokens.page_stride % 8 == 0;
  if (a.pool > 0) {
    bits |= (uintptr_t)a.blocks.keys | (uintptr_t)a.blocks.values;
    strides = strides && a.blocks.page_stride % 8 == 0;
  }
  return pieces && strides && (bits & 15) == 0;
}

static PwaCache pwa_cache(void* keys, void* values, const int* table, int table_stride, int page_size, int64_t page_stride, int num_pages) {
  PwaCache c;
  c.keys = keys; c.values = values; c.block_table = table; c.table_stride = table_stride; c.page_size = page_size;
  c.page_stride = page_stride; c.num_pages = num_pages;
  return c;
}

}  // namespace tib

using namespace tib;

// proj: [n_tokens, ld] rows holding q at q_off, k at k_off, v at v_off; q_out: [n_tokens, heads * dim]; k_pages / v_pages:
// first key / value of this layer's first page (null: only q is made).  Biases, freq and vfreq are fp32.
TIB_API int tib_rotary_kv_append(const void* proj, int64_t ld, int q_off, int k_off, int v_off, const float* q_bias,
                                 const float* k_bias, const float* v_bias, void* q_out, void* k_pages, void* v_pages,
                                 const int* positions, const int* token_slot, const int* block_table, int table_stride,
                                 const float* freq, const float* vfreq, float amplitude, int n_tokens, int heads, int kv_heads,
                                 int dim, int vdim, int rot_dim, int page_size, int64_t page_stride, int num_pages, int* error_word,
                                 int dtype, cudaStream_t stream) {
  if (n_tokens == 0) return TIB_OK;
  if (!proj || !q_out || !positions || n_tokens < 0 || heads < 1 || kv_heads < 1 || dim < 1 || vdim < 1) return TIB_E_ARG;
  if (rot_dim < 0 || rot_dim % 2 || rot_dim > dim || (rot_dim > 0 && !freq) || (vfreq && vdim % 2)) return TIB_E_SIZE;
  if (k_pages && (!v_pages || !token_slot || !block_table || page_size < 1)) return TIB_E_ARG;
  PwaAppendArgs a;
  a.ld = ld; a.q_off = q_off; a.k_off = k_off; a.v_off = v_off; a.q_bias = q_bias; a.k_bias = k_bias; a.v_bias = v_bias;
  a.positions = positions; a.token_slot = token_slot; a.freq = freq; a.vfreq = vfreq; a.amplitude = amplitude;
  a.heads = heads; a.kv_heads = kv_heads; a.dim = dim; a.vdim = vdim; a.rot_dim = rot_dim;
  a.cache = pwa_cache(k_pages, v_pages, block_table, table_stride, page_size, page_stride, num_pages);
  a.error_word = error_word;
  const int total = heads + 2 * kv_heads;
  const int threads = 32 * (total < 4 ? 4 : total > 16 ? 16 : total);
  if (dtype == TIB_F32)
    TIB_LAUNCH_DEPENDENT(pwa_append_kernel<float>, n_tokens, threads, 0, stream, (const float*)proj, (float*)q_out, a);
  else if (dtype == TIB_BF16)
    TIB_LAUNCH_DEPENDENT(pwa_append_kernel<__nv_bfloat16>, n_tokens, threads, 0, stream, (const __nv_bfloat16*)proj,
                         (__nv_bfloat16*)q_out, a);
  else
    return TIB_E_DTYPE;
  return TIB_OK;
}

// The means of the blocks of `pool` positions that the step's tokens complete, from the token pages (k_pages, v_pages,
// block_table ...) into the strided pages (bk_pages, bv_pages, b_table ...), whose entry b stands for block b.
TIB_API int tib_pool_blocks(const void* k_pages, const void* v_pages, const int* block_table, int table_stride, int page_size,
                            int64_t page_stride, int num_pages, void* bk_pages, void* bv_pages, const int* b_table,
                            int b_table_stride, int b_page_size, int64_t b_page_stride, int b_num_pages, const int* positions,
                            const int* token_slot, int n_tokens, int kv_heads, int dim, int vdim, int pool, int* error_word,
                            int dtype, cudaStream_t stream) {
  if (n_tokens == 0) return TIB_OK;
  if (!k_pages || !v_pages || !block_table || !bk_pages || !bv_pages || !b_table || !positions || !token_slot) return TIB_E_ARG;
  if (kv_heads < 1 || kv_heads > 65535 || dim < 1 || vdim < 1 || pool < 1 || page_size < 1 || b_page_size < 1) return TIB_E_SIZE;
  PwaPoolArgs a;
  a.positions = positions; a.token_slot = token_slot; a.kv_heads = kv_heads; a.dim = dim; a.vdim = vdim; a.pool = pool;
  a.tokens = pwa_cache(const_cast<void*>(k_pages), const_cast<void*>(v_pages), block_table, table_stride, page_size, page_stride, num_pages);
  a.blocks = pwa_cache(bk_pages, bv_pages, b_table, b_table_stride, b_page_size, b_page_stride, b_num_pages);
  a.error_word = error_word;
  const dim3 grid(n_tokens, kv_heads);
  if (dtype == TIB_F32) TIB_LAUNCH_DEPENDENT(pwa_pool_kernel<float>, grid, kPoolLanes * kPoolTile, 0, stream, a);
  else if (dtype == TIB_BF16) TIB_LAUNCH_DEPENDENT(pwa_pool_kernel<__nv_bfloat16>, grid, kPoolLanes * kPoolTile, 0, stream, a);
  else return TIB_E_DTYPE;
  return TIB_OK;
}

// q: [n_tokens, heads * dim]; out: [n_tokens, heads * vdim]; gate: [n_tokens, heads * vdim] logits (row stride ld_gate, its
// own dtype) or null; temp, sink: [heads] fp32 or null; vfreq: [vdim / 2] fp32 or null.  pool 0: the window alone.
// rel_bias: [heads, rel_span] fp32 or null: rel_bias[h, min(i - j, rel_span - 1)] is added to the score of token j (not
// multiplied by scale or temp; blocks get none).  n_splits > 1 (a step of single tokens only, bf16 on the tensor cores, no
// turned values and no gate): every context is shared out over n_splits blocks, whose sums go through `partial`
// [n_splits, n_tokens, heads, part floats] to a second kernel; n_tokens: rows of q.
// force_simt: the CUDA-core kernel also where the tensor-core kernel would take the step.
TIB_API int tib_pooled_window_attention(const void* q, void* out, const int* q_start, const int* kv_start, const int* slots,
                                        const void* k_pages, const void* v_pages, const int* block_table, int table_stride,
                                        int page_size, int64_t page_stride, int num_pages, const void* bk_pages,
                                        const void* bv_pages, const int* b_table, int b_table_stride, int b_page_size,
                                        int64_t b_page_stride, int b_num_pages, int n_entries, int max_q_len, int heads,
                                        int kv_heads, int dim, int vdim, int window, int pool, float scale, const float* temp,
                                        const float* sink, const float* vfreq, const void* gate, int gate_dtype, int64_t ld_gate,
                                        const float* rel_bias, int rel_span, float* partial, int n_splits, int n_tokens,
                                        int* error_word, int dtype, int force_simt, cudaStream_t stream) {
  if (n_entries == 0 || max_q_len == 0) return TIB_OK;
  if (!q || !out || !q_start || !kv_start || !slots || !k_pages || !v_pages || !block_table) return TIB_E_ARG;
  if (pool > 0 && (!bk_pages || !bv_pages || !b_table || b_page_size < 1)) return TIB_E_ARG;
  if (heads < 1 || kv_heads < 1 || heads % kv_heads || dim < 1 || vdim < 1 || page_size < 1 || window < 1 || pool < 0) return TIB_E_SIZE;
  if (dim > 256 || vdim > 256 || (vfreq && vdim % 2) || n_entries > 65535) return TIB_E_SIZE;
  if (gate && gate_dtype != TIB_F32 && gate_dtype != TIB_BF16) return TIB_E_DTYPE;
  if (rel_bias && rel_span < 1) return TIB_E_SIZE;
  PwaArgs a;
  a.q_start = q_start; a.kv_start = kv_start; a.slots = slots; a.heads = heads; a.kv_heads = kv_heads; a.dim = dim; a.vdim = vdim;
  a.window = window; a.pool = pool; a.scale = scale; a.temp = temp; a.sink = sink; a.vfreq = vfreq; a.gate = gate;
  a.gate_dtype = gate_dtype; a.ld_gate = ld_gate; a.rel_bias = rel_bias; a.rel_span = rel_span;
  a.tokens = pwa_cache(const_cast<void*>(k_pages), const_cast<void*>(v_pages), block_table, table_stride, page_size, page_stride, num_pages);
  a.blocks = pwa_cache(const_cast<void*>(bk_pages), const_cast<void*>(bv_pages), b_table, b_table_stride, b_page_size, b_page_stride, b_num_pages);
  a.error_word = error_word;
  a.partial = partial; a.n_splits = n_splits > 1 ? n_splits : 1; a.n_tokens = n_tokens;
  const int group = heads / kv_heads;
  a.group_chunk = group < kPwaRows ? group : kPwaRows;
  a.q_tile = kPwaRows / a.group_chunk;
  const int chunks = (group + a.group_chunk - 1) / a.group_chunk;
  if ((int64_t)kv_heads * chunks > 65535) return TIB_E_SIZE;
  // bf16 steps run on the tensor cores, single tokens too (their tiles come in by cp.async, 16 bytes a piece, where the
  // other kernel waits for one element at a time); 32-bit and head sizes that are no multiples of 8 run on the CUDA cores.
  if (dtype == TIB_BF16 && !force_simt && pwa_mma_takes(a, q)) {
    if (dim <= 64 && vdim <= 64) return pwa_launch_mma<64, 64>(q, out, a, n_entries, max_q_len, stream);
    if (dim <= 64) return pwa_launch_mma<64, 128>(q, out, a, n_entries, max_q_len, stream);
    if (vdim <= 64) return pwa_launch_mma<128, 64>(q, out, a, n_entries, max_q_len, stream);
    return pwa_launch_mma<128, 128>(q, out, a, n_entries, max_q_len, stream);
  }
  const int dpl = (vdim + 31) / 32;
#define TIB_PWA_DISPATCH(T)                                                              \
  (dpl <= 1 ? pwa_launch<T, 1>(q, out, a, n_entries, max_q_len, stream)                  \
   : dpl <= 2 ? pwa_launch<T, 2>(q, out, a, n_entries, max_q_len, stream)                \
   : dpl <= 4 ? pwa_launch<T, 4>(q, out, a, n_entries, max_q_len, stream)                \
              : pwa_launch<T, 8>(q, out, a, n_entries, max_q_len, stream))
  if (dtype == TIB_F32) return TIB_PWA_DISPATCH(float);
  if (dtype == TIB_BF16) return TIB_PWA_DISPATCH(__nv_bfloat16);
#undef TIB_PWA_DISPATCH
  return TIB_E_DTYPE;
}
