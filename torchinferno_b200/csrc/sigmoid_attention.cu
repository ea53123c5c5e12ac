// Attention whose weights are not a softmax: every visible key gets the weight sigmoid(score + bias of the head),
// nothing is normalised over the keys, and a head's output is multiplied by a gate of its own.
//
//   score(i, j) = (q_i . k_j) * scale                       q, k rotated and then divided by their root mean square
//   visible     = j <= i, and (chunk > 0) floor(i / chunk) == floor(j / chunk), and (window > 0) i - j < window
//   o_i         = sigmoid(gate_i) * sum over visible j of sigmoid(score(i, j) + bias) * v_j
//
// Positions count from the start of the sequence, so a chunk's edges do not move with the way a prompt was cut.
// Keys are `dim` wide and values `vdim`; a layer's pages hold [kv_heads][page_size][dim] keys and then
// [kv_heads][page_size][vdim] values.  Query head h reads kv head h / (heads / kv_heads).
//
//   qk_norm_append     rotary encoding of part of every q and k head (pairs (i, i + rot/2) or (2i, 2i + 1), angles
//                      fp32 position x fp32 frequency), then x / sqrt(mean(x^2) + eps) over the head (eps < 0: no
//                      norm), optionally times a weight per element and, for q, a temperature that grows with the
//                      logarithm of the position, all fp32; q goes to q_out, k and v (v untouched) into their page
//   sigmoid_attention  CUDA cores, every size: one warp owns a (token, head) row and walks the keys in blocks of 32
//                      aligned to absolute positions in rising order, so a row's sums are the same whatever the
//                      batch holds and however the prompt was cut.  The 32-bit path.
//   sigmoid_attention_mma   bf16 on the tensor cores (mma.sync m16n8k16): 64 query rows of one head against 64
//                      keys a step; scores, sigmoid and mask in fp32 registers; the weights enter the second
//                      product as two bf16 terms (high part and remainder), so that they keep 16 bits
#include "mma.cuh"
#include <math_constants.h>

namespace tib {

__device__ __forceinline__ float sig_f(float z) { return 1.f / (1.f + expf(-z)); }

// ------------------------------------------------------------------ append
struct QkAppendArgs {
  int64_t ld;                 // elements between rows of the projection
  int q_off, k_off, v_off;    // columns where q, k, v start in a row (k_off < 0: the row has no k and v)
  int heads, kv_heads, dim, vdim, rot_dim, interleaved;
  float eps;
  const int* positions; const int* token_slot; const int* block_table; int table_stride;
  const float* inv_freq;
  int page_size; int64_t page_stride; int num_pages;
  int* error_word;
  const float* q_weight; const float* k_weight;     // [dim] each or null: multiply the normed head (one weight for all heads)
  float temp_coef; int temp_every;                  // temp_every > 0: q times 1 + temp_coef * ln(floor((pos + 1) / temp_every) + 1)
};

template <typename T>
__global__ void __launch_bounds__(512)
qk_norm_append_kernel(const T* __restrict__ proj, T* __restrict__ q_out, T* __restrict__ k_pages, T* __restrict__ v_pages,
                      QkAppendArgs a) {
  pdl_wait();
  pdl_trigger();
  extern __shared__ float sm[];          // cos[rot/2], sin[rot/2], then one head of floats per warp
  const int tok = blockIdx.x;
  const int pos = a.positions[tok];
  const int half = a.rot_dim >> 1;
  float* cs = sm;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    float sn, cn;
    sincosf((float)pos * a.inv_freq[i], &sn, &cn);
    cs[i] = cn;
    cs[half + i] = sn;
  }
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  float* head = sm + 2 * half + warp * a.dim;
  const T* row = proj + (size_t)tok * a.ld;
  const bool write = a.k_off >= 0;
  int page = -1, off = 0;
  if (write) {
    page = a.block_table[(size_t)a.token_slot[tok] * a.table_stride + pos / a.page_size];
    off = pos % a.page_size;
    if (page < 0 || page >= a.num_pages) {
      if (a.error_word && threadIdx.x == 0) atomicExch(a.error_word, 1 + tok);
      page = -1;
    }
  }
  const int rot_heads = a.heads + (write ? a.kv_heads : 0);
  for (int hh = warp; hh < rot_heads; hh += nwarps) {
    const bool is_q = hh < a.heads;
    const int h = is_q ? hh : hh - a.heads;
    const T* src = row + (is_q ? a.q_off : a.k_off) + h * a.dim;
    for (int d = lane; d < a.dim; d += 32) head[d] = to_f32(src[d]);
    __syncwarp();
    // rotate: lane i takes pair i
    for (int i = lane; i < half; i += 32) {
      const int lo_i = a.interleaved ? 2 * i : i, hi_i = a.interleaved ? 2 * i + 1 : i + half;
      const float lo = head[lo_i], hi = head[hi_i];
      head[lo_i] = rope_lo(lo, hi, cs[i], cs[half + i]);
      head[hi_i] = rope_hi(lo, hi, cs[i], cs[half + i]);
    }
    __syncwarp();
    float inv = 1.f;
    if (a.eps >= 0.f) {
      float ss = 0.f;
      for (int d = lane; d < a.dim; d += 32) ss = fmaf(head[d], head[d], ss);
      inv = 1.f / sqrtf(warp_sum(ss) / (float)a.dim + a.eps);
    }
    T* dst = nullptr;
    if (is_q) dst = q_out + (size_t)tok * a.heads * a.dim + h * a.dim;
    else if (page >= 0) dst = k_pages + (size_t)page * a.page_stride + ((size_t)h * a.page_size + off) * a.dim;
    const float* weight = is_q ? a.q_weight : a.k_weight;
    // the query's temperature grows with the logarithm of its position, in steps of temp_every positions
    const float temp = (is_q && a.temp_every > 0) ? 1.f + a.temp_coef * logf((float)((pos + 1) / a.temp_every) + 1.f) : 1.f;
    if (dst) {
      if (weight) for (int d = lane; d < a.dim; d += 32) dst[d] = from_f32<T>(head[d] * inv * weight[d] * temp);
      else for (int d = lane; d < a.dim; d += 32) dst[d] = from_f32<T>(head[d] * inv * temp);
    }
    __syncwarp();
  }
  if (write && page >= 0) {
    const T* vsrc = row + a.v_off;
    T* vdst = v_pages + (size_t)page * a.page_stride;
    for (int w = threadIdx.x; w < a.kv_heads * a.vdim; w += blockDim.x) {
      const int h = w / a.vdim, d = w - h * a.vdim;
      vdst[((size_t)h * a.page_size + off) * a.vdim + d] = vsrc[w];
    }
  }
}

// --------------------------------------------------------------- attention
struct SigAttnArgs {
  const int* q_start;      // [n_entries + 1]
  const int* kv_start;     // [n_entries] position of the entry's first query token
  const int* slots;        // [n_entries]
  const int* block_table; int table_stride;
  int heads, kv_heads, dim, vdim;
  int page_size; int64_t page_stride; int num_pages;
  int chunk, window;       // 0: none
  float scale;
  const float* head_bias;  // [heads] or null
  const void* gate; int gate_dtype; int64_t ld_gate;    // gate logits [tokens, heads] (row stride ld_gate) or null
  int* error_word;
};

__device__ __forceinline__ int first_visible(int qpos, int chunk, int window) {
  int lo = 0;
  if (chunk > 0) lo = (qpos / chunk) * chunk;
  if (window > 0) lo = max(lo, qpos - window + 1);
  return lo;
}

constexpr int kSaWarps = 4, kSaRowsPerWarp = 4, kSaRows = kSaWarps * kSaRowsPerWarp, kSaKeys = 32;

template <typename T, int VPL>
__global__ void __launch_bounds__(kSaWarps * 32)
sigmoid_attention_simt_kernel(const T* __restrict__ q, const T* __restrict__ k_pages, const T* __restrict__ v_pages,
                              T* __restrict__ out, SigAttnArgs a, int group_chunk, int q_tile) {
  pdl_wait();
  pdl_trigger();
  extern __shared__ float smem[];
  const int d = a.dim, vd = a.vdim;
  float* q_s = smem;                          // [kSaRows][d]
  float* k_s = q_s + kSaRows * d;             // [32][d + 1]
  float* v_s = k_s + kSaKeys * (d + 1);       // [32][vd]

  const int entry = blockIdx.y;
  const int group = a.heads / a.kv_heads;
  const int chunks = (group + group_chunk - 1) / group_chunk;
  const int kvh = blockIdx.z / chunks;
  const int g0 = (blockIdx.z - kvh * chunks) * group_chunk;
  const int gc = min(group_chunk, group - g0);
  const int row0 = a.q_start[entry];
  const int q_len = a.q_start[entry + 1] - row0;
  const int t0 = blockIdx.x * q_tile;
  if (t0 >= q_len) return;
  const int nt = min(q_tile, q_len - t0);
  const int nrows = nt * gc;
  const int pos0 = a.kv_start[entry] + t0;
  const int last_pos = pos0 + nt - 1;
  const int* table = a.block_table + (size_t)a.slots[entry] * a.table_stride;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int q_width = a.heads * d;

  for (int e = threadIdx.x; e < nrows * d; e += blockDim.x) {
    const int r = e / d, dd = e - r * d;
    const int t = r / gc, g = r - t * gc;
    q_s[r * d + dd] = to_f32(q[(size_t)(row0 + t0 + t) * q_width + (kvh * group + g0 + g) * d + dd]);
  }
  float acc[kSaRowsPerWarp][VPL];
#pragma unroll
  for (int i = 0; i < kSaRowsPerWarp; ++i)
#pragma unroll
    for (int j = 0; j < VPL; ++j) acc[i][j] = 0.f;

  const int first_key = first_visible(pos0, a.chunk, a.window);      // (the lowest of the tile: positions rise)
  const int b_lo = first_key / kSaKeys, b_hi = last_pos / kSaKeys;
  for (int b = b_lo; b <= b_hi; ++b) {
    __syncthreads();
    for (int j = warp; j < kSaKeys; j += kSaWarps) {
      const int kp = b * kSaKeys + j;
      int page = -1;
      if (kp <= last_pos && kp >= first_key) {
        page = table[kp / a.page_size];
        if (page < 0 || page >= a.num_pages) {
          if (a.error_word && lane == 0) atomicExch(a.error_word, 0x10000 + entry);
          page = -1;
        }
      }
      const size_t at = (size_t)kvh * a.page_size + (kp % a.page_size);
      const T* kr = k_pages + (size_t)max(page, 0) * a.page_stride + at * d;
      const T* vr = v_pages + (size_t)max(page, 0) * a.page_stride + at * vd;
      for (int dd = lane; dd < d; dd += 32) k_s[j * (d + 1) + dd] = page >= 0 ? to_f32(kr[dd]) : 0.f;
      for (int dd = lane; dd < vd; dd += 32) v_s[j * vd + dd] = page >= 0 ? to_f32(vr[dd]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < kSaRowsPerWarp; ++i) {
      const int r = warp * kSaRowsPerWarp + i;
      if (r >= nrows) continue;
      const int t = r / gc, g = r - t * gc;
      const int qpos = pos0 + t;
      const int lo = first_visible(qpos, a.chunk, a.window);
      if (b * kSaKeys > qpos || b * kSaKeys + kSaKeys - 1 < lo) continue;
      const int kp = b * kSaKeys + lane;
      const bool allowed = kp <= qpos && kp >= lo;
      float s = 0.f;
      const float* qr = q_s + r * d;
      const float* kr = k_s + lane * (d + 1);
      for (int dd = 0; dd < d; ++dd) s = fmaf(qr[dd], kr[dd], s);
      const float bias = a.head_bias ? a.head_bias[kvh * group + g0 + g] : 0.f;
      const float p = allowed ? sig_f(s * a.scale + bias) : 0.f;
      for (int kk = 0; kk < kSaKeys; ++kk) {
        const float pk = __shfl_sync(0xffffffffu, p, kk);
#pragma unroll
        for (int j = 0; j < VPL; ++j) {
          const int dd = lane + 32 * j;
          if (dd < vd) acc[i][j] = fmaf(pk, v_s[kk * vd + dd], acc[i][j]);
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < kSaRowsPerWarp; ++i) {
    const int r = warp * kSaRowsPerWarp + i;
    if (r >= nrows) continue;
    const int t = r / gc, g = r - t * gc;
    const int head = kvh * group + g0 + g;
    const size_t tok = (size_t)(row0 + t0 + t);
    float gate = 1.f;
    if (a.gate) {
      const float z = a.gate_dtype == TIB_F32 ? reinterpret_cast<const float*>(a.gate)[tok * a.ld_gate + head]
                                              : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(a.gate)[tok * a.ld_gate + head]);
      gate = sig_f(z);
    }
    T* dst = out + tok * a.heads * vd + (size_t)head * vd;
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
      const int dd = lane + 32 * j;
      if (dd < vd) dst[dd] = from_f32<T>(acc[i][j] * gate);
    }
  }
}

template <typename T, int VPL>
static int launch_sigmoid_simt(const void* q, const void* k_pages, const void* v_pages, void* out, const SigAttnArgs& a,
                               int n_entries, int max_q_len, cudaStream_t stream) {
  const size_t smem = sizeof(float) * ((size_t)kSaRows * a.dim + (size_t)kSaKeys * (a.dim + 1) + (size_t)kSaKeys * a.vdim);
  if (smem > 227 * 1024) return TIB_E_SMEM;
  auto kern = sigmoid_attention_simt_kernel<T, VPL>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  const int group = a.heads / a.kv_heads;
  const int group_chunk = group < kSaRows ? group : kSaRows;
  const int q_tile = kSaRows / group_chunk;
  const int chunks = (group + group_chunk - 1) / group_chunk;
  if ((int64_t)a.kv_heads * chunks > 65535) return TIB_E_SIZE;
  dim3 grid(ceil_div(max_q_len, q_tile), n_entries, a.kv_heads * chunks);
  TIB_LAUNCH_DEPENDENT(kern, grid, kSaWarps * 32, smem, stream, (const T*)q, (const T*)k_pages, (const T*)v_pages, (T*)out, a,
                       group_chunk, q_tile);
  return TIB_OK;
}


// ------------------------------------------------------------ tensor cores
// 64 rows (tokens x the query heads of one kv head) against tiles of 64 keys that are aligned to absolute positions,
// four warps of 16 rows.  Keys and values of a tile come in by cp.async, row by row from their pages, two stages.
// A row's sum runs over the tiles in rising order and every key has a fixed place in its tile, so the result
// does not depend on how the prompt was cut or on what else the step holds.  Rows of values past the last position
// of the tile are zero-filled (unwritten cache may hold anything); so are the padding columns up to DK / DV.
constexpr int kSmRows = 64, kSmKeys = 64, kSmThreads = 128;

// BYKEYS: every block of the launch has at most 16 rows (single tokens, short portions).  The four warps then share a
// tile's keys, 16 each, instead of its rows, and their sums meet in shared memory at the end, in warp order.
template <int DK, int DV, bool BYKEYS>
__global__ void __launch_bounds__(kSmThreads)
sigmoid_attention_mma_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_pages,
                             const __nv_bfloat16* __restrict__ v_pages, __nv_bfloat16* __restrict__ out, SigAttnArgs a,
                             int group_chunk, int q_tile, int splits, float* __restrict__ partial) {
  // splits > 0: a step of single tokens.  blockIdx.x is then a share of the key tiles instead of a query tile, and the
  // sums of that share leave ungated in fp32, partial[split][token][head][vdim], for sigmoid_attention_sum_kernel.
  pdl_wait();
  pdl_trigger();
  constexpr int KP = DK + 8, VP = DV + 8;        // padded rows: ldmatrix rows fall in different banks
  extern __shared__ __align__(16) unsigned char sm_raw[];
  __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(sm_raw);          // [64][KP]
  __nv_bfloat16* k_s = q_s + kSmRows * KP;                                 // [2][64][KP]
  __nv_bfloat16* v_s = k_s + 2 * kSmKeys * KP;                             // [2][64][VP]
  __shared__ long long page_base[2][kSmKeys];
  __shared__ int key_row[2][kSmKeys];

  const int d = a.dim, vd = a.vdim;
  const int entry = blockIdx.y;
  const int group = a.heads / a.kv_heads;
  const int chunks = (group + group_chunk - 1) / group_chunk;
  const int kvh = blockIdx.z / chunks;
  const int g0 = (blockIdx.z - kvh * chunks) * group_chunk;
  const int gc = min(group_chunk, group - g0);
  const int row0 = a.q_start[entry];
  const int q_len = a.q_start[entry + 1] - row0;
  const int t0 = splits > 0 ? 0 : blockIdx.x * q_tile;
  if (t0 >= q_len) return;
  const int nt = min(q_tile, q_len - t0);
  const int nrows = nt * gc;
  const int pos0 = a.kv_start[entry] + t0;
  const int last_pos = pos0 + nt - 1;
  const int* table = a.block_table + (size_t)a.slots[entry] * a.table_stride;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int first_key = first_visible(pos0, a.chunk, a.window);
  int b_lo = first_key / kSmKeys, b_hi = last_pos / kSmKeys;
  if (splits > 0) {
    const int per = (b_hi - b_lo + splits) / splits;       // tiles a share, rounded up
    b_lo += (int)blockIdx.x * per;
    b_hi = min(b_hi, b_lo + per - 1);                      // (an empty share writes zeros)
  }

  auto fetch = [&](int stage, int b) {
    // where every key of the tile lives, once: its page's first element and its row in the page
    if (tid < kSmKeys) {
      const int kp = b * kSmKeys + tid;
      long long base = -1;
      int row = 0;
      if (kp <= last_pos && kp >= first_key) {
        const int logical = kp / a.page_size;
        const int page = table[logical];
        if (page < 0 || page >= a.num_pages) {
          if (a.error_word) atomicExch(a.error_word, 0x10000 + entry);
        } else {
          base = (long long)page * a.page_stride;
          row = kvh * a.page_size + (kp - logical * a.page_size);
        }
      }
      page_base[stage][tid] = base;
      key_row[stage][tid] = row;
    }
    __syncthreads();
    constexpr int KPIECES = DK / 8, VPIECES = DV / 8;
    for (int e = tid; e < kSmKeys * KPIECES; e += kSmThreads) {
      const int j = e / KPIECES, c = (e - j * KPIECES) * 8;
      const long long base = page_base[stage][j];
      const bool ok = base >= 0 && c < d;
      cp_async16(k_s + ((size_t)stage * kSmKeys + j) * KP + c, k_pages + (ok ? base + (long long)key_row[stage][j] * d + c : 0), ok);
    }
    for (int e = tid; e < kSmKeys * VPIECES; e += kSmThreads) {
      const int j = e / VPIECES, c = (e - j * VPIECES) * 8;
      const long long base = page_base[stage][j];
      const bool ok = base >= 0 && c < vd;
      cp_async16(v_s + ((size_t)stage * kSmKeys + j) * VP + c, v_pages + (ok ? base + (long long)key_row[stage][j] * vd + c : 0), ok);
    }
    cp_async_commit();
  };

  // queries: 16-byte pieces, rows past the tile's end and padding columns are zero
  {
    constexpr int QPIECES = DK / 8;
    for (int e = tid; e < kSmRows * QPIECES; e += kSmThreads) {
      const int r = e / QPIECES, c = (e - r * QPIECES) * 8;
      const bool ok = r < nrows && c < d;
      const int t = ok ? r / gc : 0, g = ok ? r - t * gc : 0;
      const __nv_bfloat16* src = q + (size_t)(row0 + t0 + t) * a.heads * d + (size_t)(kvh * group + g0 + g) * d + (ok ? c : 0);
      cp_async16(q_s + (size_t)r * KP + c, src, ok);
    }
  }
  if (b_lo <= b_hi) fetch(0, b_lo);

  // this thread's two rows: g8 and g8 + 8 of the warp's sixteen
  const int g8 = lane >> 2, t4 = lane & 3;
  int qpos[2], lo[2];
  float bias[2];
  bool live[2];
  constexpr int NT = BYKEYS ? 2 : kSmKeys / 8;      // tiles of 8 keys a warp takes of a tile of 64
  const int row_base = BYKEYS ? 0 : warp * 16, key_base = BYKEYS ? warp * 16 : 0;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = row_base + g8 + 8 * h;
    live[h] = r < nrows;
    const int t = live[h] ? r / gc : 0, g = live[h] ? r - t * gc : 0;
    qpos[h] = pos0 + t;
    lo[h] = first_visible(qpos[h], a.chunk, a.window);
    bias[h] = a.head_bias ? a.head_bias[kvh * group + g0 + g] : 0.f;
  }
  float o[DV / 8][4];
#pragma unroll
  for (int n = 0; n < DV / 8; ++n)
#pragma unroll
    for (int c = 0; c < 4; ++c) o[n][c] = 0.f;

  for (int b = b_lo; b <= b_hi; ++b) {
    const int stage = (b - b_lo) & 1;
    if (b < b_hi) {
      fetch(stage ^ 1, b + 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    // (a warp whose rows see nothing of this tile still passes the barriers)
    const int warp_first = pos0 + row_base / gc, warp_last = pos0 + min(nrows - 1, row_base + 15) / gc;
    const bool any = row_base < nrows && b * kSmKeys + key_base <= warp_last &&
                     b * kSmKeys + key_base + NT * 8 - 1 >= first_visible(warp_first, a.chunk, a.window);
    if (any) {
      const __nv_bfloat16* kt = k_s + (size_t)stage * kSmKeys * KP;
      const __nv_bfloat16* vt = v_s + (size_t)stage * kSmKeys * VP;
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
          ldmatrix_x4(bf, kt + (size_t)(key_base + j * 16 + ((lane >> 4) << 3) + (lane & 7)) * KP + kk + ((lane >> 3) & 1) * 8);
          mma_bf16(s[2 * j], af, bf[0], bf[1]);
          mma_bf16(s[2 * j + 1], af, bf[2], bf[3]);
        }
      }
      // weights in fp32; into the second product as a high bf16 part and the remainder
      uint32_t p_hi[NT / 2][4], p_lo[NT / 2][4];
#pragma unroll
      for (int n = 0; n < NT; ++n) {
        float w[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int h = c >> 1;
          const int kp = b * kSmKeys + key_base + n * 8 + 2 * t4 + (c & 1);
          const bool allowed = live[h] && kp <= qpos[h] && kp >= lo[h];
          w[c] = allowed ? __fdividef(1.f, 1.f + __expf(-(s[n][c] * a.scale + bias[h]))) : 0.f;
        }
        const int kk = n >> 1, half = (n & 1) * 2;
        const __nv_bfloat162 h01 = __floats2bfloat162_rn(w[0], w[1]), h23 = __floats2bfloat162_rn(w[2], w[3]);
        p_hi[kk][half] = *reinterpret_cast<const uint32_t*>(&h01);
        p_hi[kk][half + 1] = *reinterpret_cast<const uint32_t*>(&h23);
        const float2 f01 = bf16x2_floats(h01), f23 = bf16x2_floats(h23);
        p_lo[kk][half] = pack_bf16(w[0] - f01.x, w[1] - f01.y);
        p_lo[kk][half + 1] = pack_bf16(w[2] - f23.x, w[3] - f23.y);
      }
#pragma unroll
      for (int kk = 0; kk < NT / 2; ++kk) {
        // (the two terms of the weights go in two passes, so that products into one accumulator are not back to back)
        uint32_t bv[DV / 16][4];
#pragma unroll
        for (int dn = 0; dn < DV / 16; ++dn) {
          ldmatrix_x4_trans(bv[dn], vt + (size_t)(key_base + kk * 16 + (lane & 15)) * VP + dn * 16 + ((lane >> 4) << 3));
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
    __syncthreads();      // the stage is free for the fetch after next
  }
  if (b_lo > b_hi) {      // (an empty share: the queries' copies are still in flight)
    cp_async_commit();
    cp_async_wait<0>();
  }
  if (BYKEYS) {
    // the four warps' sums over their keys, added in warp order (the stages are free: every loop ends in a barrier)
    float* red = reinterpret_cast<float*>(k_s);         // [4][16][DV] floats over the key and value stages, which adjoin
    __syncthreads();
#pragma unroll
    for (int n = 0; n < DV / 8; ++n)
#pragma unroll
      for (int c = 0; c < 4; ++c)
        red[((size_t)warp * 16 + g8 + 8 * (c >> 1)) * DV + n * 8 + 2 * t4 + (c & 1)] = o[n][c];
    __syncthreads();
#pragma unroll
    for (int n = 0; n < DV / 8; ++n)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const size_t at = ((size_t)g8 + 8 * (c >> 1)) * DV + n * 8 + 2 * t4 + (c & 1);
        o[n][c] = ((red[at] + red[16 * DV + at]) + red[32 * DV + at]) + red[48 * DV + at];
      }
    if (warp != 0) return;      // (warp 0 writes the rows)
  }

#pragma unroll
  for (int h = 0; h < 2; ++h) {
    if (!live[h]) continue;
    const int r = row_base + g8 + 8 * h;
    const int t = r / gc, g = r - t * gc;
    const int head = kvh * group + g0 + g;
    const size_t tok = (size_t)(row0 + t0 + t);
    if (splits > 0) {
      float* dst = partial + (((size_t)blockIdx.x * a.q_start[gridDim.y] + tok) * a.heads + head) * vd;
#pragma unroll
      for (int n = 0; n < DV / 8; ++n) {
        const int col = n * 8 + 2 * t4;
        if (col < vd) dst[col] = o[n][2 * h];
        if (col + 1 < vd) dst[col + 1] = o[n][2 * h + 1];
      }
      continue;
    }
    float gate = 1.f;
    if (a.gate) {
      const float z = a.gate_dtype == TIB_F32 ? reinterpret_cast<const float*>(a.gate)[tok * a.ld_gate + head]
                                              : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(a.gate)[tok * a.ld_gate + head]);
      gate = sig_f(z);
    }
    __nv_bfloat16* dst = out + tok * a.heads * vd + (size_t)head * vd;
#pragma unroll
    for (int n = 0; n < DV / 8; ++n) {
      const int col = n * 8 + 2 * t4;
      if (col + 1 < vd)
        *reinterpret_cast<__nv_bfloat162*>(dst + col) = __floats2bfloat162_rn(o[n][2 * h] * gate, o[n][2 * h + 1] * gate);
      else if (col < vd)
        dst[col] = __float2bfloat16_rn(o[n][2 * h] * gate);
    }
  }
}

// out[tok][head] = sigmoid(gate[tok][head]) * sum over the shares, in rising order, of partial[share][tok][head]
__global__ void sigmoid_attention_sum_kernel(const float* __restrict__ partial, __nv_bfloat16* __restrict__ out, SigAttnArgs a,
                                             int splits, int n_tokens) {
  pdl_wait();
  pdl_trigger();
  const size_t tok = blockIdx.x;
  const int width = a.heads * a.vdim;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < width; c += gridDim.y * blockDim.x) {
    const int head = c / a.vdim;
    float v = 0.f;
#pragma unroll 4
    for (int s = 0; s < splits; ++s) v += partial[((size_t)s * n_tokens + tok) * width + c];
    if (a.gate) {
      const float z = a.gate_dtype == TIB_F32 ? reinterpret_cast<const float*>(a.gate)[tok * a.ld_gate + head]
                                              : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(a.gate)[tok * a.ld_gate + head]);
      v *= sig_f(z);
    }
    out[tok * width + c] = __float2bfloat16_rn(v);
  }
}

template <int DK, int DV>
static int launch_sigmoid_mma(const void* q, const void* k_pages, const void* v_pages, void* out, const SigAttnArgs& a,
                              int n_entries, int max_q_len, int splits, float* partial, cudaStream_t stream) {
  static_assert(4 * 16 * DV * sizeof(float) <= 2 * kSmKeys * (DK + 8 + DV + 8) * sizeof(__nv_bfloat16), "the warps' sums fit the stages");
  const size_t smem = sizeof(__nv_bfloat16) * ((size_t)kSmRows * (DK + 8) + 2 * (size_t)kSmKeys * (DK + 8) + 2 * (size_t)kSmKeys * (DV + 8));
  const int group = a.heads / a.kv_heads;
  const int group_chunk = group < kSmRows ? group : kSmRows;
  const bool by_keys = (int64_t)max_q_len * group_chunk <= 16;      // no block has more than 16 rows
  auto kern = by_keys ? sigmoid_attention_mma_kernel<DK, DV, true> : sigmoid_attention_mma_kernel<DK, DV, false>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  const int q_tile = by_keys ? max_q_len : kSmRows / group_chunk;
  const int chunks = (group + group_chunk - 1) / group_chunk;
  if ((int64_t)a.kv_heads * chunks > 65535) return TIB_E_SIZE;
  dim3 grid(splits > 0 ? splits : ceil_div(max_q_len, q_tile), n_entries, a.kv_heads * chunks);
  TIB_LAUNCH_DEPENDENT(kern, grid, kSmThreads, smem, stream, (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_pages,
                       (const __nv_bfloat16*)v_pages, (__nv_bfloat16*)out, a, group_chunk, q_tile, splits, partial);
  if (splits > 0)      // (a step of single tokens: one token an entry)
    TIB_LAUNCH_DEPENDENT(sigmoid_attention_sum_kernel, dim3(n_entries, ceil_div(a.heads * a.vdim, 128)), 128, 0, stream,
                         (const float*)partial, (__nv_bfloat16*)out, a, splits, n_entries);
  return TIB_OK;
}

// Whether the tensor-core kernel takes these head sizes (bf16; rows of 16-byte pieces).
static bool sigmoid_mma_takes(int dim, int vdim, int64_t page_stride, const void* q, const void* k_pages, const void* v_pages) {
  return dim % 8 == 0 && vdim % 8 == 0 && dim <= 128 && vdim <= 128 && page_stride % 8 == 0 &&
         (((uintptr_t)q | (uintptr_t)k_pages | (uintptr_t)v_pages) & 15) == 0;
}

}  // namespace tib

using namespace tib;

// proj: [n_tokens, ld] rows holding q at q_off, k at k_off, v at v_off (k_off < 0: no k, v: nothing is stored);
// q_out: [n_tokens, heads * dim]; k_pages / v_pages: first key / value of this layer's first page.  q_weight / k_weight:
// [dim] fp32 or null, multiplied into every normed head; temp_every > 0: every q is also multiplied by
// 1 + temp_coef * ln(floor((position + 1) / temp_every) + 1).
TIB_API int tib_qk_norm_append(const void* proj, int64_t ld, int q_off, int k_off, int v_off, void* q_out, void* k_pages,
                               void* v_pages, const int* positions, const int* token_slot, const int* block_table,
                               int table_stride, const float* inv_freq, int n_tokens, int heads, int kv_heads, int dim,
                               int vdim, int rot_dim, int interleaved, float eps, int page_size, int64_t page_stride,
                               int num_pages, const float* q_weight, const float* k_weight, float temp_coef, int temp_every,
                               int* error_word, int dtype, cudaStream_t stream) {
  if (n_tokens == 0) return TIB_OK;
  if (!proj || !q_out || !positions || n_tokens < 0 || heads < 1 || dim < 1) return TIB_E_ARG;
  if (rot_dim < 0 || rot_dim % 2 || rot_dim > dim || (rot_dim > 0 && !inv_freq)) return TIB_E_SIZE;
  if (k_off >= 0 && (!k_pages || !token_slot || !block_table || kv_heads < 1 || page_size < 1 || (vdim > 0 && !v_pages)))
    return TIB_E_ARG;
  QkAppendArgs a;
  a.ld = ld; a.q_off = q_off; a.k_off = k_off; a.v_off = v_off; a.heads = heads; a.kv_heads = kv_heads; a.dim = dim;
  a.vdim = vdim; a.rot_dim = rot_dim; a.interleaved = interleaved; a.eps = eps; a.positions = positions;
  a.token_slot = token_slot; a.block_table = block_table; a.table_stride = table_stride; a.inv_freq = inv_freq;
  a.page_size = page_size; a.page_stride = page_stride; a.num_pages = num_pages; a.error_word = error_word;
  a.q_weight = q_weight; a.k_weight = k_weight; a.temp_coef = temp_coef; a.temp_every = temp_every;
  const int rot_heads = heads + (k_off >= 0 ? kv_heads : 0);
  const int threads = 32 * (rot_heads < 4 ? 4 : rot_heads > 16 ? 16 : rot_heads);      // a warp a head, up to sixteen
  const size_t smem = sizeof(float) * ((size_t)rot_dim + (size_t)(threads / 32) * dim);
  if (smem > 48 * 1024) return TIB_E_SIZE;
  if (dtype == TIB_F32)
    TIB_LAUNCH_DEPENDENT(qk_norm_append_kernel<float>, n_tokens, threads, smem, stream, (const float*)proj, (float*)q_out,
                         (float*)k_pages, (float*)v_pages, a);
  else if (dtype == TIB_BF16)
    TIB_LAUNCH_DEPENDENT(qk_norm_append_kernel<__nv_bfloat16>, n_tokens, threads, smem, stream, (const __nv_bfloat16*)proj,
                         (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages, a);
  else
    return TIB_E_DTYPE;
  return TIB_OK;
}

TIB_API int tib_sigmoid_attention_takes_mma(int dim, int vdim) { return dim % 8 == 0 && vdim % 8 == 0 && dim <= 128 && vdim <= 128; }

// q: [n_tokens, heads * dim]; out: [n_tokens, heads * vdim]; gate: [n_tokens, >= heads] logits (row stride ld_gate)
// or null; head_bias: [heads] fp32 or null.  bf16 with head sizes that are multiples of 8 up to 128 runs on the tensor
// cores unless force_simt.  splits > 0 (only there, and only when every entry brings one token): the keys of a context are
// shared out over that many blocks, whose sums meet in partial [splits, n_entries, heads * vdim] fp32.

TIB_API int tib_sigmoid_attention(const void* q, const void* k_pages, const void* v_pages, void* out, const int* q_start,
                                  const int* kv_start, const int* slots, const int* block_table, int table_stride,
                                  int n_entries, int max_q_len, int heads, int kv_heads, int dim, int vdim, int page_size,
                                  int64_t page_stride, int num_pages, int chunk, int window, float scale,
                                  const float* head_bias, const void* gate, int gate_dtype, int64_t ld_gate, int* error_word,
                                  int dtype, int force_simt, int splits, float* partial, cudaStream_t stream) {
  if (n_entries == 0 || max_q_len == 0) return TIB_OK;
  if (!q || !k_pages || !v_pages || !out || !q_start || !kv_start || !slots || !block_table) return TIB_E_ARG;
  if (heads < 1 || kv_heads < 1 || heads % kv_heads || dim < 1 || vdim < 1 || page_size < 1 || chunk < 0 || window < 0)
    return TIB_E_SIZE;
  if (vdim > 256 || dim > 512 || n_entries > 65535) return TIB_E_SIZE;
  SigAttnArgs a;
  a.q_start = q_start; a.kv_start = kv_start; a.slots = slots; a.block_table = block_table; a.table_stride = table_stride;
  a.heads = heads; a.kv_heads = kv_heads; a.dim = dim; a.vdim = vdim; a.page_size = page_size; a.page_stride = page_stride;
  a.num_pages = num_pages; a.chunk = chunk; a.window = window; a.scale = scale; a.head_bias = head_bias; a.gate = gate;
  a.gate_dtype = gate_dtype; a.ld_gate = ld_gate; a.error_word = error_word;
  if (dtype == TIB_BF16 && !force_simt && sigmoid_mma_takes(dim, vdim, page_stride, q, k_pages, v_pages)) {
    if (splits > 0 && (max_q_len != 1 || !partial)) return TIB_E_ARG;
    if (dim <= 64 && vdim <= 64) return launch_sigmoid_mma<64, 64>(q, k_pages, v_pages, out, a, n_entries, max_q_len, splits, partial, stream);
    if (dim <= 64) return launch_sigmoid_mma<64, 128>(q, k_pages, v_pages, out, a, n_entries, max_q_len, splits, partial, stream);
    if (vdim <= 64) return launch_sigmoid_mma<128, 64>(q, k_pages, v_pages, out, a, n_entries, max_q_len, splits, partial, stream);
    return launch_sigmoid_mma<128, 128>(q, k_pages, v_pages, out, a, n_entries, max_q_len, splits, partial, stream);
  }
  const int vpl = (vdim + 31) / 32;
#define TIB_SA_DISPATCH(T)                                                                                   \
  (vpl <= 1 ? launch_sigmoid_simt<T, 1>(q, k_pages, v_pages, out, a, n_entries, max_q_len, stream)           \
   : vpl <= 2 ? launch_sigmoid_simt<T, 2>(q, k_pages, v_pages, out, a, n_entries, max_q_len, stream)         \
   : vpl <= 4 ? launch_sigmoid_simt<T, 4>(q, k_pages, v_pages, out, a, n_entries, max_q_len, stream)         \
              : launch_sigmoid_simt<T, 8>(q, k_pages, v_pages, out, a, n_entries, max_q_len, stream))
  if (dtype == TIB_F32) return TIB_SA_DISPATCH(float);
  if (dtype == TIB_BF16) return TIB_SA_DISPATCH(__nv_bfloat16);
#undef TIB_SA_DISPATCH
  return TIB_E_DTYPE;
}
