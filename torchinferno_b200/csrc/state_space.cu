// A state-space mixer of the Mamba-2 kind (state-space duality), after its input projection:
//
//   short_conv        u_t = silu(bias + sum_k w[:, k] * in_(t - taps + 1 + k))     per channel, causal; the last
//                     taps - 1 inputs of a request are carried in its state slot (zeros for a new request)
//   ssd_scan          per head h (its group g = h / (heads / groups)), S [N, P] in 32-bit, carried per request:
//                       dt_t = softplus(raw_t + dt_bias[h]);   a_t = exp(-exp(A_log[h]) * dt_t)
//                       S_t  = a_t * S_(t-1) + dt_t * B_t x_t^T;   y_t = S_t^T C_t + D[h] * x_t
//   gated_group_norm  out = (y * silu(z)) / rms over each of `parts` equal runs of the row * weight
//
// Step sizes, decays, the state, the sums over it, the gate and the norm are fp32 in both modes; the convolution
// accumulates in fp32 and leaves its rows in the activation type.  Every kernel takes the step's ragged batch
// through its device arrays (q_start, slots), so prompt portions and single tokens run in one launch and a decode
// step can be captured.
#include "common.cuh"

namespace tib {

__device__ __forceinline__ float ss_load(const void* p, int dtype, size_t i) {
  return dtype == TIB_F32 ? reinterpret_cast<const float*>(p)[i] : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
}
__device__ __forceinline__ void ss_store(void* p, int dtype, size_t i, float v) {
  if (dtype == TIB_F32) reinterpret_cast<float*>(p)[i] = v;
  else reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
}
__device__ __forceinline__ float ss_silu(float v) { return v / (1.f + expf(-v)); }
__device__ __forceinline__ float ss_softplus(float v) { return fmaxf(v, 0.f) + log1pf(expf(-fabsf(v))); }

// ------------------------------------------------------------------------------------------- short convolution
constexpr int kConvMaxTaps = 8;
constexpr int kConvSegment = 64;       // tokens one thread walks
constexpr int kConvChannels = 128;     // channels a block

struct ConvArgs {
  const void* in; int in_dtype; int64_t ld; int col;      // input rows: columns col .. col + channels - 1
  const float* weight; const float* bias;                  // [channels, taps], [channels] (null: none)
  float* state; int64_t state_stride; int64_t state_off;   // per slot: [taps - 1][channels] at state_off
  const int* q_start; const int* slots;
  void* out; int out_dtype;                                // [tokens, channels]
  int channels, taps, silu;
};

// grid (channel tiles, segments, entries).  The block of segment 0 alone touches the request's carried inputs: it
// reads them first and then leaves the new ones, so no other block's read can meet its write.
__global__ void __launch_bounds__(kConvChannels) short_conv_kernel(ConvArgs a) {
  pdl_wait();
  pdl_trigger();
  const int entry = blockIdx.z, seg = blockIdx.y;
  const int c = blockIdx.x * kConvChannels + threadIdx.x;
  const int row0 = a.q_start[entry], len = a.q_start[entry + 1] - row0;
  const int t0 = seg * kConvSegment;
  if (c >= a.channels || t0 >= len) return;
  const int taps = a.taps, carried = taps - 1;
  float* st = a.state + (size_t)a.slots[entry] * a.state_stride + a.state_off;
  float w[kConvMaxTaps], prev[kConvMaxTaps];      // prev[k]: the input taps - 1 - k tokens before the one at hand
#pragma unroll
  for (int k = 0; k < kConvMaxTaps; ++k) {
    w[k] = k < taps ? a.weight[(size_t)c * taps + k] : 0.f;
    prev[k] = 0.f;
  }
  const float b = a.bias ? a.bias[c] : 0.f;
  float old[kConvMaxTaps];
#pragma unroll
  for (int k = 0; k < kConvMaxTaps; ++k) old[k] = (seg == 0 && k < carried) ? st[(size_t)k * a.channels + c] : 0.f;
#pragma unroll
  for (int k = 0; k < kConvMaxTaps; ++k) {
    if (k >= carried) continue;
    const int r = t0 - carried + k;                 // row of the portion, or before it
    prev[k] = r >= 0 ? ss_load(a.in, a.in_dtype, (size_t)(row0 + r) * a.ld + a.col + c) : old[k];   // (r < 0 only in segment 0, where r = k - carried)
  }
  if (seg == 0) {                                   // what the next step finds: the last taps - 1 inputs
#pragma unroll
    for (int k = 0; k < kConvMaxTaps; ++k) {
      if (k >= carried) continue;
      const int r = len - carried + k;
      float v;
      if (r >= 0) v = ss_load(a.in, a.in_dtype, (size_t)(row0 + r) * a.ld + a.col + c);
      else {
        v = 0.f;
#pragma unroll
        for (int j = 0; j < kConvMaxTaps; ++j) if (j == k + len) v = old[j];
      }
      st[(size_t)k * a.channels + c] = v;
    }
  }
  const int t1 = min(len, t0 + kConvSegment);
  constexpr int AHEAD = 8;
  for (int t = t0; t < t1; t += AHEAD) {
    float x[AHEAD];
#pragma unroll
    for (int i = 0; i < AHEAD; ++i)
      x[i] = t + i < t1 ? ss_load(a.in, a.in_dtype, (size_t)(row0 + t + i) * a.ld + a.col + c) : 0.f;
#pragma unroll
    for (int i = 0; i < AHEAD; ++i) {
      if (t + i >= t1) break;
      float acc = b;
#pragma unroll
      for (int k = 0; k < kConvMaxTaps; ++k) {
        if (k >= carried) continue;
        acc = fmaf(w[k], prev[k], acc);
      }
#pragma unroll
      for (int k = 0; k < kConvMaxTaps; ++k) if (k == carried) acc = fmaf(w[k], x[i], acc);
#pragma unroll
      for (int k = 0; k + 1 < kConvMaxTaps; ++k) prev[k] = prev[k + 1];
#pragma unroll
      for (int k = 0; k < kConvMaxTaps; ++k) if (k == carried - 1) prev[k] = x[i];
      ss_store(a.out, a.out_dtype, (size_t)(row0 + t + i) * a.channels + c, a.silu ? ss_silu(acc) : acc);
    }
  }
}

// --------------------------------------------------------------------------------------------------- the scan
// A block of 128 threads owns 16 * CP columns of one head's state: 8 lanes share a group of CP columns along N (lane l holds
// the pairs n = 2 l, 2 l + 1, then 16 further on and so on, two values to a 64-bit register for fma.rn.f32x2), so a token's B and C are read once from shared memory for CP columns.  A step whose longest portion
// is at most one run walks every portion from its slot's state in one launch.  Longer portions are cut into runs of
// kScanRun tokens that are walked side by side: first every run from a zero state (its own sum L_r and the product of its
// decays A_r), then one thread per state element folds S_(r+1) = A_r S_r + L_r over the request's runs, leaving each run's
// starting state in the place of its sum and the last state in the slot, then every run again from its starting state,
// now with the outputs.  Cutting changes only the order of fp32 sums.
//
// Tokens are staged in shared memory a chunk at a time, in two stages: while the block walks token t of one chunk, its
// threads fetch row t of the next chunk into registers (as raw bits, so that nothing waits on the loads) and leave it in
// the other stage after the token's arithmetic.
constexpr int kScanLanesN = 8;         // lanes that share a column group along N
constexpr int kScanGroups = 16;        // column groups of a block
constexpr int kScanRun = 64;           // tokens of a run
constexpr int kScanThreads = 128;
enum { kScanWhole = 0, kScanLocal = 1, kScanFrom = 2 };

struct ScanArgs {
  const void* xbc; int xbc_dtype; int64_t ld_xbc;        // rows [x: heads * P | B: groups * N | C: groups * N]
  const void* dt; int dt_dtype; int64_t ld_dt; int dt_col;   // raw step sizes: column dt_col + h of a row
  const float* dt_bias; const float* a_log; const float* d_skip;   // [heads] each
  float* state; int64_t state_stride;                      // per slot: S [heads][N][P] at offset 0
  const int* q_start; const int* slots;
  float* y;                                                // [tokens, heads * P] fp32
  float* run_state; float* run_decay;                      // [runs][heads * N * P], [runs][heads]
  int heads, groups, N, P;
};

// The first run of an entry in the run arrays: entries' runs never overlap, since an entry of len tokens has at most
// len / kScanRun + 1 runs and the next entry starts len rows and one entry later.
__device__ __forceinline__ size_t scan_first_run(int row0, int entry) { return (size_t)(row0 / kScanRun) + entry; }

__device__ __forceinline__ unsigned ss_load_raw(const void* p, int dtype, size_t i) {
  return dtype == TIB_F32 ? reinterpret_cast<const unsigned*>(p)[i] : (unsigned)reinterpret_cast<const unsigned short*>(p)[i];
}
__device__ __forceinline__ float ss_from_raw(unsigned raw, int dtype) { return __uint_as_float(dtype == TIB_F32 ? raw : raw << 16); }

// Two fp32 values in one 64-bit register, for the packed fp32 instructions of sm_100 (each half is rounded as the scalar
// instruction rounds it).
typedef unsigned long long f32x2;
__device__ __forceinline__ f32x2 f2_pack(float lo, float hi) {
  f32x2 r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void f2_unpack(f32x2 v, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ f32x2 f2_fma(f32x2 a, f32x2 b, f32x2 c) {
  f32x2 r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ f32x2 f2_mul(f32x2 a, f32x2 b) {
  f32x2 r;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}

template <int NPT, int CP, int MODE>
__global__ void __launch_bounds__(kScanThreads) ssd_scan_kernel(ScanArgs a) {
  pdl_wait();
  pdl_trigger();
  constexpr int NP = NPT * kScanLanesN;                    // N padded
  constexpr int COLS = kScanGroups * CP;
  constexpr int CHUNK = NPT <= 16 ? 16 : 8;                // tokens of a stage
  constexpr int ROW = 2 * NP + COLS;                       // values fetched for a token
  constexpr int FETCH = (ROW + kScanThreads - 1) / kScanThreads;
  static_assert(NPT % 2 == 0, "a thread holds pairs of neighbouring n");
  constexpr int NH = NPT / 2;
  __shared__ __align__(16) float4 bc_s[2][CHUNK][NP / 2];   // (B_n, B_(n+1), C_n, C_(n+1)) for even n
  __shared__ __align__(16) float x_s[2][CHUNK][COLS];
  __shared__ float dt_s[2][CHUNK], a_s[2][CHUNK];
  const int entry = blockIdx.z;
  const int N = a.N, P = a.P, inner = a.heads * P;
  const int tiles = (P + COLS - 1) / COLS;
  const int h = blockIdx.x / tiles, p0 = (blockIdx.x - h * tiles) * COLS;
  const int row0 = a.q_start[entry], len = a.q_start[entry + 1] - row0;
  const int first = MODE == kScanWhole ? 0 : blockIdx.y * kScanRun;
  if (first >= len) return;
  const int last = MODE == kScanWhole ? len : min(len, first + kScanRun);
  const int g = h / (a.heads / a.groups);
  const int tid = threadIdx.x;
  const int ln = tid % kScanLanesN, cg = tid / kScanLanesN;
  const int p = p0 + cg * CP;                              // this thread's first column
  const size_t run = scan_first_run(row0, entry) + blockIdx.y;
  float* S = MODE == kScanWhole ? a.state + (size_t)a.slots[entry] * a.state_stride + (size_t)h * N * P
                                : a.run_state + (run * a.heads + h) * (size_t)N * P;
  // this thread's n: 2 * ln + 16 * j and the one after it, as the halves of a pair
  f32x2 s[NH][CP];
#pragma unroll
  for (int j = 0; j < NH; ++j) {
    const int n = 2 * ln + 2 * kScanLanesN * j;
#pragma unroll
    for (int c = 0; c < CP; ++c) {
      const bool in = MODE != kScanLocal && p + c < P;
      s[j][c] = f2_pack(in && n < N ? S[(size_t)n * P + p + c] : 0.f, in && n + 1 < N ? S[(size_t)(n + 1) * P + p + c] : 0.f);
    }
  }
  const float rate = expf(a.a_log[h]), bias = a.dt_bias[h], skip = a.d_skip[h];
  const int xdt = a.xbc_dtype;

  // what this thread fetches of a token's row: for piece i the column of the input row (-1: nothing, the place holds
  // zero) and the float of the stage's row it lands in
  int src[FETCH], dst[FETCH];
#pragma unroll
  for (int i = 0; i < FETCH; ++i) {
    const int col = i * kScanThreads + tid;
    src[i] = -1;
    dst[i] = -1;
    if (col < NP) {                                        // B_n
      dst[i] = (col >> 1) * 4 + (col & 1);
      if (col < N) src[i] = inner + g * N + col;
    } else if (col < 2 * NP) {                             // C_n
      const int n = col - NP;
      if (MODE != kScanLocal) {
        dst[i] = (n >> 1) * 4 + 2 + (n & 1);
        if (n < N) src[i] = inner + (a.groups + g) * N + n;
      }
    } else if (col < ROW) {                                // x
      const int cc = col - 2 * NP;
      dst[i] = 2 * NP * CHUNK + cc;                        // (told apart from the pairs below)
      if (p0 + cc < P) src[i] = h * P + p0 + cc;
    }
  }
  auto put = [&](int stage, int t, int i, float v) {
    if (dst[i] < 0) return;
    if (dst[i] >= 2 * NP * CHUNK) x_s[stage][t][dst[i] - 2 * NP * CHUNK] = v;
    else reinterpret_cast<float*>(&bc_s[stage][t][0])[dst[i]] = v;
  };
  auto put_step = [&](int stage, int t, float raw) {
    const float step = ss_softplus(raw + bias);
    dt_s[stage][t] = step;
    a_s[stage][t] = expf(-rate * step);
  };

  // the first chunk, all at once
  {
    const int nt = min(CHUNK, last - first);
    for (int tb = 0; tb < nt; tb += 4) {                   // four rows' loads in flight at a time
      unsigned got[4][FETCH];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const size_t row = (size_t)(row0 + first + min(tb + u, nt - 1)) * a.ld_xbc;
#pragma unroll
        for (int i = 0; i < FETCH; ++i) got[u][i] = src[i] >= 0 ? ss_load_raw(a.xbc, xdt, row + src[i]) : 0u;
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (tb + u >= nt) break;
#pragma unroll
        for (int i = 0; i < FETCH; ++i) put(0, tb + u, i, ss_from_raw(got[u][i], xdt));
      }
    }
    if (tid < nt) put_step(0, tid, ss_load(a.dt, a.dt_dtype, (size_t)(row0 + first + tid) * a.ld_dt + a.dt_col + h));
  }
  __syncthreads();

  float kept = 1.f;                                        // the product of the run's decays
  int stage = 0;
  for (int t0 = first; t0 < last; t0 += CHUNK, stage ^= 1) {
    const int nt = min(CHUNK, last - t0);
    const int nt_next = min(CHUNK, last - t0 - CHUNK);     // (at most 0 after the last chunk)
    // Row t of the next chunk is asked for when the walk reaches token t and put into the other stage two tokens later
    // (the last two after the walk), so that nothing waits on the loads.
    unsigned raw[2][FETCH];
    float raw_step[2];
    auto ask = [&](int t, unsigned (&r)[FETCH], float& rs) {
      if (t >= nt_next) return;
      const size_t row = (size_t)(row0 + t0 + CHUNK + t) * a.ld_xbc;
#pragma unroll
      for (int i = 0; i < FETCH; ++i) r[i] = src[i] >= 0 ? ss_load_raw(a.xbc, xdt, row + src[i]) : 0u;
      if (tid == (t & 3) * 32) rs = ss_load(a.dt, a.dt_dtype, (size_t)(row0 + t0 + CHUNK + t) * a.ld_dt + a.dt_col + h);
    };
    auto land = [&](int t, const unsigned (&r)[FETCH], float rs) {
      if (t < 0 || t >= nt_next) return;
#pragma unroll
      for (int i = 0; i < FETCH; ++i) put(stage ^ 1, t, i, ss_from_raw(r[i], xdt));
      if (tid == (t & 3) * 32) put_step(stage ^ 1, t, rs);
    };
    auto walk = [&](int t) {
      const float decay = a_s[stage][t], step = dt_s[stage][t];
      float x[CP], acc[CP];
      f32x2 dx[CP], sum[CP];
      const f32x2 decay2 = f2_pack(decay, decay);
#pragma unroll
      for (int c = 0; c < CP; ++c) {
        x[c] = x_s[stage][t][cg * CP + c];
        const float d = step * x[c];
        dx[c] = f2_pack(d, d);
        sum[c] = f2_pack(0.f, 0.f);
      }
      kept *= decay;
#pragma unroll
      for (int j = 0; j < NH; ++j) {
        const int pair = ln + kScanLanesN * j;
        if (MODE == kScanLocal) {
          const f32x2 b = reinterpret_cast<const ulonglong2*>(&bc_s[stage][t][pair])->x;
#pragma unroll
          for (int c = 0; c < CP; ++c) s[j][c] = f2_fma(decay2, s[j][c], f2_mul(dx[c], b));
        } else {
          const ulonglong2 bc = *reinterpret_cast<const ulonglong2*>(&bc_s[stage][t][pair]);
#pragma unroll
          for (int c = 0; c < CP; ++c) {
            s[j][c] = f2_fma(decay2, s[j][c], f2_mul(dx[c], bc.x));
            sum[c] = f2_fma(s[j][c], bc.y, sum[c]);
          }
        }
      }
      if (MODE != kScanLocal) {
#pragma unroll
        for (int c = 0; c < CP; ++c) {
          float even, odd;
          f2_unpack(sum[c], even, odd);
          acc[c] = even + odd;
#pragma unroll
          for (int o = kScanLanesN / 2; o > 0; o >>= 1) acc[c] += __shfl_xor_sync(0xffffffffu, acc[c], o);
          if (ln == 0 && p + c < P) a.y[(size_t)(row0 + t0 + t) * inner + h * P + p + c] = fmaf(skip, x[c], acc[c]);
        }
      }
    };
    for (int t = 0; t < nt; t += 2) {
      land(t - 2, raw[0], raw_step[0]);
      ask(t, raw[0], raw_step[0]);
      walk(t);
      if (t + 1 < nt) {
        land(t - 1, raw[1], raw_step[1]);
        ask(t + 1, raw[1], raw_step[1]);
        walk(t + 1);
      }
    }
    // (a chunk with a successor is full, so nt is even there and the rows still in registers are nt - 2 and nt - 1)
    land(nt - 2, raw[0], raw_step[0]);
    land(nt - 1, raw[1], raw_step[1]);
    __syncthreads();      // the next chunk is whole in its stage, and nobody reads this one any more
  }
  if (MODE == kScanFrom) return;
#pragma unroll
  for (int j = 0; j < NH; ++j) {
    const int n = 2 * ln + 2 * kScanLanesN * j;
#pragma unroll
    for (int c = 0; c < CP; ++c) {
      float lo, hi;
      f2_unpack(s[j][c], lo, hi);
      if (p + c < P && n < N) S[(size_t)n * P + p + c] = lo;
      if (p + c < P && n + 1 < N) S[(size_t)(n + 1) * P + p + c] = hi;
    }
  }
  if (MODE == kScanLocal && p0 == 0 && threadIdx.x == 0) a.run_decay[run * a.heads + h] = kept;
}

// grid (state elements / 256, entries): S_(r+1) = A_r S_r + L_r over the entry's runs; run_state[r] turns from L_r into S_r.
__global__ void __launch_bounds__(256) ssd_fold_runs_kernel(ScanArgs a) {
  pdl_wait();
  pdl_trigger();
  const int entry = blockIdx.y;
  const int row0 = a.q_start[entry], len = a.q_start[entry + 1] - row0;
  const size_t per_head = (size_t)a.N * a.P, width = per_head * a.heads;
  const size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (len <= 0 || e >= width) return;
  const int h = (int)(e / per_head);
  const int runs = (len + kScanRun - 1) / kScanRun;
  const size_t run0 = scan_first_run(row0, entry);
  float* slot = a.state + (size_t)a.slots[entry] * a.state_stride + e;
  float st = *slot;
  constexpr int AHEAD = 4;
  for (int r = 0; r < runs; r += AHEAD) {
    float sum[AHEAD], decay[AHEAD];
#pragma unroll
    for (int u = 0; u < AHEAD; ++u) {
      const bool in = r + u < runs;
      sum[u] = in ? a.run_state[(run0 + r + u) * width + e] : 0.f;
      decay[u] = in ? a.run_decay[(run0 + r + u) * a.heads + h] : 1.f;
    }
#pragma unroll
    for (int u = 0; u < AHEAD; ++u) {
      if (r + u >= runs) break;
      a.run_state[(run0 + r + u) * width + e] = st;
      st = fmaf(decay[u], st, sum[u]);
    }
  }
  *slot = st;
}

// -------------------------------------------------------------------------------------------- gate, then norm
// grid (rows, parts): out[t, c] = v / sqrt(mean over the part of v^2 + eps) * weight[c],  v = y[t, c] * silu(z[t, c])
__global__ void __launch_bounds__(256)
gated_group_norm_kernel(const float* __restrict__ y, const void* __restrict__ z, int z_dtype, int64_t ldz, int z_col,
                        const float* __restrict__ weight, float eps, void* __restrict__ out, int out_dtype, int width, int part) {
  pdl_wait();
  pdl_trigger();
  __shared__ float scratch[33];
  const size_t row = blockIdx.x;
  const int c0 = blockIdx.y * part;
  float ss = 0.f;
  for (int c = threadIdx.x; c < part; c += blockDim.x) {
    const float v = y[row * width + c0 + c] * ss_silu(ss_load(z, z_dtype, row * ldz + z_col + c0 + c));
    ss = fmaf(v, v, ss);
  }
  const float inv = 1.f / sqrtf(block_sum(ss, scratch) / (float)part + eps);
  for (int c = threadIdx.x; c < part; c += blockDim.x) {
    const float v = y[row * width + c0 + c] * ss_silu(ss_load(z, z_dtype, row * ldz + z_col + c0 + c));
    ss_store(out, out_dtype, row * width + c0 + c, v * inv * weight[c0 + c]);
  }
}

static inline bool ss_known(int dtype) { return dtype == TIB_F32 || dtype == TIB_BF16; }

}  // namespace tib

using namespace tib;

// in: rows of `in_dtype` with row stride ld, the convolved columns starting at col; weight [channels, taps] and bias
// [channels] fp32; state: per slot (stride state_stride floats) the carried inputs [taps - 1][channels] at state_off;
// out: [tokens, channels] in out_dtype.  max_q_len: the longest entry of the step.
TIB_API int tib_short_conv(const void* in, int in_dtype, int64_t ld, int col, const float* weight, const float* bias, float* state,
                           int64_t state_stride, int64_t state_off, const int* q_start, const int* slots, void* out, int out_dtype,
                           int channels, int taps, int silu, int n_entries, int max_q_len, cudaStream_t stream) {
  if (n_entries == 0 || max_q_len == 0 || channels == 0) return TIB_OK;
  if (!in || !weight || !state || !q_start || !slots || !out) return TIB_E_ARG;
  if (taps < 1 || taps > kConvMaxTaps || channels < 0 || n_entries > 65535) return TIB_E_SIZE;
  if (!ss_known(in_dtype) || !ss_known(out_dtype)) return TIB_E_DTYPE;
  ConvArgs a;
  a.in = in; a.in_dtype = in_dtype; a.ld = ld; a.col = col; a.weight = weight; a.bias = bias; a.state = state;
  a.state_stride = state_stride; a.state_off = state_off; a.q_start = q_start; a.slots = slots; a.out = out;
  a.out_dtype = out_dtype; a.channels = channels; a.taps = taps; a.silu = silu;
  const int segments = ceil_div(max_q_len, kConvSegment);
  if (segments > 65535) return TIB_E_SIZE;
  TIB_LAUNCH_DEPENDENT(short_conv_kernel, dim3(ceil_div(channels, kConvChannels), segments, n_entries), kConvChannels, 0, stream, a);
  return TIB_OK;
}

// The largest state size N the scan takes, and the length of a run.
TIB_API int tib_ssd_scan_max_state() { return 32 * kScanLanesN; }
TIB_API int tib_ssd_scan_run() { return kScanRun; }

template <int NPT, int CP>
static int ssd_scan_launch(const ScanArgs& a, int n_entries, int max_q_len, bool runs, cudaStream_t stream) {
  const int tiles = ceil_div(a.P, kScanGroups * CP);
  if (!runs) {
    TIB_LAUNCH_DEPENDENT((ssd_scan_kernel<NPT, CP, kScanWhole>), dim3(tiles * a.heads, 1, n_entries), kScanThreads, 0, stream, a);
    return TIB_OK;
  }
  const dim3 grid(tiles * a.heads, ceil_div(max_q_len, kScanRun), n_entries);
  TIB_LAUNCH_DEPENDENT((ssd_scan_kernel<NPT, CP, kScanLocal>), grid, kScanThreads, 0, stream, a);
  const int64_t width = (int64_t)a.heads * a.N * a.P;
  TIB_LAUNCH_DEPENDENT(ssd_fold_runs_kernel, dim3((unsigned)ceil_div64(width, 256), n_entries), 256, 0, stream, a);
  TIB_LAUNCH_DEPENDENT((ssd_scan_kernel<NPT, CP, kScanFrom>), grid, kScanThreads, 0, stream, a);
  return TIB_OK;
}

// run_state [run_capacity][heads * N * P] and run_decay [run_capacity][heads] (fp32, contents do not matter) are needed
// when max_q_len exceeds a run: run_capacity >= n_tokens / run + n_entries.  Without them every portion is walked in
// one piece.
TIB_API int tib_ssd_scan(const void* xbc, int xbc_dtype, int64_t ld_xbc, const void* dt, int dt_dtype, int64_t ld_dt, int dt_col,
                         const float* dt_bias, const float* a_log, const float* d_skip, float* state, int64_t state_stride,
                         const int* q_start, const int* slots, float* y, int heads, int groups, int N, int P, int n_entries,
                         int n_tokens, int max_q_len, float* run_state, float* run_decay, int64_t run_capacity,
                         cudaStream_t stream) {
  if (n_entries == 0 || max_q_len == 0) return TIB_OK;
  if (!xbc || !dt || !dt_bias || !a_log || !d_skip || !state || !q_start || !slots || !y) return TIB_E_ARG;
  if (heads < 1 || groups < 1 || heads % groups || N < 1 || P < 1 || N > 32 * kScanLanesN) return TIB_E_SIZE;
  if (n_entries > 65535 || n_tokens < 0 || max_q_len < 0) return TIB_E_SIZE;
  if (!ss_known(xbc_dtype) || !ss_known(dt_dtype)) return TIB_E_DTYPE;
  const bool runs = max_q_len > kScanRun && run_state && run_decay;
  if (runs && (run_capacity < n_tokens / kScanRun + n_entries || ceil_div(max_q_len, kScanRun) > 65535)) return TIB_E_SIZE;
  ScanArgs a;
  a.xbc = xbc; a.xbc_dtype = xbc_dtype; a.ld_xbc = ld_xbc; a.dt = dt; a.dt_dtype = dt_dtype; a.ld_dt = ld_dt; a.dt_col = dt_col;
  a.dt_bias = dt_bias; a.a_log = a_log; a.d_skip = d_skip; a.state = state; a.state_stride = state_stride;
  a.q_start = q_start; a.slots = slots; a.y = y; a.run_state = run_state; a.run_decay = run_decay;
  a.heads = heads; a.groups = groups; a.N = N; a.P = P;
  const int npt = ceil_div(N, kScanLanesN);
  const bool wide = P > kScanGroups;        // four columns a thread where a head has more columns than a block has groups
#define TIB_SCAN_CASE(NPT) \
  return wide ? ssd_scan_launch<NPT, 4>(a, n_entries, max_q_len, runs, stream) : ssd_scan_launch<NPT, 1>(a, n_entries, max_q_len, runs, stream)
  if (npt <= 2) TIB_SCAN_CASE(2);
  if (npt <= 4) TIB_SCAN_CASE(4);
  if (npt <= 6) TIB_SCAN_CASE(6);
  if (npt <= 8) TIB_SCAN_CASE(8);
  if (npt <= 16) TIB_SCAN_CASE(16);
  TIB_SCAN_CASE(32);
#undef TIB_SCAN_CASE
}

// y: [rows, width] fp32; z: rows of z_dtype (row stride ldz, first column z_col); weight [width] fp32; out [rows, width].
TIB_API int tib_gated_group_norm(const float* y, const void* z, int z_dtype, int64_t ldz, int z_col, const float* weight, float eps,
                                 void* out, int out_dtype, int rows, int width, int parts, cudaStream_t stream) {
  if (rows == 0 || width == 0) return TIB_OK;
  if (!y || !z || !weight || !out || rows < 0) return TIB_E_ARG;
  if (parts < 1 || width % parts || parts > 65535) return TIB_E_SIZE;
  if (!ss_known(z_dtype) || !ss_known(out_dtype)) return TIB_E_DTYPE;
  const int part = width / parts;
  const int threads = part >= 1024 ? 256 : part >= 256 ? 128 : 64;
  TIB_LAUNCH_DEPENDENT(gated_group_norm_kernel, dim3(rows, parts), threads, 0, stream, y, z, z_dtype, ldz, z_col, weight, eps, out,
                       out_dtype, width, part);
  return TIB_OK;
}
