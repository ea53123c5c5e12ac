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
constexpr int kScanLanesN = 8;         // lanes that share one column of the state along N
constexpr int kScanCols = 16;          // columns (of P) a block of 128 threads owns
constexpr int kScanChunk = 16;         // tokens staged at a time

struct ScanArgs {
  const void* xbc; int xbc_dtype; int64_t ld_xbc;        // rows [x: heads * P | B: groups * N | C: groups * N]
  const void* dt; int dt_dtype; int64_t ld_dt; int dt_col;   // raw step sizes: column dt_col + h of a row
  const float* dt_bias; const float* a_log; const float* d_skip;   // [heads] each
  float* state; int64_t state_stride;                      // per slot: S [heads][N][P] at offset 0
  const int* q_start; const int* slots;
  float* y;                                                // [tokens, heads * P] fp32
  int heads, groups, N, P;
};

template <int NPT>
__global__ void __launch_bounds__(128) ssd_scan_kernel(ScanArgs a) {
  pdl_wait();
  pdl_trigger();
  constexpr int NP = NPT * kScanLanesN;                    // N padded
  __shared__ float b_s[kScanChunk][NP], c_s[kScanChunk][NP], x_s[kScanChunk][kScanCols], dt_s[kScanChunk], a_s[kScanChunk];
  const int entry = blockIdx.z, h = blockIdx.y, p0 = blockIdx.x * kScanCols;
  const int row0 = a.q_start[entry], len = a.q_start[entry + 1] - row0;
  if (len <= 0) return;
  const int N = a.N, P = a.P, inner = a.heads * P;
  const int g = h / (a.heads / a.groups);
  const int ln = threadIdx.x % kScanLanesN, col = threadIdx.x / kScanLanesN;     // col 0..15
  const int p = p0 + col;
  const bool live = p < P;
  float* S = a.state + (size_t)a.slots[entry] * a.state_stride + (size_t)h * N * P;
  float s[NPT];
#pragma unroll
  for (int j = 0; j < NPT; ++j) {
    const int n = ln + kScanLanesN * j;
    s[j] = (live && n < N) ? S[(size_t)n * P + p] : 0.f;
  }
  const float rate = expf(a.a_log[h]), bias = a.dt_bias[h], skip = a.d_skip[h];
  for (int t0 = 0; t0 < len; t0 += kScanChunk) {
    const int nt = min(kScanChunk, len - t0);
    __syncthreads();
    for (int e = threadIdx.x; e < nt * NP; e += blockDim.x) {
      const int t = e / NP, n = e - t * NP;
      const size_t row = (size_t)(row0 + t0 + t) * a.ld_xbc;
      b_s[t][n] = n < N ? ss_load(a.xbc, a.xbc_dtype, row + inner + g * N + n) : 0.f;
      c_s[t][n] = n < N ? ss_load(a.xbc, a.xbc_dtype, row + inner + (a.groups + g) * N + n) : 0.f;
    }
    for (int e = threadIdx.x; e < nt * kScanCols; e += blockDim.x) {
      const int t = e / kScanCols, cc = e - t * kScanCols;
      x_s[t][cc] = p0 + cc < P ? ss_load(a.xbc, a.xbc_dtype, (size_t)(row0 + t0 + t) * a.ld_xbc + h * P + p0 + cc) : 0.f;
    }
    if (threadIdx.x < nt) {
      const float step = ss_softplus(ss_load(a.dt, a.dt_dtype, (size_t)(row0 + t0 + threadIdx.x) * a.ld_dt + a.dt_col + h) + bias);
      dt_s[threadIdx.x] = step;
      a_s[threadIdx.x] = expf(-rate * step);
    }
    __syncthreads();
    for (int t = 0; t < nt; ++t) {
      const float decay = a_s[t], x = x_s[t][col], dx = dt_s[t] * x;
      float acc = 0.f;
#pragma unroll
      for (int j = 0; j < NPT; ++j) {
        const int n = ln + kScanLanesN * j;
        s[j] = fmaf(decay, s[j], dx * b_s[t][n]);
        acc = fmaf(s[j], c_s[t][n], acc);
      }
#pragma unroll
      for (int o = kScanLanesN / 2; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      if (ln == 0 && live) a.y[(size_t)(row0 + t0 + t) * inner + h * P + p] = fmaf(skip, x, acc);
    }
  }
  if (live) {
#pragma unroll
    for (int j = 0; j < NPT; ++j) {
      const int n = ln + kScanLanesN * j;
      if (n < N) S[(size_t)n * P + p] = s[j];
    }
  }
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

// The largest state size N the scan takes.
TIB_API int tib_ssd_scan_max_state() { return 32 * kScanLanesN; }

TIB_API int tib_ssd_scan(const void* xbc, int xbc_dtype, int64_t ld_xbc, const void* dt, int dt_dtype, int64_t ld_dt, int dt_col,
                         const float* dt_bias, const float* a_log, const float* d_skip, float* state, int64_t state_stride,
                         const int* q_start, const int* slots, float* y, int heads, int groups, int N, int P, int n_entries,
                         cudaStream_t stream) {
  if (n_entries == 0) return TIB_OK;
  if (!xbc || !dt || !dt_bias || !a_log || !d_skip || !state || !q_start || !slots || !y) return TIB_E_ARG;
  if (heads < 1 || groups < 1 || heads % groups || N < 1 || P < 1 || N > 32 * kScanLanesN) return TIB_E_SIZE;
  if (heads > 65535 || n_entries > 65535) return TIB_E_SIZE;
  if (!ss_known(xbc_dtype) || !ss_known(dt_dtype)) return TIB_E_DTYPE;
  ScanArgs a;
  a.xbc = xbc; a.xbc_dtype = xbc_dtype; a.ld_xbc = ld_xbc; a.dt = dt; a.dt_dtype = dt_dtype; a.ld_dt = ld_dt; a.dt_col = dt_col;
  a.dt_bias = dt_bias; a.a_log = a_log; a.d_skip = d_skip; a.state = state; a.state_stride = state_stride;
  a.q_start = q_start; a.slots = slots; a.y = y; a.heads = heads; a.groups = groups; a.N = N; a.P = P;
  const dim3 grid(ceil_div(P, kScanCols), heads, n_entries);
  const int npt = ceil_div(N, kScanLanesN);
  if (npt <= 2) TIB_LAUNCH_DEPENDENT(ssd_scan_kernel<2>, grid, 128, 0, stream, a);
  else if (npt <= 4) TIB_LAUNCH_DEPENDENT(ssd_scan_kernel<4>, grid, 128, 0, stream, a);
  else if (npt <= 6) TIB_LAUNCH_DEPENDENT(ssd_scan_kernel<6>, grid, 128, 0, stream, a);
  else if (npt <= 8) TIB_LAUNCH_DEPENDENT(ssd_scan_kernel<8>, grid, 128, 0, stream, a);
  else if (npt <= 16) TIB_LAUNCH_DEPENDENT(ssd_scan_kernel<16>, grid, 128, 0, stream, a);
  else TIB_LAUNCH_DEPENDENT(ssd_scan_kernel<32>, grid, 128, 0, stream, a);
  return TIB_OK;
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
