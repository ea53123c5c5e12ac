// Layer norm with weight and bias, in the places a block with norms before and after each sublayer needs it, and
// the weighted sum over the outputs of all earlier layers (a depth average) that such a block may end with.
//
//   y = (x - mean(x)) / sqrt(mean((x - mean(x))^2) + eps) * w + b
//
// Mean, squared deviations, the scaling and every sum into the residual are fp32: a row is read once into shared
// memory as floats (or kept in registers), the mean is taken, then the deviations from it (two passes over the row,
// not the one-pass E[x^2] - E[x]^2 form, which loses digits when the mean is large).
//
//   layernorm          out[i] = LN(x[rows ? rows[i] : i])                   x: fp32 residual or activation rows
//   layernorm_tail     what follows a sublayer, as one launch, each step optional:
//                        residual[i] += LN_a(y[i])                          (without a norm a: residual[i] += y[i])
//                        next[i] = sum_{j < count} coef[j] * history[j][i], written to history[count][i], where
//                                  history[count - 1] is the residual (the running layer's stream)
//                        out[i] = LN_b(the row at hand)
//
// One block per row.  Rows wider than the staged limit are refused.
#include "common.cuh"

namespace tib {

constexpr int kLnMaxWidth = 16384;      // floats of one staged row (64 KB)

__device__ __forceinline__ float ln_load(const void* p, int dtype, size_t i) {
  return dtype == TIB_F32 ? reinterpret_cast<const float*>(p)[i] : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
}
__device__ __forceinline__ void ln_store(void* p, int dtype, size_t i, float v) {
  if (dtype == TIB_F32) reinterpret_cast<float*>(p)[i] = v;
  else reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
}

// mean and 1 / sqrt(variance + eps) of the staged row
__device__ __forceinline__ void ln_stats(const float* row, int width, float eps, float* scratch, float& mean, float& inv) {
  float s = 0.f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) s += row[c];
  mean = block_sum(s, scratch) / (float)width;
  float ss = 0.f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float d = row[c] - mean;
    ss = fmaf(d, d, ss);
  }
  inv = 1.f / sqrtf(block_sum(ss, scratch) / (float)width + eps);
}

struct LnTail {
  // residual[i] += LN(y[i]; wa, ba)      (y null: skipped; wa null: residual[i] += y[i])
  const void* y; int y_dtype; int64_t ldy; const float* wa; const float* ba;
  float* residual;                       // [n, width] fp32 (for the depth average: history[count - 1])
  // next = sum_j coef[j] history[j]     (history null: skipped, next = residual)
  float* history; int64_t slice; const float* coef; int count;
  // out[i] = LN(next[i]; wb, bb)        (out null: skipped)
  const float* wb; const float* bb; void* out; int out_dtype;
  int width; float eps;
};

__global__ void __launch_bounds__(256) layernorm_tail_kernel(LnTail a) {
  pdl_wait();
  pdl_trigger();
  extern __shared__ float row[];
  __shared__ float scratch[33];
  const size_t i = blockIdx.x;
  const int width = a.width;
  float mean, inv;
  if (a.y) {
    for (int c = threadIdx.x; c < width; c += blockDim.x) row[c] = ln_load(a.y, a.y_dtype, i * a.ldy + c);
    __syncthreads();
    if (a.wa) ln_stats(row, width, a.eps, scratch, mean, inv);
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
      const float v = a.residual[i * width + c] + (a.wa ? (row[c] - mean) * inv * a.wa[c] + a.ba[c] : row[c]);
      a.residual[i * width + c] = v;
      row[c] = v;
    }
  } else {
    for (int c = threadIdx.x; c < width; c += blockDim.x) row[c] = a.residual[i * width + c];
  }
  if (a.history) {
    // (the newest output, history[count - 1], is the row at hand)
    float* next = a.history + (size_t)a.count * a.slice + i * width;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
      float v = 0.f;
      for (int j = 0; j + 1 < a.count; ++j) v = fmaf(a.coef[j], a.history[(size_t)j * a.slice + i * width + c], v);
      v = fmaf(a.coef[a.count - 1], row[c], v);
      next[c] = v;
      row[c] = v;
    }
  }
  if (!a.out) return;
  __syncthreads();
  ln_stats(row, width, a.eps, scratch, mean, inv);
  for (int c = threadIdx.x; c < width; c += blockDim.x)
    ln_store(a.out, a.out_dtype, i * width + c, (row[c] - mean) * inv * a.wb[c] + a.bb[c]);
}

__global__ void __launch_bounds__(256)
layernorm_kernel(const void* __restrict__ x, int x_dtype, int64_t ldx, const int* __restrict__ rows, const float* __restrict__ w,
                 const float* __restrict__ b, float eps, void* __restrict__ out, int out_dtype, int width) {
  pdl_wait();
  pdl_trigger();
  extern __shared__ float row[];
  __shared__ float scratch[33];
  const size_t i = blockIdx.x;
  const size_t src = rows ? (size_t)rows[i] : i;
  for (int c = threadIdx.x; c < width; c += blockDim.x) row[c] = ln_load(x, x_dtype, src * ldx + c);
  __syncthreads();
  float mean, inv;
  ln_stats(row, width, eps, scratch, mean, inv);
  for (int c = threadIdx.x; c < width; c += blockDim.x)
    ln_store(out, out_dtype, i * width + c, (row[c] - mean) * inv * w[c] + b[c]);
}


// The same tail with the row in registers: every thread keeps up to PER pieces of four columns (16-byte loads and
// stores; a bf16 y comes in 8-byte pieces).  For widths that are multiples of 4 up to 256 x 4 x PER columns and
// 16-byte aligned rows; `rows` (only without y and history) picks the residual rows that are normed.
template <int PER>
__global__ void __launch_bounds__(256) layernorm_tail_vec_kernel(LnTail a, const int* __restrict__ rows) {
  pdl_wait();
  pdl_trigger();
  __shared__ float scratch[33];
  const size_t i = blockIdx.x;
  const int width = a.width, nvec = width >> 2, T = blockDim.x, tid = threadIdx.x;
  const size_t src = rows ? (size_t)rows[i] : i;
  float4 r[PER];
  const float4* res4 = reinterpret_cast<const float4*>(a.residual + src * width);
#pragma unroll
  for (int p = 0; p < PER; ++p) {
    const int idx = p * T + tid;
    r[p] = idx < nvec ? res4[idx] : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  auto stats = [&](const float4 (&v)[PER], float& mean, float& inv) {
    float s = 0.f;
#pragma unroll
    for (int p = 0; p < PER; ++p) s += (v[p].x + v[p].y) + (v[p].z + v[p].w);      // (pieces past the row are zero)
    mean = block_sum(s, scratch) / (float)width;
    float ss = 0.f;
#pragma unroll
    for (int p = 0; p < PER; ++p) {
      if (p * T + tid >= nvec) continue;
      const float dx = v[p].x - mean, dy = v[p].y - mean, dz = v[p].z - mean, dw = v[p].w - mean;
      ss += (dx * dx + dy * dy) + (dz * dz + dw * dw);
    }
    inv = 1.f / sqrtf(block_sum(ss, scratch) / (float)width + a.eps);
  };
  float mean, inv;
  if (a.y) {
    float4 y[PER];
#pragma unroll
    for (int p = 0; p < PER; ++p) {
      const int idx = p * T + tid;
      y[p] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (idx >= nvec) continue;
      if (a.y_dtype == TIB_F32) {
        y[p] = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(a.y) + i * a.ldy)[idx];
      } else {
        const uint2 raw = reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(a.y) + i * a.ldy)[idx];
        const float2 lo = bf16x2_floats(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
        const float2 hi = bf16x2_floats(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
        y[p] = make_float4(lo.x, lo.y, hi.x, hi.y);
      }
    }
    if (a.wa) stats(y, mean, inv);
    float4* out4 = reinterpret_cast<float4*>(a.residual + i * width);
#pragma unroll
    for (int p = 0; p < PER; ++p) {
      const int idx = p * T + tid;
      if (idx >= nvec) continue;
      if (!a.wa) {
        r[p].x += y[p].x; r[p].y += y[p].y; r[p].z += y[p].z; r[p].w += y[p].w;
        out4[idx] = r[p];
        continue;
      }
      const float4 w = reinterpret_cast<const float4*>(a.wa)[idx], b = reinterpret_cast<const float4*>(a.ba)[idx];
      r[p].x += (y[p].x - mean) * inv * w.x + b.x;
      r[p].y += (y[p].y - mean) * inv * w.y + b.y;
      r[p].z += (y[p].z - mean) * inv * w.z + b.z;
      r[p].w += (y[p].w - mean) * inv * w.w + b.w;
      out4[idx] = r[p];
    }
  }
  if (a.history) {
    float4* next = reinterpret_cast<float4*>(a.history + (size_t)a.count * a.slice + i * width);
#pragma unroll
    for (int p = 0; p < PER; ++p) {
      const int idx = p * T + tid;
      if (idx >= nvec) continue;
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int j = 0; j + 1 < a.count; ++j) {
        const float c = a.coef[j];
        const float4 h = reinterpret_cast<const float4*>(a.history + (size_t)j * a.slice + i * width)[idx];
        v.x = fmaf(c, h.x, v.x); v.y = fmaf(c, h.y, v.y); v.z = fmaf(c, h.z, v.z); v.w = fmaf(c, h.w, v.w);
      }
      const float c = a.coef[a.count - 1];
      v.x = fmaf(c, r[p].x, v.x); v.y = fmaf(c, r[p].y, v.y); v.z = fmaf(c, r[p].z, v.z); v.w = fmaf(c, r[p].w, v.w);
      next[idx] = v;
      r[p] = v;
    }
  }
  if (!a.out) return;
  stats(r, mean, inv);
#pragma unroll
  for (int p = 0; p < PER; ++p) {
    const int idx = p * T + tid;
    if (idx >= nvec) continue;
    const float4 w = reinterpret_cast<const float4*>(a.wb)[idx], b = reinterpret_cast<const float4*>(a.bb)[idx];
    const float4 v = make_float4((r[p].x - mean) * inv * w.x + b.x, (r[p].y - mean) * inv * w.y + b.y,
                                 (r[p].z - mean) * inv * w.z + b.z, (r[p].w - mean) * inv * w.w + b.w);
    if (a.out_dtype == TIB_F32) {
      reinterpret_cast<float4*>(reinterpret_cast<float*>(a.out) + i * width)[idx] = v;
    } else {
      uint2 packed;
      const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
      packed.x = *reinterpret_cast<const uint32_t*>(&lo);
      packed.y = *reinterpret_cast<const uint32_t*>(&hi);
      reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(a.out) + i * width)[idx] = packed;
    }
  }
}

// Launches the register form when the row fits it; returns false when the staged form has to run.
static bool launch_tail_vec(const LnTail& a, const int* rows, int n, cudaStream_t stream, int& status) {
  const int width = a.width;
  auto aligned = [](const void* p) { return ((uintptr_t)p & 15) == 0; };
  if (width % 4 || width > 8192 || !aligned(a.residual) || !aligned(a.history) || !aligned(a.out) || !aligned(a.wa) ||
      !aligned(a.ba) || !aligned(a.wb) || !aligned(a.bb) || (a.slice % 4) != 0)
    return false;
  if (a.y && (a.ldy % 4 || ((uintptr_t)a.y & (a.y_dtype == TIB_F32 ? 15 : 7)))) return false;
  const int nvec = width / 4;
  const int threads = nvec >= 256 ? 256 : ((nvec + 31) / 32) * 32;
  const int per = (nvec + threads - 1) / threads;
  cudaError_t e;
  if (per <= 1) e = launch_dependent(layernorm_tail_vec_kernel<1>, dim3(n), dim3(threads), 0, stream, a, rows);
  else if (per <= 2) e = launch_dependent(layernorm_tail_vec_kernel<2>, dim3(n), dim3(threads), 0, stream, a, rows);
  else if (per <= 4) e = launch_dependent(layernorm_tail_vec_kernel<4>, dim3(n), dim3(threads), 0, stream, a, rows);
  else e = launch_dependent(layernorm_tail_vec_kernel<8>, dim3(n), dim3(threads), 0, stream, a, rows);
  status = e == cudaSuccess ? TIB_OK : (int)e;
  return true;
}

static inline int ln_threads(int width) { return width >= 2048 ? 256 : width >= 512 ? 128 : 64; }

}  // namespace tib

using namespace tib;

// x: [*, width] rows (row stride ldx) in x_dtype; rows: [n] int32 or null; out: [n, width] in out_dtype.
TIB_API int tib_layernorm(const void* x, int x_dtype, int64_t ldx, const int* rows, const float* w, const float* b, float eps,
                          void* out, int out_dtype, int n, int width, cudaStream_t stream) {
  if (n == 0) return TIB_OK;
  if (!x || !w || !b || !out || n < 0 || width < 1) return TIB_E_ARG;
  if (width > kLnMaxWidth) return TIB_E_SIZE;
  if ((x_dtype != TIB_F32 && x_dtype != TIB_BF16) || (out_dtype != TIB_F32 && out_dtype != TIB_BF16)) return TIB_E_DTYPE;
  if (x_dtype == TIB_F32 && ldx == width) {
    LnTail t = {};
    t.residual = const_cast<float*>(reinterpret_cast<const float*>(x));      // (read only: no y, no history)
    t.wb = w; t.bb = b; t.out = out; t.out_dtype = out_dtype; t.width = width; t.eps = eps;
    int status = TIB_OK;
    if (launch_tail_vec(t, rows, n, stream, status)) return status;
  }
  const size_t smem = sizeof(float) * (size_t)width;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(layernorm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  TIB_LAUNCH_DEPENDENT(layernorm_kernel, n, ln_threads(width), smem, stream, x, x_dtype, ldx, rows, w, b, eps, out, out_dtype, width);
  return TIB_OK;
}

// The tail of a sublayer or of a layer (see the head of this file).  y: [n, width] rows (row stride ldy) or null;
// residual: [n, width] fp32; history: [depth, n, width] fp32 or null, with residual == history[count - 1] and
// count + 1 <= depth; coef: [count] fp32; out: [n, width] or null.
TIB_API int tib_layernorm_tail(const void* y, int y_dtype, int64_t ldy, const float* wa, const float* ba, float* residual,
                               float* history, int64_t slice, const float* coef, int count, const float* wb, const float* bb,
                               void* out, int out_dtype, int n, int width, float eps, cudaStream_t stream) {
  if (n == 0) return TIB_OK;
  if (!residual || n < 0 || width < 1) return TIB_E_ARG;
  if (y && ((wa == nullptr) != (ba == nullptr))) return TIB_E_ARG;
  if (out && (!wb || !bb)) return TIB_E_ARG;
  if (history && (!coef || count < 1 || residual != history + (size_t)(count - 1) * slice)) return TIB_E_ARG;
  if (width > kLnMaxWidth) return TIB_E_SIZE;
  if (y && y_dtype != TIB_F32 && y_dtype != TIB_BF16) return TIB_E_DTYPE;
  if (out && out_dtype != TIB_F32 && out_dtype != TIB_BF16) return TIB_E_DTYPE;
  LnTail a;
  a.y = y; a.y_dtype = y_dtype; a.ldy = ldy; a.wa = wa; a.ba = ba; a.residual = residual;
  a.history = history; a.slice = slice; a.coef = coef; a.count = count;
  a.wb = wb; a.bb = bb; a.out = out; a.out_dtype = out_dtype; a.width = width; a.eps = eps;
  int status = TIB_OK;
  if (launch_tail_vec(a, nullptr, n, stream, status)) return status;
  const size_t smem = sizeof(float) * (size_t)width;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(layernorm_tail_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  TIB_LAUNCH_DEPENDENT(layernorm_tail_kernel, n, ln_threads(width), smem, stream, a);
  return TIB_OK;
}
