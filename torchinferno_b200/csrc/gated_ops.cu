// Row-wise pieces that blocks other than the pre-norm one are put together from: sums of two sublayer
// outputs into the 32-bit residual, a unit norm added to the residual, gates (sigmoid, tanh-GELU times a
// row of a second embedding table), the square of relu, a scale, and the row pairs a layer that re-reads the
// embedding output multiplies.  Statistics, gates and sums are fp32; rows leave in the activation type.
//
// In every kernel x / y / g may be float or bf16 in memory (a dtype code each) and may be slices of a wider
// row (a row stride each), so the output of one fused projection can be taken apart without a copy.
#include "common.cuh"

namespace tib {

__device__ __forceinline__ float load_any(const void* p, int dtype, size_t i) {
  return dtype == TIB_F32 ? reinterpret_cast<const float*>(p)[i] : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
}
__device__ __forceinline__ void store_any(void* p, int dtype, size_t i, float v) {
  if (dtype == TIB_F32) reinterpret_cast<float*>(p)[i] = v;
  else reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
}
__device__ __forceinline__ float sigmoid_f(float z) { return 1.f / (1.f + expf(-z)); }
__device__ __forceinline__ float gelu_tanh_f(float z) {
  const float c = 0.7978845608028654f;     // sqrt(2 / pi)
  return 0.5f * z * (1.f + tanhf(c * (z + 0.044715f * z * z * z)));
}

// residual[t] += a[t] + b[t] (b may be null); optionally the new residual row also leaves in another type.
__global__ void add_pair_kernel(float* __restrict__ residual, const void* __restrict__ a, int a_dtype, int64_t lda,
                                const void* __restrict__ b, int b_dtype, int64_t ldb, void* __restrict__ copy,
                                int copy_dtype, int width) {
  pdl_wait();
  pdl_trigger();
  const size_t row = blockIdx.x;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    float d = load_any(a, a_dtype, row * lda + c);
    if (b) d += load_any(b, b_dtype, row * ldb + c);
    const float v = residual[row * width + c] + d;
    residual[row * width + c] = v;
    if (copy) store_any(copy, copy_dtype, row * width + c, v);
  }
}

// residual[t] += y[t] / sqrt(mean(y[t]^2) + eps) * weight
__global__ void unit_norm_add_kernel(float* __restrict__ residual, const void* __restrict__ y, int y_dtype, int64_t ldy,
                                     const float* __restrict__ weight, int width, float eps) {
  pdl_wait();
  pdl_trigger();
  __shared__ float scratch[33];
  const size_t row = blockIdx.x;
  float ss = 0.f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float v = load_any(y, y_dtype, row * ldy + c);
    ss += v * v;
  }
  const float inv = 1.f / sqrtf(block_sum(ss, scratch) / (float)width + eps);
  for (int c = threadIdx.x; c < width; c += blockDim.x)
    residual[row * width + c] += load_any(y, y_dtype, row * ldy + c) * inv * weight[c];
}

// out[t] = f(x[t]) * sigmoid(g[t]);  f = identity (weight null) or the RMS norm with `weight`.  Column c reads gate
// c / group: one gate per element (group 1) or one per run of `group` columns (a head).
__global__ void sigmoid_gate_kernel(const void* __restrict__ x, int x_dtype, int64_t ldx, const void* __restrict__ g,
                                    int g_dtype, int64_t ldg, const float* __restrict__ weight, float eps,
                                    void* __restrict__ out, int out_dtype, int width, int group) {
  pdl_wait();
  pdl_trigger();
  __shared__ float scratch[33];
  const size_t row = blockIdx.x;
  float inv = 1.f;
  if (weight) {
    float ss = 0.f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
      const float v = load_any(x, x_dtype, row * ldx + c);
      ss += v * v;
    }
    inv = 1.f / sqrtf(block_sum(ss, scratch) / (float)width + eps);
  }
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    float v = load_any(x, x_dtype, row * ldx + c) * inv;
    if (weight) v *= weight[c];
    store_any(out, out_dtype, row * width + c, v * sigmoid_f(load_any(g, g_dtype, row * ldg + (group > 1 ? c / group : c))));
  }
}

// out[t, j] = gelu_tanh(a[t, j]) * table[ids[t], first + j]; an id outside the table writes NaN.
__global__ void gelu_gate_table_kernel(const void* __restrict__ a, int a_dtype, int64_t lda, const int* __restrict__ ids,
                                       const void* __restrict__ table, int table_dtype, int64_t ld_table, int vocab,
                                       int first, void* __restrict__ out, int out_dtype, int width) {
  pdl_wait();
  pdl_trigger();
  const size_t row = blockIdx.x;
  const int id = ids[row];
  const bool known = id >= 0 && id < vocab;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float e = known ? load_any(table, table_dtype, (size_t)id * ld_table + first + c) : __int_as_float(0x7fc00000);
    store_any(out, out_dtype, row * width + c, gelu_tanh_f(load_any(a, a_dtype, row * lda + c)) * e);
  }
}

// out = relu(x)^2, element by element
__global__ void relu_squared_kernel(const void* __restrict__ x, int x_dtype, void* __restrict__ out, int out_dtype, int64_t n) {
  pdl_wait();
  pdl_trigger();
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const float v = fmaxf(load_any(x, x_dtype, i), 0.f);
    store_any(out, out_dtype, i, v * v);
  }
}

// x *= s (fp32), element by element
__global__ void scale_kernel(float* __restrict__ x, float s, int64_t n) {
  pdl_wait();
  pdl_trigger();
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) x[i] *= s;
}

// x <- cap * tanh(x / cap) (fp32), element by element
__global__ void softcap_kernel(float* __restrict__ x, float cap, int64_t n) {
  pdl_wait();
  pdl_trigger();
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
    x[i] = cap * tanhf(x[i] / cap);
}

// out[t] = [x[t] ; y[t]] in the activation type (x, y fp32 rows of `width`)
__global__ void pair_rows_kernel(const float* __restrict__ x, const float* __restrict__ y, void* __restrict__ out,
                                 int out_dtype, int width) {
  pdl_wait();
  pdl_trigger();
  const size_t row = blockIdx.x;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    store_any(out, out_dtype, row * 2 * width + c, x[row * width + c]);
    store_any(out, out_dtype, row * 2 * width + width + c, y[row * width + c]);
  }
}

// x[t] += v (one fp32 vector for every row)
__global__ void add_vector_kernel(float* __restrict__ x, const float* __restrict__ v, int width) {
  pdl_wait();
  pdl_trigger();
  const size_t row = blockIdx.x;
  for (int c = threadIdx.x; c < width; c += blockDim.x) x[row * width + c] += v[c];
}

static inline int row_threads(int width) { return width >= 1024 ? 256 : (width >= 256 ? 128 : 64); }
static inline bool known(int dtype) { return dtype == TIB_F32 || dtype == TIB_BF16; }

// out[i] = g * sigmoid(alpha * g) * (u + 1) with g = min(gu[2i], limit), u = clamp(gu[2i + 1], -limit, limit)
__global__ void glu_clamp_kernel(const void* __restrict__ gu, int gu_dtype, void* __restrict__ out, int out_dtype, int64_t n,
                                 float limit, float alpha) {
  pdl_wait();
  pdl_trigger();
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const float g = fminf(load_any(gu, gu_dtype, 2 * i), limit);
    const float u = fminf(fmaxf(load_any(gu, gu_dtype, 2 * i + 1), -limit), limit);
    store_any(out, out_dtype, i, g / (1.f + expf(-alpha * g)) * (u + 1.f));
  }
}

}  // namespace tib

using namespace tib;

TIB_API int tib_add_pair(float* residual, const void* a, int a_dtype, int64_t lda, const void* b, int b_dtype, int64_t ldb,
                         void* copy, int copy_dtype, int rows, int width, cudaStream_t stream) {
  if (rows == 0 || width == 0) return TIB_OK;
  if (!residual || !a || rows < 0 || width < 0) return TIB_E_ARG;
  if (!known(a_dtype) || (b && !known(b_dtype)) || (copy && !known(copy_dtype))) return TIB_E_DTYPE;
  TIB_LAUNCH_DEPENDENT(add_pair_kernel, rows, row_threads(width), 0, stream, residual, a, a_dtype, lda, b, b_dtype, ldb, copy,
                       copy_dtype, width);
  return TIB_OK;
}

TIB_API int tib_unit_norm_add(float* residual, const void* y, int y_dtype, int64_t ldy, const float* weight, int rows,
                              int width, float eps, cudaStream_t stream) {
  if (rows == 0 || width == 0) return TIB_OK;
  if (!residual || !y || !weight || rows < 0 || width < 0) return TIB_E_ARG;
  if (!known(y_dtype)) return TIB_E_DTYPE;
  TIB_LAUNCH_DEPENDENT(unit_norm_add_kernel, rows, row_threads(width), 0, stream, residual, y, y_dtype, ldy, weight, width, eps);
  return TIB_OK;
}

TIB_API int tib_sigmoid_gate(const void* x, int x_dtype, int64_t ldx, const void* g, int g_dtype, int64_t ldg,
                             const float* weight, float eps, void* out, int out_dtype, int rows, int width, int group,
                             cudaStream_t stream) {
  if (rows == 0 || width == 0) return TIB_OK;
  if (!x || !g || !out || rows < 0 || width < 0 || group < 1) return TIB_E_ARG;
  if (!known(x_dtype) || !known(g_dtype) || !known(out_dtype)) return TIB_E_DTYPE;
  TIB_LAUNCH_DEPENDENT(sigmoid_gate_kernel, rows, row_threads(width), 0, stream, x, x_dtype, ldx, g, g_dtype, ldg, weight, eps,
                       out, out_dtype, width, group);
  return TIB_OK;
}

TIB_API int tib_gelu_gate_table(const void* a, int a_dtype, int64_t lda, const int* ids, const void* table, int table_dtype,
                                int64_t ld_table, int vocab, int first, void* out, int out_dtype, int rows, int width,
                                cudaStream_t stream) {
  if (rows == 0 || width == 0) return TIB_OK;
  if (!a || !ids || !table || !out || rows < 0 || width < 0 || first < 0 || first + width > ld_table) return TIB_E_ARG;
  if (!known(a_dtype) || !known(table_dtype) || !known(out_dtype)) return TIB_E_DTYPE;
  TIB_LAUNCH_DEPENDENT(gelu_gate_table_kernel, rows, row_threads(width), 0, stream, a, a_dtype, lda, ids, table, table_dtype,
                       ld_table, vocab, first, out, out_dtype, width);
  return TIB_OK;
}

TIB_API int tib_relu_squared(const void* x, int x_dtype, void* out, int out_dtype, int64_t n, cudaStream_t stream) {
  if (n == 0) return TIB_OK;
  if (!x || !out || n < 0) return TIB_E_ARG;
  if (!known(x_dtype) || !known(out_dtype)) return TIB_E_DTYPE;
  const int blocks = (int)(ceil_div64(n, 256) < 148 * 8 ? ceil_div64(n, 256) : 148 * 8);
  TIB_LAUNCH_DEPENDENT(relu_squared_kernel, blocks, 256, 0, stream, x, x_dtype, out, out_dtype, n);
  return TIB_OK;
}

// gu: [rows, 2 * width] with (gate i, up i) side by side; out: [rows, width].
TIB_API int tib_glu_clamp(const void* gu, int gu_dtype, void* out, int out_dtype, int rows, int width, float limit, float alpha,
                          cudaStream_t stream) {
  const int64_t n = (int64_t)rows * width;
  if (n == 0) return TIB_OK;
  if (!gu || !out || rows < 0 || width < 0) return TIB_E_ARG;
  if (!known(gu_dtype) || !known(out_dtype)) return TIB_E_DTYPE;
  const int blocks = (int)(ceil_div64(n, 256) < 148 * 8 ? ceil_div64(n, 256) : 148 * 8);
  TIB_LAUNCH_DEPENDENT(glu_clamp_kernel, blocks, 256, 0, stream, gu, gu_dtype, out, out_dtype, n, limit, alpha);
  return TIB_OK;
}

TIB_API int tib_scale_f32(float* x, float s, int64_t n, cudaStream_t stream) {
  if (n == 0) return TIB_OK;
  if (!x || n < 0) return TIB_E_ARG;
  const int blocks = (int)(ceil_div64(n, 256) < 148 * 8 ? ceil_div64(n, 256) : 148 * 8);
  TIB_LAUNCH_DEPENDENT(scale_kernel, blocks, 256, 0, stream, x, s, n);
  return TIB_OK;
}

TIB_API int tib_softcap_f32(float* x, float cap, int64_t n, cudaStream_t stream) {
  if (n == 0) return TIB_OK;
  if (!x || n < 0 || !(cap > 0.f)) return TIB_E_ARG;
  const int blocks = (int)(ceil_div64(n, 256) < 148 * 8 ? ceil_div64(n, 256) : 148 * 8);
  TIB_LAUNCH_DEPENDENT(softcap_kernel, blocks, 256, 0, stream, x, cap, n);
  return TIB_OK;
}

TIB_API int tib_pair_rows(const float* x, const float* y, void* out, int out_dtype, int rows, int width, cudaStream_t stream) {
  if (rows == 0 || width == 0) return TIB_OK;
  if (!x || !y || !out || rows < 0 || width < 0) return TIB_E_ARG;
  if (!known(out_dtype)) return TIB_E_DTYPE;
  TIB_LAUNCH_DEPENDENT(pair_rows_kernel, rows, row_threads(width), 0, stream, x, y, out, out_dtype, width);
  return TIB_OK;
}

TIB_API int tib_add_vector(float* x, const float* v, int rows, int width, cudaStream_t stream) {
  if (rows == 0 || width == 0) return TIB_OK;
  if (!x || !v || rows < 0 || width < 0) return TIB_E_ARG;
  TIB_LAUNCH_DEPENDENT(add_vector_kernel, rows, row_threads(width), 0, stream, x, v, width);
  return TIB_OK;
}
