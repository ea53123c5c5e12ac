// A residual carried in several streams (hyper-connections), and the tanh norm.
//
// Instead of one residual x there are S copies x_1 .. x_S [S, tokens, width] in fp32.  A sublayer reads them through
// one weighted sum and writes its output y back through a small matrix:
//
//   write   x_t <- sum_s mix[s, t] x_s + out_w[t] * y          every stream from the values before the write
//   read    u = sum_s in_w[s] x_s;   rows = norm(u)
//
// One launch does a write (optional), then a read (optional) of the streams it has just made, element by element:
// a thread holds the S values of its elements in registers, so the streams are read once and written once.  With
// `rows` (a gather of token rows, for the logits) nothing is stored: the write is only looked through.
//
// The norm of the read is either none (u leaves in fp32, for a norm kernel of its own) or the tanh norm
// ("dynamic tanh"): tanh(alpha * u) * w + b, which needs no statistic of the row, so it costs nothing extra here.
// S = 1 with mix = [[1]], out_w = [1], in_w = [1] is the plain residual sum followed by the norm, which is how the
// tanh norm serves an ordinary pre-norm block.  All sums and the norm are fp32; the coefficients are fp32 tensors.
#include "common.cuh"

namespace tib {

constexpr int kMaxStreams = 8;

struct HyperArgs {
  float* streams; int64_t stream_stride;          // [S][tokens][width]; elements between streams
  int S, width;
  const void* y; int y_dtype; int64_t ldy;        // the sublayer's output rows or null (no write)
  const float* mix; const float* out_w;           // [S, S] indexed [from, to]; [S]
  const float* in_w;                              // [S] or null (no read)
  const int* rows;                                // gather of token rows or null
  int norm;                                       // 0: u in fp32; 1: tanh norm
  float alpha; const float* weight; const float* bias;
  void* out; int out_dtype;                       // [rows or tokens][width]
};

__device__ __forceinline__ float hs_load(const void* p, int dtype, size_t i) {
  return dtype == TIB_F32 ? reinterpret_cast<const float*>(p)[i] : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
}

// VEC elements a thread and pass (4 where every row starts on a 16-byte boundary: the streams then move in 16-byte
// pieces, rows in bf16 in 8-byte pieces).
template <int S, int VEC>
__global__ void __launch_bounds__(256) hyper_step_kernel(HyperArgs a) {
  pdl_wait();
  pdl_trigger();
  __shared__ float mix_s[S * S], out_s[S], in_s[S];
  if (threadIdx.x < S * S) mix_s[threadIdx.x] = a.y ? a.mix[threadIdx.x] : 0.f;
  if (threadIdx.x < S) {
    out_s[threadIdx.x] = a.y ? a.out_w[threadIdx.x] : 0.f;
    in_s[threadIdx.x] = a.in_w ? a.in_w[threadIdx.x] : 0.f;
  }
  __syncthreads();
  const size_t orow = blockIdx.x;
  const size_t srow = a.rows ? (size_t)a.rows[orow] : orow;
  const bool store = a.y && !a.rows;
  for (int c = (blockIdx.y * blockDim.x + threadIdx.x) * VEC; c < a.width; c += gridDim.y * blockDim.x * VEC) {
    float x[S][VEC];
#pragma unroll
    for (int s = 0; s < S; ++s) {
      const float* src = a.streams + (size_t)s * a.stream_stride + srow * a.width + c;
      if (VEC == 4) {
        const float4 v = *reinterpret_cast<const float4*>(src);
        x[s][0] = v.x; x[s][1] = v.y; x[s][2] = v.z; x[s][3 % VEC] = v.w;
      } else {
        x[s][0] = *src;
      }
    }
    if (a.y) {
      float yv[VEC];
      if (VEC == 4 && a.y_dtype == TIB_BF16) {
        const uint2 raw = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(a.y) + srow * a.ldy + c);
        const float2 lo = bf16x2_floats(*reinterpret_cast<const __nv_bfloat162*>(&raw.x)), hi = bf16x2_floats(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
        yv[0] = lo.x; yv[1 % VEC] = lo.y; yv[2 % VEC] = hi.x; yv[3 % VEC] = hi.y;
      } else {
#pragma unroll
        for (int e = 0; e < VEC; ++e) yv[e] = hs_load(a.y, a.y_dtype, srow * a.ldy + c + e);
      }
#pragma unroll
      for (int e = 0; e < VEC; ++e) {
        float nx[S];
#pragma unroll
        for (int t = 0; t < S; ++t) {
          float v = 0.f;
#pragma unroll
          for (int s = 0; s < S; ++s) v = fmaf(mix_s[s * S + t], x[s][e], v);
          nx[t] = fmaf(out_s[t], yv[e], v);
        }
#pragma unroll
        for (int t = 0; t < S; ++t) x[t][e] = nx[t];
      }
      if (store) {
#pragma unroll
        for (int t = 0; t < S; ++t) {
          float* dst = a.streams + (size_t)t * a.stream_stride + srow * a.width + c;
          if (VEC == 4) *reinterpret_cast<float4*>(dst) = make_float4(x[t][0], x[t][1 % VEC], x[t][2 % VEC], x[t][3 % VEC]);
          else *dst = x[t][0];
        }
      }
    }
    if (a.in_w) {
      float u[VEC];
#pragma unroll
      for (int e = 0; e < VEC; ++e) {
        u[e] = 0.f;
#pragma unroll
        for (int s = 0; s < S; ++s) u[e] = fmaf(in_s[s], x[s][e], u[e]);
        if (a.norm == 1) u[e] = fmaf(tanhf(a.alpha * u[e]), a.weight[c + e], a.bias[c + e]);
      }
      if (a.out_dtype == TIB_F32) {
        float* dst = reinterpret_cast<float*>(a.out) + orow * a.width + c;
        if (VEC == 4) *reinterpret_cast<float4*>(dst) = make_float4(u[0], u[1 % VEC], u[2 % VEC], u[3 % VEC]);
        else *dst = u[0];
      } else {
        __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(a.out) + orow * a.width + c;
        if (VEC == 4) {
          const __nv_bfloat162 lo = __floats2bfloat162_rn(u[0], u[1 % VEC]), hi = __floats2bfloat162_rn(u[2 % VEC], u[3 % VEC]);
          uint2 raw;
          raw.x = *reinterpret_cast<const uint32_t*>(&lo);
          raw.y = *reinterpret_cast<const uint32_t*>(&hi);
          *reinterpret_cast<uint2*>(dst) = raw;
        } else {
          *dst = __float2bfloat16_rn(u[0]);
        }
      }
    }
  }
}

}  // namespace tib

using namespace tib;

// streams: [S, tokens, width] fp32 (stream_stride elements apart).  y (rows of `width`, row stride ldy, its own dtype)
// with mix [S, S] and out_w [S]: the write; null: none.  in_w [S] with out: the read; null: none.  rows: int32 gather of
// n_out token rows (then nothing is stored), or null for all `n_out` = tokens rows.  norm 0: out is fp32 sums; norm 1:
// out = tanh(alpha * u) * weight + bias in out_dtype.
TIB_API int tib_hyper_step(float* streams, int64_t stream_stride, int S, int n_out, int width, const void* y, int y_dtype,
                           int64_t ldy, const float* mix, const float* out_w, const float* in_w, const int* rows, int norm,
                           float alpha, const float* weight, const float* bias, void* out, int out_dtype, cudaStream_t stream) {
  if (n_out == 0 || width == 0) return TIB_OK;
  if (!streams || n_out < 0 || width < 0 || S < 1 || S > kMaxStreams) return TIB_E_SIZE;
  if (y && (!mix || !out_w)) return TIB_E_ARG;
  if (in_w && !out) return TIB_E_ARG;
  if (!y && !in_w) return TIB_OK;
  if (norm != 0 && norm != 1) return TIB_E_ARG;
  if (norm == 1 && (!weight || !bias)) return TIB_E_ARG;
  if (in_w && norm == 0 && out_dtype != TIB_F32) return TIB_E_DTYPE;
  if ((y && y_dtype != TIB_F32 && y_dtype != TIB_BF16) || (in_w && out_dtype != TIB_F32 && out_dtype != TIB_BF16)) return TIB_E_DTYPE;
  HyperArgs a;
  a.streams = streams; a.stream_stride = stream_stride; a.S = S; a.width = width; a.y = y; a.y_dtype = y_dtype; a.ldy = ldy;
  a.mix = mix; a.out_w = out_w; a.in_w = in_w; a.rows = rows; a.norm = norm; a.alpha = alpha; a.weight = weight; a.bias = bias;
  a.out = out; a.out_dtype = out_dtype;
  // sixteen bytes a load where every row of every array starts on such a boundary
  const int64_t ybytes = y_dtype == TIB_F32 ? 4 : 2, obytes = out_dtype == TIB_F32 ? 4 : 2;
  const bool vec = width % 4 == 0 && stream_stride % 4 == 0 && ((uintptr_t)streams & 15) == 0 &&
                   (!y || ((ldy * ybytes) % 8 == 0 && ((uintptr_t)y & 15) == 0)) && (!in_w || ((uintptr_t)out & 15) == 0) &&
                   (norm == 0 || (((uintptr_t)weight | (uintptr_t)bias) & 15) == 0) && obytes > 0;
  const int per = vec ? 4 : 1;
  const int threads = width / per >= 256 ? 256 : 128;
  // (few rows: a row's columns are spread over several blocks)
  const dim3 grid(n_out, n_out < 2 * 148 ? ceil_div(width, threads * per) : 1);
  switch (S) {
#define TIB_HYPER_CASE(N)                                                                       \
  case N:                                                                                       \
    if (vec) TIB_LAUNCH_DEPENDENT((hyper_step_kernel<N, 4>), grid, threads, 0, stream, a);      \
    else TIB_LAUNCH_DEPENDENT((hyper_step_kernel<N, 1>), grid, threads, 0, stream, a);          \
    break
    TIB_HYPER_CASE(1); TIB_HYPER_CASE(2); TIB_HYPER_CASE(3); TIB_HYPER_CASE(4);
    TIB_HYPER_CASE(5); TIB_HYPER_CASE(6); TIB_HYPER_CASE(7); TIB_HYPER_CASE(8);
#undef TIB_HYPER_CASE
  }
  return TIB_OK;
}
