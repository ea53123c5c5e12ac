// Routed feed-forward (mixture of experts): routing, grouping of (token, choice) pairs by expert, the experts'
// two products over the grouped rows, and the weighted sum back per token.  Nothing here returns to the host:
// every count and offset stays on the device and grids are sized for the worst case, so a step can be captured.
//
//   moe_route    from fp32 router logits [tokens, ld]: softmax over the experts (or sigmoid), the `top` largest
//                scores (lowest index first among equals), their weights = score / (sum of the chosen + norm_eps)
//                (or the bare scores), all fp32; optionally a correction per expert that counts for the choice only, and
//                groups of neighbouring experts of which only the best few may be chosen from
//   moe_group    counting sort of the tokens * top pairs by expert: offsets [experts + 1], order[sorted] = pair,
//                place[pair] = sorted index.  The order inside an expert may differ from run to run; every row
//                of a product is computed by itself, so no value depends on it
//   moe_expert_product   y[s] = act(x[src(s)] . W_e^T) for the sorted rows s of expert e; W: [experts, n, k];
//                act: none, relu^2, silu, or a clamped gated unit over (gate, up) row pairs of W (row 2i = gate i,
//                row 2i + 1 = up i): g = min(g, limit), u = clamp(u, -limit, limit), y_i = g * sigmoid(alpha * g) * (u + 1),
//                or the plain gated unit y_i = silu(g) * u over the same pairs; either leaves n / 2 columns.  `row_scale` (per pair, may be null) multiplies the fp32 sums before the
//                activation: a router weight that belongs on the expert's input.  bf16 operands whose rows are 16-byte aligned run on the tensor cores
//                (mma.sync m16n8k16, fp32 accumulation, cp.async double buffering); everything else, and the
//                32-bit path, on fp32 FMAs in fixed k order
//   moe_combine  out[t] = sum_k weight[t, k] * y[place[t * top + k]]  (+ sigmoid(gate[t]) * shared[t]); weights may be null (1);
//                a choice whose id is `identity_from` or above has no expert: it adds weight * x[t], the input itself
#include "mma.cuh"

namespace tib {

// ----------------------------------------------------------- router logits
// out[t, e] = x[t] . w[e] in fp32 for a handful of rows w (the router, perhaps a gate row behind it): one warp per
// row and group of tokens, lanes stride over k (eight at a time where rows are 16-byte aligned), then a butterfly sum per
// token: the order of every sum is fixed by k and the alignment alone, so a token's logits do not depend on what else is
// in the step.  (The general fp32 product gives a product
// this narrow to a single block.)
// A block takes kRouterTokens tokens, so that a row of w read from the L2 serves several of them.  With 16-byte aligned
// rows (VEC) a lane takes eight consecutive k at a time: 16 bytes of a bf16 token row, 32 bytes of w.
constexpr int kRouterTokens = 4;

__device__ __forceinline__ void load8(const float* p, float (&v)[8]) {
  const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  const float2 a = bf16x2_floats(*reinterpret_cast<const __nv_bfloat162*>(&raw.x)), b = bf16x2_floats(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
  const float2 c = bf16x2_floats(*reinterpret_cast<const __nv_bfloat162*>(&raw.z)), d = bf16x2_floats(*reinterpret_cast<const __nv_bfloat162*>(&raw.w));
  v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y; v[4] = c.x; v[5] = c.y; v[6] = d.x; v[7] = d.y;
}

template <typename TX, bool VEC>
__global__ void __launch_bounds__(256)
router_logits_kernel(const TX* __restrict__ x, int64_t ldx, const float* __restrict__ w, float* __restrict__ out, int64_t ldo,
                     int tokens, int rows, int K) {
  pdl_wait();
  pdl_trigger();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int t0 = blockIdx.x * kRouterTokens;
  const int nt = min(kRouterTokens, tokens - t0);
  const int K8 = VEC ? (K / 8) * 8 : 0;
  for (int e = warp + blockIdx.y * nwarps; e < rows; e += nwarps * gridDim.y) {
    const float* wr = w + (size_t)e * K;
    float acc[kRouterTokens];
#pragma unroll
    for (int i = 0; i < kRouterTokens; ++i) acc[i] = 0.f;
    if (VEC) {
      for (int k = lane * 8; k < K8; k += 256) {
        float wv[8];
        load8(wr + k, wv);
#pragma unroll
        for (int i = 0; i < kRouterTokens; ++i) {
          if (i >= nt) continue;
          float xv[8];
          load8(x + (size_t)(t0 + i) * ldx + k, xv);
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[i] = fmaf(xv[j], wv[j], acc[i]);
        }
      }
    }
    for (int k = K8 + lane; k < K; k += 32) {
      const float wv = wr[k];
#pragma unroll
      for (int i = 0; i < kRouterTokens; ++i)
        if (i < nt) acc[i] = fmaf(to_f32(x[(size_t)(t0 + i) * ldx + k]), wv, acc[i]);
    }
#pragma unroll
    for (int i = 0; i < kRouterTokens; ++i) {
      const float v = warp_sum(acc[i]);
      if (lane == 0 && i < nt) out[(size_t)(t0 + i) * ldo + e] = v;
    }
  }
}

// ------------------------------------------------------------------- route
// One warp per token.  score(e) = softmax(z)[e] or sigmoid(z[e]); the choice looks at score + correction[e] (when a
// correction is given) and, with `groups` > 1, only at the experts of the `keep` runs of adjacent experts whose best
// corrected score ranks highest (an expert of another run is not eligible, whatever its score); the weights are made from the
// scores without the correction.  Lowest index first among equals, for groups and for experts.
constexpr int kRouteMaxGroups = 64;      // (two groups a lane)

__global__ void __launch_bounds__(128)
moe_route_kernel(const float* __restrict__ logits, int64_t ld, int experts, int top, int sigmoid_scores,
                 int normalize, float norm_eps, const float* __restrict__ correction, int groups, int keep,
                 int* __restrict__ ids, float* __restrict__ weights, int tokens) {
  pdl_wait();
  pdl_trigger();
  __shared__ unsigned char kept_s[4][kRouteMaxGroups];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int t = blockIdx.x * (blockDim.x >> 5) + warp;
  if (t >= tokens) return;
  const float* z = logits + (size_t)t * ld;
  float mx = -CUDART_INF_F;
  for (int e = lane; e < experts; e += 32) mx = fmaxf(mx, z[e]);
  mx = warp_max(mx);
  float sum = 0.f;
  for (int e = lane; e < experts; e += 32) sum += expf(z[e] - mx);
  sum = warp_sum(sum);
  auto score = [&](int e) { return sigmoid_scores ? 1.f / (1.f + expf(-z[e])) : expf(z[e] - mx) / sum; };
  const bool grouped = groups > 1 && keep < groups;
  const int per_group = grouped ? experts / groups : experts;
  if (grouped) {
    float gscore[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int g = lane + 32 * i;
      gscore[i] = -CUDART_INF_F;
      if (g < groups) {
        kept_s[warp][g] = 0;
        for (int e = g * per_group; e < (g + 1) * per_group; ++e)
          gscore[i] = fmaxf(gscore[i], score(e) + (correction ? correction[e] : 0.f));
      }
    }
    __syncwarp();
    unsigned taken = 0u;
    for (int k = 0; k < keep; ++k) {
      float best = -CUDART_INF_F;
      int best_g = 0x7fffffff;
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int g = lane + 32 * i;
        if (g < groups && !((taken >> i) & 1u) && (gscore[i] > best || best_g == 0x7fffffff)) { best = gscore[i]; best_g = g; }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int og = __shfl_xor_sync(0xffffffffu, best_g, o);
        if (og != 0x7fffffff && (best_g == 0x7fffffff || ob > best || (ob == best && og < best_g))) { best = ob; best_g = og; }
      }
      if (best_g < groups) {
        if ((best_g & 31) == lane) { taken |= 1u << (best_g >> 5); kept_s[warp][best_g] = 1; }
      }
    }
    __syncwarp();
  }
  float chosen_sum = 0.f;
  unsigned long long taken_lo = 0ull;    // lane-local mask over this lane's experts (e = lane + 32 * i, i < 64)
  for (int k = 0; k < top; ++k) {
    float best = -CUDART_INF_F, best_s = 0.f;
    int best_e = 0x7fffffff;
    for (int e = lane, i = 0; e < experts; e += 32, ++i) {
      if ((taken_lo >> i) & 1ull) continue;
      if (grouped && !kept_s[warp][e / per_group]) continue;
      const float s = score(e);
      const float c = s + (correction ? correction[e] : 0.f);
      if (c > best || best_e == 0x7fffffff) { best = c; best_s = s; best_e = e; }     // (rising e: the lowest index wins among equals)
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const float os = __shfl_xor_sync(0xffffffffu, best_s, o);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (oe != 0x7fffffff && (best_e == 0x7fffffff || ob > best || (ob == best && oe < best_e))) { best = ob; best_s = os; best_e = oe; }
    }
    if ((best_e & 31) == lane && best_e < experts) taken_lo |= 1ull << (best_e >> 5);
    chosen_sum += best_s;
    if (lane == 0) { ids[(size_t)t * top + k] = best_e < experts ? best_e : -1; weights[(size_t)t * top + k] = best_e < experts ? best_s : 0.f; }
  }
  __syncwarp();
  if (normalize && lane < top) weights[(size_t)t * top + lane] /= (chosen_sum + norm_eps);
  if (normalize) for (int k = lane + 32; k < top; k += 32) weights[(size_t)t * top + k] /= (chosen_sum + norm_eps);
}

// ------------------------------------------------------------------- group
// One block.  counts in shared memory (experts <= 1024), exclusive scan by one warp, then placement with atomics.
__global__ void __launch_bounds__(1024)
moe_group_kernel(const int* __restrict__ ids, int pairs, int experts, int* __restrict__ offsets, int* __restrict__ order,
                 int* __restrict__ place) {
  pdl_wait();
  pdl_trigger();
  __shared__ int count[1024];
  __shared__ int cursor[1024];
  for (int e = threadIdx.x; e < experts; e += blockDim.x) count[e] = 0;
  __syncthreads();
  for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
    const int e = ids[p];
    if (e >= 0 && e < experts) atomicAdd(&count[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int e = 0; e < experts; ++e) { offsets[e] = run; cursor[e] = run; run += count[e]; }
    offsets[experts] = run;
  }
  __syncthreads();
  for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
    const int e = ids[p];
    if (e >= 0 && e < experts) {
      const int s = atomicAdd(&cursor[e], 1);
      order[s] = p;
      place[p] = s;
    } else {
      place[p] = -1;
    }
  }
}

// ---------------------------------------------------------------- products
constexpr int GM = 64, GN = 64, GK = 16;
enum MoeAct : int { MOE_ACT_NONE = 0, MOE_ACT_RELU2 = 1, MOE_ACT_SILU = 2, MOE_ACT_GLU_CLAMP = 3, MOE_ACT_SWIGLU = 4 };

struct MoeEpilogue {
  int act;
  float limit, alpha;          // of the clamped gated unit
  const float* row_scale;      // [pairs] or null: sorted row s is multiplied by row_scale[order[s]] before the activation
};

__device__ __forceinline__ float moe_act(float v, int act) {
  if (act == MOE_ACT_RELU2) { v = fmaxf(v, 0.f); return v * v; }
  if (act == MOE_ACT_SILU) return v / (1.f + expf(-v));
  return v;
}
// the gated units over (gate, up) row pairs: clamped (see above), or silu(g) * u
__device__ __forceinline__ float moe_gated(float g, float u, int act, float limit, float alpha) {
  if (act == MOE_ACT_SWIGLU) return g / (1.f + expf(-g)) * u;
  g = fminf(g, limit);
  u = fminf(fmaxf(u, -limit), limit);
  return g / (1.f + expf(-alpha * g)) * (u + 1.f);
}

// Row tile `blockIdx.y` counts tiles of GM sorted rows expert by expert; it finds its expert by walking offsets.
// x_by_pair: source row of sorted row s is order[s] / top (the token), else s itself (rows already sorted).
template <typename TX, typename TW, typename TO>
__global__ void __launch_bounds__(256)
moe_expert_product_kernel(const TX* __restrict__ x, int64_t ldx, const TW* __restrict__ w, TO* __restrict__ y, int64_t ldy,
                          const int* __restrict__ offsets, const int* __restrict__ order, int experts, int top,
                          int x_by_pair, int N, int K, MoeEpilogue ep) {
  pdl_wait();
  pdl_trigger();
  __shared__ float xs[GK][GM + 4];
  __shared__ float ws[GK][GN + 4];
  __shared__ int src_row[GM];
  __shared__ int tile_info[3];     // expert, first sorted row, rows
  if (threadIdx.x == 0) {
    int tile = blockIdx.y, e = 0, found = -1, first = 0, rows = 0;
    for (; e < experts; ++e) {
      const int lo = offsets[e], n = offsets[e + 1] - lo;
      const int tiles = (n + GM - 1) / GM;
      if (tile < tiles) { found = e; first = lo + tile * GM; rows = min(GM, n - tile * GM); break; }
      tile -= tiles;
    }
    tile_info[0] = found; tile_info[1] = first; tile_info[2] = rows;
  }
  __syncthreads();
  const int expert = tile_info[0], first = tile_info[1], rows = tile_info[2];
  if (expert < 0) return;
  const int tid = threadIdx.x;
  if (tid < GM) src_row[tid] = tid < rows ? (x_by_pair ? order[first + tid] / top : first + tid) : -1;
  __syncthreads();
  const TW* we = w + (size_t)expert * N * K;
  const int tx = tid & 15, ty = tid >> 4;
  const int n0 = blockIdx.x * GN;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  for (int k0 = 0; k0 < K; k0 += GK) {
#pragma unroll
    for (int it = 0; it < 4; ++it) {
      const int e = tid + it * 256;
      const int r = e >> 4, c = e & 15;
      const int gk = k0 + c, gn = n0 + r;
      const int sr = src_row[r];
      xs[c][r] = (sr >= 0 && gk < K) ? to_f32(x[(size_t)sr * ldx + gk]) : 0.f;
      ws[c][r] = (gn < N && gk < K) ? to_f32(we[(size_t)gn * K + gk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < GK; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = xs[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = ws[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = ty * 4 + i;
    if (r >= rows) continue;
    const float rs = ep.row_scale ? ep.row_scale[order[first + r]] : 1.f;
    if (ep.act >= MOE_ACT_GLU_CLAMP) {
#pragma unroll
      for (int j = 0; j < 4; j += 2) {
        const int gn = n0 + tx * 4 + j;
        if (gn + 1 >= N) continue;
        y[(size_t)(first + r) * ldy + (gn >> 1)] = from_f32<TO>(moe_gated(acc[i][j] * rs, acc[i][j + 1] * rs, ep.act, ep.limit, ep.alpha));
      }
      continue;
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gn = n0 + tx * 4 + j;
      if (gn >= N) continue;
      y[(size_t)(first + r) * ldy + gn] = from_f32<TO>(moe_act(acc[i][j] * rs, ep.act));
    }
  }
}

// The same product on tensor cores.  64 x 64 output tile, 4 warps of 32 x 32, k in steps of 32 through two
// shared-memory stages filled by cp.async (rows of x are gathered by their source row as they are fetched).
constexpr int TK = 32, TKP = TK + 8;      // (8 elements of padding: ldmatrix rows fall in different banks)

template <typename TO>
__global__ void __launch_bounds__(128)
moe_expert_product_mma_kernel(const __nv_bfloat16* __restrict__ x, int64_t ldx, const __nv_bfloat16* __restrict__ w,
                              TO* __restrict__ y, int64_t ldy, const int* __restrict__ offsets, const int* __restrict__ order,
                              int experts, int top, int x_by_pair, int N, int K, MoeEpilogue ep) {
  pdl_wait();
  pdl_trigger();
  __shared__ __align__(16) __nv_bfloat16 xs[2][GM][TKP];
  __shared__ __align__(16) __nv_bfloat16 ws[2][GN][TKP];
  __shared__ int src_row[GM];
  __shared__ int tile_info[3];
  if (threadIdx.x == 0) {
    int tile = blockIdx.y, e = 0, found = -1, first = 0, rows = 0;
    for (; e < experts; ++e) {
      const int lo = offsets[e], n = offsets[e + 1] - lo;
      const int tiles = (n + GM - 1) / GM;
      if (tile < tiles) { found = e; first = lo + tile * GM; rows = min(GM, n - tile * GM); break; }
      tile -= tiles;
    }
    tile_info[0] = found; tile_info[1] = first; tile_info[2] = rows;
  }
  __syncthreads();
  const int expert = tile_info[0], first = tile_info[1], rows = tile_info[2];
  if (expert < 0) return;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid < GM) src_row[tid] = tid < rows ? (x_by_pair ? order[first + tid] / top : first + tid) : -1;
  __syncthreads();
  const __nv_bfloat16* we = w + (size_t)expert * N * K;
  const int n0 = blockIdx.x * GN;
  const int wm = (warp >> 1) * 32, wn = (warp & 1) * 32;
  float acc[2][4][4];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[i][j][c] = 0.f;

  // a stage: 64 rows x 32 k of each operand = 256 pieces of 16 bytes each; 128 threads, two pieces of each a thread
  auto fetch = [&](int stage, int k0) {
#pragma unroll
    for (int it = 0; it < 2; ++it) {
      const int piece = tid + it * 128;
      const int r = piece >> 2, c = (piece & 3) * 8;
      const int sr = src_row[r];
      const bool xv = sr >= 0 && k0 + c < K;
      cp_async16(&xs[stage][r][c], x + (size_t)(xv ? sr : 0) * ldx + (xv ? k0 + c : 0), xv);
      const bool wv = n0 + r < N && k0 + c < K;
      cp_async16(&ws[stage][r][c], we + (size_t)(wv ? n0 + r : 0) * K + (wv ? k0 + c : 0), wv);
    }
    cp_async_commit();
  };
  const int steps = (K + TK - 1) / TK;
  fetch(0, 0);
  for (int ks = 0; ks < steps; ++ks) {
    const int stage = ks & 1;
    if (ks + 1 < steps) {
      fetch(stage ^ 1, (ks + 1) * TK);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < TK; kk += 16) {
      uint32_t a[2][4], b[2][4];
#pragma unroll
      for (int i = 0; i < 2; ++i) ldmatrix_x4(a[i], &xs[stage][wm + i * 16 + (lane & 15)][kk + (lane >> 4) * 8]);
#pragma unroll
      for (int j = 0; j < 2; ++j)      // two n-tiles of 8 per ldmatrix: (n 0-7, k lo), (n 0-7, k hi), (n 8-15, k lo), (n 8-15, k hi)
        ldmatrix_x4(b[j], &ws[stage][wn + j * 16 + ((lane >> 4) << 3) + (lane & 7)][kk + ((lane >> 3) & 1) * 8]);
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) mma_bf16(acc[i][j], a[i], b[j >> 1][(j & 1) * 2], b[j >> 1][(j & 1) * 2 + 1]);
    }
    __syncthreads();      // the stage is free for the fetch after next
  }
  const int g = lane >> 2, t = lane & 3;
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int r = wm + i * 16 + g + (c >> 1) * 8;
        const int gn = n0 + wn + j * 8 + 2 * t + (c & 1);
        if (r >= rows || gn >= N) continue;
        const float rs = ep.row_scale ? ep.row_scale[order[first + r]] : 1.f;
        if (ep.act >= MOE_ACT_GLU_CLAMP) {      // (columns 2t and 2t + 1 of a tile sit in one thread: c and c + 1)
          if ((c & 1) == 0 && gn + 1 < N)
            y[(size_t)(first + r) * ldy + (gn >> 1)] = from_f32<TO>(moe_gated(acc[i][j][c] * rs, acc[i][j][c + 1] * rs, ep.act, ep.limit, ep.alpha));
          continue;
        }
        y[(size_t)(first + r) * ldy + gn] = from_f32<TO>(moe_act(acc[i][j][c] * rs, ep.act));
      }
}

// ----------------------------------------------------------------- combine
template <typename TS, typename TO>
__global__ void moe_combine_kernel(const float* __restrict__ y, const int* __restrict__ place, const float* __restrict__ weights,
                                   int top, const TS* __restrict__ shared, const float* __restrict__ gate, int64_t ld_gate,
                                   TO* __restrict__ out, int width, const int* __restrict__ ids, int identity_from,
                                   const TO* __restrict__ x, int64_t ldx) {
  pdl_wait();
  pdl_trigger();
  const size_t t = blockIdx.x;
  const float g = (shared && gate) ? 1.f / (1.f + expf(-gate[t * ld_gate])) : 1.f;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < width; c += gridDim.y * blockDim.x) {
    float v = 0.f;
    for (int k = 0; k < top; ++k) {
      const int s = place[t * top + k];
      if (s >= 0) v = fmaf(weights ? weights[t * top + k] : 1.f, y[(size_t)s * width + c], v);
      else if (ids && ids[t * top + k] >= identity_from) v = fmaf(weights ? weights[t * top + k] : 1.f, to_f32(x[t * ldx + c]), v);
    }
    if (shared) v = fmaf(g, to_f32(shared[t * width + c]), v);
    out[t * width + c] = from_f32<TO>(v);
  }
}

}  // namespace tib

using namespace tib;

// x: [tokens, K] (row stride ldx) float or bf16; w: [rows, K] fp32; out: [tokens, rows] fp32 (row stride ldo)
TIB_API int tib_router_logits(const void* x, int x_dtype, int64_t ldx, const float* w, float* out, int64_t ldo, int tokens,
                              int rows, int K, cudaStream_t stream) {
  if (tokens == 0 || rows == 0) return TIB_OK;
  if (!x || !w || !out || tokens < 0 || rows < 0 || K < 1) return TIB_E_ARG;
  if (tokens > 0x7fffffff / 2) return TIB_E_SIZE;
  int slices = 1;      // few tokens: the rows of w are spread over several blocks a token
  const int groups = ceil_div(tokens, kRouterTokens);
  while (groups * slices < 2 * 148 && slices * 8 < rows) slices *= 2;
  dim3 grid(groups, slices);
  const int64_t xbytes = x_dtype == TIB_F32 ? 4 : 2;
  const bool vec = K % 4 == 0 && (ldx * xbytes) % 16 == 0 && (((uintptr_t)x | (uintptr_t)w) & 15) == 0;
#define TIB_ROUTER_GO(TX, VEC) \
  TIB_LAUNCH_DEPENDENT((router_logits_kernel<TX, VEC>), grid, 256, 0, stream, (const TX*)x, ldx, w, out, ldo, tokens, rows, K)
  if (x_dtype == TIB_F32) { if (vec) TIB_ROUTER_GO(float, true); else TIB_ROUTER_GO(float, false); }
  else if (x_dtype == TIB_BF16) { if (vec) TIB_ROUTER_GO(__nv_bfloat16, true); else TIB_ROUTER_GO(__nv_bfloat16, false); }
#undef TIB_ROUTER_GO
  else
    return TIB_E_DTYPE;
  return TIB_OK;
}

// correction: [experts] fp32 added to the scores for the choice only, or null; groups > 1 with keep < groups: the experts
// are cut into `groups` equal runs of adjacent ones and only members of the best `keep` runs are eligible.
TIB_API int tib_moe_route(const float* logits, int64_t ld, int tokens, int experts, int top, int sigmoid_scores, int normalize,
                          float norm_eps, const float* correction, int groups, int keep, int* ids, float* weights,
                          cudaStream_t stream) {
  if (tokens == 0) return TIB_OK;
  if (!logits || !ids || !weights) return TIB_E_ARG;
  if (experts < 1 || experts > 2048 || top < 1 || top > experts) return TIB_E_SIZE;
  if (groups < 1 || keep < 1 || keep > groups || groups > kRouteMaxGroups || experts % groups) return TIB_E_SIZE;
  if (groups > 1 && keep < groups && top > keep * (experts / groups)) return TIB_E_SIZE;
  TIB_LAUNCH_DEPENDENT(moe_route_kernel, ceil_div(tokens, 4), 128, 0, stream, logits, ld, experts, top, sigmoid_scores, normalize,
                       norm_eps, correction, groups, keep, ids, weights, tokens);
  return TIB_OK;
}

TIB_API int tib_moe_group(const int* ids, int pairs, int experts, int* offsets, int* order, int* place, cudaStream_t stream) {
  if (!ids || !offsets || !order || !place) return TIB_E_ARG;
  if (experts < 1 || experts > 1024 || pairs < 0) return TIB_E_SIZE;
  TIB_LAUNCH_DEPENDENT(moe_group_kernel, 1, 1024, 0, stream, ids, pairs, experts, offsets, order, place);
  return TIB_OK;
}

// x: rows of K (row stride ldx) in x_dtype; w: [experts, N, K] in w_dtype; y: [pairs, N] (row stride ldy) in y_dtype
// ([pairs, N / 2] for the clamped gated unit, whose N is even); row_scale: [pairs] fp32 or null.
TIB_API int tib_moe_expert_product(const void* x, int x_dtype, int64_t ldx, const void* w, int w_dtype, void* y, int y_dtype,
                                   int64_t ldy, const int* offsets, const int* order, int pairs, int experts, int top,
                                   int x_by_pair, int N, int K, int act, float limit, float alpha, const float* row_scale,
                                   cudaStream_t stream) {
  if (pairs == 0 || N == 0) return TIB_OK;
  if (!x || !w || !y || !offsets || !order || pairs < 0 || N < 0 || K < 1 || top < 1) return TIB_E_ARG;
  if (act < MOE_ACT_NONE || act > MOE_ACT_SWIGLU || (act >= MOE_ACT_GLU_CLAMP && N % 2)) return TIB_E_SIZE;
  MoeEpilogue ep;
  ep.act = act; ep.limit = limit; ep.alpha = alpha; ep.row_scale = row_scale;
  const int row_tiles = ceil_div(pairs, GM) + experts;      // at most this many tiles hold a row
  if (row_tiles > 65535) return TIB_E_SIZE;
  dim3 grid(ceil_div(N, GN), row_tiles);
  if (x_dtype == TIB_BF16 && w_dtype == TIB_BF16 && K % 8 == 0 && ldx % 8 == 0 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)w & 15) == 0) {
    if (y_dtype == TIB_BF16)
      TIB_LAUNCH_DEPENDENT(moe_expert_product_mma_kernel<__nv_bfloat16>, grid, 128, 0, stream, (const __nv_bfloat16*)x, ldx,
                           (const __nv_bfloat16*)w, (__nv_bfloat16*)y, ldy, offsets, order, experts, top, x_by_pair, N, K, ep);
    else if (y_dtype == TIB_F32)
      TIB_LAUNCH_DEPENDENT(moe_expert_product_mma_kernel<float>, grid, 128, 0, stream, (const __nv_bfloat16*)x, ldx,
                           (const __nv_bfloat16*)w, (float*)y, ldy, offsets, order, experts, top, x_by_pair, N, K, ep);
    else
      return TIB_E_DTYPE;
    return TIB_OK;
  }
#define TIB_MOE_GO(TX, TW, TO)                                                                                             \
  TIB_LAUNCH_DEPENDENT((moe_expert_product_kernel<TX, TW, TO>), grid, 256, 0, stream, (const TX*)x, ldx, (const TW*)w, (TO*)y, \
                       ldy, offsets, order, experts, top, x_by_pair, N, K, ep)
  if (x_dtype == TIB_F32 && w_dtype == TIB_F32 && y_dtype == TIB_F32) TIB_MOE_GO(float, float, float);
  else if (x_dtype == TIB_BF16 && w_dtype == TIB_BF16 && y_dtype == TIB_BF16) TIB_MOE_GO(__nv_bfloat16, __nv_bfloat16, __nv_bfloat16);
  else if (x_dtype == TIB_BF16 && w_dtype == TIB_BF16 && y_dtype == TIB_F32) TIB_MOE_GO(__nv_bfloat16, __nv_bfloat16, float);
  else return TIB_E_DTYPE;
#undef TIB_MOE_GO
  return TIB_OK;
}

// y: [pairs, width] fp32; shared: [tokens, width] in shared_dtype or null; gate: fp32 logit per token (stride ld_gate) or
// null (the shared rows are added as they are); out: [tokens, width] in out_dtype.  ids [tokens * top] with identity_from
// and x (the experts' input rows, in out_dtype, ldx elements apart): choices of id >= identity_from add weight * x[t].
TIB_API int tib_moe_combine(const float* y, const int* place, const float* weights, int top, const void* shared,
                            int shared_dtype, const float* gate, int64_t ld_gate, void* out, int out_dtype, int tokens,
                            int width, const int* ids, int identity_from, const void* x, int64_t ldx, cudaStream_t stream) {
  if (tokens == 0 || width == 0) return TIB_OK;
  if (!y || !place || !out || top < 1 || (ids && !x)) return TIB_E_ARG;
  const int threads = width >= 1024 ? 256 : 128;
  // (few tokens: a row's columns are spread over several blocks)
  const dim3 grid(tokens, tokens < 2 * 148 ? ceil_div(width, threads) : 1);
#define TIB_COMBINE_GO(TS, TO)                                                                                       \
  TIB_LAUNCH_DEPENDENT((moe_combine_kernel<TS, TO>), grid, threads, 0, stream, y, place, weights, top, (const TS*)shared, gate, \
                       ld_gate, (TO*)out, width, ids, identity_from, (const TO*)x, ldx)
  const int sd = shared ? shared_dtype : out_dtype;
  if (sd == TIB_F32 && out_dtype == TIB_F32) TIB_COMBINE_GO(float, float);
  else if (sd == TIB_BF16 && out_dtype == TIB_BF16) TIB_COMBINE_GO(__nv_bfloat16, __nv_bfloat16);
  else if (sd == TIB_BF16 && out_dtype == TIB_F32) TIB_COMBINE_GO(__nv_bfloat16, float);
  else if (sd == TIB_F32 && out_dtype == TIB_BF16) TIB_COMBINE_GO(float, __nv_bfloat16);
  else return TIB_E_DTYPE;
#undef TIB_COMBINE_GO
  return TIB_OK;
}
