// A routed feed-forward (mixture of experts): which experts a token uses, the tokens
// sorted by expert, the experts' products over those groups of rows, the gated
// activation with clamps, and the weighted sum back into the residual stream.
//
//   route_topk     scores = softmax(router logits) over all experts (32-bit); the experts
//                  form equal groups of neighbours, a group's score is its largest expert
//                  score, only experts of the `keep` best groups are eligible, the `top`
//                  largest eligible scores are chosen; ties go to the lower index.  The
//                  weights are the chosen scores as they are, or divided by their sum.
//   route_plan     counting sort of the (token, choice) pairs by expert: each pair's row in
//                  the sorted order, each row's token, each expert's first row, and the list
//                  of row tiles (expert, first row) that the grouped products walk.
//   gather_rows    the tokens' activations in sorted order.
//   gemm_grouped   out[r] = A[r] W[expert(r)]^T with 32-bit FMA (one sequential chain per
//                  output, as gemm_simt.cu).
//   glu_clamp      y = g' sigmoid(alpha g') (u' + shift), g' = min(g, limit),
//                  u' = clamp(u, -limit, limit); limit <= 0: no clamps.
//   routed_combine x[t] += sum_j w[t, j] y[row(t, j)], in the order of j.
//
// Nothing here depends on the order in which blocks run: a pair's row inside its expert's
// group may differ from run to run, but every row is computed on its own and summed by
// token in a fixed order.
#include "api.h"
#include "common.cuh"

namespace yalm {

constexpr int RT_WARPS = 4;

// What differs between designs is a parameter: `sigmoid` (scores = sigmoid(z) instead of the softmax
// over all experts), `correction` (a stored offset per expert that is added to the scores for the
// CHOICE of groups and experts only; the weights use the scores themselves), `group_top2` (a group's
// score is the sum of its two best choice scores instead of its best one), `norm_eps` (added to the
// sum the chosen scores are divided by) and `weight_scale` (a factor on the final weights).  Choice
// scores may be negative, so "not eligible" and "taken" are minus infinity.
struct RouteRule {
  int sigmoid, group_top2, renormalise;
  float norm_eps, weight_scale;
  const float* correction;
};

__global__ void __launch_bounds__(RT_WARPS * 32)
route_topk_kernel(const float* __restrict__ z, int n_partials, long long partial_stride,
                  int n_tokens, int E, int n_groups, int keep, int top, RouteRule rule,
                  int* __restrict__ choice, float* __restrict__ weight, int* __restrict__ counts) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float rt_smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * RT_WARPS + warp;
  if (t >= n_tokens) return;
  float* score = rt_smem + (size_t)warp * (3 * E + n_groups);     // the scores the weights are made of
  float* pick = score + E;                                        // the scores the choice goes by
  float* cand = pick + E;                                         // pick of the eligible experts, taken ones removed
  float* gbest = cand + E;
  const int per = E / n_groups;

  float m = -INFINITY;
  for (int e = lane; e < E; e += 32) {
    const float v = sum_slices(z + (size_t)t * E + e, n_partials, partial_stride);
    score[e] = v;
    m = fmaxf(m, v);
  }
  if (rule.sigmoid) {
    for (int e = lane; e < E; e += 32) score[e] = 1.0f / (1.0f + expf(-score[e]));
  } else {
    m = warp_max(m);
    float sum = 0.f;
    for (int e = lane; e < E; e += 32) {
      const float p = expf(score[e] - m);
      score[e] = p;
      sum += p;
    }
    sum = warp_sum(sum);
    for (int e = lane; e < E; e += 32) score[e] = score[e] / sum;
  }
  for (int e = lane; e < E; e += 32) {
    pick[e] = score[e] + (rule.correction != nullptr ? rule.correction[e] : 0.f);
    cand[e] = -INFINITY;
  }
  __syncwarp();
  for (int g = lane; g < n_groups; g += 32) {
    float b = -INFINITY, b2 = -INFINITY;                          // the group's best and second best
    for (int i = 0; i < per; ++i) {
      const float v = pick[g * per + i];
      if (v > b) { b2 = b; b = v; }
      else if (v > b2) b2 = v;
    }
    gbest[g] = (rule.group_top2 && per > 1) ? b + b2 : b;
  }
  __syncwarp();
  // the `keep` best groups, one at a time: (largest score, lowest index)
  for (int r = 0; r < keep; ++r) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int g = lane; g < n_groups; g += 32)
      if (gbest[g] > bv) { bv = gbest[g]; bi = g; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (bi < n_groups) {
      for (int i = lane; i < per; i += 32) cand[bi * per + i] = pick[bi * per + i];
      if (lane == 0) gbest[bi] = -INFINITY;
    }
    __syncwarp();
  }
  float wsum = 0.f;
  for (int j = 0; j < top; ++j) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int e = lane; e < E; e += 32)
      if (cand[e] > bv) { bv = cand[e]; bi = e; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (bi >= E) bi = 0;                    // fewer eligible experts than `top`: refused on the host
    const float sv = score[bi];
    wsum += sv;
    if (lane == 0) {
      choice[(size_t)t * top + j] = bi;
      weight[(size_t)t * top + j] = sv;
      atomicAdd(&counts[bi], 1);
      cand[bi] = -INFINITY;
    }
    __syncwarp();
  }
  if (lane == 0) {
    if (rule.renormalise)
      for (int j = 0; j < top; ++j) weight[(size_t)t * top + j] /= (wsum + rule.norm_eps);
    if (rule.weight_scale != 1.0f)
      for (int j = 0; j < top; ++j) weight[(size_t)t * top + j] *= rule.weight_scale;
  }
}

// One block.  counts [E] comes in as the number of pairs per expert and leaves as zeros.
__global__ void __launch_bounds__(1024)
route_plan_kernel(int* __restrict__ counts, const int* __restrict__ choice, int n_pairs, int top,
                  int E, int tile_rows, int* __restrict__ first_row, int* __restrict__ pair_row,
                  int* __restrict__ row_token, int* __restrict__ tile_expert,
                  int* __restrict__ tile_row0, int* __restrict__ n_tiles) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ int rp_smem[];
  int* cursor = rp_smem;                   // [E]
  int* first_tile = rp_smem + E;           // [E + 1]
  int* first_s = first_tile + E + 1;       // [E + 1]
  if (threadIdx.x == 0) {
    int rows = 0, tiles = 0;
    for (int e = 0; e < E; ++e) {
      first_s[e] = rows;
      first_tile[e] = tiles;
      rows += counts[e];
      tiles += (counts[e] + tile_rows - 1) / tile_rows;
    }
    first_s[E] = rows;
    first_tile[E] = tiles;
    *n_tiles = tiles;
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= E; e += blockDim.x) first_row[e] = first_s[e];
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    cursor[e] = 0;
    const int t0 = first_tile[e], t1 = first_tile[e + 1];
    for (int i = t0; i < t1; ++i) {
      tile_expert[i] = e;
      tile_row0[i] = first_s[e] + (i - t0) * tile_rows;
    }
  }
  __syncthreads();
  for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
    const int e = choice[p];
    const int row = first_s[e] + atomicAdd(&cursor[e], 1);
    pair_row[p] = row;
    row_token[row] = p / top;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) counts[e] = 0;
}

template <typename T>
__global__ void gather_rows_kernel(const T* __restrict__ src, const int* __restrict__ row_token,
                                   T* __restrict__ dst, int dim, int vec) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x;
  const T* s = src + (size_t)row_token[r] * dim;
  T* d = dst + (size_t)r * dim;
  if (vec) {
    constexpr int EPV = 16 / sizeof(T);
    for (int i = threadIdx.x; i < dim / EPV; i += blockDim.x)
      reinterpret_cast<uint4*>(d)[i] = reinterpret_cast<const uint4*>(s)[i];
  } else {
    for (int i = threadIdx.x; i < dim; i += blockDim.x) d[i] = s[i];
  }
}

constexpr int GG_BM = 64, GG_BN = 64, GG_BK = 16;

// A [rows, K] in sorted order, W [E][N][K], out [rows, N]; a block takes one tile of the
// plan (rows of one expert) and 64 output features.
template <typename TA, typename TW, typename TO>
__global__ void __launch_bounds__(256)
gemm_grouped_kernel(const TA* __restrict__ A, const TW* __restrict__ W, TO* __restrict__ out,
                    const int* __restrict__ first_row, const int* __restrict__ tile_expert,
                    const int* __restrict__ tile_row0, const int* __restrict__ n_tiles, int N, int K) {
  pdl_launch_dependents();
  pdl_wait();
  if ((int)blockIdx.y >= *n_tiles) return;
  __shared__ float As[GG_BK][GG_BM + 4];
  __shared__ float Ws[GG_BK][GG_BN + 4];
  const int e = tile_expert[blockIdx.y];
  const int m0 = tile_row0[blockIdx.y];
  const int M = first_row[e + 1];                      // rows of this expert end here
  W += (size_t)e * N * K;
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
  const int n0 = blockIdx.x * GG_BN;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  for (int k0 = 0; k0 < K; k0 += GG_BK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int idx = threadIdx.x + i * 256;
      const int r = idx / GG_BK, c = idx % GG_BK;
      const int gm = m0 + r, gn = n0 + r, gk = k0 + c;
      As[c][r] = (gm < M && gk < K) ? to_float(A[(size_t)gm * K + gk]) : 0.f;
      Ws[c][r] = (gn < N && gk < K) ? to_float(W[(size_t)gn * K + gk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < GG_BK; ++k) {
      float a[4], w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[k][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) w[j] = Ws[k][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int gm = m0 + ty * 4 + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gn = n0 + tx * 4 + j;
      if (gn < N) out[(size_t)gm * N + gn] = from_float<TO>(acc[i][j]);
    }
  }
}

// gu [S][rows][2F] float32 -> out [rows][F]; gu's columns are (gate | up) or, with `paired`,
// groups of 16 gate columns each followed by the 16 up columns of the same features.  A block
// row per matrix row (blockIdx.x), VEC features per thread (4 when F is a multiple of 4).
template <typename TO, int VEC>
__global__ void glu_clamp_kernel(const float* __restrict__ gu, int n_partials, long long partial_stride,
                                 TO* __restrict__ out, int F, float alpha, float limit, float shift,
                                 int paired) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t r = blockIdx.x;
  const int f = (blockIdx.y * blockDim.x + threadIdx.x) * VEC;
  if (f >= F) return;
  const int gc = paired ? (f >> 4) * 32 + (f & 15) : f;          // the gate column of feature f
  const int up_at = paired ? 16 : F;                             // its up column lies this far on
  const float* p = gu + r * 2 * F + gc;
  float g[VEC], u[VEC];
#pragma unroll
  for (int v = 0; v < VEC; ++v) { g[v] = 0.f; u[v] = 0.f; }
  for (int s = 0; s < n_partials; ++s) {
    const float* q = p + (size_t)s * partial_stride;
    if (VEC == 4) {
      const float4 a = *reinterpret_cast<const float4*>(q), b = *reinterpret_cast<const float4*>(q + up_at);
      g[0] += a.x; g[VEC > 1 ? 1 : 0] += a.y; g[VEC > 2 ? 2 : 0] += a.z; g[VEC > 3 ? 3 : 0] += a.w;
      u[0] += b.x; u[VEC > 1 ? 1 : 0] += b.y; u[VEC > 2 ? 2 : 0] += b.z; u[VEC > 3 ? 3 : 0] += b.w;
    } else {
      g[0] += q[0];
      u[0] += q[up_at];
    }
  }
#pragma unroll
  for (int v = 0; v < VEC; ++v) {
    float gg = g[v], uu = u[v];
    if (limit > 0.f) {
      gg = fminf(gg, limit);
      uu = fminf(fmaxf(uu, -limit), limit);
    }
    out[r * F + f + v] = from_float<TO>(gg * (1.0f / (1.0f + expf(-alpha * gg))) * (uu + shift));
  }
}

constexpr int RC_MAX_TOP = 256;

__global__ void routed_combine_kernel(float* __restrict__ x, const float* __restrict__ y,
                                      const int* __restrict__ pair_row, const float* __restrict__ weight,
                                      int top, int dim) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  __shared__ int row_s[RC_MAX_TOP];
  __shared__ float w_s[RC_MAX_TOP];
  for (int j = threadIdx.x; j < top; j += blockDim.x) {
    row_s[j] = pair_row[(size_t)t * top + j];
    w_s[j] = weight[(size_t)t * top + j];
  }
  __syncthreads();
  // the rows of up to eight choices are loaded together, then added in the order of the choices
  if (dim % 4 == 0) {
    for (int i = threadIdx.x * 4; i < dim; i += blockDim.x * 4) {
      float4 v = *reinterpret_cast<const float4*>(x + (size_t)t * dim + i);
      for (int j0 = 0; j0 < top; j0 += 8) {
        float4 r[8];
#pragma unroll
        for (int j = 0; j < 8; ++j)
          r[j] = j0 + j < top ? *reinterpret_cast<const float4*>(y + (size_t)row_s[j0 + j] * dim + i)
                              : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (j0 + j < top) {
            const float w = w_s[j0 + j];
            v.x = fmaf(w, r[j].x, v.x); v.y = fmaf(w, r[j].y, v.y);
            v.z = fmaf(w, r[j].z, v.z); v.w = fmaf(w, r[j].w, v.w);
          }
      }
      *reinterpret_cast<float4*>(x + (size_t)t * dim + i) = v;
    }
    return;
  }
  for (int i = threadIdx.x; i < dim; i += blockDim.x) {
    float v = x[(size_t)t * dim + i];
    for (int j0 = 0; j0 < top; j0 += 8) {
      float r[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) r[j] = j0 + j < top ? y[(size_t)row_s[j0 + j] * dim + i] : 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (j0 + j < top) v = fmaf(w_s[j0 + j], r[j], v);
    }
    x[(size_t)t * dim + i] = v;
  }
}

}  // namespace yalm

using namespace yalm;

// z: router logits as n_partials float32 slices [n_tokens, E].  choice / weight [n_tokens, top];
// counts [E] int32, zero before the call: pairs per expert afterwards.
extern "C" int yalm_route_topk(const float* z, int n_partials, long long partial_stride, int n_tokens,
                               int E, int n_groups, int keep, int top, int renormalise, int sigmoid,
                               int group_top2, float norm_eps, float weight_scale, const float* correction,
                               int* choice, float* weight, int* counts, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (E <= 0 || n_groups <= 0 || E % n_groups || keep <= 0 || keep > n_groups || top <= 0 ||
      top > keep * (E / n_groups))
    return -2;
  const size_t smem = (size_t)RT_WARPS * (3 * E + n_groups) * sizeof(float);
  if (smem > 48 * 1024) return -2;
  const RouteRule rule = {sigmoid, group_top2, renormalise, norm_eps, weight_scale, correction};
  launch_pdl(route_topk_kernel, dim3((n_tokens + RT_WARPS - 1) / RT_WARPS), dim3(RT_WARPS * 32), smem,
             stream, z, n_partials, partial_stride, n_tokens, E, n_groups, keep, top, rule, choice,
             weight, counts);
  YALM_LAUNCH_CHECK();
  return 0;
}

// first_row [E + 1], pair_row / row_token [n_pairs], tile_expert / tile_row0
// [ceil(n_pairs / tile_rows) + E], n_tiles [1]; counts is zero again afterwards.
extern "C" int yalm_route_plan(int* counts, const int* choice, int n_pairs, int top, int E,
                               int tile_rows, int* first_row, int* pair_row, int* row_token,
                               int* tile_expert, int* tile_row0, int* n_tiles, cudaStream_t stream) {
  if (n_pairs <= 0) return 0;
  if (E <= 0 || top <= 0 || tile_rows <= 0) return -2;
  const size_t smem = (size_t)(3 * E + 2) * sizeof(int);
  if (smem > 48 * 1024) return -2;
  launch_pdl(route_plan_kernel, dim3(1), dim3(1024), smem, stream, counts, choice, n_pairs, top, E,
             tile_rows, first_row, pair_row, row_token, tile_expert, tile_row0, n_tiles);
  YALM_LAUNCH_CHECK();
  return 0;
}

extern "C" int yalm_gather_rows(const void* src, const int* row_token, void* dst, int dtype, int rows,
                                int dim, cudaStream_t stream) {
  if (rows <= 0) return 0;
  const int esz = dtype == DT_F32 ? 4 : 2;
  const int vec = (dim * esz) % 16 == 0 && (((uintptr_t)src | (uintptr_t)dst) & 15) == 0;
  if (dtype == DT_F32)
    launch_pdl(gather_rows_kernel<float>, dim3(rows), dim3(128), 0, stream, (const float*)src, row_token,
               (float*)dst, dim, vec);
  else if (dtype == DT_BF16 || dtype == DT_F16)
    launch_pdl(gather_rows_kernel<uint16_t>, dim3(rows), dim3(128), 0, stream, (const uint16_t*)src,
               row_token, (uint16_t*)dst, dim, vec);
  else
    return -3;
  YALM_LAUNCH_CHECK();
  return 0;
}

namespace yalm {
template <typename TA, typename TW>
static int launch_grouped(const void* A, const void* W, void* out, int out_dtype, const int* first_row,
                          const int* tile_expert, const int* tile_row0, const int* n_tiles,
                          int max_tiles, int N, int K, cudaStream_t stream) {
  const dim3 grid((N + GG_BN - 1) / GG_BN, max_tiles);
  if (max_tiles > 65535) return -4;
#define YALM_GG(TO)                                                                                 \
  launch_pdl(gemm_grouped_kernel<TA, TW, TO>, grid, dim3(256), 0, stream, (const TA*)A, (const TW*)W, \
             (TO*)out, first_row, tile_expert, tile_row0, n_tiles, N, K)
  if (out_dtype == DT_F32) YALM_GG(float);
  else if (out_dtype == DT_BF16) YALM_GG(__nv_bfloat16);
  else if (out_dtype == DT_F16) YALM_GG(__half);
  else return -3;
#undef YALM_GG
  YALM_LAUNCH_CHECK();
  return 0;
}
}  // namespace yalm

// out[r] = A[r] W[e]^T for the rows r of every expert e, over the tiles of a plan made with
// tile_rows = 64.  max_tiles bounds the plan's tile count (it sizes the grid).
extern "C" int yalm_gemm_grouped(const void* A, int a_dtype, const void* W, int w_dtype, void* out,
                                 int out_dtype, const int* first_row, const int* tile_expert,
                                 const int* tile_row0, const int* n_tiles, int max_tiles, int N, int K,
                                 cudaStream_t stream) {
  if (max_tiles <= 0 || N <= 0) return 0;
  if (K <= 0) return -2;
#define YALM_GGD(TA, TW)                                                                             \
  return launch_grouped<TA, TW>(A, W, out, out_dtype, first_row, tile_expert, tile_row0, n_tiles,    \
                                max_tiles, N, K, stream)
  if (a_dtype == DT_F32 && w_dtype == DT_F32) YALM_GGD(float, float);
  if (a_dtype == DT_BF16 && w_dtype == DT_BF16) YALM_GGD(__nv_bfloat16, __nv_bfloat16);
  if (a_dtype == DT_F16 && w_dtype == DT_F16) YALM_GGD(__half, __half);
  if (a_dtype == DT_F32 && w_dtype == DT_BF16) YALM_GGD(float, __nv_bfloat16);
  if (a_dtype == DT_F32 && w_dtype == DT_F16) YALM_GGD(float, __half);
#undef YALM_GGD
  return -3;
}

extern "C" int yalm_glu_clamp(const float* gu, int n_partials, long long partial_stride, void* out,
                              int out_dtype, long long rows, int F, float alpha, float limit, float shift,
                              int paired, cudaStream_t stream) {
  if (paired && F % 16 != 0) return -2;
  if (rows <= 0 || F <= 0) return 0;
  if (rows > 0x7fffffffLL) return -4;
  const bool vec = F % 4 == 0 && partial_stride % 4 == 0 && ((uintptr_t)gu & 15) == 0;
  const int per_block = 128 * (vec ? 4 : 1);
  const dim3 grid((unsigned)rows, (F + per_block - 1) / per_block);
  if (grid.y > 65535) return -4;
#define YALM_GC(TO)                                                                                  \
  do {                                                                                               \
    if (vec) launch_pdl(glu_clamp_kernel<TO, 4>, grid, dim3(128), 0, stream, gu, n_partials,         \
                        partial_stride, (TO*)out, F, alpha, limit, shift, paired);                   \
    else launch_pdl(glu_clamp_kernel<TO, 1>, grid, dim3(128), 0, stream, gu, n_partials,             \
                    partial_stride, (TO*)out, F, alpha, limit, shift, paired);                       \
  } while (0)
  if (out_dtype == DT_F32) YALM_GC(float);
  else if (out_dtype == DT_BF16) YALM_GC(__nv_bfloat16);
  else if (out_dtype == DT_F16) YALM_GC(__half);
  else return -3;
#undef YALM_GC
  YALM_LAUNCH_CHECK();
  return 0;
}

extern "C" int yalm_routed_combine(float* x, const float* y, const int* pair_row, const float* weight,
                                   int n_tokens, int top, int dim, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (top <= 0 || top > RC_MAX_TOP) return -2;
  launch_pdl(routed_combine_kernel, dim3(n_tokens), dim3(dim >= 1024 ? 256 : 128), 0, stream, x, y,
             pair_row, weight, top, dim);
  YALM_LAUNCH_CHECK();
  return 0;
}
