// Several residual copies per token ("hyper-connections"): X [copies][tokens][dim], 32-bit.
// A sublayer reads one mixture of the copies and writes into all of them:
//     u = sum_i a_i X_i,   y = f(norm(u)),   X_j <- sum_i M[i][j] X_i + m b_j y   (all j from the old X)
// One kernel does a sublayer's write and the NEXT sublayer's read and norm in one pass over the
// row (either half may be absent): the write needs nothing but the row's own element of every
// copy, the read's norm needs the whole row, which the block has in registers by then.
//   write: y is the sum of the product's split-K slices; skipped when y is null;
//   read:  u with the weights a; then h = u / sqrt(mean(u^2) + eps) * w in the storage type, or,
//          without a norm weight, u itself as 32-bit floats (the sum of the copies for the output).
#include "api.h"
#include "common.cuh"

namespace yalm {

constexpr int HC_VPT = 8;          // elements of a row a thread keeps (rows of up to 8 x 1024)

// VEC: dim is a multiple of four and every pointer 16-byte aligned; a thread then takes four
// neighbouring features (16-byte accesses), HC_VPT / 4 such groups
template <typename TO, int NS, bool VEC>
__global__ void __launch_bounds__(1024)
hc_step_kernel(float* __restrict__ X, long long copy_stride, const float* __restrict__ y,
               int n_partials, long long partial_stride, const float* __restrict__ mix,
               const float* __restrict__ out_w, float mult, const float* __restrict__ in_w,
               const float* __restrict__ norm_w, float eps, TO* __restrict__ h,
               float* __restrict__ u_out, int dim) {
  pdl_launch_dependents();
  __shared__ float scratch[33];
  __shared__ float m_s[NS * NS], b_s[NS], a_s[NS];
  // the mixing weights are model weights: read before the wait
  if (threadIdx.x < NS * NS && y != nullptr) m_s[threadIdx.x] = mix[threadIdx.x];
  if (threadIdx.x < NS) {
    b_s[threadIdx.x] = y != nullptr ? out_w[threadIdx.x] * mult : 0.f;
    a_s[threadIdx.x] = in_w != nullptr ? in_w[threadIdx.x] : 0.f;
  }
  __syncthreads();
  pdl_wait();
  const size_t r = blockIdx.x;
  constexpr int W = VEC ? 4 : 1;                      // neighbouring features per group
  constexpr int GROUPS = HC_VPT / W;
  float u[HC_VPT];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < GROUPS; ++k) {
    const int i = (threadIdx.x + k * blockDim.x) * W;
#pragma unroll
    for (int e = 0; e < W; ++e) u[k * W + e] = 0.f;
    if (i < dim) {
      float* p = X + r * dim + i;
      float v[NS][W];
#pragma unroll
      for (int c = 0; c < NS; ++c) {
        if (VEC) {
          const float4 t = *reinterpret_cast<const float4*>(p + (size_t)c * copy_stride);
          v[c][0] = t.x; v[c][W > 1 ? 1 : 0] = t.y; v[c][W > 2 ? 2 : 0] = t.z; v[c][W > 3 ? 3 : 0] = t.w;
        } else {
          v[c][0] = p[(size_t)c * copy_stride];
        }
      }
      if (y != nullptr) {
        float yv[W];
        if (VEC) {
          // each element's slices in ascending order, as sum_slices adds them
#pragma unroll
          for (int e = 0; e < W; ++e) yv[e] = 0.f;
          for (int s = 0; s < n_partials; ++s) {
            const float4 t = *reinterpret_cast<const float4*>(y + (size_t)s * partial_stride + r * dim + i);
            yv[0] += t.x; yv[W > 1 ? 1 : 0] += t.y; yv[W > 2 ? 2 : 0] += t.z; yv[W > 3 ? 3 : 0] += t.w;
          }
        } else {
          yv[0] = sum_slices(y + r * dim + i, n_partials, partial_stride);
        }
        float nv[NS][W];
#pragma unroll
        for (int j = 0; j < NS; ++j)
#pragma unroll
          for (int e = 0; e < W; ++e) {
            float acc = 0.f;
#pragma unroll
            for (int c = 0; c < NS; ++c) acc = fmaf(m_s[c * NS + j], v[c][e], acc);
            nv[j][e] = fmaf(b_s[j], yv[e], acc);
          }
#pragma unroll
        for (int j = 0; j < NS; ++j) {
#pragma unroll
          for (int e = 0; e < W; ++e) v[j][e] = nv[j][e];
          if (VEC)
            *reinterpret_cast<float4*>(p + (size_t)j * copy_stride) =
                make_float4(nv[j][0], nv[j][W > 1 ? 1 : 0], nv[j][W > 2 ? 2 : 0], nv[j][W > 3 ? 3 : 0]);
          else
            p[(size_t)j * copy_stride] = nv[j][0];
        }
      }
      if (in_w != nullptr) {
#pragma unroll
        for (int e = 0; e < W; ++e) {
          float acc = 0.f;
#pragma unroll
          for (int c = 0; c < NS; ++c) acc = fmaf(a_s[c], v[c][e], acc);
          u[k * W + e] = acc;
          ss += acc * acc;
        }
      }
    }
  }
  if (in_w == nullptr) return;
  if (norm_w == nullptr) {
#pragma unroll
    for (int k = 0; k < GROUPS; ++k) {
      const int i = (threadIdx.x + k * blockDim.x) * W;
      if (i < dim) {
        if (VEC) *reinterpret_cast<float4*>(u_out + r * dim + i) =
            make_float4(u[k * W], u[k * W + (W > 1 ? 1 : 0)], u[k * W + (W > 2 ? 2 : 0)], u[k * W + (W > 3 ? 3 : 0)]);
        else u_out[r * dim + i] = u[k];
      }
    }
    return;
  }
  const float rs = 1.0f / sqrtf(block_sum(ss, scratch) / (float)dim + eps);
#pragma unroll
  for (int k = 0; k < GROUPS; ++k) {
    const int i = (threadIdx.x + k * blockDim.x) * W;
    if (i < dim) {
      alignas(16) TO t[W];
#pragma unroll
      for (int e = 0; e < W; ++e) t[e] = from_float<TO>(u[k * W + e] * rs * norm_w[i + e]);
      if (!VEC) h[r * dim + i] = t[0];
      else if (sizeof(TO) == 4) *reinterpret_cast<float4*>(h + r * dim + i) = *reinterpret_cast<const float4*>(t);
      else *reinterpret_cast<uint2*>(h + r * dim + i) = *reinterpret_cast<const uint2*>(t);
    }
  }
}

template <typename TO>
static int launch_hc(int copies, dim3 grid, dim3 block, cudaStream_t stream, float* X, long long cs,
                     const float* y, int np, long long ps, const float* mix, const float* out_w,
                     float mult, const float* in_w, const float* norm_w, float eps, void* h,
                     float* u_out, int dim, bool vec) {
#define YALM_HC(NS)                                                                               \
  case NS:                                                                                        \
    if (vec)                                                                                      \
      launch_pdl(hc_step_kernel<TO, NS, true>, grid, block, 0, stream, X, cs, y, np, ps, mix, out_w, \
                 mult, in_w, norm_w, eps, (TO*)h, u_out, dim);                                    \
    else                                                                                          \
      launch_pdl(hc_step_kernel<TO, NS, false>, grid, block, 0, stream, X, cs, y, np, ps, mix, out_w, \
                 mult, in_w, norm_w, eps, (TO*)h, u_out, dim);                                    \
    break
  switch (copies) {
    YALM_HC(1); YALM_HC(2); YALM_HC(3); YALM_HC(4); YALM_HC(5); YALM_HC(6); YALM_HC(7); YALM_HC(8);
    default: return -2;
  }
#undef YALM_HC
  YALM_LAUNCH_CHECK();
  return 0;
}

}  // namespace yalm

using namespace yalm;

// X [copies][rows][dim] float32 (copies 1..8).  y (or null): n_partials slices [rows][dim] whose sum
// is the sublayer's output; mix [copies][copies] (from, to), out_w [copies], mult.  in_w (or null)
// [copies]: the read that follows; with norm_w [dim] its normed rows go to h (h_dtype), without to
// u_out as float32.
extern "C" int yalm_hc_step(float* X, int copies, long long rows, int dim, const float* y, int n_partials,
                            long long partial_stride, const float* mix, const float* out_w, float mult,
                            const float* in_w, const float* norm_w, float eps, void* h, int h_dtype,
                            float* u_out, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (dim <= 0 || dim > HC_VPT * 1024 || copies < 1 || copies > 8) return -2;
  if (rows > 0x7fffffffLL) return -4;
  if (y == nullptr && in_w == nullptr) return 0;
  if (in_w != nullptr && norm_w == nullptr && u_out == nullptr) return -3;
  if (in_w != nullptr && norm_w != nullptr && h == nullptr) return -3;
  // (with five copies or more the four-feature form runs out of registers: one feature per thread)
  const bool vec = copies <= 4 && dim % 4 == 0 && (partial_stride & 3) == 0 &&
                   ((((uintptr_t)X) | ((uintptr_t)y) | ((uintptr_t)u_out) | ((uintptr_t)h)) & 15) == 0;
  const int per = vec ? 4 : 1;                        // features of a thread's group
  int threads = (dim + HC_VPT - 1) / HC_VPT;
  if (rows <= 256) threads = (dim + per - 1) / per;   // a few rows: one group per thread where that fits
  threads = (threads + 31) / 32 * 32;
  if (threads > 1024) threads = 1024;
  if (threads < 64) threads = 64;
  const dim3 grid((unsigned)rows), block(threads);
  const long long cs = rows * (long long)dim;
  if (h_dtype == DT_F32)
    return launch_hc<float>(copies, grid, block, stream, X, cs, y, n_partials, partial_stride, mix, out_w,
                            mult, in_w, norm_w, eps, h, u_out, dim, vec);
  if (h_dtype == DT_BF16)
    return launch_hc<__nv_bfloat16>(copies, grid, block, stream, X, cs, y, n_partials, partial_stride, mix,
                                    out_w, mult, in_w, norm_w, eps, h, u_out, dim, vec);
  if (h_dtype == DT_F16)
    return launch_hc<__half>(copies, grid, block, stream, X, cs, y, n_partials, partial_stride, mix, out_w,
                             mult, in_w, norm_w, eps, h, u_out, dim, vec);
  return -3;
}
