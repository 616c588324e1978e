// A real-gated linear recurrent unit per channel (the recurrence of Griffin's recurrent block):
//   r = sigmoid(Ra u + ba),  i = sigmoid(Ri u + bi)        Ra, Ri block-diagonal
//   a = exp(-c r softplus(lam)),   S_t = a_t S_(t-1) + sqrt(1 - a_t^2) i_t u_t,   out_t = S_t y_t
// with y = gelu(Wy h + by) the block's other branch.  S is one 32-bit float per channel and sequence.
// Two kernels, all arithmetic 32-bit:
//  * rglru_gates: every token and channel in parallel: log a, b = sqrt(1 - a^2) i u, and y;
//  * rglru_scan: the recurrence S_t = a_t S_(t-1) + b_t.  A block owns 32 channels of one sequence
//    and cuts the step's tokens into RG_CHUNKS = 32 runs; each run is first composed into one (A, B) pair
//    (S_out = A S_in + B), the runs' pairs are chained from the sequence's state, and a second pass
//    over the run writes S_t y_t.  A decay close to 1 has few bits of its own left in a, and a state
//    that lives for a thousand tokens collects that error: so a step is S + expm1(log a) S + b, a
//    run's A is exp(sum of log a), and 1 - a^2 is -expm1(2 log a).
#include "api.h"
#include "common.cuh"

namespace yalm {

constexpr int RG_CHUNKS = 32;

// grid (tokens, parts of the channels).  gates: float32 [blocks][tokens][2 bw] (the r logits of a
// block's channels, then its i logits); yx: slices [.][tokens][yx_row] with the y logits at column 0;
// coef [3][tokens][width] receives log a, b, y.
__global__ void rglru_gates_kernel(const float* __restrict__ gates, const float* __restrict__ ra_bias,
                                   const float* __restrict__ ri_bias, const float* __restrict__ lam,
                                   const float* __restrict__ u, const float* __restrict__ yx, int n_partials,
                                   long long partial_stride, int yx_row, const float* __restrict__ y_bias,
                                   float* __restrict__ coef, int n_tokens, int width, int bw, float c_decay) {
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= width) return;
  const float sp = lam[c] > 20.f ? lam[c] : log1pf(expf(lam[c]));
  const float ba = ra_bias[c], bi = ri_bias[c], by = y_bias != nullptr ? y_bias[c] : 0.f;
  pdl_wait();
  const float* g = gates + ((size_t)(c / bw) * n_tokens + t) * 2 * bw + c % bw;
  const float r = 1.0f / (1.0f + expf(-(g[0] + ba)));
  const float i = 1.0f / (1.0f + expf(-(g[bw] + bi)));
  const float log_a = -c_decay * r * sp;
  const float b = sqrtf(-expm1f(2.0f * log_a)) * i * u[(size_t)t * width + c];
  const float* yp = yx + (size_t)t * yx_row + c;
  const float yv = (n_partials == 1 ? yp[0] : sum_slices(yp, n_partials, partial_stride)) + by;
  const float y = 0.5f * yv * (1.0f + tanhf(0.7978845608028654f * (yv + 0.044715f * yv * yv * yv)));
  const size_t plane = (size_t)n_tokens * width;
  coef[(size_t)t * width + c] = log_a;
  coef[plane + (size_t)t * width + c] = b;
  coef[2 * plane + (size_t)t * width + c] = y;
}

// grid (sequences, width / 32), block (32, RG_CHUNKS)
template <typename T>
__global__ void __launch_bounds__(32 * RG_CHUNKS)
rglru_scan_kernel(const float* __restrict__ coef, const int* __restrict__ q_start,
                  const int* __restrict__ seq_slot, float* __restrict__ state, T* __restrict__ out,
                  int n_tokens, int width) {
  pdl_launch_dependents();
  __shared__ float sA[RG_CHUNKS][32], sB[RG_CHUNKS][32];
  const int b = blockIdx.x;
  const int c = blockIdx.y * 32 + threadIdx.x, j = threadIdx.y;
  const int t0 = q_start[b], ql = q_start[b + 1] - t0;
  const int slot = seq_slot[b];
  const bool live = c < width;
  const int len = (ql + RG_CHUNKS - 1) / RG_CHUNKS;
  const int lo = j * len, hi = min(ql, lo + len);
  const size_t plane = (size_t)n_tokens * width;
  pdl_wait();
  const float* pa = coef + (size_t)t0 * width + c;
  const float* pb = pa + plane;
  const float* py = pb + plane;
  float A = 0.f, B = 0.f;                              // A: the sum of log a
  if (live) {
    int t = lo;
    for (; t + 4 <= hi; t += 4) {                       // four tokens' loads and expm1 ahead of the chain
      float la[4], bb[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) { la[u] = pa[(size_t)(t + u) * width]; bb[u] = pb[(size_t)(t + u) * width]; }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        A += la[u];
        B = fmaf(expm1f(la[u]), B, B) + bb[u];
      }
    }
    for (; t < hi; ++t) {
      const float la = pa[(size_t)t * width];
      A += la;
      B = fmaf(expm1f(la), B, B) + pb[(size_t)t * width];
    }
  }
  sA[j][threadIdx.x] = expm1f(A);
  sB[j][threadIdx.x] = B;
  __syncthreads();
  if (!live || lo >= hi) return;
  float S = state[(size_t)slot * width + c];
  for (int jj = 0; jj < j; ++jj) S = fmaf(sA[jj][threadIdx.x], S, S) + sB[jj][threadIdx.x];
  int t = lo;
  for (; t + 4 <= hi; t += 4) {
    float la[4], bb[4], yy[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      la[u] = pa[(size_t)(t + u) * width]; bb[u] = pb[(size_t)(t + u) * width]; yy[u] = py[(size_t)(t + u) * width];
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      S = fmaf(expm1f(la[u]), S, S) + bb[u];
      out[(size_t)(t0 + t + u) * width + c] = from_float<T>(S * yy[u]);
    }
  }
  for (; t < hi; ++t) {
    S = fmaf(expm1f(pa[(size_t)t * width]), S, S) + pb[(size_t)t * width];
    out[(size_t)(t0 + t) * width + c] = from_float<T>(S * py[(size_t)t * width]);
  }
  if (hi == ql) state[(size_t)slot * width + c] = S;
}

}  // namespace yalm

using namespace yalm;

// gates float32 [width / bw][tokens][2 bw]; ra_bias, ri_bias, lam [width]; u float32 [tokens][width];
// yx slices [.][tokens][yx_row] (y logits first); y_bias [width] or null; coef: float32 scratch
// [3][tokens][width]; state float32 [slots][width]; out [tokens][width] in out_dtype = S_t y_t.
extern "C" int yalm_rglru(const float* gates, const float* ra_bias, const float* ri_bias, const float* lam,
                          const float* u, const float* yx, int n_partials, long long partial_stride,
                          int yx_row, const float* y_bias, float* coef, const int* q_start,
                          const int* seq_slot, float* state, void* out, int out_dtype, int n_tokens,
                          int n_seqs, int width, int bw, float c_decay, cudaStream_t stream) {
  if (n_tokens <= 0 || n_seqs <= 0) return 0;
  if (width <= 0 || bw <= 0 || width % bw) return -2;
  const int threads = width >= 256 ? 256 : (width + 31) / 32 * 32;
  const int parts = (width + threads - 1) / threads;
  if (parts > 65535 || (width + 31) / 32 > 65535) return -4;
  launch_pdl(rglru_gates_kernel, dim3(n_tokens, parts), dim3(threads), 0, stream, gates, ra_bias, ri_bias, lam,
             u, yx, n_partials, partial_stride, yx_row, y_bias, coef, n_tokens, width, bw, c_decay);
  YALM_LAUNCH_CHECK();
  const dim3 grid(n_seqs, (width + 31) / 32), block(32, RG_CHUNKS);
  if (out_dtype == DT_F32)
    launch_pdl(rglru_scan_kernel<float>, grid, block, 0, stream, (const float*)coef, q_start, seq_slot, state,
               (float*)out, n_tokens, width);
  else if (out_dtype == DT_BF16)
    launch_pdl(rglru_scan_kernel<__nv_bfloat16>, grid, block, 0, stream, (const float*)coef, q_start, seq_slot,
               state, (__nv_bfloat16*)out, n_tokens, width);
  else if (out_dtype == DT_F16)
    launch_pdl(rglru_scan_kernel<__half>, grid, block, 0, stream, (const float*)coef, q_start, seq_slot, state,
               (__half*)out, n_tokens, width);
  else return -3;
  YALM_LAUNCH_CHECK();
  return 0;
}
