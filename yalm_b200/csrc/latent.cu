// Attention over a cached latent: a token leaves one row [c | kr] in the cache, c = norm(Wdkv h)[:rank]
// times a weight, kr the rot_dim rotated features shared by all heads.  Per head the key is
// [Wuk c | kr] and the value Wuv c, so with q = [qa | qr]
//     q . k = (Wuk^T qa) . c + qr . kr,        sum_j p_j v_j = Wuv (sum_j p_j c_j):
// queries are moved into the latent space once per token and head, the attention kernels run with
// ONE key/value head whose rows are the cache rows themselves (keys and values are the same
// rows), and the mixed latent is expanded by Wuv afterwards.  Three kernels:
//  * latent_store: sums the down projection's split-K slices, norms c, rotates kr (neighbouring
//    pairs, angle in 32 bits), writes the row to this step's buffer (as key and as value) and to
//    the cache;
//  * latent_absorb_q: q' = [Wuk_h^T qa | rot(qr) | 0] per token and head;
//  * latent_expand: out_h = (Wuv_h o_h) * sigmoid(gate), o_h the first `rank` features of the
//    attention's output for head h.
// The two per-head products keep their sums in 32 bits; a block takes LT_TOK tokens of one head so
// that a head's matrix is read once per LT_TOK tokens.
#include "api.h"
#include "common.cuh"

namespace yalm {

constexpr int LT_TOK = 8;

template <typename T>
__global__ void latent_store_kernel(const float* __restrict__ dkv, int n_partials, long long partial_stride,
                                    const float* __restrict__ c_norm, float eps,
                                    const float* __restrict__ freq, const int* __restrict__ token_seq,
                                    const int* __restrict__ q_start, const int* __restrict__ seq_slot,
                                    const int* __restrict__ slot_pos, T* __restrict__ kv_step,
                                    T* __restrict__ cache, int rank, int rd, int hd, int capacity,
                                    int write_cache, const int* __restrict__ page_table, int pps,
                                    int n_pages) {
  pdl_launch_dependents();
  extern __shared__ float row_s[];
  __shared__ float scratch[33];
  const int t = blockIdx.x;
  const int b = token_seq[t];
  const int slot = seq_slot[b];
  const int pos = slot_pos[slot] + (t - q_start[b]);
  pdl_wait();
  const int row = rank + rd;
  float ss = 0.f;
  for (int i = threadIdx.x; i < row; i += blockDim.x) {
    const float v = sum_slices(dkv + (size_t)t * row + i, n_partials, partial_stride);
    row_s[i] = v;
    if (i < rank) ss += v * v;
  }
  const float rs = 1.0f / sqrtf(block_sum(ss, scratch) / (float)rank + eps);
  const size_t off = write_cache ? kv_row_offset(page_table, pps, n_pages, slot, 0, 1, capacity, pos % capacity, hd) : 0;
  for (int i = threadIdx.x; i < hd; i += blockDim.x) {
    float v = 0.f;
    if (i < rank) {
      v = row_s[i] * rs * c_norm[i];
    } else if (i < row) {
      const int e = i - rank;
      const float ang = (float)pos * freq[e >> 1];
      const float c = cosf(ang), s = sinf(ang);
      const float me = row_s[i], other = row_s[rank + (e ^ 1)];
      v = (e & 1) ? rotate_hi(other, me, c, s) : rotate_lo(me, other, c, s);
    }
    const T val = from_float<T>(v);
    kv_step[(size_t)t * 2 * hd + i] = val;
    kv_step[(size_t)t * 2 * hd + hd + i] = val;
    if (write_cache) cache[off + i] = val;
  }
}

// grid (token tiles, heads).  q: float32 slices [tokens][H (dim + rd)]; w_uk [H][dim][rank];
// q_out [tokens][H][hd]
template <typename T>
__global__ void __launch_bounds__(256)
latent_absorb_q_kernel(const float* __restrict__ q, int n_partials, long long partial_stride,
                       const T* __restrict__ w_uk, const float* __restrict__ freq,
                       const int* __restrict__ token_seq, const int* __restrict__ q_start,
                       const int* __restrict__ seq_slot, const int* __restrict__ slot_pos,
                       T* __restrict__ q_out, int n_tokens, int H, int dim, int rd, int rank, int hd) {
  pdl_launch_dependents();
  extern __shared__ float qs[];                         // [LT_TOK][dim + rd]
  const int t0 = blockIdx.x * LT_TOK, h = blockIdx.y;
  const int qd = dim + rd;
  pdl_wait();
  for (int idx = threadIdx.x; idx < LT_TOK * qd; idx += blockDim.x) {
    const int tt = idx / qd, e = idx - tt * qd;
    const int t = t0 + tt;
    qs[idx] = t < n_tokens ? sum_slices(q + ((size_t)t * H + h) * qd + e, n_partials, partial_stride) : 0.f;
  }
  __syncthreads();
  const T* w = w_uk + (size_t)h * dim * rank;
  for (int c = threadIdx.x; c < rank; c += blockDim.x) {
    float acc[LT_TOK];
#pragma unroll
    for (int tt = 0; tt < LT_TOK; ++tt) acc[tt] = 0.f;
    for (int d = 0; d < dim; ++d) {
      const float wv = to_float(w[(size_t)d * rank + c]);
#pragma unroll
      for (int tt = 0; tt < LT_TOK; ++tt) acc[tt] = fmaf(wv, qs[tt * qd + d], acc[tt]);
    }
#pragma unroll
    for (int tt = 0; tt < LT_TOK; ++tt)
      if (t0 + tt < n_tokens) q_out[((size_t)(t0 + tt) * H + h) * hd + c] = from_float<T>(acc[tt]);
  }
  const int tail = hd - rank;
  for (int idx = threadIdx.x; idx < LT_TOK * tail; idx += blockDim.x) {
    const int tt = idx / tail, e = idx - tt * tail;
    const int t = t0 + tt;
    if (t >= n_tokens) continue;
    float v = 0.f;
    if (e < rd) {
      const int b = token_seq[t];
      const int pos = slot_pos[seq_slot[b]] + (t - q_start[b]);
      const float ang = (float)pos * freq[e >> 1];
      const float c = cosf(ang), s = sinf(ang);
      const float me = qs[tt * qd + dim + e], other = qs[tt * qd + dim + (e ^ 1)];
      v = (e & 1) ? rotate_hi(other, me, c, s) : rotate_lo(me, other, c, s);
    }
    q_out[((size_t)t * H + h) * hd + rank + e] = from_float<T>(v);
  }
}

// grid (token tiles, heads).  o [tokens][H][hd]; w_uv [H][rank][vdim] (transposed when bound);
// gate: float32 slices [tokens][H vdim] or null; out [tokens][H vdim]
template <typename T>
__global__ void __launch_bounds__(256)
latent_expand_kernel(const T* __restrict__ o, const T* __restrict__ w_uv, const float* __restrict__ gate,
                     int n_partials, long long partial_stride, T* __restrict__ out, int n_tokens, int H,
                     int rank, int vdim, int hd) {
  pdl_launch_dependents();
  extern __shared__ float xs[];                         // [LT_TOK][rank]
  const int t0 = blockIdx.x * LT_TOK, h = blockIdx.y;
  pdl_wait();
  for (int idx = threadIdx.x; idx < LT_TOK * rank; idx += blockDim.x) {
    const int tt = idx / rank, c = idx - tt * rank;
    const int t = t0 + tt;
    xs[idx] = t < n_tokens ? to_float(o[((size_t)t * H + h) * hd + c]) : 0.f;
  }
  __syncthreads();
  const T* w = w_uv + (size_t)h * rank * vdim;
  for (int idx = threadIdx.x; idx < LT_TOK * vdim; idx += blockDim.x) {
    const int tt = idx / vdim, j = idx - tt * vdim;
    const int t = t0 + tt;
    if (t >= n_tokens) continue;
    float acc = 0.f;
    const float* x = xs + tt * rank;
    for (int c = 0; c < rank; ++c) acc = fmaf(to_float(w[(size_t)c * vdim + j]), x[c], acc);
    const size_t at = ((size_t)t * H + h) * vdim + j;
    if (gate != nullptr) acc = acc / (1.0f + expf(-sum_slices(gate + at, n_partials, partial_stride)));
    out[at] = from_float<T>(acc);
  }
}

// ---- the two per-head products for many tokens: a block of 256 threads takes 64 tokens x 64
// columns of one head, a thread 4 x 4 of them; A and the head's matrix come through shared memory in
// slabs of 16 of K, so that a loaded element feeds 64 multiply-adds instead of 8.  Every output is
// the same sum, in the same order (k ascending, one fused multiply-add each), as in the kernels above.
constexpr int HP_BM = 64, HP_BN = 64, HP_BK = 16;

template <typename T, typename LoadA, typename Epi>
__device__ __forceinline__ void head_product_tile(const T* __restrict__ B, int K, int N, int t0, int n0,
                                                  int n_tokens, LoadA load_a, Epi epi) {
  __shared__ __align__(16) float As[HP_BK][HP_BM + 4];     // [k][token]
  __shared__ __align__(16) float Bs[HP_BK][HP_BN + 4];     // [k][column]
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  for (int k0 = 0; k0 < K; k0 += HP_BK) {
#pragma unroll
    for (int r = 0; r < HP_BM * HP_BK / 256; ++r) {
      const int i = threadIdx.x + r * 256;
      const int tt = i / HP_BK, kk = i % HP_BK;
      As[kk][tt] = (t0 + tt < n_tokens && k0 + kk < K) ? load_a(t0 + tt, k0 + kk) : 0.f;
    }
#pragma unroll
    for (int r = 0; r < HP_BK * HP_BN / 256; ++r) {
      const int i = threadIdx.x + r * 256;
      const int kk = i / HP_BN, nn = i % HP_BN;
      Bs[kk][nn] = (k0 + kk < K && n0 + nn < N) ? to_float(B[(size_t)(k0 + kk) * N + n0 + nn]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < HP_BK; ++kk) {
      const float4 a = *reinterpret_cast<const float4*>(&As[kk][ty * 4]);
      const float4 b = *reinterpret_cast<const float4*>(&Bs[kk][tx * 4]);
      const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(bv[j], av[i], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int t = t0 + ty * 4 + i, n = n0 + tx * 4 + j;
      if (t < n_tokens && n < N) epi(t, n, acc[i][j]);
    }
}

// grid (token tiles of 64, heads, column tiles of 64 over rank); the blocks of the first column
// tile also write the rotated part and the zero padding
template <typename T>
__global__ void __launch_bounds__(256)
latent_absorb_q_tiled_kernel(const float* __restrict__ q, int n_partials, long long partial_stride,
                             const T* __restrict__ w_uk, const float* __restrict__ freq,
                             const int* __restrict__ token_seq, const int* __restrict__ q_start,
                             const int* __restrict__ seq_slot, const int* __restrict__ slot_pos,
                             T* __restrict__ q_out, int n_tokens, int H, int dim, int rd, int rank, int hd) {
  pdl_launch_dependents();
  const int t0 = blockIdx.x * HP_BM, h = blockIdx.y, n0 = blockIdx.z * HP_BN;
  const int qd = dim + rd;
  pdl_wait();
  head_product_tile<T>(
      w_uk + (size_t)h * dim * rank, dim, rank, t0, n0, n_tokens,
      [&](int t, int k) { return sum_slices(q + ((size_t)t * H + h) * qd + k, n_partials, partial_stride); },
      [&](int t, int n, float v) { q_out[((size_t)t * H + h) * hd + n] = from_float<T>(v); });
  if (blockIdx.z != 0) return;
  const int tail = hd - rank;
  for (int idx = threadIdx.x; idx < HP_BM * tail; idx += blockDim.x) {
    const int tt = idx / tail, e = idx - tt * tail;
    const int t = t0 + tt;
    if (t >= n_tokens) continue;
    float v = 0.f;
    if (e < rd) {
      const int b = token_seq[t];
      const int pos = slot_pos[seq_slot[b]] + (t - q_start[b]);
      const float ang = (float)pos * freq[e >> 1];
      const float c = cosf(ang), s = sinf(ang);
      const float* src = q + ((size_t)t * H + h) * qd + dim;
      const float me = sum_slices(src + e, n_partials, partial_stride);
      const float other = sum_slices(src + (e ^ 1), n_partials, partial_stride);
      v = (e & 1) ? rotate_hi(other, me, c, s) : rotate_lo(me, other, c, s);
    }
    q_out[((size_t)t * H + h) * hd + rank + e] = from_float<T>(v);
  }
}

// grid (token tiles of 64, heads, column tiles of 64 over vdim)
template <typename T>
__global__ void __launch_bounds__(256)
latent_expand_tiled_kernel(const T* __restrict__ o, const T* __restrict__ w_uv, const float* __restrict__ gate,
                           int n_partials, long long partial_stride, T* __restrict__ out, int n_tokens,
                           int H, int rank, int vdim, int hd) {
  pdl_launch_dependents();
  const int t0 = blockIdx.x * HP_BM, h = blockIdx.y, n0 = blockIdx.z * HP_BN;
  pdl_wait();
  head_product_tile<T>(
      w_uv + (size_t)h * rank * vdim, rank, vdim, t0, n0, n_tokens,
      [&](int t, int k) { return to_float(o[((size_t)t * H + h) * hd + k]); },
      [&](int t, int n, float acc) {
        const size_t at = ((size_t)t * H + h) * vdim + n;
        if (gate != nullptr) acc = acc / (1.0f + expf(-sum_slices(gate + at, n_partials, partial_stride)));
        out[at] = from_float<T>(acc);
      });
}

constexpr int HP_MANY = 32;        // from this many tokens on the tiled kernels run

}  // namespace yalm

using namespace yalm;

#define YALM_BY_TYPE(dtype, CALL)                 \
  do {                                            \
    if ((dtype) == DT_F32) { CALL(float); }       \
    else if ((dtype) == DT_BF16) { CALL(__nv_bfloat16); } \
    else if ((dtype) == DT_F16) { CALL(__half); } \
    else return -3;                               \
  } while (0)

// dkv: float32 slices [tokens][rank + rd]; c_norm [rank]; freq [rd / 2]; kv_step [tokens][2][hd] and the
// cache ([slots][1][capacity][hd], or pages) in `dtype`; hd >= rank + rd (the rest is zero)
extern "C" int yalm_latent_store(const float* dkv, int n_partials, long long partial_stride,
                                 const float* c_norm, float eps, const float* freq, const int* token_seq,
                                 const int* q_start, const int* seq_slot, const int* slot_pos,
                                 void* kv_step, void* cache, int dtype, int n_tokens, int rank, int rd,
                                 int hd, int capacity, int write_cache, const int* page_table,
                                 int pages_per_slot, int n_pages, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (rank <= 0 || rd < 0 || rd % 2 || hd < rank + rd || rank + rd > 12 * 1024) return -2;
  const size_t smem = (size_t)(rank + rd) * sizeof(float);
  int threads = (hd + 31) / 32 * 32;
  if (threads > 512) threads = 512;
#define CALL(T)                                                                                         \
  launch_pdl(latent_store_kernel<T>, dim3(n_tokens), dim3(threads), smem, stream, dkv, n_partials,      \
             partial_stride, c_norm, eps, freq, token_seq, q_start, seq_slot, slot_pos, (T*)kv_step,    \
             (T*)cache, rank, rd, hd, capacity, write_cache, page_table, pages_per_slot, n_pages)
  YALM_BY_TYPE(dtype, CALL);
#undef CALL
  YALM_LAUNCH_CHECK();
  return 0;
}

extern "C" int yalm_latent_absorb_q(const float* q, int n_partials, long long partial_stride,
                                    const void* w_uk, const float* freq, const int* token_seq,
                                    const int* q_start, const int* seq_slot, const int* slot_pos,
                                    void* q_out, int dtype, int n_tokens, int H, int dim, int rd, int rank,
                                    int hd, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (H <= 0 || H > 65535 || dim <= 0 || rd < 0 || rd % 2 || rank <= 0 || hd < rank + rd) return -2;
  if (n_tokens > HP_MANY) {
    const dim3 grid((n_tokens + HP_BM - 1) / HP_BM, H, (rank + HP_BN - 1) / HP_BN), block(256);
#define CALL(T)                                                                                          \
  launch_pdl(latent_absorb_q_tiled_kernel<T>, grid, block, 0, stream, q, n_partials, partial_stride,     \
             (const T*)w_uk, freq, token_seq, q_start, seq_slot, slot_pos, (T*)q_out, n_tokens, H, dim,  \
             rd, rank, hd)
    YALM_BY_TYPE(dtype, CALL);
#undef CALL
    YALM_LAUNCH_CHECK();
    return 0;
  }
  const size_t smem = (size_t)LT_TOK * (dim + rd) * sizeof(float);
  if (smem > 48 * 1024) return -2;
  const dim3 grid((n_tokens + LT_TOK - 1) / LT_TOK, H), block(256);
#define CALL(T)                                                                                          \
  launch_pdl(latent_absorb_q_kernel<T>, grid, block, smem, stream, q, n_partials, partial_stride,        \
             (const T*)w_uk, freq, token_seq, q_start, seq_slot, slot_pos, (T*)q_out, n_tokens, H, dim,  \
             rd, rank, hd)
  YALM_BY_TYPE(dtype, CALL);
#undef CALL
  YALM_LAUNCH_CHECK();
  return 0;
}

extern "C" int yalm_latent_expand(const void* o, const void* w_uv, const float* gate, int n_partials,
                                  long long partial_stride, void* out, int dtype, int n_tokens, int H,
                                  int rank, int vdim, int hd, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (H <= 0 || H > 65535 || rank <= 0 || vdim <= 0 || hd < rank) return -2;
  if (n_tokens > HP_MANY) {
    const dim3 grid((n_tokens + HP_BM - 1) / HP_BM, H, (vdim + HP_BN - 1) / HP_BN), block(256);
#define CALL(T)                                                                                       \
  launch_pdl(latent_expand_tiled_kernel<T>, grid, block, 0, stream, (const T*)o, (const T*)w_uv, gate, \
             n_partials, partial_stride, (T*)out, n_tokens, H, rank, vdim, hd)
    YALM_BY_TYPE(dtype, CALL);
#undef CALL
    YALM_LAUNCH_CHECK();
    return 0;
  }
  const size_t smem = (size_t)LT_TOK * rank * sizeof(float);
  if (smem > 48 * 1024) return -2;
  const dim3 grid((n_tokens + LT_TOK - 1) / LT_TOK, H), block(256);
#define CALL(T)                                                                                       \
  launch_pdl(latent_expand_kernel<T>, grid, block, smem, stream, (const T*)o, (const T*)w_uv, gate,   \
             n_partials, partial_stride, (T*)out, n_tokens, H, rank, vdim, hd)
  YALM_BY_TYPE(dtype, CALL);
#undef CALL
  YALM_LAUNCH_CHECK();
  return 0;
}
