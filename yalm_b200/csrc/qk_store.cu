// What follows a q/k(/v) product whose queries and keys are normed over the WHOLE projection
// (all heads of a token at once) and rotated on a part of each head:
//  * qk_norm_rope_store: sums the product's split-K slices (plus a bias per feature of the row, if
//    the projections have one), norms q and k (each over its whole
//    row, with a weight per feature), rotates the first `dims` features of every head -- pairs
//    (i, i + dims/2) or neighbours (2i, 2i+1) -- by pos * freq[i] with cos and sin times `mult`,
//    and writes q, this step's keys and values and the cache rows in the storage type.  The
//    values are the v rows of the product, or, when it has none, the keys as projected
//    (before norm and rotation).  With head_eps >= 0 every head of q and k is, AFTER its rotation,
//    divided by its own root mean square over head_size features (a norm without a weight);
//  * pool_blocks: the mean key and the mean value of every block of `pool` positions that
//    this step completes, from the rows as the cache holds them, into a second cache that has
//    one row per block.
// Norms, angles and means are 32-bit.
#include "api.h"
#include "common.cuh"

namespace yalm {

// grid (token, part): every block of a token sums the whole row (the norms need it), and writes
// its own part of the outputs; one part when there are many tokens.  The product's row is [q: H heads | k: G heads | v: G heads (if any)],
// every head hd wide (rows beyond a head's true size are zero).  n_q / n_k: the true number of
// features of q and k (what the mean of squares divides by).
template <typename T>
__global__ void qk_norm_rope_store_kernel(
    const float* __restrict__ qkv, int n_partials, long long partial_stride,
    const float* __restrict__ bias, const float* __restrict__ q_norm, const float* __restrict__ k_norm, float n_q, float n_k, float eps,
    const float* __restrict__ freq, int dims, int neighbours, float mult, float head_eps, float head_size,
    const int* __restrict__ token_seq, const int* __restrict__ q_start,
    const int* __restrict__ seq_slot, const int* __restrict__ slot_pos, T* __restrict__ q_out,
    T* __restrict__ kv_step, T* __restrict__ k_cache, T* __restrict__ v_cache, int H, int G, int hd,
    int has_v, int capacity, int write_cache, const int* __restrict__ page_table, int pps, int n_pages) {
  pdl_launch_dependents();
  extern __shared__ float row_s[];                       // the summed row, then dims / 2 (cos, sin) pairs
  __shared__ float scratch[33];
  const int t = blockIdx.x;
  const int b = token_seq[t];
  const int slot = seq_slot[b];
  const int qs = q_start[b], q_end = q_start[b + 1];
  const int past = slot_pos[slot];
  const int pos = past + (t - qs);
  const bool keep = write_cache && pos >= past + (q_end - qs) - capacity;
  pdl_wait();
  const int nq = H * hd, nk = G * hd;
  const int row = nq + nk + (has_v ? nk : 0);
  const float* src = qkv + (size_t)t * row;
  // the token's cosines and sines, once for all heads (the angle in 32 bits)
  float2* cs = reinterpret_cast<float2*>(row_s + ((row + 1) & ~1));
  for (int i = threadIdx.x; i < (dims >> 1); i += blockDim.x) {
    const float ang = (float)pos * freq[i];
    cs[i] = make_float2(cosf(ang) * mult, sinf(ang) * mult);
  }
  float ssq = 0.f, ssk = 0.f;
  for (int i = threadIdx.x; i < row; i += blockDim.x) {
    const float v = sum_slices(src + i, n_partials, partial_stride) + (bias != nullptr ? bias[i] : 0.f);
    row_s[i] = v;
    if (i < nq) ssq += v * v;
    else if (i < nq + nk) ssk += v * v;
  }
  float rq = 1.f, rk = 1.f;
  if (q_norm != nullptr) rq = 1.0f / sqrtf(block_sum(ssq, scratch) / n_q + eps);
  if (k_norm != nullptr) rk = 1.0f / sqrtf(block_sum(ssk, scratch) / n_k + eps);
  __syncthreads();
  const int half = dims >> 1;
  // a norm per head after the rotation: the rotated row replaces the summed one first
  float* head_r = reinterpret_cast<float*>(cs + half);              // [H + G]
  if (head_eps >= 0.f) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    for (int head = warp; head < H + G; head += n_warps) {
      float* v = row_s + (size_t)head * hd;
      float ss = 0.f;
      if (neighbours) {
        for (int p = lane; p < half; p += 32) {
          const float a = v[2 * p], b2 = v[2 * p + 1];
          const float lo = rotate_lo(a, b2, cs[p].x, cs[p].y), hi = rotate_hi(a, b2, cs[p].x, cs[p].y);
          v[2 * p] = lo; v[2 * p + 1] = hi;
          ss += lo * lo + hi * hi;
        }
      } else {
        for (int p = lane; p < half; p += 32) {
          const float a = v[p], b2 = v[p + half];
          const float lo = rotate_lo(a, b2, cs[p].x, cs[p].y), hi = rotate_hi(a, b2, cs[p].x, cs[p].y);
          v[p] = lo; v[p + half] = hi;
          ss += lo * lo + hi * hi;
        }
      }
      for (int e = dims + lane; e < hd; e += 32) ss += v[e] * v[e];
      ss = warp_sum(ss);
      if (lane == 0) head_r[head] = 1.0f / sqrtf(ss / head_size + head_eps);
    }
    __syncthreads();
  }
  // this block's part of the outputs
  const int per_part = (nq + nk + gridDim.y - 1) / gridDim.y;
  const int i_lo = blockIdx.y * per_part, i_hi = min(nq + nk, i_lo + per_part);
  const int v_per = (nk + gridDim.y - 1) / gridDim.y;
  const int v_lo = blockIdx.y * v_per, v_hi = min(nk, v_lo + v_per);
  // q and k: norm, then rotate with the partner's normed value
  for (int i = i_lo + threadIdx.x; i < i_hi; i += blockDim.x) {
    const bool is_q = i < nq;
    const int j = is_q ? i : i - nq;                     // index inside q or k
    const int head = j / hd, e = j % hd;
    const float* w = is_q ? q_norm : k_norm;
    const float r = is_q ? rq : rk;
    float me = row_s[i] * (w != nullptr ? r * w[j] : 1.f);
    if (head_eps >= 0.f) {
      me *= head_r[is_q ? head : H + head];
    } else if (e < dims) {
      int pi, pair;                                       // partner's feature, pair number
      bool first;
      if (neighbours) { pi = e ^ 1; pair = e >> 1; first = !(e & 1); }
      else { first = e < half; pi = first ? e + half : e - half; pair = first ? e : e - half; }
      const int ip = i - e + pi;
      const int jp = j - e + pi;
      const float other = row_s[ip] * (w != nullptr ? r * w[jp] : 1.f);
      const float c = cs[pair].x, s = cs[pair].y;
      me = first ? rotate_lo(me, other, c, s) : rotate_hi(other, me, c, s);
    }
    const T val = from_float<T>(me);
    if (is_q) {
      q_out[(size_t)t * nq + j] = val;
    } else {
      kv_step[((size_t)t * 2 * G + head) * hd + e] = val;
      if (keep)
        k_cache[kv_row_offset(page_table, pps, n_pages, slot, head, G, capacity, pos % capacity, hd) + e] = val;
    }
  }
  // values: the v rows, or the keys as they were projected
  const float* vs = row_s + nq + (has_v ? nk : 0);
  for (int j = v_lo + threadIdx.x; j < v_hi; j += blockDim.x) {
    const int head = j / hd, e = j % hd;
    const T val = from_float<T>(vs[j]);
    kv_step[((size_t)t * 2 * G + G + head) * hd + e] = val;
    if (keep)
      v_cache[kv_row_offset(page_table, pps, n_pages, slot, head, G, capacity, pos % capacity, hd) + e] = val;
  }
}

// grid (blocks a sequence may complete in this step, G, sequences); one thread per feature.
// Block number blk of a sequence (positions blk * pool .. blk * pool + pool - 1) is complete
// after this step if its last position is one of the step's.  A position of this step is read
// from kv_step, an earlier one from the ring (the ring holds at least the last pool - 1
// positions before the step; the step's late ring write, if any, has not happened yet).
template <typename T>
__global__ void pool_blocks_kernel(const T* __restrict__ kv_step, const T* __restrict__ k_cache,
                                   const T* __restrict__ v_cache, const int* __restrict__ q_start,
                                   const int* __restrict__ seq_slot, const int* __restrict__ slot_pos,
                                   T* __restrict__ pool_k, T* __restrict__ pool_v, int G, int hd,
                                   int capacity, int pool, const int* __restrict__ page_table, int pps,
                                   int n_pages, int pool_capacity, const int* __restrict__ pool_table,
                                   int pool_pps, int pool_pages, int* __restrict__ status) {
  pdl_launch_dependents();
  pdl_wait();
  const int b = blockIdx.z, g = blockIdx.y;
  const int slot = seq_slot[b];
  const int qs = q_start[b], ql = q_start[b + 1] - qs;
  const int past = slot_pos[slot];
  const int blk = past / pool + blockIdx.x;
  if ((blk + 1) * pool > past + ql) return;               // not complete yet
  if (blk >= pool_capacity) {
    if (threadIdx.x == 0) atomicOr(status, ERR_CONTEXT_RANGE);
    return;
  }
  const size_t out = kv_row_offset(pool_table, pool_pps, pool_pages, slot, g, G, pool_capacity, blk, hd);
  const float inv = 1.0f / (float)pool;
  for (int e = threadIdx.x; e < hd; e += blockDim.x) {
    float sk = 0.f, sv = 0.f;
    for (int j = 0; j < pool; ++j) {
      const int pos = blk * pool + j;
      if (pos >= past) {
        const T* kp = kv_step + ((size_t)(qs + pos - past) * 2 * G + g) * hd + e;
        sk += to_float(kp[0]);
        sv += to_float(kp[(size_t)G * hd]);
      } else {
        const size_t off = kv_row_offset(page_table, pps, n_pages, slot, g, G, capacity, pos % capacity, hd) + e;
        sk += to_float(k_cache[off]);
        sv += to_float(v_cache[off]);
      }
    }
    pool_k[out + e] = from_float<T>(sk * inv);
    pool_v[out + e] = from_float<T>(sv * inv);
  }
}

}  // namespace yalm

using namespace yalm;

extern "C" int yalm_qk_norm_rope_store(const float* qkv, int n_partials, long long partial_stride,
                                       const float* bias, const float* q_norm, const float* k_norm, int n_q, int n_k,
                                       float eps, const float* freq, int dims, int neighbours,
                                       float mult, float head_eps, int head_size, const int* token_seq, const int* q_start,
                                       const int* seq_slot, const int* slot_pos, void* q_out,
                                       void* kv_step, void* k_cache, void* v_cache, int dtype,
                                       int n_tokens, int H, int G, int hd, int has_v, int capacity,
                                       int write_cache, const int* page_table, int pages_per_slot,
                                       int n_pages, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (hd <= 0 || dims < 0 || dims > hd || (dims & 1) || H <= 0 || G <= 0 || n_q <= 0 || n_k <= 0) return -2;
  const int row = (H + (has_v ? 2 : 1) * G) * hd;
  const size_t smem = (size_t)(((row + 1) & ~1) + dims + H + G) * sizeof(float);
  if (smem > 200 * 1024) return -2;
  if (head_eps >= 0.f && (head_size <= 0 || head_size > hd || q_norm != nullptr || k_norm != nullptr)) return -3;
  const int threads = row >= 2048 ? 512 : (row >= 512 ? 256 : 128);
  // a few tokens (a decode step): several blocks per token, each with a part of the outputs
  int parts = 1;
  if (n_tokens < 74) {
    parts = 148 / n_tokens;
    if (parts > 8) parts = 8;
    if (parts > row / 256) parts = row / 256 > 0 ? row / 256 : 1;
  }
#define YALM_QKS(T)                                                                                   \
  do {                                                                                                \
    static size_t attr = 48 * 1024;                                                                   \
    if (smem > attr) {                                                                                \
      cudaError_t e = cudaFuncSetAttribute(qk_norm_rope_store_kernel<T>,                              \
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);   \
      if (e != cudaSuccess) return (int)e;                                                            \
      attr = smem;                                                                                    \
    }                                                                                                 \
    launch_pdl(qk_norm_rope_store_kernel<T>, dim3(n_tokens, parts), dim3(threads), smem, stream, qkv, \
               n_partials, partial_stride, bias, q_norm, k_norm, (float)n_q, (float)n_k, eps, freq, dims,   \
               neighbours, mult, head_eps, (float)head_size, token_seq, q_start, seq_slot, slot_pos, (T*)q_out, (T*)kv_step,      \
               (T*)k_cache, (T*)v_cache, H, G, hd, has_v, capacity, write_cache, page_table,          \
               pages_per_slot, n_pages);                                                              \
  } while (0)
  if (dtype == DT_F32) YALM_QKS(float);
  else if (dtype == DT_BF16) YALM_QKS(__nv_bfloat16);
  else if (dtype == DT_F16) YALM_QKS(__half);
  else return -3;
#undef YALM_QKS
  YALM_LAUNCH_CHECK();
  return 0;
}

extern "C" int yalm_pool_blocks(const void* kv_step, const void* k_cache, const void* v_cache,
                                const int* q_start, const int* seq_slot, const int* slot_pos,
                                void* pool_k, void* pool_v, int dtype, int n_seqs, int max_q_len, int G,
                                int hd, int capacity, int pool, const int* page_table,
                                int pages_per_slot, int n_pages, int pool_capacity,
                                const int* pool_table, int pool_pps, int pool_pages, int* status,
                                cudaStream_t stream) {
  if (n_seqs <= 0) return 0;
  if (pool <= 0 || hd <= 0 || G <= 0 || capacity < pool - 1 || n_seqs > 65535 || G > 65535) return -2;
  const dim3 grid(max_q_len / pool + 1, G, n_seqs), block(hd >= 128 ? 128 : (hd >= 64 ? 64 : 32));
#define YALM_POOL(T)                                                                                 \
  launch_pdl(pool_blocks_kernel<T>, grid, block, 0, stream, (const T*)kv_step, (const T*)k_cache,    \
             (const T*)v_cache, q_start, seq_slot, slot_pos, (T*)pool_k, (T*)pool_v, G, hd, capacity, \
             pool, page_table, pages_per_slot, n_pages, pool_capacity, pool_table, pool_pps,          \
             pool_pages, status)
  if (dtype == DT_F32) YALM_POOL(float);
  else if (dtype == DT_BF16) YALM_POOL(__nv_bfloat16);
  else if (dtype == DT_F16) YALM_POOL(__half);
  else return -3;
#undef YALM_POOL
  YALM_LAUNCH_CHECK();
  return 0;
}
