// Prefill attention on tensor cores WITHOUT rounding the softmax weights: for mixers whose
// scores, weights and weighted sum of values have to be 32-bit.
//
//   S = Q K^T      mma.sync m16n8k16 on the 16-bit q and k as the cache holds them: every
//                  product is exact, sums are 32-bit;
//   softmax        online, 32-bit (exp2 of scaled differences), masks per element;
//   O += P V       P is NOT rounded to 16 bits: each weight is split into three 16-bit terms,
//                  p = hi + mid + lo (all 24 bits of p for bfloat16), and three tensor-core
//                  products with the same V fragment add them in 32 bits.  Twice the tensor work
//                  of the rounded form, and the result is that of 32-bit weights on 16-bit values.
//
// A block takes 64 query tokens of one head (four warps of 16 rows); keys come in blocks of 64
// through two shared-memory buffers, the next block's cp.async copies under this block's products.  A key is, in one numbering, a pooled block (one mean key / mean value
// row per `pool` positions that lie wholly before the query's window; see PoolArgs in
// attention.cu), a position before this step (the cache ring) or a position of this step (the
// step's own buffer).  Windows are sliding (window > 0) or none (0).
#include "api.h"
#include "common.cuh"

namespace yalm {

struct ExactPool {
  const void* k;
  const void* v;
  const int* table;
  int pps, n_pages, capacity, pool;
  int keep;                // > 0: beside its window a query also sees the positions below `keep`
};
__device__ __forceinline__ int exact_pooled_visible(int pos, int window, int pool) {
  if (pool <= 0 || window <= 0) return 0;
  const int n = pos - window + 1;
  return n > 0 ? n / pool : 0;
}

template <typename T> struct Mma16;
template <> struct Mma16<__nv_bfloat16> {
  static __device__ __forceinline__ void run(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
};
template <> struct Mma16<__half> {
  static __device__ __forceinline__ void run(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
};
__device__ __forceinline__ void ldmatrix_x4(uint32_t* r, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t* r, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
// (a, b) as three packed pairs of the 16-bit type whose sum is (a, b)
template <typename T>
__device__ __forceinline__ void split3(float a, float b, uint32_t& hi, uint32_t& mid, uint32_t& lo) {
  const float ah = to_float(from_float<T>(a)), bh = to_float(from_float<T>(b));
  const float ar = a - ah, br = b - bh;
  const float am = to_float(from_float<T>(ar)), bm = to_float(from_float<T>(br));
  hi = pack2<T>(ah, bh);
  mid = pack2<T>(am, bm);
  lo = pack2<T>(ar - am, br - bm);
}

constexpr int EX_BQ = 64, EX_BK = 64;

template <typename T, int HD>
__global__ void __launch_bounds__(128)
attn_exact_prefill_kernel(const T* __restrict__ q, const T* __restrict__ kv_step,
                          const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                          const int* __restrict__ q_start, const int* __restrict__ seq_slot,
                          const int* __restrict__ slot_pos, T* __restrict__ out, int H, int G,
                          int capacity, int window, float scale_log2,
                          const int* __restrict__ page_table, int pps, int n_pages, ExactPool pl) {
  constexpr int LDS = HD + 8;                          // row pitch in elements: ldmatrix without bank conflicts
  constexpr int TILE = EX_BK * LDS;                    // one block of keys (or values)
  extern __shared__ __align__(16) uint8_t exact_smem[];      // two buffers of (K block, V block)
  T* const bufs = reinterpret_cast<T*>(exact_smem);
  pdl_launch_dependents();
  pdl_wait();
  // heads run fastest, the last (longest) query tiles of a sequence first: short blocks fill the tail
  const int b = blockIdx.z, h = blockIdx.x, tile = gridDim.y - 1 - blockIdx.y;
  const int qs = q_start[b], ql = q_start[b + 1] - qs;
  if (tile * EX_BQ >= ql) return;
  const int slot = seq_slot[b];
  const int past = slot_pos[slot];
  const int gkv = h / (H / G);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int r0 = tile * EX_BQ + warp * 16 + g, r1 = r0 + 8;      // this thread's two query rows
  const int pos0 = past + r0, pos1 = past + r1;
  const int rows_here = min(EX_BQ, ql - tile * EX_BQ);
  const int p_first = past + tile * EX_BQ, p_last = p_first + rows_here - 1;
  const T* pool_k = reinterpret_cast<const T*>(pl.k);
  const T* pool_v = reinterpret_cast<const T*>(pl.v);

  uint32_t qa[HD / 16][4];
#pragma unroll
  for (int kk = 0; kk < HD / 16; ++kk) {
    const T* p0 = q + ((size_t)(qs + min(r0, ql - 1)) * H + h) * HD + kk * 16 + 2 * t;
    const T* p1 = q + ((size_t)(qs + min(r1, ql - 1)) * H + h) * HD + kk * 16 + 2 * t;
    qa[kk][0] = *reinterpret_cast<const uint32_t*>(p0);
    qa[kk][1] = *reinterpret_cast<const uint32_t*>(p1);
    qa[kk][2] = *reinterpret_cast<const uint32_t*>(p0 + 8);
    qa[kk][3] = *reinterpret_cast<const uint32_t*>(p1 + 8);
  }
  float o[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

  const int nb_max = exact_pooled_visible(p_last, window, pl.pool);
  const int j_lo = first_visible(p_first, window);
  const int n_pool_blocks = (nb_max + EX_BK - 1) / EX_BK;
  const int n_tok_blocks = (p_last - j_lo + EX_BK) / EX_BK;
  // kept first positions that lie before the tile's earliest window: blocks of their own, at their
  // own positions, visible to every row of the tile (those inside a window come with the window)
  const int n_front = pl.keep > 0 ? min(pl.keep, j_lo) : 0;
  const int n_head_blocks = n_pool_blocks + (n_front + EX_BK - 1) / EX_BK;
  const int n_blocks = n_head_blocks + n_tok_blocks;
  auto block_base = [&](int kb) {
    return kb < n_pool_blocks ? kb * EX_BK
         : kb < n_head_blocks ? (kb - n_pool_blocks) * EX_BK : j_lo + (kb - n_head_blocks) * EX_BK;
  };
  auto block_limit = [&](int kb) {
    return kb < n_pool_blocks ? nb_max : kb < n_head_blocks ? n_front : p_last + 1;
  };
  // a key block's rows into buffer (kb & 1): this thread copies half a row of K and of V in
  // 16-byte cp.async pieces; rows beyond the range are filled with zeros (source size 0)
  auto issue = [&](int kb) {
    const bool pooled = kb < n_pool_blocks;
    const int base = block_base(kb);
    const int limit = block_limit(kb);
    const int row = threadIdx.x >> 1, half = threadIdx.x & 1;
    const int key = base + row;
    const T *kp = q, *vp = q;                          // any valid address when nothing is read
    uint32_t bytes = 0;
    if (key < limit) {
      bytes = 16;
      if (pooled) {
        const size_t off = kv_row_offset(pl.table, pl.pps, pl.n_pages, slot, gkv, G, pl.capacity, key, HD);
        kp = pool_k + off;
        vp = pool_v + off;
      } else if (key >= past) {
        kp = kv_step + ((size_t)(qs + key - past) * 2 * G + gkv) * HD;
        vp = kp + (size_t)G * HD;
      } else {
        const size_t off = kv_row_offset(page_table, pps, n_pages, slot, gkv, G, capacity, key % capacity, HD);
        kp = k_cache + off;
        vp = v_cache + off;
      }
    }
    T* kd = bufs + (size_t)(kb & 1) * 2 * TILE + row * LDS;
    T* vd = kd + TILE;
#pragma unroll
    for (int c = 0; c < HD / 16; ++c) {
      const int e = half * (HD / 2) + c * 8;
      const int se = bytes ? e : 0;
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(kd + e)), "l"(kp + se), "r"(bytes) : "memory");
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(vd + e)), "l"(vp + se), "r"(bytes) : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  if (n_blocks > 0) issue(0);
  for (int kb = 0; kb < n_blocks; ++kb) {
    const bool pooled = kb < n_pool_blocks;
    const int base = block_base(kb);
    const int limit = block_limit(kb);
    if (kb + 1 < n_blocks) {                           // the next block's copies run under this block's products
      issue(kb + 1);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    const T* ks = bufs + (size_t)(kb & 1) * 2 * TILE;
    const T* vs = ks + TILE;

    // ---- S = Q K^T: 16 rows x 64 keys per warp
    float s[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
    const int mi = lane >> 3, mr = lane & 7;
#pragma unroll
    for (int kk = 0; kk < HD / 16; ++kk) {
#pragma unroll
      for (int n2 = 0; n2 < 4; ++n2) {
        uint32_t r[4];
        ldmatrix_x4(r, smem_u32(ks + (n2 * 16 + (mi >> 1) * 8 + mr) * LDS + kk * 16 + (mi & 1) * 8));
        Mma16<T>::run(s[2 * n2], qa[kk], r[0], r[1]);
        Mma16<T>::run(s[2 * n2 + 1], qa[kk], r[2], r[3]);
      }
    }
    // ---- masks, scale, online softmax (32-bit)
    const int vis0 = exact_pooled_visible(pos0, window, pl.pool), vis1 = exact_pooled_visible(pos1, window, pl.pool);
    const int lo0 = first_visible(pos0, window), lo1 = first_visible(pos1, window);
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = base + nt * 8 + 2 * t + (e & 1);
        const int rr = e >> 1;
        const int pos = rr ? pos1 : pos0;
        const bool row_ok = (rr ? r1 : r0) < ql;
        const bool see = row_ok && key < limit &&
                         (pooled ? key < (rr ? vis1 : vis0)
                                 : (key <= pos && (key >= (rr ? lo1 : lo0) || key < pl.keep)));
        const float v = see ? s[nt][e] * scale_log2 : -INFINITY;
        s[nt][e] = v;
        mx[rr] = fmaxf(mx[rr], v);
      }
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
      mx[rr] = fmaxf(mx[rr], __shfl_xor_sync(0xffffffffu, mx[rr], 1));
      mx[rr] = fmaxf(mx[rr], __shfl_xor_sync(0xffffffffu, mx[rr], 2));
      const float mn = fmaxf(m[rr], mx[rr]);
      const float corr = mn > -INFINITY ? exp2f(m[rr] - mn) : 1.f;     // exp2(-inf) = 0 on the first visible key
      m[rr] = mn;
      l[rr] *= corr;
#pragma unroll
      for (int i = 0; i < HD / 8; ++i) { o[i][2 * rr] *= corr; o[i][2 * rr + 1] *= corr; }
      float sum = 0.f;
#pragma unroll
      for (int nt = 0; nt < 8; ++nt)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const float v = s[nt][2 * rr + e];
          const float p = v > -INFINITY ? exp2f(v - mn) : 0.f;
          s[nt][2 * rr + e] = p;
          sum += p;
        }
      l[rr] += sum;
    }
    // ---- O += P V with P as three 16-bit terms
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      uint32_t hi[4], mid[4], lo[4];
      split3<T>(s[2 * kk][0], s[2 * kk][1], hi[0], mid[0], lo[0]);
      split3<T>(s[2 * kk][2], s[2 * kk][3], hi[1], mid[1], lo[1]);
      split3<T>(s[2 * kk + 1][0], s[2 * kk + 1][1], hi[2], mid[2], lo[2]);
      split3<T>(s[2 * kk + 1][2], s[2 * kk + 1][3], hi[3], mid[3], lo[3]);
#pragma unroll
      for (int n2 = 0; n2 < HD / 16; ++n2) {
        uint32_t r[4];
        ldmatrix_x4_trans(r, smem_u32(vs + (kk * 16 + (mi & 1) * 8 + mr) * LDS + n2 * 16 + (mi >> 1) * 8));
        Mma16<T>::run(o[2 * n2], lo, r[0], r[1]);
        Mma16<T>::run(o[2 * n2], mid, r[0], r[1]);
        Mma16<T>::run(o[2 * n2], hi, r[0], r[1]);
        Mma16<T>::run(o[2 * n2 + 1], lo, r[2], r[3]);
        Mma16<T>::run(o[2 * n2 + 1], mid, r[2], r[3]);
        Mma16<T>::run(o[2 * n2 + 1], hi, r[2], r[3]);
      }
    }
    __syncthreads();                                   // this buffer is copied into again two blocks on
  }
#pragma unroll
  for (int rr = 0; rr < 2; ++rr) {
    l[rr] += __shfl_xor_sync(0xffffffffu, l[rr], 1);
    l[rr] += __shfl_xor_sync(0xffffffffu, l[rr], 2);
    const int r = rr ? r1 : r0;
    if (r >= ql) continue;
    const float inv = 1.0f / l[rr];
    T* dst = out + ((size_t)(qs + r) * H + h) * HD + 2 * t;
#pragma unroll
    for (int i = 0; i < HD / 8; ++i)
      *reinterpret_cast<uint32_t*>(dst + i * 8) = pack2<T>(o[i][2 * rr] * inv, o[i][2 * rr + 1] * inv);
  }
}

}  // namespace yalm

using namespace yalm;

// Prefill attention with 32-bit softmax weights on tensor cores (dtype 1 or 2; head size 32, 64,
// 128 or 256; window >= 0).  Keys of this step come from kv_step, earlier ones from the cache ring;
// with pool > 0 the pooled rows of yalm_attention_pooled take part; with keep_first > 0 (and a
// window, no pool) the first keep_first positions stay visible beside the window, and the cache
// holds every position.  q, out [tokens, H, hd].
extern "C" int yalm_attention_exact_prefill(const void* q, const void* kv_step, const void* k_cache,
                                            const void* v_cache, const int* q_start, const int* seq_slot,
                                            const int* slot_pos, void* out, int dtype, int n_seqs,
                                            int max_q_len, int H, int G, int hd, int capacity, int window,
                                            float scale, const int* page_table, int pages_per_slot,
                                            int n_pages, const void* pool_k, const void* pool_v, int pool,
                                            int pool_capacity, const int* pool_table, int pool_pps,
                                            int pool_pages, int keep_first, cudaStream_t stream) {
  if (n_seqs <= 0 || max_q_len <= 0) return 0;
  if (hd != 32 && hd != 64 && hd != 128 && hd != 256) return -2;
  if (G <= 0 || H % G != 0 || window < 0 || (pool > 0 && window <= 0)) return -3;
  if (keep_first < 0 || (keep_first > 0 && (window <= 0 || pool > 0))) return -3;
  if (dtype != DT_BF16 && dtype != DT_F16) return -3;
  if (H > 65535 || n_seqs > 65535) return -4;
  const ExactPool pl = {pool_k, pool_v, pool_table, pool_pps, pool_pages, pool_capacity, pool > 0 ? pool : 0, keep_first};
  const dim3 grid(H, (max_q_len + EX_BQ - 1) / EX_BQ, n_seqs), block(128);
  if (grid.y > 65535) return -4;
  const size_t smem = (size_t)2 * 2 * EX_BK * (hd + 8) * 2;
  const float scale_log2 = score_scale(scale, hd) * 1.4426950408889634f;
#define YALM_EX(T, D)                                                                                \
  do {                                                                                               \
    static bool set = false;                                                                         \
    if (!set && smem > 48 * 1024) {                                                                  \
      cudaError_t e = cudaFuncSetAttribute(attn_exact_prefill_kernel<T, D>,                          \
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);  \
      if (e != cudaSuccess) return (int)e;                                                           \
      set = true;                                                                                    \
    }                                                                                                \
    launch_pdl(attn_exact_prefill_kernel<T, D>, grid, block, smem, stream, (const T*)q,              \
               (const T*)kv_step, (const T*)k_cache, (const T*)v_cache, q_start, seq_slot, slot_pos, \
               (T*)out, H, G, capacity, window, scale_log2, page_table, pages_per_slot, n_pages, pl); \
  } while (0)
  if (dtype == DT_BF16) {
    if (hd == 32) YALM_EX(__nv_bfloat16, 32);
    else if (hd == 64) YALM_EX(__nv_bfloat16, 64);
    else if (hd == 128) YALM_EX(__nv_bfloat16, 128);
    else YALM_EX(__nv_bfloat16, 256);
  } else {
    if (hd == 32) YALM_EX(__half, 32);
    else if (hd == 64) YALM_EX(__half, 64);
    else if (hd == 128) YALM_EX(__half, 128);
    else YALM_EX(__half, 256);
  }
#undef YALM_EX
  YALM_LAUNCH_CHECK();
  return 0;
}
