// A gated linear recurrence per head whose forget gate also decides what is written:
//   S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T,   o_t = S_t^T q_t,
// S [key size, value size] per head and sequence, carried from step to step in 32-bit floats.
// Everything here is 32-bit.  Two kernels:
//
//  * recurrence_gates: the fused projection [q | f | v] of a step (split-K slices) with its
//    activations applied, q = silu(.), f = l + (1 - l) sigmoid(. + bias) with a lower bound l per
//    key channel, v as it is: one pass over the step's tokens, all in parallel;
//  * recurrence_scan: the recurrence itself.  A block owns RC_COLS value columns of one
//    (sequence, head), a warp RC_CPW of them, and a lane RPT neighbouring rows of those columns'
//    state in registers.  The step's tokens of the sequence come through a three-stage cp.async ring,
//    RC_TOK tokens per stage (one block barrier per stage); a token costs a lane RPT state
//    updates and RPT multiply-adds, and the 32 partial sums of an output are added for RC_TOK
//    tokens at once, so that the shuffles of different tokens overlap.
#include "api.h"
#include "common.cuh"

namespace yalm {

constexpr int RC_CPW = 2;                 // value columns per warp
constexpr int RC_COLS = 8 * RC_CPW;       // ... per block of eight warps
constexpr int RC_TOK = 16;
constexpr int RC_STAGES = 3;

// grid (token, part of the row): a thread takes four elements of the row, a block 1,024, so that
// a decode step's few tokens still spread over many blocks.
__global__ void recurrence_gates_kernel(const float* __restrict__ proj, int n_partials,
                                        long long partial_stride, const float* __restrict__ f_bias,
                                        const float* __restrict__ lower, float* __restrict__ act,
                                        int row, int n_q) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t base = (size_t)blockIdx.x * row;
  const int e_end = min(row, (int)(blockIdx.y + 1) * 1024);
  for (int e = blockIdx.y * 1024 + threadIdx.x; e < e_end; e += blockDim.x) {
    const float z = sum_slices(proj + base + e, n_partials, partial_stride);
    float v = z;
    if (e < n_q) {
      v = z / (1.0f + expf(-z));
    } else if (e < 2 * n_q) {
      const float l = lower[e - n_q];
      v = l + (1.0f - l) * (1.0f / (1.0f + expf(-(z + f_bias[e - n_q]))));
    }
    act[base + e] = v;
  }
}

template <int BYTES>
__device__ __forceinline__ void cp_async(float* dst, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], %2;" ::"r"(smem_u32(dst)), "l"(src), "n"(BYTES) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// VEC: floats per copy (4 when every offset is a multiple of 16 bytes, else 1)
template <int RPT, int VEC>
__global__ void __launch_bounds__(256)
recurrence_scan_kernel(const float* __restrict__ act, const int* __restrict__ q_start,
                       const int* __restrict__ seq_slot, float* __restrict__ state,
                       float* __restrict__ out, int H, int dk, int dv) {
  pdl_launch_dependents();
  constexpr int DKP = 32 * RPT;                       // rows, padded
  constexpr int PER_TOK = 2 * DKP + RC_COLS;          // q, f, then this block's v columns
  extern __shared__ __align__(16) float stage[];      // [RC_STAGES][RC_TOK][PER_TOK]
  const int b = blockIdx.z, h = blockIdx.y, c0 = blockIdx.x * RC_COLS;
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int col = c0 + w * RC_CPW;
  const int slot = seq_slot[b];
  const int t0 = q_start[b], t1 = q_start[b + 1];
  const int row = 2 * H * dk + H * dv;
  // rows beyond dk: f = 0 and q = 0 for ever (never copied over); their state is not stored.
  // Value columns beyond dv are never copied either and nothing of them is stored.
  if (dk < DKP) {
    for (int i = threadIdx.x; i < RC_STAGES * RC_TOK * PER_TOK; i += blockDim.x) stage[i] = 0.f;
    __syncthreads();
  }
  // what this thread copies of every token: up to five runs of VEC floats
  const int per = 2 * dk + RC_COLS;
  int src_off[5], dst_off[5];
#pragma unroll
  for (int k = 0; k < 5; ++k) {
    const int e = (threadIdx.x + k * 256) * VEC;
    src_off[k] = dst_off[k] = -1;
    if (e < dk) { src_off[k] = h * dk + e; dst_off[k] = e; }
    else if (e < 2 * dk) { src_off[k] = H * dk + h * dk + (e - dk); dst_off[k] = DKP + (e - dk); }
    else if (e < per && c0 + (e - 2 * dk) < dv) {
      src_off[k] = 2 * H * dk + h * dv + c0 + (e - 2 * dk);
      dst_off[k] = 2 * DKP + (e - 2 * dk);
    }
  }
  pdl_wait();
  float S[RPT][RC_CPW];
  float* st = state + (((size_t)slot * H + h) * dk) * dv + col;
  // The block's part of the state is dk rows of RC_COLS neighbouring floats.  Where 16-byte
  // accesses fit, it goes through shared memory (a warp reads eight whole 64-byte runs per load)
  // instead of every lane picking its own rows out of memory 8 bytes at a time.
  constexpr int TP = RC_COLS + 1;                     // tile pitch
  const bool tiled = VEC == 4 && c0 + RC_COLS <= dv;
  float* tile_g = state + (((size_t)slot * H + h) * dk) * dv + c0;
  if (tiled) {
    for (int i = threadIdx.x; i < dk * (RC_COLS / 4); i += blockDim.x) {
      const int r = i / (RC_COLS / 4), q4 = i % (RC_COLS / 4);
      const float4 v = *reinterpret_cast<const float4*>(tile_g + (size_t)r * dv + 4 * q4);
      float* d = stage + r * TP + 4 * q4;
      d[0] = v.x; d[1] = v.y; d[2] = v.z; d[3] = v.w;
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < RPT; ++r)
#pragma unroll
      for (int c = 0; c < RC_CPW; ++c) {
        const int i = lane * RPT + r;
        S[r][c] = i < dk ? stage[i * TP + w * RC_CPW + c] : 0.f;
      }
    __syncthreads();
    if (dk < DKP) {                                   // the tile lay over rows that must read as zero
      for (int i = threadIdx.x; i < dk * TP; i += blockDim.x) stage[i] = 0.f;
      __syncthreads();
    }
  } else {
#pragma unroll
    for (int r = 0; r < RPT; ++r)
#pragma unroll
      for (int c = 0; c < RC_CPW; ++c) {
        const int i = lane * RPT + r;
        S[r][c] = (col + c < dv && i < dk) ? st[(size_t)i * dv + c] : 0.f;
      }
  }
  const int n_groups = (t1 - t0 + RC_TOK - 1) / RC_TOK;
  auto issue = [&](int g) {
    if (g < n_groups) {
      const int base = t0 + g * RC_TOK;
      const int nt = min(RC_TOK, t1 - base);
      float* dst = stage + (size_t)(g % RC_STAGES) * RC_TOK * PER_TOK;
      const float* src = act + (size_t)base * row;
#pragma unroll
      for (int k = 0; k < 5; ++k)
        if (src_off[k] >= 0)
          for (int tt = 0; tt < nt; ++tt)
            cp_async<4 * VEC>(dst + tt * PER_TOK + dst_off[k], src + (size_t)tt * row + src_off[k]);
    }
    cp_async_commit();
  };
  issue(0);
  issue(1);
  for (int g = 0; g < n_groups; ++g) {
    cp_async_wait<RC_STAGES - 2>();
    __syncthreads();                                   // stage g has landed; stage g - 1 is no longer read
    issue(g + 2);
    const int base = t0 + g * RC_TOK;
    const int nt = min(RC_TOK, t1 - base);
    const float* sg = stage + (size_t)(g % RC_STAGES) * RC_TOK * PER_TOK;
    float o[RC_TOK][RC_CPW];
#pragma unroll
    for (int tt = 0; tt < RC_TOK; ++tt) {
#pragma unroll
      for (int c = 0; c < RC_CPW; ++c) o[tt][c] = 0.f;
      if (tt < nt) {
        const float* q = sg + tt * PER_TOK + lane * RPT;
        const float* f = q + DKP;
        float vj[RC_CPW];
#pragma unroll
        for (int c = 0; c < RC_CPW; ++c) vj[c] = sg[tt * PER_TOK + 2 * DKP + w * RC_CPW + c];
#pragma unroll
        for (int r = 0; r < RPT; ++r) {
          const float fi = f[r], qi = q[r], gi = 1.0f - fi;
#pragma unroll
          for (int c = 0; c < RC_CPW; ++c) {
            S[r][c] = fmaf(fi, S[r][c], gi * vj[c]);
            o[tt][c] = fmaf(S[r][c], qi, o[tt][c]);
          }
        }
      }
    }
    // The group's RC_TOK x RC_CPW = 32 outputs, each the sum of the 32 lanes' partial sums: in every
    // round a lane hands half of its values to its partner and adds the partner's other half to its
    // own, so 16 + 8 + 4 + 2 + 1 exchanges leave lane l with the whole sum of value number l
    // (token l / RC_CPW, column l % RC_CPW).
    static_assert(RC_TOK * RC_CPW == 32, "one output per lane");
    float* ov = &o[0][0];                              // value number tt * RC_CPW + c
#pragma unroll
    for (int half = 16; half >= 1; half >>= 1) {
      const bool upper = (lane & half) != 0;
#pragma unroll
      for (int i = 0; i < half; ++i) {
        const float send = upper ? ov[i] : ov[i + half];
        const float keep = upper ? ov[i + half] : ov[i];
        ov[i] = keep + __shfl_xor_sync(0xffffffffu, send, half);
      }
    }
    {
      const int tt = lane / RC_CPW, c = lane % RC_CPW;
      if (tt < nt && col + c < dv) out[((size_t)(base + tt) * H + h) * dv + col + c] = ov[0];
    }
  }
  cp_async_wait<0>();
  if (tiled) {
    __syncthreads();                                   // the last group's rows are no longer read
#pragma unroll
    for (int r = 0; r < RPT; ++r)
#pragma unroll
      for (int c = 0; c < RC_CPW; ++c) {
        const int i = lane * RPT + r;
        if (i < dk) stage[i * TP + w * RC_CPW + c] = S[r][c];
      }
    __syncthreads();
    for (int i = threadIdx.x; i < dk * (RC_COLS / 4); i += blockDim.x) {
      const int r = i / (RC_COLS / 4), q4 = i % (RC_COLS / 4);
      const float* d = stage + r * TP + 4 * q4;
      *reinterpret_cast<float4*>(tile_g + (size_t)r * dv + 4 * q4) = make_float4(d[0], d[1], d[2], d[3]);
    }
    return;
  }
#pragma unroll
  for (int r = 0; r < RPT; ++r)
#pragma unroll
    for (int c = 0; c < RC_CPW; ++c) {
      const int i = lane * RPT + r;
      if (col + c < dv && i < dk) st[(size_t)i * dv + c] = S[r][c];
    }
}


// ---------------------------------------------------------------------------------------------
// A recurrence with a decay per key channel and a bonus for the current token ("wkv"), per head:
//   o_t = (S_(t-1) + diag(u) k_t v_t^T)^T r_t,   S_t = diag(w_t) S_(t-1) + k_t v_t^T,
// S [key size, value size] in 32-bit floats per head and sequence.  Three kernels around it:
//  * token_shift: every projection of the mixer reads its own mixture of a token's input and the
//    previous token's, h + (h' - h) mu; the previous token of a step's first token is part of the
//    sequence's state (zero for a new sequence);
//  * wkv_gates: the projections' split-K slices summed into one activated row per token,
//    (r | w | k | v) with w = exp(-exp(z + w0)), and the output gate silu(g); it also leaves the
//    step's last input of every sequence in the state for the next step's first token;
//  * wkv_scan: the recurrence, with recurrence_scan's layout (a lane owns RPT neighbouring rows of
//    two value columns, tokens through a three-stage cp.async ring).
//  * wkv_out: every head's output over its root mean square, times a weight per feature, times
//    the gate, into the storage type.

// grid (token); out [n_mix][tokens][dim] in the storage type
// four neighbouring elements of a row as floats, and back (16-byte or 8-byte accesses)
template <typename T>
__device__ __forceinline__ void load_four(const T* __restrict__ p, float* f) {
  if constexpr (sizeof(T) == 4) {
    const float4 a = *reinterpret_cast<const float4*>(p);
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w;
  } else {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    const T* e = reinterpret_cast<const T*>(&u);
#pragma unroll
    for (int j = 0; j < 4; ++j) f[j] = to_float(e[j]);
  }
}
template <typename T>
__device__ __forceinline__ void store_four(T* __restrict__ p, const float* f) {
  if constexpr (sizeof(T) == 4) {
    *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
  } else {
    uint2 u;
    T* e = reinterpret_cast<T*>(&u);
#pragma unroll
    for (int j = 0; j < 4; ++j) e[j] = from_float<T>(f[j]);
    *reinterpret_cast<uint2*>(p) = u;
  }
}
// sum_slices for four neighbouring elements (16-byte loads; each element's sum in the same order)
__device__ __forceinline__ void sum_slices_four(const float* __restrict__ p, int n_partials,
                                                long long partial_stride, float* v) {
  v[0] = v[1] = v[2] = v[3] = 0.f;
  for (int s0 = 0; s0 < n_partials; s0 += 4) {
    float4 t[4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
      t[j] = s0 + j < n_partials ? *reinterpret_cast<const float4*>(p + (size_t)(s0 + j) * partial_stride)
                                 : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int j = 0; j < 4; ++j) { v[0] += t[j].x; v[1] += t[j].y; v[2] += t[j].z; v[3] += t[j].w; }
  }
}

// VEC: dim is a multiple of four, a thread takes four neighbouring features
template <typename T, bool VEC>
__global__ void token_shift_kernel(const T* __restrict__ h, const float* __restrict__ prev,
                                   const float* __restrict__ mu, T* __restrict__ out,
                                   const int* __restrict__ token_seq, const int* __restrict__ q_start,
                                   const int* __restrict__ seq_slot, int n_tokens, int dim, int n_mix) {
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const int b = token_seq[t];
  const bool first = t == q_start[b];
  const int slot = seq_slot[b];
  pdl_wait();
  if (VEC) {
    for (int i = threadIdx.x * 4; i < dim; i += blockDim.x * 4) {
      float hv[4], pv[4], m[4], o[4];
      load_four(h + (size_t)t * dim + i, hv);
      if (first) load_four(prev + (size_t)slot * dim + i, pv);
      else load_four(h + (size_t)(t - 1) * dim + i, pv);
      for (int s = 0; s < n_mix; ++s) {
        load_four(mu + (size_t)s * dim + i, m);
#pragma unroll
        for (int j = 0; j < 4; ++j) o[j] = fmaf(pv[j] - hv[j], m[j], hv[j]);
        store_four(out + ((size_t)s * n_tokens + t) * dim + i, o);
      }
    }
  } else
  for (int i = threadIdx.x; i < dim; i += blockDim.x) {
    const float hv = to_float(h[(size_t)t * dim + i]);
    const float pv = first ? prev[(size_t)slot * dim + i] : to_float(h[(size_t)(t - 1) * dim + i]);
    const float d = pv - hv;
    for (int s = 0; s < n_mix; ++s)
      out[((size_t)s * n_tokens + t) * dim + i] = from_float<T>(fmaf(d, mu[(size_t)s * dim + i], hv));
  }
}

struct Slices {
  const float* p;
  int n;
  long long stride;
};

// grid (token, part of the row); act [tokens][3 H dk + H dv] = (r | w | k | v), gate [tokens][H dv]
// VEC: H dk and H dv are multiples of four (and the slices 16-byte aligned), a thread takes four
// neighbouring elements of one of the five parts
template <typename T, bool VEC>
__global__ void wkv_gates_kernel(Slices r, Slices k, Slices v, Slices g, Slices z,
                                 const float* __restrict__ w0, float* __restrict__ act,
                                 float* __restrict__ gate, const T* __restrict__ h,
                                 float* __restrict__ prev, const int* __restrict__ token_seq,
                                 const int* __restrict__ q_start, const int* __restrict__ seq_slot,
                                 int n_k, int n_v, int dim) {
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const int b = token_seq[t];
  const bool last = t == q_start[b + 1] - 1;
  const int slot = seq_slot[b];
  pdl_wait();
  const int row = 3 * n_k + n_v;
  const int e_end = min(row + n_v, (int)(blockIdx.y + 1) * 1024);
  if (VEC) {
    for (int e = blockIdx.y * 1024 + threadIdx.x * 4; e < e_end; e += blockDim.x * 4) {
      float a[4];
      if (e >= row) {
        const int i = e - row;
        sum_slices_four(g.p + (size_t)t * n_v + i, g.n, g.stride, a);
#pragma unroll
        for (int j = 0; j < 4; ++j) a[j] = a[j] / (1.0f + expf(-a[j]));
        store_four(gate + (size_t)t * n_v + i, a);
        continue;
      }
      if (e < n_k) {
        sum_slices_four(r.p + (size_t)t * n_k + e, r.n, r.stride, a);
      } else if (e < 2 * n_k) {
        const int i = e - n_k;
        float w[4];
        sum_slices_four(z.p + (size_t)t * n_k + i, z.n, z.stride, a);
        load_four(w0 + i, w);
#pragma unroll
        for (int j = 0; j < 4; ++j) a[j] = expf(-expf(a[j] + w[j]));
      } else if (e < 3 * n_k) {
        sum_slices_four(k.p + (size_t)t * n_k + (e - 2 * n_k), k.n, k.stride, a);
      } else {
        sum_slices_four(v.p + (size_t)t * n_v + (e - 3 * n_k), v.n, v.stride, a);
      }
      store_four(act + (size_t)t * row + e, a);
    }
  } else
  for (int e = blockIdx.y * 1024 + threadIdx.x; e < e_end; e += blockDim.x) {
    if (e < n_k) {
      act[(size_t)t * row + e] = sum_slices(r.p + (size_t)t * n_k + e, r.n, r.stride);
    } else if (e < 2 * n_k) {
      const int i = e - n_k;
      const float zz = sum_slices(z.p + (size_t)t * n_k + i, z.n, z.stride) + w0[i];
      act[(size_t)t * row + e] = expf(-expf(zz));
    } else if (e < 3 * n_k) {
      const int i = e - 2 * n_k;
      act[(size_t)t * row + e] = sum_slices(k.p + (size_t)t * n_k + i, k.n, k.stride);
    } else if (e < row) {
      const int i = e - 3 * n_k;
      act[(size_t)t * row + e] = sum_slices(v.p + (size_t)t * n_v + i, v.n, v.stride);
    } else {
      const int i = e - row;
      const float gv = sum_slices(g.p + (size_t)t * n_v + i, g.n, g.stride);
      gate[(size_t)t * n_v + i] = gv / (1.0f + expf(-gv));
    }
  }
  if (last && blockIdx.y == 0)
    for (int i = threadIdx.x; i < dim; i += blockDim.x) prev[(size_t)slot * dim + i] = to_float(h[(size_t)t * dim + i]);
}

template <int RPT, int VEC>
__global__ void __launch_bounds__(256)
wkv_scan_kernel(const float* __restrict__ act, const float* __restrict__ bonus,
                const int* __restrict__ q_start, const int* __restrict__ seq_slot,
                float* __restrict__ state, float* __restrict__ out, int H, int dk, int dv) {
  pdl_launch_dependents();
  constexpr int DKP = 32 * RPT;                       // rows, padded
  constexpr int PER_TOK = 3 * DKP + RC_COLS;          // r, w, k, then this block's v columns
  extern __shared__ __align__(16) float stage[];      // [RC_STAGES][RC_TOK][PER_TOK]
  const int b = blockIdx.z, h = blockIdx.y, c0 = blockIdx.x * RC_COLS;
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int col = c0 + w * RC_CPW;
  const int slot = seq_slot[b];
  const int t0 = q_start[b], t1 = q_start[b + 1];
  const int row = 3 * H * dk + H * dv;
  // rows beyond dk: r = k = w = 0 for ever (never copied over); their state stays zero
  if (dk < DKP) {
    for (int i = threadIdx.x; i < RC_STAGES * RC_TOK * PER_TOK; i += blockDim.x) stage[i] = 0.f;
    __syncthreads();
  }
  const int per = 3 * dk + RC_COLS;
  int src_off[4], dst_off[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int e = (threadIdx.x + k * 256) * VEC;
    src_off[k] = dst_off[k] = -1;
    if (e < 3 * dk) {
      const int which = e / dk, i = e - which * dk;
      src_off[k] = which * H * dk + h * dk + i;
      dst_off[k] = which * DKP + i;
    } else if (e < per && c0 + (e - 3 * dk) < dv) {
      src_off[k] = 3 * H * dk + h * dv + c0 + (e - 3 * dk);
      dst_off[k] = 3 * DKP + (e - 3 * dk);
    }
  }
  float U[RPT];
#pragma unroll
  for (int r = 0; r < RPT; ++r) {
    const int i = lane * RPT + r;
    U[r] = i < dk ? bonus[h * dk + i] : 0.f;
  }
  pdl_wait();
  float S[RPT][RC_CPW];
  float* st = state + (((size_t)slot * H + h) * dk) * dv + col;
#pragma unroll
  for (int r = 0; r < RPT; ++r)
#pragma unroll
    for (int c = 0; c < RC_CPW; ++c) {
      const int i = lane * RPT + r;
      S[r][c] = (col + c < dv && i < dk) ? st[(size_t)i * dv + c] : 0.f;
    }
  const int n_groups = (t1 - t0 + RC_TOK - 1) / RC_TOK;
  auto issue = [&](int g) {
    if (g < n_groups) {
      const int base = t0 + g * RC_TOK;
      const int nt = min(RC_TOK, t1 - base);
      float* dst = stage + (size_t)(g % RC_STAGES) * RC_TOK * PER_TOK;
      const float* src = act + (size_t)base * row;
#pragma unroll
      for (int k = 0; k < 4; ++k)
        if (src_off[k] >= 0)
          for (int tt = 0; tt < nt; ++tt)
            cp_async<4 * VEC>(dst + tt * PER_TOK + dst_off[k], src + (size_t)tt * row + src_off[k]);
    }
    cp_async_commit();
  };
  issue(0);
  issue(1);
  for (int g = 0; g < n_groups; ++g) {
    cp_async_wait<RC_STAGES - 2>();
    __syncthreads();                                   // stage g has landed; stage g - 1 is no longer read
    issue(g + 2);
    const int base = t0 + g * RC_TOK;
    const int nt = min(RC_TOK, t1 - base);
    const float* sg = stage + (size_t)(g % RC_STAGES) * RC_TOK * PER_TOK;
    float o[RC_TOK][RC_CPW];
#pragma unroll
    for (int tt = 0; tt < RC_TOK; ++tt) {
#pragma unroll
      for (int c = 0; c < RC_CPW; ++c) o[tt][c] = 0.f;
      if (tt < nt) {
        const float* rr = sg + tt * PER_TOK + lane * RPT;
        const float* ww = rr + DKP;
        const float* kk = rr + 2 * DKP;
        float vj[RC_CPW];
#pragma unroll
        for (int c = 0; c < RC_CPW; ++c) vj[c] = sg[tt * PER_TOK + 3 * DKP + w * RC_CPW + c];
#pragma unroll
        for (int r = 0; r < RPT; ++r) {
          const float ri = rr[r], wi = ww[r], ki = kk[r];
#pragma unroll
          for (int c = 0; c < RC_CPW; ++c) {
            const float kv = ki * vj[c];
            o[tt][c] = fmaf(ri, fmaf(U[r], kv, S[r][c]), o[tt][c]);
            S[r][c] = fmaf(wi, S[r][c], kv);
          }
        }
      }
    }
    // the 32 lanes' partial sums of the group's 32 outputs, as in recurrence_scan_kernel
    static_assert(RC_TOK * RC_CPW == 32, "one output per lane");
    float* ov = &o[0][0];
#pragma unroll
    for (int half = 16; half >= 1; half >>= 1) {
      const bool upper = (lane & half) != 0;
#pragma unroll
      for (int i = 0; i < half; ++i) {
        const float send = upper ? ov[i] : ov[i + half];
        const float keep = upper ? ov[i + half] : ov[i];
        ov[i] = keep + __shfl_xor_sync(0xffffffffu, send, half);
      }
    }
    {
      const int tt = lane / RC_CPW, c = lane % RC_CPW;
      if (tt < nt && col + c < dv) out[((size_t)(base + tt) * H + h) * dv + col + c] = ov[0];
    }
  }
  cp_async_wait<0>();
#pragma unroll
  for (int r = 0; r < RPT; ++r)
#pragma unroll
    for (int c = 0; c < RC_CPW; ++c) {
      const int i = lane * RPT + r;
      if (col + c < dv && i < dk) st[(size_t)i * dv + c] = S[r][c];
    }
}

// a warp per (token, head)
template <typename TO>
__global__ void wkv_out_kernel(const float* __restrict__ o, const float* __restrict__ w,
                               const float* __restrict__ gate, TO* __restrict__ out,
                               long long n_heads_total, int heads, int size, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  const long long head = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (head >= n_heads_total) return;
  const int lane = threadIdx.x & 31;
  const float* src = o + head * size;
  const float* wh = w + (head % heads) * size;
  float ss = 0.f;
  for (int i = lane; i < size; i += 32) ss += src[i] * src[i];
  ss = warp_sum(ss);
  const float rs = 1.0f / sqrtf(ss / (float)size + eps);
  for (int i = lane; i < size; i += 32)
    out[head * size + i] = from_float<TO>(src[i] * rs * wh[i] * gate[head * size + i]);
}

}  // namespace yalm

using namespace yalm;

// proj: float32 slices [n_partials][tokens][2 H dk + H dv] = (q | f | v); f_bias, lower [H dk];
// act: float32 scratch [tokens][2 H dk + H dv] (the activated projection); state
// [slots][H][dk][dv] float32, read at the step's start and written at its end; out float32
// [tokens][H dv].  dk up to 512.
extern "C" int yalm_gated_recurrence(const float* proj, int n_partials, long long partial_stride,
                                     const float* f_bias, const float* lower, float* act,
                                     const int* q_start, const int* seq_slot, float* state, float* out,
                                     int n_tokens, int n_seqs, int H, int dk, int dv, cudaStream_t stream) {
  if (n_seqs <= 0 || n_tokens <= 0) return 0;
  if (H <= 0 || dk <= 0 || dv <= 0 || dk > 512 || n_seqs > 65535 || H > 65535) return -2;
  const int row = 2 * H * dk + H * dv;
  if ((row + 1023) / 1024 > 65535) return -4;
  launch_pdl(recurrence_gates_kernel, dim3(n_tokens, (row + 1023) / 1024), dim3(256), 0, stream, proj,
             n_partials, partial_stride, f_bias, lower, act, row, H * dk);
  YALM_LAUNCH_CHECK();
  const dim3 grid((dv + RC_COLS - 1) / RC_COLS, H, n_seqs), block(256);
  const int rpt = (dk + 31) / 32;
  // 16-byte copies where every run starts on a 16-byte boundary; a thread copies up to five runs per token
  const bool vec = dk % 4 == 0 && dv % 4 == 0 && (((uintptr_t)act) & 15) == 0;
  if ((2 * dk + RC_COLS + (vec ? 3 : 0)) / (vec ? 4 : 1) > 5 * 256) return -2;
#define YALM_REC(R)                                                                                 \
  do {                                                                                              \
    const size_t smem = (size_t)RC_STAGES * RC_TOK * (2 * 32 * R + RC_COLS) * sizeof(float);        \
    static bool set = false;                                                                        \
    if (!set && smem > 48 * 1024) {                                                                 \
      cudaError_t e = cudaFuncSetAttribute(recurrence_scan_kernel<R, 4>,                            \
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
      if (e == cudaSuccess)                                                                         \
        e = cudaFuncSetAttribute(recurrence_scan_kernel<R, 1>,                                      \
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);           \
      if (e != cudaSuccess) return (int)e;                                                          \
      set = true;                                                                                   \
    }                                                                                               \
    if (vec)                                                                                        \
      launch_pdl(recurrence_scan_kernel<R, 4>, grid, block, smem, stream, (const float*)act,        \
                 q_start, seq_slot, state, out, H, dk, dv);                                         \
    else                                                                                            \
      launch_pdl(recurrence_scan_kernel<R, 1>, grid, block, smem, stream, (const float*)act,        \
                 q_start, seq_slot, state, out, H, dk, dv);                                         \
  } while (0)
  if (rpt <= 1) YALM_REC(1);
  else if (rpt <= 2) YALM_REC(2);
  else if (rpt <= 4) YALM_REC(4);
  else if (rpt <= 8) YALM_REC(8);
  else YALM_REC(16);
#undef YALM_REC
  YALM_LAUNCH_CHECK();
  return 0;
}

// out [n_mix][tokens][dim] = h + (h' - h) mu[s]; h' the previous token's row, for a step's first
// token the sequence's prev [slots][dim] (float32)
extern "C" int yalm_token_shift(const void* h, const float* prev, const float* mu, void* out, int dtype,
                                const int* token_seq, const int* q_start, const int* seq_slot,
                                int n_tokens, int dim, int n_mix, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (dim <= 0 || n_mix <= 0) return -2;
  const bool vec = dim % 4 == 0 && ((((uintptr_t)h) | ((uintptr_t)prev) | ((uintptr_t)mu) | ((uintptr_t)out)) & 15) == 0;
  int threads = ((vec ? dim / 4 : dim) + 31) / 32 * 32;
  if (threads > 512) threads = 512;
  const dim3 grid(n_tokens), block(threads);
#define YALM_SHIFT(T, VEC)                                                                           \
  launch_pdl(token_shift_kernel<T, VEC>, grid, block, 0, stream, (const T*)h, prev, mu, (T*)out,     \
             token_seq, q_start, seq_slot, n_tokens, dim, n_mix)
  if (dtype == DT_F32) { if (vec) YALM_SHIFT(float, true); else YALM_SHIFT(float, false); }
  else if (dtype == DT_BF16) { if (vec) YALM_SHIFT(__nv_bfloat16, true); else YALM_SHIFT(__nv_bfloat16, false); }
  else if (dtype == DT_F16) { if (vec) YALM_SHIFT(__half, true); else YALM_SHIFT(__half, false); }
  else return -3;
#undef YALM_SHIFT
  YALM_LAUNCH_CHECK();
  return 0;
}

// The recurrence of a step: r, k, z [.][tokens][H dk] and v, g [.][tokens][H dv] are float32 slices
// of the five projections (z before + w0 and exp(-exp(.))); bonus [H][dk]; act: float32 scratch
// [tokens][3 H dk + H dv]; gate: float32 out [tokens][H dv] = silu(g); state [slots][H][dk][dv];
// out float32 [tokens][H dv]; h [tokens][dim] (h_dtype) is the mixer's input, whose last row per
// sequence goes to prev [slots][dim].  dk up to 256.
extern "C" int yalm_wkv(const float* r, int nr, long long sr, const float* k, int nk, long long sk,
                        const float* v, int nv, long long sv, const float* g, int ng, long long sg,
                        const float* z, int nz, long long sz, const float* w0, const float* bonus,
                        float* act, float* gate, const void* h, int h_dtype, float* prev,
                        const int* token_seq, const int* q_start, const int* seq_slot, float* state,
                        float* out, int n_tokens, int n_seqs, int H, int dk, int dv, int dim,
                        cudaStream_t stream) {
  if (n_seqs <= 0 || n_tokens <= 0) return 0;
  if (H <= 0 || dk <= 0 || dv <= 0 || dk > 256 || n_seqs > 65535 || H > 65535 || dim <= 0) return -2;
  const int row = 3 * H * dk + H * dv;
  const int parts = (row + H * dv + 1023) / 1024;
  if (parts > 65535) return -4;
  const Slices R = {r, nr, sr}, K = {k, nk, sk}, V = {v, nv, sv}, G = {g, ng, sg}, Z = {z, nz, sz};
  const dim3 ggrid(n_tokens, parts), gblock(256);
  const bool gvec = (H * dk) % 4 == 0 && (H * dv) % 4 == 0 && ((sr | sk | sv | sg | sz) & 3) == 0 &&
                    ((((uintptr_t)r) | ((uintptr_t)k) | ((uintptr_t)v) | ((uintptr_t)g) | ((uintptr_t)z) |
                      ((uintptr_t)w0) | ((uintptr_t)act) | ((uintptr_t)gate)) & 15) == 0;
#define YALM_GATES(T, VEC)                                                                           \
  launch_pdl(wkv_gates_kernel<T, VEC>, ggrid, gblock, 0, stream, R, K, V, G, Z, w0, act, gate,       \
             (const T*)h, prev, token_seq, q_start, seq_slot, H * dk, H * dv, dim)
  if (h_dtype == DT_F32) { if (gvec) YALM_GATES(float, true); else YALM_GATES(float, false); }
  else if (h_dtype == DT_BF16) { if (gvec) YALM_GATES(__nv_bfloat16, true); else YALM_GATES(__nv_bfloat16, false); }
  else if (h_dtype == DT_F16) { if (gvec) YALM_GATES(__half, true); else YALM_GATES(__half, false); }
  else return -3;
#undef YALM_GATES
  YALM_LAUNCH_CHECK();
  const dim3 grid((dv + RC_COLS - 1) / RC_COLS, H, n_seqs), block(256);
  const int rpt = (dk + 31) / 32;
  const bool vec = dk % 4 == 0 && dv % 4 == 0 && (((uintptr_t)act) & 15) == 0;
  if ((3 * dk + RC_COLS + (vec ? 3 : 0)) / (vec ? 4 : 1) > 4 * 256) return -2;
#define YALM_WKV(R)                                                                                 \
  do {                                                                                              \
    const size_t smem = (size_t)RC_STAGES * RC_TOK * (3 * 32 * R + RC_COLS) * sizeof(float);        \
    static bool set = false;                                                                        \
    if (!set && smem > 48 * 1024) {                                                                 \
      cudaError_t e = cudaFuncSetAttribute(wkv_scan_kernel<R, 4>,                                   \
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
      if (e == cudaSuccess)                                                                         \
        e = cudaFuncSetAttribute(wkv_scan_kernel<R, 1>,                                             \
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);           \
      if (e != cudaSuccess) return (int)e;                                                          \
      set = true;                                                                                   \
    }                                                                                               \
    if (vec)                                                                                        \
      launch_pdl(wkv_scan_kernel<R, 4>, grid, block, smem, stream, (const float*)act, bonus,        \
                 q_start, seq_slot, state, out, H, dk, dv);                                         \
    else                                                                                            \
      launch_pdl(wkv_scan_kernel<R, 1>, grid, block, smem, stream, (const float*)act, bonus,        \
                 q_start, seq_slot, state, out, H, dk, dv);                                         \
  } while (0)
  if (rpt <= 1) YALM_WKV(1);
  else if (rpt <= 2) YALM_WKV(2);
  else if (rpt <= 4) YALM_WKV(4);
  else YALM_WKV(8);
#undef YALM_WKV
  YALM_LAUNCH_CHECK();
  return 0;
}

// out [rows, heads * size] = each head's `size` values of o (float32) over their root mean square,
// times w [heads * size], times gate [rows, heads * size] (float32)
extern "C" int yalm_wkv_out(const float* o, const float* w, const float* gate, void* out, int out_dtype,
                            long long rows, int heads, int size, float eps, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (heads <= 0 || size <= 0) return -2;
  const long long total = rows * heads;
  const long long blocks = (total + 7) / 8;
  if (blocks > 0x7fffffffLL) return -4;
  const dim3 grid((unsigned)blocks), block(256);
  if (out_dtype == DT_F32)
    launch_pdl(wkv_out_kernel<float>, grid, block, 0, stream, o, w, gate, (float*)out, total, heads, size, eps);
  else if (out_dtype == DT_BF16)
    launch_pdl(wkv_out_kernel<__nv_bfloat16>, grid, block, 0, stream, o, w, gate, (__nv_bfloat16*)out, total,
               heads, size, eps);
  else if (out_dtype == DT_F16)
    launch_pdl(wkv_out_kernel<__half>, grid, block, 0, stream, o, w, gate, (__half*)out, total, heads, size, eps);
  else return -3;
  YALM_LAUNCH_CHECK();
  return 0;
}
