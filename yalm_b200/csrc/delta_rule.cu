// The gated delta rule with a decay per key channel, per head with key size dk and value size dv:
//   S <- diag(g_t) S;   u = beta_t (v_t - S^T k_t);   S <- S + k_t u^T;   o_t = S^T q_t
// S [dk, dv] per head and sequence in 32-bit floats, carried from step to step.  Query/key heads may
// be fewer than value heads: head h reads q/k head h / (H / G).  Everything here is 32-bit.
//
//  * delta_prep: q and k of every token and q/k head become unit vectors (x / sqrt(sum x^2 + 1e-6)),
//    q times 1/sqrt(dk); beta = sigmoid(.); and the two low-rank projections' first halves go out in
//    the storage type as the input of their second halves;
//  * delta_decay: the decay per head and key channel, kept as g - 1 = expm1(-exp(A_h) softplus(z + dt))
//    (a decay close to 1 has few bits of its own left in g; S + (g - 1) S keeps them), and the output
//    gate sigmoid(.) per head and value channel;
//  * delta_scan: the recurrence.  As in the other scans of this library a block owns 16 value
//    columns of one (sequence, head) -- the columns of S are independent of one another -- and the
//    step's tokens come through a three-stage cp.async ring.  Unlike a plain linear recurrence the write
//    needs k.S first, so every token costs one all-reduce before its update; the outputs' sums are
//    formed for 16 tokens at once.  Key sizes up to 128 run with eight lanes per column
//    (delta_scan8_kernel), larger ones with a warp per two columns (delta_scan_kernel).
//
// The activated row of a token, float32: [q: G dk | k: G dk | v: H dv | beta: H padded to 4 | g - 1: H dk].
#include "api.h"
#include "common.cuh"

namespace yalm {

constexpr int DR_CPW = 2;
constexpr int DR_COLS = 8 * DR_CPW;
constexpr int DR_TOK = 16;
constexpr int DR_STAGES = 3;

__device__ __forceinline__ float softplus_f(float v) { return v > 20.f ? v : log1pf(expf(v)); }

// grid (tokens); a warp per q/k head for the unit vectors, then the block's threads for the rest.
// proj: slices [.][tokens][proj_row] with beta at col_b (H), the low-rank inputs at col_low (n_low)
template <typename T>
__global__ void delta_prep_kernel(float* __restrict__ act, int row, const float* __restrict__ proj,
                                  int n_partials, long long partial_stride, int proj_row, int col_b,
                                  int col_low, int n_low, T* __restrict__ low, int H, int G, int dk, int dv) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
  float* a = act + (size_t)t * row;
  const float q_scale = 1.0f / sqrtf((float)dk);
  for (int head = warp; head < 2 * G; head += n_warps) {
    float* v = a + (size_t)head * dk;                       // q heads, then k heads
    float ss = 0.f;
    for (int i = lane; i < dk; i += 32) ss += v[i] * v[i];
    ss = warp_sum(ss);
    const float r = (1.0f / sqrtf(ss + 1e-6f)) * (head < G ? q_scale : 1.0f);
    for (int i = lane; i < dk; i += 32) v[i] *= r;
  }
  const float* p = proj + (size_t)t * proj_row;
  const int beta0 = 2 * G * dk + H * dv;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    const float z = sum_slices(p + col_b + i, n_partials, partial_stride);
    a[beta0 + i] = 1.0f / (1.0f + expf(-z));
  }
  for (int i = threadIdx.x; i < n_low; i += blockDim.x)
    low[(size_t)t * n_low + i] = from_float<T>(sum_slices(p + col_low + i, n_partials, partial_stride));
}

// grid (tokens, parts); z: slices [.][tokens][H dk + H dv] = (decay logits | gate logits)
__global__ void delta_decay_kernel(float* __restrict__ act, int row, int decay0, const float* __restrict__ z,
                                   int n_partials, long long partial_stride, const float* __restrict__ dt_bias,
                                   const float* __restrict__ a_log, float* __restrict__ gate, int H, int dk,
                                   int dv) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int n_k = H * dk, n_v = H * dv;
  const float* zr = z + (size_t)t * (n_k + n_v);
  const int e_end = min(n_k + n_v, (int)(blockIdx.y + 1) * 1024);
  for (int e = blockIdx.y * 1024 + threadIdx.x; e < e_end; e += blockDim.x) {
    const float v = n_partials == 1 ? zr[e] : sum_slices(zr + e, n_partials, partial_stride);
    if (e < n_k) act[(size_t)t * row + decay0 + e] = expm1f(-expf(a_log[e / dk]) * softplus_f(v + dt_bias[e]));
    else gate[(size_t)t * n_v + (e - n_k)] = 1.0f / (1.0f + expf(-v));
  }
}

template <int BYTES>
__device__ __forceinline__ void dr_cp_async(float* dst, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], %2;" ::"r"(smem_u32(dst)), "l"(src), "n"(BYTES) : "memory");
}
__device__ __forceinline__ void dr_cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void dr_cp_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// A lane's RPT neighbouring rows of a staged vector, as one 8- or 16-byte access per two or four rows:
// single-float loads at a stride of RPT floats would meet RPT-fold bank conflicts.
template <int RPT>
__device__ __forceinline__ void lane_rows(const float* __restrict__ p, float* out) {
  if constexpr (RPT % 4 == 0) {
#pragma unroll
    for (int r = 0; r < RPT; r += 4) {
      const float4 v = *reinterpret_cast<const float4*>(p + r);
      out[r] = v.x; out[r + 1] = v.y; out[r + 2] = v.z; out[r + 3] = v.w;
    }
  } else if constexpr (RPT == 2) {
    const float2 v = *reinterpret_cast<const float2*>(p);
    out[0] = v.x; out[1] = v.y;
  } else {
#pragma unroll
    for (int r = 0; r < RPT; ++r) out[r] = p[r];
  }
}

// VEC: floats per copy (4 when every run starts on a 16-byte boundary, else 1)
template <int RPT, int VEC>
__global__ void __launch_bounds__(256)
delta_scan_kernel(const float* __restrict__ act, int row, const int* __restrict__ q_start,
                  const int* __restrict__ seq_slot, float* __restrict__ state, float* __restrict__ out,
                  int H, int G, int dk, int dv) {
  pdl_launch_dependents();
  constexpr int DKP = 32 * RPT;                       // rows, padded
  constexpr int PER_TOK = 3 * DKP + DR_COLS + 4;      // q, k, g, this block's v columns, beta (+ padding)
  extern __shared__ __align__(16) float stage[];      // [DR_STAGES][DR_TOK][PER_TOK]
  const int b = blockIdx.z, h = blockIdx.y, c0 = blockIdx.x * DR_COLS;
  const int hq = h / (H / G);
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int col = c0 + w * DR_CPW;
  const int slot = seq_slot[b];
  const int t0 = q_start[b], t1 = q_start[b + 1];
  const int hp = (H + 3) & ~3;
  // rows beyond dk: q = k = 0 for ever (never copied over), so their state stays zero
  if (dk < DKP) {
    for (int i = threadIdx.x; i < DR_STAGES * DR_TOK * PER_TOK; i += blockDim.x) stage[i] = 0.f;
    __syncthreads();
  }
  // what this thread copies of every token: up to four runs of VEC floats, and thread 0 the beta
  const int per = 3 * dk + DR_COLS;
  int src_off[4], dst_off[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int e = (threadIdx.x + k * 256) * VEC;
    src_off[k] = dst_off[k] = -1;
    if (e < dk) { src_off[k] = hq * dk + e; dst_off[k] = e; }
    else if (e < 2 * dk) { src_off[k] = G * dk + hq * dk + (e - dk); dst_off[k] = DKP + (e - dk); }
    else if (e < 3 * dk) { src_off[k] = 2 * G * dk + H * dv + hp + h * dk + (e - 2 * dk); dst_off[k] = 2 * DKP + (e - 2 * dk); }
    else if (e < per && c0 + (e - 3 * dk) < dv) {
      src_off[k] = 2 * G * dk + h * dv + c0 + (e - 3 * dk);
      dst_off[k] = 3 * DKP + (e - 3 * dk);
    }
  }
  const int beta_off = 2 * G * dk + H * dv + h;
  pdl_wait();
  float S[RPT][DR_CPW];
  float* st = state + (((size_t)slot * H + h) * dk) * dv + col;
#pragma unroll
  for (int r = 0; r < RPT; ++r)
#pragma unroll
    for (int c = 0; c < DR_CPW; ++c) {
      const int i = lane * RPT + r;
      S[r][c] = (col + c < dv && i < dk) ? st[(size_t)i * dv + c] : 0.f;
    }
  const int n_groups = (t1 - t0 + DR_TOK - 1) / DR_TOK;
  auto issue = [&](int g) {
    if (g < n_groups) {
      const int base = t0 + g * DR_TOK;
      const int nt = min(DR_TOK, t1 - base);
      float* dst = stage + (size_t)(g % DR_STAGES) * DR_TOK * PER_TOK;
      const float* src = act + (size_t)base * row;
#pragma unroll
      for (int k = 0; k < 4; ++k)
        if (src_off[k] >= 0)
          for (int tt = 0; tt < nt; ++tt)
            dr_cp_async<4 * VEC>(dst + tt * PER_TOK + dst_off[k], src + (size_t)tt * row + src_off[k]);
      if (threadIdx.x < nt)
        dr_cp_async<4>(dst + threadIdx.x * PER_TOK + 3 * DKP + DR_COLS, src + (size_t)threadIdx.x * row + beta_off);
    }
    dr_cp_commit();
  };
  issue(0);
  issue(1);
  for (int g = 0; g < n_groups; ++g) {
    dr_cp_wait<DR_STAGES - 2>();
    __syncthreads();                                   // stage g has landed; stage g - 1 is no longer read
    issue(g + 2);
    const int base = t0 + g * DR_TOK;
    const int nt = min(DR_TOK, t1 - base);
    const float* sg = stage + (size_t)(g % DR_STAGES) * DR_TOK * PER_TOK;
    float o[DR_TOK][DR_CPW];
    auto token = [&](int tt) {
      const float* qq = sg + tt * PER_TOK + lane * RPT;
      const float* kk = qq + DKP;
      const float* gg = qq + 2 * DKP;
      const float beta = sg[tt * PER_TOK + 3 * DKP + DR_COLS];
      float vj[DR_CPW], kd[DR_CPW], kr[RPT], qr[RPT], gr[RPT];
      lane_rows<RPT>(qq, qr);
      lane_rows<RPT>(kk, kr);
      lane_rows<RPT>(gg, gr);
#pragma unroll
      for (int c = 0; c < DR_CPW; ++c) { vj[c] = sg[tt * PER_TOK + 3 * DKP + w * DR_CPW + c]; kd[c] = 0.f; }
#pragma unroll
      for (int r = 0; r < RPT; ++r) {
        const float gi = gr[r];
#pragma unroll
        for (int c = 0; c < DR_CPW; ++c) {
          S[r][c] = fmaf(gi, S[r][c], S[r][c]);
          kd[c] = fmaf(kr[r], S[r][c], kd[c]);
        }
      }
#pragma unroll
      for (int off = 16; off > 0; off >>= 1)
#pragma unroll
        for (int c = 0; c < DR_CPW; ++c) kd[c] += __shfl_xor_sync(0xffffffffu, kd[c], off);
      float u[DR_CPW];
#pragma unroll
      for (int c = 0; c < DR_CPW; ++c) u[c] = beta * (vj[c] - kd[c]);
#pragma unroll
      for (int r = 0; r < RPT; ++r)
#pragma unroll
        for (int c = 0; c < DR_CPW; ++c) {
          S[r][c] = fmaf(kr[r], u[c], S[r][c]);
          o[tt][c] = fmaf(S[r][c], qr[r], o[tt][c]);
        }
    };
#pragma unroll
    for (int tt = 0; tt < DR_TOK; ++tt)
#pragma unroll
      for (int c = 0; c < DR_CPW; ++c) o[tt][c] = 0.f;
    if (nt == DR_TOK) {                                // a full group: no test between the tokens, so that a
#pragma unroll                                         // token's rows are loaded while the one before is reduced
      for (int tt = 0; tt < DR_TOK; ++tt) token(tt);
    } else {
#pragma unroll
      for (int tt = 0; tt < DR_TOK; ++tt)
        if (tt < nt) token(tt);
    }
    // the 32 lanes' partial sums of the group's 32 outputs: in every round a lane hands half of its
    // values to its partner and adds the partner's other half to its own
    static_assert(DR_TOK * DR_CPW == 32, "one output per lane");
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
      const int tt = lane / DR_CPW, c = lane % DR_CPW;
      if (tt < nt && col + c < dv) out[((size_t)(base + tt) * H + h) * dv + col + c] = ov[0];
    }
  }
  dr_cp_wait<0>();
#pragma unroll
  for (int r = 0; r < RPT; ++r)
#pragma unroll
    for (int c = 0; c < DR_CPW; ++c) {
      const int i = lane * RPT + r;
      if (col + c < dv && i < dk) st[(size_t)i * dv + c] = S[r][c];
    }
}

// The same recurrence with EIGHT lanes per value column (key sizes up to 128): a warp owns four columns,
// a lane RPL = 4, 8 or 16 neighbouring rows of one column.  The all-reduce of k.S that every token's
// write waits for then takes three exchange rounds for one value instead of five rounds for two, and
// a token costs a third fewer instructions per column (measured at 16 heads of 128 x 128, 2,048 tokens:
// 439 us with 32 lanes per column).  A block of four warps owns 16 columns, so the grid is the same.
constexpr int D8_WARPS = 4;
constexpr int D8_COLS = 4 * D8_WARPS;

template <int RPL, int VEC>
__global__ void __launch_bounds__(32 * D8_WARPS)
delta_scan8_kernel(const float* __restrict__ act, int row, const int* __restrict__ q_start,
                   const int* __restrict__ seq_slot, float* __restrict__ state, float* __restrict__ out,
                   int H, int G, int dk, int dv) {
  pdl_launch_dependents();
  constexpr int DKP = 8 * RPL;                        // rows, padded
  constexpr int PER_TOK = 3 * DKP + D8_COLS + 4;      // q, k, g - 1, this block's v columns, beta (+ padding)
  constexpr int NT = 32 * D8_WARPS;
  extern __shared__ __align__(16) float stage[];      // [DR_STAGES][DR_TOK][PER_TOK]
  const int b = blockIdx.z, h = blockIdx.y, c0 = blockIdx.x * D8_COLS;
  const int hq = h / (H / G);
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int cg = lane >> 3, sub = lane & 7;
  const int col = c0 + w * 4 + cg;
  const int slot = seq_slot[b];
  const int t0 = q_start[b], t1 = q_start[b + 1];
  const int hp = (H + 3) & ~3;
  if (dk < DKP) {                                     // rows beyond dk: q = k = 0 for ever, their state stays zero
    for (int i = threadIdx.x; i < DR_STAGES * DR_TOK * PER_TOK; i += NT) stage[i] = 0.f;
    __syncthreads();
  }
  const int per = 3 * dk + D8_COLS;
  int src_off[4], dst_off[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int e = (threadIdx.x + k * NT) * VEC;
    src_off[k] = dst_off[k] = -1;
    if (e < dk) { src_off[k] = hq * dk + e; dst_off[k] = e; }
    else if (e < 2 * dk) { src_off[k] = G * dk + hq * dk + (e - dk); dst_off[k] = DKP + (e - dk); }
    else if (e < 3 * dk) { src_off[k] = 2 * G * dk + H * dv + hp + h * dk + (e - 2 * dk); dst_off[k] = 2 * DKP + (e - 2 * dk); }
    else if (e < per && c0 + (e - 3 * dk) < dv) {
      src_off[k] = 2 * G * dk + h * dv + c0 + (e - 3 * dk);
      dst_off[k] = 3 * DKP + (e - 3 * dk);
    }
  }
  const int beta_off = 2 * G * dk + H * dv + h;
  pdl_wait();
  float S[RPL];                                       // register r holds row 4 (sub + 8 (r / 4)) + r % 4
  float* st = state + (((size_t)slot * H + h) * dk) * dv + col;
#pragma unroll
  for (int r = 0; r < RPL; ++r) {
    const int i = 4 * (sub + 8 * (r >> 2)) + (r & 3);
    S[r] = (col < dv && i < dk) ? st[(size_t)i * dv] : 0.f;
  }
  const int n_groups = (t1 - t0 + DR_TOK - 1) / DR_TOK;
  auto issue = [&](int g) {
    if (g < n_groups) {
      const int base = t0 + g * DR_TOK;
      const int nt = min(DR_TOK, t1 - base);
      float* dst = stage + (size_t)(g % DR_STAGES) * DR_TOK * PER_TOK;
      const float* src = act + (size_t)base * row;
#pragma unroll
      for (int k = 0; k < 4; ++k)
        if (src_off[k] >= 0)
          for (int tt = 0; tt < nt; ++tt)
            dr_cp_async<4 * VEC>(dst + tt * PER_TOK + dst_off[k], src + (size_t)tt * row + src_off[k]);
      if (threadIdx.x < nt)
        dr_cp_async<4>(dst + threadIdx.x * PER_TOK + 3 * DKP + D8_COLS, src + (size_t)threadIdx.x * row + beta_off);
    }
    dr_cp_commit();
  };
  issue(0);
  issue(1);
  for (int g = 0; g < n_groups; ++g) {
    dr_cp_wait<DR_STAGES - 2>();
    __syncthreads();                                   // stage g has landed; stage g - 1 is no longer read
    issue(g + 2);
    const int base = t0 + g * DR_TOK;
    const int nt = min(DR_TOK, t1 - base);
    const float* sg = stage + (size_t)(g % DR_STAGES) * DR_TOK * PER_TOK;
    float o[DR_TOK];
    auto token = [&](int tt) {
      // a lane's rows are every eighth group of four: the eight lanes of a column then read 128
      // neighbouring bytes at a time (RPL rows in a row per lane would meet four-fold bank conflicts)
      const float* qq = sg + tt * PER_TOK + 4 * sub;
      float qr[RPL], kr[RPL], gr[RPL];
#pragma unroll
      for (int j = 0; j < RPL / 4; ++j) {
        lane_rows<4>(qq + 32 * j, qr + 4 * j);
        lane_rows<4>(qq + DKP + 32 * j, kr + 4 * j);
        lane_rows<4>(qq + 2 * DKP + 32 * j, gr + 4 * j);
      }
      const float beta = sg[tt * PER_TOK + 3 * DKP + D8_COLS];
      const float vj = sg[tt * PER_TOK + 3 * DKP + w * 4 + cg];
      float kd[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int r = 0; r < RPL; ++r) {
        S[r] = fmaf(gr[r], S[r], S[r]);
        kd[r & 3] = fmaf(kr[r], S[r], kd[r & 3]);
      }
      float kdot = (kd[0] + kd[1]) + (kd[2] + kd[3]);
      kdot += __shfl_xor_sync(0xffffffffu, kdot, 4);
      kdot += __shfl_xor_sync(0xffffffffu, kdot, 2);
      kdot += __shfl_xor_sync(0xffffffffu, kdot, 1);
      const float u = beta * (vj - kdot);
      float od[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int r = 0; r < RPL; ++r) {
        S[r] = fmaf(kr[r], u, S[r]);
        od[r & 3] = fmaf(S[r], qr[r], od[r & 3]);
      }
      o[tt] = (od[0] + od[1]) + (od[2] + od[3]);
    };
#pragma unroll
    for (int tt = 0; tt < DR_TOK; ++tt) o[tt] = 0.f;
    if (nt == DR_TOK) {
#pragma unroll
      for (int tt = 0; tt < DR_TOK; ++tt) token(tt);
    } else {
#pragma unroll
      for (int tt = 0; tt < DR_TOK; ++tt)
        if (tt < nt) token(tt);
    }
    // the eight lanes' partial sums of the column's 16 outputs: in every round a lane hands half of its
    // values to its partner and adds the partner's other half to its own; two whole sums are left per lane
    static_assert(DR_TOK == 16, "two outputs per lane");
#pragma unroll
    for (int half = 4, n = 8; half >= 1; half >>= 1, n >>= 1) {
      const bool upper = (sub & half) != 0;
#pragma unroll
      for (int i = 0; i < n; ++i) {
        const float send = upper ? o[i] : o[i + n];
        const float keep = upper ? o[i + n] : o[i];
        o[i] = keep + __shfl_xor_sync(0xffffffffu, send, half);
      }
    }
    if (col < dv) {
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int tt = 2 * sub + i;
        if (tt < nt) out[((size_t)(base + tt) * H + h) * dv + col] = o[i];
      }
    }
  }
  dr_cp_wait<0>();
#pragma unroll
  for (int r = 0; r < RPL; ++r) {
    const int i = 4 * (sub + 8 * (r >> 2)) + (r & 3);
    if (col < dv && i < dk) st[(size_t)i * dv] = S[r];
  }
}

}  // namespace yalm

using namespace yalm;

// The length of a token's activated row (see the head of this file)
extern "C" int yalm_delta_row(int H, int G, int dk, int dv) {
  return 2 * G * dk + H * dv + ((H + 3) & ~3) + H * dk;
}

// act: float32 [tokens][yalm_delta_row], whose first 2 G dk + H dv columns hold q | k | v after their
// convolution and activation.  proj: slices [.][tokens][proj_row] of the mixer's first product, with
// the beta logits at column col_b and the n_low low-rank values at col_low; low [tokens][n_low] in
// low_dtype receives those.
extern "C" int yalm_delta_prep(float* act, const float* proj, int n_partials, long long partial_stride,
                               int proj_row, int col_b, int col_low, int n_low, void* low, int low_dtype,
                               int n_tokens, int H, int G, int dk, int dv, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (H <= 0 || G <= 0 || H % G || dk <= 0 || dv <= 0 || n_low < 0) return -2;
  const int row = yalm_delta_row(H, G, dk, dv);
  const dim3 grid(n_tokens), block(256);
#define YALM_DP(T)                                                                                     \
  launch_pdl(delta_prep_kernel<T>, grid, block, 0, stream, act, row, proj, n_partials, partial_stride, \
             proj_row, col_b, col_low, n_low, (T*)low, H, G, dk, dv)
  if (low_dtype == DT_F32) YALM_DP(float);
  else if (low_dtype == DT_BF16) YALM_DP(__nv_bfloat16);
  else if (low_dtype == DT_F16) YALM_DP(__half);
  else return -3;
#undef YALM_DP
  YALM_LAUNCH_CHECK();
  return 0;
}

// z: slices [.][tokens][H dk + H dv] (decay logits | gate logits); dt_bias [H dk]; a_log [H];
// gate float32 [tokens][H dv] receives sigmoid(gate logits); then the scan: state float32
// [slots][H][dk][dv], out float32 [tokens][H dv].  dk up to 256.
extern "C" int yalm_delta_scan(float* act, const float* z, int n_partials, long long partial_stride,
                               const float* dt_bias, const float* a_log, float* gate, const int* q_start,
                               const int* seq_slot, float* state, float* out, int n_tokens, int n_seqs,
                               int H, int G, int dk, int dv, cudaStream_t stream) {
  if (n_tokens <= 0 || n_seqs <= 0) return 0;
  if (H <= 0 || G <= 0 || H % G || dk <= 0 || dv <= 0 || dk > 256 || n_seqs > 65535 || H > 65535) return -2;
  const int row = yalm_delta_row(H, G, dk, dv);
  const int decay0 = row - H * dk;
  const int parts = (H * dk + H * dv + 1023) / 1024;
  if (parts > 65535) return -4;
  launch_pdl(delta_decay_kernel, dim3(n_tokens, parts), dim3(256), 0, stream, act, row, decay0, z, n_partials,
             partial_stride, dt_bias, a_log, gate, H, dk, dv);
  YALM_LAUNCH_CHECK();
  const bool vec = dk % 4 == 0 && dv % 4 == 0 && (((uintptr_t)act) & 15) == 0;
  if (dk <= 128) {
    // eight lanes per column
    const dim3 grid8((dv + D8_COLS - 1) / D8_COLS, H, n_seqs), block8(32 * D8_WARPS);
    if ((3 * dk + D8_COLS + (vec ? 3 : 0)) / (vec ? 4 : 1) > 4 * 32 * D8_WARPS) return -2;
#define YALM_D8(R)                                                                                   \
  do {                                                                                               \
    const size_t smem = (size_t)DR_STAGES * DR_TOK * (3 * 8 * R + D8_COLS + 4) * sizeof(float);      \
    static bool set = false;                                                                         \
    if (!set && smem > 48 * 1024) {                                                                  \
      cudaError_t e = cudaFuncSetAttribute(delta_scan8_kernel<R, 4>,                                 \
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);  \
      if (e == cudaSuccess)                                                                          \
        e = cudaFuncSetAttribute(delta_scan8_kernel<R, 1>,                                           \
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);            \
      if (e != cudaSuccess) return (int)e;                                                           \
      set = true;                                                                                    \
    }                                                                                                \
    if (vec)                                                                                         \
      launch_pdl(delta_scan8_kernel<R, 4>, grid8, block8, smem, stream, (const float*)act, row,      \
                 q_start, seq_slot, state, out, H, G, dk, dv);                                       \
    else                                                                                             \
      launch_pdl(delta_scan8_kernel<R, 1>, grid8, block8, smem, stream, (const float*)act, row,      \
                 q_start, seq_slot, state, out, H, G, dk, dv);                                       \
  } while (0)
    if (dk <= 32) YALM_D8(4);
    else if (dk <= 64) YALM_D8(8);
    else YALM_D8(16);
#undef YALM_D8
    YALM_LAUNCH_CHECK();
    return 0;
  }
  const dim3 grid((dv + DR_COLS - 1) / DR_COLS, H, n_seqs), block(256);
  const int rpt = (dk + 31) / 32;
#define YALM_DS(R)                                                                                  \
  do {                                                                                              \
    const size_t smem = (size_t)DR_STAGES * DR_TOK * (3 * 32 * R + DR_COLS + 4) * sizeof(float);    \
    static bool set = false;                                                                        \
    if (!set && smem > 48 * 1024) {                                                                 \
      cudaError_t e = cudaFuncSetAttribute(delta_scan_kernel<R, 4>,                                 \
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
      if (e == cudaSuccess)                                                                         \
        e = cudaFuncSetAttribute(delta_scan_kernel<R, 1>,                                           \
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);           \
      if (e != cudaSuccess) return (int)e;                                                          \
      set = true;                                                                                   \
    }                                                                                               \
    if (vec)                                                                                        \
      launch_pdl(delta_scan_kernel<R, 4>, grid, block, smem, stream, (const float*)act, row, q_start, \
                 seq_slot, state, out, H, G, dk, dv);                                               \
    else                                                                                            \
      launch_pdl(delta_scan_kernel<R, 1>, grid, block, smem, stream, (const float*)act, row, q_start, \
                 seq_slot, state, out, H, G, dk, dv);                                               \
  } while (0)
  if (rpt <= 1) YALM_DS(1);
  else if (rpt <= 2) YALM_DS(2);
  else if (rpt <= 4) YALM_DS(4);
  else YALM_DS(8);
#undef YALM_DS
  YALM_LAUNCH_CHECK();
  return 0;
}
