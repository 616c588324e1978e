// Row kernels of layers that norm a sublayer's OUTPUT before it joins the residual stream
// (x <- x + post(y)) and norm the stream again for the next sublayer (h = pre(x)):
//
//  * norm_step: one pass over a row does the write that is due and the read that follows,
//        y = f_A sum(slices A) + f_B sum(slices B)          (a mixer of two branches hands two sets)
//        x <- x + post(y),   h = pre(x)
//    where post and pre are each one of
//        tanh form ("dynamic tanh"):  n(v) = tanh(alpha v) w + b       no mean, no variance
//        rms form:                    n(v) = v / sqrt(mean(v^2) + eps) w
//        none:                        post: x <- x + y;  pre: h = x in the storage type
//    or absent.  With a row list the kernel only reads: h[r] = pre(x[rows[r]]).
//  * short_conv: a causal convolution over time on every channel of a product's output,
//        y_t = sum_j w[c, j] u_(t - taps + 1 + j)   (+ bias, then SiLU where asked)
//    over the step's tokens of each sequence; the taps - 1 inputs before a step's first token come
//    from the sequence's state (zeros for a new sequence), and short_conv_state leaves the step's
//    last taps - 1 inputs there.
//  * gated_rows: g = gelu(sum(slices)) * E[token, first .. first + dim) for a token-indexed table.
// All arithmetic is 32-bit.
#include "api.h"
#include "common.cuh"

namespace yalm {

struct NormForm {
  int kind;              // 0 absent, 1 tanh form, 2 rms form, 3 none (plain add / plain cast)
  const float* w;
  const float* b;        // tanh form only
  float alpha, eps;
};

struct SliceSet {
  const float* p;
  int n;
  long long stride;
  float factor;
};

__device__ __forceinline__ float apply_tanh_form(const NormForm& f, float v, int i) {
  return fmaf(tanhf(f.alpha * v), f.w[i], f.b[i]);
}

// four neighbouring elements of a row
__device__ __forceinline__ float4 slices4(const float* __restrict__ p, int n, long long stride) {
  float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int s0 = 0; s0 < n; s0 += 4) {
    float4 t[4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
      t[j] = s0 + j < n ? *reinterpret_cast<const float4*>(p + (size_t)(s0 + j) * stride) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int j = 0; j < 4; ++j) { v.x += t[j].x; v.y += t[j].y; v.z += t[j].z; v.w += t[j].w; }
  }
  return v;
}
template <typename T>
__device__ __forceinline__ void store4(T* __restrict__ p, float a, float b, float c, float d) {
  if constexpr (sizeof(T) == 4) {
    *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
  } else {
    uint2 u;
    T* e = reinterpret_cast<T*>(&u);
    e[0] = from_float<T>(a); e[1] = from_float<T>(b); e[2] = from_float<T>(c); e[3] = from_float<T>(d);
    *reinterpret_cast<uint2*>(p) = u;
  }
}

// VEC: dim is a multiple of four and every pointer 16-byte aligned: a thread takes four neighbouring features
template <typename T, bool VEC>
__global__ void norm_step_kernel(float* __restrict__ x, SliceSet A, SliceSet B, NormForm post, NormForm pre,
                                 T* __restrict__ h, const int* __restrict__ rows, int dim) {
  pdl_launch_dependents();
  extern __shared__ __align__(16) float row_s[];           // the row: y, then the new x
  __shared__ float scratch[33];
  pdl_wait();
  const size_t t = rows != nullptr ? (size_t)rows[blockIdx.x] : (size_t)blockIdx.x;
  float* xr = x + t * dim;
  constexpr int W = VEC ? 4 : 1;
  const int i0 = threadIdx.x * W, step = blockDim.x * W;
  if (post.kind) {
    float ss = 0.f;
    for (int i = i0; i < dim; i += step) {
      float y[W];
      if constexpr (VEC) {
        float4 ya = make_float4(0.f, 0.f, 0.f, 0.f), yb = ya;
        if (A.p != nullptr) ya = slices4(A.p + t * dim + i, A.n, A.stride);
        if (B.p != nullptr) yb = slices4(B.p + t * dim + i, B.n, B.stride);
        y[0] = fmaf(B.factor, yb.x, A.factor * ya.x); y[1] = fmaf(B.factor, yb.y, A.factor * ya.y);
        y[2] = fmaf(B.factor, yb.z, A.factor * ya.z); y[3] = fmaf(B.factor, yb.w, A.factor * ya.w);
      } else {
        y[0] = 0.f;
        if (A.p != nullptr) y[0] = A.factor * sum_slices(A.p + t * dim + i, A.n, A.stride);
        if (B.p != nullptr) y[0] = fmaf(B.factor, sum_slices(B.p + t * dim + i, B.n, B.stride), y[0]);
      }
#pragma unroll
      for (int j = 0; j < W; ++j) { row_s[i + j] = y[j]; ss += y[j] * y[j]; }
    }
    float r = 1.f;
    if (post.kind == 2) r = 1.0f / sqrtf(block_sum(ss, scratch) / (float)dim + post.eps);
    for (int i = i0; i < dim; i += step) {
      float v[W];
      if constexpr (VEC) {
        const float4 xv = *reinterpret_cast<const float4*>(xr + i);
        v[0] = xv.x; v[1] = xv.y; v[2] = xv.z; v[3] = xv.w;
      } else {
        v[0] = xr[i];
      }
#pragma unroll
      for (int j = 0; j < W; ++j) {
        const float y = row_s[i + j];
        if (post.kind == 1) v[j] += apply_tanh_form(post, y, i + j);
        else if (post.kind == 2) v[j] += y * r * post.w[i + j];
        else v[j] += y;
        row_s[i + j] = v[j];
      }
      if constexpr (VEC) *reinterpret_cast<float4*>(xr + i) = make_float4(v[0], v[1], v[2], v[3]);
      else xr[i] = v[0];
    }
  } else if (pre.kind) {
    for (int i = i0; i < dim; i += step) {
      if constexpr (VEC) *reinterpret_cast<float4*>(row_s + i) = *reinterpret_cast<const float4*>(xr + i);
      else row_s[i] = xr[i];
    }
  }
  if (!pre.kind) return;
  T* out = h + (size_t)blockIdx.x * dim;
  float r = 1.f;
  if (pre.kind == 2) {
    float ss = 0.f;
    for (int i = i0; i < dim; i += step)
#pragma unroll
      for (int j = 0; j < W; ++j) ss += row_s[i + j] * row_s[i + j];
    r = 1.0f / sqrtf(block_sum(ss, scratch) / (float)dim + pre.eps);
  }
  for (int i = i0; i < dim; i += step) {
    float o[W];
#pragma unroll
    for (int j = 0; j < W; ++j) {
      const float v = row_s[i + j];
      o[j] = pre.kind == 2 ? v * r * pre.w[i + j] : (pre.kind == 1 ? apply_tanh_form(pre, v, i + j) : v);
    }
    if constexpr (VEC) store4<T>(out + i, o[0], o[1], o[2], o[3]);
    else out[i] = from_float<T>(o[0]);
  }
}

constexpr int CONV_MAX_TAPS = 8;

struct ConvArgs {
  const float* src;          // slices [n][tokens][src_row], the channels at src_col0 ..
  int n_partials;
  long long partial_stride;
  int src_row, src_col0;
  const float* in_bias;      // added to the input (the projection's bias), or null
  const float* w;            // [channels][taps]
  const float* out_bias;     // added to the output, or null
  int taps, channels, silu;
  float* state;              // [slots][taps - 1][channels]
};

// ONE: the product came in one slice, so an input is one load (a run's loads then all go out together;
// the loop over slices would make each wait for the one before)
template <bool ONE = false>
__device__ __forceinline__ float conv_input(const ConvArgs& a, int token, int c) {
  const float* p = a.src + (size_t)token * a.src_row + a.src_col0 + c;
  const float v = ONE ? p[0] : sum_slices(p, a.n_partials, a.partial_stride);
  return a.in_bias != nullptr ? v + a.in_bias[c] : v;
}


// grid (runs of RUN tokens, parts of the channels); a block walks through its run of tokens.  out32 [tokens][out_row] at column out_col0;
// out16 (optional) in the storage type, [channels / block16][tokens][block16] (block16 = channels: one
// plain row per token).  A thread owns one channel and loads every input once: the window of the
// last TAPS - 1 inputs moves on in registers and is loaded anew only where a sequence starts.
template <typename T, int TAPS, int RUN, bool ONE>
__global__ void short_conv_kernel(ConvArgs a, const int* __restrict__ token_seq, const int* __restrict__ q_start,
                                  const int* __restrict__ seq_slot, float* __restrict__ out32, int out_row,
                                  int out_col0, T* __restrict__ out16, int block16, int n_tokens) {
  pdl_launch_dependents();
  const int t_first = blockIdx.x * RUN;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= a.channels) return;
  float w[TAPS];
#pragma unroll
  for (int k = 0; k < TAPS; ++k) w[k] = a.w[(size_t)c * TAPS + k];
  const float bias = a.out_bias != nullptr ? a.out_bias[c] : 0.f;
  // the run's index data and inputs first, all loads in flight at once; then the arithmetic in order
  int qs[RUN], ql[RUN], slot[RUN];
#pragma unroll
  for (int j = 0; j < RUN; ++j) {
    const int t = min(t_first + j, n_tokens - 1);
    const int b = token_seq[t];
    qs[j] = q_start[b];
    ql[j] = q_start[b + 1] - qs[j];
    slot[j] = seq_slot[b];
  }
  pdl_wait();
  float cur[RUN];
#pragma unroll
  for (int j = 0; j < RUN; ++j) cur[j] = conv_input<ONE>(a, min(t_first + j, n_tokens - 1), c);
  constexpr int before = TAPS - 1;
  float win[before];
#pragma unroll
  for (int j = 0; j < RUN; ++j) {
    const int t = t_first + j;
    if (t < n_tokens) {
      const int local = t - qs[j];
      float* st = a.state + (size_t)slot[j] * before * a.channels + c;
      if (j == 0 || local == 0) {
#pragma unroll
        for (int k = 0; k < before; ++k) {
          const int idx = local - before + k;
          win[k] = idx >= 0 ? conv_input<ONE>(a, qs[j] + idx, c) : st[(size_t)(before + idx) * a.channels];
        }
      }
      float y = 0.f;
#pragma unroll
      for (int k = 0; k < before; ++k) y = fmaf(w[k], win[k], y);
      y = fmaf(w[before], cur[j], y) + bias;
      if (a.silu) y = y / (1.0f + expf(-y));
      if (out32 != nullptr) out32[(size_t)t * out_row + out_col0 + c] = y;
      if (out16 != nullptr)
        out16[((size_t)(c / block16) * n_tokens + t) * block16 + c % block16] = from_float<T>(y);
#pragma unroll
      for (int k = 0; k + 1 < before; ++k) win[k] = win[k + 1];
      win[before - 1] = cur[j];
      // a sequence that brings one token: this thread has read all it needs of the state and moves it on
      if (ql[j] == 1) {
#pragma unroll
        for (int k = 0; k < before; ++k) st[(size_t)k * a.channels] = win[k];
      }
    }
  }
}

// grid (sequences, parts of the channels): the step's last taps - 1 inputs of every sequence that
// brought more than one token (some of them the state's own, when it brought fewer than taps - 1)
__global__ void short_conv_state_kernel(ConvArgs a, const int* __restrict__ q_start,
                                        const int* __restrict__ seq_slot) {
  pdl_launch_dependents();
  const int b = blockIdx.x;
  const int qs = q_start[b], ql = q_start[b + 1] - qs;
  const int slot = seq_slot[b];
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  pdl_wait();
  if (c >= a.channels || ql <= 1) return;
  const int before = a.taps - 1;
  float* st = a.state + (size_t)slot * before * a.channels + c;
  float u[CONV_MAX_TAPS];
  for (int k = 0; k < before; ++k) {
    const int idx = ql - before + k;
    u[k] = idx >= 0 ? conv_input(a, qs + idx, c) : st[(size_t)(before + idx) * a.channels];
  }
  for (int k = 0; k < before; ++k) st[(size_t)k * a.channels] = u[k];
}

// grid (tokens): out [tokens][dim] = gelu(sum of slices z [tokens][dim]) * table[token][first + i]
template <typename TT, typename T>
__global__ void gated_rows_kernel(const float* __restrict__ z, int n_partials, long long partial_stride,
                                  const int* __restrict__ tokens, const TT* __restrict__ table, int table_row,
                                  int first, T* __restrict__ out, int dim) {
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const int tok = tokens[t];
  pdl_wait();
  for (int i = threadIdx.x; i < dim; i += blockDim.x) {
    const float v = sum_slices(z + (size_t)t * dim + i, n_partials, partial_stride);
    const float g = 0.5f * v * (1.0f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)));
    out[(size_t)t * dim + i] = from_float<T>(g * to_float(table[(size_t)tok * table_row + first + i]));
  }
}

}  // namespace yalm

using namespace yalm;

// x float32 [.., dim] (changed in place when post_kind != 0).  y = fa * sum(slices a) + fb * sum(slices b)
// (either may be null).  post / pre: kind 0 absent, 1 tanh form (w, b, alpha), 2 rms form (w, eps),
// 3 none.  h [n_rows][dim] in h_dtype receives pre(x).  rows (optional, only without a post step): the
// rows of x that are read.
extern "C" int yalm_norm_step(float* x, const float* a, int na, long long sa, float fa, const float* b,
                              int nb, long long sb, float fb, int post_kind, const float* post_w,
                              const float* post_b, float post_alpha, float post_eps, int pre_kind,
                              const float* pre_w, const float* pre_b, float pre_alpha, float pre_eps,
                              void* h, int h_dtype, const int* rows, int n_rows, int dim,
                              cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (dim <= 0 || dim > 12288 || (rows != nullptr && post_kind) || (!post_kind && !pre_kind)) return -2;
  if ((post_kind && a == nullptr && b == nullptr) || (pre_kind && h == nullptr)) return -2;
  const SliceSet A = {a, na, sa, fa}, B = {b, nb, sb, fb};
  const NormForm post = {post_kind, post_w, post_b, post_alpha, post_eps};
  const NormForm pre = {pre_kind, pre_w, pre_b, pre_alpha, pre_eps};
  const bool vec = dim % 4 == 0 && (sa & 3) == 0 && (sb & 3) == 0 &&
                   ((((uintptr_t)x) | ((uintptr_t)a) | ((uintptr_t)b) | ((uintptr_t)h)) & 15) == 0;
  int threads = ((vec ? dim / 4 : dim) + 31) / 32 * 32;
  if (threads > 512) threads = 512;
  if (n_rows <= 64 && dim >= 8192 && !vec) threads = 1024;
  const dim3 grid(n_rows), block(threads);
  const size_t smem = (size_t)dim * sizeof(float);
#define YALM_NS1(T, V)                                                                                 \
  do {                                                                                                \
    static size_t attr = 48 * 1024;                                                                   \
    if (smem > attr) {                                                                                \
      cudaError_t e = cudaFuncSetAttribute(norm_step_kernel<T, V>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                           (int)smem);                                                \
      if (e != cudaSuccess) return (int)e;                                                            \
      attr = smem;                                                                                    \
    }                                                                                                 \
    launch_pdl(norm_step_kernel<T, V>, grid, block, smem, stream, x, A, B, post, pre, (T*)h, rows, dim); \
  } while (0)
#define YALM_NS(T)                \
  do {                            \
    if (vec) YALM_NS1(T, true);   \
    else YALM_NS1(T, false);      \
  } while (0)
  if (h_dtype == DT_F32) YALM_NS(float);
  else if (h_dtype == DT_BF16) YALM_NS(__nv_bfloat16);
  else if (h_dtype == DT_F16) YALM_NS(__half);
  else return -3;
#undef YALM_NS
#undef YALM_NS1
  YALM_LAUNCH_CHECK();
  return 0;
}

// src: float32 slices [n_partials][tokens][src_row], channels at columns src_col0 .. + channels;
// w [channels][taps] (the last column is the current token's); state float32 [slots][taps - 1][channels];
// out32 (optional) float32 [tokens][out_row] at out_col0; out16 (optional) [channels / block16][tokens][block16]
// in out16_dtype.  update_state: also run the kernel that leaves the step's last inputs in the state
// (needed unless every sequence brings one token).
extern "C" int yalm_short_conv(const float* src, int n_partials, long long partial_stride, int src_row,
                               int src_col0, const float* in_bias, const float* w, const float* out_bias,
                               int taps, int channels, int silu, float* state, const int* token_seq,
                               const int* q_start, const int* seq_slot, float* out32, int out_row,
                               int out_col0, void* out16, int out16_dtype, int block16, int n_tokens,
                               int n_seqs, int update_state, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (taps < 2 || taps > CONV_MAX_TAPS || channels <= 0 || (out16 != nullptr && (block16 <= 0 || channels % block16)))
    return -2;
  const ConvArgs a = {src, n_partials, partial_stride, src_row, src_col0, in_bias, w, out_bias, taps, channels,
                      silu, state};
  const int threads = channels >= 256 ? 256 : (channels + 31) / 32 * 32;
  const int parts = (channels + threads - 1) / threads;
  if (parts > 65535 || n_seqs > 0x7fffffff) return -4;
  // many tokens: a thread keeps its channel's last inputs in registers over a run of eight; few: a block per token
  const int run = n_tokens >= 1024 ? 8 : 1;
  const dim3 grid((n_tokens + run - 1) / run, parts), block(threads);
  const int b16 = out16 != nullptr ? block16 : channels;
#define YALM_CONV(T, TAPS)                                                                                \
  do {                                                                                                    \
    if (run == 8 && n_partials == 1)                                                                      \
      launch_pdl(short_conv_kernel<T, TAPS, 8, true>, grid, block, 0, stream, a, token_seq, q_start,      \
                 seq_slot, out32, out_row, out_col0, (T*)out16, b16, n_tokens);                           \
    else if (run == 8)                                                                                    \
      launch_pdl(short_conv_kernel<T, TAPS, 8, false>, grid, block, 0, stream, a, token_seq, q_start,     \
                 seq_slot, out32, out_row, out_col0, (T*)out16, b16, n_tokens);                           \
    else                                                                                                  \
      launch_pdl(short_conv_kernel<T, TAPS, 1, false>, grid, block, 0, stream, a, token_seq, q_start,     \
                 seq_slot, out32, out_row, out_col0, (T*)out16, b16, n_tokens);                           \
  } while (0)
#define YALM_CONV_T(T)                                                                                  \
  do {                                                                                                  \
    switch (taps) {                                                                                     \
      case 2: YALM_CONV(T, 2); break;                                                                   \
      case 3: YALM_CONV(T, 3); break;                                                                   \
      case 4: YALM_CONV(T, 4); break;                                                                   \
      case 5: YALM_CONV(T, 5); break;                                                                   \
      case 6: YALM_CONV(T, 6); break;                                                                   \
      case 7: YALM_CONV(T, 7); break;                                                                   \
      default: YALM_CONV(T, 8); break;                                                                  \
    }                                                                                                   \
  } while (0)
  if (out16 == nullptr || out16_dtype == DT_F32) YALM_CONV_T(float);
  else if (out16_dtype == DT_BF16) YALM_CONV_T(__nv_bfloat16);
  else if (out16_dtype == DT_F16) YALM_CONV_T(__half);
  else return -3;
#undef YALM_CONV_T
#undef YALM_CONV
  YALM_LAUNCH_CHECK();
  if (update_state) {
    launch_pdl(short_conv_state_kernel, dim3(n_seqs, parts), block, 0, stream, a, q_start, seq_slot);
    YALM_LAUNCH_CHECK();
  }
  return 0;
}

// out [tokens][dim] (out_dtype) = gelu(sum of n_partials slices of z [tokens][dim]) * table[token][first + i];
// table [vocab][table_row] in table_dtype
extern "C" int yalm_gated_rows(const float* z, int n_partials, long long partial_stride, const int* tokens,
                               const void* table, int table_dtype, int table_row, int first, void* out,
                               int out_dtype, int n_tokens, int dim, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (dim <= 0 || first < 0 || first + dim > table_row) return -2;
  const dim3 grid(n_tokens), block(dim >= 256 ? 256 : (dim + 31) / 32 * 32);
#define YALM_GR(TT, T)                                                                                 \
  launch_pdl(gated_rows_kernel<TT, T>, grid, block, 0, stream, z, n_partials, partial_stride, tokens,  \
             (const TT*)table, table_row, first, (T*)out, dim)
  if (table_dtype == DT_F32 && out_dtype == DT_F32) YALM_GR(float, float);
  else if (table_dtype == DT_BF16 && out_dtype == DT_BF16) YALM_GR(__nv_bfloat16, __nv_bfloat16);
  else if (table_dtype == DT_F16 && out_dtype == DT_F16) YALM_GR(__half, __half);
  else if (table_dtype == DT_F32 && out_dtype == DT_BF16) YALM_GR(float, __nv_bfloat16);
  else if (table_dtype == DT_F32 && out_dtype == DT_F16) YALM_GR(float, __half);
  else return -3;
#undef YALM_GR
  YALM_LAUNCH_CHECK();
  return 0;
}
