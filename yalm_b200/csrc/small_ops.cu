// Small row-wise kernels that some architectures add around the common ones:
//  * an embedding with a second, hashed table: x = E[token] + P[row], where row is a hash of
//    the previous and the current token (the previous token of a sequence's first token in a
//    step comes from a per-sequence state that the kernel also updates);
//  * a per-head output gate: o[t, h, :] *= sigmoid(g[t, h]);
//  * a soft cap on logits: v <- cap * tanh(v / cap);
//  * x += y on the residual stream, folding pending split-K partial sums in.
// All arithmetic is 32-bit.
#include "api.h"
#include "common.cuh"

namespace yalm {

template <typename T>
__global__ void embed_pair_kernel(const int* __restrict__ tokens, const int* __restrict__ token_seq,
                                  const int* __restrict__ q_start, const int* __restrict__ seq_slot,
                                  const int* __restrict__ slot_pos, const T* __restrict__ table,
                                  const T* __restrict__ pair_table, int* __restrict__ prev_token,
                                  float* __restrict__ x, float* __restrict__ x_copy, int dim, int vocab,
                                  int buckets, long long mul_prev, long long mul_cur,
                                  int* __restrict__ status) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  int tok = tokens[t];
  if (tok < 0 || tok >= vocab) {
    if (threadIdx.x == 0) atomicOr(status, ERR_TOKEN_RANGE);
    tok = tok < 0 ? 0 : vocab - 1;
  }
  const int b = token_seq[t];
  const int slot = seq_slot[b];
  const int qs = q_start[b];
  const int pos = slot_pos[slot] + (t - qs);
  // the token before this one: the step's own, or what the sequence's last step left
  int prev = t > qs ? tokens[t - 1] : prev_token[slot];
  prev = prev < 0 ? 0 : (prev >= vocab ? vocab - 1 : prev);
  long long row = buckets;                                   // a sequence's first token: the last row
  if (pos > 0) {
    row = ((long long)prev * mul_prev + (long long)tok * mul_cur) % buckets;
    if (row < 0) row += buckets;
  }
  const T* e = table + (size_t)tok * dim;
  const T* p = pair_table + (size_t)row * dim;
  float* out = x + (size_t)t * dim;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) {
    const float v = to_float(e[i]) + to_float(p[i]);
    out[i] = v;
    if (x_copy != nullptr) x_copy[(size_t)t * dim + i] = v;
  }
  // Only the block of a sequence's first token in this step reads the state, and it alone
  // writes it, after every one of its threads has read: the step's last token.
  if (t == qs) {
    __syncthreads();
    if (threadIdx.x == 0) prev_token[slot] = tokens[q_start[b + 1] - 1];
  }
}

// o [n, H, hd] *= sigmoid(sum over slices of g [S, n, H]); one block per token
template <typename T>
__global__ void head_gate_kernel(T* __restrict__ o, const float* __restrict__ g, int n_partials,
                                 long long partial_stride, int H, int hd) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float gate_s[];
  const int t = blockIdx.x;
  for (int h = threadIdx.x; h < H; h += blockDim.x) {
    const float z = sum_slices(g + (size_t)t * H + h, n_partials, partial_stride);
    gate_s[h] = 1.0f / (1.0f + expf(-z));
  }
  __syncthreads();
  T* row = o + (size_t)t * H * hd;
  // a thread takes whole runs of 8 elements of one head where the head size allows it
  if (hd % 8 == 0 && sizeof(T) == 2) {
    for (int i = threadIdx.x * 8; i < H * hd; i += blockDim.x * 8) {
      const float gt = gate_s[i / hd];
      uint4 raw = *reinterpret_cast<const uint4*>(row + i);
      T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
      for (int j = 0; j < 8; ++j) e[j] = from_float<T>(to_float(e[j]) * gt);
      *reinterpret_cast<uint4*>(row + i) = raw;
    }
    return;
  }
  for (int i = threadIdx.x; i < H * hd; i += blockDim.x)
    row[i] = from_float<T>(to_float(row[i]) * gate_s[i / hd]);
}

// o [n] *= sigmoid(sum over slices of g [S][n]), feature by feature; four features per thread
template <typename T>
__global__ void element_gate_kernel(T* __restrict__ o, const float* __restrict__ g, int n_partials,
                                    long long partial_stride, long long n4) {
  pdl_launch_dependents();
  pdl_wait();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4;
       i += (long long)gridDim.x * blockDim.x) {
    float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s = 0; s < n_partials; ++s) {
      const float4 p = *reinterpret_cast<const float4*>(g + (size_t)s * partial_stride + 4 * i);
      z.x += p.x; z.y += p.y; z.z += p.z; z.w += p.w;
    }
    T* e = o + 4 * i;
    e[0] = from_float<T>(to_float(e[0]) / (1.0f + expf(-z.x)));
    e[1] = from_float<T>(to_float(e[1]) / (1.0f + expf(-z.y)));
    e[2] = from_float<T>(to_float(e[2]) / (1.0f + expf(-z.z)));
    e[3] = from_float<T>(to_float(e[3]) / (1.0f + expf(-z.w)));
  }
}

__global__ void softcap_kernel(float* __restrict__ v, long long n, float cap) {
  pdl_launch_dependents();
  pdl_wait();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) v[i] = cap * tanhf(v[i] / cap);
}

__global__ void residual_add_kernel(float* __restrict__ x, const float* __restrict__ y,
                                    const float* __restrict__ partials, int n_partials,
                                    long long partial_stride, long long n) {
  pdl_launch_dependents();
  pdl_wait();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float v = x[i] + (n_partials ? sum_slices(partials + i, n_partials, partial_stride) : 0.f);
  x[i] = v + y[i];
}

// out [n] = act(sum over slices of z [S][n]) in the storage type: 1 = gelu in its tanh form,
// 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))), 2 = tanh
template <typename T>
__global__ void activation_rows_kernel(const float* __restrict__ z, int n_partials, long long partial_stride,
                                       T* __restrict__ out, long long n, int act) {
  pdl_launch_dependents();
  pdl_wait();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const float v = sum_slices(z + i, n_partials, partial_stride);
    float r;
    if (act == 1) r = 0.5f * v * (1.0f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)));
    else r = tanhf(v);
    out[i] = from_float<T>(r);
  }
}

}  // namespace yalm

using namespace yalm;

// x[t] = E[token t] + P[row t] (and the same into x_copy when it is given).  row = buckets
// for position 0 of a sequence, else (previous token * mul_prev + token * mul_cur) mod
// buckets; pair_table has buckets + 1 rows.  prev_token [slots]: the last token each sequence
// has been given so far (read for a step's first token, then set to the step's last).
extern "C" int yalm_embed_pair(const int* tokens, const int* token_seq, const int* q_start,
                               const int* seq_slot, const int* slot_pos, const void* table,
                               const void* pair_table, int table_dtype, int* prev_token, float* x,
                               float* x_copy, int n_tokens, int dim, int vocab, int buckets,
                               long long mul_prev, long long mul_cur, int* status,
                               cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (buckets <= 0 || dim <= 0) return -2;
  const dim3 grid(n_tokens), block(dim >= 1024 ? 256 : 128);
#define YALM_EP(T)                                                                                  \
  launch_pdl(embed_pair_kernel<T>, grid, block, 0, stream, tokens, token_seq, q_start, seq_slot,   \
             slot_pos, (const T*)table, (const T*)pair_table, prev_token, x, x_copy, dim, vocab,    \
             buckets, mul_prev, mul_cur, status)
  if (table_dtype == DT_F32) YALM_EP(float);
  else if (table_dtype == DT_BF16) YALM_EP(__nv_bfloat16);
  else if (table_dtype == DT_F16) YALM_EP(__half);
  else return -3;
#undef YALM_EP
  YALM_LAUNCH_CHECK();
  return 0;
}

extern "C" int yalm_head_gate(void* o, int dtype, const float* g, int n_partials,
                              long long partial_stride, int n_tokens, int H, int hd,
                              cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (H <= 0 || hd <= 0 || H > 12000) return -2;
  const dim3 grid(n_tokens), block(256);
  const size_t smem = (size_t)H * sizeof(float);
  if (dtype == DT_F32)
    launch_pdl(head_gate_kernel<float>, grid, block, smem, stream, (float*)o, g, n_partials, partial_stride, H, hd);
  else if (dtype == DT_BF16)
    launch_pdl(head_gate_kernel<__nv_bfloat16>, grid, block, smem, stream, (__nv_bfloat16*)o, g, n_partials,
               partial_stride, H, hd);
  else if (dtype == DT_F16)
    launch_pdl(head_gate_kernel<__half>, grid, block, smem, stream, (__half*)o, g, n_partials, partial_stride, H, hd);
  else
    return -3;
  YALM_LAUNCH_CHECK();
  return 0;
}

// o [n] *= sigmoid(sum of the n_partials slices of g [n]); n a multiple of 4, g 16-byte aligned
extern "C" int yalm_element_gate(void* o, int dtype, const float* g, int n_partials,
                                 long long partial_stride, long long n, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (n % 4 != 0 || partial_stride % 4 != 0 || (((uintptr_t)g) & 15)) return -2;
  long long blocks = (n / 4 + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  const dim3 grid((unsigned)blocks), block(256);
  if (dtype == DT_F32) launch_pdl(element_gate_kernel<float>, grid, block, 0, stream, (float*)o, g, n_partials, partial_stride, n / 4);
  else if (dtype == DT_BF16) launch_pdl(element_gate_kernel<__nv_bfloat16>, grid, block, 0, stream, (__nv_bfloat16*)o, g, n_partials, partial_stride, n / 4);
  else if (dtype == DT_F16) launch_pdl(element_gate_kernel<__half>, grid, block, 0, stream, (__half*)o, g, n_partials, partial_stride, n / 4);
  else return -3;
  YALM_LAUNCH_CHECK();
  return 0;
}

extern "C" int yalm_softcap(float* v, long long n, float cap, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (!(cap > 0.f)) return -2;
  const long long blocks = (n + 255) / 256;
  if (blocks > 0x7fffffffLL) return -4;
  launch_pdl(softcap_kernel, dim3((unsigned)blocks), dim3(256), 0, stream, v, n, cap);
  YALM_LAUNCH_CHECK();
  return 0;
}

// x += y (+ the sum of n_partials slices [n_partials][n]); all float32 of n elements
extern "C" int yalm_residual_add(float* x, const float* y, const float* partials, int n_partials,
                                 long long partial_stride, long long n, cudaStream_t stream) {
  if (n <= 0) return 0;
  const long long blocks = (n + 255) / 256;
  if (blocks > 0x7fffffffLL) return -4;
  launch_pdl(residual_add_kernel, dim3((unsigned)blocks), dim3(256), 0, stream, x, y, partials, n_partials,
             partial_stride, n);
  YALM_LAUNCH_CHECK();
  return 0;
}

extern "C" int yalm_activation_rows(const float* z, int n_partials, long long partial_stride, void* out,
                                    int out_dtype, long long n, int act, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (act != 1 && act != 2) return -3;
  long long blocks = (n + 255) / 256;
  if (blocks > 148 * 32) blocks = 148 * 32;
  const dim3 grid((unsigned)blocks), block(256);
  if (out_dtype == DT_F32) launch_pdl(activation_rows_kernel<float>, grid, block, 0, stream, z, n_partials, partial_stride, (float*)out, n, act);
  else if (out_dtype == DT_BF16) launch_pdl(activation_rows_kernel<__nv_bfloat16>, grid, block, 0, stream, z, n_partials, partial_stride, (__nv_bfloat16*)out, n, act);
  else if (out_dtype == DT_F16) launch_pdl(activation_rows_kernel<__half>, grid, block, 0, stream, z, n_partials, partial_stride, (__half*)out, n, act);
  else return -3;
  YALM_LAUNCH_CHECK();
  return 0;
}
