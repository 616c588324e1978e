// C interface of the sm_100a kernel library.  Every function launches on the
// given stream and returns 0, a cudaError_t of the launch, or a negative code
// for arguments it refuses (a size the kernel does not take).  Pointers are
// device pointers unless said otherwise.  dtype codes: 0 = float32, 1 = bfloat16,
// 2 = float16.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// a kernel whose bounded barrier wait runs out after limit_ns (<= 100 ms) and raises
// ERR_WAIT_TIMEOUT in *status: the status path, for tests
int yalm_wait_probe(unsigned long long limit_ns, int* status, cudaStream_t stream);
int yalm_copy_async(void* dst, const void* src, long long bytes, int to_device, cudaStream_t stream);
int yalm_stream_wait(cudaStream_t stream);
// x[t] = table[token t] * scale
int yalm_embed(const int* tokens, const void* table, int table_dtype, float* x, int n_tokens,
               int dim, int vocab, float scale, int* status, cudaStream_t stream);

int yalm_rmsnorm(float* x, const float* partials, int n_partials, long long partial_stride,
                 const int* rows, const float* weight, void* out, int out_dtype, int n_rows,
                 int dim, float eps, cudaStream_t stream);

int yalm_silu_mul(const float* gu, int n_partials, long long partial_stride, void* out,
                  int out_dtype, int rows, int F, int paired, cudaStream_t stream);

// `window` and `scale`, wherever an attention function takes them: window > 0, a query sees
// the last `window` positions; window < 0, the positions of its own chunk of -window
// positions (chunks counted from position 0 of the sequence); 0, every earlier position.
// scale multiplies q.k; scale <= 0 stands for 1 / sqrt(hd).
//
// The cache of a layer run, wherever it is an argument: contiguous per sequence,
// [slots][G][capacity][hd] (page_table null), or pages of 64 positions,
// [pages][G][64][hd], with page_table [slots][pages_per_slot] naming the page of rows
// 64 p .. 64 p + 63 of each sequence.  A row is a position modulo the capacity.
int yalm_rope_store(const float* qkv, int n_partials, long long partial_stride,
                    const float* inv_freq, const int* token_seq, const int* q_start,
                    const int* seq_slot, const int* slot_pos, void* q_out, void* kv_step,
                    void* k_cache, void* v_cache, int dtype, int n_tokens, int H, int G, int hd,
                    int capacity, int write_cache, const int* page_table, int pages_per_slot, int n_pages,
                    cudaStream_t stream);

// kv_step [N, 2, G, hd] -> the ring rows of the positions the ring keeps (the cache
// write of yalm_rope_store, on its own: for a ring that may only be written after the
// attention has read the rows that are replaced)
int yalm_cache_write(const void* kv_step, const int* token_seq, const int* q_start,
                     const int* seq_slot, const int* slot_pos, void* k_cache, void* v_cache,
                     int dtype, int n_tokens, int G, int hd, int capacity, const int* page_table,
                     int pages_per_slot, int n_pages, cudaStream_t stream);

int yalm_advance(const int* q_start, const int* seq_slot, int* slot_pos, int n_seqs,
                 cudaStream_t stream);

int yalm_attention(const void* q, const void* kv_step, const void* k_cache, const void* v_cache,
                   const int* token_seq, const int* q_start, const int* seq_slot,
                   const int* slot_pos, void* out, float* part_o, float* part_ml, int dtype,
                   int n_tokens, int H, int G, int hd, int capacity, int window, float scale, int nsplit,
                   const int* page_table, int pages_per_slot, int n_pages, cudaStream_t stream);

int yalm_attention_decode(const void* q, const void* k_cache, const void* v_cache,
                          const int* seq_slot, const int* slot_pos, void* out, float* part_o,
                          float* part_ml, int* counters, int* status, int dtype, int n_seqs, int H,
                          int G, int hd, int capacity, int window, float scale, int chunk, int max_context,
                          const int* page_table, int pages_per_slot, int n_pages, cudaStream_t stream);

// 16-bit attention on tensor cores (attention_mma_prefill.cu, attention_mma.cu; dtype 1 or 2): head sizes in steps of
// 16 up to 128
int yalm_attention_prefill_mma(const void* q, const void* kv_step, const void* k_cache,
                               const void* v_cache, const int* q_start, const int* seq_slot,
                               const int* slot_pos, void* out, int dtype, int n_seqs,
                               int max_q_len, int H, int G, int hd, int capacity, int window, float scale,
                               const int* page_table, int pages_per_slot, int n_pages, cudaStream_t stream);
int yalm_attention_decode_mma(const void* q, const void* k_cache, const void* v_cache,
                              const int* seq_slot, const int* slot_pos, void* out, float* part_o,
                              float* part_ml, int* counters, int* status, int dtype, int n_seqs,
                              int H, int G, int hd, int capacity, int window, float scale, int max_context,
                              int chunks_per_block, int warps, const int* page_table, int pages_per_slot,
                              int n_pages, cudaStream_t stream);
// ... compiled with two warps per block (attention_mma_two_warps.cu); yalm_attention_decode_mma
// calls it for warps = 2
int yalm_attention_decode_mma_two_warps(const void* q, const void* k_cache, const void* v_cache,
                                        const int* seq_slot, const int* slot_pos, void* out, float* part_o,
                                        float* part_ml, int* counters, int* status, int dtype, int n_seqs,
                                        int H, int G, int hd, int capacity, int window, float scale, int max_context,
                                        int chunks_per_block, const int* page_table, int pages_per_slot,
                                        int n_pages, cudaStream_t stream);
// ... with the rotary kernel's work inside (attention_mma_fused.cu): takes this step's q/k/v product
// as n_partials 32-bit slices and the step's cosines and sines, writes the new cache rows
int yalm_attention_decode_mma_fused(const float* qkv, int n_partials, long long partial_stride,
                                    const float* cos_sin, void* k_cache, void* v_cache,
                                    const int* seq_slot, const int* slot_pos, void* out, float* part_o,
                                    float* part_ml, int* counters, int* status, int dtype, int n_seqs,
                                    int H, int G, int hd, int capacity, int window, float scale, int max_context,
                                    int chunks_per_block, const int* page_table, int pages_per_slot,
                                    int n_pages, cudaStream_t stream);

// 16-bit prefill attention on tcgen05 (attention_tc.cu; dtype 1 or 2): sequences that start
// at their first token, head size 64 or 128
int yalm_attention_prefill_tc(const void* q, const void* kv_step, const int* q_start, void* out,
                              int dtype, int n_tokens, int n_seqs, int max_q_len, int H, int G,
                              int hd, int window, float scale, int* status, cudaStream_t stream);
// ... for sequences that go on from slot_pos, no one wrapping around its ring in this step:
// every key (this step's too) from the layer's cache, paged or one block per sequence
int yalm_attention_prefill_tc_cache(const void* q, const void* k_cache, const void* v_cache,
                                    const int* q_start, const int* seq_slot, const int* slot_pos,
                                    void* out, int dtype, int n_tokens, int n_seqs, int max_q_len,
                                    int n_slots, int H, int G, int hd, int capacity, int window, float scale,
                                    const int* page_table, int pages_per_slot, int n_pages, int* status,
                                    cudaStream_t stream);

int yalm_gemm_simt(const void* A, int a_dtype, const void* W, int w_dtype, void* out,
                   int out_dtype, int M, int N, int K, int accumulate, cudaStream_t stream);

// params: null, or two 64-bit words on the device that replace `seed` and `temperature`
// (the temperature's float bits in the low half of the second word)
int yalm_sample(const float* logits, int n_rows, int vocab, float temperature,
                unsigned long long seed, const unsigned long long* params, const int* row_key,
                const int* seq_slot, const int* slot_pos, int* out_tokens, cudaStream_t stream);

float yalm_uniform01(unsigned long long seed, unsigned key, unsigned counter);

// tcgen05 / TMA matrix product (operands of ab_dtype 1 or 2, 32-bit accumulation in TMEM;
// out_dtype is 0 or ab_dtype):
//   mode 0: out[M,N]  = A W^T             (out_dtype 0 or 1)
//   mode 1: out[M,N] += A W^T             (out float32: the residual stream)
//   mode 2: out[M,N/2] = silu(A Wg^T) * (A Wu^T), W = [Wg; Wu] with N rows in all
//   mode 3: out[s][M,N] = partial products of `splits` slices of K (float32 scratch)
// status: a device int that receives ERR_WAIT_TIMEOUT if a bounded wait gave up.
int yalm_gemm_tc(const void* A, const void* W, int ab_dtype, void* out, int out_dtype, int M,
                 int N, int K, int mode, int splits, int* status, cudaStream_t stream);
// modes 2 and 4 of yalm_gemm_tc / yalm_gemm_2sm with a gated activation other than SiLU:
// out = g' sigmoid(slope g') (u' + shift), g' = min(g, limit), u' = clamp(u, -limit, limit)
// (no clamps when limit <= 0)
int yalm_gemm_tc_glu(const void* A, const void* W, int ab_dtype, void* out, int out_dtype, int M,
                     int N, int K, int mode, float slope, float limit, float shift, int* status,
                     cudaStream_t stream);
int yalm_gemm_2sm_glu(const void* A, const void* W, int ab_dtype, void* out, int out_dtype, int M,
                      int N, int K, int mode, float slope, float limit, float shift, int* status,
                      cudaStream_t stream);
// yalm_gemm_2sm in mode 0 with out = act(A W^T): act 1 the tanh form of GELU, 2 tanh.
int yalm_gemm_2sm_act(const void* A, const void* W, int ab_dtype, void* out, int out_dtype, int M,
                      int N, int K, int act, int* status, cudaStream_t stream);
// 0 if the driver's tensor-map encoder was found (host-side set-up of yalm_gemm_tc).
int yalm_gemm_tc_available(void);

// cos_sin[t][i] = (cos, sin) of position(t) * inv_freq[i], positions as yalm_rope_store
// derives them: the table that yalm_gemm_2sm_rope reads, made once per step for all layers
int yalm_rope_table(const float* inv_freq, const int* token_seq, const int* q_start,
                    const int* seq_slot, const int* slot_pos, float* cos_sin, int n_tokens, int half,
                    cudaStream_t stream);

// What the rotary epilogue of yalm_gemm_2sm_rope needs: the arguments of yalm_rope_store,
// with the table of yalm_rope_table in place of the frequencies.
typedef struct yalm_rope_args {
  const float* cos_sin;      // [M][hd/2][2]
  const int* token_seq;      // [M]
  const int* q_start;        // [n_seqs + 1]
  const int* seq_slot;       // [n_seqs]
  const int* slot_pos;       // [slots]
  void* q_out;               // [M, H*hd]
  void* kv_step;             // [M, 2, G, hd]
  void* k_cache;
  void* v_cache;
  const int* page_table;     // null: a cache that is one block per sequence
  int pages_per_slot, n_pages;
  int H, G, hd, capacity, write_cache;
} yalm_rope_args;

// Two-SM (cta_group::2) variant for many tokens: mode 0 store, 1 add, 2 silu(gate)*up, 4 the
// same with interleaved rows, 3 `splits` slices of K as 32-bit partial sums [splits, M, N].
int yalm_gemm_2sm(const void* A, const void* W, int ab_dtype, void* out, int out_dtype, int M,
                  int N, int K, int mode, int splits, int* status, cudaStream_t stream);
// the token tile (256 or 240) it takes for these sizes
int yalm_gemm_2sm_token_tile(int M, int N, int splits);

// The q/k/v product of many tokens with rotary encoding and cache write in its epilogue
// (head sizes 16, 32, 64 and 128).
int yalm_gemm_2sm_rope(const void* A, const void* W, int ab_dtype, int M, int N, int K,
                       const yalm_rope_args* rope, int* status, cudaStream_t stream);

// yalm_attention with pooled blocks beside a sliding window (window > 0): pool_k / pool_v hold one
// (mean key, mean value) row per block of `pool` positions, [slots][G][pool_capacity][hd] or pages
// named by pool_table; a query at position p sees block b if b * pool + pool - 1 <= p - window, in
// the same softmax as the window's keys.
int yalm_attention_pooled(const void* q, const void* kv_step, const void* k_cache, const void* v_cache,
                          const int* token_seq, const int* q_start, const int* seq_slot,
                          const int* slot_pos, void* out, float* part_o, float* part_ml, int dtype,
                          int n_tokens, int H, int G, int hd, int capacity, int window, float scale,
                          int nsplit, const int* page_table, int pages_per_slot, int n_pages,
                          const void* pool_k, const void* pool_v, int pool, int pool_capacity,
                          const int* pool_table, int pool_pps, int pool_pages, cudaStream_t stream);
// yalm_attention with a window that keeps the first `keep` positions visible beside the last `window`
int yalm_attention_keep_first(const void* q, const void* kv_step, const void* k_cache, const void* v_cache,
                              const int* token_seq, const int* q_start, const int* seq_slot,
                              const int* slot_pos, void* out, float* part_o, float* part_ml, int dtype,
                              int n_tokens, int H, int G, int hd, int capacity, int window, int keep,
                              float scale, int nsplit, const int* page_table, int pages_per_slot,
                              int n_pages, cudaStream_t stream);

// Prefill attention with 32-bit softmax weights on tensor cores (attention_exact.cu; dtype 1 or 2,
// head size 32, 64, 128 or 256, window >= 0): S = Q K^T by mma.sync, softmax in 32 bits, P split into
// three 16-bit terms for three P V products.  pool > 0: the pooled rows take part.  keep_first > 0
// (with a window, without a pool): the first keep_first positions stay visible beside the window.
int yalm_attention_exact_prefill(const void* q, const void* kv_step, const void* k_cache,
                                 const void* v_cache, const int* q_start, const int* seq_slot,
                                 const int* slot_pos, void* out, int dtype, int n_seqs, int max_q_len,
                                 int H, int G, int hd, int capacity, int window, float scale,
                                 const int* page_table, int pages_per_slot, int n_pages,
                                 const void* pool_k, const void* pool_v, int pool, int pool_capacity,
                                 const int* pool_table, int pool_pps, int pool_pages, int keep_first,
                                 cudaStream_t stream);

// ---- qk_store.cu: after a q/k(/v) product with whole-projection norms and partial rotation ----
// qkv: float32 slices [n_partials][tokens][(H + G (+ G)) hd] = (q | k | v, v only with has_v).
// q_norm [H hd] / k_norm [G hd] (null: no norm): q <- q / sqrt(sum q^2 / n_q + eps) * q_norm over
// the whole row, likewise k.  The first `dims` features of every head are rotated by
// pos * freq[i] (freq [dims / 2]), pairs (i, i + dims/2), or (2i, 2i+1) with `neighbours`; cos and
// sin are multiplied by `mult`.  Values: the v rows, or without them the keys as projected.
int yalm_qk_norm_rope_store(const float* qkv, int n_partials, long long partial_stride,
                            const float* bias, const float* q_norm, const float* k_norm, int n_q, int n_k, float eps,
                            const float* freq, int dims, int neighbours, float mult, float head_eps,
                            int head_size, const int* token_seq, const int* q_start, const int* seq_slot,
                            const int* slot_pos, void* q_out, void* kv_step, void* k_cache,
                            void* v_cache, int dtype, int n_tokens, int H, int G, int hd, int has_v,
                            int capacity, int write_cache, const int* page_table, int pages_per_slot,
                            int n_pages, cudaStream_t stream);
// The mean key and mean value of every block of `pool` positions that this step completes, into
// the pooled cache's row of that block; positions of this step come from kv_step, earlier ones
// from the ring (capacity >= pool - 1), before the step's late ring write if there is one.
int yalm_pool_blocks(const void* kv_step, const void* k_cache, const void* v_cache, const int* q_start,
                     const int* seq_slot, const int* slot_pos, void* pool_k, void* pool_v, int dtype,
                     int n_seqs, int max_q_len, int G, int hd, int capacity, int pool,
                     const int* page_table, int pages_per_slot, int n_pages, int pool_capacity,
                     const int* pool_table, int pool_pps, int pool_pages, int* status,
                     cudaStream_t stream);

// ---- sum_norm.cu: layers that norm after the residual sum ---------------------------------
// x [rows, dim] <- n(alpha x + scale0 B0 + scale1 B1, weight), n(v, w) = v / sqrt(mean v^2 + eps) w;
// Bj is the sum of nj float32 slices (sj floats apart), itself normed with wj and branch_eps when
// wj is not null.  h (null, or [rows, dim] of h_dtype) receives the new x in that type too.
int yalm_sum_norm(float* x, float alpha, int n_branches, const float* p0, int n0, long long s0,
                  const float* w0, float scale0, const float* p1, int n1, long long s1,
                  const float* w1, float scale1, float branch_eps, const float* weight, float eps,
                  void* h, int h_dtype, int rows, int dim, cudaStream_t stream);
int yalm_cast_rows(const float* x, void* out, int out_dtype, long long n, cudaStream_t stream);
// out [rows, heads * size] = each head's `size` values of o (float32) normed with w [size]
int yalm_head_norm(const float* o, const float* w, void* out, int out_dtype, long long rows, int heads,
                   int size, float eps, cudaStream_t stream);

// ---- recurrence.cu: S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T, o_t = S_t^T q_t per head ------
// proj: float32 slices [n_partials][tokens][2 H dk + H dv] = (q | f | v) before activation:
// q = silu(.), f = lower + (1 - lower) sigmoid(. + f_bias); act: float32 scratch of one slice's
// size (the activated projection, written by a first kernel and read by the scan); state
// [slots][H][dk][dv] float32; out float32 [tokens][H dv]
int yalm_gated_recurrence(const float* proj, int n_partials, long long partial_stride,
                          const float* f_bias, const float* lower, float* act, const int* q_start,
                          const int* seq_slot, float* state, float* out, int n_tokens, int n_seqs,
                          int H, int dk, int dv, cudaStream_t stream);

// ---- small_ops.cu ---------------------------------------------------------------------
// x[t] = E[token t] + P[row t] (also into x_copy when given): row = buckets for a sequence's
// position 0, else (previous token * mul_prev + token * mul_cur) mod buckets.  prev_token
// [slots] holds the last token each sequence has been given; the kernel keeps it up to date.
int yalm_embed_pair(const int* tokens, const int* token_seq, const int* q_start, const int* seq_slot,
                    const int* slot_pos, const void* table, const void* pair_table, int table_dtype,
                    int* prev_token, float* x, float* x_copy, int n_tokens, int dim, int vocab,
                    int buckets, long long mul_prev, long long mul_cur, int* status,
                    cudaStream_t stream);
// o [n, H, hd] *= sigmoid(sum of the n_partials slices of g [n, H])
int yalm_head_gate(void* o, int dtype, const float* g, int n_partials, long long partial_stride,
                   int n_tokens, int H, int hd, cudaStream_t stream);
// o [n] *= sigmoid(sum of the n_partials slices of g [n]), feature by feature (n % 4 == 0)
int yalm_element_gate(void* o, int dtype, const float* g, int n_partials, long long partial_stride,
                      long long n, cudaStream_t stream);
// v <- cap * tanh(v / cap) over n floats
int yalm_softcap(float* v, long long n, float cap, cudaStream_t stream);
// x += y + sum of n_partials slices, n floats each
int yalm_residual_add(float* x, const float* y, const float* partials, int n_partials,
                      long long partial_stride, long long n, cudaStream_t stream);

// ---- routed.cu: a routed feed-forward ----------------------------------------------------
int yalm_route_topk(const float* z, int n_partials, long long partial_stride, int n_tokens, int E,
                    int n_groups, int keep, int top, int renormalise, int sigmoid, int group_top2,
                    float norm_eps, float weight_scale, const float* correction, int* choice,
                    float* weight, int* counts, cudaStream_t stream);
int yalm_route_plan(int* counts, const int* choice, int n_pairs, int top, int E, int tile_rows,
                    int* first_row, int* pair_row, int* row_token, int* tile_expert, int* tile_row0,
                    int* n_tiles, cudaStream_t stream);
int yalm_gather_rows(const void* src, const int* row_token, void* dst, int dtype, int rows, int dim,
                     cudaStream_t stream);
int yalm_gemm_grouped(const void* A, int a_dtype, const void* W, int w_dtype, void* out, int out_dtype,
                      const int* first_row, const int* tile_expert, const int* tile_row0,
                      const int* n_tiles, int max_tiles, int N, int K, cudaStream_t stream);
// the same product on tcgen05 (gemm_tcgen05.cu): 16-bit operands, a plan of tile_rows-row tiles
// (16, 32, 64 or 128); mode 0 stores the product, mode 2 the gated activation of W = [gate; up]
int yalm_gemm_grouped_tc(const void* A, const void* W, int ab_dtype, void* out, int out_dtype,
                         int rows_total, int E, int N, int K, int mode, int tile_rows,
                         const int* first_row, const int* tile_expert, const int* tile_row0,
                         const int* n_tiles, int max_tiles, float slope, float limit, float shift,
                         int* status, cudaStream_t stream);
int yalm_glu_clamp(const float* gu, int n_partials, long long partial_stride, void* out, int out_dtype,
                   long long rows, int F, float alpha, float limit, float shift, int paired,
                   cudaStream_t stream);
int yalm_routed_combine(float* x, const float* y, const int* pair_row, const float* weight,
                        int n_tokens, int top, int dim, cudaStream_t stream);

// ---- hyper.cu: several residual copies per token -----------------------------------------------
// X [copies][rows][dim] float32.  Write (y not null): X_j <- sum_i mix[i][j] X_i + mult out_w[j] y, y the
// sum of n_partials slices.  Read (in_w not null): u = sum_i in_w[i] X_i, normed with norm_w into h
// (h_dtype), or without norm_w stored to u_out as float32.
int yalm_hc_step(float* X, int copies, long long rows, int dim, const float* y, int n_partials,
                 long long partial_stride, const float* mix, const float* out_w, float mult,
                 const float* in_w, const float* norm_w, float eps, void* h, int h_dtype, float* u_out,
                 cudaStream_t stream);

// ---- recurrence.cu: o_t = (S_(t-1) + diag(u) k_t v_t^T)^T r_t, S_t = diag(w_t) S_(t-1) + k_t v_t^T ------
int yalm_token_shift(const void* h, const float* prev, const float* mu, void* out, int dtype,
                     const int* token_seq, const int* q_start, const int* seq_slot, int n_tokens, int dim,
                     int n_mix, cudaStream_t stream);
int yalm_wkv(const float* r, int nr, long long sr, const float* k, int nk, long long sk, const float* v,
             int nv, long long sv, const float* g, int ng, long long sg, const float* z, int nz,
             long long sz, const float* w0, const float* bonus, float* act, float* gate, const void* h,
             int h_dtype, float* prev, const int* token_seq, const int* q_start, const int* seq_slot,
             float* state, float* out, int n_tokens, int n_seqs, int H, int dk, int dv, int dim,
             cudaStream_t stream);
int yalm_wkv_out(const float* o, const float* w, const float* gate, void* out, int out_dtype,
                 long long rows, int heads, int size, float eps, cudaStream_t stream);

// ---- latent.cu: attention over a cached latent ---------------------------------------------------
int yalm_latent_store(const float* dkv, int n_partials, long long partial_stride, const float* c_norm,
                      float eps, const float* freq, const int* token_seq, const int* q_start,
                      const int* seq_slot, const int* slot_pos, void* kv_step, void* cache, int dtype,
                      int n_tokens, int rank, int rd, int hd, int capacity, int write_cache,
                      const int* page_table, int pages_per_slot, int n_pages, cudaStream_t stream);
int yalm_latent_absorb_q(const float* q, int n_partials, long long partial_stride, const void* w_uk,
                         const float* freq, const int* token_seq, const int* q_start, const int* seq_slot,
                         const int* slot_pos, void* q_out, int dtype, int n_tokens, int H, int dim, int rd,
                         int rank, int hd, cudaStream_t stream);
int yalm_latent_expand(const void* o, const void* w_uv, const float* gate, int n_partials,
                       long long partial_stride, void* out, int dtype, int n_tokens, int H, int rank,
                       int vdim, int hd, cudaStream_t stream);

// ---- small_ops.cu ---------------------------------------------------------------------------------
// out [n] = act(sum of n_partials slices of z [n]): act 1 = gelu (tanh form), 2 = tanh
int yalm_activation_rows(const float* z, int n_partials, long long partial_stride, void* out,
                         int out_dtype, long long n, int act, cudaStream_t stream);


// ---- norm_step.cu: sublayer outputs that are normed before they join the residual stream ------------
int yalm_norm_step(float* x, const float* a, int na, long long sa, float fa, const float* b, int nb,
                   long long sb, float fb, int post_kind, const float* post_w, const float* post_b,
                   float post_alpha, float post_eps, int pre_kind, const float* pre_w, const float* pre_b,
                   float pre_alpha, float pre_eps, void* h, int h_dtype, const int* rows, int n_rows, int dim,
                   cudaStream_t stream);
int yalm_short_conv(const float* src, int n_partials, long long partial_stride, int src_row, int src_col0,
                    const float* in_bias, const float* w, const float* out_bias, int taps, int channels,
                    int silu, float* state, const int* token_seq, const int* q_start, const int* seq_slot,
                    float* out32, int out_row, int out_col0, void* out16, int out16_dtype, int block16,
                    int n_tokens, int n_seqs, int update_state, cudaStream_t stream);
int yalm_gated_rows(const float* z, int n_partials, long long partial_stride, const int* tokens,
                    const void* table, int table_dtype, int table_row, int first, void* out, int out_dtype,
                    int n_tokens, int dim, cudaStream_t stream);

// ---- delta_rule.cu: the gated delta rule with a decay per key channel ------------------------------
int yalm_delta_row(int H, int G, int dk, int dv);
int yalm_delta_prep(float* act, const float* proj, int n_partials, long long partial_stride, int proj_row,
                    int col_b, int col_low, int n_low, void* low, int low_dtype, int n_tokens, int H, int G,
                    int dk, int dv, cudaStream_t stream);
int yalm_delta_scan(float* act, const float* z, int n_partials, long long partial_stride,
                    const float* dt_bias, const float* a_log, float* gate, const int* q_start,
                    const int* seq_slot, float* state, float* out, int n_tokens, int n_seqs, int H, int G,
                    int dk, int dv, cudaStream_t stream);

// ---- rglru.cu: a real-gated linear recurrent unit per channel ---------------------------------------
int yalm_rglru(const float* gates, const float* ra_bias, const float* ri_bias, const float* lam,
               const float* u, const float* yx, int n_partials, long long partial_stride, int yx_row,
               const float* y_bias, float* coef, const int* q_start, const int* seq_slot, float* state,
               void* out, int out_dtype, int n_tokens, int n_seqs, int width, int bw, float c_decay,
               cudaStream_t stream);

#ifdef __cplusplus
}
#endif
