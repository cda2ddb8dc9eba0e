// C interface of the kernel library.  Every launcher enqueues on `stream`, allocates
// nothing, and returns 0 or an error code: a positive value is a cudaError_t, a
// negative one is one of the NIB_ERR_* codes below.
#pragma once

#include <cuda_runtime.h>

#define NIB_ERR_BAD_ARGUMENT (-1)
#define NIB_ERR_UNSUPPORTED_SIZE (-2)
#define NIB_ERR_DRIVER (-3)

// Values a kernel may leave in the device status word.
#define NIB_STATUS_OK 0
#define NIB_STATUS_BAD_PAGE 1
#define NIB_STATUS_WAIT_TIMEOUT 2

// Options of the attention kernels that take them, on the scores and on the output:
//   softcap > 0:  s <- softcap tanh(s / softcap) after the scale;
//   slopes:       one number per query head, s <- s - slopes[h] (query position - key position);
//   keep_first:   with a window, keys 0 .. keep_first - 1 stay visible behind it;
//   gate:         head h's output of row t is multiplied by sigmoid(gate[t * ldg + h]);
//   out_scale:    and by this constant;
//   span > 0:     position i sees key j only if floor(i / span) == floor(j / span) (spans count from position 0 of
//                 the sequence);
//   head_scale:   one number per query head that multiplies the scale (a temperature);
//   sinks:        with `sink` set, one number per query head: the denominator's extra term is exp(sinks[h]) instead
//                 of exp(0).
struct AttnExtras {
  float softcap;
  int keep_first;
  const float* slopes;
  const float* gate;
  int ldg;
  float out_scale;
  int span;
  const float* head_scale;
  const float* sinks;
};

#ifdef __cplusplus
extern "C" {
#endif

// A negative token -(s + 1) stands for feedback[s]: the token that the step before sampled for
// slot s and left on the device (feedback may be null when no token is negative).  out = table[token] * scale
// (+ pos_table[position]).
int nib_embed(int dtype, const int* tokens, const int* positions, const void* table,
              const void* pos_table, const int* feedback, float* out, int T, int C, float scale, cudaStream_t stream);

int nib_layernorm(int out_dtype, const float* x, const int* rows, const float* gamma,
                  const float* beta, void* out, int n_rows, int C, float eps, cudaStream_t stream);

int nib_kv_append(int dtype, const void* src, int ld, int k_off, int v_off, void* cache,
                  const int* block_table, int max_blocks, const int* row_entry, const int* positions,
                  int T, int n_kv_head, int head_dim, int page_size, int n_pages, int* status,
                  cudaStream_t stream);

// out[M,N] = act(a[M,K] . w[N,K]^T + bias); with `residual` the result is added to the
// 32-bit `out` in place.  SIMT path: true 32-bit arithmetic for float inputs.
int nib_linear_simt(int in_dtype, int out_dtype, const void* a, int lda, const void* w, int ldw,
                    const float* bias, void* out, int ldo, int M, int N, int K, int act,
                    int residual, cudaStream_t stream);

// The same product for bfloat16 inputs on the tensor cores (tcgen05 + TMA); out is bfloat16 or
// float32.  nib_linear_tc_supported says whether the shape and alignment are taken.
int nib_linear_tc_supported(const void* a, int lda, const void* w, int ldw, int K);
int nib_linear_tc(int out_dtype, const void* a, int lda, const void* w, int ldw, const float* bias,
                  void* out, int ldo, int M, int N, int K, int act, int residual, int* status,
                  cudaStream_t stream);

// The general tensor-core product for steps of at most 128 rows, with three options: activations made
// in the kernel by LayerNorm of the 32-bit residual stream (ln_x), keys and values written straight
// into a cache layer (cache), and K split over blocks through caller-provided scratch
// (fix_partials / fix_counters; the counters are zero before the first call and left zero).
int nib_linear_tc_small(int out_dtype, const void* a, int lda, const void* w, int ldw, const float* bias,
                        void* out, int ldo, int M, int N, int K, int act, int residual, const float* ln_x,
                        int ln_ldx, const float* ln_gamma, const float* ln_beta, float ln_eps,
                        const int* ln_rows, void* cache, const int* block_table, int max_blocks,
                        const int* row_entry, const int* positions, int q_dim, int n_kv_head, int head_dim,
                        int page_size, int n_pages, float* fix_partials, long long fix_floats,
                        int* fix_counters, int fix_n_counters, int* status, cudaStream_t stream);

// The product for many rows by pairs of blocks that share one 256-row MMA (cta_group::2): each block
// loads its own 128 rows of the activations and half of the weight tile.  bq: columns of a tile (0:
// chosen by the library; else a multiple of 32 up to 256); splits: splits of K for residual outputs
// (0: chosen by the library).  cache != null: the fused q/k/v projection, keys and values straight
// into the rows' slots of one cache layer (q_dim a multiple of 64, head_dim of 16).
int nib_linear_tc_pair_supported(int out_dtype, const void* a, int lda, const void* w, int ldw, const void* out,
                                 int ldo, int M, int N, int K, int residual);
int nib_linear_tc_pair(int out_dtype, const void* a, int lda, const void* w, int ldw, const float* bias, void* out,
                       int ldo, int M, int N, int K, int act, int residual, int bq, int splits, void* cache,
                       const int* block_table, int max_blocks, const int* row_entry, const int* positions,
                       int q_dim, int n_kv_head, int head_dim, int page_size, int n_pages, int* status,
                       cudaStream_t stream);

// The product for steps of at most 128 rows with warp-level MMAs (bfloat16; row blocks of 16), with the same
// LayerNorm and cache options as nib_linear_tc_small.  split: blocks of a cluster that split
// K (0: chosen by the library; else 1, 2, 4 or 8).
int nib_linear_skinny_supported(int M, int K, int ldw, int ln, const void* w);
int nib_linear_skinny(int out_dtype, const void* a, int lda, const void* w, int ldw, const float* bias, void* out,
                      int ldo, int M, int N, int K, int act, int residual, const float* ln_x, int ln_ldx,
                      const float* ln_gamma, const float* ln_beta, float ln_eps, const int* ln_rows,
                      void* cache, const int* block_table, int max_blocks, const int* row_entry,
                      const int* positions, int q_dim, int n_kv_head, int head_dim, int page_size, int n_pages,
                      int split, int* status, cudaStream_t stream);

// Causal attention of T query rows over the paged cache (general SIMT kernel).  rows: the
// step's rows to process (nullptr: rows 0..T-1).  `sink` (here and in the attention kernels below): 1 adds one
// term exp(0) to the softmax's denominator, a key of score 0 that has no value.
int nib_attention_simt(int dtype, const void* q, int ldq, const void* cache, void* out, int ldo,
                       const int* block_table, int max_blocks, const int* rows, const int* row_entry,
                       const int* positions, int T, int n_head, int n_kv_head, int head_dim,
                       int page_size, int n_pages, float scale, int window, int sink, float softcap,
                       int keep_first, const float* slopes, const float* gate, int ldg, float out_scale, int span, const float* head_scale, const float* sinks, int* status,
                       cudaStream_t stream);

// tcgen05 attention for prompt portions (bfloat16, head size 64, page size a multiple of 16): tiles of
// 128 query rows, S and O in tensor memory, keys and values by TMA page by page.  q holds T rows.  With the
// options of AttnExtras.
int nib_attention_prefill_tc_supported(int head_dim, int page_size);
int nib_attention_prefill_tc(const void* q, int ldq, int T, const void* cache, void* out, int ldo,
                             const int* block_table, int max_blocks, const int* tiles, int n_tiles,
                             const int* entry_start, const int* entry_pos0, int n_head, int n_kv_head, int head_dim,
                             int page_size, int n_pages, float scale, int window, int sink, float softcap, int keep_first,
                             const float* slopes, const float* gate, int ldg, float out_scale, int span, const float* head_scale, const float* sinks, int* status,
                             cudaStream_t stream);

// Split-KV attention for single decoded tokens (float32 or bfloat16, head sizes up to 128 in steps
// of 8, pages of a multiple of 16 positions) and its scratch need.
long long nib_attention_decode_scratch(int n_rows, int n_head, int head_dim, int n_splits);
int nib_attention_decode(int dtype, const void* q, int ldq, const void* cache, float* scratch, void* out,
                         int ldo, const int* block_table, int max_blocks, const int* rows,
                         const int* row_entry, const int* positions, int n_rows, int n_head, int n_kv_head,
                         int head_dim, int page_size, int n_pages, float scale, int window, int sink, float softcap,
                         int keep_first, const float* slopes, const float* gate, int ldg, float out_scale, int span, const float* head_scale, const float* sinks, int chunk,
                         int n_splits, int* counters, int* status, cudaStream_t stream);

// Tiled tensor-core attention for prompt portions (bfloat16, head sizes 16..128 in steps of 16), with the options of
// AttnExtras.
int nib_attention_prefill_supported(int head_dim);
int nib_attention_prefill(const void* q, int ldq, const void* cache, void* out, int ldo,
                          const int* block_table, int max_blocks, const int* tiles, int n_tiles,
                          const int* entry_start, const int* entry_pos0, int n_head, int n_kv_head,
                          int head_dim, int page_size, int n_pages, float scale, int window, int sink, float softcap,
                          int keep_first, const float* slopes, const float* gate, int ldg, float out_scale, int span, const float* head_scale, const float* sinks, int* status,
                          cudaStream_t stream);

// Loading: src holds [rows, cols] values as a checkpoint stores them (src_dtype 0: 32-bit floats, 1:
// bfloat16, 2: 16-bit floats); element (r, c) is converted to dst_dtype and written to
// dst[(r0 + r) * ld + c], or with `transpose` to dst[c * ld + r0 + r].
int nib_convert(int src_dtype, const void* src, int rows, int cols, int dst_dtype, void* dst, long long ld,
                long long r0, int transpose, cudaStream_t stream);

int nib_argmax(const float* logits, int ld, int n_rows, int V, int* out, cudaStream_t stream);

// One token per logits row.  temperature, top_k and rng_state are per-slot arrays indexed by
// row_slot[r]: argmax where temperature <= 0, else temperature / top-k sampling with the
// request's own xorshift64* state (advanced by one draw).
// last_token (may be null): per-slot array that also receives each row's token, for the next step's
// embedding to read.
// scratch: 2 * n_rows 64-bit words that are zero before the first call (the kernel leaves them zero).
// teams != 0: the launch is made of clusters whose blocks share a sampled row's passes (for steps in
// which some row may be sampled; the tokens are the same either way).
int nib_sample(const float* logits, int ld, int n_rows, int V, const int* row_slot,
               const float* temperature, const int* top_k, unsigned long long* rng_state, int* out,
               int* last_token, unsigned long long* scratch, int teams, cudaStream_t stream);

// ---- layers that normalise after the sum, and a weighted average over the layers' results (stream_norm.cu)
// out[r] = x[rows[r]] / sqrt(mean(x^2) + eps) * w (rows null: x[r]).
int nib_rmsnorm(int out_dtype, const float* x, const int* rows, const float* w, void* out, int n_rows, int C,
                float eps, cudaStream_t stream);
// xn = cast(x); level0 = x (may be null); x = alpha * x.
int nib_stream_enter(int out_dtype, float* x, void* xn, float* level0, float alpha, int n_rows, int C,
                     cudaStream_t stream);
// y = rmsnorm(x) * w; with levels [n_levels][level_stride]: levels[n_levels - 1] = y and z = sum_j mix[j] *
// levels[j], else z = y; xn = cast(z) (may be null); x = alpha_next * z.
int nib_post_norm(int out_dtype, float* x, const float* w, float eps, float* levels, long long level_stride,
                  int n_levels, const float* mix, void* xn, float alpha_next, int n_rows, int C,
                  cudaStream_t stream);
// kind 1: tanh; kind 2: xIELU with prm = {p, q} on the device.  in and out may be the same buffer.
int nib_unary(int in_dtype, int out_dtype, const void* in, int ld_in, void* out, int ld_out, int n_rows,
              int n_cols, int kind, const float* prm, cudaStream_t stream);

// x += y / sqrt(mean(y^2) + eps) * w_out; y = 0; with w_next: xn = cast(x / sqrt(mean(x^2) + eps) * w_next).
int nib_add_norm(int out_dtype, float* x, float* y, const float* w_out, const float* w_next, float eps, void* xn,
                 int n_rows, int C, cudaStream_t stream);
// out[t, f] = act(pre[t, 2f]) * pre[t, 2f + 1], times sigmoid(pre[t, row_gate]) where row_gate >= 0.
int nib_glu(int in_dtype, int out_dtype, const void* pre, int ld, void* out, int ldo, int n_rows, int F, int act,
            int row_gate, cudaStream_t stream);

// ---- rotary positions with the cast and the cache append (rope.cu)
int nib_rope_append(int dtype, const float* proj, int ld, int q_off, int k_off, int v_off, int n_head, int n_kv_head,
                    int dim, int vdim, int hd, int rot_dims, const double* freqs, const int* positions,
                    const int* row_entry, void* q_out, int ldq, void* cache, const int* block_table, int max_blocks,
                    int page_size, int n_pages, int T, int* status, cudaStream_t stream);

// ---- the matrix memory of xLSTM (mlstm.cu)
long long nib_mlstm_state_floats(int dim, int vdim);
int nib_mlstm(int dtype, const float* proj, int ld, int q_off, int k_off, int v_off, int g_off, int i_off, int f_off,
              const float* bias_i, const float* bias_f, float cap, const float* norm_w, float* state,
              const int* entry_start, const int* entry_slot, int n_entries, int n_rows, int n_head, int dim, int vdim,
              float eps, float* gates, float* num, int ld_num, float* den, void* out, int ldo, cudaStream_t stream);

// ---- attention through a shared low-rank latent (latent_attention.cu)
int nib_latent_prep(int dtype, const float* proj, int ld, int q_rank, int kv_rank, int rot_dim, int rot_dims,
                    const double* freqs, const float* wq, const float* wkv, float eps, void* cq, int ld_cq,
                    void* cache, const int* block_table, int max_blocks, const int* row_entry,
                    const int* positions, int T, int page_size, int n_pages, int has_kv, int* status,
                    cudaStream_t stream);
int nib_rope_heads(int dtype, const void* q, int ldq, int nope, int rot_dim, int rot_dims, const double* freqs,
                   const int* positions, float* out, int out_dim, int out_off, int n_head, int T,
                   cudaStream_t stream);
int nib_latent_attention(int dtype, const float* q, const void* cache, void* out, int ldo, const int* block_table,
                         int max_blocks, const int* rows, const int* row_entry, const int* positions, int n_rows,
                         int n_head, int kv_rank, int D, int page_size, int n_pages, float scale, int window,
                         int* status, int n_splits, float* partials, cudaStream_t stream);

// ---- a product per head (linear_heads.cu): out[t, h, :N] = a[t, h, :K] . w[h]^T, w [n_head, N, K]
int nib_linear_heads(int dtype, int out_dtype, const void* a, int lda, int a_head_stride, const void* w, void* out,
                     int ldo, int out_head_stride, int M, int n_head, int N, int K, cudaStream_t stream);

// ---- the generalised delta rule (delta_rule.cu)
int nib_delta_rule(int dtype, float* proj, int ld, int r_off, int k_off, int v_off, int g_off, int a_off,
                   float* wl, int ld_w, const float* w0, const float* a_bias, const float* norm_w,
                   float* state, const int* entry_start, const int* entry_slot, int n_entries, int n_rows, int n_head,
                   int dim, float eps, void* out, int ldo, float* unit, cudaStream_t stream);

// ---- a routed feed-forward (moe.cu)
// score 0: softmax over all experts; 1: the sigmoids of the chosen experts' logits.  choice_bias (may be null): one
// number per expert added to the score for the choice only.  The experts n_real .. n_expert - 1 have no matrices:
// a row that chooses one gets its own input times the score added to x [T, C] here, and the id -1.
int nib_moe_route(int dtype, const void* h, int ldh, const void* w_router, int T, int C, int n_expert, int top,
                  int renorm, int score, const float* choice_bias, int n_real, float* x, int* ids, float* weights,
                  cudaStream_t stream);
// gated: w_up [experts, 2F, C], rows 2f and 2f + 1 the gate and the value of output f; inner = act(s g) * (s u) with
// s = in_weights[t * top + k] (null: 1).
int nib_moe_up(int dtype, const void* h, int ldh, const void* w_up, const int* ids, void* inner, int T, int C,
               int F, int top, int act, float act_prm, int gated, const float* in_weights, cudaStream_t stream);
int nib_moe_gate_scale(int pre_dtype, int dtype, const void* pre, void* inner, const int* ids, const float* weights,
                       int T, int n_expert, int F, int top, int act, float act_prm, int on_input, cudaStream_t stream);
int nib_moe_down(int dtype, const void* inner, const void* w_down, const int* ids, const float* weights, float* x,
                 int T, int C, int F, int top, cudaStream_t stream);
// inner [T, n_expert * F] in place: expert e's part of row t times the row's weight for e (0 where not chosen).
int nib_moe_scale(int dtype, void* inner, const int* ids, const float* weights, int T, int n_expert, int F, int top,
                  cudaStream_t stream);
// Expert-major forms for steps of many rows: phase 0 = up (out [T * top, N] in dtype; phase 3: gated, N = 2F
// interleaved rows, out [T * top, F], weights scaling the inputs), phase 1 = down into
// out float [T * top, N] (weighted), phase 2 = x[t] += the sum of row t's parts (src = the parts).
int nib_moe_grouped(int dtype, int phase, const void* src, int ld_src, const void* w, const int* ids,
                    const float* weights, void* out, float* x, int T, int top, int n_expert, int N, int K, int act,
                    float act_prm, cudaStream_t stream);

// Sinusoidal positions added to the 32-bit stream x [T, C]: entry 2i += sin(position * freqs[i]), entry 2i + 1 += cos.
int nib_add_sinusoid(float* x, const int* positions, const double* freqs, int T, int C, cudaStream_t stream);

// out[t, d] = act(pre[t, d]) * table[token_t, off + d] for d < D (tokens as in nib_embed).
int nib_gate_by_table(int dtype, const float* pre, int ld, const int* tokens, const int* feedback, const void* table,
                      int table_ld, int off, int D, int act, void* out, int ldo, int n_rows, cudaStream_t stream);

// nib_rope_append with an RMS norm of every query and key head ahead of the rotation (weights of `dim` values shared
// by the heads; either may be null).
int nib_norm_rope_append(int dtype, const float* proj, int ld, int q_off, int k_off, int v_off, int n_head,
                         int n_kv_head, int dim, int vdim, int hd, const float* wq, const float* wk, float eps,
                         int rot_dims, const double* freqs, const int* positions, const int* row_entry, void* q_out,
                         int ldq, void* cache, const int* block_table, int max_blocks, int page_size, int n_pages, int T,
                         int* status, cudaStream_t stream);

// Recurrent mixers with a matrix state per head (gated_scan.cu): the short causal convolution with its state, the
// decays and strengths (and unit queries and keys) of the rows, the recurrence itself, and the gated norm behind it.
int nib_short_conv(const float* proj, int ld, int c_off, int Cn, int taps, const float* w, const float* bias,
                   float* state, long long state_stride, const int* row_entry, const int* entry_start,
                   const int* entry_slot, float* out, int ldo, int T, int n_entries, int act, int fused,
                   void* out16, int ld16, cudaStream_t stream);
int nib_scan_prepare(const float* proj, int ld, int a_off, int w_off, const float* A_log, const float* dt_bias,
                     float* cv, int ldc, int q_off, int k_off, int N, int n_head, int n_kq, int delta, float* coef, int T,
                     cudaStream_t stream);
int nib_gated_scan_padded(int N);
int nib_gated_scan(int delta, const float* cv, int ldc, int q_off, int k_off, int v_off, int N, int V, int n_head,
                   int kq_ratio, const float* coef, const float* skip, float* state, long long state_stride,
                   long long s_off, const int* entry_start, const int* entry_slot, int n_entries, float* out, int ldo,
                   cudaStream_t stream);
int nib_gated_norm(int out_dtype, const float* o, int ldo, const float* gate, int ldg, const float* weight, int wlen,
                   int n_groups, int gs, float eps, int gate_first, float out_scale, void* out, int ld_out, int T,
                   cudaStream_t stream);

// ---- rotary positions in the halves layout (rope.cu): value i of a head's first rot_dims values pairs with value
// i + rot_dims / 2.  nib_wide_norm_rope_append: queries and keys normed over the whole projection (wq [n_head * dim],
// wk [n_kv_head * dim]; null: no norm), turned, cast, padded to hd and written to q_out and the cache (cache null:
// queries only); the values are read at v_off as they stand.  nib_rope_halves: in place on 32-bit rows, the keys
// then times k_mul, and coef[t, h] = (decay[h], 1) where coef is given.
int nib_wide_norm_rope_append(int dtype, const float* src, int ld, int q_off, int k_off, int v_off, int n_head,
                              int n_kv_head, int dim, int vdim, int hd, const float* wq, const float* wk, float eps,
                              int rot_dims, const double* freqs, const int* positions, const int* row_entry, void* q_out,
                              int ldq, void* cache, const int* block_table, int max_blocks, int page_size, int n_pages,
                              int T, int* status, cudaStream_t stream);
int nib_rope_halves(float* rows, int ld, int q_off, int k_off, int n_head, int dim, int rot_dims, const double* freqs,
                    const int* positions, float k_mul, const float* decay, float* coef, int T, cudaStream_t stream);

// ---- hyper-connections (hyper.cu): S copies of the residual stream, stream_stride floats apart.
int nib_hyper_enter(int dtype, const float* x, float* streams, long long stream_stride, int S, const float* in_w,
                    const float* w_next, float eps, void* xn, int T, int C, cudaStream_t stream);
int nib_hyper_update(int dtype, float* streams, long long stream_stride, int S, float* y, const float* gate, int ldg,
                     const float* mix, const float* out_w, const float* in_next, const float* w_next, float eps, void* xn,
                     float* total, int T, int C, cudaStream_t stream);

// ---- the selective scan of Mamba (selective_scan.cu)
long long nib_selective_scan_state_floats(int inner, int N);
int nib_selective_scan(int out_dtype, const float* dtp, int ld_dt, const float* x, int ldx, const float* bc, int ldbc,
                       int b_off, int c_off, const float* z, int ldz, const float* A_log, const float* D, float* state,
                       long long state_stride, long long s_off, const int* entry_start, const int* entry_slot,
                       int n_entries, int inner, int N, void* out, int ldo, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
