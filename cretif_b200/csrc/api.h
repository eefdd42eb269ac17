// The C interface of the kernel library.
//
// Every launcher takes raw device pointers, sizes and the CUDA stream to launch on, and
// returns 0 when the kernel was launched, a negative cretif::Status for arguments it does
// not take, or a positive cudaError_t.  Element types are passed as codes: 0 = float32,
// 1 = bfloat16.  Nothing here allocates device memory.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

// out[t, :] = table[ids[t], :] widened to float32 (+ pos_table[tok_pos[t], :] when a table of P
// learned position vectors is given).  An id outside [0, V), or a position outside [0, P), sets
// bit 1 of *fault and writes zeros.
int cretif_embed_rows(const void* table, int table_dt, const int* ids, float* out, int T, int H,
                      int V, unsigned int* fault, const void* pos_table, const int* tok_pos, int P,
                      void* stream);

// v = h[src] (+ delta[src]); if write_h, h[src] = v; out[r] = v * weight * rsqrt(mean(v^2)+eps).
// src = rows ? rows[r] : r.  delta may be null.  rows and write_h exclude each other.
int cretif_add_rmsnorm(float* h, const void* delta, int delta_dt, const float* weight, void* out,
                       int out_dt, const int* rows, int R, int H, float eps, int write_h,
                       void* stream);

// act[t, i] = silu(gate) * up; block = 0: gu row = [gate | up]; block = b: groups of b gate
// columns followed by their b up columns.
int cretif_silu_mul(const void* gu, void* act, int dt, int T, int I, int block, void* stream);

// Rotate q and k of every token by its position's angles (pairing 0: (j, j+rot/2),
// 1: (2j, 2j+1)); q in place.  write_cache bit 0: rotated k and v into the block cache;
// bit 1: k rotated in place too (encoding only; with rot_dim 0 and bit 0 it only stores).
int cretif_rope_kv_append(void* qkv, int ld, int dt, const float* cos_t, const float* sin_t,
                          int pairing, int rot_dim, int nh, int nkv, int hd, const int* tok_pos,
                          const int* tok_seq, const int* seq_slot, const int* table,
                          int table_stride, void* kc, void* vc, int bt, int write_cache, int T,
                          unsigned int* fault, void* stream);

// h[r, :] += y[r, :] * weight * rsqrt(mean(y[r]^2) + eps): a norm on a sublayer's output, fused
// with the residual addition (32-bit).  x_out (bfloat16 [R, H], may be null) receives the new rows.
int cretif_rmsnorm_add(float* h, const void* y, int y_dt, int ldy, const float* weight, int R,
                       int H, float eps, void* x_out, void* stream);

// out = h converted to the element type out_dt (the stream handed to a sublayer without a norm).
int cretif_convert_rows(const float* h, void* out, int out_dt, long long total, void* stream);

// rows [T, ld] = [q (q_dim) | k (nkv * hd) | ...].  With wq: q <- rmsnorm over all q_dim columns
// times wq, in place.  k: rmsnorm over all nkv*hd columns times wk goes to the key cache at each
// token's position; with vc, the columns as they are (before the norm) go to the value cache.
int cretif_proj_norm_kv_append(void* rows, int ld, int dt, int q_dim, const float* wq, int nkv,
                               int hd, const float* wk, float eps, const int* tok_pos,
                               const int* tok_seq, const int* seq_slot, const int* table,
                               int table_stride, void* kc, void* vc, int bt, int write_cache,
                               int T, unsigned int* fault, void* stream);

// The gated delta rule (delta_rule.cu).  proj rows (float32): [q (G d) | k (G d) | v (H e) |
// gate (H e) | b (H) | a (H)]; prep rows: [q | k | v | beta (H) | decay (H)].  conv_state and
// state point at the first sequence slot's saved inputs [C, taps-1] and matrices [H, d, e];
// state_stride is a slot's size in floats.
int cretif_delta_prepare(const float* proj, int ldp, float* prep, int ldo, const float* conv_w,
                         int taps, const float* conv_state, long long state_stride,
                         const float* a_log, const float* dt_bias, const int* tok_pos,
                         const int* tok_seq, const int* seq_slot, const int* seq_start, int H,
                         int G, int d, int e, float unit_eps, int T, void* stream);
int cretif_delta_conv_state(const float* proj, int ldp, float* conv_state, long long state_stride,
                            int taps, int C, const int* cu_seqlens, const int* seq_slot, int B,
                            void* stream);
// o_raw: float32 scratch [T, H e] for the read-outs before their norm.
int cretif_delta_recurrence(const float* prep, int ldp, const float* gate, int ldg, float* state,
                            long long state_stride, const int* cu_seqlens, const int* seq_slot,
                            int B, int H, int G, int d, int e, const float* norm_w, float eps,
                            float* o_raw, void* out, int out_dt, int ldo, int write_state, int T,
                            void* stream);

// Dynamic Tanh, dyt(x) = (tanh(alpha x) w + b) gain, a norm without statistics (pointwise_norm.cu);
// alpha points at one float on the device, gain may be null.
// dyt_rows: v = h[src] (+ delta[src]); if write_h, h[src] = v; out[r] = dyt(v); src = rows ? rows[r] : r.
int cretif_dyt_rows(float* h, const void* delta, int delta_dt, const float* w, const float* b,
                    const float* alpha, const float* gain, void* out, int out_dt, const int* rows,
                    int R, int H, int write_h, void* stream);
// h[r] += dyt(y[r]): the norm on a sublayer's output, fused with the residual sum.
int cretif_dyt_add(float* h, const void* y, int y_dt, int ldy, const float* w, const float* b,
                   const float* alpha, const float* gain, int R, int H, void* stream);
// out[t] = n[t] + (n[t-1] - n[t]) * shift with n = dyt(h) (n = h when w is null); a sequence's
// first token of the step reads the row saved in state[slot] and replaces it by the step's last.
int cretif_shift_rows(const float* h, const float* w, const float* b, const float* alpha,
                      const float* shift, float* state, long long state_stride,
                      const int* tok_seq, const int* seq_slot, const int* cu_seqlens, void* out,
                      int out_dt, int T, int H, void* stream);

// Between an attention's projections and its scores (conv_attn.cu): causal convolution over
// time of every channel of proj [q (nh hd) | k (nkv hd) | v (nkv vd)] (float32), unit RMS per q
// and k head, the query times 1 + gain_coef ln(floor((pos + 1) / gain_every) + 1) (gain_every
// 0: no gain), q into q_out, k and v into the block cache.  nkv = 0: queries only.
int cretif_conv_headnorm_kv_append(const float* proj, int ldp, const float* conv_w, int taps,
                                   const float* conv_state, long long state_stride,
                                   const int* tok_pos, const int* tok_seq, const int* seq_slot,
                                   const int* seq_start, int nh, int nkv, int hd, int vd,
                                   float eps, float gain_coef, int gain_every, void* q_out,
                                   int ldq, int dt, const int* table, int table_stride, void* kc,
                                   void* vc, int bt, int write_cache, int T, unsigned int* fault,
                                   void* stream);

// The generalized delta rule (delta_rule.cu).  proj rows (float32): [r (H d) | k (H d) | v (H e) |
// gate (H e) | a (H d) | w1 (R)]; prep rows: [u (H d) | b (H d) | w (H d)].
// z rows: W2 tanh(w1) [H d] (the expanding product of the decay's low rank).
int cretif_general_delta_prepare(const float* proj, int ldp, float* prep, int ldo,
                                 const float* a_bias, const float* z, int ldz, const float* w0,
                                 int H, int d, int e, float unit_eps, float decay_scale, int T,
                                 void* stream);
// out[t, j] = tanh(in[t * ld + j]), j < R, in the element type out_dt.
int cretif_tanh_cols(const float* in, int ld, void* out, int out_dt, int R, int T, void* stream);
int cretif_general_delta_recurrence(const float* proj, int ldp, const float* prep, int ldq,
                                    const float* gate, int ldg, float* state,
                                    long long state_stride, const int* cu_seqlens,
                                    const int* seq_slot, int B, int H, int d, int e,
                                    const float* norm_w, int per_head_weight, int gate_sigmoid,
                                    float eps, float* o_raw, void* out, int out_dt, int ldo,
                                    int write_state, int T, void* stream);

// Attention over a cached latent (latent_ops.cu).  A projection row holds
// [cq (q_rank) | c (rank) | kr (rot) | ...]: cq and c are brought to unit RMS and multiplied by wq
// and wc, kr is rotated by the token's position; cq goes to cq_out, [c | kr] into the token's row
// of the key cache (one key/value head of size rank + rot).  Of the rot channels the first rdims
// are rotated, the rest pass; pairing 0: channel i with i + rdims/2, 1: channel 2i with 2i + 1.
int cretif_latent_in(const void* proj, int ldp, int proj_dt, int q_rank, int rank, int rot,
                     int rdims, const float* wq, const float* wc, float eps, const float* cos_t,
                     const float* sin_t, int pairing, const int* tok_pos, const int* tok_seq,
                     const int* seq_slot, void* cq_out, int ldq, int dt, const int* table,
                     int table_stride, void* kc, int bt, int write_cache, int T,
                     unsigned int* fault, void* stream);
// q [T, nh (d + rot)]: the last rot channels of every head, the first rdims of them rotated, go
// to out[t, h * ldh + off ...].
int cretif_rope_heads(const void* q, int ldq, int q_dt, int nh, int d, int rot, int rdims,
                      const float* cos_t, const float* sin_t, int pairing, const int* tok_pos, void* out, int ldo,
                      int ldh, int off, int dt, int T, void* stream);
// x <- x / sqrt(mean(x^2) + eps) * w in place, float32 rows.
int cretif_rmsnorm_rows(float* x, int ld, const float* w, int R, int H, float eps, void* stream);

// Routed experts (moe.cu).
// groups > 1: the experts form that many equal groups of neighbours, a group's score is the sum
// of its two largest logistic scores, only experts of the `keep` best groups can be chosen.
// renorm: the chosen scores are divided by (their sum + sum_eps).
int cretif_moe_route(const void* x, int x_dt, int ldx, const float* router_w, int E, int H,
                     int top, int renorm, int groups, int keep, float sum_eps, int* ids,
                     float* wts, int T, void* stream);
int cretif_moe_topk(const float* logits, int ld, int E, int top, int renorm, int groups, int keep,
                    float sum_eps, int* ids, float* wts, int T, void* stream);
int cretif_moe_group(const int* ids, int P, int E, int* offsets, int* place, int* order,
                     int* tile_expert, int* tile_row0, int max_tiles, void* stream);
int cretif_moe_gemm(const void* A, int a_dt, int lda, const void* W, int w_dt, void* C, int ldc,
                    int N, int K, int top, int mode, int scale_at, const float* wts,
                    const int* order, const int* offsets, const int* tile_expert,
                    const int* tile_row0, int max_tiles, int use_mma, void* stream);
int cretif_moe_gemv(const void* A, int a_dt, int lda, const void* W, int w_dt, void* C, int ldc,
                    int N, int K, int top, int mode, int scale_at, const int* ids,
                    const float* wts, int P, void* stream);
int cretif_moe_group_padded(const int* ids, int P, int E, int tile, int* place, int* tile_expert,
                            int max_tiles, int* used, void* stream);
int cretif_moe_gather_rows(const void* x, int ldx, void* xs, int lds, const int* place,
                           const float* wts, int top, int K, int P, void* stream);
// place may be null: the rows are in the pairs' own order; wts may be null: no weights.
int cretif_moe_combine(const float* rows, int ld, const int* place, int top, const float* wts,
                       float* y, int T, int H, void* stream);

// After a decode step: ids <- sampled (if given), positions and lengths + 1.
int cretif_advance_decode(int* tok_ids, int* tok_pos, int* seq_start, const int* sampled, int B,
                          void* stream);

// C[M,N] (= or +=) A[M,K] · W[N,K]^T, 32-bit FMA on the CUDA cores.
int cretif_gemm_simt(const void* A, int a_dt, const void* W, int w_dt, void* C, int c_dt, int M,
                     int N, int K, int lda, int ldw, int ldc, int accumulate, void* stream);

// `batch` products in one launch: product z reads A + z*sa, W + z*sw and writes C + z*sc
// (strides in elements), e.g. a matrix per head applied to that head's columns of the rows.
int cretif_gemm_simt_batched(const void* A, int a_dt, const void* W, int w_dt, void* C, int c_dt,
                             int M, int N, int K, int lda, int ldw, int ldc, int batch,
                             long long sa, long long sw, long long sc, void* stream);

// The same batch in bfloat16 on the tensor cores (mma.sync through the warp-level matrix API):
// W is [batch, N, K] contiguous, A and C rows have strides lda and ldc and product z starts at
// A + z*sa and C + z*sc.  Any M, N, K.
int cretif_gemm_heads(const void* A, const void* W, void* C, int M, int N, int K, int lda, int ldc,
                      int batch, long long sa, long long sc, void* stream);

// C[M,N] (= or +=) X[M,K] · W[N,K]^T for M <= 64 rows, bfloat16 operands, streaming W once.
// K and the row strides must be multiples of 8 and the operands 16-byte aligned.
int cretif_gemm_skinny(const void* X, const void* W, void* C, int c_dt, int M, int N, int K,
                       int ldx, int ldw, int ldc, int accumulate, void* stream);
int cretif_gemm_skinny_max_rows(void);

// C[M,N] (= or +=) A[M,K] · W[N,K]^T on the tcgen05 tensor cores (TMA + TMEM), bfloat16
// operands, C bfloat16 or float32 (+= only float32).  bn = 64/128/192/256 picks the tile width,
// 0 lets the launcher choose.  The product is multiplied by alpha before it is stored or added;
// unary (0 none, 1 relu^2, 2 gelu in its tanh form, 3 silu, 4 gelu with the error function;
// stores only) is applied to the
// 32-bit sums before they are rounded.  A wait that expires sets bit 2 of *fault.
int cretif_gemm_tc(const void* A, const void* W, void* C, int c_dt, int M, int N, int K, int lda,
                   int ldw, int ldc, int accumulate, int bn, float alpha, int unary,
                   unsigned int* fault, void* stream);

// (For tests that run both.)  Epilogue warps of the tensor-core product: 4 or 8; 0, the default,
// chooses per launch.  Returns the old setting.
int cretif_set_tc_epilogue_warps(int n);

// (For tests that run both.)  Adding into a float32 matrix, and storing the SiLU product,
// through shared memory and TMA: on by default.  Returns the old setting.
int cretif_set_tc_bulk_add(int on);

// (For tests that run both.)  Two CTAs on a tile (cta_group::2) for the float32 add and the
// SiLU product: -1 where the launcher sees fit (default), 0 never, 1 wherever the kernel takes
// the product.  Returns the old setting.
int cretif_set_tc_pair(int mode);

// The same product with fused epilogues (see gemm_tc.cu): SiLU·mul for the stacked gate|up
// matrix whose rows are interleaved in blocks of 64 (I % 64 == 0), and rotary + cache write for
// the stacked q|k|v matrix (head_dim 64 or 128, rotary over the whole head).
int cretif_gemm_tc_silu(const void* A, const void* Wgu, void* act, int M, int I, int K, int lda,
                        int ldw, unsigned int* fault, void* stream);
// The same products in groups: A [M, K], M a multiple of 128, whose 128-row tiles each belong to a
// group (tile_group[M / 128]; *used_m_tiles tiles are in use, the others are left alone), and
// W [groups, N, K] ([groups, 2 I, K] interleaved as above); C float32 [M, N], act [M, I].
int cretif_gemm_tc_grouped(const void* A, const void* W, void* C, int M, int N, int K, int lda,
                           int ldw, int ldc, int groups, const int* tile_group,
                           const int* used_m_tiles, unsigned int* fault, void* stream);
// C bfloat16 [M, N] = act(A W[g]^T): unary = 1 + a kind of cretif_activation.
int cretif_gemm_tc_act_grouped(const void* A, const void* W, void* C, int M, int N, int K, int lda,
                               int ldw, int ldc, int groups, const int* tile_group,
                               const int* used_m_tiles, int unary, unsigned int* fault,
                               void* stream);
int cretif_gemm_tc_silu_grouped(const void* A, const void* Wgu, void* act, int M, int I, int K,
                                int lda, int ldw, int groups, const int* tile_group,
                                const int* used_m_tiles, unsigned int* fault, void* stream);
int cretif_gemm_tc_qkv_rope(const void* A, const void* Wqkv, void* Q, int ldq, const float* cos_t,
                            const float* sin_t, int pairing, int nh, int nkv, int hd,
                            const int* tok_pos, const int* tok_seq, const int* seq_slot,
                            const int* table, int table_stride, void* kc, void* vc, int bt,
                            int write_cache, int M, int K, int lda, int ldw, unsigned int* fault,
                            void* stream);

// Causal grouped-query attention over the block cache, any step shape.  sink (may be null):
// one float per query head, exp(sink) joins the softmax's denominator without a key or value.
// vd: size of a value head (the cache's values are [blocks, nkv, bt, vd], out rows nh * vd).
// bias (may be null): float32 [bias_rows, nh] added to the scaled score of the key n positions
// back, row = the last r with bias_edges[r] <= n (edges ascending, edges[0] = 0).
// slope (may be null): float32 [nh]; slope[h] * n is taken off that score.
// window, here and in every attention entry point: > 0 a sliding window of that many keys,
// < 0 chunks of -window positions counted from 0 (a query sees the keys of its own chunk), 0 all.
int cretif_attn_simt(const void* q, int ldq, void* out, int ldo, int dt, const void* kc,
                     const void* vc, const int* table, int table_stride, const int* tok_pos,
                     const int* tok_seq, const int* seq_slot, int nh, int nkv, int hd, float scale,
                     int window, int bt, int T, const float* sink, int vd, const float* bias,
                     const int* bias_edges, int bias_rows, const float* slope, void* stream);

// Decode attention (one query token per sequence), bfloat16, keys split into n_splits <= 64
// ranges per (sequence, kv head); part_o/part_ml are float32 scratch of the sizes that
// cretif_attn_decode_scratch_floats reports, counters is int32 [B * nkv], zero before the
// first launch and left zero by every launch.  block tokens must be 64.
int cretif_attn_decode_scratch_floats(int B, int nh, int hd, int n_splits, long long* part_o,
                                      long long* part_ml);
int cretif_attn_decode(const void* q, int ldq, void* out, int ldo, const void* kc, const void* vc,
                       const int* table, int table_stride, const int* tok_pos, const int* tok_seq,
                       const int* seq_slot, int nh, int nkv, int hd, float scale, int window,
                       int bt, int B, int n_splits, float* part_o, float* part_ml, int* counters,
                       unsigned int* fault, void* stream);

// The same operation on the tensor cores (mma.sync, TMA-swizzled tiles), head_dim <= 128;
// same scratch and counters.  n_blocks is the cache's block count.  With part_o null and at
// most 8 ranges, the ranges of a sequence form a thread-block cluster and are merged through
// distributed shared memory: no scratch, no counters.
int cretif_attn_decode_mma(const void* q, int ldq, void* out, int ldo, const void* kc,
                           const void* vc, long long n_blocks, const int* table, int table_stride,
                           const int* tok_pos, const int* tok_seq, const int* seq_slot, int nh,
                           int nkv, int hd, float scale, int window, int bt, int B, int n_splits,
                           float* part_o, float* part_ml, int* counters, unsigned int* fault,
                           void* stream);

// The same with a sink (may be null): one float per query head whose exponential joins the
// softmax's denominator where the ranges are merged.
int cretif_attn_decode_mma_sink(const void* q, int ldq, void* out, int ldo, const void* kc,
                                const void* vc, long long n_blocks, const int* table,
                                int table_stride, const int* tok_pos, const int* tok_seq,
                                const int* seq_slot, int nh, int nkv, int hd, float scale,
                                int window, int bt, int B, int n_splits, float* part_o,
                                float* part_ml, int* counters, const float* sink,
                                unsigned int* fault, void* stream);
// ... and with a bias by distance (see cretif_attn_prefill_tc_bias).  head_groups = G > 1: more
// than eight query heads on a key/value head go as G groups in one launch: B counts (sequence,
// group) items, rows of q, out, tok_pos and tok_seq are laid out by item, item b serves heads
// (b % G) * nh .. of the G * nh heads whose sink and bias rows follow one another.
int cretif_attn_decode_mma_bias(const void* q, int ldq, void* out, int ldo, const void* kc,
                                const void* vc, long long n_blocks, const int* table,
                                int table_stride, const int* tok_pos, const int* tok_seq,
                                const int* seq_slot, int nh, int nkv, int hd, float scale,
                                int window, int bt, int B, int n_splits, float* part_o,
                                float* part_ml, int* counters, const float* sink,
                                const float* bias_near, const float* bias_far, int n_far,
                                int head_groups, const float* bias_slope, unsigned int* fault,
                                void* stream);

// Fused decode projections (see decode_fused.cu).  H is the float32 residual stream; when it
// is given, x = bf16(rmsnorm(H[rows])) is computed in the kernel, else X (bfloat16) is read.
// cretif_fused_linear stores or adds alpha times the product; unary as in cretif_gemm_tc.
int cretif_fused_linear(const void* X, int ldx, const float* H, const float* norm_w,
                        const int* rows, float eps, const void* W, int ldw, void* C, int c_dt,
                        int ldc, int accumulate, float alpha, int unary, int M, int N, int K,
                        unsigned int* fault, void* stream);
int cretif_fused_qkv_rope(const float* H, const float* norm_w, float eps, const void* Wqkv, int ldw,
                          void* Q, int ldq, const float* cos_t, const float* sin_t, int pairing,
                          int nh, int nkv, int hd, const int* tok_pos, const int* tok_seq,
                          const int* seq_slot, const int* table, int table_stride, void* kc,
                          void* vc, int bt, int write_cache, int M, int K, unsigned int* fault,
                          void* stream);
int cretif_fused_gate_up_silu(const float* H, const float* norm_w, float eps, const void* Wgu,
                              int ldw, void* act, int I, int gu_block, int M, int K,
                              unsigned int* fault, void* stream);
int cretif_fused_gate_up_silu_x(const void* X, int ldx, const void* Wgu, int ldw, void* act, int I,
                                int gu_block, int M, int K, unsigned int* fault, void* stream);
int cretif_fused_smem_ok(int M, int K, int norm_prologue);
// The three switches below exist so that tests can run both variants of a kernel on one
// shape; an ordinary run never touches them.
// Programmatic dependent launch of the fused kernels on (default) or off; returns the old value.
int cretif_set_dependent_launch(int on);
// Matrices with at least k columns, or of at least min_bytes bytes (negative: unchanged), take
// the shared-memory streaming variant (decode_stream.cuh); returns the old column threshold.
int cretif_set_stream_min_k(int k, long long min_bytes);
long long cretif_stream_min_bytes(void);
// The register variant with more than eight rows and a norm prologue shares the rows'
// normalisation among the CTAs of a thread-block cluster of up to n (1: every CTA norms
// every row itself; at most 4, the default).  Returns the old value; n < 1 leaves it.
int cretif_set_fused_cluster(int n);

// Causal attention for whole prompts on tcgen05 (bfloat16, head_dim a multiple of 16 up to
// 128, 64-token cache blocks).  qkv rows hold the query heads first; sequence b brings the
// tokens cu_seqlens[b] .. cu_seqlens[b+1]-1 at positions seq_start[b] ..; max_new is the
// most tokens one sequence brings.
int cretif_attn_prefill_tc(const void* qkv, int ldq, int T, void* out, int ldo, const void* kc,
                           const void* vc, long long n_blocks, const int* table, int table_stride,
                           const int* cu_seqlens, const int* seq_start, const int* seq_slot,
                           int nh, int nkv, int hd, float scale, int window, int bt, int B,
                           int max_new, unsigned int* fault, void* stream);

// The same with a sink (may be null): one float per query head whose exponential joins each
// row's denominator (the kernel with two threads per row serves it).
int cretif_attn_prefill_tc_sink(const void* qkv, int ldq, int T, void* out, int ldo,
                                const void* kc, const void* vc, long long n_blocks,
                                const int* table, int table_stride, const int* cu_seqlens,
                                const int* seq_start, const int* seq_slot, int nh, int nkv, int hd,
                                float scale, int window, int bt, int B, int max_new,
                                const float* sink, unsigned int* fault, void* stream);
// ... and with a bias by distance: bias_near [nh, n_far] and bias_far [nh] (float32, already
// multiplied by log2 e; both null for none) are added to the scaled score of the key n positions
// back, bias_near[h, n] for n < n_far and bias_far[h] for every n beyond.  bias_slope [nh]
// (float32, times log2 e; null for none, not together with the table): n times bias_slope[h] is
// taken off that score instead, at any distance.
int cretif_attn_prefill_tc_bias(const void* qkv, int ldq, int T, void* out, int ldo,
                                const void* kc, const void* vc, long long n_blocks,
                                const int* table, int table_stride, const int* cu_seqlens,
                                const int* seq_start, const int* seq_slot, int nh, int nkv, int hd,
                                float scale, int window, int bt, int B, int max_new,
                                const float* sink, const float* bias_near, const float* bias_far,
                                int n_far, const float* bias_slope, unsigned int* fault,
                                void* stream);

// Per-head work of an attention whose projections are normed head by head (head_ops.cu).
// proj rows [q (nh hd) | k (nkv hd) | v (nkv vd) | ...] (float32 or bfloat16): + bias (null for
// none), RMS norm of every q and k head times wq / wk (hd numbers each, both null for none),
// rotation of the first rot_dim channels by the position (pairing 0: (i, i + rot_dim/2), 1:
// (2i, 2i+1)); q to q_out, k and v into the block cache (write_cache; else only q is made).
int cretif_headnorm_rope_kv_append(const void* proj, int ldp, int proj_dt, const float* bias,
                                   const float* wq, const float* wk, float eps, const float* cos_t,
                                   const float* sin_t, int pairing, int rot_dim,
                                   const int* tok_pos, const int* tok_seq, const int* seq_slot,
                                   int nh, int nkv, int hd, int vd, void* q_out, int ldq, int dt,
                                   const int* table, int table_stride, void* kc, void* vc, int bt,
                                   int write_cache, int T, unsigned int* fault, void* stream);
// o[t, h, :] *= sigmoid(g[t, h]) for nh heads of vd channels.
int cretif_gate_heads(void* o, int ldo, int dt, const float* g, int ldg, int nh, int vd, int T,
                      void* stream);
// out = act(in) element by element: kind 0 relu(z)^2, 1 gelu in its tanh form, 2 silu,
// 3 gelu with the error function.
int cretif_activation(const void* in, int ldi, int in_dt, void* out, int ldo, int out_dt, int T,
                      int width, int kind, void* stream);
// z <- cap * tanh(z / cap) in place.
int cretif_softcap(float* z, long long total, float cap, void* stream);
// h += alpha * y over `total` elements (y float32 or bfloat16).
int cretif_axpy_rows(float* h, const void* y, int y_dt, float alpha, long long total,
                     void* stream);

// Retention (retention.cu).  proj rows (float32): [q (H d) | k (H d) | ...]; prep rows: the
// rotated q and the rotated k times k_scale.  state points at the first sequence slot's
// matrices [H, d, e]; state_stride is a slot's size in floats.  o_raw [T, H e] receives the
// read-outs S^T q after S <- decay_h S + k v^T.  form: 0 lets the step's shape choose between
// the recurrence token by token (1) and 64 tokens at a time (2, refused where the sizes or
// addresses do not allow 16-byte accesses).
int cretif_retention_prepare(const float* proj, int ldp, float* prep, int ldo, const float* cos_t,
                             const float* sin_t, int pairing, int rot_dim, const int* tok_pos,
                             int H, int d, float k_scale, int T, void* stream);
int cretif_retention_recurrence(const float* prep, int ldp, const float* v, int ldv,
                                const float* decay, float* state, long long state_stride,
                                const int* cu_seqlens, const int* seq_slot, int B, int H, int d,
                                int e, float* o_raw, int write_state, int T, int form,
                                void* stream);
// out = o_raw / rms(o_raw) per head [* norm_w] * gate(gate): norm_w null, of e numbers, or of
// H e (per_head_weight); the gate is SiLU or the logistic function (gate_sigmoid).
int cretif_heads_out_norm(const float* o_raw, const float* gate, int ldg, const float* norm_w,
                          int per_head_weight, int gate_sigmoid, float eps, void* out, int out_dt,
                          int ldo, int H, int e, int T, void* stream);

// One CTA waits, with the library's bounded wait, on a barrier that nothing completes; after
// `limit` polls (at most 2^20) it gives up, sets bit 2 of *fault and returns.  *polls (may be
// null) receives `limit` when the kernel has run.  Nothing faults or hangs: it exists so that
// the path from an expired wait to the host's error can be exercised.
int cretif_wait_that_expires(unsigned int limit, unsigned int* fault, unsigned int* polls,
                             void* stream);

// (For tests that run all.)  Which kernel cretif_attn_prefill_tc gives head sizes up to 64
// without a window: -1 as the launcher sees fit (default), 0 two threads per row, 1 a thread per
// row and two query tiles per CTA, 2 a thread per row and one tile per CTA.  Returns the old
// setting.
int cretif_set_prefill_pairing(int mode);

// How often variant v of a kernel (cretif::Variant in common.cuh) has been launched; -1 for an
// unknown v.  For tests that must know which path ran.
int cretif_variant_count(int v);

// One token id per row of logits: greedy (temperature <= 0), temperature, or top-k.  The
// kernel reads the seed from *seed_dev when that is not null, else takes `seed`.
int cretif_sample(const float* logits, int ld, int rows, int V, float temperature, int top_k,
                  unsigned long long seed, const unsigned long long* seed_dev,
                  const long long* request, int* draw, int* out, void* stream);
float cretif_uniform01(unsigned long long seed, long long request, int draw);
int cretif_max_top_k(void);

#ifdef __cplusplus
}
#endif
