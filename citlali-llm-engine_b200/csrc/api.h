// The C interface of the kernel library.  Every function launches on the given stream and
// returns 0, a cudaError_t (> 0), or a refusal (< 0) whose text citlali_last_error() gives.
// dtype codes: 0 = float32, 1 = bfloat16.  All sizes are in elements unless named bytes.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

const char* citlali_last_error(void);

// 1 (default): kernels are launched so that they may start before the kernel before them has
// finished, and wait for it on the device; 0: plain stream order.
void citlali_set_dependent_launch(int enabled);

// out[m, :] = table[tokens[m], :] widened to float32 and multiplied by `scale` (1: a plain row copy).
int citlali_embed_rows(const void* table, int table_dtype, const int32_t* tokens, float* out,
                       int rows, int hidden, int vocab, float scale, int32_t* error_flag, cudaStream_t stream);

// The same into `copies` buffers `copy_stride` elements apart (the residual streams of a model that has several).
int citlali_embed_rows_copies(const void* table, int table_dtype, const int32_t* tokens, float* out, int rows, int hidden,
                              int vocab, float scale, int32_t* error_flag, int copies, size_t copy_stride, cudaStream_t stream);

// rows_out = bfloat16(x) [rows, hidden] and sumsq[r, g] = sum of x[r, 32 g .. 32 g + 31]^2 (hidden a multiple of 32):
// what citlali_gemm_tc_normed's `scale_sumsq` reads, for rows that did not come out of an emitting product.
int citlali_norm_inputs(const float* x, void* rows_out, float* sumsq, int rows, int hidden, cudaStream_t stream);

// x[0..n) *= scale.
int citlali_scale(float* x, size_t n, float scale, cudaStream_t stream);
// x = cap tanh(x / cap) over n floats, cap > 0.
int citlali_soft_cap(float* x, size_t n, float cap, cudaStream_t stream);
// out[r] = [a[r] | b[r]] for two float32 matrices [rows, width], rounded once to out's type.
int citlali_concat_rows(const float* a, const float* b, void* out, int out_dtype, int rows, int width, cudaStream_t stream);

// out[r, :] = x[idx[r], :] * rsqrt(mean(x^2) + eps) * gain   (idx may be null: identity).
int citlali_rms_norm(const float* x, const void* gain, int gain_dtype, const int32_t* row_index,
                     void* out, int out_dtype, int rows, int hidden, float eps, cudaStream_t stream);

// act[m, i] = silu(gate) * up, gate/up taken from one [rows, 2*inter] matrix whose columns
// alternate in runs of `run`: gate run, up run, gate run, ...
int citlali_swiglu(const void* gate_up, void* act, int dtype, int rows, int inter, int run,
                   cudaStream_t stream);

// y[M, N] = x[M, K] . w[N, K]^T on CUDA cores with float accumulation, k ascending.
// accumulate != 0: y (float32) += product.
int citlali_gemm_simt(const void* x, int x_dtype, const void* w, int w_dtype, void* y, int y_dtype,
                      int M, int N, int K, int accumulate, cudaStream_t stream);

// In place on a [rows, (nq + 2 nkv) d] projection: per-head RMSNorm of q and k, half-split
// rotation by the row's position, then k and v written to the paged cache of the row's slot.
// The first `rotary_dim` elements of a head are rotated in pairs (i, i + rotary_dim/2), the rest pass through.
// write_cache: 0 leaves the cache alone (a layer that reads another layer's cache); 1 stores k and v; 2 writes
// the normed, rotated k back into the row instead and leaves v alone (a second call then stores them).
int citlali_qk_norm_rope_cache(void* qkv, int dtype, const void* q_gain, const void* k_gain, int gain_dtype,
                               const float* inv_freq, int rotary_dim,
                               const int32_t* row_slot, const int32_t* row_pos,
                               const int32_t* page_table, int page_table_stride,
                               void* k_pool, void* v_pool, int cache_dtype, int page_size,
                               int rows, int nq, int nkv, int head_dim, float eps, int write_cache,
                               cudaStream_t stream);

// Causal attention of every row over the cache of its slot: keys lo..pos, lo = 0 or
// pos - window + 1.  One order of operations for prompts and for single tokens.
int citlali_attention_rows(const void* q, int q_stride, int dtype,
                           const void* k_pool, const void* v_pool, int cache_dtype,
                           const int32_t* page_table, int page_table_stride,
                           const int32_t* row_slot, const int32_t* row_pos,
                           void* out, int out_stride, int rows, int nq, int nkv, int head_dim,
                           int page_size, int window, int max_keys, float scale,
                           cudaStream_t stream);

// Attention of single new tokens (bfloat16) split over the context; positions are read on the
// device, `max_positions` bounds them and fixes the grid.  `partial` is float scratch of
// citlali_attention_decode_scratch_floats(...) elements.  `counters` (may be nullptr): `counter_ints` 32-bit
// words, at least rows * nkv * ceil((nq / nkv) / 16), zero before the first call; every call leaves them zero.
// With them, a step of many rows deals the pages of its long rows out to several blocks by the rows' lengths.
size_t citlali_attention_decode_scratch_floats(int rows, int nq, int head_dim, int page_size, int max_positions);
int citlali_attention_decode(const void* q, int q_stride, const void* k_pool, const void* v_pool,
                             const int32_t* page_table, int page_table_stride,
                             const int32_t* row_slot, const int32_t* row_pos,
                             void* out, int out_stride, float* partial, size_t partial_floats,
                             int32_t* counters, size_t counter_ints,
                             int rows, int nq, int nkv, int head_dim, int page_size, int window,
                             int max_positions, float scale, cudaStream_t stream);
void citlali_attention_decode_set_split(int split);
void citlali_attention_decode_set_by_length(int on, int run_scale_q8);
void citlali_attention_decode_set_per_warp(int on);

// Causal attention of runs of new tokens (bfloat16, pages of 64) on the tensor cores.  Sequence b
// owns rows seq_start[b] .. seq_start[b+1]-1 at positions seq_past[b] + i of slot seq_slot[b].  window > 0: a row sees
// its last `window` keys and the sequence's first `keep_first` keys.
int citlali_attention_prefill_supports(int head_dim, int page_size);
int citlali_attention_prefill(const void* q, int q_stride, const void* k_pool, const void* v_pool,
                              const int32_t* page_table, int page_table_stride,
                              const int32_t* seq_start, const int32_t* seq_slot, const int32_t* seq_past,
                              void* out, int out_stride, int sequences, int max_new,
                              int nq, int nkv, int head_dim, int page_size, int window, int keep_first, float scale,
                              float softcap, const float* gate, size_t gate_stride, cudaStream_t stream);

// The same on tcgen05 (scores and output in tensor memory), for head size 128 and pages of 64.
// total_rows: rows of q over all sequences; pool_pages: pages of the layer's key and value pools.
int citlali_attention_prefill_tc_supports(int head_dim, int page_size);
int citlali_attention_prefill_tc(const void* q, int q_stride, int total_rows,
                                 const void* k_pool, const void* v_pool, int pool_pages,
                                 const int32_t* page_table, int page_table_stride,
                                 const int32_t* seq_start, const int32_t* seq_slot, const int32_t* seq_past,
                                 void* out, int out_stride, int sequences, int max_new,
                                 int nq, int nkv, int head_dim, int page_size, int window, float scale,
                                 int32_t* error_flag, cudaStream_t stream);

// tokens[r] = argmax of logits[r, :] over finite values, lowest index on ties.
int citlali_argmax_rows(const float* logits, int32_t* tokens, int rows, int vocab, cudaStream_t stream);
// The same with 64 blocks per row; scratch holds rows * 128 floats.
int citlali_argmax_rows_wide(const float* logits, int32_t* tokens, float* scratch, int rows, int vocab,
                             cudaStream_t stream);

// tokens[r] = first index whose inclusive CDF of softmax(logits[r] / temperature[r]) exceeds
// uniform[r]; temperature[r] <= 0 means argmax.
int citlali_sample_rows(const float* logits, const float* temperature, const float* uniform,
                        int32_t* tokens, int rows, int vocab, cudaStream_t stream);

// The tensor-core product (bfloat16 operands, float accumulation).  citlali_gemm_tc_plan tells
// how a shape runs: whether the weights are the 128-row operand (*swapped), the narrow tile
// (*bn) and the K split (*splits).  force_splits > 0 replaces the plan's split (at most 8).
int citlali_gemm_tc_plan(int M, int N, int K, int sm_count, int force_splits, int* swapped, int* bn, int* splits);
// y = x[M, K] . w[N, K]^T.  mode bits: 1 = y (float32) += product; 2 = SiLU-gate epilogue (w's rows
// alternate in runs of 16 between gate and up; y is bfloat16 [M, N/2]).  K must be a multiple of 8
// and the operands 16-byte aligned.  A shape that splits K runs each tile's splits as a cluster
// that sums its partials through distributed shared memory, in split order; no scratch is needed.
// error_flag[1..2] receive the code and block of a wait that ran out.
int citlali_gemm_tc(const void* x, const void* w, void* y, int y_dtype, int M, int N, int K,
                    int mode, int force_splits, int32_t* error_flag, int sm_count, cudaStream_t stream);
// The same for few rows of x with a layer norm's work in the epilogue (gemm_tcgen05.cu says what each pointer means;
// null pointers: plain citlali_gemm_tc).
int citlali_gemm_tc_normed(const void* x, const void* w, void* y, int y_dtype, int M, int N, int K,
                           int mode, int force_splits, int32_t* error_flag, int sm_count,
                           void* emit_rows, float* emit_sumsq, const float* scale_sumsq, int scale_groups,
                           int scale_dim, float scale_eps, cudaStream_t stream);
// The same product on pairs of SMs (tcgen05.mma with cta_group::2: a [256 x BN] tile per cluster of two
// blocks, each fetching half of both operands).  With equal waves it takes 0.92-0.97 of the one-block
// kernel's time at 512 to 4,096 rows and 0.82 at 8,192, and it loses where its 256-row tiles need a wave
// more.  citlali_gemm_tc uses it from citlali_gemm_tc_set_pair_rows' number of rows on (512 unless set;
// 0: never; the call returns the number that stood before) where the waves of pairs cost less, on devices
// that run such clusters; citlali_gemm_tc_runs_on_pairs says whether a shape goes there, and
// citlali_gemm_tc_pair_plan gives the tile width and the pairs that run at once.
int citlali_gemm_tc_pair(const void* x, const void* w, void* y, int y_dtype, int M, int N, int K,
                         int mode, int32_t* error_flag, cudaStream_t stream);
int citlali_gemm_tc_pair_plan(int M, int N, int K, int* bn, int* pairs);
// Many rows: the row tiles run in bands whose rows of x (this many bytes, default 32 MiB) stay in L2 while all
// weight tiles pass by.  Sets the size and returns the one before (for tuning).
long citlali_gemm_tc_pair_set_band_bytes(long bytes);
int citlali_gemm_tc_set_pair_rows(int rows);
// The kernels' bounded wait on its own: a block waits `limit_ns` (at most one second) on a barrier on which
// nothing arrives, gives up, records code 900 in error_flag[1] and its block in error_flag[2], and leaves
// normally; result[0] = the wait's return value (0), result[1] = the block's abort word (1).
int citlali_wait_selftest(int32_t* error_flag, int* result, long long limit_ns, cudaStream_t stream);
int citlali_gemm_tc_runs_on_pairs(int M, int N, int K, int sm_count, int gate_runs);

// ---- residual streams (hyper-connections) ----------------------------------------------------------------------
// X [streams, rows, width] float32, `stream_stride` elements between streams.
// out[r, :] = u / sqrt(mean(u^2) + eps) * gain with u = sum_s w_in[s] X[s, r, :]; gain float32 [width].
int citlali_hyper_read_norm(const float* X, size_t stream_stride, int streams, const float* w_in, const float* gain,
                            void* out, int out_dtype, int rows, int width, float eps, cudaStream_t stream);
// X[t, e] <- sum_s w_mix[s * streams + t] X[s, e] + w_out[t] y[e] for the n elements of a stream, all t from the old values.
int citlali_hyper_write(float* X, size_t stream_stride, int streams, const float* y, const float* w_mix,
                        const float* w_out, size_t n, cudaStream_t stream);
// citlali_hyper_write, then citlali_hyper_read_norm of the new values with w_in and gain, in one pass over the streams.
int citlali_hyper_write_read_norm(float* X, size_t stream_stride, int streams, const float* y, const float* w_mix,
                                  const float* w_out, const float* w_in, const float* gain, void* out, int out_dtype,
                                  int rows, int width, float eps, cudaStream_t stream);
// out[i, :] = sum_s X[s, index[i], :]  (index may be null: identity).
int citlali_stream_sum(const float* X, size_t stream_stride, int streams, const int32_t* index, float* out, int rows,
                       int width, cudaStream_t stream);
// y = max(x, 0)^2 over n elements.
int citlali_relu_squared(const void* x, void* y, int dtype, size_t n, cudaStream_t stream);

// ---- the gated delta rule --------------------------------------------------------------------------------------
// proj [rows, proj_stride] float32 = q (KH D) | k (KH D) | v (H V) | gate (H V) | b (H) | a (H) per row.  Convolves the
// q, k, v channels over time (taps_w [C, taps], the last column is the current token's; earlier tokens come from the
// step's rows or from state[slot][conv_off ...], laid out [taps - 1, C]), applies SiLU, makes q and k heads unit
// vectors (q also times D^-1/2), and writes prep [rows, C + 2 H] = q | k | v | sigmoid(b) | exp(-exp(a_log) softplus(a +
// dt_bias)).  Then stores each sequence's last taps - 1 inputs in its state.  block_a_segment != 0: the form for steps of few
// rows (a block a head instead of a warp; a head's squares are summed in another order, so a caller that wants the same bits
// from every step size keeps to one form).
int citlali_delta_prepare(const float* proj, int proj_stride, const float* taps_w, int taps, float* state,
                          size_t state_stride, size_t conv_off, const int32_t* row_slot, const int32_t* seq_start,
                          const int32_t* seq_slot, int sequences, const float* a_log, const float* dt_bias, float* prep,
                          int rows, int H, int KH, int D, int V, float unit_eps, int block_a_segment, int beta_col,
                          int decay_col, const float* decay_in, int decay_stride, int channel_decay, cudaStream_t stream);
// (beta_col, decay_col: the columns of b and a in a row of proj.  decay_in (rows decay_stride floats apart) given: the
// decays' inputs come from there instead of proj.  channel_decay: one decay a head and key channel instead of one a head,
// g = exp(-exp(a_log[h]) softplus(decay_in[h D + i] + dt_bias[h D + i])); prep is then [rows, C + H + H D].)
// The recurrence over each sequence's rows, from and into state[slot][0 ...] = S [H, D, V]; out [rows, H V] float32.
// pairs != 0: a sequence's rows are taken two at a time (the same numbers up to rounding, fewer dependent steps).
// mode 0: one decay a head; 1: a decay a key channel (row i of S times g_i; prep as above); 2: no correction term,
// u = beta v, which is a state-space recurrence S <- g S + beta k v^T, o = S^T q.
int citlali_delta_rule(const float* prep, int prep_stride, float* state, size_t state_stride, const int32_t* seq_start,
                       const int32_t* seq_slot, int sequences, int H, int KH, int D, int V, float* out, int pairs, int mode,
                       cudaStream_t stream);
// y[r, h, :] = o[r, h, :] / sqrt(mean(o^2) + eps) * weight * act(gate[r * gate_stride + h V ...]); gate_act 0: SiLU, 1: sigmoid.
int citlali_delta_output(const float* o, const float* gate, int gate_stride, const float* weight, void* y, int y_dtype,
                         int rows, int H, int V, float eps, int gate_act, cudaStream_t stream);

// ---- a norm on a sub-layer's output ------------------------------------------------------------------------------
// x[r] += layer_norm(y[r]) * gain  (mean and variance of the row, variance = mean of squared deviations, no bias), float32;
// emit (may be null) receives the updated rows in emit_dtype.
int citlali_layer_norm_add(const float* y, const void* gain, int gain_dtype, float* x, void* emit, int emit_dtype, int rows,
                           int hidden, float eps, cudaStream_t stream);
// out[i] = layer_norm(x[index[i]]) * gain (index may be null: identity).
// bias (of the gain's dtype; may be null) is added.
int citlali_layer_norm_rows(const float* x, const void* gain, const void* bias, int gain_dtype, const int32_t* row_index,
                            void* out, int out_dtype, int rows, int hidden, float eps, cudaStream_t stream);
// x[r] += layer_norm(y[r] + in_bias) * g1 + b1; emit (may be null) receives the updated rows in out_dtype; with g2 also
// out2[r] = layer_norm(x[r]) * g2 + b2 in out_dtype: the norm behind a sub-layer, the sum, and the norm in front of the next
// sub-layer in one pass.  in_bias, b1 and b2 may be null; gains and biases are float32.
int citlali_layer_norm_chain(const float* y, const float* in_bias, const float* g1, const float* b1, float* x, void* emit,
                             const float* g2, const float* b2, void* out2, int out_dtype, int rows, int hidden, float eps1,
                             float eps2, cudaStream_t stream);
// out = x converted from float32.
int citlali_cast_rows(const float* x, void* out, int out_dtype, size_t n, cudaStream_t stream);
// out = a l + b r over n floats.
int citlali_scaled_sum(float a, const float* l, float b, const float* r, float* out, size_t n, cudaStream_t stream);

// ---- mixers with a state per sequence ------------------------------------------------------------------------------
// out[row, c] = act(sum_j taps_w[c, j] u(t - taps + 1 + j) + bias[c]) for channels c < C, where u of a row of this step is
// in[row, c] + in_bias[c] and u of an earlier token comes from state[slot][conv_off ...] = [taps - 1, C] (zero at a
// sequence's start).  in_bias and bias may be null; act 0: none, 1: SiLU.  keep != 0: afterwards every sequence's last
// taps - 1 inputs are stored in its state (citlali_conv_keep).
int citlali_causal_conv(const float* in, int in_stride, const float* in_bias, const float* taps_w, int taps, const float* bias,
                        int act, float* state, size_t state_stride, size_t conv_off, const int32_t* row_slot,
                        const int32_t* seq_start, const int32_t* seq_slot, int sequences, float* out, int out_stride, int rows,
                        int C, int keep, cudaStream_t stream);
int citlali_conv_keep(const float* in, int in_stride, const float* in_bias, int taps, float* state, size_t state_stride,
                      size_t conv_off, const int32_t* seq_start, const int32_t* seq_slot, int sequences, int C,
                      cudaStream_t stream);
// The state-space mixer's preparation.  proj [rows, proj_stride] = z (H P) | x (H P) | B (G N) | C (G N) | dt (H); x, B, C
// pass the convolution (with bias) and SiLU; prep [rows, 2 G N + H P + 2 H] = C | B | x | softplus(dt + dt_bias) |
// exp(-exp(a_log) dt): what citlali_delta_rule in mode 2 reads with KH = G, D = N, V = P.  Keeps the last inputs.
int citlali_ssm_prepare(const float* proj, int proj_stride, const float* taps_w, int taps, const float* conv_bias, float* state,
                        size_t state_stride, size_t conv_off, const int32_t* row_slot, const int32_t* seq_start,
                        const int32_t* seq_slot, int sequences, const float* a_log, const float* dt_bias, float* prep, int rows,
                        int H, int P, int G, int N, cudaStream_t stream);
// y = (o + skip[h] x) * silu(z), divided by the root mean square of its norm group (`groups` equal parts of a row, eps
// inside the root), times weight.  x = prep[row, x_col ...], z = proj[row, 0 ...].
int citlali_ssm_output(const float* o, const float* prep, int prep_stride, int x_col, const float* proj, int proj_stride,
                       const float* skip, const float* weight, void* y, int y_dtype, int rows, int H, int P, int groups,
                       float eps, cudaStream_t stream);
// The gates of a linear recurrent unit.  u [rows, width] in `blocks` equal parts; per part b: r = sigmoid(Wa_b u_b + ba_b),
// i = sigmoid(Wi_b u_b + bi_b), the matrices given transposed [blocks, in, out]; a = exp(-8 r softplus(lam)),
// coef = sqrt(1 - a^2) i u.
int citlali_lru_gates(const float* u, const float* wa_t, const float* ba, const float* wi_t, const float* bi, const float* lam,
                      float* a_out, float* coef_out, int rows, int width, int blocks, cudaStream_t stream);
// S <- a S + coef per channel over each sequence's rows, from and into state[slot][state_off ...]; out[row] = S *
// gelu_tanh(side[row] + side_bias).
int citlali_gated_scan(const float* a, const float* coef, const float* side, int side_stride, const float* side_bias,
                       float* state, size_t state_stride, size_t state_off, const int32_t* seq_start, const int32_t* seq_slot,
                       int sequences, void* out, int out_dtype, int width, cudaStream_t stream);

// ---- attention over a window that keeps the first tokens ------------------------------------------------------------
// proj [rows, proj_stride] float32 = q (nq d) | k (nkv d) | v (nkv vd).  Every channel passes a causal convolution (taps_w
// [C, taps], no bias; kept inputs as in citlali_causal_conv; the caller stores them afterwards with citlali_conv_keep); q and
// k heads then an RMS norm with q_gain / k_gain [d] (null: none) and the rotation of elements (2i, 2i+1), 2i < rot_dims, by
// position * inv_freq[i].  q goes to q_out [rows, nq d]; with write_cache k and v go to the paged pools
// [page, nkv, page_size, d] and [page, nkv, page_size, vd].  bias (may be null): float32 [C], added to what the
// convolution gives, ahead of the head norm.
int citlali_conv_heads_prepare(const float* proj, int proj_stride, const float* taps_w, int taps, float* state,
                               size_t state_stride, size_t conv_off, const float* q_gain, const float* k_gain,
                               const float* inv_freq, int rot_dims, const int32_t* row_slot, const int32_t* row_pos,
                               const int32_t* page_table, int table_stride, void* k_pool, void* v_pool, int cache_dtype,
                               int page_size, void* q_out, int q_dtype, int rows, int nq, int nkv, int d, int vd, float eps,
                               int write_cache, const float* bias, cudaStream_t stream);
// out [rows, nq vd]: softmax attention of every row over the keys j <= pos of its slot with pos - j < window or
// j < keep_first (window 0: all keys).  max_keys bounds the keys a row sees (shared memory).  softcap > 0: the scaled
// score s becomes softcap tanh(s / softcap).  gate (may be null): float32, out[r, c] *= sigmoid(gate[r gate_stride + c]).
int citlali_attention_window(const void* q, int q_dtype, const void* k_pool, const void* v_pool, int cache_dtype,
                             const int32_t* page_table, int table_stride, const int32_t* row_slot, const int32_t* row_pos,
                             void* out, int rows, int nq, int nkv, int d, int vd, int page_size, int window, int keep_first,
                             int max_keys, float scale, float softcap, const float* gate, size_t gate_stride,
                             cudaStream_t stream);

// ---- routed experts ----------------------------------------------------------------------------------------------------
// weights [rows, E] = softmax(logits) at the `top` best experts among those of the `keep` best of `groups` equal groups of
// neighbours (a group's score is its largest score; groups <= 1: no groups), 0 elsewhere; chosen [rows, top] (may be
// null) their indices, best first.
// The chosen experts' weights are multiplied by weight_scale.  score_kind 1: the scores are sigmoid(logits), each by itself.
int citlali_moe_route(const float* logits, float* weights, int32_t* chosen, int rows, int E, int groups, int keep, int top,
                      float weight_scale, int score_kind, cudaStream_t stream);
// act [rows, E ff + tail_ff] from gate_up [rows, 2 (E ff + tail_ff)], whose columns are, expert after expert, gate and up
// alternating in runs of `run` (the last expert, which every row uses with weight 1, in runs of `tail_run`).  kind 0:
// silu(g) u; kind 1: min(g, limit) sigmoid(alpha min(g, limit)) (clamp(u, -limit, limit) + 1).  Routed expert e's
// activations are multiplied by weights[r, e]; where that is zero they are zeros and the inputs are not read.
// kind 2: gelu_tanh(g) u.  bias (may be null): float32 [2 (E ff + tail_ff)] in the columns' order, added to gate and up
// first.  weight_input != 0: the weight multiplies what the expert reads instead of what it gives, act(w g, w u): for
// experts without biases that is the expert applied to w times its input.
int citlali_expert_gate(const void* gate_up, int in_dtype, const float* weights, void* act, int act_dtype, int rows, int E,
                        int ff, int run, int kind, float limit, float alpha, int tail_ff, int tail_run, float tail_limit,
                        const float* bias, int weight_input, cudaStream_t stream);
// out = xielu(z + bias) over [rows, n]: u > 0: ap u^2 + u / 2; u <= 0: an (exp(u) - 1 - u) + u / 2.  bias may be null.
int citlali_bias_xielu(const void* z, int z_dtype, const float* bias, float ap, float an, void* out, int out_dtype, int rows,
                       int n, cudaStream_t stream);
// y[r] += bias over float32 [rows, n].
int citlali_add_row_bias(float* y, const float* bias, int rows, int n, cudaStream_t stream);
// act[r, e, :] *= weights[r, e] over act [rows, E, ff].
int citlali_moe_scale(void* act, int dtype, const float* weights, int rows, int E, int ff, cudaStream_t stream);

// ---- attention through a shared latent -------------------------------------------------------------------------
// proj [rows, proj_stride] float32 = query latent (RQ) | latent (R) | shared key part (P) | ...; cq [rows, RQ] receives
// the normed query latent; with has_kv the normed latent and the key part, rotated by the row's position in pairs
// (2i, 2i+1) below rot_dims, go to pool [page, page_size, R + P] at the row's slot and position.
int citlali_latent_prepare(const float* proj, int proj_stride, int RQ, int R, int P, int has_kv, const float* q_weight,
                           const float* c_weight, const float* inv_freq, int rot_dims, const int32_t* row_slot,
                           const int32_t* row_pos, const int32_t* page_table, int table_stride, void* pool,
                           int cache_dtype, int page_size, void* cq, int cq_dtype, int rows, float eps, int rot_halves,
                           cudaStream_t stream);
// y[r, h, n] = sum_k x[r * x_row + h * x_head + k] M[h * m_head + k * m_k + n * m_n]; with tail > 0 the elements
// x[r, h, K .. K + tail) are rotated like a key part and copied to y[r, h, N ...]; with gate, y *= sigmoid(gate[r, h N + n])
// (gate_per_head: sigmoid(gate[r, h])).  rot_halves (here and in citlali_latent_prepare): element i < rot_dims / 2 turns
// with element i + rot_dims / 2 instead of 2i with 2i + 1.
int citlali_heads_product(const void* x, int x_dtype, size_t x_row, int x_head, const void* M, int m_dtype, size_t m_head,
                          int m_k, int m_n, void* y, int y_dtype, size_t y_row, int y_head, int rows, int heads, int K,
                          int N, int tail, const float* inv_freq, int rot_dims, const int32_t* row_pos, const float* gate,
                          size_t gate_stride, int rot_halves, int gate_per_head, cudaStream_t stream);
// out[r, h, :R] = sum_j p_j c_j over the keys lo..pos of the row's slot (lo = 0, or pos - window + 1 with a window),
// p = softmax of scale * q[r, h, :] . pool[j, :], the denominator also counting exp(sink[h]) when sink is given.
int citlali_latent_attention(const float* q, const void* pool, int cache_dtype, const int32_t* page_table,
                             int table_stride, const int32_t* row_slot, const int32_t* row_pos, const float* sink,
                             float* out, int rows, int H, int R, int E, int page_size, int window, float scale,
                             cudaStream_t stream);
// The same walk on the tensor cores for a bfloat16 cache (sixteen heads of a token are an MMA tile's rows); E a multiple
// of 16, R a multiple of 64 (citlali_latent_attention_mma_supports).  splits > 1: a (row, sixteen heads) unit's key tiles
// are dealt to that many blocks and merged by a second kernel; partial holds units * splits * 16 * (R + 2) floats.
int citlali_latent_attention_mma_supports(int R, int E);
int citlali_latent_attention_mma(const float* q, const void* pool, const int32_t* page_table, int table_stride,
                                 const int32_t* row_slot, const int32_t* row_pos, const float* sink, float* out, int rows,
                                 int H, int R, int E, int page_size, int window, float scale, int splits, float* partial,
                                 size_t partial_floats, cudaStream_t stream);


// ---- attention with sigmoid weights on scores that the heads share ---------------------------------------------------
// proj [rows, C] float32 = q (H D) | k (G D) | v (G V) | gate (H) (k and v only with has_kv, the gate only with has_gate),
// plus bias [C] (may be null).  q times the row's temperature 1 + temp_coef ln(floor((pos + 1) / temp_every) + 1)
// (temp_every 0: none) goes to q_out [rows, H D]; k and v go to the paged pools [page, G, page_size, D] / [.., V];
// gate_out [rows, H] receives the gate's sigmoid.
int citlali_biased_heads_prepare(const float* proj, const float* bias, const int32_t* row_slot, const int32_t* row_pos,
                                 const int32_t* page_table, int table_stride, void* k_pool, void* v_pool, int cache_dtype,
                                 int page_size, void* q_out, int q_dtype, float* gate_out, int rows, int H, int G, int D, int V,
                                 int has_kv, int has_gate, float temp_coef, int temp_every, cudaStream_t stream);
// out[r, h, :] = gate[r, h] sum_j sigmoid(sum_g talk[h, g] s_g(j) + head_bias[h]) v_j over the keys j of the row's slot
// with 0 <= pos - j < window (window 0: all), s_g(j) = (q_g . k_j) scale - 2^(-slope_exp (g + 1) / H) (pos - j).  talk
// [H, H] (null: identity), head_bias [H] (null: zeros), gate [rows, H] (null: ones) are float32; slope_exp 0: no distance
// bias.  runs 1: a block a row; more: a block a (row, run of citlali_sigmoid_attention_run_keys() keys) into partial
// [rows, runs, H V] and a kernel that adds the runs; both give the same bits.
int citlali_sigmoid_attention_run_keys(void);
int citlali_sigmoid_attention(const void* q, int q_dtype, const void* k_pool, const void* v_pool, int cache_dtype,
                              const int32_t* page_table, int table_stride, const int32_t* row_slot, const int32_t* row_pos,
                              const float* talk, const float* head_bias, const float* gate, void* out, float* partial, int runs,
                              int rows, int H, int G, int D, int V, int page_size, int window, float scale, float slope_exp,
                              cudaStream_t stream);

// The same attention for runs of new tokens of `sequences` sequences (rows as citlali_attention_prefill takes them) on the
// tensor cores: bfloat16 q, pools and out, pages of 64.  One kernel writes every head's weights to `weights` (scratch of
// H * groups * columns * 8 bfloat16; columns and groups from the two functions below), a second one multiplies them with the
// values.  The weights are rounded to bfloat16 for that product; everything before is float32 on bfloat16 q and keys.
int citlali_sigmoid_attention_mma_supports(int H, int G, int D, int V, int page_size);
int citlali_sigmoid_attention_mma_columns(int window, int max_keys);
int citlali_sigmoid_attention_mma_groups(int rows, int sequences);
int citlali_sigmoid_attention_mma(const void* q, const void* k_pool, const void* v_pool, const int32_t* page_table,
                                  int table_stride, const int32_t* seq_start, const int32_t* seq_slot, const int32_t* seq_past,
                                  const float* talk, const float* head_bias, const float* gate, void* out, void* weights,
                                  int columns, int groups, int sequences, int max_new, int H, int G, int D, int V, int page_size,
                                  int window, float scale, float slope_exp, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
