// C interface of the native library: every entry point validates its arguments on the host,
// launches on the given stream, allocates nothing and returns 0 or a non-zero status whose
// text ftk_last_error() gives.  Pointers are device pointers unless said otherwise.
#pragma once
#include <stdint.h>

#define FTK_F32 0
#define FTK_BF16 1
#define FTK_ACT_SILU 0
#define FTK_ACT_SWIGLUOAI 1
#define FTK_SCORE_SIGMOID 0
#define FTK_SCORE_SOFTMAX 1
#define FTK_GATE_SIGMOID 0
#define FTK_GATE_SILU 1
// the bias belongs to the logit: choice by logit + bias, weights = softmax of logit + bias over the chosen experts
#define FTK_SCORE_SOFTMAX_OF_CHOSEN 2
#define FTK_SCORE_SIGMOID_RAW 3  // sigmoid scores, the chosen experts' scores as weights without renormalising

#ifdef __cplusplus
extern "C" {
#endif

// One destination of ftk_norm_rope_store: heads [first_head, first_head + n_heads) of every
// token, optionally normed and rotated, written densely or scattered into a paged slab.
typedef struct {
  int first_head;
  int n_heads;
  const float* norm_weight;  // [head_dim] or null
  int rotate;
  void* dense_out;           // [T, n_heads, head_dim] or null
  void* slab;                // [num_pages, n_heads, page_size, head_dim] or null
  const int32_t* slot_map;   // [T] slot = page * page_size + offset; negative skips the token
  int page_size;
  int num_pages;
  const float* bias;         // [n_heads * head_dim] added to the projected heads first, or null
  const float* pos_scale;    // [pos_scale_len] factor by the token's position, applied last, or null
  int pos_scale_len;
  int dst_head_dim;          // row length at the destination (>= head_dim; the rest is written as zeros); 0 = head_dim
} FtkSection;

// What ftk_stream_add_norm adds up and writes (see stream.cu).  Dense rows, routed rows and the table share `dtype`.
typedef struct {
  float* residual;           // [T, hidden] 32-bit stream; the sum is stored back unless `rows` is given
  const void* x1;            // [T, hidden] or null
  const void* x2;            // [T, hidden] or null
  const void* y;             // [n_routes, hidden] routed rows or null: row t gets sum_j y[route_pos[t * top_k + j]]
  const int32_t* route_pos;
  int top_k;
  int n_routes;
  const void* table;         // [vocab, hidden] or null: row t gets table[ids[t]]
  const int32_t* ids;
  int vocab;
  const float* vec;          // [hidden] added to every row, or null
  int norm;                  // 0: out = the sum (or no out at all), 1: out = tanh(alpha z) * weight + bias
  const float* weight;
  const float* bias;
  const float* alpha;        // one float on the device
  void* out;                 // [n_rows, hidden] or null
  int dtype;
  const int32_t* rows;       // null, or the rows to take (out[i] belongs to rows[i]; the stream stays as it is)
  int n_rows;
  int hidden;
} FtkStreamNorm;

// Options of ftk_paged_attention_ex beyond ftk_paged_attention's.
typedef struct {
  // learned bias by distance: score(i, j) += dist_bias[head * dist_len + min(i - j, dist_len - 1)], not
  // multiplied by `scale`; null = none
  const float* dist_bias;
  int dist_len;
  // more query heads per KV head than a tile has rows: every KV head is taken as kv_split heads of the same keys,
  // each with 1 / kv_split of its query heads (plan the work list, and size the scratch, for n_kv_heads * kv_split
  // heads); 0 or 1 = as given.  Not with the tcgen05 kernels.
  int kv_split;
  // a sink in the softmax's denominator: weight_j = e^(s_j) / (e^sink_logit + sum_i e^(s_i)); the sink has no value.
  // Of the tcgen05 kernels the one with 128-row tiles takes it; not with block selection.
  int has_sink;
  float sink_logit;
  // with has_sink: one logit per query head [n_q_heads] (float32) instead of sink_logit; null = sink_logit for all
  const float* sink_heads;
} FtkAttnExtras;

const char* ftk_last_error(void);

int ftk_embedding_gather(const void* table, int dtype, const int32_t* ids, int n_tokens, int hidden,
                         int vocab, float* out, void* stream);
int ftk_add_rmsnorm(const void* x, int x_dtype, float* residual, const float* weight, void* out,
                    int out_dtype, float* out_f32, const int32_t* rows, int n_rows, int hidden,
                    float eps, int gemma, void* stream);
// The same with the row that is added taken as a sum over routes: sum_j y[route_pos[row * top_k + j]]
// (+ shared[row]), rounded to y's type (what ftk_moe_combine would have written).
int ftk_add_rmsnorm_routes(const void* y, int y_dtype, const int32_t* route_pos, int top_k, int n_routes,
                           const void* shared, float* residual, const float* weight, void* out, int out_dtype,
                           float* out_f32, const int32_t* rows, int n_rows, int hidden, float eps, int gemma,
                           void* stream);
int ftk_stream_add_norm(const FtkStreamNorm* args, void* stream);
// o[t, h, :] *= sigmoid(gates[t * gate_stride + h]) in place; o [T, n_heads, head_dim]
int ftk_head_gate(void* o, int dtype, const void* gates, long long gate_stride, int n_tokens, int n_heads,
                  int head_dim, void* stream);
// ids[t, j] = table[token_ids[t], j], weights[t, j] = weight: experts picked by a table over token ids
int ftk_table_route(const int32_t* token_ids, const int32_t* table, int n_tokens, int vocab, int top_k,
                    int n_experts, float weight, int32_t* ids, float* weights, void* stream);
int ftk_scale_f32(float* x, long long n, float s, void* stream);
// x <- cap * tanh(x / cap)
int ftk_softcap_f32(float* x, long long n, float cap, void* stream);
// A sub-layer's output joins the stream through a norm of its own, and the stream is normed for the next
// sub-layer in the same pass: residual += rms(a) w_post; out = rms(residual) w_pre (w = 1 + weight with gemma).
// a = x[row] or, with route_pos, sum_j x[route_pos[row * top_k + j]] (+ shared[row]) in 32 bits.  Without pre_w
// only the stream is updated; with `rows` only those rows are normed and the stream is left as it is.
int ftk_postnorm_add_norm(const void* x, int dtype, const int32_t* route_pos, int top_k, int n_routes,
                          const void* shared, const float* post_w, float post_eps, int post_gemma, float* residual,
                          const float* pre_w, float pre_eps, int pre_gemma, void* out, float* out_f32,
                          const int32_t* rows, int n_rows, int hidden, void* stream);
// out[t, h, :dim] = norm(x[t, h, :dim]) * act(gates[t * gate_stride + h * dim + :]); the RMS norm over the head
// (plain weight norm_w [dim]) is left out when norm_w is null; act: FTK_GATE_SIGMOID | FTK_GATE_SILU.  x is
// float32 (x_f32) or of `dtype`, rows x_stride apart; out is of `dtype`, rows out_stride apart, and may be x.
int ftk_gated_heads(const void* x, int x_f32, int x_stride, const void* gates, long long gate_stride,
                    const float* norm_w, float eps, int act, void* out, int out_stride, int dtype, int n_tokens,
                    int n_heads, int dim, void* stream);
// Gated linear attention over a step's tokens (recurrent.cu): per (request, head) S <- diag(a_t) S + k_t v_t^T,
// o_t = S^T (q_t q_scale), a_t = sigmoid(z_t + z_bias)^(1 / tau); state [n_slots, H, dim, vdim] float32, zero for
// requests whose first tokens these are (kv_len == q_len in seg_info).  chunks [n_chunks, 4] = segment, first token
// within the segment, tokens, place among the segment's chunks (consecutive per segment); seg_chunks [n_segs, 2] =
// first chunk, chunks.  carry [n_chunks, H, dim, vdim] and decay_prod [n_chunks, H, dim] are scratch for segments
// of several chunks.  out [T, H, vdim] float32.  z [T, H * dim] float32 holds the decay logits and is overwritten
// (with the decays) when a segment has several chunks.  k_fac [T, H] (or null) multiplies a token's keys per head,
// in 32 bits; a_head [T, H] (or null) gives one decay per (token, head) in place of z; with ones_col = 1 the last of
// the vdim value columns is 1 for every token and v holds vdim - 1 columns per head; with out_ones [T, H] that
// column's outputs go there and out is [T, H, vdim - 1].
int ftk_gla_scan(const void* q, long long q_stride, const void* k, long long k_stride, const void* v,
                 long long v_stride, int dtype, float* z, const float* z_bias, float tau, float q_scale,
                 float* state, int n_slots, const int32_t* state_slots, const int32_t* seg_info, int n_segs,
                 const int32_t* chunks, int n_chunks, const int32_t* seg_chunks, int any_single, int any_multi,
                 float* carry, float* decay_prod, float* out, int n_tokens, int n_heads, int dim, int vdim,
                 const float* k_fac, const float* a_head, int ones_col, float* out_ones, int qk_div, void* stream);
// (qk_div > 1: head h reads the queries and keys of head h / qk_div, and q, k hold n_heads / qk_div heads; with a_head)

// One pass over S <= 8 residual streams (hyper.cu), streams [S][T, C] float32, stream_stride floats apart; each step
// optional, in this order: every stream = init_from [T, C]; x_t <- sum_s mix[s * S + t] x_s + out_w[t] y (y [T, C]
// of y_dtype); h_out [T, C] of h_dtype = unit(sum_s in_w[s] x_s) * norm_w (division by the root mean square, eps
// inside the root); sum_out [T, C] float32 = sum_s x_s.  All sums 32-bit.
int ftk_hyper_step(float* streams, long long stream_stride, int n_streams, int n_tokens, int channels,
                   const float* init_from, const void* y, int y_dtype, const float* mix, const float* out_w,
                   const float* in_w, const float* norm_w, float eps, void* h_out, int h_dtype, float* sum_out,
                   void* stream);
// out = (1 / n) sum_i unit(xs[i]) * ws[i]: n <= 4 inputs [T, C] of `dtype`, float32 weights [C] (hyper.cu).
// xs and ws are host arrays of four device pointers.
int ftk_norm_mean(const void* const* xs, const float* const* ws, int n, int dtype, float eps, void* out, int n_tokens,
                  int channels, void* stream);
// Causal convolution over time per channel on rows of `dtype` (x rows x_stride elements apart), optional bias and
// activation (0 none, 1 silu), per-request state of the last taps - 1 inputs as in ftk_short_conv (ssm.cu).
int ftk_conv_act(const void* x, long long x_stride, int dtype, const float* w, const float* bias, int taps, int act,
                 float* state, int n_slots, const int32_t* state_slots, const int32_t* seg_info, int n_segs, void* out,
                 int n_tokens, int channels, void* stream);
// dt_out = softplus(dt + dt_bias), decay_out = exp(-exp(a_log) * dt_out), [T, H] float32 (ssm.cu).
int ftk_ssm_gates(const void* dt, long long dt_stride, int dtype, const float* dt_bias, const float* a_log, float* dt_out,
                  float* decay_out, int n_tokens, int n_heads, void* stream);
// out [T, H * P] = groupnorm((o32 + d_skip[h] * x) * silu(z)) * norm_w: norm_groups equal parts of a row, each divided
// by its root mean square (ssm.cu).
int ftk_ssm_output(const float* o32, const void* x, long long x_stride, const float* d_skip, const void* z,
                   long long z_stride, int dtype, const float* norm_w, int norm_groups, float eps, void* out,
                   int n_tokens, int n_heads, int vdim, void* stream);
// Gated delta rule (delta.cu): per (segment, head) and token in order, S <- g S; u = beta (v - S^T k); S <- S + k u^T;
// o = S^T q, with beta = sigmoid(b), g = exp(-exp(a_log) softplus(a + dt_bias)), q and k made unit vectors per head
// (x / sqrt(sum x^2 + unit_eps), q then times q_scale).  q, k hold n_kv_heads heads of `dim`; state [n_slots, n_heads,
// vdim, dim] float32 (column by column); out [T, n_heads, vdim] float32.
int ftk_delta_scan(const void* q, long long q_stride, const void* k, long long k_stride, const void* v, long long v_stride,
                   const void* b, long long b_stride, const void* a, long long a_stride, int dtype, const float* a_log,
                   const float* dt_bias, float q_scale, float unit_eps, float* state, int n_slots,
                   const int32_t* state_slots, const int32_t* seg_info, int n_segs, float* out, int n_tokens,
                   int n_heads, int n_kv_heads, int dim, int vdim, void* stream);
// Short causal convolution over time with a residual (shortconv.cu): out[t, c] = x[t, c] + sum_j w[c, j] *
// in(t - taps + 1 + j, c) over the request's own inputs; the last taps - 1 inputs of every request live in its
// state slot (state [n_slots, taps - 1, channels] float32, oldest first; zeros before the sequence's start) and are
// replaced by this call.  x float32 (the stream), out of `dtype`.
int ftk_short_conv(const float* x, const float* w, int taps, float* state, int n_slots, const int32_t* state_slots,
                   const int32_t* seg_info, int n_segs, void* out, int dtype, int n_tokens, int channels, void* stream);
// hist[n_prev] = x; x = sum_{j <= n_prev} mix[j] * hist[j] (rows of n floats, layer_stride apart; all float32).
int ftk_depth_mix(float* hist, long long layer_stride, int n_prev, const float* mix, float* x, long long n, void* stream);
// out[r, :] = weights[sorted_routes[r]] * h[sorted_routes[r] / top_k, :]: expert inputs scaled by the route's weight.
int ftk_moe_gather_scaled(const void* h, int dtype, const int32_t* sorted_routes, const float* weights, int n_routes,
                          int top_k, int hidden, void* out, void* stream);
// x <- max(x, 0)^2 in place.
int ftk_relu2(void* x, int dtype, long long n, void* stream);
// Latent attention (latent.cu).  proj rows hold [query latent q_rank | key/value latent kv_rank | rotated key part
// rot_dim]; cq_out [T, q_rank] gets the normed query latent, the token's cache row slab[slot_map[t]] (pad_dim wide)
// [normed latent | rotated part | zeros].  n_rot leading dimensions of the part turn (pairs (2i, 2i+1) when
// interleaved, else (i, i + n_rot/2)); table [max_pos, n_rot] = cos || sin.
int ftk_latent_store(const void* proj, int dtype, long long row_stride, int q_rank, int kv_rank, int rot_dim, int n_rot,
                     int interleaved, const float* wq, const float* wkv, float eps, const int32_t* positions,
                     const float* table, int max_pos, void* cq_out, void* slab, long long slab_rows,
                     const int32_t* slot_map, int pad_dim, int n_tokens, void* stream);
// q [T, heads, flat_dim + rot_dim]: every head's rotated part goes, turned, to q_out[t, head, kv_rank : kv_rank + rot_dim]
// (q_out [T, heads, pad_dim]; zeros behind it).
int ftk_latent_query_rotate(const void* q, int dtype, int n_heads, int flat_dim, int rot_dim, int n_rot, int interleaved,
                            const int32_t* positions, const float* table, int max_pos, void* q_out, int kv_rank,
                            int pad_dim, int n_tokens, void* stream);
// Matrix memory with exponential gates (mlstm.cu): see the file's header.  pre [T, 2 * heads] float32 = input gate
// then forget gate before bias and cap; m_state [n_slots, heads]; key_fac = e^(input gate), decay = e^(forget gate)
// and m_out, all [T, heads].
int ftk_mlstm_gates(const float* pre, const float* bias_i, const float* bias_f, float cap, float* m_state, int n_slots,
                    const int32_t* state_slots, const int32_t* seg_info, int n_segs, int n_heads, int n_tokens,
                    float* key_fac, float* decay, float* m_out, void* stream);
// o32 [T, heads, vdim], nq [T, heads] (n . q); out [T, heads * vdim] of `dtype`.
int ftk_mlstm_output(const float* o32, const float* nq, const float* m, const void* gates, long long gate_stride, const float* norm_w,
                     float eps, void* out, int dtype, int n_tokens, int n_heads, int vdim, void* stream);
int ftk_act_and_mul(const void* gate_up, int dtype, int n_rows, int inter, int act, float alpha,
                    float limit, void* out, void* stream);
int ftk_cast(const void* src, int src_dtype, void* dst, int dst_dtype, long long n, void* stream);
int ftk_table_update(int32_t* table, long long table_len, const int32_t* updates, int n_updates,
                     void* stream);
int ftk_copy_tokens(int32_t* dst, int dst_len, const int32_t* pairs, const int32_t* src, int src_len, int n,
                    int vocab, void* stream);
int ftk_norm_rope_store(const void* x, int dtype, int n_tokens, int row_elems, int head_dim,
                        int rotary_dim, const int32_t* positions, const float* rope_table, int max_pos,
                        float eps, int gemma, int n_sections, const FtkSection* sections, void* stream);
int ftk_paged_attention(const void* q, const void* k_slab, const void* v_slab, int dtype,
                        const int32_t* block_table, int bt_stride, const int32_t* seg_info, int n_segs,
                        const int32_t* items, int n_items, float* part_o, float* part_ml, int n_slots,
                        void* out, int n_q_heads, int n_kv_heads, int head_dim, int page_size,
                        int num_pages, int tile_rows, float scale, int window, void* stream);
// The same with options (`extras` may be null).  k_slab == v_slab is allowed (values that are the keys): the
// kernels then bring each key tile in once.
int ftk_paged_attention_ex(const void* q, const void* k_slab, const void* v_slab, int dtype,
                           const int32_t* block_table, int bt_stride, const int32_t* seg_info, int n_segs,
                           const int32_t* items, int n_items, float* part_o, float* part_ml, int n_slots,
                           void* out, int n_q_heads, int n_kv_heads, int head_dim, int page_size,
                           int num_pages, int tile_rows, float scale, int window, const FtkAttnExtras* extras,
                           void* stream);
// Long steps in bfloat16 on tcgen05: tiles of 128 query rows (plan the items with tile_rows = 128), head
// size 128, pages of a multiple of 16 tokens; n_tokens = rows of q.  ftk_attention_tc_fits says whether
// the sizes are taken.
int ftk_attention_tc_fits(int head_dim, int page_size, int group);
int ftk_paged_attention_tc(const void* q, const void* k_slab, const void* v_slab, const int32_t* block_table,
                           int bt_stride, const int32_t* seg_info, int n_segs, const int32_t* items, int n_items,
                           float* part_o, float* part_ml, int n_slots, void* out, int n_tokens, int n_q_heads,
                           int n_kv_heads, int head_dim, int page_size, int num_pages, float scale, int window,
                           void* stream);
// The 128-row form, or with few_rows the form for tiles of at most 16 rows, with options (a distance bias).  In both
// forms k_slab == v_slab (values that are the keys) makes the key tile in shared memory serve both products.
int ftk_paged_attention_tc_ex(const void* q, const void* k_slab, const void* v_slab, const int32_t* block_table,
                              int bt_stride, const int32_t* seg_info, int n_segs, const int32_t* items, int n_items,
                              float* part_o, float* part_ml, int n_slots, void* out, int n_tokens, int n_q_heads,
                              int n_kv_heads, int head_dim, int page_size, int num_pages, float scale, int window,
                              const FtkAttnExtras* extras, int few_rows, void* stream);
// Decode steps in bfloat16 on the same kernel with tiles of at most 16 query rows (plan the items with
// tile_rows = 16 and key pieces that are multiples of 128; at most 16 query heads per KV head): one
// warp takes the softmax of the tile's rows.  part_o [slots, Hkv, 16, 128], part_ml [slots, Hkv, 16, 2].
int ftk_attention_tc_few_fits(int head_dim, int page_size, int group);
int ftk_paged_attention_tc_few(const void* q, const void* k_slab, const void* v_slab, const int32_t* block_table,
                               int bt_stride, const int32_t* seg_info, int n_segs, const int32_t* items, int n_items,
                               float* part_o, float* part_ml, int n_slots, void* out, int n_tokens, int n_q_heads,
                               int n_kv_heads, int head_dim, int page_size, int num_pages, float scale, int window,
                               void* stream);
int ftk_paged_attention_sparse(const void* q, const void* k_slab, const void* v_slab, int dtype,
                               const int32_t* block_table, int bt_stride, const int32_t* seg_info, int n_segs,
                               const int32_t* items, int n_items, float* part_o, float* part_ml, int n_slots,
                               void* out, int n_q_heads, int n_kv_heads, int head_dim, int page_size,
                               int num_pages, int tile_rows, float scale, const int32_t* sel, int sel_stride,
                               int block_size, void* stream);
int ftk_sparse_select(const void* iq, const void* ik_slab, int dtype, const int32_t* block_table, int bt_stride,
                      const int32_t* seg_info, int n_segs, int n_tokens, int n_heads, int dim, int page_size,
                      int num_pages, int block_size, int topk, int local_blocks, int init_blocks, int max_blocks,
                      int live_blocks, int32_t* sel, float* scores, void* stream);
// Whether bfloat16 block scores of these sizes can be taken on the tensor cores (`scores [T, n_heads, max_blocks]`
// float32 scratch must then be given to ftk_sparse_select).
int ftk_sparse_score_fits(int n_heads, int dim, int block_size);
int ftk_router_topk(const float* logits, int n_parts, const float* bias, int n_tokens, int n_experts, int top_k,
                    int scoring, float scale, int32_t* ids, float* weights, void* stream);
// Router logits (float32 x [T, hidden] times gate_w [E, hidden]), choice and sort of the routes in one
// launch, for steps of at most 32 tokens (beyond that the
// separate kernels are faster); ftk_moe_route_fits says whether the sizes are taken.
int ftk_moe_route_fits(int n_tokens, int hidden, int n_experts, int top_k);
int ftk_moe_route(const float* x, const float* gate_w, const float* bias, int n_tokens, int hidden, int n_experts,
                  int top_k, int scoring, float scale, float* logits, int32_t* ids, float* weights,
                  int32_t* counts, int32_t* offsets, int32_t* routes, int32_t* pos, int do_sort, void* stream);
// Products of very few tokens (bfloat16): the weights are streamed once by warps of every SM (gemv.cu).
int ftk_small_linear_fits(int n_tokens, int n_out, int k);
int ftk_small_linear(const void* x, const void* w, void* out, int n_tokens, int n_out, int k, void* stream);
int ftk_moe_small_fits(int n_tokens, int hidden, int inter, int top_k);
int ftk_moe_small_gate_up(const void* h, const int32_t* ids, const void* w1, void* a, int n_tokens, int top_k,
                          int n_experts, int hidden, int inter, int act, float alpha, float limit, void* stream);
int ftk_moe_small_down(const void* a, const int32_t* ids, const float* weights, const void* w2, void* y, int n_tokens,
                       int top_k, int n_experts, int hidden, int inter, void* stream);
int ftk_moe_permute(const int32_t* topk_ids, int n_tokens, int top_k, int n_experts,
                    int32_t* expert_counts, int32_t* expert_offsets, int32_t* sorted_routes,
                    int32_t* route_pos, void* stream);
int ftk_moe_gather(const void* h, int dtype, const int32_t* sorted_routes, int n_routes, int top_k,
                   int hidden, void* out, void* stream);
int ftk_moe_gemm1_act(const void* x_sorted, const void* w1, int dtype, const int32_t* expert_offsets,
                      int n_experts, int n_routes, int hidden, int inter, int act, float alpha,
                      float limit, void* out, void* stream);
// The same from the tokens' rows x [n_tokens, hidden] in their own order (bfloat16, tensor cores): row r of
// expert order is the row of token sorted_routes[r] / top_k, gathered by the kernel (steps whose token tiles have
// at most 32 rows: ask ftk_moe_gemm1_gather_fits).
int ftk_moe_gemm1_gather_fits(int hidden, int inter, int n_experts, int n_routes);
int ftk_moe_gemm1_act_gather(const void* x, const void* w1, const int32_t* expert_offsets, const int32_t* sorted_routes,
                             int top_k, int n_tokens, int n_experts, int n_routes, int hidden, int inter, int act,
                             float alpha, float limit, void* out, void* stream);
int ftk_moe_gemm2(const void* a, const void* w2, int dtype, const int32_t* expert_offsets,
                  const int32_t* sorted_routes, const float* topk_weights, int n_experts, int n_routes,
                  int hidden, int inter, void* out, void* stream);
int ftk_moe_combine(const void* y, int dtype, const int32_t* route_pos, int n_tokens, int top_k,
                    int hidden, const void* shared, void* out, void* stream);
// Status words of the kernels' bounded waits: out[0] = first code since the last call (0 = none),
// out[1] = block that recorded it.  Synchronises with the device and clears the words.
// Kernel forms launched so far, as "name<TAB>count" lines (see ftk::note_variant); returns the bytes needed.
int ftk_variant_counts(char* buf, int cap, int reset);
int ftk_read_status(int* out);
// Writes `code` into a status word from the host (unit 0: grouped GEMM, 1: attention), so that a caller's
// handling of a given-up wait can be tested without any wait running out on the device.
int ftk_debug_set_status(int unit, int code);
// 0 sends bfloat16 grouped expert products to the CUDA-core kernels; default 1 (tcgen05).
int ftk_set_moe_tensor_cores(int enabled);
int ftk_set_moe_pairs(int enabled);
int ftk_sample(const float* logits, int n_rows, int vocab, const float* temperature,
               const int32_t* top_k, const float* top_p, const float* u, int32_t* out, void* stream);

#ifdef __cplusplus
}
#endif
