// stack.h -- layer-list decoders: a model given as a list of layers, each with one token mixer (linear attention with a
// fixed decay, a minimal gated recurrence, or latent attention over a compressed KV cache) and an optional
// feed-forward (dense or mixture of experts).  The engine's sequences, page allocator, step planner, sampler and C ABI
// are shared with the Llama path; this header holds what differs: the per-layer weights, the per-slot recurrent state,
// the latent page pools and the launchers of k_stack.cu.
#pragma once
#include <map>
#include <string>
#include <vector>

#include "../../include/dis_engine.h"
#include "common.cuh"

namespace dis {

// ---- k_stack.cu launchers.  `f32` selects the element type of activations and matrices: true = float, false = bf16
// bit patterns.  Norms, routers, scores, recurrent state and the residual are fp32 in both.
struct StackGemm {
  const void *A = nullptr;      // [M][K] activations: float when a_f32, else bf16
  const void *W = nullptr;      // [N][K] weights: float when w_f32, else bf16; applied as A W^T
  float *out = nullptr;         // [M][N] fp32
  const float *bias = nullptr;  // [N] or null
  int M = 0, N = 0, K = 0;
  long long lda = 0, ldw = 0, ldo = 0;
  bool a_f32 = true, w_f32 = true;
  // batch (blockIdx.z): element offsets added per batch index
  int batch = 1;
  long long a_bs = 0, w_bs = 0, o_bs = 0, bias_bs = 0;
  // grouped rows (mixture of experts): tiles[0] = number of row tiles, then {group, row0, rows} per tile; the group
  // selects the weight block (w_bs) -- M is then the capacity of the row space and max_tiles the grid's extent
  const int *tiles = nullptr;
  int max_tiles = 0;
  const int *a_gather = nullptr;  // row r of the row space reads A row a_gather[r]
  // a_glu > 0 (few-rows kernel only, A float): A is [M][2K] gate | up and the product's input is the gated unit (dis_mlp_act
  // a_glu - 1, clamp a_limit) of each pair, rounded to bf16 when W is bf16 -- the gated-unit kernel folded into the loader
  int a_glu = 0;
  float a_limit = 0.f;
};
cudaError_t launch_stack_gemm(const StackGemm &g, cudaStream_t st);
bool stack_gemm_few_rows(const StackGemm &g);  // launch_stack_gemm would take the few-rows kernel

struct StackSpans {  // device arrays of the pass
  const uint32_t *tokens;  // [T]
  const int *pos;          // [T] position of the token in its sequence
  const int *slot;         // [T] sequence slot
  const int *span;         // [T] index of the token's span
  const int *sp_tok0, *sp_len, *sp_pos0, *sp_slot;  // [n_spans]
  int T, n_spans;
};

// x = embed[token] * scale (+ a sinusoidal position vector when pos_freq, a table of W/2 frequencies, is given), written to each
// of the token's `streams` residual streams ([T][streams][W]); x0 (when given) receives the same rows once
cudaError_t launch_stack_embed(const void *embed, bool f32, const uint32_t *tokens, const int *pos, const double *pos_freq, float *x,
                               float *x0, float scale, int T, int W, int streams, cudaStream_t st);
// Pre-norm boundary over `streams` residual streams xs [T][streams][W]: the product before (y, as slices + bias) joins every
// stream through the coefficients `prev` of its sublayer (in | out | mix; null: x += y), then the coming sublayer's input
// u = sum_s next[s] x_s (null: x_0) is RMS-normed with the gain vector pre_w into hc (pre_w null: only the streams move on).
cudaError_t launch_stack_boundary_hc(float *xs, int streams, const float *y, int n_part, long long stride, const float *bias,
                                     const float *prev, const float *next, const float *pre_w, void *hc, bool f32, int T, int W, float eps,
                                     cudaStream_t st);
// x += unit_rms(y) * post (when y), then hn = unit_rms(x) * pre (when hn).  post / pre: device scalars.
cudaError_t launch_stack_resid_norm(float *x, const float *y, const float *post, const float *pre, float *hn, int T, int W,
                                    float eps, cudaStream_t st);
// hc = hn + causal depthwise convolution over time (taps >= 1), reading the taps-1 inputs before a span from `state`
// ([slots][taps-1][W]); then the state is replaced by the span's last taps-1 inputs (second launch inside).
cudaError_t launch_stack_canon(const float *hn, const float *w, float *state, const StackSpans &sp, void *hc, bool f32, int W,
                               int taps, cudaStream_t st);
// Passes of single tokens: residual update (y given as n_part slices + bias), both norms, convolution and tail update in one kernel
cudaError_t launch_stack_boundary_single(float *x, const float *y, int n_part, long long stride, const float *bias, const float *post,
                                         const float *pre, const float *cw, float *cstate, const StackSpans &sp, void *hc, bool f32,
                                         int W, int taps, float eps, cudaStream_t st);
// The same boundary with layer norms (weight and bias vectors) in place of the scalar-gain RMS norms: y = bias + the n_part
// slices; x += LN(y; post); cat (when given) = [x ; x0] in the compute type; LN(x; pre) -> hn (fp32, when given) and hc
// (compute type, when given).  post / pre null: that step is left out.
cudaError_t launch_stack_boundary_ln(float *x, const float *y, int n_part, long long stride, const float *bias, const float *post_w,
                                     const float *post_b, const float *pre_w, const float *pre_b, float *hn, void *hc, const float *x0,
                                     void *cat, bool f32, int T, int W, float eps, bool rms, cudaStream_t st);
// rms: both norms are v / sqrt(mean(v^2) + eps) * w (gain vectors, no mean taken off, no bias vectors)
// out = LN(x[row_map[r]]) * scale: a factor on the logits is applied to the head's input (head (s v) = s (head v)).
// b == null: the RMS form with the gain vector w
// streams > 1: the row is the sum of the token's residual streams (x is [T][streams][W])
cudaError_t launch_stack_final_ln(const float *x, const int *row_map, const float *w, const float *b, void *out, bool f32, int R, int W,
                                  float eps, float scale, int streams, cudaStream_t st);
cudaError_t launch_stack_scale(float *v, long long n, float s, cudaStream_t st);
// v = cap * tanh(v / cap)
cudaError_t launch_stack_softcap(float *v, long long n, float cap, cudaStream_t st);
cudaError_t launch_stack_copy_act(const float *hn, void *hc, bool f32, long long n, cudaStream_t st);
// proj [T][ld]: q at 0, k at H*d, v at 2*H*d (pre-activation).  state [slots][H][d][dv].  o [T][H*dv] fp32.
// seg (or null): room for stack_lightning_seg_floats() floats -- spans longer than stack_lightning_seg_tokens() (max_len: the
// longest span of the pass) are then cut into segments that run side by side, with a carry pass between them.
size_t stack_lightning_seg_floats(int cap_tokens, int max_spans, int H, int d, int dv);
int stack_lightning_seg_tokens();
// whether a pass of n_spans spans (T tokens, the longest max_len) over H heads is faster cut into segments than span by span
bool stack_lightning_segmented(int n_spans, int T, int H, int max_len);
cudaError_t launch_stack_lightning(const float *proj, long long ld, const float *decay, float *state, const StackSpans &sp,
                                   float *o, int H, int d, int dv, float *seg, int max_len, cudaStream_t st);
// Gated linear attention (per-channel decay): S = diag(a_t) S + k_t v_t^T, o_t = S^T (q_t / sqrt(d)).
// decays: dec[t][c] = sigmoid(z)^(1/tau), z = b[c] + sum_r a2[c][r] * proj[t][a_off + r]; n = H*d channels.
cudaError_t launch_stack_gla_decay(const float *proj, long long ld, int a_off, const void *a2, bool w_f32, const float *b, int T, int n,
                                   int rank, float tau, float *dec, cudaStream_t st);
// proj [T][ld] with q, k [H][d] and v [H][dv] at the given columns; dec [T][H*d]; state [slots][H][d][dv]; o [T][H*dv] fp32.
// seg / seg_a: as for lightning, plus room for stack_lightning_seg_decay_floats() floats (the segments' decay products).
size_t stack_lightning_seg_decay_floats(int cap_tokens, int max_spans, int H, int d);
cudaError_t launch_stack_gla(const float *proj, long long ld, int q_off, int k_off, int v_off, const float *dec, float *state,
                             const StackSpans &sp, float *o, int H, int d, int dv, float *seg, float *seg_a, int max_len,
                             cudaStream_t st);
// State-space mixer (DIS_MIX_SSM), three steps around the recurrence kernel of gated linear attention.
// 1. proj [T][ld] holds z | x | B | C | dt as projected.  The C = inner + 2 G N channels from x_off on pass a causal depthwise
//    convolution over time (cw [C][taps], last tap = the current token; the taps - 1 inputs before a span come from cstate
//    [slots][taps-1][C], zeros before position 0) plus cb, then SiLU -> buf [T][ld_b] (x | B | C).  dt = softplus(proj[dt_off + h]
//    + vec[h]) (vec = dt_bias | A_log | D, [3H]) -> dtv [T][H]; dec [T][H] receives the decays exp(-exp(A_log[h]) dt).  cstate
//    moves on to the span's last inputs: inside the same launch when every span is one token, else by a second one.
cudaError_t launch_stack_ssm_conv(const float *proj, long long ld, int x_off, int dt_off, int C, int H, int taps, const float *cw,
                                  const float *cb, const float *vec, float *cstate, const StackSpans &sp, float *buf, long long ld_b,
                                  float *dec, float *dtv, cudaStream_t st);
// 2. S [N][P] per head: S = dec[t][h] S + B_t (dt[t][h] x_t)^T, o_t = S^T C_t.  buf as above (B at b_off, C at c_off, x at v_off;
//    head h reads the B, C of group h / hpg); state [slots][H][N][P]; o [T][H*P]; seg / seg_a as for gated linear attention.
cudaError_t launch_stack_ssd(const float *buf, long long ld_b, int c_off, int b_off, int v_off, int hpg, const float *dec,
                             const float *dt, float *state, const StackSpans &sp, float *o, int H, int N, int P, float *seg, float *seg_a,
                             int max_len, cudaStream_t st);
// 3. y = (o + D[h] x) silu(z), RMS-normed in `parts` equal parts of H*P (each by its own mean square), times w -> out [T][H*P] in
//    the compute type.  x: buf column 0 on (row stride ld_b), z: proj column 0 on (row stride ld).
cudaError_t launch_stack_ssm_out(const float *o, const float *buf, long long ld_b, const float *z, long long ld, const float *D,
                                 const float *w, int parts, void *out, bool f32, int T, int H, int P, float eps, cudaStream_t st);
// out[t][off + h*dv + j] = scale * unit_rms_over_head(o[t][h])[j] * w[j] * silu(gate[t][h*dv + j]); out [T][ldo] compute type
cudaError_t launch_stack_headnorm_silu(const float *o, const float *w, const float *gate, long long ldg, void *out, long long ldo,
                                       int off, float scale, bool f32, int T, int H, int dv, float eps, cudaStream_t st);
// Attention over paged keys and values (k_stack_attn.cu).
struct StackAttn {
  int H, G, d, dv, rot_dims;
  unsigned flags;  // DIS_ATTN_*
  float scale, eps;
  int chunk;       // > 0: position i sees only keys from floor(i / chunk) * chunk on
  int window = 0;  // > 0: position i sees only the keys j with i - j < window
  float softcap = 0.f;  // > 0: score <- softcap * tanh(score / softcap), after the factor `scale` (softmax weights only)
};
// first key position the query at position `pos` may see (both masks are monotone in pos, so a block of consecutive queries
// starts its walk at the bound of its first token)
__host__ __device__ inline int stack_attn_row_lo(const StackAttn &c, int pos) {
  int lo = c.chunk > 0 ? pos / c.chunk * c.chunk : 0;
  if (c.window > 0 && pos - c.window + 1 > lo) lo = pos - c.window + 1;
  return lo;
}
// Per token: (bias, one entry per column of proj), query/key norm over the whole projection (gains qn [H*d], kn [G*d]) or per
// head (DIS_ATTN_QK_NORM_HEAD: gains [d] shared by the heads), rotation of the first rot_dims coordinates of every head by
// pos * freq[i] (pairs i, i + rot_dims/2); queries to qf [T][H*d]; rotated keys and the values (own projection at v_off, or the
// unrotated keys; rotated by pos * vfreq[m] over pairs m, m + dv/2 with DIS_ATTN_ROT_V) to the token's row of the pools
// ([pages*page_size][G*d] and [..][G*dv]); vrot [T][dv] receives cos | sin of the value angles for the output's rotation back.
// kpool == null: the layer reads another layer's cache -- only the queries are prepared.
// n_part > 1: proj holds split-K slices (slice stride `stride`) of n_cols columns, summed here with the bias.  gate_out (or
// null): [T][ld_gate] receives columns gate_off .. + H of every row (the logits of the output gates).
cudaError_t launch_stack_attn_prep(const float *proj, long long ld, int n_part, long long stride, int n_cols, int gate_off, float *gate_out,
                                   long long ld_gate, int q_off, int k_off, int v_off, const float *bias, const float *qn,
                                   const float *kn, const double *freq, const double *vfreq, const StackAttn &c, const StackSpans &sp,
                                   float *qf, void *kpool, void *vpool, float *vrot, bool f32, const int *page_table, int max_pages,
                                   int page_size, cudaStream_t st);
// query blocks hold at most stack_attn_block_tokens() tokens of one span (bq: the most tokens a block of this pass holds); n_split > 1: slices of keys_per_split keys (a multiple
// of 32), records of dv + 2 floats per (slice, token, head) in `part`, merged by a second kernel.  The result, times out_scale
// and rotated back when values were rotated, lands in out [T][ld_out] (compute type) at columns out_off + h * dv.
// bf16 with dim % 8 == 0, vdim % 16 == 0, both <= 128 and at most 64 query heads per key/value head: the mma.sync kernel (blocks
// of 64 (token, head) rows); otherwise the fp32-arithmetic kernel.
// sink [H] (DIS_ATTN_SINK): per-head logit in the softmax denominator.  gate [T][ld_gate] (DIS_ATTN_GATE): head h's output is
// multiplied by sigmoid(gate[t][h]).  With c.chunk > 0 a block's history starts at the chunk of its first token, and the slices
// are counted from there.
int stack_attn_block_tokens(const StackAttn &c, bool f32);
cudaError_t launch_stack_attn(const float *qf, const void *kpool, const void *vpool, bool f32, const float *temp, const float *pb,
                              const float *sink, const StackAttn &c, const StackSpans &sp, const int *qb_tok0, const int *qb_len, int n_qb,
                              int bq, const int *page_table, int max_pages, int page_size, void *out, long long ld_out, int out_off,
                              float out_scale, const float *vrot, const float *gate, long long ld_gate, int n_split,
                              int keys_per_split, float *part, cudaStream_t st);
// out = unit_rms(o) * w * sigmoid(gate) per token over n = H*dv coordinates; gate [T][ldg]
cudaError_t launch_stack_norm_gate(const float *o, const float *w, const float *gate, long long ldg, void *out, bool f32, int T,
                                   int n, float eps, cudaStream_t st);
// out = o * sigmoid(gate); heads > 0: o is [heads][T][n / heads] instead of [T][n]
cudaError_t launch_stack_gate(const float *o, const float *gate, long long ldg, void *out, bool f32, int T, int n, int heads,
                              cudaStream_t st);
// head h of src [T][ld] (columns off + h * hs .. + wd) -> dst bf16 [H][T][wd], and fp32 [H][T][wd] back into such columns
cudaError_t launch_stack_heads_pack(const float *src, long long ld, int off, int hs, int wd, int T, int H, uint16_t *dst, cudaStream_t st);
cudaError_t launch_stack_heads_unpack(const float *src, int wd, int T, int H, float *dst, long long ld, int off, int hs, cudaStream_t st);
// proj [T][ld]: z at 0, u at n, g at 2n (biases already added).  state [slots][n].
// max_len: the longest span of the pass (long spans are cut into time slices that run side by side)
// bias (or null): [3n], added to proj here when the product that made proj left it out
cudaError_t launch_stack_mingru(const float *proj, long long ld, const float *bias, float *state, const StackSpans &sp, void *out,
                                bool f32, int n, int max_len, cudaStream_t st);
// Latent attention, step 1: per token, the rotated query parts go to qf[T][H][r+dr] (+r), and -- when pool is given --
// the normed latent and the rotated shared key part go to the token's row of the page pool ([pages*page_size][r+dr]).
struct StackLatent {
  int H, d, dr, dv, r, rot_dims;
  float rot_base, scale, eps;
};
cudaError_t launch_stack_latent_prep(const float *proj, long long ld, int q_off, int dkv_off, const float *dkv_norm,
                                     const StackLatent &c, const StackSpans &sp, float *qf, void *pool, bool f32,
                                     const int *page_table, int max_pages, int page_size, cudaStream_t st);
// step 2: scores of qf against the pool rows of the sequence (causal, softmax with a per-head sink in the denominator),
// output the weighted sum of the latents: ol [T][H][r] fp32.  qb_tok0 / qb_len: query blocks (tokens of one span).
// n_split > 1: the history is cut into slices of keys_per_split keys (a multiple of 32), one CTA per (block, slice), whose
// records ([n_split][T*H][r+2] floats in `part`) a second kernel merges -- few query blocks then still fill the GPU.
int stack_latent_block_tokens(const StackLatent &c);
// the mma.sync form of the kernel applies (bf16, kv_rank % 8 == 0, (kv_rank + rot_dim) % 16 == 0, heads <= 16): query blocks
// then hold at most 16 (token, head) pairs
bool stack_latent_mma_ok(const StackLatent &c, bool f32);
cudaError_t launch_stack_latent_attn(const float *qf, const void *pool, bool f32, const float *sink, const StackLatent &c,
                                     const StackSpans &sp, const int *qb_tok0, const int *qb_len, int n_qb,
                                     const int *page_table, int max_pages, int page_size, float *ol, int n_split,
                                     int keys_per_split, float *part, cudaStream_t st);
// Long prompt portions in bf16: latents of one sequence out of their pages into cg [ctx8][D] and cgt [r][ctx8] (rows / columns
// from ctx to ctx8 zero), and softmax weights (bf16) from a block of raw score rows; the products between run on tcgen05.
cudaError_t launch_stack_latent_gather(const void *pool, const int *pt_row, int page_size, int D, int r, int ctx, int ctx8,
                                       uint16_t *cg, uint16_t *cgt, cudaStream_t st);
cudaError_t launch_stack_latent_softmax(const float *S, int rows, int ld, const float *sink, int H, int pos_first, float scale,
                                        uint16_t *P, cudaStream_t st);
// kind DIS_ACT_CLAMPED: act = g' sigmoid(1.702 g') (u' + 1), g' = min(g, limit), u' = clamp(u, -limit, limit);
// DIS_ACT_GELU_TANH: act = gelu_tanh(g) u; DIS_ACT_SILU: act = g sigmoid(g) u.  gu [M][2*ff] (gate | up)
// gu may come as n_part split-K slices (slice stride `stride`), summed here; bias (or null): [2*ff], added here when the product
// that made gu left it out
cudaError_t launch_stack_glu(const float *gu, int n_part, long long stride, const float *bias, void *act, bool f32, const int *rows_ptr,
                             int M, int ff, float limit, int kind, cudaStream_t st);
// Router: logits in fp32 from hc and the fp32 router matrix; `top` experts by value (lowest index wins a tie).
// kind DIS_ROUTE_SOFTMAX_TOP: by logit, weights = softmax over the chosen.  DIS_ROUTE_SIGMOID_GROUPS: by c = sigmoid(logit) +
// correction[e], restricted to the `keep` best of `groups` contiguous runs of experts (a run ranks by the sum of its top two c;
// groups <= 1: no restriction), weights = the chosen sigmoids over their sum (+ 1e-20).
// extra (or null): one more fp32 row [W]; its product with every token goes to extra_out [T].
cudaError_t launch_stack_route(const void *hc, bool f32, const float *router, int T, int W, int E, int top, int kind,
                               const float *correction, int groups, int keep, const float *extra, float *extra_out, int *idx, float *wt,
                               cudaStream_t st);
// Row plan of the experts: counts / cursor [E] ints (zeroed inside), perm_tok [T*top], where [T*top] (row of (t, k)),
// tiles [1 + 3 * max_tiles], rows_total[1]
cudaError_t launch_stack_moe_plan(const int *idx, int T, int top, int E, int tile_rows, int *counts, int *perm_tok, int *where,
                                  int *tiles, int max_tiles, cudaStream_t st);
cudaError_t launch_stack_moe_gather(const void *hc, const int *perm_tok, void *xs, int rows, int W, cudaStream_t st);
// y[t] = sum_k wt[t][k] * rows[where[t][k]] (+ sigmoid(shared_gate[t]) * shared[t] when shared is given; shared may come as
// n_part split-K slices of stride `stride`, summed here)
cudaError_t launch_stack_moe_combine(const float *rows, const int *where, const float *wt, const float *shared, int n_part,
                                     long long stride, const float *shared_gate, float *y, int T, int W, int top, cudaStream_t st);
cudaError_t launch_stack_final_norm(const float *x, const int *row_map, const float *g, void *out, bool f32, int R, int W, float eps,
                                    cudaStream_t st);
// out[m][n] = bias[n] + sum_s part[s][m][n]: the split-K slices of a tensor-core product, with the projection's bias
cudaError_t launch_stack_sum_bias(const float *part, int n_part, long long stride, const float *bias, float *out, int M, int N,
                                  cudaStream_t st);
constexpr int kStackGemmTile = 64;

// ---- the model
struct StackTensor {
  void *ptr = nullptr;
  size_t n = 0;
  bool f32 = true;
  std::vector<int64_t> shape;
  bool loaded = false;
};

struct StackLayer {
  dis_layer_config c{};
  std::vector<float> decay;
  // mixer
  StackTensor w_in;     // fused input projection rows (see stack.cu for the row order per mixer)
  StackTensor b_in;     // its bias (fp32) or empty
  StackTensor w_o;      // output projection
  StackTensor norm_w;   // lightning: gain of the head norm; latent: gain of the latent norm (fp32)
  StackTensor ukT;      // latent: per head [r][d] = transpose of the head's block of the key up-projection
  StackTensor uv;       // latent: [H*dv][r]
  StackTensor sink;     // latent, attention with DIS_ATTN_SINK: [H] fp32
  StackTensor decay_d;  // lightning: [H] fp32
  int n_in = 0, q_off = 0, dkv_off = 0, g_off = 0;
  float *canon1 = nullptr, *canon2 = nullptr;        // [W][taps] fp32
  float *g4 = nullptr;  // device: norm1, norm1b, norm2, norm2b (scalar gains)
  StackTensor ln_w[4], ln_b[4];  // the same four norms as layer norms: weight and bias vectors [W] fp32
  // attention (alone, or the first half of a parallel mixer): w_in rows q | k | v; qf columns follow the same order
  int k_off = 0, v_off = 0;
  StackTensor qk_norm;   // [H*d + G*d] fp32: gains of the whole-projection query and key norms; per-head norms: [d + d]
  StackTensor temp_pb;   // [2H] fp32: per-head factor on the score, then per-head bias under the sigmoid
  StackTensor b_o;       // [W] fp32: bias of the output projection
  double *freq = nullptr, *vfreq = nullptr;  // device: rotary frequencies [rot_dims/2] (scaled) and value frequencies [vdim/2]
  int n_act = 0;         // columns of the output projection's input: H*vdim (+ gla_heads*gla_vdim behind them)
  // gated linear attention (second half of a parallel mixer): w_in rows q | k | v | g | bottleneck behind the attention's
  int gq_off = 0, gk_off = 0, gv_off = 0, gg_off = 0, ga_off = 0;
  StackTensor a2, a2_b, gla_norm;  // [Hd][rank] compute type, [Hd] fp32, [gla_vdim] fp32
  // feed-forward
  StackTensor w_gu, b_gu, w_down, b_down;  // dense: [2ff][W], [2ff], [W][ff], [W]; experts: stacked per expert
  StackTensor router;                      // [E][W] fp32; with a shared expert one more row: the logit of its per-token gate
  StackTensor correction;                  // [E] fp32: added to the sigmoid scores when the experts are chosen
  StackTensor w_sgu, w_sdown;              // shared expert: [2 shared_ff][W], [W][shared_ff]
  // an ungated activation (DIS_ACT_RELU2) has no gate rows: w_gu / w_sgu hold [ff][W] per unit, named "up"
  int gu_rows = 2;                         // rows of w_gu per hidden unit: 2 (gate | up) or 1
  StackTensor hc[2];                       // residual streams: coefficients of the mixer's and the feed-forward's frame, in[S] | out[S] | mix[S][S] fp32
  // state-space mixer: w_in rows z | x | B | C | dt; norm_w = gain of the group norm [H*vdim]
  StackTensor conv_w, conv_b, ssm_vec;     // [C][taps], [C], dt_bias | A_log | D [3H], all fp32
  int x_off = 0, dt_off = 0, conv_ch = 0;
};

// One execution of a layer inside a forward pass.  Without a loop every layer runs once; a looped stretch contributes one
// run per pass and layer, all reading the layer's weights, each with its own recurrent state and cache.
struct StackRun {
  int layer = 0;
  int loop_pass = -1;       // t >= 0: the first layer of loop pass t (the loop's input projection runs in front of it)
  int kv_run = -1;          // latent, attention: the run whose pool(s) this run reads (itself when it owns them)
  void *pool = nullptr;     // latent with a pool of its own: [pages*page_size][kv_rank + rot_dim]
  void *kpool = nullptr, *vpool = nullptr;  // attention: [pages*page_size][G*dim], [..][G*vdim]
  float *state = nullptr;   // lightning / gated linear attention [slots][H][d][dv]; mingru [slots][n]
  float *cstate1 = nullptr, *cstate2 = nullptr;      // [slots][taps-1][W]
  float *conv_state = nullptr;                       // state-space mixer: the convolution's last inputs [slots][conv_taps-1][C]
};

struct StackModel {
  dis_stack_config c{};
  bool f32 = false;
  std::vector<StackLayer> layers;
  std::vector<StackRun> runs;
  StackTensor embed, head;
  float *final_g = nullptr;
  StackTensor final_w, final_b;    // layer-norm form of the final norm
  StackTensor loop_in, loop_step;  // [W][2W] compute type, [times][W] fp32
  double *pos_freq = nullptr;      // sinusoidal positions: base^(-2i/W), i < (W + 1) / 2
  float *ssm = nullptr;            // state-space mixer: x | B | C after convolution and SiLU, per token
  size_t ssm_ld = 0;
  float *x0 = nullptr;             // the scaled embedding rows of the pass (input of every loop pass)
  void *xcat = nullptr;            // [x ; x0] in the compute type
  float *dec = nullptr;            // gated linear attention: the decays of the pass [T][H*d]
  float *vrot = nullptr;           // attention with rotated values: cos | sin of every token's value angles [T][vdim]
  float *attn_part = nullptr;      // attention: slice records
  size_t attn_part_elems = 0;
  float *light_seg_a = nullptr;    // gated linear attention: decay products of the segments of long spans
  std::vector<StackTensor *> views;  // named scalars and taps: tensors that point into areas owned elsewhere
  int max_rows = 0;
  // activations
  float *x = nullptr, *y = nullptr, *hn = nullptr, *proj = nullptr, *mix = nullptr, *mix2 = nullptr, *qf = nullptr, *logits = nullptr;
  void *hc = nullptr, *act = nullptr, *xr = nullptr;
  // latent attention of long portions as matrix products: bf16 queries, gathered latents and their transpose, score block, weights
  bool lat_gemm = false;
  int lat_ctx_cap = 0;
  size_t lat_s_elems = 0;
  uint16_t *lat_qb = nullptr, *lat_cg = nullptr, *lat_cgt = nullptr, *lat_p = nullptr;
  float *lat_s = nullptr;
  float *light_seg = nullptr; // lightning: entry states of the segments of long spans
  float *lat_part = nullptr;  // latent attention: slice records
  size_t lat_part_elems = 0;
  float *scratch = nullptr;  // split-K slices of the tensor-core products
  size_t scratch_elems = 0;
  // experts
  int *r_idx = nullptr, *counts = nullptr, *perm_tok = nullptr, *where = nullptr, *tiles = nullptr;
  float *r_wt = nullptr, *rows_out = nullptr;
  float *y2 = nullptr, *r_sg = nullptr;  // shared expert: its output [T][W] and the logit of its per-token gate [T]
  void *moe_x = nullptr;       // bf16 activations in expert row order (per-expert tensor-core products of large passes)
  int *h_counts = nullptr;     // pinned: rows per expert of the layer being run
  // large passes: the experts' products run side by side on these streams (an expert's gate-up product, gated unit and down
  // product stay on one stream; the pass's stream forks before them and joins behind them)
  static constexpr int kSide = 3;
  cudaStream_t side[kSide] = {nullptr, nullptr, nullptr};
  cudaEvent_t ev_fork = nullptr, ev_join[kSide] = {nullptr, nullptr, nullptr};
  // a shared expert runs beside the router and the experts: its own stream, split-K slices, gate | up rows and activations
  cudaStream_t sh_stream = nullptr;
  cudaEvent_t ev_sh_fork = nullptr, ev_sh_join = nullptr;
  float *sh_proj = nullptr, *sh_scratch = nullptr;
  void *sh_act = nullptr;
  size_t sh_scratch_elems = 0;
  int max_tiles = 0;
  uint32_t *d_out = nullptr, *h_out = nullptr;  // [max_rows] ids then [max_rows] log-probabilities
};

}  // namespace dis
