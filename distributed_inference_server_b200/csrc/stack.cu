// stack.cu -- the layer-list decoder family inside the engine: configuration checks, allocation of weights / recurrent state /
// latent page pools, loading tensors by name, and the one forward pass (prompt chunks and decode rows together) that
// dis_engine_step, _prefill and _decode run for this family.  Sequences, page allocation, the step planner, the sampler,
// the serving loop and the C ABI are the engine's own (engine.cu, serving.cpp); the reference has no such family.
#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>

#include "engine.h"

namespace dis {

#define ENG_CUDA(expr)                                                                                \
  do {                                                                                                \
    cudaError_t _e = (expr);                                                                          \
    if (_e != cudaSuccess) {                                                                          \
      healthy = false;                                                                                \
      const char *_g = get_last_error();                                                              \
      std::string _m = (_g && *_g) ? std::string(_g) : std::string(cudaGetErrorString(_e));           \
      return fail(_e == cudaErrorMemoryAllocation ? DIS_ERR_OUT_OF_MEMORY : DIS_ERR_INFERENCE_FAILED, \
                  std::string(#expr) + ": " + _m);                                                    \
    }                                                                                                 \
  } while (0)
#define RET_CUDA(expr)                \
  do {                                \
    cudaError_t _e = (expr);          \
    if (_e != cudaSuccess) return _e; \
  } while (0)

static size_t align_up16(size_t v) { return (v + 15) / 16 * 16; }

void Engine::free_stack() {
  for (void *p : stack_allocs) cudaFree(p);
  stack_allocs.clear();
  if (stack) {
    if (stack->h_out) cudaFreeHost(stack->h_out);
    if (stack->h_counts) cudaFreeHost(stack->h_counts);
    for (int i = 0; i < StackModel::kSide; i++) {
      if (stack->side[i]) cudaStreamDestroy(stack->side[i]);
      if (stack->ev_join[i]) cudaEventDestroy(stack->ev_join[i]);
    }
    if (stack->ev_fork) cudaEventDestroy(stack->ev_fork);
    if (stack->sh_stream) cudaStreamDestroy(stack->sh_stream);
    if (stack->ev_sh_fork) cudaEventDestroy(stack->ev_sh_fork);
    if (stack->ev_sh_join) cudaEventDestroy(stack->ev_sh_join);
    for (StackTensor *v : stack->views) delete v;
    delete stack;
    stack = nullptr;
  }
}

const TmaMap *Engine::stack_map(const void *base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
  const auto key = std::make_tuple(base, rows, cols, box_rows);
  auto it = stack_maps.find(key);
  if (it != stack_maps.end()) return &it->second;
  TmaMap m;
  if (make_tma_map_2d(&m, base, rows, cols, box_rows) != cudaSuccess) return nullptr;
  return &stack_maps.emplace(key, m).first->second;
}

cudaError_t Engine::stack_meta(StepMeta &s, int cap_t, int cap_rows) {
  s.cap_tokens = cap_t;
  s.cap_rows = cap_rows;
  size_t o = 0;
  auto sec = [&](size_t bytes) { size_t at = o; o = align_up16(o + bytes); return at; };
  const size_t ct = (size_t)cap_t, cr = (size_t)cap_rows;
  s.o_tokens = sec(ct * 4); s.o_pos = sec(ct * 4); s.o_ptrow = sec(ct * 4); s.o_ctx = sec(ct * 4); s.o_span = sec(ct * 4);
  s.o_rowmap = sec(cr * 4); s.o_temp = sec(cr * 4); s.o_topp = sec(cr * 4); s.o_seed = sec(cr * 8); s.o_step = sec(cr * 8);
  s.o_qb_tok0 = sec(ct * 4); s.o_qb_len = sec(ct * 4); s.o_qb_pos0 = sec(ct * 4); s.o_qb_ptrow = sec(ct * 4);
  s.o_ab_tok0 = sec(ct * 4); s.o_ab_len = sec(ct * 4);
  s.o_kb_tok0 = sec(ct * 4); s.o_kb_len = sec(ct * 4);
  s.o_arstep = sec(16);
  s.bytes = o;
  cudaError_t e = cudaMallocHost(reinterpret_cast<void **>(&s.host), s.bytes);
  if (e != cudaSuccess) return e;
  memset(s.host, 0, s.bytes);
  e = cudaMalloc(reinterpret_cast<void **>(&s.dev), s.bytes);
  if (e == cudaSuccess) bytes_allocated += s.bytes;
  return e;
}

int Engine::init_stack(const dis_engine_config *c, const dis_stack_config *sc) {
  cfg = *c;
  if (!sc || !sc->layers || sc->n_layers <= 0 || sc->vocab <= 0 || sc->width <= 0 || sc->max_ctx <= 0)
    return fail(DIS_ERR_INVALID_ARGUMENT, "stack config: vocab, width, layers and max_ctx must be positive");
  if (c->tp_size > 1) return fail(DIS_ERR_INVALID_ARGUMENT, "stack: tensor parallelism is not available for this family");
  if (c->flags & DIS_FLAG_PREFIX_CACHE)
    return fail(DIS_ERR_INVALID_ARGUMENT, "stack: the prefix cache cannot serve a family with recurrent state (a page does not hold it)");
  if (sc->compute_dtype != DIS_F32 && sc->compute_dtype != DIS_BF16) return fail(DIS_ERR_INVALID_ARGUMENT, "stack: compute_dtype");
  if (sc->canon_taps < 0 || sc->canon_taps > 16) return fail(DIS_ERR_INVALID_ARGUMENT, "stack: canon_taps must be 0..16");
  memset(&m, 0, sizeof(m));
  m.vocab = sc->vocab; m.hidden = sc->width; m.layers = sc->n_layers; m.max_ctx = sc->max_ctx; m.rms_eps = sc->norm_eps;
  tp_rank = 0; tp_size = 1;
  vocab_l = m.vocab; vocab_off = 0;
  max_batch = c->max_batch > 0 ? c->max_batch : 32;
  cap_tokens = std::max(c->max_step_tokens > 0 ? c->max_step_tokens : 8192, max_batch);
  page_size = c->page_size > 0 ? c->page_size : 64;
  if ((page_size & (page_size - 1)) || page_size < 8) return fail(DIS_ERR_INVALID_ARGUMENT, "page_size must be a power of two >= 8");
  max_pages = (m.max_ctx + page_size - 1) / page_size;

  stack = new StackModel();
  StackModel &M = *stack;
  M.c = *sc;
  M.f32 = sc->compute_dtype == DIS_F32;
  M.max_rows = std::max(sc->max_logit_rows > 0 ? sc->max_logit_rows : max_batch, max_batch);
  M.layers.resize((size_t)sc->n_layers);
  const int W = sc->width, taps = sc->canon_taps;
  // ---- configuration checks, per layer

  for (int i = 0; i < sc->n_layers; i++) {
    StackLayer &L = M.layers[(size_t)i];
    L.c = sc->layers[i];
    const dis_layer_config &lc = L.c;
    const std::string at = "stack layer " + std::to_string(i) + ": ";
    if (lc.mixer == DIS_MIX_LIGHTNING) {
      if (lc.heads <= 0 || lc.dim <= 0 || lc.vdim <= 0 || !lc.decay) return fail(DIS_ERR_INVALID_ARGUMENT, at + "lightning needs heads, dim, vdim, decay");
      L.decay.assign(lc.decay, lc.decay + lc.heads);
      L.c.decay = nullptr;
      if (((size_t)lc.dim * lc.vdim + 2 * lc.dim + 9 * lc.vdim) * 4 > 220 * 1024) return fail(DIS_ERR_INVALID_ARGUMENT, at + "dim * vdim does not fit shared memory");
      L.n_in = 2 * lc.heads * lc.dim + 2 * lc.heads * lc.vdim;
      L.g_off = 2 * lc.heads * lc.dim + lc.heads * lc.vdim;
    } else if (lc.mixer == DIS_MIX_MINGRU) {
      if (lc.width <= 0) return fail(DIS_ERR_INVALID_ARGUMENT, at + "mingru needs width");
      L.n_in = 3 * lc.width;
    } else if (lc.mixer == DIS_MIX_LATENT) {
      if (lc.heads <= 0 || lc.dim <= 0 || lc.vdim <= 0 || lc.kv_rank <= 0 || lc.rot_dim < 0 || lc.rot_dims < 0 || lc.rot_dims > lc.rot_dim || (lc.rot_dims & 1))
        return fail(DIS_ERR_INVALID_ARGUMENT, at + "latent attention needs heads, dim, vdim, kv_rank, and an even rot_dims <= rot_dim");
      if (lc.kv_rank > 1024) return fail(DIS_ERR_INVALID_ARGUMENT, at + "kv_rank above 1024");

      if (lc.kv_from >= 0) {
        if (lc.kv_from >= i) return fail(DIS_ERR_INVALID_ARGUMENT, at + "kv_from must name an earlier layer");
        const dis_layer_config &src = M.layers[(size_t)lc.kv_from].c;
        if (src.mixer != DIS_MIX_LATENT || src.kv_from >= 0 || src.kv_rank != lc.kv_rank || src.rot_dim != lc.rot_dim)
          return fail(DIS_ERR_INVALID_ARGUMENT, at + "kv_from must name a latent layer with a cache of its own and the same kv_rank and rot_dim");
      }
      L.q_off = 0;
      L.dkv_off = lc.heads * (lc.dim + lc.rot_dim);
      L.g_off = L.dkv_off + (lc.kv_from < 0 ? lc.kv_rank + lc.rot_dim : 0);
      L.n_in = L.g_off + lc.heads * lc.vdim;
      StackLatent sl{lc.heads, lc.dim, lc.rot_dim, lc.vdim, lc.kv_rank, lc.rot_dims, lc.rot_base, lc.scale, sc->norm_eps};
      if (((size_t)32 * (lc.kv_rank + lc.rot_dim + 9) + (size_t)lc.heads * (2 * lc.kv_rank + lc.rot_dim + 2)) * 4 > 200 * 1024)
        return fail(DIS_ERR_INVALID_ARGUMENT, at + "heads * kv_rank does not fit shared memory");
      stack_bq = std::min(stack_bq, stack_latent_block_tokens(sl));
      const char *mma_env = getenv("DIS_STACK_LATENT_MMA");
      if (!(mma_env && atoi(mma_env) == 0) && stack_latent_mma_ok(sl, sc->compute_dtype == DIS_F32)) {
        stack_bq = std::min(stack_bq, std::max(1, 16 / lc.heads));
        stack_lat_mma = true;
      }
    } else if (lc.mixer == DIS_MIX_ATTENTION || lc.mixer == DIS_MIX_PARALLEL) {
      if (lc.heads <= 0 || lc.kv_heads <= 0 || lc.heads % lc.kv_heads || lc.dim <= 0 || lc.vdim <= 0 || lc.rot_dims < 0 || lc.rot_dims > lc.dim || (lc.rot_dims & 1))
        return fail(DIS_ERR_INVALID_ARGUMENT, at + "attention needs heads (a multiple of kv_heads), dim, vdim and an even rot_dims <= dim");
      if ((lc.attn_flags & DIS_ATTN_V_IS_K) && lc.vdim != lc.dim) return fail(DIS_ERR_INVALID_ARGUMENT, at + "values that are the keys need vdim == dim");
      if ((lc.attn_flags & DIS_ATTN_ROT_V) && (lc.vdim & 1)) return fail(DIS_ERR_INVALID_ARGUMENT, at + "rotated values need an even vdim");
      if (lc.rot_factor != 0.f && (lc.rot_high == lc.rot_low || lc.rot_original <= 0 || lc.rot_low <= 0.f || lc.rot_high <= 0.f))
        return fail(DIS_ERR_INVALID_ARGUMENT, at + "rotary scaling needs original > 0 and 0 < low != high");
      const unsigned fl = lc.attn_flags;
      if ((fl & DIS_ATTN_SINK) && (fl & DIS_ATTN_SIGMOID)) return fail(DIS_ERR_INVALID_ARGUMENT, at + "a sink belongs to softmax weights");
      if ((fl & DIS_ATTN_QK_NORM) && (fl & DIS_ATTN_QK_NORM_HEAD)) return fail(DIS_ERR_INVALID_ARGUMENT, at + "query/key norm: whole projection or per head, not both");
      if ((fl & DIS_ATTN_BIAS) && (fl & DIS_ATTN_BIAS_QKV)) return fail(DIS_ERR_INVALID_ARGUMENT, at + "biases: q, k, o or q, k, v, not both");
      if (lc.mask_chunk < 0 || lc.mask_window < 0) return fail(DIS_ERR_INVALID_ARGUMENT, at + "mask_chunk and mask_window must not be negative");
      if (!(lc.score_softcap >= 0.f)) return fail(DIS_ERR_INVALID_ARGUMENT, at + "score_softcap must not be negative");
      if ((fl & DIS_ATTN_SIGMOID) && (lc.score_softcap > 0.f || (fl & DIS_ATTN_SINK_UNIT))) return fail(DIS_ERR_INVALID_ARGUMENT, at + "a score soft cap and a sink belong to softmax weights");
      if ((fl & DIS_ATTN_SINK) && (fl & DIS_ATTN_SINK_UNIT)) return fail(DIS_ERR_INVALID_ARGUMENT, at + "sink: a learned logit per head or the unit term, not both");
      if (lc.kv_from >= 0) {
        if (lc.kv_from >= i) return fail(DIS_ERR_INVALID_ARGUMENT, at + "kv_from must name an earlier layer");
        const dis_layer_config &src = M.layers[(size_t)lc.kv_from].c;
        if ((src.mixer != DIS_MIX_ATTENTION && src.mixer != DIS_MIX_PARALLEL) || src.kv_from >= 0 || src.kv_heads != lc.kv_heads ||
            src.dim != lc.dim || src.vdim != lc.vdim || src.rot_dims != lc.rot_dims || src.rot_base != lc.rot_base ||
            ((src.attn_flags ^ fl) & DIS_ATTN_ROT_V))
          return fail(DIS_ERR_INVALID_ARGUMENT, at + "kv_from must name an attention layer with a cache of its own and the same kv_heads, dim, vdim and rotation");
      }
      const int H = lc.heads, G = lc.kv_heads, d = lc.dim, dv = lc.vdim;
      StackAttn sa{H, G, d, dv, lc.rot_dims, lc.attn_flags, lc.scale, sc->norm_eps, lc.mask_chunk, lc.mask_window, lc.score_softcap};
      const int bq = stack_attn_block_tokens(sa, sc->compute_dtype == DIS_F32);
      if (((size_t)32 * (d + dv + 10) + (size_t)(H / G) * (d + dv + 2)) * 4 > 200 * 1024) return fail(DIS_ERR_INVALID_ARGUMENT, at + "dim + vdim does not fit shared memory");
      stack_abq = stack_abq ? std::min(stack_abq, bq) : bq;
      stack_att_heads = std::max(stack_att_heads, H);
      stack_att_groups = stack_att_groups ? std::min(stack_att_groups, G) : G;
      stack_att_rec = std::max(stack_att_rec, (size_t)H * (dv + 2));
      // rows of the input projection: q | k | v (a layer with a cache of its own) | one gate row per head
      L.q_off = 0; L.k_off = H * d; L.v_off = L.k_off + G * d;
      L.n_in = lc.kv_from >= 0 ? H * d : L.v_off + ((lc.attn_flags & DIS_ATTN_V_IS_K) ? 0 : G * dv);
      if (lc.kv_from >= 0) L.k_off = L.v_off = 0;
      if (fl & DIS_ATTN_GATE) { L.g_off = L.n_in; L.n_in += H; }
      L.n_act = H * dv;
      if (lc.mixer == DIS_MIX_PARALLEL) {
        const int Hr = lc.gla_heads, dr = lc.gla_dim, dvr = lc.gla_vdim;
        if (Hr <= 0 || dr <= 0 || dvr <= 0 || lc.gla_rank <= 0 || lc.gla_rank > 768 || !(lc.gla_tau > 0.f)) return fail(DIS_ERR_INVALID_ARGUMENT, at + "gated linear attention needs heads, dim, vdim, a rank up to 768 and tau > 0");
        if ((dr > 128 || dvr > 128) && ((size_t)dr * dvr + 3 * dr + 9 * dvr) * 4 > 220 * 1024)
          return fail(DIS_ERR_INVALID_ARGUMENT, at + "gated linear attention: dim * vdim does not fit shared memory");
        L.gq_off = L.n_in; L.gk_off = L.gq_off + Hr * dr; L.gv_off = L.gk_off + Hr * dr; L.gg_off = L.gv_off + Hr * dvr;
        L.ga_off = L.gg_off + Hr * dvr;
        L.n_in = L.ga_off + lc.gla_rank;
        L.n_act += Hr * dvr;
      }
    } else if (lc.mixer == DIS_MIX_SSM) {
      if (L.c.ssm_norm_groups == 0) L.c.ssm_norm_groups = 1;
      const int H = lc.heads, P = lc.vdim, N = lc.ssm_state, G = lc.ssm_groups;
      if (H <= 0 || P <= 0 || N <= 0 || G <= 0 || H % G || lc.conv_taps < 1 || lc.conv_taps > 16 || L.c.ssm_norm_groups < 1 ||
          (H * P) % L.c.ssm_norm_groups)
        return fail(DIS_ERR_INVALID_ARGUMENT, at + "the state-space mixer needs heads (a multiple of ssm_groups), vdim, ssm_state, conv_taps 1..16 and ssm_norm_groups dividing heads * vdim");
      if ((N > 128 || P > 128) && ((size_t)N * P + 3 * N + 9 * P) * 4 > 220 * 1024)
        return fail(DIS_ERR_INVALID_ARGUMENT, at + "state-space mixer: ssm_state * vdim does not fit shared memory");
      if ((size_t)H * P * 4 > 160 * 1024) return fail(DIS_ERR_INVALID_ARGUMENT, at + "state-space mixer: heads * vdim above 40960");
      // rows of the input projection: z | x | B | C | dt; the convolution runs over x | B | C
      L.conv_ch = H * P + 2 * G * N;
      L.x_off = H * P; L.dt_off = L.x_off + L.conv_ch;
      L.n_in = L.dt_off + H;
    } else return fail(DIS_ERR_INVALID_ARGUMENT, at + "unknown mixer");
    if (lc.mlp_act != DIS_ACT_CLAMPED && lc.mlp_act != DIS_ACT_GELU_TANH && lc.mlp_act != DIS_ACT_SILU && lc.mlp_act != DIS_ACT_RELU2) return fail(DIS_ERR_INVALID_ARGUMENT, at + "unknown feed-forward activation");
    L.gu_rows = lc.mlp_act == DIS_ACT_RELU2 ? 1 : 2;
    if (lc.mlp == DIS_MLP_DENSE) { if (lc.ff <= 0) return fail(DIS_ERR_INVALID_ARGUMENT, at + "ff"); }
    else if (lc.mlp == DIS_MLP_MOE) {
      if (lc.ff <= 0 || lc.experts <= 0 || lc.top <= 0 || lc.top > lc.experts || lc.top > 32 || lc.experts > 1024)
        return fail(DIS_ERR_INVALID_ARGUMENT, at + "experts: 1 <= top <= min(experts, 32), experts <= 1024");
      if (lc.route_kind != DIS_ROUTE_SOFTMAX_TOP && lc.route_kind != DIS_ROUTE_SIGMOID_GROUPS && lc.route_kind != DIS_ROUTE_SOFTMAX_ALL) return fail(DIS_ERR_INVALID_ARGUMENT, at + "unknown router kind");
      if (lc.route_groups > 1) {
        if (lc.route_kind != DIS_ROUTE_SIGMOID_GROUPS || lc.experts % lc.route_groups || lc.route_keep < 1 || lc.route_keep > lc.route_groups ||
            lc.route_keep * (lc.experts / lc.route_groups) < lc.top)
          return fail(DIS_ERR_INVALID_ARGUMENT, at + "expert groups: a divisor of experts, 1 <= keep <= groups, and the kept groups must hold at least top experts");
      }
      if (lc.shared_ff < 0) return fail(DIS_ERR_INVALID_ARGUMENT, at + "shared_ff");
    } else if (lc.mlp != DIS_MLP_NONE) return fail(DIS_ERR_INVALID_ARGUMENT, at + "unknown feed-forward kind");
  }
  if (sc->norm_kind != DIS_NORM_RMS_SCALAR && sc->norm_kind != DIS_NORM_LAYER && sc->norm_kind != DIS_NORM_RMS) return fail(DIS_ERR_INVALID_ARGUMENT, "stack: norm_kind");
  if (sc->logit_softcap < 0.f) return fail(DIS_ERR_INVALID_ARGUMENT, "stack: logit_softcap must not be negative");
  const bool pre_frame = (sc->frame_flags & DIS_FRAME_PRE_NORM) != 0;
  if (pre_frame && (sc->norm_kind != DIS_NORM_RMS || sc->canon_taps != 0))
    return fail(DIS_ERR_INVALID_ARGUMENT, "stack: the pre-norm frame is built for RMS norms with gain vectors and no input convolution");
  if (sc->streams < 0 || sc->streams > 8 || (sc->streams > 0 && !pre_frame))
    return fail(DIS_ERR_INVALID_ARGUMENT, "stack: residual streams (at most 8) need the pre-norm frame");
  const bool loop_proj = sc->loop_times > 0 && !(sc->frame_flags & DIS_FRAME_LOOP_PLAIN);
  const int n_streams = std::max(1, sc->streams);
  if (sc->loop_times < 0 || (sc->loop_times > 0 && !(0 <= sc->loop_start && sc->loop_start < sc->loop_stop && sc->loop_stop <= sc->n_layers)))
    return fail(DIS_ERR_INVALID_ARGUMENT, "stack: a loop needs 0 <= loop_start < loop_stop <= n_layers");
  if (M.c.embed_scale == 0.f) M.c.embed_scale = 1.f;
  if (M.c.logit_scale == 0.f) M.c.logit_scale = 1.f;
  // ---- the layer runs of one pass: the looped stretch once per loop pass
  for (int i = 0; i < sc->n_layers; i++) {
    if (sc->loop_times > 0 && i == sc->loop_start) {
      for (int t = 0; t < sc->loop_times; t++)
        for (int j = sc->loop_start; j < sc->loop_stop; j++) { StackRun r; r.layer = j; r.loop_pass = j == sc->loop_start ? t : -1; M.runs.push_back(r); }
      i = sc->loop_stop - 1;
      continue;
    }
    StackRun r; r.layer = i;
    M.runs.push_back(r);
  }
  for (size_t ri = 0; ri < M.runs.size(); ri++) {  // a layer that borrows a cache reads the latest run of its owner
    const StackLayer &L = M.layers[(size_t)M.runs[ri].layer];
    if (L.c.mixer != DIS_MIX_LATENT && L.c.mixer != DIS_MIX_ATTENTION && L.c.mixer != DIS_MIX_PARALLEL) continue;
    M.runs[ri].kv_run = (int)ri;
    if (L.c.kv_from >= 0)
      for (size_t rj = 0; rj < ri; rj++) if (M.runs[rj].layer == L.c.kv_from) M.runs[ri].kv_run = (int)rj;
  }

  int ndev = 0;
  if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) return fail(DIS_ERR_INFERENCE_FAILED, "no CUDA device: this engine has no CPU fallback");
  if (c->device < 0 || c->device >= ndev) return fail(DIS_ERR_INVALID_ARGUMENT, "device ordinal out of range");
  ENG_CUDA(cudaSetDevice(c->device));
  cudaDeviceProp prop;
  ENG_CUDA(cudaGetDeviceProperties(&prop, c->device));
  if (prop.major != 10) return fail(DIS_ERR_INFERENCE_FAILED, "device is not sm_100; kernels are built for sm_100a only");
  if (c->stream) stream = (cudaStream_t)c->stream;
  else { ENG_CUDA(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking)); own_stream = true; }
  ENG_CUDA(cudaEventCreate(&ev0));
  ENG_CUDA(cudaEventCreate(&ev1));

  const size_t esz = M.f32 ? 4 : 2;
  auto alloc = [&](void **p, size_t bytes) -> cudaError_t {
    *p = nullptr;
    if (!bytes) return cudaSuccess;
    cudaError_t e = cudaMalloc(p, bytes);
    if (e != cudaSuccess) { set_last_error("cudaMalloc of " + std::to_string(bytes) + " bytes failed"); return e; }
    stack_allocs.push_back(*p);
    bytes_allocated += bytes;
    return cudaMemset(*p, 0, bytes);
  };
  auto tensor = [&](StackTensor &t, size_t n, bool f32) -> cudaError_t {
    t.n = n; t.f32 = f32;
    return alloc(&t.ptr, n * (f32 ? 4 : 2));
  };
  auto name = [&](const std::string &nm, StackTensor *dst, size_t off, std::vector<int64_t> shape, int layer, int transform = 0) {
    stack_names[nm] = StackTarget{dst, off, std::move(shape), transform, false, layer};
  };
  // ---- weights
  ENG_CUDA(tensor(M.embed, (size_t)sc->vocab * W, M.f32));
  name("embed", &M.embed, 0, {sc->vocab, W}, -1);
  if (sc->frame_flags & DIS_FRAME_TIED_HEAD) M.head = M.embed;  // the same memory: logits are products with the embedding rows
  else {
    ENG_CUDA(tensor(M.head, (size_t)sc->vocab * W, M.f32));
    name("head", &M.head, 0, {sc->vocab, W}, -1);
  }
  ENG_CUDA(alloc(reinterpret_cast<void **>(&M.final_g), 4));
  const bool ln = sc->norm_kind == DIS_NORM_LAYER || sc->norm_kind == DIS_NORM_RMS;  // norms with vectors
  const bool ln_bias = sc->norm_kind == DIS_NORM_LAYER;
  if (ln) {
    ENG_CUDA(tensor(M.final_w, (size_t)W, true));
    name("final.norm", &M.final_w, 0, {W}, -1);
    if (ln_bias) {
      ENG_CUDA(tensor(M.final_b, (size_t)W, true));
      name("final.norm.b", &M.final_b, 0, {W}, -1);
    }
  }
  if (loop_proj) {
    ENG_CUDA(tensor(M.loop_in, (size_t)W * 2 * W, M.f32));
    ENG_CUDA(tensor(M.loop_step, (size_t)sc->loop_times * W, true));
    name("loop.in", &M.loop_in, 0, {W, 2 * W}, -1);
    name("loop.step", &M.loop_step, 0, {sc->loop_times, W}, -1);
  }
  static StackTensor dummy;  // scalars are written through their own small tensors below
  (void)dummy;
  size_t max_proj = 1, max_mix = 1, max_act = 1, max_qf = 1, max_vrot = 0, max_dec = 0, max_ssm = 0;
  int max_top = 0, max_e = 0;
  bool any_shared = false;
  size_t max_sff = 0;
  const size_t slots = (size_t)max_batch;
  std::vector<StackTensor *> scalars;
  for (int i = 0; i < sc->n_layers; i++) {
    StackLayer &L = M.layers[(size_t)i];
    const dis_layer_config &lc = L.c;
    const std::string pre = "l" + std::to_string(i) + ".";
    ENG_CUDA(alloc(reinterpret_cast<void **>(&L.g4), 16));
    if (taps >= 1) {
      ENG_CUDA(alloc(reinterpret_cast<void **>(&L.canon1), (size_t)W * taps * 4));
      if (lc.mlp != DIS_MLP_NONE) ENG_CUDA(alloc(reinterpret_cast<void **>(&L.canon2), (size_t)W * taps * 4));
    }
    if (ln) {
      const char *gn[4] = {"norm1", "norm1b", "norm2", "norm2b"};
      for (int k = 0; k < 4; k++) {
        if (k >= 2 && lc.mlp == DIS_MLP_NONE) continue;
        if (pre_frame && (k & 1)) continue;  // no norms behind the sublayers
        ENG_CUDA(tensor(L.ln_w[k], (size_t)W, true));
        name(pre + gn[k], &L.ln_w[k], 0, {W}, i);
        if (!ln_bias) continue;
        ENG_CUDA(tensor(L.ln_b[k], (size_t)W, true));
        name(pre + gn[k] + ".b", &L.ln_b[k], 0, {W}, i);
      }
    }
    for (int q = 0; q < (lc.mlp == DIS_MLP_NONE ? 1 : 2) && sc->streams > 0; q++) {  // coefficients of the residual streams
      const int S = sc->streams;
      const std::string hp = pre + "hc" + std::to_string(q + 1) + ".";
      ENG_CUDA(tensor(L.hc[q], (size_t)(2 * S + S * S), true));
      name(hp + "in", &L.hc[q], 0, {S}, i);
      name(hp + "out", &L.hc[q], (size_t)S, {S}, i);
      name(hp + "mix", &L.hc[q], (size_t)2 * S, {S, S}, i);
    }
    ENG_CUDA(tensor(L.w_in, (size_t)L.n_in * W, M.f32));
    max_proj = std::max(max_proj, (size_t)L.n_in);
    if (lc.mixer == DIS_MIX_LIGHTNING) {
      const int H = lc.heads, d = lc.dim, dv = lc.vdim;
      name(pre + "mix.q", &L.w_in, 0, {H * d, W}, i);
      name(pre + "mix.k", &L.w_in, (size_t)H * d * W, {H * d, W}, i);
      name(pre + "mix.v", &L.w_in, (size_t)2 * H * d * W, {H * dv, W}, i);
      name(pre + "mix.g", &L.w_in, (size_t)L.g_off * W, {H * dv, W}, i);
      ENG_CUDA(tensor(L.w_o, (size_t)W * H * dv, M.f32));
      name(pre + "mix.o", &L.w_o, 0, {W, H * dv}, i);
      ENG_CUDA(tensor(L.norm_w, (size_t)H * dv, true));
      name(pre + "mix.norm", &L.norm_w, 0, {H * dv}, i);
      ENG_CUDA(tensor(L.decay_d, (size_t)H, true));
      ENG_CUDA(cudaMemcpy(L.decay_d.ptr, L.decay.data(), (size_t)H * 4, cudaMemcpyHostToDevice));
      max_mix = std::max(max_mix, (size_t)H * dv);
      max_act = std::max(max_act, (size_t)H * dv);
    } else if (lc.mixer == DIS_MIX_ATTENTION || lc.mixer == DIS_MIX_PARALLEL) {
      const int H = lc.heads, G = lc.kv_heads, d = lc.dim, dv = lc.vdim;
      const std::string a = pre + (lc.mixer == DIS_MIX_PARALLEL ? "mix.left." : "mix.");
      const bool own = lc.kv_from < 0;
      name(a + "q", &L.w_in, 0, {H * d, W}, i);
      if (own) name(a + "k", &L.w_in, (size_t)L.k_off * W, {G * d, W}, i);
      if (own && !(lc.attn_flags & DIS_ATTN_V_IS_K)) name(a + "v", &L.w_in, (size_t)L.v_off * W, {G * dv, W}, i);
      if (lc.attn_flags & DIS_ATTN_GATE) name(a + "g", &L.w_in, (size_t)L.g_off * W, {H, W}, i);
      ENG_CUDA(tensor(L.w_o, (size_t)W * L.n_act, M.f32));
      {
        name(a + "o", &L.w_o, 0, {W, H * dv}, i, 2);
        stack_names[a + "o"].ld = L.n_act;
      }
      if (lc.attn_flags & DIS_ATTN_BIAS) {
        ENG_CUDA(tensor(L.b_in, (size_t)L.n_in, true));
        name(a + "q.b", &L.b_in, 0, {H * d}, i);
        name(a + "k.b", &L.b_in, (size_t)L.k_off, {G * d}, i);
        ENG_CUDA(tensor(L.b_o, (size_t)W, true));
        name(a + "o.b", &L.b_o, 0, {W}, i);
      }
      if (lc.attn_flags & DIS_ATTN_BIAS_QKV) {
        ENG_CUDA(tensor(L.b_in, (size_t)L.n_in, true));
        name(a + "q.b", &L.b_in, 0, {H * d}, i);
        if (own) {
          name(a + "k.b", &L.b_in, (size_t)L.k_off, {G * d}, i);
          name(a + "v.b", &L.b_in, (size_t)L.v_off, {G * dv}, i);
        }
      }
      if (lc.attn_flags & DIS_ATTN_QK_NORM_HEAD) {
        ENG_CUDA(tensor(L.qk_norm, (size_t)2 * d, true));
        name(a + "q.norm", &L.qk_norm, 0, {d}, i);
        if (own) name(a + "k.norm", &L.qk_norm, (size_t)d, {d}, i);
      }
      if (lc.attn_flags & DIS_ATTN_SINK) {
        ENG_CUDA(tensor(L.sink, (size_t)H, true));
        name(a + "sink", &L.sink, 0, {H}, i);
      }
      if (lc.attn_flags & DIS_ATTN_SINK_UNIT) ENG_CUDA(tensor(L.sink, (size_t)H, true));  // zero logits: the denominator's extra 1
      if (lc.attn_flags & DIS_ATTN_QK_NORM) {
        ENG_CUDA(tensor(L.qk_norm, (size_t)(H + G) * d, true));
        name(a + "q.norm", &L.qk_norm, 0, {H * d}, i);
        name(a + "k.norm", &L.qk_norm, (size_t)H * d, {G * d}, i);
      }
      if (lc.attn_flags & DIS_ATTN_SIGMOID) {
        ENG_CUDA(tensor(L.temp_pb, (size_t)2 * H, true));
        name(a + "temp", &L.temp_pb, 0, {H}, i);
        name(a + "pb", &L.temp_pb, (size_t)H, {H}, i);
      }
      {  // frequency tables, formed in double: f_i = base^(-2i/n), rescaled by wavelength where the configuration asks
        std::vector<double> f((size_t)lc.rot_dims / 2 + 1), fv((size_t)dv / 2 + 1);
        const double kPi = 3.14159265358979323846;
        for (int k = 0; k < lc.rot_dims / 2; k++) {
          double v = std::pow((double)lc.rot_base, -2.0 * k / (double)lc.rot_dims);
          if (lc.rot_factor != 0.f) {
            const double wl = 2.0 * kPi / v, orig = (double)lc.rot_original;
            if (wl > orig / (double)lc.rot_low) v = v / (double)lc.rot_factor;
            else if (!(wl < orig / (double)lc.rot_high)) {
              const double sm = (orig / wl - (double)lc.rot_low) / ((double)lc.rot_high - (double)lc.rot_low);
              v = (1.0 - sm) * v / (double)lc.rot_factor + sm * v;
            }
          }
          f[(size_t)k] = v;
        }
        for (int k = 0; k < dv / 2; k++) fv[(size_t)k] = std::pow((double)lc.rot_base, -2.0 * k / (double)dv);
        ENG_CUDA(alloc(reinterpret_cast<void **>(&L.freq), f.size() * 8));
        ENG_CUDA(cudaMemcpy(L.freq, f.data(), f.size() * 8, cudaMemcpyHostToDevice));
        if (lc.attn_flags & DIS_ATTN_ROT_V) {
          ENG_CUDA(alloc(reinterpret_cast<void **>(&L.vfreq), fv.size() * 8));
          ENG_CUDA(cudaMemcpy(L.vfreq, fv.data(), fv.size() * 8, cudaMemcpyHostToDevice));
          max_vrot = std::max(max_vrot, (size_t)dv);
        }
      }
      max_qf = std::max(max_qf, (size_t)H * d);
      if (lc.mixer == DIS_MIX_PARALLEL) {
        const int Hr = lc.gla_heads, dr = lc.gla_dim, dvr = lc.gla_vdim, rk = lc.gla_rank;
        const std::string r = pre + "mix.right.";
        name(r + "q", &L.w_in, (size_t)L.gq_off * W, {Hr * dr, W}, i);
        name(r + "k", &L.w_in, (size_t)L.gk_off * W, {Hr * dr, W}, i);
        name(r + "v", &L.w_in, (size_t)L.gv_off * W, {Hr * dvr, W}, i);
        name(r + "g", &L.w_in, (size_t)L.gg_off * W, {Hr * dvr, W}, i);
        name(r + "a1", &L.w_in, (size_t)L.ga_off * W, {rk, W}, i);
        name(r + "o", &L.w_o, (size_t)H * dv, {W, Hr * dvr}, i, 2);
        stack_names[r + "o"].ld = L.n_act;
        ENG_CUDA(tensor(L.a2, (size_t)Hr * dr * rk, M.f32));
        name(r + "a2", &L.a2, 0, {Hr * dr, rk}, i);
        ENG_CUDA(tensor(L.a2_b, (size_t)Hr * dr, true));
        name(r + "a2.b", &L.a2_b, 0, {Hr * dr}, i);
        ENG_CUDA(tensor(L.gla_norm, (size_t)dvr, true));
        name(r + "norm", &L.gla_norm, 0, {dvr}, i);
        max_mix = std::max(max_mix, (size_t)Hr * dvr);
        max_dec = std::max(max_dec, (size_t)Hr * dr);
      }
      max_act = std::max(max_act, (size_t)L.n_act);
    } else if (lc.mixer == DIS_MIX_SSM) {
      const int H = lc.heads, P = lc.vdim, C = L.conv_ch, inner = H * P;
      name(pre + "mix.in", &L.w_in, 0, {L.n_in, W}, i);
      ENG_CUDA(tensor(L.conv_w, (size_t)C * lc.conv_taps, true));
      name(pre + "mix.conv", &L.conv_w, 0, {C, lc.conv_taps}, i);
      ENG_CUDA(tensor(L.conv_b, (size_t)C, true));
      name(pre + "mix.conv.b", &L.conv_b, 0, {C}, i);
      ENG_CUDA(tensor(L.ssm_vec, (size_t)3 * H, true));
      name(pre + "mix.dt_bias", &L.ssm_vec, 0, {H}, i);
      name(pre + "mix.A_log", &L.ssm_vec, (size_t)H, {H}, i);
      name(pre + "mix.D", &L.ssm_vec, (size_t)2 * H, {H}, i);
      ENG_CUDA(tensor(L.norm_w, (size_t)inner, true));
      name(pre + "mix.norm", &L.norm_w, 0, {inner}, i);
      ENG_CUDA(tensor(L.w_o, (size_t)W * inner, M.f32));
      name(pre + "mix.o", &L.w_o, 0, {W, inner}, i);
      max_mix = std::max(max_mix, (size_t)inner);
      max_act = std::max(max_act, (size_t)inner);
      max_ssm = std::max(max_ssm, (size_t)C);
      max_dec = std::max(max_dec, (size_t)2 * H);  // decays, then step sizes
    } else if (lc.mixer == DIS_MIX_MINGRU) {
      const int n = lc.width;
      name(pre + "mix.z", &L.w_in, 0, {n, W}, i);
      name(pre + "mix.x", &L.w_in, (size_t)n * W, {n, W}, i);
      name(pre + "mix.g", &L.w_in, (size_t)2 * n * W, {n, W}, i);
      ENG_CUDA(tensor(L.b_in, (size_t)3 * n, true));
      name(pre + "mix.z.b", &L.b_in, 0, {n}, i);
      name(pre + "mix.x.b", &L.b_in, (size_t)n, {n}, i);
      ENG_CUDA(tensor(L.w_o, (size_t)W * n, M.f32));
      name(pre + "mix.o", &L.w_o, 0, {W, n}, i);
      max_act = std::max(max_act, (size_t)n);
    } else {
      const int H = lc.heads, d = lc.dim, dr = lc.rot_dim, dv = lc.vdim, r = lc.kv_rank;
      name(pre + "mix.q", &L.w_in, 0, {H * (d + dr), W}, i);
      if (lc.kv_from < 0) {
        name(pre + "mix.dkv", &L.w_in, (size_t)L.dkv_off * W, {r + dr, W}, i);
        ENG_CUDA(tensor(L.norm_w, (size_t)r, true));
        name(pre + "mix.dkv.norm", &L.norm_w, 0, {r}, i);
      }
      name(pre + "mix.g", &L.w_in, (size_t)L.g_off * W, {H * dv, W}, i);
      ENG_CUDA(tensor(L.ukT, (size_t)H * r * d, M.f32));
      name(pre + "mix.uk", &L.ukT, 0, {H * d, r}, i, /*transpose each head's [d][r] block*/ 1);
      ENG_CUDA(tensor(L.uv, (size_t)H * dv * r, M.f32));
      name(pre + "mix.uv", &L.uv, 0, {H * dv, r}, i);
      ENG_CUDA(tensor(L.sink, (size_t)H, true));
      name(pre + "mix.sink", &L.sink, 0, {H}, i);
      ENG_CUDA(tensor(L.w_o, (size_t)W * H * dv, M.f32));
      name(pre + "mix.o", &L.w_o, 0, {W, H * dv}, i);
      max_mix = std::max(max_mix, (size_t)H * std::max(r, dv));
      max_act = std::max(max_act, (size_t)H * dv);
      max_qf = std::max(max_qf, (size_t)H * (r + dr));
      stack_lat_rec = std::max(stack_lat_rec, (size_t)H * (r + 2));
      stack_lat_heads = std::max(stack_lat_heads, H);
    }
    if (lc.mlp == DIS_MLP_DENSE) {
      const int ff = lc.ff, gr = L.gu_rows;
      ENG_CUDA(tensor(L.w_gu, (size_t)gr * ff * W, M.f32));
      ENG_CUDA(tensor(L.w_down, (size_t)W * ff, M.f32));
      if (gr == 2) name(pre + "mlp.gate", &L.w_gu, 0, {ff, W}, i);
      name(pre + "mlp.up", &L.w_gu, (size_t)(gr - 1) * ff * W, {ff, W}, i);
      name(pre + "mlp.down", &L.w_down, 0, {W, ff}, i);
      if (lc.mlp_act == DIS_ACT_CLAMPED) {  // the clamped unit carries biases, the gelu unit none
        ENG_CUDA(tensor(L.b_gu, (size_t)2 * ff, true));
        ENG_CUDA(tensor(L.b_down, (size_t)W, true));
        name(pre + "mlp.gate.b", &L.b_gu, 0, {ff}, i);
        name(pre + "mlp.up.b", &L.b_gu, (size_t)ff, {ff}, i);
        name(pre + "mlp.down.b", &L.b_down, 0, {W}, i);
      }
      max_proj = std::max(max_proj, (size_t)gr * ff);
      max_act = std::max(max_act, (size_t)ff);
    } else if (lc.mlp == DIS_MLP_MOE) {
      const int ff = lc.ff, E = lc.experts, gr = L.gu_rows;
      const bool shared_gate = lc.shared_ff > 0 && !(lc.mlp_flags & DIS_MLP_SHARED_PLAIN);
      ENG_CUDA(tensor(L.w_gu, (size_t)E * gr * ff * W, M.f32));
      ENG_CUDA(tensor(L.w_down, (size_t)E * W * ff, M.f32));
      ENG_CUDA(tensor(L.router, (size_t)(E + (shared_gate ? 1 : 0)) * W, true));
      name(pre + "mlp.router", &L.router, 0, {E, W}, i);
      if (lc.route_kind == DIS_ROUTE_SIGMOID_GROUPS) {
        ENG_CUDA(tensor(L.correction, (size_t)E, true));
        name(pre + "mlp.correction", &L.correction, 0, {E}, i);
      }
      if (lc.shared_ff > 0) {  // the shared expert: a dense unit of its own size; the logit of its gate is one more router row
        const int sf = lc.shared_ff;
        ENG_CUDA(tensor(L.w_sgu, (size_t)gr * sf * W, M.f32));
        ENG_CUDA(tensor(L.w_sdown, (size_t)W * sf, M.f32));
        if (gr == 2) name(pre + "mlp.shared.gate", &L.w_sgu, 0, {sf, W}, i);
        name(pre + "mlp.shared.up", &L.w_sgu, (size_t)(gr - 1) * sf * W, {sf, W}, i);
        name(pre + "mlp.shared.down", &L.w_sdown, 0, {W, sf}, i);
        if (shared_gate) name(pre + "mlp.shared.sg", &L.router, (size_t)E * W, {1, W}, i);
        max_proj = std::max(max_proj, (size_t)gr * sf);
        max_act = std::max(max_act, (size_t)sf);
        max_sff = std::max(max_sff, (size_t)sf);
        any_shared = true;
      }
      for (int e = 0; e < E; e++) {
        const std::string ep = pre + "mlp.e" + std::to_string(e) + ".";
        if (gr == 2) name(ep + "gate", &L.w_gu, (size_t)e * 2 * ff * W, {ff, W}, i);
        name(ep + "up", &L.w_gu, ((size_t)e * gr * ff + (size_t)(gr - 1) * ff) * W, {ff, W}, i);
        name(ep + "down", &L.w_down, (size_t)e * W * ff, {W, ff}, i);
      }
      max_proj = std::max(max_proj, (size_t)lc.top * gr * ff);
      max_act = std::max(max_act, (size_t)lc.top * ff);
      max_top = std::max(max_top, lc.top);
      max_e = std::max(max_e, E);
    }
  }
  // scalar gains and convolution taps are named too; they land in small fp32 areas through views
  // (a view is a StackTensor that does not own its memory)
  for (int i = 0; i < sc->n_layers; i++) {
    StackLayer &L = M.layers[(size_t)i];
    const std::string pre = "l" + std::to_string(i) + ".";
    const char *gn[4] = {"norm1", "norm1b", "norm2", "norm2b"};
    for (int k = 0; k < 4 && !ln; k++) {
      if (k >= 2 && L.c.mlp == DIS_MLP_NONE) continue;
      StackTensor *v = new StackTensor();
      v->ptr = L.g4 + k; v->n = 1; v->f32 = true;
      scalars.push_back(v);
      name(pre + gn[k], v, 0, {}, i);
    }
    if (taps >= 1) {
      StackTensor *v = new StackTensor();
      v->ptr = L.canon1; v->n = (size_t)W * taps; v->f32 = true;
      scalars.push_back(v);
      name(pre + "canon1", v, 0, {W, taps}, i);
      if (L.c.mlp != DIS_MLP_NONE) {
        StackTensor *v2 = new StackTensor();
        v2->ptr = L.canon2; v2->n = (size_t)W * taps; v2->f32 = true;
        scalars.push_back(v2);
        name(pre + "canon2", v2, 0, {W, taps}, i);
      }
    }
  }
  if (!ln) {
    StackTensor *v = new StackTensor();
    v->ptr = M.final_g; v->n = 1; v->f32 = true;
    scalars.push_back(v);
    name("final.norm", v, 0, {}, -1);
  }
  // ---- recurrent state of every layer run (one slot per sequence)
  for (StackRun &R : M.runs) {
    const dis_layer_config &lc = M.layers[(size_t)R.layer].c;
    if (taps > 1) {
      ENG_CUDA(alloc(reinterpret_cast<void **>(&R.cstate1), slots * (taps - 1) * W * 4));
      if (lc.mlp != DIS_MLP_NONE) ENG_CUDA(alloc(reinterpret_cast<void **>(&R.cstate2), slots * (taps - 1) * W * 4));
    }
    if (lc.mixer == DIS_MIX_LIGHTNING) ENG_CUDA(alloc(reinterpret_cast<void **>(&R.state), slots * lc.heads * lc.dim * lc.vdim * 4));
    else if (lc.mixer == DIS_MIX_MINGRU) ENG_CUDA(alloc(reinterpret_cast<void **>(&R.state), slots * lc.width * 4));
    else if (lc.mixer == DIS_MIX_PARALLEL) ENG_CUDA(alloc(reinterpret_cast<void **>(&R.state), slots * lc.gla_heads * lc.gla_dim * lc.gla_vdim * 4));
    else if (lc.mixer == DIS_MIX_SSM) {
      ENG_CUDA(alloc(reinterpret_cast<void **>(&R.state), slots * lc.heads * lc.ssm_state * lc.vdim * 4));
      if (lc.conv_taps > 1) ENG_CUDA(alloc(reinterpret_cast<void **>(&R.conv_state), slots * (lc.conv_taps - 1) * M.layers[(size_t)R.layer].conv_ch * 4));
    }
  }
  M.views.assign(scalars.begin(), scalars.end());
  // ---- activations
  const size_t cap = (size_t)cap_tokens;
  ENG_CUDA(alloc(reinterpret_cast<void **>(&M.x), cap * n_streams * W * 4));
  if (sc->frame_flags & DIS_FRAME_POS_SINUS) {  // frequencies of the position vector, formed in double
    const double base = sc->pos_base > 0.f ? (double)sc->pos_base : 10000.0;
    std::vector<double> f((size_t)(W + 1) / 2);
    for (size_t k = 0; k < f.size(); k++) f[k] = std::pow(base, -2.0 * (double)k / (double)W);
    ENG_CUDA(alloc(reinterpret_cast<void **>(&M.pos_freq), f.size() * 8));
    ENG_CUDA(cudaMemcpy(M.pos_freq, f.data(), f.size() * 8, cudaMemcpyHostToDevice));
  }
  if (max_ssm) { M.ssm_ld = max_ssm; ENG_CUDA(alloc(reinterpret_cast<void **>(&M.ssm), cap * max_ssm * 4)); }
  ENG_CUDA(alloc(reinterpret_cast<void **>(&M.y), cap * W * 4));
  ENG_CUDA(alloc(reinterpret_cast<void **>(&M.hn), cap * W * 4));
  ENG_CUDA(alloc(&M.hc, cap * W * esz));
  ENG_CUDA(alloc(reinterpret_cast<void **>(&M.proj), cap * max_proj * 4));
  ENG_CUDA(alloc(reinterpret_cast<void **>(&M.mix), cap * max_mix * 4));
  ENG_CUDA(alloc(reinterpret_cast<void **>(&M.mix2), cap * max_mix * 4));
  ENG_CUDA(alloc(reinterpret_cast<void **>(&M.qf), cap * max_qf * 4));
  ENG_CUDA(alloc(&M.act, cap * max_act * esz));
  ENG_CUDA(alloc(&M.xr, (size_t)M.max_rows * W * esz));
  if (loop_proj) {
    ENG_CUDA(alloc(reinterpret_cast<void **>(&M.x0), cap * W * 4));
    ENG_CUDA(alloc(&M.xcat, cap * 2 * W * esz));
  }
  if (max_dec) ENG_CUDA(alloc(reinterpret_cast<void **>(&M.dec), cap * max_dec * 4));
  if (max_vrot) ENG_CUDA(alloc(reinterpret_cast<void **>(&M.vrot), cap * max_vrot * 4));
  if (stack_att_rec) {
    M.attn_part_elems = (size_t)2048 * stack_att_rec;  // (tokens x slices) of one pass
    ENG_CUDA(alloc(reinterpret_cast<void **>(&M.attn_part), M.attn_part_elems * 4));
  }
  if (stack_lat_rec && !M.f32 && stack_tc) {
    bool ok = true;
    size_t max_D = 0, max_r = 0;
    for (auto &L : M.layers)
      if (L.c.mixer == DIS_MIX_LATENT) {
        ok = ok && (L.c.kv_rank % 8 == 0) && ((L.c.kv_rank + L.c.rot_dim) % 8 == 0);
        max_D = std::max(max_D, (size_t)(L.c.kv_rank + L.c.rot_dim)); max_r = std::max(max_r, (size_t)L.c.kv_rank);
      }
    if (const char *g = getenv("DIS_STACK_LATENT_PRODUCTS")) ok = ok && atoi(g) != 0;
    if (ok) {
      M.lat_gemm = true;
      M.lat_ctx_cap = (m.max_ctx + 7) / 8 * 8;
      M.lat_s_elems = std::max((size_t)16 << 20, (size_t)64 * M.lat_ctx_cap);
      ENG_CUDA(alloc(reinterpret_cast<void **>(&M.lat_qb), cap * max_qf * 2));
      ENG_CUDA(alloc(reinterpret_cast<void **>(&M.lat_cg), (size_t)M.lat_ctx_cap * max_D * 2));
      ENG_CUDA(alloc(reinterpret_cast<void **>(&M.lat_cgt), (size_t)M.lat_ctx_cap * max_r * 2));
      ENG_CUDA(alloc(reinterpret_cast<void **>(&M.lat_s), M.lat_s_elems * 4));
      ENG_CUDA(alloc(reinterpret_cast<void **>(&M.lat_p), M.lat_s_elems * 2));
    }
  }
  {
    // lightning: entry states of the segments of long spans (all layers share the buffer)
    size_t seg = 0, seg_a = 0;
    for (auto &L : M.layers) {
      if (L.c.mixer == DIS_MIX_LIGHTNING && L.c.dim <= 128 && L.c.vdim <= 128)
        seg = std::max(seg, stack_lightning_seg_floats(cap_tokens, max_batch, L.c.heads, L.c.dim, L.c.vdim));
      if (L.c.mixer == DIS_MIX_PARALLEL) {
        seg = std::max(seg, stack_lightning_seg_floats(cap_tokens, max_batch, L.c.gla_heads, L.c.gla_dim, L.c.gla_vdim));
        seg_a = std::max(seg_a, stack_lightning_seg_decay_floats(cap_tokens, max_batch, L.c.gla_heads, L.c.gla_dim));
      }
      if (L.c.mixer == DIS_MIX_SSM && L.c.ssm_state <= 128 && L.c.vdim <= 128) {
        seg = std::max(seg, stack_lightning_seg_floats(cap_tokens, max_batch, L.c.heads, L.c.ssm_state, L.c.vdim));
        seg_a = std::max(seg_a, stack_lightning_seg_decay_floats(cap_tokens, max_batch, L.c.heads, L.c.ssm_state));
      }
    }
    if (const char *g = getenv("DIS_STACK_LIGHT_SEGMENTS")) seg = atoi(g) != 0 ? seg : 0;
    if (seg) ENG_CUDA(alloc(reinterpret_cast<void **>(&M.light_seg), seg * 4));
    if (seg && seg_a) ENG_CUDA(alloc(reinterpret_cast<void **>(&M.light_seg_a), seg_a * 4));
  }
  if (stack_lat_rec) {
    M.lat_part_elems = (size_t)2048 * stack_lat_rec;  // (tokens x slices) of one pass
    ENG_CUDA(alloc(reinterpret_cast<void **>(&M.lat_part), M.lat_part_elems * 4));
  }
  if (const char *g = getenv("DIS_STACK_TC")) stack_tc = atoi(g) != 0;
  if (const char *g = getenv("DIS_STACK_PERSIST")) stack_persist = atoi(g) != 0;
  if (!M.f32 && stack_tc) {
    M.scratch_elems = 2 * cap * std::max(max_proj, (size_t)W);
    ENG_CUDA(alloc(reinterpret_cast<void **>(&M.scratch), M.scratch_elems * 4));
  }
  ENG_CUDA(alloc(reinterpret_cast<void **>(&M.logits), (size_t)M.max_rows * sc->vocab * 4));
  logits = nullptr;  // the Llama buffer is not allocated; last_logits reads stack->logits
  if (max_top > 0) {
    const size_t rows = cap * max_top;
    M.max_tiles = (int)((rows + kStackGemmTile - 1) / kStackGemmTile) + max_e;
    ENG_CUDA(alloc(reinterpret_cast<void **>(&M.r_idx), rows * 4));
    ENG_CUDA(alloc(reinterpret_cast<void **>(&M.r_wt), rows * 4));
    ENG_CUDA(alloc(reinterpret_cast<void **>(&M.counts), (size_t)max_e * 4));
    ENG_CUDA(alloc(reinterpret_cast<void **>(&M.perm_tok), rows * 4));
    ENG_CUDA(alloc(reinterpret_cast<void **>(&M.where), rows * 4));
    ENG_CUDA(alloc(reinterpret_cast<void **>(&M.tiles), (size_t)(1 + 3 * M.max_tiles) * 4));
    ENG_CUDA(alloc(reinterpret_cast<void **>(&M.rows_out), rows * W * 4));
    if (any_shared) {
      ENG_CUDA(alloc(reinterpret_cast<void **>(&M.y2), cap * W * 4));
      ENG_CUDA(alloc(reinterpret_cast<void **>(&M.r_sg), cap * 4));
      const char *lane = getenv("DIS_STACK_SHARED_LANE");  // 0: the shared expert runs in the pass's own stream (A/B runs)
      if (!(lane && atoi(lane) == 0)) {
        ENG_CUDA(alloc(reinterpret_cast<void **>(&M.sh_proj), cap * 2 * max_sff * 4));
        ENG_CUDA(alloc(&M.sh_act, cap * max_sff * esz));
        if (!M.f32 && stack_tc) {
          M.sh_scratch_elems = 2 * cap * std::max((size_t)2 * max_sff, (size_t)W);
          ENG_CUDA(alloc(reinterpret_cast<void **>(&M.sh_scratch), M.sh_scratch_elems * 4));
        }
        ENG_CUDA(cudaStreamCreateWithFlags(&M.sh_stream, cudaStreamNonBlocking));
        ENG_CUDA(cudaEventCreateWithFlags(&M.ev_sh_fork, cudaEventDisableTiming));
        ENG_CUDA(cudaEventCreateWithFlags(&M.ev_sh_join, cudaEventDisableTiming));
      }
    }
    if (!M.f32 && stack_tc) {
      ENG_CUDA(alloc(&M.moe_x, rows * W * 2));
      ENG_CUDA(cudaMallocHost(reinterpret_cast<void **>(&M.h_counts), (size_t)max_e * sizeof(int)));
      ENG_CUDA(cudaEventCreateWithFlags(&M.ev_fork, cudaEventDisableTiming));
      for (int i = 0; i < StackModel::kSide; i++) {
        ENG_CUDA(cudaStreamCreateWithFlags(&M.side[i], cudaStreamNonBlocking));
        ENG_CUDA(cudaEventCreateWithFlags(&M.ev_join[i], cudaEventDisableTiming));
      }
    }
  }
  ENG_CUDA(alloc(reinterpret_cast<void **>(&M.d_out), (size_t)2 * M.max_rows * 4));
  ENG_CUDA(cudaMallocHost(reinterpret_cast<void **>(&M.h_out), (size_t)2 * M.max_rows * 4));
  ENG_CUDA(stack_meta(meta_pre, cap_tokens, M.max_rows));
  cur_meta = &meta_pre;
  // ---- pages: one pool per latent layer that owns a cache (rows of kv_rank + rot_dim elements), a key and a value pool per
  // attention layer that owns one; a page id is valid in all
  {
    size_t row_bytes = 0;
    for (auto &R : M.runs) {
      const dis_layer_config &lc = M.layers[(size_t)R.layer].c;
      if (lc.mixer == DIS_MIX_LATENT && lc.kv_from < 0) row_bytes += (size_t)(lc.kv_rank + lc.rot_dim) * esz;
      if ((lc.mixer == DIS_MIX_ATTENTION || lc.mixer == DIS_MIX_PARALLEL) && lc.kv_from < 0) row_bytes += (size_t)lc.kv_heads * (lc.dim + lc.vdim) * esz;
    }
    int64_t want = c->kv_pages;
    const int64_t useful = (int64_t)max_batch * max_pages;
    if (want <= 0) {
      size_t free_b = 0, total_b = 0;
      ENG_CUDA(cudaMemGetInfo(&free_b, &total_b));
      const float frac = c->kv_mem_fraction > 0.f ? c->kv_mem_fraction : 0.85f;
      want = row_bytes ? (int64_t)((double)free_b * frac / (double)(row_bytes * page_size)) : useful;
      want = std::min(want, useful);
    }
    if (want < 1) return fail(DIS_ERR_OUT_OF_MEMORY, "no device memory left for the latent pages");
    n_pages = want;
    for (auto &R : M.runs) {
      const dis_layer_config &lc = M.layers[(size_t)R.layer].c;
      if (lc.mixer == DIS_MIX_LATENT && lc.kv_from < 0)
        ENG_CUDA(alloc(&R.pool, (size_t)n_pages * page_size * (lc.kv_rank + lc.rot_dim) * esz));
      if ((lc.mixer == DIS_MIX_ATTENTION || lc.mixer == DIS_MIX_PARALLEL) && lc.kv_from < 0) {
        ENG_CUDA(alloc(&R.kpool, (size_t)n_pages * page_size * lc.kv_heads * lc.dim * esz));
        ENG_CUDA(alloc(&R.vpool, (size_t)n_pages * page_size * lc.kv_heads * lc.vdim * esz));
      }
    }
    pages_ix.init(page_size, n_pages, false);
    ENG_CUDA(alloc(reinterpret_cast<void **>(&d_page_table), (size_t)max_batch * max_pages * 4));
    stack_allocs.pop_back();  // freed with the engine's own buffers
    ENG_CUDA(cudaMallocHost(reinterpret_cast<void **>(&h_page_table), (size_t)max_batch * max_pages * sizeof(int)));
    memset(h_page_table, 0, (size_t)max_batch * max_pages * sizeof(int));

  }
  seqs.resize((size_t)max_batch);
  slot_stamp.assign((size_t)max_batch, 0);
  if (const char *g = getenv("DIS_SAMPLER")) sampler_buckets = strcmp(g, "bisect") != 0;
  ENG_CUDA(cudaDeviceSynchronize());
  return DIS_OK;
}

// bf16 bit patterns or floats on the host -> the target's element type on the device, at an element offset
int Engine::load_named(const char *nm, const void *host, int dtype, const int64_t *shape, int ndim) {
  if (shut) return fail(DIS_ERR_SHUTDOWN, "engine is shut down");
  if (!stack) return fail(DIS_ERR_INVALID_ARGUMENT, "load_named: this engine holds a Llama model; use load_tensor");
  if (!nm || !host || (dtype != DIS_F32 && dtype != DIS_BF16) || ndim < 0 || (ndim > 0 && !shape))
    return fail(DIS_ERR_INVALID_ARGUMENT, "load_named: bad argument");
  auto it = stack_names.find(nm);
  if (it == stack_names.end()) return fail(DIS_ERR_INVALID_ARGUMENT, std::string("load_named: the configuration has no tensor '") + nm + "'");
  StackTarget &t = it->second;
  std::vector<int64_t> got(shape, shape + ndim);
  if (got != t.shape) return fail(DIS_ERR_INVALID_ARGUMENT, std::string("load_named: '") + nm + "' has the wrong shape");
  size_t n = 1;
  for (int64_t d : got) n *= (size_t)d;
  std::vector<float> f(n);
  if (dtype == DIS_F32) memcpy(f.data(), host, n * 4);
  else for (size_t i = 0; i < n; i++) f[i] = bf16_bits_to_float(reinterpret_cast<const uint16_t *>(host)[i]);
  if (t.transform == 1) {  // [H*d][r] -> per head [r][d]
    const dis_layer_config &lc = stack->layers[(size_t)t.layer].c;
    const size_t H = (size_t)lc.heads, d = (size_t)lc.dim, r = (size_t)lc.kv_rank;
    std::vector<float> g(n);
    for (size_t h = 0; h < H; h++)
      for (size_t a = 0; a < d; a++)
        for (size_t b = 0; b < r; b++) g[h * r * d + b * d + a] = f[(h * d + a) * r + b];
    f.swap(g);
  }
  ENG_CUDA(cudaSetDevice(cfg.device));
  // transform 2: the tensor is a block of columns of a wider matrix (row stride t.ld, first column t.off)
  const bool block = t.transform == 2 && got.size() == 2;
  const size_t cols = block ? (size_t)got[1] : n, rows = block ? (size_t)got[0] : 1, dpitch = block ? (size_t)t.ld : n;
  if (t.dst->f32) {
    float *dst = reinterpret_cast<float *>(t.dst->ptr) + t.off;
    if (block) ENG_CUDA(cudaMemcpy2D(dst, dpitch * 4, f.data(), cols * 4, cols * 4, rows, cudaMemcpyHostToDevice));
    else ENG_CUDA(cudaMemcpy(dst, f.data(), n * 4, cudaMemcpyHostToDevice));
  } else {
    std::vector<uint16_t> b(n);
    for (size_t i = 0; i < n; i++) b[i] = float_to_bf16_bits(f[i]);
    uint16_t *dst = reinterpret_cast<uint16_t *>(t.dst->ptr) + t.off;
    if (block) ENG_CUDA(cudaMemcpy2D(dst, dpitch * 2, b.data(), cols * 2, cols * 2, rows, cudaMemcpyHostToDevice));
    else ENG_CUDA(cudaMemcpy(dst, b.data(), n * 2, cudaMemcpyHostToDevice));
  }
  t.loaded = true;
  return DIS_OK;
}

int Engine::seq_extend(int slot, const uint32_t *tokens, int n, const int *probe, int n_probe) {
  if (shut) return fail(DIS_ERR_SHUTDOWN, "engine is shut down");
  if (!stack) return fail(DIS_ERR_INVALID_ARGUMENT, "seq_extend: only the layer-list family reads given tokens after the prompt");
  if (slot < 0 || slot >= max_batch || !seqs[(size_t)slot].used) return fail(DIS_ERR_INVALID_ARGUMENT, "seq_extend: no such sequence");
  if (n < 0 || (n > 0 && !tokens) || n_probe < 0 || (n_probe > 0 && !probe)) return fail(DIS_ERR_INVALID_ARGUMENT, "seq_extend: bad argument");
  Sequence &s = seqs[(size_t)slot];
  if ((long long)s.prompt.size() + n >= m.max_ctx) return fail(DIS_ERR_INVALID_ARGUMENT, "seq_extend: the sequence would not fit the context window");
  for (int i = 0; i < n; i++)
    if (tokens[i] >= (uint32_t)m.vocab) return fail(DIS_ERR_INVALID_ARGUMENT, "seq_extend: token id out of vocabulary");
  const int base = (int)s.prompt.size();
  for (int i = 0; i < n_probe; i++) {
    if (probe[i] < 0 || probe[i] >= n || (i > 0 && probe[i] <= probe[i - 1])) return fail(DIS_ERR_INVALID_ARGUMENT, "seq_extend: probes must ascend inside the given tokens");
  }
  if (!ensure_pages(s, slot, base + n)) return fail(DIS_ERR_OUT_OF_MEMORY, "seq_extend: out of pages");
  s.prompt.insert(s.prompt.end(), tokens, tokens + n);
  for (int i = 0; i < n_probe; i++) s.probes.push_back(base + probe[i]);
  if (n > 0) {
    s.prefilled = false;                 // the token sampled at the old end, if any, is dropped: the caller gave the continuation
    if (s.finish == DIS_FINISH_LENGTH || s.finish == DIS_FINISH_STOP || s.finish == DIS_FINISH_STOP_SEQUENCE) s.finish = DIS_FINISH_NONE;
  }
  return DIS_OK;
}

int Engine::seq_probe(int slot, const int *pos, int n) {
  if (shut) return fail(DIS_ERR_SHUTDOWN, "engine is shut down");
  if (!stack) return fail(DIS_ERR_INVALID_ARGUMENT, "seq_probe: only the layer-list family keeps logits of prompt positions");
  if (slot < 0 || slot >= max_batch || !seqs[(size_t)slot].used || n < 0 || (n > 0 && !pos)) return fail(DIS_ERR_INVALID_ARGUMENT, "seq_probe: bad argument");
  Sequence &s = seqs[(size_t)slot];
  for (int i = 0; i < n; i++)
    if (pos[i] < s.len || pos[i] >= (int)s.prompt.size() || (i > 0 && pos[i] <= pos[i - 1]) || (!s.probes.empty() && pos[i] <= s.probes.back() && i == 0))
      return fail(DIS_ERR_INVALID_ARGUMENT, "seq_probe: positions must ascend, lie among the tokens not yet read, and follow earlier probes");
  s.probes.insert(s.probes.end(), pos, pos + n);
  return DIS_OK;
}

// One pass.  For this family Sequence::prompt is the whole token history: tokens [0, len) are in the state and the cache,
// [len, size) are waiting; a sequence with nothing waiting feeds the token it sampled last (which then joins the history).
int Engine::stack_step(int n, const int *slots, int max_prefill_tokens, uint32_t *out_tokens, int *out_finish, int *out_produced) {
  StackModel &M = *stack;
  if (n <= 0 || n > max_batch || !slots || !out_tokens || !out_finish || !out_produced) return fail(DIS_ERR_INVALID_ARGUMENT, "step: bad argument");
  const uint64_t stamp = ++call_stamp;
  for (int i = 0; i < n; i++) {
    if (slots[i] < 0 || slots[i] >= max_batch || !seqs[(size_t)slots[i]].used) return fail(DIS_ERR_INVALID_ARGUMENT, "step: no such sequence");
    if (slot_stamp[(size_t)slots[i]] == stamp) return fail(DIS_ERR_INVALID_ARGUMENT, "step: duplicate slot");
    slot_stamp[(size_t)slots[i]] = stamp;
  }
  ENG_CUDA(cudaSetDevice(cfg.device));
  std::vector<int> idx, rem;
  for (int i = 0; i < n; i++) {
    Sequence &s = seqs[(size_t)slots[i]];
    out_tokens[i] = 0; out_produced[i] = 0; out_finish[i] = s.finish;
    if (s.finish != DIS_FINISH_NONE) continue;
    const int waiting = (int)s.prompt.size() - s.len;
    if (waiting == 0 && (!s.prefilled || s.len + 1 > m.max_ctx || !ensure_pages(s, slots[i], s.len + 1))) {
      s.finish = DIS_FINISH_FAILED; out_finish[i] = s.finish; continue;
    }
    idx.push_back(i);
    rem.push_back(waiting);
  }
  if (idx.empty()) { last_rows = 0; return DIS_OK; }
  std::vector<int> take(idx.size());
  plan_mixed_step((int)idx.size(), rem.data(), max_prefill_tokens > 0 ? max_prefill_tokens : cap_tokens, cap_tokens, take.data());
  StepMeta &mt = meta_pre;
  int T = 0, R = 0, SP = 0, QB = 0, KB = 0;
  stack_max_ctx = 0;
  stack_spans_h.clear();
  bool all_greedy = true;
  // rows first: a pass that would produce more logits rows than the engine holds is refused before anything changes
  {
    long long rows = 0;
    for (size_t k = 0; k < idx.size(); k++) {
      const Sequence &s = seqs[(size_t)slots[idx[k]]];
      if (take[k] <= 0) continue;
      const int p0 = s.len, p1 = s.len + take[k];
      for (int p : s.probes) rows += (p >= p0 && p < p1) ? 1 : 0;
      rows += (rem[k] == 0 || p1 == (int)s.prompt.size()) ? 1 : 0;
    }
    if (rows > M.max_rows) return fail(DIS_ERR_INVALID_ARGUMENT, "step: more logits rows than max_logit_rows");
  }
  ENG_CUDA(cudaEventRecord(ev0, stream));
  for (size_t k = 0; k < idx.size(); k++) {
    const int i = idx[k];
    Sequence &s = seqs[(size_t)slots[i]];
    const int tk = take[k];
    if (tk <= 0) continue;
    if (rem[k] == 0) s.prompt.push_back(s.last_token);
    const int p0 = s.len;
    stack_max_ctx = std::max(stack_max_ctx, p0 + tk);
    for (int j = 0; j < tk; j++) {
      mt.h<uint32_t>(mt.o_tokens)[T + j] = s.prompt[(size_t)(p0 + j)];
      mt.h<int>(mt.o_pos)[T + j] = p0 + j;
      mt.h<int>(mt.o_ptrow)[T + j] = slots[i];
      mt.h<int>(mt.o_span)[T + j] = SP;
    }
    mt.h<int>(mt.o_qb_tok0)[SP] = T;
    mt.h<int>(mt.o_qb_len)[SP] = tk;
    mt.h<int>(mt.o_qb_pos0)[SP] = p0;
    mt.h<int>(mt.o_qb_ptrow)[SP] = slots[i];
    SP++;
    // long portions: latent attention as matrix products; short ones and decode rows: query blocks of the paged kernel
    const bool products = M.lat_gemm && tk >= 32 && (size_t)stack_lat_heads * ((p0 + tk + 7) / 8 * 8) <= M.lat_s_elems;
    stack_spans_h.push_back({T, tk, p0, slots[i], products});
    for (int j = 0; j < tk && !products; j += stack_bq) {
      mt.h<int>(mt.o_ab_tok0)[QB] = T + j;
      mt.h<int>(mt.o_ab_len)[QB] = std::min(stack_bq, tk - j);
      QB++;
    }
    for (int j = 0; j < tk && stack_abq > 0; j += stack_abq) {
      mt.h<int>(mt.o_kb_tok0)[KB] = T + j;
      mt.h<int>(mt.o_kb_len)[KB] = std::min(stack_abq, tk - j);
      KB++;
    }
    auto row = [&](int tok, float temp, float topp, uint64_t seed, uint64_t step) {
      mt.h<int>(mt.o_rowmap)[R] = tok;
      mt.h<float>(mt.o_temp)[R] = temp;
      mt.h<float>(mt.o_topp)[R] = topp;
      mt.h<unsigned long long>(mt.o_seed)[R] = seed;
      mt.h<unsigned long long>(mt.o_step)[R] = step;
      R++;
    };
    for (int p : s.probes)
      if (p >= p0 && p < p0 + tk) row(T + (p - p0), 0.f, 1.f, 0, 0);
    if (p0 + tk == (int)s.prompt.size()) {
      row(T + tk - 1, s.temperature, s.top_p, s.seed, (uint64_t)s.generated);
      all_greedy = all_greedy && s.temperature <= 0.f;
    }
    T += tk;
  }
  if (T == 0) { last_rows = 0; return DIS_OK; }
  if (pt_dirty) {
    ENG_CUDA(cudaMemcpyAsync(d_page_table, h_page_table, (size_t)max_batch * max_pages * sizeof(int), cudaMemcpyHostToDevice, stream));
    pt_dirty = false;
  }
  ENG_CUDA(cudaMemcpyAsync(mt.dev, mt.host, mt.bytes, cudaMemcpyHostToDevice, stream));
  // latent attention: with few query blocks the history is cut into slices so that about two CTAs per SM run
  stack_lat_split = 1; stack_lat_keys = 0;
  if (QB > 0 && QB < kNumSMs && stack_max_ctx >= 256 && stack_lat_rec) {
    int sp = std::min(std::min((2 * kNumSMs + QB - 1) / QB, stack_max_ctx / (stack_lat_mma ? 64 : 32)), 64);  // a slice holds at least one tile of keys
    const int keys = ((stack_max_ctx + sp - 1) / sp + 31) / 32 * 32;
    sp = (stack_max_ctx + keys - 1) / keys;
    if (sp > 1 && (size_t)sp * T * stack_lat_rec <= M.lat_part_elems) { stack_lat_split = sp; stack_lat_keys = keys; }
  }
  // paged attention likewise: one CTA per (query block, key/value head, slice).  A layer with a chunked mask walks at most
  // its chunk (plus the block's own tokens) whatever the history's length, so it slices by that bound.
  stack_kb = KB;
  auto att_slices = [&](int ctx) -> std::pair<int, int> {
    if (!(KB > 0 && KB * stack_att_groups < kNumSMs && ctx >= 256 && stack_att_rec)) return {1, 0};
    int sp = std::min(std::min((2 * kNumSMs + KB * stack_att_groups - 1) / (KB * stack_att_groups), ctx / 64), 64);
    if (sp <= 1) return {1, 0};
    const int keys = ((ctx + sp - 1) / sp + 31) / 32 * 32;
    sp = (ctx + keys - 1) / keys;
    if (sp > 1 && (size_t)sp * T * stack_att_rec <= M.attn_part_elems) return {sp, keys};
    return {1, 0};
  };
  {
    const std::pair<int, int> whole = att_slices(stack_max_ctx);
    stack_att_split = whole.first; stack_att_keys = whole.second;
    stack_att_plan.assign(M.layers.size(), whole);
    for (size_t li = 0; li < M.layers.size(); li++) {
      const dis_layer_config &lc = M.layers[li].c;
      if (!(lc.mixer == DIS_MIX_ATTENTION || lc.mixer == DIS_MIX_PARALLEL)) continue;
      long long bound = stack_max_ctx;  // keys a query block can reach at most
      if (lc.mask_chunk > 0) bound = std::min(bound, (long long)lc.mask_chunk + stack_abq);
      if (lc.mask_window > 0) bound = std::min(bound, (long long)lc.mask_window + stack_abq);
      if (bound < stack_max_ctx) stack_att_plan[li] = att_slices((int)bound);
    }
  }
  // A pass of single tokens only (decode rows, no kept prompt positions) has the same launches whenever its size, its
  // slicing and its sampler agree: the second such pass is captured into a CUDA graph and later ones replay it.
  const bool graphable = !(cfg.flags & DIS_FLAG_NO_GRAPH) && T == SP && R == T && T <= 0xFFFF;
  if (!graphable) {
    ENG_CUDA(stack_forward(T, SP, QB, R, all_greedy));
  } else {
    // the pass's shape and every layer's slicing name the graph; `graphs` is keyed by the order in which they were first seen
    std::vector<uint64_t> shape{(uint64_t)T | ((uint64_t)stack_lat_split << 16) | ((uint64_t)(stack_lat_keys / 32) << 24) | (all_greedy ? 1ull << 60 : 0ull)};
    for (auto &pl : stack_att_plan) shape.push_back((uint64_t)pl.first | ((uint64_t)pl.second << 8));
    const uint64_t key = stack_graph_ids.emplace(shape, (uint64_t)stack_graph_ids.size()).first->second;
    auto it = graphs.find(key);
    if (it != graphs.end() && it->second) {
      ENG_CUDA(cudaGraphLaunch(it->second, stream));
      kernel_launches += graph_launches[key];
    } else if (it == graphs.end()) {
      if (graphs.size() > 256) {  // histories that grow through many slicings: start over rather than keep every graph
        for (auto &g : graphs) if (g.second) cudaGraphExecDestroy(g.second);
        graphs.clear();  // (the ids stay: an id names one shape for the engine's life)
      }
      const uint64_t before = kernel_launches;
      ENG_CUDA(stack_forward(T, SP, QB, R, all_greedy));  // first sight: plain launches (function attributes, tensor maps)
      graph_launches[key] = kernel_launches - before;
      graphs.emplace(key, nullptr);
    } else {
      const uint64_t before = kernel_launches;
      cudaGraph_t g = nullptr;
      ENG_CUDA(cudaStreamBeginCapture(stream, cudaStreamCaptureModeThreadLocal));
      stack_capturing = true;
      const cudaError_t e1 = stack_forward(T, SP, QB, R, all_greedy);
      stack_capturing = false;
      const cudaError_t e2 = cudaStreamEndCapture(stream, &g);
      if (e1 != cudaSuccess || e2 != cudaSuccess || !g) {
        if (g) cudaGraphDestroy(g);
        cudaGetLastError();
        healthy = false;
        return fail(DIS_ERR_INFERENCE_FAILED, std::string("decode graph capture failed: ") + cudaGetErrorString(e1 != cudaSuccess ? e1 : e2));
      }
      cudaGraphExec_t ex = nullptr;
      ENG_CUDA(cudaGraphInstantiate(&ex, g, 0));
      cudaGraphDestroy(g);
      kernel_launches = before + graph_launches[key];
      it->second = ex;
      ENG_CUDA(cudaGraphLaunch(ex, stream));
    }
  }
  if (R > 0) ENG_CUDA(cudaMemcpyAsync(M.h_out, M.d_out, (size_t)2 * M.max_rows * 4, cudaMemcpyDeviceToHost, stream));
  ENG_CUDA(cudaEventRecord(ev1, stream));
  ENG_CUDA(cudaEventSynchronize(ev1));
  float ms = 0.f;
  ENG_CUDA(cudaEventElapsedTime(&ms, ev0, ev1));
  last_step_ms = ms;
  last_rows = R;
  last_T = T;
  int r = 0;
  for (size_t k = 0; k < idx.size(); k++) {
    const int i = idx[k];
    Sequence &s = seqs[(size_t)slots[i]];
    const int tk = take[k];
    if (tk <= 0) continue;
    const int p0 = s.len;
    s.len += tk;
    s.prefill_pos = s.len;
    size_t keep = 0;
    for (int p : s.probes) {
      if (p >= p0 && p < s.len) r++;
      else s.probes[keep++] = p;
    }
    s.probes.resize(keep);
    if (s.len < (int)s.prompt.size()) continue;  // more chunks to come
    s.prefilled = true;
    out_tokens[i] = M.h_out[r];
    s.last_logprob = reinterpret_cast<const float *>(M.h_out + M.max_rows)[r];
    finish_check(s, M.h_out[r]);
    out_finish[i] = s.finish;
    out_produced[i] = 1;
    r++;
  }
  return DIS_OK;
}

cudaError_t Engine::stack_forward(int T, int n_spans, int n_qb, int R, bool all_greedy) {
  StackModel &M = *stack;
  StepMeta &mt = meta_pre;
  const int W = M.c.width, taps = M.c.canon_taps;
  const float eps = M.c.norm_eps;
  const bool f32 = M.f32;
  StackSpans sp{mt.d<uint32_t>(mt.o_tokens), mt.d<int>(mt.o_pos), mt.d<int>(mt.o_ptrow), mt.d<int>(mt.o_span),
                mt.d<int>(mt.o_qb_tok0), mt.d<int>(mt.o_qb_len), mt.d<int>(mt.o_qb_pos0), mt.d<int>(mt.o_qb_ptrow), T, n_spans};
  uint64_t &kl = kernel_launches;
  int pend_parts = 1;  // the product whose result the next boundary consumes: slices left unsummed, their stride, its bias
  long long pend_stride = 0;
  const float *pend_bias = nullptr, *pend_src = nullptr;
  pdl_enabled() = false;  // this family's kernels are plain launches: every kernel starts after the one before it has ended
  // Dense projection out[Mrows][N] = A[Mrows][K] W[N][K]^T (+ bias).  bf16 operands go to the tcgen05 product the Llama path
  // uses (fp32 accumulation in TMEM; split-K slices summed, with the bias, by one more kernel); float operands, and shapes a
  // TMA map cannot describe (K not a multiple of 8), to the fp32-FMA product.  a_rows: rows the buffer behind A holds.
  // later_bias: the caller's next kernel can add the bias itself; it is set to the bias when this product left it out (a
  // single-slice tensor-core product, which has no pass of its own over the result) and to null when it is already in.
  // The lane a product runs in: its stream and the room for its split-K slices.  Everything runs in the pass's own lane except
  // a shared expert, which runs beside the router and the experts in a lane of its own (stream, slices, gate | up and
  // activation buffers), forked off the pass's stream and joined in front of the combine kernel.
  cudaStream_t cur_st = stream;
  float *cur_scratch = M.scratch, *cur_proj = M.proj;
  size_t cur_scratch_elems = M.scratch_elems;
  void *cur_act = M.act;
  auto gemm = [&](const void *A, bool a_f32, long long lda, const StackTensor &Wt, size_t w_off, const float *bias, float *out,
                  int Mrows, int N, int K, int a_rows = 0, const float **later_bias = nullptr, bool later_sum = false) -> cudaError_t {
    if (later_bias) *later_bias = nullptr;
    pend_parts = 1; pend_stride = 0; pend_bias = nullptr;
    if (stack_tc && !f32 && !a_f32 && !Wt.f32 && a_rows > 0 && K % 8 == 0 && lda == K && (w_off * 2) % 16 == 0) {
      const TmaMap *xm = stack_map(A, (uint64_t)a_rows, (uint64_t)K, (uint32_t)gemm_token_tile(Mrows));
      const TmaMap *wm = stack_map(reinterpret_cast<const uint16_t *>(Wt.ptr) + w_off, (uint64_t)N, (uint64_t)K, 128);
      if (!xm || !wm) return cudaErrorInvalidValue;
      int s = gemm_pick_split_k(Mrows, N, K);
      if ((size_t)s * Mrows * N > cur_scratch_elems) s = 1;
      kl++;
      if (s == 1 && bias && later_bias) { *later_bias = bias; bias = nullptr; }
      if (s == 1 && !bias) {
        // prompt-sized products with at least two tiles per SM: the persistent kernel (one CTA per SM walks the tiles, the
        // accumulator double-buffered in TMEM), as the Llama path does
        if (stack_persist && gemm_use_persist(Mrows, N, false)) {
          const TmaMap *xm256 = stack_map(A, (uint64_t)a_rows, (uint64_t)K, 256);
          if (!xm256) return cudaErrorInvalidValue;
          return launch_gemm_persist_partial(*wm, *xm256, out, Mrows, N, K, 0, cur_st);
        }
        return launch_gemm_partial(*wm, *xm, out, Mrows, N, K, 0, 1, cur_st);
      }
      if ((size_t)s * Mrows * N > cur_scratch_elems) return cudaErrorInvalidValue;
      RET_CUDA(launch_gemm_partial(*wm, *xm, cur_scratch, Mrows, N, K, 0, s, cur_st));
      if (later_sum) {  // the boundary kernel of a single-token pass sums the slices and adds the bias
        pend_parts = s; pend_stride = (long long)Mrows * N; pend_bias = bias; pend_src = cur_scratch;
        return cudaSuccess;
      }
      kl++;
      return launch_stack_sum_bias(cur_scratch, s, (long long)Mrows * N, bias, out, Mrows, N, cur_st);
    }
    StackGemm g;
    g.A = A; g.a_f32 = a_f32; g.lda = lda;
    g.W = Wt.f32 ? (const void *)(reinterpret_cast<const float *>(Wt.ptr) + w_off) : (const void *)(reinterpret_cast<const uint16_t *>(Wt.ptr) + w_off);
    g.w_f32 = Wt.f32; g.ldw = K;
    g.out = out; g.ldo = N; g.bias = bias; g.M = Mrows; g.N = N; g.K = K;
    kl++;
    return launch_stack_gemm(g, cur_st);
  };
  const bool pre_frame = (M.c.frame_flags & DIS_FRAME_PRE_NORM) != 0;  // x += f(norm(x)), over residual streams where the model has them
  const int n_streams = std::max(1, M.c.streams);
  RET_CUDA(launch_stack_embed(M.embed.ptr, f32, sp.tokens, sp.pos, M.pos_freq, M.x, M.x0, M.c.embed_scale, T, W, n_streams, stream)); kl++;
  const float *pend_y = nullptr, *pend_post = nullptr, *pend_post_b = nullptr;
  const float *pend_hc = nullptr, *next_hc = nullptr;  // stream coefficients of the sublayer whose product is pending / of the coming one
  const bool ln = M.c.norm_kind == DIS_NORM_LAYER || M.c.norm_kind == DIS_NORM_RMS;  // norms with vectors: one boundary kernel
  const bool rms = M.c.norm_kind == DIS_NORM_RMS;
  const bool single = T == n_spans;  // every span one token long: the fused boundary kernel
  // The boundary in front of a sublayer: the product before it joins the residual through its post norm, then the pre norm (and
  // the convolution) makes the sublayer's input.  pre == null: only the residual is updated.  cat: [x ; x0] is written too.
  auto sublayer_in = [&](const float *pre, const float *pre_b, const float *cw, float *cstate, bool cat = false) -> cudaError_t {
    if (pre_frame) {  // one kernel: the pending product joins the stream(s), the coming sublayer's input is read off and normed
      kl++;
      const float *src = pend_y ? (pend_parts > 1 || pend_bias ? pend_src : pend_y) : nullptr;
      const cudaError_t e = launch_stack_boundary_hc(M.x, n_streams, src, pend_parts, pend_stride, pend_bias, pend_hc, next_hc, pre, M.hc, f32, T,
                                                     W, eps, stream);
      pend_y = nullptr; pend_parts = 1; pend_bias = nullptr; pend_hc = nullptr;
      return e;
    }
    if (ln) {  // layer norms: one kernel for passes of any shape; it sums the slices of the product before and adds its bias
      kl++;
      const float *src = pend_y ? (pend_parts > 1 || pend_bias ? pend_src : pend_y) : nullptr;
      const bool conv = pre && taps >= 1;
      const cudaError_t e = launch_stack_boundary_ln(M.x, src, pend_parts, pend_stride, pend_bias, pend_post, pend_post_b, pre, pre_b,
                                                     conv ? M.hn : nullptr, conv ? nullptr : M.hc, M.x0, cat ? M.xcat : nullptr, f32, T, W,
                                                     eps, rms, stream);
      pend_y = nullptr; pend_parts = 1; pend_bias = nullptr;
      if (e != cudaSuccess || !conv) return e;
      kl += taps > 1 ? 2 : 1;
      return launch_stack_canon(M.hn, cw, cstate, sp, M.hc, f32, W, taps, stream);
    }
    if (cat) {  // scalar-gain norms in front of a loop pass: the residual update alone, then [x ; x0]
      if (single) {
        kl++;
        RET_CUDA(launch_stack_boundary_single(M.x, pend_y ? (pend_parts > 1 || pend_bias ? pend_src : pend_y) : nullptr, pend_parts, pend_stride,
                                              pend_bias, pend_post, nullptr, nullptr, nullptr, sp, M.hc, f32, W, taps, eps, stream));
        pend_parts = 1; pend_bias = nullptr;
      } else if (pend_y) { RET_CUDA(launch_stack_resid_norm(M.x, pend_y, pend_post, nullptr, nullptr, T, W, eps, stream)); kl++; }
      pend_y = nullptr;
      kl++;
      return launch_stack_boundary_ln(M.x, nullptr, 1, 0, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, M.x0, M.xcat, f32, T, W,
                                      eps, false, stream);
    }
    if (single) {
      kl++;
      const cudaError_t e = launch_stack_boundary_single(M.x, pend_y ? (pend_parts > 1 || pend_bias ? pend_src : pend_y) : nullptr, pend_parts,
                                                         pend_stride, pend_bias, pend_post, pre, cw, cstate, sp, M.hc, f32, W, taps, eps, stream);
      pend_y = nullptr; pend_parts = 1; pend_bias = nullptr;
      return e;
    }
    RET_CUDA(launch_stack_resid_norm(M.x, pend_y, pend_post, pre, M.hn, T, W, eps, stream)); kl++;
    pend_y = nullptr;
    if (taps >= 1) { kl += taps > 1 ? 2 : 1; return launch_stack_canon(M.hn, cw, cstate, sp, M.hc, f32, W, taps, stream); }
    kl++;
    return launch_stack_copy_act(M.hn, M.hc, f32, (long long)T * W, stream);
  };
  const int lat_split = stack_lat_split, lat_keys = stack_lat_keys;
  const bool later = single || ln;  // the boundary kernel of the next sublayer sums a product's slices and adds its bias
  auto norm_w = [&](StackLayer &L, int k) { return ln ? reinterpret_cast<const float *>(L.ln_w[k].ptr) : L.g4 + k; };
  auto norm_b = [&](StackLayer &L, int k) { return ln ? reinterpret_cast<const float *>(L.ln_b[k].ptr) : nullptr; };
  int max_span = 0;
  for (auto &sh : stack_spans_h) max_span = std::max(max_span, sh.len);
  // A dense gated unit out = W_down act(W_gate h, W_up h) on the sublayer input M.hc.  later: the slices of the down projection
  // may stay unsummed for the next boundary kernel (out is then M.y, as the caller expects).
  auto dense_ff = [&](const StackTensor &w_gu, const StackTensor &b_gu, const StackTensor &w_down, const StackTensor &b_down, int ff,
                      int act_kind, float limit, float *out, bool later_ok) -> cudaError_t {
    const int gu_rows = act_kind == DIS_ACT_RELU2 ? 1 : 2;  // an ungated unit has no gate rows
    // bf16, a unit without biases (gelu_tanh or SiLU gate), prompt-sized passes: gate and up run as one tensor-core product with
    // two accumulators whose epilogue writes act(gate) * up (the product the Llama path uses with SiLU).  Decode-sized passes
    // keep the split-K product below, whose slices the gated unit sums: at these widths a single pass over K leaves each CTA a
    // long thin loop (measured: 0.337 against 0.320 ms per step of four layers at width 1024).
    if (stack_tc && !f32 && (act_kind == DIS_ACT_GELU_TANH || act_kind == DIS_ACT_SILU) && !b_gu.ptr && W % 8 == 0 && !w_gu.f32 &&
        gemm_token_tile(T) >= 128) {
      const int tc_act = act_kind == DIS_ACT_GELU_TANH ? 1 : 0;
      if (stack_persist && gemm_use_persist(T, ff, true)) {  // paired gate / up tiles on the persistent kernel
        const TmaMap *xm = stack_map(M.hc, (uint64_t)cap_tokens, (uint64_t)W, 256);
        const TmaMap *wm = stack_map(w_gu.ptr, (uint64_t)2 * ff, (uint64_t)W, 64);
        if (!xm || !wm) return cudaErrorInvalidValue;
        RET_CUDA(launch_gemm_persist_glu(*wm, *xm, reinterpret_cast<uint16_t *>(cur_act), T, ff, W, 0, tc_act, cur_st));
      } else {
        const int tr = 128;
        const TmaMap *xm = stack_map(M.hc, (uint64_t)cap_tokens, (uint64_t)W, (uint32_t)gemm_token_tile(T));
        const TmaMap *wm = stack_map(w_gu.ptr, (uint64_t)2 * ff, (uint64_t)W, (uint32_t)tr);
        if (!xm || !wm) return cudaErrorInvalidValue;
        RET_CUDA(launch_gemm_glu(*wm, *xm, reinterpret_cast<uint16_t *>(cur_act), T, ff, W, 0, tr, tc_act, cur_st));
      }
      kl++;
      return gemm(cur_act, f32, ff, w_down, 0, nullptr, out, T, W, ff, cap_tokens, nullptr, later_ok);
    }
    // an ungated unit in prompt-sized bf16 passes: the persistent product's epilogue squares the relu and writes bf16
    if (stack_tc && stack_persist && !f32 && act_kind == DIS_ACT_RELU2 && !b_gu.ptr && W % 8 == 0 && !w_gu.f32 && gemm_use_persist(T, ff, false)) {
      const TmaMap *xm = stack_map(M.hc, (uint64_t)cap_tokens, (uint64_t)W, 256);
      const TmaMap *wm = stack_map(w_gu.ptr, (uint64_t)ff, (uint64_t)W, 128);
      if (!xm || !wm) return cudaErrorInvalidValue;
      RET_CUDA(launch_gemm_persist_relu2(*wm, *xm, reinterpret_cast<uint16_t *>(cur_act), T, ff, W, 0, cur_st));
      kl++;
      return gemm(cur_act, f32, ff, w_down, 0, nullptr, out, T, W, ff, cap_tokens, nullptr, later_ok);
    }
    // the gated unit sums the slices of its input product itself and adds the bias the product left out
    const float *gu_bias = nullptr;
    RET_CUDA(gemm(M.hc, f32, W, w_gu, 0, reinterpret_cast<const float *>(b_gu.ptr), cur_proj, T, gu_rows * ff, W, cap_tokens, &gu_bias, true));
    const bool sliced = pend_parts > 1 || pend_bias;
    RET_CUDA(launch_stack_glu(sliced ? pend_src : cur_proj, sliced ? pend_parts : 1, pend_stride, sliced ? pend_bias : gu_bias, cur_act, f32, nullptr,
                              T, ff, limit, act_kind, cur_st));
    kl++;
    pend_parts = 1; pend_bias = nullptr;
    return gemm(cur_act, f32, ff, w_down, 0, reinterpret_cast<const float *>(b_down.ptr), out, T, W, ff, cap_tokens, nullptr, later_ok);
  };
  for (size_t ri = 0; ri < M.runs.size(); ri++) {
    StackRun &Rn = M.runs[ri];
    StackLayer &L = M.layers[(size_t)Rn.layer];
    const dis_layer_config &lc = L.c;
    if (Rn.loop_pass >= 0 && !(M.c.frame_flags & DIS_FRAME_LOOP_PLAIN)) {
      // in front of a loop pass: x = loop_in [x ; x0] + loop_step[pass].  The boundary kernel adds the product before to the
      // residual and writes [x ; x0]; the projection's result (with the pass's vector as its bias) replaces the residual.
      RET_CUDA(sublayer_in(nullptr, nullptr, nullptr, nullptr, true));
      RET_CUDA(gemm(M.xcat, f32, 2 * W, M.loop_in, 0, reinterpret_cast<const float *>(M.loop_step.ptr) + (size_t)Rn.loop_pass * W, M.x, T, W,
                    2 * W, cap_tokens));
    }
    next_hc = reinterpret_cast<const float *>(L.hc[0].ptr);
    RET_CUDA(sublayer_in(norm_w(L, 0), norm_b(L, 0), L.canon1, Rn.cstate1));
    const int N = L.n_in;
    const float *in_bias = nullptr;  // minGRU adds its projections' biases itself when the product left them out
    const bool is_attn = lc.mixer == DIS_MIX_ATTENTION || lc.mixer == DIS_MIX_PARALLEL;
    // a plain attention mixer's preparation kernel sums the slices of a split-K input projection itself
    const bool prep_sums = lc.mixer == DIS_MIX_ATTENTION;
    RET_CUDA(gemm(M.hc, f32, W, L.w_in, 0, L.b_in.ptr ? reinterpret_cast<const float *>(L.b_in.ptr) : nullptr, M.proj, T, N, W, cap_tokens,
                  lc.mixer == DIS_MIX_MINGRU || is_attn ? &in_bias : nullptr, prep_sums));
    const float *in_src = M.proj;
    int in_parts = 1;
    long long in_stride = 0;
    if (prep_sums && (pend_parts > 1 || pend_bias)) { in_src = pend_src; in_parts = pend_parts; in_stride = pend_stride; in_bias = pend_bias; }
    pend_parts = 1; pend_bias = nullptr;
    int n_mix = 0;
    const float *o_bias = nullptr;
    if (lc.mixer == DIS_MIX_LIGHTNING) {
      const int H = lc.heads, d = lc.dim, dv = lc.vdim;
      int max_len = 0;
      for (auto &sh : stack_spans_h) max_len = std::max(max_len, sh.len);
      const bool segments = M.light_seg && stack_lightning_segmented(sp.n_spans, T, H, max_len) && d <= 128 && dv <= 128;
      RET_CUDA(launch_stack_lightning(M.proj, N, reinterpret_cast<const float *>(L.decay_d.ptr), Rn.state, sp, M.mix, H, d, dv,
                                      segments ? M.light_seg : nullptr, max_len, stream));
      if (segments) kl += 2;
      RET_CUDA(launch_stack_norm_gate(M.mix, reinterpret_cast<const float *>(L.norm_w.ptr), M.proj + L.g_off, N, M.act, f32, T, H * dv, eps, stream));
      kl += 2;
      n_mix = H * dv;
    } else if (lc.mixer == DIS_MIX_SSM) {
      const int H = lc.heads, P = lc.vdim, Ns = lc.ssm_state, G = lc.ssm_groups, C = L.conv_ch, inner = H * P;
      const long long ld_b = C;  // x | B | C
      float *dtv = M.dec + (size_t)T * H;  // the step sizes follow the decays
      const float *vec = reinterpret_cast<const float *>(L.ssm_vec.ptr);
      RET_CUDA(launch_stack_ssm_conv(M.proj, N, L.x_off, L.dt_off, C, H, lc.conv_taps, reinterpret_cast<const float *>(L.conv_w.ptr),
                                     reinterpret_cast<const float *>(L.conv_b.ptr), vec, Rn.conv_state, sp, M.ssm, ld_b, M.dec, dtv, stream));
      kl += lc.conv_taps > 1 && T != sp.n_spans ? 2 : 1;
      const bool segments = M.light_seg && M.light_seg_a && stack_lightning_segmented(sp.n_spans, T, H, max_span) && Ns <= 128 && P <= 128;
      RET_CUDA(launch_stack_ssd(M.ssm, ld_b, inner + G * Ns, inner, 0, H / G, M.dec, dtv, Rn.state, sp, M.mix, H, Ns, P, segments ? M.light_seg : nullptr,
                                segments ? M.light_seg_a : nullptr, max_span, stream));
      kl += segments ? 3 : 1;
      RET_CUDA(launch_stack_ssm_out(M.mix, M.ssm, ld_b, M.proj, N, vec + 2 * H, reinterpret_cast<const float *>(L.norm_w.ptr), lc.ssm_norm_groups,
                                    M.act, f32, T, H, P, eps, stream));
      kl++;
      n_mix = inner;
    } else if (lc.mixer == DIS_MIX_MINGRU) {
      int max_len = 0;
      for (auto &sh : stack_spans_h) max_len = std::max(max_len, sh.len);
      RET_CUDA(launch_stack_mingru(M.proj, N, in_bias, Rn.state, sp, M.act, f32, lc.width, max_len, stream)); kl++;
      n_mix = lc.width;
    } else if (is_attn) {
      const int H = lc.heads, G = lc.kv_heads, d = lc.dim, dv = lc.vdim;
      const bool par = lc.mixer == DIS_MIX_PARALLEL;
      StackAttn sa{H, G, d, dv, lc.rot_dims, lc.attn_flags, lc.scale, eps, lc.mask_chunk, lc.mask_window, lc.score_softcap};
      const float *qkn = reinterpret_cast<const float *>(L.qk_norm.ptr), *tpb = reinterpret_cast<const float *>(L.temp_pb.ptr);
      // the gains of the key norm follow those of the query norm: [H*d] then [G*d] (whole projection), or [d] then [d] (per head)
      const float *kn = qkn ? qkn + ((lc.attn_flags & DIS_ATTN_QK_NORM_HEAD) ? (size_t)d : (size_t)H * d) : nullptr;
      const bool own = lc.kv_from < 0;  // else: the keys and values of the layer named by kv_from, as its latest run cached them
      StackRun &KV = M.runs[(size_t)Rn.kv_run];
      // the gate logits are read by the attention kernel from M.proj: when the projection came as slices the preparation writes
      // their sums there
      const bool gated = (lc.attn_flags & DIS_ATTN_GATE) != 0;
      RET_CUDA(launch_stack_attn_prep(in_src, N, in_parts, in_stride, N, L.g_off, gated && in_src != M.proj ? M.proj + L.g_off : nullptr, N, L.q_off,
                                      L.k_off, L.v_off, in_bias, qkn, kn, L.freq, L.vfreq, sa, sp, M.qf, own ? Rn.kpool : nullptr,
                                      own ? Rn.vpool : nullptr, M.vrot, f32, d_page_table, max_pages, page_size, stream));
      const std::pair<int, int> slices = stack_att_plan[(size_t)Rn.layer];
      RET_CUDA(launch_stack_attn(M.qf, KV.kpool, KV.vpool, f32, tpb, tpb ? tpb + H : nullptr, reinterpret_cast<const float *>(L.sink.ptr), sa, sp,
                                 mt.d<int>(mt.o_kb_tok0), mt.d<int>(mt.o_kb_len), stack_kb, single ? 1 : stack_abq, d_page_table, max_pages,
                                 page_size, M.act, L.n_act, 0, par ? lc.mix_scale : 1.f, M.vrot, M.proj + L.g_off, N, slices.first,
                                 slices.second, M.attn_part, stream));
      kl += slices.first > 1 ? 3 : 2;
      if (par) {
        const int Hr = lc.gla_heads, dr = lc.gla_dim, dvr = lc.gla_vdim;
        RET_CUDA(launch_stack_gla_decay(M.proj, N, L.ga_off, L.a2.ptr, L.a2.f32, reinterpret_cast<const float *>(L.a2_b.ptr), T, Hr * dr,
                                        lc.gla_rank, lc.gla_tau, M.dec, stream));
        const bool segments = M.light_seg && M.light_seg_a && stack_lightning_segmented(sp.n_spans, T, Hr, max_span);
        RET_CUDA(launch_stack_gla(M.proj, N, L.gq_off, L.gk_off, L.gv_off, M.dec, Rn.state, sp, M.mix, Hr, dr, dvr,
                                  segments ? M.light_seg : nullptr, segments ? M.light_seg_a : nullptr, max_span, stream));
        RET_CUDA(launch_stack_headnorm_silu(M.mix, reinterpret_cast<const float *>(L.gla_norm.ptr), M.proj + L.gg_off, N, M.act, L.n_act,
                                            H * dv, lc.gla_scale, f32, T, Hr, dvr, eps, stream));
        kl += segments ? 5 : 3;
      }
      o_bias = reinterpret_cast<const float *>(L.b_o.ptr);
      n_mix = L.n_act;
    } else {
      const int H = lc.heads, d = lc.dim, dr = lc.rot_dim, dv = lc.vdim, r = lc.kv_rank, D = r + dr;
      StackLatent sl{H, d, dr, dv, r, lc.rot_dims, lc.rot_base, lc.scale, eps};
      StackRun &KV = M.runs[(size_t)Rn.kv_run];
      RET_CUDA(launch_stack_latent_prep(M.proj, N, L.q_off, L.dkv_off, lc.kv_from < 0 ? reinterpret_cast<const float *>(L.norm_w.ptr) : nullptr, sl, sp,
                                        M.qf, lc.kv_from < 0 ? Rn.pool : nullptr, f32, d_page_table, max_pages, page_size, stream));
      // absorbed queries: qf[t][h][0..r) = sum_a q[t][h][a] * uk[h*d + a][.]  (one batch entry per head).  Large bf16 passes:
      // one tensor-core product per head over the head's queries packed contiguously; else the batched fp32-FMA product.
      const bool head_tc = M.lat_gemm && T >= 256 && !L.ukT.f32 && !L.uv.f32 && d % 8 == 0 && ((size_t)r * d * 2) % 16 == 0 &&
                           ((size_t)dv * r * 2) % 16 == 0 && ((size_t)T * d * 2) % 16 == 0 && ((size_t)T * r * 2) % 16 == 0;
      if (head_tc) {
        RET_CUDA(launch_stack_heads_pack(M.proj, N, L.q_off, d + dr, d, T, H, M.lat_qb, stream));
        for (int h = 0; h < H; h++) {
          TmaMap xm;
          RET_CUDA(make_tma_map_2d(&xm, M.lat_qb + (size_t)h * T * d, (uint64_t)T, (uint64_t)d, (uint32_t)gemm_token_tile(T)));
          const TmaMap *wm = stack_map(reinterpret_cast<const uint16_t *>(L.ukT.ptr) + (size_t)h * r * d, (uint64_t)r, (uint64_t)d, 128);
          if (!wm) return cudaErrorInvalidValue;
          RET_CUDA(launch_gemm_partial(*wm, xm, M.mix2 + (size_t)h * T * r, T, r, d, 0, 1, stream));
        }
        RET_CUDA(launch_stack_heads_unpack(M.mix2, r, T, H, M.qf, (long long)H * D, 0, D, stream));
        kl += H + 1;
      } else {
        StackGemm g;
        g.A = M.proj + L.q_off; g.a_f32 = true; g.lda = N; g.a_bs = d + dr;
        g.W = L.ukT.ptr; g.w_f32 = L.ukT.f32; g.ldw = d; g.w_bs = (long long)r * d;
        g.out = M.qf; g.ldo = (long long)H * D; g.o_bs = D;
        g.M = T; g.N = r; g.K = d; g.batch = H;
        RET_CUDA(launch_stack_gemm(g, stream));
      }
      RET_CUDA(launch_stack_latent_attn(M.qf, KV.pool, f32, reinterpret_cast<const float *>(L.sink.ptr), sl, sp, mt.d<int>(mt.o_ab_tok0),
                                        mt.d<int>(mt.o_ab_len), n_qb, d_page_table, max_pages, page_size, M.mix, lat_split, lat_keys,
                                        M.lat_part, stream));
      if (lat_split > 1) kl++;
      bool any_products = false;
      for (auto &sh : stack_spans_h) any_products = any_products || sh.products;
      if (any_products) {
        RET_CUDA(launch_stack_copy_act(M.qf, M.lat_qb, false, (long long)T * H * D, stream)); kl++;
        for (auto &sh : stack_spans_h) {
          if (!sh.products) continue;
          const int ctx = sh.pos0 + sh.len, ctx8 = (ctx + 7) / 8 * 8;
          RET_CUDA(launch_stack_latent_gather(KV.pool, d_page_table + (size_t)sh.slot * max_pages, page_size, D, r, ctx, ctx8, M.lat_cg,
                                              M.lat_cgt, stream));
          kl++;
          const int max_nq = (int)std::min<size_t>(M.lat_s_elems / ((size_t)H * ctx8), 4096);
          for (int j = 0; j < sh.len; j += max_nq) {
            const int nq = std::min(max_nq, sh.len - j), rows = nq * H;
            const int nkeys = (sh.pos0 + j + nq + 7) / 8 * 8;  // keys the block's last query sees, rounded up (the rest are masked)
            TmaMap qm, cm, pm, ctm;
            RET_CUDA(make_tma_map_2d(&qm, M.lat_qb + (size_t)(sh.tok0 + j) * H * D, (uint64_t)rows, (uint64_t)D, (uint32_t)gemm_token_tile(rows)));
            RET_CUDA(make_tma_map_2d(&cm, M.lat_cg, (uint64_t)nkeys, (uint64_t)D, 128));
            RET_CUDA(launch_gemm_partial(cm, qm, M.lat_s, rows, nkeys, D, 0, 1, stream));
            RET_CUDA(launch_stack_latent_softmax(M.lat_s, rows, nkeys, reinterpret_cast<const float *>(L.sink.ptr), H, sh.pos0 + j, sl.scale,
                                                 M.lat_p, stream));
            RET_CUDA(make_tma_map_2d(&pm, M.lat_p, (uint64_t)rows, (uint64_t)nkeys, (uint32_t)gemm_token_tile(rows)));
            RET_CUDA(make_tma_map_2d(&ctm, M.lat_cgt, (uint64_t)r, (uint64_t)ctx8, 128));
            RET_CUDA(launch_gemm_partial(ctm, pm, M.mix + (size_t)(sh.tok0 + j) * H * r, rows, r, nkeys, 0, 1, stream));
            kl += 3;
          }
        }
      }
      // values: mix2[t][h][0..dv) = sum_b ol[t][h][b] * uv[h*dv + .][b]
      if (head_tc) {
        RET_CUDA(launch_stack_heads_pack(M.mix, (long long)H * r, 0, r, r, T, H, M.lat_qb, stream));
        for (int h = 0; h < H; h++) {
          TmaMap xm;
          RET_CUDA(make_tma_map_2d(&xm, M.lat_qb + (size_t)h * T * r, (uint64_t)T, (uint64_t)r, (uint32_t)gemm_token_tile(T)));
          const TmaMap *wm = stack_map(reinterpret_cast<const uint16_t *>(L.uv.ptr) + (size_t)h * dv * r, (uint64_t)dv, (uint64_t)r, 128);
          if (!wm) return cudaErrorInvalidValue;
          RET_CUDA(launch_gemm_partial(*wm, xm, M.mix2 + (size_t)h * T * dv, T, dv, r, 0, 1, stream));
        }
        RET_CUDA(launch_stack_gate(M.mix2, M.proj + L.g_off, N, M.act, f32, T, H * dv, H, stream));
        kl += H;
      } else {
        StackGemm v;
        v.A = M.mix; v.a_f32 = true; v.lda = (long long)H * r; v.a_bs = r;
        v.W = L.uv.ptr; v.w_f32 = L.uv.f32; v.ldw = r; v.w_bs = (long long)dv * r;
        v.out = M.mix2; v.ldo = (long long)H * dv; v.o_bs = dv;
        v.M = T; v.N = dv; v.K = r; v.batch = H;
        RET_CUDA(launch_stack_gemm(v, stream));
        RET_CUDA(launch_stack_gate(M.mix2, M.proj + L.g_off, N, M.act, f32, T, H * dv, 0, stream));
      }
      kl += 5;
      n_mix = H * dv;
    }
    RET_CUDA(gemm(M.act, f32, n_mix, L.w_o, 0, o_bias, M.y, T, W, n_mix, cap_tokens, nullptr, later));
    pend_y = M.y; pend_post = norm_w(L, 1); pend_post_b = norm_b(L, 1); pend_hc = reinterpret_cast<const float *>(L.hc[0].ptr);
    if (lc.mlp == DIS_MLP_NONE) continue;
    next_hc = reinterpret_cast<const float *>(L.hc[1].ptr);
    RET_CUDA(sublayer_in(norm_w(L, 2), norm_b(L, 2), L.canon2, Rn.cstate2));
    if (lc.mlp == DIS_MLP_DENSE) {
      RET_CUDA(dense_ff(L.w_gu, L.b_gu, L.w_down, L.b_down, lc.ff, lc.mlp_act, lc.limit, M.y, later));
    } else {
      const int ff = lc.ff, E = lc.experts, top = lc.top, rows = T * top;
      const int gc = L.gu_rows * ff;  // columns of an expert's first product: gate | up, or up alone
      const bool shared_gate = lc.shared_ff > 0 && !(lc.mlp_flags & DIS_MLP_SHARED_PLAIN);
      // the always-on unit beside the experts: its dense product first (it borrows the buffers the experts' rows use afterwards);
      // the logit of its per-token gate is one more row of the router matrix, and the combine kernel adds it in
      const bool shared = lc.shared_ff > 0;
      const float *sh_src = M.y2;
      int sh_parts = 1;
      long long sh_stride = 0;
      const bool sh_lane = shared && M.sh_stream != nullptr;
      if (shared) {
        if (sh_lane) {  // fork: the shared expert's launches go to its own stream and buffers
          RET_CUDA(cudaEventRecord(M.ev_sh_fork, stream));
          RET_CUDA(cudaStreamWaitEvent(M.sh_stream, M.ev_sh_fork, 0));
          cur_st = M.sh_stream; cur_scratch = M.sh_scratch; cur_scratch_elems = M.sh_scratch_elems; cur_proj = M.sh_proj; cur_act = M.sh_act;
        }
        const cudaError_t se = dense_ff(L.w_sgu, StackTensor(), L.w_sdown, StackTensor(), lc.shared_ff, lc.mlp_act, lc.limit, M.y2, true);
        cur_st = stream; cur_scratch = M.scratch; cur_scratch_elems = M.scratch_elems; cur_proj = M.proj; cur_act = M.act;
        RET_CUDA(se);
        if (pend_parts > 1) { sh_src = pend_src; sh_parts = pend_parts; sh_stride = pend_stride; }  // the combine kernel sums the slices
        pend_parts = 1; pend_bias = nullptr;
      }
      auto join_shared = [&]() -> cudaError_t {
        if (!sh_lane) return cudaSuccess;
        RET_CUDA(cudaEventRecord(M.ev_sh_join, M.sh_stream));
        return cudaStreamWaitEvent(stream, M.ev_sh_join, 0);
      };
      const float *router = reinterpret_cast<const float *>(L.router.ptr);
      RET_CUDA(launch_stack_route(M.hc, f32, router, T, W, E, top, lc.route_kind, reinterpret_cast<const float *>(L.correction.ptr), lc.route_groups,
                                  lc.route_keep, shared_gate ? router + (size_t)E * W : nullptr, M.r_sg, M.r_idx, M.r_wt, stream));
      RET_CUDA(launch_stack_moe_plan(M.r_idx, T, top, E, kStackGemmTile, M.counts, M.perm_tok, M.where, M.tiles, M.max_tiles, stream));
      // Large passes in bf16: one tensor-core product per expert over its rows.  The row counts come back to the host (one
      // small copy and a wait), so this path is not taken while a decode pass is being captured into a graph.
      const float *sh_gate = shared_gate ? M.r_sg : nullptr;  // null: the shared unit joins the sum as it is
      if (M.moe_x && !stack_capturing && rows >= 64 * E && W % 8 == 0 && ff % 8 == 0) {
        RET_CUDA(launch_stack_moe_gather(M.hc, M.perm_tok, M.moe_x, rows, W, stream));
        RET_CUDA(cudaMemcpyAsync(M.h_counts, M.counts, (size_t)E * sizeof(int), cudaMemcpyDeviceToHost, stream));
        RET_CUDA(cudaStreamSynchronize(stream));
        kl += 4;
        // An expert's rows are few against the GPU (its products fill a fraction of the SMs, or one wave and a bit), so the
        // experts run side by side: the pass's stream forks into kSide more, expert e keeps to stream e mod (kSide + 1) with its
        // gate | up product, its gated unit and its down product in order, and the streams join in front of the combine kernel.
        const bool forked = M.side[0] && !getenv("DIS_STACK_MOE_SERIAL");
        auto lane = [&](int e) { const int k = e % (StackModel::kSide + 1); return forked && k > 0 ? M.side[k - 1] : stream; };
        if (forked) {
          RET_CUDA(cudaEventRecord(M.ev_fork, stream));
          for (int k = 0; k < StackModel::kSide; k++) RET_CUDA(cudaStreamWaitEvent(M.side[k], M.ev_fork, 0));
        }
        int off = 0;
        for (int e = 0; e < E; e++) {
          const int cnt = M.h_counts[e];
          if (cnt <= 0) continue;
          cudaStream_t es = lane(e);
          TmaMap xm, am;
          RET_CUDA(make_tma_map_2d(&xm, reinterpret_cast<uint16_t *>(M.moe_x) + (size_t)off * W, (uint64_t)cnt, (uint64_t)W, (uint32_t)gemm_token_tile(cnt)));
          const TmaMap *wm = stack_map(reinterpret_cast<const uint16_t *>(L.w_gu.ptr) + (size_t)e * gc * W, (uint64_t)gc, (uint64_t)W, 128);
          if (!wm) return cudaErrorInvalidValue;
          RET_CUDA(launch_gemm_partial(*wm, xm, M.proj + (size_t)off * gc, cnt, gc, W, 0, 1, es));
          RET_CUDA(launch_stack_glu(M.proj + (size_t)off * gc, 1, 0, nullptr, reinterpret_cast<uint16_t *>(M.act) + (size_t)off * ff, f32, nullptr, cnt, ff,
                                    lc.limit, lc.mlp_act, es));
          RET_CUDA(make_tma_map_2d(&am, reinterpret_cast<uint16_t *>(M.act) + (size_t)off * ff, (uint64_t)cnt, (uint64_t)ff, (uint32_t)gemm_token_tile(cnt)));
          const TmaMap *dm = stack_map(reinterpret_cast<const uint16_t *>(L.w_down.ptr) + (size_t)e * W * ff, (uint64_t)W, (uint64_t)ff, 128);
          if (!dm) return cudaErrorInvalidValue;
          RET_CUDA(launch_gemm_partial(*dm, am, M.rows_out + (size_t)off * W, cnt, W, ff, 0, 1, es));
          off += cnt; kl += 3;
        }
        kl--;  // (the count above included one gated-unit launch over all rows)
        if (forked)
          for (int k = 0; k < StackModel::kSide; k++) {
            RET_CUDA(cudaEventRecord(M.ev_join[k], M.side[k]));
            RET_CUDA(cudaStreamWaitEvent(stream, M.ev_join[k], 0));
          }
        RET_CUDA(join_shared());
        RET_CUDA(launch_stack_moe_combine(M.rows_out, M.where, M.r_wt, shared ? sh_src : nullptr, sh_parts, sh_stride, sh_gate, M.y, T, W, top, stream));
        pend_y = M.y; pend_post = norm_w(L, 3); pend_post_b = norm_b(L, 3); pend_hc = reinterpret_cast<const float *>(L.hc[1].ptr);
        continue;
      }
      const int tiles_cap = std::min(M.max_tiles, (rows + kStackGemmTile - 1) / kStackGemmTile + E);
      StackGemm g;
      g.A = M.hc; g.a_f32 = f32; g.lda = W; g.a_gather = M.perm_tok;
      g.W = L.w_gu.ptr; g.w_f32 = L.w_gu.f32; g.ldw = W; g.w_bs = (long long)gc * W;
      g.out = M.proj; g.ldo = gc; g.M = rows; g.N = gc; g.K = W;
      g.tiles = M.tiles; g.max_tiles = tiles_cap;
      RET_CUDA(launch_stack_gemm(g, stream));
      StackGemm dn;
      dn.A = M.act; dn.a_f32 = f32; dn.lda = ff;
      dn.W = L.w_down.ptr; dn.w_f32 = L.w_down.f32; dn.ldw = ff; dn.w_bs = (long long)W * ff;
      dn.out = M.rows_out; dn.ldo = W; dn.M = rows; dn.N = W; dn.K = ff;
      dn.tiles = M.tiles; dn.max_tiles = tiles_cap;
      static const bool few_glu = getenv("DIS_STACK_FEW_GLU") && atoi(getenv("DIS_STACK_FEW_GLU")) != 0;  // opt-in: measured slower (0.547 against 0.534 ms per step)
      if (few_glu && L.gu_rows == 2 && stack_gemm_few_rows(dn)) {  // a handful of rows: the down product's loader applies the gated unit to the gate | up rows
        dn.A = M.proj; dn.a_f32 = true; dn.lda = 2 * ff; dn.a_glu = lc.mlp_act + 1; dn.a_limit = lc.limit;
        kl--;
      } else RET_CUDA(launch_stack_glu(M.proj, 1, 0, nullptr, M.act, f32, nullptr, rows, ff, lc.limit, lc.mlp_act, stream));
      RET_CUDA(launch_stack_gemm(dn, stream));
      RET_CUDA(join_shared());
      RET_CUDA(launch_stack_moe_combine(M.rows_out, M.where, M.r_wt, shared ? sh_src : nullptr, sh_parts, sh_stride, sh_gate, M.y, T, W, top, stream));
      kl += 6;
    }
    pend_y = M.y; pend_post = norm_w(L, 3); pend_post_b = norm_b(L, 3); pend_hc = reinterpret_cast<const float *>(L.hc[1].ptr);
  }
  next_hc = nullptr;
  // the last sublayer's output joins the residual; rows that need logits get the final norm and the head
  if (single || ln) RET_CUDA(sublayer_in(nullptr, nullptr, nullptr, nullptr));
  else { RET_CUDA(launch_stack_resid_norm(M.x, pend_y, pend_post, nullptr, nullptr, T, W, eps, stream)); kl++; }
  if (R <= 0) return cudaSuccess;
  if (ln) RET_CUDA(launch_stack_final_ln(M.x, mt.d<int>(mt.o_rowmap), reinterpret_cast<const float *>(M.final_w.ptr),
                                         rms ? nullptr : reinterpret_cast<const float *>(M.final_b.ptr), M.xr, f32, R, W, eps, M.c.logit_scale,
                                         n_streams, stream));
  else RET_CUDA(launch_stack_final_norm(M.x, mt.d<int>(mt.o_rowmap), M.final_g, M.xr, f32, R, W, eps, stream));
  kl++;
  RET_CUDA(gemm(M.xr, f32, W, M.head, 0, nullptr, M.logits, R, M.c.vocab, W, M.max_rows));
  if (!ln && M.c.logit_scale != 1.f) { RET_CUDA(launch_stack_scale(M.logits, (long long)R * M.c.vocab, M.c.logit_scale, stream)); kl++; }
  if (M.c.logit_softcap > 0.f) { RET_CUDA(launch_stack_softcap(M.logits, (long long)R * M.c.vocab, M.c.logit_softcap, stream)); kl++; }
  const float *temp = mt.d<float>(mt.o_temp), *topp = mt.d<float>(mt.o_topp);
  const unsigned long long *seed = mt.d<unsigned long long>(mt.o_seed), *step = mt.d<unsigned long long>(mt.o_step);
  float *d_logprob = reinterpret_cast<float *>(M.d_out + M.max_rows);
  kl++;
  if (!all_greedy && sampler_buckets) {
    TpSampPeers solo{};
    solo.rank = 0; solo.tp = 1; solo.cap_rows = M.max_rows;
    return launch_tp_sample(solo, M.logits, M.c.vocab, R, M.c.vocab, temp, topp, seed, step, nullptr, 0, M.d_out, d_logprob, stream);
  }
  return launch_sample(M.logits, M.c.vocab, R, M.c.vocab, temp, topp, seed, step, M.d_out, 0, nullptr, nullptr, d_logprob, stream);
}

}  // namespace dis
