// k_stack_mix.cu -- the token mixers of the layer-list decoders: the decayed linear-attention scan, the minimal gated recurrence,
// and latent attention (query absorption happens in a batched matrix product in stack.cu; here: rotary + cache write, and the
// attention itself over the paged latents).  States and scores are fp32.
#include <cstdlib>
#include "stack_dev.cuh"

namespace dis {

__device__ __forceinline__ float silu_(float v) { return v / (1.f + expf(-v)); }

// ------------------------------------------------------------------------------------------------ linear attention
// One CTA per (span, head).  S [d][dv] lives in shared memory for the whole span; per token: S = a S + k v^T, o = S^T q.
// Warp w owns rows i = w, w + nw, ...; lanes own columns.  The partial o of every warp goes through shared memory and is added
// in warp order, so the sum's order is fixed.  A span that starts at position 0 starts from S = 0 (the slot is not read).
// GATE false: one decay per head, q, k, v through SiLU.  GATE true: the decay is a vector per token (dec [T][H*d], one factor per
// row of S), q is multiplied by qscale, no activation.
// first column of head 0's q, k, v in a row of proj.  hpg > 1: q and k are shared by groups of hpg consecutive heads (head h reads
// block h / hpg).  dec_head (gated form): the decay is one factor per token and head, dec [T][H], not one per key channel.
// vscale (or null): [T][H], a factor per token and head on the values as they are staged.
struct LightCols { int q, k, v; int hpg = 1; int dec_head = 0; const float *vscale = nullptr; };
template <bool GATE>
__global__ void __launch_bounds__(256) stack_lightning_kernel(const float *proj, long long ld, LightCols col, const float *decay,
                                                              const float *dec, float qscale, float *state, StackSpans sp, float *o, int H,
                                                              int d, int dv) {
  extern __shared__ float shm[];
  const int s = blockIdx.x, h = blockIdx.y;
  const int tok0 = sp.sp_tok0[s], len = sp.sp_len[s], pos0 = sp.sp_pos0[s], slot = sp.sp_slot[s];
  const int nw = blockDim.x >> 5, w = threadIdx.x >> 5, l = threadIdx.x & 31;
  float *S = shm;                 // [d][dv]
  float *qs = S + (size_t)d * dv; // [d]
  float *ks = qs + d;             // [d]
  float *vs = ks + d;             // [dv]
  float *part = vs + dv;          // [nw][dv]
  float *as = part + (size_t)nw * dv;  // [d] (GATE)
  float *st = state + ((long long)slot * H + h) * d * dv;
  const float a = GATE ? 1.f : decay[h];
  for (int i = threadIdx.x; i < d * dv; i += blockDim.x) S[i] = pos0 > 0 ? st[i] : 0.f;
  for (int t = 0; t < len; t++) {
    const float *row = proj + (long long)(tok0 + t) * ld;
    __syncthreads();
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
      const float qv = row[col.q + (long long)(h / col.hpg) * d + i], kv = row[col.k + (long long)(h / col.hpg) * d + i];
      qs[i] = GATE ? qv * qscale : silu_(qv);
      ks[i] = GATE ? kv : silu_(kv);
      if (GATE) as[i] = col.dec_head ? dec[(long long)(tok0 + t) * H + h] : dec[(long long)(tok0 + t) * H * d + (long long)h * d + i];
    }
    for (int j = threadIdx.x; j < dv; j += blockDim.x) {
      const float vv = row[col.v + (long long)h * dv + j];
      vs[j] = GATE ? (col.vscale ? vv * col.vscale[(long long)(tok0 + t) * H + h] : vv) : silu_(vv);
    }
    __syncthreads();
    for (int j = l; j < dv; j += 32) {
      const float vj = vs[j];
      float acc = 0.f;
      for (int i = w; i < d; i += nw) {
        const float sv = fmaf(GATE ? as[i] : a, S[(size_t)i * dv + j], ks[i] * vj);
        S[(size_t)i * dv + j] = sv;
        acc = fmaf(sv, qs[i], acc);
      }
      part[(size_t)w * dv + j] = acc;
    }
    __syncthreads();
    for (int j = threadIdx.x; j < dv; j += blockDim.x) {
      float acc = 0.f;
      for (int k = 0; k < nw; k++) acc += part[(size_t)k * dv + j];
      o[(long long)(tok0 + t) * H * dv + (long long)h * dv + j] = acc;
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < d * dv; i += blockDim.x) st[i] = S[i];
}

// The same recurrence with the state in registers: thread (warp w, lane l) owns S[w RI + ii][l + 32 jj], ii < RI, jj < RJ; q, k, v
// of eight tokens at a time are staged in shared memory while the next eight are already on their way in registers, so a group
// costs two barriers and no shared-memory traffic for the state.
// GATE false: one decay per head, q, k, v through SiLU (lightning).  GATE true: gated linear attention -- the decay is a
// vector per token and head, one factor per key channel (row of S), read from `dec` [T][H*d]; q is multiplied by qscale and
// nothing goes through an activation.
// MODE 0: a whole span, from the slot's state (zero at position 0) back into it.
// Long spans are cut into segments of kLightSeg tokens that run side by side (grid x = span * max_seg + segment):
// MODE 1: the segment's own contribution sum_s (prod_{u>s} a_u) k_s v_s^T to the state at its end (no outputs), into `seg`,
// and with GATE the product of the segment's decays per channel into `seg_a`; a carry kernel then walks the segments in order,
// S_in(c+1) = A_c S_in(c) + contribution(c), leaving S_in(c) in `seg`;
// MODE 2: the segment's outputs, starting from S_in(c).
// GATE 2 (state-space mixer): one decay per token and head, dec [T][H], and a factor per token and head on the values,
// col.vscale [T][H]; both are staged as one number per token (the first two entries of the token's decay row), so the inner loop
// reads them once instead of a vector per group of rows.
// Rows and columns beyond d and dv: shared memory starts as zeros and nobody writes those entries, so their k, q and decays are
// zero and their part of S stays zero; the inner loop needs no bounds checks.
constexpr int kLightTok = 8, kLightSeg = 64;
template <int RI, int RJ, int MODE, int GATE>
__global__ void __launch_bounds__(256, 2) stack_lightning_reg_kernel(const float *__restrict__ proj, long long ld, LightCols col,
                                                                     const float *decay, const float *__restrict__ dec, float qscale,
                                                                     float *state, StackSpans sp, float *__restrict__ o, int H, int d,
                                                                     int dv, float *seg, float *seg_a, int max_seg) {
  extern __shared__ __align__(16) float shm[];
  constexpr int DP = RI * 8, DVP = RJ * 32;
  // heads vary fastest over the grid: the CTAs that run at the same time then read whole rows of the projections rather than
  // one head's columns at a stride of a row, which would keep most memory channels idle
  const int h = blockIdx.x % H, sc = blockIdx.x / H;
  const int s = MODE == 0 ? sc : sc / max_seg;
  const int tok0 = sp.sp_tok0[s], len = sp.sp_len[s], pos0 = sp.sp_pos0[s], slot = sp.sp_slot[s];
  int first = tok0, n = len;
  float *sg = nullptr, *sga = nullptr;
  if (MODE != 0) {
    const int c = sc - s * max_seg;
    if (c * kLightSeg >= len) return;
    first = tok0 + c * kLightSeg;
    n = min(kLightSeg, len - c * kLightSeg);
    sg = seg + ((size_t)(tok0 / kLightSeg + s + c) * H + h) * d * dv;
    if (GATE) sga = seg_a + ((size_t)(tok0 / kLightSeg + s + c) * H + h) * d;
  }
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, i0 = w * RI;
  float *qs = shm;                             // [tok][DP]
  float *ks = qs + kLightTok * DP;             // [tok][DP]
  float *vs = ks + kLightTok * DP;             // [tok][DVP]
  float *part = vs + kLightTok * DVP;          // [tok][8][DVP]
  float *as = part + kLightTok * 8 * DVP;      // [tok][DP] (GATE)
  for (int i = threadIdx.x; i < kLightTok * ((GATE ? 3 : 2) * DP + 9 * DVP); i += blockDim.x) shm[i] = 0.f;  // (the loop's first barrier follows)
  float *st = state + ((long long)slot * H + h) * d * dv;
  const float a = GATE ? 1.f : decay[h];
  float S[RI][RJ];
  float A[GATE == 1 ? RI : 1];  // MODE 1: running product of the decays of this thread's rows (GATE 2: of the head)
#pragma unroll
  for (int ii = 0; ii < (GATE == 1 ? RI : 1); ii++) A[ii] = 1.f;
#pragma unroll
  for (int ii = 0; ii < RI; ii++)
#pragma unroll
    for (int jj = 0; jj < RJ; jj++) {
      const int i = i0 + ii, j = l + jj * 32;
      float v = 0.f;
      if (i < d && j < dv) {
        if (MODE == 0 && pos0 > 0) v = st[(size_t)i * dv + j];
        if (MODE == 2) v = sg[(size_t)i * dv + j];
      }
      S[ii][jj] = v;
    }
  // Staging: a token's inputs are `per` numbers (q, k, v of this head, and with GATE its d decays); per <= 512, so every thread
  // owns at most two of these columns for all tokens.  Where a column comes from and where it goes is worked out once.
  const int per = GATE == 1 ? 3 * d + dv : 2 * d + dv + (GATE == 2 ? 2 : 0);
  const float *src[2];
  long long sstride[2];
  float *sdst[2];
  int dstride[2];
  float mul[2];
#pragma unroll
  for (int u = 0; u < 2; u++) {
    const int c = threadIdx.x + u * 256;
    src[u] = nullptr; sstride[u] = ld; sdst[u] = qs; dstride[u] = DP; mul[u] = 1.f;
    if (c < d) { src[u] = proj + col.q + (long long)(h / col.hpg) * d + c; sdst[u] = qs + c; mul[u] = GATE ? qscale : 1.f; }
    else if (c < 2 * d) { src[u] = proj + col.k + (long long)(h / col.hpg) * d + (c - d); sdst[u] = ks + (c - d); }
    else if (c < 2 * d + dv) { src[u] = proj + col.v + (long long)h * dv + (c - 2 * d); sdst[u] = vs + (c - 2 * d); dstride[u] = DVP; }
    else if (GATE == 2 && c < per) {  // the head's decay, then the values' factor
      src[u] = (c == 2 * d + dv ? dec : col.vscale) + h;
      sstride[u] = H;
      sdst[u] = as + (c - 2 * d - dv);
    } else if (c < per) {  // one decay per key channel, or the head's one decay copied to every channel
      src[u] = col.dec_head ? dec + h : dec + (long long)h * d + (c - 2 * d - dv);
      sstride[u] = col.dec_head ? (long long)H : (long long)H * d;
      sdst[u] = as + (c - 2 * d - dv);
    }
  }
  float tmp[2 * kLightTok];
  auto fetch = [&](int t0) {
    const int ct = min(kLightTok, n - t0);
#pragma unroll
    for (int t = 0; t < kLightTok; t++) {
      if (t < ct) {
        if (src[0]) tmp[2 * t] = src[0][(long long)(first + t0 + t) * sstride[0]];
        if (src[1]) tmp[2 * t + 1] = src[1][(long long)(first + t0 + t) * sstride[1]];
      }
    }
  };
  fetch(0);
  for (int t0 = 0; t0 < n; t0 += kLightTok) {
    const int ct = min(kLightTok, n - t0);
    __syncthreads();
#pragma unroll
    for (int t = 0; t < kLightTok; t++) {
      if (t < ct) {
        if (src[0]) sdst[0][t * dstride[0]] = GATE ? tmp[2 * t] * mul[0] : silu_(tmp[2 * t]);
        if (src[1]) sdst[1][t * dstride[1]] = GATE ? tmp[2 * t + 1] * mul[1] : silu_(tmp[2 * t + 1]);
      }
    }
    if (t0 + kLightTok < n) fetch(t0 + kLightTok);
    __syncthreads();
    for (int t = 0; t < ct; t++) {
      float vj[RJ], acc[RJ];
      const float at = GATE == 2 ? as[t * DP] : a, ft = GATE == 2 ? as[t * DP + 1] : 1.f;
      if (GATE == 2 && MODE == 1) A[0] *= at;
#pragma unroll
      for (int jj = 0; jj < RJ; jj++) { vj[jj] = GATE == 2 ? vs[t * DVP + l + jj * 32] * ft : vs[t * DVP + l + jj * 32]; acc[jj] = 0.f; }
#pragma unroll
      for (int i4 = 0; i4 < RI; i4 += 4) {
        const float4 k4 = *reinterpret_cast<const float4 *>(ks + t * DP + i0 + i4);
        const float4 q4 = *reinterpret_cast<const float4 *>(qs + t * DP + i0 + i4);
        float4 a4 = make_float4(at, at, at, at);
        if (GATE == 1) a4 = *reinterpret_cast<const float4 *>(as + t * DP + i0 + i4);
        const float kv[4] = {k4.x, k4.y, k4.z, k4.w}, qv[4] = {q4.x, q4.y, q4.z, q4.w}, av[4] = {a4.x, a4.y, a4.z, a4.w};
#pragma unroll
        for (int u = 0; u < 4; u++) {
          if (GATE == 1 && MODE == 1) A[GATE == 1 ? i4 + u : 0] *= av[u];
#pragma unroll
          for (int jj = 0; jj < RJ; jj++) {
            S[i4 + u][jj] = fmaf(av[u], S[i4 + u][jj], kv[u] * vj[jj]);
            if (MODE != 1) acc[jj] = fmaf(S[i4 + u][jj], qv[u], acc[jj]);
          }
        }
      }
      if (MODE != 1) {
#pragma unroll
        for (int jj = 0; jj < RJ; jj++) part[(t * 8 + w) * DVP + l + jj * 32] = acc[jj];
      }
    }
    if (MODE != 1) {
      __syncthreads();
      for (int e = threadIdx.x; e < ct * dv; e += blockDim.x) {
        const int t = e / dv, j = e - t * dv;
        float acc = 0.f;
#pragma unroll
        for (int k = 0; k < 8; k++) acc += part[(t * 8 + k) * DVP + j];
        o[(long long)(first + t0 + t) * H * dv + (long long)h * dv + j] = acc;
      }
    }
  }
  if (MODE == 2) return;
  float *dst = MODE == 0 ? st : sg;
#pragma unroll
  for (int ii = 0; ii < RI; ii++)
#pragma unroll
    for (int jj = 0; jj < RJ; jj++) {
      const int i = i0 + ii, j = l + jj * 32;
      if (i < d && j < dv) dst[(size_t)i * dv + j] = S[ii][jj];
    }
  if (GATE && MODE == 1 && l == 0) {
#pragma unroll
    for (int ii = 0; ii < RI; ii++)
      if (i0 + ii < d) sga[i0 + ii] = A[GATE == 1 ? ii : 0];
  }
}

// Segment carry: one thread per state element walks the span's segments in order.  Elements vary fastest over the grid, then
// heads, so that the CTAs that run at the same time walk one contiguous stretch of every segment.  seg_a (gated form): the
// product of each segment's decays per key channel; otherwise the head's decay to the power of the segment's length.
__global__ void stack_lightning_carry_kernel(const float *decay, const float *seg_a, float *state, StackSpans sp, float *seg, int H,
                                             int d, int dv) {
  const int n_el = d * dv;
  const int nz = (n_el + blockDim.x - 1) / blockDim.x;
  const int z = blockIdx.x % nz, h = (blockIdx.x / nz) % H, s = blockIdx.x / (nz * H);
  const int e = z * blockDim.x + threadIdx.x;
  if (e >= n_el) return;
  const int tok0 = sp.sp_tok0[s], len = sp.sp_len[s], pos0 = sp.sp_pos0[s], slot = sp.sp_slot[s];
  float *st = state + ((long long)slot * H + h) * n_el;
  const float a = seg_a ? 1.f : decay[h];
  float S = pos0 > 0 ? st[e] : 0.f;
  float a64 = 1.f;
  for (int k = 0; k < kLightSeg; k++) a64 *= a;
  const int nseg = (len + kLightSeg - 1) / kLightSeg;
  float *sg0 = seg + ((size_t)(tok0 / kLightSeg + s) * H + h) * n_el + e;
  const float *sa0 = seg_a ? seg_a + ((size_t)(tok0 / kLightSeg + s) * H + h) * d + e / dv : nullptr;
  const size_t step = (size_t)H * n_el, step_a = (size_t)H * d;
  constexpr int U = 8;  // segments whose contributions are fetched together, ahead of the chain that joins them
  for (int c0 = 0; c0 < nseg; c0 += U) {
    float own[U], fa[U];
#pragma unroll
    for (int u = 0; u < U; u++) {
      own[u] = c0 + u < nseg ? sg0[(size_t)(c0 + u) * step] : 0.f;
      fa[u] = (sa0 && c0 + u < nseg) ? sa0[(size_t)(c0 + u) * step_a] : 1.f;
    }
#pragma unroll
    for (int u = 0; u < U; u++) {
      const int c = c0 + u;
      if (c < nseg) {
        const int n = min(kLightSeg, len - c * kLightSeg);
        float an = a64;
        if (sa0) an = fa[u];
        else if (n < kLightSeg) {
          an = 1.f;
          for (int k = 0; k < n; k++) an *= a;
        }
        sg0[(size_t)c * step] = S;
        S = fmaf(an, S, own[u]);
      }
    }
  }
  st[e] = S;
}

int stack_lightning_seg_tokens() { return kLightSeg; }
// Whether a pass should cut its long spans into segments.  Walking a span in one piece costs its length times three
// operations per state element, once per wave of (span, head) CTAs (two fit an SM); the segments cost five operations per
// element (contributions, then outputs) over all segment CTAs in waves, plus the carry.  Many sequences with many heads fill
// the GPU without segments and then pay less; a single long prompt needs them.
bool stack_lightning_segmented(int n_spans, int T, int H, int max_len) {
  if (max_len <= kLightSeg) return false;
  const char *force = getenv("DIS_STACK_LIGHT_SEGMENTS");  // 2: always cut (tests)
  if (force && atoi(force) == 2) return true;
  static int slots = 0;
  if (!slots) {
    int dev = 0, n_sm = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n_sm < 1) n_sm = 148;
    slots = 2 * n_sm;
  }
  const long long pairs = (long long)n_spans * H;
  const long long whole = (long long)max_len * ((pairs + slots - 1) / slots) * 3;
  const long long seg_ctas = ((long long)T / kLightSeg + n_spans) * H;
  const long long cut = ((seg_ctas + slots - 1) / slots) * kLightSeg * 5 + kLightSeg;
  return cut < whole;
}
size_t stack_lightning_seg_floats(int cap_tokens, int max_spans, int H, int d, int dv) {
  return (size_t)(cap_tokens / kLightSeg + max_spans + 1) * H * d * dv;
}
size_t stack_lightning_seg_decay_floats(int cap_tokens, int max_spans, int H, int d) {
  return (size_t)(cap_tokens / kLightSeg + max_spans + 1) * H * d;
}

template <int RI, int RJ, int GATE>
static cudaError_t lightning_reg(const float *proj, long long ld, LightCols col, const float *decay, const float *dec, float qscale,
                                 float *state, const StackSpans &sp, float *o, int H, int d, int dv, float *seg, float *seg_a,
                                 int max_len, cudaStream_t st) {
  const size_t sh = (size_t)kLightTok * ((GATE ? 3 : 2) * RI * 8 + RJ * 32 + 8 * RJ * 32) * sizeof(float);
  static DeviceOnce once;
  DIS_CUDA_TRY(once.run([&] {
    cudaError_t e = cudaFuncSetAttribute(stack_lightning_reg_kernel<RI, RJ, 0, GATE>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(stack_lightning_reg_kernel<RI, RJ, 1, GATE>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
    return e != cudaSuccess ? e : cudaFuncSetAttribute(stack_lightning_reg_kernel<RI, RJ, 2, GATE>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
  }));
  if (!seg || (GATE && !seg_a) || max_len <= kLightSeg) {
    stack_lightning_reg_kernel<RI, RJ, 0, GATE><<<sp.n_spans * H, 256, sh, st>>>(proj, ld, col, decay, dec, qscale, state, sp, o, H, d, dv, nullptr, nullptr, 1);
    return cudaGetLastError();
  }
  const int max_seg = (max_len + kLightSeg - 1) / kLightSeg;
  stack_lightning_reg_kernel<RI, RJ, 1, GATE><<<sp.n_spans * max_seg * H, 256, sh, st>>>(proj, ld, col, decay, dec, qscale, state, sp, o, H, d, dv, seg, seg_a, max_seg);
  stack_lightning_carry_kernel<<<sp.n_spans * H * ((d * dv + 255) / 256), 256, 0, st>>>(decay, GATE ? seg_a : nullptr, state, sp, seg, H, d, dv);
  stack_lightning_reg_kernel<RI, RJ, 2, GATE><<<sp.n_spans * max_seg * H, 256, sh, st>>>(proj, ld, col, decay, dec, qscale, state, sp, o, H, d, dv, seg, seg_a, max_seg);
  return cudaGetLastError();
}

cudaError_t launch_stack_lightning(const float *proj, long long ld, const float *decay, float *state, const StackSpans &sp,
                                   float *o, int H, int d, int dv, float *seg, int max_len, cudaStream_t st) {
  const int threads = 256;
  const LightCols col{0, H * d, 2 * H * d};
  if (d <= 64 && dv <= 64) return lightning_reg<8, 2, false>(proj, ld, col, decay, nullptr, 1.f, state, sp, o, H, d, dv, seg, nullptr, max_len, st);
  if (d <= 128 && dv <= 128) return lightning_reg<16, 4, false>(proj, ld, col, decay, nullptr, 1.f, state, sp, o, H, d, dv, seg, nullptr, max_len, st);
  const size_t sh = ((size_t)d * dv + 2 * d + dv + (size_t)(threads / 32) * dv) * sizeof(float);
  if (sh > 220 * 1024) return cudaErrorInvalidValue;
  static DeviceOnce once;
  DIS_CUDA_TRY(once.run([&] { return cudaFuncSetAttribute(stack_lightning_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024); }));
  stack_lightning_kernel<false><<<dim3(sp.n_spans, H), threads, sh, st>>>(proj, ld, col, decay, nullptr, 1.f, state, sp, o, H, d, dv);
  return cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------ gated linear attention
// Decays: z[c] = b[c] + sum_r A2[c][r] u[r] with u the rank-sized bottleneck (columns a_off .. of proj, fp32), then
// a[c] = sigmoid(z[c])^(1/tau) = exp(-softplus(-z[c]) / tau), everything fp32.  A block takes 16 tokens and 128 channels: the
// tokens' u sit in shared memory, a thread reads its channel's row of A2 once and uses it for all 16 tokens.
constexpr int kDecTok = 16;
template <bool WF32>
__global__ void __launch_bounds__(128) stack_gla_decay_kernel(const float *proj, long long ld, int a_off, const void *a2, const float *b,
                                                              int T, int n, int rank, float inv_tau, float *dec) {
  extern __shared__ float u[];  // [kDecTok][rank]
  const int t0 = blockIdx.x * kDecTok, nt = min(kDecTok, T - t0);
  for (int i = threadIdx.x; i < kDecTok * rank; i += blockDim.x) {
    const int tt = i / rank, r = i - tt * rank;
    u[i] = tt < nt ? proj[(long long)(t0 + tt) * ld + a_off + r] : 0.f;
  }
  __syncthreads();
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= n) return;
  float z[kDecTok];
#pragma unroll
  for (int tt = 0; tt < kDecTok; tt++) z[tt] = b[c];
  for (int r = 0; r < rank; r++) {
    const float w = ld_el<WF32>(a2, (long long)c * rank + r);
#pragma unroll
    for (int tt = 0; tt < kDecTok; tt++) z[tt] = fmaf(w, u[tt * rank + r], z[tt]);
  }
#pragma unroll
  for (int tt = 0; tt < kDecTok; tt++) {
    if (tt < nt) {
      // -log sigmoid(z) = softplus(-z) = max(-z, 0) + log1p(exp(-|z|))
      const float sp = fmaxf(-z[tt], 0.f) + log1pf(expf(-fabsf(z[tt])));
      dec[(long long)(t0 + tt) * n + c] = expf(-sp * inv_tau);
    }
  }
}
cudaError_t launch_stack_gla_decay(const float *proj, long long ld, int a_off, const void *a2, bool w_f32, const float *b, int T, int n,
                                   int rank, float tau, float *dec, cudaStream_t st) {
  if (T <= 0) return cudaSuccess;
  const dim3 grid((T + kDecTok - 1) / kDecTok, (n + 127) / 128);
  const size_t sh = (size_t)kDecTok * rank * sizeof(float);
  if (sh > 48 * 1024) return cudaErrorInvalidValue;
  if (w_f32) stack_gla_decay_kernel<true><<<grid, 128, sh, st>>>(proj, ld, a_off, a2, b, T, n, rank, 1.f / tau, dec);
  else stack_gla_decay_kernel<false><<<grid, 128, sh, st>>>(proj, ld, a_off, a2, b, T, n, rank, 1.f / tau, dec);
  return cudaGetLastError();
}

// The recurrence itself: the register kernel above in its gated form (dim, vdim <= 128).
cudaError_t launch_stack_gla(const float *proj, long long ld, int q_off, int k_off, int v_off, const float *dec, float *state,
                             const StackSpans &sp, float *o, int H, int d, int dv, float *seg, float *seg_a, int max_len,
                             cudaStream_t st) {
  const LightCols col{q_off, k_off, v_off};
  const float qscale = 1.f / sqrtf((float)d);
  // rows of S per warp (RI) and columns per lane (RJ) chosen so that all eight warps own rows: d <= 8 RI, dv <= 32 RJ
  if (d <= 32 && dv <= 64) return lightning_reg<4, 2, true>(proj, ld, col, nullptr, dec, qscale, state, sp, o, H, d, dv, seg, seg_a, max_len, st);
  if (d <= 64 && dv <= 64) return lightning_reg<8, 2, true>(proj, ld, col, nullptr, dec, qscale, state, sp, o, H, d, dv, seg, seg_a, max_len, st);
  if (d <= 64 && dv <= 128) return lightning_reg<8, 4, true>(proj, ld, col, nullptr, dec, qscale, state, sp, o, H, d, dv, seg, seg_a, max_len, st);
  if (d <= 128 && dv <= 128) return lightning_reg<16, 4, true>(proj, ld, col, nullptr, dec, qscale, state, sp, o, H, d, dv, seg, seg_a, max_len, st);
  // larger heads: the state of one head in shared memory, one CTA per (span, head)
  const int threads = 256;
  const size_t sh = ((size_t)d * dv + 3 * d + dv + (size_t)(threads / 32) * dv) * sizeof(float);
  if (sh > 220 * 1024) return cudaErrorInvalidValue;
  static DeviceOnce once;
  DIS_CUDA_TRY(once.run([&] { return cudaFuncSetAttribute(stack_lightning_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024); }));
  stack_lightning_kernel<true><<<dim3(sp.n_spans, H), threads, sh, st>>>(proj, ld, col, nullptr, dec, qscale, state, sp, o, H, d, dv);
  return cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------ state-space mixer
// The recurrence S = a_t S + B_t (dt_t x_t)^T, o_t = S^T C_t is the gated one above with a decay per token and head, keys B and
// queries C shared by the heads of a group, and values dt x: the same kernels, their staging told where to read.
cudaError_t launch_stack_ssd(const float *buf, long long ld_b, int c_off, int b_off, int v_off, int hpg, const float *dec,
                             const float *dt, float *state, const StackSpans &sp, float *o, int H, int N, int P, float *seg, float *seg_a,
                             int max_len, cudaStream_t st) {
  LightCols col{c_off, b_off, v_off};
  col.hpg = hpg < 1 ? 1 : hpg;
  col.dec_head = 1;
  col.vscale = dt;
  const int d = N, dv = P;
  if (d <= 32 && dv <= 64) return lightning_reg<4, 2, 2>(buf, ld_b, col, nullptr, dec, 1.f, state, sp, o, H, d, dv, seg, seg_a, max_len, st);
  if (d <= 64 && dv <= 64) return lightning_reg<8, 2, 2>(buf, ld_b, col, nullptr, dec, 1.f, state, sp, o, H, d, dv, seg, seg_a, max_len, st);
  if (d <= 128 && dv <= 64) return lightning_reg<16, 2, 2>(buf, ld_b, col, nullptr, dec, 1.f, state, sp, o, H, d, dv, seg, seg_a, max_len, st);
  if (d <= 64 && dv <= 128) return lightning_reg<8, 4, 2>(buf, ld_b, col, nullptr, dec, 1.f, state, sp, o, H, d, dv, seg, seg_a, max_len, st);
  if (d <= 128 && dv <= 128) return lightning_reg<16, 4, 2>(buf, ld_b, col, nullptr, dec, 1.f, state, sp, o, H, d, dv, seg, seg_a, max_len, st);
  const int threads = 256;
  const size_t sh = ((size_t)d * dv + 3 * d + dv + (size_t)(threads / 32) * dv) * sizeof(float);
  if (sh > 220 * 1024) return cudaErrorInvalidValue;
  static DeviceOnce once;
  DIS_CUDA_TRY(once.run([&] { return cudaFuncSetAttribute(stack_lightning_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024); }));
  stack_lightning_kernel<true><<<dim3(sp.n_spans, H), threads, sh, st>>>(buf, ld_b, col, nullptr, dec, 1.f, state, sp, o, H, d, dv);
  return cudaGetLastError();
}

// Convolution and SiLU over the channels x | B | C, step sizes and decays.  grid (token, stretch of channels); a thread takes
// four neighbouring channels where the layout allows 16-byte accesses (VEC).  The input at position p of the sequence comes from
// the span's own rows of proj or, before the span's start, from the slot's tail (tail[i] holds position pos0 - (taps-1) + i);
// before the sequence's start it is zero, so a slot that another sequence used before needs no clearing.  The first block of a
// token also forms dt = softplus(proj[dt_off + h] + dt_bias[h]) (no clamp) -> dtv [T][H] and the decay exp(-exp(A_log[h]) dt) -> dec.
// TAIL (passes of single tokens): the thread moves its channels' tail on by one itself, so no second launch is needed.
constexpr int kConvMaxTaps = 16;
template <bool VEC, bool TAIL>
__global__ void __launch_bounds__(256) stack_ssm_conv_kernel(const float *__restrict__ proj, long long ld, int x_off, int dt_off, int C,
                                                             int H, int taps, const float *__restrict__ cw, const float *__restrict__ cb,
                                                             const float *__restrict__ vec, float *cstate, StackSpans sp,
                                                             float *__restrict__ buf, long long ld_b, float *__restrict__ dec,
                                                             float *__restrict__ dtv) {
  constexpr int V = VEC ? 4 : 1;
  const int t = blockIdx.x;
  const int s = sp.span[t], tok0 = sp.sp_tok0[s], pos0 = sp.sp_pos0[s], slot = sp.sp_slot[s];
  const int back_in_span = t - tok0;  // tokens of the span in front of t
  const float *row = proj + (long long)t * ld;
  if (blockIdx.y == 0)
    for (int h = threadIdx.x; h < H; h += blockDim.x) {
      const float z = row[dt_off + h] + vec[h];
      const float dt = fmaxf(z, 0.f) + log1pf(expf(-fabsf(z)));
      dtv[(long long)t * H + h] = dt;
      dec[(long long)t * H + h] = expf(-expf(vec[H + h]) * dt);
    }
  float *tail = cstate + (long long)slot * (taps - 1) * C;
  const int c = (blockIdx.y * blockDim.x + threadIdx.x) * V;
  if (c >= C) return;
  float acc[V], in[kConvMaxTaps][V];
#pragma unroll
  for (int k = 0; k < V; k++) acc[k] = cb[c + k];
  for (int j = 0; j < taps; j++) {
    const int back = taps - 1 - j;
    const float *src = nullptr;
    if (back <= back_in_span) src = row + x_off + c - (long long)back * ld;
    else if (pos0 + back_in_span - back >= 0) src = tail + (long long)((taps - 1) - (back - back_in_span)) * C + c;
    if (VEC) {
      const float4 v = src ? *reinterpret_cast<const float4 *>(src) : make_float4(0.f, 0.f, 0.f, 0.f);
      in[j][0] = v.x; in[j][V > 1 ? 1 : 0] = v.y; in[j][V > 2 ? 2 : 0] = v.z; in[j][V > 3 ? 3 : 0] = v.w;
    } else in[j][0] = src ? src[0] : 0.f;
#pragma unroll
    for (int k = 0; k < V; k++) acc[k] = fmaf(cw[(long long)(c + k) * taps + j], in[j][k], acc[k]);
  }
  if (VEC) *reinterpret_cast<float4 *>(buf + (long long)t * ld_b + c) = make_float4(silu_(acc[0]), silu_(acc[V > 1 ? 1 : 0]), silu_(acc[V > 2 ? 2 : 0]), silu_(acc[V > 3 ? 3 : 0]));
  else buf[(long long)t * ld_b + c] = silu_(acc[0]);
  if (TAIL) {  // the span is this one token: tail'[i] = tail[i + 1], tail'[taps - 2] = the token's input
    for (int j = 0; j + 1 < taps; j++)
#pragma unroll
      for (int k = 0; k < V; k++) tail[(long long)j * C + c + k] = in[j + 1][k];
  }
}
// The same for passes with prompts, 2 to 4 taps: a block takes kConvTile consecutive tokens and a stretch of channels, a thread
// keeps its channels' weights and the last TAPS - 1 inputs in registers and reads every input once; the window is fetched anew
// (from the rows before, the slot's tail or zeros, as above) at the tile's first token and wherever a new span starts.  The
// products are summed in the order of the kernel above, so a position's result does not depend on which of the two ran.
constexpr int kConvTile = 16;
template <int TAPS, bool VEC>
__global__ void __launch_bounds__(256) stack_ssm_conv_tile_kernel(const float *__restrict__ proj, long long ld, int x_off, int dt_off, int C,
                                                                  int H, const float *__restrict__ cw, const float *__restrict__ cb,
                                                                  const float *__restrict__ vec, const float *__restrict__ cstate,
                                                                  StackSpans sp, float *__restrict__ buf, long long ld_b,
                                                                  float *__restrict__ dec, float *__restrict__ dtv) {
  constexpr int V = VEC ? 4 : 1;
  const int t0 = blockIdx.x * kConvTile, t1 = min(sp.T, t0 + kConvTile);
  if (blockIdx.y == 0)
    for (int e = threadIdx.x; e < (t1 - t0) * H; e += blockDim.x) {
      const int t = t0 + e / H, h = e % H;
      const float z = proj[(long long)t * ld + dt_off + h] + vec[h];
      const float dt = fmaxf(z, 0.f) + log1pf(expf(-fabsf(z)));
      dtv[(long long)t * H + h] = dt;
      dec[(long long)t * H + h] = expf(-expf(vec[H + h]) * dt);
    }
  const int c = (blockIdx.y * blockDim.x + threadIdx.x) * V;
  if (c >= C) return;
  auto ldv = [](const float *p, float (&o)[V]) {
    if (VEC) { const float4 v = *reinterpret_cast<const float4 *>(p); o[0] = v.x; o[V > 1 ? 1 : 0] = v.y; o[V > 2 ? 2 : 0] = v.z; o[V > 3 ? 3 : 0] = v.w; }
    else o[0] = p[0];
  };
  float w[TAPS][V], b[V], win[TAPS - 1][V];
#pragma unroll
  for (int k = 0; k < V; k++) {
    b[k] = cb[c + k];
#pragma unroll
    for (int j = 0; j < TAPS; j++) w[j][k] = cw[(long long)(c + k) * TAPS + j];
  }
  int prev_span = -1;
  for (int t = t0; t < t1; t++) {
    const int s = sp.span[t];
    const float *row = proj + (long long)t * ld + x_off + c;
    if (s != prev_span) {
      prev_span = s;
      const int back_in_span = t - sp.sp_tok0[s], pos0 = sp.sp_pos0[s];
      const float *tail = cstate + (long long)sp.sp_slot[s] * (TAPS - 1) * C + c;
#pragma unroll
      for (int j = 0; j < TAPS - 1; j++) {
        const int back = TAPS - 1 - j;
        if (back <= back_in_span) ldv(row - (long long)back * ld, win[j]);
        else if (pos0 + back_in_span - back >= 0) ldv(tail + (long long)((TAPS - 1) - (back - back_in_span)) * C, win[j]);
        else {
#pragma unroll
          for (int k = 0; k < V; k++) win[j][k] = 0.f;
        }
      }
    }
    float cur[V], acc[V];
    ldv(row, cur);
#pragma unroll
    for (int k = 0; k < V; k++) {
      acc[k] = b[k];
#pragma unroll
      for (int j = 0; j < TAPS - 1; j++) acc[k] = fmaf(w[j][k], win[j][k], acc[k]);
      acc[k] = silu_(fmaf(w[TAPS - 1][k], cur[k], acc[k]));
    }
    if (VEC) *reinterpret_cast<float4 *>(buf + (long long)t * ld_b + c) = make_float4(acc[0], acc[V > 1 ? 1 : 0], acc[V > 2 ? 2 : 0], acc[V > 3 ? 3 : 0]);
    else buf[(long long)t * ld_b + c] = acc[0];
#pragma unroll
    for (int k = 0; k < V; k++) {
#pragma unroll
      for (int j = 0; j + 1 < TAPS - 1; j++) win[j][k] = win[j + 1][k];
      win[TAPS - 2][k] = cur[k];
    }
  }
}
// The tail moves on to the span's last taps - 1 inputs (a span shorter than that keeps the end of the old tail in front).
__global__ void stack_ssm_tail_kernel(const float *__restrict__ proj, long long ld, int x_off, float *cstate, StackSpans sp, int C,
                                      int taps) {
  const int s = blockIdx.x;
  const int tok0 = sp.sp_tok0[s], len = sp.sp_len[s], pos0 = sp.sp_pos0[s], slot = sp.sp_slot[s];
  float *tail = cstate + (long long)slot * (taps - 1) * C;
  const int n = taps - 1;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
    float nv[kConvMaxTaps];
    for (int k = 0; k < n; k++) {
      const int rel = len - n + k;  // index relative to the span's first token of the position tail'[k] holds
      if (rel >= 0) nv[k] = proj[(long long)(tok0 + rel) * ld + x_off + c];
      else nv[k] = (pos0 + rel >= 0) ? tail[(long long)(n + rel) * C + c] : 0.f;
    }
    for (int k = 0; k < n; k++) tail[(long long)k * C + c] = nv[k];
  }
}
cudaError_t launch_stack_ssm_conv(const float *proj, long long ld, int x_off, int dt_off, int C, int H, int taps, const float *cw,
                                  const float *cb, const float *vec, float *cstate, const StackSpans &sp, float *buf, long long ld_b,
                                  float *dec, float *dtv, cudaStream_t st) {
  if (taps < 1 || taps > kConvMaxTaps) return cudaErrorInvalidValue;
  if (sp.T <= 0) return cudaSuccess;
  const bool v4 = ((C | x_off | (int)(ld & 3) | (int)(ld_b & 3)) & 3) == 0 && reinterpret_cast<uintptr_t>(proj) % 16 == 0 &&
                  reinterpret_cast<uintptr_t>(buf) % 16 == 0 && (taps == 1 || reinterpret_cast<uintptr_t>(cstate) % 16 == 0);
  const bool single = sp.T == sp.n_spans;  // every span one token long
  const int per = v4 ? 4 : 1;
  const dim3 grid(sp.T, (C + 256 * per - 1) / (256 * per));
#define DIS_CONV(V, S) stack_ssm_conv_kernel<V, S><<<grid, 256, 0, st>>>(proj, ld, x_off, dt_off, C, H, taps, cw, cb, vec, cstate, sp, buf, ld_b, dec, dtv)
#define DIS_CONV_TILE(TP, V) stack_ssm_conv_tile_kernel<TP, V><<<tgrid, 256, 0, st>>>(proj, ld, x_off, dt_off, C, H, cw, cb, vec, cstate, sp, buf, ld_b, dec, dtv)
  const dim3 tgrid((sp.T + kConvTile - 1) / kConvTile, grid.y);
  if (single && taps > 1) { if (v4) DIS_CONV(true, true); else DIS_CONV(false, true); }
  else if (!single && taps == 2) { if (v4) DIS_CONV_TILE(2, true); else DIS_CONV_TILE(2, false); }
  else if (!single && taps == 3) { if (v4) DIS_CONV_TILE(3, true); else DIS_CONV_TILE(3, false); }
  else if (!single && taps == 4) { if (v4) DIS_CONV_TILE(4, true); else DIS_CONV_TILE(4, false); }
  else { if (v4) DIS_CONV(true, false); else DIS_CONV(false, false); }
#undef DIS_CONV_TILE
#undef DIS_CONV
  if (taps > 1 && !single) stack_ssm_tail_kernel<<<dim3(sp.n_spans, (C + 1023) / 1024), 256, 0, st>>>(proj, ld, x_off, cstate, sp, C, taps);
  return cudaGetLastError();
}

// y = (o + D[h] x) silu(z), then each of `parts` equal stretches of the row is divided by its own root mean square, times w.
// One block per token, the row in shared memory.  VEC: four neighbouring columns per access (P and the stretch are multiples
// of 4).  With at least as many stretches as warps a warp normalises a stretch on its own; else the block takes them in turn.
template <bool F32, bool VEC>
__global__ void __launch_bounds__(256) stack_ssm_out_kernel(const float *__restrict__ o, const float *__restrict__ buf, long long ld_b,
                                                            const float *__restrict__ z, long long ld, const float *__restrict__ D,
                                                            const float *__restrict__ w, int parts, void *__restrict__ out, int H, int P,
                                                            float eps) {
  extern __shared__ __align__(16) float yrow[];  // [H*P]
  __shared__ float sh[32];
  constexpr int V = VEC ? 4 : 1;
  auto ldv = [](const float *p, float (&v)[V]) {
    if (VEC) { const float4 f = *reinterpret_cast<const float4 *>(p); v[0] = f.x; v[V > 1 ? 1 : 0] = f.y; v[V > 2 ? 2 : 0] = f.z; v[V > 3 ? 3 : 0] = f.w; }
    else v[0] = p[0];
  };
  const long long t = blockIdx.x;
  const int inner = H * P, per = inner / parts;
  for (int i = threadIdx.x * V; i < inner; i += blockDim.x * V) {
    float ov[V], xv[V], zv[V];
    ldv(o + t * inner + i, ov);
    ldv(buf + t * ld_b + i, xv);
    ldv(z + t * ld + i, zv);
    const float Dh = D[i / P];
#pragma unroll
    for (int k = 0; k < V; k++) yrow[i + k] = fmaf(Dh, xv[k], ov[k]) * silu_(zv[k]);
  }
  __syncthreads();
  auto put = [&](int i, float r) {  // columns i .. i + V - 1 of the row, normalised
    float yv[V], wv[V];
    ldv(yrow + i, yv);
    ldv(w + i, wv);
    if (VEC && !F32) {
      uint2 pk;
      pk.x = (uint32_t)float_to_bf16_bits(yv[0] * r * wv[0]) | ((uint32_t)float_to_bf16_bits(yv[V > 1 ? 1 : 0] * r * wv[V > 1 ? 1 : 0]) << 16);
      pk.y = (uint32_t)float_to_bf16_bits(yv[V > 2 ? 2 : 0] * r * wv[V > 2 ? 2 : 0]) | ((uint32_t)float_to_bf16_bits(yv[V > 3 ? 3 : 0] * r * wv[V > 3 ? 3 : 0]) << 16);
      *reinterpret_cast<uint2 *>(reinterpret_cast<uint16_t *>(out) + t * inner + i) = pk;
    } else if (VEC) {
      *reinterpret_cast<float4 *>(reinterpret_cast<float *>(out) + t * inner + i) =
          make_float4(yv[0] * r * wv[0], yv[V > 1 ? 1 : 0] * r * wv[V > 1 ? 1 : 0], yv[V > 2 ? 2 : 0] * r * wv[V > 2 ? 2 : 0], yv[V > 3 ? 3 : 0] * r * wv[V > 3 ? 3 : 0]);
    } else st_el<F32>(out, t * inner + i, yv[0] * r * wv[0]);
  };
  const int wp = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
  if (parts >= nw) {
    for (int g = wp; g < parts; g += nw) {
      float q = 0.f;
      for (int i = l * V; i < per; i += 32 * V) {
        float yv[V];
        ldv(yrow + g * per + i, yv);
#pragma unroll
        for (int k = 0; k < V; k++) q += yv[k] * yv[k];
      }
      const float r = rsqrtf(warp_sum(q) / (float)per + eps);
      for (int i = l * V; i < per; i += 32 * V) put(g * per + i, r);
    }
    return;
  }
  for (int g = 0; g < parts; g++) {
    float q = 0.f;
    for (int i = threadIdx.x * V; i < per; i += blockDim.x * V) {
      float yv[V];
      ldv(yrow + g * per + i, yv);
#pragma unroll
      for (int k = 0; k < V; k++) q += yv[k] * yv[k];
    }
    const float r = rsqrtf(block_sum(q, sh) / (float)per + eps);
    for (int i = threadIdx.x * V; i < per; i += blockDim.x * V) put(g * per + i, r);
  }
}
template <bool F32, bool VEC>
static cudaError_t ssm_out_go(const float *o, const float *buf, long long ld_b, const float *z, long long ld, const float *D, const float *w,
                              int parts, void *out, int T, int H, int P, float eps, cudaStream_t st) {
  static DeviceOnce once;
  DIS_CUDA_TRY(once.run([&] { return cudaFuncSetAttribute(stack_ssm_out_kernel<F32, VEC>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024); }));
  stack_ssm_out_kernel<F32, VEC><<<T, 256, (size_t)H * P * 4, st>>>(o, buf, ld_b, z, ld, D, w, parts, out, H, P, eps);
  return cudaGetLastError();
}
cudaError_t launch_stack_ssm_out(const float *o, const float *buf, long long ld_b, const float *z, long long ld, const float *D,
                                 const float *w, int parts, void *out, bool f32, int T, int H, int P, float eps, cudaStream_t st) {
  const int inner = H * P;
  if (parts < 1 || inner % parts || (size_t)inner * 4 > 160 * 1024) return cudaErrorInvalidValue;
  if (T <= 0) return cudaSuccess;
  auto al = [](const void *p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; };
  const bool vec = P % 4 == 0 && (inner / parts) % 4 == 0 && ld % 4 == 0 && ld_b % 4 == 0 && al(o) && al(buf) && al(z) && al(w) && al(out);
  if (f32) return vec ? ssm_out_go<true, true>(o, buf, ld_b, z, ld, D, w, parts, out, T, H, P, eps, st)
                      : ssm_out_go<true, false>(o, buf, ld_b, z, ld, D, w, parts, out, T, H, P, eps, st);
  return vec ? ssm_out_go<false, true>(o, buf, ld_b, z, ld, D, w, parts, out, T, H, P, eps, st)
             : ssm_out_go<false, false>(o, buf, ld_b, z, ld, D, w, parts, out, T, H, P, eps, st);
}

// out[t][off + h*dv + j] = scale * o[t][h][j] / rms(o[t][h]) * w[j] * silu(gate[t][h*dv + j]): the norm runs over one head's dv
// outputs, its gain vector is shared by the heads.  One warp per (token, head).
template <bool F32>
__global__ void __launch_bounds__(256) stack_headnorm_silu_kernel(const float *o, const float *w, const float *gate, long long ldg, void *out,
                                                                  long long ldo, int off, float scale, int rows, int H, int dv, float eps) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), l = threadIdx.x & 31;
  if (row >= rows) return;
  const int t = row / H, h = row - t * H;
  const float *r = o + (long long)row * dv;
  float s = 0.f;
  for (int j = l; j < dv; j += 32) s += r[j] * r[j];
  s = warp_sum(s);
  const float k = rsqrtf(s / (float)dv + eps) * scale;
  for (int j = l; j < dv; j += 32) {
    const float g = gate[(long long)t * ldg + (long long)h * dv + j];
    st_el<F32>(out, (long long)t * ldo + off + (long long)h * dv + j, r[j] * k * w[j] * silu_(g));
  }
}
cudaError_t launch_stack_headnorm_silu(const float *o, const float *w, const float *gate, long long ldg, void *out, long long ldo,
                                       int off, float scale, bool f32, int T, int H, int dv, float eps, cudaStream_t st) {
  const int rows = T * H;
  if (rows <= 0) return cudaSuccess;
  if (f32) stack_headnorm_silu_kernel<true><<<(rows + 7) / 8, 256, 0, st>>>(o, w, gate, ldg, out, ldo, off, scale, rows, H, dv, eps);
  else stack_headnorm_silu_kernel<false><<<(rows + 7) / 8, 256, 0, st>>>(o, w, gate, ldg, out, ldo, off, scale, rows, H, dv, eps);
  return cudaGetLastError();
}

template <bool F32>
__global__ void __launch_bounds__(256) stack_norm_gate_kernel(const float *o, const float *w, const float *gate, long long ldg,
                                                              void *out, int n, float eps) {
  __shared__ float sh[32];
  const long long t = blockIdx.x;
  const float *r = o + t * n;
  float s = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) s += r[i] * r[i];
  s = block_sum(s, sh);
  const float k = rsqrtf(s / (float)n + eps);
  for (int i = threadIdx.x; i < n; i += blockDim.x)
    st_el<F32>(out, t * n + i, r[i] * k * w[i] * sigmoid_precise(gate[t * ldg + i]));
}
cudaError_t launch_stack_norm_gate(const float *o, const float *w, const float *gate, long long ldg, void *out, bool f32, int T,
                                   int n, float eps, cudaStream_t st) {
  if (f32) stack_norm_gate_kernel<true><<<T, 256, 0, st>>>(o, w, gate, ldg, out, n, eps);
  else stack_norm_gate_kernel<false><<<T, 256, 0, st>>>(o, w, gate, ldg, out, n, eps);
  return cudaGetLastError();
}

// heads > 0: o is laid out head by head, [heads][T][n / heads] (the per-head tensor-core products write it so)
template <bool F32>
__global__ void stack_gate_kernel(const float *__restrict__ o, const float *__restrict__ gate, long long ldg, void *__restrict__ out, int T,
                                  int n, int heads) {
  const int hw = heads > 0 ? n / heads : n;
  for (int t = blockIdx.x; t < T; t += gridDim.x) {
    for (int c = threadIdx.x; c < n; c += blockDim.x) {
      const float v = heads > 0 ? o[((long long)(c / hw) * T + t) * hw + c % hw] : o[(long long)t * n + c];
      st_el<F32>(out, (long long)t * n + c, v * sigmoid_precise(gate[t * ldg + c]));
    }
  }
}
cudaError_t launch_stack_gate(const float *o, const float *gate, long long ldg, void *out, bool f32, int T, int n, int heads,
                              cudaStream_t st) {
  if (T <= 0) return cudaSuccess;
  const int grid = std::min(T, 148 * 16);
  if (f32) stack_gate_kernel<true><<<grid, 256, 0, st>>>(o, gate, ldg, out, T, n, heads);
  else stack_gate_kernel<false><<<grid, 256, 0, st>>>(o, gate, ldg, out, T, n, heads);
  return cudaGetLastError();
}

// Per-head products on the tensor cores want each head's rows contiguous: src fp32 [T][ld], head h at columns off + h * hs,
// `wd` of them -> dst bf16 [H][T][wd]; and back: src fp32 [H][T][wd] -> dst fp32 [T][ld] at columns off + h * hs.
__global__ void stack_heads_pack_kernel(const float *__restrict__ src, long long ld, int off, int hs, int wd, int T, int H,
                                        uint16_t *__restrict__ dst) {
  const int t = blockIdx.x / H, h = blockIdx.x - t * H;  // one (token, head) row per block
  const float *sr = src + (long long)t * ld + off + (long long)h * hs;
  uint16_t *dr = dst + ((long long)h * T + t) * wd;
  for (int c = threadIdx.x; c < wd; c += blockDim.x) dr[c] = float_to_bf16_bits(sr[c]);
}
__global__ void stack_heads_unpack_kernel(const float *__restrict__ src, int wd, int T, int H, float *__restrict__ dst, long long ld,
                                          int off, int hs) {
  const int t = blockIdx.x / H, h = blockIdx.x - t * H;
  const float *sr = src + ((long long)h * T + t) * wd;
  float *dr = dst + (long long)t * ld + off + (long long)h * hs;
  for (int c = threadIdx.x; c < wd; c += blockDim.x) dr[c] = sr[c];
}
cudaError_t launch_stack_heads_pack(const float *src, long long ld, int off, int hs, int wd, int T, int H, uint16_t *dst, cudaStream_t st) {
  if ((long long)T * H <= 0 || wd <= 0) return cudaSuccess;
  stack_heads_pack_kernel<<<T * H, 128, 0, st>>>(src, ld, off, hs, wd, T, H, dst);
  return cudaGetLastError();
}
cudaError_t launch_stack_heads_unpack(const float *src, int wd, int T, int H, float *dst, long long ld, int off, int hs, cudaStream_t st) {
  if ((long long)T * H <= 0 || wd <= 0) return cudaSuccess;
  stack_heads_unpack_kernel<<<T * H, 128, 0, st>>>(src, wd, T, H, dst, ld, off, hs);
  return cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------ minimal gated recurrence
// One thread per channel walks the span: z = sigmoid(pz), c = pu + 1/2 (pu >= 0) or sigmoid(pu), S = (1 - z) S + z c.
template <bool F32>
__global__ void stack_mingru_kernel(const float *__restrict__ proj, long long ld, const float *bias, float *state, StackSpans sp,
                                    void *__restrict__ out, int n) {
  const int s = blockIdx.x;
  const int i = blockIdx.y * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int tok0 = sp.sp_tok0[s], len = sp.sp_len[s], pos0 = sp.sp_pos0[s], slot = sp.sp_slot[s];
  const float bz = bias ? bias[i] : 0.f, bu = bias ? bias[n + i] : 0.f, bg = bias ? bias[2 * (long long)n + i] : 0.f;
  float S = pos0 > 0 ? state[(long long)slot * n + i] : 0.f;
  constexpr int U = 8;  // the gates read only the current token: eight tokens' inputs are fetched before the chain runs over them
  for (int t0 = 0; t0 < len; t0 += U) {
    float pz[U], pu[U], pg[U];
#pragma unroll
    for (int k = 0; k < U; k++) {
      const float *row = proj + (long long)(tok0 + min(t0 + k, len - 1)) * ld;
      pz[k] = row[i] + bz; pu[k] = row[n + i] + bu; pg[k] = row[2 * (long long)n + i] + bg;
    }
#pragma unroll
    for (int k = 0; k < U; k++) {
      if (t0 + k >= len) break;
      const float z = sigmoid_precise(pz[k]);
      const float c = pu[k] >= 0.f ? pu[k] + 0.5f : sigmoid_precise(pu[k]);
      S = (1.f - z) * S + z * c;
      st_el<F32>(out, (long long)(tok0 + t0 + k) * n + i, S * silu_(pg[k]));
    }
  }
  state[(long long)slot * n + i] = S;
}
// Long spans: a block owns 32 channels (lanes) and cuts the span into kGruSlices time slices (warps).  The update is linear in the
// state, S_t = (1 - z_t) S_(t-1) + z_t c_t, so a slice is summarised by the pair (A, B) with S_end = A S_begin + B; the warps
// exchange the pairs through shared memory, each folds the pairs of the slices before its own onto the slot's state, and
// then walks its slice a second time from that state, writing the outputs.
constexpr int kGruSlices = 16;
template <bool F32>
__global__ void __launch_bounds__(kGruSlices * 32) stack_mingru_sliced_kernel(const float *__restrict__ proj, long long ld,
                                                                              const float *bias, float *state, StackSpans sp,
                                                                              void *__restrict__ out, int n, int n_cb) {
  __shared__ float As[kGruSlices][32], Bs[kGruSlices][32];
  const int s = blockIdx.x / n_cb, cb = blockIdx.x - s * n_cb;
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  const int i = cb * 32 + l;
  const bool on = i < n;
  const int tok0 = sp.sp_tok0[s], len = sp.sp_len[s], pos0 = sp.sp_pos0[s], slot = sp.sp_slot[s];
  const int per = (len + kGruSlices - 1) / kGruSlices;
  const int t_lo = min(len, w * per), t_hi = min(len, t_lo + per);
  constexpr int U = 8;
  const float bz = bias && on ? bias[i] : 0.f, bu = bias && on ? bias[n + i] : 0.f, bg = bias && on ? bias[2 * (long long)n + i] : 0.f;
  float A = 1.f, B = 0.f;
  for (int t0 = t_lo; t0 < t_hi && on; t0 += U) {
    float pz[U], pu[U];
#pragma unroll
    for (int k = 0; k < U; k++) {
      const float *row = proj + (long long)(tok0 + min(t0 + k, t_hi - 1)) * ld;
      pz[k] = row[i] + bz; pu[k] = row[n + i] + bu;
    }
#pragma unroll
    for (int k = 0; k < U; k++) {
      if (t0 + k >= t_hi) break;
      const float z = sigmoid_precise(pz[k]);
      const float c = pu[k] >= 0.f ? pu[k] + 0.5f : sigmoid_precise(pu[k]);
      A *= 1.f - z;
      B = (1.f - z) * B + z * c;
    }
  }
  As[w][l] = A; Bs[w][l] = B;
  __syncthreads();
  if (!on) return;
  float S = pos0 > 0 ? state[(long long)slot * n + i] : 0.f;
  for (int k = 0; k < w; k++) S = fmaf(As[k][l], S, Bs[k][l]);
  for (int t0 = t_lo; t0 < t_hi; t0 += U) {
    float pz[U], pu[U], pg[U];
#pragma unroll
    for (int k = 0; k < U; k++) {
      const float *row = proj + (long long)(tok0 + min(t0 + k, t_hi - 1)) * ld;
      pz[k] = row[i] + bz; pu[k] = row[n + i] + bu; pg[k] = row[2 * (long long)n + i] + bg;
    }
#pragma unroll
    for (int k = 0; k < U; k++) {
      if (t0 + k >= t_hi) break;
      const float z = sigmoid_precise(pz[k]);
      const float c = pu[k] >= 0.f ? pu[k] + 0.5f : sigmoid_precise(pu[k]);
      S = (1.f - z) * S + z * c;
      st_el<F32>(out, (long long)(tok0 + t0 + k) * n + i, S * silu_(pg[k]));
    }
  }
  // the state after the span: the last slice that holds tokens ends at the span's end
  if (t_hi == len && t_lo < len) state[(long long)slot * n + i] = S;
}

cudaError_t launch_stack_mingru(const float *proj, long long ld, const float *bias, float *state, const StackSpans &sp, void *out,
                                bool f32, int n, int max_len, cudaStream_t st) {
  if (max_len >= 4 * kGruSlices) {
    const int n_cb = (n + 31) / 32;
    if (f32) stack_mingru_sliced_kernel<true><<<sp.n_spans * n_cb, kGruSlices * 32, 0, st>>>(proj, ld, bias, state, sp, out, n, n_cb);
    else stack_mingru_sliced_kernel<false><<<sp.n_spans * n_cb, kGruSlices * 32, 0, st>>>(proj, ld, bias, state, sp, out, n, n_cb);
    return cudaGetLastError();
  }
  dim3 grid(sp.n_spans, (n + 127) / 128);
  if (f32) stack_mingru_kernel<true><<<grid, 128, 0, st>>>(proj, ld, bias, state, sp, out, n);
  else stack_mingru_kernel<false><<<grid, 128, 0, st>>>(proj, ld, bias, state, sp, out, n);
  return cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------ latent attention
// Rotation of coordinates (i, i + rot_dims/2), i < rot_dims/2, by the angle pos * base^(-2i/rot_dims); the rest passes.  The angle
// is formed in double so that position 5000 is as exact as position 5.
__device__ __forceinline__ float rotated(const float *v, int i, int rot_dims, int pos, float base) {
  const int half = rot_dims >> 1;
  if (i >= rot_dims) return v[i];
  const int p = i < half ? i : i - half;
  const double f = exp2(-2.0 * (double)p / (double)rot_dims * log2((double)base));
  double sn, cs;
  sincos((double)pos * f, &sn, &cs);
  return i < half ? (float)((double)v[i] * cs - (double)v[i + half] * sn) : (float)((double)v[i] * cs + (double)v[i - half] * sn);
}

template <bool F32>
__global__ void __launch_bounds__(128) stack_latent_prep_kernel(const float *proj, long long ld, int q_off, int dkv_off,
                                                                const float *dkv_norm, StackLatent c, StackSpans sp, float *qf,
                                                                void *pool, const int *page_table, int max_pages, int page_size) {
  __shared__ float sh[32];
  const int t = blockIdx.x;
  const float *row = proj + (long long)t * ld;
  const int pos = sp.pos[t];
  const int D = c.r + c.dr;
  for (int i = threadIdx.x; i < c.H * c.dr; i += blockDim.x) {
    const int h = i / c.dr, k = i % c.dr;
    qf[((long long)t * c.H + h) * D + c.r + k] = rotated(row + q_off + (long long)h * (c.d + c.dr) + c.d, k, c.rot_dims, pos, c.rot_base);
  }
  if (!pool) return;
  const int slot = sp.slot[t];
  const long long prow = (long long)page_table[(long long)slot * max_pages + pos / page_size] * page_size + pos % page_size;
  const float *dk = row + dkv_off;
  float s = 0.f;
  for (int i = threadIdx.x; i < c.r; i += blockDim.x) s += dk[i] * dk[i];
  s = block_sum(s, sh);
  const float k = rsqrtf(s / (float)c.r + c.eps);
  for (int i = threadIdx.x; i < c.r; i += blockDim.x) st_el<F32>(pool, prow * D + i, dk[i] * k * dkv_norm[i]);
  for (int i = threadIdx.x; i < c.dr; i += blockDim.x) st_el<F32>(pool, prow * D + c.r + i, rotated(dk + c.r, i, c.rot_dims, pos, c.rot_base));
}
cudaError_t launch_stack_latent_prep(const float *proj, long long ld, int q_off, int dkv_off, const float *dkv_norm,
                                     const StackLatent &c, const StackSpans &sp, float *qf, void *pool, bool f32,
                                     const int *page_table, int max_pages, int page_size, cudaStream_t st) {
  if (f32) stack_latent_prep_kernel<true><<<sp.T, 128, 0, st>>>(proj, ld, q_off, dkv_off, dkv_norm, c, sp, qf, pool, page_table, max_pages, page_size);
  else stack_latent_prep_kernel<false><<<sp.T, 128, 0, st>>>(proj, ld, q_off, dkv_off, dkv_norm, c, sp, qf, pool, page_table, max_pages, page_size);
  return cudaGetLastError();
}

// One CTA per query block (tokens of one span) over all heads: 32-key tiles of the sequence's pool rows are staged in shared
// memory as fp32 and shared by every (token, head) pair of the block; one warp per pair at a time: a lane scores one key of the
// tile against the pair's query (latent part absorbed into the query, rotated part appended), the warp keeps a running maximum
// that starts at the head's sink and a running denominator that starts at exp(sink - max) = 1, and lanes own coordinates of
// the output latent.  Per-pair running state lives in shared memory between tiles.
constexpr int kLatTile = 32, kLatWarps = 8, kLatMaxR = 1024, kLatMaxSplit = 64;

int stack_latent_block_tokens(const StackLatent &c) {
  // shared memory: tile [32][D+1] + [warps][32] weights + per pair (D query + r accumulators + 2)
  const int D = c.r + c.dr;
  int bq = 8;
  while (bq > 1 && ((size_t)kLatTile * (D + 1 + kLatWarps) + (size_t)bq * c.H * (D + c.r + 2)) * 4 > 200 * 1024) bq >>= 1;
  return bq;
}

template <bool F32>
__global__ void __launch_bounds__(kLatWarps * 32) stack_latent_attn_kernel(const float *qf, const void *pool, const float *sink,
                                                                           StackLatent c, StackSpans sp, const int *qb_tok0,
                                                                           const int *qb_len, const int *page_table, int max_pages,
                                                                           int page_size, float *ol, int keys_per_split, float *part) {
  extern __shared__ float shm[];
  const int D = c.r + c.dr, DP = D + 1, r = c.r;
  const int tok0 = qb_tok0[blockIdx.x], nq = qb_len[blockIdx.x];
  const int pairs = nq * c.H;
  float *tile = shm;                                // [32][DP]
  float *qs = tile + (size_t)kLatTile * DP;        // [pairs][D]
  float *acc = qs + (size_t)pairs * D;             // [pairs][r]
  float *mx = acc + (size_t)pairs * r;             // [pairs]
  float *dn = mx + pairs;                          // [pairs]
  float *prs = dn + pairs;                         // [warps][32]
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  const int slot = sp.slot[tok0];
  const int last_pos = sp.pos[tok0 + nq - 1];
  for (int i = threadIdx.x; i < pairs * D; i += blockDim.x) qs[i] = qf[(long long)tok0 * c.H * D + i];
  for (int i = threadIdx.x; i < pairs * r; i += blockDim.x) acc[i] = 0.f;
  // the whole history in one CTA: the running maximum starts at the head's sink and the denominator at exp(sink - max) = 1;
  // one slice of the history (blockIdx.y, keys_per_split keys): both start empty and the sink joins when the slices are merged
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) { mx[i] = part ? -INFINITY : sink[i % c.H]; dn[i] = part ? 0.f : 1.f; }
  const int *pt = page_table + (long long)slot * max_pages;
  const int k_begin = part ? (int)blockIdx.y * keys_per_split : 0;
  const int k_end = part ? min(last_pos + 1, k_begin + keys_per_split) : last_pos + 1;
  for (int k0 = k_begin; k0 < k_end; k0 += kLatTile) {
    const int nk = min(kLatTile, k_end - k0);
    __syncthreads();
    if (!F32 && (D & 7) == 0) {  // a row of the pool is D bf16 values, 16-byte aligned: eight per load
      const int vpr = D >> 3;
      for (int i = threadIdx.x; i < nk * vpr; i += blockDim.x) {
        const int kk = i / vpr, cv = i - kk * vpr, kp = k0 + kk;
        const long long prow = (long long)pt[kp / page_size] * page_size + kp % page_size;
        const uint4 v = *reinterpret_cast<const uint4 *>(reinterpret_cast<const uint16_t *>(pool) + prow * D + cv * 8);
        float *dst = tile + (size_t)kk * DP + cv * 8;
        const uint32_t w4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int j = 0; j < 4; j++) {
          dst[2 * j] = __uint_as_float(w4[j] << 16);
          dst[2 * j + 1] = __uint_as_float(w4[j] & 0xffff0000u);
        }
      }
    } else {
      for (int i = threadIdx.x; i < nk * D; i += blockDim.x) {
        const int kk = i / D, cc = i % D, kp = k0 + kk;
        const long long prow = (long long)pt[kp / page_size] * page_size + kp % page_size;
        tile[(size_t)kk * DP + cc] = ld_el<F32>(pool, prow * D + cc);
      }
    }
    __syncthreads();
    for (int p = w; p < pairs; p += kLatWarps) {
      const int qpos = sp.pos[tok0 + p / c.H];
      const float *q = qs + (size_t)p * D;
      float sc = -INFINITY;
      if (l < nk && k0 + l <= qpos) {
        const float *kr = tile + (size_t)l * DP;
        float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;  // four chains, added at the end: the sum's order is fixed by D alone
        int i = 0;
        for (; i + 3 < D; i += 4) {
          s0 = fmaf(q[i], kr[i], s0); s1 = fmaf(q[i + 1], kr[i + 1], s1);
          s2 = fmaf(q[i + 2], kr[i + 2], s2); s3 = fmaf(q[i + 3], kr[i + 3], s3);
        }
        for (; i < D; i++) s0 = fmaf(q[i], kr[i], s0);
        sc = ((s0 + s1) + (s2 + s3)) * c.scale;
      }
      const float m_old = mx[p];
      const float m_new = fmaxf(m_old, warp_max(sc));
      const float pr = sc == -INFINITY ? 0.f : expf(sc - m_new);
      const float corr = m_old == -INFINITY ? 0.f : expf(m_old - m_new);
      const float psum = warp_sum(pr);
      float *a = acc + (size_t)p * r;
      float *pw = prs + w * kLatTile;  // the tile's weights of this pair: lanes own coordinates below, so every lane reads all
      pw[l] = pr;
      __syncwarp();
      for (int j = l; j < r; j += 32) {
        float v0 = a[j] * corr, v1 = 0.f, v2 = 0.f, v3 = 0.f;
        int kk = 0;
        for (; kk + 3 < nk; kk += 4) {
          v0 = fmaf(pw[kk], tile[(size_t)kk * DP + j], v0); v1 = fmaf(pw[kk + 1], tile[(size_t)(kk + 1) * DP + j], v1);
          v2 = fmaf(pw[kk + 2], tile[(size_t)(kk + 2) * DP + j], v2); v3 = fmaf(pw[kk + 3], tile[(size_t)(kk + 3) * DP + j], v3);
        }
        for (; kk < nk; kk++) v0 = fmaf(pw[kk], tile[(size_t)kk * DP + j], v0);
        a[j] = (v0 + v1) + (v2 + v3);
      }
      __syncwarp();
      if (l == 0) { mx[p] = m_new; dn[p] = dn[p] * corr + psum; }
      __syncwarp();
    }
  }
  __syncthreads();
  if (!part) {
    for (int i = threadIdx.x; i < pairs * r; i += blockDim.x) ol[(long long)tok0 * c.H * r + i] = acc[i] / dn[i / r];
    return;
  }
  // slice record per pair: r unnormalised sums, then the slice's maximum and denominator
  float *rec = part + ((long long)blockIdx.y * sp.T * c.H + (long long)tok0 * c.H) * (r + 2);
  for (int i = threadIdx.x; i < pairs * r; i += blockDim.x) rec[(long long)(i / r) * (r + 2) + i % r] = acc[i];
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) { rec[(long long)i * (r + 2) + r] = mx[i]; rec[(long long)i * (r + 2) + r + 1] = dn[i]; }
}

// ---- the same attention on mma.sync (bf16 compute type, kv_rank a multiple of 8, kv_rank + rot_dim a multiple of 16, at most 16
// (token, head) pairs per query block): the pairs are the 16 rows of m16n8k16 products.  A CTA stages 64 latents of its slice
// as bf16, warp w scores keys 8w .. 8w+7 against all pairs (K = kv_rank + rot_dim), the scores go through shared memory for the
// online softmax (fp32, two rows per warp, starting at the sink as above), and each warp then adds P C into the output
// coordinates it owns (n-tiles w, w + 8, ...), which stay in registers over the whole slice.
__device__ __forceinline__ void mma_bf16_m16n8k16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
constexpr int kMmaKeys = 64, kMmaRows = 16, kMmaPS = 72;
bool stack_latent_mma_ok(const StackLatent &c, bool f32) {
  return !f32 && c.r % 8 == 0 && (c.r + c.dr) % 16 == 0 && c.r <= kLatMaxR && c.H <= kMmaRows;
}
static size_t latent_mma_smem(const StackLatent &c) {
  const size_t DS = (size_t)c.r + c.dr + 8;
  return (kMmaRows + kMmaKeys) * DS * 2 + (size_t)kMmaRows * kMmaKeys * 4 + (size_t)kMmaRows * kMmaPS * 2 + 4 * kMmaRows * 4;
}
template <int NTW>
__global__ void __launch_bounds__(256) stack_latent_attn_mma_kernel(const float *qf, const uint16_t *pool, const float *sink, StackLatent c,
                                                                    StackSpans sp, const int *qb_tok0, const int *qb_len,
                                                                    const int *page_table, int max_pages, int page_size, float *ol,
                                                                    int keys_per_split, float *part) {
  extern __shared__ __align__(16) unsigned char smraw[];
  const int D = c.r + c.dr, r = c.r, DS = D + 8;
  uint16_t *qs = reinterpret_cast<uint16_t *>(smraw);                  // [16][DS]
  uint16_t *tile = qs + (size_t)kMmaRows * DS;                         // [64][DS]
  float *S = reinterpret_cast<float *>(tile + (size_t)kMmaKeys * DS);  // [16][64]
  uint16_t *P = reinterpret_cast<uint16_t *>(S + kMmaRows * kMmaKeys); // [16][72]
  float *mx = reinterpret_cast<float *>(P + kMmaRows * kMmaPS);        // [16]
  float *dn = mx + kMmaRows, *cr = dn + kMmaRows;                      // [16] each
  int *qp = reinterpret_cast<int *>(cr + kMmaRows);                    // [16] position of the row's query, -1 for a padding row
  __shared__ long long prow_s[kMmaKeys];
  const int tok0 = qb_tok0[blockIdx.x], nq = qb_len[blockIdx.x];
  const int pairs = nq * c.H;
  if (pairs > kMmaRows) return;  // the host cuts query blocks to fit
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, g = l >> 2, tig = l & 3;
  const int slot = sp.slot[tok0];
  const int last_pos = sp.pos[tok0 + nq - 1];
  {  // queries: four floats per load, four loads in flight per thread before the first is converted and stored
    const int n4 = kMmaRows * D / 4;
    const float4 *src = reinterpret_cast<const float4 *>(qf + (long long)tok0 * c.H * D);
    for (int i0 = threadIdx.x; i0 < n4; i0 += 4 * blockDim.x) {
      float4 v[4];
#pragma unroll
      for (int u = 0; u < 4; u++) {
        const int i = i0 + u * blockDim.x;
        v[u] = (i < n4 && i * 4 < pairs * D) ? src[i] : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int u = 0; u < 4; u++) {
        const int i = i0 + u * blockDim.x;
        if (i < n4) {
          const int row = (i * 4) / D, col = i * 4 - row * D;
          *reinterpret_cast<uint2 *>(qs + (size_t)row * DS + col) = make_uint2(float2_to_bf16x2(v[u].x, v[u].y), float2_to_bf16x2(v[u].z, v[u].w));
        }
      }
    }
  }
  if (threadIdx.x < kMmaRows) {
    const int row = threadIdx.x;
    mx[row] = part ? -INFINITY : (row < pairs ? sink[row % c.H] : 0.f);
    dn[row] = part ? 0.f : 1.f;
    qp[row] = row < pairs ? sp.pos[tok0 + row / c.H] : -1;
  }
  float acc[NTW][4];
#pragma unroll
  for (int nt = 0; nt < NTW; nt++) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
  const int *pt = page_table + (long long)slot * max_pages;
  const int k_begin = part ? (int)blockIdx.y * keys_per_split : 0;
  const int k_end = part ? min(last_pos + 1, k_begin + keys_per_split) : last_pos + 1;
  const int vpr = D >> 3;
  for (int k0 = k_begin; k0 < k_end; k0 += kMmaKeys) {
    const int nk = min(kMmaKeys, k_end - k0);
    __syncthreads();
    if (threadIdx.x < kMmaKeys) {  // pool row of every key of the tile, so that the loads below do not wait on the page table
      const int kp = k0 + threadIdx.x;
      prow_s[threadIdx.x] = threadIdx.x < nk ? (long long)pt[kp / page_size] * page_size + kp % page_size : -1;
    }
    __syncthreads();
    for (int i0 = threadIdx.x; i0 < kMmaKeys * vpr; i0 += 6 * blockDim.x) {
      uint4 v[6];
#pragma unroll
      for (int u = 0; u < 6; u++) {
        const int i = i0 + u * blockDim.x;
        v[u] = make_uint4(0u, 0u, 0u, 0u);  // rows past the slice's end are zero: their weights are zero too
        if (i < kMmaKeys * vpr) {
          const int kk = i / vpr, cv = i - kk * vpr;
          const long long prow = prow_s[kk];
          if (prow >= 0) v[u] = *reinterpret_cast<const uint4 *>(pool + prow * D + cv * 8);
        }
      }
#pragma unroll
      for (int u = 0; u < 6; u++) {
        const int i = i0 + u * blockDim.x;
        if (i < kMmaKeys * vpr) {
          const int kk = i / vpr, cv = i - kk * vpr;
          *reinterpret_cast<uint4 *>(tile + (size_t)kk * DS + cv * 8) = v[u];
        }
      }
    }
    __syncthreads();
    {  // scores of keys 8w .. 8w+7
      float sa[4] = {0.f, 0.f, 0.f, 0.f};
      const uint16_t *qa = qs + (size_t)g * DS + 2 * tig, *qb = qs + (size_t)(g + 8) * DS + 2 * tig;
      const uint16_t *kb = tile + (size_t)(w * 8 + g) * DS + 2 * tig;
      for (int k = 0; k < D; k += 16) {
        const uint32_t a0 = *reinterpret_cast<const uint32_t *>(qa + k), a1 = *reinterpret_cast<const uint32_t *>(qb + k);
        const uint32_t a2 = *reinterpret_cast<const uint32_t *>(qa + k + 8), a3 = *reinterpret_cast<const uint32_t *>(qb + k + 8);
        const uint32_t b0 = *reinterpret_cast<const uint32_t *>(kb + k), b1 = *reinterpret_cast<const uint32_t *>(kb + k + 8);
        mma_bf16_m16n8k16(sa, a0, a1, a2, a3, b0, b1);
      }
#pragma unroll
      for (int e = 0; e < 4; e++) {
        const int row = g + (e >> 1) * 8, col = w * 8 + 2 * tig + (e & 1);
        const bool seen = col < nk && k0 + col <= qp[row];
        S[row * kMmaKeys + col] = seen ? sa[e] * c.scale : -INFINITY;
      }
    }
    __syncthreads();
#pragma unroll
    for (int rr = 0; rr < 2; rr++) {
      const int row = 2 * w + rr;
      const float s0 = S[row * kMmaKeys + l], s1 = S[row * kMmaKeys + l + 32];
      const float m_old = mx[row];
      const float m_new = fmaxf(m_old, warp_max(fmaxf(s0, s1)));
      const float p0 = s0 == -INFINITY ? 0.f : expf(s0 - m_new), p1 = s1 == -INFINITY ? 0.f : expf(s1 - m_new);
      const float corr = m_old == -INFINITY ? 0.f : expf(m_old - m_new);
      const float psum = warp_sum(p0 + p1);
      P[row * kMmaPS + l] = float_to_bf16_bits(p0);
      P[row * kMmaPS + l + 32] = float_to_bf16_bits(p1);
      __syncwarp();
      if (l == 0) { mx[row] = m_new; dn[row] = dn[row] * corr + psum; cr[row] = corr; }
    }
    __syncthreads();
    const float c_lo = cr[g], c_hi = cr[g + 8];
#pragma unroll
    for (int nt = 0; nt < NTW; nt++) { acc[nt][0] *= c_lo; acc[nt][1] *= c_lo; acc[nt][2] *= c_hi; acc[nt][3] *= c_hi; }
    const int ksteps = (nk + 15) >> 4;
    for (int ks = 0; ks < ksteps; ks++) {
      const int kk = ks * 16;
      const uint32_t a0 = *reinterpret_cast<const uint32_t *>(P + g * kMmaPS + kk + 2 * tig);
      const uint32_t a1 = *reinterpret_cast<const uint32_t *>(P + (g + 8) * kMmaPS + kk + 2 * tig);
      const uint32_t a2 = *reinterpret_cast<const uint32_t *>(P + g * kMmaPS + kk + 8 + 2 * tig);
      const uint32_t a3 = *reinterpret_cast<const uint32_t *>(P + (g + 8) * kMmaPS + kk + 8 + 2 * tig);
      const uint16_t *t0 = tile + (size_t)(kk + 2 * tig) * DS + g;
#pragma unroll
      for (int nt = 0; nt < NTW; nt++) {
        const int n0 = (w + nt * 8) * 8;
        if (n0 < r) {
          const uint32_t b0 = (uint32_t)t0[n0] | ((uint32_t)t0[n0 + DS] << 16);
          const uint32_t b1 = (uint32_t)t0[n0 + 8 * (size_t)DS] | ((uint32_t)t0[n0 + 9 * (size_t)DS] << 16);
          mma_bf16_m16n8k16(acc[nt], a0, a1, a2, a3, b0, b1);
        }
      }
    }
  }
  __syncthreads();
#pragma unroll
  for (int nt = 0; nt < NTW; nt++) {
    const int n0 = (w + nt * 8) * 8;
    if (n0 >= r) continue;
#pragma unroll
    for (int e = 0; e < 4; e++) {
      const int row = g + (e >> 1) * 8, col = n0 + 2 * tig + (e & 1);
      if (row >= pairs) continue;
      if (!part) ol[((long long)tok0 * c.H + row) * r + col] = acc[nt][e] / dn[row];
      else part[((long long)blockIdx.y * sp.T * c.H + (long long)tok0 * c.H + row) * (r + 2) + col] = acc[nt][e];
    }
  }
  if (part && threadIdx.x < pairs) {
    float *rec = part + ((long long)blockIdx.y * sp.T * c.H + (long long)tok0 * c.H + threadIdx.x) * (r + 2);
    rec[r] = mx[threadIdx.x]; rec[r + 1] = dn[threadIdx.x];
  }
}

// Merge of the slices: out = sum_s acc_s e^(m_s - M) / (e^(sink - M) + sum_s l_s e^(m_s - M)), M = max(sink, max_s m_s).
__global__ void stack_latent_merge_kernel(const float *part, const float *sink, int n_split, int pairs_total, int H, int r, float *ol) {
  __shared__ float ws[kLatMaxSplit];  // per slice e^(m_s - M), 0 for an empty slice
  __shared__ float inv_den;
  const int p = blockIdx.x;
  const float sk = sink[p % H];
  float M = sk;
  for (int s = 0; s < n_split; s++) M = fmaxf(M, part[((long long)s * pairs_total + p) * (r + 2) + r]);
  for (int s = threadIdx.x; s < n_split; s += blockDim.x) {
    const float m = part[((long long)s * pairs_total + p) * (r + 2) + r];
    ws[s] = m == -INFINITY ? 0.f : expf(m - M);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float den = expf(sk - M);
    for (int s = 0; s < n_split; s++) den += part[((long long)s * pairs_total + p) * (r + 2) + r + 1] * ws[s];
    inv_den = 1.f / den;
  }
  __syncthreads();
  for (int j = threadIdx.x; j < r; j += blockDim.x) {
    float v = 0.f;
    for (int s = 0; s < n_split; s++) v = fmaf(part[((long long)s * pairs_total + p) * (r + 2) + j], ws[s], v);
    ol[(long long)p * r + j] = v * inv_den;
  }
}

// ---- latent attention of long prompt portions as matrix products (bf16 operands, fp32 accumulation): the sequence's latents
// are copied out of their pages into one contiguous matrix and its transpose, scores = Q C^T and outputs = P C run on the
// tensor-core product, and the kernel between them turns a block of score rows into softmax weights (fp32, causal, sink).
__global__ void stack_latent_gather_kernel(const uint16_t *pool, const int *pt, int page_size, int D, int r, int ctx, int ctx8,
                                           uint16_t *cg, uint16_t *cgt) {
  const int kp = blockIdx.x;
  const long long prow = kp < ctx ? (long long)pt[kp / page_size] * page_size + kp % page_size : 0;
  for (int c = threadIdx.x; c < D; c += blockDim.x) {
    const uint16_t v = kp < ctx ? pool[prow * D + c] : (uint16_t)0;
    cg[(long long)kp * D + c] = v;
    if (c < r) cgt[(long long)c * ctx8 + kp] = v;
  }
}
cudaError_t launch_stack_latent_gather(const void *pool, const int *pt_row, int page_size, int D, int r, int ctx, int ctx8,
                                       uint16_t *cg, uint16_t *cgt, cudaStream_t st) {
  stack_latent_gather_kernel<<<ctx8, 128, 0, st>>>(reinterpret_cast<const uint16_t *>(pool), pt_row, page_size, D, r, ctx, ctx8, cg, cgt);
  return cudaGetLastError();
}

// Row (t, h) of S [rows][ld] holds the raw scores of the query at position pos_first + t against keys 0 .. ld-1.
__global__ void __launch_bounds__(256) stack_latent_softmax_kernel(const float *S, int ld, const float *sink, int H, int pos_first,
                                                                   float scale, uint16_t *P) {
  __shared__ float sh[32];
  const long long row = blockIdx.x;
  const int h = (int)(row % H), qpos = pos_first + (int)(row / H);
  const float *s = S + row * ld;
  const int nk = min(ld, qpos + 1);
  const float sk = sink[h];
  float m = sk;
  for (int k = threadIdx.x; k < nk; k += blockDim.x) m = fmaxf(m, s[k] * scale);
  m = warp_max(m);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = m;
  __syncthreads();
  for (int i = 0; i < (int)(blockDim.x >> 5); i++) m = fmaxf(m, sh[i]);
  float sum = 0.f;
  for (int k = threadIdx.x; k < nk; k += blockDim.x) sum += expf(s[k] * scale - m);
  sum = block_sum(sum, sh) + expf(sk - m);
  const float inv = 1.f / sum;
  uint16_t *p = P + row * ld;
  for (int k = threadIdx.x; k < ld; k += blockDim.x) p[k] = k < nk ? float_to_bf16_bits(expf(s[k] * scale - m) * inv) : (uint16_t)0;
}
cudaError_t launch_stack_latent_softmax(const float *S, int rows, int ld, const float *sink, int H, int pos_first, float scale,
                                        uint16_t *P, cudaStream_t st) {
  if (rows <= 0) return cudaSuccess;
  stack_latent_softmax_kernel<<<rows, 256, 0, st>>>(S, ld, sink, H, pos_first, scale, P);
  return cudaGetLastError();
}

cudaError_t launch_stack_latent_attn(const float *qf, const void *pool, bool f32, const float *sink, const StackLatent &c,
                                     const StackSpans &sp, const int *qb_tok0, const int *qb_len, int n_qb, const int *page_table,
                                     int max_pages, int page_size, float *ol, int n_split, int keys_per_split, float *part,
                                     cudaStream_t st) {
  if (n_qb <= 0) return cudaSuccess;
  if (c.r > kLatMaxR) return cudaErrorInvalidValue;
  if (n_split <= 1 || !part) { n_split = 1; part = nullptr; }
  if (n_split > kLatMaxSplit) return cudaErrorInvalidValue;
  static int use_mma = -1;
  if (use_mma < 0) { const char *e = getenv("DIS_STACK_LATENT_MMA"); use_mma = (e && atoi(e) == 0) ? 0 : 1; }
  if (use_mma && stack_latent_mma_ok(c, f32)) {
    const size_t shm = latent_mma_smem(c);
    static DeviceOnce once_mma;
    DIS_CUDA_TRY(once_mma.run([&] {
      cudaError_t e = cudaFuncSetAttribute(stack_latent_attn_mma_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
      return e != cudaSuccess ? e : cudaFuncSetAttribute(stack_latent_attn_mma_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
    }));
    if (shm > 220 * 1024) return cudaErrorInvalidValue;
    const dim3 grid(n_qb, n_split);
    const uint16_t *pl = reinterpret_cast<const uint16_t *>(pool);
    if (c.r <= 512) stack_latent_attn_mma_kernel<8><<<grid, 256, shm, st>>>(qf, pl, sink, c, sp, qb_tok0, qb_len, page_table, max_pages, page_size, ol, keys_per_split, part);
    else stack_latent_attn_mma_kernel<16><<<grid, 256, shm, st>>>(qf, pl, sink, c, sp, qb_tok0, qb_len, page_table, max_pages, page_size, ol, keys_per_split, part);
    if (part) stack_latent_merge_kernel<<<sp.T * c.H, 128, 0, st>>>(part, sink, n_split, sp.T * c.H, c.H, c.r, ol);
    return cudaGetLastError();
  }
  const int D = c.r + c.dr, bq = stack_latent_block_tokens(c);
  const size_t sh = ((size_t)kLatTile * (D + 1 + kLatWarps) + (size_t)bq * c.H * (D + c.r + 2)) * sizeof(float);
  if (sh > 220 * 1024) return cudaErrorInvalidValue;
  static DeviceOnce once;
  DIS_CUDA_TRY(once.run([&] {
    cudaError_t e = cudaFuncSetAttribute(stack_latent_attn_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
    return e != cudaSuccess ? e : cudaFuncSetAttribute(stack_latent_attn_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
  }));
  const dim3 grid(n_qb, n_split);
  if (f32) stack_latent_attn_kernel<true><<<grid, kLatWarps * 32, sh, st>>>(qf, pool, sink, c, sp, qb_tok0, qb_len, page_table, max_pages, page_size, ol, keys_per_split, part);
  else stack_latent_attn_kernel<false><<<grid, kLatWarps * 32, sh, st>>>(qf, pool, sink, c, sp, qb_tok0, qb_len, page_table, max_pages, page_size, ol, keys_per_split, part);
  if (part) stack_latent_merge_kernel<<<sp.T * c.H, 128, 0, st>>>(part, sink, n_split, sp.T * c.H, c.H, c.r, ol);
  return cudaGetLastError();
}

}  // namespace dis
