// k_stack_attn.cu -- grouped-query attention over paged keys and values for the layer-list decoders (DIS_MIX_ATTENTION and the
// attention half of DIS_MIX_PARALLEL): the per-token preparation (biases, whole-projection or per-head query/key norm, partial
// rotary with a frequency table, cache write of the rotated keys and of the values -- own projection or the unrotated keys,
// optionally rotated by their position; a layer that reads another layer's cache writes nothing) and the attention itself with
// softmax (optionally with a per-head sink logit in the denominator) or per-head sigmoid weights, under a causal mask that may
// be cut into chunks of positions, over the whole visible history or a slice of it, with an optional per-head sigmoid gate on
// the output.  Scores, weights, norms and angles are fp32 (angles are formed in double) whatever the cache's element type.
#include "stack_dev.cuh"

namespace dis {

// ------------------------------------------------------------------------------------------------ preparation
// One block per token.  proj row: queries at q_off [H][d], keys at k_off [G][d], values at v_off [G][dv] (unless values are
// the keys).  `bias` (or null): one entry per column of the projection, added here when the product left it out.
// kpool == null: the layer reads another layer's cache; only the queries are prepared.
// n_part > 1: the projection comes as split-K slices (slice stride `stride`); the block first sums its token's row of n_cols
// columns (and the bias) into shared memory and works from there.  gate_out (or null): receives columns gate_off .. + H of the
// row (the logits of the output gates, which the attention kernel reads from memory).
template <bool F32>
__global__ void __launch_bounds__(128) stack_attn_prep_kernel(const float *proj, long long ld, int n_part, long long stride, int n_cols,
                                                              int gate_off, float *gate_out, long long ld_gate, int q_off, int k_off, int v_off,
                                                              const float *bias, const float *qn, const float *kn, const double *freq,
                                                              const double *vfreq, StackAttn c, StackSpans sp, float *qf, void *kpool,
                                                              void *vpool, float *vrot, const int *page_table, int max_pages,
                                                              int page_size) {
  extern __shared__ __align__(16) float tab[];  // cos [half], sin [half], value cos [dv/2], value sin [dv/2], per-head factors [H + G], summed row
  const int srow_off = (c.rot_dims + c.dv + c.H + c.G + 3) & ~3;  // the summed row starts on a 16-byte boundary
  __shared__ float sh[32];
  const int t = blockIdx.x;
  const float *row = proj + (long long)t * ld;
  if (n_part > 1) {
    float *srow = tab + srow_off;
    if ((((int)(ld & 3)) | (int)(stride & 3) | (n_cols & 3)) == 0) {  // 16-byte loads of every slice, all independent
      for (int i = threadIdx.x * 4; i < n_cols; i += blockDim.x * 4) {
        float4 v = bias ? *reinterpret_cast<const float4 *>(bias + i) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
        for (int k = 0; k < n_part; k++) {
          const float4 p = *reinterpret_cast<const float4 *>(row + (long long)k * stride + i);
          v.x += p.x; v.y += p.y; v.z += p.z; v.w += p.w;
        }
        *reinterpret_cast<float4 *>(srow + i) = v;
      }
    } else
    for (int i = threadIdx.x; i < n_cols; i += blockDim.x) {
      float v = bias ? bias[i] : 0.f;
      for (int k = 0; k < n_part; k++) v += row[(long long)k * stride + i];
      srow[i] = v;
    }
    row = srow;
    bias = nullptr;
    __syncthreads();
  }
  if (gate_out)
    for (int i = threadIdx.x; i < c.H; i += blockDim.x) gate_out[(long long)t * ld_gate + i] = row[gate_off + i];
  const int pos = sp.pos[t], slot = sp.slot[t];
  const int half = c.rot_dims >> 1, vhalf = c.dv >> 1;
  const bool rot_v = (c.flags & DIS_ATTN_ROT_V) != 0, own = kpool != nullptr;
  float *cs = tab, *sn = tab + half, *vcs = sn + half, *vsn = vcs + vhalf, *hr = vsn + vhalf;
  // the angle pos * f is formed and brought into [-pi, pi] in double (position 100000 is then as exact as position 5); sine and
  // cosine of the reduced angle are float
  auto angle = [](int p, double f, float *sn_out, float *cs_out) {
    const double a = (double)p * f;
    const double r = a - 6.283185307179586476925 * rint(a * 0.15915494309189533577);
    sincosf((float)r, sn_out, cs_out);
  };
  for (int i = threadIdx.x; i < half; i += blockDim.x) angle(pos, freq[i], &sn[i], &cs[i]);
  if (rot_v)
    for (int i = threadIdx.x; i < vhalf; i += blockDim.x) {
      float s_, c_;
      angle(pos, vfreq[i], &s_, &c_);
      vcs[i] = c_; vsn[i] = s_;
      vrot[(long long)t * c.dv + i] = c_;
      vrot[(long long)t * c.dv + vhalf + i] = s_;
    }
  const int nq = c.H * c.d, nk = c.G * c.d;
  const float *qb = bias ? bias + q_off : nullptr, *kb = bias ? bias + k_off : nullptr, *vb = bias ? bias + v_off : nullptr;
  const bool head_norm = (c.flags & DIS_ATTN_QK_NORM_HEAD) != 0;
  float rq = 1.f, rk = 1.f;
  if (c.flags & DIS_ATTN_QK_NORM) {
    float s = 0.f;
    for (int i = threadIdx.x; i < nq; i += blockDim.x) { const float v = row[q_off + i] + (qb ? qb[i] : 0.f); s += v * v; }
    rq = rsqrtf(block_sum(s, sh) / (float)nq + c.eps);
    s = 0.f;
    for (int i = threadIdx.x; i < nk; i += blockDim.x) { const float v = row[k_off + i] + (kb ? kb[i] : 0.f); s += v * v; }
    rk = rsqrtf(block_sum(s, sh) / (float)nk + c.eps);
  } else if (head_norm) {  // one factor per head: a warp per head at a time, query heads then key heads
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    for (int h = w; h < c.H + (own ? c.G : 0); h += (int)(blockDim.x >> 5)) {
      const bool isq = h < c.H;
      const int off = isq ? q_off + h * c.d : k_off + (h - c.H) * c.d;
      const float *b = isq ? (qb ? qb + h * c.d : nullptr) : (kb ? kb + (h - c.H) * c.d : nullptr);
      float s = 0.f;
      for (int i = l; i < c.d; i += 32) { const float v = row[off + i] + (b ? b[i] : 0.f); s += v * v; }
      s = warp_sum(s);
      if (l == 0) hr[h] = rsqrtf(s / (float)c.d + c.eps);
    }
  }
  __syncthreads();
  // g: the gain vector (whole projection, or [d] shared by the heads); r / rh: the factor of the projection or of each head
  auto val = [&](int off, const float *b, const float *g, float r, const float *rh, int i) {
    float v = row[off + i] + (b ? b[i] : 0.f);
    if (g) v = head_norm ? v * rh[i / c.d] * g[i % c.d] : v * r * g[i];
    return v;
  };
  auto rotated = [&](int off, const float *b, const float *g, float r, const float *rh, int i) {
    const int e = i % c.d;
    if (e >= c.rot_dims) return val(off, b, g, r, rh, i);
    if (e < half) return val(off, b, g, r, rh, i) * cs[e] - val(off, b, g, r, rh, i + half) * sn[e];
    return val(off, b, g, r, rh, i) * cs[e - half] + val(off, b, g, r, rh, i - half) * sn[e - half];
  };
  const bool normed = (c.flags & (DIS_ATTN_QK_NORM | DIS_ATTN_QK_NORM_HEAD)) != 0;
  const float *qg = normed ? qn : nullptr, *kg = normed ? kn : nullptr;
  for (int i = threadIdx.x; i < nq; i += blockDim.x) qf[(long long)t * nq + i] = rotated(q_off, qb, qg, rq, hr, i);
  if (!own) return;
  const long long prow = (long long)page_table[(long long)slot * max_pages + pos / page_size] * page_size + pos % page_size;
  for (int i = threadIdx.x; i < nk; i += blockDim.x) st_el<F32>(kpool, prow * nk + i, rotated(k_off, kb, kg, rk, hr + c.H, i));
  const int nv = c.G * c.dv;
  for (int i = threadIdx.x; i < nv; i += blockDim.x) {
    float v;
    if (c.flags & DIS_ATTN_V_IS_K) v = row[k_off + i] + (kb ? kb[i] : 0.f);  // dv == d: the keys as projected
    else if (!rot_v) v = row[v_off + i] + (vb ? vb[i] : 0.f);
    else {
      const int e = i % c.dv;
      auto vv = [&](int j) { return row[v_off + j] + (vb ? vb[j] : 0.f); };
      v = e < vhalf ? vv(i) * vcs[e] - vv(i + vhalf) * vsn[e] : vv(i) * vcs[e - vhalf] + vv(i - vhalf) * vsn[e - vhalf];
    }
    st_el<F32>(vpool, prow * nv + i, v);
  }
}
cudaError_t launch_stack_attn_prep(const float *proj, long long ld, int n_part, long long stride, int n_cols, int gate_off, float *gate_out,
                                   long long ld_gate, int q_off, int k_off, int v_off, const float *bias, const float *qn,
                                   const float *kn, const double *freq, const double *vfreq, const StackAttn &c, const StackSpans &sp,
                                   float *qf, void *kpool, void *vpool, float *vrot, bool f32, const int *page_table, int max_pages,
                                   int page_size, cudaStream_t st) {
  if (sp.T <= 0) return cudaSuccess;
  if (n_part < 1) n_part = 1;
  const size_t sh = (size_t)(((c.rot_dims + c.dv + c.H + c.G + 3) & ~3) + (n_part > 1 ? n_cols : 0)) * sizeof(float);
  if (sh > 200 * 1024) return cudaErrorInvalidValue;
  static DeviceOnce once;
  DIS_CUDA_TRY(once.run([&] {
    cudaError_t e = cudaFuncSetAttribute(stack_attn_prep_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    return e != cudaSuccess ? e : cudaFuncSetAttribute(stack_attn_prep_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
  }));
  if (f32) stack_attn_prep_kernel<true><<<sp.T, 128, sh, st>>>(proj, ld, n_part, stride, n_cols, gate_off, gate_out, ld_gate, q_off, k_off, v_off, bias, qn, kn, freq, vfreq, c, sp, qf, kpool, vpool, vrot, page_table, max_pages, page_size);
  else stack_attn_prep_kernel<false><<<sp.T, 128, sh, st>>>(proj, ld, n_part, stride, n_cols, gate_off, gate_out, ld_gate, q_off, k_off, v_off, bias, qn, kn, freq, vfreq, c, sp, qf, kpool, vpool, vrot, page_table, max_pages, page_size);
  return cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------ attention, fp32 arithmetic
// One CTA per (query block, key/value head, slice of the history).  The block's (token, query head of the group) pairs share
// 32-key tiles staged in shared memory as fp32; one warp per pair at a time: a lane scores one key, then lanes own value
// coordinates.  SIG: weight = sigmoid(score * temp[h] + pb[h]), plain sums.  Otherwise an online softmax (running maximum and
// denominator per pair).  Epilogue (whole history in one CTA) or merge kernel (slices): normalise, rotate the output back by
// the query's position when values were rotated, scale, and store into the mixer's output row.
constexpr int kAtTile = 32, kAtWarps = 8, kAtMaxSplit = 64;
bool stack_attn_mma_ok(const StackAttn &c, bool f32);
int stack_attn_mma_block_tokens(const StackAttn &c);

struct AttnOut {
  void *out;          // [T][ld] in the compute type; head h at columns off + h * dv
  long long ld;
  int off;
  float scale;        // factor on the output (weight of this mixer inside a parallel layer)
  const float *vrot;  // [T][dv]: cos | sin of the query position's value angles, or null
  const float *gate;  // [T][ldg]: logit of head h's output gate at column h, or null
  long long ldg;
};
// factor on head h's output at token tok: the mixer's weight times the head's sigmoid gate
__device__ __forceinline__ float attn_out_factor(const AttnOut &o, int tok, int h) {
  return o.gate ? o.scale * sigmoid_precise(o.gate[(long long)tok * o.ldg + h]) : o.scale;
}

template <bool F32>
__device__ __forceinline__ void attn_store(const AttnOut &o, const float *a, float inv, int tok, int h, int dv, int j) {
  float v = a[j] * inv;
  if (o.vrot) {  // rotation by minus the angle: (u, v) -> (u cos + v sin, v cos - u sin)
    const int hf = dv >> 1;
    const float *cs = o.vrot + (long long)tok * dv, *sn = cs + hf;
    v = j < hf ? (a[j] * cs[j] + a[j + hf] * sn[j]) * inv : (a[j] * cs[j - hf] - a[j - hf] * sn[j - hf]) * inv;
  }
  st_el<F32>(o.out, (long long)tok * o.ld + o.off + (long long)h * dv + j, v * attn_out_factor(o, tok, h));
}

int stack_attn_block_tokens(const StackAttn &c, bool f32) {
  if (stack_attn_mma_ok(c, f32)) return stack_attn_mma_block_tokens(c);
  const int R = c.H / c.G;
  int bq = std::max(1, 32 / R);
  while (bq > 1 && ((size_t)kAtTile * (c.d + c.dv + 2 + kAtWarps) + (size_t)bq * R * (c.d + c.dv + 2)) * 4 > 200 * 1024) bq >>= 1;
  return bq;
}
static size_t attn_smem(const StackAttn &c, int bq) {
  const int R = c.H / c.G;
  return ((size_t)kAtTile * (c.d + c.dv + 2 + kAtWarps) + (size_t)bq * R * (c.d + c.dv + 2)) * sizeof(float);
}

template <bool F32, bool SIG>
__global__ void __launch_bounds__(kAtWarps * 32) stack_attn_kernel(const float *qf, const void *kpool, const void *vpool, const float *temp,
                                                                   const float *pb, const float *sink, StackAttn c, StackSpans sp, const int *qb_tok0,
                                                                   const int *qb_len, const int *page_table, int max_pages,
                                                                   int page_size, AttnOut o, int keys_per_split, float *part) {
  extern __shared__ float shm[];
  const int d = c.d, dv = c.dv, DP = d + 1, VP = dv + 1, R = c.H / c.G, g = blockIdx.y;
  const int tok0 = qb_tok0[blockIdx.x], nq = qb_len[blockIdx.x];
  const int pairs = nq * R;
  float *kt = shm;                               // [32][DP]
  float *vt = kt + (size_t)kAtTile * DP;         // [32][VP]
  float *qs = vt + (size_t)kAtTile * VP;         // [pairs][d]
  float *acc = qs + (size_t)pairs * d;           // [pairs][dv]
  float *mx = acc + (size_t)pairs * dv;          // [pairs]
  float *dn = mx + pairs;                        // [pairs]
  float *prs = dn + pairs;                       // [warps][32]
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  const int slot = sp.slot[tok0];
  const int last_pos = sp.pos[tok0 + nq - 1];
  for (int i = threadIdx.x; i < pairs * d; i += blockDim.x) {
    const int p = i / d, e = i - p * d;
    qs[i] = qf[((long long)(tok0 + p / R) * c.H + g * R + p % R) * d + e];
  }
  for (int i = threadIdx.x; i < pairs * dv; i += blockDim.x) acc[i] = 0.f;
  const bool with_sink = !SIG && sink && blockIdx.z == 0;
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) { mx[i] = with_sink ? sink[g * R + i % R] : -INFINITY; dn[i] = with_sink ? 1.f : 0.f; }
  const int *pt = page_table + (long long)slot * max_pages;
  const int k_lo = stack_attn_row_lo(c, sp.pos[tok0]);
  const int k_begin = part ? k_lo + (int)blockIdx.z * keys_per_split : k_lo;
  const int k_end = part ? min(last_pos + 1, k_begin + keys_per_split) : last_pos + 1;
  const long long krow = (long long)c.G * d, vrow = (long long)c.G * dv;
  const float inv_cap = c.softcap > 0.f ? 1.f / c.softcap : 0.f;
  for (int k0 = k_begin; k0 < k_end; k0 += kAtTile) {
    const int nk = min(kAtTile, k_end - k0);
    __syncthreads();
    for (int i = threadIdx.x; i < nk * d; i += blockDim.x) {
      const int kk = i / d, cc = i - kk * d, kp = k0 + kk;
      const long long prow = (long long)pt[kp / page_size] * page_size + kp % page_size;
      kt[(size_t)kk * DP + cc] = ld_el<F32>(kpool, prow * krow + (long long)g * d + cc);
    }
    for (int i = threadIdx.x; i < nk * dv; i += blockDim.x) {
      const int kk = i / dv, cc = i - kk * dv, kp = k0 + kk;
      const long long prow = (long long)pt[kp / page_size] * page_size + kp % page_size;
      vt[(size_t)kk * VP + cc] = ld_el<F32>(vpool, prow * vrow + (long long)g * dv + cc);
    }
    __syncthreads();
    for (int p = w; p < pairs; p += kAtWarps) {
      const int qpos = sp.pos[tok0 + p / R], h = g * R + p % R;
      const int qlo = stack_attn_row_lo(c, qpos);
      const float *q = qs + (size_t)p * d;
      float sc = -INFINITY;
      if (l < nk && k0 + l <= qpos && k0 + l >= qlo) {
        const float *kr = kt + (size_t)l * DP;
        float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;  // four chains, added at the end: the sum's order is fixed by d alone
        int i = 0;
        for (; i + 3 < d; i += 4) {
          s0 = fmaf(q[i], kr[i], s0); s1 = fmaf(q[i + 1], kr[i + 1], s1);
          s2 = fmaf(q[i + 2], kr[i + 2], s2); s3 = fmaf(q[i + 3], kr[i + 3], s3);
        }
        for (; i < d; i++) s0 = fmaf(q[i], kr[i], s0);
        sc = ((s0 + s1) + (s2 + s3)) * c.scale;
        if (c.softcap > 0.f) sc = c.softcap * tanhf(sc * inv_cap);
      }
      float pr, corr = 1.f, psum = 0.f, m_new = 0.f;
      if (SIG) {
        pr = sc == -INFINITY ? 0.f : 1.f / (1.f + expf(-(sc * temp[h] + pb[h])));
      } else {
        const float m_old = mx[p];
        m_new = fmaxf(m_old, warp_max(sc));
        pr = sc == -INFINITY ? 0.f : expf(sc - m_new);
        corr = m_old == -INFINITY ? 0.f : expf(m_old - m_new);  // (m_new is -inf too while a pair has seen nothing: pr = 0 then)
        psum = warp_sum(pr);
      }
      float *a = acc + (size_t)p * dv;
      float *pw = prs + w * kAtTile;  // the tile's weights of this pair: lanes own coordinates below, so every lane reads all
      pw[l] = pr;
      __syncwarp();
      for (int j = l; j < dv; j += 32) {
        float v0 = a[j] * corr, v1 = 0.f, v2 = 0.f, v3 = 0.f;
        int kk = 0;
        for (; kk + 3 < nk; kk += 4) {
          v0 = fmaf(pw[kk], vt[(size_t)kk * VP + j], v0); v1 = fmaf(pw[kk + 1], vt[(size_t)(kk + 1) * VP + j], v1);
          v2 = fmaf(pw[kk + 2], vt[(size_t)(kk + 2) * VP + j], v2); v3 = fmaf(pw[kk + 3], vt[(size_t)(kk + 3) * VP + j], v3);
        }
        for (; kk < nk; kk++) v0 = fmaf(pw[kk], vt[(size_t)kk * VP + j], v0);
        a[j] = (v0 + v1) + (v2 + v3);
      }
      __syncwarp();
      if (!SIG && l == 0) { mx[p] = m_new; dn[p] = dn[p] * corr + psum; }
      __syncwarp();
    }
  }
  __syncthreads();
  if (!part) {
    for (int i = threadIdx.x; i < pairs * dv; i += blockDim.x) {
      const int p = i / dv, j = i - p * dv;
      attn_store<F32>(o, acc + (size_t)p * dv, SIG ? 1.f : 1.f / dn[p], tok0 + p / R, g * R + p % R, dv, j);
    }
    return;
  }
  // slice record per (token, head): dv unnormalised sums, then the slice's maximum and denominator
  for (int i = threadIdx.x; i < pairs * (dv + 2); i += blockDim.x) {
    const int p = i / (dv + 2), j = i - p * (dv + 2);
    float *rec = part + (((long long)blockIdx.z * sp.T + tok0 + p / R) * c.H + g * R + p % R) * (dv + 2);
    rec[j] = j < dv ? acc[(size_t)p * dv + j] : j == dv ? mx[p] : dn[p];
  }
}

// Merge of the slices of one (token, head): softmax: out = sum_s acc_s e^(m_s - M) / sum_s l_s e^(m_s - M); sigmoid: plain sum.
// Slices that lie wholly behind the token (nothing visible) wrote m = -inf, l = 0 and zeros.
template <bool F32, bool SIG>
__global__ void stack_attn_merge_kernel(const float *part, int n_split, int T, int H, int dv, AttnOut o) {
  extern __shared__ float msh[];  // [dv] merged sums, [n_split] factors
  float *a = msh, *ws = msh + dv;
  __shared__ float inv_den;
  const int p = blockIdx.x, tok = p / H, h = p - tok * H;
  const long long stride = (long long)T * H * (dv + 2);
  const float *rec = part + (long long)p * (dv + 2);
  if (!SIG) {
    float M = -INFINITY;
    for (int s = 0; s < n_split; s++) M = fmaxf(M, rec[s * stride + dv]);
    for (int s = threadIdx.x; s < n_split; s += blockDim.x) {
      const float m = rec[s * stride + dv];
      ws[s] = m == -INFINITY ? 0.f : expf(m - M);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      float den = 0.f;
      for (int s = 0; s < n_split; s++) den += rec[s * stride + dv + 1] * ws[s];
      inv_den = 1.f / den;
    }
  }
  __syncthreads();
  for (int j = threadIdx.x; j < dv; j += blockDim.x) {
    float v = 0.f;
    for (int s = 0; s < n_split; s++) v = SIG ? v + rec[s * stride + j] : fmaf(rec[s * stride + j], ws[s], v);
    a[j] = v;
  }
  __syncthreads();
  for (int j = threadIdx.x; j < dv; j += blockDim.x) attn_store<F32>(o, a, SIG ? 1.f : inv_den, tok, h, dv, j);
}

// ------------------------------------------------------------------------------------------------ attention on mma.sync
// The bf16 compute type with dim a multiple of 8, vdim a multiple of 16, both at most 128, and at most 64 query heads per
// key/value head.  A CTA of four warps owns up to 64 rows -- the (token, query head of the group) pairs of its query block,
// 16 per warp -- and walks the history in tiles of 64 keys: K and V rows of the pages are copied with cp.async into two
// shared-memory stages (the next tile is in flight while this one is used), S = Q K^T and O += P V run on m16n8k16 with fp32
// accumulators, the weights in between are fp32 (online softmax per row, or the sigmoid form) and are rounded to bf16 only as
// the operand of P V.  Slices and the epilogue are those of the kernel above.
constexpr int kMmKeys = 64, kMmWarps = 4, kMmRows = 16 * kMmWarps;
constexpr float kLog2e = 1.4426950408889634f, kLn2 = 0.6931471805599453f;

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src, int src_bytes) {  // src_bytes 0: zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {  // round to nearest even, one instruction
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
__device__ __forceinline__ float ex2_(float x) {  // 2^x, flushing results below the normal range to zero; 2^(-inf) = 0
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}

// Scores of one 64-key tile -> sigmoid weights, or scaled scores and the rows' running maxima (softmax).  MASKED: the tile
// reaches past a row's position or the slice's end, or starts before a row's chunk, so every element is checked; interior tiles
// skip the checks.
// cap2 > 0 (softmax only): the scaled score s passes cap tanh(s / cap) first; scale2 is then the plain scale over the cap, and
// tanh x = 1 - 2 / (1 + e^(2x)) is formed with one ex2 and one reciprocal (absolute error of the order of 1e-7, times the cap).
template <bool SIG, bool MASKED>
__device__ __forceinline__ void attn_tile_weights(float (&sacc)[kMmKeys / 8][4], float (&mnew)[2], int k0, int qd, const int (&r_pos)[2],
                                                  const int (&r_lo)[2], int k_end, const float (&tmp_h)[2], const float (&pb_h)[2],
                                                  float scale2, float cap2) {
#pragma unroll
  for (int j = 0; j < kMmKeys / 8; j++)
#pragma unroll
    for (int q4 = 0; q4 < 4; q4++) {
      const int e = q4 >> 1;
      bool vis = true;
      if (MASKED) { const int kp = k0 + j * 8 + qd * 2 + (q4 & 1); vis = kp <= r_pos[e] && kp < k_end && kp >= r_lo[e]; }
      float sv = sacc[j][q4];
      if (SIG) {
        float rc;
        asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(rc) : "f"(1.f + ex2_(-fmaf(sv, tmp_h[e], pb_h[e]))));
        sv = vis ? rc : 0.f;
      } else {
        sv *= scale2;
        if (cap2 > 0.f) {
          float rc;
          asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(rc) : "f"(1.f + ex2_(sv * (2.f * kLog2e))));
          sv = cap2 * fmaf(-2.f, rc, 1.f);
        }
        sv = vis ? sv : -INFINITY;
        mnew[e] = fmaxf(mnew[e], sv);
      }
      sacc[j][q4] = sv;
    }
}

bool stack_attn_mma_ok(const StackAttn &c, bool f32) {
  return !f32 && c.d % 8 == 0 && c.dv % 16 == 0 && c.d <= 128 && c.dv <= 128 && c.H / c.G <= kMmRows;
}
int stack_attn_mma_block_tokens(const StackAttn &c) { return std::max(1, kMmRows / (c.H / c.G)); }

template <int DMAX, bool SIG>
__global__ void __launch_bounds__(kMmWarps * 32, 3) stack_attn_mma_kernel(const float *__restrict__ qf, const uint16_t *__restrict__ kpool,
                                                                       const uint16_t *__restrict__ vpool, const float *temp,
                                                                       const float *pb, const float *sink, StackAttn c, StackSpans sp, const int *qb_tok0,
                                                                       const int *qb_len, const int *page_table, int max_pages,
                                                                       int page_size, AttnOut o, int keys_per_split, float *part) {
  constexpr int PITCH = DMAX + 8;  // elements per shared row: 16-byte rows land in distinct bank groups
  extern __shared__ __align__(16) uint16_t smem[];
  uint16_t *Ks = smem;                                  // [2][64][PITCH]
  uint16_t *Vs = smem + 2 * kMmKeys * PITCH;            // [2][64][PITCH]
  const int d = c.d, dv = c.dv, R = c.H / c.G, kvh = blockIdx.y;
  // the blocks of a span come in ascending position, and the later ones walk a longer history: taking the grid backwards starts
  // the long ones first, so the last CTAs to start are short
  const int qb = gridDim.x - 1 - blockIdx.x;
  const int tok0 = qb_tok0[qb], nq = qb_len[qb], rows = nq * R;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gid = lane >> 2, qd = lane & 3;
  const int slot = sp.slot[tok0], pos_first = sp.pos[tok0], last_pos = pos_first + nq - 1;
  const int *pt = page_table + (long long)slot * max_pages;
  // chunked or windowed mask: the first token's bound is where the block's history starts (later rows may start later still)
  const int k_lo = stack_attn_row_lo(c, pos_first);
  const int k_begin = part ? k_lo + (int)blockIdx.z * keys_per_split : k_lo;
  const int k_end = part ? min(last_pos + 1, k_begin + keys_per_split) : last_pos + 1;
  const int nk16 = (d + 15) >> 4, nv8 = dv >> 3, dc = d >> 3, vc = dv >> 3;  // k-steps of Q K^T, n-tiles of P V, 16-byte chunks per row
  // columns d .. 16 nk16 of the K stages are read by the last k-step: zero them once (cp.async never touches them)
  if (d & 15)
    for (int i = threadIdx.x; i < 2 * kMmKeys * 8; i += blockDim.x) Ks[(i >> 3) * PITCH + d + (i & 7)] = 0;
  // ---- this thread's rows: r0 = 16 warp + gid and r0 + 8
  int r_tok[2], r_head[2], r_pos[2], r_lo[2];
  bool r_ok[2];
  uint32_t qa[DMAX / 16][4];
#pragma unroll
  for (int e = 0; e < 2; e++) {
    const int r = warp * 16 + gid + e * 8;
    r_ok[e] = r < rows;
    r_tok[e] = tok0 + (r_ok[e] ? r / R : 0);
    r_head[e] = kvh * R + (r_ok[e] ? r % R : 0);
    r_pos[e] = r_ok[e] ? pos_first + r / R : -1;
    r_lo[e] = r_ok[e] ? stack_attn_row_lo(c, r_pos[e]) : 0;
  }
#pragma unroll
  for (int ks = 0; ks < DMAX / 16; ks++) {
#pragma unroll
    for (int e = 0; e < 2; e++) {
      const float *qr = qf + ((long long)r_tok[e] * c.H + r_head[e]) * d;
#pragma unroll
      for (int hf = 0; hf < 2; hf++) {
        const int col = ks * 16 + hf * 8 + qd * 2;
        float x0 = 0.f, x1 = 0.f;
        if (r_ok[e] && ks < nk16) {
          if (col < d) x0 = qr[col];
          if (col + 1 < d) x1 = qr[col + 1];
        }
        qa[ks][hf * 2 + e] = pack_bf16(x0, x1);
      }
    }
  }
  float oacc[DMAX / 8][4];
#pragma unroll
  for (int j = 0; j < DMAX / 8; j++) { oacc[j][0] = oacc[j][1] = oacc[j][2] = oacc[j][3] = 0.f; }
  float mrow[2] = {-INFINITY, -INFINITY}, lrow[2] = {0.f, 0.f};
  if (!SIG && sink && blockIdx.z == 0) {  // the sink term of the denominator enters as the initial state of the first slice (one lane of the four holds its 1)
#pragma unroll
    for (int e = 0; e < 2; e++) { mrow[e] = sink[r_head[e]] * kLog2e; lrow[e] = qd == 0 ? 1.f : 0.f; }
  }
  float tmp_h[2] = {1.f, 1.f}, pb_h[2] = {0.f, 0.f};
  if (SIG) {
#pragma unroll
    for (int e = 0; e < 2; e++) { tmp_h[e] = temp[r_head[e]] * c.scale * kLog2e; pb_h[e] = pb[r_head[e]] * kLog2e; }
  }
  // with a soft cap the scores are first brought to units of the cap (scale / cap), and the capped score to units of log 2
  const float cap2 = !SIG && c.softcap > 0.f ? c.softcap * kLog2e : 0.f;
  const float scale2 = cap2 > 0.f ? c.scale / c.softcap : c.scale * kLog2e;
  const bool warp_live = warp * 16 < rows;
  const int warp_last_pos = pos_first + min(rows - 1, warp * 16 + 15) / R;
  const int warp_first_pos = pos_first + (warp * 16) / R;
  const int warp_lo = stack_attn_row_lo(c, warp_first_pos);        // first key any row of the warp sees
  const int warp_lo_max = stack_attn_row_lo(c, warp_last_pos);     // first key every row of the warp sees
  const long long krow = (long long)c.G * d, vrow = (long long)c.G * dv;
  const uint32_t ks_base = (uint32_t)__cvta_generic_to_shared(Ks), vs_base = (uint32_t)__cvta_generic_to_shared(Vs);
  // two threads per key row: one page-table read per thread and tile, then the row's 16-byte chunks alternate between the two
  const int ld_row = threadIdx.x >> 1, ld_part = threadIdx.x & 1;
  const int pshift = 31 - __clz(page_size);  // page_size is a power of two
  // the page of this thread's row is read one tile ahead of the copy that needs it
  auto page_of = [&](int k0) { const int kp = k0 + ld_row; return kp < k_end ? pt[kp >> pshift] : 0; };
  int page_next = page_of(k_begin);
  auto load_tile = [&](int k0, int stage) {
    const int kp = k0 + ld_row;
    const bool ok = kp < k_end;
    const long long prow = ok ? (long long)page_next * page_size + (kp & (page_size - 1)) : 0;
    page_next = page_of(k0 + kMmKeys);
    const uint16_t *ksrc = kpool + prow * krow + (long long)kvh * d, *vsrc = vpool + prow * vrow + (long long)kvh * dv;
    const uint32_t kdst = ks_base + (uint32_t)(((stage * kMmKeys + ld_row) * PITCH) * 2), vdst = vs_base + (uint32_t)(((stage * kMmKeys + ld_row) * PITCH) * 2);
#pragma unroll 4
    for (int ch = ld_part; ch < dc; ch += 2) cp_async16(kdst + ch * 16, ksrc + ch * 8, ok ? 16 : 0);
#pragma unroll 4
    for (int ch = ld_part; ch < vc; ch += 2) cp_async16(vdst + ch * 16, vsrc + ch * 8, ok ? 16 : 0);
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  const int n_tiles = k_end > k_begin ? (k_end - k_begin + kMmKeys - 1) / kMmKeys : 0;
  if (n_tiles > 0) load_tile(k_begin, 0);
  for (int it = 0; it < n_tiles; it++) {
    const int k0 = k_begin + it * kMmKeys, stage = it & 1;
    if (it + 1 < n_tiles) {
      load_tile(k0 + kMmKeys, stage ^ 1);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    if (warp_live && k0 <= warp_last_pos && k0 + kMmKeys > warp_lo) {
      // S = Q K^T: k-steps outside, key tiles inside, so that consecutive products go to different accumulators; one ldmatrix
      // brings the fragments of two key tiles (lane l: matrix l / 8 = (tile, column half), row l % 8)
      const uint32_t kt = ks_base + (uint32_t)(stage * kMmKeys * PITCH * 2);
      float sacc[kMmKeys / 8][4];
#pragma unroll
      for (int j = 0; j < kMmKeys / 8; j++) { sacc[j][0] = sacc[j][1] = sacc[j][2] = sacc[j][3] = 0.f; }
#pragma unroll
      for (int ks = 0; ks < DMAX / 16; ks++) {
        if (ks < nk16) {
#pragma unroll
          for (int j = 0; j < kMmKeys / 8; j += 2) {
            uint32_t b0, b1, b2, b3;
            ldsm_x4(kt + (uint32_t)((((j + (lane >> 4)) * 8 + (lane & 7)) * PITCH + ks * 16 + ((lane >> 3) & 1) * 8) * 2), b0, b1, b2, b3);
            mma_bf16_16816(sacc[j], qa[ks], b0, b1);
            mma_bf16_16816(sacc[j + 1], qa[ks], b2, b3);
          }
        }
      }
      // ---- weights, fp32.  Scores are carried in units of log 2 (the factor 1 / ln 2 is folded into the scale), so every
      // exponential is one ex2.  Only a tile that reaches past a row's position or the slice's end needs the mask.
      const bool masked = k0 + kMmKeys - 1 > warp_first_pos || k0 + kMmKeys > k_end || k0 < warp_lo_max;
      float mnew[2] = {mrow[0], mrow[1]};
      if (masked) attn_tile_weights<SIG, true>(sacc, mnew, k0, qd, r_pos, r_lo, k_end, tmp_h, pb_h, scale2, cap2);
      else attn_tile_weights<SIG, false>(sacc, mnew, k0, qd, r_pos, r_lo, k_end, tmp_h, pb_h, scale2, cap2);
      if (!SIG) {
        float corr[2];
#pragma unroll
        for (int e = 0; e < 2; e++) {
          mnew[e] = fmaxf(mnew[e], __shfl_xor_sync(0xffffffffu, mnew[e], 1));
          mnew[e] = fmaxf(mnew[e], __shfl_xor_sync(0xffffffffu, mnew[e], 2));
          corr[e] = mrow[e] == -INFINITY ? 0.f : ex2_(mrow[e] - mnew[e]);
          mrow[e] = mnew[e];
          lrow[e] *= corr[e];
        }
        const float msub[2] = {mnew[0] == -INFINITY ? 0.f : mnew[0], mnew[1] == -INFINITY ? 0.f : mnew[1]};  // a row with nothing visible yet
#pragma unroll
        for (int j = 0; j < kMmKeys / 8; j++)
#pragma unroll
          for (int q4 = 0; q4 < 4; q4++) {
            const int e = q4 >> 1;
            const float pv = ex2_(sacc[j][q4] - msub[e]);  // 2^(-inf) = 0 for the masked
            sacc[j][q4] = pv;
            lrow[e] += pv;
          }
#pragma unroll
        for (int j = 0; j < DMAX / 8; j++) { oacc[j][0] *= corr[0]; oacc[j][1] *= corr[0]; oacc[j][2] *= corr[1]; oacc[j][3] *= corr[1]; }
      }
      // ---- O += P V
      const uint32_t vt = vs_base + (uint32_t)(stage * kMmKeys * PITCH * 2);
#pragma unroll
      for (int kk = 0; kk < kMmKeys / 16; kk++) {
        uint32_t pa[4];
        pa[0] = pack_bf16(sacc[2 * kk][0], sacc[2 * kk][1]);
        pa[1] = pack_bf16(sacc[2 * kk][2], sacc[2 * kk][3]);
        pa[2] = pack_bf16(sacc[2 * kk + 1][0], sacc[2 * kk + 1][1]);
        pa[3] = pack_bf16(sacc[2 * kk + 1][2], sacc[2 * kk + 1][3]);
#pragma unroll
        for (int j = 0; j < DMAX / 8; j += 2) {
          if (j < nv8) {
            // lanes 0-15: keys 16 kk + lane of columns 8 j; lanes 16-31: the same keys of columns 8 (j + 1)
            uint32_t b0, b1, b2, b3;
            ldsm_x4_trans(vt + (uint32_t)(((kk * 16 + (lane & 15)) * PITCH + (j + (lane >> 4)) * 8) * 2), b0, b1, b2, b3);
            mma_bf16_16816(oacc[j], pa, b0, b1);
            mma_bf16_16816(oacc[j + 1], pa, b2, b3);
          }
        }
      }
    }
    __syncthreads();
  }
  if (!SIG) {
#pragma unroll
    for (int e = 0; e < 2; e++) {
      lrow[e] += __shfl_xor_sync(0xffffffffu, lrow[e], 1);
      lrow[e] += __shfl_xor_sync(0xffffffffu, lrow[e], 2);
    }
  }
  // ---- results: thread holds, for row e, columns 8 j + 2 qd + {0, 1} of every n-tile j
  if (!part && o.vrot) {
    // rotation back by the query's position pairs column m with m + dv/2: the warp's 16 x dv tile goes through shared memory
    // (every key tile has been consumed; a warp reads only the rows it wrote)
    float *ot = reinterpret_cast<float *>(smem) + (size_t)warp * 16 * (dv + 1);
#pragma unroll
    for (int e = 0; e < 2; e++) {
#pragma unroll
      for (int j = 0; j < DMAX / 8; j++)
        if (j < nv8) { ot[(gid + e * 8) * (dv + 1) + j * 8 + qd * 2] = oacc[j][e * 2]; ot[(gid + e * 8) * (dv + 1) + j * 8 + qd * 2 + 1] = oacc[j][e * 2 + 1]; }
      if (qd == 0) ot[(gid + e * 8) * (dv + 1) + dv] = attn_out_factor(o, r_tok[e], r_head[e]) * (SIG ? 1.f : 1.f / lrow[e]);
    }
    __syncwarp();
    const int hf = dv >> 1;
    for (int i = lane; i < 16 * hf; i += 32) {
      const int rr = i / hf, m = i - rr * hf, r = warp * 16 + rr;
      if (r >= rows) continue;
      const int tok = tok0 + r / R, head = kvh * R + r % R;
      const float *cs = o.vrot + (long long)tok * dv, *sn = cs + hf;
      const float u = ot[rr * (dv + 1) + m], w = ot[rr * (dv + 1) + m + hf], inv = ot[rr * (dv + 1) + dv];
      uint16_t *orow = reinterpret_cast<uint16_t *>(o.out) + (long long)tok * o.ld + o.off + (long long)head * dv;
      orow[m] = float_to_bf16_bits((u * cs[m] + w * sn[m]) * inv);
      orow[m + hf] = float_to_bf16_bits((w * cs[m] - u * sn[m]) * inv);
    }
    return;
  }
#pragma unroll
  for (int e = 0; e < 2; e++) {
    if (!r_ok[e]) continue;
    if (part) {
      float *rec = part + (((long long)blockIdx.z * sp.T + r_tok[e]) * c.H + r_head[e]) * (dv + 2);
#pragma unroll
      for (int j = 0; j < DMAX / 8; j++)
        if (j < nv8) { rec[j * 8 + qd * 2] = oacc[j][e * 2]; rec[j * 8 + qd * 2 + 1] = oacc[j][e * 2 + 1]; }
      if (qd == 0) { rec[dv] = SIG ? 0.f : mrow[e] * kLn2; rec[dv + 1] = lrow[e]; }  // the maximum back in natural units
      continue;
    }
    const float inv = attn_out_factor(o, r_tok[e], r_head[e]) * (SIG ? 1.f : 1.f / lrow[e]);
    uint16_t *orow = reinterpret_cast<uint16_t *>(o.out) + (long long)r_tok[e] * o.ld + o.off + (long long)r_head[e] * dv;
#pragma unroll
    for (int j = 0; j < DMAX / 8; j++)
      if (j < nv8) *reinterpret_cast<uint32_t *>(orow + j * 8 + qd * 2) = pack_bf16(oacc[j][e * 2] * inv, oacc[j][e * 2 + 1] * inv);
  }
}

cudaError_t launch_stack_attn(const float *qf, const void *kpool, const void *vpool, bool f32, const float *temp, const float *pb,
                              const float *sink, const StackAttn &c, const StackSpans &sp, const int *qb_tok0, const int *qb_len, int n_qb,
                              int bq, const int *page_table, int max_pages, int page_size, void *out, long long ld_out, int out_off,
                              float out_scale, const float *vrot, const float *gate, long long ld_gate, int n_split,
                              int keys_per_split, float *part, cudaStream_t st) {
  if (n_qb <= 0) return cudaSuccess;
  if (!(c.flags & (DIS_ATTN_SINK | DIS_ATTN_SINK_UNIT))) sink = nullptr;  // the unit sink is a vector of zero logits
  if (!(c.flags & DIS_ATTN_GATE)) gate = nullptr;
  if (n_split <= 1 || !part) { n_split = 1; part = nullptr; }
  if (n_split > kAtMaxSplit) return cudaErrorInvalidValue;
  const bool sig = (c.flags & DIS_ATTN_SIGMOID) != 0;
  const size_t sh = attn_smem(c, bq);
  if (sh > 220 * 1024) return cudaErrorInvalidValue;
  static DeviceOnce once;
  DIS_CUDA_TRY(once.run([&] {
    cudaError_t e = cudaFuncSetAttribute(stack_attn_kernel<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(stack_attn_kernel<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(stack_attn_kernel<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
    return e != cudaSuccess ? e : cudaFuncSetAttribute(stack_attn_kernel<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
  }));
  const AttnOut o{out, ld_out, out_off, out_scale, (c.flags & DIS_ATTN_ROT_V) ? vrot : nullptr, gate, ld_gate};
  const dim3 grid(n_qb, c.G, n_split);
  static int use_mma = -1;
  if (use_mma < 0) { const char *e = getenv("DIS_STACK_ATTN_MMA"); use_mma = (e && atoi(e) == 0) ? 0 : 1; }
  // the output's 4-byte stores want even columns; bq is the block size the pass was planned with
  if (use_mma && stack_attn_mma_ok(c, f32) && bq <= stack_attn_mma_block_tokens(c) && ld_out % 2 == 0 && out_off % 2 == 0) {
    static DeviceOnce once_mma;
    DIS_CUDA_TRY(once_mma.run([&] {
      cudaError_t e = cudaFuncSetAttribute(stack_attn_mma_kernel<64, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
      if (e == cudaSuccess) e = cudaFuncSetAttribute(stack_attn_mma_kernel<64, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
      if (e == cudaSuccess) e = cudaFuncSetAttribute(stack_attn_mma_kernel<128, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
      return e != cudaSuccess ? e : cudaFuncSetAttribute(stack_attn_mma_kernel<128, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
    }));
    const bool small = c.d <= 64 && c.dv <= 64;
    const size_t shm = (size_t)4 * kMmKeys * ((small ? 64 : 128) + 8) * sizeof(uint16_t);
    const uint16_t *kp = reinterpret_cast<const uint16_t *>(kpool), *vp = reinterpret_cast<const uint16_t *>(vpool);
#define DIS_ATTN_MMA(D, S) \
  stack_attn_mma_kernel<D, S><<<grid, kMmWarps * 32, shm, st>>>(qf, kp, vp, temp, pb, sink, c, sp, qb_tok0, qb_len, page_table, max_pages, page_size, o, keys_per_split, part)
    if (small && sig) DIS_ATTN_MMA(64, true);
    else if (small) DIS_ATTN_MMA(64, false);
    else if (sig) DIS_ATTN_MMA(128, true);
    else DIS_ATTN_MMA(128, false);
#undef DIS_ATTN_MMA
    if (part) {
      const size_t msh = (size_t)(c.dv + n_split) * sizeof(float);
      if (sig) stack_attn_merge_kernel<false, true><<<sp.T * c.H, 64, msh, st>>>(part, n_split, sp.T, c.H, c.dv, o);
      else stack_attn_merge_kernel<false, false><<<sp.T * c.H, 64, msh, st>>>(part, n_split, sp.T, c.H, c.dv, o);
    }
    return cudaGetLastError();
  }
  const int th = kAtWarps * 32;
#define DIS_ATTN_LAUNCH(F, S) \
  stack_attn_kernel<F, S><<<grid, th, sh, st>>>(qf, kpool, vpool, temp, pb, sink, c, sp, qb_tok0, qb_len, page_table, max_pages, page_size, o, keys_per_split, part)
  if (f32 && sig) DIS_ATTN_LAUNCH(true, true);
  else if (f32) DIS_ATTN_LAUNCH(true, false);
  else if (sig) DIS_ATTN_LAUNCH(false, true);
  else DIS_ATTN_LAUNCH(false, false);
#undef DIS_ATTN_LAUNCH
  if (part) {
    const size_t msh = (size_t)(c.dv + n_split) * sizeof(float);
    const int rows = sp.T * c.H;
    if (f32 && sig) stack_attn_merge_kernel<true, true><<<rows, 64, msh, st>>>(part, n_split, sp.T, c.H, c.dv, o);
    else if (f32) stack_attn_merge_kernel<true, false><<<rows, 64, msh, st>>>(part, n_split, sp.T, c.H, c.dv, o);
    else if (sig) stack_attn_merge_kernel<false, true><<<rows, 64, msh, st>>>(part, n_split, sp.T, c.H, c.dv, o);
    else stack_attn_merge_kernel<false, false><<<rows, 64, msh, st>>>(part, n_split, sp.T, c.H, c.dv, o);
  }
  return cudaGetLastError();
}

}  // namespace dis
