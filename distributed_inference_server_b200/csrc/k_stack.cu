// k_stack.cu -- kernels of the layer-list decoders (stack.h): a general fp32-accumulating matrix product over float or bf16
// operands (plain, batched per head, or grouped per expert), the scalar-gain residual norms, the input convolution with its
// per-slot tail, the two recurrences, latent attention over paged latents, the clamped gated unit and the expert router.
// Everything the family defines as 32-bit -- norms, decays, recurrent state, scores and softmax, routers, the residual --
// is fp32 here whatever the element type of the matrices.
#include "stack_dev.cuh"

namespace dis {

// ------------------------------------------------------------------------------------------------ matrix product
// out[m][n] = bias[n] + sum_k A[m][k] W[n][k].  64 x 64 tile per CTA, 16-deep slices through shared memory, 4 x 4 outputs per
// thread, fp32 FMA: every output element is one k-ordered sum whatever tile it falls in, so a row's result does not depend on
// the rows beside it.
constexpr int GB = kStackGemmTile, GK = 16;

template <bool AF32, bool WF32>
__global__ void __launch_bounds__(256) stack_gemm_kernel(StackGemm g) {
  __shared__ float As[GK][GB + 4], Ws[GK][GB + 4];
  int row0, rows, grp = 0;
  if (g.tiles) {
    if ((int)blockIdx.x >= g.tiles[0]) return;
    grp = g.tiles[1 + 3 * blockIdx.x];
    row0 = g.tiles[2 + 3 * blockIdx.x];
    rows = g.tiles[3 + 3 * blockIdx.x];
  } else {
    row0 = blockIdx.x * GB;
    rows = min(GB, g.M - row0);
  }
  const int z = blockIdx.z;
  const int n0 = blockIdx.y * GB;
  const long long a_off = (long long)z * g.a_bs, w_off = (long long)z * g.w_bs + (long long)grp * (g.tiles ? g.w_bs : 0);
  const float *bias = g.bias ? g.bias + (long long)z * g.bias_bs + (g.tiles ? (long long)grp * g.bias_bs : 0) : nullptr;
  float *out = g.out + (long long)z * g.o_bs;
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  float acc[4][4] = {};
  // loader: thread -> (row = tid / 4, k = (tid % 4) * 4 .. +3)
  const int lr = tid >> 2, lk = (tid & 3) * 4;
  long long a_row = -1;
  if (lr < rows) a_row = g.a_gather ? g.a_gather[row0 + lr] : row0 + lr;
  const long long w_row = n0 + lr < g.N ? n0 + lr : -1;
  for (int k0 = 0; k0 < g.K; k0 += GK) {
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int k = k0 + lk + j;
      As[lk + j][lr] = (a_row >= 0 && k < g.K) ? ld_el<AF32>(g.A, a_off + a_row * g.lda + k) : 0.f;
      Ws[lk + j][lr] = (w_row >= 0 && k < g.K) ? ld_el<WF32>(g.W, w_off + w_row * g.ldw + k) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < GK; k++) {
      const float4 a = *reinterpret_cast<const float4 *>(&As[k][ty * 4]);
      const float4 w = *reinterpret_cast<const float4 *>(&Ws[k][tx * 4]);
      const float av[4] = {a.x, a.y, a.z, a.w}, wv[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
      for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int r = ty * 4 + i;
    if (r >= rows) continue;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int n = n0 + tx * 4 + j;
      if (n < g.N) out[(long long)(row0 + r) * g.ldo + n] = acc[i][j] + (bias ? bias[n] : 0.f);
    }
  }
}

// Few rows (decode passes, experts with a handful of tokens): the product is bound by reading W once.  A CTA takes one row tile
// and 32 output columns; eight rows of A at a time sit in shared memory as fp32 (K in chunks of kFewK), a warp owns four
// columns and its lanes stride over K eight elements at a time (16-byte loads of bf16 W), so each W element is read once per
// eight rows; the lanes' partial sums are added across the warp at the end.
constexpr int kFewK = 1024, kFewRows = 8, kFewCols = 32;
__device__ __forceinline__ float gelu_tanh_(float z) {
  return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}
// the gated unit of a feed-forward on one (gate, up) pair; kind: dis_mlp_act
__device__ __forceinline__ float glu_any(int kind, float g, float u, float limit) {
  if (kind == DIS_ACT_GELU_TANH) return gelu_tanh_(g) * u;
  if (kind == DIS_ACT_SILU) return g * sigmoid_precise(g) * u;
  g = fminf(g, limit);
  u = fminf(fmaxf(u, -limit), limit);
  return g * sigmoid_precise(1.702f * g) * (u + 1.f);
}
template <bool WF32>
__device__ __forceinline__ void ld_w8(const void *W, long long i, float (&w)[8]) {
  if (WF32) {
    const float4 a = *reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(W) + i);
    const float4 b = *reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(W) + i + 4);
    w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w; w[4] = b.x; w[5] = b.y; w[6] = b.z; w[7] = b.w;
  } else {
    const uint4 v = *reinterpret_cast<const uint4 *>(reinterpret_cast<const uint16_t *>(W) + i);
    const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; j++) { w[2 * j] = __uint_as_float(u[j] << 16); w[2 * j + 1] = __uint_as_float(u[j] & 0xffff0000u); }
  }
}
// eight consecutive W elements as they come from memory (bf16: 16 bytes in a; float: 32 bytes in a, b), unpacked at use
template <bool WF32>
struct FewRaw { uint4 a, b; };
template <bool WF32>
__device__ __forceinline__ void ld_raw8(const void *W, long long i, FewRaw<WF32> &r) {
  if (WF32) {
    const uint4 *p = reinterpret_cast<const uint4 *>(reinterpret_cast<const float *>(W) + i);
    r.a = p[0]; r.b = p[1];
  } else r.a = *reinterpret_cast<const uint4 *>(reinterpret_cast<const uint16_t *>(W) + i);
}
template <bool WF32>
__device__ __forceinline__ void unpack8(const FewRaw<WF32> &r, float (&w)[8]) {
  if (WF32) {
    w[0] = __uint_as_float(r.a.x); w[1] = __uint_as_float(r.a.y); w[2] = __uint_as_float(r.a.z); w[3] = __uint_as_float(r.a.w);
    w[4] = __uint_as_float(r.b.x); w[5] = __uint_as_float(r.b.y); w[6] = __uint_as_float(r.b.z); w[7] = __uint_as_float(r.b.w);
  } else {
    const uint32_t u[4] = {r.a.x, r.a.y, r.a.z, r.a.w};
#pragma unroll
    for (int j = 0; j < 4; j++) { w[2 * j] = __uint_as_float(u[j] << 16); w[2 * j + 1] = __uint_as_float(u[j] & 0xffff0000u); }
  }
}
template <bool AF32, bool WF32>
__global__ void __launch_bounds__(256) stack_gemm_few_kernel(StackGemm g) {
  __shared__ __align__(16) float as[kFewRows][kFewK];
  int row0, rows, grp = 0;
  if (g.tiles) {
    if ((int)blockIdx.x >= g.tiles[0]) return;
    grp = g.tiles[1 + 3 * blockIdx.x];
    row0 = g.tiles[2 + 3 * blockIdx.x];
    rows = g.tiles[3 + 3 * blockIdx.x];
  } else {
    row0 = blockIdx.x * kStackGemmTile;
    rows = min(kStackGemmTile, g.M - row0);
  }
  const int z = blockIdx.z;
  const long long a_off = (long long)z * g.a_bs, w_off = (long long)z * g.w_bs + (long long)grp * (g.tiles ? g.w_bs : 0);
  const float *bias = g.bias ? g.bias + (long long)z * g.bias_bs + (g.tiles ? (long long)grp * g.bias_bs : 0) : nullptr;
  float *out = g.out + (long long)z * g.o_bs;
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  const int n0 = blockIdx.y * kFewCols + w * 4;
  for (int r0 = 0; r0 < rows; r0 += kFewRows) {
    const int nr = min(kFewRows, rows - r0);
    float acc[4][kFewRows] = {};
    for (int k0 = 0; k0 < g.K; k0 += kFewK) {
      const int kc = min(kFewK, g.K - k0);
      // the lane's first 16 bytes of each of its four W rows are requested before A is staged: they travel while the block
      // gathers its rows, and inside the loop the next step's loads are issued before this step's products
      FewRaw<WF32> cur[4];
      auto fetch = [&](int kk, FewRaw<WF32>(&dst)[4]) {
#pragma unroll
        for (int c = 0; c < 4; c++) {
          if (n0 + c < g.N) ld_raw8<WF32>(g.W, w_off + (long long)(n0 + c) * g.ldw + k0 + kk, dst[c]);
          else dst[c].a = dst[c].b = make_uint4(0u, 0u, 0u, 0u);
        }
      };
      if (l * 8 < kc) fetch(l * 8, cur);
      __syncthreads();
      for (int rr = 0; rr < nr; rr++) {
        const long long a_row = g.a_gather ? g.a_gather[row0 + r0 + rr] : row0 + r0 + rr;
        if (g.a_glu) {  // A holds gate | up pairs: the row's input is the gated unit, rounded as the compute type would store it
          const float *ar = reinterpret_cast<const float *>(g.A) + a_off + a_row * g.lda;
          for (int kk = threadIdx.x; kk < kc; kk += blockDim.x) {
            const float v = glu_any(g.a_glu - 1, ar[k0 + kk], ar[g.K + k0 + kk], g.a_limit);
            as[rr][kk] = WF32 ? v : bf16_bits_to_float(float_to_bf16_bits(v));
          }
        } else
        for (int kk = threadIdx.x; kk < kc; kk += blockDim.x) as[rr][kk] = ld_el<AF32>(g.A, a_off + a_row * g.lda + k0 + kk);
      }
      __syncthreads();
      for (int kk = l * 8; kk < kc; kk += 256) {
        FewRaw<WF32> nxt[4];
        const bool more = kk + 256 < kc;
        if (more) fetch(kk + 256, nxt);
        float wv[4][8];
#pragma unroll
        for (int c = 0; c < 4; c++) unpack8<WF32>(cur[c], wv[c]);
#pragma unroll
        for (int r = 0; r < kFewRows; r++) {
          if (r < nr) {
            const float4 a0 = *reinterpret_cast<const float4 *>(&as[r][kk]);
            const float4 a1 = *reinterpret_cast<const float4 *>(&as[r][kk + 4]);
            const float av[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
#pragma unroll
            for (int c = 0; c < 4; c++)
#pragma unroll
              for (int j = 0; j < 8; j++) acc[c][r] = fmaf(av[j], wv[c][j], acc[c][r]);
          }
        }
        if (more) {
#pragma unroll
          for (int c = 0; c < 4; c++) cur[c] = nxt[c];
        }
      }
    }
#pragma unroll
    for (int c = 0; c < 4; c++)
#pragma unroll
      for (int r = 0; r < kFewRows; r++) {
        const float v = warp_sum(acc[c][r]);
        if (l == 0 && r < nr && n0 + c < g.N) out[(long long)(row0 + r0 + r) * g.ldo + n0 + c] = v + (bias ? bias[n0 + c] : 0.f);
      }
  }
}

// at most 64 rows in all and W rows that 16-byte loads can walk: the few-rows kernel
bool stack_gemm_few_rows(const StackGemm &g) {
  const long long wal = g.w_f32 ? 4 : 8;
  return g.M <= 64 && g.K % 8 == 0 && g.ldw % wal == 0 && g.w_bs % wal == 0 && reinterpret_cast<uintptr_t>(g.W) % 16 == 0;
}
cudaError_t launch_stack_gemm(const StackGemm &g, cudaStream_t st) {
  if (g.M <= 0 || g.N <= 0 || g.K <= 0) return cudaSuccess;
  const bool few = stack_gemm_few_rows(g);
  if (g.a_glu && (!few || !g.a_f32)) return cudaErrorInvalidValue;  // the gated input is the few-rows kernel's
  if (few) {
    dim3 grid(g.tiles ? g.max_tiles : (g.M + kStackGemmTile - 1) / kStackGemmTile, (g.N + kFewCols - 1) / kFewCols, g.batch);
    if (grid.x == 0) return cudaSuccess;
    if (g.a_f32 && g.w_f32) stack_gemm_few_kernel<true, true><<<grid, 256, 0, st>>>(g);
    else if (g.a_f32) stack_gemm_few_kernel<true, false><<<grid, 256, 0, st>>>(g);
    else if (g.w_f32) stack_gemm_few_kernel<false, true><<<grid, 256, 0, st>>>(g);
    else stack_gemm_few_kernel<false, false><<<grid, 256, 0, st>>>(g);
    return cudaGetLastError();
  }
  dim3 grid(g.tiles ? g.max_tiles : (g.M + GB - 1) / GB, (g.N + GB - 1) / GB, g.batch);
  if (grid.x == 0) return cudaSuccess;
  if (g.a_f32 && g.w_f32) stack_gemm_kernel<true, true><<<grid, 256, 0, st>>>(g);
  else if (g.a_f32) stack_gemm_kernel<true, false><<<grid, 256, 0, st>>>(g);
  else if (g.w_f32) stack_gemm_kernel<false, true><<<grid, 256, 0, st>>>(g);
  else stack_gemm_kernel<false, false><<<grid, 256, 0, st>>>(g);
  return cudaGetLastError();
}

__global__ void stack_sum_bias_kernel(const float *part, int n_part, long long stride, const float *bias, float *out, long long n,
                                      int N) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    float s = bias ? bias[i % N] : 0.f;
    for (int k = 0; k < n_part; k++) s += part[(long long)k * stride + i];
    out[i] = s;
  }
}
cudaError_t launch_stack_sum_bias(const float *part, int n_part, long long stride, const float *bias, float *out, int M, int N,
                                  cudaStream_t st) {
  const long long n = (long long)M * N;
  if (n <= 0) return cudaSuccess;
  stack_sum_bias_kernel<<<(int)std::min<long long>((n + 255) / 256, 148 * 8), 256, 0, st>>>(part, n_part, stride, bias, out, n, N);
  return cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------ embedding, norms
// x[t][s] = embed[token] * scale (+ the position vector of the token's position), the same row for every one of the S residual
// streams.  Position vector: entry 2i = sin(p f_i), entry 2i + 1 = cos(p f_i) with f_i = base^(-2i/W) from a table formed in double;
// the angle is formed and brought into [-pi, pi] in double, sine and cosine of the reduced angle are float.
template <bool F32>
__global__ void stack_embed_kernel(const void *embed, const uint32_t *tokens, const int *pos, const double *pos_freq, float *x, float *x0,
                                   float scale, int W, int S) {
  const long long t = blockIdx.x;
  const long long row = tokens[t];
  const int p = pos_freq ? pos[t] : 0;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    float v = ld_el<F32>(embed, row * W + i) * scale;
    if (pos_freq) {
      const double a = (double)p * pos_freq[i >> 1];
      const float r = (float)(a - 6.283185307179586476925 * rint(a * 0.15915494309189533577));
      v += (i & 1) ? cosf(r) : sinf(r);
    }
    for (int k = 0; k < S; k++) x[(t * S + k) * W + i] = v;
    if (x0) x0[t * W + i] = v;
  }
}
cudaError_t launch_stack_embed(const void *embed, bool f32, const uint32_t *tokens, const int *pos, const double *pos_freq, float *x,
                               float *x0, float scale, int T, int W, int streams, cudaStream_t st) {
  if (streams < 1) streams = 1;
  if (f32) stack_embed_kernel<true><<<T, 128, 0, st>>>(embed, tokens, pos, pos_freq, x, x0, scale, W, streams);
  else stack_embed_kernel<false><<<T, 128, 0, st>>>(embed, tokens, pos, pos_freq, x, x0, scale, W, streams);
  return cudaGetLastError();
}

__global__ void __launch_bounds__(256) stack_resid_norm_kernel(float *x, const float *y, const float *post, const float *pre,
                                                               float *hn, int W, float eps) {
  __shared__ float sh[32];
  const long long t = blockIdx.x;
  float *xr = x + t * W;
  if (y) {
    const float *yr = y + t * W;
    float s = 0.f;
    for (int i = threadIdx.x; i < W; i += blockDim.x) s += yr[i] * yr[i];
    s = block_sum(s, sh);
    const float r = rsqrtf(s / (float)W + eps) * post[0];
    for (int i = threadIdx.x; i < W; i += blockDim.x) xr[i] += yr[i] * r;
  }
  if (!hn) return;
  float s = 0.f;
  for (int i = threadIdx.x; i < W; i += blockDim.x) s += xr[i] * xr[i];  // each thread re-reads what it wrote itself
  s = block_sum(s, sh);
  const float r = rsqrtf(s / (float)W + eps) * pre[0];
  for (int i = threadIdx.x; i < W; i += blockDim.x) hn[t * W + i] = xr[i] * r;
}
cudaError_t launch_stack_resid_norm(float *x, const float *y, const float *post, const float *pre, float *hn, int T, int W,
                                    float eps, cudaStream_t st) {
  stack_resid_norm_kernel<<<T, 256, 0, st>>>(x, y, post, pre, hn, W, eps);
  return cudaGetLastError();
}

template <bool F32>
__global__ void stack_final_norm_kernel(const float *x, const int *row_map, const float *g, void *out, int W, float eps) {
  __shared__ float sh[32];
  const long long r = blockIdx.x;
  const float *xr = x + (long long)(row_map ? row_map[r] : r) * W;
  float s = 0.f;
  for (int i = threadIdx.x; i < W; i += blockDim.x) s += xr[i] * xr[i];
  s = block_sum(s, sh);
  const float k = rsqrtf(s / (float)W + eps) * g[0];
  for (int i = threadIdx.x; i < W; i += blockDim.x) st_el<F32>(out, r * W + i, xr[i] * k);
}
cudaError_t launch_stack_final_norm(const float *x, const int *row_map, const float *g, void *out, bool f32, int R, int W, float eps,
                                    cudaStream_t st) {
  if (f32) stack_final_norm_kernel<true><<<R, 256, 0, st>>>(x, row_map, g, out, W, eps);
  else stack_final_norm_kernel<false><<<R, 256, 0, st>>>(x, row_map, g, out, W, eps);
  return cudaGetLastError();
}

// Layer-norm form of the boundary between two sublayers, one block per token, the row in shared memory.
// y = bias + sum of the n_part slices of the product before; x += (y - mean(y)) / sqrt(var(y) + eps) * post_w + post_b;
// cat (when given) receives [x ; x0] in the compute type (input of the projection in front of a loop pass);
// h = (x - mean(x)) / sqrt(var(x) + eps) * pre_w + pre_b goes to hn (fp32, when given) and hc (compute type, when given).
// The variance is the mean of the squared deviations from the mean (second pass over the row), all in fp32.
// RMS: the norms are v / sqrt(mean(v^2) + eps) * w instead -- no mean is taken off and there is no bias vector.
template <bool F32, bool RMS>
__global__ void __launch_bounds__(256) stack_boundary_ln_kernel(float *x, const float *y, int n_part, long long stride, const float *bias,
                                                                const float *post_w, const float *post_b, const float *pre_w,
                                                                const float *pre_b, float *hn, void *hc, const float *x0, void *cat,
                                                                int W, float eps) {
  extern __shared__ __align__(16) float row[];  // [W]
  __shared__ float sh[32];
  const long long t = blockIdx.x;
  float *xr = x + t * W;
  if (((W | (int)(stride & 3)) & 3) == 0) {
    // W a multiple of 4: a thread owns groups of four neighbouring columns through every phase (16-byte accesses to the
    // slices, the residual, the gains and the outputs; at W = 1024 one group per thread)
    auto f4 = [](const float *p) { return *reinterpret_cast<const float4 *>(p); };
    const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
    if (y) {
      float s = 0.f;
      for (int i = threadIdx.x * 4; i < W; i += blockDim.x * 4) {
        float4 v = bias ? f4(bias + i) : zero;
#pragma unroll 4
        for (int k = 0; k < n_part; k++) {
          const float4 p = f4(y + (long long)k * stride + t * W + i);
          v.x += p.x; v.y += p.y; v.z += p.z; v.w += p.w;
        }
        *reinterpret_cast<float4 *>(row + i) = v;
        s += RMS ? (v.x * v.x + v.y * v.y) + (v.z * v.z + v.w * v.w) : (v.x + v.y) + (v.z + v.w);
      }
      float mean = 0.f, q = 0.f;
      if (RMS) q = s;
      else {
        mean = block_sum(s, sh) / (float)W;
        for (int i = threadIdx.x * 4; i < W; i += blockDim.x * 4) {
          const float4 v = f4(row + i);
          const float a = v.x - mean, b = v.y - mean, c = v.z - mean, d = v.w - mean;
          q += (a * a + b * b) + (c * c + d * d);
        }
      }
      const float r = rsqrtf(block_sum(q, sh) / (float)W + eps);
      for (int i = threadIdx.x * 4; i < W; i += blockDim.x * 4) {
        const float4 v = f4(row + i), g = f4(post_w + i), b = RMS ? zero : f4(post_b + i);
        float4 o = f4(xr + i);
        o.x += (v.x - mean) * r * g.x + b.x; o.y += (v.y - mean) * r * g.y + b.y;
        o.z += (v.z - mean) * r * g.z + b.z; o.w += (v.w - mean) * r * g.w + b.w;
        *reinterpret_cast<float4 *>(xr + i) = o;
        *reinterpret_cast<float4 *>(row + i) = o;
      }
    } else {
      for (int i = threadIdx.x * 4; i < W; i += blockDim.x * 4) *reinterpret_cast<float4 *>(row + i) = f4(xr + i);
    }
    if (cat) {
      __syncthreads();  // the loop below walks the row column by column
      for (int i = threadIdx.x; i < W; i += blockDim.x) {
        st_el<F32>(cat, t * 2 * W + i, row[i]);
        st_el<F32>(cat, t * 2 * W + W + i, x0[t * W + i]);
      }
    }
    if (!pre_w) return;
    float s = 0.f;
    for (int i = threadIdx.x * 4; i < W; i += blockDim.x * 4) {  // each thread re-reads what it wrote itself
      const float4 v = f4(row + i);
      s += RMS ? (v.x * v.x + v.y * v.y) + (v.z * v.z + v.w * v.w) : (v.x + v.y) + (v.z + v.w);
    }
    float mean = 0.f, q = 0.f;
    if (RMS) q = s;
    else {
      mean = block_sum(s, sh) / (float)W;
      for (int i = threadIdx.x * 4; i < W; i += blockDim.x * 4) {
        const float4 v = f4(row + i);
        const float a = v.x - mean, b = v.y - mean, c = v.z - mean, d = v.w - mean;
        q += (a * a + b * b) + (c * c + d * d);
      }
    }
    const float r = rsqrtf(block_sum(q, sh) / (float)W + eps);
    for (int i = threadIdx.x * 4; i < W; i += blockDim.x * 4) {
      const float4 v = f4(row + i), g = f4(pre_w + i), b = RMS ? zero : f4(pre_b + i);
      const float4 h = make_float4((v.x - mean) * r * g.x + b.x, (v.y - mean) * r * g.y + b.y, (v.z - mean) * r * g.z + b.z,
                                   (v.w - mean) * r * g.w + b.w);
      if (hn) *reinterpret_cast<float4 *>(hn + t * W + i) = h;
      if (hc) {
        if (F32) *reinterpret_cast<float4 *>(reinterpret_cast<float *>(hc) + t * W + i) = h;
        else {
          uint2 o;
          o.x = (uint32_t)float_to_bf16_bits(h.x) | ((uint32_t)float_to_bf16_bits(h.y) << 16);
          o.y = (uint32_t)float_to_bf16_bits(h.z) | ((uint32_t)float_to_bf16_bits(h.w) << 16);
          *reinterpret_cast<uint2 *>(reinterpret_cast<uint16_t *>(hc) + t * W + i) = o;
        }
      }
    }
    return;
  }
  if (y) {
    float s = 0.f;
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
      float v = bias ? bias[i] : 0.f;
      for (int k = 0; k < n_part; k++) v += y[(long long)k * stride + t * W + i];
      row[i] = v;
      s += RMS ? v * v : v;
    }
    float mean = 0.f, q = 0.f;
    if (RMS) q = s;
    else {
      mean = block_sum(s, sh) / (float)W;
      for (int i = threadIdx.x; i < W; i += blockDim.x) { const float dvi = row[i] - mean; q += dvi * dvi; }
    }
    const float r = rsqrtf(block_sum(q, sh) / (float)W + eps);
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
      const float v = xr[i] + ((row[i] - mean) * r * post_w[i] + (RMS ? 0.f : post_b[i]));
      xr[i] = v;
      row[i] = v;
    }
  } else {
    for (int i = threadIdx.x; i < W; i += blockDim.x) row[i] = xr[i];
  }
  if (cat) {
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
      st_el<F32>(cat, t * 2 * W + i, row[i]);
      st_el<F32>(cat, t * 2 * W + W + i, x0[t * W + i]);
    }
  }
  if (!pre_w) return;
  float s = 0.f;
  for (int i = threadIdx.x; i < W; i += blockDim.x) s += RMS ? row[i] * row[i] : row[i];  // each thread re-reads what it wrote itself
  float mean = 0.f, q = 0.f;
  if (RMS) q = s;
  else {
    mean = block_sum(s, sh) / (float)W;
    for (int i = threadIdx.x; i < W; i += blockDim.x) { const float dvi = row[i] - mean; q += dvi * dvi; }
  }
  const float r = rsqrtf(block_sum(q, sh) / (float)W + eps);
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    const float h = (row[i] - mean) * r * pre_w[i] + (RMS ? 0.f : pre_b[i]);
    if (hn) hn[t * W + i] = h;
    if (hc) st_el<F32>(hc, t * W + i, h);
  }
}
cudaError_t launch_stack_boundary_ln(float *x, const float *y, int n_part, long long stride, const float *bias, const float *post_w,
                                     const float *post_b, const float *pre_w, const float *pre_b, float *hn, void *hc, const float *x0,
                                     void *cat, bool f32, int T, int W, float eps, bool rms, cudaStream_t st) {
  if ((size_t)W * 4 > 160 * 1024) return cudaErrorInvalidValue;
  if (T <= 0) return cudaSuccess;
  static DeviceOnce once;
  DIS_CUDA_TRY(once.run([&] {
    cudaError_t e = cudaFuncSetAttribute(stack_boundary_ln_kernel<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(stack_boundary_ln_kernel<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(stack_boundary_ln_kernel<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
    return e != cudaSuccess ? e : cudaFuncSetAttribute(stack_boundary_ln_kernel<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
  }));
  const size_t shb = (size_t)W * 4;
#define DIS_BOUNDARY(F, R) \
  stack_boundary_ln_kernel<F, R><<<T, 256, shb, st>>>(x, y, n_part, stride, bias, post_w, post_b, pre_w, pre_b, hn, hc, x0, cat, W, eps)
  if (f32 && rms) DIS_BOUNDARY(true, true);
  else if (f32) DIS_BOUNDARY(true, false);
  else if (rms) DIS_BOUNDARY(false, true);
  else DIS_BOUNDARY(false, false);
#undef DIS_BOUNDARY
  return cudaGetLastError();
}

// b == null: the RMS form, x / sqrt(mean(x^2) + eps) * w.  S > 1: the row is the sum of the token's S residual streams.
template <bool F32>
__global__ void stack_final_ln_kernel(const float *x, const int *row_map, const float *w, const float *b, void *out, int W, float eps,
                                      float scale, int S) {
  extern __shared__ float frow[];  // [W] when S > 1
  __shared__ float sh[32];
  const long long r = blockIdx.x;
  const float *xr = x + (long long)(row_map ? row_map[r] : r) * S * W;
  if (S > 1) {
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
      float v = 0.f;
      for (int k = 0; k < S; k++) v += xr[(long long)k * W + i];
      frow[i] = v;
    }
    __syncthreads();
    xr = frow;
  }
  float mean = 0.f, q = 0.f;
  if (b) {
    float s = 0.f;
    for (int i = threadIdx.x; i < W; i += blockDim.x) s += xr[i];
    mean = block_sum(s, sh) / (float)W;
  }
  for (int i = threadIdx.x; i < W; i += blockDim.x) { const float dvi = xr[i] - mean; q += dvi * dvi; }
  const float k = rsqrtf(block_sum(q, sh) / (float)W + eps);
  for (int i = threadIdx.x; i < W; i += blockDim.x) st_el<F32>(out, r * W + i, ((xr[i] - mean) * k * w[i] + (b ? b[i] : 0.f)) * scale);
}
cudaError_t launch_stack_final_ln(const float *x, const int *row_map, const float *w, const float *b, void *out, bool f32, int R, int W,
                                  float eps, float scale, int streams, cudaStream_t st) {
  if (streams < 1) streams = 1;
  const size_t shb = streams > 1 ? (size_t)W * 4 : 0;
  if (shb > 160 * 1024) return cudaErrorInvalidValue;
  static DeviceOnce once;
  DIS_CUDA_TRY(once.run([&] {
    cudaError_t e = cudaFuncSetAttribute(stack_final_ln_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
    return e != cudaSuccess ? e : cudaFuncSetAttribute(stack_final_ln_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
  }));
  if (f32) stack_final_ln_kernel<true><<<R, 256, shb, st>>>(x, row_map, w, b, out, W, eps, scale, streams);
  else stack_final_ln_kernel<false><<<R, 256, shb, st>>>(x, row_map, w, b, out, W, eps, scale, streams);
  return cudaGetLastError();
}

// Pre-norm boundary over residual streams, one block per token.  xs [T][S][W].  y = bias + the n_part slices of the product before.
// prev (or null) = the coefficients of the sublayer that made y, laid out in[S] | out[S] | mix[S][S] (mix indexed [from][to]):
// every stream becomes x_t <- sum_s mix[s][t] x_s + out[t] y, all from the old streams; prev == null: the one stream gets x += y.
// Then, with pre_w: u = sum_s next[s] x_s (next = the coming sublayer's coefficients, their first S numbers; null: u = x_0), and
// h = u / sqrt(mean(u^2) + eps) * pre_w goes to hc in the compute type.  Everything is fp32.
constexpr int kHcMaxStreams = 8;
// SS: the number of streams when the compiler may know it (2, 4), else 0 and S counts at run time up to kHcMaxStreams.
// VEC: W is a multiple of 4 and every pointer 16-byte aligned, so a thread moves four neighbouring columns per access.
template <bool F32, int SS, bool VEC>
__global__ void __launch_bounds__(256) stack_boundary_hc_kernel(float *xs, int S_rt, const float *__restrict__ y, int n_part, long long stride,
                                                                const float *__restrict__ bias, const float *prev, const float *next,
                                                                const float *__restrict__ pre_w, void *hc, int W, float eps) {
  extern __shared__ __align__(16) float row[];  // [W]: u
  __shared__ float sh[32];
  __shared__ float cf[2 * kHcMaxStreams + kHcMaxStreams * kHcMaxStreams];  // out[S] | mix[S][S] of prev, then in[S] of next
  constexpr int V = VEC ? 4 : 1, SM = SS ? SS : kHcMaxStreams;
  const int S = SS ? SS : S_rt;
  const long long t = blockIdx.x;
  float *xr = xs + t * S * W;
  float *c_out = cf, *c_mix = cf + kHcMaxStreams, *c_in = c_mix + kHcMaxStreams * kHcMaxStreams;
  if (threadIdx.x < S) {
    c_out[threadIdx.x] = prev ? prev[S + threadIdx.x] : 1.f;
    c_in[threadIdx.x] = next ? next[threadIdx.x] : (threadIdx.x == 0 ? 1.f : 0.f);
  }
  if (threadIdx.x < S * S) c_mix[threadIdx.x] = prev ? prev[2 * S + threadIdx.x] : (threadIdx.x % (S + 1) == 0 ? 1.f : 0.f);
  __syncthreads();
  auto ld = [](const float *p, float (&o)[V]) {
    if (VEC) { const float4 v = *reinterpret_cast<const float4 *>(p); o[0] = v.x; o[V > 1 ? 1 : 0] = v.y; o[V > 2 ? 2 : 0] = v.z; o[V > 3 ? 3 : 0] = v.w; }
    else o[0] = p[0];
  };
  auto st = [](float *p, const float (&o)[V]) {
    if (VEC) *reinterpret_cast<float4 *>(p) = make_float4(o[0], o[V > 1 ? 1 : 0], o[V > 2 ? 2 : 0], o[V > 3 ? 3 : 0]);
    else p[0] = o[0];
  };
  float q = 0.f;
  for (int i = threadIdx.x * V; i < W; i += blockDim.x * V) {
    float old[SM][V];
#pragma unroll
    for (int k = 0; k < SM; k++) {
      if (k < S) ld(xr + (long long)k * W + i, old[k]);
      else {
#pragma unroll
        for (int e = 0; e < V; e++) old[k][e] = 0.f;
      }
    }
    float u[V];
#pragma unroll
    for (int e = 0; e < V; e++) u[e] = 0.f;
    if (y) {
      float v[V];
      if (bias) ld(bias + i, v);
      else {
#pragma unroll
        for (int e = 0; e < V; e++) v[e] = 0.f;
      }
      for (int k = 0; k < n_part; k++) {
        float p[V];
        ld(y + (long long)k * stride + t * W + i, p);
#pragma unroll
        for (int e = 0; e < V; e++) v[e] += p[e];
      }
#pragma unroll
      for (int to = 0; to < SM; to++) {
        if (to < S) {
          float nv[V];
#pragma unroll
          for (int e = 0; e < V; e++) nv[e] = c_out[to] * v[e];
#pragma unroll
          for (int from = 0; from < SM; from++)
            if (from < S) {
              const float m = c_mix[from * S + to];
#pragma unroll
              for (int e = 0; e < V; e++) nv[e] = fmaf(m, old[from][e], nv[e]);
            }
          st(xr + (long long)to * W + i, nv);
#pragma unroll
          for (int e = 0; e < V; e++) u[e] = fmaf(c_in[to], nv[e], u[e]);
        }
      }
    } else {
#pragma unroll
      for (int k = 0; k < SM; k++)
        if (k < S) {
#pragma unroll
          for (int e = 0; e < V; e++) u[e] = fmaf(c_in[k], old[k][e], u[e]);
        }
    }
    st(row + i, u);
#pragma unroll
    for (int e = 0; e < V; e++) q += u[e] * u[e];
  }
  if (!pre_w) return;
  const float r = rsqrtf(block_sum(q, sh) / (float)W + eps);
  for (int i = threadIdx.x * V; i < W; i += blockDim.x * V) {  // each thread re-reads what it wrote itself
    float u[V], g[V];
    ld(row + i, u);
    ld(pre_w + i, g);
    if (VEC && !F32) {
      uint2 o;
      o.x = (uint32_t)float_to_bf16_bits(u[0] * r * g[0]) | ((uint32_t)float_to_bf16_bits(u[V > 1 ? 1 : 0] * r * g[V > 1 ? 1 : 0]) << 16);
      o.y = (uint32_t)float_to_bf16_bits(u[V > 2 ? 2 : 0] * r * g[V > 2 ? 2 : 0]) | ((uint32_t)float_to_bf16_bits(u[V > 3 ? 3 : 0] * r * g[V > 3 ? 3 : 0]) << 16);
      *reinterpret_cast<uint2 *>(reinterpret_cast<uint16_t *>(hc) + t * W + i) = o;
    } else if (VEC) {
#pragma unroll
      for (int e = 0; e < V; e++) u[e] = u[e] * r * g[e];
      st(reinterpret_cast<float *>(hc) + t * W + i, u);
    } else st_el<F32>(hc, t * W + i, u[0] * r * g[0]);
  }
}
template <bool F32, int SS, bool VEC>
static cudaError_t boundary_hc_go(float *xs, int streams, const float *y, int n_part, long long stride, const float *bias, const float *prev,
                                  const float *next, const float *pre_w, void *hc, int T, int W, float eps, cudaStream_t st) {
  static DeviceOnce once;
  DIS_CUDA_TRY(once.run([&] { return cudaFuncSetAttribute(stack_boundary_hc_kernel<F32, SS, VEC>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024); }));
  stack_boundary_hc_kernel<F32, SS, VEC><<<T, 256, (size_t)W * 4, st>>>(xs, streams, y, n_part, stride, bias, prev, next, pre_w, hc, W, eps);
  return cudaGetLastError();
}
cudaError_t launch_stack_boundary_hc(float *xs, int streams, const float *y, int n_part, long long stride, const float *bias,
                                     const float *prev, const float *next, const float *pre_w, void *hc, bool f32, int T, int W, float eps,
                                     cudaStream_t st) {
  if (streams < 1 || streams > kHcMaxStreams || (size_t)W * 4 > 160 * 1024) return cudaErrorInvalidValue;
  if (T <= 0) return cudaSuccess;
  if (n_part < 1) n_part = 1;
  auto al = [](const void *p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; };
  const bool vec = W % 4 == 0 && stride % 4 == 0 && al(xs) && al(y) && al(bias) && al(pre_w) && al(hc);
#define DIS_HC(F, SSV, VV) return boundary_hc_go<F, SSV, VV>(xs, streams, y, n_part, stride, bias, prev, next, pre_w, hc, T, W, eps, st)
#define DIS_HC_S(F, VV) do { if (streams == 2) DIS_HC(F, 2, VV); if (streams == 4) DIS_HC(F, 4, VV); DIS_HC(F, 0, VV); } while (0)
  if (f32) { if (vec) DIS_HC_S(true, true); else DIS_HC_S(true, false); }
  else { if (vec) DIS_HC_S(false, true); else DIS_HC_S(false, false); }
#undef DIS_HC_S
#undef DIS_HC
}

__global__ void stack_scale_kernel(float *v, long long n, float s) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) v[i] *= s;
}
cudaError_t launch_stack_scale(float *v, long long n, float s, cudaStream_t st) {
  if (n <= 0) return cudaSuccess;
  stack_scale_kernel<<<(int)std::min<long long>((n + 255) / 256, 148 * 8), 256, 0, st>>>(v, n, s);
  return cudaGetLastError();
}

__global__ void stack_softcap_kernel(float *v, long long n, float cap, float inv) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    v[i] = cap * tanhf(v[i] * inv);
}
cudaError_t launch_stack_softcap(float *v, long long n, float cap, cudaStream_t st) {
  if (n <= 0 || !(cap > 0.f)) return cudaSuccess;
  stack_softcap_kernel<<<(int)std::min<long long>((n + 255) / 256, 148 * 8), 256, 0, st>>>(v, n, cap, 1.f / cap);
  return cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------ input convolution
// Input at absolute position p of the sequence: inside the span from hn, before it from the slot's tail (tail[i] holds position
// pos0 - (taps-1) + i), before the sequence's start zero.  A span that starts at position 0 never reads the tail, so a slot
// that another sequence used before needs no clearing.
constexpr int kCanonMaxTaps = 16;

template <bool F32>
__global__ void stack_canon_kernel(const float *hn, const float *w, const float *state, StackSpans sp, void *hc, int W, int taps) {
  const int t = blockIdx.x;
  const int s = sp.span[t], tok0 = sp.sp_tok0[s], pos0 = sp.sp_pos0[s], slot = sp.sp_slot[s];
  const int back_in_span = t - tok0;  // tokens of the span in front of t
  const float *tail = state + (long long)slot * (taps - 1) * W;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    const float cur = hn[(long long)t * W + i];
    float acc = cur;
    for (int j = 0; j < taps; j++) {
      const int back = taps - 1 - j;
      float v;
      if (back <= back_in_span) v = hn[(long long)(t - back) * W + i];
      else {
        const int ti = (taps - 1) - (back - back_in_span);  // index into the tail
        v = (pos0 + back_in_span - back >= 0) ? tail[(long long)ti * W + i] : 0.f;
      }
      acc = fmaf(w[(long long)i * taps + j], v, acc);
    }
    st_el<F32>(hc, (long long)t * W + i, acc);
  }
}

__global__ void stack_canon_state_kernel(const float *hn, float *state, StackSpans sp, int W, int taps) {
  const int s = blockIdx.x;
  const int tok0 = sp.sp_tok0[s], len = sp.sp_len[s], pos0 = sp.sp_pos0[s], slot = sp.sp_slot[s];
  float *tail = state + (long long)slot * (taps - 1) * W;
  const int n = taps - 1;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    float nv[kCanonMaxTaps];
    for (int k = 0; k < n; k++) {
      const int rel = len - n + k;  // index relative to the span's first token of the position tail'[k] holds
      if (rel >= 0) nv[k] = hn[(long long)(tok0 + rel) * W + i];
      else nv[k] = (pos0 + rel >= 0) ? tail[(long long)(n + rel) * W + i] : 0.f;
    }
    for (int k = 0; k < n; k++) tail[(long long)k * W + i] = nv[k];
  }
}

cudaError_t launch_stack_canon(const float *hn, const float *w, float *state, const StackSpans &sp, void *hc, bool f32, int W,
                               int taps, cudaStream_t st) {
  if (taps < 1 || taps > kCanonMaxTaps) return cudaErrorInvalidValue;
  if (f32) stack_canon_kernel<true><<<sp.T, 256, 0, st>>>(hn, w, state, sp, hc, W, taps);
  else stack_canon_kernel<false><<<sp.T, 256, 0, st>>>(hn, w, state, sp, hc, W, taps);
  if (taps > 1) stack_canon_state_kernel<<<sp.n_spans, 256, 0, st>>>(hn, state, sp, W, taps);
  return cudaGetLastError();
}

// Passes of single tokens (every span one token long): the whole boundary between two sublayers in one kernel, one block per
// token.  y = bias + sum of the n_part split-K slices of the product before (slice stride `stride`); x += post * unit_rms(y);
// hn = pre * unit_rms(x); hc = hn + convolution over the slot's tail and hn; the tail moves on by one.  pre == null: only
// the residual is updated (end of the pass).  taps == 0: no convolution.
template <bool F32>
__global__ void __launch_bounds__(256) stack_boundary_single_kernel(float *x, const float *y, int n_part, long long stride, const float *bias,
                                                                    const float *post, const float *pre, const float *cw, float *cstate,
                                                                    StackSpans sp, void *hc, int W, int taps, float eps) {
  extern __shared__ float row[];  // [W]
  __shared__ float sh[32];
  const long long t = blockIdx.x;
  float *xr = x + t * W;
  if (y) {
    float s = 0.f;
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
      float v = bias ? bias[i] : 0.f;
      for (int k = 0; k < n_part; k++) v += y[(long long)k * stride + t * W + i];
      row[i] = v;
      s += v * v;
    }
    s = block_sum(s, sh);
    const float r = rsqrtf(s / (float)W + eps) * post[0];
    for (int i = threadIdx.x; i < W; i += blockDim.x) { const float v = xr[i] + row[i] * r; xr[i] = v; row[i] = v; }
  } else {
    for (int i = threadIdx.x; i < W; i += blockDim.x) row[i] = xr[i];
  }
  if (!pre) return;
  float s = 0.f;
  for (int i = threadIdx.x; i < W; i += blockDim.x) s += row[i] * row[i];  // each thread re-reads what it wrote itself
  s = block_sum(s, sh);
  const float r = rsqrtf(s / (float)W + eps) * pre[0];
  const int pos = sp.pos[t], slot = sp.slot[t];
  float *tail = cstate + (long long)slot * (taps > 1 ? taps - 1 : 0) * W;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    const float h = row[i] * r;
    float acc = h;
    if (taps >= 1) {
      float old[kCanonMaxTaps];
      for (int j = 0; j < taps - 1; j++) old[j] = pos - (taps - 1 - j) >= 0 ? tail[(long long)j * W + i] : 0.f;
      for (int j = 0; j < taps - 1; j++) acc = fmaf(cw[(long long)i * taps + j], old[j], acc);
      acc = fmaf(cw[(long long)i * taps + taps - 1], h, acc);
      for (int j = 0; j + 2 < taps; j++) tail[(long long)j * W + i] = old[j + 1];
      if (taps > 1) tail[(long long)(taps - 2) * W + i] = h;
    }
    st_el<F32>(hc, t * W + i, acc);
  }
}
cudaError_t launch_stack_boundary_single(float *x, const float *y, int n_part, long long stride, const float *bias, const float *post,
                                         const float *pre, const float *cw, float *cstate, const StackSpans &sp, void *hc, bool f32,
                                         int W, int taps, float eps, cudaStream_t st) {
  if (taps < 0 || taps > kCanonMaxTaps || (size_t)W * 4 > 160 * 1024) return cudaErrorInvalidValue;
  static DeviceOnce once;
  DIS_CUDA_TRY(once.run([&] {
    cudaError_t e = cudaFuncSetAttribute(stack_boundary_single_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
    return e != cudaSuccess ? e : cudaFuncSetAttribute(stack_boundary_single_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
  }));
  const size_t shb = (size_t)W * 4;
  if (f32) stack_boundary_single_kernel<true><<<sp.T, 256, shb, st>>>(x, y, n_part, stride, bias, post, pre, cw, cstate, sp, hc, W, taps, eps);
  else stack_boundary_single_kernel<false><<<sp.T, 256, shb, st>>>(x, y, n_part, stride, bias, post, pre, cw, cstate, sp, hc, W, taps, eps);
  return cudaGetLastError();
}

template <bool F32>
__global__ void stack_copy_act_kernel(const float *hn, void *hc, long long n) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    st_el<F32>(hc, i, hn[i]);
}
cudaError_t launch_stack_copy_act(const float *hn, void *hc, bool f32, long long n, cudaStream_t st) {
  const int grid = (int)std::min<long long>((n + 255) / 256, 148 * 8);
  if (f32) stack_copy_act_kernel<true><<<grid, 256, 0, st>>>(hn, hc, n);
  else stack_copy_act_kernel<false><<<grid, 256, 0, st>>>(hn, hc, n);
  return cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------ gated units
template <int ACT>
__device__ __forceinline__ float glu_unit(float g, float u, float limit) {
  if (ACT == DIS_ACT_RELU2) { const float r = fmaxf(g, 0.f); return r * r; }  // ungated: there is no u
  if (ACT == DIS_ACT_GELU_TANH) return gelu_tanh_(g) * u;
  if (ACT == DIS_ACT_SILU) return g * sigmoid_precise(g) * u;
  g = fminf(g, limit);
  u = fminf(fmaxf(u, -limit), limit);
  return g * sigmoid_precise(1.702f * g) * (u + 1.f);
}
// VEC: ff is a multiple of 4 and every base pointer 16-byte aligned: a thread takes four neighbouring columns (16-byte loads of
// gate and up, one 8- or 16-byte store).  An ungated activation (DIS_ACT_RELU2) reads rows of ff columns, not 2 ff.
template <bool F32, int ACT, bool VEC>
__global__ void stack_glu_kernel(const float *__restrict__ gu, int n_part, long long stride, const float *__restrict__ bias,
                                 void *__restrict__ act, const int *rows_ptr, int M, int ff, float limit) {
  const int rows = rows_ptr ? min(M, rows_ptr[0]) : M;
  for (int r = blockIdx.x; r < rows; r += gridDim.x) {
    constexpr bool GATED = ACT != DIS_ACT_RELU2;
    const float *gr = gu + (long long)r * (GATED ? 2 : 1) * ff;
    if (VEC) {
      for (int c = (blockIdx.y * blockDim.x + threadIdx.x) * 4; c < ff; c += gridDim.y * blockDim.x * 4) {
        const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
        float4 g = *reinterpret_cast<const float4 *>(gr + c), u = GATED ? *reinterpret_cast<const float4 *>(gr + ff + c) : zero4;
        if (bias) {
          const float4 bg = *reinterpret_cast<const float4 *>(bias + c), bu = GATED ? *reinterpret_cast<const float4 *>(bias + ff + c) : zero4;
          g.x += bg.x; g.y += bg.y; g.z += bg.z; g.w += bg.w; u.x += bu.x; u.y += bu.y; u.z += bu.z; u.w += bu.w;
        }
        for (int k = 1; k < n_part; k++) {
          const float4 pg = *reinterpret_cast<const float4 *>(gr + (long long)k * stride + c);
          const float4 pu = GATED ? *reinterpret_cast<const float4 *>(gr + (long long)k * stride + ff + c) : zero4;
          g.x += pg.x; g.y += pg.y; g.z += pg.z; g.w += pg.w; u.x += pu.x; u.y += pu.y; u.z += pu.z; u.w += pu.w;
        }
        const float v0 = glu_unit<ACT>(g.x, u.x, limit), v1 = glu_unit<ACT>(g.y, u.y, limit), v2 = glu_unit<ACT>(g.z, u.z, limit),
                    v3 = glu_unit<ACT>(g.w, u.w, limit);
        if (F32) *reinterpret_cast<float4 *>(reinterpret_cast<float *>(act) + (long long)r * ff + c) = make_float4(v0, v1, v2, v3);
        else {
          uint2 o;
          o.x = (uint32_t)float_to_bf16_bits(v0) | ((uint32_t)float_to_bf16_bits(v1) << 16);
          o.y = (uint32_t)float_to_bf16_bits(v2) | ((uint32_t)float_to_bf16_bits(v3) << 16);
          *reinterpret_cast<uint2 *>(reinterpret_cast<uint16_t *>(act) + (long long)r * ff + c) = o;
        }
      }
    } else {
      for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < ff; c += gridDim.y * blockDim.x) {
        float g = gr[c] + (bias ? bias[c] : 0.f), u = GATED ? gr[ff + c] + (bias ? bias[ff + c] : 0.f) : 0.f;
        for (int k = 1; k < n_part; k++) { g += gr[(long long)k * stride + c]; if (GATED) u += gr[(long long)k * stride + ff + c]; }
        st_el<F32>(act, (long long)r * ff + c, glu_unit<ACT>(g, u, limit));
      }
    }
  }
}
cudaError_t launch_stack_glu(const float *gu, int n_part, long long stride, const float *bias, void *act, bool f32, const int *rows_ptr,
                             int M, int ff, float limit, int kind, cudaStream_t st) {
  if (M <= 0) return cudaSuccess;
  const bool vec = ff % 4 == 0 && stride % 4 == 0 && reinterpret_cast<uintptr_t>(gu) % 16 == 0 && reinterpret_cast<uintptr_t>(act) % 16 == 0 &&
                   reinterpret_cast<uintptr_t>(bias) % 16 == 0;
  const int per = vec ? 4 : 1;
  // few rows: the columns are spread over grid.y as well
  const dim3 grid(std::min(M, 148 * 16), M >= 512 ? 1 : std::min((ff + 256 * per - 1) / (256 * per), 16));
#define DIS_GLU(F, A, V) stack_glu_kernel<F, A, V><<<grid, 256, 0, st>>>(gu, n_part, stride, bias, act, rows_ptr, M, ff, limit)
#define DIS_GLU_ACT(A)                     \
  do {                                     \
    if (f32 && vec) DIS_GLU(true, A, true); \
    else if (f32) DIS_GLU(true, A, false);  \
    else if (vec) DIS_GLU(false, A, true);  \
    else DIS_GLU(false, A, false);          \
  } while (0)
  if (kind == DIS_ACT_GELU_TANH) DIS_GLU_ACT(DIS_ACT_GELU_TANH);
  else if (kind == DIS_ACT_RELU2) DIS_GLU_ACT(DIS_ACT_RELU2);
  else if (kind == DIS_ACT_SILU) DIS_GLU_ACT(DIS_ACT_SILU);
  else DIS_GLU_ACT(DIS_ACT_CLAMPED);
#undef DIS_GLU_ACT
#undef DIS_GLU
  return cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------ router and expert rows
// A block of eight warps takes TB tokens.  Logits: a warp owns a router row (fp32) at a time and forms its product with all TB
// tokens, so a row is fetched once per TB tokens; with W a multiple of 4 a lane reads 16 bytes of the row and 4 elements of
// every token per step, all loads of a row in flight together.  Choice: warp i then chooses for token i.  E <= 1024 (a token's
// scores sit in shared memory).
// DIS_ROUTE_SOFTMAX_TOP: `top` rounds of arg-max over the logits (lowest index wins a tie), weights = softmax over the chosen.
// DIS_ROUTE_SIGMOID_GROUPS: s = sigmoid(z), c = s + correction; with groups > 1 the expert indices are cut into `groups`
// contiguous runs, a run is ranked by the sum of its top two c, and experts of runs ranked below `keep` get c = -inf; `top`
// rounds of arg-max over c; weight of a chosen expert = its s over the chosen experts' sum of s (+ 1e-20).
// extra (or null): one more fp32 row [W] whose product with the token lands in extra_out[t] (the logit of a per-token gate).
constexpr int kRouteWarps = 8;
template <bool F32>
__device__ __forceinline__ void ld_act4(const void *p, long long i, float (&v)[4]) {  // 4 consecutive activations, i % 4 == 0
  if (F32) {
    const float4 a = *reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(p) + i);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
  } else {
    const uint2 u = *reinterpret_cast<const uint2 *>(reinterpret_cast<const uint16_t *>(p) + i);
    v[0] = __uint_as_float(u.x << 16); v[1] = __uint_as_float(u.x & 0xffff0000u);
    v[2] = __uint_as_float(u.y << 16); v[3] = __uint_as_float(u.y & 0xffff0000u);
  }
}
template <bool F32, int TB>
__global__ void __launch_bounds__(kRouteWarps * 32) stack_route_kernel(const void *hc, const float *__restrict__ router, int T, int W, int E,
                                                                       int top, int kind, const float *__restrict__ correction, int groups,
                                                                       int keep, const float *__restrict__ extra, float *extra_out,
                                                                       int *idx, float *wt) {
  extern __shared__ float zs[];  // per token: [E] logits (sigmoid scores), [E] choice scores, [groups] run scores, [groups] kept flags;
                                 // then [E] correction, [warps][TB] partial sums of the extra row
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  const int t0 = blockIdx.x * TB, nt = min(TB, T - t0);
  const int per_tok = 2 * E + 2 * max(groups, 1);
  float *corr_s = zs + TB * per_tok, *xpart = corr_s + E;
  const bool vec = (W & 3) == 0;
  // the correction vector comes into shared memory beside the products (the choice below then waits for no global load)
  if (correction)
    for (int e = threadIdx.x; e < E; e += blockDim.x) corr_s[e] = correction[e];
  // row `r` of the router (or the extra row) against the block's tokens over the columns first, first + step, ...: the lane's sums
  auto row_dot = [&](const float *wr, int first, int step, float (&acc)[TB]) {
#pragma unroll
    for (int j = 0; j < TB; j++) acc[j] = 0.f;
    if (vec) {
#pragma unroll 4
      for (int i = first * 4; i < W; i += step * 4) {
        const float4 r = *reinterpret_cast<const float4 *>(wr + i);
#pragma unroll
        for (int j = 0; j < TB; j++) {
          if (j < nt) {
            float v[4];
            ld_act4<F32>(hc, (long long)(t0 + j) * W + i, v);
            acc[j] = fmaf(v[0], r.x, fmaf(v[1], r.y, fmaf(v[2], r.z, fmaf(v[3], r.w, acc[j]))));
          }
        }
      }
    } else {
      for (int i = first; i < W; i += step) {
        const float r = wr[i];
#pragma unroll
        for (int j = 0; j < TB; j++)
          if (j < nt) acc[j] = fmaf(ld_el<F32>(hc, (long long)(t0 + j) * W + i), r, acc[j]);
      }
    }
  };
  for (int e = w; e < E; e += kRouteWarps) {  // a warp per expert row
    float acc[TB];
    row_dot(router + (long long)e * W, l, 32, acc);
#pragma unroll
    for (int j = 0; j < TB; j++) {
      const float sum = warp_sum(acc[j]);
      if (l == 0 && j < nt) zs[j * per_tok + e] = sum;
    }
  }
  if (extra) {  // the one extra row is shared by all warps (each an eighth of the columns), so that no warp walks a row alone
    float acc[TB];
    row_dot(extra, threadIdx.x, kRouteWarps * 32, acc);
#pragma unroll
    for (int j = 0; j < TB; j++) {
      const float sum = warp_sum(acc[j]);
      if (l == 0) xpart[w * TB + j] = sum;
    }
  }
  __syncthreads();
  if (extra && threadIdx.x < nt) {
    float sum = 0.f;
    for (int k = 0; k < kRouteWarps; k++) sum += xpart[k * TB + threadIdx.x];
    extra_out[t0 + threadIdx.x] = sum;
  }
  // ---- the choice.  Up to 32 experts: one thread per token walks its scores serially (a short chain without shuffles or
  // barriers; every token of the pass chooses at the same time); more: one warp per token.
  if (E <= 32) {
    const int j = threadIdx.x;
    if (j >= nt) return;
    const int t = t0 + j;
    float *z = zs + j * per_tok, *c = z + E, *gs = c + E;
    const bool sig = kind == DIS_ROUTE_SIGMOID_GROUPS;
    if (sig) {
      for (int e = 0; e < E; e++) {
        const float sv = sigmoid_precise(z[e]);
        z[e] = sv;
        c[e] = sv + corr_s[e];
      }
      if (groups > 1 && keep < groups) {
        const int per = E / groups;
        for (int g = 0; g < groups; g++) {
          float a = -INFINITY, b = -INFINITY;  // the two largest of the run
          for (int k = 0; k < per; k++) {
            const float v = c[g * per + k];
            if (v > a) { b = a; a = v; }
            else if (v > b) b = v;
          }
          gs[g] = per > 1 ? a + b : a;
        }
        unsigned kept = 0;  // groups <= E <= 32
        for (int k = 0; k < keep; k++) {
          float best = -INFINITY;
          int bi = -1;
          for (int g = 0; g < groups; g++)
            if (!((kept >> g) & 1u) && (bi < 0 || gs[g] > best)) { best = gs[g]; bi = g; }
          if (bi >= 0) kept |= 1u << bi;
        }
        for (int e = 0; e < E; e++)
          if (!((kept >> (e / per)) & 1u)) c[e] = -INFINITY;
      }
    }
    float *score = sig ? c : z;
    float m0 = 0.f, den = 0.f;
    for (int k = 0; k < top; k++) {
      float best = -INFINITY;
      int bi = -1;
      for (int e = 0; e < E; e++)
        if (score[e] > best) { best = score[e]; bi = e; }  // strict: the lowest index wins a tie
      if (bi < 0) bi = 0;  // nothing left to choose from (the configuration check rules it out)
      if (k == 0) m0 = best;
      const float p = sig ? z[bi] : expf(best - m0);
      den += p;
      idx[(long long)t * top + k] = bi;
      wt[(long long)t * top + k] = p;
      score[bi] = -INFINITY;
    }
    const float inv = sig ? 1.f / (den + 1e-20f) : 1.f / den;
    for (int k = 0; k < top; k++) wt[(long long)t * top + k] *= inv;
    return;
  }
  for (int j = w; j < nt; j += kRouteWarps) {
    const int t = t0 + j;
    float *z = zs + j * per_tok, *c = z + E, *gs = c + E;
    const bool sig = kind == DIS_ROUTE_SIGMOID_GROUPS;
    if (sig) {
      for (int e = l; e < E; e += 32) {
        const float sv = sigmoid_precise(z[e]);
        z[e] = sv;
        c[e] = sv + corr_s[e];
      }
      __syncwarp();
      if (groups > 1 && keep < groups) {
        const int per = E / groups;
        int *kept = reinterpret_cast<int *>(gs + groups);  // [groups]
        for (int g = l; g < groups; g += 32) {
          float a = -INFINITY, b = -INFINITY;  // the two largest of the run
          for (int k = 0; k < per; k++) {
            const float v = c[g * per + k];
            if (v > a) { b = a; a = v; }
            else if (v > b) b = v;
          }
          gs[g] = per > 1 ? a + b : a;
          kept[g] = 0;
        }
        __syncwarp();
        for (int k = 0; k < keep; k++) {  // keep rounds of arg-max over the runs not yet kept (lowest index wins a tie)
          float best = -INFINITY;
          int bi = 0x7fffffff;
          for (int g = l; g < groups; g += 32) {
            const float v = gs[g];
            if (!kept[g] && (v > best || (v == best && g < bi))) { best = v; bi = g; }
          }
          for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
          }
          if (l == 0 && bi != 0x7fffffff) kept[bi] = 1;
          __syncwarp();
        }
        for (int e = l; e < E; e += 32)
          if (!kept[e / per]) c[e] = -INFINITY;
        __syncwarp();
      }
    }
    const float *score = sig ? c : z;
    float *taken = sig ? c : z;
    float m0 = 0.f, den = 0.f, mine = 0.f;
    for (int k = 0; k < top; k++) {
      float best = -INFINITY;
      int bi = 0x7fffffff;
      for (int e = l; e < E; e += 32) {
        const float v = score[e];
        if (v > best || (v == best && e < bi)) { best = v; bi = e; }
      }
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
      }
      if (bi == 0x7fffffff) bi = 0;  // nothing left to choose from (the configuration check rules it out)
      if (k == 0) m0 = best;
      const float p = sig ? z[bi] : expf(best - m0);
      den += p;
      if (l == k % 32) mine = p;  // lane k keeps the k-th weight (top <= 32)
      __syncwarp();
      if (l == 0) { idx[(long long)t * top + k] = bi; taken[bi] = -INFINITY; }
      __syncwarp();
    }
    if (l < top) wt[(long long)t * top + l] = sig ? mine / (den + 1e-20f) : mine / den;
  }
}
cudaError_t launch_stack_route(const void *hc, bool f32, const float *router, int T, int W, int E, int top, int kind,
                               const float *correction, int groups, int keep, const float *extra, float *extra_out, int *idx, float *wt,
                               cudaStream_t st) {
  if (E > 1024 || top > 32 || top > E) return cudaErrorInvalidValue;
  // softmax over all experts, then the chosen scores over their sum: the softmax's common factor cancels, and its 1e-20 guard
  // lies below the last bit of a sum that is at least 1 / E -- the weights are the softmax over the chosen logits
  if (kind == DIS_ROUTE_SOFTMAX_ALL) kind = DIS_ROUTE_SOFTMAX_TOP;
  if (kind == DIS_ROUTE_SIGMOID_GROUPS && (!correction || groups < 0 || (groups > 1 && (E % groups || keep < 1)))) return cudaErrorInvalidValue;
  if (T <= 0) return cudaSuccess;
  // prompt-sized passes: eight tokens share every fetch of a router row; small passes keep a block per token (more blocks)
  const int per_tok = 2 * E + 2 * std::max(groups, 1);
  const int tb = T >= 1024 && (size_t)(8 * per_tok + E + 8 * kRouteWarps) * sizeof(float) <= 48 * 1024 ? 8 : 1;
  const size_t sh = (size_t)(tb * per_tok + E + tb * kRouteWarps) * sizeof(float);
  const int grid = (T + tb - 1) / tb, th = kRouteWarps * 32;
#define DIS_ROUTE(F, B) \
  stack_route_kernel<F, B><<<grid, th, sh, st>>>(hc, router, T, W, E, top, kind, correction, groups, keep, extra, extra_out, idx, wt)
  if (f32 && tb == 8) DIS_ROUTE(true, 8);
  else if (f32) DIS_ROUTE(true, 1);
  else if (tb == 8) DIS_ROUTE(false, 8);
  else DIS_ROUTE(false, 1);
#undef DIS_ROUTE
  return cudaGetLastError();
}

// Rows of the experts' matrices: the (token, choice) pairs grouped by expert, every expert's rows padded to whole row tiles in
// the tile list only (the row space itself is dense).  One block.  Inside an expert's range the pairs land in the order their
// threads arrive; a row's result does not depend on where in the range it lies, so the values are the same run to run.
__global__ void stack_moe_plan_kernel(const int *idx, int n, int top, int E, int tile_rows, int *counts, int *perm_tok, int *where,
                                      int *tiles, int max_tiles) {
  extern __shared__ int sh[];  // [E] counts, [E] cursors
  int *cnt = sh, *cur = sh + E;
  for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < n; i += blockDim.x) atomicAdd(&cnt[idx[i]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int o = 0, nt = 0;
    for (int e = 0; e < E; e++) {
      cur[e] = o;
      for (int r = 0; r < cnt[e] && nt < max_tiles; r += tile_rows) {
        tiles[1 + 3 * nt] = e; tiles[2 + 3 * nt] = o + r; tiles[3 + 3 * nt] = min(tile_rows, cnt[e] - r);
        nt++;
      }
      o += cnt[e];
      counts[e] = cnt[e];
    }
    tiles[0] = nt;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int o = atomicAdd(&cur[idx[i]], 1);
    perm_tok[o] = i / top;
    where[i] = o;
  }
}
cudaError_t launch_stack_moe_plan(const int *idx, int T, int top, int E, int tile_rows, int *counts, int *perm_tok, int *where,
                                  int *tiles, int max_tiles, cudaStream_t st) {
  stack_moe_plan_kernel<<<1, 1024, (size_t)2 * E * sizeof(int), st>>>(idx, T * top, top, E, tile_rows, counts, perm_tok, where, tiles,
                                                                      max_tiles);
  return cudaGetLastError();
}

// rows of the expert row space, in bf16: row o = activation row perm_tok[o]
__global__ void stack_moe_gather_kernel(const uint16_t *hc, const int *perm_tok, uint16_t *xs, int W) {
  const long long o = blockIdx.x;
  const uint16_t *src = hc + (long long)perm_tok[o] * W;
  for (int i = threadIdx.x; i < W; i += blockDim.x) xs[o * W + i] = src[i];
}
cudaError_t launch_stack_moe_gather(const void *hc, const int *perm_tok, void *xs, int rows, int W, cudaStream_t st) {
  if (rows <= 0) return cudaSuccess;
  stack_moe_gather_kernel<<<rows, 128, 0, st>>>(reinterpret_cast<const uint16_t *>(hc), perm_tok, reinterpret_cast<uint16_t *>(xs), W);
  return cudaGetLastError();
}

// y = sum_k wt_k * (row of choice k) [+ sigmoid(shared_gate[t]) * shared[t]]: the shared expert's output, when there is one,
// joins here behind its per-token gate
__global__ void stack_moe_combine_kernel(const float *rows, const int *where, const float *wt, const float *shared, int n_part,
                                         long long stride, const float *shared_gate, float *y, int W, int top) {
  const long long t = blockIdx.x;
  const float sg = shared ? (shared_gate ? sigmoid_precise(shared_gate[t]) : 1.f) : 0.f;  // no gate: the shared unit joins as it is
  if (((W | (int)(stride & 3)) & 3) == 0) {  // four columns per thread and step, 16-byte accesses
    for (int i = threadIdx.x * 4; i < W; i += blockDim.x * 4) {
      float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int k = 0; k < top; k++) {
        const float wk = wt[t * top + k];
        const float4 r = *reinterpret_cast<const float4 *>(rows + (long long)where[t * top + k] * W + i);
        s.x = fmaf(wk, r.x, s.x); s.y = fmaf(wk, r.y, s.y); s.z = fmaf(wk, r.z, s.z); s.w = fmaf(wk, r.w, s.w);
      }
      if (shared) {
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
        for (int k = 0; k < n_part; k++) {
          const float4 p = *reinterpret_cast<const float4 *>(shared + (long long)k * stride + t * W + i);
          v.x += p.x; v.y += p.y; v.z += p.z; v.w += p.w;
        }
        s.x = fmaf(sg, v.x, s.x); s.y = fmaf(sg, v.y, s.y); s.z = fmaf(sg, v.z, s.z); s.w = fmaf(sg, v.w, s.w);
      }
      *reinterpret_cast<float4 *>(y + t * W + i) = s;
    }
    return;
  }
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    float s = 0.f;
    for (int k = 0; k < top; k++) s = fmaf(wt[t * top + k], rows[(long long)where[t * top + k] * W + i], s);
    if (shared) {
      float v = 0.f;
      for (int k = 0; k < n_part; k++) v += shared[(long long)k * stride + t * W + i];
      s = fmaf(sg, v, s);
    }
    y[t * W + i] = s;
  }
}
cudaError_t launch_stack_moe_combine(const float *rows, const int *where, const float *wt, const float *shared, int n_part,
                                     long long stride, const float *shared_gate, float *y, int T, int W, int top, cudaStream_t st) {
  stack_moe_combine_kernel<<<T, 256, 0, st>>>(rows, where, wt, shared, n_part < 1 ? 1 : n_part, stride, shared_gate, y, W, top);
  return cudaGetLastError();
}

}  // namespace dis
