// Row operations of models whose sublayers sit between LAYER norms (weight and bias) on a 32-bit residual stream, and the
// parts of a mixture-of-experts feed-forward:
//   embed_rows     x = table[id] in fp32 (and a second copy that a looped block of layers adds back before each repeat)
//   ln_add_norm    x += mult * LN_post(y);  x += extra;  h = LN_pre(x)    (each part optional, one pass over the row)
//   ln_gather      h[r] = LN(x[rows[r]]) for the few rows whose logits are wanted
//   gated_act      out = act(gate) * up  (or act(gate) alone) on column ranges of one projection's output
//   router_topk    softmax over the experts' logits, the `top` largest (by score, or by score plus a correction), renormalised or not
//   moe_plan       (token, choice) pairs grouped by expert into row tiles
//   moe_gemm       one projection of every expert over its own rows (gather on the way in, activation or routing weight on
//                  the way out); moe_fewrows does the same for a handful of pairs with one warp per output
//   moe_gather     the experts' input rows laid out in the plan's order, for projections that want contiguous rows
//   moe_combine    y[token] = sum over its choices (+ the shared expert's output); identity experts hand the token itself back
// LN is (x - mean) / sqrt(mean((x - mean)^2) + eps) * w + b with fp32 statistics taken in two passes over a staged row.
#include <math.h>

#include "common.cuh"

namespace {

template <typename T> __device__ __forceinline__ float ldf(const T* p);
template <> __device__ __forceinline__ float ldf<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ldf<bf16>(const bf16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void stf(T* p, float v);
template <> __device__ __forceinline__ void stf<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void stf<bf16>(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

template <int NT>
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float s = 0.f;
#pragma unroll
  for (int w = 0; w < NT / 32; ++w) s += red[w];
  return s;
}

// mean and 1/sqrt(var + eps) of the W floats in `row` (shared memory; every thread reads only what it wrote itself, or
// the caller has synchronised)
__device__ __forceinline__ void row_stats(const float* row, int W, float eps, float* red, float& mean, float& inv) {
  float s = 0.f;
  for (int i = threadIdx.x; i < W; i += 256) s += row[i];
  mean = block_sum<256>(s, red) / (float)W;
  float ss = 0.f;
  for (int i = threadIdx.x; i < W; i += 256) {
    const float d = row[i] - mean;
    ss += d * d;
  }
  inv = 1.0f / sqrtf(block_sum<256>(ss, red) / (float)W + eps);
}

template <typename T>
__global__ void __launch_bounds__(256) embed_rows_kernel(const int64_t* __restrict__ ids, const T* __restrict__ table, float* __restrict__ x,
                                                         float* __restrict__ x_copy, int W, int vocab) {
  long long id = ids[blockIdx.x];
  if (id < 0 || id >= vocab) id = 0;     // the host checks the range; never read outside the table
  const T* e = table + (size_t)id * W;
  for (int i = threadIdx.x; i < W; i += 256) {
    const float v = ldf(e + i);
    x[(size_t)blockIdx.x * W + i] = v;
    if (x_copy) x_copy[(size_t)blockIdx.x * W + i] = v;
  }
}

template <typename TY, typename TH>
__global__ void __launch_bounds__(256) ln_add_norm_kernel(float* __restrict__ x, const TY* __restrict__ y, const float* __restrict__ w_post,
                                                          const float* __restrict__ b_post, float mult, const float* __restrict__ extra,
                                                          const float* __restrict__ w_pre, const float* __restrict__ b_pre, TH* __restrict__ h, int W,
                                                          float eps) {
  extern __shared__ float xs[];
  __shared__ float red[8];
  const size_t base = (size_t)blockIdx.x * W;
  float mean, inv;
  if (y != nullptr) {
    for (int i = threadIdx.x; i < W; i += 256) xs[i] = ldf(y + base + i);
    row_stats(xs, W, eps, red, mean, inv);
    for (int i = threadIdx.x; i < W; i += 256) {
      float v = x[base + i] + mult * ((xs[i] - mean) * inv * w_post[i] + b_post[i]);
      if (extra) v += extra[base + i];
      x[base + i] = v;
      xs[i] = v;
    }
  } else {
    for (int i = threadIdx.x; i < W; i += 256) {
      float v = x[base + i];
      if (extra) {
        v += extra[base + i];
        x[base + i] = v;
      }
      xs[i] = v;
    }
  }
  if (h == nullptr) return;
  row_stats(xs, W, eps, red, mean, inv);
  for (int i = threadIdx.x; i < W; i += 256) stf(h + base + i, (xs[i] - mean) * inv * w_pre[i] + b_pre[i]);
}

template <typename TH>
__global__ void __launch_bounds__(256) ln_gather_kernel(const float* __restrict__ x, const int* __restrict__ rows, const float* __restrict__ w,
                                                        const float* __restrict__ b, TH* __restrict__ h, int W, float eps) {
  extern __shared__ float xs[];
  __shared__ float red[8];
  const size_t src = (size_t)rows[blockIdx.x] * W, dst = (size_t)blockIdx.x * W;
  for (int i = threadIdx.x; i < W; i += 256) xs[i] = x[src + i];
  float mean, inv;
  row_stats(xs, W, eps, red, mean, inv);
  for (int i = threadIdx.x; i < W; i += 256) stf(h + dst + i, (xs[i] - mean) * inv * w[i] + b[i]);
}

// ---------------------------------------------------------------------------------------------------- activations
__device__ __forceinline__ float act_apply(float z, int act) {
  switch (act) {
    case LIA_ACT_RELU: return fmaxf(z, 0.f);
    case LIA_ACT_SILU: return z / (1.0f + expf(-z));
    case LIA_ACT_GELU_ERF: return 0.5f * z * (1.0f + erff(z * 0.70710678118654752440f));
    case LIA_ACT_GELU_TANH: return 0.5f * z * (1.0f + tanhf(0.79788456080286535588f * (z + 0.044715f * z * z * z)));
    default: return z;
  }
}

// the product of a gated feed-forward: act(g) * u, or (LIA_ACT_CLAMPED_SWISH, p0 = limit, p1 = alpha) with g' = min(g, limit) and
// u' = clamp(u, -limit, limit): g' * sigmoid(alpha g') * (u' + 1)
__device__ __forceinline__ float gated_apply(float g, float u, int act, float p0, float p1) {
  if (act == LIA_ACT_CLAMPED_SWISH) {
    g = fminf(g, p0);
    u = fminf(fmaxf(u, -p0), p0);
    return g / (1.0f + expf(-p1 * g)) * (u + 1.0f);
  }
  return act_apply(g, act) * u;
}

// out[m][f] = act(in[m][f]) * in[m][up_off + f]   (up_off < 0: no second factor)
template <typename T>
__global__ void gated_act_kernel(const T* __restrict__ in, int ld, int up_off, T* __restrict__ out, int M, int F, int act) {
  const size_t n = (size_t)M * F;
  for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (size_t)gridDim.x * blockDim.x) {
    const size_t m = e / F;
    const int f = (int)(e - m * F);
    float v = act_apply(ldf(in + m * ld + f), act);
    if (up_off >= 0) v *= ldf(in + m * ld + up_off + f);
    stf(out + e, v);
  }
}

// ---------------------------------------------------------------------------------------------------- router
// One warp per token: softmax over E logits (fp32), then `top` rounds of arg-max (lowest index on ties) over the scores
// plus an optional per-expert correction that takes part in the choice only; a chosen expert's weight is its plain
// score, divided by their sum (+ 1e-20) when `renorm` is set.
__global__ void __launch_bounds__(128) router_topk_kernel(const float* __restrict__ logits, const float* __restrict__ correction, int* __restrict__ idx,
                                                          float* __restrict__ wt, int M, int E, int top, int renorm) {
  extern __shared__ float sc[];          // [4 warps][2][E]: scores, choice scores
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * 4 + warp;
  if (row >= M) return;
  float* s = sc + warp * 2 * E;
  float* ch = s + E;
  const float* z = logits + (size_t)row * E;
  float mx = -INFINITY;
  for (int e = lane; e < E; e += 32) mx = fmaxf(mx, z[e]);
  mx = warp_max(mx);
  float sum = 0.f;
  for (int e = lane; e < E; e += 32) {
    const float p = expf(z[e] - mx);
    s[e] = p;
    sum += p;
  }
  sum = warp_sum(sum);
  for (int e = lane; e < E; e += 32) {
    s[e] = s[e] / sum;
    ch[e] = s[e] + (correction ? correction[e] : 0.f);
  }
  __syncwarp();
  float chosen_sum = 0.f;
  for (int t = 0; t < top; ++t) {
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      const float p = ch[e];
      if (p > best) { best = p; bi = e; }          // ascending e: the first of equal scores stays
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    const float score = s[bi];
    chosen_sum += score;
    __syncwarp();
    if (lane == 0) {
      idx[(size_t)row * top + t] = bi;
      wt[(size_t)row * top + t] = score;
      ch[bi] = -INFINITY;                           // taken
    }
    __syncwarp();
  }
  __syncwarp();
  if (renorm)
    for (int t = lane; t < top; t += 32) wt[(size_t)row * top + t] = wt[(size_t)row * top + t] / (chosen_sum + 1e-20f);
}

// ---------------------------------------------------------------------------------------------------- experts
constexpr int TM = 64;        // rows of a tile of the grouped projection

// One block.  pairs = M * top (token, choice) pairs; expert e gets ceil(count_e / TM) tiles, one after the other.
//   perm[tile * TM + r] = pair index, or -1 in the padding of an expert's last tile
//   tile_expert[tile]   = expert of the tile, -1 for the unused tiles at the end (n_tiles of them exist in all)
//   pos_of[pair]        = its place in perm (the row of the experts' intermediate buffer)
__global__ void __launch_bounds__(1024) moe_plan_kernel(const int* __restrict__ idx, int pairs, int E, int n_tiles, int* __restrict__ perm,
                                                        int* __restrict__ tile_expert, int* __restrict__ pos_of) {
  extern __shared__ int sh[];            // count[E] | offset[E]
  int* count = sh;
  int* offset = sh + E;
  for (int e = threadIdx.x; e < E; e += 1024) count[e] = 0;
  for (int i = threadIdx.x; i < n_tiles * TM; i += 1024) perm[i] = -1;
  for (int i = threadIdx.x; i < n_tiles; i += 1024) tile_expert[i] = -1;
  __syncthreads();
  for (int p = threadIdx.x; p < pairs; p += 1024) pos_of[p] = atomicAdd(&count[idx[p]], 1);      // rank inside its expert
  __syncthreads();
  if (threadIdx.x == 0) {
    int tile = 0;
    for (int e = 0; e < E; ++e) {
      offset[e] = tile * TM;
      const int nt = (count[e] + TM - 1) / TM;
      for (int t = 0; t < nt; ++t) tile_expert[tile + t] = e;
      tile += nt;
    }
  }
  __syncthreads();
  for (int p = threadIdx.x; p < pairs; p += 1024) {
    const int at = offset[idx[p]] + pos_of[p];
    perm[at] = p;
    pos_of[p] = at;
  }
}

// C[row][n] = epilogue(sum_k A[src(row)][k] * W[e][n][k]) for the rows of tile blockIdx.y (expert e = tile_expert[tile]).
//   UP   (gather by token):  src = perm[row] / top,  C = mid[row][n]      = act(sum)
//   DOWN (rows in place):    src = row,              C = ypair[perm[row]] = wt[perm[row]] * sum     (fp32)
// 64 x 64 tile, 16-wide k slabs, 4 x 4 outputs per thread, fp32 products and sums in k order (as the plain projection).
// GATED (UP only): an expert's weights are [2N][K], N gate rows then N up rows, and C = act(gate sum) * (up sum).
// Tiles of experts >= n_real (experts without weights, whose pairs the combining step serves) are skipped.
template <typename TA, typename TW, typename TC, bool UP, bool GATED>
__global__ void __launch_bounds__(256) moe_gemm_kernel(const TA* __restrict__ A, int lda, const TW* __restrict__ Wt, long long sW, TC* __restrict__ C,
                                                       int ldc, const int* __restrict__ perm, const int* __restrict__ tile_expert,
                                                       const float* __restrict__ wt, int top, int N, int K, int act, int n_real, float p0, float p1) {
  const int e = tile_expert[blockIdx.y];
  if (e < 0 || e >= n_real) return;
  __shared__ float As[16][TM + 4];
  __shared__ float Ws[16][64 + 4];
  __shared__ float Wu[GATED ? 16 : 1][64 + 4];
  __shared__ int src[TM], dstp[TM];
  const int row0 = blockIdx.y * TM, n0 = blockIdx.x * 64;
  if (threadIdx.x < TM) {
    const int p = perm[row0 + threadIdx.x];
    dstp[threadIdx.x] = p;
    src[threadIdx.x] = p < 0 ? -1 : (UP ? p / top : row0 + (int)threadIdx.x);
  }
  __syncthreads();
  Wt += (size_t)e * sW;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  float acc[4][4], accu[GATED ? 4 : 1][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      acc[i][j] = 0.f;
      if constexpr (GATED) accu[i][j] = 0.f;
    }
  for (int k0 = 0; k0 < K; k0 += 16) {
    for (int t = threadIdx.x; t < 64 * 16; t += 256) {
      const int r = t >> 4, kk = t & 15;
      const int k = k0 + kk;
      As[kk][r] = (src[r] >= 0 && k < K) ? ldf(A + (size_t)src[r] * lda + k) : 0.f;
      Ws[kk][r] = (n0 + r < N && k < K) ? ldf(Wt + (size_t)(n0 + r) * K + k) : 0.f;
      if constexpr (GATED) Wu[kk][r] = (n0 + r < N && k < K) ? ldf(Wt + (size_t)(N + n0 + r) * K + k) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < 16; ++kk) {
      float av[4], wv[4], uv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) av[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        wv[j] = Ws[kk][tx * 4 + j];
        if constexpr (GATED) uv[j] = Wu[kk][tx * 4 + j];
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
          if constexpr (GATED) accu[i][j] = fmaf(av[i], uv[j], accu[i][j]);
        }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = ty * 4 + i;
    const int p = dstp[r];
    if (p < 0) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= N) continue;
      if (UP) stf(C + (size_t)(row0 + r) * ldc + n, GATED ? gated_apply(acc[i][j], accu[i][j], act, p0, p1) : act_apply(acc[i][j], act));
      else stf(C + (size_t)p * ldc + n, acc[i][j] * wt[p]);
    }
  }
}

// 8 consecutive numbers of a row as floats
__device__ __forceinline__ void load8(const bf16* p, int k, int K, bool vec, float* f) {
  if (vec && k + 8 <= K) {
    unpack8(*reinterpret_cast<const uint4*>(p + k), f);
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = k + j < K ? __bfloat162float(p[k + j]) : 0.f;
  }
}
__device__ __forceinline__ void load8(const float* p, int k, int K, bool vec, float* f) {
  if (vec && k + 8 <= K) {
    const float4 lo = *reinterpret_cast<const float4*>(p + k), hi = *reinterpret_cast<const float4*>(p + k + 4);
    f[0] = lo.x; f[1] = lo.y; f[2] = lo.z; f[3] = lo.w; f[4] = hi.x; f[5] = hi.y; f[6] = hi.z; f[7] = hi.w;
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = k + j < K ? p[k + j] : 0.f;
  }
}

// The same projections for a handful of pairs (decoding): one warp per output n of pair p reads row n of expert idx[p]
// with 128-bit loads; memory-bound on the chosen experts' weights.  UP: A row = token p / top, C row = p, act applied.
// DOWN: A row = p, C row = p, times wt[p].  gated (UP): row N + n of the expert is the second factor, C = act(gate) * up.
// Pairs of experts >= n_real are skipped.
template <typename TA, typename TW, typename TC, bool UP>
__global__ void __launch_bounds__(128) moe_fewrows_kernel(const TA* __restrict__ A, int lda, const TW* __restrict__ Wt, long long sW, TC* __restrict__ C,
                                                          int ldc, const int* __restrict__ idx, const float* __restrict__ wt, int top, int N, int K,
                                                          int act, int gated, int n_real, float p0, float p1) {
  const int p = blockIdx.y, n = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (n >= N || idx[p] >= n_real) return;
  const TW* wr = Wt + (size_t)idx[p] * sW + (size_t)n * K;
  const TA* ar = A + (size_t)(UP ? p / top : p) * lda;
  const bool va = (reinterpret_cast<uintptr_t>(A) % 16 == 0) && ((size_t)lda * sizeof(TA)) % 16 == 0;
  const bool vw = (reinterpret_cast<uintptr_t>(Wt) % 16 == 0) && ((size_t)K * sizeof(TW)) % 16 == 0 && ((size_t)sW * sizeof(TW)) % 16 == 0;
  float acc = 0.f, accu = 0.f;
  for (int k = lane * 8; k < K; k += 256) {
    float av[8], wv[8];
    load8(ar, k, K, va, av);
    load8(wr, k, K, vw, wv);
#pragma unroll
    for (int i = 0; i < 8; ++i) acc = fmaf(av[i], wv[i], acc);
    if (UP && gated) {
      load8(wr + (size_t)N * K, k, K, vw, wv);
#pragma unroll
      for (int i = 0; i < 8; ++i) accu = fmaf(av[i], wv[i], accu);
    }
  }
  acc = warp_sum(acc);
  if (UP && gated) accu = warp_sum(accu);
  if (lane == 0) stf(C + (size_t)p * ldc + n, UP ? (gated ? gated_apply(acc, accu, act, p0, p1) : act_apply(acc, act)) : acc * wt[p]);
}

// dst[place] = src[perm[place] / top] for every place of the plan, zeros in the padding: the experts' inputs, expert by expert
template <typename T>
__global__ void moe_gather_kernel(const T* __restrict__ src, const int* __restrict__ perm, T* __restrict__ dst, int places, int W, int top) {
  const size_t n = (size_t)places * W;
  for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (size_t)gridDim.x * blockDim.x) {
    const size_t r = e / W;
    const int c = (int)(e - r * W);
    const int p = perm[r];
    dst[e] = p < 0 ? T(0.f) : src[(size_t)(p / top) * W + c];
  }
}

// y[m][c] = sum_t f(m * top + t)[c] (in the order of t) + shared[m][c];  f(pair) = ypair[pair], or, with a plan,
// wt[pair] * ypair[pos_of[pair]] (the experts' outputs still in the plan's order and not yet weighted).  A pair whose expert
// idx[pair] >= n_real is an identity expert: f(pair) = wt[pair] * h[m], and ypair is not read for it.
template <typename TY, typename TS>
__global__ void moe_combine_kernel(const TY* __restrict__ ypair, const int* __restrict__ pos_of, const float* __restrict__ wt,
                                   const TS* __restrict__ shared, float* __restrict__ y, int M, int W, int top, const int* __restrict__ idx,
                                   int n_real, const TS* __restrict__ h) {
  const size_t n = (size_t)M * W;
  for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (size_t)gridDim.x * blockDim.x) {
    const size_t m = e / W;
    const int c = (int)(e - m * W);
    float s = 0.f;
    for (int t = 0; t < top; ++t) {
      const size_t pair = m * top + t;
      if (idx && idx[pair] >= n_real) s = fmaf(wt[pair], ldf(h + e), s);
      else if (pos_of) s = fmaf(wt[pair], ldf(ypair + (size_t)pos_of[pair] * W + c), s);
      else s += ldf(ypair + pair * W + c);
    }
    if (shared) s += ldf(shared + e);
    y[e] = s;
  }
}

unsigned capped_blocks(size_t n) {
  size_t blocks = (n + 255) / 256;
  const size_t cap = (size_t)lia_sm_count() * 16;
  return (unsigned)(blocks > cap ? cap : (blocks ? blocks : 1));
}

}  // namespace

extern "C" int lia_embed_rows(const int64_t* ids, const void* table, int table_f32, float* x, float* x_copy, int rows, int W, int vocab,
                              lia_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  LIA_CHECK_ARG(ids && table && x && rows > 0 && W > 0 && vocab > 0, "lia_embed_rows: bad arguments");
  if (table_f32) embed_rows_kernel<float><<<rows, 256, 0, stream>>>(ids, reinterpret_cast<const float*>(table), x, x_copy, W, vocab);
  else embed_rows_kernel<bf16><<<rows, 256, 0, stream>>>(ids, reinterpret_cast<const bf16*>(table), x, x_copy, W, vocab);
  LIA_LAUNCH_CHECK();
  return LIA_OK;
}

extern "C" int lia_ln_add_norm(float* x, const void* y, int y_f32, const float* w_post, const float* b_post, float mult, const float* extra,
                               const float* w_pre, const float* b_pre, void* h, int h_f32, int rows, int W, float eps, lia_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  LIA_CHECK_ARG(x && (y || h || extra), "lia_ln_add_norm: nothing to do");
  LIA_CHECK_ARG(!y || (w_post && b_post), "lia_ln_add_norm: the norm after the sublayer needs a weight and a bias");
  LIA_CHECK_ARG(!h || (w_pre && b_pre), "lia_ln_add_norm: the norm before the sublayer needs a weight and a bias");
  LIA_CHECK_ARG(rows > 0 && W > 0 && (size_t)W * 4 <= 160 * 1024, "lia_ln_add_norm: bad shape rows=%d W=%d", rows, W);
  const size_t smem = (size_t)W * sizeof(float);
#define LIA_LAN(TY, TH)                                                                                                     \
  do {                                                                                                                      \
    if (smem > 48 * 1024) LIA_CUDA(cudaFuncSetAttribute(ln_add_norm_kernel<TY, TH>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
    ln_add_norm_kernel<TY, TH><<<rows, 256, smem, stream>>>(x, reinterpret_cast<const TY*>(y), w_post, b_post, mult, extra, w_pre, b_pre, \
                                                            reinterpret_cast<TH*>(h), W, eps);                              \
  } while (0)
  if (y_f32 && h_f32) LIA_LAN(float, float);
  else if (y_f32) LIA_LAN(float, bf16);
  else if (h_f32) LIA_LAN(bf16, float);
  else LIA_LAN(bf16, bf16);
#undef LIA_LAN
  LIA_LAUNCH_CHECK();
  return LIA_OK;
}

extern "C" int lia_ln_gather(const float* x, const int* rows, const float* w, const float* b, void* h, int h_f32, int n, int W, float eps,
                             lia_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  LIA_CHECK_ARG(x && rows && w && b && h && n > 0 && W > 0 && (size_t)W * 4 <= 160 * 1024, "lia_ln_gather: bad arguments");
  const size_t smem = (size_t)W * sizeof(float);
  if (h_f32) {
    if (smem > 48 * 1024) LIA_CUDA(cudaFuncSetAttribute(ln_gather_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    ln_gather_kernel<float><<<n, 256, smem, stream>>>(x, rows, w, b, reinterpret_cast<float*>(h), W, eps);
  } else {
    if (smem > 48 * 1024) LIA_CUDA(cudaFuncSetAttribute(ln_gather_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    ln_gather_kernel<bf16><<<n, 256, smem, stream>>>(x, rows, w, b, reinterpret_cast<bf16*>(h), W, eps);
  }
  LIA_LAUNCH_CHECK();
  return LIA_OK;
}

extern "C" int lia_gated_act(const void* in, int ld, int up_off, void* out, int act_f32, int M, int F, int act, lia_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  LIA_CHECK_ARG(in && out && M > 0 && F > 0 && ld >= F && (up_off < 0 || (up_off >= F && ld >= up_off + F)), "lia_gated_act: bad arguments");
  LIA_CHECK_ARG(act >= LIA_ACT_NONE && act <= LIA_ACT_GELU_TANH, "lia_gated_act: unknown activation %d", act);
  const unsigned blocks = capped_blocks((size_t)M * F);
  if (act_f32) gated_act_kernel<float><<<blocks, 256, 0, stream>>>(reinterpret_cast<const float*>(in), ld, up_off, reinterpret_cast<float*>(out), M, F, act);
  else gated_act_kernel<bf16><<<blocks, 256, 0, stream>>>(reinterpret_cast<const bf16*>(in), ld, up_off, reinterpret_cast<bf16*>(out), M, F, act);
  LIA_LAUNCH_CHECK();
  return LIA_OK;
}

extern "C" int lia_router_topk(const float* logits, int* idx, float* wt, int M, int E, int top, lia_stream_t stream_) {
  return lia_router_topk_ext(logits, nullptr, 1, idx, wt, M, E, top, stream_);
}

extern "C" int lia_router_topk_ext(const float* logits, const float* correction, int renorm, int* idx, float* wt, int M, int E, int top,
                                   lia_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  LIA_CHECK_ARG(logits && idx && wt && M > 0 && E > 0 && top > 0 && top <= E && E <= 2048, "lia_router_topk: bad arguments (E=%d top=%d)", E, top);
  router_topk_kernel<<<(M + 3) / 4, 128, (size_t)8 * E * sizeof(float), stream>>>(logits, correction, idx, wt, M, E, top, renorm);
  LIA_LAUNCH_CHECK();
  return LIA_OK;
}

extern "C" int lia_moe_tile_rows(void) { return TM; }

extern "C" int lia_moe_plan(const int* idx, int pairs, int E, int n_tiles, int* perm, int* tile_expert, int* pos_of, lia_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  LIA_CHECK_ARG(idx && perm && tile_expert && pos_of && pairs > 0 && E > 0 && E <= 4096, "lia_moe_plan: bad arguments");
  LIA_CHECK_ARG(n_tiles >= (int)(((long long)pairs + (long long)(E < pairs ? E : pairs) * (TM - 1)) / TM),
                "lia_moe_plan: %d tiles cannot hold %d pairs of %d experts", n_tiles, pairs, E);
  moe_plan_kernel<<<1, 1024, (size_t)2 * E * sizeof(int), stream>>>(idx, pairs, E, n_tiles, perm, tile_expert, pos_of);
  LIA_LAUNCH_CHECK();
  return LIA_OK;
}

// up != 0: C = act(A[token] @ W[e].T) into the experts' intermediate rows; up == 0: C[pair] = wt[pair] * A[row] @ W[e].T (fp32).
// perm == NULL: the few-rows form (rows are the pairs themselves, `idx` gives each pair's expert).
extern "C" int lia_moe_gemm(const void* A, int a_f32, int lda, const void* W, int w_f32, long long w_expert_stride, void* C, int c_f32, int ldc,
                            const int* perm, const int* tile_expert, int n_tiles, const int* idx, const float* wt, int pairs, int top, int N,
                            int K, int up, int act, lia_stream_t stream_) {
  return lia_moe_gemm_ext(A, a_f32, lda, W, w_f32, w_expert_stride, C, c_f32, ldc, perm, tile_expert, n_tiles, idx, wt, pairs, top, N, K, up, act, 0,
                          0x7fffffff, stream_);
}

extern "C" int lia_moe_gemm_ext(const void* A, int a_f32, int lda, const void* W, int w_f32, long long w_expert_stride, void* C, int c_f32, int ldc,
                                const int* perm, const int* tile_expert, int n_tiles, const int* idx, const float* wt, int pairs, int top, int N,
                                int K, int up, int act, int gated, int n_real, lia_stream_t stream_) {
  return lia_moe_gemm_act(A, a_f32, lda, W, w_f32, w_expert_stride, C, c_f32, ldc, perm, tile_expert, n_tiles, idx, wt, pairs, top, N, K, up, act, gated,
                          n_real, 0.f, 0.f, stream_);
}

// act_p0, act_p1: the activation's parameters (LIA_ACT_CLAMPED_SWISH: limit, alpha; it needs the gated form)
extern "C" int lia_moe_gemm_act(const void* A, int a_f32, int lda, const void* W, int w_f32, long long w_expert_stride, void* C, int c_f32, int ldc,
                                const int* perm, const int* tile_expert, int n_tiles, const int* idx, const float* wt, int pairs, int top, int N,
                                int K, int up, int act, int gated, int n_real, float p0, float p1, lia_stream_t stream_) {
  LIA_CHECK_ARG(act != LIA_ACT_CLAMPED_SWISH || (gated && p0 > 0.f), "lia_moe_gemm: the clamped activation needs the gated form and a positive limit");
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  LIA_CHECK_ARG(A && W && C && idx && wt && pairs > 0 && top > 0 && N > 0 && K > 0 && lda >= K && ldc >= N, "lia_moe_gemm: bad arguments");
  LIA_CHECK_ARG(!gated || up, "lia_moe_gemm: only the up projection can be gated");
  LIA_CHECK_ARG(a_f32 == w_f32, "lia_moe_gemm: activations and weights must have one type");
  LIA_CHECK_ARG(up ? c_f32 == a_f32 : c_f32 == 1, "lia_moe_gemm: the up projection writes the activations' type, the down projection fp32");
  if (perm == nullptr) {
    LIA_CHECK_ARG(pairs <= 65535, "lia_moe_gemm: too many pairs for the few-rows form");
    dim3 grid((N + 3) / 4, pairs);
    if (a_f32) {
      if (up) moe_fewrows_kernel<float, float, float, true><<<grid, 128, 0, stream>>>((const float*)A, lda, (const float*)W, w_expert_stride, (float*)C, ldc, idx, wt, top, N, K, act, gated, n_real, p0, p1);
      else moe_fewrows_kernel<float, float, float, false><<<grid, 128, 0, stream>>>((const float*)A, lda, (const float*)W, w_expert_stride, (float*)C, ldc, idx, wt, top, N, K, act, gated, n_real, p0, p1);
    } else {
      if (up) moe_fewrows_kernel<bf16, bf16, bf16, true><<<grid, 128, 0, stream>>>((const bf16*)A, lda, (const bf16*)W, w_expert_stride, (bf16*)C, ldc, idx, wt, top, N, K, act, gated, n_real, p0, p1);
      else moe_fewrows_kernel<bf16, bf16, float, false><<<grid, 128, 0, stream>>>((const bf16*)A, lda, (const bf16*)W, w_expert_stride, (float*)C, ldc, idx, wt, top, N, K, act, gated, n_real, p0, p1);
    }
    LIA_LAUNCH_CHECK();
    return LIA_OK;
  }
  LIA_CHECK_ARG(tile_expert && n_tiles > 0 && n_tiles <= 65535, "lia_moe_gemm: bad tile plan");
  dim3 grid((N + 63) / 64, n_tiles);
#define LIA_MG(TA, TC, UP_, GATED_) moe_gemm_kernel<TA, TA, TC, UP_, GATED_><<<grid, 256, 0, stream>>>((const TA*)A, lda, (const TA*)W, w_expert_stride, (TC*)C, ldc, perm, tile_expert, wt, top, N, K, act, n_real, p0, p1)
  if (a_f32) {
    if (up && gated) LIA_MG(float, float, true, true);
    else if (up) LIA_MG(float, float, true, false);
    else LIA_MG(float, float, false, false);
  } else {
    if (up && gated) LIA_MG(bf16, bf16, true, true);
    else if (up) LIA_MG(bf16, bf16, true, false);
    else LIA_MG(bf16, float, false, false);
  }
#undef LIA_MG
  LIA_LAUNCH_CHECK();
  return LIA_OK;
}

extern "C" int lia_moe_gather(const void* src, int act_f32, const int* perm, void* dst, int places, int W, int top, lia_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  LIA_CHECK_ARG(src && perm && dst && places > 0 && W > 0 && top > 0, "lia_moe_gather: bad arguments");
  const unsigned blocks = capped_blocks((size_t)places * W);
  if (act_f32) moe_gather_kernel<float><<<blocks, 256, 0, stream>>>(reinterpret_cast<const float*>(src), perm, reinterpret_cast<float*>(dst), places, W, top);
  else moe_gather_kernel<bf16><<<blocks, 256, 0, stream>>>(reinterpret_cast<const bf16*>(src), perm, reinterpret_cast<bf16*>(dst), places, W, top);
  LIA_LAUNCH_CHECK();
  return LIA_OK;
}

// The tensor-core form: every expert's contiguous rows of the gathered input through lia_gemm_bf16, one launch per expert that has
// rows, issued from here so that the launches follow each other without a trip through the caller's interpreter.
extern "C" int lia_moe_expert_gemms(const void* A, const void* W, long long w_expert_stride, void* C, const int* tiles_per_expert, int E,
                                    int tile_rows, int N, int K, void* workspace, size_t workspace_bytes, lia_stream_t stream_) {
  LIA_CHECK_ARG(A && W && C && tiles_per_expert && E > 0 && tile_rows > 0 && N > 0 && K > 0, "lia_moe_expert_gemms: bad arguments");
  const bf16* a = reinterpret_cast<const bf16*>(A);
  const bf16* w = reinterpret_cast<const bf16*>(W);
  bf16* c = reinterpret_cast<bf16*>(C);
  size_t at = 0;
  for (int e = 0; e < E; ++e) {
    const int rows = tiles_per_expert[e] * tile_rows;
    if (rows <= 0) continue;
    const int rc = lia_gemm_bf16(a + at * K, w + (size_t)e * w_expert_stride, nullptr, nullptr, c + at * N, rows, N, K, LIA_EPI_BIAS, nullptr,
                                 workspace, workspace_bytes, stream_);
    if (rc != LIA_OK) return rc;
    at += rows;
  }
  return LIA_OK;
}

extern "C" int lia_moe_combine(const void* ypair, int ypair_f32, const int* pos_of, const float* wt, const void* shared, int shared_f32, float* y,
                               int M, int W, int top, lia_stream_t stream_) {
  return lia_moe_combine_ext(ypair, ypair_f32, pos_of, wt, shared, shared_f32, nullptr, 0, nullptr, y, M, W, top, stream_);
}

extern "C" int lia_moe_combine_ext(const void* ypair, int ypair_f32, const int* pos_of, const float* wt, const void* shared, int act_f32,
                                   const int* idx, int n_real, const void* h, float* y, int M, int W, int top, lia_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  LIA_CHECK_ARG(ypair && y && M > 0 && W > 0 && top > 0 && (!pos_of || wt), "lia_moe_combine: bad arguments");
  LIA_CHECK_ARG(!idx || (h && wt && n_real >= 0), "lia_moe_combine: identity experts need the routing weights and the experts' input");
  const unsigned blocks = capped_blocks((size_t)M * W);
#define LIA_MC(TY, TS) moe_combine_kernel<TY, TS><<<blocks, 256, 0, stream>>>(reinterpret_cast<const TY*>(ypair), pos_of, wt, reinterpret_cast<const TS*>(shared), y, M, W, top, idx, n_real, reinterpret_cast<const TS*>(h))
  if (ypair_f32 && act_f32) LIA_MC(float, float);
  else if (ypair_f32) LIA_MC(float, bf16);
  else if (act_f32) LIA_MC(bf16, float);
  else LIA_MC(bf16, bf16);
#undef LIA_MC
  LIA_LAUNCH_CHECK();
  return LIA_OK;
}
