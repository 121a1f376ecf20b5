// Row operations of models that keep their residual stream in 32-bit floats: RMS norms with a scalar or a per-channel
// weight (fused with the residual add that follows a sublayer and with the norm that precedes the next one), the token
// embedding with its norm, the gated, normed residual update with a weighted mix of all earlier layers' results, the
// polynomial activation between norms, a gated feed-forward activation with clamps, a projection onto a handful of outputs with the
// gate non-linearities in its epilogue, a plain strided-batched projection on the CUDA cores (true 32-bit products and
// sums: the exact path, and the carrier of shapes the tensor-core GEMM does not take), and a 32-bit argmax.
//
// Activations are bf16 or fp32 (`act_f32`); everything a norm, a gate or the residual sum computes is fp32 either way.
#include <math.h>

#include "common.cuh"

namespace {

template <typename T> __device__ __forceinline__ float ldf(const T* p);
template <> __device__ __forceinline__ float ldf<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ldf<bf16>(const bf16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void stf(T* p, float v);
template <> __device__ __forceinline__ void stf<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void stf<bf16>(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

// sum over a block of NT threads; every thread gets the result.  `red` holds NT/32 floats.
template <int NT>
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  __syncthreads();                       // `red` may still be read from the previous call
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float s = 0.f;
#pragma unroll
  for (int w = 0; w < NT / 32; ++w) s += red[w];
  return s;
}

// x[row] = w * e / sqrt(mean(e^2) + eps), e = table[ids[row]]
template <typename T>
__global__ void __launch_bounds__(256) embed_rmsnorm_kernel(const int64_t* __restrict__ ids, const T* __restrict__ table,
                                                            const float* __restrict__ w, int w_n, float* __restrict__ x, int W,
                                                            int vocab, float eps) {
  __shared__ float red[8];
  const int row = blockIdx.x;
  long long id = ids[row];
  if (id < 0 || id >= vocab) id = 0;     // the host checks the range; never read outside the table
  const T* e = table + (size_t)id * W;
  float ss = 0.f;
  for (int i = threadIdx.x; i < W; i += 256) {
    const float v = ldf(e + i);
    ss += v * v;
  }
  ss = block_sum<256>(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)W + eps);
  for (int i = threadIdx.x; i < W; i += 256) x[(size_t)row * W + i] = ldf(e + i) * inv * w[w_n == 1 ? 0 : i];
}

// if y:  x[row] += w_post * y / sqrt(mean(y^2) + eps)          (the norm after a sublayer, then the residual sum)
// if h:  h[row]  = w_pre  * x / sqrt(mean(x^2) + eps)          (the norm before the next sublayer)
// `xs` (dynamic shared memory, W floats) keeps the updated row between the two.
template <typename TY, typename TH>
__global__ void __launch_bounds__(256) rms_add_norm_kernel(float* __restrict__ x, const TY* __restrict__ y, const float* __restrict__ w_post,
                                                           int w_post_n, const float* __restrict__ w_pre, int w_pre_n, TH* __restrict__ h,
                                                           int W, float eps) {
  extern __shared__ float xs[];
  __shared__ float red[8];
  const size_t base = (size_t)blockIdx.x * W;
  if (y != nullptr) {
    float ss = 0.f;
    for (int i = threadIdx.x; i < W; i += 256) {
      const float v = ldf(y + base + i);
      ss += v * v;
    }
    ss = block_sum<256>(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)W + eps);
    for (int i = threadIdx.x; i < W; i += 256) {
      const float v = x[base + i] + ldf(y + base + i) * inv * w_post[w_post_n == 1 ? 0 : i];
      x[base + i] = v;
      xs[i] = v;
    }
  } else {
    for (int i = threadIdx.x; i < W; i += 256) xs[i] = x[base + i];
  }
  if (h == nullptr) return;
  float ss = 0.f;
  for (int i = threadIdx.x; i < W; i += 256) ss += xs[i] * xs[i];      // each thread re-reads only what it wrote
  ss = block_sum<256>(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)W + eps);
  for (int i = threadIdx.x; i < W; i += 256) stf(h + base + i, xs[i] * inv * w_pre[w_pre_n == 1 ? 0 : i]);
}

// Pre-norm designs with learned positions and a per-channel norm weight:
//   x[row] = table[ids[row]] * scale + pos_table[position of the row]          (fp32)
//   cat (may be null): the row in the activations' type, twice side by side -- the pair [x ; x0] that a looped block's
//   input projection reads (x0 stays the embedding, the left half is overwritten as the stream moves on).
template <typename T, typename TC>
__global__ void __launch_bounds__(256) embed_scale_pos_kernel(const int64_t* __restrict__ ids, const T* __restrict__ table, float scale,
                                                              const T* __restrict__ pos_table, const int* __restrict__ meta, float* __restrict__ x,
                                                              TC* __restrict__ cat, int W, int vocab, int max_pos) {
  const int row = blockIdx.x;
  long long id = ids[row];
  if (id < 0 || id >= vocab) id = 0;     // the host checks the range; never read outside the table
  int p = meta[2 * row + 1];
  p = p < 0 ? 0 : (p >= max_pos ? max_pos - 1 : p);      // the host refuses sequences longer than the table
  const T* e = table + (size_t)id * W;
  const T* pr = pos_table ? pos_table + (size_t)p * W : nullptr;
  for (int i = threadIdx.x; i < W; i += 256) {
    const float v = fmaf(ldf(e + i), scale, pr ? ldf(pr + i) : 0.f);
    x[(size_t)row * W + i] = v;
    if (cat != nullptr) {
      stf(cat + (size_t)row * 2 * W + i, v);
      stf(cat + (size_t)row * 2 * W + W + i, v);
    }
  }
}

// The residual update of pre-norm designs, fused with the norm (or the plain cast) that the next sublayer reads:
//   x[row] = (replace ? 0 : x[row]) + y[row] + bias          (y, bias may be null; bias is one vector for all rows)
//   h[row] = w * x / sqrt(mean(x^2) + eps)                   (w null: h = x), h in the activations' type with row stride ldh
// `xs` (dynamic shared memory, W floats) keeps the updated row between the two.
template <typename TY, typename TH>
__global__ void __launch_bounds__(256) residual_norm_kernel(float* __restrict__ x, const TY* __restrict__ y, int replace, const float* __restrict__ bias,
                                                            const float* __restrict__ w, TH* __restrict__ h, long long ldh, int W, float eps) {
  extern __shared__ float xs[];
  __shared__ float red[8];
  const size_t base = (size_t)blockIdx.x * W;
  float ss = 0.f;
  for (int i = threadIdx.x; i < W; i += 256) {
    float v = replace ? 0.f : x[base + i];
    if (y != nullptr) v += ldf(y + base + i);
    if (bias != nullptr) v += bias[i];
    if (y != nullptr || bias != nullptr || replace) x[base + i] = v;
    xs[i] = v;
    ss += v * v;
  }
  if (h == nullptr) return;
  float inv = 1.0f;
  if (w != nullptr) {
    ss = block_sum<256>(ss, red);
    inv = 1.0f / sqrtf(ss / (float)W + eps);
  }
  for (int i = threadIdx.x; i < W; i += 256) stf(h + (size_t)blockIdx.x * ldh + i, w ? xs[i] * inv * w[i] : xs[i]);
}

// out[m] = w * z / sqrt(mean(z^2) + eps) over z = in[m][0..N) (a column slice with row stride ld); one warp per row
template <typename TI, typename TO>
__global__ void __launch_bounds__(128) rms_norm_rows_kernel(const TI* __restrict__ in, long long ld, const float* __restrict__ w, TO* __restrict__ out,
                                                            int M, int N, float eps) {
  const int row = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= M) return;
  const TI* z = in + (size_t)row * ld;
  float ss = 0.f;
  for (int i = lane; i < N; i += 32) {
    const float v = ldf(z + i);
    ss += v * v;
  }
  const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)N + eps);
  for (int i = lane; i < N; i += 32) stf(out + (size_t)row * N + i, ldf(z + i) * inv * w[i]);
}

// out = a * sigmoid(g), element by element over [M][F]; a and g are row-major views with their own row strides
template <typename TA, typename TG, typename TO>
__global__ void sigmoid_mul_kernel(const TA* __restrict__ a, long long lda, const TG* __restrict__ g, long long ldg, TO* __restrict__ out, int M, int F) {
  const size_t n = (size_t)M * F;
  for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (size_t)gridDim.x * blockDim.x) {
    const size_t m = e / F;
    const int f = (int)(e - m * F);
    stf(out + e, ldf(a + m * lda + f) / (1.0f + expf(-ldf(g + m * ldg + f))));
  }
}

// x = cap * tanh(x / cap) in place
__global__ void softcap_kernel(float* __restrict__ x, size_t n, float cap) {
  for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (size_t)gridDim.x * blockDim.x) x[e] = cap * tanhf(x[e] / cap);
}

// The residual update of designs that norm a sublayer's OUTPUT and gate it first, and that hand on a weighted mix of all
// earlier layers' results instead of the last one:
//   g     = y * sigmoid(r + rb)                       (r null: g = y; y null: nothing is added)
//   x_new = x + w * g / sqrt(mean(g^2) + eps)
//   stack null:  x = x_new
//   else:        stack[n_mix - 1][row] = x_new;  x = sum_{j < n_mix} mix[j] * stack[j][row]
//   h null or    h = x in the activations' type
// Block per row; `gs` (dynamic shared memory, W floats) keeps g between the two passes.
template <typename TY, typename TH>
__global__ void __launch_bounds__(256) gated_rms_add_kernel(float* __restrict__ x, const TY* __restrict__ y, const TH* __restrict__ r, int ldr,
                                                            const float* __restrict__ rb, const float* __restrict__ w, float* __restrict__ stack,
                                                            long long stack_stride, int n_mix, const float* __restrict__ mix, TH* __restrict__ h,
                                                            int W, float eps) {
  extern __shared__ float gs[];
  __shared__ float red[8];
  const size_t row = blockIdx.x, base = row * W;
  float inv = 0.f;
  if (y != nullptr) {
    float ss = 0.f;
    for (int i = threadIdx.x; i < W; i += 256) {
      float g = ldf(y + base + i);
      if (r != nullptr) g *= 1.0f / (1.0f + expf(-(ldf(r + row * ldr + i) + (rb ? rb[i] : 0.f))));
      gs[i] = g;
      ss += g * g;
    }
    ss = block_sum<256>(ss, red);
    inv = 1.0f / sqrtf(ss / (float)W + eps);
  }
  for (int i = threadIdx.x; i < W; i += 256) {
    float v = x[base + i];
    if (y != nullptr) v += gs[i] * inv * w[i];
    if (stack != nullptr) {
      stack[(size_t)(n_mix - 1) * stack_stride + base + i] = v;
      float s = 0.f;
      for (int j = 0; j < n_mix - 1; ++j) s = fmaf(mix[j], stack[(size_t)j * stack_stride + base + i], s);
      v = fmaf(mix[n_mix - 1], v, s);
    }
    if (y != nullptr || stack != nullptr) x[base + i] = v;
    if (h != nullptr) stf(h + base + i, v);
  }
}

// out = k1 R(z) + k2 R(z*z) + k3 R(z*z*z) + k0, products element by element, R(u) = u / sqrt(mean(u^2) + eps) over the row
// of F numbers; coef = {k1, k2, k3, k0} on the device.  Block per row: one pass for the three sums of squares, one for the output.
template <typename T>
__global__ void __launch_bounds__(256) poly_norm_kernel(const T* __restrict__ in, int ld, const float* __restrict__ coef, T* __restrict__ out, int F,
                                                        float eps) {
  __shared__ float red[8];
  const T* z = in + (size_t)blockIdx.x * ld;
  float s1 = 0.f, s2 = 0.f, s3 = 0.f;
  for (int i = threadIdx.x; i < F; i += 256) {
    const float v = ldf(z + i), v2 = v * v;
    s1 += v2;
    s2 += v2 * v2;
    s3 += v2 * v2 * v2;
  }
  s1 = block_sum<256>(s1, red);
  s2 = block_sum<256>(s2, red);
  s3 = block_sum<256>(s3, red);
  const float a = coef[0] / sqrtf(s1 / (float)F + eps), b = coef[1] / sqrtf(s2 / (float)F + eps), c = coef[2] / sqrtf(s3 / (float)F + eps);
  const float e = coef[3];
  for (int i = threadIdx.x; i < F; i += 256) {
    const float v = ldf(z + i);
    stf(out + (size_t)blockIdx.x * F + i, fmaf(v, fmaf(v, fmaf(v, c, b), a), e));
  }
}

// h[r] = w * x[rows[r]] / sqrt(mean^2 + eps): the norm of a few selected rows (the positions whose logits are asked for)
template <typename TH>
__global__ void __launch_bounds__(256) rms_gather_kernel(const float* __restrict__ x, const int* __restrict__ rows, const float* __restrict__ w,
                                                         int w_n, TH* __restrict__ h, int W, float eps) {
  __shared__ float red[8];
  const size_t src = (size_t)rows[blockIdx.x] * W, dst = (size_t)blockIdx.x * W;
  float ss = 0.f;
  for (int i = threadIdx.x; i < W; i += 256) ss += x[src + i] * x[src + i];
  ss = block_sum<256>(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)W + eps);
  for (int i = threadIdx.x; i < W; i += 256) stf(h + dst + i, x[src + i] * inv * w[w_n == 1 ? 0 : i]);
}

// out = g * sigmoid(alpha * g) * (u + 1),  g = min(gate, limit), u = clamp(up, -limit, limit); gate | up are the two
// column ranges of one projection's output row (row stride ld; up starts at column up_off)
template <typename T>
__global__ void clamped_glu_kernel(const T* __restrict__ gu, int ld, int up_off, T* __restrict__ out, int M, int F, float limit, float alpha) {
  const size_t n = (size_t)M * F;
  for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (size_t)gridDim.x * blockDim.x) {
    const size_t m = e / F;
    const int f = (int)(e - m * F);
    const float g = fminf(ldf(gu + m * ld + f), limit);
    const float u = fminf(fmaxf(ldf(gu + m * ld + up_off + f), -limit), limit);
    stf(out + e, g * (1.0f / (1.0f + expf(-alpha * g))) * (u + 1.0f));
  }
}

__device__ __forceinline__ float log_sigmoid(float z) { return fminf(z, 0.f) - log1pf(expf(-fabsf(z))); }

// 8 consecutive numbers of a row as floats; `vec` says that the 16-byte (bf16) / 32-byte (fp32) vector load is legal here
template <typename T> __device__ __forceinline__ void load8(const T* p, int k, int K, bool vec, float* f);
template <> __device__ __forceinline__ void load8<bf16>(const bf16* p, int k, int K, bool vec, float* f) {
  if (vec && k + 8 <= K) {
    unpack8(*reinterpret_cast<const uint4*>(p + k), f);
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = k + j < K ? __bfloat162float(p[k + j]) : 0.f;
  }
}
template <> __device__ __forceinline__ void load8<float>(const float* p, int k, int K, bool vec, float* f) {
  if (vec && k + 8 <= K) {
    const float4 lo = *reinterpret_cast<const float4*>(p + k), hi = *reinterpret_cast<const float4*>(p + k + 4);
    f[0] = lo.x; f[1] = lo.y; f[2] = lo.z; f[3] = lo.w; f[4] = hi.x; f[5] = hi.y; f[6] = hi.z; f[7] = hi.w;
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = k + j < K ? p[k + j] : 0.f;
  }
}
template <typename T> __device__ __forceinline__ bool vec_ok(const T* p, long long ld) {
  return (reinterpret_cast<uintptr_t>(p) % 16 == 0) && (ld * (long long)sizeof(T)) % 16 == 0;
}

// out[m][n] = act(sum_k a[m][k] w[n][k] + bias[n]) for a handful of outputs (gates: one per head), fp32 out.
// mode 0: identity; 1: n < N/2 -> cap*tanh(z/cap), n >= N/2 -> logsigmoid(cap*tanh(z/cap)); 2: sigmoid.
// One block of 4 warps per row: the warps split k (8 numbers per lane and sweep, 128-bit loads), 8 outputs per sweep,
// partial sums meet in shared memory in a fixed order.
template <typename TA, typename TW>
__global__ void __launch_bounds__(128) linear_small_kernel(const TA* __restrict__ a, int lda, const TW* __restrict__ w, const float* __restrict__ bias,
                                                           float* __restrict__ out, int M, int N, int K, int mode, float cap) {
  __shared__ float part[4][8];
  const int row = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const TA* ar = a + (size_t)row * lda;
  const bool va = vec_ok(a, lda), vw = vec_ok(w, K);
  for (int n0 = 0; n0 < N; n0 += 8) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int k = threadIdx.x * 8; k < K; k += 128 * 8) {
      float av[8], wv[8];
      load8(ar, k, K, va, av);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (n0 + j < N) {
          load8(w + (size_t)(n0 + j) * K, k, K, vw, wv);
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[j] = fmaf(av[i], wv[i], acc[j]);
        }
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = warp_sum(acc[j]);
    __syncthreads();
    if (lane == 0) {
#pragma unroll
      for (int j = 0; j < 8; ++j) part[warp][j] = acc[j];
    }
    __syncthreads();
    const int n = n0 + threadIdx.x;
    if (threadIdx.x < 8 && n < N) {
      float z = ((part[0][threadIdx.x] + part[1][threadIdx.x]) + (part[2][threadIdx.x] + part[3][threadIdx.x])) + (bias ? bias[n] : 0.f);
      if (mode == 1) {
        z = cap * tanhf(z / cap);
        if (n >= N / 2) z = log_sigmoid(z);
      } else if (mode == 2) {
        z = 1.0f / (1.0f + expf(-z));
      }
      out[(size_t)row * N + n] = z;
    }
  }
}

// The same projection for FEW rows (M <= 64: decoded tokens, the rows whose logits are wanted): one warp per output n reads
// its weight row with 128-bit loads and serves the rows eight at a time (the row is re-read from L1 for the next eight);
// memory-bound on the weights.
template <typename TA, typename TW, typename TC>
__global__ void __launch_bounds__(128) linear_fewrows_kernel(const TA* __restrict__ A, long long lda, long long sA, const TW* __restrict__ Wt,
                                                             long long ldw, long long sW, TC* __restrict__ C, long long ldc, long long sC, int M,
                                                             int N, int K, float scale) {
  const int b = blockIdx.y;
  A += (size_t)b * sA;
  Wt += (size_t)b * sW;
  C += (size_t)b * sC;
  const int n = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (n >= N) return;
  const TW* wr = Wt + (size_t)n * ldw;
  const bool va = vec_ok(A, lda) && (sA * (long long)sizeof(TA)) % 16 == 0, vw = vec_ok(Wt, ldw) && (sW * (long long)sizeof(TW)) % 16 == 0;
  for (int m0 = 0; m0 < M; m0 += 8) {
    float acc[8];
#pragma unroll
    for (int m = 0; m < 8; ++m) acc[m] = 0.f;
    for (int k = lane * 8; k < K; k += 32 * 8) {
      float wv[8], av[8];
      load8(wr, k, K, vw, wv);
#pragma unroll
      for (int m = 0; m < 8; ++m) {
        if (m0 + m < M) {
          load8(A + (size_t)(m0 + m) * lda, k, K, va, av);
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[m] = fmaf(av[i], wv[i], acc[m]);
        }
      }
    }
#pragma unroll
    for (int m = 0; m < 8; ++m) {
      const float sum = warp_sum(acc[m]);
      if (lane == 0 && m0 + m < M) stf(C + (size_t)(m0 + m) * ldc + n, sum * scale);
    }
  }
}

// C[b][m][n] = scale * sum_k A[b][m][k] * W[b][n][k]; 64 x 64 tile per block, 16-wide k slabs, 4 x 4 outputs per thread,
// fp32 products and sums in k order.
template <typename TA, typename TW, typename TC>
__global__ void __launch_bounds__(256) linear_plain_kernel(const TA* __restrict__ A, long long lda, long long sA, const TW* __restrict__ Wt,
                                                           long long ldw, long long sW, TC* __restrict__ C, long long ldc, long long sC, int M,
                                                           int N, int K, float scale) {
  __shared__ float As[16][64 + 4];
  __shared__ float Ws[16][64 + 4];
  const int b = blockIdx.z;
  A += (size_t)b * sA;
  Wt += (size_t)b * sW;
  C += (size_t)b * sC;
  const int m0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  for (int k0 = 0; k0 < K; k0 += 16) {
    for (int e = threadIdx.x; e < 64 * 16; e += 256) {
      const int r = e >> 4, kk = e & 15;
      const int k = k0 + kk;
      As[kk][r] = (m0 + r < M && k < K) ? ldf(A + (size_t)(m0 + r) * lda + k) : 0.f;
      Ws[kk][r] = (n0 + r < N && k < K) ? ldf(Wt + (size_t)(n0 + r) * ldw + k) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < 16; ++kk) {
      float av[4], wv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) av[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) wv[j] = Ws[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int m = m0 + ty * 4 + i, n = n0 + tx * 4 + j;
      if (m < M && n < N) stf(C + (size_t)m * ldc + n, acc[i][j] * scale);
    }
}

__global__ void __launch_bounds__(256) argmax_f32_kernel(const float* __restrict__ logits, int64_t* __restrict__ next, int V, int suppress) {
  __shared__ float sv[8];
  __shared__ int si[8];
  const float* row = logits + (size_t)blockIdx.x * V;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int idx = threadIdx.x; idx < V; idx += 256) {
    const float v = (idx == suppress) ? -INFINITY : row[idx];
    if (v > best || (v == best && idx < bi)) { best = v; bi = idx; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
  }
  if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = best; si[threadIdx.x >> 5] = bi; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 8; ++w)
      if (sv[w] > best || (sv[w] == best && si[w] < bi)) { best = sv[w]; bi = si[w]; }
    next[blockIdx.x] = bi;
  }
}

template <typename TA, typename TW>
int launch_plain(const void* A, long long lda, long long sA, const void* W, long long ldw, long long sW, void* C, long long ldc, long long sC,
                 int M, int N, int K, int batch, float scale, int c_f32, cudaStream_t stream) {
  if (M <= 64) {
    dim3 g2((N + 3) / 4, batch);
    if (c_f32)
      linear_fewrows_kernel<TA, TW, float><<<g2, 128, 0, stream>>>(reinterpret_cast<const TA*>(A), lda, sA, reinterpret_cast<const TW*>(W), ldw, sW,
                                                                   reinterpret_cast<float*>(C), ldc, sC, M, N, K, scale);
    else
      linear_fewrows_kernel<TA, TW, bf16><<<g2, 128, 0, stream>>>(reinterpret_cast<const TA*>(A), lda, sA, reinterpret_cast<const TW*>(W), ldw, sW,
                                                                  reinterpret_cast<bf16*>(C), ldc, sC, M, N, K, scale);
    LIA_LAUNCH_CHECK();
    return LIA_OK;
  }
  dim3 grid((N + 63) / 64, (M + 63) / 64, batch);
  if (c_f32)
    linear_plain_kernel<TA, TW, float><<<grid, 256, 0, stream>>>(reinterpret_cast<const TA*>(A), lda, sA, reinterpret_cast<const TW*>(W), ldw, sW,
                                                                 reinterpret_cast<float*>(C), ldc, sC, M, N, K, scale);
  else
    linear_plain_kernel<TA, TW, bf16><<<grid, 256, 0, stream>>>(reinterpret_cast<const TA*>(A), lda, sA, reinterpret_cast<const TW*>(W), ldw, sW,
                                                                reinterpret_cast<bf16*>(C), ldc, sC, M, N, K, scale);
  LIA_LAUNCH_CHECK();
  return LIA_OK;
}

}  // namespace

extern "C" int lia_embed_rmsnorm(const int64_t* ids, const void* table, int table_f32, const float* w, int w_n, float* x, int rows,
                                 int W, int vocab, float eps, lia_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  LIA_CHECK_ARG(ids && table && w && x, "lia_embed_rmsnorm: null pointer");
  LIA_CHECK_ARG(rows > 0 && W > 0 && vocab > 0 && (w_n == 1 || w_n == W), "lia_embed_rmsnorm: bad shape rows=%d W=%d w_n=%d", rows, W, w_n);
  if (table_f32)
    embed_rmsnorm_kernel<float><<<rows, 256, 0, stream>>>(ids, reinterpret_cast<const float*>(table), w, w_n, x, W, vocab, eps);
  else
    embed_rmsnorm_kernel<bf16><<<rows, 256, 0, stream>>>(ids, reinterpret_cast<const bf16*>(table), w, w_n, x, W, vocab, eps);
  LIA_LAUNCH_CHECK();
  return LIA_OK;
}

extern "C" int lia_rms_add_norm(float* x, const void* y, int y_f32, const float* w_post, int w_post_n, const float* w_pre, int w_pre_n,
                                void* h, int h_f32, int rows, int W, float eps, lia_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  LIA_CHECK_ARG(x && (y || h), "lia_rms_add_norm: nothing to do");
  LIA_CHECK_ARG(!y || (w_post && (w_post_n == 1 || w_post_n == W)), "lia_rms_add_norm: bad weight of the norm after the sublayer");
  LIA_CHECK_ARG(!h || (w_pre && (w_pre_n == 1 || w_pre_n == W)), "lia_rms_add_norm: bad weight of the norm before the sublayer");
  LIA_CHECK_ARG(rows > 0 && W > 0 && (size_t)W * 4 <= 160 * 1024, "lia_rms_add_norm: bad shape rows=%d W=%d", rows, W);
  const size_t smem = (size_t)W * sizeof(float);
#define LIA_RAN(TY, TH)                                                                                                      \
  do {                                                                                                                       \
    if (smem > 48 * 1024) LIA_CUDA(cudaFuncSetAttribute(rms_add_norm_kernel<TY, TH>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
    rms_add_norm_kernel<TY, TH><<<rows, 256, smem, stream>>>(x, reinterpret_cast<const TY*>(y), w_post, w_post_n, w_pre, w_pre_n,        \
                                                             reinterpret_cast<TH*>(h), W, eps);                              \
  } while (0)
  if (y_f32 && h_f32) LIA_RAN(float, float);
  else if (y_f32) LIA_RAN(float, bf16);
  else if (h_f32) LIA_RAN(bf16, float);
  else LIA_RAN(bf16, bf16);
#undef LIA_RAN
  LIA_LAUNCH_CHECK();
  return LIA_OK;
}

extern "C" int lia_gated_rms_add(float* x, const void* y, int y_f32, const void* r, int ldr, const float* rb, const float* w, float* stack,
                                 long long stack_stride, int n_mix, const float* mix, void* h, int act_f32, int rows, int W, float eps,
                                 lia_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  LIA_CHECK_ARG(x && (y || stack || h), "lia_gated_rms_add: nothing to do");
  LIA_CHECK_ARG(!y || w, "lia_gated_rms_add: the norm after the sublayer needs its weight");
  LIA_CHECK_ARG(!r || (y && ldr >= W), "lia_gated_rms_add: a gate needs a sublayer output and a row stride >= W");
  LIA_CHECK_ARG(!stack || (mix && n_mix >= 1 && stack_stride >= (long long)rows * W), "lia_gated_rms_add: bad stack of earlier results");
  LIA_CHECK_ARG(rows > 0 && W > 0 && (size_t)W * 4 <= 160 * 1024, "lia_gated_rms_add: bad shape rows=%d W=%d", rows, W);
  const size_t smem = (size_t)W * sizeof(float);
#define LIA_GRA(TY, TH)                                                                                                      \
  do {                                                                                                                       \
    if (smem > 48 * 1024) LIA_CUDA(cudaFuncSetAttribute(gated_rms_add_kernel<TY, TH>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
    gated_rms_add_kernel<TY, TH><<<rows, 256, smem, stream>>>(x, reinterpret_cast<const TY*>(y), reinterpret_cast<const TH*>(r), ldr, rb, w, stack, \
                                                              stack_stride, n_mix, mix, reinterpret_cast<TH*>(h), W, eps);    \
  } while (0)
  if (y_f32 && act_f32) LIA_GRA(float, float);
  else if (y_f32) LIA_GRA(float, bf16);
  else if (act_f32) LIA_GRA(bf16, float);
  else LIA_GRA(bf16, bf16);
#undef LIA_GRA
  LIA_LAUNCH_CHECK();
  return LIA_OK;
}

extern "C" int lia_poly_norm(const void* in, int ld, const float* coef, void* out, int act_f32, int M, int F, float eps, lia_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  LIA_CHECK_ARG(in && coef && out && M > 0 && F > 0 && ld >= F, "lia_poly_norm: bad arguments");
  if (act_f32) poly_norm_kernel<float><<<M, 256, 0, stream>>>(reinterpret_cast<const float*>(in), ld, coef, reinterpret_cast<float*>(out), F, eps);
  else poly_norm_kernel<bf16><<<M, 256, 0, stream>>>(reinterpret_cast<const bf16*>(in), ld, coef, reinterpret_cast<bf16*>(out), F, eps);
  LIA_LAUNCH_CHECK();
  return LIA_OK;
}

extern "C" int lia_rms_gather(const float* x, const int* rows, const float* w, int w_n, void* h, int h_f32, int n, int W, float eps,
                              lia_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  LIA_CHECK_ARG(x && rows && w && h && n > 0 && W > 0 && (w_n == 1 || w_n == W), "lia_rms_gather: bad arguments");
  if (h_f32) rms_gather_kernel<float><<<n, 256, 0, stream>>>(x, rows, w, w_n, reinterpret_cast<float*>(h), W, eps);
  else rms_gather_kernel<bf16><<<n, 256, 0, stream>>>(x, rows, w, w_n, reinterpret_cast<bf16*>(h), W, eps);
  LIA_LAUNCH_CHECK();
  return LIA_OK;
}

extern "C" int lia_clamped_glu(const void* gate_up, int ld, int up_off, void* out, int act_f32, int M, int F, float limit, float alpha,
                               lia_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  LIA_CHECK_ARG(gate_up && out && M > 0 && F > 0 && up_off >= F && ld >= up_off + F, "lia_clamped_glu: bad arguments");
  const size_t n = (size_t)M * F;
  size_t blocks = (n + 255) / 256;
  const size_t capb = (size_t)lia_sm_count() * 16;
  if (blocks > capb) blocks = capb;
  if (act_f32) clamped_glu_kernel<float><<<(unsigned)blocks, 256, 0, stream>>>(reinterpret_cast<const float*>(gate_up), ld, up_off, reinterpret_cast<float*>(out), M, F, limit, alpha);
  else clamped_glu_kernel<bf16><<<(unsigned)blocks, 256, 0, stream>>>(reinterpret_cast<const bf16*>(gate_up), ld, up_off, reinterpret_cast<bf16*>(out), M, F, limit, alpha);
  LIA_LAUNCH_CHECK();
  return LIA_OK;
}

extern "C" int lia_linear_small(const void* a, int a_f32, int lda, const void* w, int w_f32, const float* bias, float* out, int M, int N,
                                int K, int mode, float cap, lia_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  LIA_CHECK_ARG(a && w && out && M > 0 && N > 0 && K > 0 && lda >= K, "lia_linear_small: bad arguments");
  LIA_CHECK_ARG(mode >= 0 && mode <= 2 && (mode != 1 || (N % 2 == 0 && cap > 0.f)), "lia_linear_small: bad mode %d (N=%d cap=%f)", mode, N, cap);
  const int grid = M;
  if (a_f32 && w_f32) linear_small_kernel<float, float><<<grid, 128, 0, stream>>>(reinterpret_cast<const float*>(a), lda, reinterpret_cast<const float*>(w), bias, out, M, N, K, mode, cap);
  else if (a_f32) linear_small_kernel<float, bf16><<<grid, 128, 0, stream>>>(reinterpret_cast<const float*>(a), lda, reinterpret_cast<const bf16*>(w), bias, out, M, N, K, mode, cap);
  else if (w_f32) linear_small_kernel<bf16, float><<<grid, 128, 0, stream>>>(reinterpret_cast<const bf16*>(a), lda, reinterpret_cast<const float*>(w), bias, out, M, N, K, mode, cap);
  else linear_small_kernel<bf16, bf16><<<grid, 128, 0, stream>>>(reinterpret_cast<const bf16*>(a), lda, reinterpret_cast<const bf16*>(w), bias, out, M, N, K, mode, cap);
  LIA_LAUNCH_CHECK();
  return LIA_OK;
}

extern "C" int lia_linear_plain(const void* A, int a_f32, long long lda, long long sA, const void* W, int w_f32, long long ldw, long long sW,
                                void* C, int c_f32, long long ldc, long long sC, int M, int N, int K, int batch, float scale,
                                lia_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  LIA_CHECK_ARG(A && W && C && M > 0 && N > 0 && K > 0 && batch > 0 && batch <= 65535, "lia_linear_plain: bad arguments");
  LIA_CHECK_ARG(lda >= K && ldw >= K && ldc >= N, "lia_linear_plain: leading dimensions smaller than the rows");
  LIA_CHECK_ARG((M + 63) / 64 <= 65535, "lia_linear_plain: too many rows (%d)", M);
  if (a_f32 && w_f32) return launch_plain<float, float>(A, lda, sA, W, ldw, sW, C, ldc, sC, M, N, K, batch, scale, c_f32, stream);
  if (a_f32) return launch_plain<float, bf16>(A, lda, sA, W, ldw, sW, C, ldc, sC, M, N, K, batch, scale, c_f32, stream);
  if (w_f32) return launch_plain<bf16, float>(A, lda, sA, W, ldw, sW, C, ldc, sC, M, N, K, batch, scale, c_f32, stream);
  return launch_plain<bf16, bf16>(A, lda, sA, W, ldw, sW, C, ldc, sC, M, N, K, batch, scale, c_f32, stream);
}

extern "C" int lia_argmax_f32(const float* logits, int64_t* next, int B, int V, int suppress_id, lia_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  LIA_CHECK_ARG(logits && next && B > 0 && V > 0, "lia_argmax_f32: bad arguments");
  argmax_f32_kernel<<<B, 256, 0, stream>>>(logits, next, V, suppress_id);
  LIA_LAUNCH_CHECK();
  return LIA_OK;
}

extern "C" int lia_embed_scale_pos(const int64_t* ids, const void* table, const void* pos_table, int table_f32, float scale, const int* meta,
                                   float* x, void* cat, int cat_f32, int rows, int W, int vocab, int max_pos, lia_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  LIA_CHECK_ARG(ids && table && meta && x && rows > 0 && W > 0 && vocab > 0 && (!pos_table || max_pos > 0), "lia_embed_scale_pos: bad arguments");
#define LIA_ESP(T, TC) embed_scale_pos_kernel<T, TC><<<rows, 256, 0, stream>>>(ids, reinterpret_cast<const T*>(table), scale, reinterpret_cast<const T*>(pos_table), meta, x, reinterpret_cast<TC*>(cat), W, vocab, max_pos)
  if (table_f32 && cat_f32) LIA_ESP(float, float);
  else if (table_f32) LIA_ESP(float, bf16);
  else if (cat_f32) LIA_ESP(bf16, float);
  else LIA_ESP(bf16, bf16);
#undef LIA_ESP
  LIA_LAUNCH_CHECK();
  return LIA_OK;
}

extern "C" int lia_residual_norm(float* x, const void* y, int y_f32, int replace, const float* bias, const float* w, void* h, int h_f32,
                                 long long ldh, int rows, int W, float eps, lia_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  LIA_CHECK_ARG(x && (y || bias || h), "lia_residual_norm: nothing to do");
  LIA_CHECK_ARG(!replace || y, "lia_residual_norm: replacing the stream needs what replaces it");
  LIA_CHECK_ARG(rows > 0 && W > 0 && (size_t)W * 4 <= 160 * 1024 && (!h || ldh >= W), "lia_residual_norm: bad shape rows=%d W=%d", rows, W);
  const size_t smem = (size_t)W * sizeof(float);
#define LIA_RN(TY, TH)                                                                                                       \
  do {                                                                                                                       \
    if (smem > 48 * 1024) LIA_CUDA(cudaFuncSetAttribute(residual_norm_kernel<TY, TH>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
    residual_norm_kernel<TY, TH><<<rows, 256, smem, stream>>>(x, reinterpret_cast<const TY*>(y), replace, bias, w, reinterpret_cast<TH*>(h), ldh, W, eps); \
  } while (0)
  if (y_f32 && h_f32) LIA_RN(float, float);
  else if (y_f32) LIA_RN(float, bf16);
  else if (h_f32) LIA_RN(bf16, float);
  else LIA_RN(bf16, bf16);
#undef LIA_RN
  LIA_LAUNCH_CHECK();
  return LIA_OK;
}

extern "C" int lia_rms_norm_rows(const void* in, int in_f32, long long ld, const float* w, void* out, int out_f32, int M, int N, float eps,
                                 lia_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  LIA_CHECK_ARG(in && w && out && M > 0 && N > 0 && ld >= N, "lia_rms_norm_rows: bad arguments");
  const unsigned grid = (unsigned)((M + 3) / 4);
#define LIA_RNR(TI, TO) rms_norm_rows_kernel<TI, TO><<<grid, 128, 0, stream>>>(reinterpret_cast<const TI*>(in), ld, w, reinterpret_cast<TO*>(out), M, N, eps)
  if (in_f32 && out_f32) LIA_RNR(float, float);
  else if (in_f32) LIA_RNR(float, bf16);
  else if (out_f32) LIA_RNR(bf16, float);
  else LIA_RNR(bf16, bf16);
#undef LIA_RNR
  LIA_LAUNCH_CHECK();
  return LIA_OK;
}

extern "C" int lia_sigmoid_mul(const void* a, int a_f32, long long lda, const void* gate, int gate_f32, long long ldg, void* out, int out_f32,
                               int M, int F, lia_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  LIA_CHECK_ARG(a && gate && out && M > 0 && F > 0 && lda >= F && ldg >= F, "lia_sigmoid_mul: bad arguments");
  LIA_CHECK_ARG(gate_f32 == out_f32, "lia_sigmoid_mul: the gate and the output have the activations' type");
  const size_t n = (size_t)M * F;
  size_t blocks = (n + 255) / 256;
  const size_t capb = (size_t)lia_sm_count() * 16;
  if (blocks > capb) blocks = capb;
#define LIA_SM(TA, TG) sigmoid_mul_kernel<TA, TG, TG><<<(unsigned)blocks, 256, 0, stream>>>(reinterpret_cast<const TA*>(a), lda, reinterpret_cast<const TG*>(gate), ldg, reinterpret_cast<TG*>(out), M, F)
  if (a_f32 && gate_f32) LIA_SM(float, float);
  else if (a_f32) LIA_SM(float, bf16);
  else if (gate_f32) LIA_SM(bf16, float);
  else LIA_SM(bf16, bf16);
#undef LIA_SM
  LIA_LAUNCH_CHECK();
  return LIA_OK;
}

extern "C" int lia_softcap_f32(float* x, long long n, float cap, lia_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  LIA_CHECK_ARG(x && n > 0 && cap > 0.f, "lia_softcap_f32: bad arguments");
  size_t blocks = ((size_t)n + 255) / 256;
  const size_t capb = (size_t)lia_sm_count() * 16;
  if (blocks > capb) blocks = capb;
  softcap_kernel<<<(unsigned)blocks, 256, 0, stream>>>(x, (size_t)n, cap);
  LIA_LAUNCH_CHECK();
  return LIA_OK;
}
