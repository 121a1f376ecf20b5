// Attention over a compressed (latent) key/value cache.  A token caches ONE row per layer: its normalised latent c
// (kv_rank numbers) followed by one rotated key part (rot numbers) shared by all heads.  Keys and values of a head are
// linear in c (k_h = Wuk_h c, v_h = Wuv_h c), so the kernels never expand them: the query of head h is carried into the
// latent space once (q~_h = Wuk_h^T q_h, a small batched projection made by the caller) and
//     score(t, s, h) = (q~_{t,h} . c_s + qrot_{t,h} . krot_s) * scale,     out~_{t,h} = sum_s softmax_s(score) c_s,
// after which the caller applies Wuv_h to out~.  Per cached token the kernel reads kv_rank + rot numbers whatever the
// number of heads.  Scores, softmax weights and the weighted sums are fp32.
//
//   latent_prep:  RMS-norm of the latent part with its per-channel weight, rotary embedding ("rotate half": channel i is
//                 paired with i + dims/2) of the shared key part at the token's position, both written into the cache row;
//                 the same rotation of each head's rotated query part, written behind that head's q~ slot.
//                 latent_prep_pairs is the same step with the rotation of neighbouring channels (2i, 2i+1) by angles from a
//                 float64 frequency table (so that interpolated frequencies come from the host) and an amplitude on cos and sin.
//   latent_attn:  one block per (token, group of up to 8 heads, range of keys); 32 cached rows at a time are staged in shared
//                 memory as fp32, scored (warp = head, lane = key), folded into a running softmax, and accumulated.  Few rows
//                 and a long history (decoding): the keys are split over several blocks and a second kernel combines.
#include <math.h>

#include "common.cuh"

namespace {

template <typename T> __device__ __forceinline__ float ldf(const T* p);
template <> __device__ __forceinline__ float ldf<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ldf<bf16>(const bf16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void stf(T* p, float v);
template <> __device__ __forceinline__ void stf<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void stf<bf16>(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

// rotate-half rotary embedding of `src[0..n)` at position `pos`: the first `dims` channels are rotated, the rest copied.
// inv_freq[i] = base^(-2i/dims), i < dims/2 (fp32, made on the host); the angle pos * inv_freq[i] is an fp32 product.
__device__ __forceinline__ float rotate_half(const float* src, int j, int dims, float pos, const float* inv_freq) {
  if (j >= dims) return src[j];
  const int half = dims >> 1;
  const int i = j < half ? j : j - half;
  const float ang = pos * inv_freq[i];
  const float c = cosf(ang), s = sinf(ang);
  return j < half ? src[j] * c - src[j + half] * s : src[j] * c + src[j - half] * s;
}

// meta[row] = {slot, position}.  Block per token row.
template <typename T>
__global__ void __launch_bounds__(128) latent_prep_kernel(const T* __restrict__ qin, int ldq, const T* __restrict__ dkv, int ldd,
                                                          const float* __restrict__ cw, const float* __restrict__ inv_freq, const int* __restrict__ meta,
                                                          T* __restrict__ cache, long long slot_stride, float* __restrict__ qa, int H, int dim, int rot,
                                                          int rot_dims, int kv_rank, float eps) {
  extern __shared__ float sh[];                 // rot floats: one vector to rotate
  __shared__ float red[4];
  const int row = blockIdx.x;
  const int slot = meta[2 * row], p = meta[2 * row + 1];
  const float pos = (float)p;
  const int D = kv_rank + rot;
  const T* d = dkv + (size_t)row * ldd;
  T* crow = cache + (size_t)slot * slot_stride + (size_t)p * D;

  float ss = 0.f;
  for (int i = threadIdx.x; i < kv_rank; i += 128) {
    const float v = ldf(d + i);
    ss += v * v;
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  for (int i = threadIdx.x; i < rot; i += 128) sh[i] = ldf(d + kv_rank + i);
  __syncthreads();
  const float inv = 1.0f / sqrtf((red[0] + red[1] + red[2] + red[3]) / (float)kv_rank + eps);
  for (int i = threadIdx.x; i < kv_rank; i += 128) stf(crow + i, ldf(d + i) * inv * cw[i]);
  for (int i = threadIdx.x; i < rot; i += 128) stf(crow + kv_rank + i, rotate_half(sh, i, rot_dims, pos, inv_freq));
  for (int h = 0; h < H; ++h) {
    __syncthreads();
    for (int i = threadIdx.x; i < rot; i += 128) sh[i] = ldf(qin + (size_t)row * ldq + h * (dim + rot) + dim + i);
    __syncthreads();
    for (int i = threadIdx.x; i < rot; i += 128) qa[((size_t)row * H + h) * D + kv_rank + i] = rotate_half(sh, i, rot_dims, pos, inv_freq);
  }
}

// The same step with the pairwise rotation: channels (2i, 2i+1), i < rot_dims/2, turn by pos * freq[i]; cos and sin carry the
// amplitude `mag`.  The angle is a float64 product (positions in the thousands times an irrational frequency), its sine and
// cosine are rounded once to fp32 and shared by the key part and all heads' query parts.
template <typename T>
__global__ void __launch_bounds__(128) latent_prep_pairs_kernel(const T* __restrict__ qin, int ldq, const T* __restrict__ dkv, int ldd,
                                                                const float* __restrict__ cw, const double* __restrict__ freq, float mag,
                                                                const int* __restrict__ meta, T* __restrict__ cache, long long slot_stride,
                                                                float* __restrict__ qa, int H, int dim, int rot, int rot_dims, int kv_rank, float eps) {
  extern __shared__ float cs[];                 // cos | sin of the rot_dims / 2 pairs
  __shared__ float red[4];
  const int row = blockIdx.x;
  const int slot = meta[2 * row], p = meta[2 * row + 1];
  const int D = kv_rank + rot, npair = rot_dims / 2;
  const T* d = dkv + (size_t)row * ldd;
  T* crow = cache + (size_t)slot * slot_stride + (size_t)p * D;
  for (int i = threadIdx.x; i < npair; i += 128) {
    double sn, c;
    sincos((double)p * freq[i], &sn, &c);
    cs[i] = (float)c * mag;
    cs[npair + i] = (float)sn * mag;
  }
  float ss = 0.f;
  for (int i = threadIdx.x; i < kv_rank; i += 128) {
    const float v = ldf(d + i);
    ss += v * v;
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  const float inv = 1.0f / sqrtf((red[0] + red[1] + red[2] + red[3]) / (float)kv_rank + eps);
  for (int i = threadIdx.x; i < kv_rank; i += 128) stf(crow + i, ldf(d + i) * inv * cw[i]);
  // vector 0: the shared key part (into the cache); vector 1 + h: head h's rotated query part (into its q~ slot, fp32)
  for (int e = threadIdx.x; e < (H + 1) * rot; e += 128) {
    const int vec = e / rot, i = e - vec * rot;
    const T* src = vec == 0 ? d + kv_rank : qin + (size_t)row * ldq + (size_t)(vec - 1) * (dim + rot) + dim;
    float val = ldf(src + i);
    if (i < rot_dims) {
      const float other = ldf(src + (i ^ 1));
      const int pr = i >> 1;
      val = (i & 1) == 0 ? val * cs[pr] - other * cs[npair + pr] : val * cs[pr] + other * cs[npair + pr];
    }
    if (vec == 0) stf(crow + kv_rank + i, val);
    else qa[((size_t)row * H + (vec - 1)) * D + kv_rank + i] = val;
  }
}

constexpr int TK = 32;     // cached rows per stage (= one warp's lanes: lane j scores key j)
constexpr int HG = 8;      // heads per block (= warps per block: warp w scores head w)

__host__ __device__ inline int padded_row(int D) { return (D + 3) / 4 * 4 + 4; }   // smem row stride: 16-byte rows, conflict-free 128-bit reads

// one cached row segment of VEC numbers as floats (128-bit load)
__device__ __forceinline__ void load_vec(const bf16* p, float* f) { unpack8(*reinterpret_cast<const uint4*>(p), f); }
__device__ __forceinline__ void load_vec(const float* p, float* f) {
  const float4 v = *reinterpret_cast<const float4*>(p);
  f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
}
template <typename T> struct Vec { static constexpr int N = 8; };
template <> struct Vec<float> { static constexpr int N = 4; };

// qa [M][H][D] fp32, cache [slot][capacity][D], out [M][H][kv_rank] fp32, times gate[M][H] (a per-head output gate) if
// given.  RM = ceil(kv_rank / 256).  gridDim.z = nsplit: block z takes the z-th part of the row's keys; with nsplit > 1 the
// unnormalised sums go to `part` ([M][H][nsplit][kv_rank]) and (max, sum) to `part_ml`, and latent_combine_kernel finishes.
template <typename T, int RM>
__global__ void __launch_bounds__(256) latent_attn_kernel(const float* __restrict__ qa, const T* __restrict__ cache, long long slot_stride,
                                                          const int* __restrict__ meta, const float* __restrict__ gate, float* __restrict__ out,
                                                          float* __restrict__ part, float2* __restrict__ part_ml, int H, int kv_rank, int rot,
                                                          float scale) {
  extern __shared__ __align__(16) float sm[];
  const int D = kv_rank + rot, DS = padded_row(D), G4 = (DS - 4) / 4;
  float* qs = sm;                    // [HG][DS]
  float* ks = qs + HG * DS;          // [TK][DS]
  float* ps = ks + TK * DS;          // [HG][TK]
  float* alpha = ps + HG * TK;       // [HG]
  float* lsum = alpha + HG;          // [HG]
  float* msum = lsum + HG;           // [HG]
  float* red = msum + HG;            // [8 warps][HG][TK] partial dot products
  const int row = blockIdx.x, h0 = blockIdx.y * HG, z = blockIdx.z, nsplit = gridDim.z;
  const int nh = min(HG, H - h0);
  const int slot = meta[2 * row], pos = meta[2 * row + 1];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const T* crows = cache + (size_t)slot * slot_stride;
  const int tiles = (pos + TK) / TK, per = (tiles + nsplit - 1) / nsplit;
  const int j_begin = z * per * TK, j_end = min(pos + 1, (z + 1) * per * TK);
  constexpr int VEC = Vec<T>::N;
  const bool vec = (D % VEC == 0) && (slot_stride % VEC == 0) && (reinterpret_cast<uintptr_t>(cache) % 16 == 0);

  for (int e = threadIdx.x; e < HG * DS; e += 256) {
    const int hh = e / DS, d = e - hh * DS;
    qs[e] = (hh < nh && d < D) ? qa[((size_t)row * H + h0 + hh) * D + d] : 0.f;
  }
  for (int e = threadIdx.x; e < TK * (DS - D); e += 256) {          // the pad columns of the key stage stay zero
    const int j = e / (DS - D);
    ks[j * DS + D + (e - j * (DS - D))] = 0.f;
  }
  float acc[HG][RM];
#pragma unroll
  for (int hh = 0; hh < HG; ++hh)
#pragma unroll
    for (int i = 0; i < RM; ++i) acc[hh][i] = 0.f;
  float m_run = -INFINITY, l_run = 0.f;          // of head `warp`, identical in all its lanes

  for (int j0 = j_begin; j0 < j_end; j0 += TK) {
    __syncthreads();                             // previous stage fully consumed (and qs written, first time)
    const int nk = min(TK, j_end - j0);
    if (vec) {
      const int per_row = D / VEC;
      for (int e = threadIdx.x; e < TK * per_row; e += 256) {
        const int j = e / per_row, c = (e - j * per_row) * VEC;
        float f[VEC];
        if (j < nk) {
          load_vec(crows + (size_t)(j0 + j) * D + c, f);
        } else {
#pragma unroll
          for (int i = 0; i < VEC; ++i) f[i] = 0.f;
        }
#pragma unroll
        for (int i = 0; i < VEC; i += 4) *reinterpret_cast<float4*>(ks + j * DS + c + i) = make_float4(f[i], f[i + 1], f[i + 2], f[i + 3]);
      }
    } else {
      for (int e = threadIdx.x; e < TK * D; e += 256) {
        const int j = e / D, d = e - j * D;
        ks[j * DS + d] = j < nk ? ldf(crows + (size_t)(j0 + j) * D + d) : 0.f;
      }
    }
    __syncthreads();
    {
      // lane = key.  Every warp takes each 8th group of 4 channels for ALL heads of the block, so a staged key row is read
      // from shared memory once per tile and not once per head; the 8 partial sums of a (head, key) meet in `red`.
      const float4* k4 = reinterpret_cast<const float4*>(ks + lane * DS);
      float pd[HG];
#pragma unroll
      for (int hh = 0; hh < HG; ++hh) pd[hh] = 0.f;
      for (int g = warp; g < G4; g += 8) {
        const float4 b = k4[g];
#pragma unroll
        for (int hh = 0; hh < HG; ++hh) {
          if (hh < nh) {
            const float4 a = reinterpret_cast<const float4*>(qs + hh * DS)[g];
            pd[hh] = fmaf(a.x, b.x, fmaf(a.y, b.y, fmaf(a.z, b.z, fmaf(a.w, b.w, pd[hh]))));
          }
        }
      }
#pragma unroll
      for (int hh = 0; hh < HG; ++hh) red[(warp * HG + hh) * TK + lane] = pd[hh];
    }
    __syncthreads();
    if (warp < nh) {                             // warp = head: the partial sums in a fixed order, then the running softmax
      float dot = 0.f;
#pragma unroll
      for (int w = 0; w < 8; ++w) dot += red[(w * HG + warp) * TK + lane];
      const float sc = lane < nk ? dot * scale : -INFINITY;
      const float m_new = fmaxf(m_run, warp_max(sc));          // finite: the stage holds at least one visible key
      const float pr = expf(sc - m_new);
      const float a = expf(m_run - m_new);
      l_run = l_run * a + warp_sum(pr);
      m_run = m_new;
      ps[warp * TK + lane] = pr;
      if (lane == 0) alpha[warp] = a;
    }
    __syncthreads();
#pragma unroll
    for (int hh = 0; hh < HG; ++hh) {
      const float a = hh < nh ? alpha[hh] : 0.f;
#pragma unroll
      for (int i = 0; i < RM; ++i) acc[hh][i] *= a;
    }
    // four keys at a time: weights of absent keys are 0 and their staged rows are zero, so the last group may overrun nk
    for (int j = 0; j < nk; j += 4) {
      float kv[4][RM];
#pragma unroll
      for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int i = 0; i < RM; ++i) {
          const int r = threadIdx.x + 256 * i;
          kv[u][i] = r < kv_rank ? ks[(j + u) * DS + r] : 0.f;
        }
#pragma unroll
      for (int hh = 0; hh < HG; ++hh) {
        if (hh < nh) {
          const float4 pw = *reinterpret_cast<const float4*>(ps + hh * TK + j);
#pragma unroll
          for (int i = 0; i < RM; ++i) {
            acc[hh][i] = fmaf(pw.x, kv[0][i], acc[hh][i]);
            acc[hh][i] = fmaf(pw.y, kv[1][i], acc[hh][i]);
            acc[hh][i] = fmaf(pw.z, kv[2][i], acc[hh][i]);
            acc[hh][i] = fmaf(pw.w, kv[3][i], acc[hh][i]);
          }
        }
      }
    }
  }
  if (warp < nh && lane == 0) {
    lsum[warp] = l_run;
    msum[warp] = m_run;
  }
  __syncthreads();
#pragma unroll
  for (int hh = 0; hh < HG; ++hh) {
    if (hh < nh) {
      const size_t rh = (size_t)row * H + h0 + hh;
      if (nsplit == 1) {
        const float invl = (gate ? gate[rh] : 1.0f) / lsum[hh];
#pragma unroll
        for (int i = 0; i < RM; ++i) {
          const int r = threadIdx.x + 256 * i;
          if (r < kv_rank) out[rh * kv_rank + r] = acc[hh][i] * invl;
        }
      } else {
#pragma unroll
        for (int i = 0; i < RM; ++i) {
          const int r = threadIdx.x + 256 * i;
          if (r < kv_rank) part[(rh * nsplit + z) * kv_rank + r] = acc[hh][i];
        }
        if (threadIdx.x == 0) part_ml[rh * nsplit + z] = make_float2(msum[hh], lsum[hh]);
      }
    }
  }
}

// out[rh] = gate * sum_z part[rh][z] e^(m_z - m) / sum_z l_z e^(m_z - m), m = max_z m_z (a part without keys has m = -inf, l = 0)
__global__ void __launch_bounds__(128) latent_combine_kernel(const float* __restrict__ part, const float2* __restrict__ part_ml,
                                                             const float* __restrict__ gate, float* __restrict__ out, int kv_rank, int nsplit) {
  const size_t rh = blockIdx.x;
  float m = -INFINITY;
  for (int z = 0; z < nsplit; ++z) m = fmaxf(m, part_ml[rh * nsplit + z].x);
  float l = 0.f;
  for (int z = 0; z < nsplit; ++z) l += part_ml[rh * nsplit + z].y * expf(part_ml[rh * nsplit + z].x - m);
  const float g = (gate ? gate[rh] : 1.0f) / l;
  for (int r = threadIdx.x; r < kv_rank; r += 128) {
    float s = 0.f;
    for (int z = 0; z < nsplit; ++z) s = fmaf(part[(rh * nsplit + z) * kv_rank + r], expf(part_ml[rh * nsplit + z].x - m), s);
    out[rh * kv_rank + r] = s * g;
  }
}

template <typename T, int RM>
int launch_attn(const float* qa, const void* cache, long long slot_stride, const int* meta, const float* gate, float* out, float* ws, int nsplit,
                int M, int H, int kv_rank, int rot, float scale, cudaStream_t stream) {
  const int DS = padded_row(kv_rank + rot);
  const size_t smem = ((size_t)HG * DS + (size_t)TK * DS + HG * TK + 3 * HG + 8 * HG * TK) * sizeof(float);
  LIA_CHECK_ARG(smem <= 200 * 1024, "lia_latent_attn: a cache row of %d numbers does not fit the shared-memory stage", kv_rank + rot);
  if (smem > 48 * 1024) LIA_CUDA(cudaFuncSetAttribute(latent_attn_kernel<T, RM>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  dim3 grid(M, (H + HG - 1) / HG, nsplit);
  float* part = ws;
  float2* part_ml = reinterpret_cast<float2*>(ws + (size_t)M * H * nsplit * kv_rank);
  latent_attn_kernel<T, RM><<<grid, 256, smem, stream>>>(qa, reinterpret_cast<const T*>(cache), slot_stride, meta, gate, out, part, part_ml, H,
                                                         kv_rank, rot, scale);
  LIA_LAUNCH_CHECK();
  if (nsplit > 1) {
    latent_combine_kernel<<<(unsigned)((size_t)M * H), 128, 0, stream>>>(part, part_ml, gate, out, kv_rank, nsplit);
    LIA_LAUNCH_CHECK();
  }
  return LIA_OK;
}

template <typename T>
int dispatch_attn(const float* qa, const void* cache, long long slot_stride, const int* meta, const float* gate, float* out, float* ws, int nsplit,
                  int M, int H, int kv_rank, int rot, float scale, cudaStream_t stream) {
  if (kv_rank <= 256) return launch_attn<T, 1>(qa, cache, slot_stride, meta, gate, out, ws, nsplit, M, H, kv_rank, rot, scale, stream);
  if (kv_rank <= 512) return launch_attn<T, 2>(qa, cache, slot_stride, meta, gate, out, ws, nsplit, M, H, kv_rank, rot, scale, stream);
  return launch_attn<T, 4>(qa, cache, slot_stride, meta, gate, out, ws, nsplit, M, H, kv_rank, rot, scale, stream);
}

}  // namespace

extern "C" int lia_latent_prep(const void* q, int ldq, const void* dkv, int ldd, int act_f32, const float* c_norm_w, const float* inv_freq,
                               const int* meta, void* cache, long long slot_stride, float* qa, int M, int H, int dim, int rot, int rot_dims,
                               int kv_rank, float eps, lia_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  LIA_CHECK_ARG(q && dkv && c_norm_w && inv_freq && meta && cache && qa, "lia_latent_prep: null pointer");
  LIA_CHECK_ARG(M > 0 && H > 0 && dim >= 0 && rot > 0 && kv_rank > 0 && rot_dims >= 0 && rot_dims <= rot && rot_dims % 2 == 0 && rot <= 8192,
                "lia_latent_prep: bad shape H=%d dim=%d rot=%d rot_dims=%d kv_rank=%d", H, dim, rot, rot_dims, kv_rank);
  const size_t smem = (size_t)rot * sizeof(float);
  if (act_f32)
    latent_prep_kernel<float><<<M, 128, smem, stream>>>(reinterpret_cast<const float*>(q), ldq, reinterpret_cast<const float*>(dkv), ldd, c_norm_w, inv_freq,
                                                        meta, reinterpret_cast<float*>(cache), slot_stride, qa, H, dim, rot, rot_dims, kv_rank, eps);
  else
    latent_prep_kernel<bf16><<<M, 128, smem, stream>>>(reinterpret_cast<const bf16*>(q), ldq, reinterpret_cast<const bf16*>(dkv), ldd, c_norm_w, inv_freq,
                                                       meta, reinterpret_cast<bf16*>(cache), slot_stride, qa, H, dim, rot, rot_dims, kv_rank, eps);
  LIA_LAUNCH_CHECK();
  return LIA_OK;
}

extern "C" int lia_latent_prep_pairs(const void* q, int ldq, const void* dkv, int ldd, int act_f32, const float* c_norm_w, const double* freq,
                                     float mag, const int* meta, void* cache, long long slot_stride, float* qa, int M, int H, int dim, int rot,
                                     int rot_dims, int kv_rank, float eps, lia_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  LIA_CHECK_ARG(q && dkv && c_norm_w && meta && cache && qa && (freq || rot_dims == 0), "lia_latent_prep_pairs: null pointer");
  LIA_CHECK_ARG(M > 0 && H > 0 && dim >= 0 && rot > 0 && kv_rank > 0 && rot_dims >= 0 && rot_dims <= rot && rot_dims % 2 == 0 && rot <= 8192,
                "lia_latent_prep_pairs: bad shape H=%d dim=%d rot=%d rot_dims=%d kv_rank=%d", H, dim, rot, rot_dims, kv_rank);
  const size_t smem = (size_t)(rot_dims > 0 ? rot_dims : 2) * sizeof(float);
  if (act_f32)
    latent_prep_pairs_kernel<float><<<M, 128, smem, stream>>>(reinterpret_cast<const float*>(q), ldq, reinterpret_cast<const float*>(dkv), ldd, c_norm_w,
                                                              freq, mag, meta, reinterpret_cast<float*>(cache), slot_stride, qa, H, dim, rot, rot_dims, kv_rank, eps);
  else
    latent_prep_pairs_kernel<bf16><<<M, 128, smem, stream>>>(reinterpret_cast<const bf16*>(q), ldq, reinterpret_cast<const bf16*>(dkv), ldd, c_norm_w,
                                                             freq, mag, meta, reinterpret_cast<bf16*>(cache), slot_stride, qa, H, dim, rot, rot_dims, kv_rank, eps);
  LIA_LAUNCH_CHECK();
  return LIA_OK;
}

extern "C" size_t lia_latent_attn_workspace_floats(int M, int H, int kv_rank, int nsplit) {
  if (nsplit <= 1) return 0;
  return (size_t)M * H * nsplit * ((size_t)kv_rank + 2);
}

extern "C" int lia_latent_attn(const float* qa, const void* cache, int cache_f32, long long slot_stride, const int* meta, const float* gate,
                               float* out, float* workspace, int nsplit, int M, int H, int kv_rank, int rot, float scale, lia_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  LIA_CHECK_ARG(qa && cache && meta && out, "lia_latent_attn: null pointer");
  LIA_CHECK_ARG(M > 0 && H > 0 && H <= 65535 * HG && kv_rank > 0 && kv_rank <= 1024 && rot >= 0, "lia_latent_attn: bad shape M=%d H=%d kv_rank=%d rot=%d", M, H, kv_rank, rot);
  LIA_CHECK_ARG(nsplit >= 1 && nsplit <= 64 && (nsplit == 1 || workspace != nullptr), "lia_latent_attn: %d key ranges need a workspace", nsplit);
  if (cache_f32) return dispatch_attn<float>(qa, cache, slot_stride, meta, gate, out, workspace, nsplit, M, H, kv_rank, rot, scale, stream);
  return dispatch_attn<bf16>(qa, cache, slot_stride, meta, gate, out, workspace, nsplit, M, H, kv_rank, rot, scale, stream);
}
