// Matrix-memory recurrence (mLSTM) with a running-maximum stabiliser, for prompts, portions of prompts and single decoded
// tokens alike.  Per head, with log gates i_t, f_t (already capped / log-sigmoided by the gate projection's epilogue):
//     m_t = max(f_t + m_{t-1}, i_t)
//     S_t = exp(f_t + m_{t-1} - m_t) S_{t-1} + exp(i_t - m_t) k_t v_t^T          (dim x vdim)
//     n_t = exp(f_t + m_{t-1} - m_t) n_{t-1} + exp(i_t - m_t) k_t
//     o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + den_eps)
// State (S, n, m) is fp32 and lives per sequence slot; S is stored transposed, [slot][head][vdim][dim], so that the
// dim-long column a warp owns is contiguous.  Everything here is fp32 arithmetic on the CUDA cores; q, k, v arrive as the
// projection wrote them (bf16 or fp32).
//
// Work split: a warp owns CW = 2 columns of S (2 value channels) of one head of one sequence and keeps them in registers
// for the whole portion; lane l owns rows l, l+32, ...  A token costs the warp DR*CW*2 FMAs per lane and one butterfly
// reduction of CW+1 partial dot products; nothing is synchronised per token.  The 8 warps of a block share q, k and the
// gates of their head through a double-buffered shared-memory stage of TB = 8 tokens that is fetched while the previous
// 8 tokens are processed -- with 128-bit loads where the rows allow it: every block of a head re-reads that head's q and
// k, and with one load instruction (and its address arithmetic) per number the fetch cost more issue slots than the
// recurrence itself (2048 tokens, heads of 256 x 512: 1.24 -> 0.87 ms per layer).
#include <math.h>

#include "common.cuh"

namespace {

template <typename T> __device__ __forceinline__ float ldf(const T* p);
template <> __device__ __forceinline__ float ldf<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ldf<bf16>(const bf16* p) { return __bfloat162float(*p); }
// Stage loads stay where they are written (volatile asm) and return RAW bits: nothing touches the loaded register until the
// stage is stored to shared memory, so all loads of a stage are in flight together while the previous stage is processed.
// (A conversion right after each load would make the warp wait for every load in turn.)
template <typename T> struct Raw;
template <> struct Raw<float> {
  typedef float type;
  static __device__ __forceinline__ float ld(const float* p) {
    float v;
    asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(v) : "l"(p));
    return v;
  }
  static __device__ __forceinline__ float to_float(float v) { return v; }
};
template <> struct Raw<bf16> {
  typedef unsigned short type;
  static __device__ __forceinline__ unsigned short ld(const bf16* p) {
    unsigned short u;
    asm volatile("ld.global.nc.u16 %0, [%1];" : "=h"(u) : "l"(p));
    return u;
  }
  static __device__ __forceinline__ float to_float(unsigned short u) { return __uint_as_float((unsigned)u << 16); }
};
// 128-bit stage load (raw bits, same reasoning) and its unpacking into VEC floats of a 16-byte aligned shared-memory row
__device__ __forceinline__ uint4 ld_raw128(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
template <typename T> struct Vec128;
template <> struct Vec128<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void put(float* dst, uint4 v) {
    *reinterpret_cast<float4*>(dst) = make_float4(__uint_as_float(v.x), __uint_as_float(v.y), __uint_as_float(v.z), __uint_as_float(v.w));
  }
};
template <> struct Vec128<bf16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void put(float* dst, uint4 v) {
    reinterpret_cast<float4*>(dst)[0] = make_float4(__uint_as_float(v.x << 16), __uint_as_float(v.x & 0xffff0000u),
                                                    __uint_as_float(v.y << 16), __uint_as_float(v.y & 0xffff0000u));
    reinterpret_cast<float4*>(dst)[1] = make_float4(__uint_as_float(v.z << 16), __uint_as_float(v.z & 0xffff0000u),
                                                    __uint_as_float(v.w << 16), __uint_as_float(v.w & 0xffff0000u));
  }
};
template <typename T> __device__ __forceinline__ void stf(T* p, float v);
template <> __device__ __forceinline__ void stf<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void stf<bf16>(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

constexpr int TB = 8;            // tokens per stage
constexpr int CW = 2;            // columns of S per warp
constexpr int NW = 8;            // warps per block (two per scheduler: one warp alone cannot hide its own dependent-issue latency)
constexpr int CB = CW * NW;      // columns per block

// segs[s] = {slot, first position, first row, rows} of portion s.  VL: the stage is fetched with 128-bit loads (the host
// checked that every q / k / v segment of VEC numbers starts on a 16-byte boundary and is wholly inside or outside its row).
template <typename T, int DR, bool VL>
__global__ void __launch_bounds__(NW * 32, 2) mlstm_scan_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, int ld,
                                                             const float* __restrict__ gates, float* __restrict__ St, float* __restrict__ nst,
                                                             float* __restrict__ mst, const int* __restrict__ segs, int H, int dim, int vdim,
                                                             float q_scale, float den_eps, float* __restrict__ o) {
  constexpr int DP = DR * 32;                    // dim padded to whole warps
  constexpr int ROWF = 2 * DP + CB + 4;          // floats of one staged token: q | k | v (this block's columns) | i | f | 2 pad (16-byte rows)
  constexpr int VEC = Vec128<T>::N;
  constexpr int CH = (2 * DP + CB) / VEC;        // 128-bit segments of one staged token
  constexpr int NST = VL ? (TB * CH + NW * 32 - 1) / (NW * 32) : (TB * ROWF + NW * 32 - 1) / (NW * 32);
  extern __shared__ __align__(16) float stage[]; // [2][TB][ROWF]
  const int seg = blockIdx.z, h = blockIdx.y, colb = blockIdx.x * CB;
  const int slot = segs[4 * seg], row0 = segs[4 * seg + 2], len = segs[4 * seg + 3];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int col0 = colb + warp * CW;

  float S[DR][CW], n[DR];
  float* Sp = St + ((size_t)slot * H + h) * vdim * dim;
  float* np = nst + ((size_t)slot * H + h) * dim;
#pragma unroll
  for (int i = 0; i < DR; ++i) {
    const int r = lane + 32 * i;
    n[i] = r < dim ? np[r] : 0.f;
#pragma unroll
    for (int c = 0; c < CW; ++c) S[i][c] = (r < dim && col0 + c < vdim) ? Sp[(size_t)(col0 + c) * dim + r] : 0.f;
  }
  float m = mst[(size_t)slot * H + h];

  typename Raw<T>::type buf[VL ? 1 : NST];
  uint4 vbuf[VL ? NST : 1];
  float gbuf = 0.f;
  // fetch the inputs of tokens [g*TB, g*TB+TB) of the portion into registers: q | k | v elements by all threads (one
  // predicated load site, no use of the result), the 2 gates of each token by the first 2*TB threads
  auto fetch = [&](int g) {
    if constexpr (VL) {
#pragma unroll
      for (int s = 0; s < NST; ++s) {
        const int e = threadIdx.x + s * NW * 32;
        const T* p = nullptr;
        if (e < TB * CH) {
          const int t = e / CH, j = (e - t * CH) * VEC;
          const int tok = g * TB + t;
          if (tok < len) {
            const size_t row = (size_t)(row0 + tok);
            if (j < DP) { if (j < dim) p = q + row * ld + h * dim + j; }
            else if (j < 2 * DP) { if (j - DP < dim) p = k + row * ld + h * dim + (j - DP); }
            else if (colb + j - 2 * DP < vdim) p = v + row * ld + h * vdim + colb + (j - 2 * DP);
          }
        }
        vbuf[s] = make_uint4(0u, 0u, 0u, 0u);
        if (p != nullptr) vbuf[s] = ld_raw128(p);
      }
    } else {
#pragma unroll
    for (int s = 0; s < NST; ++s) {
      const int e = threadIdx.x + s * NW * 32;
      const T* p = nullptr;
      if (e < TB * ROWF) {
        const int t = e / ROWF, j = e - t * ROWF;
        const int tok = g * TB + t;
        if (tok < len) {
          const size_t row = (size_t)(row0 + tok);
          if (j < dim) p = q + row * ld + h * dim + j;
          else if (j >= DP && j - DP < dim) p = k + row * ld + h * dim + (j - DP);
          else if (j >= 2 * DP && j < 2 * DP + CB && colb + j - 2 * DP < vdim) p = v + row * ld + h * vdim + colb + (j - 2 * DP);
        }
      }
      buf[s] = typename Raw<T>::type(0);
      if (p != nullptr) buf[s] = Raw<T>::ld(p);
    }
    }
    if (threadIdx.x < 2 * TB) {
      const int tok = g * TB + (threadIdx.x >> 1);
      gbuf = 0.f;
      if (tok < len) gbuf = Raw<float>::ld(gates + (size_t)(row0 + tok) * 2 * H + (threadIdx.x & 1) * H + h);
    }
  };
  auto put = [&](int b) {
    if constexpr (VL) {
#pragma unroll
      for (int s = 0; s < NST; ++s) {
        const int e = threadIdx.x + s * NW * 32;
        if (e < TB * CH) {
          const int t = e / CH, j = (e - t * CH) * VEC;
          Vec128<T>::put(stage + b * TB * ROWF + t * ROWF + j, vbuf[s]);
        }
      }
    } else {
#pragma unroll
    for (int s = 0; s < NST; ++s) {
      const int e = threadIdx.x + s * NW * 32;
      if (e < TB * ROWF) {
        const int j = e % ROWF;
        if (j < 2 * DP + CB) stage[b * TB * ROWF + e] = Raw<T>::to_float(buf[s]);
      }
    }
    }
    if (threadIdx.x < 2 * TB) stage[b * TB * ROWF + (threadIdx.x >> 1) * ROWF + 2 * DP + CB + (threadIdx.x & 1)] = gbuf;
  };

  const int groups = (len + TB - 1) / TB;
  fetch(0);
  put(0);
  __syncthreads();
  for (int g = 0; g < groups; ++g) {
    if (g + 1 < groups) fetch(g + 1);            // in flight while this group is processed
    const float* st = stage + (g & 1) * TB * ROWF;
    const int nt = min(TB, len - g * TB);
    auto token = [&](int t) {
      const float* tk = st + t * ROWF;
      const float ig = tk[2 * DP + CB], fg = tk[2 * DP + CB + 1];
      const float m_new = fmaxf(fg + m, ig);
      const float a = expf(fg + m - m_new), b = expf(ig - m_new);
      float vc[CW];
#pragma unroll
      for (int c = 0; c < CW; ++c) vc[c] = tk[2 * DP + warp * CW + c];
      float part[CW + 1];
#pragma unroll
      for (int c = 0; c <= CW; ++c) part[c] = 0.f;
#pragma unroll
      for (int i = 0; i < DR; ++i) {
        const float qv = tk[lane + 32 * i] * q_scale, kv = tk[DP + lane + 32 * i];
        const float bk = b * kv;
        n[i] = fmaf(a, n[i], bk);
        part[CW] = fmaf(n[i], qv, part[CW]);
#pragma unroll
        for (int c = 0; c < CW; ++c) {
          S[i][c] = fmaf(a, S[i][c], bk * vc[c]);
          part[c] = fmaf(S[i][c], qv, part[c]);
        }
      }
#pragma unroll
      for (int c = 0; c <= CW; ++c) part[c] = warp_sum(part[c]);
      const float den = fmaxf(fabsf(part[CW]), expf(-m_new)) + den_eps;
      m = m_new;
      float mine = part[0];
#pragma unroll
      for (int c = 1; c < CW; ++c) mine = (lane == c) ? part[c] : mine;
      if (lane < CW && col0 + lane < vdim) o[(size_t)(row0 + g * TB + t) * H * vdim + h * vdim + col0 + lane] = mine / den;
    };
    for (int t = 0; t < nt; ++t) token(t);
    if (g + 1 < groups) put((g + 1) & 1);        // the other buffer: last read two groups ago, before the barrier below
    __syncthreads();
  }

#pragma unroll
  for (int i = 0; i < DR; ++i) {
    const int r = lane + 32 * i;
    if (r < dim) {
      if (colb == 0 && warp == 0) np[r] = n[i];
#pragma unroll
      for (int c = 0; c < CW; ++c)
        if (col0 + c < vdim) Sp[(size_t)(col0 + c) * dim + r] = S[i][c];
    }
  }
  if (colb == 0 && threadIdx.x == 0) mst[(size_t)slot * H + h] = m;
}

// out[row][h][c] = o / sqrt(mean_c(o^2) + eps) * w[h*vdim + c] * act(gate[row][h*vdim + c]), act = sigmoid (gate_silu == 0) or
// SiLU; one warp per (row, head)
template <typename T>
__global__ void __launch_bounds__(128) headnorm_gate_kernel(const float* __restrict__ o, const float* __restrict__ w, const T* __restrict__ gate, int ldg,
                                                            T* __restrict__ out, int M, int H, int vdim, float eps, int gate_silu) {
  const int pair = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (pair >= M * H) return;
  const int row = pair / H, h = pair - row * H;
  const float* orow = o + (size_t)row * H * vdim + h * vdim;
  float ss = 0.f;
  for (int c = lane; c < vdim; c += 32) ss += orow[c] * orow[c];
  ss = warp_sum(ss);
  const float inv = 1.0f / sqrtf(ss / (float)vdim + eps);
  for (int c = lane; c < vdim; c += 32) {
    float factor = 1.0f;                                    // no gate: the norm alone
    if (gate != nullptr) {
      const float g = ldf(gate + (size_t)row * ldg + h * vdim + c);
      const float sg = 1.0f / (1.0f + expf(-g));
      factor = gate_silu ? g * sg : sg;
    }
    stf(out + (size_t)row * H * vdim + h * vdim + c, orow[c] * inv * w[h * vdim + c] * factor);
  }
}

template <typename T, int DR, bool VL>
int launch_scan_as(const void* q, const void* k, const void* v, int ld, const float* gates, float* St, float* nst, float* mst, const int* segs,
                int nseg, int H, int dim, int vdim, float q_scale, float den_eps, float* o, cudaStream_t stream) {
  const size_t smem = (size_t)2 * TB * (2 * DR * 32 + CB + 4) * sizeof(float);
  if (smem > 48 * 1024) LIA_CUDA(cudaFuncSetAttribute(mlstm_scan_kernel<T, DR, VL>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  dim3 grid((vdim + CB - 1) / CB, H, nseg);
  mlstm_scan_kernel<T, DR, VL><<<grid, NW * 32, smem, stream>>>(reinterpret_cast<const T*>(q), reinterpret_cast<const T*>(k), reinterpret_cast<const T*>(v),
                                                            ld, gates, St, nst, mst, segs, H, dim, vdim, q_scale, den_eps, o);
  LIA_LAUNCH_CHECK();
  return LIA_OK;
}

template <typename T, int DR>
int launch_scan(const void* q, const void* k, const void* v, int ld, const float* gates, float* St, float* nst, float* mst, const int* segs,
                int nseg, int H, int dim, int vdim, float q_scale, float den_eps, float* o, cudaStream_t stream) {
  constexpr int VEC = Vec128<T>::N;
  const bool aligned = ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v)) % 16 == 0) &&
                       ld % VEC == 0 && dim % VEC == 0 && vdim % VEC == 0;
  if (aligned) return launch_scan_as<T, DR, true>(q, k, v, ld, gates, St, nst, mst, segs, nseg, H, dim, vdim, q_scale, den_eps, o, stream);
  return launch_scan_as<T, DR, false>(q, k, v, ld, gates, St, nst, mst, segs, nseg, H, dim, vdim, q_scale, den_eps, o, stream);
}

template <typename T>
int dispatch_scan(const void* q, const void* k, const void* v, int ld, const float* gates, float* St, float* nst, float* mst, const int* segs,
                  int nseg, int H, int dim, int vdim, float q_scale, float den_eps, float* o, cudaStream_t stream) {
  if (dim <= 32) return launch_scan<T, 1>(q, k, v, ld, gates, St, nst, mst, segs, nseg, H, dim, vdim, q_scale, den_eps, o, stream);
  if (dim <= 64) return launch_scan<T, 2>(q, k, v, ld, gates, St, nst, mst, segs, nseg, H, dim, vdim, q_scale, den_eps, o, stream);
  if (dim <= 128) return launch_scan<T, 4>(q, k, v, ld, gates, St, nst, mst, segs, nseg, H, dim, vdim, q_scale, den_eps, o, stream);
  if (dim <= 256) return launch_scan<T, 8>(q, k, v, ld, gates, St, nst, mst, segs, nseg, H, dim, vdim, q_scale, den_eps, o, stream);
  return launch_scan<T, 16>(q, k, v, ld, gates, St, nst, mst, segs, nseg, H, dim, vdim, q_scale, den_eps, o, stream);
}

}  // namespace

extern "C" int lia_mlstm_scan(const void* q, const void* k, const void* v, int act_f32, int ld, const float* gates, float* state_S,
                              float* state_n, float* state_m, const int* segs, int nseg, int H, int dim, int vdim, float q_scale,
                              float den_eps, float* o, lia_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  LIA_CHECK_ARG(q && k && v && gates && state_S && state_n && state_m && segs && o, "lia_mlstm_scan: null pointer");
  LIA_CHECK_ARG(nseg > 0 && nseg <= 65535 && H > 0 && H <= 65535 && dim > 0 && dim <= 512 && vdim > 0, "lia_mlstm_scan: bad shape nseg=%d H=%d dim=%d vdim=%d", nseg, H, dim, vdim);
  if (act_f32) return dispatch_scan<float>(q, k, v, ld, gates, state_S, state_n, state_m, segs, nseg, H, dim, vdim, q_scale, den_eps, o, stream);
  return dispatch_scan<bf16>(q, k, v, ld, gates, state_S, state_n, state_m, segs, nseg, H, dim, vdim, q_scale, den_eps, o, stream);
}

extern "C" int lia_headnorm_gate(const float* o, const float* w, const void* gate, int ldg, void* out, int act_f32, int M, int H, int vdim,
                                 float eps, int gate_silu, lia_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  LIA_CHECK_ARG(o && w && out && M > 0 && H > 0 && vdim > 0 && (!gate || ldg >= H * vdim), "lia_headnorm_gate: bad arguments");
  const long long pairs = (long long)M * H;
  const unsigned grid = (unsigned)((pairs + 3) / 4);
  if (act_f32) headnorm_gate_kernel<float><<<grid, 128, 0, stream>>>(o, w, reinterpret_cast<const float*>(gate), ldg, reinterpret_cast<float*>(out), M, H, vdim, eps, gate_silu);
  else headnorm_gate_kernel<bf16><<<grid, 128, 0, stream>>>(o, w, reinterpret_cast<const bf16*>(gate), ldg, reinterpret_cast<bf16*>(out), M, H, vdim, eps, gate_silu);
  LIA_LAUNCH_CHECK();
  return LIA_OK;
}
