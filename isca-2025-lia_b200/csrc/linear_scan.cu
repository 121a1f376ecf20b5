// Linear-attention recurrences with a matrix state per head, for prompts, portions of prompts and single decoded tokens
// alike, and what prepares their inputs.
//
//   DECAY  (a fixed decay per head):     S_t = d_h S_{t-1} + k_t v_t^T                      o_t = S_t^T q_t
//   DELTA  (gated delta rule):           S'  = g_t S_{t-1};  u_t = beta_t (v_t - S'^T k_t);  S_t = S' + k_t u_t^T;  o_t = S_t^T q_t
//   FORGET (keyless: the per-channel forget gate f_t keeps, its complement 1 - f_t writes):
//                                        row d of S:  S[d] <- f[d] S[d] + (1 - f[d]) v      o = sum_d q[d] S[d]
//
// The state is fp32, one [vdim][dim] matrix per (slot, head) -- stored transposed so that the dim-long column a warp owns
// is contiguous.  A warp keeps CW columns in registers for the whole portion, lane l owning rows l, l + 32, ...; a token
// costs one butterfly reduction (CW sums for DECAY; 2 CW + 1 for DELTA, where S'^T k, S'^T q and k . q are reduced together
// and o_t = g S_{t-1}^T q + u (k . q) needs no second pass).  The 8 warps of a block share the q and k of their head through
// a double-buffered shared-memory stage of TB tokens fetched while the previous TB are processed (128-bit loads where the rows
// allow them).  q and k may belong to a
// smaller number of heads than v (head h reads q/k head h / (H / G)); an activation (SiLU) can be applied as the inputs are
// staged, so that a projection's output feeds the recurrence directly.
//
//   conv_prep:         per token, a short causal convolution over time per channel of q | k | v (taps - 1 earlier inputs come
//                      from the rows before it in the same portion, or from the sequence's state), SiLU, q and k made unit
//                      vectors per head (q also scaled), and the per-head gates beta = sigmoid(.), g = exp(-exp(A) softplus(. + dt)).
//   conv_state_update: the last taps - 1 inputs of every portion become the sequence's new convolution state.
#include <math.h>

#include "common.cuh"

namespace {

template <typename T> __device__ __forceinline__ float ldf(const T* p);
template <> __device__ __forceinline__ float ldf<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ldf<bf16>(const bf16* p) { return __bfloat162float(*p); }

__device__ __forceinline__ float silu(float z) { return z / (1.0f + expf(-z)); }

// ---------------------------------------------------------------------------------------------------- convolution + gates
constexpr int MAX_TAPS = 16;

struct ConvCols {          // where the q, k, v channels sit in a row of the projection's output
  int q_off, k_off, v_off, nq, nk, nv;       // channels of q, of k and of v
  __device__ __forceinline__ int col(int c) const { return c < nq ? q_off + c : (c < nq + nk ? k_off + (c - nq) : v_off + (c - nq - nk)); }
};

// Block per token row.  meta[row] = {slot, position}; rows of one portion are consecutive and so are their positions.
// state [slot][taps-1][C] holds the inputs of the taps - 1 positions before the portion (zero before the sequence's start).
template <typename T>
__global__ void __launch_bounds__(256) conv_prep_kernel(const T* __restrict__ y, int ld, ConvCols cc, const float* __restrict__ wconv,
                                                        const float* __restrict__ state, const int* __restrict__ meta, float* __restrict__ gates,
                                                        const float* __restrict__ a_log, const float* __restrict__ dt_bias, float* __restrict__ qk,
                                                        float* __restrict__ v, int G, int H, int dim, int vdim, int taps, float q_scale,
                                                        float unit_eps) {
  extern __shared__ float ch[];                 // C channels after convolution and SiLU
  const int row = blockIdx.x;
  const int slot = meta[2 * row], pos = meta[2 * row + 1];
  const int C = cc.nq + cc.nk + cc.nv;
  int inside = 1;                               // rows row-1 .. row-(inside-1) belong to this portion
  while (inside < taps && row - inside >= 0 && meta[2 * (row - inside)] == slot && meta[2 * (row - inside) + 1] == pos - inside) ++inside;
  const float* st = state + (size_t)slot * (taps - 1) * C;
  for (int c = threadIdx.x; c < C; c += 256) {
    const int col = cc.col(c);
    float acc = 0.f;
    for (int j = 0; j < taps; ++j) {            // j tokens back
      const float xin = j < inside ? ldf(y + (size_t)(row - j) * ld + col) : st[(size_t)(inside - 1 - j + taps - 1) * C + c];
      acc = fmaf(wconv[(size_t)c * taps + taps - 1 - j], xin, acc);
    }
    acc = silu(acc);
    ch[c] = acc;
    if (c >= cc.nq + cc.nk) v[(size_t)row * cc.nv + c - cc.nq - cc.nk] = acc;
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int hd = warp; hd < 2 * G; hd += 8) {    // q heads, then k heads
    float ss = 0.f;
    for (int i = lane; i < dim; i += 32) ss += ch[hd * dim + i] * ch[hd * dim + i];
    ss = warp_sum(ss);
    const float inv = (hd < G ? q_scale : 1.0f) / sqrtf(ss + unit_eps);
    for (int i = lane; i < dim; i += 32) qk[(size_t)row * (cc.nq + cc.nk) + hd * dim + i] = ch[hd * dim + i] * inv;
  }
  for (int h = threadIdx.x; h < H; h += 256) {
    float* gr = gates + (size_t)row * 2 * H;
    const float zb = gr[h], za = gr[H + h] + dt_bias[h];
    const float softplus = fmaxf(za, 0.f) + log1pf(expf(-fabsf(za)));
    gr[h] = 1.0f / (1.0f + expf(-zb));
    gr[H + h] = expf(-expf(a_log[h]) * softplus);
  }
}

// segs[s] = {slot, first position, first row, rows}.  Thread per channel: the new state's entry i is the input of the
// portion's token len - (taps-1) + i, or, for a portion shorter than taps - 1, entry len + i of the old state.
template <typename T>
__global__ void __launch_bounds__(256) conv_state_update_kernel(const T* __restrict__ y, int ld, ConvCols cc, float* __restrict__ state,
                                                                const int* __restrict__ segs, int taps) {
  const int seg = blockIdx.y;
  const int slot = segs[4 * seg], row0 = segs[4 * seg + 2], len = segs[4 * seg + 3];
  const int C = cc.nq + cc.nk + cc.nv;
  const int c = blockIdx.x * 256 + threadIdx.x;
  if (c >= C) return;
  float* st = state + (size_t)slot * (taps - 1) * C;
  float keep[MAX_TAPS - 1];
#pragma unroll
  for (int i = 0; i < MAX_TAPS - 1; ++i) {
    if (i < taps - 1) {
      const int t = len - (taps - 1) + i;
      keep[i] = t >= 0 ? ldf(y + (size_t)(row0 + t) * ld + cc.col(c)) : st[(size_t)(len + i) * C + c];
    }
  }
#pragma unroll
  for (int i = 0; i < MAX_TAPS - 1; ++i)
    if (i < taps - 1) st[(size_t)i * C + c] = keep[i];
}

// ---------------------------------------------------------------------------------------------------- forget gates
// What turns the q | f | v columns of a projection's output (nq = H * dim channels of q and of f, nv of v) into the FORGET
// recurrence's fp32 inputs, row by row:  q = silu(q),  f = low + (1 - low) * sigmoid(f + f_bias)  (low: the gate's lower
// bound per channel),  v as it is;  out[row] = q | f | v.
template <typename T>
__global__ void forget_gate_prep_kernel(const T* __restrict__ y, int ld, int q_off, int f_off, int v_off, const float* __restrict__ f_bias,
                                        const float* __restrict__ low, float* __restrict__ out, int M, int nq, int nv) {
  const int C = 2 * nq + nv;
  const size_t n = (size_t)M * C;
  for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (size_t)gridDim.x * blockDim.x) {
    const size_t m = e / C;
    const int c = (int)(e - m * C);
    const T* row = y + m * ld;
    float val;
    if (c < nq) {
      val = silu(ldf(row + q_off + c));
    } else if (c < 2 * nq) {
      const int i = c - nq;
      const float l = low[i];
      val = l + (1.0f - l) / (1.0f + expf(-(ldf(row + f_off + i) + (f_bias ? f_bias[i] : 0.f))));
    } else {
      val = ldf(row + v_off + (c - 2 * nq));
    }
    out[e] = val;
  }
}

// ---------------------------------------------------------------------------------------------------- the recurrence
// Stage loads return RAW bits and nothing touches them until they are stored to shared memory, so all loads of a stage are
// in flight together while the previous stage is processed.
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

// 128-bit stage load (raw bits, same reasoning) and its unpacking into VEC floats
__device__ __forceinline__ uint4 ld_raw128(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
template <typename T> struct Vec128;
template <> struct Vec128<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void unpack(uint4 v, float* f) {
    f[0] = __uint_as_float(v.x); f[1] = __uint_as_float(v.y); f[2] = __uint_as_float(v.z); f[3] = __uint_as_float(v.w);
  }
};
template <> struct Vec128<bf16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void unpack(uint4 v, float* f) {
    f[0] = __uint_as_float(v.x << 16); f[1] = __uint_as_float(v.x & 0xffff0000u);
    f[2] = __uint_as_float(v.y << 16); f[3] = __uint_as_float(v.y & 0xffff0000u);
    f[4] = __uint_as_float(v.z << 16); f[5] = __uint_as_float(v.z & 0xffff0000u);
    f[6] = __uint_as_float(v.w << 16); f[7] = __uint_as_float(v.w & 0xffff0000u);
  }
};

constexpr int TB = 8;            // tokens per stage
constexpr int CW = 2;            // columns of S per warp
constexpr int NW = 8;            // warps per block
constexpr int CB = CW * NW;      // columns per block

// VL: the stage is fetched with 128-bit loads (the host checked that every q / k / v segment of VEC numbers starts on a
// 16-byte boundary and lies wholly inside or outside its row).
// MODE: 0 DECAY, 1 DELTA, 2 FORGET (the k slot of the stage carries f_t).
template <typename T, int DR, int MODE, bool VL>
__global__ void __launch_bounds__(NW * 32, 2) linear_scan_kernel(const T* __restrict__ q, const T* __restrict__ k, int ldqk, const T* __restrict__ v, int ldv,
                                                              int in_silu, const float* __restrict__ decay, const float* __restrict__ gates,
                                                              float* __restrict__ St, const int* __restrict__ segs, int H, int G, int dim, int vdim,
                                                              float* __restrict__ o) {
  constexpr bool DELTA = MODE == 1, FORGET = MODE == 2;
  constexpr int DP = DR * 32;                    // dim padded to whole warps
  constexpr int ROWF = 2 * DP + CB + 4;          // floats of one staged token: q | k | v (this block's columns) | beta | g | 2 pad
  constexpr int VEC = Vec128<T>::N;
  constexpr int CH = (2 * DP + CB) / VEC;        // 128-bit segments of one staged token
  constexpr int NST = VL ? (TB * CH + NW * 32 - 1) / (NW * 32) : (TB * ROWF + NW * 32 - 1) / (NW * 32);
  extern __shared__ __align__(16) float stage[]; // [2][TB][ROWF]
  const int seg = blockIdx.z, h = blockIdx.y, colb = blockIdx.x * CB;
  const int hk = h / (H / G);
  const int slot = segs[4 * seg], row0 = segs[4 * seg + 2], len = segs[4 * seg + 3];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int col0 = colb + warp * CW;

  float S[DR][CW];
  float* Sp = St + ((size_t)slot * H + h) * vdim * dim;
#pragma unroll
  for (int i = 0; i < DR; ++i) {
    const int r = lane + 32 * i;
#pragma unroll
    for (int c = 0; c < CW; ++c) S[i][c] = (r < dim && col0 + c < vdim) ? Sp[(size_t)(col0 + c) * dim + r] : 0.f;
  }
  const float dec = MODE == 0 ? decay[h] : 0.f;

  typename Raw<T>::type buf[VL ? 1 : NST];
  uint4 vbuf[VL ? NST : 1];
  float gbuf = 0.f;
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
            if (j < DP) { if (j < dim) p = q + row * ldqk + hk * dim + j; }
            else if (j < 2 * DP) { if (j - DP < dim) p = k + row * ldqk + hk * dim + (j - DP); }
            else if (colb + j - 2 * DP < vdim) p = v + row * ldv + h * vdim + colb + (j - 2 * DP);
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
          if (j < dim) p = q + row * ldqk + hk * dim + j;
          else if (j >= DP && j - DP < dim) p = k + row * ldqk + hk * dim + (j - DP);
          else if (j >= 2 * DP && j < 2 * DP + CB && colb + j - 2 * DP < vdim) p = v + row * ldv + h * vdim + colb + (j - 2 * DP);
        }
      }
      buf[s] = typename Raw<T>::type(0);
      if (p != nullptr) buf[s] = Raw<T>::ld(p);
    }
    }
    if (DELTA && threadIdx.x < 2 * TB) {
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
          float f[VEC];
          Vec128<T>::unpack(vbuf[s], f);
          if (in_silu) {
#pragma unroll
            for (int i = 0; i < VEC; ++i) f[i] = silu(f[i]);
          }
          float* dst = stage + b * TB * ROWF + t * ROWF + j;
#pragma unroll
          for (int i = 0; i < VEC; i += 4) *reinterpret_cast<float4*>(dst + i) = make_float4(f[i], f[i + 1], f[i + 2], f[i + 3]);
        }
      }
    } else {
#pragma unroll
    for (int s = 0; s < NST; ++s) {
      const int e = threadIdx.x + s * NW * 32;
      if (e < TB * ROWF) {
        const int j = e % ROWF;
        if (j < 2 * DP + CB) {
          const float x = Raw<T>::to_float(buf[s]);
          stage[b * TB * ROWF + e] = in_silu ? silu(x) : x;
        }
      }
    }
    }
    if (DELTA && threadIdx.x < 2 * TB) stage[b * TB * ROWF + (threadIdx.x >> 1) * ROWF + 2 * DP + CB + (threadIdx.x & 1)] = gbuf;
  };

  const int groups = (len + TB - 1) / TB;
  fetch(0);
  put(0);
  __syncthreads();
  for (int g = 0; g < groups; ++g) {
    if (g + 1 < groups) fetch(g + 1);            // in flight while this group is processed
    const float* st = stage + (g & 1) * TB * ROWF;
    const int nt = min(TB, len - g * TB);
    for (int t = 0; t < nt; ++t) {
      const float* tk = st + t * ROWF;
      float vc[CW], out[CW];
#pragma unroll
      for (int c = 0; c < CW; ++c) vc[c] = tk[2 * DP + warp * CW + c];
      if constexpr (DELTA) {
        const float beta = tk[2 * DP + CB], gt = tk[2 * DP + CB + 1];
        float pk[CW], pq[CW], kq = 0.f;
#pragma unroll
        for (int c = 0; c < CW; ++c) pk[c] = pq[c] = 0.f;
#pragma unroll
        for (int i = 0; i < DR; ++i) {
          const float qv = tk[lane + 32 * i], kv = tk[DP + lane + 32 * i];
          kq = fmaf(kv, qv, kq);
#pragma unroll
          for (int c = 0; c < CW; ++c) {
            pk[c] = fmaf(S[i][c], kv, pk[c]);
            pq[c] = fmaf(S[i][c], qv, pq[c]);
          }
        }
        kq = warp_sum(kq);
        float u[CW];
#pragma unroll
        for (int c = 0; c < CW; ++c) {
          pk[c] = warp_sum(pk[c]);
          pq[c] = warp_sum(pq[c]);
          u[c] = beta * (vc[c] - gt * pk[c]);
          out[c] = fmaf(u[c], kq, gt * pq[c]);
        }
#pragma unroll
        for (int i = 0; i < DR; ++i) {
          const float kv = tk[DP + lane + 32 * i];
#pragma unroll
          for (int c = 0; c < CW; ++c) S[i][c] = fmaf(gt, S[i][c], kv * u[c]);
        }
      } else {
#pragma unroll
        for (int c = 0; c < CW; ++c) out[c] = 0.f;
#pragma unroll
        for (int i = 0; i < DR; ++i) {
          const float qv = tk[lane + 32 * i], kv = tk[DP + lane + 32 * i];
#pragma unroll
          for (int c = 0; c < CW; ++c) {
            if constexpr (FORGET) S[i][c] = fmaf(kv, S[i][c], (1.0f - kv) * vc[c]);     // kv is f_t here; padded rows stay unread
            else S[i][c] = fmaf(dec, S[i][c], kv * vc[c]);
            out[c] = fmaf(S[i][c], qv, out[c]);
          }
        }
#pragma unroll
        for (int c = 0; c < CW; ++c) out[c] = warp_sum(out[c]);
      }
      float mine = out[0];
#pragma unroll
      for (int c = 1; c < CW; ++c) mine = (lane == c) ? out[c] : mine;
      if (lane < CW && col0 + lane < vdim) o[(size_t)(row0 + g * TB + t) * H * vdim + h * vdim + col0 + lane] = mine;
    }
    if (g + 1 < groups) put((g + 1) & 1);        // the other buffer: last read two groups ago, before the barrier below
    __syncthreads();
  }

#pragma unroll
  for (int i = 0; i < DR; ++i) {
    const int r = lane + 32 * i;
    if (r < dim) {
#pragma unroll
      for (int c = 0; c < CW; ++c)
        if (col0 + c < vdim) Sp[(size_t)(col0 + c) * dim + r] = S[i][c];
    }
  }
}

template <typename T, int DR, int MODE, bool VL>
int launch_scan_mode(const void* q, const void* k, int ldqk, const void* v, int ldv, int in_silu, const float* decay, const float* gates, float* St,
                     const int* segs, int nseg, int H, int G, int dim, int vdim, float* o, cudaStream_t stream) {
  const size_t smem = (size_t)2 * TB * (2 * DR * 32 + CB + 4) * sizeof(float);
  dim3 grid((vdim + CB - 1) / CB, H, nseg);
  if (smem > 48 * 1024) LIA_CUDA(cudaFuncSetAttribute(linear_scan_kernel<T, DR, MODE, VL>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  linear_scan_kernel<T, DR, MODE, VL><<<grid, NW * 32, smem, stream>>>(reinterpret_cast<const T*>(q), reinterpret_cast<const T*>(k), ldqk,
                                                                       reinterpret_cast<const T*>(v), ldv, in_silu, decay, gates, St, segs, H, G, dim, vdim, o);
  LIA_LAUNCH_CHECK();
  return LIA_OK;
}

// gates given: DELTA; decay given: DECAY; neither: FORGET
template <typename T, int DR, bool VL>
int launch_scan_as(const void* q, const void* k, int ldqk, const void* v, int ldv, int in_silu, const float* decay, const float* gates, float* St,
                   const int* segs, int nseg, int H, int G, int dim, int vdim, float* o, cudaStream_t stream) {
  if (gates != nullptr) return launch_scan_mode<T, DR, 1, VL>(q, k, ldqk, v, ldv, in_silu, decay, gates, St, segs, nseg, H, G, dim, vdim, o, stream);
  if (decay != nullptr) return launch_scan_mode<T, DR, 0, VL>(q, k, ldqk, v, ldv, in_silu, decay, gates, St, segs, nseg, H, G, dim, vdim, o, stream);
  return launch_scan_mode<T, DR, 2, VL>(q, k, ldqk, v, ldv, in_silu, decay, gates, St, segs, nseg, H, G, dim, vdim, o, stream);
}

template <typename T, int DR>
int launch_scan(const void* q, const void* k, int ldqk, const void* v, int ldv, int in_silu, const float* decay, const float* gates, float* St,
                const int* segs, int nseg, int H, int G, int dim, int vdim, float* o, cudaStream_t stream) {
  constexpr int VEC = Vec128<T>::N;
  const bool aligned = ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v)) % 16 == 0) &&
                       ldqk % VEC == 0 && ldv % VEC == 0 && dim % VEC == 0 && vdim % VEC == 0;
  if (aligned) return launch_scan_as<T, DR, true>(q, k, ldqk, v, ldv, in_silu, decay, gates, St, segs, nseg, H, G, dim, vdim, o, stream);
  return launch_scan_as<T, DR, false>(q, k, ldqk, v, ldv, in_silu, decay, gates, St, segs, nseg, H, G, dim, vdim, o, stream);
}

template <typename T>
int dispatch_scan(const void* q, const void* k, int ldqk, const void* v, int ldv, int in_silu, const float* decay, const float* gates, float* St,
                  const int* segs, int nseg, int H, int G, int dim, int vdim, float* o, cudaStream_t stream) {
  if (dim <= 32) return launch_scan<T, 1>(q, k, ldqk, v, ldv, in_silu, decay, gates, St, segs, nseg, H, G, dim, vdim, o, stream);
  if (dim <= 64) return launch_scan<T, 2>(q, k, ldqk, v, ldv, in_silu, decay, gates, St, segs, nseg, H, G, dim, vdim, o, stream);
  if (dim <= 128) return launch_scan<T, 4>(q, k, ldqk, v, ldv, in_silu, decay, gates, St, segs, nseg, H, G, dim, vdim, o, stream);
  if (dim <= 256) return launch_scan<T, 8>(q, k, ldqk, v, ldv, in_silu, decay, gates, St, segs, nseg, H, G, dim, vdim, o, stream);
  return launch_scan<T, 16>(q, k, ldqk, v, ldv, in_silu, decay, gates, St, segs, nseg, H, G, dim, vdim, o, stream);
}

}  // namespace

extern "C" int lia_conv_prep(const void* y, int y_f32, int ld, int q_off, int k_off, int v_off, const float* wconv, const float* conv_state,
                             const int* meta, float* gates, const float* a_log, const float* dt_bias, float* qk, float* v, int M, int G, int H,
                             int dim, int vdim, int taps, float q_scale, float unit_eps, lia_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  LIA_CHECK_ARG(y && wconv && conv_state && meta && gates && a_log && dt_bias && qk && v, "lia_conv_prep: null pointer");
  LIA_CHECK_ARG(M > 0 && G > 0 && H > 0 && H % G == 0 && dim > 0 && vdim > 0 && taps >= 1 && taps <= MAX_TAPS, "lia_conv_prep: bad shape G=%d H=%d dim=%d vdim=%d taps=%d", G, H, dim, vdim, taps);
  ConvCols cc{q_off, k_off, v_off, G * dim, G * dim, H * vdim};
  const size_t smem = (size_t)(cc.nq + cc.nk + cc.nv) * sizeof(float);
  LIA_CHECK_ARG(smem <= 160 * 1024, "lia_conv_prep: %d channels do not fit shared memory", cc.nq + cc.nk + cc.nv);
  if (y_f32) {
    if (smem > 48 * 1024) LIA_CUDA(cudaFuncSetAttribute(conv_prep_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    conv_prep_kernel<float><<<M, 256, smem, stream>>>(reinterpret_cast<const float*>(y), ld, cc, wconv, conv_state, meta, gates, a_log, dt_bias, qk, v, G, H, dim, vdim, taps, q_scale, unit_eps);
  } else {
    if (smem > 48 * 1024) LIA_CUDA(cudaFuncSetAttribute(conv_prep_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    conv_prep_kernel<bf16><<<M, 256, smem, stream>>>(reinterpret_cast<const bf16*>(y), ld, cc, wconv, conv_state, meta, gates, a_log, dt_bias, qk, v, G, H, dim, vdim, taps, q_scale, unit_eps);
  }
  LIA_LAUNCH_CHECK();
  return LIA_OK;
}

extern "C" int lia_conv_state_update(const void* y, int y_f32, int ld, int q_off, int k_off, int v_off, int nq, int nk, int nv, float* conv_state,
                                     const int* segs, int nseg, int taps, lia_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  LIA_CHECK_ARG(y && conv_state && segs && nseg > 0 && nseg <= 65535 && nq > 0 && nk > 0 && nv > 0 && taps >= 1 && taps <= MAX_TAPS, "lia_conv_state_update: bad arguments");
  if (taps == 1) return LIA_OK;
  ConvCols cc{q_off, k_off, v_off, nq, nk, nv};
  dim3 grid((nq + nk + nv + 255) / 256, nseg);
  if (y_f32) conv_state_update_kernel<float><<<grid, 256, 0, stream>>>(reinterpret_cast<const float*>(y), ld, cc, conv_state, segs, taps);
  else conv_state_update_kernel<bf16><<<grid, 256, 0, stream>>>(reinterpret_cast<const bf16*>(y), ld, cc, conv_state, segs, taps);
  LIA_LAUNCH_CHECK();
  return LIA_OK;
}

// gates == NULL: the DECAY recurrence with decay[H]; otherwise DELTA with gates[rows][2H] = beta | g.
extern "C" int lia_linear_scan(const void* q, const void* k, int ldqk, const void* v, int ldv, int act_f32, int in_silu, const float* decay,
                               const float* gates, float* state_S, const int* segs, int nseg, int H, int G, int dim, int vdim, float* o,
                               lia_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  LIA_CHECK_ARG(q && k && v && state_S && segs && o && (decay || gates), "lia_linear_scan: null pointer");
  LIA_CHECK_ARG(nseg > 0 && nseg <= 65535 && H > 0 && H <= 65535 && G > 0 && H % G == 0 && dim > 0 && dim <= 512 && vdim > 0,
                "lia_linear_scan: bad shape nseg=%d H=%d G=%d dim=%d vdim=%d", nseg, H, G, dim, vdim);
  if (act_f32) return dispatch_scan<float>(q, k, ldqk, v, ldv, in_silu, decay, gates, state_S, segs, nseg, H, G, dim, vdim, o, stream);
  return dispatch_scan<bf16>(q, k, ldqk, v, ldv, in_silu, decay, gates, state_S, segs, nseg, H, G, dim, vdim, o, stream);
}

extern "C" int lia_forget_gate_prep(const void* y, int y_f32, int ld, int q_off, int f_off, int v_off, const float* f_bias, const float* low,
                                    float* out, int M, int nq, int nv, lia_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  LIA_CHECK_ARG(y && low && out && M > 0 && nq > 0 && nv > 0 && ld >= nq && q_off >= 0 && f_off >= 0 && v_off >= 0, "lia_forget_gate_prep: bad arguments");
  const size_t n = (size_t)M * (2 * nq + nv);
  size_t blocks = (n + 255) / 256;
  const size_t capb = (size_t)lia_sm_count() * 16;
  if (blocks > capb) blocks = capb;
  if (y_f32) forget_gate_prep_kernel<float><<<(unsigned)blocks, 256, 0, stream>>>(reinterpret_cast<const float*>(y), ld, q_off, f_off, v_off, f_bias, low, out, M, nq, nv);
  else forget_gate_prep_kernel<bf16><<<(unsigned)blocks, 256, 0, stream>>>(reinterpret_cast<const bf16*>(y), ld, q_off, f_off, v_off, f_bias, low, out, M, nq, nv);
  LIA_LAUNCH_CHECK();
  return LIA_OK;
}

// The FORGET recurrence: q, f fp32 column slices with one row stride (H heads of dim), v fp32 (H heads of vdim).
extern "C" int lia_forget_scan(const float* q, const float* f, int ldqf, const float* v, int ldv, float* state_S, const int* segs, int nseg, int H,
                               int dim, int vdim, float* o, lia_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  LIA_CHECK_ARG(q && f && v && state_S && segs && o, "lia_forget_scan: null pointer");
  LIA_CHECK_ARG(nseg > 0 && nseg <= 65535 && H > 0 && H <= 65535 && dim > 0 && dim <= 512 && vdim > 0,
                "lia_forget_scan: bad shape nseg=%d H=%d dim=%d vdim=%d", nseg, H, dim, vdim);
  return dispatch_scan<float>(q, f, ldqf, v, ldv, 0, nullptr, nullptr, state_S, segs, nseg, H, H, dim, vdim, o, stream);
}
