// Softmax attention over a sliding window of cached keys and values (or over the whole history), with grouped key/value
// heads, a per-head temperature, a tanh soft cap on the scores, a per-head distance bias, a per-head sink in the softmax's
// denominator and an output gate; the kernel itself rotates nothing (a caller that wants rotated queries and keys hands
// them in rotated).
//
//   kv_store:     the new tokens' keys go into the key cache as they are; each value head is divided by its root mean square
//                 (fp32) and cached so.
//   window_attn:  one block per (group of token rows, group of up to 8 query heads, range of keys); a warp owns (row, head)
//                 pairs.  32 cached positions at a time are staged in shared memory as fp32 for the key/value heads the
//                 block's query heads use, once for all rows of the block that continue one sequence; lane j scores key j,
//                     s = cap * tanh((q . k) * scale * temp_h / cap) - slopes[h] * (pos - j)     (cap <= 0: no cap)
//                 over the positions j with 0 <= pos - j < window, folds the stage into a running softmax and accumulates the
//                 values (lane l owns channels l, l + 32, ...).  A sink adds exp(sink[h]) to the softmax's denominator, a term
//                 without key or value.  The output can be multiplied by a gate, one number per (row, head) or sigmoid of
//                 one pre-activation per channel.  Scores, weights and sums are fp32; the queries may be fp32 while the
//                 caches are bf16.  Few rows and a long window (decoding): the keys are split over several blocks and a
//                 second kernel combines.
//   qkv_prep:     what turns a projection's q | k | v columns into attention inputs, per token: bias, a short causal
//                 convolution along the sequence per channel, an RMS norm of q and of k (over the whole projection or per head), a
//                 position-dependent query temperature, a rotation of channel pairs, a blend of the values with the values
//                 that an earlier layer published for the same token; q goes out in fp32, k and v into the caches.
#include <math.h>

#include "common.cuh"

namespace {

template <typename T> __device__ __forceinline__ float ldf(const T* p);
template <> __device__ __forceinline__ float ldf<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ldf<bf16>(const bf16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void stf(T* p, float v);
template <> __device__ __forceinline__ void stf<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void stf<bf16>(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

// meta[row] = {slot, position}.  Block per row, warp per value head in turn.
template <typename T>
__global__ void __launch_bounds__(128) kv_store_kernel(const T* __restrict__ k, int ldk, const T* __restrict__ v, int ldv, const int* __restrict__ meta,
                                                       T* __restrict__ kcache, long long k_slot_stride, T* __restrict__ vcache, long long v_slot_stride,
                                                       int G, int dim, int vdim, float eps, int norm_values) {
  const int row = blockIdx.x;
  const int slot = meta[2 * row], pos = meta[2 * row + 1];
  T* kr = kcache + (size_t)slot * k_slot_stride + (size_t)pos * G * dim;
  T* vr = vcache + (size_t)slot * v_slot_stride + (size_t)pos * G * vdim;
  for (int i = threadIdx.x; i < G * dim; i += 128) kr[i] = k[(size_t)row * ldk + i];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int g = warp; g < G; g += 4) {
    const T* src = v + (size_t)row * ldv + g * vdim;
    float inv = 1.0f;
    if (norm_values) {
      float ss = 0.f;
      for (int c = lane; c < vdim; c += 32) {
        const float x = ldf(src + c);
        ss += x * x;
      }
      inv = 1.0f / sqrtf(warp_sum(ss) / (float)vdim + eps);
    }
    for (int c = lane; c < vdim; c += 32) stf(vr + g * vdim + c, ldf(src + c) * inv);
  }
}


// ---------------------------------------------------------------------------------------------------- attention inputs
struct PrepArgs {
  int H, G, dim, vdim;
  int q_off, k_off, v_off;       // columns of q | k | v in a row of the projection's output
  int taps;                      // of the convolution, if it has weights
  int norm_mode;                 // 0 none; 1 one RMS norm over all of q (and all of k), weights [H*dim], [G*dim]; 2 per head, weights [dim]
  int temp_every;                // > 0: q *= 1 + temp_coef * ln(floor((pos + 1) / temp_every) + 1)
  int rot_dims, rot_halves;      // channels (2i, 2i+1), i < rot_dims/2, of every head turn by pos * freq[i]; rot_halves != 0: pairs (i, i + rot_dims/2)
  int vmix_mode;                 // 0 none; 1 publish v into v_first; 2 v += lambda (v_first - v)
  float eps, temp_coef, rot_mag, lambda;
  int Gv = 0;                    // value heads (0: as many as key heads)
};

// Block per token row; meta[row] = {slot, position}; rows of one portion are consecutive and so are their positions.
// conv_state [slot][taps-1][C] holds the projection's outputs (without bias) of the taps - 1 positions before the portion;
// what lies before the sequence's start counts as zero (no bias either).
template <typename T>
__global__ void __launch_bounds__(256) qkv_prep_kernel(const T* __restrict__ y, int ld, const float* __restrict__ bias, const float* __restrict__ wconv,
                                                       const float* __restrict__ conv_state, const float* __restrict__ qnorm_w,
                                                       const float* __restrict__ knorm_w, const double* __restrict__ freq, const int* __restrict__ meta,
                                                       float* __restrict__ v_first, float* __restrict__ q_out, T* __restrict__ kcache,
                                                       long long k_slot_stride, T* __restrict__ vcache, long long v_slot_stride, PrepArgs a) {
  extern __shared__ float ch[];                 // C channels q | k | v, then cos | sin of the rotation's pairs
  __shared__ float red[8];
  const int row = blockIdx.x;
  const int slot = meta[2 * row], pos = meta[2 * row + 1];
  const int nq = a.H * a.dim, nk = a.G * a.dim, nv = (a.Gv > 0 ? a.Gv : a.G) * a.vdim, C = nq + nk + nv;
  float* cs = ch + C;
  const int npair = a.rot_dims / 2;
  for (int i = threadIdx.x; i < npair; i += 256) {
    double s, c;
    sincos((double)pos * freq[i], &s, &c);      // the angle in full: positions in the thousands times an irrational frequency
    cs[i] = (float)c * a.rot_mag;
    cs[npair + i] = (float)s * a.rot_mag;
  }
  int inside = 1;                               // rows row-1 .. row-(inside-1) belong to this portion
  while (inside < a.taps && row - inside >= 0 && meta[2 * (row - inside)] == slot && meta[2 * (row - inside) + 1] == pos - inside) ++inside;
  const float* st = conv_state ? conv_state + (size_t)slot * (a.taps - 1) * C : nullptr;
  for (int c = threadIdx.x; c < C; c += 256) {
    const int col = c < nq ? a.q_off + c : (c < nq + nk ? a.k_off + (c - nq) : a.v_off + (c - nq - nk));
    const float b = bias ? bias[c] : 0.f;
    float acc;
    if (wconv != nullptr) {
      acc = 0.f;
      for (int j = 0; j < a.taps && j <= pos; ++j) {          // j tokens back
        const float xin = j < inside ? ldf(y + (size_t)(row - j) * ld + col) : st[(size_t)(inside - 1 - j + a.taps - 1) * C + c];
        acc = fmaf(wconv[(size_t)c * a.taps + a.taps - 1 - j], xin + b, acc);
      }
    } else {
      acc = ldf(y + (size_t)row * ld + col) + b;
    }
    ch[c] = acc;
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float temp = 1.0f;
  if (a.temp_every > 0) temp = 1.0f + a.temp_coef * logf((float)((pos + 1) / a.temp_every) + 1.0f);
  if (a.norm_mode == 1) {
    float sq = 0.f, sk = 0.f;
    for (int c = threadIdx.x; c < nq; c += 256) sq += ch[c] * ch[c];
    for (int c = nq + threadIdx.x; c < nq + nk; c += 256) sk += ch[c] * ch[c];
    sq = warp_sum(sq);
    sk = warp_sum(sk);
    if (lane == 0) red[warp] = sq;
    __syncthreads();
    float tq = 0.f;
    for (int w = 0; w < 8; ++w) tq += red[w];
    __syncthreads();
    if (lane == 0) red[warp] = sk;
    __syncthreads();
    float tk = 0.f;
    for (int w = 0; w < 8; ++w) tk += red[w];
    const float iq = temp / sqrtf(tq / (float)nq + a.eps), ik = 1.0f / sqrtf(tk / (float)nk + a.eps);
    for (int c = threadIdx.x; c < nq; c += 256) ch[c] *= iq * qnorm_w[c];
    for (int c = threadIdx.x; c < nk; c += 256) ch[nq + c] *= ik * knorm_w[c];
  } else {
    for (int hd = warp; hd < a.H + a.G; hd += 8) {            // q heads, then k heads
      float* hv = ch + hd * a.dim;
      const bool is_q = hd < a.H;
      float inv = is_q ? temp : 1.0f;
      if (a.norm_mode == 2) {
        float ss = 0.f;
        for (int i = lane; i < a.dim; i += 32) ss += hv[i] * hv[i];
        inv /= sqrtf(warp_sum(ss) / (float)a.dim + a.eps);
      }
      const float* w = a.norm_mode == 2 ? (is_q ? qnorm_w : knorm_w) : nullptr;
      for (int i = lane; i < a.dim; i += 32) hv[i] *= inv * (w ? w[i] : 1.0f);
    }
  }
  __syncthreads();
  // rotation and the way out: q in fp32, k into the cache
  T* kr = kcache + (size_t)slot * k_slot_stride + (size_t)pos * nk;
  for (int e = threadIdx.x; e < nq + nk; e += 256) {
    const int hd = e / a.dim, i = e - hd * a.dim;
    float val = ch[e];
    if (i < a.rot_dims) {
      int p, mate;
      bool first;
      if (a.rot_halves) { first = i < npair; p = first ? i : i - npair; mate = first ? i + npair : i - npair; }
      else { first = (i & 1) == 0; p = i >> 1; mate = i ^ 1; }
      const float other = ch[hd * a.dim + mate];
      val = first ? val * cs[p] - other * cs[npair + p] : val * cs[p] + other * cs[npair + p];
    }
    if (e < nq) q_out[(size_t)row * nq + e] = val;
    else stf(kr + (e - nq), val);
  }
  T* vr = vcache + (size_t)slot * v_slot_stride + (size_t)pos * nv;
  for (int c = threadIdx.x; c < nv; c += 256) {
    float val = ch[nq + nk + c];
    if (a.vmix_mode == 1) v_first[(size_t)row * nv + c] = val;
    else if (a.vmix_mode == 2) val = (1.0f - a.lambda) * val + a.lambda * v_first[(size_t)row * nv + c];
    stf(vr + c, val);
  }
}

constexpr int TK = 32;     // cached positions per stage (= lanes: lane j scores key j)
constexpr int NWARP = 8;

struct WindowArgs {
  int H, G, dim, vdim, window;
  int HB, NG, QR, nsplit;      // query heads per block (spanning at most NG key/value heads), rows per block, key ranges per row
  float scale, softcap;
  int q_f32, gate_mode, ldg;   // queries in fp32; gate: 0 none, 1 fp32 [M][H] as is, 2 sigmoid of the activations' type [M][ldg], per channel
  int chunk = 0;               // > 0: a position sees only the keys of its own block of `chunk` positions (counted from the sequence's start)
  int v_div = 1;               // key head g reads value head g / v_div (the value cache holds G / v_div heads)
  int out_f32 = 0;             // the output in fp32 whatever the caches hold
};

// first position a query at `pos` sees: the window's start, and the start of its chunk if the mask is chunked
__device__ __forceinline__ int first_key(const WindowArgs& a, int pos) {
  int lo = max(0, pos - a.window + 1);
  if (a.chunk > 0) lo = max(lo, pos - pos % a.chunk);
  return lo;
}

// the output in the caches' type or, `out_f32`, in fp32
template <typename T>
__device__ __forceinline__ void store_out(T* out, size_t at, float v, const WindowArgs& a) {
  if (a.out_f32) reinterpret_cast<float*>(out)[at] = v;
  else stf(out + at, v);
}

// what the scores and the output take besides q, k, v (each may be null)
struct WindowExtras {
  const float* temp;     // [H] multiplies the scaled score
  const float* slopes;   // [H] slopes[h] * (pos - j) is taken off the score
  const float* sink;     // [H] exp(sink_h) joins the softmax's denominator
  const void* gate;      // see WindowArgs::gate_mode
};

template <typename T>
__device__ __forceinline__ float gate_of(const WindowExtras& x, const WindowArgs& a, size_t row, int h, int ch) {
  if (a.gate_mode == 1) return reinterpret_cast<const float*>(x.gate)[row * a.H + h];
  if (a.gate_mode == 2) return 1.0f / (1.0f + expf(-ldf(reinterpret_cast<const T*>(x.gate) + row * a.ldg + (size_t)h * a.vdim + ch)));
  return 1.0f;
}

__host__ __device__ inline int key_stride(int dim) { return dim % 4 == 0 ? dim + 4 : (dim | 1); }   // conflict-free rows (128-bit or scalar reads)

template <typename T> struct Vec { static constexpr int N = 8; };
template <> struct Vec<float> { static constexpr int N = 4; };
__device__ __forceinline__ void load_vec(const bf16* p, float* f) { unpack8(*reinterpret_cast<const uint4*>(p), f); }
__device__ __forceinline__ void load_vec(const float* p, float* f) {
  const float4 v = *reinterpret_cast<const float4*>(p);
  f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
}

// rows [n][G][width] of a cache -> shared memory [ng][TK][stride] as fp32, positions j0 .. j0+nk-1 (zeros behind them)
template <typename T>
__device__ __forceinline__ void stage_rows(const T* __restrict__ cache, int G, int width, int g_lo, int ng, int j0, int nk, float* dst, int stride,
                                           bool vec) {
  constexpr int VEC = Vec<T>::N;
  if (vec) {
    const int per_row = width / VEC, total = ng * TK * per_row;
    for (int e = threadIdx.x; e < total; e += NWARP * 32) {
      const int g = e / (TK * per_row), r = e - g * TK * per_row;
      const int j = r / per_row, c = (r - j * per_row) * VEC;
      float f[VEC];
      if (j < nk) {
        load_vec(cache + ((size_t)(j0 + j) * G + g_lo + g) * width + c, f);
      } else {
#pragma unroll
        for (int i = 0; i < VEC; ++i) f[i] = 0.f;
      }
      float* d = dst + (g * TK + j) * stride + c;
#pragma unroll
      for (int i = 0; i < VEC; i += 4) *reinterpret_cast<float4*>(d + i) = make_float4(f[i], f[i + 1], f[i + 2], f[i + 3]);
    }
  } else {
    const int total = ng * TK * width;
    for (int e = threadIdx.x; e < total; e += NWARP * 32) {
      const int g = e / (TK * width), r = e - g * TK * width;
      const int j = r / width, c = r - j * width;
      dst[(g * TK + j) * stride + c] = j < nk ? ldf(cache + ((size_t)(j0 + j) * G + g_lo + g) * width + c) : 0.f;
    }
  }
}

// One block: rows [blockIdx.x * QR, + QR) of the step, query heads [blockIdx.y * HB, + HB), the blockIdx.z-th part of the keys.
// Rows that continue one sequence (same slot, consecutive positions) form a run and share the staged keys and values; a block
// whose rows belong to several sequences takes the runs one after the other.  A (row, head) pair belongs to one warp, which
// keeps its running maximum, sum and value accumulators (lane l: channels l, l + 32, ...) in registers; PP pairs per warp.
// nsplit > 1: unnormalised sums to `part` [M][H][nsplit][vdim] and (max, sum) to `part_ml`; window_combine_kernel finishes.
template <typename T, int VR, int PP>
__global__ void __launch_bounds__(NWARP * 32) window_attn_kernel(const void* __restrict__ q, int ldq, const T* __restrict__ kcache, long long k_slot_stride,
                                                                const T* __restrict__ vcache, long long v_slot_stride, const int* __restrict__ meta,
                                                                WindowExtras x, T* __restrict__ out, float* __restrict__ part,
                                                                float2* __restrict__ part_ml, int M, WindowArgs a) {
  extern __shared__ __align__(16) float sm[];
  const int DKS = key_stride(a.dim);
  float* qs = sm;                                             // [QR * HB][dim]
  float* ks = qs + (a.QR * a.HB * a.dim + 3) / 4 * 4;         // [NG][TK][DKS]
  float* vs = ks + a.NG * TK * DKS;                           // [NG][TK][vdim]
  const int r_begin = blockIdx.x * a.QR, r_end = min(M, r_begin + a.QR);
  const int h0 = blockIdx.y * a.HB, z = blockIdx.z;
  const int nh = min(a.HB, a.H - h0), rep = a.H / a.G;
  const int g_lo = h0 / rep, ng = (h0 + nh - 1) / rep - g_lo + 1;
  const int gv_lo = g_lo / a.v_div, ngv = (g_lo + ng - 1) / a.v_div - gv_lo + 1;      // the value heads behind those key heads
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int VEC = Vec<T>::N;
  const bool aligned = reinterpret_cast<uintptr_t>(kcache) % 16 == 0 && reinterpret_cast<uintptr_t>(vcache) % 16 == 0 &&
                       k_slot_stride % VEC == 0 && v_slot_stride % VEC == 0;
  const bool vec_k = aligned && a.dim % VEC == 0 && a.dim % 4 == 0, vec_v = aligned && a.vdim % VEC == 0;
  const bool dot4 = a.dim % 4 == 0;
  const bool same_head = NWARP % nh == 0 && PP > 1;           // pair p = warp + 8 s belongs to head p % nh = warp % nh for every s

  int r = r_begin;
  while (r < r_end) {
    const int slot = meta[2 * r], pos_first = meta[2 * r + 1];
    int re = r + 1;
    while (re < r_end && meta[2 * re] == slot && meta[2 * re + 1] == pos_first + (re - r)) ++re;
    const int nrun = re - r, npairs = nrun * nh, pos_last = pos_first + nrun - 1;
    const T* kc = kcache + (size_t)slot * k_slot_stride;
    const T* vc = vcache + (size_t)slot * v_slot_stride;
    __syncthreads();                                          // the previous run's queries and stage are no longer read
    for (int e = threadIdx.x; e < npairs * a.dim; e += NWARP * 32) {
      const int p = e / a.dim, d = e - p * a.dim;
      const int i = p / nh, hh = p - i * nh;
      const size_t at = (size_t)(r + i) * ldq + (size_t)(h0 + hh) * a.dim + d;
      qs[e] = a.q_f32 ? reinterpret_cast<const float*>(q)[at] : ldf(reinterpret_cast<const T*>(q) + at);
    }
    float m_run[PP], l_run[PP], acc[PP][VR];
#pragma unroll
    for (int s = 0; s < PP; ++s) {
      m_run[s] = -INFINITY;
      l_run[s] = 0.f;
#pragma unroll
      for (int i = 0; i < VR; ++i) acc[s][i] = 0.f;
    }
    const int jb = first_key(a, pos_first);                 // the first key any row of the run sees (first_key grows with pos)
    const int ntiles = (pos_last - jb) / TK + 1, per = (ntiles + a.nsplit - 1) / a.nsplit;
    const int t_end = min(ntiles, (z + 1) * per);
    for (int t = z * per; t < t_end; ++t) {
      const int j0 = jb + t * TK, nk = min(TK, pos_last + 1 - j0);
      __syncthreads();                                        // previous stage fully consumed (and qs written, first time)
      stage_rows(kc, a.G, a.dim, g_lo, ng, j0, nk, ks, DKS, vec_k);
      stage_rows(vc, a.G / a.v_div, a.vdim, gv_lo, ngv, j0, nk, vs, a.vdim, vec_v);
      __syncthreads();
      if (same_head) {
        // All pairs of this warp are rows of ONE query head (nh divides the warp count): a staged key or value row is read
        // from shared memory once and serves the PP rows.
        const int hh = warp % nh, h = h0 + hh, gi = h / rep - g_lo;
        const float sc_mul = a.scale * (x.temp ? x.temp[h] : 1.0f);
        const float slope = x.slopes ? x.slopes[h] : 0.f;
        bool active[PP];
        int lo_min = 0x7fffffff, pos_max = -1;
#pragma unroll
        for (int s = 0; s < PP; ++s) {
          const int p = warp + NWARP * s;
          const int pos = pos_first + p / nh, lo = first_key(a, pos);
          active[s] = p < npairs && j0 <= pos && j0 + nk - 1 >= lo;
          if (active[s]) {
            lo_min = min(lo_min, lo);
            pos_max = max(pos_max, pos);
          }
        }
        if (pos_max >= 0) {
          float dot[PP];
#pragma unroll
          for (int s = 0; s < PP; ++s) dot[s] = 0.f;
          const float* kr = ks + (gi * TK + lane) * DKS;
          if (dot4) {
            const float4* k4 = reinterpret_cast<const float4*>(kr);
            for (int d = 0; d < a.dim / 4; ++d) {
              const float4 y = k4[d];
#pragma unroll
              for (int s = 0; s < PP; ++s) {
                const float4 x = reinterpret_cast<const float4*>(qs + (warp + NWARP * s) * a.dim)[d];
                dot[s] = fmaf(x.x, y.x, fmaf(x.y, y.y, fmaf(x.z, y.z, fmaf(x.w, y.w, dot[s]))));
              }
            }
          } else {
            for (int d = 0; d < a.dim; ++d) {
              const float y = kr[d];
#pragma unroll
              for (int s = 0; s < PP; ++s) dot[s] = fmaf(qs[(warp + NWARP * s) * a.dim + d], y, dot[s]);
            }
          }
          float pr[PP];
#pragma unroll
          for (int s = 0; s < PP; ++s) {
            pr[s] = 0.f;
            if (!active[s]) continue;                         // warp-uniform
            const int pos = pos_first + (warp + NWARP * s) / nh, lo = first_key(a, pos);
            float sc = dot[s] * sc_mul;
            if (a.softcap > 0.f) sc = a.softcap * tanhf(sc / a.softcap);
            const int j = j0 + lane;
            sc -= slope * (float)(pos - j);
            if (lane >= nk || j < lo || j > pos) sc = -INFINITY;
            const float m_new = fmaxf(m_run[s], warp_max(sc));  // finite: at least one key of the stage is visible
            pr[s] = expf(sc - m_new);
            const float al = expf(m_run[s] - m_new);
            l_run[s] = l_run[s] * al + warp_sum(pr[s]);
            m_run[s] = m_new;
#pragma unroll
            for (int c = 0; c < VR; ++c) acc[s][c] *= al;
          }
          const float* vr = vs + ((gi + g_lo) / a.v_div - gv_lo) * TK * a.vdim;
          const int jj_end = min(nk - 1, pos_max - j0);
          for (int jj = max(0, lo_min - j0); jj <= jj_end; ++jj) {
            float vv[VR];
#pragma unroll
            for (int c = 0; c < VR; ++c) {
              const int ch = lane + 32 * c;
              vv[c] = ch < a.vdim ? vr[jj * a.vdim + ch] : 0.f;
            }
#pragma unroll
            for (int s = 0; s < PP; ++s) {
              const float pw = __shfl_sync(0xffffffffu, pr[s], jj);   // 0 for a row that does not see key jj
#pragma unroll
              for (int c = 0; c < VR; ++c) acc[s][c] = fmaf(pw, vv[c], acc[s][c]);
            }
          }
        }
        continue;
      }
#pragma unroll
      for (int s = 0; s < PP; ++s) {
        const int p = warp + NWARP * s;
        if (p >= npairs) continue;
        const int i = p / nh, hh = p - i * nh;
        const int pos = pos_first + i, lo = first_key(a, pos);
        if (j0 > pos || j0 + nk - 1 < lo) continue;          // no key of this stage is visible to the row (warp-uniform)
        const int h = h0 + hh, gi = h / rep - g_lo;
        const float* kr = ks + (gi * TK + lane) * DKS;
        const float* qr = qs + p * a.dim;
        float dot = 0.f;
        if (dot4) {
          const float4* k4 = reinterpret_cast<const float4*>(kr);
          const float4* q4 = reinterpret_cast<const float4*>(qr);
          for (int d = 0; d < a.dim / 4; ++d) {
            const float4 x = q4[d], y = k4[d];
            dot = fmaf(x.x, y.x, fmaf(x.y, y.y, fmaf(x.z, y.z, fmaf(x.w, y.w, dot))));
          }
        } else {
          for (int d = 0; d < a.dim; ++d) dot = fmaf(qr[d], kr[d], dot);
        }
        float sc = dot * a.scale * (x.temp ? x.temp[h] : 1.0f);
        if (a.softcap > 0.f) sc = a.softcap * tanhf(sc / a.softcap);
        const int j = j0 + lane;
        if (x.slopes) sc -= x.slopes[h] * (float)(pos - j);
        if (lane >= nk || j < lo || j > pos) sc = -INFINITY;
        const float m_new = fmaxf(m_run[s], warp_max(sc));      // finite: at least one key of the stage is visible
        const float pr = expf(sc - m_new);
        const float al = expf(m_run[s] - m_new);
        l_run[s] = l_run[s] * al + warp_sum(pr);
        m_run[s] = m_new;
#pragma unroll
        for (int c = 0; c < VR; ++c) acc[s][c] *= al;
        const float* vr = vs + ((gi + g_lo) / a.v_div - gv_lo) * TK * a.vdim;
        const int jj_end = min(nk - 1, pos - j0);
        for (int jj = max(0, lo - j0); jj <= jj_end; ++jj) {
          const float pw = __shfl_sync(0xffffffffu, pr, jj);
#pragma unroll
          for (int c = 0; c < VR; ++c) {
            const int ch = lane + 32 * c;
            if (ch < a.vdim) acc[s][c] = fmaf(pw, vr[jj * a.vdim + ch], acc[s][c]);
          }
        }
      }
    }
#pragma unroll
    for (int s = 0; s < PP; ++s) {
      const int p = warp + NWARP * s;
      if (p >= npairs) continue;
      const int i = p / nh, hh = p - i * nh;
      const size_t rh = (size_t)(r + i) * a.H + h0 + hh;
      if (a.nsplit == 1) {
        const float invl = 1.0f / (l_run[s] + (x.sink ? expf(x.sink[h0 + hh] - m_run[s]) : 0.f));
#pragma unroll
        for (int c = 0; c < VR; ++c) {
          const int ch = lane + 32 * c;
          if (ch < a.vdim) store_out(out, rh * a.vdim + ch, acc[s][c] * invl * gate_of<T>(x, a, (size_t)(r + i), h0 + hh, ch), a);
        }
      } else {
#pragma unroll
        for (int c = 0; c < VR; ++c) {
          const int ch = lane + 32 * c;
          if (ch < a.vdim) part[(rh * a.nsplit + z) * a.vdim + ch] = acc[s][c];
        }
        if (lane == 0) part_ml[rh * a.nsplit + z] = make_float2(m_run[s], l_run[s]);
      }
    }
    r = re;
  }
}

// out[rh] = sum_z part[rh][z] e^(m_z - m) / sum_z l_z e^(m_z - m), m = max_z m_z (a part without visible keys has m = -inf, l = 0)
template <typename T>
__global__ void __launch_bounds__(128) window_combine_kernel(const float* __restrict__ part, const float2* __restrict__ part_ml, T* __restrict__ out,
                                                             int vdim, int nsplit, WindowExtras x, WindowArgs a) {
  const size_t rh = blockIdx.x;
  const int h = (int)(rh % a.H);
  const size_t row = rh / a.H;
  float m = -INFINITY;
  for (int z = 0; z < nsplit; ++z) m = fmaxf(m, part_ml[rh * nsplit + z].x);
  float l = 0.f;
  for (int z = 0; z < nsplit; ++z) {
    const float2 ml = part_ml[rh * nsplit + z];
    if (ml.y > 0.f) l += ml.y * expf(ml.x - m);
  }
  if (x.sink) l += expf(x.sink[h] - m);
  const float invl = 1.0f / l;
  for (int c = threadIdx.x; c < vdim; c += 128) {
    float s = 0.f;
    for (int z = 0; z < nsplit; ++z) {
      const float2 ml = part_ml[rh * nsplit + z];
      if (ml.y > 0.f) s = fmaf(part[(rh * nsplit + z) * vdim + c], expf(ml.x - m), s);
    }
    store_out(out, rh * vdim + c, s * invl * gate_of<T>(x, a, row, h, c), a);
  }
}

// Differential attention's last step.  `a` [M][G][2][rep][vdim] fp32 holds both maps' outputs (the query heads of key/value
// group g side by side, map 1 then map 2); head h = g * rep + r of the result is
//     o = a1 - lambda * a2,   out = mult * o / rms(o),   rms taken (with eps under the root) over that head's vdim entries.
// One warp per (row, head).
template <typename T>
__global__ void __launch_bounds__(128) diff_combine_kernel(const float* __restrict__ a, T* __restrict__ out, int M, int H, int G, int vdim,
                                                           float lambda, float mult, float eps) {
  const long long pair = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (pair >= (long long)M * H) return;
  const size_t row = pair / H;
  const int h = (int)(pair - row * H), rep = H / G, g = h / rep, r = h - g * rep;
  const float* a1 = a + (row * 2 * H + (size_t)(g * 2) * rep + r) * vdim;
  const float* a2 = a1 + (size_t)rep * vdim;
  float ss = 0.f;
  for (int c = lane; c < vdim; c += 32) {
    const float o = a1[c] - lambda * a2[c];
    ss += o * o;
  }
  const float inv = mult / sqrtf(warp_sum(ss) / (float)vdim + eps);
  for (int c = lane; c < vdim; c += 32) stf(out + (row * H + h) * vdim + c, (a1[c] - lambda * a2[c]) * inv);
}

size_t attn_smem(const WindowArgs& a) {
  return ((size_t)(a.QR * a.HB * a.dim + 3) / 4 * 4 + (size_t)a.NG * TK * (key_stride(a.dim) + a.vdim)) * sizeof(float);
}

template <typename T, int VR, int PP>
int launch_attn(const void* q, int ldq, const void* kcache, long long kss, const void* vcache, long long vss, const int* meta, const WindowExtras& x,
                void* out, float* ws, int M, const WindowArgs& a, cudaStream_t stream) {
  LIA_CHECK_ARG((a.QR * a.HB + NWARP - 1) / NWARP <= PP, "lia_window_attn: %d rows x %d heads per block are too many for value heads of %d", a.QR, a.HB, a.vdim);
  const size_t smem = attn_smem(a);
  if (smem > 48 * 1024) LIA_CUDA(cudaFuncSetAttribute(window_attn_kernel<T, VR, PP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  dim3 grid((M + a.QR - 1) / a.QR, (a.H + a.HB - 1) / a.HB, a.nsplit);
  float* part = ws;
  float2* part_ml = reinterpret_cast<float2*>(ws + (size_t)M * a.H * a.nsplit * a.vdim);
  window_attn_kernel<T, VR, PP><<<grid, NWARP * 32, smem, stream>>>(q, ldq, reinterpret_cast<const T*>(kcache), kss,
                                                                   reinterpret_cast<const T*>(vcache), vss, meta, x, reinterpret_cast<T*>(out), part,
                                                                   part_ml, M, a);
  LIA_LAUNCH_CHECK();
  if (a.nsplit > 1) {
    window_combine_kernel<T><<<(unsigned)((size_t)M * a.H), 128, 0, stream>>>(part, part_ml, reinterpret_cast<T*>(out), a.vdim, a.nsplit, x, a);
    LIA_LAUNCH_CHECK();
  }
  return LIA_OK;
}

template <typename T>
int dispatch_attn(const void* q, int ldq, const void* kcache, long long kss, const void* vcache, long long vss, const int* meta, const WindowExtras& temp,
                  void* out, float* ws, int M, const WindowArgs& a, cudaStream_t stream) {
  if (a.vdim <= 32) return launch_attn<T, 1, 4>(q, ldq, kcache, kss, vcache, vss, meta, temp, out, ws, M, a, stream);
  if (a.vdim <= 64) return launch_attn<T, 2, 4>(q, ldq, kcache, kss, vcache, vss, meta, temp, out, ws, M, a, stream);
  if (a.vdim <= 128) return launch_attn<T, 4, 4>(q, ldq, kcache, kss, vcache, vss, meta, temp, out, ws, M, a, stream);
  if (a.vdim <= 256) return launch_attn<T, 8, 2>(q, ldq, kcache, kss, vcache, vss, meta, temp, out, ws, M, a, stream);
  return launch_attn<T, 16, 1>(q, ldq, kcache, kss, vcache, vss, meta, temp, out, ws, M, a, stream);
}

}  // namespace

extern "C" int lia_kv_store(const void* k, int ldk, const void* v, int ldv, int act_f32, const int* meta, void* kcache, long long k_slot_stride,
                            void* vcache, long long v_slot_stride, int M, int G, int dim, int vdim, float eps, int norm_values,
                            lia_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  LIA_CHECK_ARG(k && v && meta && kcache && vcache && M > 0 && G > 0 && dim > 0 && vdim > 0 && ldk >= G * dim && ldv >= G * vdim, "lia_kv_store: bad arguments");
  if (act_f32)
    kv_store_kernel<float><<<M, 128, 0, stream>>>(reinterpret_cast<const float*>(k), ldk, reinterpret_cast<const float*>(v), ldv, meta,
                                                  reinterpret_cast<float*>(kcache), k_slot_stride, reinterpret_cast<float*>(vcache), v_slot_stride, G, dim, vdim, eps, norm_values);
  else
    kv_store_kernel<bf16><<<M, 128, 0, stream>>>(reinterpret_cast<const bf16*>(k), ldk, reinterpret_cast<const bf16*>(v), ldv, meta,
                                                 reinterpret_cast<bf16*>(kcache), k_slot_stride, reinterpret_cast<bf16*>(vcache), v_slot_stride, G, dim, vdim, eps, norm_values);
  LIA_LAUNCH_CHECK();
  return LIA_OK;
}

/* see lia_b200.h */
extern "C" int lia_qkv_prep(const void* y, int act_f32, int ld, int q_off, int k_off, int v_off, const float* bias, const float* wconv,
                            const float* conv_state, int taps, int norm_mode, const float* qnorm_w, const float* knorm_w, float eps,
                            float temp_coef, int temp_every, const double* freq, int rot_dims, int rot_halves, float rot_mag, int vmix_mode,
                            float lambda, float* v_first, const int* meta, float* q_out, void* kcache, long long k_slot_stride, void* vcache,
                            long long v_slot_stride, int M, int H, int G, int dim, int vdim, lia_stream_t stream_) {
  return lia_qkv_prep_heads(y, act_f32, ld, q_off, k_off, v_off, bias, wconv, conv_state, taps, norm_mode, qnorm_w, knorm_w, eps, temp_coef, temp_every,
                            freq, rot_dims, rot_halves, rot_mag, vmix_mode, lambda, v_first, meta, q_out, kcache, k_slot_stride, vcache, v_slot_stride,
                            M, H, G, G, dim, vdim, stream_);
}

// Gv value heads beside G key heads (several attention maps over one set of values have G = maps * Gv)
extern "C" int lia_qkv_prep_heads(const void* y, int act_f32, int ld, int q_off, int k_off, int v_off, const float* bias, const float* wconv,
                                  const float* conv_state, int taps, int norm_mode, const float* qnorm_w, const float* knorm_w, float eps,
                                  float temp_coef, int temp_every, const double* freq, int rot_dims, int rot_halves, float rot_mag, int vmix_mode,
                                  float lambda, float* v_first, const int* meta, float* q_out, void* kcache, long long k_slot_stride, void* vcache,
                                  long long v_slot_stride, int M, int H, int G, int Gv, int dim, int vdim, lia_stream_t stream_) {
  LIA_CHECK_ARG(Gv > 0, "lia_qkv_prep: no value heads");
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  LIA_CHECK_ARG(y && meta && q_out && kcache && vcache, "lia_qkv_prep: null pointer");
  LIA_CHECK_ARG(M > 0 && H > 0 && G > 0 && dim > 0 && vdim > 0 && taps >= 1 && taps <= 16 && (taps == 1 || (wconv && conv_state)),
                "lia_qkv_prep: bad shape H=%d G=%d dim=%d vdim=%d taps=%d", H, G, dim, vdim, taps);
  LIA_CHECK_ARG(norm_mode >= 0 && norm_mode <= 2 && (norm_mode == 0 || (qnorm_w && knorm_w)), "lia_qkv_prep: bad norm mode %d", norm_mode);
  LIA_CHECK_ARG(rot_dims >= 0 && rot_dims <= dim && rot_dims % 2 == 0 && (rot_dims == 0 || freq), "lia_qkv_prep: cannot rotate %d of %d channels", rot_dims, dim);
  LIA_CHECK_ARG(vmix_mode >= 0 && vmix_mode <= 2 && (vmix_mode == 0 || v_first), "lia_qkv_prep: bad value-mixing mode %d", vmix_mode);
  PrepArgs a{H, G, dim, vdim, q_off, k_off, v_off, taps, norm_mode, temp_every, rot_dims, rot_halves, vmix_mode, eps, temp_coef, rot_mag, lambda};
  a.Gv = Gv;
  const size_t smem = ((size_t)(H + G) * dim + (size_t)Gv * vdim + rot_dims) * sizeof(float);
  LIA_CHECK_ARG(smem <= 160 * 1024, "lia_qkv_prep: %d channels do not fit shared memory", (H + G) * dim + Gv * vdim);
  if (act_f32) {
    if (smem > 48 * 1024) LIA_CUDA(cudaFuncSetAttribute(qkv_prep_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    qkv_prep_kernel<float><<<M, 256, smem, stream>>>(reinterpret_cast<const float*>(y), ld, bias, wconv, conv_state, qnorm_w, knorm_w, freq, meta, v_first,
                                                     q_out, reinterpret_cast<float*>(kcache), k_slot_stride, reinterpret_cast<float*>(vcache), v_slot_stride, a);
  } else {
    if (smem > 48 * 1024) LIA_CUDA(cudaFuncSetAttribute(qkv_prep_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    qkv_prep_kernel<bf16><<<M, 256, smem, stream>>>(reinterpret_cast<const bf16*>(y), ld, bias, wconv, conv_state, qnorm_w, knorm_w, freq, meta, v_first,
                                                    q_out, reinterpret_cast<bf16*>(kcache), k_slot_stride, reinterpret_cast<bf16*>(vcache), v_slot_stride, a);
  }
  LIA_LAUNCH_CHECK();
  return LIA_OK;
}

// Pairs (row, head) that one warp can carry for value heads of `vdim` numbers: bounds rows_per_block * heads_per_block / 8.
extern "C" int lia_window_attn_pairs_per_warp(int vdim) { return vdim <= 128 ? 4 : (vdim <= 256 ? 2 : 1); }

extern "C" size_t lia_window_attn_smem_bytes(int heads_per_block, int kv_heads_per_block, int rows_per_block, int dim, int vdim) {
  WindowArgs a{0, 0, dim, vdim, 0, heads_per_block, kv_heads_per_block, rows_per_block, 1, 0.f, 0.f};
  return attn_smem(a);
}

extern "C" size_t lia_window_attn_workspace_floats(int M, int H, int vdim, int nsplit) {
  if (nsplit <= 1) return 0;
  return (size_t)M * H * nsplit * ((size_t)vdim + 2);
}

extern "C" int lia_window_attn_ext(const void* q, int ldq, int q_f32, int act_f32, const void* kcache, long long k_slot_stride, const void* vcache,
                                   long long v_slot_stride, const int* meta, const float* temp, const float* slopes, const float* sink,
                                   const void* gate, int gate_mode, int ldg, void* out, float* workspace, int M, int H, int G, int dim, int vdim,
                                   int window, float scale, float softcap, int heads_per_block, int rows_per_block, int nsplit,
                                   lia_stream_t stream_) {
  return lia_window_attn_masked(q, ldq, q_f32, act_f32, kcache, k_slot_stride, vcache, v_slot_stride, meta, temp, slopes, sink, gate, gate_mode, ldg, out,
                                0, workspace, M, H, G, 1, dim, vdim, window, 0, scale, softcap, heads_per_block, rows_per_block, nsplit, stream_);
}

// chunk > 0: the chunked mask; v_div: key heads per value head; out_f32: fp32 output on caches of any type
extern "C" int lia_window_attn_masked(const void* q, int ldq, int q_f32, int act_f32, const void* kcache, long long k_slot_stride, const void* vcache,
                                      long long v_slot_stride, const int* meta, const float* temp, const float* slopes, const float* sink,
                                      const void* gate, int gate_mode, int ldg, void* out, int out_f32, float* workspace, int M, int H, int G,
                                      int v_div, int dim, int vdim, int window, int chunk, float scale, float softcap, int heads_per_block,
                                      int rows_per_block, int nsplit, lia_stream_t stream_) {
  LIA_CHECK_ARG(v_div >= 1 && G % v_div == 0 && chunk >= 0, "lia_window_attn: %d key heads do not share value heads in groups of %d (chunk %d)", G, v_div, chunk);
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  LIA_CHECK_ARG(q && kcache && vcache && meta && out, "lia_window_attn: null pointer");
  LIA_CHECK_ARG(M > 0 && H > 0 && G > 0 && H % G == 0 && dim > 0 && vdim > 0 && vdim <= 512 && H <= 65535 && ldq >= H * dim,
                "lia_window_attn: bad shape H=%d G=%d dim=%d vdim=%d window=%d", H, G, dim, vdim, window);
  LIA_CHECK_ARG(gate_mode >= 0 && gate_mode <= 2 && (gate_mode == 0) == (gate == nullptr) && (gate_mode != 2 || ldg >= H * vdim),
                "lia_window_attn: bad output gate (mode %d, row stride %d)", gate_mode, ldg);
  if (window <= 0) window = 1 << 30;                             // the whole history
  const int rep = H / G, HB = heads_per_block;
  LIA_CHECK_ARG(HB >= 1 && HB <= NWARP && (HB % rep == 0 || rep % HB == 0), "lia_window_attn: %d heads per block do not fit groups of %d", HB, rep);
  LIA_CHECK_ARG(rows_per_block >= 1 && nsplit >= 1 && nsplit <= 64 && (nsplit == 1 || workspace), "lia_window_attn: bad rows per block (%d) or key ranges (%d)", rows_per_block, nsplit);
  WindowArgs a{H, G, dim, vdim, window, HB, HB >= rep ? HB / rep : 1, rows_per_block, nsplit, scale, softcap, q_f32 || act_f32, gate_mode, ldg};
  a.chunk = chunk;
  a.v_div = v_div;
  a.out_f32 = out_f32 || act_f32;
  LIA_CHECK_ARG(attn_smem(a) <= 200 * 1024, "lia_window_attn: heads of %d + %d numbers do not fit the shared-memory stage", dim, vdim);
  const WindowExtras x{temp, slopes, sink, gate};
  if (act_f32) return dispatch_attn<float>(q, ldq, kcache, k_slot_stride, vcache, v_slot_stride, meta, x, out, workspace, M, a, stream);
  return dispatch_attn<bf16>(q, ldq, kcache, k_slot_stride, vcache, v_slot_stride, meta, x, out, workspace, M, a, stream);
}

extern "C" int lia_window_attn(const void* q, int ldq, int act_f32, const void* kcache, long long k_slot_stride, const void* vcache,
                               long long v_slot_stride, const int* meta, const float* temp, void* out, float* workspace, int M, int H, int G,
                               int dim, int vdim, int window, float scale, float softcap, int heads_per_block, int rows_per_block, int nsplit,
                               lia_stream_t stream_) {
  LIA_CHECK_ARG(temp && window > 0, "lia_window_attn: needs a temperature per head and a positive window");
  return lia_window_attn_ext(q, ldq, act_f32, act_f32, kcache, k_slot_stride, vcache, v_slot_stride, meta, temp, nullptr, nullptr, nullptr, 0, 0, out,
                             workspace, M, H, G, dim, vdim, window, scale, softcap, heads_per_block, rows_per_block, nsplit, stream_);
}

extern "C" int lia_diff_combine(const float* a, void* out, int act_f32, int M, int H, int G, int vdim, float lambda, float mult, float eps,
                                lia_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  LIA_CHECK_ARG(a && out && M > 0 && H > 0 && G > 0 && H % G == 0 && vdim > 0, "lia_diff_combine: bad arguments");
  const unsigned grid = (unsigned)(((long long)M * H + 3) / 4);
  if (act_f32) diff_combine_kernel<float><<<grid, 128, 0, stream>>>(a, reinterpret_cast<float*>(out), M, H, G, vdim, lambda, mult, eps);
  else diff_combine_kernel<bf16><<<grid, 128, 0, stream>>>(a, reinterpret_cast<bf16*>(out), M, H, G, vdim, lambda, mult, eps);
  LIA_LAUNCH_CHECK();
  return LIA_OK;
}
