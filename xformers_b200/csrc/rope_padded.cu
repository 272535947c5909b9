// Rotary embeddings + KV-cache emplacement for a heterogeneous batch laid out
// as BlockDiagonalCausalWithOffsetPaddedKeysMask describes it.
//
// HBM-bound, element-wise.  One CTA owns one query token (all its heads): the
// rows of xq are rotated into out_q, the rows of xk are rotated into cache_k at
// the token's position in its sequence's slot, the rows of xv are copied into
// cache_v.  A thread owns a (real, imaginary) pair index j: it computes the
// angle seq_pos * theta^(-2j/dim) / linear_scale and its sine / cosine once and
// walks over the token's head rows, so neighbouring threads touch neighbouring
// addresses and the transcendental work is shared by all heads of the token.
// Sequence starts, lengths and positions are read from device memory.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "internal.h"

namespace xfb {

template <typename T>
struct RopeIo;
template <>
struct RopeIo<__nv_bfloat16> {
  static __device__ __forceinline__ float ld(const __nv_bfloat16* p) { return __bfloat162float(*p); }
  static __device__ __forceinline__ void st(__nv_bfloat16* p, float x) { *p = __float2bfloat16_rn(x); }
};
template <>
struct RopeIo<__half> {
  static __device__ __forceinline__ float ld(const __half* p) { return __half2float(*p); }
  static __device__ __forceinline__ void st(__half* p, float x) { *p = __float2half_rn(x); }
};
template <>
struct RopeIo<float> {
  static __device__ __forceinline__ float ld(const float* p) { return *p; }
  static __device__ __forceinline__ void st(float* p, float x) { *p = x; }
};

// frequency of pair j, with the optional wavelength-dependent rescaling
// (xformers/ops/_triton/rope_padded_kernels.py:181-203)
template <typename F>
__device__ __forceinline__ F rope_freq(const xfb200_rope_params& p, int j) {
  F freq = F(pow(F(p.theta), F(2 * j) / F(-p.dim)));
  if (p.use_dynamic_scaling) {
    const F lo_wavelen = F(p.dynamic_old_context_len) / F(p.dynamic_low_freq_factor);
    const F hi_wavelen = F(p.dynamic_old_context_len) / F(p.dynamic_high_freq_factor);
    const F wavelen = F(6.28318530718) / freq;
    const F base = freq;
    if (wavelen > lo_wavelen) freq = base / F(p.dynamic_scale_factor);
    if (hi_wavelen < wavelen && wavelen <= lo_wavelen) {
      const F smooth = (F(p.dynamic_old_context_len) / wavelen - F(p.dynamic_low_freq_factor)) /
                       (F(p.dynamic_high_freq_factor) - F(p.dynamic_low_freq_factor));
      freq = (F(1) - smooth) * base / F(p.dynamic_scale_factor) + smooth * base;
    }
  }
  return freq;
}

constexpr int kRopeThreads = 256;
constexpr int kRopeUnroll = 4;

// 16-byte vectors of T, kept as raw words between the load and the arithmetic
template <typename T>
struct RopeVec {
  static constexpr int kElems = 16 / int(sizeof(T));
  static __device__ __forceinline__ uint4 load(const T* p) { return *reinterpret_cast<const uint4*>(p); }
  static __device__ __forceinline__ void store(T* p, const uint4& w) { *reinterpret_cast<uint4*>(p) = w; }
  static __device__ __forceinline__ void unpack(const uint4& w, float (&x)[kElems]) {
    const T* t = reinterpret_cast<const T*>(&w);
#pragma unroll
    for (int i = 0; i < kElems; ++i) x[i] = RopeIo<T>::ld(t + i);
  }
  static __device__ __forceinline__ uint4 pack(const float (&x)[kElems]) {
    uint4 w;
    T* t = reinterpret_cast<T*>(&w);
#pragma unroll
    for (int i = 0; i < kElems; ++i) RopeIo<T>::st(t + i, x[i]);
    return w;
  }
};

// source and destination of row `row` (q rows, then k rows, then v rows) of one token
template <typename T>
__device__ __forceinline__ void rope_row(const xfb200_rope_params& p, int row, int qpos, int cache_pos, const T*& src, T*& dst, bool& rotate) {
  const int head = row / p.groups, g = row - head * p.groups;
  rotate = true;
  if (head < p.q_heads) {
    src = reinterpret_cast<const T*>(p.xq) + int64_t(qpos) * p.xq_m + int64_t(g) * p.xq_g + int64_t(head) * p.xq_h;
    dst = reinterpret_cast<T*>(p.out_q) + int64_t(qpos) * p.oq_m + int64_t(g) * p.oq_g + int64_t(head) * p.oq_h;
  } else if (head < p.q_heads + p.kv_heads) {
    const int hk = head - p.q_heads;
    src = reinterpret_cast<const T*>(p.xk) + int64_t(qpos) * p.xk_m + int64_t(g) * p.xk_g + int64_t(hk) * p.xk_h;
    dst = reinterpret_cast<T*>(p.cache_k) + int64_t(cache_pos) * p.ck_m + int64_t(g) * p.ck_g + int64_t(hk) * p.ck_h;
  } else {
    const int hv = head - p.q_heads - p.kv_heads;
    src = reinterpret_cast<const T*>(p.xv) + int64_t(qpos) * p.xv_m + int64_t(g) * p.xv_g + int64_t(hv) * p.xv_h;
    dst = reinterpret_cast<T*>(p.cache_v) + int64_t(cache_pos) * p.cv_m + int64_t(g) * p.cv_g + int64_t(hv) * p.cv_h;
    rotate = false;
  }
}

// kVec: every row starts on a 16-byte boundary and dim (dim / 2 for split halves)
// is a whole number of 16-byte vectors.  Shared memory: the token's table of
// (cos, sin) per pair, computed once and used by all of the token's rows.
template <typename T, bool kF64, bool kVec>
__global__ void __launch_bounds__(kRopeThreads, kVec ? 4 : 2) rope_padded_kernel(const __grid_constant__ xfb200_rope_params p) {
  extern __shared__ float2 cs_table[];
  // blockIdx.x = query inside the sequence, blockIdx.y = sequence
  const int b = blockIdx.y;
  const int q1 = p.seqstart_q[b + 1];
  const int qpos = p.seqstart_q[b] + int(blockIdx.x);
  if (qpos >= q1) return;
  const int cache_start = p.seqstart_k[b];
  const int cache_pos = cache_start + p.seqlen_k[b] - (q1 - qpos);  // the queries are the last keys of the sequence
  auto position = [&](const void* base, int64_t i) -> long long {
    return p.seqpos_i64 ? reinterpret_cast<const long long*>(base)[i * p.seqpos_stride]
                        : reinterpret_cast<const int*>(base)[i * p.seqpos_stride];
  };
  long long seq_pos;
  if (p.seqpos != nullptr)
    seq_pos = position(p.seqpos, qpos);
  else
    seq_pos = (cache_pos - cache_start) + (p.first_seqpos != nullptr ? position(p.first_seqpos, b) : 0);

  const int pairs = p.dim / 2;
  const int rows = (p.q_heads + 2 * p.kv_heads) * p.groups;
  for (int j = threadIdx.x; j < pairs; j += kRopeThreads) {
    // The frequency and the product with the position are formed in double
    // precision and reduced to [-pi, pi] there: the library is compiled with
    // fast-math, whose single-precision power, sine and cosine are only good on
    // a small range.  kF64 also takes the sine and cosine in double precision.
    const double ang = double(seq_pos) * rope_freq<double>(p, j) / double(p.linear_scale);
    float sn, cs;
    if constexpr (kF64) {
      sn = float(sin(ang)), cs = float(cos(ang));
    } else {
      const double two_pi = 6.283185307179586476925286766559;
      const float r = float(ang - two_pi * rint(ang / two_pi));
      __sincosf(r, &sn, &cs);
    }
    cs_table[j] = make_float2(cs, sn);
  }
  __syncthreads();

  if constexpr (kVec) {
    constexpr int E = RopeVec<T>::kElems;
    // an item is one vector of a row (adjacent pairs) or the two vectors holding
    // E real parts and their E imaginary parts (split halves)
    const int per_row = p.adjacents ? p.dim / E : pairs / E;
    const int items = rows * per_row;
    for (int it0 = threadIdx.x; it0 < items; it0 += kRopeThreads * kRopeUnroll) {
      uint4 xw[kRopeUnroll], yw[kRopeUnroll];
      T* dst[kRopeUnroll];
      bool rot[kRopeUnroll];
      int vec[kRopeUnroll];
#pragma unroll
      for (int u = 0; u < kRopeUnroll; ++u) {
        const int it = it0 + u * kRopeThreads;
        if (it < items) {
          const int row = it / per_row;
          vec[u] = it - row * per_row;
          const T* src;
          rope_row<T>(p, row, qpos, cache_pos, src, dst[u], rot[u]);
          dst[u] += vec[u] * E;
          xw[u] = RopeVec<T>::load(src + vec[u] * E);
          if (!p.adjacents) yw[u] = RopeVec<T>::load(src + pairs + vec[u] * E);
        }
      }
#pragma unroll
      for (int u = 0; u < kRopeUnroll; ++u) {
        const int it = it0 + u * kRopeThreads;
        if (it < items) {
          if (rot[u]) {
            float x[E], y[E];
            RopeVec<T>::unpack(xw[u], x);
            if (p.adjacents) {
#pragma unroll
              for (int i = 0; i < E / 2; ++i) {
                const float2 t = cs_table[vec[u] * (E / 2) + i];
                const float re = x[2 * i], im = x[2 * i + 1];
                x[2 * i] = re * t.x - im * t.y;
                x[2 * i + 1] = im * t.x + re * t.y;
              }
            } else {
              RopeVec<T>::unpack(yw[u], y);
#pragma unroll
              for (int i = 0; i < E; ++i) {
                const float2 t = cs_table[vec[u] * E + i];
                const float re = x[i], im = y[i];
                x[i] = re * t.x - im * t.y;
                y[i] = im * t.x + re * t.y;
              }
              yw[u] = RopeVec<T>::pack(y);
            }
            xw[u] = RopeVec<T>::pack(x);
          }
          RopeVec<T>::store(dst[u], xw[u]);
          if (!p.adjacents) RopeVec<T>::store(dst[u] + pairs, yw[u]);
        }
      }
    }
  } else {
    const int items = rows * pairs;
    for (int it = threadIdx.x; it < items; it += kRopeThreads) {
      const int row = it / pairs, j = it - row * pairs;
      const T* src;
      T* dst;
      bool rotate;
      rope_row<T>(p, row, qpos, cache_pos, src, dst, rotate);
      const int c_re = p.adjacents ? 2 * j : j;
      const int c_im = p.adjacents ? 2 * j + 1 : j + pairs;
      const float2 t = cs_table[j];
      const float re = RopeIo<T>::ld(src + c_re), im = RopeIo<T>::ld(src + c_im);
      RopeIo<T>::st(dst + c_re, rotate ? re * t.x - im * t.y : re);
      RopeIo<T>::st(dst + c_im, rotate ? im * t.x + re * t.y : im);
    }
  }
}

template <typename T>
int launch_rope(const xfb200_rope_params& p, cudaStream_t st) {
  constexpr int E = 16 / int(sizeof(T));
  auto aligned = [](const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15) == 0; };
  const int64_t strides[] = {p.xq_m, p.xq_g, p.xq_h, p.xk_m, p.xk_g, p.xk_h, p.xv_m, p.xv_g, p.xv_h,
                             p.oq_m, p.oq_g, p.oq_h, p.ck_m, p.ck_g, p.ck_h, p.cv_m, p.cv_g, p.cv_h};
  bool vec = (p.adjacents ? p.dim % E == 0 : (p.dim / 2) % E == 0) && aligned(p.xq) && aligned(p.xk) && aligned(p.xv) &&
             aligned(p.out_q) && aligned(p.cache_k) && aligned(p.cache_v);
  for (int64_t s : strides) vec = vec && s % E == 0;
  const size_t smem = size_t(p.dim / 2) * sizeof(float2);
  if (smem > 200 * 1024) return set_error(XFB200_E_UNSUPPORTED, "rope_padded: dim %d too large", p.dim);
  dim3 grid(unsigned(p.max_q_per_seq), unsigned(p.batch), 1);
  auto go = [&](auto kernel) -> int {
    if (smem > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
      if (e != cudaSuccess) return cuda_fail("rope_padded: shared memory", e);
    }
    kernel<<<grid, kRopeThreads, smem, st>>>(p);
    return check_launch("rope_padded_kernel");
  };
  if (p.internal_f64) return vec ? go(rope_padded_kernel<T, true, true>) : go(rope_padded_kernel<T, true, false>);
  return vec ? go(rope_padded_kernel<T, false, true>) : go(rope_padded_kernel<T, false, false>);
}

}  // namespace xfb

extern "C" int xfb200_rope_padded(const xfb200_rope_params* p, void* stream) {
  using namespace xfb;
  if (p == nullptr) return set_error(XFB200_E_INVALID, "rope_padded: null params");
  if (p->batch < 0 || p->max_q_per_seq < 0 || p->q_heads < 1 || p->kv_heads < 1 || p->groups < 1)
    return set_error(XFB200_E_INVALID, "rope_padded: bad extents");
  if (p->dim < 2 || p->dim % 2) return set_error(XFB200_E_INVALID, "rope_padded: dim %d must be even", p->dim);
  if (p->batch == 0 || p->max_q_per_seq == 0) return XFB200_OK;
  if (!p->xq || !p->xk || !p->xv || !p->out_q || !p->cache_k || !p->cache_v || !p->seqstart_q || !p->seqstart_k || !p->seqlen_k)
    return set_error(XFB200_E_INVALID, "rope_padded: null tensor pointer");
  if (p->first_seqpos != nullptr && p->seqpos != nullptr) return set_error(XFB200_E_INVALID, "rope_padded: seqpos and first_seqpos may not both be given");
  if (!(p->linear_scale != 0.f)) return set_error(XFB200_E_INVALID, "rope_padded: linear_scale must not be 0");
  if (p->batch > 65535) return set_error(XFB200_E_UNSUPPORTED, "rope_padded: more than 65535 sequences");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (p->dtype == XFB200_BF16) return launch_rope<__nv_bfloat16>(*p, st);
  if (p->dtype == XFB200_F16) return launch_rope<__half>(*p, st);
  if (p->dtype == XFB200_F32) return launch_rope<float>(*p, st);
  return set_error(XFB200_E_INVALID, "rope_padded: bad dtype %d", p->dtype);
}
