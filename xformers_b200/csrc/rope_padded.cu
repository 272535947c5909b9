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

#include <algorithm>

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
constexpr int kRopeMaxTok = 64;  // most tokens one CTA takes
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

// source and destination of row `row` (q rows, then k rows, then v rows) of the
// token at row `qpos` of the inputs and row `cache_pos` of the caches
// (an int4 cache has int32 rows: its strides count words)
template <typename T, int kQuant = 0>
__device__ __forceinline__ void rope_row(const xfb200_rope_params& p, int row, int qpos, int cache_pos, const T*& src, T*& dst, bool& rotate, int* kind_out = nullptr,
                                         int32_t** ss_out = nullptr) {
  int head = row, g = 0;
  if (p.groups != 1) head = row / p.groups, g = row - head * p.groups;
  const int kind = (head >= p.q_heads) + (head >= p.q_heads + p.kv_heads);  // 0 q, 1 k, 2 v
  head -= kind == 0 ? 0 : (kind == 1 ? p.q_heads : p.q_heads + p.kv_heads);
  const void* sbase = kind == 0 ? p.xq : (kind == 1 ? p.xk : p.xv);
  void* dbase = kind == 0 ? p.out_q : (kind == 1 ? p.cache_k : p.cache_v);
  if (ss_out != nullptr && kind != 0)  // fp8 caches: where this row's scale/shift word goes
    *ss_out = reinterpret_cast<int32_t*>(kind == 1 ? p.k_scale_shift : p.v_scale_shift) + int64_t(cache_pos) * (kind == 1 ? p.kss_m : p.vss_m) +
              int64_t(g) * (kind == 1 ? p.kss_g : p.vss_g) + int64_t(head) * (kind == 1 ? p.kss_h : p.vss_h);
  const int64_t s_m = kind == 0 ? p.xq_m : (kind == 1 ? p.xk_m : p.xv_m);
  const int64_t s_g = kind == 0 ? p.xq_g : (kind == 1 ? p.xk_g : p.xv_g);
  const int64_t s_h = kind == 0 ? p.xq_h : (kind == 1 ? p.xk_h : p.xv_h);
  const int64_t d_m = kind == 0 ? p.oq_m : (kind == 1 ? p.ck_m : p.cv_m);
  const int64_t d_g = kind == 0 ? p.oq_g : (kind == 1 ? p.ck_g : p.cv_g);
  const int64_t d_h = kind == 0 ? p.oq_h : (kind == 1 ? p.ck_h : p.cv_h);
  src = reinterpret_cast<const T*>(sbase) + qpos * s_m + g * s_g + head * s_h;
  const int64_t d_off = (kind == 0 ? qpos : cache_pos) * d_m + g * d_g + head * d_h;
  if (kQuant && kind != 0)
    dst = reinterpret_cast<T*>(reinterpret_cast<int32_t*>(dbase) + d_off);
  else
    dst = reinterpret_cast<T*>(dbase) + d_off;
  if (kind_out != nullptr) *kind_out = kind;
  rotate = kind != 2;
}

// kVec: every row starts on a 16-byte boundary and dim is a whole number of
// pairs of 16-byte vectors.  A CTA owns up to p.tok_per_cta
// consecutive tokens of one sequence, so the frequencies (a double-precision
// power each) are formed once per CTA and the dependent loads of the sequence
// bookkeeping are paid once.  Shared memory: (cos, sin) per (token, pair).
// kQuant (vector path, 16-bit T): cache_k / cache_v are int4 row-wise caches, a row
// = one (fp16 scale | fp16 shift << 16) word and dim / 8 words of nibbles, element
// e of a word at bits [4e, 4e + 4) (benchmarks/benchmark_attn_decoding.py:38-72):
// scale = (max - min) / 15 and shift = min of the row, both rounded to fp16,
// nibble = trunc((x - shift) / scale + 0.5).  The rotated keys are rounded to T
// first, as if a 16-bit cache had been written and quantised afterwards.
// kQuant == 2: fp8 row-wise caches (XFB200_KV_FP8_ROWWISE): int32 rows of dim / 4
// words of four e4m3 values and one (fp16 scale | fp16 shift << 16) word per row in
// a tensor of its own, x ~ fp8 * scale + shift.  shift = the row's mean, scale =
// max |x - shift| / 448, both rounded to fp16 before they are used, values rounded
// to nearest with saturation.
template <typename T, bool kF64, bool kVec, bool kAdj, int kQuant = 0>
__global__ void __launch_bounds__(kRopeThreads, kVec ? 4 : 2) rope_padded_kernel(const __grid_constant__ xfb200_rope_params p, const int tok_per_cta) {
  extern __shared__ float2 cs_table[];
  __shared__ int cache_rows[kRopeMaxTok];  // cache row of each of the CTA's tokens
  // blockIdx.x = group of queries inside the sequence, blockIdx.y = sequence
  const int b = blockIdx.y;
  const int q1 = p.seqstart_q[b + 1];
  const int first = p.seqstart_q[b] + int(blockIdx.x) * tok_per_cta;
  if (first >= q1) return;
  const int ntok = min(tok_per_cta, q1 - first);
  const int cache_start = p.seqstart_k[b];
  // the queries are the last keys of the sequence: token `first + t` is key slot_first + t of its slot,
  // which is row cache_start + slot_first + t of a flat cache, or goes through the page table
  const int slot_first = p.seqlen_k[b] - (q1 - first);
  if (int(threadIdx.x) < ntok) {
    // a key position outside the sequence's slot (lengths that do not fit the layout) is not written: row -1
    const int pos = slot_first + int(threadIdx.x);
    const int slot_rows = p.block_tables != nullptr ? p.pages_per_seq * p.page_size : p.seqstart_k[b + 1] - cache_start;
    int row = -1;
    if (pos >= 0 && pos < slot_rows)
      row = p.block_tables != nullptr ? p.block_tables[int64_t(b) * p.block_tables_stride + pos / p.page_size] * p.page_size + pos % p.page_size
                                      : cache_start + pos;
    cache_rows[threadIdx.x] = row;
  }
  auto position = [&](const void* base, int64_t i) -> long long {
    return p.seqpos_i64 ? reinterpret_cast<const long long*>(base)[i * p.seqpos_stride]
                        : reinterpret_cast<const int*>(base)[i * p.seqpos_stride];
  };
  const long long pos_first = slot_first + (p.first_seqpos != nullptr ? position(p.first_seqpos, b) : 0);

  const int pairs = p.dim / 2;
  const int rows = (p.q_heads + 2 * p.kv_heads) * p.groups;
  // The frequency and its product with the position are formed in double
  // precision and reduced to [-pi, pi] there: the library is compiled with
  // fast-math, whose single-precision power, sine and cosine are only good on
  // a small range.  kF64 also takes the sine and cosine in double precision.
  for (int j = threadIdx.x; j < pairs; j += kRopeThreads) {
    const double freq = rope_freq<double>(p, j) / double(p.linear_scale);
    for (int t = 0; t < ntok; ++t) {
      const long long seq_pos = p.seqpos != nullptr ? position(p.seqpos, first + t) : pos_first + t;
      const double ang = double(seq_pos) * freq;
      float sn, cs;
      if constexpr (kF64) {
        sn = float(sin(ang)), cs = float(cos(ang));
      } else {
        const double two_pi = 6.283185307179586476925286766559;
        const float r = float(ang - two_pi * rint(ang * (1.0 / two_pi)));
        __sincosf(r, &sn, &cs);
      }
      cs_table[t * pairs + j] = make_float2(cs, sn);
    }
  }
  __syncthreads();

  if constexpr (kVec) {
    constexpr int E = RopeVec<T>::kElems;
    // An item is E pairs of a row in two vectors, one in each half of the row:
    // E/2 pairs each (adjacent pairs), or E real parts and their E imaginary
    // parts (split halves).
    // A thread keeps its column (item index inside the row) and walks down the
    // rows of the CTA's tokens, `nslots` rows apart, (token, row) advanced
    // without a division.
        constexpr int kUnroll = 2;
    const int per_row = pairs / E;
    const int lanes = min(per_row, kRopeThreads);
    const int nslots = kRopeThreads / lanes;
    const int vx = threadIdx.x % lanes, slot = threadIdx.x / lanes;
    if (slot >= nslots) return;
    for (int v = vx; v < per_row; v += lanes) {
      const int x_off = v * E, y_off = pairs + x_off;  // the same column of the row's two halves: both loads of a warp are contiguous
      int t = 0, row = slot;
      while (row >= rows) row -= rows, ++t;
      while (t < ntok) {
        uint4 xw[kUnroll], yw[kUnroll];
        T* dst[kUnroll];
        bool to_int4[kUnroll];  // the row goes to a quantised cache
        int32_t* ss_dst[kUnroll];
        int tab[kUnroll];  // first (cos, sin) entry of the item, -1: copy only, -2: no item
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
          tab[u] = -2;
          if (t < ntok) {
            const T* src;
            bool rotate;
            int kind;
            rope_row<T, kQuant>(p, row, first + t, cache_rows[t], src, dst[u], rotate, &kind, kQuant == 2 ? &ss_dst[u] : nullptr);
            to_int4[u] = kQuant != 0 && kind != 0;
            if (kind == 0 || cache_rows[t] >= 0) {
              xw[u] = RopeVec<T>::load(src + x_off);
              yw[u] = RopeVec<T>::load(src + y_off);
              tab[u] = rotate ? t * pairs + (kAdj ? v * (E / 2) : v * E) : -1;
            }
            row += nslots;
            while (row >= rows) row -= rows, ++t;
          }
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
          if (tab[u] != -2) {
            float x[E], y[E];
            if (tab[u] >= 0 || to_int4[u]) {
              RopeVec<T>::unpack(xw[u], x);
              RopeVec<T>::unpack(yw[u], y);
            }
            if (tab[u] >= 0) {
              if constexpr (kAdj) {
#pragma unroll
                for (int i = 0; i < E / 2; ++i) {
                  const float2 w = cs_table[tab[u] + i], z = cs_table[tab[u] + pairs / 2 + i];
                  const float re = x[2 * i], im = x[2 * i + 1];
                  x[2 * i] = re * w.x - im * w.y;
                  x[2 * i + 1] = im * w.x + re * w.y;
                  const float re2 = y[2 * i], im2 = y[2 * i + 1];
                  y[2 * i] = re2 * z.x - im2 * z.y;
                  y[2 * i + 1] = im2 * z.x + re2 * z.y;
                }
              } else {
#pragma unroll
                for (int i = 0; i < E; ++i) {
                  const float2 w = cs_table[tab[u] + i];
                  const float re = x[i], im = y[i];
                  x[i] = re * w.x - im * w.y;
                  y[i] = im * w.x + re * w.y;
                }
              }
              xw[u] = RopeVec<T>::pack(x);
              yw[u] = RopeVec<T>::pack(y);
            }
            if constexpr (kQuant) {
              if (to_int4[u]) {
                if (tab[u] >= 0) {  // the values a 16-bit cache would hold
                  RopeVec<T>::unpack(xw[u], x);
                  RopeVec<T>::unpack(yw[u], y);
                }
                float mn = x[0], mx = x[0];
#pragma unroll
                for (int i = 0; i < E; ++i) {
                  mn = fminf(mn, fminf(x[i], y[i]));
                  mx = fmaxf(mx, fmaxf(x[i], y[i]));
                }
                // the `lanes` threads of a row are neighbours in their warp and reach this point together
                const unsigned gmask = (lanes >= 32 ? 0xffffffffu : ((1u << lanes) - 1u)) << ((threadIdx.x & 31) & ~(lanes - 1));
                if constexpr (kQuant == 2) {
                  float sum = 0.f;
#pragma unroll
                  for (int i = 0; i < E; ++i) sum += x[i] + y[i];
                  for (int o = 1; o < lanes; o <<= 1) sum += __shfl_xor_sync(gmask, sum, o);
                  const __half shift_h = __float2half_rn(__fdiv_rn(sum, float(p.dim)));
                  const float sh = __half2float(shift_h);
                  float amax = 0.f;
#pragma unroll
                  for (int i = 0; i < E; ++i) {
                    x[i] -= sh, y[i] -= sh;
                    amax = fmaxf(amax, fmaxf(fabsf(x[i]), fabsf(y[i])));
                  }
                  for (int o = 1; o < lanes; o <<= 1) amax = fmaxf(amax, __shfl_xor_sync(gmask, amax, o));
                  __half scale_h = __float2half_rn(__fdiv_rn(amax, 448.f));
                  if (__half2float(scale_h) == 0.f) scale_h = __float2half_rn(1.f);  // a constant row: every value is 0 * 1 + shift
                  const float inv = __fdiv_rn(1.f, __half2float(scale_h));
                  auto e4m3x4 = [&](float a0, float a1, float a2, float a3) {
                    uint32_t lo, hi;
                    asm("{\n\t.reg .b16 t;\n\tcvt.rn.satfinite.e4m3x2.f32 t, %2, %1;\n\tcvt.u32.u16 %0, t;\n\t}" : "=r"(lo) : "f"(a0 * inv), "f"(a1 * inv));
                    asm("{\n\t.reg .b16 t;\n\tcvt.rn.satfinite.e4m3x2.f32 t, %2, %1;\n\tcvt.u32.u16 %0, t;\n\t}" : "=r"(hi) : "f"(a2 * inv), "f"(a3 * inv));
                    return lo | (hi << 16);
                  };
                  int32_t* drow = reinterpret_cast<int32_t*>(dst[u]);
                  // x holds the elements [8 v, 8 v + 8) of the row, y the same of its second half: two words each
                  *reinterpret_cast<uint2*>(drow + 2 * v) = make_uint2(e4m3x4(x[0], x[1], x[2], x[3]), e4m3x4(x[4], x[5], x[6], x[7]));
                  *reinterpret_cast<uint2*>(drow + 2 * per_row + 2 * v) = make_uint2(e4m3x4(y[0], y[1], y[2], y[3]), e4m3x4(y[4], y[5], y[6], y[7]));
                  if (v == 0) *ss_dst[u] = int32_t(uint32_t(__half_as_ushort(scale_h)) | (uint32_t(__half_as_ushort(shift_h)) << 16));
                  continue;
                }
                for (int o = 1; o < lanes; o <<= 1) {
                  mn = fminf(mn, __shfl_xor_sync(gmask, mn, o));
                  mx = fmaxf(mx, __shfl_xor_sync(gmask, mx, o));
                }
                const __half scale_h = __float2half_rn(__fdiv_rn(mx - mn, 15.f)), shift_h = __float2half_rn(mn);
                const float sc = __half2float(scale_h), sh = __half2float(shift_h);
                auto nibbles = [&](const float (&z)[E]) {
                  uint32_t w = 0;
#pragma unroll
                  for (int i = 0; i < E; ++i) {
                    const float qf = __fadd_rn(__fdiv_rn(__fsub_rn(z[i], sh), sc), 0.5f);
                    const uint32_t qi = qf > 0.f ? uint32_t(qf) : 0u;  // truncation; NaN (a constant row: 0 / 0) gives 0
                    w |= (qi & 0xFu) << (4 * i);
                  }
                  return w;
                };
                int32_t* drow = reinterpret_cast<int32_t*>(dst[u]);
                drow[1 + v] = int32_t(nibbles(x));
                drow[1 + per_row + v] = int32_t(nibbles(y));
                if (v == 0) drow[0] = int32_t(uint32_t(__half_as_ushort(scale_h)) | (uint32_t(__half_as_ushort(shift_h)) << 16));
                continue;
              }
            }
            RopeVec<T>::store(dst[u] + x_off, xw[u]);
            RopeVec<T>::store(dst[u] + y_off, yw[u]);
          }
        }
      }
    }
  } else {
    const int per_tok = rows * pairs;
    const int items = ntok * per_tok;
    for (int it = threadIdx.x; it < items; it += kRopeThreads) {
      const int t = it / per_tok, rem = it - t * per_tok;
      const int row = rem / pairs, j = rem - row * pairs;
      const T* src;
      T* dst;
      bool rotate;
      int kind;
      rope_row<T>(p, row, first + t, cache_rows[t], src, dst, rotate, &kind);
      if (kind != 0 && cache_rows[t] < 0) continue;
      const int c_re = kAdj ? 2 * j : j;
      const int c_im = kAdj ? 2 * j + 1 : j + pairs;
      const float2 w = cs_table[t * pairs + j];
      const float re = RopeIo<T>::ld(src + c_re), im = RopeIo<T>::ld(src + c_im);
      RopeIo<T>::st(dst + c_re, rotate ? re * w.x - im * w.y : re);
      RopeIo<T>::st(dst + c_im, rotate ? im * w.x + re * w.y : im);
    }
  }
}

template <typename T>
int launch_rope(const xfb200_rope_params& p, cudaStream_t st) {
  constexpr int E = 16 / int(sizeof(T));
  auto aligned = [](const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15) == 0; };
  const int64_t strides[] = {p.xq_m, p.xq_g, p.xq_h, p.xk_m, p.xk_g, p.xk_h, p.xv_m, p.xv_g, p.xv_h,
                             p.oq_m, p.oq_g, p.oq_h, p.ck_m, p.ck_g, p.ck_h, p.cv_m, p.cv_g, p.cv_h};
  const bool quant = p.cache_format != 0;  // int32 rows, written word by word (fp8: 8 bytes at a time, checked below)
  bool vec = p.dim % (2 * E) == 0 && aligned(p.xq) && aligned(p.xk) && aligned(p.xv) && aligned(p.out_q) &&
             (quant || (aligned(p.cache_k) && aligned(p.cache_v)));
  for (int i = 0; i < 18; ++i) vec = vec && ((quant && i >= 12) || strides[i] % E == 0);
  const int pairs = p.dim / 2;
  // Tokens per CTA: about 128 KB of rows, while the (cos, sin) table stays within
  // 16 KB and the grid keeps a few CTAs per SM slot.
  const int64_t tok_bytes = int64_t(p.q_heads + 2 * p.kv_heads) * p.groups * p.dim * int64_t(sizeof(T));
  const int64_t by_grid = int64_t(p.max_q_per_seq) * p.batch / (int64_t(sm_count()) * 16);
  const int tok_per_cta = int(std::max<int64_t>(1, std::min<int64_t>({(128 * 1024 + tok_bytes - 1) / tok_bytes, 2048 / pairs, p.max_q_per_seq, by_grid, kRopeMaxTok})));
  const size_t smem = size_t(tok_per_cta) * pairs * sizeof(float2);
  if (smem > 200 * 1024) return set_error(XFB200_E_UNSUPPORTED, "rope_padded: dim %d too large", p.dim);
  dim3 grid(unsigned((p.max_q_per_seq + tok_per_cta - 1) / tok_per_cta), unsigned(p.batch), 1);
  auto go = [&](auto kernel) -> int {
    if (smem > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
      if (e != cudaSuccess) return cuda_fail("rope_padded: shared memory", e);
    }
    kernel<<<grid, kRopeThreads, smem, st>>>(p, tok_per_cta);
    return check_launch("rope_padded_kernel");
  };
  if (p.cache_format == 2) {
    const int per_row = pairs / E;
    if constexpr (sizeof(T) != 2) {
      return set_error(XFB200_E_UNSUPPORTED, "rope_padded: an fp8 cache needs bf16 or f16 inputs");
    } else {
      if (!vec || per_row > 32 || (per_row & (per_row - 1)) != 0)
        return set_error(XFB200_E_UNSUPPORTED, "rope_padded: an fp8 cache needs dim 32, 64, 128, 256 or 512 and 16-byte aligned input rows");
      if (p.internal_f64) return p.adjacents ? go(rope_padded_kernel<T, true, true, true, 2>) : go(rope_padded_kernel<T, true, true, false, 2>);
      return p.adjacents ? go(rope_padded_kernel<T, false, true, true, 2>) : go(rope_padded_kernel<T, false, true, false, 2>);
    }
  }
  if (p.cache_format == 1) {
    // int4 caches: the vector path with a row's threads inside one warp, 16-bit inputs
    const int per_row = pairs / E;
    if constexpr (sizeof(T) != 2) {
      return set_error(XFB200_E_UNSUPPORTED, "rope_padded: an int4 cache needs bf16 or f16 inputs");
    } else {
      if (!vec || per_row > 32 || (per_row & (per_row - 1)) != 0)
        return set_error(XFB200_E_UNSUPPORTED, "rope_padded: an int4 cache needs dim 32, 64, 128, 256 or 512 and 16-byte aligned input rows");
      if (p.internal_f64) return p.adjacents ? go(rope_padded_kernel<T, true, true, true, 1>) : go(rope_padded_kernel<T, true, true, false, 1>);
      return p.adjacents ? go(rope_padded_kernel<T, false, true, true, 1>) : go(rope_padded_kernel<T, false, true, false, 1>);
    }
  }
#define XFB_ROPE(F64, VEC)                                                                   \
  return p.adjacents ? go(rope_padded_kernel<T, F64, VEC, true>) : go(rope_padded_kernel<T, F64, VEC, false>)
  if (p.internal_f64) {
    if (vec) XFB_ROPE(true, true);
    XFB_ROPE(true, false);
  }
  if (vec) XFB_ROPE(false, true);
  XFB_ROPE(false, false);
#undef XFB_ROPE
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
  if (p->cache_format < 0 || p->cache_format > 2) return set_error(XFB200_E_INVALID, "rope_padded: cache_format %d", p->cache_format);
  if (p->cache_format == 2) {
    if (p->k_scale_shift == nullptr || p->v_scale_shift == nullptr) return set_error(XFB200_E_INVALID, "rope_padded: an fp8 cache needs its scale/shift tensors");
    const int64_t st[] = {p->ck_m, p->ck_g, p->ck_h, p->cv_m, p->cv_g, p->cv_h};
    bool ok = (reinterpret_cast<uintptr_t>(p->cache_k) & 7) == 0 && (reinterpret_cast<uintptr_t>(p->cache_v) & 7) == 0;
    for (int64_t s : st) ok = ok && s % 2 == 0;
    if (!ok) return set_error(XFB200_E_UNSUPPORTED, "rope_padded: fp8 cache rows must be 8-byte aligned");
  }
  if (p->block_tables != nullptr && p->pages_per_seq < 1) return set_error(XFB200_E_INVALID, "rope_padded: pages_per_seq %d with a page table", p->pages_per_seq);
  if (p->block_tables != nullptr && p->page_size < 1) return set_error(XFB200_E_INVALID, "rope_padded: page_size %d with a page table", p->page_size);
  if (!(p->linear_scale != 0.f)) return set_error(XFB200_E_INVALID, "rope_padded: linear_scale must not be 0");
  if (p->batch > 65535) return set_error(XFB200_E_UNSUPPORTED, "rope_padded: more than 65535 sequences");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (p->dtype == XFB200_BF16) return launch_rope<__nv_bfloat16>(*p, st);
  if (p->dtype == XFB200_F16) return launch_rope<__half>(*p, st);
  if (p->dtype == XFB200_F32) return launch_rope<float>(*p, st);
  return set_error(XFB200_E_INVALID, "rope_padded: bad dtype %d", p->dtype);
}
