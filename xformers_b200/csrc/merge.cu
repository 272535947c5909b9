// LSE-weighted merge of partial attentions (HBM-bound, element-wise over rows).
//
//   m = max_s lse_s; w_s = exp(lse_s - m); out = sum_s w_s O_s / sum_s w_s;
//   lse = m + log sum_s w_s
//
// One warp owns one output row (b, m, g, h): it reads the S log-sum-exps once,
// then streams the S partial rows with 128-bit loads and accumulates in fp32
// in a fixed order (s = 0..S-1), so results are bit-reproducible.
// A partial with lse = -inf contributes exactly nothing (selected out, never
// multiplied), so NaN/garbage in such a partial cannot leak.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "internal.h"

namespace xfb {

struct MergeArgs {
  const void* attn[XFB200_MERGE_MAX_PTRS];
  const float* lse[XFB200_MERGE_MAX_PTRS];
  int32_t num_splits;
  int32_t stacked;
  int64_t attn_stride_s, lse_stride_s;
  xfb200_strides as;
  int64_t li_b, li_g, li_h;
  void* out;
  float* lse_out;
  xfb200_strides os;
  int64_t lo_b, lo_g, lo_h;
  int32_t B, M, G, H, D;
};

template <typename T>
__device__ __forceinline__ float to_f32(T x);
template <>
__device__ __forceinline__ float to_f32<float>(float x) { return x; }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }
template <>
__device__ __forceinline__ float to_f32<__half>(__half x) { return __half2float(x); }

template <typename T>
__device__ __forceinline__ T from_f32(float x);
template <>
__device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }
template <>
__device__ __forceinline__ __half from_f32<__half>(float x) { return __float2half_rn(x); }

template <typename T, int V>
struct alignas(sizeof(T) * V) Vec {
  T v[V];
};

constexpr int kMergeWarps = 8;
constexpr int kMaxSplitsInRegs = 32;

template <typename Tin, typename Tout, int V>
__global__ void __launch_bounds__(kMergeWarps * 32) merge_kernel(const __grid_constant__ MergeArgs a) {
  const int lane = threadIdx.x & 31;
  const int64_t row = int64_t(blockIdx.x) * kMergeWarps + (threadIdx.x >> 5);
  const int64_t rows = int64_t(a.B) * a.M * a.G * a.H;
  if (row >= rows) return;
  // m fastest so that the lse reads of neighbouring warps are contiguous
  int64_t r = row;
  const int m = int(r % a.M);
  r /= a.M;
  const int h = int(r % a.H);
  r /= a.H;
  const int g = int(r % a.G);
  const int b = int(r / a.G);

  const int S = a.num_splits;
  const int64_t lse_off = b * a.li_b + g * a.li_g + h * a.li_h + m;
  const int64_t att_off = b * a.as.b + int64_t(m) * a.as.m + g * a.as.g + h * a.as.h;

  // lane s holds lse of split s (+32, +64, ... for larger S)
  float mx = -INFINITY;
  for (int s = lane; s < S; s += 32) {
    const float* lp = a.stacked ? a.lse[0] + s * a.lse_stride_s : a.lse[s];
    float l = lp[lse_off];
    if (l != l) l = -INFINITY;  // NaN lse: treat as an empty partial
    mx = fmaxf(mx, l);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  const bool any = mx > -INFINITY;

  constexpr int kChunks = 4;  // up to 4 column chunks of 32*V per lane kept in registers
  float acc[V * kChunks];
#pragma unroll
  for (int i = 0; i < V * kChunks; ++i) acc[i] = 0.f;
  float den = 0.f;

  for (int d0 = 0; d0 < a.D; d0 += 32 * V * kChunks) {
    den = 0.f;
#pragma unroll
    for (int i = 0; i < V * kChunks; ++i) acc[i] = 0.f;
    for (int s = 0; s < S; ++s) {
      const float* lp = a.stacked ? a.lse[0] + s * a.lse_stride_s : a.lse[s];
      float l = lp[lse_off];
      if (l != l) l = -INFINITY;
      const float w = (any && l > -INFINITY) ? __expf(l - mx) : 0.f;
      den += w;
      if (w == 0.f) continue;  // warp-uniform: all lanes read the same lse
      const Tin* ap = reinterpret_cast<const Tin*>(a.stacked ? a.attn[0] : a.attn[s]) +
                      (a.stacked ? s * a.attn_stride_s : 0) + att_off;
#pragma unroll
      for (int c = 0; c < kChunks; ++c) {
        const int d = d0 + (c * 32 + lane) * V;
        if (d < a.D) {
          Vec<Tin, V> x = *reinterpret_cast<const Vec<Tin, V>*>(ap + d);
#pragma unroll
          for (int i = 0; i < V; ++i) acc[c * V + i] += w * to_f32<Tin>(x.v[i]);
        }
      }
    }
    const float inv = den > 0.f ? 1.f / den : 0.f;
    Tout* op = reinterpret_cast<Tout*>(a.out) + b * a.os.b + int64_t(m) * a.os.m + g * a.os.g + h * a.os.h;
#pragma unroll
    for (int c = 0; c < kChunks; ++c) {
      const int d = d0 + (c * 32 + lane) * V;
      if (d < a.D) {
        Vec<Tout, V> y;
#pragma unroll
        for (int i = 0; i < V; ++i) y.v[i] = from_f32<Tout>(acc[c * V + i] * inv);
        *reinterpret_cast<Vec<Tout, V>*>(op + d) = y;
      }
    }
  }
  if (a.lse_out != nullptr && lane == 0) {
    if (a.D == 0) {
      den = 0.f;
      for (int s = 0; s < S; ++s) {
        const float* lp = a.stacked ? a.lse[0] + s * a.lse_stride_s : a.lse[s];
        float l = lp[lse_off];
        den += (any && l > -INFINITY) ? __expf(l - mx) : 0.f;
      }
    }
    a.lse_out[b * a.lo_b + g * a.lo_g + h * a.lo_h + m] = den > 0.f ? mx + __logf(den) : -INFINITY;
  }
}

template <typename Tin, typename Tout>
static int launch_merge_v(const MergeArgs& a, int vec, cudaStream_t stream) {
  const int64_t rows = int64_t(a.B) * a.M * a.G * a.H;
  if (rows == 0) return XFB200_OK;
  const unsigned grid = unsigned((rows + kMergeWarps - 1) / kMergeWarps);
  if (vec == 4)
    merge_kernel<Tin, Tout, 4><<<grid, kMergeWarps * 32, 0, stream>>>(a);
  else
    merge_kernel<Tin, Tout, 1><<<grid, kMergeWarps * 32, 0, stream>>>(a);
  return check_launch("merge_kernel");
}

template <typename Tin>
static int launch_merge_in(const MergeArgs& a, int out_dtype, int vec, cudaStream_t stream) {
  switch (out_dtype) {
    case XFB200_F32: return launch_merge_v<Tin, float>(a, vec, stream);
    case XFB200_BF16: return launch_merge_v<Tin, __nv_bfloat16>(a, vec, stream);
    case XFB200_F16: return launch_merge_v<Tin, __half>(a, vec, stream);
  }
  return set_error(XFB200_E_INVALID, "merge: bad out_dtype %d", out_dtype);
}

static size_t dtype_size(int dt) { return dt == XFB200_F32 ? 4 : 2; }

}  // namespace xfb

extern "C" int xfb200_merge_attentions(const xfb200_merge_params* p, void* stream) {
  using namespace xfb;
  if (p == nullptr) return set_error(XFB200_E_INVALID, "merge: null params");
  if (p->num_splits < 1) return set_error(XFB200_E_INVALID, "merge: num_splits must be >= 1, got %d", p->num_splits);
  if (!p->stacked && p->num_splits > XFB200_MERGE_MAX_PTRS)
    return set_error(XFB200_E_UNSUPPORTED, "merge: %d separate partials exceed the limit of %d; pass a stacked tensor",
                     p->num_splits, XFB200_MERGE_MAX_PTRS);
  if (p->B < 0 || p->M < 0 || p->G < 0 || p->H < 0 || p->D < 0) return set_error(XFB200_E_INVALID, "merge: negative extent");
  if (p->attn_ptrs == nullptr || p->lse_ptrs == nullptr || p->out == nullptr)
    return set_error(XFB200_E_INVALID, "merge: null tensor pointer");
  MergeArgs a{};
  const int np = p->stacked ? 1 : p->num_splits;
  for (int s = 0; s < np; ++s) {
    a.attn[s] = p->attn_ptrs[s];
    a.lse[s] = p->lse_ptrs[s];
    if (a.attn[s] == nullptr || a.lse[s] == nullptr) return set_error(XFB200_E_INVALID, "merge: null partial %d", s);
  }
  a.num_splits = p->num_splits;
  a.stacked = p->stacked;
  a.attn_stride_s = p->attn_stride_s;
  a.lse_stride_s = p->lse_stride_s;
  a.as = p->attn_strides;
  a.li_b = p->lse_in_stride_b;
  a.li_g = p->lse_in_stride_g;
  a.li_h = p->lse_in_stride_h;
  a.out = p->out;
  a.lse_out = p->lse_out;
  a.os = p->out_strides;
  a.lo_b = p->lse_out_stride_b;
  a.lo_g = p->lse_out_stride_g;
  a.lo_h = p->lse_out_stride_h;
  a.B = p->B;
  a.M = p->M;
  a.G = p->G;
  a.H = p->H;
  a.D = p->D;

  // 4-wide vectors need every row start aligned to 4 elements of both dtypes
  auto aligned4 = [](const xfb200_strides& s, int64_t extra) {
    return s.b % 4 == 0 && s.m % 4 == 0 && s.g % 4 == 0 && s.h % 4 == 0 && extra % 4 == 0;
  };
  int vec = 1;
  if (p->D % 4 == 0 && aligned4(a.as, p->stacked ? a.attn_stride_s : 0) && aligned4(a.os, 0)) {
    vec = 4;
    const size_t in_al = 4 * dtype_size(p->in_dtype), out_al = 4 * dtype_size(p->out_dtype);
    for (int s = 0; s < np; ++s)
      if (reinterpret_cast<uintptr_t>(a.attn[s]) % in_al) vec = 1;
    if (reinterpret_cast<uintptr_t>(a.out) % out_al) vec = 1;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (p->in_dtype) {
    case XFB200_F32: return launch_merge_in<float>(a, p->out_dtype, vec, st);
    case XFB200_BF16: return launch_merge_in<__nv_bfloat16>(a, p->out_dtype, vec, st);
    case XFB200_F16: return launch_merge_in<__half>(a, p->out_dtype, vec, st);
  }
  return set_error(XFB200_E_INVALID, "merge: bad in_dtype %d", p->in_dtype);
}
