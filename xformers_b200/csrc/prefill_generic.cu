// Generic attention-forward kernel on warp-level mma.sync (m16n8k16).
//
// Covers every shape the tcgen05 kernels do not take:
// head dims other than 64/128 (any multiple of 8 up to 256), different
// value head dim is not supported.  Same mask model, same outputs.
//
// One CTA = 4 warps = one 64-row query tile of one (sequence, head); key tiles
// of 64 rows are staged in shared memory with cp.async (zero-filled past the
// end), masked tiles are skipped, the online softmax runs in registers in the
// log2 domain.  K/V heads are indexed, never expanded (head stride may be 0).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "internal.h"
#include "ptx.cuh"

namespace xfb {

struct GenericArgs {
  xfb200_prefill_params p;
  float scale_log2;
};

constexpr int kGenBM = 64;
constexpr int kGenBN = 64;
constexpr int kGenThreads = 128;

template <bool kBf16>
__device__ __forceinline__ uint32_t gen_pack2(float lo, float hi) {
  if constexpr (kBf16) {
    __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&t);
  } else {
    __half2 t = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&t);
  }
}

template <int DP, bool kBf16>
__global__ void __launch_bounds__(kGenThreads) prefill_generic_kernel(const __grid_constant__ GenericArgs ga) {
  const xfb200_prefill_params& p = ga.p;
  constexpr int kRow = DP * 2 + 16;  // padded row stride in bytes
  constexpr int KS = DP / 16;
  constexpr int NT = DP / 8;
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* q_s = smem;
  uint8_t* k_s = q_s + kGenBM * kRow;
  uint8_t* v_s = k_s + kGenBN * kRow;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = lane >> 2, c = lane & 3;
  const int qt = blockIdx.x;
  const int gh = blockIdx.y;
  const int g = gh / p.heads_per_group, h = gh % p.heads_per_group;
  const int b = blockIdx.z;
  const int D = p.head_dim;

  // sequence geometry
  int64_t q_row0, k_row0;  // first row of this sequence in the q / k tensors (dim 1)
  int qlen, klen;
  int64_t qb = 0, kb = 0;  // batch index used for the batch stride
  if (p.seqstart_q != nullptr) {
    q_row0 = p.seqstart_q[b];
    qlen = p.seqstart_q[b + 1] - p.seqstart_q[b];
    k_row0 = p.seqstart_k[b];
    klen = p.seqlen_k != nullptr ? p.seqlen_k[b] : p.seqstart_k[b + 1] - p.seqstart_k[b];
  } else {
    q_row0 = 0, k_row0 = 0, qlen = p.mq, klen = p.mkv, qb = b, kb = b;
  }
  const int m0 = qt * kGenBM;
  if (m0 >= qlen) return;
  // query i sees key j iff i + shift - window_left <= j <= i + shift + wr (each bound only when it is >= 0)
  const int shift = (p.mask_type >= XFB200_MASK_CAUSAL_BOTTOM_RIGHT ? klen - qlen : 0) - p.kv_offset;
  const int wr = p.mask_type == XFB200_MASK_NONE ? -1 : p.mask_type == XFB200_MASK_LOCAL_BOTTOM_RIGHT ? p.window_right : 0;
  const bool causal = wr >= 0;

  // key range that any row of this tile can see
  int n_hi = klen;
  if (causal) n_hi = min(n_hi, m0 + kGenBM - 1 + shift + wr + 1);
  int n_lo = 0;
  if (p.window_left >= 0) n_lo = max(0, m0 + shift - p.window_left);
  n_lo = n_lo / kGenBN * kGenBN;

  const int esz = 2;
  const uint8_t* qg = reinterpret_cast<const uint8_t*>(p.q) + (qb * p.q_strides.b + q_row0 * p.q_strides.m + int64_t(g) * p.q_strides.g + int64_t(h) * p.q_strides.h) * esz;
  const uint8_t* kg = reinterpret_cast<const uint8_t*>(p.k) + (kb * p.k_strides.b + k_row0 * p.k_strides.m + int64_t(g) * p.k_strides.g + int64_t(h) * p.k_strides.h) * esz;
  const uint8_t* vg = reinterpret_cast<const uint8_t*>(p.v) + (kb * p.v_strides.b + k_row0 * p.v_strides.m + int64_t(g) * p.v_strides.g + int64_t(h) * p.v_strides.h) * esz;

  auto load_tile = [&](uint8_t* dst, const uint8_t* src, int64_t stride_m, int row_first, int row_limit) {
    // 64 rows x DP/8 chunks of 16 B; rows >= row_limit and columns >= D are zero-filled
    for (int i = threadIdx.x; i < 64 * (DP / 8); i += kGenThreads) {
      const int rr = i / (DP / 8), ch = i % (DP / 8);
      const int row = row_first + rr;
      const bool ok = row < row_limit && ch * 8 < D;
      const uint8_t* s = src + (int64_t(ok ? row : 0) * stride_m + (ok ? ch * 8 : 0)) * esz;
      cp_async_16(dst + rr * kRow + ch * 16, s, ok);
    }
  };

  load_tile(q_s, qg, p.q_strides.m, m0, qlen);
  cp_async_commit();

  float acc[NT][4];
#pragma unroll
  for (int j = 0; j < NT; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const int i0 = m0 + warp * 16 + r, i1 = i0 + 8;  // local query indices of this thread's rows
  // additive bias: rows of this thread's two query rows (dense batches only), or null
  const uint8_t* bias_row[2] = {nullptr, nullptr};
  const int bias_esz = p.bias_dtype == XFB200_F32 ? 4 : 2;
  if (p.bias != nullptr) {
    const int64_t base = int64_t(b) * p.bias_stride_b + int64_t(g) * p.bias_stride_g + int64_t(h) * p.bias_stride_h;
    if (i0 < qlen) bias_row[0] = reinterpret_cast<const uint8_t*>(p.bias) + (base + int64_t(i0) * p.bias_stride_m) * bias_esz;
    if (i1 < qlen) bias_row[1] = reinterpret_cast<const uint8_t*>(p.bias) + (base + int64_t(i1) * p.bias_stride_m) * bias_esz;
  }
  auto load_bias = [&](const uint8_t* row, int col) -> float {
    if (p.bias_dtype == XFB200_F32) return reinterpret_cast<const float*>(row)[col];
    if (p.bias_dtype == XFB200_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(row)[col]);
    return __half2float(reinterpret_cast<const __half*>(row)[col]);
  };

  for (int n0 = n_lo; n0 < n_hi; n0 += kGenBN) {
    __syncthreads();  // previous tile fully consumed
    load_tile(k_s, kg, p.k_strides.m, n0, klen);
    load_tile(v_s, vg, p.v_strides.m, n0, klen);
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();

    float s[kGenBN / 8][4];
#pragma unroll
    for (int j = 0; j < kGenBN / 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      uint32_t qf[4];
      ldmatrix_x4(qf, smem_u32(q_s + (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * kRow + (ks * 16 + (lane >> 4) * 8) * 2));
#pragma unroll
      for (int j = 0; j < kGenBN / 8; j += 2) {
        uint32_t kf[4];
        ldmatrix_x4(kf, smem_u32(k_s + (j * 8 + (lane & 7) + (lane >> 4) * 8) * kRow + (ks * 16 + ((lane >> 3) & 1) * 8) * 2));
        mma_16816<kBf16>(s[j], qf, kf[0], kf[1]);
        mma_16816<kBf16>(s[j + 1], qf, kf[2], kf[3]);
      }
    }

    // additive bias + mask + online softmax
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int j = 0; j < kGenBN / 8; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int col = n0 + j * 8 + 2 * c + (e & 1);
        const int i = (e >> 1) ? i1 : i0;
        bool vis = col < klen;
        if (causal) vis = vis && col <= i + shift + wr;
        if (p.window_left >= 0) vis = vis && col >= i + shift - p.window_left;
        float x = -INFINITY;
        if (vis) {
          x = s[j][e] * ga.scale_log2;
          if (bias_row[e >> 1] != nullptr) x = fmaf(load_bias(bias_row[e >> 1], col), 1.4426950408889634f, x);
        }
        s[j][e] = x;
        mx[e >> 1] = fmaxf(mx[e >> 1], x);
      }
    float alpha[2], m_use[2];
#pragma unroll
    for (int hlf = 0; hlf < 2; ++hlf) {
      mx[hlf] = fmaxf(mx[hlf], __shfl_xor_sync(0xffffffffu, mx[hlf], 1));
      mx[hlf] = fmaxf(mx[hlf], __shfl_xor_sync(0xffffffffu, mx[hlf], 2));
      const float m_new = fmaxf(m_run[hlf], mx[hlf]);
      m_use[hlf] = m_new == -INFINITY ? 0.f : m_new;
      alpha[hlf] = fast_exp2(m_run[hlf] - m_use[hlf]);
      m_run[hlf] = m_new;
    }
    float psum[2] = {0.f, 0.f};
    uint32_t pa[kGenBN / 16][4];
#pragma unroll
    for (int j = 0; j < kGenBN / 8; ++j) {
      const float p0 = fast_exp2(s[j][0] - m_use[0]), p1 = fast_exp2(s[j][1] - m_use[0]);
      const float p2 = fast_exp2(s[j][2] - m_use[1]), p3 = fast_exp2(s[j][3] - m_use[1]);
      psum[0] += p0 + p1;
      psum[1] += p2 + p3;
      pa[j >> 1][(j & 1) * 2 + 0] = gen_pack2<kBf16>(p0, p1);
      pa[j >> 1][(j & 1) * 2 + 1] = gen_pack2<kBf16>(p2, p3);
    }
    l_run[0] = l_run[0] * alpha[0] + psum[0];
    l_run[1] = l_run[1] * alpha[1] + psum[1];
#pragma unroll
    for (int j = 0; j < NT; ++j) {
      acc[j][0] *= alpha[0];
      acc[j][1] *= alpha[0];
      acc[j][2] *= alpha[1];
      acc[j][3] *= alpha[1];
    }
    // O += P V   (rows of V past klen are zero-filled, so 0 * garbage cannot occur)
#pragma unroll
    for (int kk = 0; kk < kGenBN / 16; ++kk) {
#pragma unroll
      for (int j = 0; j < NT; j += 2) {
        uint32_t vf[4];
        ldmatrix_x4_trans(vf, smem_u32(v_s + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * kRow + (j * 8 + (lane >> 4) * 8) * 2));
        mma_16816<kBf16>(acc[j], pa[kk], vf[0], vf[1]);
        mma_16816<kBf16>(acc[j + 1], pa[kk], vf[2], vf[3]);
      }
    }
  }
  cp_async_wait<0>();

  // epilogue
#pragma unroll
  for (int hlf = 0; hlf < 2; ++hlf) {
    l_run[hlf] += __shfl_xor_sync(0xffffffffu, l_run[hlf], 1);
    l_run[hlf] += __shfl_xor_sync(0xffffffffu, l_run[hlf], 2);
  }
  uint8_t* og = reinterpret_cast<uint8_t*>(p.out);
  const int osz = p.out_dtype == XFB200_F32 ? 4 : 2;
#pragma unroll
  for (int hlf = 0; hlf < 2; ++hlf) {
    const int i = hlf ? i1 : i0;
    if (i >= qlen) continue;
    const float inv = l_run[hlf] > 0.f ? 1.f / l_run[hlf] : 0.f;
    const int64_t off = qb * p.o_strides.b + (q_row0 + i) * p.o_strides.m + int64_t(g) * p.o_strides.g + int64_t(h) * p.o_strides.h;
#pragma unroll
    for (int j = 0; j < NT; ++j) {
      const int d = j * 8 + 2 * c;
      if (d >= D) continue;
      const float x0 = acc[j][hlf * 2] * inv, x1 = acc[j][hlf * 2 + 1] * inv;
      uint8_t* dst = og + (off + d) * osz;
      if (p.out_dtype == XFB200_F32) {
        *reinterpret_cast<float2*>(dst) = make_float2(x0, x1);
      } else if (p.out_dtype == XFB200_BF16) {
        *reinterpret_cast<uint32_t*>(dst) = gen_pack2<true>(x0, x1);
      } else {
        *reinterpret_cast<uint32_t*>(dst) = gen_pack2<false>(x0, x1);
      }
    }
    if (p.lse != nullptr && c == 0) {
      const float lse = l_run[hlf] > 0.f ? (m_run[hlf] + log2f(l_run[hlf])) * 0.6931471805599453f : -INFINITY;
      const int64_t lo = p.seqstart_q != nullptr ? int64_t(g) * p.lse_stride_g + int64_t(h) * p.lse_stride_h + q_row0 + i
                                                 : int64_t(b) * p.lse_stride_b + int64_t(g) * p.lse_stride_g + int64_t(h) * p.lse_stride_h + i;
      p.lse[lo] = lse;
    }
  }
}

template <int DP, bool kBf16>
static int launch_generic_t(const GenericArgs& ga, cudaStream_t stream) {
  const xfb200_prefill_params& p = ga.p;
  auto kern = prefill_generic_kernel<DP, kBf16>;
  const size_t smem = size_t(kGenBM + 2 * kGenBN) * (DP * 2 + 16);
  static bool configured[kMaxDevices] = {false};  // the attribute belongs to the device's context
  if (first_use_on_device(configured)) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    if (e != cudaSuccess) return cuda_fail("prefill(generic): cudaFuncSetAttribute", e);
  }
  dim3 grid((p.mq + kGenBM - 1) / kGenBM, p.groups * p.heads_per_group, p.batch);
  if (grid.x == 0 || grid.y == 0 || grid.z == 0) return XFB200_OK;
  if (grid.y > 65535 || grid.z > 65535) return set_error(XFB200_E_UNSUPPORTED, "prefill(generic): more than 65535 heads or sequences");
  kern<<<grid, kGenThreads, smem, stream>>>(ga);
  return check_launch("prefill_generic_kernel");
}

int prefill_generic_launch(const xfb200_prefill_params* p, cudaStream_t stream) {
  GenericArgs ga;
  ga.p = *p;
  ga.scale_log2 = p->scale * 1.4426950408889634f;
  const bool bf16 = p->dtype == XFB200_BF16;
  const int D = p->head_dim;
  if (D <= 32) return bf16 ? launch_generic_t<32, true>(ga, stream) : launch_generic_t<32, false>(ga, stream);
  if (D <= 64) return bf16 ? launch_generic_t<64, true>(ga, stream) : launch_generic_t<64, false>(ga, stream);
  if (D <= 128) return bf16 ? launch_generic_t<128, true>(ga, stream) : launch_generic_t<128, false>(ga, stream);
  if (D <= 256) return bf16 ? launch_generic_t<256, true>(ga, stream) : launch_generic_t<256, false>(ga, stream);
  return set_error(XFB200_E_UNSUPPORTED, "prefill: head_dim %d > 256", D);
}

}  // namespace xfb
