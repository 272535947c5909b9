// Attention forward (prefill) on the 5th-generation tensor cores of sm_100a.
//
// One CTA = one 128-row query tile of one (sequence, query head).  Warp roles:
//   warp 0      : TMA producer  (Q once; K and V tiles of 128 keys into a 2-deep ring)
//   warp 1      : MMA issuer    (one elected lane issues tcgen05.mma)
//   warps 2..5  : softmax       (thread <-> query row <-> TMEM lane)
// Tensor memory (512 columns): S0 | S1 (fp32 scores, double buffered) | O (fp32).
//   S_j = Q K_j^T        SS-MMA, both operands K-major in 128B-swizzled smem
//   O  += P_j V_j        SS-MMA, P (bf16/f16) K-major from smem, V MN-major as TMA delivered it
// The MMA warp issues S_{j+1} before it waits for P_j, so the tensor pipe works
// on the next scores while the softmax warps work on the current ones.
// The running maximum is only raised when it grows by more than 2^8 (the
// accumulator rescale is a TMEM round trip), which keeps exp2 arguments <= 8.
//
// Masks: none / causal top-left / causal bottom-right (+ key offset for
// sequence-sharded keys, + left window); tiles that are entirely masked are
// never loaded or multiplied; GQA/MQA by indexing the KV head in the TMA
// coordinate, K/V are never expanded.
//
// Every mbarrier wait is bounded; on a timeout the CTA records a code in the
// device status word, drains, frees its tensor memory and returns.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "internal.h"
#include "prefill_sm100.h"
#include "ptx.cuh"

namespace xfb {

constexpr int kBM = 128;  // query rows per CTA
constexpr int kBN = 128;  // keys per tile
constexpr int kStages = 2;
constexpr int kSoftmaxWarps = 4;
constexpr int kThreads = (2 + kSoftmaxWarps) * 32;
constexpr float kRescaleThreshold = 8.0f;  // log2 units

struct __align__(8) Sm100Barriers {
  uint64_t q_full;
  uint64_t k_full[kStages], v_full[kStages], k_empty[kStages], v_empty[kStages];
  uint64_t s_full[2], s_free[2];
  uint64_t p_full, pv_done;
  uint32_t tmem_base;
  uint32_t abort_flag;
};

template <int D>
struct Sm100Smem {
  static constexpr int kQBytes = kBM * D * 2;
  static constexpr int kKVBytes = kBN * D * 2;
  static constexpr int kPBytes = kBM * kBN * 2;
  static constexpr int kQ = 0;
  static constexpr int kK = kQ + kQBytes;
  static constexpr int kV = kK + kStages * kKVBytes;
  static constexpr int kP = kV + kStages * kKVBytes;
  static constexpr int kBar = kP + kPBytes;
  static constexpr int kTotal = kBar + 256 + 1024;  // + slack to align the base to 1024 B
};

template <int D, bool kBf16>
__global__ void __launch_bounds__(kThreads, 1) prefill_sm100_kernel(const __grid_constant__ Sm100Args a) {
  using L = Sm100Smem<D>;
  constexpr int kHalves = D / 64;          // 64-element (128-byte) column blocks of Q/K/V
  constexpr uint32_t kHalfBytes = 128 * 128;  // 128 rows x 128 B
  extern __shared__ uint8_t smem_dyn[];
  uint8_t* smem = smem_dyn + ((1024u - (smem_u32(smem_dyn) & 1023u)) & 1023u);  // an offset, so that the compiler keeps seeing shared memory
  Sm100Barriers* bar = reinterpret_cast<Sm100Barriers*>(smem + L::kBar);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qt = a.q_tiles - 1 - int(blockIdx.x);  // heaviest (latest) query tiles first
  const int gh = blockIdx.y;
  const int g = gh / a.heads_per_group, h = gh % a.heads_per_group;
  const int b = blockIdx.z;

  // ---- geometry of this sequence (read from device memory: graph-replay safe)
  int q_row0 = 0, k_row0 = 0, qlen = a.mq, klen = a.mkv, tb = b;
  if (a.seqstart_q != nullptr) {
    q_row0 = a.seqstart_q[b];
    qlen = a.seqstart_q[b + 1] - q_row0;
    k_row0 = a.seqstart_k[b];
    klen = a.seqlen_k != nullptr ? a.seqlen_k[b] : a.seqstart_k[b + 1] - k_row0;
    tb = 0;
  }
  const int m0 = qt * kBM;
  if (m0 >= qlen) return;
  const bool causal = a.mask_type != XFB200_MASK_NONE;
  const int shift = (a.mask_type == XFB200_MASK_CAUSAL_BOTTOM_RIGHT ? klen - qlen : 0) - a.kv_offset;
  int n_hi = klen;
  if (causal) n_hi = min(n_hi, m0 + kBM + shift);
  int n_lo = 0;
  if (a.window_left >= 0) n_lo = max(0, m0 + shift - a.window_left) / kBN * kBN;
  const int n_tiles = n_hi > n_lo ? (n_hi - n_lo + kBN - 1) / kBN : 0;
  const int kv_g = g, kv_h = a.kv_h_is_broadcast ? 0 : h;

  // ---- set-up
  if (threadIdx.x == 0) {
    mbar_init(&bar->q_full, 1);
    for (int i = 0; i < kStages; ++i) {
      mbar_init(&bar->k_full[i], 1);
      mbar_init(&bar->v_full[i], 1);
      mbar_init(&bar->k_empty[i], 1);
      mbar_init(&bar->v_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bar->s_full[i], 1);
      mbar_init(&bar->s_free[i], kSoftmaxWarps * 32);
    }
    mbar_init(&bar->p_full, kSoftmaxWarps * 32);
    mbar_init(&bar->pv_done, 1);
    bar->abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(&bar->tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bar->tmem_base;
  const uint32_t tmem_s[2] = {tmem, tmem + 128};
  const uint32_t tmem_o = tmem + 256;
  volatile uint32_t* abort_flag = &bar->abort_flag;

  if (warp == 0) {
    // ============================================================ TMA producer
    if (lane == 0 && n_tiles > 0) {
      prefetch_tensormap(&a.tm_q);
      prefetch_tensormap(&a.tm_k);
      prefetch_tensormap(&a.tm_v);
      mbar_expect_tx(&bar->q_full, L::kQBytes);
#pragma unroll
      for (int hf = 0; hf < kHalves; ++hf)
        tma_load_4d(smem + L::kQ + hf * kHalfBytes, &a.tm_q, &bar->q_full, hf * 64, g * a.heads_per_group + h, q_row0 + m0, tb);
      for (int j = 0; j < n_tiles; ++j) {
        const int st = j % kStages, use = j / kStages;
        const int row = k_row0 + n_lo + j * kBN;
        if (use > 0 && !mbar_wait(&bar->k_empty[st], (use - 1) & 1, abort_flag)) {
          atomicExch(a.status, 11);
          *abort_flag = 1;
          break;
        }
        mbar_expect_tx(&bar->k_full[st], L::kKVBytes);
#pragma unroll
        for (int hf = 0; hf < kHalves; ++hf)
          tma_load_4d(smem + L::kK + st * L::kKVBytes + hf * kHalfBytes, &a.tm_k, &bar->k_full[st], hf * 64,
                      kv_g * (a.kv_h_is_broadcast ? 1 : a.heads_per_group) + kv_h, row, tb);
        if (use > 0 && !mbar_wait(&bar->v_empty[st], (use - 1) & 1, abort_flag)) {
          atomicExch(a.status, 12);
          *abort_flag = 1;
          break;
        }
        mbar_expect_tx(&bar->v_full[st], L::kKVBytes);
#pragma unroll
        for (int hf = 0; hf < kHalves; ++hf)
          tma_load_4d(smem + L::kV + st * L::kKVBytes + hf * kHalfBytes, &a.tm_v, &bar->v_full[st], hf * 64,
                      kv_g * (a.kv_h_is_broadcast ? 1 : a.heads_per_group) + kv_h, row, tb);
      }
    }
  } else if (warp == 1) {
    // ============================================================== MMA issuer
    constexpr uint32_t idesc_qk = umma_idesc(kBM, kBN, kBf16, false, false);
    constexpr uint32_t idesc_pv = umma_idesc(kBM, D, kBf16, false, true);
    const uint32_t q_addr = smem_u32(smem + L::kQ);
    const uint32_t p_addr = smem_u32(smem + L::kP);
    bool ok = true;

    auto issue_qk = [&](int j) {
      const int st = j % kStages;
      const uint32_t k_addr = smem_u32(smem + L::kK + st * L::kKVBytes);
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        const uint32_t off = (kk / 4) * kHalfBytes + (kk % 4) * 32;
        umma_ss(tmem_s[j & 1], umma_desc_sw128(q_addr + off, 16, 1024), umma_desc_sw128(k_addr + off, 16, 1024), idesc_qk, kk > 0);
      }
    };

    if (n_tiles > 0) {
      ok = mbar_wait(&bar->q_full, 0, abort_flag) && mbar_wait(&bar->k_full[0], 0, abort_flag);
      if (!ok && lane == 0) atomicExch(a.status, 21);
      if (ok) {
        tc_fence_after();
        if (lane == 0) {
          issue_qk(0);
          tc_commit(&bar->s_full[0]);
          tc_commit(&bar->k_empty[0]);
        }
        __syncwarp();
      }
      for (int j = 0; ok && j < n_tiles; ++j) {
        const int st = j % kStages, use = j / kStages;
        if (j + 1 < n_tiles) {
          const int j1 = j + 1, st1 = j1 % kStages, use1 = j1 / kStages;
          ok = mbar_wait(&bar->k_full[st1], use1 & 1, abort_flag);
          if (ok && j1 >= 2) ok = mbar_wait(&bar->s_free[j1 & 1], ((j1 >> 1) - 1) & 1, abort_flag);
          if (!ok) {
            if (lane == 0) atomicExch(a.status, 22);
            break;
          }
          tc_fence_after();
          if (lane == 0) {
            issue_qk(j1);
            tc_commit(&bar->s_full[j1 & 1]);
            tc_commit(&bar->k_empty[st1]);
          }
          __syncwarp();
        }
        ok = mbar_wait(&bar->v_full[st], use & 1, abort_flag);
        if (!ok) {
          if (lane == 0) atomicExch(a.status, 23);
          break;
        }
        // keys past the end of the sequence: their V rows may hold anything
        // (next sequence, padding, NaN); P is exactly 0 there, so zero the rows
        const int n0 = n_lo + j * kBN;
        if (n0 + kBN > klen) {
          const int first = max(klen - n0, 0);
          uint8_t* vt = smem + L::kV + st * L::kKVBytes;
          for (int hf = 0; hf < kHalves; ++hf)
            for (int i = first * 8 + lane; i < kBN * 8; i += 32)
              *reinterpret_cast<uint4*>(vt + hf * kHalfBytes + i * 16) = make_uint4(0, 0, 0, 0);
          fence_proxy_async_smem();
          __syncwarp();
        }
        ok = mbar_wait(&bar->p_full, j & 1, abort_flag);
        if (!ok) {
          if (lane == 0) atomicExch(a.status, 24);
          break;
        }
        tc_fence_after();
        if (lane == 0) {
          const uint32_t v_addr = smem_u32(smem + L::kV + st * L::kKVBytes);
#pragma unroll
          for (int kk = 0; kk < kBN / 16; ++kk) {
            const uint64_t pd = umma_desc_sw128(p_addr + (kk / 4) * kHalfBytes + (kk % 4) * 32, 16, 1024);
            const uint64_t vd = umma_desc_sw128(v_addr + kk * 16 * 128, kHalfBytes, 1024);
            umma_ss(tmem_o, pd, vd, idesc_pv, (j > 0 || kk > 0) ? 1u : 0u);
          }
          tc_commit(&bar->pv_done);
          tc_commit(&bar->v_empty[st]);
        }
        __syncwarp();
      }
      if (!ok) *abort_flag = 1;
    }
  } else {
    // ================================================================ softmax
    const int row = (warp & 3) * 32 + lane;  // TMEM lane == query row inside the tile
    const uint32_t lane_sel = uint32_t((warp & 3) * 32) << 16;
    const int i_loc = m0 + row;  // query index inside the sequence
    const int col_hi = causal ? min(klen, i_loc + shift + 1) : klen;
    const int col_lo = a.window_left >= 0 ? i_loc + shift - a.window_left : 0;
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;

    for (int j = 0; j < n_tiles; ++j) {
      const int n0 = n_lo + j * kBN;
      ok = mbar_wait(&bar->s_full[j & 1], (j >> 1) & 1, abort_flag);
      if (!ok) {
        atomicExch(a.status, 31);
        break;
      }
      tc_fence_after();
      uint32_t sr[kBN];
#pragma unroll
      for (int cblk = 0; cblk < kBN / 32; ++cblk) {
        uint32_t* dst = sr + cblk * 32;
        XFB_TMEM_LD_32(tmem_s[j & 1] + lane_sel + cblk * 32, dst);
      }
      tc_wait_ld();
      tc_fence_before();
      mbar_arrive(&bar->s_free[j & 1]);

      float* s = reinterpret_cast<float*>(sr);
      const bool need_mask = (n0 + kBN > klen) || (causal && n0 + kBN - 1 > m0 + shift) ||
                             (a.window_left >= 0 && n0 < m0 + kBM - 1 + shift - a.window_left);
      if (need_mask) {
#pragma unroll
        for (int cidx = 0; cidx < kBN; ++cidx) {
          const int col = n0 + cidx;
          s[cidx] = (col >= col_lo && col < col_hi) ? s[cidx] : -INFINITY;
        }
      }
      float mx = -INFINITY;
#pragma unroll
      for (int cidx = 0; cidx < kBN; ++cidx) mx = fmaxf(mx, s[cidx]);
      mx *= a.scale_log2;  // scale > 0 is guaranteed by the host side
      // raise the running maximum only when it moved by more than the threshold
      float alpha = 1.f;
      bool raise = mx > m_run + kRescaleThreshold || (m_run == -INFINITY && mx > -INFINITY);
      const float m_new = raise ? mx : m_run;
      if (raise) alpha = m_run == -INFINITY ? 0.f : fast_exp2(m_run - m_new);
      const float m_use = m_new == -INFINITY ? 0.f : m_new;

      // P tile (and O) are in use by PV_{j-1} until it completes
      if (j > 0) {
        ok = mbar_wait(&bar->pv_done, (j - 1) & 1, abort_flag);
        if (!ok) {
          atomicExch(a.status, 32);
          break;
        }
        tc_fence_after();
      }
      if (j > 0 && __any_sync(0xffffffffu, raise)) {
#pragma unroll
        for (int cblk = 0; cblk < D / 32; ++cblk) {
          uint32_t orr[32];
          XFB_TMEM_LD_32(tmem_o + lane_sel + cblk * 32, orr);
          tc_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) orr[i] = __float_as_uint(__uint_as_float(orr[i]) * alpha);
          XFB_TMEM_ST_32(tmem_o + lane_sel + cblk * 32, orr);
        }
        tc_wait_st();
      }
      l_run *= alpha;
      m_run = m_new;

      float psum = 0.f;
      uint8_t* prow = smem + L::kP + row * 128;
#pragma unroll
      for (int ch = 0; ch < kBN / 8; ++ch) {
        uint32_t w[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float p0 = fast_exp2(fmaf(s[ch * 8 + 2 * e], a.scale_log2, -m_use));
          const float p1 = fast_exp2(fmaf(s[ch * 8 + 2 * e + 1], a.scale_log2, -m_use));
          psum += p0 + p1;
          if constexpr (kBf16) {
            __nv_bfloat162 t = __floats2bfloat162_rn(p0, p1);
            w[e] = *reinterpret_cast<uint32_t*>(&t);
          } else {
            __half2 t = __floats2half2_rn(p0, p1);
            w[e] = *reinterpret_cast<uint32_t*>(&t);
          }
        }
        // K-major, 128B swizzle: 16-byte chunk x of row r sits at chunk x ^ (r % 8)
        const int half = ch / 8, x = ch % 8;
        *reinterpret_cast<uint4*>(prow + half * kHalfBytes + ((x ^ (row & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
      }
      l_run += psum;
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(&bar->p_full);
    }

    // ---- epilogue: O / l -> global, LSE
    if (ok && n_tiles > 0) {
      ok = mbar_wait(&bar->pv_done, (n_tiles - 1) & 1, abort_flag);
      if (!ok) atomicExch(a.status, 33);
      tc_fence_after();
    }
    const bool valid_row = i_loc < qlen;
    const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
    const int64_t o_off = int64_t(tb) * a.os.b + int64_t(q_row0 + i_loc) * a.os.m + int64_t(g) * a.os.g + int64_t(h) * a.os.h;
#pragma unroll
    for (int cblk = 0; cblk < D / 32; ++cblk) {
      uint32_t orr[32];
      if (ok && n_tiles > 0) {
        XFB_TMEM_LD_32(tmem_o + lane_sel + cblk * 32, orr);
        tc_wait_ld();
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) orr[i] = 0;
      }
      if (valid_row) {
        if (a.out_dtype == XFB200_F32) {
          float* dst = reinterpret_cast<float*>(a.out) + o_off + cblk * 32;
#pragma unroll
          for (int i = 0; i < 32; i += 4)
            *reinterpret_cast<float4*>(dst + i) = make_float4(__uint_as_float(orr[i]) * inv, __uint_as_float(orr[i + 1]) * inv,
                                                              __uint_as_float(orr[i + 2]) * inv, __uint_as_float(orr[i + 3]) * inv);
        } else {
          uint16_t* dst = reinterpret_cast<uint16_t*>(a.out) + o_off + cblk * 32;
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint32_t w[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float x0 = __uint_as_float(orr[i + 2 * e]) * inv, x1 = __uint_as_float(orr[i + 2 * e + 1]) * inv;
              if (a.out_dtype == XFB200_BF16) {
                __nv_bfloat162 t = __floats2bfloat162_rn(x0, x1);
                w[e] = *reinterpret_cast<uint32_t*>(&t);
              } else {
                __half2 t = __floats2half2_rn(x0, x1);
                w[e] = *reinterpret_cast<uint32_t*>(&t);
              }
            }
            *reinterpret_cast<uint4*>(dst + i) = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      }
    }
    if (valid_row && a.lse != nullptr) {
      const float lse = l_run > 0.f ? (m_run + log2f(l_run)) * 0.6931471805599453f : -INFINITY;
      const int64_t lo = a.seqstart_q != nullptr ? int64_t(g) * a.lse_g + int64_t(h) * a.lse_h + q_row0 + i_loc
                                                 : int64_t(b) * a.lse_b + int64_t(g) * a.lse_g + int64_t(h) * a.lse_h + i_loc;
      a.lse[lo] = lse;
    }
    tc_fence_before();
  }

  // ---- teardown: everyone is done with tensor memory before it is freed
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

// ------------------------------------------------------------------ host side
// Tensor map over [D, heads, rows, batch] (innermost first); box = 64 x 1 x box_rows x 1, 128B swizzle.
static int make_map(CUtensorMap* tm, const void* base, int dtype, int D, int64_t heads, int64_t head_stride, int64_t rows,
                    int64_t row_stride, int64_t batch, int64_t batch_stride, const char* what, int box_rows = 128) {
  EncodeTiledFn enc = encode_tiled_fn();
  if (enc == nullptr) return set_error(XFB200_E_CUDA, "prefill: cuTensorMapEncodeTiled is not available from this driver");
  const cuuint64_t dims[4] = {cuuint64_t(D), cuuint64_t(heads), cuuint64_t(rows), cuuint64_t(batch)};
  // a dimension of extent 1 never contributes to an address; give it a legal stride
  auto st = [&](int64_t s, int64_t extent) { return cuuint64_t((extent > 1 ? s : int64_t(D)) * 2); };
  const cuuint64_t strides[3] = {st(head_stride, heads), st(row_stride, rows), st(batch_stride, batch)};
  const cuuint32_t box[4] = {64, 1, cuuint32_t(box_rows), 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(tm, dtype == XFB200_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4,
                   const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return set_error(XFB200_E_CUDA, "prefill: cuTensorMapEncodeTiled(%s) failed with CUresult %d", what, int(r));
  return XFB200_OK;
}

static int32_t* prefill_status_word() {
  static int32_t* words[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (words[dev] == nullptr) {
    int32_t* p = nullptr;
    if (cudaMalloc(&p, 256) != cudaSuccess) return nullptr;
    cudaMemset(p, 0, 256);
    words[dev] = p;
  }
  return words[dev];
}

// Heads of q form one tensor-map dimension only if (g, h) flatten to a single stride.
static bool heads_flatten(const xfb200_strides& s, int G, int H, int64_t* stride, int64_t* count) {
  if (G == 1) { *stride = s.h; *count = H; return true; }
  if (H == 1) { *stride = s.g; *count = G; return true; }
  if (s.g == s.h * H) { *stride = s.h; *count = int64_t(G) * H; return true; }
  return false;
}

int prefill_sm100_supported(const xfb200_prefill_params* p) {
  if (p->head_dim != 64 && p->head_dim != 128) return 0;
  if (!(p->scale > 0.f)) return 0;
  if (p->mq < 1 || p->batch < 1) return 0;
  int64_t hs, hc;
  if (!heads_flatten(p->q_strides, p->groups, p->heads_per_group, &hs, &hc)) return 0;
  const bool kbc = p->heads_per_group > 1 && p->k_strides.h == 0;
  if (kbc != (p->heads_per_group > 1 && p->v_strides.h == 0)) return 0;
  if (!kbc && !(heads_flatten(p->k_strides, p->groups, p->heads_per_group, &hs, &hc) &&
                heads_flatten(p->v_strides, p->groups, p->heads_per_group, &hs, &hc)))
    return 0;
  auto al = [](int64_t e) { return (e * 2) % 16 == 0; };
  const xfb200_strides* ss[3] = {&p->q_strides, &p->k_strides, &p->v_strides};
  for (auto s : ss)
    if (!al(s->b) || !al(s->m) || !al(s->g) || !al(s->h)) return 0;
  if ((reinterpret_cast<uintptr_t>(p->q) | reinterpret_cast<uintptr_t>(p->k) | reinterpret_cast<uintptr_t>(p->v) |
       reinterpret_cast<uintptr_t>(p->out)) & 15)
    return 0;
  const int osz = p->out_dtype == XFB200_F32 ? 4 : 2;
  if ((p->o_strides.b * osz) % 16 || (p->o_strides.m * osz) % 16 || (p->o_strides.g * osz) % 16 || (p->o_strides.h * osz) % 16) return 0;
  return 1;
}

template <int D, bool kBf16>
static int launch_sm100_t(const Sm100Args& a, cudaStream_t stream) {
  auto kern = prefill_sm100_kernel<D, kBf16>;
  constexpr int smem = Sm100Smem<D>::kTotal;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return cuda_fail("prefill(sm100): cudaFuncSetAttribute", e);
    configured = true;
  }
  dim3 grid(a.q_tiles, a.groups * a.heads_per_group, a.batch);
  if (grid.y > 65535 || grid.z > 65535) return set_error(XFB200_E_UNSUPPORTED, "prefill: more than 65535 heads or sequences");
  kern<<<grid, kThreads, smem, stream>>>(a);
  return check_launch("prefill_sm100_kernel");
}

int prefill_sm100_launch(const xfb200_prefill_params* p, cudaStream_t stream) {
  Sm100Args a{};
  const int G = p->groups, H = p->heads_per_group, D = p->head_dim;
  const bool varlen = p->seqstart_q != nullptr;
  int64_t hs = 0, hc = 0;
  heads_flatten(p->q_strides, G, H, &hs, &hc);
  const int64_t q_rows = varlen ? p->total_q : p->mq;
  const int64_t k_rows = p->mkv;
  const int64_t nb = varlen ? 1 : p->batch;
  int rc = make_map(&a.tm_q, p->q, p->dtype, D, hc, hs, q_rows, p->q_strides.m, nb, p->q_strides.b, "q");
  if (rc) return rc;
  const bool kbc = H > 1 && p->k_strides.h == 0;
  int64_t khs = p->k_strides.g, khc = G, vhs = p->v_strides.g;
  if (!kbc) {
    heads_flatten(p->k_strides, G, H, &khs, &khc);
    heads_flatten(p->v_strides, G, H, &vhs, &khc);
  }
  // keys per K/V copy: 128 (a tile of the 128-key kernels) or 64 (a stage of the 64-key-step kernel)
  const int kv_box = prefill_path_override() == 5 ? 64 : 128;
  rc = make_map(&a.tm_k, p->k, p->dtype, D, khc, khs, k_rows, p->k_strides.m, nb, p->k_strides.b, "k", kv_box);
  if (rc) return rc;
  rc = make_map(&a.tm_v, p->v, p->dtype, D, khc, vhs, k_rows, p->v_strides.m, nb, p->v_strides.b, "v", kv_box);
  if (rc) return rc;
  a.out = p->out, a.lse = p->lse;
  a.seqstart_q = p->seqstart_q, a.seqstart_k = p->seqstart_k, a.seqlen_k = p->seqlen_k;
  a.status = prefill_status_word();
  if (a.status == nullptr) return set_error(XFB200_E_CUDA, "prefill: cannot allocate the device status word");
  a.batch = p->batch, a.mq = p->mq, a.mkv = p->mkv, a.groups = G, a.heads_per_group = H;
  a.kv_h_is_broadcast = kbc ? 1 : 0;
  a.os = p->o_strides;
  a.lse_b = p->lse_stride_b, a.lse_g = p->lse_stride_g, a.lse_h = p->lse_stride_h;
  a.mask_type = p->mask_type, a.kv_offset = p->kv_offset, a.window_left = p->window_left, a.out_dtype = p->out_dtype;
  a.scale_log2 = p->scale * 1.4426950408889634f;
  a.q_tiles = (p->mq + kBM - 1) / kBM;
  const bool bf16 = p->dtype == XFB200_BF16;
  if (prefill_path_override() != 3) {
    a.q_tiles = (p->mq + 255) / 256;
    if (prefill_path_override() == 5) return prefill_sm100_s64_launch(a, D, bf16, stream);
    return prefill_sm100_m256_launch(a, D, bf16, stream);
  }
  if (D == 128) return bf16 ? launch_sm100_t<128, true>(a, stream) : launch_sm100_t<128, false>(a, stream);
  return bf16 ? launch_sm100_t<64, true>(a, stream) : launch_sm100_t<64, false>(a, stream);
}

}  // namespace xfb

extern "C" int xfb200_prefill_device_status(void* stream, int32_t* status_out) {
  using namespace xfb;
  if (status_out == nullptr) return set_error(XFB200_E_INVALID, "status_out is null");
  int32_t* w = prefill_status_word();
  if (w == nullptr) return set_error(XFB200_E_CUDA, "cannot allocate the device status word");
  cudaError_t e = cudaMemcpyAsync(status_out, w, sizeof(int32_t), cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream));
  if (e == cudaSuccess) e = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail("prefill_device_status", e);
  return XFB200_OK;
}

