// Split-K decode attention: few queries per sequence against a long KV cache.
//
// HBM-bound.  One CTA owns (sequence b, key chunk s, block of kv heads): a
// producer warp streams that chunk of the cache into a 3-deep shared-memory
// ring with 1-D bulk TMA copies (whole token stripes, all heads of the block
// at once when they are contiguous, so every request is >= 256 B and
// 16-B aligned), 8 consumer warps do QK^T and PV with warp-level
// mma.sync.m16n8k16 (query heads of a GQA group are the M rows, tokens the N
// columns; K/V are never expanded), the online softmax lives in registers.
// The int4 row-wise cache is unpacked in registers: nibbles become bf16/f16
// values 16 + n by one shift+lop3 per element pair, and scale/shift are folded
// into the scores (K) and into the probabilities (V) so no per-element FMA is
// spent on dequantisation.
//
// Each CTA writes a normalised partial (O_s fp32, LSE_s) to caller-provided
// scratch; the row-merge kernel (merge.cu arithmetic) combines the chunks that
// exist for each sequence in a fixed order, so results are bit-reproducible.
// Lengths and page tables are read from device memory at run time; the grid
// depends on static bounds only.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "internal.h"
#include "ptx.cuh"

namespace xfb {

constexpr int kDecConsumerWarps = 8;
constexpr int kDecThreads = (kDecConsumerWarps + 1) * 32;
constexpr int kDecChunkAlign = 128;  // chunk size granularity in tokens (= largest stage)

struct DecodeArgs {
  // copy_mode 3 only: the K and V caches as 3-D tensors {64 elements, token rows, 128-byte column groups}
  CUtensorMap tm_k, tm_v;
  // fp8 with ss_tma: the scale/shift words as 3-D int32 tensors {4 words, kv heads, token rows}
  CUtensorMap tm_kss, tm_vss;
  const void* q;
  const void* k;
  const void* v;
  void* out;
  float* lse;
  float* part_o;    // [batch, split, kv_heads, R, D]
  float* part_lse;  // [batch, split, kv_heads, R]
  int32_t* status;  // device status word (timed-out waits)
  const int32_t* seqlen_k;
  const int32_t* kv_start;  // gappy caches: first key row of every sequence (padded: absolute row; paged: row inside its block table)
  const int32_t* block_tables;
  int32_t batch, mq, kv_heads, q_per_kv;
  int32_t kv_padding, page_size, bt_stride;
  int32_t split_k, chunk_tokens;
  int32_t hb;          // kv heads per CTA (1, 2, 4 or 8)
  int32_t rows;        // R = mq * q_per_kv
  int32_t row_blocks;  // ceil(R / (16*MT))
  int32_t copy_mode;   // 0: one bulk copy per token stripe of hb heads; 1: per (token, head); 2: word copies (no TMA);
                       // 3: tiled TMA, a whole run of tokens per copy, 128-byte swizzled in shared memory (16-bit cache)
  int32_t box_tok;     // mode 3: tokens per tiled copy (power of two, 8..256, divides the stage)
  int32_t kv_bytes;    // bytes of the K (or V) part of a stage
  int32_t stage_bytes; // bytes of a whole stage (K part, V part, fp8: the scale/shift words of both)
  const int32_t* k_ss; // fp8: scale/shift words of K and V, strides in words
  const int32_t* v_ss;
  int64_t kss_m, kss_g, vss_m, vss_g;
  int32_t ss_tma;      // fp8: the scale/shift words come by tiled copies: 1 = 16 bytes per (token, head), the word first;
                       // 2 = compact tensors, the words of the hb heads of a token adjacent
  int32_t ss_bytes;    // fp8: bytes of the scale/shift words of K (or V) in a stage
  int32_t copy_group;  // tokens per bulk copy (int4 only, mode 0)
  int32_t stages;         // depth of the shared-memory ring
  int32_t q_first_stage;  // stages >= this one hold the staged Q until q_done
  int64_t q_sm, q_sg, q_sh;
  int64_t k_sm, k_sg, v_sm, v_sg;
  int64_t o_sm, o_sg, o_sh;
  int64_t lse_sg, lse_sh;
  int32_t causal;
  int32_t out_dtype;
  float scale_log2;
  int32_t window_size;  // 0: none; else query i of a sequence sees the window_size keys that end at its own position
  int32_t window_span;  // window_size + mq - 1: the keys any query of a sequence sees (0 without a window)
  // additive bias (16-bit cache, plain layout): element strides of [batch, kv_heads, q_per_kv, mq, keys]; bias / scale is
  // added to q k^T, so that the softmax sees q k^T * scale + bias
  const void* bias;
  int32_t bias_dtype;
  float inv_scale;
  int64_t bias_b, bias_kvh, bias_q, bias_m;
};

template <bool kBf16>
struct Half2Type;
template <>
struct Half2Type<true> {
  using T = __nv_bfloat16;
  using T2 = __nv_bfloat162;
};
template <>
struct Half2Type<false> {
  using T = __half;
  using T2 = __half2;
};

template <bool kBf16>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  if constexpr (kBf16) {
    __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&t);
  } else {
    __half2 t = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&t);
  }
}
template <bool kBf16>
__device__ __forceinline__ float2 unpack2(uint32_t x) {
  if constexpr (kBf16) {
    return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&x));
  } else {
    return __half22float2(*reinterpret_cast<__half2*>(&x));
  }
}
__device__ __forceinline__ float half_bits_to_float(uint32_t bits16) {
  return __half2float(__ushort_as_half(static_cast<unsigned short>(bits16)));
}

// Shared-memory geometry of one stage.
// cache formats (the template parameter kFmt of what follows)
constexpr int kFmtPlain = 0, kFmtInt4 = 1, kFmtFp8 = 2;
// the plain layout read by the variant of its consumer that knows additive biases and per-row lower limits (windows with
// several queries per sequence): a kernel of its own, so that the common one stays as lean as it is
constexpr int kFmtPlainX = 3;

template <int D, int kFmt, int NG = 1>
struct DecStage {
  // plain: one row per token = hb heads * D elements (+16 B pad against bank conflicts; unpadded and
  //        swizzled when the stage is filled by a tiled copy)
  // int4 : one row per token = hb heads * (NG + D/8) words (NG quantisation groups), unpadded
  // fp8  : [head][token][D bytes] boxes (tiled copy, 128-byte swizzle), then the scale/shift words
  __host__ __device__ static int row_bytes(int hb) {
    return kFmt == kFmtInt4 ? hb * (NG + D / 8) * 4 : kFmt == kFmtFp8 ? hb * D : hb * D * 2 + 16;
  }
  // sub-tiles of 16 tokens each warp takes from one stage: the int4 cache is 4x
  // denser, so its stages hold more tokens to keep the per-stage overhead
  // (barrier round trip, page-table look-ups of the producer) off the critical path
#ifndef XFB_FP8_SUBTILES
#define XFB_FP8_SUBTILES 1
#endif
#ifndef XFB_FP8_CTAS
#define XFB_FP8_CTAS 2
#endif
  static constexpr int kSubTiles = kFmt == kFmtInt4 ? 2 : kFmt == kFmtFp8 ? XFB_FP8_SUBTILES : 1;
  __host__ __device__ static int tokens(int hb) { return 16 * kSubTiles * (kDecConsumerWarps / hb); }
  __host__ __device__ static int kv_bytes(int hb) {  // K or V part of a stage, rounded to 128 B
    return (row_bytes(hb) * tokens(hb) + 127) & ~127;
  }
  // fp8: scale/shift words of the K (or V) rows of a stage, one per token and head
  __host__ __device__ static int ss_bytes(int hb) { return kFmt == kFmtFp8 ? tokens(hb) * hb * 4 : 0; }
};

constexpr int kDecMaxStages = 12;
// Bytes of cache in flight per SM are what hide the HBM latency.  The 16-bit
// kernel runs one CTA per SM with a ~212 KB ring.  The int4 kernel does 4x the
// arithmetic per byte and each warp's sub-tile is one long dependency chain, so
// it runs two CTAs per SM (twice the warps to interleave) with half the ring each;
// so does the fp8 kernel, which shares its structure.
template <int kFmt>
struct DecOccupancy {
  static constexpr int kCtasPerSm = kFmt == kFmtInt4 ? 2 : kFmt == kFmtFp8 ? XFB_FP8_CTAS : 1;
  static constexpr int kRingBudget = kCtasPerSm == 2 ? 108 * 1024 : 212 * 1024;
};

// What a consumer warp needs to know about its CTA.
struct DecWarp {
  const uint8_t* qs;          // this warp's staged Q rows (ROWS x D, 16-bit)
  const uint8_t* stage_base;  // the ring
  uint64_t* full_bar;
  uint64_t* empty_bar;
  uint64_t* q_done_bar;
  float* mine;  // this warp's slot of the combine area: [ROWS][D + 2]
  int lane, hw, sub, wph, row0;
  int b, head;  // sequence and kv head of this warp
  int chunk_lo, chunk_hi, kv_len, n_tiles;
  int tok_per_stage, kv_bytes, stage_bytes, row_bytes, stages;
};

__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t x) {
  uint32_t y;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(y) : "r"(x));
  return y;
}

// ---------------------------------------------------------------------------
// 16-bit cache.  Query rows (heads of the GQA group x queries) are the M rows
// of the MMAs, tokens the N columns of QK^T and the K dimension of PV.
// Leaves the un-normalised partial (acc, running max, row sum) in w.mine.
// ---------------------------------------------------------------------------
template <int D, int MT, bool kBf16, bool kExtras>
__device__ __forceinline__ void consume_plain(const DecodeArgs& a, const DecWarp& w) {
  constexpr int KS = D / 16;  // k-steps of the QK^T product
  constexpr int NT = D / 8;   // n-tiles of the PV product
  constexpr int kCmbRow = D + 2;
  constexpr int kSps = DecStage<D, kFmtPlain>::kSubTiles;
  const int lane = w.lane, r = lane >> 2, c = lane & 3;
  const int R = a.rows, hw = w.hw, row_bytes = w.row_bytes;
  // Tiled copies leave a stage as boxes of [column group][token][128 B] with the
  // 16-byte chunks of every row XOR-ed by (token & 7); bulk copies leave padded
  // token rows.  Either way ldmatrix sees no bank conflicts.
  const bool swz = a.copy_mode == 3;
  const int box_shift = __ffs(a.box_tok) - 1;
  const int cg_stride = a.box_tok * 128;
  const int box_bytes = cg_stride * (a.hb * (D / 64));

  // A fragments of Q straight from global memory (rows r and r + 8 of each
  // m-tile, element pairs 2c and 2c + 8 of each k-step); rows beyond R are zero.
  uint32_t qf[MT][KS][4];
  {
    using T = typename Half2Type<kBf16>::T;
    const T* qg = reinterpret_cast<const T*>(a.q);
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int hlf = 0; hlf < 2; ++hlf) {
        const int row = w.row0 + mt * 16 + r + hlf * 8;
        const bool live = row < R;
        const int qi = live ? row / a.q_per_kv : 0, h = live ? row % a.q_per_kv : 0;
        const uint32_t* src = reinterpret_cast<const uint32_t*>(
            qg + (int64_t(w.b) * a.mq + qi) * a.q_sm + int64_t(w.head) * a.q_sg + int64_t(h) * a.q_sh + 2 * c);
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
          qf[mt][ks][hlf] = live ? __ldg(src + ks * 8) : 0u;
          qf[mt][ks][2 + hlf] = live ? __ldg(src + ks * 8 + 4) : 0u;
        }
      }
  }

  // per-row visibility limits: token t visible iff lo <= t < lim (lo > 0 only with a window and several queries per sequence)
  int lim[MT][2], lo[MT][2];
  const bool has_lo = kExtras && a.window_size > 0 && a.mq > 1;  // uniform
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int hlf = 0; hlf < 2; ++hlf) {
      const int row = w.row0 + mt * 16 + r + hlf * 8;
      int l = w.chunk_hi, f = 0;
      if (a.causal && row < R) {
        const int own = w.kv_len - a.mq + row / a.q_per_kv + 1;  // one past the row's own position
        l = min(l, own);
        if (has_lo) f = max(own - a.window_size, 0);
      }
      lim[mt][hlf] = l, lo[mt][hlf] = f;
    }

  float acc[MT][NT][4];
  float m_run[MT][2], l_run[MT][2];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
    for (int j = 0; j < NT; ++j) acc[mt][j][0] = acc[mt][j][1] = acc[mt][j][2] = acc[mt][j][3] = 0.f;
    m_run[mt][0] = m_run[mt][1] = -INFINITY;
    l_run[mt][0] = l_run[mt][1] = 0.f;
  }

  for (int tile = 0; tile < w.n_tiles; ++tile) {
    const int st = tile % w.stages;
    if (!mbar_wait(&w.full_bar[st], (tile / w.stages) & 1)) {
      if (lane == 0) atomicCAS(a.status, 0, 2);
      break;
    }
    for (int sp = 0; sp < kSps; ++sp) {
      const int usub = w.sub + w.wph * sp;                                // this warp's sub-tile of the stage
      const int t_sub = w.chunk_lo + tile * w.tok_per_stage + usub * 16;  // its first token
      if (t_sub >= w.chunk_hi) continue;
      const uint8_t* ks_ = w.stage_base + st * w.stage_bytes;
      const uint8_t* vs_ = ks_ + w.kv_bytes;
      const bool ragged = t_sub + 16 > w.chunk_hi;

      // ------------------------------------------------ S = Q K^T (16*MT x 16)
      float s[MT][2][4];
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int j = 0; j < 2; ++j) s[mt][j][0] = s[mt][j][1] = s[mt][j][2] = s[mt][j][3] = 0.f;
      {
        const int tok = usub * 16 + (lane & 7) + (lane >> 4) * 8;
        const int ti = tok & (a.box_tok - 1);
        const uint32_t kaddr = swz ? smem_u32(ks_) + (tok >> box_shift) * box_bytes + hw * (D / 64) * cg_stride + ti * 128
                                   : smem_u32(ks_ + tok * row_bytes + hw * D * 2 + ((lane >> 3) & 1) * 16);
        const int xh = (ti & 7) ^ ((lane >> 3) & 1);
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
          uint32_t kf[4];
          // byte column ks*32 + half*16 of this head: column group ks/4, chunk (2 ks + half) & 7
          ldmatrix_x4(kf, swz ? kaddr + (ks >> 2) * cg_stride + ((((2 * ks) & 7) ^ xh) << 4) : kaddr + ks * 32);
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            mma_16816<kBf16>(s[mt][0], qf[mt][ks], kf[0], kf[1]);
            mma_16816<kBf16>(s[mt][1], qf[mt][ks], kf[2], kf[3]);
          }
        }
      }

      if (kExtras && a.bias != nullptr) {
        // additive bias: one value per (query row, token), read where it lies (plain loads: this path is for small inputs)
        const int esz = a.bias_dtype == XFB200_F32 ? 4 : 2;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
          for (int hlf = 0; hlf < 2; ++hlf) {
            const int row = w.row0 + mt * 16 + r + hlf * 8;
            if (row >= R) continue;
            const uint8_t* brow = reinterpret_cast<const uint8_t*>(a.bias) +
                                  (int64_t(w.b) * a.bias_b + int64_t(w.head) * a.bias_kvh + int64_t(row % a.q_per_kv) * a.bias_q +
                                   int64_t(row / a.q_per_kv) * a.bias_m) * esz;
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
              for (int e = 0; e < 2; ++e) {
                const int t = t_sub + j * 8 + 2 * c + e;
                if (t >= w.chunk_hi) continue;
                float bv;
                if (a.bias_dtype == XFB200_F32) bv = reinterpret_cast<const float*>(brow)[t];
                else if (a.bias_dtype == XFB200_BF16) bv = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(brow)[t]);
                else bv = __half2float(reinterpret_cast<const __half*>(brow)[t]);
                s[mt][j][hlf * 2 + e] = fmaf(bv, a.inv_scale, s[mt][j][hlf * 2 + e]);
              }
          }
      }
      // -------------------------------- scale, mask, online softmax (log2 domain)
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int t = t_sub + j * 8 + 2 * c + e;
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            s[mt][j][e] = t < lim[mt][0] ? s[mt][j][e] * a.scale_log2 : -INFINITY;
            s[mt][j][2 + e] = t < lim[mt][1] ? s[mt][j][2 + e] * a.scale_log2 : -INFINITY;
          }
        }
      if (has_lo && t_sub < a.mq) {
        // (the lower limits lie within the first mq - 1 tokens of the window: one sub-tile or two of the first chunk)
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int t = t_sub + j * 8 + 2 * c + e;
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
              if (t < lo[mt][0]) s[mt][j][e] = -INFINITY;
              if (t < lo[mt][1]) s[mt][j][2 + e] = -INFINITY;
            }
          }
      }

      uint32_t pa[MT][4];
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        float alpha[2];
#pragma unroll
        for (int hlf = 0; hlf < 2; ++hlf) {
          float mx = fmaxf(fmaxf(s[mt][0][2 * hlf], s[mt][0][2 * hlf + 1]), fmaxf(s[mt][1][2 * hlf], s[mt][1][2 * hlf + 1]));
          mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
          mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
          const float m_new = fmaxf(m_run[mt][hlf], mx);
          const float m_use = m_new == -INFINITY ? 0.f : m_new;
          alpha[hlf] = fast_exp2(m_run[mt][hlf] - m_use);  // exp2(-inf) = 0 on the first tile
          m_run[mt][hlf] = m_new;
          const float p00 = fast_exp2(s[mt][0][2 * hlf] - m_use), p01 = fast_exp2(s[mt][0][2 * hlf + 1] - m_use);
          const float p10 = fast_exp2(s[mt][1][2 * hlf] - m_use), p11 = fast_exp2(s[mt][1][2 * hlf + 1] - m_use);
          l_run[mt][hlf] = l_run[mt][hlf] * alpha[hlf] + ((p00 + p01) + (p10 + p11));
          pa[mt][hlf] = pack2<kBf16>(p00, p01);      // k = 2c, 2c+1   (rows r / r+8)
          pa[mt][2 + hlf] = pack2<kBf16>(p10, p11);  // k = 2c+8, 2c+9
        }
        // rescale the running output only when some row's maximum moved
        const bool moved = alpha[0] != 1.f || alpha[1] != 1.f;
        if (__any_sync(0xffffffffu, moved)) {
#pragma unroll
          for (int j = 0; j < NT; ++j) {
            acc[mt][j][0] *= alpha[0];
            acc[mt][j][1] *= alpha[0];
            acc[mt][j][2] *= alpha[1];
            acc[mt][j][3] *= alpha[1];
          }
        }
      }

      // ------------------------------------------------------- O += P V
      if (ragged) {
        // rows of tokens past the end were not copied: zero them so that
        // 0 * garbage cannot produce NaN
        for (int i = lane; i < 16 * (D / 8); i += 32) {
          const int tt = i / (D / 8), ch = i % (D / 8);
          if (t_sub + tt >= w.chunk_hi) {
            const int tk = usub * 16 + tt;
            // (all eight chunks of a 128-byte row are cleared, so the swizzle does not matter)
            const int off = swz ? (tk >> box_shift) * box_bytes + (hw * (D / 64) + (ch >> 3)) * cg_stride + (tk & (a.box_tok - 1)) * 128 + (ch & 7) * 16
                                : tk * row_bytes + hw * D * 2 + ch * 16;
            *reinterpret_cast<uint4*>(const_cast<uint8_t*>(vs_) + off) = make_uint4(0, 0, 0, 0);
          }
        }
        __syncwarp();
      }
      const int tok = usub * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
      const int tiv = tok & (a.box_tok - 1);
      const uint32_t vaddr = swz ? smem_u32(vs_) + (tok >> box_shift) * box_bytes + hw * (D / 64) * cg_stride + tiv * 128
                                 : smem_u32(vs_ + tok * row_bytes + hw * D * 2 + (lane >> 4) * 16);
      const int xv = (tiv & 7) ^ (lane >> 4);
#pragma unroll
      for (int j = 0; j < NT; j += 2) {
        uint32_t vf[4];
        // byte column (j + hi)*16 of this head: column group j/8, chunk (j & 7) | hi
        ldmatrix_x4_trans(vf, swz ? vaddr + (j >> 3) * cg_stride + (((j & 7) ^ xv) << 4) : vaddr + j * 16);
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          mma_16816<kBf16>(acc[mt][j], pa[mt], vf[0], vf[1]);
          mma_16816<kBf16>(acc[mt][j + 1], pa[mt], vf[2], vf[3]);
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&w.empty_bar[st]);
  }

  // full row sums (each thread of a quad saw 4 of the 16 tokens of a tile)
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int hlf = 0; hlf < 2; ++hlf) {
      float l = l_run[mt][hlf];
      l += __shfl_xor_sync(0xffffffffu, l, 1);
      l += __shfl_xor_sync(0xffffffffu, l, 2);
      l_run[mt][hlf] = l;
    }

  // the ring is no longer in use once every consumer warp got here
  asm volatile("bar.sync 1, %0;" ::"n"(kDecConsumerWarps * 32) : "memory");
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int rr = mt * 16 + r + (e >> 1) * 8;
        w.mine[rr * kCmbRow + j * 8 + 2 * c + (e & 1)] = acc[mt][j][e];
      }
    if (c == 0) {
      w.mine[(mt * 16 + r) * kCmbRow + D] = m_run[mt][0];
      w.mine[(mt * 16 + r) * kCmbRow + D + 1] = l_run[mt][0];
      w.mine[(mt * 16 + r + 8) * kCmbRow + D] = m_run[mt][1];
      w.mine[(mt * 16 + r + 8) * kCmbRow + D + 1] = l_run[mt][1];
    }
  }
}

// ---------------------------------------------------------------------------
// int4 row-wise cache.  The integer pipe that unpacks the nibbles is what
// bounds this path, so everything is arranged to spend as few logic
// operations per nibble as possible:
//  * The products are taken transposed: tokens are the M rows of S^T = K Q^T
//    and the K dimension of O^T = V^T P^T, the query rows (8 per n-tile) are
//    the N columns.  One 16-token sub-tile costs D/16 + D/16 MMAs per n-tile
//    and no MMA row is padding when the GQA group has 8 query heads.
//  * Both products run in f16 whatever the type of Q.  With 10 mantissa bits a
//    nibble can be read where it already sits: (w & 0x000F000F) | 0x64006400
//    is the pair (1024 + n_e, 1024 + n_{e+4}) and (w & 0x00F000F0) | 0x64006400
//    the pair (1024 + 16 n), so a word costs one shift (w >> 8, for the upper
//    byte of each half) and four logic operations.  One half2 subtraction or
//    fused multiply-add per pair, on the otherwise idle FMA pipe, brings the
//    values back to exactly n, so the accumulators never see the offset.
//    bf16 queries are converted to f16 after scaling each row by a power of
//    two that keeps it below 2^15; the factor returns with the softmax scale.
//  * K: thread (r, c) reads word 4i + c of tokens r and r + 8; its nibble pairs
//    (e, e + 4) are the k-slots (2c, 2c+1) / (2c+8, 2c+9) of k-steps 2i and
//    2i + 1.  Q^T is loaded in the same permuted order of d.
//  * V: thread (r, c) reads words WPT*r + wi of tokens 2c, 2c+1, 2c+8, 2c+9;
//    a byte permute first puts the same half-word of two neighbouring tokens
//    side by side, so that unpacking yields A-fragment registers directly:
//    m-tile wi*4 + e holds d = 8*(WPT*r + wi) + e in row r, d + 4 in row r + 8.
//  * K's scale and shift are applied to the scores (shift times the row sum
//    of q), V's scale is folded into P and its shift is a per-row term
//    sum_t p_t * shift_t added at the end.  P^T reaches the B operand of the
//    second product through movmatrix.
//  * The running maximum is refreshed (cross-lane reduction, rescaling) only
//    when some score exceeds it by more than 2^8; otherwise probabilities are
//    taken against the stale maximum, which is exact in floating point.
// ---------------------------------------------------------------------------
template <int D, int NTQ, bool kBf16>
__device__ __forceinline__ void consume_int4(const DecodeArgs& a, const DecWarp& w) {
  using T = typename Half2Type<kBf16>::T;
  constexpr int W = 1 + D / 8;  // words per row (scale/shift word + nibbles)
  constexpr int KS = D / 16;    // k-steps of K Q^T
  constexpr int MTV = D / 16;   // m-tiles of V^T P^T
  constexpr int WPT = D / 64;   // V words per thread and token
  constexpr int kQRowBytes = D * 2;
  constexpr int kCmbRow = D + 2;
  constexpr int kSps = DecStage<D, kFmtInt4>::kSubTiles;
  // log2 of the largest probability taken against a stale maximum; P * scale(V)
  // is an f16 value, so 2^kLazy * scale must stay below 65504
  constexpr float kLazy = 4.f;
  const int lane = w.lane, r = lane >> 2, c = lane & 3;
  const int R = a.rows, hw = w.hw, row_bytes = w.row_bytes;

  // nibble pairs (e, e+4), e = 0..3, of a packed word as two f16 values n
  auto unpack4 = [](uint32_t x, uint32_t (&out)[4]) {
    constexpr uint32_t kMagic = 0x64006400u;                   // 1024.0 | 1024.0
    const __half2 k1024 = __half2half2(__ushort_as_half(0x6400));
    const __half2 k64 = __half2half2(__ushort_as_half(0x5400));   // 64.0
    const __half2 k16th = __half2half2(__ushort_as_half(0x2C00));  // 1/16
    const uint32_t hi = x >> 8;
    uint32_t v0 = (x & 0x000F000Fu) | kMagic, v1 = (x & 0x00F000F0u) | kMagic;
    uint32_t v2 = (hi & 0x000F000Fu) | kMagic, v3 = (hi & 0x00F000F0u) | kMagic;
    __half2 h0 = __hsub2(*reinterpret_cast<__half2*>(&v0), k1024);
    __half2 h1 = __hfma2(*reinterpret_cast<__half2*>(&v1), k16th, __hneg2(k64));
    __half2 h2 = __hsub2(*reinterpret_cast<__half2*>(&v2), k1024);
    __half2 h3 = __hfma2(*reinterpret_cast<__half2*>(&v3), k16th, __hneg2(k64));
    out[0] = *reinterpret_cast<uint32_t*>(&h0);
    out[1] = *reinterpret_cast<uint32_t*>(&h1);
    out[2] = *reinterpret_cast<uint32_t*>(&h2);
    out[3] = *reinterpret_cast<uint32_t*>(&h3);
  };

  // B fragments of Q^T (n = query row nt*8 + r) in the permuted order of d, as
  // f16 of q * 2^-k with k chosen per row so that nothing overflows
  uint32_t qf[NTQ][KS][2];
  float qsum[NTQ][2];  // sum over d of the scaled q, for the rows 2c, 2c+1 of each n-tile
  float qfac[NTQ][2];  // 2^k * softmax scale * log2(e) of those rows
#pragma unroll
  for (int nt = 0; nt < NTQ; ++nt) {
    const T* qrow = reinterpret_cast<const T*>(w.qs + (nt * 8 + r) * kQRowBytes);
    float amax = 0.f;
    for (int d = c; d < D; d += 4) amax = fmaxf(amax, fabsf(float(qrow[d])));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    int kexp = 0;
    if (amax >= 32768.f && amax < INFINITY) kexp = int(__float_as_uint(amax) >> 23) - 127 - 14;
    const float qmul = __uint_as_float(uint32_t(127 - kexp) << 23);  // 2^-k
    float sr = 0.f;  // the quad of row r adds up that row, then rows 2c, 2c+1 are fetched
    for (int d = c; d < D; d += 4) sr += __half2float(__float2half_rn(float(qrow[d]) * qmul));
    sr += __shfl_xor_sync(0xffffffffu, sr, 1);
    sr += __shfl_xor_sync(0xffffffffu, sr, 2);
    const float fac = __uint_as_float(uint32_t(127 + kexp) << 23) * a.scale_log2;
    qsum[nt][0] = __shfl_sync(0xffffffffu, sr, 8 * c);
    qsum[nt][1] = __shfl_sync(0xffffffffu, sr, 8 * c + 4);
    qfac[nt][0] = __shfl_sync(0xffffffffu, fac, 8 * c);
    qfac[nt][1] = __shfl_sync(0xffffffffu, fac, 8 * c + 4);
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      const T* q0 = qrow + (4 * (ks >> 1) + c) * 8;
      const int e0 = (ks & 1) * 2;
      auto pk = [qmul](const T* p, int i0, int i1) {
        const __half2 h = __floats2half2_rn(float(p[i0]) * qmul, float(p[i1]) * qmul);
        return *reinterpret_cast<const uint32_t*>(&h);
      };
      qf[nt][ks][0] = pk(q0, e0, e0 + 4);
      qf[nt][ks][1] = pk(q0, e0 + 1, e0 + 5);
    }
  }
  // Q now lives in registers: release the staging area to the producer
  __syncwarp();
  if (lane == 0) mbar_arrive(w.q_done_bar);

  // per-query-row visibility limit: token t visible iff t < lim
  // per-query-row visibility limit: token t visible iff t < lim (a window with several queries per sequence, which
  // also has lower limits, is served by the 16-bit consumer only)
  int lim[NTQ][2];
  int lim_min = w.chunk_hi;  // below it nothing is masked for any row of this warp
#pragma unroll
  for (int nt = 0; nt < NTQ; ++nt)
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int row = w.row0 + nt * 8 + 2 * c + e;
      int l = w.chunk_hi;
      if (a.causal && row < R) l = min(l, w.kv_len - a.mq + row / a.q_per_kv + 1);
      lim[nt][e] = l;
      lim_min = min(lim_min, l);
    }
  lim_min = min(lim_min, __shfl_xor_sync(0xffffffffu, lim_min, 1));
  lim_min = min(lim_min, __shfl_xor_sync(0xffffffffu, lim_min, 2));

  float acc[MTV][NTQ][4];
  float m_run[NTQ][2], l_run[NTQ][2], corr[NTQ][2];
#pragma unroll
  for (int nt = 0; nt < NTQ; ++nt) {
#pragma unroll
    for (int mt = 0; mt < MTV; ++mt) acc[mt][nt][0] = acc[mt][nt][1] = acc[mt][nt][2] = acc[mt][nt][3] = 0.f;
    m_run[nt][0] = m_run[nt][1] = -INFINITY;
    l_run[nt][0] = l_run[nt][1] = 0.f;
    corr[nt][0] = corr[nt][1] = 0.f;
  }

  const int rw = row_bytes / 4;  // words per token row of the stage
  for (int tile = 0; tile < w.n_tiles; ++tile) {
    const int st = tile % w.stages;
    if (!mbar_wait(&w.full_bar[st], (tile / w.stages) & 1)) {
      if (lane == 0) atomicCAS(a.status, 0, 2);
      break;
    }
    const uint32_t* kst = reinterpret_cast<const uint32_t*>(w.stage_base + st * w.stage_bytes) + hw * W;
    const uint32_t* vst = kst + w.kv_bytes / 4;
#pragma unroll 1
    for (int sp = 0; sp < kSps; ++sp) {
      const int usub = w.sub + w.wph * sp;                                // this warp's sub-tile of the stage
      const int t_sub = w.chunk_lo + tile * w.tok_per_stage + usub * 16;  // its first token
      if (t_sub >= w.chunk_hi) continue;
      const uint32_t* k0 = kst + (usub * 16 + r) * rw;  // token r; token r + 8 is 8 rows on
      const uint32_t* v0 = vst + (usub * 16 + r) * rw;

      // ------------------------------------------- S^T = K Q^T (16 tokens x 8*NTQ)
      float s[NTQ][4], s2[NTQ][4];  // two chains of dependent MMAs instead of one
#pragma unroll
      for (int nt = 0; nt < NTQ; ++nt) {
        s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
        s2[nt][0] = s2[nt][1] = s2[nt][2] = s2[nt][3] = 0.f;
      }
#pragma unroll
      for (int i = 0; i < KS / 2; ++i) {
        uint32_t u0[4], u1[4];
        unpack4(k0[1 + 4 * i + c], u0);
        unpack4(k0[8 * rw + 1 + 4 * i + c], u1);
        const uint32_t ka[4] = {u0[0], u1[0], u0[1], u1[1]};
        const uint32_t kb[4] = {u0[2], u1[2], u0[3], u1[3]};
#pragma unroll
        for (int nt = 0; nt < NTQ; ++nt) {
          mma_16816<false>(s[nt], ka, qf[nt][2 * i][0], qf[nt][2 * i][1]);
          mma_16816<false>(s2[nt], kb, qf[nt][2 * i + 1][0], qf[nt][2 * i + 1][1]);
        }
      }

      // ------------------ scale/shift of tokens r, r+8; mask; online softmax
      const uint32_t kw0 = k0[0], kw1 = k0[8 * rw], vw0 = v0[0], vw1 = v0[8 * rw];
      const float ksc0 = half_bits_to_float(kw0 & 0xFFFFu), ksh0 = half_bits_to_float(kw0 >> 16);
      const float ksc1 = half_bits_to_float(kw1 & 0xFFFFu), ksh1 = half_bits_to_float(kw1 >> 16);
      float vsc0 = half_bits_to_float(vw0 & 0xFFFFu), vsh0 = half_bits_to_float(vw0 >> 16);
      float vsc1 = half_bits_to_float(vw1 & 0xFFFFu), vsh1 = half_bits_to_float(vw1 >> 16);
      const bool all_visible = t_sub + 16 <= lim_min;  // warp-uniform
      float sc0[NTQ][2], sc1[NTQ][2];                  // scores of tokens r / r+8, log2 domain
      bool need = false;
#pragma unroll
      for (int nt = 0; nt < NTQ; ++nt)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          sc0[nt][e] = fmaf(ksc0, s[nt][e] + s2[nt][e], ksh0 * qsum[nt][e]) * qfac[nt][e];
          sc1[nt][e] = fmaf(ksc1, s[nt][2 + e] + s2[nt][2 + e], ksh1 * qsum[nt][e]) * qfac[nt][e];
        }
      if (!all_visible) {
        const int t0 = t_sub + r, t1 = t_sub + r + 8;
        // tokens past the end were not copied: their scale words are garbage
        if (t0 >= w.chunk_hi) vsc0 = 0.f, vsh0 = 0.f;
        if (t1 >= w.chunk_hi) vsc1 = 0.f, vsh1 = 0.f;
#pragma unroll
        for (int nt = 0; nt < NTQ; ++nt)
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            if (t0 >= lim[nt][e]) sc0[nt][e] = -INFINITY;
            if (t1 >= lim[nt][e]) sc1[nt][e] = -INFINITY;
          }
      }
#pragma unroll
      for (int nt = 0; nt < NTQ; ++nt)
#pragma unroll
        for (int e = 0; e < 2; ++e) need |= fmaxf(sc0[nt][e], sc1[nt][e]) > m_run[nt][e] + kLazy;
      if (__any_sync(0xffffffffu, need)) {
        // some row's maximum grew by more than the slack: refresh all of them
#pragma unroll
        for (int nt = 0; nt < NTQ; ++nt) {
          float alpha[2];
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            float mx = fmaxf(sc0[nt][e], sc1[nt][e]);
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
            const float m_new = fmaxf(m_run[nt][e], mx);
            alpha[e] = fast_exp2(m_run[nt][e] - (m_new == -INFINITY ? 0.f : m_new));  // exp2(-inf) = 0 at first
            m_run[nt][e] = m_new;
            l_run[nt][e] *= alpha[e];
            corr[nt][e] *= alpha[e];
          }
#pragma unroll
          for (int mt = 0; mt < MTV; ++mt) {
            acc[mt][nt][0] *= alpha[0];
            acc[mt][nt][1] *= alpha[1];
            acc[mt][nt][2] *= alpha[0];
            acc[mt][nt][3] *= alpha[1];
          }
        }
      }
      uint32_t pb[NTQ][2];
#pragma unroll
      for (int nt = 0; nt < NTQ; ++nt) {
        float p0[2], p1[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const float m_use = m_run[nt][e] == -INFINITY ? 0.f : m_run[nt][e];
          p0[e] = fast_exp2(sc0[nt][e] - m_use);
          p1[e] = fast_exp2(sc1[nt][e] - m_use);
          l_run[nt][e] += p0[e] + p1[e];
          corr[nt][e] = fmaf(p0[e], vsh0, fmaf(p1[e], vsh1, corr[nt][e]));
        }
        // V's scale rides on the probabilities
        pb[nt][0] = movmatrix_trans(pack2<false>(p0[0] * vsc0, p0[1] * vsc0));  // tokens 2c, 2c+1   of row r
        pb[nt][1] = movmatrix_trans(pack2<false>(p1[0] * vsc1, p1[1] * vsc1));  // tokens 2c+8, 2c+9 of row r
      }

      // ------------------------------------------------- O^T += V^T P^T
      const uint32_t* va = vst + (usub * 16 + 2 * c) * rw + 1 + WPT * r;
#pragma unroll
      for (int wi = 0; wi < WPT; ++wi) {
        const uint32_t x0 = va[wi], x1 = va[rw + wi], x2 = va[8 * rw + wi], x3 = va[9 * rw + wi];
        // low / high half-words of two neighbouring tokens side by side
        uint32_t ylo[4], yhi[4], zlo[4], zhi[4];
        unpack4(__byte_perm(x0, x1, 0x5410), ylo);  // nibbles e   of tokens 2c,   2c+1 -> rows r
        unpack4(__byte_perm(x0, x1, 0x7632), yhi);  // nibbles e+4 of tokens 2c,   2c+1 -> rows r+8
        unpack4(__byte_perm(x2, x3, 0x5410), zlo);  // nibbles e   of tokens 2c+8, 2c+9
        unpack4(__byte_perm(x2, x3, 0x7632), zhi);
        // unpack4 pairs nibble e of the low half with nibble e of the high half
        // (its "e + 4"), i.e. the same element of the two tokens: out[0..3] are
        // elements 0, 1, 2, 3 of the half-word
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const uint32_t vf[4] = {ylo[e], yhi[e], zlo[e], zhi[e]};
#pragma unroll
          for (int nt = 0; nt < NTQ; ++nt) mma_16816<false>(acc[wi * 4 + e][nt], vf, pb[nt][0], pb[nt][1]);
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&w.empty_bar[st]);
  }

  // full row sums (each thread saw tokens r and r+8 of every sub-tile)
#pragma unroll
  for (int nt = 0; nt < NTQ; ++nt)
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      float l = l_run[nt][e], cs = corr[nt][e];
#pragma unroll
      for (int o = 4; o < 32; o <<= 1) {
        l += __shfl_xor_sync(0xffffffffu, l, o);
        cs += __shfl_xor_sync(0xffffffffu, cs, o);
      }
      l_run[nt][e] = l;
      corr[nt][e] = cs;
    }

  // the ring is no longer in use once every consumer warp got here
  asm volatile("bar.sync 1, %0;" ::"n"(kDecConsumerWarps * 32) : "memory");
#pragma unroll
  for (int nt = 0; nt < NTQ; ++nt) {
#pragma unroll
    for (int mt = 0; mt < MTV; ++mt)
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int d = 8 * (WPT * r + (mt >> 2)) + (mt & 3) + (q >> 1) * 4;
        const int rr = nt * 8 + 2 * c + (q & 1);
        w.mine[rr * kCmbRow + d] = acc[mt][nt][q] + corr[nt][q & 1];
      }
    if (r == 0) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        w.mine[(nt * 8 + 2 * c + e) * kCmbRow + D] = m_run[nt][e];
        w.mine[(nt * 8 + 2 * c + e) * kCmbRow + D + 1] = l_run[nt][e];
      }
    }
  }
}

// ---------------------------------------------------------------------------
// int4 row-wise cache with NG > 1 quantisation groups per row (the first NG
// words of a row are the (scale | shift << 16) words of its groups of D / NG
// elements).  Same products as consume_int4, but a scale now belongs to a
// (token, group) pair.  K: the products of every group are accumulated on their
// own and scaled in fp32 afterwards (the scores, hence the log-sum-exp, see no
// rounding of K).  V: an output tile may mix groups along the token axis, so the
// scales are folded into the unpacked elements themselves (one more half2
// multiply per nibble pair, on the FMA pipe).  The shifts become per-group
// terms: shift_g x (sum of q over group g) for K, sum_t p_t x shift_{t,g} added
// to the columns of group g for V.
// ---------------------------------------------------------------------------
template <int D, int NTQ, bool kBf16, int NG>
__device__ __forceinline__ void consume_int4_groups(const DecodeArgs& a, const DecWarp& w) {
  using T = typename Half2Type<kBf16>::T;
  constexpr int W = NG + D / 8;      // words per row
  constexpr int KS = D / 16;         // k-steps of K Q^T
  constexpr int MTV = D / 16;        // m-tiles of V^T P^T
  constexpr int WPT = D / 64;        // V words per thread and token
  constexpr int GW = (D / 8) / NG;   // nibble words per group
  static_assert(GW >= WPT && GW >= 1 && (D / 8) % NG == 0, "groups of at least 16 elements");
  constexpr int kQRowBytes = D * 2;
  constexpr int kCmbRow = D + 2;
  constexpr int kSps = DecStage<D, kFmtInt4, NG>::kSubTiles;
  constexpr float kLazy = 4.f;
  const int lane = w.lane, r = lane >> 2, c = lane & 3;
  const int R = a.rows, hw = w.hw, row_bytes = w.row_bytes;

  // nibble pairs (e, e+4), e = 0..3, of a packed word as f16 pairs n * mul (mul: one factor per half)
  auto unpack4s = [](uint32_t x, __half2 mul, uint32_t (&out)[4]) {
    constexpr uint32_t kMagic = 0x64006400u;
    const __half2 k1024 = __half2half2(__ushort_as_half(0x6400));
    const __half2 k64 = __half2half2(__ushort_as_half(0x5400));
    const __half2 k16th = __half2half2(__ushort_as_half(0x2C00));
    const uint32_t hi = x >> 8;
    uint32_t v0 = (x & 0x000F000Fu) | kMagic, v1 = (x & 0x00F000F0u) | kMagic;
    uint32_t v2 = (hi & 0x000F000Fu) | kMagic, v3 = (hi & 0x00F000F0u) | kMagic;
    __half2 h0 = __hmul2(__hsub2(*reinterpret_cast<__half2*>(&v0), k1024), mul);
    __half2 h1 = __hmul2(__hfma2(*reinterpret_cast<__half2*>(&v1), k16th, __hneg2(k64)), mul);
    __half2 h2 = __hmul2(__hsub2(*reinterpret_cast<__half2*>(&v2), k1024), mul);
    __half2 h3 = __hmul2(__hfma2(*reinterpret_cast<__half2*>(&v3), k16th, __hneg2(k64)), mul);
    out[0] = *reinterpret_cast<uint32_t*>(&h0);
    out[1] = *reinterpret_cast<uint32_t*>(&h1);
    out[2] = *reinterpret_cast<uint32_t*>(&h2);
    out[3] = *reinterpret_cast<uint32_t*>(&h3);
  };
  auto scale_of = [](uint32_t word) { return __ushort_as_half(static_cast<unsigned short>(word & 0xFFFFu)); };

  uint32_t qf[NTQ][KS][2];
  float qsum[NTQ][NG][2];  // per group: sum of the scaled q, rows 2c, 2c+1 of each n-tile
  float qfac[NTQ][2];
#pragma unroll
  for (int nt = 0; nt < NTQ; ++nt) {
    const T* qrow = reinterpret_cast<const T*>(w.qs + (nt * 8 + r) * kQRowBytes);
    float amax = 0.f;
    for (int d = c; d < D; d += 4) amax = fmaxf(amax, fabsf(float(qrow[d])));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    int kexp = 0;
    if (amax >= 32768.f && amax < INFINITY) kexp = int(__float_as_uint(amax) >> 23) - 127 - 14;
    const float qmul = __uint_as_float(uint32_t(127 - kexp) << 23);
    const float fac = __uint_as_float(uint32_t(127 + kexp) << 23) * a.scale_log2;
    qfac[nt][0] = __shfl_sync(0xffffffffu, fac, 8 * c);
    qfac[nt][1] = __shfl_sync(0xffffffffu, fac, 8 * c + 4);
#pragma unroll
    for (int g = 0; g < NG; ++g) {
      float sr = 0.f;
      for (int d = g * (D / NG) + c; d < (g + 1) * (D / NG); d += 4) sr += __half2float(__float2half_rn(float(qrow[d]) * qmul));
      sr += __shfl_xor_sync(0xffffffffu, sr, 1);
      sr += __shfl_xor_sync(0xffffffffu, sr, 2);
      qsum[nt][g][0] = __shfl_sync(0xffffffffu, sr, 8 * c);
      qsum[nt][g][1] = __shfl_sync(0xffffffffu, sr, 8 * c + 4);
    }
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      const T* q0 = qrow + (4 * (ks >> 1) + c) * 8;
      const int e0 = (ks & 1) * 2;
      auto pk = [qmul](const T* p, int i0, int i1) {
        const __half2 h = __floats2half2_rn(float(p[i0]) * qmul, float(p[i1]) * qmul);
        return *reinterpret_cast<const uint32_t*>(&h);
      };
      qf[nt][ks][0] = pk(q0, e0, e0 + 4);
      qf[nt][ks][1] = pk(q0, e0 + 1, e0 + 5);
    }
  }
  __syncwarp();
  if (lane == 0) mbar_arrive(w.q_done_bar);

  // per-query-row visibility limit: token t visible iff t < lim (a window with several queries per sequence, which
  // also has lower limits, is served by the 16-bit consumer only)
  int lim[NTQ][2];
  int lim_min = w.chunk_hi;  // below it nothing is masked for any row of this warp
#pragma unroll
  for (int nt = 0; nt < NTQ; ++nt)
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int row = w.row0 + nt * 8 + 2 * c + e;
      int l = w.chunk_hi;
      if (a.causal && row < R) l = min(l, w.kv_len - a.mq + row / a.q_per_kv + 1);
      lim[nt][e] = l;
      lim_min = min(lim_min, l);
    }
  lim_min = min(lim_min, __shfl_xor_sync(0xffffffffu, lim_min, 1));
  lim_min = min(lim_min, __shfl_xor_sync(0xffffffffu, lim_min, 2));

  float acc[MTV][NTQ][4];
  float m_run[NTQ][2], l_run[NTQ][2], corr[NTQ][NG][2];
#pragma unroll
  for (int nt = 0; nt < NTQ; ++nt) {
#pragma unroll
    for (int mt = 0; mt < MTV; ++mt) acc[mt][nt][0] = acc[mt][nt][1] = acc[mt][nt][2] = acc[mt][nt][3] = 0.f;
    m_run[nt][0] = m_run[nt][1] = -INFINITY;
    l_run[nt][0] = l_run[nt][1] = 0.f;
#pragma unroll
    for (int g = 0; g < NG; ++g) corr[nt][g][0] = corr[nt][g][1] = 0.f;
  }
  const int gv = (WPT * r) / GW;  // group of the V words this thread unpacks (both words of a token share it)

  const int rw = row_bytes / 4;
  for (int tile = 0; tile < w.n_tiles; ++tile) {
    const int st = tile % w.stages;
    if (!mbar_wait(&w.full_bar[st], (tile / w.stages) & 1)) {
      if (lane == 0) atomicCAS(a.status, 0, 2);
      break;
    }
    const uint32_t* kst = reinterpret_cast<const uint32_t*>(w.stage_base + st * w.stage_bytes) + hw * W;
    const uint32_t* vst = kst + w.kv_bytes / 4;
#pragma unroll 1
    for (int sp = 0; sp < kSps; ++sp) {
      const int usub = w.sub + w.wph * sp;
      const int t_sub = w.chunk_lo + tile * w.tok_per_stage + usub * 16;
      if (t_sub >= w.chunk_hi) continue;
      const uint32_t* k0 = kst + (usub * 16 + r) * rw;  // token r; token r + 8 is 8 rows on
      const uint32_t* v0 = vst + (usub * 16 + r) * rw;
      const bool all_visible = t_sub + 16 <= lim_min;
      const int t0 = t_sub + r, t1 = t_sub + r + 8;
      const bool in0 = t0 < w.chunk_hi, in1 = t1 < w.chunk_hi;  // tokens past the end were not copied

      // ------------------------------------------- S^T = K Q^T, one fp32 partial sum per group
      // A scale belongs to a (token, group) pair.  The nibbles go into the MMAs as they are (exact in f16), the
      // products of every group are accumulated on their own and take their scale in fp32 afterwards, so that
      // nothing of K is rounded before the scores exist.  The words of iteration i (4i .. 4i+3, one per thread
      // of a quad) lie in one group when a group has at least four words; with two-word groups words c < 2 and
      // c >= 2 belong to different groups and each takes its own pair of MMAs, the other threads feeding zeros.
      float sc0[NTQ][2], sc1[NTQ][2];
#pragma unroll
      for (int nt = 0; nt < NTQ; ++nt) sc0[nt][0] = sc0[nt][1] = sc1[nt][0] = sc1[nt][1] = 0.f;
      auto unpack4 = [](uint32_t x, uint32_t (&out)[4]) {
        constexpr uint32_t kMagic = 0x64006400u;
        const __half2 k1024 = __half2half2(__ushort_as_half(0x6400));
        const __half2 k64 = __half2half2(__ushort_as_half(0x5400));
        const __half2 k16th = __half2half2(__ushort_as_half(0x2C00));
        const uint32_t hi = x >> 8;
        uint32_t v0 = (x & 0x000F000Fu) | kMagic, v1 = (x & 0x00F000F0u) | kMagic;
        uint32_t v2 = (hi & 0x000F000Fu) | kMagic, v3 = (hi & 0x00F000F0u) | kMagic;
        __half2 h0 = __hsub2(*reinterpret_cast<__half2*>(&v0), k1024);
        __half2 h1 = __hfma2(*reinterpret_cast<__half2*>(&v1), k16th, __hneg2(k64));
        __half2 h2 = __hsub2(*reinterpret_cast<__half2*>(&v2), k1024);
        __half2 h3 = __hfma2(*reinterpret_cast<__half2*>(&v3), k16th, __hneg2(k64));
        out[0] = *reinterpret_cast<uint32_t*>(&h0);
        out[1] = *reinterpret_cast<uint32_t*>(&h1);
        out[2] = *reinterpret_cast<uint32_t*>(&h2);
        out[3] = *reinterpret_cast<uint32_t*>(&h3);
      };
      auto add_group = [&](const float (&s)[NTQ][4], const float (&s2)[NTQ][4], int g) {
        const float ksc0 = half_bits_to_float(k0[g] & 0xFFFFu), ksc1 = half_bits_to_float(k0[8 * rw + g] & 0xFFFFu);
#pragma unroll
        for (int nt = 0; nt < NTQ; ++nt)
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            sc0[nt][e] = fmaf(ksc0, s[nt][e] + s2[nt][e], sc0[nt][e]);
            sc1[nt][e] = fmaf(ksc1, s[nt][2 + e] + s2[nt][2 + e], sc1[nt][e]);
          }
      };
      if constexpr (GW % 4 == 0) {
        constexpr int IPG = GW / 4;  // iterations (four words each) per group
#pragma unroll
        for (int g = 0; g < NG; ++g) {
          float s[NTQ][4], s2[NTQ][4];
#pragma unroll
          for (int nt = 0; nt < NTQ; ++nt) {
            s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
            s2[nt][0] = s2[nt][1] = s2[nt][2] = s2[nt][3] = 0.f;
          }
#pragma unroll
          for (int ii = 0; ii < IPG; ++ii) {
            const int i = g * IPG + ii;
            uint32_t u0[4], u1[4];
            unpack4(k0[NG + 4 * i + c], u0);
            unpack4(k0[8 * rw + NG + 4 * i + c], u1);
            const uint32_t ka[4] = {u0[0], u1[0], u0[1], u1[1]};
            const uint32_t kb[4] = {u0[2], u1[2], u0[3], u1[3]};
#pragma unroll
            for (int nt = 0; nt < NTQ; ++nt) {
              mma_16816<false>(s[nt], ka, qf[nt][2 * i][0], qf[nt][2 * i][1]);
              mma_16816<false>(s2[nt], kb, qf[nt][2 * i + 1][0], qf[nt][2 * i + 1][1]);
            }
          }
          add_group(s, s2, g);
        }
      } else {
        static_assert(GW == 2, "groups of two words (16 elements) or of a multiple of four words");
#pragma unroll
        for (int i = 0; i < KS / 2; ++i) {
          uint32_t u0[4], u1[4];
          unpack4(k0[NG + 4 * i + c], u0);
          unpack4(k0[8 * rw + NG + 4 * i + c], u1);
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            const bool mine = (c >> 1) == half;  // this thread's word belongs to group 2i + half
            const uint32_t ka[4] = {mine ? u0[0] : 0u, mine ? u1[0] : 0u, mine ? u0[1] : 0u, mine ? u1[1] : 0u};
            const uint32_t kb[4] = {mine ? u0[2] : 0u, mine ? u1[2] : 0u, mine ? u0[3] : 0u, mine ? u1[3] : 0u};
            float s[NTQ][4], s2[NTQ][4];
#pragma unroll
            for (int nt = 0; nt < NTQ; ++nt) {
              s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
              s2[nt][0] = s2[nt][1] = s2[nt][2] = s2[nt][3] = 0.f;
              mma_16816<false>(s[nt], ka, qf[nt][2 * i][0], qf[nt][2 * i][1]);
              mma_16816<false>(s2[nt], kb, qf[nt][2 * i + 1][0], qf[nt][2 * i + 1][1]);
            }
            add_group(s, s2, 2 * i + half);
          }
        }
      }
      // shifts of K: one term per group
#pragma unroll
      for (int g = 0; g < NG; ++g) {
        const float ksh0 = half_bits_to_float(k0[g] >> 16), ksh1 = half_bits_to_float(k0[8 * rw + g] >> 16);
#pragma unroll
        for (int nt = 0; nt < NTQ; ++nt)
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            sc0[nt][e] = fmaf(ksh0, qsum[nt][g][e], sc0[nt][e]);
            sc1[nt][e] = fmaf(ksh1, qsum[nt][g][e], sc1[nt][e]);
          }
      }
      bool need = false;
#pragma unroll
      for (int nt = 0; nt < NTQ; ++nt)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          sc0[nt][e] *= qfac[nt][e];
          sc1[nt][e] *= qfac[nt][e];
          if (!all_visible) {
            if (t0 >= lim[nt][e]) sc0[nt][e] = -INFINITY;
            if (t1 >= lim[nt][e]) sc1[nt][e] = -INFINITY;
          }
          need |= fmaxf(sc0[nt][e], sc1[nt][e]) > m_run[nt][e] + kLazy;
        }
      if (__any_sync(0xffffffffu, need)) {
#pragma unroll
        for (int nt = 0; nt < NTQ; ++nt) {
          float alpha[2];
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            float mx = fmaxf(sc0[nt][e], sc1[nt][e]);
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
            const float m_new = fmaxf(m_run[nt][e], mx);
            alpha[e] = fast_exp2(m_run[nt][e] - (m_new == -INFINITY ? 0.f : m_new));
            m_run[nt][e] = m_new;
            l_run[nt][e] *= alpha[e];
#pragma unroll
            for (int g = 0; g < NG; ++g) corr[nt][g][e] *= alpha[e];
          }
#pragma unroll
          for (int mt = 0; mt < MTV; ++mt) {
            acc[mt][nt][0] *= alpha[0];
            acc[mt][nt][1] *= alpha[1];
            acc[mt][nt][2] *= alpha[0];
            acc[mt][nt][3] *= alpha[1];
          }
        }
      }
      uint32_t pb[NTQ][2];
      float p0[NTQ][2], p1[NTQ][2];
#pragma unroll
      for (int nt = 0; nt < NTQ; ++nt) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const float m_use = m_run[nt][e] == -INFINITY ? 0.f : m_run[nt][e];
          p0[nt][e] = fast_exp2(sc0[nt][e] - m_use);
          p1[nt][e] = fast_exp2(sc1[nt][e] - m_use);
          l_run[nt][e] += p0[nt][e] + p1[nt][e];
        }
        pb[nt][0] = movmatrix_trans(pack2<false>(p0[nt][0], p0[nt][1]));  // tokens 2c, 2c+1   of row r
        pb[nt][1] = movmatrix_trans(pack2<false>(p1[nt][0], p1[nt][1]));  // tokens 2c+8, 2c+9 of row r
      }
      // shifts of V: sum_t p_t shift_{t,g}, one accumulator per group
#pragma unroll
      for (int g = 0; g < NG; ++g) {
        const float vsh0 = in0 ? half_bits_to_float(v0[g] >> 16) : 0.f;
        const float vsh1 = in1 ? half_bits_to_float(v0[8 * rw + g] >> 16) : 0.f;
#pragma unroll
        for (int nt = 0; nt < NTQ; ++nt)
#pragma unroll
          for (int e = 0; e < 2; ++e) corr[nt][g][e] = fmaf(p0[nt][e], vsh0, fmaf(p1[nt][e], vsh1, corr[nt][g][e]));
      }

      // ------------------------------------------------- O^T += V^T P^T with V already scaled
      {
        const uint32_t* va = vst + (usub * 16 + 2 * c) * rw;  // token 2c; +rw: 2c+1; +8rw: 2c+8; +9rw: 2c+9
        const int tv = t_sub + 2 * c;
        // scales of the four tokens for this thread's group (0 past the end: garbage words there)
        const __half hz = __ushort_as_half(0);
        const __half2 ma = __halves2half2(tv < w.chunk_hi ? scale_of(va[gv]) : hz, tv + 1 < w.chunk_hi ? scale_of(va[rw + gv]) : hz);
        const __half2 mb = __halves2half2(tv + 8 < w.chunk_hi ? scale_of(va[8 * rw + gv]) : hz, tv + 9 < w.chunk_hi ? scale_of(va[9 * rw + gv]) : hz);
#pragma unroll
        for (int wi = 0; wi < WPT; ++wi) {
          const int wd = NG + WPT * r + wi;
          const uint32_t x0 = va[wd], x1 = va[rw + wd], x2 = va[8 * rw + wd], x3 = va[9 * rw + wd];
          uint32_t ylo[4], yhi[4], zlo[4], zhi[4];
          unpack4s(__byte_perm(x0, x1, 0x5410), ma, ylo);
          unpack4s(__byte_perm(x0, x1, 0x7632), ma, yhi);
          unpack4s(__byte_perm(x2, x3, 0x5410), mb, zlo);
          unpack4s(__byte_perm(x2, x3, 0x7632), mb, zhi);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const uint32_t vf[4] = {ylo[e], yhi[e], zlo[e], zhi[e]};
#pragma unroll
            for (int nt = 0; nt < NTQ; ++nt) mma_16816<false>(acc[wi * 4 + e][nt], vf, pb[nt][0], pb[nt][1]);
          }
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&w.empty_bar[st]);
  }

#pragma unroll
  for (int nt = 0; nt < NTQ; ++nt)
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      float l = l_run[nt][e];
#pragma unroll
      for (int o = 4; o < 32; o <<= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
      l_run[nt][e] = l;
#pragma unroll
      for (int g = 0; g < NG; ++g) {
        float cs = corr[nt][g][e];
#pragma unroll
        for (int o = 4; o < 32; o <<= 1) cs += __shfl_xor_sync(0xffffffffu, cs, o);
        corr[nt][g][e] = cs;
      }
    }

  asm volatile("bar.sync 1, %0;" ::"n"(kDecConsumerWarps * 32) : "memory");
#pragma unroll
  for (int nt = 0; nt < NTQ; ++nt) {
    // the columns this thread holds all belong to group gv
    float cv[2] = {0.f, 0.f};
#pragma unroll
    for (int g = 0; g < NG; ++g)
      if (g == gv) cv[0] = corr[nt][g][0], cv[1] = corr[nt][g][1];
#pragma unroll
    for (int mt = 0; mt < MTV; ++mt)
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int d = 8 * (WPT * r + (mt >> 2)) + (mt & 3) + (q >> 1) * 4;
        const int rr = nt * 8 + 2 * c + (q & 1);
        w.mine[rr * kCmbRow + d] = acc[mt][nt][q] + cv[q & 1];
      }
    if (r == 0) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        w.mine[(nt * 8 + 2 * c + e) * kCmbRow + D] = m_run[nt][e];
        w.mine[(nt * 8 + 2 * c + e) * kCmbRow + D + 1] = l_run[nt][e];
      }
    }
  }
}

// ---------------------------------------------------------------------------
// fp8 row-wise cache (four e4m3 values per int32 word, one fp16 scale / shift
// pair per token and kv head in a tensor of its own; tests/utils.py:311-340 of
// the reference).  Same structure as the int4 consumer: transposed products in
// f16, tokens = M rows of S^T = K Q^T and K dimension of O^T = V^T P^T, K's
// scale/shift applied to the scores, V's scale folded into P, its shift a
// per-row term.  A stage is [head][token][128 B] as the tiled copy left it
// (16-byte chunks XOR-ed with token & 7).
//   K: thread (r, c) reads word c of chunk ks of tokens r and r + 8: elements
//      d = 16 ks + 4 c + {0, 1 | 2, 3} are the k-slots (2c, 2c+1 | 2c+8, 2c+9)
//      of k-step ks; one cvt.f16x2.e4m3x2 per pair.
//   V: thread (r, c) reads word r + 8 wj of tokens 2c, 2c+1, 2c+8, 2c+9; a byte
//      permute puts the same element of two neighbouring tokens side by side,
//      so that the conversion yields A-fragment registers: m-tile 2 wj + p
//      holds d = 4 (r + 8 wj) + p in row r and d + 2 in row r + 8.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void cvt_e4m3x4(uint32_t w, uint32_t& lo, uint32_t& hi) {
  asm("{\n\t.reg .b16 l, h;\n\tmov.b32 {l, h}, %2;\n\tcvt.rn.f16x2.e4m3x2 %0, l;\n\tcvt.rn.f16x2.e4m3x2 %1, h;\n\t}" : "=r"(lo), "=r"(hi) : "r"(w));
}

template <int D, int NTQ, bool kBf16>
__device__ __forceinline__ void consume_fp8(const DecodeArgs& a, const DecWarp& w) {
  static_assert(D == 128, "fp8 rows are one 128-byte swizzle row");
  using T = typename Half2Type<kBf16>::T;
  constexpr int KS = D / 16;   // k-steps of K Q^T
  constexpr int MTV = D / 16;  // m-tiles of V^T P^T
  constexpr int WJ = D / 32;   // V words per thread and token
  constexpr int kQRowBytes = D * 2;
  constexpr int kCmbRow = D + 2;
  constexpr int kSps = DecStage<D, kFmtFp8>::kSubTiles;
  constexpr float kLazy = 4.f;  // as in the int4 consumer
  const int lane = w.lane, r = lane >> 2, c = lane & 3;
  const int R = a.rows, hw = w.hw, hb = a.hb;
  const int box_shift = __ffs(a.box_tok) - 1;
  const int head_bytes = a.box_tok * 128;      // one head of a box
  const int box_bytes = head_bytes * hb;

  // B fragments of Q^T (n = query row nt*8 + r): f16 of q * 2^-k, k per row so that nothing overflows
  uint32_t qf[NTQ][KS][2];
  float qsum[NTQ][2];  // sum over d of the scaled q, rows 2c, 2c+1 of each n-tile
  float qfac[NTQ][2];  // 2^k * softmax scale * log2(e) of those rows
#pragma unroll
  for (int nt = 0; nt < NTQ; ++nt) {
    const T* qrow = reinterpret_cast<const T*>(w.qs + (nt * 8 + r) * kQRowBytes);
    float amax = 0.f;
    for (int d = c; d < D; d += 4) amax = fmaxf(amax, fabsf(float(qrow[d])));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    int kexp = 0;
    if (amax >= 32768.f && amax < INFINITY) kexp = int(__float_as_uint(amax) >> 23) - 127 - 14;
    const float qmul = __uint_as_float(uint32_t(127 - kexp) << 23);  // 2^-k
    float sr = 0.f;
    for (int d = c; d < D; d += 4) sr += __half2float(__float2half_rn(float(qrow[d]) * qmul));
    sr += __shfl_xor_sync(0xffffffffu, sr, 1);
    sr += __shfl_xor_sync(0xffffffffu, sr, 2);
    const float fac = __uint_as_float(uint32_t(127 + kexp) << 23) * a.scale_log2;
    qsum[nt][0] = __shfl_sync(0xffffffffu, sr, 8 * c);
    qsum[nt][1] = __shfl_sync(0xffffffffu, sr, 8 * c + 4);
    qfac[nt][0] = __shfl_sync(0xffffffffu, fac, 8 * c);
    qfac[nt][1] = __shfl_sync(0xffffffffu, fac, 8 * c + 4);
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      const T* q0 = qrow + 16 * ks + 4 * c;
      const __half2 h01 = __floats2half2_rn(float(q0[0]) * qmul, float(q0[1]) * qmul);
      const __half2 h23 = __floats2half2_rn(float(q0[2]) * qmul, float(q0[3]) * qmul);
      qf[nt][ks][0] = *reinterpret_cast<const uint32_t*>(&h01);
      qf[nt][ks][1] = *reinterpret_cast<const uint32_t*>(&h23);
    }
  }
  // Q now lives in registers: release the staging area to the producer
  __syncwarp();
  if (lane == 0) mbar_arrive(w.q_done_bar);

  // per-query-row visibility limit: token t visible iff t < lim (a window with several queries per sequence, which
  // also has lower limits, is served by the 16-bit consumer only)
  int lim[NTQ][2];
  int lim_min = w.chunk_hi;  // below it nothing is masked for any row of this warp
#pragma unroll
  for (int nt = 0; nt < NTQ; ++nt)
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int row = w.row0 + nt * 8 + 2 * c + e;
      int l = w.chunk_hi;
      if (a.causal && row < R) l = min(l, w.kv_len - a.mq + row / a.q_per_kv + 1);
      lim[nt][e] = l;
      lim_min = min(lim_min, l);
    }
  lim_min = min(lim_min, __shfl_xor_sync(0xffffffffu, lim_min, 1));
  lim_min = min(lim_min, __shfl_xor_sync(0xffffffffu, lim_min, 2));

  float acc[MTV][NTQ][4];
  float m_run[NTQ][2], l_run[NTQ][2], corr[NTQ][2];
#pragma unroll
  for (int nt = 0; nt < NTQ; ++nt) {
#pragma unroll
    for (int mt = 0; mt < MTV; ++mt) acc[mt][nt][0] = acc[mt][nt][1] = acc[mt][nt][2] = acc[mt][nt][3] = 0.f;
    m_run[nt][0] = m_run[nt][1] = -INFINITY;
    l_run[nt][0] = l_run[nt][1] = 0.f;
    corr[nt][0] = corr[nt][1] = 0.f;
  }

  for (int tile = 0; tile < w.n_tiles; ++tile) {
    const int st = tile % w.stages;
    if (!mbar_wait(&w.full_bar[st], (tile / w.stages) & 1)) {
      if (lane == 0) atomicCAS(a.status, 0, 2);
      break;
    }
    const uint8_t* kst = w.stage_base + st * w.stage_bytes;
    const uint8_t* vst = kst + w.kv_bytes;
    // scale/shift words: [head][token] after the 4-byte copies, [token][head][4 words] after the tiled ones
    // scale/shift words of a stage: [token][head][4 words] (tiled copies of replicated words), [token][head]
    // (tiled copies of compact words) or [head][token] (4-byte copies)
    const uint32_t* ssk = reinterpret_cast<const uint32_t*>(kst + 2 * w.kv_bytes) + (a.ss_tma == 1 ? hw * 4 : a.ss_tma == 2 ? hw : hw * w.tok_per_stage);
    const uint32_t* ssv = ssk + a.ss_bytes / 4;
    const int ss_step = a.ss_tma == 1 ? hb * 4 : a.ss_tma == 2 ? hb : 1;  // words from one token to the next
#pragma unroll 1
    for (int sp = 0; sp < kSps; ++sp) {
      const int usub = w.sub + w.wph * sp;                                // this warp's sub-tile of the stage
      const int t_sub = w.chunk_lo + tile * w.tok_per_stage + usub * 16;  // its first token
      if (t_sub >= w.chunk_hi) continue;
      const int tok0 = usub * 16;  // first token of the sub-tile inside the stage (a multiple of 16 inside its box)
      const int boff = (tok0 >> box_shift) * box_bytes + hw * head_bytes + (tok0 & (a.box_tok - 1)) * 128;

      // ------------------------------------------- S^T = K Q^T (16 tokens x 8*NTQ)
      float s[NTQ][4], s2[NTQ][4];  // two chains of dependent MMAs instead of one
#pragma unroll
      for (int nt = 0; nt < NTQ; ++nt) {
        s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
        s2[nt][0] = s2[nt][1] = s2[nt][2] = s2[nt][3] = 0.f;
      }
      {
        const uint8_t* k0 = kst + boff + r * 128 + c * 4;  // token r (chunk swizzle r & 7 = r); token r + 8 is 8 rows on, same swizzle
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
          const int co = (ks ^ r) * 16;
          const uint32_t w0 = *reinterpret_cast<const uint32_t*>(k0 + co);
          const uint32_t w1 = *reinterpret_cast<const uint32_t*>(k0 + 8 * 128 + co);
          uint32_t ka[4];
          cvt_e4m3x4(w0, ka[0], ka[2]);
          cvt_e4m3x4(w1, ka[1], ka[3]);
#pragma unroll
          for (int nt = 0; nt < NTQ; ++nt) mma_16816<false>((ks & 1) ? s2[nt] : s[nt], ka, qf[nt][ks][0], qf[nt][ks][1]);
        }
      }

      // ------------------ scale/shift of tokens r, r+8; mask; online softmax
      const uint32_t kw0 = ssk[(tok0 + r) * ss_step], kw1 = ssk[(tok0 + r + 8) * ss_step];
      const uint32_t vw0 = ssv[(tok0 + r) * ss_step], vw1 = ssv[(tok0 + r + 8) * ss_step];
      const float ksc0 = half_bits_to_float(kw0 & 0xFFFFu), ksh0 = half_bits_to_float(kw0 >> 16);
      const float ksc1 = half_bits_to_float(kw1 & 0xFFFFu), ksh1 = half_bits_to_float(kw1 >> 16);
      float vsc0 = half_bits_to_float(vw0 & 0xFFFFu), vsh0 = half_bits_to_float(vw0 >> 16);
      float vsc1 = half_bits_to_float(vw1 & 0xFFFFu), vsh1 = half_bits_to_float(vw1 >> 16);
      const bool all_visible = t_sub + 16 <= lim_min;  // warp-uniform
      float sc0[NTQ][2], sc1[NTQ][2];                  // scores of tokens r / r+8, log2 domain
      bool need = false;
#pragma unroll
      for (int nt = 0; nt < NTQ; ++nt)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          sc0[nt][e] = fmaf(ksc0, s[nt][e] + s2[nt][e], ksh0 * qsum[nt][e]) * qfac[nt][e];
          sc1[nt][e] = fmaf(ksc1, s[nt][2 + e] + s2[nt][2 + e], ksh1 * qsum[nt][e]) * qfac[nt][e];
        }
      if (!all_visible) {
        const int t0 = t_sub + r, t1 = t_sub + r + 8;
        // tokens past the end were not copied: their scale words are garbage
        if (t0 >= w.chunk_hi) vsc0 = 0.f, vsh0 = 0.f;
        if (t1 >= w.chunk_hi) vsc1 = 0.f, vsh1 = 0.f;
#pragma unroll
        for (int nt = 0; nt < NTQ; ++nt)
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            if (t0 >= lim[nt][e]) sc0[nt][e] = -INFINITY;
            if (t1 >= lim[nt][e]) sc1[nt][e] = -INFINITY;
          }
      }
#pragma unroll
      for (int nt = 0; nt < NTQ; ++nt)
#pragma unroll
        for (int e = 0; e < 2; ++e) need |= fmaxf(sc0[nt][e], sc1[nt][e]) > m_run[nt][e] + kLazy;
      if (__any_sync(0xffffffffu, need)) {
#pragma unroll
        for (int nt = 0; nt < NTQ; ++nt) {
          float alpha[2];
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            float mx = fmaxf(sc0[nt][e], sc1[nt][e]);
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
            const float m_new = fmaxf(m_run[nt][e], mx);
            alpha[e] = fast_exp2(m_run[nt][e] - (m_new == -INFINITY ? 0.f : m_new));
            m_run[nt][e] = m_new;
            l_run[nt][e] *= alpha[e];
            corr[nt][e] *= alpha[e];
          }
#pragma unroll
          for (int mt = 0; mt < MTV; ++mt) {
            acc[mt][nt][0] *= alpha[0];
            acc[mt][nt][1] *= alpha[1];
            acc[mt][nt][2] *= alpha[0];
            acc[mt][nt][3] *= alpha[1];
          }
        }
      }
      uint32_t pb[NTQ][2];
#pragma unroll
      for (int nt = 0; nt < NTQ; ++nt) {
        float p0[2], p1[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const float m_use = m_run[nt][e] == -INFINITY ? 0.f : m_run[nt][e];
          p0[e] = fast_exp2(sc0[nt][e] - m_use);
          p1[e] = fast_exp2(sc1[nt][e] - m_use);
          l_run[nt][e] += p0[e] + p1[e];
          corr[nt][e] = fmaf(p0[e], vsh0, fmaf(p1[e], vsh1, corr[nt][e]));
        }
        pb[nt][0] = movmatrix_trans(pack2<false>(p0[0] * vsc0, p0[1] * vsc0));  // tokens 2c, 2c+1   of row r
        pb[nt][1] = movmatrix_trans(pack2<false>(p1[0] * vsc1, p1[1] * vsc1));  // tokens 2c+8, 2c+9 of row r
      }

      // ------------------------------------------------- O^T += V^T P^T
      {
        const uint8_t* v0 = vst + boff + (2 * c) * 128 + (r & 3) * 4;  // token 2c; +128: 2c+1; +1024: 2c+8; +1152: 2c+9
        const int x0s = (2 * c) & 7, x1s = (2 * c + 1) & 7;            // chunk swizzles of the even / odd token
        // Bytes of tokens past the end were never copied and may hold the NaN patterns of
        // e4m3 (0 x NaN = NaN): they are cleared before the conversion.  After the byte
        // permute, bytes 0 and 2 belong to the even token, bytes 1 and 3 to the odd one.
        uint32_t vmask_a = 0xFFFFFFFFu, vmask_b = 0xFFFFFFFFu;
        if (!all_visible) {
          const int tv = t_sub + 2 * c;
          vmask_a = (tv < w.chunk_hi ? 0x00FF00FFu : 0u) | (tv + 1 < w.chunk_hi ? 0xFF00FF00u : 0u);
          vmask_b = (tv + 8 < w.chunk_hi ? 0x00FF00FFu : 0u) | (tv + 9 < w.chunk_hi ? 0xFF00FF00u : 0u);
        }
#pragma unroll
        for (int wj = 0; wj < WJ; ++wj) {
          const int ch = (r >> 2) + 2 * wj;  // 16-byte chunk of word r + 8 wj
          const uint32_t xa = *reinterpret_cast<const uint32_t*>(v0 + (ch ^ x0s) * 16);
          const uint32_t xb = *reinterpret_cast<const uint32_t*>(v0 + 128 + (ch ^ x1s) * 16);
          const uint32_t xc = *reinterpret_cast<const uint32_t*>(v0 + 1024 + (ch ^ x0s) * 16);
          const uint32_t xd = *reinterpret_cast<const uint32_t*>(v0 + 1152 + (ch ^ x1s) * 16);
          // bytes (a0 b0 a1 b1) and (a2 b2 a3 b3): element e of the two tokens side by side
          uint32_t y01[2], y23[2], z01[2], z23[2];
          cvt_e4m3x4(__byte_perm(xa, xb, 0x5140) & vmask_a, y01[0], y01[1]);
          cvt_e4m3x4(__byte_perm(xa, xb, 0x7362) & vmask_a, y23[0], y23[1]);
          cvt_e4m3x4(__byte_perm(xc, xd, 0x5140) & vmask_b, z01[0], z01[1]);
          cvt_e4m3x4(__byte_perm(xc, xd, 0x7362) & vmask_b, z23[0], z23[1]);
#pragma unroll
          for (int p = 0; p < 2; ++p) {
            const uint32_t vf[4] = {y01[p], y23[p], z01[p], z23[p]};  // rows r: d = 4(r+8wj)+p, rows r+8: d+2
#pragma unroll
            for (int nt = 0; nt < NTQ; ++nt) mma_16816<false>(acc[wj * 2 + p][nt], vf, pb[nt][0], pb[nt][1]);
          }
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&w.empty_bar[st]);
  }

  // full row sums (each thread saw tokens r and r+8 of every sub-tile)
#pragma unroll
  for (int nt = 0; nt < NTQ; ++nt)
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      float l = l_run[nt][e], cs = corr[nt][e];
#pragma unroll
      for (int o = 4; o < 32; o <<= 1) {
        l += __shfl_xor_sync(0xffffffffu, l, o);
        cs += __shfl_xor_sync(0xffffffffu, cs, o);
      }
      l_run[nt][e] = l;
      corr[nt][e] = cs;
    }

  // the ring is no longer in use once every consumer warp got here
  asm volatile("bar.sync 1, %0;" ::"n"(kDecConsumerWarps * 32) : "memory");
#pragma unroll
  for (int nt = 0; nt < NTQ; ++nt) {
#pragma unroll
    for (int mt = 0; mt < MTV; ++mt)
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int d = 4 * (r + 8 * (mt >> 1)) + (mt & 1) + (q >> 1) * 2;
        const int rr = nt * 8 + 2 * c + (q & 1);
        w.mine[rr * kCmbRow + d] = acc[mt][nt][q] + corr[nt][q & 1];
      }
    if (r == 0) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        w.mine[(nt * 8 + 2 * c + e) * kCmbRow + D] = m_run[nt][e];
        w.mine[(nt * 8 + 2 * c + e) * kCmbRow + D + 1] = l_run[nt][e];
      }
    }
  }
}

template <int D, int MT, int kFmt, bool kBf16, int NG = 1>
__global__ void __launch_bounds__(kDecThreads, DecOccupancy<kFmt>::kCtasPerSm) decode_splitk_kernel(const __grid_constant__ DecodeArgs a) {
  using Stage = DecStage<D, kFmt, NG>;
  constexpr bool kInt4 = kFmt == kFmtInt4, kFp8 = kFmt == kFmtFp8, kQuant = kFmt == kFmtInt4 || kFmt == kFmtFp8;
  using T = typename Half2Type<kBf16>::T;
  constexpr int W = NG + D / 8;  // int4 words per row (NG scale/shift words, then the nibbles)
  // query rows of one kv head per CTA: MT m-tiles of 16 (16-bit cache) or MT
  // n-tiles of 8 (int4 and fp8 caches, transposed products)
  constexpr int ROWS = kQuant ? 8 * MT : 16 * MT;

  // bytes in flight per SM are what hide HBM latency: the ring takes ~200 KB,
  // i.e. 3 stages of 64 KB (bf16, D = 128) up to 12 stages of 17 KB (int4)
  const int kDecStages = a.stages;
  extern __shared__ __align__(128) uint8_t smem_raw[];
  __shared__ uint64_t full_bar[kDecMaxStages];
  __shared__ uint64_t empty_bar[kDecMaxStages];
  __shared__ uint64_t q_done_bar;

  const int split = blockIdx.x;
  const int b = blockIdx.y;
  const int hblk = blockIdx.z / a.row_blocks;
  const int rblk = blockIdx.z % a.row_blocks;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int hb = a.hb;
  const int wph = kDecConsumerWarps / hb;  // consumer warps per kv head
  constexpr int kSps = Stage::kSubTiles;
  const int TOK = 16 * wph * kSps;

  int kv_len = a.seqlen_k != nullptr ? min(max(a.seqlen_k[b], 0), a.kv_padding) : a.kv_padding;
  // a window is a sequence that starts win_skip keys later: the first key the first query of the sequence sees
  const int win_skip = a.window_size > 0 ? max(kv_len - a.window_span, 0) : 0;
  kv_len -= win_skip;
  const int chunk_lo = split * a.chunk_tokens;
  const int chunk_hi = min(chunk_lo + a.chunk_tokens, kv_len);
  if (chunk_lo >= chunk_hi) {
    // nothing for this CTA (uniform: the whole CTA leaves).  Without a merge
    // pass the rows of an empty sequence still have to be defined: out = 0,
    // lse = -inf.
    if (a.split_k == 1 && split == 0) {
      const int nrows = min(ROWS, a.rows - rblk * ROWS);
      for (int i = threadIdx.x; i < hb * nrows * D; i += blockDim.x) {
        const int d = i % D, rr = (i / D) % nrows, hh = i / (D * nrows);
        const int row = rblk * ROWS + rr, head = hblk * hb + hh;
        const int qi = row / a.q_per_kv, h = row % a.q_per_kv;
        const int64_t off = (int64_t(b) * a.mq + qi) * a.o_sm + int64_t(head) * a.o_sg + int64_t(h) * a.o_sh + d;
        if (a.out_dtype == XFB200_F32)
          reinterpret_cast<float*>(a.out)[off] = 0.f;
        else
          reinterpret_cast<unsigned short*>(a.out)[off] = 0;
        if (d == 0 && a.lse != nullptr) a.lse[int64_t(head) * a.lse_sg + int64_t(h) * a.lse_sh + int64_t(b) * a.mq + qi] = -INFINITY;
      }
    }
    return;
  }
  const int n_tiles = (chunk_hi - chunk_lo + TOK - 1) / TOK;

  const int kv_bytes = a.kv_bytes, stage_bytes = a.stage_bytes;
  const int row_bytes = Stage::row_bytes(hb);
  // swizzled tiles want 1024-byte aligned stages; the static barriers precede the dynamic part
  // (an offset from the array, not a cast of a rounded integer: the compiler must keep seeing shared memory)
  uint8_t* stage_base = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  // Q is staged once in the region of the LAST stages; the producer does not
  // fill those before every consumer warp has taken its Q fragments
  uint8_t* q_smem = stage_base + a.q_first_stage * stage_bytes;     // 8 warps * 16*MT rows * D*2 B
  constexpr int kQRowBytes = D * 2;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kDecStages; ++i) {
      mbar_init(&full_bar[i], kFp8 ? 33 : 1);  // fp8: + one arrival per lane of the copy warp (scale/shift copies)
      mbar_init(&empty_bar[i], kDecConsumerWarps);
    }
    mbar_init(&q_done_bar, kDecConsumerWarps);
    mbar_fence_init();
  }
  __syncthreads();

  if (warp == kDecConsumerWarps) {
    // ------------------------------------------------------------ producer
    const uint8_t* kg = reinterpret_cast<const uint8_t*>(a.k);
    const uint8_t* vg = reinterpret_cast<const uint8_t*>(a.v);
    constexpr int kElem = kQuant ? 4 : 2;  // bytes per element of the k/v tensors (int32 words when quantised)
    constexpr int kHeadBytes = kInt4 ? W * 4 : kFp8 ? D : D * 2;
    const int head0 = hblk * hb;
    // physical row of token t; the page-table entry is kept while t stays on its page,
    // so that a lane waits for that load once per page instead of once per stage
    int cached_page = -1;
    int64_t cached_base = 0;
    const int64_t kv_base = (a.kv_start != nullptr ? int64_t(a.kv_start[b]) : int64_t(b) * a.kv_padding) + win_skip;  // padded / gappy cache
    const int t_shift = ((a.block_tables != nullptr && a.kv_start != nullptr) ? a.kv_start[b] : 0) + win_skip;       // paged gappy cache
    auto row_of = [&](int t_rel) -> int64_t {
      if (a.block_tables == nullptr) return kv_base + t_rel;
      const int t = t_rel + t_shift;
      const int pg = t / a.page_size;
      if (pg != cached_page) {
        cached_page = pg;
        cached_base = int64_t(a.block_tables[int64_t(b) * a.bt_stride + pg]) * a.page_size;
      }
      return cached_base + (t - pg * a.page_size);
    };
    for (int tile = 0; tile < n_tiles; ++tile) {
      const int st = tile % kDecStages;
      if (tile >= kDecStages) {
        if (!mbar_wait(&empty_bar[st], ((tile / kDecStages) - 1) & 1)) {
          if (lane == 0) atomicCAS(a.status, 0, 1);
          return;
        }
      } else if (kQuant && tile == a.q_first_stage) {
        if (!mbar_wait(&q_done_bar, 0)) {
          if (lane == 0) atomicCAS(a.status, 0, 3);
          return;
        }
      }
      const int t0 = chunk_lo + tile * TOK;
      const int nvalid = min(TOK, chunk_hi - t0);
      uint8_t* ks = stage_base + st * stage_bytes;
      uint8_t* vs = ks + kv_bytes;
      if (a.copy_mode == 3) {
        // one tiled copy per run of box_tok tokens: {64 elements} x {box_tok rows} x {hb*D/64 column groups}
        if (lane == 0) {
          const int nbox = (nvalid + a.box_tok - 1) / a.box_tok;
          const uint32_t box_bytes = uint32_t(a.box_tok) * hb * kHeadBytes;
          const bool ss_tma = kFp8 && a.ss_tma;
          const uint32_t box_ss = uint32_t(a.box_tok) * hb * (a.ss_tma == 2 ? 4u : 16u);  // per (token, head): the word, or the word and three replicas
          mbar_expect_tx(&full_bar[st], uint32_t(nbox) * (box_bytes + (ss_tma ? box_ss : 0u)) * 2u);
          for (int bx = 0; bx < nbox; ++bx) {
            const int64_t row = row_of(t0 + bx * a.box_tok);
            // third coordinate: 128-byte column group (16-bit cache) or kv head (fp8: a head is one 128-byte row)
            const int c2 = kFp8 ? head0 : head0 * (D / 64);
            tma_load_3d(ks + bx * box_bytes, &a.tm_k, &full_bar[st], 0, int(row), c2);
            tma_load_3d(vs + bx * box_bytes, &a.tm_v, &full_bar[st], 0, int(row), c2);
            if (ss_tma) {
              uint8_t* ss = ks + 2 * kv_bytes;
              if (a.ss_tma == 2) {  // compact: {kv heads, token rows}
                tma_load_3d(ss + bx * box_ss, &a.tm_kss, &full_bar[st], head0, int(row), 0);
                tma_load_3d(ss + a.ss_bytes + bx * box_ss, &a.tm_vss, &full_bar[st], head0, int(row), 0);
              } else {  // {4 words, kv heads, token rows}
                tma_load_3d(ss + bx * box_ss, &a.tm_kss, &full_bar[st], 0, head0, int(row));
                tma_load_3d(ss + a.ss_bytes + bx * box_ss, &a.tm_vss, &full_bar[st], 0, head0, int(row));
              }
            }
          }
        }
        if constexpr (kFp8) {
          // The scale/shift words (one per token and head, 128 per tensor and stage)
          // go straight from global to shared memory with 4-byte asynchronous copies,
          // [head][token] behind the K and V parts of the stage.  Every lane then lets
          // the full barrier count the completion of its copies (the barrier expects
          // 32 such arrivals besides the one that carries the TMA byte count), so the
          // copy warp never waits for this data itself.
          uint32_t* ssk = reinterpret_cast<uint32_t*>(ks + 2 * kv_bytes);
          uint32_t* ssv = ssk + hb * TOK;
          for (int i = lane; i < (a.ss_tma ? 0 : nvalid * hb); i += 32) {
            const int tok = i / hb, hh = i % hb;  // heads fastest: neighbouring lanes read neighbouring words
            const int64_t row = row_of(t0 + tok);
            cp_async_4(ssk + hh * TOK + tok, a.k_ss + row * a.kss_m + (head0 + hh) * a.kss_g);
            cp_async_4(ssv + hh * TOK + tok, a.v_ss + row * a.vss_m + (head0 + hh) * a.vss_g);
          }
          cp_async_mbar_arrive_noinc(&full_bar[st]);
        }
        __syncwarp();
        continue;
      }
      if (a.copy_mode == 2) {
        // no TMA: 32-bit loads (rows that are not 16-B aligned)
        const int words_per_head = kHeadBytes / 4;
        const int total = nvalid * hb * words_per_head;
        for (int i = lane; i < total; i += 32) {
          const int tok = i / (hb * words_per_head);
          const int rem = i % (hb * words_per_head);
          const int hh = rem / words_per_head, wd = rem % words_per_head;
          const int t = t0 + tok;
          const int64_t row = row_of(t);
          const int64_t ko = (row * a.k_sm + (head0 + hh) * a.k_sg) * kElem + wd * 4;
          const int64_t vo = (row * a.v_sm + (head0 + hh) * a.v_sg) * kElem + wd * 4;
          *reinterpret_cast<uint32_t*>(ks + tok * row_bytes + hh * kHeadBytes + wd * 4) = __ldg(reinterpret_cast<const uint32_t*>(kg + ko));
          *reinterpret_cast<uint32_t*>(vs + tok * row_bytes + hh * kHeadBytes + wd * 4) = __ldg(reinterpret_cast<const uint32_t*>(vg + vo));
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&full_bar[st]);
        continue;
      }
      const int grp = (kInt4 && a.copy_mode == 0) ? a.copy_group : 1;
      const int ngroups = (nvalid + grp - 1) / grp;  // a group is always copied whole
      const int per_tok_copies = a.copy_mode == 0 ? 1 : hb;
      const uint32_t seg_bytes = a.copy_mode == 0 ? uint32_t(hb * kHeadBytes * grp) : uint32_t(kHeadBytes);
      if (lane == 0) mbar_expect_tx(&full_bar[st], uint32_t(ngroups) * per_tok_copies * seg_bytes * 2u);
      __syncwarp();
      for (int i = lane; i < ngroups * per_tok_copies; i += 32) {
        const int gi = i / per_tok_copies;
        const int hh = i % per_tok_copies;
        const int tok = gi * grp;
        const int t = t0 + tok;
        const int64_t row = row_of(t);
        const int64_t ko = (row * a.k_sm + (head0 + hh) * a.k_sg) * kElem;
        const int64_t vo = (row * a.v_sm + (head0 + hh) * a.v_sg) * kElem;
        bulk_g2s(ks + tok * row_bytes + hh * kHeadBytes, kg + ko, seg_bytes, &full_bar[st]);
        bulk_g2s(vs + tok * row_bytes + hh * kHeadBytes, vg + vo, seg_bytes, &full_bar[st]);
      }
    }
    return;
  }

  // -------------------------------------------------------------- consumers
  const int hw = warp % hb;   // kv head of this warp inside the block
  const int sub = warp / hb;  // 16-token sub-tile of each stage
  const int head = hblk * hb + hw;
  const int row0 = rblk * ROWS;  // first query row (of this kv head) handled here
  const int R = a.rows;

  // ---- int4 path: stage Q (this warp's head) in shared memory, zero rows beyond R.
  // (The 16-bit path reads its fragments from global memory: a fragment load that
  // nothing consumes yet could still be in flight when the staging area is handed
  // back to the copy engine.  The int4 path converts what it loads before it
  // arrives on q_done, so its loads have returned by then.)
  if constexpr (kQuant) {
    uint8_t* qs = q_smem + warp * ROWS * kQRowBytes;
    const T* qg = reinterpret_cast<const T*>(a.q);
    for (int i = lane; i < ROWS * (D / 8); i += 32) {
      const int rr = i / (D / 8), ch = i % (D / 8);
      const int row = row0 + rr;
      uint4 val = make_uint4(0, 0, 0, 0);
      if (row < R) {
        const int qi = row / a.q_per_kv, h = row % a.q_per_kv;
        const int64_t off = (int64_t(b) * a.mq + qi) * a.q_sm + int64_t(head) * a.q_sg + int64_t(h) * a.q_sh + ch * 8;
        val = *reinterpret_cast<const uint4*>(qg + off);
      }
      *reinterpret_cast<uint4*>(qs + rr * kQRowBytes + ch * 16) = val;
    }
    __syncwarp();
  }
  // Partial results of the warps meet in shared memory once the ring is drained.
  float* cmb = reinterpret_cast<float*>(smem_raw);  // [warp][ROWS][D + 2]  (acc, m, l)
  constexpr int kCmbRow = D + 2;
  DecWarp w;
  w.qs = q_smem + warp * ROWS * kQRowBytes;
  w.stage_base = stage_base;
  w.full_bar = full_bar, w.empty_bar = empty_bar, w.q_done_bar = &q_done_bar;
  w.mine = cmb + size_t(warp) * ROWS * kCmbRow;
  w.lane = lane, w.hw = hw, w.sub = sub, w.wph = wph, w.row0 = row0;
  w.b = b, w.head = head;
  w.chunk_lo = chunk_lo, w.chunk_hi = chunk_hi, w.kv_len = kv_len, w.n_tiles = n_tiles;
  w.tok_per_stage = TOK, w.kv_bytes = kv_bytes, w.stage_bytes = stage_bytes, w.row_bytes = row_bytes, w.stages = kDecStages;
  if constexpr (kInt4 && NG == 1)
    consume_int4<D, MT, kBf16>(a, w);
  else if constexpr (kInt4)
    consume_int4_groups<D, MT, kBf16, NG>(a, w);
  else if constexpr (kFp8)
    consume_fp8<D, MT, kBf16>(a, w);
  else
    consume_plain<D, MT, kBf16, kFmt == kFmtPlainX>(a, w);
  asm volatile("bar.sync 1, %0;" ::"n"(kDecConsumerWarps * 32) : "memory");
  // warps of head hw share the rows: warp `sub` finalises rows sub, sub+wph, ...
  const bool direct = a.split_k == 1;
  for (int rr = sub; rr < ROWS; rr += wph) {
    const int row = row0 + rr;
    if (row >= R) break;
    float mx = -INFINITY;
    for (int w2 = 0; w2 < wph; ++w2) mx = fmaxf(mx, cmb[size_t(w2 * hb + hw) * ROWS * kCmbRow + rr * kCmbRow + D]);
    const float m_use = mx == -INFINITY ? 0.f : mx;
    float den = 0.f;
    float o[D / 32];
#pragma unroll
    for (int i = 0; i < D / 32; ++i) o[i] = 0.f;
    for (int w2 = 0; w2 < wph; ++w2) {
      const float* src = cmb + size_t(w2 * hb + hw) * ROWS * kCmbRow + rr * kCmbRow;
      const float mw = src[D];
      if (mw == -INFINITY) continue;
      const float wgt = fast_exp2(mw - m_use);
      den += wgt * src[D + 1];
#pragma unroll
      for (int i = 0; i < D / 32; ++i) o[i] += wgt * src[i * 32 + lane];
    }
    const float inv = den > 0.f ? 1.f / den : 0.f;
    const float lse = den > 0.f ? (m_use + log2f(den)) * 0.6931471805599453f : -INFINITY;
    const int qi = row / a.q_per_kv, h = row % a.q_per_kv;
    if (direct) {
      const int64_t off = (int64_t(b) * a.mq + qi) * a.o_sm + int64_t(head) * a.o_sg + int64_t(h) * a.o_sh;
#pragma unroll
      for (int i = 0; i < D / 32; ++i) {
        const float val = o[i] * inv;
        const int d = i * 32 + lane;
        if (a.out_dtype == XFB200_F32)
          reinterpret_cast<float*>(a.out)[off + d] = val;
        else if (a.out_dtype == XFB200_BF16)
          reinterpret_cast<__nv_bfloat16*>(a.out)[off + d] = __float2bfloat16_rn(val);
        else
          reinterpret_cast<__half*>(a.out)[off + d] = __float2half_rn(val);
      }
      if (a.lse != nullptr && lane == 0) a.lse[int64_t(head) * a.lse_sg + int64_t(h) * a.lse_sh + int64_t(b) * a.mq + qi] = lse;
    } else {
      const int64_t prow = ((int64_t(b) * a.split_k + split) * a.kv_heads + head) * R + row;
      float* po = a.part_o + prow * D;
#pragma unroll
      for (int i = 0; i < D / 32; ++i) po[i * 32 + lane] = o[i] * inv;
      if (lane == 0) a.part_lse[prow] = lse;
    }
  }
}

// ---------------------------------------------------------------------------
// Merge of the per-chunk partials of each sequence.  One warp per output row
// (b, kv head, query row); chunks are visited in order, so the result is
// deterministic.  Only the chunks that exist for sequence b are read.
// ---------------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(256) decode_merge_kernel(const __grid_constant__ DecodeArgs a) {
  const int lane = threadIdx.x & 31;
  const int64_t gw = int64_t(blockIdx.x) * 8 + (threadIdx.x >> 5);
  const int R = a.rows;
  const int64_t total = int64_t(a.batch) * a.kv_heads * R;
  if (gw >= total) return;
  const int row = int(gw % R);
  const int head = int((gw / R) % a.kv_heads);
  const int b = int(gw / (int64_t(R) * a.kv_heads));
  int kv_len = a.seqlen_k != nullptr ? min(max(a.seqlen_k[b], 0), a.kv_padding) : a.kv_padding;
  if (a.window_size > 0) kv_len = min(kv_len, a.window_span);
  const int nsplit = min(a.split_k, (kv_len + a.chunk_tokens - 1) / a.chunk_tokens);

  float mx = -INFINITY;
  for (int s = lane; s < nsplit; s += 32) {
    const float l = a.part_lse[((int64_t(b) * a.split_k + s) * a.kv_heads + head) * R + row];
    mx = fmaxf(mx, l);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  constexpr int V = D / 32;
  float acc[V];
#pragma unroll
  for (int i = 0; i < V; ++i) acc[i] = 0.f;
  float den = 0.f;
  if (mx > -INFINITY) {
    for (int s = 0; s < nsplit; ++s) {
      const int64_t prow = ((int64_t(b) * a.split_k + s) * a.kv_heads + head) * R + row;
      const float l = a.part_lse[prow];
      if (!(l > -INFINITY)) continue;
      const float w = __expf(l - mx);
      den += w;
      const float* po = a.part_o + prow * D + lane * V;
      if constexpr (V == 4) {
        const float4 x = *reinterpret_cast<const float4*>(po);
        acc[0] += w * x.x, acc[1] += w * x.y, acc[2] += w * x.z, acc[3] += w * x.w;
      } else if constexpr (V == 2) {
        const float2 x = *reinterpret_cast<const float2*>(po);
        acc[0] += w * x.x, acc[1] += w * x.y;
      } else {
#pragma unroll
        for (int i = 0; i < V; ++i) acc[i] += w * po[i];
      }
    }
  }
  const float inv = den > 0.f ? 1.f / den : 0.f;
  const int qi = row / a.q_per_kv, h = row % a.q_per_kv;
  const int64_t off = (int64_t(b) * a.mq + qi) * a.o_sm + int64_t(head) * a.o_sg + int64_t(h) * a.o_sh + lane * V;
#pragma unroll
  for (int i = 0; i < V; ++i) {
    const float val = acc[i] * inv;
    if (a.out_dtype == XFB200_F32)
      reinterpret_cast<float*>(a.out)[off + i] = val;
    else if (a.out_dtype == XFB200_BF16)
      reinterpret_cast<__nv_bfloat16*>(a.out)[off + i] = __float2bfloat16_rn(val);
    else
      reinterpret_cast<__half*>(a.out)[off + i] = __float2half_rn(val);
  }
  if (a.lse != nullptr && lane == 0)
    a.lse[int64_t(head) * a.lse_sg + int64_t(h) * a.lse_sh + int64_t(b) * a.mq + qi] = den > 0.f ? mx + __logf(den) : -INFINITY;
}

// ------------------------------------------------------------------ host side
int decode_chunk_tokens(int kv_bound, int split_k) {
  int c = (kv_bound + split_k - 1) / split_k;
  c = (c + kDecChunkAlign - 1) / kDecChunkAlign * kDecChunkAlign;
  return c < kDecChunkAlign ? kDecChunkAlign : c;
}

template <int D, int MT, int kFmt, bool kBf16, int NG = 1>
static int launch_decode_t(const DecodeArgs& a_in, int head_blocks, cudaStream_t stream) {
  using Stage = DecStage<D, kFmt, NG>;
  constexpr bool kQuant = kFmt == kFmtInt4 || kFmt == kFmtFp8;
  constexpr int ROWS = kQuant ? 8 * MT : 16 * MT;
  // tiled copies need no row padding
  const int kv_bytes = kFmt == kFmtFp8      ? Stage::tokens(a_in.hb) * a_in.hb * D
                       : a_in.copy_mode == 3 ? Stage::tokens(a_in.hb) * a_in.hb * D * 2
                                             : Stage::kv_bytes(a_in.hb);
  const int ss_bytes = Stage::ss_bytes(a_in.hb) * (a_in.ss_tma == 1 ? 4 : 1);  // 16 bytes per entry when the replicas come along
  const size_t stage_bytes = 2 * size_t(kv_bytes) + 2 * size_t(ss_bytes);
  const size_t qbytes = size_t(kDecConsumerWarps) * ROWS * (D * 2);
  const size_t cmb = size_t(kDecConsumerWarps) * ROWS * (D + 2) * 4;
  int stages = int(DecOccupancy<kFmt>::kRingBudget / stage_bytes);
  stages = stages > kDecMaxStages ? kDecMaxStages : stages;
  const int q_stages = kQuant ? int((qbytes + stage_bytes - 1) / stage_bytes) : 0;  // only the quantised paths stage Q
  if (stages < 2 || q_stages > stages) return set_error(XFB200_E_UNSUPPORTED, "decode: shared-memory ring too small for this shape");
  DecodeArgs a = a_in;
  a.stages = stages;
  a.q_first_stage = stages - q_stages;
  a.kv_bytes = kv_bytes;
  a.stage_bytes = int(stage_bytes);
  a.ss_bytes = ss_bytes;
  const size_t ring = stages * stage_bytes + 1024;  // the kernel aligns the ring to 1024 B
  const size_t smem = ring > cmb ? ring : cmb;
  auto kern = decode_splitk_kernel<D, MT, kFmt, kBf16, NG>;
  // 227 KB per CTA includes the static part (the mbarriers)
  if (smem + 1024 > size_t(227 * 1024) / DecOccupancy<kFmt>::kCtasPerSm) return set_error(XFB200_E_UNSUPPORTED, "decode: shared memory %zu B exceeds 227 KB", smem);
  // per instantiation and device (the attribute belongs to the device's context): largest size opted into so far
  static size_t configured[kMaxDevices] = {0};
  const int dev = current_device();
  if (dev < 0 || smem > configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    if (e != cudaSuccess) return cuda_fail("decode: cudaFuncSetAttribute", e);
    if (dev >= 0) configured[dev] = smem;
  }
  dim3 grid(a.split_k, a.batch, head_blocks * a.row_blocks);
  kern<<<grid, kDecThreads, smem, stream>>>(a);
  int rc = check_launch("decode_splitk_kernel");
  if (rc != XFB200_OK) return rc;
  if (a.split_k > 1) {
    const int64_t rows = int64_t(a.batch) * a.kv_heads * a.rows;
    decode_merge_kernel<D><<<unsigned((rows + 7) / 8), 256, 0, stream>>>(a);
    rc = check_launch("decode_merge_kernel");
  }
  return rc;
}

template <int D, int kFmt, bool kBf16, int NG = 1>
static int launch_decode_mt(const DecodeArgs& a, int mt, int head_blocks, cudaStream_t stream) {
  if (mt == 1) return launch_decode_t<D, 1, kFmt, kBf16, NG>(a, head_blocks, stream);
  return launch_decode_t<D, 2, kFmt, kBf16, NG>(a, head_blocks, stream);
}

}  // namespace xfb

extern "C" size_t xfb200_decode_scratch_bytes(int32_t batch, int32_t mq, int32_t kv_heads, int32_t q_per_kv, int32_t head_dim,
                                              int32_t split_k) {
  if (split_k <= 1) return 0;
  const size_t rows = size_t(batch) * split_k * kv_heads * mq * q_per_kv;
  const size_t o = (rows * head_dim * 4 + 255) & ~size_t(255);
  const size_t l = (rows * 4 + 255) & ~size_t(255);
  return o + l;
}

extern "C" int xfb200_decode_forward(const xfb200_decode_params* p, void* stream) {
  using namespace xfb;
  if (p == nullptr) return set_error(XFB200_E_INVALID, "decode: null params");
  if (p->batch < 0 || p->mq < 1 || p->kv_heads < 1 || p->q_per_kv < 1) return set_error(XFB200_E_INVALID, "decode: bad extents");
  if (p->batch == 0) return XFB200_OK;
  if (p->q == nullptr || p->k == nullptr || p->v == nullptr || p->out == nullptr)
    return set_error(XFB200_E_INVALID, "decode: null tensor pointer");
  if (p->head_dim != 64 && p->head_dim != 128)
    return set_error(XFB200_E_UNSUPPORTED, "decode: head_dim %d not in {64, 128}", p->head_dim);
  if (p->dtype != XFB200_BF16 && p->dtype != XFB200_F16) return set_error(XFB200_E_INVALID, "decode: q dtype must be bf16 or f16");
  const bool int4 = p->kv_format == XFB200_KV_INT4_ROWWISE;
  const bool fp8 = p->kv_format == XFB200_KV_FP8_ROWWISE;
  const int ng = int4 ? p->num_quant_groups : 1;
  if (int4 && (ng != 1 && ng != 2 && ng != 4 && ng != 8))
    return set_error(XFB200_E_UNSUPPORTED, "decode: int4 cache with %d quantisation groups per row (1, 2, 4 or 8)", ng);
  if (int4 && p->head_dim / ng < 16)
    return set_error(XFB200_E_UNSUPPORTED, "decode: int4 groups of %d elements (at least 16)", p->head_dim / ng);
  if (!int4 && !fp8 && p->kv_format != XFB200_KV_PLAIN) return set_error(XFB200_E_INVALID, "decode: bad kv_format %d", p->kv_format);
  if (fp8 && (p->k_scale_shift == nullptr || p->v_scale_shift == nullptr))
    return set_error(XFB200_E_INVALID, "decode: an fp8 cache needs k_scale_shift and v_scale_shift");
  if (fp8 && p->head_dim != 128) return set_error(XFB200_E_UNSUPPORTED, "decode: fp8 cache with head_dim %d (only 128)", p->head_dim);
  if (p->split_k < 1 || p->split_k > 1024) return set_error(XFB200_E_INVALID, "decode: split_k %d out of range", p->split_k);
  if (p->kv_padding < 1) return set_error(XFB200_E_INVALID, "decode: kv_padding must be positive");
  if (p->block_tables != nullptr && (p->page_size < 1 || p->block_table_stride < 1))
    return set_error(XFB200_E_INVALID, "decode: paged cache needs page_size and block_table_stride");
  if (p->mask_type != XFB200_MASK_NONE && p->mask_type != XFB200_MASK_CAUSAL_BOTTOM_RIGHT)
    return set_error(XFB200_E_UNSUPPORTED, "decode: mask_type %d", p->mask_type);
  const int R = p->mq * p->q_per_kv;
  // query rows of one kv head per CTA: 16 or 32 (16-bit cache), 8 or 16 (int4 cache)
  const int tile_rows = (int4 || fp8) ? 8 : 16;
  const int mt = R <= tile_rows ? 1 : 2;
  const int row_blocks = (R + tile_rows * mt - 1) / (tile_rows * mt);
  if (p->split_k > 1 && p->scratch == nullptr) return set_error(XFB200_E_INVALID, "decode: split_k > 1 needs scratch");
  if (p->split_k > 1 && (reinterpret_cast<uintptr_t>(p->scratch) & 255)) return set_error(XFB200_E_INVALID, "decode: scratch must be 256-B aligned");

  DecodeArgs a{};
  a.q = p->q, a.k = p->k, a.v = p->v, a.out = p->out, a.lse = p->lse;
  a.seqlen_k = p->seqlen_k, a.block_tables = p->block_tables, a.kv_start = p->kv_seqstart;
  a.batch = p->batch, a.mq = p->mq, a.kv_heads = p->kv_heads, a.q_per_kv = p->q_per_kv;
  a.kv_padding = p->kv_padding, a.page_size = p->page_size, a.bt_stride = p->block_table_stride;
  a.split_k = p->split_k;
  // with a window no sequence has more than window_size + mq - 1 keys to read: the chunks divide that
  const int window_span = p->window_size > 0 ? p->window_size + p->mq - 1 : 0;
  a.chunk_tokens = decode_chunk_tokens(window_span > 0 && window_span < p->kv_padding ? window_span : p->kv_padding, p->split_k);
  a.rows = R, a.row_blocks = row_blocks;
  a.q_sm = p->q_stride_m, a.q_sg = p->q_stride_g, a.q_sh = p->q_stride_h;
  a.k_sm = p->k_stride_m, a.k_sg = p->k_stride_g, a.v_sm = p->v_stride_m, a.v_sg = p->v_stride_g;
  if (p->kv_heads == 1) a.k_sg = a.v_sg = 0;  // the stride of an extent-1 axis is meaningless
  a.o_sm = p->o_stride_m, a.o_sg = p->o_stride_g, a.o_sh = p->o_stride_h;
  a.lse_sg = p->lse_stride_g, a.lse_sh = p->lse_stride_h;
  a.k_ss = p->k_scale_shift, a.v_ss = p->v_scale_shift;
  a.kss_m = p->ks_stride_m, a.kss_g = p->kv_heads == 1 ? 0 : p->ks_stride_g;
  a.vss_m = p->vs_stride_m, a.vss_g = p->kv_heads == 1 ? 0 : p->vs_stride_g;
  a.causal = p->mask_type == XFB200_MASK_CAUSAL_BOTTOM_RIGHT;
  a.out_dtype = p->out_dtype;
  a.scale_log2 = p->scale * 1.4426950408889634f;
  if (p->split_k > 1) {
    const size_t rows = size_t(p->batch) * p->split_k * p->kv_heads * R;
    a.part_o = reinterpret_cast<float*>(p->scratch);
    a.part_lse = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(p->scratch) + ((rows * p->head_dim * 4 + 255) & ~size_t(255)));
  }
  {
    int32_t* words = device_words();
    if (words == nullptr) return set_error(XFB200_E_CUDA, "decode: cannot resolve the device status word");
    a.status = words + kWordDecodeStatus;
  }

  // kv heads per CTA: the largest of 8, 4, 2, 1 that divides kv_heads
  int hb = 8;
  while (p->kv_heads % hb) hb >>= 1;
  a.hb = hb;
  const int head_blocks = p->kv_heads / hb;

  // how the producer may copy: whole stripes by TMA when alignment allows
  const int elem = (int4 || fp8) ? 4 : 2;
  const int head_elems = int4 ? (ng + p->head_dim / 8) : fp8 ? p->head_dim / 4 : p->head_dim;
  const bool heads_contig = hb == 1 || (a.k_sg == head_elems && a.v_sg == head_elems);
  auto al16 = [&](int64_t elems) { return (elems * elem) % 16 == 0; };
  const bool base_al = (reinterpret_cast<uintptr_t>(p->k) % 16 == 0) && (reinterpret_cast<uintptr_t>(p->v) % 16 == 0);
  a.copy_group = 1;
  const bool moved_start = p->kv_seqstart != nullptr || p->window_size > 0;  // a sequence's first key is not the first row of its slot
  if (!base_al) {
    a.copy_mode = 2;
  } else if (heads_contig && al16(p->k_stride_m) && al16(p->v_stride_m) && al16(int64_t(hb) * head_elems) &&
             al16(a.k_sg * hb) && al16(a.v_sg * hb)) {
    a.copy_mode = 0;
    // The copy engine's throughput is set by the number of copies, not by
    // their bytes, and a packed token stripe is only hb * 68 B: when the
    // tokens of a page (or of the padded row) follow one another in memory,
    // copy runs of up to 64 tokens at once.
    // (not for gappy caches: a run could cross a page, or the end of the tensor)
    if (int4 && !moved_start && head_blocks == 1 && p->k_stride_m == int64_t(hb) * head_elems && p->v_stride_m == p->k_stride_m) {
      const int span = p->block_tables ? p->page_size : p->kv_padding;
      // a run must fit the stage it is copied into (a power of two of tokens)
      const int stage_tokens = p->head_dim == 128 ? DecStage<128, kFmtInt4>::tokens(hb) : DecStage<64, kFmtInt4>::tokens(hb);
      int g = stage_tokens < 64 ? stage_tokens : 64;
      while (g > 1 && span % g) g >>= 1;
      a.copy_group = g;
    }
  } else if (al16(p->k_stride_m) && al16(p->v_stride_m) && al16(a.k_sg) && al16(a.v_sg) && al16(head_elems)) {
    a.copy_mode = 1;
  } else if (int4 && !moved_start && heads_contig && head_blocks == 1 && p->k_stride_m == int64_t(hb) * head_elems &&
             p->v_stride_m == p->k_stride_m) {
    // tokens are contiguous: copy groups of 2 or 4 tokens so that each copy is a multiple of 16 B
    int g = 2;
    while (g <= 4 && !al16(int64_t(g) * p->k_stride_m)) g <<= 1;
    const bool starts_ok = p->block_tables ? (p->page_size % g == 0) : (p->kv_padding % g == 0);
    if (g <= 4 && starts_ok) {
      a.copy_mode = 0;
      a.copy_group = g;
    } else {
      a.copy_mode = 2;
    }
  } else {
    a.copy_mode = 2;
  }
  if (!int4 && a.copy_mode == 2) return set_error(XFB200_E_INVALID, "decode: K/V rows must be 16-byte aligned");
  if (fp8 && a.copy_mode != 0) return set_error(XFB200_E_UNSUPPORTED, "decode: the heads of an fp8 cache row must be contiguous");
  a.box_tok = 16;
  a.bias = p->bias, a.bias_dtype = p->bias_dtype, a.inv_scale = p->scale > 0.f ? 1.f / p->scale : 0.f;
  a.bias_b = p->bias_stride_b, a.bias_kvh = p->bias_stride_kvh, a.bias_q = p->bias_stride_q, a.bias_m = p->bias_stride_m;
  if (p->bias != nullptr) {
    if (int4 || fp8) return set_error(XFB200_E_UNSUPPORTED, "decode: an additive bias needs a 16-bit cache");
    if (p->seqlen_k != nullptr || p->block_tables != nullptr || p->kv_seqstart != nullptr)
      return set_error(XFB200_E_UNSUPPORTED, "decode: an additive bias needs the plain cache layout (no sequence lengths, no page table)");
    if (p->bias_dtype != XFB200_BF16 && p->bias_dtype != XFB200_F16 && p->bias_dtype != XFB200_F32)
      return set_error(XFB200_E_INVALID, "decode: bad bias_dtype %d", p->bias_dtype);
    if (!(p->scale > 0.f)) return set_error(XFB200_E_UNSUPPORTED, "decode: an additive bias needs a positive scale");
  }
  a.window_size = p->window_size, a.window_span = window_span;
  if (p->window_size < 0) return set_error(XFB200_E_INVALID, "decode: window_size %d", p->window_size);
  if (p->window_size > 0 && p->mask_type != XFB200_MASK_CAUSAL_BOTTOM_RIGHT)
    return set_error(XFB200_E_UNSUPPORTED, "decode: a window needs the bottom-right causal mask");
  if (p->window_size > 0 && p->mq != 1 && (int4 || fp8))
    return set_error(XFB200_E_UNSUPPORTED, "decode: a window over a quantised cache needs one query per sequence");
  // a window moves the first key of a sequence like a gappy start does
  const bool gappy = p->kv_seqstart != nullptr || p->window_size > 0;
  if (gappy && p->block_tables == nullptr && p->kv_seqstart != nullptr && p->kv_rows <= 0)
    return set_error(XFB200_E_INVALID, "decode: a gappy cache needs kv_rows, the number of key rows of the tensor");
  // (a run of a paged gappy cache may start anywhere inside a page: per-token copies there)
  if (!int4 && a.copy_mode == 0 && !(gappy && p->block_tables != nullptr) &&
      (p->kv_heads == 1 || (a.k_sg == head_elems && a.v_sg == head_elems))) {
    // The copy engine's throughput is set by the number of copies: one tiled
    // copy per run of tokens that is contiguous in the cache (a whole stage, or
    // what a page allows) instead of one bulk copy per token.
    const int stage_tokens = 16 * (kDecConsumerWarps / hb);
    int box = stage_tokens;
    if (p->block_tables != nullptr)
      while (box > 1 && p->page_size % box) box >>= 1;
    EncodeTiledFn enc = encode_tiled_fn();
    if (box >= (fp8 ? 16 : 8) && enc != nullptr) {
      // token rows: all of a padded cache (rows past the end read as zero); a paged pool's
      // size when the caller states it (kv_rows), so that a bad table entry reads zeros
      // instead of foreign memory; a copy never leaves its page
      const cuuint64_t rows = p->kv_rows > 0              ? cuuint64_t(p->kv_rows)
                              : p->block_tables != nullptr ? (cuuint64_t(1) << 31)
                                                           : cuuint64_t(p->batch) * p->kv_padding;
      // 16-bit cache: {64 elements, token rows, 128-byte column groups}; fp8: {128 bytes, token rows, kv heads}
      const cuuint64_t dims[3] = {cuuint64_t(fp8 ? 128 : 64), rows, fp8 ? cuuint64_t(p->kv_heads) : cuuint64_t(p->kv_heads) * (p->head_dim / 64)};
      const cuuint32_t bx[3] = {cuuint32_t(fp8 ? 128 : 64), cuuint32_t(box), cuuint32_t(fp8 ? hb : hb * (p->head_dim / 64))};
      const cuuint32_t estr[3] = {1, 1, 1};
      const CUtensorMapDataType dt = fp8                      ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                     : p->dtype == XFB200_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                               : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
      const cuuint64_t ks[2] = {cuuint64_t(p->k_stride_m) * elem, 128}, vs[2] = {cuuint64_t(p->v_stride_m) * elem, 128};
      const CUresult rk = enc(&a.tm_k, dt, 3, const_cast<void*>(p->k), dims, ks, bx, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
      const CUresult rv = enc(&a.tm_v, dt, 3, const_cast<void*>(p->v), dims, vs, bx, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
      if (rk == CUDA_SUCCESS && rv == CUDA_SUCCESS) {  // otherwise stay with the per-token bulk copies
        a.copy_mode = 3;
        a.box_tok = box;
      }
    }
  }

  a.ss_tma = 0;
  if (fp8 && a.copy_mode == 3 && p->ss_words >= 4) {
    // The caller vouches for at least 4 consecutive int32 at every (token, kv head)
    // entry of the scale/shift tensors (the word and its replicas for the query
    // heads of the group): 16 bytes per entry can then come by tiled copies, one
    // per tensor and run of tokens, instead of one 4-byte copy per word.
    auto ok16 = [](const void* ptr, int64_t m, int64_t g, int heads) {
      return (reinterpret_cast<uintptr_t>(ptr) & 15) == 0 && m % 4 == 0 && m > 0 && (heads == 1 || (g % 4 == 0 && g > 0));
    };
    EncodeTiledFn enc = encode_tiled_fn();
    if (enc != nullptr && ok16(a.k_ss, a.kss_m, a.kss_g, p->kv_heads) && ok16(a.v_ss, a.vss_m, a.vss_g, p->kv_heads)) {
      const cuuint64_t rows = p->kv_rows > 0              ? cuuint64_t(p->kv_rows)
                              : p->block_tables != nullptr ? (cuuint64_t(1) << 31)
                                                           : cuuint64_t(p->batch) * p->kv_padding;
      const cuuint64_t dims[3] = {4, cuuint64_t(p->kv_heads), rows};
      const cuuint32_t bx[3] = {4, cuuint32_t(hb), cuuint32_t(a.box_tok)};
      const cuuint32_t estr[3] = {1, 1, 1};
      const cuuint64_t ks[2] = {cuuint64_t(p->kv_heads == 1 ? 4 : a.kss_g) * 4, cuuint64_t(a.kss_m) * 4};
      const cuuint64_t vs[2] = {cuuint64_t(p->kv_heads == 1 ? 4 : a.vss_g) * 4, cuuint64_t(a.vss_m) * 4};
      const CUresult rk = enc(&a.tm_kss, CU_TENSOR_MAP_DATA_TYPE_INT32, 3, const_cast<int32_t*>(a.k_ss), dims, ks, bx, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                              CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
      const CUresult rv = enc(&a.tm_vss, CU_TENSOR_MAP_DATA_TYPE_INT32, 3, const_cast<int32_t*>(a.v_ss), dims, vs, bx, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                              CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
      if (rk == CUDA_SUCCESS && rv == CUDA_SUCCESS) a.ss_tma = 1;
    }
  }
  if (fp8 && a.copy_mode == 3 && a.ss_tma == 0 && hb >= 4) {
    // Compact scale/shift tensors: one word per (token, kv head), the heads of a token adjacent (a [rows, kv
    // heads] tensor, or the same expanded over the query heads with stride 0).  The words of the hb heads of a
    // run of tokens then come by one tiled copy of hb * 4 >= 16 bytes per token: no byte of a replica is read.
    auto compact = [&](const void* ptr, int64_t m, int64_t g) {
      return (reinterpret_cast<uintptr_t>(ptr) & 15) == 0 && g == 1 && m % 4 == 0 && m >= p->kv_heads;
    };
    EncodeTiledFn enc = encode_tiled_fn();
    if (enc != nullptr && compact(a.k_ss, a.kss_m, a.kss_g) && compact(a.v_ss, a.vss_m, a.vss_g)) {
      const cuuint64_t rows = p->kv_rows > 0              ? cuuint64_t(p->kv_rows)
                              : p->block_tables != nullptr ? (cuuint64_t(1) << 31)
                                                           : cuuint64_t(p->batch) * p->kv_padding;
      const cuuint64_t dims[3] = {cuuint64_t(p->kv_heads), rows, 1};
      const cuuint32_t bx[3] = {cuuint32_t(hb), cuuint32_t(a.box_tok), 1};
      const cuuint32_t estr[3] = {1, 1, 1};
      const cuuint64_t ks[2] = {cuuint64_t(a.kss_m) * 4, cuuint64_t(a.kss_m) * 4 * rows};
      const cuuint64_t vs[2] = {cuuint64_t(a.vss_m) * 4, cuuint64_t(a.vss_m) * 4 * rows};
      const CUresult rk = enc(&a.tm_kss, CU_TENSOR_MAP_DATA_TYPE_INT32, 3, const_cast<int32_t*>(a.k_ss), dims, ks, bx, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                              CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
      const CUresult rv = enc(&a.tm_vss, CU_TENSOR_MAP_DATA_TYPE_INT32, 3, const_cast<int32_t*>(a.v_ss), dims, vs, bx, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                              CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
      if (rk == CUDA_SUCCESS && rv == CUDA_SUCCESS) a.ss_tma = 2;
    }
  }

  if (fp8 && a.copy_mode != 3)
    return set_error(XFB200_E_UNSUPPORTED, "decode: fp8 cache needs tiled copies (16-byte aligned rows, pages that are multiples of 16 tokens)");

  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool bf16 = p->dtype == XFB200_BF16;
  const bool extras = p->bias != nullptr || (p->window_size > 0 && p->mq > 1);  // 16-bit cache: the consumer variant that knows them
#define XFB_DISPATCH(DD)                                                                                          \
  if (int4) {                                                                                                     \
    return bf16 ? launch_decode_mt<DD, kFmtInt4, true>(a, mt, head_blocks, st)                                    \
                : launch_decode_mt<DD, kFmtInt4, false>(a, mt, head_blocks, st);                                  \
  } else if (extras) {                                                                                            \
    return bf16 ? launch_decode_mt<DD, kFmtPlainX, true>(a, mt, head_blocks, st)                                  \
                : launch_decode_mt<DD, kFmtPlainX, false>(a, mt, head_blocks, st);                                \
  } else {                                                                                                        \
    return bf16 ? launch_decode_mt<DD, kFmtPlain, true>(a, mt, head_blocks, st)                                   \
                : launch_decode_mt<DD, kFmtPlain, false>(a, mt, head_blocks, st);                                 \
  }
  if (fp8)
    return bf16 ? launch_decode_mt<128, kFmtFp8, true>(a, mt, head_blocks, st) : launch_decode_mt<128, kFmtFp8, false>(a, mt, head_blocks, st);
  if (int4 && ng > 1) {
#define XFB_DISPATCH_NG(DD, GG) \
  return bf16 ? launch_decode_mt<DD, kFmtInt4, true, GG>(a, mt, head_blocks, st) : launch_decode_mt<DD, kFmtInt4, false, GG>(a, mt, head_blocks, st);
    if (p->head_dim == 128) {
      if (ng == 2) { XFB_DISPATCH_NG(128, 2) }
      if (ng == 4) { XFB_DISPATCH_NG(128, 4) }
      XFB_DISPATCH_NG(128, 8)
    }
    if (ng == 2) { XFB_DISPATCH_NG(64, 2) }
    XFB_DISPATCH_NG(64, 4)
#undef XFB_DISPATCH_NG
  }
  if (p->head_dim == 128) {
    XFB_DISPATCH(128)
  } else {
    XFB_DISPATCH(64)
  }
#undef XFB_DISPATCH
}

// ---------------------------------------------------------------------------
// Split-K decode for callers that cannot allocate device memory.
//
// The partial outputs of the key chunks go to a fixed array that is part of the
// library image instead of caller-provided scratch (the status word of the
// bounded waits is part of the image for every entry point).  It is a
// file-scope __device__ array: in host code its name is a host-side stand-in,
// not a device address, so the address the kernels receive is looked up once
// per device with cudaGetSymbolAddress while that device is current.
// ---------------------------------------------------------------------------
namespace xfb {

static __device__ __align__(256) unsigned char g_static_scratch[XFB200_DECODE_STATIC_SCRATCH_BYTES];

struct StaticScratchAddr {
  void* scratch = nullptr;
};

// Device address of the array on the current device; resolved on the first
// call per device (a symbol look-up, not an allocation) and cached.
static int static_scratch_addresses(StaticScratchAddr* out) {
  static StaticScratchAddr per_device[64];
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_fail("decode(static scratch): cudaGetDevice", e);
  if (dev < 0 || dev >= 64) return set_error(XFB200_E_UNSUPPORTED, "decode(static scratch): device index %d out of range", dev);
  StaticScratchAddr& slot = per_device[dev];
  if (slot.scratch == nullptr) {
    void* scratch = nullptr;
    e = cudaGetSymbolAddress(&scratch, g_static_scratch);
    if (e != cudaSuccess) return cuda_fail("decode(static scratch): cudaGetSymbolAddress(scratch)", e);
    slot.scratch = scratch;
  }
  *out = slot;
  return XFB200_OK;
}

}  // namespace xfb

extern "C" int xfb200_decode_forward_static_scratch(const xfb200_decode_params* p, void* stream) {
  using namespace xfb;
  if (p == nullptr) return set_error(XFB200_E_INVALID, "decode(static scratch): null params");
  if (p->batch < 0 || p->mq < 1 || p->kv_heads < 1 || p->q_per_kv < 1 || p->split_k < 1 || p->head_dim < 1)
    return set_error(XFB200_E_INVALID, "decode(static scratch): bad extents");
  const size_t need = xfb200_decode_scratch_bytes(p->batch, p->mq, p->kv_heads, p->q_per_kv, p->head_dim, p->split_k);
  if (need > size_t(XFB200_DECODE_STATIC_SCRATCH_BYTES))
    return set_error(XFB200_E_INVALID,
                     "decode(static scratch): this shape needs %zu bytes of split-K scratch, the built-in array holds %zu; "
                     "use fewer splits or xfb200_decode_forward with your own scratch",
                     need, size_t(XFB200_DECODE_STATIC_SCRATCH_BYTES));
  if (p->batch == 0) return XFB200_OK;
  StaticScratchAddr addr;
  int rc = static_scratch_addresses(&addr);
  if (rc != XFB200_OK) return rc;
  xfb200_decode_params q = *p;
  q.scratch = addr.scratch;
  return xfb200_decode_forward(&q, stream);
}
