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
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "internal.h"
#include "ptx.cuh"

namespace xfb {

constexpr int kDecConsumerWarps = 8;
constexpr int kDecThreads = (kDecConsumerWarps + 1) * 32;
constexpr int kDecChunkAlign = 128;  // chunk size granularity in tokens (= largest stage)

struct DecodeArgs {
  const void* q;
  const void* k;
  const void* v;
  void* out;
  float* lse;
  float* part_o;    // [batch, split, kv_heads, R, D]
  float* part_lse;  // [batch, split, kv_heads, R]
  int32_t* status;  // device status word (timed-out waits)
  const int32_t* seqlen_k;
  const int32_t* block_tables;
  int32_t batch, mq, kv_heads, q_per_kv;
  int32_t kv_padding, page_size, bt_stride;
  int32_t split_k, chunk_tokens;
  int32_t hb;          // kv heads per CTA (1, 2, 4 or 8)
  int32_t rows;        // R = mq * q_per_kv
  int32_t row_blocks;  // ceil(R / (16*MT))
  int32_t copy_mode;   // 0: one bulk copy per token stripe of hb heads; 1: per (token, head); 2: word copies (no TMA)
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
template <int D, bool kInt4>
struct DecStage {
  // plain: one row per token = hb heads * D elements (+16 B pad against bank conflicts)
  // int4 : one row per token = hb heads * (1 + D/8) words, unpadded
  __host__ __device__ static int row_bytes(int hb) { return kInt4 ? hb * (1 + D / 8) * 4 : hb * D * 2 + 16; }
  // sub-tiles of 16 tokens each warp takes from one stage: the packed cache is 4x
  // denser, so its stages hold 4x the tokens to keep the per-stage overhead
  // (barrier round trip, page-table look-ups of the producer) off the critical path
  static constexpr int kSubTiles = kInt4 ? 4 : 1;
  __host__ __device__ static int tokens(int hb) { return 16 * kSubTiles * (kDecConsumerWarps / hb); }
  __host__ __device__ static int kv_bytes(int hb) {  // K or V part of a stage, rounded to 128 B
    return (row_bytes(hb) * tokens(hb) + 127) & ~127;
  }
};

constexpr int kDecMaxStages = 12;
constexpr int kDecRingBudget = 212 * 1024;  // bytes of cache in flight per SM

template <int D, int MT, bool kInt4, bool kBf16>
__global__ void __launch_bounds__(kDecThreads, 1) decode_splitk_kernel(const __grid_constant__ DecodeArgs a) {
  using Stage = DecStage<D, kInt4>;
  using T = typename Half2Type<kBf16>::T;
  constexpr int W = 1 + D / 8;  // int4 words per row (one quantisation group)
  constexpr int KS = D / 16;    // k-steps of the QK^T product
  constexpr int NT = D / 8;     // n-tiles of the PV product

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
  constexpr int kSps = DecStage<D, kInt4>::kSubTiles;
  const int TOK = 16 * wph * kSps;

  const int kv_len = a.seqlen_k != nullptr ? min(max(a.seqlen_k[b], 0), a.kv_padding) : a.kv_padding;
  const int chunk_lo = split * a.chunk_tokens;
  const int chunk_hi = min(chunk_lo + a.chunk_tokens, kv_len);
  if (chunk_lo >= chunk_hi) {
    // nothing for this CTA (uniform: the whole CTA leaves).  Without a merge
    // pass the rows of an empty sequence still have to be defined: out = 0,
    // lse = -inf.
    if (a.split_k == 1 && split == 0) {
      const int nrows = min(16 * MT, a.rows - rblk * 16 * MT);
      for (int i = threadIdx.x; i < hb * nrows * D; i += blockDim.x) {
        const int d = i % D, rr = (i / D) % nrows, hh = i / (D * nrows);
        const int row = rblk * 16 * MT + rr, head = hblk * hb + hh;
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

  const int kv_bytes = Stage::kv_bytes(hb);
  const int row_bytes = Stage::row_bytes(hb);
  uint8_t* stage_base = smem_raw;                                  // kDecStages * 2 * kv_bytes
  // Q is staged once in the region of the LAST stages; the producer does not
  // fill those before every consumer warp has taken its Q fragments
  uint8_t* q_smem = smem_raw + a.q_first_stage * 2 * kv_bytes;     // 8 warps * 16*MT rows * D*2 B
  constexpr int kQRowBytes = D * 2;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kDecStages; ++i) {
      mbar_init(&full_bar[i], 1);
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
    constexpr int kElem = kInt4 ? 4 : 2;
    constexpr int kHeadBytes = kInt4 ? W * 4 : D * 2;
    const int head0 = hblk * hb;
    for (int tile = 0; tile < n_tiles; ++tile) {
      const int st = tile % kDecStages;
      if (tile >= kDecStages) {
        if (!mbar_wait(&empty_bar[st], ((tile / kDecStages) - 1) & 1)) {
          if (lane == 0) atomicExch(a.status, 1);
          return;
        }
      } else if (tile == a.q_first_stage) {
        if (!mbar_wait(&q_done_bar, 0)) {
          if (lane == 0) atomicExch(a.status, 3);
          return;
        }
      }
      const int t0 = chunk_lo + tile * TOK;
      const int nvalid = min(TOK, chunk_hi - t0);
      uint8_t* ks = stage_base + st * 2 * kv_bytes;
      uint8_t* vs = ks + kv_bytes;
      if (a.copy_mode == 2) {
        // no TMA: 32-bit loads (rows that are not 16-B aligned)
        const int words_per_head = kHeadBytes / 4;
        const int total = nvalid * hb * words_per_head;
        for (int i = lane; i < total; i += 32) {
          const int tok = i / (hb * words_per_head);
          const int rem = i % (hb * words_per_head);
          const int hh = rem / words_per_head, wd = rem % words_per_head;
          const int t = t0 + tok;
          const int64_t row = a.block_tables ? int64_t(a.block_tables[int64_t(b) * a.bt_stride + t / a.page_size]) * a.page_size + t % a.page_size
                                             : int64_t(b) * a.kv_padding + t;
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
        const int64_t row = a.block_tables ? int64_t(a.block_tables[int64_t(b) * a.bt_stride + t / a.page_size]) * a.page_size + t % a.page_size
                                           : int64_t(b) * a.kv_padding + t;
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
  const int r = lane >> 2, c = lane & 3;
  const int row0 = rblk * 16 * MT;  // first query row (of this kv head) handled here
  const int R = a.rows;

  // ---- stage Q (this warp's head) in shared memory, zero rows beyond R
  {
    uint8_t* qs = q_smem + warp * (16 * MT) * kQRowBytes;
    const T* qg = reinterpret_cast<const T*>(a.q);
    for (int i = lane; i < 16 * MT * (D / 8); i += 32) {
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
  const uint8_t* qs = q_smem + warp * (16 * MT) * kQRowBytes;

  // A fragments of Q.  Plain cache: natural k order.  int4 cache: k-slot
  // (ks, 2c+e [+8]) of thread c <-> d = 8*(4*(ks/2)... see kperm() below.
  uint32_t qf[MT][KS][4];
  float qsum[MT][2];  // int4: sum over d of q[row][d] (rows r, r+8)
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) qsum[mt][0] = qsum[mt][1] = 0.f;
  if constexpr (!kInt4) {
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
        const int rr = mt * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
        const int cc = ks * 16 + (lane >> 4) * 8;
        ldmatrix_x4(qf[mt][ks], smem_u32(qs + rr * kQRowBytes + cc * 2));
      }
  } else {
    // Thread c unpacks words c, c+4, c+8, ... of a K row; word i (= 4*j + c)
    // feeds k-steps 2j and 2j+1: k-step 2j holds elements (0,4 | 1,5), k-step
    // 2j+1 holds (2,6 | 3,7) of that word.  Q must use the same order.
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
        const int word = 4 * (ks >> 1) + c;
        const int e0 = (ks & 1) * 2;
        const T* q0 = reinterpret_cast<const T*>(qs + (mt * 16 + r) * kQRowBytes) + word * 8;
        const T* q1 = reinterpret_cast<const T*>(qs + (mt * 16 + r + 8) * kQRowBytes) + word * 8;
        auto pk = [](const T* p, int i0, int i1) {
          uint32_t lo = *reinterpret_cast<const unsigned short*>(p + i0);
          uint32_t hi = *reinterpret_cast<const unsigned short*>(p + i1);
          return lo | (hi << 16);
        };
        qf[mt][ks][0] = pk(q0, e0, e0 + 4);
        qf[mt][ks][1] = pk(q1, e0, e0 + 4);
        qf[mt][ks][2] = pk(q0, e0 + 1, e0 + 5);
        qf[mt][ks][3] = pk(q1, e0 + 1, e0 + 5);
      }
    // row sums over all d (every thread of a quad needs them for its rows)
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      const T* q0 = reinterpret_cast<const T*>(qs + (mt * 16 + r) * kQRowBytes);
      const T* q1 = reinterpret_cast<const T*>(qs + (mt * 16 + r + 8) * kQRowBytes);
      float s0 = 0.f, s1 = 0.f;
      for (int d = c; d < D; d += 4) {
        s0 += float(q0[d]);
        s1 += float(q1[d]);
      }
      s0 += __shfl_xor_sync(0xffffffffu, s0, 1);
      s0 += __shfl_xor_sync(0xffffffffu, s0, 2);
      s1 += __shfl_xor_sync(0xffffffffu, s1, 1);
      s1 += __shfl_xor_sync(0xffffffffu, s1, 2);
      qsum[mt][0] = s0;
      qsum[mt][1] = s1;
    }
  }

  // Q now lives in registers: release the staging area to the producer
  __syncwarp();
  if (lane == 0) mbar_arrive(&q_done_bar);

  // per-row visibility limit: token t visible iff t < lim
  int lim[MT][2];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int hlf = 0; hlf < 2; ++hlf) {
      const int row = row0 + mt * 16 + r + hlf * 8;
      int l = chunk_hi;
      if (a.causal && row < R) l = min(l, kv_len - a.mq + row / a.q_per_kv + 1);
      lim[mt][hlf] = l;
    }

  float acc[MT][NT][4];
  float m_run[MT][2], l_run[MT][2], corr[MT][2];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
    for (int j = 0; j < NT; ++j) acc[mt][j][0] = acc[mt][j][1] = acc[mt][j][2] = acc[mt][j][3] = 0.f;
    m_run[mt][0] = m_run[mt][1] = -INFINITY;
    l_run[mt][0] = l_run[mt][1] = 0.f;
    corr[mt][0] = corr[mt][1] = 0.f;
  }
  // A nibble n dropped into the top four mantissa bits of 16.0 reads as 16 + n
  // exactly (bf16: mantissa bits [3,7); f16: bits [6,10)).  The offset is of the
  // size of the values themselves, so removing it later costs no precision.
  constexpr uint32_t kMagic = kBf16 ? 0x41804180u : 0x4C004C00u;
  constexpr uint32_t kNibMask = kBf16 ? 0x00780078u : 0x03C003C0u;
  constexpr int kNibPos = kBf16 ? 3 : 6;
  constexpr float kMagicF = 16.f;
  // nibble pair (e, e+4) of a packed word, e = 0..3, as two 16-bit floats 16+n
  auto unpack_pair = [](uint32_t w, int e) -> uint32_t {
    const int sh = 4 * e - kNibPos;  // compile-time after unrolling
    const uint32_t t = sh >= 0 ? (w >> sh) : (w << (-sh));
    return (t & kNibMask) | kMagic;
  };

  for (int tile = 0; tile < n_tiles; ++tile) {
    const int st = tile % kDecStages;
    if (!mbar_wait(&full_bar[st], (tile / kDecStages) & 1)) {
      if (lane == 0) atomicExch(a.status, 2);
      break;
    }
    for (int sp = 0; sp < kSps; ++sp) {
    const int usub = sub + wph * sp;                      // this warp's sub-tile of the stage
    const int t_sub = chunk_lo + tile * TOK + usub * 16;  // its first token
    if (t_sub < chunk_hi) {
      const uint8_t* ks_ = stage_base + st * 2 * kv_bytes;
      const uint8_t* vs_ = ks_ + kv_bytes;
      const bool ragged = t_sub + 16 > chunk_hi;

      // ------------------------------------------------ S = Q K^T (16*MT x 16)
      float s[MT][2][4];
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int j = 0; j < 2; ++j) s[mt][j][0] = s[mt][j][1] = s[mt][j][2] = s[mt][j][3] = 0.f;

      if constexpr (!kInt4) {
        const int tok = usub * 16 + (lane & 7) + (lane >> 4) * 8;
        const uint32_t kaddr = smem_u32(ks_ + tok * row_bytes + hw * D * 2 + ((lane >> 3) & 1) * 16);
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
          uint32_t kf[4];
          ldmatrix_x4(kf, kaddr + ks * 32);
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            mma_16816<kBf16>(s[mt][0], qf[mt][ks], kf[0], kf[1]);
            mma_16816<kBf16>(s[mt][1], qf[mt][ks], kf[2], kf[3]);
          }
        }
      } else {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const uint32_t* krow = reinterpret_cast<const uint32_t*>(ks_ + (usub * 16 + j * 8 + r) * row_bytes + hw * W * 4) + 1;
#pragma unroll
          for (int i = 0; i < KS / 2; ++i) {
            const uint32_t w = krow[4 * i + c];
            const uint32_t b00 = unpack_pair(w, 0);  // elements 0,4
            const uint32_t b01 = unpack_pair(w, 1);  // elements 1,5
            const uint32_t b10 = unpack_pair(w, 2);  // elements 2,6
            const uint32_t b11 = unpack_pair(w, 3);  // elements 3,7
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
              mma_16816<kBf16>(s[mt][j], qf[mt][2 * i], b00, b01);
              mma_16816<kBf16>(s[mt][j], qf[mt][2 * i + 1], b10, b11);
            }
          }
        }
      }

      // -------------------------------- scale, mask, online softmax (log2 domain)
      float vsc[2][2] = {{1.f, 1.f}, {1.f, 1.f}}, vsh[2][2] = {{0.f, 0.f}, {0.f, 0.f}};  // V scale/shift of tokens (j, 2c+e)
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int tl = usub * 16 + j * 8 + 2 * c + e;
          const int t = t_sub + j * 8 + 2 * c + e;
          if constexpr (kInt4) {
            const uint32_t kw = *reinterpret_cast<const uint32_t*>(ks_ + tl * row_bytes + hw * W * 4);
            const uint32_t vw = *reinterpret_cast<const uint32_t*>(vs_ + tl * row_bytes + hw * W * 4);
            const float ksc = half_bits_to_float(kw & 0xFFFFu), ksh = half_bits_to_float(kw >> 16);
            const bool tv = t < chunk_hi;
            vsc[j][e] = tv ? half_bits_to_float(vw & 0xFFFFu) : 0.f;
            vsh[j][e] = tv ? half_bits_to_float(vw >> 16) : 0.f;
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
              s[mt][j][e] = ksc * s[mt][j][e] + (ksh - kMagicF * ksc) * qsum[mt][0];
              s[mt][j][2 + e] = ksc * s[mt][j][2 + e] + (ksh - kMagicF * ksc) * qsum[mt][1];
            }
          }
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            s[mt][j][e] = t < lim[mt][0] ? s[mt][j][e] * a.scale_log2 : -INFINITY;
            s[mt][j][2 + e] = t < lim[mt][1] ? s[mt][j][2 + e] * a.scale_log2 : -INFINITY;
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
          float psum = 0.f, csum = 0.f;
          float p[2][2];
#pragma unroll
          for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const float pv = fast_exp2(s[mt][j][2 * hlf + e] - m_use);
              psum += pv;
              if constexpr (kInt4) {
                // fold the V scale into P; the shift (and the 2^k offset of the
                // unpacked nibbles) becomes a per-row correction that uses the
                // ROUNDED weight so that the offset cancels exactly
                const float pw = pv * vsc[j][e];
                const uint32_t one = pack2<kBf16>(pw, 0.f);
                const float pw_r = unpack2<kBf16>(one).x;
                csum += pv * vsh[j][e] - kMagicF * pw_r;
                p[j][e] = pw;
              } else {
                p[j][e] = pv;
              }
            }
          l_run[mt][hlf] = l_run[mt][hlf] * alpha[hlf] + psum;
          corr[mt][hlf] = corr[mt][hlf] * alpha[hlf] + csum;
          pa[mt][hlf] = pack2<kBf16>(p[0][0], p[0][1]);      // k = 2c, 2c+1   (rows r / r+8)
          pa[mt][2 + hlf] = pack2<kBf16>(p[1][0], p[1][1]);  // k = 2c+8, 2c+9
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
      if constexpr (!kInt4) {
        if (ragged) {
          // rows of tokens past the end were not copied: zero them so that
          // 0 * garbage cannot produce NaN
          for (int i = lane; i < 16 * (D / 8); i += 32) {
            const int tt = i / (D / 8), ch = i % (D / 8);
            if (t_sub + tt >= chunk_hi)
              *reinterpret_cast<uint4*>(const_cast<uint8_t*>(vs_) + (usub * 16 + tt) * row_bytes + hw * D * 2 + ch * 16) = make_uint4(0, 0, 0, 0);
          }
          __syncwarp();
        }
        const int tok = usub * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
        const uint32_t vaddr = smem_u32(vs_ + tok * row_bytes + hw * D * 2 + (lane >> 4) * 16);
#pragma unroll
        for (int j = 0; j < NT; j += 2) {
          uint32_t vf[4];
          ldmatrix_x4_trans(vf, vaddr + j * 16);
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            mma_16816<kBf16>(acc[mt][j], pa[mt], vf[0], vf[1]);
            mma_16816<kBf16>(acc[mt][j + 1], pa[mt], vf[2], vf[3]);
          }
        }
      } else {
        // Thread (r, c) unpacks words 2r', 2r'+1 ... of tokens 2c, 2c+1, 2c+8,
        // 2c+9: virtual output column (n-tile j, col r) <-> d = (D/8)*r + j.
        constexpr int WPT = D / 64;  // words per thread and token (2 for D = 128)
#pragma unroll
        for (int wi = 0; wi < WPT; ++wi) {
          uint32_t x[4][4];  // [token 2c,2c+1,2c+8,2c+9][element pair i,(i+4)]
#pragma unroll
          for (int tk = 0; tk < 4; ++tk) {
            const int tl = usub * 16 + 2 * c + (tk & 1) + (tk >> 1) * 8;
            const uint32_t w = *(reinterpret_cast<const uint32_t*>(vs_ + tl * row_bytes + hw * W * 4) + 1 + WPT * r + wi);
            x[tk][0] = unpack_pair(w, 0);
            x[tk][1] = unpack_pair(w, 1);
            x[tk][2] = unpack_pair(w, 2);
            x[tk][3] = unpack_pair(w, 3);
          }
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            // element i (low halves) and element i+4 (high halves) of this word
            const uint32_t b0_lo = __byte_perm(x[0][i], x[1][i], 0x5410);
            const uint32_t b1_lo = __byte_perm(x[2][i], x[3][i], 0x5410);
            const uint32_t b0_hi = __byte_perm(x[0][i], x[1][i], 0x7632);
            const uint32_t b1_hi = __byte_perm(x[2][i], x[3][i], 0x7632);
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
              mma_16816<kBf16>(acc[mt][wi * 8 + i], pa[mt], b0_lo, b1_lo);
              mma_16816<kBf16>(acc[mt][wi * 8 + i + 4], pa[mt], b0_hi, b1_hi);
            }
          }
        }
      }
    }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty_bar[st]);
  }

  // ------------------------------------------------------------- epilogue
  // full row sums (each thread of a quad saw 4 of the 16 tokens of a tile)
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int hlf = 0; hlf < 2; ++hlf) {
      float l = l_run[mt][hlf], cs = corr[mt][hlf];
      l += __shfl_xor_sync(0xffffffffu, l, 1);
      l += __shfl_xor_sync(0xffffffffu, l, 2);
      cs += __shfl_xor_sync(0xffffffffu, cs, 1);
      cs += __shfl_xor_sync(0xffffffffu, cs, 2);
      l_run[mt][hlf] = l;
      corr[mt][hlf] = cs;
    }

  // Combine the warps that share a kv head through shared memory (the ring is
  // no longer in use once every consumer warp got here).
  asm volatile("bar.sync 1, %0;" ::"n"(kDecConsumerWarps * 32) : "memory");
  float* cmb = reinterpret_cast<float*>(smem_raw);  // [warp][16*MT][D + 2]  (acc, m, l)
  constexpr int kCmbRow = D + 2;
  {
    float* mine = cmb + size_t(warp) * (16 * MT) * kCmbRow;
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
      for (int j = 0; j < NT; ++j) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int rr = mt * 16 + r + (e >> 1) * 8;
          const int col = 2 * c + (e & 1);
          const int d = kInt4 ? (D / 8) * col + j : j * 8 + col;
          float val = acc[mt][j][e];
          if constexpr (kInt4) val += corr[mt][e >> 1];
          mine[rr * kCmbRow + d] = val;
        }
      }
      if (c == 0) {
        mine[(mt * 16 + r) * kCmbRow + D] = m_run[mt][0];
        mine[(mt * 16 + r) * kCmbRow + D + 1] = l_run[mt][0];
        mine[(mt * 16 + r + 8) * kCmbRow + D] = m_run[mt][1];
        mine[(mt * 16 + r + 8) * kCmbRow + D + 1] = l_run[mt][1];
      }
    }
  }
  asm volatile("bar.sync 1, %0;" ::"n"(kDecConsumerWarps * 32) : "memory");

  // warps of head hw share the rows: warp `sub` finalises rows sub, sub+wph, ...
  const bool direct = a.split_k == 1;
  for (int rr = sub; rr < 16 * MT; rr += wph) {
    const int row = row0 + rr;
    if (row >= R) break;
    float mx = -INFINITY;
    for (int w2 = 0; w2 < wph; ++w2) mx = fmaxf(mx, cmb[size_t(w2 * hb + hw) * (16 * MT) * kCmbRow + rr * kCmbRow + D]);
    const float m_use = mx == -INFINITY ? 0.f : mx;
    float den = 0.f;
    float o[D / 32];
#pragma unroll
    for (int i = 0; i < D / 32; ++i) o[i] = 0.f;
    for (int w2 = 0; w2 < wph; ++w2) {
      const float* src = cmb + size_t(w2 * hb + hw) * (16 * MT) * kCmbRow + rr * kCmbRow;
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
  const int kv_len = a.seqlen_k != nullptr ? min(max(a.seqlen_k[b], 0), a.kv_padding) : a.kv_padding;
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
static int32_t* decode_status_word() {
  // one status word per device, allocated on first use and kept
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

// Set only while xfb200_decode_forward_static_scratch runs on this thread: the
// status word then lives in the library's own device memory as well.
static thread_local int32_t* t_status_override = nullptr;

int decode_chunk_tokens(int kv_bound, int split_k) {
  int c = (kv_bound + split_k - 1) / split_k;
  c = (c + kDecChunkAlign - 1) / kDecChunkAlign * kDecChunkAlign;
  return c < kDecChunkAlign ? kDecChunkAlign : c;
}

template <int D, int MT, bool kInt4, bool kBf16>
static int launch_decode_t(const DecodeArgs& a_in, int head_blocks, cudaStream_t stream) {
  using Stage = DecStage<D, kInt4>;
  const size_t stage_bytes = 2 * size_t(Stage::kv_bytes(a_in.hb));
  const size_t qbytes = size_t(kDecConsumerWarps) * 16 * MT * (D * 2);
  const size_t cmb = size_t(kDecConsumerWarps) * 16 * MT * (D + 2) * 4;
  int stages = int(kDecRingBudget / stage_bytes);
  stages = stages > kDecMaxStages ? kDecMaxStages : stages;
  const int q_stages = int((qbytes + stage_bytes - 1) / stage_bytes);
  if (stages < 2 || q_stages > stages) return set_error(XFB200_E_UNSUPPORTED, "decode: shared-memory ring too small for this shape");
  DecodeArgs a = a_in;
  a.stages = stages;
  a.q_first_stage = stages - q_stages;
  const size_t ring = stages * stage_bytes;
  const size_t smem = ring > cmb ? ring : cmb;
  auto kern = decode_splitk_kernel<D, MT, kInt4, kBf16>;
  // 227 KB per CTA includes the static part (the mbarriers)
  if (smem + 1024 > 227 * 1024) return set_error(XFB200_E_UNSUPPORTED, "decode: shared memory %zu B exceeds 227 KB", smem);
  static size_t configured = 0;  // per instantiation: largest size opted into so far
  if (smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    if (e != cudaSuccess) return cuda_fail("decode: cudaFuncSetAttribute", e);
    configured = smem;
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

template <int D, bool kInt4, bool kBf16>
static int launch_decode_mt(const DecodeArgs& a, int mt, int head_blocks, cudaStream_t stream) {
  if (mt == 1) return launch_decode_t<D, 1, kInt4, kBf16>(a, head_blocks, stream);
  return launch_decode_t<D, 2, kInt4, kBf16>(a, head_blocks, stream);
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
  if (int4 && p->num_quant_groups != 1)
    return set_error(XFB200_E_UNSUPPORTED, "decode: int4 cache with %d quantisation groups per row (only 1)", p->num_quant_groups);
  if (!int4 && p->kv_format != XFB200_KV_PLAIN) return set_error(XFB200_E_INVALID, "decode: bad kv_format %d", p->kv_format);
  if (p->split_k < 1 || p->split_k > 1024) return set_error(XFB200_E_INVALID, "decode: split_k %d out of range", p->split_k);
  if (p->kv_padding < 1) return set_error(XFB200_E_INVALID, "decode: kv_padding must be positive");
  if (p->block_tables != nullptr && (p->page_size < 1 || p->block_table_stride < 1))
    return set_error(XFB200_E_INVALID, "decode: paged cache needs page_size and block_table_stride");
  if (p->mask_type != XFB200_MASK_NONE && p->mask_type != XFB200_MASK_CAUSAL_BOTTOM_RIGHT)
    return set_error(XFB200_E_UNSUPPORTED, "decode: mask_type %d", p->mask_type);
  const int R = p->mq * p->q_per_kv;
  const int mt = R <= 16 ? 1 : 2;
  const int row_blocks = (R + 16 * mt - 1) / (16 * mt);
  if (p->split_k > 1 && p->scratch == nullptr) return set_error(XFB200_E_INVALID, "decode: split_k > 1 needs scratch");
  if (p->split_k > 1 && (reinterpret_cast<uintptr_t>(p->scratch) & 255)) return set_error(XFB200_E_INVALID, "decode: scratch must be 256-B aligned");

  DecodeArgs a{};
  a.q = p->q, a.k = p->k, a.v = p->v, a.out = p->out, a.lse = p->lse;
  a.seqlen_k = p->seqlen_k, a.block_tables = p->block_tables;
  a.batch = p->batch, a.mq = p->mq, a.kv_heads = p->kv_heads, a.q_per_kv = p->q_per_kv;
  a.kv_padding = p->kv_padding, a.page_size = p->page_size, a.bt_stride = p->block_table_stride;
  a.split_k = p->split_k;
  a.chunk_tokens = decode_chunk_tokens(p->kv_padding, p->split_k);
  a.rows = R, a.row_blocks = row_blocks;
  a.q_sm = p->q_stride_m, a.q_sg = p->q_stride_g, a.q_sh = p->q_stride_h;
  a.k_sm = p->k_stride_m, a.k_sg = p->k_stride_g, a.v_sm = p->v_stride_m, a.v_sg = p->v_stride_g;
  if (p->kv_heads == 1) a.k_sg = a.v_sg = 0;  // the stride of an extent-1 axis is meaningless
  a.o_sm = p->o_stride_m, a.o_sg = p->o_stride_g, a.o_sh = p->o_stride_h;
  a.lse_sg = p->lse_stride_g, a.lse_sh = p->lse_stride_h;
  a.causal = p->mask_type == XFB200_MASK_CAUSAL_BOTTOM_RIGHT;
  a.out_dtype = p->out_dtype;
  a.scale_log2 = p->scale * 1.4426950408889634f;
  if (p->split_k > 1) {
    const size_t rows = size_t(p->batch) * p->split_k * p->kv_heads * R;
    a.part_o = reinterpret_cast<float*>(p->scratch);
    a.part_lse = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(p->scratch) + ((rows * p->head_dim * 4 + 255) & ~size_t(255)));
  }
  a.status = t_status_override != nullptr ? t_status_override : decode_status_word();
  if (a.status == nullptr) return set_error(XFB200_E_CUDA, "decode: cannot allocate the device status word");

  // kv heads per CTA: the largest of 8, 4, 2, 1 that divides kv_heads
  int hb = 8;
  while (p->kv_heads % hb) hb >>= 1;
  a.hb = hb;
  const int head_blocks = p->kv_heads / hb;

  // how the producer may copy: whole stripes by TMA when alignment allows
  const int elem = int4 ? 4 : 2;
  const int head_elems = int4 ? (1 + p->head_dim / 8) : p->head_dim;
  const bool heads_contig = hb == 1 || (a.k_sg == head_elems && a.v_sg == head_elems);
  auto al16 = [&](int64_t elems) { return (elems * elem) % 16 == 0; };
  const bool base_al = (reinterpret_cast<uintptr_t>(p->k) % 16 == 0) && (reinterpret_cast<uintptr_t>(p->v) % 16 == 0);
  a.copy_group = 1;
  if (!base_al) {
    a.copy_mode = 2;
  } else if (heads_contig && al16(p->k_stride_m) && al16(p->v_stride_m) && al16(int64_t(hb) * head_elems) &&
             al16(a.k_sg * hb) && al16(a.v_sg * hb)) {
    a.copy_mode = 0;
  } else if (al16(p->k_stride_m) && al16(p->v_stride_m) && al16(a.k_sg) && al16(a.v_sg) && al16(head_elems)) {
    a.copy_mode = 1;
  } else if (int4 && heads_contig && head_blocks == 1 && p->k_stride_m == int64_t(hb) * head_elems &&
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

  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool bf16 = p->dtype == XFB200_BF16;
#define XFB_DISPATCH(DD)                                                                           \
  if (int4) {                                                                                      \
    return bf16 ? launch_decode_mt<DD, true, true>(a, mt, head_blocks, st)                         \
                : launch_decode_mt<DD, true, false>(a, mt, head_blocks, st);                       \
  } else {                                                                                         \
    return bf16 ? launch_decode_mt<DD, false, true>(a, mt, head_blocks, st)                        \
                : launch_decode_mt<DD, false, false>(a, mt, head_blocks, st);                      \
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
// library image instead of caller-provided scratch, and the status word of the
// bounded waits sits next to it.  Both are file-scope __device__ arrays: in
// host code their names are host-side stand-ins, not device addresses, so the
// addresses the kernels receive are looked up once per device with
// cudaGetSymbolAddress while that device is current.
// ---------------------------------------------------------------------------
namespace xfb {

static __device__ __align__(256) unsigned char g_static_scratch[XFB200_DECODE_STATIC_SCRATCH_BYTES];
static __device__ __align__(256) int32_t g_static_status[64];

struct StaticScratchAddr {
  void* scratch = nullptr;
  int32_t* status = nullptr;
};

// Device addresses of the two arrays on the current device; resolved on the
// first call per device (a symbol look-up, not an allocation) and cached.
static int static_scratch_addresses(StaticScratchAddr* out) {
  static StaticScratchAddr per_device[64];
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_fail("decode(static scratch): cudaGetDevice", e);
  if (dev < 0 || dev >= 64) return set_error(XFB200_E_UNSUPPORTED, "decode(static scratch): device index %d out of range", dev);
  StaticScratchAddr& slot = per_device[dev];
  if (slot.scratch == nullptr) {
    void* scratch = nullptr;
    void* status = nullptr;
    e = cudaGetSymbolAddress(&scratch, g_static_scratch);
    if (e != cudaSuccess) return cuda_fail("decode(static scratch): cudaGetSymbolAddress(scratch)", e);
    e = cudaGetSymbolAddress(&status, g_static_status);
    if (e != cudaSuccess) return cuda_fail("decode(static scratch): cudaGetSymbolAddress(status)", e);
    slot.status = static_cast<int32_t*>(status);
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
  t_status_override = addr.status;
  rc = xfb200_decode_forward(&q, stream);
  t_status_override = nullptr;
  return rc;
}
