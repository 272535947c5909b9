// Attention forward (prefill) on tcgen05, 256 query rows per CTA, 64-key steps.
//
// Two 128-row query tiles share every K/V stage (64 keys) that TMA brings in.
// Each query tile has its own softmax warpgroup, its own MMA-issuing warp and
// TWO score buffers in tensor memory, and works in steps of 64 keys:
//
//   MMA warp t   : ... PV(t,n-2), QK(t,n), [wait P(n-1)], PV(t,n-1), QK(t,n+1) ...
//   softmax WG t : ... S(n) -> P(n) in place, S(n+1) -> P(n+1) ...
//
// QK^T runs two steps ahead of PV, so the softmax of step n+1 finds its scores
// ready the moment it has handed over P(n).  A 128x64x16 MMA takes 48 clocks
// instead of 32 (operand fetch from shared memory bounds it), so the tensor
// pipe needs 1280 clocks per step for both tiles against 1024 with 128 keys.
//
// Status: an alternative schedule, selected with xfb200_debug_set_prefill_path(5)
// and covered by the same tests; the default stays the 128-key-step kernel.
// Measured on the causal 4096 x 128 headline case both run at the same speed
// (~2000 clocks per 64-key step here).  Per step and tile the softmax warps
// spend ~370 clocks on load + max, 650 on the exponentials when the two tiles
// are half a step apart (1000-1100 when their 2^x phases coincide: the units
// are shared) and 55 on the hand-over; each MMA-issuing lane spends ~640 on
// its own MMAs, as much again blocked behind the other tile's, and ~700 in
// three barrier waits.  With the softmax replaced by a constant the step still
// takes ~1700 clocks, while the same MMA sequence alone sustains 1260-1330:
// the issuing lanes, not a pipe, set the pace.  Neither strict alternation of
// the two lanes (with the token handed over early) nor deeper K/V rings moved it.
//
//   warps 0-3   softmax of query tile 0   (thread <-> row <-> TMEM lane)
//   warps 4-7   softmax of query tile 1
//   warp 8, 9   MMA issuer of tile 0, 1 (one lane issues); the two pass a token so
//               that their blocks (PV of step n-2, QK^T of step n) alternate on the
//               tensor pipe, which keeps the two softmax warpgroups half a step
//               apart: they share the 2^x units of their schedulers
//   warp 10     TMA producer of Q (both tiles, once) and of the K stages
//   warp 11     TMA producer of the V stages (V is used two steps after K: separate
//               rings and producers, so that neither load waits for the other's stage)
// The third warpgroup hands most of its registers to the softmax warpgroups
// with setmaxnreg (which only moves registers inside what the CTA was launched
// with; a request beyond that never returns, see kRegs* below).
//
// Tensor memory (all 512 columns), per tile t at column 256 t:
//   S[0] 64 | S[1] 64 | O 128   (fp32).  P(n) overwrites the first 32 columns
// of S[n & 1] as packed bf16/f16 pairs and feeds PV straight from tensor memory.
// tcgen05 operations issued by one thread complete in order: QK(n+2), issued
// after PV(n), may overwrite S[n & 1] without a further hand-shake.  O is
// rescaled by the softmax threads only after PV(n-1) has completed (pv_done)
// and before P(n) is handed over, so no product is in flight on it.
//
// Softmax arithmetic as in the 128-key kernel: packed f32x2 FMA/ADD, exp2 with
// the scale folded in, lazy running maximum (raised only when it grows by more
// than 2^8).  Masks, GQA indexing, NaN hygiene and bounded waits likewise.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "internal.h"
#include "prefill_sm100.h"
#include "ptx.cuh"

namespace xfb {
namespace s64 {

constexpr int kBM = 128;      // rows per query tile
constexpr int kTiles = 2;     // query tiles per CTA
constexpr int kBN = 128;      // alignment of the first key a CTA touches
constexpr int kStep = 64;     // keys per QK^T / softmax / PV step = keys per K (or V) stage in shared memory
// A stage is refilled kStages steps ahead of its use, and a TMA load takes a few
// thousand clocks to land while a step should take ~1300: four stages each.
#ifndef XFB_KSTAGES
#define XFB_KSTAGES 4
#endif
#ifndef XFB_VSTAGES
#define XFB_VSTAGES 4
#endif
constexpr int kStagesK = XFB_KSTAGES, kStagesV = XFB_VSTAGES;
constexpr int kSoftmaxWarps = 8;  // 4 per query tile
constexpr int kMmaWarp0 = 8, kTmaWarp = 10;  // warps 8 and 9 issue the MMAs of query tile 0 and 1
constexpr int kThreads = 384;
// registers per thread after setmaxnreg: 8 softmax warps grow, 4 other warps shrink;
// the sum must fit what 384 threads were launched with (168 each)
constexpr int kRegsLaunch = 168, kRegsSoftmax = 208, kRegsAux = 88;
static_assert(8 * kRegsSoftmax + 4 * kRegsAux <= 12 * kRegsLaunch, "setmaxnreg would ask for more registers than the CTA owns");
constexpr float kRescaleThreshold = 8.0f;
constexpr uint32_t kHalfBytes = 128 * 128;  // one 64-column block of a 128-row Q tile
constexpr uint32_t kKvHalfBytes = kStep * 128;  // one 64-column block of a 64-key K or V stage

struct __align__(8) Barriers {
  uint64_t q_full;
  uint64_t k_full[kStagesK], v_full[kStagesV], k_empty[kStagesK], v_empty[kStagesV];
  uint64_t s_full[kTiles][2], p_full[kTiles][2], pv_done[kTiles];
  uint64_t turn[kTiles];  // token of the tensor pipe: the two MMA warps issue their blocks alternately
  uint32_t tmem_base;
  uint32_t abort_flag;
};

template <int D>
struct Smem {
  static constexpr int kQTile = kBM * D * 2;
  static constexpr int kKV = kStep * D * 2;
  static constexpr int kQ = 0;
  static constexpr int kK = kQ + kTiles * kQTile;
  static constexpr int kV = kK + kStagesK * kKV;
  static constexpr int kBar = kV + kStagesV * kKV;
  static constexpr int kTotal = kBar + int(sizeof(Barriers)) + 1024;
};

// Packed fp32 pairs live in 64-bit registers; building and splitting them with
// mov.b64 keeps everything in registers (no address-taken locals).
__device__ __forceinline__ uint64_t f2_pack(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void f2_unpack(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t ffma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t fadd2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ uint64_t fmul2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
template <bool kBf16>
__device__ __forceinline__ uint32_t pack_pair(float lo, float hi) {
  if constexpr (kBf16) {
    __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&t);
  } else {
    __half2 t = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&t);
  }
}

template <int D, bool kBf16>
__global__ void __launch_bounds__(kThreads, 1) prefill_sm100_s64_kernel(const __grid_constant__ Sm100Args a) {
  using L = Smem<D>;
  constexpr int kHalves = D / 64;
  extern __shared__ uint8_t smem_dyn[];
  uint8_t* smem = smem_dyn + ((1024u - (smem_u32(smem_dyn) & 1023u)) & 1023u);  // an offset, so that the compiler keeps seeing shared memory
  Barriers* bar = reinterpret_cast<Barriers*>(smem + L::kBar);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // CTAs are handed out with blockIdx.x fastest: all (batch, head) pairs of the
  // heaviest (latest) row block first, the lightest row block last, so that the
  // tail of the grid is made of short CTAs
  const int qt = a.q_tiles - 1 - int(blockIdx.y);
  const int n_heads = a.groups * a.heads_per_group;
  const int gh = int(blockIdx.x) % n_heads;
  const int g = gh / a.heads_per_group, h = gh % a.heads_per_group;
  const int b = int(blockIdx.x) / n_heads;

  if (*reinterpret_cast<volatile int32_t*>(a.status) != 0) return;  // an earlier CTA gave up: drain the grid

  int q_row0 = 0, k_row0 = 0, qlen = a.mq, klen = a.mkv, tb = b;
  if (a.seqstart_q != nullptr) {
    q_row0 = a.seqstart_q[b];
    qlen = a.seqstart_q[b + 1] - q_row0;
    k_row0 = a.seqstart_k[b];
    klen = a.seqlen_k != nullptr ? a.seqlen_k[b] : a.seqstart_k[b + 1] - k_row0;
    tb = 0;
  }
  const int m0 = qt * kBM * kTiles;
  if (m0 >= qlen) return;
  const bool causal = a.mask_type != XFB200_MASK_NONE;
  const int shift = (a.mask_type == XFB200_MASK_CAUSAL_BOTTOM_RIGHT ? klen - qlen : 0) - a.kv_offset;

  // Step range [slo_t, shi_t) of each query tile, in units of kStep keys from
  // n_base (a multiple of kBN); the CTA loads the steps [S0, S1) of their union.
  int slo[kTiles], shi[kTiles];
  int n_base = 0;
  if (a.window_left >= 0) n_base = max(0, m0 + shift - a.window_left) / kBN * kBN;
  int s_min = 0x7fffffff, s_max = 0;
#pragma unroll
  for (int t = 0; t < kTiles; ++t) {
    const int mt0 = m0 + t * kBM;
    int hi = klen, lo = n_base;
    if (causal) hi = min(hi, mt0 + kBM + shift);
    if (a.window_left >= 0) lo = max(n_base, max(0, mt0 + shift - a.window_left) / kStep * kStep);
    if (mt0 >= qlen) hi = lo;  // no valid row in this tile
    slo[t] = (lo - n_base) / kStep;
    shi[t] = hi > lo ? (hi - n_base + kStep - 1) / kStep : slo[t];
    if (shi[t] > slo[t]) s_min = min(s_min, slo[t]), s_max = max(s_max, shi[t]);
  }
  const int S0 = s_max > 0 ? s_min : 0, S1 = s_max;  // steps this CTA loads
  const int kv_head = g * (a.kv_h_is_broadcast ? 1 : a.heads_per_group) + (a.kv_h_is_broadcast ? 0 : h);

  if (threadIdx.x == 0) {
    mbar_init(&bar->q_full, 1);
    for (int i = 0; i < kStagesK; ++i) {
      mbar_init(&bar->k_full[i], 1);
      mbar_init(&bar->k_empty[i], kTiles);  // released by both MMA warps
    }
    for (int i = 0; i < kStagesV; ++i) {
      mbar_init(&bar->v_full[i], 1);
      mbar_init(&bar->v_empty[i], kTiles);
    }
    for (int t = 0; t < kTiles; ++t) {
      for (int i = 0; i < 2; ++i) {
        mbar_init(&bar->s_full[t][i], 1);
        mbar_init(&bar->p_full[t][i], 128);
      }
      mbar_init(&bar->pv_done[t], 1);
      mbar_init(&bar->turn[t], 1);
    }
    bar->abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == kMmaWarp0) {
    tmem_alloc(&bar->tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bar->tmem_base;
  volatile uint32_t* abort_flag = &bar->abort_flag;

  if (warp >= kSoftmaxWarps) {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsAux));
  if (warp == kTmaWarp || warp == kTmaWarp + 1) {
    // =========================================== TMA producers: K (and Q) / V
    const bool is_v = warp == kTmaWarp + 1;
    if (lane == 0 && S1 > S0) {
      if (!is_v) {
        prefetch_tensormap(&a.tm_q);
        prefetch_tensormap(&a.tm_k);
        mbar_expect_tx(&bar->q_full, kTiles * L::kQTile);
#pragma unroll
        for (int t = 0; t < kTiles; ++t)
#pragma unroll
          for (int hf = 0; hf < kHalves; ++hf)
            tma_load_4d(smem + L::kQ + t * L::kQTile + hf * kHalfBytes, &a.tm_q, &bar->q_full, hf * 64, g * a.heads_per_group + h,
                        q_row0 + m0 + t * kBM, tb);
      } else {
        prefetch_tensormap(&a.tm_v);
      }
      const int stages = is_v ? kStagesV : kStagesK;
      uint64_t* full = is_v ? bar->v_full : bar->k_full;
      uint64_t* empty = is_v ? bar->v_empty : bar->k_empty;
      uint8_t* ring = smem + (is_v ? L::kV : L::kK);
      const CUtensorMap* tm = is_v ? &a.tm_v : &a.tm_k;
      int st = 0, use = 0;
      for (int sg = S0; sg < S1; ++sg) {
        const int row = k_row0 + n_base + sg * kStep;
        if (use > 0 && !mbar_wait(&empty[st], (use - 1) & 1, abort_flag)) {
          atomicExch(a.status, is_v ? 12 : 11);
          *abort_flag = 1;
          break;
        }
        mbar_expect_tx(&full[st], L::kKV);
#pragma unroll
        for (int hf = 0; hf < kHalves; ++hf)
          tma_load_4d(ring + st * L::kKV + hf * kKvHalfBytes, tm, &full[st], hf * 64, kv_head, row, tb);
        if (++st == stages) st = 0, ++use;
      }
    }
  } else if (warp == kMmaWarp0 || warp == kMmaWarp0 + 1) {
    // ===================================================== MMA issuer of tile t
    // tcgen05.mma is issued almost synchronously (the queue in front of the
    // tensor pipe is about one instruction deep) and a satisfied mbarrier wait
    // costs the issuing lane ~90 clocks: one issuing warp per query tile, so
    // that while one waits for its softmax the other keeps the pipe fed.
    const int t = warp - kMmaWarp0;
    constexpr uint32_t idesc_qk = umma_idesc(kBM, kStep, kBf16, false, false);
    constexpr uint32_t idesc_pv = umma_idesc(kBM, D, kBf16, false, true);
    bool ok = true;
    // Shared-memory descriptors: the upper word is constant (stride between
    // 8-row groups = 1024 B, version 1, 128B swizzle); the lower word holds
    // (address >> 4) and the leading-dimension offset, so stepping through a
    // tile is one 32-bit add per operand.
    constexpr uint32_t kDescHi = 64u | (1u << 14) | (2u << 29);
    auto desc = [](uint32_t lo) -> uint64_t {
      uint64_t d;
      asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(lo), "r"(kDescHi));
      return d;
    };
    const uint32_t q_lo = (smem_u32(smem + L::kQ + t * L::kQTile) >> 4) | (1u << 16);
    const uint32_t k_lo0 = (smem_u32(smem + L::kK) >> 4) | (1u << 16);
    const uint32_t v_lo0 = (smem_u32(smem + L::kV) >> 4) | ((kKvHalfBytes >> 4) << 16);
    const uint32_t tmem_t = tmem + t * 256, tmem_o = tmem_t + 128;
    // S[buf] = Q_t K^T for the 64 keys in `k_stage`
    auto issue_qk = [&](int k_stage, int buf, int kk_lo, int kk_hi) {
      const uint32_t kl = k_lo0 + k_stage * (L::kKV >> 4);
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        if (kk < kk_lo || kk >= kk_hi) continue;
        const uint32_t qoff = ((kk / 4) * kHalfBytes + (kk % 4) * 32) >> 4;
        const uint32_t koff = ((kk / 4) * kKvHalfBytes + (kk % 4) * 32) >> 4;
        umma_ss(tmem_t + buf * kStep, desc(q_lo + qoff), desc(kl + koff), idesc_qk, kk > 0);
      }
    };
    // O += P V for the keys in `v_stage`; A = P: packed 16-bit pairs, 8 columns of tensor memory per 16 keys
    auto issue_pv = [&](int v_stage, int buf, bool accumulate) {
      const uint32_t vl = v_lo0 + v_stage * (L::kKV >> 4);
#pragma unroll
      for (int kk = 0; kk < kStep / 16; ++kk)
        umma_ts(tmem_o, tmem_t + buf * kStep + kk * 8, desc(vl + ((kk * 16 * 128) >> 4)), idesc_pv, (accumulate || kk > 0) ? 1u : 0u);
    };

    // One lane does everything, waits included: lanes that merely spin on the same
    // barriers would share the warp's issue slots with the lane that feeds the tensor pipe.
    if (S1 > S0 && lane == 0) {
      ok = mbar_wait(&bar->q_full, 0, abort_flag);
      if (!ok) atomicExch(a.status, 21);
      // The first blocks are issued alternately by the two warps, tile 0 first, so
      // that the tiles start half a step apart: their softmax warps share the 2^x
      // units and should be in different phases.  (Alternating throughout costs a
      // hand-over of several hundred clocks per block: measured slower.)
      int turn_ph = 0;
      if (t == 1) mbar_arrive(&bar->turn[0]);
#ifndef XFB_S64_TURNS
#define XFB_S64_TURNS 2
#endif
#ifndef XFB_S64_PASS_AT
#define XFB_S64_PASS_AT 4
#endif
#define XFB_S64_TAKE_TURN                                        \
  if (s2 < S0 + XFB_S64_TURNS) {                                 \
    ok = mbar_wait(&bar->turn[t], turn_ph, abort_flag);          \
    turn_ph ^= 1;                                                \
    if (!ok) {                                                   \
      atomicExch(a.status, 27 + t);                              \
      break;                                                     \
    }                                                            \
  }
      // QK of step s2 and, two steps behind it, PV of step s2 - 2.  Steps outside
      // [slo, shi) of this tile issue nothing but still take part in the release of
      // the K/V stages (after seeing them full, so that this warp can never arrive
      // twice for the same use of a stage).
      int ks = 0, kuse = 0, vs = 0, vuse = 0;
      for (int s2 = S0; ok && s2 < S1 + 2; ++s2) {
        const int sp = s2 - 2;
        // Waits first -- the operand stages (long since full, but even a satisfied
        // wait costs the lane ~100 clocks), then the probabilities, which arrive
        // last -- so that PV and QK^T are issued back to back.
        if (sp >= S0) {
          ok = mbar_wait(&bar->v_full[vs], vuse & 1, abort_flag);
          if (!ok) {
            atomicExch(a.status, 22);
            break;
          }
          const int n0 = n_base + sp * kStep;
          if (n0 + kStep > klen) {
            // V rows past the end of the sequence may hold anything; P is 0 there.
            // Both MMA warps write the same zeros: no ordering between them is needed.
            const int first = max(klen - n0, 0);
            uint8_t* vt = smem + L::kV + vs * L::kKV;
            for (int hf = 0; hf < kHalves; ++hf)
              for (int i = first * 8; i < kStep * 8; ++i) *reinterpret_cast<uint4*>(vt + hf * kKvHalfBytes + i * 16) = make_uint4(0, 0, 0, 0);
            fence_proxy_async_smem();
          }
        }
        if (s2 < S1) {
          ok = mbar_wait(&bar->k_full[ks], kuse & 1, abort_flag);
          if (!ok) {
            atomicExch(a.status, 26);
            break;
          }
        }
        const bool act_pv = sp >= S0 && sp >= slo[t] && sp < shi[t];
        const bool act_qk = s2 < S1 && s2 >= slo[t] && s2 < shi[t];
        const int np = sp - slo[t], nq = s2 - slo[t];
        if (act_pv) {
          ok = mbar_wait(&bar->p_full[t][np & 1], (np >> 1) & 1, abort_flag);
          if (!ok) {
            atomicExch(a.status, 23 + t);
            break;
          }
        }
        tc_fence_after();
        XFB_S64_TAKE_TURN
        {
          if (act_pv) {
            issue_pv(vs, np & 1, np > 0);
            tc_commit(&bar->pv_done[t]);
          }
          if (sp >= S0) tc_commit(&bar->v_empty[vs]);
          // the token goes to the other warp a few MMAs before the end of the block,
          // so that the hand-over latency is hidden behind them
          if (act_qk) {
            issue_qk(ks, nq & 1, 0, XFB_S64_PASS_AT);
            if (s2 < S0 + XFB_S64_TURNS) mbar_arrive(&bar->turn[1 - t]);
            issue_qk(ks, nq & 1, XFB_S64_PASS_AT, D / 16);
            tc_commit(&bar->s_full[t][nq & 1]);
          } else if (s2 < S0 + XFB_S64_TURNS) {
            mbar_arrive(&bar->turn[1 - t]);
          }
          if (s2 < S1) tc_commit(&bar->k_empty[ks]);
        }
        if (sp >= S0 && ++vs == kStagesV) vs = 0, ++vuse;
        if (s2 < S1 && ++ks == kStagesK) ks = 0, ++kuse;
      }
      if (!ok) *abort_flag = 1;
    }
  }
  } else {
    // ================================================================ softmax
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsSoftmax));
    const int t = warp >> 2;                      // query tile of this warpgroup
    const int row = (warp & 3) * 32 + lane;       // TMEM lane == row inside the tile
    const uint32_t lane_sel = uint32_t((warp & 3) * 32) << 16;
    const uint32_t tmem_t = tmem + t * 256 + lane_sel;
    const uint32_t tmem_o = tmem_t + 128;
    const int mt0 = m0 + t * kBM;
    const int i_loc = mt0 + row;
    const int col_hi = causal ? min(klen, i_loc + shift + 1) : klen;
    const int col_lo = a.window_left >= 0 ? i_loc + shift - a.window_left : 0;
    const float sl2 = a.scale_log2;
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
    int cnt = 0;

    for (int sg = slo[t]; sg < shi[t]; ++sg, ++cnt) {
      const int n0 = n_base + sg * kStep;
      const int buf = cnt & 1;
      const uint32_t tmem_s = tmem_t + buf * kStep;
      ok = mbar_wait(&bar->s_full[t][buf], (cnt >> 1) & 1, abort_flag);
      if (!ok) {
        atomicExch(a.status, 31 + t);
        *abort_flag = 1;
        break;
      }
      tc_fence_after();
      uint32_t sr[kStep];
#pragma unroll
      for (int cblk = 0; cblk < kStep / 32; ++cblk) {
        uint32_t* dst = sr + cblk * 32;
        XFB_TMEM_LD_32(tmem_s + cblk * 32, dst);
      }
      tc_wait_ld();
      float* s = reinterpret_cast<float*>(sr);

      const bool need_mask = (n0 + kStep > klen) || (causal && n0 + kStep - 1 > mt0 + shift) ||
                             (a.window_left >= 0 && n0 < mt0 + kBM - 1 + shift - a.window_left);
      if (need_mask) {
#pragma unroll
        for (int c = 0; c < kStep; ++c) {
          const int col = n0 + c;
          s[c] = (col >= col_lo && col < col_hi) ? s[c] : -INFINITY;
        }
      }
      // row maximum: four independent chains of three-input max
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int c = 0; c < kStep; c += 8) {
        mx4[0] = fmax3(mx4[0], s[c], s[c + 1]);
        mx4[1] = fmax3(mx4[1], s[c + 2], s[c + 3]);
        mx4[2] = fmax3(mx4[2], s[c + 4], s[c + 5]);
        mx4[3] = fmax3(mx4[3], s[c + 6], s[c + 7]);
      }
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * sl2;  // scale > 0 (host guarantees)
      const bool raise = mx > m_run + kRescaleThreshold;  // also true on the first visible key (m_run = -inf)
      const float m_new = raise ? mx : m_run;
      const float alpha = raise ? (m_run == -INFINITY ? 0.f : fast_exp2(m_run - m_new)) : 1.f;
      const float m_use = m_new == -INFINITY ? 0.f : m_new;

      if (cnt > 0 && __any_sync(0xffffffffu, raise)) {
        // O_t may only be touched while no product accumulates into it: PV(cnt-1)
        // has to be complete (PV(cnt) cannot start before this thread hands over P).
        // The scores of this step prove PV(cnt-2) complete, so the parity wait is
        // unambiguous.
        ok = mbar_wait(&bar->pv_done[t], (cnt - 1) & 1, abort_flag);
        if (!ok) {
          atomicExch(a.status, 35 + t);
          *abort_flag = 1;
          break;
        }
        tc_fence_after();
        const uint64_t al2 = f2_pack(alpha, alpha);
#pragma unroll
        for (int cblk = 0; cblk < D / 32; ++cblk) {
          uint32_t orr[32];
          XFB_TMEM_LD_32(tmem_o + cblk * 32, orr);
          tc_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            float x0, x1;
            f2_unpack(fmul2(f2_pack(__uint_as_float(orr[i]), __uint_as_float(orr[i + 1])), al2), x0, x1);
            orr[i] = __float_as_uint(x0);
            orr[i + 1] = __float_as_uint(x1);
          }
          XFB_TMEM_ST_32(tmem_o + cblk * 32, orr);
        }
      }
      l_run *= alpha;
      m_run = m_new;

      // P = exp2(s * scale - m), packed pairs, straight back into tensor memory
      const uint64_t sc2 = f2_pack(sl2, sl2), nm2 = f2_pack(-m_use, -m_use);
      uint32_t pr[kStep / 2];
      // A lone warp per scheduler hides no latency by itself: the loop is written
      // in blocks of 16 independent elements (all FMAs, then all exp2, then the
      // sums and packs) with four independent sum chains.
      constexpr int kEB = 16;
      uint64_t sum2[4] = {f2_pack(0.f, 0.f), f2_pack(0.f, 0.f), f2_pack(0.f, 0.f), f2_pack(0.f, 0.f)};
#pragma unroll
      for (int c = 0; c < kStep; c += kEB) {
        float e[kEB];
#pragma unroll
        for (int i = 0; i < kEB; i += 2) f2_unpack(ffma2(f2_pack(s[c + i], s[c + i + 1]), sc2, nm2), e[i], e[i + 1]);
#pragma unroll
        for (int i = 0; i < kEB; ++i) e[i] = fast_exp2(e[i]);
#pragma unroll
        for (int i = 0; i < kEB; i += 2) {
          sum2[(i / 2) & 3] = fadd2(sum2[(i / 2) & 3], f2_pack(e[i], e[i + 1]));
          pr[(c + i) / 2] = pack_pair<kBf16>(e[i], e[i + 1]);
        }
      }
      {
        float x0, x1, y0, y1;
        f2_unpack(fadd2(sum2[0], sum2[1]), x0, x1);
        f2_unpack(fadd2(sum2[2], sum2[3]), y0, y1);
        l_run += (x0 + x1) + (y0 + y1);
      }
      XFB_TMEM_ST_32(tmem_s, pr);
      tc_wait_st();
      tc_fence_before();
      mbar_arrive(&bar->p_full[t][buf]);
    }

    // ---- epilogue
    const bool have = cnt > 0;
    if (ok && have) {
      // The last scores seen only prove that PV(cnt-3) is complete.  A parity
      // wait can tell apart two neighbouring phases, not three: wait for
      // PV(cnt-2) first, then for PV(cnt-1).
      if (cnt >= 2) ok = mbar_wait(&bar->pv_done[t], (cnt - 2) & 1, abort_flag);
      if (ok) ok = mbar_wait(&bar->pv_done[t], (cnt - 1) & 1, abort_flag);
      if (!ok) atomicExch(a.status, 33 + t);
      tc_fence_after();
    }
    const bool valid_row = i_loc < qlen;
    const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
    const int64_t o_off = int64_t(tb) * a.os.b + int64_t(q_row0 + i_loc) * a.os.m + int64_t(g) * a.os.g + int64_t(h) * a.os.h;
#pragma unroll
    for (int cblk = 0; cblk < D / 32; ++cblk) {
      uint32_t orr[32];
      if (ok && have) {
        XFB_TMEM_LD_32(tmem_o + cblk * 32, orr);
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
              w[e] = a.out_dtype == XFB200_BF16 ? pack_pair<true>(x0, x1) : pack_pair<false>(x0, x1);
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

  __syncthreads();
  if (warp == kMmaWarp0) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

template <int D, bool kBf16>
static int launch_t(const Sm100Args& a, cudaStream_t stream) {
  auto kern = prefill_sm100_s64_kernel<D, kBf16>;
  constexpr int smem = Smem<D>::kTotal;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return cuda_fail("prefill(sm100, 64-key steps): cudaFuncSetAttribute", e);
    configured = true;
  }
  const int64_t bh = int64_t(a.groups) * a.heads_per_group * a.batch;
  if (bh > 0x7fffffff || a.q_tiles > 65535) return set_error(XFB200_E_UNSUPPORTED, "prefill: grid too large");
  dim3 grid(unsigned(bh), a.q_tiles, 1);
  kern<<<grid, kThreads, smem, stream>>>(a);
  return check_launch("prefill_sm100_s64_kernel");
}

}  // namespace s64

int prefill_sm100_s64_launch(Sm100Args a, int head_dim, bool bf16, cudaStream_t stream) {
  if (head_dim == 128) return bf16 ? s64::launch_t<128, true>(a, stream) : s64::launch_t<128, false>(a, stream);
  return bf16 ? s64::launch_t<64, true>(a, stream) : s64::launch_t<64, false>(a, stream);
}

}  // namespace xfb
