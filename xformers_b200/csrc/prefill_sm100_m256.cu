// Attention forward (prefill) on tcgen05, 256 query rows per CTA.
//
// Two 128-row query tiles share every K/V tile that TMA brings in, and two
// softmax warpgroups work out of phase so that the tensor pipe always has
// either a QK^T or a PV product to run:
//
//   warps 0-3   softmax of query tile 0   (thread <-> row <-> TMEM lane)
//   warps 4-7   softmax of query tile 1
//   warp 8      MMA issuer of tile 0: ... PV(0,j), QK(0,j+1) ...   (one lane issues)
//   warp 9      MMA issuer of tile 1; the two pass a token so that their blocks
//               of MMAs alternate on the tensor pipe (an issuing thread stalls on
//               every barrier it waits for, two of them hide each other's stalls)
//   warp 10     TMA producer: Q (both tiles) once, then K_j / V_j into 2-deep rings
//   warp 11     idle
// The third warpgroup (warps 8-11) hands most of its registers to the two
// softmax warpgroups with setmaxnreg, so that a whole score row (128 fp32)
// stays in registers.  setmaxnreg only moves registers inside what the CTA was
// launched with; a request beyond that never returns (see kRegs* below).
//
// Tensor memory (all 512 columns): S0 | S1 | O0 | O1, fp32.  The probabilities
// P_t overwrite the first 64 columns of S_t as packed bf16/f16 pairs and feed
// the PV product straight from tensor memory (A operand in TMEM), so P never
// touches shared memory.  tcgen05 operations issued by one thread complete in
// order: when the barrier of QK(t,j) fires, PV(t,j-1) has finished, hence the
// softmax may rescale O_t and overwrite S_t/P_t without further hand-shakes.
//
// Softmax arithmetic runs on packed f32x2 FMA/ADD, exp2 with the scale folded
// in, four independent max/sum chains per thread, and a lazy running maximum
// (raised only when it grows by more than 2^8) so that rescaling the
// accumulator in tensor memory is rare.
//
// Masks are index arithmetic on (row, key) positions; K/V heads of a GQA group are
// indexed, never expanded; V rows past a sequence's end are zeroed in shared memory
// and K garbage is masked by select, so NaN in padding cannot leak; every wait is bounded.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "internal.h"
#include "prefill_sm100.h"
#include "ptx.cuh"

namespace xfb {
namespace m256 {

constexpr int kBM = 128;      // rows per query tile
constexpr int kTiles = 2;     // query tiles per CTA
constexpr int kBN = 128;      // keys per tile
// depth of the K and V rings (a third V stage measured no gain)
#ifndef XFB_KSTAGES
#define XFB_KSTAGES 2
#endif
#ifndef XFB_VSTAGES
#define XFB_VSTAGES 2
#endif
constexpr int kStagesK = XFB_KSTAGES, kStagesV = XFB_VSTAGES;
constexpr int kThreads = 384;  // warps 0-3 / 4-7: softmax of tile 0 / 1; 8, 9: MMA of tile 0 / 1; 10: TMA; 11 idle
constexpr int kMmaWarp0 = 8, kTmaWarp = 10;  // warps 8 and 9 issue the MMAs of query tile 0 and 1
// registers per thread after setmaxnreg: 8 softmax warps grow, 4 other warps shrink;
// the sum must fit what 384 threads were launched with (168 each)
constexpr int kRegsLaunch = 168, kRegsSoftmax = 208, kRegsAux = 88;
static_assert(8 * kRegsSoftmax + 4 * kRegsAux <= 12 * kRegsLaunch, "setmaxnreg would ask for more registers than the CTA owns");
constexpr float kRescaleThreshold = 8.0f;
constexpr uint32_t kHalfBytes = 128 * 128;  // one 64-column block of a 128-row tile

struct __align__(8) Barriers {
  uint64_t q_full;
  uint64_t k_full[kStagesK], v_full[kStagesV], k_empty[kStagesK], v_empty[kStagesV];
  uint64_t s_full[kTiles], p_full[kTiles], pv_done[kTiles];
  uint64_t turn[kTiles];  // token of the tensor pipe: the two MMA warps issue their blocks alternately
  uint32_t tmem_base;
  uint32_t abort_flag;
};

template <int D>
struct Smem {
  static constexpr int kQTile = kBM * D * 2;
  static constexpr int kKV = kBN * D * 2;
  static constexpr int kQ = 0;
  static constexpr int kK = kQ + kTiles * kQTile;
  static constexpr int kV = kK + kStagesK * kKV;
  static constexpr int kBar = kV + kStagesV * kKV;
  static constexpr int kTotal = kBar + 256 + 1024;
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

// Records the first code a launch gives up with (kept until the host reads it) and marks the
// launch, so that its remaining CTAs leave at once.
__device__ __forceinline__ void give_up(const Sm100Args& a, int code) {
  atomicCAS(a.status, 0, code);
  reinterpret_cast<volatile int32_t*>(a.status)[1] = int32_t(a.epoch);
}

template <int D, bool kBf16>
__global__ void __launch_bounds__(kThreads, 1) prefill_sm100_m256_kernel(const __grid_constant__ Sm100Args a) {
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

  if (reinterpret_cast<volatile int32_t*>(a.status)[1] == int32_t(a.epoch)) return;  // a CTA of this launch gave up: drain the grid

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
  // query i sees key j iff i + shift - window_left <= j <= i + shift + wr (each bound only when it is >= 0)
  const int wr = a.window_right;
  const bool causal = wr >= 0;
  const int shift = (a.bottom_right ? klen - qlen : 0) - a.kv_offset;

  // Key-tile range [jlo_t, jhi_t) of each query tile, in units of kBN keys from n_base.
  int jlo[kTiles], jhi[kTiles];
  int n_base = 0;
  if (a.window_left >= 0) n_base = max(0, m0 + shift - a.window_left) / kBN * kBN;
  int j_end = 0;
#pragma unroll
  for (int t = 0; t < kTiles; ++t) {
    const int mt0 = m0 + t * kBM;
    int hi = klen, lo = n_base;
    if (causal) hi = min(hi, mt0 + kBM + shift + wr);
    if (a.window_left >= 0) lo = max(n_base, max(0, mt0 + shift - a.window_left) / kBN * kBN);
    if (mt0 >= qlen) hi = lo;  // no valid row in this tile
    jlo[t] = (lo - n_base) / kBN;
    jhi[t] = hi > lo ? (hi - n_base + kBN - 1) / kBN : jlo[t];
    j_end = max(j_end, jhi[t]);
  }
  const int j_begin = min(jlo[0], jlo[1]);
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
      mbar_init(&bar->s_full[t], 1);
      mbar_init(&bar->p_full[t], 128);
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

  if (warp >= 8) {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsAux));
  if (warp == kTmaWarp) {
    // ============================================================ TMA producer
    if (lane == 0 && j_end > j_begin) {
      prefetch_tensormap(&a.tm_q);
      prefetch_tensormap(&a.tm_k);
      prefetch_tensormap(&a.tm_v);
      mbar_expect_tx(&bar->q_full, kTiles * L::kQTile);
#pragma unroll
      for (int t = 0; t < kTiles; ++t)
#pragma unroll
        for (int hf = 0; hf < kHalves; ++hf)
          tma_load_4d(smem + L::kQ + t * L::kQTile + hf * kHalfBytes, &a.tm_q, &bar->q_full, hf * 64, g * a.heads_per_group + h,
                      q_row0 + m0 + t * kBM, tb);
      for (int j = j_begin; j < j_end; ++j) {
        const int it = j - j_begin, st = it % kStagesK, use = it / kStagesK;
        const int sv = it % kStagesV, use_v = it / kStagesV;
        const int row = k_row0 + n_base + j * kBN;
        if (use > 0 && !mbar_wait(&bar->k_empty[st], (use - 1) & 1, abort_flag, a.wait_budget)) {
          give_up(a, 11);
          *abort_flag = 1;
          break;
        }
        // (testing aid: the first CTA leaves out its last key tile, so that the wait for it runs out)
        if (!((a.debug_flags & 1) && blockIdx.x == 0 && blockIdx.y == 0 && j == j_end - 1)) {
          mbar_expect_tx(&bar->k_full[st], L::kKV);
#pragma unroll
          for (int hf = 0; hf < kHalves; ++hf)
            tma_load_4d(smem + L::kK + st * L::kKV + hf * kHalfBytes, &a.tm_k, &bar->k_full[st], hf * 64, kv_head, row, tb);
        }
        if (use_v > 0 && !mbar_wait(&bar->v_empty[sv], (use_v - 1) & 1, abort_flag, a.wait_budget)) {
          give_up(a, 12);
          *abort_flag = 1;
          break;
        }
        {
          mbar_expect_tx(&bar->v_full[sv], L::kKV);
#pragma unroll
          for (int hf = 0; hf < kHalves; ++hf)
            tma_load_4d(smem + L::kV + sv * L::kKV + hf * kHalfBytes, &a.tm_v, &bar->v_full[sv], hf * 64, kv_head, row, tb);
        }
      }
    }
  } else if (warp == kMmaWarp0 || warp == kMmaWarp0 + 1) {
    // ===================================================== MMA issuer of tile t
    // tcgen05.mma is issued almost synchronously (the queue in front of the
    // tensor pipe is about one instruction deep), so every clock this lane
    // spends on anything else -- a satisfied mbarrier wait alone costs ~90 --
    // is a clock the tensor pipe idles.  Hence one issuing warp per query tile:
    // while one waits for its softmax, the other keeps the pipe fed.
    const int t = warp - kMmaWarp0;
    constexpr uint32_t idesc_qk = umma_idesc(kBM, kBN, kBf16, false, false);
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
    const uint32_t v_lo0 = (smem_u32(smem + L::kV) >> 4) | ((kHalfBytes >> 4) << 16);
    const uint32_t tmem_s = tmem + t * 128, tmem_o = tmem + 256 + t * 128;
    auto issue_qk_part = [&](int k_stage, int kk_lo, int kk_hi) {
      const uint32_t kl = k_lo0 + k_stage * (L::kKV >> 4);
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        if (kk < kk_lo || kk >= kk_hi) continue;
        const uint32_t off = ((kk / 4) * kHalfBytes + (kk % 4) * 32) >> 4;
        umma_ss(tmem_s, desc(q_lo + off), desc(kl + off), idesc_qk, kk > 0);
      }
    };
    auto issue_qk = [&](int k_stage) { issue_qk_part(k_stage, 0, D / 16); };
    auto issue_pv = [&](int v_stage, bool accumulate) {
      const uint32_t vl = v_lo0 + v_stage * (L::kKV >> 4);
#pragma unroll
      for (int kk = 0; kk < kBN / 16; ++kk) {
        // A = P_t: packed 16-bit pairs, 8 columns of tensor memory per 16 keys
        umma_ts(tmem_o, tmem_s + kk * 8, desc(vl + ((kk * 16 * 128) >> 4)), idesc_pv, (accumulate || kk > 0) ? 1u : 0u);
      }
    };

    if (j_end > j_begin) {
      // ring positions advance by one per key tile (no divisions in the loop)
      int ks = 0, kph = 0;  // K stage / phase of tile j
      int vs = 0, vph = 0;  // V stage / phase of tile j
      int cnt = 0;          // products of this query tile so far
      ok = mbar_wait(&bar->q_full, 0, abort_flag, a.wait_budget) && mbar_wait(&bar->k_full[0], 0, abort_flag, a.wait_budget);
      if (!ok && lane == 0) give_up(a, 21);
      if (ok) {
        tc_fence_after();
        if (lane == 0) {
          if (j_begin >= jlo[t] && j_begin < jhi[t]) {
            issue_qk(0);
            tc_commit(&bar->s_full[t]);
          }
          tc_commit(&bar->k_empty[0]);
          if (t == 1) mbar_arrive(&bar->turn[0]);  // tile 0 opens every iteration
        }
      }
      int turn_ph = 0;
      for (int j = j_begin; ok && j < j_end; ++j) {
        const bool has_next = j + 1 < j_end;
        const bool act = j >= jlo[t] && j < jhi[t];
        const bool act_next = has_next && (j + 1) >= jlo[t] && (j + 1) < jhi[t];
        int ks1 = ks + 1, kph1 = kph;
        if (ks1 == kStagesK) ks1 = 0, kph1 ^= 1;
        ok = mbar_wait(&bar->v_full[vs], vph, abort_flag, a.wait_budget);
        if (ok && has_next) ok = mbar_wait(&bar->k_full[ks1], kph1, abort_flag, a.wait_budget);
        if (!ok) {
          if (lane == 0) give_up(a, 22);
          break;
        }
        const int n0 = n_base + j * kBN;
        if (n0 + kBN > klen) {
          // V rows past the end of the sequence may hold anything; P is 0 there.
          // Both MMA warps write the same zeros: no ordering between them is needed.
          const int first = max(klen - n0, 0);
          uint8_t* vt = smem + L::kV + vs * L::kKV;
          for (int hf = 0; hf < kHalves; ++hf)
            for (int i = first * 8 + lane; i < kBN * 8; i += 32) *reinterpret_cast<uint4*>(vt + hf * kHalfBytes + i * 16) = make_uint4(0, 0, 0, 0);
          fence_proxy_async_smem();
          __syncwarp();
        }
        if (act) {
          ok = mbar_wait(&bar->p_full[t], cnt & 1, abort_flag, a.wait_budget);
          if (!ok) {
            if (lane == 0) give_up(a, 23 + t);
            break;
          }
          tc_fence_after();
        }
        // If both warps issued at will, their MMAs would interleave one by one,
        // both tiles would finish together and both softmaxes would run at the
        // same time with the tensor pipe idle.  Blocks (PV, next QK) are
        // therefore issued alternately, which keeps the two tiles half a period
        // apart; the token is passed a few MMAs before the end of a block so
        // that the hand-over latency is hidden.
        ok = mbar_wait(&bar->turn[t], turn_ph, abort_flag, a.wait_budget);
        turn_ph ^= 1;
        if (!ok) {
          if (lane == 0) give_up(a, 25 + t);
          break;
        }
        if (lane == 0) {
          if (act) {
            issue_pv(vs, cnt > 0);
            tc_commit(&bar->pv_done[t]);
          }
          tc_commit(&bar->v_empty[vs]);
          if (act_next) {
            issue_qk_part(ks1, 0, D / 32);
            mbar_arrive(&bar->turn[1 - t]);
            issue_qk_part(ks1, D / 32, D / 16);
            tc_commit(&bar->s_full[t]);
          } else {
            mbar_arrive(&bar->turn[1 - t]);
          }
          if (has_next) tc_commit(&bar->k_empty[ks1]);
        }
        if (act) ++cnt;
        ks = ks1, kph = kph1;
        if (++vs == kStagesV) vs = 0, vph ^= 1;
      }
      if (!ok) *abort_flag = 1;
    }
  }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsSoftmax));
    // ================================================================ softmax
    const int t = warp >> 2;                      // query tile of this warpgroup
    const int row = (warp & 3) * 32 + lane;       // TMEM lane == row inside the tile
    const uint32_t lane_sel = uint32_t((warp & 3) * 32) << 16;
    const uint32_t tmem_s = tmem + t * 128 + lane_sel;
    const uint32_t tmem_o = tmem + 256 + t * 128 + lane_sel;
    const int mt0 = m0 + t * kBM;
    const int i_loc = mt0 + row;
    const int col_hi = causal ? min(klen, i_loc + shift + wr + 1) : klen;
    const int col_lo = a.window_left >= 0 ? i_loc + shift - a.window_left : 0;
    const float sl2 = a.scale_log2;
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
    int cnt = 0;

    for (int j = jlo[t]; j < jhi[t]; ++j, ++cnt) {
      const int n0 = n_base + j * kBN;
      ok = mbar_wait(&bar->s_full[t], cnt & 1, abort_flag, a.wait_budget);
      if (!ok) {
        give_up(a, 31 + t);
        *abort_flag = 1;
        break;
      }
      tc_fence_after();
      uint32_t sr[kBN];
#pragma unroll
      for (int cblk = 0; cblk < kBN / 32; ++cblk) {
        uint32_t* dst = sr + cblk * 32;
        XFB_TMEM_LD_32(tmem_s + cblk * 32, dst);
      }
      tc_wait_ld();
      float* s = reinterpret_cast<float*>(sr);

      const bool need_mask = (n0 + kBN > klen) || (causal && n0 + kBN - 1 > mt0 + shift + wr) ||
                             (a.window_left >= 0 && n0 < mt0 + kBM - 1 + shift - a.window_left);
      if (need_mask) {
#pragma unroll
        for (int c = 0; c < kBN; ++c) {
          const int col = n0 + c;
          s[c] = (col >= col_lo && col < col_hi) ? s[c] : -INFINITY;
        }
      }
      // row maximum: four independent chains
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int c = 0; c < kBN; c += 8) {  // three-input max: two elements per instruction
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

      // QK(t,j) completing implies PV(t,j-1) completed: O_t is quiescent here
      if (cnt > 0 && __any_sync(0xffffffffu, raise)) {
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
      uint32_t pr[kBN / 2];
      // A lone warp per scheduler hides no latency by itself: the loop is written
      // in blocks of XFB_EXP_BLOCK independent elements (all FMAs, then all exp2,
      // then the sums and packs) with four independent sum chains.
#ifndef XFB_EXP_BLOCK
#define XFB_EXP_BLOCK 16
#endif
      constexpr int kEB = XFB_EXP_BLOCK;
      uint64_t sum2[4] = {f2_pack(0.f, 0.f), f2_pack(0.f, 0.f), f2_pack(0.f, 0.f), f2_pack(0.f, 0.f)};
#pragma unroll
      for (int c = 0; c < kBN; c += kEB) {
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
      {
        uint32_t* p0 = pr;
        uint32_t* p1 = pr + 32;
        XFB_TMEM_ST_32(tmem_s, p0);
        XFB_TMEM_ST_32(tmem_s + 32, p1);
      }
      tc_wait_st();
      tc_fence_before();
      mbar_arrive(&bar->p_full[t]);
    }

    // ---- epilogue
    const bool have = cnt > 0;
    if (ok && have) {
      ok = mbar_wait(&bar->pv_done[t], (cnt - 1) & 1, abort_flag, a.wait_budget);
      if (!ok) give_up(a, 33 + t);
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
  auto kern = prefill_sm100_m256_kernel<D, kBf16>;
  constexpr int smem = Smem<D>::kTotal;
  static bool configured[kMaxDevices] = {false};  // the attribute belongs to the device's context
  if (first_use_on_device(configured)) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return cuda_fail("prefill(sm100, 256 rows): cudaFuncSetAttribute", e);
  }
  const int64_t bh = int64_t(a.groups) * a.heads_per_group * a.batch;
  if (bh > 0x7fffffff || a.q_tiles > 65535) return set_error(XFB200_E_UNSUPPORTED, "prefill: grid too large");
  dim3 grid(unsigned(bh), a.q_tiles, 1);
  kern<<<grid, kThreads, smem, stream>>>(a);
  return check_launch("prefill_sm100_m256_kernel");
}

}  // namespace m256

int prefill_sm100_m256_launch(Sm100Args a, int head_dim, bool bf16, cudaStream_t stream) {
  if (head_dim == 128) return bf16 ? m256::launch_t<128, true>(a, stream) : m256::launch_t<128, false>(a, stream);
  return bf16 ? m256::launch_t<64, true>(a, stream) : m256::launch_t<64, false>(a, stream);
}

}  // namespace xfb
