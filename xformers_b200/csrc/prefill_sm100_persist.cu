// Attention forward (prefill) on tcgen05: one persistent CTA per SM.
//
// A work item is a block of 256 query rows of one (sequence, query head): two
// 128-row query tiles that share every K/V tile TMA brings in.  Items are
// handed out by one atomic counter, heaviest first (the last row block of every
// head, then the one before, ...) inside groups of heads whose keys and values
// fit the L2 together, so the SMs stay evenly loaded whatever the sequence
// lengths are, a K/V tile comes from DRAM once and from the L2 for the other row
// blocks of its head, and everything a CTA sets up -- tensor memory, barriers,
// tensor-map prefetch -- is paid once per SM instead of once per block of rows.
// The roles of the 16 warps:
//
//   warps 0-3    softmax of query tile 0   (thread <-> row <-> TMEM lane)
//   warps 4-7    softmax of query tile 1
//   warps 8-11   output: O_t / l -> global memory, log-sum-exp.  They work on
//                item i while every other warp is already on item i + 1, so
//                the tensor pipe does not wait for the write-back.
//   warp 12/13   MMA issuer of tile 0 / 1 (one lane issues); the two pass a
//                token so that their blocks of MMAs alternate on the tensor pipe
//   warp 14      scheduler + TMA producer: pulls the next item one item ahead of
//                time, works out its geometry once and announces it to the other
//                warps through a small ring of descriptors in shared memory,
//                loads Q (per tile) and the K/V tiles into 2-deep rings that run
//                on across item boundaries.  Items in which no query sees any
//                key (possible when the key axis is sharded) never enter the
//                ring: this warp writes their zeros and -inf itself.
//   warp 15      idle
//
// Tensor memory (all 512 columns): S0 | S1 | O0 | O1, fp32.  The probabilities
// P_t overwrite the last 64 columns of S_t as packed 16-bit pairs (keys 64-127
// in columns 64-95, keys 0-63 in columns 96-127) and feed the PV product
// straight from tensor memory.  tcgen05 operations issued by one
// thread complete in order: when the barrier of QK(t, j) fires, PV(t, j-1) has
// finished, so the softmax may rescale O_t and overwrite S_t / P_t without
// further hand-shakes; across items the first PV of a tile waits until the
// output warps have read the previous O_t out of tensor memory.
//
// Softmax: thread = row.  A step reads the row's 128 scores out of tensor memory
// twice.  First for their maximum: if it exceeds the row's reference maximum by
// more than 2^8 the row is re-based at once (O_t is quiescent at that point, see
// above), otherwise the reference stays and nothing is rescaled -- one vote and
// one rarely taken branch per step.  Then for the probabilities, which are stored
// back as P chunk by chunk.  The second pass starts with the two chunks (of 32
// columns) the first one ended with, straight from registers, and P goes into
// columns 64-127 in the order in which it is produced (keys 64-127 first), so
// that only the first 64 columns are read a second time and their loads fly
// behind the exponentials of the other half.  A warp runs almost alone on its
// scheduler: every vote, branch or wait it executes is a bubble nobody fills, so
// the step has no loop and no per-chunk test.  On diagonal and ragged tiles a
// small loop first writes -inf over the hidden scores in tensor memory; the step
// itself is one piece of code for every tile, which the instruction cache likes.
// An additive bias is folded into the scores the same way (bias / scale added in
// tensor memory).  When the first half of P (keys 64-127) is stored the softmax
// arrives on a barrier of its own and the MMA warp issues that half of PV while
// the other half is still being computed.  Measured
// alternatives on the causal 4k case: one pass with a stale reference, a vote per
// chunk and a fix-up path (10 % slower: the votes and branches); the whole row in
// registers as in the one-CTA-per-block kernel; two threads per row; part of the
// exponentials as a cubic on the FMA pipe (slower at every fraction).
//
// Masks are index arithmetic on (row, key) positions; K/V heads of a GQA group
// are indexed, never expanded; V rows past a sequence's end are zeroed in
// shared memory and K garbage is masked by select, so NaN in padding cannot
// leak.  Every wait is bounded: a wait that runs out records a code in the
// device status word, all warps leave their loops, tensor memory is freed and
// the CTA returns.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "internal.h"
#include "prefill_sm100.h"
#include "ptx.cuh"

namespace xfb {
namespace pst {

constexpr int kBM = 128;    // rows per query tile
constexpr int kTiles = 2;   // query tiles per item
constexpr int kBN = 128;    // keys per step
constexpr int kStages = 2;  // depth of the K and of the V ring
constexpr int kSched = 4;   // depth of the ring that announces work items
constexpr int kThreads = 512;
constexpr int kOutWarp0 = 8, kMmaWarp0 = 12, kTmaWarp = 14;
constexpr int kItemReaders = 14;  // warps that read every announced item (all but the scheduler and the idle one)
// registers per thread after setmaxnreg; the sum over the 16 warps must fit what the CTA was launched with
#ifndef XFB_PST_REGS_SOFTMAX
#define XFB_PST_REGS_SOFTMAX 176
#endif
#ifndef XFB_PST_REGS_OUT
#define XFB_PST_REGS_OUT 80
#endif
#ifndef XFB_PST_REGS_AUX
#define XFB_PST_REGS_AUX 80
#endif
constexpr int kRegsLaunch = 128, kRegsSoftmax = XFB_PST_REGS_SOFTMAX, kRegsOut = XFB_PST_REGS_OUT, kRegsAux = XFB_PST_REGS_AUX;
static_assert(8 * kRegsSoftmax + 4 * kRegsOut + 4 * kRegsAux <= 16 * kRegsLaunch, "setmaxnreg would ask for more registers than the CTA owns");
constexpr float kRescaleThreshold = 8.0f;  // a row is re-based when its maximum grew by more than 2^8: probabilities stay below 2^8
constexpr uint32_t kHalfBytes = 128 * 128;  // one 64-column block of a 128-row tile

// Geometry of a work item, worked out once by the scheduler warp and read by the others from shared memory.
struct Item {
  int idx;  // item number, -1 = no more work
  int b, head, kv_head, tb;
  int g, h;
  int q_row0, k_row0, qlen, klen;
  int m0, shift, n_base;
  int shift2;  // two key ranges in one tensor: what `shift` is for the keys from row kv_split on
  int jlo[kTiles], jhi[kTiles];  // key-step range of each query tile, in steps of kBN keys from n_base
  int j_begin, j_end;            // steps any tile takes part in
};

struct __align__(8) Barriers {
  uint64_t sched_full[kSched], sched_empty[kSched];
  uint64_t q_full[kTiles], q_empty[kTiles];
  uint64_t k_full[kStages], v_full[kStages], k_empty[kStages], v_empty[kStages];
  uint64_t s_full[kTiles], p_half[kTiles], p_full[kTiles];  // p_half: the probabilities of keys 64-127 are stored
  uint64_t o_full[kTiles], o_empty[kTiles];
  uint64_t stats_full[kTiles], stats_empty[kTiles];
  uint64_t turn[kTiles];  // token of the tensor pipe: the two MMA warps issue their blocks alternately
  Item sched_item[kSched];
  uint32_t tmem_base;
  uint32_t abort_flag;
};

template <int D>
struct Smem {
  static constexpr int kQTile = kBM * D * 2;
  static constexpr int kKV = kBN * D * 2;
  static constexpr int kQ = 0;
  static constexpr int kK = kQ + kTiles * kQTile;
  static constexpr int kV = kK + kStages * kKV;
  static constexpr int kStats = kV + kStages * kKV;          // float2 [kTiles][kBM]: running maximum (log2 units), row sum
  static constexpr int kBar = kStats + kTiles * kBM * 8;
  static constexpr int kTotal = kBar + 1024 + 1024;
};
static_assert(sizeof(Barriers) <= 1024, "barrier block");

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
__device__ __forceinline__ void unpack_pair(uint32_t x, float& lo, float& hi) {
  if constexpr (kBf16) {
    lo = __uint_as_float(x << 16);
    hi = __uint_as_float(x & 0xffff0000u);
  } else {
    const float2 f = __half22float2(*reinterpret_cast<__half2*>(&x));
    lo = f.x, hi = f.y;
  }
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

#ifdef XFB_PST_PROFILE
// Timing build only: per-CTA cycle counters of the softmax warps (8 slots each, 0-63) and, with
// -DXFB_PST_PROFILE_MMA, of the two MMA issuers (64-79 / 80-95), read back with xfb200_debug_read_prefill_profile.
__device__ long long g_prof[160][96];
#define XFB_PROF_DECL(n) long long prof_acc[n] = {0}; long long prof_t = clock64();
#define XFB_PROF_LAP(k) { const long long _n = clock64(); prof_acc[k] += _n - prof_t; prof_t = _n; }
#define XFB_PROF_COUNT(k) { prof_acc[k] += 1; }
#define XFB_PROF_STORE(base, n) { if (lane == 0 && blockIdx.x < 160) for (int _i = 0; _i < (n); ++_i) g_prof[blockIdx.x][(base) + _i] += prof_acc[_i]; }
#else
#define XFB_PROF_DECL(n)
#define XFB_PROF_LAP(k)
#define XFB_PROF_COUNT(k)
#define XFB_PROF_STORE(base, n)
#endif

// Records the first code a launch gives up with (kept until the host reads it) and marks the
// launch, so that CTAs that have not started yet leave at once.
__device__ __forceinline__ void give_up(const Sm100Args& a, int code) {
  atomicCAS(a.status, 0, code);
  reinterpret_cast<volatile int32_t*>(a.status)[1] = int32_t(a.epoch);
}

// Returns false when the item has no query row at all (a row block past the end of its sequence).
__device__ __forceinline__ bool decode_item(const Sm100Args& a, int idx, Item& it) {
  it.idx = idx;
  const int n_heads = a.groups * a.heads_per_group;
  const int n_bh = n_heads * a.batch;
  // Heaviest (latest) row blocks first, but not over all heads at once: the CTAs of a launch run side by side, and
  // the keys and values they read should fit the L2 (a K/V tile is read once per row block of its head: from DRAM
  // the first time only, if it is still there).  Heads are taken in groups of heads_per_wave; inside a group the
  // row blocks go from the last to the first, so the launch still ends with light items.
  const int kHeadsPerWave = a.heads_per_wave;
  const int grp = idx / (kHeadsPerWave * a.q_tiles);
  const int first_bh = grp * kHeadsPerWave;
  const int in_grp = min(kHeadsPerWave, n_bh - first_bh);
  const int rr = idx - grp * kHeadsPerWave * a.q_tiles;
  const int qt = a.q_tiles - 1 - rr / in_grp;
  const int bh = first_bh + rr % in_grp;
  it.b = bh / n_heads;
  it.head = bh % n_heads;
  it.g = it.head / a.heads_per_group, it.h = it.head % a.heads_per_group;
  it.kv_head = it.g * (a.kv_h_is_broadcast ? 1 : a.heads_per_group) + (a.kv_h_is_broadcast ? 0 : it.h);
  it.q_row0 = 0, it.k_row0 = 0, it.qlen = a.mq, it.klen = a.mkv, it.tb = it.b;
  if (a.seqstart_q != nullptr) {
    it.q_row0 = a.seqstart_q[it.b];
    it.qlen = a.seqstart_q[it.b + 1] - it.q_row0;
    it.k_row0 = a.seqstart_k[it.b];
    it.klen = a.seqlen_k != nullptr ? a.seqlen_k[it.b] : a.seqstart_k[it.b + 1] - it.k_row0;
    it.tb = 0;
  }
  it.m0 = qt * kBM * kTiles;
  if (it.m0 >= it.qlen) return false;
  it.shift = (a.bottom_right ? it.klen - it.qlen : 0) - a.kv_offset;
  it.shift2 = -a.kv_offset2;
  it.n_base = 0;
  if (a.window_left >= 0) it.n_base = max(0, it.m0 + it.shift - a.window_left) / kBN * kBN;
  it.j_begin = 0x7fffffff, it.j_end = 0;
#pragma unroll
  for (int t = 0; t < kTiles; ++t) {
    const int mt0 = it.m0 + t * kBM;
    int hi = it.klen, lo = it.n_base;
    if (a.window_right >= 0) hi = min(hi, mt0 + kBM + it.shift + a.window_right);
    if (a.kv_split > 0) {
      // Two key ranges back to back (causal, the second one later in the sequence): rows that see any key of the
      // second range see all of the first, so the visible keys are still one run of rows of the tensor.
      const int hi1 = min(it.klen - a.kv_split, mt0 + kBM + it.shift2);
      hi = hi1 > 0 ? a.kv_split + hi1 : min(a.kv_split, mt0 + kBM + it.shift);
    }
    if (a.window_left >= 0) lo = max(it.n_base, max(0, mt0 + it.shift - a.window_left) / kBN * kBN);
    if (mt0 >= it.qlen) hi = lo;  // no valid row in this tile
    it.jlo[t] = (lo - it.n_base) / kBN;
    it.jhi[t] = hi > lo ? (hi - it.n_base + kBN - 1) / kBN : it.jlo[t];
    if (it.jhi[t] > it.jlo[t]) {
      it.j_begin = min(it.j_begin, it.jlo[t]);
      it.j_end = max(it.j_end, it.jhi[t]);
    }
  }
  if (it.j_end == 0) it.j_begin = 0;
  return true;
}

template <int D, bool kBf16>
__global__ void __launch_bounds__(kThreads, 1) prefill_sm100_persist_kernel(const __grid_constant__ Sm100Args a) {
  using L = Smem<D>;
  constexpr int kHalves = D / 64;
  extern __shared__ uint8_t smem_dyn[];
  uint8_t* smem = smem_dyn + ((1024u - (smem_u32(smem_dyn) & 1023u)) & 1023u);  // an offset, so that the compiler keeps seeing shared memory
  Barriers* bar = reinterpret_cast<Barriers*>(smem + L::kBar);
  float2* stats = reinterpret_cast<float2*>(smem + L::kStats);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_items = a.q_tiles * a.groups * a.heads_per_group * a.batch;
  const long long budget = a.wait_budget;

  // a CTA of this launch already gave up: take no work (the counters are still settled below)
  const bool drained = reinterpret_cast<volatile int32_t*>(a.status)[1] == int32_t(a.epoch);

  if (!drained) {
    if (threadIdx.x == 0) {
      for (int i = 0; i < kSched; ++i) {
        mbar_init(&bar->sched_full[i], 1);
        mbar_init(&bar->sched_empty[i], kItemReaders);
      }
      for (int i = 0; i < kStages; ++i) {
        mbar_init(&bar->k_full[i], 1);
        mbar_init(&bar->k_empty[i], kTiles);  // released by both MMA warps
        mbar_init(&bar->v_full[i], 1);
        mbar_init(&bar->v_empty[i], kTiles);
      }
      for (int t = 0; t < kTiles; ++t) {
        mbar_init(&bar->q_full[t], 1);
        mbar_init(&bar->q_empty[t], 1);
        mbar_init(&bar->s_full[t], 1);
        mbar_init(&bar->p_half[t], 4);  // one arrival per softmax warp of the tile
        mbar_init(&bar->p_full[t], 4);
        mbar_init(&bar->o_full[t], 1);
        mbar_init(&bar->o_empty[t], 128);
        mbar_init(&bar->stats_full[t], 128);
        mbar_init(&bar->stats_empty[t], 128);
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

    // Next announced item (every announced item has key steps): its number, -1 after the last one, -2 when the
    // wait ran out.  `take` copies what the caller needs out of the descriptor before the slot is handed back.
    auto pop_item = [&](int& seq, auto&& take) -> int {
      const int slot = seq % kSched;
      if (!mbar_wait(&bar->sched_full[slot], (seq / kSched) & 1, abort_flag, budget)) return -2;
      const Item* d = &bar->sched_item[slot];
      const int idx = d->idx;
      if (idx >= 0) take(*d);
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar->sched_empty[slot]);
      ++seq;
      return idx;
    };

    if (warp >= kMmaWarp0) {
      asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsAux));
      if (warp == kTmaWarp) {
        // ============================================ scheduler + TMA producer
        // Lane 0 waits and issues; all lanes run the loop, because pulling an item (a broadcast)
        // and writing the rows of an item without visible keys are done by the whole warp.
        if (lane == 0) {
          prefetch_tensormap(&a.tm_q);
          prefetch_tensormap(&a.tm_k);
          prefetch_tensormap(&a.tm_v);
        }
        int seq = 0;              // items announced
        int kstep = 0;            // K/V steps loaded, over all items
        int aq[kTiles] = {0, 0};  // items in which tile t took part so far
        bool ok = true;
        // Pulls item numbers until one has key steps.  Row blocks past the end of their sequence are
        // skipped; blocks whose rows see no key at all get their result here: zeros and -inf.
        auto next_item = [&](Item& it) {
          for (;;) {
            int idx = 0;
            if (lane == 0) idx = atomicAdd(a.counters, 1);
            idx = __shfl_sync(0xffffffffu, idx, 0);
            if (idx >= n_items) {
              it.idx = -1;
              return;
            }
            if (!decode_item(a, idx, it)) continue;
            if (it.j_end > it.j_begin) return;
            const int nrows = min(kBM * kTiles, it.qlen - it.m0);
            const int osz = a.out_dtype == XFB200_F32 ? 4 : 2;
            const int chunks = D * osz / 16;
            uint8_t* ob = reinterpret_cast<uint8_t*>(a.out);
            const int64_t base = int64_t(it.tb) * a.os.b + int64_t(it.q_row0 + it.m0) * a.os.m + int64_t(it.g) * a.os.g + int64_t(it.h) * a.os.h;
            for (int i = lane; i < nrows * chunks; i += 32) {
              const int r = i / chunks, c = i % chunks;
              *reinterpret_cast<uint4*>(ob + (base + int64_t(r) * a.os.m) * osz + c * 16) = make_uint4(0, 0, 0, 0);
            }
            if (a.lse != nullptr) {
              const int64_t lo = a.seqstart_q != nullptr ? int64_t(it.g) * a.lse_g + int64_t(it.h) * a.lse_h + it.q_row0 + it.m0
                                                         : int64_t(it.b) * a.lse_b + int64_t(it.g) * a.lse_g + int64_t(it.h) * a.lse_h + it.m0;
              for (int r = lane; r < nrows; r += 32) a.lse[lo + r] = -INFINITY;
            }
          }
        };
        Item cur, nxt;
        next_item(cur);
        while (ok) {
          const int slot = seq % kSched;
          if (lane == 0) {
            if (seq >= kSched && !mbar_wait(&bar->sched_empty[slot], (seq / kSched - 1) & 1, abort_flag, budget)) {
              give_up(a, 10);
              ok = false;
            } else {
              bar->sched_item[slot] = cur;
              mbar_arrive(&bar->sched_full[slot]);  // (release: the descriptor is visible to whoever sees the phase)
            }
          }
          ok = __shfl_sync(0xffffffffu, int(ok), 0) != 0;
          ++seq;
          if (!ok || cur.idx < 0) break;
          // Loads are issued in the order in which what they wait for comes free at the end of the previous
          // item: the K tile of the first step (its stage is released one step before the end), Q of tile 0,
          // the V tile of the first step, Q of tile 1, then the remaining steps.  A Q load that waited for
          // the very last QK of the previous item must not hold back the first K tile.
          auto load_q = [&](int t) {
            if (!ok || (t == 0 ? cur.jhi[0] <= cur.jlo[0] : cur.jhi[1] <= cur.jlo[1])) return;
            if (aq[t] > 0 && !mbar_wait(&bar->q_empty[t], (aq[t] - 1) & 1, abort_flag, budget)) {
              give_up(a, 13);
              ok = false;
              return;
            }
            ++aq[t];
            mbar_expect_tx(&bar->q_full[t], L::kQTile);
#pragma unroll
            for (int hf = 0; hf < kHalves; ++hf)
              tma_load_4d(smem + L::kQ + t * L::kQTile + hf * kHalfBytes, &a.tm_q, &bar->q_full[t], hf * 64, cur.head,
                          cur.q_row0 + cur.m0 + t * kBM, cur.tb);
          };
          bool have_next = false;
          for (int j = cur.j_begin; j < cur.j_end; ++j, ++kstep) {
            if (lane == 0 && ok) {
              const int st = kstep % kStages, use = kstep / kStages;
              const int row = cur.k_row0 + cur.n_base + j * kBN;
              if (use > 0 && !mbar_wait(&bar->k_empty[st], (use - 1) & 1, abort_flag, budget)) {
                give_up(a, 11);
                ok = false;
              }
              // (testing aid: the CTA that got the first item leaves out its last key tile, so that the wait for it runs out)
              if (ok && !((a.debug_flags & 1) && cur.idx == 0 && j == cur.j_end - 1)) {
                mbar_expect_tx(&bar->k_full[st], L::kKV);
#pragma unroll
                for (int hf = 0; hf < kHalves; ++hf)
                  tma_load_4d(smem + L::kK + st * L::kKV + hf * kHalfBytes, &a.tm_k, &bar->k_full[st], hf * 64, cur.kv_head, row, cur.tb);
              }
              if (j == cur.j_begin) load_q(0);
              if (ok && use > 0 && !mbar_wait(&bar->v_empty[st], (use - 1) & 1, abort_flag, budget)) {
                give_up(a, 12);
                ok = false;
              }
              if (ok) {
                mbar_expect_tx(&bar->v_full[st], L::kKV);
#pragma unroll
                for (int hf = 0; hf < kHalves; ++hf)
                  tma_load_4d(smem + L::kV + st * L::kKV + hf * kHalfBytes, &a.tm_v, &bar->v_full[st], hf * 64, cur.kv_head, row, cur.tb);
              }
              if (j == cur.j_begin) load_q(1);
            }
            ok = __shfl_sync(0xffffffffu, int(ok), 0) != 0;
            if (!ok) break;
            // The first two steps fit the rings at once; from here on every load waits for a stage to
            // come free, so this is the moment to pull the next item: its latency costs nothing.
            if (!have_next && (j == cur.j_begin + 1 || j == cur.j_end - 1)) {
              next_item(nxt);
              have_next = true;
            }
          }
          if (!ok) break;
          cur = nxt;
        }
        if (!ok) *abort_flag = 1;
      } else if (warp == kMmaWarp0 || warp == kMmaWarp0 + 1) {
        // ================================================= MMA issuer of tile t
        // tcgen05.mma is issued almost synchronously (the queue in front of the
        // tensor pipe is about one instruction deep), so every clock this lane
        // spends on anything else -- a satisfied mbarrier wait alone costs ~90 --
        // is a clock the tensor pipe idles.  Hence one issuing warp per query tile:
        // while one waits for its softmax, the other keeps the pipe fed.
#if !defined(XFB_PST_PROFILE_MMA)
#define XFB_MPROF_DECL(n)
#define XFB_MPROF_LAP(k)
#define XFB_MPROF_COUNT(k)
#define XFB_MPROF_STORE(b, n)
#else
#define XFB_MPROF_DECL(n) XFB_PROF_DECL(n)
#define XFB_MPROF_LAP(k) XFB_PROF_LAP(k)
#define XFB_MPROF_COUNT(k) XFB_PROF_COUNT(k)
#define XFB_MPROF_STORE(b, n) XFB_PROF_STORE(b, n)
#endif
        const int t = warp - kMmaWarp0;
        constexpr uint32_t idesc_qk = umma_idesc(kBM, kBN, kBf16, false, false);
        constexpr uint32_t idesc_pv = umma_idesc(kBM, D, kBf16, false, true);
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
        // the part of P_t V_j over keys [16 kk_lo, 16 kk_hi) of the step; `accumulate` false: its first product overwrites O_t
        auto issue_pv = [&](int v_stage, int kk_lo, int kk_hi, bool accumulate) {
          const uint32_t vl = v_lo0 + v_stage * (L::kKV >> 4);
#pragma unroll
          for (int kk = 0; kk < kBN / 16; ++kk) {
            if (kk < kk_lo || kk >= kk_hi) continue;
            // A = P_t: packed 16-bit pairs, 8 columns of tensor memory per 16 keys
            // (the pairs of keys 0-63 sit in columns 96-127, those of keys 64-127 in columns 64-95)
            umma_ts(tmem_o, tmem_s + (kk < 4 ? 96 + kk * 8 : 32 + kk * 8), desc(vl + ((kk * 16 * 128) >> 4)), idesc_pv, (accumulate || kk > kk_lo) ? 1u : 0u);
          }
        };

        int seq = 0;
        bool ok = true;
        // what this warp needs to know about an item: its key steps, the ones its tile takes part in, the sequence end
        struct Steps {
          int j_begin, j_end, jlo, jhi, n_base, klen;
        };
        Steps cur, nxt;
        auto pop_with_steps = [&](Steps& st) -> int {
          return pop_item(seq, [&](const Item& it) {
            st.j_begin = it.j_begin, st.j_end = it.j_end, st.n_base = it.n_base, st.klen = it.klen;
            st.jlo = t == 0 ? it.jlo[0] : it.jlo[1];
            st.jhi = t == 0 ? it.jhi[0] : it.jhi[1];
          });
        };
        int ci = pop_with_steps(cur);
        if (ci == -2) {
          if (lane == 0) give_up(a, 20);
          ok = false;
        }
        if (ci >= 0) {
          int j = cur.j_begin;
          int ks = 0, kph = 0;  // K stage / phase of step (cur, j)
          int vs = 0, vph = 0;  // V stage / phase of step (cur, j)
          int cnt = 0;          // products of this query tile so far, over all items
          int kq = 0;           // items whose first QK of this tile has been issued
          int kp = 0;           // items whose last PV of this tile has been issued
          int turn_ph = 0;
          XFB_MPROF_DECL(16)
          {
            // the very first step: nothing to multiply by V yet
            const bool act = j >= cur.jlo && j < cur.jhi;
            if (act) ok = mbar_wait(&bar->q_full[t], 0, abort_flag, budget);
            ok = ok && mbar_wait(&bar->k_full[0], 0, abort_flag, budget);
            if (!ok && lane == 0) give_up(a, 21);
            if (ok) {
              tc_fence_after();
              if (lane == 0) {
                if (act) {
                  issue_qk_part(0, 0, D / 16);
                  tc_commit(&bar->s_full[t]);
                  if (j == cur.jhi - 1) tc_commit(&bar->q_empty[t]);
                }
                tc_commit(&bar->k_empty[0]);
                if (t == 1) mbar_arrive(&bar->turn[0]);  // tile 0 opens every iteration
              }
              if (act) ++kq;
            }
          }
          while (ok) {
            XFB_MPROF_LAP(0)
            // ---- the step after (cur, j): same item, or the first step of the next item with steps
            bool has_next = true, same_item = true;
            int nj = j + 1;
            if (nj >= cur.j_end) {
              same_item = false;
              const int ni = pop_with_steps(nxt);
              if (ni == -2) {
                if (lane == 0) give_up(a, 20);
                ok = false;
                break;
              }
              has_next = ni >= 0;
              nj = nxt.j_begin;
            }
            XFB_MPROF_LAP(1)  // pulling the next item
            const int nx_jlo = same_item ? cur.jlo : nxt.jlo, nx_jhi = same_item ? cur.jhi : nxt.jhi;
            const bool act = j >= cur.jlo && j < cur.jhi;
            const bool act_next = has_next && nj >= nx_jlo && nj < nx_jhi;
            const bool first_qk_next = act_next && nj == nx_jlo;
            int ks1 = ks + 1, kph1 = kph;
            if (ks1 == kStages) ks1 = 0, kph1 ^= 1;
            ok = mbar_wait(&bar->v_full[vs], vph, abort_flag, budget);
            if (ok && has_next) ok = mbar_wait(&bar->k_full[ks1], kph1, abort_flag, budget);
            if (!ok) {
              if (lane == 0) give_up(a, 22);
              break;
            }
            // The first QK of the next item needs its Q tile.  If that has not landed yet, the token is not
            // held back for it: the block ends after the PV and the QK follows out of turn (late_qk).
            XFB_MPROF_LAP(2)  // waits for V and the next K
            bool late_qk = false;
            if (first_qk_next) {
              int ready = 0;
              if (lane == 0) ready = mbar_try_wait(&bar->q_full[t], kq & 1) ? 1 : 0;
              late_qk = __shfl_sync(0xffffffffu, ready, 0) == 0;
            }
            const int n0 = cur.n_base + j * kBN;
            if (n0 + kBN > cur.klen) {
              // V rows past the end of the sequence may hold anything; P is 0 there.
              // Both MMA warps write the same zeros: no ordering between them is needed.
              const int first = max(cur.klen - n0, 0);
              uint8_t* vt = smem + L::kV + vs * L::kKV;
              for (int hf = 0; hf < kHalves; ++hf)
                for (int i = first * 8 + lane; i < kBN * 8; i += 32) *reinterpret_cast<uint4*>(vt + hf * kHalfBytes + i * 16) = make_uint4(0, 0, 0, 0);
              fence_proxy_async_smem();
              __syncwarp();
            }
            // If both warps issued at will, their MMAs would interleave one by one,
            // both tiles would finish together and both softmaxes would run at the
            // same time with the tensor pipe idle.  Blocks (PV, next QK) are
            // therefore issued alternately, which keeps the two tiles half a period
            // apart; the token is passed a few MMAs before the end of a block so
            // that the hand-over latency is hidden.  The token is waited for before
            // P: it normally arrives first, and even a satisfied wait costs ~90 clocks
            // that would otherwise sit between the softmax and its PV.
            ok = mbar_wait(&bar->turn[t], turn_ph, abort_flag, budget);
            turn_ph ^= 1;
            if (!ok) {
              if (lane == 0) give_up(a, 25 + t);
              break;
            }
            XFB_MPROF_LAP(4)  // wait for the token
            if (act) {
              // The probabilities of keys 64-127 are stored first: their half of the product runs while the
              // softmax is still busy with keys 0-63.
              ok = mbar_wait(&bar->p_half[t], cnt & 1, abort_flag, budget);
              // the first PV of an item overwrites O_t: the output warps must have read the previous one
              if (ok && j == cur.jlo && kp > 0) ok = mbar_wait(&bar->o_empty[t], (kp - 1) & 1, abort_flag, budget);
              if (ok) {
                tc_fence_after();
                if (lane == 0) issue_pv(vs, kBN / 32, kBN / 16, j > cur.jlo);
                ok = mbar_wait(&bar->p_full[t], cnt & 1, abort_flag, budget);
              }
              if (!ok) {
                if (lane == 0) give_up(a, 23 + t);
                break;
              }
              tc_fence_after();
            }
            XFB_MPROF_LAP(3)  // V tail, wait for P (and for the output warps at the first PV of an item)
            if (lane == 0) {
              if (act) {
                issue_pv(vs, 0, kBN / 32, true);
                if (j == cur.jhi - 1) tc_commit(&bar->o_full[t]);
              }
              tc_commit(&bar->v_empty[vs]);
              if (act_next && !late_qk) {
                issue_qk_part(ks1, 0, D / 32);
                mbar_arrive(&bar->turn[1 - t]);
                issue_qk_part(ks1, D / 32, D / 16);
                tc_commit(&bar->s_full[t]);
                if (nj == nx_jhi - 1) tc_commit(&bar->q_empty[t]);
              } else {
                mbar_arrive(&bar->turn[1 - t]);
              }
              if (has_next && !late_qk) tc_commit(&bar->k_empty[ks1]);
            }
            XFB_MPROF_LAP(5)  // issuing the block
            if (late_qk) {
              XFB_MPROF_COUNT(8)
              ok = mbar_wait(&bar->k_full[ks1], kph1, abort_flag, budget);
              if (ok && first_qk_next) ok = mbar_wait(&bar->q_full[t], kq & 1, abort_flag, budget);
              if (!ok) {
                if (lane == 0) give_up(a, 27 + t);
                break;
              }
              tc_fence_after();
              if (lane == 0) {
                issue_qk_part(ks1, 0, D / 16);
                tc_commit(&bar->s_full[t]);
                if (nj == nx_jhi - 1) tc_commit(&bar->q_empty[t]);
                tc_commit(&bar->k_empty[ks1]);
              }
            }
            XFB_MPROF_LAP(6)  // a QK issued out of turn
            XFB_MPROF_COUNT(7)
            if (act) {
              ++cnt;
              if (j == cur.jhi - 1) ++kp;
            }
            if (first_qk_next) ++kq;
            if (!has_next) break;
            if (!same_item) cur = nxt;
            j = nj;
            ks = ks1, kph = kph1;
            if (++vs == kStages) vs = 0, vph ^= 1;
          }
          XFB_MPROF_STORE(64 + t * 16, 16)
        }
        if (!ok) *abort_flag = 1;
      }
    } else if (warp >= kOutWarp0) {
      asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsOut));
      // ================================================================ output
      const int row = (warp & 3) * 32 + lane;  // TMEM lane == row inside the tile
      const uint32_t lane_sel = uint32_t((warp & 3) * 32) << 16;
      int seq = 0;
      int ko[kTiles] = {0, 0};  // items in which tile t took part so far
      bool ok = true;
      while (ok) {
        Item it;
        const int idx = pop_item(seq, [&](const Item& d) { it = d; });
        if (idx < 0) {
          if (idx == -2) {
            give_up(a, 40);
            ok = false;
          }
          break;
        }
#pragma unroll
        for (int t = 0; t < kTiles; ++t) {
          const int i_loc = it.m0 + t * kBM + row;
          const bool valid_row = i_loc < it.qlen;
          const bool active = it.jhi[t] > it.jlo[t];
          if (!active && it.m0 + t * kBM >= it.qlen) continue;  // no row of this tile exists
          float m_run = -INFINITY, l_run = 0.f;
          const uint32_t tmem_o = tmem + 256 + t * 128 + lane_sel;
          if (active) {
            const int k = ko[t]++;
            ok = mbar_wait(&bar->stats_full[t], k & 1, abort_flag, budget);
            if (ok) {
              const float2 st = stats[t * kBM + row];
              m_run = st.x, l_run = st.y;
              mbar_arrive(&bar->stats_empty[t]);
              ok = mbar_wait(&bar->o_full[t], k & 1, abort_flag, budget);
            }
            if (!ok) {
              give_up(a, 41 + t);
              break;
            }
            tc_fence_after();
          }
          const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
          const int64_t o_off = int64_t(it.tb) * a.os.b + int64_t(it.q_row0 + i_loc) * a.os.m + int64_t(it.g) * a.os.g + int64_t(it.h) * a.os.h;
#pragma unroll
          for (int cblk = 0; cblk < D / 32; ++cblk) {
            uint32_t orr[32];
            if (active) {
              XFB_TMEM_LD_32(tmem_o + cblk * 32, orr);
              XFB_TMEM_WAIT_LD_32(orr);
              if (cblk == D / 32 - 1) {
                // O_t is in registers: the next item's first PV may overwrite it
                tc_fence_before();
                mbar_arrive(&bar->o_empty[t]);
              }
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
            const int64_t lo = a.seqstart_q != nullptr ? int64_t(it.g) * a.lse_g + int64_t(it.h) * a.lse_h + it.q_row0 + i_loc
                                                       : int64_t(it.b) * a.lse_b + int64_t(it.g) * a.lse_g + int64_t(it.h) * a.lse_h + i_loc;
            a.lse[lo] = lse;
          }
        }
      }
      if (!ok) *abort_flag = 1;
      tc_fence_before();
    } else {
      asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsSoftmax));
      // ================================================================ softmax
      const int t = warp >> 2;                  // query tile of this warpgroup
      const int row = (warp & 3) * 32 + lane;   // TMEM lane == row inside the tile
      const uint32_t lane_sel = uint32_t((warp & 3) * 32) << 16;
      const uint32_t tmem_s = tmem + t * 128 + lane_sel;
      const uint32_t tmem_o = tmem + 256 + t * 128 + lane_sel;
      const float sl2 = a.scale_log2;
      const uint64_t sc2 = f2_pack(sl2, sl2);
      int seq = 0;
      int cnt = 0;  // steps of this tile so far, over all items
      int ka = 0;   // items in which this tile took part so far
      bool ok = true;
      XFB_PROF_DECL(16)

      // visibility of the 32 columns starting at key `col0` for this thread's row: hidden scores become -inf
      int col_lo = 0, col_hi = 0;
      auto mask_chunk = [&](float* sc, int col0) {
        // one bit per column, then a test and a select per score
        const int hr = col_hi - col0, lr = col_lo - col0;
        const uint32_t below_hi = hr >= 32 ? 0xffffffffu : (hr <= 0 ? 0u : (1u << hr) - 1u);
        const uint32_t from_lo = lr <= 0 ? 0xffffffffu : (lr >= 32 ? 0u : ~((1u << lr) - 1u));
        const uint32_t vis = below_hi & from_lo;
#pragma unroll
        for (int c = 0; c < 32; ++c) sc[c] = (vis & (1u << c)) != 0u ? sc[c] : -INFINITY;
      };
      auto chunk_max = [](const float* sc) -> float {
        float m0 = fmax3(sc[0], sc[1], sc[2]), m1 = fmax3(sc[3], sc[4], sc[5]), m2 = fmax3(sc[6], sc[7], sc[8]), m3 = fmax3(sc[9], sc[10], sc[11]);
        m0 = fmax3(m0, sc[12], sc[13]), m1 = fmax3(m1, sc[14], sc[15]), m2 = fmax3(m2, sc[16], sc[17]), m3 = fmax3(m3, sc[18], sc[19]);
        m0 = fmax3(m0, sc[20], sc[21]), m1 = fmax3(m1, sc[22], sc[23]), m2 = fmax3(m2, sc[24], sc[25]), m3 = fmax3(m3, sc[26], sc[27]);
        m0 = fmax3(m0, sc[28], sc[29]), m1 = fmax3(m1, sc[30], sc[31]);
        return fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
      };
      // 32 score columns -> 16 packed probability pairs against the maximum -m (nm2 = (-m, -m)), summed into
      // sum2 and stored to the 16 columns of S_t that start at `col`
      auto exp_store = [&](const uint32_t* sr, int col, uint64_t nm2, uint64_t (&sum2)[4]) {
        uint32_t pr[16];
        // (blocks of 16 independent elements: all FMAs, then all exp2, then the sums and packs -- a lone warp per
        // scheduler hides no latency by switching warps, the instruction stream has to)
#pragma unroll
        for (int h = 0; h < 32; h += 16) {
          float e[16];
#pragma unroll
          for (int i = 0; i < 16; i += 2)
            f2_unpack(ffma2(f2_pack(__uint_as_float(sr[h + i]), __uint_as_float(sr[h + i + 1])), sc2, nm2), e[i], e[i + 1]);
#pragma unroll
          for (int i = 0; i < 16; ++i) e[i] = fast_exp2(e[i]);
#pragma unroll
          for (int i = 0; i < 16; i += 2) {
            sum2[(i / 2) & 3] = fadd2(sum2[(i / 2) & 3], f2_pack(e[i], e[i + 1]));
            pr[(h + i) / 2] = pack_pair<kBf16>(e[i], e[i + 1]);
          }
        }
        XFB_TMEM_ST_16(tmem_s + col, pr);
      };
      // O_t *= alpha (per row), through registers
      auto rescale_o = [&](float alpha) {
        const uint64_t al2 = f2_pack(alpha, alpha);
#pragma unroll
        for (int cblk = 0; cblk < D / 32; ++cblk) {
          uint32_t orr[32];
          XFB_TMEM_LD_32(tmem_o + cblk * 32, orr);
          XFB_TMEM_WAIT_LD_32(orr);
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            float x0, x1;
            f2_unpack(fmul2(f2_pack(__uint_as_float(orr[i]), __uint_as_float(orr[i + 1])), al2), x0, x1);
            orr[i] = __float_as_uint(x0);
            orr[i + 1] = __float_as_uint(x1);
          }
          XFB_TMEM_ST_32(tmem_o + cblk * 32, orr);
        }
        tc_wait_st();
      };

      while (ok) {
        struct {
          int jlo, jhi, m0, shift, shift2, n_base, klen, qlen;
          int64_t bias_off;  // of the item's (batch, head) in the additive bias, in elements
        } it;
        const int idx = pop_item(seq, [&](const Item& d) {
          it.jlo = t == 0 ? d.jlo[0] : d.jlo[1];
          it.jhi = t == 0 ? d.jhi[0] : d.jhi[1];
          it.m0 = d.m0, it.shift = d.shift, it.shift2 = d.shift2, it.n_base = d.n_base, it.klen = d.klen, it.qlen = d.qlen;
          it.bias_off = a.bias != nullptr ? int64_t(d.b) * a.bias_b + int64_t(d.g) * a.bias_g + int64_t(d.h) * a.bias_h : 0;
        });
        if (idx < 0) {
          if (idx == -2) {
            give_up(a, 30);
            ok = false;
          }
          break;
        }
        const int jlo = it.jlo, jhi = it.jhi;
        if (jhi <= jlo) continue;  // this tile sees no key in this item
        const int mt0 = it.m0 + t * kBM;
        const int i_loc = mt0 + row;
        const bool causal = a.window_right >= 0;
        col_hi = causal ? min(it.klen, i_loc + it.shift + a.window_right + 1) : it.klen;
        col_lo = a.window_left >= 0 ? i_loc + it.shift - a.window_left : 0;
        // this thread's row of the additive bias (dense batches only), or null
        const uint8_t* bias_row = nullptr;
        if (a.bias != nullptr && i_loc < it.qlen)
          bias_row = reinterpret_cast<const uint8_t*>(a.bias) + (it.bias_off + int64_t(i_loc) * a.bias_m) * (a.bias_dtype == XFB200_F32 ? 4 : 2);
        // m_run: the reference maximum the probabilities and O_t are taken against (log2 units; at most 2^8 below
        // the true running maximum); l_run: the row sum against m_run
        float m_run = -INFINITY, l_run = 0.f;

        XFB_PROF_LAP(0)  // between items: statistics hand-over, next descriptor
        for (int j = jlo; j < jhi; ++j, ++cnt) {
          int n0 = it.n_base + j * kBN;
          int klen = it.klen, shift = it.shift;
          if (a.kv_split > 0) {
            // which of the two key ranges this step lies in: positions and limits are relative to that range
            const bool second = n0 >= a.kv_split;
            klen = second ? it.klen - a.kv_split : a.kv_split;
            shift = second ? it.shift2 : it.shift;
            n0 -= second ? a.kv_split : 0;
            col_hi = min(klen, i_loc + shift + 1);
          }
          const bool need_mask = (n0 + kBN > klen) || (causal && n0 + kBN - 1 > mt0 + shift + a.window_right) ||
                                 (a.window_left >= 0 && n0 < mt0 + kBM - 1 + shift - a.window_left);
          ok = mbar_wait(&bar->s_full[t], cnt & 1, abort_flag, budget);
          XFB_PROF_LAP(1)  // wait for the scores
          if (!ok) {
            give_up(a, 31 + t);
            break;
          }
          tc_fence_after();
          if (a.bias != nullptr) {  // (warp-uniform: the tensor-memory accesses below are warp-wide)
            // An additive bias is folded into the scores where they lie (as bias / scale, so that the step's
            // scale * log2 e applies to the sum); rows past the end of the queries and keys past the end of the
            // keys are left alone (the former are never written, the latter are masked below).
            uint32_t sm[32];
#pragma unroll 1
            for (int c = 0; c < kBN / 32; ++c) {
              const int col0 = n0 + c * 32;
              XFB_TMEM_LD_32(tmem_s + c * 32, sm);
              XFB_TMEM_WAIT_LD_32(sm);
#pragma unroll
              for (int i = 0; i < 32; ++i) {
                float bv = 0.f;
                if (bias_row != nullptr && col0 + i < klen) {
                  if (a.bias_dtype == XFB200_F32) bv = reinterpret_cast<const float*>(bias_row)[col0 + i];
                  else if (a.bias_dtype == XFB200_BF16) bv = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(bias_row)[col0 + i]);
                  else bv = __half2float(reinterpret_cast<const __half*>(bias_row)[col0 + i]);
                }
                sm[i] = __float_as_uint(fmaf(bv, a.inv_scale, __uint_as_float(sm[i])));
              }
              XFB_TMEM_ST_32(tmem_s + c * 32, sm);
              tc_wait_st();  // (the registers are written again in the next round)
            }
          }
          if (need_mask) {
            // Diagonal and ragged tiles: hidden scores are turned into -inf where they lie, in tensor memory, by this
            // small loop; the step itself then is the same code for every tile (one copy of it in the instruction
            // cache).  The rows of a warp are consecutive and both limits grow with the row, so the limits of the
            // first and the last row tell which chunks are fully visible to the warp (left alone) or fully hidden
            // (overwritten without being read).
            const int hi_first = __shfl_sync(0xffffffffu, col_hi, 0), hi_last = __shfl_sync(0xffffffffu, col_hi, 31);
            const int lo_first = __shfl_sync(0xffffffffu, col_lo, 0), lo_last = __shfl_sync(0xffffffffu, col_lo, 31);
            uint32_t sm[32], ninf[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) ninf[i] = 0xff800000u;
#pragma unroll 1
            for (int c = 0; c < kBN / 32; ++c) {
              const int col0 = n0 + c * 32;
              if (col0 >= lo_last && col0 + 32 <= hi_first) continue;  // every row of the warp sees the whole chunk
              if (col0 >= hi_last || col0 + 32 <= lo_first) {
                // no row of the warp sees any of it (the same eight registers serve every store: nothing to wait for)
#pragma unroll
                for (int i = 0; i < 4; ++i) XFB_TMEM_ST_8(tmem_s + c * 32 + i * 8, ninf);
              } else {
                tc_wait_st();  // (an earlier round's store may still be reading the registers)
                XFB_TMEM_LD_32(tmem_s + c * 32, sm);
                XFB_TMEM_WAIT_LD_32(sm);
                mask_chunk(reinterpret_cast<float*>(sm), col0);
                XFB_TMEM_ST_32(tmem_s + c * 32, sm);
              }
            }
            tc_wait_st();
            XFB_PROF_COUNT(5)
            XFB_PROF_LAP(3)  // the visibility test
          }
          {
            uint32_t sa[32], sb[32];
            // ---- first pass: the maximum of the scores
            XFB_TMEM_LD_32(tmem_s, sa);
            XFB_TMEM_LD_32(tmem_s + 32, sb);
            XFB_TMEM_WAIT_LD_32(sa);
            XFB_TMEM_WAIT_LD_32(sb);
            float mx = fmaxf(chunk_max(reinterpret_cast<float*>(sa)), chunk_max(reinterpret_cast<float*>(sb)));
            XFB_TMEM_LD_32(tmem_s + 64, sa);
            XFB_TMEM_LD_32(tmem_s + 96, sb);
            XFB_TMEM_WAIT_LD_32(sa);
            XFB_TMEM_WAIT_LD_32(sb);
            mx = fmaxf(mx, fmaxf(chunk_max(reinterpret_cast<float*>(sa)), chunk_max(reinterpret_cast<float*>(sb))));
            const float ms = mx * sl2;  // scale > 0 (host guarantees)
            // ---- the reference follows the maximum only when it has to (a fresh row: from -inf).  QK(t,j) completing
            // implies PV(t,j-1) completed: O_t is quiescent here.
            if (__any_sync(0xffffffffu, ms > m_run + kRescaleThreshold)) {
              XFB_PROF_COUNT(7)
              const float m_new = ms > m_run + kRescaleThreshold ? ms : m_run;
              const float alpha = m_new == m_run ? 1.f : (m_run == -INFINITY ? 0.f : fast_exp2(m_run - m_new));
              if (j > jlo) rescale_o(alpha);
              l_run *= alpha;
              m_run = m_new;
            }
            // ---- second pass: probabilities.  Keys 64-127 are in registers; keys 0-63 come back behind them.
            const float m_use = m_run == -INFINITY ? 0.f : m_run;
            const uint64_t nm2 = f2_pack(-m_use, -m_use);
            uint64_t sum2[4] = {f2_pack(0.f, 0.f), f2_pack(0.f, 0.f), f2_pack(0.f, 0.f), f2_pack(0.f, 0.f)};
            exp_store(sa, 64, nm2, sum2);
            XFB_TMEM_LD_32(tmem_s, sa);
            exp_store(sb, 80, nm2, sum2);
            XFB_TMEM_LD_32(tmem_s + 32, sb);
            tc_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bar->p_half[t]);
            XFB_TMEM_WAIT_LD_32(sa);
            XFB_TMEM_WAIT_LD_32(sb);
            exp_store(sa, 96, nm2, sum2);
            exp_store(sb, 112, nm2, sum2);
            {
              float x0, x1, y0, y1;
              f2_unpack(fadd2(sum2[0], sum2[1]), x0, x1);
              f2_unpack(fadd2(sum2[2], sum2[3]), y0, y1);
              l_run += (x0 + x1) + (y0 + y1);
            }
          }
          XFB_PROF_LAP(2)  // the step proper
          XFB_PROF_COUNT(6)
          tc_wait_st();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&bar->p_full[t]);
          XFB_PROF_LAP(4)  // storing P
        }
        if (!ok) break;
        // hand the row's statistics to the output warps
        if (ka > 0 && !mbar_wait(&bar->stats_empty[t], (ka - 1) & 1, abort_flag, budget)) {
          give_up(a, 33 + t);
          ok = false;
          break;
        }
        ++ka;
        stats[t * kBM + row] = make_float2(m_run, l_run);
        mbar_arrive(&bar->stats_full[t]);
      }
      if (!ok) *abort_flag = 1;
      tc_fence_before();
      XFB_PROF_STORE(warp * 8, 8)
    }

    __syncthreads();
    if (warp == kMmaWarp0) {
      tc_fence_after();
      tmem_dealloc(tmem, 512);
    }
  }

  // The last CTA to finish puts the work counters back to zero for the next launch.
  if (threadIdx.x == 0) {
    __threadfence();
    const int done = atomicAdd(a.counters + 1, 1);
    if (done == int(gridDim.x) - 1) {
      atomicExch(a.counters, 0);
      atomicExch(a.counters + 1, 0);
    }
  }
}

template <int D, bool kBf16>
static int launch_t(const Sm100Args& a, cudaStream_t stream) {
  auto kern = prefill_sm100_persist_kernel<D, kBf16>;
  constexpr int smem = Smem<D>::kTotal;
  static bool configured[kMaxDevices] = {false};  // the attribute belongs to the device's context
  if (first_use_on_device(configured)) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return cuda_fail("prefill(sm100, persistent): cudaFuncSetAttribute", e);
  }
  const int64_t items = int64_t(a.groups) * a.heads_per_group * a.batch * a.q_tiles;
  if (items > 0x3fffffff) return set_error(XFB200_E_UNSUPPORTED, "prefill: too many blocks of query rows");
  int sms = sm_count() - a.sm_margin;
  if (sms < 1) sms = 1;
  const unsigned grid = unsigned(items < sms ? items : sms);
  kern<<<grid, kThreads, smem, stream>>>(a);
  return check_launch("prefill_sm100_persist_kernel");
}

}  // namespace pst

#ifdef XFB_PST_PROFILE
extern "C" __attribute__((visibility("default"))) int xfb200_debug_read_prefill_profile(long long* out, int clear) {
  cudaDeviceSynchronize();
  cudaError_t e = cudaMemcpyFromSymbol(out, pst::g_prof, sizeof(long long) * 160 * 96);
  if (e == cudaSuccess && clear) {
    static long long zeros[160 * 96] = {0};
    e = cudaMemcpyToSymbol(pst::g_prof, zeros, sizeof(zeros));
  }
  return e == cudaSuccess ? 0 : -3;
}
#endif

int prefill_sm100_persist_launch(Sm100Args a, int head_dim, bool bf16, cudaStream_t stream) {
  if (head_dim == 128) return bf16 ? pst::launch_t<128, true>(a, stream) : pst::launch_t<128, false>(a, stream);
  return bf16 ? pst::launch_t<64, true>(a, stream) : pst::launch_t<64, false>(a, stream);
}

}  // namespace xfb
