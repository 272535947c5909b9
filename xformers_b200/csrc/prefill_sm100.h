// Kernel arguments shared by the tcgen05 prefill kernels.
#pragma once

#include <cuda.h>

#include "internal.h"

namespace xfb {

struct Sm100Args {
  CUtensorMap tm_q, tm_k, tm_v;
  void* out;
  float* lse;
  const int32_t* seqstart_q;
  const int32_t* seqstart_k;
  const int32_t* seqlen_k;
  int32_t* status;    // [0] first code a launch gave up with, [1] epoch of that launch
  int32_t* counters;  // persistent kernel: [0] next work item, [1] CTAs that have finished; zero between launches
  int32_t batch, mq, mkv, groups, heads_per_group;
  int32_t kv_h_is_broadcast;  // K/V head stride 0: KV head index is g only
  xfb200_strides os;
  int64_t lse_b, lse_g, lse_h;
  // query i of a block sees key j iff i + shift - window_left <= j <= i + shift + window_right, each bound only
  // when it is >= 0; shift = (bottom_right ? keys - queries of the block : 0) - kv_offset
  int32_t bottom_right, kv_offset, window_left, window_right;
  // two key ranges in one tensor (persistent kernel, dense causal only): rows [0, kv_split) of k/v start at global key
  // kv_offset, rows from kv_split on at kv_offset2; 0 = one range
  int32_t kv_split, kv_offset2;
  int32_t sm_margin;  // persistent kernel: SMs left free for kernels of other streams
  int32_t heads_per_wave;  // persistent kernel: (batch, head) pairs whose row blocks are handed out together (>= 1)
  int32_t out_dtype;
  float scale_log2;
  int32_t q_tiles;  // blocks of 256 query rows per sequence (static bound)
  uint32_t epoch;   // differs from launch to launch, never 0
  int32_t debug_flags;
  long long wait_budget;  // SM clocks after which a wait gives up
  // additive bias (persistent kernel, dense batches): element strides of [batch, G, H, mq, mkv], unit stride on mkv;
  // the kernel adds bias / scale to q k^T, so that the softmax sees q k^T * scale + bias
  const void* bias;
  int32_t bias_dtype;
  float inv_scale;
  int64_t bias_b, bias_g, bias_h, bias_m;
};

// One CTA per block of 256 query rows (two 128-row tiles sharing every K/V tile), 128-key steps.
int prefill_sm100_m256_launch(Sm100Args a, int head_dim, bool bf16, cudaStream_t stream);
// The same tile shape run by one persistent CTA per SM that pulls blocks from a work counter,
// with the output of a block written by its own warps while the next block computes.
int prefill_sm100_persist_launch(Sm100Args a, int head_dim, bool bf16, cudaStream_t stream);

}  // namespace xfb
