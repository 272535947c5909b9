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
  int32_t* status;
  int32_t batch, mq, mkv, groups, heads_per_group;
  int32_t kv_h_is_broadcast;  // K/V head stride 0: KV head index is g only
  xfb200_strides os;
  int64_t lse_b, lse_g, lse_h;
  int32_t mask_type, kv_offset, window_left, out_dtype;
  float scale_log2;
  int32_t q_tiles;
};

// 256 query rows per CTA (two 128-row tiles sharing every K/V tile), 128-key steps, one score buffer per tile.
int prefill_sm100_m256_launch(Sm100Args a, int head_dim, bool bf16, cudaStream_t stream);
// The same CTA shape with 64-key steps and two score buffers per tile.
int prefill_sm100_s64_launch(Sm100Args a, int head_dim, bool bf16, cudaStream_t stream);

// 0 = default kernel choice; 3 = the 128-rows-per-CTA kernel, 4 = 256 rows with 128-key steps, 5 = 256 rows with 64-key steps (testing knobs).
int prefill_path_override();

}  // namespace xfb
