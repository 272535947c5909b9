// Host side of the tcgen05 prefill kernels: what they cover, their tensor maps and arguments.
#include <cuda.h>

#include "internal.h"
#include "prefill_sm100.h"

namespace xfb {

constexpr long long kDefaultWaitBudgetCycles = 400000000LL;  // ~0.2 s of SM clock

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
  rc = make_map(&a.tm_k, p->k, p->dtype, D, khc, khs, k_rows, p->k_strides.m, nb, p->k_strides.b, "k");
  if (rc) return rc;
  rc = make_map(&a.tm_v, p->v, p->dtype, D, khc, vhs, k_rows, p->v_strides.m, nb, p->v_strides.b, "v");
  if (rc) return rc;
  a.out = p->out, a.lse = p->lse;
  a.seqstart_q = p->seqstart_q, a.seqstart_k = p->seqstart_k, a.seqlen_k = p->seqlen_k;
  int32_t* words = device_words();
  if (words == nullptr) return set_error(XFB200_E_CUDA, "prefill: cannot resolve the device status words");
  a.status = words + kWordPrefillStatus;
  a.epoch = next_launch_epoch();
  // launches that may overlap on the GPU (several streams) must not share a work counter: hand the slots out in turn
  a.counters = words + kWordPrefillCounters + 2 * int(a.epoch % uint32_t(kPrefillCounterSlots));
  a.batch = p->batch, a.mq = p->mq, a.mkv = p->mkv, a.groups = G, a.heads_per_group = H;
  a.kv_h_is_broadcast = kbc ? 1 : 0;
  a.os = p->o_strides;
  a.lse_b = p->lse_stride_b, a.lse_g = p->lse_stride_g, a.lse_h = p->lse_stride_h;
  a.bottom_right = p->mask_type >= XFB200_MASK_CAUSAL_BOTTOM_RIGHT ? 1 : 0;
  a.kv_offset = p->kv_offset, a.window_left = p->window_left, a.out_dtype = p->out_dtype;
  a.window_right = p->mask_type == XFB200_MASK_NONE ? -1 : p->mask_type == XFB200_MASK_LOCAL_BOTTOM_RIGHT ? p->window_right : 0;
  a.kv_split = p->kv_split, a.kv_offset2 = p->kv_offset2;
  a.sm_margin = p->sm_margin > 0 ? p->sm_margin : 0;
  {
    // Work items are handed out heaviest first inside groups of (batch, head) pairs whose keys and values fit the L2
    // together (measured on 4 x 4096 x 32 heads: 945 -> 1020 TFLOP/s causal with 16 or 32 heads per group against all
    // 128 at once, 990 -> 1140-1200 without a mask with 8; on 16 packed sequences of 256..4096 tokens 872 with 64,
    // 900 with 128, 830-840 with 8..32).  Causal launches take larger groups: their items differ in weight, and the
    // more of them run side by side the shorter the tail of a group.
    const double keys = varlen ? double(p->mkv) / double(p->batch > 0 ? p->batch : 1) : double(p->mkv);
    const double per_head = 2.0 * keys * D * 2.0 / (kbc ? H : 1);  // K and V, 2 bytes per element; a GQA group shares them
    const double budget = (p->mask_type == XFB200_MASK_NONE ? 16.0 : 64.0) * 1024.0 * 1024.0;
    int hpw = 1;
    while (hpw < 256 && 2.0 * hpw * per_head <= budget) hpw *= 2;
    if (kbc && hpw < H) hpw = H;  // the heads of a GQA group read the same keys: keep them together
    a.heads_per_wave = hpw;
  }
  a.scale_log2 = p->scale * 1.4426950408889634f;
  a.q_tiles = (p->mq + 255) / 256;
  a.debug_flags = p->debug_flags;
  a.wait_budget = p->wait_budget_kcycles > 0 ? 1000LL * p->wait_budget_kcycles : kDefaultWaitBudgetCycles;
  a.bias = p->bias, a.bias_dtype = p->bias_dtype, a.inv_scale = 1.f / p->scale;
  a.bias_b = p->bias_stride_b, a.bias_g = p->bias_stride_g, a.bias_h = p->bias_stride_h, a.bias_m = p->bias_stride_m;
  const bool bf16 = p->dtype == XFB200_BF16;
  if (p->kernel_path == XFB200_PREFILL_TCGEN05_CTA) {
    if (p->kv_split > 0) return set_error(XFB200_E_UNSUPPORTED, "prefill: two key ranges in one call need the persistent kernel");
    if (p->bias != nullptr) return set_error(XFB200_E_UNSUPPORTED, "prefill: an additive bias needs the persistent or the mma.sync kernel");
    return prefill_sm100_m256_launch(a, D, bf16, stream);
  }
  return prefill_sm100_persist_launch(a, D, bf16, stream);
}

}  // namespace xfb

