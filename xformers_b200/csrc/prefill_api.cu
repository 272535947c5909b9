// xfb200_prefill_forward: host-side validation and kernel selection.
#include "internal.h"

extern "C" int xfb200_prefill_forward(const xfb200_prefill_params* p, void* stream) {
  using namespace xfb;
  if (p == nullptr) return set_error(XFB200_E_INVALID, "prefill: null params");
  if (p->dtype != XFB200_BF16 && p->dtype != XFB200_F16) return set_error(XFB200_E_INVALID, "prefill: dtype must be bf16 or f16");
  if (p->out_dtype != XFB200_BF16 && p->out_dtype != XFB200_F16 && p->out_dtype != XFB200_F32)
    return set_error(XFB200_E_INVALID, "prefill: bad out_dtype %d", p->out_dtype);
  if (p->batch < 0 || p->mq < 0 || p->mkv < 0 || p->groups < 1 || p->heads_per_group < 1)
    return set_error(XFB200_E_INVALID, "prefill: bad extents");
  if (p->head_dim < 8 || p->head_dim % 8 != 0 || p->head_dim > 256)
    return set_error(XFB200_E_UNSUPPORTED, "prefill: head_dim %d (need a multiple of 8 in [8, 256])", p->head_dim);
  if (p->batch == 0 || p->mq == 0 || p->total_q == 0) return XFB200_OK;  // empty output
  if (p->q == nullptr || p->out == nullptr) return set_error(XFB200_E_INVALID, "prefill: null q/out");
  if (p->mkv > 0 && (p->k == nullptr || p->v == nullptr)) return set_error(XFB200_E_INVALID, "prefill: null k/v");
  if ((p->seqstart_q == nullptr) != (p->seqstart_k == nullptr))
    return set_error(XFB200_E_INVALID, "prefill: seqstart_q and seqstart_k go together");
  if (p->seqlen_k != nullptr && p->seqstart_k == nullptr) return set_error(XFB200_E_INVALID, "prefill: seqlen_k needs seqstart_k");
  if (p->mask_type < 0 || p->mask_type > XFB200_MASK_LOCAL_BOTTOM_RIGHT) return set_error(XFB200_E_INVALID, "prefill: bad mask_type %d", p->mask_type);
  if (p->mask_type >= XFB200_MASK_CAUSAL_BOTTOM_RIGHT && p->kv_offset != 0)
    return set_error(XFB200_E_INVALID, "prefill: kv_offset needs the top-left causal mask");
  if (p->mask_type == XFB200_MASK_LOCAL_BOTTOM_RIGHT && (p->window_left < 0 || p->window_right < 0))
    return set_error(XFB200_E_INVALID, "prefill: the local mask needs window_left >= 0 and window_right >= 0");
  if (p->kernel_path != XFB200_PREFILL_AUTO && p->kernel_path != XFB200_PREFILL_MMA_SYNC && p->kernel_path != XFB200_PREFILL_TCGEN05 &&
      p->kernel_path != XFB200_PREFILL_TCGEN05_CTA && p->kernel_path != XFB200_PREFILL_TCGEN05_PERSISTENT)
    return set_error(XFB200_E_INVALID, "prefill: bad kernel_path %d", p->kernel_path);
  if (p->window_left >= 0 && p->mask_type == XFB200_MASK_NONE)
    return set_error(XFB200_E_UNSUPPORTED, "prefill: a left window without a causal mask");
  // 16-byte vector loads / cp.async need aligned rows
  auto al8 = [](const xfb200_strides& s) { return s.b % 8 == 0 && s.m % 8 == 0 && s.g % 8 == 0 && s.h % 8 == 0; };
  if (!al8(p->q_strides) || !al8(p->k_strides) || !al8(p->v_strides))
    return set_error(XFB200_E_INVALID, "prefill: q/k/v strides must be multiples of 8 elements (16 bytes)");
  if ((reinterpret_cast<uintptr_t>(p->q) | reinterpret_cast<uintptr_t>(p->k) | reinterpret_cast<uintptr_t>(p->v)) & 15)
    return set_error(XFB200_E_INVALID, "prefill: q/k/v must be 16-byte aligned");
  const int osz = p->out_dtype == XFB200_F32 ? 4 : 2;
  if (((p->o_strides.b | p->o_strides.m | p->o_strides.g | p->o_strides.h) * osz) % 8 || (reinterpret_cast<uintptr_t>(p->out) & 7))
    return set_error(XFB200_E_INVALID, "prefill: out rows must be 8-byte aligned");

  if (p->kv_split != 0) {
    if (p->kv_split < 0 || p->kv_split >= p->mkv || p->kv_split % 128 != 0)
      return set_error(XFB200_E_INVALID, "prefill: kv_split %d must be a multiple of 128 inside (0, mkv)", p->kv_split);
    if (p->mask_type != XFB200_MASK_CAUSAL_TOP_LEFT || p->window_left >= 0 || p->seqstart_q != nullptr || p->bias != nullptr)
      return set_error(XFB200_E_UNSUPPORTED, "prefill: two key ranges need dense inputs and the plain top-left causal mask");
    if (int64_t(p->kv_offset2) < int64_t(p->kv_offset) + p->kv_split)
      return set_error(XFB200_E_INVALID, "prefill: the second key range must lie behind the first (kv_offset2 >= kv_offset + kv_split)");
  }

  if (p->bias != nullptr) {
    if (p->seqstart_q != nullptr) return set_error(XFB200_E_UNSUPPORTED, "prefill: an additive bias with concatenated sequences");
    if (p->bias_dtype != XFB200_BF16 && p->bias_dtype != XFB200_F16 && p->bias_dtype != XFB200_F32)
      return set_error(XFB200_E_INVALID, "prefill: bad bias_dtype %d", p->bias_dtype);
  }

  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // (of the tcgen05 kernels only the persistent one takes an additive bias)
  const bool can100 = p->kernel_path != XFB200_PREFILL_MMA_SYNC && p->mkv > 0 &&
                      (p->bias == nullptr || p->kernel_path != XFB200_PREFILL_TCGEN05_CTA) && prefill_sm100_supported(p);
  if (p->kernel_path >= XFB200_PREFILL_TCGEN05 && !can100) return set_error(XFB200_E_UNSUPPORTED, "prefill: the tcgen05 kernel does not cover this input");
  if (can100) return prefill_sm100_launch(p, st);
  if (p->kv_split != 0) return set_error(XFB200_E_UNSUPPORTED, "prefill: two key ranges in one call need the tcgen05 kernel (head dim 64 or 128)");
  return prefill_generic_launch(p, st);
}
