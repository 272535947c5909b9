"""CPU oracle for the attention-forward path.  TEST INFRASTRUCTURE ONLY.

Nothing in the shipped package imports this directory.  It restates, in plain
fp32 PyTorch / numpy on the CPU, the arithmetic that the reference's tests use
to judge its attention operators.  The reference's own ``ref_attention`` lives
in the un-vendored ``mslk`` package (xformers/attn_bias_utils.py:7-12) and can
not be imported, so every function here follows a formula spelled out in the
reference's test-suite and cites it.

Parity status: pinned through the known-answer tensors held by the reference's
tests (tests/golden/mask_kats.json, transcribed from
tests/test_mem_eff_attention.py), through the test-local closed-form formulas
(logsumexp, merge-with-self = lse + ln 2, chunked == full) and through
``torch.nn.functional.scaled_dot_product_attention`` as an independent
implementation of the same softmax(QK^T*scale+bias)V definition.
"""

from .ref_attention import (  # noqa: F401
    ref_attention,
    ref_attention_bmhk,
    ref_attention_with_lse,
)
from .masks import (  # noqa: F401
    causal_mask,
    block_diagonal_mask,
    padded_keys_mask,
    local_mask,
)
from .int4 import quantize_kv_int4, dequantize_kv_int4  # noqa: F401
from .fp8 import (  # noqa: F401
    quantize_fp8_asymmetric,
    dequantize_fp8_asymmetric,
    combine_scale_shift,
    split_scale_shift,
    pack_fp8_words,
    unpack_fp8_words,
)
from .paged import gather_paged, scatter_to_pages, physical_rows  # noqa: F401
from .merge import merge_attentions_ref  # noqa: F401
from .splitk import ref_attention_splitk  # noqa: F401
from .rope import rope_frequencies, rope_rotate, rope_padded as rope_padded_ref  # noqa: F401
