"""superl8_b200 -- the reference's int8 attention hot path on B200 (sm_100a).

Public names follow the reference package (reference superl8/__init__.py):
``attn_int8_fwd``, ``attn_int8_decode`` (alias ``attn_decode``), ``attn_fp16_fwd``,
``quantize_i8_rowwise``, ``attn``, ``attn_ref``, and the ``quant`` helpers.
"""

from . import _C, quant  # noqa: F401
from .autograd import attn, attn_ref  # noqa: F401
from .ops import (  # noqa: F401
    attn_decode,
    attn_decode_cached,
    attn_decode_int8_cache,
    attn_fp16_fwd,
    attn_int8_decode,
    attn_int8_fwd,
    attn_int8_fwd_host,
    attn_int8_varlen,
    backward_cuda,
    quantize_i8_rowwise,
    quantize_kv_cache,
)
from .quant import (  # noqa: F401
    LOG2E,
    Q_MAX,
    detect_q_outlier_domination,
    quantize_int8_rowwise,
    quantize_qk,
    smooth_k,
)

__all__ = [
    "attn", "attn_ref", "attn_decode", "attn_decode_cached", "attn_decode_int8_cache", "quantize_kv_cache", "attn_fp16_fwd", "attn_int8_decode", "attn_int8_fwd",
    "attn_int8_fwd_host", "attn_int8_varlen", "backward_cuda", "quantize_i8_rowwise", "quantize_int8_rowwise", "quantize_qk", "smooth_k", "detect_q_outlier_domination",
    "LOG2E", "Q_MAX",
]
