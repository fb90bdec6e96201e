"""B200-native absorbed-MLA decode over an FP8 / MXFP4 / hybrid latent KV cache.

Public surface (mirrors the reference's mixed-mla problem definition):

* ``custom_kernel(data)`` - the submission entry point, same 5-tuple as the reference
  (mixed-mla/submission.py:626).
* ``generate_input`` / ``quantize_fp8`` / ``quantize_mxfp4`` / ``dequantize_mxfp4`` - host-side
  mirrors of competitor_submissions/mi355x_reference/reference.py:65-154,288-346.
* ``mla_decode`` / ``combine_partials`` / ``quantize_q_fp8`` / ``kv_append`` - thin wrappers over the
  C ABI of libb200mla.so (include/b200_mla.h).

The compute path is hand-written CUDA for sm_100a behind that C ABI; there is no CPU or Triton
fallback.  The library-backed names are resolved on first access (so that the build module can be
imported before the library exists); if libb200mla.so has not been built, that access raises.
"""
from .inputs import (generate_input, quantize_fp8, quantize_mxfp4, dequantize_mxfp4, quantize_hybrid,
                     QK_HEAD_DIM, V_HEAD_DIM, KV_LORA_RANK, QK_ROPE_HEAD_DIM)

_LIB_BACKED = ("custom_kernel", "mla_decode", "combine_partials", "quantize_q_fp8", "q_amax_parts", "kv_append")


def __getattr__(name):
    if name in _LIB_BACKED or name in ("submission", "_cabi", "distributed"):
        import importlib
        if name in _LIB_BACKED:
            return getattr(importlib.import_module(".submission", __name__), name)
        return importlib.import_module("." + name, __name__)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")

__all__ = [
    "custom_kernel", "mla_decode", "combine_partials", "quantize_q_fp8", "q_amax_parts", "kv_append",
    "generate_input", "quantize_fp8", "quantize_mxfp4", "dequantize_mxfp4", "quantize_hybrid",
    "QK_HEAD_DIM", "V_HEAD_DIM", "KV_LORA_RANK", "QK_ROPE_HEAD_DIM",
]
