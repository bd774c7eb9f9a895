"""B200-native attention / KV-cache hot path behind a C ABI (libtc_attn.so).

`capi` binds the shared library (and raises when it is missing -- there is no
fallback), `ops` wraps each entry point for torch device tensors, `engine`
mirrors the reference engine's per-layer attention dispatch on top of `ops`,
`sharding` partitions the work over the GPUs of one box.
"""
from . import capi, ops  # noqa: F401

__all__ = ["capi", "ops"]
