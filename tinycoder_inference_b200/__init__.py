"""B200-native attention / KV-cache hot path behind a C ABI (libtc_attn.so).

`capi` binds the shared library (and raises when it is missing -- there is no
fallback), `ops` wraps each entry point for torch device tensors (the driver of the
tests and of the bench; `ops.KvSession` is the view of the C session that mirrors
the reference engine's per-layer attention dispatch), `sharding` partitions the work
over the GPUs of one box, `synth` draws the seeded benchmark inputs.
"""
from . import capi, ops  # noqa: F401

__all__ = ["capi", "ops"]
