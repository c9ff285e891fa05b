"""B200-native paged full-attention KV-cache hot path (append, paged GQA decode,
packed prefill, prefix reuse with GDN hybrid-state snapshot / restore)."""

__version__ = "0.1.0"
