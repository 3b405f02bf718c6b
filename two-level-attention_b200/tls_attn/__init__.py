"""Mirror of the reference's ``tls_attn`` prototype operators (contiguous KV cache)."""
