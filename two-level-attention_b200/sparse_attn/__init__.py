"""Mirror of the reference's ``sparse_attn`` operator surface for the decode hot path."""
