"""Mirror of the reference package ``flash_attn_triton`` (module names and
public functions are the reference's)."""
