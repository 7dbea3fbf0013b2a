"""GPU KV storage and fused attention operators (sm_100a CUDA behind a C ABI)."""
