"""Version-pinned vLLM integration; importing this package does not load CUDA."""
