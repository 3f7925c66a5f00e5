"""LLM engine: paged KV pool, model runner with CUDA-graph decode, decode loops and continuous batching."""
