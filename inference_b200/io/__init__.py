"""Checkpoint IO: safetensors (mmap, sharded, tensor-parallel slicing on read), GGUF (container, block
dequantisers, Q4_K / Q8_0 quantisers), tokenizer reconstruction and snapshot preparation."""
