"""B200-native CUDA backend for zllm's decode/prefill kernel path."""
