"""Engine runtime: requests, paged KV-cache manager, continuous-batching scheduler,
model runner with CUDA-graph dispatch, and the step loop behind ``LLM``."""
