"""infer_b200: a small, whole inference engine for one GPU (NVIDIA B200, sm_100a).

Everything between a request's tokens and its next token: typed configuration and architecture
registry, safetensors weights, layers put together from parts, a paged cache manager, one step
function for mixed batches, a scheduler, sampling, and hand-written CUDA kernels underneath.
"""
__version__ = "0.1.0"
