"""binfer_b200: a small, whole inference engine for one GPU (B200, sm_100a).

From a model folder (config.json + safetensors) to next-token logits and
generated tokens: typed configuration and architecture registry, weights by
tensor name, layers put together from parts, a paged cache manager, one step
function for mixed batches, a continuous-batching scheduler, device sampling,
and hand-written CUDA kernels.  There is no CPU path.
"""
__version__ = "0.1.0"
