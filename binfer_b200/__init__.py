"""binfer_b200: a small, whole inference engine for one GPU (B200, sm_100a).

From a model folder (config.json + safetensors) to next-token logits and
generated tokens: typed configuration and architecture registry, weights by
tensor name, layers put together from parts, a paged cache manager, one step
function for mixed batches, a continuous-batching scheduler, device sampling,
and hand-written CUDA kernels.  There is no CPU path.
"""
__version__ = "0.1.0"


def __getattr__(name):
    # heavy imports (torch, the CUDA library) only when something is used
    if name == "Engine":
        from .engine.engine import Engine
        return Engine
    if name == "SamplingParams":
        from .sampling.params import SamplingParams
        return SamplingParams
    if name in ("Qwen3Config", "register_architecture", "load_config"):
        from . import config
        return getattr(config, name)
    raise AttributeError(name)


def generate(model_dir, prompts, dtype="bfloat16", **kwargs):
    """One-call convenience: load ``model_dir`` and generate for ``prompts`` (token ids).
    Engine options (``page_size``, ``num_pages``, ``max_seq_len``, ...) and sampling
    options (``max_tokens``, ``temperature``, ``top_k``, ``top_p``, ``seed``, ...) may be
    mixed in ``kwargs``."""
    from .engine.engine import Engine
    engine_keys = {"random_seed", "random_std", "max_kv_memory_gb", "num_pages", "page_size",
                   "max_seq_len", "max_batch_size", "max_tokens_per_step", "cuda_graphs", "device"}
    ekw = {k: v for k, v in kwargs.items() if k in engine_keys}
    gkw = {k: v for k, v in kwargs.items() if k not in engine_keys}
    return Engine(model_dir, dtype, **ekw).generate(prompts, **gkw)
