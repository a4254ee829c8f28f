"""Engine: loading, the step function, the scheduler and the public generate() entry."""
from .loading import make_env, make_runner, model_from_dir, model_from_seed, parse_dtype
from .runner import ModelRunner, StepError, StepItem

__all__ = ["make_env", "make_runner", "model_from_dir", "model_from_seed", "parse_dtype",
           "ModelRunner", "StepError", "StepItem"]
