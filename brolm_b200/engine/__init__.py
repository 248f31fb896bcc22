from .context import StepContext
from .model import DecoderModel, as_dtype, load_model, write_random_model
from .generate import generate, plan_batches
from .step import Engine, StepError

__all__ = ["StepContext", "DecoderModel", "as_dtype", "load_model", "write_random_model", "Engine", "StepError", "generate", "plan_batches"]
