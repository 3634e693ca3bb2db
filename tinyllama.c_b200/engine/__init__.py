from .generate import Continuation, EngineBackend, GenerationResult, generate, plan_batches  # noqa: F401
from .step import StepEntry, StepError, step  # noqa: F401
