from .engine import Engine, OutOfPages, SamplingInputs, StepContext, StepEntry, StepResult  # noqa: F401
from .model import Model  # noqa: F401
