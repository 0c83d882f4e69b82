from .engine import Engine, OutOfPages, StepContext, StepEntry  # noqa: F401
from .model import Model  # noqa: F401
