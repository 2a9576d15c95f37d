from .batch import StepBatch, StepEntry  # noqa: F401
from .engine import Engine, StreamEvent  # noqa: F401
from .request import Request, RequestState  # noqa: F401
from .runner import ModelRunner  # noqa: F401
from .scheduler import Plan, PlannedEntry, Scheduler  # noqa: F401
