from .batch import RowSampling, Segment, StepContext
from .engine import Engine
from .runner import EngineError, ModelRunner
from .scheduler import Scheduler, SchedulerConfig, Sequence, StepPlan
