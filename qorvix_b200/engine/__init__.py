from .batch import BatchBuilder, StepContext, StepEntry
from .runner import ModelRunner, parse_dtype
from .generate import LLM
from .scheduler import RequestResult, Scheduler, SchedulerConfig
