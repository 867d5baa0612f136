from .batch import BatchBuilder, StepContext, StepEntry
from .runner import ModelRunner, parse_dtype
