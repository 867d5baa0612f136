"""qorvix_b200: a small, whole inference engine for the Llama dense decoder on one B200."""
from . import models            # registers the architectures
from .config import LlamaConfig, load_config, register_architecture
from .engine import LLM, ModelRunner, Scheduler, SchedulerConfig, StepEntry
from .sampling import SamplingParams
from .weights import write_random_model

__version__ = "0.1.0"
