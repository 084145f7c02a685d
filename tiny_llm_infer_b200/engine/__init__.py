from .batch import Segment, StepContext, StepEntry
from .llm_engine import LLM, EngineConfig, GenerationResult, LLMEngine
from .runner import DTYPES, ModelRunner, StepError, load_model, random_model
from .scheduler import BatchPlan, Scheduler, SchedulerConfig, SchedulerError, Sequence, Status
