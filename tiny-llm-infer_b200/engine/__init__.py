from .batch import Segment, StepContext, StepEntry
from .runner import DTYPES, ModelRunner, StepError, load_model, random_model
