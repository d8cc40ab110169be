from .context import StepContext
from .load import load_model, parse_dtype
from .model import Model
from .runner import ModelRunner, StepEntry
from .workspace import Workspace
