from .engine import Engine
from .model import DecoderModel, ignorable_tensors, tensor_declarations
from .step import GroupMeta, StepContext, StepPlanner
from .generate import generate, plan_batches, finished
