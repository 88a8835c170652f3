from .batch import StepBatch, BatchStager
from .model import DecoderModel, Layer, tensor_requirements
from .engine import Engine, StepEntry
