from .batch import StepBatch, BatchStager
from .model import DecoderModel, Layer, tensor_requirements
from .engine import Engine, StepEntry
from .generate import GenerationRequest, GenerationResult, GenerationStats, Generator, plan_batches
