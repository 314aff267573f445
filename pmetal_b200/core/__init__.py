from .config import (DatasetConfig, DistributedTrainingConfig, FullTrainingConfig, LoraConfig, ModelConfig,
                     TrainingConfig)
from .scheduler import LearningRateScheduler
from .types import EvalMetrics, StepMetrics
