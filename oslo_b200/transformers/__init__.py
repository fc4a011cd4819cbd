from .oslo_init import OsloTrainerConfig, init_oslo_features
from .profiler import FlopsProfiler, get_model_profile
from .trainer import Trainer
from .trainer_callback import (CallbackHandler, EarlyStoppingCallback, PredictionOutput, TrainerCallback, TrainerControl,
                               TrainerMemoryTracker)
from .training_args import TrainingArguments

__all__ = ["Trainer", "TrainingArguments", "OsloTrainerConfig", "init_oslo_features", "FlopsProfiler", "get_model_profile",
           "TrainerCallback", "TrainerControl", "CallbackHandler", "EarlyStoppingCallback", "TrainerMemoryTracker",
           "PredictionOutput"]
