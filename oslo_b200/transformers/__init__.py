from .data_collator import DataCollatorWithPadding, default_data_collator
from .oslo_init import OsloTrainerConfig, init_oslo_features
from .profiler import FlopsProfiler, get_model_profile
from .trainer import Trainer
from .trainer_callback import (CallbackHandler, EarlyStoppingCallback, PredictionOutput, TrainerCallback, TrainerControl,
                               TrainerMemoryTracker)
from .trainer_utils import IntervalStrategy, OptimizerNames, SchedulerType, create_optimizer, get_scheduler, log_dist
from .training_args import TrainingArguments

__all__ = ["Trainer", "TrainingArguments", "OsloTrainerConfig", "init_oslo_features", "FlopsProfiler", "get_model_profile",
           "TrainerCallback", "TrainerControl", "CallbackHandler", "EarlyStoppingCallback", "TrainerMemoryTracker",
           "PredictionOutput", "SchedulerType", "OptimizerNames", "IntervalStrategy", "get_scheduler", "create_optimizer",
           "log_dist", "default_data_collator", "DataCollatorWithPadding"]
