"""``TrainingArguments``: the knobs of :class:`oslo_b200.transformers.Trainer`.

A compact counterpart of the reference's Hugging-Face-style dataclass (oslo/transformers/training_args.py): the fields
the trainer acts on, plus ``oslo_config_path_or_dict`` whose parsing builds the ``ParallelContext`` and the wrapper
recipes in ``__post_init__`` exactly once.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional, Union


@dataclass
class TrainingArguments:
    output_dir: str = "output"
    oslo_config_path_or_dict: Union[str, dict, None] = None
    do_train: bool = True
    do_eval: bool = False
    per_device_train_batch_size: int = 8
    per_device_eval_batch_size: int = 8
    gradient_accumulation_steps: int = 1
    learning_rate: float = 5e-5
    weight_decay: float = 0.0
    adam_beta1: float = 0.9
    adam_beta2: float = 0.999
    adam_epsilon: float = 1e-8
    max_grad_norm: float = 1.0
    num_train_epochs: float = 1.0
    max_steps: int = -1
    lr_scheduler_type: str = "linear"  # see trainer_utils.SchedulerType
    lr_scheduler_num_cycles: float = 0.5  # cosine: half-waves / 2; cosine_with_restarts: number of restarts
    lr_scheduler_power: float = 1.0  # polynomial
    warmup_ratio: float = 0.0
    warmup_steps: int = 0
    logging_strategy: str = "steps"  # no | steps | epoch
    logging_steps: int = 10
    logging_first_step: bool = False
    logging_dir: Optional[str] = None  # when set, every log record is also appended to <logging_dir>/log.jsonl
    save_strategy: str = "steps"  # no | steps | epoch
    save_steps: int = 0
    save_total_limit: Optional[int] = None
    evaluation_strategy: str = "steps"  # no | steps | epoch
    eval_steps: int = 0
    eval_accumulation_steps: Optional[int] = None  # predict(): move gathered outputs to the host every this many batches
    load_best_model_at_end: bool = False
    label_names: Optional[list] = None  # batch keys handed to compute_metrics as labels (default ["labels"])
    label_smoothing_factor: float = 0.0
    remove_unused_columns: bool = True  # drop batch keys the model's forward does not take
    ignore_data_skip: bool = False  # resume: do not fast-forward the data loader to the saved step
    group_by_length: bool = False  # batches drawn from length-sorted buckets (needs a "length" or "input_ids" column)
    overwrite_output_dir: bool = False
    local_rank: int = -1
    report_to: Optional[list] = None  # "jsonl" (logging_dir) is the only built-in sink
    disable_tqdm: bool = True
    seed: int = 42
    bf16: bool = False
    fp16: bool = False
    fp16_init_scale: float = 65536.0  # dynamic loss scaling (fp16 only): initial scale ...
    fp16_growth_interval: int = 2000  # ... doubled after this many overflow-free steps, halved on overflow
    dataloader_drop_last: bool = True
    dataloader_num_workers: int = 0
    dataloader_pin_memory: bool = True
    optim: str = "adam"  # see trainer_utils.OptimizerNames
    resume_from_checkpoint: Optional[str] = None
    metric_for_best_model: Optional[str] = None
    greater_is_better: bool = False
    skip_memory_metrics: bool = True  # False: per-stage host / device memory deltas are added to the metrics
    flops_profiler: bool = False
    flops_profiler_step: int = 1
    flops_profiler_output_path: Optional[str] = None
    parallel_context: Any = field(default=None, repr=False)
    wrapper_recipes: Any = field(default=None, repr=False)
    oslo_config: Any = field(default=None, repr=False)

    def __post_init__(self):
        from .trainer_utils import IntervalStrategy, OptimizerNames, SchedulerType

        if self.bf16 and self.fp16:
            raise ValueError("choose one of bf16 / fp16")
        SchedulerType(self.lr_scheduler_type)
        OptimizerNames(str(self.optim).lower())
        for name in ("logging_strategy", "save_strategy", "evaluation_strategy"):
            setattr(self, name, IntervalStrategy(getattr(self, name)).value)
        if self.load_best_model_at_end and self.metric_for_best_model is None:
            self.metric_for_best_model = "eval_loss"
        if not 0.0 <= self.label_smoothing_factor < 1.0:
            raise ValueError("label_smoothing_factor must be in [0, 1)")
        if self.label_names is None:
            self.label_names = ["labels"]
        if self.oslo_config_path_or_dict is not None and self.parallel_context is None:
            from .oslo_init import OsloTrainerConfig, init_oslo_features

            self.oslo_config = OsloTrainerConfig(self.oslo_config_path_or_dict)
            self.parallel_context, self.wrapper_recipes = init_oslo_features(self.oslo_config)
        mp = getattr(self.oslo_config, "mixed_precision", None) if self.oslo_config is not None else None
        if mp and mp.get("enable", True):
            # the configuration's mixed_precision section selects the compute dtype like the bf16 / fp16 flags do
            want = mp.get("dtype", "bf16")
            if (want == "bf16" and self.fp16) or (want == "fp16" and self.bf16):
                raise ValueError(f"mixed_precision.dtype={want} contradicts the bf16 / fp16 flags")
            self.bf16, self.fp16 = want == "bf16", want == "fp16"

    @property
    def dtype(self):
        import torch

        return torch.bfloat16 if self.bf16 else (torch.float16 if self.fp16 else torch.float32)
