"""Trainer callbacks, control flags and the memory tracker.

``TrainerCallback`` subclasses receive the events of the training loop (``on_train_begin``, ``on_epoch_begin``,
``on_step_begin``, ``on_step_end``, ``on_log``, ``on_evaluate``, ``on_predict``, ``on_save``, ``on_train_end``) and may steer
it through ``TrainerControl`` (``should_training_stop / should_save / should_evaluate / should_log``), as in the
reference trainer's handler (oslo/transformers/trainer.py:230-330, trainer_callback usage throughout).
``TrainerMemoryTracker`` measures host RSS and device memory deltas of the init / train / evaluate / predict stages and
adds them to the returned metrics (reference: the ``_memory_tracker`` calls in oslo/transformers/trainer.py).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

import torch


@dataclass
class TrainerControl:
    should_training_stop: bool = False
    should_epoch_stop: bool = False
    should_save: bool = False
    should_evaluate: bool = False
    should_log: bool = False

    def _new_step(self):
        self.should_save = self.should_evaluate = self.should_log = False


class TrainerCallback:
    """Override any of the ``on_*`` methods; each gets ``(args, state, control, **kwargs)`` and may return ``control``."""

    def on_init_end(self, args, state, control, **kwargs): ...
    def on_train_begin(self, args, state, control, **kwargs): ...
    def on_train_end(self, args, state, control, **kwargs): ...
    def on_epoch_begin(self, args, state, control, **kwargs): ...
    def on_epoch_end(self, args, state, control, **kwargs): ...
    def on_step_begin(self, args, state, control, **kwargs): ...
    def on_step_end(self, args, state, control, **kwargs): ...
    def on_evaluate(self, args, state, control, **kwargs): ...
    def on_predict(self, args, state, control, **kwargs): ...
    def on_save(self, args, state, control, **kwargs): ...
    def on_log(self, args, state, control=None, logs=None, **kwargs): ...


class CallbackHandler:
    def __init__(self, callbacks, model=None, optimizer=None, lr_scheduler=None):
        self.callbacks: List = []
        for cb in callbacks or []:
            self.add_callback(cb)
        self.model, self.optimizer, self.lr_scheduler = model, optimizer, lr_scheduler

    def add_callback(self, cb):
        self.callbacks.append(cb() if isinstance(cb, type) else cb)

    def remove_callback(self, cb):
        self.callbacks = [c for c in self.callbacks if c is not cb and not (isinstance(cb, type) and isinstance(c, cb))]

    def call_event(self, event: str, args, state, control: TrainerControl, **kwargs) -> TrainerControl:
        for cb in self.callbacks:
            fn = getattr(cb, event, None)
            if fn is None:
                continue
            if event == "on_log":
                try:
                    result = fn(args, state, control, logs=kwargs.get("logs"))
                except TypeError:  # legacy signature on_log(args, state, logs)
                    result = fn(args, state, kwargs.get("logs"))
            else:
                result = fn(args, state, control, model=self.model, optimizer=self.optimizer, lr_scheduler=self.lr_scheduler,
                            **kwargs)
            if isinstance(result, TrainerControl):
                control = result
        return control


class EarlyStoppingCallback(TrainerCallback):
    """Stop when the tracked metric has not improved for ``patience`` evaluations."""

    def __init__(self, early_stopping_patience: int = 1, early_stopping_threshold: float = 0.0):
        self.patience, self.threshold = early_stopping_patience, early_stopping_threshold
        self.bad, self.best = 0, None

    def on_evaluate(self, args, state, control, metrics=None, **kwargs):
        key = args.metric_for_best_model or "eval_loss"
        if not metrics or key not in metrics:
            return control
        v = metrics[key]
        improved = self.best is None or ((v - self.best) > self.threshold if args.greater_is_better else (self.best - v) > self.threshold)
        if improved:
            self.best, self.bad = v, 0
        else:
            self.bad += 1
            if self.bad >= self.patience:
                control.should_training_stop = True
        return control


class TrainerMemoryTracker:
    """``start(stage)`` / ``stop_and_update_metrics(stage, metrics)``: host RSS and device memory deltas per stage."""

    def __init__(self, skip_memory_metrics: bool = False, device=None):
        self.skip = skip_memory_metrics
        self.device = device
        self._begin: Dict[str, dict] = {}
        self.metrics: Dict[str, int] = {}
        try:
            import psutil

            self._proc = psutil.Process()
        except Exception:
            self._proc = None

    def _cpu(self) -> int:
        return int(self._proc.memory_info().rss) if self._proc is not None else 0

    def _gpu(self):
        if torch.cuda.is_available() and (self.device is None or torch.device(self.device).type == "cuda"):
            return int(torch.cuda.memory_allocated(self.device)), int(torch.cuda.max_memory_allocated(self.device))
        return 0, 0

    def start(self, stage: str):
        if self.skip:
            return
        if torch.cuda.is_available():
            torch.cuda.reset_peak_memory_stats(self.device)
        alloc, _ = self._gpu()
        self._begin[stage] = {"cpu": self._cpu(), "gpu": alloc}

    def stop_and_update_metrics(self, stage: str, metrics: Optional[dict] = None) -> dict:
        if self.skip or stage not in self._begin:
            return metrics if metrics is not None else {}
        b = self._begin.pop(stage)
        alloc, peak = self._gpu()
        out = {f"{stage}_mem_cpu_alloc_delta": self._cpu() - b["cpu"], f"{stage}_mem_gpu_alloc_delta": alloc - b["gpu"],
               f"{stage}_mem_gpu_peaked_delta": max(0, peak - alloc)}
        self.metrics.update(out)
        if metrics is not None:
            metrics.update(out)
        return out


@dataclass
class PredictionOutput:
    predictions: Optional[torch.Tensor]
    label_ids: Optional[torch.Tensor]
    metrics: Dict[str, float]
