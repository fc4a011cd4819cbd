"""``Trainer``: training / evaluation loop over the parallel wrappers.

Covers what the reference trainer does (oslo/transformers/trainer.py:91-1871) in a compact form: distributed samplers
over the DATA group, gradient accumulation (``no_sync`` on DDP), clipping, LR schedules, logging history, evaluation,
checkpoints (per-rank model shards through ``save_pretrained``, ``optimizer.pt``, ``scheduler.pt``,
``trainer_state.json``, per-rank ``rng_state_{rank}.pth``), resume (skips the batches already seen), best-model tracking,
one-step FLOPs profiling, and the pipeline generator protocol.
"""
from __future__ import annotations

import json
import math
import os
import random
import shutil
import time
from typing import Callable, Dict, List, Optional

import numpy as np
import torch
import torch.distributed as dist
from torch.utils.data import DataLoader, Dataset
from torch.utils.data.distributed import DistributedSampler

import oslo_b200
from oslo_b200.distributed import ParallelMode
from oslo_b200.utils.logging import get_dist_logger

from .trainer_callback import (CallbackHandler, PredictionOutput, TrainerCallback, TrainerControl,  # noqa: F401
                               TrainerMemoryTracker)
from .trainer_utils import IntervalStrategy, create_optimizer, get_scheduler  # noqa: F401
from .training_args import TrainingArguments


def _scheduler(optimizer, kind: str, warmup: int, total: int, num_cycles: float = 0.5, power: float = 1.0):
    return get_scheduler(kind, optimizer, warmup, total, num_cycles=num_cycles, power=power)


class LengthGroupedSampler(torch.utils.data.Sampler):
    """Distributed sampler whose batches hold examples of similar length: a seeded shuffle, cut into mega-batches of
    ``50 x batch_size x replicas`` examples that are sorted by length, then dealt to the replicas batch by batch (so every
    replica's k-th batch comes from the same length neighbourhood and padding is short everywhere)."""

    def __init__(self, dataset, batch_size: int, num_replicas: int = 1, rank: int = 0, seed: int = 0, drop_last: bool = True,
                 lengths: Optional[List[int]] = None):
        self.n, self.bs, self.world, self.rank, self.seed, self.epoch = len(dataset), batch_size, num_replicas, rank, seed, 0
        if lengths is None:
            def length(ex):
                if isinstance(ex, dict):
                    return int(ex["length"]) if "length" in ex else len(ex["input_ids"])
                return len(ex)
            lengths = [length(dataset[i]) for i in range(self.n)]
        self.lengths = lengths
        per = self.bs * self.world
        self.total = (self.n // per) * per if drop_last else (self.n + per - 1) // per * per

    def set_epoch(self, epoch: int):
        self.epoch = epoch

    def __len__(self):
        return self.total // self.world

    def __iter__(self):
        g = torch.Generator().manual_seed(self.seed + self.epoch)
        order = torch.randperm(self.n, generator=g).tolist()
        order = (order + order[: self.total - self.n])[: self.total]
        mega = 50 * self.bs * self.world
        out = []
        for s in range(0, self.total, mega):
            chunk = sorted(order[s : s + mega], key=lambda i: -self.lengths[i])
            for b in range(0, len(chunk), self.bs * self.world):
                out.extend(chunk[b + self.rank * self.bs : b + (self.rank + 1) * self.bs])
        return iter(out)


class TrainerState:
    def __init__(self):
        self.global_step = 0
        self.epoch = 0.0
        self.log_history: List[dict] = []
        self.best_metric = None
        self.best_model_checkpoint = None

    def to_json(self):
        return json.dumps(self.__dict__, indent=2)


class Trainer:
    def __init__(self, model, args: TrainingArguments, train_dataset: Optional[Dataset] = None,
                 eval_dataset: Optional[Dataset] = None, data_collator: Optional[Callable] = None,
                 optimizers=(None, None), compute_metrics: Optional[Callable] = None, callbacks=None):
        self.args = args
        self.pc = args.parallel_context
        self.logger = get_dist_logger("oslo_b200.trainer")
        self.train_dataset, self.eval_dataset = train_dataset, eval_dataset
        self.data_collator = data_collator
        self.compute_metrics = compute_metrics
        self.callbacks = callbacks or []
        self.callback_handler = CallbackHandler(self.callbacks, model=model)
        self.control = TrainerControl()
        self._memory_tracker = TrainerMemoryTracker(getattr(args, "skip_memory_metrics", True))
        self._memory_tracker.start("init")
        self.state = TrainerState()
        self.base_model = model
        if args.dtype != torch.float32:
            model.to(args.dtype)
        self.model = model
        self.zero = None
        self.hetero = None
        self.scaler = None  # DynamicLossScaler, built with the optimizer when fp16 is on
        if self.pc is not None:
            from .oslo_init import apply_wrappers

            self.model = apply_wrappers(model, self.pc, args.wrapper_recipes or [])
            cfg = args.oslo_config
            dp = cfg.data_parallelism if cfg else None
            stage = (dp or {}).get("zero_stage", 0)
            self.hetero = None
            if stage == 3:
                # chunked ZeRO-3: parameters live in chunks sharded over the DATA group and are gathered around each module
                from oslo_b200.parallel.data_parallel.zero.hetero import HeteroDataParallel

                params = {k: v for k, v in ((dp or {}).get("params") or {}).items()
                          if k in ("placement_policy", "chunk_size_mb", "pin_memory", "min_free_fraction", "device_budget_bytes")}
                if (dp or {}).get("params", {}).get("cpu_offload"):
                    params.setdefault("placement_policy", "cpu")
                self.hetero = self.model = HeteroDataParallel(self.model, self.pc, **params)
            if self.pc.data_parallel_size > 1 and stage == 0:
                from oslo_b200.parallel import DistributedDataParallel

                self.model = DistributedDataParallel(model if self.model is model else self.model, self.pc) \
                    if self.model is model else self._ddp_over(self.model)
            oslo_b200.ready(self.model, self.pc)
            if cfg and cfg.activation_checkpointing:
                from oslo_b200.utils.checkpoint import ActivationCheckpointing

                ac = cfg.activation_checkpointing
                ActivationCheckpointing(model, self.pc, ac.get("partitioned", False), ac.get("contiguous", False), ac.get("cpu", False))
        elif torch.cuda.is_available():
            model.to("cuda")
        self.optimizer, self.lr_scheduler = optimizers
        self.is_pipeline = self.pc is not None and self.pc.pipeline_parallel_size > 1
        self.profiler = None
        self._memory_tracker.stop_and_update_metrics("init")
        self.control = self.callback_handler.call_event("on_init_end", self.args, self.state, self.control)

    def add_callback(self, callback):
        self.callback_handler.add_callback(callback)

    def remove_callback(self, callback):
        self.callback_handler.remove_callback(callback)

    def _event(self, name: str, **kwargs):
        self.callback_handler.optimizer, self.callback_handler.lr_scheduler = self.optimizer, self.lr_scheduler
        self.control = self.callback_handler.call_event(name, self.args, self.state, self.control, **kwargs)

    def _ddp_over(self, wrapped):
        from oslo_b200.parallel.data_parallel import _DistributedDataParallel

        _DistributedDataParallel(self.base_model, self.pc)  # registers itself on the base module
        return wrapped

    # ------------------------------------------------------------------ setup
    @property
    def device(self):
        return self.pc.device if self.pc is not None else next(self.base_model.parameters()).device

    def _dp(self):
        if self.pc is None:
            return 1, 0
        return self.pc.get_world_size(ParallelMode.DATA), self.pc.get_local_rank(ParallelMode.DATA)

    def get_train_dataloader(self) -> DataLoader:
        world, rank = self._dp()
        if self.args.group_by_length:
            sampler = LengthGroupedSampler(self.train_dataset, self.args.per_device_train_batch_size, num_replicas=world, rank=rank,
                                           seed=self.args.seed, drop_last=self.args.dataloader_drop_last)
        else:
            sampler = DistributedSampler(self.train_dataset, num_replicas=world, rank=rank, shuffle=True, seed=self.args.seed,
                                         drop_last=self.args.dataloader_drop_last)
        return DataLoader(self.train_dataset, batch_size=self.args.per_device_train_batch_size, sampler=sampler,
                          collate_fn=self.data_collator, drop_last=self.args.dataloader_drop_last,
                          num_workers=self.args.dataloader_num_workers,
                          pin_memory=self.args.dataloader_pin_memory and torch.cuda.is_available())

    def get_eval_dataloader(self, dataset=None) -> DataLoader:
        dataset = dataset or self.eval_dataset
        world, rank = self._dp()
        sampler = DistributedSampler(dataset, num_replicas=world, rank=rank, shuffle=False)
        return DataLoader(dataset, batch_size=self.args.per_device_eval_batch_size, sampler=sampler,
                          collate_fn=self.data_collator)

    def create_optimizer(self):
        if self.optimizer is not None:
            return self.optimizer
        a = self.args
        params = [p for p in self.base_model.parameters() if p.requires_grad and (p.numel() > 0 or self.hetero is not None)]
        opt = None if self.hetero is not None else create_optimizer(a.optim, params, lr=a.learning_rate, weight_decay=a.weight_decay, betas=(a.adam_beta1, a.adam_beta2),
                               eps=a.adam_epsilon, max_grad_norm=a.max_grad_norm, master_weights=a.dtype != torch.float32)
        cfg = a.oslo_config
        dp = (cfg.data_parallelism if cfg else None) or {}
        if self.pc is not None and dp.get("zero_stage", 0) in (1, 2):
            from oslo_b200.parallel import ZeroRedundancyOptimizer

            inner = torch.optim.AdamW(params, lr=a.learning_rate, betas=(a.adam_beta1, a.adam_beta2), eps=a.adam_epsilon,
                                      weight_decay=a.weight_decay)
            scaling = dict(initial_scale=a.fp16_init_scale, growth_interval=a.fp16_growth_interval) if a.fp16 else {}
            self.zero = opt = ZeroRedundancyOptimizer(inner, parallel_context=self.pc, partition_grad=dp["zero_stage"] == 2,
                                                      clip_grad_norm=a.max_grad_norm, **scaling, **(dp.get("params") or {}))
        if self.hetero is not None:
            from oslo_b200.parallel.data_parallel.zero.hetero import HeteroOptimizer

            inner = torch.optim.AdamW(params, lr=a.learning_rate, betas=(a.adam_beta1, a.adam_beta2), eps=a.adam_epsilon,
                                      weight_decay=a.weight_decay)
            self.zero = opt = HeteroOptimizer(self.hetero, inner, clip_grad_norm=a.max_grad_norm)
        self.optimizer = opt
        if a.fp16 and self.zero is None and self.scaler is None:
            from oslo_b200.optim.loss_scaler import DynamicLossScaler

            group = dist.group.WORLD if (self.pc is not None and dist.is_initialized()) else None
            self.scaler = DynamicLossScaler(init_scale=a.fp16_init_scale, growth_interval=a.fp16_growth_interval, group=group)
        return opt

    # ------------------------------------------------------------- train loop
    def _forward_keys(self):
        """Argument names of the model's forward, or None when it takes ``**kwargs`` (then nothing is dropped)."""
        if not hasattr(self, "_fwd_keys"):
            import inspect

            sig = inspect.signature(self.base_model.forward)
            open_ended = any(p.kind == p.VAR_KEYWORD for p in sig.parameters.values())
            self._fwd_keys = None if open_ended else set(sig.parameters)
        return self._fwd_keys

    def _move(self, batch: Dict[str, torch.Tensor]):
        keys = self._forward_keys() if self.args.remove_unused_columns else None
        if keys is not None:
            batch = {k: v for k, v in batch.items() if k in keys}
        return {k: (v.to(self.device, non_blocking=True) if torch.is_tensor(v) else v) for k, v in batch.items()}

    def compute_loss(self, batch) -> torch.Tensor:
        """The model's own loss, or, with ``label_smoothing_factor``, (1 - eps) * NLL + eps * mean over the vocabulary of
        -log p, taken on the logits with the labels withheld from the model (decoder-only models: shifted by one)."""
        eps = self.args.label_smoothing_factor
        if not eps or "labels" not in batch:
            return self.model(**batch).loss
        labels = batch["labels"]
        out = self.model(**{k: v for k, v in batch.items() if k != "labels"})
        logits = out.logits if hasattr(out, "logits") else out[0]
        if logits.dim() == 3 and logits.shape[1] == labels.shape[-1] and getattr(self.base_model, "shift_labels", self._is_causal()):
            logits, labels = logits[:, :-1], labels[:, 1:]
        logp = torch.log_softmax(logits.float(), dim=-1)
        valid = labels.ne(-100)
        safe = labels.clamp(min=0).unsqueeze(-1)
        nll = -logp.gather(-1, safe).squeeze(-1)
        smooth = -logp.mean(dim=-1)
        n = valid.sum().clamp(min=1)
        return ((1.0 - eps) * (nll * valid).sum() + eps * (smooth * valid).sum()) / n

    def _is_causal(self) -> bool:
        name = type(self.base_model).__name__
        return "CausalLM" in name or "LMHeadModel" in name

    def training_step(self, batch) -> torch.Tensor:
        batch = self._move(batch)
        accum = self.args.gradient_accumulation_steps
        if self.is_pipeline:
            total = torch.zeros((), device=self.device)
            for _, out in self.model(**batch):
                if torch.is_tensor(out.loss):
                    part = out.loss / accum
                    (self.scaler.scale(part) if self.scaler is not None else part).backward()
                    total += out.loss.detach()
            return self._from_last_stage(total)
        loss = self.compute_loss(batch) / accum
        if self.zero is not None:
            self.zero.backward(loss)  # the ZeRO optimizer scales the loss itself
        elif self.scaler is not None:
            self.scaler.scale(loss).backward()
        else:
            loss.backward()
        return loss.detach() * accum

    def _from_last_stage(self, value) -> torch.Tensor:
        """Under pipeline parallelism only the last stage computes the loss: hand it to every stage (the others add
        zero), so logs, best-model tracking and early stopping see the same number on all ranks."""
        t = torch.zeros((), device=self.device) if value is None else value.detach().float().to(self.device).reshape(())
        if self.pc is not None and self.pc.pipeline_parallel_size > 1:
            t = t.clone()
            dist.all_reduce(t, group=self.pc.get_group(ParallelMode.PIPELINE))
        return t

    def _clip(self):
        if self.zero is not None or not self.args.max_grad_norm:
            return
        params = [p for p in self.base_model.parameters() if p.grad is not None]
        if params:
            torch.nn.utils.clip_grad_norm_(params, self.args.max_grad_norm)

    def train(self, resume_from_checkpoint: Optional[str] = None):
        a = self.args
        loader = self.get_train_dataloader()
        steps_per_epoch = max(1, len(loader) // a.gradient_accumulation_steps)
        max_steps = a.max_steps if a.max_steps > 0 else int(math.ceil(a.num_train_epochs * steps_per_epoch))
        opt = self.create_optimizer()
        inner = opt.optim if self.zero is not None else opt
        if self.lr_scheduler is None:
            warm = a.warmup_steps or int(a.warmup_ratio * max_steps)
            self.lr_scheduler = _scheduler(inner, a.lr_scheduler_type, warm, max_steps, a.lr_scheduler_num_cycles, a.lr_scheduler_power)
        resume = resume_from_checkpoint or a.resume_from_checkpoint
        skip_batches = 0
        if resume:
            done_steps = self._load_checkpoint(resume)
            # the loop restarts in the epoch the checkpoint was taken in: skip only what that epoch had already consumed
            self.state.epoch = float(done_steps // steps_per_epoch)
            skip_batches = (done_steps % steps_per_epoch) * a.gradient_accumulation_steps
            if a.ignore_data_skip:
                skip_batches = 0
        self.base_model.train()
        self._memory_tracker.start("train")
        self._event("on_train_begin")
        t0 = time.time()
        tokens = 0
        running, epoch, last_logged = 0.0, int(self.state.epoch), self.state.global_step
        done = False
        while not done:
            if hasattr(loader.sampler, "set_epoch"):
                loader.sampler.set_epoch(epoch)
            self._event("on_epoch_begin")
            for i, batch in enumerate(loader):
                if skip_batches > 0:
                    skip_batches -= 1
                    continue
                sync_now = (i + 1) % a.gradient_accumulation_steps == 0
                if i % a.gradient_accumulation_steps == 0:
                    self.control._new_step()
                    self._event("on_step_begin")
                profile = a.flops_profiler and self.state.global_step == a.flops_profiler_step and self._rank() == 0
                if profile:
                    from .profiler import FlopsProfiler

                    self.profiler = FlopsProfiler(self.base_model)
                    self.profiler.start_profile()
                ctx = self.model.no_sync() if (not sync_now and hasattr(self.model, "no_sync")) else _null()
                zctx = self.zero.no_sync() if (not sync_now and self.zero is not None and hasattr(self.zero, "no_sync")) else _null()
                with ctx, zctx:
                    running += float(self.training_step(batch))
                if profile:
                    self.profiler.stop_profile()
                    self.profiler.print_model_profile(output_file=a.flops_profiler_output_path)
                if "input_ids" in batch:
                    tokens += batch["input_ids"].numel()
                if not sync_now:
                    continue
                if self.scaler is not None:
                    # fp16: un-scale, skip the update (and the schedule step) when any rank's gradients overflowed
                    overflow = self.scaler.unscale_(opt)
                    if not overflow:
                        self._clip()
                    self.scaler.step(opt)
                    self.scaler.update()
                    if not overflow:
                        self.lr_scheduler.step()
                else:
                    self._clip()
                    opt.step()
                    self.lr_scheduler.step()
                if self.zero is not None:
                    opt.zero_grad()
                elif hasattr(self.model, "zero_grad") and hasattr(self.model, "flats"):
                    self.model.zero_grad()
                else:
                    opt.zero_grad()
                self.state.global_step += 1
                self.state.epoch = epoch + (i + 1) / len(loader)
                self._event("on_step_end")
                first = a.logging_first_step and self.state.global_step == 1
                if (a.logging_strategy == "steps" and a.logging_steps and self.state.global_step % a.logging_steps == 0) \
                        or first or self.control.should_log:
                    n = max(1, self.state.global_step - last_logged) * a.gradient_accumulation_steps
                    last_logged = self.state.global_step
                    self.log({"loss": self._mean_over_dp(running / n), "learning_rate": self.lr_scheduler.get_last_lr()[0],
                              "epoch": round(self.state.epoch, 3), "step": self.state.global_step})
                    running = 0.0
                if self.eval_dataset is not None and ((a.evaluation_strategy == "steps" and a.eval_steps
                                                       and self.state.global_step % a.eval_steps == 0)
                                                      or self.control.should_evaluate):
                    self._track_best(self.evaluate())
                    self.base_model.train()
                if (a.save_strategy == "steps" and a.save_steps and self.state.global_step % a.save_steps == 0) \
                        or self.control.should_save:
                    self.save_checkpoint()
                if self.state.global_step >= max_steps or self.control.should_training_stop:
                    done = True
                    break
            self._event("on_epoch_end")
            if a.logging_strategy == "epoch" and self.state.global_step > last_logged:
                n = (self.state.global_step - last_logged) * a.gradient_accumulation_steps
                last_logged = self.state.global_step
                self.log({"loss": self._mean_over_dp(running / n), "learning_rate": self.lr_scheduler.get_last_lr()[0],
                          "epoch": round(self.state.epoch, 3), "step": self.state.global_step})
                running = 0.0
            if a.evaluation_strategy == "epoch" and self.eval_dataset is not None:
                self._track_best(self.evaluate())
                self.base_model.train()
            if a.save_strategy == "epoch":
                self.save_checkpoint()
            if self.control.should_training_stop:
                done = True
            epoch += 1
        if a.load_best_model_at_end and self.state.best_model_checkpoint:
            self._load_checkpoint(self.state.best_model_checkpoint, weights_only=True)
        elapsed = time.time() - t0
        dp_world, _ = self._dp()
        metrics = {"train_runtime": elapsed, "train_steps_per_second": self.state.global_step / max(elapsed, 1e-9),
                   "train_tokens_per_second": tokens * dp_world / max(elapsed, 1e-9)}
        self._memory_tracker.stop_and_update_metrics("train", metrics)
        self._event("on_train_end")
        self.log(metrics)
        return metrics

    def _rank(self):
        return self.pc.get_global_rank() if self.pc is not None else 0

    def _mean_over_dp(self, value: float) -> float:
        if self.pc is None or self.pc.data_parallel_size == 1:
            return value
        t = torch.tensor([value], device=self.device)
        dist.all_reduce(t, group=self.pc.get_group(ParallelMode.DATA))
        return float(t) / self.pc.data_parallel_size

    def log(self, logs: dict):
        self.state.log_history.append(dict(logs))
        self.logger.info(json.dumps(logs), ranks=[0])
        if self.args.logging_dir and self._rank() == 0:
            os.makedirs(self.args.logging_dir, exist_ok=True)
            with open(os.path.join(self.args.logging_dir, "log.jsonl"), "a") as f:
                f.write(json.dumps(logs) + "\n")
        self._event("on_log", logs=logs)

    # ------------------------------------------------------------- evaluation
    @torch.no_grad()
    def evaluate(self, eval_dataset=None, metric_key_prefix: str = "eval") -> Dict[str, float]:
        self.base_model.eval()
        self._memory_tracker.start(metric_key_prefix)
        losses = []
        for batch in self.get_eval_dataloader(eval_dataset):
            batch = self._move(batch)
            if self.is_pipeline:
                total = None
                for _, out in self.model(**batch):
                    if torch.is_tensor(out.loss):
                        total = out.loss if total is None else total + out.loss
                losses.append(float(self._from_last_stage(total)))
            else:
                losses.append(float(self.model(**batch).loss))
        loss = self._mean_over_dp(sum(losses) / max(1, len(losses)))
        metrics = {f"{metric_key_prefix}_loss": loss, f"{metric_key_prefix}_ppl": math.exp(min(loss, 50.0))}
        if self.compute_metrics:
            metrics.update(self.compute_metrics(metrics))
        self._memory_tracker.stop_and_update_metrics(metric_key_prefix, metrics)
        self.log(metrics)
        self._event("on_evaluate", metrics=metrics)
        return metrics

    @torch.no_grad()
    def predict(self, test_dataset, metric_key_prefix: str = "test") -> PredictionOutput:
        """Run the model over ``test_dataset`` and return the gathered predictions (``argmax`` of the logits), the labels
        when the dataset has them, and metrics (loss over the batches that carry labels, ``compute_metrics`` on
        ``(predictions, label_ids)`` when given).  Under pipeline parallelism only the loss is available."""
        self.base_model.eval()
        self._memory_tracker.start(metric_key_prefix)
        preds, labels, losses = [], [], []
        for batch in self.get_eval_dataloader(test_dataset):
            batch = self._move(batch)
            if self.is_pipeline:
                total = None
                for _, out in self.model(**batch):
                    if torch.is_tensor(out.loss):
                        total = out.loss if total is None else total + out.loss
                losses.append(float(self._from_last_stage(total)))
                continue
            out = self.model(**batch)
            if getattr(out, "loss", None) is not None:
                losses.append(float(out.loss))
            logits = getattr(out, "logits", None)
            if logits is None and "labels" in batch:  # the fused loss consumed the logits: run once more without labels
                logits = self.model(**{k: v for k, v in batch.items() if k != "labels"}).logits
            if logits is not None:
                if self.pc is not None and self.pc.tensor_parallel_size > 1 and logits.dim() >= 2:
                    # tensor-parallel heads may return a vocabulary (and, in the N-D layouts, batch) shard
                    from oslo_b200.lightseq.inference import _whole_logits

                    flat = _whole_logits(self.model, logits.reshape(-1, logits.shape[-1]))
                    logits = flat.reshape(-1, *logits.shape[1:-1], flat.shape[-1]) if logits.dim() > 2 else flat
                preds.append(logits.argmax(-1).cpu())
            if "labels" in batch:
                labels.append(batch["labels"].cpu())
        metrics: Dict[str, float] = {}
        if losses:
            loss = self._mean_over_dp(sum(losses) / len(losses))
            metrics[f"{metric_key_prefix}_loss"] = loss
        predictions = torch.cat(preds) if preds else None
        label_ids = torch.cat(labels) if labels else None
        if self.compute_metrics is not None and predictions is not None:
            try:
                extra = self.compute_metrics((predictions, label_ids))
            except Exception:
                extra = self.compute_metrics(metrics)
            metrics.update({k if k.startswith(metric_key_prefix) else f"{metric_key_prefix}_{k}": v for k, v in (extra or {}).items()})
        self._memory_tracker.stop_and_update_metrics(metric_key_prefix, metrics)
        self.log(metrics)
        self._event("on_predict", metrics=metrics)
        return PredictionOutput(predictions, label_ids, metrics)

    def _track_best(self, metrics):
        key = self.args.metric_for_best_model or "eval_loss"
        if key not in metrics:
            return
        v = metrics[key]
        better = self.state.best_metric is None or (v > self.state.best_metric if self.args.greater_is_better else v < self.state.best_metric)
        if better:
            self.state.best_metric = v
            self.state.best_model_checkpoint = self.save_checkpoint()

    # ------------------------------------------------------------ checkpoints
    def save_checkpoint(self) -> str:
        a = self.args
        out = os.path.join(a.output_dir, f"checkpoint-{self.state.global_step}")
        os.makedirs(out, exist_ok=True)
        if self.hetero is not None:
            full = self.hetero.state_dict()  # collective: every chunk is gathered
            if self._rank() == 0:
                torch.save(full, os.path.join(out, "pytorch_model.bin"))
        elif hasattr(self.model, "save_pretrained") and self.pc is not None:
            self.model.save_pretrained(out)
        elif self._rank() == 0:
            self.base_model.save_pretrained(out) if hasattr(self.base_model, "save_pretrained") else torch.save(
                self.base_model.state_dict(), os.path.join(out, "pytorch_model.bin"))
        rank = self._rank()
        torch.save(self.optimizer.state_dict(), os.path.join(out, f"optimizer_{rank}.pt" if self.pc is not None else "optimizer.pt"))
        rng = {"python": random.getstate(), "numpy": np.random.get_state(), "cpu": torch.get_rng_state()}
        if torch.cuda.is_available():
            rng["cuda"] = torch.cuda.get_rng_state()
        torch.save(rng, os.path.join(out, f"rng_state_{rank}.pth"))
        if rank == 0:
            torch.save(self.lr_scheduler.state_dict(), os.path.join(out, "scheduler.pt"))
            if self.scaler is not None:
                torch.save(self.scaler.state_dict(), os.path.join(out, "scaler.pt"))
            with open(os.path.join(out, "trainer_state.json"), "w") as f:
                f.write(self.state.to_json())
            torch.save(self.args.__dict__.get("oslo_config_path_or_dict"), os.path.join(out, "training_args.bin"))
            self._rotate()
        if dist.is_initialized():
            dist.barrier()
        self._event("on_save")
        return out

    def _rotate(self):
        limit = self.args.save_total_limit
        if not limit:
            return
        ckpts = sorted((d for d in os.listdir(self.args.output_dir) if d.startswith("checkpoint-")), key=lambda d: int(d.split("-")[1]))
        for d in ckpts[:-limit]:
            full = os.path.join(self.args.output_dir, d)
            if full != self.state.best_model_checkpoint:
                shutil.rmtree(full, ignore_errors=True)

    def _load_checkpoint(self, path: str, weights_only: bool = False) -> int:
        """Restores model shards, optimizer, scheduler, RNG and trainer state; returns the steps already done.
        ``weights_only`` reloads the model alone (best-model reload at the end of training)."""
        rank = self._rank()
        if self.hetero is not None:
            self.hetero.load_state_dict(torch.load(os.path.join(path, "pytorch_model.bin"), map_location="cpu"))
            if self.zero is not None:
                self.zero._built = False  # the fp32 masters are rebuilt from the loaded shards
        elif self.pc is not None and hasattr(self.model, "from_parallelized"):
            self.model.from_parallelized(path)
        else:
            self.base_model.load_state_dict(torch.load(os.path.join(path, "pytorch_model.bin"), map_location="cpu"))
        if weights_only:
            if self.zero is not None and hasattr(self.zero, "resync_master"):
                self.zero.resync_master()
            return self.state.global_step
        opt_file = os.path.join(path, f"optimizer_{rank}.pt" if self.pc is not None else "optimizer.pt")
        if os.path.exists(opt_file):
            self.optimizer.load_state_dict(torch.load(opt_file, map_location="cpu", weights_only=False))
        elif self.zero is not None and hasattr(self.zero, "resync_master"):
            self.zero.resync_master()  # the fp32 master shards must follow the weights that were just loaded
        sched = os.path.join(path, "scheduler.pt")
        if os.path.exists(sched):
            self.lr_scheduler.load_state_dict(torch.load(sched))
        scaler = os.path.join(path, "scaler.pt")
        if self.scaler is not None and os.path.exists(scaler):
            self.scaler.load_state_dict(torch.load(scaler))
        rng_file = os.path.join(path, f"rng_state_{rank}.pth")
        if os.path.exists(rng_file):
            rng = torch.load(rng_file, weights_only=False)
            random.setstate(rng["python"])
            np.random.set_state(rng["numpy"])
            torch.set_rng_state(rng["cpu"])
            if "cuda" in rng and torch.cuda.is_available():
                torch.cuda.set_rng_state(rng["cuda"])
        with open(os.path.join(path, "trainer_state.json")) as f:
            saved = json.load(f)
        self.state.global_step = saved["global_step"]
        self.state.epoch = saved["epoch"]
        self.state.log_history = saved["log_history"]
        self.state.best_metric = saved.get("best_metric")
        return self.state.global_step


class _null:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False
