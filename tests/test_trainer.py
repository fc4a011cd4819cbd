"""Trainer: loss goes down, checkpoint + resume reproduces the uninterrupted run, config validation, profiler."""
import json
import math
import os
import tempfile

import pytest
import torch
from torch.utils.data import Dataset


class _Toy(Dataset):
    def __init__(self, n=64, seq=16, vocab=64):
        g = torch.Generator().manual_seed(0)
        base = torch.randint(0, vocab, (n, seq // 2), generator=g)
        self.ids = torch.cat([base, base], dim=1)  # second half repeats the first: learnable

    def __len__(self):
        return len(self.ids)

    def __getitem__(self, i):
        return {"input_ids": self.ids[i], "labels": self.ids[i]}


def _model():
    from oslo_b200.models import GPT2Config, GPT2LMHeadModel

    torch.manual_seed(0)
    return GPT2LMHeadModel(GPT2Config(vocab_size=64, n_positions=16, n_embd=32, n_layer=2, n_head=4, resid_pdrop=0.0,
                                      embd_pdrop=0.0, attn_pdrop=0.0))


def test_trainer_trains_and_resumes_identically():
    from oslo_b200.transformers import Trainer, TrainingArguments

    with tempfile.TemporaryDirectory() as tmp:
        args = TrainingArguments(output_dir=tmp, per_device_train_batch_size=8, learning_rate=3e-3, max_steps=12,
                                 logging_steps=4, save_steps=6, lr_scheduler_type="cosine", seed=1)
        t = Trainer(_model(), args, train_dataset=_Toy(), eval_dataset=_Toy(16))
        t.train()
        losses = [h["loss"] for h in t.state.log_history if "loss" in h]
        assert losses[-1] < losses[0]
        ev = t.evaluate()
        assert ev["eval_loss"] > 0
        final = {k: v.clone() for k, v in t.base_model.state_dict().items()}
        assert os.path.isdir(os.path.join(tmp, "checkpoint-6"))
        # resume from step 6 and finish: same final weights
        args2 = TrainingArguments(output_dir=tmp, per_device_train_batch_size=8, learning_rate=3e-3, max_steps=12,
                                  logging_steps=4, save_steps=0, lr_scheduler_type="cosine", seed=1)
        t2 = Trainer(_model(), args2, train_dataset=_Toy())
        t2.train(resume_from_checkpoint=os.path.join(tmp, "checkpoint-6"))
        for k, v in t2.base_model.state_dict().items():
            assert torch.allclose(v, final[k], rtol=1e-5, atol=1e-6), k


def test_config_validation():
    from oslo_b200.transformers import OsloTrainerConfig

    cfg = OsloTrainerConfig({"tensor_parallelism": {"parallel_size": 4, "parallel_mode": "2.5d", "params": {"parallel_depth_2.5d": 1}},
                             "data_parallelism": {"parallel_size": 2, "zero_stage": 2}})
    assert cfg.size("tensor_parallelism") == 4 and cfg.size("pipeline_parallelism") == 1
    with pytest.raises(KeyError):
        OsloTrainerConfig({"tensor_parallelism": {"paralel_size": 2}})
    with pytest.raises(ValueError):
        OsloTrainerConfig({"tensor_parallelism": {"parallel_mode": "4d"}})
    with pytest.raises(ValueError):
        OsloTrainerConfig({"data_parallelism": {"zero_stage": 7}})


def test_flops_profiler_counts_linear_layers():
    from oslo_b200.transformers import get_model_profile

    m = _model()
    ids = torch.randint(0, 64, (2, 16))
    flops, params, _ = get_model_profile(m, {"input_ids": ids})
    tokens = 32
    dense = 2 * tokens * (2 * (4 * 32 * 32 + 2 * 32 * 128) + 32 * 64)
    assert flops >= dense and flops < 3 * dense
    assert params == sum(p.numel() for p in m.parameters())


def test_flops_profiler_counts_functional_ops_and_reports_by_depth():
    """Activations, softmax, normalisation, convolution and scaled-dot-product attention are counted whichever Python
    entry point reaches them; MACs are tracked beside FLOPs and the report can be cut at a module depth."""
    import torch.nn as nn
    import torch.nn.functional as F

    from oslo_b200.transformers.profiler import FlopsProfiler, flops_to_string

    class Net(nn.Module):
        def __init__(self):
            super().__init__()
            self.conv = nn.Conv1d(8, 16, 3, padding=1)
            self.norm = nn.LayerNorm(16)
            self.fc = nn.Linear(16, 16)

        def forward(self, x):                       # x: [2, 8, 10]
            h = F.relu(self.conv(x)).transpose(1, 2)  # [2, 10, 16]
            h = self.norm(h)
            q = self.fc(h).view(2, 10, 2, 8).transpose(1, 2)
            a = F.scaled_dot_product_attention(q, q, q)
            return F.softmax(a, dim=-1).sum()

    net = Net()
    prof = FlopsProfiler(net)
    prof.start_profile()
    with torch.no_grad():
        net(torch.randn(2, 8, 10))
    prof.stop_profile()
    conv_macs = 2 * 16 * 10 * 8 * 3
    fc_macs = 2 * 10 * 16 * 16
    attn_macs = 2 * (2 * 2 * 10 * 10 * 8)
    assert prof.get_total_macs() >= conv_macs + fc_macs + attn_macs
    assert prof.macs["conv"] == conv_macs and prof.macs["fc"] == fc_macs
    # element-wise work on top of the multiply-accumulates: relu (320) + layer norm (5 x 320) + softmax (>= 320)
    assert prof.get_total_flops() >= 2 * prof.get_total_macs() + 320 + 5 * 320 + 320
    assert prof.flops["norm"] == 5 * 320
    text = prof.print_model_profile(module_depth=1, top_modules=3, output_file=None)
    assert "fwd FLOPs" in text and "conv" in text and "FLOPs" in flops_to_string(1e9)


def test_trainer_callbacks_predict_and_memory_metrics():
    """Callbacks see the loop's events and can stop it; ``predict`` returns predictions, labels and metrics; memory
    deltas are reported per stage when asked for."""
    from oslo_b200.transformers import EarlyStoppingCallback, Trainer, TrainerCallback, TrainingArguments

    class Recorder(TrainerCallback):
        def __init__(self):
            self.events = []

        def on_train_begin(self, args, state, control, **kw):
            self.events.append("train_begin")

        def on_step_end(self, args, state, control, **kw):
            self.events.append(("step_end", state.global_step))
            if state.global_step == 3:
                control.should_evaluate = True
            if state.global_step == 5:
                control.should_training_stop = True
            return control

        def on_evaluate(self, args, state, control, metrics=None, **kw):
            self.events.append(("evaluate", sorted(metrics)))

        def on_log(self, args, state, control, logs=None, **kw):
            self.events.append(("log", sorted(logs)))

        def on_train_end(self, args, state, control, **kw):
            self.events.append("train_end")

    with tempfile.TemporaryDirectory() as tmp:
        rec = Recorder()
        args = TrainingArguments(output_dir=tmp, per_device_train_batch_size=8, learning_rate=3e-3, max_steps=50, logging_steps=2,
                                 save_steps=0, seed=1, skip_memory_metrics=False)
        t = Trainer(_model(), args, train_dataset=_Toy(), eval_dataset=_Toy(16), callbacks=[rec, EarlyStoppingCallback(3)])
        metrics = t.train()
        assert t.state.global_step == 5  # stopped by the callback, not by max_steps
        assert rec.events[0] == "train_begin" and rec.events[-2] == "train_end"
        assert ("step_end", 3) in rec.events and any(e[0] == "evaluate" for e in rec.events if isinstance(e, tuple))
        assert "train_mem_cpu_alloc_delta" in metrics
        out = t.predict(_Toy(16))
        assert out.predictions.shape == out.label_ids.shape == (16, 16)
        assert out.metrics["test_loss"] > 0 and "test_mem_cpu_alloc_delta" in out.metrics


def test_scheduler_types_and_optimizer_names():
    from oslo_b200.transformers.trainer_utils import (OptimizerNames, SchedulerType, create_optimizer, get_scheduler, lr_factor,
                                                      log_dist)

    # closed forms of each schedule (warm-up 2 of 10 steps)
    assert lr_factor("linear", 0, 2, 10) == 0.5 and lr_factor("linear", 1, 2, 10) == 1.0
    assert abs(lr_factor("linear", 6, 2, 10) - 0.5) < 1e-12 and lr_factor("linear", 10, 2, 10) == 0.0
    assert abs(lr_factor("cosine", 6, 2, 10) - 0.5) < 1e-12
    assert abs(lr_factor("polynomial", 6, 2, 10, power=2.0) - 0.25) < 1e-12
    assert lr_factor("constant", 0, 2, 10) == 1.0 and lr_factor("constant_with_warmup", 0, 2, 10) == 0.5
    assert lr_factor("constant_with_warmup", 9, 2, 10) == 1.0
    # two restarts: the factor returns to 1 at the middle of the decay phase
    assert abs(lr_factor("cosine_with_restarts", 6, 2, 10, num_cycles=2) - 1.0) < 1e-12
    assert lr_factor("cosine_with_restarts", 5, 2, 10, num_cycles=2) < 0.2
    with pytest.raises(ValueError):
        SchedulerType("nope")
    assert OptimizerNames("lamb") == "lamb"
    w = torch.nn.Parameter(torch.ones(4))
    for name in ("adam", "adamw", "sgd", "adagrad", "adadelta", "cpu_adam", "cpu_adagrad"):
        w.grad = torch.ones(4)
        before = w.detach().clone()
        opt = create_optimizer(name, [w], lr=0.1)
        opt.step()
        assert (w.detach() < before).all(), name
    sched = get_scheduler("linear", torch.optim.SGD([w], lr=1.0), 0, 4)
    seen = []
    for _ in range(4):
        seen.append(sched.get_last_lr()[0])
        sched.optimizer.step()
        sched.step()
    assert seen == [1.0, 0.75, 0.5, 0.25]
    assert log_dist("hello", rank=0) and not log_dist("hello", rank=3)


def test_epoch_strategies_best_model_reload_and_log_sink():
    from oslo_b200.transformers import Trainer, TrainingArguments

    with tempfile.TemporaryDirectory() as tmp:
        args = TrainingArguments(output_dir=tmp, per_device_train_batch_size=8, learning_rate=3e-3, num_train_epochs=2,
                                 logging_strategy="epoch", evaluation_strategy="epoch", save_strategy="epoch",
                                 load_best_model_at_end=True, logging_dir=os.path.join(tmp, "logs"), seed=1)
        assert args.metric_for_best_model == "eval_loss"
        t = Trainer(_model(), args, train_dataset=_Toy(), eval_dataset=_Toy(16))
        t.train()
        steps_per_epoch = len(_Toy()) // 8
        assert os.path.isdir(os.path.join(tmp, f"checkpoint-{steps_per_epoch}"))
        assert os.path.isdir(os.path.join(tmp, f"checkpoint-{2 * steps_per_epoch}"))
        losses = [h for h in t.state.log_history if "loss" in h]
        evals = [h for h in t.state.log_history if "eval_loss" in h]
        assert len(losses) == 2 and len(evals) == 2
        assert t.state.best_model_checkpoint is not None
        # the reloaded weights are those of the best checkpoint
        best = torch.load(os.path.join(t.state.best_model_checkpoint, "pytorch_model.bin"), map_location="cpu")
        for k, v in t.base_model.state_dict().items():
            assert torch.equal(v.cpu(), best[k]), k
        with open(os.path.join(tmp, "logs", "log.jsonl")) as f:
            lines = [json.loads(line) for line in f]
        assert len(lines) == len(t.state.log_history)
    with pytest.raises(ValueError):
        TrainingArguments(save_strategy="sometimes")
    with pytest.raises(ValueError):
        TrainingArguments(optim="adamz")


def test_label_smoothing_unused_columns_and_length_grouping():
    from oslo_b200.transformers import Trainer, TrainingArguments
    from oslo_b200.transformers.trainer import LengthGroupedSampler

    class _Extra(_Toy):
        def __getitem__(self, i):
            d = super().__getitem__(i)
            d["not_a_model_argument"] = torch.zeros(1)
            return d

    class _Strict(torch.nn.Module):
        shift_labels = True

        def __init__(self):
            super().__init__()
            self.inner = _model()

        def forward(self, input_ids, labels=None):
            return self.inner(input_ids=input_ids, labels=labels)

    with tempfile.TemporaryDirectory() as tmp:
        model = _Strict()
        t = Trainer(model, TrainingArguments(output_dir=tmp, label_smoothing_factor=0.1, max_steps=1, save_steps=0), train_dataset=_Extra())
        batch = {"input_ids": torch.arange(16).view(1, 16) % 64, "labels": torch.arange(16).view(1, 16) % 64,
                 "not_a_model_argument": torch.zeros(1)}
        moved = t._move(batch)
        assert "not_a_model_argument" not in moved
        with torch.no_grad():
            got = t.compute_loss(moved)
            logits = model(input_ids=moved["input_ids"]).logits[:, :-1].float()
            want = torch.nn.functional.cross_entropy(logits.reshape(-1, 64), moved["labels"][:, 1:].reshape(-1), label_smoothing=0.1)
        assert torch.allclose(got, want, rtol=1e-5, atol=1e-6)
        t.train()  # the extra column does not reach the model
    lengths = [int(x) for x in torch.randint(1, 100, (64,), generator=torch.Generator().manual_seed(0))]
    parts = [list(LengthGroupedSampler(list(range(64)), 4, num_replicas=2, rank=r, seed=3, lengths=lengths)) for r in (0, 1)]
    assert sorted(parts[0] + parts[1]) == list(range(64))
    spread = [max(lengths[i] for i in parts[0][b:b + 4]) - min(lengths[i] for i in parts[0][b:b + 4]) for b in range(0, 32, 4)]
    assert sum(spread) / len(spread) < 25  # random batches of four would spread over ~60


def test_fp16_training_uses_the_dynamic_loss_scaler_and_checkpoints_it():
    from oslo_b200.transformers import Trainer, TrainingArguments

    with tempfile.TemporaryDirectory() as tmp:
        args = TrainingArguments(output_dir=tmp, per_device_train_batch_size=8, learning_rate=1e-3, max_steps=8, logging_steps=2,
                                 save_steps=8, fp16=True, fp16_init_scale=2.0 ** 40, fp16_growth_interval=3, seed=1)
        t = Trainer(_model(), args, train_dataset=_Toy())
        t.train()
        assert t.scaler is not None and next(t.base_model.parameters()).dtype == torch.float16
        # 2^40 overflows fp16 gradients: the first steps are skipped (weights untouched) while the scale backs off
        assert t.scaler.skipped_steps >= 1 and t.scaler.get_scale() < 2.0 ** 40
        assert all(torch.isfinite(p).all() for p in t.base_model.parameters())
        losses = [h["loss"] for h in t.state.log_history if "loss" in h]
        assert all(math.isfinite(v) for v in losses)
        saved = torch.load(os.path.join(tmp, "checkpoint-8", "scaler.pt"))
        assert saved["scale"] == t.scaler.get_scale() and saved["skipped_steps"] == t.scaler.skipped_steps
        # the schedule advanced only on the steps that were taken
        assert t.lr_scheduler.last_epoch == 8 - t.scaler.skipped_steps
        t2 = Trainer(_model(), TrainingArguments(output_dir=tmp, per_device_train_batch_size=8, max_steps=9, fp16=True, save_steps=0, seed=1),
                     train_dataset=_Toy())
        t2.train(resume_from_checkpoint=os.path.join(tmp, "checkpoint-8"))
        assert t2.scaler.skipped_steps >= t.scaler.skipped_steps


_DIST_CONFIGS = {
    "tp1d_sp": (2, {"tensor_parallelism": {"parallel_size": 2, "parallel_mode": "1d", "sequence_parallel": True}}),
    "zero2": (2, {"data_parallelism": {"parallel_size": 2, "zero_stage": 2}}),
    "zero3": (2, {"data_parallelism": {"parallel_size": 2, "zero_stage": 3}}),
    "pp": (2, {"pipeline_parallelism": {"parallel_size": 2, "params": {"num_micro_batches": 2}}}),
    "tp2d": (4, {"tensor_parallelism": {"parallel_size": 4, "parallel_mode": "2d"}}),
    "tp_dp_ckpt": (4, {"tensor_parallelism": {"parallel_size": 2, "parallel_mode": "1d"},
                       "data_parallelism": {"parallel_size": 2, "zero_stage": 1},
                       "activation_checkpointing": {"partitioned": True}}),
}


def _dist_trainer_worker(rank, world, name, tmp):
    """``Trainer`` driven by a configuration dict on CPU ranks: trains, logs the same finite loss on every rank (under
    pipeline parallelism too, where only the last stage computes it), evaluates, checkpoints, and a second trainer resumed
    from the mid-run checkpoint ends with the same loss."""
    import torch.distributed as dist

    from oslo_b200.transformers import Trainer, TrainingArguments

    cfg = dict(_DIST_CONFIGS[name][1], backend={"name": "gloo"})
    common = dict(output_dir=tmp, per_device_train_batch_size=8, learning_rate=3e-3, logging_steps=2, seed=1)
    args = TrainingArguments(max_steps=6, save_steps=4, oslo_config_path_or_dict=cfg, **common)
    t = Trainer(_model(), args, train_dataset=_Toy(), eval_dataset=_Toy(16))
    t.train()
    losses = [h["loss"] for h in t.state.log_history if "loss" in h]
    assert len(losses) == 3 and all(math.isfinite(v) and v > 0 for v in losses), (name, losses)
    gathered = [None] * world
    dist.all_gather_object(gathered, losses)
    dp = cfg.get("data_parallelism", {}).get("parallel_size", 1)
    assert all(max(abs(a - b) for a, b in zip(g, gathered[0])) < 1e-5 for g in gathered) or dp > 1, gathered
    ev = t.evaluate()
    assert math.isfinite(ev["eval_loss"]) and ev["eval_loss"] > 0
    assert os.path.isdir(os.path.join(tmp, "checkpoint-4"))
    dist.barrier()
    args2 = TrainingArguments(max_steps=6, save_steps=0, parallel_context=args.parallel_context, wrapper_recipes=args.wrapper_recipes,
                              oslo_config=args.oslo_config, **common)
    t2 = Trainer(_model(), args2, train_dataset=_Toy())
    t2.train(resume_from_checkpoint=os.path.join(tmp, "checkpoint-4"))
    resumed = [h["loss"] for h in t2.state.log_history if "loss" in h]
    assert abs(resumed[-1] - losses[-1]) < 2e-4, (name, resumed, losses)


@pytest.mark.parametrize("name", list(_DIST_CONFIGS))
def test_trainer_under_parallel_configurations(name):
    from dist_utils import run_dist

    with tempfile.TemporaryDirectory() as tmp:
        run_dist(_dist_trainer_worker, _DIST_CONFIGS[name][0], name, tmp, timeout=600)


def _predict_tp_worker(rank, world, mode, tmp):
    from oslo_b200.transformers import Trainer, TrainingArguments

    cfg = {"tensor_parallelism": {"parallel_size": world, "parallel_mode": mode}, "backend": {"name": "gloo"}}
    args = TrainingArguments(output_dir=tmp, per_device_eval_batch_size=8, oslo_config_path_or_dict=cfg)
    ref = _model().eval()
    out = Trainer(_model(), args, eval_dataset=_Toy(16)).predict(_Toy(16))
    data = _Toy(16)
    ids = torch.stack([data[i]["input_ids"] for i in range(16)])
    with torch.no_grad():
        want = ref(input_ids=ids).logits.argmax(-1)
    assert out.predictions.shape == want.shape and torch.equal(out.predictions, want)  # not the argmax of a vocabulary shard


@pytest.mark.parametrize("mode,world", [("1d", 2), ("2d", 4)])
def test_predict_under_tensor_parallelism_sees_whole_logits(mode, world):
    from dist_utils import run_dist

    with tempfile.TemporaryDirectory() as tmp:
        run_dist(_predict_tp_worker, world, mode, tmp, timeout=600)


def test_mixed_precision_section_selects_the_compute_dtype(monkeypatch):
    from oslo_b200.transformers import TrainingArguments

    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "MASTER_ADDR", "MASTER_PORT"):
        monkeypatch.delenv(k, raising=False)
    cfg = {"mixed_precision": {"enable": True, "dtype": "bf16"}, "backend": {"name": "gloo"}}
    args = TrainingArguments(output_dir="unused", oslo_config_path_or_dict=cfg)
    try:
        assert args.bf16 and not args.fp16 and args.dtype == torch.bfloat16
        with pytest.raises(ValueError):
            TrainingArguments(output_dir="unused", fp16=True, oslo_config=args.oslo_config, parallel_context=args.parallel_context)
        off = TrainingArguments(output_dir="unused", parallel_context=args.parallel_context,
                                oslo_config=type(args.oslo_config)({"mixed_precision": {"enable": False, "dtype": "bf16"}}))
        assert off.dtype == torch.float32
    finally:
        args.parallel_context.destroy()
