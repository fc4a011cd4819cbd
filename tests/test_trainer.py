"""Trainer: loss goes down, checkpoint + resume reproduces the uninterrupted run, config validation, profiler."""
import json
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
