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
