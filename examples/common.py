"""Shared pieces of the example scripts: argument parsing, model presets, synthetic / text data.

The three scripts mirror the reference's end-to-end examples (tests/training.py, tests/merge.py, tests/inference.py with
tests/util/arg_parser.py): train a model under a chosen mix of data / tensor / pipeline parallelism, merge the per-rank
checkpoint shards into one file, and run inference from either form.  They run on GPUs (NCCL) or, with ``--cpu``, on CPU
ranks (gloo), and need no download: models are random-initialised presets and the data is synthetic unless ``--text-file``
is given.
"""
from __future__ import annotations

import argparse
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

TASKS = ("causal-lm", "sequence-classification", "seq2seq")
PRESETS = {
    # name -> (family, keyword arguments of the config)
    "gpt2-tiny": ("gpt2", dict(vocab_size=512, n_positions=128, n_embd=64, n_layer=2, n_head=4, resid_pdrop=0.0, embd_pdrop=0.0,
                               attn_pdrop=0.0)),
    "gpt2": ("gpt2", dict(vocab_size=50304, n_positions=1024, n_embd=768, n_layer=12, n_head=12)),
    "gpt-neox-tiny": ("gpt_neox", dict(vocab_size=512, hidden_size=64, num_hidden_layers=2, num_attention_heads=4,
                                       intermediate_size=256, max_position_embeddings=128)),
    "gpt-neox-1.3b": ("gpt_neox", dict(vocab_size=50304, hidden_size=2048, num_hidden_layers=24, num_attention_heads=16,
                                       intermediate_size=8192, max_position_embeddings=2048)),
    "bert-tiny": ("bert", dict(vocab_size=512, hidden_size=64, num_hidden_layers=2, num_attention_heads=4, intermediate_size=128,
                               max_position_embeddings=128, hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0)),
    "bert-base": ("bert", dict(vocab_size=30528)),
    "t5-tiny": ("t5", dict(vocab_size=512, d_model=64, d_kv=16, d_ff=128, num_layers=2, num_decoder_layers=2, num_heads=4,
                           dropout_rate=0.0)),
    "t5-base": ("t5", dict(vocab_size=32128, d_model=768, d_kv=64, d_ff=3072, num_layers=12, num_heads=12)),
}
MODES = {"1d": "TENSOR_1D", "2d": "TENSOR_2D", "2.5d": "TENSOR_2P5D", "3d": "TENSOR_3D"}


def get_args(description: str, training: bool = True):
    ap = argparse.ArgumentParser(description=description)
    ap.add_argument("--model", default="gpt2-tiny", choices=sorted(PRESETS))
    ap.add_argument("--task", default="causal-lm", choices=TASKS)
    ap.add_argument("--tensor_parallel_size", type=int, default=1)
    ap.add_argument("--tensor_parallel_mode", default="1d", choices=sorted(MODES))
    ap.add_argument("--tensor_parallel_depth", type=int, default=1)
    ap.add_argument("--data_parallel_size", type=int, default=1)
    ap.add_argument("--pipeline_parallel_size", type=int, default=1)
    ap.add_argument("--sequence_length", type=int, default=32)
    ap.add_argument("--batch_size", type=int, default=4, help="per data-parallel rank")
    ap.add_argument("--cpu", action="store_true", help="gloo ranks on the CPU")
    ap.add_argument("--dtype", default=None, choices=["fp32", "bf16"], help="default: bf16 on GPUs, fp32 on CPU")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--save_dir", default="example_ckpt")
    if training:
        ap.add_argument("--train_step", type=int, default=20)
        ap.add_argument("--save_interval", type=int, default=0, help="0: save once at the end")
        ap.add_argument("--lr", type=float, default=1e-3)
        ap.add_argument("--micro_batches", type=int, default=2, help="pipeline micro-batches")
        ap.add_argument("--zero_stage", type=int, default=0, choices=[0, 1, 2])
        ap.add_argument("--text-file", default=None, help="train on this text (byte-level) instead of synthetic tokens")
        ap.add_argument("--merge", action="store_true", help="also write the merged single-file checkpoint")
        ap.add_argument("--check_parity", action="store_true",
                        help="train an unsharded twin on the same global batches (every rank, fp32 recommended) and fail if the "
                             "losses drift apart by more than --parity_tol")
        ap.add_argument("--parity_tol", type=float, default=2e-3)
    return ap


def build_context(args):
    from oslo_b200 import ParallelContext, ParallelMode

    return ParallelContext.from_torch(
        data_parallel_size=args.data_parallel_size, tensor_parallel_size=args.tensor_parallel_size,
        pipeline_parallel_size=args.pipeline_parallel_size, tensor_parallel_mode=getattr(ParallelMode, MODES[args.tensor_parallel_mode]),
        tensor_parallel_depth=args.tensor_parallel_depth if args.tensor_parallel_mode == "2.5d" else None,
        backend="gloo" if args.cpu else "nccl", seed=args.seed)


def build_model(args):
    """Random-initialised model of the preset, with the head the task needs (same seed on every rank)."""
    from oslo_b200 import models

    family, kw = PRESETS[args.model]
    torch.manual_seed(args.seed)
    if family == "gpt2":
        return models.GPT2LMHeadModel(models.GPT2Config(**kw))
    if family == "gpt_neox":
        from oslo_b200.models.config import GPTNeoXConfig
        from oslo_b200.models.gpt_neox import GPTNeoXForCausalLM

        return GPTNeoXForCausalLM(GPTNeoXConfig(**kw))
    if family == "bert":
        cfg = models.BertConfig(**kw, num_labels=3)
        return models.BertForSequenceClassification(cfg) if args.task == "sequence-classification" else models.BertForMaskedLM(cfg)
    if family == "t5":
        return models.T5ForConditionalGeneration(models.T5Config(**kw))
    raise ValueError(family)


def dtype_of(args):
    name = args.dtype or ("fp32" if args.cpu else "bf16")
    return torch.float32 if name == "fp32" else torch.bfloat16


def batches(args, vocab: int, dp_rank: int, device, steps: int):
    """Yield ``steps`` batches of this data-parallel rank: a cyclic arithmetic token pattern the models can learn, or
    windows of ``--text-file`` bytes."""
    g = torch.Generator().manual_seed(1000 + args.seed + dp_rank)
    data = None
    if getattr(args, "text_file", None):
        with open(args.text_file, "rb") as f:
            data = torch.tensor(list(f.read()), dtype=torch.long) % vocab
    b, s = args.batch_size, args.sequence_length
    for _ in range(steps):
        if data is not None and data.numel() > s + 1:
            starts = torch.randint(0, data.numel() - s, (b,), generator=g)
            ids = torch.stack([data[i : i + s] for i in starts.tolist()])
        else:
            start = torch.randint(0, vocab, (b, 1), generator=g)
            stride = torch.randint(1, 4, (b, 1), generator=g)
            ids = (start + stride * torch.arange(s)) % vocab
        batch = {"input_ids": ids.to(device)}
        if args.task == "causal-lm":
            batch["labels"] = batch["input_ids"]
        elif args.task == "sequence-classification":
            batch["labels"] = (ids[:, 1] - ids[:, 0]).remainder(vocab).clamp(max=3).sub(1).clamp(min=0).to(device)
        else:  # seq2seq: reproduce the input shifted by its stride
            batch["labels"] = ((ids + (ids[:, 1:2] - ids[:, 0:1])) % vocab).to(device)
        yield batch
