"""Reference arm of ``bench.py``: the unmodified EleutherAI/oslo package, driven through its own public API.

The package is installed (``pip install --no-deps --target baseline/_ref``) and its files are left byte-identical.
What runs is the reference's stock 1-D tensor-parallel path:

    ParallelContext.from_torch(tensor_parallel_size=N)          oslo/torch/distributed/parallel_context.py:182-245
    TensorParallel(model, parallel_context)                     oslo/torch/nn/parallel/tensor_parallel/tensor_parallel.py:51-62
    oslo.ready(model, parallel_context)                         oslo/__init__.py:5-6
    ColLinear1D / RowLinear1D / VocabParallelEmbedding1D        oslo/torch/nn/modules/linear.py:73-160

on a Hugging Face ``GPTNeoXForCausalLM`` of the benchmark's dimensions (the reference has a GPTNeoX mapping,
oslo/transformers/mapping_utils.py:174-180), bf16 weights, ``torch.optim.AdamW``, same batch, same timing rules
and the same JSON keys as the repository's own arm.  None of this repository's models, kernels or engine is
imported here.

One shim is needed and is declared in the JSON line under ``"shims"``: ``import oslo`` JIT-compiles a
generation-only n-gram blocking extension (oslo/torch/nn/modules/ngram_repeat_block.py:12-19) that does not
compile against torch 2.11 headers.  The reference already falls back when that import raises ``ImportError``;
the binder class is replaced, in ``sys.modules`` only, by a stand-in that raises exactly that.
"""
from __future__ import annotations

import json
import os
import sys
import time
import traceback

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")

SHIMS = ["oslo.torch._C.NgramRepeatBlockBinder -> stand-in raising ImportError (generation-only JIT extension "
         "does not compile on torch 2.11; the reference's own except-ImportError fallback then applies)",
         "oslo.lightseq2 OpBuilder.load -> placeholder (import-time JIT of all LightSeq kernels, pulled in "
         "by the BERT fork, refuses nvcc 12.9 with a cu128 torch; no LightSeq kernel is on this path)"]


def _install_shim():
    """Patch two reference modules the moment the import system has executed them (they import ``oslo`` themselves, so
    they cannot be loaded ahead of the package).  A meta-path finder wraps those modules' loaders:

    * ``oslo.torch._C``: the n-gram binder becomes a class whose construction raises ImportError;
    * ``oslo.lightseq2.training.ops.pytorch.builder.builder``: ``OpBuilder.load`` (run at import
      time by the LightSeq layers that the BERT fork imports, oslo/transformers/models/bert/modeling_bert.py:19)
      returns a placeholder instead of JIT-compiling every LightSeq kernel; the build refuses this image outright
      (nvcc 12.9 vs a cu128 torch, builder.py:66) and no LightSeq kernel is on the GPT-NeoX training path."""
    import importlib.abc
    import importlib.machinery

    class NgramRepeatBlockBinder:  # stand-in
        def __init__(self, *a, **k):
            raise ImportError("n-gram blocking extension not built (bench shim)")

    class _NotBuilt:
        def __getattr__(self, name):
            raise ImportError(f"LightSeq extension not built (bench shim): {name}")

    def _patch_c(module):
        module.NgramRepeatBlockBinder = NgramRepeatBlockBinder

    def _patch_ls(module):
        module.OpBuilder.load = lambda self, verbose=True: _NotBuilt()

    patches = {
        "oslo.torch._C": _patch_c,
        "oslo.lightseq2.training.ops.pytorch.builder.builder": _patch_ls,
    }

    class _Loader(importlib.abc.Loader):
        def __init__(self, inner, patch):
            self.inner, self.patch = inner, patch

        def create_module(self, spec):
            return self.inner.create_module(spec)

        def exec_module(self, module):
            self.inner.exec_module(module)
            self.patch(module)

    class _Finder(importlib.abc.MetaPathFinder):
        def find_spec(self, name, path, target=None):
            if name not in patches:
                return None
            spec = importlib.machinery.PathFinder.find_spec(name, path, target)
            if spec is not None and spec.loader is not None:
                spec.loader = _Loader(spec.loader, patches[name])
            return spec

    sys.meta_path.insert(0, _Finder())
    _install_missing_dependencies()


def _install_missing_dependencies():
    """Third-party packages that the reference lists in its requirements but that are neither in this image nor in the
    offline wheelhouse get an empty stand-in, so that modules which import them at top level (the pipeline partitioner,
    not on the tensor-parallel training path) still import.  Using one of the stand-ins raises."""
    import importlib
    import types

    def _absent(name):
        try:
            importlib.import_module(name)
            return False
        except ImportError:
            return True

    if _absent("anytree"):
        mod = types.ModuleType("anytree")

        class Node:  # placeholder for anytree.Node
            def __init__(self, *a, **k):
                raise ImportError("anytree is not installed (bench stand-in)")

        mod.Node = Node
        sys.modules["anytree"] = mod
        SHIMS.append("anytree (absent from the image and the wheelhouse) -> empty stand-in module; only imported "
                     "by the pipeline partitioner, never used on this path")

    # Names that the reference's model forks import from Hugging Face transformers and that transformers 5.x removed.
    # `oslo/transformers/__init__.py` imports every fork, and the tensor-parallel wrapper imports that package, so the
    # names must resolve; none of them is called on the GPT-NeoX training path.
    import transformers  # noqa: F401

    def _placeholder(qualname):
        class _Removed:
            def __init__(self, *a, **k):
                raise ImportError(f"{qualname} was removed from transformers 5.x (bench stand-in)")

        _Removed.__name__ = qualname.rsplit(".", 1)[-1]
        return _Removed

    removed = {
        "transformers.modeling_utils": ["SequenceSummary", "find_pruneable_heads_and_indices", "prune_conv1d_layer"],
        "transformers.pytorch_utils": ["find_pruneable_heads_and_indices"],
        "transformers.models.albert": ["load_tf_weights_in_albert"],
        "transformers.models.bert.modeling_bert": ["load_tf_weights_in_bert"],
        "transformers.models.gpt2.modeling_gpt2": ["load_tf_weights_in_gpt2"],
        "transformers.models.t5": ["load_tf_weights_in_t5"],
    }
    added = []
    for modname, names in removed.items():
        mod = importlib.import_module(modname)
        for n in names:
            if not hasattr(mod, n):
                setattr(mod, n, _placeholder(f"{modname}.{n}"))
                added.append(f"{modname}.{n}")
    for modname in ("transformers.deepspeed", "transformers.generation_utils",
                    "transformers.generation_logits_process", "transformers.models.bart.modeling_flax_bart"):
        if _absent(modname):
            mod = types.ModuleType(modname)
            mod.__getattr__ = lambda n, _m=modname: _placeholder(f"{_m}.{n}")
            sys.modules[modname] = mod
            parent, _, leaf = modname.rpartition(".")
            try:
                setattr(importlib.import_module(parent), leaf, mod)
            except Exception:
                pass
            added.append(modname)
    if added:
        SHIMS.append("Hugging Face names removed in transformers 5.x, imported at top level by the reference's model "
                     "forks, -> placeholders that raise if called: " + ", ".join(added))


def _one_line(text: str, limit: int = 600) -> str:
    text = " | ".join(l.strip() for l in text.strip().splitlines() if l.strip())
    return text[-limit:]


def run(args, configs, model_flops_per_token, ClockSampler) -> int:
    rank = int(os.environ.get("RANK", "0"))
    try:
        return _run(args, configs, model_flops_per_token, ClockSampler)
    except BaseException as e:  # the line must still be printed, with this attempt's own traceback
        if isinstance(e, KeyboardInterrupt):
            raise
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": _one_line(traceback.format_exc()),
                              "shims": SHIMS}), flush=True)
        return 0


def _run(args, configs, model_flops_per_token, ClockSampler) -> int:
    if not os.path.isdir(os.path.join(REF, "oslo")):
        raise RuntimeError("baseline/_ref/oslo is missing: run `python -m pip install --no-index "
                           "--no-build-isolation --no-deps --find-links /opt/wheelhouse --target baseline/_ref "
                           "<copy of the reference>` first")
    args.warmup = max(args.warmup, 3)
    if "RANK" not in os.environ:
        if args.gpus != 1:
            raise SystemExit("for --gpus N > 1 launch with torch.distributed.run (one rank per GPU)")
        os.environ.update(RANK="0", LOCAL_RANK="0", WORLD_SIZE="1", LOCAL_WORLD_SIZE="1",
                          MASTER_ADDR="127.0.0.1", MASTER_PORT=str(29500 + os.getpid() % 2000))
    os.environ.setdefault("LOCAL_WORLD_SIZE", os.environ["WORLD_SIZE"])
    world = int(os.environ["WORLD_SIZE"])
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}"

    import warnings

    warnings.filterwarnings("ignore")
    import torch
    import torch.distributed as dist

    sys.path.insert(0, REF)
    _install_shim()
    import oslo  # the reference package
    from oslo.torch.distributed import ParallelContext, ParallelMode
    from oslo.torch.nn.parallel import TensorParallel
    from transformers import GPTNeoXConfig, GPTNeoXForCausalLM

    assert os.path.realpath(oslo.__file__).startswith(os.path.realpath(REF)), oslo.__file__

    pc = ParallelContext.from_torch(tensor_parallel_size=world, tensor_parallel_mode=ParallelMode.TENSOR_1D,
                                    backend="nccl", seed=1234)
    rank = dist.get_rank()
    dev = torch.device("cuda", torch.cuda.current_device())
    cfg = dict(configs[args.model])
    B, S = cfg.pop("global_batch"), cfg.pop("seq_len")
    hf_cfg = GPTNeoXConfig(use_parallel_residual=True, hidden_act="gelu", hidden_dropout=0.0,
                           attention_dropout=0.0, use_cache=False, tie_word_embeddings=False, **cfg)

    torch.manual_seed(1234)
    model = GPTNeoXForCausalLM(hf_cfg).to(torch.bfloat16)
    n_params = sum(p.numel() for p in model.parameters())
    model = TensorParallel(model, parallel_context=pc)
    oslo.ready(model, pc)  # shards the weights and moves the model to this rank's GPU
    model.train()
    opt = torch.optim.AdamW(model.parameters(), lr=1e-4, weight_decay=0.01, fused=True)

    gen = torch.Generator().manual_seed(99)
    host_ids = [torch.randint(0, hf_cfg.vocab_size, (B, S), generator=gen).pin_memory() for _ in range(4)]
    dev_ids = [t.to(dev) for t in host_ids]

    def step(ids):
        opt.zero_grad()
        loss = model(input_ids=ids, labels=ids).loss
        loss.backward()
        opt.step()
        return loss

    def timed(n_steps, e2e: bool):
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        e0.record()
        last = None
        for i in range(n_steps):
            if e2e:
                ids = host_ids[i % len(host_ids)].to(dev, non_blocking=True)
                last = float(step(ids))
            else:
                last = step(dev_ids[i % len(dev_ids)])
        e1.record()
        torch.cuda.synchronize()
        wall = (time.perf_counter() - t0) * 1e3
        dist.barrier()
        t = torch.tensor([e0.elapsed_time(e1), wall], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t[0].item(), t[1].item(), float(last)

    for i in range(args.warmup):
        step(dev_ids[i % len(dev_ids)])
    torch.cuda.synchronize()

    sampler = ClockSampler(torch.cuda.current_device())
    sampler.start()
    ms, _, loss_val = timed(args.steps, e2e=False)
    ms_e2e, wall_e2e, _ = timed(args.steps, e2e=True)
    clocks = sampler.stop()

    tokens = B * S * args.steps
    value = tokens / (ms / 1e3)
    e2e_value = tokens / (max(ms_e2e, wall_e2e) / 1e3)
    flops_tok = model_flops_per_token(dict(cfg, seq_len=S))
    if rank == 0:
        out = {
            "metric": "train tokens/sec (device-timed, max over ranks), 1D tensor parallel + sequence parallel",
            "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic uniform token ids, random-init N(0, 0.02) weights",
            "impl": "reference", "shims": SHIMS,
            "config": {
                "model": f"GPT-NeoX-style {args.model} ({n_params / 1e9:.2f}B params), Hugging Face "
                         "GPTNeoXForCausalLM under the reference's TensorParallel",
                "global_batch": B, "seq_len": S,
                "parallelism": f"tp{world} (the reference's 1-D mode has no sequence parallelism)",
                "optimizer": "torch.optim.AdamW(fused=True) on bf16 parameters",
                "attention": str(getattr(hf_cfg, "_attn_implementation", None)),
                "l2_policy": "inputs larger than L2: every step streams > 126 MB of weights and activations",
            },
            "mfu": {"model_tflops_per_s": value * flops_tok / 1e12,
                    "per_gpu_tflops": value * flops_tok / 1e12 / world},
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": B * S * 8,
                    "d2h_bytes_per_step": 4, "ms_per_step": max(ms_e2e, wall_e2e) / args.steps},
            "gpu_launches": 0,
            "loss": loss_val,
        }
        print(json.dumps(out), flush=True)
    dist.barrier()
    torch.cuda.synchronize()
    dist.destroy_process_group()
    return 0
