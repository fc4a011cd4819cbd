"""Train a preset model under data / tensor / pipeline parallelism and save per-rank checkpoint shards.

    python -m torch.distributed.run --nproc-per-node 4 --master-addr 127.0.0.1 examples/train.py \
        --model gpt-neox-tiny --tensor_parallel_size 2 --data_parallel_size 2 --train_step 50 --merge

``--check_parity`` additionally trains an unsharded copy of the model on the same global batches on every rank and compares
the two losses step by step (the reference's loss-parity scripts do this against a plain / DDP model).  ``--cpu`` runs the
same thing on gloo ranks.  Rank 0 prints the loss every few steps and, at the end, where the
checkpoint went (``pytorch_model_tp_{t}_pp_{p}_ep_{e}.bin`` per rank, plus ``pytorch_model.bin`` with ``--merge``).
"""
from __future__ import annotations

import json

from common import batches, build_context, build_model, dtype_of, get_args

import torch


def main(argv=None):
    args = get_args(__doc__).parse_args(argv)
    import oslo_b200
    from oslo_b200 import ParallelMode
    from oslo_b200.optim import FusedAdam
    from oslo_b200.parallel import DistributedDataParallel, PipelineParallel, TensorParallel, ZeroRedundancyOptimizer

    pc = build_context(args)
    rank = pc.get_global_rank()
    model = build_model(args).to(dtype_of(args))
    vocab = model.config.vocab_size
    wrapped = model
    if args.tensor_parallel_size > 1:
        wrapped = TensorParallel(wrapped, pc)
    if args.pipeline_parallel_size > 1:
        wrapped = PipelineParallel(wrapped, pc, num_micro_batches=args.micro_batches)
    if args.data_parallel_size > 1 and args.zero_stage == 0 and args.pipeline_parallel_size == 1:
        wrapped = DistributedDataParallel(wrapped, pc)
    oslo_b200.ready(wrapped, pc)
    params = [p for p in model.parameters() if p.requires_grad and p.numel() > 0]
    if args.zero_stage:
        opt = ZeroRedundancyOptimizer(torch.optim.AdamW(params, lr=args.lr), parallel_context=pc, partition_grad=args.zero_stage == 2)
    else:
        opt = FusedAdam(params, lr=args.lr, master_weights=dtype_of(args) != torch.float32)
    dp_rank = pc.get_local_rank(ParallelMode.DATA)
    history = []
    twin = twin_opt = None
    streams = [batches(args, vocab, r, pc.device, args.train_step) for r in range(args.data_parallel_size)]
    if args.check_parity:
        # built BEFORE the wrappers shard anything would be ideal; the presets are seeded, so building again is the same model
        twin = build_model(args).to(dtype_of(args)).to(pc.device)
        twin_opt = torch.optim.AdamW(twin.parameters(), lr=args.lr, weight_decay=0.0)
    worst = 0.0
    for step in range(1, args.train_step + 1):
        per_rank = [next(s) for s in streams]
        batch = per_rank[dp_rank]
        twin_loss = None
        if twin is not None:
            full = {k: torch.cat([b[k] for b in per_rank]) for k in batch}
            twin_opt.zero_grad()
            twin_loss = twin(**full).loss
            twin_loss.backward()
            twin_opt.step()
        opt.zero_grad()
        if args.pipeline_parallel_size > 1:
            loss = None
            for _, out in wrapped(**batch):
                if torch.is_tensor(getattr(out, "loss", None)):
                    (out.loss / args.micro_batches).backward()
                    loss = out.loss.detach() if loss is None else loss + out.loss.detach()
            loss = loss / args.micro_batches if loss is not None else None
        else:
            loss = wrapped(**batch).loss
            if args.zero_stage:
                opt.backward(loss)
            else:
                loss.backward()
        opt.step()
        if loss is not None and twin_loss is not None:
            # the parallel loss is this rank's data-parallel share; average the shares before comparing
            mine = loss.detach().float().clone()
            if args.data_parallel_size > 1:
                import torch.distributed as dist

                dist.all_reduce(mine, group=pc.get_group(ParallelMode.DATA))
                mine /= args.data_parallel_size
            twin_loss = twin_loss.detach()
            worst = max(worst, abs(float(mine) - float(twin_loss)))
            loss = mine  # report the data-parallel mean, which is what the twin computes
        if loss is not None and (step % 5 == 0 or step == 1 or step == args.train_step):
            history.append((step, float(loss)))
            if rank == 0 or (args.pipeline_parallel_size > 1 and pc.is_last_rank(ParallelMode.PIPELINE) and dp_rank == 0
                             and pc.get_local_rank(ParallelMode.TENSOR) == 0):
                extra = f"  twin {float(twin_loss):.4f}" if twin_loss is not None else ""
                print(f"step {step:5d}{extra}  loss {float(loss):.4f}", flush=True)
        if args.save_interval and step % args.save_interval == 0:
            wrapped.save_pretrained(f"{args.save_dir}/step_{step}")
    wrapped.save_pretrained(args.save_dir)
    if args.merge:
        wrapped.save_pretrained(args.save_dir + "_merged", merge_checkpoints=True)
    if history and rank == pc.get_world_size(ParallelMode.GLOBAL) - 1:
        with open(f"{args.save_dir}/losses.json", "w") as f:
            json.dump(history, f)
    if args.check_parity and args.pipeline_parallel_size == 1:
        if rank == 0:
            print(f"parity: max |parallel loss - unsharded loss| = {worst:.2e} over {args.train_step} steps", flush=True)
        if worst > args.parity_tol:
            raise SystemExit(f"loss parity violated on rank {rank}: {worst:.3e} > {args.parity_tol:.1e}")
    if rank == 0:
        print(f"saved shards to {args.save_dir}" + (f" and a merged checkpoint to {args.save_dir}_merged" if args.merge else ""), flush=True)
    pc.destroy()


if __name__ == "__main__":
    main()
