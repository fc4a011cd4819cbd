"""Run a trained preset model: next-token generation (causal-lm, seq2seq) or classification.

    python examples/inference.py --model gpt-neox-tiny --load example_ckpt_merged --cpu            # merged, one process
    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 examples/inference.py \
        --model gpt-neox-tiny --tensor_parallel_size 2 --load example_ckpt --sharded                  # per-rank shards

Prints the prompt and the continuation (token ids) on rank 0.
"""
from __future__ import annotations

import os

from common import batches, build_context, build_model, dtype_of, get_args

import torch


def main(argv=None):
    ap = get_args(__doc__, training=False)
    ap.add_argument("--load", required=True, help="directory written by train.py / merge.py")
    ap.add_argument("--sharded", action="store_true", help="--load holds per-rank shards (launch with the training layout)")
    ap.add_argument("--max_new_tokens", type=int, default=8)
    args = ap.parse_args(argv)
    import oslo_b200
    from oslo_b200 import ParallelMode
    from oslo_b200.parallel import TensorParallel

    distributed = args.sharded or args.tensor_parallel_size > 1 or "RANK" in os.environ
    pc = build_context(args) if distributed else None
    device = pc.device if pc is not None else torch.device("cpu" if args.cpu or not torch.cuda.is_available() else "cuda")
    model = build_model(args).to(dtype_of(args))
    wrapped = model
    if not args.sharded:
        state = torch.load(os.path.join(args.load, "pytorch_model.bin"), map_location="cpu")
        model.load_state_dict(state, strict=False)
    if pc is not None and args.tensor_parallel_size > 1:
        wrapped = TensorParallel(model, pc)
    if pc is not None:
        oslo_b200.ready(wrapped, pc)
    else:
        model.to(device)
    if args.sharded:
        wrapped.from_parallelized(args.load)
    model.eval()
    args.batch_size = 2
    batch = next(batches(args, model.config.vocab_size, 0, device, 1))
    ids = batch["input_ids"][:, : max(4, args.sequence_length // 2)]
    rank0 = pc is None or pc.get_global_rank() == 0
    with torch.no_grad():
        if args.task == "sequence-classification":
            logits = wrapped(input_ids=ids).logits
            if rank0:
                print("input", ids.tolist(), "\nclass", logits.argmax(-1).tolist(), flush=True)
        elif args.task == "seq2seq":
            out = model.generate(ids, max_new_tokens=args.max_new_tokens)
            if rank0:
                print("input", ids.tolist(), "\noutput", out.tolist(), flush=True)
        else:
            out = ids
            for _ in range(args.max_new_tokens):
                logits = wrapped(input_ids=out).logits
                if pc is not None and args.tensor_parallel_size > 1 and logits.shape[-1] != model.config.vocab_size:
                    from oslo_b200.distributed import comm

                    logits = comm.all_gather(logits, dim=-1, parallel_context=pc, parallel_mode=ParallelMode.TENSOR_1D)
                nxt = logits[:, -1, : model.config.vocab_size].argmax(-1, keepdim=True)
                out = torch.cat([out, nxt], dim=1)
            if rank0:
                print("prompt", ids.tolist(), "\ncontinuation", out[:, ids.shape[1]:].tolist(), flush=True)
    if pc is not None:
        pc.destroy()


if __name__ == "__main__":
    main()
