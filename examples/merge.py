"""Merge the per-rank checkpoint shards written by ``train.py`` into one ``pytorch_model.bin``.

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 examples/merge.py \
        --model gpt-neox-tiny --tensor_parallel_size 2 --save_dir example_ckpt --merge_dir example_ckpt_merged

Launch it with the same parallel sizes as the training run (every rank loads its own shard); rank 0 writes the merged file
and its config, which ``inference.py`` (or any single-process ``from_pretrained``) reads.
"""
from __future__ import annotations

from common import build_context, build_model, dtype_of, get_args


def main(argv=None):
    ap = get_args(__doc__, training=False)
    ap.add_argument("--merge_dir", required=True)
    args = ap.parse_args(argv)
    import oslo_b200
    from oslo_b200.parallel import PipelineParallel, TensorParallel

    pc = build_context(args)
    model = build_model(args).to(dtype_of(args))
    wrapped = model
    if args.tensor_parallel_size > 1:
        wrapped = TensorParallel(wrapped, pc)
    if args.pipeline_parallel_size > 1:
        wrapped = PipelineParallel(wrapped, pc)
    oslo_b200.ready(wrapped, pc)
    wrapped.from_parallelized(args.save_dir)
    wrapped.save_pretrained(args.merge_dir, merge_checkpoints=True)
    if pc.get_global_rank() == 0:
        print(f"merged {args.save_dir} into {args.merge_dir}", flush=True)
    pc.destroy()


if __name__ == "__main__":
    main()
