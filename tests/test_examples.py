"""The example scripts end to end on CPU ranks: train with tensor x data parallelism, merge the shards, run inference from
the merged file in one process and from the shards in two, and get the same continuation."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EX = os.path.join(ROOT, "examples")


def _run(script, *args, nproc=1, port=None):
    from dist_utils import free_port

    port = free_port()  # (the argument is kept for readability of the call sites; a free port is always taken)
    env = dict(os.environ, OMP_NUM_THREADS="1", PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    if nproc == 1:
        cmd = [sys.executable, os.path.join(EX, script), *args]
        for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "MASTER_ADDR", "MASTER_PORT"):
            env.pop(k, None)
    else:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
               "--master-port", str(port), os.path.join(EX, script), *args]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=EX)
    assert res.returncode == 0, res.stdout[-2000:] + "\n" + res.stderr[-3000:]
    return res.stdout


def test_train_merge_and_infer_examples(tmp_path):
    ckpt = str(tmp_path / "ckpt")
    common = ["--model", "gpt-neox-tiny", "--cpu", "--sequence_length", "16", "--save_dir", ckpt]
    out = _run("train.py", *common, "--tensor_parallel_size", "2", "--data_parallel_size", "2", "--train_step", "30", "--lr", "3e-3",
               "--merge", "--check_parity", nproc=4, port=29713)
    parity = [line for line in out.splitlines() if line.startswith("parity:")]
    assert parity and float(parity[0].split("=")[1].split()[0]) < 2e-3, parity  # sharded run tracks the unsharded twin
    losses = [float(line.split()[-1]) for line in out.splitlines() if line.startswith("step")]
    assert len(losses) >= 3 and losses[-1] < losses[0] - 0.3, losses
    assert os.path.exists(os.path.join(ckpt, "pytorch_model_tp_0_pp_0_ep_0.bin")) and os.path.exists(os.path.join(ckpt, "pytorch_model_tp_1_pp_0_ep_0.bin"))
    assert os.path.exists(os.path.join(ckpt + "_merged", "pytorch_model.bin"))
    with open(os.path.join(ckpt, "losses.json")) as f:
        assert len(json.load(f)) == len(losses)
    # merging afterwards from the shards gives the file that --merge wrote
    import torch

    merged2 = str(tmp_path / "merged2")
    _run("merge.py", *common, "--tensor_parallel_size", "2", "--merge_dir", merged2, nproc=2, port=29715)
    a = torch.load(os.path.join(ckpt + "_merged", "pytorch_model.bin"))
    b = torch.load(os.path.join(merged2, "pytorch_model.bin"))
    assert a.keys() == b.keys() and all(torch.equal(a[k], b[k]) for k in a)
    single = _run("inference.py", *common, "--load", merged2)
    sharded = _run("inference.py", *common, "--tensor_parallel_size", "2", "--load", ckpt, "--sharded", nproc=2, port=29717)
    pick = lambda text: [line for line in text.splitlines() if line.startswith("continuation")]  # noqa: E731
    assert pick(single) and pick(single) == pick(sharded)


def test_pipeline_and_zero_example_runs(tmp_path):
    out = _run("train.py", "--model", "gpt2-tiny", "--cpu", "--sequence_length", "16", "--save_dir", str(tmp_path / "pp"),
               "--pipeline_parallel_size", "2", "--train_step", "6", "--micro_batches", "2", nproc=2, port=29719)
    assert "saved shards" in out
    out = _run("train.py", "--model", "bert-tiny", "--task", "sequence-classification", "--cpu", "--sequence_length", "16",
               "--save_dir", str(tmp_path / "z"), "--data_parallel_size", "2", "--zero_stage", "2", "--train_step", "6", nproc=2, port=29721)
    assert "saved shards" in out
    out = _run("train.py", "--model", "t5-tiny", "--task", "seq2seq", "--cpu", "--sequence_length", "16", "--save_dir", str(tmp_path / "t5"),
               "--train_step", "4", "--merge")
    assert "saved shards" in out
    out = _run("inference.py", "--model", "t5-tiny", "--task", "seq2seq", "--cpu", "--sequence_length", "16", "--load", str(tmp_path / "t5_merged"))
    assert "output [[" in out
    _run("train.py", "--model", "bert-tiny", "--task", "sequence-classification", "--cpu", "--sequence_length", "16", "--save_dir",
         str(tmp_path / "cls"), "--train_step", "3", "--merge")
    out = _run("inference.py", "--model", "bert-tiny", "--task", "sequence-classification", "--cpu", "--sequence_length", "16", "--load",
               str(tmp_path / "cls_merged"))
    assert "class [" in out
