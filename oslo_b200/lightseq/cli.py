"""Command-line entry points for the LightSeq-interface models: train, validate, generate, export, serve.

    python -m oslo_b200.lightseq.cli train    --arch transformer-base --data pairs.tsv --save ckpt.pt --epochs 3
    python -m oslo_b200.lightseq.cli validate --load ckpt.pt --data pairs.tsv
    python -m oslo_b200.lightseq.cli generate --load ckpt.pt --input src.txt --beam 4
    python -m oslo_b200.lightseq.cli export   --load ckpt.pt --out model.lsw --int8
    python -m oslo_b200.lightseq.cli serve    --load ckpt.pt --port 8000           (decoder-only checkpoints)

Counterpart of the reference's ``lightseq-train / -validate / -generate / -infer`` commands
(oslo/lightseq2/training/cli/*.py), which are fairseq / DeepSpeed launchers; neither package is assumed here.  Data files
hold one example per line as whitespace-separated token ids; translation pairs are ``source<TAB>target``.
"""
from __future__ import annotations

import argparse
import sys
from typing import List, Tuple

import torch

from .models import LSGpt, LSTransformer, get_config


def read_pairs(path: str) -> List[Tuple[List[int], List[int]]]:
    out = []
    with open(path) as f:
        for line in f:
            line = line.rstrip("\n")
            if not line:
                continue
            src, _, trg = line.partition("\t")
            out.append(([int(t) for t in src.split()], [int(t) for t in trg.split()]))
    return out


def batches(pairs, batch_size: int, pad: int, bos: int, eos: int, device):
    for i in range(0, len(pairs), batch_size):
        chunk = pairs[i : i + batch_size]
        s_len = max(len(s) for s, _ in chunk)
        t_len = max(len(t) for _, t in chunk) + 1
        src = torch.full((len(chunk), s_len), pad, dtype=torch.long)
        trg_in = torch.full((len(chunk), t_len), pad, dtype=torch.long)
        labels = torch.full((len(chunk), t_len), pad, dtype=torch.long)
        for r, (s, t) in enumerate(chunk):
            src[r, : len(s)] = torch.tensor(s)
            trg_in[r, : len(t) + 1] = torch.tensor([bos] + t)
            labels[r, : len(t) + 1] = torch.tensor(t + [eos])
        yield src.to(device), trg_in.to(device), labels.to(device)


def _save(model, path):
    torch.save({"config": vars(model.config), "kind": type(model).__name__, "state": model.state_dict()}, path)


def _load(path, device):
    blob = torch.load(path, map_location="cpu")
    cfg = get_config(**blob["config"])
    model = {"LSTransformer": LSTransformer, "LSGpt": LSGpt}[blob["kind"]](cfg)
    model.load_state_dict(blob["state"])
    return model.to(device)


def cmd_train(a) -> int:
    device = torch.device(a.device)
    pairs = read_pairs(a.data)
    vocab = a.vocab_size or (max(max(s + t) for s, t in pairs) + 1)
    cfg = get_config(model=a.arch, vocab_size=vocab, padding_idx=a.pad, bos_id=a.bos, eos_id=a.eos, max_seq_len=a.max_len,
                     **({"hidden_size": a.hidden, "intermediate_size": 4 * a.hidden, "nhead": a.heads} if a.hidden else {}),
                     **({"num_encoder_layer": a.layers, "num_decoder_layer": a.layers} if a.layers else {}))
    torch.manual_seed(a.seed)
    model = LSTransformer(cfg).to(device)
    from oslo_b200.optim import FusedAdam

    opt = FusedAdam(model.parameters(), lr=a.lr) if device.type == "cuda" else torch.optim.Adam(model.parameters(), lr=a.lr)
    for epoch in range(a.epochs):
        total, n = 0.0, 0
        for src, trg_in, labels in batches(pairs, a.batch_size, a.pad, a.bos, a.eos, device):
            loss, _ = model(src, trg_in, labels)
            opt.zero_grad()
            loss.backward()
            opt.step()
            total, n = total + loss.item(), n + 1
        print(f"epoch {epoch + 1}: loss {total / max(1, n):.4f}", flush=True)
    _save(model, a.save)
    return 0


def cmd_validate(a) -> int:
    device = torch.device(a.device)
    model = _load(a.load, device).eval()
    cfg = model.config
    tot, ntok = 0.0, 0
    with torch.no_grad():
        for src, trg_in, labels in batches(read_pairs(a.data), a.batch_size, cfg.padding_idx, cfg.bos_id, cfg.eos_id, device):
            logits = model(src, trg_in)
            _, nll = model.criterion(logits, labels)
            tot += nll.item()
            ntok += int((labels != cfg.padding_idx).sum())
    print(f"nll per token {tot / max(1, ntok):.4f}  perplexity {torch.tensor(tot / max(1, ntok)).exp().item():.3f}")
    return 0


def cmd_generate(a) -> int:
    device = torch.device(a.device)
    model = _load(a.load, device).eval()
    cfg = model.config
    with open(a.input) as f:
        rows = [[int(t) for t in line.split()] for line in f if line.strip()]
    for i in range(0, len(rows), a.batch_size):
        chunk = rows[i : i + a.batch_size]
        width = max(len(r) for r in chunk)
        src = torch.full((len(chunk), width), cfg.padding_idx, dtype=torch.long)
        for r, ids in enumerate(chunk):
            src[r, : len(ids)] = torch.tensor(ids)
        if isinstance(model, LSTransformer):
            out = model.infer(src.to(device), max_new_tokens=a.max_new_tokens, beam_size=a.beam)
        else:
            out = model.infer(src.to(device), max_new_tokens=a.max_new_tokens, num_beams=a.beam)
        for row in out.tolist():
            toks = [t for t in row if t not in (cfg.padding_idx, cfg.bos_id)]
            if cfg.eos_id in toks:
                toks = toks[: toks.index(cfg.eos_id)]
            print(" ".join(map(str, toks)))
    return 0


def cmd_export(a) -> int:
    from .export import export_model

    model = _load(a.load, torch.device("cpu"))
    header = export_model(model, a.out, quantize=a.int8)
    print(f"wrote {a.out}: {len(header['tensors'])} tensors, quantized={header['quantized']}")
    return 0


def cmd_serve(a) -> int:
    from .serving import serve

    serve(_load(a.load, torch.device(a.device)).eval(), host=a.host, port=a.port, max_batch=a.max_batch)
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="oslo_b200.lightseq.cli")
    sub = ap.add_subparsers(dest="cmd", required=True)
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    t = sub.add_parser("train")
    t.add_argument("--arch", default="transformer-base")
    t.add_argument("--data", required=True)
    t.add_argument("--save", required=True)
    for name, typ, default in (("epochs", int, 1), ("batch-size", int, 32), ("lr", float, 1e-3), ("seed", int, 0), ("pad", int, 0),
                               ("bos", int, 1), ("eos", int, 2), ("max-len", int, 256), ("vocab-size", int, 0), ("hidden", int, 0),
                               ("heads", int, 8), ("layers", int, 0)):
        t.add_argument(f"--{name}", type=typ, default=default)
    t.set_defaults(fn=cmd_train)
    v = sub.add_parser("validate")
    v.add_argument("--load", required=True)
    v.add_argument("--data", required=True)
    v.add_argument("--batch-size", type=int, default=32)
    v.set_defaults(fn=cmd_validate)
    g = sub.add_parser("generate")
    g.add_argument("--load", required=True)
    g.add_argument("--input", required=True)
    g.add_argument("--beam", type=int, default=1)
    g.add_argument("--max-new-tokens", type=int, default=64)
    g.add_argument("--batch-size", type=int, default=32)
    g.set_defaults(fn=cmd_generate)
    e = sub.add_parser("export")
    e.add_argument("--load", required=True)
    e.add_argument("--out", required=True)
    e.add_argument("--int8", action="store_true")
    e.set_defaults(fn=cmd_export)
    s = sub.add_parser("serve")
    s.add_argument("--load", required=True)
    s.add_argument("--host", default="127.0.0.1")
    s.add_argument("--port", type=int, default=8000)
    s.add_argument("--max-batch", type=int, default=8)
    s.set_defaults(fn=cmd_serve)
    for p in (t, v, g, e, s):  # (export always works on the host copy; it takes the flag so scripts can pass one set of options)
        p.add_argument("--device", default=dev)
    a = ap.parse_args(argv)
    return a.fn(a)


if __name__ == "__main__":
    sys.exit(main())
