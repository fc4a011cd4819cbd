"""Corpus loading, tokenizer training and corpus serialisation for the task processors.

Parity: oslo/transformers/tasks/data_utils.py (``CorpusType``, ``batch_iterator``, ``load_corpora``, ``train_tokenizer``,
``serialize_corpora``) and oslo/transformers/tasks/loading/sent_text.py (one sentence per line, a blank line between
documents).  The reference leans on the ``datasets`` library; here a corpus is a :class:`Corpus`, a small column store with
the handful of operations the pipeline needs (``map`` / ``select`` / ``rename_column`` / ``save_to_disk``), so the data
path has no dependency beyond the standard library and, for tokenizer training, the ``tokenizers`` package.  Tokenizers are
trained from scratch (BPE, WordPiece or Unigram by model family): nothing is fetched from a hub.
"""
from __future__ import annotations

import enum
import json
import os
import random
from pathlib import Path
from typing import Any, Callable, Dict, Iterable, Iterator, List, Optional, Sequence, Union


class CorpusType(str, enum.Enum):
    DOCU_TEXT = "docu_text"  # *.txt, one document per line
    DOCU_JSON = "docu_json"  # *.json, one JSON object per line (or one JSON array per file)
    SENT_TEXT = "sent_text"  # *.txt, one sentence per line, documents separated by blank lines
    SENT_JSON = "sent_json"  # *.json, objects with a list of sentences under "sentences" (or "text")
    DATASET = "dataset"  # a directory written by Corpus.save_to_disk


class Corpus:
    """Column store: ``{column: [values]}`` with equal-length columns.  Indexing with an int gives a row dict, with a slice
    or a column name gives lists, like the ``datasets`` objects the processors were written against."""

    def __init__(self, columns: Dict[str, List[Any]]):
        lengths = {len(v) for v in columns.values()}
        if len(lengths) > 1:
            raise ValueError(f"columns differ in length: { {k: len(v) for k, v in columns.items()} }")
        self._cols = {k: list(v) for k, v in columns.items()}

    # ------------------------------------------------------------------ access
    @property
    def column_names(self) -> List[str]:
        return list(self._cols)

    def __len__(self) -> int:
        return len(next(iter(self._cols.values()))) if self._cols else 0

    def __getitem__(self, key):
        if isinstance(key, str):
            return self._cols[key]
        if isinstance(key, slice):
            return {k: v[key] for k, v in self._cols.items()}
        if key < 0:
            key += len(self)
        return {k: v[key] for k, v in self._cols.items()}

    def __iter__(self) -> Iterator[Dict[str, Any]]:
        return (self[i] for i in range(len(self)))

    # -------------------------------------------------------------- transforms
    def select(self, indices: Iterable[int]) -> "Corpus":
        idx = list(indices)
        return Corpus({k: [v[i] for i in idx] for k, v in self._cols.items()})

    def rename_column(self, old: str, new: str) -> "Corpus":
        if new in self._cols:
            raise ValueError(f"column {new!r} exists")
        return Corpus({(new if k == old else k): v for k, v in self._cols.items()})

    def map(self, fn: Callable[[Dict[str, List[Any]]], Dict[str, List[Any]]], batched: bool = True, batch_size: int = 1000,
            remove_columns: Optional[Sequence[str]] = None, **_unused) -> "Corpus":
        """Apply ``fn`` to batches (dict of lists; may return a different number of rows) or to single rows.  Columns in
        ``remove_columns`` are dropped; others are kept only when the row count is unchanged."""
        out: Dict[str, List[Any]] = {}
        drop = set(remove_columns or ())
        kept = [k for k in self._cols if k not in drop]
        n = len(self)
        step = batch_size if batched else 1
        for s in range(0, n, step):
            batch = self[s : s + step]
            res = fn(batch) if batched else {k: [v] for k, v in fn({k: v[0] for k, v in batch.items()}).items()}
            rows = len(next(iter(res.values()))) if res else 0
            same = rows == len(next(iter(batch.values())))
            for k, v in res.items():
                out.setdefault(k, []).extend(v)
            for k in kept:
                if k in res:
                    continue
                if not same:
                    raise ValueError(f"map changed the row count; list column {k!r} in remove_columns")
                out.setdefault(k, []).extend(batch[k])
        return Corpus(out)

    def train_test_split(self, test_size: float = 0.1, seed: int = 0) -> Dict[str, "Corpus"]:
        idx = list(range(len(self)))
        random.Random(seed).shuffle(idx)
        cut = int(round(len(idx) * (1.0 - test_size)))
        return {"train": self.select(sorted(idx[:cut])), "test": self.select(sorted(idx[cut:]))}

    # ------------------------------------------------------------------- disk
    def save_to_disk(self, path: str) -> None:
        os.makedirs(path, exist_ok=True)
        with open(os.path.join(path, "data.jsonl"), "w", encoding="utf-8") as f:
            for row in self:
                f.write(json.dumps(row, ensure_ascii=False) + "\n")
        with open(os.path.join(path, "corpus_info.json"), "w") as f:
            json.dump({"columns": self.column_names, "num_rows": len(self)}, f)

    @classmethod
    def load_from_disk(cls, path: str) -> "Corpus":
        with open(os.path.join(path, "corpus_info.json")) as f:
            info = json.load(f)
        cols: Dict[str, List[Any]] = {k: [] for k in info["columns"]}
        with open(os.path.join(path, "data.jsonl"), encoding="utf-8") as f:
            for line in f:
                row = json.loads(line)
                for k in cols:
                    cols[k].append(row.get(k))
        return cls(cols)


def batch_iterator(corpus, key: str = "text", batch_size: int = 1000) -> Iterator[List[Any]]:
    """Lists of ``batch_size`` values of column ``key`` (what tokenizer trainers consume)."""
    return (corpus[i : i + batch_size][key] for i in range(0, len(corpus), batch_size))


def _json_records(path: Path) -> Iterator[dict]:
    text = path.read_text(encoding="utf-8")
    stripped = text.lstrip()
    if stripped.startswith("["):
        yield from json.loads(text)
        return
    for line in text.splitlines():
        if line.strip():
            yield json.loads(line)


def read_sent_text(path: Union[str, Path], encoding: str = "utf-8") -> List[str]:
    """Documents of a sentence-per-line file: consecutive non-empty lines joined by one space; blank lines separate."""
    docs, cur = [], []
    with open(path, encoding=encoding) as f:
        for line in f:
            line = line.rstrip("\n").rstrip()
            if line:
                cur.append(line)
            elif cur:
                docs.append(" ".join(cur))
                cur = []
    if cur:
        docs.append(" ".join(cur))
    return docs


def load_corpora(dir_path: str, corpus_type: Union[str, CorpusType] = "docu_json") -> Corpus:
    """All ``*.txt`` / ``*.json`` files under ``dir_path`` (recursively, in sorted order) as one :class:`Corpus`."""
    kind = CorpusType(corpus_type)
    root = Path(dir_path).absolute()
    if kind == CorpusType.DATASET:
        return Corpus.load_from_disk(str(root / "train") if (root / "train").is_dir() else str(root))
    ext = "*.json" if kind.value.endswith("json") else "*.txt"
    files = sorted(root.rglob(ext))
    if not files:
        raise FileNotFoundError(f"no {ext} file under {root}")
    cols: Dict[str, List[Any]] = {}

    def add(row: dict):
        for k in set(cols) | set(row):
            cols.setdefault(k, [None] * n_rows[0]).append(row.get(k))
        n_rows[0] += 1

    n_rows = [0]
    for path in files:
        if kind == CorpusType.DOCU_TEXT:
            with open(path, encoding="utf-8") as f:
                for line in f:
                    if line.strip():
                        add({"text": line.rstrip("\n")})
        elif kind == CorpusType.SENT_TEXT:
            for doc in read_sent_text(path):
                add({"text": doc})
        elif kind == CorpusType.DOCU_JSON:
            for rec in _json_records(path):
                add(rec)
        else:  # SENT_JSON
            for rec in _json_records(path):
                sents = rec.get("sentences", rec.get("text"))
                rec = dict(rec)
                rec.pop("sentences", None)
                rec["text"] = " ".join(sents) if isinstance(sents, (list, tuple)) else sents
                add(rec)
    return Corpus(cols)


#: tokenizer algorithm per model family: (model, pre-tokenizer, special tokens in id order)
_FAMILIES = {
    "gpt2": ("bpe", ["<|endoftext|>"]),
    "gpt_neox": ("bpe", ["<|endoftext|>", "<|padding|>"]),
    "roberta": ("bpe", ["<s>", "<pad>", "</s>", "<unk>", "<mask>"]),
    "bart": ("bpe", ["<s>", "<pad>", "</s>", "<unk>", "<mask>"]),
    "mbart": ("unigram", ["<s>", "<pad>", "</s>", "<unk>", "<mask>"]),
    "bert": ("wordpiece", ["[PAD]", "[UNK]", "[CLS]", "[SEP]", "[MASK]"]),
    "distilbert": ("wordpiece", ["[PAD]", "[UNK]", "[CLS]", "[SEP]", "[MASK]"]),
    "electra": ("wordpiece", ["[PAD]", "[UNK]", "[CLS]", "[SEP]", "[MASK]"]),
    "albert": ("unigram", ["<pad>", "<unk>", "[CLS]", "[SEP]", "[MASK]"]),
    "t5": ("unigram", ["<pad>", "</s>", "<unk>"]),
    "mt5": ("unigram", ["<pad>", "</s>", "<unk>"]),
}


def _family(model_name: str) -> str:
    name = model_name.lower().replace("-", "_")
    for fam in sorted(_FAMILIES, key=len, reverse=True):
        if fam in name:
            return fam
    raise ValueError(f"cannot tell the tokenizer family of {model_name!r}; known: {sorted(_FAMILIES)}")


def train_tokenizer(model_name: str, vocab_size: int, min_frequency: int = 2, corpora_dir: Optional[str] = None,
                    corpus_type: Union[str, CorpusType] = "docu_text", sampling_ratio: float = 1.0, save_dir: Optional[str] = None,
                    additional_special_tokens: Optional[List[str]] = None, batch_size: int = 1000, corpora: Optional[Corpus] = None,
                    seed: int = 0):
    """Train a tokenizer of ``model_name``'s family on a corpus and save it with ``save_pretrained``.

    A directory that already holds a tokenizer (``model_name`` is a path) is retrained with its own algorithm through
    ``train_new_from_iterator``; otherwise the algorithm and special tokens follow the family named in ``model_name``.
    Returns the ``transformers`` fast tokenizer."""
    if sampling_ratio <= 0:
        raise ValueError("sampling_ratio must be greater than 0")
    if corpora is None:
        if corpora_dir is None:
            raise ValueError("give corpora_dir or corpora")
        corpora = load_corpora(corpora_dir, corpus_type)
    if sampling_ratio < 1.0:
        k = max(1, int(len(corpora) * sampling_ratio))
        corpora = corpora.select(sorted(random.Random(seed).sample(range(len(corpora)), k)))
    extra = list(additional_special_tokens or [])
    if len(extra) != len(set(extra)):
        raise ValueError("additional special tokens must be unique")
    if save_dir is None:
        save_dir = f"tokenizers/{Path(model_name).name}_{Path(corpora_dir).name if corpora_dir else 'corpus'}"

    if os.path.isdir(model_name):
        from transformers import AutoTokenizer

        base = AutoTokenizer.from_pretrained(model_name)
        if set(base.all_special_tokens) & set(extra):
            raise ValueError("additional special tokens repeat the tokenizer's own")
        kwargs = {"new_special_tokens": extra} if extra else {}
        tok = base.train_new_from_iterator(batch_iterator(corpora, batch_size=batch_size), vocab_size=vocab_size,
                                           min_frequency=min_frequency, **kwargs)
        tok.save_pretrained(save_dir)
        return tok

    from tokenizers import Tokenizer, decoders, models, normalizers, pre_tokenizers, processors, trainers
    from transformers import PreTrainedTokenizerFast

    fam = _family(model_name)
    algo, specials = _FAMILIES[fam]
    if set(specials) & set(extra):
        raise ValueError("additional special tokens repeat the tokenizer's own")
    specials = specials + extra
    if algo == "bpe":
        tk = Tokenizer(models.BPE(unk_token="<unk>" if "<unk>" in specials else None))
        tk.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False)
        tk.decoder = decoders.ByteLevel()
        trainer = trainers.BpeTrainer(vocab_size=vocab_size, min_frequency=min_frequency, special_tokens=specials,
                                      initial_alphabet=pre_tokenizers.ByteLevel.alphabet())
    elif algo == "wordpiece":
        tk = Tokenizer(models.WordPiece(unk_token="[UNK]"))
        tk.normalizer = normalizers.BertNormalizer(lowercase=True)
        tk.pre_tokenizer = pre_tokenizers.BertPreTokenizer()
        tk.decoder = decoders.WordPiece()
        trainer = trainers.WordPieceTrainer(vocab_size=vocab_size, min_frequency=min_frequency, special_tokens=specials)
    else:
        tk = Tokenizer(models.Unigram())
        tk.normalizer = normalizers.NFKC()
        tk.pre_tokenizer = pre_tokenizers.Metaspace()
        tk.decoder = decoders.Metaspace()
        trainer = trainers.UnigramTrainer(vocab_size=vocab_size, special_tokens=specials, unk_token="<unk>")
    tk.train_from_iterator(batch_iterator(corpora, batch_size=batch_size), trainer=trainer)

    names: Dict[str, Any] = {}
    if fam in ("gpt2", "gpt_neox"):
        names = dict(bos_token="<|endoftext|>", eos_token="<|endoftext|>", unk_token="<|endoftext|>")
        if fam == "gpt_neox":
            names["pad_token"] = "<|padding|>"
    elif algo == "wordpiece" or fam == "albert":
        names = dict(pad_token=specials[0], unk_token=specials[1], cls_token="[CLS]", sep_token="[SEP]", mask_token="[MASK]")
        cls_id, sep_id = tk.token_to_id("[CLS]"), tk.token_to_id("[SEP]")
        tk.post_processor = processors.TemplateProcessing(single="[CLS] $A [SEP]", pair="[CLS] $A [SEP] $B:1 [SEP]:1",
                                                          special_tokens=[("[CLS]", cls_id), ("[SEP]", sep_id)])
    elif fam in ("t5", "mt5"):
        names = dict(pad_token="<pad>", eos_token="</s>", unk_token="<unk>")
        tk.post_processor = processors.TemplateProcessing(single="$A </s>", pair="$A </s> $B </s>",
                                                          special_tokens=[("</s>", tk.token_to_id("</s>"))])
    else:  # roberta, bart, mbart
        names = dict(bos_token="<s>", pad_token="<pad>", eos_token="</s>", unk_token="<unk>", mask_token="<mask>",
                     cls_token="<s>", sep_token="</s>")
        tk.post_processor = processors.TemplateProcessing(single="<s> $A </s>", pair="<s> $A </s> </s> $B </s>",
                                                          special_tokens=[("<s>", tk.token_to_id("<s>")), ("</s>", tk.token_to_id("</s>"))])
    tok = PreTrainedTokenizerFast(tokenizer_object=tk, additional_special_tokens=extra or None, **names)
    tok.save_pretrained(save_dir)
    return tok


def _processors() -> Dict[str, Any]:
    from . import (ProcessorForAlbertPretraining, ProcessorForBartPretraining, ProcessorForBertPretraining, ProcessorForCausalLM,
                   ProcessorForMaskedLM, ProcessorForSequenceClassification, ProcessorForSummarization, ProcessorForT5Pretraining,
                   ProcessorForTokenClassification)

    return {
        "causal_lm": ProcessorForCausalLM,
        "masked_lm": ProcessorForMaskedLM,
        "sequence_classification": ProcessorForSequenceClassification,
        "token_classification": ProcessorForTokenClassification,
        "summarization": ProcessorForSummarization,
        "bert_pretraining": ProcessorForBertPretraining,
        "albert_pretraining": ProcessorForAlbertPretraining,
        "roberta_pretraining": ProcessorForMaskedLM,
        "bart_pretraining": ProcessorForBartPretraining,
        "t5_pretraining": ProcessorForT5Pretraining,
    }


def serialize_corpora(model_type: str, task_type: str, tokenizer_dir, corpora_dir: Optional[str] = None,
                      corpus_type: Union[str, CorpusType] = "docu_text", max_seq_length: int = 512, save_dir: Optional[str] = None,
                      batched: bool = True, batch_size: int = 1000, corpora: Optional[Corpus] = None, **processor_kwargs) -> Corpus:
    """Tokenise a corpus with the processor of ``task_type`` and write the result (plus the tokenizer) to ``save_dir``.
    ``tokenizer_dir`` is a directory saved by :func:`train_tokenizer` / ``save_pretrained`` or a tokenizer object."""
    table = _processors()
    if task_type not in table:
        raise ValueError(f"{task_type!r} must be one of {sorted(table)}")
    if save_dir is None:
        save_dir = f"datasets/{model_type}_{task_type}"
    if corpora is None:
        if corpora_dir is None:
            raise ValueError("give corpora_dir or corpora")
        corpora = load_corpora(corpora_dir, corpus_type)
    for old in ("label", "label_ids"):
        if old in corpora.column_names and "labels" not in corpora.column_names:
            corpora = corpora.rename_column(old, "labels")
    tokenizer = tokenizer_dir
    if isinstance(tokenizer_dir, (str, os.PathLike)):
        from transformers import AutoTokenizer

        tokenizer = AutoTokenizer.from_pretrained(str(tokenizer_dir))
    processor = table[task_type](tokenizer, max_seq_length, **processor_kwargs)
    out = corpora.map(processor, batched=batched, batch_size=batch_size, remove_columns=corpora.column_names)
    out.save_to_disk(save_dir)
    processor.save_tokenizer(save_dir)
    return out


__all__ = ["CorpusType", "Corpus", "batch_iterator", "read_sent_text", "load_corpora", "train_tokenizer", "serialize_corpora"]
