"""Pre-training objectives beyond plain MLM: BERT (MLM + next-sentence), ALBERT (MLM + sentence order), BART (text
infilling + sentence permutation) and T5 (span corruption with sentinel tokens)."""
from __future__ import annotations

import random
from typing import List

import torch

from .data_base import BaseProcessor, pad_sequences
from .data_masked_lm import DataCollatorForMaskedLM


def _split_sentences(text: str) -> List[str]:
    out, cur = [], []
    for tok in text.replace("\n", " ").split(" "):
        cur.append(tok)
        if tok.endswith((".", "!", "?")):
            out.append(" ".join(cur).strip())
            cur = []
    if cur:
        out.append(" ".join(cur).strip())
    return [s for s in out if s]


class ProcessorForBertPretraining(BaseProcessor):
    """Pairs of consecutive sentence segments; ``next_sentence_label`` 1 when the second segment was swapped in from
    another document (NSP) — ``sentence_order=True`` instead swaps the two segments (ALBERT's SOP)."""

    def __init__(self, tokenizer, max_length: int = 512, sentence_order: bool = False, seed: int = 0):
        super().__init__(tokenizer, max_length)
        self.sentence_order = sentence_order
        self.rng = random.Random(seed)

    def __call__(self, examples):
        docs = [[self._encode(s) for s in _split_sentences(t)] for t in examples["text"]]
        docs = [d for d in docs if len(d) >= 2]
        tk = self._tokenizer
        out = {"input_ids": [], "token_type_ids": [], "next_sentence_label": []}
        budget = self._max_length - 3
        for di, doc in enumerate(docs):
            for i in range(0, len(doc) - 1, 2):
                a, b = list(doc[i]), list(doc[i + 1])
                label = 0
                if self.rng.random() < 0.5:
                    label = 1
                    if self.sentence_order:
                        a, b = b, a
                    elif len(docs) > 1:
                        other = docs[self.rng.choice([j for j in range(len(docs)) if j != di])]
                        b = list(self.rng.choice(other))
                while len(a) + len(b) > budget:
                    (a if len(a) > len(b) else b).pop()
                ids = [tk.cls_token_id] + a + [tk.sep_token_id] + b + [tk.sep_token_id]
                out["input_ids"].append(ids)
                out["token_type_ids"].append([0] * (len(a) + 2) + [1] * (len(b) + 1))
                out["next_sentence_label"].append(label)
        return out


class ProcessorForAlbertPretraining(ProcessorForBertPretraining):
    def __init__(self, tokenizer, max_length: int = 512, seed: int = 0):
        super().__init__(tokenizer, max_length, sentence_order=True, seed=seed)


class DataCollatorForBertPretraining(DataCollatorForMaskedLM):
    label_key = "next_sentence_label"

    def __call__(self, features):
        batch = super().__call__(features)
        batch["token_type_ids"] = pad_sequences([f["token_type_ids"] for f in features], 0)
        batch[self.label_key] = torch.as_tensor([f["next_sentence_label"] for f in features])
        return batch


class DataCollatorForAlbertPretraining(DataCollatorForBertPretraining):
    label_key = "sentence_order_label"


class ProcessorForT5Pretraining(BaseProcessor):
    """Fixed-length chunks; the collator corrupts spans."""

    def __call__(self, examples):
        out = {"input_ids": []}
        for text in examples["text"]:
            self._buffer.extend(self._encode(text))
            while len(self._buffer) >= self._chunk_size:
                out["input_ids"].append(self._buffer[: self._chunk_size])
                self._buffer = self._buffer[self._chunk_size :]
        return out


class DataCollatorForT5Pretraining:
    """Span corruption: ~``noise_density`` of the tokens, in spans of mean length ``mean_span``, are replaced by sentinel
    ids counting down from ``vocab_size - 1``; the target lists each sentinel followed by the removed span."""

    def __init__(self, processor, noise_density: float = 0.15, mean_span: float = 3.0, label_pad_token_id: int = -100, seed: int = 0):
        self.tokenizer = processor._tokenizer
        self.noise_density, self.mean_span = noise_density, mean_span
        self.label_pad_token_id = label_pad_token_id
        self.rng = random.Random(seed)

    def _corrupt(self, ids: List[int]):
        vocab = getattr(self.tokenizer, "vocab_size", None) or len(self.tokenizer)
        n = len(ids)
        n_noise = max(1, int(round(n * self.noise_density)))
        n_spans = max(1, int(round(n_noise / self.mean_span)))
        starts = sorted(self.rng.sample(range(n), min(n_spans, n)))
        noise = [False] * n
        per = max(1, n_noise // len(starts))
        for s in starts:
            for j in range(s, min(n, s + per)):
                noise[j] = True
        inp, tgt, sentinel, prev = [], [], vocab - 1, False
        for tok, z in zip(ids, noise):
            if z:
                if not prev:
                    inp.append(sentinel)
                    tgt.append(sentinel)
                    sentinel -= 1
                tgt.append(tok)
            else:
                inp.append(tok)
            prev = z
        eos = getattr(self.tokenizer, "eos_token_id", None)
        if eos is not None:
            inp.append(eos)
            tgt.append(eos)
        return inp, tgt

    def __call__(self, features):
        pad = getattr(self.tokenizer, "pad_token_id", 0) or 0
        pairs = [self._corrupt(f["input_ids"]) for f in features]
        ids = pad_sequences([p[0] for p in pairs], pad)
        labels = pad_sequences([p[1] for p in pairs], self.label_pad_token_id)
        return {"input_ids": ids, "attention_mask": (ids != pad).long(), "labels": labels}


class ProcessorForBartPretraining(ProcessorForT5Pretraining):
    pass


class DataCollatorForBartPretraining:
    """Text infilling (spans with Poisson(3) lengths replaced by ONE mask token) and sentence permutation; the target
    is the original sequence."""

    def __init__(self, processor, mlm_probability: float = 0.3, poisson_lambda: float = 3.0, permute_sentences: bool = True,
                 label_pad_token_id: int = -100, seed: int = 0):
        self.tokenizer = processor._tokenizer
        self.p, self.lam, self.permute = mlm_probability, poisson_lambda, permute_sentences
        self.label_pad_token_id = label_pad_token_id
        self.rng = random.Random(seed)
        self.gen = torch.Generator().manual_seed(seed)

    def _infill(self, ids: List[int]) -> List[int]:
        mask_id = self.tokenizer.mask_token_id
        n, out, i = len(ids), [], 0
        to_mask = int(round(n * self.p))
        while i < n:
            if to_mask > 0 and self.rng.random() < self.p / max(self.lam, 1.0):
                span = int(torch.poisson(torch.tensor([self.lam]), generator=self.gen).item())
                span = min(span, to_mask, n - i)
                out.append(mask_id)
                i += span
                to_mask -= span
                if span == 0:
                    out.append(ids[i])
                    i += 1
            else:
                out.append(ids[i])
                i += 1
        return out

    def _permute(self, ids: List[int]) -> List[int]:
        eos = getattr(self.tokenizer, "eos_token_id", None)
        if eos is None or eos not in ids:
            return ids
        sents, cur = [], []
        for t in ids:
            cur.append(t)
            if t == eos:
                sents.append(cur)
                cur = []
        if cur:
            sents.append(cur)
        self.rng.shuffle(sents)
        return [t for s in sents for t in s]

    def __call__(self, features):
        pad = getattr(self.tokenizer, "pad_token_id", 0) or 0
        originals = [f["input_ids"] for f in features]
        noisy = [self._infill(self._permute(list(o)) if self.permute else list(o)) for o in originals]
        ids = pad_sequences(noisy, pad)
        labels = pad_sequences(originals, self.label_pad_token_id)
        return {"input_ids": ids, "attention_mask": (ids != pad).long(), "labels": labels}
