"""Task processors / collators with a toy whitespace tokenizer."""
import torch


class ToyTokenizer:
    pad_token_id, cls_token_id, sep_token_id, mask_token_id, eos_token_id, bos_token_id = 0, 1, 2, 3, 4, None
    vocab_size = 200

    def __call__(self, text, add_special_tokens=False):
        return {"input_ids": [5 + (hash(w) % 150) for w in text.split()]}

    def __len__(self):
        return self.vocab_size


TEXT = {"text": ["the quick brown fox jumps. over the lazy dog again! and again and again?"] * 6}


def test_causal_lm_chunks_and_labels():
    from oslo_b200.transformers.tasks import DataCollatorForCausalLM, ProcessorForCausalLM

    proc = ProcessorForCausalLM(ToyTokenizer(), max_length=8)
    feats = proc(TEXT)["input_ids"]
    assert feats and all(len(f) == 8 for f in feats)
    batch = DataCollatorForCausalLM(proc)([{"input_ids": f} for f in feats[:3]])
    assert batch["input_ids"].shape == (3, 8) and torch.equal(batch["labels"], batch["input_ids"])


def test_masked_lm_masks_about_15_percent():
    from oslo_b200.transformers.tasks import DataCollatorForMaskedLM, ProcessorForMaskedLM

    proc = ProcessorForMaskedLM(ToyTokenizer(), max_length=16)
    feats = [{"input_ids": f} for f in proc({"text": TEXT["text"] * 20})["input_ids"]]
    batch = DataCollatorForMaskedLM(proc, seed=0)(feats)
    frac = (batch["labels"] != -100).float().mean().item()
    assert 0.05 < frac < 0.25
    assert (batch["input_ids"][:, 0] == 1).all()  # [CLS] never masked


def test_pretraining_and_classification_collators():
    from oslo_b200.transformers import tasks as T

    tk = ToyTokenizer()
    bert = T.ProcessorForBertPretraining(tk, max_length=32)
    feats = bert(TEXT)
    rows = [{k: v[i] for k, v in feats.items()} for i in range(len(feats["input_ids"]))]
    b = T.DataCollatorForBertPretraining(bert, seed=1)(rows)
    assert set(b) >= {"input_ids", "labels", "token_type_ids", "next_sentence_label"}
    t5 = T.ProcessorForT5Pretraining(tk, max_length=16)
    b5 = T.DataCollatorForT5Pretraining(t5)([{"input_ids": f} for f in t5({"text": TEXT["text"] * 4})["input_ids"]])
    assert (b5["input_ids"] >= 190).any() and (b5["labels"] >= 190).any()  # sentinels on both sides
    bart = T.ProcessorForBartPretraining(tk, max_length=16)
    bb = T.DataCollatorForBartPretraining(bart)([{"input_ids": f} for f in bart({"text": TEXT["text"] * 4})["input_ids"]])
    assert bb["labels"].shape[0] == bb["input_ids"].shape[0]
    sc = T.ProcessorForSequenceClassification(tk, 16)({"text": ["a b c", "d e"], "labels": [0, 1]})
    bs = T.DataCollatorForSequenceClassification(T.ProcessorForSequenceClassification(tk, 16))(
        [{"input_ids": i, "labels": l} for i, l in zip(sc["input_ids"], sc["labels"])])
    assert bs["labels"].tolist() == [0, 1]
    tc = T.ProcessorForTokenClassification(tk, 16)({"tokens": [["a", "b"]], "labels": [[1, 2]]})
    assert tc["labels"][0] == [1, 2]
    sm = T.ProcessorForSummarization(tk, 16, 8)({"text": ["a b c d"], "summary": ["a b"]})
    bsm = T.DataCollatorForSummarization(T.ProcessorForSummarization(tk, 16, 8))([{"input_ids": sm["input_ids"][0], "labels": sm["labels"][0]}])
    assert bsm["decoder_input_ids"].shape == bsm["labels"].shape


def test_fused_norm_swaps():
    import torch.nn as nn

    from oslo_b200.transformers.kernel_fusion_utils import fused_layer_norm

    m = nn.Sequential(nn.Linear(8, 8), nn.LayerNorm(8))
    x = torch.randn(2, 8)
    want = m(x)
    fused_layer_norm(m)
    assert m[1].__class__.__name__ == "FusedLayerNorm" and torch.allclose(m(x), want, atol=1e-6)


def _write_corpus(root):
    import json
    import os

    os.makedirs(os.path.join(root, "docs", "sub"), exist_ok=True)
    os.makedirs(os.path.join(root, "sents"), exist_ok=True)
    os.makedirs(os.path.join(root, "json"), exist_ok=True)
    lines = [f"document number {i} talks about the quick brown fox and the lazy dog {i % 7} times." for i in range(120)]
    with open(os.path.join(root, "docs", "a.txt"), "w") as f:
        f.write("\n".join(lines[:60]) + "\n")
    with open(os.path.join(root, "docs", "sub", "b.txt"), "w") as f:
        f.write("\n".join(lines[60:]) + "\n")
    with open(os.path.join(root, "sents", "s.txt"), "w") as f:
        f.write("first sentence of one.\nsecond sentence of one.\n\nonly sentence of two.\n\n\nthree a.\nthree b.\nthree c.")
    with open(os.path.join(root, "json", "j.json"), "w") as f:
        for i in range(10):
            f.write(json.dumps({"text": lines[i], "label": i % 2}) + "\n")
    return lines


def test_corpus_loading_and_column_store(tmp_path):
    from oslo_b200.transformers.tasks.data_utils import Corpus, CorpusType, batch_iterator, load_corpora

    lines = _write_corpus(str(tmp_path))
    docs = load_corpora(str(tmp_path / "docs"), "docu_text")
    assert len(docs) == 120 and docs[0]["text"] == lines[0] and docs.column_names == ["text"]
    sents = load_corpora(str(tmp_path / "sents"), CorpusType.SENT_TEXT)
    assert sents["text"] == ["first sentence of one. second sentence of one.", "only sentence of two.", "three a. three b. three c."]
    js = load_corpora(str(tmp_path / "json"), "docu_json")
    assert js.column_names == ["text", "label"] or set(js.column_names) == {"text", "label"}
    assert js.rename_column("label", "labels")["labels"] == [i % 2 for i in range(10)]
    assert [len(b) for b in batch_iterator(docs, batch_size=50)] == [50, 50, 20]
    doubled = docs.map(lambda b: {"n": [len(t) for t in b["text"]]}, batch_size=32)
    assert doubled.column_names == ["n", "text"] or set(doubled.column_names) == {"n", "text"}
    grown = docs.map(lambda b: {"piece": [w for t in b["text"] for w in t.split()[:2]]}, remove_columns=["text"])
    assert len(grown) == 240
    docs.save_to_disk(str(tmp_path / "saved"))
    again = load_corpora(str(tmp_path / "saved"), "dataset")
    assert again["text"] == docs["text"]
    split = docs.train_test_split(0.25, seed=1)
    assert len(split["train"]) == 90 and len(split["test"]) == 30
    import pytest

    with pytest.raises(FileNotFoundError):
        load_corpora(str(tmp_path / "sents"), "docu_json")
    with pytest.raises(ValueError):
        Corpus({"a": [1], "b": [1, 2]})


def test_train_tokenizer_and_serialize_corpora(tmp_path):
    from oslo_b200.transformers.tasks import DataCollatorForBertPretraining, DataCollatorForCausalLM
    from oslo_b200.transformers.tasks.data_utils import load_corpora, serialize_corpora, train_tokenizer

    _write_corpus(str(tmp_path))
    docs = str(tmp_path / "docs")
    gpt = train_tokenizer("gpt2", 400, 1, docs, "docu_text", 0.5, save_dir=str(tmp_path / "tok_gpt2"), additional_special_tokens=["<extra>"])
    assert gpt.eos_token == "<|endoftext|>" and "<extra>" in gpt.get_vocab() and len(gpt) <= 400
    text = "the quick brown fox 17"
    assert gpt.decode(gpt(text)["input_ids"]) == text  # byte-level BPE round-trips any string
    bert = train_tokenizer("bert-base", 300, 1, docs, save_dir=str(tmp_path / "tok_bert"))
    enc = bert("the lazy dog")["input_ids"]
    assert enc[0] == bert.cls_token_id and enc[-1] == bert.sep_token_id and bert.pad_token_id == 0
    t5 = train_tokenizer("t5-small", 200, 1, docs, save_dir=str(tmp_path / "tok_t5"))
    assert t5("fox")["input_ids"][-1] == t5.eos_token_id
    # retraining a saved tokenizer keeps its algorithm and special tokens
    re = train_tokenizer(str(tmp_path / "tok_bert"), 280, 1, docs, save_dir=str(tmp_path / "tok_bert2"))
    assert re.cls_token == "[CLS]" and len(re) <= 280

    out = serialize_corpora("gpt2", "causal_lm", str(tmp_path / "tok_gpt2"), docs, "docu_text", max_seq_length=32,
                            save_dir=str(tmp_path / "ds_clm"))
    assert len(out) > 10 and all(len(r["input_ids"]) == 32 for r in out)
    reloaded = load_corpora(str(tmp_path / "ds_clm"), "dataset")
    assert reloaded["input_ids"] == out["input_ids"]
    import os

    assert os.path.exists(tmp_path / "ds_clm" / "tokenizer.json")
    batch = DataCollatorForCausalLM(type("P", (), {"_tokenizer": gpt})())([out[0], out[1]])
    assert batch["input_ids"].shape == (2, 32)
    pre = serialize_corpora("bert", "bert_pretraining", bert, corpora=load_corpora(str(tmp_path / "sents"), "sent_text"),
                            max_seq_length=24, save_dir=str(tmp_path / "ds_bert"))
    assert len(pre) >= 1 and "input_ids" in pre.column_names
    import pytest

    with pytest.raises(ValueError):
        serialize_corpora("bert", "no_such_task", bert, docs)
    with pytest.raises(ValueError):
        train_tokenizer("bert", 100, 1, docs, additional_special_tokens=["[CLS]"], save_dir=str(tmp_path / "x"))


def test_default_and_padding_collators():
    from oslo_b200.transformers import DataCollatorWithPadding, default_data_collator

    feats = [{"input_ids": [1, 2, 3], "label": 1, "name": "a", "skip": None}, {"input_ids": [4, 5, 6], "label": 0, "name": "b", "skip": None}]
    b = default_data_collator(feats)
    assert set(b) == {"input_ids", "labels"} and b["labels"].dtype == torch.long and b["input_ids"].shape == (2, 3)
    reg = default_data_collator([{"x": torch.ones(2), "label": 0.5}, {"x": torch.zeros(2), "label": 1.5}], return_tensors="np")
    assert reg["labels"].dtype.kind == "f" and reg["x"].shape == (2, 2)
    pad = DataCollatorWithPadding(ToyTokenizer(), pad_to_multiple_of=4)
    out = pad([{"input_ids": [5, 6, 7, 8, 9], "label": 2}, {"input_ids": [5, 6], "label": 1}])
    assert out["input_ids"].shape == (2, 8) and out["input_ids"][1].tolist() == [5, 6, 0, 0, 0, 0, 0, 0]
    assert out["attention_mask"].sum(1).tolist() == [5, 2] and out["labels"].tolist() == [2, 1]
    tok = ToyTokenizer()
    tok.padding_side = "left"
    out = DataCollatorWithPadding(tok, padding="max_length", max_length=6)([{"input_ids": [5, 6, 7], "labels": [1, 2, 3]}, {"input_ids": [9], "labels": [4]}])
    assert out["input_ids"].tolist() == [[0, 0, 0, 5, 6, 7], [0, 0, 0, 0, 0, 9]] and out["labels"][1].tolist() == [-100] * 5 + [4]
