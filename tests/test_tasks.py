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
