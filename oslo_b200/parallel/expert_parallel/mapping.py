"""Which linears of a model's feed-forward blocks become the front / behind halves of a mixture-of-experts layer.

``Front(names..., layer="transformer.h")`` marks the first FFN linear (it gets the router, the dispatch and the experts'
first GEMM), ``Behind`` the second (experts' second GEMM and the combine).  ``layer`` is the dotted path of the
``ModuleList`` holding the transformer layers, used to read the layer index from a module name; ``enc_name`` /
``dec_name`` tell encoder stacks from decoder stacks.  Parity: oslo/torch/nn/parallel/expert_parallel/mapping.py.
"""
from __future__ import annotations

from typing import List, Optional


class ExpertParallelInfo:
    def __init__(self, *name, layer: str, enc_name: Optional[str] = None, dec_name: Optional[str] = None, reversed: bool = False):
        self.name = name
        self.layer = layer
        self.enc_name, self.dec_name = enc_name, dec_name
        self.reversed = reversed


class Front(ExpertParallelInfo):
    pass


class Behind(ExpertParallelInfo):
    pass


class ExpertParallelMapping:
    __MAPPING__ = {
        "GPT2": [Front("mlp.c_fc", layer="transformer.h", dec_name="transformer", reversed=True),
                 Behind("mlp.c_proj", layer="transformer.h", dec_name="transformer", reversed=True)],
        "MoEGPT": [Front("mlp.c_fc", layer="transformer.h", dec_name="transformer", reversed=True),
                   Behind("mlp.c_proj", layer="transformer.h", dec_name="transformer", reversed=True)],
        "GPTNeoX": [Front("mlp.dense_h_to_4h", layer="gpt_neox.layers", dec_name="gpt_neox"),
                    Behind("mlp.dense_4h_to_h", layer="gpt_neox.layers", dec_name="gpt_neox")],
        "Bert": [Front("intermediate.dense", layer="bert.encoder.layer", enc_name="encoder"),
                 Behind("output.dense", layer="bert.encoder.layer", enc_name="encoder")],
        "Roberta": [Front("intermediate.dense", layer="roberta.encoder.layer", enc_name="encoder"),
                    Behind("output.dense", layer="roberta.encoder.layer", enc_name="encoder")],
        "Albert": [Front("ffn", layer="albert.encoder.albert_layer_groups.albert_layers", enc_name="encoder"),
                   Behind("ffn_output", layer="albert.encoder.albert_layer_groups.albert_layers", enc_name="encoder")],
        "T5": [Front("DenseReluDense.wi", layer="block", enc_name="encoder", dec_name="decoder"),
               Behind("DenseReluDense.wo", layer="block", enc_name="encoder", dec_name="decoder")],
        "Bart": [Front("fc1", layer="layers", enc_name="encoder", dec_name="decoder"),
                 Behind("fc2", layer="layers", enc_name="encoder", dec_name="decoder")],
        "Blenderbot": [Front("fc1", layer="layers", enc_name="encoder", dec_name="decoder"),
                       Behind("fc2", layer="layers", enc_name="encoder", dec_name="decoder")],
        "Electra": [Front("intermediate.dense", layer="electra.encoder.layer", enc_name="encoder"),
                    Behind("output.dense", layer="electra.encoder.layer", enc_name="encoder")],
        "DistilBert": [Front("ffn.lin1", layer="distilbert.transformer.layer", enc_name="transformer"),
                       Behind("ffn.lin2", layer="distilbert.transformer.layer", enc_name="transformer")],
        "GPTNeo": [Front("mlp.c_fc", layer="transformer.h", dec_name="transformer"),
                   Behind("mlp.c_proj", layer="transformer.h", dec_name="transformer")],
        "GPTJ": [Front("mlp.fc_in", layer="transformer.h", dec_name="transformer"),
                 Behind("mlp.fc_out", layer="transformer.h", dec_name="transformer")],
        "OPT": [Front("fc1", layer="model.decoder.layers", dec_name="decoder"),
                Behind("fc2", layer="model.decoder.layers", dec_name="decoder")],
        "ViT": [Front("intermediate.dense", layer="vit.encoder.layer", enc_name="encoder"),
                Behind("output.dense", layer="vit.encoder.layer", enc_name="encoder")],
    }
    # families that share a table
    __MAPPING__["BlenderbotSmall"] = __MAPPING__["Blenderbot"]
    __MAPPING__["MBart"] = __MAPPING__["Bart"]
    __MAPPING__["MT5"] = __MAPPING__["T5"]

    def __init__(self, mapping: Optional[dict] = None):
        self._table = dict(self.__MAPPING__)
        if mapping:
            self._table.update(mapping)

    def get_mapping(self, model) -> List[ExpertParallelInfo]:
        best = None
        for cls in type(model).__mro__:
            for key, entries in self._table.items():
                if cls.__name__.startswith(key) and (best is None or len(key) > best[0]):
                    best = (len(key), entries)
            if best:
                break
        if best is None:
            raise ValueError(f"{type(model).__name__} has no expert-parallel mapping; pass one explicitly")
        return best[1]

    def match(self, model, module_name: str):
        """``(info, layer_index, stack)`` for a module name, or None."""
        for info in self.get_mapping(model):
            for n in info.name:
                if module_name.endswith("." + n) or module_name == n:
                    prefix = module_name[: -len(n)].rstrip(".")
                    parts = prefix.split(".")
                    # the name must be everything after the layer index: ``layer.3.output.dense`` is the feed-forward
                    # output, ``layer.3.attention.output.dense`` (same suffix) is not
                    if not parts or not parts[-1].isdigit():
                        continue
                    idx = int(parts[-1])
                    stack = "dec"
                    if info.enc_name and info.enc_name in module_name.split("."):
                        stack = "enc"
                    elif info.dec_name and info.dec_name in module_name.split("."):
                        stack = "dec"
                    return info, idx, stack
        return None
