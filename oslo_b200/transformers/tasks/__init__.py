from .data_base import BaseProcessor, pad_sequences
from .data_causal_lm import DataCollatorForCausalLM, ProcessorForCausalLM
from .data_classification import (
    DataCollatorForSequenceClassification,
    DataCollatorForSummarization,
    DataCollatorForTokenClassification,
    ProcessorForSequenceClassification,
    ProcessorForSummarization,
    ProcessorForTokenClassification,
)
from .data_masked_lm import DataCollatorForMaskedLM, ProcessorForMaskedLM
from .data_pretraining import (
    DataCollatorForAlbertPretraining,
    DataCollatorForBartPretraining,
    DataCollatorForBertPretraining,
    DataCollatorForT5Pretraining,
    ProcessorForAlbertPretraining,
    ProcessorForBartPretraining,
    ProcessorForBertPretraining,
    ProcessorForT5Pretraining,
)
from .data_utils import Corpus, CorpusType, batch_iterator, load_corpora, read_sent_text, serialize_corpora, train_tokenizer
