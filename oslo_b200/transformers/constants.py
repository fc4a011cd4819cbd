"""Which keyword arguments of a model's ``forward`` carry a batch dimension, and where.

Used by the N-D tensor-parallel wrappers (inputs are split over the batch-holding groups) and by the pipeline
wrapper (inputs are split into micro-batches).  Parity: oslo/transformers/constants.py:1-27.
"""
BATCH_DIMENSIONS_TP = {
    "input_ids": 0,
    "attention_mask": 0,
    "token_type_ids": 0,
    "position_ids": 0,
    "inputs_embeds": 0,
    "labels": 0,
    "decoder_input_ids": 0,
    "decoder_attention_mask": 0,
    "decoder_inputs_embeds": 0,
    "encoder_hidden_states": 0,
    "encoder_attention_mask": 0,
    "pixel_values": 0,
    "start_positions": 0,
    "end_positions": 0,
}

BATCH_DIMENSIONS_PP = dict(BATCH_DIMENSIONS_TP)
BATCH_DIMENSIONS_PP.update({"head_mask": 1, "decoder_head_mask": 1, "cross_attn_head_mask": 1, "past_key_values": 2})
