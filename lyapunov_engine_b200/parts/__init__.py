from . import (attention, base, block, delta_rule, differential_attention, embedding, feedforward, hyper,  # noqa: F401  (registers the kinds)
               latent_attention, mlstm, moe, norm, rope, short_conv, side_by_side, state_space, stream_inputs)
from .base import (BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, INPUT_FILTERS, MIXERS, NORMS, POSITION_ENCODINGS, STREAM_INPUTS, Block,
                   FeedForward, InputFilter, NormedAddend, ScaledAddend, StreamInput, register_input_filter, register_stream_input,
                   KVNeed, LayerSpec, Mixer, ModelSpec, Norm, Part, PartSpec, PositionEncoding, ResidualStream,
                   RunSpec, StateNeed, TensorDecl, register_block, register_embedding, register_feed_forward,
                   register_head, register_mixer, register_norm, register_position_encoding)
