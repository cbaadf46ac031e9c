"""Parts a model is put together from: mixers, feed-forwards, norms, position encodings, blocks."""
from .base import (Block, Embedding, FeedForward, Head, LazyNorm, Mixer, Norm, PagedKVBinding,
                   PagedKVSpec, Part, PositionEncoding, StateBinding, StateSpec, StepContext, Summed,
                   TensorSpec,
                   make_part, register_block, register_feed_forward, register_mixer,
                   register_norm, register_part, register_position, register_stream_input,
                   StreamInput)
from .plan import LayerSpec, ModelPlan, PartSpec, RunEntry, sequential_run
from . import (attention, block, delta_rule, embedding, feed_forward, gated_attention,  # noqa: F401
               latent_attention, linear_attention, norm, position, routed, state_space,
               stream_input, wide_attention)
from .model import DecoderModel
