"""Parts a model is put together from: mixers, feed-forwards, norms, position
encodings and block arrangements, each registered under a kind and built from a
``PartSpec`` of sizes and constants."""

from .registry import (BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITION_ENCODINGS,
                       STREAM_ADDENDS, BuildContext, register_stream_addend, register_block, register_embedding, register_feed_forward,
                       register_head, register_mixer, register_norm, register_position_encoding)
from .spec import (CompositeSpec, LayerSpec, ModelPlan, PagedKVSpec, PartSpec, ScheduleEntry, StateSpec,
                   TensorSpec)
from . import (attention, block, delta_rule, embedding, feed_forward, gated_delta_rule, gated_linear_recurrence,
               latent_attention, masked_attention, norm, parallel, position, routed_experts, sigmoid_attention,
               state_space)  # noqa: F401  (register the kinds)
