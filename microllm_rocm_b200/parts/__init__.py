from .base import (Runtime, WeightSpec, PagedKVNeed, PagedRowsNeed, FixedStateNeed, CompositeNeed, RunEntry, RUN_ENTRIES, register_run_entry, PagedKVView, StateView, StepContext, Part, Norm,
                   PositionEncoding, RotaryTable, Mixer, FeedForward, Block, NORMS, POSITION_ENCODINGS, MIXERS,
                   FEED_FORWARDS, BLOCKS, EMBEDDINGS, HEADS, register_norm, register_position_encoding,
                   register_mixer, register_feed_forward, register_block, register_embedding, register_head)
from . import norm, rotary, positions, attention, latent_attention, mlp, routed, embedding, block, loop, delta_rule, linear_attention, parallel  # noqa: F401  (register the built-in kinds)
from .build import Model, build_model
