"""Parts a model is put together from.  Importing the package registers the built-in kinds."""
from . import attention, block, embedding, ffn, norm, position  # noqa: F401
from .base import (CacheRequest, FeedForward, Mixer, Norm, Part, Runtime, StepBatch, TensorRequest)
from .registry import (part_class, register_arrangement, register_embedding, register_ffn, register_head,
                       register_mixer, register_norm, register_part, register_position)
from .spec import (AttentionSpec, EmbeddingSpec, GatedMlpSpec, HeadSpec, LayerSpec, ModelSpec,
                   NormSpec, RopeSpec, ScheduleEntry)
from .workspace import Workspace
