"""Parts a layer is made of.  Importing this package registers the built-in parts."""
from . import norm, position, attention, mlp, block, retention, streams, latent, moe, recurrent, parallel, embedding, linear_attention, state_space  # noqa: F401  (registration)
from .base import (Part, Norm, PositionEncoding, Mixer, SplitMixer, FeedForward, Block, Connector, EmbeddingExtra, LayerContext,
                   WeightSpec, KVNeed, StateNeed, MATRIX, VECTOR, INT_TABLE)
from .description import PartSpec, LayerSpec, ScheduleEntry, ModelDescription
from .model import Model, CacheBinding, build_part
from .streams import ResidualStreams
