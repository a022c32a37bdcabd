from .model_config import (ModelConfig, Qwen3Config, ConfigError, read_config_json, write_config_json,
                           FULL_ATTENTION, SLIDING_ATTENTION, architecture_name)
from .tipezen_config import TipezenConfig, TipezenLayer, RotaryConfig
from .dominex_config import DominexConfig, DominexLayer, DominexExperts
from .sadupel_config import SadupelConfig, SadupelLayer, SadupelExperts
from .nugosun_config import NugosunConfig, NugosunLayer, NugosunMlp
from .engine_config import EngineConfig
