from .engine_config import EngineConfig, SamplingParams
from .model_config import ConfigError, Qwen3Config, preset, preset_names
from .gamilorn_config import GamilornConfig
from .zatirax_config import ZatiraxConfig
from .kipezen_config import KipezenConfig
from .bovitar_config import BovitarConfig
