from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleStep
from .qwen3 import ARCHITECTURE, QwenConfig, read_config_json
from .lanizen import LanizenConfig
from . import lanizen as _lanizen
from .gidirax import GidiraxConfig
from . import gidirax as _gidirax
from .sobunex import SobunexConfig
from . import sobunex as _sobunex
from .pivavik import PivavikConfig
from . import pivavik as _pivavik
from .registry import (config_class_for, config_from_dict, config_from_model_dir,
                       register_architecture, registered_architectures, unregister_architecture)

register_architecture(ARCHITECTURE, QwenConfig)
register_architecture(_lanizen.ARCHITECTURE, LanizenConfig)
register_architecture(_gidirax.ARCHITECTURE, GidiraxConfig)
register_architecture(_sobunex.ARCHITECTURE, SobunexConfig)
register_architecture(_pivavik.ARCHITECTURE, PivavikConfig)
