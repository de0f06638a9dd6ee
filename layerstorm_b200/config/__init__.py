from .loader import (ConfigError, PRESET_OVERLAYS, apply_env, deep_merge, fill_model_from_checkpoint, get_path, load_config,
                     model_config_from, model_section_from, parse_pin, set_path, validate)
from .schema import SCHEMA, defaults, json_schema, leaf_paths, live_changeable_fields
