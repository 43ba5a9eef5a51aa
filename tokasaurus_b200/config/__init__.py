from tokasaurus_b200.config.model_config import (  # noqa: F401
    ConfigError,
    LlamaConfig,
    RopeScaling,
    read_config_json,
    read_eos_token_ids,
)
from tokasaurus_b200.config.engine_config import (  # noqa: F401
    EngineConfig,
    OptionError,
    parse_overrides,
    parse_rope_scaling_override,
)
from tokasaurus_b200.config.registry import (  # noqa: F401
    Architecture,
    UnknownArchitectureError,
    known_architectures,
    lookup_architecture,
    register_architecture,
    unregister_architecture,
)
