"""Typed configuration, the block-by-block model description, and the architecture registry."""
from .spec import (BiasAttentionSpec, MlstmSpec, MoeSpec, PostNormBlockSpec)  # noqa: F401
from .spec import (DeltaRuleSpec, LatentAttentionSpec, ParallelBlockSpec, RotaryPairsSpec, TokenSideSpec)  # noqa: F401
from .spec import (LimitedMlpSpec, SigmoidAttentionSpec)  # noqa: F401
from .spec import (NormedAttentionSpec, RotaryBlendSpec, SandwichBlockSpec)  # noqa: F401
from .spec import (AttentionSpec, BlockSpec, ConfigError, GatedMlpSpec, LinearHeadSpec, ModelSpec, NoPositionSpec,
                   RmsNormSpec, RotarySpec, ScheduleEntry)
from .registry import (Architecture, architecture, architecture_of, known_architectures,
                       read_config_json, register_architecture, unregister_architecture)
from . import llama as _llama
from .llama import LlamaConfig

register_architecture(Architecture(
    name=_llama.ARCHITECTURE,
    read_config=LlamaConfig.from_dict,
    to_spec=LlamaConfig.to_spec,
    tensor_name=_llama.tensor_name,
    cap_positions=LlamaConfig.with_max_positions,
    config_to_dict=LlamaConfig.to_dict,
))

from . import fesorax as _fesorax
from .fesorax import FesoraxConfig

register_architecture(Architecture(
    name=_fesorax.ARCHITECTURE,
    read_config=FesoraxConfig.from_dict,
    to_spec=FesoraxConfig.to_spec,
    tensor_name=_fesorax.tensor_name,
    cap_positions=FesoraxConfig.with_max_positions,
    config_to_dict=FesoraxConfig.to_dict,
    complete_config=_fesorax.with_sizes_of,
))

from . import lotilix as _lotilix
from .lotilix import LotilixConfig

register_architecture(Architecture(
    name=_lotilix.ARCHITECTURE,
    read_config=LotilixConfig.from_dict,
    to_spec=LotilixConfig.to_spec,
    tensor_name=_lotilix.tensor_name,
    cap_positions=LotilixConfig.with_max_positions,
    config_to_dict=LotilixConfig.to_dict,
    complete_config=_lotilix.with_sizes_of,
))

from . import mekevik as _mekevik
from .mekevik import MekevikConfig

register_architecture(Architecture(
    name=_mekevik.ARCHITECTURE,
    read_config=MekevikConfig.from_dict,
    to_spec=MekevikConfig.to_spec,
    tensor_name=_mekevik.tensor_name,
    cap_positions=MekevikConfig.with_max_positions,
    config_to_dict=MekevikConfig.to_dict,
    complete_config=_mekevik.with_sizes_of,
))

from . import netanex as _netanex
from .netanex import NetanexConfig

register_architecture(Architecture(
    name=_netanex.ARCHITECTURE,
    read_config=NetanexConfig.from_dict,
    to_spec=NetanexConfig.to_spec,
    tensor_name=_netanex.tensor_name,
    cap_positions=NetanexConfig.with_max_positions,
    config_to_dict=NetanexConfig.to_dict,
))

__all__ = [
    "NetanexConfig", "NormedAttentionSpec", "RotaryBlendSpec", "SandwichBlockSpec",
    "AttentionSpec", "BlockSpec", "ConfigError", "GatedMlpSpec", "LinearHeadSpec", "ModelSpec", "NoPositionSpec",
    "RmsNormSpec", "RotarySpec", "ScheduleEntry", "Architecture", "architecture", "architecture_of",
    "known_architectures", "read_config_json", "register_architecture", "unregister_architecture",
    "LlamaConfig", "FesoraxConfig", "BiasAttentionSpec", "MlstmSpec", "MoeSpec", "PostNormBlockSpec",
    "MekevikConfig", "SigmoidAttentionSpec", "LimitedMlpSpec",
    "LotilixConfig", "DeltaRuleSpec", "LatentAttentionSpec", "ParallelBlockSpec", "RotaryPairsSpec", "TokenSideSpec",
]
