"""Configuration: the typed per-architecture readers, the neutral `ModelSpec`, and the registry."""

from .lfm2_moe import ARCHITECTURES as _LFM2_ARCHS
from .lfm2_moe import MODEL_TYPES as _LFM2_TYPES
from .lfm2_moe import Lfm2MoeConfig
from .registry import (REGISTRY, Architecture, architecture_of, read_model_config, register, resolve_model_folder,
                       spec_of, unregister)
from .niralix import ARCHITECTURES as _NIRALIX_ARCHS
from .niralix import MODEL_TYPES as _NIRALIX_TYPES
from .niralix import NiralixConfig
from .puripel import ARCHITECTURES as _PURIPEL_ARCHS
from .puripel import MODEL_TYPES as _PURIPEL_TYPES
from .puripel import PuripelConfig
from .sebilorn import ARCHITECTURES as _SEBILORN_ARCHS
from .sebilorn import MODEL_TYPES as _SEBILORN_TYPES
from .sebilorn import SebilornConfig
from .sifupel import ARCHITECTURES as _SIFUPEL_ARCHS
from .sifupel import MODEL_TYPES as _SIFUPEL_TYPES
from .sifupel import SifupelConfig
from .spec import LayerSpec, ModelSpec, PartSpec, Site, StreamAdd, plain_schedule

register(Architecture(name="lfm2_moe", architectures=_LFM2_ARCHS, model_types=_LFM2_TYPES,
                      read_config=Lfm2MoeConfig.from_dict))

register(Architecture(name="sifupel", architectures=_SIFUPEL_ARCHS, model_types=_SIFUPEL_TYPES,
                      read_config=SifupelConfig.from_dict))

register(Architecture(name="puripel", architectures=_PURIPEL_ARCHS, model_types=_PURIPEL_TYPES,
                      read_config=PuripelConfig.from_dict))

register(Architecture(name="sebilorn", architectures=_SEBILORN_ARCHS, model_types=_SEBILORN_TYPES,
                      read_config=SebilornConfig.from_dict))

register(Architecture(name="niralix", architectures=_NIRALIX_ARCHS, model_types=_NIRALIX_TYPES,
                      read_config=NiralixConfig.from_dict))

__all__ = ["NiralixConfig", "PuripelConfig", "SebilornConfig", "REGISTRY", "Architecture", "architecture_of", "read_model_config", "register", "unregister",
           "resolve_model_folder", "spec_of", "LayerSpec", "ModelSpec", "PartSpec", "Site", "StreamAdd", "plain_schedule",
           "Lfm2MoeConfig", "SifupelConfig"]
