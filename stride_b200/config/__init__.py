from .llama import ConfigError, LlamaConfig, RopeScaling
from .registry import Architecture, register_architecture, registered_architectures, resolve_architecture
from . import llama_spec as _llama_spec  # registers LlamaForCausalLM
from . import keralorn as _keralorn      # registers Keralorn
from . import ganupel as _ganupel        # registers Ganupel
from . import pusisun as _pusisun        # registers Pusisun
from . import sitivik as _sitivik        # registers Sitivik

__all__ = ["ConfigError", "LlamaConfig", "RopeScaling", "Architecture", "register_architecture",
           "registered_architectures", "resolve_architecture"]
