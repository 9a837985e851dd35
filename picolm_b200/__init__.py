"""picolm_b200: a small model library with generation of its own for one NVIDIA
B200, after whoreson/picolm's Llama engine."""
from . import architectures  # noqa: F401
from .config import LlamaConfig, read_config, register_architecture, spec_of
from .parts import register_part

__version__ = "0.1.0"
__all__ = ["LlamaConfig", "read_config", "register_architecture", "spec_of", "register_part", "__version__"]
