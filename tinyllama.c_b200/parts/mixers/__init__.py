from .attention import AttentionMixer  # noqa: F401
from .mamba2 import Mamba2Mixer  # noqa: F401
