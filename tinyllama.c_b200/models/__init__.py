from .model import Model  # noqa: F401
from . import falcon_h1  # noqa: F401  (registers FalconH1ForCausalLM)
