"""Architectures as data.  Importing the package registers the built-in architecture."""

from .plan import LayerRun, LayerSpec, ModelPlan  # noqa: F401
from .model import Model  # noqa: F401
from . import llama  # noqa: F401,E402
