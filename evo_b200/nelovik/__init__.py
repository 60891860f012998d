"""Nelovik: layers that run mixer and feed-forward side by side on an fp32 stream; gated delta rule, state-space-duality and
pooled-window attention mixers; the model class follows the framework's object protocol."""
from .config import NelovikConfig
from .model import Nelovik

__all__ = ["Nelovik", "NelovikConfig"]
