"""Gakupel model family: layer norms on the sublayers' outputs, a learned mix of all earlier layers' results, causal attention whose
values are its keys, biased attention with a sink beside a matrix memory, the gated delta rule, and grouped expert routing."""
from .config import GakupelConfig
from .model import Gakupel

__all__ = ["Gakupel", "GakupelConfig"]
