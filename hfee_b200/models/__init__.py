"""Architectures: each module registers itself in ``hfee_b200.config.registry``."""
from . import llama  # noqa: F401
