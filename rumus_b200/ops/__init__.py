"""Operator layer: ``functional`` (differentiable ops), ``native`` (raw kernel launchers)."""
from . import _lib
from .functional import *  # noqa: F401,F403
from . import functional
