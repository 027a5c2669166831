"""rumus_b200 — a Blackwell (sm_100a) native deep-learning framework with the capabilities of
the RUMUS reference: PyTorch is the tensor/autograd layer, every hot operator is a hand-written
CUDA kernel, and multi-GPU paths fuse their collectives with the adjacent compute."""
__version__ = "0.1.0"

from . import ops  # noqa: F401
