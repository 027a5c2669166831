"""Parallelism strategies (reference: rumus/src/nn/{parallel,fsdp}.rs, rumus-distributed/)."""
from .flat import FlatUnit, build_units, default_units
from .fsdp import FSDP
from .cp import ring_attention, ulysses_attention
from .collective import AllReduceHandle, all_reduce, async_all_reduce
