"""Graph ops (reference: rumus-graph/): CSR ``Graph`` and differentiable ``spmm``."""
from .graph import Graph, SparseTensor, spmm
