"""Data engine (reference: rumus/src/data/): Dataset / DataItem / DataLoader and the `.rrec`
record format."""
from .dataset import DataItem, Dataset, TensorDataset, SyntheticTokens, SyntheticImages
from .dataloader import DataLoader, collate
from .record import RecordWriter, RecordDataset
from .native_loader import NativeBatchLoader

RecordReader = RecordDataset   # the reference's name for the mmap reader (rumus/src/data/record.rs)
