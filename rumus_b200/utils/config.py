"""Configuration: dataclass configs loadable from YAML / dicts, named presets for the five
benchmark configurations, and the ``RB_BACKEND={fused,nccl,cpu}`` switch between the fused
collective kernels, the NCCL baseline and CPU (gloo) ranks.

The reference configures everything through constructor arguments, Cargo features and seven
hand-parsed server flags (rumus-serve/src/main.rs:13-62)."""
from __future__ import annotations

from dataclasses import asdict, dataclass, field
from typing import Optional


@dataclass
class ParallelConfig:
    dp: int = 1
    tp: int = 1
    pp: int = 1
    fsdp: bool = False
    micro_batches: int = 1
    backend: str = "fused"      # fused | nccl | cpu
    reshard_after_forward: bool = False   # FSDP: keep only shards between a block's forward and backward (nccl / cpu backends)


@dataclass
class PrecisionConfig:
    compute: str = "bf16"       # fp32 | bf16 | fp16
    master_weights: bool = True
    loss_scaling: bool = False  # dynamic loss scaling (fp16)
    init_scale: float = 65536.0


@dataclass
class ModelPreset:
    family: str                 # gpt | llama | resnet50
    kwargs: dict = field(default_factory=dict)


@dataclass
class TrainConfig:
    name: str
    model: ModelPreset
    parallel: ParallelConfig = field(default_factory=ParallelConfig)
    precision: PrecisionConfig = field(default_factory=PrecisionConfig)
    optimizer: str = "adam"
    lr: float = 1e-3
    momentum: float = 0.0
    seqs_per_gpu: int = 8
    global_batch: Optional[int] = None
    steps: int = 50
    seed: int = 0

    def to_dict(self) -> dict:
        return asdict(self)


PRESETS = {
    "tiny-decoder-cpu": TrainConfig(
        "tiny-decoder-cpu",
        ModelPreset("gpt", dict(vocab_size=1024, seq_len=64, d_model=128, num_heads=4, num_layers=2,
                                ffn_dim=512, activation="relu")),
        precision=PrecisionConfig("fp32", False), lr=1e-3, seqs_per_gpu=8, steps=50),
    "gpt-1.3b-fsdp": TrainConfig(
        "gpt-1.3b-fsdp",
        ModelPreset("gpt", dict(vocab_size=50304, seq_len=2048, d_model=2048, num_heads=16, num_layers=24,
                                ffn_dim=8192, activation="gelu")),
        ParallelConfig(dp=8, fsdp=True), PrecisionConfig("bf16", True), lr=1e-4, seqs_per_gpu=8),
    "llama-7b-tp4-pp2": TrainConfig(
        "llama-7b-tp4-pp2",
        ModelPreset("llama", dict(vocab_size=32000, seq_len=4096, d_model=4096, num_heads=32,
                                  num_kv_heads=32, num_layers=32, ffn_dim=11008)),
        ParallelConfig(tp=4, pp=2, micro_batches=8), PrecisionConfig("bf16", True), lr=1e-4,
        global_batch=64),
    "resnet50-dp-fp16": TrainConfig(
        "resnet50-dp-fp16", ModelPreset("resnet50", dict(num_classes=1000)),
        ParallelConfig(dp=8), PrecisionConfig("fp16", True, True), optimizer="sgd", lr=0.1, momentum=0.9,
        seqs_per_gpu=256),
    "llama-7b-int4-serve-tp8": TrainConfig(
        "llama-7b-int4-serve-tp8",
        ModelPreset("llama", dict(vocab_size=32000, seq_len=4096, d_model=4096, num_heads=32,
                                  num_kv_heads=32, num_layers=32, ffn_dim=11008)),
        ParallelConfig(tp=8), PrecisionConfig("bf16", False)),
}


def load_config(source) -> TrainConfig:
    """``source``: preset name, dict, or path to a YAML file with the same fields."""
    if isinstance(source, str) and source in PRESETS:
        return PRESETS[source]
    if isinstance(source, str):
        import yaml
        with open(source) as f:
            source = yaml.safe_load(f)
    d = dict(source)
    d["model"] = ModelPreset(**d["model"])
    d["parallel"] = ParallelConfig(**d.get("parallel", {}))
    d["precision"] = PrecisionConfig(**d.get("precision", {}))
    return TrainConfig(**d)
