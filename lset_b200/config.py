"""YAML configuration with dotted command-line overrides.

Same user-facing surface as the reference's config (lset/config.py:27-317): seventeen sections with
the same field names and defaults, ``from_yaml`` / ``apply_overrides`` / ``validate`` / ``to_yaml``
/ ``to_dict``, ``parse_overrides`` for ``--section.field value`` arguments. Unknown YAML sections and
keys are ignored; an unknown override is an error. A few fields are additions of this framework
(marked "extension") for features that the reference keeps as library-only code.

The implementation is schema driven: every value, whether it comes from YAML or from the command
line, goes through ``convert(value, annotation)``.
"""
from __future__ import annotations

import dataclasses
import typing
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, List, Optional

_NONE_WORDS = ("null", "none", "")
_TRUE_WORDS = ("true", "1", "yes")


def convert(value: Any, annotation: Any) -> Any:
    """Coerce ``value`` (usually a string) to the type described by ``annotation``."""
    origin = typing.get_origin(annotation)
    args = typing.get_args(annotation)
    if origin is typing.Union:  # Optional[X]
        inner = [a for a in args if a is not type(None)]
        if value is None or (isinstance(value, str) and value.lower() in _NONE_WORDS):
            return None
        return convert(value, inner[0]) if inner else value
    if origin in (list, List):
        inner = args[0] if args else str
        if value is None or (isinstance(value, str) and value.lower() in _NONE_WORDS):
            return None
        items = [s.strip() for s in value.split(",")] if isinstance(value, str) else list(value)
        return [convert(i, inner) for i in items]
    if annotation is bool:
        if isinstance(value, str):
            return value.lower() in _TRUE_WORDS
        return bool(value)
    if annotation is int and isinstance(value, str):
        return int(value)
    if annotation is float and isinstance(value, (str, int)) and not isinstance(value, bool):
        return float(value)
    return value


@dataclass
class ModelSection:
    path: str = ""
    pooling: str = "auto"  # auto | last_token | mean | cls | weighted_mean
    padding_side: str = "auto"  # auto | left | right
    fused_projections: bool = False


@dataclass
class DataSection:
    train_path: str = ""
    max_seq_length: int = 128
    num_hard_negatives: Optional[int] = None
    length_sorted: bool = False  # extension: longest-query-first ordering inside a batch
    use_template: bool = False  # extension: apply the model family's query/document template


@dataclass
class TrainingSection:
    batch_size: int = 8
    lr: float = 2e-5
    max_steps: Optional[int] = None
    epochs: int = 1
    scheduler: str = "cosine"  # cosine | linear | wsd | constant
    warmup_steps: int = 0
    grad_clip: float = 1.0
    gradient_accumulation_steps: int = 1
    seed: int = 42
    temperature: float = 0.02
    top_k: Optional[int] = None
    cascade: bool = False
    cascade_d_small: int = 64
    cascade_K_prime: int = 256
    matryoshka_dims: Optional[List[int]] = None
    learnable_temperature: bool = False  # extension
    weight_decay: float = 0.01  # extension (reference uses the AdamW default 0.01)


@dataclass
class PackingSection:
    enabled: bool = False


@dataclass
class GradCacheSection:
    enabled: bool = False
    token_budget: int = 4096
    chunk_size: Optional[int] = None
    selective_backward_keep: float = 1.0


@dataclass
class CompileSection:
    enabled: bool = False
    dynamic: bool = True
    backend: str = "inductor"
    mode: str = "default"


@dataclass
class ActivationCheckpointSection:
    enabled: bool = False
    mode: str = "selective"  # selective | full
    ratio: float = 1.0


@dataclass
class CudaGraphSection:
    enabled: bool = False
    token_budget: Optional[int] = None


@dataclass
class KernelsSection:
    fused: bool = True
    fused_residual_rmsnorm: bool = True
    fused_pool_normalize: bool = True
    fused_layernorm: bool = False


@dataclass
class AttentionSection:
    backend: str = "auto"  # auto | native | sdpa (flash_attn / varlen_attn are accepted aliases)


@dataclass
class DistributedSection:
    dp_size: int = 1
    tp_size: int = 1
    async_tp: bool = False  # sequence-parallel TP with collectives fused into the GEMMs (no torch.compile needed)
    # extension: shard the layers' parameters and gradients over the data-parallel ranks as well
    # (ZeRO-3; the default keeps a resident bf16 replica and shards gradients + optimizer state)
    reshard_after_forward: bool = False
    max_restarts: int = 0  # extension: passed to the launcher; resume from the newest checkpoint
    step_timeout_s: float = 0.0  # extension: watchdog limit for one step (0 = off)


@dataclass
class LoraSection:
    enabled: bool = False
    r: int = 8
    alpha: float = 16.0
    dropout: float = 0.0
    targets: Optional[List[str]] = None


@dataclass
class QloraSection:
    enabled: bool = False
    block_size: int = 64


@dataclass
class Fp8Section:
    enabled: bool = False
    recipe: str = "rowwise"


@dataclass
class CheckpointSection:
    save_steps: int = 0
    output_dir: str = "output/"
    resume_from: Optional[str] = None


@dataclass
class LoggingSection:
    log_interval: int = 10
    wandb: bool = False
    wandb_project: str = "lset"
    jsonl: bool = True  # extension: write metrics.jsonl beside the checkpoints


@dataclass
class EvalSection:
    tasks: Optional[List[str]] = None
    batch_size: int = 32
    max_length: int = 512


@dataclass
class LSETConfig:
    model: ModelSection = field(default_factory=ModelSection)
    data: DataSection = field(default_factory=DataSection)
    training: TrainingSection = field(default_factory=TrainingSection)
    packing: PackingSection = field(default_factory=PackingSection)
    grad_cache: GradCacheSection = field(default_factory=GradCacheSection)
    compile: CompileSection = field(default_factory=CompileSection)
    cuda_graph: CudaGraphSection = field(default_factory=CudaGraphSection)
    kernels: KernelsSection = field(default_factory=KernelsSection)
    attention: AttentionSection = field(default_factory=AttentionSection)
    activation_checkpoint: ActivationCheckpointSection = field(
        default_factory=ActivationCheckpointSection)
    distributed: DistributedSection = field(default_factory=DistributedSection)
    lora: LoraSection = field(default_factory=LoraSection)
    qlora: QloraSection = field(default_factory=QloraSection)
    fp8: Fp8Section = field(default_factory=Fp8Section)
    checkpoint: CheckpointSection = field(default_factory=CheckpointSection)
    logging: LoggingSection = field(default_factory=LoggingSection)
    eval: EvalSection = field(default_factory=EvalSection)

    # ------------------------------------------------------------------ construction
    @classmethod
    def from_yaml(cls, path) -> "LSETConfig":
        import yaml

        with open(path) as fh:
            tree = yaml.safe_load(fh) or {}
        return cls._from_dict(tree)

    @classmethod
    def _from_dict(cls, tree: dict) -> "LSETConfig":
        cfg = cls()
        for sec_name, body in (tree or {}).items():
            section = getattr(cfg, sec_name, None) if isinstance(sec_name, str) else None
            if section is None or not dataclasses.is_dataclass(section) or not isinstance(body, dict):
                continue
            hints = typing.get_type_hints(type(section))
            for key, raw in body.items():
                if key in hints:
                    ann = hints[key]
                    # YAML already typed most scalars; numeric strings ("2e-5") and comma-separated
                    # lists written as one string ("64,128") need help.
                    if isinstance(raw, str):
                        base = [a for a in typing.get_args(ann) if a is not type(None)] or [ann]
                        if base[0] in (int, float) or typing.get_origin(base[0]) in (list, List):
                            raw = convert(raw, ann)
                    setattr(section, key, raw)
        return cfg

    # ------------------------------------------------------------------ overrides
    def apply_overrides(self, overrides) -> None:
        for dotted, raw in overrides:
            sec_name, sep, key = dotted.partition(".")
            if not sep or not key:
                raise ValueError(f"Override key must be section.field: {dotted}")
            section = getattr(self, sec_name, None)
            if section is None or not dataclasses.is_dataclass(section):
                raise ValueError(f"Unknown config section: {sec_name}")
            hints = typing.get_type_hints(type(section))
            if key not in hints:
                raise ValueError(f"Unknown field {key} in section {sec_name}")
            setattr(section, key, convert(raw, hints[key]))

    # ------------------------------------------------------------------ validation
    def validate(self) -> None:
        cg, d = self.cuda_graph, self.distributed
        if cg.enabled and self.packing.enabled and not cg.token_budget:
            raise ValueError("cuda_graph.enabled + packing.enabled requires cuda_graph.token_budget")
        if self.qlora.enabled and d.tp_size > 1:
            raise ValueError("QLoRA + TP is not supported (NF4 weights are not tensor-parallel)")
        if self.fp8.enabled and (self.lora.enabled or self.qlora.enabled):
            raise ValueError("FP8 + LoRA/QLoRA is not supported")
        if cg.enabled and self.compile.enabled:
            raise ValueError("CUDA graph + torch.compile is redundant (use one or the other)")
        if cg.enabled and self.grad_cache.enabled:
            raise ValueError("CUDA graph + GradCache is not supported")
        if d.dp_size < 1 or d.tp_size < 1:
            raise ValueError("distributed.dp_size and distributed.tp_size must be >= 1")
        if self.training.gradient_accumulation_steps < 1:
            raise ValueError("training.gradient_accumulation_steps must be >= 1")

    # ------------------------------------------------------------------ serialisation
    def to_dict(self) -> dict:
        return dataclasses.asdict(self)

    def to_yaml(self, path) -> None:
        import yaml

        Path(path).parent.mkdir(parents=True, exist_ok=True)
        with open(path, "w") as fh:
            yaml.dump(self.to_dict(), fh, default_flow_style=False, sort_keys=False)


def parse_overrides(argv) -> list:
    """Collect ``--section.field value`` pairs; a bare ``--section.field`` means ``true``."""
    out, i = [], 0
    argv = list(argv)
    while i < len(argv):
        tok = argv[i]
        if tok.startswith("--") and "." in tok and tok != "--config":
            nxt = argv[i + 1] if i + 1 < len(argv) else None
            if nxt is not None and not nxt.startswith("--"):
                out.append((tok[2:], nxt))
                i += 2
                continue
            out.append((tok[2:], "true"))
        i += 1
    return out


def resolve_path(p: str) -> str:
    return str(Path(p).expanduser()) if p else p
