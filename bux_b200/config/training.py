"""Training settings: data, optimizer, schedule, precision, mesh, layout, methods, ...

Field names and defaults are the language's public surface and enter the run id, so
they follow the reference schema (``src/bux/train/config.py:61-1362``). The
B200-specific meaning of the "how" settings (mesh / layout / methods / compiler),
which stay outside the id, is documented on each class.
"""

from __future__ import annotations

import itertools
import math
from typing import Annotated, Literal, Optional, Union

from pydantic import AfterValidator, BeforeValidator, Field, model_validator

from .layers import Config, RoPEScalingConfig, tags_of

Positive = Annotated[int, Field(gt=0)]
Fraction = Annotated[float, Field(ge=0, le=1)]
UnitOpen = Annotated[float, Field(gt=0, lt=1)]


def _as_tuple(v):
    return (v,) if isinstance(v, (str, int)) else v


def _start_before_end(split):
    if split[0] >= split[1]:
        raise ValueError("a split is [start, end], with start < end")
    return split


Split = Annotated[tuple[Fraction, Fraction], AfterValidator(_start_before_end)]


# ---------------------------------------------------------------- data
class TextConfig(Config):
    type: Literal["text"] = "text"
    path: str
    column: str = "text"
    bos: bool = False
    eos: bool = True
    split: Split = (0.0, 1.0)


class ChatConfig(Config):
    type: Literal["chat"] = "chat"
    path: str
    column: str = "messages"
    template: Optional[str] = None
    train_on: Literal["assistant", "last", "all"] = "assistant"
    split: Split = (0.0, 1.0)


class TokensConfig(Config):
    type: Literal["tokens"] = "tokens"
    path: str
    dtype: Literal["uint16", "uint32"] = "uint16"
    header: int = 0


class SyntheticConfig(Config):
    type: Literal["synthetic"] = "synthetic"


Source = Annotated[
    Union[TextConfig, ChatConfig, TokensConfig, SyntheticConfig], Field(discriminator="type")
]


class Weighted(Config):
    weight: Annotated[float, Field(gt=0)]
    source: Source


class MixtureConfig(Config):
    type: Literal["mix"] = "mix"
    sources: tuple[Weighted, ...]


DataConfig = Annotated[
    Union[TextConfig, ChatConfig, TokensConfig, SyntheticConfig, MixtureConfig],
    Field(discriminator="type"),
]
SOURCES = (TextConfig, ChatConfig, TokensConfig, SyntheticConfig, MixtureConfig)
DOCUMENTS = (TextConfig, ChatConfig)


class TokenizerConfig(Config):
    type: Literal["tokenizer"] = "tokenizer"
    name: str
    bos: str = "<|endoftext|>"
    eos: str = "<|endoftext|>"
    added: tuple[str, ...] = ()


class ConcatPacking(Config):
    type: Literal["concat"] = "concat"
    doc_mask: bool = False
    chunk: Positive = 16_000_000


class GreedyPacking(Config):
    type: Literal["greedy"] = "greedy"
    doc_mask: bool = True
    long: Literal["drop", "truncate", "split"] = "drop"
    max_docs: Optional[Positive] = None
    chunk: Positive = 16_000_000


class BestFitPacking(Config):
    type: Literal["best_fit"] = "best_fit"
    doc_mask: bool = True
    long: Literal["drop", "truncate", "split"] = "split"
    max_docs: Optional[Positive] = None
    sort: bool = True
    chunk: Positive = 16_000_000


PackingConfig = Annotated[
    Union[ConcatPacking, GreedyPacking, BestFitPacking], Field(discriminator="type")
]


# ---------------------------------------------------------------- optimizers
class AdamWConfig(Config):
    type: Literal["adamw"] = "adamw"
    lr: float
    b1: float = 0.9
    b2: float = 0.95
    eps: float = 1e-8
    weight_decay: float = 0.1
    cautious_weight_decay: bool = False


class MuonConfig(Config):
    type: Literal["muon"] = "muon"
    lr: float
    momentum: float = 0.95
    nesterov: bool = True
    ns_steps: int = 5
    ns_coefficients: str = "jordan"
    ns_algorithm: str = "standard"
    ns_restarts: Optional[Annotated[tuple[Positive, ...], BeforeValidator(_as_tuple)]] = None
    ns_dtype: Literal["float32", "bfloat16"] = "bfloat16"
    weight_decay: float = 0.1
    cautious_weight_decay: bool = False
    consistent_rms: Optional[float] = 0.2
    adam: Optional[AdamWConfig] = None


class NorMuonConfig(MuonConfig):
    type: Literal["normuon"] = "normuon"  # type: ignore[assignment]
    b2: float = 0.95
    eps: float = 1e-10


OptimizerConfig = Annotated[
    Union[AdamWConfig, MuonConfig, NorMuonConfig], Field(discriminator="type")
]


class EMAConfig(Config):
    type: Literal["ema"] = "ema"
    window: Union[Positive, UnitOpen] = 0.25
    blend: Fraction = 0.65

    def steps(self, steps: int) -> int:
        window = self.window if isinstance(self.window, int) else self.window * steps
        return min(max(round(window), 1), steps)


# ---------------------------------------------------------------- schedules
def _warmup_from_zero(warmup):
    if warmup < 0:
        raise ValueError("a warmup is a count of steps from 0, or a share of them below 1")
    return warmup


Warmup = Annotated[Union[int, UnitOpen], AfterValidator(_warmup_from_zero)]
Shape = Literal["linear", "sqrt", "cosine", "exp", "geometric", "constant"]


def _increasing(shares):
    if any(a >= b for a, b in itertools.pairwise(shares)):
        raise ValueError("the shares of the steps must increase")
    return shares


def _geometric_needs_positive(shape, *ends):
    if shape == "geometric" and min(ends) <= 0:
        raise ValueError("a geometric cooldown or piece starts and ends above 0")


class ConstantSchedule(Config):
    type: Literal["constant"] = "constant"
    warmup: Warmup = 0


class CosineSchedule(Config):
    type: Literal["cosine"] = "cosine"
    warmup: Warmup = 0
    final: float = 0.1
    horizon: Annotated[float, Field(gt=0)] = 1.0


class WSDSchedule(Config):
    type: Literal["wsd"] = "wsd"
    warmup: Warmup = 0
    decay: Fraction = 0.2
    final: float = 0.0
    shape: Shape = "linear"

    def cooldown(self, steps: int) -> int:
        return round(self.decay * steps)

    @model_validator(mode="after")
    def _ends(self):
        _geometric_needs_positive(self.shape, self.final)
        return self


class LinearDecaySchedule(Config):
    type: Literal["linear_decay"] = "linear_decay"
    warmup: Warmup = 0
    final: float = 0.0


class MultiStepSchedule(Config):
    type: Literal["multistep"] = "multistep"
    warmup: Warmup = 0
    at: Annotated[tuple[Fraction, ...], AfterValidator(_increasing)] = (0.8, 0.9)
    factor: float = 0.316


class PowerSchedule(Config):
    type: Literal["power"] = "power"
    warmup: Warmup = 0
    a: float = 4.0
    b: float = -0.51
    decay: Fraction = 0.1
    final: float = 0.0
    shape: Shape = "exp"

    def cooldown(self, steps: int) -> int:
        return round(self.decay * steps)

    @model_validator(mode="after")
    def _ends(self):
        _geometric_needs_positive(self.shape, self.final)
        return self


class Piece(Config):
    type: Literal["piece"] = "piece"
    until: Fraction = 1.0
    to: Optional[float] = None
    shape: Shape = "constant"


def levels(pieces) -> list:
    """Multiplier at the start of each piece and after the last one."""
    found = [1.0]
    for p in pieces:
        found.append(found[-1] if p.to is None else p.to)
    return found


def _pieces_ordered(pieces):
    if not pieces or pieces[-1].until != 1:
        raise ValueError("the last piece ends at 1, the end of the run")
    _increasing(tuple(p.until for p in pieces))
    for p, start in zip(pieces, levels(pieces)):
        _geometric_needs_positive(p.shape, start, start if p.to is None else p.to)
    return pieces


class PiecewiseSchedule(Config):
    type: Literal["piecewise"] = "piecewise"
    warmup: Warmup = 0
    pieces: Annotated[tuple[Piece, ...], AfterValidator(_pieces_ordered)]

    def cooldown(self, steps: int) -> int:
        return steps - round(self.pieces[0].until * steps)


ScheduleConfig = Annotated[
    Union[
        ConstantSchedule, CosineSchedule, WSDSchedule, LinearDecaySchedule,
        MultiStepSchedule, PowerSchedule, PiecewiseSchedule,
    ],
    Field(discriminator="type"),
]
COOLED = (WSDSchedule, PowerSchedule, PiecewiseSchedule)


def warmup_steps(c, steps: int) -> int:
    return round(c.warmup * steps) if isinstance(c.warmup, float) else c.warmup


# ---------------------------------------------------------------- curriculum
At = Union[Annotated[int, Field(gt=0)], UnitOpen]


class PhaseConfig(Config):
    type: Literal["phase"] = "phase"
    at: At
    seq_len: Optional[Annotated[int, Field(ge=2)]] = None
    batch: Optional[Positive] = None
    data: Optional[DataConfig] = None
    rope_scaling: Optional[RoPEScalingConfig] = None
    rope_base: Optional[Annotated[float, Field(gt=0)]] = None

    def start(self, steps: int) -> int:
        return round(self.at * steps) if isinstance(self.at, float) else self.at


class RampConfig(Config):
    type: Literal["ramp"] = "ramp"
    start: Positive
    steps: Positive
    multiple: Optional[Positive] = None


def _one_phase(v):
    return (v,) if isinstance(v, PhaseConfig) else v


Phases = Annotated[tuple[PhaseConfig, ...], BeforeValidator(_one_phase)]


class PrefixConfig(Config):
    type: Literal["prefix"] = "prefix"
    weight: Annotated[float, Field(ge=0)] = 0.25
    hold: Fraction = 1 / 3
    decay: Fraction = 1 / 3


class LossConfig(Config):
    type: Literal["loss"] = "loss"
    z: float = 0.0
    mtp: float = 0.3
    prefix: Optional[PrefixConfig] = None


def _ascending(v):
    if any(a >= b for a, b in itertools.pairwise(v)):
        raise ValueError(f"positions go up, one after another: {list(v)}")
    return v


Positions = Annotated[
    tuple[Positive, ...], BeforeValidator(_as_tuple), AfterValidator(_ascending)
]


class EvalConfig(Config):
    type: Literal["eval"] = "eval"
    name: Annotated[str, Field(min_length=1)] = "eval"
    data: DataConfig
    every: Positive = 1000
    batches: Positive = 10
    seq_len: Optional[Annotated[int, Field(ge=2)]] = None
    batch: Optional[Positive] = None
    positions: Positions = ()


def buckets(positions) -> list:
    return [f"{p // 1024}k" if p and p % 1024 == 0 else str(p) for p in (0, *positions)]


def metrics(e: EvalConfig, bpb: bool) -> list:
    """Names of the metrics an eval logs (per position bucket too)."""
    found = [f"{e.name}_{k}" for k in (["loss", "bpb"] if bpb else ["loss"])]
    return found + [f"{m}_{b}" for m in found for b in buckets(e.positions)]


def _each(evals):
    return () if evals is None else evals if isinstance(evals, tuple) else (evals,)


def _distinct_names(evals):
    names = [e.name for e in _each(evals)]
    if len(set(names)) < len(names):
        raise ValueError('each eval needs a name of its own: eval(name="web", ...)')
    return evals


Evals = Annotated[
    Union[EvalConfig, tuple[EvalConfig, ...], None], AfterValidator(_distinct_names)
]


# ---------------------------------------------------------------- watching a run
class CheckpointConfig(Config):
    type: Literal["checkpoint"] = "checkpoint"
    every: Positive = 1000
    keep: Positive = 2


class WandbConfig(Config):
    type: Literal["wandb"] = "wandb"
    project: str = "bux"
    entity: Optional[str] = None
    group: Optional[str] = None
    tags: tuple[str, ...] = ()
    mode: Optional[Literal["online", "offline", "disabled"]] = None


class TensorBoardConfig(Config):
    type: Literal["tensorboard"] = "tensorboard"


Tracker = Annotated[Union[WandbConfig, TensorBoardConfig], Field(discriminator="type")]


class LogConfig(Config):
    type: Literal["log"] = "log"
    every: Positive = 10
    trackers: tuple[Tracker, ...] = ()


class ObserveConfig(Config):
    type: Literal["observe"] = "observe"
    every: Positive = 100
    histograms: bool = False


class ProfileConfig(Config):
    """``tool``: ``torch`` (alias ``jax`` kept for source compatibility) traces with
    the CUPTI-backed torch profiler; ``nsys`` / ``ncu`` relaunch under the tool."""

    type: Literal["profile"] = "profile"
    start: Annotated[int, Field(ge=0)] = 10
    steps: Positive = 5
    tool: str = "jax"
    options: str = ""


# ---------------------------------------------------------------- precision
Pass = Literal["fprop", "dgrad", "wgrad"]
PASSES = ("fprop", "dgrad", "wgrad")
GROUPED = ("compute", "mxfp8", "mxfp8_2d")


def _grouped_format(fmt):
    if fmt not in (None, *GROUPED):
        raise ValueError(
            f"the routed experts multiply in {', '.join(GROUPED)}: bux has no grouped "
            f"GEMM in {fmt}"
        )
    return fmt


Branches = Union[Annotated[int, Field(ge=0)], UnitOpen]


class RolesConfig(Config):
    type: Literal["roles"] = "roles"
    q: Optional[str] = None
    kv: Optional[str] = None
    o: Optional[str] = None
    mlp: Optional[str] = None
    experts: Annotated[Optional[str], AfterValidator(_grouped_format)] = None
    latent: Optional[str] = None
    recurrence: Optional[str] = None
    recurrence_out: Optional[str] = None
    mtp: Optional[str] = None


class SwitchConfig(Config):
    type: Literal["switch"] = "switch"
    at: UnitOpen
    passes: tuple[Pass, ...] = ()


class PrecisionConfig(Config):
    type: Literal["precision"] = "precision"
    compute: Literal["float32", "bfloat16"] = "bfloat16"
    matmuls: str = "compute"
    roles: RolesConfig = RolesConfig()
    first: Branches = 0
    last: Branches = 0
    passes: tuple[Pass, ...] = PASSES
    switch: Optional[SwitchConfig] = None
    eval: Literal["train", "compute"] = "train"
    moments: Literal["float32", "bfloat16"] = "float32"
    reduce: Literal["compute", "float32"] = "compute"
    dispatch: Literal["compute", "mxfp8"] = "compute"

    def experts(self) -> Optional[str]:
        """Format of the routed experts' grouped GEMMs; None = the compute dtype."""
        if self.roles.experts is None and self.matmuls in GROUPED:
            return None if self.matmuls == "compute" else self.matmuls
        return self.roles.experts


# ---------------------------------------------------------------- how a run is split
Axis = Literal["data", "stage", "fsdp", "context", "expert", "tensor"]
Axes = Union[Axis, tuple[Axis, ...], None]


class MeshConfig(Config):
    """Device grid: one rank per GPU, axes in the fixed order
    (stage, data, fsdp, context, expert, tensor); ``data=None`` takes what is left."""

    type: Literal["mesh"] = "mesh"
    data: Optional[Positive] = None
    stage: Positive = 1
    fsdp: Positive = 1
    context: Positive = 1
    expert: Positive = 1
    tensor: Positive = 1


class LayoutConfig(Config):
    type: Literal["layout"] = "layout"
    batch: Axes = ("data", "fsdp", "expert")
    seq: Axes = "context"
    stream: Axes = "context"
    embed: Axes = None
    vocab: Axes = "tensor"
    heads: Axes = "tensor"
    kv_heads: Axes = "tensor"
    mlp: Axes = "tensor"
    experts: Axes = "expert"
    latent: Axes = None
    layers: Axes = None
    stages: Axes = "stage"
    fsdp: Axes = ("fsdp", "context", "expert")
    zero: Literal[1, 3] = 3


def _none_as_name(v):
    return "none" if v is None else v


Names = Annotated[tuple[str, ...], BeforeValidator(_as_tuple)]


class RematConfig(Config):
    type: Literal["remat"] = "remat"
    save: Names = ()
    offload: Names = ()
    first: Optional[Annotated[int, Field(ge=0)]] = None


class MethodsConfig(Config):
    """Which algorithm each communicating part uses. On B200 ``moe`` additionally
    takes ``fused_ep`` (in-kernel NVLink dispatch/combine) and ``tensor`` takes
    ``fused`` (all-gather→GEMM / GEMM→reduce-scatter kernels); the reference's
    names (``sorted``, ``all_to_all``, ``ragged_all_to_all``, ``nccl_ep``,
    ``gspmd``, ``chunked``) keep their meaning."""

    type: Literal["methods"] = "methods"
    attention: str = "auto"
    moe: str = "sorted"
    capacity: Optional[Annotated[float, Field(gt=0)]] = None
    moe_chunks: Positive = 1
    moe_stream: bool = False
    recurrence: str = "scan"
    states: Literal["keep", "recompute"] = "keep"
    repeat: str = "unroll"
    remat: Annotated[Union[str, RematConfig], BeforeValidator(_none_as_name)] = "auto"
    pipeline: str = "1f1b"
    rounds: Positive = 1
    stages: Optional[list[Positive]] = None
    orthogonalize: str = "owner"
    loss: str = "chunks"
    tensor: str = "gspmd"
    tensor_chunks: Positive = 2
    microbatches: Positive = 1
    interleave: bool = False
    gather: Literal["step", "layer"] = "step"
    accumulate: Literal["auto", "unreduced", "reduced"] = "auto"
    donate: bool = True


def _flag_syntax(options):
    for option in options.split():
        if "=" not in option:
            raise ValueError(f"an option is --name=value, not {option!r}")
    return options


class CompilerConfig(Config):
    """Kept for source compatibility. There is no tracing compiler here:
    ``preset`` selects CUDA-graph capture policy (``default`` = capture the step's
    launch-bound regions), ``reductions=early`` launches each layer's gradient
    reduction right after its weight-gradient kernel on a side stream."""

    type: Literal["compiler"] = "compiler"
    preset: str = "default"
    options: Annotated[str, AfterValidator(_flag_syntax)] = ""
    reductions: Literal["early", "xla"] = "early"


# ---------------------------------------------------------------- search
DIGITS = 3


def significant(x: float) -> float:
    return float(f"{x:.{DIGITS}g}")


class _Range(Config):
    @model_validator(mode="after")
    def _low_below_high(self):
        if not self.low < self.high:  # type: ignore[attr-defined]
            raise ValueError("low must be less than high")
        return self

    def _clip(self, x):
        return min(max(significant(x), self.low), self.high)  # type: ignore[attr-defined]


class UniformConfig(_Range):
    type: Literal["uniform"] = "uniform"
    low: float
    high: float

    def value(self, u):
        return self._clip(self.low + u * (self.high - self.low))

    def unit(self, x):
        return (x - self.low) / (self.high - self.low)


class LogUniformConfig(_Range):
    type: Literal["log_uniform"] = "log_uniform"
    low: Annotated[float, Field(gt=0)]
    high: float

    def value(self, u):
        return self._clip(self.low * (self.high / self.low) ** u)

    def unit(self, x):
        return math.log(x / self.low) / math.log(self.high / self.low)


class IntUniformConfig(_Range):
    type: Literal["int_uniform"] = "int_uniform"
    low: int
    high: int
    log: bool = False

    def _ends(self):
        if self.log:
            return math.log(self.low - 0.5), math.log(self.high + 0.5)
        return self.low - 0.5, self.high + 0.5

    def value(self, u):
        lo, hi = self._ends()
        x = lo + u * (hi - lo)
        x = math.exp(x) if self.log else x
        return min(max(round(x), self.low), self.high)

    def unit(self, x):
        lo, hi = self._ends()
        return ((math.log(x) if self.log else x) - lo) / (hi - lo)

    @model_validator(mode="after")
    def _log_positive(self):
        if self.log and self.low < 1:
            raise ValueError("int_uniform(log=true) needs low >= 1")
        return self


class ChoiceConfig(Config):
    type: Literal["choice"] = "choice"
    options: Annotated[tuple[str, ...], Field(min_length=2)]

    def value(self, u):
        return min(int(u * len(self.options)), len(self.options) - 1)

    def unit(self, x):
        return (x + 0.5) / len(self.options)


Distribution = Annotated[
    Union[UniformConfig, LogUniformConfig, IntUniformConfig, ChoiceConfig],
    Field(discriminator="type"),
]


class RandomSearch(Config):
    type: Literal["random"] = "random"


class HaltonSearch(Config):
    type: Literal["halton"] = "halton"


class SobolSearch(Config):
    type: Literal["sobol"] = "sobol"


class TPESearch(Config):
    type: Literal["tpe"] = "tpe"
    startup: Positive = 10
    candidates: Positive = 24
    gamma: UnitOpen = 0.1
    multivariate: bool = True


class GPSearch(Config):
    type: Literal["gp"] = "gp"
    startup: Positive = 5
    acquisition: Literal["log_ei", "ucb"] = "log_ei"
    beta: Annotated[float, Field(gt=0)] = 2.0


SearchMethod = Annotated[
    Union[RandomSearch, HaltonSearch, SobolSearch, TPESearch, GPSearch],
    Field(discriminator="type"),
]


class HalvingConfig(Config):
    type: Literal["halving"] = "halving"
    eta: Annotated[int, Field(ge=2)] = 3
    rungs: Annotated[int, Field(ge=2)] = 3
    brackets: Positive = 1

    @model_validator(mode="after")
    def _fits(self):
        if self.brackets > self.rungs:
            raise ValueError("halving needs brackets <= rungs")
        return self

    def steps(self, steps: int, rung: int) -> int:
        return max(1, round(steps / self.eta ** (self.rungs - 1 - rung)))


class SearchConfig(Config):
    type: Literal["search"] = "search"
    method: SearchMethod = GPSearch()
    trials: Positive = 16
    parallel: Optional[Positive] = None
    halving: Optional[HalvingConfig] = None
    seed: Annotated[int, Field(ge=0)] = 0


class Term(Config):
    metric: str
    weight: float


class ObjectiveConfig(Config):
    type: Literal["objective"] = "objective"
    terms: Annotated[tuple[Term, ...], Field(min_length=1)]
    constant: float = 0.0


# ---------------------------------------------------------------- the run
class TrainConfig(Config):
    data: DataConfig
    tokenizer: Optional[TokenizerConfig] = None
    packing: PackingConfig = BestFitPacking()
    optimizer: OptimizerConfig
    schedule: ScheduleConfig = ConstantSchedule()
    seq_len: Annotated[int, Field(ge=2)]
    batch: Positive
    batch_ramp: Optional[RampConfig] = None
    steps: Positive
    curriculum: Phases = ()
    seed: int = 0
    clip: Annotated[Optional[float], Field(gt=0)] = 1.0
    ema: Optional[EMAConfig] = None
    loss: LossConfig = LossConfig()
    eval: Evals = None
    checkpoint: Optional[CheckpointConfig] = None
    log: LogConfig = LogConfig()
    observe: Optional[ObserveConfig] = None
    profile: Optional[ProfileConfig] = None
    precision: PrecisionConfig = PrecisionConfig()
    mesh: MeshConfig = MeshConfig()
    layout: LayoutConfig = LayoutConfig()
    methods: MethodsConfig = MethodsConfig()
    compiler: CompilerConfig = CompilerConfig()
    objective: Optional[ObjectiveConfig] = None
    search: SearchConfig = SearchConfig()

    @model_validator(mode="after")
    def _prefix_needs_tokenizer(self):
        if self.loss.prefix is not None and self.tokenizer is None:
            raise ValueError(
                "loss(prefix=...) predicts each target's prefix token, by its bytes: "
                "it takes a tokenizer = tokenizer(...)"
            )
        return self


_SETTING_CLASSES = (
    TextConfig, ChatConfig, TokensConfig, SyntheticConfig, TokenizerConfig, ConcatPacking,
    GreedyPacking, BestFitPacking, AdamWConfig, MuonConfig, NorMuonConfig, EMAConfig,
    ConstantSchedule, CosineSchedule, WSDSchedule, LinearDecaySchedule, MultiStepSchedule,
    PowerSchedule, PiecewiseSchedule, Piece, PhaseConfig, RampConfig, LossConfig,
    PrefixConfig, EvalConfig, CheckpointConfig, LogConfig, WandbConfig, TensorBoardConfig,
    ObserveConfig, ProfileConfig, PrecisionConfig, RolesConfig, SwitchConfig, MeshConfig,
    LayoutConfig, RematConfig, MethodsConfig, CompilerConfig, UniformConfig,
    LogUniformConfig, IntUniformConfig, ChoiceConfig, RandomSearch, HaltonSearch,
    SobolSearch, TPESearch, GPSearch, HalvingConfig, SearchConfig,
)
TRAINING = tags_of(_SETTING_CLASSES)
DISTRIBUTIONS = tags_of((UniformConfig, LogUniformConfig, IntUniformConfig, ChoiceConfig))


def leaves(c) -> tuple:
    """The plain sources of `c`: a mixture's parts, or `c` itself."""
    return tuple(w.source for w in c.sources) if isinstance(c, MixtureConfig) else (c,)


def evals(t: TrainConfig) -> tuple:
    return _each(t.eval)


def evaluated(t: TrainConfig, e: EvalConfig) -> TrainConfig:
    shape = {k: getattr(e, k) for k in ("seq_len", "batch") if getattr(e, k) is not None}
    return t.model_copy(update=shape) if shape else t


def objective(t: TrainConfig) -> ObjectiveConfig:
    """The run's objective, defaulting to the first eval's loss/bpb or the loss."""
    if t.objective is not None:
        return t.objective
    first = next(iter(evals(t)), None)
    if first is None:
        metric = "loss"
    else:
        metric = f"{first.name}_{'bpb' if t.tokenizer is not None else 'loss'}"
    return ObjectiveConfig(terms=(Term(metric=metric, weight=1.0),))
