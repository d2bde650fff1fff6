"""Layer settings: one frozen pydantic model per layer a ``.bux`` file can call.

The field names and defaults are the public surface of the language (a run id is a
hash of their JSON dump), so they follow the reference schema field for field
(reference: ``src/bux/config.py``, classes at lines 33-1513). Everything else about
this file is this project's own: the models are declared compactly, validators are
small functions shared between classes, and `TAGS` gives the name → class tables
the compiler needs without introspecting unions.
"""

from __future__ import annotations

from typing import Annotated, ClassVar, Literal, Optional, Union

from pydantic import BaseModel, ConfigDict, Field, model_validator

Positive = Annotated[int, Field(gt=0)]
NonNeg = Annotated[int, Field(ge=0)]
PosFloat = Annotated[float, Field(gt=0)]

ACTIVATIONS = (
    "relu", "relu2", "gelu", "gelu_tanh", "swish", "sigmoid", "tanh", "softplus",
    "situ", "quick_gelu",
)
Activation = Literal[
    "relu", "relu2", "gelu", "gelu_tanh", "swish", "sigmoid", "tanh", "softplus",
    "situ", "quick_gelu",
]


class Config(BaseModel):
    """Base of every settings model: immutable, unknown keys rejected.

    `ports` names the internal tensors a layer can send or take through taps
    (``gqa(v=@v1)``).
    """

    model_config = ConfigDict(extra="forbid", frozen=True)
    ports: ClassVar[frozenset] = frozenset()


def _fail(condition: bool, message: str) -> None:
    if condition:
        raise ValueError(message)


# ---------------------------------------------------------------- norms / positions
class NormalizationConfig(Config):
    type: Literal["layernorm", "rmsnorm"]
    eps: float = 1e-6
    affine: bool = True
    bias: bool = False
    zero_centered: bool = False
    gain_init: float = 1.0
    scale_input: bool = False


class DyTConfig(Config):
    type: Literal["dyt"] = "dyt"
    alpha_init: float = 0.5


class PositionInterpolationConfig(Config):
    type: Literal["pi"] = "pi"
    factor: float


class YaRNConfig(Config):
    type: Literal["yarn"] = "yarn"
    factor: float
    original_max_len: int
    beta_fast: float = 32.0
    beta_slow: float = 1.0
    attention_factor: Optional[float] = None
    attention_factor_on: Literal["rotary", "softmax"] = "rotary"


class Llama3RoPEScalingConfig(Config):
    type: Literal["llama3"] = "llama3"
    factor: float
    original_max_len: int = 8192
    low_freq_factor: float = 1.0
    high_freq_factor: float = 4.0


RoPEScalingConfig = Annotated[
    Union[PositionInterpolationConfig, YaRNConfig, Llama3RoPEScalingConfig],
    Field(discriminator="type"),
]


class RoPEConfig(Config):
    type: Literal["rope"] = "rope"
    base: float = 10000.0
    fraction: float = 1.0
    layout: Literal["half", "interleaved"] = "half"
    scaling: Optional[RoPEScalingConfig] = None


class RelativeBiasConfig(Config):
    type: Literal["relbias"] = "relbias"
    rank: int = 16
    extent: int = 1024


# ---------------------------------------------------------------- feed-forward
class MLPConfig(Config):
    type: Literal["mlp", "gated_mlp"]
    intermediate_size: int
    activation: Activation
    dropout: float = 0.0
    bias: bool = False
    limit: Optional[float] = None
    up_softcap: Optional[float] = None
    up_offset: float = 0.0


class MoEConfig(Config):
    type: Literal["moe"] = "moe"
    num_experts: int
    top_k: int
    expert: MLPConfig
    num_shared_experts: int = 0
    shared_expert: Optional[MLPConfig] = None
    shared_expert_gate: bool = False
    router: Literal["softmax", "sigmoid", "sqrtsoftplus"] = "softmax"
    router_bias: bool = False
    router_logit_scale: float = 1.0
    random_logits: bool = False
    normalize_top_k: bool = True
    routed_scaling_factor: float = 1.0
    num_groups: Positive = 1
    top_k_groups: Positive = 1
    load_balancing: Literal["aux_loss", "aux_free", "smebu"] = "aux_loss"
    bias_update_rate: Annotated[float, Field(ge=0)] = 1e-3
    center_bias: bool = False
    bias_softclamp: PosFloat = 2.0
    bias_momentum: Annotated[float, Field(ge=0, lt=1)] = 0.5
    aux_loss_coef: Optional[Annotated[float, Field(ge=0)]] = None
    aux_loss_scope: Literal["batch", "sequence"] = "batch"
    latent_size: Optional[int] = None
    latent_input_norm: Optional[NormalizationConfig] = None
    latent_output_norm: Optional[NormalizationConfig] = None
    expert_norm: Optional[NormalizationConfig] = None
    shared_expert_sink: bool = False
    num_zero_experts: NonNeg = 0
    ffn_experts_per_token: Optional[float] = None

    @property
    def ffn_budget(self) -> float:
        """Routed (non-zero) experts a token is expected to pass through."""
        if self.ffn_experts_per_token is not None:
            return self.ffn_experts_per_token
        return self.top_k * self.num_experts / (self.num_experts + self.num_zero_experts)

    @property
    def aux_loss_weight(self) -> float:
        if self.aux_loss_coef is not None:
            return self.aux_loss_coef
        return 1e-2 if self.load_balancing == "aux_loss" else 0.0

    @model_validator(mode="after")
    def _consistent(self):
        n, g, picked = self.num_experts, self.num_groups, self.top_k_groups
        scored = n + self.num_zero_experts
        _fail(
            n % g != 0 or picked > g or self.top_k > picked * (scored // g),
            f"{g} groups of {n} experts, {picked} of them picked, cannot hold "
            f"the top {self.top_k}",
        )
        shared_only = [
            k for k, on in (
                ("shared_expert", self.shared_expert is not None),
                ("shared_expert_gate", self.shared_expert_gate),
                ("shared_expert_sink", self.shared_expert_sink),
            ) if on
        ]
        _fail(
            bool(shared_only) and not self.num_shared_experts,
            f"{', '.join(shared_only)} set the shared experts, of which there are "
            "none: set num_shared_experts",
        )
        if not self.num_zero_experts:
            _fail(self.ffn_experts_per_token is not None,
                  "ffn_experts_per_token needs num_zero_experts")
            return self
        _fail(not 0 < self.ffn_budget < self.top_k,
              f"ffn_experts_per_token={self.ffn_budget} is not between 0 and "
              f"top_k={self.top_k}")
        refused = [
            k for k, on in (
                ("load_balancing=smebu", self.load_balancing == "smebu"),
                ("center_bias", self.center_bias),
                ("num_groups", self.num_groups > 1),
            ) if on
        ]
        _fail(bool(refused),
              f"num_zero_experts with {', '.join(refused)}: the zero experts' bias "
              "stays 0, which centering would move, and they are in no group")
        return self


# ---------------------------------------------------------------- attention
class AttentionConfig(Config):
    """Common base of every token mixer."""


class SparseIndexerConfig(Config):
    type: Literal["indexer"] = "indexer"
    num_heads: int = 64
    head_dim: int = 128
    top_k: int = 2048
    block_size: int = 1
    pool: Literal["mean", "max"] = "mean"
    per_group: bool = False
    relu: bool = True
    weighted: bool = True
    norm: Optional[NormalizationConfig] = None
    rope_layout: Literal["half", "interleaved"] = "half"
    candidate_block_size: int = 8
    candidate_top_k: int = 2048
    loss_weight: Annotated[float, Field(ge=0)] = 1.0
    loss_over: Literal["own", "served"] = "own"

    @model_validator(mode="after")
    def _selection(self):
        blocks = self.block_size > 1
        _fail(self.per_group and self.weighted,
              "indexer(per_group=true) scores each group by its own head, which no "
              "weight sums with others: set weighted=false")
        _fail(self.per_group and blocks and self.pool == "mean",
              "indexer(per_group=true) with blocks takes pool=max: QSA's mean-pooled "
              "blocks are one pick for all heads")
        _fail(self.loss_over == "served" and (self.per_group or blocks),
              "indexer(loss_over=served) distills one pick of single keys for all "
              "heads: set block_size=1 and per_group=false")
        _fail(blocks and self.top_k < self.block_size,
              f"indexer keeps top_k // block_size blocks: top_k={self.top_k} is less "
              f"than one block of {self.block_size}")
        return self


class QuadraticAttentionConfig(AttentionConfig):
    sliding_window_size: Optional[int] = None
    attention_dropout: float = 0.0
    output_dropout: float = 0.0
    gated: bool = False
    gate_per_head: bool = False
    gate_activation: Activation = "sigmoid"
    gate_head_bias: bool = False
    gate_input_rank: Optional[int] = None
    gate_output_rank: Optional[int] = None
    gate_cross_head: bool = False
    output_norm: Optional[NormalizationConfig] = None
    qk_norm: Optional[NormalizationConfig] = None
    softcap: Optional[float] = None
    sinks: bool = False
    scale: Optional[float] = None
    log_scale: Optional[float] = None
    log_scale_floor: int = 8192
    relative_bias: Optional[RelativeBiasConfig] = None
    indexer: Optional[SparseIndexerConfig] = None

    @model_validator(mode="after")
    def _gate(self):
        given = [
            k for k, on in (
                ("gate_per_head", self.gate_per_head),
                ("gate_head_bias", self.gate_head_bias),
                ("gate_activation", self.gate_activation != "sigmoid"),
                ("gate_input_rank", self.gate_input_rank is not None),
                ("gate_output_rank", self.gate_output_rank is not None),
                ("gate_cross_head", self.gate_cross_head),
            ) if on
        ]
        _fail(bool(given) and not self.gated,
              f"{', '.join(given)} set the gate, which gated=true adds")
        ranks = self.gate_input_rank is not None or self.gate_output_rank is not None
        _fail(ranks and self.gate_per_head,
              "gate_input_rank and gate_output_rank gate each dim of a head: not with "
              "gate_per_head")
        if self.indexer is not None and self.indexer.per_group:
            kv = getattr(self, "num_kv_heads", None)
            _fail(kv is None,
                  "indexer(per_group=true) picks for each kv head's group of query "
                  "heads, which gqa has alone")
            _fail(self.indexer.num_heads != kv,
                  f"indexer(per_group=true) has a head for each of the layer's {kv} kv "
                  f"heads: num_heads={self.indexer.num_heads} is not {kv}")
        return self


class GQAConfig(QuadraticAttentionConfig):
    ports: ClassVar[frozenset] = frozenset({"v", "kv", "index", "ve"})
    type: Literal["gqa"] = "gqa"
    num_heads: int
    num_kv_heads: int
    head_dim: Optional[int] = None
    v_head_dim: Optional[int] = None
    bias: bool = False
    output_bias: Optional[bool] = None
    fused_qkv: bool = False
    qk_norm_all_heads: bool = False
    rope: Optional[RoPEConfig] = None
    power_scale: Optional[float] = None
    power_scale_length: int = 2048
    kv_conv_size: Optional[int] = None
    value_residual: Literal["fixed", "learned", "convex"] = "fixed"
    exclusive: Union[bool, Literal["learned"]] = False
    value_embed_gate: Optional[Positive] = 6
    k_eq_v: bool = False
    differential: bool = False
    paired: bool = False
    mimetic_vo: Optional[PosFloat] = None
    mimetic_noise: float = 0.01

    @model_validator(mode="after")
    def _heads(self):
        _fail(self.num_kv_heads < 1 or self.num_heads % self.num_kv_heads != 0,
              f"{self.num_kv_heads} key and value heads do not divide "
              f"{self.num_heads} query heads")
        _fail(self.k_eq_v and self.v_head_dim not in (None, self.head_dim),
              "gqa(k_eq_v=true) makes the values from the keys, so v_head_dim is "
              f"head_dim: give no v_head_dim (got {self.v_head_dim})")
        clash = [k for k, v in (("indexer", self.indexer),
                                ("relative_bias", self.relative_bias)) if v is not None]
        _fail(self.differential and bool(clash),
              f"gqa: differential with {', '.join(clash)} not yet")
        if self.paired:
            _fail(self.num_heads % 2 != 0 or self.num_kv_heads % 2 != 0,
                  "gqa: paired takes an even number of heads and kv heads, not "
                  f"{self.num_heads} and {self.num_kv_heads}")
            clash = [
                k for k, on in (
                    ("indexer", self.indexer is not None),
                    ("relative_bias", self.relative_bias is not None),
                    ("log_scale", self.log_scale is not None),
                    ("attention_dropout", self.attention_dropout > 0),
                    ("sinks", self.sinks),
                    ("differential", self.differential),
                    ("exclusive", bool(self.exclusive)),
                ) if on
            ]
            _fail(bool(clash), f"gqa: paired with {', '.join(clash)} not yet")
        _fail(self.mimetic_noise != 0.01 and self.mimetic_vo is None,
              "mimetic_noise sets the init that mimetic_vo adds")
        _fail(self.mimetic_vo is not None and self.k_eq_v,
              "gqa: mimetic_vo starts the v projection, which k_eq_v has not")
        return self


class MLAConfig(QuadraticAttentionConfig):
    ports: ClassVar[frozenset] = frozenset({"index"})
    type: Literal["mla"] = "mla"
    num_heads: int
    q_lora_rank: Optional[int] = None
    kv_lora_rank: int = 512
    qk_nope_head_dim: int = 128
    qk_rope_head_dim: int = 64
    v_head_dim: int = 128
    rope: Optional[RoPEConfig] = RoPEConfig()


class CSAConfig(QuadraticAttentionConfig):
    ports: ClassVar[frozenset] = frozenset({"kv", "index", "candidates"})
    type: Literal["csa"] = "csa"
    num_heads: int
    head_dim: int = 512
    q_lora_rank: Optional[int] = None
    o_lora_rank: Optional[int] = None
    o_groups: int = 1
    compress_ratio: Optional[int] = None
    rope: Optional[RoPEConfig] = RoPEConfig()
    latent_norm: NormalizationConfig = NormalizationConfig(type="rmsnorm")


Gate = Optional[Literal["swish", "sigmoid"]]


class LinearAttentionConfig(AttentionConfig):
    num_heads: int
    head_dim: int
    num_v_heads: Optional[int] = None
    v_head_dim: Optional[int] = None
    conv_size: Optional[int] = 4
    output_gate: Gate = "swish"
    norm_eps: float = 1e-6


class GLAConfig(LinearAttentionConfig):
    type: Literal["gla"] = "gla"
    gate_rank: int = 16
    conv_size: Optional[int] = None


class DeltaNetConfig(LinearAttentionConfig):
    type: Literal["deltanet"] = "deltanet"


class GatedDeltaNetConfig(LinearAttentionConfig):
    type: Literal["gdn"] = "gdn"


class KDAConfig(LinearAttentionConfig):
    type: Literal["kda"] = "kda"
    gate_rank: Optional[int] = None
    output_gate: Gate = "sigmoid"
    output_gate_rank: Optional[int] = None
    gate_lower_bound: Optional[float] = None


class GatedDeltaNet2Config(LinearAttentionConfig):
    type: Literal["gdn2"] = "gdn2"
    gate_rank: Optional[int] = None
    output_gate_rank: Optional[int] = None
    norm_eps: float = 1e-5
    negative_eigenvalues: bool = False
    gate_lower_bound: Optional[float] = None


class LightningAttentionConfig(LinearAttentionConfig):
    type: Literal["lightning"] = "lightning"
    conv_size: Optional[int] = None
    output_gate: Gate = "sigmoid"


class RWKV7Config(LinearAttentionConfig):
    ports: ClassVar[frozenset] = frozenset({"v"})
    type: Literal["rwkv7"] = "rwkv7"
    conv_size: Optional[int] = None
    output_gate: Gate = "sigmoid"
    norm_eps: float = 1e-5
    decay_rank: int = 64
    a_rank: int = 64
    v_rank: int = 32
    gate_rank: int = 128


class StateSpaceConfig(AttentionConfig):
    state_size: int
    expand: int = 2
    conv_size: Positive = 4
    dt_min: float = 1e-3
    dt_max: float = 1e-1


class MambaConfig(StateSpaceConfig):
    type: Literal["mamba"] = "mamba"
    state_size: int = 16
    dt_rank: Optional[int] = None


class Mamba2Config(StateSpaceConfig):
    type: Literal["mamba2"] = "mamba2"
    state_size: int = 128
    head_dim: int = 64
    num_heads: Optional[int] = None
    num_groups: int = 1


class ConvConfig(AttentionConfig):
    type: Literal["conv"] = "conv"
    size: Positive = 4
    bias: bool = False


class ShortConvConfig(AttentionConfig):
    type: Literal["short_conv"] = "short_conv"
    conv_size: Positive = 3
    bias: bool = False


# ---------------------------------------------------------------- small layers
class LinearConfig(Config):
    type: Literal["linear"] = "linear"
    features: int
    bias: bool = False


class ActivationConfig(Config):
    type: Literal["act"] = "act"
    fn: Activation


class ScaleConfig(Config):
    type: Literal["scale"] = "scale"
    init: float = 1.0
    per_channel: bool = False


class DropoutConfig(Config):
    type: Literal["dropout"] = "dropout"
    rate: float


class EmbeddingConfig(Config):
    type: Literal["embed"] = "embed"
    max_positions: Optional[int] = None
    scale_by_sqrt_dim: bool = False
    norm: Optional[NormalizationConfig] = None
    dropout: float = 0.0


class ValueEmbeddingConfig(Config):
    ports: ClassVar[frozenset] = frozenset({"ve"})
    type: Literal["value_embed"] = "value_embed"
    features: Positive
    std: float = 0.01


class CopyPointerConfig(Config):
    type: Literal["copy_pointer"] = "copy_pointer"
    dim: Positive = 128
    token: Optional[NonNeg] = None
    window: Optional[Positive] = None


class LMHeadConfig(Config):
    type: Literal["head"] = "head"
    tied: bool = False
    bias: bool = False
    softcap: Optional[float] = None
    pointer: Optional[CopyPointerConfig] = None


class NextNConfig(Config):
    type: Literal["nextn"] = "nextn"
    norm: NormalizationConfig = NormalizationConfig(type="rmsnorm")


class EngramConfig(Config):
    type: Literal["engram"] = "engram"
    head_dim: int
    table_size: int
    max_ngram_size: Annotated[int, Field(ge=2)] = 3
    num_heads: int = 8
    norm: NormalizationConfig = NormalizationConfig(type="rmsnorm")
    conv_size: Optional[int] = 4
    vocab_classes: Optional[int] = None
    boundary_token: Optional[int] = None


class DocCopyConfig(Config):
    ports: ClassVar[frozenset] = frozenset({"copy"})
    type: Literal["doc_copy"] = "doc_copy"
    gain: float = 0.5
    lengths: tuple[Positive, ...] = (1, 2, 3, 4, 6, 8, 12, 16, 24, 32)
    counts: Positive = 3


# ---------------------------------------------------------------- init
INIT_ROLES = ("embed", "head", "out")


class InitConfig(Config):
    embed: Optional["Init"] = None
    head: Optional["Init"] = None
    out: Optional["Init"] = None

    @model_validator(mode="after")
    def _flat_roles(self):
        for role in INIT_ROLES:
            sub = getattr(self, role)
            _fail(sub is not None and any(getattr(sub, r) is not None for r in INIT_ROLES),
                  f"the init of '{role}' sets roles of its own; set them all on "
                  "the model's init")
        return self


class NormalInitConfig(InitConfig):
    type: Literal["normal"] = "normal"
    std: PosFloat = 0.02
    truncate: Optional[PosFloat] = None


class FanInitConfig(InitConfig):
    type: Literal["fan_in", "fan_out", "fan_avg"]
    scale: PosFloat = 1.0
    distribution: Literal["truncated", "gaussian", "uniform"] = "truncated"


class ZerosInitConfig(InitConfig):
    type: Literal["zeros"] = "zeros"


Init = Annotated[
    Union[NormalInitConfig, FanInitConfig, ZerosInitConfig], Field(discriminator="type")
]
for _c in (InitConfig, NormalInitConfig, FanInitConfig, ZerosInitConfig):
    _c.model_rebuild()


# ---------------------------------------------------------------- residual algebras
class HyperConnectionsConfig(Config):
    type: Literal["hc", "mhc"]
    expansion: Annotated[int, Field(ge=2)] = 4
    dynamic: bool = True
    sinkhorn_iters: Positive = 20
    pre_bias: float = 1.0
    post_bias: float = 1.0
    res_bias: float = -8.0
    single_pass: bool = False
    norm_eps: float = 1e-6


class GatedResidualConfig(Config):
    type: Literal["gr"] = "gr"
    rank: Positive
    expansion: Positive = 4
    norm_eps: float = 1e-6


class AttentionResidualConfig(Config):
    type: Literal["attnres"] = "attnres"
    block_size: Optional[Positive] = None
    norm_eps: float = 1e-6


class MultiStreamAttentionResidualConfig(Config):
    type: Literal["msar"] = "msar"
    block_size: Optional[Positive] = None
    kernel_sizes: tuple[Positive, ...] = (4, 8, 12)
    norm_eps: float = 1e-6


class ResidualGateConfig(Config):
    type: Literal["vpgate"] = "vpgate"
    temperature: PosFloat = 0.3
    eps: PosFloat = 1e-3


class MergeConfig(Config):
    type: Literal["merge"] = "merge"


ResidualConfig = Annotated[
    Union[
        HyperConnectionsConfig, GatedResidualConfig, AttentionResidualConfig,
        MultiStreamAttentionResidualConfig, ResidualGateConfig,
    ],
    Field(discriminator="type"),
]

_LAYER_CLASSES = (
    NormalizationConfig, DyTConfig, MLPConfig, MoEConfig, GQAConfig, MLAConfig, CSAConfig,
    GLAConfig, DeltaNetConfig, GatedDeltaNetConfig, KDAConfig, GatedDeltaNet2Config,
    LightningAttentionConfig, RWKV7Config, MambaConfig, Mamba2Config, ConvConfig,
    ShortConvConfig, LinearConfig, ActivationConfig, ScaleConfig, DropoutConfig,
    EmbeddingConfig, ValueEmbeddingConfig, LMHeadConfig, NextNConfig, EngramConfig,
    DocCopyConfig, MergeConfig,
)
LayerConfig = Annotated[Union[_LAYER_CLASSES], Field(discriminator="type")]  # type: ignore[valid-type]

_SUB_CLASSES = (
    RoPEConfig, PositionInterpolationConfig, YaRNConfig, Llama3RoPEScalingConfig,
    RelativeBiasConfig, CopyPointerConfig, SparseIndexerConfig, HyperConnectionsConfig,
    GatedResidualConfig, AttentionResidualConfig, MultiStreamAttentionResidualConfig,
    ResidualGateConfig, NormalInitConfig, FanInitConfig, ZerosInitConfig,
)


def tags_of(classes) -> dict:
    """Map every ``type`` tag of `classes` to its class (a class may own several)."""
    from typing import get_args

    table = {}
    for cls in classes:
        for tag in get_args(cls.model_fields["type"].annotation):
            table[tag] = cls
    return table


LAYERS = tags_of(_LAYER_CLASSES)
SUBCONFIGS = tags_of(_SUB_CLASSES)
RESIDUALS = tags_of((HyperConnectionsConfig, GatedResidualConfig, AttentionResidualConfig,
                     MultiStreamAttentionResidualConfig, ResidualGateConfig))
INITS = tags_of((NormalInitConfig, FanInitConfig, ZerosInitConfig))
