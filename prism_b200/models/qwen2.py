"""Qwen2 / Qwen2.5 dense decoder: its typed configuration, its layer plan and
its entry in the architecture registry.  Everything this engine knows about
the architecture by name is in this file.

What andre-fu/prism's executor computes (engine/executor.py:106-130) and
which tensors it reads (engine/weight_pool.py:156-199), written as data:
per layer a pre-norm block of RMSNorm, grouped-query attention with q/k/v
bias and rotary positions, RMSNorm, SwiGLU; then a final RMSNorm and a linear
head that shares the embedding when ``tie_word_embeddings`` is set.  The
configuration restates the keys and defaults the executor reads with
``getattr`` (engine/executor.py:34-48, engine/weight_pool.py:34-40) and the
validation rules of the upload path (engine/model_upload.py:93-107).
"""

from __future__ import annotations

from dataclasses import asdict, dataclass
from typing import Optional, Tuple

from ..config.model_config import ConfigError
from ..model_registry import register_architecture
from ..parts.base import PartSpec
from .decoder import ModelSpec

ARCHITECTURE = "Qwen2ForCausalLM"


@dataclass(frozen=True)
class Qwen2Config:
    """Keys of a Qwen2 / Qwen2.5 ``config.json``.

    Defaults follow the executor where it has one: ``rms_norm_eps`` 1e-6
    (engine/executor.py:43), ``rope_theta`` 10000.0 (executor.py:48),
    ``max_position_embeddings`` 4096 (executor.py:46, without its cap),
    ``num_key_value_heads`` = heads (engine/model_upload.py:97),
    ``tie_word_embeddings`` False (engine/weight_manager.py:84).
    ``head_dim`` defaults to ``hidden_size // num_attention_heads``
    (executor.py:37) and may be given explicitly.
    """

    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    max_position_embeddings: int = 4096
    tie_word_embeddings: bool = False
    attention_bias: bool = True
    hidden_act: str = "silu"
    use_sliding_window: bool = False
    sliding_window: Optional[int] = None
    max_window_layers: Optional[int] = None
    eos_token_id: Tuple[int, ...] = ()       # every id that ends a sequence (config.json gives one id or a list)
    bos_token_id: Optional[int] = None
    torch_dtype: str = "bfloat16"
    architectures: tuple = (ARCHITECTURE,)
    model_type: str = "qwen2"

    REQUIRED = ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                "num_attention_heads")

    # ---- derived sizes -------------------------------------------------
    @property
    def q_size(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_key_value_heads * self.head_dim

    def layer_window(self, layer: int) -> Optional[int]:
        """Sliding window of one layer (None: all keys).  With
        ``use_sliding_window`` the layers from ``max_window_layers`` on see
        the last ``sliding_window`` positions; the executor itself never
        reads these keys and always attends to everything."""
        if not self.use_sliding_window or self.sliding_window is None:
            return None
        first = self.max_window_layers if self.max_window_layers is not None else self.num_hidden_layers
        return int(self.sliding_window) if layer >= first else None

    # ---- construction ----------------------------------------------------
    @classmethod
    def from_dict(cls, raw: dict) -> "Qwen2Config":
        missing = [k for k in cls.REQUIRED if k not in raw]
        if missing:
            raise ConfigError(f"config.json missing required field(s): {', '.join(missing)}")
        nh = int(raw["num_attention_heads"])
        nkv = int(raw.get("num_key_value_heads") or nh)
        hs = int(raw["hidden_size"])
        if raw.get("head_dim"):
            hd = int(raw["head_dim"])
        else:
            if hs % nh != 0:
                raise ConfigError(f"hidden_size ({hs}) not divisible by num_attention_heads ({nh})")
            hd = hs // nh
        if nh <= 0 or nkv <= 0 or nh % nkv != 0:
            raise ConfigError(f"num_attention_heads ({nh}) not divisible by num_key_value_heads ({nkv})")
        if hd <= 0 or hd % 2 != 0:
            raise ConfigError(f"head_dim ({hd}) must be even for rotary pairs")
        if raw.get("rope_scaling") not in (None, {}):
            raise ConfigError("rope_scaling is set; scaled rotary embeddings are not computed by this engine")
        act = raw.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"hidden_act={act!r}; this architecture's feed-forward is SwiGLU with silu")
        usw = bool(raw.get("use_sliding_window", False))
        sw = raw.get("sliding_window")
        if usw and (sw is None or int(sw) <= 0):
            raise ConfigError("use_sliding_window is true but sliding_window is not a positive integer")
        for key in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers"):
            if int(raw[key]) <= 0:
                raise ConfigError(f"{key} must be positive, got {raw[key]}")
        eos = raw.get("eos_token_id")
        eos = () if eos is None else tuple(int(e) for e in (eos if isinstance(eos, (list, tuple)) else [eos]))
        archs = raw.get("architectures") or [ARCHITECTURE]
        return cls(
            vocab_size=int(raw["vocab_size"]), hidden_size=hs,
            intermediate_size=int(raw["intermediate_size"]),
            num_hidden_layers=int(raw["num_hidden_layers"]),
            num_attention_heads=nh, num_key_value_heads=nkv, head_dim=hd,
            rms_norm_eps=float(raw.get("rms_norm_eps", 1e-6)),
            rope_theta=float(raw.get("rope_theta", 10000.0)),
            max_position_embeddings=int(raw.get("max_position_embeddings", 4096)),
            tie_word_embeddings=bool(raw.get("tie_word_embeddings", False)),
            attention_bias=bool(raw.get("attention_bias", True)),
            hidden_act=act, use_sliding_window=usw,
            sliding_window=None if sw is None else int(sw),
            max_window_layers=None if raw.get("max_window_layers") is None else int(raw["max_window_layers"]),
            eos_token_id=eos, bos_token_id=raw.get("bos_token_id"),
            torch_dtype=str(raw.get("torch_dtype", "bfloat16")),
            architectures=tuple(archs), model_type=str(raw.get("model_type", "qwen2")),
        )

    def to_dict(self) -> dict:
        d = asdict(self)
        d["architectures"] = list(self.architectures)
        d["eos_token_id"] = list(self.eos_token_id) if len(self.eos_token_id) != 1 else self.eos_token_id[0]
        return d


def qwen2_spec(cfg: Qwen2Config) -> ModelSpec:
    H = cfg.hidden_size
    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        mixer = PartSpec("gqa_attention", dict(
            hidden_size=H, num_heads=cfg.num_attention_heads, num_kv_heads=cfg.num_key_value_heads,
            head_dim=cfg.head_dim, qkv_bias=cfg.attention_bias, o_bias=False,
            window=cfg.layer_window(i),
            position=PartSpec("rotary", dict(head_dim=cfg.head_dim, theta=cfg.rope_theta))),
            prefix=p + "self_attn.")
        ff = PartSpec("swiglu", dict(hidden_size=H, intermediate_size=cfg.intermediate_size), prefix=p + "mlp.")
        layers.append(PartSpec("prenorm", dict(
            mixer=mixer, feed_forward=ff,
            mixer_norm=PartSpec("rmsnorm", dict(width=H, eps=cfg.rms_norm_eps), prefix=p + "input_layernorm."),
            ff_norm=PartSpec("rmsnorm", dict(width=H, eps=cfg.rms_norm_eps), prefix=p + "post_attention_layernorm."))))
    return ModelSpec(
        architecture=ARCHITECTURE, hidden_size=H, vocab_size=cfg.vocab_size,
        max_positions=cfg.max_position_embeddings,
        embedding=PartSpec("token", dict(vocab_size=cfg.vocab_size, hidden_size=H), prefix="model."),
        layers=layers,
        final_norm=PartSpec("rmsnorm", dict(width=H, eps=cfg.rms_norm_eps), prefix="model.norm."),
        head=PartSpec("linear", dict(vocab_size=cfg.vocab_size, hidden_size=H,
                                     tied_to="embedding.weight" if cfg.tie_word_embeddings else None),
                      prefix="lm_head."),
        eos_token_id=cfg.eos_token_id)


register_architecture(ARCHITECTURE, Qwen2Config.from_dict, qwen2_spec)
