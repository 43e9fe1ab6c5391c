"""`params.json` schema (mirror of mistral_inference/args.py:29-59 and moe.py:10-13).

`simple_parsing` is not a dependency here: `from_dict` is a few lines (the reference only uses
`Serializable.from_dict`, transformer.py:306-307).
"""
from dataclasses import dataclass, fields
from typing import List, Optional, Union


@dataclass
class MoeArgs:
    num_experts: int
    num_experts_per_tok: int

    @classmethod
    def from_dict(cls, d: dict) -> "MoeArgs":
        return cls(**{f.name: d[f.name] for f in fields(cls) if f.name in d})


@dataclass
class LoraArgs:
    rank: int
    scaling: float

    @classmethod
    def from_dict(cls, d: dict) -> "LoraArgs":
        return cls(**{f.name: d[f.name] for f in fields(cls) if f.name in d})


@dataclass
class TransformerArgs:
    dim: int
    n_layers: int
    head_dim: int
    hidden_dim: int
    n_heads: int
    n_kv_heads: int
    norm_eps: float
    vocab_size: int

    max_batch_size: int = 0

    # For rotary embeddings. If not set, 1e6 is used (transformer.py:115).
    rope_theta: Optional[float] = None
    # If this is set, MoE layers replace the dense FeedForward.
    moe: Optional[MoeArgs] = None
    lora: Optional[LoraArgs] = None
    sliding_window: Union[None, int, List[Optional[int]]] = None
    _sliding_window: Union[None, int, List[Optional[int]]] = None
    model_type: str = "transformer"

    vision_encoder: Optional[dict] = None

    def __post_init__(self) -> None:
        assert self.model_type == "transformer", self.model_type
        assert self.sliding_window is None or self._sliding_window is None
        # same aliasing as args.py:58-59
        self.sliding_window = self.sliding_window if self.sliding_window is not None else self._sliding_window
        if self.vision_encoder is not None:
            raise NotImplementedError("vision_encoder (Pixtral) is outside the accelerated hot path (SURVEY.md 2, row 10)")
        if isinstance(self.moe, dict):
            self.moe = MoeArgs.from_dict(self.moe)
        if isinstance(self.lora, dict):
            self.lora = LoraArgs.from_dict(self.lora)

    @classmethod
    def from_dict(cls, d: dict) -> "TransformerArgs":
        known = {f.name for f in fields(cls)}
        return cls(**{k: v for k, v in d.items() if k in known})


# ----------------------------------------------------------------------------- layered decoders (config.json)
@dataclass
class BiasedAttentionArgs:
    """Softmax attention without rotation: per-head RMS norm of q and k, a query temperature that grows with the position,
    a learned additive bias by (bucketed) distance, optional mixing of the values with an earlier layer's."""
    heads: int
    kv_heads: int
    dim: int            # per-head query/key size
    vdim: int           # per-head value size
    scale: float        # multiplies q.k (not the bias)
    bias_max: float     # distance at which the logarithmic part of the bias buckets ends
    temp_coef: float = 0.0
    temp_every: int = 0  # 0: no temperature
    v_mix: bool = False

    @classmethod
    def from_dict(cls, d: dict) -> "BiasedAttentionArgs":
        qt = d.get("q_temp") or {}
        return cls(heads=int(d["heads"]), kv_heads=int(d["kv_heads"]), dim=int(d["dim"]), vdim=int(d["vdim"]), scale=float(d["scale"]),
                   bias_max=float(d["bias_max"]), temp_coef=float(qt.get("coef", 0.0)), temp_every=int(qt.get("every", 0)),
                   v_mix=bool(d.get("v_mix", False)))


@dataclass
class LightningArgs:
    """Linear attention with one fixed decay per head and an fp32 state [heads, dim, vdim] per sequence."""
    heads: int
    dim: int
    vdim: int
    decay: List[float]

    @classmethod
    def from_dict(cls, d: dict) -> "LightningArgs":
        a = cls(heads=int(d["heads"]), dim=int(d["dim"]), vdim=int(d["vdim"]), decay=[float(x) for x in d["decay"]])
        assert len(a.decay) == a.heads, "one decay per head"
        return a


@dataclass
class ClampedGluArgs:
    """Dense feed-forward y = g * sigmoid(alpha * g) * (u + 1) with g = min(gate, limit), u = clamp(up, -limit, limit)."""
    ff: int
    limit: float
    alpha: float = 1.702

    @classmethod
    def from_dict(cls, d: dict) -> "ClampedGluArgs":
        assert d.get("kind", "dense") == "dense", f"unknown feed-forward kind {d.get('kind')}"
        return cls(ff=int(d["ff"]), limit=float(d["limit"]))


@dataclass
class LayerArgs:
    type: str                                             # "attention" | "lightning"
    mixer: Union[BiasedAttentionArgs, LightningArgs]
    mlp: Optional[ClampedGluArgs]


MIXER_ARGS = {"attention": BiasedAttentionArgs, "lightning": LightningArgs}


@dataclass
class LayeredArgs:
    """config.json of a layered decoder (architecture "Fesenex"): a list of layers, each naming its mixer kind."""
    architecture: str
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    layers: List[LayerArgs]
    max_batch_size: int = 0

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @classmethod
    def from_dict(cls, d: dict) -> "LayeredArgs":
        layers = []
        for L in d["layers"]:
            if L["type"] not in MIXER_ARGS:
                raise ValueError(f"unknown mixer type {L['type']!r}")
            layers.append(LayerArgs(type=L["type"], mixer=MIXER_ARGS[L["type"]].from_dict(L["mixer"]),
                                    mlp=ClampedGluArgs.from_dict(L["mlp"]) if L.get("mlp") is not None else None))
        return cls(architecture=d["architecture"], vocab=int(d["vocab"]), width=int(d["width"]),
                   embedding_scale=float(d["embedding"]["scale"]), norm_eps=float(d["norm"]["eps"]), layers=layers)
