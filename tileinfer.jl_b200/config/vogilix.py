"""Typed configuration of the Vogilix design and its lowering to per-layer records.

A Vogilix model is a decoder whose config.json lists its layers one by one (``layers``: ``type``, ``mixer``,
``mlp``), so every layer may have sizes of its own. What the design fixes lives here and in the parts; what
config.json gives is read from it and nowhere else:

* the stream starts as token embedding + a learned position vector and is kept in 32-bit;
* a layer normalises the OUTPUT of each sublayer (an RMS norm whose gain is 1 + the stored weight) and adds it,
  times ``residual_mult``, to the stream; the sublayers read the stream itself;
* mixer ``latent_attention``: queries and keys/values through low-rank latents, no positions inside, a
  sliding window of ``mask.size`` keys, only the key/value latent cached;
* feed-forward ``dense`` (up, exact GELU, down) or ``moe`` (sigmoid router, ``top`` experts whose score scales
  their INPUT, an always-on shared expert; experts are clamped gated units), or none;
* with ``token_side`` every layer ends by adding a gated, normalised projection of a per-token vector.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from .apertus import ConfigError, _require
from .spec import FeedForwardSpec, LayerSpec, MixerSpec, ModelSpec, NormSpec, TokenInputSpec

# Constants of the design's expert unit: y = g * sigmoid(SIGMOID_SLOPE * g) * (u + UP_SHIFT).
EXPERT_SIGMOID_SLOPE = 1.702
EXPERT_UP_SHIFT = 1.0


@dataclass(frozen=True)
class LatentMixerConfig:
    heads: int
    dim: int                       # query/key size of a head
    vdim: int                      # value size of a head
    q_rank: int
    kv_rank: int
    scale: float
    window: Optional[int]          # mask.size; None: every earlier position is visible

    @classmethod
    def from_dict(cls, m: Mapping[str, Any], where: str) -> "LatentMixerConfig":
        get = lambda k: _need(m, k, where)
        mask = m.get("mask")
        window = None if not mask else int(_need(mask, "size", where + ".mask"))
        out = cls(int(get("heads")), int(get("dim")), int(get("vdim")), int(get("q_rank")), int(get("kv_rank")),
                  float(get("scale")), window)
        for name in ("heads", "dim", "vdim", "q_rank", "kv_rank"):
            if getattr(out, name) < 1:
                raise ConfigError(f"{where}.{name} must be positive")
        if window is not None and window < 1:
            raise ConfigError(f"{where}.mask.size must be positive")
        return out

    def to_dict(self) -> dict:
        d = {"dim": self.dim, "heads": self.heads, "kv_rank": self.kv_rank, "q_rank": self.q_rank, "scale": self.scale,
             "vdim": self.vdim}
        if self.window is not None:
            d["mask"] = {"size": self.window}
        return d


@dataclass(frozen=True)
class ExpertConfig:
    ff: int
    limit: float


@dataclass(frozen=True)
class MlpConfig:
    kind: str                      # "dense" | "moe"
    ff: int = 0                    # dense
    experts: int = 0               # moe
    top: int = 0
    expert: Optional[ExpertConfig] = None
    shared: Optional[ExpertConfig] = None

    @classmethod
    def from_dict(cls, m: Mapping[str, Any], where: str) -> "MlpConfig":
        kind = _need(m, "kind", where)
        if kind == "dense":
            return cls("dense", ff=int(_need(m, "ff", where)))
        if kind == "moe":
            r = _need(m, "router", where)
            e = _need(m, "expert", where)
            s = m.get("shared")
            out = cls("moe", experts=int(_need(r, "experts", where + ".router")), top=int(_need(r, "top", where + ".router")),
                      expert=ExpertConfig(int(_need(e, "ff", where + ".expert")), float(_need(e, "limit", where + ".expert"))),
                      shared=None if not s else ExpertConfig(int(_need(s, "ff", where + ".shared")),
                                                             float(_need(s, "limit", where + ".shared"))))
            if not 1 <= out.top <= out.experts:
                raise ConfigError(f"{where}.router: top {out.top} of {out.experts} experts")
            return out
        raise ConfigError(f"{where}.kind \"{kind}\" is not a feed-forward of this design (dense, moe)")

    def to_dict(self) -> dict:
        if self.kind == "dense":
            return {"ff": self.ff, "kind": "dense"}
        d = {"expert": {"ff": self.expert.ff, "limit": self.expert.limit}, "kind": "moe",
             "router": {"experts": self.experts, "top": self.top}}
        if self.shared is not None:
            d["shared"] = {"ff": self.shared.ff, "limit": self.shared.limit}
        return d


@dataclass(frozen=True)
class VogilixLayerConfig:
    type: str
    mixer: LatentMixerConfig
    mlp: Optional[MlpConfig]


def _need(m: Mapping[str, Any], key: str, where: str):
    if not isinstance(m, Mapping) or key not in m or m[key] is None:
        raise ConfigError(f"config.json: {where} has no \"{key}\"")
    return m[key]


@dataclass(frozen=True)
class VogilixConfig:
    vocab: int
    width: int
    max_positions: int
    norm_eps: float
    residual_mult: float
    token_side_dim: Optional[int]
    layers: Tuple[VogilixLayerConfig, ...]
    eos_token_ids: Tuple[int, ...] = ()

    architecture = "Vogilix"
    model_type = "vogilix"

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @classmethod
    def from_dict(cls, c: Mapping[str, Any]) -> "VogilixConfig":
        layers = []
        for i, l in enumerate(_require(c, "layers")):
            where = f"layers[{i}]"
            kind = _need(l, "type", where)
            if kind != "latent_attention":
                raise ConfigError(f"{where}.type \"{kind}\" is not a mixer of this design (latent_attention)")
            mlp = l.get("mlp")
            layers.append(VogilixLayerConfig(kind, LatentMixerConfig.from_dict(_need(l, "mixer", where), where + ".mixer"),
                                             None if mlp is None else MlpConfig.from_dict(mlp, where + ".mlp")))
        side = c.get("token_side")
        eos = c.get("eos_token_id", ())
        eos = (eos,) if isinstance(eos, int) else tuple(eos or ())
        out = cls(vocab=int(_require(c, "vocab")), width=int(_require(c, "width")), max_positions=int(_require(c, "max_positions")),
                  norm_eps=float(_need(_require(c, "norm"), "eps", "norm")), residual_mult=float(c.get("residual_mult", 1.0)),
                  token_side_dim=None if not side else int(_need(side, "dim", "token_side")), layers=tuple(layers),
                  eos_token_ids=eos)
        if out.vocab < 1 or out.width < 1 or out.max_positions < 1:
            raise ConfigError("vocab, width and max_positions must be positive")
        return out

    def to_dict(self) -> dict:
        d = {"architecture": self.architecture,
             "layers": [{"mixer": l.mixer.to_dict(), "mlp": None if l.mlp is None else l.mlp.to_dict(), "type": l.type}
                        for l in self.layers],
             "max_positions": self.max_positions, "norm": {"eps": self.norm_eps}, "residual_mult": self.residual_mult,
             "vocab": self.vocab, "width": self.width}
        if self.token_side_dim is not None:
            d["token_side"] = {"dim": self.token_side_dim}
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d

    def model_spec(self) -> ModelSpec:
        W, eps = self.width, self.norm_eps
        std = lambda fan_in: 1.0 / math.sqrt(fan_in)          # random weights that keep activations near one
        norm = lambda name: NormSpec("rmsnorm32", W, eps, name, {"offset": True, "init_std": 0.1})
        layers = []
        n_layers = len(self.layers)
        for i, l in enumerate(self.layers):
            p = f"l{i}."
            m = l.mixer
            mixer = MixerSpec(
                kind="latent_attention", prefix=p + "mix.", hidden_size=W, num_heads=m.heads, num_kv_heads=1, head_dim=m.dim,
                scale=m.scale, window=m.window,
                tensor_names={"dq": "dq", "dq_norm": "dq.norm", "uq": "uq", "dkv": "dkv", "dkv_norm": "dkv.norm", "uk": "uk",
                              "uv": "uv", "o": "o"},
                options={"value_dim": m.vdim, "q_rank": m.q_rank, "kv_rank": m.kv_rank, "latent_norm_eps": eps})
            ffn = ffn_norm = None
            if l.mlp is not None and l.mlp.kind == "dense":
                ffn = FeedForwardSpec("gelu_mlp", p + "mlp.", W, l.mlp.ff, {"up": "up", "down": "down"},
                                      {"activation": "gelu_erf", "init_std_up": std(W), "init_std_down": std(l.mlp.ff)})
            elif l.mlp is not None:
                x = l.mlp
                ffn = FeedForwardSpec(
                    "routed_experts", p + "mlp.", W, x.expert.ff,
                    {"router": "router", "expert": "e{}.", "shared": "shared.", "gate": "gate", "up": "up", "down": "down"},
                    {"experts": x.experts, "top": x.top, "limit": x.expert.limit, "score": "sigmoid", "renormalize": False,
                     "scale_input": True, "sigmoid_slope": EXPERT_SIGMOID_SLOPE, "up_shift": EXPERT_UP_SHIFT,
                     "shared_size": x.shared.ff if x.shared else 0, "shared_limit": x.shared.limit if x.shared else 0.0})
            if ffn is not None:
                ffn_norm = norm(p + "norm2")
            side = None
            if self.token_side_dim is not None:
                d = self.token_side_dim
                side = TokenInputSpec("gated_embedding", p + "side.", W, d, self.vocab, "side.embed", n_layers * d, i * d, eps,
                                      {"gate": "gate", "proj": "proj", "norm": "norm"}, {"activation": "gelu_tanh"})
            layers.append(LayerSpec("post_norm", mixer, norm(p + "norm1"), ffn, ffn_norm, side,
                                    {"residual_mult": self.residual_mult}))
        return ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab, hidden_size=W, layers=tuple(layers),
            order=tuple(range(n_layers)), final_norm=norm("final.norm"), embed_name="embed", lm_head_name="head",
            max_positions=self.max_positions, eos_token_ids=self.eos_token_ids, init_std=std(W),
            embedding_kind="lookup_learned_positions", head_kind="linear",
            options={"residual_dtype": "float32", "position_table": "pos", "embed_init_std": 1.0, "position_init_std": 0.5})
