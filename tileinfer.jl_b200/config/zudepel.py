"""Typed configuration of the Zudepel design and its lowering to per-layer records.

A Zudepel model is a decoder whose config.json lists its layers one by one (``layers``: ``type``, ``mixer``, ``mlp``), so every
layer may have sizes of its own. What the design fixes lives here and in the parts; what config.json gives is read from it and
nowhere else:

* the stream starts as the token's embedding row and is kept in 32-bit; the model ends with an RMS norm and the head;
* a layer has ONE RMS norm (plain weight), whose output both the mixer and the feed-forward read; both results are added;
* mixer ``lightning``: linear attention with a decay per head (``decay``) and a matrix state per head carried from token to
  token; SiLU on queries, keys and values, an RMS norm over all heads' outputs and a sigmoid output gate;
* mixer ``attention``: grouped-query attention (``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``) with biases on q, k, v, a
  causal convolution of ``conv`` taps over time on every projected channel, RMS norms over the whole q and k rows, a rotation
  of the first ``rot.dims`` elements of every head (half-split pairs, base ``rot.base``), a learned sink per head in the softmax's
  denominator and a sigmoid output gate; with ``kv_from`` the layer reads the keys and values of an earlier layer;
* feed-forward ``dense``: down(gelu_tanh(gate h) * up h); ``moe``: a softmax router over experts and ``identity`` pass-through
  outputs, a correction added for the choice, ``groups`` of neighbours of which the best stay, the ``top`` choices with weights
  divided by their sum, SiLU-gated experts, and a shared expert scaled by a sigmoid gate; or none.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from .apertus import ConfigError, _require
from .spec import FeedForwardSpec, LayerSpec, MixerSpec, ModelSpec, NormSpec, PositionSpec

DEFAULT_MAX_POSITIONS = 131072       # config.json gives no limit; tables are sized by the engine's max_context below this


def _need(m: Mapping[str, Any], key: str, where: str):
    if not isinstance(m, Mapping) or key not in m or m[key] is None:
        raise ConfigError(f"config.json: {where} has no \"{key}\"")
    return m[key]


@dataclass(frozen=True)
class LightningConfig:
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]

    @classmethod
    def from_dict(cls, m, where):
        out = cls(int(_need(m, "heads", where)), int(_need(m, "dim", where)), int(_need(m, "vdim", where)),
                  tuple(float(a) for a in _need(m, "decay", where)))
        if min(out.heads, out.dim, out.vdim) < 1:
            raise ConfigError(f"{where}: heads, dim and vdim must be positive")
        if len(out.decay) != out.heads:
            raise ConfigError(f"{where}.decay has {len(out.decay)} entries for {out.heads} heads")
        return out

    def to_dict(self):
        return {"decay": list(self.decay), "dim": self.dim, "heads": self.heads, "vdim": self.vdim}


@dataclass(frozen=True)
class AttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    conv: int                          # taps of the convolution; 0: none
    rot_dims: int                      # 0: no rotation
    rot_base: float
    kv_from: Optional[int]

    @classmethod
    def from_dict(cls, m, where):
        rot = m.get("rot")
        out = cls(int(_need(m, "heads", where)), int(m.get("kv_heads") or _need(m, "heads", where)), int(_need(m, "dim", where)),
                  int(m.get("vdim") or _need(m, "dim", where)), float(_need(m, "scale", where)), int(m.get("conv") or 0),
                  int(_need(rot, "dims", where + ".rot")) if rot else 0, float(_need(rot, "base", where + ".rot")) if rot else 10000.0,
                  None if m.get("kv_from") is None else int(m["kv_from"]))
        if min(out.heads, out.kv_heads, out.dim, out.vdim) < 1 or out.heads % out.kv_heads:
            raise ConfigError(f"{where}: {out.heads} query heads do not divide into {out.kv_heads} key/value heads")
        if out.rot_dims % 2 or out.rot_dims > out.dim:
            raise ConfigError(f"{where}.rot.dims {out.rot_dims} must be even and at most dim {out.dim}")
        if out.conv < 0:
            raise ConfigError(f"{where}.conv must not be negative")
        return out

    def to_dict(self):
        d = {"dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads, "scale": self.scale, "vdim": self.vdim}
        if self.conv:
            d["conv"] = self.conv
        if self.rot_dims:
            d["rot"] = {"base": self.rot_base, "dims": self.rot_dims}
        if self.kv_from is not None:
            d["kv_from"] = self.kv_from
        return d


@dataclass(frozen=True)
class MlpConfig:
    kind: str                          # "dense" | "moe"
    ff: int = 0                        # dense: inner size; moe: an expert's
    experts: int = 0
    identity: int = 0
    top: int = 0
    groups: int = 1
    keep: int = 1
    shared_ff: int = 0                 # 0: no shared expert

    @classmethod
    def from_dict(cls, m, where):
        kind = _need(m, "kind", where)
        if kind == "dense":
            return cls("dense", ff=int(_need(m, "ff", where)))
        if kind != "moe":
            raise ConfigError(f"{where}.kind \"{kind}\" is not a feed-forward of this design (dense, moe)")
        r = _need(m, "router", where)
        g = r.get("groups") or {}
        s = m.get("shared") or {}
        out = cls("moe", ff=int(_need(_need(m, "expert", where), "ff", where + ".expert")), experts=int(_need(r, "experts", where + ".router")),
                  identity=int(r.get("identity") or 0), top=int(_need(r, "top", where + ".router")), groups=int(g.get("count") or 1),
                  keep=int(g.get("keep") or g.get("count") or 1), shared_ff=int(s.get("ff") or 0))
        total = out.experts + out.identity
        if out.experts < 1 or not 1 <= out.top <= total:
            raise ConfigError(f"{where}.router: top {out.top} of {total} router outputs")
        if total % out.groups or not 1 <= out.keep <= out.groups or out.keep * (total // out.groups) < out.top:
            raise ConfigError(f"{where}.router.groups: {out.keep} of {out.groups} groups over {total} router outputs for top {out.top}")
        return out

    def to_dict(self):
        if self.kind == "dense":
            return {"ff": self.ff, "kind": "dense"}
        r = {"experts": self.experts, "top": self.top}
        if self.groups > 1:
            r["groups"] = {"count": self.groups, "keep": self.keep}
        if self.identity:
            r["identity"] = self.identity
        d = {"expert": {"ff": self.ff}, "kind": "moe", "router": r}
        if self.shared_ff:
            d["shared"] = {"ff": self.shared_ff}
        return d


@dataclass(frozen=True)
class ZudepelLayerConfig:
    type: str                          # "lightning" | "attention"
    mixer: Any
    mlp: Optional[MlpConfig]


@dataclass(frozen=True)
class ZudepelConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[ZudepelLayerConfig, ...]
    max_positions: int = DEFAULT_MAX_POSITIONS
    eos_token_ids: Tuple[int, ...] = ()

    architecture = "Zudepel"
    model_type = "zudepel"

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @classmethod
    def from_dict(cls, c: Mapping[str, Any]) -> "ZudepelConfig":
        layers = []
        for i, l in enumerate(_require(c, "layers")):
            where = f"layers[{i}]"
            kind = _need(l, "type", where)
            if kind == "lightning":
                mixer = LightningConfig.from_dict(_need(l, "mixer", where), where + ".mixer")
            elif kind == "attention":
                mixer = AttentionConfig.from_dict(_need(l, "mixer", where), where + ".mixer")
                j = mixer.kv_from
                if j is not None:
                    src = layers[j].mixer if 0 <= j < i and layers[j].type == "attention" else None
                    if src is None or src.kv_from is not None:
                        raise ConfigError(f"{where}.mixer.kv_from {j} must name an earlier attention layer with keys and values of its own")
                    if (src.kv_heads, src.dim, src.vdim) != (mixer.kv_heads, mixer.dim, mixer.vdim):
                        raise ConfigError(f"{where}.mixer: key/value heads and sizes differ from those of layer {j}, whose keys and values it reads")
            else:
                raise ConfigError(f"{where}.type \"{kind}\" is not a mixer of this design (lightning, attention)")
            mlp = l.get("mlp")
            layers.append(ZudepelLayerConfig(kind, mixer, None if mlp is None else MlpConfig.from_dict(mlp, where + ".mlp")))
        eos = c.get("eos_token_id", ())
        eos = (eos,) if isinstance(eos, int) else tuple(eos or ())
        out = cls(vocab=int(_require(c, "vocab")), width=int(_require(c, "width")), norm_eps=float(_need(_require(c, "norm"), "eps", "norm")),
                  layers=tuple(layers), max_positions=int(c.get("max_positions") or DEFAULT_MAX_POSITIONS), eos_token_ids=eos)
        if out.vocab < 1 or out.width < 1 or not layers:
            raise ConfigError("vocab and width must be positive and layers not empty")
        return out

    def to_dict(self) -> dict:
        d = {"architecture": self.architecture,
             "layers": [{"mixer": l.mixer.to_dict(), "mlp": None if l.mlp is None else l.mlp.to_dict(), "type": l.type} for l in self.layers],
             "norm": {"eps": self.norm_eps}, "vocab": self.vocab, "width": self.width}
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            d["max_positions"] = self.max_positions
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d

    def model_spec(self) -> ModelSpec:
        W, eps = self.width, self.norm_eps
        norm = lambda name: NormSpec("rmsnorm32", W, eps, name, {"init_std": 0.1})
        layers = []
        for i, l in enumerate(self.layers):
            p = f"l{i}."
            m = l.mixer
            if l.type == "lightning":
                mixer = MixerSpec(kind="lightning", prefix=p + "mix.", hidden_size=W, num_heads=m.heads, head_dim=m.dim,
                                  tensor_names={"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "norm": "norm"},
                                  options={"value_dim": m.vdim, "decay": m.decay, "norm_eps": eps, "gate": True, "activation": "silu"})
            else:
                position = PositionSpec(kind="none")
                if m.rot_dims:
                    position = PositionSpec(kind="rope", head_dim=m.dim, theta=m.rot_base, max_positions=self.max_positions,
                                            options={"rotary_dim": m.rot_dims, "pairing": "half", "table_dtype": "float32", "angles": "float64"})
                mixer = MixerSpec(kind="conv_attention", prefix=p + "mix.", hidden_size=W, num_heads=m.heads, num_kv_heads=m.kv_heads,
                                  head_dim=m.dim, qk_norm=True, qk_norm_eps=eps, scale=m.scale, kv_source=m.kv_from, position=position,
                                  tensor_names={"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "sink": "sink", "bias_suffix": ".b",
                                                "conv_suffix": ".conv", "norm_suffix": ".norm"},
                                  options={"value_dim": m.vdim, "conv_taps": m.conv, "bias": True, "row_norm": True, "sink": True, "gate": True})
            ffn = None
            x = l.mlp
            if x is not None and x.kind == "dense":
                ffn = FeedForwardSpec("gated_mlp", p + "mlp.", W, x.ff, {"gate": "gate", "up": "up", "down": "down"}, {"activation": "gelu_tanh"})
            elif x is not None:
                ffn = FeedForwardSpec(
                    "routed_experts", p + "mlp.", W, x.ff,
                    {"router": "router", "correction": "correction", "expert": "e{}.", "shared": "shared.", "shared_gate": "shared.sg",
                     "gate": "gate", "up": "up", "down": "down"},
                    {"experts": x.experts, "top": x.top, "limit": None, "score": "softmax", "renormalize": True, "correction": True,
                     "groups": (x.groups, x.keep), "pass_through": x.identity, "scale_input": False, "sigmoid_slope": 1.0, "up_shift": 0.0,
                     "shared_size": x.shared_ff, "shared_limit": None, "shared_gate": bool(x.shared_ff)})
            layers.append(LayerSpec("parallel", mixer, norm(p + "norm1"), ffn, None))
        return ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab, hidden_size=W, layers=tuple(layers), order=tuple(range(len(layers))),
            final_norm=norm("final.norm"), embed_name="embed", lm_head_name="head", max_positions=self.max_positions,
            eos_token_ids=self.eos_token_ids, init_std=W ** -0.5, embedding_kind="lookup32", head_kind="linear",
            options={"residual_dtype": "float32", "embed_init_std": 1.0})
