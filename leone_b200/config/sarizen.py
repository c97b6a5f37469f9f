"""Typed configuration of the Sarizen decoder.

Its ``config.json`` names the model under ``architecture`` and describes every layer on its own
(``layers``: a list of ``{"type", "mixer", "mlp"}``), so layers may differ in kind, sizes and
constants.  Top-level keys: ``vocab``, ``width``, ``norm.eps``, ``logit_scale``.  Mixer types:

``lightning``: ``heads``, ``dim``, ``vdim``, ``decay`` (one factor per head).
``latent_attention``: ``heads``, ``dim`` (unrotated), ``rot_dim`` (rotated), ``vdim``, ``kv_rank``,
``scale``, optional ``mask.size`` (sliding window), ``rot``: ``base``, ``dims`` and optional
``scaling`` (``factor``, ``original``, ``fast``, ``slow``).

``mlp`` is ``null``, ``{"kind": "dense", "ff"}`` or ``{"kind": "moe", "expert": {"ff"}, "router":
{"experts", "top"}, "shared": {"ff"} or null}``.

The file gives no limit on positions; ``max_positions`` (not a key of the design) bounds the
engine's block tables and defaults to 2**20.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from .base import ConfigReader, InvalidValue, ModelConfig, UnsupportedField, WrongType

DEFAULT_MAX_POSITIONS = 1 << 20


@dataclass(frozen=True)
class RotaryScaling:
    factor: float
    original: float
    fast: float
    slow: float


@dataclass(frozen=True)
class LightningMixer:
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]

    def to_json(self):
        return {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "decay": list(self.decay)}


@dataclass(frozen=True)
class LatentAttentionMixer:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    window: Optional[int]
    rot_base: float
    rot_dims: int
    rot_scaling: Optional[RotaryScaling]

    def to_json(self):
        rot = {"base": self.rot_base, "dims": self.rot_dims}
        if self.rot_scaling is not None:
            s = self.rot_scaling
            rot["scaling"] = {"factor": s.factor, "original": s.original, "fast": s.fast, "slow": s.slow}
        out = {"heads": self.heads, "dim": self.dim, "rot_dim": self.rot_dim, "vdim": self.vdim,
               "kv_rank": self.kv_rank, "scale": self.scale, "rot": rot}
        if self.window is not None:
            out["mask"] = {"size": self.window}
        return out


@dataclass(frozen=True)
class DenseMlp:
    ff: int

    def to_json(self):
        return {"kind": "dense", "ff": self.ff}


@dataclass(frozen=True)
class MoeMlp:
    expert_ff: int
    experts: int
    top: int
    shared_ff: Optional[int]

    def to_json(self):
        return {"kind": "moe", "expert": {"ff": self.expert_ff}, "router": {"experts": self.experts, "top": self.top},
                "shared": None if self.shared_ff is None else {"ff": self.shared_ff}}


@dataclass(frozen=True)
class SarizenLayer:
    type: str
    mixer: object
    mlp: object            # DenseMlp, MoeMlp or None

    def to_json(self):
        return {"type": self.type, "mixer": self.mixer.to_json(), "mlp": None if self.mlp is None else self.mlp.to_json()}


def _read_mixer(kind: str, r: ConfigReader):
    if kind == "lightning":
        heads = r.positive_int("heads")
        decay = r.raw.get("decay")
        if not isinstance(decay, list) or len(decay) != heads:
            raise InvalidValue(f"{r.where}: 'decay' must list one factor per head ({heads})")
        values = []
        for d in decay:
            if isinstance(d, bool) or not isinstance(d, (int, float)) or not 0.0 <= float(d) < float("inf"):
                raise InvalidValue(f"{r.where}: a decay factor must be a finite number >= 0, got {d!r}")
            values.append(float(d))
        return LightningMixer(heads, r.positive_int("dim"), r.positive_int("vdim"), tuple(values))
    if kind == "latent_attention":
        rot_dim = r.positive_int("rot_dim")
        rot = r.section("rot")
        dims = rot.positive_int("dims")
        if dims % 2 or dims > rot_dim:
            raise InvalidValue(f"{rot.where}: 'dims' ({dims}) must be even and at most rot_dim ({rot_dim})")
        sc = rot.section("scaling", optional=True)
        scaling = None if sc is None else RotaryScaling(sc.positive_float("factor"), sc.positive_float("original"),
                                                        sc.positive_float("fast"), sc.positive_float("slow"))
        mask = r.section("mask", optional=True)
        return LatentAttentionMixer(r.positive_int("heads"), r.positive_int("dim"), rot_dim, r.positive_int("vdim"),
                                    r.positive_int("kv_rank"), r.positive_float("scale"),
                                    None if mask is None else mask.positive_int("size"),
                                    rot.positive_float("base"), dims, scaling)
    raise UnsupportedField(f"{r.where}: mixer type '{kind}' is not supported (lightning, latent_attention)")


def _read_mlp(r: Optional[ConfigReader]):
    if r is None:
        return None
    kind = r.string("kind")
    if kind == "dense":
        return DenseMlp(r.positive_int("ff"))
    if kind == "moe":
        router = r.section("router")
        experts, top = router.positive_int("experts"), router.positive_int("top")
        if top > experts:
            raise InvalidValue(f"{router.where}: 'top' ({top}) exceeds 'experts' ({experts})")
        shared = r.section("shared", optional=True)
        return MoeMlp(r.section("expert").positive_int("ff"), experts, top,
                      None if shared is None else shared.positive_int("ff"))
    raise UnsupportedField(f"{r.where}: mlp kind '{kind}' is not supported (dense, moe)")


@dataclass(frozen=True)
class SarizenConfig(ModelConfig):
    vocab: int = 0
    width: int = 0
    norm_eps: float = 0.0
    logit_scale: float = 1.0
    layers: Tuple[SarizenLayer, ...] = ()
    max_positions: int = DEFAULT_MAX_POSITIONS

    ARCHITECTURE = "Sarizen"

    def to_json_dict(self) -> dict:
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
               "norm": {"eps": self.norm_eps}, "logit_scale": self.logit_scale,
               "layers": [layer.to_json() for layer in self.layers]}
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            out["max_positions"] = self.max_positions
        return out

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "SarizenConfig":
        r = ConfigReader(raw)
        layers_raw = raw.get("layers")
        if not isinstance(layers_raw, list) or not layers_raw:
            raise WrongType("config.json: 'layers' must be a non-empty list of layer descriptions")
        layers = []
        for i, entry in enumerate(layers_raw):
            lr = ConfigReader(entry, f"config.json: layers[{i}]")
            kind = lr.string("type")
            layers.append(SarizenLayer(kind, _read_mixer(kind, lr.section("mixer")),
                                       _read_mlp(lr.section("mlp", optional=True))))
        return cls(architecture=cls.ARCHITECTURE, vocab=r.positive_int("vocab"), width=r.positive_int("width"),
                   norm_eps=r.section("norm").positive_float("eps"), logit_scale=r.number("logit_scale", 1.0),
                   layers=tuple(layers), max_positions=r.positive_int("max_positions", DEFAULT_MAX_POSITIONS))
