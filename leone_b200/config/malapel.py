"""Typed configuration of the Malapel decoder.

Its ``config.json`` names the model under ``architecture`` and describes every layer on its own
(``layers``: a list of ``{"type", "mixer", "mlp"}``).  Top-level keys: ``vocab``, ``width``,
``norm.eps`` and, optionally, ``loop`` (``start``, ``stop``, ``times``: layers ``start .. stop-1``
run ``times`` times in a row with the same weights).

The three mixer types share their keys: ``heads``, ``kv_heads``, ``dim`` (query/key width of a
head), ``vdim`` (value width), ``scale``, ``rot`` (``base``, ``dims``), and ``mask.size`` where the
type has a mask of a size:

``attention``: chunks of ``mask.size`` positions; ``attention_2``: causal; ``attention_3``: a
sliding window of ``mask.size`` positions.

``mlp`` is ``null``, ``{"kind": "dense", "ff", "limit"}`` or ``{"kind": "moe", "expert": {"ff"},
"router": {"experts", "top", "scale", "groups": {"count", "keep"}}}``.

The file gives no limit on positions; ``max_positions`` (not a key of the design) bounds the
engine's block tables and defaults to 2**20.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from .base import ConfigReader, InvalidValue, ModelConfig, UnsupportedField, WrongType

DEFAULT_MAX_POSITIONS = 1 << 20
MIXER_TYPES = ("attention", "attention_2", "attention_3")
MASKED_TYPES = ("attention", "attention_3")       # the types whose mask has a size


@dataclass(frozen=True)
class AttentionMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot_base: float
    rot_dims: int
    mask_size: Optional[int]

    def to_json(self):
        out = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim,
               "scale": self.scale, "rot": {"base": self.rot_base, "dims": self.rot_dims}}
        if self.mask_size is not None:
            out["mask"] = {"size": self.mask_size}
        return out


@dataclass(frozen=True)
class DenseMlp:
    ff: int
    limit: float

    def to_json(self):
        return {"kind": "dense", "ff": self.ff, "limit": self.limit}


@dataclass(frozen=True)
class MoeMlp:
    expert_ff: int
    experts: int
    top: int
    scale: float
    group_count: int
    group_keep: int
    grouped: bool        # whether the file spelled the groups out

    def to_json(self):
        router = {"experts": self.experts, "top": self.top, "scale": self.scale}
        if self.grouped:
            router["groups"] = {"count": self.group_count, "keep": self.group_keep}
        return {"kind": "moe", "expert": {"ff": self.expert_ff}, "router": router}


@dataclass(frozen=True)
class Loop:
    start: int
    stop: int
    times: int

    def to_json(self):
        return {"start": self.start, "stop": self.stop, "times": self.times}


@dataclass(frozen=True)
class MalapelLayer:
    type: str
    mixer: AttentionMixer
    mlp: object            # DenseMlp, MoeMlp or None

    def to_json(self):
        return {"type": self.type, "mixer": self.mixer.to_json(), "mlp": None if self.mlp is None else self.mlp.to_json()}


def _read_mixer(kind: str, r: ConfigReader) -> AttentionMixer:
    if kind not in MIXER_TYPES:
        raise UnsupportedField(f"{r.where}: mixer type '{kind}' is not supported ({', '.join(MIXER_TYPES)})")
    heads, kv_heads, dim = r.positive_int("heads"), r.positive_int("kv_heads"), r.positive_int("dim")
    if heads % kv_heads:
        raise InvalidValue(f"{r.where}: 'heads' ({heads}) must be a multiple of 'kv_heads' ({kv_heads})")
    rot = r.section("rot")
    dims = rot.positive_int("dims")
    if dims % 2 or dims > dim:
        raise InvalidValue(f"{rot.where}: 'dims' ({dims}) must be even and at most dim ({dim})")
    mask = r.section("mask", optional=kind not in MASKED_TYPES)
    return AttentionMixer(heads, kv_heads, dim, r.positive_int("vdim"), r.positive_float("scale"),
                          rot.positive_float("base"), dims,
                          mask.positive_int("size") if mask is not None and kind in MASKED_TYPES else None)


def _read_mlp(r: Optional[ConfigReader]):
    if r is None:
        return None
    kind = r.string("kind")
    if kind == "dense":
        return DenseMlp(r.positive_int("ff"), r.positive_float("limit"))
    if kind == "moe":
        router = r.section("router")
        experts, top = router.positive_int("experts"), router.positive_int("top")
        groups = router.section("groups", optional=True)
        count = 1 if groups is None else groups.positive_int("count")
        keep = count if groups is None else groups.positive_int("keep")
        if experts % count or keep > count:
            raise InvalidValue(f"{router.where}: {experts} experts do not form {count} equal groups of which {keep} are kept")
        if top > experts // count * keep:
            raise InvalidValue(f"{router.where}: 'top' ({top}) exceeds the experts of the kept groups ({experts // count * keep})")
        return MoeMlp(r.section("expert").positive_int("ff"), experts, top, router.number("scale", 1.0), count, keep,
                      groups is not None)
    raise UnsupportedField(f"{r.where}: mlp kind '{kind}' is not supported (dense, moe)")


@dataclass(frozen=True)
class MalapelConfig(ModelConfig):
    vocab: int = 0
    width: int = 0
    norm_eps: float = 0.0
    layers: Tuple[MalapelLayer, ...] = ()
    loop: Optional[Loop] = None
    max_positions: int = DEFAULT_MAX_POSITIONS

    ARCHITECTURE = "Malapel"

    def to_json_dict(self) -> dict:
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
               "norm": {"eps": self.norm_eps}, "layers": [layer.to_json() for layer in self.layers]}
        if self.loop is not None:
            out["loop"] = self.loop.to_json()
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            out["max_positions"] = self.max_positions
        return out

    def run_order(self) -> Tuple[int, ...]:
        """Layer indices in the order they run."""
        n = len(self.layers)
        if self.loop is None:
            return tuple(range(n))
        lp = self.loop
        return tuple(range(lp.start)) + tuple(range(lp.start, lp.stop)) * lp.times + tuple(range(lp.stop, n))

    def pass_starts(self) -> Tuple[int, ...]:
        """Positions of the run order at which a pass over the looped layers begins."""
        if self.loop is None:
            return ()
        lp = self.loop
        return tuple(lp.start + k * (lp.stop - lp.start) for k in range(lp.times))

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "MalapelConfig":
        r = ConfigReader(raw)
        layers_raw = raw.get("layers")
        if not isinstance(layers_raw, list) or not layers_raw:
            raise WrongType("config.json: 'layers' must be a non-empty list of layer descriptions")
        layers = []
        for i, entry in enumerate(layers_raw):
            lr = ConfigReader(entry, f"config.json: layers[{i}]")
            kind = lr.string("type")
            layers.append(MalapelLayer(kind, _read_mixer(kind, lr.section("mixer")),
                                       _read_mlp(lr.section("mlp", optional=True))))
        loop = None
        lr = r.section("loop", optional=True)
        if lr is not None:
            start = lr.optional_int("start")
            stop, times = lr.positive_int("stop"), lr.positive_int("times")
            if start is None or not 0 <= start < stop <= len(layers):
                raise InvalidValue(f"{lr.where}: layers {start} .. {stop} - 1 are not a span of the {len(layers)} layers")
            loop = Loop(start, stop, times)
        return cls(architecture=cls.ARCHITECTURE, vocab=r.positive_int("vocab"), width=r.positive_int("width"),
                   norm_eps=r.section("norm").positive_float("eps"), layers=tuple(layers), loop=loop,
                   max_positions=r.positive_int("max_positions", DEFAULT_MAX_POSITIONS))
