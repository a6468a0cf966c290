"""Typed view of a Kamelorn ``config.json``.

Kamelorn is a pre-norm decoder whose layers are listed one by one: each has a mixer (a
state-space recurrence, "mamba2", or attention over a cached latent, "latent_attention") and a
feed-forward (dense and gated, routed experts, or none).  A span of layers may run several times
in a row with the same weights (``loop``), every sublayer's output enters the residual times
``residual_mult``, and with ``streams`` the residual is several streams that every sublayer reads
and rewrites through learned coefficients.  Every size and every constant that may differ between
models is a key of the file; nothing here has a default that stands in for a missing size.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional

from tandem_b200.config.fumanex_config import NO_POSITION_LIMIT, _number
from tandem_b200.config.model_config import ConfigError, _positive_int, _require

MIXER_TYPES = ("mamba2", "latent_attention")
MLP_KINDS = ("dense", "moe")

__all__ = ["KamelornConfig", "KamelornLayer", "KamelornMamba", "KamelornLatent", "KamelornMLP", "NO_POSITION_LIMIT"]


def _int(d: dict, key: str, where: str) -> int:
    return _positive_int(d, where + key, _require(d, key))


@dataclass(frozen=True)
class KamelornMamba:
    heads: int
    vdim: int
    state: int
    groups: int
    conv: int
    norm_groups: int

    @classmethod
    def from_dict(cls, m: dict, where: str) -> "KamelornMamba":
        c = cls(heads=_int(m, "heads", where), vdim=_int(m, "vdim", where), state=_int(m, "state", where),
                groups=_positive_int(m, where + "groups", m.get("groups") or 1), conv=_int(m, "conv", where),
                norm_groups=_positive_int(m, where + "norm_groups", m.get("norm_groups") or 1))
        if c.heads % c.groups:
            raise ConfigError(f"config.json: {where}heads ({c.heads}) must be a multiple of groups ({c.groups})")
        if (c.heads * c.vdim) % c.norm_groups:
            raise ConfigError(f"config.json: {where}norm_groups ({c.norm_groups}) must divide heads * vdim ({c.heads * c.vdim})")
        return c

    def to_dict(self) -> dict:
        return {"heads": self.heads, "vdim": self.vdim, "state": self.state, "groups": self.groups, "conv": self.conv,
                "norm_groups": self.norm_groups}


@dataclass(frozen=True)
class KamelornLatent:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    rot_dims: int
    rot_base: float

    @classmethod
    def from_dict(cls, m: dict, where: str) -> "KamelornLatent":
        rot = _require(m, "rot")
        c = cls(heads=_int(m, "heads", where), dim=_int(m, "dim", where), rot_dim=_int(m, "rot_dim", where),
                vdim=_int(m, "vdim", where), kv_rank=_int(m, "kv_rank", where), scale=_number(m, "scale", where),
                rot_dims=_int(rot, "dims", where + "rot."), rot_base=_number(rot, "base", where + "rot."))
        if c.rot_dims > c.rot_dim or c.rot_dims % 2:
            raise ConfigError(f"config.json: {where}rot.dims ({c.rot_dims}) must be even and at most rot_dim ({c.rot_dim})")
        return c

    def to_dict(self) -> dict:
        return {"heads": self.heads, "dim": self.dim, "rot_dim": self.rot_dim, "vdim": self.vdim, "kv_rank": self.kv_rank,
                "scale": self.scale, "rot": {"dims": self.rot_dims, "base": self.rot_base}}


@dataclass(frozen=True)
class KamelornMLP:
    kind: str
    ff: int  # width of the dense feed-forward, or of one expert
    experts: int = 0
    top: int = 0
    route_scale: float = 1.0

    @classmethod
    def from_dict(cls, m: dict, where: str) -> "KamelornMLP":
        kind = _require(m, "kind")
        if kind not in MLP_KINDS:
            raise ConfigError(f"config.json: {where}kind {kind!r} is not supported (supported: {list(MLP_KINDS)})")
        if kind == "dense":
            return cls("dense", _int(m, "ff", where))
        router, expert = _require(m, "router"), _require(m, "expert")
        c = cls("moe", _int(expert, "ff", where + "expert."), experts=_int(router, "experts", where + "router."),
                top=_int(router, "top", where + "router."),
                route_scale=_number(router, "scale", where + "router.") if "scale" in router else 1.0)
        if c.top > c.experts:
            raise ConfigError(f"config.json: {where}router.top ({c.top}) exceeds router.experts ({c.experts})")
        return c

    def to_dict(self) -> dict:
        if self.kind == "dense":
            return {"kind": "dense", "ff": self.ff}
        return {"kind": "moe", "expert": {"ff": self.ff},
                "router": {"experts": self.experts, "top": self.top, "scale": self.route_scale}}


@dataclass(frozen=True)
class KamelornLayer:
    type: str
    mixer: Any  # KamelornMamba | KamelornLatent
    mlp: Optional[KamelornMLP]

    def to_dict(self) -> dict:
        return {"type": self.type, "mixer": self.mixer.to_dict(), "mlp": None if self.mlp is None else self.mlp.to_dict()}


@dataclass(frozen=True)
class KamelornConfig:
    architecture: str
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    residual_mult: float
    streams: Optional[int]  # None: one plain residual stream, no hyper-connection tensors
    layers: tuple  # of KamelornLayer
    loop: Optional[tuple]  # (start, stop, times): layers start .. stop-1 run `times` times in a row
    eos_token_ids: tuple = ()
    extra: dict = field(default_factory=dict, compare=False)

    @classmethod
    def from_dict(cls, d: dict) -> "KamelornConfig":
        entries = _require(d, "layers")
        if not isinstance(entries, list) or not entries:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, e in enumerate(entries):
            where = f"layers[{i}]."
            kind = _require(e, "type")
            if kind not in MIXER_TYPES:
                raise ConfigError(f"config.json: {where}type {kind!r} is not supported (supported: {list(MIXER_TYPES)})")
            m = _require(e, "mixer")
            mixer = KamelornMamba.from_dict(m, where + "mixer.") if kind == "mamba2" else KamelornLatent.from_dict(m, where + "mixer.")
            mlp = e.get("mlp")
            layers.append(KamelornLayer(kind, mixer, None if mlp is None else KamelornMLP.from_dict(mlp, where + "mlp.")))
        loop = d.get("loop")
        if loop is not None:
            start, stop = int(_require(loop, "start")), int(_require(loop, "stop"))
            times = _positive_int(loop, "loop.times", _require(loop, "times"))
            if not 0 <= start <= stop <= len(layers):
                raise ConfigError(f"config.json: loop {start} .. {stop} does not lie within the {len(layers)} layers")
            loop = (start, stop, times)
        streams = d.get("streams")
        if streams is not None:
            _positive_int(d, "streams", streams)
        eos = d.get("eos_token_id")
        known = {"architecture", "vocab", "width", "embedding", "norm", "residual_mult", "streams", "layers", "loop", "eos_token_id"}
        return cls(
            architecture=d.get("architecture", "Kamelorn"),
            vocab=_positive_int(d, "vocab", _require(d, "vocab")),
            width=_positive_int(d, "width", _require(d, "width")),
            embedding_scale=_number(d["embedding"], "scale", "embedding.") if d.get("embedding") else 1.0,
            norm_eps=_number(_require(d, "norm"), "eps", "norm."),
            residual_mult=_number(d, "residual_mult", "") if "residual_mult" in d else 1.0,
            streams=streams,
            layers=tuple(layers),
            loop=loop,
            eos_token_ids=() if eos is None else ((eos,) if isinstance(eos, int) else tuple(eos)),
            extra={k: v for k, v in d.items() if k not in known},
        )

    def run_order(self) -> list:
        """Layer indices in running order: the looped span repeated in place."""
        n = len(self.layers)
        if self.loop is None:
            return list(range(n))
        start, stop, times = self.loop
        return list(range(start)) + list(range(start, stop)) * times + list(range(stop, n))

    def to_dict(self) -> dict:
        d: dict = dict(self.extra)
        d.update(architecture=self.architecture, vocab=self.vocab, width=self.width,
                 embedding={"scale": self.embedding_scale}, norm={"eps": self.norm_eps}, residual_mult=self.residual_mult,
                 layers=[l.to_dict() for l in self.layers])
        if self.streams is not None:
            d["streams"] = self.streams
        if self.loop is not None:
            d["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids) if len(self.eos_token_ids) > 1 else self.eos_token_ids[0]
        return d
