"""Typed view of a Fumanex ``config.json``.

Fumanex is a decoder of parallel layers (one norm, mixer and feed-forward side by side) whose
mixers are listed layer by layer: softmax attention with a window, kept first tokens, a bias by
distance and a sink ("attention"), or linear attention with a fixed decay per head, in two
dressings ("retention", "lightning").  Every size and every constant that may differ between
models is a key of the file; nothing here has a default that stands in for a missing size.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional

from tandem_b200.config.model_config import ConfigError, _positive_int, _require

MIXER_TYPES = ("attention", "retention", "lightning")
NO_POSITION_LIMIT = 1 << 24  # the design has no table of positions; float32 holds every position below this exactly


def _number(d: dict, key: str, where: str) -> float:
    v = _require(d, key)
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json: {where}{key!r} must be a number, got {v!r}")
    return float(v)


@dataclass(frozen=True)
class FumanexAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: Optional[float]
    bias_max: int
    window: Optional[int]
    keep_first: int
    v_mix: bool
    bias_buckets: int = 32  # rows of the distance-bias table; the checkpoint's tensor decides where there is one

    @classmethod
    def from_dict(cls, m: dict, where: str) -> "FumanexAttention":
        heads = _positive_int(m, "heads", _require(m, "heads"))
        kv = _positive_int(m, "kv_heads", m.get("kv_heads") or heads)
        if heads % kv:
            raise ConfigError(f"config.json: {where}heads ({heads}) must be a multiple of kv_heads ({kv})")
        mask = m.get("mask") or {}
        window = mask.get("size")
        if window is not None:
            _positive_int(mask, "mask.size", window)
        keep = int(mask.get("keep_first") or 0)
        if keep < 0:
            raise ConfigError(f"config.json: {where}mask.keep_first must not be negative")
        cap = m.get("softcap")
        return cls(heads=heads, kv_heads=kv, dim=_positive_int(m, "dim", _require(m, "dim")),
                   vdim=_positive_int(m, "vdim", m.get("vdim") or m["dim"]), scale=_number(m, "scale", where),
                   softcap=None if cap is None else float(cap), bias_max=_positive_int(m, "bias_max", _require(m, "bias_max")),
                   window=window, keep_first=keep, v_mix=bool(m.get("v_mix", False)),
                   bias_buckets=_positive_int(m, "bias_buckets", m.get("bias_buckets") or 32))

    def to_dict(self) -> dict:
        d: dict = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale,
                   "bias_max": self.bias_max, "v_mix": self.v_mix, "bias_buckets": self.bias_buckets}
        if self.softcap is not None:
            d["softcap"] = self.softcap
        if self.window is not None:
            d["mask"] = {"size": self.window, "keep_first": self.keep_first}
        return d


@dataclass(frozen=True)
class FumanexRecurrence:
    heads: int
    dim: int
    vdim: int
    decay: tuple
    rot_dims: int = 0  # retention only
    rot_base: float = 10000.0

    @classmethod
    def from_dict(cls, m: dict, where: str, kind: str) -> "FumanexRecurrence":
        heads = _positive_int(m, "heads", _require(m, "heads"))
        decay = tuple(float(x) for x in _require(m, "decay"))
        if len(decay) != heads:
            raise ConfigError(f"config.json: {where}decay has {len(decay)} entries for {heads} heads")
        dim = _positive_int(m, "dim", _require(m, "dim"))
        rot = m.get("rot") if kind == "retention" else None
        dims, base = 0, 10000.0
        if rot:
            dims = _positive_int(rot, "rot.dims", _require(rot, "dims"))
            base = _number(rot, "base", where + "rot.")
            if dims % 2 or dims > dim:
                raise ConfigError(f"config.json: {where}rot.dims ({dims}) must be even and at most dim ({dim})")
        return cls(heads=heads, dim=dim, vdim=_positive_int(m, "vdim", m.get("vdim") or dim), decay=decay, rot_dims=dims,
                   rot_base=base)

    def to_dict(self) -> dict:
        d: dict = {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "decay": list(self.decay)}
        if self.rot_dims:
            d["rot"] = {"dims": self.rot_dims, "base": self.rot_base}
        return d


@dataclass(frozen=True)
class FumanexLayer:
    type: str
    mixer: Any  # FumanexAttention | FumanexRecurrence
    ff: Optional[int]  # width of the dense feed-forward, None: the layer has none

    def to_dict(self) -> dict:
        return {"type": self.type, "mixer": self.mixer.to_dict(),
                "mlp": None if self.ff is None else {"kind": "dense", "ff": self.ff}}


@dataclass(frozen=True)
class FumanexConfig:
    architecture: str
    vocab: int
    width: int
    embedding_scale: float
    logit_scale: float
    norm_eps: float
    layers: tuple  # of FumanexLayer
    eos_token_ids: tuple = ()
    extra: dict = field(default_factory=dict, compare=False)

    @classmethod
    def from_dict(cls, d: dict) -> "FumanexConfig":
        layers = []
        entries = _require(d, "layers")
        if not isinstance(entries, list) or not entries:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        for i, e in enumerate(entries):
            where = f"layers[{i}]."
            kind = _require(e, "type")
            if kind not in MIXER_TYPES:
                raise ConfigError(f"config.json: {where}type {kind!r} is not supported (supported: {list(MIXER_TYPES)})")
            m = _require(e, "mixer")
            mixer = FumanexAttention.from_dict(m, where) if kind == "attention" else FumanexRecurrence.from_dict(m, where, kind)
            mlp = e.get("mlp")
            ff = None
            if mlp is not None:
                if mlp.get("kind") != "dense":
                    raise ConfigError(f"config.json: {where}mlp.kind {mlp.get('kind')!r} is not supported (dense)")
                ff = _positive_int(mlp, "mlp.ff", _require(mlp, "ff"))
            layers.append(FumanexLayer(kind, mixer, ff))
        mixing = [l.mixer for l in layers if l.type == "attention" and l.mixer.v_mix]
        if any((m.kv_heads, m.vdim) != (mixing[0].kv_heads, mixing[0].vdim) for m in mixing):
            raise ConfigError("config.json: layers with v_mix must agree in kv_heads and vdim (they mix one another's values)")
        eos = d.get("eos_token_id")
        known = {"architecture", "vocab", "width", "embedding", "logit_scale", "norm", "layers", "eos_token_id"}
        return cls(
            architecture=d.get("architecture", "Fumanex"),
            vocab=_positive_int(d, "vocab", _require(d, "vocab")),
            width=_positive_int(d, "width", _require(d, "width")),
            embedding_scale=_number(d.get("embedding") or {}, "scale", "embedding.") if d.get("embedding") else 1.0,
            logit_scale=float(d.get("logit_scale", 1.0)),
            norm_eps=_number(_require(d, "norm"), "eps", "norm."),
            layers=tuple(layers),
            eos_token_ids=() if eos is None else ((eos,) if isinstance(eos, int) else tuple(eos)),
            extra={k: v for k, v in d.items() if k not in known},
        )

    def with_checkpoint_shapes(self, shapes: Optional[dict]) -> "FumanexConfig":
        """Sizes that only a tensor's shape gives: the rows of each attention layer's distance-bias table."""
        from dataclasses import replace

        if not shapes:
            return self
        layers = []
        for i, l in enumerate(self.layers):
            rel = shapes.get(f"l{i}.mix.rel")
            if l.type == "attention" and rel is not None and len(rel) == 2:
                l = replace(l, mixer=replace(l.mixer, bias_buckets=int(rel[0])))
            layers.append(l)
        return replace(self, layers=tuple(layers))

    def to_dict(self) -> dict:
        d: dict = dict(self.extra)
        d.update(architecture=self.architecture, vocab=self.vocab, width=self.width,
                 embedding={"scale": self.embedding_scale}, logit_scale=self.logit_scale, norm={"eps": self.norm_eps},
                 layers=[l.to_dict() for l in self.layers])
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids) if len(self.eos_token_ids) > 1 else self.eos_token_ids[0]
        return d
