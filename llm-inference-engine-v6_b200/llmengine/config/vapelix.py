"""Typed configuration of the Vapelix decoder, read from its config.json.

Keys: `architecture` ("Vapelix"), `vocab`, `width`, `norm.eps`, `layers` (a list; each entry has `type`,
`mixer` with the mixer's sizes, and `mlp`: null, `{kind: dense, ff}` or `{kind: moe, expert: {ff}, router:
{experts, top}}`), optional `loop` (`start`, `stop`, `times`: layers start .. stop-1 run `times` times in a row),
optional `token_side` (`dim`), optional `max_positions` (the design itself has no position limit; the engine
needs one for its rotation tables) and optional `eos_token_ids`. Every size is read from here; nothing about
sizes stands in code.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, FrozenSet, Optional, Tuple

from .files import ConfigError

DEFAULT_MAX_POSITIONS = 131072


def _need(d: Dict[str, Any], key: str, where: str):
    if not isinstance(d, dict) or key not in d or d[key] is None:
        raise ConfigError(f"config.json: missing key '{key}' in {where}")
    return d[key]


@dataclass(frozen=True)
class RotaryRamp:
    factor: float
    original: float
    fast: float
    slow: float


@dataclass(frozen=True)
class Rotary:
    dims: int
    base: float
    scaling: Optional[RotaryRamp] = None


@dataclass(frozen=True)
class LatentMixer:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    q_rank: int
    scale: float
    rot: Rotary


@dataclass(frozen=True)
class FeedForwardConfig:
    kind: str  # "dense" | "moe"
    ff: int
    experts: int = 0
    top: int = 0


@dataclass(frozen=True)
class LayerConfig:
    type: str
    mixer: LatentMixer
    mlp: Optional[FeedForwardConfig]


@dataclass(frozen=True)
class Loop:
    start: int
    stop: int
    times: int


@dataclass(frozen=True)
class VapelixConfig:
    architecture: str
    vocab: int
    width: int
    eps: float
    layers: Tuple[LayerConfig, ...]
    loop: Optional[Loop] = None
    side_dim: int = 0  # 0: no per-layer token input
    max_positions: int = DEFAULT_MAX_POSITIONS
    eos_token_ids: FrozenSet[int] = field(default_factory=frozenset)

    # names shared with the other configurations (the command line and the scheduler read them)
    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    @property
    def max_position_embeddings(self) -> int:
        return self.max_positions

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, j: Dict[str, Any], generation: Optional[Dict[str, Any]] = None) -> "VapelixConfig":
        width, vocab = int(_need(j, "width", "config.json")), int(_need(j, "vocab", "config.json"))
        eps = float(_need(_need(j, "norm", "config.json"), "eps", "norm"))
        raw_layers = _need(j, "layers", "config.json")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, e in enumerate(raw_layers):
            where = f"layers[{i}]"
            kind = _need(e, "type", where)
            if kind != "latent_attention":
                raise ConfigError(f"config.json: {where}: unknown layer type '{kind}' (latent_attention)")
            m = _need(e, "mixer", where)
            r = _need(m, "rot", where + ".mixer")
            sc = r.get("scaling")
            ramp = None
            if sc:
                ramp = RotaryRamp(float(_need(sc, "factor", "rot.scaling")), float(_need(sc, "original", "rot.scaling")),
                                  float(_need(sc, "fast", "rot.scaling")), float(_need(sc, "slow", "rot.scaling")))
            rot = Rotary(int(_need(r, "dims", "rot")), float(_need(r, "base", "rot")), ramp)
            mixer = LatentMixer(heads=int(_need(m, "heads", where)), dim=int(_need(m, "dim", where)),
                                rot_dim=int(_need(m, "rot_dim", where)), vdim=int(_need(m, "vdim", where)),
                                kv_rank=int(_need(m, "kv_rank", where)), q_rank=int(_need(m, "q_rank", where)),
                                scale=float(_need(m, "scale", where)), rot=rot)
            f = e.get("mlp")
            mlp = None
            if f:
                fk = _need(f, "kind", where + ".mlp")
                if fk == "dense":
                    mlp = FeedForwardConfig("dense", int(_need(f, "ff", where + ".mlp")))
                elif fk == "moe":
                    router = _need(f, "router", where + ".mlp")
                    mlp = FeedForwardConfig("moe", int(_need(_need(f, "expert", where + ".mlp"), "ff", "expert")),
                                            int(_need(router, "experts", "router")), int(_need(router, "top", "router")))
                else:
                    raise ConfigError(f"config.json: {where}.mlp: unknown kind '{fk}' (dense, moe)")
            layers.append(LayerConfig(kind, mixer, mlp))
        loop = None
        if j.get("loop"):
            lp = j["loop"]
            loop = Loop(int(_need(lp, "start", "loop")), int(_need(lp, "stop", "loop")), int(_need(lp, "times", "loop")))
        side = j.get("token_side")
        eos = j.get("eos_token_ids") or []
        cfg = cls(architecture=j.get("architecture", "Vapelix"), vocab=vocab, width=width, eps=eps, layers=tuple(layers), loop=loop,
                  side_dim=int(_need(side, "dim", "token_side")) if side else 0,
                  max_positions=int(j.get("max_positions") or DEFAULT_MAX_POSITIONS),
                  eos_token_ids=frozenset(int(t) for t in eos))
        cfg.check()
        return cfg

    def check(self) -> None:
        if self.width <= 0 or self.vocab <= 0 or self.eps < 0 or self.side_dim < 0 or self.max_positions <= 0:
            raise ConfigError("config.json: width, vocab and max_positions must be positive, eps and token_side.dim not negative")
        for i, l in enumerate(self.layers):
            m = l.mixer
            if min(m.heads, m.dim, m.vdim, m.kv_rank, m.q_rank) <= 0 or m.rot_dim < 0:
                raise ConfigError(f"config.json: layers[{i}].mixer: sizes must be positive")
            if m.rot.dims < 0 or m.rot.dims % 2 or m.rot.dims > m.rot_dim:
                raise ConfigError(f"config.json: layers[{i}].mixer: rot.dims must be even and at most rot_dim")
            if l.mlp is not None and (l.mlp.ff <= 0 or (l.mlp.kind == "moe" and not 1 <= l.mlp.top <= l.mlp.experts)):
                raise ConfigError(f"config.json: layers[{i}].mlp: bad sizes")
        if self.loop is not None:
            lp = self.loop
            if not (0 <= lp.start < lp.stop <= len(self.layers)) or lp.times < 1:
                raise ConfigError("config.json: loop: need 0 <= start < stop <= number of layers and times >= 1")

    # ------------------------------------------------------------------ writing
    def to_dict(self) -> Dict[str, Any]:
        layers = []
        for l in self.layers:
            m = l.mixer
            rot: Dict[str, Any] = {"dims": m.rot.dims, "base": m.rot.base}
            if m.rot.scaling is not None:
                s = m.rot.scaling
                rot["scaling"] = {"factor": s.factor, "original": s.original, "fast": s.fast, "slow": s.slow}
            mlp = None
            if l.mlp is not None:
                mlp = {"kind": "dense", "ff": l.mlp.ff} if l.mlp.kind == "dense" else \
                    {"kind": "moe", "expert": {"ff": l.mlp.ff}, "router": {"experts": l.mlp.experts, "top": l.mlp.top}}
            layers.append({"type": l.type, "mixer": {"heads": m.heads, "dim": m.dim, "rot_dim": m.rot_dim, "vdim": m.vdim,
                                                      "kv_rank": m.kv_rank, "q_rank": m.q_rank, "scale": m.scale, "rot": rot}, "mlp": mlp})
        out: Dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
                               "layers": layers, "max_positions": self.max_positions}
        if self.loop is not None:
            out["loop"] = {"start": self.loop.start, "stop": self.loop.stop, "times": self.loop.times}
        if self.side_dim:
            out["token_side"] = {"dim": self.side_dim}
        if self.eos_token_ids:
            out["eos_token_ids"] = sorted(self.eos_token_ids)
        return out
