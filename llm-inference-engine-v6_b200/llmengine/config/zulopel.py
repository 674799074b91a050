"""Typed configuration of the Zulopel decoder, read from its config.json.

Keys: `architecture` ("Zulopel"), `vocab`, `width`, `norm.eps`, `embedding.scale`, `layers` (a list; each entry has
`type`: "attention" or "mamba1", `mixer` with that mixer's sizes and constants, and `mlp`: null or `{kind: moe, expert:
{ff}, router: {experts, top, groups: {count, keep}}, shared: {ff}}`), optional `max_positions` (the design has no position
limit; the engine needs one for its rotation tables) and optional `eos_token_ids`. Every size and constant is read from here.

attention mixer: heads, kv_heads, dim (queries and keys), vdim (values), scale, rot {dims, base, scaling {factor, original,
fast, slow}}, mask {size} (chunks; absent: plain causal), v_mix (bool). mamba1 mixer: inner, state, conv (taps), dt_rank.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, FrozenSet, Optional, Tuple, Union

from .files import ConfigError
from .vapelix import DEFAULT_MAX_POSITIONS, Rotary, RotaryRamp, _need


@dataclass(frozen=True)
class AttentionMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: Rotary
    chunk: int = 0      # mask.size; 0: every earlier position is seen
    v_mix: bool = False


@dataclass(frozen=True)
class ScanMixer:
    inner: int
    state: int
    taps: int
    dt_rank: int


@dataclass(frozen=True)
class MoEConfig:
    ff: int
    experts: int
    top: int
    groups: int = 1
    keep: int = 1
    shared_ff: int = 0  # 0: no shared expert


@dataclass(frozen=True)
class ZulopelLayer:
    type: str  # "attention" | "mamba1"
    mixer: Union[AttentionMixer, ScanMixer]
    mlp: Optional[MoEConfig]


@dataclass(frozen=True)
class ZulopelConfig:
    architecture: str
    vocab: int
    width: int
    eps: float
    embedding_scale: float
    layers: Tuple[ZulopelLayer, ...]
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
    def from_dict(cls, j: Dict[str, Any], generation: Optional[Dict[str, Any]] = None) -> "ZulopelConfig":
        width, vocab = int(_need(j, "width", "config.json")), int(_need(j, "vocab", "config.json"))
        eps = float(_need(_need(j, "norm", "config.json"), "eps", "norm"))
        emb = j.get("embedding") or {}
        raw_layers = _need(j, "layers", "config.json")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, e in enumerate(raw_layers):
            where = f"layers[{i}]"
            kind = _need(e, "type", where)
            m = _need(e, "mixer", where)
            if kind == "attention":
                r = _need(m, "rot", where + ".mixer")
                sc = r.get("scaling")
                ramp = None
                if sc:
                    ramp = RotaryRamp(float(_need(sc, "factor", "rot.scaling")), float(_need(sc, "original", "rot.scaling")),
                                      float(_need(sc, "fast", "rot.scaling")), float(_need(sc, "slow", "rot.scaling")))
                mask = m.get("mask")
                mixer = AttentionMixer(heads=int(_need(m, "heads", where)), kv_heads=int(_need(m, "kv_heads", where)),
                                       dim=int(_need(m, "dim", where)), vdim=int(_need(m, "vdim", where)),
                                       scale=float(_need(m, "scale", where)),
                                       rot=Rotary(int(_need(r, "dims", "rot")), float(_need(r, "base", "rot")), ramp),
                                       chunk=int(_need(mask, "size", where + ".mixer.mask")) if mask else 0, v_mix=bool(m.get("v_mix", False)))
            elif kind == "mamba1":
                mixer = ScanMixer(inner=int(_need(m, "inner", where)), state=int(_need(m, "state", where)),
                                  taps=int(_need(m, "conv", where)), dt_rank=int(_need(m, "dt_rank", where)))
            else:
                raise ConfigError(f"config.json: {where}: unknown layer type '{kind}' (attention, mamba1)")
            f = e.get("mlp")
            mlp = None
            if f:
                fk = f.get("kind", "moe")
                if fk != "moe":
                    raise ConfigError(f"config.json: {where}.mlp: unknown kind '{fk}' (moe)")
                router = _need(f, "router", where + ".mlp")
                groups = router.get("groups") or {}
                shared = f.get("shared")
                mlp = MoEConfig(ff=int(_need(_need(f, "expert", where + ".mlp"), "ff", "expert")),
                                experts=int(_need(router, "experts", "router")), top=int(_need(router, "top", "router")),
                                groups=int(groups.get("count", 1)), keep=int(groups.get("keep", groups.get("count", 1))),
                                shared_ff=int(_need(shared, "ff", where + ".mlp.shared")) if shared else 0)
            layers.append(ZulopelLayer(kind, mixer, mlp))
        eos = j.get("eos_token_ids") or []
        cfg = cls(architecture=j.get("architecture", "Zulopel"), vocab=vocab, width=width, eps=eps,
                  embedding_scale=float(emb.get("scale", 1.0)), layers=tuple(layers),
                  max_positions=int(j.get("max_positions") or DEFAULT_MAX_POSITIONS), eos_token_ids=frozenset(int(t) for t in eos))
        cfg.check()
        return cfg

    def check(self) -> None:
        if self.width <= 0 or self.vocab <= 0 or self.eps < 0 or self.max_positions <= 0:
            raise ConfigError("config.json: width, vocab and max_positions must be positive, eps not negative")
        mixed = None
        for i, l in enumerate(self.layers):
            m, where = l.mixer, f"config.json: layers[{i}]"
            if l.type == "attention":
                if min(m.heads, m.kv_heads, m.dim, m.vdim) <= 0 or m.heads % m.kv_heads or m.chunk < 0:
                    raise ConfigError(f"{where}.mixer: sizes must be positive and heads a multiple of kv_heads")
                if m.rot.dims < 0 or m.rot.dims % 2 or m.rot.dims > m.dim:
                    raise ConfigError(f"{where}.mixer: rot.dims must be even and at most dim")
                if m.v_mix:
                    if mixed is not None and mixed != (m.kv_heads, m.vdim):
                        raise ConfigError(f"{where}.mixer: layers that mix values must agree in kv_heads and vdim")
                    mixed = (m.kv_heads, m.vdim)
            elif min(m.inner, m.state, m.taps, m.dt_rank) <= 0:
                raise ConfigError(f"{where}.mixer: sizes must be positive")
            f = l.mlp
            if f is not None:
                if f.ff <= 0 or not 1 <= f.top <= f.experts or f.shared_ff < 0:
                    raise ConfigError(f"{where}.mlp: bad sizes")
                if f.groups < 1 or f.experts % f.groups or not 1 <= f.keep <= f.groups or f.keep * (f.experts // f.groups) < f.top:
                    raise ConfigError(f"{where}.mlp.router.groups: {f.experts} experts, {f.groups} groups of which {f.keep} stay, {f.top} chosen")

    # ------------------------------------------------------------------ writing
    def to_dict(self) -> Dict[str, Any]:
        layers = []
        for l in self.layers:
            m = l.mixer
            if l.type == "attention":
                rot: Dict[str, Any] = {"dims": m.rot.dims, "base": m.rot.base}
                if m.rot.scaling is not None:
                    s = m.rot.scaling
                    rot["scaling"] = {"factor": s.factor, "original": s.original, "fast": s.fast, "slow": s.slow}
                mixer: Dict[str, Any] = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "scale": m.scale,
                                         "rot": rot, "v_mix": m.v_mix}
                if m.chunk:
                    mixer["mask"] = {"size": m.chunk}
            else:
                mixer = {"inner": m.inner, "state": m.state, "conv": m.taps, "dt_rank": m.dt_rank}
            mlp = None
            if l.mlp is not None:
                f = l.mlp
                mlp = {"kind": "moe", "expert": {"ff": f.ff},
                       "router": {"experts": f.experts, "top": f.top, "groups": {"count": f.groups, "keep": f.keep}}}
                if f.shared_ff:
                    mlp["shared"] = {"ff": f.shared_ff}
            layers.append({"type": l.type, "mixer": mixer, "mlp": mlp})
        out: Dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
                               "embedding": {"scale": self.embedding_scale}, "layers": layers, "max_positions": self.max_positions}
        if self.eos_token_ids:
            out["eos_token_ids"] = sorted(self.eos_token_ids)
        return out
