"""The Vapelix decoder ("architecture": "Vapelix") as a description in parts.

Tensors: `embed` [vocab, width] (also the output head), `final.norm`; per layer i `l<i>.norm1`, `l<i>.norm2`,
the mixer's `l<i>.mix.{dq, dq.norm, uq, dkv, dkv.norm, uk, uv, g, o}`, the feed-forward's `l<i>.mlp.{gate, up, down}`
(dense) or `l<i>.mlp.{router, router.b, e<k>.up, e<k>.down}` (routed); with a per-layer token input `side.embed`
[vocab, layers * dim] and `l<i>.side.{gate, proj, norm}`.

A layer is a parallel block (both norms read the same stream) with latent attention as its mixer. A loop in the
configuration repeats a range of layers with the same weights; every repetition is a run of its own in the layer
order, so it owns its cache, and the first layer of every repetition but the first adds the embedding's output to
the stream before it runs.
"""
from __future__ import annotations

from ..config.registry import Architecture, register_architecture
from ..config.vapelix import VapelixConfig
from ..parts.spec import (BlockSpec, EmbeddingSpec, GatedMLPSpec, HeadSpec, LatentAttentionSpec, LayerRun, ModelSpec, NormSpec,
                          RoutedMLPSpec, ScaledRotarySpec, TokenSideSpec)


def layer_order(cfg: VapelixConfig):
    L = len(cfg.layers)
    if cfg.loop is None:
        return tuple(LayerRun(i) for i in range(L))
    lp = cfg.loop
    order = [LayerRun(i) for i in range(lp.start)]
    for k in range(lp.times):
        order += [LayerRun(i, add_embedding=(k > 0 and i == lp.start)) for i in range(lp.start, lp.stop)]
    return tuple(order + [LayerRun(i) for i in range(lp.stop, L)])


def describe_vapelix(cfg: VapelixConfig) -> ModelSpec:
    layers, ignore = [], []
    L = len(cfg.layers)
    for i, l in enumerate(cfg.layers):
        p, m = f"l{i}.", l.mixer
        sc = m.rot.scaling
        position = ScaledRotarySpec(kind="rope_ramp", dims=m.rot.dims, base=m.rot.base, max_positions=cfg.max_positions,
                                    factor=sc.factor if sc else 0.0, original=sc.original if sc else 0.0,
                                    fast=sc.fast if sc else 0.0, slow=sc.slow if sc else 0.0)
        mixer = LatentAttentionSpec(kind="latent_attention", hidden=cfg.width, heads=m.heads, dim=m.dim, rot_dim=m.rot_dim, vdim=m.vdim,
                                    kv_rank=m.kv_rank, q_rank=m.q_rank, scale=m.scale, eps=cfg.eps, position=position,
                                    dq_weight=p + "mix.dq", dq_norm=p + "mix.dq.norm", uq_weight=p + "mix.uq",
                                    dkv_weight=p + "mix.dkv", dkv_norm=p + "mix.dkv.norm", uk_weight=p + "mix.uk",
                                    uv_weight=p + "mix.uv", gate_weight=p + "mix.g", o_weight=p + "mix.o")
        ff = norm2 = None
        if l.mlp is None:
            ignore.append(p + "norm2")  # a layer without a feed-forward has no use for its second norm
        else:
            norm2 = NormSpec("rmsnorm", cfg.width, cfg.eps, p + "norm2")
            if l.mlp.kind == "dense":
                ff = GatedMLPSpec(kind="gated_mlp", hidden=cfg.width, intermediate=l.mlp.ff, gate_weight=p + "mlp.gate",
                                  up_weight=p + "mlp.up", down_weight=p + "mlp.down", activation="gelu_tanh")
            else:
                ff = RoutedMLPSpec(kind="routed_mlp", hidden=cfg.width, intermediate=l.mlp.ff, experts=l.mlp.experts, top=l.mlp.top,
                                   router_weight=p + "mlp.router", router_bias=p + "mlp.router.b",
                                   up_weights=tuple(f"{p}mlp.e{k}.up" for k in range(l.mlp.experts)),
                                   down_weights=tuple(f"{p}mlp.e{k}.down" for k in range(l.mlp.experts)), activation="gelu")
        side = None
        if cfg.side_dim:
            side = TokenSideSpec(kind="gated_side", hidden=cfg.width, dim=cfg.side_dim, vocab_size=cfg.vocab, table="side.embed",
                                 table_width=L * cfg.side_dim, col0=i * cfg.side_dim, gate_weight=p + "side.gate",
                                 proj_weight=p + "side.proj", norm_weight=p + "side.norm", eps=cfg.eps)
        layers.append(BlockSpec(kind="parallel", norm1=NormSpec("rmsnorm", cfg.width, cfg.eps, p + "norm1"), mixer=mixer,
                                norm2=norm2, feed_forward=ff, token_input=side))
    return ModelSpec(
        architecture=cfg.architecture,
        embedding=EmbeddingSpec("embed", cfg.vocab, cfg.width),
        layers=tuple(layers),
        order=layer_order(cfg),
        final_norm=NormSpec("rmsnorm", cfg.width, cfg.eps, "final.norm"),
        head=HeadSpec("embed", cfg.vocab, cfg.width),
        max_positions=cfg.max_positions,
        eos_token_ids=cfg.eos_token_ids,
        ignore=tuple(ignore),
    )


VAPELIX = Architecture(name="Vapelix", parse_config=VapelixConfig.from_dict, describe=describe_vapelix,
                       config_to_json=lambda cfg: cfg.to_dict())
register_architecture(VAPELIX, replace=True)
