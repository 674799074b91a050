"""The Zulopel decoder ("architecture": "Zulopel") as a description in parts.

Tensors: `embed` [vocab, width], `head` [vocab, width], `final.norm`; per layer i `l<i>.norm1`, `l<i>.ls1` and, with a
feed-forward, `l<i>.norm2`, `l<i>.ls2`; an attention mixer's `l<i>.mix.{q, k, v, q.norm, k.norm, sink, g, o}` and, with
value mixing, `l<i>.mix.vmix`; a recurrent mixer's `l<i>.mix.{in, conv, conv.b, x, dt, dt.b, A_log, D, o}`; the
feed-forward's `l<i>.mlp.{router, correction, e<k>.gate, e<k>.up, e<k>.down}` and `l<i>.mlp.shared.{gate, up, down}`.

The stream starts as the embedding row times a constant. A layer is a post-norm block with layer scales:
x += ls1 * norm1(mixer(x)); x += ls2 * norm2(ff(x)). The mixers are gated attention (query/key norm, rotation of a part of
each head with a frequency ramp, chunked mask, a sink in the softmax, value mixing with the first such layer's values, an
output gate) and the selective scan; the feed-forward is the group-limited mixture of gated experts with a shared expert.
"""
from __future__ import annotations

from ..config.registry import Architecture, register_architecture
from ..config.zulopel import ZulopelConfig
from ..parts.spec import (BlockSpec, EmbeddingSpec, GatedAttentionSpec, GatedMLPSpec, GroupRoutedMLPSpec, HeadSpec, LayerRun, ModelSpec,
                          NormSpec, ScaledRotarySpec, SelectiveScanSpec)


def describe_zulopel(cfg: ZulopelConfig) -> ModelSpec:
    layers, ignore = [], []
    first_mix = True
    for i, l in enumerate(cfg.layers):
        p, m = f"l{i}.", l.mixer
        if l.type == "attention":
            sc = m.rot.scaling
            position = ScaledRotarySpec(kind="rope_ramp", dims=m.rot.dims, base=m.rot.base, max_positions=cfg.max_positions,
                                        factor=sc.factor if sc else 0.0, original=sc.original if sc else 0.0,
                                        fast=sc.fast if sc else 0.0, slow=sc.slow if sc else 0.0)
            role = None
            if m.v_mix:
                role = "first" if first_mix else "mix"
                first_mix = False
            if role != "mix":
                ignore.append(p + "mix.vmix")  # present in a file, read only by the layers that mix
            mixer = GatedAttentionSpec(kind="gated_attention", hidden=cfg.width, num_heads=m.heads, num_kv_heads=m.kv_heads,
                                       head_dim=m.dim, value_dim=m.vdim, scale=m.scale, eps=cfg.eps, position=position,
                                       q_weight=p + "mix.q", k_weight=p + "mix.k", v_weight=p + "mix.v", o_weight=p + "mix.o",
                                       q_norm=p + "mix.q.norm", k_norm=p + "mix.k.norm", sink=p + "mix.sink", gate_weight=p + "mix.g",
                                       value_mix=role, value_mix_weight=p + "mix.vmix" if role == "mix" else None, chunk=m.chunk)
        else:
            mixer = SelectiveScanSpec(kind="selective_scan", hidden=cfg.width, inner=m.inner, state=m.state, taps=m.taps,
                                      dt_rank=m.dt_rank, in_weight=p + "mix.in", conv_weight=p + "mix.conv", conv_bias=p + "mix.conv.b",
                                      x_weight=p + "mix.x", dt_weight=p + "mix.dt", dt_bias=p + "mix.dt.b", a_log=p + "mix.A_log",
                                      skip=p + "mix.D", o_weight=p + "mix.o")
        ff = norm2 = None
        if l.mlp is None:
            ignore += [p + "norm2", p + "ls2"]  # a layer without a feed-forward has no use for them
        else:
            f = l.mlp
            norm2 = NormSpec("rmsnorm", cfg.width, cfg.eps, p + "norm2")
            shared = None
            if f.shared_ff:
                shared = GatedMLPSpec(kind="gated_mlp", hidden=cfg.width, intermediate=f.shared_ff, gate_weight=p + "mlp.shared.gate",
                                      up_weight=p + "mlp.shared.up", down_weight=p + "mlp.shared.down", activation="silu")
            ff = GroupRoutedMLPSpec(kind="group_routed_mlp", hidden=cfg.width, intermediate=f.ff, experts=f.experts, top=f.top,
                                    router_weight=p + "mlp.router", correction=p + "mlp.correction",
                                    gate_weights=tuple(f"{p}mlp.e{k}.gate" for k in range(f.experts)),
                                    up_weights=tuple(f"{p}mlp.e{k}.up" for k in range(f.experts)),
                                    down_weights=tuple(f"{p}mlp.e{k}.down" for k in range(f.experts)),
                                    groups=f.groups, keep_groups=f.keep, norm_eps=1e-20, activation="silu", shared=shared)
        layers.append(BlockSpec(kind="post_norm", norm1=NormSpec("rmsnorm", cfg.width, cfg.eps, p + "norm1"), mixer=mixer,
                                norm2=norm2, feed_forward=ff, scale1=p + "ls1", scale2=p + "ls2"))
    return ModelSpec(
        architecture=cfg.architecture,
        embedding=EmbeddingSpec("embed", cfg.vocab, cfg.width, scale=cfg.embedding_scale),
        layers=tuple(layers),
        order=tuple(LayerRun(i) for i in range(len(layers))),
        final_norm=NormSpec("rmsnorm", cfg.width, cfg.eps, "final.norm"),
        head=HeadSpec("head", cfg.vocab, cfg.width),
        max_positions=cfg.max_positions,
        eos_token_ids=cfg.eos_token_ids,
        ignore=tuple(ignore),
    )


ZULOPEL = Architecture(name="Zulopel", parse_config=ZulopelConfig.from_dict, describe=describe_zulopel,
                       config_to_json=lambda cfg: cfg.to_dict())
register_architecture(ZULOPEL, replace=True)
