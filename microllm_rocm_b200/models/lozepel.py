"""The Lozepel decoder as data: which parts, with which sizes, in which order.

token embedding plus a row of a second table chosen by the token and the one before it -> layers of
[x += norm(mixer(norm(x))); x += norm(ff(norm(x)))] -> rms norm -> head -> a cap on the logits.  Every norm of the stream
stores its weight minus one.  A layer's mixer is one of: grouped-query softmax attention whose values are the projected
keys, with biases on q and k, interleaved rotation, one added to the softmax's denominator and one sigmoid gate per head;
two mixers side by side added with fixed weights (softmax attention with q and k normalised over their whole rows, a
learned sink per head and a gate per head; linear attention with one fixed decay per head, silu on q, k and v, a norm over
all heads together and a sigmoid gate); softmax attention with rotation, then q and k divided by their root mean square
per head, capped scores and a learned sink, which may read the keys and values of an earlier layer instead of projecting
its own.  The feed-forward is a gated one with a clamped activation, routed experts (softmax over all router outputs, a
correction that only steers the choice, outputs without an expert that pass the input on), or none.

Tensor names: `embed`, `bigram`, `final.norm`, `head`; layer i: `l<i>.norm1`, `.norm1b`, `.norm2`, `.norm2b`;
`l<i>.mix.{q,q.b,k,k.b,g,o}`; `l<i>.mix.left.{q,k,v,q.norm,k.norm,sink,g,o}` and `l<i>.mix.right.{q,k,v,g,o,norm}`;
`l<i>.mix.{q,k,v,sink,o}`; `l<i>.mlp.{gate,up,down}` or `l<i>.mlp.{router,correction,e<j>.gate,e<j>.up,e<j>.down}`.

This file only describes; the parts it names live in `parts/` and know nothing of it.
"""
from __future__ import annotations

from ..config.lozepel import ARCHITECTURE, PRESETS, LozepelConfig
from ..config.registry import Architecture, register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec, RunSpec

NAMES = dict(q="q", k="k", v="v", o="o", gate="g", q_bias="q.b", k_bias="k.b", q_norm="q.norm", k_norm="k.norm", sink="sink")
LIGHTNING_NAMES = dict(q="q", k="k", v="v", gate="g", o="o", norm="norm")


def _softmax_mixer(cfg: LozepelConfig, m: dict, prefix: str, **options) -> PartSpec:
    params = dict(prefix=prefix, hidden_size=cfg.width, num_heads=m["heads"], num_kv_heads=m["kv_heads"], dim=m["dim"], vdim=m["vdim"],
                  scale=float(m["scale"]), eps=float(cfg.norm_eps), conv=1, names=NAMES, **options)
    rot = m.get("rot")
    if rot:
        params["position"] = PartSpec("rotary", dict(head_dim=m["dim"], rotary_dim=int(rot["dims"]), theta=float(rot["base"]),
                                                     layout="interleaved"))
    return PartSpec("normed_attention", params)


def _mixer(cfg: LozepelConfig, layer: dict) -> PartSpec:
    m = layer["mixer"]
    if layer["type"] == "attention":
        return _softmax_mixer(cfg, m, "mix.", values="keys", bias=True, qk_norm=False, gate="head", sink="zero")
    if layer["type"] == "attention_2":
        return _softmax_mixer(cfg, m, "mix.", values="projected", qk_norm=True, qk_norm_weight=False, qk_norm_where="after", gate=False,
                              sink="learned", softcap=m.get("softcap"), kv_shared=m.get("kv_from") is not None)
    right = m["right"]
    return PartSpec("parallel", dict(
        prefix="mix.", hidden_size=cfg.width,
        branches=(("left", float(m["left_scale"]), _softmax_mixer(cfg, m["left"], "left.", values="projected", qk_norm="row", gate="head",
                                                                  sink="learned")),
                  ("right", float(m["right_scale"]), PartSpec("lightning_attention", dict(
                      prefix="right.", hidden_size=cfg.width, num_heads=right["heads"], dim=right["dim"], vdim=right["vdim"],
                      decay=tuple(float(d) for d in right["decay"]), eps=float(cfg.norm_eps), names=LIGHTNING_NAMES))))))


def _feed_forward(cfg: LozepelConfig, mlp) -> PartSpec:
    if mlp is None:
        return PartSpec("none")
    if mlp["kind"] == "dense":
        return PartSpec("swiglu", dict(prefix="mlp.", hidden_size=cfg.width, intermediate_size=mlp["ff"], names=("gate", "up", "down"),
                                       activation="clamped_swish", limit=float(mlp["limit"])))
    router = mlp["router"]
    return PartSpec("routed_experts", dict(prefix="mlp.", hidden_size=cfg.width, experts=router["experts"], top=router["top"],
                                           identity=int(router.get("identity", 0)), expert_size=mlp["expert"]["ff"],
                                           expert_names=("e{}.gate", "e{}.up", "e{}.down"), router_name="router",
                                           router_bias_name="correction", scoring="softmax_all"))


def build_spec(cfg: LozepelConfig) -> ModelSpec:
    cfg.validate()
    w, eps = cfg.width, float(cfg.norm_eps)
    norm = lambda name, **more: PartSpec("rmsnorm", dict(prefix="", name=name, size=w, eps=eps, one_plus=True, **more))
    layers, order, tolerated = [], [], []
    for i, layer in enumerate(cfg.layers):
        mlp = layer.get("mlp")
        layers.append(LayerSpec(prefix=f"l{i}.",
                                block=PartSpec("sandwich_residual", dict(size=w, eps=eps, post_names=("norm1b", "norm2b"), one_plus=True)),
                                mixer_norm=norm("norm1"), mixer=_mixer(cfg, layer),
                                ffn_norm=norm("norm2", absent=mlp is None), feed_forward=_feed_forward(cfg, mlp)))
        # (run i is layer i: a layer that reads another layer's keys and values reads the cache of that layer's run)
        order.append(RunSpec(layer=i, read_cache_of=layer["mixer"].get("kv_from") if layer["type"] == "attention_2" else None))
        if mlp is None:
            tolerated += [f"l{i}.norm2", f"l{i}.norm2b"]
    embedding = dict(name="embed", vocab_size=cfg.vocab, hidden_size=w)
    if cfg.bigram:
        embedding["bigram"] = dict(name="bigram", **{k: int(cfg.bigram[k]) for k in ("buckets", "mul_prev", "mul_cur")})
    spec = ModelSpec(
        architecture=ARCHITECTURE, hidden_size=w, vocab_size=cfg.vocab, max_position=cfg.max_positions,
        embedding=PartSpec("token_embedding", embedding), position=PartSpec("none"), layers=layers, order=order,
        final_norm=norm("final.norm"),
        head=PartSpec("lm_head", dict(name="head", vocab_size=cfg.vocab, hidden_size=w, softcap=cfg.logit_softcap)),
        tolerated_tensors=tuple(tolerated))
    spec.validate()
    return spec


register_architecture(Architecture(name=ARCHITECTURE, config_class=LozepelConfig, build_spec=build_spec, presets=PRESETS), replace=True)
