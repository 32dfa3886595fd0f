"""The Fonuvik decoder as data: which parts, with which sizes, in which order.

token embedding -> rms norm -> layers of [x += norm(mixer(norm(x))); x += norm(experts(norm(x)))] -> rms norm -> head with
the embedding table.  A layer's mixer is either two mixers side by side on the same input whose results are added with
fixed weights (softmax attention in blocks of positions, q and k rotated in interleaved pairs with rescaled frequencies
and then divided by their root mean square per head; and linear attention with a decay per key channel), or a
token-shift recurrence with a bonus on the present token.  The feed-forward is routed experts with a router bias and a
shared expert that every token runs, or none.

Tensor names: `embed`, `embed.norm`, `final.norm`; layer i: `l<i>.norm1`, `.norm1b`, `.norm2`, `.norm2b`,
`l<i>.mix.left.{q,k,v,o}` and `l<i>.mix.right.{q,k,v,g,o,norm,a1,a2,a2.b}`, or
`l<i>.mix.{r,k,v,g,o,w1,w2,w0,u,norm,mu.r,mu.k,mu.v,mu.g,mu.w}`;
`l<i>.mlp.{router,router.b,e<j>.gate,e<j>.up,e<j>.down,shared.gate,shared.up,shared.down}`.

This file only describes; the parts it names live in `parts/` and know nothing of it.
"""
from __future__ import annotations

from ..config.fonuvik import ARCHITECTURE, PRESETS, FonuvikConfig, sizes_from_tensors
from ..config.registry import Architecture, register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec, RunSpec

SOFTMAX_NAMES = dict(q="q", k="k", v="v", o="o")
DECAY_NAMES = dict(q="q", k="k", v="v", gate="g", o="o", a1="a1", a2="a2", a_bias="a2.b", norm="norm")
WKV_NAMES = dict(r="r", k="k", v="v", g="g", o="o", w1="w1", w2="w2", w0="w0", u="u", norm="norm", mu_r="mu.r", mu_k="mu.k",
                 mu_v="mu.v", mu_g="mu.g", mu_w="mu.w")


def _left(cfg: FonuvikConfig, m: dict) -> PartSpec:
    params = dict(prefix="left.", hidden_size=cfg.width, num_heads=m["heads"], num_kv_heads=m["kv_heads"], dim=m["dim"],
                  vdim=m["vdim"], scale=float(m["scale"]), eps=float(cfg.norm_eps), values="projected", conv=1, gate=False,
                  qk_norm=True, qk_norm_weight=False, qk_norm_where="after", names=SOFTMAX_NAMES)
    if m.get("mask"):
        params["chunk"] = int(m["mask"]["size"])
    rot = m.get("rot")
    if rot:
        position = dict(head_dim=m["dim"], rotary_dim=int(rot["dims"]), theta=float(rot["base"]), layout="interleaved")
        if rot.get("scaling"):
            position["rescale"] = {k: float(rot["scaling"][k]) for k in ("factor", "low", "high", "original")}
        params["position"] = PartSpec("rotary", position)
    return PartSpec("normed_attention", params)


def _mixer(cfg: FonuvikConfig, layer: dict) -> PartSpec:
    m, w, eps = layer["mixer"], cfg.width, float(cfg.norm_eps)
    if layer["type"] == "wkv":
        return PartSpec("token_shift_wkv", dict(prefix="mix.", hidden_size=w, num_heads=m["heads"], dim=m["dim"], w_rank=m["w_rank"],
                                                eps=eps, names=WKV_NAMES))
    right = m["right"]
    return PartSpec("parallel", dict(
        prefix="mix.", hidden_size=w,
        branches=(("left", float(m["left_scale"]), _left(cfg, m["left"])),
                  ("right", float(m["right_scale"]), PartSpec("gated_linear_attention", dict(
                      prefix="right.", hidden_size=w, num_heads=right["heads"], dim=right["dim"], vdim=right["vdim"],
                      a_rank=right["a_rank"], tau=float(right["tau"]), eps=eps, names=DECAY_NAMES))))))


def _feed_forward(cfg: FonuvikConfig, mlp) -> PartSpec:
    if mlp is None:
        return PartSpec("none")
    params = dict(prefix="mlp.", hidden_size=cfg.width, experts=mlp["router"]["experts"], top=mlp["router"]["top"],
                  expert_size=mlp["expert"]["ff"], expert_names=("e{}.gate", "e{}.up", "e{}.down"), router_name="router",
                  router_bias_name="router.b")
    if mlp.get("shared") is not None:
        params["shared"] = PartSpec("swiglu", dict(prefix="shared.", hidden_size=cfg.width,
                                                   intermediate_size=mlp["shared"]["ff"], names=("gate", "up", "down")))
    return PartSpec("routed_experts", params)


def build_spec(cfg: FonuvikConfig) -> ModelSpec:
    cfg.validate()
    w, eps = cfg.width, float(cfg.norm_eps)
    norm = lambda name, **more: PartSpec("rmsnorm", dict(prefix="", name=name, size=w, eps=eps, **more))
    layers, tolerated = [], []
    for i, layer in enumerate(cfg.layers):
        mlp = layer.get("mlp")
        layers.append(LayerSpec(prefix=f"l{i}.",
                                block=PartSpec("sandwich_residual", dict(size=w, eps=eps, post_names=("norm1b", "norm2b"))),
                                mixer_norm=norm("norm1"), mixer=_mixer(cfg, layer),
                                ffn_norm=norm("norm2", absent=mlp is None), feed_forward=_feed_forward(cfg, mlp)))
        if mlp is None:
            tolerated += [f"l{i}.norm2", f"l{i}.norm2b"]
    spec = ModelSpec(
        architecture=ARCHITECTURE, hidden_size=w, vocab_size=cfg.vocab, max_position=cfg.max_positions,
        embedding=PartSpec("token_embedding", dict(name="embed", vocab_size=cfg.vocab, hidden_size=w, norm=("embed.norm", eps))),
        position=PartSpec("none"), layers=layers, order=[RunSpec(layer=i) for i in range(len(layers))],
        final_norm=norm("final.norm"),
        head=PartSpec("lm_head", dict(name="head", vocab_size=cfg.vocab, hidden_size=w, tied_to="embed")),
        tolerated_tensors=tuple(tolerated))
    spec.validate()
    return spec


register_architecture(Architecture(name=ARCHITECTURE, config_class=FonuvikConfig, build_spec=build_spec,
                                   presets=PRESETS, sizes_from_tensors=sizes_from_tensors), replace=True)
