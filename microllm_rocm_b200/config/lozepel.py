"""Typed configuration of the Lozepel decoder, read from its own config.json keys.

  architecture          "Lozepel"
  vocab, width          vocabulary and residual width
  norm.eps              eps of every norm of the model
  embedding.bigram      {buckets, mul_prev, mul_cur} | absent: a second table whose row is chosen by the token and the one before it
  logit_softcap         logits <- c * tanh(logits / c) (absent or null: none)
  layers[i]             type ("attention" | "parallel" | "attention_2"), mixer (its sizes), mlp (dense, moe, or null for none)
  max_positions         optional: the longest sequence the engine admits (no table depends on it)

Mixer "attention": heads, kv_heads, dim, vdim (= dim: the values are the projected keys), scale, rot {base, dims} | null.
Mixer "parallel": left {heads, kv_heads, dim, vdim, scale}, right {heads, dim, vdim, decay [one per head]}, left_scale, right_scale.
Mixer "attention_2": heads, kv_heads, dim, vdim, scale, softcap | null, rot {base, dims} | null, kv_from (index of an EARLIER
"attention_2" layer with projections of its own and the same head counts, widths and rotation) | absent.
mlp "dense": ff, limit.  mlp "moe": router {experts, top, identity}, expert {ff}.
Every size and constant comes from here or from a tensor's shape; nothing in the engine carries one.
"""
from __future__ import annotations

import copy
import json
import os
from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple

from .matidra import _number, _positive_int
from .qwen2 import ConfigError

ARCHITECTURE = "Lozepel"
MIXER_KINDS = ("attention", "parallel", "attention_2")
DEFAULT_MAX_POSITIONS = 1 << 20


def _mapping(value, where: str) -> Mapping[str, Any]:
    if not isinstance(value, Mapping):
        raise ConfigError(f"{where} is missing")
    return value


def _heads(m: Mapping[str, Any], where: str) -> None:
    for key in ("heads", "kv_heads", "dim", "vdim"):
        _positive_int(m.get(key), f"{where}.{key}")
    if m["heads"] % m["kv_heads"]:
        raise ConfigError(f"{where}.heads must be a multiple of kv_heads")
    _number(m.get("scale"), f"{where}.scale", positive=True)


def _rot(m: Mapping[str, Any], where: str) -> None:
    rot = m.get("rot")
    if rot is None:
        return
    _number(_mapping(rot, f"{where}.rot").get("base"), f"{where}.rot.base", positive=True)
    dims = rot.get("dims")
    if not isinstance(dims, int) or isinstance(dims, bool) or dims <= 0 or dims % 2 or dims > m["dim"]:
        raise ConfigError(f"{where}.rot.dims must be even, positive and at most dim")


@dataclass(frozen=True)
class LozepelConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[Dict[str, Any], ...]
    bigram: Optional[Dict[str, int]] = None
    logit_softcap: Optional[float] = None
    max_positions: int = DEFAULT_MAX_POSITIONS
    torch_dtype: str = "bfloat16"

    # ---- what the engine asks of any configuration ------------------------------------
    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def max_position_embeddings(self) -> int:
        return self.max_positions

    eos_token_id = None

    # ---- validation ----------------------------------------------------------------
    def validate(self) -> None:
        _positive_int(self.vocab, "vocab"); _positive_int(self.width, "width"); _positive_int(self.max_positions, "max_positions")
        _number(self.norm_eps, "norm.eps", positive=True)
        if self.bigram is not None:
            for key in ("buckets", "mul_prev", "mul_cur"):
                _positive_int(_mapping(self.bigram, "embedding.bigram").get(key), f"embedding.bigram.{key}")
        if self.logit_softcap is not None:
            _number(self.logit_softcap, "logit_softcap", positive=True)
        if not self.layers:
            raise ConfigError("layers must list at least one layer")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            kind = layer.get("type")
            if kind not in MIXER_KINDS:
                raise ConfigError(f"{where}.type {kind!r} is not one of {', '.join(MIXER_KINDS)}")
            m = _mapping(layer.get("mixer"), f"{where}.mixer")
            if kind == "attention":
                _heads(m, f"{where}.mixer"); _rot(m, f"{where}.mixer")
                if m["vdim"] != m["dim"]:
                    raise ConfigError(f"{where}.mixer.vdim must equal dim: the values are the projected keys")
            elif kind == "attention_2":
                _heads(m, f"{where}.mixer"); _rot(m, f"{where}.mixer")
                if m.get("softcap") is not None:
                    _number(m["softcap"], f"{where}.mixer.softcap", positive=True)
                src = m.get("kv_from")
                if src is not None:
                    if not isinstance(src, int) or isinstance(src, bool) or not 0 <= src < i:
                        raise ConfigError(f"{where}.mixer.kv_from must name an earlier layer")
                    other = self.layers[src]
                    if other.get("type") != "attention_2" or other["mixer"].get("kv_from") is not None:
                        raise ConfigError(f"{where}.mixer.kv_from must name an attention_2 layer with projections of its own")
                    for key in ("kv_heads", "dim", "vdim", "rot"):
                        if other["mixer"].get(key) != m.get(key):
                            raise ConfigError(f"{where}.mixer.{key} differs from layer {src}'s, whose keys and values it reads")
            else:
                left = _mapping(m.get("left"), f"{where}.mixer.left")
                _heads(left, f"{where}.mixer.left")
                right = _mapping(m.get("right"), f"{where}.mixer.right")
                for key in ("heads", "dim", "vdim"):
                    _positive_int(right.get(key), f"{where}.mixer.right.{key}")
                decay = right.get("decay")
                if not isinstance(decay, (list, tuple)) or len(decay) != right["heads"]:
                    raise ConfigError(f"{where}.mixer.right.decay must list one number per head")
                for d in decay:
                    _number(d, f"{where}.mixer.right.decay", positive=True)
                _number(m.get("left_scale"), f"{where}.mixer.left_scale"); _number(m.get("right_scale"), f"{where}.mixer.right_scale")
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            kind = _mapping(mlp, f"{where}.mlp").get("kind")
            if kind == "dense":
                _positive_int(mlp.get("ff"), f"{where}.mlp.ff"); _number(mlp.get("limit"), f"{where}.mlp.limit", positive=True)
            elif kind == "moe":
                router = _mapping(mlp.get("router"), f"{where}.mlp.router")
                _positive_int(router.get("experts"), f"{where}.mlp.router.experts"); _positive_int(router.get("top"), f"{where}.mlp.router.top")
                identity = router.get("identity", 0)
                if not isinstance(identity, int) or isinstance(identity, bool) or identity < 0:
                    raise ConfigError(f"{where}.mlp.router.identity must be a non-negative integer")
                if router["top"] > router["experts"] + identity:
                    raise ConfigError(f"{where}.mlp.router.top must be at most experts + identity")
                _positive_int(_mapping(mlp.get("expert"), f"{where}.mlp.expert").get("ff"), f"{where}.mlp.expert.ff")
            else:
                raise ConfigError(f"{where}.mlp.kind {kind!r} is not 'dense' or 'moe'")

    # ---- (de)serialisation -----------------------------------------------------------
    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "LozepelConfig":
        missing = [k for k in ("vocab", "width", "layers", "norm") if k not in raw]
        if missing:
            raise ConfigError("config.json is missing " + ", ".join(missing))
        if not isinstance(raw["layers"], list):
            raise ConfigError("layers must be a list")
        bigram = (raw.get("embedding") or {}).get("bigram")
        cfg = cls(vocab=raw["vocab"], width=raw["width"], norm_eps=(raw["norm"] or {}).get("eps"),
                  layers=tuple(copy.deepcopy(l) for l in raw["layers"]), bigram=dict(bigram) if bigram else None,
                  logit_softcap=raw.get("logit_softcap"), max_positions=raw.get("max_positions", DEFAULT_MAX_POSITIONS),
                  torch_dtype=raw.get("torch_dtype", "bfloat16"))
        cfg.validate()
        return cfg

    @classmethod
    def from_json(cls, path: str) -> "LozepelConfig":
        if os.path.isdir(path):
            path = os.path.join(path, "config.json")
        with open(path, "r", encoding="utf-8") as f:
            return cls.from_dict(json.load(f))

    def to_dict(self) -> Dict[str, Any]:
        out = {"architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
               "layers": [copy.deepcopy(l) for l in self.layers], "logit_softcap": self.logit_softcap,
               "max_positions": self.max_positions, "torch_dtype": self.torch_dtype}
        if self.bigram:
            out["embedding"] = {"bigram": dict(self.bigram)}
        return out

    def __hash__(self):
        return hash(json.dumps(self.to_dict(), sort_keys=True))


# ---- presets: a tiny one for smoke runs, and two whose layers have the sizes of real models' layers ---------------
def dense(ff, limit=7.0):
    return {"kind": "dense", "ff": ff, "limit": limit}


def moe(experts, top, ff, identity=0):
    return {"kind": "moe", "router": {"experts": experts, "top": top, "identity": identity}, "expert": {"ff": ff}}


def attention_layer(heads, kv_heads, dim, mlp, rot_dims=None, base=10000.0, scale=None):
    return {"type": "attention", "mlp": mlp,
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale or dim ** -0.5,
                      "rot": {"base": base, "dims": rot_dims} if rot_dims else None}}


def capped_layer(heads, kv_heads, dim, vdim, mlp, rot_dims=None, base=1000000.0, scale=None, softcap=50.0, kv_from=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale or dim ** -0.5, "softcap": softcap,
         "rot": {"base": base, "dims": rot_dims} if rot_dims else None}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention_2", "mixer": m, "mlp": mlp}


def parallel_layer(heads, kv_heads, dim, vdim, r_heads, r_dim, r_vdim, mlp, scale=None, left_scale=1.0, right_scale=1.0, decay=None):
    decay = decay or [1.0 - 2.0 ** (-(1 + 7.0 * h / max(1, r_heads - 1))) for h in range(r_heads)]
    return {"type": "parallel", "mlp": mlp,
            "mixer": {"left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale or dim ** -0.5},
                      "right": {"heads": r_heads, "dim": r_dim, "vdim": r_vdim, "decay": decay},
                      "left_scale": left_scale, "right_scale": right_scale}}


def _preset(vocab, width, layers, buckets):
    return {"architecture": ARCHITECTURE, "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "layers": layers,
            "embedding": {"bigram": {"buckets": buckets, "mul_prev": 36313, "mul_cur": 27191}}, "logit_softcap": 25.0}


PRESETS: Dict[str, Dict[str, Any]] = {
    "lozepel-tiny": _preset(320, 96, [attention_layer(4, 2, 16, dense(80, 3.0), rot_dims=8),
                                      parallel_layer(4, 2, 32, 48, 2, 16, 32, moe(4, 2, 48, identity=1), left_scale=1.1, right_scale=0.8),
                                      capped_layer(3, 1, 32, 16, moe(4, 2, 48, identity=1), rot_dims=16),
                                      capped_layer(3, 1, 32, 16, None, rot_dims=16, kv_from=2)], buckets=211),
    "lozepel-small": _preset(32000, 1024, [attention_layer(16, 4, 64, dense(2816), rot_dims=64),
                                           parallel_layer(16, 4, 64, 64, 8, 64, 128, moe(16, 2, 704, identity=2)),
                                           capped_layer(16, 4, 64, 64, moe(16, 2, 704, identity=2), rot_dims=64),
                                           capped_layer(16, 4, 64, 64, moe(16, 2, 704, identity=2), rot_dims=64, kv_from=2)], buckets=32749),
    "lozepel-3b-layers": _preset(102400, 2048, [attention_layer(16, 4, 128, dense(5632), rot_dims=128),
                                                parallel_layer(16, 4, 128, 128, 16, 64, 128, moe(32, 4, 704, identity=2)),
                                                capped_layer(16, 4, 128, 128, moe(32, 4, 704, identity=2), rot_dims=128),
                                                capped_layer(16, 4, 128, 128, moe(32, 4, 704, identity=2), rot_dims=128, kv_from=2)],
                                 buckets=65521),
}
