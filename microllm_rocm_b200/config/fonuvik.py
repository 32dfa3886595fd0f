"""Typed configuration of the Fonuvik decoder, read from its own config.json keys.

  architecture          "Fonuvik"
  vocab, width          vocabulary and residual width
  norm.eps              eps of every norm of the model (the stream's rms norms and the per-head ones)
  layers[i]             type ("parallel" | "wkv"), mixer (its sizes), mlp ({kind: "moe", ...} or null for none)
  max_positions         optional: the longest sequence the engine admits (no table depends on it)

Mixer "parallel": left {heads, kv_heads, dim, vdim, scale, rot {base, dims, scaling {factor, low, high, original} | null} | null,
mask {size} | null}, right {heads, dim, vdim, tau}, left_scale, right_scale.
Mixer "wkv": heads, dim.
mlp: router {experts, top}, expert {ff}, shared {ff} | null.
The inner widths of the two-step decay projections stand in no key: they are the first extent of `<layer>.mix.right.a1`
and `<layer>.mix.w1` in the weight file (`sizes_from_tensors` writes them into the raw configuration as `a_rank` and
`w_rank`; presets name them).  Every size and constant comes from here or from a tensor's shape.
"""
from __future__ import annotations

import copy
import json
import os
from dataclasses import dataclass
from typing import Any, Dict, Mapping, Sequence, Tuple

from .matidra import _number, _positive_int
from .qwen2 import ConfigError

ARCHITECTURE = "Fonuvik"
MIXER_KINDS = ("parallel", "wkv")
DEFAULT_MAX_POSITIONS = 1 << 20


def _mapping(value, where: str) -> Mapping[str, Any]:
    if not isinstance(value, Mapping):
        raise ConfigError(f"{where} is missing")
    return value


def _check_left(left: Mapping[str, Any], where: str) -> None:
    for key in ("heads", "kv_heads", "dim", "vdim"):
        _positive_int(left.get(key), f"{where}.{key}")
    if left["heads"] % left["kv_heads"]:
        raise ConfigError(f"{where}.heads must be a multiple of kv_heads")
    _number(left.get("scale"), f"{where}.scale", positive=True)
    rot = left.get("rot")
    if rot is not None:
        _number(_mapping(rot, f"{where}.rot").get("base"), f"{where}.rot.base", positive=True)
        dims = rot.get("dims")
        if not isinstance(dims, int) or isinstance(dims, bool) or dims <= 0 or dims % 2 or dims > left["dim"]:
            raise ConfigError(f"{where}.rot.dims must be even, positive and at most dim")
        sc = rot.get("scaling")
        if sc is not None:
            for key in ("factor", "low", "high", "original"):
                _number(_mapping(sc, f"{where}.rot.scaling").get(key), f"{where}.rot.scaling.{key}", positive=True)
            if not sc["high"] > sc["low"]:
                raise ConfigError(f"{where}.rot.scaling.high must be above low")
    mask = left.get("mask")
    if mask is not None:
        _positive_int(_mapping(mask, f"{where}.mask").get("size"), f"{where}.mask.size")


@dataclass(frozen=True)
class FonuvikConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[Dict[str, Any], ...]
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
        if not self.layers:
            raise ConfigError("layers must list at least one layer")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            kind = layer.get("type")
            if kind not in MIXER_KINDS:
                raise ConfigError(f"{where}.type {kind!r} is not one of {', '.join(MIXER_KINDS)}")
            m = _mapping(layer.get("mixer"), f"{where}.mixer")
            if kind == "parallel":
                _check_left(_mapping(m.get("left"), f"{where}.mixer.left"), f"{where}.mixer.left")
                right = _mapping(m.get("right"), f"{where}.mixer.right")
                for key in ("heads", "dim", "vdim"):
                    _positive_int(right.get(key), f"{where}.mixer.right.{key}")
                _number(right.get("tau"), f"{where}.mixer.right.tau", positive=True)
                _positive_int(right.get("a_rank"), f"{where}.mixer.right.a_rank (or the shape of the matching tensor)")
                _number(m.get("left_scale"), f"{where}.mixer.left_scale"); _number(m.get("right_scale"), f"{where}.mixer.right_scale")
            else:
                _positive_int(m.get("heads"), f"{where}.mixer.heads"); _positive_int(m.get("dim"), f"{where}.mixer.dim")
                _positive_int(m.get("w_rank"), f"{where}.mixer.w_rank (or the shape of the matching tensor)")
            mlp = layer.get("mlp")
            if mlp is not None:
                if _mapping(mlp, f"{where}.mlp").get("kind") != "moe":
                    raise ConfigError(f"{where}.mlp.kind {mlp.get('kind')!r} is not 'moe'")
                router = _mapping(mlp.get("router"), f"{where}.mlp.router")
                _positive_int(router.get("experts"), f"{where}.mlp.router.experts"); _positive_int(router.get("top"), f"{where}.mlp.router.top")
                if router["top"] > router["experts"]:
                    raise ConfigError(f"{where}.mlp.router.top must be at most experts")
                _positive_int(_mapping(mlp.get("expert"), f"{where}.mlp.expert").get("ff"), f"{where}.mlp.expert.ff")
                if mlp.get("shared") is not None:
                    _positive_int(_mapping(mlp["shared"], f"{where}.mlp.shared").get("ff"), f"{where}.mlp.shared.ff")

    # ---- (de)serialisation -----------------------------------------------------------
    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "FonuvikConfig":
        missing = [k for k in ("vocab", "width", "layers", "norm") if k not in raw]
        if missing:
            raise ConfigError("config.json is missing " + ", ".join(missing))
        if not isinstance(raw["layers"], list):
            raise ConfigError("layers must be a list")
        cfg = cls(vocab=raw["vocab"], width=raw["width"], norm_eps=(raw["norm"] or {}).get("eps"),
                  layers=tuple(copy.deepcopy(l) for l in raw["layers"]),
                  max_positions=raw.get("max_positions", DEFAULT_MAX_POSITIONS), torch_dtype=raw.get("torch_dtype", "bfloat16"))
        cfg.validate()
        return cfg

    @classmethod
    def from_json(cls, path: str) -> "FonuvikConfig":
        if os.path.isdir(path):
            path = os.path.join(path, "config.json")
        with open(path, "r", encoding="utf-8") as f:
            return cls.from_dict(json.load(f))

    def to_dict(self) -> Dict[str, Any]:
        return {"architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
                "layers": [copy.deepcopy(l) for l in self.layers], "max_positions": self.max_positions,
                "torch_dtype": self.torch_dtype}

    def __hash__(self):
        return hash(json.dumps(self.to_dict(), sort_keys=True))


def sizes_from_tensors(raw: Dict[str, Any], shapes: Mapping[str, Sequence[int]]) -> Dict[str, Any]:
    """config.json completed with the sizes that only the weight file knows (tensor name -> shape)."""
    raw = copy.deepcopy(raw)
    for i, layer in enumerate(raw.get("layers") or []):
        if not isinstance(layer, dict) or not isinstance(layer.get("mixer"), dict):
            continue
        if layer.get("type") == "parallel":
            target, key, tensor = layer["mixer"].get("right"), "a_rank", f"l{i}.mix.right.a1"
        elif layer.get("type") == "wkv":
            target, key, tensor = layer["mixer"], "w_rank", f"l{i}.mix.w1"
        else:
            continue
        if isinstance(target, dict) and key not in target and tensor in shapes and len(shapes[tensor]) == 2:
            target[key] = int(shapes[tensor][0])
    return raw


# ---- presets: a tiny one for smoke runs, and two whose layers have the sizes of real models' layers ---------------
def moe(experts, top, ff, shared_ff=None):
    return {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff},
            "shared": {"ff": shared_ff} if shared_ff else None}


def wkv_layer(heads, dim, mlp, rank=None):
    return {"type": "wkv", "mixer": {"heads": heads, "dim": dim, "w_rank": rank or dim}, "mlp": mlp}


def parallel_layer(heads, kv_heads, dim, vdim, r_heads, r_dim, r_vdim, mlp, block=None, rot_dims=None, base=500000.0, scaling=None,
                   scale=None, tau=16.0, rank=None, left_scale=1.0, right_scale=1.0):
    rot = {"base": base, "dims": rot_dims, "scaling": scaling} if rot_dims else None
    return {"type": "parallel",
            "mixer": {"left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale or dim ** -0.5,
                               "rot": rot, "mask": {"size": block} if block else None},
                      "right": {"heads": r_heads, "dim": r_dim, "vdim": r_vdim, "tau": tau, "a_rank": rank or r_dim},
                      "left_scale": left_scale, "right_scale": right_scale},
            "mlp": mlp}


def _preset(vocab, width, layers):
    return {"architecture": ARCHITECTURE, "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "layers": layers}


_SLOWED = {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}
PRESETS: Dict[str, Dict[str, Any]] = {
    "fonuvik-tiny": _preset(320, 96, [wkv_layer(3, 16, moe(4, 2, 48, 64), rank=8),
                                      parallel_layer(4, 2, 32, 48, 2, 16, 32, moe(4, 2, 48, 64), block=24, rot_dims=16,
                                                     scaling={"factor": 4.0, "low": 1.0, "high": 4.0, "original": 64}, rank=8,
                                                     left_scale=1.1, right_scale=0.8),
                                      wkv_layer(3, 16, None, rank=8)]),
    "fonuvik-small": _preset(32000, 1024, [wkv_layer(16, 64, moe(16, 2, 704, 1408), rank=64),
                                           parallel_layer(16, 4, 64, 64, 8, 64, 128, moe(16, 2, 704, 1408), block=2048, rot_dims=64,
                                                          scaling=_SLOWED, rank=64),
                                           wkv_layer(16, 64, moe(16, 2, 704, 1408), rank=64),
                                           parallel_layer(16, 4, 64, 64, 8, 64, 128, moe(16, 2, 704, 1408), block=2048, rot_dims=64,
                                                          scaling=_SLOWED, rank=64)]),
    "fonuvik-3b-layers": _preset(102400, 2048, [wkv_layer(32, 64, moe(32, 4, 704, 2816), rank=64),
                                                parallel_layer(16, 4, 128, 128, 16, 64, 128, moe(32, 4, 704, 2816), block=4096,
                                                               rot_dims=128, scaling=_SLOWED, rank=64),
                                                wkv_layer(32, 64, moe(32, 4, 704, 2816), rank=64),
                                                parallel_layer(16, 4, 128, 128, 16, 64, 128, moe(32, 4, 704, 2816), block=4096,
                                                               rot_dims=128, scaling=_SLOWED, rank=64)]),
}
