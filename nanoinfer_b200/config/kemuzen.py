"""Kemuzen's configuration: a list of layers, each with a mixer of one of three kinds (attention with a soft cap on
its scores and a window that keeps the first tokens; the gated delta rule; attention with a distance bias beside a
Mamba-2 recurrence) and an optional gated feed-forward, read from the nested keys of its config.json:

    {"architecture": "Kemuzen", "vocab": V, "width": C, "embedding": {"scale": s}, "norm": {"eps": e},
     "logit_softcap": c, "token_side": {"dim": D},
     "layers": [{"type": "attention",
                 "mixer": {"heads": H, "kv_heads": G, "dim": d, "vdim": v, "scale": s, "softcap": c,
                           "mask": {"size": W, "keep_first": K}, "kv_from": j},
                 "mlp": {"kind": "dense", "ff": F}},
                {"type": "delta", "mixer": {"heads": H, "kv_heads": G, "dim": d, "vdim": v, "conv": taps}, "mlp": ...},
                {"type": "parallel",
                 "mixer": {"left": {"heads": H, "kv_heads": G, "dim": d, "vdim": v, "scale": s, "mask": {"size": W}},
                           "right": {"heads": H, "vdim": v, "state": N, "groups": G, "norm_groups": P, "conv": taps},
                           "left_scale": a, "right_scale": b},
                 "mlp": null}]}

Every size and constant comes from the file.  Left out, ``kv_heads`` is ``heads``, ``softcap`` and ``logit_softcap``
mean no cap, ``mask`` all keys, ``mask.keep_first`` 0, ``kv_from`` keys and values of the layer's own,
``token_side`` no per-layer token input, ``left_scale`` and ``right_scale`` 1.
"""
from __future__ import annotations

import dataclasses
from typing import ClassVar, List, Optional, Tuple

from .base import ConfigError, ModelConfig, field
from .mulavik import _positive
from .vadonex import _get

MIXER_KINDS = ("attention", "delta", "parallel")


def _attention_keys(m: dict, bad: List[str], w: str) -> None:
    heads = _positive(m, "heads", int, bad, w)
    g = _positive(m, "kv_heads", int, bad, w, default=heads)
    if isinstance(heads, int) and isinstance(g, int) and g > 0 and heads % g:
        bad.append(f"{w}.heads {heads} must be a multiple of kv_heads {g}")
    for key in ("dim", "vdim"):
        v = _positive(m, key, int, bad, w)
        if isinstance(v, int) and v % 2:
            bad.append(f"{w}.{key} {v} must be even")
    _get(m, "scale", float, bad, w)
    cap = _get(m, "softcap", float, bad, w, default=None)
    if cap is not None and not cap > 0.0:
        bad.append(f"{w}.softcap must be positive, got {cap}")
    if m.get("mask") is not None:
        _positive(m, "mask.size", int, bad, w)
        keep = _get(m, "mask.keep_first", int, bad, w, default=0)
        if isinstance(keep, int) and keep < 0:
            bad.append(f"{w}.mask.keep_first must not be negative")


@dataclasses.dataclass
class KemuzenConfig(ModelConfig):
    architecture_names: ClassVar[Tuple[str, ...]] = ("Kemuzen",)

    vocab: int = field()
    width: int = field()
    layers: list = field()
    norm: dict = field()
    embedding: dict = field()
    logit_softcap: Optional[float] = field(default=None)
    token_side: Optional[dict] = field(default=None)

    def validate(self) -> None:
        bad: List[str] = []
        if self.vocab <= 0 or self.width <= 0:
            bad.append("vocab and width must be positive")
        _positive(self.norm, "eps", float, bad, "norm")
        _get(self.embedding, "scale", float, bad, "embedding")
        if self.logit_softcap is not None and (isinstance(self.logit_softcap, bool)
                                               or not isinstance(self.logit_softcap, (int, float))
                                               or not self.logit_softcap > 0):
            bad.append(f"logit_softcap must be a positive number, got {self.logit_softcap!r}")
        if self.token_side is not None:
            if not isinstance(self.token_side, dict):
                bad.append("token_side: expected an object with 'dim'")
            else:
                _positive(self.token_side, "dim", int, bad, "token_side")
        if not self.layers:
            bad.append("layers: at least one layer is needed")
        for i, layer in enumerate(self.layers):
            w = f"layers[{i}]"
            if not isinstance(layer, dict) or not isinstance(layer.get("mixer"), dict):
                bad.append(f"{w}: expected an object with 'type', 'mixer' and 'mlp'")
                continue
            kind, m = layer.get("type"), layer["mixer"]
            if kind not in MIXER_KINDS:
                bad.append(f"{w}.type {kind!r} is not one of {MIXER_KINDS}")
                continue
            if kind == "attention":
                _attention_keys(m, bad, f"{w}.mixer")
                j = m.get("kv_from")
                if j is not None:
                    ok = isinstance(j, int) and not isinstance(j, bool) and 0 <= j < i \
                        and isinstance(self.layers[j], dict) and self.layers[j].get("type") == "attention" \
                        and isinstance(self.layers[j].get("mixer"), dict) \
                        and self.layers[j]["mixer"].get("kv_from") is None
                    if not ok:
                        bad.append(f"{w}.mixer.kv_from {j!r} must name an earlier attention layer with keys and "
                                   "values of its own")
                    else:
                        o = self.layers[j]["mixer"]
                        same = all(m.get(k, m.get("heads") if k == "kv_heads" else None)
                                   == o.get(k, o.get("heads") if k == "kv_heads" else None)
                                   for k in ("heads", "kv_heads", "dim", "vdim"))
                        if not same:
                            bad.append(f"{w}.mixer: head counts and sizes must equal those of layer {j}, whose keys "
                                       "and values it reads")
            elif kind == "delta":
                heads = _positive(m, "heads", int, bad, f"{w}.mixer")
                g = _positive(m, "kv_heads", int, bad, f"{w}.mixer", default=heads)
                if isinstance(heads, int) and isinstance(g, int) and g > 0 and heads % g:
                    bad.append(f"{w}.mixer.heads {heads} must be a multiple of kv_heads {g}")
                for key in ("dim", "vdim", "conv"):
                    _positive(m, key, int, bad, f"{w}.mixer")
            else:
                if not isinstance(m.get("left"), dict) or not isinstance(m.get("right"), dict):
                    bad.append(f"{w}.mixer: expected 'left' and 'right' objects")
                    continue
                _attention_keys(m["left"], bad, f"{w}.mixer.left")
                r, wr = m["right"], f"{w}.mixer.right"
                heads = _positive(r, "heads", int, bad, wr)
                vdim = _positive(r, "vdim", int, bad, wr)
                _positive(r, "state", int, bad, wr)
                _positive(r, "conv", int, bad, wr)
                groups = _positive(r, "groups", int, bad, wr, default=1)
                parts = _positive(r, "norm_groups", int, bad, wr, default=1)
                if isinstance(heads, int) and isinstance(groups, int) and groups > 0 and heads % groups:
                    bad.append(f"{wr}.heads {heads} must be a multiple of groups {groups}")
                if all(isinstance(v, int) and v > 0 for v in (heads, vdim, parts)) and (heads * vdim) % parts:
                    bad.append(f"{wr}: heads * vdim must be a multiple of norm_groups {parts}")
                _get(m, "left_scale", float, bad, f"{w}.mixer", default=1.0)
                _get(m, "right_scale", float, bad, f"{w}.mixer", default=1.0)
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            if not isinstance(mlp, dict) or mlp.get("kind") != "dense":
                bad.append(f"{w}.mlp.kind must be 'dense' (or mlp null)")
                continue
            _positive(mlp, "ff", int, bad, f"{w}.mlp")
        if bad:
            raise ConfigError("config.json: " + "; ".join(bad))

    @property
    def eps(self) -> float:
        return float(self.norm["eps"])

    @property
    def embedding_scale(self) -> float:
        return float(self.embedding["scale"])

    @property
    def side_dim(self) -> int:
        return int(self.token_side["dim"]) if self.token_side is not None else 0

    @property
    def n_layer(self) -> int:
        return len(self.layers)

    def to_dict(self):
        out = {"architecture": self.architecture_names[0], "vocab": self.vocab, "width": self.width,
               "embedding": dict(self.embedding), "norm": dict(self.norm), "layers": self.layers}
        if self.logit_softcap is not None:
            out["logit_softcap"] = self.logit_softcap
        if self.token_side is not None:
            out["token_side"] = dict(self.token_side)
        return out
