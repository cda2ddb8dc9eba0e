"""Nagilix's configuration: learned absolute positions, several copies of the residual stream (hyper-connections)
with a gate on every sublayer's result, a list of layers each with a mixer of one of two kinds (Mamba's selective
scan; attention inside spans of positions beside retention) and an optional routed feed-forward, read from the
nested keys of its config.json:

    {"architecture": "Nagilix", "vocab": V, "width": C, "max_positions": P, "streams": S, "norm": {"eps": e},
     "logit_scale": s,
     "layers": [{"type": "mamba1", "mixer": {"inner": I, "state": N, "dt_rank": R, "conv": taps},
                 "mlp": {"kind": "moe", "expert": {"ff": F, "limit": L},
                         "router": {"experts": E, "identity": J, "top": K}}},
                {"type": "parallel",
                 "mixer": {"left": {"heads": H, "kv_heads": G, "dim": d, "vdim": d, "scale": s, "conv": taps,
                                    "mask": {"size": W}, "rot": {"dims": r, "base": b}},
                           "right": {"heads": H, "dim": d, "vdim": v, "decay": [..H numbers..],
                                     "rot": {"dims": r, "base": b}}},
                 "mlp": null}]}

Every size and constant comes from the file.  Left out, ``streams`` is 1, ``logit_scale`` 1, ``kv_heads`` is
``heads``, ``vdim`` is ``dim``, ``conv`` of the left mixer means no convolution, ``mask`` all keys, ``rot`` no
rotation, ``router.identity`` 0.
"""
from __future__ import annotations

import dataclasses
from typing import ClassVar, List, Optional, Tuple

from .base import ConfigError, ModelConfig, field
from .mulavik import _positive
from .vadonex import _get

MIXER_KINDS = ("mamba1", "parallel")


def _rot_keys(m: dict, bad: List[str], w: str, dim) -> None:
    if m.get("rot") is None:
        return
    dims = _get(m, "rot.dims", int, bad, w)
    _positive(m, "rot.base", float, bad, w)
    if isinstance(dims, int) and (dims < 0 or dims % 2 or (isinstance(dim, int) and dims > dim)):
        bad.append(f"{w}.rot.dims {dims} must be even, not negative and at most dim")


@dataclasses.dataclass
class NagilixConfig(ModelConfig):
    architecture_names: ClassVar[Tuple[str, ...]] = ("Nagilix",)

    vocab: int = field()
    width: int = field()
    max_positions: int = field()
    layers: list = field()
    norm: dict = field()
    streams: int = field(default=1)
    logit_scale: float = field(default=1.0)

    def validate(self) -> None:
        bad: List[str] = []
        if self.vocab <= 0 or self.width <= 0 or self.max_positions <= 0:
            bad.append("vocab, width and max_positions must be positive")
        if not 1 <= self.streams <= 8:
            bad.append(f"streams must lie between 1 and 8, got {self.streams}")
        _positive(self.norm, "eps", float, bad, "norm")
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
            if kind == "mamba1":
                for key in ("inner", "state", "dt_rank", "conv"):
                    _positive(m, key, int, bad, f"{w}.mixer")
                n = m.get("state")
                if isinstance(n, int) and n > 256:
                    bad.append(f"{w}.mixer.state {n} is larger than 256")
            else:
                if not isinstance(m.get("left"), dict) or not isinstance(m.get("right"), dict):
                    bad.append(f"{w}.mixer: expected 'left' and 'right' objects")
                    continue
                a, wl = m["left"], f"{w}.mixer.left"
                heads = _positive(a, "heads", int, bad, wl)
                g = _positive(a, "kv_heads", int, bad, wl, default=heads)
                if isinstance(heads, int) and isinstance(g, int) and g > 0 and heads % g:
                    bad.append(f"{wl}.heads {heads} must be a multiple of kv_heads {g}")
                dim = _positive(a, "dim", int, bad, wl)
                vdim = _positive(a, "vdim", int, bad, wl, default=dim)
                if isinstance(dim, int) and (dim % 2 or dim > 256):
                    bad.append(f"{wl}.dim {dim} must be even and at most 256")
                if isinstance(dim, int) and isinstance(vdim, int) and vdim != dim:
                    bad.append(f"{wl}.vdim {vdim} must equal dim {dim}: the values are the keys")
                _get(a, "scale", float, bad, wl)
                taps = _get(a, "conv", int, bad, wl, default=0)
                if isinstance(taps, int) and taps < 0:
                    bad.append(f"{wl}.conv must not be negative")
                if a.get("mask") is not None:
                    _positive(a, "mask.size", int, bad, wl)
                _rot_keys(a, bad, wl, dim)
                r, wr = m["right"], f"{w}.mixer.right"
                heads = _positive(r, "heads", int, bad, wr)
                dim = _positive(r, "dim", int, bad, wr)
                _positive(r, "vdim", int, bad, wr, default=dim)
                if isinstance(dim, int) and dim > 256:
                    bad.append(f"{wr}.dim {dim} is larger than 256")
                decay = r.get("decay")
                if not isinstance(decay, list) or (isinstance(heads, int) and len(decay) != heads) or any(
                        isinstance(d, bool) or not isinstance(d, (int, float)) or not 0.0 < d <= 1.0 for d in decay):
                    bad.append(f"{wr}.decay must list one number in (0, 1] per head")
                _rot_keys(r, bad, wr, dim)
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            if not isinstance(mlp, dict) or mlp.get("kind") != "moe":
                bad.append(f"{w}.mlp.kind must be 'moe' (or mlp null)")
                continue
            _positive(mlp, "expert.ff", int, bad, f"{w}.mlp")
            _positive(mlp, "expert.limit", float, bad, f"{w}.mlp")
            e = _positive(mlp, "router.experts", int, bad, f"{w}.mlp")
            j = _get(mlp, "router.identity", int, bad, f"{w}.mlp", default=0)
            top = _positive(mlp, "router.top", int, bad, f"{w}.mlp")
            if isinstance(j, int) and j < 0:
                bad.append(f"{w}.mlp.router.identity must not be negative")
            elif all(isinstance(v, int) for v in (e, j, top)) and top > e + j:
                bad.append(f"{w}.mlp.router.top {top} is more than the router's {e + j} outputs")
        if bad:
            raise ConfigError("config.json: " + "; ".join(bad))

    @property
    def eps(self) -> float:
        return float(self.norm["eps"])

    @property
    def n_layer(self) -> int:
        return len(self.layers)

    def to_dict(self):
        return {"architecture": self.architecture_names[0], "vocab": self.vocab, "width": self.width,
                "max_positions": self.max_positions, "streams": self.streams, "norm": dict(self.norm),
                "logit_scale": self.logit_scale, "layers": self.layers}
