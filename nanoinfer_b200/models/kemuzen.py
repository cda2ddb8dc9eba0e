"""Kemuzen as a ModelSpec: a token embedding times a constant plus fixed sinusoidal positions; layers whose
sublayers read the stream itself and are normed on their OUTPUT only (``output_norm``), each with a mixer, an
optional gated SiLU feed-forward and, where the model has a second embedding table, a per-layer input gated by the
row's own token; a final norm, a head tied to the embedding table, and a soft cap on the logits.  The model's norms
are RMS norms whose weight is stored around zero.

Mixers: ``attention`` (biases, query/key norm, capped scores, a window that keeps the first tokens; a layer may read
an earlier layer's keys and values), ``delta`` (the gated delta rule), ``parallel`` (attention with a distance bias
and a per-head output gate beside a Mamba-2 recurrence).

Tensor names: ``embed``, ``side.embed``, ``final.norm``, ``l<i>.norm1``, ``l<i>.norm2``,
``l<i>.mlp.{gate, up, down}``, ``l<i>.side.{gate, proj, norm}``; attention ``l<i>.mix.{q, k, v, o}`` with
``.b`` biases and ``l<i>.mix.{q, k}.norm``; delta ``l<i>.mix.{q, k, v}`` with ``.conv`` each,
``l<i>.mix.{b, a, A_log, dt_bias, g, norm, o}``; parallel ``l<i>.mix.left.{q, k, v, q.norm, k.norm, g, o}`` and
``l<i>.mix.right.{in, conv, conv.b, dt_bias, A_log, D, norm, o}``.  Matrices are stored [out, in].
"""
from __future__ import annotations

from ..config.kemuzen import KemuzenConfig
from ..parts.base import TensorRef
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

#: the distance bias of the attention beside the recurrence: slope_h = 2^(-8 (h + 1) / heads)
DISTANCE_BIAS = 8.0


def _refs(prefix: str, names: dict) -> dict:
    return {key: TensorRef(prefix + name) for key, name in names.items()}


def _attention_args(c: int, m: dict, eps: float) -> dict:
    mask = m.get("mask") or {}
    return dict(width=c, n_head=m["heads"], n_kv_head=m.get("kv_heads") or m["heads"], head_dim=m["dim"],
                v_dim=m["vdim"], scale=float(m["scale"]), eps=eps, window=int(mask.get("size") or 0),
                keep_first=int(mask.get("keep_first") or 0), softcap=float(m.get("softcap") or 0.0), qk_norm=True)


def build_kemuzen_spec(cfg: KemuzenConfig) -> ModelSpec:
    c, eps, side = cfg.width, cfg.eps, cfg.side_dim

    def norm(name: str, one_plus: bool = True) -> PartSpec:
        return PartSpec("rmsnorm", dict(width=c, eps=eps, one_plus=one_plus), {"weight": TensorRef(name)})

    layers, schedule = [], []
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}.", layer["mixer"]
        parts = {"norm_1": norm(p + "norm1")}
        cache_of = None
        if layer["type"] == "attention":
            own = m.get("kv_from") is None
            cache_of = None if own else int(m["kv_from"])
            names = {"q_weight": "mix.q", "q_bias": "mix.q.b", "q_norm": "mix.q.norm", "out_weight": "mix.o",
                     "out_bias": "mix.o.b"}
            if own:
                names.update({"k_weight": "mix.k", "k_bias": "mix.k.b", "k_norm": "mix.k.norm", "v_weight": "mix.v",
                              "v_bias": "mix.v.b"})
            parts["mixer"] = PartSpec("normed_attention", dict(_attention_args(c, m, eps), bias=True, own_kv=own),
                                      _refs(p, names))
        elif layer["type"] == "delta":
            parts["mixer"] = PartSpec("gated_delta", dict(
                width=c, n_head=m["heads"], n_kq_head=m.get("kv_heads") or m["heads"], head_dim=m["dim"],
                v_dim=m["vdim"], taps=m["conv"], eps=eps),
                _refs(p, {"q_weight": "mix.q", "k_weight": "mix.k", "v_weight": "mix.v", "g_weight": "mix.g",
                          "b_weight": "mix.b", "a_weight": "mix.a", "q_conv": "mix.q.conv", "k_conv": "mix.k.conv",
                          "v_conv": "mix.v.conv", "A_log": "mix.A_log", "dt_bias": "mix.dt_bias",
                          "out_norm": "mix.norm", "out_weight": "mix.o"}))
        else:
            r = m["right"]
            left = dict(kind="normed_attention", args=dict(_attention_args(c, m["left"], eps), bias=False,
                                                           distance_bias=DISTANCE_BIAS, head_gate=True))
            right = dict(kind="state_space", args=dict(
                width=c, n_head=r["heads"], v_dim=r["vdim"], state=r["state"], groups=r.get("groups") or 1,
                norm_groups=r.get("norm_groups") or 1, taps=r["conv"], eps=eps))
            names = {"left.q_weight": "mix.left.q", "left.k_weight": "mix.left.k", "left.v_weight": "mix.left.v",
                     "left.q_norm": "mix.left.q.norm", "left.k_norm": "mix.left.k.norm",
                     "left.gate_weight": "mix.left.g", "left.out_weight": "mix.left.o",
                     "right.in_weight": "mix.right.in", "right.conv_weight": "mix.right.conv",
                     "right.conv_bias": "mix.right.conv.b", "right.dt_bias": "mix.right.dt_bias",
                     "right.A_log": "mix.right.A_log", "right.D": "mix.right.D", "right.out_norm": "mix.right.norm",
                     "right.out_weight": "mix.right.o"}
            parts["mixer"] = PartSpec("parallel", dict(
                width=c, left=left, right=right, left_scale=float(m.get("left_scale", 1.0)),
                right_scale=float(m.get("right_scale", 1.0))), _refs(p, names))
        mlp = layer.get("mlp")
        if mlp is not None:
            parts["norm_2"] = norm(p + "norm2")
            parts["feed_forward"] = PartSpec(
                "gated_mlp", dict(width=c, inner=mlp["ff"], activation="silu"),
                _refs(p, {"gate_weight": "mlp.gate", "up_weight": "mlp.up", "down_weight": "mlp.down"}))
        if side:
            parts["norm_3"] = norm(p + "side.norm", one_plus=False)
            parts["token_input"] = PartSpec(
                "token_gated_input", dict(width=c, dim=side, table_width=side * cfg.n_layer, offset=i * side,
                                          vocab_size=cfg.vocab, activation="tanh"),
                {"table": TensorRef("side.embed"), "gate_weight": TensorRef(p + "side.gate"),
                 "proj_weight": TensorRef(p + "side.proj")})
        layers.append(LayerSpec("output_norm", parts))
        schedule.append(ScheduleEntry(i, cache_of=cache_of))
    return ModelSpec(
        width=c,
        embedding=PartSpec("token_embedding", dict(vocab_size=cfg.vocab, width=c, scale=cfg.embedding_scale),
                           {"table": TensorRef("embed")}),
        position=PartSpec("sinusoidal", dict(width=c)),
        layers=layers,
        schedule=schedule,
        final_norm=norm("final.norm"),
        head=PartSpec("linear_head", dict(vocab_size=cfg.vocab, width=c, softcap=float(cfg.logit_softcap or 0.0)),
                      {"weight": TensorRef("embed")}),
        max_positions=None,
    )
