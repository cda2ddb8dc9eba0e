"""Nagilix as a ModelSpec: a token embedding plus learned absolute positions; ``streams`` copies of the residual
stream (hyper-connections) with a gate on every sublayer's result; pre-norm layers whose norms are RMS norms with ONE
number as weight, each with a mixer and an optional routed feed-forward; a final norm of the copies' sum, a head of
its own and a constant on the logits.

Mixers: ``mamba1`` (the selective scan) and ``parallel``: attention inside spans of positions (a short convolution
and a norm over the whole projection on queries and keys, rotary halves, a temperature and a learned sink per head,
the keys as values) beside retention (one fixed decay per head), each side's output normed over the width, the result
half their sum.  Feed-forward: experts chosen by softmax scores plus a learned correction, weighted by the scores
themselves, some of the router's outputs standing for experts that hand their input on; an expert is a gated unit
with capped gate and value.

Tensor names: ``embed``, ``pos``, ``final.norm``, ``head``, ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.hc<q>.{in, out,
mix}`` and ``l<i>.rg<q>`` with ``.b`` (q = 1: the mixer, 2: the feed-forward); mamba1 ``l<i>.mix.{in, conv, conv.b,
x, dt, dt.b, A_log, D, o}``; parallel ``l<i>.mix.left.{q, k, q.conv, k.conv, q.norm, k.norm, temp, sink, o, out}`` and
``l<i>.mix.right.{q, k, v, g, o, out}``; ``l<i>.mlp.{router, correction}`` and ``l<i>.mlp.e<j>.{gate, up, down}``.
Matrices are stored [out, in].
"""
from __future__ import annotations

from ..config.nagilix import NagilixConfig
from ..parts.base import TensorRef
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry


def _refs(prefix: str, names: dict) -> dict:
    return {key: TensorRef(prefix + name) for key, name in names.items()}


def build_nagilix_spec(cfg: NagilixConfig) -> ModelSpec:
    c, eps, S = cfg.width, cfg.eps, cfg.streams

    def norm(name: str) -> PartSpec:
        return PartSpec("scalar_rmsnorm", dict(width=c, eps=eps), {"weight": TensorRef(name)})

    def connect(p: str, q: int) -> PartSpec:
        return PartSpec("hyper_connection", dict(width=c, streams=S, gated=True),
                        _refs(p, {"in": f"hc{q}.in", "out": f"hc{q}.out", "mix": f"hc{q}.mix", "gate_weight": f"rg{q}",
                                  "gate_bias": f"rg{q}.b"}))

    layers, schedule = [], []
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}.", layer["mixer"]
        parts = {"norm_1": norm(p + "norm1"), "connect_1": connect(p, 1)}
        if layer["type"] == "mamba1":
            parts["mixer"] = PartSpec("selective_scan", dict(
                width=c, inner=m["inner"], state=m["state"], dt_rank=m["dt_rank"], taps=m["conv"]),
                _refs(p, {"in_weight": "mix.in", "conv_weight": "mix.conv", "conv_bias": "mix.conv.b",
                          "x_weight": "mix.x", "dt_weight": "mix.dt", "dt_bias": "mix.dt.b", "A_log": "mix.A_log",
                          "D": "mix.D", "out_weight": "mix.o"}))
        else:
            a, r = m["left"], m["right"]
            taps = int(a.get("conv") or 0)
            rot_a, rot_r = a.get("rot") or {}, r.get("rot") or {}
            left = dict(kind="span_attention", args=dict(
                width=c, n_head=a["heads"], n_kv_head=a.get("kv_heads") or a["heads"], head_dim=a["dim"],
                v_dim=a.get("vdim") or a["dim"], scale=float(a["scale"]), eps=eps,
                span=int((a.get("mask") or {}).get("size") or 0), taps=taps, wide_norm=True,
                rot_dims=int(rot_a.get("dims") or 0), rot_base=float(rot_a.get("base") or 10000.0),
                values_are_keys=True, head_temperature=True, learned_sink=True))
            right = dict(kind="retention", args=dict(
                width=c, n_head=r["heads"], head_dim=r["dim"], v_dim=r.get("vdim") or r["dim"],
                decay=[float(d) for d in r["decay"]], eps=eps, rot_dims=int(rot_r.get("dims") or 0),
                rot_base=float(rot_r.get("base") or 10000.0)))
            names = {"left.q_weight": "mix.left.q", "left.k_weight": "mix.left.k", "left.q_norm": "mix.left.q.norm",
                     "left.k_norm": "mix.left.k.norm", "left.temperature": "mix.left.temp", "left.sink": "mix.left.sink",
                     "left.out_weight": "mix.left.o", "left.out_norm": "mix.left.out",
                     "right.q_weight": "mix.right.q", "right.k_weight": "mix.right.k", "right.v_weight": "mix.right.v",
                     "right.g_weight": "mix.right.g", "right.out_weight": "mix.right.o", "right.out_norm": "mix.right.out"}
            if taps > 0:
                names.update({"left.q_conv": "mix.left.q.conv", "left.k_conv": "mix.left.k.conv"})
            # the result is half the sum of the two sides' normed outputs
            parts["mixer"] = PartSpec("parallel", dict(width=c, left=left, right=right, left_scale=0.5, right_scale=0.5,
                                                       out_norm_eps=eps), _refs(p, names))
        mlp = layer.get("mlp")
        if mlp is not None:
            E, J = int(mlp["router"]["experts"]), int(mlp["router"].get("identity") or 0)
            names = {"router": "mlp.router", "choice_bias": "mlp.correction"}
            for e in range(E):
                names.update({f"expert{e}_gate": f"mlp.e{e}.gate", f"expert{e}_up": f"mlp.e{e}.up",
                              f"expert{e}_down": f"mlp.e{e}.down"})
            parts["norm_2"] = norm(p + "norm2")
            parts["connect_2"] = connect(p, 2)
            parts["feed_forward"] = PartSpec("routed_experts", dict(
                width=c, n_expert=E, top=int(mlp["router"]["top"]), inner=int(mlp["expert"]["ff"]),
                activation="swiglu_capped", act_limit=float(mlp["expert"]["limit"]), renorm=False, score="softmax",
                gated=True, choice_bias=True, n_identity=J), _refs(p, names))
        layers.append(LayerSpec("hyper_connections", parts))
        schedule.append(ScheduleEntry(i))
    return ModelSpec(
        width=c,
        embedding=PartSpec("token_embedding", dict(vocab_size=cfg.vocab, width=c), {"table": TensorRef("embed")}),
        position=PartSpec("learned_absolute", dict(n_positions=cfg.max_positions, width=c), {"table": TensorRef("pos")}),
        layers=layers,
        schedule=schedule,
        final_norm=norm("final.norm"),
        head=PartSpec("linear_head", dict(vocab_size=cfg.vocab, width=c, scale=float(cfg.logit_scale)),
                      {"weight": TensorRef("head")}),
        max_positions=cfg.max_positions,
    )
