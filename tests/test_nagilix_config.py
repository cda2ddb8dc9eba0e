"""Nagilix without a GPU: the configuration's reader and its errors, the model as data (parts, tensors, cache and
state needs), and the plain implementation's own checks against formulas written out element by element."""
import json
import math

import pytest
import torch

from nagilix_util import config, moe, pair_layer, scan_layer, write_model


def build(cfg_dict):
    from nanoinfer_b200.config import NagilixConfig
    from nanoinfer_b200.models.model import Model
    from nanoinfer_b200.registry import get_architecture

    cfg = NagilixConfig.from_dict(json.loads(json.dumps(cfg_dict)))
    return Model(get_architecture(cfg.architecture).build_spec(cfg), cfg)


def test_the_architecture_is_registered():
    from nanoinfer_b200 import architectures
    from nanoinfer_b200.config.base import architecture_name

    assert {"Nagilix", "Kemuzen", "Mulavik", "Vadonex", "GPT2LMHeadModel"} <= set(architectures())
    assert architecture_name({"architecture": "Nagilix"}) == "Nagilix"


def test_all_problems_of_a_configuration_come_in_one_error():
    from nanoinfer_b200.config import ConfigError, NagilixConfig

    bad = config([pair_layer(heads=3, kv_heads=2), scan_layer(), dict(type="conv", mixer={}),
                  scan_layer(mlp=moe(experts=2, identity=1, top=4)), pair_layer(dim=8, rot=10),
                  pair_layer(r_heads=2, decay=[0.5, 1.5]), pair_layer(mlp=dict(kind="dense", ff=8))], streams=9)
    del bad["layers"][1]["mixer"]["dt_rank"]
    bad["layers"][4]["mixer"]["left"]["vdim"] = 12
    bad["norm"] = {}
    with pytest.raises(ConfigError) as e:
        NagilixConfig.from_dict(bad)
    text = str(e.value)
    for piece in ("norm.eps", "streams", "layers[0].mixer.left.heads", "layers[1].mixer.dt_rank", "layers[2].type",
                  "router.top", "layers[4].mixer.left.rot.dims", "layers[4].mixer.left.vdim", "layers[5].mixer.right.decay",
                  "layers[6].mlp.kind"):
        assert piece in text, (piece, text)


def test_defaults_of_keys_that_may_be_left_out():
    cfg = config([pair_layer(conv=0, span=0, rot=0, r_rot=0, mlp=moe(identity=0))])
    left, right = cfg["layers"][0]["mixer"]["left"], cfg["layers"][0]["mixer"]["right"]
    del left["kv_heads"], left["vdim"], right["vdim"], cfg["streams"], cfg["logit_scale"]
    del cfg["layers"][0]["mlp"]["router"]["identity"]
    m = build(cfg)
    att, ret = m.layers[0].mixer.children["left"], m.layers[0].mixer.children["right"]
    assert att.n_kv_head == att.n_head and att.span == 0 and att.taps == 0 and att.rotary.dims == 0
    assert att.state_spec() is None and ret.n_val == ret.n_key and ret.rotary.dims == 0
    assert m.layers[0].streams == 1 and m.head.scale == 1.0 and m.layers[0].feed_forward.n_identity == 0


def test_parts_tensors_cache_and_state_of_a_mixed_stack():
    from nanoinfer_b200.cache import CacheManager
    from nanoinfer_b200.kernels.ops import gated_scan_state_floats, selective_scan_padded

    layers = [scan_layer(inner=40, state=12, dt_rank=5, conv=3, mlp=moe(experts=5, identity=2, top=3, ff=24)),
              pair_layer(heads=4, kv_heads=2, dim=16, conv=3, span=24, r_heads=3, r_dim=12, r_vdim=20, mlp=None),
              pair_layer(heads=2, kv_heads=1, dim=40, conv=0, span=0, r_heads=1, r_dim=64, r_vdim=8, mlp=moe(identity=0, top=1))]
    m = build(config(layers, vocab=99, width=64, streams=3))
    kinds = [type(b).__name__ for b in m.layers]
    assert kinds == ["HyperConnectionBlock"] * 3 and all(b.streams == 3 for b in m.layers)
    assert m.layers[1].feed_forward is None and m.layers[0].feed_forward.n_routes == 7
    names = {b.ref.name: tuple(b.spec.shape) for b in m.bindings()}
    assert names["l0.norm1"] == () and names["final.norm"] == () and names["pos"] == (600, 64)
    assert names["l0.hc2.mix"] == (3, 3) and names["l0.rg1"] == (64, 64) and names["l0.rg2.b"] == (64,)
    assert names["l0.mix.x"] == (5 + 24, 40) and names["l0.mix.dt"] == (40, 5) and names["l0.mix.A_log"] == (40, 12)
    assert names["l0.mlp.router"] == (7, 64) and names["l0.mlp.correction"] == (7,) and names["l0.mlp.e4.down"] == (64, 24)
    assert names["l1.mix.left.q"] == (64, 64) and names["l1.mix.left.k"] == (32, 64) and names["l1.mix.left.q.norm"] == (64,)
    assert names["l1.mix.left.k.conv"] == (32, 3) and names["l1.mix.left.temp"] == (4,) and names["l1.mix.left.sink"] == (4,)
    assert names["l1.mix.left.o"] == (64, 64) and names["l1.mix.left.out"] == (64,) and names["l1.mix.right.out"] == (64,)
    assert names["l1.mix.right.v"] == (60, 64) and names["l1.mix.right.g"] == (60, 64) and names["l1.mix.right.o"] == (64, 60)
    assert "l1.mix.left.v" not in names and "l2.mix.left.q.conv" not in names and "l1.hc2.in" not in names
    # keys and values: the two attention sides, heads padded to 16s; every layer keeps state
    kv = dict(m.kv_needs())
    assert set(kv) == {1, 2} and (kv[1].n_kv_head, kv[1].head_dim, kv[1].window) == (2, 16, 0) and kv[2].head_dim == 48
    st = dict(m.state_needs())
    assert st[0].shape == (2 * 40 + 40 * selective_scan_padded(12),)
    conv_floats = 2 * (64 + 32)
    assert st[1].shape == (conv_floats + gated_scan_state_floats(0, 0, 3, 12, 20),)
    assert st[2].shape == (gated_scan_state_floats(0, 0, 1, 64, 8),)
    cm = CacheManager(m.kv_needs(), m.state_needs(), max_tokens=128, max_requests=2, page_size=16)
    assert len(cm.groups) == 2


def test_random_weights_fit_the_model_and_the_plain_model_reads_them(tmp_path):
    from plain_nagilix import PlainNagilix

    cfg = config([scan_layer(mlp=moe()), pair_layer(mlp=moe(top=1))], vocab=70, width=32, streams=2)
    d = write_model(cfg, str(tmp_path), torch.float32, seed=2)
    out = PlainNagilix(d).logits(list(range(30)))
    assert out.shape == (30, 70) and bool(torch.isfinite(out).all()) and float(out.std()) > 0.1


# --------------------------------------------------------------------------- the plain model against written-out formulas
def test_plain_span_attention_element_by_element():
    import plain_nagilix as P

    torch.manual_seed(0)
    n, C, H, G, d, span, eps = 11, 10, 2, 1, 4, 4, 1e-5
    m = dict(heads=H, kv_heads=G, dim=d, scale=0.7, conv=2, mask=dict(size=span), rot=dict(dims=2, base=10.0))
    w = {k: torch.randn(*s, dtype=torch.float64) for k, s in
         {"q": (H * d, C), "k": (G * d, C), "q.conv": (H * d, 2), "k.conv": (G * d, 2), "q.norm": (H * d,), "k.norm": (G * d,),
          "temp": (H,), "sink": (H,), "o": (C, H * d)}.items()}
    h = torch.randn(n, C, dtype=torch.float64)
    got = P.chunked_sink_attention(h, w, "", m, eps)
    q0, k0 = h @ w["q"].T, h @ w["k"].T
    want = torch.zeros(n, H * d, dtype=torch.float64)
    conv = lambda x, cw, t: x[t] * cw[:, 1] + (x[t - 1] * cw[:, 0] if t > 0 else 0.0)
    qc = torch.stack([conv(q0, w["q.conv"], t) for t in range(n)])
    kc = torch.stack([conv(k0, w["k.conv"], t) for t in range(n)])

    def prepared(x, wn, t, heads):
        y = x[t] / math.sqrt(float((x[t] ** 2).mean()) + eps) * wn
        y = y.view(heads, d).clone()
        a = t * 10.0 ** 0.0
        u, v = y[:, 0].clone(), y[:, 1].clone()
        y[:, 0], y[:, 1] = u * math.cos(a) - v * math.sin(a), v * math.cos(a) + u * math.sin(a)
        return y

    for i in range(n):
        qi = prepared(qc, w["q.norm"], i, H)
        for a in range(H):
            js = [j for j in range(i + 1) if j // span == i // span]
            s = torch.tensor([float(qi[a] @ prepared(kc, w["k.norm"], j, G)[0]) * 0.7 * float(w["temp"][a]) for j in js], dtype=torch.float64)
            den = torch.exp(s).sum() + math.exp(float(w["sink"][a]))
            for jj, j in enumerate(js):
                want[i, a * d:(a + 1) * d] += torch.exp(s[jj]) / den * kc[j].view(G, d)[0]
    assert float((got - want @ w["o"].T).abs().max()) < 1e-9


def test_plain_retention_and_scan_element_by_element():
    import plain_nagilix as P

    torch.manual_seed(1)
    n, C, eps = 6, 8, 1e-5
    m = dict(heads=2, dim=2, vdim=3, decay=[0.5, 0.9])
    w = {k: torch.randn(*s, dtype=torch.float64) for k, s in
         {"q": (4, C), "k": (4, C), "v": (6, C), "g": (6, C), "o": (C, 6)}.items()}
    h = torch.randn(n, C, dtype=torch.float64)
    got = P.retention(h, w, "", m, eps)
    q, k, v = (h @ w["q"].T).view(n, 2, 2), (h @ w["k"].T).view(n, 2, 2) / math.sqrt(2), (h @ w["v"].T).view(n, 2, 3)
    o = torch.zeros(n, 2, 3, dtype=torch.float64)
    for t in range(n):
        for a in range(2):
            for j in range(t + 1):
                o[t, a] += m["decay"][a] ** (t - j) * float(q[t, a] @ k[j, a]) * v[j, a]
    o = o / torch.sqrt((o ** 2).mean(-1, keepdim=True) + eps)
    g = h @ w["g"].T
    assert float((got - (o.reshape(n, 6) * g * torch.sigmoid(g)) @ w["o"].T).abs().max()) < 1e-9
    # the scan: one channel, two states, written out
    ms = dict(inner=1, state=2, dt_rank=1, conv=1)
    ws = {k: torch.randn(*s, dtype=torch.float64) for k, s in
          {"in": (2, C), "conv": (1, 1), "conv.b": (1,), "x": (5, 1), "dt": (1, 1), "dt.b": (1,), "A_log": (1, 2), "D": (1,),
           "o": (C, 1)}.items()}
    got = P.selective_scan(h, ws, "", ms)
    S, want = [0.0, 0.0], []
    for t in range(n):
        xz = ws["in"] @ h[t]
        x = float(xz[0]) * float(ws["conv"][0, 0]) + float(ws["conv.b"][0])
        x = x / (1 + math.exp(-x))
        dbc = ws["x"][:, 0] * x
        dt = math.log1p(math.exp(float(dbc[0]) * float(ws["dt"][0, 0]) + float(ws["dt.b"][0])))
        y = float(ws["D"][0]) * x
        for j in range(2):
            S[j] = math.exp(-dt * math.exp(float(ws["A_log"][0, j]))) * S[j] + dt * x * float(dbc[1 + j])
            y += S[j] * float(dbc[3 + j])
        z = float(xz[1])
        want.append(y * z / (1 + math.exp(-z)))
    assert float((got - torch.tensor(want, dtype=torch.float64)[:, None] * ws["o"][:, 0][None, :]).abs().max()) < 1e-9


def test_plain_routing_and_copies_element_by_element():
    import plain_nagilix as P

    torch.manual_seed(2)
    C, F = 6, 3
    m = dict(expert=dict(ff=F, limit=0.5), router=dict(experts=2, identity=1, top=2))
    w = {"router": torch.randn(3, C, dtype=torch.float64), "correction": torch.tensor([0.0, 0.0, 5.0], dtype=torch.float64)}
    for e in range(2):
        w.update({f"e{e}.gate": torch.randn(F, C, dtype=torch.float64), f"e{e}.up": torch.randn(F, C, dtype=torch.float64),
                  f"e{e}.down": torch.randn(C, F, dtype=torch.float64)})
    h = torch.randn(1, C, dtype=torch.float64)
    picked = []
    got = P.routed(h, w, "", m, picked)
    s = torch.softmax(w["router"] @ h[0], 0)
    assert 2 in picked[0][0].tolist()                                    # the correction makes the choice ...
    other = 0 if s[0] > s[1] else 1
    g = torch.clamp(w[f"e{other}.gate"] @ h[0], max=0.5)
    u = torch.clamp(w[f"e{other}.up"] @ h[0], -0.5, 0.5)
    want = s[2] * h[0] + s[other] * (w[f"e{other}.down"] @ (g / (1 + torch.exp(-1.702 * g)) * (u + 1)))   # ... not the weight
    assert float((got[0] - want).abs().max()) < 1e-12
