"""Kemuzen without a GPU: the configuration's reader and its errors, the model as data (parts, tensors, cache and
state needs), the cache manager's pages behind a window that keeps the first tokens, and the plain
implementation's own checks against formulas written out element by element."""
import json
import math

import pytest
import torch

from kemuzen_util import attention_layer, config, delta_layer, dense, parallel_layer, write_model


def build(cfg_dict):
    from nanoinfer_b200.config.kemuzen import KemuzenConfig
    from nanoinfer_b200.models.model import Model
    from nanoinfer_b200.registry import get_architecture

    cfg = KemuzenConfig.from_dict(json.loads(json.dumps(cfg_dict)))
    return Model(get_architecture(cfg.architecture).build_spec(cfg), cfg)


def test_the_architecture_is_registered():
    from nanoinfer_b200 import architectures

    assert {"Kemuzen", "Mulavik", "Vadonex", "GPT2LMHeadModel"} <= set(architectures())


def test_all_problems_of_a_configuration_come_in_one_error():
    from nanoinfer_b200.config import ConfigError
    from nanoinfer_b200.config.kemuzen import KemuzenConfig

    bad = config([attention_layer(heads=3, kv_heads=2), delta_layer(), dict(type="conv", mixer={}),
                  attention_layer(kv_from=1), parallel_layer(r_heads=3, groups=2), attention_layer(dim=7),
                  attention_layer(heads=2, kv_heads=2, kv_from=0), parallel_layer(r_heads=3, r_vdim=5, norm_groups=2)])
    del bad["layers"][1]["mixer"]["conv"]
    bad["layers"][5]["mixer"]["mask"]["size"] = 0
    bad["norm"] = {}
    del bad["embedding"]["scale"]
    bad["logit_softcap"] = -1.0
    bad["token_side"] = {"dim": 0}
    with pytest.raises(ConfigError) as e:
        KemuzenConfig.from_dict(bad)
    text = str(e.value)
    for piece in ("norm.eps", "embedding.scale", "logit_softcap", "token_side.dim", "layers[0].mixer.heads",
                  "layers[1].mixer.conv", "layers[2].type", "layers[3].mixer.kv_from", "layers[4].mixer.right.heads",
                  "layers[5].mixer.dim", "layers[5].mixer.mask.size", "layers[6].mixer: head counts",
                  "layers[7].mixer.right: heads * vdim"):
        assert piece in text, (piece, text)


def test_defaults_of_keys_that_may_be_left_out():
    cfg = config([attention_layer(softcap=None, window=None), delta_layer(), parallel_layer(window=None)], side=0,
                 logit_softcap=None)
    del cfg["layers"][0]["mixer"]["kv_heads"], cfg["layers"][1]["mixer"]["kv_heads"]
    for key in ("groups", "norm_groups"):
        del cfg["layers"][2]["mixer"]["right"][key]
    del cfg["layers"][2]["mixer"]["left_scale"], cfg["layers"][2]["mixer"]["right_scale"]
    m = build(cfg)
    att, delta, par = (blk.mixer for blk in m.layers)
    assert att.n_kv_head == att.n_head and att.window == 0 and att.softcap == 0.0 and att.keep_first == 0
    assert delta.n_kq == delta.n_head
    assert par.children["right"].n_kq == 1 and par.children["right"].norm_groups == 1
    assert par.left_scale == par.right_scale == 1.0 and par.children["left"].distance_bias == 8.0
    assert m.head.softcap == 0.0 and all(len(blk.sublayers) == 1 for blk in m.layers)
    assert m.kv_needs()[0][1].window == 0 and m.config.to_dict() == cfg


def test_parts_tensors_cache_and_state_of_a_mixed_stack():
    from nanoinfer_b200.cache import CacheManager
    from nanoinfer_b200.kernels.ops import gated_scan_state_floats

    layers = [delta_layer(heads=4, kv_heads=2, dim=24, vdim=40, conv=3, mlp=dense(80)),
              attention_layer(heads=4, kv_heads=2, dim=16, vdim=40, window=30, keep_first=2, mlp=None),
              parallel_layer(heads=4, kv_heads=1, dim=48, vdim=8, window=20, r_heads=6, r_vdim=10, state=20, groups=2,
                             norm_groups=3, conv=4, mlp=dense(32)),
              attention_layer(heads=4, kv_heads=2, dim=16, vdim=40, window=50, keep_first=7, kv_from=1, mlp=dense(16)),
              attention_layer(heads=4, kv_heads=2, dim=16, vdim=40, window=10, keep_first=None, kv_from=1, mlp=None)]
    m = build(config(layers, vocab=99, width=64, side=6))
    names = {b.ref.name: tuple(b.spec.shape) for b in m.bindings()}
    assert names["embed"] == (99, 64) and names["side.embed"] == (99, 30) and names["final.norm"] == (64,)
    assert names["l0.mix.q"] == (48, 64) and names["l0.mix.v"] == (160, 64) and names["l0.mix.q.conv"] == (48, 3)
    assert names["l0.mix.b"] == names["l0.mix.a"] == (4, 64) and names["l0.mix.A_log"] == names["l0.mix.dt_bias"] == (4,)
    assert names["l0.mix.norm"] == (40,) and names["l0.mix.o"] == (64, 160) and names["l0.mlp.gate"] == (80, 64)
    assert names["l1.mix.q.b"] == (64,) and names["l1.mix.k.norm"] == (16,) and names["l1.mix.o.b"] == (64,)
    assert names["l2.mix.left.g"] == (4, 64) and names["l2.mix.left.k"] == (48, 64)
    assert names["l2.mix.right.in"] == (60 + 60 + 40 + 40 + 6, 64) and names["l2.mix.right.conv"] == (140, 4)
    assert names["l2.mix.right.conv.b"] == (140,) and names["l2.mix.right.norm"] == (60,) and names["l2.mix.right.D"] == (6,)
    assert names["l3.side.gate"] == (6, 64) and names["l3.side.proj"] == (64, 6) and names["l3.side.norm"] == (64,)
    assert not any(n.startswith(("l3.mix.k", "l3.mix.v", "l4.mix.k", "l4.mix.v")) for n in names)
    assert "l1.norm2" not in names and "l2.norm2" in names
    # layer 1 owns the pages that 3 and 4 read: kept for the widest window and the most first tokens of the three
    kv = dict(m.kv_needs())
    assert sorted(kv) == [1, 2] and (kv[1].window, kv[1].keep_first, kv[1].head_dim, kv[1].n_kv_head) == (50, 7, 48, 2)
    assert (kv[2].window, kv[2].keep_first, kv[2].head_dim, kv[2].n_kv_head) == (20, 0, 48, 1)
    assert [e.cache_of for e in m.schedule] == [None, None, None, 1, 1]
    st = dict(m.state_needs())
    assert sorted(st) == [0, 2]
    assert st[0].shape == (gated_scan_state_floats(3, 2 * 48 + 160, 4, 24, 40),) == (2 * 256 + 4 * 40 * 32,)
    assert st[2].shape == (gated_scan_state_floats(4, 140, 6, 20, 10),) == (420 + 6 * 10 * 32,)
    assert m.capture_safe()
    cache = CacheManager(m.kv_needs(), m.state_needs(), max_tokens=256, max_requests=2)
    assert len(cache.groups) == 2


def test_pages_behind_a_window_go_back_but_those_of_the_kept_tokens_stay():
    from nanoinfer_b200.cache import CacheManager
    from nanoinfer_b200.parts.base import KVCacheSpec

    cache = CacheManager([(0, KVCacheSpec(1, 16, window=40, keep_first=18)), (1, KVCacheSpec(1, 16, window=40))], [],
                         max_tokens=160, max_requests=2, page_size=16)
    r = cache.open_request()
    for n in (50, 1, 1, 30, 1, 60, 1):
        cache.append([(r, n)])
        cache.commit(r, n)
        cache.check()
        first = max(0, r.n_tokens - 40 + 1) // 16
        held = [[b for b, p in enumerate(blocks) if p >= 0] for blocks in r.blocks]
        last = (r.n_tokens - 1) // 16
        assert held[1] == list(range(first, last + 1))
        assert held[0] == sorted(set([0, 1]) | set(range(first, last + 1)))
    assert r.n_tokens == 144 and cache.pages_used() == [5, 3]
    cache.close_request(r)
    assert cache.pages_used() == [0, 0]


def test_the_plain_model_against_formulas_written_out(tmp_path):
    from plain_kemuzen import PlainKemuzen, capped_attention, distance_attention, short_conv, sinusoid, visible

    assert visible(6, 3, 1).tolist() == [[True, False, False, False, False, False], [True, True, False, False, False, False],
                                         [True, True, True, False, False, False], [True, True, True, True, False, False],
                                         [True, False, True, True, True, False], [True, False, False, True, True, True]]
    s = sinusoid(torch.tensor([0, 3]), 6)
    assert s[0].tolist() == [0, 1, 0, 1, 0, 1] and abs(float(s[1, 2]) - math.sin(3 * 10000 ** (-2 / 6))) < 1e-12
    x, w = torch.arange(8.0, dtype=torch.float64).view(4, 2), torch.tensor([[1.0, 10.0, 100.0], [0.0, 0.0, 1.0]], dtype=torch.float64)
    assert short_conv(x, w).tolist() == [[0.0, 1.0], [200.0, 3.0], [420.0, 5.0], [642.0, 7.0]]
    assert short_conv(x[2:], w, before=x[:2]).tolist() == [[420.0, 5.0], [642.0, 7.0]]
    # one attention head by hand: two tokens, a cap, biases
    torch.manual_seed(0)
    W = {k: torch.randn(*shape, dtype=torch.float64) for k, shape in
         {"q": (4, 4), "k": (4, 4), "v": (4, 4), "o": (4, 4), "q.b": (4,), "k.b": (4,), "v.b": (4,), "o.b": (4,),
          "q.norm": (4,), "k.norm": (4,), "g": (1, 4)}.items()}
    h = torch.randn(2, 4, dtype=torch.float64)
    m = dict(heads=1, kv_heads=1, dim=4, vdim=4, scale=0.7, softcap=2.0)
    unit = lambda v, wt: v / math.sqrt(float((v * v).mean()) + 1e-5) * wt
    q = [unit(W["q"] @ h[i] + W["q.b"], W["q.norm"]) for i in range(2)]
    k = [unit(W["k"] @ h[i] + W["k.b"], W["k.norm"]) for i in range(2)]
    v = [W["v"] @ h[i] + W["v.b"] for i in range(2)]
    s = [2.0 * math.tanh(float(q[1] @ k[j]) * 0.7 / 2.0) for j in range(2)]
    p = [math.exp(s[j]) / (math.exp(s[0]) + math.exp(s[1])) for j in range(2)]
    want = W["o"] @ (p[0] * v[0] + p[1] * v[1]) + W["o.b"]
    got = capped_attention(h, W, "", m, 1e-5)
    assert float((got[1] - want).abs().max()) < 1e-12 and float((got[0] - (W["o"] @ v[0] + W["o.b"])).abs().max()) < 1e-12
    # the distance bias: one head, slope 2^-8; the gate
    del m["softcap"]
    kk = [unit(W["k"] @ h[i], W["k.norm"]) for i in range(2)]
    qq = unit(W["q"] @ h[1], W["q.norm"])
    s = [float(qq @ kk[0]) * 0.7 - 2.0 ** -8 * 1, float(qq @ kk[1]) * 0.7]
    p = [math.exp(s[j]) / (math.exp(s[0]) + math.exp(s[1])) for j in range(2)]
    gate = 1 / (1 + math.exp(-float(W["g"][0] @ h[1])))
    want = W["o"] @ ((p[0] * (W["v"] @ h[0]) + p[1] * (W["v"] @ h[1])) * gate)
    assert float((distance_attention(h, W, "", m, 1e-5)[1] - want).abs().max()) < 1e-12
    # a whole model: a sequence's logits do not depend on what follows, and greedy decoding repeats itself
    d = write_model(config([delta_layer(mlp=dense()), parallel_layer(), attention_layer()], vocab=60, width=32), str(tmp_path))
    plain = PlainKemuzen(d)
    t = list(range(5, 45))
    full = plain.logits(t)
    assert float((plain.logits(t[:17]) - full[:17]).abs().max()) < 1e-9
    assert plain.greedy(t[:9], 4) == plain.greedy(t[:9], 6)[:4]
    assert float(full.abs().max()) <= 25.0 and float(full.std()) > 0.5
