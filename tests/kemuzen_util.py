"""Helpers of the Kemuzen tests: small configurations, model folders with seeded weights made so that faults
show, and the error measure."""
import json
import os

import torch

from mulavik_util import TOL, assert_close, rel_err, row_errs  # noqa: F401  (the same measure and bounds)


def dense(ff=48):
    return dict(kind="dense", ff=ff)


def attention_layer(heads=4, kv_heads=2, dim=16, vdim=16, scale=None, softcap=12.0, window=24, keep_first=3,
                    kv_from=None, mlp=None):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale if scale is not None else dim ** -0.5)
    if softcap:
        m["softcap"] = softcap
    if window:
        m["mask"] = dict(size=window)
        if keep_first is not None:
            m["mask"]["keep_first"] = keep_first
    if kv_from is not None:
        m["kv_from"] = kv_from
    return dict(type="attention", mixer=m, mlp=mlp)


def delta_layer(heads=2, kv_heads=2, dim=16, vdim=24, conv=4, mlp=None):
    return dict(type="delta", mixer=dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, conv=conv), mlp=mlp)


def parallel_layer(heads=4, kv_heads=1, dim=16, vdim=16, scale=None, window=20, r_heads=3, r_vdim=16, state=16,
                   groups=1, norm_groups=1, conv=4, left_scale=1.3, right_scale=0.6, mlp=None):
    left = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale if scale is not None else dim ** -0.5)
    if window:
        left["mask"] = dict(size=window)
    right = dict(heads=r_heads, vdim=r_vdim, state=state, groups=groups, norm_groups=norm_groups, conv=conv)
    return dict(type="parallel", mixer=dict(left=left, right=right, left_scale=left_scale, right_scale=right_scale),
                mlp=mlp)


def config(layers, vocab=200, width=64, scale=4.0, eps=1e-5, logit_softcap=25.0, side=8):
    out = dict(architecture="Kemuzen", vocab=vocab, width=width, embedding=dict(scale=scale), norm=dict(eps=eps),
               layers=layers)
    if logit_softcap:
        out["logit_softcap"] = logit_softcap
    if side:
        out["token_side"] = dict(dim=side)
    return out


def write_model(cfg_dict, out_dir, dtype=torch.float32, seed=1, sharpen=3.0, long_memory=False):
    """A model folder from the product's random-weights rule, then reshaped so that faults show: embeddings of
    ordinary size; the weights of the query and key norms scaled so that the softmax leans on single keys (queries
    and keys are normed, so scaling their projections would do nothing); biases, gates and convolution taps of
    ordinary size; the rates of the recurrences spread so that some heads forget within a few tokens and others
    remember for hundreds (``long_memory``: all remember); norm weights that are stored around zero far enough from
    it that a missing one shows."""
    from nanoinfer_b200.config.kemuzen import KemuzenConfig
    from nanoinfer_b200.models.model import Model
    from nanoinfer_b200.registry import get_architecture
    from nanoinfer_b200.weights import random_tensors, write_safetensors

    cfg = KemuzenConfig.from_dict(json.loads(json.dumps(cfg_dict)))
    model = Model(get_architecture(cfg.architecture).build_spec(cfg), cfg)
    tensors = random_tensors(model, seed, 0.02, torch.float32)
    g = torch.Generator().manual_seed(seed + 99)
    for name, t in tensors.items():
        leaf = name.split(".", 1)[1] if name.startswith("l") and name[1].isdigit() else name
        if name == "embed":
            t *= 50.0 / abs(cfg.embedding_scale)
        elif name == "side.embed":
            t *= 50.0
        elif leaf in ("norm1", "norm2", "final.norm"):
            t *= 15.0                                    # stored around zero: 1 + w between 0.1 and 1.9
        elif leaf.endswith((".q.norm", ".k.norm")):
            t.copy_((1.0 + 0.3 * torch.randn(t.shape, generator=g)) * sharpen)
        elif leaf.endswith(".b") and not leaf.endswith(("mix.b", "conv.b")):
            t.copy_(torch.randn(t.shape, generator=g) * 0.5)       # biases of q, k, v, o
        elif leaf.endswith(("conv", "conv.b")):
            t.copy_(torch.randn(t.shape, generator=g) * 0.5)
        elif leaf.endswith("A_log"):
            t.copy_(torch.rand(t.shape, generator=g) * 4.5 - 4.0)
            if long_memory:
                t.copy_(torch.rand(t.shape, generator=g) - 7.0)
        elif leaf.endswith("dt_bias"):
            t.copy_(torch.rand(t.shape, generator=g) * 4.0 - 3.0)
        elif leaf.endswith(".D"):
            t.copy_(torch.randn(t.shape, generator=g))
        elif leaf in ("mix.b", "mix.a", "mix.g", "mix.left.g"):
            t *= 10.0
        elif leaf.startswith(("mlp.", "side.")) and not leaf.endswith("norm"):
            t *= 5.0
        elif leaf.startswith("mix.") and leaf.split(".")[-1] in ("q", "k", "v", "in"):
            t *= 5.0
    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(out_dir, "config.json"), "w") as fh:
        json.dump(cfg.to_dict(), fh)
    write_safetensors(os.path.join(out_dir, "model.safetensors"), {k: v.to(dtype) for k, v in tensors.items()})
    return out_dir
