"""Helpers of the Nagilix tests: small configurations, model folders with seeded weights made so that faults show,
and the error measure."""
import json
import os

import torch

from mulavik_util import TOL, rel_err, row_errs  # noqa: F401  (the same measure and 32-bit bound)


def assert_close(errs: torch.Tensor, dtype: str, what: str = "") -> None:
    """32-bit: every position within the bound; this is the sharp check.  bfloat16: a sublayer here is a chain of up
    to six rounded products (projection, step sizes, output, gate, router, experts), the test weights lean on single
    keys, and what one position rounds differently stays in the recurrent states for the positions behind it; so the
    median stays below the bound, at most one position in ten lies over twice the bound, none over eight times.  (A
    wrong key, state or expert moves every position behind it by about 1.)"""
    errs = errs.flatten()
    if dtype == "float32":
        assert float(errs.max()) <= TOL[dtype], f"{what}: {float(errs.max()):.3e} at {int(errs.argmax())}"
        return
    over = int((errs > 2 * TOL[dtype]).sum())
    assert float(errs.median()) <= TOL[dtype], f"{what}: median {float(errs.median()):.3e}"
    assert over <= max(2, len(errs) // 10), f"{what}: {over} of {len(errs)} positions over {2 * TOL[dtype]}"
    assert float(errs.max()) <= 8 * TOL[dtype], f"{what}: {float(errs.max()):.3e} at {int(errs.argmax())}"


def moe(experts=5, identity=2, top=3, ff=24, limit=0.8):
    return dict(kind="moe", expert=dict(ff=ff, limit=limit), router=dict(experts=experts, identity=identity, top=top))


def scan_layer(inner=40, state=12, dt_rank=5, conv=3, mlp=None):
    return dict(type="mamba1", mixer=dict(inner=inner, state=state, dt_rank=dt_rank, conv=conv), mlp=mlp)


def pair_layer(heads=4, kv_heads=2, dim=16, scale=None, conv=3, span=24, rot=8, base=5000.0, r_heads=3, r_dim=12,
               r_vdim=20, decay=None, r_rot=6, r_base=70000.0, mlp=None):
    left = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=dim, scale=scale if scale is not None else dim ** -0.5)
    if conv:
        left["conv"] = conv
    if span:
        left["mask"] = dict(size=span)
    if rot:
        left["rot"] = dict(dims=rot, base=base)
    right = dict(heads=r_heads, dim=r_dim, vdim=r_vdim,
                 decay=decay if decay is not None else [1.0 - 2.0 ** -(3 + 2 * h) for h in range(r_heads)])
    if r_rot:
        right["rot"] = dict(dims=r_rot, base=r_base)
    return dict(type="parallel", mixer=dict(left=left, right=right), mlp=mlp)


def config(layers, vocab=200, width=48, streams=3, eps=1e-5, logit_scale=1.7, max_positions=600):
    return dict(architecture="Nagilix", vocab=vocab, width=width, max_positions=max_positions, streams=streams,
                norm=dict(eps=eps), logit_scale=logit_scale, layers=layers)


def write_model(cfg_dict, out_dir, dtype=torch.float32, seed=1, sharpen=3.0, long_memory=False):
    """A model folder from the product's random-weights rule, then reshaped so that faults show: embeddings and
    positions of ordinary size; the weights of the query and key norms scaled so that the softmax leans on single keys
    or, where all scores are low, on the sink (queries and keys are normed, so scaling their projections would do
    nothing); temperatures and sinks spread per head; convolution taps of ordinary size; the scan's rates spread so
    that some channels forget within a few tokens and others remember for hundreds (``long_memory``: all remember); a
    router whose scores differ, with a correction large enough to move choices; the copies' weights far from one another and from
    1; the one-number norm weights far from 1."""
    from nanoinfer_b200.config import NagilixConfig
    from nanoinfer_b200.models.model import Model
    from nanoinfer_b200.registry import get_architecture
    from nanoinfer_b200.weights import random_tensors, write_safetensors

    cfg = NagilixConfig.from_dict(json.loads(json.dumps(cfg_dict)))
    model = Model(get_architecture(cfg.architecture).build_spec(cfg), cfg)
    tensors = random_tensors(model, seed, 0.02, torch.float32)
    g = torch.Generator().manual_seed(seed + 99)
    rn = lambda t, s=1.0: torch.randn(t.shape, generator=g) * s
    ru = lambda t: torch.rand(t.shape, generator=g)
    S = cfg.streams
    for name, t in tensors.items():
        leaf = name.split(".", 1)[1] if name.startswith("l") and name[1].isdigit() else name
        if name == "embed":
            t *= 50.0
        elif name == "pos":
            t *= 25.0
        elif name == "head":
            t *= 5.0
        elif leaf in ("norm1", "norm2", "final.norm"):
            t.copy_(0.4 + 1.6 * ru(t))
        elif leaf.endswith((".q.norm", ".k.norm")):
            t.copy_((1.0 + 0.3 * rn(t)) * sharpen)
        elif leaf.endswith(".temp"):
            t.copy_(0.5 + 1.5 * ru(t))
        elif leaf.endswith(".sink"):
            t.copy_(rn(t, 2.0) + 1.0)
        elif leaf.endswith(("conv", "conv.b")):
            t.copy_(rn(t, 0.5))
        elif leaf.endswith(("left.out", "right.out")):
            t.copy_(0.3 + 1.5 * ru(t))
        elif leaf.endswith("A_log"):
            t.copy_(ru(t) * 4.5 - 4.0 if not long_memory else ru(t) - 7.0)
        elif leaf.endswith("dt.b"):
            t.copy_(ru(t) * 4.0 - 3.0)
        elif leaf.endswith(".D"):
            t.copy_(rn(t))
        elif leaf.endswith(".in") and ".hc" in "." + leaf:
            t.copy_(0.3 + 0.7 * ru(t))
        elif leaf.endswith(".out") and ".hc" in "." + leaf:
            t.copy_(0.5 + rn(t, 0.5))
        elif leaf.endswith(".mix") and ".hc" in "." + leaf:
            t.copy_(0.7 * torch.eye(S) + rn(t, 0.15))
        elif leaf.startswith("rg") and leaf.endswith(".b"):
            t.copy_(rn(t))
        elif leaf.startswith("rg"):
            t *= 8.0
        elif leaf == "mlp.router":
            t *= 6.0            # (scores that differ, yet few choices that hang on the rounding of a 16-bit input)
        elif leaf == "mlp.correction":
            t.copy_(rn(t, 0.15))
        elif leaf.startswith("mlp."):
            t *= 6.0
        elif leaf.startswith("mix.") and leaf.split(".")[-1] in ("q", "k", "v", "g", "in", "x", "dt"):
            t *= 5.0
    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(out_dir, "config.json"), "w") as fh:
        json.dump(cfg.to_dict(), fh)
    write_safetensors(os.path.join(out_dir, "model.safetensors"), {k: v.to(dtype) for k, v in tensors.items()})
    return out_dir
