"""Tiny Malapel configurations for the tests, and random weights for them.

They differ from one another in every size and option, and avoid coincidences: key and value widths
differ, rotated dimensions are not all rotated, windows and chunks are no multiples of the page
sizes, the looped span starts at layer 0 or later and covers one layer or several, a model has no
loop at all, groups of experts are kept all or in part, heads share key/value heads in different
ratios, and a layer has no feed-forward."""
import torch

from leone_b200.engine.model import weight_specs_for_config
from leone_b200.registry import config_from_dict
from leone_b200.weights.random_init import random_tensors


def mixer(heads, kv_heads, dim, vdim, scale, rot_dims=None, base=10000.0, mask=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
         "rot": {"base": base, "dims": dim if rot_dims is None else rot_dims}}
    if mask:
        m["mask"] = {"size": mask}
    return m


def dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def moe(ff, experts, top, scale, groups=None):
    router = {"experts": experts, "top": top, "scale": scale}
    if groups:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "expert": {"ff": ff}, "router": router}


def layer(kind, m, mlp):
    return {"type": kind, "mixer": m, "mlp": mlp}


TINY = {
    # all three mixers, a loop over the first two layers, window 9 and chunk 11 over pages of 4
    "A": {"architecture": "Malapel", "vocab": 97, "width": 64, "norm": {"eps": 1e-5},
          "loop": {"start": 0, "stop": 2, "times": 3}, "layers": [
        layer("attention_3", mixer(6, 2, 16, 24, 0.2, rot_dims=8, mask=9), dense(96, 1.5)),
        layer("attention", mixer(4, 4, 24, 16, 0.15, rot_dims=24, base=500.0, mask=11), moe(48, 6, 2, 1.5, (3, 2))),
        layer("attention_2", mixer(3, 1, 16, 40, 0.25, rot_dims=4), None),
        layer("attention_2", mixer(2, 2, 32, 8, 0.1, base=100000.0), moe(32, 4, 3, 0.5))]},
    # a loop in the middle over one layer, sizes that are no multiple of 8, a window of 1, a chunk of 1,
    # every group kept, one expert of three
    "B": {"architecture": "Malapel", "vocab": 131, "width": 72, "norm": {"eps": 3e-6},
          "loop": {"start": 1, "stop": 2, "times": 2}, "layers": [
        layer("attention", mixer(1, 1, 20, 28, 0.3, rot_dims=12, mask=1), moe(36, 3, 1, 2.5, (3, 3))),
        layer("attention_3", mixer(5, 5, 12, 10, 0.35, rot_dims=6, base=100.0, mask=500), dense(100, 0.75)),
        layer("attention_3", mixer(2, 1, 36, 36, 0.2, rot_dims=36, mask=1), dense(60, 4.0)),
        layer("attention", mixer(3, 3, 8, 8, 0.4, rot_dims=2, mask=7), None)]},
    # no loop; head sizes the tensor-core paths like (64, 128, 32), a window of 32 and a chunk of 48 over
    # pages of 16, eight query heads on one key/value head
    "C": {"architecture": "Malapel", "vocab": 256, "width": 128, "norm": {"eps": 1e-6}, "layers": [
        layer("attention_2", mixer(4, 2, 64, 64, 0.125, base=20000.0), moe(64, 8, 2, 1.0, (4, 1))),
        layer("attention_3", mixer(8, 1, 32, 64, 0.18, rot_dims=16, mask=32), dense(256, 2.0)),
        layer("attention", mixer(4, 2, 128, 32, 0.09, rot_dims=64, mask=48), dense(128, 1.0)),
        layer("attention_2", mixer(2, 2, 48, 80, 0.14, rot_dims=48), moe(32, 12, 4, 2.0, (6, 3)))]},
    # the whole model looped once (the pass still starts with the injection); 18 query heads, wide heads
    "D": {"architecture": "Malapel", "vocab": 200, "width": 96, "norm": {"eps": 2e-6},
          "loop": {"start": 0, "stop": 3, "times": 1}, "layers": [
        layer("attention", mixer(18, 6, 16, 16, 0.2, rot_dims=8, base=1000.0, mask=70), None),
        layer("attention_3", mixer(2, 1, 144, 48, 0.08, rot_dims=100, mask=70), moe(24, 6, 6, 1.25, (2, 2))),
        layer("attention_2", mixer(5, 5, 32, 32, 0.17, rot_dims=16), dense(64, 2.5))]},
    # windows, chunks and the sigmoid rule at the head sizes of the tcgen05 prompt kernel (64 and 128, values as
    # wide as keys), looped, with a window and a chunk that end inside a key tile
    "E": {"architecture": "Malapel", "vocab": 180, "width": 128, "norm": {"eps": 1e-6},
          "loop": {"start": 0, "stop": 2, "times": 2}, "layers": [
        layer("attention_3", mixer(4, 2, 64, 64, 0.12, rot_dims=32, mask=40), dense(192, 3.0)),
        layer("attention", mixer(2, 1, 128, 128, 0.09, rot_dims=128, base=50000.0, mask=50), moe(48, 8, 2, 2.0, (4, 2))),
        layer("attention", mixer(6, 2, 64, 64, 0.12, rot_dims=16, mask=130), dense(96, 1.0))]},
}
PAGE_TOKENS = {"A": 4, "B": 8, "C": 16, "D": 32, "E": 16}


def tiny_config(which):
    return config_from_dict(TINY[which])


def tiny_tensors(which, seed=5, gain=4.0, raw=None):
    """fp32 random tensors; matrices are scaled up so that scores, gates and routers are far from
    uniform and every mechanism matters to the logits."""
    specs = weight_specs_for_config(config_from_dict(raw) if raw is not None else tiny_config(which))
    tensors = random_tensors(specs, seed)
    for name, t in tensors.items():
        if name == "embed":
            tensors[name] = t * 40.0
        elif name == "loop.in":
            tensors[name] = t * 25.0          # keeps the stream's size through the passes
        elif t.dim() == 2:
            tensors[name] = t * gain
    return tensors


def as_bf16(tensors):
    return {k: (v.to(torch.bfloat16).float() if v.dim() == 2 else v) for k, v in tensors.items()}
