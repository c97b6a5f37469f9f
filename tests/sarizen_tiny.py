"""Tiny Sarizen configurations for the tests, and random weights for them.

They differ from one another in every size and option, and avoid coincidences: head sizes differ
between keys and values, rotated dimensions are not all rotated, several experts are chosen, the
shared expert is wider than the routed ones or absent, a layer has no feed-forward, a latent layer
has no window or no frequency scaling, decay factors include 1 and a small one."""
import torch

from leone_b200.engine.model import weight_specs_for_config
from leone_b200.registry import config_from_dict
from leone_b200.weights.random_init import random_tensors


def latent(heads, dim, rot_dim, vdim, rank, scale, window=None, base=10000.0, dims=None, scaling=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "scale": scale,
         "rot": {"base": base, "dims": rot_dim if dims is None else dims}}
    if window:
        m["mask"] = {"size": window}
    if scaling:
        m["rot"]["scaling"] = scaling
    return m


def lightning(heads, dim, vdim, decay):
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay}


def moe(ff, experts, top, shared):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top},
            "shared": None if shared is None else {"ff": shared}}


YARN = {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}

TINY = {
    # window 9 (not a multiple of any page size), partial rotation with YaRN, 3 heads, two of five experts
    "P": {"architecture": "Sarizen", "vocab": 97, "width": 64, "norm": {"eps": 1e-5}, "logit_scale": 0.5, "layers": [
        {"type": "latent_attention", "mixer": latent(3, 16, 8, 24, 40, 0.2, window=9, dims=4, scaling=YARN),
         "mlp": {"kind": "dense", "ff": 96}},
        {"type": "lightning", "mixer": lightning(2, 16, 32, [0.9, 1.0]), "mlp": moe(48, 5, 2, 80)},
        {"type": "lightning", "mixer": lightning(3, 24, 16, [0.3, 0.97, 0.999]), "mlp": None},
        {"type": "latent_attention", "mixer": latent(2, 24, 16, 16, 32, 0.15, base=500.0),
         "mlp": moe(32, 4, 3, None)}]},
    # sizes that are no multiple of 8, one head, one expert of three, a window of 1 and a window past the prompts
    "Q": {"architecture": "Sarizen", "vocab": 131, "width": 72, "norm": {"eps": 3e-6}, "logit_scale": 2.0, "layers": [
        {"type": "lightning", "mixer": lightning(1, 40, 24, [0.95]), "mlp": moe(40, 3, 1, 24)},
        {"type": "latent_attention", "mixer": latent(1, 20, 12, 28, 36, 0.3, window=1, dims=12, scaling=YARN),
         "mlp": None},
        {"type": "latent_attention", "mixer": latent(5, 8, 4, 8, 24, 0.35, window=500, base=100.0),
         "mlp": {"kind": "dense", "ff": 100}}]},
    # head sizes the tensor-core paths like (64), a window of 32 over pages of 16, more experts
    "R": {"architecture": "Sarizen", "vocab": 256, "width": 128, "norm": {"eps": 1e-6}, "logit_scale": 1.0, "layers": [
        {"type": "latent_attention", "mixer": latent(4, 64, 32, 64, 64, 0.1, window=32, base=20000.0,
                                                     scaling={"factor": 5.0, "original": 128, "fast": 24.0, "slow": 2.0}),
         "mlp": moe(64, 8, 2, 64)},
        {"type": "lightning", "mixer": lightning(4, 64, 64, [0.6, 0.9, 0.99, 0.999]), "mlp": {"kind": "dense", "ff": 256}}]},
    # 18 heads (two groups of query rows on the tensor-core attention), no window on one latent layer,
    # value width 128, keys of 80 and 144 elements, a wide lightning head
    "S": {"architecture": "Sarizen", "vocab": 200, "width": 96, "norm": {"eps": 2e-6}, "logit_scale": 0.75, "layers": [
        {"type": "latent_attention", "mixer": latent(18, 16, 16, 8, 64, 0.2, base=1000.0, dims=8), "mlp": None},
        {"type": "lightning", "mixer": lightning(2, 136, 40, [0.8, 0.99]), "mlp": moe(24, 6, 6, 16)},
        {"type": "latent_attention", "mixer": latent(5, 32, 16, 32, 128, 0.12, window=70, scaling=YARN),
         "mlp": {"kind": "dense", "ff": 64}}]},
}
PAGE_TOKENS = {"P": 4, "Q": 8, "R": 16, "S": 32}


def tiny_config(which):
    return config_from_dict(TINY[which])


def tiny_tensors(which, seed=5, gain=4.0):
    """fp32 random tensors; matrices are scaled up so that scores, gates and routers are far from
    uniform and every mechanism matters to the logits."""
    specs = weight_specs_for_config(tiny_config(which))
    tensors = random_tensors(specs, seed)
    for name, t in tensors.items():
        if t.dim() == 2 and name != "embed":
            tensors[name] = t * gain
        elif name == "embed":
            tensors[name] = t * 40.0
    return tensors


def as_bf16(tensors):
    return {k: (v.to(torch.bfloat16).float() if v.dim() == 2 else v) for k, v in tensors.items()}
