"""The Malapel decoder through the engine against the plain implementation (tests/plain/malapel.py).

Without a GPU the engine runs on the stand-in kernels (tests/emulated_ops.py), which checks the
configuration, the model description, the loop's run order and injections, the parts' use of the
cache, and the step function's cutting and batching; on a B200 the same traces run on the CUDA
kernels in 32-bit and in bfloat16, together with tests that aim at single mechanisms."""
import copy
import os

import numpy as np
import pytest
import torch

from leone_b200.engine.engine import Engine
from leone_b200.registry import config_from_dict, spec_from_config
from tests import replay
from tests.malapel_tiny import PAGE_TOKENS, TINY, as_bf16, dense, layer, mixer, moe, tiny_config, tiny_tensors
from tests.plain import malapel as plain

FP32 = dict(rtol=3e-5, atol_scale=3e-5)
# bfloat16: the gained weights make scores and routers sharp, which also amplifies rounding; the 32-bit
# runs are the sharp tests, these catch a wrong path or operand
BF16 = dict(rtol=1e-1, atol_scale=1e-1)
LENGTHS = [40, 7, 75, 33, 1, 64, 50]


def _plain(which, tensors, bf16=False, raw=None):
    return plain.PlainMalapel(raw or TINY[which], as_bf16(tensors) if bf16 else tensors)


def _engine(which, tensors, dtype, device, ops=None, max_tokens=512, page=None, raw=None, **kw):
    spec = spec_from_config(config_from_dict(raw) if raw is not None else tiny_config(which))
    return Engine(spec, dict(tensors), dtype=dtype, device=device, ops=ops, page_tokens=page or PAGE_TOKENS[which],
                  max_tokens=max_tokens, max_requests=kw.pop("max_requests", 4),
                  max_batch_tokens=kw.pop("max_batch_tokens", 128), **kw)


def _requests(vocab, lengths=LENGTHS, seed=100):
    return {f"r{i}": replay.random_tokens(vocab, n, seed + i) for i, n in enumerate(lengths)}


def _traces(reqs):
    return {"whole": replay.trace_whole(reqs), "tail": replay.trace_decode_tail(reqs, tail=20),
            "portions": replay.trace_portions(reqs), "mixed": replay.trace_mixed(reqs, seed=3)}


def _one_layer(kind, m, mlp=None, vocab=64, width=32, loop=None):
    raw = {"architecture": "Malapel", "vocab": vocab, "width": width, "norm": {"eps": 1e-6},
           "layers": [layer(kind, m, mlp)]}
    if loop:
        raw["loop"] = loop
    return raw


def _random(raw, seed, gain=5.0):
    from leone_b200.engine.model import weight_specs_for_config
    from leone_b200.weights.random_init import random_tensors
    tensors = random_tensors(weight_specs_for_config(config_from_dict(raw)), seed)
    return {k: (v * gain if v.dim() == 2 and k != "loop.in" else (v * 25.0 if k == "loop.in" else v))
            for k, v in tensors.items()}


# -- configuration and description (CPU) ---------------------------------------------------------
def test_config_round_trip_and_spec():
    for which, raw in TINY.items():
        cfg = config_from_dict(raw)
        assert cfg.to_json_dict() == raw
        spec = spec_from_config(cfg)
        assert all(ls.mixer.kind == "attention" and ls.block == "pre_norm" for ls in spec.layers)
        assert [ls.feed_forward is None for ls in spec.layers] == [e["mlp"] is None for e in raw["layers"]]
        assert [(i, pos in dict(spec.injections)) for pos, i in enumerate(spec.run_order)] == plain.run_order(raw)


def test_run_order_of_loops():
    cfg = tiny_config("A")
    assert cfg.run_order() == (0, 1, 0, 1, 0, 1, 2, 3) and cfg.pass_starts() == (0, 2, 4)
    cfg = tiny_config("B")
    assert cfg.run_order() == (0, 1, 1, 2, 3) and cfg.pass_starts() == (1, 2)
    assert tiny_config("C").run_order() == (0, 1, 2, 3) and tiny_config("C").pass_starts() == ()
    assert tiny_config("D").run_order() == (0, 1, 2) and tiny_config("D").pass_starts() == (0,)


def test_config_rejections():
    from leone_b200.config.base import ConfigError
    for patch in (lambda c: c["layers"][0]["mixer"].update(kv_heads=4),
                  lambda c: c["layers"][0]["mixer"]["rot"].update(dims=3),
                  lambda c: c["layers"][0]["mixer"].pop("mask"),
                  lambda c: c["layers"][0].update(type="conv"),
                  lambda c: c["layers"][1]["mlp"]["router"].update(top=5),
                  lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(count=4),
                  lambda c: c["layers"][0]["mlp"].pop("limit"),
                  lambda c: c["loop"].update(stop=9), lambda c: c["loop"].update(start=2),
                  lambda c: c.pop("width"), lambda c: c.update(layers=[])):
        raw = copy.deepcopy(TINY["A"])
        patch(raw)
        with pytest.raises(ConfigError):
            config_from_dict(raw)


# -- the plain implementation's own mechanisms, against their definitions (CPU) -----------------------
def test_plain_masks_and_weight_rules():
    pos = list(range(10))
    assert plain.seen_window(pos, 3)[5].tolist() == [False] * 3 + [True] * 3 + [False] * 4
    assert plain.seen_chunked(pos, 4)[5].tolist() == [False] * 4 + [True] * 2 + [False] * 4
    assert plain.seen_chunked(pos, 4)[4].tolist() == [False] * 4 + [True] + [False] * 5
    s = torch.tensor([[0.3, -1.0, 2.0]], dtype=torch.float64)
    seen = torch.tensor([[True, True, False]])
    w = plain.weights_softmax_with_silent_zero(s, seen)
    e = torch.exp(s[0, :2])
    assert torch.allclose(w[0, :2], e / (1 + e.sum())) and w[0, 2] == 0
    # the weights sum to less than one, by the silent member's share; large scores of either sign are safe
    w = plain.weights_softmax_with_silent_zero(torch.tensor([[5.0, 4.0]], dtype=torch.float64), torch.tensor([[True, True]]))
    assert abs(float(w.sum()) - (1.0 - 1.0 / (1.0 + np.exp(5.0) + np.exp(4.0)))) < 1e-12
    for big in (800.0, -800.0):
        w = plain.weights_softmax_with_silent_zero(torch.tensor([[big]], dtype=torch.float64), torch.tensor([[True]]))
        assert float(w) == (1.0 if big > 0 else 0.0)
    w = plain.weights_sigmoid(s[None], seen[None], torch.tensor([0.5], dtype=torch.float64))
    assert torch.allclose(w[0, 0, :2], torch.sigmoid(s[0, :2] + 0.5)) and w[0, 0, 2] == 0


def test_plain_router_groups():
    # 6 experts in 3 groups worth 0.30, 0.25 and 0.20; two are kept: expert 4 (0.20) cannot be chosen
    # although it scores above expert 0 (0.05), which can
    z = torch.log(torch.tensor([[0.05, 0.30, 0.25, 0.02, 0.20, 0.18]], dtype=torch.float64))
    W = {"router": torch.eye(6, dtype=torch.float64)}
    idx, wt = plain.router_choice(z, W, {"experts": 6, "top": 3, "scale": 2.0, "groups": {"count": 3, "keep": 2}})
    assert idx.tolist() == [[1, 2, 0]] and torch.allclose(wt, torch.tensor([[0.6, 0.5, 0.1]], dtype=torch.float64))
    idx, wt = plain.router_choice(z, W, {"experts": 6, "top": 3, "scale": 1.0})
    assert idx.tolist() == [[1, 2, 4]] and torch.allclose(wt, torch.tensor([[0.3, 0.25, 0.2]], dtype=torch.float64))


# -- the step function on stand-in kernels (CPU) ------------------------------------------------
@pytest.mark.parametrize("which", ["A", "B", "D"])
@pytest.mark.parametrize("mode", ["whole", "portions", "mixed"])
def test_replay_on_stand_in_kernels(which, mode):
    from tests.emulated_ops import EmulatedOps
    tensors = tiny_tensors(which)
    reqs = _requests(TINY[which]["vocab"], [23, 7, 30, 1, 12])
    steps = _traces(reqs)[mode]
    eng = _engine(which, tensors, "float32", "cpu", EmulatedOps(), max_tokens=replay.max_live_tokens(steps))
    out = replay.run_trace_engine(eng, steps)
    replay.compare(steps, out, _plain(which, tensors), reqs, what=f"{which} {mode} stand-in", rtol=2e-5, atol_scale=2e-5)
    assert all(f == eng.num_pages for f in eng.cache.free_pages())


def test_cache_requests_of_the_mixers():
    from tests.emulated_ops import EmulatedOps
    eng = _engine("A", tiny_tensors("A"), "float32", "cpu", EmulatedOps())
    # every run of a looped layer owns a cache; the window layer gives its pages back as the window passes
    kinds = sorted((g.spec.kind, g.spec.head_dim, g.spec.window, len(g.spec.layers)) for g in eng.cache.groups)
    assert kinds == [("full", 16, None, 1), ("full", 24, None, 3), ("full", 32, None, 1), ("window", 16, 9, 3)]
    widths = sorted((k.shape[-1], v.shape[-1]) for k, v in eng.pools)
    assert widths == [(16, 24), (16, 40), (24, 16), (32, 8)]


# -- on the GPU ----------------------------------------------------------------------------------
@pytest.mark.gpu
@pytest.mark.parametrize("which", ["A", "B", "C", "D", "E"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("mode", ["whole", "tail", "portions", "mixed"])
def test_replay_on_the_gpu(which, dtype, mode):
    tensors = tiny_tensors(which)
    reqs = _requests(TINY[which]["vocab"])
    steps = _traces(reqs)[mode]
    pool = replay.max_live_tokens(steps)
    eng = _engine(which, tensors, dtype, "cuda:0", max_tokens=pool)
    out = replay.run_trace_engine(eng, steps)
    tol = FP32 if dtype == "float32" else BF16
    replay.compare(steps, out, _plain(which, tensors, dtype == "bfloat16"), reqs, what=f"{which}/{dtype}/{mode}", **tol)
    if mode == "mixed":
        blocks = sum(-(-len(t) // eng.page_tokens) for t in reqs.values())
        assert blocks > eng.num_pages and len(reqs) > eng.max_requests, "pages and slots must be used again"
    assert all(f == eng.num_pages for f in eng.cache.free_pages())


@pytest.mark.gpu
@pytest.mark.parametrize("switch", ["LEONE_NO_MASKED_MMA", "LEONE_NO_MASKED_TC", "LEONE_NO_EXPERT_MMA", "LEONE_NO_TENSOR_CORES",
                                    "LEONE_NO_TILED_ATTENTION", "LEONE_NO_FUSED_NORM"])
@pytest.mark.parametrize("which", ["C", "D", "E"])
def test_bfloat16_kernel_switches(which, switch, monkeypatch):
    """Every bfloat16 kernel has an any-size form behind a switch; with the switch thrown the same
    traces still agree with the plain implementation (prompt portions of 100 tokens and decode)."""
    monkeypatch.setenv(switch, "1")
    tensors = tiny_tensors(which)
    reqs = _requests(TINY[which]["vocab"], [130, 40, 75])
    steps = replay.trace_portions(reqs, sizes=(100, 2, 1, 1, 30)) + []
    eng = _engine(which, tensors, "bfloat16", "cuda:0", max_tokens=replay.max_live_tokens(steps), max_batch_tokens=128)
    out = replay.run_trace_engine(eng, steps)
    replay.compare(steps, out, _plain(which, tensors, True), reqs, what=f"{which} with {switch}", **BF16)


@pytest.mark.gpu
@pytest.mark.parametrize("which,index", [(w, i) for w in ("A", "B", "C") for i in range(4)])
def test_each_layer_alone(which, index):
    """A model of one layer (looped twice where the configuration has a loop): its mixer and
    feed-forward with nothing else to hide behind."""
    raw = copy.deepcopy(TINY[which])
    raw["layers"] = [raw["layers"][index]]
    if "loop" in raw:
        raw["loop"] = {"start": 0, "stop": 1, "times": 2}
    tensors = {k.replace(f"l{index}.", "l0."): v for k, v in tiny_tensors(which).items()
               if not k.startswith("l") or k.startswith(f"l{index}.") or k == "loop.in"}
    reqs = _requests(raw["vocab"], [45, 2, 19])
    steps = replay.trace_portions(reqs, sizes=(2, 7, 1, 2, 13))
    eng = _engine(which, tensors, "float32", "cuda:0", raw=raw, max_tokens=192, max_requests=2, max_batch_tokens=64)
    out = replay.run_trace_engine(eng, steps)
    replay.compare(steps, out, plain.PlainMalapel(raw, tensors), reqs, what=f"{which} layer {index}", **FP32)


@pytest.mark.gpu
def test_long_prompt_and_long_decode():
    """A prompt of many pages, then 150 single-token steps across pages, windows and chunks;
    position 0 alone first."""
    for dtype, tol in (("float32", FP32), ("bfloat16", BF16)):
        tensors = tiny_tensors("C")
        reqs = {"one": replay.random_tokens(256, 1, 5), "long": replay.random_tokens(256, 460, 77)}
        steps = replay.trace_decode_tail(reqs, tail=150)
        eng = _engine("C", tensors, dtype, "cuda:0", max_tokens=512, max_batch_tokens=512)
        out = replay.run_trace_engine(eng, steps)
        replay.compare(steps, out, _plain("C", tensors, dtype == "bfloat16"), reqs, what=f"long {dtype}", **tol)


@pytest.mark.gpu
def test_page_size_and_batching_do_not_change_fp32_logits_beyond_rounding():
    tensors = tiny_tensors("A")
    reqs = _requests(97, [50, 21, 64])
    steps = replay.trace_mixed(reqs, seed=5)
    outs = []
    for pt in (4, 16, 64):
        eng = _engine("A", tensors, "float32", "cuda:0", max_tokens=replay.max_live_tokens(steps), page=pt)
        outs.append(replay.run_trace_engine(eng, steps))
    for k in outs[0]:
        assert np.array_equal(outs[0][k], outs[1][k]) and np.array_equal(outs[0][k], outs[2][k])


def _seen(kind, size, q_pos, k_pos):
    """The design's rule, stated once more for the test's own premise."""
    if k_pos > q_pos:
        return False
    if kind == "attention":
        return q_pos // size == k_pos // size
    if kind == "attention_3":
        return q_pos - k_pos < size
    return True


@pytest.mark.gpu
@pytest.mark.parametrize("kind,size,q_pos,k_pos", [
    ("attention_2", None, 299, 0), ("attention_2", None, 70, 63), ("attention_2", None, 70, 64),
    ("attention_3", 40, 60, 21), ("attention_3", 40, 60, 20), ("attention_3", 17, 48, 32), ("attention_3", 17, 48, 31),
    ("attention_3", 16, 47, 32), ("attention_3", 16, 47, 31), ("attention_3", 300, 200, 0),
    ("attention", 40, 95, 80), ("attention", 40, 95, 79), ("attention", 16, 40, 32), ("attention", 16, 40, 31),
    ("attention", 25, 99, 75), ("attention", 25, 100, 99), ("attention", 25, 100, 100), ("attention", 300, 250, 0)])
def test_one_key_that_stands_out(kind, size, q_pos, k_pos):
    """A one-layer model whose token 7 (and no other) makes a key that token 9's query scores far
    above all others: the logits at ``q_pos`` change a lot when that key sits at ``k_pos`` and the
    query may see it (just inside a window or a chunk, at a page border, hundreds of tokens back),
    and not at all when it may not.  Checked for the position in a prompt and decoded alone."""
    m = mixer(2, 1, 8, 12, 0.5, rot_dims=4, mask=size)
    raw = _one_layer(kind, m)
    tensors = _random(raw, 3)
    # token 7 is all coordinate 0 and token 9 all coordinate 1 (the norms keep directions); key dimension 4
    # (not rotated) reads coordinate 0 and query dimension 4 of head 0 reads coordinate 1
    for tok, coord in ((7, 0), (9, 1)):
        tensors["embed"][tok] = 0.0
        tensors["embed"][tok, coord] = 1.0
    tensors["l0.mix.k"][4, 0] += 30.0
    tensors["l0.mix.q"][4, 1] += 30.0
    if kind == "attention_3":
        tensors["l0.mix.pb"] = torch.tensor([-6.0, 0.3])       # the ordinary keys of head 0 weigh next to nothing
    length = q_pos + 4
    base = [t if t not in (7, 9) else 8 for t in replay.random_tokens(64, length, 9)]
    base[q_pos] = 9
    marked = list(base)
    if k_pos != q_pos:
        marked[k_pos] = 7
    model = plain.PlainMalapel(raw, tensors)
    delta = float((model.logits(marked)[q_pos] - model.logits(base)[q_pos]).abs().max())
    if k_pos != q_pos:
        assert (delta > 1e-3) == _seen(kind, size, q_pos, k_pos), "the test's own premise"
    eng = _engine(None, tensors, "float32", "cuda:0", raw=raw, page=16, max_tokens=704, max_requests=2,
                  max_batch_tokens=352)
    for name, toks in (("marked", marked), ("base", base)):
        want = model.logits(toks)[q_pos]
        bound = 3e-5 * float(want.abs().max())
        whole = eng.step([(name, toks, [q_pos])])[0].cpu()
        eng.close(name)
        assert float((whole.double() - want).abs().max()) <= bound, (name, "prompt")
        cut = max(1, q_pos - 2)
        eng.step([(name, toks[:cut], [])])
        for p in range(cut, q_pos + 1):
            last = eng.step([(name, [toks[p]], [0])])[0].cpu()
        eng.close(name)
        assert float((last.double() - want).abs().max()) <= bound, (name, "decoded")


@pytest.mark.gpu
def test_the_silent_member_and_the_first_tokens():
    """The first token of a chunk sees only itself: with the silent member its weight is
    e^s / (1 + e^s), not 1, so the first positions (and every chunk's first) tell the two rules apart."""
    raw = _one_layer("attention", mixer(3, 3, 8, 8, 0.3, rot_dims=8, mask=5))
    tensors = _random(raw, 11)
    toks = replay.random_tokens(64, 13, 4)
    model = plain.PlainMalapel(raw, tensors)
    want = model.logits(toks)
    # premise: an ordinary softmax would give other logits at a chunk's first position
    saved = plain.weights_softmax_with_silent_zero
    try:
        plain.weights_softmax_with_silent_zero = plain.weights_softmax
        other = plain.PlainMalapel(raw, tensors).logits(toks)
    finally:
        plain.weights_softmax_with_silent_zero = saved
    assert float((want[[0, 5, 10]] - other[[0, 5, 10]]).abs().max()) > 1e-2 * float(want.abs().max())
    for dtype, tol in (("float32", 3e-5), ("bfloat16", 5e-2)):
        eng = _engine(None, tensors, dtype, "cuda:0", raw=raw, page=4, max_tokens=64, max_requests=2, max_batch_tokens=64)
        ref = _plain(None, tensors, dtype == "bfloat16", raw=raw).logits(toks)
        got = eng.step([("s", toks, list(range(13)))]).cpu().double()
        assert float((got - ref).abs().max()) <= tol * float(ref.abs().max())
        eng.close("s")
        rows = [eng.step([("t", [t], [0])])[0].cpu().double() for t in toks]         # every position decoded alone
        assert float((torch.stack(rows) - ref).abs().max()) <= tol * float(ref.abs().max())


@pytest.mark.gpu
def test_attention_kernels_against_the_plain_rules():
    """The preparation kernel and the attention kernel alone, in 32-bit, over pages: every mask and
    weight rule, both norm forms, key and value widths that differ, a partial rotation."""
    from types import SimpleNamespace
    from leone_b200.ops.cuda import CudaOps
    from leone_b200.parts.base import PagedCacheView
    ops = CudaOps("cuda:0", torch.float32)
    g = torch.Generator().manual_seed(2)
    n, n_q, n_kv, dk, dv, rot, page = 37, 6, 2, 12, 20, 8, 8
    dev = "cuda:0"
    for norm in (None, "per_head", "whole"):
        for pairing in ("half_split", "adjacent"):
            qkv = torch.randn(n, (n_q + n_kv) * dk + n_kv * dv, generator=g)
            q_w = torch.rand((n_q * dk) if norm == "whole" else dk, generator=g) + 0.5
            k_w = torch.rand((n_kv * dk) if norm == "whole" else dk, generator=g) + 0.5
            freqs = torch.tensor([100.0 ** (-2.0 * i / rot) for i in range(rot // 2)], dtype=torch.float64).float()
            ctx = SimpleNamespace(positions=torch.arange(n, dtype=torch.int32, device=dev), n_seqs=1,
                                  seq_of_token=torch.zeros(n, dtype=torch.int32, device=dev),
                                  status=torch.zeros(4, dtype=torch.int32, device=dev))
            pages = -(-n // page)
            table = torch.randperm(pages, generator=g).to(torch.int32).view(1, pages).to(dev)
            cache = PagedCacheView(torch.zeros(pages, n_kv, page, dk, device=dev), torch.zeros(pages, n_kv, page, dv, device=dev),
                                   table, page)
            work = qkv.to(dev)
            ops.attention_prepare(ctx, work, n_q, n_kv, dk, dv, norm, None if norm is None else q_w.to(dev),
                                  None if norm is None else k_w.to(dev), 1e-5, freqs.to(dev), pairing, cache)
            x = qkv.double()
            q, k, v = x[:, :n_q * dk], x[:, n_q * dk:(n_q + n_kv) * dk], x[:, (n_q + n_kv) * dk:].view(n, n_kv, dv)
            if norm == "whole":
                q, k = plain.norm_plain(q, q_w.double(), 1e-5), plain.norm_plain(k, k_w.double(), 1e-5)
            q, k = q.reshape(n, n_q, dk), k.reshape(n, n_kv, dk)
            if norm == "per_head":
                q, k = plain.norm_plain(q, q_w.double(), 1e-5), plain.norm_plain(k, k_w.double(), 1e-5)
            if pairing == "half_split":
                q = plain.rotate_half_split(q, list(range(n)), rot, 100.0, torch.float64)
                k = plain.rotate_half_split(k, list(range(n)), rot, 100.0, torch.float64)
            else:
                def turn(t):
                    ang = torch.arange(n, dtype=torch.float64)[:, None] * freqs.double()[None, :]
                    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
                    out = t.clone()
                    out[..., 0:rot:2] = t[..., 0:rot:2] * c - t[..., 1:rot:2] * s
                    out[..., 1:rot:2] = t[..., 1:rot:2] * c + t[..., 0:rot:2] * s
                    return out
                q, k = turn(q), turn(k)
            got = work.cpu().double()
            assert torch.allclose(got[:, :n_q * dk], q.reshape(n, -1), rtol=1e-5, atol=2e-5), (norm, pairing, "q")
            assert torch.allclose(got[:, n_q * dk:(n_q + n_kv) * dk], k.reshape(n, -1), rtol=1e-5, atol=2e-5), (norm, pairing, "k")
            pos = torch.arange(n)
            slot = table[0].cpu().long()[pos // page]
            assert torch.allclose(cache.k_pool.cpu().double()[slot, :, pos % page, :], k, rtol=1e-5, atol=2e-5)
            assert torch.equal(cache.v_pool.cpu().double()[slot, :, pos % page, :], v)
            if norm is not None or pairing != "half_split":
                continue
            bias = torch.tensor([0.5, -1.0, 0.0, 2.0, -3.0, 1.0])
            for mask, size in (("causal", 0), ("window", 5), ("window", 8), ("chunk", 7), ("chunk", 8), ("chunk", 1)):
                for weights in ("softmax", "softmax_plus_one", "sigmoid"):
                    out = torch.zeros(n, n_q * dv, device=dev)
                    ops.attention_masked(ctx, work, out, n_q, n_kv, dk, dv, 0.4, mask, size, weights,
                                         bias.to(dev) if weights == "sigmoid" else None, cache)
                    kk = k.repeat_interleave(n_q // n_kv, dim=1)
                    vv = v.repeat_interleave(n_q // n_kv, dim=1)
                    sc = torch.einsum("thd,shd->hts", q, kk) * 0.4
                    seen = {"causal": plain.seen_causal(pos), "window": plain.seen_window(pos, size or 1),
                            "chunk": plain.seen_chunked(pos, size or 1)}[mask][None]
                    w = {"softmax": lambda: plain.weights_softmax(sc, seen),
                         "softmax_plus_one": lambda: plain.weights_softmax_with_silent_zero(sc, seen),
                         "sigmoid": lambda: plain.weights_sigmoid(sc, seen, bias.double())}[weights]()
                    want = torch.einsum("hts,shv->thv", w, vv).reshape(n, -1)
                    assert torch.allclose(out.cpu().double(), want, rtol=2e-5, atol=2e-5), (mask, size, weights)


@pytest.mark.gpu
@pytest.mark.parametrize("n_q,n_kv,dk,dv", [(6, 2, 32, 48), (4, 4, 96, 96), (8, 1, 128, 16), (2, 1, 16, 128),
                                            (8, 2, 128, 128), (3, 1, 64, 64)])
def test_tensor_core_attention_against_the_plain_rules(n_q, n_kv, dk, dv):
    """The bfloat16 tensor-core kernel alone: three sequences of unequal lengths as prompt portions
    that start in the middle of a sequence, and as a decode step with and without split keys, for
    every mask and weight rule; against the plain rules on the same bfloat16 values."""
    from types import SimpleNamespace
    from leone_b200.ops.cuda import CudaOps
    from leone_b200.parts.base import PagedCacheView
    ops = CudaOps("cuda:0", torch.bfloat16)
    g = torch.Generator().manual_seed(dk + dv)
    dev, page = "cuda:0", 16
    ctx_lens, q_lens = [300, 77, 130], [130, 77, 1]
    pages = sum(-(-c // page) for c in ctx_lens)
    order = torch.randperm(pages, generator=g)
    table = torch.full((3, -(-max(ctx_lens) // page)), -1, dtype=torch.int32)
    k_pool = torch.zeros(pages, n_kv, page, dk, dtype=torch.bfloat16)
    v_pool = torch.zeros(pages, n_kv, page, dv, dtype=torch.bfloat16)
    keys, vals, at = [], [], 0
    for s_, c in enumerate(ctx_lens):
        kk = (torch.randn(c, n_kv, dk, generator=g)).to(torch.bfloat16)
        vv = torch.randn(c, n_kv, dv, generator=g).to(torch.bfloat16)
        keys.append(kk.double()), vals.append(vv.double())
        for b in range(-(-c // page)):
            table[s_, b] = order[at]
            rows = slice(b * page, min((b + 1) * page, c))
            k_pool[order[at], :, :rows.stop - rows.start] = kk[rows].transpose(0, 1)
            v_pool[order[at], :, :rows.stop - rows.start] = vv[rows].transpose(0, 1)
            at += 1
    cache = PagedCacheView(k_pool.to(dev), v_pool.to(dev), table.to(dev), page)
    bias = torch.linspace(-2.0, 2.0, n_q)

    def run(q_lens_now, mask, size, weights):
        n = sum(q_lens_now)
        q = (torch.randn(n, n_q, dk, generator=g) * 1.5).to(torch.bfloat16)
        qkv = torch.zeros(n, (n_q + n_kv) * dk + n_kv * dv, dtype=torch.bfloat16)
        qkv[:, :n_q * dk] = q.reshape(n, -1)
        starts = [0]
        for x in q_lens_now:
            starts.append(starts[-1] + x)
        pos = torch.cat([torch.arange(c - x, c) for c, x in zip(ctx_lens, q_lens_now)])
        seq = torch.cat([torch.full((x,), i) for i, x in enumerate(q_lens_now)])
        ctx = SimpleNamespace(positions=pos.to(torch.int32).to(dev), seq_of_token=seq.to(torch.int32).to(dev), n_seqs=3,
                              q_start=torch.tensor(starts, dtype=torch.int32, device=dev),
                              ctx_len=torch.tensor(ctx_lens, dtype=torch.int32, device=dev), max_q_len=max(q_lens_now),
                              max_ctx_len=max(ctx_lens), decode_only=max(q_lens_now) == 1,
                              status=torch.zeros(4, dtype=torch.int32, device=dev))
        out = torch.zeros(n, n_q * dv, dtype=torch.bfloat16, device=dev)
        before = ops.launches
        ops.attention_masked(ctx, qkv.to(dev), out, n_q, n_kv, dk, dv, 0.2, mask, size, weights,
                             bias.to(dev) if weights == "sigmoid" else None, cache)
        assert int(ctx.status[0]) == 0
        want = torch.zeros(n, n_q, dv, dtype=torch.float64)
        for i, x in enumerate(q_lens_now):
            c = ctx_lens[i]
            allpos = torch.arange(c)
            seen = {"causal": plain.seen_causal(allpos), "window": plain.seen_window(allpos, size or 1),
                    "chunk": plain.seen_chunked(allpos, size or 1)}[mask][c - x:][None]
            kk = keys[i].repeat_interleave(n_q // n_kv, dim=1)
            vv = vals[i].repeat_interleave(n_q // n_kv, dim=1)
            sc = torch.einsum("thd,shd->hts", q[starts[i]:starts[i + 1]].double(), kk) * 0.2
            w = {"softmax": lambda: plain.weights_softmax(sc, seen),
                 "softmax_plus_one": lambda: plain.weights_softmax_with_silent_zero(sc, seen),
                 "sigmoid": lambda: plain.weights_sigmoid(sc, seen, bias.double())}[weights]()
            want[starts[i]:starts[i + 1]] = torch.einsum("hts,shv->thv", w, vv)
        got = out.cpu().double().view(n, n_q, dv)
        err = float((got - want).abs().max()) / float(want.abs().max())
        assert err < 1.5e-2, (q_lens_now, mask, size, weights, err)

    for mask, size in (("causal", 0), ("window", 70), ("window", 64), ("chunk", 100), ("chunk", 64), ("chunk", 1)):
        for weights in ("softmax", "softmax_plus_one", "sigmoid"):
            run(q_lens, mask, size, weights)
            run([1, 1, 1], mask, size, weights)


@pytest.mark.gpu
def test_router_groups_scale_and_ungated_experts():
    """The router kernel against the plain choice (softmax scores, best groups, scaled weights),
    and the grouped products of ungated experts against the plain sum, in both dtypes."""
    from leone_b200.ops.cuda import CudaOps
    from leone_b200.parts.base import Runtime
    g = torch.Generator().manual_seed(1)
    x = torch.randn(50, 72, generator=g)
    ops = CudaOps("cuda:0", torch.float32)
    for experts, top, groups, keep, scale in ((12, 4, 4, 3, 2.0), (12, 3, 6, 2, 0.5), (11, 11, 1, 1, 1.0), (8, 1, 8, 1, 3.0),
                                              (16, 4, 4, 4, 1.5), (6, 2, 2, 1, 1.0)):
        w = torch.randn(experts, 72, generator=g) * 0.3
        chosen = torch.zeros(50 * top, dtype=torch.int32, device="cuda:0")
        weight = torch.zeros(50 * top, dtype=torch.float32, device="cuda:0")
        ops.experts_route(x.cuda(), w.cuda(), chosen, weight, top, True, False, groups=groups, groups_kept=keep,
                          weight_scale=scale)
        router = {"experts": experts, "top": top, "scale": scale, "groups": {"count": groups, "keep": keep}}
        want_e, want_w = plain.router_choice(x.double(), {"router": w.double()}, router)
        assert torch.equal(chosen.cpu().view(50, top).long(), want_e), (experts, top, groups, keep)
        assert torch.allclose(weight.cpu().view(50, top).double(), want_w, rtol=1e-5, atol=1e-7)
    for dtype, tol in ((torch.float32, 2e-5), (torch.bfloat16, 3e-2)):
        ops = CudaOps("cuda:0", dtype)
        rt = Runtime("cuda:0", dtype, ops, 64)
        for width, ff, experts, top in ((72, 40, 5, 2), (64, 96, 7, 3)):
            up = (torch.randn(experts, ff, width, generator=g) * 0.2).to(dtype)
            down = (torch.randn(experts, width, ff, generator=g) * 0.2).to(dtype)
            xin = torch.randn(50, width, generator=g).to(dtype)
            idx = torch.stack([torch.randperm(experts, generator=g)[:top] for _ in range(50)])
            wt = torch.rand(50, top, generator=g) + 0.1
            hidden = torch.randn(50, width, generator=g)
            want = hidden.double().clone()
            for t in range(50):
                for e, s in zip(idx[t].tolist(), wt[t].tolist()):
                    want[t] += s * plain.linear(plain.relu_squared(plain.linear(xin[t].double()[None], up[e].double())),
                                                down[e].double())[0]
            got = hidden.cuda()
            ops.experts_forward(xin.cuda(), None, up.cuda(), down.cuda(), idx.reshape(-1).to(torch.int32).cuda(),
                                wt.reshape(-1).cuda(), top, False, got, rt)
            assert float((got.cpu().double() - want).abs().max()) <= tol * float(want.abs().max()), (dtype, width)


@pytest.mark.gpu
def test_clamped_gate_against_the_plain_formula():
    """The gated layer with a steeper sigmoid, clamped inputs and a shifted up branch, through the
    part: inputs large enough that both clamps bind."""
    raw = _one_layer("attention_2", mixer(2, 2, 8, 8, 0.3), dense(48, 0.6), width=32)
    tensors = _random(raw, 21, gain=8.0)
    toks = replay.random_tokens(64, 40, 3)
    for dtype, tol in (("float32", 3e-5), ("bfloat16", 5e-2)):
        model = _plain(None, tensors, dtype == "bfloat16", raw=raw)
        h = plain.norm_around_one(model.residuals(toks)[0], model.t["l0.norm2"], 1e-6)
        pre = plain.linear(h, model.t["l0.mlp.gate"])
        assert float((pre > 0.6).double().mean()) > 0.1 and float((plain.linear(h, model.t["l0.mlp.up"]) < -0.6).double().mean()) > 0.1
        eng = _engine(None, tensors, dtype, "cuda:0", raw=raw, page=16, max_tokens=64, max_requests=2, max_batch_tokens=64)
        got = eng.step([("g", toks, list(range(40)))]).cpu().double()
        want = model.logits(toks)
        assert float((got - want).abs().max()) <= tol * float(want.abs().max())


@pytest.mark.gpu
@pytest.mark.parametrize("which", ["A", "C", "E"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_scheduler(dtype, which, tmp_path):
    """generate(): admission, prompt portions mixed with decode, captured decode steps (with the
    looped layers, their injections and windows whose pages go back while decoding), finish."""
    from leone_b200 import generate
    from leone_b200.weights.safetensors import write_safetensors
    folder = str(tmp_path / "model")
    cfg = tiny_config(which)
    cfg.write(folder)
    tensors = tiny_tensors(which)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors)
    model = _plain(which, tensors, dtype == "bfloat16")
    prompts = [replay.random_tokens(TINY[which]["vocab"], n, 60 + n) for n in (1, 9, 40, 23, 5)]
    for kw in (dict(), dict(prefill_chunk=7, max_batch_tokens=16, use_graphs=False, prefill_first=False)):
        got = generate(folder, prompts, 10, dtype=dtype, eos_token_id=-1, max_running=3, **kw)
        for p, toks in zip(prompts, got):
            assert len(toks) == 10
            seq = list(p)
            for t in toks:
                logits = model.logits(seq)[-1]
                gap = float(logits.max() - logits[t])
                assert gap <= (1e-4 if dtype == "float32" else 0.04) * float(logits.abs().max()), (kw, seq, t, gap)
                seq.append(t)


@pytest.mark.gpu
def test_trace_program_on_a_written_model(tmp_path):
    """bin/trace_run as a user runs it: a folder with config.json and model.safetensors, steps over stdin."""
    from leone_b200.weights.safetensors import write_safetensors
    folder, out = str(tmp_path / "model"), str(tmp_path / "out")
    tiny_config("A").write(folder)
    tensors = {k: (v.to(torch.bfloat16) if v.dtype == torch.float32 else v) for k, v in tiny_tensors("A").items()}
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors)
    reqs = _requests(97, [30, 5, 41, 17, 8])
    steps = replay.trace_mixed(reqs, seed=11)
    got = replay.run_trace_program(folder, "float32", steps, out, replay.max_live_tokens(steps), extra=("--page-tokens", "4"))
    model = plain.PlainMalapel(TINY["A"], {k: v.float() for k, v in tensors.items()})
    replay.compare(steps, got, model, reqs, what="trace program", **FP32)
