"""Small Borosun configurations for the tests, and model folders and runners made from them."""

from __future__ import annotations

import copy

import torch

import plain_borosun as pb
from conftest import device
from ludalix_helpers import replay, write_model  # noqa: F401  (step plans replayed through the step function)


def rot(dims, base=10000.0, scaling=None):
    r = dict(dims=dims, base=base)
    if scaling:
        r["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    return r


def attention(heads, kv_heads, dim, vdim, scale, rotation=None, conv=None, v_mix=False):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale)
    if rotation:
        m["rot"] = rotation
    if conv:
        m["conv"] = conv
    if v_mix:
        m["v_mix"] = True
    return m


def attention_2(heads, kv_heads, dim, vdim, scale, size, rotation=None, softcap=None, v_mix=False):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale, mask=dict(size=size))
    if rotation:
        m["rot"] = rotation
    if softcap:
        m["softcap"] = softcap
    if v_mix:
        m["v_mix"] = True
    return m


def gla(heads, dim, vdim, tau):
    return dict(heads=heads, dim=dim, vdim=vdim, tau=tau)


def dense(ff):
    return dict(kind="dense", ff=ff)


def config(width, vocab, layers, side=None, cap=None, eps=2e-6):
    c = dict(architecture="Borosun", vocab=vocab, width=width, norm=dict(eps=eps),
             layers=[dict(type=t, mixer=m, mlp=f) for t, m, f in layers])
    if side:
        c["token_side"] = dict(dim=side)
    if cap:
        c["logit_softcap"] = cap
    return c


# A: all three mixers, values mixed between the two kinds of attention (first the convolved one), rotation over a
# part of the head with rescaled frequencies, a window of 9 over pages of 8, a state layer without feed-forward
CFG_A = config(72, 211, [
    ("attention", attention(4, 2, 24, 20, 0.25, rot(16, 900.0, (4.0, 1.0, 3.0, 48)), conv=4, v_mix=True), dense(96)),
    ("gla", gla(3, 20, 28, 7.0), None),
    ("attention_2", attention_2(4, 2, 32, 20, 0.15, 9, rot(32, 5000.0), softcap=6.0, v_mix=True), dense(64)),
    ("gla", gla(2, 40, 16, 3.0), dense(80)),
], side=10, cap=9.0)
# B: the first layer that mixes values is a windowed one and a convolved one follows; one kv head, and as many kv
# heads as heads; a convolution of two taps and one of one tap (no memory); no token side input, no logit cap;
# a window larger than most prompts; rescaled frequencies under the window, none without it
CFG_B = config(64, 97, [
    ("attention_2", attention_2(6, 1, 16, 24, 0.4, 40, rot(8, 300.0, (2.0, 1.0, 4.0, 16)), softcap=20.0, v_mix=True), None),
    ("attention", attention(3, 3, 16, 8, 0.3, rot(16, 1e4), conv=2, v_mix=True), dense(48)),
    ("attention", attention(2, 1, 40, 24, 0.2, None, conv=1, v_mix=True), dense(40)),
    ("gla", gla(1, 64, 32, 16.0), dense(56)),
], eps=1e-5)
# C: head sizes the tensor-core kernels like (64, 128), a window of one page, no value mixing, attention without
# a convolution, a wide state head, sizes that are no multiple of 8
CFG_C = config(100, 130, [
    ("attention_2", attention_2(4, 2, 128, 64, 0.03, 16, rot(64, 5e5), softcap=30.0), dense(52)),
    ("gla", gla(2, 128, 24, 9.0), dense(36)),
    ("attention", attention(2, 1, 64, 64, 0.125, rot(64, 1e4, (8.0, 1.0, 4.0, 64))), None),
    ("gla", gla(1, 136, 72, 2.0), None),
], side=3, cap=30.0)

# D: the sizes the tensor-core attention kernels take in bfloat16 (values as wide as keys, 64 and 128): mixed heads
# over two kv heads behind a convolution, capped scores under a window of 40, values mixed between the two
CFG_D = config(96, 150, [
    ("attention", attention(4, 2, 64, 64, 0.125, rot(32, 1e4, (4.0, 1.0, 4.0, 32)), conv=3, v_mix=True), dense(72)),
    ("attention_2", attention_2(8, 2, 64, 64, 0.05, 40, rot(64, 1e4), softcap=2.5, v_mix=True), None),
    ("gla", gla(2, 32, 48, 8.0), dense(40)),
    ("attention_2", attention_2(4, 2, 128, 128, 0.02, 24, rot(64, 5e5), softcap=1.5), dense(64)),
    ("attention", attention(2, 2, 128, 128, 0.09, None, conv=2), None),
], side=20, cap=20.0)

CONFIGS = {"A": (CFG_A, 8), "B": (CFG_B, 4), "C": (CFG_C, 16), "D": (CFG_D, 16)}  # config, page size


# (The token side input is divided by its own root mean square: with a share of only a few columns it nearly
# vanishes at some positions and 16-bit rounding is amplified there, in any evaluation of the design.  D, with five
# layers, has a share of 20 columns for that reason; C keeps a share of 3.)
SEEDS: dict = {}


def weights_for(tag: str, dtype: str, seed: int | None = None):
    cfg, page = CONFIGS[tag]
    seed = SEEDS.get(tag, 0) if seed is None else seed
    w = pb.random_weights(cfg, seed=seed + sum(map(ord, tag)))
    if dtype != "float32":
        w = {n: t.to(getattr(torch, dtype)) for n, t in w.items()}
    return copy.deepcopy(cfg), w, page


def make_runner(tmp_path, cfg, w, page, dtype, num_pages=64, max_requests=4, name="m", **kw):
    from ullm_b200.engine import ModelRunner

    d = write_model(str(tmp_path / f"{name}_{dtype}"), cfg, w)
    return ModelRunner(d, dtype=dtype, device=device(), page_size=page, num_pages=num_pages, max_requests=max_requests,
                       max_context=num_pages * page, max_step_tokens=64, poison_cache=True, **kw)


def oracle(ids, w, cfg) -> torch.Tensor:
    """Logits at every position, 64-bit arithmetic on the weights as given (rounded ones stay rounded)."""
    return pb.forward(cfg, {n: t.double() for n, t in w.items()}, ids).float()
