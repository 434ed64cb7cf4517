"""Small Ludalix configurations for the tests, model folders made from them, and a replay of step plans through
the engine's step function."""

from __future__ import annotations

import copy
import json
import os

import torch

import plain_ludalix as pl
from conftest import device


def attention(heads, kv_heads, dim, vdim, size, keep_first, scale, kv_from=None):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, mask=dict(size=size, keep_first=keep_first), scale=scale)
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def mlstm(heads, dim, vdim, gate_cap):
    return dict(heads=heads, dim=dim, vdim=vdim, gate_cap=gate_cap)


def dense(ff, limit):
    return dict(kind="dense", ff=ff, limit=limit)


def moe(experts, top, ff):
    return dict(kind="moe", expert=dict(ff=ff), router=dict(experts=experts, top=top))


def config(width, vocab, layers, mult=0.6, scale=9.0, eps=2e-6):
    return dict(architecture="Ludalix", vocab=vocab, width=width, residual_mult=mult, embedding=dict(scale=scale),
                norm=dict(eps=eps), layers=[dict(type=t, mixer=m, mlp=f) for t, m, f in layers])


# P: an attention layer first (as many kv heads as heads, values wider than keys, two experts per token), a state
# layer without feed-forward, a layer that borrows layer 0's keys and values under a LARGER window without kept
# tokens, a state layer whose head size is no multiple of anything
CFG_P = config(72, 211, [
    ("attention", attention(4, 4, 24, 40, 9, 3, 0.31), moe(5, 2, 48)),
    ("mlstm", mlstm(3, 20, 28, 7.5), None),
    ("attention", attention(4, 4, 24, 40, 17, 0, 0.2, kv_from=0), dense(100, 0.8)),
    ("mlstm", mlstm(2, 40, 16, 15.0), moe(3, 3, 32)),
])
# Q: one head of state with keys wider than values, grouped attention whose kept tokens outnumber its window,
# odd vocabulary, multiplier 1
CFG_Q = config(64, 97, [
    ("mlstm", mlstm(1, 64, 32, 4.0), dense(80, 3.0)),
    ("attention", attention(6, 2, 16, 16, 5, 11, 0.25), moe(4, 1, 24)),
    ("attention", attention(6, 2, 16, 16, 40, 2, 0.25, kv_from=1), None),
], mult=1.0, scale=1.0, eps=1e-5)
# R: head sizes the tensor-core paths like (64), a window of one page, sizes that are no multiple of 8
CFG_R = config(100, 130, [
    ("attention", attention(2, 1, 64, 64, 16, 16, 0.125), dense(52, 1.5)),
    ("mlstm", mlstm(2, 12, 36, 12.0), moe(6, 2, 20)),
], mult=0.8, scale=4.0)

# S: state heads of 128 and 256 rows (the recurrence kernel's forms without bounds checks), many value columns
CFG_S = config(96, 77, [
    ("mlstm", mlstm(2, 128, 24, 9.0), dense(64, 2.0)),
    ("mlstm", mlstm(1, 256, 136, 9.0), None),
], mult=0.7, scale=5.0)

# T: windows without kept tokens at the head sizes of the tensor-core attention kernels (the paths the rotary
# models take, here without any rotation), one of them read again by a later layer under another window
CFG_T = config(96, 150, [
    ("attention", attention(4, 2, 128, 128, 40, 0, 0.09), dense(72, 4.0)),
    ("attention", attention(2, 2, 64, 64, 24, 0, 0.125), None),
    ("attention", attention(4, 2, 128, 128, 100, 0, 0.09, kv_from=0), moe(4, 2, 40)),
], mult=0.65, scale=6.0)

CONFIGS = {"P": (CFG_P, 8), "Q": (CFG_Q, 4), "R": (CFG_R, 16), "S": (CFG_S, 16), "T": (CFG_T, 16)}  # config, page size


def weights_for(tag: str, dtype: str, seed: int = 0, std_scale: float = 1.0):
    cfg, page = CONFIGS[tag]
    w = pl.random_weights(cfg, seed=seed + sum(map(ord, tag)), std_scale=std_scale)
    if dtype != "float32":
        w = {n: t.to(getattr(torch, dtype)) for n, t in w.items()}
    return copy.deepcopy(cfg), w, page


def write_model(path: str, cfg: dict, w: dict) -> str:
    from ullm_b200.weights import save_tensors

    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_tensors(os.path.join(path, "model.safetensors"), {n: t.contiguous() for n, t in w.items()})
    return path


def make_runner(tmp_path, cfg, w, page, dtype, num_pages=64, max_requests=4, name="m", **kw):
    from ullm_b200.engine import ModelRunner

    d = write_model(str(tmp_path / f"{name}_{dtype}"), cfg, w)
    return ModelRunner(d, dtype=dtype, device=device(), page_size=page, num_pages=num_pages, max_requests=max_requests,
                       max_context=num_pages * page, max_step_tokens=64, poison_cache=True, **kw)


def oracle(ids, w, cfg) -> torch.Tensor:
    """Logits at every position, float64 arithmetic on the weights as given (rounded ones stay rounded)."""
    return pl.forward_logits(ids, {n: t.double() for n, t in w.items()}, cfg).float()


def replay(runner, requests: dict[str, list[int]], plan) -> dict[str, torch.Tensor]:
    """plan: steps, each a list of (request id, token count); a request is admitted at its first entry and ended
    when its tokens are used up.  Returns the logits at every position of every request."""
    from ullm_b200.engine import StepEntry

    at = {r: 0 for r in requests}
    got = {r: [] for r in requests}
    for step in plan:
        entries = []
        for rid, n in step:
            if not runner.has_request(rid):
                assert runner.add_request(rid) is not None, "no free request slot"
            lo = at[rid]
            entries.append(StepEntry(rid, requests[rid][lo:lo + n], list(range(n))))
            at[rid] = lo + n
        lg = runner.step(entries).float().cpu().clone()
        runner.check_device_status()
        row = 0
        for rid, n in step:
            got[rid].append(lg[row:row + n])
            row += n
            if at[rid] == len(requests[rid]):
                runner.end_request(rid)
        runner.cache.check_invariants()
    assert all(at[r] == len(requests[r]) for r in requests), "the plan does not use up every request"
    return {r: torch.cat(v) for r, v in got.items()}


def router_margins(ids, w, cfg) -> torch.Tensor:
    """Per position, the smallest gap (in score) between the last chosen and the first rejected expert over all
    routed layers, from the plain model in 64-bit; infinity where nothing is routed."""
    margins = torch.full((len(ids),), float("inf"), dtype=torch.float64)
    keep = pl.router_choice

    def watching(h, w_, pre, top):
        s = torch.sigmoid(h @ w_[pre + "router"].T).sort(-1, descending=True).values
        if top < s.shape[1]:
            margins.copy_(torch.minimum(margins, s[:, top - 1] - s[:, top]))
        return keep(h, w_, pre, top)

    pl.router_choice = watching
    try:
        pl.forward_stream(ids, {n: t.double() for n, t in w.items()}, cfg)
    finally:
        pl.router_choice = keep
    return margins


def assert_rows_close(got, ref, dtype: str, what: str = "", margins=None):
    """32-bit: the fixed limits of tests/helpers.py on every row.  16-bit: the same rms limit over all rows that
    count, and the max limit on all of them but at most one in fifty (at least one), which may reach three times
    the limit: a head's read-out is divided by its own root mean square, so at a position where the read-out
    nearly vanishes the rounding of q, k and v is amplified, as it is in any 16-bit evaluation of the design.
    Rows whose router decision is a close call in the plain model (`margins` below 0.005) do not count: 16-bit
    rounding may send them to another expert."""
    from helpers import TOL, TOL_RMS, assert_close

    if dtype == "float32":
        return assert_close(got, ref, dtype, what)
    assert got.shape == ref.shape and torch.isfinite(got.float()).all(), f"{what}: shape or non-finite values"
    got = got.detach().float().cpu()
    counted = torch.ones(len(ref), dtype=torch.bool) if margins is None else margins >= 0.005
    assert counted.sum() >= 0.8 * len(ref), f"{what}: too many close calls of the router for a meaningful comparison"
    scale = max(ref.abs().max().item(), 1e-6)
    d = (got - ref)[counted]
    per_row = d.abs().max(-1).values / scale
    rms = d.pow(2).mean().sqrt().item() / scale
    over = int((per_row > TOL[dtype]).sum())
    assert rms <= TOL_RMS[dtype], f"{what}: rms {rms:.3e} (limit {TOL_RMS[dtype]:.0e}) of scale"
    assert over <= max(1, len(per_row) // 50) and per_row.max() <= 3 * TOL[dtype], (
        f"{what}: {over} of {len(per_row)} rows over {TOL[dtype]:.0e}, worst {per_row.max():.3e} of scale"
        + ("" if margins is None else f" (router margin there {float(margins[counted][per_row.argmax()]):.3f})"))
