"""The Borosun decoder in the engine against the plain implementation (tests/plain_borosun.py): each mechanism
alone, whole prompts against token-by-token decoding and portions down to two tokens, unequal batches with pages
and state slots that are used again, the edges of the window and of pages (with weights made so that one key
decides), far keys and far memory, the first tokens of a sequence, long decoding, and greedy generation through
the entry point and the scheduler."""

import copy

import pytest
import torch

import plain_borosun as pb
from borosun_helpers import (attention, attention_2, config, dense, gla, make_runner, oracle, replay, rot,
                             weights_for, write_model)
from conftest import device
from helpers import TOL, assert_close, errors, random_ids
from ludalix_helpers import assert_rows_close

pytestmark = pytest.mark.gpu


def close(got, ref, dtype, what):
    """A part alone: 32-bit to 3e-5 of the largest value; bfloat16 within the limits the whole models get."""
    if dtype != "float32":
        return assert_close(got, ref, dtype, what)
    mx, _ = errors(got, ref)
    assert torch.isfinite(got.float()).all(), f"{what}: non-finite"
    assert mx <= 3e-5, f"{what}: max err {mx:.2e} of scale"


def rand(shape, seed, dtype, scale=1.0):
    t = torch.randn(*shape, generator=torch.Generator().manual_seed(seed)) * scale
    return t.to(getattr(torch, dtype)).to(device())


def cast(w, dtype):
    return w if dtype == "float32" else {n: t.to(getattr(torch, dtype)) for n, t in w.items()}


# ---------------------------------------------------------------------------------------------------------
# each mechanism alone
# ---------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tag,layer", [("A", 0), ("A", 2), ("B", 0), ("B", 1), ("B", 2), ("C", 0), ("C", 2), ("D", 0),
                                       ("D", 1), ("D", 3), ("D", 4)])
def test_attention_mixers_alone(tmp_path, dtype, tag, layer):
    """Both kinds of attention on random rows in four steps (1, 36, 2 and 1 tokens: the convolution's memory is
    younger than its taps at first, and a later step brings fewer rows than it has taps), with the first layer's
    values given where the layer mixes them in."""
    from ullm_b200.engine import StepEntry

    cfg, w, page = weights_for(tag, dtype)
    r = make_runner(tmp_path, cfg, w, page, dtype)
    n = 40
    L = cfg["layers"][layer]
    m, pre = L["mixer"], f"l{layer}.mix."
    mixer = r.model.blocks[layer].mixer
    x = rand((n, cfg["width"]), 6, dtype)
    vf = rand((n, m["kv_heads"] * m["vdim"]), 7, dtype)
    wd = {k: t.double() for k, t in w.items()}
    shared = {"v_first": vf.double().cpu()} if mixer.value_mix == "mix" else {}
    if L["type"] == "attention":
        ref = pb.attention_conv_talk(x.double().cpu(), m, wd, pre, shared)
    else:
        ref = pb.attention_window_capped(x.double().cpu(), m, wd, pre, shared, cfg["norm"]["eps"])
    got = []
    r.add_request("a")
    for a, b in ((0, 1), (1, 37), (37, 39), (39, 40)):
        e = [StepEntry("a", [0] * (b - a), [])]
        ctx = r.prepare(e)
        ctx.shared = {"attn.v_first": vf[a:b].contiguous()} if mixer.value_mix == "mix" else {}
        caches = r.cache.layer_caches(ctx.groups)
        got.append(mixer.forward(x[a:b].clone(), ctx, caches[layer]).float().cpu().clone())
        if mixer.value_mix == "first":
            assert ctx.shared["attn.v_first"].shape == (b - a, m["kv_heads"] * m["vdim"])
        r.commit(e)
    r.check_device_status()
    close(torch.cat(got), ref.float(), dtype, f"{L['type']} mixer")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tag,layer", [("A", 1), ("A", 3), ("B", 3), ("C", 1), ("C", 3)])
def test_gla_mixer_alone(tmp_path, dtype, tag, layer):
    """The mixer on random rows in three steps (13, 1 and 9 tokens) against the recurrence run whole."""
    from ullm_b200.engine import StepEntry

    cfg, w, page = weights_for(tag, dtype)
    r = make_runner(tmp_path, cfg, w, page, dtype)
    x = rand((23, cfg["width"]), 5, dtype)
    wd = {n: t.double() for n, t in w.items()}
    ref = pb.gla(x.double().cpu(), cfg["layers"][layer]["mixer"], wd, f"l{layer}.mix.", cfg["norm"]["eps"]).float()
    got = []
    r.add_request("a")
    for a, b in ((0, 13), (13, 14), (14, 23)):
        e = [StepEntry("a", [0] * (b - a), [])]
        ctx = r.prepare(e)
        caches = r.cache.layer_caches(ctx.groups)
        got.append(r.model.blocks[layer].mixer.forward(x[a:b].clone(), ctx, caches[layer]).float().cpu().clone())
        r.commit(e)
    r.check_device_status()
    close(torch.cat(got), ref, dtype, "gated linear attention mixer")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tag,layer", [("A", 1), ("A", 3), ("C", 3), ("B", 3)])
def test_parallel_gated_block_alone(tmp_path, dtype, tag, layer):
    """One layer on a random 32-bit stream: both sub-layers from one norm, each through its gate, then the layer's
    share of the token side input (A, C) or none (B); a layer without feed-forward has one gate."""
    from ullm_b200.engine import StepEntry

    cfg, w, page = weights_for(tag, dtype)
    r = make_runner(tmp_path, cfg, w, page, dtype)
    n = 19
    ids = random_ids(cfg["vocab"], n, 3)
    x = rand((n, cfg["width"]), 8, "float32", 2.0)
    wd = {k: t.double() for k, t in w.items()}
    ref = pb.layer(x.double().cpu(), torch.tensor(ids), layer, cfg["layers"][layer], cfg, wd, {}).float()
    r.add_request("a")
    e = [StepEntry("a", ids, [])]
    ctx = r.prepare(e)
    ctx.token_side, ctx.shared = r.model.token_side, {}
    stream = x.clone()
    y, out = r.model.blocks[layer].forward(None, stream, ctx, r.cache.layer_caches(ctx.groups)[layer])
    r.check_device_status()
    assert y is None and out.dtype == torch.float32
    close(out.cpu(), ref, dtype, "parallel gated block")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_convolution_longer_than_the_steps(tmp_path, dtype):
    """Eleven taps: the memory outlives several steps of one to three tokens, and a first step is shorter than it."""
    cfg = config(48, 61, [("attention", attention(4, 2, 16, 12, 0.25, rot(8, 50.0), conv=11, v_mix=True), dense(32))], side=8)
    w = cast(pb.random_weights(cfg, seed=1), dtype)
    ids = random_ids(61, 60, 3)
    r = make_runner(tmp_path, cfg, w, 8, dtype)
    plan = [[("a", 3)], [("a", 1)], [("a", 2)], [("a", 30)], [("a", 5)]] + [[("a", 1)] for _ in range(19)]
    assert_rows_close(replay(r, {"a": ids}, plan)["a"], oracle(ids, w, cfg), dtype, "eleven taps")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_capped_logits_of_the_tied_head(tmp_path, dtype):
    """A (cap 9) against the same weights without a cap: the engine follows the configuration, and the cap matters."""
    cfg, w, page = weights_for("A", dtype)
    ids = random_ids(cfg["vocab"], 12, 2)
    ref = oracle(ids, w, cfg)
    free = copy.deepcopy(cfg)
    free.pop("logit_softcap")
    assert ref.abs().max() < 9.0 < oracle(ids, w, free).abs().max()
    for c, name in ((cfg, "capped"), (free, "free")):
        r = make_runner(tmp_path, c, w, page, dtype, name=name)
        assert_rows_close(replay(r, {"a": ids}, [[("a", 12)]])["a"], oracle(ids, w, c), dtype, name)


# ---------------------------------------------------------------------------------------------------------
# whole prompts, token-by-token decoding, portions
# ---------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tag", ["A", "B", "C", "D"])
def test_whole_decode_and_portions_agree_with_the_plain_model(tmp_path, dtype, tag):
    cfg, w, page = weights_for(tag, dtype)
    r = make_runner(tmp_path, cfg, w, page, dtype)
    n = 75
    ids = random_ids(cfg["vocab"], n, 11)
    ref = oracle(ids, w, cfg)
    plans = {
        "whole": [[("a", n)]],
        "decode": [[("b", 3)]] + [[("b", 1)] for _ in range(n - 3)],
        "portions": [[("c", k)] for k in (2, 2, 3, 7, 2, 16, 1, 1, 2, 31, 8)],
        "one by one": [[("d", 1)] for _ in range(n)],
    }
    assert sum(k for (_, k), in plans["portions"]) == n
    for name, plan in plans.items():
        rid = plan[0][0][0]
        got = replay(r, {rid: ids}, plan)[rid]
        assert_rows_close(got, ref, dtype, f"{tag} {name}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tag,pages", [("A", 22), ("D", 12)])
def test_unequal_batches_with_pages_and_slots_used_again(tmp_path, dtype, tag, pages):
    """Three state slots and a pool that cannot hold all requests at once: six requests of unequal length come
    and go, portions of some beside single tokens of others; every request equals itself run alone."""
    cfg, w, page = weights_for(tag, dtype)
    r = make_runner(tmp_path, cfg, w, page, dtype, num_pages=pages, max_requests=3)
    lens = dict(a=50, b=9, c=61, d=2, e=33, f=17)
    reqs = {k: random_ids(cfg["vocab"], n, 40 + n) for k, n in lens.items()}
    plan = [
        [("a", 20), ("b", 2)],
        [("a", 1), ("b", 5), ("c", 30)],
        [("b", 2), ("a", 9), ("c", 1)],          # b ends: its slot and pages go back
        [("d", 2), ("c", 1), ("a", 1)],          # d takes them, and ends at once
        [("e", 16), ("a", 19)],                  # a ends
        [("c", 29), ("e", 1), ("f", 2)],         # c ends; f starts on a slot that held state
        [("f", 15), ("e", 16)],
    ]
    got = replay(r, reqs, plan)
    for k in reqs:
        if tag == "A" or dtype == "float32":
            assert_rows_close(got[k], oracle(reqs[k], w, cfg), dtype, f"request {k}")
        # and against the same request run alone, whole, through the same engine
        alone = replay(r, {k + "'": reqs[k]}, [[(k + "'", len(reqs[k]))]])[k + "'"]
        assert_rows_close(got[k], alone, dtype, f"request {k} in the batch against itself alone")
    assert not r.cache.requests and all(r.cache.num_free_pages(g) == pages for g in range(len(r.cache.groups)))


# ---------------------------------------------------------------------------------------------------------
# edges: the window, page borders, far keys; weights made so that one key decides
# ---------------------------------------------------------------------------------------------------------
def one_key_window_model(size, dtype, dim=16, vdim=24, cap=None):
    """One windowed layer without feed-forward whose scale is large: with unit-RMS queries and keys the scores
    spread over +- scale x dim, the softmax is nearly one-hot, and a key that is wrongly seen or wrongly hidden
    changes the logits by much more than any tolerance."""
    scale = (14.0 if dtype == "float32" else 12.0) / dim
    cfg = config(48, 61, [("attention_2", attention_2(2, 1, dim, vdim, scale, size, rot(dim // 2, 100.0), softcap=cap), None)])
    w = pb.random_weights(cfg, seed=size * 31 + dim)
    w["l0.mix.o"] = w["l0.mix.o"] * 2.0  # (the mixer's share of the stream beside the embedding)
    return cfg, cast(w, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("size", [1, 8, 16, 5, 17])
@pytest.mark.parametrize("dim,vdim", [(16, 24), (64, 64), (128, 128)])  # the last two: tensor-core kernels in bfloat16
def test_window_edges_in_prompts_and_decoding(tmp_path, dtype, size, dim, vdim):
    page = 8
    cfg, w = one_key_window_model(size, dtype, dim, vdim)
    n = 70
    # the test has power: a window one token longer or shorter is far off
    for seed in range(5, 25):
        ids = random_ids(cfg["vocab"], n, seed)
        ref = oracle(ids, w, cfg)
        offs = []
        for ds in (1, -1):
            if size + ds < 1:
                continue
            other = copy.deepcopy(cfg)
            other["layers"][0]["mixer"]["mask"]["size"] = size + ds
            offs.append(float((oracle(ids, w, other) - ref).abs().max() / ref.abs().max()))
        if min(offs) > 5 * TOL[dtype]:
            break
    else:
        raise AssertionError(f"no token sequence makes both edges decisive (last: {offs})")
    r = make_runner(tmp_path, cfg, w, page, dtype, num_pages=12)
    # portions that end on, one before and one after page borders and window edges; then single tokens
    plan = [[("a", k)] for k in (7, 1, 1, 8, 9, 2, size, 3)]
    used = sum(k for (_, k), in plan)
    plan += [[("a", 1)] for _ in range(n - used)]
    got = replay(r, {"a": ids}, plan)["a"]
    assert_close(got, ref, dtype, f"window {size}")
    assert r.cache.num_free_pages(0) == 12  # pages the window left behind went back while the request ran


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("dim,vdim", [(16, 24), (64, 64), (128, 128)])
def test_score_cap_decides(tmp_path, dtype, dim, vdim):
    """Scores far beyond the cap: without it the softmax is one-hot, with it the best keys tie."""
    cfg, w = one_key_window_model(24, dtype, dim, vdim, cap=2.0)
    ids = random_ids(cfg["vocab"], 50, 4)
    ref = oracle(ids, w, cfg)
    free = copy.deepcopy(cfg)
    free["layers"][0]["mixer"].pop("softcap")
    assert (oracle(ids, w, free) - ref).abs().max() > 5 * TOL[dtype] * ref.abs().max()
    r = make_runner(tmp_path, cfg, w, 8, dtype, num_pages=12)
    got = replay(r, {"a": ids}, [[("a", 30)], [("a", 2)]] + [[("a", 1)] for _ in range(18)])["a"]
    assert_close(got, ref, dtype, "capped scores")


@pytest.mark.parametrize("dim", [64, 128])
def test_scores_deep_inside_the_cap_on_the_tensor_cores(tmp_path, dim):
    """bfloat16, head sizes of the tensor-core kernels, |score| at most a sixth of the cap: the prompt kernel's
    short form of the cap must agree with the plain model as its exact form does (prompt portions and decoding)."""
    from ullm_b200.csrc import kernels

    cfg = config(64, 83, [("attention_2", attention_2(4, 2, dim, dim, 1.3 / dim, 50, rot(dim // 2, 1e4), softcap=8.0), dense(48))])
    w = cast(pb.random_weights(cfg, seed=dim), "bfloat16")
    ids = random_ids(cfg["vocab"], 120, 6)
    r = make_runner(tmp_path, cfg, w, 16, "bfloat16", num_pages=12)
    got = replay(r, {"a": ids}, [[("a", 70)], [("a", 3)], [("a", 40)]] + [[("a", 1)] for _ in range(7)])["a"]
    assert_rows_close(got, oracle(ids, w, cfg), "bfloat16", "cap in its linear regime")
    if device() != "cpu":
        r2 = make_runner(tmp_path, cfg, w, 16, "bfloat16", num_pages=12, name="p")
        replay(r2, {"b": ids}, [[("b", 120)]])
        assert kernels().attention_path == ("prefill" if dim == 64 else "prefill_tcgen05")


def far_key_model(dtype, dim=16, vdim=12):
    """One causal layer (convolution, mixed heads, two kv heads) with a large scale, without feed-forward."""
    scale = (1.1 if dtype == "float32" else 0.7) * (16 / dim) ** 0.5
    cfg = config(48, 61, [("attention", attention(4, 2, dim, vdim, scale, rot(8, 50.0, (4.0, 1.0, 2.0, 16)), conv=3), None)])
    w = pb.random_weights(cfg, seed=5)
    w["l0.mix.talk"] = torch.tensor([[0.2, 0.9, -0.4, 0.3], [0.0, 1.0, 0.0, 0.0], [0.5, 0.1, 0.6, -0.2],
                                     [-0.3, 0.2, 0.8, 0.3]])
    w["l0.mix.o"] = w["l0.mix.o"] * 2.5  # (the mixer's share of the stream beside the embedding)
    return cfg, cast(w, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("dim,vdim", [(16, 12), (64, 64), (128, 128)])  # the last two: tensor-core kernels in bfloat16
def test_far_keys_and_mixed_heads_over_two_kv_heads(tmp_path, dtype, dim, vdim):
    """A causal layer over 300 tokens and many pages: the first tokens stay visible to the end, and the head
    mixer is no symmetric matrix, so its transpose, or a head that reads the other kv head's values, shows."""
    cfg, w = far_key_model(dtype, dim, vdim)
    n = 300
    # the test has power: the token at position 2 decides logits among the last twenty, three hundred keys later
    # (the first of a few token sequences for which it does), and so does the mixer's orientation
    for seed in range(8, 40):
        ids = random_ids(cfg["vocab"], n, seed)
        ref = oracle(ids, w, cfg)
        changed = list(ids)
        changed[2] = (ids[2] + 1) % cfg["vocab"]
        if (oracle(changed, w, cfg)[-20:] - ref[-20:]).abs().max() > 5 * TOL[dtype] * ref.abs().max():
            break
    else:
        raise AssertionError("no token sequence makes the key at position 2 decisive at the end")
    wt = dict(w)
    wt["l0.mix.talk"] = w["l0.mix.talk"].T.contiguous()
    assert (oracle(ids, wt, cfg) - ref).abs().max() > 5 * TOL[dtype] * ref.abs().max(), "the mixer's transpose must show"
    r = make_runner(tmp_path, cfg, w, 8, dtype, num_pages=40)
    plan = [[("a", 3)], [("a", 60)], [("a", 64)], [("a", 2)], [("a", 131)]] + [[("a", 1)] for _ in range(40)]
    got = replay(r, {"a": ids}, plan)["a"]
    assert_rows_close(got, ref, dtype, "far keys")


@pytest.mark.parametrize("dtype", ["float32"])
def test_state_layers_remember_far_tokens(tmp_path, dtype):
    """Decays close to one: what the token at position 2 wrote still decides the logits two hundred tokens later,
    through portions, decoding and a slot that held another request's state before."""
    cfg = config(40, 53, [("gla", gla(2, 12, 20, 4.0), None), ("gla", gla(1, 24, 8, 16.0), dense(48))], side=4)
    w = pb.random_weights(cfg, seed=21)
    for l in (0, 1):
        w[f"l{l}.mix.a2.b"] = torch.full_like(w[f"l{l}.mix.a2.b"], 7.0)   # decay about 1 - 1e-3 / tau
        w[f"l{l}.mix.a2"] = w[f"l{l}.mix.a2"] * 0.05
    w["embed"][51:] *= 6.0
    w = cast(w, dtype)
    n = 230
    ids = [t % 51 for t in random_ids(53, n, 13)]
    ids[2] = 51
    ref = oracle(ids, w, cfg)
    changed = list(ids)
    changed[2] = 52
    assert (oracle(changed, w, cfg)[-20:] - ref[-20:]).abs().max() > 5 * TOL[dtype] * ref.abs().max(), (
        "token 2 must matter at the end")
    r = make_runner(tmp_path, cfg, w, 16, dtype, num_pages=32, max_requests=2)
    got = replay(r, {"x": changed[:40], "a": ids}, [
        [("x", 40)],                                  # leaves state in slot 0, which "a" then takes
        [("a", 3)], [("a", 60)], [("a", 64)], [("a", 2)], [("a", 61)]] + [[("a", 1)] for _ in range(40)])
    assert_rows_close(got["a"], ref, dtype, "far memory")


def test_long_decoding_in_32_bit(tmp_path):
    """One prompt token, then 300 tokens one by one: windows slide over decoded tokens, pages come and go."""
    cfg, w, page = weights_for("B", "float32")
    r = make_runner(tmp_path, cfg, w, page, "float32", num_pages=90)
    ids = random_ids(cfg["vocab"], 301, 17)
    got = replay(r, {"a": ids}, [[("a", 1)] for _ in range(301)])["a"]
    assert_close(got, oracle(ids, w, cfg), "float32", "long decoding")


@pytest.mark.needs_cuda
def test_tensor_core_attention_agrees_with_the_general_kernel(tmp_path):
    """D in bfloat16 with the general path's tensor-core kernels on (the default) and off: the same logits within
    rounding, through a prompt, two portions and decoding; and the kernels that ran are the ones meant."""
    from ullm_b200.csrc import kernels

    cfg, w, page = weights_for("D", "bfloat16")
    ids = random_ids(cfg["vocab"], 90, 31)
    plan = [[("a", 50)], [("a", 2)], [("a", 20)]] + [[("a", 1)] for _ in range(18)]
    K = kernels()
    got = {}
    try:
        for on in (True, False):
            K.general_attention_tc = on
            r = make_runner(tmp_path, cfg, w, page, "bfloat16", name=f"tc{on}")
            got[on] = replay(r, {"a": ids}, plan)["a"]
            assert K.attention_path == ("decode" if on else "generic")
    finally:
        K.general_attention_tc = True
    ref = oracle(ids, w, cfg)
    assert_rows_close(got[True], ref, "bfloat16", "tensor-core kernels")
    assert_rows_close(got[False], ref, "bfloat16", "general kernel")
    mx, rms = errors(got[True], got[False])
    assert rms <= 1e-2, f"the two paths differ by {rms:.2e} rms of scale"


# ---------------------------------------------------------------------------------------------------------
# generation through the entry point and the scheduler
# ---------------------------------------------------------------------------------------------------------
def check_greedy(prompts, outs, w, cfg, count):
    wd = {n: t.double() for n, t in w.items()}
    for p, o in zip(prompts, outs):
        assert len(o.token_ids) == count
        seq = list(p)
        for tok in o.token_ids:
            lg = pb.forward(cfg, wd, seq)[-1]
            top2 = torch.topk(lg, 2).values
            if top2[0] - top2[1] > 1e-3 * lg.abs().max():
                assert tok == int(torch.argmax(lg)), f"prompt of {len(p)}: token {len(seq) - len(p)} differs"
            seq.append(tok)


@pytest.mark.parametrize("eager", [True, False])
@pytest.mark.parametrize("tag", ["A", "B"])
def test_greedy_generation_through_the_entry_point(tmp_path, tag, eager):
    """Five prompts, three request slots, a token budget of 16 per step: prompts are cut into portions and run
    beside decoding requests; decode steps come from CUDA graphs unless `eager`."""
    from ullm_b200 import LLM, EngineConfig, SamplingParams

    cfg, w, page = weights_for(tag, "float32")
    d = write_model(str(tmp_path / f"gen{tag}{eager}"), cfg, w)
    ec = EngineConfig(model=d, max_bs=3, context_len=128, page_size=page, num_pages=48, max_num_batched_tokens=16,
                      dtype="float32", enforce_eager=eager)
    if device() == "cpu":
        type(ec).device = property(lambda self: "cpu")
    llm = LLM(ec)
    prompts = [random_ids(cfg["vocab"], n, 90 + n) for n in (1, 6, 23, 40, 17)]
    outs = llm.generate_batch(prompts, SamplingParams(temperature=0.0, max_new_tokens=14, ignore_eos=True))
    check_greedy(prompts, outs, w, cfg, 14)
    llm.engine.runner.cache.check_invariants()


@pytest.mark.parametrize("eager", [True, False])
def test_preempted_requests_start_again_from_zeroed_state(tmp_path, eager):
    """A pool too small for three requests of about 60 tokens: some are preempted, take a slot again later (their
    state rows zeroed, their prompt and generated tokens recomputed) and still produce the plain model's tokens."""
    from ullm_b200 import LLM, EngineConfig, SamplingParams

    cfg, w, page = weights_for("B", "float32")
    d = write_model(str(tmp_path / f"pre{eager}"), cfg, w)
    ec = EngineConfig(model=d, max_bs=3, context_len=96, page_size=page, num_pages=34, max_num_batched_tokens=32,
                      dtype="float32", enforce_eager=eager)
    if device() == "cpu":
        type(ec).device = property(lambda self: "cpu")
    llm = LLM(ec)
    prompts = [random_ids(cfg["vocab"], n, 200 + n) for n in (30, 22, 35)]
    outs = llm.generate_batch(prompts, SamplingParams(temperature=0.0, max_new_tokens=30, ignore_eos=True))
    assert llm.engine.stats()["preemptions"] >= 1, "34 pages of 4 tokens cannot hold three requests of 52 to 65 tokens"
    check_greedy(prompts, outs, w, cfg, 30)
    llm.engine.runner.cache.check_invariants()
