"""The Ludalix decoder in the engine against the plain implementation (tests/plain_ludalix.py): each mechanism
alone, whole prompts against token-by-token decoding and portions down to two tokens, unequal batches with pages
and state slots that are used again, the edges of windows and of the kept first tokens (with weights made so
that one key decides), far memory of the state layers, long decoding, and greedy generation through the entry
point and the scheduler."""

import pytest
import torch

import plain_ludalix as pl
from conftest import device
from helpers import TOL, assert_close, errors, random_ids
from ludalix_helpers import (CONFIGS, assert_rows_close, router_margins, attention, config, dense, make_runner, mlstm, moe, oracle,
                             replay, weights_for)

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


# ---------------------------------------------------------------------------------------------------------
# each mechanism alone
# ---------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_embedding_with_added_sinusoid(tmp_path, dtype):
    from ullm_b200.engine import StepEntry

    cfg, w, page = weights_for("P", dtype)
    r = make_runner(tmp_path, cfg, w, page, dtype)
    ids = random_ids(cfg["vocab"], 30, 1)
    r.add_request("a")
    first = 0
    for a, b in ((0, 19), (19, 30)):  # the second portion starts at position 19
        ctx = r.prepare([StepEntry("a", ids[a:b], [])])
        stream = torch.empty(b - a, cfg["width"], dtype=torch.float32, device=r.device)
        copy = torch.empty(b - a, cfg["width"], dtype=r.dtype, device=r.device) if dtype != "float32" else None
        r.model.embedding.forward_stream(ctx.token_ids, stream, copy, ctx)
        ref = pl.embed(ids[a:b], w["embed"].double(), cfg["embedding"]["scale"], first_position=a).float()
        assert (stream.cpu() - ref).abs().max() <= 2e-6 * ref.abs().max(), "32-bit stream of the embedding"
        if copy is not None:
            assert torch.equal(copy.cpu(), stream.cpu().to(copy.dtype))
        r.commit([StepEntry("a", ids[a:b], [])])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tag,layer", [("P", 1), ("P", 3), ("Q", 0), ("R", 1), ("S", 0), ("S", 1)])
def test_mlstm_mixer_alone(tmp_path, dtype, tag, layer):
    """The mixer on random rows in three steps (13, 1 and 9 tokens) against the recurrence run whole."""
    from ullm_b200.engine import StepEntry

    cfg, w, page = weights_for(tag, dtype)
    r = make_runner(tmp_path, cfg, w, page, dtype)
    x = rand((23, cfg["width"]), 5, dtype)
    wd = {n: t.double() for n, t in w.items()}
    ref = pl.mlstm_mixer(x.double().cpu(), wd, f"l{layer}.mix.", cfg["layers"][layer]["mixer"], cfg["norm"]["eps"]).float()
    got = []
    r.add_request("a")
    for a, b in ((0, 13), (13, 14), (14, 23)):
        e = [StepEntry("a", [0] * (b - a), [])]
        ctx = r.prepare(e)
        caches = r.cache.layer_caches(ctx.groups)
        got.append(r.model.blocks[layer].mixer.forward(x[a:b].clone(), ctx, caches[layer]).float().cpu().clone())
        r.commit(e)
    r.check_device_status()
    close(torch.cat(got), ref, dtype, "mLSTM mixer")


def test_mlstm_gates_take_both_branches_of_the_running_maximum():
    """The oracle's own recurrence against a direct evaluation without any maximum, in 64-bit; and the case
    where the maximum stays at its start value 0 (all gates far below zero) against the case where it moves."""
    g = torch.Generator().manual_seed(3)
    T, Hn, d, dv = 17, 2, 5, 3
    q, k = torch.randn(T, Hn, d, generator=g).double(), torch.randn(T, Hn, d, generator=g).double()
    v = torch.randn(T, Hn, dv, generator=g).double()
    for shift in (-6.0, 3.0):
        i = torch.randn(T, Hn, generator=g).double() + shift
        f = -torch.rand(T, Hn, generator=g).double()
        o = pl.mlstm_recurrence(q, k, v, i, f)
        F = torch.cumsum(f, 0)
        for t in (0, 5, T - 1):
            for h in range(Hn):
                wgt = torch.exp(F[t, h] - F[: t + 1, h] + i[: t + 1, h])  # unnormalized weights of the pairs
                S = torch.einsum("s,sd,sv->dv", wgt, k[: t + 1, h], v[: t + 1, h])
                n = torch.einsum("s,sd->d", wgt, k[: t + 1, h])
                m = torch.maximum(torch.cummax(F[t, h] - F[: t + 1, h] + i[: t + 1, h], 0).values[-1], F[t, h])
                m = torch.maximum(m, torch.tensor(0.0).double() + F[t, h])
                # the running maximum started at 0: m_t = max(F_t, max_s(F_t - F_s + i_s))
                den = torch.maximum((n @ q[t, h]).abs() * torch.exp(-m), torch.exp(-m)) + 1e-6
                ref = (S.T @ q[t, h]) * torch.exp(-m) / den
                assert torch.allclose(o[t, h], ref, rtol=1e-9, atol=1e-12), (shift, t, h)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tag,layer", [("P", 0), ("Q", 1), ("R", 0)])
def test_attention_mixer_alone(tmp_path, dtype, tag, layer):
    """Keys wider or narrower than values, as many kv heads as heads, kept tokens beyond the window: 37 tokens,
    then 2, then 1 more."""
    from ullm_b200.engine import StepEntry

    cfg, w, page = weights_for(tag, dtype)
    r = make_runner(tmp_path, cfg, w, page, dtype)
    n = 40
    x = rand((n, cfg["width"]), 6, dtype)
    wd = {k: t.double() for k, t in w.items()}
    mix, eps, pre = cfg["layers"][layer]["mixer"], cfg["norm"]["eps"], f"l{layer}.mix."
    xd = x.double().cpu()
    ref = pl.attention_mixer(xd, wd, pre, mix, eps, pl.attention_keys_values(xd, wd, pre, mix, eps)).float()
    got = []
    r.add_request("a")
    for a, b in ((0, 37), (37, 39), (39, 40)):
        e = [StepEntry("a", [0] * (b - a), [])]
        ctx = r.prepare(e)
        caches = r.cache.layer_caches(ctx.groups)
        got.append(r.model.blocks[layer].mixer.forward(x[a:b].clone(), ctx, caches[layer]).float().cpu().clone())
        r.commit(e)
    r.check_device_status()
    close(torch.cat(got), ref, dtype, "attention mixer")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_feed_forwards_alone(tmp_path, dtype):
    from ullm_b200.engine.batch import Workspace

    for tag, layers in (("P", (0, 2, 3)), ("Q", (0, 1)), ("R", (1,))):
        cfg, w, page = weights_for(tag, dtype)
        r = make_runner(tmp_path, cfg, w, page, dtype, name=tag)

        class Ctx:
            workspace = Workspace(r.device, max_tokens=32, max_requests=4)

        x = rand((21, cfg["width"]), 8, dtype, 1.5)
        wd = {k: t.double() for k, t in w.items()}
        for l in layers:
            mlp = cfg["layers"][l]["mlp"]
            ref = pl.feed_forward(x.double().cpu(), wd, f"l{l}.mlp.", mlp).float()
            got = r.model.blocks[l].feed_forward.forward(x.clone(), Ctx())
            if mlp["kind"] == "moe" and dtype != "float32":
                # a close call of the router may fall the other way after rounding: compare the rows that agree
                s = torch.sigmoid(x.double().cpu() @ wd[f"l{l}.mlp.router"].T).sort(-1, descending=True).values
                top = mlp["router"]["top"]
                clear = (s[:, top - 1] - s[:, top]).abs() > 0.02 if top < s.shape[1] else torch.ones(21, dtype=torch.bool)
                assert clear.sum() >= 10
                close(got.float().cpu()[clear], ref[clear], dtype, f"{tag} layer {l} {mlp['kind']}")
            else:
                close(got, ref, dtype, f"{tag} layer {l} {mlp['kind']}")


@pytest.mark.needs_cuda
def test_routed_experts_on_tensor_cores_agree_with_the_plain_grouped_product(tmp_path):
    """Sizes that allow 16-byte pieces take the tensor-core grouped product in bfloat16; the same step with that
    kernel switched off must give the same rows up to the order of additions, and both follow the plain model.
    300 and 90 tokens over 5 experts: tiles of 64 places with ragged ends, and an expert's columns that end inside
    a tile."""
    from ullm_b200.csrc import kernels
    from ullm_b200.engine.batch import Workspace

    cfg = config(72, 64, [("mlstm", mlstm(1, 8, 8, 5.0), moe(5, 2, 88))])
    w = {n: t.to(torch.bfloat16) for n, t in pl.random_weights(cfg, seed=8).items()}
    r = make_runner(tmp_path, cfg, w, 8, "bfloat16")

    class Ctx:
        workspace = Workspace(r.device, max_tokens=320, max_requests=4)

    ff = r.model.blocks[0].feed_forward
    for rows in (300, 90):
        x = rand((rows, 72), 3 + rows, "bfloat16", 1.5)
        fast = ff.forward(x.clone(), Ctx()).float().cpu().clone()
        kernels().moe_force_plain(True)
        try:
            slow = ff.forward(x.clone(), Ctx()).float().cpu().clone()
        finally:
            kernels().moe_force_plain(False)
        assert (fast - slow).abs().max() <= 2e-2 * slow.abs().max()
        ref = pl.feed_forward(x.double().cpu(), {n: t.double() for n, t in w.items()}, "l0.mlp.",
                              cfg["layers"][0]["mlp"]).float()
        s = torch.sigmoid(x.double().cpu() @ w["l0.mlp.router"].double().T).sort(-1, descending=True).values
        clear = (s[:, 1] - s[:, 2]) > 0.005
        assert clear.sum() > 0.75 * rows
        assert_close(fast[clear], ref[clear], "bfloat16", f"routed experts on tensor cores, {rows} rows")


def test_router_weight_multiplies_the_experts_input_not_its_output():
    """The oracle's own reading: with one expert per token the two readings differ, and the engine follows the
    first (checked through the whole model elsewhere; here the plain functions are pinned)."""
    cfg, w, _ = weights_for("Q", "float32")
    wd = {k: t.double() for k, t in w.items()}
    x = torch.randn(6, cfg["width"], generator=torch.Generator().manual_seed(2)).double()
    pre = "l1.mlp."
    score, index = pl.router_choice(x, wd, pre, 1)
    on_input = pl.moe_ff(x, wd, pre, 4, 1)
    on_output = torch.stack([score[t, 0] * pl.expert_ff(x[t], wd, f"{pre}e{int(index[t, 0])}.") for t in range(6)])
    assert (on_input - on_output).abs().max() > 1e-3 * on_input.abs().max()


# ---------------------------------------------------------------------------------------------------------
# whole prompts, token-by-token decoding, portions
# ---------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tag", ["P", "Q", "R", "S", "T"])
def test_whole_decode_and_portions_agree_with_the_plain_model(tmp_path, dtype, tag):
    cfg, w, page = weights_for(tag, dtype)
    r = make_runner(tmp_path, cfg, w, page, dtype)
    n = 75 if tag != "T" else 150  # (T: the windows of 40 and 100 must pass over prompt and decoded tokens)
    ids = random_ids(cfg["vocab"], n, 11)
    ref = oracle(ids, w, cfg)
    margins = router_margins(ids, w, cfg)
    plans = {
        "whole": [[("a", n)]],
        "decode": [[("b", 3)]] + [[("b", 1)] for _ in range(n - 3)],
        "portions": [[("c", k)] for k in (2, 2, 3, 7, 2, 16, 1, 1, 2, 31, 8) + ((70, 5) if n == 150 else ())],
        "one by one": [[("d", 1)] for _ in range(n)],
    }
    assert sum(k for (_, k), in plans["portions"]) == n
    for name, plan in plans.items():
        rid = plan[0][0][0]
        got = replay(r, {rid: ids}, plan)[rid]
        assert_rows_close(got, ref, dtype, f"{tag} {name}", margins)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unequal_batches_with_pages_and_slots_used_again(tmp_path, dtype):
    """Three state slots and a pool that cannot hold all requests at once: six requests of unequal length come
    and go, portions of some beside single tokens of others; every request equals itself run alone."""
    cfg, w, page = weights_for("P", dtype)
    r = make_runner(tmp_path, cfg, w, page, dtype, num_pages=22, max_requests=3)
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
        assert_rows_close(got[k], oracle(reqs[k], w, cfg), dtype, f"request {k}", router_margins(reqs[k], w, cfg))
    assert not r.cache.requests and r.cache.num_free_pages(0) == 22


# ---------------------------------------------------------------------------------------------------------
# edges: the window, the kept first tokens, page borders; weights made so that one key decides
# ---------------------------------------------------------------------------------------------------------
def one_key_model(size, keep_first, dtype, page, dim=32, vdim=24):
    """One attention layer without feed-forward whose query norm is scaled up: the softmax is nearly one-hot, so
    a key that is wrongly seen or wrongly hidden changes the logits by much more than any tolerance."""
    cfg = config(48, 61, [("attention", attention(2, 1, dim, vdim, size, keep_first, 1.0), None)], mult=1.0, scale=3.0)
    w = pl.random_weights(cfg, seed=size * 31 + keep_first)
    w["l0.mix.q.norm"] = w["l0.mix.q.norm"] * (4.0 if dtype == "float32" else 2.5)
    if dtype != "float32":
        w = {n: t.to(getattr(torch, dtype)) for n, t in w.items()}
    return cfg, w


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("size,keep_first", [(8, 3), (16, 0), (5, 16), (17, 9)])
@pytest.mark.parametrize("dim,vdim", [(32, 24), (64, 64)])  # the second: the sizes the tensor-core kernels take
def test_window_and_kept_tokens_edges_in_prompts_and_decoding(tmp_path, dtype, size, keep_first, dim, vdim):
    page = 8
    cfg, w = one_key_model(size, keep_first, dtype, page, dim, vdim)
    n = 70
    # the test has power: a window one token longer or shorter, or one kept token more or less, is far off
    # (the first of a few token sequences for which all four are)
    for seed in range(5, 25):
        ids = random_ids(cfg["vocab"], n, seed)
        ref = oracle(ids, w, cfg)
        offs = []
        for ds, dk in ((1, 0), (-1, 0), (0, 1), (0, -1)):
            if keep_first + dk < 0:
                continue
            other = config(48, 61, [("attention", attention(2, 1, dim, vdim, size + ds, keep_first + dk, 1.0), None)],
                           mult=1.0, scale=3.0)
            offs.append(float((oracle(ids, w, other) - ref).abs().max() / ref.abs().max()))
        if min(offs) > 5 * TOL[dtype]:
            break
    else:
        raise AssertionError(f"no token sequence makes every edge decisive (last: {offs})")
    r = make_runner(tmp_path, cfg, w, page, dtype, num_pages=12)
    # portions that end on, one before and one after page borders and window edges; then single tokens
    plan = [[("a", k)] for k in (7, 1, 1, 8, 9, 2, size, 3)]
    used = sum(k for (_, k), in plan)
    plan += [[("a", 1)] for _ in range(n - used)]
    got = replay(r, {"a": ids}, plan)["a"]
    assert_close(got, ref, dtype, f"window {size}, first {keep_first} kept")
    # pages that the window left behind went back to the pool while the request ran, the kept ones did not
    assert r.cache.num_free_pages(0) == 12


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_borrowed_keys_and_values_follow_the_reader_with_the_larger_window(tmp_path, dtype):
    """Layer 1 reads layer 0's keys and values under a window four times as long: the pages must stay as long as
    the reader reaches them, and its own mask decides what it sees."""
    cfg = config(48, 61, [("attention", attention(3, 3, 16, 16, 6, 0, 0.6), None),
                          ("attention", attention(3, 3, 16, 16, 24, 5, 0.6, kv_from=0), None)], mult=1.0, scale=3.0)
    w = pl.random_weights(cfg, seed=77)
    for l in (0, 1):
        w[f"l{l}.mix.q.norm"] = w[f"l{l}.mix.q.norm"] * (3.0 if dtype == "float32" else 2.0)
    if dtype != "float32":
        w = {n: t.to(getattr(torch, dtype)) for n, t in w.items()}
    ids = random_ids(61, 66, 9)
    ref = oracle(ids, w, cfg)
    same_mask = config(48, 61, [("attention", attention(3, 3, 16, 16, 6, 0, 0.6), None),
                                ("attention", attention(3, 3, 16, 16, 6, 0, 0.6, kv_from=0), None)], mult=1.0, scale=3.0)
    assert (oracle(ids, w, same_mask) - ref).abs().max() > 5 * TOL[dtype] * ref.abs().max()
    r = make_runner(tmp_path, cfg, w, 4, dtype, num_pages=20)
    assert len(r.cache.groups) == 1 and r.cache.groups[0].need.window == 24 and r.cache.groups[0].need.keep_first == 5
    plan = [[("a", 30)], [("a", 2)]] + [[("a", 1)] for _ in range(34)]
    assert_close(replay(r, {"a": ids}, plan)["a"], ref, dtype, "reader with the larger window")


@pytest.mark.parametrize("dtype", ["float32"])
def test_state_layers_remember_far_tokens(tmp_path, dtype):
    """(32-bit only: with the state all but one outer product, a head's normed read-out is a sign times a fixed
    vector, and a 16-bit rounding of q or k may flip the sign.  The state path in 16 bits is covered by the
    schedule tests above.)  Forget gates close to one, and input gates that open wide for one marked token only (its embedding points
    along the input gate's weight): what the token at position 2 wrote dominates the state two hundred tokens
    later, through portions, decoding and a slot that held another request's state before."""
    cfg = config(40, 53, [("mlstm", mlstm(2, 12, 20, 6.0), None), ("mlstm", mlstm(1, 24, 8, 6.0), dense(48, 2.0))],
                 mult=0.9, scale=2.0)
    w = pl.random_weights(cfg, seed=21)
    u = torch.nn.functional.normalize(torch.randn(40, generator=torch.Generator().manual_seed(4)), dim=0)
    marked = (51, 52)
    for z in marked:
        w["embed"][z] += 40.0 * u / cfg["embedding"]["scale"]
    w["l0.mix.i"] = 0.5 * u.repeat(2, 1)
    w["l0.mix.i.b"] = torch.full_like(w["l0.mix.i.b"], -3.0)
    for l in (0, 1):
        w[f"l{l}.mix.f.b"] = torch.full_like(w[f"l{l}.mix.f.b"], 5.5)   # log forget gate about -0.004
        w[f"l{l}.mix.f"] = w[f"l{l}.mix.f"] * 0.05
    if dtype != "float32":
        w = {n: t.to(getattr(torch, dtype)) for n, t in w.items()}
    n = 230
    ids = [t % 51 for t in random_ids(53, n, 13)]
    ids[2] = marked[0]
    ref = oracle(ids, w, cfg)
    changed = list(ids)
    changed[2] = marked[1]
    assert (oracle(changed, w, cfg)[-20:] - ref[-20:]).abs().max() > 5 * TOL[dtype] * ref.abs().max(), (
        "token 2 must matter at the end")
    r = make_runner(tmp_path, cfg, w, 16, dtype, num_pages=32, max_requests=2)
    got = replay(r, {"x": changed[:40], "a": ids}, [
        [("x", 40)],                                  # leaves state in slot 0, which "a" then takes
        [("a", 3)], [("a", 60)], [("a", 64)], [("a", 2)], [("a", 61)]] + [[("a", 1)] for _ in range(40)])
    assert_rows_close(got["a"], ref, dtype, "far memory")


def test_long_decoding_in_32_bit(tmp_path):
    """One prompt token, then 300 tokens one by one: windows slide over decoded tokens, pages come and go."""
    cfg, w, page = weights_for("Q", "float32")
    r = make_runner(tmp_path, cfg, w, page, "float32", num_pages=90)
    ids = random_ids(cfg["vocab"], 301, 17)
    got = replay(r, {"a": ids}, [[("a", 1)] for _ in range(301)])["a"]
    assert_close(got, oracle(ids, w, cfg), "float32", "long decoding")


# ---------------------------------------------------------------------------------------------------------
# generation through the entry point and the scheduler
# ---------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("eager", [True, False])
@pytest.mark.parametrize("tag", ["P", "R"])
def test_greedy_generation_through_the_entry_point(tmp_path, tag, eager):
    """Five prompts under a token budget of 16 and three request slots (prompts are cut into portions, requests
    wait for a slot, decode steps are replayed from CUDA graphs unless eager), greedy, against the plain model
    run on the growing sequence.  A step's choice is compared only where the plain model's margin is clear."""
    from helpers import write_model_dir  # noqa: F401  (same folder layout)
    from ludalix_helpers import write_model
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
    wd = {n: t.double() for n, t in w.items()}
    for p, o in zip(prompts, outs):
        assert len(o.token_ids) == 14
        seq = list(p)
        for tok in o.token_ids:
            lg = pl.forward_logits(seq, wd, cfg)[-1]
            top2 = torch.topk(lg, 2).values
            if top2[0] - top2[1] > 1e-3 * lg.abs().max():
                assert tok == int(torch.argmax(lg)), f"prompt of {len(p)}: token {len(seq) - len(p)} differs"
            seq.append(tok)
    llm.engine.runner.cache.check_invariants()


@pytest.mark.parametrize("eager", [True, False])
def test_preempted_requests_start_again_from_zeroed_state(tmp_path, eager):
    """A pool too small for three requests of about 60 tokens: some are preempted, take a slot again later (their
    state rows zeroed, their prompt and generated tokens recomputed) and still produce the plain model's tokens."""
    from ludalix_helpers import write_model
    from ullm_b200 import LLM, EngineConfig, SamplingParams

    cfg, w, page = weights_for("Q", "float32")
    d = write_model(str(tmp_path / f"pre{eager}"), cfg, w)
    ec = EngineConfig(model=d, max_bs=3, context_len=96, page_size=page, num_pages=34, max_num_batched_tokens=32,
                      dtype="float32", enforce_eager=eager)
    if device() == "cpu":
        type(ec).device = property(lambda self: "cpu")
    llm = LLM(ec)
    prompts = [random_ids(cfg["vocab"], n, 200 + n) for n in (30, 22, 35)]
    outs = llm.generate_batch(prompts, SamplingParams(temperature=0.0, max_new_tokens=30, ignore_eos=True))
    assert llm.engine.stats()["preemptions"] >= 1, "34 pages of 4 tokens cannot hold three requests of 52 to 65 tokens"
    wd = {n: t.double() for n, t in w.items()}
    for p, o in zip(prompts, outs):
        assert len(o.token_ids) == 30
        seq = list(p)
        for tok in o.token_ids:
            lg = pl.forward_logits(seq, wd, cfg)[-1]
            top2 = torch.topk(lg, 2).values
            if top2[0] - top2[1] > 1e-3 * lg.abs().max():
                assert tok == int(torch.argmax(lg)), f"prompt of {len(p)}: token {len(seq) - len(p)} differs"
            seq.append(tok)
    llm.engine.runner.cache.check_invariants()
