"""Host-side pieces of the Borosun decoder that need no GPU: the config.json reader, the tensor names the model
declares, the sizes a tensor's shape gives, the cache groups and state rows, and the rotation's frequencies."""

import copy
import math

import pytest
import torch

import plain_borosun as pb
from borosun_helpers import CFG_A, CFG_B, CFG_C, weights_for, write_model


def test_the_model_declares_exactly_the_checkpoints_tensors():
    from ullm_b200.config import load_model_spec
    from ullm_b200.parts.model import DecoderModel

    for cfg in (CFG_A, CFG_B, CFG_C):
        _, spec = load_model_spec(copy.deepcopy(cfg))
        model = DecoderModel(spec)
        got = {n: tuple(d.shape) for n, d in model.all_decls().items()}
        assert got == pb.tensor_shapes(cfg, decay_rank=16)
        assert spec.stream_dtype == "float32" and spec.tie_embeddings
        assert spec.logit_softcap == cfg.get("logit_softcap")
        assert (spec.token_side is None) == ("token_side" not in cfg)


def test_the_decay_projections_inner_size_is_read_from_the_files(tmp_path):
    from ullm_b200.config import load_model_spec
    from ullm_b200.parts.model import DecoderModel

    cfg, w, _ = weights_for("A", "float32")
    d = write_model(str(tmp_path / "m"), cfg, w)
    _, spec = load_model_spec(d)
    got = {n: tuple(x.shape) for n, x in DecoderModel(spec).all_decls().items()}
    assert got == {n: tuple(t.shape) for n, t in w.items()}
    assert spec.layers[1].mixer.args["decay_rank"] == 5


def test_allocated_tensors_are_32_bit_where_the_arithmetic_is():
    from ullm_b200.config import load_model_spec
    from ullm_b200.parts.model import DecoderModel

    _, spec = load_model_spec(copy.deepcopy(CFG_A))
    model = DecoderModel(spec)
    model.allocate("cpu", torch.bfloat16)
    for n, v in model.all_tensors().items():
        is32 = n.endswith(("norm1", ".norm", "rg1.b", "rg2.b", "a2.b", "talk", "vmix"))
        assert v.dtype == (torch.float32 if is32 else torch.bfloat16), n


def test_which_layer_leaves_its_values_and_which_mix_them_in():
    from ullm_b200.config import load_model_spec

    _, spec = load_model_spec(copy.deepcopy(CFG_B))
    assert [L.mixer.args.get("value_mix") for L in spec.layers] == ["first", "mix", "mix", None]
    _, spec = load_model_spec(copy.deepcopy(CFG_C))
    assert [L.mixer.args.get("value_mix") for L in spec.layers] == [None, None, None, None]


def test_cache_groups_and_state_rows():
    from ullm_b200.cache.manager import plan_groups
    from ullm_b200.config import load_model_spec
    from ullm_b200.parts.model import DecoderModel

    _, spec = load_model_spec(copy.deepcopy(CFG_A))
    needs = DecoderModel(spec).cache_needs()
    groups, where = plan_groups(needs)
    assert [(g.need.window, g.need.head_dim, g.need.v_dim) for g in groups] == [(None, 24, 20), (9, 32, 20)]
    assert where[1] is None and where[3] is None
    # the convolved attention keeps taps - 1 projected rows, a state layer its matrices
    assert needs[0][1].shape == (3 * (4 * 24 + 2 * 24 + 2 * 20),)
    assert needs[1][1].shape == (3 * 20 * 28,) and needs[2][1] is None
    _, spec = load_model_spec(copy.deepcopy(CFG_B))
    needs = DecoderModel(spec).cache_needs()
    assert needs[1][1].shape == (3 * 16 + 3 * 16 + 3 * 8,) and needs[2][1] is None  # two taps: one row; one tap: none


@pytest.mark.parametrize("change,needle", [
    (lambda c: c.pop("width"), "width"),
    (lambda c: c["norm"].pop("eps"), "eps"),
    (lambda c: c["layers"][0].update(type="conv"), "type"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "multiple"),
    (lambda c: c["layers"][2]["mixer"]["mask"].pop("size"), "size"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=26), "dims"),
    (lambda c: c["layers"][0]["mixer"]["rot"]["scaling"].pop("low"), "low"),
    (lambda c: c["layers"][1]["mixer"].pop("tau"), "tau"),
    (lambda c: c["layers"][2]["mixer"].update(vdim=8), "value mixing"),
    (lambda c: c["layers"][0]["mlp"].update(kind="moe"), "kind"),
    (lambda c: c.update(logit_softcap=0), "logit_softcap"),
    (lambda c: c["token_side"].update(dim=0), "dim"),
])
def test_config_errors_name_the_key(change, needle):
    from ullm_b200.config import BorosunConfigError, load_model_spec

    cfg = copy.deepcopy(CFG_A)
    change(cfg)
    with pytest.raises(BorosunConfigError, match=needle):
        load_model_spec(cfg)


def test_rescaled_frequencies_keep_short_waves_slow_long_ones_and_blend_between():
    from ullm_b200.parts.position import scaled_frequencies

    dims, base = 32, 1000.0
    plain = scaled_frequencies(dims, base)
    assert torch.allclose(plain, torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=torch.float64))
    factor, low, high, orig = 4.0, 1.0, 4.0, 64
    f = scaled_frequencies(dims, base, dict(factor=factor, low=low, high=high, original=orig))
    kinds = set()
    for a, b in zip(plain.tolist(), f.tolist()):
        wave = 2 * math.pi / a
        if wave < orig / high:
            assert b == a
            kinds.add("kept")
        elif wave > orig / low:
            assert abs(b - a / factor) < 1e-15
            kinds.add("slowed")
        else:
            s = (orig / wave - low) / (high - low)
            assert abs(b - ((1 - s) * a / factor + s * a)) < 1e-15 and a / factor <= b <= a
            kinds.add("blended")
    assert kinds == {"kept", "slowed", "blended"}
    assert torch.equal(f, pb.rotary_frequencies(dims, base, dict(factor=factor, low=low, high=high, original=orig)))


def test_plain_recurrence_equals_the_sum_over_decayed_pairs():
    """The oracle's own state recurrence against the closed form o_t = sum_s (prod_{s<u<=t} alpha_u * k_s) . q_t v_s."""
    g = torch.Generator().manual_seed(3)
    T, N, d, dv = 11, 2, 5, 3
    q, k = torch.randn(T, N, d, generator=g).double(), torch.randn(T, N, d, generator=g).double()
    v = torch.randn(T, N, dv, generator=g).double()
    alpha = torch.rand(T, N, d, generator=g).double() * 0.5 + 0.5
    o = pb.gla_recurrence(q, k, v, alpha)
    for t in (0, 4, T - 1):
        ref = torch.zeros(N, dv).double()
        for s in range(t + 1):
            decay = alpha[s + 1:t + 1].prod(0) if s < t else torch.ones(N, d).double()
            ref += ((decay * k[s] * q[t]).sum(-1))[:, None] * v[s]
        assert torch.allclose(o[t], ref, rtol=1e-10, atol=1e-12)


def test_plain_convolution_reads_only_the_past():
    u = torch.arange(12.0).view(6, 2)
    w = torch.tensor([[1.0, 10.0, 100.0], [0.0, 0.0, 1.0]])
    y = pb.short_conv(u, w)
    assert torch.equal(y[:, 1], u[:, 1])  # a filter that keeps the present tap only
    assert y[0, 0] == 100 * u[0, 0] and y[2, 0] == u[0, 0] + 10 * u[1, 0] + 100 * u[2, 0]


def test_random_model_folder_round_trip(tmp_path):
    """`random-model` writes a folder from the configuration alone; reading it back finds every size again,
    the decay projection's inner size from the tensor it wrote."""
    import json

    from ullm_b200.config import load_model_spec
    from ullm_b200.engine.cli import main
    from ullm_b200.parts.model import DecoderModel
    from ullm_b200.weights.safetensors_io import open_model_files

    cfg = copy.deepcopy(CFG_B)
    cfg["layers"][3]["mixer"]["decay_rank"] = 7
    path = tmp_path / "cfg.json"
    path.write_text(json.dumps(cfg))
    out = str(tmp_path / "model")
    assert main(["random-model", "--out", out, "--config", str(path), "--seed", "3", "--dtype", "bfloat16"]) == 0
    files = open_model_files(out)
    shapes = {n: tuple(f.shape(n)) for f in files for n in f.names()}
    for f in files:
        f.close()
    assert shapes == pb.tensor_shapes(cfg)
    assert shapes["l3.mix.a1"] == (7, cfg["width"])
    del cfg["layers"][3]["mixer"]["decay_rank"]  # a folder made elsewhere does not carry the key
    (tmp_path / "model" / "config.json").write_text(json.dumps(cfg))
    _, spec = load_model_spec(out)
    assert {n: tuple(d.shape) for n, d in DecoderModel(spec).all_decls().items()} == shapes
