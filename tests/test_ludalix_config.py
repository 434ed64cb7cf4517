"""Host-side pieces of the Ludalix decoder that need no GPU: the config.json reader, the tensor names the model
declares, what the cache manager plans for windows with kept first tokens and for borrowed keys and values, and
the state rows."""

import copy

import pytest
import torch

import plain_ludalix as pl
from ludalix_helpers import CFG_P, CFG_Q, CFG_R


def test_the_model_declares_exactly_the_checkpoints_tensors():
    from ullm_b200.config import load_model_spec
    from ullm_b200.parts.model import DecoderModel

    for cfg in (CFG_P, CFG_Q, CFG_R):
        _, spec = load_model_spec(copy.deepcopy(cfg))
        model = DecoderModel(spec)
        got = {n: tuple(d.shape) for n, d in model.all_decls().items()}
        assert got == pl.tensor_shapes(cfg)
        assert spec.stream_dtype == "float32" and spec.embedding_scale == cfg["embedding"]["scale"]
        assert [e.cache_of for e in spec.schedule] == [L["mixer"].get("kv_from") for L in cfg["layers"]]


def test_allocated_tensors_have_the_declared_names_and_32_bit_where_the_arithmetic_is():
    from ullm_b200.config import load_model_spec
    from ullm_b200.parts.model import DecoderModel

    _, spec = load_model_spec(copy.deepcopy(CFG_P))
    model = DecoderModel(spec)
    model.allocate("cpu", torch.bfloat16)
    t = model.all_tensors()
    assert {n: tuple(v.shape) for n, v in t.items()} == pl.tensor_shapes(CFG_P)
    for n, v in t.items():
        is32 = n.endswith(("norm1", "norm2", ".norm", "i.b", "f.b"))
        assert v.dtype == (torch.float32 if is32 else torch.bfloat16), n


@pytest.mark.parametrize("change,needle", [
    (lambda c: c.pop("width"), "width"),
    (lambda c: c["embedding"].pop("scale"), "scale"),
    (lambda c: c["layers"][0].update(type="conv"), "type"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "multiple"),
    (lambda c: c["layers"][0]["mixer"]["mask"].pop("size"), "size"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=1), "no keys"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=2), "earlier"),
    (lambda c: c["layers"][2]["mixer"].update(vdim=8), "differ"),
    (lambda c: c["layers"][1]["mixer"].pop("gate_cap"), "gate_cap"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=9), "top"),
    (lambda c: c["layers"][2]["mlp"].update(limit=0), "limit"),
])
def test_config_errors_name_the_key(change, needle):
    from ullm_b200.config import LudalixConfigError, load_model_spec

    cfg = copy.deepcopy(CFG_P)
    change(cfg)
    with pytest.raises(LudalixConfigError, match=needle):
        load_model_spec(cfg)


def _needs(cfg):
    from ullm_b200.config import load_model_spec
    from ullm_b200.parts.model import DecoderModel

    _, spec = load_model_spec(copy.deepcopy(cfg))
    return DecoderModel(spec).cache_needs()


def test_a_borrowed_cache_is_kept_for_its_widest_reader_and_state_layers_ask_for_rows():
    from ullm_b200.cache import plan_groups
    from ullm_b200.parts.mlstm import mlstm_state_floats

    needs = _needs(CFG_P)
    groups, where = plan_groups(needs)
    # layer 0 writes (window 9, 3 kept), layer 2 reads it under a window of 17 with none kept
    assert len(groups) == 1 and groups[0].need.window == 17 and groups[0].need.keep_first == 3
    assert groups[0].need.head_dim == 24 and groups[0].need.v_dim == 40
    assert where[0] == where[2] == (0, 0) and where[1] is None and where[3] is None
    assert needs[1][1].shape == (mlstm_state_floats(3, 20, 28),) and needs[3][1].shape == (2 * 16 * 40 + 2 * 40 + 2,)
    assert needs[0][1] is None


def test_pages_behind_the_window_go_back_but_not_those_of_the_kept_tokens():
    from ullm_b200.cache import CacheManager
    from ullm_b200.parts.base import CacheNeed

    need = CacheNeed(2, 8, window=10, value_dim=12, keep_first=5)
    cm = CacheManager([(need, None, None)], page_size=4, num_pages=16, max_requests=2, max_pages_per_request=16)
    rc = cm.admit("a")
    for n in (3, 9, 1, 20, 1, 1):
        cm.reserve(rc, n)
        cm.commit(rc, n)
        cm.check_invariants()
        held = [i for i, p in enumerate(rc.pages[0]) if p >= 0]
        # pages 0 and 1 hold positions 0..4; the next token (position num_tokens) reaches back to num_tokens - 9
        first_window_page = max(0, rc.num_tokens - 10 + 1) // 4
        assert held[:2] == [0, 1][: len(held)]
        assert all(i < 2 or i >= first_window_page for i in held)
        assert all(i in held for i in range(first_window_page, -(-rc.num_tokens // 4)))
    cm.release(rc)
    assert cm.num_free_pages(0) == 16
    assert CacheManager.bytes_per_page([(need, None, None)], 4, 2) == 4 * 2 * (8 + 12) * 2
