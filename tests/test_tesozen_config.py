"""Tesozen on the host: configuration, registry, the model as data, cache groups, tensor names, the pages that
a chunked attention holds, and the plain implementation's own routing and recurrence."""

import copy

import numpy as np
import pytest
import torch

import plain_tesozen as plain

_MOE = {"kind": "moe", "router": {"experts": 8, "top": 2, "scale": 1.5, "groups": {"count": 4, "keep": 2}},
        "expert": {"ff": 24}, "shared": {"ff": 40}}
_ATT = {"type": "attention", "mlp": {"kind": "dense", "ff": 56},
        "mixer": {"heads": 6, "kv_heads": 3, "dim": 12, "vdim": 20, "scale": 0.3, "diff": 0.25, "mask": {"size": 21}}}
_MLSTM = {"type": "mlstm", "mlp": _MOE, "mixer": {"heads": 3, "dim": 10, "vdim": 14, "gate_cap": 9.0}}
_LAT = {"type": "latent_attention", "mlp": None, "mixer": {"heads": 5, "dim": 12, "vdim": 8, "kv_rank": 24, "scale": 0.2}}
BASE = {"architecture": "Tesozen", "vocab": 97, "width": 48, "norm": {"eps": 1e-5}, "embedding": {"scale": 3.0},
        "layers": [_MLSTM, _ATT, _LAT, _ATT, _MLSTM]}


def build(document, dtype=torch.bfloat16):
    from ayaka_py_b200 import models, parts  # noqa: F401
    from ayaka_py_b200.models.model import Model
    from ayaka_py_b200.registry import architecture_for
    arch = architecture_for(document)
    config = arch.config_class.from_dict(document)
    return arch, config, Model(arch.build_spec(config), dtype, "meta")


def test_registry_and_round_trip():
    arch, config, _ = build(BASE)
    assert arch.name == "Tesozen"
    again = arch.config_class.from_dict(config.to_dict())
    assert again.to_dict() == config.to_dict() and again.to_dict()["architecture"] == "Tesozen"


def test_tensor_names_and_shapes():
    arch, config, model = build(BASE)
    rows = {r.source.name: tuple(r.decl.shape) for r in model.tensor_rows()}
    assert rows == plain.tensor_shapes(BASE)
    # the head is the embedding table itself
    assert [r.source.name for r in model.tensor_rows() if r.part is model.head] == ["embed"]
    # a layer without feed-forward has neither its tensors nor its two norms, and passes them over in a checkpoint
    assert "l2.norm2" not in rows and "l2.norm2.b" not in rows and "l1.norm2b.b" in rows
    assert arch.normalize_name("l2.norm2b.b", config) is None and arch.normalize_name("l1.norm2b", config) == "l1.norm2b"
    assert arch.normalize_name("l2.mlp.up", config) is None and arch.normalize_name("embed", config) == "embed"


def test_cache_groups_and_constants():
    from ayaka_py_b200.parts import KVNeed, StateNeed
    _, _, model = build(BASE)
    assert [b.KIND for b in model.blocks] == ["double_norm", "double_norm", "double_norm_mixer_only", "double_norm", "double_norm"]
    needs = {g.need: g.layers for g in model.groups}
    assert needs == {StateNeed((3, 10 * 14 + 10 + 4)): 2,
                     KVNeed(kv_heads=6, head_dim=12, value_heads=3, value_dim=20, chunk=21): 2,
                     KVNeed(kv_heads=1, head_dim=0, value_heads=1, value_dim=24): 1}
    att, rec, lat = model.blocks[1].mixer, model.blocks[0].mixer, model.blocks[2].mixer
    assert (att.KIND, att.chunk, att.window, att.head_gate, att.diff, att.scale) == ("differential_attention", 21, None, True, 0.25, 0.3)
    assert (rec.KIND, rec.cap, rec.eps, rec.heads, rec.dim, rec.vdim) == ("mlstm", 9.0, 1e-5, 3, 10, 14)
    assert (lat.KIND, lat.rot_dim, lat.rotary, lat.gate_width, lat.rank, lat.scale) == ("latent_attention", 0, None, 40, 24, 0.2)
    moe, dense = model.blocks[0].ffn, model.blocks[1].ffn
    assert (moe.router, moe.groups, moe.keep, moe.route_scale, moe.slope, moe.plus, moe.shared_gated, moe.limit) == \
        ("sigmoid_groups", 4, 2, 1.5, 1.0, 0.0, False, float("inf"))
    assert (dense.activation, dense.has_bias, dense.inner) == ("relu2", False, 56)
    assert model.embedding.scale == 3.0 and model.head.scale == 1.0 and model.final_norm.KIND == "layernorm"
    # no mask: every earlier key; no shared expert; no groups
    doc = copy.deepcopy(BASE)
    del doc["layers"][1]["mixer"]["mask"]
    doc["layers"][0]["mlp"]["shared"] = None
    del doc["layers"][0]["mlp"]["router"]["groups"]
    _, _, other = build(doc)
    assert other.blocks[1].mixer.chunk is None and other.blocks[0].ffn.shared_inner == 0 and other.blocks[0].ffn.groups == 1
    assert "l0.mlp.shared.up" not in {r.source.name for r in other.tensor_rows()}


@pytest.mark.parametrize("path,value", [(("layers", 1, "type"), "attention_2"), (("layers", 1, "mixer", "kv_heads"), 4),
                                        (("layers", 1, "mixer", "diff"), None), (("layers", 1, "mixer", "mask", "size"), 0),
                                        (("layers", 1, "mlp", "kind"), "gated"), (("layers", 0, "mixer", "gate_cap"), 0),
                                        (("layers", 0, "mlp", "router", "top"), 9), (("layers", 0, "mlp", "router", "groups", "count"), 3),
                                        (("layers", 0, "mlp", "router", "groups", "keep"), 5), (("layers", 2, "mixer", "kv_rank"), None),
                                        (("layers", 0, "mlp", "expert", "ff"), 0), (("embedding", "scale"), "big"), (("width",), 0)])
def test_bad_values_are_refused(path, value):
    from ayaka_py_b200.config.model import ConfigError, TesozenConfig
    doc = copy.deepcopy(BASE)
    at = doc
    for key in path[:-1]:
        at = at[key]
    at[path[-1]] = value
    with pytest.raises(ConfigError):
        TesozenConfig.from_dict(doc)


def test_pages_before_the_chunk_of_the_next_position_come_back():
    """Page size 4, chunks of 10: after every step the request holds exactly the pages from the one with the
    first position of the next token's chunk on, and closing it returns every page once."""
    from ayaka_py_b200.cache import CacheGroupSpec, CacheManager
    from ayaka_py_b200.parts.base import KVNeed
    m = CacheManager([CacheGroupSpec("c", KVNeed(2, 8, chunk=10), 1)], kv_pages=9, page_size=4, max_requests=2,
                     max_len=64, device=None)
    a = m.open("a")
    n = 0
    for step in (3, 2, 7, 1, 1, 9, 1, 6, 1, 5, 1, 3):
        m.commit(m.reserve([(a, n, step)]))
        n += step
        m.check_invariants()
        held = [p for p in range(-(-n // 4)) if m.tables[0][a, p] > 0]
        assert held == list(range((n // 10 * 10) // 4, -(-n // 4))), (n, held)
    b = m.open("b")
    m.commit(m.reserve([(b, 0, 13)]))
    m.check_invariants()
    m.close(a)
    m.close(b)
    m.assert_clean()


def test_routing_of_the_plain_model():
    """Groups shut experts out altogether (a negative ranking score still beats an expert of a dropped group),
    the mixing weights come from the uncorrected scores and add up to the factor."""
    z = np.array([3.0, 2.5, -4.0, -4.0, 2.9, -9.0, -9.0, -9.0])
    corr = np.array([0.0, 0.0, -2.0, -2.0, 0.0, 0.0, 0.0, 0.0])
    # groups of two: scores ~ (1.87, -3.96, 0.95, 0.0002); keep 2 -> groups 0 and 2; top 3 -> experts 0, 4, 1
    chosen, w = plain.route(z, corr, 3, 4, 2, 2.0)
    assert chosen == [0, 4, 1] and abs(w.sum() - 2.0) < 1e-12
    s = plain.sigmoid(z)
    assert np.allclose(w, s[[0, 4, 1]] / s[[0, 4, 1]].sum() * 2.0)
    # with a group kept whose scores are negative, its expert is chosen before any expert of a dropped group
    chosen, _ = plain.route(np.array([0.0, 0.0, 5.0, -9.0, 1.0, 1.0]), np.array([-3.0, -3.0, 0.0, 0.0, -3.0, -3.0]), 2, 3, 1, 1.0)
    assert chosen == [2, 3]
    # one group: the plain top-k of the corrected scores
    chosen, _ = plain.route(np.array([0.1, 0.2, 0.3, 0.4]), np.array([1.0, 0.0, 0.0, 0.0]), 2, 1, 1, 1.0)
    assert chosen == [0, 3]


def test_the_recurrence_of_the_plain_model_against_its_unstabilized_form():
    """With small gates nothing overflows, and the running maximum cancels but for the floor of the denominator:
    m starts at 0, so the first tokens divide by exp(-m) while |n . q| is small."""
    rs = np.random.RandomState(5)
    T, H, D, Dv = 12, 2, 6, 5
    q, k, v = rs.randn(T, H, D), rs.randn(T, H, D), rs.randn(T, H, Dv)
    i, f = 0.5 * rs.randn(T, H), plain.log_sigmoid(2.0 + rs.randn(T, H))
    got = plain.mlstm_recurrence(q, k, v, i, f)
    S, n, m = np.zeros((H, D, Dv)), np.zeros((H, D)), np.zeros(H)
    for t in range(T):
        S = np.exp(f[t])[:, None, None] * S + np.exp(i[t])[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        n = np.exp(f[t])[:, None] * n + np.exp(i[t])[:, None] * k[t]
        m = np.maximum(f[t] + m, i[t])
        num = np.einsum("hdv,hd->hv", S, q[t]) * np.exp(-m)[:, None]
        den = np.maximum(np.abs(np.einsum("hd,hd->h", n, q[t])) * np.exp(-m), np.exp(-m)) + 1e-6
        assert np.allclose(got[t], num / den[:, None], rtol=1e-9, atol=1e-12)


def test_plain_model_is_causal_and_respects_its_chunks():
    """Changing a token moves the logits of later positions only, and with nothing but chunked attention only
    those of its own chunk."""
    att = {"type": "attention", "mlp": {"kind": "dense", "ff": 16},
           "mixer": {"heads": 2, "kv_heads": 1, "dim": 6, "vdim": 8, "scale": 0.4, "diff": 0.3, "mask": {"size": 7}}}
    cfg = {"architecture": "Tesozen", "vocab": 50, "width": 24, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.0}, "layers": [att, att]}
    t = {k: v.astype(np.float64) for k, v in plain.random_tensors(cfg, 3).items()}
    toks = np.random.RandomState(0).randint(0, 50, 30).tolist()
    base = plain.forward(cfg, t, toks)
    other = list(toks)
    other[9] = (other[9] + 1) % 50
    moved = np.abs(plain.forward(cfg, t, other) - base).max(axis=1)
    assert (moved[:9] == 0).all() and (moved[9:14] > 0).all() and (moved[14:] == 0).all()
    cfg2 = dict(cfg, layers=[att, {"type": "mlstm", "mlp": None, "mixer": {"heads": 2, "dim": 4, "vdim": 6, "gate_cap": 8.0}}])
    t2 = {k: v.astype(np.float64) for k, v in plain.random_tensors(cfg2, 4).items()}
    moved = np.abs(plain.forward(cfg2, t2, other) - plain.forward(cfg2, t2, toks)).max(axis=1)
    assert (moved[:9] == 0).all() and (moved[9:] > 0).all()          # the recurrence carries it on
