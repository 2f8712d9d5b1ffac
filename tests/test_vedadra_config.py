"""Vedadra on the host: configuration, registry, the model as data, run order, cache groups, tensor names,
and the pages that a window with kept first tokens holds."""

import copy

import numpy as np
import pytest
import torch

import plain_vedadra as plain

_FF = {"kind": "dense", "ff": 40}
_TALK = {"type": "attention", "mlp": _FF,
         "mixer": {"heads": 6, "kv_heads": 3, "dim": 12, "vdim": 12, "scale": 0.3, "mask": {"size": 21}}}
_DIFF = {"type": "attention_2", "mlp": None,
         "mixer": {"heads": 4, "kv_heads": 2, "dim": 10, "vdim": 14, "scale": 0.25, "diff": 0.2, "mask": {"size": 9, "keep_first": 3}}}
BASE = {"architecture": "Vedadra", "vocab": 97, "width": 48, "norm": {"eps": 1e-5, "groups": 3},
        "loop": {"start": 1, "stop": 3, "times": 3}, "layers": [_DIFF, _TALK, _DIFF, _TALK]}


def build(document, dtype=torch.bfloat16):
    from ayaka_py_b200 import models, parts  # noqa: F401
    from ayaka_py_b200.models.model import Model
    from ayaka_py_b200.registry import architecture_for
    arch = architecture_for(document)
    config = arch.config_class.from_dict(document)
    return arch, config, Model(arch.build_spec(config), dtype, "meta")


def test_registry_and_round_trip():
    arch, config, _ = build(BASE)
    assert arch.name == "Vedadra"
    again = arch.config_class.from_dict(config.to_dict())
    assert again.to_dict() == config.to_dict() and again.to_dict()["architecture"] == "Vedadra"


def test_tensor_names_and_shapes():
    arch, config, model = build(BASE)
    rows = {r.source.name: tuple(r.decl.shape) for r in model.tensor_rows()}
    assert rows == plain.tensor_shapes(BASE)
    # a layer without feed-forward has neither its tensors nor its two norms, and passes them over in a checkpoint
    assert "l0.norm2" not in rows and "l0.mlp.up" not in rows and "l1.norm2b" in rows
    assert arch.normalize_name("l0.norm2b", config) is None and arch.normalize_name("l1.norm2b", config) == "l1.norm2b"
    assert arch.normalize_name("l2.mlp.gate", config) is None and arch.normalize_name("head", config) == "head"


def test_the_loop_names_layers_once_per_pass_with_caches_of_their_own():
    from ayaka_py_b200.parts import KVNeed
    _, config, model = build(BASE)
    assert config.run_order() == plain.run_order(BASE)
    order = model.spec.order
    assert [s.layer for s in order] == [0, 1, 2, 1, 2, 1, 2, 3] and len(model.blocks) == 4
    assert [s.add_input for s in order] == [False, False, False, True, False, True, False, False]
    assert [b.KIND for b in model.blocks] == ["double_norm_mixer_only", "double_norm", "double_norm_mixer_only", "double_norm"]
    needs = {g.need: g.layers for g in model.groups}
    assert needs == {KVNeed(kv_heads=4, head_dim=10, window=9, value_heads=2, value_dim=14, keep_first=3): 4,
                     KVNeed(kv_heads=3, head_dim=12, window=21, value_heads=3, value_dim=12): 4}
    seen = set()
    for binding in model.bindings:
        key = (binding["mixer"].group, binding["mixer"].layer)
        assert binding["mixer"].writes and key not in seen
        seen.add(key)
    for doc, want in (({**BASE, "loop": None}, [0, 1, 2, 3]), ({**BASE, "loop": {"start": 0, "stop": 4, "times": 2}}, [0, 1, 2, 3] * 2),
                      ({**BASE, "loop": {"start": 2, "stop": 2, "times": 5}}, [0, 1, 2, 3]),
                      ({**BASE, "loop": {"start": 3, "stop": 4, "times": 1}}, [0, 1, 2, 3])):
        _, _, m = build(doc)
        assert [s.layer for s in m.spec.order] == want
        assert [s.add_input for s in m.spec.order] == [k >= 4 and k % 4 == 0 for k in range(len(want))]


def test_constants_reach_the_parts():
    _, _, model = build(BASE)
    diff, talk = model.blocks[0].mixer, model.blocks[1].mixer
    assert (diff.KIND, diff.window, diff.keep_first, diff.diff, diff.scale, diff.vdim) == ("differential_attention", 9, 3, 0.2, 0.25, 14)
    assert (talk.KIND, talk.window, talk.scale, talk.slope_exponent, talk.heads, talk.kv_heads) == ("talking_attention", 21, 0.3, 8.0, 6, 3)
    assert model.blocks[1].norm1b.groups == 3 and model.final_norm.groups == 3 and model.final_norm.eps == 1e-5
    assert model.blocks[1].ffn.activation == "gelu_tanh" and model.blocks[1].ffn.inner == 40


@pytest.mark.parametrize("path,value", [(("layers", 1, "type"), "attention_3"), (("layers", 1, "mixer", "kv_heads"), 4),
                                        (("layers", 1, "mixer", "vdim"), 16), (("layers", 0, "mixer", "diff"), None),
                                        (("layers", 0, "mixer", "mask", "size"), 0), (("layers", 1, "mlp", "kind"), "moe"),
                                        (("norm", "groups"), 5), (("loop", "stop"), 5), (("loop", "times"), 0),
                                        (("layers", 1, "mixer", "scale"), "big"), (("width",), 0)])
def test_bad_values_are_refused(path, value):
    from ayaka_py_b200.config.model import ConfigError, VedadraConfig
    doc = copy.deepcopy(BASE)
    at = doc
    for key in path[:-1]:
        at = at[key]
    at[path[-1]] = value
    with pytest.raises(ConfigError):
        VedadraConfig.from_dict(doc)


def test_kept_first_pages_stay_while_the_window_moves_on():
    """Page size 4, window 6, the first 5 tokens kept: pages 0 and 1 stay for good, the pages between them and
    the window's first page go back to the pool, and closing the request returns every page once."""
    from ayaka_py_b200.cache import CacheGroupSpec, CacheManager
    from ayaka_py_b200.parts.base import KVNeed
    m = CacheManager([CacheGroupSpec("w", KVNeed(2, 8, 6, keep_first=5), 1)], kv_pages=12, page_size=4, max_requests=2,
                     max_len=64, device=None)
    a = m.open("a")
    m.commit(m.reserve([(a, 0, 3)]))
    m.check_invariants()
    n = 3
    for step in (2, 7, 1, 1, 9, 1, 1, 1, 5, 1):
        m.commit(m.reserve([(a, n, step)]))
        n += step
        m.check_invariants()
        held = [p for p in range(-(-n // 4)) if m.tables[0][a, p] > 0]
        first_needed = max(0, n - 6 + 1) // 4
        assert held == sorted(set([p for p in (0, 1) if p < -(-n // 4)]) | set(range(first_needed, -(-n // 4))))
    b = m.open("b")
    m.commit(m.reserve([(b, 0, 13)]))
    m.check_invariants()
    m.close(a)
    m.check_invariants()
    m.close(b)
    m.assert_clean()


def test_plain_model_is_causal_and_respects_its_windows():
    """The oracle itself: changing a token that no later position can reach through any layer's mask leaves
    those positions' logits alone, and changing a reachable one does not."""
    cfg = {"architecture": "Vedadra", "vocab": 50, "width": 24, "norm": {"eps": 1e-5, "groups": 2}, "loop": None,
           "layers": [{"type": "attention_2", "mlp": None,
                       "mixer": {"heads": 2, "kv_heads": 1, "dim": 6, "vdim": 8, "scale": 0.4, "diff": 0.3, "mask": {"size": 3, "keep_first": 2}}},
                      {"type": "attention", "mlp": {"kind": "dense", "ff": 16},
                       "mixer": {"heads": 2, "kv_heads": 2, "dim": 6, "vdim": 6, "scale": 0.4, "mask": {"size": 4}}}]}
    t = {k: v.astype(np.float64) for k, v in plain.random_tensors(cfg, 3).items()}
    toks = np.random.RandomState(0).randint(0, 50, 30).tolist()
    base = plain.forward(cfg, t, toks)
    other = list(toks)
    other[10] = (other[10] + 1) % 50
    moved = np.abs(plain.forward(cfg, t, other) - base).max(axis=1)
    # token 10 is not kept (keep_first 2); it reaches i <= 12 in the first layer and i <= 15 through the second
    assert (moved[:10] == 0).all() and moved[10] > 0 and moved[15] > 0 and (moved[16:] == 0).all()
    other = list(toks)
    other[1] = (other[1] + 1) % 50
    assert np.abs(plain.forward(cfg, t, other) - base).max(axis=1)[29] > 0          # a kept token reaches everything
