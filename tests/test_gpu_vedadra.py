"""Vedadra: every mechanism alone against the plain functions of ``plain_vedadra``, then whole
models of several shapes replayed whole, decoded, in portions and mixed, and greedy generation
through the engine's own entry point."""

import copy
import json
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import plain_vedadra as plain
import trace_tools

pytestmark = pytest.mark.gpu

DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def dev(a, dtype=torch.float32):
    return torch.as_tensor(np.ascontiguousarray(a)).to(dtype).cuda()


def host(t):
    return t.double().cpu().numpy()


def tol(dtype, scale=1.0):
    return (2e-5 if dtype == "float32" else 2e-2) * scale


# ------------------------------------------------------------------ configs --

def ff(n):
    return {"kind": "dense", "ff": n}


def talking(heads, kv, dim, size, scale, mlp):
    return {"type": "attention", "mlp": mlp,
            "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": dim, "scale": scale, "mask": {"size": size}}}


def differential(heads, kv, dim, vdim, size, keep, scale, diff, mlp):
    return {"type": "attention_2", "mlp": mlp,
            "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "diff": diff,
                      "mask": {"size": size, "keep_first": keep}}}


# A: odd sizes, three norm groups, a loop that starts after the first layer and runs three times, a layer
# without feed-forward, values narrower than keys, two key/value heads under the differential maps,
# windows shorter than two pages, kept tokens within the first page.
CONFIG_A = {"architecture": "Vedadra", "vocab": 211, "width": 72, "norm": {"eps": 1e-5, "groups": 3},
            "loop": {"start": 1, "stop": 3, "times": 3},
            "layers": [differential(4, 2, 20, 12, 11, 3, 0.22, 0.25, ff(40)), talking(6, 3, 10, 23, 0.3, ff(52)),
                       differential(2, 2, 12, 28, 30, 0, 0.3, 0.1, None), talking(3, 1, 24, 9, 0.2, ff(36))]}
# B: one norm group, no loop, every head with keys of its own, a window of one token (a query sees itself
# and the kept tokens), kept tokens over several pages, a window longer than any request, values wider than keys.
CONFIG_B = {"architecture": "Vedadra", "vocab": 130, "width": 64, "norm": {"eps": 1e-6, "groups": 1}, "loop": None,
            "layers": [talking(4, 4, 16, 1000, 0.25, ff(48)), differential(3, 3, 16, 40, 1, 20, 0.25, 0.4, ff(30)),
                       talking(2, 1, 32, 1, 0.2, None), differential(4, 1, 8, 16, 13, 13, 0.35, 0.05, ff(64))]}
# C: sizes of the tensor-core kernels (heads of 64, eight query heads on two key/value heads), the whole
# model looped three times, windows of a few pages.
CONFIG_C = {"architecture": "Vedadra", "vocab": 300, "width": 128, "norm": {"eps": 1e-6, "groups": 4},
            "loop": {"start": 0, "stop": 3, "times": 3},
            "layers": [talking(8, 2, 64, 100, 0.125, ff(192)), differential(8, 2, 64, 128, 70, 5, 0.125, 0.35, ff(160)),
                       differential(4, 4, 32, 32, 40, 17, 0.18, 0.2, None)]}
CONFIGS = {"A": CONFIG_A, "B": CONFIG_B, "C": CONFIG_C}
LENGTHS = {"A": [1, 2, 19, 77, 150], "B": [3, 33, 64, 129], "C": [5, 48, 100, 300]}
PAGE = {"A": 16, "B": 8, "C": 16}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    base = tmp_path_factory.mktemp("vedadra")
    out = {}
    for tag, cfg in CONFIGS.items():
        tensors = plain.random_tensors(cfg, seed=60 + ord(tag))
        folder = plain.write_folder(base / tag, cfg, tensors)
        rs = np.random.RandomState(ord(tag))
        reqs = {f"{tag.lower()}{i}": rs.randint(0, cfg["vocab"], n).tolist() for i, n in enumerate(LENGTHS[tag])}
        t64 = {k: v.astype(np.float64) for k, v in tensors.items()}
        want = {rid: plain.forward(cfg, t64, toks) for rid, toks in reqs.items()}
        out[tag] = (folder, cfg, t64, reqs, want)
    return out


def limit(dtype, want):
    """The 16-bit limit leaves room for the difference of two maps that nearly cancel before it is divided by
    its root mean square; such a position's error is the same however the request is cut."""
    big = max(float(np.abs(w).max()) for w in want.values())
    return (2e-5 if dtype == "float32" else 0.05) * big


def replay(folder, dtype, trace, page_size, max_tokens=None):
    from ayaka_py_b200.replay import ReplaySession
    session = ReplaySession(folder, dtype, max_tokens or trace_tools.tokens_needed(trace), page_size)
    outputs = []
    for record in trace:
        logits = session.step(record)
        outputs.append(None if logits is None or logits.shape[0] == 0 else logits.cpu().numpy())
    session.cache.assert_clean()
    return outputs, session


def check(models, tag, dtype, trace, want=None, **kw):
    """Every position of every request agrees with the plain model's whole-sequence logits."""
    folder = models[tag][0]
    want = want or models[tag][4]
    outputs, session = replay(folder, dtype, trace, PAGE[tag], **kw)
    got = trace_tools.collect(trace, outputs)
    bad = trace_tools.first_difference(got, want, limit(dtype, want))
    assert bad is None, f"first wrong place: request {bad[0]} position {bad[1]} |diff| {bad[2]:.3e} (limit {limit(dtype, want):.3e})"
    return session


# ---------------------------------------------------------- a step context --

def context_for(groups, dtype, max_requests=4, page_size=8, pages=64, positions=1024):
    from ayaka_py_b200.cache import CacheManager
    from ayaka_py_b200.engine.step import StepRunner
    cache = CacheManager(groups, kv_pages=pages, page_size=page_size, max_requests=max_requests, max_len=positions,
                         dtype=DT[dtype], device="cuda")
    model = SimpleNamespace(device="cuda", dtype=DT[dtype], max_positions=positions, vocab_size=10)
    return cache, StepRunner(model, cache, max_tokens=positions)


def step_of(cache, runner, counts):
    """A reserved step in which request i brings counts[i] tokens."""
    from ayaka_py_b200.engine.step import StepEntry
    entries = []
    for i, n in counts.items():
        slot = cache.slot_of.get(i)
        if slot is None:
            slot = cache.open(i)
        entries.append(StepEntry(slot, int(cache.length[slot]), [0] * n, []))
    res = cache.reserve([(e.slot, e.start, len(e.tokens)) for e in entries])
    return runner.prepare(entries), res


def run_cut(cache, runner, rows, cuts, fn):
    """Feeds rows[i] (one array per request) in portions: cuts is a list of {request: count} steps;
    fn(ctx, packed rows of the step) returns the step's output rows.  Gives back per-request outputs."""
    at = {i: 0 for i in rows}
    got = {i: [] for i in rows}
    for counts in cuts:
        ctx, res = step_of(cache, runner, counts)
        order = [int(i) for i in ctx.host["order"]]
        ids = list(counts)
        packed = [ids[k] for k in order]
        x = torch.cat([rows[i][at[i]:at[i] + counts[i]] for i in packed])
        y = fn(ctx, x)
        a = 0
        for i in packed:
            got[i].append(y[a:a + counts[i]].float().cpu().numpy())
            a += counts[i]
            at[i] += counts[i]
        cache.commit(res)
    return {i: np.concatenate(v) for i, v in got.items()}


def cuts_for(lengths, sizes):
    out, k = [], 0
    for i, n in lengths.items():
        p = 0
        while p < n:
            c = min(sizes[k % len(sizes)], n - p)
            out.append({i: c})
            p += c
            k += 1
    return out


PLANS = [lambda L: cuts_for(L, [1000]), lambda L: cuts_for(L, [1]), lambda L: cuts_for(L, [2, 1, 3, 5, 2, 2, 1, 8, 70]),
         lambda L: [{0: 5, 1: 1}, {0: 1, 1: 2, 2: L[2]}, {0: 2, 1: 1}, {0: L[0] - 8, 1: L[1] - 4}]]


def layer_tensors(layer, d, seed, prefix="l0.mix."):
    cfg = {"vocab": 4, "width": d, "layers": [layer]}
    t = plain.random_tensors(cfg, seed)
    return {k: v.astype(np.float64) for k, v in t.items()}, {k[len(prefix):]: v for k, v in t.items() if k.startswith(prefix)}


def bind(part, tensors, names, dtype):
    decl = part.tensors()
    part.bind({names[k]: dev(v, DT[dtype] if decl[names[k]].kind == "matrix" else torch.float32) for k, v in tensors.items()})


def mixer_alone(part, dtype, d, want_fn, lengths, seed=5, rows=None, page_size=8):
    """A mixer part over several requests, cut four ways (whole, token by token, ragged, batched with
    unequal requests), and once more in slots and pages that were used before."""
    from ayaka_py_b200.cache import CacheBinding, CacheGroupSpec
    rs = np.random.RandomState(seed)
    xs = rows or {i: plain.round_bf16(rs.randn(n, d).astype(np.float32)) for i, n in lengths.items()}
    want = {i: want_fn(x.astype(np.float64)) for i, x in xs.items()}
    big = max(float(np.abs(w).max()) for w in want.values())
    rows_d = {i: dev(x, DT[dtype]) for i, x in xs.items()}
    binding = CacheBinding(0, "g", 0, True)
    fn = lambda ctx, x: part.forward(x.contiguous(), None, ctx, binding)
    for n, plan in enumerate(PLANS):
        cache, runner = context_for([CacheGroupSpec("g", part.cache_need(), 1)], dtype, max_requests=3, page_size=page_size,
                                    pages=768 // page_size)
        got = run_cut(cache, runner, rows_d, plan(lengths), fn)
        for i in lengths:
            worst = float(np.abs(got[i] - want[i]).max())
            assert worst < tol(dtype, 3 * big), (n, i, int(np.abs(got[i] - want[i]).max(axis=1).argmax()), worst)
        for i in list(cache.slot_of):
            cache.close(cache.slot_of[i])
        got = run_cut(cache, runner, rows_d, cuts_for(lengths, [4, 1, 33]), fn)      # slots and pages used again
        for i in lengths:
            assert np.abs(got[i] - want[i]).max() < tol(dtype, 3 * big)
        cache.check_invariants() if hasattr(cache, "check_invariants") else None
    return want


# ------------------------------------------------------- mechanisms alone --

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("d,groups", [(72, 3), (64, 1), (128, 4), (40, 40), (1536, 2), (6, 2)])
def test_norm_in_groups_alone_and_added_to_the_stream(dtype, d, groups):
    from ayaka_py_b200.parts import PartSpec, make_part
    for n_rows in (9, 2048 // groups + 8):          # few rows: a block per group; many: a warp per group
        norm_cases(dtype, d, groups, n_rows)


def norm_cases(dtype, d, groups, n_rows):
    from ayaka_py_b200.parts import PartSpec, make_part
    rs = np.random.RandomState(d + groups)
    x = rs.randn(n_rows, d).astype(np.float32) * 3
    x[:, :d // groups] *= 20                                            # a group's size must not leak into the next
    w = (1.0 + 0.2 * rs.randn(d)).astype(np.float32)
    norm = make_part(PartSpec("rmsnorm", {"width": d, "eps": 1e-5, "groups": groups}), DT[dtype], "cuda")
    norm.bind({"weight": dev(w)})
    want = plain.grouped_norm(x.astype(np.float64), w.astype(np.float64), groups, 1e-5)
    got = norm.forward(dev(x), None)
    assert got.dtype == DT[dtype]
    assert np.abs(host(got) - want).max() < (1e-5 if dtype == "float32" else 1e-2) * np.abs(want).max()
    base = rs.randn(n_rows, d).astype(np.float32)
    assert np.abs(host(norm.add_normed(dev(base), dev(x))) - (base + want)).max() < 2e-5 * np.abs(want).max()
    # added to the stream and the next norm of the sum, one kernel
    w2 = (1.0 + 0.2 * rs.randn(d)).astype(np.float32)
    after = make_part(PartSpec("rmsnorm", {"width": d, "eps": 3e-5, "groups": groups}), DT[dtype], "cuda")
    after.bind({"weight": dev(w2)})
    stream = dev(base)
    got = norm.add_normed_then(stream, dev(x), after)
    assert got.dtype == DT[dtype]
    assert np.abs(host(stream) - (base + want)).max() < 2e-5 * np.abs(want).max()
    want2 = plain.grouped_norm(base + want, w2.astype(np.float64), groups, 3e-5)
    assert np.abs(host(got) - want2).max() < (1e-5 if dtype == "float32" else 1e-2) * np.abs(want2).max()
    if groups > 1:                                                      # one group would be another function
        other = plain.grouped_norm(x.astype(np.float64), w.astype(np.float64), 1, 1e-5)
        assert np.abs(other - want).max() > 0.1


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("d,inner", [(72, 40), (64, 30), (128, 192), (48, 7)])
def test_gated_feed_forward_alone(dtype, d, inner):
    from ayaka_py_b200.parts import PartSpec, make_part
    rs = np.random.RandomState(3)
    layer = talking(2, 1, 8, 4, 0.1, ff(inner))
    t64, w = layer_tensors(layer, d, 19, prefix="l0.mlp.")
    part = make_part(PartSpec("gated_mlp", {"width": d, "inner": inner, "activation": "gelu_tanh"}), DT[dtype], "cuda")
    bind(part, w, {"gate": "gate_weight", "up": "up_weight", "down": "down_weight"}, dtype)
    for n in (1, 5, 150):
        h = plain.round_bf16(rs.randn(n, d).astype(np.float32) * 2)
        want = plain.gated_ff(h.astype(np.float64), t64, "l0.mlp.")
        got = part.forward(dev(h, DT[dtype]), None, None)
        assert got.dtype == torch.float32
        assert np.abs(host(got) - want).max() < tol(dtype, 3 * float(np.abs(want).max()))
    base = rs.randn(n, d).astype(np.float32)
    got = part.forward(dev(h, DT[dtype]), dev(base), None)
    assert np.abs(host(got) - (base + want)).max() < tol(dtype, 3 * float(np.abs(want).max()))


TALK_NAMES = {"q": "q_weight", "q.b": "q_bias", "k": "k_weight", "k.b": "k_bias", "q.norm": "q_norm", "k.norm": "k_norm",
              "talk": "talk", "temp": "temp", "g": "gate_weight", "o": "out_weight", "o.b": "out_bias"}
DIFF_NAMES = {"q": "q_weight", "k": "k_weight", "v": "v_weight", "q.norm": "q_norm", "k.norm": "k_norm", "lq1": "lq1",
              "lk1": "lk1", "lq2": "lq2", "lk2": "lk2", "o": "out_weight"}


def talking_part(layer, d, dtype, eps=1e-5):
    from ayaka_py_b200.parts import PartSpec, make_part
    mx = layer["mixer"]
    return make_part(PartSpec("talking_attention", {"width": d, "heads": mx["heads"], "kv_heads": mx["kv_heads"], "dim": mx["dim"],
                                                    "scale": mx["scale"], "eps": eps, "window": mx["mask"]["size"]}), DT[dtype], "cuda")


def differential_part(layer, d, dtype, eps=1e-5):
    from ayaka_py_b200.parts import PartSpec, make_part
    mx = layer["mixer"]
    return make_part(PartSpec("differential_attention",
                              {"width": d, "heads": mx["heads"], "kv_heads": mx["kv_heads"], "dim": mx["dim"], "vdim": mx["vdim"],
                               "scale": mx["scale"], "diff": mx["diff"], "eps": eps, "window": mx["mask"]["size"],
                               "keep_first": mx["mask"]["keep_first"]}), DT[dtype], "cuda")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,D,size", [(6, 3, 10, 23), (4, 4, 16, 1000), (2, 1, 32, 1), (8, 2, 64, 100), (3, 1, 24, 9),
                                        (16, 4, 32, 64), (1, 1, 128, 40)])
def test_talking_attention_alone(dtype, H, G, D, size):
    d = 48
    layer = talking(H, G, D, size, 1.5 / np.sqrt(D), None)
    t64, w = layer_tensors(layer, d, 23)
    part = talking_part(layer, d, dtype)
    bind(part, w, TALK_NAMES, dtype)
    mixer_alone(part, dtype, d, lambda h: plain.biased_attention(h, t64, "l0.mix.", layer["mixer"], 1e-5), {0: 150, 1: 9, 2: 70})


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,D,Dv,size,keep", [(4, 2, 20, 12, 11, 3), (3, 3, 16, 40, 1, 20), (4, 1, 8, 16, 13, 13),
                                                (8, 2, 64, 128, 70, 5), (2, 2, 12, 28, 30, 0), (4, 4, 32, 32, 40, 17),
                                                (2, 1, 128, 64, 1000, 2), (5, 1, 16, 256, 24, 1)])
def test_differential_attention_alone(dtype, H, G, D, Dv, size, keep):
    d = 48
    layer = differential(H, G, D, Dv, size, keep, 1.5 / np.sqrt(D), 0.45, None)
    t64, w = layer_tensors(layer, d, 29)
    part = differential_part(layer, d, dtype)
    bind(part, w, DIFF_NAMES, dtype)
    mixer_alone(part, dtype, d, lambda h: plain.differential_attention(h, t64, "l0.mix.", layer["mixer"], 1e-5),
                {0: 150, 1: 9, 2: 70})


# ------------------------------------------- keys that stand out from the rest --

def standing_out_rows(rs, n, d, places):
    """Random rows; at ``places`` a strong common part plus a part of the row's own.  With keys made from the
    queries' matrix those places score high against one another, everything else around zero, and their
    values still differ, so that one key too many or too few moves the output."""
    x = rs.randn(n, d).astype(np.float32)
    common = rs.randn(d).astype(np.float32)
    for p in places:
        x[p] = 2.0 * common + x[p]
    return plain.round_bf16(x)


def edge_places(P, size, keep, n):
    """The first tokens, page borders, a pair just inside and just outside the window, the border of the
    kept tokens, and the end."""
    far = n - 30
    out = {0, 2, P - 1, P, P + 1, 5 * P - 1, 5 * P, far, n - 1}
    if size < n:
        out |= {far - size, far - size + 1}                     # the query at ``far`` sees the second only
        out |= {n - 1 - size, n - size}
    if keep:
        out |= {keep - 1, keep}
    return sorted(p for p in out if 0 <= p < n)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,D,size", [(4, 2, 20, 19), (3, 3, 16, 1000), (8, 2, 64, 100), (2, 1, 48, 8)])
def test_talking_attention_with_keys_that_stand_out(dtype, H, G, D, size):
    rs = np.random.RandomState(13)
    d, P = 48, 8
    layer = talking(H, G, D, size, 8.0 / D, None)
    t64, w = layer_tensors(layer, d, 31)
    per = H // G
    w["k"] = np.concatenate([w["q"][g * per * D:(g * per + 1) * D] for g in range(G)])
    w["q.b"][:], w["k.b"][:] = 0, 0
    w["q.norm"][:], w["k.norm"][:] = 1, 1
    for k, v in w.items():
        t64["l0.mix." + k] = v.astype(np.float64)
    part = talking_part(layer, d, dtype)
    bind(part, w, TALK_NAMES, dtype)
    lengths = {0: 330, 1: 9, 2: 70}
    places = {0: edge_places(P, size, 0, 330), 1: [0, 8], 2: [3, 2 * P, 69]}
    rows = {i: standing_out_rows(rs, n, d, places[i]) for i, n in lengths.items()}
    want = mixer_alone(part, dtype, d, lambda h: plain.biased_attention(h, t64, "l0.mix.", layer["mixer"], 1e-5),
                       lengths, rows=rows, page_size=P)
    if size < 330:                                                   # one key more in the window is another output
        wider = copy.deepcopy(layer["mixer"])
        wider["mask"]["size"] = size + 1
        other = plain.biased_attention(rows[0].astype(np.float64), t64, "l0.mix.", wider, 1e-5)
        assert np.abs(other[300] - want[0][300]).max() > 0.004 * np.abs(want[0]).max()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,D,Dv,size,keep", [(4, 2, 20, 12, 37, 3), (3, 3, 16, 40, 1, 20), (8, 2, 64, 128, 70, 9),
                                                (2, 1, 32, 64, 1000, 0), (4, 1, 8, 16, 24, 1)])
def test_differential_attention_with_keys_that_stand_out(dtype, H, G, D, Dv, size, keep):
    rs = np.random.RandomState(17)
    d, P = 48, 8
    layer = differential(H, G, D, Dv, size, keep, 8.0 / D, 0.35, None)
    t64, w = layer_tensors(layer, d, 37)
    per = H // G
    # the first map's keys are the first map's queries of the group's first head; the second map stays random
    k = w["k"].reshape(G, 2, D, d).copy()
    q = w["q"].reshape(H, 2, D, d)
    for g in range(G):
        k[g, 0] = q[g * per, 0]
    w["k"] = k.reshape(G * 2 * D, d)
    w["q.norm"][:], w["k.norm"][:] = 1, 1
    for name, v in w.items():
        t64["l0.mix." + name] = v.astype(np.float64)
    part = differential_part(layer, d, dtype)
    bind(part, w, DIFF_NAMES, dtype)
    lengths = {0: 330, 1: 9, 2: 70}
    places = {0: edge_places(P, size, keep, 330), 1: [0, 8], 2: [3, 2 * P, 69]}
    rows = {i: standing_out_rows(rs, n, d, places[i]) for i, n in lengths.items()}
    want = mixer_alone(part, dtype, d, lambda h: plain.differential_attention(h, t64, "l0.mix.", layer["mixer"], 1e-5),
                       lengths, rows=rows, page_size=P)
    for change in ([("size", size + 1)] if size < 300 else []) + ([("keep_first", keep + 1)] if keep else []):
        other_mx = copy.deepcopy(layer["mixer"])
        other_mx["mask"][change[0]] = change[1]
        other = plain.differential_attention(rows[0].astype(np.float64), t64, "l0.mix.", other_mx, 1e-5)
        assert np.abs(other[300] - want[0][300]).max() > 0.015 * np.abs(want[0]).max(), change


@pytest.mark.parametrize("step", ["prompts", "single", "mixed"])
@pytest.mark.parametrize("QH,KH,VH,DK,DV,window,keep,maps", [
    (8, 1, 2, 256, 128, 100, 0, 1), (16, 1, 4, 512, 128, None, 0, 1), (8, 4, 2, 64, 64, 70, 9, 2), (4, 2, 1, 24, 40, 33, 3, 2),
    (6, 1, 3, 48, 16, 1, 0, 1), (12, 1, 1, 96, 96, 300, 0, 1), (2, 2, 1, 128, 128, 520, 40, 2)])
def test_attention_on_the_tensor_cores_against_the_fp32_pipes(step, QH, KH, VH, DK, DV, window, keep, maps):
    """The two kernels of the grouped softmax attention on the same bfloat16 queries and pages: wide keys
    (tiles of 32 keys), padded head sizes, long contexts cut into parts, windows and kept tokens."""
    from ayaka_py_b200 import ops
    from ayaka_py_b200.cache import CacheGroupSpec
    from ayaka_py_b200.parts.base import KVNeed
    torch.manual_seed(QH * 131 + DK)
    need = KVNeed(kv_heads=KH, head_dim=DK, window=window, value_heads=VH, value_dim=DV, keep_first=keep if window else 0)
    cache, runner = context_for([CacheGroupSpec("g", need, 1)], "bfloat16", max_requests=3, page_size=16, pages=160)
    kpages, vpages = cache.kv_layer(0, 0)
    kpages.copy_(torch.randn(kpages.shape, device="cuda") * 0.7)
    vpages.copy_(torch.randn(vpages.shape, device="cuda"))
    before = {"prompts": {0: 0, 1: 300, 2: 5}, "single": {0: 699, 1: 300, 2: 0}, "mixed": {0: 650, 1: 17, 2: 200}}[step]
    brings = {"prompts": {0: 700, 1: 37, 2: 2}, "single": {0: 1, 1: 1, 2: 1}, "mixed": {0: 1, 1: 130, 2: 1}}[step]
    for i, n in before.items():
        slot = cache.open(i)
        if n:
            cache.commit(cache.reserve([(slot, 0, n)]))
    ctx, res = step_of(cache, runner, brings)
    T = ctx.num_rows
    q = (torch.randn(T, QH * DK, device="cuda") * (2.0 / DK ** 0.5)).to(torch.bfloat16)
    slopes = torch.rand(QH, device="cuda") * 0.05 if maps == 1 else None
    gate = torch.randn(T, QH * DV + 8, device="cuda") if maps == 1 else None
    kw = dict(heads=QH, key_heads=KH, key_dim=DK, scale=0.8, slopes=slopes, window=window, keep_first=keep, gate=gate,
              maps=maps, lam=0.4 if maps == 2 else 0.0, post_scale=0.6 if maps == 2 else 1.0, eps=1e-5)
    table = ctx.tables[0]
    got = ops.grouped_attention(q, kpages, vpages, table, ctx, tensor_cores=True, **kw).float()
    want = ops.grouped_attention(q, kpages, vpages, table, ctx, tensor_cores=False, **kw).float()
    assert torch.isfinite(got).all()
    assert float((got - want).abs().max()) < 1.5e-2 * float(want.abs().max())
    cache.rollback(res)


def test_lambda_and_the_scaling_after_the_difference():
    """The layer's factor from its four vectors, and values the given sizes would hide: diff 0 and a
    second map that weighs more than the first."""
    from ayaka_py_b200.parts import PartSpec, make_part
    d = 40
    for diff, gain in ((0.0, 1.0), (0.6, 6.0)):
        layer = differential(2, 1, 16, 24, 12, 2, 0.3, diff, None)
        t64, w = layer_tensors(layer, d, 41)
        for name in ("lq2", "lk2"):
            w[name] = plain.round_bf16(np.abs(w[name]) * gain)
            t64["l0.mix." + name] = w[name].astype(np.float64)
        lam = plain.differential_lambda(t64, "l0.mix.", diff)
        part = differential_part(layer, d, "float32")
        bind(part, w, DIFF_NAMES, "float32")
        assert abs(part.lam - lam) < 1e-6 * max(1.0, abs(lam))
        if gain > 1:
            assert lam < 0
        mixer_alone(part, "float32", d, lambda h: plain.differential_attention(h, t64, "l0.mix.", layer["mixer"], 1e-5), {0: 40, 1: 6, 2: 17})


# --------------------------------------------------------------- whole models --

def test_layers_one_by_one_in_32_bit(models):
    """The residual stream after every layer run (a looped layer counts every time) against the plain model."""
    from ayaka_py_b200.engine.step import StepEntry
    from ayaka_py_b200.replay import ReplaySession
    for tag in CONFIGS:
        folder, cfg, t64, reqs, _ = models[tag]
        toks = list(reqs.values())[2]
        after = []
        plain.forward(cfg, t64, toks, after)
        s = ReplaySession(folder, "float32", 256, PAGE[tag])
        seen = []
        for block in s.model.blocks:
            inner = block.forward
            def outer(x, ctx, caches, inner=inner):
                y = inner(x, ctx, caches)
                seen.append(host(y))
                return y
            block.forward = outer
        s.step({"step": 0, "entries": [{"id": "x", "tokens": toks, "want": [0]}], "end": ["x"]})
        assert len(seen) == len(after) == len(plain.run_order(cfg))
        for i, (got, want) in enumerate(zip(seen, after)):
            assert np.abs(got - want).max() < 1e-4 * max(1.0, float(np.abs(want).max())), (tag, i)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tag", ["A", "B", "C"])
def test_each_request_alone_and_whole(models, tag, dtype):
    check(models, tag, dtype, trace_tools.whole(models[tag][3]))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tag", ["A", "B", "C"])
def test_prefill_against_token_by_token_decoding(models, tag, dtype):
    check(models, tag, dtype, trace_tools.tail_decoded(models[tag][3], 40))
    few = dict(list(models[tag][3].items())[:3])
    check(models, tag, dtype, trace_tools.tail_decoded(few, 10_000), want={k: models[tag][4][k] for k in few})


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tag", ["A", "B", "C"])
def test_portions_down_to_two_tokens(models, tag, dtype):
    check(models, tag, dtype, trace_tools.portions(models[tag][3]))
    check(models, tag, dtype, trace_tools.portions(models[tag][3], sizes=(2, 2, 1, 2, 3, 2)))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tag", ["A", "B", "C"])
def test_mixed_batches_with_pages_and_slots_used_again(models, tag, dtype):
    reqs = dict(models[tag][3])
    extra = {f"{rid}+": toks[::-1] for rid, toks in reqs.items()}      # more requests than slots
    _, cfg, t64, _, want = models[tag]
    want = dict(want)
    want.update({rid: plain.forward(cfg, t64, toks) for rid, toks in extra.items()})
    reqs.update(extra)
    for seed in (0, 1):
        trace = trace_tools.mixed(reqs, seed=seed)
        assert max(len(s["entries"]) for s in trace) >= 3
        session = check(models, tag, dtype, trace, want=want)
        assert any(g["reused"] > 0 for g in session.cache.stats()["groups"].values())
    longer = {rid: toks for rid, toks in reqs.items() if len(toks) >= 19}
    check(models, tag, dtype, trace_tools.reopened(longer, seed=3), want={rid: want[rid] for rid in longer})


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_past_every_window(models, dtype):
    folder, cfg, t64, _, _ = models["B"]
    toks = np.random.RandomState(11).randint(0, cfg["vocab"], 420).tolist()
    want = {"long": plain.forward(cfg, t64, toks)}
    check(models, "B", dtype, trace_tools.tail_decoded({"long": toks}, 400), want=want)


def test_the_batch_does_not_change_a_request(models):
    """A request alone, cut one way, and the same request beside others, cut another way (32-bit)."""
    folder, cfg, _, reqs, _ = models["A"]
    alone = trace_tools.portions({"a4": reqs["a4"]}, sizes=(16, 1, 5))
    out_alone, _ = replay(folder, "float32", alone, 16)
    got_alone = trace_tools.collect(alone, out_alone)["a4"]
    both = trace_tools.mixed(reqs, seed=4)
    out_both, _ = replay(folder, "float32", both, 16)
    got_both = trace_tools.collect(both, out_both)["a4"]
    worst = max(float(np.abs(got_alone[p] - got_both[p]).max()) for p in got_alone)
    assert worst < 2e-5


def test_pages_behind_the_window_come_back_and_kept_pages_stay(models):
    """A long request in a pool smaller than its length: pages that every window has passed are handed out
    again while the pages of the kept first tokens stay."""
    folder, cfg, t64, _, _ = models["B"]
    toks = np.random.RandomState(12).randint(0, cfg["vocab"], 300).tolist()
    want = {"long": plain.forward(cfg, t64, toks)}
    trace = trace_tools.portions({"long": toks}, sizes=(5, 2, 11, 1, 1, 7))
    outputs, session = replay(folder, "float32", trace, PAGE["B"], max_tokens=320)
    got = trace_tools.collect(trace, outputs)
    assert trace_tools.first_difference(got, want, limit("float32", want)) is None
    stats = session.cache.stats()["groups"]
    short = [stats[g.name] for g in session.cache.groups if g.need.window is not None and g.need.window < 100]
    assert short and all(g["high_water"] < 300 // PAGE["B"] // 2 and g["reused"] > 0 for g in short)


# --------------------------------------------- the engine's own entry point --

@pytest.mark.parametrize("graphs", [True, False])
def test_greedy_generation_through_the_scheduler(models, graphs):
    from ayaka_py_b200.engine.llm import LLM
    from ayaka_py_b200.engine.request import StopCriteria
    from ayaka_py_b200.sampling.params import SamplingParams
    folder, cfg, t64, reqs, _ = models["A"]
    prompts = [reqs["a2"], reqs["a3"][:40], reqs["a0"], reqs["a3"][5:30], reqs["a1"], reqs["a4"][:70]]
    llm = LLM(folder, dtype="float32", kv_pages=24, page_size=16, max_requests=3, batch_tokens=48, prefill_chunk=20,
              max_model_len=128, decode_graph=graphs)
    results = llm.generate(prompts, SamplingParams(temperature=0.0), StopCriteria(max_tokens=12, ignore_eos=True))
    for prompt, result in zip(prompts, results):
        want = plain.greedy_generate(cfg, t64, prompt, 12)
        k = next((i for i, (a, b) in enumerate(zip(result.token_ids, want)) if a != b), None)
        if k is not None:                     # a near tie may turn a token
            logits = plain.forward(cfg, t64, prompt + want[:k])[-1]
            assert abs(logits[result.token_ids[k]] - logits[want[k]]) < 1e-3
        else:
            assert result.token_ids == want
    llm.engine.cache.assert_clean()


def test_bfloat16_generation_with_decode_graphs_equals_eager(models):
    from ayaka_py_b200.engine.llm import LLM
    from ayaka_py_b200.engine.request import StopCriteria
    from ayaka_py_b200.sampling.params import SamplingParams
    folder, cfg, _, reqs, _ = models["C"]
    prompts = [reqs["c1"], reqs["c0"], reqs["c2"][:33]]
    out = []
    for graphs in (True, False):
        llm = LLM(folder, dtype="bfloat16", kv_pages=40, page_size=16, max_requests=4, max_model_len=160, decode_graph=graphs)
        out.append([r.token_ids for r in llm.generate(prompts, SamplingParams(temperature=0.0),
                                                      StopCriteria(max_tokens=16, ignore_eos=True))])
    assert out[0] == out[1]


def test_random_weights_mode_and_command_line(tmp_path):
    """A folder written by the engine's own random-weights mode loads and generates from the command line."""
    import subprocess
    import sys
    from pathlib import Path
    from ayaka_py_b200.config.model import VedadraConfig
    from ayaka_py_b200.weights import write_random_model
    folder = write_random_model(tmp_path / "m", VedadraConfig.from_dict(CONFIG_B), seed=3)
    assert json.loads((folder / "config.json").read_text())["architecture"] == "Vedadra"
    root = Path(__file__).resolve().parent.parent
    proc = subprocess.run([sys.executable, "-m", "ayaka_py_b200", "generate", str(folder), "--prompt-ids", "1,2,3,4,5",
                           "--max-tokens", "5", "--temperature", "0", "--ignore-eos", "--max-model-len", "64", "--kv-pages", "16"],
                          cwd=root, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    line = json.loads(proc.stdout.strip().splitlines()[-1])
    assert len(line["token_ids"]) == 5
