"""Tesozen: every mechanism alone against the plain functions of ``plain_tesozen``, then whole models of
several shapes replayed whole, decoded, in portions and mixed, and greedy generation through the engine's own
entry point."""

import copy
import json

import numpy as np
import pytest
import torch

import plain_tesozen as plain
import trace_tools
from test_gpu_vedadra import DT, bind, context_for, dev, host, mixer_alone, standing_out_rows, step_of, tol

pytestmark = pytest.mark.gpu


# ------------------------------------------------------------------ configs --

def dense(n):
    return {"kind": "dense", "ff": n}


def moe(experts, top, count, keep, ff, shared, scale=2.0):
    return {"kind": "moe", "router": {"experts": experts, "top": top, "scale": scale, "groups": {"count": count, "keep": keep}},
            "expert": {"ff": ff}, "shared": {"ff": shared} if shared else None}


def attention(heads, kv, dim, vdim, size, scale, diff, mlp):
    mixer = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "diff": diff}
    if size is not None:
        mixer["mask"] = {"size": size}
    return {"type": "attention", "mlp": mlp, "mixer": mixer}


def mlstm(heads, dim, vdim, cap, mlp):
    return {"type": "mlstm", "mlp": mlp, "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}}


def latent(heads, dim, vdim, rank, scale, mlp):
    return {"type": "latent_attention", "mlp": mlp, "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": rank, "scale": scale}}


# A: odd sizes; a chunk that is no multiple of a page; a layer without feed-forward; experts in groups of one; the
# recurrence first, so that its state meets the first tokens of the stream.
CONFIG_A = {"architecture": "Tesozen", "vocab": 211, "width": 72, "norm": {"eps": 1e-5}, "embedding": {"scale": 4.0},
            "layers": [mlstm(3, 10, 14, 9.0, moe(6, 2, 6, 3, 20, 28)), attention(4, 2, 20, 12, 23, 0.22, 0.25, dense(40)),
                       latent(3, 12, 10, 20, 0.3, None), attention(2, 2, 12, 28, 7, 0.3, 0.1, moe(8, 3, 2, 1, 16, 0, 1.0))]}
# B: every head with keys of its own; a chunk of one token (a query sees itself only); a chunk longer than any
# request; an attention without a mask; one group of experts; embedding scale 1.
CONFIG_B = {"architecture": "Tesozen", "vocab": 130, "width": 64, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0},
            "layers": [attention(4, 4, 16, 16, 1000, 0.25, 0.4, dense(48)), latent(2, 32, 16, 40, 0.18, moe(4, 4, 1, 1, 24, 16)),
                       attention(3, 3, 16, 40, 1, 0.25, 0.0, None), mlstm(1, 32, 64, 3.0, dense(30)),
                       attention(4, 1, 8, 16, None, 0.35, 0.05, moe(12, 2, 4, 2, 8, 40, 0.5))]}
# C: sizes of the tensor-core kernels (heads of 64 and 128, eight query heads on two key/value heads, a latent of
# 128), chunks of a few pages, sixteen experts in eight groups.
CONFIG_C = {"architecture": "Tesozen", "vocab": 300, "width": 128, "norm": {"eps": 1e-6}, "embedding": {"scale": 11.3},
            "layers": [attention(8, 2, 64, 128, 80, 0.125, 0.35, moe(16, 4, 8, 3, 64, 96, 2.5)), mlstm(2, 64, 128, 15.0, dense(192)),
                       latent(4, 64, 64, 128, 0.125, moe(16, 4, 8, 3, 64, 96, 2.5)), mlstm(4, 32, 32, 12.0, None),
                       attention(4, 4, 32, 32, 48, 0.18, 0.2, dense(160))]}
CONFIGS = {"A": CONFIG_A, "B": CONFIG_B, "C": CONFIG_C}
LENGTHS = {"A": [1, 2, 19, 77, 150], "B": [3, 33, 64, 129], "C": [5, 48, 100, 300]}
PAGE = {"A": 16, "B": 8, "C": 16}


class Logits(np.ndarray):
    """Logits [T, V] with ``close``: the places where a router's choice was a close call."""


def oracle(cfg, t64, toks):
    margins = []
    out = plain.forward(cfg, t64, toks, margins=margins).view(Logits)
    out.close = np.min(np.stack(margins), axis=0) < 0.01 if margins else np.zeros(len(toks), dtype=bool)
    return out


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    base = tmp_path_factory.mktemp("tesozen")
    out = {}
    for tag, cfg in CONFIGS.items():
        tensors = plain.random_tensors(cfg, seed=90 + ord(tag))
        folder = plain.write_folder(base / tag, cfg, tensors)
        rs = np.random.RandomState(ord(tag))
        reqs = {f"{tag.lower()}{i}": rs.randint(0, cfg["vocab"], n).tolist() for i, n in enumerate(LENGTHS[tag])}
        t64 = {k: v.astype(np.float64) for k, v in tensors.items()}
        want = {rid: oracle(cfg, t64, toks) for rid, toks in reqs.items()}
        out[tag] = (folder, cfg, t64, reqs, want)
    return out


def limit(dtype, want):
    big = max(float(np.abs(w).max()) for w in want.values())
    return (3e-5 if dtype == "float32" else 0.05) * big


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
    """In 32-bit every position must agree.  In bfloat16 rounding can turn a router's close call, which moves
    that position's logits visibly and, through the caches and the recurrence, later ones a little: the places
    that the plain model marks as close calls are not compared, and of the others at most 2 in 100 may differ,
    which a lost state, a wrong page or a wrong edge would exceed at once."""
    folder = models[tag][0]
    want = want or models[tag][4]
    outputs, session = replay(folder, dtype, trace, PAGE[tag], **kw)
    got = trace_tools.collect(trace, outputs)
    if dtype == "float32":
        bad = trace_tools.first_difference(got, want, limit(dtype, want))
        assert bad is None, f"first wrong place: request {bad[0]} position {bad[1]} |diff| {bad[2]:.3e} (limit {limit(dtype, want):.3e})"
        return session
    over, total, first = 0, 0, None
    for rid, rows in want.items():
        for p in range(rows.shape[0]):
            assert p in got.get(rid, {}), f"request {rid} position {p} was not answered"
            if rows.close[p]:
                continue
            d = float(np.abs(got[rid][p] - np.asarray(rows[p])).max())
            total += 1
            if not d <= limit(dtype, want):
                over += 1
                first = first or (rid, p, d)
    assert over <= 0.02 * total, f"{over} of {total} places differ; the first: request {first[0]} position {first[1]} |diff| {first[2]:.3e}"
    return session


def layer_tensors(layer, d, seed, prefix="l0.mix."):
    cfg = {"vocab": 4, "width": d, "layers": [layer]}
    t = plain.random_tensors(cfg, seed)
    return {k: v.astype(np.float64) for k, v in t.items()}, {k[len(prefix):]: v for k, v in t.items() if k.startswith(prefix)}


def put(t64, w, prefix="l0.mix."):
    for name, v in w.items():
        t64[prefix + name] = v.astype(np.float64)


# ------------------------------------------------------- mechanisms alone --

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("d", [72, 64, 6, 1537, 1])
def test_layer_norm_alone_added_to_the_stream_and_followed_by_the_next(dtype, d):
    from ayaka_py_b200.parts import PartSpec, make_part
    rs = np.random.RandomState(d)
    for n_rows in (1, 37):
        x = (rs.randn(n_rows, d) * 3 + 50.0).astype(np.float32)                     # a mean far from zero: the variance is about the mean
        w, b = (1.0 + 0.2 * rs.randn(d)).astype(np.float32), (0.3 * rs.randn(d)).astype(np.float32)
        norm = make_part(PartSpec("layernorm", {"width": d, "eps": 1e-5}), DT[dtype], "cuda")
        norm.bind({"weight": dev(w), "bias": dev(b)})
        want = plain.layer_norm(x.astype(np.float64), w.astype(np.float64), b.astype(np.float64), 1e-5)
        scale = max(1.0, float(np.abs(want).max()))
        got = norm.forward(dev(x), None)
        assert got.dtype == DT[dtype]
        assert np.abs(host(got) - want).max() < (2e-4 if dtype == "float32" else 2e-2) * scale
        base = rs.randn(n_rows, d).astype(np.float32)
        assert np.abs(host(norm.add_normed(dev(base), dev(x))) - (base + want)).max() < 2e-4 * scale
        w2, b2 = (1.0 + 0.2 * rs.randn(d)).astype(np.float32), (0.3 * rs.randn(d)).astype(np.float32)
        after = make_part(PartSpec("layernorm", {"width": d, "eps": 3e-5}), DT[dtype], "cuda")
        after.bind({"weight": dev(w2), "bias": dev(b2)})
        stream = dev(base)
        got = norm.add_normed_then(stream, dev(x), after)
        assert got.dtype == DT[dtype]
        assert np.abs(host(stream) - (base + want)).max() < 2e-4 * scale
        want2 = plain.layer_norm(base + want, w2.astype(np.float64), b2.astype(np.float64), 3e-5)
        assert np.abs(host(got) - want2).max() < (5e-4 if dtype == "float32" else 2e-2) * max(1.0, float(np.abs(want2).max()))
    if d > 1:                                                                        # an RMS norm would be another function
        assert np.abs(plain.unit_rms(x.astype(np.float64), 1e-5) * w + b - want).max() > 0.1


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("d,inner", [(72, 40), (64, 30), (128, 192), (48, 7)])
def test_squared_relu_feed_forward_alone(dtype, d, inner):
    from ayaka_py_b200.parts import PartSpec, make_part
    rs = np.random.RandomState(3)
    t64, w = layer_tensors(attention(2, 1, 8, 8, 4, 0.1, 0.2, dense(inner)), d, 19, prefix="l0.mlp.")
    part = make_part(PartSpec("mlp", {"width": d, "inner": inner, "activation": "relu2", "bias": False}), DT[dtype], "cuda")
    bind(part, w, {"up": "up_weight", "down": "down_weight"}, dtype)
    for n in (1, 5, 150):
        h = plain.round_bf16(rs.randn(n, d).astype(np.float32) * 2)
        want = plain.dense_ff(h.astype(np.float64), t64, "l0.mlp.")
        base = rs.randn(n, d).astype(np.float32)
        got = part.forward(dev(h, DT[dtype]), dev(base), None)
        assert got.dtype == torch.float32
        assert np.abs(host(got) - (base + want)).max() < tol(dtype, 3 * float(np.abs(want).max()))
    z = h.astype(np.float64) @ t64["l0.mlp.up"].T                                     # a plain ReLU, or a square without it, is another function
    assert np.abs(np.maximum(z, 0) @ t64["l0.mlp.down"].T - want).max() > 0.05 and np.abs((z * z) @ t64["l0.mlp.down"].T - want).max() > 0.05


MOE_CASES = [(12, 3, 3, 2, 16, 24), (8, 2, 1, 1, 24, 0), (16, 4, 8, 3, 8, 40), (6, 2, 6, 2, 20, 8), (4, 4, 2, 2, 64, 16), (64, 6, 8, 4, 8, 8)]


def moe_part(mlp, d, dtype):
    from ayaka_py_b200.parts import PartSpec, make_part
    r, sf = mlp["router"], (mlp["shared"]["ff"] if mlp["shared"] else 0)
    return make_part(PartSpec("moe", {"width": d, "experts": r["experts"], "top": r["top"], "inner": mlp["expert"]["ff"], "limit": None,
                                      "shared_inner": sf, "shared_limit": None, "router": "sigmoid_groups",
                                      "groups": r["groups"]["count"], "keep": r["groups"]["keep"], "route_scale": r["scale"],
                                      "slope": 1.0, "plus": 0.0, "shared_gated": False}), DT[dtype], "cuda")


def moe_names(mlp):
    names = {"router": "router_weight", "correction": "correction"}
    if mlp["shared"]:
        names.update({"shared.gate": "shared_gate", "shared.up": "shared_up", "shared.down": "shared_down"})
    for e in range(mlp["router"]["experts"]):
        names.update({f"e{e}.gate": f"gate_{e}", f"e{e}.up": f"up_{e}", f"e{e}.down": f"down_{e}"})
    return names


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("E,top,count,keep,ff,shared", MOE_CASES)
def test_experts_routed_by_scores_in_groups_alone(dtype, E, top, count, keep, ff, shared):
    """Routing and output for a single token, a few and many (the experts' products run through different kernels);
    corrections large enough to matter, some negative enough that an allowed expert's ranking score is below zero."""
    from ayaka_py_b200 import ops
    d = 48
    mlp = moe(E, top, count, keep, ff, shared, 1.7)
    t64, w = layer_tensors(attention(2, 1, 8, 8, 4, 0.1, 0.2, mlp), d, 100 + E, prefix="l0.mlp.")
    rs = np.random.RandomState(E)
    w["correction"] = plain.round_bf16((rs.randn(E) * 0.4 - 1.3).astype(np.float32))        # most ranking scores are below zero
    w["router"] = plain.round_bf16(w["router"] * 2)
    put(t64, w, "l0.mlp.")
    part = moe_part(mlp, d, dtype)
    bind(part, w, moe_names(mlp), dtype)
    below_zero = False
    for n in (1, 7, 150):
        h = plain.round_bf16(rs.randn(n, d).astype(np.float32) * 1.5)
        margins = []
        want = plain.moe_ff(h.astype(np.float64), t64, "l0.mlp.", mlp, margins)
        clear = margins[0] > 1e-4
        z = h.astype(np.float64) @ t64["l0.mlp.router"].T
        route = ops.moe_route(dev(z.astype(np.float32)), E, top, {"correction": dev(w["correction"]), "groups": count, "keep": keep, "factor": 1.7})
        ids, weights = route.ids.cpu().numpy(), host(route.weights)
        for t in np.flatnonzero(clear):
            chosen, wt = plain.route(z[t], t64["l0.mlp.correction"], top, count, keep, 1.7)
            assert ids[t].tolist() == chosen, (t, ids[t], chosen)
            assert np.abs(weights[t] - wt).max() < 1e-5
            below_zero = below_zero or (plain.sigmoid(z[t]) + t64["l0.mlp.correction"])[chosen].min() < 0
        got = host(part.forward(dev(h, DT[dtype]), None, None))
        big = float(np.abs(want).max())
        assert np.abs(got - want)[clear].max() < tol(dtype, 4 * big), n
        assert clear.mean() > 0.9
    assert below_zero              # chosen experts with ranking scores below zero: a dropped group counted as 0 would have won


ATT_NAMES = {"q": "q_weight", "k": "k_weight", "v": "v_weight", "q.norm": "q_norm", "k.norm": "k_norm", "lq1": "lq1",
             "lk1": "lk1", "lq2": "lq2", "lk2": "lk2", "g": "gate_weight", "o": "out_weight"}
MLSTM_NAMES = {"q": "q_weight", "k": "k_weight", "v": "v_weight", "i": "i_weight", "i.b": "i_bias", "f": "f_weight", "f.b": "f_bias",
               "g": "gate_weight", "norm": "norm_weight", "o": "out_weight"}
LATENT_NAMES = {"q": "q_weight", "dkv": "down_weight", "dkv.norm": "down_norm", "uk": "uk_weight", "uv": "uv_weight",
                "g": "gate_weight", "o": "out_weight"}


def attention_part(layer, d, dtype, eps=1e-5):
    from ayaka_py_b200.parts import PartSpec, make_part
    mx = layer["mixer"]
    return make_part(PartSpec("differential_attention",
                              {"width": d, "heads": mx["heads"], "kv_heads": mx["kv_heads"], "dim": mx["dim"], "vdim": mx["vdim"],
                               "scale": mx["scale"], "diff": mx["diff"], "eps": eps, "chunk": (mx.get("mask") or {}).get("size"),
                               "head_gate": True}), DT[dtype], "cuda")


def mlstm_part(layer, d, dtype, eps=1e-5):
    from ayaka_py_b200.parts import PartSpec, make_part
    mx = layer["mixer"]
    return make_part(PartSpec("mlstm", {"width": d, "heads": mx["heads"], "dim": mx["dim"], "vdim": mx["vdim"],
                                        "gate_cap": mx["gate_cap"], "eps": eps}), DT[dtype], "cuda")


def latent_part(layer, d, dtype, eps=1e-5):
    from ayaka_py_b200.parts import PartSpec, make_part
    mx = layer["mixer"]
    return make_part(PartSpec("latent_attention", {"width": d, "heads": mx["heads"], "dim": mx["dim"], "rot_dim": 0, "vdim": mx["vdim"],
                                                   "kv_rank": mx["kv_rank"], "scale": mx["scale"], "eps": eps, "rot": None,
                                                   "gate": "element"}), DT[dtype], "cuda")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,D,Dv,size", [(4, 2, 20, 12, 23), (3, 3, 16, 40, 1), (4, 1, 8, 16, None), (8, 2, 64, 128, 80),
                                           (2, 2, 12, 28, 7), (4, 4, 32, 32, 48), (2, 1, 128, 64, 1000), (5, 1, 16, 256, 16)])
def test_chunked_differential_attention_alone(dtype, H, G, D, Dv, size):
    d = 48
    layer = attention(H, G, D, Dv, size, 1.5 / np.sqrt(D), 0.45, None)
    t64, w = layer_tensors(layer, d, 29)
    part = attention_part(layer, d, dtype)
    bind(part, w, ATT_NAMES, dtype)
    mixer_alone(part, dtype, d, lambda h: plain.chunked_differential_attention(h, t64, "l0.mix.", layer["mixer"], 1e-5),
                {0: 150, 1: 9, 2: 70})


def chunk_edge_places(P, size, n):
    """The first tokens, page borders, the first and last position of chunks, and the end."""
    last = (n - 1) // size * size
    out = {0, 2, P - 1, P, P + 1, 5 * P - 1, 5 * P, n - 1, last, last - 1, last + 1, last - size, size - 1, size, size + 1}
    return sorted(p for p in out if 0 <= p < n)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,D,Dv,size", [(4, 2, 20, 12, 37), (8, 2, 64, 128, 70), (2, 1, 32, 64, 1000), (4, 1, 8, 16, 24), (3, 3, 16, 24, 100)])
def test_chunked_attention_with_keys_that_stand_out(dtype, H, G, D, Dv, size):
    """Keys made from the queries' matrix at chosen places score high against one another: the first and last
    key of a chunk, page borders, a key far back in a long chunk.  A chunk that is one position longer or
    shorter gives another output at the checked place."""
    rs = np.random.RandomState(17)
    d, P = 48, 8
    layer = attention(H, G, D, Dv, size, 8.0 / D, 0.35, None)
    t64, w = layer_tensors(layer, d, 37)
    per = H // G
    k = w["k"].reshape(G, 2, D, d).copy()
    q = w["q"].reshape(H, 2, D, d)
    for g in range(G):
        k[g, 0] = q[g * per, 0]
    w["k"] = k.reshape(G * 2 * D, d)
    w["q.norm"][:], w["k.norm"][:] = 1, 1
    put(t64, w)
    part = attention_part(layer, d, dtype)
    bind(part, w, ATT_NAMES, dtype)
    lengths = {0: 330, 1: 9, 2: 70}
    places = {0: chunk_edge_places(P, size, 330), 1: [0, 8], 2: [3, 2 * P, 69]}
    rows = {i: standing_out_rows(rs, n, d, places[i]) for i, n in lengths.items()}
    want = mixer_alone(part, dtype, d, lambda h: plain.chunked_differential_attention(h, t64, "l0.mix.", layer["mixer"], 1e-5),
                       lengths, rows=rows, page_size=P)
    if size < 330:
        last = 329 // size * size                           # the last chunk's first query sees itself only; the key before it stands out
        for other_size in (size + 1, size - 1):
            other_mx = copy.deepcopy(layer["mixer"])
            other_mx["mask"]["size"] = other_size
            other = plain.chunked_differential_attention(rows[0].astype(np.float64), t64, "l0.mix.", other_mx, 1e-5)
            assert np.abs(other[last] - want[0][last]).max() > 0.01 * np.abs(want[0]).max(), other_size


def test_head_gate_and_lambda():
    """The layer's factor from its four vectors, with diff 0 and with a second map that weighs more than the
    first (values that one model's sizes would hide)."""
    d = 40
    for diff, gain in ((0.0, 1.0), (0.6, 6.0)):
        layer = attention(2, 1, 16, 24, 12, 0.3, diff, None)
        t64, w = layer_tensors(layer, d, 41)
        for name in ("lq2", "lk2"):
            w[name] = plain.round_bf16(np.abs(w[name]) * gain)
        put(t64, w)
        lam = plain.differential_lambda(t64, "l0.mix.", diff)
        part = attention_part(layer, d, "float32")
        bind(part, w, ATT_NAMES, "float32")
        assert abs(part.lam - lam) < 1e-6 * max(1.0, abs(lam))
        if gain > 1:
            assert lam < 0
        mixer_alone(part, "float32", d, lambda h: plain.chunked_differential_attention(h, t64, "l0.mix.", layer["mixer"], 1e-5),
                    {0: 40, 1: 6, 2: 17})


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,D,Dv,cap", [(3, 10, 14, 9.0), (1, 32, 64, 3.0), (2, 64, 128, 15.0), (4, 32, 32, 12.0), (2, 7, 5, 1.0),
                                        (1, 20, 256, 6.0), (1, 800, 8, 8.0)])
def test_mlstm_alone(dtype, H, D, Dv, cap):
    """Whole, token by token, in ragged portions (the chunked kernel meets chunks of every length), batched, and
    in slots that were used before; heads of 800 numbers take the token-by-token kernel for prompts too."""
    d = 48
    layer = mlstm(H, D, Dv, cap, None)
    t64, w = layer_tensors(layer, d, 43)
    part = mlstm_part(layer, d, dtype)
    bind(part, w, MLSTM_NAMES, dtype)
    mixer_alone(part, dtype, d, lambda h: plain.mlstm(h, t64, "l0.mix.", layer["mixer"], 1e-5), {0: 150, 1: 9, 2: 70})


@pytest.mark.parametrize("f_bias,i_bias,i_gain", [(6.0, 0.0, 1.0), (-6.0, 0.0, 1.0), (2.0, 8.0, 6.0), (0.0, -8.0, 6.0)])
def test_mlstm_with_strong_gates_and_long_memory(f_bias, i_bias, i_gain):
    """A forget gate near one (a token 300 back still counts), near zero (only the last tokens do), input gates
    that reach the cap from both sides (the running maximum moves; the first tokens divide by exp(-m) with m from
    0): 32-bit, whole against token by token against portions, and the two kernels against one another."""
    from ayaka_py_b200 import ops
    d, H, D, Dv = 48, 2, 16, 24
    layer = mlstm(H, D, Dv, 10.0, None)
    t64, w = layer_tensors(layer, d, 47)
    w["f.b"][:] = f_bias
    w["i.b"][:] = i_bias
    w["i"] = plain.round_bf16(w["i"] * i_gain)
    put(t64, w)
    part = mlstm_part(layer, d, "float32")
    bind(part, w, MLSTM_NAMES, "float32")
    rs = np.random.RandomState(3)
    rows = {0: standing_out_rows(rs, 330, d, [5, 29]), 1: standing_out_rows(rs, 9, d, [0]), 2: standing_out_rows(rs, 70, d, [3])}
    want = mixer_alone(part, "float32", d, lambda h: plain.mlstm(h, t64, "l0.mix.", layer["mixer"], 1e-5), {0: 330, 1: 9, 2: 70}, rows=rows)
    if f_bias >= 6.0:                                    # the token at place 5 is still felt 300 tokens later
        x = rows[0].astype(np.float64).copy()
        x[5] = 0.0
        other = plain.mlstm(x, t64, "l0.mix.", layer["mixer"], 1e-5)
        assert np.abs(other[320] - want[0][320]).max() > 1e-3 * np.abs(want[0]).max()
    # the chunked kernel and the token-by-token kernel on the same rows and an empty state
    from ayaka_py_b200.cache import CacheGroupSpec
    out = []
    for chunked, cols in ((True, 16), (True, 32), (False, 0)):       # blocks of 16 and of 32 value columns, and the walk
        cache, runner = context_for([CacheGroupSpec("g", part.cache_need(), 1)], "float32", max_requests=2, page_size=8, pages=8)
        ctx, res = step_of(cache, runner, {0: 330})
        proj = ops.linear(dev(rows[0]), part.in_weight, part.in_bias, out_dtype=torch.float32)
        out.append(host(ops.mlstm(proj, cache.state_layer(0, 0), part.norm_weight, ctx, H, D, Dv, 10.0, 1e-5, torch.float32,
                                  chunked=chunked, slice_cols=cols)))
        out.append(host(cache.state_layer(0, 0)[cache.slot_of[0]]))
        cache.commit(res)
    for k in (0, 2):
        assert np.abs(out[k] - out[4]).max() < 2e-4 * np.abs(out[4]).max()
        assert np.abs(out[k + 1] - out[5]).max() < 2e-4 * max(1.0, np.abs(out[5]).max())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,D,Dv,rank", [(3, 12, 10, 20), (2, 32, 16, 40), (4, 64, 64, 128), (1, 16, 48, 8), (8, 64, 48, 96), (2, 24, 256, 36)])
def test_latent_attention_without_rotation_alone(dtype, H, D, Dv, rank):
    d = 48
    layer = latent(H, D, Dv, rank, 1.5 / np.sqrt(D), None)
    t64, w = layer_tensors(layer, d, 53)
    part = latent_part(layer, d, dtype)
    bind(part, w, LATENT_NAMES, dtype)
    mixer_alone(part, dtype, d, lambda h: plain.plain_latent_attention(h, t64, "l0.mix.", layer["mixer"], 1e-5), {0: 150, 1: 9, 2: 70})


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_latent_attention_with_a_key_far_back(dtype):
    """The latent of two places is made to stand out against one query direction: a key 320 positions back, at a
    page's last cell, among hundreds of others, must carry the output."""
    rs = np.random.RandomState(19)
    d, H, D, Dv, rank, P = 48, 2, 16, 24, 32, 8
    layer = latent(H, D, Dv, rank, 0.4 / D, None)
    t64, w = layer_tensors(layer, d, 59)
    # keys k = U_k c and queries q = W_q h: with U_k U_k^T ~ I and W_q = U_k W_dkv the score is about c_i . c_j
    uk = np.linalg.qr(rs.randn(rank, rank))[0][:D].astype(np.float32)
    w["uk"] = plain.round_bf16(np.tile(uk, (H, 1)) * 4)
    w["q"] = plain.round_bf16((w["uk"].astype(np.float64) @ w["dkv"].astype(np.float64)).astype(np.float32))
    w["dkv.norm"][:] = 1
    put(t64, w)
    part = latent_part(layer, d, dtype)
    bind(part, w, LATENT_NAMES, dtype)
    lengths = {0: 330, 1: 9, 2: 70}
    places = {0: [7, 8, 5 * P - 1, 328], 1: [0, 8], 2: [3, 2 * P, 69]}
    rows = {i: standing_out_rows(rs, n, d, places[i]) for i, n in lengths.items()}
    want = mixer_alone(part, dtype, d, lambda h: plain.plain_latent_attention(h, t64, "l0.mix.", layer["mixer"], 1e-5),
                       lengths, rows=rows, page_size=P)
    x = rows[0].astype(np.float64).copy()
    x[7] = rs.randn(d)                                          # without that far key the output at 328 is another
    other = plain.plain_latent_attention(x, t64, "l0.mix.", layer["mixer"], 1e-5)
    assert np.abs(other[328] - want[0][328]).max() > 0.02 * np.abs(want[0]).max()


# --------------------------------------------------------------- whole models --

def test_layers_one_by_one_in_32_bit(models):
    """The residual stream after every layer against the plain model."""
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
        assert len(seen) == len(after) == len(cfg["layers"])
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
    want.update({rid: oracle(cfg, t64, toks) for rid, toks in extra.items()})
    reqs.update(extra)
    for seed in (0, 1):
        trace = trace_tools.mixed(reqs, seed=seed)
        assert max(len(s["entries"]) for s in trace) >= 3
        session = check(models, tag, dtype, trace, want=want)
        assert any(g["reused"] > 0 for g in session.cache.stats()["groups"].values())
    longer = {rid: toks for rid, toks in reqs.items() if len(toks) >= 19}
    check(models, tag, dtype, trace_tools.reopened(longer, seed=3), want={rid: want[rid] for rid in longer})


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tag", ["A", "C"])
def test_long_decoding_past_many_chunks(models, tag, dtype):
    folder, cfg, t64, _, _ = models[tag]
    toks = np.random.RandomState(11).randint(0, cfg["vocab"], 420).tolist()
    want = {"long": oracle(cfg, t64, toks)}
    check(models, tag, dtype, trace_tools.tail_decoded({"long": toks}, 400), want=want)


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
    assert worst < 5e-5


def test_pages_behind_the_chunk_come_back(models):
    """A model of chunked attentions only, a long request in a pool smaller than its length: the pages of chunks
    that are over are handed out again."""
    cfg = {"architecture": "Tesozen", "vocab": 90, "width": 48, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.0},
           "layers": [attention(4, 2, 12, 16, 37, 0.3, 0.3, dense(40)), attention(2, 1, 16, 8, 37, 0.3, 0.1, None)]}
    tensors = plain.random_tensors(cfg, 77)
    import tempfile
    with tempfile.TemporaryDirectory() as tmp:
        folder = plain.write_folder(tmp, cfg, tensors)
        t64 = {k: v.astype(np.float64) for k, v in tensors.items()}
        toks = np.random.RandomState(12).randint(0, cfg["vocab"], 300).tolist()
        want = {"long": plain.forward(cfg, t64, toks)}
        trace = trace_tools.portions({"long": toks}, sizes=(5, 2, 11, 1, 1, 7))
        outputs, session = replay(folder, "float32", trace, 8, max_tokens=320)
        got = trace_tools.collect(trace, outputs)
        assert trace_tools.first_difference(got, want, limit("float32", want)) is None
        stats = session.cache.stats()["groups"]
        assert stats and all(g["high_water"] < 300 // 8 // 2 and g["reused"] > 0 for g in stats.values())


def moe_plain_topk(experts, top, ff, scale):
    """Experts without groups and without a shared expert."""
    return {"kind": "moe", "router": {"experts": experts, "top": top, "scale": scale}, "expert": {"ff": ff}}


OTHER_SHAPES = {
    # no attention at all: no pages, only state slots
    "only_mlstm": dict(vocab=101, width=50, layers=[mlstm(2, 9, 11, 5.0, dense(33)), mlstm(5, 6, 10, 20.0, None)]),
    # only the latent attention; experts without groups or shared expert, one expert chosen
    "only_latent": dict(vocab=333, width=96, layers=[latent(3, 24, 16, 48, 0.2, dense(100)), latent(6, 16, 32, 64, 0.25, moe_plain_topk(5, 1, 24, 3.0))]),
    # a width that is no multiple of 8, heads of 50 and 20, every group kept
    "odd_width": dict(vocab=257, width=100, layers=[attention(5, 5, 20, 20, 33, 0.2, 0.8, moe(9, 3, 3, 3, 28, 12)), mlstm(2, 50, 50, 12.0, dense(77)),
                                                    latent(2, 50, 50, 56, 0.14, None), attention(6, 2, 16, 48, 64, 0.25, 0.5, dense(64))]),
    # values of 320 numbers in the recurrence (the chunked kernel also takes the single-token steps), of 256 in the attention
    "wide_values": dict(vocab=64, width=64, layers=[mlstm(1, 16, 320, 8.0, dense(64)), attention(2, 1, 32, 256, 300, 0.17, 0.3, None)]),
    # 32 experts of which 8 are chosen from 2 of 4 groups; 24 in 12 groups of two; two experts, both chosen
    "many_experts": dict(vocab=512, width=128, layers=[attention(2, 1, 64, 64, 128, 0.125, 0.7, moe(32, 8, 4, 2, 32, 64, 1.0)),
                                                       mlstm(8, 16, 16, 10.0, moe(24, 6, 12, 3, 16, 16, 2.5)), latent(16, 8, 8, 16, 0.35, moe(2, 2, 2, 2, 8, 8))]),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(OTHER_SHAPES))
def test_other_shapes_whole_decoded_in_portions_and_mixed(tmp_path, name, dtype):
    c = OTHER_SHAPES[name]
    cfg = {"architecture": "Tesozen", "vocab": c["vocab"], "width": c["width"], "norm": {"eps": 1e-6},
           "embedding": {"scale": float(c["width"]) ** 0.5}, "layers": c["layers"]}
    tensors = plain.random_tensors(cfg, seed=len(name))
    t64 = {k: v.astype(np.float64) for k, v in tensors.items()}
    rs = np.random.RandomState(1)
    reqs = {f"r{i}": rs.randint(0, c["vocab"], n).tolist() for i, n in enumerate([1, 37, 130])}
    want = {rid: oracle(cfg, t64, toks) for rid, toks in reqs.items()}
    folder = plain.write_folder(tmp_path / name, cfg, tensors)
    models = {name: (folder, cfg, t64, reqs, want)}
    PAGE[name] = 16
    for trace in (trace_tools.whole(reqs), trace_tools.tail_decoded(reqs, 40), trace_tools.portions(reqs), trace_tools.mixed(reqs, seed=2)):
        check(models, name, dtype, trace)


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
    """A folder written by the engine's own random-weights mode loads, generates from the command line and replays a trace."""
    import subprocess
    import sys
    from pathlib import Path
    from ayaka_py_b200.config.model import TesozenConfig
    from ayaka_py_b200.weights import write_random_model
    folder = write_random_model(tmp_path / "m", TesozenConfig.from_dict(CONFIG_B), seed=3)
    assert json.loads((folder / "config.json").read_text())["architecture"] == "Tesozen"
    root = Path(__file__).resolve().parent.parent
    proc = subprocess.run([sys.executable, "-m", "ayaka_py_b200", "generate", str(folder), "--prompt-ids", "1,2,3,4,5",
                           "--max-tokens", "5", "--temperature", "0", "--ignore-eos", "--max-model-len", "64", "--kv-pages", "16"],
                          cwd=root, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    line = json.loads(proc.stdout.strip().splitlines()[-1])
    assert len(line["token_ids"]) == 5
    steps = "\n".join(json.dumps(s) for s in [{"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []},
                                              {"step": 1, "entries": [{"id": "a", "tokens": [9], "want": [0]}], "end": ["a"]}])
    proc = subprocess.run([str(root / "bin" / "trace_run"), "--model", str(folder), "--dtype", "float32", "--out", str(tmp_path / "out"),
                           "--max-tokens", "64"], input=steps + "\n", cwd=root, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert "done 0" in proc.stdout and "done 1" in proc.stdout
    assert np.fromfile(tmp_path / "out" / "0.f32", dtype="<f4").shape == (2 * CONFIG_B["vocab"],)
