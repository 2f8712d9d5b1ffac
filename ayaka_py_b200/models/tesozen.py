"""Tesozen as data: which parts, with which constants, bound to which tensors.

A layer is a ``double_norm`` arrangement with layer norms (weight and bias) in front of and behind each
sublayer: x += norm1b(mixer(norm1(x))); x += norm2b(ff(norm2(x))).  The mixer is, by the layer's ``type``,
a ``differential_attention`` whose keys are visible inside the query's chunk only and whose heads pass a
gate of one number each (``attention``), an ``mlstm``, or a ``latent_attention`` without a rotated part and
with a gate per output number.  The feed-forward is ``mlp`` with the squared-ReLU activation and no biases
(``dense``), a ``moe`` routed by sigmoid scores in groups with silu-gated experts and an ungated shared
expert, or absent.  The embedding is multiplied by a constant; the head is the embedding table itself.
Layer i's tensors start with ``l<i>.``: ``norm1 norm1b norm2 norm2b`` (biases with ``.b`` added) and
``mix.*`` / ``mlp.*``; the model's own are ``embed`` and ``final.norm``.  Linear weights are [out, in]."""

from __future__ import annotations

import math

from ..config.model import TesozenConfig
from ..parts.base import Init, LayerSpec, ModelSpec, PartSpec, RunStep, Source
from ..registry import Architecture, register_architecture

_GAMMA = Init(std=0.1, mean=1.0)
_BETA = Init(std=0.1)


def tesozen_spec(config: TesozenConfig) -> ModelSpec:
    d, eps = config.width, float(config.norm["eps"])

    def matrix(name: str, fan_in: int, gain: float = 1.0) -> Source:
        return Source(name, init=Init(std=gain / math.sqrt(fan_in)))

    def norm(name: str) -> PartSpec:
        return PartSpec("layernorm", {"width": d, "eps": eps},
                        {"weight": Source(name, init=_GAMMA), "bias": Source(name + ".b", init=_BETA)})

    layers = []
    for i, layer in enumerate(config.layers):
        p, mx = f"l{i}.", layer["mixer"]
        m = p + "mix."
        if layer["type"] == "attention":
            H, G, D, Dv = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
            lam = Init(std=0.15)
            mixer = PartSpec("differential_attention",
                             {"width": d, "heads": H, "kv_heads": G, "dim": D, "vdim": Dv, "scale": float(mx["scale"]),
                              "diff": float(mx["diff"]), "eps": eps, "chunk": (mx.get("mask") or {}).get("size"),
                              "head_gate": True},
                             {"q_weight": matrix(m + "q", d), "k_weight": matrix(m + "k", d), "v_weight": matrix(m + "v", d),
                              "q_norm": Source(m + "q.norm", init=_GAMMA), "k_norm": Source(m + "k.norm", init=_GAMMA),
                              "lq1": Source(m + "lq1", init=lam), "lk1": Source(m + "lk1", init=lam),
                              "lq2": Source(m + "lq2", init=lam), "lk2": Source(m + "lk2", init=lam),
                              "gate_weight": matrix(m + "g", d), "out_weight": matrix(m + "o", H * Dv)})
        elif layer["type"] == "mlstm":
            H, D, Dv = mx["heads"], mx["dim"], mx["vdim"]
            mixer = PartSpec("mlstm",
                             {"width": d, "heads": H, "dim": D, "vdim": Dv, "gate_cap": float(mx["gate_cap"]), "eps": eps},
                             {"q_weight": matrix(m + "q", d), "k_weight": matrix(m + "k", d), "v_weight": matrix(m + "v", d),
                              "i_weight": matrix(m + "i", d), "i_bias": Source(m + "i.b", init=Init(std=0.5)),
                              "f_weight": matrix(m + "f", d), "f_bias": Source(m + "f.b", init=Init(std=1.0, mean=2.0)),
                              "gate_weight": matrix(m + "g", d), "norm_weight": Source(m + "norm", init=_GAMMA),
                              "out_weight": matrix(m + "o", H * Dv)})
        else:
            H, D, Dv, R = mx["heads"], mx["dim"], mx["vdim"], mx["kv_rank"]
            mixer = PartSpec("latent_attention",
                             {"width": d, "heads": H, "dim": D, "rot_dim": 0, "vdim": Dv, "kv_rank": R,
                              "scale": float(mx["scale"]), "eps": eps, "rot": None, "gate": "element"},
                             {"q_weight": matrix(m + "q", d), "down_weight": matrix(m + "dkv", d),
                              "down_norm": Source(m + "dkv.norm", init=_GAMMA), "uk_weight": matrix(m + "uk", R),
                              "uv_weight": matrix(m + "uv", R), "gate_weight": matrix(m + "g", d),
                              "out_weight": matrix(m + "o", H * Dv)})
        parts = [("norm1", norm(p + "norm1")), ("mixer", mixer), ("norm1b", norm(p + "norm1b"))]
        mlp = layer.get("mlp")
        if mlp is None:
            layers.append(LayerSpec(tuple(parts), "double_norm_mixer_only"))
            continue
        f = p + "mlp."
        if mlp["kind"] == "dense":
            ffn = PartSpec("mlp", {"width": d, "inner": mlp["ff"], "activation": "relu2", "bias": False},
                           {"up_weight": matrix(f + "up", d), "down_weight": matrix(f + "down", mlp["ff"])})
        else:
            router, shared = mlp["router"], mlp.get("shared")
            E, ff, sf = router["experts"], mlp["expert"]["ff"], (shared["ff"] if shared else 0)
            groups = router.get("groups") or {"count": 1, "keep": 1}
            sources = {"router_weight": matrix(f + "router", d, 2.0), "correction": Source(f + "correction", init=Init(std=0.2))}
            if sf:
                sources.update({"shared_gate": matrix(f + "shared.gate", d), "shared_up": matrix(f + "shared.up", d),
                                "shared_down": matrix(f + "shared.down", sf)})
            for e in range(E):
                sources[f"gate_{e}"] = matrix(f"{f}e{e}.gate", d)
                sources[f"up_{e}"] = matrix(f"{f}e{e}.up", d)
                sources[f"down_{e}"] = matrix(f"{f}e{e}.down", ff)
            ffn = PartSpec("moe", {"width": d, "experts": E, "top": router["top"], "inner": ff, "limit": None,
                                   "shared_inner": sf, "shared_limit": None, "router": "sigmoid_groups",
                                   "groups": groups["count"], "keep": groups["keep"],
                                   "route_scale": float(router.get("scale", 1.0)), "slope": 1.0, "plus": 0.0,
                                   "shared_gated": False}, sources)
        parts += [("norm2", norm(p + "norm2")), ("ffn", ffn), ("norm2b", norm(p + "norm2b"))]
        layers.append(LayerSpec(tuple(parts), "double_norm"))

    table = Source("embed", init=Init(std=0.5))
    return ModelSpec(
        vocab_size=config.vocab, hidden_size=d, max_positions=None,
        embedding=PartSpec("token_embedding", {"vocab": config.vocab, "width": d, "scale": float(config.embedding["scale"])},
                           {"weight": table}),
        position=PartSpec("no_positions", {}, {}),
        layers=tuple(layers), order=tuple(RunStep(i) for i in range(len(layers))),
        final_norm=norm("final.norm"),
        head=PartSpec("lm_head", {"vocab": config.vocab, "width": d}, {"weight": table}))


def tesozen_normalize_name(name: str, config: TesozenConfig) -> str | None:
    """Tensors of the feed-forward sublayer of a layer that has none are passed over."""
    if name.startswith("l"):
        index, _, rest = name[1:].partition(".")
        if index.isdigit() and int(index) < len(config.layers) and config.layers[int(index)].get("mlp") is None:
            if rest in ("norm2", "norm2b", "norm2.b", "norm2b.b") or rest.startswith("mlp."):
                return None
    return name


register_architecture(Architecture(
    name="Tesozen", model_type="tesozen", config_class=TesozenConfig,
    build_spec=tesozen_spec, normalize_name=tesozen_normalize_name))
