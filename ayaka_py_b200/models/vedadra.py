"""Vedadra as data: which parts, with which constants, bound to which tensors.

A layer is a ``double_norm`` arrangement: a grouped RMS norm (the row in ``norm.groups`` runs, each with
its own root mean square) in front of and behind each sublayer, x += norm1b(mixer(norm1(x))); x +=
norm2b(ff(norm2(x))).  The mixer is, by the layer's ``type``, a ``talking_attention`` (``attention``:
the values are the projected keys, a distance bias per head, scores mixed across heads, an output
gate) or a ``differential_attention`` (``attention_2``: two score maps per head, a window that keeps
the first tokens); neither rotates.  The feed-forward is down(gelu_tanh(gate h) * (up h)) or absent.
``loop`` runs a stretch of layers several times with the same tensors: the run order names those
layers once per pass, every pass has caches of its own, and every pass but the first starts by adding
the embedding's output to the stream.  Layer i's tensors start with ``l<i>.``: ``norm1 norm1b norm2
norm2b`` and ``mix.*`` / ``mlp.*``; the model's own are ``embed``, ``final.norm`` and ``head``.
Linear weights are [out, in]."""

from __future__ import annotations

import math

from ..config.model import VedadraConfig
from ..parts.base import Init, LayerSpec, ModelSpec, PartSpec, RunStep, Source
from ..registry import Architecture, register_architecture

_GAMMA = Init(std=0.1, mean=1.0)
_BIAS = Init(std=0.3)


def vedadra_spec(config: VedadraConfig) -> ModelSpec:
    d, eps, groups = config.width, float(config.norm["eps"]), int(config.norm.get("groups", 1))

    def matrix(name: str, fan_in: int) -> Source:
        return Source(name, init=Init(std=1.0 / math.sqrt(fan_in)))

    def norm(name: str) -> PartSpec:
        return PartSpec("rmsnorm", {"width": d, "eps": eps, "groups": groups}, {"weight": Source(name, init=_GAMMA)})

    layers = []
    for i, layer in enumerate(config.layers):
        p, mx = f"l{i}.", layer["mixer"]
        H, G, D, Dv = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
        mask = mx.get("mask") or {}
        common = {"q_norm": Source(p + "mix.q.norm", init=_GAMMA), "k_norm": Source(p + "mix.k.norm", init=_GAMMA),
                  "out_weight": matrix(p + "mix.o", H * Dv)}
        if layer["type"] == "attention":
            mixer = PartSpec("talking_attention",
                             {"width": d, "heads": H, "kv_heads": G, "dim": D, "scale": float(mx["scale"]), "eps": eps,
                              "window": mask.get("size")},
                             {"q_weight": matrix(p + "mix.q", d), "q_bias": Source(p + "mix.q.b", init=_BIAS),
                              "k_weight": matrix(p + "mix.k", d), "k_bias": Source(p + "mix.k.b", init=_BIAS),
                              "talk": Source(p + "mix.talk", init=Init(std=0.5 / math.sqrt(H), mean=0.0)),
                              "temp": Source(p + "mix.temp", init=Init(std=0.2, mean=1.0)),
                              "gate_weight": matrix(p + "mix.g", d),
                              "out_bias": Source(p + "mix.o.b", init=_BIAS), **common})
        else:
            lam = Init(std=0.15)
            mixer = PartSpec("differential_attention",
                             {"width": d, "heads": H, "kv_heads": G, "dim": D, "vdim": Dv, "scale": float(mx["scale"]),
                              "diff": float(mx["diff"]), "eps": eps, "window": mask.get("size"),
                              "keep_first": int(mask.get("keep_first", 0))},
                             {"q_weight": matrix(p + "mix.q", d), "k_weight": matrix(p + "mix.k", d),
                              "v_weight": matrix(p + "mix.v", d),
                              "lq1": Source(p + "mix.lq1", init=lam), "lk1": Source(p + "mix.lk1", init=lam),
                              "lq2": Source(p + "mix.lq2", init=lam), "lk2": Source(p + "mix.lk2", init=lam), **common})
        parts = [("norm1", norm(p + "norm1")), ("mixer", mixer), ("norm1b", norm(p + "norm1b"))]
        if layer.get("mlp") is not None:
            ff = layer["mlp"]["ff"]
            ffn = PartSpec("gated_mlp", {"width": d, "inner": ff, "activation": "gelu_tanh"},
                           {"gate_weight": matrix(p + "mlp.gate", d), "up_weight": matrix(p + "mlp.up", d),
                            "down_weight": matrix(p + "mlp.down", ff)})
            parts += [("norm2", norm(p + "norm2")), ("ffn", ffn), ("norm2b", norm(p + "norm2b"))]
            layers.append(LayerSpec(tuple(parts), "double_norm"))
        else:
            layers.append(LayerSpec(tuple(parts), "double_norm_mixer_only"))

    return ModelSpec(
        vocab_size=config.vocab, hidden_size=d, max_positions=None,
        embedding=PartSpec("token_embedding", {"vocab": config.vocab, "width": d}, {"weight": Source("embed", init=Init(std=0.5))}),
        position=PartSpec("no_positions", {}, {}),
        layers=tuple(layers), order=tuple(RunStep(i, add_input=again) for i, again in config.run_order()),
        final_norm=norm("final.norm"),
        head=PartSpec("lm_head", {"vocab": config.vocab, "width": d}, {"weight": matrix("head", d)}))


def vedadra_normalize_name(name: str, config: VedadraConfig) -> str | None:
    """Tensors of the feed-forward sublayer of a layer that has none are passed over."""
    if name.startswith("l"):
        index, _, rest = name[1:].partition(".")
        if index.isdigit() and int(index) < len(config.layers) and config.layers[int(index)].get("mlp") is None:
            if rest in ("norm2", "norm2b") or rest.startswith("mlp."):
                return None
    return name


register_architecture(Architecture(
    name="Vedadra", model_type="vedadra", config_class=VedadraConfig,
    build_spec=vedadra_spec, normalize_name=vedadra_normalize_name))
