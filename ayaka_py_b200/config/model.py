"""Model configurations, read from the architecture's own ``config.json`` keys.

``GPT2Config`` keeps the Hugging Face short names (``n_layer``, ``n_embd`` ...)
and also accepts the long spellings the reference uses
(``models/gpt2.py:68-75``).  Defaults and checks follow ``models/gpt2.py:91-134``
with one difference: ``scale_attn_by_inverse_layer_idx`` is supported here (the
reference raises on it, ``models/gpt2.py:131-132``).
"""

from __future__ import annotations

import dataclasses
import json
import math
from dataclasses import dataclass
from pathlib import Path
from typing import Any, ClassVar, Mapping


class ConfigError(ValueError):
    """A configuration value is missing, of the wrong type or out of range."""


def _require_int(value: Any, name: str, minimum: int = 1) -> int:
    if isinstance(value, bool) or not isinstance(value, int):
        raise ConfigError(f"{name} must be an integer, got {value!r}")
    if value < minimum:
        raise ConfigError(f"{name} must be >= {minimum}, got {value}")
    return value


@dataclass(frozen=True)
class ModelConfig:
    """Base of every architecture's configuration.

    ``from_dict`` renames aliases, keeps the keys the dataclass declares and
    drops the rest (``models/_common.py:82-111``)."""

    ALIASES: ClassVar[Mapping[str, str]] = {}
    ARCHITECTURE: ClassVar[str] = ""

    @classmethod
    def from_dict(cls, values: Mapping[str, Any]):
        names = {f.name for f in dataclasses.fields(cls)}
        picked: dict[str, Any] = {}
        for key, value in values.items():
            key = cls.ALIASES.get(key, key)
            if key in names:
                if key in picked and picked[key] != value:
                    raise ConfigError(f"{key} is given twice with different values")
                picked[key] = value
        return cls(**picked)

    @classmethod
    def from_folder(cls, folder):
        return cls.from_dict(json.loads((Path(folder) / "config.json").read_text(encoding="utf-8")))

    def to_dict(self) -> dict[str, Any]:
        """The config.json document of this configuration."""
        doc = {"architectures": [self.ARCHITECTURE]}
        doc.update(dataclasses.asdict(self))
        return doc


_GPT2_ACTIVATIONS = ("gelu", "gelu_new", "gelu_fast", "gelu_pytorch_tanh", "quick_gelu")


@dataclass(frozen=True)
class GPT2Config(ModelConfig):
    ALIASES: ClassVar[Mapping[str, str]] = {
        "hidden_size": "n_embd",
        "num_hidden_layers": "n_layer",
        "num_attention_heads": "n_head",
        "max_position_embeddings": "n_positions",
        "intermediate_size": "n_inner",
        "layer_norm_eps": "layer_norm_epsilon",
    }
    ARCHITECTURE: ClassVar[str] = "GPT2LMHeadModel"

    vocab_size: int = 50257
    n_positions: int = 1024
    n_embd: int = 768
    n_layer: int = 12
    n_head: int = 12
    n_inner: int | None = None
    activation_function: str = "gelu_new"
    layer_norm_epsilon: float = 1e-5
    scale_attn_weights: bool = True
    scale_attn_by_inverse_layer_idx: bool = False
    reorder_and_upcast_attn: bool = False
    tie_word_embeddings: bool = True
    bos_token_id: int = 50256
    eos_token_id: int = 50256
    model_type: str = "gpt2"

    def __post_init__(self) -> None:
        for name in ("vocab_size", "n_positions", "n_embd", "n_layer", "n_head"):
            _require_int(getattr(self, name), name)
        if self.n_inner is not None:
            _require_int(self.n_inner, "n_inner")
        if self.n_embd % self.n_head:
            raise ConfigError(f"n_embd ({self.n_embd}) must be divisible by n_head ({self.n_head})")
        if self.activation_function not in _GPT2_ACTIVATIONS:
            raise ConfigError(
                f"unsupported activation_function {self.activation_function!r}; "
                f"expected one of {sorted(_GPT2_ACTIVATIONS)}")
        eps = self.layer_norm_epsilon
        if isinstance(eps, bool) or not isinstance(eps, (int, float)) or not math.isfinite(eps) or eps <= 0:
            raise ConfigError("layer_norm_epsilon must be finite and positive")
        for name in ("scale_attn_weights", "scale_attn_by_inverse_layer_idx",
                     "reorder_and_upcast_attn", "tie_word_embeddings"):
            if not isinstance(getattr(self, name), bool):
                raise ConfigError(f"{name} must be true or false")
        if self.reorder_and_upcast_attn:
            # It only asks for 32-bit attention scores, which every kernel here
            # computes anyway (the reference refuses it, models/gpt2.py:133-134).
            pass

    @property
    def head_dim(self) -> int:
        return self.n_embd // self.n_head

    @property
    def inner_size(self) -> int:
        """``n_inner``, or 4 * n_embd when it is null (models/gpt2.py:140-145)."""
        return self.n_inner if self.n_inner is not None else 4 * self.n_embd

    def attention_scale(self, layer: int) -> float:
        """Dh^-0.5 when ``scale_attn_weights`` (models/gpt2.py:147-149), divided
        by (layer + 1) when ``scale_attn_by_inverse_layer_idx``."""
        scale = self.head_dim ** -0.5 if self.scale_attn_weights else 1.0
        if self.scale_attn_by_inverse_layer_idx:
            scale /= float(layer + 1)
        return scale


def _require_number(value: Any, name: str, positive: bool = False) -> float:
    if isinstance(value, bool) or not isinstance(value, (int, float)) or not math.isfinite(value):
        raise ConfigError(f"{name} must be a finite number, got {value!r}")
    if positive and value <= 0:
        raise ConfigError(f"{name} must be positive, got {value}")
    return float(value)


_RAKALIX_MIXERS = {"latent_attention": ("heads", "dim", "rot_dim", "vdim", "kv_rank"),
                   "hgrn2": ("heads", "dim", "vdim")}


@dataclass(frozen=True)
class RakalixConfig(ModelConfig):
    """Rakalix: ``layers`` lists the layers in order, each {"type": which mixer, "mixer": its sizes
    and constants, "mlp": {"kind": "dense", "ff": n} or null}; ``norm.eps``, ``canon.taps``
    (the taps of the convolution over time in front of every sublayer), ``embedding.scale`` and
    ``residual_mult`` are the model-wide constants.  The document names the design under
    ``architecture``.  The model has no position limit of its own."""

    ARCHITECTURE: ClassVar[str] = "Rakalix"

    vocab: int = 0
    width: int = 0
    layers: tuple = ()
    norm: Mapping[str, Any] = dataclasses.field(default_factory=lambda: {"eps": 1e-6})
    canon: Mapping[str, Any] = dataclasses.field(default_factory=lambda: {"taps": 4})
    embedding: Mapping[str, Any] = dataclasses.field(default_factory=lambda: {"scale": 1.0})
    residual_mult: float = 1.0

    def __post_init__(self) -> None:
        _require_int(self.vocab, "vocab")
        _require_int(self.width, "width")
        if not isinstance(self.layers, (list, tuple)) or not self.layers:
            raise ConfigError("layers must be a non-empty list")
        object.__setattr__(self, "layers", tuple(self.layers))
        _require_number(self.norm.get("eps"), "norm.eps", positive=True)
        _require_int(self.canon.get("taps"), "canon.taps")
        _require_number(self.embedding.get("scale"), "embedding.scale")
        _require_number(self.residual_mult, "residual_mult")
        for i, layer in enumerate(self.layers):
            kind = layer.get("type") if isinstance(layer, Mapping) else None
            if kind not in _RAKALIX_MIXERS:
                raise ConfigError(f"layers[{i}].type must be one of {sorted(_RAKALIX_MIXERS)}, got {kind!r}")
            mixer = layer.get("mixer")
            if not isinstance(mixer, Mapping):
                raise ConfigError(f"layers[{i}].mixer must give the mixer's sizes")
            for key in _RAKALIX_MIXERS[kind]:
                _require_int(mixer.get(key), f"layers[{i}].mixer.{key}")
            if kind == "latent_attention":
                _require_number(mixer.get("scale"), f"layers[{i}].mixer.scale")
                rot = mixer.get("rot")
                if not isinstance(rot, Mapping):
                    raise ConfigError(f"layers[{i}].mixer.rot must give the rotation's constants")
                dims = _require_int(rot.get("dims"), f"layers[{i}].mixer.rot.dims")
                _require_number(rot.get("base"), f"layers[{i}].mixer.rot.base", positive=True)
                if dims % 2 or dims > mixer["rot_dim"]:
                    raise ConfigError(f"layers[{i}].mixer.rot.dims must be even and at most rot_dim")
                scaling = rot.get("scaling")
                if scaling is not None:
                    for key in ("factor", "original", "fast", "slow"):
                        _require_number(scaling.get(key) if isinstance(scaling, Mapping) else None,
                                        f"layers[{i}].mixer.rot.scaling.{key}", positive=True)
            mlp = layer.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, Mapping) or mlp.get("kind") != "dense":
                    raise ConfigError(f"layers[{i}].mlp.kind must be 'dense' (or mlp null), got {mlp!r}")
                _require_int(mlp.get("ff"), f"layers[{i}].mlp.ff")

    def to_dict(self) -> dict[str, Any]:
        return {"architecture": self.ARCHITECTURE, "vocab": self.vocab, "width": self.width,
                "layers": [json.loads(json.dumps(layer)) for layer in self.layers], "norm": dict(self.norm),
                "canon": dict(self.canon), "embedding": dict(self.embedding), "residual_mult": self.residual_mult}


_LUPORAX_MIXERS = {"attention": ("heads", "kv_heads", "dim", "vdim"),
                   "rglru": ("width", "blocks", "conv"),
                   "mingru": ("width",)}


@dataclass(frozen=True)
class LuporaxConfig(ModelConfig):
    """Luporax: ``layers`` lists the layer runs in order, each {"type": "attention" | "rglru" |
    "mingru", "mixer": its sizes and constants, "mlp": {"kind": "moe", "router": {experts, top},
    "expert": {ff, limit}, "shared": {ff, limit}} or null}; an entry with ``weights_of``: j runs
    layer j's tensors once more, with a cache and state of its own.  ``norm.eps``,
    ``residual_mult`` and ``logit_scale`` are the model-wide constants.  The document names the
    design under ``architecture``.  The model has no position limit of its own."""

    ARCHITECTURE: ClassVar[str] = "Luporax"

    vocab: int = 0
    width: int = 0
    layers: tuple = ()
    norm: Mapping[str, Any] = dataclasses.field(default_factory=lambda: {"eps": 1e-6})
    residual_mult: float = 1.0
    logit_scale: float = 1.0

    def __post_init__(self) -> None:
        _require_int(self.vocab, "vocab")
        _require_int(self.width, "width")
        if not isinstance(self.layers, (list, tuple)) or not self.layers:
            raise ConfigError("layers must be a non-empty list")
        object.__setattr__(self, "layers", tuple(self.layers))
        _require_number(self.norm.get("eps") if isinstance(self.norm, Mapping) else None, "norm.eps", positive=True)
        _require_number(self.residual_mult, "residual_mult")
        _require_number(self.logit_scale, "logit_scale")
        for i, layer in enumerate(self.layers):
            kind = layer.get("type") if isinstance(layer, Mapping) else None
            if kind not in _LUPORAX_MIXERS:
                raise ConfigError(f"layers[{i}].type must be one of {sorted(_LUPORAX_MIXERS)}, got {kind!r}")
            mixer = layer.get("mixer")
            if not isinstance(mixer, Mapping):
                raise ConfigError(f"layers[{i}].mixer must give the mixer's sizes")
            for key in _LUPORAX_MIXERS[kind]:
                _require_int(mixer.get(key), f"layers[{i}].mixer.{key}")
            if kind == "attention":
                if mixer["heads"] % mixer["kv_heads"]:
                    raise ConfigError(f"layers[{i}].mixer: {mixer['heads']} heads cannot share {mixer['kv_heads']} key/value heads")
                _require_number(mixer.get("scale"), f"layers[{i}].mixer.scale")
                _require_number(mixer.get("softcap"), f"layers[{i}].mixer.softcap", positive=True)
                rot = mixer.get("rot")
                if not isinstance(rot, Mapping):
                    raise ConfigError(f"layers[{i}].mixer.rot must give the rotation's constants")
                dims = _require_int(rot.get("dims"), f"layers[{i}].mixer.rot.dims")
                _require_number(rot.get("base"), f"layers[{i}].mixer.rot.base", positive=True)
                if dims % 2 or dims > mixer["dim"]:
                    raise ConfigError(f"layers[{i}].mixer.rot.dims must be even and at most dim")
            elif kind == "rglru" and mixer["width"] % mixer["blocks"]:
                raise ConfigError(f"layers[{i}].mixer: width {mixer['width']} is not {mixer['blocks']} equal blocks")
            source = layer.get("weights_of")
            if source is not None:
                _require_int(source, f"layers[{i}].weights_of", minimum=0)
                if source >= i or "weights_of" in self.layers[source]:
                    raise ConfigError(f"layers[{i}].weights_of must name an earlier layer that has tensors of its own")
                theirs = self.layers[source]
                if layer["type"] != theirs["type"] or dict(mixer) != dict(theirs["mixer"]) or layer.get("mlp") != theirs.get("mlp"):
                    raise ConfigError(f"layers[{i}] runs layer {source}'s tensors but describes another layer")
            mlp = layer.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, Mapping) or mlp.get("kind") != "moe":
                    raise ConfigError(f"layers[{i}].mlp.kind must be 'moe' (or mlp null), got {mlp!r}")
                for group, keys in (("router", ("experts", "top")), ("expert", ("ff",)), ("shared", ("ff",))):
                    if not isinstance(mlp.get(group), Mapping):
                        raise ConfigError(f"layers[{i}].mlp.{group} is missing")
                    for key in keys:
                        _require_int(mlp[group].get(key), f"layers[{i}].mlp.{group}.{key}")
                for group in ("expert", "shared"):
                    _require_number(mlp[group].get("limit"), f"layers[{i}].mlp.{group}.limit", positive=True)
                if mlp["router"]["top"] > mlp["router"]["experts"]:
                    raise ConfigError(f"layers[{i}].mlp.router: top exceeds experts")

    def to_dict(self) -> dict[str, Any]:
        return {"architecture": self.ARCHITECTURE, "vocab": self.vocab, "width": self.width,
                "layers": [json.loads(json.dumps(layer)) for layer in self.layers], "norm": dict(self.norm),
                "residual_mult": self.residual_mult, "logit_scale": self.logit_scale}


_VEDADRA_MIXERS = {"attention": "talking_attention", "attention_2": "differential_attention"}


@dataclass(frozen=True)
class VedadraConfig(ModelConfig):
    """Vedadra: ``layers`` lists the layers in order, each {"type": "attention" | "attention_2", "mixer":
    {heads, kv_heads, dim, vdim, scale, mask: {size[, keep_first]}[, diff]}, "mlp": {"kind": "dense",
    "ff": n} or null}.  ``loop`` {start, stop, times} (or null): the layers start .. stop-1 run ``times``
    times in a row with the same tensors and a cache per pass.  ``norm`` {eps, groups}: every norm of the
    stream cuts the row into ``groups`` runs.  The document names the design under ``architecture``.  The
    model has no position limit of its own."""

    ARCHITECTURE: ClassVar[str] = "Vedadra"

    vocab: int = 0
    width: int = 0
    layers: tuple = ()
    loop: Mapping[str, Any] | None = None
    norm: Mapping[str, Any] = dataclasses.field(default_factory=lambda: {"eps": 1e-6, "groups": 1})

    def __post_init__(self) -> None:
        _require_int(self.vocab, "vocab")
        _require_int(self.width, "width")
        if not isinstance(self.layers, (list, tuple)) or not self.layers:
            raise ConfigError("layers must be a non-empty list")
        object.__setattr__(self, "layers", tuple(self.layers))
        if not isinstance(self.norm, Mapping):
            raise ConfigError("norm must give eps and groups")
        _require_number(self.norm.get("eps"), "norm.eps", positive=True)
        groups = _require_int(self.norm.get("groups", 1), "norm.groups")
        if self.width % groups:
            raise ConfigError(f"width {self.width} is not {groups} equal norm groups")
        if self.loop is not None:
            if not isinstance(self.loop, Mapping):
                raise ConfigError("loop must give start, stop and times (or be null)")
            start = _require_int(self.loop.get("start"), "loop.start", minimum=0)
            stop = _require_int(self.loop.get("stop"), "loop.stop", minimum=0)
            _require_int(self.loop.get("times"), "loop.times")
            if not start <= stop <= len(self.layers):
                raise ConfigError(f"loop runs layers {start} .. {stop - 1}; the model has {len(self.layers)}")
        for i, layer in enumerate(self.layers):
            kind = layer.get("type") if isinstance(layer, Mapping) else None
            if kind not in _VEDADRA_MIXERS:
                raise ConfigError(f"layers[{i}].type must be one of {sorted(_VEDADRA_MIXERS)}, got {kind!r}")
            mixer = layer.get("mixer")
            if not isinstance(mixer, Mapping):
                raise ConfigError(f"layers[{i}].mixer must give the mixer's sizes")
            for key in ("heads", "kv_heads", "dim", "vdim"):
                _require_int(mixer.get(key), f"layers[{i}].mixer.{key}")
            if mixer["heads"] % mixer["kv_heads"]:
                raise ConfigError(f"layers[{i}].mixer: {mixer['heads']} heads cannot share {mixer['kv_heads']} key/value heads")
            _require_number(mixer.get("scale"), f"layers[{i}].mixer.scale")
            mask = mixer.get("mask")
            if mask is not None:
                if not isinstance(mask, Mapping):
                    raise ConfigError(f"layers[{i}].mixer.mask must give the window's size")
                _require_int(mask.get("size"), f"layers[{i}].mixer.mask.size")
                _require_int(mask.get("keep_first", 0), f"layers[{i}].mixer.mask.keep_first", minimum=0)
            if kind == "attention":
                if mixer["vdim"] != mixer["dim"]:
                    raise ConfigError(f"layers[{i}].mixer: the values are the keys, vdim must equal dim")
                if mask is not None and mask.get("keep_first"):
                    raise ConfigError(f"layers[{i}].mixer.mask: this mixer's window keeps no first tokens")
            else:
                _require_number(mixer.get("diff"), f"layers[{i}].mixer.diff")
            mlp = layer.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, Mapping) or mlp.get("kind") != "dense":
                    raise ConfigError(f"layers[{i}].mlp.kind must be 'dense' (or mlp null), got {mlp!r}")
                _require_int(mlp.get("ff"), f"layers[{i}].mlp.ff")

    def run_order(self) -> list[tuple[int, bool]]:
        """[(layer, the embedding's output is added first)] in the order in which the layers run."""
        n = len(self.layers)
        if self.loop is None:
            return [(i, False) for i in range(n)]
        start, stop, times = self.loop["start"], self.loop["stop"], self.loop["times"]
        order = [(i, False) for i in range(start)]
        for rep in range(times):
            order += [(i, rep > 0 and i == start) for i in range(start, stop)]
        return order + [(i, False) for i in range(stop, n)]

    def to_dict(self) -> dict[str, Any]:
        return {"architecture": self.ARCHITECTURE, "vocab": self.vocab, "width": self.width,
                "layers": [json.loads(json.dumps(layer)) for layer in self.layers],
                "loop": dict(self.loop) if self.loop is not None else None, "norm": dict(self.norm)}


_TESOZEN_MIXERS = {"attention": ("heads", "kv_heads", "dim", "vdim"),
                   "mlstm": ("heads", "dim", "vdim"),
                   "latent_attention": ("heads", "dim", "vdim", "kv_rank")}


@dataclass(frozen=True)
class TesozenConfig(ModelConfig):
    """Tesozen: ``layers`` lists the layers in order, each {"type": "attention" | "mlstm" | "latent_attention",
    "mixer": its sizes and constants, "mlp": {"kind": "dense", "ff": n}, {"kind": "moe", "router": {experts, top,
    scale, groups: {count, keep}}, "expert": {ff}, "shared": {ff}} or null}.  ``attention``: heads, kv_heads, dim,
    vdim, scale, diff and mask.size (the chunk inside which keys are seen; without ``mask`` every earlier key is);
    ``mlstm``: heads, dim, vdim, gate_cap; ``latent_attention``: heads, dim, vdim, kv_rank, scale.  ``norm.eps``
    and ``embedding.scale`` are the model-wide constants.  The document names the design under ``architecture``.
    The model has no position limit of its own."""

    ARCHITECTURE: ClassVar[str] = "Tesozen"

    vocab: int = 0
    width: int = 0
    layers: tuple = ()
    norm: Mapping[str, Any] = dataclasses.field(default_factory=lambda: {"eps": 1e-6})
    embedding: Mapping[str, Any] = dataclasses.field(default_factory=lambda: {"scale": 1.0})

    def __post_init__(self) -> None:
        _require_int(self.vocab, "vocab")
        _require_int(self.width, "width")
        if not isinstance(self.layers, (list, tuple)) or not self.layers:
            raise ConfigError("layers must be a non-empty list")
        object.__setattr__(self, "layers", tuple(self.layers))
        _require_number(self.norm.get("eps") if isinstance(self.norm, Mapping) else None, "norm.eps", positive=True)
        _require_number(self.embedding.get("scale") if isinstance(self.embedding, Mapping) else None, "embedding.scale")
        for i, layer in enumerate(self.layers):
            kind = layer.get("type") if isinstance(layer, Mapping) else None
            if kind not in _TESOZEN_MIXERS:
                raise ConfigError(f"layers[{i}].type must be one of {sorted(_TESOZEN_MIXERS)}, got {kind!r}")
            mixer = layer.get("mixer")
            if not isinstance(mixer, Mapping):
                raise ConfigError(f"layers[{i}].mixer must give the mixer's sizes")
            for key in _TESOZEN_MIXERS[kind]:
                _require_int(mixer.get(key), f"layers[{i}].mixer.{key}")
            if kind == "attention":
                if mixer["heads"] % mixer["kv_heads"]:
                    raise ConfigError(f"layers[{i}].mixer: {mixer['heads']} heads cannot share {mixer['kv_heads']} key/value heads")
                _require_number(mixer.get("scale"), f"layers[{i}].mixer.scale")
                _require_number(mixer.get("diff"), f"layers[{i}].mixer.diff")
                mask = mixer.get("mask")
                if mask is not None:
                    if not isinstance(mask, Mapping):
                        raise ConfigError(f"layers[{i}].mixer.mask must give the chunk's size")
                    _require_int(mask.get("size"), f"layers[{i}].mixer.mask.size")
            elif kind == "mlstm":
                _require_number(mixer.get("gate_cap"), f"layers[{i}].mixer.gate_cap", positive=True)
            else:
                _require_number(mixer.get("scale"), f"layers[{i}].mixer.scale")
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            if not isinstance(mlp, Mapping) or mlp.get("kind") not in ("dense", "moe"):
                raise ConfigError(f"layers[{i}].mlp.kind must be 'dense' or 'moe' (or mlp null), got {mlp!r}")
            if mlp["kind"] == "dense":
                _require_int(mlp.get("ff"), f"layers[{i}].mlp.ff")
                continue
            router, expert, shared = mlp.get("router"), mlp.get("expert"), mlp.get("shared")
            if not isinstance(router, Mapping) or not isinstance(expert, Mapping):
                raise ConfigError(f"layers[{i}].mlp must give router and expert")
            experts = _require_int(router.get("experts"), f"layers[{i}].mlp.router.experts")
            top = _require_int(router.get("top"), f"layers[{i}].mlp.router.top")
            _require_number(router.get("scale", 1.0), f"layers[{i}].mlp.router.scale")
            _require_int(expert.get("ff"), f"layers[{i}].mlp.expert.ff")
            if shared is not None:
                if not isinstance(shared, Mapping):
                    raise ConfigError(f"layers[{i}].mlp.shared must give the shared expert's size (or be null)")
                _require_int(shared.get("ff"), f"layers[{i}].mlp.shared.ff")
            groups = router.get("groups")
            count = keep = 1
            if groups is not None:
                if not isinstance(groups, Mapping):
                    raise ConfigError(f"layers[{i}].mlp.router.groups must give count and keep")
                count = _require_int(groups.get("count"), f"layers[{i}].mlp.router.groups.count")
                keep = _require_int(groups.get("keep"), f"layers[{i}].mlp.router.groups.keep")
            if experts % count or keep > count or keep * (experts // count) < top or top > experts:
                raise ConfigError(f"layers[{i}].mlp.router: {experts} experts in {count} groups of which {keep} are kept "
                                  f"cannot give {top} choices")

    def to_dict(self) -> dict[str, Any]:
        return {"architecture": self.ARCHITECTURE, "vocab": self.vocab, "width": self.width,
                "layers": [json.loads(json.dumps(layer)) for layer in self.layers], "norm": dict(self.norm),
                "embedding": dict(self.embedding)}
