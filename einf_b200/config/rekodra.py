"""Typed configuration of the Rekodra decoder: pre-norm layers with routed feed-forwards, a span
of layers that runs several times, and two mixers.

``config.json`` carries ``architecture: "Rekodra"``, ``vocab``, ``width``, ``norm.eps``,
``embedding.scale``, ``logit_scale``, ``loop`` (``start``, ``stop``, ``times``; optional) and ``layers``, a
list with one entry per layer: ``type`` (``parallel`` or ``attention``), ``mixer`` (that mixer's sizes
and constants) and ``mlp`` (``{"kind": "moe", "expert": {"ff": n}, "router": {"experts": E, "top": k,
"identity": I, "groups": {"count": c, "keep": k}}, "shared": {"ff": n}}``, or null for a layer without
a feed-forward).

The embedding row is multiplied by ``embedding.scale``.  A layer computes ``x += mixer(norm1 x);
x += ff(norm2 x)`` with RMS norms of plain weight.  Layers ``start .. stop - 1`` run ``times`` times in a
row with the same weights and a cache of their own each time; before every repeat the embedding
output is added to the stream.  The output matrix is the embedding table, unscaled; logits are
multiplied by ``logit_scale``.

``attention``: grouped-query softmax attention, causal, whose values are the keys as projected
(no value projection); queries and keys are RMS-normed over the whole projection with stored
weights, then the first ``rot.dims`` dimensions of every head are rotated (dimension i paired with
i + dims / 2, frequencies ``rot.base^(-2i/dims)``); a stored sink per head joins the softmax's denominator.

``parallel``: two mixers on one input.  ``left``: grouped-query softmax attention without rotation,
queries and keys RMS-normed head by head with one stored weight of the head's size each, a sliding
window of ``mask.size`` keys.  ``right``: a matrix memory with exponential gates capped at ``gate_cap``
(see the ``matrix_memory`` mixer).  The mixer's output is half the sum of the two branches' outputs,
each RMS-normed over the model width with a stored weight.

The feed-forward routes by softmax scores over ``experts + identity`` router outputs; the choice
adds a stored correction to the scores and is limited to the best ``groups.keep`` of ``groups.count``
groups of neighbouring outputs; the last ``identity`` outputs are experts that hand the token through;
weights are the scores, not renormalised; a shared expert with a sigmoid gate of its own is added.

Checkpoint names are ``embed``, ``l<i>.norm1|norm2``, ``l<i>.mix.<name>`` (``left.<name>``, ``right.<name>``,
``left.out``, ``right.out`` in a parallel layer), ``l<i>.mlp.router|correction``, ``l<i>.mlp.e<j>.gate|up|down``,
``l<i>.mlp.shared.gate|up|down|sg``, ``final.norm``.
"""
from __future__ import annotations

import dataclasses
from typing import Any, ClassVar, Optional

from .base import ConfigError, ModelConfig
from .specs import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

#: the design's fixed number: what is added to the matrix memory's denominator
MEMORY_DENOMINATOR_EPS = 1e-6
#: the mean of the two branches of a parallel mixer
PARALLEL_JOIN_SCALE = 0.5

_SINK_ATTENTION_NAMES = {
    "q_proj.weight": "q", "k_proj.weight": "k", "o_proj.weight": "o", "q_norm.weight": "q.norm",
    "k_norm.weight": "k.norm", "sink": "sink",
}
_WINDOW_ATTENTION_NAMES = {
    "q_proj.weight": "q", "k_proj.weight": "k", "v_proj.weight": "v", "o_proj.weight": "o",
    "q_norm.weight": "q.norm", "k_norm.weight": "k.norm",
}
_MEMORY_NAMES = {
    "q_proj.weight": "q", "k_proj.weight": "k", "v_proj.weight": "v", "g_proj.weight": "g", "o_proj.weight": "o",
    "i_proj.weight": "i", "i_proj.bias": "i.b", "f_proj.weight": "f", "f_proj.bias": "f.b", "norm.weight": "norm",
}


def _positive(where: str, value: Any) -> int:
    if not isinstance(value, int) or isinstance(value, bool) or value <= 0:
        raise ConfigError(f"{where} must be a positive integer, got {value!r}")
    return value


def _count(where: str, value: Any) -> int:
    if not isinstance(value, int) or isinstance(value, bool) or value < 0:
        raise ConfigError(f"{where} must be a count, got {value!r}")
    return value


def _number(where: str, value: Any) -> float:
    if isinstance(value, bool) or not isinstance(value, (int, float)):
        raise ConfigError(f"{where} must be a number, got {value!r}")
    return float(value)


def _require(where: str, data: Any, keys) -> None:
    if not isinstance(data, dict):
        raise ConfigError(f"{where} must be an object")
    missing = [key for key in keys if key not in data]
    if missing:
        raise ConfigError(f"{where} lacks {', '.join(missing)}")


def _heads(where: str, m: dict) -> None:
    _require(where, m, ("heads", "kv_heads", "dim", "vdim", "scale"))
    for key in ("heads", "kv_heads", "dim", "vdim"):
        _positive(f"{where}.{key}", m[key])
    _number(f"{where}.scale", m["scale"])
    if m["heads"] % m["kv_heads"]:
        raise ConfigError(f"{where}: {m['heads']} heads are not a multiple of {m['kv_heads']} kv_heads")


@dataclasses.dataclass(frozen=True)
class RekodraConfig(ModelConfig):
    architecture: ClassVar[str] = "Rekodra"

    vocab: int
    width: int
    layers: list
    norm: dict
    embedding: Optional[dict] = None
    logit_scale: float = 1.0
    loop: Optional[dict] = None

    def validate(self) -> None:
        _positive("vocab", self.vocab)
        _positive("width", self.width)
        if not isinstance(self.norm, dict) or not (float(self.norm.get("eps", 0)) > 0):
            raise ConfigError(f"norm.eps must be positive, got {self.norm!r}")
        if self.embedding is not None:
            _require("embedding", self.embedding, ("scale",))
            _number("embedding.scale", self.embedding["scale"])
        _number("logit_scale", self.logit_scale)
        if not isinstance(self.layers, (list, tuple)) or not self.layers:
            raise ConfigError("layers must be a non-empty list")
        if self.loop is not None:
            _require("loop", self.loop, ("start", "stop", "times"))
            start, stop = _count("loop.start", self.loop["start"]), _count("loop.stop", self.loop["stop"])
            _positive("loop.times", self.loop["times"])
            if not start < stop <= len(self.layers):
                raise ConfigError(f"loop must span layers inside the model, got {start} .. {stop} of {len(self.layers)}")
        for index, layer in enumerate(self.layers):
            where = f"layers[{index}]"
            if not isinstance(layer, dict):
                raise ConfigError(f"{where} must be an object")
            kind, mixer = layer.get("type"), layer.get("mixer")
            if kind not in ("parallel", "attention"):
                raise ConfigError(f"{where}.type must be parallel or attention, got {kind!r}")
            if kind == "attention":
                _heads(f"{where}.mixer", mixer)
                if mixer["vdim"] != mixer["dim"]:
                    raise ConfigError(f"{where}.mixer: the values are the keys, so vdim must equal dim")
                rot = mixer.get("rot")
                if rot is not None:
                    _require(f"{where}.mixer.rot", rot, ("base", "dims"))
                    dims = _positive(f"{where}.mixer.rot.dims", rot["dims"])
                    if dims % 2 or dims > mixer["dim"]:
                        raise ConfigError(f"{where}.mixer.rot.dims must be even and at most {mixer['dim']}, got {dims}")
                    if not _number(f"{where}.mixer.rot.base", rot["base"]) > 0:
                        raise ConfigError(f"{where}.mixer.rot.base must be positive")
            else:
                _require(f"{where}.mixer", mixer, ("left", "right"))
                left, right = mixer["left"], mixer["right"]
                _heads(f"{where}.mixer.left", left)
                if left.get("mask") is not None:
                    _positive(f"{where}.mixer.left.mask.size", (left["mask"] or {}).get("size"))
                _require(f"{where}.mixer.right", right, ("heads", "dim", "vdim", "gate_cap"))
                for key in ("heads", "dim", "vdim"):
                    _positive(f"{where}.mixer.right.{key}", right[key])
                if not _number(f"{where}.mixer.right.gate_cap", right["gate_cap"]) > 0:
                    raise ConfigError(f"{where}.mixer.right.gate_cap must be positive")
            mlp = layer.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind") != "moe":
                    raise ConfigError(f"{where}.mlp.kind must be 'moe', got {(mlp or {}).get('kind')!r}")
                _positive(f"{where}.mlp.expert.ff", (mlp.get("expert") or {}).get("ff"))
                router = mlp.get("router") or {}
                experts = _positive(f"{where}.mlp.router.experts", router.get("experts"))
                top = _positive(f"{where}.mlp.router.top", router.get("top"))
                outputs = experts + _count(f"{where}.mlp.router.identity", router.get("identity", 0))
                per_group, keep = outputs, 1
                if router.get("groups") is not None:
                    _require(f"{where}.mlp.router.groups", router["groups"], ("count", "keep"))
                    count = _positive(f"{where}.mlp.router.groups.count", router["groups"]["count"])
                    keep = _positive(f"{where}.mlp.router.groups.keep", router["groups"]["keep"])
                    if outputs % count or keep > count:
                        raise ConfigError(f"{where}.mlp.router: {outputs} outputs do not form {count} equal groups "
                                          f"of which {keep} are kept")
                    per_group = outputs // count
                if top > keep * per_group:
                    raise ConfigError(f"{where}.mlp.router: top {top} exceeds the {keep * per_group} outputs that can be chosen")
                if mlp.get("shared") is not None:
                    _positive(f"{where}.mlp.shared.ff", (mlp["shared"] or {}).get("ff"))

    def to_dict(self) -> dict[str, Any]:
        data = {"architecture": self.architecture}
        data.update(dataclasses.asdict(self))
        return data

    @property
    def eps(self) -> float:
        return float(self.norm["eps"])

    @property
    def init_std(self) -> float:
        # random matrices that keep activations of order one, so that scores spread
        return float(self.width) ** -0.5

    # The part-by-part description --------------------------------------
    def _norm(self, name: str) -> PartSpec:
        return PartSpec("rmsnorm", {"size": self.width, "eps": self.eps, "tensor_names": {"weight": ""}}, name)

    def _sink_attention(self, m: dict, prefix: str) -> PartSpec:
        rot = m.get("rot")
        position = PartSpec("none", {}) if rot is None else PartSpec(
            "rope", {"rotary_dim": int(rot["dims"]), "theta": float(rot["base"]), "layout": "halves"})
        return PartSpec(
            "attention",
            {
                "hidden_size": self.width, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"],
                "head_size": m["dim"], "value_head_size": m["vdim"], "qkv_bias": False, "out_bias": False,
                "scale": float(m["scale"]), "window": None, "values": "keys", "qk_unit_eps": self.eps,
                "qk_norm_weight": "row", "sink": True, "position": position,
                "tensor_names": _SINK_ATTENTION_NAMES,
            },
            prefix,
        )

    def _parallel(self, m: dict, prefix: str) -> PartSpec:
        left, right = m["left"], m["right"]
        attention = PartSpec(
            "attention",
            {
                "hidden_size": self.width, "num_heads": left["heads"], "num_kv_heads": left["kv_heads"],
                "head_size": left["dim"], "value_head_size": left["vdim"], "qkv_bias": False, "out_bias": False,
                "scale": float(left["scale"]), "window": (left.get("mask") or {}).get("size"),
                "qk_unit_eps": self.eps, "qk_norm_weight": "head", "position": PartSpec("none", {}),
                "tensor_names": _WINDOW_ATTENTION_NAMES,
            },
            prefix + "left.",
        )
        memory = PartSpec(
            "matrix_memory",
            {
                "hidden_size": self.width, "num_heads": right["heads"], "head_size": right["dim"],
                "value_head_size": right["vdim"], "gate_cap": float(right["gate_cap"]),
                "query_scale": float(right["dim"]) ** -0.5, "eps": self.eps,
                "denominator_eps": MEMORY_DENOMINATOR_EPS, "tensor_names": _MEMORY_NAMES,
            },
            prefix + "right.",
        )
        return PartSpec(
            "side_by_side",
            {"mixers": (attention, memory), "hidden_size": self.width,
             "join_norm": {"eps": self.eps, "scale": PARALLEL_JOIN_SCALE},
             "tensor_names": {"out.0": "left.out", "out.1": "right.out"}},
            prefix,
        )

    def _feed_forward(self, mlp: dict, prefix: str) -> PartSpec:
        router = mlp["router"]
        experts = int(router["experts"])
        names = {"router.weight": "router", "router.correction": "correction",
                 "shared.gate_proj.weight": "shared.gate", "shared.up_proj.weight": "shared.up",
                 "shared.down_proj.weight": "shared.down", "shared.gate.weight": "shared.sg"}
        for e in range(experts):
            for local, stored in (("gate_proj", "gate"), ("up_proj", "up"), ("down_proj", "down")):
                names[f"experts.{e}.{local}.weight"] = f"e{e}.{stored}"
        shared = mlp.get("shared")
        groups = router.get("groups")
        return PartSpec(
            "routed_mlp",
            {
                "hidden_size": self.width, "intermediate_size": int(mlp["expert"]["ff"]), "num_experts": experts,
                "num_identity": int(router.get("identity", 0)), "top_k": int(router["top"]), "score": "softmax",
                "renormalise": False, "weight_on": "output", "correction": True,
                "groups": None if groups is None else {"count": int(groups["count"]), "keep": int(groups["keep"])},
                "shared": None if shared is None else int(shared["ff"]), "shared_gate": shared is not None,
                "tensor_names": names,
            },
            prefix,
        )

    def layer_runs(self) -> list[tuple[int, bool]]:
        """The layers in the order they run, each with whether the embedding output is added ahead of it."""
        count = len(self.layers)
        if self.loop is None:
            return [(index, False) for index in range(count)]
        start, stop, times = int(self.loop["start"]), int(self.loop["stop"]), int(self.loop["times"])
        runs = [(index, False) for index in range(start)]
        for turn in range(times):
            runs += [(index, turn > 0 and index == start) for index in range(start, stop)]
        return runs + [(index, False) for index in range(stop, count)]

    def model_spec(self) -> ModelSpec:
        layers = []
        for index, layer in enumerate(self.layers):
            prefix = f"l{index}."
            build = self._parallel if layer["type"] == "parallel" else self._sink_attention
            parts = {
                "mixer_norm": self._norm(prefix + "norm1"),
                "mixer": build(layer["mixer"], prefix + "mix."),
            }
            mlp = layer.get("mlp")
            if mlp is not None:
                parts["feed_forward_norm"] = self._norm(prefix + "norm2")
                parts["feed_forward"] = self._feed_forward(mlp, prefix + "mlp.")
            layers.append(LayerSpec("prenorm" if mlp is not None else "prenorm_mixer", parts))
        schedule = tuple(ScheduleEntry(index, add_embedding=again) for index, again in self.layer_runs())
        scale = 1.0 if self.embedding is None else float(self.embedding["scale"])
        return ModelSpec(
            hidden_size=self.width,
            vocab_size=self.vocab,
            embedding=PartSpec(
                "embedding",
                {"vocab_size": self.vocab, "hidden_size": self.width, "scale": scale, "tensor_names": {"weight": "embed"}},
                "",
            ),
            layers=tuple(layers),
            schedule=schedule,
            final_norm=self._norm("final.norm"),
            head=PartSpec(
                "linear_head",
                {"vocab_size": self.vocab, "hidden_size": self.width, "tied_to": "embed",
                 "scale": float(self.logit_scale), "tensor_names": {"weight": "head"}},
                "",
            ),
        )
