"""Typed configuration of the Kanavik decoder: pre-norm layers whose mixer is softmax attention
and a gated linear recurrence side by side, with a short convolution in front of every sublayer,
a per-layer token input and a weighted sum over the depth.

``config.json`` carries ``architecture: "Kanavik"``, ``vocab``, ``width``, ``max_positions``,
``norm.eps``, ``residual_mult``, ``canon.taps``, ``token_side.dim`` and ``layers``, a list with one
entry per layer: ``type`` (``parallel``), ``mixer`` (``left``, ``right``, ``left_scale``,
``right_scale``) and ``mlp`` (``{"kind": "dense", "ff": n}``, or null for a layer without a
feed-forward).

The embedding is the token's row plus a learned vector per position.  A layer computes
``x += m mixer(c(norm1 x)); x += m ff(c(norm2 x))`` with ``c(h) = h + conv(h)``, a causal
convolution of ``canon.taps`` taps per channel; then ``x += m rms(proj(gelu(gate x) * e)) w`` with e
the layer's slice of a second embedding table; then x becomes a learned weighted sum of the
embedding output and all layers' results so far.

``left``: grouped-query softmax attention without rotation: scores ``scale q.k - slope_h (i - j)``
with ``slope_h = 2^(-8 (h + 1) / heads)``, the heads' scores mixed by a stored matrix, a sliding
window of ``mask.size`` keys, one stored sink per head in the softmax's denominator.
``right``: ``y = gelu(W_y h + b)``, ``u = conv(W_x h + b)``; block-diagonal gates ``r, i =
sigmoid(W u + b)``; ``a = exp(-8 r softplus(lam))``; ``S <- a S + sqrt(1 - a^2) i u``; output
``W_o (S y)``.  The mixer's output is ``left_scale left + right_scale right``.

Checkpoint names are ``embed``, ``pos``, ``side.embed``, ``l<i>.norm1|norm2|canon1|canon2|dwa``,
``l<i>.mix.left.<name>``, ``l<i>.mix.right.<name>``, ``l<i>.mlp.gate|up|down``,
``l<i>.side.gate|proj|norm``, ``final.norm``, ``head``.
"""
from __future__ import annotations

import dataclasses
from typing import Any, ClassVar, Optional

from .base import ConfigError, ModelConfig
from .specs import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

#: the design's fixed numbers: the factor in the decay's logarithm and the base of the distance slopes
DECAY_CONSTANT = 8.0
SLOPE_EXPONENT = 8.0

_LEFT_NAMES = {
    "q_proj.weight": "q", "k_proj.weight": "k", "v_proj.weight": "v", "o_proj.weight": "o",
    "talk": "talk", "sink": "sink",
}
_RIGHT_NAMES = {
    "y_proj.weight": "y", "y_proj.bias": "y.b", "x_proj.weight": "x", "x_proj.bias": "x.b",
    "conv.weight": "conv", "conv.bias": "conv.b", "gate_a.weight": "ra", "gate_a.bias": "ra.b",
    "gate_i.weight": "ri", "gate_i.bias": "ri.b", "lam": "lam", "o_proj.weight": "o",
}
_MLP_NAMES = {"gate_proj.weight": "gate", "up_proj.weight": "up", "down_proj.weight": "down"}


def _positive(where: str, value: Any) -> int:
    if not isinstance(value, int) or isinstance(value, bool) or value <= 0:
        raise ConfigError(f"{where} must be a positive integer, got {value!r}")
    return value


def _number(where: str, value: Any) -> float:
    if isinstance(value, bool) or not isinstance(value, (int, float)):
        raise ConfigError(f"{where} must be a number, got {value!r}")
    return float(value)


def distance_slopes(heads: int) -> tuple[float, ...]:
    """``2^(-8 (h + 1) / heads)`` for head h."""
    return tuple(2.0 ** (-SLOPE_EXPONENT * (h + 1) / heads) for h in range(heads))


@dataclasses.dataclass(frozen=True)
class KanavikConfig(ModelConfig):
    architecture: ClassVar[str] = "Kanavik"

    vocab: int
    width: int
    max_positions: int
    layers: list
    norm: dict
    residual_mult: float = 1.0
    canon: Optional[dict] = None
    token_side: Optional[dict] = None

    def validate(self) -> None:
        _positive("vocab", self.vocab)
        _positive("width", self.width)
        _positive("max_positions", self.max_positions)
        _number("residual_mult", self.residual_mult)
        if not isinstance(self.norm, dict) or not (float(self.norm.get("eps", 0)) > 0):
            raise ConfigError(f"norm.eps must be positive, got {self.norm!r}")
        if self.canon is not None:
            _positive("canon.taps", (self.canon or {}).get("taps"))
        if self.token_side is not None:
            _positive("token_side.dim", (self.token_side or {}).get("dim"))
        if not isinstance(self.layers, (list, tuple)) or not self.layers:
            raise ConfigError("layers must be a non-empty list")
        for index, layer in enumerate(self.layers):
            where = f"layers[{index}]"
            if layer.get("type") != "parallel":
                raise ConfigError(f"{where}.type must be parallel, got {layer.get('type')!r}")
            mixer = layer.get("mixer")
            if not isinstance(mixer, dict) or not isinstance(mixer.get("left"), dict) or \
                    not isinstance(mixer.get("right"), dict):
                raise ConfigError(f"{where}.mixer must give left and right")
            for key in ("left_scale", "right_scale"):
                if key not in mixer:
                    raise ConfigError(f"{where}.mixer lacks {key}")
                _number(f"{where}.mixer.{key}", mixer[key])
            left, right = mixer["left"], mixer["right"]
            missing = [key for key in ("heads", "kv_heads", "dim", "vdim", "scale") if key not in left]
            missing += [key for key in ("width", "blocks", "conv") if key not in right]
            if missing:
                raise ConfigError(f"{where}.mixer lacks {', '.join(missing)}")
            for key in ("heads", "kv_heads", "dim", "vdim"):
                _positive(f"{where}.mixer.left.{key}", left[key])
            _number(f"{where}.mixer.left.scale", left["scale"])
            if left["heads"] % left["kv_heads"]:
                raise ConfigError(f"{where}: {left['heads']} heads are not a multiple of {left['kv_heads']} kv_heads")
            if left.get("mask") is not None:
                _positive(f"{where}.mixer.left.mask.size", left["mask"].get("size"))
            for key in ("width", "blocks", "conv"):
                _positive(f"{where}.mixer.right.{key}", right[key])
            if right["width"] % right["blocks"]:
                raise ConfigError(f"{where}: a width of {right['width']} is not a multiple of {right['blocks']} blocks")
            mlp = layer.get("mlp")
            if mlp is not None:
                if mlp.get("kind") != "dense":
                    raise ConfigError(f"{where}.mlp.kind must be 'dense', got {mlp.get('kind')!r}")
                _positive(f"{where}.mlp.ff", mlp.get("ff"))

    def to_dict(self) -> dict[str, Any]:
        data = {"architecture": self.architecture}
        data.update(dataclasses.asdict(self))
        return data

    @property
    def eps(self) -> float:
        return float(self.norm["eps"])

    @property
    def max_position_embeddings(self) -> int:
        return int(self.max_positions)

    @property
    def init_std(self) -> float:
        return float(self.width) ** -0.5

    # The part-by-part description --------------------------------------
    def _norm(self, name: str) -> PartSpec:
        return PartSpec("rmsnorm", {"size": self.width, "eps": self.eps, "tensor_names": {"weight": ""}}, name)

    def _conv(self, name: str) -> PartSpec:
        return PartSpec("causal_conv_input", {"size": self.width, "taps": int(self.canon["taps"]),
                                              "tensor_names": {"weight": ""}}, name)

    def _mixer(self, m: dict, prefix: str) -> PartSpec:
        left, right = m["left"], m["right"]
        attention = PartSpec(
            "attention",
            {
                "hidden_size": self.width,
                "num_heads": left["heads"],
                "num_kv_heads": left["kv_heads"],
                "head_size": left["dim"],
                "value_head_size": left["vdim"],
                "qkv_bias": False,
                "out_bias": False,
                "scale": float(left["scale"]),
                "window": (left.get("mask") or {}).get("size"),
                "distance_slopes": distance_slopes(int(left["heads"])),
                "talking_heads": True,
                "sink": True,
                "output_scale": float(m["left_scale"]),
                "position": PartSpec("none", {}),
                "tensor_names": _LEFT_NAMES,
            },
            prefix + "left.",
        )
        recurrence = PartSpec(
            "gated_linear_recurrence",
            {
                "hidden_size": self.width,
                "width": right["width"],
                "blocks": right["blocks"],
                "conv_taps": right["conv"],
                "decay_constant": DECAY_CONSTANT,
                "output_scale": float(m["right_scale"]),
                "tensor_names": _RIGHT_NAMES,
            },
            prefix + "right.",
        )
        return PartSpec("side_by_side", {"mixers": (attention, recurrence)}, prefix)

    def model_spec(self) -> ModelSpec:
        layers, schedule = [], []
        count = len(self.layers)
        for index, layer in enumerate(self.layers):
            prefix = f"l{index}."
            parts = {
                "mixer_norm": self._norm(prefix + "norm1"),
                "mixer": self._mixer(layer["mixer"], prefix + "mix."),
            }
            if self.canon is not None:
                parts["mixer_conv"] = self._conv(prefix + "canon1")
            mlp = layer.get("mlp")
            if mlp is not None:
                parts["feed_forward_norm"] = self._norm(prefix + "norm2")
                if self.canon is not None:
                    parts["feed_forward_conv"] = self._conv(prefix + "canon2")
                parts["feed_forward"] = PartSpec(
                    "gated_mlp",
                    {"hidden_size": self.width, "intermediate_size": int(mlp["ff"]), "activation": "gelu_tanh",
                     "tensor_names": _MLP_NAMES},
                    prefix + "mlp.",
                )
            if self.token_side is not None:
                dim = int(self.token_side["dim"])
                parts["token_input"] = PartSpec(
                    "token_side_input",
                    {"hidden_size": self.width, "size": dim, "vocab_size": self.vocab, "table_width": dim * count,
                     "table_offset": dim * index, "eps": self.eps,
                     "tensor_names": {"table": "side.embed", "gate.weight": prefix + "side.gate",
                                      "proj.weight": prefix + "side.proj", "norm.weight": prefix + "side.norm"}},
                    "",
                )
            parts["depth_mix"] = PartSpec(
                "depth_average", {"index": index, "layers": count, "tensor_names": {"weight": ""}}, prefix + "dwa"
            )
            layers.append(LayerSpec("prenorm_stream", parts, {"residual_mult": float(self.residual_mult)}))
            schedule.append(ScheduleEntry(index))
        return ModelSpec(
            hidden_size=self.width,
            vocab_size=self.vocab,
            embedding=PartSpec(
                "embedding",
                {"vocab_size": self.vocab, "hidden_size": self.width, "max_positions": int(self.max_positions),
                 "tensor_names": {"weight": "embed", "positions": "pos"}},
                "",
            ),
            layers=tuple(layers),
            schedule=tuple(schedule),
            final_norm=self._norm("final.norm"),
            head=PartSpec(
                "linear_head",
                {"vocab_size": self.vocab, "hidden_size": self.width, "tensor_names": {"weight": "head"}},
                "",
            ),
        )
