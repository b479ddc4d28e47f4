"""Typed configuration of the Vomotar decoder, read from its config.json.

The file names every size and every constant that differs between models of the design:

    {"architecture": "Vomotar", "vocab": V, "width": D,
     "norm": {"eps": e, "groups": n},
     "layers": [{"type": "channel_delta" | "parallel", "mixer": {...}, "mlp": {...} | null}, ...]}

* ``channel_delta`` mixer: ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``conv`` (taps); the rank of
  its two low-rank projections is the shape of their tensors (an optional ``rank`` key is only
  what the random-weights mode draws them with).
* ``parallel`` mixer: ``left`` (softmax attention inside chunks of ``mask.size`` positions:
  ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``) and ``right`` (retention: ``heads``,
  ``dim``, ``vdim``, ``decay`` one per head, ``rot.dims`` and ``rot.base``).
* ``mlp``: ``{"kind": "dense", "ff": F}`` or null for a layer without a feed-forward.

Layer i's tensors are named ``l<i>.*``; the layers map onto the engine's parts as
``layer_specs`` says.  A model of this design has no position limit of its own.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping

from .model import (ConfigError, LayerSpec, ModelConfig, PartSpec, positive, require,
                    number as _number, positive_int as _int, section as _section)

NAME = "Vomotar"
MAX_POSITIONS = 1 << 20          # the design names none; positions are exact in float32 far beyond


def _delta(m: Mapping[str, Any], where: str) -> tuple:
    heads, kv_heads = _int(m, "heads", where), _int(m, "kv_heads", where)
    if heads % kv_heads:
        raise ConfigError(f"config.json: {where}heads ({heads}) must be a multiple of "
                          f"kv_heads ({kv_heads})")
    rank = m.get("rank")
    if rank is not None and (type(rank) is not int or rank <= 0):
        raise ConfigError(f"config.json: '{where}rank' must be a positive integer")
    return ("channel_delta", heads, kv_heads, _int(m, "dim", where), _int(m, "vdim", where),
            _int(m, "conv", where), rank)


def _parallel(m: Mapping[str, Any], where: str) -> tuple:
    a, b = _section(m, "left", where), _section(m, "right", where)
    wa, wb = where + "left.", where + "right."
    heads, kv_heads = _int(a, "heads", wa), _int(a, "kv_heads", wa)
    if heads % kv_heads:
        raise ConfigError(f"config.json: {wa}heads ({heads}) must be a multiple of kv_heads "
                          f"({kv_heads})")
    left = (heads, kv_heads, _int(a, "dim", wa), _int(a, "vdim", wa), _number(a, "scale", wa),
            _int(_section(a, "mask", wa), "size", wa + "mask."))
    rheads, rdim = _int(b, "heads", wb), _int(b, "dim", wb)
    decay = b.get("decay")
    if (not isinstance(decay, list) or len(decay) != rheads
            or any(isinstance(x, bool) or not isinstance(x, (int, float)) for x in decay)):
        raise ConfigError(f"config.json: '{wb}decay' must list one number for each of the "
                          f"{rheads} heads")
    rot = _section(b, "rot", wb)
    dims = rot.get("dims")
    if type(dims) is not int or dims < 0 or dims % 2 or dims > rdim:
        raise ConfigError(f"config.json: '{wb}rot.dims' ({dims!r}) must be an even number from 0 "
                          f"to '{wb}dim' ({rdim})")
    right = (rheads, rdim, _int(b, "vdim", wb), tuple(float(x) for x in decay), dims,
             _number(rot, "base", wb + "rot."))
    return ("parallel", left, right)


@dataclass(frozen=True)
class VomotarConfig(ModelConfig):
    vocab: int
    model_width: int
    eps: float
    groups: int
    # per layer: (mixer tuple as _delta / _parallel return it, feed-forward width or None)
    layers: tuple

    # ------------------------------------------------------------------ parsing
    @staticmethod
    def from_json(data: Mapping[str, Any]) -> "VomotarConfig":
        width = positive("width", require(data, "width", int))
        norm = _section(data, "norm", "")
        eps = _number(norm, "eps", "norm.")
        groups = _int(norm, "groups", "norm.")
        if eps <= 0 or width % groups:
            raise ConfigError(f"config.json: 'norm.eps' must be positive and 'norm.groups' "
                              f"({groups}) must divide 'width' ({width})")
        entries = data.get("layers")
        if not isinstance(entries, list) or not entries:
            raise ConfigError("config.json: 'layers' must be a nonempty list")
        layers = []
        for i, entry in enumerate(entries):
            where = f"layers[{i}]."
            if not isinstance(entry, Mapping):
                raise ConfigError(f"config.json: 'layers[{i}]' must be an object")
            kind = entry.get("type")
            mixer = _section(entry, "mixer", where)
            if kind == "channel_delta":
                parsed = _delta(mixer, where + "mixer.")
            elif kind == "parallel":
                parsed = _parallel(mixer, where + "mixer.")
            else:
                raise ConfigError(f"config.json: '{where}type' is '{kind}'; this design has "
                                  f"'channel_delta' and 'parallel'")
            mlp = entry.get("mlp")
            ff = None
            if mlp is not None:
                if not isinstance(mlp, Mapping) or mlp.get("kind") != "dense":
                    raise ConfigError(f"config.json: '{where}mlp' must be null or of kind 'dense'")
                ff = _int(mlp, "ff", where + "mlp.")
            layers.append((parsed, ff))
        return VomotarConfig(architecture=NAME, vocab=positive("vocab", require(data, "vocab", int)),
                             model_width=width, eps=eps, groups=groups, layers=tuple(layers))

    def to_json(self) -> dict[str, Any]:
        layers = []
        for mixer, ff in self.layers:
            if mixer[0] == "channel_delta":
                _, heads, kv_heads, dim, vdim, taps, rank = mixer
                m: dict[str, Any] = {"heads": heads, "kv_heads": kv_heads, "dim": dim,
                                     "vdim": vdim, "conv": taps}
                if rank is not None:
                    m["rank"] = rank
            else:
                _, a, b = mixer
                m = {"left": {"heads": a[0], "kv_heads": a[1], "dim": a[2], "vdim": a[3],
                              "scale": a[4], "mask": {"size": a[5]}},
                     "right": {"heads": b[0], "dim": b[1], "vdim": b[2], "decay": list(b[3]),
                               "rot": {"dims": b[4], "base": b[5]}}}
            layers.append({"type": mixer[0], "mixer": m,
                           "mlp": None if ff is None else {"kind": "dense", "ff": ff}})
        return {"architecture": NAME, "vocab": self.vocab, "width": self.model_width,
                "norm": {"eps": self.eps, "groups": self.groups}, "layers": layers}

    # ------------------------------------------------------------------ the model as data
    @property
    def width(self) -> int:
        return self.model_width

    @property
    def vocabulary(self) -> int:
        return self.vocab

    @property
    def max_positions(self) -> int:
        return MAX_POSITIONS

    @property
    def tied_output(self) -> bool:
        return False

    def _norm(self, tensor: str) -> PartSpec:
        return PartSpec.of("rmsnorm", width=self.model_width, eps=self.eps, groups=self.groups,
                           tensor=tensor)

    def layer_specs(self) -> list[LayerSpec]:
        """A pre-norm block per layer.  ``channel_delta`` is the gated delta rule with a decay
        per key channel; ``parallel`` runs chunk-masked softmax attention beside retention and
        averages their normalised outputs."""
        specs, d = [], self.model_width
        for i, (mixer, ff) in enumerate(self.layers):
            base = f"l{i}."
            if mixer[0] == "channel_delta":
                _, heads, kv_heads, dim, vdim, taps, rank = mixer
                part = PartSpec.of("gated_delta_rule", width=d, heads=heads, kv_heads=kv_heads,
                                   key_dim=dim, value_dim=vdim, taps=taps, rank=rank,
                                   eps=self.eps)
            else:
                _, a, b = mixer
                left = PartSpec.of("chunk_attention", width=d, heads=a[0], kv_heads=a[1],
                                   key_dim=a[2], value_dim=a[3], scale=a[4], chunk=a[5],
                                   eps=self.eps)
                right = PartSpec.of("retention", width=d, heads=b[0], key_dim=b[1],
                                    value_dim=b[2], decay=b[3], rotary_dim=b[4], theta=b[5],
                                    eps=self.eps)
                part = PartSpec.of("parallel", width=d, eps=self.eps,
                                   branches=(("left", left), ("right", right)))
            feed_forward = None
            if ff is not None:
                feed_forward = PartSpec.of("gated_mlp", width=d, inner=ff, activation="silu",
                                           names=("gate", "up", "down"))
            specs.append(LayerSpec(
                block="prenorm", mixer=part, feed_forward=feed_forward, norm=self._norm("norm1"),
                feed_forward_norm=self._norm("norm2"),
                prefixes=(("mixer", base + "mix."), ("feed_forward", base + "mlp."),
                          ("mixer_norm", base), ("feed_forward_norm", base))))
        return specs

    def final_norm(self) -> PartSpec:
        return self._norm("norm")

    def tensor_names(self) -> dict[str, str]:
        return {"embedding": "embed", "final_norm": "final.", "output": "head"}
