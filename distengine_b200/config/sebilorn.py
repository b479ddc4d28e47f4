"""Typed configuration of the Sebilorn decoder, read from its config.json.

The file names every size and every constant that differs between models of the design:

    {"architecture": "Sebilorn", "vocab": V, "width": D, "norm": {"eps": e},
     "embedding": {"scale": s}, "logit_softcap": c,
     "layers": [{"type": "attention" | "parallel" | "lightning", "mixer": {...},
                 "mlp": {"kind": "dense", "ff": F} | null}, ...]}

* ``attention`` mixer: ``heads``, ``kv_heads``, ``dim``, ``vdim`` (where absent: ``dim``),
  ``scale``, ``softcap`` (optional), ``mask`` (``size`` of the sliding window, ``keep_first``
  tokens that stay visible; without a mask every earlier token is seen), ``rot``
  (``dims``, ``base``, optional ``scaling`` with ``factor``, ``low``, ``high``, ``original``), and
  optionally ``kv_from``: the index of the earlier layer whose keys and values it reads instead of
  having matrices of its own.  Values are rotated by position and the heads' results turned back.
* ``parallel`` mixer: ``left`` (causal softmax attention with an output gate: ``heads``,
  ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``rot``) beside ``right`` (the generalized delta
  rule: ``heads``, ``dim``; the rank of its decay projection is the shape of its tensors), summed
  with ``left_scale`` and ``right_scale``.
* ``lightning`` mixer: ``heads``, ``dim``, ``vdim``, ``decay`` (one per head).
* ``mlp``: down(relu(up x)^2), or null for a layer without a feed-forward.

All norms are layer norms with weight and bias.  Layer i's tensors are named ``l<i>.*``; the
layers map onto the engine's parts as ``layer_specs`` says.  A model of this design has no
position limit of its own.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping

from .model import (ConfigError, LayerSpec, ModelConfig, PartSpec, PlanEntry, positive, require,
                    number as _number, positive_int as _int, section as _section)

NAME = "Sebilorn"
MAX_POSITIONS = 1 << 20          # the design names none; positions are exact in float32 far beyond


def _rotation(m: Mapping[str, Any], where: str, dim: int) -> tuple:
    """(dims, base, scaling or None) of a mixer's ``rot`` section."""
    rot = _section(m, "rot", where)
    dims = rot.get("dims")
    if type(dims) is not int or dims < 0 or dims % 2 or dims > dim:
        raise ConfigError(f"config.json: '{where}rot.dims' ({dims!r}) must be an even number from "
                          f"0 to '{where}dim' ({dim})")
    scaling = rot.get("scaling")
    if scaling is not None:
        sc = _section(rot, "scaling", where + "rot.")
        w = where + "rot.scaling."
        scaling = (_number(sc, "factor", w), _number(sc, "low", w), _number(sc, "high", w),
                   _number(sc, "original", w))
        if scaling[0] <= 0 or scaling[1] == scaling[2] or scaling[3] <= 0:
            raise ConfigError(f"config.json: '{where}rot.scaling' needs a positive factor and "
                              f"original, and low other than high")
    return dims, _number(rot, "base", where + "rot."), scaling


def _heads(m: Mapping[str, Any], where: str) -> tuple[int, int]:
    heads, kv_heads = _int(m, "heads", where), _int(m, "kv_heads", where)
    if heads % kv_heads:
        raise ConfigError(f"config.json: {where}heads ({heads}) must be a multiple of kv_heads "
                          f"({kv_heads})")
    return heads, kv_heads


def _attention(m: Mapping[str, Any], where: str, index: int) -> dict:
    heads, kv_heads = _heads(m, where)
    dim = _int(m, "dim", where)
    vdim = _int(m, "vdim", where) if m.get("vdim") is not None else dim
    if vdim % 2:
        raise ConfigError(f"config.json: '{where}vdim' ({vdim}) must be even: values are rotated "
                          f"in pairs")
    window, keep = None, 0                           # no mask: every earlier token is seen
    if m.get("mask") is not None:
        mask = _section(m, "mask", where)
        keep = mask.get("keep_first", 0)
        if type(keep) is not int or keep < 0:
            raise ConfigError(f"config.json: '{where}mask.keep_first' must be an integer >= 0")
        window = _int(mask, "size", where + "mask.")
    softcap = m.get("softcap")
    if softcap is not None:
        softcap = _number(m, "softcap", where)
        if softcap <= 0:
            raise ConfigError(f"config.json: '{where}softcap' must be positive")
    kv_from = m.get("kv_from")
    if kv_from is not None and (type(kv_from) is not int or not 0 <= kv_from < index):
        raise ConfigError(f"config.json: '{where}kv_from' ({kv_from!r}) must name an earlier layer")
    return {"kind": "attention", "heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
            "scale": _number(m, "scale", where), "softcap": softcap,
            "window": window, "keep_first": keep,
            "rot": _rotation(m, where, dim), "kv_from": kv_from}


def _parallel(m: Mapping[str, Any], where: str) -> dict:
    a, b = _section(m, "left", where), _section(m, "right", where)
    wa, wb = where + "left.", where + "right."
    heads, kv_heads = _heads(a, wa)
    dim = _int(a, "dim", wa)
    rank = b.get("rank")
    if rank is not None and (type(rank) is not int or rank <= 0):
        raise ConfigError(f"config.json: '{wb}rank' must be a positive integer")
    return {"kind": "parallel",
            "left": {"heads": heads, "kv_heads": kv_heads, "dim": dim,
                     "vdim": _int(a, "vdim", wa) if a.get("vdim") is not None else dim,
                     "scale": _number(a, "scale", wa),
                     "rot": _rotation(a, wa, dim)},
            "right": {"heads": _int(b, "heads", wb), "dim": _int(b, "dim", wb), "rank": rank},
            "left_scale": _number(m, "left_scale", where),
            "right_scale": _number(m, "right_scale", where)}


def _lightning(m: Mapping[str, Any], where: str) -> dict:
    heads = _int(m, "heads", where)
    decay = m.get("decay")
    if (not isinstance(decay, list) or len(decay) != heads
            or any(isinstance(x, bool) or not isinstance(x, (int, float)) for x in decay)):
        raise ConfigError(f"config.json: '{where}decay' must list one number for each of the "
                          f"{heads} heads")
    dim = _int(m, "dim", where)
    return {"kind": "lightning", "heads": heads, "dim": dim,
            "vdim": _int(m, "vdim", where) if m.get("vdim") is not None else dim,
            "decay": tuple(float(x) for x in decay)}


def _freeze(value):
    if isinstance(value, dict):
        return tuple(sorted((k, _freeze(v)) for k, v in value.items()))
    return value


def _thaw(value):
    if isinstance(value, tuple) and value and all(isinstance(x, tuple) and len(x) == 2
                                                  and isinstance(x[0], str) for x in value):
        return {k: _thaw(v) for k, v in value}
    return value


def _rot_json(rot: tuple) -> dict:
    dims, base, scaling = rot
    out: dict[str, Any] = {"dims": dims, "base": base}
    if scaling is not None:
        out["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    return out


@dataclass(frozen=True)
class SebilornConfig(ModelConfig):
    vocab: int
    model_width: int
    eps: float
    embed_scale: float
    softcap: "float | None"
    # per layer: (the mixer's parsed keys, frozen; feed-forward width or None)
    layers: tuple

    # ------------------------------------------------------------------ parsing
    @staticmethod
    def from_json(data: Mapping[str, Any]) -> "SebilornConfig":
        width = positive("width", require(data, "width", int))
        eps = _number(_section(data, "norm", ""), "eps", "norm.")
        if eps <= 0:
            raise ConfigError("config.json: 'norm.eps' must be positive")
        embed_scale = 1.0
        if data.get("embedding") is not None:
            embed_scale = _number(_section(data, "embedding", ""), "scale", "embedding.")
        softcap = data.get("logit_softcap")
        if softcap is not None:
            softcap = _number(data, "logit_softcap", "")
            if softcap <= 0:
                raise ConfigError("config.json: 'logit_softcap' must be positive")
        entries = data.get("layers")
        if not isinstance(entries, list) or not entries:
            raise ConfigError("config.json: 'layers' must be a nonempty list")
        layers, parsed_all = [], []
        for i, entry in enumerate(entries):
            where = f"layers[{i}]."
            if not isinstance(entry, Mapping):
                raise ConfigError(f"config.json: 'layers[{i}]' must be an object")
            kind = entry.get("type")
            mixer = _section(entry, "mixer", where)
            if kind == "attention":
                parsed = _attention(mixer, where + "mixer.", i)
                source = parsed["kv_from"]
                if source is not None:
                    theirs = parsed_all[source]
                    if theirs["kind"] != "attention" or theirs["kv_from"] is not None:
                        raise ConfigError(f"config.json: '{where}mixer.kv_from' must name an "
                                          f"attention layer with keys and values of its own")
                    same = ("kv_heads", "dim", "vdim", "rot")
                    if any(parsed[k] != theirs[k] for k in same):
                        raise ConfigError(f"config.json: layer {i} reads layer {source}'s keys "
                                          f"and values, so {', '.join(same)} must be equal")
            elif kind == "parallel":
                parsed = _parallel(mixer, where + "mixer.")
            elif kind == "lightning":
                parsed = _lightning(mixer, where + "mixer.")
            else:
                raise ConfigError(f"config.json: '{where}type' is '{kind}'; this design has "
                                  f"'attention', 'parallel' and 'lightning'")
            mlp = entry.get("mlp")
            ff = None
            if mlp is not None:
                if not isinstance(mlp, Mapping) or mlp.get("kind") != "dense":
                    raise ConfigError(f"config.json: '{where}mlp' must be null or of kind 'dense'")
                ff = _int(mlp, "ff", where + "mlp.")
            parsed_all.append(parsed)
            layers.append((_freeze(parsed), ff))
        return SebilornConfig(architecture=NAME,
                              vocab=positive("vocab", require(data, "vocab", int)),
                              model_width=width, eps=eps, embed_scale=embed_scale,
                              softcap=softcap, layers=tuple(layers))

    def to_json(self) -> dict[str, Any]:
        layers = []
        for frozen, ff in self.layers:
            m = _thaw(frozen)
            if m["kind"] == "attention":
                mixer: dict[str, Any] = {
                    "heads": m["heads"], "kv_heads": m["kv_heads"], "dim": m["dim"],
                    "vdim": m["vdim"], "scale": m["scale"], "rot": _rot_json(m["rot"])}
                if m["window"] is not None:
                    mixer["mask"] = {"size": m["window"], "keep_first": m["keep_first"]}
                if m["softcap"] is not None:
                    mixer["softcap"] = m["softcap"]
                if m["kv_from"] is not None:
                    mixer["kv_from"] = m["kv_from"]
            elif m["kind"] == "parallel":
                a, b = m["left"], m["right"]
                right = {"heads": b["heads"], "dim": b["dim"]}
                if b["rank"] is not None:
                    right["rank"] = b["rank"]
                mixer = {"left": {"heads": a["heads"], "kv_heads": a["kv_heads"], "dim": a["dim"],
                                  "vdim": a["vdim"], "scale": a["scale"],
                                  "rot": _rot_json(a["rot"])},
                         "right": right, "left_scale": m["left_scale"],
                         "right_scale": m["right_scale"]}
            else:
                mixer = {"heads": m["heads"], "dim": m["dim"], "vdim": m["vdim"],
                         "decay": list(m["decay"])}
            layers.append({"type": m["kind"], "mixer": mixer,
                           "mlp": None if ff is None else {"kind": "dense", "ff": ff}})
        out: dict[str, Any] = {"architecture": NAME, "vocab": self.vocab,
                               "width": self.model_width, "norm": {"eps": self.eps},
                               "embedding": {"scale": self.embed_scale}, "layers": layers}
        if self.softcap is not None:
            out["logit_softcap"] = self.softcap
        return out

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

    @property
    def embedding_scale(self) -> float:
        return self.embed_scale

    @property
    def logit_softcap(self) -> "float | None":
        return self.softcap

    def _norm(self, tensor: str) -> PartSpec:
        return PartSpec.of("layernorm", width=self.model_width, eps=self.eps, tensor=tensor,
                           bias=tensor + ".b")

    def _mixers(self) -> list[dict]:
        return [_thaw(frozen) for frozen, _ in self.layers]

    def layer_specs(self) -> list[LayerSpec]:
        """A pre-norm block per layer.  ``attention``: windowed attention with kept first tokens,
        soft cap and rotated values; ``parallel``: gated causal attention beside the generalized
        delta rule, summed with fixed weights; ``lightning``: a decayed state per head."""
        specs, d, mixers = [], self.model_width, self._mixers()
        # what the pages of an attention layer must keep: the widest window and the most kept
        # first tokens among the layer and those that read its keys and values
        window = {i: m["window"] for i, m in enumerate(mixers) if m["kind"] == "attention"}
        kept = {i: m["keep_first"] for i, m in enumerate(mixers) if m["kind"] == "attention"}
        for i, m in enumerate(mixers):
            if m["kind"] == "attention" and m["kv_from"] is not None:
                j = m["kv_from"]
                both = window[j] is not None and m["window"] is not None
                window[j] = max(window[j], m["window"]) if both else None
                kept[j] = max(kept[j], m["keep_first"])
        for i, (m, (_, ff)) in enumerate(zip(mixers, self.layers)):
            base = f"l{i}."
            if m["kind"] == "attention":
                owner = i if m["kv_from"] is None else m["kv_from"]
                dims, theta, scaling = m["rot"]
                part = PartSpec.of("window_attention", width=d, heads=m["heads"],
                                   kv_heads=m["kv_heads"], key_dim=m["dim"], value_dim=m["vdim"],
                                   scale=m["scale"], rotary_dim=dims, theta=theta, scaling=scaling,
                                   window=m["window"], keep_first=m["keep_first"],
                                   softcap=m["softcap"], rotate_values=True,
                                   owns_kv=m["kv_from"] is None, cache_window=window[owner],
                                   cache_keep_first=kept[owner])
            elif m["kind"] == "parallel":
                a, b = m["left"], m["right"]
                dims, theta, scaling = a["rot"]
                left = PartSpec.of("window_attention", width=d, heads=a["heads"],
                                   kv_heads=a["kv_heads"], key_dim=a["dim"], value_dim=a["vdim"],
                                   scale=a["scale"], rotary_dim=dims, theta=theta, scaling=scaling,
                                   gated=True)
                right = PartSpec.of("generalized_delta_rule", width=d, heads=b["heads"],
                                    key_dim=b["dim"], rank=b["rank"], eps=self.eps)
                part = PartSpec.of("parallel", width=d, eps=self.eps, combine="weighted_sum",
                                   scales=(m["left_scale"], m["right_scale"]),
                                   branches=(("left", left), ("right", right)))
            else:
                part = PartSpec.of("lightning_attention", width=d, heads=m["heads"],
                                   key_dim=m["dim"], value_dim=m["vdim"], decay=m["decay"],
                                   eps=self.eps)
            feed_forward = None
            if ff is not None:
                feed_forward = PartSpec.of("dense_mlp", width=d, inner=ff, activation="relu2",
                                           names=("up", "down"))
            specs.append(LayerSpec(
                block="prenorm", mixer=part, feed_forward=feed_forward, norm=self._norm("norm1"),
                feed_forward_norm=self._norm("norm2"),
                prefixes=(("mixer", base + "mix."), ("feed_forward", base + "mlp."),
                          ("mixer_norm", base), ("feed_forward_norm", base))))
        return specs

    def plan(self) -> list[PlanEntry]:
        """Every layer runs once, in order; a layer with ``kv_from`` reads that layer's cache."""
        return [PlanEntry(i, reads_cache_of=m["kv_from"] if m["kind"] == "attention" else None)
                for i, m in enumerate(self._mixers())]

    def final_norm(self) -> PartSpec:
        return self._norm("norm")

    def tensor_names(self) -> dict[str, str]:
        return {"embedding": "embed", "final_norm": "final.", "output": "head"}
