"""Typed configuration of the Fivitar decoder.

A Fivitar config.json names its model class as the string `architecture` and
gives `vocab`, `width`, `norm.eps` and a list `layers`; every entry of the list
has a `type` (which mixer), the mixer's sizes under `mixer`, a feed-forward
under `mlp` (or null) and, optionally, `weights_of: j`: the layer then runs
layer j's tensors on a cache entry of its own.  Nothing else is read: an
unknown mixer or feed-forward kind is refused by name, a key outside the
design is ignored with a warning.

The layer (x is the float32 residual stream, which every sublayer reads as it
is; there is no norm in front of a sublayer):

    x += norm1( sigmoid(R1 x + r1) * mixer(x) )
    x += norm2( sigmoid(R2 x + r2) * ff(x) )          (when the layer has a feed-forward)

Three mixers: `lightning` (linear attention with one fixed decay per head),
`latent_attention` (keys and values expanded from a cached low-rank latent,
one rotated key part shared by the heads, YaRN-scaled interleaved rotary
positions, a softmax whose denominator holds a learned sink per head) and
`delta` (the gated delta rule behind short causal convolutions).  The
feed-forward is a two-matrix MLP with the xIELU activation.

The design gives no limit on positions; `MAX_POSITIONS` is this library's
(positions are int32 on the device and are turned into float32 angles).
"""
from __future__ import annotations

import copy
import json
import warnings
from dataclasses import dataclass, field
from typing import Optional

from .base import ConfigError, LayerSpec, ModelPlan, PartSpec, ScheduleEntry, coerce, require

ARCHITECTURE = "Fivitar"
MAX_POSITIONS = 1 << 22

_MIXER_KEYS = {
    "lightning": {"heads": int, "dim": int, "vdim": int, "decay": list},
    "latent_attention": {"heads": int, "dim": int, "rot_dim": int, "vdim": int, "kv_rank": int, "scale": float,
                         "rot": dict},
    "delta": {"heads": int, "kv_heads": int, "dim": int, "vdim": int, "conv": int},
}


def _typed(d: dict, keys: dict, where: str) -> dict:
    """The listed keys of `d`, each of its type.  A key this library does not know is left out with a warning."""
    if not isinstance(d, dict):
        raise ConfigError(f"{where}: must be an object, found {d!r}")
    unknown = sorted(set(d) - set(keys))
    if unknown:
        warnings.warn(f"{where}: keys {unknown} are not part of the design and are ignored", stacklevel=3)
    out = {}
    for k, typ in keys.items():
        if typ is dict:
            if not isinstance(d.get(k), dict):
                raise ConfigError(f"{where}: key '{k}' must be an object")
            out[k] = copy.deepcopy(d[k])
        else:
            out[k] = require(d, k, typ, where)
    return out


def _rotary(rot: dict, where: str) -> dict:
    out = _typed({k: v for k, v in rot.items() if k != "scaling"}, {"base": float, "dims": int}, where)
    out["scaling"] = None
    if rot.get("scaling") is not None:
        out["scaling"] = _typed(rot["scaling"], {"factor": float, "original": float, "fast": float, "slow": float},
                                where + ".scaling")
    return out


@dataclass
class FivitarConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: list = field(default_factory=list)      # the entries of config.json's `layers`, checked
    max_position_embeddings: int = MAX_POSITIONS    # not a key of the design: this library's own limit

    def __post_init__(self):
        self.validate()

    # ---- reading and writing -------------------------------------------------
    @classmethod
    def from_dict(cls, cfg: dict, where: str = "config.json") -> "FivitarConfig":
        norm = cfg.get("norm")
        if not isinstance(norm, dict):
            raise ConfigError(f"{where}: key 'norm' must be an object with 'eps'")
        raw = require(cfg, "layers", list, where)
        layers = []
        for i, entry in enumerate(raw):
            w = f"{where}: layers[{i}]"
            if not isinstance(entry, dict):
                raise ConfigError(f"{w}: must be an object")
            unknown = sorted(set(entry) - {"type", "mixer", "mlp", "weights_of"})
            if unknown:
                warnings.warn(f"{w}: keys {unknown} are not part of the design and are ignored", stacklevel=2)
            typ = require(entry, "type", str, w)
            if typ not in _MIXER_KEYS:
                raise ConfigError(f"{w}: mixer type {typ!r} is not one of {sorted(_MIXER_KEYS)}")
            mixer = _typed(entry.get("mixer"), _MIXER_KEYS[typ], w + ".mixer")
            if typ == "latent_attention":
                mixer["rot"] = _rotary(mixer["rot"], w + ".mixer.rot")
            if typ == "lightning":
                mixer["decay"] = [coerce(v, "decay", float, w + ".mixer") for v in mixer["decay"]]
            mlp = entry.get("mlp")
            if mlp is not None:
                mlp = _typed(mlp, {"kind": str, "ff": int}, w + ".mlp")
                if mlp["kind"] != "dense":
                    raise ConfigError(f"{w}.mlp: kind {mlp['kind']!r} is not computed (only 'dense')")
            out = {"type": typ, "mixer": mixer, "mlp": mlp}
            if entry.get("weights_of") is not None:
                out["weights_of"] = require(entry, "weights_of", int, w)
            layers.append(out)
        return cls(vocab=require(cfg, "vocab", int, where), width=require(cfg, "width", int, where),
                   norm_eps=require(norm, "eps", float, where + ": norm"), layers=layers)

    def to_dict(self) -> dict:
        layers = copy.deepcopy(self.layers)
        for layer in layers:                          # an absent scaling stays absent
            rot = layer["mixer"].get("rot")
            if rot is not None and rot.get("scaling") is None:
                rot.pop("scaling", None)
        return {"architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width,
                "norm": {"eps": self.norm_eps}, "layers": layers}

    # ---- checks ----------------------------------------------------------------
    def validate(self) -> None:
        bad = []
        if self.vocab <= 0 or self.width <= 0:
            bad.append("vocab and width must be positive")
        if not self.norm_eps > 0:
            bad.append(f"norm.eps must be positive, found {self.norm_eps}")
        if not self.layers:
            bad.append("'layers' is empty")
        for i, layer in enumerate(self.layers):
            m, typ = layer["mixer"], layer["type"]
            for k, v in m.items():
                if isinstance(v, int) and not isinstance(v, bool) and v <= 0:
                    bad.append(f"layers[{i}].mixer.{k} must be positive, found {v}")
            if typ == "lightning" and len(m["decay"]) != m["heads"]:
                bad.append(f"layers[{i}]: {len(m['decay'])} decays for {m['heads']} heads")
            if typ == "delta":
                if m["heads"] % m["kv_heads"]:
                    bad.append(f"layers[{i}]: {m['heads']} heads are no multiple of {m['kv_heads']} kv_heads")
                if m["conv"] > 16:
                    bad.append(f"layers[{i}]: a convolution of {m['conv']} taps is beyond this library's 16")
            if typ == "latent_attention":
                rot = m["rot"]
                if rot["dims"] % 2 or rot["dims"] > m["rot_dim"]:
                    bad.append(f"layers[{i}]: rot.dims {rot['dims']} must be even and at most rot_dim {m['rot_dim']}")
            j = layer.get("weights_of")
            if j is not None:
                if not 0 <= j < len(self.layers) or j == i or self.layers[j].get("weights_of") is not None:
                    bad.append(f"layers[{i}].weights_of = {j} must name another layer that has tensors of its own")
                elif {k: v for k, v in self.layers[j].items() if k != "weights_of"} != \
                        {k: v for k, v in layer.items() if k != "weights_of"}:
                    bad.append(f"layers[{i}] uses the weights of layer {j} but its entry differs from that layer's")
        if bad:
            raise ConfigError("config: " + "; ".join(bad))

    # ---- the plan ----------------------------------------------------------------
    def _mixer_spec(self, i: int, layer: dict) -> PartSpec:
        m, p, eps = layer["mixer"], f"l{i}.mix.", self.norm_eps
        names = lambda *ns: {n: p + n for n in ns}
        if layer["type"] == "lightning":
            return PartSpec("decay_linear_attention",
                            dict(hidden_size=self.width, n_heads=m["heads"], key_dim=m["dim"], value_dim=m["vdim"],
                                 decay=tuple(m["decay"]), eps=eps, feature_map="silu", out_gate="sigmoid"),
                            names("q", "k", "v", "g", "o", "norm"))
        if layer["type"] == "delta":
            return PartSpec("gated_delta_rule",
                            dict(hidden_size=self.width, n_heads=m["heads"], n_kv_heads=m["kv_heads"],
                                 key_dim=m["dim"], value_dim=m["vdim"], conv_taps=m["conv"], eps=eps,
                                 unit_eps=1e-6),
                            names("q", "k", "v", "q.conv", "k.conv", "v.conv", "b", "a", "A_log", "dt_bias", "g",
                                  "o", "norm"))
        return PartSpec("latent_attention",
                        dict(hidden_size=self.width, n_heads=m["heads"], plain_dim=m["dim"], rot_dim=m["rot_dim"],
                             value_dim=m["vdim"], kv_rank=m["kv_rank"], softmax_scale=m["scale"], eps=eps,
                             sink=True),
                        names("q", "dkv", "dkv.norm", "uk", "uv", "sink", "o"))

    def plan(self) -> ModelPlan:
        eps, w = self.norm_eps, self.width
        own = [i for i, layer in enumerate(self.layers) if layer.get("weights_of") is None]
        index_of = {i: k for k, i in enumerate(own)}          # config layer -> index into the plan's layers
        specs, positions = [], {}
        for i in own:
            layer, p = self.layers[i], f"l{i}."
            norms = {"post_mixer": PartSpec("rms_norm", dict(size=w, eps=eps), dict(weight=p + "norm1"))}
            gates = {"mixer": PartSpec("sigmoid_gate", dict(hidden_size=w),
                                       dict(weight=p + "rg1", bias=p + "rg1.b"))}
            ff = None
            if layer["mlp"] is not None:
                ff = PartSpec("xielu_mlp", dict(hidden_size=w, intermediate_size=layer["mlp"]["ff"]),
                              dict(up=p + "mlp.up", down=p + "mlp.down", act=p + "mlp.act"))
                norms["post_ff"] = PartSpec("rms_norm", dict(size=w, eps=eps), dict(weight=p + "norm2"))
                gates["ff"] = PartSpec("sigmoid_gate", dict(hidden_size=w), dict(weight=p + "rg2", bias=p + "rg2.b"))
            position = None
            if layer["type"] == "latent_attention":
                # one table-less rotary part per distinct set of constants; angles are made from the position
                # in float32 where they are used, so no limit on positions enters
                rot, m = layer["mixer"]["rot"], layer["mixer"]
                params = dict(head_dim=m["rot_dim"], rotary_dim=rot["dims"], theta=rot["base"],
                              max_positions=self.max_position_embeddings, layout="interleaved",
                              yarn=rot["scaling"], tables=False)
                position = "rotary:" + json.dumps(params, sort_keys=True)
                positions.setdefault(position, PartSpec("rotary", params))
            specs.append(LayerSpec("post_norm_gated_residual", self._mixer_spec(i, layer), ff, norms, position, gates))
        schedule = tuple(ScheduleEntry(layer=index_of[layer.get("weights_of", i) if layer.get("weights_of") is not None
                                                      else i], cache=i)
                         for i, layer in enumerate(self.layers))
        return ModelPlan(
            architecture=ARCHITECTURE, hidden_size=w, vocab_size=self.vocab,
            max_positions=self.max_position_embeddings,
            embedding=PartSpec("token_embedding", dict(vocab_size=self.vocab, hidden_size=w), dict(weight="embed")),
            positions=positions, layers=tuple(specs), schedule=schedule,
            final_norm=PartSpec("rms_norm", dict(size=w, eps=eps), dict(weight="final.norm")),
            head=PartSpec("linear_head", dict(hidden_size=w, vocab_size=self.vocab), dict(weight="head")))
