"""Typed configuration of the Zogulorn decoder.

A Zogulorn config.json names its model class as the string `architecture` and
gives `vocab`, `width`, `norm.eps`, `embedding.scale` and a list `layers`; every
entry has a `type` (which mixer), the mixer's sizes and constants under `mixer`
and a feed-forward under `mlp` (or null).  An unknown mixer or feed-forward kind
is refused by name; a key outside the design is ignored with a warning.

    x0 = E[token] * embedding.scale
    x += s1 * mixer(dyt1(x));   x += s2 * ff(dyt2(x))              dyt(z) = tanh(alpha z) * w + b

Mixers.  `parallel`: a rotary, chunk-masked grouped-query attention with a
sigmoid gate per head (`left`) beside a gated delta rule behind short
convolutions whose decay is one number per head and key channel and whose
decay and output-gate projections are products of two thin matrices (`right`);
their results are summed with `left_scale` and `right_scale`.  `attention`:
chunk-masked differential attention behind short convolutions on q, k and v,
without rotation; with `kv_from: j` the layer has no keys and values of its own
and reads those of layer j's cache.
Feed-forwards.  `dense`: down(gelu_tanh(gate x) * (up x)).  `moe`: `top` of
`experts` two-matrix experts with the square of relu, router weights a softmax
over the chosen logits.

The design gives no limit on positions; `MAX_POSITIONS` is this library's
(positions are int32 on the device and are turned into float32 angles).
"""
from __future__ import annotations

import copy
import json
import warnings
from dataclasses import dataclass, field

from .base import ConfigError, LayerSpec, ModelPlan, PartSpec, ScheduleEntry, require

ARCHITECTURE = "Zogulorn"
MAX_POSITIONS = 1 << 22
UNIT_EPS = 1e-6            # under the root that makes q and k of the delta rule unit vectors: fixed by the design

_LEFT = {"heads": int, "kv_heads": int, "dim": int, "vdim": int, "scale": float, "mask": dict, "rot": dict}
_RIGHT = {"heads": int, "kv_heads": int, "dim": int, "vdim": int, "conv": int}
_ATTENTION = {"heads": int, "kv_heads": int, "dim": int, "vdim": int, "scale": float, "mask": dict, "conv": int,
              "diff": float}


def _typed(d, keys: dict, where: str, optional: tuple = ()) -> dict:
    """The listed keys of `d`, each of its type.  A key this library does not know is left out with a warning."""
    if not isinstance(d, dict):
        raise ConfigError(f"{where}: must be an object, found {d!r}")
    unknown = sorted(set(d) - set(keys) - set(optional))
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


def _attention_like(d, keys, where, optional=()):
    out = _typed(d, keys, where, optional)
    out["mask"] = _typed(out["mask"], {"size": int}, where + ".mask")
    if "rot" in out:
        out["rot"] = _typed(out["rot"], {"base": float, "dims": int}, where + ".rot")
    return out


@dataclass
class ZogulornConfig:
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float = 1.0
    layers: list = field(default_factory=list)      # the entries of config.json's `layers`, checked
    max_position_embeddings: int = MAX_POSITIONS    # not a key of the design: this library's own limit

    def __post_init__(self):
        self.validate()

    # ---- reading and writing -------------------------------------------------
    @classmethod
    def from_dict(cls, cfg: dict, where: str = "config.json") -> "ZogulornConfig":
        norm, emb = cfg.get("norm"), cfg.get("embedding")
        if not isinstance(norm, dict):
            raise ConfigError(f"{where}: key 'norm' must be an object with 'eps'")
        if not isinstance(emb, dict):
            raise ConfigError(f"{where}: key 'embedding' must be an object with 'scale'")
        layers = []
        for i, entry in enumerate(require(cfg, "layers", list, where)):
            w = f"{where}: layers[{i}]"
            if not isinstance(entry, dict):
                raise ConfigError(f"{w}: must be an object")
            unknown = sorted(set(entry) - {"type", "mixer", "mlp"})
            if unknown:
                warnings.warn(f"{w}: keys {unknown} are not part of the design and are ignored", stacklevel=2)
            typ = require(entry, "type", str, w)
            m = entry.get("mixer")
            if typ == "parallel":
                mixer = _typed(m, {"left": dict, "right": dict, "left_scale": float, "right_scale": float}, w + ".mixer")
                mixer["left"] = _attention_like(mixer["left"], _LEFT, w + ".mixer.left")
                rank = mixer["right"].get("rank") if isinstance(mixer["right"], dict) else None
                mixer["right"] = _typed(mixer["right"], _RIGHT, w + ".mixer.right", optional=("rank",))
                if rank is not None:             # this library's own key, written with random models (see thin_rank)
                    mixer["right"]["rank"] = require({"rank": rank}, "rank", int, w + ".mixer.right")
            elif typ == "attention":
                mixer = _attention_like(m, _ATTENTION, w + ".mixer", optional=("kv_from",))
                if isinstance(m, dict) and m.get("kv_from") is not None:
                    mixer["kv_from"] = require(m, "kv_from", int, w + ".mixer")
            else:
                raise ConfigError(f"{w}: mixer type {typ!r} is neither 'parallel' nor 'attention'")
            mlp = entry.get("mlp")
            if mlp is not None:
                kind = require(mlp, "kind", str, w + ".mlp")
                if kind == "dense":
                    mlp = _typed(mlp, {"kind": str, "ff": int}, w + ".mlp")
                elif kind == "moe":
                    mlp = _typed(mlp, {"kind": str, "expert": dict, "router": dict}, w + ".mlp")
                    mlp["expert"] = _typed(mlp["expert"], {"ff": int}, w + ".mlp.expert")
                    mlp["router"] = _typed(mlp["router"], {"experts": int, "top": int}, w + ".mlp.router")
                else:
                    raise ConfigError(f"{w}.mlp: kind {kind!r} is neither 'dense' nor 'moe'")
            layers.append({"type": typ, "mixer": mixer, "mlp": mlp})
        return cls(vocab=require(cfg, "vocab", int, where), width=require(cfg, "width", int, where),
                   norm_eps=require(norm, "eps", float, where + ": norm"),
                   embedding_scale=require(emb, "scale", float, where + ": embedding"), layers=layers)

    def to_dict(self) -> dict:
        return {"architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width,
                "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.norm_eps},
                "layers": copy.deepcopy(self.layers)}

    # ---- checks ----------------------------------------------------------------
    def validate(self) -> None:
        bad = []
        if self.vocab <= 0 or self.width <= 0:
            bad.append("vocab and width must be positive")
        if not self.norm_eps > 0:
            bad.append(f"norm.eps must be positive, found {self.norm_eps}")
        if not self.layers:
            bad.append("'layers' is empty")

        def heads(m, at):
            for k in ("heads", "kv_heads", "dim", "vdim"):
                if m[k] <= 0:
                    bad.append(f"{at}.{k} must be positive, found {m[k]}")
            if m["kv_heads"] > 0 and m["heads"] % m["kv_heads"]:
                bad.append(f"{at}: {m['heads']} heads are no multiple of {m['kv_heads']} kv_heads")

        def attention(m, at):
            heads(m, at)
            if m["mask"]["size"] <= 0:
                bad.append(f"{at}.mask.size must be positive, found {m['mask']['size']}")

        for i, layer in enumerate(self.layers):
            m, at = layer["mixer"], f"layers[{i}].mixer"
            if layer["type"] == "parallel":
                attention(m["left"], at + ".left")
                rot = m["left"]["rot"]
                if rot["dims"] % 2 or not 0 <= rot["dims"] <= m["left"]["dim"] or rot["base"] <= 0:
                    bad.append(f"{at}.left.rot: dims {rot['dims']} must be even and at most dim {m['left']['dim']}, "
                               "the base positive")
                heads(m["right"], at + ".right")
                if not 1 <= m["right"]["conv"] <= 16:
                    bad.append(f"{at}.right.conv = {m['right']['conv']} taps is outside this library's 1 to 16")
            else:
                attention(m, at)
                if not 1 <= m["conv"] <= 16:
                    bad.append(f"{at}.conv = {m['conv']} taps is outside this library's 1 to 16")
                j = m.get("kv_from")
                if j is not None:
                    src = self.layers[j] if 0 <= j < i else None
                    if src is None or src["type"] != "attention" or src["mixer"].get("kv_from") is not None:
                        bad.append(f"{at}.kv_from = {j} must name an earlier attention layer with keys and values "
                                   "of its own")
                    elif any(src["mixer"][k] != m[k] for k in ("heads", "kv_heads", "dim", "vdim")):
                        bad.append(f"{at}.kv_from = {j}: that layer's head counts and sizes differ from this one's")
            mlp = layer["mlp"]
            if mlp is not None and mlp["kind"] == "moe":
                r = mlp["router"]
                if not 0 < r["top"] <= r["experts"] or mlp["expert"]["ff"] <= 0:
                    bad.append(f"layers[{i}].mlp: top {r['top']} of {r['experts']} experts of {mlp['expert']['ff']}")
            elif mlp is not None and mlp["ff"] <= 0:
                bad.append(f"layers[{i}].mlp.ff must be positive")
        if bad:
            raise ConfigError("config: " + "; ".join(bad))

    # ---- the plan ----------------------------------------------------------------
    def _left(self, m: dict) -> dict:
        return dict(hidden_size=self.width, n_heads=m["heads"], n_kv_heads=m["kv_heads"], key_dim=m["dim"],
                    value_dim=m["vdim"], softmax_scale=m["scale"], mask={"kind": "chunk", "size": m["mask"]["size"]},
                    head_gate=True)

    def _right(self, m: dict) -> dict:
        # the inner size of the thin products is no key of the design: the tensors' shapes give it (`with_shapes`,
        # which the loader calls); without a file it is `rank` if the configuration carries one, else `thin_rank`
        return dict(hidden_size=self.width, n_heads=m["heads"], n_kv_heads=m["kv_heads"], key_dim=m["dim"],
                    value_dim=m["vdim"], conv_taps=m["conv"], eps=self.norm_eps, unit_eps=UNIT_EPS,
                    decay_per="channel", decay_rank=m.get("rank", self.thin_rank(m)),
                    gate_rank=m.get("rank", self.thin_rank(m)), out_gate="sigmoid")

    @staticmethod
    def thin_rank(m: dict) -> int:
        """The inner size of the two thin products of the delta rule when no file says otherwise (random models):
        an eighth of the read-out width, at least 8, a multiple of 8."""
        return max(8, (m["heads"] * m["vdim"] // 8 + 7) // 8 * 8)

    def with_shapes(self, shapes: dict) -> "ZogulornConfig":
        """The same configuration with the sizes that only the tensors give (the inner size of the delta rule's
        thin products, from `l<i>.mix.right.a1`) taken from `shapes` {tensor name: shape}."""
        out = copy.deepcopy(self)
        for i, layer in enumerate(out.layers):
            if layer["type"] == "parallel":
                name = f"l{i}.mix.right.a1"
                if name in shapes:
                    layer["mixer"]["right"]["rank"] = int(shapes[name][0])
        return out

    def _mixer_spec(self, i: int, layer: dict):
        m, p = layer["mixer"], f"l{i}.mix."
        if layer["type"] == "parallel":
            left, right = self._left(m["left"]), self._right(m["right"])
            params = dict(left={"kind": "masked_attention", "params": left},
                          right={"kind": "gated_delta_rule", "params": right},
                          left_scale=m["left_scale"], right_scale=m["right_scale"])
            names = ["left." + n for n in ("q", "k", "v", "g", "o")] + \
                    ["right." + n for n in ("q", "k", "v", "q.conv", "k.conv", "v.conv", "b", "A_log", "norm", "a1", "a2",
                                            "dt_bias", "g1", "g2", "o")]
            rot = m["left"]["rot"]
            rp = dict(head_dim=m["left"]["dim"], rotary_dim=rot["dims"], theta=rot["base"],
                      max_positions=self.max_position_embeddings, layout="interleaved", tables=False)
            return PartSpec("parallel_mixers", params, {n: p + n for n in names}), (rp if rot["dims"] else None)
        own = m.get("kv_from") is None
        params = dict(hidden_size=self.width, n_heads=m["heads"], n_kv_heads=m["kv_heads"], key_dim=m["dim"],
                      value_dim=m["vdim"], softmax_scale=m["scale"], mask={"kind": "chunk", "size": m["mask"]["size"]},
                      maps=2, diff=m["diff"], sub_norm_eps=self.norm_eps, out_mul=1.0 - m["diff"], conv_taps=m["conv"],
                      head_gate=True, own_kv=own)
        names = ["q", "q.conv", "lq1", "lk1", "lq2", "lk2", "g", "o"] + (["k", "v", "k.conv", "v.conv"] if own else [])
        return PartSpec("masked_attention", params, {n: p + n for n in names}), None

    def plan(self) -> ModelPlan:
        w = self.width
        norm = lambda name: PartSpec("dyt_norm", dict(size=w), dict(weight=name, bias=name + ".b", alpha=name + ".alpha"))
        scale = lambda name: PartSpec("channel_scale", dict(hidden_size=w), dict(weight=name))
        specs, positions, schedule = [], {}, []
        for i, layer in enumerate(self.layers):
            p = f"l{i}."
            mixer, rot = self._mixer_spec(i, layer)
            position = None
            if rot is not None:
                position = "rotary:" + json.dumps(rot, sort_keys=True)
                positions.setdefault(position, PartSpec("rotary", rot))
            norms, gates, ff = {"input": norm(p + "norm1")}, {"mixer": scale(p + "ls1")}, None
            mlp = layer["mlp"]
            if mlp is not None:
                norms["post_mixer"], gates["ff"] = norm(p + "norm2"), scale(p + "ls2")
                if mlp["kind"] == "dense":
                    ff = PartSpec("glu_mlp", dict(hidden_size=w, intermediate_size=mlp["ff"], activation="gelu_tanh"),
                                  {n: p + "mlp." + n for n in ("gate", "up", "down")})
                else:
                    E = mlp["router"]["experts"]
                    names = ["router"] + [f"e{e}.{n}" for e in range(E) for n in ("up", "down")]
                    ff = PartSpec("routed_experts",
                                  dict(hidden_size=w, expert_size=mlp["expert"]["ff"], n_experts=E,
                                       top=mlp["router"]["top"], activation="relu_squared"),
                                  {n: p + "mlp." + n for n in names})
            specs.append(LayerSpec("pre_norm_scaled_residual", mixer, ff, norms, position, gates))
            schedule.append(ScheduleEntry(layer=i, cache=i, kv_cache=layer["mixer"].get("kv_from")))
        return ModelPlan(
            architecture=ARCHITECTURE, hidden_size=w, vocab_size=self.vocab,
            max_positions=self.max_position_embeddings,
            embedding=PartSpec("token_embedding", dict(vocab_size=self.vocab, hidden_size=w,
                                                       scale=self.embedding_scale), dict(weight="embed")),
            positions=positions, layers=tuple(specs), schedule=tuple(schedule),
            final_norm=norm("final.norm"),
            head=PartSpec("linear_head", dict(hidden_size=w, vocab_size=self.vocab), dict(weight="head")))
