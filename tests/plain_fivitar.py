"""Plain, slow restatement of the Fivitar decoder, used only by the tests.

Whole sequences, no cache, token-by-token loops for the recurrences, one
function per mechanism, torch on the CPU in float32 (or float64 when asked).
It shares no code with the package under test: its own reader for config.json
and safetensors, its own arithmetic.

The design in this file's notation (x is the float32 residual stream, h what a
sublayer reads, which is x itself; there is no norm in front of a sublayer):

    layer:      x += norm1( sigmoid(R1 h + r1) * mixer(h) );  x += norm2( sigmoid(R2 h + r2) * ff(h) )
    norm:       y = x / sqrt(mean(x^2) + eps) * w
    ff:         D act(U h),  act(z) = softplus(p) z^2 + z/2                      for z > 0
                                      (1/2 + softplus(q)) (e^z - 1 - z) + z/2    for z <= 0
    lightning:  q, k, v = silu(W h);  S_t = lam_h S_(t-1) + k_t v_t^T;  o_t = S_t^T q_t;
                y = Wo( norm(concat o) * sigmoid(Wg h) )
    latent:     q = Wq h = [plain | rotated] per head;  [c | kr] = Wdkv h,  c <- norm(c);
                k_h = Wuk c,  v_h = Wuv c;  score = (q_plain . k_h + rot(q_rot) . rot(kr)) * scale;
                causal softmax whose denominator also holds exp(sink_h);  y = Wo concat(sum_j w_j v_h,j)
    delta:      q, k, v = silu(conv(W h));  q, k <- unit vectors per head, q *= dim^-1/2;
                beta = sigmoid(Wb h);  g = exp(-exp(A) softplus(Wa h + dt));
                S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q;
                y = Wo( o / rms(o) * w * silu(Wg h) )
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np
import torch

_ST_DTYPES = {"F32": np.float32, "BF16": np.uint16, "F16": np.float16, "I32": np.int32, "I64": np.int64}


# --------------------------------------------------------------------------
# files
# --------------------------------------------------------------------------
def read_safetensors(path) -> dict[str, torch.Tensor]:
    """8-byte little-endian header length, a JSON header, raw tensors; floating tensors come back as float32."""
    raw = Path(path).read_bytes()
    (hlen,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + hlen].decode("utf-8"))
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        arr = np.frombuffer(raw[8 + hlen + lo:8 + hlen + hi], dtype=_ST_DTYPES[info["dtype"]]).reshape(info["shape"])
        if info["dtype"] == "BF16":
            out[name] = torch.from_numpy((arr.astype(np.uint32).reshape(-1) << 16).view(np.float32).copy()).reshape(info["shape"])
        elif info["dtype"] in ("F32", "F16"):
            out[name] = torch.from_numpy(arr.astype(np.float32))
        else:
            out[name] = torch.from_numpy(arr.copy())
    return out


def read_model_dir(model_dir):
    model_dir = Path(model_dir)
    return json.loads((model_dir / "config.json").read_text()), read_safetensors(model_dir / "model.safetensors")


# --------------------------------------------------------------------------
# small functions
# --------------------------------------------------------------------------
def rms_norm(x: torch.Tensor, w, eps: float) -> torch.Tensor:
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if w is None else y * w


def silu(z):
    return z / (1.0 + torch.exp(-z))


def sigmoid(z):
    return 1.0 / (1.0 + torch.exp(-z))


def softplus(z):
    return torch.where(z > 20.0, z, torch.log1p(torch.exp(torch.clamp(z, max=20.0))))


def xielu(z: torch.Tensor, p: float, q: float) -> torch.Tensor:
    ap = math.log1p(math.exp(p))
    an = 0.5 + math.log1p(math.exp(q))
    pos = ap * z * z + 0.5 * z
    neg = an * (torch.expm1(torch.clamp(z, max=0.0)) - z) + 0.5 * z
    return torch.where(z > 0, pos, neg)


def dense_ff(h, up, down, act) -> torch.Tensor:
    return xielu(h @ up.T, float(act[0]), float(act[1])) @ down.T


# --------------------------------------------------------------------------
# rotary positions with YaRN
# --------------------------------------------------------------------------
def yarn_frequencies(dims: int, base: float, scaling) -> tuple[list, float]:
    """Per pair i < dims/2 the angle per position, and the factor on cos and sin."""
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    if not scaling:
        return f, 1.0
    factor, orig = float(scaling["factor"]), float(scaling["original"])

    def turn_dim(t):
        return dims * math.log(orig / (2.0 * math.pi * t)) / (2.0 * math.log(base))

    lo = max(math.floor(turn_dim(float(scaling["fast"]))), 0)
    hi = min(math.ceil(turn_dim(float(scaling["slow"]))), dims - 1)
    out = []
    for i, fi in enumerate(f):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(fi / factor * ramp + fi * (1.0 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


def rotate_pairs(x: torch.Tensor, positions: torch.Tensor, freq, mscale: float, n_rot: int) -> torch.Tensor:
    """x [..., T, D]: dimensions (2i, 2i+1), i < n_rot/2, turn by position * freq[i]; the rest pass.  Angles are
    products in x's precision (float32 unless the caller works in float64)."""
    out = x.clone()
    f = torch.tensor(freq, dtype=torch.float64).to(x.dtype)
    ang = positions.to(x.dtype)[:, None] * f[None, :]
    c, s = torch.cos(ang) * mscale, torch.sin(ang) * mscale
    u, v = x[..., 0:n_rot:2], x[..., 1:n_rot:2]
    out[..., 0:n_rot:2] = u * c - v * s
    out[..., 1:n_rot:2] = v * c + u * s
    return out


# --------------------------------------------------------------------------
# mixers: h [T, width] -> [T, width]; `first` is the position of h[0]
# --------------------------------------------------------------------------
def lightning_mixer(h, w, m, eps):
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = silu(h @ w["q"].T).view(T, H, d)
    k = silu(h @ w["k"].T).view(T, H, d)
    v = silu(h @ w["v"].T).view(T, H, dv)
    lam = torch.tensor(m["decay"], dtype=h.dtype)
    S = torch.zeros(H, d, dv, dtype=h.dtype)
    o = torch.empty(T, H, dv, dtype=h.dtype)
    for t in range(T):
        S = lam[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    o = rms_norm(o.reshape(T, H * dv), w["norm"], eps) * sigmoid(h @ w["g"].T)
    return o @ w["o"].T


def latent_attention_mixer(h, w, m, eps):
    H, d, dr, dv, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    T = h.shape[0]
    rot = m["rot"]
    freq, mscale = yarn_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
    pos = torch.arange(T)
    q = (h @ w["q"].T).view(T, H, d + dr)
    q_plain, q_rot = q[..., :d], q[..., d:]
    ckr = h @ w["dkv"].T
    c = rms_norm(ckr[:, :r], w["dkv.norm"], eps)
    kr = ckr[:, r:]
    k = (c @ w["uk"].T).view(T, H, d)
    v = (c @ w["uv"].T).view(T, H, dv)
    q_rot = rotate_pairs(q_rot.transpose(0, 1), pos, freq, mscale, rot["dims"])         # [H, T, dr]
    kr = rotate_pairs(kr, pos, freq, mscale, rot["dims"])                                # [T, dr]
    s = (torch.einsum("thd,jhd->htj", q_plain, k) + torch.einsum("htd,jd->htj", q_rot, kr)) * m["scale"]
    s = s.masked_fill(pos[None, None, :] > pos[None, :, None], float("-inf"))
    sink = w["sink"].to(h.dtype)
    top = torch.maximum(s.max(-1).values, sink[:, None])
    e = torch.exp(s - top[..., None])
    p = e / (e.sum(-1) + torch.exp(sink[:, None] - top))[..., None]
    o = torch.einsum("htj,jhv->thv", p, v).reshape(T, H * dv)
    return o @ w["o"].T


def causal_conv(x, taps):
    """x [T, C], taps [C, K] with the last column on the current token; zeros before the start."""
    T, K = x.shape[0], taps.shape[1]
    pad = torch.cat([torch.zeros(K - 1, x.shape[1], dtype=x.dtype), x])
    return sum(pad[j:j + T] * taps[:, j] for j in range(K))


def delta_mixer(h, w, m, eps):
    H, Hk, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = silu(causal_conv(h @ w["q"].T, w["q.conv"])).view(T, Hk, d)
    k = silu(causal_conv(h @ w["k"].T, w["k.conv"])).view(T, Hk, d)
    v = silu(causal_conv(h @ w["v"].T, w["v.conv"])).view(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    rep = H // Hk
    q, k = q.repeat_interleave(rep, dim=1), k.repeat_interleave(rep, dim=1)
    beta = sigmoid(h @ w["b"].T)                                                        # [T, H]
    g = torch.exp(-torch.exp(w["A_log"]) * softplus(h @ w["a"].T + w["dt_bias"]))       # [T, H]
    S = torch.zeros(H, d, dv, dtype=h.dtype)
    o = torch.empty(T, H, dv, dtype=h.dtype)
    for t in range(T):
        S = g[t][:, None, None] * S
        u = beta[t][:, None] * (v[t] - torch.einsum("hdv,hd->hv", S, k[t]))
        S = S + k[t][:, :, None] * u[:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    o = rms_norm(o, w["norm"], eps) * silu(h @ w["g"].T).view(T, H, dv)
    return o.reshape(T, H * dv) @ w["o"].T


MIXERS = {"lightning": lightning_mixer, "latent_attention": latent_attention_mixer, "delta": delta_mixer}


# --------------------------------------------------------------------------
# the model
# --------------------------------------------------------------------------
def layer_weights(weights, i: int, dtype) -> dict:
    p = f"l{i}."
    return {n[len(p):]: t.to(dtype) if t.is_floating_point() else t for n, t in weights.items() if n.startswith(p)}


def layer_step(x, lw, spec, eps):
    mw = {n[4:]: t for n, t in lw.items() if n.startswith("mix.")}
    y = MIXERS[spec["type"]](x, mw, spec["mixer"], eps)
    y = y * sigmoid(x @ lw["rg1"].T + lw["rg1.b"])
    x = x + rms_norm(y, lw["norm1"], eps)
    if spec.get("mlp") is not None:
        y = dense_ff(x, lw["mlp.up"], lw["mlp.down"], lw["mlp.act"])
        y = y * sigmoid(x @ lw["rg2"].T + lw["rg2.b"])
        x = x + rms_norm(y, lw["norm2"], eps)
    return x


def forward(cfg: dict, weights: dict, tokens, dtype=torch.float32, layers_out: list | None = None) -> torch.Tensor:
    """Logits [T, vocab] for one sequence from position 0; `layers_out` collects the stream after each layer."""
    eps = cfg["norm"]["eps"]
    x = weights["embed"].to(dtype)[torch.as_tensor(tokens, dtype=torch.long)]
    for i, spec in enumerate(cfg["layers"]):
        x = layer_step(x, layer_weights(weights, spec.get("weights_of", i), dtype), spec, eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    return rms_norm(x, weights["final.norm"].to(dtype), eps) @ weights["head"].to(dtype).T
