"""Plain, slow restatement of the Zogulorn decoder, used only by the tests.

Whole sequences, no cache, token-by-token loops for the recurrence, one
function per mechanism, torch on the CPU in float32 (or float64 when asked).
It shares no code with the package under test (the file reader is the other
plain model's).

The design in this file's notation (x is the float32 residual stream):

    x0          = E[token] * embedding.scale
    layer:      x += s1 * mixer(dyt1(x));   x += s2 * ff(dyt2(x))           s1, s2: a learned factor per channel
    dyt:        tanh(alpha z) * w + b                                       alpha one learned number; no statistics
    attend:     softmax_j( q_i . k_j * scale ) v_j  over j <= i with floor(i / c) = floor(j / c);
                query head h reads key/value head h // (H / G)
    left:       q, k rotated: pairs (2r, 2r+1), r < dims/2, turn by i * base^(-2r/dims); the other dimensions pass;
                y = Wo( attend * sigmoid(Wg h)_head )
    right:      q, k, v = silu(conv(W h));  q, k <- unit vectors per head, q *= dim^-1/2;  beta = sigmoid(Wb h);
                g = exp(-exp(A_head) softplus(Wa2 Wa1 h + dt))  per head and key channel;
                S <- diag(g) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q;
                y = Wo( o / rms(o) * w * sigmoid(Wg2 Wg1 h) )
    parallel:   a_left * left(h) + a_right * right(h)
    attention:  q, k, v = conv(W h), no activation; two maps per head over the same values:
                lam = exp(lq1 . lk1) - exp(lq2 . lk2) + diff;  o = attend_1 - lam attend_2;
                o <- o / rms(o) * (1 - diff);  y = Wo( o * sigmoid(Wg h)_head );
                with kv_from = j the keys and values are layer j's (after its convolutions)
    dense ff:   Wd( gelu_tanh(Wg h) * (Wu h) )
    moe ff:     z = Wr h;  the `top` largest z are chosen, their weights softmax over the chosen z alone;
                sum_e weight_e Wd_e relu(Wu_e h)^2
    logits      = head dyt_final(x)
"""
from __future__ import annotations

import math

import torch

from plain_fivitar import read_model_dir, read_safetensors  # noqa: F401  (file readers only)


# --------------------------------------------------------------------------
# small functions
# --------------------------------------------------------------------------
def sigmoid(z):
    return 1.0 / (1.0 + torch.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return torch.where(z > 20.0, z, torch.log1p(torch.exp(torch.clamp(z, max=20.0))))


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rms_div(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def dyt(x, w, b, alpha):
    return torch.tanh(alpha * x) * w + b


def causal_conv(x, taps):
    """x [T, C], taps [C, K] with the last column on the current token; zeros before the start."""
    T, K = x.shape[0], taps.shape[1]
    pad = torch.cat([torch.zeros(K - 1, x.shape[1], dtype=x.dtype), x])
    return sum(pad[j:j + T] * taps[:, j] for j in range(K))


def rotate_pairs(x, dims: int, base: float):
    """x [T, heads, D]: dimensions (2r, 2r+1), r < dims/2, of the token at position i turn by i * base^(-2r/dims)."""
    T = x.shape[0]
    out = x.clone()
    f = torch.tensor([base ** (-2.0 * r / dims) for r in range(dims // 2)], dtype=torch.float64).to(x.dtype)
    ang = torch.arange(T).to(x.dtype)[:, None] * f[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def chunk_mask(T: int, size: int):
    """[T, T] True where query i may see key j."""
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    return (j <= i) & (i // size == j // size)


def attend(q, k, v, scale: float, seen):
    """q [T, H, d], k [T, G, d], v [T, G, dv] -> [T, H, dv]; softmax over the keys `seen` [T, T] allows."""
    H, G = q.shape[1], k.shape[1]
    k, v = k.repeat_interleave(H // G, dim=1), v.repeat_interleave(H // G, dim=1)
    s = torch.einsum("ihd,jhd->hij", q, k) * scale
    s = s.masked_fill(~seen[None], float("-inf"))
    p = torch.softmax(s, dim=-1)
    return torch.einsum("hij,jhv->ihv", p, v)


# --------------------------------------------------------------------------
# mixers: h [T, width] -> [T, width]; a sequence from position 0
# --------------------------------------------------------------------------
def rotary_attention(h, w, m):
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = rotate_pairs((h @ w["q"].T).view(T, H, d), m["rot"]["dims"], m["rot"]["base"])
    k = rotate_pairs((h @ w["k"].T).view(T, G, d), m["rot"]["dims"], m["rot"]["base"])
    v = (h @ w["v"].T).view(T, G, dv)
    o = attend(q, k, v, m["scale"], chunk_mask(T, m["mask"]["size"]))
    o = o * sigmoid(h @ w["g"].T)[:, :, None]
    return o.reshape(T, H * dv) @ w["o"].T


def delta_rule(q, k, v, beta, g):
    """q, k [T, H, d], v [T, H, dv], beta [T, H], g [T, H, d] -> o [T, H, dv]; the state starts at zero."""
    T, H, d = q.shape
    S = torch.zeros(H, d, v.shape[2], dtype=q.dtype)
    o = torch.empty_like(v)
    for t in range(T):
        S = g[t][:, :, None] * S
        u = beta[t][:, None] * (v[t] - torch.einsum("hdv,hd->hv", S, k[t]))
        S = S + k[t][:, :, None] * u[:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    return o


def gated_delta(h, w, m, eps):
    H, Hk, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = silu(causal_conv(h @ w["q"].T, w["q.conv"])).view(T, Hk, d)
    k = silu(causal_conv(h @ w["k"].T, w["k.conv"])).view(T, Hk, d)
    v = silu(causal_conv(h @ w["v"].T, w["v.conv"])).view(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    q, k = q.repeat_interleave(H // Hk, dim=1), k.repeat_interleave(H // Hk, dim=1)
    beta = sigmoid(h @ w["b"].T)
    a = ((h @ w["a1"].T) @ w["a2"].T + w["dt_bias"]).view(T, H, d)
    g = torch.exp(-torch.exp(w["A_log"])[None, :, None] * softplus(a))
    o = delta_rule(q, k, v, beta, g)
    gate = sigmoid((h @ w["g1"].T) @ w["g2"].T).view(T, H, dv)
    o = rms_div(o, eps) * w["norm"] * gate
    return o.reshape(T, H * dv) @ w["o"].T


def parallel_mixer(h, w, m, eps, shared=None, index=None):
    sub = lambda side: {n[len(side) + 1:]: t for n, t in w.items() if n.startswith(side + ".")}
    return m["left_scale"] * rotary_attention(h, sub("left"), m["left"]) + \
        m["right_scale"] * gated_delta(h, sub("right"), m["right"], eps)


def differential_attention(h, w, m, eps, shared, index):
    """`shared` {layer: (k, v)} holds the keys and values (after their convolutions) of the layers run so far."""
    H, G, d, dv, diff = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["diff"]
    T = h.shape[0]
    q = causal_conv(h @ w["q"].T, w["q.conv"]).view(T, H, 2, d)
    if m.get("kv_from") is not None:
        k, v = shared[m["kv_from"]]
    else:
        k = causal_conv(h @ w["k"].T, w["k.conv"]).view(T, G, 2, d)
        v = causal_conv(h @ w["v"].T, w["v.conv"]).view(T, G, dv)
    shared[index] = (k, v)
    seen = chunk_mask(T, m["mask"]["size"])
    a1 = attend(q[:, :, 0], k[:, :, 0], v, m["scale"], seen)
    a2 = attend(q[:, :, 1], k[:, :, 1], v, m["scale"], seen)
    lam = torch.exp((w["lq1"] * w["lk1"]).sum()) - torch.exp((w["lq2"] * w["lk2"]).sum()) + diff
    o = rms_div(a1 - lam * a2, eps) * (1.0 - diff)
    o = o * sigmoid(h @ w["g"].T)[:, :, None]
    return o.reshape(T, H * dv) @ w["o"].T


# --------------------------------------------------------------------------
# feed-forwards
# --------------------------------------------------------------------------
def dense_ff(h, w):
    return (gelu_tanh(h @ w["gate"].T) * (h @ w["up"].T)) @ w["down"].T


def route(z, top: int):
    """z [T, E] -> (chosen experts [T, top], weights [T, top]): softmax over the chosen logits alone."""
    val, idx = torch.topk(z, top, dim=-1)
    return idx, torch.softmax(val, dim=-1)


def moe_ff(h, w, mlp):
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    idx, wt = route(h @ w["router"].T, top)
    out = torch.zeros_like(h)
    for e in range(E):
        y = (torch.relu(h @ w[f"e{e}.up"].T) ** 2) @ w[f"e{e}.down"].T
        out = out + y * (wt * (idx == e)).sum(-1, keepdim=True)
    return out


# --------------------------------------------------------------------------
# the model
# --------------------------------------------------------------------------
MIXERS = {"parallel": parallel_mixer, "attention": differential_attention}


def under(weights: dict, prefix: str, dtype) -> dict:
    return {n[len(prefix):]: (t.to(dtype) if t.is_floating_point() else t) for n, t in weights.items()
            if n.startswith(prefix)}


def norm_of(lw: dict, name: str):
    return lambda x: dyt(x, lw[name], lw[name + ".b"], lw[name + ".alpha"])


def forward(cfg: dict, weights: dict, tokens, dtype=torch.float32, layers_out: list | None = None) -> torch.Tensor:
    """Logits [T, vocab] for one sequence from position 0; `layers_out` collects the stream after each layer."""
    eps = cfg["norm"]["eps"]
    x = weights["embed"].to(dtype)[torch.as_tensor(tokens, dtype=torch.long)] * cfg["embedding"]["scale"]
    shared: dict = {}
    for i, spec in enumerate(cfg["layers"]):
        lw = under(weights, f"l{i}.", dtype)
        h = norm_of(lw, "norm1")(x)
        x = x + lw["ls1"] * MIXERS[spec["type"]](h, under(lw, "mix.", dtype), spec["mixer"], eps, shared, i)
        if spec.get("mlp") is not None:
            h = norm_of(lw, "norm2")(x)
            mw = under(lw, "mlp.", dtype)
            y = dense_ff(h, mw) if spec["mlp"]["kind"] == "dense" else moe_ff(h, mw, spec["mlp"])
            x = x + lw["ls2"] * y
        if layers_out is not None:
            layers_out.append(x.clone())
    fw = under(weights, "final.", dtype)
    return norm_of(fw, "norm")(x) @ weights["head"].to(dtype).T
