"""ORACLE — TEST INFRASTRUCTURE ONLY. Not imported by the product path.

Plain, slow restatement of the Sonulorn decoder, one function per mechanism, written from the design's
equations with torch on the CPU.  It shares no code with mlx_vlm_b200/: no cache, no state objects, no
batching; every call recomputes the whole sequence token by token where the design is recurrent.

Notation: x (T, W) residual stream, e the scaled embedding rows.  A layer is pre-norm with both sublayers
reading the same normed input:  n = N(x);  x <- x + mixer(n) + ff(n),  N(y) = y / sqrt(mean(y^2) + eps) * w.
Mixers: softmax attention with a per-head sink logit (causal or block-local keys, grouped key/value heads,
rotate-half rotary on the leading dims, optional short convolutions, a sigmoid gate per element or per head),
a gated delta rule, a decayed outer-product state ("lightning"), and the weighted sum of an attention and a
delta rule that read the same input.  A span of layers may repeat; before every repetition the stream is
re-mixed with e through a (W, 2W) matrix and a per-repetition vector is added.

Weights: dict name -> tensor with the checkpoint's names ('embed', 'l<i>.norm1', 'l<i>.mix...', 'final.norm',
'head', 'loop.in', 'loop.step').
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch
import torch.nn.functional as F


# ------------------------------------------------------------------------------------------------ pieces
def rms(y: torch.Tensor, eps: float) -> torch.Tensor:
    return y / torch.sqrt((y * y).mean(-1, keepdim=True) + eps)


def norm(y, w, eps):
    return rms(y, eps) * w


def rotate_half(v: torch.Tensor, pos: torch.Tensor, base: float, dims: int) -> torch.Tensor:
    """v (T, heads, D): the first `dims` of D turn, element i with i + dims/2, angle pos * base^(-2i/dims)"""
    half = dims // 2
    if half == 0:
        return v.clone()
    f = base ** (-2.0 * torch.arange(half, dtype=torch.float64) / dims)
    a = pos.to(torch.float64)[:, None] * f[None, :]
    cos, sin = torch.cos(a).to(v.dtype)[:, None, :], torch.sin(a).to(v.dtype)[:, None, :]
    lo, hi = v[..., :half], v[..., half:dims]
    out = v.clone()
    out[..., :half] = lo * cos - hi * sin
    out[..., half:dims] = hi * cos + lo * sin
    return out


def short_conv(u: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """u (T, C), w (C, taps): y[t] = sum_j w[:, j] u[t - (taps - 1) + j], nothing before the first token"""
    T, taps = u.shape[0], w.shape[1]
    y = torch.zeros_like(u)
    for j in range(taps):
        back = taps - 1 - j
        if back < T:
            y[back:] += w[:, j] * u[:T - back]
    return y


def visible(T: int, block: Optional[int]) -> torch.Tensor:
    """(T, T) bool: query i sees key j <= i, and with `block` only keys of its own block of positions"""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    ok = j <= i
    if block:
        ok &= (i // block) == (j // block)
    return ok


def sink_softmax_attention(q, k, v, scale, sink, block=None):
    """q (T, H, d), k (T, G, d), v (T, G, dv), sink (H,): softmax over the visible keys and one extra logit per
    head that has no key and no value"""
    T, H, _ = q.shape
    G = k.shape[1]
    rep = H // G
    ok = visible(T, block)
    out = torch.zeros(T, H, v.shape[-1], dtype=q.dtype)
    for h in range(H):
        g = h // rep
        s = (q[:, h] @ k[:, g].T) * scale
        s = s.masked_fill(~ok, float("-inf"))
        s = torch.cat([s, sink[h].expand(T, 1).to(s.dtype)], dim=1)
        p = torch.softmax(s, dim=-1)[:, :T]
        out[:, h] = p @ v[:, g]
    return out


def attention_mixer(n, W, p, m, pos, gate="element"):
    """p: tensor prefix ending in '.', m: the mixer's sizes"""
    T = n.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q, k, v = n @ W[p + "q"].T, n @ W[p + "k"].T, n @ W[p + "v"].T
    if m.get("conv"):
        q, k, v = (short_conv(t, W[p + name + ".conv"]) for t, name in ((q, "q"), (k, "k"), (v, "v")))
    q, k, v = q.view(T, H, d), k.view(T, G, d), v.view(T, G, dv)
    rot = m.get("rot") or {}
    if rot.get("dims"):
        q = rotate_half(q, pos, rot["base"], rot["dims"])
        k = rotate_half(k, pos, rot["base"], rot["dims"])
    block = (m.get("mask") or {}).get("size")
    o = sink_softmax_attention(q, k, v, m["scale"], W[p + "sink"], block)
    z = torch.sigmoid(n @ W[p + "g"].T)
    o = o * (z.view(T, H, dv) if gate == "element" else z.view(T, H, 1))
    return o.reshape(T, H * dv) @ W[p + "o"].T


def delta_rule(q, k, v, decay, beta):
    """q, k (T, H, d), v (T, H, dv), decay, beta (T, H): per head a (d, dv) state S; per token
    S <- decay S;  S <- S + k (beta (v - S^T k))^T;  o = S^T q"""
    T, H, d = q.shape
    dv = v.shape[-1]
    S = torch.zeros(H, d, dv, dtype=q.dtype)
    out = torch.zeros(T, H, dv, dtype=q.dtype)
    for t in range(T):
        S = S * decay[t][:, None, None]
        seen = torch.einsum("hdv,hd->hv", S, k[t])
        u = beta[t][:, None] * (v[t] - seen)
        S = S + torch.einsum("hd,hv->hdv", k[t], u)
        out[t] = torch.einsum("hdv,hd->hv", S, q[t])
    return out


def delta_mixer(n, W, p, m, eps):
    T = n.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    rep = H // G
    q = F.silu(short_conv(n @ W[p + "q"].T, W[p + "q.conv"])).view(T, G, d)
    k = F.silu(short_conv(n @ W[p + "k"].T, W[p + "k.conv"])).view(T, G, d)
    v = F.silu(short_conv(n @ W[p + "v"].T, W[p + "v.conv"])).view(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    q, k = q.repeat_interleave(rep, dim=1), k.repeat_interleave(rep, dim=1)
    beta = torch.sigmoid(n @ W[p + "b"].T)
    decay = torch.exp(-torch.exp(W[p + "A_log"]) * F.softplus(n @ W[p + "a"].T + W[p + "dt_bias"]))
    o = delta_rule(q, k, v, decay, beta)
    o = rms(o, eps) * W[p + "norm"] * F.silu(n @ W[p + "g"].T).view(T, H, dv)
    return o.reshape(T, H * dv) @ W[p + "o"].T


def decayed_state(q, k, v, decay):
    """q, k (T, H, d), v (T, H, dv), decay (H,): S <- decay S + k v^T;  o = S^T q"""
    T, H, d = q.shape
    S = torch.zeros(H, d, v.shape[-1], dtype=q.dtype)
    out = torch.zeros(T, H, v.shape[-1], dtype=q.dtype)
    for t in range(T):
        S = S * decay[:, None, None] + torch.einsum("hd,hv->hdv", k[t], v[t])
        out[t] = torch.einsum("hdv,hd->hv", S, q[t])
    return out


def lightning_mixer(n, W, p, m, eps):
    T = n.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = F.silu(n @ W[p + "q"].T).view(T, H, d)
    k = F.silu(n @ W[p + "k"].T).view(T, H, d)
    v = F.silu(n @ W[p + "v"].T).view(T, H, dv)
    o = decayed_state(q, k, v, torch.tensor(m["decay"], dtype=n.dtype)).reshape(T, H * dv)
    o = norm(o, W[p + "norm"], eps) * torch.sigmoid(n @ W[p + "g"].T)
    return o @ W[p + "o"].T


def side_by_side_mixer(n, W, p, m, eps, pos):
    left = attention_mixer(n, W, p + "left.", m["left"], pos, gate="head")
    right = delta_mixer(n, W, p + "right.", m["right"], eps)
    return m["left_scale"] * left + m["right_scale"] * right


def clamped_glu(n, W, p, f):
    lim = f["limit"]
    g = torch.clamp(n @ W[p + "gate"].T, max=lim)
    u = torch.clamp(n @ W[p + "up"].T, -lim, lim)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ W[p + "down"].T


def layer(x, W, i, L, eps, pos):
    p = f"l{i}."
    n = norm(x, W[p + "norm1"], eps)
    kind = L["type"]
    if kind == "attention":
        y = attention_mixer(n, W, p + "mix.", L["mixer"], pos, gate="element")
    elif kind == "parallel":
        y = side_by_side_mixer(n, W, p + "mix.", L["mixer"], eps, pos)
    elif kind == "lightning":
        y = lightning_mixer(n, W, p + "mix.", L["mixer"], eps)
    else:
        raise ValueError(kind)
    if L.get("mlp") is not None:
        y = y + clamped_glu(n, W, p + "mlp.", L["mlp"])
    return x + y


def layer_runs(cfg) -> List[tuple]:
    """(layer index, repetition or None, first of its repetition) in the order the layers run"""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None, False) for i in range(n)]
    a, b, times = loop["start"], loop["stop"], loop["times"]
    runs = [(i, None, False) for i in range(a)]
    for t in range(times):
        runs += [(i, t, i == a) for i in range(a, b)]
    return runs + [(i, None, False) for i in range(b, n)]


def forward(cfg, W: Dict[str, torch.Tensor], tokens, dtype=torch.float64, layers_out: Optional[list] = None):
    """logits (T, vocab) of every position of ONE sequence"""
    W = {k: v.to(dtype) for k, v in W.items()}
    ids = torch.as_tensor(tokens, dtype=torch.long)
    T = ids.shape[0]
    pos = torch.arange(T)
    eps = cfg["norm"]["eps"]
    e = W["embed"][ids] * cfg["embedding"]["scale"]
    x = e
    for i, t, first in layer_runs(cfg):
        if first:
            x = torch.cat([x, e], dim=-1) @ W["loop.in"].T + W["loop.step"][t]
        x = layer(x, W, i, cfg["layers"][i], eps, pos)
        if layers_out is not None:
            layers_out.append(x.clone())
    return norm(x, W["final.norm"], eps) @ W["head"].T


# ------------------------------------------------------------------------------------------------ weights
def tensor_shapes(cfg) -> Dict[str, tuple]:
    Wd, V = cfg["width"], cfg["vocab"]
    out = {"embed": (V, Wd), "final.norm": (Wd,), "head": (V, Wd)}
    if cfg.get("loop"):
        out["loop.in"] = (Wd, 2 * Wd)
        out["loop.step"] = (cfg["loop"]["times"], Wd)

    def attn(p, m, gate_rows):
        H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        out.update({p + "q": (H * d, Wd), p + "k": (G * d, Wd), p + "v": (G * dv, Wd), p + "sink": (H,),
                    p + "g": (gate_rows, Wd), p + "o": (Wd, H * dv)})
        if m.get("conv"):
            out.update({p + "q.conv": (H * d, m["conv"]), p + "k.conv": (G * d, m["conv"]),
                        p + "v.conv": (G * dv, m["conv"])})

    def delta(p, m):
        H, G, d, dv, c = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
        out.update({p + "q": (G * d, Wd), p + "k": (G * d, Wd), p + "v": (H * dv, Wd), p + "q.conv": (G * d, c),
                    p + "k.conv": (G * d, c), p + "v.conv": (H * dv, c), p + "b": (H, Wd), p + "a": (H, Wd),
                    p + "A_log": (H,), p + "dt_bias": (H,), p + "norm": (dv,), p + "g": (H * dv, Wd),
                    p + "o": (Wd, H * dv)})

    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        out[p + "norm1"] = (Wd,)
        if L["type"] == "attention":
            attn(p + "mix.", m, m["heads"] * m["vdim"])
        elif L["type"] == "parallel":
            attn(p + "mix.left.", m["left"], m["left"]["heads"])
            delta(p + "mix.right.", m["right"])
        elif L["type"] == "lightning":
            H, d, dv = m["heads"], m["dim"], m["vdim"]
            out.update({p + "mix.q": (H * d, Wd), p + "mix.k": (H * d, Wd), p + "mix.v": (H * dv, Wd),
                        p + "mix.g": (H * dv, Wd), p + "mix.o": (Wd, H * dv), p + "mix.norm": (H * dv,)})
        if L.get("mlp") is not None:
            ff = L["mlp"]["ff"]
            out.update({p + "mlp.gate": (ff, Wd), p + "mlp.up": (ff, Wd), p + "mlp.down": (Wd, ff)})
    return out


def random_weights(cfg, seed: int = 0, gain: float = 1.0) -> Dict[str, torch.Tensor]:
    """bf16-valued tensors: matrices N(0, gain / fan-in), norm weights around one, sinks / decays of order one"""
    g = torch.Generator().manual_seed(seed)
    W = {}
    for name, shape in tensor_shapes(cfg).items():
        last = name.rsplit(".", 1)[-1]
        if last in ("norm1", "norm") or name == "final.norm":
            t = 1.0 + 0.2 * torch.randn(shape, generator=g)
        elif last in ("sink", "dt_bias", "A_log"):
            t = torch.randn(shape, generator=g)
        elif last == "conv":
            t = torch.randn(shape, generator=g) * 0.6
        elif name == "embed":
            t = torch.randn(shape, generator=g) / cfg["embedding"]["scale"]
        elif name == "loop.step":
            t = torch.randn(shape, generator=g) * 0.3
        else:
            t = torch.randn(shape, generator=g) * (gain / math.sqrt(shape[-1]))
        W[name] = t.to(torch.bfloat16)
    return W
