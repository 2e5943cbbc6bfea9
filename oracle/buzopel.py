"""ORACLE — TEST INFRASTRUCTURE ONLY. Not imported by the product path.

Plain, slow restatement of the Buzopel decoder (a post-norm decoder whose mixer is a latent
attention and whose feed-forward is a mixture of small experts), one function per mechanism,
written from the design's equations with torch on the CPU.  It shares no code with
mlx_vlm_b200/: no cache, no batching, every call recomputes the whole sequence.

Notation: x (T, W) residual stream; per layer  x <- x + N1(mixer(x));  x <- x + N2(ff(x))
with N(y) = y / sqrt(mean(y^2) + eps) * (1 + w).

Weights are a dict name -> tensor with the checkpoint's names
('embed', 'l<i>.norm1', 'l<i>.mix.dq', ..., 'final.norm', 'head').
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def rms(y: torch.Tensor, eps: float) -> torch.Tensor:
    return y / torch.sqrt((y * y).mean(-1, keepdim=True) + eps)


def norm_offset(y, w, eps):
    """the layers' norm: weight stored around zero"""
    return rms(y, eps) * (1.0 + w)


def norm_plain(y, w, eps):
    """the latents' norm: plain weight"""
    return rms(y, eps) * w


def rotate_half(v: torch.Tensor, pos: torch.Tensor, base: float, dims: int) -> torch.Tensor:
    """v (..., T, D); the first `dims` of D are rotated: element i pairs with i + dims/2,
    angle = pos * base^(-2i/dims)."""
    half = dims // 2
    i = torch.arange(half, dtype=torch.float64)
    f = base ** (-2.0 * i / dims)
    a = pos.to(torch.float64)[:, None] * f[None, :]          # (T, half)
    cos, sin = torch.cos(a).to(v.dtype), torch.sin(a).to(v.dtype)
    u, w = v[..., :half], v[..., half:dims]
    out = v.clone()
    out[..., :half] = u * cos - w * sin
    out[..., half:dims] = w * cos + u * sin
    return out


def latent_kv(h, W, pre, m, eps, pos):
    """what a layer with its own W_dkv caches: (c (T, kv_rank), k_rot (T, rot_dim) rotated)"""
    r = m["kv_rank"]
    d = h @ W[pre + "dkv"].T
    c = norm_plain(d[:, :r], W[pre + "dkv.norm"], eps)
    k_rot = rotate_half(d[:, r:], pos, m["rot"]["base"], m["rot"]["dims"])
    return c, k_rot


def latent_attention(h, W, pre, m, eps, pos, kv):
    """h (T, W) -> (T, W).  kv = (c, k_rot) of this layer or of the layer it borrows from."""
    T = h.shape[0]
    H, dn, dr, dv = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    cq = norm_plain(h @ W[pre + "dq"].T, W[pre + "dq.norm"], eps)
    q = (cq @ W[pre + "uq"].T).view(T, H, dn + dr)
    q_n, q_r = q[..., :dn], q[..., dn:]
    q_r = rotate_half(q_r.transpose(0, 1), pos, m["rot"]["base"], m["rot"]["dims"]).transpose(0, 1)
    c, k_rot = kv
    k_n = (c @ W[pre + "uk"].T).view(T, H, dn)
    v = (c @ W[pre + "uv"].T).view(T, H, dv)
    s = torch.einsum("ihd,jhd->hij", q_n, k_n) + torch.einsum("ihd,jd->hij", q_r, k_rot)
    s = s * m["scale"]
    causal = torch.ones(T, T, dtype=torch.bool).tril()
    s = s.masked_fill(~causal, float("-inf"))
    p = torch.softmax(s, dim=-1)
    o = torch.einsum("hij,jhd->ihd", p, v).reshape(T, H * dv)
    return o @ W[pre + "o"].T


def router(h, Wr, b, top):
    """-> (indices (T, top), weights (T, top)): softmax over the chosen logits only"""
    z = h.float() @ Wr.float().T + b.float()
    val, idx = torch.topk(z, top, dim=-1)
    return idx, torch.softmax(val, dim=-1)


def expert(h, up, down):
    return torch.relu(h @ up.T).square() @ down.T


def moe(h, W, pre, f):
    E, top = f["router"]["experts"], f["router"]["top"]
    idx, wgt = router(h, W[pre + "router"], W[pre + "router.b"], top)
    out = torch.zeros_like(h)
    for e in range(E):
        hit = (idx == e)
        rows = hit.any(-1).nonzero().flatten()
        if rows.numel() == 0:
            continue
        y = expert(h[rows], W[pre + f"e{e}.up"], W[pre + f"e{e}.down"])
        out[rows] += y * (wgt[rows] * hit[rows]).sum(-1, keepdim=True).to(h.dtype)
    return out


def forward(config: dict, W: Dict[str, torch.Tensor], tokens: List[int], dtype=torch.float64,
            layers_out: Optional[list] = None) -> torch.Tensor:
    """logits (T, vocab) of one sequence, everything in `dtype`"""
    W = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in W.items()}
    eps = config["norm"]["eps"]
    ids = torch.as_tensor(tokens, dtype=torch.long)
    pos = torch.arange(len(tokens))
    x = W["embed"][ids] * config["embedding"]["scale"]
    kept = {}
    for i, L in enumerate(config["layers"]):
        pre, m = f"l{i}.mix.", L["mixer"]
        assert L["type"] == "latent_attention"
        if "kv_from" in m and m["kv_from"] is not None:
            kv = kept[m["kv_from"]]
        else:
            kv = kept[i] = latent_kv(x, W, pre, m, eps, pos)
        x = x + norm_offset(latent_attention(x, W, pre, m, eps, pos, kv), W[f"l{i}.norm1"], eps)
        if L.get("mlp") is not None:
            assert L["mlp"]["kind"] == "moe"
            x = x + norm_offset(moe(x, W, f"l{i}.mlp.", L["mlp"]), W[f"l{i}.norm2"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    y = norm_offset(x, W["final.norm"], eps) @ W["head"].T
    cap = config.get("logit_softcap")
    if cap:
        y = cap * torch.tanh(y / cap)
    return y


def random_weights(config: dict, seed: int = 0, scale: float = 1.0) -> Dict[str, torch.Tensor]:
    """bf16-valued random weights with the checkpoint's names and shapes"""
    g = torch.Generator().manual_seed(seed)
    Wd, V = config["width"], config["vocab"]

    def lin(o, i, s=1.0):
        return (torch.randn(o, i, generator=g) * (s * scale / math.sqrt(i))).bfloat16()

    def vec(n, s=0.1, mean=0.0):
        return (mean + torch.randn(n, generator=g) * s).bfloat16()

    W = {"embed": (torch.randn(V, Wd, generator=g) / config["embedding"]["scale"]).bfloat16(),
         "final.norm": vec(Wd), "head": lin(V, Wd)}
    for i, L in enumerate(config["layers"]):
        m, p = L["mixer"], f"l{i}."
        H, dn, dr, dv, r, qr = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
        W[p + "norm1"] = vec(Wd)
        W[p + "mix.dq"] = lin(qr, Wd)
        W[p + "mix.dq.norm"] = vec(qr, mean=1.0)
        W[p + "mix.uq"] = lin(H * (dn + dr), qr, 2.0)
        if m.get("kv_from") is None:
            W[p + "mix.dkv"] = lin(r + dr, Wd)
            W[p + "mix.dkv.norm"] = vec(r, mean=1.0)
        W[p + "mix.uk"] = lin(H * dn, r, 2.0)
        W[p + "mix.uv"] = lin(H * dv, r)
        W[p + "mix.o"] = lin(Wd, H * dv)
        f = L.get("mlp")
        if f is not None:
            W[p + "norm2"] = vec(Wd)
            E, ff = f["router"]["experts"], f["expert"]["ff"]
            W[p + "mlp.router"] = lin(E, Wd, 2.0)
            W[p + "mlp.router.b"] = vec(E, 0.5)
            for e in range(E):
                W[p + f"mlp.e{e}.up"] = lin(ff, Wd, 2.0)
                W[p + f"mlp.e{e}.down"] = lin(Wd, ff)
    return W
