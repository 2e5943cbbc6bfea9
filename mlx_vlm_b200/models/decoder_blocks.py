"""Decoder mechanisms that a design picks by name in its configuration, each with its sizes and constants as
parameters, its packed weight layout and its launch sequence over the layer ops (layer_ops.py):

  mixers         MIXERS["latent_attention"]  -> LatentAttention
  feed-forwards  FEEDFORWARDS["moe"]         -> ExpertMixture
  layer          PostNormLayer: x += norm(mixer(x)); x += norm(ff(x)), weights of the norms stored around zero

A block declares `manifest(prefix)` (packed name, shape) and `pack(prefix, checkpoint tensors, arena)`; the model
packs all blocks into ONE device arena (the layout the other models of this package use).  `forward(ctx, x)`
enqueues the block's kernels; `ctx` carries the per-token slot / position arrays of the step and the cache pool,
so a prompt, a portion of a prompt, a decoded token and a batch of unequal requests are the same code.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch

from .._native import B200Error as _B200Error
from .layer_ops import EPI_RELU2, LayerOps


@dataclass
class StepCtx:
    ops: LayerOps
    slot: torch.Tensor            # (T,) int32 device: cache slot of every token of the step
    pos: torch.Tensor             # (T,) int32 device: position of every token in its sequence
    pool: object                  # LatentPool
    eps: float
    segments: Optional[List] = None   # host view of the step: (first token, tokens, slot, first position) per request
    _rope: Dict = field(default_factory=dict)

    def rope(self, base: float, dims: int) -> torch.Tensor:
        key = (float(base), int(dims))
        if key not in self._rope:
            self._rope[key] = self.ops.rope_table(self.pos, base, dims)
        return self._rope[key]


class LatentAttention:
    """Attention whose keys and values are expanded from one cached latent row per token.

    q = W_uq rmsnorm(W_dq h);  [c | r] = W_dkv h, c rms-normed, r rotated: the cache row of the token;
    per head  k = [W_uk c | r],  v = W_uv c;  softmax(scale * q.k) over the causal prefix;  W_o on the heads.
    `kv_from = j`: no W_dkv, the rows that layer j cached are read instead (same rank and rotation).
    The rotation is rotate-half on the first `rot_dims` of the rotated part, frequency base `rot_base`."""

    def __init__(self, index: int, cfg: dict, width: int):
        self.index, self.W = index, width
        self.H, self.dim, self.rot_dim, self.vdim = cfg["heads"], cfg["dim"], cfg["rot_dim"], cfg["vdim"]
        self.kv_rank, self.q_rank, self.scale = cfg["kv_rank"], cfg["q_rank"], float(cfg["scale"])
        rot = cfg.get("rot") or {}
        self.rot_base, self.rot_dims = float(rot.get("base", 10000.0)), int(rot.get("dims", self.rot_dim))
        self.kv_from: Optional[int] = cfg.get("kv_from")
        self.cache_index = -1     # set by the model: which caching layer of the pool this mixer reads (and writes)
        self.w: Dict[str, torch.Tensor] = {}

    @property
    def own_kv(self) -> bool:
        return self.kv_from is None

    @property
    def row_dim(self) -> int:
        return self.kv_rank + self.rot_dim

    def manifest(self, p: str):
        n_down = self.q_rank + (self.row_dim if self.own_kv else 0)
        out = [(p + "down", (n_down, self.W)), (p + "dq.norm", (self.q_rank,)),
               (p + "uq", (self.H * (self.dim + self.rot_dim), self.q_rank)),
               (p + "ukT", (self.H, self.kv_rank, self.dim)), (p + "uv", (self.H * self.vdim, self.kv_rank)),
               (p + "o", (self.W, self.H * self.vdim))]
        if self.own_kv:
            out.append((p + "dkv.norm", (self.kv_rank,)))
        return out

    def pack(self, p: str, ck: Dict[str, torch.Tensor], view):
        """ck: checkpoint tensors '<p>dq', '<p>dq.norm', '<p>uq', '<p>dkv', '<p>dkv.norm', '<p>uk', '<p>uv', '<p>o'"""
        down = view(p + "down")
        down[:self.q_rank].copy_(ck[p + "dq"])
        if self.own_kv:
            down[self.q_rank:].copy_(ck[p + "dkv"])          # one product for both down-projections
            view(p + "dkv.norm").copy_(ck[p + "dkv.norm"])
        for n in ("dq.norm", "uq", "uv", "o"):
            view(p + n).copy_(ck[p + n])
        # the key up-projection per head, transposed: it is applied to the QUERY (absorbed form)
        view(p + "ukT").copy_(ck[p + "uk"].view(self.H, self.dim, self.kv_rank).transpose(1, 2))
        self.bind(p, view)

    def bind(self, p: str, view):
        self.w = {n[len(p):]: view(n) for n, _ in self.manifest(p)}

    def forward(self, ctx: StepCtx, x: torch.Tensor) -> torch.Tensor:
        ops, w, T = ctx.ops, self.w, x.shape[0]
        H, dn, dr, r, dv = self.H, self.dim, self.rot_dim, self.kv_rank, self.vdim
        Dl = r + dr
        D = ops.linear(x, w["down"])
        cache_layer = ctx.pool.buf[self.cache_index][..., :Dl]    # a pool row may be wider than this layer's
        cs = ctx.rope(self.rot_base, self.rot_dims)
        cq = ops.empty((T, self.q_rank))
        ops.latent_post(D, w["dq.norm"], w.get("dkv.norm"), ctx.eps, cq, cache_layer if self.own_kv else None,
                        ctx.slot, ctx.pos, cs, self.q_rank, r, dr, self.rot_dims)
        q = ops.linear(cq, w["uq"])
        qa = ops.empty((T, H * Dl))
        heads_tc = ops.tc_ok(T, dn, dn + dr, r) and dn % 64 == 0 and r % 64 == 0 and Dl % 4 == 0 and dv % 4 == 0
        if heads_tc:     # a prompt: the heads' products as ONE tcgen05 launch (inner sizes are whole k-blocks)
            try:
                qb = ops.to_bf16(q, H * (dn + dr))
                ops.tc_gemm_heads(qb, w["ukT"], qa, H=H, N_=r, K=dn, x_cols=qb.shape[1], x_group_cols=dn + dr,
                                  c_group_cols=Dl)
            except _B200Error as e:
                ops.tc_refused(e)
                heads_tc = False
        if not heads_tc:
            ops.gemm(q, w["ukT"], qa, M=T, N_=r, K=dn, xb=dn + dr, ldw=dn, wb=r * dn, yb=Dl, batch=H)
        ops.rope_q(q, qa, cs, H, dn, dr, self.rot_dims, r)
        ol = ops.empty((T, H * r))
        segs = ctx.segments or []
        done = False
        if any(ops.tc_ok(n, Dl, r, cache_layer.stride(1)) for _, n, _, _ in segs) and cache_layer.dtype == torch.bfloat16:
            try:
                for start, n, slot, p0 in segs:      # long portions on the tensor cores, the rest on the row kernel
                    sl = slice(start, start + n)
                    if ops.tc_ok(n, Dl, r, cache_layer.stride(1)):
                        self._attend_prompt(ops, qa[sl], cache_layer[slot], ctx.pos[sl], ol[sl], p0 + n)
                    else:
                        ops.latent_attention(qa[sl], cache_layer, ctx.slot[sl], ctx.pos[sl], ol[sl], H, r, self.scale)
                done = True
            except _B200Error as e:
                ops.tc_refused(e)
        if not done:
            ops.latent_attention(qa, cache_layer, ctx.slot, ctx.pos, ol, H, r, self.scale)
        att = ops.empty((T, H * dv))
        if heads_tc:
            try:
                ob = ops.to_bf16(ol, H * r)
                ops.tc_gemm_heads(ob, w["uv"], att, H=H, N_=dv, K=r, x_cols=ob.shape[1], x_group_cols=r, c_group_cols=dv)
            except _B200Error as e:
                ops.tc_refused(e)
                heads_tc = False
        if not heads_tc:
            ops.gemm(ol, w["uv"], att, M=T, N_=dv, K=r, xb=r, ldw=r, wb=dv * r, yb=dv, batch=H)
        return ops.linear(att, w["o"])


    def _attend_prompt(self, ops: LayerOps, qa, rows, pos, ol, S: int):
        """A portion of a prompt against the S cached rows of its slot as two tcgen05 products: the cache rows are
        the weight-major operand of the scores (absorbed queries x rows), the causal softmax runs in fp32 over the
        score rows, and the transposed latent columns are the operand of the weighted sum.  Queries are taken in
        chunks that bound the score buffer."""
        H, r, Dl = self.H, self.kv_rank, self.kv_rank + self.rot_dim
        n, Sp = qa.shape[0], (S + 63) // 64 * 64
        ct = ops.cache_transpose(rows, S, Sp, r)
        step = max(1, min(n, (1 << 27) // (H * Sp)))
        for a in range(0, n, step):
            m = min(step, n - a)
            qb = ops.to_bf16(qa[a:a + m].view(m * H, Dl), Dl)
            sc = ops.empty((m * H, S))
            ops.tc_gemm(qb, rows, sc, N_=S, K=Dl, ldw=rows.stride(0))
            P = ops.empty((m * H, Sp), torch.bfloat16)
            ops.masked_softmax_bf16(sc, pos[a:a + m], H, self.scale, P)
            ops.tc_gemm(P, ct, ol[a:a + m].view(m * H, r), N_=r, K=Sp)


class ExpertMixture:
    """`experts` small feed-forwards W_down relu(W_up h)^2 without biases; a token uses the `top` experts with the
    largest router logits (fp32, with a bias), weighted by the softmax over those logits only."""

    def __init__(self, index: int, cfg: dict, width: int):
        self.index, self.W = index, width
        self.E, self.top, self.ff = cfg["router"]["experts"], cfg["router"]["top"], cfg["expert"]["ff"]
        self.w: Dict[str, torch.Tensor] = {}

    def manifest(self, p: str):
        return [(p + "router", (self.E, self.W)), (p + "router.b", (self.E,)), (p + "up", (self.E, self.ff, self.W)),
                (p + "down", (self.E, self.W, self.ff))]

    def pack(self, p: str, ck: Dict[str, torch.Tensor], view):
        view(p + "router").copy_(ck[p + "router"])
        view(p + "router.b").copy_(ck[p + "router.b"])
        up, down = view(p + "up"), view(p + "down")
        for e in range(self.E):
            up[e].copy_(ck[p + f"e{e}.up"])
            down[e].copy_(ck[p + f"e{e}.down"])
        self.bind(p, view)

    def bind(self, p: str, view):
        self.w = {n[len(p):]: view(n) for n, _ in self.manifest(p)}

    def forward(self, ctx: StepCtx, x: torch.Tensor):
        """-> (rows (T * top, W) of the chosen experts' outputs, weights (T, top)): the layer's norm sums them"""
        ops, w, T = ctx.ops, self.w, x.shape[0]
        z = ops.linear(x, w["router"], bias=w["router.b"])
        idx, wgt = ops.router_topk(z, self.top)
        lists, count = ops.moe_group(idx, self.E)
        if ops.tc_ok(T, self.W, self.ff):
            try:
                return self._experts_prompt(ops, x, lists, count), wgt
            except _B200Error as e:
                ops.tc_refused(e)
        hid = ops.empty((T * self.top, self.ff))
        ops.gemm(x, w["up"], hid, M=T, N_=self.ff, K=self.W, wb=self.ff * self.W, batch=self.E, lists=lists,
                 count=count, x_div=self.top, epi=EPI_RELU2, compact=min(self.E, T * self.top))
        out = ops.empty((T * self.top, self.W))
        ops.gemm(hid, w["down"], out, M=T, N_=self.W, K=self.ff, wb=self.W * self.ff, batch=self.E, lists=lists,
                 count=count, x_div=1, compact=min(self.E, T * self.top))
        return out, wgt


    def _experts_prompt(self, ops: LayerOps, x, lists, count):
        """A prompt step on the tensor cores, without the host knowing how the tokens spread over the experts: the
        (token, choice) entries are sorted by expert into segments padded to whole token tiles, with the expert of
        every tile in a device table; ONE launch gathers and rounds all input rows in that order, ONE grouped tcgen05
        launch per projection multiplies every tile by its expert's weights (empty tiles leave at once), ONE launch
        applies relu^2 and rounds the hidden rows, ONE launch scatters the outputs back to entry order."""
        w, T = self.w, x.shape[0]
        n_all = T * self.top
        order, group = ops.moe_tiles(lists, count, n_all)
        n_rows = order.shape[0]
        xs = ops.to_bf16(x, self.W, rows=n_rows, row_map=order, div=self.top)
        hs = ops.empty((n_rows, self.ff))
        ops.tc_gemm_grouped(xs, w["up"], hs, group, N_=self.ff, K=self.W, n_groups=self.E)
        hb = ops.to_bf16(hs, self.ff, relu2=True)
        ys = ops.empty((n_rows, self.W))
        ops.tc_gemm_grouped(hb, w["down"], ys, group, N_=self.W, K=self.ff, n_groups=self.E)
        out = ops.empty((n_all, self.W))
        ops.rows_scatter(ys, order, out, n_rows)
        return out


MIXERS = {"latent_attention": LatentAttention}
FEEDFORWARDS = {"moe": ExpertMixture}


class PostNormLayer:
    """x <- x + N1(mixer(x)); x <- x + N2(ff(x)), N = RMS norm with weight (1 + w); the sublayers read x itself."""

    def __init__(self, index: int, cfg: dict, width: int):
        self.index, self.W = index, width
        if cfg["type"] not in MIXERS:
            raise ValueError(f"layer {index}: unknown mixer type {cfg['type']!r} (have {sorted(MIXERS)})")
        self.mixer = MIXERS[cfg["type"]](index, cfg["mixer"], width)
        f = cfg.get("mlp")
        if f is not None and f.get("kind") not in FEEDFORWARDS:
            raise ValueError(f"layer {index}: unknown feed-forward kind {f.get('kind')!r} (have {sorted(FEEDFORWARDS)})")
        self.ff = None if f is None else FEEDFORWARDS[f["kind"]](index, f, width)
        self.w: Dict[str, torch.Tensor] = {}

    def manifest(self, p: str):
        out = [(p + "norm1", (self.W,))] + self.mixer.manifest(p + "mix.")
        if self.ff is not None:
            out += [(p + "norm2", (self.W,))] + self.ff.manifest(p + "mlp.")
        return out

    def pack(self, p: str, ck, view):
        view(p + "norm1").copy_(ck[p + "norm1"])
        self.mixer.pack(p + "mix.", ck, view)
        if self.ff is not None:
            view(p + "norm2").copy_(ck[p + "norm2"])
            self.ff.pack(p + "mlp.", ck, view)
        self.bind(p, view)

    def bind(self, p: str, view):
        """point the blocks at their views of the arena (after packing a checkpoint or filling the arena directly)"""
        self.w["norm1"] = view(p + "norm1")
        self.mixer.bind(p + "mix.", view)
        if self.ff is not None:
            self.w["norm2"] = view(p + "norm2")
            self.ff.bind(p + "mlp.", view)

    def forward(self, ctx: StepCtx, x: torch.Tensor):
        ops = ctx.ops
        y = self.mixer.forward(ctx, x)
        ops.norm_rows(y, self.w["norm1"], ctx.eps, x, w_offset=1.0, add=True)
        if self.ff is not None:
            rows, wgt = self.ff.forward(ctx, x)
            ops.norm_rows(rows, self.w["norm2"], ctx.eps, x, w_offset=1.0, add=True, combine=wgt, top=self.ff.top)


def assign_cache_layers(layers: List[PostNormLayer]) -> int:
    """number the layers that cache rows of their own; a borrowing layer gets its source's number"""
    n = 0
    for L in layers:
        if L.mixer.own_kv:
            L.mixer.cache_index = n
            n += 1
    for L in layers:
        m = L.mixer
        if not m.own_kv:
            if not 0 <= m.kv_from < m.index:
                raise ValueError(f"layer {m.index} borrows the latent of layer {m.kv_from}, which does not run before it")
            src = layers[m.kv_from].mixer
            if not src.own_kv or (src.kv_rank, src.rot_dim, src.rot_base, src.rot_dims) != \
                    (m.kv_rank, m.rot_dim, m.rot_base, m.rot_dims):
                raise ValueError(f"layer {m.index} borrows the latent of layer {m.kv_from}, which does not fit")
            m.cache_index = src.cache_index
    return n
