"""Decoder mechanisms that a design picks by name in its configuration, each with its sizes and constants as
parameters, its packed weight layout and its launch sequence over the layer ops (layer_ops.py):

  mixers         MIXERS["latent_attention"]  -> LatentAttention
  feed-forwards  FEEDFORWARDS["moe"]         -> ExpertMixture
  layer          PostNormLayer: x += norm(mixer(x)); x += norm(ff(x)), weights of the norms stored around zero

and, for layers whose sublayers all read ONE normed input (so that all their input projections are one product and
all their output projections another), the parts of a `SharedInputLayer`:

  mixers         FUSED_MIXERS["attention"]  -> SinkAttention   (grouped heads, sink logit, block-local keys, gate)
                 FUSED_MIXERS["lightning"]  -> DecayedState    (outer-product state with a fixed decay per head)
                 FUSED_MIXERS["parallel"]   -> an attention and a GatedDeltaRule side by side, weighted
  feed-forwards  FUSED_FEEDFORWARDS["dense"] -> ClampedGLU
  layer          SharedInputLayer: n = norm(x); x += sum of the parts' outputs

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
    _seq: Optional[tuple] = None

    def seq_tables(self):
        """(first (T,), seqs (G, 2), G): the sequences of the step for the mixers that walk them in order; without a
        host view every token is a sequence of its own (a decode step)"""
        if self._seq is None:
            self._seq = self.ops.seq_tables(self.segments, self.pos.shape[0])
        return self._seq

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


# ----------------------------------------------------------------------------------------------------------------
# Parts of a layer whose sublayers share their input.  A part names the rows it adds to the layer's input projection
# (`in_names`, stacked in that order; `n_in` rows in all), the columns it adds to the output projection (`out_name`,
# `n_out`), its other tensors (`small`), what it keeps per request (`kv_dim` numbers per cached token, `state_floats`
# fp32 numbers per slot), and `forward(ctx, D, cat, kv_layer, state_off, out_scale)`: D (T, n_in) its columns of the
# projected rows (scratch: it may overwrite them), cat (T, n_out) its columns of the output projection's input.
class SinkAttention:
    """Softmax attention with `heads` query heads over `kv_heads` key/value heads (query head h reads key/value head
    h // (heads / kv_heads)), rotate-half rotary on the first `rot.dims` numbers of every query and key head, an
    optional short causal convolution on q, k, v before the rotation (`conv` taps), keys limited to the query's own
    block of `mask.size` positions (absent: all earlier positions), a learned logit per head that joins the softmax's
    denominator without a key or a value (`sink`), and a sigmoid gate on the heads' outputs computed from the layer's
    input: one number per output element (`gate="element"`) or per head (`gate="head"`)."""

    def __init__(self, index: int, cfg: dict, width: int, gate: str = "element"):
        self.index, self.W, self.gate = index, width, gate
        self.H, self.dim = int(cfg["heads"]), int(cfg["dim"])
        self.G, self.vdim = int(cfg.get("kv_heads", self.H)), int(cfg.get("vdim", self.dim))
        if self.H % self.G:
            raise ValueError(f"layer {index}: {self.H} query heads do not divide over {self.G} key/value heads")
        self.scale = float(cfg.get("scale", float(self.dim) ** -0.5))
        rot = cfg.get("rot") or {}
        self.rot_base, self.rot_dims = float(rot.get("base", 10000.0)), int(rot.get("dims", 0))
        self.chunk = int((cfg.get("mask") or {}).get("size", 0))
        self.window = int(cfg.get("window", 0))
        self.taps = int(cfg.get("conv") or 0)
        self.n_q, self.n_k, self.n_v = self.H * self.dim, self.G * self.dim, self.G * self.vdim
        self.n_gate = self.H * self.vdim if gate == "element" else self.H
        self.in_names, self.out_name = ["q", "k", "v", "g"], "o"
        self.n_in, self.n_out = self.n_q + self.n_k + self.n_v + self.n_gate, self.H * self.vdim
        self.kv_dim = self.n_k + self.n_v
        self.state_floats = max(self.taps - 1, 0) * (self.n_q + self.n_k + self.n_v)
        self.w: Dict[str, torch.Tensor] = {}

    def in_rows(self, name: str) -> int:
        return {"q": self.n_q, "k": self.n_k, "v": self.n_v, "g": self.n_gate}[name]

    def small(self):
        out = [("sink", (self.H,))]
        if self.taps:
            out.append(("conv", (self.n_q + self.n_k + self.n_v, self.taps)))
        return out

    def checkpoint_small(self):
        """packed name -> the checkpoint tensors it is stacked from"""
        out = {"sink": ["sink"]}
        if self.taps:
            out["conv"] = ["q.conv", "k.conv", "v.conv"]
        return out

    def forward(self, ctx: StepCtx, D, cat, kv_layer: int, state_off: int, out_scale: float = 1.0):
        ops, w, T = ctx.ops, self.w, D.shape[0]
        nq, nk, nv = self.n_q, self.n_k, self.n_v
        src = D
        if self.taps:
            src = ops.short_conv(D[:, :nq + nk + nv], w["conv"], ctx.pool.state[:, state_off:state_off + self.state_floats],
                                 ctx)
        q, k, v = src[:, :nq], src[:, nq:nq + nk], src[:, nq + nk:nq + nk + nv]
        rows = ctx.pool.buf[kv_layer][..., :self.kv_dim]
        ops.qkv_post(q, k, v, rows, ctx.slot, ctx.pos, ctx.rope(self.rot_base, self.rot_dims), self.H, self.G, self.dim,
                     self.vdim, self.rot_dims)
        o = ops.empty((T, self.n_out))
        segs = ctx.segments or []
        done = False
        if rows.dtype == torch.bfloat16 and not self.window and any(self._tc_portion(ops, n, rows) for _, n, _, _ in segs):
            try:
                for start, n, slot, p0 in segs:      # long portions on the tensor cores, the rest on the row kernel
                    sl = slice(start, start + n)
                    if self._tc_portion(ops, n, rows):
                        self._attend_prompt(ctx, q[sl], rows, slot, ctx.slot[sl], ctx.pos[sl], o[sl], p0, n)
                    else:
                        self._attend_rows(ctx, q[sl], rows, ctx.slot[sl], ctx.pos[sl], o[sl], prompt=True)
                done = True
            except _B200Error as e:
                ops.tc_refused(e)
        if not done:
            self._attend_rows(ctx, q, rows, ctx.slot, ctx.pos, o, prompt=ctx.segments is not None)
        ops.head_post(o, cat, dv=self.vdim, gate=D[:, nq + nk + nv:], gate_per_head=self.gate == "head", scale=out_scale)

    def _tc_portion(self, ops: LayerOps, n: int, rows) -> bool:
        return ops.tc_ok(n, self.dim, rows.stride(1)) and rows.stride(0) % 8 == 0

    def _attend_rows(self, ctx: StepCtx, q, rows, slot, pos, o, prompt: bool):
        """the row kernel: every query finds its keys by (slot, position); a step of few tokens (decoding) spreads the
        keys of a query over several blocks"""
        ctx.ops.sink_attention(q, rows, slot, pos, o, self.w["sink"], self.H, self.G, self.dim, self.vdim, self.scale,
                               chunk=self.chunk, window=self.window, n_split=1 if prompt and q.shape[0] > 16 else None)

    def _attend_prompt(self, ctx: StepCtx, q, all_rows, slot_index: int, slot, pos, o, p0: int, n: int):
        """A portion of a prompt (positions p0 .. p0 + n - 1 of one slot) as two tcgen05 products per key/value head:
        the cached key columns of that head are the weight-major operand of the scores of the query heads that share
        it, an fp32 softmax over the visible keys (with the sink logit in the denominator) writes bf16 probabilities,
        and the head's value columns, transposed, are the operand of the weighted sum.  With block-local keys the
        portion is taken block by block, each against the keys of its own block only.  Queries are taken in chunks
        that bound the score buffer; a block's share of fewer rows than a tile goes to the row kernel."""
        ops, H, G, d, dv = ctx.ops, self.H, self.G, self.dim, self.vdim
        rep, rows = H // G, all_rows[slot_index]
        if self.chunk:
            spans = [(max(p0, b * self.chunk), min(p0 + n, (b + 1) * self.chunk), b * self.chunk)
                     for b in range(p0 // self.chunk, (p0 + n - 1) // self.chunk + 1)]
        else:
            spans = [(p0, p0 + n, 0)]
        for qa, qb, key0 in spans:
            m, a0 = qb - qa, qa - p0
            if not ops.tc_ok(m, d):
                sl = slice(a0, a0 + m)
                self._attend_rows(ctx, q[sl], all_rows, slot[sl], pos[sl], o[sl], prompt=True)
                continue
            S = qb - key0
            Sp = (S + 63) // 64 * 64
            step = max(1, min(m, (1 << 27) // (rep * Sp)))
            for g in range(G):
                keys = rows[key0:key0 + S, g * d:(g + 1) * d]
                vt = ops.cache_transpose(rows[key0:, G * d + g * dv:], S, Sp, dv)
                for a in range(a0, a0 + m, step):
                    mm = min(step, a0 + m - a)
                    qb16 = ops.heads_to_bf16(q[a:a + mm, g * rep * d:], rep, d)
                    sc = ops.empty((mm * rep, S))
                    ops.tc_gemm(qb16, keys, sc, N_=S, K=d, ldw=rows.stride(0))
                    P = ops.empty((mm * rep, Sp), torch.bfloat16)
                    ops.sink_softmax_bf16(sc, pos[a:a + mm], rep, self.w["sink"][g * rep:], self.scale, self.chunk, 0, key0, P)
                    og = ops.empty((mm * rep, dv))
                    ops.tc_gemm(P, vt, og, N_=dv, K=Sp)
                    ops.head_post(og.view(mm, rep * dv), o[a:a + mm, g * rep * dv:(g + 1) * rep * dv], dv=dv)


STATE_ROWS = 8     # rows of a matrix state's column that one thread holds (csrc/mixer_ops.cu: LS_R)


def state_lanes(dim: int) -> int:
    """threads that share a column of a matrix state (STATE_ROWS rows each; a power of two up to a warp): it fixes
    the layout of the state in the slot, [heads][STATE_ROWS][vdim][lanes]"""
    if dim > 32 * STATE_ROWS:
        raise ValueError(f"a matrix state with {dim} rows is not supported (at most {32 * STATE_ROWS})")
    lanes = 1
    while lanes * STATE_ROWS < dim:
        lanes *= 2
    return lanes


def state_floats(heads: int, dim: int, vdim: int) -> int:
    return heads * STATE_ROWS * vdim * state_lanes(dim)


class GatedDeltaRule:
    """Gated delta rule: per head a (dim, vdim) state with  S <- g S;  S <- S + k (beta (v - S^T k))^T;  o = S^T q.
    q, k (`kv_heads` heads, shared by heads / kv_heads value heads) and v pass a short causal convolution and silu; q, k
    are then scaled to unit length (q also by dim^-1/2); beta = sigmoid(W_b n); g = exp(-exp(A_log) softplus(W_a n +
    dt_bias)); every head's output is RMS-normed over vdim, weighted, and gated by silu(W_g n)."""

    def __init__(self, index: int, cfg: dict, width: int, unit_eps: float = 1e-6):
        self.index, self.W, self.unit_eps = index, width, unit_eps
        self.H, self.dim, self.taps = int(cfg["heads"]), int(cfg["dim"]), int(cfg.get("conv") or 1)
        self.G, self.vdim = int(cfg.get("kv_heads", self.H)), int(cfg.get("vdim", self.dim))
        if self.H % self.G:
            raise ValueError(f"layer {index}: {self.H} value heads do not divide over {self.G} query/key heads")
        self.n_qk, self.n_v = self.G * self.dim, self.H * self.vdim
        self.n_conv = 2 * self.n_qk + self.n_v
        self.in_names, self.out_name = ["q", "k", "v", "b", "a", "g"], "o"
        self.n_in, self.n_out = self.n_conv + 2 * self.H + self.n_v, self.n_v
        self.kv_dim = 0
        self.conv_floats = max(self.taps - 1, 0) * self.n_conv
        self.state_floats = self.conv_floats + state_floats(self.H, self.dim, self.vdim)
        self.w: Dict[str, torch.Tensor] = {}

    def in_rows(self, name: str) -> int:
        return {"q": self.n_qk, "k": self.n_qk, "v": self.n_v, "b": self.H, "a": self.H, "g": self.n_v}[name]

    def small(self):
        return [("conv", (self.n_conv, self.taps)), ("A_log", (self.H,)), ("dt_bias", (self.H,)), ("norm", (self.vdim,))]

    def checkpoint_small(self):
        return {"conv": ["q.conv", "k.conv", "v.conv"], "A_log": ["A_log"], "dt_bias": ["dt_bias"], "norm": ["norm"]}

    def forward(self, ctx: StepCtx, D, cat, kv_layer: int, state_off: int, out_scale: float = 1.0):
        ops, w, T = ctx.ops, self.w, D.shape[0]
        n, nc, H = self.n_qk, self.n_conv, self.H
        st = ctx.pool.state
        c = ops.short_conv(D[:, :nc], w["conv"], st[:, state_off:state_off + self.conv_floats], ctx, act=True)
        o = ops.empty((T, self.n_out))
        ops.linear_state(c[:, :n], c[:, n:2 * n], c[:, 2 * n:], o, st[:, state_off + self.conv_floats:state_off + self.state_floats],
                         ctx, H=H, rep=H // self.G, dim=self.dim, vdim=self.vdim, unit_eps=self.unit_eps,
                         q_scale=float(self.dim) ** -0.5, a=D[:, nc + H:nc + 2 * H], A_log=w["A_log"], dt_bias=w["dt_bias"],
                         b=D[:, nc:nc + H], delta=True)
        ops.head_post(o, cat, dv=self.vdim, gate=D[:, nc + 2 * H:], gate_silu=True, w=w["norm"], eps=ctx.eps, span=self.vdim,
                      scale=out_scale)


class DecayedState:
    """Outer-product state with a fixed decay per head:  S <- decay_h S + k v^T,  o = S^T q,  q, k, v = silu of their
    projections; the heads' outputs are RMS-normed together, weighted, and gated by sigmoid(W_g n)."""

    def __init__(self, index: int, cfg: dict, width: int):
        self.index, self.W = index, width
        self.H, self.dim = int(cfg["heads"]), int(cfg["dim"])
        self.vdim = int(cfg.get("vdim", self.dim))
        decay = cfg["decay"]
        self.decay = [float(d) for d in decay] if isinstance(decay, (list, tuple)) else [float(decay)] * self.H
        if len(self.decay) != self.H:
            raise ValueError(f"layer {index}: {len(self.decay)} decays for {self.H} heads")
        self.n_qk, self.n_v = self.H * self.dim, self.H * self.vdim
        self.in_names, self.out_name = ["q", "k", "v", "g"], "o"
        self.n_in, self.n_out = 2 * self.n_qk + 2 * self.n_v, self.n_v
        self.kv_dim = 0
        self.state_floats = state_floats(self.H, self.dim, self.vdim)
        self.w: Dict[str, torch.Tensor] = {}
        self._decay_dev = None

    def in_rows(self, name: str) -> int:
        return {"q": self.n_qk, "k": self.n_qk, "v": self.n_v, "g": self.n_v}[name]

    def small(self):
        return [("norm", (self.n_v,))]

    def checkpoint_small(self):
        return {"norm": ["norm"]}

    def forward(self, ctx: StepCtx, D, cat, kv_layer: int, state_off: int, out_scale: float = 1.0):
        ops, T = ctx.ops, D.shape[0]
        n, nv = self.n_qk, self.n_v
        if self._decay_dev is None:       # first used by a prompt step, never inside a captured decode step
            import numpy as np
            self._decay_dev = ops.to_device(np.asarray(self.decay, dtype=np.float32), np.float32)
        o = ops.empty((T, nv))
        ops.linear_state(D[:, :n], D[:, n:2 * n], D[:, 2 * n:2 * n + nv], o,
                         ctx.pool.state[:, state_off:state_off + self.state_floats], ctx, H=self.H, rep=1, dim=self.dim,
                         vdim=self.vdim, act=True, decay_const=self._decay_dev)
        ops.head_post(o, cat, dv=self.vdim, gate=D[:, 2 * n + nv:], w=self.w["norm"], eps=ctx.eps, span=nv, scale=out_scale)


class ClampedGLU:
    """Gated feed-forward with clamps: g = min(W_gate n, limit), u = clamp(W_up n, -limit, limit),
    W_down (g sigmoid(alpha g) (u + 1))."""

    def __init__(self, index: int, cfg: dict, width: int, alpha: float = 1.702):
        self.index, self.W, self.alpha = index, width, alpha
        self.ff, self.limit = int(cfg["ff"]), float(cfg["limit"])
        self.in_names, self.out_name = ["gate", "up"], "down"
        self.n_in, self.n_out = 2 * self.ff, self.ff
        self.kv_dim = self.state_floats = 0
        self.w: Dict[str, torch.Tensor] = {}

    def in_rows(self, name: str) -> int:
        return self.ff

    def small(self):
        return []

    def checkpoint_small(self):
        return {}

    def forward(self, ctx: StepCtx, D, cat, kv_layer: int, state_off: int, out_scale: float = 1.0):
        ctx.ops.glu_clamp(D[:, :self.ff], D[:, self.ff:], self.limit, self.alpha, cat)


def _side_by_side(index: int, cfg: dict, width: int):
    """an attention (gate per head) and a gated delta rule reading the same input; their outputs are weighted"""
    return [("left.", SinkAttention(index, cfg["left"], width, gate="head"), float(cfg["left_scale"])),
            ("right.", GatedDeltaRule(index, cfg["right"], width), float(cfg["right_scale"]))]


FUSED_MIXERS = {"attention": lambda i, c, w: [("", SinkAttention(i, c, w, gate="element"), 1.0)],
                "lightning": lambda i, c, w: [("", DecayedState(i, c, w), 1.0)],
                "parallel": _side_by_side}
FUSED_FEEDFORWARDS = {"dense": ClampedGLU}


class SharedInputLayer:
    """n = rmsnorm(x) * w;  x <- x + sum_parts scale_part * part(n).  The parts' input projections are stacked into ONE
    weight (one product per layer gives every part its rows), their output projections are laid side by side into ONE
    weight whose input is the parts' outputs side by side — the sum over the parts and the residual add happen inside
    that product.  A part's scale is applied to its output before the product."""

    def __init__(self, index: int, cfg: dict, width: int):
        self.index, self.W = index, width
        if cfg["type"] not in FUSED_MIXERS:
            raise ValueError(f"layer {index}: unknown mixer type {cfg['type']!r} (have {sorted(FUSED_MIXERS)})")
        self.parts = [("mix." + p, part, s) for p, part, s in FUSED_MIXERS[cfg["type"]](index, cfg["mixer"], width)]
        f = cfg.get("mlp")
        if f is not None:
            if f.get("kind") not in FUSED_FEEDFORWARDS:
                raise ValueError(f"layer {index}: unknown feed-forward kind {f.get('kind')!r} (have {sorted(FUSED_FEEDFORWARDS)})")
            self.parts.append(("mlp.", FUSED_FEEDFORWARDS[f["kind"]](index, f, width), 1.0))
        self.n_in = sum(part.n_in for _, part, _ in self.parts)
        self.n_out = sum(part.n_out for _, part, _ in self.parts)
        self.kv_layers = sum(1 for _, part, _ in self.parts if part.kv_dim)
        self.kv_dim = max(part.kv_dim for _, part, _ in self.parts)
        self.state_floats = sum(part.state_floats for _, part, _ in self.parts)
        self.w: Dict[str, torch.Tensor] = {}

    def manifest(self, p: str):
        out = [(p + "norm1", (self.W,)), (p + "in", (self.n_in, self.W)), (p + "out", (self.W, self.n_out))]
        for pre, part, _ in self.parts:
            out += [(p + pre + n, shape) for n, shape in part.small()]
        return out

    def checkpoint_tensors(self, p: str):
        """checkpoint name -> shape of everything this layer reads"""
        out = {p + "norm1": (self.W,)}
        for pre, part, _ in self.parts:
            for n in part.in_names:
                out[p + pre + n] = (part.in_rows(n), self.W)
            out[p + pre + part.out_name] = (self.W, part.n_out)
            shapes = dict(part.small())
            for packed, names in part.checkpoint_small().items():
                if len(names) == 1:
                    out[p + pre + names[0]] = shapes[packed]
                else:       # the convolutions of q, k, v stacked: rows split like the projections'
                    for n in names:
                        out[p + pre + n] = (part.in_rows(n.split(".")[0]), shapes[packed][1])
        return out

    def pack(self, p: str, ck, view):
        view(p + "norm1").copy_(ck[p + "norm1"])
        w_in, w_out = view(p + "in"), view(p + "out")
        r = c = 0
        for pre, part, _ in self.parts:
            for n in part.in_names:
                t = ck[p + pre + n]
                w_in[r:r + t.shape[0]].copy_(t)
                r += t.shape[0]
            w_out[:, c:c + part.n_out].copy_(ck[p + pre + part.out_name])
            c += part.n_out
            for packed, names in part.checkpoint_small().items():
                dst, at = view(p + pre + packed), 0
                for n in names:
                    t = ck[p + pre + n]
                    dst[at:at + t.shape[0]].copy_(t)
                    at += t.shape[0]
        self.bind(p, view)

    def bind(self, p: str, view):
        self.w = {n: view(p + n) for n in ("norm1", "in", "out")}
        for pre, part, _ in self.parts:
            part.w = {n: view(p + pre + n) for n, _ in part.small()}

    def forward(self, ctx: StepCtx, x: torch.Tensor, kv_base: int = 0, state_base: int = 0):
        """kv_base: the pool's caching layer of this RUN's first attention; state_base: its offset in the slot's state"""
        ops, T = ctx.ops, x.shape[0]
        n = ops.empty((T, self.W))
        ops.norm_rows(x, self.w["norm1"], ctx.eps, n)
        D = ops.linear(n, self.w["in"])
        cat = ops.empty((T, self.n_out))
        a = c = 0
        for _, part, scale in self.parts:
            part.forward(ctx, D[:, a:a + part.n_in], cat[:, c:c + part.n_out], kv_base, state_base, scale)
            a, c = a + part.n_in, c + part.n_out
            kv_base += 1 if part.kv_dim else 0
            state_base += part.state_floats
        ops.linear(cat, self.w["out"], out=x, add=True)


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
