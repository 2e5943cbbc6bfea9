"""Sonulorn on the GPU against the plain restatement in oracle/sonulorn.py: every mechanism alone (with inputs made
so that a fault shows: one key that stands out, far back, at a staging tile's edge, just inside and just outside a
block of visible keys; a sink that takes most of the weight), whole prompts with the residual stream after every
layer run, prefill against token-by-token decoding, portions, batches of unequal requests, slots released and used
again, long decoding, other sizes, and greedy generation through generate_step and the batch scheduler.  Small
random configurations; none of them is a real model's."""
import copy
import types

import numpy as np
import pytest
import torch

from oracle import sonulorn as O

pytestmark = pytest.mark.gpu


# ------------------------------------------------------------------------------------------------ configurations
def attn(heads=4, kv_heads=2, dim=16, vdim=24, rot=8, base=5000.0, block=None, conv=None, scale=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "rot": {"base": base, "dims": rot},
         "scale": scale if scale is not None else 1.0 / float(dim) ** 0.5}
    if block:
        m["mask"] = {"size": block}
    if conv:
        m["conv"] = conv
    return m


def delta(heads=4, kv_heads=2, dim=24, vdim=16, conv=3):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}


def mlp(ff=40, limit=1.25):
    return {"kind": "dense", "ff": ff, "limit": limit}


def L_attn(ff=True, **kw):
    return {"type": "attention", "mixer": attn(**kw), "mlp": mlp() if ff else None}


def L_par(ff=True, left=None, right=None, ls=0.7, rs=0.6):
    return {"type": "parallel", "mlp": mlp() if ff else None,
            "mixer": {"left": left or attn(heads=3, kv_heads=3, dim=16, vdim=8, rot=16, conv=2), "left_scale": ls,
                      "right": right or delta(), "right_scale": rs}}


def L_light(ff=True, heads=3, dim=16, vdim=24, decay=None):
    return {"type": "lightning", "mlp": mlp() if ff else None,
            "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay or [0.5 + 0.49 * i / heads for i in range(heads)]}}


def config(layers=None, loop=(0, 3, 2), width=72, vocab=101, scale=3.0, eps=1e-5):
    layers = layers or [L_par(), L_light(), L_attn(block=11), L_par(ff=False), L_attn(rot=4)]
    c = {"architecture": "Sonulorn", "vocab": vocab, "width": width, "layers": layers, "embedding": {"scale": scale},
         "norm": {"eps": eps}}
    if loop:
        c["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return c


_MODELS = {}


def build(cfg, dtype="float32", seed=1):
    from mlx_vlm_b200.models.sonulorn import Model, ModelConfig
    key = (repr(cfg), dtype, seed)
    if key not in _MODELS:
        W = O.random_weights(cfg, seed)
        _MODELS[key] = (Model(ModelConfig.from_dict(copy.deepcopy(cfg)), dtype=dtype).load_weights(W), W)
    return _MODELS[key]


def host(eng, t):
    eng.stream.synchronize()
    return t.detach().to("cpu", torch.float64)


def rel_rows(got, want):
    d = got - want
    d = d - d.mean(-1, keepdim=True)
    return d.square().mean(-1).sqrt() / (want - want.mean(-1, keepdim=True)).square().mean(-1).sqrt()


def rel(got, want):
    return rel_rows(got, want).max().item()


TOL = {"float32": 3e-5, "bfloat16": 8e-2}


def tokens(n, vocab, seed=0):
    return np.random.default_rng(seed).integers(0, vocab, n).tolist()


def run_alone(model, toks, cuts=None):
    """one request in its own fresh pool, its tokens cut into portions; logits of every position"""
    lm = model.language_model
    cache = lm.make_cache()
    out, at = [], 0
    for n in (cuts or [len(toks)]):
        part = toks[at:at + n]
        out.append(host(model.engine, lm.step([part], [cache], want=[list(range(len(part)))])))
        at += n
    assert at == len(toks)
    return torch.cat(out)


# ------------------------------------------------------------------------------------------------ mechanisms
def _eng():
    from mlx_vlm_b200.layer_engine import LayerEngine
    if "eng" not in _MODELS:
        _MODELS["eng"] = LayerEngine("cuda:0", exact=True)
    return _MODELS["eng"]


def dev(a, dtype=torch.float32):
    return torch.as_tensor(a).to(device="cuda:0", dtype=dtype).contiguous()


class _Pool:
    """what the mixers read of a pool: rows (caching layers, slots, capacity, row) and state (slots, floats)"""

    def __init__(self, slots=3, capacity=0, row=0, state=0):
        self.buf = torch.zeros((1, slots, max(capacity, 1), max(row, 1)), device="cuda:0")
        self.state = torch.full((slots, max(state, 1)), 7.0, device="cuda:0")     # stale numbers: never to be read
        torch.cuda.synchronize()


def _ctx(eng, pool, segments):
    """segments: (first row, rows, slot, first position) per sequence"""
    from mlx_vlm_b200.models.decoder_blocks import StepCtx
    T = sum(n for _, n, _, _ in segments)
    slot, pos = np.zeros(T, np.int32), np.zeros(T, np.int32)
    for a, n, s, p0 in segments:
        slot[a:a + n], pos[a:a + n] = s, np.arange(p0, p0 + n)
    return StepCtx(eng.ops, dev(slot, torch.int32), dev(pos, torch.int32), pool, 1e-5, segments)


@pytest.mark.parametrize("taps", [1, 2, 4])
@pytest.mark.parametrize("cuts", [[30], [1] * 12, [2, 1, 3, 24], [5, 25]])
def test_short_convolution_carries_its_last_inputs(taps, cuts):
    """two sequences in one launch, cut at different places, in slots that hold stale numbers"""
    eng = _eng()
    C, T = 37, sum(cuts)
    g = torch.Generator().manual_seed(taps)
    u = torch.randn(2, T, C, generator=g)
    w = torch.randn(C, taps, generator=g).bfloat16()
    pool = _Pool(slots=3, state=(taps - 1) * C + 6)
    st = pool.state[:, 5:5 + max((taps - 1) * C, 1)]
    got, at = [[], []], [0, 0]
    for na, nb in zip(cuts, cuts[::-1]):
        segs = [(0, na, 2, at[0]), (na, nb, 0, at[1])]
        rows = torch.cat([u[0, at[0]:at[0] + na], u[1, at[1]:at[1] + nb]])
        y = host(eng, eng.ops.short_conv(dev(rows), dev(w, torch.bfloat16), st, _ctx(eng, pool, segs), act=False))
        got[0].append(y[:na])
        got[1].append(y[na:])
        at = [at[0] + na, at[1] + nb]
    for i in (0, 1):
        assert (torch.cat(got[i]) - O.short_conv(u[i].double(), w.double())).abs().max() < 1e-5
    y = host(eng, eng.ops.short_conv(dev(u[0]), dev(w, torch.bfloat16), st, _ctx(eng, pool, [(0, T, 0, 0)]), act=True))
    assert (y - torch.nn.functional.silu(O.short_conv(u[0].double(), w.double()))).abs().max() < 1e-5


def _attend(eng, H, G, d, dv, k, v, q, qpos, slot=1, sink=None, scale=1.0, chunk=0, n_split=None, rot=0, base=10.0):
    """k, v (S, G, d / dv) written through qkv_post into slot `slot`, then q (n, H, d) at positions qpos"""
    S = k.shape[0]
    pool = _Pool(slots=2, capacity=S + 3, row=G * (d + dv) + 2)
    rows = pool.buf[0][..., :G * (d + dv)]
    ops = eng.ops
    pos = dev(np.arange(S), torch.int32)
    sl = dev(np.full(S, slot), torch.int32)
    junk = dev(torch.zeros(S, H * d))
    ops.qkv_post(junk, dev(k.reshape(S, -1)), dev(v.reshape(S, -1)), rows, sl, pos, ops.rope_table(pos, base, rot), H, G, d, dv, rot)
    n = q.shape[0]
    qd, qp = dev(q.reshape(n, -1)), dev(np.asarray(qpos), torch.int32)
    qs = dev(np.full(n, slot), torch.int32)
    zk, zv = dev(torch.zeros(n, G * d)), dev(torch.zeros(n, G * dv))
    scratch = _Pool(slots=2, capacity=S + 3, row=G * (d + dv) + 2)
    ops.qkv_post(qd, zk, zv, scratch.buf[0][..., :G * (d + dv)], qs, qp, ops.rope_table(qp, base, rot), H, G, d, dv, rot)
    out = dev(torch.zeros(n, H * dv))
    ops.sink_attention(qd, rows, qs, qp, out, None if sink is None else dev(sink, torch.bfloat16), H, G, d, dv, scale,
                       chunk=chunk, n_split=n_split)
    return host(eng, out).view(n, H, dv)


def _attend_plain(k, v, q, qpos, sink, scale, block, rot=0, base=10.0):
    """the restatement on one query at a time: the query sits at the end of the keys it may see"""
    H, out = q.shape[1], []
    for i, p in enumerate(qpos):
        T = p + 1
        kk = O.rotate_half(k[:T].double(), torch.arange(T), base, rot)
        qq = O.rotate_half(q[i:i + 1].double().expand(T, -1, -1).clone(), torch.arange(T), base, rot)
        s = sink.double() if sink is not None else torch.full((H,), -1e30, dtype=torch.float64)
        out.append(O.sink_softmax_attention(qq, kk, v[:T].double(), scale, s, block)[-1])
    return torch.stack(out)


@pytest.mark.parametrize("d,dv", [(16, 24), (15, 33)])
def test_attention_far_key_tile_edges_and_heads(d, dv):
    """keys are staged 32 at a time: a key that stands out is found at the first row, at both sides of a tile's edge
    and far back among hundreds; the row one past the query is never seen; every query head reads its own kv head"""
    eng = _eng()
    H, G, S = 6, 3, 700
    g = torch.Generator().manual_seed(d)
    k = torch.nn.functional.normalize(torch.randn(S, G, d, generator=g), dim=-1)
    v = torch.randn(S, G, dv, generator=g)
    sink = torch.randn(H, generator=g).bfloat16()
    for key in (0, 31, 32, 33, 63, 64, 350, 698):
        for qpos in (key, key + 1, 699):
            q = torch.randn(1, H, d, generator=g) * 0.3
            q[0, 3] = k[key, 1] * 120.0                      # head 3 (kv head 1) points at row `key`
            for split in (1, None):
                got = _attend(eng, H, G, d, dv, k, v, q, [qpos], sink=sink, n_split=split)
                want = _attend_plain(k, v, q, [qpos], sink, 1.0, None)
                assert (got - want).abs().max() < 2e-5
                assert (got[0, 3] - v[key, 1].double()).abs().max() < 1e-3
    q = torch.zeros(1, H, d)
    q[0, :] = k[40, 0] * 120.0
    got = _attend(eng, H, G, d, dv, k, v, q, [39], sink=sink)
    assert (got - _attend_plain(k, v, q, [39], sink, 1.0, None)).abs().max() < 2e-5
    assert (got[0, 0] - v[40, 0].double()).abs().max() > 0.05


@pytest.mark.parametrize("block", [1, 7, 32, 50])
def test_attention_block_of_visible_keys(block):
    """a query sees the keys of its own block of positions only: a key that stands out takes all the weight when it is
    the first key of the query's block and none when it is the last key of the block before, in prompts (many queries
    in a launch) and for a single decoded query, with and without splits"""
    eng = _eng()
    H, G, d, dv, S = 2, 1, 8, 8, 160
    g = torch.Generator().manual_seed(block)
    k = torch.nn.functional.normalize(torch.randn(S, G, d, generator=g), dim=-1)
    v = torch.randn(S, G, dv, generator=g)
    qpos = list(range(S))
    q = torch.randn(S, H, d, generator=g) * 0.2
    for p in qpos:        # head 1 of every query points at the last key BEFORE its block (invisible) ...
        start = (p // block) * block
        if start > 0:
            q[p, 1] = k[start - 1, 0] * 100.0
    got = _attend(eng, H, G, d, dv, k, v, q, qpos, chunk=block, n_split=1)
    want = _attend_plain(k, v, q, qpos, None, 1.0, block)
    assert (got - want).abs().max() < 2e-5
    for p in (block, S - 1):
        start = (p // block) * block
        if 0 < start < S:
            assert (got[p, 1] - v[start - 1, 0].double()).abs().max() > 0.05
    for p in qpos:        # ... and now at the first key OF its block (visible)
        q[p, 1] = k[(p // block) * block, 0] * 100.0
    got = _attend(eng, H, G, d, dv, k, v, q, qpos, chunk=block, n_split=1)
    assert (got - _attend_plain(k, v, q, qpos, None, 1.0, block)).abs().max() < 2e-5
    for p in (S - 1, S // 2):
        one = _attend(eng, H, G, d, dv, k, v, q[p:p + 1], [p], chunk=block)
        assert (one[0] - got[p]).abs().max() < 2e-6
        assert (one[0, 1] - v[(p // block) * block, 0].double()).abs().max() < 1e-3


def test_attention_sink_counts_once_and_rotation():
    eng = _eng()
    H, G, d, dv, S = 4, 2, 16, 8, 90
    g = torch.Generator().manual_seed(5)
    k, v = torch.randn(S, G, d, generator=g), torch.randn(S, G, dv, generator=g)
    q = torch.randn(3, H, d, generator=g)
    sink = torch.tensor([12.0, -30.0, 0.0, 2.0]).bfloat16()       # head 0: the sink takes nearly everything
    qpos = [0, 40, 89]
    for split in (1, 4, 64):
        got = _attend(eng, H, G, d, dv, k, v, q, qpos, sink=sink, scale=0.3, n_split=split, rot=12, base=77.0)
        want = _attend_plain(k, v, q, qpos, sink, 0.3, None, rot=12, base=77.0)
        assert (got - want).abs().max() < 2e-5
    none = _attend(eng, H, G, d, dv, k, v, q, qpos, sink=None, scale=0.3, rot=12, base=77.0)
    assert none[:, 0].abs().max() > 10 * got[:, 0].abs().max()      # without the sink head 0 is not damped
    assert (none[:, 1] - got[:, 1]).abs().max() < 1e-5               # a sink of -30 changes nothing


@pytest.mark.parametrize("d,dv,H,rep", [(16, 24, 3, 1), (24, 16, 4, 2), (64, 40, 2, 2), (100, 130, 2, 1), (160, 8, 1, 1)])
@pytest.mark.parametrize("kind", ["delta", "plain"])
def test_matrix_state_in_portions_and_slots(d, dv, H, rep, kind):
    """the state of a sequence survives from step to step in its slot; a slot that held another sequence starts anew"""
    eng = _eng()
    ops = eng.ops
    from mlx_vlm_b200.models.decoder_blocks import state_floats
    T, Hk = 45, H // rep
    g = torch.Generator().manual_seed(d + dv)
    q, k = torch.randn(T, Hk, d, generator=g), torch.randn(T, Hk, d, generator=g)
    v = torch.randn(T, H, dv, generator=g)
    a, b = torch.randn(T, H, generator=g), torch.randn(T, H, generator=g)
    A_log, dt = (torch.randn(H, generator=g) * 0.5).bfloat16(), torch.randn(H, generator=g).bfloat16()
    decay_h = torch.rand(H, generator=g) * 0.5 + 0.5
    floats = state_floats(H, d, dv)
    pool = _Pool(slots=3, state=floats + 3)
    st = pool.state[:, 3:3 + floats]
    if kind == "delta":
        qn = q.double() / torch.sqrt((q.double() ** 2).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
        kn = k.double() / torch.sqrt((k.double() ** 2).sum(-1, keepdim=True) + 1e-6)
        dec = torch.exp(-torch.exp(A_log.double()) * torch.nn.functional.softplus(a.double() + dt.double()))
        want = O.delta_rule(qn.repeat_interleave(rep, 1), kn.repeat_interleave(rep, 1), v.double(), dec, torch.sigmoid(b.double()))
    else:
        f = torch.nn.functional.silu
        want = O.decayed_state(f(q.double()).repeat_interleave(rep, 1), f(k.double()).repeat_interleave(rep, 1), f(v.double()),
                               decay_h.double())
    for cuts in ([T], [1] * 6 + [17, 2, 20]):
        got, at = [], 0
        for n in cuts:
            ctx = _ctx(eng, pool, [(0, n, 1, at)])
            o = dev(torch.zeros(n, H * dv))
            sl = slice(at, at + n)
            if kind == "delta":
                ops.linear_state(dev(q[sl].reshape(n, -1)), dev(k[sl].reshape(n, -1)), dev(v[sl].reshape(n, -1)), o, st, ctx,
                                 H=H, rep=rep, dim=d, vdim=dv, unit_eps=1e-6, q_scale=d ** -0.5, a=dev(a[sl]),
                                 A_log=dev(A_log, torch.bfloat16), dt_bias=dev(dt, torch.bfloat16), b=dev(b[sl]), delta=True)
            else:
                ops.linear_state(dev(q[sl].reshape(n, -1)), dev(k[sl].reshape(n, -1)), dev(v[sl].reshape(n, -1)), o, st, ctx,
                                 H=H, rep=rep, dim=d, vdim=dv, act=True, decay_const=dev(decay_h))
            got.append(host(eng, o).view(n, H, dv))
            at += n
        err = (torch.cat(got) - want).abs().max() / want.abs().max()
        assert err < 2e-5, (cuts, err)


def test_head_post_and_clamped_activation():
    eng = _eng()
    ops = eng.ops
    g = torch.Generator().manual_seed(2)
    T, H, dv = 5, 3, 20
    o, gate, gh = torch.randn(T, H * dv, generator=g) * 3, torch.randn(T, H * dv, generator=g), torch.randn(T, H, generator=g)
    w1, wall = torch.randn(dv, generator=g).bfloat16(), torch.randn(H * dv, generator=g).bfloat16()
    out = dev(torch.zeros(T, H * dv + 4))
    ops.head_post(dev(o), out[:, 4:], dv=dv, gate=dev(gate))
    assert (host(eng, out)[:, 4:] - o.double() * torch.sigmoid(gate.double())).abs().max() < 1e-5
    ops.head_post(dev(o), out[:, 4:], dv=dv, gate=dev(gh), gate_per_head=True, scale=0.7)
    want = (o.double().view(T, H, dv) * torch.sigmoid(gh.double())[:, :, None]).reshape(T, -1) * 0.7
    assert (host(eng, out)[:, 4:] - want).abs().max() < 1e-5
    ops.head_post(dev(o), out[:, 4:], dv=dv, gate=dev(gate), gate_silu=True, w=dev(w1, torch.bfloat16), eps=1e-3, span=dv)
    want = (O.rms(o.double().view(T, H, dv), 1e-3) * w1.double()).reshape(T, -1) * torch.nn.functional.silu(gate.double())
    assert (host(eng, out)[:, 4:] - want).abs().max() < 1e-5
    ops.head_post(dev(o), out[:, 4:], dv=dv, gate=dev(gate), w=dev(wall, torch.bfloat16), eps=1e-3, span=H * dv)
    want = O.norm(o.double(), wall.double(), 1e-3) * torch.sigmoid(gate.double())
    assert (host(eng, out)[:, 4:] - want).abs().max() < 1e-5
    # a norm group longer than a warp's share is summed by a whole block
    big, gbig, wbig = torch.randn(T, 3000, generator=g), torch.randn(T, 3000, generator=g), torch.randn(3000, generator=g).bfloat16()
    out = dev(torch.zeros(T, 3000))
    ops.head_post(dev(big), out, dv=1500, gate=dev(gbig), w=dev(wbig, torch.bfloat16), eps=1e-5, span=3000, scale=0.5)
    assert (host(eng, out) - O.norm(big.double(), wbig.double(), 1e-5) * torch.sigmoid(gbig.double()) * 0.5).abs().max() < 1e-5
    a, b = torch.randn(T, 700, generator=g) * 2, torch.randn(T, 700, generator=g) * 2
    y = dev(torch.zeros(T, 700))
    ops.glu_clamp(dev(a), dev(b), 1.25, 1.702, y)
    gg, uu = a.double().clamp(max=1.25), b.double().clamp(-1.25, 1.25)
    assert (host(eng, y) - gg * torch.sigmoid(1.702 * gg) * (uu + 1)).abs().max() < 1e-5
    # many rows of whole 16-byte vectors (a prompt step) take four columns per thread; column ranges of wider rows
    wide = torch.randn(40, 3 * 64, generator=g) * 2
    wd, y = dev(wide), dev(torch.zeros(40, 64 + 4))
    ops.glu_clamp(wd[:, :64], wd[:, 128:], 1.25, 1.702, y[:, 4:])
    gg, uu = wide[:, :64].double().clamp(max=1.25), wide[:, 128:].double().clamp(-1.25, 1.25)
    assert (host(eng, y)[:, 4:] - gg * torch.sigmoid(1.702 * gg) * (uu + 1)).abs().max() < 1e-5


@pytest.mark.parametrize("M", [1, 3, 12, 40, 150])
def test_product_added_to_its_output_rows(M):
    """x += y . W^T on column ranges of wider rows, on every row kernel and (serving mode, many rows) the tensor cores"""
    from mlx_vlm_b200.layer_engine import LayerEngine
    if "eng16" not in _MODELS:
        _MODELS["eng16"] = LayerEngine("cuda:0", exact=False)
    g = torch.Generator().manual_seed(M)
    K, N_ = 48, 40
    wide = (torch.randn(N_, 2 * K, generator=g) / 7).bfloat16()
    y, x0 = torch.randn(M, K + 8, generator=g), torch.randn(M, N_, generator=g)
    bias = torch.randn(N_, generator=g).bfloat16()
    for eng, yy, tol in ((_eng(), y, 1e-5), (_MODELS["eng16"], y.bfloat16().float(), 1e-5)):
        x = dev(x0)
        eng.ops.linear(dev(yy)[:, 8:], dev(wide, torch.bfloat16)[:, K:], out=x, add=True)
        want = x0.double() + yy[:, 8:].double() @ wide[:, K:].double().T
        assert (host(eng, x) - want).abs().max() < tol * 10
        z = eng.ops.linear(dev(yy)[:, 8:], dev(wide, torch.bfloat16)[:, :K], bias=dev(bias, torch.bfloat16))
        assert (host(eng, z) - (yy[:, 8:].double() @ wide[:, :K].double().T + bias.double())).abs().max() < tol * 10


@pytest.mark.parametrize("M", [1, 2, 4, 7])
def test_product_with_long_rows_and_few_of_them(M):
    """a decode-step product whose weight has few rows of many columns (several staging chunks per row)"""
    eng = _eng()
    g = torch.Generator().manual_seed(M)
    K, N_ = 4104, 24
    W = (torch.randn(N_, K, generator=g) / 64).bfloat16()
    y, x0 = torch.randn(M, K, generator=g), torch.randn(M, N_, generator=g)
    x = dev(x0)
    eng.ops.linear(dev(y), dev(W, torch.bfloat16), out=x, add=True)
    assert (host(eng, x) - (x0.double() + y.double() @ W.double().T)).abs().max() < 1e-4


# ------------------------------------------------------------------------------------------------ the model
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_prompt_and_every_layer_run(dtype):
    cfg = config()
    model, W = build(cfg, dtype)
    toks = tokens(150, cfg["vocab"], 1)
    layers_ref = []
    ref = O.forward(cfg, W, toks, torch.float64, layers_ref)
    assert rel(run_alone(model, toks), ref) < TOL[dtype]
    if dtype == "float32":
        from mlx_vlm_b200.models.decoder_blocks import StepCtx
        eng, lm = model.engine, model.language_model
        pool = lm.make_pool(1, 256)
        T = len(toks)
        ctx = StepCtx(eng.ops, dev(torch.zeros(T), torch.int32), dev(torch.arange(T), torch.int32), pool, model.eps,
                      [(0, T, 0, 0)])
        x = eng.ops.embed(dev(toks, torch.int32), model.embed, model.embed_scale)
        seen = []
        real = [L.forward for L in model.layers]
        try:
            for L, f in zip(model.layers, real):
                def wrapped(c, xx, kv, st, f=f):
                    f(c, xx, kv, st)
                    seen.append(host(eng, xx))
                L.forward = wrapped
            model.run_layers(ctx, x, lambda: eng.ops.embed(dev(toks, torch.int32), model.embed, model.embed_scale))
        finally:
            for L, f in zip(model.layers, real):
                L.forward = f
        assert len(seen) == len(layers_ref) == 8
        for got, want in zip(seen, layers_ref):
            assert (got - want).abs().max() < 3e-4 * max(1.0, want.abs().max().item())


def test_first_tokens():
    cfg = config()
    model, W = build(cfg)
    for n in (1, 2, 3, 4):
        toks = tokens(n, cfg["vocab"], 10 + n)
        assert rel(run_alone(model, toks), O.forward(cfg, W, toks)) < TOL["float32"]
        assert rel(run_alone(model, toks, [1] * n), O.forward(cfg, W, toks)) < TOL["float32"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prefill_then_token_by_token(dtype):
    cfg = config()
    model, W = build(cfg, dtype)
    toks = tokens(90, cfg["vocab"], 2)
    ref = O.forward(cfg, W, toks)
    got = run_alone(model, toks, [50] + [1] * 40)       # the decoded tokens cross several blocks of visible keys
    assert rel(got, ref) < TOL[dtype]
    if dtype == "float32":
        assert rel(got, run_alone(model, toks)) < TOL[dtype]
        assert rel(run_alone(model, toks, [1] * 90), ref) < TOL[dtype]


@pytest.mark.parametrize("cuts", [[2] * 35, [3, 64, 3], [31, 1, 32, 6], [33, 2, 35], [69, 1], [11, 11, 22, 26]])
def test_portions(cuts):
    cfg = config()
    model, W = build(cfg)
    toks = tokens(70, cfg["vocab"], 3)
    assert rel(run_alone(model, toks, cuts), O.forward(cfg, W, toks)) < TOL["float32"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unequal_batch_against_each_alone(dtype):
    cfg = config()
    model, W = build(cfg, dtype)
    lm, eng = model.language_model, model.engine
    lens = [1, 45, 130, 18]
    reqs = [tokens(n + 12, cfg["vocab"], 20 + n) for n in lens]
    pool = lm.make_pool(4, 64)                       # too short on purpose: it grows under the batch
    caches = [lm.make_cache_row(pool, s) for s in (2, 0, 3, 1)]
    first = host(eng, lm.step([r[:n] for r, n in zip(reqs, lens)], caches, want=[list(range(n)) for n in lens]))
    got = list(torch.split(first, lens))
    for k in range(12):                              # then all go on by one token, together
        step = host(eng, lm.step([[r[n + k]] for r, n in zip(reqs, lens)], caches))
        got = [torch.cat([g, step[i:i + 1]]) for i, g in enumerate(got)]
    for g, r in zip(got, reqs):
        assert rel(g, O.forward(cfg, W, r)) < TOL[dtype]
        if dtype == "float32":
            assert rel(g, run_alone(model, r)) < TOL[dtype]


def test_slots_released_and_used_again_and_more_slots():
    from mlx_vlm_b200.models.cache import SlotTable
    cfg = config()
    model, W = build(cfg)
    lm, eng = model.language_model, model.engine
    pool, table = lm.make_pool(2, 64), SlotTable(2)
    a, b, c, d = (tokens(n, cfg["vocab"], 40 + n) for n in (40, 25, 33, 50))
    ca, cb = lm.make_cache_row(pool, table.acquire("a")), lm.make_cache_row(pool, table.acquire("b"))
    lm.step([a[:30], b], [ca, cb])
    table.release("b")                                   # b is finished; c takes its slot (and b's stale state)
    cc = lm.make_cache_row(pool, table.acquire("c"))
    assert cc[0]._row == 1 and cc[0].offset == 0
    got = host(eng, lm.step([a[30:], c], [ca, cc], want=[list(range(10)), list(range(33))]))
    assert rel(got[:10], O.forward(cfg, W, a)[30:]) < TOL["float32"]
    assert rel(got[10:], O.forward(cfg, W, c)) < TOL["float32"]
    with torch.cuda.stream(eng.stream):                  # a third live request: the pool gets more slots
        pool.add_slots(4, live_tokens=pool.capacity)
    table.grow(4)
    cd = lm.make_cache_row(pool, table.acquire("d"))
    assert cd[0]._row == 2
    got = host(eng, lm.step([[a[0]], d], [ca, cd], want=[[], list(range(50))]))
    assert rel(got, O.forward(cfg, W, d)) < TOL["float32"]
    got = host(eng, lm.step([[5]], [cc]))                # c's rows and state survived the move
    assert rel(got, O.forward(cfg, W, c + [5])[-1:]) < TOL["float32"]
    # a slot copied to another row (the scheduler's compaction) carries rows and state
    eng.kv_copy_row(pool, 3, pool, 1, cc[0].offset)
    moved = lm.make_cache_row(pool, 3)
    for m in moved:
        m.offset = cc[0].offset
    got = host(eng, lm.step([[9]], [moved]))
    assert rel(got, O.forward(cfg, W, c + [5, 9])[-1:]) < TOL["float32"]


def test_long_prompt_paths_of_the_serving_mode():
    """prompts of 128 tokens and more take the tensor-core products; a long portion after a cached prefix; a batch
    whose short member stays on the row kernels"""
    cfg = config()
    model, W = build(cfg, "bfloat16", seed=4)
    exact, _ = build(cfg, "float32", seed=4)
    lm, eng = model.language_model, model.engine
    toks = tokens(330, cfg["vocab"], 9)
    ref = O.forward(cfg, W, toks)
    assert rel(run_alone(model, toks, [140, 150, 40]), ref) < TOL["bfloat16"]
    assert rel(run_alone(exact, toks, [140, 150, 40]), ref) < TOL["float32"]
    # blocks of visible keys as long as a tile: a block's share of a portion runs against that block's keys only
    wide = config([L_attn(block=150, heads=6, kv_heads=2), L_par(left=attn(heads=4, kv_heads=2, dim=16, vdim=8, rot=16, conv=3, block=200))],
                  loop=(0, 2, 2))
    m2, W2 = build(wide, "bfloat16", seed=6)
    ref2 = O.forward(wide, W2, toks)
    assert rel(run_alone(m2, toks, [140, 150, 40]), ref2) < TOL["bfloat16"]
    assert rel(run_alone(m2, toks), ref2) < TOL["bfloat16"]
    pool = lm.make_pool(2, 512)
    ca, cb = lm.make_cache_row(pool, 0), lm.make_cache_row(pool, 1)
    both = host(eng, lm.step([toks[:200], toks[:30]], [ca, cb], want=[list(range(200)), list(range(30))]))
    assert rel(both[:200], ref[:200]) < TOL["bfloat16"] and rel(both[200:], ref[:30]) < TOL["bfloat16"]


def test_long_decoding():
    cfg = config()
    model, W = build(cfg)
    toks = tokens(330, cfg["vocab"], 5)
    got = run_alone(model, toks, [20] + [1] * 310)
    assert rel(got, O.forward(cfg, W, toks)) < TOL["float32"]


OTHER = {
    "no repeated span": config([L_attn(block=5), L_par(), L_light()], loop=None),
    "the span starts late and runs three times": config([L_light(), L_attn(), L_par(), L_light(ff=False)], loop=(1, 3, 3)),
    "one run of the span, one layer": config([L_par()], loop=(0, 1, 1)),
    "one head everywhere": config([L_attn(heads=1, kv_heads=1, block=9), L_light(heads=1),
                                   L_par(left=attn(heads=1, kv_heads=1, conv=2), right=delta(heads=1, kv_heads=1, conv=2))],
                                  loop=(0, 2, 2)),
    "one tap, no feed-forward anywhere": config([L_par(ff=False, left=attn(heads=2, kv_heads=1, dim=12, vdim=20, rot=6, conv=1),
                                                       right=delta(heads=3, kv_heads=3, dim=20, vdim=12, conv=1)),
                                                 L_attn(ff=False, heads=5, kv_heads=5, dim=10, vdim=14, rot=10, block=2), L_light(ff=False)],
                                                loop=(0, 2, 2), width=50, vocab=37),
    "equal sizes": config([L_attn(heads=2, kv_heads=2, dim=32, vdim=32, rot=32, block=32), L_light(heads=2, dim=32, vdim=32),
                           L_par(left=attn(heads=2, kv_heads=2, dim=32, vdim=32, rot=32, conv=4),
                                 right=delta(heads=2, kv_heads=2, dim=32, vdim=32, conv=4), ls=1.0, rs=1.0)],
                          loop=(0, 3, 1), width=32, vocab=32, scale=1.0),
    "nothing rotated, wide keys": config([L_attn(heads=6, kv_heads=2, dim=72, vdim=8, rot=0), L_light(heads=2, dim=80, vdim=40),
                                          L_par(left=attn(heads=2, kv_heads=1, dim=8, vdim=40, rot=2, block=3, conv=5),
                                                right=delta(heads=6, kv_heads=2, dim=136, vdim=8, conv=2))],
                                         loop=(2, 3, 2), eps=1e-3),
}


@pytest.mark.parametrize("name", sorted(OTHER))
def test_other_sizes(name):
    cfg = OTHER[name]
    model, W = build(cfg, seed=7)
    toks = tokens(75, cfg["vocab"], 6)
    ref = O.forward(cfg, W, toks)
    assert rel(run_alone(model, toks), ref) < TOL["float32"]
    assert rel(run_alone(model, toks, [40] + [1] * 35), ref) < TOL["float32"]
    assert rel(run_alone(model, toks, [7, 2, 66]), ref) < TOL["float32"]
    served, _ = build(cfg, "bfloat16", seed=7)
    assert rel(run_alone(served, toks, [40] + [1] * 35), ref) < TOL["bfloat16"]


# ------------------------------------------------------------------------------------------------ generation
def oracle_greedy(cfg, W, prompt, n):
    toks, margins = list(prompt), []
    for _ in range(n):
        z = O.forward(cfg, W, toks)[-1]
        top2 = torch.topk(z, 2).values
        margins.append(float(top2[0] - top2[1]))
        toks.append(int(torch.argmax(z)))
    return toks[len(prompt):], margins


def same_until_tie(got, want, margins, what):
    for i, (g, w) in enumerate(zip(got, want)):
        if margins[i] < 1e-3:
            return
        assert g == w, f"{what}: token {i} is {g}, the plain implementation says {w}"


def test_greedy_generate_step():
    from mlx_vlm_b200.generate import generate_step
    cfg = config()
    model, W = build(cfg)
    prompt = tokens(21, cfg["vocab"], 8)
    want, margins = oracle_greedy(cfg, W, prompt, 10)
    got = [t for t, _ in generate_step(np.asarray([prompt]), model, None, None, max_tokens=10)]
    same_until_tie(got, want, margins, "generate_step")
    from mlx_vlm_b200.sample_utils import make_sampler
    got = [t for t, _ in generate_step(np.asarray([prompt]), model, None, None, max_tokens=6,
                                       sampler=make_sampler(temp=0.0), logit_bias={0: 0.0})]
    same_until_tie(got, want[:6], margins, "generate_step with a sampler")


def test_batch_scheduler_lock_step_rows():
    from mlx_vlm_b200.generate_batch import BatchGenerator
    cfg = config()
    model, W = build(cfg)
    model.config.eos_token_id = []
    prompts = [tokens(n, cfg["vocab"], 60 + n) for n in (5, 30, 12, 44, 9)]
    n_new = [6, 9, 4, 7, 5]
    proc = types.SimpleNamespace(tokenizer=types.SimpleNamespace(stopping_criteria=None))
    g = BatchGenerator(model, proc, completion_batch_size=3, prefill_batch_size=2, decode_slice=2)
    uids = g.insert(prompts, n_new)
    out = {u: [] for u in uids}
    while g.has_work:
        for r in g.next()[1]:
            out[r.uid].append(r.token)
    for u, p, n in zip(uids, prompts, n_new):
        want, margins = oracle_greedy(cfg, W, p, n)
        assert len(out[u]) == n
        same_until_tie(out[u], want, margins, f"row {u}")


def test_trace_runner_from_a_checkpoint_folder(tmp_path):
    """bin/trace_run on a checkpoint folder: the registry picks the class from `architecture`, requests are prefilled
    together, decoded together, one ends and a later one takes its slot; both number formats"""
    import json
    import os
    import subprocess
    import sys
    from safetensors.torch import save_file
    cfg = config()
    W = O.random_weights(cfg, 11)
    model_dir = tmp_path / "model"
    model_dir.mkdir()
    (model_dir / "config.json").write_text(json.dumps(cfg))
    save_file({k: v.contiguous() for k, v in W.items()}, str(model_dir / "model.safetensors"))
    a, b, c = (tokens(n, cfg["vocab"], 70 + n) for n in (40, 9, 25))
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:30], "want": [0, 29]}, {"id": "b", "tokens": b[:8], "want": [7]}],
              "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[30:31], "want": [0]}, {"id": "b", "tokens": b[8:], "want": [0]}],
              "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": a[31:32], "want": []}], "end": []},
             {"step": 3, "entries": [{"id": "a", "tokens": a[32:], "want": [7]}, {"id": "c", "tokens": c, "want": [0, 24]}],
              "end": ["a", "c"]}]
    want = {0: [(a, 0), (a, 29), (b, 7)], 1: [(a, 30), (b, 8)], 3: [(a, 39), (c, 0), (c, 24)]}
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for dtype in ("bfloat16", "float32"):
        out = tmp_path / dtype
        r = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", str(model_dir), "--dtype", dtype,
                            "--out", str(out), "--max-tokens", "80"], input="".join(json.dumps(x) + "\n" for x in steps),
                           capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stderr[-2000:]
        assert [ln for ln in r.stdout.splitlines() if ln.startswith("done")] == [f"done {i}" for i in range(4)]
        assert not (out / "2.f32").exists()
        for st, rows in want.items():
            got = torch.from_numpy(np.fromfile(out / f"{st}.f32", dtype="<f4").reshape(len(rows), cfg["vocab"])).double()
            ref = torch.stack([O.forward(cfg, W, t)[i] for t, i in rows])
            assert rel(got, ref) < TOL[dtype]
