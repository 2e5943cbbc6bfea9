"""Buzopel on the GPU against the plain restatement in oracle/buzopel.py: every mechanism alone, whole prompts,
prefill against token-by-token decoding, portions, batches of unequal requests, slots that are released and used
again, pools that grow, keys far away and at the edges of the attention kernel's key tiles, long decoding, other
sizes, and greedy generation through generate_step and the batch scheduler.  Small random configurations; none of
them is a real model's."""
import copy
import types

import numpy as np
import pytest
import torch

from oracle import buzopel as O

pytestmark = pytest.mark.gpu


def layer(heads=3, dim=16, rot=8, vdim=24, kv_rank=40, q_rank=48, base=5000.0, kv_from=None, experts=5, top=2, ff=24,
          mlp=True):
    m = {"heads": heads, "dim": dim, "rot_dim": rot, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
         "rot": {"base": base, "dims": rot}, "scale": 1.0 / float(dim + rot) ** 0.5}
    if kv_from is not None:
        m["kv_from"] = kv_from
    f = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}} if mlp else None
    return {"type": "latent_attention", "mixer": m, "mlp": f}


def config(layers=None, width=96, vocab=101, scale=6.0, cap=9.0, eps=1e-5):
    layers = layers or [layer(), layer(), layer(kv_from=1), layer(mlp=False), layer(kv_from=3)]
    c = {"architecture": "Buzopel", "vocab": vocab, "width": width, "layers": layers, "embedding": {"scale": scale},
         "norm": {"eps": eps}}
    if cap:
        c["logit_softcap"] = cap
    return c


_MODELS = {}


def build(cfg, dtype="float32", seed=1):
    from mlx_vlm_b200.models.buzopel import Model, ModelConfig
    key = (repr(cfg), dtype, seed)
    if key not in _MODELS:
        W = O.random_weights(cfg, seed)
        _MODELS[key] = (Model(ModelConfig.from_dict(copy.deepcopy(cfg)), dtype=dtype).load_weights(W), W)
    return _MODELS[key]


def host(eng, t):
    eng.stream.synchronize()
    return t.detach().to("cpu", torch.float64)


def rel_rows(got, want):
    """per row: rms of the difference (mean over the row taken off) / rms of the reference"""
    d = got - want
    d = d - d.mean(-1, keepdim=True)
    return d.square().mean(-1).sqrt() / (want - want.mean(-1, keepdim=True)).square().mean(-1).sqrt()


def rel(got, want, dtype="float32"):
    """float32: the worst row.  bfloat16: the row at the 85th percentile — with random weights a few tokens sit
    on a close call of a router, and under bf16 rounding such a token takes another expert (a different, equally
    valid output); the exact mode has no such excuse and is held to every row."""
    e = rel_rows(got, want)
    return e.max().item() if dtype == "float32" else torch.quantile(e, 0.85).item()


TOL = {"float32": 3e-5, "bfloat16": 6e-2}


def tokens(n, vocab, seed=0):
    return np.random.default_rng(seed).integers(0, vocab, n).tolist()


def run_alone(model, toks, cuts=None, want_all=True):
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
def _ops():
    from mlx_vlm_b200.layer_engine import LayerEngine
    if "eng" not in _MODELS:
        _MODELS["eng"] = LayerEngine("cuda:0", exact=True)
    return _MODELS["eng"]


def dev(a, dtype=torch.float32):
    return torch.as_tensor(a).to(device="cuda:0", dtype=dtype).contiguous()


@pytest.mark.parametrize("n", [7, 96, 1000])
def test_norm_rows(n):
    eng = _ops()
    g = torch.Generator().manual_seed(n)
    y = torch.randn(5, n, generator=g) * 3
    w = (torch.randn(n, generator=g) * 0.2).bfloat16()
    x0 = torch.randn(5, n, generator=g)
    for off, ref in ((1.0, O.norm_offset), (0.0, O.norm_plain)):
        x = dev(x0)
        eng.ops.norm_rows(dev(y), dev(w, torch.bfloat16), 1e-5, x, w_offset=off, add=True)
        want = x0.double() + ref(y.double(), w.double(), 1e-5)
        assert (host(eng, x) - want).abs().max() < 1e-5
    # the weighted sum of `top` rows per token, then the norm; and a gathered row list without the add
    top, wg = 3, torch.rand(5, 3, generator=g)
    rows = torch.randn(15, n, generator=g)
    x = dev(x0)
    eng.ops.norm_rows(dev(rows), dev(w, torch.bfloat16), 1e-5, x, w_offset=1.0, add=True, combine=dev(wg), top=top)
    comb = (rows.view(5, top, n).double() * wg.double()[:, :, None]).sum(1)
    assert (host(eng, x) - (x0.double() + O.norm_offset(comb, w.double(), 1e-5))).abs().max() < 1e-5
    out = dev(torch.zeros(2, n))
    eng.ops.norm_rows(dev(y), dev(w, torch.bfloat16), 1e-5, out, w_offset=1.0, rows=dev([4, 1], torch.int32))
    assert (host(eng, out) - O.norm_offset(y[[4, 1]].double(), w.double(), 1e-5)).abs().max() < 1e-5


@pytest.mark.parametrize("dims,base", [(8, 5000.0), (2, 10.0), (64, 250000.0)])
def test_rotation_far_positions(dims, base):
    """rotate-half at positions up to 100k: the angle must not lose precision"""
    eng = _ops()
    pos = torch.tensor([0, 1, 2, 31, 32, 1023, 4097, 99999], dtype=torch.int32)
    T, q_rank, kv_rank = pos.shape[0], 4, 6
    g = torch.Generator().manual_seed(dims)
    D = torch.randn(T, q_rank + kv_rank + dims, generator=g)
    one = dev(torch.ones(64), torch.bfloat16)
    cache = dev(torch.zeros(1, 100000, kv_rank + dims))
    cs = eng.ops.rope_table(dev(pos, torch.int32), base, dims)
    cq = dev(torch.zeros(T, q_rank))
    eng.ops.latent_post(dev(D), one, one, 1e-5, cq, cache, dev(torch.zeros(T), torch.int32), dev(pos, torch.int32), cs,
                        q_rank, kv_rank, dims, dims)
    got = host(eng, cache[0][pos.long()])
    want_r = O.rotate_half(D[:, q_rank + kv_rank:].double(), pos, base, dims)
    assert (got[:, kv_rank:] - want_r).abs().max() < 2e-6
    assert (got[:, :kv_rank] - O.rms(D[:, q_rank:q_rank + kv_rank].double(), 1e-5)).abs().max() < 2e-6
    assert (host(eng, cq) - O.rms(D[:, :q_rank].double(), 1e-5)).abs().max() < 2e-6


@pytest.mark.parametrize("E,top", [(5, 2), (1, 1), (7, 7), (70, 4)])
def test_router(E, top):
    eng = _ops()
    g = torch.Generator().manual_seed(E)
    h = torch.randn(33, 20, generator=g)
    Wr, b = (torch.randn(E, 20, generator=g)).bfloat16(), torch.randn(E, generator=g).bfloat16()
    z = eng.ops.linear(dev(h), dev(Wr, torch.bfloat16), bias=dev(b, torch.bfloat16))
    idx, wgt = eng.ops.router_topk(z, top)
    ridx, rw = O.router(h.double(), Wr.double(), b.double(), top)
    eng.stream.synchronize()
    assert torch.equal(idx.cpu().long(), ridx)
    assert (wgt.cpu().double() - rw).abs().max() < 1e-6
    lists, count = eng.ops.moe_group(idx, E)
    eng.stream.synchronize()
    flat = ridx.reshape(-1)
    for e in range(E):
        assert lists[e, :int(count[e])].cpu().tolist() == (flat == e).nonzero().flatten().tolist()


def test_router_tie_takes_lowest_index():
    eng = _ops()
    z = dev([[1.0, 3.0, 3.0, 0.0, 3.0]])
    idx, wgt = eng.ops.router_topk(z, 2)
    eng.stream.synchronize()
    assert idx.cpu().tolist() == [[1, 2]] and (wgt.cpu() - 0.5).abs().max() < 1e-7


@pytest.mark.parametrize("T", [1, 9, 70])
def test_expert_mixture(T):
    from mlx_vlm_b200.models.decoder_blocks import ExpertMixture, StepCtx
    eng = _ops()
    f = {"kind": "moe", "router": {"experts": 6, "top": 3}, "expert": {"ff": 20}}
    g = torch.Generator().manual_seed(T)
    W = {"router": torch.randn(6, 36, generator=g).bfloat16(), "router.b": torch.randn(6, generator=g).bfloat16()}
    for e in range(6):
        W[f"e{e}.up"] = (torch.randn(20, 36, generator=g) / 6).bfloat16()
        W[f"e{e}.down"] = (torch.randn(36, 20, generator=g) / 4).bfloat16()
    mix = ExpertMixture(0, f, 36)
    store = {n: dev(torch.zeros(s), torch.bfloat16) for n, s in mix.manifest("")}
    mix.pack("", {k: dev(v, torch.bfloat16) for k, v in W.items()}, store.__getitem__)
    h = torch.randn(T, 36, generator=g)
    rows, wgt = mix.forward(StepCtx(eng.ops, None, None, None, 1e-5), dev(h))
    got = (host(eng, rows).view(T, 3, 36) * host(eng, wgt)[:, :, None]).sum(1)
    want = O.moe(h.double(), {k: v.double() for k, v in W.items()}, "", f)
    assert (got - want).abs().max() < 1e-5


@pytest.mark.parametrize("M,N,K,batch", [(1, 5, 7, 1), (16, 130, 33, 1), (17, 64, 64, 1), (150, 70, 100, 3), (3, 9, 40, 4)])
def test_row_gemm_both_kernels(M, N, K, batch):
    eng = _ops()
    g = torch.Generator().manual_seed(M * N)
    X, W = torch.randn(batch, M, K, generator=g), torch.randn(batch, N, K, generator=g).bfloat16()
    Y = dev(torch.zeros(batch, M, N))
    eng.ops.gemm(dev(X), dev(W, torch.bfloat16), Y, M=M, N_=N, K=K, ldx=K, xb=M * K, wb=N * K, ldy=N, yb=M * N, batch=batch)
    want = torch.einsum("bmk,bnk->bmn", X.double(), W.double())
    assert (host(eng, Y) - want).abs().max() < 1e-4


def test_grouped_tensor_core_gemm_over_padded_segments():
    """entries sorted by expert into segments padded to whole tiles; an expert with several tiles, one with a partial
    tile, one with none; every row against a plain product with its own expert's weights"""
    from mlx_vlm_b200.layer_engine import LayerEngine
    if "eng16" not in _MODELS:
        _MODELS["eng16"] = LayerEngine("cuda:0", exact=False)
    eng = _MODELS["eng16"]
    ops = eng.ops
    E, K, N_, top = 4, 72, 40, 1
    g = torch.Generator().manual_seed(8)
    counts = [300, 0, 130, 5]
    idx = torch.cat([torch.full((c,), e) for e, c in enumerate(counts)])[torch.randperm(sum(counts), generator=g)]
    T = idx.shape[0]
    x = torch.randn(T, K, generator=g)
    W = (torch.randn(E, N_, K, generator=g) / 8).bfloat16()
    lists, count = ops.moe_group(dev(idx.view(T, 1), torch.int32), E)
    order, group = ops.moe_tiles(lists, count, T)
    xs = ops.to_bf16(dev(x), K, rows=order.shape[0], row_map=order, div=top)
    ys = ops.empty((order.shape[0], N_))
    ops.tc_gemm_grouped(xs, dev(W, torch.bfloat16), ys, group, N_=N_, K=K, n_groups=E)
    out = ops.empty((T, N_))
    ops.rows_scatter(ys, order, out, order.shape[0])
    eng.stream.synchronize()
    assert group.cpu().tolist()[:6] == [0, 0, 0, 2, 2, 3] and set(group.cpu().tolist()[6:]) <= {-1}
    want = torch.einsum("tk,tnk->tn", x.bfloat16().double(), W.double()[idx])
    assert (host(eng, out) - want).abs().max() < 2e-3


def _attend(eng, cache, q, slot, pos, H, r, scale):
    out = dev(torch.zeros(q.shape[0], H * r))
    eng.ops.latent_attention(dev(q), cache, dev(slot, torch.int32), dev(pos, torch.int32), out, H, r, scale)
    return host(eng, out).view(q.shape[0], H, r)


@pytest.mark.parametrize("r,dr", [(12, 4), (13, 2)])
def test_attention_far_key_and_tile_edges(r, dr):
    """the kernel stages keys 32 at a time: a key that stands out is found wherever it lies (first row, last of a
    tile, first of the next, far back among hundreds), the row just past the query's position is never seen, and
    the result matches a plain softmax"""
    eng = _ops()
    H, S = 2, 700          # rows of 16 numbers (128-bit shared loads) and of 15 (the scalar path)
    g = torch.Generator().manual_seed(3)
    rows = torch.nn.functional.normalize(torch.randn(2, S, r + dr, generator=g), dim=-1)   # a row's best match is itself
    cache = dev(rows)
    for key in (0, 31, 32, 33, 63, 64, 350, 698):
        for qpos in (key, key + 1, 699):
            q = torch.randn(1, H, r + dr, generator=g) * 0.3
            q[0, 1] = rows[1, key] * 120.0                       # head 1 points at row `key` of slot 1
            got = _attend(eng, cache, q.view(1, -1), [1], [qpos], H, r, 1.0)
            s = torch.einsum("hd,jd->hj", q[0].double(), rows[1, :qpos + 1].double())
            want = torch.softmax(s, -1) @ rows[1, :qpos + 1, :r].double()
            assert (got[0] - want).abs().max() < 1e-5
            assert (got[0, 1] - rows[1, key, :r].double()).abs().max() < 1e-3   # head 1 returns that row's latent
    # a row that stands out but lies one past the query's position must not be seen
    q = torch.zeros(1, H, r + dr)
    q[0, :] = rows[0, 40] * 120.0
    got = _attend(eng, cache, q.view(1, -1), [0], [39], H, r, 1.0)
    want = torch.softmax(torch.einsum("hd,jd->hj", q[0].double(), rows[0, :40].double()), -1) @ rows[0, :40, :r].double()
    assert (got[0] - want).abs().max() < 1e-5 and (got[0, 0] - rows[0, 40, :r].double()).abs().max() > 0.05


# ------------------------------------------------------------------------------------------------ the model
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_prompt_and_every_layer(dtype):
    cfg = config()
    model, W = build(cfg, dtype)
    toks = tokens(150, cfg["vocab"], 1)
    layers_ref = []
    ref = O.forward(cfg, W, toks, torch.float64, layers_ref)
    assert rel(run_alone(model, toks), ref, dtype) < TOL[dtype]
    if dtype == "float32":      # the residual stream after every layer
        from mlx_vlm_b200.models.decoder_blocks import StepCtx
        eng, lm = model.engine, model.language_model
        pool = lm.make_pool(1, 256)
        T = len(toks)
        ctx = StepCtx(eng.ops, dev(torch.zeros(T), torch.int32), dev(torch.arange(T), torch.int32), pool, model.eps)
        x = eng.ops.embed(dev(toks, torch.int32), model.embed, model.embed_scale)
        for L, want in zip(model.layers, layers_ref):
            L.forward(ctx, x)
            assert (host(eng, x) - want).abs().max() < 2e-4


def test_first_tokens():
    cfg = config()
    model, W = build(cfg)
    for n in (1, 2, 3):
        toks = tokens(n, cfg["vocab"], 10 + n)
        assert rel(run_alone(model, toks), O.forward(cfg, W, toks)) < TOL["float32"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prefill_then_token_by_token(dtype):
    cfg = config()
    model, W = build(cfg, dtype)
    toks = tokens(90, cfg["vocab"], 2)
    ref = O.forward(cfg, W, toks)
    got = run_alone(model, toks, [50] + [1] * 40)
    assert rel(got, ref, dtype) < TOL[dtype]
    if dtype == "float32":       # decoding gives what one pass gives, up to the order of the sums
        assert rel(got, run_alone(model, toks)) < TOL[dtype]


@pytest.mark.parametrize("cuts", [[2] * 35, [3, 64, 3], [31, 1, 32, 6], [33, 2, 35], [69, 1]])
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
    first = host(eng, lm.step([r[:n] for r, n in zip(reqs, lens)], caches,
                              want=[list(range(n)) for n in lens]))
    got = list(torch.split(first, lens))
    for k in range(12):                              # then all go on by one token, together
        step = host(eng, lm.step([[r[n + k]] for r, n in zip(reqs, lens)], caches))
        got = [torch.cat([g, step[i:i + 1]]) for i, g in enumerate(got)]
    for g, r in zip(got, reqs):
        assert rel(g, O.forward(cfg, W, r), dtype) < TOL[dtype]
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
    table.release("b")                                   # b is finished; c takes its slot while a goes on
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
    got = host(eng, lm.step([[a[0]], d], [ca, cd], want=[[], list(range(50))]))    # a's cache survived the move
    assert rel(got, O.forward(cfg, W, d)) < TOL["float32"]
    got = host(eng, lm.step([[5]], [cc]))
    assert rel(got, O.forward(cfg, W, c + [5])[-1:]) < TOL["float32"]


def test_long_prompt_paths_of_the_serving_mode():
    """prompts of 128 tokens and more take the tensor-core products (projections, attention against the cached
    rows, experts over sorted segments): a long portion after a cached prefix, experts that get one or two tokens
    or none, sizes that are multiples of 8 but not of 64, a batch whose short member stays on the row kernels"""
    cfg = config([layer(heads=3, dim=24, rot=8, vdim=16, kv_rank=40, q_rank=56, experts=48, top=1, ff=40),
                  layer(heads=3, dim=24, rot=8, vdim=16, kv_rank=40, q_rank=56, experts=3, top=2, ff=24, kv_from=0)],
                 width=72, vocab=90)
    model, W = build(cfg, "bfloat16", seed=4)
    exact, _ = build(cfg, "float32", seed=4)
    lm, eng = model.language_model, model.engine
    toks = tokens(330, cfg["vocab"], 9)
    ref = O.forward(cfg, W, toks)
    got = run_alone(model, toks, [140, 150, 40])
    assert rel(got, ref, "bfloat16") < TOL["bfloat16"]
    assert rel(run_alone(exact, toks, [140, 150, 40]), ref) < TOL["float32"]
    pool = lm.make_pool(2, 512)
    ca, cb = lm.make_cache_row(pool, 0), lm.make_cache_row(pool, 1)
    both = host(eng, lm.step([toks[:200], toks[:30]], [ca, cb], want=[list(range(200)), list(range(30))]))
    assert rel(both[:200], ref[:200], "bfloat16") < TOL["bfloat16"] and rel(both[200:], ref[:30], "bfloat16") < TOL["bfloat16"]


def test_row_kernels_take_over_when_the_tensor_core_gemm_refuses():
    """a product whose arguments the tcgen05 GEMM rejects (its checks run before any launch) is redone on the row
    kernels and the tensor-core path stays off: same logits within the serving mode's noise"""
    from mlx_vlm_b200 import _native
    cfg = config([layer(), layer(kv_from=0)])
    model, W = build(cfg, "bfloat16", seed=5)
    ops = model.engine.ops
    toks = tokens(160, cfg["vocab"], 12)
    ref = O.forward(cfg, W, toks)
    real, calls = ops.tc_gemm, []

    def refuse(*a, **k):
        calls.append(1)
        raise _native.B200Error("refused for the test")

    ops.tc_gemm = refuse
    try:
        got = run_alone(model, toks)
    finally:
        ops.tc_gemm = real
    assert calls and not ops.tc_enabled
    assert rel(got, ref, "bfloat16") < TOL["bfloat16"]
    ops.tc_enabled = True
    assert rel(run_alone(model, toks), ref, "bfloat16") < TOL["bfloat16"]


def test_long_decoding():
    cfg = config(layers=[layer(), layer(kv_from=0)])
    model, W = build(cfg)
    toks = tokens(420, cfg["vocab"], 5)
    got = run_alone(model, toks, [20] + [1] * 400)
    assert rel(got, O.forward(cfg, W, toks)) < TOL["float32"]


OTHER = {
    "one head, one expert": config([layer(heads=1, experts=1, top=1), layer(heads=1, kv_from=0, experts=2, top=2)]),
    "wide heads, small rotation": config([layer(heads=9, dim=8, rot=2, vdim=5, kv_rank=70, q_rank=11, ff=50)], width=40,
                                         vocab=33, scale=1.0, cap=None),
    "layers of different sizes": config([layer(kv_rank=40, rot=8), layer(kv_rank=24, rot=16, heads=2, base=100.0),
                                         layer(kv_from=0), layer(kv_from=1, heads=2, kv_rank=24, rot=16, base=100.0,
                                                                 mlp=False)], eps=1e-3),
    "nothing rotated": config([layer(rot=0), layer(rot=0, kv_from=0)]),
    "equal sizes": config([layer(heads=2, dim=32, rot=32, vdim=32, kv_rank=32, q_rank=32, experts=4, top=4, ff=32)],
                          width=32, vocab=32),
}


@pytest.mark.parametrize("name", sorted(OTHER))
def test_other_sizes(name):
    cfg = OTHER[name]
    model, W = build(cfg, seed=7)
    toks = tokens(75, cfg["vocab"], 6)
    ref = O.forward(cfg, W, toks)
    assert rel(run_alone(model, toks), ref) < TOL["float32"]
    assert rel(run_alone(model, toks, [40] + [1] * 35), ref) < TOL["float32"]


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
    # the sampler path (temperature 0 through an explicit sampler reads the logits on the host side of the loop)
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
    """bin/trace_run on a checkpoint folder (config.json + model.safetensors, bf16 tensors with the design's names):
    the registry picks the class from `architecture`, requests are prefilled together, decoded together, one ends
    and a later one takes its slot; both number formats against the plain restatement"""
    import json
    import os
    import subprocess
    import sys
    from safetensors.torch import save_file
    cfg = config([layer(), layer(kv_from=0), layer(mlp=False)])
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
            assert rel(got, ref, dtype) < TOL[dtype]
