"""Host-side parts of the Sonulorn integration (no GPU): configuration, registry, the order of layer runs, the packed
layout of a shared-input layer, the state pool and its cache views on CPU tensors, and sanity properties of the plain
restatement the GPU tests compare with."""
import pytest
import torch

from oracle import sonulorn as O


def attn(block=None, conv=None, **kw):
    m = {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 6, "rot": {"base": 100.0, "dims": 4}, "scale": 0.3}
    m.update(kw)
    if block:
        m["mask"] = {"size": block}
    if conv:
        m["conv"] = conv
    return m


def delta(**kw):
    m = {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 6, "conv": 3}
    m.update(kw)
    return m


MLP = {"kind": "dense", "ff": 12, "limit": 2.0}


def layers():
    return [{"type": "parallel", "mlp": MLP, "mixer": {"left": attn(conv=2), "left_scale": 0.9, "right": delta(), "right_scale": 0.4}},
            {"type": "lightning", "mlp": None, "mixer": {"heads": 2, "dim": 8, "vdim": 10, "decay": [0.9, 0.99]}},
            {"type": "attention", "mlp": MLP, "mixer": attn(block=5)}]


def config(loop=(0, 2, 3)):
    c = {"architecture": "Sonulorn", "vocab": 29, "width": 20, "embedding": {"scale": 3.0}, "norm": {"eps": 1e-5},
         "layers": layers()}
    if loop:
        c["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return c


def test_config_registry_and_run_order():
    from mlx_vlm_b200.models.sonulorn import ModelConfig
    from mlx_vlm_b200.utils import get_model_and_args
    c = ModelConfig.from_dict(config())
    assert (c.vocab, c.width, c.embedding_scale, c.norm_eps) == (29, 20, 3.0, 1e-5)
    assert ModelConfig.from_dict(c.to_dict()).to_dict() == c.to_dict()
    arch, name = get_model_and_args(config())
    assert name == "sonulorn" and hasattr(arch, "Model")
    assert c.layer_runs() == [(0, 0, True), (1, 0, False), (0, 1, True), (1, 1, False), (0, 2, True), (1, 2, False),
                              (2, None, False)]
    assert c.layer_runs() == O.layer_runs(config()) and c.num_hidden_layers == 7
    late = ModelConfig.from_dict(config(loop=(1, 3, 2)))
    assert [r[0] for r in late.layer_runs()] == [0, 1, 2, 1, 2] and [r[2] for r in late.layer_runs()] == [False, True, False, True, False]
    assert [r[0] for r in ModelConfig.from_dict(config(loop=None)).layer_runs()] == [0, 1, 2]
    for bad in ((2, 2, 1), (0, 4, 2), (0, 2, 0)):
        with pytest.raises(ValueError):
            ModelConfig.from_dict(config(loop=bad))
    with pytest.raises(ValueError):
        ModelConfig.from_dict({"vocab": 3})


def test_model_layout_matches_the_checkpoint_names():
    from mlx_vlm_b200.models.sonulorn import Model, ModelConfig
    cfg = config()
    m = Model(ModelConfig.from_dict(cfg), device="cpu")       # no engine is made until something runs
    assert m.checkpoint_tensors() == O.tensor_shapes(cfg)
    L0, L1, L2 = m.layers
    # one stacked input projection and one side-by-side output projection per layer
    names = dict(L0.manifest("l0."))
    n_left, n_right = 32 + 16 + 12 + 4, 16 + 16 + 24 + 4 + 4 + 24
    assert names["l0.in"] == (n_left + n_right + 24, 20) and names["l0.out"] == (20, 24 + 24 + 12)
    assert names["l0.mix.left.conv"] == (60, 2) and names["l0.mix.right.conv"] == (56, 3) and names["l0.mix.right.norm"] == (6,)
    assert dict(L1.manifest("l1."))["l1.out"] == (20, 20) and dict(L2.manifest("l2."))["l2.in"] == (32 + 16 + 12 + 24 + 24, 20)
    # every run has its own cache rows and state: 3 runs of the pair, then the last layer
    assert [(r.layer, r.repetition, r.kv_base) for r in m.runs] == [(0, 0, 0), (1, 0, 1), (0, 1, 1), (1, 1, 2), (0, 2, 2),
                                                                    (1, 2, 3), (2, None, 3)]
    assert m.n_cache_layers == 4 and m.row_dim == 28
    s0 = 1 * 60 + 2 * 56 + 4 * 8 * 6 * 1
    s1 = 2 * 8 * 10 * 1
    assert (L0.state_floats, L1.state_floats, L2.state_floats) == (s0, s1, 0)
    assert [r.state_base for r in m.runs] == [0, s0, s0 + s1, 2 * s0 + s1, 2 * (s0 + s1), 3 * s0 + 2 * s1, 3 * (s0 + s1)]
    assert m.state_floats == 3 * (s0 + s1)
    from mlx_vlm_b200.models.decoder_blocks import SharedInputLayer, state_lanes
    assert [state_lanes(d) for d in (1, 8, 9, 16, 17, 64, 65, 128, 129, 256)] == [1, 1, 2, 2, 4, 8, 16, 16, 32, 32]
    with pytest.raises(ValueError):
        state_lanes(257)
    with pytest.raises(ValueError):
        SharedInputLayer(0, {"type": "other", "mixer": {}}, 20)
    with pytest.raises(ValueError):
        SharedInputLayer(0, {"type": "attention", "mixer": attn(heads=3), "mlp": None}, 20)
    with pytest.raises(ValueError):
        SharedInputLayer(0, {"type": "attention", "mixer": attn(), "mlp": {"kind": "other"}}, 20)


def test_packing_stacks_the_projections():
    from mlx_vlm_b200.models.decoder_blocks import SharedInputLayer
    cfg = config()
    W = O.random_weights(cfg, 2)
    L = SharedInputLayer(0, cfg["layers"][0], 20)
    store = {n: torch.zeros(s, dtype=torch.bfloat16) for n, s in L.manifest("l0.")}
    L.pack("l0.", W, store.__getitem__)
    rows = [W["l0.mix.left." + n] for n in "qkvg"] + [W["l0.mix.right." + n] for n in "qkvbag"] + [W["l0.mlp.gate"], W["l0.mlp.up"]]
    assert torch.equal(store["l0.in"], torch.cat(rows))
    assert torch.equal(store["l0.out"], torch.cat([W["l0.mix.left.o"], W["l0.mix.right.o"], W["l0.mlp.down"]], dim=1))
    assert torch.equal(store["l0.mix.right.conv"], torch.cat([W["l0.mix.right." + n + ".conv"] for n in "qkv"]))
    assert L.parts[0][1].w["sink"] is store["l0.mix.left.sink"] and L.w["in"] is store["l0.in"]


def test_state_pool_and_cache_views():
    from mlx_vlm_b200.models.cache import RunCache, StatePool
    pool = StatePool(2, 6, 9, "cpu", batch=2, capacity=10, dtype=torch.float32)
    assert pool.buf.shape == (2, 2, 256, 6) and pool.state.shape == (2, 9) and pool.state.dtype == torch.float32
    pool.buf[1, 1, :5] = torch.arange(30.0).view(5, 6)
    pool.state[1] = torch.arange(9.0)
    assert pool.reserve(300, live_tokens=5) and pool.capacity == 512 and pool.buf[1, 1, 4, 5] == 29 and pool.state[1, 8] == 8
    assert pool.add_slots(5, live_tokens=5) and pool.buf.shape == (2, 5, 512, 6) and pool.state.shape == (5, 9)
    assert pool.buf[1, 1, 4, 5] == 29 and pool.state[1, 8] == 8 and pool.state[4].abs().sum() == 0
    pool.copy_slot(4, pool, 1, 5)
    assert torch.equal(pool.buf[:, 4, :5], pool.buf[:, 1, :5]) and torch.equal(pool.state[4], pool.state[1])
    both = RunCache(pool, 1, kv_layer=1, kv_dim=4, state_off=2, state_len=3)
    both.offset = 5
    k, s = both.state
    assert k.shape == (1, 5, 4) and s.tolist() == [2.0, 3.0, 4.0] and not both.is_trimmable() and both.trim(2) == 0
    rows_only = RunCache(pool, 1, kv_layer=0, kv_dim=6)
    rows_only.offset = 5
    assert rows_only.is_trimmable() and rows_only.trim(2) == 2 and rows_only.size() == 3 and rows_only.recurrent is None
    state_only = RunCache(pool, 1, state_off=0, state_len=9)
    assert state_only.keys is None and state_only.nbytes == 36 and state_only.empty()
    empty = StatePool(0, 0, 0, "cpu", batch=1, capacity=4)      # a design without attention or without state still has buffers
    assert empty.buf.numel() > 0 and empty.state.numel() > 0


# ---- the plain restatement itself ---------------------------------------------------------------------------
def test_restatement_is_causal_and_blocks_hide_earlier_keys():
    cfg = config()
    W = O.random_weights(cfg, 3)
    toks = [3, 1, 4, 1, 5, 9, 2, 6, 5, 3, 5, 8]
    full = O.forward(cfg, W, toks)
    assert torch.allclose(O.forward(cfg, W, toks[:7]), full[:7], atol=1e-10)
    ok = O.visible(12, 5)
    assert ok[4, 0] and not ok[5, 4] and ok[9, 5] and not ok[10, 9] and not ok[3, 4] and O.visible(3, None).sum() == 6
    # the sink only shrinks the weights; a very low sink is no sink
    g = torch.Generator().manual_seed(1)
    q, k, v = (torch.randn(6, 2, 4, generator=g, dtype=torch.float64) for _ in range(3))
    low = O.sink_softmax_attention(q, k, v, 0.5, torch.tensor([-1e9, -1e9]))
    plain = torch.stack([torch.softmax((q[:, h] @ k[:, h].T * 0.5).masked_fill(~O.visible(6, None), -1e30), -1) @ v[:, h]
                         for h in range(2)], 1)
    assert torch.allclose(low, plain, atol=1e-12)
    high = O.sink_softmax_attention(q, k, v, 0.5, torch.tensor([30.0, -1e9]))
    assert high[:, 0].abs().max() < 1e-6 and torch.allclose(high[:, 1], plain[:, 1])


def test_restatement_pieces():
    g = torch.Generator().manual_seed(0)
    u = torch.randn(9, 3, generator=g, dtype=torch.float64)
    w = torch.randn(3, 4, generator=g, dtype=torch.float64)
    y = O.short_conv(u, w)
    assert torch.allclose(y[0], w[:, 3] * u[0]) and torch.allclose(y[5], sum(w[:, j] * u[2 + j] for j in range(4)))
    assert torch.allclose(O.short_conv(u, w[:, 3:]), w[:, 3] * u)
    # the delta rule with beta = 1, no decay and orthonormal keys stores and returns each value exactly
    k = torch.eye(4, dtype=torch.float64)[:, None, :]
    v = torch.randn(4, 1, 5, generator=g, dtype=torch.float64)
    one = torch.ones(4, 1, dtype=torch.float64)
    assert torch.allclose(O.delta_rule(k, k, v, one, one), v)
    again = O.delta_rule(torch.cat([k, k]), torch.cat([k, k]), torch.cat([v, -v]), torch.ones(8, 1, dtype=torch.float64),
                         torch.ones(8, 1, dtype=torch.float64))
    assert torch.allclose(again[4:], -v)                     # a key written again replaces its value
    # the decayed state of one key is a geometric sum
    q1 = torch.ones(5, 1, 1, dtype=torch.float64)
    out = O.decayed_state(q1, q1, q1, torch.tensor([0.5], dtype=torch.float64))
    assert torch.allclose(out.flatten(), torch.tensor([1, 1.5, 1.75, 1.875, 1.9375], dtype=torch.float64))
    r = O.rotate_half(torch.randn(3, 2, 8, generator=g, dtype=torch.float64), torch.tensor([0, 1, 7]), 100.0, 0)
    assert r.shape == (3, 2, 8)
    n = torch.randn(4, 20, generator=g, dtype=torch.float64) * 4
    W = {"gate": torch.randn(12, 20, generator=g, dtype=torch.float64), "up": torch.randn(12, 20, generator=g, dtype=torch.float64),
         "down": torch.eye(12, dtype=torch.float64)}
    y = O.clamped_glu(n, W, "", MLP)
    assert y.max() <= 2.0 * 1.0 * 3.0 + 1e-9                 # g <= limit, sigmoid <= 1, u + 1 <= limit + 1
