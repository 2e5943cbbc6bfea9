"""Host-side parts of the Buzopel integration (no GPU): configuration, registry, block layout, the latent pool
and its slot table on CPU tensors, and sanity properties of the plain restatement the GPU tests compare with."""
import pytest
import torch

from oracle import buzopel as O


def layer(kv_from=None, mlp=True, **kw):
    m = {"heads": 2, "dim": 8, "rot_dim": 4, "vdim": 6, "kv_rank": 10, "q_rank": 12,
         "rot": {"base": 100.0, "dims": 4}, "scale": 0.3}
    m.update(kw)
    if kv_from is not None:
        m["kv_from"] = kv_from
    f = {"kind": "moe", "router": {"experts": 4, "top": 2}, "expert": {"ff": 6}} if mlp else None
    return {"type": "latent_attention", "mixer": m, "mlp": f}


def config(layers=None):
    return {"architecture": "Buzopel", "vocab": 29, "width": 20, "embedding": {"scale": 3.0}, "norm": {"eps": 1e-5},
            "logit_softcap": 7.0, "layers": layers or [layer(), layer(kv_from=0), layer(mlp=False)]}


def test_config_and_registry():
    from mlx_vlm_b200.models.buzopel import ModelConfig
    from mlx_vlm_b200.utils import get_model_and_args
    c = ModelConfig.from_dict(config())
    assert (c.vocab, c.width, c.embedding_scale, c.norm_eps, c.logit_softcap) == (29, 20, 3.0, 1e-5, 7.0)
    assert ModelConfig.from_dict(c.to_dict()).to_dict() == c.to_dict()
    arch, name = get_model_and_args(config())           # no model_type: the architecture names the class
    assert name == "buzopel" and hasattr(arch, "Model")
    with pytest.raises(ValueError):
        ModelConfig.from_dict({"vocab": 3})
    with pytest.raises(ValueError):
        get_model_and_args({})


def test_block_layout_and_borrowed_latents():
    from mlx_vlm_b200.models.decoder_blocks import PostNormLayer, assign_cache_layers
    layers = [PostNormLayer(i, c, 20) for i, c in enumerate(config()["layers"])]
    assert assign_cache_layers(layers) == 2
    assert [L.mixer.cache_index for L in layers] == [0, 0, 1]
    names = dict(layers[0].manifest("l0."))
    assert names["l0.mix.down"] == (12 + 10 + 4, 20) and names["l0.mix.ukT"] == (2, 10, 8)
    assert names["l0.mlp.up"] == (4, 6, 20) and names["l0.mlp.down"] == (4, 20, 6)
    assert dict(layers[1].manifest("l1."))["l1.mix.down"] == (12, 20)      # a borrowing layer has no kv projection
    assert "l2.norm2" not in dict(layers[2].manifest("l2."))
    for bad in ([layer(kv_from=1), layer()], [layer(), layer(kv_from=0, kv_rank=12)], [layer(), layer(kv_from=0), layer(kv_from=1)]):
        with pytest.raises(ValueError):
            assign_cache_layers([PostNormLayer(i, c, 20) for i, c in enumerate(bad)])
    with pytest.raises(ValueError):
        PostNormLayer(0, {"type": "other", "mixer": {}}, 20)


def test_slot_table():
    from mlx_vlm_b200.models.cache import SlotTable
    t = SlotTable(2)
    assert t.acquire("a") == 0 and t.acquire("b") == 1 and t.free == 0
    with pytest.raises(RuntimeError):
        t.acquire("c")
    with pytest.raises(KeyError):
        t.acquire("a")
    assert t.release("a") == 0 and "a" not in t and "b" in t
    assert t.acquire("c") == 0                       # the released slot is used again
    t.grow(4)
    assert t.acquire("d") == 2 and t.slot_of("d") == 2 and len(t) == 3


def test_latent_pool_and_cache_views():
    from mlx_vlm_b200.models.cache import LatentCache, LatentPool
    pool = LatentPool(2, 6, "cpu", batch=2, capacity=10, dtype=torch.float32)
    assert pool.buf.shape == (2, 2, 256, 6)
    pool.buf[1, 1, :5] = torch.arange(30.0).view(5, 6)
    assert pool.reserve(300, live_tokens=5) and pool.capacity == 512 and pool.buf[1, 1, 4, 5] == 29
    assert pool.add_slots(5, live_tokens=5) and pool.buf.shape == (2, 5, 512, 6) and pool.buf[1, 1, 4, 5] == 29
    pool.copy_slot(4, pool, 1, 5)
    assert torch.equal(pool.buf[:, 4, :5], pool.buf[:, 1, :5])
    own, shared = LatentCache(pool, 1, 1, latent_dim=4), LatentCache(pool, 1, 1, latent_dim=4, shared=True)
    own.offset = 5
    k, v = own.state
    assert k.shape == (1, 5, 6) and v.shape == (1, 5, 4) and own.trim(2) == 2 and own.size() == 3
    assert shared.nbytes == 0 and own.nbytes > 0 and own.is_trimmable()


# ---- the plain restatement itself ---------------------------------------------------------------------------
def test_restatement_is_causal_and_borrowing_reads_the_source_latent():
    cfg = config()
    W = O.random_weights(cfg, 3)
    toks = [3, 1, 4, 1, 5, 9, 2, 6, 5, 3, 5]
    full = O.forward(cfg, W, toks)
    assert torch.allclose(O.forward(cfg, W, toks[:6]), full[:6], atol=1e-10)
    # layer 1 borrows layer 0's latent: giving it its own copy of layer 0's projection AFTER layer 0 changed x differs
    own = config([layer(), layer(), layer(mlp=False)])
    W2 = dict(W)
    W2["l1.mix.dkv"], W2["l1.mix.dkv.norm"] = W["l0.mix.dkv"], W["l0.mix.dkv.norm"]
    assert not torch.allclose(O.forward(own, W2, toks), full, atol=1e-6)


def test_restatement_pieces():
    g = torch.Generator().manual_seed(0)
    v = torch.randn(5, 8, generator=g, dtype=torch.float64)
    pos = torch.tensor([0, 1, 7, 100, 5000])
    r = O.rotate_half(v, pos, 100.0, 6)
    assert torch.equal(r[0], v[0]) and torch.equal(r[:, 6:], v[:, 6:])          # position 0, and the unrotated tail
    assert torch.allclose(r[:, :6].norm(dim=-1), v[:, :6].norm(dim=-1))
    a = 7 * 100.0 ** (-2.0 / 6)                                                  # pair (1, 4) at position 7
    assert torch.allclose(r[2, 1], v[2, 1] * torch.cos(torch.tensor(a)) - v[2, 4] * torch.sin(torch.tensor(a)))
    idx, w = O.router(v, torch.randn(6, 8, generator=g), torch.zeros(6), 3)
    assert torch.allclose(w.sum(-1), torch.ones(5)) and (w[:, 0] >= w[:, 1]).all() and idx.shape == (5, 3)
    y = torch.randn(4, 8, generator=g, dtype=torch.float64)
    assert torch.allclose(O.norm_offset(y, torch.zeros(8), 0.0).square().mean(-1), torch.ones(4, dtype=torch.float64))
    assert torch.allclose(O.norm_plain(y, torch.ones(8), 1e-5), O.norm_offset(y, torch.zeros(8), 1e-5))
