"""What of the Kaditar design needs no GPU: config.json key by key, the layers'
run order, what the cache must hold, and the plain implementation's own
pieces against each other."""
import copy

import pytest
import torch

import plain_kaditar as pk
from lyapunov_engine_b200.config.base import ConfigError
from lyapunov_engine_b200.config.kaditar import KaditarConfig
from lyapunov_engine_b200.models.model import Model
from lyapunov_engine_b200.registry import spec_for

CFG = {"architecture": "Kaditar", "vocab": 50, "width": 32, "norm": {"eps": 1e-5}, "streams": 2, "logit_softcap": 9.0,
       "loop": {"start": 1, "stop": 2, "times": 3},
       "layers": [{"type": "attention",
                   "mixer": {"heads": 2, "kv_heads": 1, "dim": 8, "vdim": 24, "scale": 0.3, "diff": 0.2,
                             "rot": {"dims": 4, "base": 100.0}, "mask": {"size": 6}},
                   "mlp": {"kind": "dense", "ff": 48}},
                  {"type": "attention",
                   "mixer": {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 8, "scale": 0.3, "diff": 0.2,
                             "rot": {"dims": 8, "base": 100.0}, "mask": {"size": 6}},
                   "mlp": {"kind": "moe", "expert": {"ff": 16}, "router": {"experts": 3, "top": 2}, "shared": {"ff": 8}}},
                  {"type": "attention",
                   "mixer": {"heads": 2, "kv_heads": 2, "dim": 8, "vdim": 8, "scale": 0.3, "diff": 0.2,
                             "rot": {"dims": 8, "base": 100.0}, "mask": {"size": 6}},
                   "mlp": None}]}


def test_config_is_read_key_by_key():
    c = KaditarConfig.from_dict(CFG)
    assert (c.vocab, c.width, c.streams, c.logit_softcap, c.loop) == (50, 32, 2, 9.0, (1, 2, 3))
    assert c.run_order() == [0, 1, 1, 1, 2] == pk.run_order(CFG)
    assert c.layers[1].feed_forward.experts == 3 and c.layers[1].feed_forward.shared_ff == 8
    assert c.layers[2].feed_forward is None and c.layers[0].mixer.window == 6
    for path in (("vocab",), ("width",), ("norm",), ("layers", 0, "mixer", "heads"), ("layers", 0, "mixer", "diff"),
                 ("layers", 0, "mixer", "scale"), ("layers", 0, "mixer", "vdim"), ("layers", 1, "mlp", "router"),
                 ("layers", 1, "mlp", "expert"), ("layers", 0, "mlp", "ff"), ("layers", 0, "mixer", "rot", "base"),
                 ("loop", "times")):
        broken = copy.deepcopy(CFG)
        at = broken
        for key in path[:-1]:
            at = at[key]
        del at[path[-1]]
        with pytest.raises(ConfigError, match=str(path[-1])):
            KaditarConfig.from_dict(broken)
    for path, value in ((("layers", 0, "mixer", "kv_heads"), 3), (("layers", 0, "mixer", "rot", "dims"), 5),
                        (("layers", 0, "mixer", "rot", "dims"), 10), (("layers", 1, "mlp", "router", "top"), 4),
                        (("loop", "stop"), 4), (("layers", 0, "type"), "other"), (("layers", 0, "mlp", "kind"), "other")):
        broken = copy.deepcopy(CFG)
        at = broken
        for key in path[:-1]:
            at = at[key]
        at[path[-1]] = value
        with pytest.raises(ConfigError):
            KaditarConfig.from_dict(broken)


def test_keys_that_may_be_absent():
    cfg = copy.deepcopy(CFG)
    for key in ("streams", "loop", "logit_softcap"):
        del cfg[key]
    del cfg["layers"][0]["mixer"]["mask"], cfg["layers"][0]["mixer"]["rot"], cfg["layers"][1]["mlp"]["shared"]
    c = KaditarConfig.from_dict(cfg)
    assert c.streams == 0 and c.loop is None and c.logit_softcap == 0.0 and c.run_order() == [0, 1, 2]
    assert c.layers[0].mixer.window == 0 and c.layers[0].mixer.rot_dims == 0 and c.layers[1].feed_forward.shared_ff == 0
    model = Model(spec_for(cfg))
    assert {d.name: tuple(d.shape) for d in model.tensors()} == pk.tensor_shapes(cfg)
    assert not any(".hc" in d.name or "shared" in d.name for d in model.tensors())
    assert model.groups[0].window is None


def test_the_cache_plan_has_a_pool_pair_per_pass():
    model = Model(spec_for(CFG))
    assert {d.name: tuple(d.shape) for d in model.tensors()} == pk.tensor_shapes(CFG)
    assert [r.layer for r in model.runs] == [0, 1, 1, 1, 2]
    # two maps of 8 beside values of 24 -> heads of 32 in the cache; of 8 -> 16
    assert [(g.num_kv_heads, g.head_dim, g.window) for g in model.groups] == [(1, 32, 6), (2, 16, 6)]
    assert model.streams_per_group == [1, 4]
    assert len({(r.group, r.stream) for r in model.runs}) == 5 and all(r.writes for r in model.runs)
    assert model.states == []


def test_plain_pieces_agree_with_each_other():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(5, 12, generator=g, dtype=torch.float64)
    w, b = torch.randn(12, generator=g, dtype=torch.float64), torch.randn(12, generator=g, dtype=torch.float64)
    ref = torch.nn.functional.layer_norm(x, (12,), w, b, 1e-5)
    torch.testing.assert_close(pk.layer_norm(x, w, b, 1e-5), ref)
    # a turn by an angle keeps each pair's length, and position 0 turns nothing
    v = torch.randn(7, 10, generator=g, dtype=torch.float64)
    r = pk.rotate_pairs(v, torch.arange(7), 6, 100.0)
    assert torch.equal(r[0], v[0]) and torch.equal(r[:, 6:], v[:, 6:])
    torch.testing.assert_close(r[:, 0:6].view(7, 3, 2).norm(dim=-1), v[:, 0:6].view(7, 3, 2).norm(dim=-1))
    # scores of turned queries and keys depend on the distance only
    q, k = torch.randn(1, 6, generator=g, dtype=torch.float64), torch.randn(1, 6, generator=g, dtype=torch.float64)
    a = pk.rotate_pairs(q, torch.tensor([9]), 6, 50.0) @ pk.rotate_pairs(k, torch.tensor([4]), 6, 50.0).T
    c = pk.rotate_pairs(q, torch.tensor([105]), 6, 50.0) @ pk.rotate_pairs(k, torch.tensor([100]), 6, 50.0).T
    torch.testing.assert_close(a, c)
    m = pk.window_mask(6, 3)
    assert m[5].tolist() == [False, False, False, True, True, True] and m[1].tolist() == [True, True, False, False, False, False]
    # whole sequences against prefixes: position t depends on tokens up to t only
    w_ = pk.random_weights(CFG, seed=1)
    ids = list(range(3, 20))
    full = pk.forward(CFG, w_, ids)
    torch.testing.assert_close(pk.forward(CFG, w_, ids[:9]), full[:9])
