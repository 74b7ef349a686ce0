"""What of the Sulepel design needs no GPU: reading its config.json, the
description and cache plan that follow from it, the cache manager's chunked
groups, and the plain implementation's own mechanisms against one another."""
import copy

import pytest
import torch

import plain_sulepel as ps
from lyapunov_engine_b200 import build
from lyapunov_engine_b200.config import ConfigError, SulepelConfig
from lyapunov_engine_b200.models.model import Model
from lyapunov_engine_b200.registry import spec_for

CFG = {"architecture": "Sulepel", "vocab": 50, "width": 48, "norm": {"eps": 1e-5, "groups": 2}, "canon": {"taps": 3},
       "layers": [{"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 8, "mask": {"size": 12},
                                                  "scale": 0.25}, "mlp": {"kind": "dense", "ff": 64, "limit": 2.0}},
                  {"type": "latent_attention", "mixer": {"heads": 2, "dim": 8, "vdim": 24, "kv_rank": 40, "scale": 0.3},
                   "mlp": None}]}


def test_config_is_read_key_by_key():
    c = SulepelConfig.from_dict(CFG)
    assert (c.vocab, c.width, c.norm_groups, c.taps, len(c.layers)) == (50, 48, 2, 3, 2)
    assert c.layers[0].mixer.chunk == 12 and c.layers[0].feed_forward.limit == 2.0
    assert c.layers[1].mixer.kv_rank == 40 and c.layers[1].feed_forward is None
    for path, value, word in ((("width",), None, "width"), (("norm", "groups"), None, "groups"),
                              (("canon", "taps"), None, "taps"), (("layers", 0, "mixer", "mask", "size"), None, "size"),
                              (("layers", 0, "mixer", "scale"), None, "scale"), (("layers", 1, "mixer", "kv_rank"), None, "kv_rank"),
                              (("layers", 0, "type"), "sliding", "sliding"), (("layers", 0, "mlp", "kind"), "routed", "routed"),
                              (("norm", "groups"), 5, "groups"), (("layers", 0, "mixer", "kv_heads"), 3, "kv_heads")):
        bad = copy.deepcopy(CFG)
        at = bad
        for k in path[:-1]:
            at = at[k]
        if value is None:
            del at[path[-1]]
        else:
            at[path[-1]] = value
        with pytest.raises(ConfigError, match=word):
            SulepelConfig.from_dict(bad)


def test_description_and_cache_plan():
    model = Model(spec_for(CFG))
    assert {d.name: tuple(d.shape) for d in model.tensors()} == ps.tensor_shapes(CFG)
    # chunked keys and values at the larger of the two head sizes; one pool of latents, padded to a multiple of 16
    assert [(g.num_kv_heads, g.head_dim, g.window, g.chunk, g.values) for g in model.groups] == \
        [(2, 16, None, 12, True), (1, 48, None, None, False)]
    assert [tuple(s.shape) for s in model.states] == [(2, 48), (2, 48)]          # taps - 1 inputs per layer and request
    assert [r.extra_states for r in model.runs] == [(("mixer_input", 0),), (("mixer_input", 1),)]
    assert 16 in model.tile_sizes


def test_a_config_without_convolution_or_mask_describes_a_model_without_them():
    bare = copy.deepcopy(CFG)
    del bare["canon"]
    del bare["layers"][0]["mixer"]["mask"]
    model = Model(spec_for(bare))
    assert {d.name: tuple(d.shape) for d in model.tensors()} == ps.tensor_shapes(bare)
    assert not any(d.name.endswith("canon1") for d in model.tensors()) and model.states == []
    assert [(g.window, g.chunk) for g in model.groups] == [(None, None), (None, None)]


def test_cache_manager_gives_back_pages_before_the_current_chunk():
    host = build.load_host()
    groups = [host.CacheGroupSpec(block_size=4, window=0, num_blocks=40),
              host.CacheGroupSpec(block_size=4, chunk=10, num_blocks=40)]
    bm = host.BlockSpaceManager(groups, 2)
    seq = host.Sequence(0, list(range(60)), host.SamplingParams())
    for n in (3, 9, 10, 11, 19, 20, 37, 40, 60):
        assert bm.grow(seq, n)
        seq.set_num_computed_tokens(n)
        bm.release_passed(seq)
        # the next query stands at n: its chunk starts at n // 10 * 10; pages wholly before that are dead
        first_needed = n // 10 * 10
        live = (n + 3) // 4 - first_needed // 4
        assert bm.get_num_used_blocks(1) == live, (n, bm.get_num_used_blocks(1), live)
        assert bm.get_num_used_blocks(0) == (n + 3) // 4
        assert bm.audit() == ""
        table = seq.get_block_tables()[1]
        assert all(p < 0 for p in table[:first_needed // 4]) and all(p >= 0 for p in table[first_needed // 4:(n + 3) // 4])
    bm.free(seq)
    assert bm.get_num_free_blocks(0) == 40 and bm.get_num_free_blocks(1) == 40
    with pytest.raises(ValueError):
        host.BlockSpaceManager([host.CacheGroupSpec(block_size=4, window=5, chunk=10, num_blocks=8)], 1)


def test_plain_mechanisms_agree_with_their_definitions():
    g = torch.Generator().manual_seed(0)
    # the convolution, token by token from kept inputs, against the whole sequence
    h, w = torch.randn(9, 5, generator=g, dtype=torch.float64), torch.randn(5, 3, generator=g, dtype=torch.float64)
    whole = ps.causal_taps(h, w)
    for t in range(9):
        acc = h[t].clone()
        for j in range(3):
            src = t - 2 + j
            if src >= 0:
                acc += w[:, j] * h[src]
        torch.testing.assert_close(whole[t], acc)
    # chunks: query 12 of chunks of 5 sees keys 10, 11, 12 only
    mask = ps.chunk_mask(14, 5)
    assert mask[12].nonzero().flatten().tolist() == [10, 11, 12] and mask[4].nonzero().flatten().tolist() == [0, 1, 2, 3, 4]
    # the position vector: sin and cos of the same angle side by side
    s = ps.sinusoid(torch.tensor([0, 3]), 6, torch.float64)
    assert s[0].tolist() == [0.0, 1.0, 0.0, 1.0, 0.0, 1.0]
    torch.testing.assert_close(s[1, 2] ** 2 + s[1, 3] ** 2, torch.tensor(1.0, dtype=torch.float64))
    torch.testing.assert_close(s[1, 2], torch.sin(torch.tensor(3.0 * 10000.0 ** (-2.0 / 6.0), dtype=torch.float64)))
    # the norm in groups: every part has unit mean square before the weight
    x = torch.randn(2, 12, generator=g, dtype=torch.float64)
    n = ps.grouped_rmsnorm(x, torch.ones(12, dtype=torch.float64), 0.0, 3).view(2, 3, 4)
    torch.testing.assert_close(n.pow(2).mean(-1), torch.ones(2, 3, dtype=torch.float64))
    # prefix property of the whole model: a position's logits do not depend on later tokens
    wts = ps.random_weights(CFG, 1)
    ids = torch.randint(0, 50, (30,), generator=g).tolist()
    full = ps.forward(CFG, wts, ids)
    torch.testing.assert_close(ps.forward(CFG, wts, ids[:17])[-1], full[16])
