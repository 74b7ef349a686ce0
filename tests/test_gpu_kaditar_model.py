"""Kaditar models through the framework (its loader, cache manager, step
function and kernels, driven by the trace replay program and by the generation
entry point) against the plain implementation of tests/plain_kaditar.py:
whole prompts, token-by-token decoding, portions down to two tokens, mixed
batches on a pool whose pages and slots are used again, long decoding over
window and page borders from the first token on, greedy generation.  The
configurations differ from one another in every size; one takes the values that
make mechanisms vanish (one stream copy, a loop that runs once, one expert
chosen of one, all experts chosen, one key/value head, a window of one key and
one longer than any sequence, no rotary width, diff 0), one leaves out every
key that may be absent, one has sizes the tensor-core kernels take whole.
Scores are scaled up so that single keys decide a softmax: a window that is
off by one key moves the logits far beyond the tolerance (asserted)."""
import copy
import json
import os

import numpy as np
import pytest
import torch

import plain_kaditar as pk
import replay_util as ru

pytestmark = pytest.mark.gpu


def attn(heads, kv_heads, dim, vdim, window, rot, base, scale, diff, mlp):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "diff": diff}
    if window:
        mixer["mask"] = {"size": window}
    if rot is not None:
        mixer["rot"] = {"dims": rot, "base": base}
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, shared):
    out = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared:
        out["shared"] = {"ff": shared}
    return out


CONFIGS = {
    # every size its own; value sizes above and below two maps; the looped stretch ends with a layer without feed-forward
    "a": ({"architecture": "Kaditar", "vocab": 211, "width": 96, "norm": {"eps": 1e-5}, "streams": 3, "logit_softcap": 12.0,
           "loop": {"start": 1, "stop": 3, "times": 2},
           "layers": [attn(4, 2, 16, 40, 10, 8, 1e4, 0.9, 0.25, dense(160)),
                      attn(2, 1, 24, 24, 33, 24, 5e5, 0.7, 0.4, moe(6, 2, 48, 64)),
                      attn(3, 3, 8, 16, 5, 4, 100.0, 1.2, 0.1, None),
                      attn(6, 2, 8, 24, 21, 6, 1e3, 1.0, 0.35, moe(5, 3, 24, 0))]}, 8),
    # the values that make a mechanism vanish
    "b": ({"architecture": "Kaditar", "vocab": 97, "width": 64, "norm": {"eps": 1e-6}, "streams": 1, "logit_softcap": 50.0,
           "loop": {"start": 0, "stop": 2, "times": 1},
           "layers": [attn(1, 1, 16, 16, 1, 0, 1e4, 0.5, 0.0, moe(1, 1, 32, 16)),
                      attn(2, 1, 8, 32, 100000, 8, 1e4, 0.8, 0.5, moe(3, 3, 16, 0)),
                      attn(4, 4, 16, 8, 2, 2, 7.0, 0.6, 0.2, dense(40))]}, 4),
    # sizes the tensor-core kernels take whole (heads of 64 and 128 in the cache, 128 rows and more per step), pages of 16
    "c": ({"architecture": "Kaditar", "vocab": 300, "width": 128, "norm": {"eps": 1e-5}, "streams": 2, "logit_softcap": 20.0,
           "layers": [attn(2, 1, 32, 64, 100, 16, 1e4, 0.5, 0.3, dense(256)),
                      attn(2, 2, 64, 128, 150, 64, 5e5, 0.35, 0.2, moe(8, 2, 128, 128)),
                      attn(4, 2, 32, 32, 40, 32, 1e4, 0.5, 0.3, dense(128))]}, 16),
    # every key that may be absent is absent (one stream with plain additions, no loop, no cap, all keys visible, no
    # rotary, no shared expert); sizes no kernel takes in 16-byte pieces; heads beyond the tensor-core kernels' sizes
    "d": ({"architecture": "Kaditar", "vocab": 130, "width": 100, "norm": {"eps": 1e-5},
           "layers": [attn(2, 1, 20, 12, 0, None, 0, 0.6, 0.3, moe(4, 2, 36, 0)),
                      attn(2, 2, 72, 100, 25, 10, 1e4, 0.3, 0.15, dense(44))]}, 8),
}
LENGTHS = {"a": (23, 47, 75, 141), "b": (9, 70, 35, 101), "c": (40, 130, 301, 215), "d": (12, 66, 31, 90)}
PROMPTS = {"a": (3, 30, 41, 100), "b": (1, 64, 2, 67), "c": (8, 128, 260, 101), "d": (2, 40, 30, 51)}


def write_folder(folder, cfg, weights, dtype):
    from safetensors.torch import save_file
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as f:
        json.dump(cfg, f)
    save_file({k: v.to(dtype).contiguous() for k, v in weights.items()}, os.path.join(folder, "model.safetensors"))


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for name, (cfg, page) in CONFIGS.items():
        w = pk.random_weights(cfg, seed=len(name) + cfg["width"])
        folders = {}
        for dtype in (torch.float32, torch.bfloat16):
            d = str(tmp_path_factory.mktemp(f"kaditar_{name}_{'f32' if dtype == torch.float32 else 'bf16'}"))
            write_folder(d, cfg, w, dtype)
            folders["float32" if dtype == torch.float32 else "bfloat16"] = d
        g = torch.Generator().manual_seed(7)
        requests = {f"r{i}": torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for i, n in enumerate(LENGTHS[name])}
        exact = {r: pk.forward(cfg, w, ids, torch.float64) for r, ids in requests.items()}
        rounded = {r: pk.forward(cfg, w, ids, torch.float64, round_to=torch.bfloat16) for r, ids in requests.items()}
        noise = float(np.sqrt(np.mean([float((rounded[r] - exact[r]).pow(2).mean()) for r in requests])))
        out[name] = dict(cfg=cfg, page=page, w=w, folders=folders, requests=requests, exact=exact, rounded=rounded, noise=noise,
                         prompt_lens={f"r{i}": n for i, n in enumerate(PROMPTS[name])})
    return out


def check(m, trace, dtype, out_dir, pool=None, what="", extra=()):
    """Runs the trace and compares every wanted place.  float32: tight.
    bfloat16: in units of what rounding activations to bfloat16 moves the plain
    implementation's own logits by (root mean square over all places)."""
    pool = pool or sum((len(v) + 63) // 64 * 64 for v in m["requests"].values())
    got = ru.run_trace(trace, m["folders"][dtype], dtype, str(out_dir), pool, m["page"], extra=extra)
    assert len(got) == sum(len(w) for w in trace.wanted)
    ref = {r: v.float() for r, v in m["exact"].items()}
    if dtype == "float32":
        return ru.compare(got, ref, atol=3e-4, rtol=3e-4, what=what)
    # Sharp scores and a router's choice make rounding noise heavy-tailed: the plain implementation's own rounded run
    # lies up to 20 units from its exact one at single places (a router logit that rounding pushes past another, and
    # the places after it that see that token through their windows), with a median of 0.5 to 1.1.  So: the median, a
    # cap that a key wrongly seen or missed (50 units and more) still breaks, and no more loud places than twice what
    # the plain implementation's rounded run has at the same places.
    units, own = [], []
    for (rid, p), row in sorted(got.items()):
        assert np.all(np.isfinite(row))
        d = row.astype(np.float64) - m["exact"][rid][p].numpy()
        units.append(float(np.sqrt(np.mean(d * d))) / m["noise"])
        own.append(float((m["rounded"][rid][p] - m["exact"][rid][p]).pow(2).mean().sqrt()) / m["noise"])
    worst = int(np.argmax(units))
    assert units[worst] <= 30.0, f"{what}: place {sorted(got)[worst]}: {units[worst]:.1f} units of rounding noise"
    assert float(np.median(units)) <= 1.5, f"{what}: the median place lies {np.median(units):.2f} units of rounding noise off"
    loud, loud_own = sum(u > 4.0 for u in units), sum(u > 4.0 for u in own)
    assert loud <= 2 * loud_own + max(2, len(units) // 50), \
        f"{what}: {loud} of {len(units)} places above 4 units of rounding noise (the plain rounded run: {loud_own})"
    return float(np.median(units))


def test_the_model_is_described_from_its_config(models):
    from lyapunov_engine_b200.models.model import Model
    from lyapunov_engine_b200.registry import spec_for
    for name, m in models.items():
        model = Model(spec_for(m["cfg"]))
        assert {d.name: tuple(d.shape) for d in model.tensors()} == pk.tensor_shapes(m["cfg"])
        assert [r.layer for r in model.runs] == pk.run_order(m["cfg"])
        assert model.states == []
    a = Model(spec_for(models["a"]["cfg"]))
    # a cache group per geometry and window; the looped layers have a pool pair per pass
    assert sorted((g.num_kv_heads, g.head_dim, g.window) for g in a.groups) == [(1, 48, 33), (2, 32, 21), (2, 48, 10), (3, 16, 5)]
    assert sorted(a.streams_per_group) == [1, 1, 2, 2]
    d = Model(spec_for(models["d"]["cfg"]))
    assert sorted((g.num_kv_heads, g.head_dim, g.window) for g in d.groups) == [(1, 48, None), (2, 144, 25)]


def test_a_window_that_is_one_key_off_would_show(models):
    """The plain implementation with every window one key longer or shorter
    moves the logits by far more than the comparisons allow."""
    m = models["a"]
    ids = m["requests"]["r2"]
    for delta in (1, -1):
        cfg = copy.deepcopy(m["cfg"])
        for layer in cfg["layers"]:
            layer["mixer"]["mask"]["size"] += delta
        other = pk.forward(cfg, m["w"], ids, torch.float64)
        moved = (other - m["exact"]["r2"]).abs().amax(dim=-1)
        assert float(moved[40:].median()) > 100 * 3e-4 and float(moved[40:].pow(2).mean().sqrt()) > 10 * m["noise"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_whole_prompts(models, name, dtype, tmp_path):
    m = models[name]
    check(m, ru.whole_trace(m["requests"]), dtype, tmp_path, what=f"{name} {dtype} whole")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_prefill_then_token_by_token(models, name, dtype, tmp_path):
    m = models[name]
    check(m, ru.tail_trace(m["requests"], tail=44), dtype, tmp_path, what=f"{name} {dtype} decode")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_portions_down_to_two_tokens(models, name, dtype, tmp_path):
    m = models[name]
    check(m, ru.portions_trace(m["requests"]), dtype, tmp_path, what=f"{name} {dtype} portions")
    check(m, ru.portions_trace(m["requests"], sizes=(2, 2, 3, 2, 129, 2)), dtype, tmp_path, what=f"{name} {dtype} small portions")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_mixed_batches_on_a_pool_that_is_used_again(models, name, dtype, tmp_path):
    """Twice the requests, up to four live, on a pool that just holds the peak:
    late requests get pages that others gave back with their keys still in them."""
    m = models[name]
    requests, prompts, exact, rounded = dict(m["requests"]), dict(m["prompt_lens"]), dict(m["exact"]), dict(m["rounded"])
    g = torch.Generator().manual_seed(11)
    for rid, ids in list(m["requests"].items()):
        requests[rid + "x"] = torch.randint(0, m["cfg"]["vocab"], (len(ids),), generator=g).tolist()
        prompts[rid + "x"] = m["prompt_lens"][rid]
        exact[rid + "x"] = pk.forward(m["cfg"], m["w"], requests[rid + "x"], torch.float64)
        rounded[rid + "x"] = pk.forward(m["cfg"], m["w"], requests[rid + "x"], torch.float64, round_to=torch.bfloat16)
    trace = ru.mixed_trace(requests, prompts, chunk=16, max_live=4, seed=5)
    assert any(len(s["entries"]) >= 3 for s in trace.steps)
    m2 = dict(m, requests=requests, exact=exact, rounded=rounded)
    check(m2, trace, dtype, tmp_path, pool=ru.peak_pool_tokens(trace, m["page"]), what=f"{name} {dtype} mixed",
          extra=("--max-num-seqs", "4"))
    pages = ru.read_pages(str(tmp_path))
    assert pages["allocations"] > pages["pool_pages"] and pages["reuses"] > 0, pages


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_and_long_decoding(models, dtype, tmp_path):
    """One request token by token from its first token on, far past every
    window and many pages (the captured decode step serves it), beside a
    second request that joins late."""
    m = models["a"]
    g = torch.Generator().manual_seed(3)
    ids = torch.randint(0, m["cfg"]["vocab"], (170,), generator=g).tolist()
    other = m["requests"]["r1"]
    exact = {"long": pk.forward(m["cfg"], m["w"], ids, torch.float64), "r1": m["exact"]["r1"]}
    rounded = {"long": pk.forward(m["cfg"], m["w"], ids, torch.float64, round_to=torch.bfloat16), "r1": m["rounded"]["r1"]}
    t = ru.Trace()
    for i, tok in enumerate(ids):
        entries = [("long", [tok], [0])]
        j = i - 100
        if 0 <= j < len(other):
            entries.append(("r1", [other[j]], [0]))
        t.step(entries, end=(["long"] if i == len(ids) - 1 else []) + (["r1"] if j == len(other) - 1 else []))
    check(dict(m, exact=exact, rounded=rounded), t, dtype, tmp_path, pool=256, what=f"a {dtype} long decoding")


def test_window_pages_are_given_back_while_a_request_lives(models, tmp_path):
    """Every pass of a windowed layer holds one request's window, not its whole context."""
    from lyapunov_engine_b200 import build
    from lyapunov_engine_b200.cache import DeviceCache
    from lyapunov_engine_b200.engine.llm_engine import load_model
    from lyapunov_engine_b200.engine.step import ModelRunner
    m = models["a"]
    host = build.load_host()
    loaded = load_model(m["folders"]["float32"], "float32", "cuda:0", max_model_len=256)
    cache = DeviceCache(loaded.model, loaded.runtime, num_blocks=32, block_size=8, max_num_seqs=2)
    runner = ModelRunner(loaded.model, cache, loaded.runtime, 256, 2, 256, use_cuda_graphs=False, check_status=True)
    ids = m["requests"]["r3"]
    seq = host.Sequence(0, ids, host.SamplingParams())
    got, pos = [], 0
    for n in (50, 3, 1, 1, 40, 2, 44):
        assert cache.manager.grow(seq, pos + n)
        got.append(runner.step([host.StepEntry(seq, pos, n, list(range(n)))]).cpu())
        pos += n
        seq.set_num_computed_tokens(pos)
        cache.manager.release_passed(seq)
        for gi, group in enumerate(loaded.model.groups):
            assert cache.manager.get_num_used_blocks(gi) <= (group.window + 7) // 8 + 1
        assert cache.manager.audit() == ""
    torch.testing.assert_close(torch.cat(got), m["exact"]["r3"].float(), atol=3e-4, rtol=3e-4)


def test_the_stream_after_every_layer_run(models):
    """The sum of the stream's copies after every run of a layer (looped layers
    count each time) against the plain implementation."""
    from lyapunov_engine_b200 import build
    from lyapunov_engine_b200.cache import DeviceCache
    from lyapunov_engine_b200.engine.llm_engine import load_model
    from lyapunov_engine_b200.engine.step import ModelRunner
    m = models["a"]
    host = build.load_host()
    loaded = load_model(m["folders"]["float32"], "float32", "cuda:0", max_model_len=128)
    cache = DeviceCache(loaded.model, loaded.runtime, num_blocks=16, block_size=8, max_num_seqs=1)
    runner = ModelRunner(loaded.model, cache, loaded.runtime, 128, 1, 128, use_cuda_graphs=False, check_status=True)
    ids = m["requests"]["r1"]
    S, W = m["cfg"]["streams"], m["cfg"]["width"]
    seen = []

    def observe(index, stream):
        x = stream.resid.view(-1, S, W)
        y = stream.pending
        y = (y.sum(0) if y.dim() == 3 else y).float()
        link = stream.update
        new = torch.einsum("st,bsw->btw", link.mix.view(S, S), x) + link.post.view(1, S, 1) * y[:, None, :]
        seen.append(new.sum(1).cpu())

    forward = loaded.model.forward
    loaded.model.forward = lambda ctx, c: forward(ctx, c, observe=observe)
    seq = host.Sequence(0, ids, host.SamplingParams())
    assert cache.manager.grow(seq, len(ids))
    runner.step([host.StepEntry(seq, 0, len(ids), [0])])
    want = []
    pk.forward(m["cfg"], m["w"], ids, torch.float64, layers_out=want)
    assert len(seen) == len(want) == 6
    for got, ref in zip(seen, want):
        torch.testing.assert_close(got, ref.float(), atol=2e-4, rtol=2e-4)


@pytest.mark.parametrize("name", ["a", "b"])
def test_greedy_generation_through_the_entry_point(models, name):
    """Five requests through LLMEngine.generate with its scheduler, two
    requests live at a time and small pages: the same tokens as the plain
    implementation picks."""
    from lyapunov_engine_b200 import LLMEngine, SamplingParams
    m = models[name]
    engine = LLMEngine.from_pretrained(m["folders"]["float32"], dtype="float32", num_blocks=40, block_size=m["page"],
                                       max_num_seqs=2, max_num_batched_tokens=24, max_model_len=160)
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(0, m["cfg"]["vocab"], (n,), generator=g).tolist() for n in (3, 37, 1, 26, 12)]
    outs = engine.generate(prompts, SamplingParams(temperature=0.0, max_tokens=9, ignore_eos=True))
    for p, o in zip(prompts, outs):
        assert o.output_tokens == pk.greedy(m["cfg"], m["w"], p, 9), (p, o.output_tokens)
        assert o.finish_reason == "length"
    assert engine.block_manager.audit() == ""


def test_command_line_generates_from_random_weights(tmp_path):
    """`generate --random-weights` builds a Kaditar model from a config.json alone."""
    import subprocess
    import sys
    cfg = CONFIGS["b"][0]
    folder = tmp_path / "cfg"
    folder.mkdir()
    (folder / "config.json").write_text(json.dumps(cfg))
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    proc = subprocess.run([sys.executable, os.path.join(root, "bin", "lyapunov"), "generate", "--model", str(folder),
                           "--random-weights", "--prompt-ids", "5,6,7", "--max-tokens", "6", "--temperature", "0"],
                          capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
