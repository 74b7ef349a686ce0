"""Sulepel models through the framework (its loader, cache manager, step
function and kernels, driven by the trace replay program and by the generation
entry point) against the plain implementation of tests/plain_sulepel.py:
whole prompts, token-by-token decoding, portions down to two tokens, mixed
batches on a pool whose pages and slots are used again, long decoding over
chunk and page borders, greedy generation.  The configurations differ from one
another in every size; some take the values that make mechanisms vanish
(one norm group, one key/value head, as many as heads, chunks of one key or
shorter than a page, two taps, a layer without feed-forward)."""
import json
import os

import numpy as np
import pytest
import torch

import plain_sulepel as ps
import replay_util as ru

pytestmark = pytest.mark.gpu


def latent(heads, dim, vdim, rank, scale, mlp):
    return {"type": "latent_attention", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": rank, "scale": scale},
            "mlp": mlp}


def chunked(heads, kv_heads, dim, vdim, size, scale, mlp):
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
                                           "mask": {"size": size}, "scale": scale}, "mlp": mlp}


def dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


CONFIGS = {
    # every size its own; a latent that needs padding (20 -> 32); value sizes above and below the key size; a layer
    # without feed-forward; chunks shorter than a page (7 < 8)
    "a": ({"architecture": "Sulepel", "vocab": 211, "width": 96, "norm": {"eps": 1e-5, "groups": 3}, "canon": {"taps": 4},
           "layers": [chunked(6, 3, 16, 32, 10, 0.3, dense(160, 1.5)),
                      latent(3, 24, 40, 48, 0.2, None),
                      latent(2, 16, 16, 20, 0.25, dense(64, 3.0)),
                      chunked(4, 4, 32, 16, 7, 0.2, dense(96, 0.7))]}, 8),
    # the values that make a mechanism vanish: one norm group, two taps, one key/value head, chunks of one key,
    # heads = kv heads, one head
    "b": ({"architecture": "Sulepel", "vocab": 97, "width": 64, "norm": {"eps": 1e-6, "groups": 1}, "canon": {"taps": 2},
           "layers": [latent(1, 16, 48, 64, 0.25, dense(80, 2.5)),
                      chunked(2, 1, 48, 24, 33, 0.15, None),
                      chunked(3, 3, 16, 16, 1, 0.25, dense(48, 1.0)),
                      latent(4, 8, 8, 16, 0.35, dense(40, 4.0))]}, 4),
    # sizes the tensor-core kernels take whole (latent 64 and heads of 64: the tcgen05 prefill; 128 rows and more per
    # step: the tcgen05 product), pages of 16, no taps beyond the token itself
    "c": ({"architecture": "Sulepel", "vocab": 300, "width": 128, "norm": {"eps": 1e-5, "groups": 4}, "canon": {"taps": 1},
           "layers": [latent(4, 32, 32, 64, 0.18, dense(256, 2.0)),
                      chunked(4, 2, 64, 64, 100, 0.125, dense(256, 2.0)),
                      latent(2, 64, 32, 128, 0.12, dense(128, 1.2))]}, 16),
    # sizes no kernel takes in 16-byte pieces (heads of 20 and 12), a latent beyond the tensor-core kernels' head sizes
    # (136 -> 144: the FP32-pipe attention also in bfloat16), five taps, a width of 72 in three parts
    "d": ({"architecture": "Sulepel", "vocab": 130, "width": 72, "norm": {"eps": 1e-5, "groups": 3}, "canon": {"taps": 5},
           "layers": [latent(2, 20, 12, 136, 0.22, dense(56, 1.8)),
                      chunked(2, 1, 12, 20, 25, 0.3, dense(40, 2.2))]}, 8),
    # a width that is no multiple of 8 (no product kernel of the package takes its rows in 16-byte pieces: the
    # library's and the FP32-pipe products run), heads of 8 and 12, an odd vocabulary
    "e": ({"architecture": "Sulepel", "vocab": 77, "width": 100, "norm": {"eps": 1e-5, "groups": 5}, "canon": {"taps": 3},
           "layers": [chunked(2, 2, 8, 8, 5, 0.35, dense(36, 2.0)),
                      latent(2, 12, 12, 24, 0.3, dense(44, 1.5))]}, 4),
    # a model whose config names neither the convolution nor a mask: plain causal attention, no state at all
    "f": ({"architecture": "Sulepel", "vocab": 90, "width": 48, "norm": {"eps": 1e-5, "groups": 2},
           "layers": [{"type": "attention", "mixer": {"heads": 3, "kv_heads": 1, "dim": 16, "vdim": 16, "scale": 0.25},
                       "mlp": dense(64, 2.0)},
                      latent(3, 16, 16, 32, 0.25, dense(64, 2.0))]}, 8),
}
LENGTHS = {"a": (23, 47, 75, 141), "b": (9, 70, 35, 101), "c": (40, 130, 301, 215), "d": (12, 66, 31, 90), "e": (7, 45, 29, 70), "f": (5, 40, 18, 77)}
PROMPTS = {"a": (3, 30, 41, 100), "b": (1, 64, 2, 67), "c": (8, 128, 260, 101), "d": (2, 40, 30, 51), "e": (2, 33, 20, 40), "f": (3, 20, 10, 50)}


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
        w = ps.random_weights(cfg, seed=len(name) + cfg["width"])
        if name == "b":
            w["l1.mix.temp"] = torch.tensor([1.25, -0.75])          # a negative factor: the loudest key becomes the faintest
        folders = {}
        for dtype in (torch.float32, torch.bfloat16):
            d = str(tmp_path_factory.mktemp(f"sulepel_{name}_{'f32' if dtype == torch.float32 else 'bf16'}"))
            write_folder(d, cfg, w, dtype)
            folders["float32" if dtype == torch.float32 else "bfloat16"] = d
        g = torch.Generator().manual_seed(7)
        requests = {f"r{i}": torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for i, n in enumerate(LENGTHS[name])}
        exact = {r: ps.forward(cfg, w, ids, torch.float64) for r, ids in requests.items()}
        rounded = {r: ps.forward(cfg, w, ids, torch.float64, round_to=torch.bfloat16) for r, ids in requests.items()}
        noise = float(np.sqrt(np.mean([float((rounded[r] - exact[r]).pow(2).mean()) for r in requests])))
        out[name] = dict(cfg=cfg, page=page, w=w, folders=folders, requests=requests, exact=exact, noise=noise,
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
        return ru.compare(got, ref, atol=2e-4, rtol=2e-4, what=what)
    total, n = 0.0, 0
    for (rid, p), row in sorted(got.items()):
        assert np.all(np.isfinite(row))
        d = row.astype(np.float64) - m["exact"][rid][p].numpy()
        rms = float(np.sqrt(np.mean(d * d)))
        assert rms <= 2.5 * m["noise"], f"{what}: request {rid} position {p}: {rms / m['noise']:.2f} units of rounding noise"
        total += float(np.sum(d * d)); n += d.size
    assert (total / n) ** 0.5 <= 1.5 * m["noise"], f"{what}: {(total / n) ** 0.5 / m['noise']:.2f} units of rounding noise overall"
    return (total / n) ** 0.5 / m["noise"]


def test_the_model_is_described_from_its_config(models):
    from lyapunov_engine_b200.models.model import Model
    from lyapunov_engine_b200.registry import spec_for
    for name, m in models.items():
        model = Model(spec_for(m["cfg"]))
        assert {d.name: tuple(d.shape) for d in model.tensors()} == ps.tensor_shapes(m["cfg"])
    a = Model(spec_for(models["a"]["cfg"]))
    # two groups of chunked pages (each with keys and values), two of latents (one pool each, 48 and 20 -> 32 wide)
    assert sorted((g.num_kv_heads, g.head_dim, g.chunk, g.values) for g in a.groups) == \
        sorted([(3, 32, 10, True), (1, 48, None, False), (1, 32, None, False), (4, 32, 7, True)])
    assert len(a.states) == 4 and all(tuple(s.shape) == (3, 96) for s in a.states)
    assert Model(spec_for(models["c"]["cfg"])).states == []       # one tap keeps nothing


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_whole_prompts(models, name, dtype, tmp_path):
    m = models[name]
    check(m, ru.whole_trace(m["requests"]), dtype, tmp_path, what=f"{name} {dtype} whole")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_prefill_then_token_by_token(models, name, dtype, tmp_path):
    m = models[name]
    check(m, ru.tail_trace(m["requests"], tail=36), dtype, tmp_path, what=f"{name} {dtype} decode")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_portions_down_to_two_tokens(models, name, dtype, tmp_path):
    m = models[name]
    check(m, ru.portions_trace(m["requests"]), dtype, tmp_path, what=f"{name} {dtype} portions")
    check(m, ru.portions_trace(m["requests"], sizes=(2, 2, 3, 2, 129, 2)), dtype, tmp_path, what=f"{name} {dtype} small portions")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_mixed_batches_on_a_pool_that_is_used_again(models, name, dtype, tmp_path):
    """Twice the requests, up to four live, on a pool that just holds the peak
    and with four state slots: late requests get pages and slots that others
    gave back with their keys and inputs still in them."""
    m = models[name]
    requests, prompts, exact = dict(m["requests"]), dict(m["prompt_lens"]), dict(m["exact"])
    g = torch.Generator().manual_seed(11)
    for rid, ids in list(m["requests"].items()):
        requests[rid + "x"] = torch.randint(0, m["cfg"]["vocab"], (len(ids),), generator=g).tolist()
        prompts[rid + "x"] = m["prompt_lens"][rid]
        exact[rid + "x"] = ps.forward(m["cfg"], m["w"], requests[rid + "x"], torch.float64)
    trace = ru.mixed_trace(requests, prompts, chunk=16, max_live=4, seed=5)
    assert any(len(s["entries"]) >= 3 for s in trace.steps)
    m2 = dict(m, requests=requests, exact=exact)
    check(m2, trace, dtype, tmp_path, pool=ru.peak_pool_tokens(trace, m["page"]), what=f"{name} {dtype} mixed",
          extra=("--max-num-seqs", "4"))
    pages = ru.read_pages(str(tmp_path))
    assert pages["allocations"] > pages["pool_pages"] and pages["reuses"] > 0, pages


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_and_long_decoding(models, dtype, tmp_path):
    """One request token by token from its first token on, far past several
    chunks and pages (the captured decode step serves it), beside a second
    request that joins late."""
    m = models["a"]
    g = torch.Generator().manual_seed(3)
    ids = torch.randint(0, m["cfg"]["vocab"], (170,), generator=g).tolist()
    other = m["requests"]["r1"]
    exact = {"long": ps.forward(m["cfg"], m["w"], ids, torch.float64), "r1": m["exact"]["r1"]}
    t = ru.Trace()
    for i, tok in enumerate(ids):
        entries = [("long", [tok], [0])]
        j = i - 100
        if 0 <= j < len(other):
            entries.append(("r1", [other[j]], [0]))
        t.step(entries, end=(["long"] if i == len(ids) - 1 else []) + (["r1"] if j == len(other) - 1 else []))
    check(dict(m, exact=exact), t, dtype, tmp_path, pool=256, what=f"a {dtype} long decoding")


def test_chunk_pages_are_given_back_while_a_request_lives(models, tmp_path):
    """The pools of the chunked layers hold one request's current chunk, not its whole context."""
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
    chunked_groups = [i for i, g in enumerate(loaded.model.groups) if g.chunk]
    full_groups = [i for i, g in enumerate(loaded.model.groups) if not g.chunk]
    got, pos = [], 0
    for n in (50, 3, 1, 1, 40, 2, 44):
        assert cache.manager.grow(seq, pos + n)
        got.append(runner.step([host.StepEntry(seq, pos, n, list(range(n)))]).cpu())
        pos += n
        seq.set_num_computed_tokens(pos)
        cache.manager.release_passed(seq)
        for gi in chunked_groups:
            size = loaded.model.groups[gi].chunk
            assert cache.manager.get_num_used_blocks(gi) <= (size + 7) // 8 + 1
        for gi in full_groups:
            assert cache.manager.get_num_used_blocks(gi) == (pos + 7) // 8
        assert cache.manager.audit() == ""
    torch.testing.assert_close(torch.cat(got), m["exact"]["r3"].float(), atol=2e-4, rtol=2e-4)


@pytest.mark.parametrize("name", ["a", "b"])
def test_greedy_generation_through_the_entry_point(models, name):
    """Five requests through LLMEngine.generate with its scheduler, two state
    slots and small pages: the same tokens as the plain implementation picks."""
    from lyapunov_engine_b200 import LLMEngine, SamplingParams
    m = models[name]
    engine = LLMEngine.from_pretrained(m["folders"]["float32"], dtype="float32", num_blocks=40, block_size=m["page"],
                                       max_num_seqs=2, max_num_batched_tokens=24, max_model_len=160)
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(0, m["cfg"]["vocab"], (n,), generator=g).tolist() for n in (3, 37, 1, 26, 12)]
    outs = engine.generate(prompts, SamplingParams(temperature=0.0, max_tokens=9, ignore_eos=True))
    for p, o in zip(prompts, outs):
        assert o.output_tokens == ps.greedy(m["cfg"], m["w"], p, 9), (p, o.output_tokens)
        assert o.finish_reason == "length"
    assert engine.block_manager.audit() == ""


def test_command_line_generates_from_random_weights(tmp_path):
    """`generate --random-weights` builds a Sulepel model from a config.json alone."""
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
