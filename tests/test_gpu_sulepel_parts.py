"""Each mechanism of the Sulepel design alone, the kernel against the plain
function of tests/plain_sulepel.py (or plain torch): the sinusoidal embedding,
the norm in groups, the short convolution with its per-request state under
every cut, the clamped gated activation in its three kernels, the per-head
products, the cache writes, and attention over chunks with a factor per head
(every kernel that serves it), with inputs made so that one key at a chunk's
edge decides the result."""
import math

import pytest
import torch

import plain_sulepel as ps

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def test_sinusoid_embedding():
    from lyapunov_engine_b200 import ops
    for width, vocab in ((10, 7), (96, 50), (130, 11)):
        g = torch.Generator().manual_seed(width)
        table = torch.randn(vocab, width, generator=g)
        ids = torch.randint(0, vocab, (9,), generator=g, dtype=torch.int32)
        pos = torch.tensor([0, 1, 2, 63, 64, 500, 1023, 4097, 70000], dtype=torch.int32)
        i = torch.arange(0, width, 2, dtype=torch.float64)
        rates = torch.pow(torch.tensor(10000.0, dtype=torch.float64), -i / width).float()
        out = torch.zeros(9, width, device=DEV)
        status = ops.new_status(DEV)
        ops.embed_sinusoid(out, table.to(DEV), ids.to(DEV), pos.to(DEV), rates.to(DEV), status)
        ops.check_status(status)
        want = table[ids.long()] + ps.sinusoid(pos, width, torch.float64).float()
        # the angle itself is 32-bit: at position p it carries an error of p * 2^-24
        torch.testing.assert_close(out.cpu()[:7], want[:7], atol=2e-4, rtol=0)
        torch.testing.assert_close(out.cpu(), want, atol=1e-2, rtol=0)
        assert float((out.cpu()[0] - table[ids[0].long()])[0::2].abs().max()) == 0.0     # sin(0), exactly


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width,groups", [(96, 1), (96, 3), (360, 5), (66, 2), (4096, 4)])
def test_norm_in_groups(width, groups, dtype):
    from lyapunov_engine_b200 import ops
    g = torch.Generator().manual_seed(width + groups)
    x = torch.randn(5, width, generator=g) * torch.tensor([1.0, 30.0, 0.01, 3.0, 1.0])[:, None]
    x[:, : width // groups] *= 7.0                       # one part much larger than the others: a whole-row norm shows
    delta = torch.randn(5, width, generator=g).to(dtype)
    w = 1.0 + 0.3 * torch.randn(width, generator=g)
    resid = x.clone().to(DEV)
    out = torch.zeros(5, width, dtype=dtype, device=DEV)
    ops.rmsnorm(out, resid, delta.to(DEV), w.to(DEV), 1e-5, groups=groups)
    summed = x + delta.float()
    want = ps.grouped_rmsnorm(summed.double(), w.double(), 1e-5, groups).float()
    torch.testing.assert_close(resid.cpu(), summed, atol=1e-6, rtol=1e-6)
    tol = dict(atol=1e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=1e-2, rtol=1e-2)
    torch.testing.assert_close(out.float().cpu(), want, **tol)
    rows = torch.tensor([3, 0], dtype=torch.int32, device=DEV)
    some = torch.zeros(2, width, dtype=dtype, device=DEV)
    ops.rmsnorm(some, resid, None, w.to(DEV), 1e-5, rows, groups=groups)
    torch.testing.assert_close(some.float().cpu(), want[[3, 0]], **tol)


def _tiles(q_lens, size):
    req, q0 = [], []
    for b, n in enumerate(q_lens):
        for s in range(0, n, size):
            req.append(b); q0.append(s)
    return (torch.tensor(req, dtype=torch.int32, device=DEV), torch.tensor(q0, dtype=torch.int32, device=DEV), len(req))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("taps,C", [(1, 200), (2, 200), (3, 200), (4, 200), (7, 200), (3, 52), (17, 36)])
def test_short_convolution_under_every_cut(taps, C, dtype):
    """Three requests are fed in cuts of unequal sizes (down to one token, and
    shorter than the taps), in batches, with state slots that another request
    left its inputs in; the result equals the convolution of each whole sequence."""
    from lyapunov_engine_b200 import ops
    g = torch.Generator().manual_seed(taps)       # (52 and 36 channels: no 16-byte pieces, one channel a thread)
    w = (0.5 * torch.randn(C, taps, generator=g))
    seqs = [torch.randn(n, C, generator=g).to(dtype) for n in (37, 5, 64)]
    want = [ps.causal_taps(s.double(), w.double()).float() for s in seqs]
    cuts = [[1, 1, 2, 1, 17, 1, 2, 12], [2, 1, 1, 1], [33, 1, 1, 1, 16, 1, 11]]
    slots_of = [2, 0, 3]
    state = torch.full((5, max(taps - 1, 1), C), 9.0, device=DEV) if taps > 1 else None    # stale inputs of earlier requests
    wt = w.t().contiguous().to(DEV)
    got = [[] for _ in seqs]
    at = [0, 0, 0]
    step = 0
    while any(at[r] < len(seqs[r]) for r in range(3)):
        live = [r for r in range(3) if step < len(cuts[r])]
        q_lens = [cuts[r][step] for r in live]
        h = torch.cat([seqs[r][at[r]:at[r] + n] for r, n in zip(live, q_lens)]).to(DEV)
        cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32, device=DEV)
        slots = torch.tensor([slots_of[r] for r in live], dtype=torch.int32, device=DEV)
        before = torch.tensor([at[r] for r in live], dtype=torch.int32, device=DEV)
        if state is not None:
            ops.zero_fresh_state(state, slots, before, len(live))       # what the framework does before a step
        out = torch.zeros_like(h)
        tr, tq, n = _tiles(q_lens, ops.SHORT_CONV_TILE)
        if all(x == 1 for x in q_lens) and step % 2:
            ops.short_conv(out, h, wt, state, slots, cu, None, None, len(q_lens))     # the form for steps of single tokens
        else:
            ops.short_conv(out, h, wt, state, slots, cu, tr, tq, n)
        o = 0
        for r, n in zip(live, q_lens):
            got[r].append(out[o:o + n].float().cpu())
            o += n
            at[r] += n
        step += 1
    tol = dict(atol=1e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=3e-2, rtol=2e-2)
    for r in range(3):
        torch.testing.assert_close(torch.cat(got[r]), want[r], **tol)
    # a row that stands for no request sees zeros before it and keeps nothing
    if state is not None:
        kept = state.clone()
        h = seqs[0][:1].to(DEV)
        out = torch.zeros_like(h)
        tr, tq, n = _tiles([1], ops.SHORT_CONV_TILE)
        ops.short_conv(out, h, wt, state, torch.tensor([-1], dtype=torch.int32, device=DEV),
                       torch.tensor([0, 1], dtype=torch.int32, device=DEV), tr, tq, n)
        torch.testing.assert_close(out.float().cpu(), want[0][:1], **tol)
        assert torch.equal(kept, state)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width,groups,taps,partials", [(96, 3, 4, 0), (2048, 4, 4, 2), (352, 1, 2, 1), (4096, 2, 3, 4), (128, 4, 1, 3),
                                                        (256, 2, 6, 2), (64, 1, 5, 5)])
def test_norm_and_convolution_as_one_kernel(width, groups, taps, partials, dtype):
    """Decode steps run the norm and the short convolution as one kernel: the
    same bits as the two kernels, outputs and state, over several steps, with
    a row that stands for no request."""
    from lyapunov_engine_b200 import ops
    assert ops.rmsnorm_taps_applies(width, groups)
    g = torch.Generator().manual_seed(width + taps)
    B = 5
    w = (1.0 + 0.3 * torch.randn(width, generator=g)).to(DEV)
    wt = (0.5 * torch.randn(taps, width, generator=g)).to(DEV)
    slots = torch.tensor([3, 0, -1, 5, 1], dtype=torch.int32, device=DEV)
    cu = torch.arange(B + 1, dtype=torch.int32, device=DEV)
    states = [torch.randn(7, max(taps - 1, 1), width, generator=g).to(DEV) if taps > 1 else None for _ in range(2)]
    if taps > 1:
        states[1].copy_(states[0])
    for step in range(4):
        x = torch.randn(B, width, generator=g)
        if partials == 0:
            delta = None
        elif partials == 1:
            delta = torch.randn(B, width, generator=g).to(dtype).to(DEV)
        else:
            delta = torch.randn(partials, B, width, generator=g).to(DEV)
        resid = [x.clone().to(DEV), x.clone().to(DEV)]
        normed = torch.zeros(B, width, dtype=dtype, device=DEV)
        two = torch.zeros(B, width, dtype=dtype, device=DEV)
        ops.rmsnorm(normed, resid[0], delta, w, 1e-5, groups=groups)
        ops.short_conv(two, normed, wt, states[0], slots, cu, None, None, B)
        one = torch.zeros(B, width, dtype=dtype, device=DEV)
        ops.rmsnorm_taps(one, resid[1], delta, w, 1e-5, groups, wt, states[1], slots)
        assert torch.equal(one, two) and torch.equal(resid[0], resid[1])
        if taps > 1:
            assert torch.equal(states[0], states[1])
    assert not ops.rmsnorm_taps_applies(66, 2)       # parts that are no multiple of four values: the two kernels run


@pytest.mark.parametrize("rows", [1, 7, 16, 29, 64, 200, 700])
def test_clamped_gated_activation_in_every_kernel(rows):
    """The stand-alone kernel (both types), and in bfloat16 the product kernels
    that carry it in their epilogue: weight-streaming (few rows) and tcgen05."""
    from lyapunov_engine_b200 import ops
    from lyapunov_engine_b200.engine.runtime import Workspace
    K, I, limit, slope = 256, 384, 1.5, 1.702
    g = torch.Generator().manual_seed(rows)
    x = torch.randn(rows, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(2 * I, K, generator=g) * 0.15).to(torch.bfloat16)      # products well beyond the limit on both sides
    gu = x.double() @ w.double().t()
    gate, up = gu[:, :I].clamp(max=limit), gu[:, I:].clamp(min=-limit, max=limit)
    want = (gate * torch.sigmoid(slope * gate) * (up + 1.0)).float()
    assert float((gu[:, :I] > limit).float().mean()) > 0.05 and float((gu[:, I:] < -limit).float().mean()) > 0.05
    act = (ops.GLU_CLAMPED, slope, limit)
    for dtype in (torch.float32, torch.bfloat16):
        out = torch.zeros(rows, I, dtype=dtype, device=DEV)
        ops.glu(out, gu.to(dtype).to(DEV), *act)
        tol = dict(atol=1e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=3e-2, rtol=2e-2)
        torch.testing.assert_close(out.float().cpu(), want, **tol)
    ws = Workspace(torch.device(DEV))
    out = torch.zeros(rows, I, dtype=torch.bfloat16, device=DEV)
    ops.gated_linear(out, x.to(DEV), w.to(DEV), ws, ops.new_status(DEV), act)       # the kernel the step would take
    torch.testing.assert_close(out.float().cpu(), want, atol=2e-2, rtol=2e-2)
    out.zero_()
    ops.gemm_tc(out, x.to(DEV), w.to(DEV), gated=True, activation=act)
    ops.check_status(ops.tc_status(DEV))
    torch.testing.assert_close(out.float().cpu(), want, atol=2e-2, rtol=2e-2)
    if rows <= 64:
        out.zero_()
        ops.gemm_skinny(out, x.to(DEV), w.to(DEV), gated=True, activation=act)
        torch.testing.assert_close(out.float().cpu(), want, atol=2e-2, rtol=2e-2)
    # the plain SiLU form is what it was
    out.zero_()
    ops.gated_linear(out, x.to(DEV), w.to(DEV), ws, ops.new_status(DEV))
    silu = (torch.nn.functional.silu(gu[:, :I]) * gu[:, I:]).float()
    torch.testing.assert_close(out.float().cpu(), silu, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,heads,N,K", [(1, 3, 48, 24), (19, 5, 7, 130), (100, 2, 96, 40), (33, 1, 64, 64), (8, 6, 50, 64),
                                            (32, 2, 128, 16)])
def test_per_head_products(rows, heads, N, K, dtype):
    from lyapunov_engine_b200 import ops
    g = torch.Generator().manual_seed(rows + K)
    wide = torch.randn(rows, heads * K + 8, generator=g).to(dtype)         # the operand is a column range of a wider buffer
    w = (torch.randn(heads, N, K, generator=g) / math.sqrt(K)).to(dtype)
    gate = torch.randn(rows, heads + 3, generator=g).to(dtype)
    a_dev = wide.to(DEV)[:, :heads * K]
    want = torch.einsum("thk,hnk->thn", wide[:, :heads * K].double().view(rows, heads, K), w.double())
    tol = dict(atol=1e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)
    out = torch.zeros(rows, heads * N, dtype=dtype, device=DEV)
    ops.gemm_heads(out, a_dev, w.to(DEV))
    torch.testing.assert_close(out.float().cpu(), want.reshape(rows, -1).float(), **tol)
    out.zero_()
    ops.gemm_heads(out, a_dev, w.to(DEV), gate.to(DEV)[:, 1:1 + heads])
    gated = want * torch.sigmoid(gate[:, 1:1 + heads].double())[:, :, None]
    torch.testing.assert_close(out.float().cpu(), gated.reshape(rows, -1).float(), **tol)
    # the gate alone, as the many-row path applies it
    plain = want.reshape(rows, -1).to(dtype).to(DEV).contiguous()
    ops.head_gate(plain, gate.to(DEV)[:, 1:1 + heads], heads, N)
    torch.testing.assert_close(plain.float().cpu(), gated.reshape(rows, -1).float(), **tol)
    if dtype == torch.float32:
        # a row's result does not depend on the rows beside it (the kernel has a form for up to 32 rows and one for more)
        few = 1 if rows <= 32 else 33
        part = torch.zeros(few, heads * N, dtype=dtype, device=DEV)
        ops.gemm_heads(part, a_dev[rows - few:], w.to(DEV), gate.to(DEV)[rows - few:, 1:1 + heads])
        assert torch.equal(part[-1], out[rows - 1])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_cache_writes(dtype):
    from lyapunov_engine_b200 import ops
    g = torch.Generator().manual_seed(3)
    page, pages, nkv, hd, rank, padded = 4, 9, 2, 16, 20, 32
    positions = torch.tensor([0, 1, 2, 7, 8, 5], dtype=torch.int32)
    request = torch.tensor([0, 0, 0, 1, 1, 2], dtype=torch.int32)
    table = torch.tensor([[3, 8, 8], [1, 0, 6], [8, 5, 8]], dtype=torch.int32)
    src = torch.randn(6, 100, generator=g).to(dtype)
    status = ops.new_status(DEV)
    k = torch.full((pages, nkv, page, hd), 5.0, dtype=dtype, device=DEV)
    v = torch.full((pages, nkv, page, hd), 5.0, dtype=dtype, device=DEV)
    ops.kv_store(src.to(DEV), 8, 8 + nkv * hd, k, v, positions.to(DEV), request.to(DEV), table.to(DEV), nkv, hd, page, status)
    latent = torch.full((pages, 1, page, padded), 5.0, dtype=dtype, device=DEV)
    weight = 1.0 + 0.3 * torch.randn(rank, generator=g)
    ops.latent_norm_store(src.to(DEV), 72, rank, weight.to(DEV), 1e-5, latent, positions.to(DEV), request.to(DEV),
                          table.to(DEV), page, status)
    ops.check_status(status)
    written = set()
    tol = dict(atol=1e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)
    for t in range(6):
        p, b = int(positions[t]), int(request[t])
        pg, off = int(table[b, p // page]), p % page
        written.add((pg, off))
        assert torch.equal(k[pg, :, off].cpu().reshape(-1), src[t, 8:8 + nkv * hd])
        assert torch.equal(v[pg, :, off].cpu().reshape(-1), src[t, 8 + nkv * hd:8 + 2 * nkv * hd])
        c = src[t, 72:72 + rank].double()
        c = c / torch.sqrt(c.pow(2).mean() + 1e-5) * weight.double()
        torch.testing.assert_close(latent[pg, 0, off, :rank].float().cpu(), c.float(), **tol)
        assert float(latent[pg, 0, off, rank:].float().abs().max()) == 0.0
    for pg in range(pages):
        for off in range(page):
            if (pg, off) not in written:
                assert float((k[pg, :, off].float() - 5.0).abs().max()) == 0.0 and float((latent[pg, 0, off].float() - 5.0).abs().max()) == 0.0
    # a page outside the pool is refused, not followed
    bad = table.clone(); bad[0, 0] = 99
    ops.kv_store(src.to(DEV), 8, 8 + nkv * hd, k, v, positions.to(DEV), request.to(DEV), bad.to(DEV), nkv, hd, page, status)
    with pytest.raises(ops.KernelError):
        ops.check_status(status)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,heads,d,rank", [(1, 3, 24, 48), (8, 8, 32, 128), (19, 2, 16, 20), (32, 5, 64, 72)])
def test_latent_prepare_equals_its_two_kernels(rows, heads, d, rank, dtype):
    from lyapunov_engine_b200 import ops
    g = torch.Generator().manual_seed(rows + rank)
    padded = (rank + 15) // 16 * 16
    col = (heads * d + 7) // 8 * 8
    src = torch.randn(rows, col + (rank + 7) // 8 * 8 + 8, generator=g).to(dtype).to(DEV)
    w_into = torch.zeros(heads, padded, d)
    w_into[:, :rank] = torch.randn(heads, rank, d, generator=g) / math.sqrt(d)
    w_into = w_into.to(dtype).to(DEV)
    weight = (1.0 + 0.3 * torch.randn(rank, generator=g)).to(DEV)
    page, pages = 4, 12
    positions = torch.arange(5, 5 + rows, dtype=torch.int32, device=DEV)
    request = torch.zeros(rows, dtype=torch.int32, device=DEV)
    table = torch.randperm(pages - 1, generator=g)[:10].to(torch.int32).view(1, 10).to(DEV)
    status = ops.new_status(DEV)
    caches = [torch.full((pages, 1, page, padded), 3.0, dtype=dtype, device=DEV) for _ in range(2)]
    two = torch.zeros(rows, heads * padded, dtype=dtype, device=DEV)
    ops.latent_norm_store(src, col, rank, weight, 1e-5, caches[0], positions, request, table, page, status)
    ops.gemm_heads(two, src[:, :heads * d], w_into)
    one = torch.zeros_like(two)
    assert ops.latent_prepare_applies(src, d)
    ops.latent_prepare(one, src, w_into, col, rank, weight, 1e-5, caches[1], positions, request, table, page, status)
    ops.check_status(status)
    assert torch.equal(one, two) and torch.equal(caches[0], caches[1])
    want = torch.einsum("thk,hnk->thn", src[:, :heads * d].double().cpu().view(rows, heads, d), w_into.double().cpu())
    tol = dict(atol=1e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)
    torch.testing.assert_close(one.float().cpu(), want.reshape(rows, -1).float(), **tol)
    # a run that reads another run's cache stores nothing
    kept = caches[1].clone()
    caches[1].fill_(1.0)
    ops.latent_prepare(one, src, w_into, col, rank, weight, 1e-5, None, positions, request, table, page, status)
    assert float((caches[1].float() - 1.0).abs().max()) == 0.0 and torch.equal(one, two) and kept is not None


# ---------------------------------------------------------------- attention over chunks, a factor per head
def chunk_case(dtype, nh, nkv, hd, page, q_lens, ctx_before, chunk, seed, head_scale, latent=False):
    """Keys and values of every request in scattered pages (stale values
    elsewhere), queries for the step's tokens, and the plain result.  For every
    request the key at the start of the last query's chunk answers that query
    strongly, and so does the key just before it, which the query must not
    see.  ``latent``: one pool is keys and values."""
    g = torch.Generator().manual_seed(seed)
    B = len(q_lens)
    totals = [c + q for c, q in zip(ctx_before, q_lens)]
    max_blocks = max((t + page - 1) // page for t in totals) + 1
    need = sum((t + page - 1) // page for t in totals)
    num_pages = need + 3
    perm = torch.randperm(num_pages - 1, generator=g)[:need].tolist()
    table = torch.full((B, max_blocks), num_pages - 1, dtype=torch.int32)
    k_cache = torch.randn(num_pages, nkv, page, hd, generator=g).to(dtype)
    v_cache = k_cache if latent else torch.randn(num_pages, nkv, page, hd, generator=g).to(dtype)
    T = sum(q_lens)
    q = torch.randn(T, nh * hd, generator=g)
    want = torch.zeros(T, nh * hd, dtype=torch.float64)
    scale = 0.9 / math.sqrt(hd)
    nxt, t0 = 0, 0
    for b in range(B):
        n = totals[b]
        k = torch.randn(nkv, n, hd, generator=g)
        last = n - 1
        start = last // chunk * chunk if chunk else 0
        t_last = t0 + q_lens[b] - 1
        for h in range(nh):
            sign = 1.0 if head_scale is None else math.copysign(1.0, float(head_scale[h]))
            spike = q[t_last, h * hd:(h + 1) * hd] * 1.5 * sign
            if h % (nh // nkv) == 0:
                k[h // (nh // nkv), start] = spike                     # just inside
                if start > 0:
                    k[h // (nh // nkv), start - 1] = spike * 1.3       # just outside, and louder
        k = k.to(dtype)
        v = k if latent else torch.randn(nkv, n, hd, generator=g).to(dtype)
        for i in range((n + page - 1) // page):
            pg = perm[nxt]; nxt += 1
            table[b, i] = pg
            m = min(page, n - i * page)
            k_cache[pg, :, :m] = k[:, i * page:i * page + m]
            if not latent:
                v_cache[pg, :, :m] = v[:, i * page:i * page + m]
        qb = q[t0:t0 + q_lens[b]].to(dtype).double().view(q_lens[b], nh, hd).transpose(0, 1)
        pos = torch.arange(ctx_before[b], n)
        keys = torch.arange(n)
        visible = keys[None, :] <= pos[:, None]
        if chunk:
            visible &= (keys[None, :] // chunk) == (pos[:, None] // chunk)
        s = scale * (torch.tensor(head_scale, dtype=torch.float64) if head_scale is not None else 1.0)
        o = ps.masked_softmax_attention(qb, k.double().repeat_interleave(nh // nkv, 0),
                                        v.double().repeat_interleave(nh // nkv, 0), s, visible)
        want[t0:t0 + q_lens[b]] = o.transpose(0, 1).reshape(q_lens[b], nh * hd)
        t0 += q_lens[b]
    cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32)
    hs = torch.tensor(head_scale, dtype=torch.float32, device=DEV) if head_scale is not None else None
    k_dev = k_cache.to(DEV)
    return dict(q=q.to(dtype).to(DEV), k=k_dev, v=k_dev if latent else v_cache.to(DEV), table=table.to(DEV),
                cu=cu.to(DEV), ctx=torch.tensor(ctx_before, dtype=torch.int32, device=DEV), want=want.float(), T=T,
                scale=scale, head_scale=hs)


CHUNK_CASES = [
    # nh, nkv, hd, page, q_lens, ctx_before, chunk, head_scale, latent
    (4, 2, 16, 4, [5, 1, 17, 1], [0, 9, 3, 10], 10, [1.0, 0.5, 2.0, 1.5], False),
    (6, 3, 48, 16, [40, 1, 1, 1, 2], [100, 119, 120, 121, 239], 120, [1.3, 0.7, 1.0, 1.9, 0.6, 1.1], False),
    (2, 2, 32, 8, [1, 1, 1], [63, 64, 65], 64, [1.0, -0.8], False),               # a negative factor turns the order of scores
    (4, 1, 64, 16, [130, 1, 3], [200, 511, 30], 96, [0.5, 1.0, 1.5, 2.0], False),   # tcgen05 prefill with factors
    (8, 1, 128, 16, [150, 1, 1, 2], [0, 700, 129, 64], None, None, True),           # latents: all heads on one pool
    (3, 1, 80, 8, [9, 1], [30, 77], 33, None, True),
    (5, 1, 160, 16, [20, 1], [3, 300], None, None, True),                           # beyond the tensor-core kernels
]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("case", CHUNK_CASES)
def test_chunks_and_head_factors_fp32_pipe_kernel(case, dtype):
    from lyapunov_engine_b200 import ops
    nh, nkv, hd, page, q_lens, ctx_before, chunk, head_scale, latent = case
    c = chunk_case(dtype, nh, nkv, hd, page, q_lens, ctx_before, chunk, hd + page, head_scale, latent)
    out = torch.zeros(c["T"], nh * hd, dtype=dtype, device=DEV)
    status = ops.new_status(DEV)
    tr, tq, n = _tiles(q_lens, 16)
    ops.attention_generic(out, c["q"], c["q"].stride(0), c["k"], c["v"], c["table"], c["cu"], c["ctx"], tr, tq, n,
                          nh, nkv, hd, page, ops.reach_code(chunk=chunk), c["scale"], status, head_scale=c["head_scale"])
    ops.check_status(status)
    tol = dict(atol=3e-5, rtol=1e-4) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)
    torch.testing.assert_close(out.float().cpu(), c["want"], **tol)


@pytest.mark.parametrize("case", [c for c in CHUNK_CASES if c[2] <= 128])
def test_chunks_and_head_factors_tensor_core_kernels(case):
    """Requests with several tokens through the prefill kernels (mma.sync, and
    tcgen05 where it exists and the factors are positive), single tokens
    through the split-key kernel with several split counts."""
    from lyapunov_engine_b200 import ops
    nh, nkv, hd, page, q_lens, ctx_before, chunk, head_scale, latent = case
    dtype = torch.bfloat16
    c = chunk_case(dtype, nh, nkv, hd, page, q_lens, ctx_before, chunk, hd + page + 1, head_scale, latent)
    reach = ops.reach_code(chunk=chunk)
    multi = [b for b, n in enumerate(q_lens) if n > 1]
    single = [b for b, n in enumerate(q_lens) if n == 1]
    variants = [(1, ops.attention_prefill_bf16), (3, ops.attention_prefill_bf16), (12, ops.attention_prefill_bf16)]
    if ops.attention_tc_available(hd, page) and (head_scale is None or min(head_scale) > 0):
        variants.append((2, ops.attention_prefill_tc_bf16))
    for splits, prefill in variants:
        status = ops.new_status(DEV)
        out = torch.full((c["T"], nh * hd), 7.0, dtype=dtype, device=DEV)
        if multi:
            req, q0 = [], []
            for b in multi:
                for s in range(0, q_lens[b], 128):
                    req.append(b); q0.append(s)
            prefill(out, c["q"], c["q"].stride(0), c["k"], c["v"], c["table"], c["cu"], c["ctx"],
                    torch.tensor(req, dtype=torch.int32, device=DEV), torch.tensor(q0, dtype=torch.int32, device=DEV),
                    len(req), nh, nkv, hd, page, reach, c["scale"], status, head_scale=c["head_scale"])
        if single:
            floats = ops.attention_decode_scratch_floats(hd, len(single), nh, splits)
            scratch = torch.zeros(max(floats, 1), dtype=torch.float32, device=DEV)
            ops.attention_decode_bf16(out, scratch, c["q"], c["q"].stride(0), c["k"], c["v"], c["table"], c["cu"], c["ctx"],
                                      torch.tensor(single, dtype=torch.int32, device=DEV), len(single), nh, nkv, hd, page,
                                      reach, c["scale"], splits, status, head_scale=c["head_scale"])
        ops.check_status(status)
        torch.testing.assert_close(out.float().cpu(), c["want"], atol=2.5e-2, rtol=2.5e-2)
