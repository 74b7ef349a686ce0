"""Each mechanism of the Kaditar design alone, the kernel against the plain
function of tests/plain_kaditar.py (or plain torch in 64 bits): the stream in
several copies with its norm, rotary pairs over segmented heads with bias and
cache write, the combination of a head's maps, the relu gate in its kernels,
the router, the grouping of pairs by expert, the experts' products, the
weighted sum, and the capped logits."""
import pytest
import torch

import plain_kaditar as pk

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("W,S,parts", [(96, 3, 0), (208, 4, 2), (100, 1, 1), (2048, 2, 0), (66, 8, 3), (4096, 4, 1)])
def test_stream_copies_update_read_and_layer_norm(W, S, parts, dtype):
    from lyapunov_engine_b200 import ops
    g = torch.Generator().manual_seed(W + S)
    T = 7
    x = torch.randn(T, S, W, generator=g) * 5.0 + 3.0         # a mean far from zero: a norm without the mean shows
    y = torch.randn(parts or 1, T, W, generator=g)
    delta = (y if parts else y[0].to(dtype)).contiguous()
    mix = torch.eye(S) + 0.3 * torch.randn(S, S, generator=g)
    post, pre = torch.randn(S, generator=g), torch.randn(S, generator=g)
    w, b = 1.0 + 0.3 * torch.randn(W, generator=g), 0.5 * torch.randn(W, generator=g)
    ysum = delta.double().sum(0) if parts else delta.double()
    new = torch.einsum("st,bsw->btw", mix.double(), x.double()) + post.double()[None, :, None] * ysum[:, None, :]
    u = torch.einsum("s,bsw->bw", pre.double(), new)
    want = pk.layer_norm(u, w.double(), b.double(), 1e-5).float()
    streams = x.clone().to(DEV)
    out = torch.zeros(T, W, dtype=dtype, device=DEV)
    ops.stream_norm(out, streams, w.to(DEV), b.to(DEV), 1e-5, delta=delta.to(DEV), mix=mix.to(DEV).contiguous(),
                    post=post.to(DEV), pre=pre.to(DEV))
    tol = dict(atol=2e-5, rtol=2e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)
    torch.testing.assert_close(streams.cpu(), new.float(), atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(out.float().cpu(), want, **tol)
    # chosen rows, the plain sum of the copies, nothing written back; the update is still pending
    kept = x.clone().to(DEV)
    rows = torch.tensor([5, 0, 2], dtype=torch.int32, device=DEV)
    some = torch.zeros(3, W, dtype=dtype, device=DEV)
    ops.stream_norm(some, kept, w.to(DEV), b.to(DEV), 1e-5, delta=delta.to(DEV), mix=mix.to(DEV).contiguous(),
                    post=post.to(DEV), pre=None, rows=rows)
    assert torch.equal(kept.cpu(), x)
    want_sum = pk.layer_norm(new.sum(1), w.double(), b.double(), 1e-5).float()[[5, 0, 2]]
    torch.testing.assert_close(some.float().cpu(), want_sum, **tol)
    # every copy starts as one row; without bias the norm is the root-mean-square one
    first = torch.randn(T, W, generator=g)
    fresh = torch.full((T, S, W), 9.0, device=DEV)
    ops.stream_norm(out, fresh, w.to(DEV), None, 1e-5, pre=pre.to(DEV), init=first.to(DEV))
    assert torch.equal(fresh.cpu(), first[:, None, :].expand(T, S, W))
    u = first.double() * pre.double().sum()
    rms = u / torch.sqrt((u * u).mean(-1, keepdim=True) + 1e-5) * w.double()
    torch.testing.assert_close(out.float().cpu(), rms.float(), **tol)
    total = torch.zeros(T, W, device=DEV)
    ops.stream_sum(total, streams)
    torch.testing.assert_close(total.cpu(), new.sum(1).float(), atol=1e-4, rtol=1e-5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,segs,d,e,rot,base", [(4, 2, 2, 40, 80, 16, 1e6), (2, 1, 2, 20, 12, 10, 1e4), (3, 3, 1, 16, 16, 16, 1e4),
                                                   (2, 2, 2, 8, 40, 0, 1.0), (1, 1, 3, 10, 7, 6, 50.0)])
def test_rotary_pairs_bias_spread_queries_and_cache_write(H, G, segs, d, e, rot, base, dtype):
    from lyapunov_engine_b200 import ops
    g = torch.Generator().manual_seed(H * 100 + d)
    hd = (max(segs * d, e) + 15) // 16 * 16
    page, pages = 4, 9
    pos = torch.tensor([0, 1, 2, 3, 4, 5, 17, 33, 1000, 30001], dtype=torch.int32)
    # two requests; tokens of request 1 sit at large positions (their pages are given below)
    req = torch.tensor([0, 0, 0, 0, 0, 0, 1, 1, 1, 1], dtype=torch.int32)
    T = pos.numel()
    table = torch.full((2, 30001 // page + 1), pages, dtype=torch.int32)
    table[0, 0], table[0, 1] = 3, 5
    table[1, 17 // page], table[1, 33 // page], table[1, 1000 // page], table[1, 30001 // page] = 0, 7, 2, 8
    cols = (H + G) * segs * d + G * e
    src = torch.randn(T, cols, generator=g).to(dtype)
    bias = torch.randn(cols, generator=g)
    k_cache = torch.full((pages + 1, G, page, hd), 7.0, dtype=dtype, device=DEV)
    v_cache = torch.full((pages + 1, G, page, hd), 7.0, dtype=dtype, device=DEV)
    q_out = torch.full((T, H * segs * hd), 7.0, dtype=dtype, device=DEV)
    i = torch.arange(0, rot, 2, dtype=torch.float64)
    rates = torch.pow(torch.tensor(base, dtype=torch.float64), -i / max(rot, 1)).float()
    status = ops.new_status(DEV)
    ops.rope_pairs_store(q_out, src.to(DEV), bias.to(DEV), k_cache, v_cache, rates.to(DEV), pos.to(DEV), req.to(DEV),
                         table.to(DEV), H, G, segs, d, e, rot, hd, page, True, status)
    ops.check_status(status)
    x = src.double() + bias.double()
    q = x[:, :H * segs * d].view(T, H * segs, d).transpose(0, 1)
    k = x[:, H * segs * d:(H + G) * segs * d].view(T, G * segs, d).transpose(0, 1)
    v = x[:, (H + G) * segs * d:].view(T, G, e)
    # (the kernel's angle is the 32-bit product position * rate)
    q, k = pk.rotate_pairs(q, pos, rot, base), pk.rotate_pairs(k, pos, rot, base)
    tol = dict(atol=3e-3, rtol=1e-5) if dtype == torch.float32 else dict(atol=3e-2, rtol=2e-2)
    got_q = q_out.float().cpu().view(T, H * segs, hd)
    for qh in range(H * segs):
        seg = qh % segs
        torch.testing.assert_close(got_q[:, qh, seg * d:(seg + 1) * d], q[qh].float(), **tol)
        rest = torch.cat([got_q[:, qh, :seg * d], got_q[:, qh, (seg + 1) * d:]], dim=1)
        assert float(rest.abs().max()) == 0.0 if rest.numel() else True
    small = slice(0, 8)                       # positions where the 32-bit angle is all but exact
    tight = dict(atol=2e-5, rtol=1e-5) if dtype == torch.float32 else tol
    torch.testing.assert_close(got_q[small, 0, :d], q[0][small].float(), **tight)
    for t in range(T):
        pg = int(table[int(req[t]), int(pos[t]) // page])
        for kvh in range(G):
            row_k = k_cache[pg, kvh, int(pos[t]) % page].float().cpu()
            row_v = v_cache[pg, kvh, int(pos[t]) % page].float().cpu()
            want_k = torch.cat([k[kvh * segs + s][t] for s in range(segs)]).float()
            torch.testing.assert_close(row_k[:segs * d], want_k, **tol)
            torch.testing.assert_close(row_v[:e], v[t, kvh].float(), **(tight if dtype == torch.float32 else tol))
            assert float(row_k[segs * d:].abs().max() if segs * d < hd else 0.0) == 0.0
            assert float(row_v[e:].abs().max() if e < hd else 0.0) == 0.0
    # a page outside the pool is refused, not followed
    table[0, 0] = pages + 5
    ops.rope_pairs_store(q_out, src.to(DEV), None, k_cache, v_cache, rates.to(DEV), pos.to(DEV), req.to(DEV), table.to(DEV),
                         H, G, segs, d, e, rot, hd, page, True, status)
    with pytest.raises(ops.KernelError):
        ops.check_status(status)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,segs,hd,e", [(4, 2, 80, 80), (3, 2, 48, 12), (1, 2, 16, 7), (2, 3, 64, 40)])
def test_maps_of_a_head_combined(H, segs, hd, e, dtype):
    from lyapunov_engine_b200 import ops
    g = torch.Generator().manual_seed(hd + e)
    T = 6
    attn = torch.randn(T, H * segs * hd, generator=g).to(dtype)
    coef = torch.tensor([1.0, -0.73, 0.4][:segs])
    out = torch.zeros(T, H * e, dtype=dtype, device=DEV)
    ops.maps_combine(out, attn.to(DEV), coef.to(DEV), H, segs, hd, e, 1e-5, 0.7)
    a = attn.double().view(T, H, segs, hd)[..., :e]
    o = (a * coef.double()[None, None, :, None]).sum(2)
    want = (o / torch.sqrt((o * o).mean(-1, keepdim=True) + 1e-5) * 0.7).reshape(T, H * e).float()
    tol = dict(atol=1e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)
    torch.testing.assert_close(out.float().cpu(), want, **tol)
    ops.maps_combine(out, attn.to(DEV), coef.to(DEV), H, segs, hd, e, None, 2.0)
    torch.testing.assert_close(out.float().cpu(), (2.0 * o).reshape(T, H * e).float(), **tol)


def test_differential_attention_maps_through_the_paged_kernels():
    """Two maps per head as twice the query heads over keys that hold both maps
    side by side: every attention kernel of the package against the plain
    softmax per map, with one loud key just outside the window and a fainter
    one just inside (a window one key too long would hear the loud one)."""
    from lyapunov_engine_b200 import ops
    from lyapunov_engine_b200.parts import attention_kernels  # noqa: F401
    H, G, d, e, window, page = 2, 1, 16, 32, 9, 4
    hd = 32
    T = 40
    g = torch.Generator().manual_seed(1)
    q = torch.randn(H, 2, T, d, generator=g, dtype=torch.float64)
    k = torch.randn(G, 2, T, d, generator=g, dtype=torch.float64)
    v = torch.randn(T, G, e, generator=g, dtype=torch.float64)
    t0 = 30
    k[0, 0, t0 - window] = 6.0 * q[0, 0, t0]            # just outside: must not be heard
    k[0, 0, t0 - window + 1] = 3.0 * q[0, 0, t0]        # just inside: decides map 1 of head 0
    visible = pk.window_mask(T, window)
    want = torch.stack([pk.softmax_attention(q[h, m], k[0, m], v[:, 0], 0.5, visible) for h in range(H) for m in range(2)], dim=1)
    assert float((torch.softmax((q[0, 0, t0] @ k[0, 0].T * 0.5).masked_fill(~visible[t0], -1e30), -1))[t0 - window + 1]) > 0.99
    for dtype in (torch.float32, torch.bfloat16):
        q_wide = torch.zeros(T, H * 2, hd, dtype=torch.float64)
        for h in range(H):
            for m in range(2):
                q_wide[:, h * 2 + m, m * d:(m + 1) * d] = q[h, m]
        pages = (T + page - 1) // page
        k_cache = torch.zeros(pages + 1, G, page, hd, dtype=dtype, device=DEV)
        v_cache = torch.zeros(pages + 1, G, page, hd, dtype=dtype, device=DEV)
        perm = torch.randperm(pages, generator=g)
        for t in range(T):
            k_cache[perm[t // page], 0, t % page] = torch.cat([k[0, 0, t], k[0, 1, t]]).to(dtype)
            v_cache[perm[t // page], 0, t % page] = v[t, 0].to(dtype)
        table = perm.to(torch.int32)[None, :].contiguous().to(DEV)
        qd = q_wide.view(T, -1).to(dtype).to(DEV)
        out = torch.zeros(T, H * 2 * hd, dtype=dtype, device=DEV)
        status = ops.new_status(DEV)
        cu = torch.tensor([0, T], dtype=torch.int32, device=DEV)
        before = torch.tensor([0], dtype=torch.int32, device=DEV)
        tile = 16
        tr = torch.zeros((T + tile - 1) // tile, dtype=torch.int32, device=DEV)
        tq = torch.arange(0, T, tile, dtype=torch.int32, device=DEV)
        ops.attention_generic(out, qd, qd.stride(0), k_cache, v_cache, table, cu, before, tr, tq, tr.numel(), H * 2, G, hd,
                              page, window, 0.5, status)
        ops.check_status(status)
        tol = dict(atol=2e-5, rtol=2e-5) if dtype == torch.float32 else dict(atol=3e-2, rtol=3e-2)
        torch.testing.assert_close(out.float().cpu().view(T, H * 2, hd), want.float(), **tol)
        if dtype == torch.bfloat16:
            out2 = torch.zeros_like(out)
            tr = torch.zeros(1, dtype=torch.int32, device=DEV)
            tq = torch.zeros(1, dtype=torch.int32, device=DEV)
            ops.attention_prefill_bf16(out2, qd, qd.stride(0), k_cache, v_cache, table, cu, before, tr, tq, 1, H * 2, G, hd,
                                       page, window, 0.5, status)
            ops.check_status(status)
            torch.testing.assert_close(out2.float().cpu().view(T, H * 2, hd), want.float(), **tol)
            # the last token alone, as a decoded one, with every split count
            for splits in (1, 2, 3):
                one = torch.zeros(1, H * 2 * hd, dtype=dtype, device=DEV)
                scratch = torch.zeros(max(1, ops.attention_decode_scratch_floats(hd, 1, H * 2, splits)), device=DEV)
                ops.attention_decode_bf16(one, scratch, qd[t0:t0 + 1], qd.stride(0), k_cache, v_cache, table,
                                          torch.tensor([0, 1], dtype=torch.int32, device=DEV),
                                          torch.tensor([t0], dtype=torch.int32, device=DEV), None, 1, H * 2, G, hd, page,
                                          window, 0.5, splits, status)
                ops.check_status(status)
                torch.testing.assert_close(one.float().cpu().view(H * 2, hd), want[t0].float(), **tol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_relu_gate_in_every_gated_kernel(dtype):
    from lyapunov_engine_b200 import ops
    from lyapunov_engine_b200.engine.runtime import Workspace
    g = torch.Generator().manual_seed(5)
    ws = Workspace(DEV)
    for T in (3, 200):
        K, F = 128, 256
        x = torch.randn(T, K, generator=g).to(dtype)
        w = (torch.randn(2 * F, K, generator=g) / K ** 0.5).to(dtype)
        out = torch.zeros(T, F, dtype=dtype, device=DEV)
        ops.gated_linear(out, x.to(DEV), w.to(DEV), ws, None, (ops.GLU_RELU, 1.0, 0.0))
        gu = x.double() @ w.double().T
        want = (torch.relu(gu[:, :F]) * gu[:, F:]).float()
        tol = dict(atol=1e-4, rtol=1e-4) if dtype == torch.float32 else dict(atol=3e-2, rtol=3e-2)
        torch.testing.assert_close(out.float().cpu(), want, **tol)
        assert float((out.float().cpu()[gu[:, :F] < -0.05]).abs().max()) == 0.0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,W,E,top,F,shared", [(5, 64, 6, 2, 24, 40), (70, 176, 12, 2, 56, 120), (9, 100, 3, 3, 20, 0),
                                                (33, 72, 1, 1, 16, 0), (300, 128, 40, 4, 36, 0), (700, 64, 4, 2, 200, 0)])
def test_routed_experts_step_by_step(T, W, E, top, F, shared, dtype):
    """Router, grouping, both products and the weighted sum, each against plain
    arithmetic, and the whole against the plain feed-forward."""
    from lyapunov_engine_b200 import ops
    g = torch.Generator().manual_seed(T + W + E)
    h = torch.randn(T, W, generator=g).to(dtype)
    wr = torch.randn(E, W, generator=g) / W ** 0.5 * 3.0
    br = torch.randn(E, generator=g)
    sg = torch.randn(W, generator=g) / W ** 0.5
    w = {"router": wr, "router.b": br}
    for e in range(E):
        w[f"e{e}.gate"] = (torch.randn(F, W, generator=g) / W ** 0.5).to(dtype).float()
        w[f"e{e}.up"] = (torch.randn(F, W, generator=g) / W ** 0.5).to(dtype).float()
        w[f"e{e}.down"] = (torch.randn(W, F, generator=g) / F ** 0.5).to(dtype).float()
    ids = torch.zeros(T, top, dtype=torch.int32, device=DEV)
    share = torch.zeros(T, top, device=DEV)
    gate = torch.zeros(T, device=DEV)
    ops.moe_route(ids, share, gate, h.to(DEV), wr.to(DEV), br.to(DEV), sg.to(DEV), top)
    z = h.double() @ wr.double().T + br.double()
    chosen = torch.topk(z, top, dim=-1)
    assert torch.equal(ids.cpu().long(), chosen.indices)
    torch.testing.assert_close(share.cpu(), torch.softmax(chosen.values, -1).float(), atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(gate.cpu(), torch.sigmoid(h.double() @ sg.double()).float(), atol=1e-5, rtol=1e-5)
    pairs = T * top
    wgu = torch.stack([torch.cat([w[f"e{e}.gate"], w[f"e{e}.up"]]) for e in range(E)]).to(dtype).to(DEV)
    wd = torch.stack([w[f"e{e}.down"] for e in range(E)]).to(dtype).to(DEV)
    flat = ids.cpu().view(-1)
    # the usual row tiles and, in bfloat16 with rows in 16-byte pieces, the wide ones of the tensor-core form
    for wide in ((False, True) if dtype == torch.bfloat16 and W % 8 == 0 and F % 8 == 0 else (False,)):
        max_tiles = ops.moe_max_tiles(pairs, E, wide)
        slots = torch.full((pairs,), -1, dtype=torch.int32, device=DEV)
        tiles = torch.zeros(3, max_tiles, dtype=torch.int32, device=DEV)
        meta = torch.zeros(4, dtype=torch.int32, device=DEV)
        ops.moe_group(ids, E, slots, tiles, meta, wide)
        n_tiles = int(meta[0])
        assert sorted(slots.cpu().tolist()) == list(range(pairs))             # every pair once
        assert torch.equal(flat[slots.cpu().long()], flat.sort().values)      # in expert order
        covered = []
        for i in range(n_tiles):
            e, first, rows = (int(tiles[j, i]) for j in range(3))
            assert 1 <= rows <= ops.moe_tile_rows(wide) and all(int(flat[slots[first + r]]) == e for r in range(rows))
            covered += list(range(first, first + rows))
        assert covered == list(range(pairs)) and n_tiles <= max_tiles
        act = torch.zeros(pairs, F, dtype=dtype, device=DEV)
        ops.moe_grouped(act, h.to(DEV), wgu, slots, tiles, meta, max_tiles, src_div=top, scatter=False, gated=True,
                        activation=(ops.GLU_SILU, 1.0, 0.0), wide=wide)
        y = torch.zeros(pairs, W, device=DEV)
        ops.moe_grouped(y, act, wd, slots, tiles, meta, max_tiles, src_div=0, scatter=True, pair_weight=share.view(-1), wide=wide)
        if wide:
            torch.testing.assert_close(y, y_narrow, atol=2e-2, rtol=2e-2)
        y_narrow = y
    shared_out = torch.randn(T, W, generator=g).to(dtype) if shared else None
    out = torch.zeros(T, W, dtype=dtype, device=DEV)
    ops.moe_combine(out, y, top, shared_out.to(DEV) if shared else None, gate if shared else None)
    cfg = {"router": {"experts": E, "top": top}}
    want = pk.routed_ff(h.double(), {k: v.double() for k, v in w.items()}, "", cfg)
    if shared:
        want = want + torch.sigmoid(h.double() @ sg.double())[:, None] * shared_out.double()
    tol = dict(atol=1e-4, rtol=1e-4) if dtype == torch.float32 else dict(atol=4e-2, rtol=4e-2)
    torch.testing.assert_close(out.float().cpu(), want.float(), **tol)
    if dtype == torch.bfloat16 and W % 8 == 0 and F % 8 == 0:
        # the form for many rows per expert: slots padded to whole tiles of 128, rows gathered, the tcgen05 product
        # in its grouped form twice, the weighted sum through each pair's slot
        max_tiles = ops.moe_max_tiles(pairs, E, True)
        rows = max_tiles * ops.moe_tile_rows(True)
        slots = torch.full((rows,), 12345, dtype=torch.int32, device=DEV)
        pair_slot = torch.full((pairs,), -7, dtype=torch.int32, device=DEV)
        tiles = torch.full((3, max_tiles), 99, dtype=torch.int32, device=DEV)
        ops.moe_group(ids, E, slots, tiles, meta, True, padded=True, pair_slot=pair_slot)
        n_tiles = int(meta[0])
        sl, ps = slots.cpu(), pair_slot.cpu()
        assert sorted(ps.tolist()) == sorted(i for i in range(n_tiles * 128) if sl[i] >= 0) and len(set(ps.tolist())) == pairs
        for pair in range(pairs):
            slot = int(ps[pair])
            assert int(sl[slot]) == pair and int(tiles[0, slot // 128]) == int(flat[pair])
        assert all(int(v) in (-1,) or 0 <= int(v) < pairs for v in sl[:n_tiles * 128])
        status = ops.new_status(DEV)
        x_sorted = torch.full((rows, W), 3.0, dtype=dtype, device=DEV)
        ops.moe_gather(x_sorted, h.to(DEV), slots, meta, top)
        for pair in (0, pairs // 2, pairs - 1):
            assert torch.equal(x_sorted[int(ps[pair])].cpu(), h[pair // top])
        act2 = torch.zeros(rows, F, dtype=dtype, device=DEV)
        ops.gemm_tc_grouped(act2, x_sorted, wgu, tiles[0], meta, gated=True, status=status, activation=(ops.GLU_SILU, 1.0, 0.0))
        y2 = torch.zeros(rows, W, device=DEV)
        ops.gemm_tc_grouped(y2, act2, wd, tiles[0], meta, status=status)
        ops.check_status(status)
        out2 = torch.zeros(T, W, dtype=dtype, device=DEV)
        ops.moe_combine_sorted(out2, y2, pair_slot, share, top, shared_out.to(DEV) if shared else None, gate if shared else None)
        torch.testing.assert_close(out2.float().cpu(), want.float(), **tol)


def test_router_prefers_the_lower_index_on_a_tie_and_ignores_the_rest():
    from lyapunov_engine_b200 import ops
    W, E = 32, 5
    wr = torch.zeros(E, W)
    wr[1, 0] = wr[3, 0] = 2.0        # experts 1 and 3 tie, expert 4 follows through its bias
    br = torch.tensor([0.0, 0.0, -1.0, 0.0, 1.5])
    h = torch.zeros(2, W)
    h[0, 0] = 1.0
    h[1, 0] = -1.0
    ids = torch.zeros(2, 3, dtype=torch.int32, device=DEV)
    share = torch.zeros(2, 3, device=DEV)
    ops.moe_route(ids, share, None, h.to(DEV), wr.to(DEV), br.to(DEV), None, 3)
    assert ids.cpu().tolist() == [[1, 3, 4], [4, 0, 2]]
    z = torch.tensor([[2.0, 2.0, 1.5], [1.5, 0.0, -1.0]])
    torch.testing.assert_close(share.cpu(), torch.softmax(z, -1), atol=1e-6, rtol=1e-6)


def test_capped_logits():
    from lyapunov_engine_b200 import ops
    x = torch.tensor([[-1000.0, -30.0, -1.0, 0.0, 0.5, 14.0, 29.0, 1e6]])
    got = x.clone().to(DEV)
    ops.softcap(got, 15.0)
    torch.testing.assert_close(got.cpu(), (15.0 * torch.tanh(x.double() / 15.0)).float(), atol=1e-5, rtol=1e-6)
