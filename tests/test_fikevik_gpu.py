"""Fikevik on the GPU: every mechanism's kernels against the plain implementation's function for it, then
whole models through the engine's step function, cache and state slots, scheduler and entry point."""
import math
import os

import numpy as np
import pytest
import torch

import plain_fikevik as P
import replay_util as R
from tiny_fikevik import TINY, load_folder, write_tiny

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def K():
    from rosellm_b200.ops import kernels

    return kernels


def rel(a: torch.Tensor, b: torch.Tensor) -> float:
    return float((a.double().cpu() - b.double().cpu()).abs().max() / (b.double().abs().max() + 1e-30))


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


# ---- mechanisms alone ------------------------------------------------------------------------------

def test_token_rows_are_scaled_in_float32():
    g = torch.Generator().manual_seed(1)
    table = torch.randn(30, 24, generator=g).to(torch.bfloat16)
    ids = torch.randint(0, 30, (11,), generator=g).to(torch.int32)
    for scale in (1.0, 7.3):
        out = torch.empty(11, 24, device=DEV)
        K().embed(ids.to(DEV), torch.arange(11, dtype=torch.int32, device=DEV), table.to(DEV), None, out, scale=scale)
        assert rel(out, P.embed(table.double(), ids.tolist(), scale)) < 1e-7


@pytest.mark.parametrize("width", [8, 100, 1000, 12000])
def test_join_of_stream_and_gated_results_with_the_norm_after_the_sum(width):
    """One result and two with a weight each, with and without a gate, stream weights of 1 and others; the
    bfloat16 copy of the new rows; rows too wide to be kept on chip between the two passes."""
    g = torch.Generator().manual_seed(width)
    n = 5
    x, y0, y1, z = (torch.randn(n, width, generator=g) * s for s in (1.0, 3.0, 0.5, 2.0))
    gamma = 1 + 0.2 * torch.randn(width, generator=g)
    for alpha, s0, s1, two, gate in ((2.0, 1.0, 0.0, False, True), (1.0, 0.6, 1.1, True, True), (0.5, 1.3, 0.2, True, False)):
        xs = x.to(DEV).clone()
        copy = torch.empty(n, width, dtype=torch.bfloat16, device=DEV)
        K().gated_join_norm(y0.to(DEV), s0, y1.to(DEV) if two else None, s1, z.to(DEV) if gate else None, gamma.to(DEV), 1e-5,
                            alpha, xs, copy)
        y = s0 * y0.double() + (s1 * y1.double() if two else 0.0)
        gt = torch.sigmoid(z.double()) if gate else 1.0
        want = P.unit(alpha * x.double() + gt * y, 1e-5) * gamma.double()
        assert rel(xs, want) < 2e-6
        assert rel(copy.float(), want) < 5e-3


def test_join_matches_the_plain_sublayer_join():
    """The gate's logits come from a product of the sublayer's input, as the part computes them."""
    g = torch.Generator().manual_seed(3)
    n, width = 9, 40
    x, y = torch.randn(n, width, generator=g), torch.randn(n, width, generator=g)
    w = {"rg": torch.randn(width, width, generator=g).double() * 0.3, "rg.b": torch.randn(width, generator=g).double(),
         "nw": 1 + 0.1 * torch.randn(width, generator=g).double()}
    z = (x.double() @ w["rg"].T + w["rg.b"]).float()
    xs = x.to(DEV).clone()
    K().gated_join_norm(y.to(DEV), 1.0, None, 0.0, z.to(DEV), w["nw"].float().to(DEV), 1e-6, 2.5, xs, None)
    assert rel(xs, P.sublayer_join(x.double(), y.double(), w, "rg", "nw", 2.5, 1e-6)) < 2e-6


@pytest.mark.parametrize("H,G,dk,dv,rot", [(6, 2, 20, 12, 12), (4, 4, 64, 32, 64), (7, 1, 9, 5, 8), (3, 3, 16, 24, 0),
                                           (2, 1, 136, 130, 136), (5, 5, 6, 6, 2)])
def test_norms_and_rotation_of_queries_keys_and_values(H, G, dk, dv, rot):
    """In place on columns of a wider matrix; pairs (2i, 2i + 1) of the first ``rot`` entries only; positions from
    0 to far out; with and without the norms' weights and the values' norm."""
    g = torch.Generator().manual_seed(H * dk)
    n = 13
    pos = torch.tensor([0, 1, 2, 3, 15, 16, 17, 100, 1000, 4097, 30000, 7, 8], dtype=torch.int32)
    widths = (H * dk, G * dk, G * dv)
    offs = (3, 3 + widths[0] + 5, 3 + widths[0] + 5 + widths[1] + 2)
    packed = torch.randn(n, offs[2] + widths[2] + 4, generator=g)
    qn, kn = 1 + 0.3 * torch.randn(dk, generator=g), 1 + 0.3 * torch.randn(dk, generator=g)
    base, eps = 700.0, 1e-5
    freq = torch.tensor([base ** (-2.0 * i / rot) for i in range(rot // 2)], dtype=torch.float32) if rot else None
    for normed, unit_v in ((True, True), (False, False), (True, False)):
        buf = packed.to(DEV).clone()
        q, k, v = (buf[:, o:o + w] for o, w in zip(offs, widths))
        K().qkv_norm_rotate(q, k, v, pos.to(DEV), n_heads=H, n_kv=G, dk=dk, dv=dv, eps=eps,
                            q_norm=qn.to(DEV) if normed else None, k_norm=kn.to(DEV) if normed else None,
                            freq=None if freq is None else freq.to(DEV), rot_dims=rot, unit_values=unit_v)
        pq, pk, pv = (packed[:, o:o + w].double() for o, w in zip(offs, widths))
        pq, pk, pv = pq.view(n, H, dk), pk.view(n, G, dk), pv.view(n, G, dv)
        if normed:
            pq, pk = P.unit(pq, eps) * qn.double(), P.unit(pk, eps) * kn.double()
        if rot:
            pq, pk = P.rotate_pairs(pq, pos, rot, base), P.rotate_pairs(pk, pos, rot, base)
        if unit_v:
            pv = P.unit(pv, eps)
        # the angle is a float32 product of a position up to 30000: half a unit in its last place is 1e-3 rad
        tol = 2e-6 if not rot else 2e-3
        assert rel(q.reshape(n, H, dk), pq) < tol and rel(k.reshape(n, G, dk), pk) < tol and rel(v.reshape(n, G, dv), pv) < 2e-6
        near = pos < 200  # where the angle is exact to 1e-5
        assert rel(q.reshape(n, H, dk)[near], pq[near]) < 2e-5
        keep = torch.ones(buf.shape[1], dtype=torch.bool)
        for o, w in zip(offs, widths):
            keep[o:o + w] = False
        assert torch.equal(buf[:, keep].cpu(), packed[:, keep])  # nothing beside the three is touched


def _window_case(dtype, H, G, dk, dv, lens_new, lens_old, page, scale, window, seed, stand_out=None, splits=1, mma=False):
    """Requests with ``lens_old`` cached tokens bring ``lens_new`` more.  All tokens' cache rows are written by the
    store kernel; then the pages that the window has passed before this step are taken away (their table
    entries -1, their rows overwritten with huge numbers), as the cache manager does.  Returns the kernel's
    output [tokens, H, dv] and the plain result from the same (rounded) keys and values."""
    from rosellm_b200.engine.context import build_host_batch

    dt = DTYPES[dtype]
    g = torch.Generator().manual_seed(seed)
    v_at = -(-dk // 8) * 8
    row = -(-(v_at + dv) // 8) * 8
    n_req = len(lens_new)
    totals = [a + b for a, b in zip(lens_new, lens_old)]
    pages_per = [-(-t // page) for t in totals]
    n_pages = sum(pages_per) + 3
    order = torch.randperm(n_pages, generator=g).tolist()
    table = torch.full((n_req + 1, max(pages_per)), -1, dtype=torch.int32)
    at = 0
    for r in range(n_req):
        for lp in range(pages_per[r]):
            table[r + 1, lp] = order[at]
            at += 1
    pool = torch.full((n_pages, 1, G, page, row), 9.0, dtype=dt, device=DEV)
    ks = [torch.randn(t, G, dk, generator=g) * 0.7 for t in totals]
    vs = [torch.randn(t, G, dv, generator=g) for t in totals]
    n_tok = sum(lens_new)
    q = torch.randn(n_tok, H, dk, generator=g) * 0.8
    temp = 0.5 + 1.5 * torch.rand(H, generator=g)
    if stand_out is not None:  # request 0's last query points hard at one key
        key, head = stand_out
        ks[0][key, head // (H // G)] = q[lens_new[0] - 1, head] * 40.0
    full = table.to(DEV)
    for new, old in ((lens_old, [0] * n_req), (lens_new, lens_old)):
        ents = [(r + 1, old[r], [0] * new[r], []) for r in range(n_req) if new[r] > 0]
        if not ents:
            continue
        hb = build_host_batch(ents)
        kk = torch.cat([ks[r][old[r]:old[r] + new[r]] for r in range(n_req) if new[r] > 0]).reshape(-1, G * dk)
        vv = torch.cat([vs[r][old[r]:old[r] + new[r]] for r in range(n_req) if new[r] > 0]).reshape(-1, G * dv)
        K().bias_kv_store(kk.to(DEV), vv.to(DEV), pool, full, dev(hb.positions), dev(hb.req_of_token), dev(hb.slots),
                          v_at=v_at, max_pos=max(totals))
    if window is not None:
        for r in range(n_req):
            gone = max(0, lens_old[r] - window + 1) // page
            for lp in range(gone):
                pool[int(table[r + 1, lp])] = 1e4
                table[r + 1, lp] = -1
    table = table.to(DEV)
    mma = mma and K().bias_attention_tensor_cores(dt, dk, dv)
    wide = K().bias_attention_shape(H // G, mma)[1] > 16
    tiles, n_tiles = (hb.tiles_wide, len(hb.tiles_wide)) if wide else (hb.tiles, len(hb.tiles))
    out = torch.full((n_tok, H * dv), 5.0, dtype=dt, device=DEV)
    part_o = part_ml = None
    if splits > 1:
        part_o = torch.full((len(hb.decode_reqs) * H * splits, dv), float("nan"), device=DEV)
        part_ml = torch.full((len(hb.decode_reqs) * H * splits, 2), float("nan"), device=DEV)
    K().bias_attention(q.reshape(n_tok, H * dk).to(DEV), None, pool, table, dev(hb.q_start), dev(hb.kv_len), dev(hb.slots), out,
                       n_heads=H, dk=dk, dv=dv, v_at=v_at, scale=scale, tiles=dev(tiles.reshape(-1)), n_tiles=n_tiles,
                       tile_tokens=64 if wide else 16, decode_reqs=dev(hb.decode_reqs), n_decode=len(hb.decode_reqs),
                       max_pos=max(totals), n_splits=splits, part_o=part_o, part_ml=part_ml, tensor_cores=mma,
                       window=window or 0, head_scale=temp.to(DEV))
    K().check_status(torch.device(DEV))
    want = torch.empty(n_tok, H, dv, dtype=torch.float64)
    t0 = 0
    for r in range(n_req):
        kc, vc = ks[r].to(dt).double(), vs[r].to(dt).double()  # what the cache holds
        qq = torch.zeros(totals[r], H, dk, dtype=torch.float64)
        qq[lens_old[r]:] = q[t0:t0 + lens_new[r]].double()
        want[t0:t0 + lens_new[r]] = P.window_softmax(qq, kc, vc, scale, temp.double(), window)[lens_old[r]:]
        t0 += lens_new[r]
    return out.float().cpu().view(n_tok, H, dv), want, vs


def _tol(dtype, mma=False):
    # with bfloat16 operands on the tensor cores the queries and the probabilities are rounded too
    return 2e-5 if dtype == "float32" else (2.5e-2 if mma else 1e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window", [1, 2, 7, 16, 17, 40, 100, 5000, None])
def test_windowed_attention_prompt_portions_and_single_tokens(dtype, window):
    """Windows of one key, within a page, of a page and one more, of several key tiles, wider than any context and
    none; portions that start inside a page, end on a page's border and are longer than the window, beside
    single tokens; one to forty heads a key/value head; pages the window has passed are gone."""
    for mma in ((False,) if dtype == "float32" else (False, True)):
        for H, G, dk, dv, page in ((6, 2, 20, 12, 16), (4, 4, 64, 32, 8), (40, 1, 8, 8, 32), (2, 1, 136, 130, 16), (16, 4, 128, 128, 16),
                                   (3, 1, 24, 200, 16)):
            got, want, _ = _window_case(dtype, H, G, dk, dv, [40, 1, 2, 17, 1, 16], [5, 130, 0, 15, 0, 16], page, 0.3, window, seed=H,
                                        mma=mma)
            assert rel(got, want) < _tol(dtype, mma), (H, G, dk, dv, mma)
            got, want, _ = _window_case(dtype, H, G, dk, dv, [33, 16, 2, 70, 130], [0, 31, 70, 63, 200], page, 0.2, window, seed=H + 9,
                                        mma=mma)
            assert rel(got, want) < _tol(dtype, mma), (H, G, dk, dv, mma, "portions only")
            got, want, _ = _window_case(dtype, H, G, dk, dv, [1, 1, 1, 1], [0, 31, 32, 300], page, 0.2, window, seed=H + 50, mma=mma)
            assert rel(got, want) < _tol(dtype, mma), (H, G, dk, dv, mma, "single tokens")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("splits", [2, 3, 8, 32])
@pytest.mark.parametrize("window", [40, 300, None])
def test_decoded_tokens_with_the_windows_keys_cut_into_parts(dtype, splits, window):
    """More parts than a window has tiles of keys (empty parts), parts that end inside a tile, windows that begin
    inside a tile, beside a prompt portion that is not cut."""
    got, want, _ = _window_case(dtype, 6, 2, 20, 10, [1, 1, 5, 1, 1], [700, 0, 40, 63, 64], 16, 0.25, window, seed=splits,
                                splits=splits)
    assert rel(got, want) < _tol(dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window", [1, 5, 16, 33, 64, 250])
def test_a_key_that_stands_out_counts_just_inside_the_window_and_not_just_outside(dtype, window):
    """One key is scored far above the rest.  As the earliest key the window keeps, the output is (nearly) its
    value; one position earlier it must leave no trace.  From a prompt portion's last query (on the CUDA cores
    and on the tensor cores) and from a decoded token's (whole and cut into parts), at contexts where the window's
    edge falls inside a page, on its border and in a page that is partly gone."""
    H, G, dk, dv, head = 4, 2, 24, 12, 3
    for total in (window + 3, 333, 900):
        last = total - 1
        for new, splits, mma in ((4, 1, False), (4, 1, True), (1, 1, False), (1, 5, False), (min(total, 70), 1, False)):
            old = total - new
            for key, inside in ((last - window + 1, True), (last - window, False)):
                if key < 0:
                    continue
                got, want, vs = _window_case(dtype, H, G, dk, dv, [new], [old], 16, 0.5, window, seed=key, stand_out=(key, head),
                                             splits=splits, mma=mma)
                # on the tensor cores the queries are rounded to bfloat16 too: the other rows of the portion, whose
                # scores with the scaled key are large and random, then differ by more than the key they should
                # see or not see would explain; the last row's do not
                rows = slice(-1, None) if mma and dtype == "bfloat16" else slice(None)
                assert rel(got[rows], want[rows]) < _tol(dtype, mma), (total, new, splits, mma, key, inside)
                value = vs[0][key, head // (H // G)].to(DTYPES[dtype]).double()
                hit = float((got[-1, head].double() - value).abs().max())
                if inside:
                    assert hit < 1e-2, (total, new, splits, mma, "the earliest key of the window was not seen")
                elif window > 1:
                    assert hit > 0.3, (total, new, splits, mma, "a key before the window was seen")


def _state_case(mode, dtype, H, dk, dv, lens, cuts, seed, rank=4, tau=4.0, cap=5.0, gate_spread=3.0, stale=True):
    """Requests of ``lens`` tokens run through the kernels in steps of ``cuts`` tokens each, their state carried in
    slots (which a slot's new owner finds zeroed, as the cache manager leaves them); compares with the plain
    recurrence on the whole sequences.  Returns the largest relative difference."""
    from rosellm_b200.engine.context import build_host_batch

    g = torch.Generator().manual_seed(seed)
    dt = DTYPES[dtype]
    n_req = len(lens)
    wk, wv = H * dk, H * dv
    if mode == "decayed_keys":
        names, widths = ("r", "k", "v", "g", "w"), (wk, wk, wv, wv, rank)
    else:
        names, widths = ("r", "k", "v", "g", "a", "w"), (wk, wk, wv, wv, H, H)
    offs, at = {}, 0
    for nme, w in zip(names, widths):
        offs[nme] = at
        at += -(-w // 8) * 8
    proj = [torch.randn(n, at, generator=g) for n in lens]
    for p_ in proj:
        if mode == "matrix_memory":  # gate logits on both sides of their cap
            p_[:, offs["a"]:offs["a"] + H] *= gate_spread
            p_[:, offs["w"]:offs["w"] + H] *= gate_spread
    eps, qscale = 1e-5, dk ** -0.5
    if mode == "decayed_keys":
        bias, w2 = 1.0 + 2.0 * torch.randn(wk, generator=g), torch.randn(wk, rank, generator=g)
        out_w = 1 + 0.3 * torch.randn(dv, generator=g)
        state = torch.zeros(n_req + 1, H, dk, dv, device=DEV)
    else:
        bi, bf = torch.randn(H, generator=g), 2.0 + torch.randn(H, generator=g)
        out_w = 1 + 0.3 * torch.randn(wv, generator=g)
        state = torch.zeros(n_req + 1, H * dk * (dv + 1) + H, device=DEV)
    got = [[] for _ in lens]
    done = [0] * n_req
    k = 0
    while any(d < n for d, n in zip(done, lens)):
        ents, take = [], []
        for r in range(n_req):
            if done[r] < lens[r]:
                n = min(cuts[k % len(cuts)], lens[r] - done[r])
                k += 1
                ents.append((r + 1, done[r], [0] * n, []))
                take.append((r, n))
        hb = build_host_batch(ents)
        pj = torch.cat([proj[r][done[r]:done[r] + n] for r, n in take]).to(DEV)
        out = torch.full((pj.shape[0], wv), 3.0, dtype=dt, device=DEV)
        m = K().RECURRENCES[mode]
        dvs = dv + 1 if mode == "matrix_memory" else dv
        prep = torch.full((H * pj.shape[0] * K().recurrence_record(m, dk, dvs),), float("nan"), device=DEV)
        oraw = torch.full((pj.shape[0], H * dvs), float("nan"), device=DEV)
        kw = dict(n_reqs=len(ents), n_heads=H, dk=dk, dv=dv, eps=eps, out_weight=out_w.to(DEV), qscale=qscale)
        if mode == "decayed_keys":
            kw.update(a_bias=bias.to(DEV), w0=bias.to(DEV), w2t=w2.t().contiguous().to(DEV), rank=rank, tau=tau)
        else:
            kw.update(a_bias=bi.to(DEV), w0=bf.to(DEV), cap=cap, floor_eps=1e-6,
                      gates=torch.full((pj.shape[0] * H * 4,), float("nan"), device=DEV))
        K().recurrence(m, pj, offs, state, out, dev(hb.q_start), dev(hb.slots), prep, oraw, **kw)
        at = 0
        for r, n in take:
            got[r].append(out[at:at + n].float().cpu())
            at += n
            done[r] += n
    K().check_status(torch.device(DEV))
    worst = 0.0
    for r, n in enumerate(lens):
        pr = proj[r].double()
        col = lambda nme, w: pr[:, offs[nme]:offs[nme] + w]
        qq, kk, vv = col("r", wk).view(n, H, dk) * qscale, col("k", wk).view(n, H, dk), col("v", wv).view(n, H, dv)
        if mode == "decayed_keys":
            z = (col("w", rank) @ w2.double().T + bias.double()).view(n, H, dk)
            o = P.unit(P.decay_recurrence(qq, kk, vv, torch.sigmoid(z) ** (1.0 / tau)), eps) * out_w.double()
            gl = col("g", wv).view(n, H, dv)
            want = o * gl * torch.sigmoid(gl)
        else:
            gi, gf = P.capped_log_gates(col("a", H) + bi.double(), col("w", H) + bf.double(), cap)
            o = P.unit(P.memory_recurrence(qq, kk, vv, gi, gf), eps)
            want = o * out_w.double().view(H, dv) * torch.sigmoid(col("g", wv).view(n, H, dv))
        worst = max(worst, rel(torch.cat(got[r]).view(n, H, dv), want))
    return worst


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("mode", ["decayed_keys", "matrix_memory"])
def test_state_mixers_whole_in_portions_and_token_by_token(mode, dtype):
    """Square and oblong states, sizes on both sides of the kernel's register tiers, portions that end on and
    inside the kernel's chunks of tokens, portions of two, single tokens; several requests a step."""
    tol = 5e-5 if dtype == "float32" else 6e-3
    for H, dk, dv in ((3, 24, 10), (2, 8, 40), (1, 64, 64), (6, 32, 64), (3, 128, 16), (2, 12, 136), (1, 130, 130), (4, 48, 64)):
        for cuts in ((1000,), (16, 1, 15, 17, 2, 33), (2,), (1,)):
            lens = [70, 1, 33] if cuts not in ((1,), (2,)) else [20, 3]
            assert _state_case(mode, dtype, H, dk, dv, lens, cuts, seed=dk + len(cuts)) < tol, (H, dk, dv, cuts)


@pytest.mark.parametrize("cuts", [(1000,), (1,), (7, 1, 64, 2)])
def test_the_memorys_running_maximum_over_a_long_sequence(cuts):
    """Wide gates (logits far beyond the cap, which then binds) and a narrow cap, over 400 tokens: the maximum
    starts at zero, rises with strong inputs and sinks with forgetting; its value is carried between steps."""
    for cap, spread in ((0.5, 5.0), (15.0, 8.0), (3.0, 0.2)):
        assert _state_case("matrix_memory", "float32", 2, 16, 24, [400, 37], cuts, seed=int(cap * 10), cap=cap,
                           gate_spread=spread) < 1e-4, (cap, spread)


@pytest.mark.parametrize("cuts", [(2000,), (511, 2, 513), (512,), (1024, 1)])
def test_the_memorys_gates_over_the_kernels_rounds_of_tokens(cuts):
    """The kernel of the running maximum takes a request's tokens in rounds of 512: portions longer than a round,
    and portions that end a token before a round's end, on it and a token after it; three requests a step."""
    assert _state_case("matrix_memory", "float32", 3, 16, 24, [1100, 513, 512], cuts, seed=3, cap=6.0,
                       gate_spread=3.0) < 1e-4, cuts
    assert _state_case("decayed_keys", "float32", 2, 16, 24, [1100, 513], cuts, seed=4, tau=8.0, rank=5) < 1e-4, cuts


@pytest.mark.parametrize("tau", [1.0, 16.0, 0.25])
def test_decays_from_nearly_none_to_nearly_all(tau):
    """tau stretches the decays towards one (a long memory) or squeezes them towards zero; 300 tokens whole
    against portions and single tokens."""
    for cuts in ((1000,), (1,), (5, 2, 90)):
        assert _state_case("decayed_keys", "float32", 3, 16, 8, [300, 2], cuts, seed=7, tau=tau, rank=6) < 5e-5, cuts


# ---- whole models through the step function ------------------------------------------------------------

@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = str(tmp_path_factory.mktemp("fikevik"))
    return {name: write_tiny(name, root) for name in TINY}


_plain: dict = {}


def plain_logits(folder, toks, how="exact"):
    """``exact``: float64.  ``float32``: the same functions on float32 tensors.  ``bfloat16``: float64 with the
    activations rounded to bfloat16 where a 16-bit engine stores them.  The last two show how far rounding alone
    moves the logits of this very sequence, which is what the tolerances below are tied to."""
    key = (folder, tuple(toks), how)
    if key not in _plain:
        if folder not in _plain:
            cfg, w = load_folder(folder)
            _plain[folder] = (cfg, w, {k: v.float() for k, v in w.items()})
        cfg, w, w32 = _plain[folder]
        if how == "float32":
            _plain[key] = P.forward(cfg, w32, toks).double()
        else:
            _plain[key] = P.forward(cfg, w, toks, rounding=P.to_bfloat16_and_back if how == "bfloat16" else None)
    return _plain[key]


def centred_rms(d):
    d = d - d.mean()
    return float(d.pow(2).mean().sqrt())


def row_limit(folder, toks, pos, dtype):
    """float32: 3e-4 on a logit, or five times what float32 rounding moves this row in the plain implementation.
    bfloat16: the row's error (mean taken off, root mean square over the vocabulary, over that of the plain row)
    0.12, or three times what bfloat16 storage moves this row.  The second figures matter where the model itself
    magnifies rounding: a matrix memory whose state one token dominates, read by a query nearly at right angles to
    that token's key, has an output whose direction the remaining small terms decide, and the heads' norm
    scales it up to full size."""
    ref = plain_logits(folder, toks)[pos]
    if dtype == "float32":
        return max(3e-4, 5.0 * float((plain_logits(folder, toks, "float32")[pos] - ref).abs().max()))
    return max(0.12, 3.0 * centred_rms(plain_logits(folder, toks, "bfloat16")[pos] - ref) / centred_rms(ref))


def check(folder, reqs, trace, got, dtype):
    """Every wanted row within ``row_limit`` of the plain logits: in float32 all rows, in bfloat16 all but 3 %;
    and no more than a tenth of the rows may owe their limit to the model's own magnification."""
    over, total, lifted, errs = 0, 0, 0, []
    for s, want in zip(trace.steps, trace.wanted):
        if not want:
            continue
        arr = torch.from_numpy(got[s["step"]].astype(np.float64)).view(len(want), -1)
        for row, (rid, pos) in enumerate(want):
            ref = plain_logits(folder, reqs[rid])[pos]
            assert torch.isfinite(arr[row]).all()
            total += 1
            limit = row_limit(folder, reqs[rid], pos, dtype)
            lifted += limit > (3e-4 if dtype == "float32" else 0.12)
            if dtype == "float32":
                diff = float((arr[row] - ref).abs().max())
                assert diff <= limit, (f"step {s['step']}: request {rid} position {pos}: |logits - plain| = {diff:.3e} > "
                                       f"{limit:.1e}; entries {[(e['id'], len(e['tokens'])) for e in s['entries']]}")
            else:
                errs.append(centred_rms(arr[row] - ref) / centred_rms(ref))
                over += errs[-1] > limit
    assert over <= 0.03 * total + 1, (f"{over} of {total} rows differ from the plain logits beyond bfloat16 rounding; "
                                      f"quantiles 50/90/99 %: {np.quantile(errs, [0.5, 0.9, 0.99])}")
    assert lifted <= 0.1 * total + 2, f"{lifted} of {total} rows are judged by the model's magnification of rounding"


def requests_for(name, lens, seed):
    rng = np.random.default_rng(seed)
    return {f"r{i}": rng.integers(0, TINY[name]["raw"]["vocab"], size=n).tolist() for i, n in enumerate(lens)}


def replay(folder, name, dtype, trace, out, **kw):
    return R.replay(folder, dtype, trace, str(out), page_size=TINY[name]["page_size"], **kw)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(TINY))
def test_whole_prompts(folders, tmp_path, name, dtype):
    reqs = requests_for(name, [1, 2, 5, 16, 17, 33, 150, 300], 1)
    tr = R.whole(reqs)
    check(folders[name], reqs, tr, replay(folders[name], name, dtype, tr, tmp_path), dtype)


def test_every_layer_run_against_the_plain_stream(folders):
    """The stream after each run of a layer (a layer whose tensors run twice counts twice), in 32 bits."""
    from rosellm_b200.config.engine import EngineConfig
    from rosellm_b200.engine.runner import ModelRunner, StepEntry

    for name in ("A", "B", "D"):
        runner = ModelRunner.from_folder(folders[name], EngineConfig(dtype="float32", page_size=TINY[name]["page_size"],
                                                                     kv_cache_tokens=256, max_num_seqs=2, cuda_graphs=False,
                                                                     capture_graphs_at_start=False, device=DEV))
        caught = []
        for layer in runner.model.layers:
            def wrapped(ctx, run, lyr, x, inner=layer.block.forward):
                inner(ctx, run, lyr, x)
                caught.append(x.detach().cpu().clone())
            layer.block.forward = wrapped
        toks = requests_for(name, [45], 11)["r0"]
        slot = runner.cache.new_request()
        runner.step([StepEntry(slot, toks, [len(toks) - 1])])
        runner.check_status()
        cfg, w = load_folder(folders[name])
        streams = []
        P.forward(cfg, w, toks, streams)
        assert len(caught) == len(streams) == len(cfg["layers"])
        for i, (mine, want) in enumerate(zip(caught, streams)):
            assert rel(mine, want) < 2e-5, (name, i)


@pytest.mark.parametrize("graphs", [False, True], ids=["walked", "graphs"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(TINY))
def test_prefill_against_token_by_token_decoding(folders, tmp_path, name, dtype, graphs):
    """The last 40 tokens one by one (with ``graphs``: as CUDA-graph replays, the way generation runs them), over
    page borders and with windows passing over decoded tokens."""
    reqs = requests_for(name, [41, 72, 104, 3], 2)
    tr = R.tail_decoded(reqs, tail=40)
    stats = {}
    got = replay(folders[name], name, dtype, tr, tmp_path, cuda_graphs=graphs, stats=stats)
    check(folders[name], reqs, tr, got, dtype)
    assert (stats["graph_replays"] > 0) == graphs


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(TINY))
def test_portions_down_to_two_tokens(folders, tmp_path, name, dtype):
    reqs = requests_for(name, [100, 37, 64, 129], 3)
    for sizes in ((7, 2, 16, 3, 2, 5, 33, 2, 1, 17), (2,), (15, 1, 16, 17)):
        tr = R.portions(reqs, sizes=sizes)
        got = replay(folders[name], name, dtype, tr, tmp_path / f"s{len(sizes)}{sizes[0]}")
        check(folders[name], reqs, tr, got, dtype)


@pytest.mark.parametrize("graphs", [False, True], ids=["walked", "graphs"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(TINY))
def test_mixed_batches_with_pages_and_slots_used_again(folders, tmp_path, name, dtype, graphs):
    """Up to four live requests, portions beside single tokens, in a pool so small that pages and state slots come
    round again; every row is compared with the request run alone (the plain implementation knows no batch): a
    state, a running maximum or a key left over by a slot's or a page's earlier owner would show."""
    lens = [120, 9, 200, 33, 70, 2, 193, 64, 20, 101]
    reqs = requests_for(name, lens, 4)
    prompt_lens = {rid: max(1, len(t) - (8 if i % 2 else 40)) for i, (rid, t) in enumerate(reqs.items())}
    tr = R.mixed(reqs, prompt_lens, max_live=4, seed=5)
    peak = R.peak_tokens(tr)
    assert sum(-(-len(t) // 64) * 64 for t in reqs.values()) > 1.5 * peak
    got = replay(folders[name], name, dtype, tr, tmp_path, max_tokens=peak, cuda_graphs=graphs)
    check(folders[name], reqs, tr, got, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_and_long_decoding(folders, tmp_path, dtype):
    reqs = requests_for("A", [1, 2, 3, 4], 9)
    for i, tr in enumerate((R.whole(reqs), R.tail_decoded(reqs, tail=10), R.portions(reqs, sizes=(2, 1)))):
        check(folders["A"], reqs, tr, replay(folders["A"], "A", dtype, tr, tmp_path / f"f{i}"), dtype)
    reqs = requests_for("B", [420], 10)
    tr = R.tail_decoded(reqs, tail=417)
    check(folders["B"], reqs, tr, replay(folders["B"], "B", dtype, tr, tmp_path / "long", cuda_graphs=True), dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_wide_model_with_long_contexts(tmp_path, dtype):
    """Width 1024: the products' tensor-core paths with float32 outputs, prompts of 600 and 350 tokens whole and in
    portions of up to 256, the last tokens one by one, windows of many key tiles, states of 64 and 128 columns."""
    from tiny_fikevik import WIDE

    folder = write_tiny("WIDE", str(tmp_path))
    rng = np.random.default_rng(3)
    reqs = {f"r{i}": rng.integers(0, WIDE["raw"]["vocab"], size=n).tolist() for i, n in enumerate([600, 350])}
    for i, tr in enumerate((R.whole(reqs), R.tail_decoded(reqs, tail=6), R.portions(reqs, sizes=(256, 3, 130, 64, 200)))):
        wanted = {rid: {len(t) - 1, len(t) - 2, len(t) // 2, 0, 1} for rid, t in reqs.items()}
        for s_, w_ in zip(tr.steps, tr.wanted):  # keep a few rows a request: the logits of 950 rows are not needed
            keep = [k for k, (rid, pos) in enumerate(w_) if pos in wanted[rid] or len(s_["entries"][0]["tokens"]) == 1]
            at = 0
            for e in s_["entries"]:
                n = len(e["want"])
                e["want"] = [e["want"][k - at] for k in keep if at <= k < at + n]
                at += n
            w_[:] = [w_[k] for k in keep]
        got = R.replay(folder, dtype, tr, str(tmp_path / f"w{i}"), page_size=16)
        check(folder, reqs, tr, got, dtype)


def test_trace_program_as_a_child_process(folders, tmp_path):
    reqs = requests_for("A", [40, 90, 3], 6)
    tr = R.mixed(reqs, {rid: len(t) - 5 for rid, t in reqs.items()}, max_live=2, seed=1)
    got = R.replay(folders["A"], "float32", tr, str(tmp_path), subprocess_mode=True, page_size=16)
    check(folders["A"], reqs, tr, got, "float32")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(TINY))
def test_greedy_generation_through_the_entry_point(folders, name, dtype):
    """Prompts of unequal length through ``InferenceEngine.generate_batch`` (scheduler, portions of 16 tokens,
    decode graphs, tokens chosen on the device and fed back without the host reading them): every generated
    token is the plain arg-max given the tokens before it, or within the precision's reach."""
    from rosellm_b200.engine.llm import InferenceEngine

    rng = np.random.default_rng(7)
    vocab = TINY[name]["raw"]["vocab"]
    prompts = [rng.integers(0, vocab, n).tolist() for n in (5, 37, 1, 64)]
    eng = InferenceEngine(folders[name], dtype=dtype, page_size=TINY[name]["page_size"], max_batch_size=4,
                          kv_cache_max_tokens=512, prefill_chunk_size=16, max_position_embeddings=256)
    outs = eng.generate_batch(prompts, max_new_tokens=12, stop_on_eos=False)
    assert [len(o) for o in outs] == [12] * 4
    for prompt, out in zip(prompts, outs):
        ids = list(prompt)
        for tok in out:
            ref = plain_logits(folders[name], ids)[-1]
            gap = float(ref.max() - ref[tok])
            limit = row_limit(folders[name], ids, len(ids) - 1, dtype)  # on a logit, or on the row's relative error
            assert gap <= (2 * limit if dtype == "float32" else 1.4 * limit * centred_rms(ref)), (gap, limit)
            ids.append(tok)


@pytest.mark.parametrize("stream", [False, True], ids=["whole", "stream"])
def test_the_command_line_generates_the_plain_greedy_tokens(folders, stream):
    """``python -m rosellm_b200.cli_generate`` as a child process, in 32 bits, on a model whose layers run other
    layers' tensors: the ids it prints are the plain arg-max, token after token."""
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    prompt = np.random.default_rng(12).integers(0, TINY["B"]["raw"]["vocab"], 23).tolist()
    env = dict(os.environ, PYTHONPATH=root + os.pathsep + os.environ.get("PYTHONPATH", ""))
    res = subprocess.run([sys.executable, "-m", "rosellm_b200.cli_generate", "--model", folders["B"], "--prompt-ids",
                          ",".join(map(str, prompt)), "--max-new-tokens", "6", "--no-stop-on-eos", "--dtype", "fp32",
                          "--max-num-batched-tokens", "64", "--max-num-seqs", "2", "--page-size", str(TINY["B"]["page_size"]),
                          "--kv-cache-max-tokens", "256", *(["--stream"] if stream else [])],
                         capture_output=True, text=True, timeout=600, env=env, cwd=root)
    assert res.returncode == 0, res.stderr[-3000:]
    if stream:
        line = next(l for l in res.stdout.splitlines() if l.startswith("[rosellm_b200] streaming output: "))
        got = [int(t) for t in line.split(": ", 1)[1].split()]
    else:
        import ast

        line = next(l for l in res.stdout.splitlines() if l.startswith("[rosellm_b200] output: "))
        got = list(ast.literal_eval(line.split(": ", 1)[1]))
    assert len(got) == 6
    ids = list(prompt)
    for tok in got:
        ref = plain_logits(folders["B"], ids)[-1]
        assert float(ref.max() - ref[tok]) <= 2 * row_limit(folders["B"], ids, len(ids) - 1, "float32")
        ids.append(tok)
