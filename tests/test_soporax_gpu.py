"""Soporax on the GPU: every mechanism's kernels against the plain implementation's function for it, then whole
models through the engine's step function, cache, scheduler and entry point."""
import math
import os
import types

import numpy as np
import pytest
import torch

import plain_soporax as P
import replay_util as R
from tiny_soporax import TINY, WIDE, load_folder, write_tiny

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

@pytest.mark.parametrize("width", [8, 100, 1000, 12000])
def test_what_is_added_to_the_stream_ahead_of_a_pass(width):
    """The row of the pass, the kept token rows, both or neither; keeping the rows as they were; rows of a wider
    matrix."""
    g = torch.Generator().manual_seed(width)
    n = 7
    x, again = torch.randn(n, width + 8, generator=g), torch.randn(n, width, generator=g)
    vec = torch.randn(width, generator=g)
    for use_vec, use_again, use_keep in ((1, 0, 1), (1, 1, 0), (0, 0, 1), (0, 1, 0), (1, 1, 1)):
        buf = x.to(DEV).clone()
        keep = torch.full((n, width), 9.0, device=DEV) if use_keep else None
        K().stream_inject(buf[:, :width], vec=vec.to(DEV) if use_vec else None, again=again.to(DEV) if use_again else None,
                          keep=keep)
        want = x[:, :width].double() + (vec.double() if use_vec else 0.0) + (again.double() if use_again else 0.0)
        assert rel(buf[:, :width], want) < 1e-7 and torch.equal(buf[:, width:].cpu(), x[:, width:])
        if use_keep:
            assert torch.equal(keep.cpu(), x[:, :width])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_output_gate_on_merged_heads(dtype):
    g = torch.Generator().manual_seed(2)
    for n, width in ((5, 30), (33, 512), (1, 7)):
        o = torch.randn(n, width + 2, generator=g).to(DTYPES[dtype])
        z = torch.randn(n, width + 5, generator=g) * 4.0
        buf = o.to(DEV).clone()
        K().gate_mul(buf[:, :width], z.to(DEV)[:, 3:3 + width])
        want = o[:, :width].double() * torch.sigmoid(z[:, 3:3 + width].double())
        assert rel(buf[:, :width].float(), want) < (1e-6 if dtype == "float32" else 5e-3)
        assert torch.equal(buf[:, width:].cpu(), o[:, width:])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("experts,top,n", [(5, 2, 150), (1, 1, 9), (9, 1, 3), (3, 3, 70), (16, 4, 1), (8, 2, 600), (6, 3, 2800)])
def test_experts_named_by_a_table_of_token_ids(dtype, experts, top, n):
    """The part itself on a step's tokens: few tokens (every expert's weights streamed once) and many (tiles), also
    more pairs than the one-launch routing takes (three launches then); all experts a token, one, and a single
    expert; token ids the engine feeds back from the device; a second run of the part in the same step, which
    finds the step's routing again."""
    from rosellm_b200.engine.context import Workspace
    from rosellm_b200.parts.gated import MixtureOfExperts

    g = torch.Generator().manual_seed(experts * 7 + top)
    dt, hid, ff, vocab = DTYPES[dtype], 48, 20, 37
    part = MixtureOfExperts(hidden_size=hid, inner_size=ff, num_experts=experts, top=top, gate="silu", routing="table",
                            vocab_size=vocab)
    table = torch.rand(vocab, experts, generator=g).argsort(dim=1)[:, :top].to(torch.int32)
    gu = (torch.randn(experts * 2 * ff, hid, generator=g) * 0.3).to(torch.bfloat16)
    down = (torch.randn(experts * hid, ff, generator=g) * 0.3).to(torch.bfloat16)
    part.bind({"table": table.to(DEV), "gate_up_weight": gu.to(dt).to(DEV), "down_weight": down.to(dt).to(DEV)})
    toks = torch.randint(0, vocab, (n,), generator=g).to(torch.int32)
    h = torch.randn(n, hid, generator=g).to(dt)
    w = {"m.table": table}
    for e in range(experts):
        w[f"m.e{e}.gate"], w[f"m.e{e}.up"] = gu[e * 2 * ff:e * 2 * ff + ff].double(), gu[e * 2 * ff + ff:(e + 1) * 2 * ff].double()
        w[f"m.e{e}.down"] = down[e * hid:(e + 1) * hid].double()
    want = P.table_experts(h.double(), toks.tolist(), w, "m.", top)
    for feedback in (False, True):
        ids = toks.clone()
        extras = {}
        if feedback:  # ids below zero name rows of the buffer the sampler wrote
            ids = -(torch.arange(n, dtype=torch.int32) + 1)
            extras["token_feedback"] = toks.to(DEV)
        ctx = types.SimpleNamespace(n_tokens=n, token_ids=ids.to(DEV), act_dtype=dt, extras=extras,
                                    workspace=Workspace(torch.device(DEV)))
        x0 = torch.randn(n, hid, generator=g)
        x = x0.to(DEV).clone()
        part.forward(ctx, h.to(DEV), x, add=True)
        K().check_status(torch.device(DEV))
        assert rel(x.cpu().double() - x0.double(), want) < (2e-5 if dtype == "float32" else 1.5e-2)
        before = K().launches()
        x2 = torch.zeros(n, hid, device=DEV)
        part.forward(ctx, h.to(DEV), x2, add=False)  # the same step again: no routing launches, the same result
        assert K().launches() - before == 3 and rel(x2, want) < (2e-5 if dtype == "float32" else 1.5e-2)


@pytest.mark.parametrize("H,G,dk,dv,rot", [(6, 2, 20, 12, 12), (4, 4, 64, 32, 0), (7, 1, 9, 5, 8), (2, 1, 136, 130, 136)])
def test_unit_queries_and_keys_and_stretched_rotations(H, G, dk, dv, rot):
    """Queries and keys divided by their root mean square without a weight; rotation with frequencies of both
    scalings, at positions below and far beyond the scaling's original length; values untouched."""
    g = torch.Generator().manual_seed(H * dk)
    n = 12
    pos = torch.tensor([0, 1, 2, 3, 15, 16, 17, 100, 1000, 4097, 7, 8], dtype=torch.int32)
    q, k, v = (torch.randn(n, w, generator=g) for w in (H * dk, G * dk, G * dv))
    eps = 1e-5
    scalings = [None]
    if rot:
        scalings += [dict(kind="wavelength", factor=4.0, low=1.0, high=4.0, original=16),
                     dict(kind="ramp", factor=8.0, original=32, fast=16.0, slow=2.0)]
    from rosellm_b200.parts.standard import RotaryPositions

    for sc in scalings:
        for unit in (True, False):
            bq, bk, bv = q.to(DEV).clone(), k.to(DEV).clone(), v.to(DEV).clone()
            rp = RotaryPositions(dims=rot, base=700.0, scaling=sc) if rot else None
            K().qkv_norm_rotate(bq, bk, bv, pos.to(DEV), n_heads=H, n_kv=G, dk=dk, dv=dv, eps=eps,
                                freq=rp.frequencies(DEV) if rot else None, rot_dims=rot, unit_qk=unit)
            pq, pk = q.double().view(n, H, dk), k.double().view(n, G, dk)
            if unit:
                pq, pk = P.unit(pq, eps), P.unit(pk, eps)
            if rot:
                rd = {"dims": rot, "base": 700.0}
                if sc is not None:
                    rd["scaling"] = {a: b for a, b in sc.items() if a != "kind"}
                freqs, mult = P.rotation_constants(rd)
                assert mult == pytest.approx(rp.mult)
                pq, pk = P.rotate_pairs(pq, pos, freqs), P.rotate_pairs(pk, pos, freqs)
            near = pos < 200
            assert rel(bq.view(n, H, dk)[near], pq[near]) < 2e-5 and rel(bk.view(n, G, dk)[near], pk[near]) < 2e-5
            assert rel(bq.view(n, H, dk), pq) < 2e-3 and torch.equal(bv.cpu(), v)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,dk,dv,rot,unit_v", [(6, 2, 20, 12, 12, False), (4, 4, 64, 32, 0, True), (7, 1, 9, 5, 8, False),
                                                  (2, 1, 136, 130, 136, True)])
def test_keys_and_values_into_their_pages_by_the_pass_that_normalises_them(dtype, H, G, dk, dv, rot, unit_v):
    """The pass with a cache target against the pass in place followed by the store kernel: the same pages bit for
    bit, the same queries; requests that start inside a page and cross page borders; a padding row (slot -1) writes
    nothing."""
    from rosellm_b200.engine.context import build_host_batch
    from rosellm_b200.parts.standard import RotaryPositions

    dt = DTYPES[dtype]
    g = torch.Generator().manual_seed(H + dk)
    page, v_at = 8, -(-dk // 8) * 8
    row = -(-(v_at + dv) // 8) * 8
    hb = build_host_batch([(1, 5, [0] * 20, []), (2, 0, [0] * 3, []), (3, 31, [0], []), (-1, 0, [0], [])])
    n = len(hb.positions)
    table = torch.full((4, 8), -1, dtype=torch.int32)
    table[1:, :] = torch.randperm(24, generator=g).view(3, 8).to(torch.int32)
    q, k, v = (torch.randn(n, w, generator=g) for w in (H * dk, G * dk, G * dv))
    freq = RotaryPositions(dims=rot, base=300.0).frequencies(DEV) if rot else None
    pools, queries = [], []
    for fused in (False, True):
        pool = torch.full((24, 1, G, page, row), 7.0, dtype=dt, device=DEV)
        bq, bk, bv = q.to(DEV).clone(), k.to(DEV).clone(), v.to(DEV).clone()
        cache = K().QkvCache(pool, table.to(DEV), dev(hb.req_of_token), dev(hb.slots), v_at, 64) if fused else None
        K().qkv_norm_rotate(bq, bk, bv, dev(hb.positions), n_heads=H, n_kv=G, dk=dk, dv=dv, eps=1e-5, freq=freq, rot_dims=rot,
                            unit_values=unit_v, unit_qk=True, cache=cache)
        if fused:
            assert torch.equal(bk.cpu(), k) and torch.equal(bv.cpu(), v)  # not written back
        else:
            K().bias_kv_store(bk, bv, pool, table.to(DEV), dev(hb.positions), dev(hb.req_of_token), dev(hb.slots), v_at=v_at,
                              max_pos=64)
        K().check_status(torch.device(DEV))
        pools.append(pool.float().cpu())
        queries.append(bq.cpu())
    assert torch.equal(pools[0], pools[1]) and torch.equal(queries[0], queries[1])
    assert (pools[1] != 7.0).sum() == (n - 1) * G * (dk + dv)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_latent_rows_and_queries_with_scaled_cosines(dtype):
    """The cache rows and the queries' turned parts with a factor on cosines and sines, frequencies of the ramp."""
    from rosellm_b200.parts.standard import RotaryPositions

    dt = DTYPES[dtype]
    g = torch.Generator().manual_seed(5)
    n, rank, rot_dim, H, plain, page = 9, 18, 6, 3, 12, 16
    rows_w = -(-(rank + rot_dim) // 8) * 8
    sc = dict(kind="ramp", factor=8.0, original=32, fast=16.0, slow=2.0)
    rp = RotaryPositions(dims=rot_dim, base=10000.0, scaling=sc)
    freqs, mult = P.rotation_constants({"dims": rot_dim, "base": 10000.0, "scaling": {a: b for a, b in sc.items() if a != "kind"}})
    assert mult == pytest.approx(rp.mult) and mult > 1.1
    pos = torch.tensor([0, 1, 5, 31, 32, 33, 100, 640, 64], dtype=torch.int32)
    dkv = torch.randn(n, rank + rot_dim + 3, generator=g)
    gamma = 1 + 0.2 * torch.randn(rank, generator=g)
    pool = torch.zeros(60, 1, 1, page, rows_w, dtype=dt, device=DEV)
    table = torch.arange(1, 60, dtype=torch.int32).view(1, -1)
    table = torch.cat([torch.full_like(table, -1), table]).to(DEV)
    zeros = torch.zeros(n, dtype=torch.int32, device=DEV)
    K().latent_kv_write(dkv.to(DEV)[:, :rank + rot_dim], gamma.to(DEV), 1e-5, rp.frequencies(DEV), rot_dim, pool, table,
                        pos.to(DEV), zeros, torch.ones(1, dtype=torch.int32, device=DEV), rank=rank, rot_dim=rot_dim,
                        max_pos=1024, rot_mult=rp.mult)
    K().check_status(torch.device(DEV))
    c = P.unit(dkv[:, :rank].double(), 1e-5) * gamma.double()
    kr = P.rotate_pairs(dkv[:, rank:rank + rot_dim].double(), pos, freqs, mult)
    tol = 2e-5 if dtype == "float32" else 6e-3
    for i, p_ in enumerate(pos.tolist()):
        row = pool[1 + p_ // page, 0, 0, p_ % page].float().cpu()
        assert rel(row[:rank], c[i]) < tol and rel(row[rank:rank + rot_dim], kr[i]) < tol
        assert not row[rank + rot_dim:].any()
    q = torch.randn(n, H * (plain + rot_dim), generator=g).to(dt)
    rows = torch.full((n, H * rows_w), 3.0, dtype=dt, device=DEV)
    K().latent_q_rope(q.to(DEV), rows, rp.frequencies(DEV), pos.to(DEV), n_heads=H, head_in=plain + rot_dim, plain=plain,
                      rank=rank, rot_dim=rot_dim, rot_dims=rot_dim, row_width=rows_w, rot_mult=rp.mult)
    want = P.rotate_pairs(q.double().view(n, H, plain + rot_dim)[..., plain:], pos, freqs, mult)
    assert rel(rows.view(n, H, rows_w)[..., rank:rank + rot_dim].float(), want) < tol


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key", [0, 15, 16, 512, 897])
def test_latent_attention_with_a_plain_softmax_finds_a_far_key(dtype, key):
    """The latent mixer of this design has no sink: among 900 cached rows one is scored far above the rest, as the
    first key, at a page's border and far back, from a prompt portion's query and from a decoded token's (keys cut
    into parts); the case builder is the one of the latent kernels' own tests."""
    from test_lebedra_gpu import _attention_case as latent_case

    for new, old, by_request, splits in (([4], [896], False, 1), ([1], [899], True, 4), ([1], [899], True, 1)):
        got, want = latent_case(dtype, 2, 24, 8, new, old, 16, None, 1.0, by_request, splits, seed=key,
                                stand_out=(new[0] - 1, key))
        assert rel(got, want) < (2e-5 if dtype == "float32" else 2e-2)
        assert (want[-1, 0].abs() > 0.05).any()


def _attn_case(dtype, H, G, dk, dv, lens_new, lens_old, page, scale, window, seed, stand_out=None, splits=1, mma=False,
               sink="random", gate=None):
    """Requests with ``lens_old`` cached tokens bring ``lens_new`` more.  All tokens' cache rows are written by the
    store kernel; then the pages that the window has passed before this step are taken away (their table
    entries -1, their rows overwritten with huge numbers), as the cache manager does.  ``sink``: ``None``, a
    number for all heads, or ``"random"``; ``gate``: ``None``, ``"head"`` or ``"element"``.  Returns the kernel's
    output [tokens, H, dv], the plain result from the same (rounded) keys and values, and the values."""
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
    if sink == "random":
        sinks = torch.randn(H, generator=g) * 2.0
    else:
        sinks = None if sink is None else torch.full((H,), float(sink))
    gates = None
    if gate is not None:
        gates = torch.randn(n_tok, H if gate == "head" else H * dv, generator=g) * 3.0
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
    K().bias_attention(q.reshape(n_tok, H * dk).to(DEV), None if gates is None else gates.to(DEV), pool, table, dev(hb.q_start),
                       dev(hb.kv_len), dev(hb.slots), out, n_heads=H, dk=dk, dv=dv, v_at=v_at, scale=scale,
                       tiles=dev(tiles.reshape(-1)), n_tiles=n_tiles, tile_tokens=64 if wide else 16,
                       decode_reqs=dev(hb.decode_reqs), n_decode=len(hb.decode_reqs), max_pos=max(totals), n_splits=splits,
                       part_o=part_o, part_ml=part_ml, tensor_cores=mma, window=window or 0,
                       sink=None if sinks is None else sinks.to(DEV), gate_per_head=gate == "head")
    K().check_status(torch.device(DEV))
    want = torch.empty(n_tok, H, dv, dtype=torch.float64)
    t0 = 0
    for r in range(n_req):
        kc, vc = ks[r].to(dt).double(), vs[r].to(dt).double()  # what the cache holds
        qq = torch.zeros(totals[r], H, dk, dtype=torch.float64)
        qq[lens_old[r]:] = q[t0:t0 + lens_new[r]].double()
        want[t0:t0 + lens_new[r]] = P.softmax_attention(qq, kc, vc, scale, window, None if sinks is None else sinks.double())[lens_old[r]:]
        t0 += lens_new[r]
    if gate == "head":
        want = want * torch.sigmoid(gates.double())[:, :, None]
    elif gate == "element":
        want = want * torch.sigmoid(gates.double()).view(n_tok, H, dv)
    return out.float().cpu().view(n_tok, H, dv), want, vs


def _tol(dtype, mma=False):
    # with bfloat16 operands on the tensor cores the queries and the probabilities are rounded too
    return 2e-5 if dtype == "float32" else (2.5e-2 if mma else 1e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window", [1, 7, 16, 17, 100, None])
@pytest.mark.parametrize("gate", [None, "head", "element"])
def test_attention_with_a_sink_and_gates(dtype, window, gate):
    """Learned sinks on both sides of zero with windows of one key, within a page, of a page and one more, of
    several key tiles and none; a gate per head, per element, or none; portions that start inside a page and end
    on a border beside single tokens; one to forty heads a key/value head; CUDA cores and tensor cores."""
    for mma in ((False,) if dtype == "float32" else (False, True)):
        for H, G, dk, dv, page in ((6, 2, 20, 12, 16), (40, 1, 8, 8, 32), (2, 1, 136, 130, 16), (16, 4, 128, 128, 16)):
            got, want, _ = _attn_case(dtype, H, G, dk, dv, [40, 1, 2, 17, 1, 16], [5, 130, 0, 15, 0, 16], page, 0.3, window,
                                      seed=H, mma=mma, gate=gate)
            assert rel(got, want) < _tol(dtype, mma), (H, G, dk, dv, mma)
            got, want, _ = _attn_case(dtype, H, G, dk, dv, [1, 1, 1, 1], [0, 31, 32, 300], page, 0.2, window, seed=H + 50,
                                      mma=mma, gate=gate)
            assert rel(got, want) < _tol(dtype, mma), (H, G, dk, dv, mma, "single tokens")


@pytest.mark.parametrize("window", [None, 1, 100])
def test_both_forms_of_the_tensor_core_prompt_tiles(window):
    """Key and value tiles by cp.async through two stages (portions of one to many tiles, contexts that begin
    inside a tile, tiles that are partly or wholly outside the window) against the form that copies them through
    registers, and both against the plain result."""
    for H, G, dk, dv, page in ((8, 2, 64, 64, 16), (4, 1, 48, 24, 8), (16, 4, 128, 128, 16), (3, 3, 16, 120, 32)):
        got = {}
        for on in (True, False):
            K().bias_attention_async(on)
            try:
                got[on], want, _ = _attn_case("bfloat16", H, G, dk, dv, [200, 1, 2, 65, 64, 700], [5, 130, 0, 63, 64, 330], page, 0.3,
                                              window, seed=H, mma=True, gate="head")
            finally:
                K().bias_attention_async(True)
            assert rel(got[on], want) < _tol("bfloat16", True), (H, G, dk, dv, on)
        assert rel(got[True], got[False]) < 1e-2


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("sink", [None, 0.0, -30.0, 4.0, 25.0])
def test_sinks_of_every_size(dtype, sink):
    """No sink, a sink of score zero (one more unit in the denominator), one too small to count, and sinks that
    take most or nearly all of the weight; for prompt portions, single tokens, and keys cut into parts."""
    for splits, mma in ((1, False), (1, True), (4, False)):
        got, want, _ = _attn_case(dtype, 6, 3, 24, 16, [1, 20, 1, 3], [200, 9, 0, 64], 16, 0.25, None, seed=3, sink=sink,
                                  splits=splits, mma=mma, gate="head")
        tol = _tol(dtype, mma) * (1.0 if sink is None or sink < 10 else 3.0)  # nearly nothing is left of the output
        assert rel(got, want) < tol, (splits, mma)
    if sink == 0.0:  # a first token sees itself and the sink alike: half its value
        got, _, vs = _attn_case(dtype, 2, 1, 16, 8, [1], [0], 16, 0.0, None, seed=1, sink=0.0)
        assert rel(got[0, 0], vs[0][0, 0].to(DTYPES[dtype]).double() / 2) < _tol(dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("splits", [2, 3, 8, 32])
@pytest.mark.parametrize("window", [40, None])
def test_decoded_tokens_with_keys_cut_into_parts_and_a_sink(dtype, splits, window):
    """The sink counts once, whatever the number of parts (more parts than tiles of keys too), beside a prompt
    portion that is not cut."""
    got, want, _ = _attn_case(dtype, 6, 2, 20, 10, [1, 1, 5, 1, 1], [700, 0, 40, 63, 64], 16, 0.25, window, seed=splits,
                              splits=splits, gate="element")
    assert rel(got, want) < _tol(dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window", [1, 5, 16, 33, 96, None])
def test_a_key_that_stands_out_just_inside_the_window_just_outside_and_far_back(dtype, window):
    """One key is scored far above the rest and the sink.  As the earliest key the window keeps (with no window:
    as the sequence's first key, hundreds back, and at a page's border), the output is (nearly) its value; one
    position earlier it must leave no trace.  From a prompt portion's last query (CUDA cores and tensor cores) and
    from a decoded token's (whole and cut into parts)."""
    H, G, dk, dv, head = 4, 2, 24, 12, 3
    for total in (window + 3 if window else 40, 333, 900):
        last = total - 1
        for new, splits, mma in ((4, 1, False), (4, 1, True), (1, 1, False), (1, 5, False), (min(total, 70), 1, False)):
            old = total - new
            cases = ((last - window + 1, True), (last - window, False)) if window else ((0, True), (last - (last % 16) - 1, True))
            for key, inside in cases:
                if key < 0:
                    continue
                got, want, vs = _attn_case(dtype, H, G, dk, dv, [new], [old], 16, 0.5, window, seed=key, stand_out=(key, head),
                                           splits=splits, mma=mma, sink=1.0)
                rows = slice(-1, None) if mma and dtype == "bfloat16" else slice(None)
                assert rel(got[rows], want[rows]) < _tol(dtype, mma), (total, new, splits, mma, key, inside)
                value = vs[0][key, head // (H // G)].to(DTYPES[dtype]).double()
                hit = float((got[-1, head].double() - value).abs().max())
                if inside:
                    assert hit < 1e-2, (total, new, splits, mma, "a key the query sees was not seen")
                elif window > 1:
                    assert hit > 0.3, (total, new, splits, mma, "a key before the window was seen")


# ---- whole models through the step function ------------------------------------------------------------

@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = str(tmp_path_factory.mktemp("soporax"))
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
            _plain[folder] = (cfg, w, {k: (v.float() if v.is_floating_point() else v) for k, v in w.items()})
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
    """float32: 3e-4 on a logit (times the logits' multiplier where that exceeds one), or five times what float32
    rounding moves this row in the plain implementation.  bfloat16: the row's error (mean taken off, root mean
    square over the vocabulary, over that of the plain row) 0.08, or three times what bfloat16 storage moves it."""
    ref = plain_logits(folder, toks)[pos]
    if dtype == "float32":
        floor = 3e-4 * max(1.0, float(ref.abs().max()) / 10.0)
        return max(floor, 5.0 * float((plain_logits(folder, toks, "float32")[pos] - ref).abs().max()))
    return max(0.08, 3.0 * centred_rms(plain_logits(folder, toks, "bfloat16")[pos] - ref) / centred_rms(ref))


def check(folder, reqs, trace, got, dtype):
    """Every wanted row within ``row_limit`` of the plain logits: in float32 all rows, in bfloat16 all but 2 %."""
    over, total, errs = 0, 0, []
    for s, want in zip(trace.steps, trace.wanted):
        if not want:
            continue
        arr = torch.from_numpy(got[s["step"]].astype(np.float64)).view(len(want), -1)
        for row, (rid, pos) in enumerate(want):
            ref = plain_logits(folder, reqs[rid])[pos]
            assert torch.isfinite(arr[row]).all()
            total += 1
            limit = row_limit(folder, reqs[rid], pos, dtype)
            if dtype == "float32":
                diff = float((arr[row] - ref).abs().max())
                assert diff <= limit, (f"step {s['step']}: request {rid} position {pos}: |logits - plain| = {diff:.3e} > "
                                       f"{limit:.1e}; entries {[(e['id'], len(e['tokens'])) for e in s['entries']]}")
            else:
                errs.append(centred_rms(arr[row] - ref) / centred_rms(ref))
                over += errs[-1] > limit
    assert over <= 0.02 * total + 1, (f"{over} of {total} rows differ from the plain logits beyond bfloat16 rounding; "
                                      f"quantiles 50/90/99 %: {np.quantile(errs, [0.5, 0.9, 0.99])}")


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
    """The stream after each run of a layer (a layer of the repeated stretch counts every pass), in 32 bits."""
    from rosellm_b200.config.engine import EngineConfig
    from rosellm_b200.engine.runner import ModelRunner, StepEntry

    for name in ("A", "C", "D", "F"):
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
        P.forward(cfg, w, toks, streams=streams)
        assert len(caught) == len(streams) == len(P.run_order(cfg)) > len(cfg["layers"])
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
    """Up to four live requests, portions beside single tokens, in a pool so small that pages and slots come
    round again; every row is compared with the request run alone (the plain implementation knows no batch): a
    key left over by a page's earlier owner, or a page the window gave back too early, would show."""
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
    portions of up to 256, the last tokens one by one, a window of many key tiles, a latent of 256."""
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
    decode graphs, tokens chosen on the device and fed back without the host reading them, which the experts'
    table has to follow): every generated token is the plain arg-max given the tokens before it, or within the
    precision's reach."""
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


def test_the_command_line_generates_the_plain_greedy_tokens(folders):
    """``python -m rosellm_b200.cli_generate`` as a child process, in 32 bits, on a model with a repeated stretch:
    the ids it prints are the plain arg-max, token after token."""
    import ast
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    prompt = np.random.default_rng(12).integers(0, TINY["A"]["raw"]["vocab"], 23).tolist()
    env = dict(os.environ, PYTHONPATH=root + os.pathsep + os.environ.get("PYTHONPATH", ""))
    res = subprocess.run([sys.executable, "-m", "rosellm_b200.cli_generate", "--model", folders["A"], "--prompt-ids",
                          ",".join(map(str, prompt)), "--max-new-tokens", "6", "--no-stop-on-eos", "--dtype", "fp32",
                          "--max-num-batched-tokens", "64", "--max-num-seqs", "2", "--page-size", str(TINY["A"]["page_size"]),
                          "--kv-cache-max-tokens", "256"],
                         capture_output=True, text=True, timeout=600, env=env, cwd=root)
    assert res.returncode == 0, res.stderr[-3000:]
    line = next(l for l in res.stdout.splitlines() if l.startswith("[rosellm_b200] output: "))
    got = list(ast.literal_eval(line.split(": ", 1)[1]))
    assert len(got) == 6
    ids = list(prompt)
    for tok in got:
        ref = plain_logits(folders["A"], ids)[-1]
        assert float(ref.max() - ref[tok]) <= 2 * row_limit(folders["A"], ids, len(ids) - 1, "float32")
        ids.append(tok)
