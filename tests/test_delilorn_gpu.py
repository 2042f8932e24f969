"""Delilorn on the device against the plain implementation (tests/plain_delilorn.py): each
mechanism alone through its kernel, then whole models through the step function: whole prompts,
prompts against token-by-token decoding, portions down to two tokens, mixed batches with pages and
state slots that are used again, keys at the edges of the window and of the kept first tokens, far
keys, sinks and long memories that the weights are made to show, long decoding, and greedy
generation through the entry point."""
import json
import math
import os
from types import SimpleNamespace

import numpy as np
import pytest
import torch
from safetensors.torch import load_file, save_file

import plain_delilorn as plain
from delilorn_configs import DELILORN_TINY, decisive_routers, make_delilorn_dir, random_delilorn_config_dict
from helpers import (collect_logits, lines_of, max_live_tokens, random_ids, schedule_mixed, schedule_portions,
                     schedule_tail_decode, schedule_whole)

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
# Largest |logit difference|, and largest root-mean-square difference over the vocabulary at one
# position, over the largest plain |logit|.  float32: 32-bit sums against float64, the sharp test of
# every schedule.  bfloat16: products and activations rounded to 8 bits through tiny random layers
# whose norms (four per block) carry a rounding of a small sub-layer output into the stream at full
# size; it catches a kernel that is wrong, not one that rounds elsewhere.
TOLERANCE = {"float32": 5e-5, "bfloat16": 2e-1}
RMS_TOLERANCE = {"float32": 1.7e-5, "bfloat16": 6e-2}
MEASURED = {}


def draws(*shape, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).bfloat16().double()


def on_device(x, dtype):
    return x.to(dtype).to(DEV).contiguous()


class Tables:
    def __init__(self, rot, n):
        from tinyserve_b200.parts.rotary import Rotary
        part = Rotary(rot["dims"], rot["base"], "half", rot.get("scaling"))
        self.rotary_dim, self.interleaved = rot["dims"], False
        cos, sin = Rotary.tables(part.rotary_dim, part.theta, n, part.scaling)
        self.cos, self.sin = cos.to(DEV), sin.to(DEV)


# ----------------------------------------------------------------------------- mechanisms alone
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-6), (torch.bfloat16, 1e-2)])
@pytest.mark.parametrize("n", [40, 200, 1000])
def test_norm_of_the_output_add_and_next_norm_in_one_kernel(dtype, tol, n):
    from tinyserve_b200.kernels import ops
    T = 23
    r, y = draws(T, n, seed=1, scale=3.0), draws(T, n, seed=2, scale=0.05)
    wa, wb = draws(n, seed=3, scale=0.1), draws(n, seed=4, scale=0.1)
    residual = on_device(r, torch.float32)
    addend = ops.NormedAddend(on_device(y, dtype), on_device(1 + wa, torch.float32), 1e-5)
    out = ops.normed_add_rmsnorm(addend, residual, on_device(1 + wb, torch.float32), 1e-6, dtype)
    stream = r + plain.norm_around_zero(y, wa, 1e-5)
    want = plain.norm_around_zero(stream, wb, 1e-6)
    assert (out.double().cpu() - want).abs().max() <= tol * want.abs().max()
    assert (residual.double().cpu() - stream).abs().max() <= (1e-6 if dtype == torch.float32 else 1e-2) * stream.abs().max()
    assert (addend.materialize().double().cpu() - plain.norm_around_zero(y, wa, 1e-5)).abs().max() <= tol * 2
    rows = torch.tensor([5, 0, 22], dtype=torch.int32, device=DEV)
    before = residual.clone()
    some = ops.normed_add_rmsnorm(addend, residual, on_device(1 + wb, torch.float32), 1e-6, dtype, rows=rows)
    assert torch.equal(before, residual), "with rows the residual is left as it is"
    want = plain.norm_around_zero(before.double().cpu() + plain.norm_around_zero(y, wa, 1e-5), wb, 1e-6)[[5, 0, 22]]
    assert (some.double().cpu() - want).abs().max() <= tol * want.abs().max()


def test_offset_norm_weight_is_summed_in_32_bit():
    from tinyserve_b200.parts.norm import RMSNorm
    norm = RMSNorm(8, 1e-6, offset=1.0)
    w = torch.tensor([0.00390625 * 0.75] * 8).bfloat16()        # 1 + w is no bfloat16 number
    norm.bind({"weight": w})
    weight, eps = norm.rms_parameters()
    assert weight.dtype == torch.float32 and torch.equal(weight, 1.0 + w.float()) and eps == 1e-6


def _paged(rows, page, num_pages, seed):
    """Per-request rows [n, heads, width] scattered into shuffled pages; unused slots hold large
    values, so that reading them shows."""
    heads, width = rows[0].shape[1:]
    g = torch.Generator().manual_seed(seed)
    order = (torch.randperm(num_pages - 1, generator=g) + 1).tolist()
    cache = torch.full((num_pages, heads, page, width), 40.0, dtype=rows[0].dtype)
    table = torch.zeros(len(rows), max(-(-x.shape[0] // page) for x in rows) + 2, dtype=torch.int32)
    for b, x in enumerate(rows):
        for i in range(-(-x.shape[0] // page)):
            pg = order.pop()
            table[b, i] = pg
            n = min(page, x.shape[0] - i * page)
            cache[pg, :, :n] = x[i * page:i * page + n].transpose(0, 1)
    return cache.to(DEV), table.to(DEV)


def _attention_plain(q, k, v, q_lens, scale, mask, sinks):
    """Request b's last q_lens[b] positions attend to its keys; float64."""
    out, at = [], 0
    for kb, vb, n in zip(k, v, q_lens):
        kv, H, G = kb.shape[0], q.shape[1], kb.shape[1]
        o = torch.zeros(n, H, vb.shape[2], dtype=torch.float64)
        for i in range(n):
            pos = kv - n + i
            js = [j for j in range(kv) if plain.visible(pos, j, mask)]
            for a in range(H):
                g = a // (H // G)
                s = (kb[js, g].double() @ q[at + i, a].double()) * scale
                sink = sinks[a].double() if sinks is not None else torch.tensor(-math.inf, dtype=torch.float64)
                top = torch.maximum(s.max(), sink)
                e = torch.exp(s - top)
                o[i, a] = (e @ vb[js, g].double()) / (e.sum() + torch.exp(sink - top))
        out.append(o)
        at += n
    return torch.cat(out)


def _run_attention(q, kc, vc, table, q_lens, kv_lens, page, scale, mask, sinks, splits=None, backend=None):
    from tinyserve_b200.kernels import ops
    cu = torch.tensor([0] + list(np.cumsum(q_lens)), dtype=torch.int32, device=DEV)
    ctx = SimpleNamespace(cu_q=cu, kv_lens=torch.tensor(kv_lens, dtype=torch.int32, device=DEV), num_requests=len(q_lens),
                          max_q_len=max(q_lens), max_kv_len=max(kv_lens), host={}, tile_cache={})
    view = SimpleNamespace(block_table=table, page_size=page)
    mask = mask or {}
    return ops.paged_attention(q, kc, vc, view, ctx, scale, mask.get("size", 0), num_splits=splits, backend=backend,
                               keep_first=mask.get("keep_first", 0), sinks=sinks)


def attention_backends(dtype, D, page, mask, sinks):
    """The kernels that can run this case: the one the engine picks by head size, and the slower
    ones below it (the engine reaches those at other head sizes)."""
    from tinyserve_b200.kernels import ops
    chosen = ops.attention_backend(dtype, D, page)
    return {"tcgen05": ["tcgen05", "mma", "simt"], "mma": ["mma", "simt"], "simt": ["simt"]}[chosen]


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 3e-6), (torch.bfloat16, 1.5e-2)])
@pytest.mark.parametrize("H,G,D,page", [(4, 2, 32, 8), (3, 1, 48, 16), (8, 8, 64, 4), (6, 2, 128, 32)])
@pytest.mark.parametrize("mask", [{"size": 23, "keep_first": 5}, {"size": 8, "keep_first": 20}, {"size": 1, "keep_first": 1},
                                  {"size": 40, "keep_first": 0}, None])
@pytest.mark.parametrize("with_sinks", [False, True])
def test_attention_with_kept_first_keys_and_sinks(dtype, tol, H, G, D, page, mask, with_sinks):
    """Sharp scores (a large scale), so that one key more or less at an edge of the window or of the
    kept tokens moves the output: a whole prompt, single tokens at and around the edges, a portion
    after a prefix, two tokens, and a request of one token."""
    kv_lens, q_lens = [70, 24, 97, 9, 150, 1], [70, 1, 29, 2, 1, 1]
    if mask:
        kv_lens[1] = mask["size"] + mask["keep_first"]          # the decoded token's window ends right behind the kept ones
    k = [draws(n, G, D, seed=10 + i).to(dtype) for i, n in enumerate(kv_lens)]
    v = [draws(n, G, D, seed=20 + i).to(dtype) for i, n in enumerate(kv_lens)]
    q = draws(sum(q_lens), H, D, seed=30).to(dtype)
    sinks = (draws(H, seed=31, scale=3.0) + 2.0).float() if with_sinks else None
    kc, table = _paged(k, page, sum(-(-n // page) for n in kv_lens) + 3, seed=1)
    vc, _ = _paged(v, page, sum(-(-n // page) for n in kv_lens) + 3, seed=1)
    scale = 3.0 / math.sqrt(D)
    want = _attention_plain(q, k, v, q_lens, scale, mask, sinks)
    for backend in attention_backends(dtype, D, page, mask, sinks):
        for splits in (None, 3):
            if splits and backend == "tcgen05":
                continue                       # prefill has no key ranges
            out = _run_attention(q.to(DEV), kc, vc, table, q_lens, kv_lens, page, scale, mask,
                                 sinks.to(DEV) if with_sinks else None, splits, backend)
            assert (out.double().cpu() - want).abs().max() <= tol * want.abs().max(), (backend, splits)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 3e-6), (torch.bfloat16, 1.5e-2)])
@pytest.mark.parametrize("H,G,D,page", [(4, 2, 64, 16), (2, 1, 128, 64), (6, 3, 32, 8)])
@pytest.mark.parametrize("mask", [{"size": 50, "keep_first": 7}, {"size": 130, "keep_first": 129}, {"size": 200, "keep_first": 140}])
def test_long_prompt_walks_the_kept_tiles_first(dtype, tol, H, G, D, page, mask):
    """A prompt of 420 tokens in one portion, and the same prompt's last 150 tokens after a prefix:
    the window's first tile lies behind the kept keys' tiles in every kernel (key tiles of 32, 64
    and 128), kept keys fill a tile, end in the middle of one, and reach into the window's first tile."""
    kv_lens, q_lens = [420, 420], [420, 150]
    k = [draws(n, G, D, seed=50 + i).to(dtype) for i, n in enumerate(kv_lens)]
    v = [draws(n, G, D, seed=60 + i).to(dtype) for i, n in enumerate(kv_lens)]
    q = draws(sum(q_lens), H, D, seed=70).to(dtype)
    sinks = (draws(H, seed=71, scale=2.0) + 1.0).float()
    kc, table = _paged(k, page, sum(-(-n // page) for n in kv_lens) + 3, seed=3)
    vc, _ = _paged(v, page, sum(-(-n // page) for n in kv_lens) + 3, seed=3)
    scale = 3.0 / math.sqrt(D)
    want = _attention_plain(q, k, v, q_lens, scale, mask, sinks)
    for backend in attention_backends(dtype, D, page, mask, sinks):
        out = _run_attention(q.to(DEV), kc, vc, table, q_lens, kv_lens, page, scale, mask, sinks.to(DEV), None, backend)
        assert (out.double().cpu() - want).abs().max() <= tol * want.abs().max(), backend


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_sees_exactly_the_window_and_the_kept_keys(dtype):
    """One key stands out (its score is far above all others): the output is its value when it is
    visible and something else when it is not: just inside and just outside the window, the last
    kept key and the first that is not kept, at a page's border and in its middle."""
    H, G, D, page, n = 2, 1, 32, 16, 300
    direction = torch.ones(D) / math.sqrt(D)
    size, keep = 64, 16
    for marked, seen in ((n - size, True), (n - size - 1, False), (keep - 1, True), (keep, False), (0, True),
                         (n - 1, True), (n - 50, True), (n - 140, False)):
        k = draws(n, G, D, seed=1, scale=0.1).to(dtype)
        v = draws(n, G, D, seed=2).to(dtype)
        k[marked] = (direction * 40).to(dtype)
        q = (direction * 40).to(dtype).repeat(1, H, 1)
        kc, table = _paged([k], page, 40, seed=2)
        vc, _ = _paged([v], page, 40, seed=2)
        for splits in (None, 4):
            out = _run_attention(q.to(DEV), kc, vc, table, [1], [n], page, 1.0, {"size": size, "keep_first": keep}, None, splits)
            miss = (out[0].float().cpu() - v[marked].float()).abs().max().item()
            assert (miss < 2e-2) == seen, (marked, seen, miss)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 3e-6), (torch.bfloat16, 1e-2)])
@pytest.mark.parametrize("H,n,nr,nv,qr,r", [(3, 16, 8, 24, 40, 24), (2, 8, 8, 16, 16, 24), (4, 32, 16, 32, 64, 48), (1, 20, 0, 6, 8, 12)])
def test_latent_rows_and_query_rows(dtype, tol, H, n, nr, nv, qr, r):
    """What the cache keeps of a token (normed latent, rotated shared key part, zeros behind), the
    normed query latent, and the query rows the attention kernel reads; a request that stands at
    position 40 and one that starts, slots in shuffled pages, one token that writes nothing."""
    from tinyserve_b200.kernels import ops
    T, page, eps = 9, 4, 1e-5
    stored = -(-(r + nr) // 16) * 16
    rot = {"base": 100.0, "dims": nr}
    tables = Tables(rot, 64) if nr else None
    pos = torch.tensor([40, 41, 42, 43, 44, 0, 1, 2, 3], dtype=torch.int32)
    gate_cols = 5
    proj = draws(T, qr + r + nr + gate_cols, seed=1, scale=2.0)
    wq, wk = draws(qr, seed=2) + 1, draws(r, seed=3) + 1
    slots = torch.tensor([37, 2, 19, -1, 8, 11, 30, 4, 25], dtype=torch.int32)
    cache = torch.full((10, 1, page, stored), 7.0).to(dtype).to(DEV)
    ql = ops.latent_prepare(on_device(proj, dtype), qr, on_device(wq, dtype), eps, kv_rank=r, rot_dim=nr,
                            kv_weight=on_device(wk, dtype), rotary=tables, positions=pos.to(DEV), cache=cache,
                            slot_mapping=slots.to(DEV))
    want_q = plain.norm_plain(proj[:, :qr], wq, eps)
    assert (ql.double().cpu() - want_q).abs().max() <= tol * want_q.abs().max()
    c = plain.norm_plain(proj[:, qr:qr + r], wk, eps)
    kr = plain.rotate(proj[:, None, qr + r:qr + r + nr], pos, rot)[:, 0] if nr else proj[:, :0]
    flat = cache.view(-1, stored).double().cpu()
    for t in range(T):
        if slots[t] < 0:
            continue
        row = flat[slots[t]]
        assert (row[:r] - c[t]).abs().max() <= tol * c.abs().max()
        assert nr == 0 or (row[r:r + nr] - kr[t]).abs().max() <= tol * kr.abs().max()
        assert (row[r + nr:] == 0).all()
    untouched = [s for s in range(10 * page) if s not in slots.tolist()]
    assert (flat[untouched] == 7.0).all(), "only the step's slots are written"
    # without a key/value latent of its own the layer makes the query latent only
    alone = ops.latent_prepare(on_device(proj[:, :qr], dtype), qr, on_device(wq, dtype), eps)
    assert torch.equal(alone, ql)
    # query rows
    q = draws(T, H * (n + nr), seed=4)
    w_uk = draws(H * n, r, seed=5)
    carried = ops.batched_matmul(on_device(q, dtype).view(T, H, n + nr)[:, :, :n].transpose(0, 1), on_device(w_uk, dtype).view(H, n, r))
    rows = ops.latent_query(carried, on_device(q, dtype), H, n, nr, stored, tables, pos.to(DEV))
    qv = q.view(T, H, n + nr)
    want = torch.einsum("thd,hdr->thr", qv[..., :n], w_uk.view(H, n, r))
    assert (rows[..., :r].double().cpu() - want).abs().max() <= tol * want.abs().max()
    if nr:
        assert (rows[..., r:r + nr].double().cpu() - plain.rotate(qv[..., n:], pos, rot)).abs().max() <= tol * q.abs().max()
    assert (rows[..., r + nr:] == 0).all()
    # the values' side: every head's weighted latent expanded and gated
    mixed = draws(T, H, stored, seed=6)
    w_uv = draws(H * nv, r, seed=7)
    gate = draws(T, H * nv + 3, seed=8)
    values = ops.batched_matmul(on_device(mixed, dtype)[:, :, :r].transpose(0, 1), on_device(w_uv, dtype).view(H, nv, r).transpose(1, 2))
    got = ops.gate_heads(values, on_device(gate, dtype)[:, 3:])
    want = (torch.einsum("thr,hvr->thv", mixed[..., :r], w_uv.view(H, nv, r)).reshape(T, H * nv) * torch.sigmoid(gate[:, 3:]))
    assert (got.double().cpu() - want).abs().max() <= 2 * tol * want.abs().max()


class Batch:
    """What the scan needs of a step: requests of given lengths, each from position ``starts[b]``,
    with state slots ``slots[b]``."""

    def __init__(self, lengths, starts=None, slots=None):
        starts = starts or [0] * len(lengths)
        self.num_requests = len(lengths)
        self.max_q_len = max(lengths)
        cu = np.concatenate([[0], np.cumsum(lengths)])
        self.cu_q = torch.tensor(cu, dtype=torch.int32, device=DEV)
        self.positions = torch.tensor(np.concatenate([np.arange(s, s + n) for s, n in zip(starts, lengths)]),
                                      dtype=torch.int32, device=DEV)
        self.state_slots = torch.tensor(slots or list(range(len(lengths))), dtype=torch.int32, device=DEV)
        self.fresh = torch.tensor([int(s == 0) for s in starts], dtype=torch.int32, device=DEV)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 1e-2)])
@pytest.mark.parametrize("H,n,nv", [(2, 16, 32), (3, 20, 24), (1, 64, 128), (2, 36, 30), (6, 64, 64)])
@pytest.mark.parametrize("segment", [0, 16])
def test_lightning_scan_in_portions_from_and_to_slots(dtype, tol, H, n, nv, segment):
    """silu on q, k and v, one decay per head, the heads normed together, a sigmoid gate: a prompt in
    one go against the same prompt in three portions through a state slot that another request
    used before, beside a second request."""
    from tinyserve_b200.kernels import ops
    T, eps = 50, 1e-5
    decay = [1.0 - 2.0 ** -(2 + a) for a in range(H)]
    proj = draws(T, 2 * H * n + 2 * H * nv, seed=3)
    w = draws(H * nv, seed=4, scale=0.2) + 1
    q, k, v, g = (proj[:, :H * n], proj[:, H * n:2 * H * n], proj[:, 2 * H * n:2 * H * n + H * nv], proj[:, 2 * H * n + H * nv:])
    out = torch.zeros(T, H, nv, dtype=torch.float64)
    for a in range(H):
        S = torch.zeros(n, nv, dtype=torch.float64)
        for t in range(T):
            S = decay[a] * S + torch.outer(plain.silu(k[t, a * n:(a + 1) * n]), plain.silu(v[t, a * nv:(a + 1) * nv]))
            out[t, a] = S.T @ plain.silu(q[t, a * n:(a + 1) * n])
    want = plain.norm_plain(out.reshape(T, H * nv), w, eps) * torch.sigmoid(g)
    state = torch.full((3, H, n, nv), 9.0, dtype=torch.float32, device=DEV)
    dproj = on_device(proj, dtype)
    cols = lambda x, a, b: x[:, a:b]
    call = lambda rows, batch: ops.linear_attention(
        cols(rows, 0, H * n), cols(rows, H * n, 2 * H * n), cols(rows, 2 * H * n, 2 * H * n + H * nv),
        cols(rows, 2 * H * n + H * nv, 2 * H * n + 2 * H * nv), state, batch, H, n, nv, dtype,
        decay=torch.tensor(decay, dtype=torch.float32, device=DEV), norm_weight=on_device(w, torch.float32), eps=eps,
        segment=segment, input_activation="silu", gate_activation="sigmoid", joint_norm=True)
    whole = call(dproj, Batch([T], slots=[1]))
    assert (whole.double().cpu() - want).abs().max() <= tol * want.abs().max()
    kept = state[1].clone()
    # portions of 17, 1 and 32 tokens in slot 2, which holds another request's leftovers; beside it the first 9 tokens again
    got = []
    for at, m in ((0, 17), (17, 1), (18, 32)):
        rows = torch.cat([dproj[at:at + m], dproj[:9]])
        res = call(rows, Batch([m, 9], starts=[at, 0], slots=[2, 0]))
        got.append(res[:m])
        assert (res[m:].double().cpu() - want[:9]).abs().max() <= tol * want.abs().max()
    got = torch.cat(got)
    assert (got.double().cpu() - want).abs().max() <= tol * want.abs().max()
    assert (state[2] - kept).abs().max() <= 1e-5 * kept.abs().max(), "the state after portions is the state after the whole"


@pytest.mark.parametrize("E,top", [(8, 2), (5, 5), (1, 1), (40, 7), (3, 1)])
def test_router_keeps_the_largest_probabilities_as_they_are(E, top):
    from tinyserve_b200.kernels import ops
    z = torch.randn(33, E, generator=torch.Generator().manual_seed(E), dtype=torch.float64) * 2.0      # (no two alike)
    z[4] = 0.0                                   # all equal: the lowest numbers win
    gates = ops.moe_route(on_device(z, torch.float32), top).double().cpu()
    s = torch.softmax(z, -1)
    w, idx = torch.topk(s, top, -1)
    want = torch.zeros_like(s).scatter(1, idx, w)
    want[4] = 0.0
    want[4, :top] = 1.0 / E
    assert (gates - want).abs().max() < 1e-6
    assert ((gates > 0).sum(-1) == top).all()
    # the activation kernel routes by itself when it gets the logits: the same numbers in one launch
    for dtype in (torch.float32, torch.bfloat16):
        a = draws(33, E * 24, seed=3)
        two = ops.moe_activate_(on_device(a, dtype), ops.moe_route(on_device(z, torch.float32), top), E)
        one = ops.moe_activate_(on_device(a, dtype), None, E, logits=on_device(z, torch.float32), top=top)
        assert torch.equal(one, two)
        expect = torch.relu(a).pow(2).view(33, E, 24) * want[:, :, None]
        assert (one.double().cpu().view(33, E, 24) - expect).abs().max() <= (1e-6 if dtype == torch.float32 else 8e-3) * expect.abs().max()


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("E,top,ff,width", [(4, 2, 40, 64), (6, 1, 24, 64), (1, 1, 48, 96), (7, 4, 72, 96), (16, 5, 32, 128),
                                            (40, 7, 16, 64)])
@pytest.mark.parametrize("T", [29, 300])
def test_mixture_of_experts_against_the_plain_one(dtype, tol, E, top, ff, width, T):
    """A few tokens (all experts on all tokens, the unchosen ones times zero) and a step of 300 tokens
    (in bfloat16: rows sorted by expert, ragged groups, some experts with few rows or none)."""
    from tinyserve_b200.parts.moe import MixtureOfExperts
    h = draws(T, width, seed=1)
    W = {"router": draws(E, width, seed=2, scale=0.5)}
    for e in range(E):
        W[f"e{e}.up"], W[f"e{e}.down"] = draws(ff, width, seed=10 + e, scale=0.2), draws(width, ff, seed=40 + e, scale=0.2)
    part = MixtureOfExperts(width, ff, E, top)
    part.bind({"router.weight": on_device(W["router"], dtype),
               "up.weight": on_device(torch.cat([W[f"e{e}.up"] for e in range(E)]), dtype),
               "down.weight": on_device(torch.cat([W[f"e{e}.down"] for e in range(E)]), dtype)})
    from tinyserve_b200.kernels import ops
    got = ops.materialize(part.forward(on_device(h, dtype), None))
    want = plain.experts(h, W, "", {"router": {"experts": E, "top": top}})
    # (in bfloat16 a token whose router scores are a rounding apart may take another expert: one row in fifty may differ)
    err = (got.double().cpu() - want).abs().max(-1).values
    allowed = T // 50 if dtype == torch.bfloat16 else 0
    assert int((err > tol * want.abs().max()).sum()) <= allowed
    if dtype == torch.bfloat16 and T >= ops.MOE_GROUPED_MIN_TOKENS and top < E:
        # the other form on the same input: all experts on all tokens
        keep, ops.MOE_GROUPED_MIN_TOKENS = ops.MOE_GROUPED_MIN_TOKENS, 10 ** 9
        try:
            dense = ops.materialize(part.forward(on_device(h, dtype), None))
        finally:
            ops.MOE_GROUPED_MIN_TOKENS = keep
        assert (got.double() - dense.double()).abs().max() <= tol * want.abs().max(), "both forms route alike and agree to a rounding"


# ----------------------------------------------------------------------------- whole models
LENGTHS = {"P": [5, 37, 40, 70, 2, 1, 33], "Q": [1, 9, 64, 100, 31, 48], "R": [150, 130, 57, 3, 129]}


@pytest.fixture(scope="module", params=sorted(DELILORN_TINY))
def model(request, tmp_path_factory):
    name = request.param
    folder = make_delilorn_dir(tmp_path_factory.mktemp(f"delilorn{name}"), name, seed=41)
    cfg, weights = plain.load_folder(folder)
    reqs = {f"r{i}": random_ids(cfg["vocab"], n, seed=300 + i) for i, n in enumerate(LENGTHS[name])}
    ref = {rid: plain.logits(cfg, weights, ids) for rid, ids in reqs.items()}
    return {"name": name, "folder": folder, "cfg": cfg, "weights": weights, "requests": reqs, "ref": ref}


def run_replay(folder, dtype, steps, out_dir, page=16, max_live=4, graphs=False):
    from tinyserve_b200.engine import replay
    runner = replay.make_runner(folder, dtype, max_live_tokens(steps, max(64, page)), block_size=page,
                                max_live=max_live, use_cuda_graphs=graphs)
    done = []
    replay.replay(runner, lines_of(steps), str(out_dir), done.append)
    assert done == [f"done {s['step']}" for s in steps]
    runner.manager.check_invariants()
    assert not runner.manager.requests and all(p.num_free == p.num_usable for p in runner.manager.pools)
    outputs = {}
    for s in steps:
        wanted = sum(len(e["want"]) for e in s["entries"])
        if wanted:
            data = np.fromfile(os.path.join(str(out_dir), f"{s['step']}.f32"), dtype="<f4")
            outputs[s["step"]] = torch.from_numpy(data.reshape(wanted, runner.model.vocab_size))
    return outputs, runner


def check(model, dtype, steps, out_dir, slack=1.0, **kw):
    outputs, runner = run_replay(model["folder"], dtype, steps, out_dir, **kw)
    got = collect_logits(steps, outputs, model["cfg"]["vocab"])
    # In bfloat16 a token whose router scores lie within a rounding of one another may take another
    # expert than the plain model does, and the norm behind the experts carries that choice into the
    # stream at full size; such a token is no fault (measured on a B200, configuration R with 16 experts:
    # 2 to 4 of 150 positions, the same ones in every schedule, at a median difference of 0.003).  One
    # position in twenty may differ for that reason; none in 32-bit, where every schedule is held to
    # the plain model at every position.
    positions = sum(out.shape[0] for out in got.values())
    allowed = positions // 20 if dtype == "bfloat16" else 0
    over = []
    for rid, out in got.items():
        ref = model["ref"][rid.rstrip("x")]
        assert out.shape == ref.shape
        scale = ref.abs().max().item()
        err = (out.double() - ref).abs().max(-1).values / scale
        rms = (out.double() - ref).pow(2).mean(-1).sqrt() / scale
        bad = ((err > slack * TOLERANCE[dtype]) | (rms > slack * RMS_TOLERANCE[dtype]))
        seen = MEASURED.setdefault((model["name"], dtype), [0.0, 0.0])
        if (~bad).any():
            seen[0], seen[1] = max(seen[0], err[~bad].max().item()), max(seen[1], rms[~bad].max().item())
        over += [(rid, int(i), err[int(i)].item(), rms[int(i)].item()) for i in bad.nonzero()]
    assert len(over) <= allowed, (f"{model['name']} {dtype}: {len(over)} of {positions} positions differ; the first is place "
                                  f"{over[0][1]} of request {over[0][0]} (error {over[0][2]:.3e}, rms {over[0][3]:.3e})")
    return runner


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_prompts(model, dtype, tmp_path):
    check(model, dtype, schedule_whole(model["requests"]), tmp_path)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prompt_against_token_by_token(model, dtype, tmp_path):
    """The last 32 tokens one by one; and everything but the first token one by one (the first
    tokens of a sequence, a window that passes over decoded tokens, a long run of decoding)."""
    check(model, dtype, schedule_tail_decode(model["requests"], 32), tmp_path / "tail")
    longest = max(model["requests"], key=lambda r: len(model["requests"][r]))
    one = {longest: model["requests"][longest]}
    check(model, dtype, schedule_tail_decode(one, len(one[longest]) - 1), tmp_path / "all", graphs=dtype == "bfloat16")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_portions_down_to_two_tokens(model, dtype, tmp_path):
    check(model, dtype, schedule_portions(model["requests"]), tmp_path / "a")
    check(model, dtype, schedule_portions(model["requests"], sizes=(2,)), tmp_path / "twos")
    check(model, dtype, schedule_portions(model["requests"], sizes=(16, 1, 15, 17, 32, 3)), tmp_path / "edges", page=8)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", [0, 1])
def test_mixed_batches_reuse_pages_and_slots(model, dtype, seed, tmp_path):
    reqs = dict(model["requests"])
    more = {f"{rid}x": ids for rid, ids in reqs.items()}
    steps = schedule_mixed({**reqs, **more}, max_live=4, seed=seed)
    assert max(len(s["entries"]) for s in steps) >= 3
    assert any(len({len(e["tokens"]) == 1 for e in s["entries"]}) == 2 for s in steps), "portions beside single tokens"
    runner = check(model, dtype, steps, tmp_path, max_live=4)
    assert len(reqs) + len(more) > runner.manager.slots.num_slots == 4, "state slots are used again"
    total = sum(-(-len(i) // 16) for i in {**reqs, **more}.values())
    assert total > runner.manager.pools[0].num_usable, "the pool is too small to avoid reuse"


def test_batch_of_unequal_requests_equals_each_alone(model, tmp_path):
    reqs = model["requests"]
    together = [{"step": 0, "entries": [{"id": r, "tokens": ids, "want": list(range(len(ids)))} for r, ids in reqs.items()],
                 "end": list(reqs)}]
    out_a, _ = run_replay(model["folder"], "float32", together, tmp_path / "a", max_live=len(reqs))
    out_b, _ = run_replay(model["folder"], "float32", schedule_whole(reqs), tmp_path / "b")
    a = collect_logits(together, out_a, model["cfg"]["vocab"])
    b = collect_logits(schedule_whole(reqs), out_b, model["cfg"]["vocab"])
    for rid in reqs:
        # (the attention kernel cuts a request's keys into ranges by how full the batch is: the
        # order of its sums, not what is summed, depends on the batch)
        assert (a[rid] - b[rid]).abs().max() <= 1e-5 * b[rid].abs().max()


@pytest.mark.parametrize("seed", range(10))
def test_drawn_configurations(seed, tmp_path):
    """Configurations drawn from a seed (odd head sizes, head counts, ranks, windows, orders, shared
    caches): whole prompts, portions and a mixed batch against the plain implementation."""
    from tinyserve_b200.config import config_from_dict
    from tinyserve_b200.weights import write_random_model
    raw = random_delilorn_config_dict(seed)
    folder = decisive_routers(write_random_model(config_from_dict(raw), str(tmp_path / "model"), seed=seed))
    cfg, weights = plain.load_folder(folder)
    reqs = {f"r{i}": random_ids(cfg["vocab"], n, seed=700 + 10 * seed + i) for i, n in enumerate((37, 5, 66, 1))}
    ref = {rid: plain.logits(cfg, weights, ids) for rid, ids in reqs.items()}
    model = {"name": f"drawn{seed}", "folder": folder, "cfg": cfg, "requests": reqs, "ref": ref}
    check(model, "float32", schedule_whole(reqs), tmp_path / "whole", slack=2.0)
    check(model, "float32", schedule_portions(reqs, sizes=(17, 2, 16, 1, 3)), tmp_path / "portions", slack=2.0)
    check(model, "float32", schedule_mixed(reqs, max_live=3, seed=seed), tmp_path / "mixed", slack=2.0, max_live=3)
    check(model, "bfloat16", schedule_mixed(reqs, max_live=3, seed=seed), tmp_path / "mixed16", slack=2.0, max_live=3)


# ----------------------------------------------------------------------------- weights that show a fault
def sharpened(folder, out, cfg):
    """The same model with its memories made long and its attention sharp: lightning decays near one,
    large attention scales (a far key, a key at a window's edge or a wrong position then moves the
    logits), and sinks of unequal, large size (a sink that is left out, or given to the wrong head,
    changes how much of the values gets through)."""
    weights = load_file(os.path.join(folder, "model.safetensors"))
    cfg = {**cfg, "layers": [dict(layer) for layer in cfg["layers"]]}
    for i, layer in enumerate(cfg["layers"]):
        m = dict(layer["mixer"])
        if layer["type"] == "lightning":
            m["decay"] = [1.0 - 2.0 ** -(6 + a) for a in range(m["heads"])]
        else:
            m["scale"] = 12.0 if layer["type"] == "attention" else 6.0
        if layer["type"] == "latent_attention":
            weights[f"l{i}.mix.sink"] = torch.tensor([1.5 * (-1) ** a * (1 + a) for a in range(m["heads"])]).bfloat16()
        layer["mixer"] = m
    os.makedirs(out, exist_ok=True)
    save_file(weights, os.path.join(out, "model.safetensors"))
    with open(os.path.join(out, "config.json"), "w") as fh:
        json.dump(cfg, fh)
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["P", "R"])
def test_far_keys_window_edges_sinks_and_long_memories(dtype, name, tmp_path):
    folder = make_delilorn_dir(tmp_path / "base", name, seed=43)
    cfg, _ = plain.load_folder(folder)
    sharp = sharpened(folder, str(tmp_path / "sharp"), cfg)
    cfg, weights = plain.load_folder(sharp)
    ids = random_ids(cfg["vocab"], 200, seed=7)
    ids[130] = ids[199] = ids[3]              # a token that comes back far behind
    reqs = {"far": ids, "near": ids[:70]}
    ref = {rid: plain.logits(cfg, weights, t) for rid, t in reqs.items()}
    short = plain.logits(cfg, weights, ids[60:])                 # the same tail without what lies far back
    assert (short[-1] - ref["far"][-1]).abs().max() > 0.02 * ref["far"].abs().max(), "the far tokens matter here"
    # the plain model with one key more in every window, and without its sinks, is another model
    wider = {**cfg, "layers": [{**l, "mixer": ({**l["mixer"], "mask": {**l["mixer"]["mask"], "size": l["mixer"]["mask"]["size"] + 1}}
                                               if l["mixer"].get("mask") else l["mixer"])} for l in cfg["layers"]]}
    assert (plain.logits(wider, weights, ids) - ref["far"]).abs().max() > 1e-3 * ref["far"].abs().max(), "one key at the edge matters"
    no_sink = {k: (torch.full_like(v, -30.0) if k.endswith(".sink") else v) for k, v in weights.items()}
    assert (plain.logits(cfg, no_sink, ids) - ref["far"]).abs().max() > 1e-2 * ref["far"].abs().max(), "the sinks matter"
    model = {"name": name + "sharp", "folder": sharp, "cfg": cfg, "requests": reqs, "ref": ref}
    slack = 2.0 if dtype == "float32" else 3.0
    check(model, dtype, schedule_whole(reqs), tmp_path / "whole", slack=slack)
    check(model, dtype, schedule_tail_decode(reqs, 90), tmp_path / "tail", slack=slack)
    check(model, dtype, schedule_portions(reqs, sizes=(63, 2, 1, 64, 5, 16, 15)), tmp_path / "portions", slack=slack)
    check(model, dtype, schedule_mixed({**reqs, "farx": ids, "nearx": ids[:70]}, max_live=3, seed=5), tmp_path / "mixed",
          slack=slack, max_live=3)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_head_sizes_of_real_models(dtype, tmp_path):
    """Cache rows of 256 and of 128, attention heads of 128 behind a window beside kept tokens, state heads
    of 128 x 256, pages of 64: the kernels that real layer sizes reach (tcgen05 prefill, mma.sync with wide
    heads, decode by whole pages), prompts longer than two key tiles of any kernel."""
    from delilorn_configs import _latent, _moe
    from tinyserve_b200.config import config_from_dict
    from tinyserve_b200.weights import write_random_model
    raw = {"architecture": "Delilorn", "vocab": 1000, "width": 512, "norm": {"eps": 1e-6}, "layers": [
        {"type": "latent_attention", "mlp": _moe(256, 8, 2), "mixer": _latent(4, 128, 64, 128, 256, 192, 0.08, 1e4)},
        {"type": "lightning", "mlp": _moe(256, 8, 2), "mixer": {"heads": 2, "dim": 128, "vdim": 256, "decay": [0.97, 0.999]}},
        {"type": "latent_attention", "mlp": _moe(256, 8, 2), "mixer": _latent(4, 128, 32, 128, 256, 96, 0.08, 1e4)},
        {"type": "attention", "mlp": _moe(256, 8, 2), "mixer": {
            "heads": 4, "kv_heads": 1, "dim": 128, "vdim": 128, "scale": 0.09,
            "rot": {"base": 1e6, "dims": 64, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 256}},
            "mask": {"size": 150, "keep_first": 4}}},
        {"type": "latent_attention", "mlp": None, "mixer": _latent(8, 64, 64, 64, 128, 192, 0.1, 1e4, kv_from=0)},
    ]}
    folder = decisive_routers(write_random_model(config_from_dict(raw), str(tmp_path / "model"), seed=5))
    cfg, weights = plain.load_folder(folder)
    reqs = {"a": random_ids(1000, 420, seed=1), "b": random_ids(1000, 130, seed=2)}
    ref = {rid: plain.logits(cfg, weights, ids) for rid, ids in reqs.items()}
    model = {"name": "real", "folder": folder, "cfg": cfg, "requests": reqs, "ref": ref}
    check(model, dtype, schedule_tail_decode(reqs, 40), tmp_path / "tail", page=64)
    check(model, dtype, schedule_mixed(reqs, max_live=2, seed=1, chunk_sizes=(200, 2, 129, 64, 1)), tmp_path / "mixed", max_live=2)


# ----------------------------------------------------------------------------- the entry point
def test_greedy_generation_through_the_scheduler(tmp_path):
    """Five prompts of unequal length through LLM.generate with three state slots and at most
    48 tokens a step (prompts in portions beside decoding requests, slots and pages used again)."""
    from tinyserve_b200 import LLM, SamplingParams
    folder = make_delilorn_dir(tmp_path, "P", seed=44)
    cfg, weights = plain.load_folder(folder)
    prompts = [random_ids(cfg["vocab"], n, seed=500 + n) for n in (3, 60, 17, 1, 90)]
    params = SamplingParams(temperature=0.0, max_tokens=12, repetition_penalty=1.0, ignore_eos=True)
    llm = LLM(folder, dtype="float32", max_model_len=128, block_size=16, max_num_seqs=3, max_num_batched_tokens=48,
              num_blocks=20, use_cuda_graphs=False)
    outs = llm.generate(prompts, params)
    for prompt, out in zip(prompts, outs):
        want, gaps = plain.greedy(cfg, weights, prompt, 12)
        assert out.finished and len(out.token_ids) == 12
        for j, (a, b, gap) in enumerate(zip(out.token_ids, want, gaps)):
            if gap < 1e-3:
                break                        # a near tie: either side is a right answer, the rest differs
            assert a == b, (len(prompt), j)
    outs16 = LLM(folder, dtype="bfloat16", max_model_len=128, block_size=16, max_num_seqs=3,
                 max_num_batched_tokens=48, num_blocks=20, use_cuda_graphs=True).generate(prompts, params)
    for prompt, out in zip(prompts, outs16):
        ids = list(prompt)
        for tok in out.token_ids:
            row = plain.logits(cfg, weights, ids)[-1]
            assert row[tok] >= row.max() - 0.05 * row.abs().max()
            ids.append(tok)


def test_programs_replay_and_generate(tmp_path):
    """bin/trace_run and ``python -m tinyserve_b200 generate`` as programs on a Delilorn folder: the
    architecture is chosen by config.json; stdin to files, 'done' lines, exit code 0; greedy tokens."""
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    folder = make_delilorn_dir(tmp_path / "m", "Q", seed=2)
    cfg, weights = plain.load_folder(folder)
    reqs = {"p": random_ids(cfg["vocab"], 45, seed=1), "q": random_ids(cfg["vocab"], 30, seed=2)}
    steps = schedule_mixed(reqs, max_live=2, seed=0)
    out = tmp_path / "out"
    proc = subprocess.run(
        [sys.executable, os.path.join(root, "bin", "trace_run"), "--model", folder, "--dtype", "float32",
         "--out", str(out), "--max-tokens", str(max_live_tokens(steps))],
        input="\n".join(lines_of(steps)) + "\n", capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert proc.stdout.split("\n")[:-1] == [f"done {s['step']}" for s in steps]
    outputs = {}
    for s in steps:
        wanted = sum(len(e["want"]) for e in s["entries"])
        outputs[s["step"]] = torch.from_numpy(np.fromfile(out / f"{s['step']}.f32", dtype="<f4").reshape(wanted, cfg["vocab"]))
    got = collect_logits(steps, outputs, cfg["vocab"])
    for rid, ids in reqs.items():
        ref = plain.logits(cfg, weights, ids)
        assert (got[rid].double() - ref).abs().max().item() < TOLERANCE["float32"] * ref.abs().max().item()
    prompt = reqs["q"][:9]
    proc = subprocess.run(
        [sys.executable, "-m", "tinyserve_b200", "generate", "--model", folder, "--dtype", "float32", "--prompt-ids",
         ",".join(map(str, prompt)), "--max-tokens", "5", "--repetition-penalty", "1.0", "--ignore-eos", "--max-model-len", "64",
         "--max-num-seqs", "2", "--max-num-batched-tokens", "32", "--num-blocks", "16", "--block-size", "16"],
        capture_output=True, text=True, timeout=600, cwd=root)
    assert proc.returncode == 0, proc.stderr[-2000:]
    tokens = [int(t) for t in proc.stdout.strip().split("\n")[-1].split()]
    want, gaps = plain.greedy(cfg, weights, prompt, 5)
    for a, b, gap in zip(tokens, want, gaps):
        if gap < 1e-3:
            break
        assert a == b, (tokens, want)
    assert len(tokens) == 5


def test_measured_differences_are_reported():
    print({k: (f"{v[0]:.2e}", f"{v[1]:.2e}") for k, v in sorted(MEASURED.items())})
