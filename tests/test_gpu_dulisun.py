"""The Dulisun design in the engine against its plain implementation (``plain_dulisun``): each
mechanism alone, then whole models under every way of cutting the work, in float32 and bfloat16.

The configurations are small and differ from one another in every size and constant: head
counts and groups, key and value sizes, how many dimensions rotate, chunk sizes that are a
page, less than a page and no multiple of a page, expert counts, groups and top counts
(also values that make groups or the top count 1), a layer without a feed-forward, a
feed-forward without a shared expert.  Where random weights would hide a fault the inputs are
made so that it shows: one key is scaled until its score stands out, a sink is made large.
"""
import json
import math
import os

import numpy as np
import pytest
import torch

import helpers as H
import plain_dulisun as pd

pytestmark = pytest.mark.gpu


def _attn(heads, kv, dim, vdim, rot, chunk, scale, base=10000.0):
    return {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "rot": {"base": base, "dims": rot} if rot else None,
            "mask": {"size": chunk} if chunk else None, "scale": scale}


def _moe(experts, top, count, keep, ff, shared):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "groups": {"count": count, "keep": keep}}}
    m["shared"] = {"ff": shared} if shared else None
    return m


CONFIGS = {
    # grouped heads, value shorter than key, half of the head rotates, a chunk that is no multiple of a page,
    # a layer without feed-forward in the middle
    "P": {"architecture": "Dulisun", "vocab": 333, "width": 96, "norm": {"eps": 1e-5}, "layers": [
        {"type": "attention", "mixer": _attn(4, 2, 32, 24, 16, 24, 0.2), "mlp": _moe(8, 3, 4, 2, 40, 56)},
        {"type": "attention", "mixer": _attn(4, 2, 32, 24, 16, 24, 0.2), "mlp": None},
        {"type": "attention", "mixer": _attn(4, 4, 32, 32, 32, 40, 0.15, 500.0), "mlp": _moe(6, 2, 1, 1, 48, 0)}]},
    # one key/value head, the whole head rotates, chunk = one page, top 1, groups that keep one expert group of two
    "Q": {"architecture": "Dulisun", "vocab": 257, "width": 72, "norm": {"eps": 3e-6}, "layers": [
        {"type": "attention", "mixer": _attn(3, 1, 48, 48, 48, 16, 0.1, 1e6), "mlp": _moe(4, 1, 2, 1, 24, 24)},
        {"type": "attention", "mixer": _attn(6, 3, 16, 16, 8, 7, 0.3), "mlp": _moe(4, 4, 1, 1, 32, 8)}]},
    # sizes the tensor-core kernels take (multiples of 64), head 64, chunk 128, more experts
    "R": {"architecture": "Dulisun", "vocab": 512, "width": 128, "norm": {"eps": 1e-6}, "layers": [
        {"type": "attention", "mixer": _attn(4, 2, 64, 64, 32, 128, 0.125), "mlp": _moe(16, 4, 4, 2, 64, 128)},
        {"type": "attention", "mixer": _attn(2, 1, 128, 128, 64, 48, 0.09), "mlp": _moe(8, 2, 2, 2, 128, 64)}]},
    # sizes no fast kernel takes: width and vocabulary that are no multiple of 4, heads of 20 and 6, experts' hidden sizes of 30
    # and 14, three experts; one layer without a mask (every earlier key is seen), one with chunks of 5, one without rotation
    "S": {"architecture": "Dulisun", "vocab": 101, "width": 90, "norm": {"eps": 1e-5}, "layers": [
        {"type": "attention", "mixer": _attn(3, 3, 20, 20, 10, 0, 0.25), "mlp": _moe(3, 2, 1, 1, 30, 14)},
        {"type": "attention", "mixer": _attn(4, 2, 6, 6, 6, 5, 0.5, 77.0), "mlp": _moe(3, 1, 3, 2, 14, 0)},
        {"type": "attention", "mixer": _attn(2, 1, 16, 16, 0, 33, 0.2), "mlp": None}]},
    # no mask with heads the tensor-core attention kernels take (64: tcgen05; 48: mma.sync), sinks alone
    "U": {"architecture": "Dulisun", "vocab": 320, "width": 64, "norm": {"eps": 1e-5}, "layers": [
        {"type": "attention", "mixer": _attn(2, 1, 64, 64, 16, 0, 0.125), "mlp": _moe(4, 2, 2, 1, 32, 32)},
        {"type": "attention", "mixer": _attn(4, 2, 48, 48, 48, 0, 0.15), "mlp": None}]},
}
PAGE = {"P": 16, "Q": 16, "R": 32, "S": 8, "U": 16}
LENGTHS = {"P": [1, 9, 50, 131], "Q": [3, 20, 77], "R": [5, 140, 300], "S": [2, 31, 90], "U": [7, 150, 260]}
FP32_TOL, BF16_TOL = 1e-4, 4e-2


def load_plain(folder):
    from aien_sovereign_core_mv_b200.weights.safetensors_io import CheckpointFiles
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    files = CheckpointFiles(folder)
    tensors = {n: files.tensor(n).float().numpy().astype(np.float64) for n in files.names()}
    files.close()
    return cfg, tensors


def tokens(which, n, seed):
    return [int(t) for t in np.random.default_rng(seed).integers(0, CONFIGS[which]["vocab"], n)]


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    from aien_sovereign_core_mv_b200 import write_random_model
    root = tmp_path_factory.mktemp("dulisun")
    out = {}
    for i, which in enumerate(CONFIGS):
        d = write_random_model(os.path.join(str(root), which), CONFIGS[which], 40 + i)
        cfg, tensors = load_plain(d)
        reqs = {j + 1: tokens(which, n, 100 * i + n) for j, n in enumerate(LENGTHS[which])}
        want = {rid: pd.forward(cfg, tensors, toks) for rid, toks in reqs.items()}
        out[which] = (d, reqs, want)
    return out


def check(collected, want, tol, what):
    """float32: every row within ``tol``.  bfloat16: a router whose two best candidates lie closer
    than the rounding of its input may choose the other expert, which changes that token by far
    more than rounding does; such rows are counted, and at most one in 25 (or one) may be over."""
    assert collected, f"{what}: nothing was collected"
    strict = tol <= FP32_TOL
    over, total = [], 0
    for rid, rows in collected.items():
        pos = sorted(rows)
        got, ref = np.stack([rows[p] for p in pos]), want[rid][pos]
        if strict:
            H.assert_close(got, ref, tol, f"{what} request {rid} (positions {pos[0]}..{pos[-1]})")
            continue
        assert np.isfinite(got).all(), f"{what}: non-finite values"
        bad = np.abs(got - ref).max(axis=1) > tol * np.abs(ref).max()
        over += [(rid, pos[i]) for i in np.where(bad)[0]]
        total += len(pos)
    assert len(over) <= max(1, total // 25), f"{what}: {len(over)} of {total} rows over the bound: {over[:12]}"


DTYPES = [("float32", FP32_TOL), ("bfloat16", BF16_TOL)]


# ------------------------------------------------------------------ mechanisms alone
def make_ctx(dtype, positions, seq_of_token, q_start, ctx_len, groups=()):
    from test_gpu_parts import make_ctx as mk
    return mk(dtype, positions, seq_of_token, q_start, ctx_len, groups)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width", [72, 2304])
def test_offset_norm_on_a_branch_output(dtype, width):
    from aien_sovereign_core_mv_b200.registry import make_part
    norm = make_part("norm", "rmsnorm", size=width, eps=1e-5, weight_offset=1.0)
    g = torch.Generator().manual_seed(3)
    w = ((torch.rand(width, generator=g) - 0.5) * 0.4).to(torch.bfloat16)
    norm.bind({"weight": w.cuda()})
    T = 5
    ctx = make_ctx(dtype, list(range(T)), [0] * T, [0, T], [T])
    x = torch.randn(T, width, generator=g).cuda()
    parts = torch.randn(3, T, width, generator=g).cuda()                 # float32 parts, as routed experts leave them
    b = torch.randn(T, width, generator=g).to(dtype).cuda()
    x0 = x.clone()
    h = norm.add_normed(ctx, x, parts, b, want_copy=True)
    y = parts.double().sum(0).cpu().numpy() + b.double().cpu().numpy()
    want = x0.double().cpu().numpy() + pd.offset_rmsnorm(y, w.double().numpy(), 1e-5)
    H.assert_close(x.cpu().numpy(), want, 2e-6, "stream after the branch norm")
    H.assert_close(h.float().cpu().numpy(), want, 1e-6 if dtype == torch.float32 else 8e-3, "copy of the stream")
    assert (h is x) == (dtype == torch.float32)
    # one tensor, no second source; then the norm of the stream in place
    x1 = x0.clone()
    norm.add_normed(ctx, x1, b)
    H.assert_close(x1.cpu().numpy(), x0.double().cpu().numpy() + pd.offset_rmsnorm(b.double().cpu().numpy(), w.double().numpy(), 1e-5), 2e-6, "one source")
    x2 = x0.clone()
    norm.norm_stream(ctx, x2)
    H.assert_close(x2.cpu().numpy(), pd.offset_rmsnorm(x0.double().cpu().numpy(), w.double().numpy(), 1e-5), 2e-6, "norm in place")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hd,hdv,rot,nq,nkv", [(32, 24, 16, 4, 2), (64, 64, 64, 3, 1), (20, 20, 0, 2, 2), (128, 128, 32, 2, 1)])
def test_rotation_of_pairs_unit_norm_and_cache_write(dtype, hd, hdv, rot, nq, nkv):
    from aien_sovereign_core_mv_b200 import kernels as K
    g = torch.Generator().manual_seed(hd + rot)
    T, eps, base = 7, 1e-5, 777.0
    pos = [0, 1, 5, 63, 64, 1000, 70001]
    qk = torch.randn(2, T, (nq + nkv) * hd, generator=g).cuda()          # two float32 parts, as a product cut over K leaves them
    q, k = qk[..., :nq * hd], qk[..., nq * hd:]
    cos = sin = None
    if rot:
        inv = np.array([base ** (-2.0 * i / rot) for i in range(rot // 2)])
        ang = np.asarray(pos, dtype=np.float64)[:, None] * inv[None]
        cos, sin = torch.tensor(np.cos(ang), dtype=torch.float32).cuda(), torch.tensor(np.sin(ang), dtype=torch.float32).cuda()
    slots = torch.tensor([3, 9, 0, -1, 5, 8, 1], dtype=torch.int32).cuda()
    kc = torch.zeros(12, nkv, hd, dtype=dtype).cuda()
    vc = torch.zeros(12, nkv, hdv, dtype=dtype).cuda()
    qo = torch.empty(T, nq * hd, dtype=dtype).cuda()
    K.qk_rope_pairs_unit_kv_write(q, k, None, hd, hdv, True, eps, cos, sin, rot, slots, kc, vc, qo)
    qs = qk.double().sum(0).cpu().numpy()
    qh, kh = qs[:, :nq * hd].reshape(T, nq, hd), qs[:, nq * hd:].reshape(T, nkv, hd)
    wq = pd.unit_rms(pd.rotate_interleaved(qh, pos, base, rot), eps)
    wk = pd.unit_rms(pd.rotate_interleaved(kh, pos, base, rot), eps)
    tol = 3e-6 if dtype == torch.float32 else 8e-3
    H.assert_close(qo.float().cpu().numpy().reshape(T, nq, hd), wq, tol, "q")
    for t, s in enumerate(slots.tolist()):
        if s < 0:
            continue
        H.assert_close(kc[s].float().cpu().numpy(), wk[t], tol, f"key of token {t}")
        H.assert_close(vc[s].float().cpu().numpy(), kh[t][:, :hdv], tol, f"value of token {t}: the key as projected")
    used = [s for s in slots.tolist() if s >= 0]
    assert all(float(kc[s].abs().max()) == 0.0 for s in range(12) if s not in used)      # a token without a slot writes nothing


def _paged(keys, vals, page, order):
    """Scatter [n, g, d] rows into pages taken in ``order``; returns caches and the block table row."""
    n = keys.shape[0]
    nb = (n + page - 1) // page
    kc = torch.zeros((max(order) + 1) * page, *keys.shape[1:], dtype=keys.dtype)
    vc = torch.zeros((max(order) + 1) * page, *vals.shape[1:], dtype=vals.dtype)
    for j in range(n):
        s = order[j // page] * page + j % page
        kc[s], vc[s] = keys[j], vals[j]
    return kc, vc, order[:nb]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("chunk,page,hd,hdv,nq,nkv", [(24, 16, 32, 24, 4, 2), (16, 16, 64, 64, 6, 2), (64, 16, 64, 64, 2, 2), (100, 32, 128, 128, 2, 1)])
def test_attention_sees_its_chunk_and_the_sink(dtype, chunk, page, hd, hdv, nq, nkv):
    """Keys just inside and just outside the chunk's edge are scaled until their scores stand out; a
    mask that is one position off changes the output by orders of magnitude more than the bound."""
    from aien_sovereign_core_mv_b200 import kernels as K
    g = torch.Generator().manual_seed(chunk + hd)
    n = 3 * chunk + 5
    keys = torch.randn(n, nkv, hd, generator=g)
    vals = torch.randn(n, nkv, hdv, generator=g)
    qpos = [0, 1, chunk - 1, chunk, chunk + 1, 2 * chunk - 1, 2 * chunk, 3 * chunk, n - 1]
    for p in (chunk - 1, chunk, 2 * chunk - 1, 2 * chunk, 3 * chunk - 1, 3 * chunk, 0):
        keys[p] *= 3.0                                               # the edges stand out
    q = torch.randn(len(qpos), nq, hd, generator=g)
    q = q.to(dtype).float(); keys = keys.to(dtype).float(); vals = vals.to(dtype).float()
    sinks = torch.tensor([(-1.0) ** h * (0.5 + 2.5 * h) for h in range(nq)])          # one large, one far below
    scale = 0.4 / math.sqrt(hd)
    order = list(reversed(range((n + page - 1) // page + 2)))         # pages in descending order with two unused ones
    kc, vc, row = _paged(keys, vals, page, order)
    mb = len(row) + 3
    bt = torch.full((2, mb), -1, dtype=torch.int32)
    bt[1, :len(row)] = torch.tensor(row, dtype=torch.int32)
    out = torch.empty(len(qpos), nq * hdv, dtype=dtype).cuda()
    K.paged_attention_generic(q.reshape(len(qpos), -1).to(dtype).cuda(), kc.to(dtype).cuda(), vc.to(dtype).cuda(), bt.cuda(), mb,
                              torch.ones(len(qpos), dtype=torch.int32).cuda(), torch.tensor(qpos, dtype=torch.int32).cuda(), out,
                              nq, nkv, hd, page, 0, scale, chunk=chunk, sinks=sinks.cuda(), value_dim=hdv)
    want = pd.chunk_sink_attention(q.double().numpy(), keys.double().numpy(), vals.double().numpy(), qpos, list(range(n)), scale, chunk,
                                   sinks.double().numpy())
    H.assert_close(out.float().cpu().numpy().reshape(len(qpos), nq, hdv), want, 2e-5 if dtype == torch.float32 else 1.5e-2, "attention")
    # the same without a sink and without a chunk differs: both are in the result
    out2 = torch.empty_like(out)
    K.paged_attention_generic(q.reshape(len(qpos), -1).to(dtype).cuda(), kc.to(dtype).cuda(), vc.to(dtype).cuda(), bt.cuda(), mb,
                              torch.ones(len(qpos), dtype=torch.int32).cuda(), torch.tensor(qpos, dtype=torch.int32).cuda(), out2,
                              nq, nkv, hd, page, 0, scale, chunk=chunk, sinks=None, value_dim=hdv)
    assert float((out2.float() - out.float()).abs().max()) > 0.05


@pytest.mark.parametrize("impl", ["tc", "mma"])
@pytest.mark.parametrize("chunk,page,hd,nq,nkv,offset,qlen", [(24, 16, 32, 4, 2, 0, 150), (64, 16, 64, 8, 2, 37, 300), (128, 32, 128, 2, 1, 200, 129),
                                                              (100, 16, 48, 3, 3, 99, 2), (16, 16, 64, 2, 2, 15, 131), (1000, 16, 128, 4, 2, 700, 520),
                                                              (300, 16, 64, 3, 1, 1, 400)])
def test_tiled_prefill_attention_sees_its_chunk_and_the_sink(chunk, page, hd, nq, nkv, offset, qlen, impl):
    """A portion of ``qlen`` queries that starts at position ``offset`` of its request, through the
    tensor-core kernels (tcgen05 where the head size allows, else and on request mma.sync): the keys at every chunk's two edges stand out, so a warp that skips a block
    it needs, or a row that sees across its chunk's edge, shows."""
    from aien_sovereign_core_mv_b200 import kernels as K
    g = torch.Generator().manual_seed(chunk * 3 + hd)
    n = offset + qlen
    keys = torch.randn(n, nkv, hd, generator=g)
    vals = torch.randn(n, nkv, hd, generator=g)
    for p in range(0, n, chunk):
        keys[p] *= 3.0
        if p > 0:
            keys[p - 1] *= 3.0
    qpos = list(range(offset, n))
    q = torch.randn(qlen, nq, hd, generator=g).to(torch.bfloat16)
    keys, vals = keys.to(torch.bfloat16), vals.to(torch.bfloat16)
    sinks = torch.tensor([(-1.0) ** h * (0.5 + 1.5 * h) for h in range(nq)])
    scale = 0.5 / math.sqrt(hd)
    order = list(reversed(range((n + page - 1) // page + 1)))
    kc, vc, row = _paged(keys, vals, page, order)
    mb = len(row) + 2
    bt = torch.full((2, mb), -1, dtype=torch.int32)
    bt[1, :len(row)] = torch.tensor(row, dtype=torch.int32)
    i32 = lambda a: torch.tensor(a, dtype=torch.int32).cuda()
    tiles = list(range(0, qlen, 128))
    out = torch.zeros(3 + qlen, nq * hd, dtype=torch.bfloat16).cuda()          # three tokens of another request come first
    qfull = torch.zeros(3 + qlen, nq * hd, dtype=torch.bfloat16)
    qfull[3:] = q.reshape(qlen, -1)
    K.paged_attention_prefill(qfull.cuda(), kc.cuda(), vc.cuda(), bt.cuda(), mb, i32([0, 3, 3 + qlen]), i32([3, n]), i32([1] * len(tiles)),
                              i32(tiles), len(tiles), out, nq, nkv, hd, page, 0, scale, chunk=chunk, sinks=sinks.cuda(), impl=impl)
    want = pd.chunk_sink_attention(q.double().numpy(), keys.double().numpy(), vals.double().numpy(), qpos, list(range(n)), scale, chunk,
                                   sinks.double().numpy())
    H.assert_close(out[3:].float().cpu().numpy().reshape(qlen, nq, hd), want, 2e-2, "tiled attention")


@pytest.mark.parametrize("chunk,page,hd,nq,nkv", [(24, 16, 32, 4, 2), (64, 16, 64, 8, 2), (128, 32, 128, 2, 1), (100, 16, 48, 3, 3), (16, 16, 64, 2, 2),
                                                  (1000, 16, 128, 8, 2), (300, 16, 64, 16, 1), (129, 8, 16, 2, 1)])
def test_split_key_decode_attention_sees_its_chunk_and_the_sink(chunk, page, hd, nq, nkv):
    """Single tokens at the first, second and last position of a chunk, next to every edge, through the
    split-key kernel, whose blocks of 128 keys are counted from the block that holds the chunk's start."""
    from aien_sovereign_core_mv_b200 import kernels as K
    g = torch.Generator().manual_seed(chunk * 5 + hd)
    n = min(3 * chunk + 7, 2600)
    keys = torch.randn(n, nkv, hd, generator=g)
    vals = torch.randn(n, nkv, hd, generator=g)
    for p in range(0, n, chunk):
        keys[p] *= 3.0
        if p > 0:
            keys[p - 1] *= 3.0
    edges = sorted({p for c in range(0, n, chunk) for p in (c - 1, c, c + 1, c + chunk // 2) if 0 <= p < n} | {0, n - 1, 127, 128} & set(range(n)))
    T = len(edges)
    q = torch.randn(T, nq, hd, generator=g).to(torch.bfloat16)
    keys, vals = keys.to(torch.bfloat16), vals.to(torch.bfloat16)
    sinks = torch.tensor([(-1.0) ** h * (0.5 + 0.7 * h) for h in range(nq)])
    scale = 0.5 / math.sqrt(hd)
    order = list(reversed(range((n + page - 1) // page + 1)))
    kc, vc, row = _paged(keys, vals, page, order)
    mb = len(row) + 2
    bt = torch.full((2, mb), -1, dtype=torch.int32)
    bt[1, :len(row)] = torch.tensor(row, dtype=torch.int32)
    i32 = lambda a: torch.tensor(a, dtype=torch.int32).cuda()
    splits = K.decode_splits(n, chunk)
    part_out = torch.empty(T * nq * splits * hd, dtype=torch.float32).cuda()
    part_ml = torch.empty(T * nq * splits * 2, dtype=torch.float32).cuda()
    out = torch.zeros(T, nq * hd, dtype=torch.bfloat16).cuda()
    K.paged_attention_decode(q.reshape(T, -1).cuda(), kc.cuda(), vc.cuda(), bt.cuda(), mb, i32([1] * T), i32(edges), out, part_out, part_ml,
                             nq, nkv, hd, page, 0, scale, splits, impl="direct", chunk=chunk, sinks=sinks.cuda())
    want = pd.chunk_sink_attention(q.double().numpy(), keys.double().numpy(), vals.double().numpy(), edges, list(range(n)), scale, chunk,
                                   sinks.double().numpy())
    H.assert_close(out.float().cpu().numpy().reshape(T, nq, hd), want, 2e-2, "split-key attention")
    # a second launch finds the tickets at zero again and gives the same bits
    out2 = torch.zeros_like(out)
    K.paged_attention_decode(q.reshape(T, -1).cuda(), kc.cuda(), vc.cuda(), bt.cuda(), mb, i32([1] * T), i32(edges), out2, part_out, part_ml,
                             nq, nkv, hd, page, 0, scale, splits, impl="direct", chunk=chunk, sinks=sinks.cuda())
    assert torch.equal(out, out2)


@pytest.mark.parametrize("E,count,keep,top", [(8, 4, 2, 3), (12, 3, 2, 2), (4, 1, 1, 1), (6, 6, 2, 2), (64, 8, 3, 6), (5, 1, 1, 5)])
def test_router_choice(E, count, keep, top):
    from aien_sovereign_core_mv_b200 import kernels as K
    g = torch.Generator().manual_seed(E * 7 + top)
    T = 33
    z = (torch.randn(T, E, generator=g) * 2.0).cuda()
    ids = torch.empty(T, top, dtype=torch.int32).cuda()
    wts = torch.empty(T, top, dtype=torch.float32).cuda()
    K.moe_route(z, count, keep, top, False, ids, wts)
    for t in range(T):
        chosen, weights = pd.route(z[t].double().cpu().numpy(), top, count, keep)
        assert ids[t].tolist() == chosen, (t, ids[t].tolist(), chosen)
        H.assert_close(wts[t].cpu().numpy(), np.array(weights), 1e-5, "router weights")
        if keep < count:                                              # the best expert overall is always eligible; the rest share few groups
            assert len({e // (E // count) for e in ids[t].tolist()}) <= keep


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T", [3, 70, 400])
@pytest.mark.parametrize("shared,D,F,E,top", [(0, 96, 40, 8, 3), (56, 96, 40, 8, 3), (64, 256, 256, 8, 3), (0, 128, 72, 16, 2)])
def test_routed_feed_forward_part(dtype, T, shared, D, F, E, top):
    """Sizes that take the plain products, the products that stream a few tokens' experts (width and
    hidden size multiples of 256, few tokens) and the grouped tensor-core products (many tokens)."""
    from aien_sovereign_core_mv_b200.registry import make_part
    ff = make_part("feed_forward", "routed_experts", hidden_size=D, expert_ff=F, num_experts=E, top=top, group_count=4, group_keep=2,
                   shared_ff=shared)
    g = torch.Generator().manual_seed(T + shared)
    ws = {n: (torch.randn(s, generator=g) / math.sqrt(s[1])).to(torch.bfloat16) for n, (s, _) in ff.param_shapes().items()}
    ws["router"] = (ws["router"].float() * 6.0).to(torch.bfloat16)       # decided choices
    ff.bind({n: (t.cuda() if dtype == torch.bfloat16 else t.float().cuda()) for n, t in ws.items()})
    h = torch.randn(T, D, generator=g).to(dtype).cuda()
    ctx = make_ctx(dtype, list(range(T)), [0] * T, [0, T], [T])
    parts, sh = ff.forward(ctx, h)
    got = parts.double().sum(0)
    if sh is not None:
        got = got + (sh.double().sum(0) if sh.dim() == 3 else sh.double())
    W = {"router": ws["router"].double().numpy()}
    for e in range(E):
        W[f"e{e}.up"], W[f"e{e}.down"] = ws[f"experts.{e}.up"].double().numpy(), ws[f"experts.{e}.down"].double().numpy()
    mlp = {"router": {"experts": E, "top": top, "groups": {"count": 4, "keep": 2}}, "expert": {"ff": F}, "shared": None}
    if shared:
        W["shared.up"], W["shared.down"] = ws["shared.up"].double().numpy(), ws["shared.down"].double().numpy()
        mlp["shared"] = {"ff": shared}
    want = pd.moe_ff(h.double().cpu().numpy(), W, mlp)
    H.assert_close(got.cpu().numpy(), want, 2e-5 if dtype == torch.float32 else 2e-2, "routed feed-forward")


@pytest.mark.parametrize("M,N,K", [(3, 192, 256), (12, 1536, 512), (70, 200, 128), (600, 1536, 2048), (2048, 1536, 2048), (2048, 768, 1024)])
@pytest.mark.parametrize("act", [0, 1])
def test_products_with_the_activation_in_their_epilogue(M, N, K, act):
    """The streamed decode product (few rows) and every form of the tensor-core product (tiles, persistent,
    256-row tiles) with the gelu of both forms in the epilogue, against a float64 product and activation."""
    from aien_sovereign_core_mv_b200.parts.linear import linear
    g = torch.Generator().manual_seed(M + N)
    a = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).to(torch.bfloat16)
    ctx = make_ctx(torch.bfloat16, list(range(M)), [0] * M, [0, M], [M])
    y = linear(ctx, a.cuda(), w.cuda(), act=act)
    z = a.double().numpy() @ w.double().numpy().T
    want = pd.gelu_erf(z) if act == 0 else pd.gelu_tanh(z)
    H.assert_close(y.float().cpu().numpy(), want, 8e-3, "product with activation")


# ------------------------------------------------------------------ whole models
@pytest.mark.parametrize("dtype,tol", DTYPES)
@pytest.mark.parametrize("which", list(CONFIGS))
def test_whole_requests(models, which, dtype, tol):
    d, reqs, want = models[which]
    eng = H.engine_for(d, dtype, PAGE[which], 512)
    steps = [([(rid, toks, list(range(len(toks))))], [rid]) for rid, toks in reqs.items()]
    check(H.run_steps(eng, steps), want, tol, f"{which} {dtype} whole")
    assert eng.cache_state()["check"] == "" and eng.cache_state()["requests"] == 0


@pytest.mark.parametrize("dtype,tol", DTYPES)
@pytest.mark.parametrize("which", list(CONFIGS))
def test_prefill_then_token_by_token(models, which, dtype, tol):
    """Most of the longest request in one step, then 40 tokens one by one: the decoded tokens pass
    over chunk edges, and pages before a chunk are given back while the request runs."""
    d, reqs, want = models[which]
    eng = H.engine_for(d, dtype, PAGE[which], 512)
    rid = max(reqs, key=lambda r: len(reqs[r]))
    toks = reqs[rid]
    cut = len(toks) - 40
    steps = [([(rid, toks[:cut], [0, cut - 1])], [])] + [([(rid, [toks[i]], [0])], []) for i in range(cut, len(toks))]
    check(H.run_steps(eng, steps), want, tol, f"{which} {dtype} decode")
    state = eng.cache_state()
    assert state["check"] == "" and (which == "U" or state["metrics"]["window_releases"] > 0)     # pages of earlier chunks went back


@pytest.mark.parametrize("dtype,tol", DTYPES)
@pytest.mark.parametrize("which", list(CONFIGS))
def test_first_tokens_one_by_one(models, which, dtype, tol):
    d, reqs, want = models[which]
    eng = H.engine_for(d, dtype, PAGE[which], 512)
    rid = max(reqs, key=lambda r: len(reqs[r]))
    toks = reqs[rid][:45]
    steps = [([(rid, [t], [0])], []) for t in toks]
    check(H.run_steps(eng, steps), want, tol, f"{which} {dtype} from the first token")


@pytest.mark.parametrize("dtype,tol", DTYPES)
@pytest.mark.parametrize("which", list(CONFIGS))
def test_changing_portions(models, which, dtype, tol):
    d, reqs, want = models[which]
    eng = H.engine_for(d, dtype, PAGE[which], 512)
    sizes = [7, 2, 13, 3, 2, 29, 5, 2, 16, 17, 1, 8, 64, 2, 31]
    for rid, toks in reqs.items():
        steps, at, k = [], 0, rid
        while at < len(toks):
            n = min(sizes[k % len(sizes)], len(toks) - at)
            steps.append(([(rid, toks[at:at + n], list(range(n)))], []))
            at += n
            k += 1
        steps[-1] = (steps[-1][0], [rid])
        check(H.run_steps(eng, steps), want, tol, f"{which} {dtype} portions of request {rid}")
    assert eng.cache_state()["check"] == "" and eng.cache_state()["requests"] == 0


@pytest.mark.parametrize("dtype,tol", DTYPES)
@pytest.mark.parametrize("which", list(CONFIGS))
def test_mixed_batches_on_few_pages(models, which, dtype, tol):
    """Unequal requests side by side, portions beside single tokens, in a pool so small that pages
    and request rows are used again; every logit equals the request's alone."""
    d, reqs, want = models[which]
    page = PAGE[which]
    longest = max(len(t) for t in reqs.values())
    pool = ((longest + page - 1) // page + 6) * page
    if which == "U":                                               # no mask: every key stays, so the three live requests must fit whole
        pool = (sum((len(t) + page - 1) // page + 1 for t in reqs.values()) + 2) * page
    eng = H.engine_for(d, dtype, page, pool, max_requests=3)
    rng = np.random.default_rng(5)
    at = {rid: 0 for rid in reqs}
    waiting, live, steps = sorted(reqs, key=lambda r: len(reqs[r])), [], []
    held = lambda: sum((at[r] + page - 1) // page + 1 for r in live)
    while waiting or live:
        while waiting and len(live) < 3 and (held() + (len(reqs[waiting[0]]) + page - 1) // page + 2) * page <= pool:
            live.append(waiting.pop(0))
        if not live:
            live.append(waiting.pop(0))
        entries, end = [], []
        for rid in list(live):
            left = len(reqs[rid]) - at[rid]
            n = 1 if rng.random() < 0.4 else int(min(left, rng.integers(2, 40)))
            n = min(n, left)
            entries.append((rid, reqs[rid][at[rid]:at[rid] + n], list(range(n))))
            at[rid] += n
            if at[rid] == len(reqs[rid]):
                end.append(rid)
                live.remove(rid)
        steps.append((entries, end))
    check(H.run_steps(eng, steps), want, tol, f"{which} {dtype} mixed")
    state = eng.cache_state()
    assert state["check"] == "" and state["requests"] == 0


def test_a_chunk_group_gives_pages_back_and_takes_them_again(models):
    """A request far longer than the pool runs, because only its current chunk is held; a second request
    then reuses the pages, and its logits are its own."""
    d, reqs, want = models["P"]                                     # chunks of 24 and 40 positions, pages of 16
    eng = H.engine_for(d, "float32", 16, 7 * 16, max_requests=2, max_batch_tokens=64)
    toks = reqs[4]                                                  # 131 tokens through a pool of 112
    steps, at = [], 0
    for n in [30, 2, 17, 1, 1, 40, 9, 31]:
        steps.append(([(4, toks[at:at + n], list(range(n)))], []))
        at += n
    assert at == len(toks)
    steps[-1] = (steps[-1][0], [4])
    steps.append(([(3, reqs[3], list(range(len(reqs[3]))))], [3]))
    check(H.run_steps(eng, steps), want, FP32_TOL, "P float32 through a pool smaller than the request")
    assert eng.cache_state()["check"] == "" and eng.cache_state()["metrics"]["window_releases"] >= 3


def test_long_decoding_bfloat16_graphs(models):
    """200 decode-only steps of two requests (captured graphs, several buckets of context): along
    the given tokens the logits stay with the plain implementation."""
    d, reqs, want = models["R"]
    eng = H.engine_for(d, "bfloat16", 32, 1024)
    a, b = reqs[3], reqs[2]
    steps = [([(3, a[:100], [99]), (2, b[:4], [3])], [])]
    for i in range(130):
        steps.append(([(3, [a[100 + i]], [0]), (2, [b[4 + i]], [0])], []))
    check(H.run_steps(eng, steps), want, BF16_TOL, "R bfloat16 long decoding")


def test_greedy_generation_through_the_entry_point(models):
    from aien_sovereign_core_mv_b200.engine.generate import generate
    from aien_sovereign_core_mv_b200.sampling import SamplingParams
    d, reqs, _ = models["P"]
    cfg, tensors = load_plain(d)
    prompts = [reqs[2], reqs[3][:30], reqs[1]]
    n_new = 10
    want = []
    for p in prompts:
        seq, out = list(p), []
        for _ in range(n_new):
            row = pd.forward(cfg, tensors, seq)[-1]
            t = int(np.argmax(row))
            seq.append(t); out.append(t)
        want.append(out)
    eng = H.engine_for(d, "float32", 16, 512, prefill_chunk_size=16, max_prefill_tokens=32)
    got = generate(eng, prompts, SamplingParams(temperature=0.0, max_tokens=n_new, stop_token_ids=[]))
    assert got == want
    assert eng.cache_state()["requests"] == 0 and eng.cache_state()["check"] == ""


def test_sampling_and_the_command_line(models):
    """Sampling through the scheduler (temperature, top-p, top-k) runs and repeats under the same seed; the
    command line generates the plain implementation's greedy tokens and describes the model."""
    import subprocess
    from aien_sovereign_core_mv_b200.engine.generate import Generator
    from aien_sovereign_core_mv_b200.sampling import SamplingParams
    d, reqs, _ = models["Q"]
    eng = H.engine_for(d, "bfloat16", 16, 512)
    params = SamplingParams(temperature=0.8, top_p=0.9, top_k=40, max_tokens=12, stop_token_ids=[], seed=7)
    a = Generator(eng).generate([reqs[2], reqs[1]], params, request_ids=[5, 6])
    b = Generator(eng).generate([reqs[2], reqs[1]], params, request_ids=[5, 6])
    assert [r.tokens for r in a] == [r.tokens for r in b] and all(len(r.tokens) == 12 for r in a)
    cfg, tensors = load_plain(d)
    seq, want = list(reqs[1]), []
    for _ in range(5):
        t = int(np.argmax(pd.forward(cfg, tensors, seq)[-1]))
        seq.append(t); want.append(t)
    exe = os.path.join(H.ROOT, "bin", "aien-b200")
    out = subprocess.run([exe, "generate", "--model-dir", d, "--dtype", "float32", "--prompt-ids", ",".join(map(str, reqs[1])),
                          "--max-tokens", "5", "--temperature", "0", "--stop-token-ids", "", "--json"], capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    assert json.loads(out.stdout.strip().splitlines()[-1])["tokens"] == [want]
    info = subprocess.run([exe, "info", "--model-dir", d], capture_output=True, text=True, timeout=600)
    assert info.returncode == 0, info.stderr[-2000:]
    rec = json.loads(info.stdout.strip().splitlines()[-1])
    assert rec["architecture"] == "Dulisun" and rec["layers"] == 2 and rec["cache_groups"] == ["chunk", "chunk"]


def test_trace_replay_from_the_command(models, tmp_path):
    d, reqs, want = models["Q"]
    toks = reqs[3]
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": toks[:50], "want": [0, 49]}, {"id": 7, "tokens": reqs[1], "want": [2]}], "end": [7]},
             {"step": 1, "entries": [{"id": "x", "tokens": toks[50:52], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "x", "tokens": toks[52:], "want": [len(toks) - 53]}], "end": ["x"]}]
    out = H.run_trace(d, "float32", str(tmp_path / "out"), 192, steps)
    assert sorted(out) == [0, 2]
    H.assert_close(out[0], np.stack([want[3][0], want[3][49], want[1][2]]), FP32_TOL, "trace step 0")
    H.assert_close(out[2], want[3][-1:], FP32_TOL, "trace step 2")


def test_config_errors_name_the_field():
    from aien_sovereign_core_mv_b200 import ConfigError, model_spec_for
    import copy
    bad = copy.deepcopy(CONFIGS["Q"]); bad["layers"][0]["type"] = "conv"
    with pytest.raises(ConfigError, match=r"layers\[0\]\.type"):
        model_spec_for(bad)
    bad = copy.deepcopy(CONFIGS["Q"]); del bad["layers"][1]["mixer"]["scale"]
    with pytest.raises(ConfigError, match=r"layers\[1\]\.mixer\.scale"):
        model_spec_for(bad)
    bad = copy.deepcopy(CONFIGS["Q"]); del bad["norm"]
    with pytest.raises(ConfigError, match="norm"):
        model_spec_for(bad)
