"""The mechanisms of the Nomudra design one at a time: each kernel against the plain function of the same mechanism
(float64 on the CPU), in packed batches of unequal requests, in portions down to one token, with pages in shuffled
places of a poisoned pool and state slots that are used again.  Where random numbers would hide a fault (a key just
outside a chunk, a far key among many, a masked group whose score is negative), the inputs are made so that it shows."""
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import plain_nomudra as pn

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]
F64 = torch.float64


@pytest.fixture(scope="module")
def ops():
    from nanohybrid_vlm_b200.kernels import ops
    return ops


def dev(t):
    return t.cuda()


def i32(x):
    return torch.tensor(x, dtype=torch.int32).cuda()


def step_batch(news, starts, slots):
    cu = [0, *np.cumsum(news).tolist()]
    return SimpleNamespace(cu_q=i32(cu), q_start=i32(starts), state_slots=i32(slots), n_seqs=len(news),
                           n_tokens=int(sum(news)), kv_len=i32([s + n for s, n in zip(starts, news)]),
                           n_prefill_tokens=sum(n for n in news if n > 1), n_prefill_seqs=sum(1 for n in news if n > 1),
                           n_decode_seqs=sum(1 for n in news if n == 1), max_kv_len=max(s + n for s, n in zip(starts, news)))


def portions_of(lengths, cuts):
    """Step i brings the i-th portion of every request that still has one: (requests, their starts, their sizes)."""
    bounds = [[0, *c, L] for L, c in zip(lengths, cuts)]
    for i in range(max(len(b) for b in bounds) - 1):
        who = [r for r, b in enumerate(bounds) if i + 1 < len(b)]
        yield who, [bounds[r][i] for r in who], [bounds[r][i + 1] - bounds[r][i] for r in who]


def tol(dtype, f32=2e-5, bf16=2e-2):
    return dict(rtol=f32, atol=f32) if dtype == torch.float32 else dict(rtol=bf16, atol=bf16)


# ---------------------------------------------------------------- Dynamic Tanh
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [96, 100, 1030])
def test_dyntanh_forms(ops, dtype, width):
    g = torch.Generator().manual_seed(width)
    T = 9

    def triple():
        return ((0.3 + torch.rand(1, generator=g)).to(dtype), (1 + 0.3 * torch.randn(width, generator=g)).to(dtype),
                (0.3 * torch.randn(width, generator=g)).to(dtype))

    pre, post = triple(), triple()
    f = lambda x, p: pn.dyntanh(x.to(F64), *(t.to(F64) for t in p))     # noqa: E731
    x = (2 * torch.randn(T, width, generator=g)).to(dtype)
    for x_in, out_dtype in ((x, dtype), (x, torch.float32), (x.float(), dtype), (x.float(), torch.float32)):
        out = torch.empty(T, width, dtype=out_dtype, device="cuda")
        ops.dyntanh(out, dev(x_in), *map(dev, pre))
        torch.testing.assert_close(out.cpu().to(F64), f(x_in, pre), **tol(out_dtype))
    # the embedding through the norm
    table = torch.randn(50, width, generator=g).to(dtype)
    ids = torch.randint(0, 50, (T,), generator=g, dtype=torch.int32)
    out = torch.empty(T, width, dtype=torch.float32, device="cuda")
    ops.embed_dyntanh(out, dev(table), dev(ids), *map(dev, pre))
    torch.testing.assert_close(out.cpu().to(F64), f(table[ids.long()], pre), **tol(torch.float32))
    # over the stream: nothing pending; a pending output with its own norm; gathered rows that write nothing back
    stream = 3 * torch.randn(T, width, generator=g)
    a = (2 * torch.randn(T, width, generator=g)).to(dtype)
    s_dev = dev(stream.clone())
    out = torch.empty(T, width, dtype=dtype, device="cuda")
    ops.dyntanh_stream(out, s_dev, tuple(map(dev, pre)))
    torch.testing.assert_close(out.cpu().to(F64), f(stream, pre), **tol(dtype))
    assert torch.equal(s_dev.cpu(), stream)
    ops.dyntanh_stream(out, s_dev, tuple(map(dev, pre)), dev(a), tuple(map(dev, post)))
    summed = stream.to(F64) + f(a, post)
    torch.testing.assert_close(s_dev.cpu().to(F64), summed, **tol(torch.float32))          # the stream stays 32-bit
    torch.testing.assert_close(out.cpu().to(F64), f(summed, pre), **tol(dtype))
    rows = torch.tensor([7, 0, 3], dtype=torch.int32)
    before = s_dev.clone()
    out = torch.empty(3, width, dtype=dtype, device="cuda")
    ops.dyntanh_stream(out, s_dev, tuple(map(dev, pre)), dev(a), tuple(map(dev, post)), rows=dev(rows), write_stream=False)
    torch.testing.assert_close(out.cpu().to(F64), f(summed + f(a, post), pre)[rows.long()], **tol(dtype))
    assert torch.equal(s_dev, before)


# ---------------------------------------------------------------- small gated steps
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n,skip", [(70, 3), (72, 8), (1032, 16)], ids=["one_column_a_thread", "eight", "eight_wide"])
def test_gates_bias_and_clamped_unit(ops, dtype, n, skip):
    g = torch.Generator().manual_seed(5)
    T = 6
    wide = (2 * torch.randn(T, 2 * n + skip, generator=g)).to(dtype)
    x = torch.randn(T, n, generator=g).to(dtype)
    out = torch.empty(T, n, dtype=dtype, device="cuda")
    ops.sigmoid_mul(out, dev(x), dev(wide)[:, skip:skip + n])
    want = x.to(F64) * torch.sigmoid(wide[:, skip:skip + n].to(F64))
    torch.testing.assert_close(out.cpu().to(F64), want, **tol(dtype))
    inplace = dev(x.clone())
    ops.sigmoid_mul(inplace, inplace, dev(wide)[:, skip:skip + n])               # the attention layer gates its heads in place
    torch.testing.assert_close(inplace.cpu().to(F64), want, **tol(dtype))
    b = torch.randn(n, generator=g).to(dtype)
    y = dev(x.clone())
    ops.add_row_bias(y, dev(b))
    torch.testing.assert_close(y.cpu().to(F64), x.to(F64) + b.to(F64), **tol(dtype))
    gu = (3 * torch.randn(T, 2 * n, generator=g)).to(dtype)          # well beyond the limit on both sides
    ops.clamped_glu(out, dev(gu), 1.5, 1.702)
    gg, uu = gu[:, :n].to(F64).clamp(max=1.5), gu[:, n:].to(F64).clamp(-1.5, 1.5)
    torch.testing.assert_close(out.cpu().to(F64), gg * torch.sigmoid(1.702 * gg) * (uu + 1), **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("groups,size", [(2, 48), (3, 40), (1, 300)])
def test_gated_rmsnorm_with_a_sigmoid_gate(ops, dtype, groups, size):
    g = torch.Generator().manual_seed(size)
    T, n = 5, groups * size
    y = 3 * torch.randn(T, n, generator=g)
    z = torch.randn(T, n + 7, generator=g).to(dtype)
    w = (1 + 0.2 * torch.randn(n, generator=g)).to(dtype)
    out = torch.empty(T, n, dtype=dtype, device="cuda")
    ops.gated_rmsnorm(out, dev(y), dev(z)[:, 7:], dev(w), groups, 1e-5, gate_first=False, gate="sigmoid")
    yy = y.to(F64).view(T, groups, size)
    yy = (yy / torch.sqrt((yy * yy).mean(-1, keepdim=True) + 1e-5)).reshape(T, n)
    torch.testing.assert_close(out.cpu().to(F64), yy * w.to(F64) * torch.sigmoid(z[:, 7:].to(F64)), **tol(dtype))


# ---------------------------------------------------------------- chunked attention whose values are its keys
def rotary_table(dims, base, n_pos):
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=F64)
    ang = torch.arange(n_pos, dtype=F64)[:, None] * f[None, :]
    return torch.cat((ang.cos(), ang.sin()), -1).float()


def plain_chunked(x, bias, nq, nkv, d, rot, base, chunk, scale):
    """x [T, (nq + nkv) d + extra]: projected q and k rows -> [T, nq d]."""
    T = x.shape[0]
    x = x.to(F64)[:, :(nq + nkv) * d] + bias.to(F64)
    q, k = x[:, :nq * d].view(T, nq, d), x[:, nq * d:].view(T, nkv, d)
    v = k
    if rot:
        q, k = pn.rotate_half(q, torch.arange(T), base, rot), pn.rotate_half(k, torch.arange(T), base, rot)
    vis = pn.chunk_mask(T, chunk)
    heads = []
    for h in range(nq):
        s = (q[:, h] @ k[:, h // (nq // nkv)].T * scale).masked_fill(~vis, -float("inf"))
        heads.append(torch.softmax(s, -1) @ v[:, h // (nq // nkv)])
    return torch.cat(heads, -1)


def run_chunked(ops, dtype, xs, bias, cuts, nq, nkv, d, page, rot, table, chunk, scale, simt, seed=0):
    """Requests' projected rows through bias + rotation + cache store and the attention kernel, in portions, with
    shuffled pages in a poisoned pool."""
    rng = np.random.default_rng(seed)
    lengths = [x.shape[0] for x in xs]
    n_pages = sum(-(-L // page) for L in lengths) + 3
    pages = torch.full((n_pages, 2, nkv, page, d), float("nan"), dtype=dtype, device="cuda")
    free = list(rng.permutation(n_pages))
    tables = [[int(free.pop()) for _ in range(-(-L // page))] for L in lengths]
    width = max(len(t) for t in tables)
    got = [torch.zeros(L, nq * d, dtype=dtype) for L in lengths]
    for who, starts, news in portions_of(lengths, cuts):
        x = torch.cat([xs[r][s:s + n] for r, s, n in zip(who, starts, news)])
        pos = [p for s, n in zip(starts, news) for p in range(s, s + n)]
        slots = [tables[r][p // page] * page + p % page for r, s, n in zip(who, starts, news) for p in range(s, s + n)]
        bt = torch.full((len(who), width), -1, dtype=torch.int32)
        for i, r in enumerate(who):
            bt[i, :len(tables[r])] = torch.tensor(tables[r], dtype=torch.int32)
        q = torch.full((x.shape[0], nq * d), float("nan"), dtype=dtype, device="cuda")
        ops.rope_norm_store(dev(x), q, pages, i32(slots), i32(pos), None if table is None else dev(table), rot, nq, nkv,
                            d, d, None, bias=dev(bias), values_from_keys=True)
        out = torch.full((x.shape[0], nq * d), float("nan"), dtype=dtype, device="cuda")
        b = step_batch(news, starts, [-1] * len(who))
        if simt:
            ops.attention_sink_simt(out, q, pages, dev(bt), b.cu_q, b.kv_len, len(who), x.shape[0], nq, nkv, d, d, scale,
                                    None, 0, chunk or 0)
        else:       # the dispatcher: the tensor-core kernels where the shape allows them
            ops.attention_sink(out, q, pages, SimpleNamespace(block_tables=dev(bt)), b, nq, nkv, d, d, scale, None, 0,
                               chunk or 0)
        at = 0
        for r, s, n in zip(who, starts, news):
            got[r][s:s + n] = out[at:at + n].cpu()
            at += n
    return got


def planted(g, L, nq, nkv, d, extra, chunk, dtype):
    """Random projected rows in which some queries would, but for the mask, give nearly all their weight to one key:
    the last key of the chunk before theirs (just outside), the first key of their own chunk (just inside, far back
    when the query ends its chunk), and their own position.  The spike sits in the last element of the head, which no
    rotation touches, so it shows whatever the positions."""
    x = 0.5 * torch.randn(L, (nq + nkv) * d + extra, generator=g)
    if chunk:
        for c0 in range(chunk, L, chunk):
            for kh in range(nkv):
                x[c0 - 1, nq * d + kh * d + d - 1] += 5.0         # the key just outside
                x[c0, nq * d + kh * d + d - 1] += 3.0             # the first key inside
            for i in {c0, min(c0 + 1, L - 1), min(c0 + chunk - 1, L - 1)}:
                for h in range(nq):
                    x[i, h * d + d - 1] += 4.0
    return x.to(dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("simt", [True, False], ids=["cuda_cores", "dispatcher"])
@pytest.mark.parametrize("nq,nkv,d,rot,page,chunk", [
    (4, 2, 32, 16, 8, 24), (2, 1, 64, 64, 64, 7), (6, 6, 16, 8, 5, 33), (3, 1, 48, 0, 16, None), (4, 4, 128, 32, 64, 96),
    (3, 1, 20, 10, 3, 50), (8, 2, 64, 32, 16, 64)])
def test_chunked_attention_in_portions_against_plain(ops, dtype, simt, nq, nkv, d, rot, page, chunk):
    """Portions that start and end in the middle of chunks and pages, single tokens at a chunk's first and last
    position, a request of two tokens; in bfloat16 the dispatcher takes the tensor-core kernels (mma.sync for pages of
    any size, tcgen05 and the TMA decode kernel for pages of 64 keys and heads in steps of 64)."""
    g = torch.Generator().manual_seed(nq * 10 + d)
    c = chunk or 40
    lengths = [3 * c + 5, c + 1, 2, 2 * c]
    cuts = [[c - 1, c, c + 1, 2 * c - 2, 2 * c - 1, 2 * c, 3 * c + 4], [c], [1], [3, 5, c - 1, 2 * c - 1]]
    xs = [planted(g, L, nq, nkv, d, 5, chunk, dtype) for L in lengths]
    bias = (0.5 * torch.randn((nq + nkv) * d, generator=g)).to(dtype)
    table = rotary_table(rot, 10000.0, 4 * c + 8) if rot else None
    got = run_chunked(ops, dtype, xs, bias, cuts, nq, nkv, d, page, rot, table, chunk, 0.3, simt)
    for r, x in enumerate(xs):
        want = plain_chunked(x, bias, nq, nkv, d, rot, 10000.0, chunk, 0.3)
        # bfloat16: a planted score of 6 carries the rounding of its query and key (2^-8 each), so a weight is off by
        # up to a few percent; a key that is wrongly seen or missed moves the outputs by whole units
        torch.testing.assert_close(got[r].to(F64), want, **(tol(dtype) if dtype == torch.float32 else dict(rtol=5e-2, atol=8e-2)))


# ---------------------------------------------------------------- mLSTM
def mlstm_inputs(g, T, H, d, dv, dtype, spread):
    proj = torch.randn(T, 2 * H * d + H * dv + 3, generator=g).to(dtype)         # three columns that are not read
    gates = spread * torch.randn(T, 2 * H, generator=g)
    return proj, gates


def plain_scan(proj, gates, bias, cap, H, d, dv):
    T = proj.shape[0]
    x = proj.to(F64)
    q = x[:, :H * d].view(T, H, d) * d ** -0.5
    k = x[:, H * d:2 * H * d].view(T, H, d)
    v = x[:, 2 * H * d:2 * H * d + H * dv].view(T, H, dv)
    raw = gates.to(F64) + bias.to(F64)
    i = cap * torch.tanh(raw[:, :H] / cap)
    f = torch.nn.functional.logsigmoid(cap * torch.tanh(raw[:, H:] / cap))
    return pn.mlstm_recurrence(q, k, v, i, f).reshape(T, H * dv)


@pytest.fixture(params=[0, 8, 16], ids=lambda p: f"lanes{p}")
def lanes(request, ops):
    """Both forms of the scan: a column of the memory in 8 or in 16 lanes (0: the kernel's choice)."""
    ops.MLSTM_LANES = request.param
    yield request.param
    ops.MLSTM_LANES = 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,d,dv,cap,spread", [(2, 24, 40, 15.0, 6.0), (1, 100, 16, 4.0, 8.0), (3, 16, 130, 10.0, 1.0),
                                               (1, 256, 8, 15.0, 3.0), (2, 7, 5, 2.0, 3.0), (2, 128, 128, 15.0, 4.0),
                                               (1, 64, 24, 15.0, 4.0), (1, 512, 16, 15.0, 2.0)])
def test_mlstm_scan_over_portions_and_reused_slots(ops, lanes, dtype, H, d, dv, cap, spread):
    """Three requests cut into portions of 1, 2 and more tokens, their states in slots 1, 3, 0 of a poisoned pool; gates
    spread so wide that the cap and the running maximum matter (input gates far above and below the forget gates);
    then a new request in a used slot, which must start from zeros and a maximum of 0."""
    g = torch.Generator().manual_seed(H * 1000 + d)
    lengths, cuts, slots = [41, 19, 6], [[2, 3, 20, 37], [18], [1, 2, 3, 4, 5]], [1, 3, 0]
    ins = [mlstm_inputs(g, L, H, d, dv, dtype, spread) for L in lengths]
    bias = torch.cat((torch.randn(H, generator=g), 2 + torch.randn(H, generator=g)))
    want = [plain_scan(p, gt, bias, cap, H, d, dv) for p, gt in ins]
    state = torch.full((4, ops.mlstm_state_floats(H, d, dv) + 3), float("nan"), dtype=torch.float32, device="cuda")
    got = [torch.zeros(L, H * dv) for L in lengths]
    for who, starts, news in portions_of(lengths, cuts):
        proj = torch.cat([ins[r][0][s:s + n] for r, s, n in zip(who, starts, news)])
        gates = torch.cat([ins[r][1][s:s + n] for r, s, n in zip(who, starts, news)])
        o = torch.full((proj.shape[0], H * dv), float("nan"), dtype=torch.float32, device="cuda")
        ops.mlstm_scan(o, dev(proj), dev(gates), dev(bias), cap, state, step_batch(news, starts, [slots[r] for r in who]),
                       H, d, dv)
        at = 0
        for r, s, n in zip(who, starts, news):
            got[r][s:s + n] = o[at:at + n].cpu()
            at += n
    for r in range(3):
        torch.testing.assert_close(got[r].to(F64), want[r], rtol=2e-4, atol=2e-5)
    proj, gates = mlstm_inputs(g, 5, H, d, dv, dtype, spread)
    o = torch.full((5, H * dv), float("nan"), dtype=torch.float32, device="cuda")
    ops.mlstm_scan(o, dev(proj), dev(gates), dev(bias), cap, state, step_batch([5], [0], [3]), H, d, dv)
    torch.testing.assert_close(o.cpu().to(F64), plain_scan(proj, gates, bias, cap, H, d, dv), rtol=2e-4, atol=2e-5)
    # a request without a slot is skipped and its outputs are cleared
    ops.mlstm_scan(o, dev(proj), dev(gates), dev(bias), cap, state, step_batch([5], [0], [-1]), H, d, dv)
    assert (o == 0).all()


# ---------------------------------------------------------------- the router
@pytest.mark.parametrize("N,count,keep,top,identity", [(10, 2, 1, 3, 2), (64, 8, 4, 8, 0), (12, 1, 1, 4, 3), (7, 7, 3, 3, 1),
                                                       (5, 1, 1, 5, 0), (130, 13, 2, 6, 2), (4, 2, 2, 1, 1)])
def test_router_against_plain(ops, N, count, keep, top, identity):
    """Logits spaced so that no choice is a close call, and a correction that pushes every choice score below zero: a
    masked group counted as 0 instead of minus infinity would win every time."""
    g = torch.Generator().manual_seed(N)
    T, W = 37, 24
    h = torch.randn(T, W, generator=g).to(F64)
    router_w = (torch.randn(N, W, generator=g) * 0.8).to(F64)
    correction = (-1.0 - 0.3 * torch.rand(N, generator=g)).float()
    r = dict(experts=N - identity, identity=identity, top=top, groups=dict(count=count, keep=keep))
    ids_want, w_want, _ = pn.route(h, router_w, correction.to(F64), r)
    logits = torch.full((T, N + 2), float("nan"))
    logits[:, :N] = (h @ router_w.T).float()
    ids = torch.empty(T, top, dtype=torch.int32, device="cuda")
    weights = torch.empty(T, top, dtype=torch.float32, device="cuda")
    ops.moe_route(ids, weights, dev(logits)[:, :N], dev(correction), N, count, keep)
    ids, weights = ids.cpu().long(), weights.cpu().to(F64)
    for t in range(T):
        want = dict(zip(ids_want[t].tolist(), w_want[t].tolist()))
        assert sorted(ids[t].tolist()) == sorted(want), f"token {t}: chose {ids[t].tolist()}, the plain router {sorted(want)}"
        for e, wt in zip(ids[t].tolist(), weights[t].tolist()):
            assert abs(wt - want[e]) < 1e-5
    torch.testing.assert_close(weights.sum(-1), torch.ones(T, dtype=F64), rtol=1e-5, atol=1e-5)


# ---------------------------------------------------------------- the experts and their sum
def plain_moe_sum(x, gate, up, down, ids, weights, limit, shared, sg):
    E = gate.shape[0]
    out = torch.zeros_like(x)
    for t in range(x.shape[0]):
        for e, wt in zip(ids[t].tolist(), weights[t]):
            out[t] += wt * (x[t] if e >= E else pn.clamped_unit(x[t:t + 1], gate[e], up[e], down[e], limit)[0])
    if shared is not None:
        out = out + shared * torch.sigmoid(sg)[:, None]
    return out


@pytest.mark.parametrize("path", ["float32", "bfloat16_cuda_cores", "bfloat16_tile16", "bfloat16_tile64", "bfloat16_tile128",
                                  "bfloat16_tcgen05", "bfloat16_auto"])
@pytest.mark.parametrize("T,E,I0,top,W,ff", [(1, 8, 2, 3, 64, 48), (5, 4, 0, 2, 128, 40), (300, 6, 2, 3, 96, 72),
                                            (70, 16, 1, 4, 200, 136), (9, 3, 1, 2, 100, 36)])
def test_experts_and_their_sum(ops, path, T, E, I0, top, W, ff):
    """Every path of the experts' products (CUDA cores in both types; mma.sync with tiles of 16, 64 and 128 rows; tcgen05) with
    identity choices, an expert that no token chooses, and the gated shared term.  The tokens' choices are drawn, not
    routed: each token gets `top` different outputs."""
    dtype = torch.float32 if path == "float32" else torch.bfloat16
    if path.startswith(("bfloat16_tile", "bfloat16_tcgen05")) and (W % 8 or ff % 8):
        pytest.skip("the tensor-core products take sizes in steps of 8")
    g = torch.Generator().manual_seed(T * 7 + E)
    x = torch.randn(T, W, generator=g).to(dtype)
    gate = (torch.randn(E, ff, W, generator=g) * 2.5 / W ** 0.5).to(dtype)
    up = (torch.randn(E, ff, W, generator=g) * 2.5 / W ** 0.5).to(dtype)
    down = (torch.randn(E, W, ff, generator=g) / ff ** 0.5).to(dtype)
    N = E + I0
    ids = torch.stack([torch.randperm(N - 1, generator=g)[:top] + 1 for _ in range(T)]).int()      # expert 0 is never chosen
    if N - 1 < top:
        ids = torch.stack([torch.randperm(N, generator=g)[:top] for _ in range(T)]).int()
    weights = torch.rand(T, top, generator=g)
    weights = weights / weights.sum(-1, keepdim=True)
    shared = torch.randn(T, W, generator=g).to(dtype)
    sg = torch.full((T, 3), float("nan"))
    sg[:, 1] = torch.randn(T, generator=g)
    ops.MOE_ON_TENSOR_CORES = path != "bfloat16_cuda_cores"
    ops.MOE_TILE = {"bfloat16_tile16": 16, "bfloat16_tile64": 64, "bfloat16_tile128": 128}.get(path, 0)
    ops.MOE_TCGEN05 = True if path == "bfloat16_tcgen05" else None
    try:
        y, slot_pos = ops.moe_experts(dev(x), dev(gate), dev(up), dev(down), dev(ids), 1.5, 1.702)
        ops.raise_wait_errors()
    finally:
        ops.MOE_ON_TENSOR_CORES, ops.MOE_TILE, ops.MOE_TCGEN05 = True, 0, None
    out = torch.full((T, W), float("nan"), dtype=dtype, device="cuda")
    ops.moe_combine(out, y, dev(x), dev(ids), dev(weights), slot_pos, E, dev(shared), dev(sg)[:, 1])
    want = plain_moe_sum(x.to(F64), gate.to(F64), up.to(F64), down.to(F64), ids, weights.to(F64), 1.5, shared.to(F64),
                         sg[:, 1].to(F64))
    torch.testing.assert_close(out.cpu().to(F64), want, **tol(dtype, f32=5e-5, bf16=4e-2))
    # without a shared term, and with one that has no gate
    ops.moe_combine(out, y, dev(x), dev(ids), dev(weights), slot_pos, E)
    want = plain_moe_sum(x.to(F64), gate.to(F64), up.to(F64), down.to(F64), ids, weights.to(F64), 1.5, None, None)
    torch.testing.assert_close(out.cpu().to(F64), want, **tol(dtype, f32=5e-5, bf16=4e-2))


def test_experts_tensor_core_paths_equal_the_cuda_cores(ops):
    """In bfloat16 the tensor-core products round where the CUDA-core products round, so every tile and the tcgen05
    products give nearly the same numbers as the CUDA cores (sums in another order), far closer than bfloat16 is to float64."""
    g = torch.Generator().manual_seed(1)
    T, E, top, W, ff = 150, 5, 2, 128, 96
    x = torch.randn(T, W, generator=g).bfloat16()
    gate, up = (torch.randn(2, E, ff, W, generator=g) * 0.2).bfloat16()
    down = (torch.randn(E, W, ff, generator=g) * 0.1).bfloat16()
    ids = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(T)]).int()
    outs = []
    for on, tile, tc in ((False, 0, False), (True, 16, False), (True, 64, False), (True, 128, False), (True, 0, True)):
        ops.MOE_ON_TENSOR_CORES, ops.MOE_TILE, ops.MOE_TCGEN05 = on, tile, tc
        try:
            y, pos = ops.moe_experts(dev(x), dev(gate), dev(up), dev(down), dev(ids), 1.5, 1.702)
        finally:
            ops.MOE_ON_TENSOR_CORES, ops.MOE_TILE, ops.MOE_TCGEN05 = True, 0, None
        outs.append(y[pos.long()].float().cpu())
    for other in outs[1:]:
        torch.testing.assert_close(other, outs[0], rtol=1e-2, atol=2e-3)
