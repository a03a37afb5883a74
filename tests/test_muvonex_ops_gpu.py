"""The mechanisms of the Muvonex design one at a time: each kernel against the plain function of the same
mechanism (float64 on the CPU), in packed batches of unequal requests, with per-request state that is carried
over portions and slots that are used again.  Sizes are odd on purpose: heads whose sizes are no multiple of 32,
groups of several heads, one tap, many taps."""
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import plain_muvonex as pm

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
    """The facts of one packed step that the recurrent kernels read."""
    cu = [0, *np.cumsum(news).tolist()]
    return SimpleNamespace(cu_q=i32(cu), q_start=i32(starts), state_slots=i32(slots), n_seqs=len(news),
                           n_tokens=int(sum(news)), kv_len=i32([s + n for s, n in zip(starts, news)]),
                           n_prefill_tokens=sum(n for n in news if n > 1), n_prefill_seqs=sum(1 for n in news if n > 1),
                           n_decode_seqs=sum(1 for n in news if n == 1), max_kv_len=max(s + n for s, n in zip(starts, news)))


def portions_of(lengths, cuts):
    """Steps over several requests: request r is cut at ``cuts[r]``; step i brings the i-th portion of every request
    that still has one.  Yields (requests in the step, their starts, their portion sizes)."""
    bounds = [[0, *c, L] for L, c in zip(lengths, cuts)]
    for i in range(max(len(b) for b in bounds) - 1):
        who = [r for r, b in enumerate(bounds) if i + 1 < len(b)]
        yield who, [bounds[r][i] for r in who], [bounds[r][i + 1] - bounds[r][i] for r in who]


def tol(dtype, f32=2e-5, bf16=2e-2):
    return dict(rtol=f32, atol=f32) if dtype == torch.float32 else dict(rtol=bf16, atol=bf16)


# ---------------------------------------------------------------- short convolution
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("C,K,bias", [(70, 4, True), (33, 1, False), (200, 2, False), (129, 7, True), (64, 8, True)])
def test_short_conv_over_portions_and_reused_slots(ops, dtype, C, K, bias):
    """Three requests cut into portions of 1, 2 and more tokens (shorter than the filter too), their states in
    slots 2, 0, 1 of a poisoned pool; then a new request in a used slot, which must start from zeros."""
    g = torch.Generator().manual_seed(C + K)
    lengths, cuts, slots = [23, 9, 14], [[2, 3, 10, 11], [1], [5, 7, 9, 11, 13]], [2, 0, 1]
    w = (torch.randn(C, K, generator=g) * 0.5).to(dtype)
    b = (torch.randn(C, generator=g) * 0.3).to(dtype) if bias else None
    xs = [torch.randn(L, C, generator=g).to(dtype) for L in lengths]
    want = [pm.silu(pm.short_conv(x.to(F64), w.to(F64), None if b is None else b.to(F64))) for x in xs]
    state = torch.full((4, max(K - 1, 1) * C), float("nan"), dtype=torch.float32, device="cuda")
    got = [torch.zeros(L, C, dtype=dtype) for L in lengths]
    for who, starts, news in portions_of(lengths, cuts):
        x = torch.cat([xs[r][s:s + n] for r, s, n in zip(who, starts, news)])
        wide = torch.full((x.shape[0], C + 5), float("nan"), dtype=dtype, device="cuda")     # a view with a row stride
        wide[:, 3:3 + C] = dev(x)
        out = torch.empty(x.shape[0], C, dtype=dtype, device="cuda")
        ops.short_conv_silu(out, wide[:, 3:3 + C], dev(w), None if b is None else dev(b), state,
                            step_batch(news, starts, [slots[r] for r in who]))
        at = 0
        for r, s, n in zip(who, starts, news):
            got[r][s:s + n] = out[at:at + n].cpu()
            at += n
    for r in range(3):
        torch.testing.assert_close(got[r].to(F64), want[r], **tol(dtype))
    # slot 2 held request 0's last inputs: a new request there must not see them
    # (its output in float32, as the recurrent mixers ask for it: nothing is rounded to the inputs' type)
    x = torch.randn(3, C, generator=g).to(dtype)
    out = torch.empty(3, C, dtype=torch.float32, device="cuda")
    ops.short_conv_silu(out, dev(x), dev(w), None if b is None else dev(b), state, step_batch([3], [0], [2]))
    torch.testing.assert_close(out.cpu().to(F64), pm.silu(pm.short_conv(x.to(F64), w.to(F64), None if b is None else b.to(F64))),
                               **tol(torch.float32))


# ---------------------------------------------------------------- gated delta rule
def delta_inputs(g, T, G, H, d, dv, dtype):
    qkv = torch.randn(T, 2 * G * d + H * dv, generator=g).to(dtype)
    ba = torch.randn(T, 2 * H, generator=g)
    a_log = torch.rand(H, generator=g) * 1.5 - 1.0
    dt_bias = torch.randn(H, generator=g) * 0.3
    return qkv, ba, a_log, dt_bias


def plain_delta(qkv, ba, a_log, dt_bias, G, H, d, dv):
    T = qkv.shape[0]
    x = qkv.to(F64)
    q, k, v = x[:, :G * d].view(T, G, d), x[:, G * d:2 * G * d].view(T, G, d), x[:, 2 * G * d:].view(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(ba[:, :H].to(F64))
    decay = torch.exp(-torch.exp(a_log.to(F64)) * pm.softplus(ba[:, H:].to(F64) + dt_bias.to(F64)))
    return pm.delta_recurrence(q, k, v, beta, decay).reshape(T, H * dv)


@pytest.fixture(params=[(0, -1, 0), (4, 0, 1), (8, 0, 1), (16, 0, 1), (32, 0, 1), (0, 1, 1), (0, 0, 2), (0, 0, 4)],
                ids=lambda p: f"lanes{p[0]}_group{p[1]}_columns{p[2]}")
def lanes(request, ops):
    """Every form of the scans: a state column over 4 to 32 lanes (0: the kernel's choice), the delta rule one token
    or four tokens per round of its chain (-1: the kernel's choice), one, two or four columns per lane."""
    ops.SCAN_LANES, ops.SCAN_GROUP4, ops.SCAN_COLUMNS = request.param
    yield request.param
    ops.SCAN_LANES, ops.SCAN_GROUP4, ops.SCAN_COLUMNS = 0, -1, 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("G,H,d,dv", [(2, 4, 24, 40), (3, 3, 48, 16), (1, 5, 100, 72), (2, 2, 16, 130), (1, 1, 256, 8),
                                      (2, 2, 30, 18), (1, 2, 128, 128), (1, 3, 7, 5)])
def test_delta_rule_over_portions_and_reused_slots(ops, lanes, dtype, G, H, d, dv):
    g = torch.Generator().manual_seed(G * 1000 + d)
    lengths, cuts, slots = [41, 19, 6], [[2, 3, 20, 37], [18], [1, 2, 3, 4, 5]], [1, 3, 0]
    ins = [delta_inputs(g, L, G, H, d, dv, dtype) for L in lengths]
    a_log, dt_bias = ins[0][2], ins[0][3]
    want = [plain_delta(qkv, ba, a_log, dt_bias, G, H, d, dv) for qkv, ba, _, _ in ins]
    state = torch.full((4, H * dv * d + 3), float("nan"), dtype=torch.float32, device="cuda")
    got = [torch.zeros(L, H * dv) for L in lengths]
    for who, starts, news in portions_of(lengths, cuts):
        qkv = torch.cat([ins[r][0][s:s + n] for r, s, n in zip(who, starts, news)])
        ba = torch.cat([ins[r][1][s:s + n] for r, s, n in zip(who, starts, news)])
        o = torch.full((qkv.shape[0], H * dv), float("nan"), dtype=torch.float32, device="cuda")
        ops.delta_rule(o, dev(qkv), dev(ba), dev(a_log), dev(dt_bias), state,
                       step_batch(news, starts, [slots[r] for r in who]), G, H, d, dv)
        at = 0
        for r, s, n in zip(who, starts, news):
            got[r][s:s + n] = o[at:at + n].cpu()
            at += n
    for r in range(3):
        torch.testing.assert_close(got[r].to(F64), want[r], **tol(torch.float32, f32=3e-5))
    # a new request in a slot that was used starts from zeros; a request without a slot writes zeros and no state
    qkv, ba, _, _ = delta_inputs(g, 4, G, H, d, dv, dtype)
    before = state.clone()
    o = torch.full((8, H * dv), float("nan"), dtype=torch.float32, device="cuda")
    ops.delta_rule(o, dev(torch.cat([qkv, qkv])), dev(torch.cat([ba, ba])), dev(a_log), dev(dt_bias), state,
                   step_batch([4, 4], [0, 7], [1, -1]), G, H, d, dv)
    torch.testing.assert_close(o[:4].cpu().to(F64), plain_delta(qkv, ba, a_log, dt_bias, G, H, d, dv), **tol(torch.float32, f32=3e-5))
    assert torch.equal(o[4:].cpu(), torch.zeros(4, H * dv))
    keep = [0, 2, 3]
    assert torch.equal(torch.nan_to_num(state[keep]), torch.nan_to_num(before[keep]))


def test_delta_rule_recalls_a_value_written_long_ago(ops, lanes):
    """With beta = 1 and no decay the state is an associative memory: the value written under one key hundreds of
    tokens back (in an earlier portion) comes out again for a query along that key, and a later write under the
    same key replaces it.  Keys in between are orthogonal to it."""
    G = H = 1
    d, dv, T = 64, 48, 300
    g = torch.Generator().manual_seed(5)
    qkv = torch.zeros(T, 2 * d + dv)
    for t in range(T):
        qkv[t, d + 1 + t % (d - 1)] = 3.0                    # keys e_1 .. e_63 in turn
        qkv[t, t % (d - 1) + 1] = 1.0                        # queries that look elsewhere
    qkv[:, 2 * d:] = torch.randn(T, dv, generator=g)
    qkv[0, d:2 * d] = 0
    qkv[0, d] = 2.0                                          # token 0 writes v_0 under e_0 ...
    qkv[T - 1, :d] = 0
    qkv[T - 1, 0] = 5.0                                      # ... and the last token asks for e_0
    qkv[T - 1, d:2 * d] = 0
    qkv[T - 1, d + 5] = 1.0
    ba = torch.zeros(T, 2 * H)
    ba[:, 0] = 40.0                                          # beta = 1
    ba[:, 1] = -200.0                                        # softplus = 0: decay = 1
    a_log, dt_bias = torch.zeros(H), torch.zeros(H)
    state = torch.full((2, H * dv * d), float("nan"), dtype=torch.float32, device="cuda")
    o_last = None
    for s, n in [(0, 150), (150, 149), (299, 1)]:            # the last token is decoded alone
        o = torch.empty(n, dv, dtype=torch.float32, device="cuda")
        ops.delta_rule(o, dev(qkv[s:s + n]), dev(ba[s:s + n]), dev(a_log), dev(dt_bias), state,
                       step_batch([n], [s], [1]), G, H, d, dv)
        o_last = o[-1].cpu()
    torch.testing.assert_close(o_last, qkv[0, 2 * d:] * d ** -0.5, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(o_last.to(F64), plain_delta(qkv, ba, a_log, dt_bias, G, H, d, dv)[-1], rtol=1e-4, atol=1e-5)


# ---------------------------------------------------------------- Mamba-2 recurrence
def plain_ssd(xbc, dt_raw, dt_bias, a_log, skip, H, P, N, G):
    T = xbc.shape[0]
    x = xbc.to(F64)
    return pm.ssd_recurrence(x[:, :H * P].view(T, H, P), x[:, H * P:H * P + G * N].view(T, G, N),
                             x[:, H * P + G * N:].view(T, G, N), dt_raw.to(F64), dt_bias.to(F64), a_log.to(F64),
                             skip.to(F64)).reshape(T, H * P)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,P,N,G", [(4, 24, 16, 2), (6, 40, 48, 3), (3, 130, 20, 1), (2, 8, 256, 2), (5, 64, 7, 5),
                                     (2, 64, 128, 1), (3, 20, 100, 3)])
def test_ssd_scan_over_portions_and_reused_slots(ops, lanes, dtype, H, P, N, G):
    g = torch.Generator().manual_seed(H * 100 + N)
    lengths, cuts, slots = [37, 12, 5], [[2, 3, 19, 36], [11], [1, 2, 3, 4]], [3, 0, 2]
    dt_bias, a_log = torch.randn(H, generator=g) * 0.5, torch.rand(H, generator=g) * 1.5 - 1.0
    skip = 1 + torch.randn(H, generator=g) * 0.2
    xs = [torch.randn(L, H * P + 2 * G * N, generator=g).to(dtype) for L in lengths]
    dts = [torch.randn(L, H, generator=g) * 2 for L in lengths]
    want = [plain_ssd(x, dt, dt_bias, a_log, skip, H, P, N, G) for x, dt in zip(xs, dts)]
    state = torch.full((4, H * P * N), float("nan"), dtype=torch.float32, device="cuda")
    got = [torch.zeros(L, H * P) for L in lengths]
    for who, starts, news in portions_of(lengths, cuts):
        x = torch.cat([xs[r][s:s + n] for r, s, n in zip(who, starts, news)])
        dt = torch.cat([dts[r][s:s + n] for r, s, n in zip(who, starts, news)])
        y = torch.full((x.shape[0], H * P), float("nan"), dtype=torch.float32, device="cuda")
        ops.ssd_scan(y, dev(x), dev(dt), dev(dt_bias), dev(a_log), dev(skip), state,
                     step_batch(news, starts, [slots[r] for r in who]), H, P, N, G)
        at = 0
        for r, s, n in zip(who, starts, news):
            got[r][s:s + n] = y[at:at + n].cpu()
            at += n
    for r in range(3):
        torch.testing.assert_close(got[r].to(F64), want[r], **tol(torch.float32, f32=5e-5))
    x, dt = torch.randn(3, H * P + 2 * G * N, generator=g).to(dtype), torch.randn(3, H, generator=g)
    y = torch.empty(6, H * P, dtype=torch.float32, device="cuda")
    ops.ssd_scan(y, dev(torch.cat([x, x])), dev(torch.cat([dt, dt])), dev(dt_bias), dev(a_log), dev(skip), state,
                 step_batch([3, 3], [0, 9], [3, -1]), H, P, N, G)
    torch.testing.assert_close(y[:3].cpu().to(F64), plain_ssd(x, dt, dt_bias, a_log, skip, H, P, N, G), **tol(torch.float32, f32=5e-5))
    assert torch.equal(y[3:].cpu(), torch.zeros(3, H * P))


def test_ssd_scan_keeps_an_input_from_long_ago(ops, lanes):
    """With a decay of almost one the state still holds the first token's write after 400 tokens whose B is
    orthogonal to the last C: the output is dt_0 x_0 (B_0 . C_last), through a portion's edge and single tokens."""
    H, P, N, G, T = 1, 16, 32, 1, 400
    g = torch.Generator().manual_seed(2)
    xbc = torch.zeros(T, P + 2 * N)
    xbc[:, :P] = torch.randn(T, P, generator=g)
    for t in range(1, T):
        xbc[t, P + 1 + t % (N - 1)] = 1.0                   # B_t = e_1 .. e_31
        xbc[t, P + N + 1 + (t + 3) % (N - 1)] = 1.0         # C_t elsewhere
    xbc[0, P] = 2.0                                          # B_0 = 2 e_0
    xbc[T - 1, P + N:] = 0
    xbc[T - 1, P + N] = 3.0                                  # C_last = 3 e_0
    dt_raw = torch.full((T, 1), 1.0)
    dt_bias, a_log, skip = torch.zeros(1), torch.full((1,), -30.0), torch.zeros(1)
    state = torch.full((1, P * N), float("nan"), dtype=torch.float32, device="cuda")
    y_last = None
    for s, n in [(0, 1), (1, 2), (3, 300), (303, 96), (399, 1)]:
        y = torch.empty(n, P, dtype=torch.float32, device="cuda")
        ops.ssd_scan(y, dev(xbc[s:s + n]), dev(dt_raw[s:s + n]), dev(dt_bias), dev(a_log), dev(skip), state,
                     step_batch([n], [s], [0]), H, P, N, G)
        y_last = y[-1].cpu()
    dt0 = float(pm.softplus(torch.tensor(1.0, dtype=F64)))
    torch.testing.assert_close(y_last, xbc[0, :P] * dt0 * 6.0, rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("groups,size,period,gate_first", [(1, 96, 96, True), (3, 40, 120, True), (4, 72, 72, False),
                                                            (2, 300, 600, True), (5, 16, 16, False)])
def test_gated_rmsnorm(ops, dtype, groups, size, period, gate_first):
    g = torch.Generator().manual_seed(size)
    T, n = 5, groups * size
    y = torch.randn(T, n, generator=g) * 3
    z = torch.randn(T, n + 7, generator=g).to(dtype)
    w = (1 + 0.2 * torch.randn(period, generator=g)).to(dtype)
    out = torch.empty(T, n, dtype=dtype, device="cuda")
    ops.gated_rmsnorm(out, dev(y), dev(z)[:, 7:], dev(w), groups, 1e-5, gate_first)
    want = pm.gated_norm(y.to(F64), z[:, 7:].to(F64), w.to(F64), groups, 1e-5, gate_first)
    torch.testing.assert_close(out.cpu().to(F64), want, **tol(dtype))


# ---------------------------------------------------------------- rotation, unit norm, attention with a sink
def rotary_table(dims, base, scaling, n_pos):
    f = pm.rotary_frequencies(dims, base, scaling)
    ang = torch.arange(n_pos, dtype=F64)[:, None] * f[None, :]
    return torch.cat((ang.cos(), ang.sin()), -1).float()


def run_attention(ops, dtype, qkvs, cuts, nq, nkv, dk, dv, page, rot, table, eps, scale, sink, seed=0, simt=True):
    """Requests' projected rows [L, nq dk + nkv dk + nkv dv] through rotation + norm + cache store and the attention
    kernel, in portions, with shuffled pages in a poisoned pool.  Returns per request [L, nq dv]."""
    rng = np.random.default_rng(seed)
    lengths = [x.shape[0] for x in qkvs]
    row = max(dk, dv)
    n_pages = sum(-(-L // page) for L in lengths) + 3
    pages = torch.full((n_pages, 2, nkv, page, row), float("nan"), dtype=dtype, device="cuda")
    free = list(rng.permutation(n_pages))
    tables = [[int(free.pop()) for _ in range(-(-L // page))] for L in lengths]
    width = max(len(t) for t in tables)
    got = [torch.zeros(L, nq * dv, dtype=dtype) for L in lengths]
    for who, starts, news in portions_of(lengths, cuts):
        x = torch.cat([qkvs[r][s:s + n] for r, s, n in zip(who, starts, news)])
        pos = [p for s, n in zip(starts, news) for p in range(s, s + n)]
        slots = [tables[r][p // page] * page + p % page for r, s, n in zip(who, starts, news) for p in range(s, s + n)]
        bt = torch.full((len(who), width), -1, dtype=torch.int32)
        for i, r in enumerate(who):
            bt[i, :len(tables[r])] = torch.tensor(tables[r], dtype=torch.int32)
        q = torch.full((x.shape[0], nq * dk), float("nan"), dtype=dtype, device="cuda")
        ops.rope_norm_store(dev(x), q, pages, i32(slots), i32(pos), None if table is None else dev(table), rot, nq, nkv,
                            dk, dv, eps)
        out = torch.full((x.shape[0], nq * dv), float("nan"), dtype=dtype, device="cuda")
        b = step_batch(news, starts, [-1] * len(who))
        if simt:
            ops.attention_sink_simt(out, q, pages, dev(bt), b.cu_q, b.kv_len, len(who), x.shape[0], nq, nkv, dk, dv, scale,
                                    None if sink is None else dev(sink))
        else:       # the dispatcher: the tensor-core kernels where the shape allows them
            ops.attention_sink(out, q, pages, SimpleNamespace(block_tables=dev(bt)), b, nq, nkv, dk, dv, scale,
                               None if sink is None else dev(sink))
        at = 0
        for r, s, n in zip(who, starts, news):
            got[r][s:s + n] = out[at:at + n].cpu()
            at += n
    return got


def plain_attention(x, nq, nkv, dk, dv, rot, freqs, eps, scale, sink):
    T = x.shape[0]
    x = x.to(F64)
    q, k = x[:, :nq * dk].view(T, nq, dk), x[:, nq * dk:(nq + nkv) * dk].view(T, nkv, dk)
    v = x[:, (nq + nkv) * dk:].view(T, nkv, dv)
    if rot:
        q, k = pm.rotate(q, torch.arange(T), freqs, rot), pm.rotate(k, torch.arange(T), freqs, rot)
    if eps is not None:
        q, k = pm.rms_unit(q, eps), pm.rms_unit(k, eps)
    s = torch.full((nq,), -1e30, dtype=F64) if sink is None else sink.to(F64)
    return pm.sink_attention(q, k, v, s, scale).reshape(T, nq * dv)


SCALING = dict(factor=8.0, low=1.0, high=4.0, original=64)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq,nkv,dk,dv,rot,page,scaling,sink", [
    (6, 2, 40, 72, 20, 8, SCALING, True), (4, 1, 64, 32, 64, 16, None, True), (3, 3, 24, 24, 8, 5, SCALING, False),
    (8, 4, 128, 16, 128, 64, SCALING, True), (2, 2, 16, 200, 0, 1, None, True)])
def test_sink_attention_in_portions_against_plain(ops, dtype, nq, nkv, dk, dv, rot, page, scaling, sink):
    g = torch.Generator().manual_seed(nq * 10 + dk)
    lengths, cuts = [75, 33, 2, 18], [[40, 42, 43, 74], [32], [1], [3, 5, 16, 17]]
    qkvs = [torch.randn(L, (nq + nkv) * dk + nkv * dv, generator=g).to(dtype) for L in lengths]
    sinks = torch.randn(nq, generator=g) * 2 if sink else None
    freqs = pm.rotary_frequencies(rot, 10000.0, scaling) if rot else None
    table = rotary_table(rot, 10000.0, scaling, 128) if rot else None
    got = run_attention(ops, dtype, qkvs, cuts, nq, nkv, dk, dv, page, rot, table, 1e-5, 0.3, sinks)
    for r, x in enumerate(qkvs):
        want = plain_attention(x, nq, nkv, dk, dv, rot, freqs, 1e-5, 0.3, sinks)
        torch.testing.assert_close(got[r].to(F64), want, **tol(dtype, f32=3e-5, bf16=3e-2))


@pytest.mark.parametrize("nq,nkv,d,page,which", [(4, 1, 64, 16, "mma"), (8, 2, 128, 64, "tcgen05"), (6, 2, 64, 128, "tcgen05"),
                                                  (3, 3, 48, 8, "mma"), (16, 4, 128, 256, "tcgen05"), (8, 2, 128, 64, "mma")])
def test_sink_attention_on_the_tensor_cores(ops, nq, nkv, d, page, which):
    """bfloat16 with key and value heads of one size: prompt portions and single tokens of long and short requests
    in one step through the tensor-core kernels (tcgen05 / TMA where the shape allows, else mma.sync), each with
    the sink in its head's sum exactly once, also where a request's keys are shared between several blocks."""
    g = torch.Generator().manual_seed(nq + d)
    lengths = [900, 130, 301, 40]
    cuts = [[600, 897, 898, 899], [64, 129], [300], [1, 2, 39]]
    qkvs = [torch.randn(L, (nq + 2 * nkv) * d, generator=g).to(torch.bfloat16) for L in lengths]
    sinks = torch.randn(nq, generator=g) * 3
    ops.USE_TCGEN05_ATTENTION = ops.USE_TMA_DECODE = which == "tcgen05"
    try:
        got = run_attention(ops, torch.bfloat16, qkvs, cuts, nq, nkv, d, d, page, 0, None, 1e-6, 0.25, sinks, simt=False)
    finally:
        ops.USE_TCGEN05_ATTENTION = ops.USE_TMA_DECODE = True
    assert ops.take_wait_errors() == [], "a bounded wait of a kernel ran out"
    for r, x in enumerate(qkvs):
        want = plain_attention(x, nq, nkv, d, d, 0, None, 1e-6, 0.25, sinks)
        torch.testing.assert_close(got[r].to(F64), want, rtol=3e-2, atol=3e-2)
    # without the sink the same rows differ: the test would see a sink that was left out
    assert not torch.allclose(plain_attention(qkvs[3], nq, nkv, d, d, 0, None, 1e-6, 0.25, None), got[3].to(F64), atol=3e-2)


@pytest.mark.parametrize("page", [7, 16, 64])
def test_sink_attention_finds_one_far_key_and_weighs_the_sink(ops, page):
    """No rotation, no norm: among 500 quiet keys, one loud key next to a page's edge takes nearly all the weight of
    the last (decoded) query; a loud sink takes it all away again; the first token alone shares its weight with the
    sink as exp(s) / (exp(s) + exp(sink))."""
    nq, nkv, dk, dv, T = 2, 1, 32, 48, 500
    g = torch.Generator().manual_seed(page)
    for far in (page - 1, page, 3 * page + 1):
        x = torch.randn(T, (nq + nkv) * dk + nkv * dv, generator=g) * 0.1
        x[T - 1, :nq * dk] = 0
        x[T - 1, 0], x[T - 1, dk] = 6.0, 6.0                     # both query heads along e_0
        x[far, nq * dk] = 8.0                                    # the loud key
        x[far, (nq + nkv) * dk:] = 5.0
        x[0, (nq + nkv) * dk:] = 1.0
        sinks = torch.tensor([-3.0, 60.0])                       # head 1's sink outweighs the loud key (score 48)
        got = run_attention(ops, torch.float32, [x], [[1, T - 1]], nq, nkv, dk, dv, page, 0, None, None, 1.0, sinks,
                            seed=far)[0]
        want = plain_attention(x, nq, nkv, dk, dv, 0, None, None, 1.0, sinks)
        torch.testing.assert_close(got.to(F64), want, rtol=1e-4, atol=2e-5)
        assert (got[-1, :dv] > 4.9).all() and (got[-1, dv:].abs() < 1e-3).all()
        s0 = float((x[0, :dk] * x[0, nq * dk:nq * dk + dk]).sum())
        share = np.exp(s0) / (np.exp(s0) + np.exp(-3.0))
        torch.testing.assert_close(got[0, :dv], torch.full((dv,), share, dtype=torch.float32), rtol=1e-4, atol=1e-5)


def test_banded_rotary_table(ops):
    """The table of the position part against frequencies written out here: every band occurs (kept, divided,
    blended), and without bands the plain geometric frequencies."""
    from nanohybrid_vlm_b200.parts import POSITIONS, BuildEnv, part
    env = BuildEnv(hidden_size=64, dtype=torch.float32, device="cuda", max_position=300)
    for scaling in (SCALING, dict(factor=3.0, low=2.0, high=6.0, original=500), None):
        spec = part("rope_banded", theta=5000.0, rotary_dim=48, **(scaling or {}))
        table, dims = POSITIONS.get(spec.kind)(spec, env).rotary()
        want = rotary_table(48, 5000.0, scaling, 300)
        assert dims == 48
        torch.testing.assert_close(table.cpu(), want, rtol=0, atol=1e-6)
    f, fs = pm.rotary_frequencies(48, 5000.0, None), pm.rotary_frequencies(48, 5000.0, SCALING)
    kinds = {("kept" if a == b else "divided" if abs(a / b - 8.0) < 1e-9 else "blended") for a, b in zip(f.tolist(), fs.tolist())}
    assert kinds == {"kept", "divided", "blended"}


# ---------------------------------------------------------------- small projections with 32-bit results
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("M,N,K", [(1, 6, 272), (8, 32, 2048), (70, 12, 136), (3, 650, 200), (600, 40, 264), (5, 3, 36)])
def test_linear_f32_keeps_the_sums(ops, dtype, M, N, K):
    """x W^T with float32 sums handed on unrounded, for one row and for many, also as a view of a wider matrix; a
    row's result does not depend on the rows beside it."""
    g = torch.Generator().manual_seed(M + N)
    wide = torch.randn(M, K + 8, generator=g).to(dtype)
    w = torch.randn(N, K, generator=g).to(dtype)
    x = dev(wide)[:, 8:] if K % 8 == 0 else dev(wide[:, 8:].contiguous())
    out = torch.empty(M, N, dtype=torch.float32, device="cuda")
    ops.linear_f32(out, x, dev(w))
    want = wide[:, 8:].to(F64) @ w.to(F64).T
    torch.testing.assert_close(out.cpu().to(F64), want, rtol=1e-4, atol=1e-4 * K ** 0.5)
    if M > 1:
        one = torch.empty(1, N, dtype=torch.float32, device="cuda")
        ops.linear_f32(one, x[M - 1:], dev(w))
        if dtype == torch.float32 or M * N <= ops.LINEAR_F32_ROWS_LIMIT:
            assert torch.equal(one[0], out[M - 1])
