"""A plain, slow restatement of the Muvonex design in float64 on the CPU: one function per mechanism,
token-by-token loops where the design has a recurrence, no cache, no batching.  The tests compare the engine
with it; it shares nothing with the engine's code.

Notation.  A layer's input is h [T, W].  Linear weights are [out, in] and applied as h @ W.T.  ``cfg`` is the
config.json dictionary, ``w`` maps tensor names to float64 tensors.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


# ---------------------------------------------------------------- small pieces
def rms_unit(x, eps):
    """x scaled to root mean square 1 over its last dimension (eps inside the root)."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm_around_zero(x, weight, eps):
    """RMS norm whose stored weight is an offset from one."""
    return rms_unit(x, eps) * (1.0 + weight)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.logaddexp(z, torch.zeros_like(z))


def gated_mlp(h, gate, up, down):
    return (gelu_tanh(h @ gate.T) * (h @ up.T)) @ down.T


def short_conv(x, taps_weight, bias=None):
    """Causal convolution over time, one filter per channel.  x [T, C]; taps_weight [C, K] whose last column
    multiplies the current token; inputs before the sequence are zero."""
    T, C = x.shape
    K = taps_weight.shape[1]
    padded = torch.cat([torch.zeros(K - 1, C, dtype=x.dtype), x], 0)
    y = torch.zeros(T, C, dtype=x.dtype)
    for j in range(K):
        y = y + padded[j:j + T] * taps_weight[:, j]
    if bias is not None:
        y = y + bias
    return y


# ---------------------------------------------------------------- rotary angles
def rotary_frequencies(dims, base, scaling=None):
    """f_i = base^(-2i/dims), i < dims/2, then rescaled by wavelength bands when ``scaling`` is given."""
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=F64)
    if scaling is None:
        return f
    factor, low, high, original = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
    out = f.clone()
    for i in range(dims // 2):
        wavelength = 2.0 * math.pi / float(f[i])
        if wavelength < original / high:
            continue
        if wavelength > original / low:
            out[i] = f[i] / factor
        else:
            s = (original / wavelength - low) / (high - low)
            out[i] = (1.0 - s) * f[i] / factor + s * f[i]
    return out


def rotate(x, positions, freqs, dims):
    """x [T, heads, d]; the first ``dims`` elements of each head rotate, element i with i + dims/2."""
    half = dims // 2
    ang = positions.to(F64)[:, None] * freqs[None, :]          # [T, half]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., dims:]], -1)


# ---------------------------------------------------------------- attention with a sink
def sink_attention(q, k, v, sink, scale):
    """q [T, H, d], k [T, G, d], v [T, G, dv], sink [H].  Causal; the softmax denominator holds exp(sink_h) too."""
    T, H, _ = q.shape
    G = k.shape[1]
    rep = H // G
    out = torch.zeros(T, H, v.shape[-1], dtype=q.dtype)
    for h in range(H):
        g = h // rep
        for i in range(T):
            s = (k[:i + 1, g] @ q[i, h]) * scale
            m = max(float(s.max()), float(sink[h]))
            e = torch.exp(s - m)
            denom = e.sum() + math.exp(float(sink[h]) - m)
            out[i, h] = (e[:, None] * v[:i + 1, g]).sum(0) / denom
    return out


def attention_side(h, w, pre, m, eps, positions):
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = (h @ w[pre + "q"].T).view(T, H, d)
    k = (h @ w[pre + "k"].T).view(T, G, d)
    v = (h @ w[pre + "v"].T).view(T, G, dv)
    rot = m["rot"]
    f = rotary_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
    q = rms_unit(rotate(q, positions, f, rot["dims"]), eps)
    k = rms_unit(rotate(k, positions, f, rot["dims"]), eps)
    o = sink_attention(q, k, v, w[pre + "sink"], m["scale"])
    return o.reshape(T, H * dv) @ w[pre + "o"].T


# ---------------------------------------------------------------- state-space side
def ssd_recurrence(x, B, C, dt_raw, dt_bias, a_log, skip, S0=None):
    """x [T, heads, P], B and C [T, G, N], dt_raw [T, heads] -> y [T, heads, P] (and the last state with S0 given).
    Per head: S <- exp(-exp(a_log) dt) S + dt B x^T, y = S^T C + skip x, dt = softplus(dt_raw + dt_bias)."""
    T, heads, P = x.shape
    G, N = B.shape[1], B.shape[2]
    dt = softplus(dt_raw + dt_bias)
    rate = torch.exp(a_log)
    y = torch.zeros(T, heads, P, dtype=x.dtype)
    last = torch.zeros(heads, N, P, dtype=x.dtype)
    for hd in range(heads):
        g = hd // (heads // G)
        S = torch.zeros(N, P, dtype=x.dtype) if S0 is None else S0[hd].clone()
        for t in range(T):
            S = torch.exp(-rate[hd] * dt[t, hd]) * S + dt[t, hd] * torch.outer(B[t, g], x[t, hd])
            y[t, hd] = S.T @ C[t, g] + skip[hd] * x[t, hd]
        last[hd] = S
    return y if S0 is None else (y, last)


def gated_norm(y, z, weight, parts, eps, gate_first):
    """y, z [T, n]; gate_first: unit_rms(y silu(z)) w in ``parts`` equal parts; else unit_rms(y) w silu(z), w tiled."""
    T, n = y.shape
    if gate_first:
        y = y * silu(z)
    y = rms_unit(y.view(T, parts, n // parts), eps).reshape(T, n) * weight.repeat(n // weight.numel())
    return y if gate_first else y * silu(z)


def ssd_side(h, w, pre, m, eps):
    heads, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = heads * P
    T = h.shape[0]
    proj = h @ w[pre + "in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(short_conv(xbc, w[pre + "conv"], w[pre + "conv.b"]))
    x = xbc[:, :inner].view(T, heads, P)
    B = xbc[:, inner:inner + G * N].view(T, G, N)
    C = xbc[:, inner + G * N:].view(T, G, N)
    y = ssd_recurrence(x, B, C, dt, w[pre + "dt_bias"], w[pre + "A_log"], w[pre + "D"])
    y = y.reshape(T, inner) * silu(z)
    parts = m["norm_groups"]
    y = rms_unit(y.view(T, parts, inner // parts), eps).reshape(T, inner) * w[pre + "norm"]
    return y @ w[pre + "o"].T


def parallel_mixer(h, w, pre, m, eps, positions):
    return (m["left_scale"] * attention_side(h, w, pre + "left.", m["left"], eps, positions)
            + m["right_scale"] * ssd_side(h, w, pre + "right.", m["right"], eps))


# ---------------------------------------------------------------- gated delta rule
def delta_recurrence(q, k, v, beta, decay, S0=None):
    """q, k [T, G, d] (already unit vectors), v [T, H, dv], beta and decay [T, H] -> o [T, H, dv] (and the last
    state with S0 given).  Per head: S <- decay S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q."""
    T, H, dv = v.shape
    G, d = q.shape[1], q.shape[2]
    o = torch.zeros(T, H, dv, dtype=v.dtype)
    last = torch.zeros(H, d, dv, dtype=v.dtype)
    for hd in range(H):
        g = hd // (H // G)
        S = torch.zeros(d, dv, dtype=v.dtype) if S0 is None else S0[hd].clone()
        for t in range(T):
            S = decay[t, hd] * S
            u = beta[t, hd] * (v[t, hd] - S.T @ k[t, g])
            S = S + torch.outer(k[t, g], u)
            o[t, hd] = S.T @ q[t, g]
        last[hd] = S
    return o if S0 is None else (o, last)


def delta_mixer(h, w, pre, m, eps):
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = silu(short_conv(h @ w[pre + "q"].T, w[pre + "q.conv"])).view(T, G, d)
    k = silu(short_conv(h @ w[pre + "k"].T, w[pre + "k.conv"])).view(T, G, d)
    v = silu(short_conv(h @ w[pre + "v"].T, w[pre + "v.conv"])).view(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w[pre + "b"].T)
    decay = torch.exp(-torch.exp(w[pre + "A_log"]) * softplus(h @ w[pre + "a"].T + w[pre + "dt_bias"]))
    o = delta_recurrence(q, k, v, beta, decay)
    o = rms_unit(o, eps) * w[pre + "norm"]
    o = o.reshape(T, H * dv) * silu(h @ w[pre + "g"].T)
    return o @ w[pre + "o"].T


# ---------------------------------------------------------------- the model
def forward(cfg, w, tokens, return_layers=False):
    """tokens: list of ids of ONE sequence -> logits [T, vocab] (and the residual stream after every layer)."""
    eps = cfg["norm"]["eps"]
    mult = cfg["residual_mult"]
    ids = torch.tensor(tokens, dtype=torch.long)
    positions = torch.arange(len(tokens))
    x = w["embed"][ids] * cfg["embedding"]["scale"]
    layers = []
    for i, layer in enumerate(cfg["layers"]):
        pre = f"l{i}."
        h = norm_around_zero(x, w[pre + "norm1"], eps)
        if layer["type"] == "parallel":
            mixed = parallel_mixer(h, w, pre + "mix.", layer["mixer"], eps, positions)
        elif layer["type"] == "delta":
            mixed = delta_mixer(h, w, pre + "mix.", layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        ff = 0.0
        if layer.get("mlp") is not None:
            ff = gated_mlp(h, w[pre + "mlp.gate"], w[pre + "mlp.up"], w[pre + "mlp.down"])
        x = x + mult * (mixed + ff)
        layers.append(x)
    logits = norm_around_zero(x, w["final.norm"], eps) @ w["embed"].T
    return (logits, torch.stack(layers)) if return_layers else logits


# ---------------------------------------------------------------- random models for the tests
def tensor_shapes(cfg):
    """name -> shape of every tensor of a model with this config."""
    W = cfg["width"]
    shapes = {"embed": (cfg["vocab"], W), "final.norm": (W,)}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        shapes[p + "norm1"] = (W,)
        if layer["type"] == "delta":
            H, G, d, dv, K = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
            for n, rows in (("q", G * d), ("k", G * d), ("v", H * dv)):
                shapes[p + "mix." + n] = (rows, W)
                shapes[p + "mix." + n + ".conv"] = (rows, K)
            shapes.update({p + "mix.b": (H, W), p + "mix.a": (H, W), p + "mix.A_log": (H,), p + "mix.dt_bias": (H,),
                           p + "mix.norm": (dv,), p + "mix.g": (H * dv, W), p + "mix.o": (W, H * dv)})
        else:
            a, s = m["left"], m["right"]
            q = p + "mix.left."
            shapes.update({q + "q": (a["heads"] * a["dim"], W), q + "k": (a["kv_heads"] * a["dim"], W),
                           q + "v": (a["kv_heads"] * a["vdim"], W), q + "sink": (a["heads"],),
                           q + "o": (W, a["heads"] * a["vdim"])})
            r = p + "mix.right."
            inner, gn = s["heads"] * s["vdim"], s["groups"] * s["state"]
            shapes.update({r + "in": (2 * inner + 2 * gn + s["heads"], W), r + "conv": (inner + 2 * gn, s["conv"]),
                           r + "conv.b": (inner + 2 * gn,), r + "dt_bias": (s["heads"],), r + "A_log": (s["heads"],),
                           r + "D": (s["heads"],), r + "norm": (inner,), r + "o": (W, inner)})
        if layer.get("mlp") is not None:
            ff = layer["mlp"]["ff"]
            shapes.update({p + "mlp.gate": (ff, W), p + "mlp.up": (ff, W), p + "mlp.down": (W, ff)})
    return shapes


def random_weights(cfg, seed, dtype=torch.bfloat16):
    """Random tensors (rounded to ``dtype``, returned in that dtype) sized so that activations stay of order one."""
    gen = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        leaf = name.split(".")[-1]
        if len(shape) == 2 and leaf != "conv":
            t = torch.randn(shape, generator=gen) * (1.0 / math.sqrt(shape[1]) if name != "embed" else 0.05)
        elif leaf == "conv":
            t = torch.randn(shape, generator=gen) * 0.4
        elif leaf in ("norm1", "norm") and "right" not in name and "mix.norm" not in name:
            t = torch.randn(shape, generator=gen) * 0.1                 # stored around zero
        elif leaf == "norm":
            t = 1.0 + torch.randn(shape, generator=gen) * 0.1
        elif leaf == "A_log":
            t = torch.rand(shape, generator=gen) * 1.5 - 1.0
        elif leaf == "sink":
            t = torch.randn(shape, generator=gen)
        elif leaf == "D":
            t = 1.0 + torch.randn(shape, generator=gen) * 0.2
        else:                                                           # dt_bias, conv bias
            t = torch.randn(shape, generator=gen) * 0.3
        out[name] = t.to(dtype)
    return out
