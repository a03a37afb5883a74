"""Nomudra in plain PyTorch on the CPU, in float64, one function per mechanism, written from the design's equations.
It shares no code with the engine: it is what the engine's kernels are compared with.

Notation: x [T, W] rows of one request, positions 0 .. T-1; p(name) a tensor of the checkpoint.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64
EXPERT_ALPHA = 1.702


def dyntanh(x, alpha, w, b):
    """A norm without statistics: tanh(alpha x) * w + b."""
    return torch.tanh(alpha * x) * w + b


def rotate_half(x, positions, base, dims):
    """x [T, heads, d]: element i < dims/2 is paired with element i + dims/2; the pair turns by position * base^(-2i/dims).
    Elements from dims on pass unchanged."""
    half = dims // 2
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F64)
    ang = positions.to(F64)[:, None] * freq[None, :]
    c, s = ang.cos()[:, None, :], ang.sin()[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def chunk_mask(n, size):
    """visible[i, j]: j <= i and both in the same chunk of `size` positions counted from 0 (size None: causal only)."""
    i = torch.arange(n)
    vis = i[None, :] <= i[:, None]
    if size is not None:
        vis &= (i[None, :] // size) == (i[:, None] // size)
    return vis


def chunked_attention(h, m, q_w, q_b, k_w, k_b, g_w, o_w, o_b):
    """Grouped-query attention whose values are the keys as projected (before the rotation), chunked, with a sigmoid
    gate on the concatenated heads."""
    T = h.shape[0]
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    q = (h @ q_w.T + q_b).view(T, H, d)
    k = (h @ k_w.T + k_b).view(T, G, d)
    v = k
    pos = torch.arange(T)
    qr = rotate_half(q, pos, m["rot"]["base"], m["rot"]["dims"])
    kr = rotate_half(k, pos, m["rot"]["base"], m["rot"]["dims"])
    vis = chunk_mask(T, m["mask"]["size"] if m.get("mask") else None)
    heads = []
    for hh in range(H):
        g = hh // (H // G)
        score = (qr[:, hh] @ kr[:, g].T) * m["scale"]
        score = score.masked_fill(~vis, -math.inf)
        heads.append(torch.softmax(score, dim=-1) @ v[:, g])
    cat = torch.cat(heads, dim=-1) * torch.sigmoid(h @ g_w.T)
    return cat @ o_w.T + o_b


def mlstm_gates(h, i_w, i_b, f_w, f_b, cap):
    """Log input gate and log forget gate per head, both capped through tanh."""
    i = cap * torch.tanh((h @ i_w.T + i_b) / cap)
    f = torch.nn.functional.logsigmoid(cap * torch.tanh((h @ f_w.T + f_b) / cap))
    return i, f


def mlstm_recurrence(q, k, v, i, f):
    """q, k [T, H, d] (q already scaled), v [T, H, dv], gates [T, H] -> o [T, H, dv], token by token."""
    T, H, d = k.shape
    dv = v.shape[-1]
    out = torch.zeros(T, H, dv, dtype=F64)
    for hh in range(H):
        S = torch.zeros(d, dv, dtype=F64)
        n = torch.zeros(d, dtype=F64)
        m = torch.zeros((), dtype=F64)
        for t in range(T):
            m_new = torch.maximum(f[t, hh] + m, i[t, hh])
            keep, take = torch.exp(f[t, hh] + m - m_new), torch.exp(i[t, hh] - m_new)
            S = keep * S + take * torch.outer(k[t, hh], v[t, hh])
            n = keep * n + take * k[t, hh]
            m = m_new
            den = torch.maximum((n @ q[t, hh]).abs(), torch.exp(-m)) + 1e-6
            out[t, hh] = (S.T @ q[t, hh]) / den
    return out


def mlstm(h, m, eps, q_w, k_w, v_w, g_w, i_w, i_b, f_w, f_b, norm_w, o_w):
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = (h @ q_w.T).view(T, H, d) * d ** -0.5
    k = (h @ k_w.T).view(T, H, d)
    v = (h @ v_w.T).view(T, H, dv)
    i, f = mlstm_gates(h, i_w, i_b, f_w, f_b, m["gate_cap"])
    o = mlstm_recurrence(q, k, v, i, f)
    o = o / torch.sqrt((o * o).mean(dim=-1, keepdim=True) + eps)
    return (o.reshape(T, H * dv) * norm_w * torch.sigmoid(h @ g_w.T)) @ o_w.T


def clamped_unit(h, gate_w, up_w, down_w, limit):
    g = torch.clamp(h @ gate_w.T, max=limit)
    u = torch.clamp(h @ up_w.T, min=-limit, max=limit)
    return (g * torch.sigmoid(EXPERT_ALPHA * g) * (u + 1.0)) @ down_w.T


def route(h, router_w, correction, r):
    """(ids [T, top], weights [T, top], scores [T, N]) of the router: softmax scores; the choice by score + correction
    among the outputs of the best groups; weights from the scores without the correction."""
    N = r["experts"] + r.get("identity", 0)
    s = torch.softmax(h @ router_w.T, dim=-1)
    choice = s + correction
    groups = r.get("groups") or {}
    count = groups.get("count", 1)
    keep = groups.get("keep", count)
    per = N // count
    best = choice.view(-1, count, per).max(dim=-1).values.topk(keep, dim=-1).indices
    allowed = torch.zeros(h.shape[0], count, dtype=torch.bool).scatter_(1, best, True)
    allowed = allowed[:, :, None].expand(-1, -1, per).reshape(-1, N)
    ids = choice.masked_fill(~allowed, -math.inf).topk(r["top"], dim=-1).indices
    w = s.gather(1, ids)
    return ids, w / (w.sum(dim=-1, keepdim=True) + 1e-20), s


def moe(h, mlp, p):
    """p(name) gives the tensor ``<layer>.mlp.<name>``."""
    r = mlp["router"]
    E = r["experts"]
    ids, w, _ = route(h, p("router"), p("correction"), r)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, wt in zip(ids[t].tolist(), w[t]):
            if e >= E:
                out[t] += wt * h[t]                  # an identity expert
            else:
                out[t] += wt * clamped_unit(h[t:t + 1], p(f"e{e}.gate"), p(f"e{e}.up"), p(f"e{e}.down"),
                                            mlp["expert"]["limit"])[0]
    if mlp.get("shared") is not None:
        sh = clamped_unit(h, p("shared.gate"), p("shared.up"), p("shared.down"), mlp["shared"]["limit"])
        out = out + sh * torch.sigmoid(h @ p("shared.sg").T)
    return out


def forward(cfg, w, tokens, return_stream=False):
    """Logits [T, vocab] of one request (float64).  ``w``: the checkpoint's tensors in float64."""
    def norm(x, name):
        return dyntanh(x, w[name + ".alpha"], w[name], w[name + ".b"])

    x = norm(w["embed"][torch.as_tensor(tokens)], "embed.norm")
    eps = cfg["norm"]["eps"]
    streams = []
    for li, layer in enumerate(cfg["layers"]):
        pre = f"l{li}."
        mx = lambda n: w[pre + "mix." + n]          # noqa: E731
        h = norm(x, pre + "norm1")
        m = layer["mixer"]
        if layer["type"] == "attention":
            a = chunked_attention(h, m, mx("q"), mx("q.b"), mx("k"), mx("k.b"), mx("g"), mx("o"), mx("o.b"))
        else:
            a = mlstm(h, m, eps, mx("q"), mx("k"), mx("v"), mx("g"), mx("i"), mx("i.b"), mx("f"), mx("f.b"), mx("norm"),
                      mx("o"))
        x = x + norm(a, pre + "norm1b")
        if layer.get("mlp") is not None:
            y = moe(norm(x, pre + "norm2"), layer["mlp"], lambda n: w[pre + "mlp." + n])
            x = x + norm(y, pre + "norm2b")
        streams.append(x)
    logits = norm(x, "final.norm") @ w["head"].T
    return (logits, streams) if return_stream else logits


def tensor_shapes(cfg) -> dict:
    W, V = cfg["width"], cfg["vocab"]
    out = {"embed": (V, W), "head": (V, W)}

    def norm(name):
        out[name], out[name + ".b"], out[name + ".alpha"] = (W,), (W,), ()

    norm("embed.norm")
    norm("final.norm")
    for li, layer in enumerate(cfg["layers"]):
        pre, m = f"l{li}.", layer["mixer"]
        norm(pre + "norm1")
        norm(pre + "norm1b")
        mix = pre + "mix."
        if layer["type"] == "attention":
            H, G, d = m["heads"], m["kv_heads"], m["dim"]
            out.update({mix + "q": (H * d, W), mix + "q.b": (H * d,), mix + "k": (G * d, W), mix + "k.b": (G * d,),
                        mix + "g": (H * m["vdim"], W), mix + "o": (W, H * m["vdim"]), mix + "o.b": (W,)})
        else:
            H, d, dv = m["heads"], m["dim"], m["vdim"]
            out.update({mix + "q": (H * d, W), mix + "k": (H * d, W), mix + "v": (H * dv, W), mix + "g": (H * dv, W),
                        mix + "o": (W, H * dv), mix + "norm": (H * dv,), mix + "i": (H, W), mix + "i.b": (H,),
                        mix + "f": (H, W), mix + "f.b": (H,)})
        mlp = layer.get("mlp")
        if mlp is not None:
            norm(pre + "norm2")
            norm(pre + "norm2b")
            r, ff, mp = mlp["router"], mlp["expert"]["ff"], pre + "mlp."
            N = r["experts"] + r.get("identity", 0)
            for e in range(r["experts"]):
                out.update({f"{mp}e{e}.gate": (ff, W), f"{mp}e{e}.up": (ff, W), f"{mp}e{e}.down": (W, ff)})
            out.update({mp + "router": (N, W), mp + "correction": (N,)})
            if mlp.get("shared") is not None:
                sf = mlp["shared"]["ff"]
                out.update({mp + "shared.gate": (sf, W), mp + "shared.up": (sf, W), mp + "shared.down": (W, sf),
                            mp + "shared.sg": (1, W)})
    return out


def random_weights(cfg, seed, dtype=torch.bfloat16) -> dict:
    """Random tensors (rounded to ``dtype``, returned in that dtype) sized so that activations stay of order one, gates
    differ between heads, the router spreads its choices and the experts' limits are reached now and then."""
    gen = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        leaf = name.split(".")[-1]
        if leaf == "alpha":
            t = 0.4 + 0.5 * torch.rand(shape, generator=gen)
        elif leaf == "embed":
            t = torch.randn(shape, generator=gen) * 1.5
        elif leaf == "router":
            t = torch.randn(shape, generator=gen) * (3.0 / math.sqrt(shape[1]))
        elif leaf == "correction":
            t = torch.randn(shape, generator=gen) * 0.1
        elif leaf in ("gate", "up") or (leaf in ("i", "f") and len(shape) == 2):
            t = torch.randn(shape, generator=gen) * (2.5 / math.sqrt(shape[1]))
        elif len(shape) == 2:
            t = torch.randn(shape, generator=gen) * (1.0 / math.sqrt(shape[1]))
        elif name.endswith("i.b"):
            t = torch.randn(shape, generator=gen)
        elif name.endswith("f.b"):
            t = 2.0 + torch.randn(shape, generator=gen)
        elif leaf == "b":
            t = torch.randn(shape, generator=gen) * 0.2
        else:                                        # norm weights
            t = 1.0 + torch.randn(shape, generator=gen) * 0.2
        out[name] = t.to(dtype)
    return out
