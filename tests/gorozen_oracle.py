"""Slow, plain float64 statement of the Gorozen equations, one function per mechanism. Shares no code with the package:
it takes a config dict (the checkpoint's ``config.json`` schema) and a dict of tensors under the checkpoint's names.

Notation: n tokens, W width, H query heads, G key/value heads, D head size, R rotated dims, E experts, K chosen experts.
"""
import math

import torch


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm(x, w, eps):
    """RMS norm whose gain is stored as a distance from one."""
    return unit_rms(x, eps) * (1.0 + w)


def rotary_frequencies(rot):
    """f_i = base^(-2i/R), then three bands by wavelength 2 pi / f against the original context length."""
    R = rot["dims"]
    f = torch.tensor([rot["base"] ** (-2.0 * i / R) for i in range(R // 2)], dtype=torch.float64)
    sc = rot.get("scaling")
    if not sc:
        return f
    out = []
    for fi in f.tolist():
        lam = 2 * math.pi / fi
        if lam < sc["original"] / sc["high"]:
            out.append(fi)
        elif lam > sc["original"] / sc["low"]:
            out.append(fi / sc["factor"])
        else:
            s = (sc["original"] / lam - sc["low"]) / (sc["high"] - sc["low"])
            out.append((1 - s) * fi / sc["factor"] + s * fi)
    return torch.tensor(out, dtype=torch.float64)


def rotate(x, positions, rot):
    """x [n, heads, D]; neighbours (2i, 2i+1) of the first R dims turn by positions * f_i; the rest stays."""
    R = rot["dims"]
    if R == 0:
        return x.clone()
    f = rotary_frequencies(rot)
    y = x.clone()
    for t, p in enumerate(positions):
        for i in range(R // 2):
            a = p * float(f[i])
            c, s = math.cos(a), math.sin(a)
            u, v = x[t, :, 2 * i].clone(), x[t, :, 2 * i + 1].clone()
            y[t, :, 2 * i] = u * c - v * s
            y[t, :, 2 * i + 1] = v * c + u * s
    return y


def sink_softmax_attention(q, k, v, scale, sink):
    """q [n, H, D] (rotated), k [n, G, D] (rotated), v [n, G, D]; causal; the denominator also holds exp(sink_h)."""
    n, H, D = q.shape
    G = k.shape[1]
    out = torch.zeros(n, H, D, dtype=q.dtype)
    for h in range(H):
        g = h // (H // G)
        for i in range(n):
            sc = (k[:i + 1, g] @ q[i, h]) * scale
            m = max(float(sc.max()), float(sink[h]))
            e = torch.exp(sc - m)
            den = e.sum() + math.exp(float(sink[h]) - m)
            out[i, h] = (e / den) @ v[:i + 1, g]
    return out


def attention(h, W, pre, mc, positions=None):
    n = h.shape[0]
    H, G, D = mc["heads"], mc["kv_heads"], mc["dim"]
    positions = list(range(n)) if positions is None else positions
    q = (h @ W[pre + "q"].T).view(n, H, D)
    k = (h @ W[pre + "k"].T).view(n, G, D)
    v = k.clone()                                          # the values are the keys as projected, not rotated
    q, k = rotate(q, positions, mc["rot"]), rotate(k, positions, mc["rot"])
    o = sink_softmax_attention(q, k, v, mc["scale"], W[pre + "sink"])
    return o.reshape(n, H * D) @ W[pre + "o"].T


def dense_ff(h, W, pre, fc):
    lim = fc["limit"]
    g = torch.clamp(h @ W[pre + "gate"].T, max=lim)
    u = torch.clamp(h @ W[pre + "up"].T, -lim, lim)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ W[pre + "down"].T


def router(h, W, pre, fc):
    """(chosen experts [n, K], weights [n, K]): softmax over the K largest logits only."""
    z = h @ W[pre + "router"].T + W[pre + "router.b"]
    K = fc["router"]["top"]
    order = torch.argsort(z, dim=-1, descending=True, stable=True)[:, :K]
    zs = torch.gather(z, 1, order)
    e = torch.exp(zs - zs.max(-1, keepdim=True).values)
    return order, e / e.sum(-1, keepdim=True)


def moe_ff(h, W, pre, fc):
    idx, wts = router(h, W, pre, fc)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(idx.shape[1]):
            p = f"{pre}e{int(idx[t, j])}."
            a = h[t] @ W[p + "gate"].T
            y = (a * torch.sigmoid(a) * (h[t] @ W[p + "up"].T)) @ W[p + "down"].T
            out[t] += wts[t, j] * y
    return out


def forward(cfg, W, tokens, residuals=None):
    """Logits [n, vocab] of one sequence; ``residuals`` receives the stream after every layer."""
    W = {k: v.double() for k, v in W.items()}
    eps = cfg["norm"]["eps"]
    x = W["embed"][torch.as_tensor(tokens)]
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        x = x + norm(attention(norm(x, W[p + "norm1"], eps), W, p + "mix.", L["mixer"]), W[p + "norm1b"], eps)
        f = L.get("mlp")
        if f is not None:
            hin = norm(x, W[p + "norm2"], eps)
            y = dense_ff(hin, W, p + "mlp.", f) if f["kind"] == "dense" else moe_ff(hin, W, p + "mlp.", f)
            x = x + norm(y, W[p + "norm2b"], eps)
        if residuals is not None:
            residuals.append(x.clone())
    z = norm(x, W["final.norm"], eps) @ W["head"].T
    cap = cfg.get("logit_softcap")
    return cap * torch.tanh(z / cap) if cap else z


def greedy(cfg, W, prompt, new_tokens):
    toks = list(prompt)
    for _ in range(new_tokens):
        toks.append(int(forward(cfg, W, toks)[-1].argmax()))
    return toks


# ------------------------------------------------------------------------------------------------------------------
# small random models
# ------------------------------------------------------------------------------------------------------------------
def make_config(width=64, vocab=96, layers=None, eps=1e-5, softcap=12.0):
    return {"architecture": "Gorozen", "layers": layers, "logit_softcap": softcap, "norm": {"eps": eps}, "vocab": vocab, "width": width}


def attn_layer(heads=4, kv_heads=2, dim=32, rot_dims=16, base=10000.0, scaling=None, scale=None, mlp=None):
    rot = {"base": base, "dims": rot_dims}
    if scaling:
        rot["scaling"] = scaling
    return {"type": "attention", "mixer": {"dim": dim, "heads": heads, "kv_heads": kv_heads, "vdim": dim, "rot": rot,
                                           "scale": scale if scale is not None else dim ** -0.5}, "mlp": mlp}


def dense(ff=80, limit=2.0):
    return {"kind": "dense", "ff": ff, "limit": limit}


def moe(experts=4, top=2, ff=48):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def random_weights(cfg, seed=0, std=None, dtype=torch.bfloat16):
    """Tensors under the checkpoint's names, rounded to ``dtype`` (so that a bf16 model and the oracle see the same values)."""
    g = torch.Generator().manual_seed(seed)
    W, V = cfg["width"], cfg["vocab"]
    rn = lambda *s, sd=1.0: (torch.randn(*s, generator=g) * sd).to(dtype)          # noqa: E731
    out = {"embed": rn(V, W), "final.norm": rn(W, sd=0.2), "head": rn(V, W, sd=W ** -0.5)}
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        for nm in ("norm1", "norm1b"):
            out[p + nm] = rn(W, sd=0.2)
        out[p + "mix.q"] = rn(m["heads"] * m["dim"], W, sd=std or W ** -0.5)
        out[p + "mix.k"] = rn(m["kv_heads"] * m["dim"], W, sd=std or W ** -0.5)
        out[p + "mix.o"] = rn(W, m["heads"] * m["dim"], sd=(m["heads"] * m["dim"]) ** -0.5)
        out[p + "mix.sink"] = rn(m["heads"])
        f = L.get("mlp")
        if f is None:
            continue
        for nm in ("norm2", "norm2b"):
            out[p + nm] = rn(W, sd=0.2)
        if f["kind"] == "dense":
            out[p + "mlp.gate"], out[p + "mlp.up"] = rn(f["ff"], W, sd=2 * W ** -0.5), rn(f["ff"], W, sd=2 * W ** -0.5)
            out[p + "mlp.down"] = rn(W, f["ff"], sd=f["ff"] ** -0.5)
        else:
            E, F = f["router"]["experts"], f["expert"]["ff"]
            out[p + "mlp.router"], out[p + "mlp.router.b"] = rn(E, W, sd=W ** -0.5), rn(E)
            for e in range(E):
                q = f"{p}mlp.e{e}."
                out[q + "gate"], out[q + "up"], out[q + "down"] = rn(F, W, sd=W ** -0.5), rn(F, W, sd=W ** -0.5), rn(W, F, sd=F ** -0.5)
    return out
