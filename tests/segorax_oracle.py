"""Slow, plain float64 statement of the Segorax equations, one function per mechanism. Shares no code with the package:
it takes a config dict (the checkpoint's ``config.json`` schema) and a dict of tensors under the checkpoint's names.

Notation: n tokens, W width, H heads, D un-rotated and R rotated query/key dims per head, Dv value dims per head, C the
latent size, Cq the query latent size, E experts, K chosen experts.

This oracle expands keys and values per head from the latent (the direct reading of the equations); the package never
does that, it attends over the cached latent rows.
"""
import math

import torch


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm(x, w, eps):
    return unit_rms(x, eps) * w


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def gelu_erf(z):
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def rotary_frequencies(rot):
    """(f [R / 2], magnitude): f_i = base^(-2i/R); with ``scaling`` the slow dims are divided by ``factor`` through a ramp
    between two dim indices found from the wavelengths ``original / fast`` and ``original / slow``, and cos / sin grow by
    0.1 ln(factor) + 1."""
    R, base = rot["dims"], rot["base"]
    f = [base ** (-2.0 * i / R) for i in range(R // 2)]
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    where = lambda t: R * math.log(sc["original"] / (2 * math.pi * t)) / (2 * math.log(base))          # noqa: E731
    lo = max(math.floor(where(sc["fast"])), 0)
    hi = min(math.ceil(where(sc["slow"])), R - 1)
    out = []
    for i, fi in enumerate(f):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(fi / sc["factor"] * ramp + fi * (1 - ramp))
    return out, 0.1 * math.log(sc["factor"]) + 1.0


def rotate(x, positions, rot):
    """x [n, heads, R']: neighbours (2i, 2i+1) of the first R dims turn by positions * f_i; the rest stays."""
    R = rot["dims"]
    f, mag = rotary_frequencies(rot)
    y = x.clone()
    for t, p in enumerate(positions):
        for i in range(R // 2):
            a = p * f[i]
            c, s = math.cos(a) * mag, math.sin(a) * mag
            u, v = x[t, :, 2 * i].clone(), x[t, :, 2 * i + 1].clone()
            y[t, :, 2 * i] = u * c - v * s
            y[t, :, 2 * i + 1] = v * c + u * s
    return y


def causal_attention(q, k, v, scale, sink=None):
    """q, k [n, H, Dq]; v [n, H, Dv]; position i sees j <= i; ``sink`` [H] adds exp(sink_h) to the denominator only."""
    n, H, _ = q.shape
    out = torch.zeros(n, H, v.shape[2], dtype=q.dtype)
    for h in range(H):
        for i in range(n):
            sc = (k[:i + 1, h] @ q[i, h]) * scale
            m = float(sc.max()) if sink is None else max(float(sc.max()), float(sink[h]))
            e = torch.exp(sc - m)
            den = e.sum() + (0.0 if sink is None else math.exp(float(sink[h]) - m))
            out[i, h] = (e / den) @ v[:i + 1, h]
    return out


def latent_attention(h, W, pre, mc, eps, kind, positions=None):
    """``kind`` "latent_attention": queries through a normed latent, sinks; "latent_attention_2": direct queries, scaled
    rotary frequencies, no sink."""
    n = h.shape[0]
    H, D, R, Dv, C = mc["heads"], mc["dim"], mc["rot_dim"], mc["vdim"], mc["kv_rank"]
    positions = list(range(n)) if positions is None else positions
    if kind == "latent_attention":
        q = norm(h @ W[pre + "dq"].T, W[pre + "dq.norm"], eps) @ W[pre + "uq"].T
    else:
        q = h @ W[pre + "q"].T
    q = q.view(n, H, D + R)
    kv = h @ W[pre + "dkv"].T
    c = norm(kv[:, :C], W[pre + "dkv.norm"], eps)
    k_rot = rotate(kv[:, None, C:], positions, mc["rot"])                       # [n, 1, R], one for all heads
    q_rot = rotate(q[:, :, D:], positions, mc["rot"])
    k = torch.cat([(c @ W[pre + "uk"].T).view(n, H, D), k_rot.expand(n, H, R)], -1)
    v = (c @ W[pre + "uv"].T).view(n, H, Dv)
    o = causal_attention(torch.cat([q[:, :, :D], q_rot], -1), k, v, mc["scale"], W.get(pre + "sink") if kind == "latent_attention" else None)
    return o.reshape(n, H * Dv) @ W[pre + "o"].T


def dense_ff(h, W, pre):
    return (gelu_tanh(h @ W[pre + "gate"].T) * (h @ W[pre + "up"].T)) @ W[pre + "down"].T


def plain_expert(h, W, pre):
    return gelu_erf(h @ W[pre + "up"].T) @ W[pre + "down"].T


def router(h, W, pre, rc):
    """(chosen experts [n, K], weights [n, K]). s = sigmoid(z); the choice is made on s + correction among the experts of
    the ``keep`` groups whose two largest choice scores sum highest; the weights are s of the chosen, as they are."""
    s = torch.sigmoid(h @ W[pre + "router"].T)
    choice = s + W[pre + "correction"]
    n, E = s.shape
    K = rc["top"]
    g = rc.get("groups") or {"count": 1, "keep": 1}
    per = E // g["count"]
    idx = torch.zeros(n, K, dtype=torch.long)
    wts = torch.zeros(n, K, dtype=s.dtype)
    for t in range(n):
        gs = [sum(sorted(choice[t, j * per:(j + 1) * per].tolist(), reverse=True)[:2]) for j in range(g["count"])]
        kept = sorted(range(g["count"]), key=lambda j: (-gs[j], j))[:g["keep"]]
        cand = [e for e in range(E) if e // per in kept]
        cand.sort(key=lambda e: (-float(choice[t, e]), e))
        for j, e in enumerate(cand[:K]):
            idx[t, j], wts[t, j] = e, s[t, e]
    return idx, wts


def moe_ff(h, W, pre, fc):
    idx, wts = router(h, W, pre, fc["router"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(idx.shape[1]):
            out[t] += wts[t, j] * plain_expert(h[t], W, f"{pre}e{int(idx[t, j])}.")
    if fc.get("shared"):
        out = out + torch.sigmoid(h @ W[pre + "shared.sg"].T) * plain_expert(h, W, pre + "shared.")
    return out


def forward(cfg, W, tokens, residuals=None):
    """Logits [n, vocab] of one sequence; ``residuals`` receives the stream after every layer."""
    W = {k: v.double() for k, v in W.items()}
    eps, m = cfg["norm"]["eps"], cfg["residual_mult"]
    x = W["embed"][torch.as_tensor(tokens)] * cfg["embedding"]["scale"]
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        x = x + m * norm(latent_attention(x, W, p + "mix.", L["mixer"], eps, L["type"]), W[p + "norm1"], eps)
        f = L.get("mlp")
        if f is not None:
            y = dense_ff(x, W, p + "mlp.") if f["kind"] == "dense" else moe_ff(x, W, p + "mlp.", f)
            x = x + m * norm(y, W[p + "norm2"], eps)
        if residuals is not None:
            residuals.append(x.clone())
    return norm(x, W["final.norm"], eps) @ W["head"].T * cfg["logit_scale"]


def greedy(cfg, W, prompt, new_tokens):
    toks = list(prompt)
    for _ in range(new_tokens):
        toks.append(int(forward(cfg, W, toks)[-1].argmax()))
    return toks


# ------------------------------------------------------------------------------------------------------------------
# small random models
# ------------------------------------------------------------------------------------------------------------------
def make_config(width=64, vocab=96, layers=None, eps=1e-5, embed_scale=3.0, residual_mult=0.7, logit_scale=0.8):
    return {"architecture": "Segorax", "embedding": {"scale": embed_scale}, "layers": layers, "logit_scale": logit_scale,
            "norm": {"eps": eps}, "residual_mult": residual_mult, "vocab": vocab, "width": width}


def latent_layer(kind="latent_attention", heads=4, dim=24, rot_dim=8, vdim=16, kv_rank=40, q_rank=32, base=10000.0, scaling=None,
                 scale=None, mlp=None):
    rot = {"base": base, "dims": rot_dim}
    if scaling:
        rot["scaling"] = scaling
    mixer = {"dim": dim, "heads": heads, "kv_rank": kv_rank, "rot": rot, "rot_dim": rot_dim, "vdim": vdim,
             "scale": scale if scale is not None else (dim + rot_dim) ** -0.5}
    if kind == "latent_attention":
        mixer["q_rank"] = q_rank
    return {"type": kind, "mixer": mixer, "mlp": mlp}


def dense(ff=80):
    return {"kind": "dense", "ff": ff}


def moe(experts=6, top=2, ff=48, groups=3, keep=2, shared_ff=40):
    d = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "groups": {"count": groups, "keep": keep}}}
    if shared_ff:
        d["shared"] = {"ff": shared_ff}
    return d


def random_weights(cfg, seed=0, dtype=torch.bfloat16):
    """Tensors under the checkpoint's names, rounded to ``dtype`` (so that a bf16 model and the oracle see the same values)."""
    g = torch.Generator().manual_seed(seed)
    W, V = cfg["width"], cfg["vocab"]
    rn = lambda *s, sd=1.0, mean=0.0: (torch.randn(*s, generator=g) * sd + mean).to(dtype)          # noqa: E731
    out = {"embed": rn(V, W, sd=0.5), "final.norm": rn(W, sd=0.2, mean=1.0), "head": rn(V, W, sd=W ** -0.5)}
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        H, D, R, Dv, C = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
        out[p + "norm1"] = rn(W, sd=0.2, mean=1.0)
        if L["type"] == "latent_attention":
            Cq = m["q_rank"]
            out[p + "mix.dq"], out[p + "mix.dq.norm"] = rn(Cq, W, sd=W ** -0.5), rn(Cq, sd=0.2, mean=1.0)
            out[p + "mix.uq"] = rn(H * (D + R), Cq, sd=2 * Cq ** -0.5)
            out[p + "mix.sink"] = rn(H)
        else:
            out[p + "mix.q"] = rn(H * (D + R), W, sd=2 * W ** -0.5)
        out[p + "mix.dkv"], out[p + "mix.dkv.norm"] = rn(C + R, W, sd=W ** -0.5), rn(C, sd=0.2, mean=1.0)
        out[p + "mix.uk"], out[p + "mix.uv"] = rn(H * D, C, sd=C ** -0.5), rn(H * Dv, C, sd=C ** -0.5)
        out[p + "mix.o"] = rn(W, H * Dv, sd=(H * Dv) ** -0.5)
        f = L.get("mlp")
        if f is None:
            continue
        out[p + "norm2"] = rn(W, sd=0.2, mean=1.0)
        if f["kind"] == "dense":
            out[p + "mlp.gate"], out[p + "mlp.up"] = rn(f["ff"], W, sd=2 * W ** -0.5), rn(f["ff"], W, sd=2 * W ** -0.5)
            out[p + "mlp.down"] = rn(W, f["ff"], sd=f["ff"] ** -0.5)
        else:
            E, F = f["router"]["experts"], f["expert"]["ff"]
            out[p + "mlp.router"], out[p + "mlp.correction"] = rn(E, W, sd=W ** -0.5), rn(E, sd=0.3)
            for e in range(E):
                q = f"{p}mlp.e{e}."
                out[q + "up"], out[q + "down"] = rn(F, W, sd=2 * W ** -0.5), rn(W, F, sd=F ** -0.5)
            if f.get("shared"):
                Fs = f["shared"]["ff"]
                out[p + "mlp.shared.up"], out[p + "mlp.shared.down"] = rn(Fs, W, sd=2 * W ** -0.5), rn(W, Fs, sd=Fs ** -0.5)
                out[p + "mlp.shared.sg"] = rn(1, W, sd=W ** -0.5)
    return out
