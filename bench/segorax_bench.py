"""Segorax beside Gorozen (the framework's other design on the ragged paged step) at equal layer sizes, random weights:
prefill and decode throughput through each model's own generator, and the time of each Segorax kernel next to the Gorozen
kernel that does the like job, as fractions of the measured roofline (``MEASURED_PEAKS.json``: copy bandwidth and cuBLAS
bf16 rate of this pool's B200).

    python bench.py --workload segorax [--steps K --warmup W]

Timing: CUDA events on the launching stream, W >= 3 warm-up iterations; the single-kernel rows (both designs) are replayed
from a CUDA graph, since they run for less time than the host needs to issue them, with an L2 flush (a 256 MB write)
between timed iterations; the end-to-end rows run steps whose weights and caches together exceed L2.
"""
from __future__ import annotations

import json
import time

import torch

from gorozen_bench import Timer, _peaks, gorozen_config

SIZES = {
    # name: (width, heads, un-rotated dim, rotated dim, value dim, kv latent, q latent (0: direct), ff, layers, vocab,
    #        Gorozen head size, Gorozen kv heads)
    "2.5k wide, 40 heads, latent 256": (2560, 40, 64, 32, 64, 256, 768, 6400, 4, 32768, 96, 8),
    "2k wide, 16 heads, latent 128": (2048, 16, 64, 64, 64, 128, 0, 6144, 4, 32768, 128, 8),
}


class GraphTimer(Timer):
    """Times ``fn`` replayed from a CUDA graph: the single kernels here run for tens of microseconds, less than the host
    needs to issue them (allocation of the outputs, the ctypes call), so an eagerly timed call would measure the host."""

    def __call__(self, fn, steps, warmup):
        for _ in range(max(3, warmup)):
            fn()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            fn()
        return super().__call__(g.replay, steps, warmup)


def segorax_config(width, heads, dim, rot, vdim, kv_rank, q_rank, ff, layers, vocab, moe=False):
    kind = "latent_attention" if q_rank else "latent_attention_2"
    r = {"base": 10000.0, "dims": rot}
    mixer = {"dim": dim, "heads": heads, "kv_rank": kv_rank, "rot": r, "rot_dim": rot, "scale": (dim + rot) ** -0.5, "vdim": vdim}
    if q_rank:
        mixer["q_rank"] = q_rank
    else:
        r["scaling"] = {"factor": 4.0, "original": 4096, "fast": 32.0, "slow": 1.0}
    mlp = ({"kind": "moe", "expert": {"ff": ff // 4}, "router": {"experts": 16, "top": 4, "groups": {"count": 4, "keep": 2}},
            "shared": {"ff": ff // 4}} if moe else {"kind": "dense", "ff": ff})
    return {"architecture": "Segorax", "embedding": {"scale": width ** 0.5}, "layers": [{"type": kind, "mixer": mixer, "mlp": mlp}] * layers,
            "logit_scale": 0.5, "norm": {"eps": 1e-6}, "residual_mult": 0.5, "vocab": vocab, "width": width}


def build_models(size, dev, moe=False):
    from llm_in_practise_b200.models.gorozen import GorozenConfig, GorozenForCausalLM
    from llm_in_practise_b200.models.segorax import SegoraxConfig, SegoraxForCausalLM
    W, H, D, R, Dv, C, Cq, F, L, V, gD, gG = SIZES[size]
    torch.manual_seed(0)
    sg = SegoraxForCausalLM(SegoraxConfig.from_dict(segorax_config(W, H, D, R, Dv, C, Cq, F, L, V, moe)), dtype=torch.bfloat16, device=dev).eval()
    for n, p in sg.named_parameters():
        if p.dim() == 1 and p.dtype == torch.bfloat16:
            p.data.normal_(mean=1.0, std=0.1)
        elif n.endswith(("w_uk", "w_uv", "experts_up", "experts_down")):
            p.data.normal_(std=0.02)
        elif n.endswith("router"):
            p.data.normal_(std=0.05)
    gz = GorozenForCausalLM(GorozenConfig.from_dict(gorozen_config(W, H, gG, gD, F, L, V, moe)), dtype=torch.bfloat16, device=dev).eval()
    for p in gz.parameters():
        if p.dim() == 1 and p.dtype == torch.bfloat16:
            p.data.normal_(std=0.1)
    return sg, gz


@torch.no_grad()
def end_to_end(size, dev, steps, warmup, prompt=2048, batch=32, ctx=1024, moe=False):
    """tokens/s of (a) one prompt of ``prompt`` tokens, (b) one decode step of ``batch`` sequences at context ``ctx``."""
    from llm_in_practise_b200.inference import RaggedGenerator
    t = Timer(dev, flush=False)
    out = {}
    V = SIZES[size][9]
    toks = torch.randint(0, V, (prompt,)).tolist()
    for name, model in zip(("segorax", "gorozen"), build_models(size, dev, moe)):
        g = RaggedGenerator(model, None, max(prompt, ctx + 64))
        per = -(-max(prompt, ctx + 64) // 64)
        cache = g.make_cache(batch * per, 64, batch, per * 64)
        for b in range(batch):
            g.set_block_row(cache, b, list(range(1 + b * per, 1 + (b + 1) * per)))
        ms = t(lambda: g.step([(0, 0, toks, [prompt - 1])], cache), steps, warmup)
        out[f"{name}_prefill_tok_s"] = prompt / ms * 1e3
        last = [1] * batch
        ms = t(lambda: g.decode(last, [ctx] * batch, list(range(batch)), cache), steps * 4, warmup)
        out[f"{name}_decode_tok_s"] = batch / ms * 1e3
        out[f"{name}_decode_ms"] = ms
        out[f"{name}_kv_bytes_per_token"] = g.kv_token_bytes()
        del g, cache, model
        torch.cuda.empty_cache()
    return out


@torch.no_grad()
def kernel_rows(size, dev, steps, warmup, root):
    """Single kernels at the layer sizes: (name, Segorax ms, fraction of roofline, Gorozen like-kernel, ms, fraction, bound)."""
    from llm_in_practise_b200.inference.ragged import TILE_Q, Pieces
    from llm_in_practise_b200.ops import elementwise as ew
    from llm_in_practise_b200.ops.latent_attention import latent_attention, latent_kv_store, latent_q_rope
    from llm_in_practise_b200.ops.moe import route_sigmoid_grouped, route_topk
    from llm_in_practise_b200.ops.norm import sandwich_norm
    from llm_in_practise_b200.ops.paged_attention import paged_attention, rope_paged_store
    hbm, tf, which = _peaks(root)
    W, H, D, R, Dv, C, Cq, F, L, V, gD, gG = SIZES[size]
    Dk = C + R
    t = GraphTimer(dev)
    rows = []
    bf = torch.bfloat16
    T = 4096

    def frac_bw(nbytes, ms):
        return nbytes / (ms * 1e-3) / 1e9 / hbm

    def frac_fl(flops, ms):
        return flops / (ms * 1e-3) / 1e12 / tf

    def frac_both(nbytes, flops, ms):
        """Against the slower of the two bounds (a latent cache is read once for all heads, so the bound may be either)."""
        return max(nbytes / (hbm * 1e9), flops / (tf * 1e12)) / (ms * 1e-3)

    # --- post-norm + residual (+ cast for the next GEMM) vs post-norm + residual + pre-norm
    y32, res = torch.randn(T, W, device=dev), torch.randn(T, W, device=dev)
    w1, w2 = torch.ones(W, dtype=bf, device=dev), torch.zeros(W, dtype=bf, device=dev)
    ms_s = t(lambda: sandwich_norm(y32, w1, res, None, 1e-6, 0.0, bf, branch_mult=0.5, cast_next=True), steps, warmup)
    ms_g = t(lambda: sandwich_norm(y32, w2, res, w2, 1e-6, 1.0, bf), steps, warmup)
    rows.append(("post-norm + scaled residual add + cast", ms_s, frac_bw(T * W * 14, ms_s), "post-norm + residual + pre-norm", ms_g,
                 frac_bw(T * W * 14, ms_g), "HBM"))
    # --- latent norms + rotary + cache row store (+ query rotary) vs rotary + K/V page store
    BS = 64
    nb = T // BS
    cache = torch.zeros(nb + 1, 1, BS, Dk, dtype=bf, device=dev)
    table = torch.arange(1, nb + 1, dtype=torch.int32, device=dev).view(1, nb)
    pos = torch.arange(T, dtype=torch.int32, device=dev)
    slot = torch.zeros(T, dtype=torch.int32, device=dev)
    proj = torch.randn(T, Cq + Dk, device=dev)
    wq, wkv = torch.ones(max(Cq, 1), dtype=bf, device=dev), torch.ones(C, dtype=bf, device=dev)
    cos, sin = ew.rope_tables_partial(T, R, 1e4, dev)
    q = torch.randn(T, H * (D + R), device=dev).to(bf)
    qx = torch.randn(T, H, Dk, device=dev).to(bf)

    def seg_store():
        latent_kv_store(proj, 0, Cq, Cq, C, R, R, wq if Cq else None, wkv, 1e-6, cos, sin, pos, slot, cache, table, bf)
        latent_q_rope(q, cos, sin, pos, qx, H, D, R, R, C)
    ms_s = t(seg_store, steps, warmup)
    by_s = T * ((Cq + Dk) * 4 + (Cq + Dk) * 2 + H * R * 2 * 2)
    ck, cv = torch.zeros(nb + 1, gG, BS, gD, dtype=bf, device=dev), torch.zeros(nb + 1, gG, BS, gD, dtype=bf, device=dev)
    qk = torch.randn(T, (H + gG) * gD, device=dev).to(bf)
    cos2, sin2 = ew.rope_tables_partial(T, gD, 1e6, dev)
    ms_g = t(lambda: rope_paged_store(qk, cos2, sin2, pos, slot, ck, cv, table, H, gG, gD, gD, True, True), steps, warmup)
    rows.append(("latent norms + rotary + cache row store, query rotary", ms_s, frac_bw(by_s, ms_s), "rotary + K/V page store", ms_g,
                 frac_bw(T * ((H + gG) * gD * 2 * 2 + 2 * gG * gD * 2), ms_g), "HBM"))
    # --- prompt attention: 4096 tokens of one sequence, causal
    tiles = torch.tensor([[q0, min(TILE_Q, T - q0), q0, 0] for q0 in range(0, T, TILE_Q)], dtype=torch.int32, device=dev)
    pieces = Pieces(tiles, tiles.shape[0], T)
    sinks = torch.zeros(H, device=dev)
    cache.normal_()
    ms_s = t(lambda: latent_attention(qx, cache, table, pos, slot, H, C, Dk ** -0.5, sinks=sinks, max_pos=T - 1, pieces=pieces), steps, warmup)
    ck.normal_()
    cv.normal_()
    ms_g = t(lambda: paged_attention(qk, ck, cv, table, pos, slot, H, gG, gD, gD ** -0.5, sinks=sinks, max_pos=T - 1, pieces=pieces), steps, warmup)
    rows.append(("prompt attention over latent rows (mma.sync)", ms_s, frac_fl(2 * H * (Dk + C) * T * T / 2, ms_s),
                 "prompt attention (paged, sinks, mma.sync)", ms_g, frac_fl(4 * H * gD * T * T / 2, ms_g), "bf16 tensor"))
    # --- decode attention: 64 sequences at context 4032
    Bq, ctx = 64, 4032
    nbd = Bq * (ctx // BS + 1)
    cached = torch.randn(nbd + 1, 1, BS, Dk, device=dev).to(bf)
    tabd = torch.arange(1, nbd + 1, dtype=torch.int32, device=dev).view(Bq, -1)
    posd = torch.full((Bq,), ctx, dtype=torch.int32, device=dev)
    slotd = torch.arange(Bq, dtype=torch.int32, device=dev)
    qd = torch.randn(Bq, H, Dk, device=dev).to(bf)
    ms_s = t(lambda: latent_attention(qd, cached, tabd, posd, slotd, H, C, Dk ** -0.5, sinks=sinks, max_pos=ctx), steps, warmup)
    del cached
    ckd, cvd = torch.randn(nbd + 1, gG, BS, gD, device=dev).to(bf), torch.randn(nbd + 1, gG, BS, gD, device=dev).to(bf)
    qgd = torch.randn(Bq, (H + gG) * gD, device=dev).to(bf)
    ms_g = t(lambda: paged_attention(qgd, ckd, cvd, tabd, posd, slotd, H, gG, gD, gD ** -0.5, sinks=sinks, max_pos=ctx), steps, warmup)
    rows.append(("decode attention over latent rows", ms_s, frac_both(Bq * (ctx + 1) * Dk * 2, 2 * Bq * H * (ctx + 1) * (Dk + C), ms_s),
                 "decode attention (paged, sinks)", ms_g, frac_bw(Bq * gG * (ctx + 1) * gD * 2 * 2, ms_g), "HBM / bf16 tensor, the slower"))
    del ckd, cvd
    # --- gated activation
    gu = torch.randn(T, 2 * F, device=dev).to(bf)
    ms_s = t(lambda: ew.act_glu(gu, "gelu_tanh"), steps, warmup)
    ms_g = t(lambda: ew.clamped_glu(gu, 7.0, 1.702, 1.0), steps, warmup)
    rows.append(("tanh-GELU gated unit", ms_s, frac_bw(T * F * 2 * 3, ms_s), "clamped gated unit", ms_g, frac_bw(T * F * 2 * 3, ms_g), "HBM"))
    # --- router: 64 experts
    E = 64
    h = torch.randn(T, W, device=dev).to(bf)
    wr, corr = torch.randn(E + 1, W, device=dev) * 0.05, torch.randn(E, device=dev) * 0.1
    ms_s = t(lambda: route_sigmoid_grouped(h, wr, corr, 6, 8, 4, 2, gate_rows=1), steps, warmup)
    ms_g = t(lambda: route_topk(h, wr[:E], corr, 6), steps, warmup)
    rows.append(("sigmoid router, 8 groups keep 4, shared gate", ms_s, frac_bw(T * W * 2, ms_s), "top-k softmax router", ms_g, frac_bw(T * W * 2, ms_g), "HBM"))
    return rows, which


def run(args, root):
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    from llm_in_practise_b200.ops import _native as nv
    nv.lib()
    n0 = nv.launch_count
    t0 = time.time()
    res = {"metric": "Segorax vs Gorozen at equal layer sizes: prefill / decode tok/s", "unit": "tok/s", "n_gpus": 1,
           "steps": args.steps, "warmup": max(3, args.warmup), "dtype": "bf16", "data": "synthetic", "sizes": {}, "kernels": {}}
    first = next(iter(SIZES))
    for size in SIZES:
        res["sizes"][size] = {k: round(v, 2) for k, v in end_to_end(size, dev, args.steps, args.warmup).items()}
        torch.cuda.empty_cache()
    moe = end_to_end(first, dev, args.steps, args.warmup, moe=True)
    res["sizes"][first + ", 16 experts top 4"] = {k: round(v, 2) for k, v in moe.items()}
    torch.cuda.empty_cache()
    for size in SIZES:
        rows, which = kernel_rows(size, dev, args.steps, args.warmup, root)
        res["kernels"][size] = [{"segorax": a, "ms": round(b, 4), "of_roofline": round(c, 3), "gorozen": d, "gorozen_ms": round(e, 4),
                                 "gorozen_of_roofline": round(f, 3), "bound": g, "gap_ratio": round(f / c, 2) if c else None}
                                for a, b, c, d, e, f, g in rows]
        res["roofline"] = which
        torch.cuda.empty_cache()
    res["gpu_launches"] = nv.launch_count - n0
    res["seconds"] = round(time.time() - t0, 1)
    res["value"] = res["sizes"][first]["segorax_decode_tok_s"]
    res["config"] = {"model": "segorax dense, 4 layers of each size", "sizes": {k: list(v) for k, v in SIZES.items()},
                     "l2": "single kernels: replayed from a CUDA graph, 256 MB flush between iterations; steps: weights + cache exceed L2"}
    print(json.dumps(res))
    return 0
