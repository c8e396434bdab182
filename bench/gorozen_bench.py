"""Gorozen beside Qwen3 at equal layer sizes (random weights): prefill and decode throughput through each model's own
generator, and the time of each Gorozen kernel next to the Qwen3 kernel that does the like job, as fractions of the measured
roofline (``MEASURED_PEAKS.json``: copy bandwidth and cuBLAS bf16 rate of this pool's B200).

    python bench.py --workload gorozen [--steps K --warmup W]

Timing: CUDA events on the launching stream, W >= 3 warm-up iterations, an L2 flush (a 256 MB write) between timed
iterations of the single-kernel rows; the end-to-end rows run steps whose weights and caches together exceed L2.
"""
from __future__ import annotations

import json
import math
import os
import statistics
import time

import torch

SIZES = {
    # name: (width, heads, kv heads, head size, ff, layers, vocab)
    "1.7b-like": (2048, 16, 8, 128, 6144, 4, 32768),
    "8b-like": (4096, 32, 8, 128, 12288, 4, 32768),
}


def _peaks(root):
    try:
        with open(os.path.join(root, "MEASURED_PEAKS.json")) as f:
            d = json.load(f)
        return d["hbm_gbs"], d["bf16_tflops"], "measured"
    except Exception:
        return 6650.0, 1590.0, "fallback"


def gorozen_config(width, heads, kv, dim, ff, layers, vocab, moe=False):
    rot = {"base": 1000000.0, "dims": dim, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}
    mlp = ({"kind": "moe", "expert": {"ff": ff // 4}, "router": {"experts": 16, "top": 4}} if moe
           else {"kind": "dense", "ff": ff, "limit": 7.0})
    layer = {"type": "attention", "mixer": {"dim": dim, "heads": heads, "kv_heads": kv, "vdim": dim, "rot": rot, "scale": dim ** -0.5}, "mlp": mlp}
    return {"architecture": "Gorozen", "layers": [layer] * layers, "logit_softcap": 30.0, "norm": {"eps": 1e-6}, "vocab": vocab, "width": width}


class Timer:
    def __init__(self, dev, flush=True):
        self.flush_buf = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev) if flush else None

    def __call__(self, fn, steps, warmup):
        for _ in range(max(3, warmup)):
            fn()
        ts = []
        for _ in range(steps):
            if self.flush_buf is not None:
                self.flush_buf.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b))
        return statistics.median(ts)


def build_models(size, dev, moe=False):
    from llm_in_practise_b200.models.gorozen import GorozenConfig, GorozenForCausalLM
    from llm_in_practise_b200.models.qwen3 import Qwen3Config, Qwen3ForCausalLM
    W, H, G, D, F, L, V = SIZES[size]
    torch.manual_seed(0)
    gz = GorozenForCausalLM(GorozenConfig.from_dict(gorozen_config(W, H, G, D, F, L, V, moe)), dtype=torch.bfloat16, device=dev).eval()
    for p in gz.parameters():
        if p.dim() == 1 and p.dtype == torch.bfloat16:
            p.data.normal_(std=0.1)
    qw = Qwen3ForCausalLM(Qwen3Config(vocab_size=V, hidden_size=W, intermediate_size=F, num_hidden_layers=L, num_attention_heads=H,
                                      num_key_value_heads=G, head_dim=D, max_position_embeddings=8192), dtype=torch.bfloat16, device=dev).eval()
    return gz, qw


@torch.no_grad()
def end_to_end(size, dev, steps, warmup, prompt=2048, batch=32, ctx=1024, moe=False):
    """tokens/s of (a) one prompt of ``prompt`` tokens, (b) one decode step of ``batch`` sequences at context ``ctx``."""
    from llm_in_practise_b200.inference import Generator, KVCache, RaggedGenerator
    gz, qw = build_models(size, dev, moe)
    W, H, G, D, F, L, V = SIZES[size]
    t = Timer(dev, flush=False)
    out = {}
    toks = torch.randint(0, V, (prompt,)).tolist()
    # ---- Gorozen
    g = RaggedGenerator(gz, None, max(prompt, ctx + 64))
    per = -(-max(prompt, ctx + 64) // 64)
    cache = g.make_cache(batch * per, 64, batch, per * 64)
    for b in range(batch):
        g.set_block_row(cache, b, list(range(1 + b * per, 1 + (b + 1) * per)))
    ms = t(lambda: g.step([(0, 0, toks, [prompt - 1])], cache), steps, warmup)
    out["gorozen_prefill_tok_s"] = prompt / ms * 1e3
    last = [1] * batch
    ms = t(lambda: g.decode(last, [ctx] * batch, list(range(batch)), cache), steps * 4, warmup)
    out["gorozen_decode_tok_s"] = batch / ms * 1e3
    out["gorozen_decode_ms"] = ms
    del g, cache
    # ---- Qwen3, same sizes
    q = Generator(qw, None, max(prompt, ctx + 64))
    kv = KVCache(L, batch + 1, G, max(prompt, ctx + 64), D, torch.bfloat16, dev)
    ids = torch.tensor([toks], device=dev)
    ms = t(lambda: q._prefill(ids, kv, torch.zeros(1, dtype=torch.long, device=dev)), steps, warmup)
    out["qwen3_prefill_tok_s"] = prompt / ms * 1e3
    tok = torch.ones(batch, dtype=torch.long, device=dev)
    pos = torch.full((batch,), ctx, dtype=torch.int32, device=dev)
    slots = torch.arange(batch, dtype=torch.int32, device=dev)
    ms = t(lambda: q.decode_graphed(tok, kv, pos, slots), steps * 4, warmup)
    out["qwen3_decode_tok_s"] = batch / ms * 1e3
    out["qwen3_decode_ms"] = ms
    return out


@torch.no_grad()
def kernel_rows(size, dev, steps, warmup, root):
    """Single kernels at the layer sizes: (name, Gorozen ms, fraction of roofline, Qwen3 like-kernel ms, fraction)."""
    from llm_in_practise_b200.inference.generate import KVCache, _decode_attn
    from llm_in_practise_b200.inference.ragged import TILE_Q, Pieces
    from llm_in_practise_b200.ops import elementwise as ew
    from llm_in_practise_b200.ops.flash import flash_attention_varlen
    from llm_in_practise_b200.ops.norm import rms_norm, sandwich_norm
    from llm_in_practise_b200.ops.paged_attention import paged_attention, rope_paged_store
    hbm, tf, which = _peaks(root)
    W, H, G, D, F, L, V = SIZES[size]
    t = Timer(dev)
    rows = []
    bf = torch.bfloat16
    T = 4096

    def frac_bw(nbytes, ms):
        return nbytes / (ms * 1e-3) / 1e9 / hbm

    def frac_fl(flops, ms):
        return flops / (ms * 1e-3) / 1e12 / tf

    # --- norms: sandwich (reads y fp32 + stream fp32, writes stream fp32 + h bf16) vs add + RMSNorm on a 16-bit stream
    y32, res = torch.randn(T, W, device=dev), torch.randn(T, W, device=dev)
    w1, w2 = torch.zeros(W, dtype=bf, device=dev), torch.zeros(W, dtype=bf, device=dev)
    ms_g = t(lambda: sandwich_norm(y32, w1, res, w2, 1e-6, 1.0, bf), steps, warmup)
    y16, r16 = y32.to(bf), res.to(bf)
    ms_q = t(lambda: rms_norm(y16, w1, 1e-6, r16), steps, warmup)
    rows.append(("post-norm + residual + pre-norm", ms_g, frac_bw(T * W * (4 + 4 + 4 + 2), ms_g), "add + RMSNorm (16-bit stream)", ms_q,
                 frac_bw(T * W * 2 * 4, ms_q), "HBM"))
    # --- rotary + cache store vs qk-norm + rotary (+ the separate cache scatter Qwen3's prefill does)
    BS = 64
    nb = T // BS
    ck, cv = torch.zeros(nb + 1, G, BS, D, dtype=bf, device=dev), torch.zeros(nb + 1, G, BS, D, dtype=bf, device=dev)
    table = torch.arange(1, nb + 1, dtype=torch.int32, device=dev).view(1, nb)
    pos = torch.arange(T, dtype=torch.int32, device=dev)
    slot = torch.zeros(T, dtype=torch.int32, device=dev)
    qk = torch.randn(T, (H + G) * D, device=dev).to(bf)
    cos, sin = ew.rope_tables_partial(T, D, 1e6, dev)
    ms_g = t(lambda: rope_paged_store(qk, cos, sin, pos, slot, ck, cv, table, H, G, D, D, True, True), steps, warmup)
    qkv = torch.randn(T, (H + 2 * G) * D, device=dev).to(bf)
    qn, kn = torch.ones(D, dtype=bf, device=dev), torch.ones(D, dtype=bf, device=dev)
    cs2, sn2 = ew.rope_tables(T, D, 1e6, dev)
    kvc = KVCache(1, 1, G, T, D, bf, dev)

    def qwen_rope():
        o = ew.qknorm_rope(qkv, qn, kn, cs2, sn2, pos, H, G, D, False, 1e-6)
        tt = o.view(T, H + 2 * G, D)
        kvc.store(0, slot.long(), pos.long(), tt[:, H:H + G], tt[:, H + G:])
    ms_q = t(qwen_rope, steps, warmup)
    rows.append(("rotary + K/V page store", ms_g, frac_bw(T * ((H + G) * D * 2 * 2 + 2 * G * D * 2), ms_g), "qk-norm + rotary, cache scatter", ms_q,
                 frac_bw(T * ((H + 2 * G) * D * 2 * 2 + 4 * G * D * 2), ms_q), "HBM"))
    # --- prompt attention: 4096 tokens of one sequence, causal
    tiles = torch.tensor([[q0, min(TILE_Q, T - q0), q0, 0] for q0 in range(0, T, TILE_Q)], dtype=torch.int32, device=dev)
    pieces = Pieces(tiles, tiles.shape[0], T)
    sinks = torch.zeros(H, device=dev)
    ms_g = t(lambda: paged_attention(qk, ck, cv, table, pos, slot, H, G, D, D ** -0.5, sinks=sinks, max_pos=T - 1, pieces=pieces), steps, warmup)
    cu = torch.tensor([0, T], dtype=torch.int32, device=dev)
    ms_q = t(lambda: flash_attention_varlen(qkv, cu, T, H, G, D, D ** -0.5), steps, warmup)
    fl = 4 * H * D * T * T / 2
    rows.append(("prompt attention (paged, sinks, mma.sync)", ms_g, frac_fl(fl, ms_g), "varlen flash attention (mma.sync)", ms_q, frac_fl(fl, ms_q), "bf16 tensor"))
    # --- decode attention: 64 sequences at context 4032
    Bq, ctx = 64, 4032
    nbd = Bq * (ctx // BS + 1)
    ckd, cvd = torch.randn(nbd + 1, G, BS, D, device=dev).to(bf), torch.randn(nbd + 1, G, BS, D, device=dev).to(bf)
    tabd = torch.arange(1, nbd + 1, dtype=torch.int32, device=dev).view(Bq, -1)
    posd = torch.full((Bq,), ctx, dtype=torch.int32, device=dev)
    slotd = torch.arange(Bq, dtype=torch.int32, device=dev)
    qd = torch.randn(Bq, (H + G) * D, device=dev).to(bf)
    ms_g = t(lambda: paged_attention(qd, ckd, cvd, tabd, posd, slotd, H, G, D, D ** -0.5, sinks=sinks, max_pos=ctx), steps, warmup)
    kq = torch.randn(Bq, G, ctx + 64, D, device=dev).to(bf)
    vq = torch.randn(Bq, G, ctx + 64, D, device=dev).to(bf)
    qkvd = torch.randn(Bq, (H + 2 * G) * D, device=dev).to(bf)
    ms_q = t(lambda: _decode_attn(qkvd, kq, vq, posd, H, G, D, D ** -0.5, slotd), steps, warmup)
    by = Bq * G * (ctx + 1) * D * 2 * 2
    rows.append(("decode attention (paged, sinks)", ms_g, frac_bw(by, ms_g), "decode attention (slot rows, split)", ms_q, frac_bw(by, ms_q), "HBM"))
    # --- gated activation
    gu = torch.randn(T, 2 * F, device=dev).to(bf)
    ms_g = t(lambda: ew.clamped_glu(gu, 7.0, 1.702, 1.0), steps, warmup)
    ms_q = t(lambda: ew.swiglu(gu), steps, warmup)
    rows.append(("clamped gated unit", ms_g, frac_bw(T * F * 2 * 3, ms_g), "SwiGLU", ms_q, frac_bw(T * F * 2 * 3, ms_q), "HBM"))
    return rows, which


def run(args, root):
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    from llm_in_practise_b200.ops import _native as nv
    nv.lib()
    n0 = nv.launch_count
    t0 = time.time()
    res = {"metric": "Gorozen vs Qwen3 at equal layer sizes: prefill / decode tok/s", "unit": "tok/s", "n_gpus": 1,
           "steps": args.steps, "warmup": max(3, args.warmup), "dtype": "bf16", "data": "synthetic", "sizes": {}, "kernels": {}}
    for size in SIZES:
        res["sizes"][size] = {k: round(v, 2) for k, v in end_to_end(size, dev, args.steps, args.warmup).items()}
        torch.cuda.empty_cache()
    moe = end_to_end("1.7b-like", dev, args.steps, args.warmup, moe=True)
    res["sizes"]["1.7b-like, 16 experts top 4"] = {k: round(v, 2) for k, v in moe.items() if k.startswith("gorozen")}
    torch.cuda.empty_cache()
    for size in SIZES:
        rows, which = kernel_rows(size, dev, args.steps, args.warmup, root)
        res["kernels"][size] = [{"gorozen": a, "ms": round(b, 4), "of_roofline": round(c, 3), "qwen3": d, "qwen3_ms": round(e, 4),
                                 "qwen3_of_roofline": round(f, 3), "bound": g, "gap_ratio": round(f / c, 2) if c else None}
                                for a, b, c, d, e, f, g in rows]
        res["roofline"] = which
        torch.cuda.empty_cache()
    res["gpu_launches"] = nv.launch_count - n0
    res["seconds"] = round(time.time() - t0, 1)
    res["value"] = res["sizes"]["8b-like"]["gorozen_decode_tok_s"]
    res["config"] = {"model": "gorozen dense, 4 layers of each size", "sizes": {k: list(v) for k, v in SIZES.items()},
                     "l2": "single kernels: 256 MB flush between iterations; steps: weights + cache exceed L2"}
    print(json.dumps(res))
    return 0
