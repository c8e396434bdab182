"""Gorozen against the plain float64 oracle in ``gorozen_oracle.py``: every mechanism alone, then the model through the ragged
step, the serving engine's block / slot pools and its scheduler. Small random models of several shapes; the same tests run
on the CPU path and (marked ``gpu``) on the CUDA kernels in fp32 and bf16."""
import json

import pytest
import torch

import gorozen_oracle as O

CASES = [("cpu", torch.float32), pytest.param("cuda", torch.float32, marks=pytest.mark.gpu),
         pytest.param("cuda", torch.bfloat16, marks=pytest.mark.gpu)]


def tol(dtype):
    return 2e-4 if dtype == torch.float32 else 6e-2


def rel_err(got, want):
    """RMS difference over RMS of the oracle, means over the last axis removed (a shift of all logits changes nothing)."""
    got, want = got.double().cpu(), want.double().cpu()
    d = got - want
    d = d - d.mean(-1, keepdim=True)
    w = want - want.mean(-1, keepdim=True)
    return float(d.pow(2).mean().sqrt() / w.pow(2).mean().sqrt())


def row_errs(got, want):
    got, want = got.double().cpu(), want.double().cpu()
    d = got - want
    d = d - d.mean(-1, keepdim=True)
    w = want - want.mean(-1, keepdim=True)
    return d.pow(2).mean(-1).sqrt() / w.pow(2).mean().sqrt()


def assert_rows(got, want, dtype, what=""):
    """Every position against the oracle. In fp32 each row must agree. In 16 bits a router logit that the oracle decides by a
    hair can fall the other way and move that token's row by far more than rounding, so there the bulk of the rows is held
    to the tolerance (nine in ten, and the median to half of it) — the logic itself is pinned by the fp32 run."""
    e = row_errs(got, want)
    if dtype == torch.float32:
        assert float(e.max()) < tol(dtype), (what, float(e.max()), int(e.argmax()))
    else:
        assert float(e.quantile(0.9)) < tol(dtype) and float(e.median()) < tol(dtype) / 2, (what, float(e.quantile(0.9)), float(e.median()))


def build(tmp_path, cfg, W, device, dtype, name="m"):
    from llm_in_practise_b200.io.hf import from_pretrained
    from llm_in_practise_b200.io.safetensors import save_file
    d = tmp_path / name
    d.mkdir(exist_ok=True)
    (d / "config.json").write_text(json.dumps(cfg))
    save_file(W, str(d / "model.safetensors"))
    return from_pretrained(str(d), dtype=dtype, device=torch.device(device))


def fresh_cache(gen, n_seqs, max_len, block=64, order=None):
    """A cache whose rows list their blocks in a scrambled physical order."""
    per = -(-max_len // block)
    cache = gen.make_cache(n_seqs * per, block, n_seqs, per * block)
    ids = list(range(1, n_seqs * per + 1))
    if order is None:
        ids = ids[::-1]
    for s in range(n_seqs):
        gen.set_block_row(cache, s, ids[s::n_seqs][:per])
    return cache


SCALING = {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}      # with base 100 and 16 dims: all three bands occur

VARIANTS = {
    "mixed": lambda: O.make_config(64, 96, [O.attn_layer(4, 2, 32, 16, 100.0, SCALING, mlp=O.dense()),
                                            O.attn_layer(4, 2, 32, 16, 100.0, SCALING, mlp=O.moe(4, 2, 48)),
                                            O.attn_layer(4, 2, 32, 16, 100.0, SCALING, mlp=None)]),
    "mha_fullrot": lambda: O.make_config(48, 80, [O.attn_layer(3, 3, 16, 16, 50.0, None, scale=0.3, mlp=O.moe(3, 3, 24)),
                                                  O.attn_layer(6, 1, 16, 8, 1000.0, None, mlp=O.dense(40, 0.7))], softcap=None),
    "odd_heads": lambda: O.make_config(40, 64, [O.attn_layer(2, 1, 24, 4, 10.0, None, mlp=O.moe(5, 1, 16)),
                                                O.attn_layer(8, 4, 48, 0, 10.0, None, mlp=O.dense(56, 3.0))], eps=1e-3, softcap=5.0),
}


SC2 = {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 128}
# sizes that are not multiples of the kernels' vector widths: width % 8 != 0 (no TMA rows), odd vocabulary, head sizes that
# are not whole 16-byte chunks, 3 / 5 / 10 heads, 7 experts
ODD = {
    "w72": lambda: O.make_config(72, 75, [O.attn_layer(3, 1, 40, 10, 1e4, SC2, mlp=O.dense(100, 1.5)),
                                          O.attn_layer(3, 1, 40, 10, 1e4, SC2, mlp=O.moe(3, 2, 36))]),
    "w100": lambda: O.make_config(100, 130, [O.attn_layer(5, 5, 36, 36, 1e6, None, mlp=O.moe(7, 3, 52)),
                                             O.attn_layer(10, 2, 20, 2, 1e6, None, mlp=O.dense(90, 9.0))], softcap=50.0),
}


# ------------------------------------------------------------------------------------------------------------------
# mechanisms alone
# ------------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("device,dtype", CASES)
def test_sandwich_norm(device, dtype):
    from llm_in_practise_b200.ops.norm import sandwich_norm
    g = torch.Generator().manual_seed(1)
    n, W, eps = 5, 72, 1e-5
    y, res = torch.randn(n, W, generator=g) * 3, torch.randn(n, W, generator=g)
    wp, wn = (torch.randn(W, generator=g) * 0.3).to(dtype), (torch.randn(W, generator=g) * 0.3).to(dtype)
    h, x = sandwich_norm(y.to(device), wp.to(device), res.to(device), wn.to(device), eps, 1.0, dtype)
    x_ref = res.double() + O.norm(y.double(), wp.double(), eps)
    assert x.dtype == torch.float32
    torch.testing.assert_close(x.cpu().double(), x_ref, rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(h.cpu().double(), O.norm(x_ref, wn.double(), eps), rtol=tol(dtype) / 4, atol=tol(dtype) / 4)
    # entering the stream (no post-norm, no residual) and leaving it (no next norm)
    h0, x0 = sandwich_norm(y.to(device, dtype), None, None, wn.to(device), eps, 1.0, dtype)
    torch.testing.assert_close(x0.cpu(), y.to(dtype).float())
    h1, x1 = sandwich_norm(y.to(device), wp.to(device), res.to(device), None, eps, 1.0, dtype)
    assert h1 is None
    torch.testing.assert_close(x1.cpu().double(), x_ref, rtol=1e-5, atol=1e-5)


def test_rotary_bands_all_present():
    rot = {"base": 100.0, "dims": 16, "scaling": SCALING}
    f0 = O.rotary_frequencies({"base": 100.0, "dims": 16})
    f = O.rotary_frequencies(rot)
    ratio = (f / f0).tolist()
    assert any(abs(r - 1.0) < 1e-12 for r in ratio) and any(abs(r - 1 / 8) < 1e-12 for r in ratio)
    assert any(1 / 8 + 1e-6 < r < 1 - 1e-6 for r in ratio)


@pytest.mark.parametrize("device,dtype", CASES)
@pytest.mark.parametrize("D,R,scaling", [(32, 16, SCALING), (24, 24, None), (20, 6, None), (16, 0, None)])
def test_rope_paged_store(device, dtype, D, R, scaling):
    from llm_in_practise_b200.models.gorozen import _hf_rope_scaling
    from llm_in_practise_b200.ops.elementwise import rope_tables_partial
    from llm_in_practise_b200.ops.paged_attention import rope_paged_store
    g = torch.Generator().manual_seed(2)
    H, G, BS = 4, 2, 8
    positions = [0, 1, 7, 8, 9, 63, 200, 1023]
    slots = [1, 0, 1, 1, 0, 0, 1, 0]
    n = len(positions)
    qk = torch.randn(n, (H + G) * D, generator=g).to(dtype)
    rot = {"base": 100.0, "dims": R}
    if scaling:
        rot["scaling"] = scaling
    if R:
        cos, sin = rope_tables_partial(1024, R, 100.0, device, _hf_rope_scaling(scaling))
    else:
        cos = sin = torch.zeros(1, 1, device=device)
    nb = 2 * 128
    ck = torch.zeros(nb + 1, G, BS, D, dtype=dtype, device=device)
    cv = torch.zeros_like(ck)
    table = (torch.randperm(nb, generator=g).view(2, 128) + 1).to(torch.int32).to(device)
    out = rope_paged_store(qk.clone().to(device), cos, sin, torch.tensor(positions, dtype=torch.int32, device=device),
                           torch.tensor(slots, dtype=torch.int32, device=device), ck, cv, table, H, G, D, R, interleaved=True, v_from_k=True)
    x = qk.double().view(n, H + G, D)
    ref = O.rotate(x, positions, rot)
    t = tol(dtype) / 4
    torch.testing.assert_close(out.cpu().double().view(n, H + G, D), ref, rtol=t, atol=t)
    for i, (p, s) in enumerate(zip(positions, slots)):
        blk = int(table[s, p // BS])
        torch.testing.assert_close(ck[blk, :, p % BS].cpu().double(), ref[i, H:], rtol=t, atol=t)
        torch.testing.assert_close(cv[blk, :, p % BS].cpu().double(), x[i, H:], rtol=0, atol=0)      # values: the un-rotated keys


def _fill_cache(k, v, BS, device, dtype, seed=0):
    """k, v [n, G, D] of ONE sequence -> (cache_k, cache_v, table) with scrambled pages, sequence in row 1 of 2."""
    n, G, D = k.shape
    nb = -(-n // BS)
    perm = torch.randperm(nb + 3, generator=torch.Generator().manual_seed(seed))[:nb] + 1
    ck = torch.full((nb + 5, G, BS, D), float("nan"), dtype=dtype, device=device)       # unread pages hold NaN
    cv = torch.full_like(ck, float("nan"))
    table = torch.zeros(2, nb, dtype=torch.int32, device=device)
    table[1] = perm.to(torch.int32)
    for j in range(nb):
        lo, hi = j * BS, min(n, (j + 1) * BS)
        ck[perm[j], :, :hi - lo] = k[lo:hi].transpose(0, 1).to(device, dtype)
        cv[perm[j], :, :hi - lo] = v[lo:hi].transpose(0, 1).to(device, dtype)
        ck[perm[j], :, hi - lo:] = 0          # the tail of the last page is never a valid key; finite filler
        cv[perm[j], :, hi - lo:] = 0
    return ck, cv, table


def _pieces(device, runs):
    from llm_in_practise_b200.inference.ragged import TILE_Q, Pieces
    tiles, base = [], 0
    for pos0, n in runs:
        for q0 in range(0, n, TILE_Q):
            tiles.append([base + q0, min(TILE_Q, n - q0), pos0 + q0, 1])
        base += n
    return Pieces(torch.tensor(tiles, dtype=torch.int32, device=device), len(tiles), max(n for _, n in runs))


@pytest.mark.parametrize("device,dtype", CASES)
@pytest.mark.parametrize("H,G,D,BS", [(4, 2, 32, 64), (3, 3, 24, 16), (6, 2, 48, 64), (2, 1, 128, 32)])
def test_paged_attention_with_sinks(device, dtype, H, G, D, BS):
    from llm_in_practise_b200.ops.paged_attention import paged_attention
    g = torch.Generator().manual_seed(3)
    n = 150
    q = torch.randn(n, H, D, generator=g).to(dtype)
    k = torch.randn(n, G, D, generator=g).to(dtype)
    v = torch.randn(n, G, D, generator=g).to(dtype)
    sink = torch.randn(H, generator=g) * 2
    scale = 0.21
    ref = O.sink_softmax_attention(q.double(), k.double(), v.double(), scale, sink.double()).reshape(n, H * D)
    ck, cv, table = _fill_cache(k, v, BS, device, dtype)
    # (a) the last 90 positions as one piece over 60 cached ones, (b) the same positions one token at a time
    pos = torch.arange(60, n, dtype=torch.int32, device=device)
    slot = torch.ones_like(pos)
    qq = q[60:].reshape(-1, H * D).to(device)
    out = paged_attention(qq, ck, cv, table, pos, slot, H, G, D, scale, sinks=sink.to(device), max_pos=n - 1,
                          pieces=_pieces(device, [(60, n - 60)]))
    assert rel_err(out, ref[60:]) < tol(dtype) / 2
    assert float(row_errs(out, ref[60:]).max()) < tol(dtype) / 2          # no single row (a page border, the piece's start) is off
    for t in (0, 1, 63, 64, 65, n - 1):
        o1 = paged_attention(q[t:t + 1].reshape(1, H * D).to(device), ck, cv, table, torch.tensor([t], dtype=torch.int32, device=device),
                             torch.ones(1, dtype=torch.int32, device=device), H, G, D, scale, sinks=sink.to(device), max_pos=t)
        assert rel_err(o1, ref[t:t + 1]) < tol(dtype) / 2, t
    # without sinks the rows are plain softmax averages
    out0 = paged_attention(qq, ck, cv, table, pos, slot, H, G, D, scale, sinks=None, max_pos=n - 1, pieces=_pieces(device, [(60, n - 60)]))
    ref0 = O.sink_softmax_attention(q.double(), k.double(), v.double(), scale, torch.full((H,), -1e30, dtype=torch.float64)).reshape(n, H * D)
    assert rel_err(out0, ref0[60:]) < tol(dtype) / 2


@pytest.mark.parametrize("device,dtype", CASES)
@pytest.mark.parametrize("as_piece", [True, False])
def test_one_far_key_dominates(device, dtype, as_piece):
    """One key gets a score far above the rest: the output must be its value — for keys hundreds back, on both sides of a
    page border, the first key and the query's own; a dominant sink must leave (almost) nothing."""
    from llm_in_practise_b200.ops.paged_attention import paged_attention
    g = torch.Generator().manual_seed(4)
    H, G, D, BS, n = 2, 1, 32, 64, 700
    k = (torch.randn(n, G, D, generator=g) * 0.1)
    v = torch.randn(n, G, D, generator=g)
    qdir = torch.nn.functional.normalize(torch.randn(D, generator=g), dim=0)
    targets = {699: 0, 698: 63, 697: 64, 696: 65, 695: 127, 694: 128, 693: 300, 692: 692, 691: 690, 640: 639, 650: 1}
    q = torch.randn(n, H, D, generator=g) * 0.1
    for qp, kp in targets.items():
        q[qp] = qdir * 60
    kk = k.clone()
    vv = v.clone()
    sink = torch.zeros(H)
    # every target query gets its own copy of the cache with only ITS key boosted
    for qp, kp in targets.items():
        kb = kk.clone()
        kb[kp, 0] = qdir * 4
        ck, cv, table = _fill_cache(kb.to(dtype), vv.to(dtype), BS, device, dtype, seed=qp)
        if as_piece:
            lo = max(0, qp - 20)
            pos = torch.arange(lo, qp + 1, dtype=torch.int32, device=device)
            out = paged_attention(q[lo:qp + 1].reshape(-1, H * D).to(device, dtype), ck, cv, table, pos, torch.ones_like(pos), H, G, D, 1.0,
                                  sinks=sink.to(device), max_pos=qp, pieces=_pieces(device, [(lo, qp + 1 - lo)]))[-1]
        else:
            out = paged_attention(q[qp:qp + 1].reshape(1, H * D).to(device, dtype), ck, cv, table, torch.tensor([qp], dtype=torch.int32, device=device),
                                  torch.ones(1, dtype=torch.int32, device=device), H, G, D, 1.0, sinks=sink.to(device), max_pos=qp)[0]
        want = vv[kp, 0].to(dtype).float().repeat(H)
        torch.testing.assert_close(out.float().cpu(), want, rtol=2e-2, atol=2e-2, msg=f"query {qp} key {kp}")
    # a key one step in the future must not be seen: boost key qp + 1
    kb = kk.clone()
    kb[401, 0] = qdir * 4
    ck, cv, table = _fill_cache(kb.to(dtype), vv.to(dtype), BS, device, dtype)
    qq = (qdir * 60).repeat(H).view(1, H * D)
    seen = paged_attention(qq.to(device, dtype), ck, cv, table, torch.tensor([401], dtype=torch.int32, device=device),
                           torch.ones(1, dtype=torch.int32, device=device), H, G, D, 1.0, sinks=sink.to(device), max_pos=401)[0]
    unseen = paged_attention(qq.to(device, dtype), ck, cv, table, torch.tensor([400], dtype=torch.int32, device=device),
                             torch.ones(1, dtype=torch.int32, device=device), H, G, D, 1.0, sinks=sink.to(device), max_pos=400)[0]
    torch.testing.assert_close(seen.float().cpu(), vv[401, 0].to(dtype).float().repeat(H), rtol=2e-2, atol=2e-2)
    assert float((unseen.float().cpu() - vv[401, 0].repeat(H)).abs().max()) > 0.5
    big = paged_attention(qq.to(device, dtype), ck, cv, table, torch.tensor([400], dtype=torch.int32, device=device),
                          torch.ones(1, dtype=torch.int32, device=device), H, G, D, 1.0, sinks=torch.full((H,), 300.0, device=device), max_pos=400)[0]
    assert float(big.float().abs().max()) < 1e-3


@pytest.mark.parametrize("device,dtype", CASES)
def test_long_context_decode_splits(device, dtype):
    """A single token over thousands of keys (the key range is cut over several CTAs on the GPU) equals the oracle."""
    from llm_in_practise_b200.ops.paged_attention import paged_attention
    g = torch.Generator().manual_seed(5)
    H, G, D, BS, n = 4, 2, 32, 64, 2500
    k, v = torch.randn(n, G, D, generator=g).to(dtype), torch.randn(n, G, D, generator=g).to(dtype)
    q = torch.randn(1, H, D, generator=g).to(dtype)
    sink = torch.randn(H, generator=g)
    ck, cv, table = _fill_cache(k, v, BS, device, dtype)
    out = paged_attention(q.reshape(1, H * D).to(device), ck, cv, table, torch.tensor([n - 1], dtype=torch.int32, device=device),
                          torch.ones(1, dtype=torch.int32, device=device), H, G, D, 0.3, sinks=sink.to(device), max_pos=n - 1)
    qf = torch.zeros(n, H, D, dtype=torch.float64)
    qf[-1] = q[0].double()
    sc = torch.einsum("hd,nhd->hn", q[0].double(), k.double().repeat_interleave(H // G, 1)) * 0.3
    m = torch.maximum(sc.max(-1).values, sink.double())
    e = torch.exp(sc - m[:, None])
    ref = torch.einsum("hn,nhd->hd", e / (e.sum(-1) + torch.exp(sink.double() - m))[:, None], v.double().repeat_interleave(H // G, 1))
    assert rel_err(out, ref.reshape(1, H * D)) < tol(dtype) / 2


@pytest.mark.parametrize("device,dtype", CASES)
def test_clamped_glu_and_softcap(device, dtype):
    from llm_in_practise_b200.ops.elementwise import clamped_glu, softcap_
    g = torch.Generator().manual_seed(6)
    gu = (torch.randn(7, 2 * 36, generator=g) * 3).to(dtype)
    y = clamped_glu(gu.to(device), 1.5, 1.702, 1.0)
    a, b = gu[:, :36].double().clamp(max=1.5), gu[:, 36:].double().clamp(-1.5, 1.5)
    torch.testing.assert_close(y.cpu().double(), a * torch.sigmoid(1.702 * a) * (b + 1), rtol=tol(dtype) / 4, atol=tol(dtype) / 4)
    assert float(a.max()) == 1.5 and float(b.min()) == -1.5                        # the clamps were exercised
    y2 = clamped_glu(gu.to(device))                                                 # defaults: SwiGLU
    a, b = gu[:, :36].double(), gu[:, 36:].double()
    torch.testing.assert_close(y2.cpu().double(), a * torch.sigmoid(a) * b, rtol=tol(dtype) / 4, atol=tol(dtype) / 2)
    z = torch.randn(3, 50, generator=g) * 30
    torch.testing.assert_close(softcap_(z.clone().to(device), 15.0).cpu(), 15 * torch.tanh(z / 15), rtol=1e-5, atol=1e-5)
    assert torch.equal(softcap_(z.clone().to(device), None).cpu(), z)


@pytest.mark.parametrize("device,dtype", CASES)
@pytest.mark.parametrize("E,K", [(4, 2), (5, 1), (3, 3), (16, 4)])
def test_router_and_experts(device, dtype, E, K):
    from llm_in_practise_b200.ops.elementwise import clamped_glu
    from llm_in_practise_b200.ops.moe import gated_moe_ffn, route_topk
    g = torch.Generator().manual_seed(7)
    n, W, F = 9, 40, 24
    fc = {"router": {"experts": E, "top": K}, "expert": {"ff": F}}
    Wt = {"router": torch.randn(E, W, generator=g).to(torch.bfloat16), "router.b": torch.randn(E, generator=g).to(torch.bfloat16)}
    for e in range(E):
        Wt[f"e{e}.gate"], Wt[f"e{e}.up"] = (torch.randn(F, W, generator=g) * W ** -0.5).to(dtype), (torch.randn(F, W, generator=g) * W ** -0.5).to(dtype)
        Wt[f"e{e}.down"] = (torch.randn(W, F, generator=g) * F ** -0.5).to(dtype)
    h = torch.randn(n, W, generator=g).to(dtype)
    Wd = {k: v.double() for k, v in Wt.items()}
    idx_ref, w_ref = O.router(h.double(), Wd, "", fc)
    ti, tp = route_topk(h.to(device), Wt["router"].float().to(device), Wt["router.b"].float().to(device), K)
    assert tp.dtype == torch.float32
    assert torch.equal(ti.cpu(), idx_ref)
    torch.testing.assert_close(tp.cpu().double(), w_ref, rtol=1e-5, atol=1e-6)
    gu = torch.stack([torch.cat([Wt[f"e{e}.gate"], Wt[f"e{e}.up"]], 0) for e in range(E)]).to(device)
    dn = torch.stack([Wt[f"e{e}.down"] for e in range(E)]).to(device)
    y = gated_moe_ffn(h.to(device), ti, tp, gu, dn, clamped_glu)
    assert y.dtype == torch.float32
    assert rel_err(y, O.moe_ff(h.double(), Wd, "", fc)) < tol(dtype) / 2


# ------------------------------------------------------------------------------------------------------------------
# the model through the ragged step
# ------------------------------------------------------------------------------------------------------------------
def _tokens(n, vocab, seed):
    return torch.randint(0, vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


@pytest.mark.parametrize("device,dtype", CASES)
@pytest.mark.parametrize("variant", list(VARIANTS))
def test_whole_prompt_and_residuals(tmp_path, device, dtype, variant):
    from llm_in_practise_b200.inference.ragged import RaggedGenerator
    cfg = VARIANTS[variant]()
    W = O.random_weights(cfg, seed=11)
    model = build(tmp_path, cfg, W, device, dtype)
    toks = _tokens(70, cfg["vocab"], 1)
    res_ref = []
    ref = O.forward(cfg, W, toks, res_ref)
    gen = RaggedGenerator(model, None, 128)
    cache = fresh_cache(gen, 1, 128)
    res = []
    got = gen.step([(0, 0, toks, list(range(len(toks))))], cache, layer_outputs=res)
    assert got.dtype == torch.float32
    for a, b in zip(res, res_ref):
        assert_rows(a, b, dtype, variant)
    assert_rows(got, ref, dtype, variant)
    # the first tokens of a sequence: a one-token request and the start of a longer one agree with the oracle row by row
    one = gen.step([(0, 0, toks[:1], [0])], fresh_cache(gen, 1, 64))
    assert rel_err(one, ref[:1]) < 2 * tol(dtype)
    assert rel_err(got[:3], ref[:3]) < 2 * tol(dtype)


@pytest.mark.parametrize("device,dtype", CASES)
@pytest.mark.parametrize("name", list(ODD))
def test_odd_sizes(tmp_path, device, dtype, name):
    from llm_in_practise_b200.inference.ragged import RaggedGenerator
    cfg = ODD[name]()
    W = O.random_weights(cfg, seed=3)
    model = build(tmp_path, cfg, W, device, dtype)
    n = 140
    toks = _tokens(n, cfg["vocab"], 2)
    ref = O.forward(cfg, W, toks)
    gen = RaggedGenerator(model, None, 192)
    cache = fresh_cache(gen, 2, 192)
    p, outs = 0, []
    for c in [30, 34, 2, 3, 61, 1, 1, 1, 7]:
        outs.append(gen.step([(1, p, toks[p:p + c], list(range(c)))], cache))
        p += c
    assert_rows(torch.cat(outs, 0), ref, dtype, name)


@pytest.mark.parametrize("device,dtype", CASES)
def test_portions_decode_and_long_decode(tmp_path, device, dtype):
    """Whatever way a sequence is cut into steps — whole, portions down to two tokens that straddle page borders, one token
    at a time for 150 tokens — every position's logits equal the oracle's for the whole sequence."""
    from llm_in_practise_b200.inference.ragged import RaggedGenerator
    cfg = VARIANTS["mixed"]()
    W = O.random_weights(cfg, seed=12, std=0.6 if dtype == torch.float32 else 0.2)     # sharp attention: a misplaced key shows
    model = build(tmp_path, cfg, W, device, dtype)
    n = 230
    toks = _tokens(n, cfg["vocab"], 2)
    ref = O.forward(cfg, W, toks)
    gen = RaggedGenerator(model, None, 256)
    for cuts in ([60, 2, 2, 3, 61, 1, 2, 64, 35], [63, 2, 64, 101], [80] + [1] * 150):
        assert sum(cuts) == n
        cache = fresh_cache(gen, 1, 256)
        p, outs = 0, []
        for c in cuts:
            outs.append(gen.step([(0, p, toks[p:p + c], list(range(c)))], cache))
            p += c
        assert_rows(torch.cat(outs, 0), ref, dtype, cuts[:4])


@pytest.mark.parametrize("device,dtype", CASES)
def test_mixed_batch_equals_each_alone(tmp_path, device, dtype):
    from llm_in_practise_b200.inference.ragged import RaggedGenerator
    cfg = VARIANTS["mixed"]()
    W = O.random_weights(cfg, seed=13, std=0.5 if dtype == torch.float32 else 0.2)
    model = build(tmp_path, cfg, W, device, dtype)
    lens = [150, 9, 70, 1]
    seqs = [_tokens(L, cfg["vocab"], 20 + i) for i, L in enumerate(lens)]
    refs = [O.forward(cfg, W, s) for s in seqs]
    gen = RaggedGenerator(model, None, 192)
    cache = fresh_cache(gen, 4, 192)
    # step plans: per sequence a list of portion sizes; sequences join and pause at different steps
    plans = [[64, 2, 0, 50, 1, 1, 32], [0, 9, 0, 0, 0, 0, 0], [3, 1, 60, 1, 1, 2, 2], [0, 0, 1, 0, 0, 0, 0]]
    done = [0] * 4
    outs = [[] for _ in seqs]
    for step in range(7):
        entries, who = [], []
        for s, plan in enumerate(plans):
            c = plan[step]
            if c:
                entries.append((s, done[s], seqs[s][done[s]:done[s] + c], list(range(c))))
                who.append((s, c))
                done[s] += c
        got = gen.step(entries, cache)
        o = 0
        for s, c in who:
            outs[s].append(got[o:o + c])
            o += c
    assert done == lens
    for s in range(4):
        assert_rows(torch.cat(outs[s], 0), refs[s], dtype, s)


@pytest.mark.parametrize("device,dtype", CASES)
def test_engine_replay_reuses_pages_and_slots(tmp_path, device, dtype):
    """The engine's own slot pool (4 rows) and block pool (sized for the live requests only): six requests come and go, so
    rows and pages are handed out again while neighbours are still using theirs."""
    from llm_in_practise_b200.serve.engine import EngineArgs, LLMEngine
    cfg = VARIANTS["odd_heads"]()
    W = O.random_weights(cfg, seed=14, std=0.5 if dtype == torch.float32 else 0.2)
    model = build(tmp_path, cfg, W, device, dtype)
    lens = {"a": 130, "b": 64, "c": 65, "d": 20, "e": 128, "f": 70}
    seqs = {k: _tokens(L, cfg["vocab"], 30 + i) for i, (k, L) in enumerate(lens.items())}
    refs = {k: O.forward(cfg, W, s) for k, s in seqs.items()}
    eng = LLMEngine(model, None, EngineArgs(max_num_seqs=4, max_model_len=192, block_size=64, num_kv_blocks=7,
                                            enable_prefix_caching=False, warmup=False))
    done = {k: 0 for k in lens}
    outs = {k: [] for k in lens}

    def run(parts, end=()):
        entries = []
        for k, c in parts:
            entries.append((k, seqs[k][done[k]:done[k] + c], list(range(c))))
            done[k] += c
        got = eng.replay_step(entries, end)
        o = 0
        for k, c in parts:
            outs[k].append(got[o:o + c])
            o += c

    run([("a", 100), ("b", 30)])                       # a: 2 pages, b: 1
    run([("a", 30), ("b", 34), ("c", 65)], end=["b"])  # a: 3, b: 1, c: 2 -> 6 of 7 pages; b leaves
    run([("d", 20), ("c", 0), ("e", 60)], end=["a"])   # d and e take b's row / page and fresh ones
    run([("e", 68), ("d", 0)], end=["d", "c"])
    run([("f", 2)])
    run([("f", 62), ("e", 0)])
    run([("f", 6)], end=["e", "f"])
    assert done == lens
    for k in lens:
        assert_rows(torch.cat([o for o in outs[k] if o.shape[0]], 0), refs[k], dtype, k)
    assert len(eng.free) == 4 and len(eng._free_blocks) == 7       # everything went back to the pools


@pytest.mark.parametrize("device,dtype", [("cpu", torch.float32), pytest.param("cuda", torch.float32, marks=pytest.mark.gpu)])
def test_greedy_generation_through_engine_and_generate(tmp_path, device, dtype):
    from llm_in_practise_b200.inference import GenerationConfig
    from llm_in_practise_b200.serve.engine import EngineArgs, LLMEngine
    cfg = VARIANTS["mixed"]()
    W = O.random_weights(cfg, seed=15)
    model = build(tmp_path, cfg, W, device, dtype)
    prompts = [_tokens(L, cfg["vocab"], 40 + i) for i, L in enumerate([5, 70, 17, 33, 2, 64])]
    new = 12
    refs = [O.greedy(cfg, W, p, new) for p in prompts]
    # scheduler: 4 rows for 6 requests, 24 prompt tokens per iteration, so prompts are cut and mixed with decode tokens
    eng = LLMEngine(model, None, EngineArgs(max_num_seqs=4, max_model_len=128, max_prefill_tokens=24, block_size=64,
                                            enable_prefix_caching=True, warmup=False))
    reqs = eng.generate(prompts, GenerationConfig(max_new_tokens=new, ignore_eos=True))
    for r, p, ref in zip(reqs, prompts, refs):
        assert r.finish_reason == "length"
        assert p + r.output_ids == ref
    # a second wave repeats two prompts: the prefix cache shares their pages, the result must not change
    again = eng.generate([prompts[1], prompts[5]], GenerationConfig(max_new_tokens=new, ignore_eos=True))
    assert prompts[1] + again[0].output_ids == refs[1] and prompts[5] + again[1].output_ids == refs[5]
    assert eng.metrics.prefix_hits > 0
    out = model.generate(torch.tensor([prompts[2], prompts[2][::-1]], device=device), max_new_tokens=new)
    assert out[0].tolist() == refs[2]
    assert out[1].tolist() == O.greedy(cfg, W, prompts[2][::-1], new)
    lg = model(torch.tensor([prompts[3]], device=device))["logits"][0]
    assert rel_err(lg, O.forward(cfg, W, prompts[3])) < tol(dtype)


def test_checkpoint_names_round_trip(tmp_path):
    from llm_in_practise_b200.models.gorozen import GorozenConfig, gorozen_state_dict
    cfg = VARIANTS["mixed"]()
    W = O.random_weights(cfg, seed=16)
    model = build(tmp_path, cfg, W, "cpu", torch.bfloat16)
    sd = gorozen_state_dict(model)
    assert set(sd) == set(W)
    for k in W:
        assert torch.equal(sd[k].to(torch.bfloat16).cpu(), W[k]), k
    c = GorozenConfig.from_dict(cfg)
    assert [l.mlp.kind if l.mlp else None for l in c.layers] == ["dense", "moe", None]
    with pytest.raises(ValueError):
        bad = json.loads(json.dumps(cfg))
        bad["layers"][0]["type"] = "recurrent"
        GorozenConfig.from_dict(bad)
