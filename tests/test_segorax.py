"""Segorax against the plain float64 oracle in ``segorax_oracle.py``: every mechanism alone, then the model through the ragged
step, the serving engine's block / slot pools and its scheduler. Small random models of several shapes; the same tests run
on the CPU path and (marked ``gpu``) on the CUDA kernels in fp32 and bf16. The oracle expands keys and values per head; the
package attends over the cached latent rows, so agreement also checks the absorbed form."""
import json
import math

import pytest
import torch

import segorax_oracle as O

CASES = [("cpu", torch.float32), pytest.param("cuda", torch.float32, marks=pytest.mark.gpu),
         pytest.param("cuda", torch.bfloat16, marks=pytest.mark.gpu)]


def tol(dtype):
    return 2e-4 if dtype == torch.float32 else 6e-2


def row_errs(got, want):
    """Per row: RMS difference over RMS of the oracle, means over the last axis removed."""
    got, want = got.double().cpu(), want.double().cpu()
    d = got - want
    d = d - d.mean(-1, keepdim=True)
    w = want - want.mean(-1, keepdim=True)
    return d.pow(2).mean(-1).sqrt() / w.pow(2).mean().sqrt()


def rel_err(got, want):
    return float(row_errs(got.reshape(1, -1), want.reshape(1, -1))[0])


def assert_rows(got, want, dtype, what=""):
    """Every position against the oracle. In fp32 each row must agree. In 16 bits a router score that the oracle decides by a
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


def fresh_cache(gen, n_seqs, max_len, block=64):
    """A cache whose rows list their blocks in a scrambled physical order."""
    per = -(-max_len // block)
    cache = gen.make_cache(n_seqs * per, block, n_seqs, per * block)
    ids = list(range(1, n_seqs * per + 1))[::-1]
    for s in range(n_seqs):
        gen.set_block_row(cache, s, ids[s::n_seqs][:per])
    return cache


SCALING = {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}      # with base 100 and 16 dims: kept, blended and divided dims

VARIANTS = {
    # both mixers, both feed-forwards, a layer without one; sizes the tensor-core kernel takes (48 and 64 values per cached row)
    "mixed": lambda: O.make_config(64, 96, [
        O.latent_layer("latent_attention", 4, 24, 8, 16, 40, 32, mlp=O.dense(80)),
        O.latent_layer("latent_attention_2", 4, 16, 16, 32, 48, base=100.0, scaling=SCALING, mlp=O.moe(6, 2, 48, 3, 2, 40)),
        O.latent_layer("latent_attention", 4, 24, 8, 16, 40, 32, mlp=None)]),
    # one head; values wider than keys; every group kept; one expert chosen; no shared expert; multipliers of 1
    "one_head": lambda: O.make_config(48, 80, [
        O.latent_layer("latent_attention_2", 1, 16, 16, 56, 32, base=50.0, scaling={"factor": 1.5, "original": 32, "fast": 4.0, "slow": 2.0},
                       scale=0.3, mlp=O.moe(4, 1, 24, 2, 2, 0)),
        O.latent_layer("latent_attention", 3, 32, 16, 8, 16, 56, mlp=O.dense(40))], embed_scale=1.0, residual_mult=1.0, logit_scale=1.0),
    # one group; all experts of the kept groups chosen; query latent wider than the KV latent
    "all_chosen": lambda: O.make_config(40, 64, [
        O.latent_layer("latent_attention", 8, 8, 8, 8, 24, 40, mlp=O.moe(3, 3, 16, 1, 1, 24)),
        O.latent_layer("latent_attention_2", 2, 40, 8, 24, 56, base=10.0, scaling=None, mlp=O.moe(8, 2, 16, 4, 1, 8))], eps=1e-3),
}

# sizes that are not multiples of the kernels' vector widths: rows of 42 and 30 cached values, head sizes 26 and 18, widths and
# latent sizes that TMA cannot address, 5 and 3 heads
ODD = {
    "w72": lambda: O.make_config(72, 75, [
        O.latent_layer("latent_attention", 5, 20, 6, 10, 36, 20, mlp=O.dense(100)),
        O.latent_layer("latent_attention_2", 3, 12, 6, 14, 24, base=1e4, scaling=SCALING, mlp=O.moe(6, 3, 36, 2, 1, 20))]),
    "w100": lambda: O.make_config(100, 130, [
        O.latent_layer("latent_attention_2", 3, 30, 2, 22, 50, base=1e6, scaling=None, mlp=O.moe(9, 2, 52, 3, 2, 28)),
        O.latent_layer("latent_attention", 10, 10, 10, 10, 22, 12, mlp=O.dense(90))], logit_scale=2.0),
}


# ------------------------------------------------------------------------------------------------------------------
# mechanisms alone
# ------------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("device,dtype", CASES)
def test_post_norm_residual_with_multiplier(device, dtype):
    from llm_in_practise_b200.ops.norm import sandwich_norm
    g = torch.Generator().manual_seed(1)
    n, W, eps = 5, 72, 1e-5
    y, res = torch.randn(n, W, generator=g) * 3, torch.randn(n, W, generator=g)
    wp = (1 + torch.randn(W, generator=g) * 0.3).to(dtype)
    h, x = sandwich_norm(y.to(device), wp.to(device), res.to(device), None, eps, 0.0, dtype, branch_mult=0.35, cast_next=True)
    x_ref = res.double() + 0.35 * O.norm(y.double(), wp.double(), eps)
    assert x.dtype == torch.float32 and h.dtype == dtype
    torch.testing.assert_close(x.cpu().double(), x_ref, rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(h.cpu().double(), x_ref, rtol=tol(dtype) / 4, atol=tol(dtype) / 4)       # h is the stream itself
    # entering the stream: y * scale, nothing normed
    emb = torch.randn(n, W, generator=g).to(dtype)
    h0, x0 = sandwich_norm(emb.to(device), None, None, None, eps, 0.0, dtype, branch_mult=7.5, cast_next=True)
    torch.testing.assert_close(x0.cpu().double(), emb.double() * 7.5, rtol=1e-6, atol=1e-6)
    # leaving it: the final norm of the stream
    wn = (1 + torch.randn(W, generator=g) * 0.3).to(dtype)
    h2, _ = sandwich_norm(None, None, x, wn.to(device), eps, 0.0, dtype)
    torch.testing.assert_close(h2.cpu().double(), O.norm(x.cpu().double(), wn.double(), eps), rtol=tol(dtype) / 4, atol=tol(dtype) / 4)


def test_scaled_frequencies_have_three_bands():
    from llm_in_practise_b200.models.segorax import _yarn_scaling
    from llm_in_practise_b200.ops.elementwise import rope_inv_freq
    rot = {"base": 100.0, "dims": 16, "scaling": SCALING}
    f0, _ = O.rotary_frequencies({"base": 100.0, "dims": 16})
    f, mag = O.rotary_frequencies(rot)
    ratio = [a / b for a, b in zip(f, f0)]
    assert any(abs(r - 1.0) < 1e-12 for r in ratio) and any(abs(r - 1 / 4) < 1e-12 for r in ratio)
    assert any(1 / 4 + 1e-6 < r < 1 - 1e-6 for r in ratio)
    assert abs(mag - (0.1 * math.log(4.0) + 1)) < 1e-12
    for r in (rot, {"base": 50.0, "dims": 16, "scaling": {"factor": 1.5, "original": 32, "fast": 4.0, "slow": 2.0}},
              {"base": 1e4, "dims": 6, "scaling": SCALING}, {"base": 7.0, "dims": 4, "scaling": {"factor": 0.5, "original": 4096, "fast": 64.0, "slow": 32.0}}):
        inv, att = rope_inv_freq(r["dims"], r["base"], _yarn_scaling(r["scaling"]), dtype=torch.float64)
        fr, m = O.rotary_frequencies(r)
        torch.testing.assert_close(inv, torch.tensor(fr, dtype=torch.float64), rtol=1e-6, atol=0)
        assert abs(att - m) < 1e-12


@pytest.mark.parametrize("device,dtype", CASES)
@pytest.mark.parametrize("C,R,rot,Cq,scaling", [(40, 8, 8, 32, None), (48, 16, 16, 0, SCALING), (36, 6, 6, 20, None), (24, 8, 4, 12, None)])
def test_latent_store_and_query_rotation(device, dtype, C, R, rot, Cq, scaling):
    from llm_in_practise_b200.models.segorax import _yarn_scaling
    from llm_in_practise_b200.ops.elementwise import rope_tables_partial
    from llm_in_practise_b200.ops.latent_attention import latent_kv_store, latent_q_rope
    g = torch.Generator().manual_seed(2)
    H, D, BS, eps = 3, 12, 8, 1e-5
    positions = [0, 1, 7, 8, 9, 63, 200, 1023]
    slots = [1, 0, 1, 1, 0, 0, 1, 0]
    n = len(positions)
    proj = torch.randn(n, Cq + C + R, generator=g) * 2
    wq = (1 + torch.randn(max(Cq, 1), generator=g) * 0.3).to(dtype)
    wkv = (1 + torch.randn(C, generator=g) * 0.3).to(dtype)
    rd = {"base": 100.0, "dims": rot}
    if scaling:
        rd["scaling"] = scaling
    cos, sin = rope_tables_partial(1024, rot, 100.0, device, _yarn_scaling(scaling))
    nb = 2 * 128
    cache = torch.zeros(nb + 1, 1, BS, C + R, dtype=dtype, device=device)
    table = (torch.randperm(nb, generator=g).view(2, 128) + 1).to(torch.int32).to(device)
    pos_t = torch.tensor(positions, dtype=torch.int32, device=device)
    cq = latent_kv_store(proj.to(device), 0, Cq, Cq, C, R, rot, wq.to(device) if Cq else None, wkv.to(device), eps, cos, sin, pos_t,
                         torch.tensor(slots, dtype=torch.int32, device=device), cache, table, dtype)
    t = tol(dtype) / 4
    pd = proj.double()
    c_ref = O.norm(pd[:, Cq:Cq + C], wkv.double(), eps)
    r_ref = O.rotate(pd[:, None, Cq + C:], positions, rd)[:, 0]
    for i, (p, s) in enumerate(zip(positions, slots)):
        row = cache[int(table[s, p // BS]), 0, p % BS].cpu().double()
        torch.testing.assert_close(row[:C], c_ref[i], rtol=t, atol=t)
        torch.testing.assert_close(row[C:], r_ref[i], rtol=t, atol=t)
    if Cq:
        torch.testing.assert_close(cq.cpu().double(), O.norm(pd[:, :Cq], wq.double(), eps), rtol=t, atol=t)
    else:
        assert cq is None
    q = torch.randn(n, H * (D + R), generator=g).to(dtype)
    qx = torch.zeros(n, H, C + R, dtype=dtype, device=device)
    latent_q_rope(q.to(device), cos, sin, pos_t, qx, H, D, R, rot, C)
    q_ref = O.rotate(q.double().view(n, H, D + R)[:, :, D:], positions, rd)
    torch.testing.assert_close(qx[:, :, C:].cpu().double(), q_ref, rtol=t, atol=t)
    assert float(qx[:, :, :C].abs().max()) == 0


@pytest.mark.parametrize("device,dtype", CASES)
@pytest.mark.parametrize("w_kn", [True, False])
@pytest.mark.parametrize("H,K,N,extra", [(4, 24, 40, 8), (3, 20, 36, 6), (1, 64, 16, 0)])
def test_head_linear(device, dtype, w_kn, H, K, N, extra):
    from llm_in_practise_b200.ops.gemm import head_linear
    g = torch.Generator().manual_seed(3)
    T = 11
    full = torch.randn(T, H, K + extra, generator=g).to(dtype)
    w = (torch.randn(H, K, N, generator=g) if w_kn else torch.randn(H, N, K, generator=g)).to(dtype)
    wide = torch.zeros(T, H, N + extra, dtype=dtype, device=device)
    out = head_linear(full.to(device)[:, :, :K], w.to(device), w_kn=w_kn, out=wide[:, :, :N])
    ref = torch.einsum("thk,hkn->thn" if w_kn else "thk,hnk->thn", full[:, :, :K].double(), w.double())
    assert rel_err(out, ref) < tol(dtype) / 4
    assert float(wide[:, :, N:].abs().max()) == 0 if extra else True


def _fill_rows(rows, BS, device, dtype, seed=0):
    """rows [n, Dk] of ONE sequence -> (cache, table) with scrambled pages, sequence in row 1 of 2."""
    n, Dk = rows.shape
    nb = -(-n // BS)
    perm = torch.randperm(nb + 3, generator=torch.Generator().manual_seed(seed))[:nb] + 1
    cache = torch.full((nb + 5, 1, BS, Dk), float("nan"), dtype=dtype, device=device)        # unread pages hold NaN
    table = torch.zeros(2, nb, dtype=torch.int32, device=device)
    table[1] = perm.to(torch.int32)
    for j in range(nb):
        lo, hi = j * BS, min(n, (j + 1) * BS)
        cache[perm[j], 0, :hi - lo] = rows[lo:hi].to(device, dtype)
        cache[perm[j], 0, hi - lo:] = 0          # the tail of the last page is never a valid key; finite filler
    return cache, table


def _pieces(device, runs):
    from llm_in_practise_b200.inference.ragged import TILE_Q, Pieces
    tiles, base = [], 0
    for pos0, n in runs:
        for q0 in range(0, n, TILE_Q):
            tiles.append([base + q0, min(TILE_Q, n - q0), pos0 + q0, 1])
        base += n
    return Pieces(torch.tensor(tiles, dtype=torch.int32, device=device), len(tiles), max(n for _, n in runs))


def _latent_reference(q, rows, C, scale, sink):
    """Multi-query attention in the latent space, float64: q [n, H, Dk], rows [n, Dk] -> [n, H, C]."""
    n, H, _ = q.shape
    k = rows[:, None, :].expand(n, H, rows.shape[1])
    return O.causal_attention(q, k, k[:, :, :C], scale, sink)


@pytest.mark.parametrize("device,dtype", CASES)
@pytest.mark.parametrize("H,C,R,BS", [(4, 40, 8, 64), (3, 36, 6, 16), (6, 64, 32, 64), (1, 16, 16, 32), (16, 32, 16, 64), (80, 16, 0, 64),
                                      (2, 320, 16, 64), (20, 272, 16, 64), (40, 128, 32, 64)])
@pytest.mark.parametrize("with_sink", [True, False])
def test_latent_attention(device, dtype, H, C, R, BS, with_sink):
    from llm_in_practise_b200.ops.latent_attention import latent_attention
    g = torch.Generator().manual_seed(4)
    n, Dk = 150, C + R
    q = torch.randn(n, H, Dk, generator=g).to(dtype)
    rows = torch.randn(n, Dk, generator=g).to(dtype)
    sink = torch.randn(H, generator=g) * 2 if with_sink else None
    scale = 0.21
    ref = _latent_reference(q.double(), rows.double(), C, scale, sink.double() if with_sink else None)
    cache, table = _fill_rows(rows, BS, device, dtype)
    sk = sink.to(device) if with_sink else None
    # (a) the last 90 positions as one piece over 60 cached ones, (b) single tokens, (c) pieces and single tokens in one call
    pos = torch.arange(60, n, dtype=torch.int32, device=device)
    out = latent_attention(q[60:].contiguous().to(device), cache, table, pos, torch.ones_like(pos), H, C, scale, sinks=sk, max_pos=n - 1,
                           pieces=_pieces(device, [(60, n - 60)]))
    assert float(row_errs(out.reshape(n - 60, -1), ref[60:].reshape(n - 60, -1)).max()) < tol(dtype) / 2
    for t in (0, 1, 63, 64, 65, n - 1):
        o1 = latent_attention(q[t:t + 1].contiguous().to(device), cache, table, torch.tensor([t], dtype=torch.int32, device=device),
                              torch.ones(1, dtype=torch.int32, device=device), H, C, scale, sinks=sk, max_pos=t)
        assert rel_err(o1, ref[t:t + 1]) < tol(dtype) / 2, t
    idx = list(range(10, 13)) + [100] + list(range(64, 66)) + [5]
    posm = torch.tensor(idx, dtype=torch.int32, device=device)
    outm = latent_attention(q[idx].contiguous().to(device), cache, table, posm, torch.ones_like(posm), H, C, scale, sinks=sk, max_pos=100,
                            pieces=_pieces(device, [(10, 3), (100, 1), (64, 2), (5, 1)]))
    assert float(row_errs(outm.reshape(len(idx), -1), ref[idx].reshape(len(idx), -1)).max()) < tol(dtype) / 2


@pytest.mark.parametrize("device,dtype", CASES)
@pytest.mark.parametrize("as_piece", [True, False])
def test_one_far_row_dominates(device, dtype, as_piece):
    """One cached row gets a score far above the rest: the output must be its latent — for rows hundreds back, on both sides
    of a page border, the first row and the query's own; a row one step ahead must stay unseen; a dominant sink must leave
    (almost) nothing."""
    from llm_in_practise_b200.ops.latent_attention import latent_attention
    g = torch.Generator().manual_seed(5)
    H, C, R, BS, n = 2, 32, 16, 64, 700
    Dk = C + R
    rows = torch.randn(n, Dk, generator=g)
    rows[:, C:] *= 0.05                                     # the scores are decided by the rotated part
    qdir = torch.nn.functional.normalize(torch.randn(R, generator=g), dim=0)
    targets = {699: 0, 698: 63, 697: 64, 696: 65, 695: 127, 694: 128, 693: 300, 692: 692, 691: 690, 640: 639, 650: 1}
    q = torch.zeros(n, H, Dk)
    q[:, :, C:] = torch.randn(n, H, R, generator=g) * 0.05
    for qp in targets:
        q[qp, :, C:] = qdir * 60
    sink = torch.zeros(H)
    one = lambda p: torch.tensor([p], dtype=torch.int32, device=device)          # noqa: E731
    for qp, kp in targets.items():
        rb = rows.clone()
        rb[kp, C:] = qdir * 4
        cache, table = _fill_rows(rb.to(dtype), BS, device, dtype, seed=qp)
        if as_piece:
            lo = max(0, qp - 20)
            pos = torch.arange(lo, qp + 1, dtype=torch.int32, device=device)
            out = latent_attention(q[lo:qp + 1].contiguous().to(device, dtype), cache, table, pos, torch.ones_like(pos), H, C, 1.0,
                                   sinks=sink.to(device), max_pos=qp, pieces=_pieces(device, [(lo, qp + 1 - lo)]))[-1]
        else:
            out = latent_attention(q[qp:qp + 1].contiguous().to(device, dtype), cache, table, one(qp), one(1), H, C, 1.0,
                                   sinks=sink.to(device), max_pos=qp)[0]
        want = rb[kp, :C].to(dtype).float().expand(H, C)
        torch.testing.assert_close(out.float().cpu(), want, rtol=2e-2, atol=2e-2, msg=f"query {qp} row {kp}")
    rb = rows.clone()
    rb[401, C:] = qdir * 4
    cache, table = _fill_rows(rb.to(dtype), BS, device, dtype)
    qq = torch.zeros(1, H, Dk)
    qq[:, :, C:] = qdir * 60
    qq = qq.to(device, dtype)
    seen = latent_attention(qq, cache, table, one(401), one(1), H, C, 1.0, sinks=sink.to(device), max_pos=401)[0]
    unseen = latent_attention(qq, cache, table, one(400), one(1), H, C, 1.0, sinks=sink.to(device), max_pos=400)[0]
    torch.testing.assert_close(seen.float().cpu(), rb[401, :C].to(dtype).float().expand(H, C), rtol=2e-2, atol=2e-2)
    assert float((unseen.float().cpu() - rb[401, :C]).abs().max()) > 0.5
    big = latent_attention(qq, cache, table, one(400), one(1), H, C, 1.0, sinks=torch.full((H,), 300.0, device=device), max_pos=400)[0]
    assert float(big.float().abs().max()) < 1e-3


@pytest.mark.parametrize("device,dtype", CASES)
@pytest.mark.parametrize("with_sink", [True, False])
def test_long_context_decode_splits(device, dtype, with_sink):
    """Single tokens over thousands of rows (on the GPU the rows are cut into ranges over several CTAs) equal the oracle."""
    from llm_in_practise_b200.ops.latent_attention import latent_attention
    g = torch.Generator().manual_seed(6)
    H, C, R, BS, n = 4, 32, 16, 64, 2500
    rows = torch.randn(n, C + R, generator=g).to(dtype)
    q = torch.randn(2, H, C + R, generator=g).to(dtype)
    sink = torch.randn(H, generator=g) if with_sink else None
    cache, table = _fill_rows(rows, BS, device, dtype)
    posl = [n - 1, 1300]
    out = latent_attention(q.to(device), cache, table, torch.tensor(posl, dtype=torch.int32, device=device),
                           torch.ones(2, dtype=torch.int32, device=device), H, C, 0.3, sinks=sink.to(device) if with_sink else None, max_pos=n - 1)
    for i, p in enumerate(posl):
        sc = (q[i].double() @ rows[:p + 1].double().t()) * 0.3
        m = sc.max(-1).values if sink is None else torch.maximum(sc.max(-1).values, sink.double())
        e = torch.exp(sc - m[:, None])
        den = e.sum(-1) + (0 if sink is None else torch.exp(sink.double() - m))
        ref = (e / den[:, None]) @ rows[:p + 1, :C].double()
        assert rel_err(out[i], ref) < tol(dtype) / 2, p


@pytest.mark.parametrize("device,dtype", CASES)
def test_activations(device, dtype):
    from llm_in_practise_b200.ops.elementwise import act_glu, gelu
    g = torch.Generator().manual_seed(7)
    for F in (36, 64):
        gu = (torch.randn(7, 2 * F, generator=g) * 3).to(dtype)
        a, b = gu[:, :F].double(), gu[:, F:].double()
        t = tol(dtype) / 4
        torch.testing.assert_close(act_glu(gu.to(device), "gelu_tanh").cpu().double(), O.gelu_tanh(a) * b, rtol=t, atol=2 * t)
        torch.testing.assert_close(act_glu(gu.to(device), "gelu").cpu().double(), O.gelu_erf(a) * b, rtol=t, atol=2 * t)
        torch.testing.assert_close(act_glu(gu.to(device), "silu").cpu().double(), a * torch.sigmoid(a) * b, rtol=t, atol=2 * t)
        torch.testing.assert_close(gelu(gu.to(device)).cpu().double(), O.gelu_erf(gu.double()), rtol=t, atol=t)
    z = torch.tensor([[1.0, 1.0]], dtype=torch.float64)     # the two forms differ: 0.8412 (tanh form) vs 0.8413 (erf)
    assert abs(float(O.gelu_tanh(z)[0, 0]) - float(O.gelu_erf(z)[0, 0])) > 1e-4


@pytest.mark.parametrize("device,dtype", CASES)
@pytest.mark.parametrize("E,K,groups,keep,shared", [(6, 2, 3, 2, 40), (8, 2, 2, 1, 16), (4, 1, 2, 2, 0), (3, 3, 1, 1, 24), (12, 3, 4, 1, 8),
                                                     (16, 4, 4, 2, 0)])
def test_router_and_experts(device, dtype, E, K, groups, keep, shared):
    from llm_in_practise_b200.ops.elementwise import gelu
    from llm_in_practise_b200.ops.gemm import linear_exact
    from llm_in_practise_b200.ops.moe import gated_moe_ffn, route_sigmoid_grouped
    g = torch.Generator().manual_seed(8)
    n, W, F = 19, 40, 24
    fc = {"router": {"experts": E, "top": K, "groups": {"count": groups, "keep": keep}}, "expert": {"ff": F}}
    Wt = {"router": torch.randn(E, W, generator=g).to(torch.bfloat16),
          "correction": (torch.randn(E, generator=g) * 0.5 - 1.2).to(torch.bfloat16)}        # most choice scores are negative
    for e in range(E):
        Wt[f"e{e}.up"] = (torch.randn(F, W, generator=g) * W ** -0.5).to(dtype)
        Wt[f"e{e}.down"] = (torch.randn(W, F, generator=g) * F ** -0.5).to(dtype)
    if shared:
        fc["shared"] = {"ff": shared}
        Wt["shared.up"] = (torch.randn(shared, W, generator=g) * W ** -0.5).to(dtype)
        Wt["shared.down"] = (torch.randn(W, shared, generator=g) * shared ** -0.5).to(dtype)
        Wt["shared.sg"] = torch.randn(1, W, generator=g).to(torch.bfloat16)
    h = torch.randn(n, W, generator=g).to(dtype)
    Wd = {k: v.double() for k, v in Wt.items()}
    idx_ref, w_ref = O.router(h.double(), Wd, "", fc["router"])
    assert float((torch.sigmoid(h.double() @ Wd["router"].T) + Wd["correction"]).gather(1, idx_ref).min()) < 0
    wr = torch.cat([Wt["router"]] + ([Wt["shared.sg"]] if shared else []), 0).float().to(device)
    ti, tp, gate = route_sigmoid_grouped(h.to(device), wr, Wt["correction"].float().to(device), K, groups, keep, 2, gate_rows=1 if shared else 0)
    assert tp.dtype == torch.float32
    assert torch.equal(ti.cpu(), idx_ref)
    torch.testing.assert_close(tp.cpu().double(), w_ref, rtol=1e-5, atol=1e-6)
    if keep < groups:                                        # every chosen expert of a token lies in at most `keep` groups
        assert int((ti.cpu() // (E // groups)).sort(-1).values.diff(dim=-1).ne(0).sum(-1).max()) <= keep - 1
    sh = None
    if shared:
        torch.testing.assert_close(gate.cpu().double(), torch.sigmoid(h.double() @ Wd["shared.sg"].T), rtol=1e-5, atol=1e-6)
        sh = linear_exact(gelu(linear_exact(h.to(device), Wt["shared.up"].to(device))), Wt["shared.down"].to(device))
    up = torch.stack([Wt[f"e{e}.up"] for e in range(E)]).to(device)
    dn = torch.stack([Wt[f"e{e}.down"] for e in range(E)]).to(device)
    y = gated_moe_ffn(h.to(device), ti, tp, up, dn, gelu, shared=sh, gate=gate)
    assert y.dtype == torch.float32
    assert rel_err(y, O.moe_ff(h.double(), Wd, "", fc)) < tol(dtype) / 2


def test_group_limit_beats_a_larger_score_outside():
    """An expert with the single largest choice score sits in a group whose top-two sum loses: it must not be chosen."""
    from llm_in_practise_b200.ops.moe import route_sigmoid_grouped
    W = 4
    h = torch.eye(W)[:1]
    z = torch.tensor([3.0, -9.0, 1.0, 1.0, -1.0, -1.0])     # group 0: one high score; group 1: two good ones; group 2: weak
    wr = torch.zeros(6, W)
    wr[:, 0] = z
    ti, tp, _ = route_sigmoid_grouped(h, wr, torch.zeros(6), 2, 3, 1, 2)
    assert sorted(ti[0].tolist()) == [2, 3]
    torch.testing.assert_close(tp[0], torch.sigmoid(torch.tensor([1.0, 1.0])))
    ti1, _, _ = route_sigmoid_grouped(h, wr, torch.zeros(6), 2, 3, 1, 1)      # ranked by the single largest instead: group 0 wins
    assert sorted(ti1[0].tolist()) == [0, 1]


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
    assert all(v.shape[3] == 0 for v in cache.v)            # only the latent rows are cached
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
    W = O.random_weights(cfg, seed=12)
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
    W = O.random_weights(cfg, seed=13)
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
    cfg = VARIANTS["all_chosen"]()
    W = O.random_weights(cfg, seed=14)
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
    from llm_in_practise_b200.models.segorax import SegoraxConfig, segorax_state_dict
    cfg = VARIANTS["mixed"]()
    W = O.random_weights(cfg, seed=16)
    model = build(tmp_path, cfg, W, "cpu", torch.bfloat16)
    sd = segorax_state_dict(model)
    assert set(sd) == set(W)
    for k in W:
        assert torch.equal(sd[k].to(torch.bfloat16).cpu(), W[k]), k
    c = SegoraxConfig.from_dict(cfg)
    assert [l.mlp.kind if l.mlp else None for l in c.layers] == ["dense", "moe", None]
    assert [l.mixer.q_rank for l in c.layers] == [32, 0, 32] and c.layers[1].mixer.rot_scaling == SCALING
    with pytest.raises(ValueError):
        bad = json.loads(json.dumps(cfg))
        bad["layers"][0]["type"] = "recurrent"
        SegoraxConfig.from_dict(bad)
