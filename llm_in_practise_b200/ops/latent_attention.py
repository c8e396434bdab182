"""Ragged attention over a paged cache of latent rows (``csrc/latent_attn.cu``): multi-head latent attention the way a
serving engine runs it, with the up-projections of keys and values absorbed into the query and the output.

A layer of this kind caches ONE row per token, ``[c | r]``: the normed latent ``c`` [C] from which every head's keys and
values would be expanded (``k_h = W_uk_h c``, ``v_h = W_uv_h c``) and a rotated key part ``r`` [R] shared by all heads. The
expanded keys and values are never formed: head h's query is carried into the latent space,
``q'_h = [W_uk_h^T q_h | rot(q_h)]`` (``ops.gemm.head_linear`` + ``latent_q_rope``), the attention is multi-query attention
of ``q'`` over the cached rows with the rows' first C columns as values (``latent_attention``), and the context
``sum_j p_j c_j`` is expanded by ``W_uv_h`` afterwards. The cache pool is ``[blocks, 1, block_size, C + R]`` per layer with
no value pool, the block table and the (position, cache row) arrays are those of ``ops.paged_attention``.

Options other designs can use: a query latent with its own norm (or none), rotation of only the first ``rot`` of the R
columns, per-head attention sinks, any sizes (the tensor-core kernel takes C + R a multiple of 16 and C <= 512; everything
else runs on the fp32-arithmetic kernel).
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from . import _native as nv
from .paged_attention import _rotate

vp, i32, i64, f32 = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float


def _unit_rms(x, eps):
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def latent_kv_store(proj: torch.Tensor, q_off: int, q_rank: int, kv_off: int, kv_rank: int, rot_dim: int, rot_dims: int,
                    q_norm: Optional[torch.Tensor], kv_norm: torch.Tensor, eps: float, cos: torch.Tensor, sin: torch.Tensor,
                    pos: torch.Tensor, slot: torch.Tensor, cache: torch.Tensor, table: torch.Tensor,
                    dtype: torch.dtype) -> Optional[torch.Tensor]:
    """``proj`` fp32 [T, >= ...]: the down-projections of a step's tokens, query latent in columns ``q_off .. + q_rank``
    (``q_rank`` 0: none), KV latent in ``kv_off .. + kv_rank`` followed by ``rot_dim`` columns of the shared key part. Norms
    the latents (RMS, plain gains, fp32 statistics), turns the first ``rot_dims`` columns of the key part by the token's
    position (interleaved pairs; ``cos`` / ``sin`` fp32 [max_pos, rot_dims / 2]) and writes ``[c | r]`` to position ``pos[t]``
    of cache row ``slot[t]`` (``cache`` [blocks, 1, block_size, kv_rank + rot_dim]). Returns the normed query latent
    [T, q_rank] in ``dtype`` (None without one)."""
    T = proj.shape[0]
    C, R, Cq = kv_rank, rot_dim, q_rank
    BS = cache.shape[2]
    if nv.use_native(proj):
        if proj.dtype != torch.float32 or proj.stride(1) != 1 or cache.dtype != dtype:
            raise ValueError("latent_kv_store: fp32 projections with contiguous rows, cache in the compute dtype")
        cq = torch.empty(T, Cq, dtype=dtype, device=proj.device) if Cq else None
        fn = nv.proto("b200_latent_kv_store", [vp, i64, i32, i32, i32, i32, i32, i32, vp, vp, f32, vp, vp, vp, vp, vp, i32, i32, vp, vp,
                                               i32, i32, i32, vp])
        nv.check(fn(nv.ptr(proj), proj.stride(0), q_off, Cq, kv_off, C, R, rot_dims, nv.ptr(q_norm), nv.ptr(kv_norm), eps, nv.ptr(cos),
                    nv.ptr(sin), nv.ptr(pos), nv.ptr(slot), nv.ptr(table), table.shape[1], BS, nv.ptr(cq), nv.ptr(cache), T,
                    nv.dtype_code(dtype), nv.dtype_code(kv_norm.dtype), nv.stream()), "latent_kv_store")
        nv.count_launch()
        return cq
    pl, sl = pos.long(), slot.long()
    pf = proj.float()
    c = _unit_rms(pf[:, kv_off:kv_off + C], eps) * kv_norm.float()
    r = pf[:, None, kv_off + C:kv_off + C + R]
    if rot_dims:
        r = _rotate(r, cos[pl], sin[pl], rot_dims, True)
    blk = table[sl, pl // BS].long()
    cache[blk, 0, pl % BS] = torch.cat([c, r[:, 0]], -1).to(cache.dtype)
    if not Cq:
        return None
    return (_unit_rms(pf[:, q_off:q_off + Cq], eps) * q_norm.float()).to(dtype)


def latent_q_rope(q: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, pos: torch.Tensor, qx: torch.Tensor, n_heads: int,
                  dim: int, rot_dim: int, rot_dims: int, kv_rank: int) -> torch.Tensor:
    """The last ``rot_dim`` columns of every head of ``q`` [T, H * (dim + rot_dim)], turned like the keys' shared part, into
    columns ``kv_rank ..`` of the latent-space queries ``qx`` [T, H, kv_rank + rot_dim]. Returns ``qx``."""
    T = q.shape[0]
    H, D, R, C = n_heads, dim, rot_dim, kv_rank
    if R == 0:
        return qx
    if nv.use_native(q):
        if q.stride(1) != 1 or not qx.is_contiguous() or qx.dtype != q.dtype:
            raise ValueError("latent_q_rope: contiguous rows and one dtype")
        fn = nv.proto("b200_latent_q_rope", [vp, i64, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, vp])
        nv.check(fn(nv.ptr(q), q.stride(0), nv.ptr(cos), nv.ptr(sin), nv.ptr(pos), nv.ptr(qx), T, H, D, R, rot_dims, C,
                    nv.dtype_code(q.dtype), nv.stream()), "latent_q_rope")
        nv.count_launch()
        return qx
    r = q.view(T, H, D + R)[:, :, D:].float()
    if rot_dims:
        pl = pos.long()
        r = _rotate(r, cos[pl], sin[pl], rot_dims, True)
    qx[:, :, C:] = r.to(qx.dtype)
    return qx


_SPLIT_KEYS = int(os.environ.get("B200_LATENT_SPLIT_KEYS", "256"))      # keys per split of a decode-only batch


def latent_attention(qx: torch.Tensor, cache: torch.Tensor, table: torch.Tensor, pos: torch.Tensor, slot: torch.Tensor,
                     n_heads: int, kv_rank: int, scale: float, sinks: Optional[torch.Tensor] = None, max_pos: int = 0,
                     pieces=None) -> torch.Tensor:
    """Context in the latent space [T, H, kv_rank]: token t's heads over rows ``0 .. pos[t]`` of cache row ``slot[t]``,
    scores ``qx . row * scale``, values the rows' first ``kv_rank`` columns. ``qx`` [T, H, Dk] contiguous, ``cache``
    [blocks, 1, block_size, Dk]; ``sinks`` fp32 [H]: per-head logit in the softmax denominator only. ``pieces``: the step's
    runs of consecutive tokens (``inference.ragged.Pieces``); None: every token is alone (a decode batch), and ``max_pos``
    (an upper bound of ``pos`` known on the host) decides into how many key ranges a small batch is cut."""
    T, H, Dk = qx.shape
    Dv = kv_rank
    BS = cache.shape[2]
    if nv.use_native(qx):
        if not qx.is_contiguous() or cache.dtype != qx.dtype:
            raise ValueError("latent_attention: contiguous queries in the cache's dtype")
        out = torch.empty(T, H, Dv, dtype=qx.dtype, device=qx.device)
        mma_ok = (qx.dtype == torch.bfloat16 and Dk % 16 == 0 and Dv % 2 == 0 and Dv <= 512 and scale > 0 and BS & (BS - 1) == 0
                  and (Dk + 8) * 2 * 192 <= 227 * 1024 and os.environ.get("B200_LATENT_MMA", "1") != "0")
        if mma_ok:
            fn = nv.proto("b200_latent_attn_mma", [vp, vp, vp, i32, vp, vp, vp, i32, vp, vp, vp, i32, i32, i32, i32, f32, i32, i32, vp])
            if pieces is not None:
                nv.check(fn(nv.ptr(qx), nv.ptr(cache), nv.ptr(pieces.tiles), pieces.n_tiles, None, None, nv.ptr(table), table.shape[1],
                            nv.ptr(sinks), nv.ptr(out), None, H, Dk, Dv, BS, scale, 1, nv.dtype_code(qx.dtype), nv.stream()),
                         "latent_attn_mma")
                nv.count_launch()
                return out
            hb = 1
            while hb < min(H, 64):
                hb *= 2
            ctas = T * -(-H // hb)
            nsplit = 1
            if max_pos > 2 * _SPLIT_KEYS and ctas < 296:
                nsplit = min(32, -(-max_pos // _SPLIT_KEYS), max(1, 296 // ctas))
            part = torch.empty(T * H * nsplit * (Dv + 2), dtype=torch.float32, device=qx.device) if nsplit > 1 else None
            nv.check(fn(nv.ptr(qx), nv.ptr(cache), None, T, nv.ptr(pos), nv.ptr(slot), nv.ptr(table), table.shape[1], nv.ptr(sinks),
                        nv.ptr(out), nv.ptr(part), H, Dk, Dv, BS, scale, nsplit, nv.dtype_code(qx.dtype), nv.stream()),
                     "latent_attn_mma")
            nv.count_launch(2 if nsplit > 1 else 1)
            return out
        fn = nv.proto("b200_latent_attn", [vp, vp, vp, vp, vp, i32, vp, vp, i32, i32, i32, i32, i32, f32, i32, vp])
        nv.check(fn(nv.ptr(qx), nv.ptr(cache), nv.ptr(pos), nv.ptr(slot), nv.ptr(table), table.shape[1], nv.ptr(sinks), nv.ptr(out),
                    T, H, Dk, Dv, BS, scale, nv.dtype_code(qx.dtype), nv.stream()), "latent_attn")
        nv.count_launch()
        return out
    # PyTorch path (CPU): one token at a time over its own row
    out = torch.empty(T, H, Dv, dtype=qx.dtype, device=qx.device)
    pl, sl = pos.tolist(), slot.tolist()
    for t in range(T):
        n = pl[t] + 1
        nb = -(-n // BS)
        rows = cache[table[sl[t], :nb].long(), 0].reshape(nb * BS, Dk)[:n].float()
        sc = (qx[t].float() @ rows.t()) * scale
        if sinks is not None:
            sc = torch.cat([sc, sinks.float().view(H, 1)], 1)
        p = sc.softmax(-1)
        if sinks is not None:
            p = p[:, :-1]
        out[t] = (p @ rows[:, :Dv]).to(qx.dtype)
    return out
