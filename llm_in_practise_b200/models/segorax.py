"""Segorax: a decoder-only language model of latent-attention layers on an un-normed residual stream.

Layer i (tensors ``l<i>.*``) works on a residual stream x kept in fp32. The sublayers read x itself; only their outputs are
normed (RMS, plain gains), scaled by the config's ``residual_mult`` m and added:

    x <- x + m * norm1(mixer(x))          x <- x + m * norm2(ff(x))          (the second line only if the layer has an ff)

The stream starts as ``embed[token] * embedding.scale``; the output is ``head(final_norm(x)) * logit_scale``.

* mixer, both kinds: the token is projected to a latent c = RMSnorm(W_dkv h)[:C] and one rotated key part r (the last R rows
  of W_dkv h, not normed, rotary in the interleaved pair layout) shared by all heads; head h's key is [W_uk_h c | r], its
  value W_uv_h c, its query [q_h (D un-rotated dims) | rot(q_h) (R dims)]; causal; score scale from the config.
  - ``latent_attention``: the queries come through a latent too, q = W_uq RMSnorm(W_dq h); a learned per-head sink logit
    sits in the softmax denominator.
  - ``latent_attention_2``: q = W_q h; the rotary frequencies are rescaled (``rot.scaling``: slow dims divided by
    ``factor`` through a ramp between the dims whose wavelengths are ``original / fast`` and ``original / slow``; cos and
    sin grow by 0.1 ln(factor) + 1); ordinary softmax.
* ff, dense: W_down (gelu_tanh(W_gate h) * W_up h).
* ff, mixture of experts: sigmoid router in fp32; the choice is made on the scores plus a per-expert correction, within the
  ``groups.keep`` best of ``groups.count`` groups of neighbouring experts (a group's rank: the sum of its two largest
  choice scores); the weights are the chosen experts' plain scores; experts are W_down gelu(W_up h) (erf form); a shared
  expert of the same form runs for every token, weighted by sigmoid(W_sg h).

Only [c | r] is cached (``kv_layout``: one row of C + R per token and layer, no value pool), and the compute path never
expands keys or values: ``forward_ragged`` carries the queries into the latent space (``ops.gemm.head_linear`` with W_uk),
attends over the cached rows (``ops.latent_attention``) and expands the latent context with W_uv. The post-norm, the
residual add and the cast for the next GEMM are one pass (``ops.norm.sandwich_norm``); W_dq | W_dkv, gate | up and
router | shared gate are single projections; experts run as grouped GEMMs (``ops.moe.gated_moe_ffn``).
``inference/ragged.RaggedGenerator`` and ``serve/engine.LLMEngine`` drive it.
"""
from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass, field
from typing import List, Optional

import torch
from torch import nn

from ..ops import elementwise as ew
from ..ops.gemm import head_linear, linear_exact
from ..ops.latent_attention import latent_attention, latent_kv_store, latent_q_rope
from ..ops.linear import FusedLinear
from ..ops.moe import gated_moe_ffn, route_sigmoid_grouped
from ..ops.norm import sandwich_norm

GROUP_TOP = 2                     # a group of experts is ranked by the sum of its two largest choice scores: fixed by the design
MIXERS = ("latent_attention", "latent_attention_2")


@dataclass
class SegoraxAttention:
    kind: str                                   # "latent_attention" (query latent, sinks) | "latent_attention_2" (scaled rotary)
    heads: int
    dim: int                                    # un-rotated query / key dims per head
    rot_dim: int                                # rotated query / key dims per head (the key's are shared by all heads)
    vdim: int
    kv_rank: int
    q_rank: int                                 # 0: queries are projected directly
    scale: float
    rot_dims: int
    rot_base: float
    rot_scaling: Optional[dict] = None          # {"factor", "original", "fast", "slow"} or None

    @property
    def has_sink(self) -> bool:
        return self.kind == "latent_attention"


@dataclass
class SegoraxFF:
    kind: str                                   # "dense" | "moe"
    ff: int
    experts: int = 0
    top: int = 0
    groups: int = 1
    keep: int = 1
    shared_ff: int = 0


@dataclass
class SegoraxLayerSpec:
    type: str
    mixer: SegoraxAttention
    mlp: Optional[SegoraxFF]


@dataclass
class SegoraxConfig:
    vocab_size: int
    hidden_size: int
    layers: List[SegoraxLayerSpec]
    norm_eps: float
    embed_scale: float = 1.0
    residual_mult: float = 1.0
    logit_scale: float = 1.0
    model_type: str = "segorax"
    raw: dict = field(default_factory=dict, repr=False)

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    def to_dict(self) -> dict:
        return dict(self.raw)

    @classmethod
    def from_dict(cls, d: dict) -> "SegoraxConfig":
        layers = []
        for L in d["layers"]:
            if L["type"] not in MIXERS:
                raise ValueError(f"Segorax has no mixer {L['type']!r}")
            m = L["mixer"]
            rot = m.get("rot") or {}
            kind = L["type"]
            att = SegoraxAttention(kind=kind, heads=int(m["heads"]), dim=int(m["dim"]), rot_dim=int(m["rot_dim"]), vdim=int(m["vdim"]),
                                   kv_rank=int(m["kv_rank"]), q_rank=int(m["q_rank"]) if kind == "latent_attention" else 0,
                                   scale=float(m["scale"]), rot_dims=int(rot.get("dims", m["rot_dim"])),
                                   rot_base=float(rot.get("base", 10000.0)),
                                   rot_scaling=(rot.get("scaling") or None) if kind == "latent_attention_2" else None)
            if att.rot_dims % 2 or att.rot_dims > att.rot_dim:
                raise ValueError("bad rotary sizes")
            f = L.get("mlp")
            ff = None
            if f is not None:
                if f["kind"] == "dense":
                    ff = SegoraxFF("dense", int(f["ff"]))
                elif f["kind"] == "moe":
                    r = f["router"]
                    g = r.get("groups") or {}
                    ff = SegoraxFF("moe", int(f["expert"]["ff"]), experts=int(r["experts"]), top=int(r["top"]), groups=int(g.get("count", 1)),
                                   keep=int(g.get("keep", g.get("count", 1))), shared_ff=int((f.get("shared") or {}).get("ff", 0)))
                    if ff.experts % ff.groups or ff.keep > ff.groups or ff.top > ff.keep * (ff.experts // ff.groups):
                        raise ValueError("bad expert groups")
                else:
                    raise ValueError(f"unknown feed-forward kind {f['kind']!r}")
            layers.append(SegoraxLayerSpec(kind, att, ff))
        return cls(vocab_size=int(d["vocab"]), hidden_size=int(d["width"]), layers=layers, norm_eps=float(d["norm"]["eps"]),
                   embed_scale=float((d.get("embedding") or {}).get("scale", 1.0)), residual_mult=float(d.get("residual_mult", 1.0)),
                   logit_scale=float(d.get("logit_scale", 1.0)), raw=d)


def _yarn_scaling(s: Optional[dict]) -> Optional[dict]:
    """The design's {factor, original, fast, slow} in the key names ``ops.elementwise.rope_inv_freq`` reads; cos and sin are
    multiplied by 0.1 ln(factor) + 1 whatever the factor."""
    if not s:
        return None
    return {"rope_type": "yarn", "factor": float(s["factor"]), "original_max_position_embeddings": int(s["original"]),
            "beta_fast": float(s["fast"]), "beta_slow": float(s["slow"]), "attention_factor": 0.1 * math.log(float(s["factor"])) + 1.0}


class SegoraxLayer(nn.Module):
    def __init__(self, cfg: SegoraxConfig, idx: int, dtype, device):
        super().__init__()
        spec = cfg.layers[idx]
        a, f, W = spec.mixer, spec.mlp, cfg.hidden_size
        self.spec, self.idx = spec, idx
        mk = lambda *n, dt=dtype: nn.Parameter(torch.zeros(*n, dtype=dt, device=device))          # noqa: E731
        self.norm1 = mk(W)
        H, D, R, C = a.heads, a.dim, a.rot_dim, a.kv_rank
        # W_dq | W_dkv as one projection (fp32 out: its rows are normed next); direct queries ride in front of W_dkv instead
        if a.q_rank:
            self.down_proj_a = FusedLinear(W, [("dq", a.q_rank), ("dkv", C + R)], dtype=dtype, device=device)
            self.q_norm = mk(a.q_rank)
            self.uq_proj = FusedLinear(a.q_rank, [("uq", H * (D + R))], dtype=dtype, device=device)
        else:
            self.down_proj_a = FusedLinear(W, [("dkv", C + R)], dtype=dtype, device=device)
            self.q_proj = FusedLinear(W, [("q", H * (D + R))], dtype=dtype, device=device)
        self.kv_norm = mk(C)
        self.w_uk = mk(H, D, C)                        # per head [D, C]: applied transposed to carry q into the latent space
        self.w_uv = mk(H, a.vdim, C)
        self.o_proj = FusedLinear(H * a.vdim, [("o", W)], dtype=dtype, device=device)
        if a.has_sink:
            self.sink = mk(H, dt=torch.float32)
        if f is not None:
            self.norm2 = mk(W)
        if f is not None and f.kind == "dense":
            self.gate_up_proj = FusedLinear(W, [("gate", f.ff), ("up", f.ff)], dtype=dtype, device=device)
            self.down_proj = FusedLinear(f.ff, [("down", W)], dtype=dtype, device=device)
        elif f is not None:
            gate_rows = 1 if f.shared_ff else 0
            self.router = mk(f.experts + gate_rows, W, dt=torch.float32)         # router rows, then the shared expert's gate row
            self.correction = mk(f.experts, dt=torch.float32)
            self.experts_up = mk(f.experts, f.ff, W)
            self.experts_down = mk(f.experts, W, f.ff)
            if f.shared_ff:
                self.shared_up = FusedLinear(W, [("up", f.shared_ff)], dtype=dtype, device=device)
                self.shared_down = FusedLinear(f.shared_ff, [("down", W)], dtype=dtype, device=device)

    def fused_linears(self):
        d = {"down_proj_a": self.down_proj_a, "o_proj": self.o_proj}
        for n in ("uq_proj", "q_proj", "gate_up_proj", "down_proj", "shared_up", "shared_down"):
            if hasattr(self, n):
                d[n] = getattr(self, n)
        return d

    def mixer(self, h, cos, sin, pos, slot, cache_rows, table, eps, max_pos, pieces):
        """h [T, W] (the stream in the compute dtype) -> the mixer's output in fp32 [T, W]; the step's [c | r] rows are
        stored in ``cache_rows`` on the way."""
        a = self.spec.mixer
        H, D, R, C, T = a.heads, a.dim, a.rot_dim, a.kv_rank, h.shape[0]
        dt = h.dtype
        low = linear_exact(h, self.down_proj_a.weight, out_dtype=torch.float32)
        cq = latent_kv_store(low, 0, a.q_rank, a.q_rank, C, R, a.rot_dims, self.q_norm if a.q_rank else None, self.kv_norm, eps,
                             cos, sin, pos, slot, cache_rows, table, dt)
        q = linear_exact(cq, self.uq_proj.weight) if a.q_rank else linear_exact(h, self.q_proj.weight)
        qx = torch.empty(T, H, C + R, dtype=dt, device=h.device)
        head_linear(q.view(T, H, D + R)[:, :, :D], self.w_uk, w_kn=True, out=qx[:, :, :C])
        latent_q_rope(q, cos, sin, pos, qx, H, D, R, a.rot_dims, C)
        ctx = latent_attention(qx, cache_rows, table, pos, slot, H, C, a.scale, sinks=self.sink if a.has_sink else None,
                               max_pos=max_pos, pieces=pieces)
        v = head_linear(ctx, self.w_uv)
        return linear_exact(v.view(T, H * a.vdim), self.o_proj.weight, out_dtype=torch.float32)

    def feed_forward(self, h: torch.Tensor) -> torch.Tensor:
        """h [T, W] -> the sublayer's output in fp32 [T, W]."""
        f = self.spec.mlp
        if f.kind == "dense":
            gu = linear_exact(h, self.gate_up_proj.weight)
            return linear_exact(ew.act_glu(gu, "gelu_tanh"), self.down_proj.weight, out_dtype=torch.float32)
        top_i, top_p, gate = route_sigmoid_grouped(h, self.router, self.correction, f.top, f.groups, f.keep, GROUP_TOP,
                                                   gate_rows=1 if f.shared_ff else 0)
        shared = None
        if f.shared_ff:
            shared = linear_exact(ew.gelu(linear_exact(h, self.shared_up.weight)), self.shared_down.weight)
        return gated_moe_ffn(h, top_i, top_p, self.experts_up, self.experts_down, ew.gelu, shared=shared, gate=gate)


class SegoraxForCausalLM(nn.Module):
    """``forward_ragged`` is the serving step; ``forward(input_ids)`` runs whole sequences through the same step."""
    ragged = True                                   # served by inference.ragged.RaggedGenerator

    def __init__(self, cfg: SegoraxConfig, dtype=torch.bfloat16, device=None, init_std: float = 0.02):
        super().__init__()
        self.config = cfg
        self.dtype_ = dtype
        W, V = cfg.hidden_size, cfg.vocab_size
        self.embed_tokens = nn.Parameter(torch.empty(V, W, dtype=dtype, device=device).normal_(std=init_std))
        self.layers = nn.ModuleList([SegoraxLayer(cfg, i, dtype, device) for i in range(len(cfg.layers))])
        self.norm = nn.Parameter(torch.ones(W, dtype=dtype, device=device))
        self.lm_head = nn.Parameter(torch.empty(V, W, dtype=dtype, device=device).normal_(std=init_std))
        self._rope = {}

    @property
    def device(self) -> torch.device:
        return self.embed_tokens.device

    def head_weight(self) -> torch.Tensor:
        return self.lm_head

    def kv_layout(self):
        """(kv heads, key row size, value row size) of every layer: one latent row per token, no value pool."""
        return [(1, s.mixer.kv_rank + s.mixer.rot_dim, 0) for s in self.config.layers]

    def rope(self, li: int, device, need: int):
        a = self.config.layers[li].mixer
        key = (a.rot_dims, a.rot_base, json.dumps(a.rot_scaling, sort_keys=True), str(device))
        t = self._rope.get(key)
        if t is None or t[0].shape[0] < need:
            n = max(need, 4096)
            t = self._rope[key] = ew.rope_tables_partial(n, a.rot_dims, a.rot_base, device, _yarn_scaling(a.rot_scaling))
        return t

    @torch.no_grad()
    def forward_ragged(self, ids: torch.Tensor, pos: torch.Tensor, slot: torch.Tensor, cache, want: Optional[torch.Tensor] = None,
                       max_pos: int = 0, pieces=None, layer_outputs: Optional[list] = None) -> torch.Tensor:
        """One serving step over a flat token list: ``ids`` long [T], ``pos`` / ``slot`` int32 [T] (position in its sequence
        and cache row of every token), ``cache`` a ``PagedKVCache`` whose table rows cover those positions. Returns fp32
        logits of the rows ``want`` (long [n]; default all). ``max_pos`` >= every position (host-side bound that sizes the
        rotary tables). ``layer_outputs``: a list that receives the residual stream after every layer."""
        cfg = self.config
        dt = self.embed_tokens.dtype
        eps, m = cfg.norm_eps, cfg.residual_mult
        dev = ids.device
        need = max(int(max_pos) + 1, cache.max_len)
        # the stream enters as embed * scale in fp32; h is the stream in the GEMMs' dtype (the stream itself in an fp32 run)
        h, x = sandwich_norm(ew.embedding(ids, self.embed_tokens), None, None, None, eps, 0.0, dt, branch_mult=cfg.embed_scale,
                             cast_next=True)
        for li, layer in enumerate(self.layers):
            a = layer.spec.mixer
            if a.rot_dims:
                cos, sin = self.rope(li, dev, need)
            else:
                cos = sin = torch.zeros(1, 1, dtype=torch.float32, device=dev)
            y = layer.mixer(h, cos, sin, pos, slot, cache.k[li], cache.table, eps, max_pos, pieces)
            h, x = sandwich_norm(y, layer.norm1, x, None, eps, 0.0, dt, branch_mult=m, cast_next=True)
            if layer.spec.mlp is not None:
                h, x = sandwich_norm(layer.feed_forward(h), layer.norm2, x, None, eps, 0.0, dt, branch_mult=m, cast_next=True)
            if layer_outputs is not None:
                layer_outputs.append(x)
        if want is not None:
            x = x.index_select(0, want)
        h, _ = sandwich_norm(None, None, x.contiguous(), self.norm, eps, 0.0, dt)
        return linear_exact(h, self.lm_head, out_dtype=torch.float32).mul_(cfg.logit_scale)

    @torch.no_grad()
    def forward(self, input_ids: torch.Tensor, labels=None, **_) -> dict:
        """Whole sequences [B, S] through the serving step with a throw-away cache: ``{"logits": [B, S, V]}`` (fp32)."""
        if labels is not None:
            raise NotImplementedError("Segorax is an inference model here: no loss / backward")
        from ..inference.ragged import RaggedGenerator
        B, S = input_ids.shape
        gen = RaggedGenerator(self, None, max_len=S)
        per = -(-S // 64)
        cache = gen.make_cache(num_blocks=B * per, block_size=64, max_seqs=B, max_len=S)
        for b in range(B):
            gen.set_block_row(cache, b, list(range(1 + b * per, 1 + (b + 1) * per)))
        logits = gen.step([(b, 0, input_ids[b].tolist(), list(range(S))) for b in range(B)], cache)
        return {"logits": logits.view(B, S, -1)}

    @torch.no_grad()
    def generate(self, input_ids: torch.Tensor, max_new_tokens: int = 256, **kw) -> torch.Tensor:
        from ..inference.ragged import RaggedGenerator
        g = self.__dict__.get("_generator")
        need = input_ids.shape[1] + int(max_new_tokens)
        if g is None or g.max_len < need:
            g = self.__dict__["_generator"] = RaggedGenerator(self, None, max(need, 4096))
        return g.generate(input_ids.to(self.device), max_new_tokens=max_new_tokens, **kw)

    def num_parameters(self, only_trainable: bool = False) -> int:
        return sum(p.numel() for p in self.parameters() if p.requires_grad or not only_trainable)


# ------------------------------------------------------------------------------------------------------------------
# checkpoint: config.json + model.safetensors with the design's own tensor names
# ------------------------------------------------------------------------------------------------------------------
def _tensor_map(model: SegoraxForCausalLM):
    """(checkpoint name, parameter, slice of its first dim or None, shape in the file or None) for every tensor."""
    out = [("embed", model.embed_tokens, None, None), ("final.norm", model.norm, None, None), ("head", model.lm_head, None, None)]
    for i, layer in enumerate(model.layers):
        p, a, f = f"l{i}.", layer.spec.mixer, layer.spec.mlp
        H, D, R, C = a.heads, a.dim, a.rot_dim, a.kv_rank
        out.append((p + "norm1", layer.norm1, None, None))
        if a.q_rank:
            out += [(p + "mix.dq", layer.down_proj_a.weight, slice(0, a.q_rank), None),
                    (p + "mix.dkv", layer.down_proj_a.weight, slice(a.q_rank, a.q_rank + C + R), None),
                    (p + "mix.dq.norm", layer.q_norm, None, None), (p + "mix.uq", layer.uq_proj.weight, None, None)]
        else:
            out += [(p + "mix.dkv", layer.down_proj_a.weight, None, None), (p + "mix.q", layer.q_proj.weight, None, None)]
        out += [(p + "mix.dkv.norm", layer.kv_norm, None, None), (p + "mix.uk", layer.w_uk, None, (H * D, C)),
                (p + "mix.uv", layer.w_uv, None, (H * a.vdim, C)), (p + "mix.o", layer.o_proj.weight, None, None)]
        if a.has_sink:
            out.append((p + "mix.sink", layer.sink, None, None))
        if f is None:
            continue
        out.append((p + "norm2", layer.norm2, None, None))
        if f.kind == "dense":
            out += [(p + "mlp.gate", layer.gate_up_proj.weight, slice(0, f.ff), None),
                    (p + "mlp.up", layer.gate_up_proj.weight, slice(f.ff, 2 * f.ff), None),
                    (p + "mlp.down", layer.down_proj.weight, None, None)]
            continue
        out += [(p + "mlp.router", layer.router, slice(0, f.experts), None), (p + "mlp.correction", layer.correction, None, None)]
        for e in range(f.experts):
            out += [(f"{p}mlp.e{e}.up", layer.experts_up, e, None), (f"{p}mlp.e{e}.down", layer.experts_down, e, None)]
        if f.shared_ff:
            out += [(p + "mlp.shared.up", layer.shared_up.weight, None, None), (p + "mlp.shared.down", layer.shared_down.weight, None, None),
                    (p + "mlp.shared.sg", layer.router, slice(f.experts, f.experts + 1), None)]
    return out


@torch.no_grad()
def load_segorax_weights(model: SegoraxForCausalLM, path: str) -> None:
    from ..io.safetensors import safe_open
    with safe_open(os.path.join(path, "model.safetensors")) as f:
        names = set(f.keys())
        used = set()
        for name, param, sl, shape in _tensor_map(model):
            used.add(name)
            dst = param if sl is None else param[sl]
            t = f.get_tensor(name).to(param.device, param.dtype)
            dst.copy_(t.view(dst.shape) if shape is not None else t)
        missing = names - used
        if missing:
            raise ValueError(f"checkpoint tensors the model has no place for: {sorted(missing)[:8]}")


def segorax_from_pretrained(path: str, dtype=torch.bfloat16, device=None) -> SegoraxForCausalLM:
    with open(os.path.join(path, "config.json")) as f:
        cfg = SegoraxConfig.from_dict(json.load(f))
    model = SegoraxForCausalLM(cfg, dtype=dtype, device=device)
    load_segorax_weights(model, path)
    model.name_or_path = path
    return model.eval()


@torch.no_grad()
def segorax_state_dict(model: SegoraxForCausalLM) -> dict:
    """Tensors under the checkpoint's names (the inverse of ``load_segorax_weights``)."""
    out = {}
    for name, param, sl, shape in _tensor_map(model):
        t = param if sl is None else param[sl]
        out[name] = (t.reshape(shape) if shape is not None else t).detach().contiguous()
    return out
