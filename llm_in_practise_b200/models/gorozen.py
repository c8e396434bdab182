"""Gorozen: a decoder-only language model of attention layers whose values are their own keys.

Layer i (tensors ``l<i>.*``), on a residual stream x kept in fp32, with an RMS norm before AND after each sublayer
(gains stored around zero, applied as 1 + w):

    x <- x + norm1b(attn(norm1(x)))          x <- x + norm2b(ff(norm2(x)))      (the second line only if the layer has an ff)

* attention: q = W_q h, k = W_k h, no value projection — the value of a key position is k as projected, before it is
  rotated. Grouped query heads; rotary embedding on the first ``rot.dims`` dimensions of q and k in the interleaved pair
  layout, with the three-band frequency rescaling of ``rot.scaling`` (short wavelengths kept, long ones divided by
  ``factor``, a linear blend between); causal; score scale from the config; a learned per-head sink logit in the softmax
  denominator.
* ff, dense: g = min(W_g h, limit), u = clamp(W_u h, ±limit), W_d (g · sigmoid(1.702 g) · (u + 1)).
* ff, mixture of experts: fp32 router with bias, the ``top`` largest logits, softmax over those; SwiGLU experts.
* output: final norm, head, then logits <- cap · tanh(logits / cap).

Everything the config gives per layer (head counts and sizes, rotary sizes, ff kind and sizes, layer order) is read per
layer, so the KV cache is sized layer by layer too. The compute path is the ragged serving step
(``forward_ragged``): tokens of any mix of sequences, K/V in the paged cache (``ops/paged_attention.py``), the
sandwich norms fused around the fp32 stream (``ops/norm.sandwich_norm``), q|k and gate|up as single projections, experts
as grouped GEMMs (``ops/moe.gated_moe_ffn``). ``inference/ragged.RaggedGenerator`` and ``serve/engine.LLMEngine`` drive it.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import List, Optional

import torch
from torch import nn

from ..ops import elementwise as ew
from ..ops.gemm import linear_exact
from ..ops.linear import FusedLinear
from ..ops.moe import ROUTE_SOFTMAX_SELECTED, gated_moe_ffn, route_topk
from ..ops.norm import sandwich_norm
from ..ops.paged_attention import paged_attention, rope_paged_store

GELU_SIGMOID_ALPHA = 1.702        # g * sigmoid(1.702 g): the sigmoid approximation of GELU, fixed by the design


@dataclass
class GorozenAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot_dims: int
    rot_base: float
    rot_scaling: Optional[dict] = None          # {"factor", "low", "high", "original"} or None


@dataclass
class GorozenFF:
    kind: str                                   # "dense" | "moe"
    ff: int
    limit: float = 0.0                          # dense: clamp of gate / up
    experts: int = 0
    top: int = 0


@dataclass
class GorozenLayerSpec:
    type: str
    mixer: GorozenAttention
    mlp: Optional[GorozenFF]


@dataclass
class GorozenConfig:
    vocab_size: int
    hidden_size: int
    layers: List[GorozenLayerSpec]
    norm_eps: float
    logit_softcap: Optional[float] = None
    model_type: str = "gorozen"
    raw: dict = field(default_factory=dict, repr=False)

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    def to_dict(self) -> dict:
        return dict(self.raw)

    @classmethod
    def from_dict(cls, d: dict) -> "GorozenConfig":
        layers = []
        for L in d["layers"]:
            if L["type"] != "attention":
                raise ValueError(f"Gorozen has no mixer {L['type']!r}")
            m = L["mixer"]
            rot = m.get("rot") or {}
            att = GorozenAttention(heads=int(m["heads"]), kv_heads=int(m["kv_heads"]), dim=int(m["dim"]),
                                   vdim=int(m.get("vdim", m["dim"])), scale=float(m["scale"]), rot_dims=int(rot.get("dims", 0)),
                                   rot_base=float(rot.get("base", 10000.0)), rot_scaling=rot.get("scaling") or None)
            if att.vdim != att.dim:
                raise ValueError("values are the keys: vdim must equal dim")
            if att.heads % att.kv_heads or att.rot_dims % 2 or att.rot_dims > att.dim:
                raise ValueError("bad head / rotary sizes")
            f = L.get("mlp")
            ff = None
            if f is not None:
                if f["kind"] == "dense":
                    ff = GorozenFF("dense", int(f["ff"]), limit=float(f["limit"]))
                elif f["kind"] == "moe":
                    ff = GorozenFF("moe", int(f["expert"]["ff"]), experts=int(f["router"]["experts"]), top=int(f["router"]["top"]))
                else:
                    raise ValueError(f"unknown feed-forward kind {f['kind']!r}")
            layers.append(GorozenLayerSpec(L["type"], att, ff))
        return cls(vocab_size=int(d["vocab"]), hidden_size=int(d["width"]), layers=layers, norm_eps=float(d["norm"]["eps"]),
                   logit_softcap=d.get("logit_softcap"), raw=d)


def _hf_rope_scaling(s: Optional[dict]) -> Optional[dict]:
    """The design's {factor, low, high, original} in the key names ``ops.elementwise.rope_inv_freq`` reads."""
    if not s:
        return None
    return {"rope_type": "llama3", "factor": float(s["factor"]), "low_freq_factor": float(s["low"]),
            "high_freq_factor": float(s["high"]), "original_max_position_embeddings": int(s["original"])}


class GorozenLayer(nn.Module):
    def __init__(self, cfg: GorozenConfig, idx: int, dtype, device):
        super().__init__()
        spec = cfg.layers[idx]
        a, f, W = spec.mixer, spec.mlp, cfg.hidden_size
        self.spec, self.idx = spec, idx
        mk = lambda n: nn.Parameter(torch.zeros(n, dtype=dtype, device=device))          # noqa: E731
        self.norm1, self.norm1b = mk(W), mk(W)
        self.qk_proj = FusedLinear(W, [("q", a.heads * a.dim), ("k", a.kv_heads * a.dim)], dtype=dtype, device=device)
        self.o_proj = FusedLinear(a.heads * a.vdim, [("o", W)], dtype=dtype, device=device)
        self.sink = nn.Parameter(torch.zeros(a.heads, dtype=torch.float32, device=device))
        if f is not None:
            self.norm2, self.norm2b = mk(W), mk(W)
        if f is not None and f.kind == "dense":
            self.gate_up_proj = FusedLinear(W, [("gate", f.ff), ("up", f.ff)], dtype=dtype, device=device)
            self.down_proj = FusedLinear(f.ff, [("down", W)], dtype=dtype, device=device)
        elif f is not None:
            self.router = nn.Parameter(torch.zeros(f.experts, W, dtype=torch.float32, device=device))
            self.router_bias = nn.Parameter(torch.zeros(f.experts, dtype=torch.float32, device=device))
            self.experts_gate_up = nn.Parameter(torch.empty(f.experts, 2 * f.ff, W, dtype=dtype, device=device).normal_(std=0.02))
            self.experts_down = nn.Parameter(torch.empty(f.experts, W, f.ff, dtype=dtype, device=device).normal_(std=0.02))

    def fused_linears(self):
        d = {"qk_proj": self.qk_proj, "o_proj": self.o_proj}
        if hasattr(self, "gate_up_proj"):
            d.update(gate_up_proj=self.gate_up_proj, down_proj=self.down_proj)
        return d

    def feed_forward(self, h: torch.Tensor) -> torch.Tensor:
        """h [T, W] (already normed) -> the sublayer's output in fp32 [T, W]."""
        f = self.spec.mlp
        if f.kind == "dense":
            gu = linear_exact(h, self.gate_up_proj.weight)
            return linear_exact(ew.clamped_glu(gu, f.limit, GELU_SIGMOID_ALPHA, 1.0), self.down_proj.weight, out_dtype=torch.float32)
        top_i, top_p = route_topk(h, self.router, self.router_bias, f.top, ROUTE_SOFTMAX_SELECTED)
        return gated_moe_ffn(h, top_i, top_p, self.experts_gate_up, self.experts_down, ew.clamped_glu)


class GorozenForCausalLM(nn.Module):
    """``forward_ragged`` is the serving step; ``forward(input_ids)`` runs whole sequences through the same step."""
    ragged = True                                   # served by inference.ragged.RaggedGenerator

    def __init__(self, cfg: GorozenConfig, dtype=torch.bfloat16, device=None, init_std: float = 0.02):
        super().__init__()
        self.config = cfg
        self.dtype_ = dtype
        W, V = cfg.hidden_size, cfg.vocab_size
        self.embed_tokens = nn.Parameter(torch.empty(V, W, dtype=dtype, device=device).normal_(std=init_std))
        self.layers = nn.ModuleList([GorozenLayer(cfg, i, dtype, device) for i in range(len(cfg.layers))])
        self.norm = nn.Parameter(torch.zeros(W, dtype=dtype, device=device))
        self.lm_head = nn.Parameter(torch.empty(V, W, dtype=dtype, device=device).normal_(std=init_std))
        self._rope = {}

    @property
    def device(self) -> torch.device:
        return self.embed_tokens.device

    def head_weight(self) -> torch.Tensor:
        return self.lm_head

    def kv_layout(self):
        """(kv heads, head size) of every layer: what the cache manager sizes its per-layer pools from."""
        return [(s.mixer.kv_heads, s.mixer.dim) for s in self.config.layers]

    def rope(self, li: int, device, need: int):
        a = self.config.layers[li].mixer
        key = (a.rot_dims, a.rot_base, json.dumps(a.rot_scaling, sort_keys=True), str(device))
        t = self._rope.get(key)
        if t is None or t[0].shape[0] < need:
            n = max(need, 4096)
            t = self._rope[key] = ew.rope_tables_partial(n, a.rot_dims, a.rot_base, device, _hf_rope_scaling(a.rot_scaling))
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
        eps = cfg.norm_eps
        dev = ids.device
        need = max(int(max_pos) + 1, cache.max_len)
        layers = self.layers
        h, x = sandwich_norm(ew.embedding(ids, self.embed_tokens), None, None, layers[0].norm1 if len(layers) else self.norm, eps, 1.0, dt)
        for li, layer in enumerate(layers):
            a = layer.spec.mixer
            nxt = layers[li + 1].norm1 if li + 1 < len(layers) else self.norm
            qk = linear_exact(h, layer.qk_proj.weight)
            if a.rot_dims:
                cos, sin = self.rope(li, dev, need)
            else:
                cos = sin = torch.zeros(1, 1, dtype=torch.float32, device=dev)
            rope_paged_store(qk, cos, sin, pos, slot, cache.k[li], cache.v[li], cache.table, a.heads, a.kv_heads, a.dim,
                             a.rot_dims, interleaved=True, v_from_k=True)
            ctx = paged_attention(qk, cache.k[li], cache.v[li], cache.table, pos, slot, a.heads, a.kv_heads, a.dim, a.scale,
                                  sinks=layer.sink, max_pos=max_pos, pieces=pieces)
            y = linear_exact(ctx, layer.o_proj.weight, out_dtype=torch.float32)
            if layer.spec.mlp is None:
                h, x = sandwich_norm(y, layer.norm1b, x, nxt, eps, 1.0, dt)
            else:
                h, x = sandwich_norm(y, layer.norm1b, x, layer.norm2, eps, 1.0, dt)
                h, x = sandwich_norm(layer.feed_forward(h), layer.norm2b, x, nxt, eps, 1.0, dt)
            if layer_outputs is not None:
                layer_outputs.append(x)
        if want is not None:
            h = h.index_select(0, want)
        logits = linear_exact(h.contiguous(), self.lm_head, out_dtype=torch.float32)
        return ew.softcap_(logits, cfg.logit_softcap)

    @torch.no_grad()
    def forward(self, input_ids: torch.Tensor, labels=None, **_) -> dict:
        """Whole sequences [B, S] through the serving step with a throw-away cache: ``{"logits": [B, S, V]}`` (fp32)."""
        if labels is not None:
            raise NotImplementedError("Gorozen is an inference model here: no loss / backward")
        from ..inference.ragged import RaggedGenerator
        B, S = input_ids.shape
        gen = RaggedGenerator(self, None, max_len=S)
        cache = gen.make_cache(num_blocks=B * (-(-S // 64)), block_size=64, max_seqs=B, max_len=S)
        for b in range(B):
            gen.set_block_row(cache, b, list(range(1 + b * (-(-S // 64)), 1 + (b + 1) * (-(-S // 64)))))
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
@torch.no_grad()
def load_gorozen_weights(model: GorozenForCausalLM, path: str) -> None:
    from ..io.safetensors import safe_open
    dev, dt = model.embed_tokens.device, model.embed_tokens.dtype
    with safe_open(os.path.join(path, "model.safetensors")) as f:
        names = set(f.keys())
        used = set()

        def get(name, dtype=dt):
            used.add(name)
            return f.get_tensor(name).to(dev, dtype)

        model.embed_tokens.copy_(get("embed"))
        model.norm.copy_(get("final.norm"))
        model.lm_head.copy_(get("head"))
        for i, layer in enumerate(model.layers):
            p = f"l{i}."
            spec = layer.spec
            layer.norm1.copy_(get(p + "norm1"))
            layer.norm1b.copy_(get(p + "norm1b"))
            layer.qk_proj.weight.copy_(torch.cat([get(p + "mix.q"), get(p + "mix.k")], 0))
            layer.o_proj.weight.copy_(get(p + "mix.o"))
            layer.sink.copy_(get(p + "mix.sink", torch.float32))
            if spec.mlp is None:
                continue
            layer.norm2.copy_(get(p + "norm2"))
            layer.norm2b.copy_(get(p + "norm2b"))
            if spec.mlp.kind == "dense":
                layer.gate_up_proj.weight.copy_(torch.cat([get(p + "mlp.gate"), get(p + "mlp.up")], 0))
                layer.down_proj.weight.copy_(get(p + "mlp.down"))
            else:
                layer.router.copy_(get(p + "mlp.router", torch.float32))
                layer.router_bias.copy_(get(p + "mlp.router.b", torch.float32))
                for e in range(spec.mlp.experts):
                    q = f"{p}mlp.e{e}."
                    layer.experts_gate_up[e].copy_(torch.cat([get(q + "gate"), get(q + "up")], 0))
                    layer.experts_down[e].copy_(get(q + "down"))
        missing = names - used
        if missing:
            raise ValueError(f"checkpoint tensors the model has no place for: {sorted(missing)[:8]}")


def gorozen_from_pretrained(path: str, dtype=torch.bfloat16, device=None) -> GorozenForCausalLM:
    with open(os.path.join(path, "config.json")) as f:
        cfg = GorozenConfig.from_dict(json.load(f))
    model = GorozenForCausalLM(cfg, dtype=dtype, device=device)
    load_gorozen_weights(model, path)
    model.name_or_path = path
    return model.eval()


@torch.no_grad()
def gorozen_state_dict(model: GorozenForCausalLM) -> dict:
    """Tensors under the checkpoint's names (the inverse of ``load_gorozen_weights``)."""
    out = {"embed": model.embed_tokens, "final.norm": model.norm, "head": model.lm_head}
    for i, layer in enumerate(model.layers):
        p, a, f = f"l{i}.", layer.spec.mixer, layer.spec.mlp
        out[p + "norm1"], out[p + "norm1b"] = layer.norm1, layer.norm1b
        nq = a.heads * a.dim
        out[p + "mix.q"], out[p + "mix.k"] = layer.qk_proj.weight[:nq], layer.qk_proj.weight[nq:]
        out[p + "mix.o"], out[p + "mix.sink"] = layer.o_proj.weight, layer.sink
        if f is None:
            continue
        out[p + "norm2"], out[p + "norm2b"] = layer.norm2, layer.norm2b
        if f.kind == "dense":
            out[p + "mlp.gate"], out[p + "mlp.up"] = layer.gate_up_proj.weight[:f.ff], layer.gate_up_proj.weight[f.ff:]
            out[p + "mlp.down"] = layer.down_proj.weight
        else:
            out[p + "mlp.router"], out[p + "mlp.router.b"] = layer.router, layer.router_bias
            for e in range(f.experts):
                out[f"{p}mlp.e{e}.gate"], out[f"{p}mlp.e{e}.up"] = layer.experts_gate_up[e, :f.ff], layer.experts_gate_up[e, f.ff:]
                out[f"{p}mlp.e{e}.down"] = layer.experts_down[e]
    return {k: v.detach().contiguous() for k, v in out.items()}
