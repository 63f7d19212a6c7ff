"""Grouped-query attention over paged keys and values.

In execution order, as the reference runs it (crates/airun-core/src/runtime.rs:3833-4122):
q = Wq h, k = Wk h, v = Wv h without bias, head i in columns [i*hd, (i+1)*hd);
per-head RMSNorm of q and k with one shared weight vector each (when
``qk_norm``); the position encoding on q and k; k and v into the cache;
head h attends through KV head h / (num_heads / num_kv_heads) with
s_j = scale * q.K_j over keys j <= pos (and pos - j < window when window > 0);
then the output projection.  The three input projections run as one product
over the stacked matrix [Wq; Wk; Wv].

An entry of the execution order that reads another entry's cache computes q
only and attends over that cache.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import ops
from ..weights.loader import WeightSpec
from .base import Mixer, NormedActivations, PagedKVSpec, make_part, register_part
from .linear import linear, linear_into_residual


class GQAAttention(Mixer):
    device_driven = True

    fuses_norms = True        # takes NormedActivations as input and a ResidualSink for its output

    def __init__(self, prefix: str, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 scale: float, window: int = 0, qk_norm: bool = True, qk_norm_eps: float = 1e-6,
                 position: str = "rotary_neox", position_args: Optional[dict] = None,
                 dtype: torch.dtype = torch.bfloat16, device=None,
                 names: Optional[Dict[str, str]] = None):
        if num_heads % num_kv_heads:
            raise ValueError(f"num_heads ({num_heads}) must be a multiple of num_kv_heads ({num_kv_heads})")
        if head_dim > 256:
            raise ValueError(f"head_dim {head_dim} is above the attention kernels' limit of 256")
        self.prefix = prefix
        self.H, self.nh, self.nkv, self.hd = int(hidden_size), int(num_heads), int(num_kv_heads), int(head_dim)
        self.scale, self.window = float(scale), int(window)
        self.qk_norm, self.qk_norm_eps = bool(qk_norm), float(qk_norm_eps)
        self.dtype, self.device = dtype, device
        self.pos = make_part("position", position, prefix=prefix, dtype=dtype, device=device,
                             **(position_args or {}))
        n = dict(q="q_proj.weight", k="k_proj.weight", v="v_proj.weight", o="o_proj.weight",
                 q_norm="q_norm.weight", k_norm="k_norm.weight")
        n.update(names or {})
        self.names = {k: f"{prefix}.{v}" for k, v in n.items()}
        self.w_qkv = self.w_q = self.w_o = self.q_norm_w = self.k_norm_w = None

    # ---- weights ----
    def weight_specs(self) -> List[WeightSpec]:
        nm, H, qd, kd = self.names, self.H, self.nh * self.hd, self.nkv * self.hd
        specs = [WeightSpec(nm["q"], (qd, H)), WeightSpec(nm["k"], (kd, H)), WeightSpec(nm["v"], (kd, H)),
                 WeightSpec(nm["o"], (H, qd))]
        if self.qk_norm:
            specs += [WeightSpec(nm["q_norm"], (self.hd,), storage="float32", init="norm"),
                      WeightSpec(nm["k_norm"], (self.hd,), storage="float32", init="norm")]
        return specs + self.pos.weight_specs()

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        nm = self.names
        self.w_qkv = torch.cat([tensors.pop(nm["q"]), tensors.pop(nm["k"]), tensors.pop(nm["v"])], dim=0).contiguous()
        self.w_q = self.w_qkv[: self.nh * self.hd]
        self.w_o = tensors.pop(nm["o"])
        if self.qk_norm:
            self.q_norm_w, self.k_norm_w = tensors[nm["q_norm"]], tensors[nm["k_norm"]]
        self.pos.load_weights(tensors)

    # ---- cache ----
    def cache_spec(self):
        return PagedKVSpec(self.nkv, self.hd, self.window)

    # ---- compute ----
    def forward(self, ctx, h, cache, sink=None):
        T = h.h.shape[0] if isinstance(h, NormedActivations) else h.shape[0]
        ws = ctx.ws
        owns = not cache.shared
        width = (self.nh + 2 * self.nkv) * self.hd if owns else self.nh * self.hd
        qkv = ws.alloc((T, width), torch.float32)
        linear(ctx, h, self.w_qkv if owns else self.w_q, qkv)
        q = ws.alloc((T, self.nh * self.hd), self.dtype)
        kind, rdim, inv_freq = self.pos.fused()
        ops.qkv_post(qkv, q, self.q_norm_w, self.k_norm_w, self.qk_norm_eps, ctx.positions, ctx.req_of_token,
                     kind, rdim, inv_freq, cache.pool, cache.block_table, ctx.num_reqs, cache.page_size,
                     self.nh, self.nkv, self.hd, ctx.err, store=owns, kv_in_row=owns,
                     rope_positions=self.pos.rotation_positions(ctx))
        attn = ws.alloc((T, self.nh * self.hd), self.dtype)
        self.attend(ctx, q, attn, cache)
        fused = linear_into_residual(ctx, attn, self.w_o, sink)
        if fused is not None:
            return fused
        delta = ws.alloc((T, self.H), torch.float32)
        linear(ctx, attn, self.w_o, delta)
        return delta

    def attend(self, ctx, q: torch.Tensor, out: torch.Tensor, cache) -> None:
        if q.dtype == torch.bfloat16:
            from ..kernels import fast
            if fast.attention_bf16(ctx, q, out, cache, self.nh, self.nkv, self.hd, self.scale, self.window):
                return
        ops.attention_generic(q, out, cache.pool, cache.block_table, ctx.positions, ctx.req_of_token,
                              ctx.num_reqs, self.nh, self.nkv, self.hd, self.scale, self.window, ctx.err)


register_part("mixer", "gqa_attention", GQAAttention)
