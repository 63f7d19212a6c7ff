"""A decoder put together from parts, layer by layer, from a configuration.

The model is: token embedding, a list of layers (each an arrangement of norm,
mixer, feed-forward chosen by the configuration's ``layer_specs()``), an
execution order (a list of :class:`LayerCall`, which may name a layer twice or
let an entry read an earlier entry's cache), a final norm and an output head.
Tensor names come from the configuration's ``tensor_names()``.  The reference
assembles the same pieces per layer (crates/airun-core/src/model.rs:612-628,
crates/airun-core/src/runtime.rs:3482-3602) and keeps the output norm fused with
the last residual add (runtime.rs:3745-3746).
"""
from __future__ import annotations

import os
import sys
from typing import Dict, List, Optional, Tuple

import torch

from ..config.base import LayerCall, ModelConfig
from ..parts.base import make_part
from ..parts import embedding as _embedding_parts      # noqa: F401  (registers the embedding and head parts)
from ..weights.loader import (DictSource, TensorSource, WeightSpec, load_tensors, random_tensors)

# AIRUN_TRACE_LAYERS=1 prints the residual stream's rms and mean after every block (the reference's
# switch of the same name, crates/airun-core/src/runtime.rs:5265-5302).  Off by default.
TRACE_LAYERS = os.environ.get("AIRUN_TRACE_LAYERS", "") not in ("", "0")

DEFAULT_NAMES = dict(embed="model.embed_tokens.weight", layer="model.layers.{i}", mixer="self_attn",
                     ffn="mlp", norm1="input_layernorm", norm2="post_attention_layernorm",
                     final_norm="model.norm", head="lm_head.weight")


class DecoderModel:
    def __init__(self, config: ModelConfig, dtype: torch.dtype, device):
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"the engine computes in float32 or bfloat16, not {dtype}")
        self.config, self.dtype, self.device = config, dtype, torch.device(device)
        names = dict(DEFAULT_NAMES)
        names.update(getattr(config, "tensor_names", lambda: {})())
        self.names = names
        V, H = config.vocab_size, config.hidden_size
        self.V, self.H = V, H
        emb_name, emb_args = config.embedding() if hasattr(config, "embedding") else ("token_embedding", {})
        self.embedding = make_part("embedding", emb_name, prefix=names["embed"], vocab_size=V, hidden_size=H,
                                   dtype=dtype, device=self.device, **emb_args)
        self.layers = []
        for i, spec in enumerate(config.layer_specs()):
            p = names["layer"].format(i=i)
            common = dict(dtype=dtype, device=self.device)
            norm1 = make_part("norm", spec.norm, prefix=f"{p}.{names['norm1']}", **spec.norm_args, **common)
            norm2 = make_part("norm", spec.norm, prefix=f"{p}.{names['norm2']}", **spec.norm_args, **common)
            mixer = make_part("mixer", spec.mixer, prefix=f"{p}.{names['mixer']}", **spec.mixer_args, **common)
            ffn = make_part("feed_forward", spec.feed_forward, prefix=f"{p}.{names['ffn']}", **spec.ffn_args, **common)
            self.layers.append(make_part("arrangement", spec.arrangement, norm1=norm1, mixer=mixer,
                                         norm2=norm2, ffn=ffn, dtype=dtype))
        self.order: List[LayerCall] = list(config.execution_order())
        for c in self.order:
            if not (0 <= c.layer < len(self.layers)):
                raise ValueError(f"the execution order names layer {c.layer}, the model has {len(self.layers)}")
        fn_name, fn_args = config.final_norm() if hasattr(config, "final_norm") else \
            ("rmsnorm", dict(size=H, eps=config.rms_norm_eps))
        self.final_norm = make_part("norm", fn_name, prefix=names["final_norm"], dtype=dtype,
                                    device=self.device, **fn_args)
        tied = bool(getattr(config, "tie_word_embeddings", False))
        head_name, head_args = config.head() if hasattr(config, "head") else ("lm_head", {})
        self.head = make_part("head", head_name, prefix=names["head"], vocab_size=V, hidden_size=H,
                              tied_to=self.embedding if tied else None, dtype=dtype, device=self.device, **head_args)
        self.tied = tied

    # ---- weights ----
    def parts(self):
        return [self.embedding] + self.layers + [self.final_norm, self.head]

    def weight_specs(self) -> List[WeightSpec]:
        return [s for p in self.parts() for s in p.weight_specs()]

    def ignorable_tensors(self) -> List[str]:
        # a tied model's file may still carry the head; it is the same matrix
        return [self.names["head"]] if self.tied else []

    def load(self, source: TensorSource) -> None:
        tensors = load_tensors(self.weight_specs(), source, self.dtype, self.device, self.ignorable_tensors())
        for p in self.parts():
            p.load_weights(tensors)
        del tensors
        if self.device.type == "cuda":
            self.pack_weights()

    ARENA_ALIGN = 256

    def pack_weights(self) -> None:
        """Moves every tensor the parts hold (weights as the parts keep them: stacked, interleaved, tables)
        into ONE allocation, each at a 256-byte boundary, and gives the memory they came from back.  The
        reference keeps a layer's weights in one arena with 256-byte aligned sub-allocations for the same
        reasons: one allocation instead of hundreds, none of the allocator's rounding per tensor, and
        addresses that suit vector and bulk loads (crates/airun-core/src/model.rs:1332-1393).  Tensors that
        share memory (a tied head and the table; the q rows of the stacked q/k/v matrix) still do afterwards.
        Parts are found by walking the attributes of the model's parts, so a part needs nothing for it."""
        slots = []                                           # (holder, key, tensor): holder[key] or holder.key
        seen = set()

        def walk(obj):
            if id(obj) in seen:
                return
            seen.add(id(obj))
            items = vars(obj).items() if hasattr(obj, "__dict__") else ()
            for key, val in list(items):
                if isinstance(val, torch.Tensor):
                    if val.device == self.device:
                        slots.append((obj, key, val))
                elif isinstance(val, (list, tuple)):
                    if isinstance(val, list):
                        for i, v in enumerate(val):
                            if isinstance(v, torch.Tensor) and v.device == self.device:
                                slots.append((val, i, v))
                            elif hasattr(v, "weight_specs"):
                                walk(v)
                    else:
                        for v in val:
                            if hasattr(v, "weight_specs"):
                                walk(v)
                elif hasattr(val, "weight_specs"):
                    walk(val)

        for p in self.parts():
            walk(p)
        if not slots:
            return
        storages = {}                                        # storage address -> (bytes, offset in the arena)
        total = 0
        for _, _, t in slots:
            st = t.untyped_storage()
            if st.data_ptr() not in storages:
                storages[st.data_ptr()] = (st, total)
                total += (st.nbytes() + self.ARENA_ALIGN - 1) // self.ARENA_ALIGN * self.ARENA_ALIGN
        arena = torch.empty(total + self.ARENA_ALIGN, dtype=torch.uint8, device=self.device)
        base = (-arena.data_ptr()) % self.ARENA_ALIGN        # torch aligns to 512 bytes already; be sure of it
        moved = {}
        for ptr, (st, off) in storages.items():
            n = st.nbytes()
            dst = arena[base + off: base + off + n]
            dst.copy_(torch.empty(0, dtype=torch.uint8, device=self.device).set_(st, 0, (n,), (1,)))
            moved[ptr] = dst
        for holder, key, t in slots:
            dst = moved[t.untyped_storage().data_ptr()]
            esz = t.element_size()
            view = dst.view(t.dtype) if dst.numel() % esz == 0 else dst[: dst.numel() // esz * esz].view(t.dtype)
            new = torch.as_strided(view, t.shape, t.stride(), view.storage_offset() + t.storage_offset())
            if isinstance(holder, list):
                holder[key] = new
            else:
                setattr(holder, key, new)
        self.weight_arena = arena
        del storages, moved, slots
        torch.cuda.empty_cache()

    def load_random(self, seed: int) -> None:
        """Seeded random weights made on the model's device, through the same loading path."""
        tensors = random_tensors(self.weight_specs(), seed, self.device,
                                 torch.bfloat16)
        self.load(DictSource(tensors))

    def device_driven(self) -> bool:
        """True if every layer reads the batch's layout from the device arrays only, so that a step
        of a given padded size always launches the same kernels (and can be replayed from a graph)."""
        return all(getattr(l, "device_driven", lambda: False)() for l in self.layers) \
            and getattr(self.final_norm, "device_driven", False)

    def graph_safe(self) -> bool:
        """False if a part has said that its forward must not be captured into a CUDA graph (it
        decides on the host what to launch from values it reads back from the device)."""
        return all(getattr(l, "graph_safe", lambda: True)() for l in self.layers)

    # ---- cache needs ----
    def cache_specs(self) -> Tuple[List[object], List[Optional[int]]]:
        return ([self.layers[c.layer].cache_spec() for c in self.order],
                [c.cache_from for c in self.order])

    # ---- one pass over the given tokens ----
    def forward(self, ctx, want_rows: Optional[torch.Tensor], n_want: int) -> Optional[torch.Tensor]:
        T = ctx.num_tokens
        ctx.ws_main.reset()
        x = ctx.ws_main.alloc((T, self.H), torch.float32)
        self.embedding.forward(ctx, ctx.token_ids[:T], x)
        delta = None
        trace = TRACE_LAYERS and not torch.cuda.is_current_stream_capturing()
        for ci, call in enumerate(self.order):
            ctx.ws = ctx.ws_pair[ci % 2]
            ctx.ws.reset()
            nxt = self.layers[self.order[ci + 1].layer] if ci + 1 < len(self.order) else None
            next_norm = nxt.norm1 if (nxt is not None and getattr(nxt, "accepts_normed", lambda: False)()) else None
            if next_norm is not None:
                delta = self.layers[call.layer].forward(ctx, x, delta, ctx.caches[ci], next_norm=next_norm)
            else:
                delta = self.layers[call.layer].forward(ctx, x, delta, ctx.caches[ci])
            if trace:           # synchronises after every block: a debugging aid, as the reference's AIRUN_TRACE_LAYERS
                r = x[:ctx.num_tokens] if not isinstance(delta, torch.Tensor) else (x[:ctx.num_tokens] + delta[:ctx.num_tokens])
                print(f"[airun_b200] entry {ci} layer {call.layer}: rms {float(r.pow(2).mean().sqrt()):.6f} "
                      f"mean {float(r.mean()):+.6f}", file=sys.stderr)
        if n_want == 0:
            return None
        ctx.ws = ctx.ws_pair[len(self.order) % 2]
        ctx.ws.reset()
        hsel = ctx.ws.alloc((n_want, self.H), self.dtype)
        self.final_norm.forward(ctx, x, hsel, delta=delta, rows=want_rows[:n_want])
        logits = ctx.ws_main.alloc((n_want, self.V), torch.float32)
        self.head.forward(ctx, hsel, logits)
        return logits


def build_decoder(config: ModelConfig, dtype: torch.dtype, device) -> DecoderModel:
    return DecoderModel(config, dtype, device)
