"""A toy mixer with state of its own, a toy architecture that uses it, and an execution
order that names a layer twice and lets an entry read another entry's cache: all
registered from here, built and stepped without a change to the framework's files."""
from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass
from typing import Dict, List

import numpy as np
import pytest
import torch

import plain_qwen3 as P
from helpers import TINY, assert_close, random_tokens

pytestmark = pytest.mark.gpu


# ----------------------------------------------------------------------------- the toy parts
def define_toy():
    from airun_b200.config.base import LayerCall, LayerSpec, ModelConfig, register_architecture
    from airun_b200.config.qwen3 import Qwen3Config
    from airun_b200.engine.model import build_decoder
    from airun_b200.parts.base import Mixer, StateSpec, register_part
    from airun_b200.parts.linear import linear
    from airun_b200.weights.loader import WeightSpec

    class RunningMean(Mixer):
        """out[t] = W * mean(h[0..t]) of the request: the state is the running sum of h, one
        vector per request, zero when the request starts.  Works on any mix of portions and
        single tokens; padding rows (request -1) are ignored."""

        def __init__(self, prefix, hidden_size, dtype, device):
            self.prefix, self.H, self.dtype, self.device = prefix, hidden_size, dtype, device
            self.name = f"{prefix}.mix.weight"
            self.w = None

        def weight_specs(self):
            return [WeightSpec(self.name, (self.H, self.H))]

        def load_weights(self, tensors):
            self.w = tensors[self.name]

        def cache_spec(self):
            return StateSpec((self.H,), torch.float32)

        def forward(self, ctx, h, cache):
            T = h.shape[0]
            req = ctx.req_of_token[:T].long()
            valid = (req >= 0).unsqueeze(1)
            reqc = req.clamp(min=0)
            slots = ctx.state_slots.long()[reqc]
            hf = torch.where(valid, h.float(), torch.zeros((), device=h.device))
            c = torch.cumsum(hf, dim=0)
            start = ctx.cu_tokens.long()[reqc]                          # first row of the row's request
            before = torch.where((start > 0).unsqueeze(1), c[(start - 1).clamp(min=0)], torch.zeros((), device=h.device))
            total = cache.state[slots] + (c - before)                   # sum of h[0..t] of the request
            mean = total / (ctx.positions[:T].clamp(min=0).float().unsqueeze(1) + 1.0)
            cache.state.index_add_(0, slots, hf)                        # the state after this step
            out = ctx.ws.alloc((T, self.H), torch.float32)
            linear(ctx, mean.to(self.dtype), self.w, out)
            return out

    @dataclass(frozen=True)
    class ToyConfig(Qwen3Config):
        """Layer 0 is Qwen3 attention, layer 1 the running mean, layer 2 attention again; the
        order runs layer 2 twice, the second time reading the first run's cache."""

        def layer_specs(self):
            specs = Qwen3Config.layer_specs(self)
            s = specs[1]
            specs[1] = LayerSpec("toy_running_mean", dict(hidden_size=self.hidden_size), s.feed_forward,
                                 s.ffn_args, s.norm, s.norm_args)
            return specs

        def execution_order(self):
            return [LayerCall(0), LayerCall(1), LayerCall(2), LayerCall(2, cache_from=2)]

    register_part("mixer", "toy_running_mean", RunningMean)
    register_architecture("ToyMeanForCausalLM", ToyConfig, build_decoder)
    return ToyConfig


def plain_toy_forward(cfg: dict, W: Dict[str, torch.Tensor], tokens: List[int]) -> torch.Tensor:
    """The toy model, plainly: whole sequence, float32."""
    c = P.config_values(cfg)
    dt = torch.float32
    T = len(tokens)
    pos = list(range(T))
    x = P.plain_embedding(W["model.embed_tokens.weight"], tokens, dt)
    kvs = {}
    for entry, (l, src) in enumerate([(0, None), (1, None), (2, None), (2, 2)]):
        p = f"model.layers.{l}"
        h = P.plain_rmsnorm(x, W[f"{p}.input_layernorm.weight"], c["eps"])
        if l == 1:
            mean = torch.cumsum(h, 0) / torch.arange(1, T + 1, dtype=dt).unsqueeze(1)
            a = mean @ W[f"{p}.self_attn.mix.weight"].to(dt).T
        else:
            a, kv = P.plain_attention_layer(h, W, f"{p}.self_attn", c, pos, 0,
                                            kv_override=None if src is None else kvs[src])
            kvs[entry] = kv
        x = x + a
        h = P.plain_rmsnorm(x, W[f"{p}.post_attention_layernorm.weight"], c["eps"])
        x = x + P.plain_swiglu_ffn(h, W[f"{p}.mlp.gate_proj.weight"].to(dt), W[f"{p}.mlp.up_proj.weight"].to(dt),
                                   W[f"{p}.mlp.down_proj.weight"].to(dt))
    h = P.plain_rmsnorm(x, W["model.norm.weight"], c["eps"])
    return h @ W["lm_head.weight"].to(dt).T


@pytest.fixture(scope="module")
def toy(tmp_path_factory):
    ToyConfig = define_toy()
    from airun_b200.engine.model import DecoderModel
    from airun_b200.weights import write_model_folder
    d = dict(TINY["B"]["cfg"], architectures=["ToyMeanForCausalLM"])
    cfg = ToyConfig.from_dict(d)
    folder = str(tmp_path_factory.mktemp("toy") / "m")
    model = DecoderModel(cfg, torch.float32, "cpu")
    write_model_folder(folder, cfg, model.weight_specs(), seed=5)
    with open(os.path.join(folder, "config.json")) as f:
        assert json.load(f)["architectures"] == ["ToyMeanForCausalLM"]
    return folder


def test_toy_model_is_registered_built_and_stepped(toy):
    import airun_b200
    from airun_b200 import StepEntry
    cfg, W = P.read_model_folder(toy)
    seqs = [random_tokens(n, cfg["vocab_size"], 300 + i) for i, n in enumerate((37, 21))]
    want = [plain_toy_forward(cfg, W, s).numpy() for s in seqs]
    eng = airun_b200.Engine.from_folder(toy, dtype="float32", page_size=8, cache_tokens=256, max_batch_tokens=64,
                                        max_requests=4)
    m = eng.manager
    assert [b.kind for b in m.bindings] == ["paged", "state", "paged", "paged"]
    assert m.bindings[3].shared and m.bindings[3].index == m.bindings[2].index
    assert len(m.state) == 1 and m.state[0].spec.shape == (96,)

    def run(rid, toks, want_all=True):
        out = eng.runner.step([StepEntry(rid, toks, tuple(range(len(toks))))])
        return out.cpu().numpy()

    def start(rid):
        eng.storage.zero_state_slot(m.add_request(rid).slot)

    # whole
    start("w")
    assert_close(run("w", seqs[0]), want[0], "float32", "toy whole")
    m.free_request("w")
    # portions, then single tokens (replayed from a CUDA graph), in a slot that was used before
    start("c")
    got = [run("c", seqs[0][:13]), run("c", seqs[0][13:15]), run("c", seqs[0][15:30])]
    got += [run("c", [t]) for t in seqs[0][30:]]
    assert_close(np.concatenate(got), want[0], "float32", "toy portions and single tokens")
    # two requests side by side: a portion of one beside single tokens of the other
    start("d")
    got_d = [run("d", seqs[1][:5])]
    got_c2 = []
    m.free_request("c")
    start("e")
    got_e = []
    pe, pd = 0, 5
    while pe < len(seqs[0]) or pd < len(seqs[1]):
        entries = []
        if pe < len(seqs[0]):
            n = min(9, len(seqs[0]) - pe)
            entries.append(StepEntry("e", seqs[0][pe:pe + n], tuple(range(n))))
        if pd < len(seqs[1]):
            entries.append(StepEntry("d", [seqs[1][pd]], (0,)))
        out = eng.runner.step(entries).cpu().numpy()
        r = 0
        if pe < len(seqs[0]):
            got_e.append(out[:n]); r = n; pe += n
        if pd < len(seqs[1]):
            got_d.append(out[r:r + 1]); pd += 1
    assert_close(np.concatenate(got_e), want[0], "float32", "toy mixed, portions")
    assert_close(np.concatenate(got_d), want[1], "float32", "toy mixed, single tokens")
    eng.runner.raise_on_device_error()
    # and through the scheduler: greedy generation equals the plain model's
    res = eng.generate(seqs[1][:10], airun_b200.SamplingParams.greedy(), max_new_tokens=5)
    toks = list(seqs[1][:10])
    for _ in range(5):
        toks.append(P.plain_argmax(plain_toy_forward(cfg, W, toks)[-1].tolist()))
    assert res.token_ids == toks[10:]


def test_unknown_parts_and_architectures_are_named():
    from airun_b200.config import ConfigError, lookup_architecture
    from airun_b200.parts.base import make_part, registered_parts
    with pytest.raises(KeyError) as e:
        make_part("mixer", "no_such_mixer")
    assert "gqa_attention" in str(e.value)
    assert "swiglu" in registered_parts("feed_forward") and "rmsnorm" in registered_parts("norm")
    assert "rotary_neox" in registered_parts("position")
    with pytest.raises(ConfigError):
        lookup_architecture("NoSuchForCausalLM")


# ----------------------------------------------------------------------------- a routed feed-forward, another position encoding
def define_routed_toy():
    """A toy feed-forward with routing (every token goes to the one of three small SwiGLU experts
    its router picks, weighted by the router's probability) and a toy position encoding (rotary
    over half of each head, positions stretched by a factor), again registered from here."""
    from airun_b200.config.base import LayerSpec, register_architecture
    from airun_b200.config.qwen3 import Qwen3Config
    from airun_b200.engine.model import build_decoder
    from airun_b200.kernels import ops
    from airun_b200.parts.base import FeedForward, PositionEncoding, register_part
    from airun_b200.parts.linear import linear
    from airun_b200.weights.loader import WeightSpec

    class Top1Experts(FeedForward):
        graph_safe = False        # which experts run is decided on the host, from values read back

        def __init__(self, prefix, hidden_size, expert_size, num_experts, dtype, device):
            self.prefix, self.H, self.E, self.n, self.dtype = prefix, hidden_size, expert_size, num_experts, dtype

        def weight_specs(self):
            specs = [WeightSpec(f"{self.prefix}.router.weight", (self.n, self.H), storage="float32")]
            for e in range(self.n):
                specs += [WeightSpec(f"{self.prefix}.experts.{e}.gate_up.weight", (2 * self.E, self.H)),
                          WeightSpec(f"{self.prefix}.experts.{e}.down.weight", (self.H, self.E))]
            return specs

        def load_weights(self, tensors):
            self.router = tensors[f"{self.prefix}.router.weight"]
            self.gu = [tensors[f"{self.prefix}.experts.{e}.gate_up.weight"] for e in range(self.n)]
            self.down = [tensors[f"{self.prefix}.experts.{e}.down.weight"] for e in range(self.n)]

        def forward(self, ctx, h):
            T = h.shape[0]
            logits = h.float() @ self.router.T                          # router logits in float32
            prob = torch.softmax(logits, -1)
            top = prob.argmax(-1)
            out = ctx.ws.alloc((T, self.H), torch.float32)
            out.zero_()
            for e in range(self.n):                                     # the engine's own products, expert by expert
                rows = (top == e).nonzero().flatten()
                if rows.numel() == 0:
                    continue
                he = h[rows].contiguous()
                gu = torch.empty(rows.numel(), 2 * self.E, dtype=torch.float32, device=h.device)
                linear(ctx, he, self.gu[e], gu)
                g, u = gu[:, :self.E], gu[:, self.E:]
                act = (g / (1 + torch.exp(-g)) * u).to(self.dtype)
                y = torch.empty(rows.numel(), self.H, dtype=torch.float32, device=h.device)
                linear(ctx, act, self.down[e], y)
                out[rows] = y * prob[rows, e].unsqueeze(1)
            return out

    class StretchedHalfRotary(PositionEncoding):
        """NeoX rotation of the first half of every head only, with the position divided by a factor:
        the fused q/k kernel takes both as parameters (rotary_dim < head_dim, inv_freq as given)."""

        def __init__(self, prefix="", head_dim=0, theta=10000.0, factor=1.0, dtype=None, device=None):
            self.rotary_dim = head_dim // 2
            i = torch.arange(0, self.rotary_dim // 2, dtype=torch.float64)
            self.inv_freq = (torch.pow(torch.tensor(theta, dtype=torch.float64), -2.0 * i / self.rotary_dim)
                             / factor).to(torch.float32).to(device)

        def fused(self):
            return ops.ROPE_NEOX, self.rotary_dim, self.inv_freq

    class RoutedConfig(Qwen3Config):
        def layer_specs(self):
            specs = Qwen3Config.layer_specs(self)
            out = []
            for i, s in enumerate(specs):
                mixer_args = dict(s.mixer_args, position="toy_stretched_half_rotary",
                                  position_args=dict(head_dim=self.head_dim, theta=self.rope_theta, factor=4.0))
                if i % 2 == 1:                                          # every other layer is routed
                    out.append(LayerSpec(s.mixer, mixer_args, "toy_top1_experts",
                                         dict(hidden_size=self.hidden_size, expert_size=40, num_experts=3),
                                         s.norm, s.norm_args))
                else:
                    out.append(LayerSpec(s.mixer, mixer_args, s.feed_forward, s.ffn_args, s.norm, s.norm_args))
            return out

    register_part("feed_forward", "toy_top1_experts", Top1Experts)
    register_part("position", "toy_stretched_half_rotary", StretchedHalfRotary)
    register_architecture("ToyRoutedForCausalLM", RoutedConfig, build_decoder)
    return RoutedConfig


def plain_routed_forward(cfg: dict, W: Dict[str, torch.Tensor], tokens: List[int]) -> torch.Tensor:
    c = P.config_values(cfg)
    dt = torch.float32
    T = len(tokens)
    hd, nh, nkv = c["hd"], c["nh"], c["nkv"]
    rdim = hd // 2
    x = P.plain_embedding(W["model.embed_tokens.weight"], tokens, dt)
    for l in range(c["L"]):
        p = f"model.layers.{l}"
        h = P.plain_rmsnorm(x, W[f"{p}.input_layernorm.weight"], c["eps"])
        q = (h @ W[f"{p}.self_attn.q_proj.weight"].to(dt).T).view(T, nh, hd)
        k = (h @ W[f"{p}.self_attn.k_proj.weight"].to(dt).T).view(T, nkv, hd)
        v = (h @ W[f"{p}.self_attn.v_proj.weight"].to(dt).T).view(T, nkv, hd)
        q = P.plain_rmsnorm(q, W[f"{p}.self_attn.q_norm.weight"], c["eps"])
        k = P.plain_rmsnorm(k, W[f"{p}.self_attn.k_norm.weight"], c["eps"])
        half = rdim // 2
        inv = torch.tensor([c["theta"] ** (-2.0 * i / rdim) for i in range(half)], dtype=torch.float64).float() / 4.0
        ang = torch.arange(T, dtype=dt).unsqueeze(1) * inv.float().unsqueeze(0)
        cs, sn = ang.cos().unsqueeze(1), ang.sin().unsqueeze(1)

        def rot(t):
            a, b, rest = t[..., :half], t[..., half:rdim], t[..., rdim:]
            return torch.cat([a * cs - b * sn, a * sn + b * cs, rest], -1)

        q, k = rot(q), rot(k)
        att = torch.zeros(T, nh, hd)
        for t in range(T):
            for hh in range(nh):
                kv = hh // (nh // nkv)
                s = (k[:t + 1, kv] @ q[t, hh]) / math.sqrt(hd)
                att[t, hh] = torch.softmax(s, 0) @ v[:t + 1, kv]
        x = x + att.view(T, nh * hd) @ W[f"{p}.self_attn.o_proj.weight"].to(dt).T
        h = P.plain_rmsnorm(x, W[f"{p}.post_attention_layernorm.weight"], c["eps"])
        if l % 2 == 1:
            prob = torch.softmax(h @ W[f"{p}.mlp.router.weight"].to(dt).T, -1)
            y = torch.zeros_like(h)
            for t in range(T):
                e = int(prob[t].argmax())
                gu = W[f"{p}.mlp.experts.{e}.gate_up.weight"].to(dt) @ h[t]
                g, u = gu[:40], gu[40:]
                y[t] = (W[f"{p}.mlp.experts.{e}.down.weight"].to(dt) @ (g / (1 + torch.exp(-g)) * u)) * prob[t, e]
            x = x + y
        else:
            x = x + P.plain_swiglu_ffn(h, W[f"{p}.mlp.gate_proj.weight"].to(dt), W[f"{p}.mlp.up_proj.weight"].to(dt),
                                       W[f"{p}.mlp.down_proj.weight"].to(dt))
    h = P.plain_rmsnorm(x, W["model.norm.weight"], c["eps"])
    return h @ W["lm_head.weight"].to(dt).T


def test_routed_feed_forward_and_another_position_encoding(tmp_path):
    import math  # noqa: F401  (used by the plain model above through the module's namespace)
    import airun_b200
    from airun_b200 import StepEntry
    from airun_b200.engine.model import DecoderModel
    from airun_b200.weights import write_model_folder
    RoutedConfig = define_routed_toy()
    cfg_obj = RoutedConfig.from_dict(dict(TINY["B"]["cfg"], architectures=["ToyRoutedForCausalLM"]))
    folder = str(tmp_path / "routed")
    write_model_folder(folder, cfg_obj, DecoderModel(cfg_obj, torch.float32, "cpu").weight_specs(), seed=9)
    cfg, W = P.read_model_folder(folder)
    seqs = [random_tokens(n, cfg["vocab_size"], 400 + i) for i, n in enumerate((29, 18))]
    want = [plain_routed_forward(cfg, W, s).numpy() for s in seqs]
    eng = airun_b200.Engine.from_folder(folder, dtype="float32", page_size=8, cache_tokens=256, max_batch_tokens=64,
                                        max_requests=4)
    assert not eng.runner.use_graphs            # the toy feed-forward forbids capture: every step runs kernel by kernel
    for rid in ("a", "b"):
        eng.manager.add_request(rid)
    got_a = [eng.runner.step([StepEntry("a", seqs[0][:11], tuple(range(11)))]).cpu().numpy()]
    rows_b = []
    pa, pb = 11, 0
    while pa < len(seqs[0]) or pb < len(seqs[1]):
        entries = []
        if pa < len(seqs[0]):
            entries.append(StepEntry("a", [seqs[0][pa]], (0,)))
        nb = min(5, len(seqs[1]) - pb)
        if nb > 0:
            entries.append(StepEntry("b", seqs[1][pb:pb + nb], tuple(range(nb))))
        out = eng.runner.step(entries).cpu().numpy()
        r = 0
        if pa < len(seqs[0]):
            got_a.append(out[:1]); r = 1; pa += 1
        if nb > 0:
            rows_b.append(out[r:r + nb]); pb += nb
    eng.runner.raise_on_device_error()
    assert_close(np.concatenate(got_a), want[0], "float32", "routed toy, portion then single tokens")
    assert_close(np.concatenate(rows_b), want[1], "float32", "routed toy, portions beside single tokens")


# ----------------------------------------------------------------------------- parts only the registries reach
def define_scaled_toy():
    """A toy architecture whose embedding is scaled, whose logits are soft-capped, and whose rotary
    encoding pairs neighbouring dimensions and turns by positions that are not the cache positions."""
    from airun_b200.config.base import LayerSpec, register_architecture
    from airun_b200.config.qwen3 import Qwen3Config
    from airun_b200.engine.model import build_decoder
    from airun_b200.kernels import ops
    from airun_b200.parts.base import PositionEncoding, register_part

    class ShiftedInterleavedRotary(PositionEncoding):
        """Pairs (2i, 2i + 1); a row at cache position p is rotated by p // 2 + 3."""

        def __init__(self, prefix="", head_dim=0, theta=10000.0, dtype=None, device=None):
            self.rotary_dim = head_dim
            i = torch.arange(0, head_dim // 2, dtype=torch.float64)
            self.inv_freq = torch.pow(torch.tensor(theta, dtype=torch.float64), -2.0 * i / head_dim).float().to(device)

        def fused(self):
            return ops.ROPE_INTERLEAVED, self.rotary_dim, self.inv_freq

        def rotation_positions(self, ctx):
            pos = ctx.positions[:ctx.num_tokens]
            return (torch.div(pos.clamp(min=0), 2, rounding_mode="floor") + 3).to(torch.int32).contiguous()

    class ScaledConfig(Qwen3Config):
        def embedding(self):
            return "token_embedding", dict(scale=math.sqrt(self.hidden_size))

        def head(self):
            return "lm_head", dict(soft_cap=0.5)

        def layer_specs(self):
            out = []
            for s in Qwen3Config.layer_specs(self):
                mixer_args = dict(s.mixer_args, position="toy_shifted_interleaved_rotary",
                                  position_args=dict(head_dim=self.head_dim, theta=self.rope_theta))
                out.append(LayerSpec(s.mixer, mixer_args, s.feed_forward, s.ffn_args, s.norm, s.norm_args))
            return out

    register_part("position", "toy_shifted_interleaved_rotary", ShiftedInterleavedRotary)
    register_architecture("ToyScaledForCausalLM", ScaledConfig, build_decoder)
    return ScaledConfig


def plain_scaled_forward(cfg: dict, W: Dict[str, torch.Tensor], tokens: List[int], round_to=None) -> torch.Tensor:
    c = P.config_values(cfg)
    dt = torch.float32
    T = len(tokens)
    hd, nh, nkv = c["hd"], c["nh"], c["nkv"]
    r = (lambda t: t) if round_to is None else (lambda t: t.to(round_to).to(dt))
    x = P.plain_embedding(W["model.embed_tokens.weight"], tokens, dt) * torch.tensor(math.sqrt(c["H"]), dtype=dt)
    rpos = [p // 2 + 3 for p in range(T)]
    for l in range(c["L"]):
        p = f"model.layers.{l}"
        h = r(P.plain_rmsnorm(x, W[f"{p}.input_layernorm.weight"], c["eps"]))
        q = (h @ W[f"{p}.self_attn.q_proj.weight"].to(dt).T).view(T, nh, hd)
        k = (h @ W[f"{p}.self_attn.k_proj.weight"].to(dt).T).view(T, nkv, hd)
        v = r((h @ W[f"{p}.self_attn.v_proj.weight"].to(dt).T).view(T, nkv, hd))
        q = r(P.plain_rope_interleaved(P.plain_rmsnorm(q, W[f"{p}.self_attn.q_norm.weight"], c["eps"]), rpos, c["theta"], hd))
        k = r(P.plain_rope_interleaved(P.plain_rmsnorm(k, W[f"{p}.self_attn.k_norm.weight"], c["eps"]), rpos, c["theta"], hd))
        att = r(P.plain_attention(q, k, v, list(range(T)), hd ** -0.5, 0)).reshape(T, nh * hd)
        x = x + att @ W[f"{p}.self_attn.o_proj.weight"].to(dt).T
        h = r(P.plain_rmsnorm(x, W[f"{p}.post_attention_layernorm.weight"], c["eps"]))
        x = x + P.plain_swiglu_ffn(h, W[f"{p}.mlp.gate_proj.weight"].to(dt), W[f"{p}.mlp.up_proj.weight"].to(dt),
                                   W[f"{p}.mlp.down_proj.weight"].to(dt), round_to)
    h = r(P.plain_rmsnorm(x, W["model.norm.weight"], c["eps"]))
    logits = h @ W["lm_head.weight"].to(dt).T
    return 0.5 * torch.tanh(logits / 0.5)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_scaled_embedding_capped_head_and_rotation_positions_of_their_own(dtype, tmp_path):
    """The embedding and the head come from the part registries with their constants as parameters; the
    position encoding asks the fused prologue for the interleaved pairing and gives it rotation positions
    that are not the cache positions.  Whole, in portions and token by token (graph replay), against a
    plain implementation of the toy."""
    import airun_b200
    from airun_b200 import StepEntry
    from airun_b200.engine.model import DecoderModel
    from airun_b200.weights import write_model_folder
    from helpers import bf16_noise
    ScaledConfig = define_scaled_toy()
    cfg_obj = ScaledConfig.from_dict(dict(TINY["B"]["cfg"], architectures=["ToyScaledForCausalLM"]))
    folder = str(tmp_path / "scaled")
    write_model_folder(folder, cfg_obj, DecoderModel(cfg_obj, torch.float32, "cpu").weight_specs(), seed=10)
    cfg, W = P.read_model_folder(folder)
    seq = random_tokens(41, cfg["vocab_size"], 500)
    exact = plain_scaled_forward(cfg, W, seq).numpy()
    want = exact if dtype == "float32" else plain_scaled_forward(cfg, W, seq, torch.bfloat16).numpy()
    noise = bf16_noise(want, exact)
    assert 0.3 < float(np.abs(exact).max()) < 0.5                # the cap does bend these logits
    eng = airun_b200.Engine.from_folder(folder, dtype=dtype, page_size=8, cache_tokens=256, max_batch_tokens=64,
                                        max_requests=4)
    assert eng.model.embedding.scale == math.sqrt(cfg["hidden_size"]) and eng.model.head.soft_cap == 0.5
    eng.manager.add_request("w")
    whole = eng.runner.step([StepEntry("w", seq, tuple(range(len(seq))))]).cpu().numpy()
    eng.manager.add_request("c")
    rows = [eng.runner.step([StepEntry("c", seq[:13], tuple(range(13)))]).cpu().numpy(),
            eng.runner.step([StepEntry("c", seq[13:15], (0, 1))]).cpu().numpy()]
    for t in seq[15:]:
        rows.append(eng.runner.step([StepEntry("c", [t], (0,))]).cpu().numpy())
    eng.runner.raise_on_device_error()
    assert_close(whole, want, dtype, "scaled toy, whole", noise)
    assert_close(np.concatenate(rows), want, dtype, "scaled toy, portions then single tokens", noise)
