"""A toy mixer with state of its own, a toy architecture that uses it, and an execution
order that names a layer twice and lets an entry read another entry's cache: all
registered from here, built and stepped without a change to the framework's files."""
from __future__ import annotations

import json
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
