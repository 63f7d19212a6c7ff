"""The reference's own CUDA kernels, compiled unmodified, behind their C entry points.

The reference project is a Rust workspace whose runtime cannot be built without cargo.
Its kernels, however, are plain CUDA behind ``extern "C"`` launchers with fixed-width
types (crates/airun-cuda/kernels/ops.cu:2222-2578, matmul.cu:2277-2531, airun.cuh:1-4).
This module

* builds ``ops.cu`` and ``matmul.cu`` (copied, not edited) into one shared library with
  the reference's own compiler flags (crates/airun-cuda/build.rs:73-84), for sm_100;
* binds the entry points a dense Qwen3 decoder uses with ctypes;
* restates, in :class:`ReferenceDecoder`, the ORDER in which the reference's runtime calls
  them: whole-prompt portions (crates/airun-core/src/runtime.rs:3507-3602, :3833-4120 the
  non-mixed branch, :2601-2655) and one decode step for several conversations
  (runtime.rs:3050-3147 and the mixed branch of run_attention).  The Rust code around the
  calls (memory planning, graphs, scheduling) is not restated.

Nothing of the product package is imported here; tensors are torch tensors only as device
memory.  Used by the tests that pin the plain implementation on the reference's kernels
and by ``bench.py --impl reference``.
"""
from __future__ import annotations

import ctypes
import os
import shutil
import subprocess
import sys
import time
from ctypes import c_float, c_int32, c_int64, c_uint64, c_void_p
from typing import Dict, List, Optional, Sequence

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")
LIB_PATH = os.path.join(REF_DIR, "libairun_ref_kernels.so")
SOURCES = ("ops.cu", "matmul.cu")

TYPE_F32, TYPE_F16, TYPE_BF16 = 0, 1, 30          # dequant.cuh:693-710
KV_F16 = 0                                         # ops.cu:288


class RopeParams(ctypes.Structure):
    """airun_rope_params (airun.cuh:120-143), passed by value."""
    _fields_ = [("base", c_float), ("freq_scale", c_float), ("ext_factor", c_float), ("mscale", c_float),
                ("corr_lo", c_float), ("corr_hi", c_float), ("shift", c_void_p), ("mpos", c_void_p),
                ("n_tok", c_int32), ("sections", c_int32 * 3)]


def plain_rope(base: float) -> RopeParams:
    """RopeParams::plain(base, 1.0): no scaling, positions are the cache slots."""
    return RopeParams(float(base), 1.0, 0.0, 1.0, 0.0, 0.0, None, None, 0, (c_int32 * 3)(0, 0, 0))


def build(reference_dir: str, verbose: bool = True) -> str:
    """Copies the reference's kernels folder beside this file and compiles the two sources."""
    src = os.path.join(reference_dir, "crates", "airun-cuda", "kernels")
    if not os.path.isdir(src):
        raise FileNotFoundError(f"{src} is not the reference's kernels folder")
    dst = os.path.join(REF_DIR, "kernels")
    os.makedirs(REF_DIR, exist_ok=True)
    if os.path.isdir(dst):
        shutil.rmtree(dst)
    shutil.copytree(src, dst)
    flags = ["-O3", "--use_fast_math", "-std=c++17", "--extended-lambda", "-allow-unsupported-compiler",
             "-diag-suppress=177", "-Xcompiler", "-fPIC", "-I", dst, "-gencode=arch=compute_100,code=sm_100"]
    procs = []
    for s in SOURCES:
        obj = os.path.join(REF_DIR, s.replace(".cu", ".o"))
        cmd = ["nvcc", *flags, "-c", os.path.join(dst, s), "-o", obj]
        if verbose:
            print("building", s, "(matmul.cu takes several minutes)", file=sys.stderr, flush=True)
        procs.append((s, obj, subprocess.Popen(cmd)))
    objs = []
    for s, obj, p in procs:
        t0 = time.time()
        while p.poll() is None:
            time.sleep(5)
            if verbose and time.time() - t0 > 60:
                print("  still compiling", s, file=sys.stderr, flush=True)
                t0 = time.time()
        if p.returncode != 0:
            raise RuntimeError(f"nvcc failed on {s}")
        objs.append(obj)
    subprocess.check_call(["nvcc", "-shared", "-o", LIB_PATH, *objs, "-lcudart"])
    return LIB_PATH


_LIB = None


def available() -> bool:
    return os.path.exists(LIB_PATH)


def load():
    global _LIB
    if _LIB is None:
        if not available():
            raise FileNotFoundError(
                f"{LIB_PATH} is missing: run `python baseline/reference_kernels.py --build <reference checkout>`")
        lib = ctypes.CDLL(LIB_PATH)
        P, I, F, L = c_void_p, c_int32, c_float, c_int64
        sig = {
            "airun_rmsnorm": [P, P, P, I, I, F, P],
            "airun_add_rmsnorm": [P, P, P, P, I, I, F, P],
            "airun_add": [P, P, L, P],
            "airun_swiglu": [P, P, L, P],
            "airun_argmax": [P, I, P, P, P, P],
            "airun_rope": [P, P, I, I, I, I, RopeParams, I, P],
            "airun_embed": [I, P, P, P, I, I, c_uint64, I, P],
            "airun_kv_store": [P, P, P, P, P, I, I, I, I, I, P],
            "airun_qk_norm_rope_store": [P, P, P, P, P, P, P, P, I, I, I, I, I, F, I, RopeParams, I, I, I, P],
            "airun_attention": [P, P, P, P, P, I, I, I, I, I, F, I, I, P, I, I, P],
            "airun_attention_split": [P, P, P, P, P, P, I, I, I, I, F, I, I, I, P, P],
            "airun_attention_split_rows": [P, P, P, P, P, I, I, I, I, F, I, I, I, I, P],
            "airun_matvec": [I, P, P, P, I, I, I, c_uint64, P],
            "airun_matvec_glu": [I, P, P, P, P, I, I, c_uint64, P],
            "airun_matvec3": [I, P, P, P, P, P, P, P, I, I, I, I, c_uint64, P],
        }
        for name, args in sig.items():
            f = getattr(lib, name)
            f.argtypes = args
            f.restype = c_int32
        _LIB = lib
    return _LIB


def _ok(status: int, what: str) -> None:
    if status != 0:
        raise RuntimeError(f"reference kernel {what} returned status {status}")


def _stream():
    import torch
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _p(t):
    return None if t is None else c_void_p(t.data_ptr())


def attention_splits(ctx: int) -> int:
    """crates/airun-cuda/src/ops.rs:1207."""
    return min(256, max(16, -(-ctx // 64)))


# ----------------------------------------------------------------------------- thin calls
def rmsnorm(out, x, w, n, rows, eps):
    _ok(load().airun_rmsnorm(_p(out), _p(x), _p(w), n, rows, eps, _stream()), "rmsnorm")


def add_rmsnorm(out, x, b, w, n, rows, eps):
    _ok(load().airun_add_rmsnorm(_p(out), _p(x), _p(b), _p(w), n, rows, eps, _stream()), "add_rmsnorm")


def swiglu(gate, up, n):
    _ok(load().airun_swiglu(_p(gate), _p(up), n, _stream()), "swiglu")


def argmax(x, n, out, scratch):
    _ok(load().airun_argmax(_p(x), n, _p(out), _p(scratch), None, _stream()), "argmax")


def rope(x, positions, n_tokens, n_heads, head_dim, rope_dim, base, interleaved=False):
    _ok(load().airun_rope(_p(x), _p(positions), n_tokens, n_heads, head_dim, rope_dim, plain_rope(base),
                          1 if interleaved else 0, _stream()), "rope")


def embed(out, table, tokens, n_tokens, n_embd, vocab, type_id=TYPE_BF16):
    row_bytes = n_embd * (4 if type_id == TYPE_F32 else 2)
    _ok(load().airun_embed(type_id, _p(out), _p(table), _p(tokens), n_tokens, n_embd, row_bytes, vocab, _stream()),
        "embed")


def qk_norm_rope_store(q, k, v, q_norm, k_norm, k_cache, v_cache, positions, n_tokens, nh, nkv, hd, max_seq, eps,
                       rope_dim, base, interleaved=False, rope_on=True):
    _ok(load().airun_qk_norm_rope_store(_p(q), _p(k), _p(v), _p(q_norm), _p(k_norm), _p(k_cache), _p(v_cache),
                                        _p(positions), n_tokens, nh, nkv, hd, max_seq, eps, rope_dim,
                                        plain_rope(base), 1 if interleaved else 0, 1 if rope_on else 0, KV_F16,
                                        _stream()), "qk_norm_rope_store")


def attention(out, q, k_cache, v_cache, positions, n_tokens, nh, nkv, hd, max_seq, scale, window, keys):
    _ok(load().airun_attention(_p(out), _p(q), _p(k_cache), _p(v_cache), _p(positions), n_tokens, nh, nkv, hd,
                               max_seq, scale, window, KV_F16, None, 0, keys, _stream()), "attention")


def attention_split(out, partial, q, k_cache, v_cache, positions, nh, nkv, hd, max_seq, scale, window, splits):
    _ok(load().airun_attention_split(_p(out), _p(partial), _p(q), _p(k_cache), _p(v_cache), _p(positions), nh, nkv,
                                     hd, max_seq, scale, window, splits, KV_F16, None, _stream()), "attention_split")


def attention_split_rows(out, partial, q, kv_rows, positions, nh, nkv, hd, max_seq, scale, window, splits, rows):
    _ok(load().airun_attention_split_rows(_p(out), _p(partial), _p(q), _p(kv_rows), _p(positions), nh, nkv, hd,
                                          max_seq, scale, window, splits, KV_F16, rows, _stream()),
        "attention_split_rows")


def matvec(w, x, y, k, n_rows, n_tokens, type_id=TYPE_BF16, x_off=0, y_off=0):
    """y[t] = W x[t]; ``x_off`` / ``y_off`` are float offsets into x and y."""
    row_bytes = k * (4 if type_id == TYPE_F32 else 2)
    _ok(load().airun_matvec(type_id, _p(w), c_void_p(x.data_ptr() + 4 * x_off), c_void_p(y.data_ptr() + 4 * y_off),
                            k, n_rows, n_tokens, row_bytes, _stream()), "matvec")


def matvec_glu(wg, wu, x, y, k, n_rows, type_id=TYPE_BF16):
    row_bytes = k * (4 if type_id == TYPE_F32 else 2)
    _ok(load().airun_matvec_glu(type_id, _p(wg), _p(wu), _p(x), _p(y), k, n_rows, row_bytes, _stream()), "matvec_glu")


def matvec3(w0, w1, w2, x, y0, y1, y2, k, n0, n1, n2, type_id=TYPE_BF16):
    row_bytes = k * (4 if type_id == TYPE_F32 else 2)
    _ok(load().airun_matvec3(type_id, _p(w0), _p(w1), _p(w2), _p(x), _p(y0), _p(y1), _p(y2), k, n0, n1, n2, row_bytes,
                             _stream()), "matvec3")


# ----------------------------------------------------------------------------- the order of calls
class ReferenceDecoder:
    """A dense Qwen3 decoder whose every computation is one of the reference's kernels.

    ``weights`` maps the HF tensor names to device tensors: matrices bfloat16 (or float32 with
    ``weight_type=TYPE_F32``), norm vectors float32.  Activations are float32 and each slot owns a
    contiguous float16 cache ``[nkv][ctx][hd]`` per layer for K and for V, as in the reference
    (runtime.rs:1033-1037).  ``max_batch`` bounds the tokens of one pass."""

    def __init__(self, cfg: dict, weights: Dict[str, "torch.Tensor"], ctx: int, slots: int = 1, max_batch: int = 512,
                 weight_type: int = TYPE_BF16, device: str = "cuda:0", logit_rows: int = 0):
        import torch
        self.torch = torch
        self.L, self.H = cfg["num_hidden_layers"], cfg["hidden_size"]
        self.nh = cfg["num_attention_heads"]
        self.nkv = cfg.get("num_key_value_heads") or self.nh
        self.hd = cfg.get("head_dim") or self.H // self.nh
        self.I, self.V = cfg["intermediate_size"], cfg["vocab_size"]
        self.eps = float(cfg.get("rms_norm_eps") or 1e-6)
        self.theta = float(cfg.get("rope_theta") or 10000.0)
        self.tied = bool(cfg.get("tie_word_embeddings", False))
        self.W, self.ctx, self.wt, self.dev = weights, ctx, weight_type, torch.device(device)
        self.max_batch = max_batch
        f32 = dict(dtype=torch.float32, device=self.dev)
        n = max_batch
        self.x = torch.zeros(n, self.H, **f32)
        self.xb = torch.zeros(n, self.H, **f32)
        self.xb2 = torch.zeros(n, self.H, **f32)
        self.q = torch.zeros(n, self.nh * self.hd, **f32)
        self.k = torch.zeros(n, self.nkv * self.hd, **f32)
        self.v = torch.zeros(n, self.nkv * self.hd, **f32)
        self.attn = torch.zeros(n, self.nh * self.hd, **f32)
        self.gate = torch.zeros(n, self.I, **f32)
        self.up = torch.zeros(n, self.I, **f32)
        self.tokens = torch.zeros(n, dtype=torch.int32, device=self.dev)
        self.positions = torch.zeros(n, dtype=torch.int32, device=self.dev)
        self.splits = attention_splits(ctx)
        self.partial = torch.zeros(n * self.nh * self.splits * (self.hd + 2), **f32)
        # [slot][layer] K and V caches
        self.kc = torch.zeros(slots, self.L, self.nkv, ctx, self.hd, dtype=torch.float16, device=self.dev)
        self.vc = torch.zeros(slots, self.L, self.nkv, ctx, self.hd, dtype=torch.float16, device=self.dev)
        self.n_past = [0] * slots
        self.rows_tab = torch.zeros(self.L, 2 * max(slots, 1), dtype=torch.int64, device=self.dev)
        self.logits = torch.zeros(logit_rows or n, self.V, **f32)
        self.argmax_scratch = torch.zeros(4096, dtype=torch.int32, device=self.dev)
        self.argmax_out = torch.zeros(n, dtype=torch.int32, device=self.dev)

    # -- helpers
    def _w(self, name):
        return self.W[name]

    def _mv(self, name, x, y, n):
        w = self._w(name)
        matvec(w, x, y, w.shape[1], w.shape[0], n, self.wt)

    def _head_name(self):
        return "model.embed_tokens.weight" if self.tied else "lm_head.weight"

    def _ffn(self, p, n):
        """dense_ffn (runtime.rs:688-747) for float weights: one token takes the fused gate/up/SwiGLU
        matvec, several take gate, up, swiglu."""
        wg, wu = self._w(f"{p}.mlp.gate_proj.weight"), self._w(f"{p}.mlp.up_proj.weight")
        if n == 1:
            matvec_glu(wg, wu, self.xb, self.gate, wg.shape[1], wg.shape[0], self.wt)
        else:
            self._mv(f"{p}.mlp.gate_proj.weight", self.xb, self.gate, n)
            self._mv(f"{p}.mlp.up_proj.weight", self.xb, self.up, n)
            swiglu(self.gate, self.up, n * self.I)
        self._mv(f"{p}.mlp.down_proj.weight", self.gate, self.xb2, n)

    def _next_norm(self, l):
        return self._w(f"model.layers.{l + 1}.input_layernorm.weight") if l + 1 < self.L else self._w("model.norm.weight")

    def _qkv(self, p, n):
        a = f"{p}.self_attn"
        wq, wk, wv = (self._w(f"{a}.{x}_proj.weight") for x in "qkv")
        if n == 1 and wq.shape[0] % 4 == 0 and wk.shape[0] % 4 == 0:       # matvec3 wants whole warps of 4 rows
            matvec3(wq, wk, wv, self.xb, self.q, self.k, self.v, wq.shape[1], wq.shape[0], wk.shape[0], wv.shape[0], self.wt)
        else:
            self._mv(f"{a}.q_proj.weight", self.xb, self.q, n)
            self._mv(f"{a}.k_proj.weight", self.xb, self.k, n)
            self._mv(f"{a}.v_proj.weight", self.xb, self.v, n)

    def _embed_and_first_norm(self, n):
        embed(self.x, self._w("model.embed_tokens.weight"), self.tokens, n, self.H, self.V, self.wt)
        rmsnorm(self.xb, self.x, self._w("model.layers.0.input_layernorm.weight"), self.H, n, self.eps)

    # -- one sequence, n tokens at positions n_past.. (runtime.rs:2424 queue_forward, non-mixed branch)
    def forward(self, slot: int, token_ids: Sequence[int], all_logits: bool = False):
        """Feeds ``token_ids`` to ``slot`` in passes of at most ``max_batch`` tokens; returns the last
        token's logits [V], or with ``all_logits`` every token's [n, V] (forward_all, runtime.rs:1642-1681)."""
        torch = self.torch
        outs = []
        ids = list(token_ids)
        for s in range(0, len(ids), self.max_batch):
            part = ids[s:s + self.max_batch]
            n = len(part)
            past = self.n_past[slot]
            self.tokens[:n].copy_(torch.tensor(part, dtype=torch.int32))
            self.positions[:n].copy_(torch.arange(past, past + n, dtype=torch.int32))
            self._pass_single(slot, n, past)
            self.n_past[slot] = past + n
            if all_logits:
                for r0 in range(0, n, 8):
                    m = min(8, n - r0)
                    w = self._w(self._head_name())
                    matvec(w, self.xb, self.logits, self.H, self.V, m, self.wt, x_off=r0 * self.H, y_off=r0 * self.V)
                outs.append(self.logits[:n].clone())
            elif s + n == len(ids):
                w = self._w(self._head_name())
                matvec(w, self.xb, self.logits, self.H, self.V, 1, self.wt, x_off=(n - 1) * self.H)
                outs.append(self.logits[:1].clone())
        return torch.cat(outs) if all_logits else outs[-1][0]

    def _pass_single(self, slot, n, past):
        self._embed_and_first_norm(n)
        scale = self.hd ** -0.5
        for l in range(self.L):
            p = f"model.layers.{l}"
            a = f"{p}.self_attn"
            self._qkv(p, n)
            kc, vc = self.kc[slot, l], self.vc[slot, l]
            qk_norm_rope_store(self.q, self.k, self.v, self._w(f"{a}.q_norm.weight"), self._w(f"{a}.k_norm.weight"),
                               kc, vc, self.positions, n, self.nh, self.nkv, self.hd, self.ctx, self.eps, self.hd,
                               self.theta)
            if n == 1:
                attention_split(self.attn, self.partial, self.q, kc, vc, self.positions, self.nh, self.nkv, self.hd,
                                self.ctx, scale, 0, self.splits)
            else:
                attention(self.attn, self.q, kc, vc, self.positions, n, self.nh, self.nkv, self.hd, self.ctx, scale, 0,
                          past + n)
            self._mv(f"{a}.o_proj.weight", self.attn, self.xb2, n)
            add_rmsnorm(self.xb, self.x, self.xb2, self._w(f"{p}.post_attention_layernorm.weight"), self.H, n, self.eps)
            self._ffn(p, n)
            add_rmsnorm(self.xb, self.x, self.xb2, self._next_norm(l), self.H, n, self.eps)

    # -- one token for each of several slots (runtime.rs:3050-3147 decode_rows)
    def prepare_rows(self, slots: Sequence[int]) -> None:
        """fill_rows_tab (runtime.rs:3152-3173): per layer the K pointers of the rows, then the V pointers."""
        torch = self.torch
        n = len(slots)
        host = torch.zeros(self.L, 2 * n, dtype=torch.int64)
        for l in range(self.L):
            for b, s in enumerate(slots):
                host[l, b] = self.kc[s, l].data_ptr()
                host[l, n + b] = self.vc[s, l].data_ptr()
        self.rows_tab = host.to(self.dev)
        self._row_slots = list(slots)

    def set_row_inputs(self, token_ids: Sequence[int]) -> None:
        torch = self.torch
        n = len(token_ids)
        self.tokens[:n].copy_(torch.tensor(list(token_ids), dtype=torch.int32))
        self.positions[:n].copy_(torch.tensor([self.n_past[s] for s in self._row_slots], dtype=torch.int32))

    def launch_rows(self, head: bool = True) -> None:
        """The kernels of one decode step for the prepared rows, on the current stream (capturable)."""
        slots = self._row_slots
        n = len(slots)
        if n == 1:
            self._pass_single(slots[0], 1, None)
            if head:
                w = self._w(self._head_name())
                matvec(w, self.xb, self.logits, self.H, self.V, 1, self.wt)
            return
        self._embed_and_first_norm(n)
        scale = self.hd ** -0.5
        qw, kw = self.nh * self.hd, self.nkv * self.hd
        batched = self.nh // self.nkv <= 8 and self.hd in (64, 128, 256)       # attention_split_rows_ok, ops.rs:1242
        for l in range(self.L):
            p = f"model.layers.{l}"
            a = f"{p}.self_attn"
            self._qkv(p, n)
            for b, s in enumerate(slots):
                pos = self.positions[b:b + 1]
                qk_norm_rope_store(self.q[b:b + 1], self.k[b:b + 1], self.v[b:b + 1], self._w(f"{a}.q_norm.weight"),
                                   self._w(f"{a}.k_norm.weight"), self.kc[s, l], self.vc[s, l], pos, 1, self.nh,
                                   self.nkv, self.hd, self.ctx, self.eps, self.hd, self.theta)
                if not batched:
                    attention_split(self.attn[b:b + 1], self.partial, self.q[b:b + 1], self.kc[s, l], self.vc[s, l], pos,
                                    self.nh, self.nkv, self.hd, self.ctx, scale, 0, self.splits)
            if batched:
                attention_split_rows(self.attn, self.partial, self.q, self.rows_tab[l], self.positions, self.nh,
                                     self.nkv, self.hd, self.ctx, scale, 0, self.splits, n)
            self._mv(f"{a}.o_proj.weight", self.attn, self.xb2, n)
            add_rmsnorm(self.xb, self.x, self.xb2, self._w(f"{p}.post_attention_layernorm.weight"), self.H, n, self.eps)
            self._ffn(p, n)
            add_rmsnorm(self.xb, self.x, self.xb2, self._next_norm(l), self.H, n, self.eps)
        if head:
            w = self._w(self._head_name())
            for r0 in range(0, n, 8):
                m = min(8, n - r0)
                matvec(w, self.xb, self.logits, self.H, self.V, m, self.wt, x_off=r0 * self.H, y_off=r0 * self.V)

    def decode_rows(self, rows: Sequence[tuple]):
        """rows: (slot, token).  Returns logits [n, V] on the device."""
        self.prepare_rows([s for s, _ in rows])
        self.set_row_inputs([t for _, t in rows])
        self.launch_rows()
        for s, _ in rows:
            self.n_past[s] += 1
        return self.logits[:len(rows)]


if __name__ == "__main__":
    import argparse
    ap = argparse.ArgumentParser(description="build the reference's CUDA kernels for sm_100 beside this file")
    ap.add_argument("--build", metavar="REFERENCE_CHECKOUT", required=True)
    a = ap.parse_args()
    print(build(a.build))
