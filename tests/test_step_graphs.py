"""Steps replayed from CUDA graphs against the same steps run kernel by kernel and against the
plain implementation: prompt portions beside decoded tokens, padded batches, the attention work
lists made on the device."""
import numpy as np
import pytest
import torch

import plain_qwen3 as P
from helpers import TINY, assert_close, bf16_noise, make_model_folder, random_tokens

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("graph_models")
    return {n: make_model_folder(n, str(root)) for n in TINY}


def schedule(seqs):
    """Steps whose shapes come again and again: a portion of 6 or 11 tokens of one prompt beside the
    single tokens of the others; every request ends with 6 single tokens."""
    pos = [0] * len(seqs)
    steps, k = [], 0
    while any(p < len(s) for p, s in zip(pos, seqs)):
        entries = []
        filler = k % len(seqs)
        for i, s in enumerate(seqs):
            left = len(s) - pos[i]
            if left == 0:
                continue
            if left > 6 and i == filler:
                n = min(left - 6, 6 if k % 3 else 11)
            elif left <= 6 or pos[i] > 0 and k % 2:
                n = 1
            else:
                continue
            entries.append((i, pos[i], n))
            pos[i] += n
        k += 1
        if entries:
            steps.append(entries)
    return steps


@pytest.mark.parametrize("name,dtype", [(n, d) for n in ("A", "B") for d in ("float32", "bfloat16")])
def test_graph_replayed_steps_match_eager_steps_and_the_plain_model(name, dtype, folders):
    import airun_b200
    from airun_b200.engine.step import StepEntry
    cfg, W = P.read_model_folder(folders[name])
    V = cfg["vocab_size"]
    seqs = [random_tokens(n, V, 300 + i) for i, n in enumerate((61, 47, 38, 55))]
    exact = [P.plain_forward(cfg, W, s).numpy() for s in seqs]
    want = exact if dtype == "float32" else \
        [P.plain_forward(cfg, W, s, torch.float32, round_to=torch.bfloat16).numpy() for s in seqs]
    steps = schedule(seqs)
    got = {}
    for graphs in (False, True):
        eng = airun_b200.Engine.from_folder(folders[name], dtype=dtype, page_size=TINY[name]["page_size"],
                                            cache_tokens=512, max_batch_tokens=64, max_requests=4)
        eng.runner.use_graphs = graphs
        for i in range(len(seqs)):
            eng.manager.add_request(i)
        rows = {i: [] for i in range(len(seqs))}
        for entries in steps:
            out = eng.runner.step([StepEntry(i, seqs[i][p:p + n], (n - 1,)) for i, p, n in entries]).cpu().numpy()
            for r, (i, p, n) in enumerate(entries):
                rows[i].append((p + n - 1, out[r]))
        eng.runner.raise_on_device_error()
        got[graphs] = rows
        if graphs:
            mixed = [k for k in eng.runner.graphs if isinstance(k, tuple) and k[0] == "mixed"]
            assert mixed, "no step with a prompt portion was captured"
            assert eng.runner.graph_launches > 0
    for i in range(len(seqs)):
        noise = bf16_noise(want[i], exact[i]) if dtype == "bfloat16" else None
        for graphs in (False, True):
            where = [p for p, _ in got[graphs][i]]
            logits = np.stack([l for _, l in got[graphs][i]])
            assert_close(logits, want[i][where], dtype, f"{name} {dtype} graphs={graphs} request {i}",
                         None if noise is None else noise[where])
        a = np.stack([l for _, l in got[False][i]])
        b = np.stack([l for _, l in got[True][i]])
        assert_close(b, a, dtype, f"{name} {dtype} replayed vs kernel by kernel, request {i}",
                     None if noise is None else noise[where])


def test_attention_work_lists_made_on_the_device():
    """The plan kernel against the same lists made on the host."""
    from airun_b200.engine.batch import StepContext, Workspace
    from airun_b200.kernels import fast
    dev = torch.device("cuda:0")
    rng = np.random.default_rng(5)
    for trial in range(12):
        R = int(rng.integers(1, 40))
        qlens = [int(rng.choice([0, 1, 1, 2, 7, 33, 64, 65, 300])) for _ in range(R)]
        if trial == 11:
            qlens = [1500] * 3 + [1] * 5          # more tiles than the kernel sorts: any order, same set
            R = len(qlens)
        ctxlens = [q + int(rng.integers(0, 500)) for q in qlens]
        cu = np.concatenate([[0], np.cumsum(qlens)]).astype(np.int32)
        T = int(cu[-1]) + 5
        per = int(rng.choice([1, 4, 16, 64, 128])) if trial != 11 else 1
        ctx = StepContext(num_tokens=T, num_reqs=R + 3, token_ids=None, positions=None, req_of_token=None,
                          cu_tokens=torch.tensor(np.concatenate([cu, [cu[-1]] * 3]).astype(np.int32), device=dev),
                          context_lens=torch.tensor(ctxlens + [0] * 3, dtype=torch.int32, device=dev),
                          state_slots=None, err=torch.zeros(1, dtype=torch.int32, device=dev))
        max_tiles = T // per + R + 4
        tiles = torch.full((max_tiles, 4), -7, dtype=torch.int32, device=dev)
        rows = torch.full((R + 3,), -7, dtype=torch.int32, device=dev)
        counts = torch.zeros(4, dtype=torch.int32, device=dev)
        fast.attn_plan(ctx, per, tiles, rows, counts)
        want_rows, want_tiles = [], []
        for r, (n, c) in enumerate(zip(qlens, ctxlens)):
            if n == 1:
                want_rows.append(int(cu[r]))
            elif n > 1:
                for s in range(0, n, per):
                    k = min(per, n - s)
                    want_tiles.append((r, int(cu[r]) + s, k, c - n + s + k))
        nt, nr = counts[:2].tolist()
        assert int(ctx.err.item()) == 0
        assert nr == len(want_rows) and rows[:nr].tolist() == want_rows
        assert nt == len(want_tiles)
        got_tiles = [tuple(t) for t in tiles[:nt].tolist()]
        if nt <= 1024:
            assert got_tiles == sorted(want_tiles, key=lambda x: -x[3])      # stable, the most keys first
        else:
            assert sorted(got_tiles) == sorted(want_tiles)
    # lists that are too short: nothing is run and the error flag says so
    ctx.err.zero_()
    fast.attn_plan(ctx, per, tiles[:2], rows, counts)
    assert counts[:2].tolist() == [0, 0] and int(ctx.err.item()) != 0
