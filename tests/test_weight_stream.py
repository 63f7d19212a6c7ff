"""The host-side bookkeeping of the weight prefetch: which bytes a kernel is told to ask into L2."""
import random

import torch

from airun_b200.engine.batch import WeightStream


def make(sizes, max_ahead):
    ts = [torch.empty(n, dtype=torch.uint8) for n in sizes]
    return ts, WeightStream(ts, max_ahead=max_ahead)


def test_ranges_follow_the_order_of_the_pass_and_stay_within_the_limit():
    ts, ws = make([1000 * 256, 300 * 256 + 100, 2000 * 256], 500 * 256)
    p, n = ws.claim(100 * 256)                           # before any product: the first matrix
    assert (p, n) == (ts[0].data_ptr(), 100 * 256)
    ws.consume(ts[0])                                    # the matrix being read is never asked for again
    p, n = ws.claim(400 * 256)
    assert (p, n) == (ts[1].data_ptr(), 300 * 256)       # inside one matrix, whole 256-byte units
    p, n = ws.claim(400 * 256)                           # the ragged 100 bytes are skipped; the limit cuts the range
    assert p == ts[2].data_ptr() and n == (500 * 256 - 300 * 256 - 100) // 256 * 256
    assert ws.claim(400 * 256) == (0, 0)                 # nothing more until a product moves on
    ws.consume(ts[1])
    p2, n2 = ws.claim(10 ** 9)
    assert p2 == p + n and n2 > 0
    ws.consume(ts[2])
    p3, n3 = ws.claim(64 * 256)                          # after the last matrix comes the first: the next pass's
    assert (p3, n3) == (ts[0].data_ptr(), 64 * 256)
    ws.reset()
    p4, n4 = ws.claim(64 * 256)                          # the new pass goes on where the old one's requests ended
    assert (p4, n4) == (ts[0].data_ptr() + 64 * 256, 64 * 256)


def test_random_claims_never_overlap_never_run_behind_and_cover_each_matrix_once():
    rnd = random.Random(3)
    sizes = [rnd.randrange(1, 400) * 256 + rnd.choice([0, 16, 250]) for _ in range(12)]
    ts, ws = make(sizes, 64 * 1024)
    base = {t.data_ptr(): i for i, t in enumerate(ts)}
    for _pass in range(3):
        ws.reset()
        seen = {i: [] for i in range(len(ts))}
        for i, t in enumerate(ts):
            for _ in range(rnd.randrange(0, 4)):
                p, n = ws.claim(rnd.randrange(1, 200) * 256)
                if n:
                    j = max((k for k in base if k <= p), key=lambda k: k)
                    j = base[j]
                    off = p - ts[j].data_ptr()
                    assert off % 256 == 0 and n % 256 == 0 and off + n <= sizes[j]
                    assert j != ws_current(ws, ts)        # never the matrix being read
                    seen[j].append((off, n))
            ws.consume(t)
            assert ws.front - ws.cur_end <= ws.max_ahead
        for j, ranges in seen.items():
            ranges.sort()
            for (a, n), (b, _) in zip(ranges, ranges[1:]):
                assert a + n <= b, "a range was handed out twice"


def ws_current(ws, ts):
    if ws.cur_start < 0:
        return -1
    return ws.starts.index(ws.cur_start % ws.total) if (ws.cur_start % ws.total) in ws.starts else -1


def test_a_matrix_used_twice_in_a_pass_and_unknown_matrices():
    ts, ws = make([256 * 10, 256 * 20, 256 * 30], 1 << 20)
    twice = WeightStream([ts[0], ts[1], ts[0], ts[2]], max_ahead=1 << 20)
    twice.consume(ts[0])
    assert twice.cur_start == 0
    twice.consume(ts[1])
    twice.consume(ts[0])                                 # its second place in the order
    assert twice.cur_start == 256 * 30
    twice.consume(torch.empty(16, dtype=torch.uint8))    # not part of the stream: ignored
    assert twice.cur_start == 256 * 30
