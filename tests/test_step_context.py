"""The work lists that the kernels for long portions get from the step context (host logic, on the CPU)."""
import random

import numpy as np
import torch

from logssms_b200.parts.context import SHORT_PORTION, StepContext


def context(lens, starts):
    T, B = int(sum(lens)), len(lens)
    z = lambda n: torch.zeros(n, dtype=torch.int32)
    return StepContext(num_tokens=T, num_requests=B, max_len=max(lens), token_ids=z(T), positions=z(T), token_req=z(T),
                       cu_seqlens=z(B + 1), start_pos=z(B), slots=z(B), block_tables=[], slot_mappings=[], logit_rows=z(0),
                       cache=None, host_lens=np.asarray(lens), host_starts=np.asarray(starts))


def test_tiles_cover_every_long_portion_once_heaviest_first():
    rng = random.Random(5)
    for _ in range(50):
        B = rng.randint(1, 6)
        lens = [rng.choice([1, 2, SHORT_PORTION, SHORT_PORTION + 1, 64, 65, 127, 128, 300, 700]) for _ in range(B)]
        starts = [rng.choice([0, 3, 64, 1000]) for _ in range(B)]
        ctx = context(lens, starts)
        for tile in (64, 128):
            tiles, n = ctx.long_portion_tiles(tile)
            assert tiles.shape == (n, 2) and tiles.dtype == torch.int32
            got = sorted(map(tuple, tiles.tolist()))
            want = sorted((b, t0) for b, m in enumerate(lens) if m > SHORT_PORTION for t0 in range(0, m, tile))
            assert got == want
            seen = [starts[b] + min(t0 + tile, lens[b]) for b, t0 in tiles.tolist()]       # keys the tile's last row sees
            assert seen == sorted(seen, reverse=True)
            assert ctx.long_portion_tiles(tile)[0] is tiles                               # built once per step


def test_chunks_and_request_lists():
    lens, starts = [300, 1, 128, 5, 129], [0, 77, 64, 0, 9]
    ctx = context(lens, starts)
    assert ctx.has_long_portions
    chunks, n, per_request, m = ctx.long_portion_chunks(128)
    assert n == 3 + 1 + 2 and m == 3
    assert chunks.tolist() == [[0, 0], [0, 128], [0, 256], [2, 0], [4, 0], [4, 128]]
    assert per_request.tolist() == [[0, 0, 3], [2, 3, 1], [4, 4, 2]]
    long_r, nl, short_r, ns = ctx.requests_by_portion()
    assert (long_r.tolist(), nl, short_r.tolist(), ns) == ([0, 2, 4], 3, [1, 3], 2)
    tokens, nt = ctx.short_portion_tokens()
    assert nt == 6 and tokens.tolist() == [300] + list(range(429, 434))       # request 1's token, request 3's five


def test_a_step_of_short_portions_has_no_long_ones():
    ctx = context([1, 1, SHORT_PORTION], [10, 20, 30])
    assert not ctx.has_long_portions
    tokens, n = ctx.short_portion_tokens()
    assert n == 2 + SHORT_PORTION and tokens.tolist() == list(range(n))
