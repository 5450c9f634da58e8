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


def test_buckets_leave_room_for_the_dummy_requests_and_hold_every_list():
    """Any step fits the bucket chosen for it: at least one dummy single token and a dummy portion of more than
    SHORT_PORTION tokens behind the real requests, and the fixed list lengths hold the real work plus the dummies'."""
    from logssms_b200.engine.plan import bucket_for
    from logssms_b200.parts.context import Padding, chunk_lists, request_lists, short_token_list, tile_list
    rng = random.Random(11)
    seen = set()
    for _ in range(300):
        B = rng.randint(1, 40)
        lens = [rng.choice([1, 1, 1, 2, SHORT_PORTION, SHORT_PORTION + 1, 40, 64, 129, 300, 512, 700]) for _ in range(B)]
        starts = [rng.choice([0, 3, 64, 1000]) for _ in range(B)]
        wanted = rng.randint(0, B)
        bk = bucket_for(lens, wanted)
        assert bk is not None and bk.requests >= B + 2 and bk.requests >= wanted
        singles = bk.requests - B - 1
        portion = bk.tokens - sum(lens) - singles
        assert singles >= 1 and portion > SHORT_PORTION
        assert bk.tokens % 64 == 0 and bk.requests % 4 == 0
        seen.add(bk)
        # the step as the planner pads it
        plens = np.asarray(lens + [1] * singles + [portion])
        pstarts = np.asarray(starts + [0] * (singles + 1))
        pad = Padding(B, bk.long_cap, bk.short_cap)
        dummy_single_request, dummy_single_token = B, sum(lens)
        for tile in (64, 128):
            cap = -(-bk.tokens // tile) + pad.long_cap
            tiles = tile_list(plens, pstarts, tile, cap)
            real = sorted((b, t0) for b, m in enumerate(plens) if m > SHORT_PORTION for t0 in range(0, int(m), tile))
            assert tiles.shape == (cap, 2) and sorted(map(tuple, tiles[:len(real)].tolist())) == real
            assert all(tuple(t) == (-1, 0) for t in tiles[len(real):].tolist())                    # entries without work
            chunks, per_request = chunk_lists(plens, tile, cap, pad.long_cap)
            assert chunks.shape == (cap, 2) and per_request.shape == (pad.long_cap, 3)
            n_long = sum(1 for m in plens if m > SHORT_PORTION)
            assert all(tuple(r) == (-1, 0, 0) for r in per_request[n_long:].tolist())
            assert per_request[n_long - 1][0] == bk.requests - 1 and all(c[0] == -1 for c in chunks[len(real):].tolist())
        short = short_token_list(plens, pad.short_cap, dummy_single_token)
        n_short = sum(int(m) for m in plens if m <= SHORT_PORTION)
        assert short.shape == (pad.short_cap,) and n_short <= pad.short_cap and set(short[n_short:].tolist()) <= {dummy_single_token}
        long_r, short_r = request_lists(plens, pad.long_cap, min(pad.short_cap, bk.requests), dummy_single_request)
        assert long_r.shape == (pad.long_cap,) and long_r[-1] == bk.requests - 1
        assert set(short_r[sum(1 for m in plens if m <= SHORT_PORTION):].tolist()) <= {dummy_single_request}
    # the shapes of chunked serving (some decoding requests beside one prompt portion under a budget of 512 tokens):
    # a thousand different shapes, a few dozen buckets (requests x tokens)
    shapes = {(d, rng.randint(SHORT_PORTION + 1, 512 - d)) for d in (rng.randint(0, 32) for _ in range(1500))}
    buckets = {bucket_for([1] * d + [n], d + 1) for d, n in shapes}
    assert len(shapes) > 1000 and len(buckets) <= 60, (len(shapes), len(buckets))
    assert bucket_for([5, 5], 3) is not None and bucket_for([5], 9) is None      # more wanted places than the bucket has requests
