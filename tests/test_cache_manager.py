"""The cache manager on the CPU: no page lost, held twice or freed twice, under random orders."""
import random

import pytest
import torch

from logssms_b200.cache import CacheManager, CacheNeeds, FreeList, KVNeed, OutOfPages, PagedNeed, PagedTensor, StateNeed

FULL = KVNeed(2, 16)
WINDOW = KVNeed(2, 16, window=40)


def manager(needs, pages=12, page=16, max_requests=4, max_seq=256, **kw):
    return CacheManager(needs, page_size=page, num_pages=pages, max_requests=max_requests, max_seq_len=max_seq,
                        dtype=torch.float32, device="cpu", **kw)


def test_free_list_refuses_misuse():
    fl = FreeList(3)
    a = fl.alloc(2)
    with pytest.raises(OutOfPages):
        fl.alloc(2)
    fl.free(a[:1])
    with pytest.raises(ValueError, match="twice"):
        fl.free(a[:1])
    with pytest.raises(ValueError, match="does not exist"):
        fl.free([7])
    fl.check()
    assert fl.num_free == 2 and fl.num_held == 1


def test_groups_are_formed_by_need():
    needs = [CacheNeeds(kv=FULL), CacheNeeds(kv=WINDOW), CacheNeeds(kv=FULL, states=(StateNeed("s", (3, 2)),)),
             CacheNeeds(states=(StateNeed("only", (5,), torch.float32),))]
    m = manager(needs)
    assert len(m.groups) == 2
    assert m.groups[0].layers == [0, 2] and m.groups[1].layers == [1]
    assert {n: tuple(t.shape) for n, t in m.groups[0].storage.items()} == {"k": (2, 13, 16, 2, 16), "v": (2, 13, 16, 2, 16)}   # 12 pages and the dummy page
    assert m.states[2]["s"].shape == (5, 3, 2) and m.states[3]["only"].dtype == torch.float32
    k, v, gi = m.kv(2)
    assert gi == 0 and k.shape == (13, 16, 2, 16)
    assert m.dummy_row == 4 and (m.groups[0].block_table[4] == 12).all()     # the dummy request's row names the dummy page


def test_pages_follow_length_and_return_at_release():
    m = manager([CacheNeeds(kv=FULL)])
    a = m.admit()
    m.extend(a, 17)
    assert m.groups[0].pool.num_held == 2
    m.extend(a, 32)
    assert m.groups[0].pool.num_held == 2
    m.extend(a, 33)
    assert m.groups[0].pool.num_held == 3
    assert m.slot_of(0, a, 20) == int(m.groups[0].block_table[a.row, 1]) * 16 + 4
    m.check_integrity()
    m.release(a)
    assert m.groups[0].pool.num_held == 0 and m.rows.num_free == 4
    with pytest.raises(ValueError, match="twice"):
        m.release(a)
    m.check_integrity()


def test_window_group_gives_pages_back_as_the_window_passes():
    m = manager([CacheNeeds(kv=FULL), CacheNeeds(kv=WINDOW)], pages=16)
    a = m.admit()
    m.extend(a, 100)                              # one step of 100 tokens: nothing behind it yet
    full, win = m.groups
    assert full.pool.num_held == 7 and win.pool.num_held == 7
    m.extend(a, 101)                              # next token at position 100 sees keys >= 61: pages 0..2 go
    assert win.pool.num_held == 7 - 3 and full.pool.num_held == 7
    assert (win.block_table[a.row, :3] == -1).all() and win.block_table[a.row, 3] >= 0
    m.check_integrity()
    for n in range(102, 200):
        m.extend(a, n)
        m.check_integrity()
        assert win.pool.num_held <= 4             # window 40 + one token spans at most 4 pages of 16
    m.release(a)
    m.check_integrity()
    assert win.pool.num_held == 0 and full.pool.num_held == 0


def test_extending_again_to_the_same_length_from_the_same_first_position_changes_nothing():
    """A step planned ahead and then dropped has grown its requests; the same step planned again names the position
    of its first token, and neither takes pages nor gives back a page that this token still sees."""
    m = manager([CacheNeeds(kv=FULL), CacheNeeds(kv=WINDOW)], pages=16)
    a = m.admit(reserve_tokens=200)
    m.extend(a, 103)
    full, win = m.groups
    for pos in range(103, 140):                   # position 103: the window's oldest key, 64, is the first of page 4
        m.extend(a, pos + 1, first_pos=pos)
        held = (full.pool.num_held, win.pool.num_held, a.length, dict(a.reserved))
        table = win.block_table[a.row].copy()
        oldest_seen = pos - 40 + 1
        assert win.block_table[a.row, oldest_seen // 16] >= 0
        m.extend(a, pos + 1, first_pos=pos)       # once more: the cache already holds pos + 1 tokens
        assert (full.pool.num_held, win.pool.num_held, a.length, dict(a.reserved)) == held
        assert (win.block_table[a.row] == table).all()
        m.check_room([(a, pos + 1)])
        m.check_integrity()
    m.release(a)
    m.check_integrity()


def test_reservation_blocks_admission_not_running_requests():
    m = manager([CacheNeeds(kv=FULL)], pages=10)
    a = m.admit(reserve_tokens=100)               # 7 pages set aside
    assert not m.can_admit(80) and m.can_admit(48)
    b = m.admit(reserve_tokens=48)                # 3 pages
    assert not m.can_admit(1)
    with pytest.raises(OutOfPages):
        m.admit(1)
    m.extend(a, 100)
    m.extend(b, 48)                               # both can always grow to what they reserved
    m.check_integrity()
    m.release(a)
    assert m.can_admit(100)
    m.release(b)
    m.check_integrity()
    assert not m.fits_at_all(10 * 16 + 1) and m.fits_at_all(160)


def test_unreserved_growth_fails_loudly_when_the_pool_is_dry():
    m = manager([CacheNeeds(kv=FULL)], pages=3)
    a, b = m.admit(), m.admit()
    m.extend(a, 32)
    m.extend(b, 16)
    with pytest.raises(OutOfPages):
        m.extend(b, 17)
    with pytest.raises(OutOfPages):
        m.extend(a, 10_000)
    with pytest.raises(ValueError, match="shrinks"):
        m.extend(a, 5)


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_of_requests_keep_every_page_accounted(seed):
    rng = random.Random(seed)
    m = manager([CacheNeeds(kv=FULL), CacheNeeds(kv=WINDOW, states=(StateNeed("s", (2,)),))], pages=20,
                max_requests=5, max_seq=200)
    live = []
    for _ in range(400):
        action = rng.random()
        if action < 0.25 and m.rows.num_free:
            reserve = rng.choice([0, 0, rng.randrange(1, 120)])
            if m.can_admit(reserve):
                live.append([m.admit(reserve), reserve])
        elif action < 0.85 and live:
            rc, reserve = rng.choice(live)
            limit = reserve if reserve else 200
            new_len = min(limit, rc.length + rng.choice([1, 1, 1, 2, 7, 30]))
            try:
                m.extend(rc, new_len)
            except OutOfPages:
                assert reserve == 0                # a reserved request never runs dry
        elif live:
            rc, _ = live.pop(rng.randrange(len(live)))
            m.release(rc)
        m.check_integrity()
        for g in m.groups:
            held = sum(int(g.num_pages_of[rc.row] - g.first_page[rc.row]) for rc, _ in live)
            assert held == g.pool.num_held
    for rc, _ in live:
        m.release(rc)
    m.check_integrity()
    assert all(g.pool.num_free == 20 for g in m.groups) and m.rows.num_free == 5


def test_integrity_check_sees_a_corrupted_table():
    m = manager([CacheNeeds(kv=FULL)])
    a, b = m.admit(), m.admit()
    m.extend(a, 20)
    m.extend(b, 20)
    m.groups[0].block_table[b.row, 0] = m.groups[0].block_table[a.row, 0]
    with pytest.raises(AssertionError):
        m.check_integrity()


def test_poison_marks_freed_memory():
    m = manager([CacheNeeds(kv=FULL, states=(StateNeed("s", (2,)),))], poison_on_free=True)
    a = m.admit()
    m.extend(a, 5)
    page = int(m.groups[0].block_table[a.row, 0])
    m.release(a)
    assert all(torch.isnan(t[:, page]).all() for t in m.groups[0].storage.values()) and torch.isnan(m.states[0]["s"][a.row]).all()


def test_check_room_refuses_a_step_whose_third_request_runs_dry_and_changes_nothing():
    m = manager([CacheNeeds(kv=FULL), CacheNeeds(kv=WINDOW)], pages=6)
    a, b, c = m.admit(), m.admit(), m.admit()
    for rc in (a, b, c):
        m.extend(rc, 10)                       # one page each in both groups
    before = [(rc.length, int(m.groups[0].num_pages_of[rc.row])) for rc in (a, b, c)]
    growth = [(a, 30), (b, 30), (c, 40)]       # 1 + 1 + 2 more pages of the full group; three are free
    with pytest.raises(OutOfPages):
        m.check_room(growth)
    assert [(rc.length, int(m.groups[0].num_pages_of[rc.row])) for rc in (a, b, c)] == before
    m.check_integrity()
    m.check_room(growth[:2])
    for rc, n in growth[:2]:
        m.extend(rc, n)
    m.check_integrity()


def test_check_room_agrees_with_what_extend_does():
    rng = random.Random(5)
    for trial in range(200):
        needs = [CacheNeeds(kv=FULL)] + ([CacheNeeds(kv=WINDOW)] if trial % 2 else [])
        m = manager(needs, pages=rng.randint(3, 10), max_seq=160)
        reqs = []
        for _ in range(rng.randint(1, 4)):
            reserve = rng.choice([0, 0, 40, 90])
            if m.can_admit(reserve):
                reqs.append(m.admit(reserve))
        # a few steps so that requests hold pages and windows have passed some
        for _ in range(rng.randint(0, 3)):
            for rc in reqs:
                try:
                    m.extend(rc, min(rc.length + rng.randint(1, 50), 160))
                except OutOfPages:
                    pass
        growth = [(rc, min(rc.length + rng.randint(1, 60), 160)) for rc in reqs]
        try:
            m.check_room(growth)
            fits = True
        except OutOfPages:
            fits = False
        ran_dry = False
        for rc, n in growth:
            try:
                m.extend(rc, n)
            except OutOfPages:
                ran_dry = True
                break
        assert fits != ran_dry, (trial, fits, ran_dry)
        m.check_integrity()


def test_paged_needs_other_than_equal_keys_and_values():
    """A cache of latents (one tensor per token, of its own dtype), keys and values of different head sizes, and the
    usual pair: three groups with their own pools, storage shapes and block tables, paged alike."""
    latent = PagedNeed((PagedTensor("latent", (40,), torch.float32), PagedTensor("rope_key", (8,))), window=None)
    uneven = KVNeed(2, 24, value_head_dim=16)
    needs = [CacheNeeds(kv=latent), CacheNeeds(kv=uneven), CacheNeeds(kv=FULL), CacheNeeds(kv=latent)]
    m = CacheManager(needs, page_size=16, num_pages=6, max_requests=2, max_seq_len=64, dtype=torch.bfloat16, device="cpu",
                     poison_on_free=True)
    assert len(m.groups) == 3 and m.groups[0].layers == [0, 3]
    g = m.groups[0]
    assert g.tensor("latent", 3).shape == (7, 16, 40) and g.tensor("latent", 3).dtype == torch.float32
    assert g.tensor("rope_key", 0).shape == (7, 16, 8) and g.tensor("rope_key", 0).dtype == torch.bfloat16
    k, v, gi = m.kv(1)
    assert gi == 1 and k.shape == (7, 16, 2, 24) and v.shape == (7, 16, 2, 16)
    item = 2
    assert CacheManager.bytes_per_page(needs, 16, torch.bfloat16) == 16 * (2 * (40 * 4 + 8 * item) + (48 + 32) * item + 64 * item)
    a = m.admit()
    m.extend(a, 40)
    assert all(int(gr.num_pages_of[a.row]) == 3 for gr in m.groups)
    pages = [int(p) for p in g.block_table[a.row, :3]]
    g.tensor("latent", 0)[pages[0]] = 1.0
    m.release(a)
    m.check_integrity()
    assert torch.isnan(g.tensor("latent", 0)[pages[0]]).all() and torch.isnan(g.tensor("rope_key", 3)[pages[2]]).all()
