"""Every CUDA kernel alone against its plain reference, at sizes other than the tiny models'.

References are the per-part functions of tests/plain (or a few lines of torch where the kernel has
no counterpart there), computed on the CPU in float64 for the 32-bit kernels and in float32 with
bfloat16 rounding points for the bfloat16 kernels.
"""
import math

import pytest
import torch

from plain import falcon_h1_plain as P

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]
TOL = {torch.float32: 2e-5, torch.bfloat16: 2e-2}


def K():
    from logssms_b200.ops import kernels
    return kernels


def dev(t):
    return t.cuda()


def close(got, want, dtype, scale=None, tol=None):
    got, want = got.double().cpu(), want.double().cpu()
    assert got.shape == want.shape, (got.shape, want.shape)
    assert torch.isfinite(got).all()
    denom = want.abs().max().clamp_min(1e-30) if scale is None else scale
    err = float((got - want).abs().max() / denom)
    assert err <= (TOL[dtype] if tol is None else tol), f"error {err:.3g}"


def rnd_of(dtype):
    return P._rounder(None if dtype == torch.float32 else dtype)


def ref_dtype(dtype):
    return torch.float64 if dtype == torch.float32 else torch.float32


def randn(gen, *shape, dtype=torch.float32, scale=1.0):
    return (torch.randn(*shape, generator=gen) * scale).to(dtype)


# --------------------------------------------------------------------------- embedding
@pytest.mark.parametrize("dtype", DTYPES)
def test_embed_gather_and_gather_rows(dtype):
    g = torch.Generator().manual_seed(0)
    V, H = 301, 200
    table = randn(g, V, H, dtype=dtype)
    ids = torch.randint(0, V, (37,), generator=g, dtype=torch.int32)
    out = K().embed_gather(dev(table), dev(ids), 3.5)
    want = rnd_of(dtype)(table.to(ref_dtype(dtype))[ids.long()] * 3.5)
    close(out, want, dtype, tol=1e-7 if dtype == torch.float32 else 1e-6)   # one rounding of the product
    rows = torch.tensor([5, 0, 36, 5], dtype=torch.int32)
    picked = K().gather_rows(out, dev(rows))
    assert torch.equal(picked.cpu(), out.cpu()[rows.long()])


# --------------------------------------------------------------------------- norms
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H", [40, 100, 1000, 3000, 4104])
@pytest.mark.parametrize("two_inputs", [False, True])
def test_add_rmsnorm(dtype, H, two_inputs):
    g = torch.Generator().manual_seed(H)
    rows = 7
    x, other, res = (randn(g, rows, H, dtype=dtype) for _ in range(3))
    w = 1 + 0.1 * torch.randn(H, generator=g)
    rd = ref_dtype(dtype)
    outs, new_res = K().add_rmsnorm(dev(x), dev(w), 1e-5, dev(res.clone()), other=dev(other) if two_inputs else None,
                                    in_scales=(0.8, 0.7), out_scales=(1.5, 1.2))
    # one input: its multiplier is the output multiplier of the product before, applied (and rounded) while x is read
    x_in = x.to(rd) if two_inputs else rnd_of(dtype)(x.to(rd) * 0.8)
    want_outs, want_res = P.rms_norm_branches(x_in, w.to(rd), 1e-5, res.to(rd), other.to(rd) if two_inputs else None,
                                              (0.8, 0.7), (1.5, 1.2), rnd_of(dtype))
    close(new_res, want_res, dtype)
    for a, b in zip(outs, want_outs):
        close(a, b, dtype)
    # first layer: no residual yet, one output
    (o,), r = K().add_rmsnorm(dev(x), dev(w), 1e-5)
    (wo,), wr = P.rms_norm_branches(x.to(rd), w.to(rd), 1e-5, rnd=rnd_of(dtype))
    close(o, wo, dtype)
    close(r, wr, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("mode", ["gate_only", "before", "after"])
def test_gated_rmsnorm(dtype, mode):
    g = torch.Generator().manual_seed(1)
    rows, groups, width = 5, 3, 120
    k = K()
    y = randn(g, rows, groups * width, dtype=dtype)
    wide = randn(g, rows, groups * width + 50, dtype=dtype)
    gate = wide[:, 20:20 + groups * width]                       # a column view, as the mixer passes it
    w = 1 + 0.1 * torch.randn(groups * width, generator=g)
    rd = ref_dtype(dtype)
    gate_dev = dev(wide)[:, 20:20 + groups * width]
    if mode == "gate_only":
        out = k.gated_rmsnorm(dev(y), gate_dev, None, 1e-6, 1, 0.6, k.GATE_ONLY)
        want = P.silu_gate(y.to(rd), gate.to(rd), 0.6, rnd_of(dtype))
    else:
        out = k.gated_rmsnorm(dev(y), gate_dev, dev(w), 1e-6, groups, 0.6,
                              k.NORM_BEFORE_GATE if mode == "before" else k.NORM_AFTER_GATE)
        want = P.gated_group_norm(y.to(rd), gate.to(rd), w.to(rd), 1e-6, groups, mode == "before", 0.6, rnd_of(dtype))
    close(out, want, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("I", [333, 328])                  # odd width / a multiple of 8 (the 16-byte form)
def test_swiglu_and_scale(dtype, I):
    g = torch.Generator().manual_seed(2)
    rows = 9
    gu = randn(g, rows, 2 * I, dtype=dtype)
    rd, rnd = ref_dtype(dtype), rnd_of(dtype)
    out = K().swiglu(dev(gu), 0.9)
    gg, uu = gu.to(rd)[:, :I], gu.to(rd)[:, I:]
    close(out, rnd(rnd(P.silu(rnd(gg * 0.9))) * uu), dtype)
    close(K().scale(dev(gu), 1.1), rnd(gu.to(rd) * 1.1), dtype)
    f32 = K().scale(dev(gu), 0.25, to_f32=True)
    assert f32.dtype == torch.float32
    close(f32, gu.to(rd) * 0.25, torch.float32)


# --------------------------------------------------------------------------- rotation + cache store
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hd,rotary", [(16, 16), (48, 24), (64, 32), (80, 80), (128, 64)])
def test_rope_kv_store(dtype, hd, rotary):
    g = torch.Generator().manual_seed(hd)
    k = K()
    Hq, Hkv, T, page, pages = 6, 3, 11, 16, 5
    theta = 1e4
    inv = P.rope_inv_freq(rotary, theta)
    table = k.rope_table(dev(inv), 200)
    pos_all = torch.arange(200, dtype=torch.float32)[:, None] * inv[None]
    close(table, torch.cat([pos_all.cos(), pos_all.sin()], 1), torch.float32, tol=2e-6)
    qkv = randn(g, T, (Hq + 2 * Hkv) * hd + 8, dtype=dtype)[:, :(Hq + 2 * Hkv) * hd]      # row-strided view
    positions = torch.randint(0, 200, (T,), generator=g, dtype=torch.int32)
    slots = torch.randperm(page * pages, generator=g)[:T].to(torch.int32)
    slots[3] = -1                                                                        # a token without a slot
    kc = torch.zeros(pages, page, Hkv, hd, dtype=dtype)
    vc = torch.zeros_like(kc)
    qkv_dev = dev(torch.cat([qkv, qkv.new_zeros(T, 8)], 1))[:, :(Hq + 2 * Hkv) * hd]
    kcd, vcd = dev(kc), dev(vc)
    q_out = k.rope_kv_store(qkv_dev, Hq, Hkv, hd, dev(positions), dev(slots), table, kcd, vcd, 0.5)
    rd, rnd = ref_dtype(dtype), rnd_of(dtype)
    q, kk, v = qkv.to(rd).split([Hq * hd, Hkv * hd, Hkv * hd], 1)
    want_q = P.rope_apply(q.reshape(T, Hq, hd), positions, inv, rotary, rnd)
    want_k = P.rope_apply(rnd(kk.reshape(T, Hkv, hd) * 0.5), positions, inv, rotary, rnd)
    close(q_out, want_q, dtype)
    want_kc, want_vc = kc.to(rd).reshape(-1, Hkv, hd), vc.to(rd).reshape(-1, Hkv, hd)
    for t in range(T):
        if slots[t] >= 0:
            want_kc[slots[t]] = want_k[t]
            want_vc[slots[t]] = v.reshape(T, Hkv, hd)[t]
    close(kcd.reshape(-1, Hkv, hd), want_kc, dtype)
    close(vcd.reshape(-1, Hkv, hd), want_vc, dtype, tol=0 if dtype == torch.float32 else 1e-6)


# --------------------------------------------------------------------------- attention over pages
def paged_case(g, dtype, Hq, Hkv, hd, page, lengths, new_tokens, plant=False, key_ramp=0.0):
    """Requests of `lengths` tokens whose last `new_tokens[r]` tokens are this step's queries, keys and
    values scattered over shuffled pages.  Returns device inputs and, per query row, (request, position)."""
    total_pages = sum(-(-n // page) for n in lengths) + 3
    perm = torch.randperm(total_pages, generator=g).tolist()
    kc = torch.full((total_pages, page, Hkv, hd), float("nan"), dtype=dtype)
    vc = torch.full_like(kc, float("nan"))
    max_pages = max(-(-n // page) for n in lengths) + 2
    bt = torch.full((len(lengths), max_pages), -1, dtype=torch.int32)
    keys, values, rows = [], [], []
    for r, n in enumerate(lengths):
        k = randn(g, n, Hkv, hd, dtype=dtype)
        v = randn(g, n, Hkv, hd, dtype=dtype)
        if plant and n > 40:
            k[3] *= 6.0                                  # one far key that the query below will pick
        if key_ramp:                                     # scores that rise (or fall) steadily with the key's position
            k[:, :, 0] = (key_ramp * torch.arange(n) / 64.0)[:, None].to(dtype)
        for p in range(-(-n // page)):
            page_id = perm.pop()
            bt[r, p] = page_id
            lo, hi = p * page, min(n, (p + 1) * page)
            kc[page_id, :hi - lo] = k[lo:hi]
            vc[page_id, :hi - lo] = v[lo:hi]
        keys.append(k)
        values.append(v)
        rows += [(r, pos) for pos in range(n - new_tokens[r], n)]
    q = randn(g, len(rows), Hq, hd, dtype=dtype)
    if key_ramp:
        q[:, :, 0] = 8.0
    if plant:
        for i, (r, pos) in enumerate(rows):
            if lengths[r] > 40 and pos >= 3:
                q[i] = (keys[r][3].float().repeat_interleave(Hq // Hkv, 0) * 0.5).to(dtype)
    token_req = torch.tensor([r for r, _ in rows], dtype=torch.int32)
    positions = torch.tensor([p for _, p in rows], dtype=torch.int32)
    return dict(q=q, kc=kc, vc=vc, bt=bt, token_req=token_req, positions=positions, keys=keys, values=values, rows=rows)


def attention_reference(case, scale, window, rd):
    q = case["q"].to(rd)
    Hq, Hkv = q.shape[1], case["keys"][0].shape[1]
    out = torch.zeros_like(q)
    for i, (r, pos) in enumerate(case["rows"]):
        lo = max(0, pos - window + 1) if window else 0
        k = case["keys"][r].to(rd)[lo:pos + 1].repeat_interleave(Hq // Hkv, 1)
        v = case["values"][r].to(rd)[lo:pos + 1].repeat_interleave(Hq // Hkv, 1)
        s = torch.einsum("hd,shd->hs", q[i], k) * scale
        out[i] = torch.einsum("hs,shd->hd", torch.softmax(s, -1), v)
    return out


ATTN_SHAPES = [  # Hq, Hkv, hd, page
    (4, 2, 16, 16), (3, 1, 32, 64), (8, 2, 64, 64), (6, 6, 48, 16), (16, 1, 80, 32), (5, 1, 128, 64), (2, 1, 256, 16),
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", ATTN_SHAPES)
@pytest.mark.parametrize("kernel", ["split1", "split5", "split_auto"])
def test_paged_attention_kernels(dtype, shape, kernel):
    Hq, Hkv, hd, page = shape
    g = torch.Generator().manual_seed(hd + Hq)
    lengths, new = [70, 1, 333, 64, 129], [5, 1, 1, 64, 2]
    case = paged_case(g, dtype, Hq, Hkv, hd, page, lengths, new)
    k = K()
    scale = hd ** -0.5
    args = (dev(case["q"]), dev(case["kc"]), dev(case["vc"]), dev(case["bt"]), dev(case["token_req"]), dev(case["positions"]), scale)
    splits = {"split1": 1, "split5": 5}.get(kernel) or k.attention_splits(len(case["rows"]), Hq, Hkv, max(lengths))
    out = k.attention_decode(*args, splits=splits)
    close(out, rnd_of(dtype)(attention_reference(case, scale, 0, ref_dtype(dtype))), dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("splits", [1, 7])
def test_attention_finds_a_far_key_and_honours_a_window(dtype, splits):
    g = torch.Generator().manual_seed(5)
    Hq, Hkv, hd, page = 8, 2, 64, 64
    case = paged_case(g, dtype, Hq, Hkv, hd, page, [700, 50, 257], [3, 2, 1], plant=True)
    k = K()
    scale = hd ** -0.5
    args = (dev(case["q"]), dev(case["kc"]), dev(case["vc"]), dev(case["bt"]), dev(case["token_req"]), dev(case["positions"]), scale)
    rd = ref_dtype(dtype)
    want = attention_reference(case, scale, 0, rd)
    # the planted key really dominates: the output is close to that key's value row
    v3 = case["values"][0].to(rd)[3].repeat_interleave(Hq // Hkv, 0)
    assert float((want[0] - v3).abs().max()) < 0.05
    close(k.attention_decode(*args, splits=splits), rnd_of(dtype)(want), dtype)
    for window in (1, 64, 65, 300):
        want_w = rnd_of(dtype)(attention_reference(case, scale, window, rd))
        close(k.attention_decode(*args, window, splits=splits), want_w, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_decode_token_list_leaves_other_rows(dtype):
    g = torch.Generator().manual_seed(6)
    Hq, Hkv, hd, page = 4, 1, 32, 16
    case = paged_case(g, dtype, Hq, Hkv, hd, page, [90, 40], [6, 3])
    k = K()
    scale = hd ** -0.5
    out = torch.full_like(dev(case["q"]), 7.0)
    picked = torch.tensor([8, 0, 5], dtype=torch.int32)
    k.attention_decode(dev(case["q"]), dev(case["kc"]), dev(case["vc"]), dev(case["bt"]), dev(case["token_req"]),
                       dev(case["positions"]), scale, splits=3, token_list=dev(picked), out=out)
    want = rnd_of(dtype)(attention_reference(case, scale, 0, ref_dtype(dtype)))
    mask = torch.zeros(len(case["rows"]), dtype=torch.bool)
    mask[picked.long()] = True
    close(out[dev(mask)], want[mask], dtype)
    assert bool((out[dev(~mask)] == 7.0).all())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", ATTN_SHAPES)
@pytest.mark.parametrize("splits", [1, 3, 40])
def test_attention_decode_step_rotates_stores_attends_and_merges(dtype, shape, splits):
    """One launch against the three-kernel chain: rotate + store, attention, merge."""
    Hq, Hkv, hd, page = shape
    g = torch.Generator().manual_seed(hd + Hq + splits)
    lengths = [70, 1, 333, 64, 129, 700]
    case = paged_case(g, dtype, Hq, Hkv, hd, page, lengths, [1] * len(lengths))
    k = K()
    tokens = len(lengths)
    qkv = randn(g, tokens, (Hq + 2 * Hkv) * hd + 8, dtype=dtype)[:, :(Hq + 2 * Hkv) * hd]        # a row-strided view
    rotary = hd // 2 if hd % 32 == 0 else hd
    inv = 1.0 / (1e4 ** (torch.arange(0, rotary, 2, dtype=torch.float32) / rotary))
    table = k.rope_table(dev(inv), 1024)
    positions = case["positions"]
    slots = torch.tensor([int(case["bt"][r, p // page]) * page + p % page for r, p in case["rows"]], dtype=torch.int32)
    qkv_d = dev(torch.cat([qkv, torch.zeros(tokens, 8, dtype=dtype)], 1))[:, :(Hq + 2 * Hkv) * hd]
    scale = hd ** -0.5
    for window in (0, 100):
        kc1, vc1, kc2, vc2 = dev(case["kc"]), dev(case["vc"]), dev(case["kc"]), dev(case["vc"])
        q = k.rope_kv_store(qkv_d, Hq, Hkv, hd, dev(positions), dev(slots), table, kc1, vc1, 0.5)
        want = k.attention_decode(q, kc1, vc1, dev(case["bt"]), dev(case["token_req"]), dev(positions), scale, window, splits=2)
        got = k.attention_decode_step(qkv_d, Hq, Hkv, hd, dev(positions), dev(slots), table, kc2, vc2, dev(case["bt"]),
                                      dev(case["token_req"]), scale, 0.5, window, splits=splits)
        close(got, want, dtype)
        held = torch.isfinite(kc1.float())                                    # pages nobody owns stay NaN in the case
        assert torch.equal(torch.isfinite(kc2.float()), held)
        assert torch.equal(kc2[held], kc1[held]) and torch.equal(vc2[held], vc1[held])   # the same keys and values were stored
        # write_kv off: nothing is stored, and the own position is read from the cache (stored by someone else)
        kc3, vc3 = kc1.clone(), vc1.clone()
        again = k.attention_decode_step(qkv_d, Hq, Hkv, hd, dev(positions), dev(slots), table, kc3, vc3, dev(case["bt"]),
                                        dev(case["token_req"]), scale, 0.5, window, write_kv=False, splits=splits)
        close(again, want, dtype)
        assert torch.equal(kc3[held], kc1[held])
    assert int(k._counters_for(torch.device("cuda", torch.cuda.current_device()), 1).abs().sum()) == 0


def prefill_inputs(case, lengths, new, tile=64):
    cu = torch.tensor([0] + list(torch.tensor(new).cumsum(0)), dtype=torch.int32)
    start = torch.tensor([n - m for n, m in zip(lengths, new)], dtype=torch.int32)
    tiles = torch.tensor([(b, t0) for b, m in enumerate(new) for t0 in range(0, m, tile)], dtype=torch.int32)
    return cu, start, tiles


@pytest.mark.parametrize("shape", ATTN_SHAPES)
def test_attention_prefill_kernel_over_pages_and_earlier_portions(shape):
    Hq, Hkv, hd, page = shape
    dtype = torch.bfloat16
    g = torch.Generator().manual_seed(hd * 3 + Hq)
    lengths, new = [70, 333, 64, 129, 200, 9], [70, 100, 64, 65, 13, 9]      # whole prompts and later portions
    case = paged_case(g, dtype, Hq, Hkv, hd, page, lengths, new)
    cu, start, tiles = prefill_inputs(case, lengths, new)
    k = K()
    scale = hd ** -0.5
    out = k.attention_prefill(dev(case["q"]), dev(case["kc"]), dev(case["vc"]), dev(case["bt"]), dev(cu), dev(start),
                              dev(tiles), tiles.shape[0], scale)
    close(out, rnd_of(dtype)(attention_reference(case, scale, 0, ref_dtype(dtype))), dtype)


def test_attention_prefill_finds_a_far_key_honours_a_window_and_leaves_other_rows():
    dtype = torch.bfloat16
    g = torch.Generator().manual_seed(15)
    Hq, Hkv, hd, page = 8, 2, 64, 64
    lengths, new = [700, 50, 257], [130, 50, 70]
    case = paged_case(g, dtype, Hq, Hkv, hd, page, lengths, new, plant=True)
    cu, start, tiles = prefill_inputs(case, lengths, new)
    k = K()
    scale = hd ** -0.5
    args = (dev(case["q"]), dev(case["kc"]), dev(case["vc"]), dev(case["bt"]), dev(cu), dev(start))
    rd = ref_dtype(dtype)
    want = attention_reference(case, scale, 0, rd)
    v3 = case["values"][0].to(rd)[3].repeat_interleave(Hq // Hkv, 0)
    assert float((want[0] - v3).abs().max()) < 0.05          # the planted far key dominates
    close(k.attention_prefill(*args, dev(tiles), tiles.shape[0], scale), rnd_of(dtype)(want), dtype)
    for window in (1, 64, 65, 300):
        want_w = rnd_of(dtype)(attention_reference(case, scale, window, rd))
        close(k.attention_prefill(*args, dev(tiles), tiles.shape[0], scale, window), want_w, dtype)
    # only the second request's tile: the other rows stay as they were
    out = torch.full_like(dev(case["q"]), 7.0)
    only = torch.tensor([[1, 0]], dtype=torch.int32)
    k.attention_prefill(*args, dev(only), 1, scale, out=out)
    lo, hi = int(cu[1]), int(cu[2])
    close(out[lo:hi], rnd_of(dtype)(want)[lo:hi], dtype)
    assert bool((out[:lo] == 7.0).all()) and bool((out[hi:] == 7.0).all())


@pytest.mark.parametrize("shape", [(8, 2, 64, 64), (3, 3, 64, 128), (4, 1, 64, 64), (6, 2, 128, 64), (3, 1, 128, 128)])
def test_attention_prefill_on_tcgen05_over_pages_and_earlier_portions(shape):
    """The tcgen05 form (head size 64, pages of a multiple of 64 tokens): whole prompts and later portions, tiles
    that end inside a page whose other rows hold NaN (what a reused page holds in the replay tests), a planted far
    key, windows."""
    Hq, Hkv, hd, page = shape
    dtype = torch.bfloat16
    k = K()
    g = torch.Generator().manual_seed(hd * 3 + Hq)
    lengths, new = [70, 333, 64, 129, 700, 9, 300], [70, 100, 64, 65, 130, 9, 300]
    case = paged_case(g, dtype, Hq, Hkv, hd, page, lengths, new, plant=True)
    assert k.attention_prefill_tc_ok(dev(case["q"]), dev(case["kc"]))
    cu, start, tiles = prefill_inputs(case, lengths, new, 128)
    scale = hd ** -0.5
    kc, vc = dev(case["kc"]).clone(), dev(case["vc"]).clone()
    # rows of the requests' last pages beyond their lengths: stale memory
    for r, n in enumerate(lengths):
        last_page = int(case["bt"][r, (n - 1) // page])
        if n % page:
            kc[last_page, n % page:] = float("nan")
            vc[last_page, n % page:] = float("nan")
    args = (dev(case["q"]), kc, vc, dev(case["bt"]), dev(cu), dev(start))
    rd = ref_dtype(dtype)
    want = attention_reference(case, scale, 0, rd)
    got = k.attention_prefill_tc(*args, dev(tiles), tiles.shape[0], scale)
    k.check_kernel_errors()
    close(got, rnd_of(dtype)(want), dtype)
    close(k.attention_prefill_tc(*args, dev(tiles), tiles.shape[0], scale, splits=2), rnd_of(dtype)(want), dtype)   # ranges, some empty
    for window in (1, 64, 65, 300):
        want_w = rnd_of(dtype)(attention_reference(case, scale, window, rd))
        close(k.attention_prefill_tc(*args, dev(tiles), tiles.shape[0], scale, window), want_w, dtype)
        close(k.attention_prefill_tc(*args, dev(tiles), tiles.shape[0], scale, window, splits=4), want_w, dtype)
    k.check_kernel_errors()
    # only one request's tiles: the other rows stay as they were
    out = torch.full_like(dev(case["q"]), 7.0)
    only = torch.tensor([[1, 0]], dtype=torch.int32)
    k.attention_prefill_tc(*args, dev(only), 1, scale, out=out)
    lo, hi = int(cu[1]), int(cu[2])
    close(out[lo:hi], rnd_of(dtype)(want)[lo:hi], dtype)
    assert bool((out[:lo] == 7.0).all()) and bool((out[hi:] == 7.0).all())


@pytest.mark.parametrize("ramp", [8.3, -8.3, 1.0])
def test_attention_prefill_on_tcgen05_when_the_row_maximum_keeps_moving(ramp):
    """Scores that grow by about 2^12 per 64-key tile make every tile rescale the output row that the kernel keeps in
    tensor memory (with random scores that happens in the first tiles only); falling scores never do after the first
    tile, and leave later tiles with weights that underflow; a slow rise stays below the kernel's threshold, so the
    weights exceed 1 for many tiles."""
    Hq, Hkv, hd, page = 4, 2, 64, 64
    dtype = torch.bfloat16
    k = K()
    g = torch.Generator().manual_seed(7)
    lengths, new = [700, 333, 130], [700, 200, 2]
    case = paged_case(g, dtype, Hq, Hkv, hd, page, lengths, new, key_ramp=ramp)
    cu, start, tiles = prefill_inputs(case, lengths, new, 128)
    tiles64 = prefill_inputs(case, lengths, new, 64)[2]
    scale = hd ** -0.5
    args = (dev(case["q"]), dev(case["kc"]), dev(case["vc"]), dev(case["bt"]), dev(cu), dev(start))
    rd = ref_dtype(dtype)
    for window in (0, 200):
        want = rnd_of(dtype)(attention_reference(case, scale, window, rd))
        close(k.attention_prefill_tc(*args, dev(tiles), tiles.shape[0], scale, window), want, dtype)
        close(k.attention_prefill(*args, dev(tiles64), tiles64.shape[0], scale, window), want, dtype)     # and the mma.sync form
    k.check_kernel_errors()


def test_attention_prefill_on_tcgen05_refuses_other_shapes():
    k = K()
    q = torch.zeros(4, 2, 48, dtype=torch.bfloat16, device="cuda")
    assert not k.attention_prefill_tc_ok(q, torch.zeros(2, 64, 2, 48, dtype=torch.bfloat16, device="cuda"))       # head size 48
    q = torch.zeros(4, 2, 64, dtype=torch.bfloat16, device="cuda")
    assert not k.attention_prefill_tc_ok(q, torch.zeros(2, 16, 2, 64, dtype=torch.bfloat16, device="cuda"))       # pages of 16
    assert not k.attention_prefill_tc_ok(q.float(), torch.zeros(2, 64, 2, 64, device="cuda"))                     # float32


# --------------------------------------------------------------------------- Mamba2: conv and scan
def packed_batch(lens, starts):
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
    return cu, torch.tensor(starts, dtype=torch.int32)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("Kc", [2, 3, 4])
@pytest.mark.parametrize("layout", [(50, 30, 40, 3, 6), (64, 32, 48, 8, 16)])       # odd sizes / 16-byte aligned
def test_causal_conv1d_portions_resume_from_state(dtype, Kc, layout):
    """Three requests; each is run as two portions (the second resumes from the saved window) and must
    equal the conv over the whole sequence.  Lengths include portions shorter than the kernel."""
    g = torch.Generator().manual_seed(Kc)
    k = K()
    C, e0, e1, lead, extra = layout
    scales = (1.1, 0.9, 1.3)
    full = [70, 5, 131]
    first = [69, 1, 64]
    w = randn(g, C, Kc, scale=0.3)
    b = randn(g, C, scale=0.1)
    xs = [randn(g, n, C + extra, dtype=dtype)[:, lead:lead + C] for n in full]
    rd, rnd = ref_dtype(dtype), rnd_of(dtype)
    scale_vec = torch.cat([torch.full((e0,), scales[0]), torch.full((e1 - e0,), scales[1]), torch.full((C - e1,), scales[2])])
    want = [P.causal_conv_silu(rnd(x.to(rd) * scale_vec.to(rd)), w.to(rd), b.to(rd), rnd) for x in xs]
    state = torch.full((5, C, Kc - 1), float("nan"), dtype=dtype).cuda()
    slots = torch.tensor([4, 0, 2], dtype=torch.int32)
    got = [[] for _ in full]
    for part in range(2):
        pieces = [x[:f] if part == 0 else x[f:] for x, f in zip(xs, first)]
        lens = [p.shape[0] for p in pieces]
        starts = [0 if part == 0 else f for f in first]
        cu, sp = packed_batch(lens, starts)
        wide = torch.cat([torch.zeros(sum(lens), lead, dtype=dtype), torch.cat(pieces).contiguous(),
                          torch.zeros(sum(lens), extra - lead, dtype=dtype)], 1).cuda()
        out = k.causal_conv1d(wide[:, lead:lead + C], dev(w), dev(b), state, dev(cu), dev(sp), dev(slots), 3, max(lens),
                              (e0, e1), scales)
        for r in range(3):
            got[r].append(out[int(cu[r]):int(cu[r + 1])].cpu())
    for r in range(3):
        close(torch.cat(got[r]), want[r], dtype)
    # the saved window is the last K-1 scaled inputs, oldest first
    for r in range(3):
        tail = rnd(xs[r].to(rd) * scale_vec.to(rd))[-(Kc - 1):].T
        close(state[int(slots[r])], tail, dtype, tol=1e-6)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(4, 16, 16, 1), (6, 24, 32, 2), (3, 64, 128, 1), (2, 40, 256, 2), (5, 8, 20, 5)])
def test_ssm_scan_portions_resume_from_state(dtype, shape):
    nh, Pd, N, G = shape
    g = torch.Generator().manual_seed(nh * N)
    k = K()
    inner, C = nh * Pd, nh * Pd + 2 * G * N
    full, first = [45, 2, 71], [44, 1, 16]
    A_log = torch.log(1 + 15 * torch.rand(nh, generator=g))
    dt_bias = randn(g, nh, scale=0.5) - 2.0
    D = 1 + 0.1 * torch.randn(nh, generator=g)
    convs = [randn(g, n, C, dtype=dtype) for n in full]
    dts = [randn(g, n, nh + 3, dtype=dtype)[:, 1:1 + nh] for n in full]
    rd, rnd = ref_dtype(dtype), rnd_of(dtype)
    want = []
    for c, d in zip(convs, dts):
        n = c.shape[0]
        x, B, Cm = c.to(rd).split([inner, G * N, G * N], 1)
        y = P.ssm_recurrence(x.reshape(n, nh, Pd), d.to(rd), A_log.to(rd), dt_bias.to(rd), B.reshape(n, G, N),
                             Cm.reshape(n, G, N), D.to(rd), 0.8, rnd)
        want.append(y.reshape(n, inner))
    state = torch.full((4, nh, Pd, N), float("nan"), dtype=torch.float32).cuda()
    slots = torch.tensor([3, 1, 0], dtype=torch.int32)
    got = [[] for _ in full]
    for part in range(2):
        cs = [c[:f] if part == 0 else c[f:] for c, f in zip(convs, first)]
        ds = [d[:f] if part == 0 else d[f:] for d, f in zip(dts, first)]
        lens = [c.shape[0] for c in cs]
        cu, sp = packed_batch(lens, [0 if part == 0 else f for f in first])
        dt_wide = torch.cat([torch.cat(ds), torch.zeros(sum(lens), 5, dtype=dtype)], 1).cuda()
        y = k.ssm_scan(torch.cat(cs).cuda(), dt_wide[:, :nh], dev(A_log), dev(dt_bias), dev(D), state, dev(cu),
                       dev(sp), dev(slots), 3, nh, Pd, N, G, 0.8)
        for r in range(3):
            got[r].append(y[int(cu[r]):int(cu[r + 1])].cpu())
    for r in range(3):
        close(torch.cat(got[r]), want[r], dtype)


def chunk_lists(lens, L):
    chunks, per_request = [], []
    for b, n in enumerate(lens):
        first = len(chunks)
        chunks += [(b, t0) for t0 in range(0, n, L)]
        per_request.append((b, first, len(chunks) - first))
    return torch.tensor(chunks, dtype=torch.int32), torch.tensor(per_request, dtype=torch.int32)


@pytest.mark.parametrize("shape", [(4, 16, 16, 1, 8), (6, 24, 32, 2, 16), (3, 64, 128, 1, 128), (2, 40, 256, 2, 64),
                                   (2, 128, 64, 1, 32), (5, 8, 24, 5, 256),
                                   # head size 64 with chunks of 128: the tcgen05 chunk scan, state sizes 64 to 256
                                   (4, 64, 64, 2, 128), (2, 64, 192, 1, 128), (2, 64, 256, 2, 256), (3, 64, 128, 1, 64),
                                   # ... and heads of 128 as two pieces of 64
                                   (2, 128, 128, 1, 128), (3, 128, 256, 3, 128)])
def test_ssd_prefill_in_chunks_resumes_from_state_and_matches_the_recurrence(shape):
    ssd_case(shape, [150, 40, 300], [70, 17, 129])


@pytest.mark.parametrize("shape", [(3, 64, 128, 1, 128), (2, 128, 256, 1, 128), (2, 64, 256, 2, 128), (2, 48, 64, 1, 64)])
def test_ssd_prefill_over_dozens_of_chunks(shape):
    """The state pass over 33 and 32 chunks of one request (and a short neighbour), as a 4,096-token portion and the
    4,133 tokens that follow it."""
    ssd_case(shape, [8229, 40, 2300], [4096, 17, 2048])


def ssd_case(shape, full, first):
    nh, Pd, N, G, chunk = shape
    dtype = torch.bfloat16
    k = K()
    L = k.ssd_chunk_len(chunk, Pd, N)
    assert 0 < L <= chunk
    g = torch.Generator().manual_seed(nh * 31 + N)
    inner = nh * Pd
    convs = [randn(g, n, inner + 2 * G * N, dtype=dtype) for n in full]
    dts = [randn(g, n, nh, dtype=dtype) for n in full]
    zs = [randn(g, n, inner, dtype=dtype) for n in full]
    A_log = torch.log(1 + 15 * torch.rand(nh, generator=g))
    dt_bias = torch.randn(nh, generator=g) - 3.0
    D = torch.randn(nh, generator=g)
    rd, rnd = ref_dtype(dtype), rnd_of(dtype)
    want = []
    for c, d in zip(convs, dts):
        n = c.shape[0]
        x, B, Cm = c.to(rd).split([inner, G * N, G * N], 1)
        want.append(P.ssm_recurrence(x.reshape(n, nh, Pd), d.to(rd), A_log.to(rd), dt_bias.to(rd), B.reshape(n, G, N),
                                     Cm.reshape(n, G, N), D.to(rd), 0.8, rnd).reshape(n, inner))
    state = torch.full((4, nh, Pd, N), float("nan"), dtype=torch.float32).cuda()
    state_seq = torch.full((4, nh, Pd, N), float("nan"), dtype=torch.float32).cuda()
    slots = torch.tensor([3, 1, 0], dtype=torch.int32)
    got, got_gated = [[] for _ in full], [[] for _ in full]
    for part in range(2):
        cut = lambda ts: [t[:f] if part == 0 else t[f:] for t, f in zip(ts, first)]
        cs, ds, zz = cut(convs), cut(dts), cut(zs)
        lens = [c.shape[0] for c in cs]
        cu, sp = packed_batch(lens, [0 if part == 0 else f for f in first])
        chunks, per_request = chunk_lists(lens, L)
        common = (dev(A_log), dev(dt_bias), dev(D))
        conv_d, dt_d, z_d = torch.cat(cs).cuda(), torch.cat(ds).cuda(), torch.cat(zz).cuda()
        lists = (dev(cu), dev(sp), dev(slots), dev(chunks), chunks.shape[0], dev(per_request), per_request.shape[0], L)
        st_before, st_before2 = state.clone(), state.clone()
        y = k.ssd_prefill(conv_d, dt_d, *common, state, *lists, nh, Pd, N, G, 0.8)
        yg = k.ssd_prefill(conv_d, dt_d, *common, st_before, *lists, nh, Pd, N, G, 0.8, z_d, 0.6)
        y_then_gate = k.gated_rmsnorm(y, z_d, None, 1e-5, 1, 0.6, k.GATE_ONLY)
        if k.ssd_chunk_scan_tc_ok(Pd, N, L):             # that kernel's SiLU is the fast one: a last bit may differ
            close(yg, y_then_gate, dtype, tol=1e-2)
        else:
            assert torch.equal(yg, y_then_gate)
        # the gate as a view whose rows start on no 16-byte boundary (the kernel copies it piece by piece then)
        z_wide = torch.zeros(z_d.shape[0], inner + 12, dtype=dtype, device="cuda")
        z_view = z_wide[:, 4:4 + inner]
        z_view.copy_(z_d)
        y_view = k.ssd_prefill(conv_d, dt_d, *common, st_before2, *lists, nh, Pd, N, G, 0.8, z_view, 0.6)
        assert torch.equal(y_view, yg)
        k.ssm_scan(conv_d, dt_d, *common, state_seq, dev(cu), dev(sp), dev(slots), 3, nh, Pd, N, G, 0.8)
        for r in range(3):
            got[r].append(y[int(cu[r]):int(cu[r + 1])].cpu())
    for r in range(3):
        close(torch.cat(got[r]), want[r], dtype)
    live = [3, 1, 0]
    close(state[live], state_seq[live], dtype)           # the state left behind equals the token-by-token kernel's


def test_ssm_scan_request_list_leaves_other_rows():
    g = torch.Generator().manual_seed(13)
    nh, Pd, N, G = 4, 16, 16, 1
    inner = nh * Pd
    k = K()
    lens = [3, 5, 2]
    n = sum(lens)
    conv = randn(g, n, inner + 2 * G * N, dtype=torch.bfloat16).cuda()
    dt = randn(g, n, nh, dtype=torch.bfloat16).cuda()
    consts = [dev(torch.rand(nh, generator=g)), dev(torch.randn(nh, generator=g) - 2), dev(torch.randn(nh, generator=g))]
    cu, sp = packed_batch(lens, [0, 0, 0])
    slots = dev(torch.tensor([0, 1, 2], dtype=torch.int32))
    st_all, st_some = torch.zeros(3, nh, Pd, N).cuda(), torch.zeros(3, nh, Pd, N).cuda()
    y_all = k.ssm_scan(conv, dt, *consts, st_all, dev(cu), dev(sp), slots, 3, nh, Pd, N, G, 1.0)
    out = torch.full_like(y_all, 7.0)
    picked = dev(torch.tensor([2, 0], dtype=torch.int32))
    k.ssm_scan(conv, dt, *consts, st_some, dev(cu), dev(sp), slots, 3, nh, Pd, N, G, 1.0, request_list=picked, num_listed=2, out=out)
    assert torch.equal(out[:3], y_all[:3]) and torch.equal(out[8:], y_all[8:]) and bool((out[3:8] == 7.0).all())
    assert torch.equal(st_some[[0, 2]], st_all[[0, 2]]) and bool((st_some[1] == 0).all())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(24, 64, 128, 1, 9), (20, 40, 256, 2, 12), (37, 24, 20, 1, 20)])
def test_ssm_scan_beside_other_kernels_gives_the_same_bits(dtype, shape):
    """The form for listed requests that shares the GPU with other kernels (a grid that is resident at once, every CTA
    walking its items with the next state on its way) against one CTA per item: the same threads, the same order of
    sums, the same outputs and states; a list entry that names no request is skipped."""
    nh, Pd, N, G, B = shape
    g = torch.Generator().manual_seed(B * 3 + N)
    k = K()
    inner, C = nh * Pd, nh * Pd + 2 * G * N
    lens = [1 + (r * 5) % 4 for r in range(B)]
    starts = [0 if r % 4 == 1 else 11 for r in range(B)]
    n = sum(lens)
    conv = dev(randn(g, n, C + 8, dtype=dtype))[:, :C]
    dt = dev(randn(g, n, nh, dtype=dtype))
    consts = [dev(torch.log(1 + 15 * torch.rand(nh, generator=g))), dev(randn(g, nh, scale=0.5) - 2.0),
              dev(1 + 0.1 * torch.randn(nh, generator=g))]
    cu, sp = packed_batch(lens, starts)
    slots = torch.randperm(B + 3, generator=g)[:B].to(torch.int32)
    state = randn(g, B + 3, nh, Pd, N)
    for r in range(B):
        if starts[r] == 0:
            state[int(slots[r])] = float("nan")          # a request at position 0 never reads its slot
    listed = [r for r in range(B) if r % 3 != 2]          # some requests of the batch only
    st_a, st_b = dev(state), dev(state)
    y_a = torch.full((n, inner), 7.0, dtype=dtype, device="cuda")
    y_b = y_a.clone()
    common = (conv, dt, *consts)
    k.ssm_scan(*common, st_a, dev(cu), dev(sp), dev(slots), B, nh, Pd, N, G, 0.8,
               request_list=dev(torch.tensor(listed, dtype=torch.int32)), num_listed=len(listed), out=y_a)
    with_gap = listed[:2] + [-1] + listed[2:]
    k.ssm_scan(*common, st_b, dev(cu), dev(sp), dev(slots), B, nh, Pd, N, G, 0.8,
               request_list=dev(torch.tensor(with_gap, dtype=torch.int32)), num_listed=len(with_gap), out=y_b, beside=True)
    assert torch.equal(y_a, y_b)
    assert torch.equal(st_a.nan_to_num(nan=-1.0), st_b.nan_to_num(nan=-1.0))
    rows = torch.cat([torch.arange(int(cu[r]), int(cu[r + 1])) for r in listed])
    assert not bool(torch.isnan(y_b[rows.cuda()].float()).any()) and bool((y_b[rows.cuda()] != 7.0).any())


@pytest.mark.parametrize("shape", [(6, 64, 128, 1, 128), (3, 128, 256, 1, 128), (4, 24, 20, 2, 16)])
def test_a_state_kept_in_bfloat16_is_the_float32_state_rounded_once_per_call(shape):
    """The recurrent state kept in the activation dtype between steps (as the reference keeps it): every kernel that
    reads or writes it (the chunked prompt kernels, the token-by-token kernel in both of its forms) must give the very
    outputs of the 32-bit-state run whose state is rounded to bfloat16 by hand after each call."""
    nh, Pd, N, G, chunk = shape
    dtype = torch.bfloat16
    k = K()
    L = k.ssd_chunk_len(chunk, Pd, N)
    g = torch.Generator().manual_seed(nh + N)
    inner, C = nh * Pd, nh * Pd + 2 * G * N
    consts = [dev(torch.log(1 + 15 * torch.rand(nh, generator=g))), dev(torch.randn(nh, generator=g) - 3.0),
              dev(torch.randn(nh, generator=g))]
    B = 3
    slots = dev(torch.tensor([2, 0, 3], dtype=torch.int32))
    st16 = torch.full((5, nh, Pd, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    st32 = torch.full((5, nh, Pd, N), float("nan"), dtype=torch.float32, device="cuda")
    pos = [0, 0, 0]
    # a prompt portion each (chunked where the sizes allow), a second portion, then single tokens in both scan forms
    for step, lens in enumerate([[150, 40, 300], [129, 17, 33], [1, 1, 1], [1, 1, 1], [3, 1, 2]]):
        n = sum(lens)
        conv, dt = dev(randn(g, n, C, dtype=dtype)), dev(randn(g, n, nh, dtype=dtype))
        cu, sp = packed_batch(lens, pos)
        args = (dev(cu), dev(sp), slots)
        outs = []
        for st in (st16, st32):
            if step < 2 and L > 0:
                chunks, per_request = chunk_lists(lens, L)
                outs.append(k.ssd_prefill(conv, dt, *consts, st, *args, dev(chunks), chunks.shape[0], dev(per_request),
                                          per_request.shape[0], L, nh, Pd, N, G, 0.8))
            else:
                outs.append(k.ssm_scan(conv, dt, *consts, st, *args, B, nh, Pd, N, G, 0.8, beside=step == 3))
        live = [2, 0, 3]
        st32[live] = st32[live].bfloat16().float()          # what keeping the state in bfloat16 does, by hand
        assert torch.equal(outs[0], outs[1]), f"step {step}"
        assert torch.equal(st16[live].float(), st32[live]), f"step {step}"
        pos = [p + m for p, m in zip(pos, lens)]
    assert bool(torch.isnan(st16[[1, 4]].float()).all())      # nobody else's slot was touched


# --------------------------------------------------------------------------- 32-bit matrix product
def test_gemm_f32_is_true_32_bit():
    g = torch.Generator().manual_seed(9)
    M, N, Kd = 37, 150, 1000
    a = randn(g, M, Kd + 4)[:, :Kd]
    w, b = randn(g, N, Kd), randn(g, N)
    out = K().gemm_f32(dev(torch.cat([a, torch.zeros(M, 4)], 1))[:, :Kd], dev(w), dev(b), 0.5)
    want = (a.double() @ w.double().T + b.double()) * 0.5
    # a reduced-precision matrix mode (10-bit mantissa inputs) would err by ~1e-3 here
    close(out, want, torch.float32, tol=3e-6)


# --------------------------------------------------------------------------- products of a few rows
@pytest.mark.parametrize("M", [1, 7, 8, 13, 33, 64])
@pytest.mark.parametrize("N,Kd", [(16, 64), (100, 1000), (3352, 1024), (1030, 2048)])
def test_linear_skinny_plain_bias_scale_and_f32(M, N, Kd):
    g = torch.Generator().manual_seed(M * 7 + N)
    x = randn(g, M, Kd + 8, dtype=torch.bfloat16)[:, :Kd]          # a row-strided view
    w = randn(g, N, Kd, dtype=torch.bfloat16, scale=0.05)
    b = randn(g, N, dtype=torch.bfloat16)
    k = K()
    xd = dev(torch.cat([x, torch.zeros(M, 8, dtype=torch.bfloat16)], 1))[:, :Kd]
    rnd = rnd_of(torch.bfloat16)
    acc = x.float() @ w.float().T
    close(k.linear_skinny(xd, dev(w)), rnd(acc), torch.bfloat16, tol=4e-3)           # one bfloat16 ulp of the largest
    close(k.linear_skinny(xd, dev(w), dev(b), out_scale=0.7), rnd(rnd(acc + b.float()) * 0.7), torch.bfloat16, tol=8e-3)
    out32 = k.linear_skinny(xd, dev(w), out_scale=0.25, out_f32=True)
    assert out32.dtype == torch.float32
    close(out32, rnd(acc) * 0.25, torch.bfloat16, tol=4e-3)
    # the dispatcher sends these sizes to the same kernel, and more rows to the library
    if M <= k.SKINNY_MAX_ROWS:
        assert torch.equal(k.linear(xd, dev(w)), k.linear_skinny(xd, dev(w)))
    else:
        close(k.linear(xd, dev(w)), rnd(acc), torch.bfloat16, tol=8e-3)


@pytest.mark.parametrize("M", [1, 8, 20, 64])
@pytest.mark.parametrize("I,Kd", [(16, 64), (200, 96), (2048, 1024)])
def test_linear_skinny_swiglu_matches_the_unfused_chain(M, I, Kd):
    g = torch.Generator().manual_seed(M + I)
    x = randn(g, M, Kd, dtype=torch.bfloat16)
    w = randn(g, 2 * I, Kd, dtype=torch.bfloat16, scale=0.1)
    k = K()
    rnd = rnd_of(torch.bfloat16)
    gu = rnd(x.float() @ w.float().T)
    gate = rnd(gu[:, :I] * 0.9)
    want = rnd(rnd(P.silu(gate)) * gu[:, I:])
    close(k.linear_skinny(dev(x), dev(w), swiglu_scale=0.9), want, torch.bfloat16, tol=1e-2)
    close(k.linear_swiglu(dev(x), dev(w), 0.9), want, torch.bfloat16, tol=1e-2)


@pytest.mark.parametrize("M", [1, 8, 13, 16])
@pytest.mark.parametrize("N,Kd", [(16, 64), (1030, 1000), (768, 2048)])
@pytest.mark.parametrize("two_inputs", [False, True])
def test_linear_skinny_with_the_norm_in_its_prologue(M, N, Kd, two_inputs):
    """Residual add + RMSNorm inside the product against the norm kernel followed by the product."""
    g = torch.Generator().manual_seed(M * 3 + N)
    x, other, res = (randn(g, M, Kd, dtype=torch.bfloat16) for _ in range(3))
    nw = (1 + 0.1 * torch.randn(Kd, generator=g)).cuda()
    w = randn(g, N, Kd, dtype=torch.bfloat16, scale=0.05).cuda()
    w2 = randn(g, 2 * N, Kd, dtype=torch.bfloat16, scale=0.05).cuda()
    b = randn(g, N, dtype=torch.bfloat16).cuda()
    k = K()
    oth = dev(other) if two_inputs else None
    (a0, a1), want_res = k.add_rmsnorm(dev(x), nw, 1e-5, dev(res), other=oth, in_scales=(0.8, 0.7), out_scales=(1.5, 1.2), in_place=False)
    shared = {"residual_out": torch.empty_like(dev(x)), "written": False}
    n0 = k.NormedRows(dev(x), oth, dev(res), nw, 1e-5, (0.8, 0.7), 1.5, shared)
    n1 = k.NormedRows(dev(x), oth, dev(res), nw, 1e-5, (0.8, 0.7), 1.2, shared)
    close(k.linear(n0, w, b, out_scale=0.7), k.linear_skinny(a0, w, b, out_scale=0.7), torch.bfloat16, tol=8e-3)
    assert shared["written"]
    close(shared["residual_out"], want_res, torch.bfloat16, tol=1e-6)
    shared["residual_out"].fill_(7.0)                      # the second consumer must leave the residual alone
    close(k.linear_swiglu(n1, w2, 0.9), k.linear_skinny(a1, w2, swiglu_scale=0.9), torch.bfloat16, tol=1.6e-2)
    assert bool((shared["residual_out"] == 7.0).all())
    # no residual wanted, float32 out (the output head)
    lone = k.NormedRows(dev(x), None, None, nw, 1e-6, (1.0, 1.0), 1.0, {"residual_out": None, "written": False})
    (h,), _ = k.add_rmsnorm(dev(x), nw, 1e-6, None, want_residual=False)
    close(k.linear(lone, w, out_scale=0.25, out_f32=True), k.linear_skinny(h, w, out_scale=0.25, out_f32=True), torch.bfloat16, tol=8e-3)
    # any other use falls back to the norm kernel
    close(n1.tensor(), a1, torch.bfloat16, tol=1e-6)


@pytest.mark.parametrize("M", [1, 8, 13, 16])
@pytest.mark.parametrize("N,Kd", [(16, 64), (1024, 512), (1008, 2048)])
@pytest.mark.parametrize("two_inputs", [False, True])
def test_linear_join_leaves_summed_rows_that_later_products_norm_themselves(M, N, Kd, two_inputs):
    """A product that joins the residual stream in its epilogue, then products that take the summed rows and norm
    their own columns, against product -> norm kernel -> product."""
    g = torch.Generator().manual_seed(M * 11 + N)
    k = K()
    x = randn(g, M, Kd, dtype=torch.bfloat16).cuda()
    w = randn(g, N, Kd, dtype=torch.bfloat16, scale=0.05).cuda()
    b = randn(g, N, dtype=torch.bfloat16).cuda()
    other, res = (randn(g, M, N, dtype=torch.bfloat16).cuda() for _ in range(2))
    nw = (1 + 0.1 * torch.randn(N, generator=g)).cuda()
    N2 = 48
    w2 = randn(g, N2, N, dtype=torch.bfloat16, scale=0.05).cuda()
    w3 = randn(g, 2 * N2, N, dtype=torch.bfloat16, scale=0.05).cuda()
    b2 = randn(g, N2, dtype=torch.bfloat16).cuda()
    oth = other if two_inputs else None
    join = k.ResidualJoin(res, (lambda: oth) if two_inputs else None, (0.8, 0.7))
    assert k.linear_join_ok(x, w, b, join)
    rows = k.linear_join(x, w, b, join, out_scale=1.1)
    y = k.linear_skinny(x, w, b, out_scale=1.1)
    if not two_inputs:            # a lone input is not scaled by the norm kernel either
        (n0, n1), want_res = k.add_rmsnorm(y, nw, 1e-5, res, out_scales=(1.5, 1.2), in_place=False)
    else:
        (n0, n1), want_res = k.add_rmsnorm(y, nw, 1e-5, res, other=oth, in_scales=(0.8, 0.7), out_scales=(1.5, 1.2), in_place=False)
    assert torch.equal(rows.residual, want_res)
    assert torch.equal(rows.vsum.to(torch.bfloat16), want_res)
    close(rows.partial.sum(0), (rows.vsum.double() ** 2).sum(-1), torch.float32, tol=1e-5)
    shared = {"residual_out": None, "written": True}
    a0 = k.NormedRows(rows, None, None, nw, 1e-5, (1.0, 1.0), 1.5, shared)
    a1 = k.NormedRows(rows, None, None, nw, 1e-5, (1.0, 1.0), 1.2, shared)
    assert k.deferred_norm_ok(rows) == (M <= k.DEFERRED_NORM_MAX_ROWS)
    # the rows' factors come from sums in another order than the norm kernel's: a value may round the other way
    close(k.linear(a0, w2, b2, out_scale=0.7), k.linear_skinny(n0, w2, b2, out_scale=0.7), torch.bfloat16, tol=8e-3)
    close(k.linear_swiglu(a1, w3, 0.9), k.linear_skinny(n1, w3, swiglu_scale=0.9), torch.bfloat16, tol=1e-2)
    close(k.linear(a0, w2, out_scale=0.25, out_f32=True), k.linear_skinny(n0, w2, out_scale=0.25, out_f32=True), torch.bfloat16, tol=4e-3)
    close(a1.tensor(), n1, torch.bfloat16, tol=4e-3)
    # with the conv step in the epilogue of the consumer
    taps, C, first = 4, 32, 8
    cw, cb = randn(g, C, taps, scale=0.4).cuda(), randn(g, C, scale=0.1).cuda()
    slots = torch.randperm(M + 2, generator=g)[:M].to(torch.int32).cuda()
    start = torch.tensor([0 if i % 3 == 0 else 5 + i for i in range(M)], dtype=torch.int32).cuda()
    state0 = randn(g, M + 2, C, taps - 1, dtype=torch.bfloat16).cuda()
    st_a, st_b = state0.clone(), state0.clone()
    got = k.linear_conv_step(a0, w2, b2, cw, cb, st_a, slots, start, first, first + C, (8, 20), (1.1, 0.9, 1.3))
    want = k.linear_conv_step(n0, w2, b2, cw, cb, st_b, slots, start, first, first + C, (8, 20), (1.1, 0.9, 1.3))
    close(got, want, torch.bfloat16, tol=8e-3)
    close(st_a, st_b, torch.bfloat16, tol=8e-3)


def test_linear_join_is_refused_where_it_does_not_fit():
    k = K()
    x = torch.zeros(4, 64, dtype=torch.bfloat16, device="cuda")
    res = torch.zeros(4, 24, dtype=torch.bfloat16, device="cuda")
    assert not k.linear_join_ok(x, torch.zeros(24, 64, dtype=torch.bfloat16, device="cuda"), None, k.ResidualJoin(res))      # 24 columns
    x17 = torch.zeros(17, 64, dtype=torch.bfloat16, device="cuda")
    assert not k.linear_join_ok(x17, torch.zeros(32, 64, dtype=torch.bfloat16, device="cuda"), None,
                                k.ResidualJoin(torch.zeros(17, 32, dtype=torch.bfloat16, device="cuda")))                  # 17 rows
    assert not k.linear_join_ok(x, torch.zeros(32, 64, dtype=torch.bfloat16, device="cuda"), None, None)


@pytest.mark.parametrize("M", [1, 5, 16, 40])
@pytest.mark.parametrize("taps", [2, 4])
@pytest.mark.parametrize("normed", [False, True])
def test_linear_with_the_conv_step_in_its_epilogue(M, taps, normed):
    """Projection + conv step of a decode batch in one launch against projection, then the conv kernel."""
    if normed and M > 16:
        pytest.skip("the norm prologue takes at most 16 rows")
    g = torch.Generator().manual_seed(M * 5 + taps)
    Kd, first, C, tail = 96, 24, 56, 10                     # output: 24 plain columns | 56 conv channels | 10 plain
    N = first + C + tail
    k = K()
    x = randn(g, M, Kd, dtype=torch.bfloat16).cuda()
    w = randn(g, N, Kd, dtype=torch.bfloat16, scale=0.2).cuda()
    b = randn(g, N, dtype=torch.bfloat16).cuda()
    cw, cb = randn(g, C, taps, scale=0.4).cuda(), randn(g, C, scale=0.1).cuda()
    slots = torch.randperm(M + 3, generator=g)[:M].to(torch.int32).cuda()
    start = torch.tensor([0 if i % 3 == 0 else 5 + i for i in range(M)], dtype=torch.int32).cuda()     # some requests are new
    state0 = randn(g, M + 3, C, taps - 1, dtype=torch.bfloat16).cuda()
    ends, scales = (24, 40), (1.1, 0.9, 1.3)
    if normed:
        nw = (1 + 0.1 * torch.randn(Kd, generator=g)).cuda()
        res = randn(g, M, Kd, dtype=torch.bfloat16).cuda()
        (xin,), _ = k.add_rmsnorm(x, nw, 1e-5, res, out_scales=(1.2,), in_place=False)
        arg = k.NormedRows(x, None, res, nw, 1e-5, (1.0, 1.0), 1.2, {"residual_out": torch.empty_like(x), "written": False})
    else:
        xin = arg = x
    proj = k.linear_skinny(xin, w, b)
    st_want = state0.clone()
    cu = torch.arange(M + 1, dtype=torch.int32).cuda()
    conv = k.causal_conv1d(proj[:, first:first + C], cw, cb, st_want, cu, start, slots, M, 1, ends, scales)
    st_got = state0.clone()
    got = k.linear_conv_step(arg, w, b, cw, cb, st_got, slots, start, first, first + C, ends, scales)
    assert torch.equal(got[:, :first], proj[:, :first]) and torch.equal(got[:, first + C:], proj[:, first + C:])
    close(got[:, first:first + C], conv, torch.bfloat16, tol=8e-3)
    used = slots.long()
    close(st_got[used], st_want[used], torch.bfloat16, tol=8e-3)
    others = torch.ones(M + 3, dtype=torch.bool)
    others[used.cpu()] = False
    assert torch.equal(st_got[others.cuda()], state0[others.cuda()])


def test_linear_many_rows_goes_to_the_library_with_the_same_epilogues():
    g = torch.Generator().manual_seed(4)
    x = randn(g, 130, 256, dtype=torch.bfloat16)
    w = randn(g, 2 * 96, 256, dtype=torch.bfloat16, scale=0.1)
    k = K()
    rnd = rnd_of(torch.bfloat16)
    acc = rnd(x.float() @ w.float().T)
    close(k.linear(dev(x), dev(w), out_scale=1.1), rnd(acc * 1.1), torch.bfloat16, tol=8e-3)
    close(k.linear_swiglu(dev(x), dev(w), 0.9), rnd(rnd(P.silu(rnd(acc[:, :96] * 0.9))) * acc[:, 96:]), torch.bfloat16, tol=1e-2)


@pytest.mark.parametrize("shape", [(128, 128, 64), (130, 200, 72), (65, 72, 1000), (300, 1024, 2048), (2048, 3352, 1024)])
def test_gemm_tcgen05_plain_bias_scale_and_f32(shape):
    M, N, Kd = shape
    g = torch.Generator().manual_seed(M + N)
    x = randn(g, M, Kd + 8, dtype=torch.bfloat16)[:, :Kd]          # a row-strided view
    w = randn(g, N, Kd, dtype=torch.bfloat16, scale=0.05)
    b = randn(g, N, dtype=torch.bfloat16)
    k = K()
    xd = dev(torch.cat([x, torch.zeros(M, 8, dtype=torch.bfloat16)], 1))[:, :Kd]
    rnd = rnd_of(torch.bfloat16)
    acc = x.float() @ w.float().T
    close(k.gemm_tcgen05(xd, dev(w)), rnd(acc), torch.bfloat16, tol=8e-3)            # one bfloat16 ulp of the largest
    close(k.gemm_tcgen05(xd, dev(w), dev(b), out_scale=0.7), rnd(rnd(acc + b.float()) * 0.7), torch.bfloat16, tol=1.6e-2)
    out32 = k.gemm_tcgen05(xd, dev(w), out_scale=0.25, out_f32=True)
    assert out32.dtype == torch.float32
    close(out32, rnd(acc) * 0.25, torch.bfloat16, tol=8e-3)
    k.check_kernel_errors()
    # exact structure: one hot rows of x pick single rows of w, whatever tile and k-block they sit in
    eye = torch.zeros(M, Kd, dtype=torch.bfloat16)
    cols = torch.randint(0, Kd, (M,), generator=g)
    eye[torch.arange(M), cols] = 1.0
    assert torch.equal(k.gemm_tcgen05(dev(eye), dev(w)).cpu(), w[:, cols].T.contiguous())


@pytest.mark.parametrize("shape", [(128, 64, 64), (200, 200, 96), (2048, 2048, 1024)])
def test_gemm_tcgen05_swiglu_matches_the_unfused_chain(shape):
    M, I, Kd = shape
    g = torch.Generator().manual_seed(M + I)
    x = randn(g, M, Kd, dtype=torch.bfloat16)
    w = randn(g, 2 * I, Kd, dtype=torch.bfloat16, scale=0.1)
    k = K()
    rnd = rnd_of(torch.bfloat16)
    gu = rnd(x.float() @ w.float().T)
    want = rnd(rnd(P.silu(rnd(gu[:, :I] * 0.9))) * gu[:, I:])
    close(k.gemm_tcgen05(dev(x), dev(w), swiglu_scale=0.9), want, torch.bfloat16, tol=1.6e-2)
    k.check_kernel_errors()


def test_ssm_scan_with_the_gate_in_its_epilogue():
    g = torch.Generator().manual_seed(12)
    nh, Pd, N, G = 6, 24, 32, 2
    inner = nh * Pd
    k = K()
    for dtype in DTYPES:
        n = 9
        conv = randn(g, n, inner + 2 * G * N, dtype=dtype)
        z = randn(g, n, inner + 3, dtype=dtype)
        dt = randn(g, n, nh, dtype=dtype)
        A_log, dt_bias, D = torch.rand(nh, generator=g), torch.randn(nh, generator=g) - 2, torch.randn(nh, generator=g)
        cu, sp = packed_batch([5, 4], [0, 0])
        args = (dev(A_log), dev(dt_bias), dev(D))
        rest = (dev(cu), dev(sp), dev(torch.tensor([1, 0], dtype=torch.int32)), 2, nh, Pd, N, G, 0.8)
        st1 = torch.zeros(2, nh, Pd, N).cuda()
        st2 = torch.zeros(2, nh, Pd, N).cuda()
        y = k.ssm_scan(dev(conv), dev(dt), *args, st1, *rest)
        zd = dev(z)[:, :inner]
        fused = k.ssm_scan(dev(conv), dev(dt), *args, st2, *rest, gate=zd, gate_scale=0.6)
        unfused = k.gated_rmsnorm(y, zd, None, 1e-5, 1, 0.6, k.GATE_ONLY)
        assert torch.equal(fused, unfused)
        assert torch.equal(st1, st2)


# --------------------------------------------------------------------------- sampling
def test_sample_greedy_is_argmax_lowest_index():
    from logssms_b200.sampling import sample_tokens
    g = torch.Generator().manual_seed(3)
    logits = torch.randn(6, 1003, generator=g)
    logits[2, 77] = logits[2, 500] = 9.0                    # a tie: the lower index wins
    out = sample_tokens(dev(logits), None, None, None, None, None).cpu()
    want = logits.argmax(-1)
    want[2] = 77
    assert out.tolist() == want.tolist()


def test_sample_temperature_frequencies_and_reproducibility():
    from logssms_b200.sampling import sample_tokens
    rows = 4000
    base = torch.tensor([1.0, 0.0, -1.0, 2.0, 0.5])
    logits = dev(base.repeat(rows, 1).contiguous())
    temp = dev(torch.full((rows,), 0.7))
    topk = dev(torch.zeros(rows, dtype=torch.int32))
    topp = dev(torch.ones(rows))
    seeds = dev(torch.full((rows,), 1234, dtype=torch.int64))
    counters = dev(torch.arange(rows, dtype=torch.int64))
    a = sample_tokens(logits, temp, topk, topp, seeds, counters).cpu()
    b = sample_tokens(logits, temp, topk, topp, seeds, counters).cpu()
    assert torch.equal(a, b)
    freq = torch.bincount(a.long(), minlength=5).double() / rows
    want = torch.softmax(base.double() / 0.7, 0)
    assert float((freq - want).abs().max()) < 0.03
    # top_k = 2 keeps the two most likely tokens only; top_p = 0.5 keeps the most likely one (p = 0.66)
    a2 = sample_tokens(logits, temp, dev(torch.full((rows,), 2, dtype=torch.int32)), topp, seeds, counters).cpu()
    assert set(a2.tolist()) == {0, 3}
    a3 = sample_tokens(logits, temp, topk, dev(torch.full((rows,), 0.5)), seeds, counters).cpu()
    assert set(a3.tolist()) == {3}
    # temperature -> 0 is greedy
    a4 = sample_tokens(logits, dev(torch.full((rows,), 1e-6)), topk, topp, seeds, counters).cpu()
    assert set(a4.tolist()) == {3}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H", [40, 1000, 3072])
def test_summed_rmsnorm_norms_32_bit_residual_sums(dtype, H):
    """Rows left by a product that joined the residual, for a consumer that cannot norm them itself."""
    from plain import falcon_h1_plain as P
    k = K()
    g = torch.Generator().manual_seed(H)
    v = randn(g, 5, H, scale=3.0)
    w = 1.0 + 0.1 * randn(g, H)
    rows = k.SummedRows(dev(v), dev(v).to(dtype), None)
    got = k.summed_rmsnorm(rows, dev(w), 1e-5, (1.5, 0.7))
    rd = ref_dtype(dtype)
    want, _ = P.rms_norm_branches(v.to(rd), w.to(rd), 1e-5, out_scales=(1.5, 0.7), rnd=rnd_of(dtype))
    assert got[0].dtype == dtype and len(got) == 2
    for a, b in zip(got, want):
        close(a, b, dtype)


# --------------------------------------------------------------------------- the attention kernels at long contexts
LONG_ATTN_SHAPES = [(8, 2, 64, 64), (12, 2, 128, 64), (6, 2, 128, 128), (3, 1, 32, 64)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", LONG_ATTN_SHAPES)
def test_decode_attention_kernels_over_thousands_of_keys(dtype, shape):
    """Single new tokens over 8,192, 5,000 and 2,065 keys (block tables of up to 128 pages): the split-KV kernel
    against the reference, with a planted far key, and the one-launch decode-step kernel (cluster merge of 8 ranges,
    and more ranges than a cluster holds) against the three-kernel chain."""
    Hq, Hkv, hd, page = shape
    g = torch.Generator().manual_seed(hd + 7 * Hq)
    lengths = [8192, 5000, 2065, 3]
    case = paged_case(g, dtype, Hq, Hkv, hd, page, lengths, [1] * len(lengths), plant=True)
    k = K()
    scale = hd ** -0.5
    rd = ref_dtype(dtype)
    want = attention_reference(case, scale, 0, rd)
    v3 = case["values"][0].to(rd)[3].repeat_interleave(Hq // Hkv, 0)
    assert float((want[0] - v3).abs().max()) < 0.05          # key 3 of 8,192 decides the first row
    args = (dev(case["q"]), dev(case["kc"]), dev(case["vc"]), dev(case["bt"]), dev(case["token_req"]), dev(case["positions"]), scale)
    for splits in (1, k.attention_splits(len(lengths), Hq, Hkv, max(lengths)), 64):
        close(k.attention_decode(*args, splits=splits), rnd_of(dtype)(want), dtype)
    tokens = len(lengths)
    qkv = randn(g, tokens, (Hq + 2 * Hkv) * hd, dtype=dtype)
    inv = 1.0 / (1e4 ** (torch.arange(0, hd, 2, dtype=torch.float32) / hd))
    table = k.rope_table(dev(inv), 8192)
    slots = torch.tensor([int(case["bt"][r, p // page]) * page + p % page for r, p in case["rows"]], dtype=torch.int32)
    for splits in (k.decode_step_splits(tokens, Hq, Hkv, 8192), 8, 40):
        kc1, vc1, kc2, vc2 = dev(case["kc"]), dev(case["vc"]), dev(case["kc"]), dev(case["vc"])
        q = k.rope_kv_store(dev(qkv), Hq, Hkv, hd, dev(case["positions"]), dev(slots), table, kc1, vc1, 0.5)
        chain = k.attention_decode(q, kc1, vc1, dev(case["bt"]), dev(case["token_req"]), dev(case["positions"]), scale, splits=4)
        step = k.attention_decode_step(dev(qkv), Hq, Hkv, hd, dev(case["positions"]), dev(slots), table, kc2, vc2,
                                       dev(case["bt"]), dev(case["token_req"]), scale, 0.5, splits=splits)
        close(step, chain, dtype)


@pytest.mark.parametrize("shape", LONG_ATTN_SHAPES)
def test_prompt_attention_kernels_over_thousands_of_keys(shape):
    """A 2,048-token portion behind 2,148 earlier tokens, a whole 2,300-token prompt and a short neighbour: the
    tensor-core prompt kernels (tcgen05 where it takes the shape) against the reference, a planted far key."""
    Hq, Hkv, hd, page = shape
    dtype = torch.bfloat16
    g = torch.Generator().manual_seed(hd + 11 * Hq)
    lengths, new = [4196, 2300, 50], [2048, 2300, 50]
    case = paged_case(g, dtype, Hq, Hkv, hd, page, lengths, new, plant=True)
    k = K()
    scale = hd ** -0.5
    want = rnd_of(dtype)(attention_reference(case, scale, 0, ref_dtype(dtype)))
    args = (dev(case["q"]), dev(case["kc"]), dev(case["vc"]), dev(case["bt"]))
    cu, start, tiles = prefill_inputs(case, lengths, new, 64)
    close(k.attention_prefill(*args, dev(cu), dev(start), dev(tiles), tiles.shape[0], scale), want, dtype)
    if k.attention_prefill_tc_ok(args[0], args[1]):
        cu, start, tiles = prefill_inputs(case, lengths, new, k.ATTENTION_TC_TILE)
        close(k.attention_prefill_tc(*args, dev(cu), dev(start), dev(tiles), tiles.shape[0], scale), want, dtype)
        # the keys of every tile cut into ranges with a CTA each, merged by a second kernel (few tiles, long contexts)
        for splits in (3, 16):
            close(k.attention_prefill_tc(*args, dev(cu), dev(start), dev(tiles), tiles.shape[0], scale, splits=splits), want, dtype)
        assert k.prefill_splits(4, 6, 4096) == 6 and k.prefill_splits(40, 8, 4096) == 1 and k.prefill_splits(2, 4, 700) == 1
        k.check_kernel_errors()


def test_attention_prefill_on_tcgen05_when_only_some_warps_keep_rescaling():
    """Rows 0..31 of every 128-query tile see scores that rise steeply along the keys (their warp fetches, scales and
    puts back its output rows at every tile), the other rows see random scores (their warps run ahead, up to a tile):
    the products must still wait for every warp's rows of P.  Several launches, since the order of the warps is a
    matter of timing."""
    Hq, Hkv, hd, page = 4, 2, 64, 64
    dtype = torch.bfloat16
    k = K()
    g = torch.Generator().manual_seed(23)
    lengths, new = [2300, 1500], [2300, 1100]
    case = paged_case(g, dtype, Hq, Hkv, hd, page, lengths, new, key_ramp=8.3)
    calm = torch.tensor([(pos - (lengths[r] - new[r])) % 128 >= 32 for r, pos in case["rows"]])
    case["q"][calm, :, 0] = 0.0
    cu, start, tiles = prefill_inputs(case, lengths, new, 128)
    scale = hd ** -0.5
    args = (dev(case["q"]), dev(case["kc"]), dev(case["vc"]), dev(case["bt"]), dev(cu), dev(start))
    want = rnd_of(dtype)(attention_reference(case, scale, 0, ref_dtype(dtype)))
    for _ in range(5):
        close(k.attention_prefill_tc(*args, dev(tiles), tiles.shape[0], scale), want, dtype)
    k.check_kernel_errors()


@pytest.mark.parametrize("shape", [(8, 2, 64, 64), (12, 2, 128, 64), (3, 1, 32, 64), (16, 1, 80, 32), (6, 6, 48, 16)])
@pytest.mark.parametrize("splits", [1, 5, 8, 20])
def test_attention_decode_listed_runs_the_listed_rows_with_rotated_queries(shape, splits):
    """The decode step's tensor-core kernel on some rows of a step (queries rotated and keys stored beforehand):
    equal to the reference on the listed rows, other rows untouched; short and long contexts, a planted far key."""
    Hq, Hkv, hd, page = shape
    dtype = torch.bfloat16
    g = torch.Generator().manual_seed(hd + 3 * Hq + splits)
    lengths, new = [70, 1, 2065, 64, 129, 700], [3, 1, 1, 2, 1, 4]
    case = paged_case(g, dtype, Hq, Hkv, hd, page, lengths, new, plant=True)
    k = K()
    scale = hd ** -0.5
    assert k.attention_decode_listed_ok(dev(case["q"]), dev(case["kc"]))
    want = rnd_of(dtype)(attention_reference(case, scale, 0, ref_dtype(dtype)))
    rows = len(case["rows"])
    listed = torch.tensor([r for r in range(rows) if r % 3 != 1], dtype=torch.int32)
    out = torch.full_like(dev(case["q"]), 7.0)
    k.attention_decode_listed(dev(case["q"]), dev(case["kc"]), dev(case["vc"]), dev(case["bt"]), dev(case["token_req"]),
                              dev(case["positions"]), dev(listed), listed.numel(), scale, splits=splits, out=out)
    mask = torch.zeros(rows, dtype=torch.bool)
    mask[listed.long()] = True
    close(out[dev(mask)], want[mask], dtype)
    assert bool((out[dev(~mask)] == 7.0).all())
    for window in (1, 65, 300):
        want_w = rnd_of(dtype)(attention_reference(case, scale, window, ref_dtype(dtype)))
        got = k.attention_decode_listed(dev(case["q"]), dev(case["kc"]), dev(case["vc"]), dev(case["bt"]), dev(case["token_req"]),
                                        dev(case["positions"]), dev(listed), listed.numel(), scale, window, splits=splits)
        close(got[dev(mask)], want_w[mask], dtype)
    assert int(k._counters_for(torch.device("cuda", torch.cuda.current_device()), 1).abs().sum()) == 0
