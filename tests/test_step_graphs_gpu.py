"""Steps whose shape comes again are replayed from CUDA graphs: the logits must be those of the same steps
run kernel by kernel, for other requests, other tokens, other pages and other places in the sequence than
the ones the graph was captured with."""
import pytest
import torch

from tiny import TINY, TOL, make_model_dir, plain_logits

pytestmark = pytest.mark.gpu


def run_steps(engine, plan, prompts):
    """`plan`: a list of steps, each a list of (request name, number of tokens, wanted places); the tokens are
    taken from the request's prompt in order.  Returns the logits of every step (on the host)."""
    from logssms_b200.engine import StepEntry
    live, done, out = {}, {}, []
    for step in plan:
        entries = []
        for name, n, want in step:
            if name not in live:
                live[name], done[name] = engine.new_request(), 0
            ids = prompts[name][done[name]:done[name] + n]
            assert len(ids) == n
            done[name] += n
            entries.append(StepEntry(live[name], ids, want))
        out.append(engine.step(entries).float().cpu().clone())
        for name in [nm for nm, _, _ in step if done[nm] == len(prompts[nm])]:
            engine.release(live.pop(name))
    for r in live.values():
        engine.release(r)
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_steps_of_a_repeated_shape_replay_from_a_graph_with_the_same_logits(tmp_path, name, dtype):
    from logssms_b200.engine import Engine as _Engine

    def Engine(*a, **kw):
        e = _Engine(*a, **kw)
        e.exact_after = 0          # a shape gets a graph of its own at once (by default only after some steps through its bucket's)
        return e
    raw = TINY[name]
    model_dir = make_model_dir(tmp_path / "m", raw, seed=41, dtype=torch.float32 if dtype == "float32" else torch.bfloat16)
    g = torch.Generator().manual_seed(9)
    prompts = {k: torch.randint(0, raw["vocab_size"], (n,), generator=g).tolist()
               for k, n in (("a", 120), ("b", 80), ("c", 80), ("d", 47), ("e", 47), ("f", 47), ("g", 47))}
    plan = []
    # one prompt in equal portions of 40 (the same shape at other places of the sequence)
    plan += [[("a", 40, [39])] for _ in range(3)]
    # the same prompt length again and again, for other requests
    plan += [[(k, 47, [46])] for k in ("d", "e", "f", "g")]
    # a mixed shape again and again: a portion of 20 beside a portion of 3 and a single token
    plan += [[("b", 20, [19]), ("c", 3, []), ("d2", 1, [0])] for _ in range(4)]
    prompts["d2"] = torch.randint(0, raw["vocab_size"], (4,), generator=g).tolist()
    results = {}
    for graphs in (False, True):
        engine = Engine(model_dir, dtype, max_requests=4, max_seq_len=128, num_pages=8, use_graphs=graphs, poison_on_free=True)
        results[graphs] = run_steps(engine, plan, prompts)
        engine.cache.check_integrity()
        if graphs:
            captured = {k for k, slot in engine._shape_graphs.items() if slot.graph is not None}
            assert ((40,), 1) in captured and ((47,), 1) in captured and ((20, 3, 1), 2) in captured
        del engine
    # the same kernels; a replayed step may cut the keys of single tokens into other ranges than the step run
    # kernel by kernel (it is planned for the longest context), which moves float32 sums by a rounding
    tol = 1e-5 if dtype == "float32" else TOL[dtype]
    for i, (a, b) in enumerate(zip(results[False], results[True])):
        assert a.shape == b.shape, f"step {i}"
        scale = float(a.abs().max()) or 1.0
        assert float((a - b).abs().max()) <= tol * scale, f"step {i}: graph replay differs from the kernel-by-kernel run"


def test_step_graphs_are_bounded_in_number_and_in_tokens(tmp_path):
    from logssms_b200.engine import Engine, StepEntry
    raw = TINY["A"]
    model_dir = make_model_dir(tmp_path / "m", raw, seed=42)
    engine = Engine(model_dir, "float32", max_requests=2, max_seq_len=128, num_pages=4, max_shape_graphs=2, max_graph_tokens=16)
    engine.exact_after = 0             # every shape straight to a graph of its own
    for n in (10, 11, 12, 20):
        for _ in range(3):
            r = engine.new_request()
            engine.step([StepEntry(r, list(range(n)), [n - 1])])
            engine.release(r)
    assert len(engine._shape_graphs) == 2 and all(k[0][0] <= 16 for k in engine._shape_graphs)


def test_shapes_that_never_recur_push_no_captured_graph_out(tmp_path):
    """One-off shapes take no slot and no device tables; a shape that came only twice goes before a captured one;
    among captured graphs the one used longest ago goes."""
    from logssms_b200.engine import Engine, StepEntry
    raw = TINY["A"]
    model_dir = make_model_dir(tmp_path / "m", raw, seed=43)
    engine = Engine(model_dir, "float32", max_requests=2, max_seq_len=128, num_pages=4, max_shape_graphs=2, max_graph_tokens=64)
    engine.exact_after = 0             # every shape straight to a graph of its own

    def prompt(n):
        r = engine.new_request()
        engine.step([StepEntry(r, list(range(n)), [n - 1])])
        engine.release(r)

    def captured():
        return {k[0][0] for k, slot in engine._shape_graphs.items() if slot.graph is not None}

    for n in (10, 11):
        for _ in range(3):
            prompt(n)
    assert captured() == {10, 11}
    for n in range(20, 40):            # twenty shapes that come once
        prompt(n)
    assert captured() == {10, 11} and len(engine._shape_graphs) == 2
    prompt(12)
    prompt(12)                         # a second sight takes a slot: the graph used longest ago (10) makes room
    assert captured() == {11} and set(k[0][0] for k in engine._shape_graphs) == {11, 12}
    prompt(13)
    prompt(13)                         # ... and the slot without a graph (12) goes before the captured one
    assert captured() == {11} and set(k[0][0] for k in engine._shape_graphs) == {11, 13}
    assert len(engine._sightings) <= 64


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["B", "D", "E"])
def test_steps_of_new_shapes_replay_the_graph_of_their_bucket(tmp_path, name, dtype):
    """Mixed steps none of whose shapes comes twice (decoding requests beside prompt portions of changing length):
    filled up with dummy requests to the sizes of a bucket, they are captured once per bucket and replayed.  The
    logits must be those of the same steps run kernel by kernel without any filling, and the plain model's."""
    from logssms_b200.engine import Engine
    from tiny import plain_logits, rel_err
    raw = TINY[name]
    model_dir = make_model_dir(tmp_path / "m", raw, seed=44, dtype=torch.float32 if dtype == "float32" else torch.bfloat16)
    g = torch.Generator().manual_seed(19)
    sizes = {"p": 700, "q": 520, "r": 74 + 81 + 60, "d0": 40, "d1": 23, "d2": 31}
    prompts = {k: torch.randint(0, raw["vocab_size"], (n,), generator=g).tolist() for k, n in sizes.items()}
    plan = [[("d0", 12, [11]), ("d1", 9, [8]), ("d2", 10, [9])]]
    # prompt p in portions of 100 + i beside the three decoding requests; then q beside two of them
    portions_p = [100, 101, 99, 102, 98, 103, 97]
    for n in portions_p:
        plan.append([("d0", 1, [0]), ("d1", 1, [0]), ("d2", 1, [0]), ("p", n, [n - 1])])
    for n in (150, 133):
        plan.append([("d0", 1, [0]), ("q", n, [n - 1]), ("d2", 1, [0])])
    # two prompt portions in one step: q goes on while r starts (a new request behind a continuing one) and goes on
    for n, m in ((129, 74), (108, 81)):
        plan.append([("d0", 1, [0]), ("q", n, [n - 1]), ("r", m, [m - 1]), ("d2", 1, [0])])
    plan.append([("r", 60, [59]), ("d0", 1, [0])])
    results = {}
    for graphs in (False, True):
        engine = Engine(model_dir, dtype, max_requests=6, max_seq_len=1024, num_pages=24, use_graphs=graphs, poison_on_free=True)
        results[graphs] = run_steps(engine, plan, prompts)
        engine.cache.check_integrity()
        if graphs:
            replayed = sum(max(0, slot.seen - 1) for slot in engine._bucket_graphs.values() if slot.graph is not None)
            assert replayed >= 7, {k: slot.seen for k, slot in engine._bucket_graphs.items()}
            assert not engine._shape_graphs                      # no shape came twice
        del engine
    tol = 2e-5 if dtype == "float32" else TOL[dtype]
    for i, (a, b) in enumerate(zip(results[False], results[True])):
        assert a.shape == b.shape, f"step {i}"
        scale = float(a.abs().max()) or 1.0
        assert float((a - b).abs().max()) <= tol * scale, f"step {i}: the bucket's graph differs from the kernel-by-kernel run"
    # and against the plain model: the last token of every portion of p
    want = plain_logits(model_dir, prompts["p"], dtype)
    ends = [sum(portions_p[:i + 1]) - 1 for i in range(len(portions_p))]
    got = torch.stack([results[True][1 + i][3] for i in range(len(portions_p))])
    assert rel_err(got, want[ends]) <= TOL[dtype]


def test_decoded_tokens_state_update_beside_the_chunked_kernels_of_a_portion(tmp_path):
    """In a captured step the Mamba2 mixer puts the token-by-token state update of the decoded tokens on a stream of
    its own beside the chunked kernels of the prompt portion, as a grid that is resident at once.  That form is taken
    only with hundreds of (request, head) items: a model with 40 small SSM heads and a dozen decoding requests.  The
    replayed steps must give the logits of the same steps run kernel by kernel on one stream, and the plain model's."""
    import copy
    from logssms_b200.engine import Engine
    from tiny import plain_logits, rel_err
    raw = copy.deepcopy(TINY["D"])
    raw.update({"mamba_n_heads": 40, "mamba_d_head": 16, "mamba_d_ssm": 640, "mamba_d_state": 64})
    dtype = "bfloat16"
    model_dir = make_model_dir(tmp_path / "m", raw, seed=47, dtype=torch.bfloat16)
    g = torch.Generator().manual_seed(23)
    decoders = [f"d{i}" for i in range(12)]
    portions_p = [100, 101, 99, 102, 98, 103]
    sizes = {"p": sum(portions_p), **{d: 20 + 3 * i + len(portions_p) for i, d in enumerate(decoders)}}
    prompts = {k: torch.randint(0, raw["vocab_size"], (n,), generator=g).tolist() for k, n in sizes.items()}
    plan = [[(d, 20 + 3 * i, [19 + 3 * i]) for i, d in enumerate(decoders)]]
    for n in portions_p:
        plan.append([*((d, 1, [0]) for d in decoders), ("p", n, [n - 1])])
    results = {}
    for graphs in (False, True):
        engine = Engine(model_dir, dtype, max_requests=16, max_seq_len=1024, num_pages=40, use_graphs=graphs, poison_on_free=True)
        results[graphs] = run_steps(engine, plan, prompts)
        engine.cache.check_integrity()
        if graphs:
            replayed = sum(max(0, slot.seen - 1) for slot in engine._bucket_graphs.values() if slot.graph is not None)
            assert replayed >= 3 and engine._aux_streams is not None, {k: slot.seen for k, slot in engine._bucket_graphs.items()}
        del engine
    for i, (a, b) in enumerate(zip(results[False], results[True])):
        assert a.shape == b.shape and bool(torch.isfinite(b).all()), f"step {i}"
        scale = float(a.abs().max()) or 1.0
        assert float((a - b).abs().max()) <= TOL[dtype] * scale, f"step {i}: the graph differs from the kernel-by-kernel run"
    want_p = plain_logits(model_dir, prompts["p"], dtype)
    ends = [sum(portions_p[:i + 1]) - 1 for i in range(len(portions_p))]
    got_p = torch.stack([results[True][1 + i][len(decoders)] for i in range(len(portions_p))])
    assert rel_err(got_p, want_p[ends]) <= TOL[dtype]
    for j in (0, 7, 11):                                   # ... and the decoded tokens of some of the decoding requests
        d = decoders[j]
        want_d = plain_logits(model_dir, prompts[d], dtype)
        first = 20 + 3 * j
        got_d = torch.stack([results[True][1 + i][j] for i in range(len(portions_p))])
        assert rel_err(got_d, want_d[first:first + len(portions_p)]) <= TOL[dtype]


def test_decode_graphs_captured_ahead_and_the_largest_batch_with_a_graph(tmp_path):
    """`cuda_graph_max_bs` as the reference has it: the decode graphs of batch sizes 1, 2, 4, 8, ... up to it can be
    captured before the first request; a larger decode batch runs kernel by kernel; 0 switches graphs off.  Tokens are
    the same either way."""
    from logssms_b200.engine import LLM
    from logssms_b200.sampling import SamplingParams
    model_dir = make_model_dir(tmp_path / "m", TINY["B"], seed=3)
    prompts = [[3 + i, 9, 27 + i] for i in range(6)]
    sp = SamplingParams(max_tokens=6, ignore_eos=True)
    plain = LLM(model_dir, "float32", max_running_requests=8, max_seq_len_override=128, num_pages=12, cuda_graph_max_bs=0)
    assert not plain.engine.use_graphs
    want = [o.token_ids for o in plain.generate(prompts, sp)]
    del plain
    llm = LLM(model_dir, "float32", max_running_requests=8, max_seq_len_override=128, num_pages=12, cuda_graph_max_bs=4)
    assert sorted(n for n, g in llm.engine._graphs.items() if g.graph is not None) == [1, 2, 4]      # captured at start
    assert not llm.engine.cache.live
    llm.engine.cache.check_integrity()
    assert [o.token_ids for o in llm.generate(prompts, sp)] == want          # six decode together: beyond 4, no graph
    assert 6 not in llm.engine._graphs
    assert [o.token_ids for o in llm.generate(prompts[:2], sp)] == want[:2]  # two: the graph captured at start
    assert llm.engine.capture_decode_graphs([3]) == [3] and llm.engine.capture_decode_graphs([7]) == []


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_decode_batch_without_a_graph_rides_in_the_graph_of_a_larger_one(tmp_path, dtype):
    """With the usual batch sizes captured at start, a decode batch of another size is filled up with dummy requests
    and replayed from the next larger graph: no step of the run is launched kernel by kernel or captured, the dummy
    requests change nobody's tokens, and only a size that keeps coming earns a graph of its own."""
    from logssms_b200.engine import LLM
    from logssms_b200.sampling import SamplingParams
    store = torch.float32 if dtype == "float32" else torch.bfloat16
    model_dir = make_model_dir(tmp_path / "m", TINY["B"], seed=5, dtype=store)
    prompts = [[3 + i, 9, 27 + i] for i in range(7)]
    sp = SamplingParams(max_tokens=7, ignore_eos=True)
    plain = LLM(model_dir, dtype, max_running_requests=8, max_seq_len_override=128, num_pages=12, cuda_graph_max_bs=0)
    want = {k: [o.token_ids for o in plain.generate(prompts[:k], sp)] for k in (3, 5, 6, 7)}
    del plain

    def same(got, ref):
        # float32: the very tokens.  bfloat16: the key ranges of the attention follow the batch size of the graph, so
        # sums round differently and a greedy choice between near-equal logits of a random model may flip, after
        # which that request goes its own way: every token must be the plain implementation's choice after the
        # request's own tokens so far, or within the tolerance of it; the float32 run is the one that proves the mechanism
        if dtype == "float32":
            return got == ref
        for prompt, toks in zip(prompts, got):
            logits = plain_logits(model_dir, prompt + toks[:-1], dtype)[len(prompt) - 1:]
            for tok, row in zip(toks, logits):
                if float(row.max() - row[tok]) / float(row.abs().max()) > TOL[dtype]:
                    return False
        return len(got) == len(ref) and all(len(g) == len(r) for g, r in zip(got, ref))
    llm = LLM(model_dir, dtype, max_running_requests=8, max_seq_len_override=128, num_pages=12, cuda_graph_max_bs=8)
    eng = llm.engine
    assert sorted(n for n, g in eng._graphs.items() if g.graph is not None) == [1, 2, 4, 8]
    eager = {"n": 0}
    run = eng._run

    def counting(ctx, device_tokens):
        eager["n"] += ctx.max_len == 1                      # decode steps only: the prompts' own steps do not count
        return run(ctx, device_tokens)
    eng._run = counting
    for overlap in (True, False):
        llm.scheduler.overlap = overlap
        for k in (3, 5, 6, 7):
            assert same([o.token_ids for o in llm.generate(prompts[:k], sp)], want[k]), (overlap, k)
    assert eager["n"] == 0
    assert sorted(n for n, g in eng._graphs.items() if g.graph is not None) == [1, 2, 4, 8]
    assert not eng.cache.live
    eng.cache.check_integrity()
    eng.exact_after = 2                                     # now a size that keeps coming gets a graph of its own
    for _ in range(2):
        assert same([o.token_ids for o in llm.generate(prompts[:3], sp)], want[3])
    assert eng._graphs.get(3) is not None and eng._graphs[3].graph is not None
