"""The kernel families that the environment switches select for comparisons (`LOGSSMS_B200_ATTN_TC=0`, `_SSD_TC=0`,
`_GEMM=tcgen05`) at model level: a prompt in portions and a few decoded tokens against the plain implementation."""
import pytest
import torch

from tiny import TINY, TOL, make_model_dir, plain_logits, rel_err

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("switch", [("ATTENTION_TC", False), ("SSD_TC", False), ("GEMM_MODE", "tcgen05")])
@pytest.mark.parametrize("name", ["D", "E"])
def test_the_other_kernel_families_give_the_plain_models_logits(tmp_path, monkeypatch, name, switch):
    from logssms_b200.engine import Engine, StepEntry
    from logssms_b200.ops import kernels as K
    monkeypatch.setattr(K, switch[0], switch[1])          # read at every call; the chunk length at the engine's start
    raw = TINY[name]
    model_dir = make_model_dir(tmp_path / "m", raw, seed=61, dtype=torch.bfloat16)
    g = torch.Generator().manual_seed(13)
    ids = torch.randint(0, raw["vocab_size"], (333,), generator=g).tolist()
    want = plain_logits(model_dir, ids, "bfloat16")
    engine = Engine(model_dir, "bfloat16", max_requests=2, max_seq_len=512, num_pages=8, poison_on_free=True)
    launched = []
    if switch[0] == "GEMM_MODE":
        inner = K.gemm_tcgen05
        monkeypatch.setattr(K, "gemm_tcgen05", lambda *a, **kw: (launched.append(1), inner(*a, **kw))[1])
    r = engine.new_request()
    got, at = [], 0
    for n in (200, 70, 55, 1, 1, 1, 1, 1, 1, 1, 1):
        got.append(engine.step([StepEntry(r, ids[at:at + n], list(range(n)))]).float().cpu())
        at += n
    assert at == len(ids)
    K.check_kernel_errors(engine.device)
    engine.release(r)
    engine.cache.check_integrity()
    err = rel_err(torch.cat(got), want)
    assert err <= TOL["bfloat16"], f"{name} with {switch[0]} = {switch[1]}: error {err:.3g}"
    if switch[0] == "GEMM_MODE":
        assert launched, "no product went to the tcgen05 kernel"
