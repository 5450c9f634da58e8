"""A mixer that the framework has never seen, with per-request state of its own, defined HERE:
registered, built from a config.json, given random weights, stepped in portions and token by token
(CUDA-graph decode steps included) and through the scheduler, without touching a file of the package.

The toy mixer is an exponential moving average over the tokens of a request followed by a projection:
    s_t = a * s_{t-1} + x_t          (a = sigmoid(decay_logit), per channel; s is the request's state)
    y_t = s_t W^T
Its state is one float32 vector per request, kept in the cache manager's state slots.  It is written
with torch tensor operations only (a test part, not a product kernel), shaped so that nothing depends
on host-side lengths: that is what lets a captured decode step replay it.
"""
from dataclasses import dataclass

import pytest
import torch

from plain import falcon_h1_plain as P

pytestmark = pytest.mark.gpu

ARCH = "ToyEmaForCausalLM"


@dataclass(frozen=True)
class EmaSpec:
    hidden_size: int
    kind: str = "toy_ema"


def define_toy():
    """Registers the toy mixer and a toy architecture (idempotent); returns the config class."""
    from logssms_b200 import registry
    from logssms_b200.cache import CacheNeeds, StateNeed
    from logssms_b200.config.specs import BlockSpec, GatedMLPSpec, MixerSlot, ModelSpec, NormSpec
    from logssms_b200.models import register_architecture
    from logssms_b200.ops import kernels as K
    from logssms_b200.parts import MATRIX, VECTOR, ParamSpec, Part
    from logssms_b200.parts.base import normal_init

    class EmaMixer(Part):
        kernels = ("linear_skinny",)

        def __init__(self, spec, perturb_init=False, shared=None):
            self.spec = spec
            self.decay_logit = self.proj_weight = None

        def param_specs(self):
            H = self.spec.hidden_size
            return {"decay_logit": ParamSpec((H,), VECTOR, normal_init(1.0)), "proj.weight": ParamSpec((H, H), MATRIX, normal_init(0.1))}

        def setup(self, rt):
            pass

        def cache_needs(self):
            return CacheNeeds(states=(StateNeed("ema", (self.spec.hidden_size,), torch.float32),))

        def forward(self, x, ctx, cache_layer, writes_cache=True):
            state = ctx.cache.states[cache_layer]["ema"]                       # [slots, H] float32
            a = torch.sigmoid(self.decay_logit)                                # [H]
            req = ctx.token_req.long()
            slots = ctx.slots.long()
            since_start = (ctx.positions - ctx.start_pos[req]).float()         # 0 for the first token of the portion
            t = torch.arange(ctx.num_tokens, device=x.device)
            same = (req[:, None] == req[None, :]) & (t[None, :] <= t[:, None])
            gap = (t[:, None] - t[None, :]).clamp_min(0).float()
            weights = torch.where(same[..., None], a[None, None, :] ** gap[..., None], torch.zeros((), device=x.device))
            s = torch.einsum("tsh,sh->th", weights, x.float())
            carried = state[slots] * (ctx.start_pos > 0).float()[:, None]      # a request at position 0 starts from zero
            s = s + carried[req] * a[None, :] ** (since_start[:, None] + 1)
            last = (ctx.cu_seqlens[1:] - 1).long()
            state.index_copy_(0, slots, s[last])
            return K.linear(s.to(x.dtype).contiguous(), self.proj_weight)

    if "toy_ema" not in registry.MIXERS:
        registry.MIXERS.register("toy_ema")(EmaMixer)

    @dataclass(frozen=True)
    class ToyConfig:
        num_hidden_layers: int
        hidden_size: int
        intermediate_size: int
        vocab_size: int
        rms_norm_eps: float
        architectures: tuple = (ARCH,)
        torch_dtype: str = "bfloat16"
        max_position_embeddings: int = 512

        @classmethod
        def from_dict(cls, raw):
            return cls(raw["num_hidden_layers"], raw["hidden_size"], raw["intermediate_size"], raw["vocab_size"], raw["rms_norm_eps"])

        def to_dict(self):
            return {"architectures": [ARCH], "num_hidden_layers": self.num_hidden_layers, "hidden_size": self.hidden_size,
                    "intermediate_size": self.intermediate_size, "vocab_size": self.vocab_size, "rms_norm_eps": self.rms_norm_eps}

        def model_spec(self):
            norm = NormSpec(self.hidden_size, self.rms_norm_eps)
            layers = tuple(BlockSpec(prefix=f"layers.{i}.", mixers=(MixerSlot(EmaSpec(self.hidden_size), "ema."),),
                                     mixer_norm=norm, mixer_norm_name="norm1.", feed_forward=GatedMLPSpec(self.hidden_size, self.intermediate_size),
                                     feed_forward_name="mlp.", feed_forward_norm=norm, feed_forward_norm_name="norm2.")
                           for i in range(self.num_hidden_layers))
            return ModelSpec(vocab_size=self.vocab_size, hidden_size=self.hidden_size, embedding_name="embed.",
                             embedding_multiplier=1.0, lm_head_name="head.", lm_head_multiplier=1.0, tie_word_embeddings=True,
                             final_norm=norm, final_norm_name="final_norm.", layers=layers)

    register_architecture(ARCH, ToyConfig, replace=True)
    return ToyConfig


RAW = {"architectures": [ARCH], "num_hidden_layers": 2, "hidden_size": 40, "intermediate_size": 72, "vocab_size": 131,
       "rms_norm_eps": 1e-5}


def toy_reference(tensors, ids, rd, rnd):
    w = {k: v.to(rd) for k, v in tensors.items()}
    lin = lambda a, m, b=None: rnd(a @ m.T)
    x = rnd(w["embed.weight"][torch.tensor(ids)])
    res = None
    for i in range(RAW["num_hidden_layers"]):
        p = f"layers.{i}."
        (n1,), res = P.rms_norm_branches(x, w[p + "norm1.weight"], 1e-5, res, rnd=rnd)
        a = torch.sigmoid(w[p + "ema.decay_logit"].float()).to(rd)
        s, rows = torch.zeros_like(n1[0]), []
        for t in range(n1.shape[0]):
            s = a * s + n1[t]
            rows.append(s)
        y = lin(rnd(torch.stack(rows)), w[p + "ema.proj.weight"])
        (n2,), res = P.rms_norm_branches(y, w[p + "norm2.weight"], 1e-5, res, rnd=rnd)
        x = P.gated_mlp(n2, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"], 1.0, 1.0, rnd, lin)
    (hN,), _ = P.rms_norm_branches(x, w["final_norm.weight"], 1e-5, res, rnd=rnd)
    return lin(hN, w["embed.weight"]).float()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_mixer_is_registered_built_and_stepped(tmp_path, dtype):
    Config = define_toy()
    from logssms_b200.config import make_model_config
    from logssms_b200.engine import Engine, StepEntry
    from logssms_b200.weights import read_checkpoint, write_random_model
    config = make_model_config(RAW)
    assert isinstance(config, Config)
    store = torch.float32 if dtype == "float32" else torch.bfloat16
    model_dir = write_random_model(config, str(tmp_path / "toy"), seed=2, dtype=store, perturb=True)
    engine = Engine(model_dir, dtype, max_requests=3, max_seq_len=128, page_size=16, num_pages=4)
    assert not engine.cache.groups                                   # no keys or values anywhere in this model
    assert all(set(s) == {"ema"} for s in engine.cache.states)
    g = torch.Generator().manual_seed(3)
    seqs = [torch.randint(0, 131, (n,), generator=g).tolist() for n in (50, 23)]
    tensors = read_checkpoint(model_dir)
    rd = torch.float64 if dtype == "float32" else torch.float32
    rnd = P._rounder(None if dtype == "float32" else torch.bfloat16)
    want = [toy_reference(tensors, ids, rd, rnd) for ids in seqs]
    tol = 1e-4 if dtype == "float32" else 2e-2
    # both requests side by side: portions of changing size, then single tokens (graph replays after the first)
    reqs = [engine.new_request() for _ in seqs]
    done, got = [0, 0], [[], []]
    plan = [(20, 3), (2, 9), (17, 1), (1, 1), (1, 1), (1, 1), (8, 1), (1, 6)]
    for step in plan:
        entries, spans = [], []
        for r, n in enumerate(step):
            n = min(n, len(seqs[r]) - done[r])
            if n:
                entries.append(StepEntry(reqs[r], seqs[r][done[r]:done[r] + n], list(range(n))))
                spans.append((r, n))
        logits = engine.step(entries).cpu()
        at = 0
        for r, n in spans:
            got[r].append(logits[at:at + n].clone())
            at += n
            done[r] += n
    for r in range(2):
        g_r = torch.cat(got[r])
        err = float((g_r.double() - want[r][:g_r.shape[0]].double()).abs().max() / want[r].abs().max())
        assert err <= tol, f"request {r}: error {err:.3g}"
    assert any(slot.graph is not None for slot in engine._graphs.values()), "no decode step was replayed from a graph"
    # a released slot is used again by a new request, which must start from zero whatever the slot holds
    engine.release(reqs[0])
    again = engine.new_request()
    assert again.row == reqs[0].row
    logits = engine.step([StepEntry(again, seqs[0][:7], list(range(7)))]).cpu()
    assert float((logits.double() - want[0][:7].double()).abs().max() / want[0].abs().max()) <= tol


def test_toy_model_generates_through_the_scheduler(tmp_path):
    define_toy()
    from logssms_b200.config import make_model_config
    from logssms_b200.engine import LLM
    from logssms_b200.sampling import SamplingParams
    from logssms_b200.weights import read_checkpoint, write_random_model
    model_dir = write_random_model(make_model_config(RAW), str(tmp_path / "toy"), seed=4, dtype=torch.float32, perturb=True)
    llm = LLM(model_dir, "float32", max_running_requests=2, max_seq_len_override=64, page_size=16, num_pages=4, max_prefill_tokens=16)
    prompts = [[5, 9, 100, 3], list(range(30)), [7]]
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True))
    tensors = read_checkpoint(model_dir)
    for prompt, out in zip(prompts, outs):
        ids = list(prompt)
        for tok in out.token_ids:
            logits = toy_reference(tensors, ids, torch.float64, lambda t: t)[-1]
            assert float(logits.max() - logits[tok]) / float(logits.abs().max()) < 1e-4
            ids.append(tok)
        assert len(out.token_ids) == 5 and out.finish_reason == "length"
