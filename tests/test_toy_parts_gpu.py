"""Parts that the framework has never seen, defined HERE and registered from outside the package: a feed-forward
with routing (top-1 over small experts), another position encoding (rotation with linearly spaced frequencies), an
output head of another kind (its own matrix and a bias per vocabulary entry), and
a stateful mixer whose scan is a CUDA kernel of its own that lies beside this test.  They are chosen layer by layer
in one toy architecture (layer 0: the toy mixer + the built-in gated MLP; layer 1: attention with the toy encoding
+ the routed feed-forward, last, so that a token whose two best experts nearly tie moves its own logits only), built from a config.json, given random weights, stepped in portions and single
tokens (graph replays included) and compared with a plain computation.  None of this is a model of anybody's.
"""
import os
from ctypes import c_int, c_void_p
from dataclasses import dataclass

import pytest
import torch

from plain import falcon_h1_plain as P

pytestmark = pytest.mark.gpu

ARCH = "ToyPartsForCausalLM"
EMA_CU = os.path.join(os.path.dirname(os.path.abspath(__file__)), "toy_kernels", "toy_ema.cu")
H, HEADS, HD, EXPERTS, EI, I2, V = 48, 3, 16, 3, 40, 56, 97


@dataclass(frozen=True)
class LinearRopeSpec:
    head_dim: int
    rotary_dim: int
    kind: str = "toy_linear_rope"


@dataclass(frozen=True)
class RoutedSpec:
    hidden_size: int
    experts: int
    expert_size: int
    kind: str = "toy_routed"


@dataclass(frozen=True)
class EmaSpec:
    hidden_size: int
    kind: str = "toy_ema_cuda"


def toy_inv_freq(rotary_dim):
    return 1.0 / (1.0 + torch.arange(rotary_dim // 2, dtype=torch.float32))          # linearly spaced wavelengths


def define_toys():
    from logssms_b200 import registry
    from logssms_b200.cache import CacheNeeds, StateNeed
    from logssms_b200.config.specs import AttentionSpec, BlockSpec, GatedMLPSpec, MixerSlot, ModelSpec, NormSpec
    from logssms_b200.models import register_architecture
    from logssms_b200.ops import build
    from logssms_b200.ops import kernels as K
    from logssms_b200.parts import MATRIX, VECTOR, ParamSpec, Part
    from logssms_b200.parts.base import normal_init

    class LinearRope(Part):
        """Another position encoding: it only has to fill the cos|sin table that the rotate-and-store kernels read."""
        kernels = ("rope",)

        def __init__(self, spec):
            self.spec, self.table = spec, None

        def setup(self, rt):
            self.table = K.rope_table(toy_inv_freq(self.spec.rotary_dim).to(rt.device), max(rt.max_seq_len, 1))

    class RoutedFeedForward(Part):
        """Top-1 routing: the router's logits in 32-bit, the chosen expert's output times its softmax weight."""

        def __init__(self, spec, perturb_init=False, shared=None):
            self.spec = spec

        def param_specs(self):
            s = self.spec
            specs = {"router.weight": ParamSpec((s.experts, s.hidden_size), VECTOR, normal_init(0.5))}
            for e in range(s.experts):
                specs[f"experts.{e}.up.weight"] = ParamSpec((s.expert_size, s.hidden_size), MATRIX, normal_init(0.1))
                specs[f"experts.{e}.down.weight"] = ParamSpec((s.hidden_size, s.expert_size), MATRIX, normal_init(0.1))
            return specs

        def bind(self, t):
            self.router = t["router.weight"]
            self.up = [t[f"experts.{e}.up.weight"] for e in range(self.spec.experts)]
            self.down = [t[f"experts.{e}.down.weight"] for e in range(self.spec.experts)]

        def setup(self, rt):
            pass

        def forward(self, x):
            # no host decision depends on the routing (a captured step replays it): every expert runs on all rows
            # and the rows it was not chosen for are masked away
            weights = torch.softmax(x.float() @ self.router.t(), -1)                       # [T, E] float32
            top = weights.argmax(-1)
            out = torch.zeros_like(x)
            for e in range(self.spec.experts):
                h = K.linear(x, self.up[e])
                h = (h.float() * torch.sigmoid(h.float())).to(x.dtype)
                y = K.linear(h, self.down[e])
                pick = (top == e).to(x.dtype)[:, None]
                out = out + (y.float() * weights[:, e:e + 1]).to(x.dtype) * pick
            return out

    class EmaCudaMixer(Part):
        kernels = (EMA_CU, "linear_skinny")                # its own source by path, and one of the package's

        def __init__(self, spec, perturb_init=False, shared=None):
            self.spec = spec

        def param_specs(self):
            n = self.spec.hidden_size
            return {"decay_logit": ParamSpec((n,), VECTOR, normal_init(1.0)), "proj.weight": ParamSpec((n, n), MATRIX, normal_init(0.1))}

        def setup(self, rt):
            self.scan = build.load(EMA_CU).toy_ema_scan
            self.scan.argtypes = [c_void_p] * 7 + [c_int, c_int, c_int, c_void_p]
            self.scan.restype = c_int

        def cache_needs(self):
            return CacheNeeds(states=(StateNeed("ema", (self.spec.hidden_size,), torch.float32),))

        def forward(self, x, ctx, cache_layer, writes_cache=True):
            state = ctx.cache.states[cache_layer]["ema"]
            x = x.contiguous()
            y = torch.empty(x.shape, dtype=torch.float32, device=x.device)
            rc = self.scan(x.data_ptr(), y.data_ptr(), state.data_ptr(), self.decay_logit.data_ptr(), ctx.cu_seqlens.data_ptr(),
                           ctx.start_pos.data_ptr(), ctx.slots.data_ptr(), ctx.num_requests, x.shape[1],
                           int(x.dtype == torch.bfloat16), torch.cuda.current_stream().cuda_stream)
            assert rc == 0
            return K.linear(y.to(x.dtype), self.proj_weight)

    class BiasedHead(Part):
        """An output head of another kind: never tied to the embedding, and with a bias per vocabulary entry."""
        kernels = ("linear_skinny",)

        def __init__(self, vocab_size, hidden_size, multiplier, tied_to):
            assert tied_to is None
            self.vocab_size, self.hidden_size, self.multiplier = vocab_size, hidden_size, multiplier

        def param_specs(self):
            return {"weight": ParamSpec((self.vocab_size, self.hidden_size), MATRIX),
                    "bias": ParamSpec((self.vocab_size,), MATRIX, normal_init(0.5))}

        def forward(self, h):
            return K.linear(h, self.weight, self.bias, out_scale=self.multiplier, out_f32=True)

    for reg, name, cls in ((registry.HEADS, "toy_biased_head", BiasedHead),
                           (registry.POSITION_ENCODINGS, "toy_linear_rope", LinearRope),
                           (registry.FEED_FORWARDS, "toy_routed", RoutedFeedForward),
                           (registry.MIXERS, "toy_ema_cuda", EmaCudaMixer)):
        if name not in reg:
            reg.register(name)(cls)

    @dataclass(frozen=True)
    class ToyConfig:
        rms_norm_eps: float
        architectures: tuple = (ARCH,)
        torch_dtype: str = "bfloat16"
        max_position_embeddings: int = 512

        @classmethod
        def from_dict(cls, raw):
            return cls(raw["rms_norm_eps"])

        def to_dict(self):
            return {"architectures": [ARCH], "rms_norm_eps": self.rms_norm_eps}

        def model_spec(self):
            norm = NormSpec(H, self.rms_norm_eps)
            attention = AttentionSpec(hidden_size=H, num_heads=HEADS, num_kv_heads=1, head_dim=HD,
                                      position=LinearRopeSpec(HD, HD // 2), key_scale=1.0)
            common = dict(mixer_norm=norm, mixer_norm_name="norm1.", feed_forward_norm=norm, feed_forward_norm_name="norm2.",
                          feed_forward_name="ff.")
            layers = (
                BlockSpec(prefix="layers.0.", mixers=(MixerSlot(EmaSpec(H), "ema."),), feed_forward=GatedMLPSpec(H, I2), **common),
                BlockSpec(prefix="layers.1.", mixers=(MixerSlot(attention, "attn."),), feed_forward=RoutedSpec(H, EXPERTS, EI), **common),
            )
            return ModelSpec(vocab_size=V, hidden_size=H, embedding_name="embed.", embedding_multiplier=1.0, lm_head_name="head.",
                             lm_head_multiplier=1.0, tie_word_embeddings=False, final_norm=norm, final_norm_name="final_norm.",
                             layers=layers, lm_head_kind="toy_biased_head")

    register_architecture(ARCH, ToyConfig, replace=True)
    return ToyConfig


def toy_reference(tensors, ids, rd, rnd):
    w = {k: v.to(rd) for k, v in tensors.items()}
    lin = lambda a, m, b=None: rnd(a @ m.T)
    T = len(ids)
    x = rnd(w["embed.weight"][torch.tensor(ids)])
    # layer 0: the toy mixer, gated MLP
    (n1,), res = P.rms_norm_branches(x, w["layers.0.norm1.weight"], 1e-5, None, rnd=rnd)
    a = torch.sigmoid(w["layers.0.ema.decay_logit"].float()).to(rd)
    s, rows = torch.zeros_like(n1[0]), []
    for t in range(T):
        s = a * s + n1[t]
        rows.append(s)
    y = lin(rnd(torch.stack(rows)), w["layers.0.ema.proj.weight"])
    (n2,), res = P.rms_norm_branches(y, w["layers.0.norm2.weight"], 1e-5, res, rnd=rnd)
    x = P.gated_mlp(n2, w["layers.0.ff.gate_proj.weight"], w["layers.0.ff.up_proj.weight"], w["layers.0.ff.down_proj.weight"], 1.0, 1.0, rnd, lin)
    # layer 1: attention with the toy encoding, routed feed-forward
    (n1,), res = P.rms_norm_branches(x, w["layers.1.norm1.weight"], 1e-5, res, rnd=rnd)
    q = lin(n1, w["layers.1.attn.q_proj.weight"]).reshape(T, HEADS, HD)
    k = lin(n1, w["layers.1.attn.k_proj.weight"]).reshape(T, 1, HD)
    v = lin(n1, w["layers.1.attn.v_proj.weight"]).reshape(T, 1, HD)
    pos, inv = torch.arange(T), toy_inv_freq(HD // 2)
    q, k = P.rope_apply(q, pos, inv, HD // 2, rnd), P.rope_apply(k, pos, inv, HD // 2, rnd)
    att = lin(P.causal_attention(q, k, v, HD ** -0.5, None, rnd).reshape(T, HEADS * HD), w["layers.1.attn.o_proj.weight"])
    (n2,), res = P.rms_norm_branches(att, w["layers.1.norm2.weight"], 1e-5, res, rnd=rnd)
    weights = torch.softmax(n2.float() @ w["layers.1.ff.router.weight"].float().T, -1).to(rd)
    top = weights.argmax(-1)
    x = torch.zeros_like(n2)
    for e in range(EXPERTS):
        h = lin(n2, w[f"layers.1.ff.experts.{e}.up.weight"])
        y = lin(rnd(h * torch.sigmoid(h)), w[f"layers.1.ff.experts.{e}.down.weight"])
        x = x + rnd(y * weights[:, e:e + 1]) * (top == e).to(rd)[:, None]
    x = rnd(x)
    (hN,), _ = P.rms_norm_branches(x, w["final_norm.weight"], 1e-5, res, rnd=rnd)
    return rnd(hN @ w["head.weight"].T + w["head.bias"]).float()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_parts_are_chosen_layer_by_layer_built_and_stepped(tmp_path, dtype):
    Config = define_toys()
    from logssms_b200.config import make_model_config
    from logssms_b200.engine import Engine, StepEntry
    from logssms_b200.ops import build
    from logssms_b200.weights import read_checkpoint, write_random_model
    config = make_model_config({"architectures": [ARCH], "rms_norm_eps": 1e-5})
    assert isinstance(config, Config)
    assert EMA_CU in build.all_libraries()                         # a registered part's own source is among the libraries
    store = torch.float32 if dtype == "float32" else torch.bfloat16
    model_dir = write_random_model(config, str(tmp_path / "toy"), seed=6, dtype=store, perturb=True)
    engine = Engine(model_dir, dtype, max_requests=3, max_seq_len=128, page_size=64, num_pages=4)
    assert os.path.basename(build.library_path(EMA_CU)).startswith("lb200_toy_ema-")
    assert len(engine.cache.groups) == 1 and engine.cache.groups[0].layers == [1]          # only layer 1 keeps keys and values
    assert set(engine.cache.states[0]) == {"ema"} and not engine.cache.states[1]
    g = torch.Generator().manual_seed(8)
    seqs = [torch.randint(0, V, (n,), generator=g).tolist() for n in (60, 31)]
    tensors = read_checkpoint(model_dir)
    rd = torch.float64 if dtype == "float32" else torch.float32
    rnd = P._rounder(None if dtype == "float32" else torch.bfloat16)
    want = [toy_reference(tensors, ids, rd, rnd) for ids in seqs]
    tol = 1e-4 if dtype == "float32" else 2e-2
    reqs = [engine.new_request() for _ in seqs]
    done, got = [0, 0], [[], []]
    for step in [(25, 4), (2, 11), (20, 1), (1, 1), (1, 1), (1, 1), (9, 1), (1, 10)]:
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
        w_r = want[r][:g_r.shape[0]]
        # a routed feed-forward is discontinuous where two experts nearly tie: leave out the rare tokens whose choice
        # hangs on a rounding, compare all others
        err = (g_r.double() - w_r.double()).abs().amax(1) / w_r.abs().max()
        assert float((err <= tol).float().mean()) >= 0.95 and float(err.median()) <= tol / 4, f"request {r}: {err.max():.3g}"
    assert any(slot.graph is not None for slot in engine._graphs.values()), "no decode step was replayed from a graph"
