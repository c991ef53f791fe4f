"""Parts alone against their plain counterparts, and the generality of the assembly:
a toy architecture, defined here and registered without touching the framework, whose
layers mix a mixer with state of its own, a windowed attention in a page group of its
own, a layer that reads another layer's cache, and a block that runs twice."""
from dataclasses import dataclass

import pytest
import torch

import plain_llama as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def rnd(*shape, dtype=torch.float32, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (scale * torch.randn(*shape, generator=g)).to(dtype).to(DEV)


def runtime(dtype):
    from mstar_b200.parts import Runtime
    return Runtime(dtype=dtype, device=torch.device(DEV))


def simple_ctx(q_lens, starts):
    """A StepContext for requests that bring q_lens tokens after ``starts`` cached ones."""
    from mstar_b200.parts import StepContext

    token_req = [i for i, n in enumerate(q_lens) for _ in range(n)]
    pos = [s + k for s, n in zip(starts, q_lens) for k in range(n)]
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    indptr = [0]
    for n in q_lens:
        indptr.append(indptr[-1] + n)
    return StepContext(num_tokens=len(pos), num_entries=len(q_lens), token_req=i32(token_req),
                       positions=i32(pos), cache_pos=i32(pos), qo_indptr=i32(indptr),
                       kv_len=i32([s + n for s, n in zip(starts, q_lens)]),
                       slots=i32(list(range(len(q_lens)))), q_lens=list(q_lens),
                       kv_lens=[s + n for s, n in zip(starts, q_lens)],
                       host_slots=list(range(len(q_lens))), max_q_len=max(q_lens),
                       max_kv_len=max(s + n for s, n in zip(starts, q_lens)),
                       num_decode=0)


@pytest.mark.parametrize("dtype", DTYPES)
def test_norm_part(dtype):
    from mstar_b200.config.layout import NormSpec
    from mstar_b200.parts import ResidualStream, build_part

    spec = NormSpec(size=200, eps=1e-4)
    w = (1 + 0.2 * rnd(200, seed=1))
    norm = build_part("norm", spec, {"weight": w}, runtime(dtype))
    h, d = rnd(6, 200, seed=2), rnd(6, 200, dtype=dtype, seed=3)
    stream = ResidualStream(h.clone())
    stream.push(d)
    out = norm.add_norm(stream)
    want = P.plain_rms_norm((h.double() + d.double()).cpu(), w.cpu(), 1e-4)
    assert stream.delta is None and out.dtype == dtype
    assert (out.double().cpu() - want).abs().max() < (1e-5 if dtype == torch.float32 else 3e-2)


@pytest.mark.parametrize("dtype", DTYPES)
def test_gated_mlp_part(dtype):
    from mstar_b200.config.layout import GatedMLPSpec
    from mstar_b200.parts import build_part

    spec = GatedMLPSpec(hidden_size=72, intermediate_size=200)
    gu, dn = rnd(400, 72, dtype=dtype, seed=4, scale=0.1), rnd(72, 200, dtype=dtype, seed=5, scale=0.1)
    mlp = build_part("ffn", spec, {"gate_up.weight": gu, "down.weight": dn}, runtime(dtype))
    x = rnd(9, 72, dtype=dtype, seed=6)
    want = P.plain_swiglu(x.cpu(), gu[:200].cpu(), gu[200:].cpu(), dn.cpu())
    got = mlp.forward(x, None)
    assert (got.double().cpu() - want).abs().max() < (1e-5 if dtype == torch.float32 else 2e-2)
    with pytest.raises(ValueError, match="gelu"):
        build_part("ffn", GatedMLPSpec(hidden_size=72, intermediate_size=200, activation="gelu"),
                   {"gate_up.weight": gu, "down.weight": dn}, runtime(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding_and_head_parts(dtype):
    """The two ends of the residual stream alone: a table with a row multiplier (tokens that
    only the device holds included), and a linear head with a logit scale and a soft cap."""
    from mstar_b200.config.layout import EmbeddingSpec, HeadSpec
    from mstar_b200.parts import build_part

    V, H = 150, 72
    table = rnd(V, H, dtype=dtype, seed=1)
    emb = build_part("embedding", EmbeddingSpec(vocab_size=V, hidden_size=H, multiplier=3.0),
                     {"weight": table}, runtime(dtype))
    assert emb.graph_safe is True
    ids = torch.tensor([5, 149, 0, 7], dtype=torch.int32, device=DEV)
    ctx = simple_ctx([4], [0])
    h = emb.forward(ids, ctx)
    assert h.dtype == torch.float32 and torch.equal(h, table[ids.long()].float() * 3.0)
    # token 1 and 3 come from the device: their ids in `ids` are not to be used
    ctx.token_source = (torch.tensor([-1, 1, -1, 0], dtype=torch.int32, device=DEV),
                        torch.tensor([100, 33], dtype=torch.int32, device=DEV))
    h2 = emb.forward(ids, ctx)
    want_ids = torch.tensor([5, 33, 0, 100], device=DEV)
    assert torch.equal(h2, table[want_ids].float() * 3.0)

    w = rnd(V, H, dtype=dtype, seed=2, scale=0.3)
    x = rnd(6, H, dtype=dtype, seed=3)
    plain = (x.double() @ w.double().T).cpu()
    tol = 1e-4 if dtype == torch.float32 else 2e-2
    head = build_part("head", HeadSpec(vocab_size=V, hidden_size=H), {"weight": w}, runtime(dtype))
    logits = head.forward(x)
    assert logits.dtype == torch.float32 and (logits.double().cpu() - plain).abs().max() < tol
    capped = build_part("head", HeadSpec(vocab_size=V, hidden_size=H, logit_scale=2.0, softcap=3.0),
                        {"weight": w}, runtime(dtype))
    want = 3.0 * torch.tanh(plain * 2.0 / 3.0)
    assert (capped.forward(x).double().cpu() - want).abs().max() < tol


def test_rope_part_holds_the_hand_computed_frequencies_on_the_device():
    """The position part's table, as the kernels read it (float on the device), against
    values worked out by hand from the llama3 rule (tests/test_plain.py; the rule itself is
    compared with the library call the reference makes in tests/test_gpu_library_anchor.py),
    and against the plain rule for a head size and base without scaling."""
    from test_plain import ORPHEUS_FREQS, TINY_B_FREQS

    from mstar_b200.config.layout import PositionSpec, RopeScalingSpec
    from mstar_b200.parts import build_part

    for hd, theta, sc, pins in ((128, 500000.0, (32.0, 1.0, 4.0, 8192), ORPHEUS_FREQS),
                                (32, 500000.0, (8.0, 1.0, 4.0, 32), TINY_B_FREQS),
                                (48, 10000.0, None, {0: 1.0, 12: 0.01, 23: 10000.0 ** (-46 / 48)})):
        scaling = None if sc is None else RopeScalingSpec("llama3", *sc)
        part = build_part("position", PositionSpec("rope", hd, hd, theta, scaling), {},
                          runtime(torch.float32))
        assert part.inv_freq.is_cuda and part.inv_freq.dtype == torch.float32
        table = part.inv_freq.cpu().double()
        assert table.numel() == hd // 2
        for j, value in pins.items():
            assert abs(table[j].item() / value - 1) < 1e-7, (hd, j, table[j].item(), value)


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_part_with_its_cache(dtype):
    """The mixer alone: a prompt portion, then another portion, against whole-sequence
    plain attention with the same weights."""
    from mstar_b200.config.layout import AttentionSpec, PositionSpec
    from mstar_b200.parts import LayerCache, build_part

    H, nh, nkv, hd, page = 80, 6, 2, 48, 4
    spec = AttentionSpec(hidden_size=H, num_heads=nh, num_kv_heads=nkv, head_dim=hd,
                         position=PositionSpec("rope", hd, hd, 10000.0))
    qkv = rnd((nh + 2 * nkv) * hd, H, dtype=dtype, seed=7, scale=0.15)
    o = rnd(H, nh * hd, dtype=dtype, seed=8, scale=0.1)
    attn = build_part("mixer", spec, {"qkv.weight": qkv, "o.weight": o}, runtime(dtype))
    x = rnd(23, H, dtype=dtype, seed=9)
    kv = torch.zeros(8, 2, nkv, page, hd, dtype=dtype, device=DEV)
    table = torch.tensor([[5, 1, 7, 2, 0, 6]], dtype=torch.int32, device=DEV)
    cache = LayerCache(kv=kv, page_size=page, block_table=table)
    first = attn.forward(x[:14].contiguous(), simple_ctx([14], [0]), cache)
    second = attn.forward(x[14:].contiguous(), simple_ctx([9], [14]), cache)
    got = torch.cat([first, second]).double().cpu()
    w = {"a.q_proj.weight": qkv[:nh * hd].cpu(), "a.k_proj.weight": qkv[nh * hd:(nh + nkv) * hd].cpu(),
         "a.v_proj.weight": qkv[(nh + nkv) * hd:].cpu(), "a.o_proj.weight": o.cpu()}
    cfg = dict(num_attention_heads=nh, num_key_value_heads=nkv, head_dim=hd, hidden_size=H,
               rope_theta=10000.0)
    want = P.plain_self_attention(x.cpu(), w, "a", cfg, torch.arange(23),
                                  P.plain_rope_frequencies(cfg))
    assert (got - want).abs().max() < (2e-5 if dtype == torch.float32 else 5e-2)


# ----------------------------------------------------------------- toy architecture
@dataclass(frozen=True)
class RunningMeanSpec:
    """Toy mixer: y_t = W . mean(x_0 .. x_t).  Its state is the running sum."""
    kind: str = "toy_running_mean"
    hidden_size: int = 0
    shares_kv: bool = False


class RunningMeanMixer:
    @classmethod
    def param_specs(cls, spec):
        from mstar_b200.weights.names import ParamSpec
        return {"w.weight": ParamSpec((spec.hidden_size, spec.hidden_size))}

    @classmethod
    def cache_need(cls, spec):
        from mstar_b200.parts import CacheNeed, StateNeed
        return CacheNeed(state=StateNeed(shape=(spec.hidden_size,), dtype="float32"))

    def __init__(self, spec, params, runtime):
        self.w = params["w.weight"]

    def forward(self, x, ctx, cache):
        out = torch.empty_like(x)
        xf, t0 = x.float(), 0
        for i, n in enumerate(ctx.q_lens):
            slot, before = ctx.host_slots[i], ctx.kv_lens[i] - n
            sums = torch.cumsum(xf[t0:t0 + n], 0) + cache.state[slot]
            cache.state[slot] = sums[-1]
            count = torch.arange(before + 1, before + n + 1, device=x.device)[:, None].float()
            out[t0:t0 + n] = ((sums / count) @ self.w.float().T).to(x.dtype)
            t0 += n
        return out


@dataclass(frozen=True)
class TopOneExpertsSpec:
    """Toy feed-forward with routing: a float router picks one of `experts` small
    relu(x W1) W2 experts per token; its output is weighted by the router's softmax."""
    kind: str = "toy_top1_experts"
    hidden_size: int = 0
    expert_size: int = 0
    experts: int = 0


class TopOneExperts:
    @classmethod
    def param_specs(cls, spec):
        from mstar_b200.weights.names import ParamSpec
        return {"router.weight": ParamSpec((spec.experts, spec.hidden_size)),
                "w1.weight": ParamSpec((spec.experts * spec.expert_size, spec.hidden_size)),
                "w2.weight": ParamSpec((spec.experts * spec.hidden_size, spec.expert_size))}

    def __init__(self, spec, params, runtime):
        self.spec = spec
        self.router, self.w1, self.w2 = (params[k] for k in ("router.weight", "w1.weight",
                                                             "w2.weight"))

    def forward(self, x, ctx):
        s = self.spec
        scores = torch.softmax(x.float() @ self.router.float().T, dim=-1)   # router in float
        weight, expert = scores.max(dim=-1)
        out = torch.zeros_like(x)
        for e in range(s.experts):
            rows = (expert == e).nonzero().flatten()
            if rows.numel() == 0:
                continue
            w1 = self.w1[e * s.expert_size:(e + 1) * s.expert_size].float()
            w2 = self.w2[e * s.hidden_size:(e + 1) * s.hidden_size].float()
            y = torch.relu(x[rows].float() @ w1.T) @ w2.T
            out[rows] = (weight[rows, None] * y).to(x.dtype)
        return out


@dataclass(frozen=True)
class QueryGrowthSpec:
    """Toy position encoding: no rotation; the query of position p is scaled by
    1 + rate * p (keys and values are written as they are)."""
    kind: str = "toy_query_growth"
    head_dim: int = 0
    rate: float = 0.0


class QueryGrowth:
    @classmethod
    def param_specs(cls, spec):
        return {}

    def __init__(self, spec, params, runtime):
        self.spec = spec

    def apply(self, qkv, ctx, kv_cache, block_table, page_size, num_heads, num_kv_heads):
        from mstar_b200 import ops
        nq = num_heads * self.spec.head_dim
        grow = 1.0 + self.spec.rate * ctx.positions.float()
        qkv[:, :nq] = (qkv[:, :nq].float() * grow[:, None]).to(qkv.dtype)
        ops.rope_kv_write(qkv, ctx.positions, ctx.cache_pos, ctx.token_req, block_table, None,
                          kv_cache, num_heads, num_kv_heads, self.spec.head_dim, 0, False,
                          page_size)


class ToyConfig:
    architecture = "ToyMixedForCausalLM"
    EXPERTS, EXPERT_SIZE, RATE = 3, 40, 0.02
    EMBED_MULT, LOGIT_SCALE, SOFTCAP = 1.5, 0.5, 4.0     # a scaled embedding, a capped head
    H, NH, NKV, HD, INTER, VOCAB, WINDOW, EPS = 64, 4, 2, 16, 96, 128, 8, 1e-5

    def to_dict(self):
        return {"architectures": [self.architecture]}

    @classmethod
    def from_dict(cls, raw):
        return cls()

    def stop_token_ids(self):
        return ()

    def layout(self):
        from mstar_b200.config.layout import (AttentionSpec, BlockSpec, EmbeddingSpec,
                                              GatedMLPSpec, HeadSpec, ModelLayout, NormSpec,
                                              PositionSpec, RunEntry)
        pos = PositionSpec("rope", self.HD, self.HD, 10000.0)
        norm = NormSpec(size=self.H, eps=self.EPS)
        ffn = GatedMLPSpec(hidden_size=self.H, intermediate_size=self.INTER)

        def attn(**kw):
            return AttentionSpec(hidden_size=self.H, num_heads=self.NH, num_kv_heads=self.NKV,
                                 head_dim=self.HD, position=pos, **kw)

        routed = TopOneExpertsSpec(hidden_size=self.H, expert_size=self.EXPERT_SIZE,
                                   experts=self.EXPERTS)
        grown = AttentionSpec(hidden_size=self.H, num_heads=self.NH, num_kv_heads=self.NKV,
                              head_dim=self.HD,
                              position=QueryGrowthSpec(head_dim=self.HD, rate=self.RATE))
        blocks = [BlockSpec("prenorm", attn(), ffn, norm, norm),
                  BlockSpec("prenorm", RunningMeanSpec(hidden_size=self.H), ffn, norm, norm),
                  BlockSpec("prenorm", attn(shares_kv=True), ffn, norm, norm),
                  BlockSpec("prenorm", attn(window=self.WINDOW), ffn, norm, norm),
                  BlockSpec("prenorm", grown, routed, norm, norm)]
        # block 2 reads the cache block 0 wrote; block 1 runs twice, with a state each time;
        # block 4 has a position encoding and a routed feed-forward of the test's own
        order = [RunEntry(0, 0), RunEntry(1, 1), RunEntry(2, 0), RunEntry(3, 2), RunEntry(1, 3),
                 RunEntry(4, 4)]
        return ModelLayout(vocab_size=self.VOCAB, hidden_size=self.H, blocks=blocks, order=order,
                           final_norm=norm, tie_word_embeddings=True,
                           embedding=EmbeddingSpec(vocab_size=self.VOCAB, hidden_size=self.H,
                                                   multiplier=self.EMBED_MULT),
                           head=HeadSpec(vocab_size=self.VOCAB, hidden_size=self.H,
                                         logit_scale=self.LOGIT_SCALE, softcap=self.SOFTCAP))


def toy_checkpoint_map(config, layout):
    from mstar_b200.engine.model import model_param_specs
    from mstar_b200.weights.names import CheckpointMap, TensorSource

    sources = [TensorSource("toy." + name, name, 0, spec.shape[0])
               for name, spec in model_param_specs(layout).items()]
    return CheckpointMap(sources=sources, aliases={"head.weight": "embed.weight"},
                         optional=frozenset({"toy.head.weight"}))


def toy_plain_logits(w, cfg: ToyConfig, ids, margins=None):
    """Whole-sequence plain forward of the toy model, from the plain part functions.
    ``margins``: a list that receives, per token, the gap between the router's two largest
    logits in the routed feed-forward (a choice inside rounding noise is not a fault)."""
    T = len(ids)
    pos = torch.arange(T)
    rope_cfg = dict(head_dim=cfg.HD, rope_theta=10000.0, hidden_size=cfg.H,
                    num_attention_heads=cfg.NH)
    inv = P.plain_rope_frequencies(rope_cfg)
    h = w["toy.embed.weight"].double()[torch.tensor(ids)] * cfg.EMBED_MULT
    kv_of_cache = {}

    def heads(x, mat, n):
        return (x @ mat.double().T).view(T, n, cfg.HD)

    for block, cache in ((0, 0), (1, 1), (2, 0), (3, 2), (1, 3), (4, 4)):
        p = f"toy.blocks.{block}"
        x = P.plain_rms_norm(h, w[f"{p}.norm1.weight"], cfg.EPS)
        if block == 1:
            mean = torch.cumsum(x, 0) / torch.arange(1, T + 1)[:, None]
            a = mean @ w[f"{p}.mixer.w.weight"].double().T
        else:
            nq = cfg.NH * cfg.HD
            if block == 2:
                q = P.plain_apply_rope(heads(x, w[f"{p}.mixer.q.weight"], cfg.NH), pos, inv)
                k, v = kv_of_cache[cache]
            else:
                qkv = w[f"{p}.mixer.qkv.weight"]
                nk = cfg.NKV * cfg.HD
                if block == 4:          # the toy position encoding: queries grow with p
                    q = heads(x, qkv[:nq], cfg.NH) * (1 + cfg.RATE * pos.double())[:, None, None]
                    k = heads(x, qkv[nq:nq + nk], cfg.NKV)
                else:
                    q = P.plain_apply_rope(heads(x, qkv[:nq], cfg.NH), pos, inv)
                    k = P.plain_apply_rope(heads(x, qkv[nq:nq + nk], cfg.NKV), pos, inv)
                v = heads(x, qkv[nq + nk:], cfg.NKV)
                kv_of_cache[cache] = (k, v)
            att = P.plain_attention(q, k, v, window=cfg.WINDOW if block == 3 else None)
            a = att.reshape(T, nq) @ w[f"{p}.mixer.o.weight"].double().T
        h = h + a
        y = P.plain_rms_norm(h, w[f"{p}.norm2.weight"], cfg.EPS)
        if block == 4:                  # the toy routed feed-forward
            router_logits = y @ w[f"{p}.ffn.router.weight"].double().T
            scores = torch.softmax(router_logits, dim=-1)
            weight, expert = scores.max(dim=-1)
            if margins is not None:
                best2 = torch.topk(router_logits, 2, dim=-1).values
                margins.extend((best2[:, 0] - best2[:, 1]).tolist())
            m = torch.zeros_like(y)
            for t in range(T):
                e = int(expert[t])
                w1 = w[f"{p}.ffn.w1.weight"].double()[e * cfg.EXPERT_SIZE:(e + 1) * cfg.EXPERT_SIZE]
                w2 = w[f"{p}.ffn.w2.weight"].double()[e * cfg.H:(e + 1) * cfg.H]
                m[t] = weight[t] * (torch.relu(y[t] @ w1.T) @ w2.T)
            h = h + m
            continue
        gu = w[f"{p}.ffn.gate_up.weight"]
        h = h + P.plain_swiglu(y, gu[:cfg.INTER], gu[cfg.INTER:], w[f"{p}.ffn.down.weight"])
    logits = P.plain_rms_norm(h, w["toy.final_norm.weight"], cfg.EPS) @ w["toy.embed.weight"].double().T
    return cfg.SOFTCAP * torch.tanh(logits * cfg.LOGIT_SCALE / cfg.SOFTCAP)


@pytest.fixture
def toy_registered():
    from mstar_b200.config.registry import register_architecture, unregister_architecture
    from mstar_b200.parts import register_part, unregister_part

    register_part("mixer", "toy_running_mean", RunningMeanMixer)
    register_part("ffn", "toy_top1_experts", TopOneExperts)
    register_part("position", "toy_query_growth", QueryGrowth)
    register_architecture("ToyMixedForCausalLM", ToyConfig, toy_checkpoint_map)
    yield
    unregister_architecture("ToyMixedForCausalLM")
    unregister_part("mixer", "toy_running_mean")
    unregister_part("ffn", "toy_top1_experts")
    unregister_part("position", "toy_query_growth")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_architecture_is_registered_built_and_stepped(toy_registered, dtype):
    import helpers as H
    from mstar_b200.cache.storage import plan_groups
    from mstar_b200.engine.model import load_model, model_param_specs
    from mstar_b200.engine.step import make_stepper

    cfg = ToyConfig()
    layout = cfg.layout()
    g = torch.Generator().manual_seed(5)
    tensors = {}
    for name, spec in model_param_specs(layout).items():
        if name == "head.weight":
            continue
        if spec.init == "ones":
            t = 1 + 0.1 * torch.randn(spec.shape, generator=g)
        else:
            t = 0.05 * torch.randn(spec.shape, generator=g)
            if ".ffn.router" in name:
                t *= 40            # a router that decides: few tokens near a tie
            if ".mixer.q" in name:
                t[:cfg.NH * cfg.HD + (0 if name.endswith("q.weight") else cfg.NKV * cfg.HD)] *= 3
        tensors["toy." + name] = t.to(torch.bfloat16)
    model = load_model(None, dtype=dtype, device=DEV, config=cfg, tensors=tensors)
    # two page groups (all keys / window of 8) and two state caches
    windows, group_of = plan_groups(model.cache_needs)
    assert windows == [None, 8] and group_of == [0, None, 1, None, 0]
    assert [n.state is not None for n in model.cache_needs] == [False, True, False, True, False]

    reqs = {f"t{i}": H.request_tokens(cfg.VOCAB, n, seed=40 + i) for i, n in enumerate([3, 21, 50, 77])}
    # the routed feed-forward sits in the last block, so a token whose two best experts are
    # within rounding noise of each other differs in its own logits only: those are left out
    want, close = {}, 0
    noise = 1e-4 if dtype == "float32" else 0.3       # of router logits as large as 20
    for rid, toks in reqs.items():
        margins = []
        logits = toy_plain_logits(tensors, cfg, toks, margins)
        for i in range(len(toks)):
            if margins[i] < noise:
                close += 1
            else:
                want[(rid, i)] = logits[i]
    assert close <= 0.1 * sum(len(t) for t in reqs.values())
    # the group of windowed layers has pages of its own size (2 tokens) in the last two runs
    for steps, what, page1 in ((H.whole(reqs), "toy whole", 4), (H.portions(reqs), "toy portions", 4),
                               (H.prefill_then_decode(reqs, 32), "toy prefill + decode", 2),
                               (H.mixed(reqs, seed=2), "toy mixed", 2)):
        pages = [H.max_tokens_of(steps, 4) // 4, H.max_tokens_of(steps, page1) // page1]
        stepper = make_stepper(model, page_size=[4, page1], num_pages=pages, num_slots=4)
        assert stepper.storage.state_bytes_per_request() == 2 * cfg.H * 4
        assert not stepper.cuda_graphs        # the toy parts do not say that they may be captured
        got = H.run_steps_in_process(stepper, steps)
        H.compare({k: v for k, v in got.items() if k in want}, want, dtype, what)
        mgr = stepper.manager
        assert mgr.check() == 0 and mgr.free_pages(0) == pages[0] and mgr.free_pages(1) == pages[1]


def test_a_failed_step_leaves_state_and_lengths_as_they_were(toy_registered):
    """Mixers update their per-request state in place; a forward pass that fails after they
    did (here: the routed feed-forward of the last block raises) must leave the state, like
    the lengths, where the step found them, so that the same step can be run again."""
    import helpers as H
    from mstar_b200.engine.model import load_model, model_param_specs
    from mstar_b200.engine.step import StepEntry, make_stepper

    cfg = ToyConfig()
    g = torch.Generator().manual_seed(6)
    tensors = {"toy." + name: ((torch.ones(spec.shape) if spec.init == "ones"
                                else 0.05 * torch.randn(spec.shape, generator=g))).to(torch.bfloat16)
               for name, spec in model_param_specs(cfg.layout()).items() if name != "head.weight"}
    model = load_model(None, dtype="float32", device=DEV, config=cfg, tensors=tensors)
    toks = {r: H.request_tokens(cfg.VOCAB, 12, seed=60 + i) for i, r in enumerate("ab")}

    def run(fail_at_step):
        stepper = make_stepper(model, page_size=4, num_pages=16, num_slots=2)
        for r in toks:
            stepper.add_request(r)
        outs = []
        for step, (lo, hi) in enumerate(((0, 5), (5, 6), (6, 12))):
            entries = [StepEntry(r, toks[r][lo:hi], (hi - lo - 1,)) for r in toks]
            if step == fail_at_step:
                before = [s.clone() for s in stepper.storage.state if s is not None]
                real = TopOneExperts.forward
                TopOneExperts.forward = lambda *a, **k: (_ for _ in ()).throw(RuntimeError("boom"))
                try:
                    with pytest.raises(RuntimeError, match="boom"):
                        stepper.step(entries)
                finally:
                    TopOneExperts.forward = real
                after = [s for s in stepper.storage.state if s is not None]
                assert len(before) == 2 and all(torch.equal(x, y) for x, y in zip(before, after))
                assert [stepper.manager.length(r) for r in toks] == [lo, lo]
            outs.append(stepper.step(entries).clone())
        return outs

    clean = run(None)
    for fail_at in (0, 1, 2):
        for x, y in zip(clean, run(fail_at)):
            assert torch.equal(x, y)


def test_llama_has_an_empty_state_slot(model_folders):
    from mstar_b200.engine.model import load_model
    from mstar_b200.engine.step import make_stepper

    model = load_model(model_folders["tiny_a"][0], dtype="float32", device=DEV)
    stepper = make_stepper(model, page_size=4, num_pages=4, num_slots=3)
    assert stepper.storage.state_bytes_per_request() == 0
    assert stepper.add_request("x") == 0 and stepper.manager.free_slots() == 2
