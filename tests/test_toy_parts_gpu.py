"""Parts that are not the architecture's, defined in this file only: a mixer with state
of its own (a decaying sum, no cache), a feed-forward with routing (two experts, the
router's logits in float32) and a position encoding (a learned table added to q and k).
They are registered, built into a model beside an attention layer, loaded by tensor
name and stepped in portions through the engine, with no change to the framework's
files; the result is compared with a restatement in this file."""

import os
from dataclasses import dataclass

import numpy as np
import pytest
import torch

import plain_llama as P
from gpu_utils import rel_max

pytestmark = pytest.mark.gpu

H, V, HQ, HKV, D, I, E = 64, 97, 4, 2, 16, 48, 2
DECAY = 0.9


@dataclass(frozen=True)
class DecayParams:
    hidden: int
    decay: float


def register_toys():
    from redline_b200.parts import (FeedForward, Mixer, PositionEncoding, StateSpec, TensorSpec, register)

    @register("mixer", "toy_decay_sum")
    class DecaySum(Mixer):
        """s_t = decay * s_{t-1} + W x_t, y_t = s_t; s lives in the request's state slot."""

        def state_spec(self):
            return StateSpec((self.params.hidden,), "float32")

        def tensors(self):
            return {"w": TensorSpec((self.params.hidden, self.params.hidden))}

        def load(self, tensors):
            self.w = tensors["w"].float()

        def forward(self, x, ctx, cache, state):
            assert cache is None and state is not None
            out = torch.empty_like(x)
            z = x.float() @ self.w.T
            for start, n, slot in zip(ctx.host.q_start, ctx.host.q_len, ctx.host.state_slot):
                s = state[slot].clone()
                for t in range(start, start + n):
                    s = self.params.decay * s + z[t]
                    out[t] = s.to(x.dtype)
                state[slot] = s
            return out

    @register("ffn", "toy_routed")
    class Routed(FeedForward):
        """Each token goes to the expert whose router logit (float32) is larger."""

        def tensors(self):
            h, i, e = self.params
            return {"router": TensorSpec((e, h)), "up": TensorSpec((e, i, h)), "down": TensorSpec((e, h, i))}

        def load(self, tensors):
            self.router, self.up, self.down = (tensors[n].float() for n in ("router", "up", "down"))

        def forward(self, x, ctx):
            xf = x.float()
            choice = (xf @ self.router.T).argmax(-1)
            y = torch.zeros_like(xf)
            for e in range(self.params[2]):
                m = choice == e
                y[m] = torch.relu(xf[m] @ self.up[e].T) @ self.down[e].T
            return y.to(x.dtype)

    @register("position", "toy_learned")
    class Learned(PositionEncoding):
        """table[pos] is added to every q and k head (nothing is rotated)."""

        def __init__(self, spec, rt):
            super().__init__(spec, rt)
            g = torch.Generator().manual_seed(spec.params["seed"])
            self.table = (torch.randn(rt.max_seq_len, spec.params["head_dim"], generator=g) * 0.5).to(rt.device)

        def apply(self, qkv, num_heads, num_kv_heads, head_dim, ctx):
            T = ctx.T
            add = self.table[ctx.positions[:T].long()]
            v = qkv[:, :(num_heads + num_kv_heads) * head_dim].view(T, num_heads + num_kv_heads, head_dim)
            v.copy_((v.float() + add[:, None, :]).to(qkv.dtype))


def toy_spec():
    from redline_b200.parts import LayerCall, LayerSpec, ModelSpec, PartSpec
    from redline_b200.parts.attention import AttentionParams
    from redline_b200.parts.embedding import EmbeddingParams, HeadParams
    from redline_b200.parts.mlp import GatedMLPParams
    from redline_b200.parts.rmsnorm import RMSNormParams

    def norm(name):
        return PartSpec("rmsnorm", RMSNormParams(H, 1e-5), {"weight": name})

    l0 = LayerSpec("prenorm", norm("l0.n1"), PartSpec("toy_decay_sum", DecayParams(H, DECAY), {"w": "l0.mix.w"}),
                   norm("l0.n2"), PartSpec("toy_routed", (H, I, E), {"router": "l0.ffn.router", "up": "l0.ffn.up",
                                                                      "down": "l0.ffn.down"}))
    att = AttentionParams(H, HQ, HKV, D, PartSpec("toy_learned", {"seed": 5, "head_dim": D}))
    l1 = LayerSpec("prenorm", norm("l1.n1"), PartSpec("gqa_attention", att, {n: f"l1.att.{n}" for n in "qkvo"}),
                   norm("l1.n2"), PartSpec("swiglu_mlp", GatedMLPParams(H, I), {n: f"l1.mlp.{n}" for n in ("gate", "up", "down")}))
    return ModelSpec(H, V, 256, PartSpec("token_embedding", EmbeddingParams(V, H), {"weight": "emb"}),
                     (l0, l1), (LayerCall(0), LayerCall(1), LayerCall(0)), norm("fn"),
                     PartSpec("lm_head", HeadParams(V, H, False), {"weight": "head"}))


def toy_weights():
    g = torch.Generator().manual_seed(0)
    r = lambda *s: (torch.randn(*s, generator=g) * 0.2).to(torch.bfloat16).float()  # noqa: E731
    n = lambda: (1 + 0.1 * torch.randn(H, generator=g)).to(torch.bfloat16).float()  # noqa: E731
    return {"emb": r(V, H), "head": r(V, H), "fn": n(), "l0.n1": n(), "l0.n2": n(), "l1.n1": n(), "l1.n2": n(),
            "l0.mix.w": r(H, H), "l0.ffn.router": r(E, H) * 5, "l0.ffn.up": r(E, I, H), "l0.ffn.down": r(E, H, I),
            "l1.att.q": r(HQ * D, H) * 4, "l1.att.k": r(HKV * D, H) * 4, "l1.att.v": r(HKV * D, H), "l1.att.o": r(H, HQ * D),
            "l1.mlp.gate": r(I, H), "l1.mlp.up": r(I, H), "l1.mlp.down": r(H, I)}


def toy_oracle(w, toks, table):
    """float64 restatement; the decay layer is called twice, each call with a state of its own."""
    T = len(toks)
    h = w["emb"][toks].double()

    def decay_layer(h):
        z = P.rmsnorm(h, w["l0.n1"], 1e-5) @ w["l0.mix.w"].double().T
        s = torch.zeros(H, dtype=torch.float64)
        out = []
        for t in range(T):
            s = DECAY * s + z[t]
            out.append(s)
        h = h + torch.stack(out)
        x = P.rmsnorm(h, w["l0.n2"], 1e-5)
        choice = (x @ w["l0.ffn.router"].double().T).argmax(-1)
        y = torch.zeros_like(x)
        for e in range(E):
            m = choice == e
            y[m] = torch.relu(x[m] @ w["l0.ffn.up"][e].double().T) @ w["l0.ffn.down"][e].double().T
        return h + y

    h = decay_layer(h)
    x = P.rmsnorm(h, w["l1.n1"], 1e-5)
    add = table[:T].double()[:, None, :]
    q = P.linear(x, w["l1.att.q"]).view(T, HQ, D) + add
    k = P.linear(x, w["l1.att.k"]).view(T, HKV, D) + add
    v = P.linear(x, w["l1.att.v"]).view(T, HKV, D)
    h = h + P.linear(P.causal_attention(q, k, v, D ** -0.5).reshape(T, -1), w["l1.att.o"])
    x = P.rmsnorm(h, w["l1.n2"], 1e-5)
    h = h + P.linear(P.swiglu(P.linear(x, w["l1.mlp.gate"]), P.linear(x, w["l1.mlp.up"])), w["l1.mlp.down"])
    h = decay_layer(h)
    return (P.rmsnorm(h, w["fn"], 1e-5) @ w["head"].double().T).numpy()


def toy_engine(tmp_path, **options):
    """(engine, weights) of the toy model in float32; the model folder is written once per test."""
    from redline_b200.config import EngineConfig
    from redline_b200.config.model_config import ModelConfig
    from redline_b200.engine.engine import Engine
    from redline_b200.engine.runner import ModelRunner
    register_toys()
    w = toy_weights()
    d = str(tmp_path / "toy")
    if not os.path.isdir(d):
        os.makedirs(d)
        P.write_safetensors(os.path.join(d, "model.safetensors"), w)
    opts = dict(dtype="float32", kv_cache_tokens=256, max_seq_len=256, max_num_seqs=3, max_num_batched_tokens=128,
                max_logit_rows=128, cuda_graphs=False, async_scheduling=False)
    opts.update(options)
    runner = ModelRunner(EngineConfig.from_options(d, opts), ModelConfig("ToyForTests", V, H, 256, -1, ()), toy_spec())
    return Engine.from_runner(runner), w


def oracle_greedy(w, table, prompt, outputs):
    """Whether ``outputs`` are the arg max of the restatement's logits after every prefix."""
    seq = list(prompt) + list(outputs)
    ref = toy_oracle(w, seq[:-1], table)
    return [int(ref[len(prompt) - 1 + i].argmax()) for i in range(len(outputs))] == list(outputs)


def test_toy_parts_are_registered_built_loaded_and_stepped(tmp_path):
    eng, w = toy_engine(tmp_path)
    runner = eng.runner
    assert sorted(runner.states.pools) == [0, 2] and runner.states.pools[0].shape == (3, H)
    assert len(runner.groups) == 1 and runner.groups[0].owners == [1]
    table = runner.model.blocks[1].mixer.position.table.cpu()
    rng = np.random.RandomState(3)
    a, b = rng.randint(0, V, 90).tolist(), rng.randint(0, V, 61).tolist()
    ref_a, ref_b = toy_oracle(w, a, table), toy_oracle(w, b, table)
    whole = eng.step_tokens([("w", a, list(range(len(a))))]).cpu().numpy()
    eng.close_request("w")
    assert rel_max(whole, ref_a) < 1e-4
    # portions of a beside portions and single tokens of b; the state carries from step to step
    got = {"a": [], "b": []}
    ia = ib = 0
    for na, nb in [(33, 1), (2, 1), (1, 17), (40, 1), (14, 41)]:
        out = eng.step_tokens([("a", a[ia:ia + na], list(range(na))), ("b", b[ib:ib + nb], list(range(nb)))]).cpu().numpy()
        got["a"].append(out[:na]), got["b"].append(out[na:])
        ia, ib = ia + na, ib + nb
    assert ia == len(a) and ib == len(b)
    assert rel_max(np.concatenate(got["a"]), ref_a) < 1e-4 and rel_max(np.concatenate(got["b"]), ref_b) < 1e-4
    eng.close_request("a"), eng.close_request("b")
    # a slot that is handed out again starts from zero state
    again = eng.step_tokens([("c", b, [len(b) - 1])]).cpu().numpy()
    assert rel_max(again, ref_b[-1:]) < 1e-4
    eng.close_request("c")
    # and generation through the scheduler works with these parts too
    outs = eng.generate([a[:20], b[:9]], max_new_tokens=5, ignore_eos=True)
    assert oracle_greedy(w, table, a[:20], outs[0]["output_ids"])
    assert oracle_greedy(w, table, b[:9], outs[1]["output_ids"])


def test_state_keeping_mixer_with_cuda_graphs_asked_for(tmp_path):
    """With per-request state in the model the engine steps eagerly even when CUDA graphs are on (a
    graph's padding rows would share slot 0 with a live request, and capturing runs a step more than
    once): generation with graphs and asynchronous scheduling asked for gives the restatement's tokens."""
    eng, w = toy_engine(tmp_path, cuda_graphs=True, async_scheduling=True, max_num_seqs=4)
    table = eng.runner.model.blocks[1].mixer.position.table.cpu()
    rng = np.random.RandomState(11)
    prompts = [rng.randint(0, V, n).tolist() for n in (20, 9, 33, 14)]
    outs = eng.generate(prompts, max_new_tokens=12, ignore_eos=True)
    assert eng.runner.num_graph_steps == 0 and eng.runner.num_eager_steps > 0
    for p, o in zip(prompts, outs):
        assert oracle_greedy(w, table, p, o["output_ids"]), o["id"]


def test_state_keeping_mixer_under_recompute_preemption(tmp_path):
    """A pool of 160 tokens for four requests that grow to 70 each: the newest are preempted, their
    pages and state slots given back, and later recomputed from prompt + generated tokens.  A slot
    that is handed out again starts from zero, so the recomputed state is the restatement's."""
    eng, w = toy_engine(tmp_path, kv_cache_tokens=160, max_num_seqs=4, max_num_batched_tokens=64,
                        async_scheduling=True)
    table = eng.runner.model.blocks[1].mixer.position.table.cpu()
    rng = np.random.RandomState(12)
    prompts = [rng.randint(0, V, n).tolist() for n in (40, 38, 35, 30)]
    outs = eng.generate(prompts, max_new_tokens=30, ignore_eos=True)
    assert eng.num_preemptions > 0 and sum(o["num_preemptions"] for o in outs) > 0
    for p, o in zip(prompts, outs):
        assert len(o["output_ids"]) == 30 and oracle_greedy(w, table, p, o["output_ids"]), o["id"]
    assert eng.runner.cache.num_open() == 0
    eng.runner.cache.check_invariants()


# ---------------------------------------------------------------------------------------------
# A mixer whose cache is not keys and values: ONE latent vector per token.

Z = 24


def register_latent_toy():
    from redline_b200.parts import CacheSpec, CacheTensor, Mixer, TensorSpec, register

    @register("mixer", "toy_latent_mean")
    class LatentMean(Mixer):
        """z_t = W x_t is cached (one tensor "z" of Z numbers per token, no heads); y_t = U mean_{j <= t} z_j."""

        def cache_spec(self):
            return CacheSpec("full", (CacheTensor("z", (Z,)),))

        def tensors(self):
            return {"w": TensorSpec((Z, H)), "u": TensorSpec((H, Z))}

        def load(self, tensors):
            self.w, self.u = tensors["w"].float(), tensors["u"].float()

        def forward(self, x, ctx, cache, state):
            g = ctx.groups[cache.group]
            zc = cache.tensors["z"]                                    # [pages, page_size, Z]
            assert zc.shape[1:] == (self.rt.page_size, Z) and "k" not in cache.tensors
            T = ctx.T
            z = x.float() @ self.w.T
            flat = zc.view(-1, Z)
            flat[g.slots[:T].long()] = z.to(zc.dtype)
            out = torch.empty_like(x)
            for si, (start, n, p) in enumerate(zip(ctx.host.q_start, ctx.host.q_len, ctx.host.start_pos)):
                blocks = (p + n + self.rt.page_size - 1) // self.rt.page_size
                seen = zc[g.block_table[si, :blocks].long()].reshape(-1, Z)[:p + n].float()
                mean = seen.cumsum(0)[p:] / torch.arange(p + 1, p + n + 1, device=x.device)[:, None]
                out[start:start + n] = (mean @ self.u.T).to(x.dtype)
            return out


def latent_spec():
    from redline_b200.parts import LayerCall, LayerSpec, ModelSpec, PartSpec
    from redline_b200.parts.attention import AttentionParams
    from redline_b200.parts.embedding import EmbeddingParams, HeadParams
    from redline_b200.parts.mlp import GatedMLPParams
    from redline_b200.parts.rmsnorm import RMSNormParams
    from redline_b200.parts.rope import RotaryParams
    from redline_b200.config.model_config import RopeScaling

    def norm(name):
        return PartSpec("rmsnorm", RMSNormParams(H, 1e-5), {"weight": name})

    mlp = lambda i: PartSpec("swiglu_mlp", GatedMLPParams(H, I), {n: f"l{i}.mlp.{n}" for n in ("gate", "up", "down")})  # noqa: E731
    l0 = LayerSpec("prenorm", norm("l0.n1"), PartSpec("toy_latent_mean", None, {"w": "l0.mix.w", "u": "l0.mix.u"}),
                   norm("l0.n2"), mlp(0))
    att = AttentionParams(H, HQ, HKV, D, PartSpec("rope", RotaryParams(D, 1e4, RopeScaling(), 256)))
    l1 = LayerSpec("prenorm", norm("l1.n1"), PartSpec("gqa_attention", att, {n: f"l1.att.{n}" for n in "qkvo"}))   # no feed-forward
    return ModelSpec(H, V, 256, PartSpec("token_embedding", EmbeddingParams(V, H), {"weight": "emb"}),
                     (l0, l1), (LayerCall(0), LayerCall(1)), norm("fn"),
                     PartSpec("lm_head", HeadParams(V, H, True), {"weight": "head"}))


def latent_oracle(w, toks):
    T = len(toks)
    h = w["emb"][toks].double()
    z = P.rmsnorm(h, w["l0.n1"], 1e-5) @ w["l0.mix.w"].double().T
    mean = z.cumsum(0) / torch.arange(1, T + 1, dtype=torch.float64)[:, None]
    h = h + mean @ w["l0.mix.u"].double().T
    x = P.rmsnorm(h, w["l0.n2"], 1e-5)
    h = h + P.linear(P.swiglu(P.linear(x, w["l0.mlp.gate"]), P.linear(x, w["l0.mlp.up"])), w["l0.mlp.down"])
    x = P.rmsnorm(h, w["l1.n1"], 1e-5)
    pc = P.PlainConfig(V, H, I, 2, HQ, HKV, D, 1e-5, 1e4, None, True, 256)
    cos, sin = P.rope_tables(pc, T)
    q = P.rope_rotate(P.linear(x, w["l1.att.q"]).view(T, HQ, D), cos, sin)
    k = P.rope_rotate(P.linear(x, w["l1.att.k"]).view(T, HKV, D), cos, sin)
    v = P.linear(x, w["l1.att.v"]).view(T, HKV, D)
    h = h + P.linear(P.causal_attention(q, k, v, D ** -0.5).reshape(T, -1), w["l1.att.o"])     # the layer has no feed-forward
    return (P.rmsnorm(h, w["fn"], 1e-5) @ w["emb"].double().T).numpy()                         # tied head


def test_a_cache_that_is_not_keys_and_values_and_a_layer_without_a_feed_forward(tmp_path):
    """Two cache groups with tensors of different shapes in one model (a latent vector per token beside
    keys and values), each with pages and block tables of its own; a layer that has a mixer only; a head
    tied to the embedding.  Stepped in portions beside single tokens in a pool so small that pages are
    handed out again, against a restatement in float64."""
    from redline_b200.config import EngineConfig
    from redline_b200.config.model_config import ModelConfig
    from redline_b200.engine.engine import Engine
    from redline_b200.engine.runner import ModelRunner
    register_latent_toy()
    g = torch.Generator().manual_seed(7)
    r = lambda *s: (torch.randn(*s, generator=g) * 0.2).to(torch.bfloat16).float()  # noqa: E731
    n = lambda: (1 + 0.1 * torch.randn(H, generator=g)).to(torch.bfloat16).float()  # noqa: E731
    w = {"emb": r(V, H), "fn": n(), "l0.n1": n(), "l0.n2": n(), "l1.n1": n(), "l0.mix.w": r(Z, H), "l0.mix.u": r(H, Z),
         "l0.mlp.gate": r(I, H), "l0.mlp.up": r(I, H), "l0.mlp.down": r(H, I),
         "l1.att.q": r(HQ * D, H) * 4, "l1.att.k": r(HKV * D, H) * 4, "l1.att.v": r(HKV * D, H), "l1.att.o": r(H, HQ * D)}
    d = str(tmp_path / "latent")
    os.makedirs(d)
    P.write_safetensors(os.path.join(d, "model.safetensors"), w)
    cfg = EngineConfig.from_options(d, dict(dtype="float32", kv_cache_tokens=192, max_seq_len=160, max_num_seqs=3,
                                            max_num_batched_tokens=128, max_logit_rows=128, cuda_graphs=False,
                                            async_scheduling=False))
    runner = ModelRunner(cfg, ModelConfig("LatentToyForTests", V, H, 256, -1, ()), latent_spec())
    eng = Engine.from_runner(runner)
    assert [[(t.name, t.shape) for t in grp.spec.tensors] for grp in runner.groups] == \
        [[("z", (Z,))], [("k", (HKV, D)), ("v", (HKV, D))]]
    assert runner.model.blocks[1].ffn is None and runner.model.head.weight.data_ptr() == runner.model.embedding.weight.data_ptr()
    rng = np.random.RandomState(5)
    seqs = {k: rng.randint(0, V, n_).tolist() for k, n_ in (("a", 90), ("b", 61), ("c", 70))}
    refs = {k: latent_oracle(w, t) for k, t in seqs.items()}
    got = {k: [] for k in seqs}
    pos = {k: 0 for k in seqs}
    for step in [{"a": 33, "b": 1}, {"a": 2, "b": 1}, {"a": 1, "b": 17}, {"a": 40, "b": 1}, {"a": 14, "b": 41}]:
        out = eng.step_tokens([(k, seqs[k][pos[k]:pos[k] + m], list(range(m))) for k, m in step.items()]).cpu().numpy()
        at = 0
        for k, m in step.items():
            got[k].append(out[at:at + m])
            at += m
            pos[k] += m
    eng.close_request("a"), eng.close_request("b")
    out = eng.step_tokens([("c", seqs["c"], list(range(70)))]).cpu().numpy()       # on pages that a and b gave back
    got["c"].append(out)
    eng.close_request("c")
    for k in seqs:
        assert rel_max(np.concatenate(got[k]), refs[k]) < 1e-4, k
    runner.cache.check_invariants()
    assert runner.cache.num_open() == 0
