"""Each part of a layer alone, against the plain function of the same name, at sizes of
its own; then parts put together in other ways than the architecture does: a layer
named twice, a layer reading another layer's cache, a window, no position encoding;
and a toy mixer with state of its own, a toy feed-forward with routing and a toy
position encoding, defined here, registered, built and stepped without a change to
the framework's files."""

import dataclasses
import math

import numpy as np
import pytest
import torch

import plain_llama as P
import tiny_configs as C
from gpu_utils import F32_REL, check_logits, make_model, oracle_logits, random_tokens, rel_max

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda")


def runtime(dtype=torch.float32, max_tokens=128):
    from redline_b200.parts.base import Runtime
    return Runtime(DEV, dtype, max_tokens, 4, 256, 16)


class Harness:
    """A cache manager, storage and batch builder for one attention-like part."""

    def __init__(self, cache_spec, dtype):
        from redline_b200.cache import CacheManager, GroupInfo
        from redline_b200.cache.storage import CacheStorage
        from redline_b200.engine.batch import BatchBuilder
        groups = [GroupInfo(cache_spec, [0])]
        self.cache = CacheManager(groups, [40], 16, 4)
        self.storage = CacheStorage(groups, [40], 16, dtype, DEV)
        self.builder = BatchBuilder(self.cache, 128, 4, 16, 256, DEV)

    def ctx(self, segs):
        from redline_b200.engine.batch import Segment
        out = []
        for key, start, n in segs:
            rc = self.cache.get(key) if self.cache.is_open(key) else self.cache.open(key)
            assert self.cache.reserve(rc, start + n)
            out.append(Segment(rc, [0] * n, start))
        return self.builder.build(out)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_embedding_head_mlp(dtype):
    from redline_b200.parts import PartSpec, build_part
    from redline_b200.parts.embedding import EmbeddingParams, HeadParams
    from redline_b200.parts.mlp import GatedMLPParams
    from redline_b200.parts.rmsnorm import RMSNormParams
    rt = runtime(dtype)
    tol = 1e-5 if dtype == torch.float32 else 1.5e-2
    H, I, V, T = 200, 328, 331, 23
    g = torch.Generator().manual_seed(0)
    r = lambda *s: torch.randn(*s, generator=g)  # noqa: E731
    # norm
    norm = build_part("norm", PartSpec("rmsnorm", RMSNormParams(H, 3e-6), {"weight": "n"}), rt)
    assert norm.tensors()["weight"].shape == (H,)
    wn = (1 + 0.1 * r(H)).to(dtype)
    norm.load({"weight": wn.to(DEV)})
    res, delta = r(T, H), r(T, H).to(dtype)
    out = torch.empty(T, H, device=DEV, dtype=dtype)
    res_d = res.to(DEV)
    norm.add_norm(res_d, delta.to(DEV), out)
    assert rel_max(out.double().cpu().numpy(), P.rmsnorm(res.double() + delta.double(), wn, 3e-6).numpy()) < tol
    # embedding
    harness = Harness(__import__("redline_b200.parts.spec", fromlist=["CacheSpec"]).CacheSpec.keys_values("full", 1, 16), dtype)
    emb = build_part("embedding", PartSpec("token_embedding", EmbeddingParams(V, H), {"weight": "e"}), rt)
    table = r(V, H).to(dtype)
    emb.load({"weight": table.to(DEV)})
    ctx = harness.ctx([("a", 0, T)])
    ids = torch.randint(0, V, (T,), generator=g, dtype=torch.int32)
    ctx.token_ids[:T].copy_(ids)
    stream = torch.empty(T, H, device=DEV)
    emb.forward(ctx, stream)
    assert torch.equal(stream.cpu(), P.embedding(ids.tolist(), table).float())
    # head, tied to the table and with a weight of its own
    head = build_part("head", PartSpec("lm_head", HeadParams(V, H, True), {"weight": "h"}), rt)
    head.load({})
    head.tie(emb.table())
    x = r(5, H).to(dtype)
    logits = torch.empty(8, V, device=DEV)
    head.forward(x.to(DEV), 5, logits)
    assert rel_max(logits[:5].double().cpu().numpy(), P.linear(x, table).numpy()) < (1e-5 if dtype == torch.float32 else 1e-3)
    # feed-forward
    mlp = build_part("ffn", PartSpec("swiglu_mlp", GatedMLPParams(H, I), {}), rt)
    wg, wu, wd = (r(I, H) * 0.1).to(dtype), (r(I, H) * 0.1).to(dtype), (r(H, I) * 0.1).to(dtype)
    mlp.load({"gate": wg.to(DEV), "up": wu.to(DEV), "down": wd.to(DEV)})
    xin = r(T, H).to(dtype)
    y = mlp.forward(xin.to(DEV), ctx)
    P.STORE_DTYPE = dtype if dtype == torch.bfloat16 else None
    try:
        want = P.linear(P.swiglu(P.linear(xin, wg), P.linear(xin, wu)), wd)
    finally:
        P.STORE_DTYPE = None
    assert rel_max(y.double().cpu().numpy(), want.numpy()) < tol


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("Hq,Hkv,D,window", [(5, 5, 48, 0), (6, 2, 32, 0), (4, 1, 64, 20)])
def test_attention_part_with_rotary_and_without(dtype, Hq, Hkv, D, window):
    from redline_b200.config.model_config import RopeScaling
    from redline_b200.parts import PartSpec, build_part
    from redline_b200.parts.attention import AttentionParams
    from redline_b200.parts.rope import RotaryParams
    H = 136
    for pos_kind in ("rope", "none"):
        rt = runtime(dtype)
        pos = PartSpec("rope", RotaryParams(D, 3e4, RopeScaling("linear", 1.5), 512)) if pos_kind == "rope" \
            else PartSpec("none")
        att = build_part("mixer", PartSpec("gqa_attention", AttentionParams(H, Hq, Hkv, D, pos, window=window), {}), rt)
        cs = att.cache_spec()
        assert (cs.kind, cs.window) == ("window" if window else "full", window)
        assert [(t.name, t.shape) for t in cs.tensors] == [("k", (Hkv, D)), ("v", (Hkv, D))]
        g = torch.Generator().manual_seed(1)
        w = {n: (torch.randn(s, generator=g) * 0.15).to(dtype) for n, s in
             {"q": (Hq * D, H), "k": (Hkv * D, H), "v": (Hkv * D, H), "o": (H, Hq * D)}.items()}
        assert {n: t.shape for n, t in att.tensors().items() if not t.optional} == {n: tuple(x.shape) for n, x in w.items()}
        att.load({n: x.to(DEV) for n, x in w.items()})
        hs = Harness(cs, dtype)
        cache = hs.storage.of_owner(0, True)
        T = 75
        x = torch.randn(T, H, generator=g).to(dtype)
        # run as 40 tokens, then 34, then 1 (prefill, prefill over a past, decode)
        outs = []
        for start, n in [(0, 40), (40, 34), (74, 1)]:
            ctx = hs.ctx([("s", start, n)])
            outs.append(att.forward(x[start:start + n].to(DEV), ctx, cache, None).clone())
        got = torch.cat(outs).double().cpu()
        P.STORE_DTYPE = dtype if dtype == torch.bfloat16 else None
        try:
            q = P.linear(x, w["q"]).view(T, Hq, D)
            k = P.linear(x, w["k"]).view(T, Hkv, D)
            v = P.linear(x, w["v"]).view(T, Hkv, D)
            if pos_kind == "rope":
                pc = P.PlainConfig(0, H, 0, 0, Hq, Hkv, D, 0, 3e4, {"type": "linear", "factor": 1.5}, False, 512)
                cos, sin = P.rope_tables(pc, T)
                q, k = P.rope_rotate(q, cos, sin), P.rope_rotate(k, cos, sin)
            a = P.causal_attention(q, k, v, 1 / math.sqrt(D), window)
            want = P.linear(a.reshape(T, -1), w["o"])
        finally:
            P.STORE_DTYPE = None
        assert rel_max(got.numpy(), want.numpy()) < (2e-5 if dtype == torch.float32 else 2e-2), pos_kind


def spec_with(cfg_json, **changes):
    """The architecture's spec with the attention parameters of every layer changed."""
    from redline_b200.config import config_from_dict, model_spec
    spec = model_spec(config_from_dict(cfg_json))
    layers = []
    for ls in spec.layers:
        mixer = dataclasses.replace(ls.mixer, params=dataclasses.replace(ls.mixer.params, **changes))
        layers.append(dataclasses.replace(ls, mixer=mixer))
    return dataclasses.replace(spec, layers=tuple(layers))


def engine_from_spec(model_dir, cfg_json, spec, dtype, **kw):
    from redline_b200.config import EngineConfig, config_from_dict
    from redline_b200.engine.engine import Engine
    from redline_b200.engine.runner import ModelRunner
    opts = dict(dtype=dtype, kv_cache_tokens=512, max_seq_len=512, max_num_seqs=4, max_num_batched_tokens=256,
                max_logit_rows=256, cuda_graphs=False, async_scheduling=False)
    opts.update(kw)
    cfg = EngineConfig.from_options(model_dir, opts)
    return Engine.from_runner(ModelRunner(cfg, config_from_dict(cfg_json), spec))


def replay_in_portions(eng, toks, key="x"):
    outs, i = [], 0
    for s in [33, 2, 1, 40, 1, 1, 17, 64, 64, 64]:
        s = min(s, len(toks) - i)
        if s <= 0:
            break
        outs.append(eng.step_tokens([(key, toks[i:i + s], list(range(s)))]).cpu().numpy())
        i += s
    eng.close_request(key)
    return np.concatenate(outs)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_layer_named_twice_and_a_layer_that_reads_another_layers_cache(dtype, tmp_path):
    from redline_b200.parts.spec import LayerCall
    # (bfloat16 noise grows with depth and with the sharpness of attention: four layer calls at
    # sharpness 6 reach 4e-2 of max |logit| from flipped roundings alone, so the 16-bit run uses 3)
    d, w = make_model(tmp_path, C.TINY_B, seed=50, sharpen=6.0 if dtype == "float32" else 3.0)
    base = spec_with(C.TINY_B)
    # layer 1 runs twice with caches of its own; the last call runs layer 2's weights on call 0's cache
    order = (LayerCall(0), LayerCall(1), LayerCall(1), LayerCall(2, cache_of=0))
    spec = dataclasses.replace(base, order=order)
    eng = engine_from_spec(d, C.TINY_B, spec, dtype)
    assert len(eng.runner.groups) == 1 and eng.runner.groups[0].owners == [0, 1, 2]
    toks = random_tokens(1000, 140, 1)
    got = replay_in_portions(eng, toks)
    pc = P.plain_config(C.TINY_B)
    pc.layer_order = [(0, -1), (1, -1), (1, -1), (2, 0)]
    check_logits(got, C.TINY_B, w, toks, dtype, pc=pc)
    with pytest.raises(ValueError, match="does not come before"):
        engine_from_spec(d, C.TINY_B, dataclasses.replace(base, order=(LayerCall(0, cache_of=1), LayerCall(1))), dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_window_layers_beside_full_layers_give_pages_back(dtype, tmp_path):
    """Layers 0 and 2 keep a window of 24 keys, layer 1 keeps all: two cache groups with
    pages of their own; the window group's pages come back while the request still runs."""
    d, w = make_model(tmp_path, C.TINY_B, seed=51, sharpen=6.0 if dtype == "float32" else 3.0)
    base = spec_with(C.TINY_B)
    layers = list(base.layers)
    for i in (0, 2):
        m = layers[i].mixer
        layers[i] = dataclasses.replace(layers[i], mixer=dataclasses.replace(m, params=dataclasses.replace(m.params, window=24)))
    eng = engine_from_spec(d, C.TINY_B, dataclasses.replace(base, layers=tuple(layers)), dtype, kv_cache_tokens=256)
    kinds = sorted((g.spec.kind, tuple(g.owners)) for g in eng.runner.groups)
    assert kinds == [("full", (1,)), ("window", (0, 2))]
    wg = [i for i, g in enumerate(eng.runner.groups) if g.spec.kind == "window"][0]
    toks = random_tokens(1000, 200, 2)
    outs, i, freed_early = [], 0, False
    for s in [33, 2, 1, 40, 1, 1, 17, 30, 30, 30, 15]:
        outs.append(eng.step_tokens([("x", toks[i:i + s], list(range(s)))]).cpu().numpy())
        i += s
        rc = eng.runner.cache.get("x")
        freed_early |= rc.released_upto[wg] > 0
        eng.runner.cache.check_invariants()
    assert i == 200 and freed_early and rc.released_upto[wg] == (200 - 24 + 1) // 16
    assert eng.runner.cache.num_free_pages(wg) > eng.runner.cache.num_free_pages(1 - wg)
    eng.close_request("x")

    # oracle: per-layer windows
    pc = P.plain_config(C.TINY_B)
    got = np.concatenate(outs)

    def forward_with_windows(tokens, rounded):
        P.STORE_DTYPE = rounded
        try:
            T = len(tokens)
            cos, sin = P.rope_tables(pc, T)
            h = P.embedding(tokens, w["model.embed_tokens.weight"])
            for layer in range(3):
                pc.sliding_window = 24 if layer in (0, 2) else 0
                p = f"model.layers.{layer}."
                a, _ = P.attention_block(pc, w, layer, P.rmsnorm(h, w[p + "input_layernorm.weight"], pc.rms_norm_eps), cos, sin)
                h = h + a
                h = h + P.mlp_block(pc, w, layer, P.rmsnorm(h, w[p + "post_attention_layernorm.weight"], pc.rms_norm_eps))
            xn = P.rmsnorm(h, w["model.norm.weight"], pc.rms_norm_eps)
            return (xn.double() @ w["model.embed_tokens.weight"].double().T).numpy()
        finally:
            P.STORE_DTYPE = None
            pc.sliding_window = 0

    ref = forward_with_windows(toks, torch.bfloat16 if dtype == "bfloat16" else None)
    assert rel_max(got, ref) < (F32_REL if dtype == "float32" else 3e-2)
    # and the window matters: the full-attention oracle differs
    assert rel_max(got, oracle_logits(C.TINY_B, w, toks)) > 1e-2
