"""Plain, slow implementation of the Llama decoder used as the oracle of the tests.

Whole sequences, no cache, no batching, one function for each part, float64
arithmetic unless the reference fixes a narrower type (RoPE angles are formed in
float32).  It runs where its weights lie: on the CPU in nearly all tests; the tests
at the real layer sizes hand it weights on the GPU, where the same torch float64
operations are fast enough for thousands of tokens.  It shares no code with ``redline_b200``: it has its own
reading of ``config.json``, its own weight generator, its own safetensors writer.

Every function cites the place in the reference project (Neil456/Redline, paths
relative to that project) whose formula it restates.  ``tests/golden`` holds
logits of the reference's own CPU model for two tiny random models;
``tests/test_plain.py`` checks this file against them, so this file does not
rest on the formulas alone.
"""

from __future__ import annotations

import json
import math
import os
import struct
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

F64 = torch.float64

# When set to a 16-bit type, every tensor that a 16-bit engine stores in that type
# (outputs of norms, projections, the rotation, attention and the gated product; the
# cached keys and values) is rounded to it here as well, while all arithmetic stays in
# double precision and the residual stream and the logits stay unrounded.  With it the
# oracle differs from a 16-bit engine only by the order of its sums.
STORE_DTYPE: Optional[torch.dtype] = None


def stored(x: torch.Tensor) -> torch.Tensor:
    return x if STORE_DTYPE is None else x.to(STORE_DTYPE).to(F64)


# --------------------------------------------------------------------------
# configuration (python/redline/convert.py:86-150, src/core/model_config.cpp:25-59)
# --------------------------------------------------------------------------


@dataclass
class PlainConfig:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_layers: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    rms_norm_eps: float
    rope_theta: float
    rope_scaling: Optional[dict]
    tie_word_embeddings: bool
    max_position_embeddings: int
    # The reference model has neither; they exist so that tests of the
    # framework's general parts (a window, a layer order) have an oracle.
    sliding_window: int = 0
    layer_order: Optional[List[Tuple[int, int]]] = None  # (layer, cache owner call)


def plain_config(cfg: dict) -> PlainConfig:
    """HF ``config.json`` keys and defaults as python/redline/convert.py:108-150."""
    params = cfg.get("rope_parameters") or {}
    scaling = cfg.get("rope_scaling") or params or None
    theta = cfg.get("rope_theta", params.get("rope_theta", 10000.0))
    rs = None
    if scaling:
        rtype = scaling.get("rope_type", scaling.get("type", "default"))
        if rtype == "linear":
            rs = {"type": "linear", "factor": float(scaling["factor"])}
        elif rtype == "llama3":
            rs = {
                "type": "llama3",
                "factor": float(scaling["factor"]),
                "low_freq_factor": float(scaling.get("low_freq_factor", 1.0)),
                "high_freq_factor": float(scaling.get("high_freq_factor", 4.0)),
                "original_max_position_embeddings": int(
                    scaling.get("original_max_position_embeddings", 8192)),
            }
        elif rtype not in ("default", None):
            raise NotImplementedError(rtype)
    heads = cfg["num_attention_heads"]
    return PlainConfig(
        vocab_size=cfg["vocab_size"],
        hidden_size=cfg["hidden_size"],
        intermediate_size=cfg["intermediate_size"],
        num_layers=cfg["num_hidden_layers"],
        num_heads=heads,
        num_kv_heads=cfg.get("num_key_value_heads") or heads,
        head_dim=cfg.get("head_dim") or cfg["hidden_size"] // heads,
        rms_norm_eps=cfg.get("rms_norm_eps", 1e-5),
        rope_theta=float(theta),
        rope_scaling=rs,
        tie_word_embeddings=bool(cfg.get("tie_word_embeddings", False)),
        max_position_embeddings=cfg.get("max_position_embeddings", 4096),
    )


# --------------------------------------------------------------------------
# position encoding (src/core/model_config.cpp:126-169)
# --------------------------------------------------------------------------


def rope_inv_freq(head_dim: int, theta: float, scaling: Optional[dict]) -> List[float]:
    """Inverse frequencies in double precision, src/core/model_config.cpp:126-152."""
    half = head_dim // 2
    inv = [1.0 / (theta ** ((2.0 * i) / head_dim)) for i in range(half)]
    if scaling is None:
        return inv
    if scaling["type"] == "linear":
        return [f / scaling["factor"] for f in inv]
    assert scaling["type"] == "llama3"
    old_ctx = float(scaling["original_max_position_embeddings"])
    low, high, factor = scaling["low_freq_factor"], scaling["high_freq_factor"], scaling["factor"]
    low_freq_wavelen = old_ctx / low
    high_freq_wavelen = old_ctx / high
    out = []
    for f in inv:
        wavelen = 2.0 * math.pi / f
        if wavelen < high_freq_wavelen:
            out.append(f)
        elif wavelen > low_freq_wavelen:
            out.append(f / factor)
        else:
            smooth = (old_ctx / wavelen - low) / (high - low)
            out.append((1.0 - smooth) * f / factor + smooth * f)
    return out


def rope_tables(cfg: PlainConfig, num_pos: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """cos/sin [num_pos, D/2]; the angle is float32(pos) * float32(inv_freq), formed
    in float32 (src/core/model_config.cpp:155-169)."""
    inv = np.asarray(rope_inv_freq(cfg.head_dim, cfg.rope_theta, cfg.rope_scaling), dtype=np.float64)
    inv32 = inv.astype(np.float32)
    pos32 = np.arange(num_pos, dtype=np.float32)
    angle = (pos32[:, None] * inv32[None, :]).astype(np.float32)
    ang64 = angle.astype(np.float64)
    return torch.from_numpy(np.cos(ang64)), torch.from_numpy(np.sin(ang64))


def rope_rotate(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotate-half on [T, heads, D]: pairs (i, i + D/2), src/cpu/reference_model.cpp:174-183."""
    half = x.shape[-1] // 2
    x0, x1 = x[..., :half], x[..., half:]
    c, s = cos[:, None, :], sin[:, None, :]
    return stored(torch.cat([x0 * c - x1 * s, x1 * c + x0 * s], dim=-1))


# --------------------------------------------------------------------------
# parts
# --------------------------------------------------------------------------


def embedding(ids: Sequence[int], table: torch.Tensor) -> torch.Tensor:
    """Pure row gather, no scaling (src/cpu/reference_model.cpp:165-168)."""
    return table[torch.as_tensor(list(ids), dtype=torch.long, device=table.device)].to(F64)


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """y = x * rsqrt(mean(x^2) + eps) * w (src/cpu/reference_model.cpp:145-155)."""
    x = x.to(F64)
    inv = 1.0 / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return stored(x * inv * w.to(F64))


def linear(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y = x W^T (+ b), W stored [out, in] (src/cpu/reference_model.cpp:132-143)."""
    y = x.to(F64) @ w.to(F64).T
    if b is not None:
        y = stored(y) + b.to(F64)
    return stored(y)


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                     window: int = 0) -> torch.Tensor:
    """Grouped-query causal attention over a whole sequence.

    q [T, Hq, D], k and v [T, Hkv, D]; query head h reads kv head h // (Hq / Hkv);
    scores (q.k) * scale for keys j <= t, softmax with the maximum taken off,
    weighted sum of v (src/cpu/reference_model.cpp:191-218).  ``window`` > 0 keeps
    only keys with t - j < window (not in the reference).
    """
    T, Hq, D = q.shape
    Hkv = k.shape[1]
    G = Hq // Hkv
    out = torch.zeros(T, Hq, D, dtype=F64, device=q.device)
    for h in range(Hq):
        kh = h // G
        s = (q[:, h, :] @ k[:, kh, :].T) * scale  # [T, T]
        idx = torch.arange(T, device=q.device)
        mask = idx[None, :] > idx[:, None]
        if window > 0:
            mask = mask | (idx[:, None] - idx[None, :] >= window)
        s = s.masked_fill(mask, float("-inf"))
        s = s - s.max(dim=-1, keepdim=True).values
        p = torch.exp(s)
        p = p / p.sum(dim=-1, keepdim=True)
        out[:, h, :] = p @ v[:, kh, :]
    return stored(out)


def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """silu(g) * u with silu(g) = g / (1 + exp(-g)) (src/cpu/reference_model.cpp:222-229)."""
    return stored(gate / (1.0 + torch.exp(-gate)) * up)


# --------------------------------------------------------------------------
# the whole model (src/cpu/reference_model.cpp:157-238)
# --------------------------------------------------------------------------


def attention_block(cfg: PlainConfig, w: Dict[str, torch.Tensor], layer: int, x: torch.Tensor,
                    cos: torch.Tensor, sin: torch.Tensor,
                    kv_from: Optional[Tuple[torch.Tensor, torch.Tensor]] = None):
    """Projections, RoPE on q and k (not v), attention, output projection
    (src/cpu/reference_model.cpp:170-220).  Returns (output, (k, v))."""
    p = f"model.layers.{layer}.self_attn."
    T = x.shape[0]
    q = linear(x, w[p + "q_proj.weight"], w.get(p + "q_proj.bias")).view(T, cfg.num_heads, cfg.head_dim)
    q = rope_rotate(q, cos, sin)
    if kv_from is None:
        k = linear(x, w[p + "k_proj.weight"], w.get(p + "k_proj.bias")).view(T, cfg.num_kv_heads, cfg.head_dim)
        v = linear(x, w[p + "v_proj.weight"], w.get(p + "v_proj.bias")).view(T, cfg.num_kv_heads, cfg.head_dim)
        k = rope_rotate(k, cos, sin)
    else:
        k, v = kv_from
    scale = 1.0 / math.sqrt(cfg.head_dim)
    a = causal_attention(q, k, v, scale, cfg.sliding_window)
    return linear(a.reshape(T, -1), w[p + "o_proj.weight"]), (k, v)


def mlp_block(cfg: PlainConfig, w: Dict[str, torch.Tensor], layer: int, x: torch.Tensor) -> torch.Tensor:
    """down(silu(gate(x)) * up(x)) (src/cpu/reference_model.cpp:222-232)."""
    p = f"model.layers.{layer}.mlp."
    g = linear(x, w[p + "gate_proj.weight"])
    u = linear(x, w[p + "up_proj.weight"])
    return linear(swiglu(g, u), w[p + "down_proj.weight"])


def hidden_states(cfg: PlainConfig, w: Dict[str, torch.Tensor], tokens: Sequence[int]) -> torch.Tensor:
    """Embedding and the layer loop with pre-norm residual blocks; the result is
    the residual stream before the final norm (src/cpu/reference_model.cpp:157-233)."""
    T = len(tokens)
    h = embedding(tokens, w["model.embed_tokens.weight"])
    cos, sin = (t.to(h.device) for t in rope_tables(cfg, T))
    order = cfg.layer_order or [(i, -1) for i in range(cfg.num_layers)]
    kv_of_call: List[Tuple[torch.Tensor, torch.Tensor]] = []
    for layer, kv_owner in order:
        p = f"model.layers.{layer}."
        xn = rmsnorm(h, w[p + "input_layernorm.weight"], cfg.rms_norm_eps)
        a, kv = attention_block(cfg, w, layer, xn, cos, sin,
                                kv_of_call[kv_owner] if kv_owner >= 0 else None)
        kv_of_call.append(kv)
        h = h + a
        xn = rmsnorm(h, w[p + "post_attention_layernorm.weight"], cfg.rms_norm_eps)
        h = h + mlp_block(cfg, w, layer, xn)
    return h


def forward(cfg: PlainConfig, w: Dict[str, torch.Tensor], tokens: Sequence[int]) -> torch.Tensor:
    """Logits [T, V] in float64: final norm, then the head, which is the embedding
    table when the file has no ``lm_head.weight`` (src/cpu/reference_model.cpp:120-127,234-237)."""
    h = hidden_states(cfg, w, tokens)
    xn = rmsnorm(h, w["model.norm.weight"], cfg.rms_norm_eps)
    head = w["lm_head.weight"] if "lm_head.weight" in w else w["model.embed_tokens.weight"]
    return xn.to(F64) @ head.to(F64).T


def greedy_generate(cfg: PlainConfig, w: Dict[str, torch.Tensor], prompt: Sequence[int], n: int) -> List[int]:
    """Full recompute per token, argmax with the smaller index on ties
    (src/cpu/reference_model.cpp:240-252)."""
    seq = list(prompt)
    out = []
    for _ in range(n):
        last = forward(cfg, w, seq)[-1]
        nxt = int(torch.argmax(last))
        out.append(nxt)
        seq.append(nxt)
    return out


# --------------------------------------------------------------------------
# sampling (src/cuda/kernels/sampling.cu:53-203, src/cuda/kernels/common.cuh:112-140)
# --------------------------------------------------------------------------


def warped_distribution(logits: np.ndarray, temperature: float, top_k: int, top_p: float) -> np.ndarray:
    """The distribution a non-greedy row is drawn from: temperature, then top-k
    (ties at the k-th value kept), then top-p over what top-k kept: the smallest
    set of largest logits whose mass reaches top_p (ties at the threshold kept)
    (src/cuda/kernels/sampling.cu:129-171; order as tests/cuda/test_sampling.cu:53)."""
    l = logits.astype(np.float64)
    V = l.shape[0]
    keep = np.ones(V, dtype=bool)
    if 0 < top_k < V:
        kth = np.sort(l)[::-1][top_k - 1]
        keep &= l >= kth
    z = np.where(keep, np.exp((l - l.max()) / temperature), 0.0)
    if top_p < 1.0:
        order = np.argsort(-l, kind="stable")
        total = z.sum()
        cum = 0.0
        thr = None
        for i in order:
            if not keep[i]:
                continue
            cum += z[i]
            if cum >= top_p * total:
                thr = l[i]
                break
        if thr is not None:
            keep &= l >= thr
        z = np.where(keep, z, 0.0)
    return z / z.sum()


def _mulhilo(a: int, b: int) -> Tuple[int, int]:
    p = a * b
    return (p >> 32) & 0xFFFFFFFF, p & 0xFFFFFFFF


def philox4x32_10(ctr: Tuple[int, int, int, int], key: Tuple[int, int]) -> Tuple[int, int, int, int]:
    """Philox4x32-10 (src/cuda/kernels/common.cuh:112-125)."""
    M0, M1, W0, W1 = 0xD2511F53, 0xCD9E8D57, 0x9E3779B9, 0xBB67AE85
    x, y, z, w = ctr
    k0, k1 = key
    for _ in range(10):
        hi0, lo0 = _mulhilo(M0, x)
        hi1, lo1 = _mulhilo(M1, z)
        x, y, z, w = (hi1 ^ y ^ k0) & 0xFFFFFFFF, lo1, (hi0 ^ w ^ k1) & 0xFFFFFFFF, lo0
        k0 = (k0 + W0) & 0xFFFFFFFF
        k1 = (k1 + W1) & 0xFFFFFFFF
    return x, y, z, w


def uniform01(seed: int, position: int, stream: int, index: int) -> float:
    """Uniform in (0, 1) for (seed, position, stream, token index)
    (src/cuda/kernels/common.cuh:128-134)."""
    r = philox4x32_10((index, position, stream, 0x52444C4E), (seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF))
    return float(np.float32(np.float32(r[0] >> 8) + np.float32(0.5)) * np.float32(1.0 / 16777216.0))


def gumbel_draw(logits: np.ndarray, temperature: float, top_k: int, top_p: float, seed: int,
                position: int, stream: int = 0) -> int:
    """The token the reference draws: argmax over the kept set of
    (l - max) / T - log(-log(u_i)), u_i from Philox keyed by the seed with the
    position of the token being generated (src/cuda/kernels/sampling.cu:177-187)."""
    p = warped_distribution(logits, temperature, top_k, top_p)
    l = logits.astype(np.float64)
    best, best_i = -np.inf, None
    for i in np.nonzero(p > 0)[0]:
        u = uniform01(seed, position, stream, int(i))
        val = (l[i] - l.max()) / temperature - math.log(-math.log(u))
        if val > best:
            best, best_i = val, int(i)
    return best_i


# --------------------------------------------------------------------------
# test models: weights, folders
# --------------------------------------------------------------------------


def random_weights(cfg_json: dict, seed: int, sharpen: float = 1.0,
                   dtype: torch.dtype = torch.float32) -> Dict[str, torch.Tensor]:
    """Seeded weights by HF tensor name: matrices N(0, 0.02^2), norm weights
    1 + N(0, 0.1^2).  ``sharpen`` multiplies q_proj and k_proj so that attention
    is far from uniform (with 0.02-sized weights every score is about 0 and a
    fault in the choice of keys would not show).  Values are rounded to bfloat16
    so that every storage type holds the same numbers."""
    c = plain_config(cfg_json)
    g = torch.Generator().manual_seed(seed)

    def mat(n, k, s=0.02):
        return (torch.randn(n, k, generator=g) * s).to(torch.bfloat16).to(dtype)

    def norm(n):
        return (1.0 + 0.1 * torch.randn(n, generator=g)).to(torch.bfloat16).to(dtype)

    H, D, I = c.hidden_size, c.head_dim, c.intermediate_size
    w = {"model.embed_tokens.weight": mat(c.vocab_size, H)}
    for i in range(c.num_layers):
        p = f"model.layers.{i}."
        w[p + "input_layernorm.weight"] = norm(H)
        w[p + "self_attn.q_proj.weight"] = mat(c.num_heads * D, H, 0.02 * sharpen)
        w[p + "self_attn.k_proj.weight"] = mat(c.num_kv_heads * D, H, 0.02 * sharpen)
        w[p + "self_attn.v_proj.weight"] = mat(c.num_kv_heads * D, H)
        w[p + "self_attn.o_proj.weight"] = mat(H, c.num_heads * D)
        w[p + "post_attention_layernorm.weight"] = norm(H)
        w[p + "mlp.gate_proj.weight"] = mat(I, H)
        w[p + "mlp.up_proj.weight"] = mat(I, H)
        w[p + "mlp.down_proj.weight"] = mat(H, I)
    w["model.norm.weight"] = norm(H)
    if not c.tie_word_embeddings:
        w["lm_head.weight"] = mat(c.vocab_size, H)
    return w


_ST_NAME = {torch.float32: "F32", torch.bfloat16: "BF16", torch.float16: "F16", torch.int32: "I32"}


def write_safetensors(path: str, tensors: Dict[str, torch.Tensor], metadata: Optional[Dict[str, str]] = None):
    """A minimal safetensors writer of the tests' own: 8-byte little-endian header
    length, JSON header with dtype / shape / data_offsets, then the raw data."""
    header = {}
    if metadata:
        header["__metadata__"] = metadata
    blobs = []
    off = 0
    for name, t in tensors.items():
        t = t.contiguous()
        raw = t.view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _ST_NAME[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * ((8 - len(hj) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)


def write_model_dir(path: str, cfg_json: dict, weights: Dict[str, torch.Tensor]):
    """A model folder as HF lays it out: config.json and model.safetensors."""
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg_json, f, indent=1)
    write_safetensors(os.path.join(path, "model.safetensors"), weights, {"format": "pt"})
