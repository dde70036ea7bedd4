"""Plain, slow implementation of Qwen3 dense: whole sequences, no cache, CPU.

It is the oracle of the test-suite.  One function for each part, written from
the formulas of the reference (each cites the reference's file:line); it shares
no code with the package: it reads config.json and model.safetensors by itself.
``tests/golden/`` holds logits of the reference's own model code for two tiny
models, made once on the CPU by ``tests/golden/make_golden.py``; the test
``test_plain.py`` checks this file against them.

All arithmetic is done in ``dtype`` (float32 by default) with the 32-bit inner
steps that the reference has; with ``dtype=torch.bfloat16`` the roundings fall
where the reference's bf16 service puts them, which gives the tests a measured
bf16-vs-fp32 distance to judge the engine's bf16 path by.
"""

from __future__ import annotations

import json
import math
import os

import torch
from safetensors import safe_open


# --------------------------------------------------------------------------- reading
def read_folder(folder: str) -> tuple[dict, dict[str, torch.Tensor]]:
    """config.json as a dict and every tensor of model.safetensors as float32."""
    with open(os.path.join(folder, "config.json"), "r", encoding="utf-8") as fh:
        cfg = json.load(fh)
    tensors: dict[str, torch.Tensor] = {}
    with safe_open(os.path.join(folder, "model.safetensors"), framework="pt", device="cpu") as fh:
        for name in fh.keys():
            tensors[name] = fh.get_tensor(name).to(torch.float32)
    return cfg, tensors


def sizes(cfg: dict) -> dict:
    """Sizes with the reference's defaults (acvram/engine/config.py:891-906, 177-179)."""
    heads = cfg.get("num_attention_heads", 32)
    hidden = cfg.get("hidden_size", 4096)
    return dict(
        L=cfg.get("num_hidden_layers", 32), H=hidden, NH=heads,
        NKV=cfg.get("num_key_value_heads", heads),
        D=cfg.get("head_dim", 0) or hidden // heads,
        I=cfg.get("intermediate_size", 11008), V=cfg.get("vocab_size", 32000),
        eps=cfg.get("rms_norm_eps", cfg.get("norm_epsilon", 1e-5)),
        theta=cfg.get("rope_theta", 10000.0),
        tied=bool(cfg.get("tie_word_embeddings", False)),
    )


# --------------------------------------------------------------------------- parts
def embed(table: torch.Tensor, ids: torch.Tensor, dtype) -> torch.Tensor:
    """x = E[token], cast to the model dtype (acvram/engine/model.py:161-164)."""
    return table[ids].to(dtype)


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """Variance, rsqrt and scaling in 32-bit; the normalised value is cast to the
    model dtype before the multiply by the weight, which is plain ``w``
    (acvram/engine/layers.py:625-630)."""
    dtype = x.dtype
    x32 = x.to(torch.float32)
    var = x32.pow(2).mean(-1, keepdim=True)
    x32 = x32 * torch.rsqrt(var + eps)
    return x32.to(dtype) * w.to(dtype)


def rotary_tables(positions: torch.Tensor, head_dim: int, theta: float) -> tuple[torch.Tensor, torch.Tensor]:
    """inv_freq[i] = 1/theta^(2i/D); angle = position * inv_freq; cos and sin of
    cat(angle, angle), all in 32-bit (acvram/engine/layers.py:727-730, 824-830).
    The tables stay float32 here, as the engine keeps them."""
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
    ang = torch.outer(positions.to(torch.float32), inv)
    emb = torch.cat((ang, ang), dim=-1)
    return emb.cos(), emb.sin()


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    """cat(-x[D/2:], x[:D/2]) (acvram/engine/layers.py:934-936)."""
    half = x.shape[-1] // 2
    return torch.cat((-x[..., half:], x[..., :half]), dim=-1)


def qk_norm_rotary(x: torch.Tensor, w: torch.Tensor, eps: float, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Per-head RMS norm over D, then the rotation, with one rounding at the end:
    a = v*inv*w in 32-bit, out = a*cos + rotate_half(a)*sin
    (fused kernel: acvram/kernels/acvram_kernels.cu:4397-4430; the order norm
    before rotation: acvram/engine/attention.py:353-359).  x: [T, heads, D]."""
    dtype = x.dtype
    x32 = x.to(torch.float32)
    inv = torch.rsqrt(x32.pow(2).mean(-1, keepdim=True) + eps)
    a = x32 * inv * w.to(torch.float32)
    out = a * cos[:, None, :] + rotate_half(a) * sin[:, None, :]
    return out.to(dtype)


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, window: int = 0) -> torch.Tensor:
    """q: [T, NH, D]; k, v: [T, NKV, D]; q-head h reads kv-head h // (NH/NKV)
    (acvram/engine/layers.py:1012-1017).  s = scale*q.k; key j is visible to the
    query at position i iff j <= i (acvram/engine/layers.py:1020-1041), and, with a
    window w > 0, j > i - w; softmax in 32-bit over the visible keys; o = p.v."""
    T, NH, D = q.shape
    rep = NH // k.shape[1]
    k32 = k.to(torch.float32).repeat_interleave(rep, dim=1)
    v32 = v.to(torch.float32).repeat_interleave(rep, dim=1)
    s = torch.einsum("qhd,khd->hqk", q.to(torch.float32), k32) * scale
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    hidden = j > i
    if window > 0:
        hidden = hidden | (j <= i - window)
    s = s.masked_fill(hidden[None], float("-inf"))
    p = torch.softmax(s, dim=-1)
    return torch.einsum("hqk,khd->qhd", p, v32).to(q.dtype)


def linear(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor | None = None) -> torch.Tensor:
    """y = x @ W^T (+ b), W is [out, in] (acvram/engine/layers.py:463-558).  A bias exists where the file holds a
    ``.bias`` tensor beside the weight (acvram/engine/loader.py:269-270); Qwen3's files hold none.  The product is
    rounded to the model dtype, then the bias is added in 32-bit and the sum rounded."""
    y = (x.to(torch.float32) @ w.to(torch.float32).T).to(x.dtype)
    if b is not None:
        y = (y.to(torch.float32) + b.to(torch.float32)).to(x.dtype)
    return y


def proj(x: torch.Tensor, t: dict, name: str) -> torch.Tensor:
    """The projection stored as ``name + "weight"`` (and ``name + "bias"`` when present)."""
    return linear(x, t[name + "weight"], t.get(name + "bias"))


def attention_block(h: torch.Tensor, t: dict, p: str, s: dict, positions: torch.Tensor, window: int = 0) -> torch.Tensor:
    """q/k/v projections, QK-norm, rotation, attention, o projection
    (acvram/engine/attention.py:290-365, 519-584)."""
    T = h.shape[0]
    q = proj(h, t, p + "self_attn.q_proj.").view(T, s["NH"], s["D"])
    k = proj(h, t, p + "self_attn.k_proj.").view(T, s["NKV"], s["D"])
    v = proj(h, t, p + "self_attn.v_proj.").view(T, s["NKV"], s["D"])
    cos, sin = rotary_tables(positions, s["D"], s["theta"])
    q = qk_norm_rotary(q, t[p + "self_attn.q_norm.weight"], s["eps"], cos, sin)
    k = qk_norm_rotary(k, t[p + "self_attn.k_norm.weight"], s["eps"], cos, sin)
    o = causal_attention(q, k, v, s["D"] ** -0.5, window)
    return proj(o.reshape(T, s["NH"] * s["D"]), t, p + "self_attn.o_proj.")


def swiglu_mlp(h: torch.Tensor, t: dict, p: str) -> torch.Tensor:
    """y = (silu(g) * u) @ Wd^T with silu(g) = g/(1+exp(-g)) in 32-bit, rounded to
    the model dtype before the product (acvram/engine/attention.py:745-761;
    kernel acvram/kernels/acvram_kernels.cu:8441-8452)."""
    g = proj(h, t, p + "mlp.gate_proj.")
    u = proj(h, t, p + "mlp.up_proj.")
    g32 = g.to(torch.float32)
    act = (g32 / (1.0 + torch.exp(-g32))).to(h.dtype)
    return proj(act * u, t, p + "mlp.down_proj.")


def residual_add(x: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
    """The sum is made in 32-bit and rounded once (acvram/engine/couches.py:427-443)."""
    return (x.to(torch.float32) + y.to(torch.float32)).to(x.dtype)


def decoder_layer(x: torch.Tensor, t: dict, i: int, s: dict, positions: torch.Tensor, window: int = 0) -> torch.Tensor:
    """Pre-norm block: x += Attn(RMS(x)); x += MLP(RMS(x)) (acvram/engine/couches.py:404-425)."""
    p = f"model.layers.{i}."
    h = rms_norm(x, t[p + "input_layernorm.weight"], s["eps"])
    x = residual_add(x, attention_block(h, t, p, s, positions, window))
    h = rms_norm(x, t[p + "post_attention_layernorm.weight"], s["eps"])
    return residual_add(x, swiglu_mlp(h, t, p))


def output_logits(x: torch.Tensor, t: dict, s: dict) -> torch.Tensor:
    """Final norm, then logits = float32(x) @ W^T in 32-bit; W is lm_head, or the
    embedding when tied (acvram/engine/model.py:211-221, 369-410;
    acvram/engine/loader.py:1138-1150)."""
    x = rms_norm(x, t["model.norm.weight"], s["eps"])
    w = t["model.embed_tokens.weight"] if s["tied"] or "lm_head.weight" not in t else t["lm_head.weight"]
    return x.to(torch.float32) @ w.to(torch.float32).T


# --------------------------------------------------------------------------- whole model
def forward_logits(cfg: dict, t: dict, ids, dtype=torch.float32, window: int = 0, schedule=None) -> torch.Tensor:
    """Logits [T, V] (float32) at every position of one whole sequence.

    ``schedule`` lists the layers in the order in which they run (default: each
    once, in order)."""
    s = sizes(cfg)
    ids = torch.as_tensor(ids, dtype=torch.long)
    positions = torch.arange(ids.numel())
    x = embed(t["model.embed_tokens.weight"], ids, dtype)
    for i in (range(s["L"]) if schedule is None else schedule):
        x = decoder_layer(x, t, i, s, positions, window)
    return output_logits(x, t, s)


def greedy_generate(cfg: dict, t: dict, prompt, n_new: int, dtype=torch.float32) -> list[int]:
    """Greedy continuation, recomputing the whole sequence for each token."""
    ids = list(prompt)
    out = []
    for _ in range(n_new):
        nxt = int(forward_logits(cfg, t, ids, dtype)[-1].argmax())
        out.append(nxt)
        ids.append(nxt)
    return out


# --------------------------------------------------------------------------- sampling
def philox_uniform(seed: int, counter: int) -> float:
    """Philox-4x32-10 (Salmon et al., SC'11) keyed by the 64-bit seed, counter =
    (counter, 0, 0, 0); the first output word mapped to (0, 1): (w + 0.5) / 2^32."""
    M0, M1 = 0xD2511F53, 0xCD9E8D57
    W0, W1 = 0x9E3779B9, 0xBB67AE85
    mask = 0xFFFFFFFF
    c = [counter & mask, (counter >> 32) & mask, 0, 0]
    k = [seed & mask, (seed >> 32) & mask]
    for _ in range(10):
        p0 = M0 * c[0]
        p1 = M1 * c[2]
        c = [((p1 >> 32) ^ c[1] ^ k[0]) & mask, p1 & mask, ((p0 >> 32) ^ c[3] ^ k[1]) & mask, p0 & mask]
        k = [(k[0] + W0) & mask, (k[1] + W1) & mask]
    return (c[0] + 0.5) / 4294967296.0


def penalised(logits: torch.Tensor, history: list[int], repetition: float, presence: float, frequency: float) -> torch.Tensor:
    """Penalties on the raw logits: for tokens already seen, divide a positive logit
    by the repetition penalty and multiply a negative one; subtract the presence
    penalty once and the frequency penalty times the count
    (acvram/engine/sampler.py:48-70)."""
    out = logits.clone().to(torch.float32)
    if not history:
        return out
    ids = torch.tensor(sorted(set(history)), dtype=torch.long)
    if repetition != 1.0:
        vals = out[ids]
        out[ids] = torch.where(vals > 0, vals / repetition, vals * repetition)
    if presence:
        out[ids] -= presence
    if frequency:
        counts = torch.bincount(torch.tensor(history, dtype=torch.long), minlength=out.numel()).to(out.dtype)
        out -= frequency * counts
    return out


def filtered_distribution(logits: torch.Tensor, temperature: float, top_k: int, min_p: float, top_p: float) -> torch.Tensor:
    """Scaled logits with the dropped tokens at -inf, in the reference's order:
    / max(T, 1e-5); top-k keeps values >= the k-th; min-p drops p < min_p * p_max;
    top-p sorts descending and drops where (cumulative - p) > top_p, so that the
    token that crosses the threshold stays (acvram/engine/sampler.py:225-246)."""
    scaled = logits.to(torch.float32) / max(temperature, 1e-5)
    V = scaled.numel()
    if top_k and top_k < V:
        kth = torch.topk(scaled, top_k).values[-1]
        scaled = torch.where(scaled < kth, torch.full_like(scaled, float("-inf")), scaled)
    if min_p > 0:
        probs = torch.softmax(scaled, dim=-1)
        scaled = torch.where(probs < min_p * probs.max(), torch.full_like(scaled, float("-inf")), scaled)
    if 0.0 < top_p < 1.0:
        sorted_logits, sorted_idx = torch.sort(scaled, descending=True)
        sm = torch.softmax(sorted_logits, dim=-1)
        drop = sm.cumsum(-1) - sm > top_p
        sorted_logits[drop] = float("-inf")
        scaled = torch.full_like(scaled, float("-inf")).scatter(0, sorted_idx, sorted_logits)
    return scaled


def draw(scaled: torch.Tensor, u: float) -> int:
    """Inverse-CDF draw over the kept tokens in index order: the first index whose
    cumulative probability reaches u (the reference draws with torch.multinomial
    and no per-request generator, acvram/engine/sampler.py:248-249; the engine uses
    a counter-based generator per request instead, so this is its plain form)."""
    probs = torch.softmax(scaled.to(torch.float64), dim=-1)
    cum = probs.cumsum(-1)
    idx = int(torch.searchsorted(cum, torch.tensor(u * float(cum[-1]), dtype=torch.float64), right=False))
    kept = torch.nonzero(probs > 0).flatten()
    idx = min(idx, int(kept[-1]))
    while probs[idx] == 0:
        idx += 1
    return idx
