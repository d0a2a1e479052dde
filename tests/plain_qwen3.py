"""A plain, slow implementation of the Qwen3 dense decoder, for tests only.

Whole sequences, no cache, no batching, one function per part, written from the reference's formulas
(every function cites the file and lines it restates).  It shares no code with ``cuinfer_b200``: it reads
``config.json`` and ``model.safetensors`` by itself (through the ``safetensors`` package) and computes with
torch on the CPU.  The reference's own model code cannot run on a CPU: every op exists only as a CUDA kernel
with fixed sizes (hidden 1024/2048, head_dim 128; csrc/ops/embedding.cu:74-88, csrc/ops/qk_norm_rope_fused.cu:278)
and the model constructor copies to a GPU (csrc/model/causal_lm.cpp:24-33), so this file is written from the formulas.
It is anchored on the reference all the same: ``tests/golden/reference_tokens.json`` holds greedy tokens that the
unmodified reference engine generated on a B200 for a small random model (``tests/golden/make_reference_tokens.py``
made it), and ``tests/test_plain.py`` checks this implementation against them.

Intermediate roundings that the reference's bfloat16 kernels make (after the norm product, between q/k norm
and RoPE, of the softmax weights before they multiply V) are left out on purpose: this is the exact
arithmetic that both the 32-bit path and the bfloat16 path of the engine are measured against.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Sequence

import torch


def load_folder(model_dir: str, dtype: torch.dtype = torch.float32):
    """(config dict, {name: tensor in ``dtype``}) of a model folder."""
    from safetensors.torch import load_file

    with open(os.path.join(model_dir, "config.json")) as fh:
        cfg = json.load(fh)
    tensors = {k: v.to(dtype) for k, v in load_file(os.path.join(model_dir, "model.safetensors")).items()}
    return cfg, tensors


def embed(table: torch.Tensor, ids: Sequence[int]) -> torch.Tensor:
    """x[t] = E[id_t], no scaling (csrc/ops/embedding.cu:31-35; csrc/model/causal_lm.cpp:74-80)."""
    return table[torch.tensor(list(ids), dtype=torch.long)]


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """x * rsqrt(mean(x^2) + eps) * w over the last axis; eps inside the root, weight multiplies directly
    (csrc/ops/rms_norm.cu:43-71)."""
    var = (x * x).mean(dim=-1, keepdim=True)
    return x * torch.rsqrt(var + eps) * weight


def rope_cos_sin(theta: float, rotary_dim: int, positions: torch.Tensor):
    """cos/sin of p * f_i with f_i = 1 / theta^(2i / rotary_dim), frequencies and angles in float32
    (csrc/model/rope_cache.cpp:15-24, :47-58)."""
    half = rotary_dim // 2
    exponent = torch.arange(half, dtype=torch.float32) * 2.0 / float(rotary_dim)
    inv_freq = 1.0 / torch.pow(torch.tensor(float(theta), dtype=torch.float32), exponent)
    angle = positions.to(torch.float32)[:, None] * inv_freq[None, :]
    return torch.cos(angle), torch.sin(angle)


def apply_rope(u: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotate-half over the first 2*half elements of every head: u'[i] = u[i] cos - u[i+half] sin,
    u'[i+half] = u[i+half] cos + u[i] sin (csrc/ops/qk_norm_rope_fused.cu:114-139).  u: [n, heads, d]."""
    half = cos.shape[-1]
    c = cos.to(u.dtype)[:, None, :]
    s = sin.to(u.dtype)[:, None, :]
    a, b, rest = u[..., :half], u[..., half:2 * half], u[..., 2 * half:]
    return torch.cat((a * c - b * s, b * c + a * s, rest), dim=-1)


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                     window: Optional[int] = None) -> torch.Tensor:
    """softmax(q k^T * scale + causal mask) v; query head a uses kv head a // (nq / nkv)
    (csrc/ops/paged_attention.cu:204, :239-276, :283-340; scale 1/sqrt(d) at :163-164).
    q: [n, nq, d]; k, v: [n, nkv, d] -> [n, nq, d].  ``window`` w keeps keys j with p - w < j <= p."""
    n, nq, d = q.shape
    nkv = k.shape[1]
    g = nq // nkv
    out = torch.empty_like(q)
    idx = torch.arange(n)
    mask = idx[None, :] > idx[:, None]
    if window is not None:
        mask = mask | (idx[None, :] <= idx[:, None] - window)
    for a in range(nq):
        h = a // g
        s = (q[:, a, :] @ k[:, h, :].T) * scale
        s = s.masked_fill(mask, float("-inf"))
        out[:, a, :] = torch.softmax(s, dim=-1) @ v[:, h, :]
    return out


def attention_layer(x: torch.Tensor, w: Dict[str, torch.Tensor], prefix: str, cfg: dict,
                    positions: torch.Tensor) -> torch.Tensor:
    """q/k/v projections without bias, per-head q_norm/k_norm with eps = rms_norm_eps, RoPE, causal GQA
    attention, output projection (csrc/model/layers/attention.cpp:44-105; qk-norm
    csrc/ops/qk_norm_rope_fused.cu:88-112)."""
    nq, nkv = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    d = cfg.get("head_dim") or cfg["hidden_size"] // nq
    n = x.shape[0]
    q = (x @ w[f"{prefix}.q_proj.weight"].T).view(n, nq, d)
    k = (x @ w[f"{prefix}.k_proj.weight"].T).view(n, nkv, d)
    v = (x @ w[f"{prefix}.v_proj.weight"].T).view(n, nkv, d)
    q = rms_norm(q, w[f"{prefix}.q_norm.weight"], cfg["rms_norm_eps"])
    k = rms_norm(k, w[f"{prefix}.k_norm.weight"], cfg["rms_norm_eps"])
    cos, sin = rope_cos_sin(cfg["rope_theta"], d, positions)
    q = apply_rope(q, cos, sin)
    k = apply_rope(k, cos, sin)
    o = causal_attention(q, k, v, 1.0 / math.sqrt(d))
    return o.reshape(n, nq * d) @ w[f"{prefix}.o_proj.weight"].T


def swiglu(x: torch.Tensor, w: Dict[str, torch.Tensor], prefix: str) -> torch.Tensor:
    """down( g * u / (1 + exp(-g)) ) with g = gate(x), u = up(x), no bias
    (csrc/model/layers/mlp.cpp:21-27; csrc/ops/swiglu.cu:23-32)."""
    g = x @ w[f"{prefix}.gate_proj.weight"].T
    u = x @ w[f"{prefix}.up_proj.weight"].T
    return (g / (1.0 + torch.exp(-g)) * u) @ w[f"{prefix}.down_proj.weight"].T


def decoder_layer(x: torch.Tensor, w: Dict[str, torch.Tensor], i: int, cfg: dict, positions: torch.Tensor) -> torch.Tensor:
    """x += attn(norm(x)); x += mlp(norm(x)) (csrc/model/causal_lm.cpp:138-188)."""
    p = f"model.layers.{i}"
    eps = cfg["rms_norm_eps"]
    x = x + attention_layer(rms_norm(x, w[f"{p}.input_layernorm.weight"], eps), w, f"{p}.self_attn", cfg, positions)
    x = x + swiglu(rms_norm(x, w[f"{p}.post_attention_layernorm.weight"], eps), w, f"{p}.mlp")
    return x


def forward(cfg: dict, w: Dict[str, torch.Tensor], ids: Sequence[int]) -> torch.Tensor:
    """Logits [n, vocab] at every position of one whole sequence: embedding, layers, final norm, output
    head = embedding when tied (csrc/model/causal_lm.cpp:67-115, :35-38)."""
    x = embed(w["model.embed_tokens.weight"], ids)
    positions = torch.arange(len(ids))
    for i in range(cfg["num_hidden_layers"]):
        x = decoder_layer(x, w, i, cfg, positions)
    x = rms_norm(x, w["model.norm.weight"], cfg["rms_norm_eps"])
    head = w["model.embed_tokens.weight"] if cfg["tie_word_embeddings"] else w["lm_head.weight"]
    return x @ head.T


def logits_at(cfg: dict, w: Dict[str, torch.Tensor], ids: Sequence[int], positions: Sequence[int]) -> torch.Tensor:
    """The rows ``positions`` of ``forward``'s result, with the output head applied to those rows only (for
    vocabularies where the whole [n, vocab] matrix would be large)."""
    x = embed(w["model.embed_tokens.weight"], ids)
    pos = torch.arange(len(ids))
    for i in range(cfg["num_hidden_layers"]):
        x = decoder_layer(x, w, i, cfg, pos)
    x = rms_norm(x[torch.tensor(list(positions), dtype=torch.long)], w["model.norm.weight"], cfg["rms_norm_eps"])
    head = w["model.embed_tokens.weight"] if cfg["tie_word_embeddings"] else w["lm_head.weight"]
    return x @ head.T


def greedy_generate(cfg: dict, w: Dict[str, torch.Tensor], prompt: Sequence[int], num_new: int) -> List[int]:
    """Argmax decoding by recomputing the whole sequence each time; ties go to the lowest id
    (csrc/ops/sampler.cu:31-38)."""
    ids = list(prompt)
    out = []
    for _ in range(num_new):
        logits = forward(cfg, w, ids)[-1]
        nxt = int(torch.argmax(logits))          # torch.argmax returns the first maximal index
        out.append(nxt)
        ids.append(nxt)
    return out


def sample_plain(logits: torch.Tensor, temperature: float, top_k: int, top_p: float, u: float) -> int:
    """One draw with the options' meaning of csrc/ops/sampler.cu:207-386: temperature 0 -> argmax (lowest id);
    top_k keeps values >= the k-th largest (ties kept); top_p keeps the smallest set of most probable kept
    tokens whose mass reaches top_p (ties at the edge kept); the token is the first index whose running kept
    mass exceeds u * kept mass."""
    x = logits.double()
    if temperature <= 0 or top_k == 1:
        return int(torch.argmax(x))
    keep = torch.ones_like(x, dtype=torch.bool)
    V = x.numel()
    if 0 < top_k < V:
        kth = torch.sort(x, descending=True).values[top_k - 1]
        keep &= x >= kth
    wgt = torch.exp((x - x.max()) / temperature) * keep
    if 0 < top_p < 1:
        order = torch.argsort(wgt, descending=True, stable=True)
        csum = torch.cumsum(wgt[order], 0)
        need = top_p * wgt.sum()
        cut = int(torch.searchsorted(csum, need.reshape(1)).item())
        cut = min(cut, V - 1)
        thresh = wgt[order][cut]
        wgt = wgt * (wgt >= thresh)
    csum = torch.cumsum(wgt, 0)
    target = u * csum[-1]
    return int(torch.searchsorted(csum, target.reshape(1), right=True).item())
