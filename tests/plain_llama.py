"""Plain, slow, whole-sequence implementation of the dense Llama decoder.

It is the yardstick of the test-suite: no cache, no batching, no kernels, one
function for each part, written from the formulas of IanConery/lyapunov-engine
(each function cites the file and lines it follows).  It shares no code with
the product package: it reads a model folder with the ``safetensors`` library
and ``json`` and computes in float32 (or float64) with plain torch ops on the
CPU.

The llama3 frequency scaling is not in the reference (its model builds plain
``inv_freq`` only, python/lyapunov_engine/models/llama.py:180-184); it is
written here from the definition of the ``rope_scaling`` keys of config.json
(``factor``, ``low_freq_factor``, ``high_freq_factor``,
``original_max_position_embeddings``).  Everything else was compared once with
the reference's own model code on the CPU; tests/golden/ holds the outputs and
the script that made them.
"""
from __future__ import annotations

import json
import math
import os

import torch


# --------------------------------------------------------------------------
# model folder
# --------------------------------------------------------------------------
def read_model_folder(folder: str, dtype=torch.float32):
    """config.json as a dict and every tensor of every *.safetensors file,
    later files overwriting earlier ones in sorted order
    (python/lyapunov_engine/models/weight_loader.py:10-21, 49-57)."""
    from safetensors.torch import load_file

    with open(os.path.join(folder, "config.json"), "r", encoding="utf-8") as f:
        cfg = json.load(f)
    tensors = {}
    for name in sorted(os.listdir(folder)):
        if name.endswith(".safetensors"):
            tensors.update(load_file(os.path.join(folder, name)))
    tensors = {k: v.to(dtype) for k, v in tensors.items()}
    return cfg, tensors


def head_dim_of(cfg: dict) -> int:
    """head_dim, by default hidden_size // num_attention_heads
    (python/lyapunov_engine/models/weight_loader.py:29-34)."""
    return int(cfg.get("head_dim") or cfg["hidden_size"] // cfg["num_attention_heads"])


# --------------------------------------------------------------------------
# parts
# --------------------------------------------------------------------------
def plain_embedding(ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """h0[t] = E[id_t] (python/lyapunov_engine/models/llama.py:172,205)."""
    return table[ids.long()]


def plain_rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """x * rsqrt(mean(x^2) + eps) * w (python/lyapunov_engine/ops.py:49-50;
    csrc/kernels/fused_rmsnorm_swiglu.cu:83-101)."""
    variance = x.pow(2).mean(-1, keepdim=True)
    return x * torch.rsqrt(variance + eps) * weight


def plain_inv_freq(head_dim: int, theta: float, rope_scaling: dict | None) -> torch.Tensor:
    """f_j = theta^(-2j/hd) in float32
    (python/lyapunov_engine/models/llama.py:180-184); then, for
    rope_type "llama3", the piecewise scaling by wavelength."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2).float() / head_dim))
    if not rope_scaling:
        return inv_freq
    kind = rope_scaling.get("rope_type", rope_scaling.get("type", "default"))
    if kind == "default":
        return inv_freq
    if kind != "llama3":
        raise ValueError(f"plain implementation knows no rope_type {kind!r}")
    factor = float(rope_scaling["factor"])
    low = float(rope_scaling["low_freq_factor"])
    high = float(rope_scaling["high_freq_factor"])
    orig = float(rope_scaling["original_max_position_embeddings"])
    out = []
    for f in inv_freq.tolist():
        wavelen = 2.0 * math.pi / f
        if wavelen < orig / high:
            out.append(f)
        elif wavelen > orig / low:
            out.append(f / factor)
        else:
            smooth = (orig / wavelen - low) / (high - low)
            out.append((1.0 - smooth) * f / factor + smooth * f)
    return torch.tensor(out, dtype=torch.float32)


def plain_cos_sin(positions: torch.Tensor, inv_freq: torch.Tensor):
    """angles = outer(p, f) in float32, doubled along the last axis, cos and
    sin of it (python/lyapunov_engine/models/llama.py:186-194)."""
    t = positions.to(inv_freq.dtype)
    freqs = torch.outer(t, inv_freq)
    emb = torch.cat((freqs, freqs), dim=-1)
    return emb.cos(), emb.sin()


def plain_rotate_half(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x*cos + cat(-x2, x1)*sin (python/lyapunov_engine/models/llama.py:23-31).
    x: [heads, T, hd]; cos, sin: [T, hd]."""
    d = x.shape[-1]
    x1 = x[..., : d // 2]
    x2 = x[..., d // 2:]
    rotated = torch.cat((-x2, x1), dim=-1)
    return x * cos + rotated * sin


def plain_attention(q, k, v, window: int | None = None, prob_dtype=None, prob_shift: float = 0.0) -> torch.Tensor:
    """Causal grouped-query attention over a whole sequence
    (python/lyapunov_engine/ops.py:100-121): scale 1/sqrt(hd), kv heads
    repeated for their group, keys after the query masked, softmax, times V.
    q: [nh, T, hd]; k, v: [nkv, T, hd].  ``window`` (not in the reference):
    a query at p sees keys p-window+1 .. p only.  ``prob_dtype`` models a
    pipeline that stores exp(score - max) in that type before it multiplies by
    V (and still divides by the unrounded sum); ``prob_shift`` one that scales
    its numerators by another bound than the row's true maximum, exp(score -
    max - shift): the same mathematics, other roundings."""
    nh, T, hd = q.shape
    nkv = k.shape[0]
    scale = 1.0 / (hd ** 0.5)
    if nh != nkv:
        ratio = nh // nkv
        k = k.repeat_interleave(ratio, dim=0)
        v = v.repeat_interleave(ratio, dim=0)
    scores = torch.matmul(q, k.transpose(-1, -2)) * scale
    mask = torch.triu(torch.ones(T, T, dtype=torch.bool), diagonal=1)
    if window is not None:
        mask |= torch.tril(torch.ones(T, T, dtype=torch.bool), diagonal=-window)
    scores = scores.masked_fill(mask, float("-inf"))
    if prob_dtype is not None:
        p = torch.exp(scores - scores.max(dim=-1, keepdim=True).values - prob_shift)
        return torch.matmul(rounded(p, prob_dtype), v) / p.sum(dim=-1, keepdim=True)
    probs = torch.softmax(scores, dim=-1)
    return torch.matmul(probs, v)


def rounded(x: torch.Tensor, act_dtype) -> torch.Tensor:
    """What storing an activation in ``act_dtype`` does to it (nothing when
    act_dtype is None).  With act_dtype=torch.bfloat16 the plain implementation
    models a pipeline whose activations between matrix products are bfloat16
    while the residual stream, norms, softmax and rotation stay 32-bit."""
    return x if act_dtype is None else x.to(act_dtype).to(x.dtype)


def plain_attention_layer(x, wq, wk, wv, wo, nh, nkv, hd, cos, sin, window=None, act_dtype=None, prob_dtype=None,
                          prob_shift=0.0):
    """q/k/v projections, head split, RoPE on q and k, attention, o projection
    (python/lyapunov_engine/models/llama.py:61-106)."""
    T = x.shape[0]
    q = rounded(x @ wq.T, act_dtype).view(T, nh, hd).transpose(0, 1)
    k = rounded(x @ wk.T, act_dtype).view(T, nkv, hd).transpose(0, 1)
    v = rounded(x @ wv.T, act_dtype).view(T, nkv, hd).transpose(0, 1)
    q = rounded(plain_rotate_half(q, cos, sin), act_dtype)
    k = rounded(plain_rotate_half(k, cos, sin), act_dtype)
    o = rounded(plain_attention(q, k, v, window, prob_dtype, prob_shift), act_dtype)
    o = o.transpose(0, 1).contiguous().view(T, nh * hd)
    return rounded(o @ wo.T, act_dtype)


def plain_swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """silu(gate) * up (python/lyapunov_engine/ops.py:71-73;
    csrc/kernels/fused_rmsnorm_swiglu.cu:170-176)."""
    return gate / (1.0 + torch.exp(-gate)) * up


def plain_mlp(x, w_gate, w_up, w_down, act_dtype=None) -> torch.Tensor:
    """down(silu(gate(x)) * up(x)) (python/lyapunov_engine/models/llama.py:119-122)."""
    act = plain_swiglu(rounded(x @ w_gate.T, act_dtype), rounded(x @ w_up.T, act_dtype))
    return rounded(rounded(act, act_dtype) @ w_down.T, act_dtype)


def plain_block(h, w: dict, prefix: str, cfg: dict, cos, sin, window=None, act_dtype=None, prob_dtype=None,
                prob_shift=0.0):
    """Pre-norm residual block (python/lyapunov_engine/models/llama.py:136-165)."""
    eps = float(cfg["rms_norm_eps"])
    nh = cfg["num_attention_heads"]
    nkv = cfg.get("num_key_value_heads", nh)
    hd = head_dim_of(cfg)
    n = rounded(plain_rmsnorm(h, w[prefix + "input_layernorm.weight"], eps), act_dtype)
    a = plain_attention_layer(
        n,
        w[prefix + "self_attn.q_proj.weight"],
        w[prefix + "self_attn.k_proj.weight"],
        w[prefix + "self_attn.v_proj.weight"],
        w[prefix + "self_attn.o_proj.weight"],
        nh, nkv, hd, cos, sin, window, act_dtype, prob_dtype, prob_shift,
    )
    h = h + a
    n = rounded(plain_rmsnorm(h, w[prefix + "post_attention_layernorm.weight"], eps), act_dtype)
    m = plain_mlp(
        n,
        w[prefix + "mlp.gate_proj.weight"],
        w[prefix + "mlp.up_proj.weight"],
        w[prefix + "mlp.down_proj.weight"],
        act_dtype,
    )
    return h + m


def plain_forward(cfg: dict, w: dict, ids, windows=None, act_dtype=None, prob_dtype=None, prob_shift=0.0) -> torch.Tensor:
    """Logits [T, V] of one whole sequence starting at position 0
    (python/lyapunov_engine/models/llama.py:196-225).  The output head is
    ``lm_head.weight`` when the folder has it, else the embedding matrix
    (python/lyapunov_engine/models/weight_loader.py:102-109).  ``act_dtype``:
    see ``rounded``."""
    ids = torch.as_tensor(ids)
    T = ids.shape[0]
    dtype = w["model.embed_tokens.weight"].dtype
    h = plain_embedding(ids, w["model.embed_tokens.weight"])
    inv_freq = plain_inv_freq(head_dim_of(cfg), float(cfg.get("rope_theta", 500000.0)),
                              cfg.get("rope_scaling"))
    cos, sin = plain_cos_sin(torch.arange(T), inv_freq)
    cos, sin = cos.to(dtype), sin.to(dtype)
    for i in range(cfg["num_hidden_layers"]):
        window = windows[i] if windows is not None else None
        h = plain_block(h, w, f"model.layers.{i}.", cfg, cos, sin, window, act_dtype, prob_dtype, prob_shift)
    n = rounded(plain_rmsnorm(h, w["model.norm.weight"], float(cfg["rms_norm_eps"])), act_dtype)
    head = w.get("lm_head.weight", w["model.embed_tokens.weight"])
    return n @ head.T


# --------------------------------------------------------------------------
# sampling
# --------------------------------------------------------------------------
def plain_filtered_probs(logits: torch.Tensor, temperature: float, top_k: int, top_p: float):
    """The distribution the reference draws from
    (python/lyapunov_engine/engine/sampling.py:40-68): logits / T, keep values
    not below the k-th largest, then drop the sorted tail whose preceding
    cumulative probability exceeds top_p, softmax."""
    x = logits.double() / temperature
    if top_k > 0 and top_k < x.shape[-1]:
        kth = torch.topk(x, top_k).values[-1]
        x = torch.where(x < kth, torch.tensor(float("-inf"), dtype=x.dtype), x)
    if top_p < 1.0:
        sorted_logits, sorted_idx = torch.sort(x, descending=True)
        cum = torch.cumsum(torch.softmax(sorted_logits, dim=-1), dim=-1)
        remove = cum > top_p
        remove[1:] = remove[:-1].clone()
        remove[0] = False
        x[sorted_idx[remove]] = float("-inf")
    return torch.softmax(x, dim=-1)


def plain_greedy(logits: torch.Tensor) -> int:
    """argmax, the first of equal maxima
    (python/lyapunov_engine/engine/sampling.py:34-38)."""
    return int(torch.argmax(logits).item())


def plain_greedy_generate(cfg: dict, w: dict, prompt, steps: int):
    """Greedy continuation by whole-sequence forwards, one per new token."""
    ids = list(prompt)
    out = []
    for _ in range(steps):
        logits = plain_forward(cfg, w, ids)
        tok = plain_greedy(logits[-1])
        out.append(tok)
        ids.append(tok)
    return out
