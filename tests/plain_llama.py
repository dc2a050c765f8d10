"""Plain, slow restatement of the dense Llama decoder, whole sequences, no cache.

This file is the oracle of the test-suite.  It shares no code with the
``zllm_b200`` package: it reads ``config.json`` and ``model.safetensors`` with
its own few lines, computes every part with ordinary torch tensor arithmetic on
the CPU and recomputes the whole sequence for every query.  One function per
part; each cites the lines of fankh/zllm it restates.

It rests on the formulas only: the reference is Rust (candle + WGSL shaders),
no Rust toolchain or GGUF model is available where this suite runs, so the
reference's model code can be neither imported nor compiled, and it ships no
golden numbers.  What anchors this file is (1) the cited formulas, (2) the
identities the reference's own tests assert, restated in ``test_plain.py``,
(3) a second statement written along the reference's own path
(``plain_reference_path.py``: permuted weights with interleaved rotation, a
table of frequency divisors, a cache that grows token by token) with which it
must agree to rounding (``test_two_statements.py``), and (4) the numbers under
``tests/golden/``, which pin both against drift.
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import torch

# --------------------------------------------------------------------------
# reading a model folder (own reader: no code shared with the package)
# --------------------------------------------------------------------------

_ST_DTYPES = {
    "F32": torch.float32,
    "BF16": torch.bfloat16,
    "F16": torch.float16,
    "F64": torch.float64,
    "I32": torch.int32,
    "I64": torch.int64,
}


def read_safetensors(path) -> dict:
    """name -> tensor, every floating tensor widened to float32."""
    raw = Path(path).read_bytes()
    (hlen,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8 : 8 + hlen])
    base = 8 + hlen
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        lo, hi = meta["data_offsets"]
        t = torch.frombuffer(bytearray(raw[base + lo : base + hi]), dtype=_ST_DTYPES[meta["dtype"]])
        t = t.reshape(meta["shape"])
        out[name] = t.float() if t.is_floating_point() else t
    return out


def read_model_dir(model_dir):
    model_dir = Path(model_dir)
    cfg = json.loads((model_dir / "config.json").read_text())
    weights = read_safetensors(model_dir / "model.safetensors")
    return cfg, weights


# --------------------------------------------------------------------------
# parts
# --------------------------------------------------------------------------


def llama3_divisors(head_dim: int, theta: float, scaling: dict) -> list:
    """The divisors f_j a converter stores in ``rope_freqs.weight`` for llama3 scaling (the
    reference only consumes them, fork.rs:584-590, 722-734).  With wavelength lambda_j =
    2*pi/theta_j: f_j = 1 if lambda_j < L/hi, f_j = F if lambda_j > L/lo, else theta_j / theta'_j
    with theta'_j = (1-s) theta_j/F + s theta_j and s = (L/lambda_j - lo)/(hi - lo).  Python floats
    (double), one value per pair."""
    F = float(scaling["factor"])
    lo = float(scaling["low_freq_factor"])
    hi = float(scaling["high_freq_factor"])
    L = float(scaling["original_max_position_embeddings"])
    out = []
    for j in range(0, head_dim, 2):
        th = float(theta) ** (-j / head_dim)
        lam = 2.0 * math.pi / th
        if lam < L / hi:
            out.append(1.0)
        elif lam > L / lo:
            out.append(F)
        else:
            s = (L / lam - lo) / (hi - lo)
            out.append(th / ((1.0 - s) * th / F + s * th))
    return out


def rope_inv_freq(head_dim: int, theta: float, scaling: dict | None, dtype=torch.float32) -> torch.Tensor:
    """theta_j = 1 / base^(i/head_dim) for i = 0, 2, 4, ..., divided by per-pair divisors f_j.

    zllm src/backend/candle/quantized_llama_fork.rs:579-583 computes theta_j with every operand
    f32 (``1f32 / freq_base.powf(i as f32 / head_dim as f32)``) and :584-590 divides by the f32
    divisors in f32; ``dtype`` float32 does exactly that, float64 the same in double (for
    comparisons).  ``linear`` scaling multiplies every theta_j by 1/F (fork.rs:592-597).
    """
    i = torch.arange(0, head_dim, 2, dtype=dtype)
    inv = 1.0 / torch.pow(torch.tensor(float(theta), dtype=dtype), i / torch.tensor(float(head_dim), dtype=dtype))
    if scaling:
        kind = scaling.get("rope_type", scaling.get("type"))
        if kind == "llama3":
            f = torch.tensor(llama3_divisors(head_dim, theta, scaling), dtype=dtype)
            inv = inv / f
        elif kind == "linear":
            inv = inv * (torch.tensor(1.0, dtype=dtype) / float(scaling["factor"]))
        elif kind in (None, "default"):
            pass
        else:
            raise ValueError(f"plain implementation: rope scaling {kind!r} not restated")
    return inv


def rope_tables(inv_freq: torch.Tensor, positions: torch.Tensor):
    """cos/sin of pos * theta_j, the product taken in float32.

    fork.rs:631-638: arange(max_seq) (f32) x theta (f32) then cos, sin.
    """
    ang = positions.to(inv_freq.dtype)[:, None] * inv_freq[None, :]
    return ang.cos(), ang.sin()


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, interleaved: bool) -> torch.Tensor:
    """x [T, heads, head_dim]; cos/sin [T, head_dim/2].

    interleaved (zllm ``rope_i``; src/backend/gpu/shaders.rs:576-586): the pair
    (x[2j], x[2j+1]) -> (a c - b s, a s + b c).
    half-split (zllm ``rope_neox``; fork.rs:447-451): the pair (x[j], x[j+hd/2]),
    same rotation.  A model folder in safetensors layout uses half-split.
    """
    c = cos[:, None, :]
    s = sin[:, None, :]
    if interleaved:
        a = x[..., 0::2]
        b = x[..., 1::2]
        out = torch.empty_like(x)
        out[..., 0::2] = a * c - b * s
        out[..., 1::2] = a * s + b * c
        return out
    half = x.shape[-1] // 2
    a = x[..., :half]
    b = x[..., half:]
    return torch.cat([a * c - b * s, a * s + b * c], dim=-1)


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """y = x * rsqrt(mean(x^2) + eps) * w   (shaders.rs:555-562)."""
    inv = torch.rsqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return x * inv * w


def causal_attention(q, k, v, n_heads, n_kv_heads, positions, window: int | None = None):
    """q [T, nh, hd], k,v [T, nkv, hd] -> [T, nh*hd].

    fork.rs:518-533: repeat_kv, scores = q k^T / sqrt(hd), masked_fill(-inf)
    where key j > query position (mask: fork.rs:846-853), softmax over keys,
    att v, heads concatenated.  ``window`` (not in the reference's Llama) also
    hides keys older than ``window`` positions: key j visible iff
    p - window < j <= p.
    """
    T, _, hd = q.shape
    rep = n_heads // n_kv_heads
    kk = k.repeat_interleave(rep, dim=1)  # kv head h // rep serves query head h
    vv = v.repeat_interleave(rep, dim=1)
    att = torch.einsum("thd,shd->hts", q, kk) / math.sqrt(hd)
    pq = positions[:, None]
    pk = positions[None, :]
    hidden = pk > pq
    if window is not None:
        hidden = hidden | (pk <= pq - window)
    att = att.masked_fill(hidden[None], float("-inf"))
    att = torch.softmax(att, dim=-1)
    y = torch.einsum("hts,shd->thd", att, vv)
    return y.reshape(T, n_heads * hd)


def silu(x):
    """g / (1 + exp(-g))   (shaders.rs:984-988)."""
    return x / (1.0 + torch.exp(-x))


def swiglu_mlp(x, w_gate, w_up, w_down):
    """w2( silu(w1 x) * (w3 x) )   (fork.rs:394-400)."""
    return (silu(x @ w_gate.T) * (x @ w_up.T)) @ w_down.T


# --------------------------------------------------------------------------
# whole model
# --------------------------------------------------------------------------


def forward_all_positions(cfg: dict, w: dict, tokens, dtype=torch.float32, interleaved=False,
                          window=None, return_hidden=False):
    """Logits [T, V] for every position of one sequence.

    fork.rs:1240-1269 (= the forward of fork.rs:920-987 without the last-row
    select): embed, per layer {attn_norm, q/k/v, rope, attention, wo, residual,
    ffn_norm, mlp, residual}, final norm, output head (tied to the embedding
    when the folder holds no lm_head, fork.rs:761-764).
    """
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    T = tokens.numel()
    H = cfg["hidden_size"]
    nh = cfg["num_attention_heads"]
    nkv = cfg.get("num_key_value_heads", nh)
    hd = cfg.get("head_dim") or H // nh
    eps = cfg["rms_norm_eps"]
    W = {k: v.to(dtype) if v.is_floating_point() else v for k, v in w.items()}
    pos = torch.arange(T)
    # float32 theta_j and a float32 product, as the reference; all in double when asked for double
    inv = rope_inv_freq(hd, cfg.get("rope_theta", 10000.0), cfg.get("rope_scaling"),
                        torch.float64 if dtype == torch.float64 else torch.float32)
    cos, sin = rope_tables(inv, pos)
    cos, sin = cos.to(dtype), sin.to(dtype)
    x = W["model.embed_tokens.weight"][tokens]
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        h = rmsnorm(x, W[p + "input_layernorm.weight"], eps)
        q = (h @ W[p + "self_attn.q_proj.weight"].T).reshape(T, nh, hd)
        k = (h @ W[p + "self_attn.k_proj.weight"].T).reshape(T, nkv, hd)
        v = (h @ W[p + "self_attn.v_proj.weight"].T).reshape(T, nkv, hd)
        q = apply_rope(q, cos, sin, interleaved)
        k = apply_rope(k, cos, sin, interleaved)
        a = causal_attention(q, k, v, nh, nkv, pos, window)
        x = x + a @ W[p + "self_attn.o_proj.weight"].T
        h = rmsnorm(x, W[p + "post_attention_layernorm.weight"], eps)
        x = x + swiglu_mlp(h, W[p + "mlp.gate_proj.weight"], W[p + "mlp.up_proj.weight"],
                           W[p + "mlp.down_proj.weight"])
    xn = rmsnorm(x, W["model.norm.weight"], eps)
    head = W.get("lm_head.weight")            # tied iff the folder has no head tensor (fork.rs:761-764)
    if head is None:
        head = W["model.embed_tokens.weight"]
    logits = xn @ head.T
    if return_hidden:
        return logits, x
    return logits


# --------------------------------------------------------------------------
# sampling
# --------------------------------------------------------------------------

_M32 = 0xFFFFFFFF


def argmax_lowest(logits) -> int:
    """Strict '>' scan: the lowest index among equal maxima (shaders.rs:907-909)."""
    best, bi = None, 0
    for i, v in enumerate(logits.tolist() if hasattr(logits, "tolist") else logits):
        if best is None or v > best:
            best, bi = v, i
    return bi


def hash_u32(x: int) -> int:
    """The 2-multiply xorshift of shaders.rs:805-811."""
    h = x & _M32
    h ^= h >> 16
    h = (h * 0x7FEB352D) & _M32
    h ^= h >> 15
    h = (h * 0x846CA68B) & _M32
    h ^= h >> 16
    return h


def rand01(seed: int, i: int) -> float:
    """u = ((hash(seed ^ hash(i)) >> 8) + 0.5) / 2^24, strictly in (0,1) (shaders.rs:812-815)."""
    r = hash_u32((seed ^ hash_u32(i)) & _M32)
    return ((r >> 8) + 0.5) / 16777216.0


def step_seed(base: int, gen_idx: int) -> int:
    """seed_n = base + n * 0x9E3779B1, wrapping (src/backend/gpu/sampling.rs:7-9)."""
    return (base + gen_idx * 0x9E3779B1) & _M32


def gumbel_sample(logits, temperature: float, seed: int) -> int:
    """argmax_i(logit_i / temp - log(-log u_i)); temp <= 0 -> plain argmax (shaders.rs:816-836)."""
    vals = logits.tolist()
    if temperature <= 0:
        return argmax_lowest(vals)
    inv_t = 1.0 / temperature
    best, bi = -1e30, 0
    f32 = torch.float32
    for i, v in enumerate(vals):
        u = torch.tensor(rand01(seed, i), dtype=f32)
        g = -torch.log(-torch.log(u))
        s = float(torch.tensor(v, dtype=f32) * torch.tensor(inv_t, dtype=f32) + g)
        if s > best:
            best, bi = s, i
    return bi


def topk_desc(logits, k: int):
    """K rounds of 'largest strictly below the previous winner', value desc, index asc
    (shaders.rs:852-905)."""
    vals = logits.tolist()
    order = sorted(range(len(vals)), key=lambda i: (-vals[i], i))[:k]
    return [vals[i] for i in order], order


def rng01_splitmix(seed: int) -> float:
    """splitmix64 -> uniform (0,1)  (sampling.rs:24-30)."""
    M = (1 << 64) - 1
    z = ((seed & _M32) * 0x9E3779B97F4A7C15 + 0x9E3779B97F4A7C15) & M
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & M
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & M
    z ^= z >> 31
    return ((z >> 40) + 0.5) / 16777216.0


def sample_topk(vals, idxs, temperature: float, top_k: int, top_p: float, seed: int) -> int:
    """Temperature, top-k, top-p over a descending candidate pool, inverse CDF draw
    (sampling.rs:35-56)."""
    n = 0
    for v in vals:
        if v > -3.0e37:
            n += 1
        else:
            break
    n = min(n, len(idxs))
    if n == 0 or temperature <= 0:
        return idxs[0]
    kk = n if top_k == 0 else min(top_k, n)
    f = torch.float32
    v = torch.tensor(vals[:kk], dtype=f)
    probs = torch.exp((v - v[0]) / torch.tensor(temperature, dtype=f))
    probs = (probs / probs.sum()).tolist()
    cut = kk
    if 0.0 < top_p < 1.0:
        cum = 0.0
        for i, p in enumerate(probs):
            cum += p
            if cum >= top_p:
                cut = i + 1
                break
    zc = sum(probs[:cut])
    target = rng01_splitmix(seed) * zc
    acc = 0.0
    for i in range(cut):
        acc += probs[i]
        if acc >= target:
            return idxs[i]
    return idxs[cut - 1]


def greedy_generate(cfg, w, prompt, n_new, dtype=torch.float32):
    """Whole-sequence recompute per token; argmax with lowest-index ties."""
    toks = list(prompt)
    out = []
    for _ in range(n_new):
        logits = forward_all_positions(cfg, w, toks, dtype=dtype)[-1]
        first = int((logits == logits.max()).nonzero()[0])   # the lowest index among equal maxima
        out.append(first)
        toks.append(first)
    return out
