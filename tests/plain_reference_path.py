"""A second plain statement of the dense Llama decoder, written along the
REFERENCE'S OWN path rather than along ``plain_llama.py``'s, so that the two
can only agree if both read the formulas the same way.

Where ``plain_llama.py`` is torch, whole sequences, half-split rotation on the
folder's weights and the llama3 blend applied to theta_j, this file is

* NumPy only, double precision, scalar loops over heads and keys;
* a cache that grows token by token, one query at a time, as the reference's
  decode path runs (zllm src/backend/candle/quantized_llama_fork.rs:495-510 and
  src/backend/candle/sdpa_cpu.rs:123-165: scores, maximum, exponentials, sum,
  weighted values, query head h reads kv head h // (nh/nkv));
* the reference's rotary convention: the rows of Wq and Wk are permuted the way
  a GGUF converter permutes them and pairs (x[2j], x[2j+1]) are rotated
  (``rope_i``, src/backend/arch.rs:25-35; src/backend/gpu/shaders.rs:576-586);
* the reference's llama3 mechanism: a table of divisors f_j, as
  ``rope_freqs.weight`` holds them, by which theta_j is divided unless f_j is 0
  (fork.rs:584-590) -- the divisors are derived here from the wavelength rule
  on their own, in the form "interpolate the divisor's reciprocal";
* the softmax in its online form where asked (running maximum and sum,
  shaders.rs:703-723).

It shares no code with ``plain_llama.py`` or with the package and reads the
model folder with its own few lines.  Like ``plain_llama.py`` it rests on the
formulas only: the reference is Rust and can be neither imported nor compiled
where this suite runs.
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np

_NP = {"F32": np.float32, "F64": np.float64, "F16": np.float16, "I32": np.int32, "I64": np.int64}


def _bf16_to_f64(raw: bytes, shape):
    u = np.frombuffer(raw, dtype=np.uint16).astype(np.uint32) << 16
    return u.view(np.float32).astype(np.float64).reshape(shape)


def read_folder(model_dir):
    """(config dict, name -> float64 array).  Container: 8-byte length, JSON header, raw data."""
    d = Path(model_dir)
    cfg = json.loads((d / "config.json").read_text())
    blob = (d / "model.safetensors").read_bytes()
    (n,) = struct.unpack("<Q", blob[:8])
    head = json.loads(blob[8:8 + n])
    out = {}
    for name, m in head.items():
        if name == "__metadata__":
            continue
        a, b = m["data_offsets"]
        raw = blob[8 + n + a:8 + n + b]
        if m["dtype"] == "BF16":
            out[name] = _bf16_to_f64(raw, m["shape"])
        else:
            out[name] = np.frombuffer(raw, dtype=_NP[m["dtype"]]).reshape(m["shape"]).astype(np.float64)
    return cfg, out


def gguf_row_order(n_heads: int, head_dim: int):
    """Row order that turns half-split pairs (j, j + hd/2) of each head into neighbours
    (2j, 2j+1): what a GGUF converter does to Wq and Wk of this family (arch.rs:25-28)."""
    order = []
    for h in range(n_heads):
        for j in range(head_dim // 2):
            order += [h * head_dim + j, h * head_dim + j + head_dim // 2]
    return np.array(order)


def freq_divisors(cfg):
    """The table ``rope_freqs.weight`` would hold: one divisor per pair, 1 where nothing changes."""
    hd = cfg.get("head_dim") or cfg["hidden_size"] // cfg["num_attention_heads"]
    sc = cfg.get("rope_scaling")
    n = hd // 2
    if not sc or sc.get("rope_type", sc.get("type")) in (None, "default"):
        return [1.0] * n
    kind = sc.get("rope_type", sc.get("type"))
    if kind == "linear":
        return [float(sc["factor"])] * n
    if kind != "llama3":
        raise ValueError(kind)
    F, lo, hi = float(sc["factor"]), float(sc["low_freq_factor"]), float(sc["high_freq_factor"])
    L = float(sc["original_max_position_embeddings"])
    base = float(cfg.get("rope_theta", 10000.0))
    out = []
    for j in range(n):
        turns = L / (2.0 * math.pi * base ** (2.0 * j / hd))      # rotations within the original context
        if turns > hi:
            out.append(1.0)
        elif turns < lo:
            out.append(F)
        else:
            t = (turns - lo) / (hi - lo)                          # 0 at the slow end, 1 at the fast end
            out.append(1.0 / ((1.0 - t) / F + t))                 # the reciprocal is what is interpolated
    return out


def rotate_pairs(x, pos, theta):
    """(x[2j], x[2j+1]) -> (a c - b s, a s + b c), angle pos * theta_j (shaders.rs:576-586)."""
    y = np.empty_like(x)
    for j, th in enumerate(theta):
        c, s = math.cos(pos * th), math.sin(pos * th)
        a, b = x[2 * j], x[2 * j + 1]
        y[2 * j] = a * c - b * s
        y[2 * j + 1] = a * s + b * c
    return y


def rms(x, w, eps):
    """x / sqrt(mean(x^2) + eps) * w (shaders.rs:555-562)."""
    return x / math.sqrt(float(np.dot(x, x)) / x.size + eps) * w


def attend_two_pass(q, keys, vals, scale):
    """sdpa_cpu.rs:131-165: scores, their maximum, exponentials, their sum, weighted values."""
    s = [float(np.dot(q, k)) * scale for k in keys]
    m = max(s)
    e = [math.exp(v - m) for v in s]
    z = sum(e)
    out = np.zeros_like(vals[0])
    for w, v in zip(e, vals):
        out += (w / z) * v
    return out


def attend_online(q, keys, vals, scale):
    """shaders.rs:703-723: one pass with a running maximum, sum and accumulator."""
    m, z, acc = -math.inf, 0.0, np.zeros_like(vals[0])
    for k, v in zip(keys, vals):
        s = float(np.dot(q, k)) * scale
        m2 = max(m, s)
        c = math.exp(m - m2) if m > -math.inf else 0.0
        p = math.exp(s - m2)
        z = z * c + p
        acc = acc * c + p * v
        m = m2
    return acc / z


def logits_token_by_token(cfg, w, tokens, online=False, window=None):
    """Logits [T, V] (float64), feeding one token at a time against a growing cache."""
    H = cfg["hidden_size"]
    nh = cfg["num_attention_heads"]
    nkv = cfg.get("num_key_value_heads", nh)
    hd = cfg.get("head_dim") or H // nh
    L = cfg["num_hidden_layers"]
    eps = cfg["rms_norm_eps"]
    base = float(cfg.get("rope_theta", 10000.0))
    theta = [base ** (-2.0 * j / hd) for j in range(hd // 2)]
    theta = [t / f if f != 0 else t for t, f in zip(theta, freq_divisors(cfg))]
    qo, ko = gguf_row_order(nh, hd), gguf_row_order(nkv, hd)
    scale = 1.0 / math.sqrt(hd)
    attend = attend_online if online else attend_two_pass
    emb = w["model.embed_tokens.weight"]
    head = w["lm_head.weight"] if "lm_head.weight" in w else emb     # tied iff absent (fork.rs:761-764)
    cache_k = [[[] for _ in range(nkv)] for _ in range(L)]
    cache_v = [[[] for _ in range(nkv)] for _ in range(L)]
    out = []
    for pos, tok in enumerate(tokens):
        x = emb[tok].copy()
        for l in range(L):
            p = f"model.layers.{l}."
            h = rms(x, w[p + "input_layernorm.weight"], eps)
            q = w[p + "self_attn.q_proj.weight"][qo] @ h
            k = w[p + "self_attn.k_proj.weight"][ko] @ h
            v = w[p + "self_attn.v_proj.weight"] @ h
            for g in range(nkv):
                cache_k[l][g].append(rotate_pairs(k[g * hd:(g + 1) * hd], pos, theta))
                cache_v[l][g].append(v[g * hd:(g + 1) * hd])
            first = 0 if window is None else max(0, pos - window + 1)
            y = np.empty(nh * hd)
            for hq in range(nh):
                g = hq // (nh // nkv)
                qh = rotate_pairs(q[hq * hd:(hq + 1) * hd], pos, theta)
                y[hq * hd:(hq + 1) * hd] = attend(qh, cache_k[l][g][first:], cache_v[l][g][first:], scale)
            x = x + w[p + "self_attn.o_proj.weight"] @ y
            h = rms(x, w[p + "post_attention_layernorm.weight"], eps)
            gate = w[p + "mlp.gate_proj.weight"] @ h
            up = w[p + "mlp.up_proj.weight"] @ h
            x = x + w[p + "mlp.down_proj.weight"] @ (gate / (1.0 + np.exp(-gate)) * up)
        out.append(head @ rms(x, w["model.norm.weight"], eps))
    return np.stack(out)
