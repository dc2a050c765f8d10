"""The plain implementation itself: the identities the reference's own tests assert,
restated (CPU).  They anchor ``plain_llama.py`` to zllm's kernel math."""
import math

import pytest
import torch

import plain_llama as P
from configs import TINY, make_model_dir, random_prompt


def test_online_softmax_equals_two_pass():
    """shaders.rs:703-723 (running max / sum) vs sdpa_cpu.rs:138-165 (two passes)."""
    g = torch.Generator().manual_seed(0)
    q = torch.randn(16, generator=g)
    K = torch.randn(70, 16, generator=g)
    V = torch.randn(70, 16, generator=g)
    s = K @ q / 4.0
    two = torch.softmax(s, 0) @ V
    m, l, acc = -math.inf, 0.0, torch.zeros(16)
    for j in range(70):
        m_new = max(m, float(s[j]))
        corr = math.exp(m - m_new)
        p = math.exp(float(s[j]) - m_new)
        l = l * corr + p
        acc = acc * corr + p * V[j]
        m = m_new
    assert torch.allclose(acc / l, two, atol=1e-5)


def test_gqa_by_index_equals_repeat_kv():
    """sdpa_cpu.rs:296-304: kv head h // (nh/nkv) == repeat_kv then per-head."""
    g = torch.Generator().manual_seed(1)
    T, nh, nkv, hd = 9, 6, 2, 16
    q, k, v = torch.randn(T, nh, hd, generator=g), torch.randn(T, nkv, hd, generator=g), torch.randn(T, nkv, hd, generator=g)
    pos = torch.arange(T)
    out = P.causal_attention(q, k, v, nh, nkv, pos).reshape(T, nh, hd)
    for h in range(nh):
        kvh = h // (nh // nkv)
        s = (q[:, h] @ k[:, kvh].T) / math.sqrt(hd)
        s = s.masked_fill(pos[None, :] > pos[:, None], -math.inf)
        assert torch.allclose(torch.softmax(s, -1) @ v[:, kvh], out[:, h], atol=1e-5)


def test_interleaved_on_permuted_rows_equals_half_split():
    """arch.rs:25-35: GGUF converters permute the rows of Wq/Wk so that interleaved rotation of the
    permuted projection equals half-split rotation of the original one."""
    g = torch.Generator().manual_seed(2)
    hd, H, T = 16, 24, 5
    W = torch.randn(hd, H, generator=g)
    x = torch.randn(T, H, generator=g)
    inv = P.rope_inv_freq(hd, 10000.0, None)
    cos, sin = P.rope_tables(inv, torch.arange(T))
    perm = torch.stack([torch.arange(hd // 2), torch.arange(hd // 2) + hd // 2], 1).reshape(-1)  # 0,8,1,9,...
    a = P.apply_rope((x @ W.T)[:, None, :], cos, sin, interleaved=False)[:, 0]
    b = P.apply_rope((x @ W[perm].T)[:, None, :], cos, sin, interleaved=True)[:, 0]
    assert torch.allclose(a[:, perm], b, atol=1e-6)
    k = torch.randn(T, hd, generator=g)
    ka = P.apply_rope(k[:, None, :], cos, sin, False)[:, 0]
    kb = P.apply_rope(k[:, perm][:, None, :], cos, sin, True)[:, 0]
    assert torch.allclose(a @ ka.T, b @ kb.T, atol=1e-5)      # the scores agree


def test_llama3_divisors():
    inv0 = P.rope_inv_freq(32, 500000.0, None, torch.float64)
    sc = dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0, original_max_position_embeddings=64)
    inv = P.rope_inv_freq(32, 500000.0, sc, torch.float64)
    lam = 2 * math.pi / inv0
    assert torch.equal(inv[lam < 16], inv0[lam < 16])                       # short wavelengths untouched
    assert torch.allclose(inv[lam > 64], inv0[lam > 64] / 8.0)              # long ones divided by the factor
    mid = (lam >= 16) & (lam <= 64)
    assert mid.any() and ((inv[mid] <= inv0[mid]) & (inv[mid] >= inv0[mid] / 8.0)).all()
    # the package's own rotary part states the same formula independently (float32, as the reference)
    from zllm_b200.parts.rotary import inverse_frequencies
    got = inverse_frequencies(32, 500000.0, sc)
    assert got.dtype == torch.float32 and torch.allclose(got.double(), inv, rtol=3e-7, atol=0)
    assert torch.allclose(got, P.rope_inv_freq(32, 500000.0, sc), rtol=2.5e-7, atol=0)
    lin = P.rope_inv_freq(32, 10000.0, dict(rope_type="linear", factor=4.0), torch.float64)
    assert torch.allclose(lin, P.rope_inv_freq(32, 10000.0, None, torch.float64) / 4.0)


def test_theta_in_float32_as_the_reference_and_how_far_double_precision_tables_are():
    """fork.rs:579-583 computes theta_j in f32; tables made from double-precision theta_j rounded
    once differ from the reference's by up to an ulp of theta_j times the position.  Stated here
    for the largest sizes in use (head size 64, base 500000, llama3 factor 32, 131072 positions)."""
    sc = dict(rope_type="llama3", factor=32.0, low_freq_factor=1.0, high_freq_factor=4.0,
              original_max_position_embeddings=8192)
    f32 = P.rope_inv_freq(64, 500000.0, sc)
    f64 = P.rope_inv_freq(64, 500000.0, sc, torch.float64)
    assert f32.dtype == torch.float32
    rel = ((f32.double() - f64) / f64).abs().max()
    assert float(rel) < 2.4e-7                                  # two float32 roundings and a powf
    far = float(((f32.double() - f64.float().double()).abs() * 131071).max())
    assert far < 0.02                                           # radians at the last position: 0.003 typical
    # the engine's tables are the float32 product of the float32 theta_j (fork.rs:631-637)
    from zllm_b200.parts.rotary import inverse_frequencies
    assert torch.allclose(inverse_frequencies(64, 500000.0, sc), f32, rtol=2.5e-7, atol=0)
    ff = [0.0, 2.0] + [1.0] * 30                                # explicit divisors; 0 leaves a pair alone
    e = inverse_frequencies(64, 10000.0, None, ff)
    b = inverse_frequencies(64, 10000.0, None)
    assert e[0] == b[0] and e[1] == b[1] / 2 and torch.equal(e[2:], b[2:])


def test_portions_with_rectangular_masks_equal_single_shot(tmp_path):
    """backend.rs:198-205: a prompt fed in chunks against a growing cache equals one call.
    Here: logits at position i of the whole sequence equal the last logits of the prefix 0..i."""
    cfg, w = P.read_model_dir(make_model_dir(tmp_path, "A"))
    toks = random_prompt(cfg["vocab_size"], 23, 3)
    whole = P.forward_all_positions(cfg, w, toks)
    for i in (0, 6, 22):
        assert torch.allclose(P.forward_all_positions(cfg, w, toks[:i + 1])[-1], whole[i], atol=2e-6)


def test_float64_agrees_with_float32(tmp_path):
    for name in ("A", "B"):
        cfg, w = P.read_model_dir(make_model_dir(tmp_path, name))
        toks = random_prompt(cfg["vocab_size"], 40, 4)
        a = P.forward_all_positions(cfg, w, toks)
        b = P.forward_all_positions(cfg, w, toks, dtype=torch.float64)
        assert float((a - b.float()).abs().max()) < 2e-5


def test_window_hides_old_keys():
    g = torch.Generator().manual_seed(5)
    T, hd = 12, 16
    q, k, v = (torch.randn(T, 1, hd, generator=g) for _ in range(3))
    pos = torch.arange(T)
    w4 = P.causal_attention(q, k, v, 1, 1, pos, window=4)
    for t in (0, 3, 11):
        lo = max(0, t - 3)
        s = (k[lo:t + 1, 0] @ q[t, 0]) / 4.0
        assert torch.allclose(torch.softmax(s, 0) @ v[lo:t + 1, 0], w4[t], atol=1e-5)


def test_argmax_takes_the_lowest_index():
    assert P.argmax_lowest(torch.tensor([1.0, 3.0, 3.0, 2.0, 3.0])) == 1


def test_gumbel_sampling():
    """gpu/mod.rs:3830-3837: temp 0 is greedy whatever the seed; same (params, seed) reproduces."""
    g = torch.Generator().manual_seed(6)
    lg = torch.randn(300, generator=g)
    assert P.gumbel_sample(lg, 0.0, 123) == int(lg.argmax()) == P.gumbel_sample(lg, -1.0, 9)
    a = [P.gumbel_sample(lg, 0.8, P.step_seed(7, n)) for n in range(6)]
    assert a == [P.gumbel_sample(lg, 0.8, P.step_seed(7, n)) for n in range(6)]
    assert len(set(a)) > 1
    assert all(0.0 < P.rand01(5, i) < 1.0 for i in range(1000))
    assert P.step_seed(0xFFFFFFFF, 3) == (0xFFFFFFFF + 3 * 0x9E3779B1) % 2 ** 32


def test_gumbel_sampling_follows_the_distribution():
    lg = torch.tensor([2.0, 1.0, 0.0, -1.0])
    n = 4000
    counts = torch.zeros(4)
    for s in range(n):
        counts[P.gumbel_sample(lg, 1.0, P.hash_u32(s))] += 1
    assert float((counts / n - torch.softmax(lg, 0)).abs().max()) < 0.03


def test_topk_order_with_ties():
    """gpu_btopk_kernel (gpu/mod.rs:3848): value descending, index ascending."""
    lg = torch.tensor([0.5, 2.0, 2.0, -1.0, 2.0, 0.5])
    v, i = P.topk_desc(lg, 4)
    assert i == [1, 2, 4, 0] and v == [2.0, 2.0, 2.0, 0.5]
    assert P.sample_topk(v, i, 0.0, 0, 1.0, 5) == 1
    picks = {P.sample_topk(v, i, 1.0, 2, 1.0, s) for s in range(50)}
    assert picks <= {1, 2} and len(picks) == 2
