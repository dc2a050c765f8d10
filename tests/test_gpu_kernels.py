"""Each CUDA kernel alone against its plain torch statement (``ref_ops``), at sizes other
than the engine configurations': odd widths, head sizes in steps of 16, any head and group
counts, page sizes that are no power of two, row counts around every tile edge."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

from gpu_util import DEV, CpuCacheView, cpu_ctx, make_cache, make_ctx
from ref_ops import RefOps
from zllm_b200.parts.feedforward import interleave_gate_up


@pytest.fixture(scope="module")
def ops():
    from zllm_b200.kernels.ops import CudaOps
    o = CudaOps(DEV)
    o.configure(torch.bfloat16)
    return o


REF = RefOps()


def rnd(shape, dtype, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype)


@pytest.mark.parametrize("wdtype", [torch.float32, torch.bfloat16])
def test_embedding(ops, wdtype):
    table = rnd((517, 72), wdtype, 0)
    tok = torch.tensor([0, 516, 3, 3, 100], dtype=torch.int32)
    out = torch.empty(5, 72, device=DEV)
    ops.embedding(tok.to(DEV), table.to(DEV), out)
    assert torch.equal(out.cpu(), table[tok.long()].float())


@pytest.mark.parametrize("H,T", [(72, 3), (2048, 5), (1000, 1), (8200, 2)])
@pytest.mark.parametrize("wdtype,odtype", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16),
                                           (torch.float32, torch.bfloat16)])
def test_rmsnorm(ops, H, T, wdtype, odtype):
    x = rnd((T, H), torch.float32, 1, 3.0)
    w = (1 + rnd((H,), torch.float32, 2, 0.1)).to(wdtype)
    out = torch.empty(T, H, dtype=odtype, device=DEV)
    ops.rmsnorm(x.to(DEV), w.to(DEV), 1e-6, out)
    want = torch.empty(T, H, dtype=odtype)
    REF.rmsnorm(x, w, 1e-6, want)
    tol = 2e-6 if odtype == torch.float32 else 2 ** -7
    assert float((out.cpu().float() - want.float()).abs().max()) <= tol * float(want.float().abs().max())


@pytest.mark.parametrize("H", [72, 2048, 8200])
def test_rmsnorm_of_chosen_rows(ops, H):
    """The norm of x[rows]: the rows whose logits are wanted go straight to the head's input (a
    row may be named twice, the order is free)."""
    x = rnd((9, H), torch.float32, 1, 3.0)
    w = 1 + rnd((H,), torch.float32, 2, 0.1)
    rows = torch.tensor([8, 0, 3, 3, 5], dtype=torch.int32)
    out = torch.empty(5, H, dtype=torch.bfloat16, device=DEV)
    ops.rmsnorm(x.to(DEV), w.to(DEV), 1e-6, out, rows=rows.to(DEV))
    want = torch.empty(5, H, dtype=torch.bfloat16)
    REF.rmsnorm(x[rows.long()], w, 1e-6, want)
    assert torch.equal(out.cpu(), want) or float((out.cpu().float() - want.float()).abs().max()) <= 2 ** -7 * float(want.float().abs().max())
    whole = torch.empty(9, H, dtype=torch.bfloat16, device=DEV)
    ops.rmsnorm(x.to(DEV), w.to(DEV), 1e-6, whole)
    assert torch.equal(out.cpu(), whole.cpu()[rows.long()])           # the same numbers as the rows of the whole


@pytest.mark.parametrize("M,N", [(3, 264), (5, 40000)])               # the fused product, and the norm as a kernel of its own
def test_linear_normed_of_chosen_rows(ops, M, N):
    from zllm_b200.engine.batch import Workspace
    K = 256
    x = rnd((12, K), torch.float32, 1, 2.0)
    nw = 1 + rnd((K,), torch.float32, 2, 0.1)
    w = rnd((N, K), torch.bfloat16, 3, K ** -0.5)
    rows = torch.tensor([11, 2, 7, 7, 0][:M], dtype=torch.int32)
    ws = Workspace(64, DEV)
    out = torch.zeros(M, N, dtype=torch.float32, device=DEV)
    ops.linear_normed(x.to(DEV), nw.to(DEV), 1e-5, w.to(DEV), out, "store", ws, rows=rows.to(DEV))
    gathered = torch.zeros(M, N, dtype=torch.float32, device=DEV)
    ops.linear_normed(x[rows.long()].contiguous().to(DEV), nw.to(DEV), 1e-5, w.to(DEV), gathered, "store", ws)
    assert torch.equal(out.cpu(), gathered.cpu())
    want = torch.zeros(M, N)
    REF.linear_normed(x, nw, 1e-5, w, want, "store", None, rows=rows)
    assert float((out.cpu() - want).abs().max()) <= 2 ** -7 * max(1.0, float(want.abs().max()))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_silu_mul(ops, dtype):
    a, b = rnd((7, 333), dtype, 3, 2.0), rnd((7, 333), dtype, 4)
    out = torch.empty(7, 333, dtype=dtype, device=DEV)
    ops.silu_mul(a.to(DEV), b.to(DEV), out)
    want = torch.empty(7, 333, dtype=dtype)
    REF.silu_mul(a, b, want)
    assert float((out.cpu().float() - want.float()).abs().max()) <= (1e-6 if dtype == torch.float32 else 2 ** -7 * 4)


LINEAR_SHAPES = [(1, 72, 64), (3, 200, 136), (8, 264, 520), (9, 96, 256), (16, 1000, 72), (17, 136, 2048),
                 (5, 264, 8200), (8, 2048, 16384), (2, 40, 10240),      # few rows, long K: two CTAs share the passes over K
                 (64, 520, 264), (65, 72, 72), (127, 256, 192), (128, 384, 128), (129, 640, 320), (300, 1536, 448),
                 (515, 200, 1024)]


@pytest.mark.parametrize("M,N,K", LINEAR_SHAPES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("mode", ["store", "add", "swiglu"])
def test_linear(ops, M, N, K, dtype, mode):
    x = rnd((M, K), dtype, 5)
    if mode == "swiglu":
        w = interleave_gate_up(rnd((N, K), dtype, 6, K ** -0.5), rnd((N, K), dtype, 7, K ** -0.5))
    else:
        w = rnd((N, K), dtype, 6, K ** -0.5)
    odt = torch.float32 if mode == "add" else dtype
    base = rnd((M, N), odt, 8)
    out = base.clone().to(DEV)
    ops.linear(x.to(DEV), w.to(DEV), out, mode)
    want = base.clone().float()
    REF.linear(x, w, want, mode)           # float32 accumulation, unrounded output
    err = float((out.cpu().float() - want).abs().max())
    ops.check_async_errors()
    scale = float(want.abs().max())
    if dtype == torch.float32:
        assert err <= 2e-5 * max(scale, 1.0)
    else:
        assert err <= (2 ** -8) * max(scale, 1.0) * 1.5     # output rounding to bf16 plus accumulation order


STREAM_SHAPES = [  # rows, N, K, epilogue: what the TMA-fed streaming product takes (9..64 rows), at sizes with one and
    # several weight tiles, K split over clusters of 1 to 8 CTAs, ragged last tiles and k steps
    (12, 4096, 3072, "store"), (9, 2048, 8192, "add"), (16, 8192, 1536, "swiglu"), (17, 48, 24, "store"),
    (33, 3072, 2048, "store"), (40, 2048, 8192, "add"), (64, 1000, 1032, "store"), (64, 4104, 520, "swiglu"),
    (23, 264, 4104, "add"), (32, 30000, 72, "store"),
    # few rows on matrices that are large on both sides (from 5 rows; from one row with 50 M weights and a K of 4096)
    (5, 3072, 3072, "add"), (8, 5120, 3072, "store"), (7, 3072, 8192, "add"), (6, 4096, 3072, "swiglu"),
    (1, 12296, 4096, "store"), (3, 4096, 12296, "add"),
]


@pytest.mark.parametrize("M,N,K,mode", STREAM_SHAPES)
def test_streaming_product(ops, M, N, K, mode):
    dtype = torch.bfloat16
    x = rnd((M, K), dtype, 5)
    if mode == "swiglu":
        w = interleave_gate_up(rnd((N, K), dtype, 6, K ** -0.5), rnd((N, K), dtype, 7, K ** -0.5))
    else:
        w = rnd((N, K), dtype, 6, K ** -0.5)
    assert ops._streams(M, w) or M > 16
    for odt in ((torch.float32,) if mode == "add" else (torch.float32, torch.bfloat16)):
        base = rnd((M, N), odt, 8)
        out = base.clone().to(DEV)
        before = ops.launches
        ops.linear(x.to(DEV), w.to(DEV), out, mode)
        assert ops.launches == before + 1
        ops.check_async_errors()
        want = base.clone().float()
        REF.linear(x, w, want, mode)
        err = float((out.cpu().float() - want).abs().max())
        scale = max(float(want.abs().max()), 1.0)
        assert err <= (2e-5 if odt == torch.float32 else 2 ** -8 * 1.5) * scale, (odt, err)


SPLIT_K_SHAPES = [  # rows, N, K, epilogue: few tiles, so the many-row kernel takes tiles of 128 weight rows, splits K (2..16
    # slices, the last slice ragged or empty) and a second kernel sums the slices in order
    (128, 2048, 8192, "add"), (200, 2048, 2048, "add"), (70, 3072, 2048, "store"), (512, 2048, 8192, "add"),
    (300, 264, 4104, "store"), (96, 520, 1352, "swiglu"), (130, 1000, 2056, "store"),
]


STREAM_K_SHAPES = [  # more tiles than SMs, so that the tile width is chosen by the waves it makes (192, 195, 320 tiles of
    # 256 weight rows, the last ones ragged; 128 tiles of a long K)
    (2048, 3072, 2048, "store"), (1900, 3080, 1032, "store"), (1280, 4096, 1024, "swiglu"), (2048, 2048, 8192, "add"),
    (2047, 3072, 2048, "add"),
]


@pytest.mark.parametrize("pair", [-1, 0])
@pytest.mark.parametrize("tile", [0, 128, 192, 256])
@pytest.mark.parametrize("M,N,K,mode", SPLIT_K_SHAPES + STREAM_K_SHAPES +
                         [(700, 1288, 520, "store"), (1100, 640, 264, "swiglu"), (640, 904, 1032, "add")])
def test_many_row_product_with_split_k(ops, M, N, K, mode, tile, pair):
    """``tile``: the kernel's tile width forced to 128, 192 or 256 weight rows (0: chosen by the sizes),
    so that both shapes run at every size.  ``pair``: -1, pairs of CTAs on tiles of 256 rows wherever
    there is more than one row tile (a last row tile without a partner included: 300, 640, 700,
    1100, 1900 rows); 0, single CTAs on tiles of 128 rows everywhere."""
    lib = ops.lib("gemm_tc")
    assert lib.zllm_gemm_tc_force_tile(tile) == 0 and lib.zllm_gemm_tc_force_pair(pair) == 0
    try:
        _many_row_product(ops, M, N, K, mode)
    finally:
        lib.zllm_gemm_tc_force_tile(0)
        lib.zllm_gemm_tc_force_pair(-1)


@pytest.mark.parametrize("slices", [1, 3, 5, 32])
@pytest.mark.parametrize("M,N,K,mode", [(128, 2048, 2048, "add"), (300, 264, 4104, "store"), (512, 2048, 8192, "add"),
                                        (96, 520, 1352, "swiglu"), (1024, 2048, 8192, "add")])
def test_many_row_product_with_forced_slices(ops, M, N, K, mode, slices):
    """The number of slices of K is chosen by a model of the kernel's time; here it is forced: one
    slice, counts that do not divide the k steps (ragged and empty last slices), and more than
    the product allows (clamped to one slice per four k steps and to the scratch)."""
    lib = ops.lib("gemm_tc")
    assert lib.zllm_gemm_tc_force_splits(slices) == 0
    try:
        _many_row_product(ops, M, N, K, mode)
    finally:
        lib.zllm_gemm_tc_force_splits(0)


def _many_row_product(ops, M, N, K, mode):
    dtype = torch.bfloat16
    x = rnd((M, K), dtype, 5)
    if mode == "swiglu":
        w = interleave_gate_up(rnd((N, K), dtype, 6, K ** -0.5), rnd((N, K), dtype, 7, K ** -0.5))
    else:
        w = rnd((N, K), dtype, 6, K ** -0.5)
    for odt in ((torch.float32,) if mode == "add" else (torch.float32, torch.bfloat16)):
        base = rnd((M, N), odt, 8)
        outs = []
        for _ in range(2):                      # twice: the sum over the slices has a fixed order
            out = base.clone().to(DEV)
            ops.linear(x.to(DEV), w.to(DEV), out, mode)
            ops.check_async_errors()
            outs.append(out.cpu())
        assert torch.equal(outs[0], outs[1])
        want = base.clone().float()
        REF.linear(x, w, want, mode)
        err = float((outs[0].float() - want).abs().max())
        scale = max(float(want.abs().max()), 1.0)
        assert err <= (2e-5 if odt == torch.float32 else 2 ** -8 * 1.5) * scale, (odt, err)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_linear_plain_matches_too(ops, dtype):
    x, w = rnd((33, 100), dtype, 1), rnd((77, 100), dtype, 2, 0.1)
    out = torch.zeros(33, 77, dtype=dtype, device=DEV)
    ops.linear_plain(x.to(DEV), w.to(DEV), out, "store")
    assert float((out.cpu().float() - x.float() @ w.float().T).abs().max()) < (1e-5 if dtype == torch.float32 else 0.02)


def test_float32_products_do_not_depend_on_the_batch(ops):
    """The 32-bit path: a row's result is bit-identical whatever else is in the batch."""
    x, w = rnd((130, 200), torch.float32, 1).to(DEV), rnd((300, 200), torch.float32, 2).to(DEV)
    full = torch.empty(130, 300, device=DEV)
    ops.linear(x, w, full, "store")
    for rows in ([0], [64, 65], list(range(100, 130))):
        part = torch.empty(len(rows), 300, device=DEV)
        ops.linear(x[rows].contiguous(), w, part, "store")
        assert torch.equal(part, full[rows])


ROPE_CASES = [(4, 2, 16, 16, False), (3, 1, 32, 32, True), (5, 5, 48, 32, False), (8, 2, 64, 64, False), (2, 1, 128, 128, True)]


@pytest.mark.parametrize("nq,nkv,hd,rd,inter", ROPE_CASES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rope_and_cache_write(ops, nq, nkv, hd, rd, inter, dtype):
    from zllm_b200.parts.rotary import Rotary
    from zllm_b200.models.decoder import Runtime
    rot = Rotary(rd, 10000.0, 200, interleaved=inter)
    rot.bind(Runtime(dtype, torch.device(DEV), ops))
    bs = 6
    cm = make_cache(nkv, hd, bs, 40, 3, 120, dtype)
    s0, s1 = cm.admit(), cm.admit()
    make_ctx(cm, [(s0, 11)])                                  # s0 already holds 11 positions
    ctx = make_ctx(cm, [(s0, 9), (s1, 1), ])
    T = 10
    qkv = rnd((T, (nq + 2 * nkv) * hd), dtype, 9)
    dq = qkv.clone().to(DEV)
    view = cm.view(0)
    view.k_pages.zero_(); view.v_pages.zero_()
    ops.rope_kv_store(dq, ctx, rot.rotary(), view, nq, nkv, hd, True)
    # plain
    import copy
    crot = copy.copy(rot.rotary()); crot.cos = crot.cos.cpu(); crot.sin = crot.sin.cpu()
    cview = CpuCacheView(view); cview.k_pages.zero_(); cview.v_pages.zero_()
    want = qkv.clone().float()
    REF.rope_kv_store(want, cpu_ctx(ctx), crot, cview, nq, nkv, hd, True)
    tol = 1e-6 if dtype == torch.float32 else 2 ** -7
    sc = float(want.abs().max())
    assert float((dq.cpu().float() - want).abs().max()) <= tol * sc
    assert float((view.k_pages.float().cpu() - cview.k_pages).abs().max()) <= tol * sc
    assert float((view.v_pages.float().cpu() - cview.v_pages).abs().max()) <= tol * sc
    assert float(cview.k_pages.abs().sum()) > 0
    # without store nothing is written
    view.k_pages.zero_()
    ops.rope_kv_store(qkv.clone().to(DEV), ctx, rot.rotary(), view, nq, nkv, hd, False)
    assert float(view.k_pages.abs().sum()) == 0.0


ATT_CASES = [  # nq, nkv, hd, page size, window
    (4, 2, 16, 16, None), (3, 1, 32, 8, None), (8, 2, 64, 16, None), (32, 8, 64, 16, None), (6, 6, 48, 5, None),
    (16, 2, 128, 16, None), (5, 1, 80, 7, None), (8, 2, 64, 16, 37), (4, 4, 96, 12, 20), (8, 1, 112, 16, None),
    (2, 1, 256, 16, None),
    # page sizes and groups of the TMA / tcgen05 kernels (head sizes 64 and 128): one box per page, pages
    # smaller and larger than a block of keys, a group of one head, the largest group
    (8, 2, 64, 8, None), (8, 2, 64, 32, None), (6, 6, 64, 64, None), (4, 2, 64, 128, None), (8, 1, 64, 256, None),
    (4, 2, 128, 32, None), (8, 1, 128, 128, None),
]


@pytest.mark.parametrize("nq,nkv,hd,bs,window", ATT_CASES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_mixed_batch(ops, nq, nkv, hd, bs, window, dtype):
    """Decoded rows at long and short contexts beside portions that start anywhere."""
    cm = make_cache(nkv, hd, bs, 1300 // bs + 12, 6, 700, dtype, window)
    slots = [cm.admit() for _ in range(5)]
    view = cm.view(0)
    g = torch.Generator().manual_seed(11)
    view.k_pages.copy_(torch.randn(view.k_pages.shape, generator=g).to(dtype))
    view.v_pages.copy_(torch.randn(view.v_pages.shape, generator=g).to(dtype))
    # earlier contents of every request (pages handed out in interleaved order, so tables are scattered)
    for rounds in range(3):
        for s, n in zip(slots, (100, 3, 40, 170, 1)):
            make_ctx(cm, [(s, n)])
    ctx = make_ctx(cm, [(slots[0], 1), (slots[1], 70), (slots[2], 1), (slots[3], 2), (slots[4], 130), ])
    T = ctx.T
    qkv = rnd((T, (nq + 2 * nkv) * hd), dtype, 12)
    out = torch.full((T, nq * hd), 7.0, dtype=dtype, device=DEV)
    scale = 1.0 / math.sqrt(hd)
    ops.paged_attention(qkv.to(DEV), out, ctx, view, nq, nkv, hd, scale, window)
    want = torch.zeros(T, nq * hd)
    REF.paged_attention(qkv.float(), want, cpu_ctx(ctx), CpuCacheView(view), nq, nkv, hd, scale, window)
    err = float((out.cpu().float() - want).abs().max())
    assert err <= (2e-5 if dtype == torch.float32 else 0.02), err


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_finds_a_far_key_among_hundreds(ops, dtype):
    """One key far back is made to stand out (query and that key scaled up): the output must be
    that key's value, whatever page it lies in.  Random data would hide a missed key."""
    nq, nkv, hd, bs = 8, 2, 64, 16
    cm = make_cache(nkv, hd, bs, 80, 2, 1100, dtype)
    s = cm.admit()
    view = cm.view(0)
    g = torch.Generator().manual_seed(13)
    view.k_pages.copy_((torch.randn(view.k_pages.shape, generator=g) * 0.1).to(dtype))
    view.v_pages.copy_(torch.randn(view.v_pages.shape, generator=g).to(dtype))
    make_ctx(cm, [(s, 1000)])
    ctx = make_ctx(cm, [(s, 1)])                 # one decoded row at position 1000
    for far in (0, 15, 16, 255, 256, 257, 511, 777, 999):
        page = int(view.block_table[s, far // bs])
        qkv = torch.zeros(1, (nq + 2 * nkv) * hd)
        direction = torch.randn(hd, generator=g)
        direction /= direction.norm()
        saved = view.k_pages[page, :, far % bs].clone()
        view.k_pages[page, :, far % bs] = (direction * 40).to(dtype)
        qkv[0, :nq * hd] = (direction * 40).repeat(nq)
        out = torch.zeros(1, nq * hd, dtype=dtype, device=DEV)
        ops.paged_attention(qkv.to(dtype).to(DEV), out, ctx, view, nq, nkv, hd, 1.0, None)
        got = out.float().cpu().reshape(nq, hd)
        for h in range(nq):
            v = view.v_pages[page, h // (nq // nkv), far % bs].float().cpu()
            assert float((got[h] - v).abs().max()) < 0.02, f"far key {far} head {h}"
        view.k_pages[page, :, far % bs] = saved


@pytest.mark.parametrize("hd", [64, 80, 128])                 # 80: the mma.sync kernel, the others by TMA
@pytest.mark.parametrize("n_ctx", [8200, 9100, 65500, 66000, 70100])    # 33, 36, 256, 258 and 274 splits of 256 keys
def test_decode_attention_over_many_splits(ops, hd, n_ctx):
    """Up to 32 splits are merged by one warp per (row, head), up to 255 by a block, from 256 on in
    two passes (groups of 32, then the groups): eight full groups, a ninth group of two splits and
    one of eighteen; beside a short row in the same launch (one split, one group).  One far key
    per long row is made to stand out as well."""
    nq, nkv, bs, dtype = 4, 2, 16, torch.bfloat16
    cm = make_cache(nkv, hd, bs, n_ctx // bs + 40, 2, n_ctx + 300, dtype)
    a, b = cm.admit(), cm.admit()
    view = cm.view(0)
    g = torch.Generator().manual_seed(17)
    view.k_pages.copy_((torch.randn(view.k_pages.shape, generator=g) * 0.3).to(dtype))
    view.v_pages.copy_(torch.randn(view.v_pages.shape, generator=g).to(dtype))
    for slot, n in ((a, n_ctx - 1), (b, 200)):                # earlier contents: pages handed out, lengths advanced
        assert cm.ensure(slot, n)
        cm.advance(slot, n)
    ctx = make_ctx(cm, [(a, 1), (b, 1)])
    qkv = rnd((2, (nq + 2 * nkv) * hd), dtype, 18)
    scale = 1.0 / math.sqrt(hd)
    out = torch.zeros(2, nq * hd, dtype=dtype, device=DEV)
    ops.paged_attention(qkv.to(DEV), out, ctx, view, nq, nkv, hd, scale, None)
    want = torch.zeros(2, nq * hd)
    REF.paged_attention(qkv.float(), want, cpu_ctx(ctx), CpuCacheView(view), nq, nkv, hd, scale, None)
    assert float((out.cpu().float() - want).abs().max()) <= 0.02
    # a far key in the last group's last split, and one in the first split
    for far in (n_ctx - 300, 5):
        page = int(view.block_table[a, far // bs])
        direction = torch.randn(hd, generator=g)
        direction /= direction.norm()
        saved = view.k_pages[page, :, far % bs].clone()
        view.k_pages[page, :, far % bs] = (direction * 40).to(dtype)
        q2 = qkv.clone()
        q2[0, :nq * hd] = (direction * 40).repeat(nq).to(dtype)
        ops.paged_attention(q2.to(DEV), out, ctx, view, nq, nkv, hd, 1.0, None)
        got = out[0].float().cpu().reshape(nq, hd)
        for h in range(nq):
            v = view.v_pages[page, h // (nq // nkv), far % bs].float().cpu()
            assert float((got[h] - v).abs().max()) < 0.02, f"far key {far} head {h}"
        view.k_pages[page, :, far % bs] = saved


@pytest.mark.parametrize("slope", [0.0, 0.5, 3.0, -2.0])
@pytest.mark.parametrize("hd,nq,nkv", [(64, 8, 2), (128, 4, 1)])
def test_prefill_attention_when_the_maximum_keeps_moving(ops, slope, hd, nq, nkv):
    """The scores of a row grow (or fall) with the key's position at a chosen rate, so the running
    maximum of the softmax moves from block to block: slowly (the kernel may keep a stale reference),
    fast (it has to rescale what it has summed at every block) or never (the first block holds it).
    A portion of 300 rows behind a prefix of 500; random data would leave the maximum where it is."""
    dtype = torch.bfloat16
    bs = 16
    cm = make_cache(nkv, hd, bs, 70, 2, 900, dtype)
    s = cm.admit()
    view = cm.view(0)
    g = torch.Generator().manual_seed(15)
    make_ctx(cm, [(s, 500)])
    ctx = make_ctx(cm, [(s, 300)])
    direction = torch.randn(hd, generator=g)
    direction /= direction.norm()
    k = torch.randn(view.k_pages.shape, generator=g) * 0.3
    for pos in range(800):
        page = int(view.block_table[s, pos // bs])
        k[page, :, pos % bs] += direction * slope * pos / math.sqrt(hd) * 8.0 / 40.0
    view.k_pages.copy_(k.to(dtype))
    view.v_pages.copy_(torch.randn(view.v_pages.shape, generator=g).to(dtype))
    qkv = torch.randn(300, (nq + 2 * nkv) * hd, generator=g) * 0.3
    qkv[:, :nq * hd] += (direction * 40.0).repeat(nq)
    qkv = qkv.to(dtype)
    out = torch.zeros(300, nq * hd, dtype=dtype, device=DEV)
    scale = 1.0 / math.sqrt(hd)
    ops.paged_attention(qkv.to(DEV), out, ctx, view, nq, nkv, hd, scale, None)
    ops.check_async_errors()
    want = torch.zeros(300, nq * hd)
    REF.paged_attention(qkv.float(), want, cpu_ctx(ctx), CpuCacheView(view), nq, nkv, hd, scale, None)
    err = float((out.cpu().float() - want).abs().max())
    assert err <= 0.03, err


@pytest.mark.parametrize("hd", [64, 128])
def test_prefill_attention_of_a_partial_tile_does_not_depend_on_what_ran_before(ops, hd):
    """A portion of 69 rows fills half a tile: the tile's other rows are another request's queries
    (large ones here), and the key boxes beyond position 68 are never loaded.  Whatever an earlier
    kernel left in shared memory there must not reach the real rows (not even their rounding, by
    way of a decision the rows of a warp take together): the same step gives the same bits before
    and after attention over large and very different data."""
    dtype = torch.bfloat16
    nq, nkv, bs = 8, 2, 16
    scale = 1.0 / math.sqrt(hd)
    g = torch.Generator().manual_seed(21)
    cm = make_cache(nkv, hd, bs, 200, 3, 1400, dtype)
    view = cm.view(0)
    view.k_pages.copy_(torch.randn(view.k_pages.shape, generator=g).to(dtype))
    view.v_pages.copy_(torch.randn(view.v_pages.shape, generator=g).to(dtype))
    s, s_b = cm.admit(), cm.admit()
    ctx = make_ctx(cm, [(s, 69), (s_b, 100)])
    qkv = torch.randn(169, (nq + 2 * nkv) * hd, generator=g) * 0.5
    qkv[69:] *= 8.0
    qkv = qkv.to(dtype).to(DEV)
    outs = []
    for big in (30.0, -50.0, None):
        out = torch.zeros(169, nq * hd, dtype=dtype, device=DEV)
        ops.paged_attention(qkv, out, ctx, view, nq, nkv, hd, scale, None)
        outs.append(out.cpu().clone())
        if big is None:
            break
        # dirty every SM's shared memory: 1,024 rows of scores of the size ``big``
        cm2 = make_cache(nkv, hd, bs, 80, 2, 1100, dtype)
        s2 = cm2.admit()
        v2 = cm2.view(0)
        v2.k_pages.fill_(big)
        v2.v_pages.fill_(big)
        ctx2 = make_ctx(cm2, [(s2, 1024)])
        q2 = torch.full((1024, (nq + 2 * nkv) * hd), abs(big), dtype=dtype, device=DEV)
        ops.paged_attention(q2, torch.zeros(1024, nq * hd, dtype=dtype, device=DEV), ctx2, v2, nq, nkv, hd, scale, None)
    ops.check_async_errors()
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
    want = torch.zeros(169, nq * hd)
    REF.paged_attention(qkv.cpu().float(), want, cpu_ctx(ctx), CpuCacheView(view), nq, nkv, hd, scale, None)
    assert float((outs[0].float() - want).abs().max()) <= 0.03


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_window_edge(ops, dtype):
    """The key just outside the window is made dominant: it must NOT be seen; the one just
    inside must."""
    nq, nkv, hd, bs, window = 4, 1, 32, 8, 21
    cm = make_cache(nkv, hd, bs, 40, 2, 300, dtype, window)
    s = cm.admit()
    view = cm.view(0)
    g = torch.Generator().manual_seed(14)
    for n in (90, 1, 1, 1, 5):
        make_ctx(cm, [(s, n)])
    view.k_pages.copy_((torch.randn(view.k_pages.shape, generator=g) * 0.1).to(dtype))
    view.v_pages.copy_(torch.randn(view.v_pages.shape, generator=g).to(dtype))
    ctx = make_ctx(cm, [(s, 1)])
    p = int(ctx.positions[0])
    direction = torch.ones(hd) / math.sqrt(hd)
    qkv = torch.zeros(1, (nq + 2) * hd)
    qkv[0, :nq * hd] = (direction * 40).repeat(nq)
    for key, visible in ((p - window, False), (p - window + 1, True)):
        page = int(view.block_table[s, key // bs])
        if page < 0:
            assert not visible
            continue
        saved = view.k_pages[page, 0, key % bs].clone()
        view.k_pages[page, 0, key % bs] = (direction * 40).to(dtype)
        out = torch.zeros(1, nq * hd, dtype=dtype, device=DEV)
        ops.paged_attention(qkv.to(dtype).to(DEV), out, ctx, view, nq, nkv, hd, 1.0, window)
        v = view.v_pages[page, 0, key % bs].float().cpu()
        close = float((out.float().cpu().reshape(nq, hd)[0] - v).abs().max()) < 0.02
        assert close == visible, f"key {key} visible={visible}"
        view.k_pages[page, 0, key % bs] = saved


def test_sampling_kernels(ops):
    import plain_llama as P
    g = torch.Generator().manual_seed(15)
    V = 5003
    lg = torch.randn(6, V, generator=g)
    lg[1, 4000] = lg[1, 77] = 9.0              # a tie: the lowest index wins
    lg[2] = 0.0                                # all equal: token 0
    temps = torch.tensor([0.0, 0.0, 0.0, 0.8, 1.3, 0.8])
    seeds = torch.tensor([1, 2, 3, 12345, 99, 12345], dtype=torch.int64).to(torch.int32)
    out = torch.zeros(6, dtype=torch.int32, device=DEV)
    ops.sample(lg.to(DEV), temps.to(DEV), seeds.to(DEV), out)
    got = out.cpu().tolist()
    assert got[0] == int(lg[0].argmax()) and got[1] == 77 and got[2] == 0
    for r in (3, 4, 5):
        assert got[r] == P.gumbel_sample(lg[r], float(temps[r]), int(seeds[r]))
    vals = torch.zeros(6, 64, device=DEV)
    idx = torch.zeros(6, 64, dtype=torch.int32, device=DEV)
    ops.topk(lg.to(DEV), 64, vals, idx)
    for r in range(6):
        v, i = P.topk_desc(lg[r], 64)
        assert idx[r].cpu().tolist() == i and vals[r].cpu().tolist() == v
    # a large vocabulary: many blocks per row, the last one to arrive picks the winner
    big = torch.randn(3, 40003, generator=g)
    big[0, 39999] = big[0, 123] = 11.0
    tb, sb = torch.tensor([0.0, 0.9, 0.0]), torch.tensor([0, 77, 5], dtype=torch.int32)
    ob = torch.zeros(3, dtype=torch.int32, device=DEV)
    for _ in range(2):                          # twice: the arrival counters must be back at zero
        ops.sample(big.to(DEV), tb.to(DEV), sb.to(DEV), ob)
        gb = ob.cpu().tolist()
        assert gb[0] == 123 and gb[2] == int(big[2].argmax())
        assert gb[1] == P.gumbel_sample(big[1], 0.9, 77)
    small = torch.tensor([[1.0, 5.0, 5.0]])
    v3 = torch.zeros(1, 5, device=DEV); i3 = torch.zeros(1, 5, dtype=torch.int32, device=DEV)
    ops.topk(small.to(DEV), 5, v3, i3)
    assert i3.cpu().tolist() == [[1, 2, 0, -1, -1]]


def test_topk_in_two_stages_and_the_draw_among_the_candidates(ops):
    """A vocabulary large enough for the two-stage top-k (64 stretches per row, then a merge), with
    ties across stretches and rows with fewer than 64 finite entries; then the device's draw among
    the candidates against the host's (sampling/sampler.py::sample_from_pool), parameter by parameter."""
    import plain_llama as P
    from zllm_b200.sampling.sampler import sample_from_pool
    from zllm_b200.sampling.params import SamplingParams
    g = torch.Generator().manual_seed(21)
    V = 40003
    lg = torch.randn(9, V, generator=g) * 3
    lg[0, 5] = lg[0, 20000] = lg[0, 39990] = 50.0          # ties in three different stretches
    lg[1, :] = float("-inf"); lg[1, 777] = 1.0; lg[1, 30000] = 2.0      # two finite entries
    lg[2, 1000:1070] = 40.0                                 # more than 64 equal values in one stretch
    vals = torch.zeros(9, 64, device=DEV)
    idx = torch.zeros(9, 64, dtype=torch.int32, device=DEV)
    for _ in range(2):
        before = ops.launches
        ops.topk(lg.to(DEV), 64, vals, idx)
        assert ops.launches == before + 4                   # group maxima, stretches, two merges
        for r in range(9):
            v, i = P.topk_desc(lg[r], 64)
            v = v + [-3.0e38] * (64 - len(v)); i = i + [-1] * (64 - len(i))
            assert idx[r].cpu().tolist() == i, r
            assert [float(x) for x in vals[r].cpu()] == [float(torch.tensor(x, dtype=torch.float32)) for x in v]
    cases = [(0.8, 0, 0.9), (1.3, 5, 1.0), (0.7, 40, 0.5), (2.0, 64, 0.999), (0.01, 3, 0.3), (1.0, 1, 1.0), (0.9, 0, 0.05),
             (0.0, 7, 0.9), (1.1, 10, 0.0)]
    for trial in range(20):
        seeds = [int(x) for x in torch.randint(0, 2 ** 31 - 1, (9,), generator=g)]
        ptemp = torch.tensor([c[0] for c in cases], dtype=torch.float64)
        topk = torch.tensor([c[1] for c in cases], dtype=torch.int32)
        topp = torch.tensor([c[2] for c in cases], dtype=torch.float64)
        out = torch.full((9,), -7, dtype=torch.int32, device=DEV)
        ops.pool_draw(vals, idx, ptemp.to(DEV), topk.to(DEV), topp.to(DEV), torch.tensor(seeds, dtype=torch.int32).to(DEV), out)
        got = out.cpu().tolist()
        hv, hi = vals.cpu().tolist(), idx.cpu().tolist()
        for r, (t, k, pp) in enumerate(cases):
            if t <= 0.0:
                assert got[r] == -7                         # not a pool row: left as it was
            else:
                want = sample_from_pool(hv[r], hi[r], SamplingParams(temperature=t, top_k=k, top_p=pp), seeds[r])
                assert got[r] == want, (trial, r)


def test_kernels_refuse_what_they_cannot_run(ops):
    from zllm_b200.errors import BackendError
    x = torch.zeros(4, 64, device=DEV)
    with pytest.raises(BackendError):
        ops.linear(x, torch.zeros(8, 63, device=DEV), torch.zeros(4, 8, device=DEV), "store")
    with pytest.raises(BackendError):
        ops.linear(x.bfloat16(), torch.zeros(8, 64, device=DEV).bfloat16(), torch.zeros(4, 8, device=DEV).bfloat16(), "add")
    with pytest.raises(BackendError):
        ops.rmsnorm(x.t(), torch.ones(64, device=DEV), 1e-5, torch.zeros(64, 4, device=DEV))   # not contiguous
    with pytest.raises(BackendError):
        ops.embedding(torch.zeros(4, dtype=torch.int64, device=DEV), x, torch.zeros(4, 64, device=DEV))


@pytest.mark.parametrize("M", [1, 5, 8, 9, 16, 17, 40])
@pytest.mark.parametrize("N,K,mode", [(72, 64, "store"), (136, 200, "add"), (96, 264, "swiglu"), (2048, 2304, "store"),
                                      (264, 4104, "add"), (1000, 520, "store")])
@pytest.mark.parametrize("wdtype", [torch.float32, torch.bfloat16])
def test_linear_with_norm_prologue(ops, M, N, K, mode, wdtype):
    """rmsnorm folded into the product (decode batches) against norm-then-product."""
    from gpu_util import DEV
    from zllm_b200.engine.batch import Workspace
    x = rnd((M, K), torch.float32, 21, 3.0)
    nw = (1 + rnd((K,), torch.float32, 22, 0.2)).to(wdtype)
    w = rnd((N, K), torch.bfloat16, 23, K ** -0.5)
    if mode == "swiglu":
        w = interleave_gate_up(w, rnd((N, K), torch.bfloat16, 24, K ** -0.5))
    odt = torch.float32 if mode == "add" else torch.bfloat16
    base = rnd((M, N), odt, 25)
    out = base.clone().to(DEV)
    ops.linear_normed(x.to(DEV), nw.to(DEV), 1e-5, w.to(DEV), out, mode, Workspace(64, DEV))
    want = base.clone().float()
    h = torch.empty(M, K)
    REF.rmsnorm(x, nw, 1e-5, h)
    REF.linear(h, w, want, mode)
    err = float((out.cpu().float() - want).abs().max())
    assert err <= 2 ** -7 * max(1.0, float(want.abs().max())), err


@pytest.mark.parametrize("M", [1, 3, 8, 13, 16, 20, 70, 200, 333])      # 70 and more: the epilogue of the tensor-core product
@pytest.mark.parametrize("nq,nkv,hd,inter", [(4, 2, 16, False), (3, 1, 32, True), (8, 2, 64, False), (2, 1, 128, False),
                                             (5, 5, 48, True), (5, 1, 64, False), (3, 3, 128, False)])
@pytest.mark.parametrize("with_norm", [False, True])
def test_qkv_product_with_rope_and_cache_write(ops, M, nq, nkv, hd, inter, with_norm, monkeypatch):
    """The fused QKV product (norm prologue, rotation and cache write in the epilogue) against
    the composition of the separate kernels' plain statements.  The engine sends only products of
    thousands of rows to the tensor-core kernel's fused epilogue (where it pays); here the limit
    is lowered so that 70, 200 and 333 rows take it: single CTAs and pairs, a last row tile
    without a partner, portions that start mid-page."""
    import copy
    monkeypatch.setattr(ops, "ROPE_IN_PRODUCT_MIN_ROWS", 65)
    from zllm_b200.engine.batch import Workspace
    from zllm_b200.models.decoder import Runtime
    from zllm_b200.parts.rotary import Rotary
    dtype = torch.bfloat16
    H = 200
    rot = Rotary(hd, 10000.0, 300, interleaved=inter)
    rot.bind(Runtime(dtype, torch.device(DEV), ops))
    bs = 6
    if M <= 20:
        cm = make_cache(nkv, hd, bs, 500, M + 1, 200, dtype)
        slots = [cm.admit() for _ in range(M)]
        for i, s in enumerate(slots):
            make_ctx(cm, [(s, 3 + 5 * i)])               # every request at another position
        ctx = make_ctx(cm, [(s, 1) for s in slots])
    else:
        # many rows: three portions that start anywhere (a page's edge, mid-page) beside two decoded rows
        cm = make_cache(nkv, hd, bs, 500, 6, 280, dtype)
        slots = [cm.admit() for _ in range(5)]
        for s, n in zip(slots, (12, 5, 30, 7, 1)):
            make_ctx(cm, [(s, n)])
        a = (M - 2) // 3
        ctx = make_ctx(cm, [(slots[0], a), (slots[1], 1), (slots[2], a), (slots[3], 1), (slots[4], M - 2 - 2 * a)])
        assert ctx.T == M
    N = (nq + 2 * nkv) * hd
    w = rnd((N, H), dtype, 31, H ** -0.5)
    x32 = rnd((M, H), torch.float32, 32, 2.0)
    nw = 1 + rnd((H,), torch.float32, 33, 0.2)
    view = cm.view(0)
    view.k_pages.zero_(); view.v_pages.zero_()
    qkv = torch.zeros(M, N, dtype=dtype, device=DEV)
    ws = Workspace(64, DEV)
    if with_norm:
        ops.qkv_rope_store(x32.to(DEV), (nw.to(DEV), 1e-6), w.to(DEV), qkv, ctx, rot.rotary(), view, nq, nkv, hd, True, ws)
        xin = torch.empty(M, H)
        REF.rmsnorm(x32, nw, 1e-6, xin)
    else:
        xin = x32.to(dtype)
        ops.qkv_rope_store(xin.to(DEV), None, w.to(DEV), qkv, ctx, rot.rotary(), view, nq, nkv, hd, True, ws)
        xin = xin.float()
    crot = copy.copy(rot.rotary()); crot.cos = crot.cos.cpu(); crot.sin = crot.sin.cpu()
    cview = CpuCacheView(view); cview.k_pages.zero_(); cview.v_pages.zero_()
    want = torch.zeros(M, N)
    REF.linear(xin, w.float(), want, "store")
    REF.rope_kv_store(want, cpu_ctx(ctx), crot, cview, nq, nkv, hd, True)
    sc = max(1.0, float(want.abs().max()))
    qk = (nq + nkv) * hd                                  # q and k are compared in the buffer, v in the cache
    assert float((qkv.cpu().float()[:, :qk] - want[:, :qk]).abs().max()) <= 2 ** -7 * sc
    assert float((view.k_pages.float().cpu() - cview.k_pages).abs().max()) <= 2 ** -7 * sc
    assert float((view.v_pages.float().cpu() - cview.v_pages).abs().max()) <= 2 ** -7 * sc
    assert float(cview.k_pages.abs().sum()) > 0 and float(cview.v_pages.abs().sum()) > 0


# ---- bounded waits: the give-up path of each kernel family -----------------------------------
def _run_family(ops, family):
    """One ordinary launch of the family's kernel; returns (got, want, tolerance)."""
    g = torch.Generator().manual_seed(21)
    if family in ("gemm_tc", "gemm_stream"):
        M = 300 if family == "gemm_tc" else 40
        N, K = 512, 1024
        x, w = rnd((M, K), torch.bfloat16, 31), rnd((N, K), torch.bfloat16, 32, K ** -0.5)
        out = torch.zeros(M, N, dtype=torch.float32, device=DEV)
        ops.linear(x.to(DEV), w.to(DEV), out, "store")
        want = torch.zeros(M, N)
        REF.linear(x, w, want, "store")
        return out, want, 2 ** -8 * 1.5 * max(1.0, float(want.abs().max()))
    nq, nkv, hd, bs = 8, 2, 64, 16
    cm = make_cache(nkv, hd, bs, 64, 2, 700, torch.bfloat16)
    s = cm.admit()
    view = cm.view(0)
    view.k_pages.copy_(torch.randn(view.k_pages.shape, generator=g).to(torch.bfloat16))
    view.v_pages.copy_(torch.randn(view.v_pages.shape, generator=g).to(torch.bfloat16))
    make_ctx(cm, [(s, 300)])
    ctx = make_ctx(cm, [(s, 1)] if family == "attention_decode_tma" else [(s, 150)])
    T = ctx.T
    qkv = rnd((T, (nq + 2 * nkv) * hd), torch.bfloat16, 33)
    out = torch.zeros(T, nq * hd, dtype=torch.bfloat16, device=DEV)
    ops.paged_attention(qkv.to(DEV), out, ctx, view, nq, nkv, hd, 0.125, None)
    want = torch.zeros(T, nq * hd)
    REF.paged_attention(qkv.float(), want, cpu_ctx(ctx), CpuCacheView(view), nq, nkv, hd, 0.125, None)
    return out, want, 0.02


@pytest.mark.parametrize("family", ["gemm_tc", "gemm_stream", "attention_decode_tma", "attention_prefill_tc"])
def test_a_wait_that_runs_out_is_reported_and_the_kernel_recovers(ops, family):
    """The kernels with mbarrier waits bound every wait.  Here the family's producer is told to
    issue no copy at all and the limit is a few hundred polls, so every wait for data runs out
    with nothing in flight: the kernel must return by itself, the error must reach the host (the
    device flag and its pinned mirror), and the next ordinary launch must be right again."""
    from zllm_b200.errors import BackendError
    got, want, tol = _run_family(ops, family)                     # an ordinary launch first
    assert float((got.float().cpu() - want).abs().max()) <= tol
    ops.check_async_errors()
    ops.set_wait_test_hook(family, limit=300, skip_loads=True)
    try:
        _run_family(ops, family)                                  # returns although nothing ever arrives
        torch.cuda.synchronize()
        with pytest.raises(BackendError, match="bounded wait ran out"):
            ops.raise_if_a_wait_gave_up()                         # seen through the pinned mirror, no copy
    finally:
        ops.set_wait_test_hook(family, limit=0, skip_loads=False)
    ops.check_async_errors()                                      # reading cleared the flags
    assert not bool(ops._error_words.any())
    got, want, tol = _run_family(ops, family)                     # the same kernel, right again
    assert float((got.float().cpu() - want).abs().max()) <= tol
    ops.check_async_errors()
