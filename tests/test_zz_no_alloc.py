"""The entry point for callers that cannot allocate device memory
(``zllm_attention_decode_bf16_noalloc``, csrc/attention_noalloc.h): called through its
exported C symbol and compared with the regular entry point and with the plain statement of
attention, twice in a row, at three head sizes and with a window.

Such callers exist: code running inside a stream capture or under a locked memory pool, a
plug-in that is handed only input and output buffers, a latency-critical loop that must stay
away from the allocator.  For them the kernel's scratch (per-split partial results) sits in
a fixed 16 MiB array inside the library instead of in buffers the caller provides.

This file is named so that pytest collects it last: if it failed, a run that stops at the
first failure has already run every other test.  It passes alone in a fresh process and after
the others (the first call on the device does the one-time address lookup)."""
import ctypes
import math
from ctypes import c_float, c_int, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu

from gpu_util import DEV, make_cache, make_ctx

TOO_LARGE = 10002


def ptr(t):
    return c_void_p(t.data_ptr())


def call_noalloc(lib, qkv, out, ctx, view, nq, nkv, hd, scale, window, n_splits, n_rows=None):
    msg = ctypes.create_string_buffer(256)
    tb = view.block_table
    rc = lib.zllm_attention_decode_bf16_noalloc(
        ptr(qkv), ptr(out), ptr(ctx.decode_rows), c_int(ctx.n_decode if n_rows is None else n_rows), ptr(ctx.positions),
        ptr(ctx.row_slot), ptr(view.k_pages), ptr(view.v_pages), ptr(tb), c_int(tb.shape[1]), c_int(view.block_size),
        c_int(nq), c_int(nkv), c_int(hd), c_float(scale), c_int(window or 0), c_int(n_splits),
        c_void_p(torch.cuda.current_stream().cuda_stream), msg, c_int(256))
    return rc, msg.value.decode()


@pytest.mark.parametrize("nq,nkv,hd,bs,window", [(8, 2, 64, 16, None), (6, 2, 96, 16, None), (4, 1, 128, 8, 300)])
def test_no_alloc_entry_point_matches_the_regular_one_twice(nq, nkv, hd, bs, window):
    from ref_ops import RefOps
    from gpu_util import CpuCacheView, cpu_ctx
    from zllm_b200.kernels.ops import CudaOps
    ops = CudaOps(DEV)
    ops.configure(torch.bfloat16)
    lib = ops.lib("attention_bf16")
    dtype = torch.bfloat16
    cm = make_cache(nkv, hd, bs, 3200 // bs, 6, 1400, dtype, window)
    slots = [cm.admit() for _ in range(5)]
    view = cm.view(0)
    g = torch.Generator().manual_seed(3)
    view.k_pages.copy_(torch.randn(view.k_pages.shape, generator=g).to(dtype))
    view.v_pages.copy_(torch.randn(view.v_pages.shape, generator=g).to(dtype))
    for s, n in zip(slots, (900, 3, 300, 1, 620)):          # one to four splits of 256 keys
        make_ctx(cm, [(s, n)])
    scale = 1.0 / math.sqrt(hd)
    for call in range(2):                                     # two calls in a row: the scratch is reused
        ctx = make_ctx(cm, [(s, 1) for s in slots])           # one decoded row per request, one position further
        T = ctx.T
        qkv = (torch.randn(T, (nq + 2 * nkv) * hd, generator=g) * (1 + call)).to(dtype).to(DEV)
        regular = torch.zeros(T, nq * hd, dtype=dtype, device=DEV)
        ops.paged_attention(qkv, regular, ctx, view, nq, nkv, hd, scale, window)   # the engine's entry point
        plain = torch.zeros(T, nq * hd)                        # the plain statement, float32 on the CPU
        RefOps().paged_attention(qkv.float().cpu(), plain, cpu_ctx(ctx), CpuCacheView(view), nq, nkv, hd, scale, window)
        got = torch.full((T, nq * hd), 7.0, dtype=dtype, device=DEV)
        before = torch.cuda.memory_allocated()
        rc, msg = call_noalloc(lib, qkv, got, ctx, view, nq, nkv, hd, scale, window, ops.decode_splits(ctx.max_context))
        assert rc == 0, msg
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        # the tolerance of the attention kernel tests: against the plain statement ...
        err = float((got.float().cpu() - plain).abs().max())
        assert err <= 0.02 * max(1.0, float(plain.abs().max())), f"call {call}: {err} from the plain statement"
        # ... and against the regular entry point (which may be another kernel for this head size)
        err = float((got.float() - regular.float()).abs().max())
        assert err <= 0.02, f"call {call}: {err} from the regular entry point"
        assert float(plain.abs().max()) > 0.1


def test_no_alloc_entry_point_refuses_what_does_not_fit():
    from zllm_b200.kernels.ops import CudaOps
    ops = CudaOps(DEV)
    ops.configure(torch.bfloat16)
    lib = ops.lib("attention_bf16")
    nq, nkv, hd, bs = 32, 8, 128, 16
    cm = make_cache(nkv, hd, bs, 8, 2, 64, torch.bfloat16)
    s = cm.admit()
    make_ctx(cm, [(s, 5)])
    ctx = make_ctx(cm, [(s, 1)])
    qkv = torch.zeros(1, (nq + 2 * nkv) * hd, dtype=torch.bfloat16, device=DEV)
    out = torch.zeros(1, nq * hd, dtype=torch.bfloat16, device=DEV)
    # 1 row x 32 heads x 2048 splits x 130 floats = 8.5 M floats > 4 Mi: refused, nothing launched
    rc, msg = call_noalloc(lib, qkv, out, ctx, cm.view(0), nq, nkv, hd, 0.1, None, 2048)
    assert rc == TOO_LARGE and "exceeds the built-in scratch" in msg
    rc, msg = call_noalloc(lib, qkv, out, ctx, cm.view(0), nq, nkv, 72, 0.1, None, 1)
    assert rc == 10001 and "head size" in msg
    view = cm.view(0)
    tb = view.block_table
    msgbuf = ctypes.create_string_buffer(256)                 # a page size of 0 is refused, not divided by
    rc = lib.zllm_attention_decode_bf16_noalloc(
        ptr(qkv), ptr(out), ptr(ctx.decode_rows), c_int(1), ptr(ctx.positions), ptr(ctx.row_slot), ptr(view.k_pages),
        ptr(view.v_pages), ptr(tb), c_int(tb.shape[1]), c_int(0), c_int(nq), c_int(nkv), c_int(hd), c_float(0.1), c_int(0),
        c_int(1), c_void_p(torch.cuda.current_stream().cuda_stream), msgbuf, c_int(256))
    assert rc == 10001 and "page size" in msgbuf.value.decode()
    torch.cuda.synchronize()
