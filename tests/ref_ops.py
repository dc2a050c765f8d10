"""Plain torch statements of every kernel the engine calls, one function per kernel.

Two uses: (1) each CUDA kernel is compared alone with the function of the same
name here; (2) given to the engine as its kernel table, they let the host side
(cache, tables, batch description, step, scheduler) run on the CPU in tests.
They are never chosen by the package itself: the product path has CUDA only.

Formulas cite zllm's kernels (src/backend/gpu/shaders.rs) where one exists.
"""
from __future__ import annotations

import math

import torch

GROUP = 8


def deinterleave_gate_up(w):
    """[2I, K] in groups of (8 gate rows, 8 up rows) -> gate [I,K], up [I,K]."""
    two_i, K = w.shape
    w = w.reshape(two_i // (2 * GROUP), 2, GROUP, K)
    return w[:, 0].reshape(-1, K), w[:, 1].reshape(-1, K)


class RefOps:
    decode_split_keys = 256

    def __init__(self, device="cpu"):
        self.device = torch.device(device)
        self.dtype = torch.float32

    def configure(self, dtype):
        self.dtype = dtype

    def decode_splits(self, max_ctx):
        return max(1, -(-max_ctx // self.decode_split_keys))

    # ---- embedding: x[t] = E[token[t]] (fork.rs:935) -------------------------------
    def embedding(self, token_ids, table, out):
        out.copy_(table[token_ids.long()].float())

    # ---- BNORM (shaders.rs:545-564) --------------------------------------------------
    def rmsnorm(self, x, weight, eps, out, rows=None):
        xf = x.float() if rows is None else x[rows.long()].float()
        inv = torch.rsqrt((xf * xf).mean(dim=-1, keepdim=True) + eps)
        out.copy_((xf * inv * weight.float()).to(out.dtype))

    # ---- products out = x W^T with the three epilogues --------------------------------
    def linear(self, x, w, out, mode):
        xf, wf = x.float(), w.float()
        if mode == "store":
            out.copy_((xf @ wf.T).to(out.dtype))
        elif mode == "add":
            out.add_((xf @ wf.T).to(out.dtype))
        elif mode == "swiglu":
            g, u = deinterleave_gate_up(wf)
            gv = xf @ g.T
            out.copy_((gv / (1.0 + torch.exp(-gv)) * (xf @ u.T)).to(out.dtype))
        else:
            raise ValueError(mode)

    # ---- SILU_MUL (shaders.rs:976-990) -------------------------------------------------
    def silu_mul(self, a, b, out):
        af = a.float()
        out.copy_((af / (1.0 + torch.exp(-af)) * b.float()).to(out.dtype))

    # ---- BROPE + BKV_PACK (shaders.rs:566-587, 727-756) -------------------------------
    def rope_kv_store(self, qkv, ctx, rot, cache, nq, nkv, hd, write_cache=True):
        T = qkv.shape[0]
        pos = ctx.positions.long()
        x = qkv.float().reshape(T, nq + 2 * nkv, hd)
        q, k, v = x[:, :nq], x[:, nq:nq + nkv], x[:, nq + nkv:]
        if rot is not None:
            c = rot.cos[pos][:, None, :]
            s = rot.sin[pos][:, None, :]
            rd = rot.rot_dim

            def rotate(t):
                t = t.clone()
                r = t[..., :rd]
                if rot.interleaved:
                    a, b = r[..., 0::2], r[..., 1::2]
                    o = torch.empty_like(r)
                    o[..., 0::2] = a * c - b * s
                    o[..., 1::2] = a * s + b * c
                else:
                    a, b = r[..., :rd // 2], r[..., rd // 2:]
                    o = torch.cat([a * c - b * s, a * s + b * c], dim=-1)
                t[..., :rd] = o
                return t
            q, k = rotate(q), rotate(k)
        out = torch.cat([q, k, v], dim=1).reshape(T, -1)
        qkv.copy_(out.to(qkv.dtype))
        if not write_cache:
            return
        bs = cache.block_size
        kq = qkv.reshape(T, nq + 2 * nkv, hd)
        for t in range(T):
            slot = int(ctx.row_slot[t])
            if slot < 0:
                continue
            p = int(pos[t])
            page = int(cache.block_table[slot, p // bs])
            assert page >= 0, "write to a position without a page"
            cache.k_pages[page, :, p % bs, :] = kq[t, nq:nq + nkv].to(cache.k_pages.dtype)
            cache.v_pages[page, :, p % bs, :] = kq[t, nq + nkv:].to(cache.v_pages.dtype)

    # ---- BDSDPA_PAGED (shaders.rs:670-725) ----------------------------------------------
    def paged_attention(self, qkv, out, ctx, cache, nq, nkv, hd, scale, window):
        T = qkv.shape[0]
        bs = cache.block_size
        q = qkv.float().reshape(T, nq + 2 * nkv, hd)[:, :nq]
        rep = nq // nkv
        for t in range(T):
            slot = int(ctx.row_slot[t])
            if slot < 0:
                out[t].zero_()
                continue
            p = int(ctx.positions[t])
            lo = 0 if not window else max(0, p - window + 1)
            idx = torch.arange(lo, p + 1)
            pages = cache.block_table[slot, (idx // bs).long()].long()
            assert (pages >= 0).all(), "read of a position whose page was given back"
            K = cache.k_pages[pages, :, (idx % bs).long(), :].float()   # [n, nkv, hd]
            V = cache.v_pages[pages, :, (idx % bs).long(), :].float()
            K = K.repeat_interleave(rep, dim=1)
            V = V.repeat_interleave(rep, dim=1)
            s = torch.einsum("hd,nhd->hn", q[t], K) * scale
            pr = torch.softmax(s, dim=-1)
            o = torch.einsum("hn,nhd->hd", pr, V)
            out[t].copy_(o.reshape(-1).to(out.dtype))

    # ---- fused forms (the compositions they stand for) ----------------------------------------
    def linear_normed(self, x, norm_w, eps, w, out, mode, ws, rows=None):
        h = torch.empty((out.shape[0], x.shape[1]), dtype=w.dtype)
        self.rmsnorm(x, norm_w, eps, h, rows=rows)
        self.linear(h, w, out, mode)

    def qkv_rope_store(self, x, norm, w_qkv, qkv, ctx, rot, cache, nq, nkv, hd, write_cache, ws):
        if norm is not None:
            h = torch.empty(x.shape, dtype=w_qkv.dtype)
            self.rmsnorm(x, norm[0], norm[1], h)
            x = h
        self.linear(x, w_qkv, qkv, "store")
        self.rope_kv_store(qkv, ctx, rot, cache, nq, nkv, hd, write_cache)

    def gather_rows(self, x, rows, out):
        out.copy_(x[rows.long()])

    # ---- BSAMPLE / BARGMAX (shaders.rs:758-850) -----------------------------------------
    def sample(self, logits, temps, seeds, out):
        from plain_llama import gumbel_sample
        for r in range(logits.shape[0]):
            out[r] = gumbel_sample(logits[r].float().cpu(), float(temps[r]), int(seeds[r]) & 0xFFFFFFFF)

    # ---- BTOPK (shaders.rs:852-905) -------------------------------------------------------
    def topk(self, logits, k, vals, idx):
        from plain_llama import topk_desc
        for r in range(logits.shape[0]):
            v, i = topk_desc(logits[r].float().cpu(), k)
            n = len(v)
            vals[r, :n] = torch.tensor(v)
            idx[r, :n] = torch.tensor(i, dtype=idx.dtype)
            if n < k:
                vals[r, n:] = -3.0e38
                idx[r, n:] = -1
