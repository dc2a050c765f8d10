"""The step function: one batch of (request, its next tokens) through the model,
from the cache, logits at the wanted places.

After the reference's ``BatchedDecoder`` step (zllm src/backend/gpu/mod.rs:2180-2243:
write inputs -> prepare paging -> layers -> final norm -> head -> select) and its
prefill chunk (mod.rs:2383-2421), with one difference: portions of prompts and
single decoded tokens of other requests go through ONE forward, cut anywhere.
A step runs only the tokens it is given; every earlier position comes from the
cache.  Pool exhaustion is an error return (MemoryError_) raised before
anything is launched, where the reference panics (mod.rs:2508-2509).

Decode-only steps replay a captured CUDA graph per (rows, split-count) bucket,
since at small batch the step is bound by launches, not by memory.  Steps with
prompt portions are captured too, per shape bucket (rows, decoded rows, wanted
rows, splits, the parts' own table sizes), once a shape has been seen twice: a
forward is more than a hundred launches, which the driver then issues in one
call where the host would need a millisecond.  The reference records a whole
step into one command buffer and submits it once (mod.rs:2193-2208).
"""
from __future__ import annotations

from pathlib import Path
from typing import Dict, List, Optional, Sequence

import torch

from ..cache.manager import CacheManager
from ..config.engine_config import EngineConfig
from ..config.model_config import read_config_json
from ..config.registry import architecture_of
from ..errors import BackendError, ConfigError, MemoryError_, RequestError
from ..models.decoder import DecoderModel, Runtime
from ..weights.loader import load_checked, target_dtype
from ..weights.random_init import random_tensor
from .batch import StepBuffers, StepContext, StepEntry, Workspace, fill_step, make_context

_TORCH_DTYPE = {"bfloat16": torch.bfloat16, "float32": torch.float32}


def _default_ops(device):
    from ..kernels.ops import CudaOps
    return CudaOps(device)


class ModelRunner:
    """Model + cache + step function on one device."""

    def __init__(self, model_dir=None, *, config=None, seed: Optional[int] = None,
                 engine_config: Optional[EngineConfig] = None, ops=None, init_std=None, norm_std=None,
                 random_on_device: bool = False):
        self.ecfg = (engine_config or EngineConfig()).validate()
        self.device = torch.device(self.ecfg.device)
        self.dtype = _TORCH_DTYPE[self.ecfg.dtype]
        if ops is None:
            if self.device.type != "cuda":
                raise BackendError("the engine runs on a CUDA device only; there is no CPU path")
            ops = _default_ops(self.device)
        self.ops = ops
        ops.configure(self.dtype)
        if getattr(ops, "profiling", False) and self.ecfg.cuda_graphs:
            # per-operation timers bracket every launch with events, which a captured graph cannot hold
            import dataclasses
            self.ecfg = dataclasses.replace(self.ecfg, cuda_graphs=False)
        if model_dir is not None:
            raw = read_config_json(model_dir)
            arch = architecture_of(raw)
            self.config = arch.read_config(raw)
        elif config is not None:
            from ..config.registry import architecture
            arch = architecture(config.architecture)
            self.config = config
        else:
            raise ConfigError("ModelRunner needs a model folder or a configuration")
        self.spec = arch.build_spec(self.config)
        rt = Runtime(self.dtype, self.device, ops)
        self.model = DecoderModel(self.spec, rt)
        if model_dir is not None:
            tensors = load_checked(model_dir, self.model.required_tensors(), self.dtype, self.device,
                                   optional=self.model.optional_tensors(), ignored=self.spec.ignored_tensors)
        else:
            tensors = {}
            for name, ws in self.model.expected_tensors().items():
                dt = target_dtype(torch.bfloat16 if self.dtype == torch.bfloat16 else torch.float32, ws.role, self.dtype)
                # drawn on the CPU (the same values everywhere) unless the caller asks for speed
                t = random_tensor(name, ws, seed or 0, dt, self.device if random_on_device else "cpu", init_std, norm_std)
                tensors[name] = t.to(self.device)
        self.model.load_weights(tensors)
        del tensors

        self.max_len = min(self.ecfg.max_model_len or self.spec.max_position, self.spec.max_position)
        bs = self.ecfg.block_size
        needs = self.model.cache_needs()
        num_blocks = self.ecfg.num_blocks
        if num_blocks is None:
            num_blocks = self.ecfg.max_num_seqs * (-(-self.max_len // bs))
            num_blocks = min(num_blocks, self._blocks_that_fit(needs, bs))
        self.cache = CacheManager(needs, bs, num_blocks, self.ecfg.max_num_seqs, self.max_len, self.dtype, self.device,
                                  prefix_sharing=self.ecfg.prefix_sharing)
        self.max_rows = self.ecfg.max_num_batched_tokens
        self.ws = Workspace(self.max_rows, self.device)
        self.buffers = StepBuffers(self.max_rows, self.max_rows, self.device)
        self._planners = self.model.step_planners()
        self._graphs: Dict[tuple, dict] = {}
        # graphs of steps with prompt portions, by shape bucket; a shape is captured when it comes
        # a second time.  Only for models all of whose parts say they can be captured.
        self._step_graphs: Dict[tuple, dict] = {}
        self._step_seen: Dict[tuple, int] = {}
        self._side_stream = None
        self._graph_pool = None
        self._last_captured = None
        self.step_graphs_on = bool(self.ecfg.cuda_graphs and self.ecfg.step_graphs and self.device.type == "cuda"
                                   and self.model.capturable())
        self.step_graph_replays = 0
        self._token_ring = None
        self._last_key = None
        self.steps = 0
        self.tokens_run = 0

    # ------------------------------------------------------------------
    def _blocks_that_fit(self, needs, bs) -> int:
        if self.device.type != "cuda":
            return 1 << 30
        per_block = 0
        el = 2 if self.dtype == torch.bfloat16 else 4
        for spec, cache_of in needs:
            if cache_of is None and spec is not None and hasattr(spec, "n_kv_heads"):
                per_block += 2 * bs * spec.n_kv_heads * spec.head_dim * el
        if per_block == 0:
            return 1
        free, _ = torch.cuda.mem_get_info(self.device)
        return max(1, int(free * 0.6) // per_block)

    # ---- slots -----------------------------------------------------------
    def admit(self) -> Optional[int]:
        return self.cache.admit()

    def release(self, slot: int) -> None:
        self.cache.free_slot(slot)

    def cached_len(self, slot: int) -> int:
        return self.cache.length[slot]

    def truncate(self, slot: int, new_len: int) -> None:
        """Forget the slot's positions from ``new_len`` on; the next step continues there."""
        self.cache.truncate(slot, new_len)

    # ---- the step ----------------------------------------------------------
    def _prepare(self, entries: Sequence[StepEntry]):
        if not entries:
            raise RequestError("a step needs at least one entry")
        total = 0
        seen = set()
        for e in entries:
            n = len(e.tokens)
            if n == 0:
                raise RequestError(f"slot {e.slot}: an entry needs at least one token")
            if e.slot in seen:
                raise RequestError(f"slot {e.slot} appears twice in one step")
            seen.add(e.slot)
            if not self.cache.live[e.slot]:
                raise RequestError(f"slot {e.slot} is not live")
            if self.cache.length[e.slot] + n > self.max_len:
                raise RequestError(f"slot {e.slot}: position {self.cache.length[e.slot] + n} exceeds the "
                                   f"maximum length {self.max_len}")
            total += n
        if total > self.max_rows:
            raise RequestError(f"step of {total} tokens exceeds max_num_batched_tokens {self.max_rows}")
        # pages for everything, or nothing is run
        if not self.cache.can_fit([(e.slot, self.cache.length[e.slot] + len(e.tokens)) for e in entries]):
            raise MemoryError_(f"cache pool exhausted: free pages {self.cache.free_pages()} do not cover this step")
        starts = []
        for e in entries:
            start = self.cache.length[e.slot]
            ok = self.cache.ensure(e.slot, start + len(e.tokens))
            assert ok
            starts.append(start)
        return starts

    def step(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """Run the entries as one batch.  Returns float32 logits [wanted, vocab] on the
        device, in the order of the entries and of their ``want`` (None if nothing is wanted).
        The tensor is a view of a reused buffer: read it before the next step."""
        starts = self._prepare(entries)
        if self.step_graphs_on:
            logits = self._step_through_graph(entries, starts)
            if logits is not NotImplemented:
                return logits
        buf = self.buffers
        T, R, nd, plans, max_ctx = fill_step(buf, entries, starts, planners=self._planners)
        buf.upload()
        self.cache.sync_tables()
        ctx = make_context(buf, T, R, nd, plans, max_ctx, self.ws, entries, starts)
        logits = self._forward(ctx)
        for e, s in zip(entries, starts):
            self.cache.advance(e.slot, s + len(e.tokens))
        self.steps += 1
        self.tokens_run += T
        return logits

    # ---- steps with prompt portions through captured graphs -----------------------------------
    STEP_GRAPH_CAP = 64                     # graphs kept; beyond that new shapes run launch by launch

    @staticmethod
    def _row_bucket(n: int) -> int:
        """Rows of a captured step: 16, 32, 64, 128, then multiples of 128 up to 1024, then of 256."""
        if n <= 128:
            return max(16, _bucket(n))
        if n <= 1024:
            return -(-n // 128) * 128
        return -(-n // 256) * 256

    def _step_through_graph(self, entries, starts):
        """Run the step by replaying the graph of its shape bucket; NotImplemented when the shape
        has no graph (yet) and the caller should launch the kernels one by one."""
        T = sum(len(e.tokens) for e in entries)
        nd = sum(1 for e in entries if len(e.tokens) == 1)
        if nd == len(entries):
            return NotImplemented                           # decode-only steps have their own graphs
        R = sum(len(e.want) for e in entries)
        nd_b = _bucket(nd) if nd else 0
        T_b = self._row_bucket(T + (nd_b - nd))             # padding rows stand in for the missing decoded rows
        if T_b > self.max_rows:
            return NotImplemented
        R_b = _bucket(R) if R else 0
        max_ctx = max(s + len(e.tokens) for e, s in zip(entries, starts))
        sp_b = _bucket(self.ops.decode_splits(max_ctx)) if nd else 0
        # the parts' tables: their sizes are part of the shape
        probe = StepBuffers.table_shapes(entries, starts, self._planners)
        key = (T_b, nd_b, R_b, sp_b, probe)
        g = self._step_graphs.get(key)
        if g is None:
            seen = self._step_seen.get(key, 0) + 1
            self._step_seen[key] = seen
            if seen < 2 or len(self._step_graphs) >= self.STEP_GRAPH_CAP:
                return NotImplemented
            g = self._step_graphs[key] = self._capture_step(key, entries, starts)
        buf = g["buf"]
        fill_step(buf, entries, starts, pad_rows=T_b, planners=self._planners, pad_decode=nd_b, pad_want=R_b,
                  bucketed=True)
        buf.upload()
        self.cache.sync_tables()
        g["graph"].replay()
        for e, s in zip(entries, starts):
            self.cache.advance(e.slot, s + len(e.tokens))
        self.steps += 1
        self.tokens_run += T
        self.step_graph_replays += 1
        return g["logits"][:R] if R else None

    def _capture_step(self, key, entries, starts):
        T_b, nd_b, R_b, sp_b, _ = key
        buf = StepBuffers(T_b, max(R_b, 1), self.device)
        _, R, nd, plans, _ = fill_step(buf, entries, starts, pad_rows=T_b, planners=self._planners, pad_decode=nd_b,
                                       pad_want=R_b, bucketed=True)
        ctx = make_context(buf, T_b, R, nd, plans, 0, self.ws)          # no host-side description: a replay has other entries
        ctx.max_context = sp_b * self.ops.decode_split_keys
        ctx.fixed_splits = sp_b
        # warm-up and capture run on neutral contents: every row padding, every tile empty, so that
        # nothing is written to the cache; the real contents are uploaded before each replay
        buf.host_section("row_slot")[:] = -1
        buf.host_section("token_ids")[:] = 0
        buf.host_section("positions")[:] = 0
        for name, (off, shape) in plans.items():
            n = 1
            for d in shape:
                n *= d
            self._neutral_table(buf.host_section("aux")[off:off + n], name)
        buf.upload()
        self.cache.sync_tables()
        logits = self._capture(lambda: self._forward(ctx))
        return {"buf": buf, "graph": self._last_captured, "logits": logits, "ctx": ctx}

    def _capture(self, body):
        """Run ``body`` once on a side stream (it sizes every workspace buffer), then capture it
        into a graph (``self._last_captured``) and return what it returned.  The graphs share one
        memory pool; ``capture_begin`` is used directly because the ``torch.cuda.graph`` context
        collects garbage and empties the allocator's cache on entry, which costs tens of
        milliseconds per capture."""
        cur = torch.cuda.current_stream(self.device)
        if self._side_stream is None:
            self._side_stream = torch.cuda.Stream(self.device)
            self._graph_pool = torch.cuda.graph_pool_handle()
        side = self._side_stream
        side.wait_stream(cur)
        with torch.cuda.stream(side):
            body()
            side.synchronize()
            graph = torch.cuda.CUDAGraph()
            graph.capture_begin(pool=self._graph_pool)
            try:
                out = body()
            finally:
                graph.capture_end()
        cur.wait_stream(side)
        self._last_captured = graph
        return out

    @staticmethod
    def _neutral_table(host, name):
        # a part's table made harmless for the warm-up and capture runs: the attention path's tiles
        # become empty tiles; any other table is zeroed
        if name == "query_tiles":
            host.reshape(-1, 4)[:] = (0, 0, -1, 0)
        else:
            host[:] = 0

    def _forward(self, ctx):
        bind = getattr(self.ops, "bind_stream", None)
        if bind is None:
            return self.model.forward(ctx, self.cache.views)
        bind()                                  # one stream lookup for the whole forward
        try:
            return self.model.forward(ctx, self.cache.views)
        finally:
            self.ops.unbind_stream()

    # ---- decode-only steps through a captured graph ----------------------------
    def decode_step(self, slots: Sequence[int], tokens: Sequence[int], temps: Sequence[float],
                    seeds: Sequence[int], pool=None) -> torch.Tensor:
        """One decoded token for each slot; samples on the device (temperature <= 0: argmax)
        and returns the int32 token ids [len(slots)] on the device.  The logits of the step
        stay in ``self.last_logits`` ([bucket, vocab], first len(slots) rows valid).

        ``pool`` = (temperatures, top_ks, top_ps) per slot: rows with a temperature > 0 there are
        drawn among their 64 best candidates on the device (top-k / top-p sampling); their entry in
        ``temps`` must then be 0.  Needs CUDA graphs."""
        entries = [StepEntry(s, (t,), (0,)) for s, t in zip(slots, tokens)]
        starts = self._prepare(entries)
        n = len(entries)
        use_graph = self.ecfg.cuda_graphs and self.device.type == "cuda"
        bucket = _bucket(n) if use_graph else n
        max_ctx = max(starts) + 1
        split_bucket = _bucket(self.ops.decode_splits(max_ctx)) if use_graph else 0
        if pool is not None and not use_graph:
            raise BackendError("sampling from the candidate pool on the device needs CUDA graphs")
        key = (bucket, split_bucket, pool is not None)
        g = self._graphs.get(key)
        if g is None:
            g = self._make_decode_graph(bucket, split_bucket, use_graph, pool is not None)
            self._graphs[key] = g
        buf = g["buf"]
        fill_step(buf, entries, starts, pad_rows=bucket)
        if pool is not None:
            pt = buf.host_section("pool_temp").view("float64")
            pp = buf.host_section("pool_topp").view("float64")
            pk = buf.host_section("pool_topk")
            pt[:bucket] = 0.0
            pt[:n], pk[:n], pp[:n] = pool[0], pool[1], pool[2]
        # every row of the bucket is "wanted" so that the graph's shapes never change
        want = buf.host_section("want_rows")
        want[:bucket] = range(bucket)
        tf = buf.host_section("temps").view("float32")
        tf[:bucket] = 0.0
        tf[:n] = temps
        sd = buf.host_section("seeds").view("uint32")
        sd[:bucket] = 0
        sd[:n] = [s & 0xFFFFFFFF for s in seeds]
        buf.upload()
        self.cache.sync_tables()
        if use_graph:
            g["graph"].replay()
        else:
            g["ctx"].max_context = max_ctx          # no captured shape to honour: size the step as it is
            g["ctx"].fixed_splits = 0
            g["ctx"].entries, g["ctx"].starts = list(entries), list(starts)
            self._decode_body(g)
        for e, s in zip(entries, starts):
            self.cache.advance(e.slot, s + 1)
        self.steps += 1
        self.tokens_run += n
        self.last_logits = g["logits"]
        self._last_key = key
        return g["out"][:n]

    # ---- decode steps whose tokens are read later (host work overlaps the device) ----------
    def decode_launch(self, slots: Sequence[int], tokens: Sequence[int], temps: Sequence[float],
                      seeds: Sequence[int], pool=None):
        """``decode_step`` that does not wait: the sampled tokens are copied to pinned host memory
        behind the step and a handle is returned; ``decode_collect(handle)`` waits and reads them."""
        out = self.decode_step(slots, tokens, temps, seeds, pool)
        return self._token_handle(out, len(slots), self._last_key, list(slots))

    def decode_continue(self, handle):
        """Launch the step AFTER the one in ``handle`` for the same slots without knowing its
        tokens yet: the step's inputs were advanced on the device (token <- sampled token,
        position + 1, seed + 0x9E3779B1).  Returns a new handle, or None when that is not
        possible (another graph bucket would be needed, a page is missing, length limit)."""
        if not (self.ecfg.cuda_graphs and self.device.type == "cuda"):
            return None
        slots = handle["slots"]
        key = handle["key"]
        g = self._graphs.get(key)
        if g is None or g["graph"] is None:
            return None
        new_ctx = max(self.cache.length[s] for s in slots) + 1
        if _bucket(self.ops.decode_splits(new_ctx)) != key[1]:
            return None
        if any(self.cache.length[s] + 1 > self.max_len for s in slots):
            return None
        if not self.cache.can_fit([(s, self.cache.length[s] + 1) for s in slots]):
            return None
        for s in slots:
            ok = self.cache.ensure(s, self.cache.length[s] + 1)
            assert ok
        self.cache.sync_tables()
        g["graph"].replay()
        for s in slots:
            self.cache.advance(s, self.cache.length[s] + 1)
        self.steps += 1
        self.tokens_run += len(slots)
        self.last_logits = g["logits"]
        return self._token_handle(g["out"][:len(slots)], len(slots), key, slots)

    def _token_handle(self, out, n, key, slots):
        ring = self._token_ring
        if ring is None:
            ring = self._token_ring = [torch.zeros(max(self.ecfg.max_num_seqs, 1), dtype=torch.int32).pin_memory()
                                       if self.device.type == "cuda" else torch.zeros(self.ecfg.max_num_seqs, dtype=torch.int32)
                                       for _ in range(4)]
            self._token_ring_next = 0
        host = ring[self._token_ring_next % len(ring)]
        self._token_ring_next += 1
        host[:n].copy_(out, non_blocking=True)
        ev = None
        if self.device.type == "cuda":
            ev = torch.cuda.Event()
            ev.record()
        return {"host": host, "event": ev, "n": n, "key": key, "slots": slots}

    def decode_collect(self, handle) -> List[int]:
        if handle["event"] is not None:
            handle["event"].synchronize()
        check = getattr(self.ops, "raise_if_a_wait_gave_up", None)
        if check is not None:
            check()                 # a kernel whose bounded wait ran out has flagged it by now
        return handle["host"][:handle["n"]].tolist()

    def _decode_body(self, g):
        ctx = g["ctx"]
        logits = self._forward(ctx)
        g["logits"] = logits
        buf = g["buf"]
        B = ctx.T
        seeds = buf.dev_section("seeds", B)
        self.ops.sample(logits, buf.dev_section("temps", B).view(torch.float32), seeds, g["out"])
        if g.get("pool_vals") is not None:
            # top-k / top-p rows: the 64 best candidates, then the draw among them, all on the device
            self.ops.topk(logits, g["pool_vals"].shape[1], g["pool_vals"], g["pool_idx"])
            self.ops.pool_draw(g["pool_vals"], g["pool_idx"], buf.dev_section("pool_temp", 2 * B).view(torch.float64),
                               buf.dev_section("pool_topk", B), buf.dev_section("pool_topp", 2 * B).view(torch.float64),
                               seeds, g["out"])
        if hasattr(self.ops, "advance_decode"):
            # the step's inputs become those of the next step: a burst replays without the host
            self.ops.advance_decode(ctx.token_ids, ctx.positions, ctx.row_slot, seeds, g["out"], g["hist"], g["counter"])

    def decode_burst(self, slots: Sequence[int], tokens: Sequence[int], temps: Sequence[float],
                     seeds: Sequence[int], n_steps: int) -> torch.Tensor:
        """``n_steps`` decode steps back to back on the device: each step's sampled token is the
        next step's input, positions and seeds advance on the device, and the host reads the
        tokens [n_steps, len(slots)] once at the end.  Pages for all steps are taken up front.
        Stop tokens are not looked at in between: the caller cuts the streams afterwards."""
        if not (self.ecfg.cuda_graphs and self.device.type == "cuda"):
            raise BackendError("decode_burst needs CUDA graphs")
        if n_steps < 1 or n_steps > self.BURST_CAP:
            raise RequestError(f"a burst has 1..{self.BURST_CAP} steps")
        entries = [StepEntry(s, (t,), (0,)) for s, t in zip(slots, tokens)]
        # pages for the whole burst, or nothing is run
        if not self.cache.can_fit([(s, self.cache.length[s] + n_steps) for s in slots]):
            raise MemoryError_(f"cache pool exhausted: free pages {self.cache.free_pages()} do not cover the burst")
        starts = self._prepare(entries)
        for s in slots:
            if self.cache.length[s] + n_steps > self.max_len:
                raise RequestError(f"slot {s}: the burst exceeds the maximum length {self.max_len}")
            ok = self.cache.ensure(s, self.cache.length[s] + n_steps)
            assert ok
        n = len(entries)
        bucket = _bucket(n)
        split_bucket = _bucket(self.ops.decode_splits(max(starts) + n_steps))
        key = (bucket, split_bucket, False)
        g = self._graphs.get(key)
        if g is None:
            g = self._graphs[key] = self._make_decode_graph(bucket, split_bucket, True)
        buf = g["buf"]
        fill_step(buf, entries, starts, pad_rows=bucket)
        buf.host_section("want_rows")[:bucket] = range(bucket)
        tf = buf.host_section("temps").view("float32")
        tf[:bucket] = 0.0
        tf[:n] = temps
        sd = buf.host_section("seeds").view("uint32")
        sd[:bucket] = 0
        sd[:n] = [s & 0xFFFFFFFF for s in seeds]
        buf.upload()
        self.cache.sync_tables()
        g["counter"].zero_()
        for _ in range(n_steps):
            g["graph"].replay()
        for s, st in zip(slots, starts):
            self.cache.advance(s, st + n_steps)
        self.steps += n_steps
        self.tokens_run += n * n_steps
        self.last_logits = g["logits"]
        return g["hist"][:n_steps, :n]

    BURST_CAP = 1024

    def _make_decode_graph(self, bucket: int, split_bucket: int, use_graph: bool, pool: bool = False):
        buf = StepBuffers(bucket, bucket, self.device)
        ctx = make_context(buf, bucket, bucket, bucket, None, 0, self.ws)
        ctx.max_context = split_bucket * self.ops.decode_split_keys if split_bucket else 0
        ctx.fixed_splits = split_bucket
        out = torch.zeros(bucket, dtype=torch.int32, device=self.device)
        g = {"buf": buf, "ctx": ctx, "out": out, "logits": None, "graph": None,
             "hist": torch.zeros((self.BURST_CAP, bucket), dtype=torch.int32, device=self.device),
             "counter": torch.zeros(1, dtype=torch.int32, device=self.device), "launches": 0,
             "pool_vals": None, "pool_idx": None}
        if pool:
            k = min(64, self.spec.vocab_size)
            g["pool_vals"] = torch.zeros((bucket, k), dtype=torch.float32, device=self.device)
            g["pool_idx"] = torch.zeros((bucket, k), dtype=torch.int32, device=self.device)
        if not use_graph:
            return g
        # neutral contents for warm-up and capture: every row is padding
        buf.begin_fill()
        buf.host_section("row_slot")[:] = -1
        buf.host_section("decode_rows")[:bucket] = range(bucket)
        buf.host_section("want_rows")[:bucket] = range(bucket)
        buf.upload()
        before = getattr(self.ops, "launches", 0)
        self._capture(lambda: self._decode_body(g))
        g["launches"] = (getattr(self.ops, "launches", 0) - before) // 2     # kernels in one replay (warm-up + capture)
        graph = self._last_captured
        g["graph"] = graph
        return g

    def capture_decode_graphs(self, max_batch: Optional[int] = None, max_context: Optional[int] = None,
                              pool: bool = False) -> int:
        """Capture the decode graphs of every (rows, splits) bucket up to ``max_batch`` rows and
        ``max_context`` positions now, so that no step pays for a capture later (a capture takes a
        few milliseconds).  ``pool``: also the variants that draw top-k / top-p tokens on the device.
        Returns the number of graphs captured."""
        if not (self.ecfg.cuda_graphs and self.device.type == "cuda"):
            return 0
        max_batch = min(max_batch or self.ecfg.max_num_seqs, self.ecfg.max_num_seqs)
        max_context = min(max_context or self.max_len, self.max_len)
        n = 0
        b = 1
        while True:
            sb = 1
            while True:
                for with_pool in ((False, True) if pool else (False,)):
                    if (b, sb, with_pool) not in self._graphs:
                        self._graphs[(b, sb, with_pool)] = self._make_decode_graph(b, sb, True, with_pool)
                        n += 1
                if sb >= self.ops.decode_splits(max_context):
                    break
                sb *= 2
            if b >= max_batch:
                break
            b *= 2
        return n

    # ---- numbers for measurement ------------------------------------------------
    def weight_bytes(self) -> int:
        seen = set()
        total = 0
        def add(t):
            nonlocal total
            if isinstance(t, torch.Tensor) and t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                total += t.numel() * t.element_size()
        add(self.model.embedding if self.model.head is not self.model.embedding else None)
        add(self.model.head)
        for layer in self.model.layers:
            for part in layer.parts().values():
                for v in vars(part).values():
                    add(v)
        for v in vars(self.model.final_norm).values():
            add(v)
        return total


def _bucket(n: int) -> int:
    b = 1
    while b < n:
        b *= 2
    return b
