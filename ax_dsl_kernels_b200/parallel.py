"""Multi-GPU host logic: one process per GPU, torch.distributed for the plumbing (NCCL on GPUs; the same code runs
over gloo on CPU in the tests, with the local compute injected).  Two forms: expert parallelism of the MoE block
(below) and tensor parallelism of the dense hybrid stack (second half of the file).

Expert parallelism for decode-sized batches.  Experts are sharded contiguously (rank r owns experts
[r * NE / N, (r + 1) * NE / N)), router and shared expert are replicated, sequences stay on their rank.
Exchange per step, all fixed-size (no host round trip for counts):
  1. all-gather of every rank's post-norm hidden rows h2 [T, H] bf16, expert ids and routing weights;
  2. every rank runs ITS experts over the gathered tokens (ids stay global, `expert_base` tells the kernel where this
     rank's planes start) and produces fp32 partial sums [N * T, H];
  3. reduce-scatter (sum) returns to each rank the sums of its own T tokens; out = bf16(base + sum).
This moves the same bytes as an exact all-to-all dispatch/return of the routed rows (T * K rows out, T * K rows back)
when T * K / N >= T, which holds for top-8 routing on up to 8 GPUs.
In the reference the same exchange happens between the 4 NPU cores through shared on-chip memory
(models/qwen35_2b/whole/src/q35_layer_mc.py:830-886: logits gathered, expert partial sums added).

Prefill-sized batches (thousands of tokens per rank) use `forward_all_to_all` instead: every routed row goes only to
the rank that owns its expert and comes back weighted, T * K rows each way.
"""
import torch
import torch.distributed as dist


def shard_range(n_experts, rank, world):
    per = n_experts // world
    if per * world != n_experts:
        raise ValueError(f"{n_experts} experts do not divide over {world} ranks")
    return rank * per, (rank + 1) * per


def local_ids(ids, lo, hi):
    """global expert ids -> ids inside this rank's planes; pairs owned by other ranks become -1 (skipped)"""
    inside = (ids >= lo) & (ids < hi)
    return torch.where(inside, ids - lo, torch.full_like(ids, -1))


class ExpertParallelMoE:
    """w: the block's weights with FULL-size expert planes e_gw / e_gs / e_dw / e_ds [NE, ...]; only this rank's
    slice is kept (as a view when already on the device)."""

    def __init__(self, w, top_k, group=None, n_experts=None, exchange="auto"):
        """exchange: "peer" = the two exchanges of forward() through this library's peer-memory kernels (roles
        ep.publish / ep.wait / ep.reduce over a symmetric buffer every rank maps), "nccl" = all-gather + reduce-scatter,
        "auto" = peer when the ranks are GPUs of one node and symmetric memory can be set up, else nccl."""
        self.exchange = exchange
        self._peer = None
        self.group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(self.group), dist.get_world_size(self.group)
        self.top_k = top_k
        self.n_experts = int(n_experts if n_experts is not None else w["w_router"].shape[0])
        self.lo, self.hi = shard_range(self.n_experts, self.rank, self.world)
        self.w = dict(w)
        for n in ("e_gw", "e_gs", "e_dw", "e_ds"):
            t = w[n]
            self.w[n] = t[self.lo:self.hi].contiguous() if t.shape[0] == self.n_experts else t
        self._buf = {}
        self._coalesce = None

    # -- the local compute pieces; the CPU tests override them with the oracle ------------------------------------
    def _dense_part(self, x1):
        """-> (base = bf16(x1 + shared expert), h2, ids, rw, event after which base is ready or None).  On the GPU the
        shared expert runs on a second stream and is only waited for before the closing sum."""
        from . import _lib, moe
        T, H = x1.shape
        dev = x1.device
        w = self.w
        base, h2 = self._get("base", (T, H), x1.dtype, dev), self._get("h2", (T, H), x1.dtype, dev)
        logits = self._get("logits", (T, self.n_experts), torch.float32, dev)
        gate = self._get("gate", (T,), torch.float32, dev)
        ids = self._get("ids", (T, self.top_k), torch.int32, dev)
        rw = self._get("rw", (T, self.top_k), torch.float32, dev)
        # (role moe.front does norm, router, gate dot, softmax and top-k in one launch; measured here it is the slower
        # choice: the shared expert on the second stream can only start once that whole kernel is through, 47 us
        # against 33 us for this part at 2 GPUs, so the short norm + router kernel stays in front of the fork)
        one_launch = False
        if one_launch:
            _lib.run("moe.front", x1=x1, ln2=w["ln2"], w_router=w["w_router"], w_shg=w["w_shg"].reshape(-1), h2_out=h2,
                     logits_out=logits, gate_out=gate, ids=ids, rw=rw)
        else:
            _lib.run("moe.norm_router", x1=x1, ln2=w["ln2"], w_router=w["w_router"], w_shg=w["w_shg"].reshape(-1),
                     h2_out=h2, logits_out=logits, gate_out=gate)
        main, side = torch.cuda.current_stream(dev), moe._side_stream(dev)
        side.wait_stream(main)
        with torch.cuda.stream(side):
            _lib.run("moe.shared", x1=x1, h2=h2, gate=gate, w_gate=w["w_gate"], s_gate=moe._u8(w["s_gate"]),
                     w_up=w["w_up"], s_up=moe._u8(w["s_up"]), w_down=w["w_down"], s_down=moe._u8(w["s_down"]), out=base)
            ready = side.record_event()
        if not one_launch:
            moe.route(logits, self.top_k, ids, rw)
        return base, h2, ids, rw, ready

    def _local_experts(self, h2_all, ids_all, rw_all):
        """fp32 sums over THIS rank's experts for every gathered token; ids are global"""
        from . import _lib, moe
        w = self.w
        partial = self._get("partial", h2_all.shape, torch.float32, h2_all.device)
        if "expert_base" not in self._buf:
            self._buf["expert_base"] = torch.tensor([self.lo], dtype=torch.int32, device=h2_all.device)
        if "e_gs_tiled" not in w and w["e_gs"].is_cuda:  # load-time re-layout of this rank's scales, once
            w["e_gs_tiled"], w["e_ds_tiled"] = moe.tile_scales(w["e_gs"], True), moe.tile_scales(w["e_ds"], False)
        kw = dict(e_gs_tiled=w["e_gs_tiled"], e_ds_tiled=w["e_ds_tiled"]) if "e_gs_tiled" in w else {}
        _lib.run("moe.experts", h2=h2_all, ids=ids_all, rw=rw_all, e_gw=moe._u8(w["e_gw"]), e_gs=moe._u8(w["e_gs"]),
                 e_dw=moe._u8(w["e_dw"]), e_ds=moe._u8(w["e_ds"]), expert_base=self._buf["expert_base"],
                 partial_out=partial, **kw)
        return partial

    def _finish(self, base, mine, out, ready):
        from . import _lib
        if ready is not None:
            torch.cuda.current_stream(base.device).wait_event(ready)
        _lib.run("moe.finish", base=base, partial=mine, out=out)
        return out

    # -------------------------------------------------------------------------------------------------------------
    def _get(self, name, shape, dtype, device):
        key = (name, tuple(shape), dtype)
        if key not in self._buf:
            self._buf[key] = torch.empty(tuple(shape), dtype=dtype, device=device)
        return self._buf[key]

    def _gather(self, pairs):
        """all-gather of several tensors; on NCCL the three go out as ONE grouped launch (torch's coalescing manager,
        the mechanism FSDP uses), which matters at 8 ranks where each collective costs about 20 us of latency"""
        if self._coalesce is None:
            self._coalesce = pairs[0][1].is_cuda and hasattr(dist, "_coalescing_manager")
        if self._coalesce:
            try:
                with dist._coalescing_manager(group=self.group, async_ops=False):
                    for dst, src in pairs:
                        dist.all_gather_into_tensor(dst, src.contiguous(), group=self.group)
                return
            except (RuntimeError, ValueError, TypeError, AttributeError):
                self._coalesce = False  # this torch cannot coalesce them: separate collectives below
        for dst, src in pairs:
            dist.all_gather_into_tensor(dst, src.contiguous(), group=self.group)

    # -- the exchanges through peer memory -----------------------------------------------------------------------
    def _peer_setup(self, x1):
        """One symmetric buffer per rank (torch's symmetric memory: cuMem allocations every rank of the node maps),
        laid out as ep_exchange expects: 1 KB header, then h2_all, ids_all, rw_all, partial.  Returns None when it
        cannot be had (CPU tensors, no symmetric memory): the caller then takes the NCCL exchange."""
        if self._peer is not None:
            return self._peer or None
        self._peer = False
        if self.exchange == "nccl" or not x1.is_cuda:
            return None
        try:
            import torch.distributed._symmetric_memory as symm_mem
            T, H = x1.shape
            N, K = self.world, self.top_k
            al = lambda n: (n + 255) // 256 * 256  # noqa: E731
            o_h2 = 1024
            o_ids = o_h2 + al(N * T * H * 2)
            o_rw = o_ids + al(N * T * K * 4)
            o_par = o_rw + al(N * T * K * 4)
            total = o_par + al(N * T * H * 4)
            buf = symm_mem.empty(total, dtype=torch.uint8, device=x1.device)
            name = self.group.group_name if hasattr(self.group, "group_name") else self.group
            hdl = symm_mem.rendezvous(buf, name)
            buf.zero_()
            torch.cuda.synchronize(x1.device)
            dist.barrier(group=self.group)  # nobody publishes into a buffer that is still being cleared
            view = lambda off, n, dt, shape: buf[off:off + n].view(dt).view(shape)  # noqa: E731
            self._peer = dict(
                T=T, buf=buf, hdl=hdl,
                peers=torch.tensor([int(p) for p in hdl.buffer_ptrs], dtype=torch.int64, device=x1.device).view(torch.uint8),
                rank=torch.tensor([self.rank], dtype=torch.int32, device=x1.device),
                h2_all=view(o_h2, N * T * H * 2, torch.bfloat16, (N * T, H)),
                ids_all=view(o_ids, N * T * K * 4, torch.int32, (N * T, K)),
                rw_all=view(o_rw, N * T * K * 4, torch.float32, (N * T, K)),
                partial=view(o_par, N * T * H * 4, torch.float32, (N * T, H)))
            # the gathered-token buffers of the step ARE the regions of the exchange buffer
            self._buf[("partial", (N * T, H), torch.float32)] = self._peer["partial"]
        except Exception as e:  # noqa: BLE001  (any failure of the optional path: fall back, but say so once)
            if self.exchange == "peer":
                raise
            import warnings
            warnings.warn(f"expert-parallel exchange falls back to NCCL: {type(e).__name__}: {e}")
            self._peer = False
        return self._peer or None

    def _forward_peer(self, x1, out, px, mark):
        from . import _lib
        base, h2, ids, rw, ready = self._dense_part(x1)
        mark("norm + router + route (shared expert on a second stream)")
        common = dict(exchange=px["buf"], peers=px["peers"], rank=px["rank"])
        _lib.run("ep.publish", h2=h2, ids=ids, rw=rw, h2_all=px["h2_all"], ids_all=px["ids_all"], rw_all=px["rw_all"],
                 **common)  # returns in stream order once every rank's rows are here
        mark("rows, ids, weights to every rank (peer stores) and the wait for everybody's")
        partial = self._local_experts(px["h2_all"], px["ids_all"], px["rw_all"])
        assert partial.data_ptr() == px["partial"].data_ptr()
        mark("moe.experts on the gathered tokens, local experts")
        if ready is not None:
            torch.cuda.current_stream(base.device).wait_event(ready)
        _lib.run("ep.reduce", base=base, partial=partial, out=out, **common)
        mark("partial sums of my tokens from every rank (peer loads) + closing sum")
        return out

    def forward(self, x1, out=None, marks=None):
        """marks: a list; when given, a (phase name, CUDA event) pair is appended after every phase of the step, so a
        caller can time the phases on the device (the first entry marks the start)."""
        def mark(name):
            if marks is not None and x1.is_cuda:
                ev = torch.cuda.Event(enable_timing=True)
                ev.record()
                marks.append((name, ev))

        T, H = x1.shape
        N, K = self.world, self.top_k
        mark("start")
        px = self._peer_setup(x1)
        if px is not None and px["T"] == T:
            return self._forward_peer(x1, torch.empty_like(x1) if out is None else out, px, mark)
        base, h2, ids, rw, ready = self._dense_part(x1)
        mark("norm + router + route (shared expert on a second stream)")
        h2_all = self._get("h2_all", (N * T, H), h2.dtype, h2.device)
        ids_all = self._get("ids_all", (N * T, K), ids.dtype, ids.device)
        rw_all = self._get("rw_all", (N * T, K), rw.dtype, rw.device)
        self._gather(((h2_all, h2), (ids_all, ids), (rw_all, rw)))
        mark("all-gather of rows, ids, weights")
        partial = self._local_experts(h2_all, ids_all, rw_all)
        mark("moe.experts on the gathered tokens, local experts")
        mine = self._get("mine", (T, H), torch.float32, x1.device)
        dist.reduce_scatter_tensor(mine, partial, op=dist.ReduceOp.SUM, group=self.group)
        mark("reduce-scatter of the fp32 partial sums")
        out = torch.empty_like(x1) if out is None else out
        out = self._finish(base, mine, out, ready)
        mark("closing sum (waits for the shared expert)")
        return out

    def phases(self, x1, out):
        """[(name, callable)]: the pieces of forward() on the same buffers, each callable on its own (a benchmark
        captures each into a CUDA graph and times its replays; events cannot be placed inside one replayed graph).
        The first piece joins the second stream at its end, so the shared expert's time shows in it instead of
        hiding behind the exchange as it does in forward()."""
        T, H = x1.shape
        N, K = self.world, self.top_k
        st = {}

        def dense():
            st["base"], st["h2"], st["ids"], st["rw"], ready = self._dense_part(x1)
            if ready is not None:
                torch.cuda.current_stream(x1.device).wait_event(ready)

        dense()
        px = self._peer_setup(x1)
        if px is not None and px["T"] == T:
            from . import _lib
            common = dict(exchange=px["buf"], peers=px["peers"], rank=px["rank"])

            def publish():
                _lib.run("ep.publish", h2=st["h2"], ids=st["ids"], rw=st["rw"], h2_all=px["h2_all"],
                         ids_all=px["ids_all"], rw_all=px["rw_all"], **common)

            def experts_p():
                self._local_experts(px["h2_all"], px["ids_all"], px["rw_all"])

            def reduce():
                _lib.run("ep.reduce", base=st["base"], partial=px["partial"], out=out, **common)

            publish(); experts_p(); reduce()  # noqa: E702
            return [("norm + router + route + shared expert (joined)", dense),
                    ("rows, ids, weights to every rank (peer stores) + wait for everybody's", publish),
                    ("moe.experts on the gathered tokens, local experts", experts_p),
                    ("partial sums of my tokens from every rank (peer loads) + closing sum", reduce)]
        h2_all = self._get("h2_all", (N * T, H), st["h2"].dtype, x1.device)
        ids_all = self._get("ids_all", (N * T, K), st["ids"].dtype, x1.device)
        rw_all = self._get("rw_all", (N * T, K), st["rw"].dtype, x1.device)
        mine = self._get("mine", (T, H), torch.float32, x1.device)

        def gather():
            self._gather(((h2_all, st["h2"]), (ids_all, st["ids"]), (rw_all, st["rw"])))

        def experts():
            st["partial"] = self._local_experts(h2_all, ids_all, rw_all)

        def scatter():
            dist.reduce_scatter_tensor(mine, st["partial"], op=dist.ReduceOp.SUM, group=self.group)

        def finish():
            self._finish(st["base"], mine, out, None)

        gather(); experts(); scatter(); finish()  # noqa: E702  (every buffer exists before anything is captured)
        return [("norm + router + route + shared expert (joined)", dense), ("all-gather of rows, ids, weights", gather),
                ("moe.experts on the gathered tokens, local experts", experts),
                ("reduce-scatter of the fp32 partial sums", scatter), ("closing sum", finish)]

    # -- prefill-sized batches: a true all-to-all ---------------------------------------------------------------------
    def _combine(self, base, loc, rows, out):
        from . import _lib
        _lib.run("moe.combine", base=base, loc=loc, sout=rows, out=out)
        return out

    def forward_all_to_all(self, x1, out=None, marks=None):
        """The block on THIS rank's T tokens (every rank holds different tokens) with every token's row sent only to
        the ranks that own one of its experts, once per rank: dispatch all-to-all of (row, its K expert ids, its K
        weights) sorted by destination; the owner runs its experts on the rows it received (landed in its own memory
        first; ids of other ranks' experts are skipped, as in the decode form) and returns ONE weighted partial sum per
        received row; the token's rank adds the returned rows onto the dense part in fp32 (moe_combine arithmetic,
        models/qwen35_2b/whole/src/q35_moe_prefill.py:201-214, with the rank as the slot).  Moves at most
        min(K, N) rows per token each way instead of the N * T rows per rank the all-gather form replicates, which is
        what a prefill of thousands of tokens per rank needs; the per-destination row counts cross the host once per
        call (one small device-to-host copy)."""
        def mark(name):
            if marks is not None and x1.is_cuda:
                ev = torch.cuda.Event(enable_timing=True)
                ev.record()
                marks.append((name, ev))

        T, H = x1.shape
        N, K = self.world, self.top_k
        per = self.n_experts // N
        mark("start")
        base, h2, ids, rw, ready = self._dense_part(x1)
        mark("norm + router + route (shared expert on a second stream)")
        dest = torch.div(ids.long(), per, rounding_mode="floor")                      # [T, K] owning rank of each pick
        member = torch.zeros((N, T), dtype=torch.bool, device=x1.device)
        member[dest.t().reshape(-1), torch.arange(T, device=x1.device).repeat(K)] = True  # rank r owns a pick of token t
        rk, tok = member.nonzero(as_tuple=True)                                        # sorted by rank, then token
        send_counts = member.sum(1)
        counts = torch.empty_like(send_counts)
        dist.all_to_all_single(counts, send_counts, group=self.group)
        both = torch.stack([send_counts, counts]).cpu()          # the one host round trip: split sizes of the exchange
        s_split, r_split = both[0].tolist(), both[1].tolist()
        S, R = int(sum(s_split)), int(sum(r_split))
        send_rows = h2[tok]
        meta = torch.cat([ids[tok].float(), rw[tok].float()], 1).contiguous()          # [S, 2 K]
        rows = torch.empty((R, H), dtype=h2.dtype, device=h2.device)
        rmeta = torch.empty((R, 2 * K), dtype=torch.float32, device=h2.device)
        dist.all_to_all_single(rows, send_rows, r_split, s_split, group=self.group)
        dist.all_to_all_single(rmeta, meta, r_split, s_split, group=self.group)
        mark("dispatch all-to-all (rows, ids, weights)")
        if R:
            partial = self._local_experts(rows, rmeta[:, :K].to(torch.int32).contiguous(), rmeta[:, K:].contiguous())
            res = partial.to(h2.dtype)                           # weighted sums travel back in bf16
        else:
            res = rows
        mark("expert GEMMs on the received rows")
        back = torch.empty((S, H), dtype=h2.dtype, device=h2.device)
        dist.all_to_all_single(back, res, s_split, r_split, group=self.group)
        mark("return all-to-all")
        loc = torch.full((N, T), -1, dtype=torch.int32, device=x1.device)              # slot of (rank, token) or -1
        loc[rk, tok] = torch.arange(S, dtype=torch.int32, device=x1.device)
        out = torch.empty_like(x1) if out is None else out
        if ready is not None:
            torch.cuda.current_stream(base.device).wait_event(ready)
        self._combine(base, loc, back, out)
        mark("combine (waits for the shared expert)")
        return out


    def forward_prefill(self, x1, out=None, form="auto", marks=None, gather_limit_bytes=4 << 30):
        """A prefill-sized call through one of the two exchanges.  form "all_gather": forward() -- every rank receives
        every rank's rows and returns fp32 partial sums of all of them; fixed sizes, no counts, no host round trip, and
        on the peer-memory kernels two launches.  form "all_to_all": forward_all_to_all() -- at most min(K, N) rows per
        token each way, but a count exchange, a host round trip and the index building in front of it.  Inside one
        NVSwitch node the first is the faster one as long as the gathered rows fit (measured at 8192 tokens over 2-8
        GPUs); "auto" takes it while the N * T gathered rows with their fp32 partial sums (6 bytes per element) stay
        under gather_limit_bytes, and the all-to-all beyond."""
        if form == "auto":
            T, H = x1.shape
            form = "all_gather" if self.world * T * H * 6 <= gather_limit_bytes else "all_to_all"
        if form == "all_gather":
            return self.forward(x1, out, marks)
        if form == "all_to_all":
            return self.forward_all_to_all(x1, out, marks)
        raise ValueError(f"form {form!r}: 'auto', 'all_gather' or 'all_to_all'")


# ----------------------------------------------------------------------------------------------------------------
# Tensor parallelism of the dense hybrid stack (27B-class decode group: heads split across 2 / 4 / 8 GPUs).
# The reference splits the same way across its 4 NPU cores: projection rows by head, FFN rows by column block,
# partial sums of the output projections added (models/qwen35_2b/whole/src/q35_layer_mc.py:129-136, 242-423).
# Every sublayer ends in ONE all-reduce of the fp32 partial [tokens, H] of its output projection; the residual is
# added after the sum.  Nothing else crosses GPUs: GDN state, conv state and KV cache are sharded by head.

def _rows(w, s, lo, hi):
    """rows [lo, hi) of a quantised matrix: block scales [N, K/32] and per-row scales [N] follow the rows"""
    return w[lo:hi].contiguous(), s[lo:hi].contiguous()


def _cols(w, s, lo, hi):
    """input columns [lo, hi) (multiples of 32) of a quantised matrix [N, K]: MXFP4 bytes hold two columns each, block
    scales one per 32 columns, per-row fp32 scales are unchanged"""
    if lo % 32 or hi % 32:
        raise ValueError("column shards of quantised weights must be multiples of 32")
    packed = w.dtype == torch.uint8 and s.dim() == 2 and w.shape[1] * 2 == s.shape[1] * 32
    wc = w[:, lo // 2:hi // 2] if packed else w[:, lo:hi]
    sc = s if s.dim() == 1 else s[:, lo // 32:hi // 32]
    return wc.contiguous(), sc.contiguous()


def shard_gdn_weights(w, rank, world, head_dim=128):
    """this rank's value heads [rank * NV / N, ...) and the key heads they use (grouped map kh = vh // (NV / NK))"""
    NV = w["a_log"].numel()
    NK = w["w_q"].shape[0] // head_dim
    if NV % world or NK % world:
        raise ValueError(f"{NV} value / {NK} key heads do not divide over {world} ranks")
    v0, v1 = rank * NV // world, (rank + 1) * NV // world
    k0, k1 = rank * NK // world, (rank + 1) * NK // world
    out = dict(input_norm_w=w["input_norm_w"], o_norm_w=w["o_norm_w"], a_log=w["a_log"][v0:v1].contiguous(),
               dt_bias=w["dt_bias"][v0:v1].contiguous())
    for n, (lo, hi) in (("q", (k0 * head_dim, k1 * head_dim)), ("k", (k0 * head_dim, k1 * head_dim)),
                        ("v", (v0 * head_dim, v1 * head_dim)), ("z", (v0 * head_dim, v1 * head_dim)),
                        ("a", (v0, v1)), ("b", (v0, v1))):
        out["w_" + n], out["s_" + n] = _rows(w["w_" + n], w["s_" + n], lo, hi)
    for n, (lo, hi) in (("q", (k0, k1)), ("k", (k0, k1)), ("v", (v0, v1))):
        out[f"w_{n}_conv"] = w[f"w_{n}_conv"][lo * head_dim:hi * head_dim].contiguous()
    out["w_o"], out["s_o"] = _cols(w["w_o"], w["s_o"], v0 * head_dim, v1 * head_dim)
    return out


def shard_attention_weights(w, rank, world, heads, kv_heads, head_dim, gated=True):
    """this rank's query heads; its KV heads while world <= kv_heads, else the single KV head its query heads belong to
    (ranks sharing a KV head each keep that head's cache: no exchange inside the attention).
    Returns (weights, local heads, local kv heads)."""
    if heads % world:
        raise ValueError(f"{heads} query heads do not divide over {world} ranks")
    hl = heads // world
    h0 = rank * hl
    per_q = head_dim * (2 if gated else 1)  # rows per head in w_q: [q | gate]
    if kv_heads % world == 0:
        kl = kv_heads // world
        kv0 = rank * kl
    else:
        group = heads // kv_heads
        if world % kv_heads or group % hl:
            raise ValueError(f"{heads} / {kv_heads} heads cannot be split over {world} ranks by whole KV-head groups")
        kl, kv0 = 1, h0 // group
    out = dict(ln1=w["ln1"], q_norm=w["q_norm"], k_norm=w["k_norm"])
    out["w_q"], out["s_q"] = _rows(w["w_q"], w["s_q"], h0 * per_q, (h0 + hl) * per_q)
    for n in ("k", "v"):
        out["w_" + n], out["s_" + n] = _rows(w["w_" + n], w["s_" + n], kv0 * head_dim, (kv0 + kl) * head_dim)
    out["w_o"], out["s_o"] = _cols(w["w_o"], w["s_o"], h0 * head_dim, (h0 + hl) * head_dim)
    return out, hl, kl


def shard_mlp_weights(w, rank, world):
    """rows [rank * F / N, ...) of gate and up, the same columns of down"""
    F = w["w_gate"].shape[0]
    if F % (32 * world):
        raise ValueError(f"intermediate size {F} does not divide over {world} ranks in multiples of 32")
    lo, hi = rank * F // world, (rank + 1) * F // world
    out = dict(ln2=w["ln2"])
    for n in ("gate", "up"):
        out["w_" + n], out["s_" + n] = _rows(w["w_" + n], w["s_" + n], lo, hi)
    out["w_down"], out["s_down"] = _cols(w["w_down"], w["s_down"], lo, hi)
    return out


def shard_stack_weights(layers, kinds, rank, world, *, heads, kv_heads, head_dim, gated=True, gdn_head_dim=128):
    """per-layer shards of a hybrid stack; returns (layers, local heads, local kv heads)"""
    out, hl, kl = [], heads // world, max(1, kv_heads // world)
    for w, kind in zip(layers, kinds):
        if kind == "g":
            lw = shard_gdn_weights(w, rank, world, gdn_head_dim)
        else:
            lw, hl, kl = shard_attention_weights(w, rank, world, heads, kv_heads, head_dim, gated)
        lw.update(shard_mlp_weights(w, rank, world))
        out.append(lw)
    return out, hl, kl


def all_reduce_sum(group=None):
    """the `reduce` hook of the sublayers: in-place sum of the fp32 partial over the group"""
    def reduce(partial):
        dist.all_reduce(partial, op=dist.ReduceOp.SUM, group=group)
        return partial
    return reduce


class PeerAllReduce:
    """The `reduce` hook through this library's one-kernel all-reduce over peer memory (role ar.oneshot): every rank
    stores its fp32 partial into a slot of every rank's symmetric buffer, flags, waits, and adds the slots in rank
    order.  Made for the few hundred kilobytes a decode step reduces after each output projection, where a collective's
    latency is the cost.  Tensors of another size than the first one seen, CPU tensors and hosts without symmetric
    memory take dist.all_reduce."""

    def __init__(self, group=None, mode="auto"):
        self.group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(self.group), dist.get_world_size(self.group)
        self.mode = mode
        self._px = None

    def _setup(self, partial):
        if self._px is not None:
            return self._px or None
        self._px = False
        if self.mode == "nccl" or not partial.is_cuda or partial.numel() % 4 or partial.dtype != torch.float32:
            return None
        try:
            import torch.distributed._symmetric_memory as symm_mem
            slot = (partial.numel() * 4 + 255) // 256 * 256
            buf = symm_mem.empty(1024 + 2 * self.world * slot, dtype=torch.uint8, device=partial.device)
            name = self.group.group_name if hasattr(self.group, "group_name") else self.group
            hdl = symm_mem.rendezvous(buf, name)
            buf.zero_()
            torch.cuda.synchronize(partial.device)
            dist.barrier(group=self.group)
            self._px = dict(numel=partial.numel(), buf=buf, hdl=hdl, out=torch.empty_like(partial),
                            peers=torch.tensor([int(p) for p in hdl.buffer_ptrs], dtype=torch.int64,
                                               device=partial.device).view(torch.uint8),
                            rank=torch.tensor([self.rank], dtype=torch.int32, device=partial.device))
        except Exception as e:  # noqa: BLE001
            if self.mode == "peer":
                raise
            import warnings
            warnings.warn(f"tensor-parallel all-reduce falls back to NCCL: {type(e).__name__}: {e}")
            self._px = False
        return self._px or None

    def __call__(self, partial):
        px = self._setup(partial)
        if px is None or px["numel"] != partial.numel():
            dist.all_reduce(partial, op=dist.ReduceOp.SUM, group=self.group)
            return partial
        from . import _lib
        out = px["out"].view(partial.shape)
        _lib.run("ar.oneshot", x=partial.contiguous(), peers=px["peers"], rank=px["rank"], exchange=px["buf"], out=out)
        return out


def tensor_parallel_stack(layers, kinds, *, heads, kv_heads, head_dim, group=None, gated=True, **stack_kw):
    """layers.HybridStack over this rank's shards with an all-reduce after each of the two sublayers of a layer"""
    from .layers import HybridStack
    g = group if group is not None else dist.group.WORLD
    rank, world = dist.get_rank(g), dist.get_world_size(g)
    shards, hl, kl = shard_stack_weights(layers, kinds, rank, world, heads=heads, kv_heads=kv_heads, head_dim=head_dim,
                                         gated=gated)
    return HybridStack(shards, kinds, heads=hl, kv_heads=kl, head_dim=head_dim, gated=gated, reduce=all_reduce_sum(g),
                       **stack_kw)


def tensor_parallel_decode_group(layers, kinds, *, batch, heads, kv_heads, head_dim, group=None, gated=True,
                                 reduce="auto", **group_kw):
    """layers.DecodeGroup (B sequences, one token each per step) over this rank's shards: heads, GDN value heads and FFN
    columns split over the group, one all-reduce of the fp32 partial [B, H] after each sublayer's output projection --
    the split of the 27B-class decode group over 2 / 4 / 8 devices (models/qwen38_27b/decode/q35_group.py:128-137)."""
    from .layers import DecodeGroup
    g = group if group is not None else dist.group.WORLD
    rank, world = dist.get_rank(g), dist.get_world_size(g)
    shards, hl, kl = shard_stack_weights(layers, kinds, rank, world, heads=heads, kv_heads=kv_heads, head_dim=head_dim,
                                         gated=gated)
    # reduce: "auto" / "peer" = the one-kernel all-reduce over peer memory (PeerAllReduce), "nccl" = dist.all_reduce
    hook = all_reduce_sum(g) if reduce == "nccl" else PeerAllReduce(g, reduce)
    return DecodeGroup(shards, kinds, batch=batch, heads=hl, kv_heads=kl, head_dim=head_dim, gated=gated,
                       reduce=hook, **group_kw)


# ----------------------------------------------------------------------------------------------------------------
# Paged attention decode split over GPUs (the standalone attention configuration: batch 64, 16 q / 2 kv heads).
# Query heads go with their KV head.  While there are at least as many KV heads as ranks, a rank owns whole KV heads
# and nothing is exchanged inside the attention.  With more ranks than KV heads, the S = world / HKV ranks that share
# a KV head split every sequence's PAGES among themselves (contiguous shares), each computes the unnormalised
# partial (m, l, o) over its pages (role attn.paged_decode with part_* outputs), the partials are all-gathered and
# merged by log-sum-exp (role attn.lse_merge) -- the pair scheme of the reference's multi-core attention
# (models/qwen35_35b_a3b/sgl/python/sgl_kernel_axera/attention/flash_attn.py:2393-2474;
#  models/qwen35_2b/whole/src/q35_layer_mc.py:308-379).

def attention_split(heads, kv_heads, world, rank):
    """-> dict(kv0, kv1: this rank's KV heads [kv0, kv1); q0, q1: its query heads; share, shares: its part of the pages)"""
    group = heads // kv_heads
    if world <= kv_heads:
        if kv_heads % world:
            raise ValueError(f"{kv_heads} KV heads do not divide over {world} ranks")
        per = kv_heads // world
        kv0 = rank * per
        return dict(kv0=kv0, kv1=kv0 + per, q0=kv0 * group, q1=(kv0 + per) * group, share=0, shares=1)
    if world % kv_heads:
        raise ValueError(f"{world} ranks do not divide over {kv_heads} KV heads")
    shares = world // kv_heads
    kv0 = rank // shares
    return dict(kv0=kv0, kv1=kv0 + 1, q0=kv0 * group, q1=(kv0 + 1) * group, share=rank % shares, shares=shares)


def split_page_table(indptr, indices, last_page_len, page, share, shares):
    """the contiguous share `share` of `shares` of every sequence's pages (host tensors in, host tensors out): pages
    [share * n / shares, (share + 1) * n / shares) of a sequence with n pages; only the rank that holds a sequence's final
    page sees its partial fill, the others see full pages.  Returns (indptr, indices, last_page_len)."""
    ip, out_idx, out_last = [0], [], []
    for b in range(indptr.numel() - 1):
        a0, a1 = int(indptr[b]), int(indptr[b + 1])
        n = a1 - a0
        lo, hi = share * n // shares, (share + 1) * n // shares
        out_idx.extend(indices[a0 + lo:a0 + hi].tolist())
        ip.append(ip[-1] + (hi - lo))
        out_last.append(int(last_page_len[b]) if hi == n else page)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32)  # noqa: E731
    return i32(ip), i32(out_idx or [0]), i32(out_last)


class HeadSplitAttention:
    """paged attention decode over the ranks of a group: q [B, HQ, D] (replicated) -> out [B, HQ, D] (replicated).
    The rank's cache holds ITS KV heads only ([pages, 2, P, kv_local, D]) and its page table ITS share of the pages.
    local / merge: the compute pieces (default: the library's roles; the CPU tests inject the oracle)."""

    def __init__(self, heads, kv_heads, group=None, local=None, merge=None):
        self.group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(self.group), dist.get_world_size(self.group)
        self.heads, self.kv_heads = heads, kv_heads
        self.plan = attention_split(heads, kv_heads, self.world, self.rank)
        self._local = local or self._gpu_partial
        self._merge = merge or self._gpu_merge
        self._buf = {}

    def _get(self, name, shape, dtype, device):
        key = (name, tuple(shape), dtype)
        if key not in self._buf:
            self._buf[key] = torch.empty(tuple(shape), dtype=dtype, device=device)
        return self._buf[key]

    def _gpu_partial(self, q, cache, indptr, indices, last_page_len, sm_scale, kv_scale, packed):
        from . import _lib
        kw = dict(q=q, paged_kv_cache=cache, indptr=indptr, indices=indices, last_page_len=last_page_len,
                  part_packed=packed)  # the kernel writes o | m | l of every row straight into the message
        if sm_scale is not None:
            kw["sm_scale"] = sm_scale
        if kv_scale is not None:
            kw["kv_scale"] = kv_scale
        _lib.run("attn.paged_decode", **kw)

    def _gpu_merge(self, gathered, out):
        from . import _lib
        B = out.shape[0]
        _lib.run("attn.lse_merge", packed=gathered.reshape(self.world, B, -1, gathered.shape[-1]), out=out)

    @staticmethod
    def unpack(gathered, world, shares):
        """gathered [world * B, Hq, D + 2] (ranks along dim 0, KV group major) -> (m, l, o) as [shares, B, HQ] and
        [shares, B, HQ, D]: the separate-tensor form of the merge (what a CPU merge takes)"""
        B, Hq, W = gathered.shape[0] // world, gathered.shape[1], gathered.shape[2]
        n_kv = world // shares
        g = gathered.reshape(n_kv, shares, B, Hq, W).permute(1, 2, 0, 3, 4).reshape(shares, B, n_kv * Hq, W)
        return g[..., W - 2].contiguous(), g[..., W - 1].contiguous(), g[..., :W - 2].contiguous()

    def forward(self, q, cache, indptr, indices, last_page_len, out=None, sm_scale=None, kv_scale=None):
        """q [B, HQ, D]: every rank passes the full query; cache / page table: this rank's (see class docstring)"""
        B, HQ, D = q.shape
        p = self.plan
        ql = q[:, p["q0"]:p["q1"]].contiguous()
        Hq = ql.shape[1]
        packed = self._get("packed", (B, Hq, D + 2), torch.float32, q.device)  # o | m | l, one message per rank
        self._local(ql, cache, indptr, indices, last_page_len, sm_scale, kv_scale, packed)
        gathered = self._get("gathered", (self.world * B, Hq, D + 2), torch.float32, q.device)  # ranks along dim 0
        dist.all_gather_into_tensor(gathered, packed, group=self.group)
        out = torch.empty((B, HQ, D), dtype=q.dtype, device=q.device) if out is None else out
        self._merge(gathered, out)
        return out
