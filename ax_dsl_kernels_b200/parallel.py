"""Multi-GPU host logic: one process per GPU, torch.distributed for the plumbing (NCCL on GPUs; the same code runs
over gloo on CPU in the tests, with the local compute injected).

Expert parallelism for decode-sized batches.  Experts are sharded contiguously (rank r owns experts
[r * NE / N, (r + 1) * NE / N)), router and shared expert are replicated, sequences stay on their rank.
Exchange per step, all fixed-size (no host round trip for counts):
  1. all-gather of every rank's post-norm hidden rows h2 [T, H] bf16, expert ids and routing weights;
  2. every rank runs ITS experts over the gathered tokens and produces fp32 partial sums [N * T, H];
  3. reduce-scatter (sum) returns to each rank the sums of its own T tokens; out = bf16(base + sum).
This moves the same bytes as an exact all-to-all dispatch/return of the routed rows (T * K rows out, T * K rows back)
when T * K / N >= T, which holds for top-8 routing on up to 8 GPUs.
In the reference the same exchange happens between the 4 NPU cores through shared on-chip memory
(models/qwen35_2b/whole/src/q35_layer_mc.py:830-886: logits gathered, expert partial sums added).
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

    def __init__(self, w, top_k, group=None, n_experts=None):
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

    # -- the three local compute pieces; the CPU tests override them with the oracle ------------------------------
    def _dense_part(self, x1):
        from . import moe
        T, H = x1.shape
        base, h2 = torch.empty_like(x1), torch.empty_like(x1)
        logits = torch.empty((T, self.n_experts), dtype=torch.float32, device=x1.device)
        w = self.w
        moe.moe_pre(x1, w["ln2"], w["w_gate"], w["s_gate"], w["w_up"], w["s_up"], w["w_down"], w["s_down"],
                    w["w_router"], w["w_shg"], base, h2, logits)
        ids, rw = moe.route(logits, self.top_k)
        return base, h2, ids, rw

    def _local_experts(self, h2_all, ids_local, rw_all):
        from . import _lib
        w = self.w
        partial = self._get("partial", h2_all.shape, torch.float32, h2_all.device)
        _lib.run("moe.experts", h2=h2_all, ids=ids_local, rw=rw_all, e_gw=w["e_gw"], e_gs=w["e_gs"], e_dw=w["e_dw"],
                 e_ds=w["e_ds"], partial_out=partial)
        return partial

    # -------------------------------------------------------------------------------------------------------------
    def _get(self, name, shape, dtype, device):
        key = (name, tuple(shape), dtype)
        if key not in self._buf:
            self._buf[key] = torch.empty(tuple(shape), dtype=dtype, device=device)
        return self._buf[key]

    def forward(self, x1, out=None):
        T, H = x1.shape
        N, K = self.world, self.top_k
        base, h2, ids, rw = self._dense_part(x1)
        h2_all = self._get("h2_all", (N * T, H), h2.dtype, h2.device)
        ids_all = self._get("ids_all", (N * T, K), ids.dtype, ids.device)
        rw_all = self._get("rw_all", (N * T, K), rw.dtype, rw.device)
        dist.all_gather_into_tensor(h2_all, h2.contiguous(), group=self.group)
        dist.all_gather_into_tensor(ids_all, ids.contiguous(), group=self.group)
        dist.all_gather_into_tensor(rw_all, rw.contiguous(), group=self.group)
        partial = self._local_experts(h2_all, local_ids(ids_all, self.lo, self.hi), rw_all)
        mine = self._get("mine", (T, H), torch.float32, x1.device)
        dist.reduce_scatter_tensor(mine, partial, op=dist.ReduceOp.SUM, group=self.group)
        out = torch.empty_like(x1) if out is None else out
        out.copy_((base.float() + mine).to(out.dtype))
        return out
