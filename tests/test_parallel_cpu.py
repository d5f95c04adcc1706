"""Expert-parallel host logic on CPU: 2 ranks over gloo, the per-rank compute supplied by the CPU oracle.
Checks the sharding, the id remapping and the all-gather / reduce-scatter plumbing against the unsharded oracle."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from ax_dsl_kernels_b200 import parallel
from oracle import codecs, moe as omoe


def _weights(seed, NE=8, H=64, FE=32, FS=32):
    g = torch.Generator().manual_seed(seed)
    w = dict(ln2=torch.ones(H), w_router=(torch.randn((NE, H), generator=g) / 8).to(torch.bfloat16),
             w_shg=(torch.randn((H,), generator=g) / 8).to(torch.bfloat16))
    w["e_gw"], w["e_gs"] = codecs.random_mxfp4((NE, 2 * FE, H), g, -3, 0)
    w["e_dw"], w["e_ds"] = codecs.random_mxfp4((NE, H, FE), g, -3, 0)
    for n, shp in (("gate", (FS, H)), ("up", (FS, H)), ("down", (H, FS))):
        w["w_" + n], w["s_" + n] = codecs.random_mxfp4(shp, g, -3, 0)
    return w


class OracleEP(parallel.ExpertParallelMoE):
    def _dense_part(self, x1):
        w = self.w
        deq = [codecs.dequant_mxfp4(w["w_" + n], w["s_" + n]) for n in ("gate", "up", "down")]
        base, h2, logits = omoe.moe_pre(x1, w["ln2"], *deq, w["w_router"], w["w_shg"])
        ids, rw = omoe.route(logits, self.top_k)
        return base, h2, ids, rw, None

    def _finish(self, base, mine, out, ready):
        out.copy_((base.float() + mine).to(out.dtype))
        return out

    def _local_experts(self, h2_all, ids_all, rw_all):
        ids_local = parallel.local_ids(ids_all, self.lo, self.hi)
        w = self.w
        partial = torch.zeros(h2_all.shape)
        zero = torch.zeros_like(h2_all)
        for t in range(h2_all.shape[0]):
            keep = ids_local[t] >= 0
            if keep.any():
                o = omoe.experts_decode(h2_all[t:t + 1], zero[t:t + 1], ids_local[t:t + 1, keep], rw_all[t:t + 1, keep],
                                        w["e_gw"], w["e_gs"], w["e_dw"], w["e_ds"])
                # experts_decode rounds to bf16; redo the sum in fp32 for the partial
                acc = torch.zeros(h2_all.shape[1])
                FE = w["e_gw"].shape[1] // 2
                for i in keep.nonzero().flatten().tolist():
                    e = int(ids_local[t, i])
                    wc, wd = codecs.dequant_mxfp4(w["e_gw"][e], w["e_gs"][e]), codecs.dequant_mxfp4(w["e_dw"][e], w["e_ds"][e])
                    gu = omoe.bf(wc @ h2_all[t].float())
                    a = omoe.bf(torch.nn.functional.silu(gu[:FE]) * gu[FE:])
                    acc += rw_all[t, i] * (wd @ a)
                partial[t] = acc
                del o
        return partial


    def _combine(self, base, loc, rows, out):
        acc = base.float()
        for k in range(loc.shape[0]):
            have = loc[k] >= 0
            acc[have] += rows[loc[k][have].long()].float()
        out.copy_(acc.to(out.dtype))
        return out


def _a2a_worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        w = _weights(5)
        g = torch.Generator().manual_seed(200 + rank)
        T = 5 + 2 * rank  # a different number of tokens on every rank
        x1 = torch.randn((T, 64), generator=g).to(torch.bfloat16)
        ep = OracleEP(w, top_k=3)
        out = ep.forward_all_to_all(x1)
        deq = [codecs.dequant_mxfp4(w["w_" + n], w["s_" + n]) for n in ("gate", "up", "down")]
        ref, _, _, _ = omoe.moe_block(x1, w["ln2"], *deq, w["w_router"], w["w_shg"], w["e_gw"], w["e_gs"], w["e_dw"],
                                      w["e_ds"], 3)
        ret[rank] = float((out.float() - ref.float()).abs().max() / ref.float().square().mean().sqrt())
    finally:
        dist.destroy_process_group()


def test_expert_parallel_all_to_all_dispatch_two_and_four_ranks_gloo():
    """prefill form: every routed row travels only to the rank that owns its expert and comes back weighted; ranks hold
    different token counts; the result equals the single-process golden block"""
    for world in (2, 4):
        s = socket.socket()
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
        s.close()
        ret = mp.Manager().dict()
        mp.spawn(_a2a_worker, args=(world, port, ret), nprocs=world, join=True)
        assert len(ret) == world and all(v <= 2e-2 for v in ret.values()), dict(ret)


def _worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        w = _weights(5)
        g = torch.Generator().manual_seed(100 + rank)
        x1 = torch.randn((3, 64), generator=g).to(torch.bfloat16)
        ep = OracleEP(w, top_k=3)
        assert (ep.lo, ep.hi) == (rank * 4, rank * 4 + 4) and ep.w["e_gw"].shape[0] == 4
        out = ep.forward(x1)
        deq = [codecs.dequant_mxfp4(w["w_" + n], w["s_" + n]) for n in ("gate", "up", "down")]
        ref, _, _, _ = omoe.moe_block(x1, w["ln2"], *deq, w["w_router"], w["w_shg"], w["e_gw"], w["e_gs"], w["e_dw"],
                                      w["e_ds"], 3)
        err = (out.float() - ref.float()).abs().max() / ref.float().square().mean().sqrt()
        # the prefill entry: the same exchange under "auto" while the gathered rows fit, the all-to-all beyond
        same = ep.forward_prefill(x1)
        a2a = ep.forward_prefill(x1, gather_limit_bytes=0)
        assert torch.equal(same, out)
        err2 = (a2a.float() - ref.float()).abs().max() / ref.float().square().mean().sqrt()
        ret[rank] = float(max(err, err2))
    finally:
        dist.destroy_process_group()


def test_expert_parallel_two_ranks_gloo():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(2, port, ret), nprocs=2, join=True)
    assert len(ret) == 2 and all(v <= 2e-2 for v in ret.values()), dict(ret)


def test_shard_range_and_local_ids():
    assert parallel.shard_range(256, 3, 8) == (96, 128)
    with pytest.raises(ValueError):
        parallel.shard_range(10, 0, 4)
    ids = torch.tensor([[0, 5, 9], [4, 7, 8]], dtype=torch.int32)
    assert parallel.local_ids(ids, 4, 8).tolist() == [[-1, 1, -1], [0, 3, -1]]


# ----------------------------------------------------------------------------------------------------------------
# tensor parallelism: the sharding of heads / FFN columns and the all-reduce, with the oracle as the local compute
def _deq(w):
    out = {}
    for k, v in w.items():
        if k.startswith("w_") and ("s_" + k[2:]) in w:
            out[k] = codecs.dequant_fp8_rowwise(v, w["s_" + k[2:]])
        elif not k.startswith("s_"):
            out[k] = v
    return out


def _tp_worker(rank, world, port, ret):
    import sys
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from _cases import stack_case
    from oracle import attention as oattn, gdn as ogdn, stack as ostack
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        H, heads, kv_heads, D, NK, NV, DV = 256, 4, 1, 64, 2, 4, 32  # kv_heads < world: the KV head is replicated
        kw, ow = stack_case("ga", H=H, F=128, heads=heads, kv_heads=kv_heads, head_dim=D, NK=NK, NV=NV, DV=DV, seed=3)
        reduce = parallel.all_reduce_sum()
        g = torch.Generator().manual_seed(9)
        x = (torch.randn((2, 1, H), generator=g) * 0.5).to(torch.bfloat16)
        errs = {}

        def rel(a, b):
            return float((a.float() - b.float()).abs().max() / b.float().square().mean().sqrt())

        # GDN sublayer: value heads [rank * 2, rank * 2 + 2), key head rank
        lw = _deq(parallel.shard_gdn_weights(kw[0], rank, world, head_dim=DV))
        assert lw["w_v"].shape[0] == NV // world * DV and lw["w_o"].shape == (H, NV // world * DV)
        st = torch.randn((2, NV, DV, DV), generator=g) * 0.03
        cs = (torch.randn((2, 3, 2 * NK * DV + NV * DV), generator=g) * 0.1).to(torch.bfloat16)
        zero = torch.zeros_like(x)
        full, st_full, _ = ogdn.gdn_sublayer(x, zero, ow[0], st, cs)
        k0, v0 = rank * NK // world * DV, rank * NV // world * DV
        kd, vd = NK * DV, NV * DV
        cs_l = torch.cat((cs[..., k0:k0 + kd // world], cs[..., kd + k0:kd + k0 + kd // world],
                          cs[..., 2 * kd + v0:2 * kd + v0 + vd // world]), -1)
        st_l = st[:, rank * NV // world:(rank + 1) * NV // world]
        part, st_out, _ = ogdn.gdn_sublayer(x, zero, lw, st_l, cs_l)
        partial = part.float() - x.float()  # the sublayer adds the residual; take it off again
        out = (x.float() + reduce(partial)).to(torch.bfloat16)
        errs["gdn"] = rel(out, full)
        errs["gdn_state"] = rel(st_out, st_full[:, rank * NV // world:(rank + 1) * NV // world])

        # attention sublayer (decode, 5 tokens of history)
        aw, hl, kl = parallel.shard_attention_weights(kw[1], rank, world, heads, kv_heads, D)
        assert (hl, kl) == (2, 1) and aw["w_q"].shape[0] == 2 * 2 * D and aw["w_o"].shape == (H, 2 * D)
        cache = (torch.randn((2, 2, 8, kv_heads, D), generator=g)).to(torch.bfloat16)
        indptr, indices = torch.tensor([0, 1, 2], dtype=torch.int32), torch.tensor([0, 1], dtype=torch.int32)
        last = torch.tensor([5, 5], dtype=torch.int32)
        loc = torch.tensor([[0, 5], [1, 5]], dtype=torch.int32)
        cos, sin = oattn.rope_cos_sin(torch.tensor([5, 5]), 16, 1e7)
        x2 = x.reshape(2, H)
        kwa = dict(head_dim=D, rot=16, gated=True)
        full = ostack.attn_sublayer(x2, ow[1], cache.clone(), indptr, indices, last, cos, sin, heads=heads,
                                    kv_heads=kv_heads, cache_location=loc, **kwa)
        part = ostack.attn_sublayer(x2, _deq(aw), cache.clone(), indptr, indices, last, cos, sin, heads=hl, kv_heads=kl,
                                    cache_location=loc, **kwa)
        out = (x2.float() + reduce(part.float() - x2.float())).to(torch.bfloat16)
        errs["attn"] = rel(out, full)

        # dense FFN
        mw = _deq(parallel.shard_mlp_weights(kw[0], rank, world))
        full = ostack.dense_mlp(x2, ow[0]["ln2"], ow[0]["w_gate"], ow[0]["w_up"], ow[0]["w_down"])
        part = ostack.dense_mlp(x2, mw["ln2"], mw["w_gate"], mw["w_up"], mw["w_down"])
        out = (x2.float() + reduce(part.float() - x2.float())).to(torch.bfloat16)
        errs["mlp"] = rel(out, full)
        ret[rank] = errs
    finally:
        dist.destroy_process_group()


def test_tensor_parallel_shards_two_ranks_gloo():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ret = mp.Manager().dict()
    mp.spawn(_tp_worker, args=(2, port, ret), nprocs=2, join=True)
    assert len(ret) == 2
    for errs in ret.values():
        # each rank's partial went through one extra bf16 rounding (the oracle sublayer rounds before the residual)
        assert all(v <= 3e-2 for v in errs.values()), dict(ret)


def test_column_shard_of_block_scaled_weights():
    g = torch.Generator().manual_seed(1)
    w, s = codecs.random_mxfp4((8, 128), g, -3, 0)
    wc, sc = parallel._cols(w, s, 64, 128)
    assert torch.equal(codecs.dequant_mxfp4(wc, sc), codecs.dequant_mxfp4(w, s)[:, 64:128])
    with pytest.raises(ValueError):
        parallel._cols(w, s, 16, 128)


# ----------------------------------------------------------------------------------------------------------------
# attention split over ranks: KV heads per rank, pages split inside a KV head, LSE merge of the all-gathered partials
def _attn_worker(rank, world, port, ret):
    import sys
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from _cases import paged_case
    from oracle import attention as oattn
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        HQ, HKV, D, P = 8, 2, 64, 16
        q, cache, indptr, indices, last, _ = paged_case([5, 40, 333, 0, 16], P=P, HKV=HKV, HQ=HQ, D=D, seed=7)
        ref = oattn.paged_decode(q, cache, indptr, indices, last)

        def local(ql, c, ip, ix, lp, sm, kvs, packed):
            m, ln, o = oattn.paged_decode_partial(ql, c, ip, ix, lp)
            packed[..., :D], packed[..., D], packed[..., D + 1] = o, m, ln

        def merge(gathered, out):
            pm, pl, po = parallel.HeadSplitAttention.unpack(gathered, world, world // HKV)
            out.copy_(oattn.lse_merge(pm, pl, po))

        att = parallel.HeadSplitAttention(HQ, HKV, local=local, merge=merge)
        pl_ = att.plan
        assert (pl_["shares"], pl_["kv0"], pl_["share"]) == (world // HKV, rank // (world // HKV), rank % (world // HKV))
        my_cache = cache[:, :, :, pl_["kv0"]:pl_["kv1"]].contiguous()
        ip, ix, lp = parallel.split_page_table(indptr, indices, last, P, pl_["share"], pl_["shares"])
        out = att.forward(q, my_cache, ip, ix, lp)
        ret[rank] = float((out.float() - ref.float()).abs().max() / ref.float().square().mean().sqrt())
    finally:
        dist.destroy_process_group()


def test_attention_pages_split_inside_kv_heads_four_ranks_gloo():
    """4 ranks, 2 KV heads: two ranks share each KV head and split every sequence's pages; the all-gathered partials
    merged by log-sum-exp equal the unsplit golden on every rank"""
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ret = mp.Manager().dict()
    mp.spawn(_attn_worker, args=(4, port, ret), nprocs=4, join=True)
    assert len(ret) == 4 and all(v <= 1e-2 for v in ret.values()), dict(ret)


def test_attention_split_plan_and_page_shares():
    assert parallel.attention_split(16, 2, 2, 1) == dict(kv0=1, kv1=2, q0=8, q1=16, share=0, shares=1)
    assert parallel.attention_split(16, 2, 8, 5) == dict(kv0=1, kv1=2, q0=8, q1=16, share=1, shares=4)
    assert parallel.attention_split(24, 4, 2, 0) == dict(kv0=0, kv1=2, q0=0, q1=12, share=0, shares=1)
    with pytest.raises(ValueError):
        parallel.attention_split(16, 2, 3, 0)
    indptr = torch.tensor([0, 5, 5, 6], dtype=torch.int32)
    indices = torch.tensor([9, 8, 7, 6, 5, 4], dtype=torch.int32)
    last = torch.tensor([3, 0, 11], dtype=torch.int32)
    got = [parallel.split_page_table(indptr, indices, last, 16, s, 2) for s in range(2)]
    assert got[0][0].tolist() == [0, 2, 2, 2] and got[0][1].tolist() == [9, 8] and got[0][2].tolist() == [16, 0, 16]
    assert got[1][0].tolist() == [0, 3, 3, 4] and got[1][1].tolist() == [7, 6, 5, 4] and got[1][2].tolist() == [3, 0, 11]
