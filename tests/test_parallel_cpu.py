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
        return base, h2, ids, rw

    def _local_experts(self, h2_all, ids_local, rw_all):
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
        ret[rank] = float(err)
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
