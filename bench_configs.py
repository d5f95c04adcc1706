"""The other configurations of the hot path as benchmark lines (`python bench.py --config NAME`), one JSON line each in
the schema of the headline line:

  c2, c2_fp8   paged attention decode alone: batch 64, contexts uniform in [1024, 16384] (seed 1), page 64, permuted
               pages, bf16 KV / FP8 E4M3 KV with per-head scales
  c3_decode    GDN recurrent state update, batch 64, 32 value / 16 key heads
  c3_prefill   GDN chunked prefill of 16384 tokens, chunk 64
  c4_decode    MoE block at decode batch 64 (256 experts, top-8, shared expert)
  c4_prefill   MoE block on 8192 tokens, against the block-scaled tensor-core peak measured in the same run
  c5, c5_fp8   27B-class dense decode group: 16 layers (g g g a x 4), hidden 5120, batch 8, every sequence at a context
               of 131072 tokens, FP8 per-row weights, bf16 / FP8 KV; with --gpus N the heads, GDN value heads and FFN
               columns are split over N GPUs (one all-reduce per sublayer, strong scaling)

A step is one pass of the configuration over its synthetic seeded inputs; timing as in bench.py (rounds of K steps, CUDA
events, median round, max over ranks); `e2e` copies the step's activations from pinned host memory and its result back
inside the timed region.
"""
import json
import math
import os

import torch

import bench as hb

PAGE, HQ, HKV, D = 64, 16, 2, 256


def _finish(args, name, metric, unit_items, step, ins, outs, roofline, config, dist=None, dev=None, extra=None,
            scaling="weak", graph_ok=True):
    """times `step` (graph replay on one GPU), the end-to-end variant, samples clocks, prints the line on rank 0"""
    import ax_dsl_kernels_b200 as q35
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    L = q35._lib.lib()

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def agree(ms):
        if dist is None:
            return ms
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    clocks = hb.ClockSampler(torch.cuda.current_device()) if rank == 0 else None
    if clocks:
        clocks.start()
    warm = max(args.warmup, 3)
    for _ in range(warm):
        step()
    barrier()
    n0 = L.q35_launch_count()
    step()
    launches = L.q35_launch_count() - n0
    # several ranks: the NCCL collectives are captured too; a step with a host round trip cannot be captured
    graph = hb.capture(step) if graph_ok and not args.no_graph else None
    run = graph.replay if graph is not None else step
    barrier()
    rounds = hb.timed_rounds(run, args.steps, barrier, agree=agree)
    ms = hb.median(rounds)
    # end to end: inputs from pinned host memory, result back
    host_in = [t.detach().cpu().pin_memory() for t in ins]
    host_out = [torch.empty_like(t, device="cpu").pin_memory() for t in outs]

    def step_e2e():
        for d, h in zip(ins, host_in):
            d.copy_(h, non_blocking=True)
        run()
        for d, h in zip(outs, host_out):
            h.copy_(d, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    for _ in range(3):
        step_e2e()
    e2e_ms = hb.median(hb.timed_rounds(step_e2e, args.steps, barrier, agree=agree))
    t = torch.tensor([ms, e2e_ms], device=dev or "cuda")
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, e2e_ms = t.tolist()
    status = q35.device_status()
    if rank == 0:
        per_step = ms / args.steps
        line = {
            "metric": metric, "value": unit_items * args.steps / (ms * 1e-3), "unit": "tok/s", "n_gpus": world,
            "steps": args.steps, "warmup": warm, "ms_per_step": per_step, "rounds": len(rounds),
            "higher_is_better": True, "scaling": scaling, "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic (seeded, on-device)", "config": dict(config, name=name),
            "launch": "cuda graph replay" if graph is not None else "eager",
            "timing": f"median of {len(rounds)} rounds of {args.steps} steps, CUDA events, max over ranks",
            "e2e": {"value": unit_items * args.steps / (e2e_ms * 1e-3), "unit": "tok/s",
                    "h2d_bytes_per_step": sum(x.numel() * x.element_size() for x in ins),
                    "d2h_bytes_per_step": sum(x.numel() * x.element_size() for x in outs)},
            "gpu_launches": int(launches * args.steps), "gpu_launches_per_step": int(launches),
            "roofline": roofline(per_step), "clocks": hb.clocks_summary(clocks), "device_status": status,
        }
        if extra:
            line.update(extra(per_step))
        print(json.dumps(line), flush=True)
    if dist is not None:
        if graph is not None:  # captured collectives keep the communicator busy at teardown: leave without it
            barrier()
            os._exit(0)
        dist.destroy_process_group()


def _hbm(nbytes, kernel):
    peak, _, src = hb.measured_peaks()
    peak *= int(os.environ.get("WORLD_SIZE", 1))  # whole-job bytes against the GPUs' aggregate bandwidth

    def f(ms):
        gbs = nbytes / (ms * 1e-3) / 1e9
        return {"bound": "hbm", "kernel": kernel, "achieved": gbs, "peak": peak, "unit": "GB/s", "frac": gbs / peak,
                "frac_of_nominal_8tbs": gbs / hb.NOMINAL_GBS, "peak_source": src, "traffic": None,
                "algorithmic_bytes": int(nbytes), "ms_per_launch": ms}
    return f


def run_c2(args, fp8):
    import ax_dsl_kernels_b200 as q35
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import datetime
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=180))
    B = 64
    ctxs = torch.randint(1024, 16385, (B,), generator=torch.Generator().manual_seed(1)).tolist()
    n_pages = [(c + PAGE - 1) // PAGE for c in ctxs]
    indptr = torch.tensor([0, *torch.tensor(n_pages).cumsum(0).tolist()], dtype=torch.int32)
    last = torch.tensor([c - (n - 1) * PAGE for c, n in zip(ctxs, n_pages)], dtype=torch.int32)
    kv_local = HKV
    if world > 1:  # this rank's KV heads and its share of every sequence's pages (see parallel.HeadSplitAttention)
        from ax_dsl_kernels_b200 import parallel
        plan = parallel.attention_split(HQ, HKV, world, rank)
        kv_local = plan["kv1"] - plan["kv0"]
        indptr, _, last = parallel.split_page_table(indptr, torch.arange(sum(n_pages), dtype=torch.int32), last, PAGE,
                                                    plan["share"], plan["shares"])
    total = int(indptr[-1])
    g = torch.Generator(device=dev).manual_seed(1 + rank)
    cache = torch.empty((total, 2, PAGE, kv_local, D), dtype=torch.bfloat16, device=dev)
    for i in range(0, total, 2048):
        cache[i:i + 2048] = torch.randn((min(2048, total - i), 2, PAGE, kv_local, D), generator=g, device=dev).to(torch.bfloat16)
    indices = torch.randperm(total, generator=g, device=dev).to(torch.int32)  # physical pages: a random permutation
    indptr, last = indptr.to(dev), last.to(dev)
    q = torch.randn((B, HQ, D), generator=torch.Generator(device=dev).manual_seed(11), device=dev).to(torch.bfloat16)
    kvs = None
    if fp8:
        amax = torch.stack([cache[i:i + 2048].float().abs().amax((0, 2, 4)) for i in range(0, total, 2048)]).amax(0)
        kvs = (amax / 448.0).contiguous()
        c8 = torch.empty(cache.shape, dtype=torch.float8_e4m3fn, device=dev)
        for i in range(0, total, 2048):
            c8[i:i + 2048] = (cache[i:i + 2048].float() / kvs.reshape(1, 2, 1, kv_local, 1)).to(torch.float8_e4m3fn)
        cache = c8
    out = torch.empty_like(q)
    scale = torch.tensor([1.0 / 16], device=dev)
    if world > 1:
        att = parallel.HeadSplitAttention(HQ, HKV)
        step = lambda: att.forward(q, cache, indptr, indices, last, out, sm_scale=scale, kv_scale=kvs)  # noqa: E731
    else:
        step = lambda: q35.paged_attention_decode(q, cache, indptr, indices, last, out, sm_scale=scale, kv_scale=kvs)  # noqa: E731
    nbytes = sum(ctxs) * 2 * HKV * D * (1 if fp8 else 2)
    _finish(args, "c2_fp8" if fp8 else "c2", "paged attention decode tok/s (batch 64, contexts 1024..16384)", B, step,
            [q], [out], _hbm(nbytes, f"attn_decode_kernel<256,{'e4m3' if fp8 else 'bf16'}> (+ plan and merge)"),
            {"workload": f"attn.paged_decode alone, batch {B}, contexts uniform in [1024, 16384] (seed 1, {sum(ctxs)} "
             f"tokens), {HQ} q / {HKV} kv heads, head_dim {D}, page {PAGE}, permuted pages, "
             f"{'FP8 E4M3 KV with per-head scales' if fp8 else 'bf16 KV'}", "l2": "KV larger than L2",
             "parallelism": "1 GPU" if world == 1 else f"query heads with their KV head over {min(world, HKV)} groups of "
             f"ranks; {max(1, world // HKV)} ranks share a KV head and split every sequence's pages, one all-gather of "
             "the unnormalised partials [64, 8, 258] fp32 per rank and a log-sum-exp merge"},
            dist=dist, dev=dev, scaling="strong")


def run_c3_decode(args):
    import ax_dsl_kernels_b200 as q35
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    wl = hb.Workload(dev, seed=2, attn=False)
    step = lambda: q35.gdn_recurrent_step(wl.gq, wl.gk, wl.gv, wl.gg, wl.gbeta, wl.state, wl.g_out, wl.state)  # noqa: E731
    _finish(args, "c3_decode", "GDN recurrent decode tok/s (batch 64)", hb.B, step, [wl.gq, wl.gk, wl.gv, wl.gg, wl.gbeta],
            [wl.g_out], _hbm(wl.gdn_bytes(), "gdn_step_kernel"),
            {"workload": f"gdn.step, batch {hb.B}, {hb.NV} value / {hb.NK} key heads, d 128, fp32 state read and written "
             "in place", "l2": "state (268 MB) larger than L2"}, dev=dev)


def run_c3_prefill(args):
    import ax_dsl_kernels_b200 as q35
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    T, NK, NV, GD = 16384, hb.NK, hb.NV, hb.GD
    g = torch.Generator(device=dev).manual_seed(2)
    rn = lambda *s: torch.randn(s, generator=g, device=dev)  # noqa: E731
    nrm = lambda t: t / torch.sqrt(t.square().sum(-1, keepdim=True) + 1e-6)  # noqa: E731
    q = (nrm(rn(1, T, NK, GD)) * GD ** -0.5).to(torch.bfloat16)
    k = nrm(rn(1, T, NK, GD)).to(torch.bfloat16)
    v = rn(1, T, NV, GD).to(torch.bfloat16)
    gg = -torch.nn.functional.softplus(rn(1, T, NV))
    beta = torch.sigmoid(rn(1, T, NV)).to(torch.bfloat16)
    s0 = torch.zeros((1, NV, GD, GD), device=dev)
    o, s1 = torch.empty_like(v), torch.empty_like(s0)
    step = lambda: q35.gdn_chunk_prefill(q, k, v, gg, beta, s0, o, s1)  # noqa: E731
    C = 64
    flop = (2 * C * C * GD + 2 * C * C * 2 * GD + 2 * 2 * C * GD * GD + 2 * C * C * GD + 2 * C * C * GD + 2 * C * GD * GD) * NV * (T // C)
    io = T * ((2 * NK * GD + NV * GD) * 2 + NV * GD * 2 + NV * 6) + 2 * NV * GD * GD * 4
    _, tf, src = hb.measured_peaks()

    def roof(ms):
        t = flop / (ms * 1e-3) / 1e12
        return {"bound": "tensor", "kernel": "gdn_chunk_prep_kernel + gdn_chunk_scan_kernel", "achieved": t, "peak": tf,
                "unit": "TFLOP/s", "frac": t / tf, "peak_source": src + " (bf16 GEMM)", "traffic": None,
                "algorithmic_flop": flop, "io_gbs": io / (ms * 1e-3) / 1e9, "algorithmic_io_bytes": io}
    _finish(args, "c3_prefill", "GDN chunked prefill tok/s (16384 tokens, chunk 64)", T, step, [q, k, v, gg, beta], [o],
            roof, {"workload": f"gdn.chunk_prefill, one sequence of {T} tokens, {NV} value / {NK} key heads, d 128, chunk 64, "
                   "bf16 inputs, fp32 state"}, dev=dev)


def run_c4_prefill_ep(args):
    """MoE prefill over several GPUs: experts sharded, the 8192 tokens split evenly; both exchange forms are timed and
    compared, the timed step runs the one `ExpertParallelMoE.forward_prefill` picks"""
    import datetime
    import torch.distributed as dist
    import ax_dsl_kernels_b200 as q35
    from ax_dsl_kernels_b200 import parallel
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=180))
    wl = hb.Workload(dev, seed=3, attn=False)  # the same weights on every rank; each keeps its experts
    ep = parallel.ExpertParallelMoE(wl.w, hb.TOPK, dist.group.WORLD)
    T = 8192 // world
    g = torch.Generator(device=dev).manual_seed(3 + rank)
    x1 = torch.randn((T, hb.H), generator=g, device=dev).to(torch.bfloat16)
    out = torch.empty_like(x1)
    flop = 8192 * hb.TOPK * 6 * hb.H * hb.FE + 8192 * 6 * hb.H * hb.FS + 8192 * 2 * hb.H * hb.NE
    _, tf, src = hb.measured_peaks()

    def roof(ms):
        t = flop / (ms * 1e-3) / 1e12
        return {"bound": "tensor", "kernel": "tc_gemm_kernel (routed gate-up, down on the received rows; shared expert)",
                "achieved": t, "peak": tf * world, "unit": "TFLOP/s", "frac": t / (tf * world),
                "peak_source": src + " (bf16 GEMM) x GPUs", "traffic": None, "algorithmic_flop": flop}

    # Both exchanges on the same tokens: phase times of each (every rank takes part: the steps hold collectives; rank
    # 0's medians are reported), their whole-step times, and how far their results are apart.  The timed step is the
    # library's own choice (forward_prefill, form "auto").
    forms, outs = {}, {}
    for form in ("all_to_all", "all_gather"):
        o = torch.empty_like(x1)
        per, whole = {}, []
        for it in range(12):
            marks = []
            ep.forward_prefill(x1, o, form=form, marks=marks)
            torch.cuda.synchronize()
            if it >= 4:
                for (_, a), (nm, b) in zip(marks[:-1], marks[1:]):
                    per.setdefault(nm, []).append(a.elapsed_time(b))
                whole.append(marks[0][1].elapsed_time(marks[-1][1]))
        t = torch.tensor([hb.median(whole)], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        forms[form] = {"ms_max_over_ranks": round(float(t.item()), 4),
                       "phases_us_rank0": {nm: round(hb.median(v) * 1e3, 1) for nm, v in per.items()}}
        outs[form] = o
    diff = (outs["all_to_all"].float() - outs["all_gather"].float()).abs().max() / outs["all_gather"].float().square().mean().sqrt()
    d = torch.tensor([float(diff)], device=dev)
    dist.all_reduce(d, op=dist.ReduceOp.MAX)
    chosen = "all_gather" if world * T * hb.H * 6 <= (4 << 30) else "all_to_all"
    step = lambda: ep.forward_prefill(x1, out)  # noqa: E731
    extra = lambda _ms: {"ep_forms": forms, "ep_forms_max_diff_over_rms": float(d.item()), "ep_form_timed": chosen}  # noqa: E731
    _finish(args, "c4_prefill", "MoE block prefill tok/s (8192 tokens, 256 experts top-8); % of FP4/FP8 TC peak", 8192, step,
            [x1], [out], roof,
            {"workload": f"MoE block, 8192 tokens ({T} per GPU), {hb.NE} experts top-{hb.TOPK} MXFP4 + shared expert, "
             f"hidden {hb.H}", "parallelism": f"experts sharded x{world}, tokens split x{world}; exchange form '{chosen}' "
             "(all_gather: every rank's rows to every rank and fp32 partial sums back, through peer memory or NCCL; "
             "all_to_all: every token's row once to each rank that owns one of its experts, one weighted sum back per "
             "row, row counts through the host); both are timed in ep_forms"},
            dist=dist, dev=dev, scaling="strong", graph_ok=False, extra=extra)


def run_c4(args, prefill):
    import ax_dsl_kernels_b200 as q35
    if prefill and int(os.environ.get("WORLD_SIZE", 1)) > 1:
        return run_c4_prefill_ep(args)
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    wl = hb.Workload(dev, seed=3, attn=False)
    q35.prepare_moe_weights(wl.w)
    T = 8192 if prefill else hb.B
    g = torch.Generator(device=dev).manual_seed(3)
    x1 = torch.randn((T, hb.H), generator=g, device=dev).to(torch.bfloat16)
    out = torch.empty_like(x1)
    step = lambda: q35.moe_block(x1, wl.w, hb.TOPK, out)  # noqa: E731
    ids = q35.moe_block(x1, wl.w, hb.TOPK, out)[1]
    distinct = int(torch.unique(ids).numel())
    wbytes = distinct * hb.EXPERT_BYTES + hb.EXPERT_BYTES + hb.NE * hb.H * 2 + 2 * T * hb.H * 2
    if not prefill:
        _finish(args, "c4_decode", "MoE block decode tok/s (batch 64, 256 experts top-8)", T, step, [x1], [out],
                _hbm(wbytes, "moe_front + moe_decode_quant + moe_decode_kernel + moe_block_combine"),
                {"workload": f"MoE block, {T} tokens, {hb.NE} experts top-{hb.TOPK} MXFP4 + shared expert, hidden {hb.H}, "
                 f"{distinct} distinct experts hit", "l2": "expert weights (0.43 GB) larger than L2"}, dev=dev)
        return
    # the block-scaled tensor-core peak, measured now on this GPU
    iters = torch.tensor([20000], dtype=torch.int32, device=dev)
    done = torch.zeros(1, dtype=torch.int32, device=dev)
    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    q35.run("debug.tc_peak", iters=iters, done=done)
    torch.cuda.synchronize()
    best = None
    for _ in range(3):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        q35.run("debug.tc_peak", iters=iters, done=done)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        best = ms if best is None else min(best, ms)
    tc_peak = sms * 20000 * 4 * 2 * 128 * 256 * 32 / (best * 1e-3) / 1e12
    flop = T * hb.TOPK * 6 * hb.H * hb.FE + T * 6 * hb.H * hb.FS + T * 2 * hb.H * hb.NE
    _, tf, src = hb.measured_peaks()

    def roof(ms):
        t = flop / (ms * 1e-3) / 1e12
        return {"bound": "tensor", "kernel": "tc_gemm_kernel<64, *> (routed gate-up, down; shared expert) + router",
                "achieved": t, "peak": tc_peak, "unit": "TFLOP/s", "frac": t / tc_peak,
                "peak_source": "tcgen05 kind::mxf8f6f4.block_scale 128x256x32 issued back to back from shared memory on "
                "every SM, measured in this run (debug.tc_peak)", "frac_of_measured_bf16_gemm": t / tf,
                "bf16_gemm_peak": tf, "traffic": None, "algorithmic_flop": flop,
                "note": "algorithmic FLOP of bf16 x MXFP4; the kernel issues twice the MMA work (activations as two E4M3 terms)"}
    _finish(args, "c4_prefill", "MoE block prefill tok/s (8192 tokens, 256 experts top-8); % of FP4/FP8 TC peak", T, step,
            [x1], [out], roof,
            {"workload": f"MoE block, {T} tokens, {hb.NE} experts top-{hb.TOPK} MXFP4 + shared expert, hidden {hb.H}"},
            dev=dev)


def _fp8_rows(g, dev, n, k):
    w = torch.randn((n, k), generator=g, device=dev) * 0.02
    s = (w.abs().amax(-1) / 448.0).clamp_min(1e-12)
    return (w / s[:, None]).to(torch.float8_e4m3fn).contiguous(), s.float().contiguous()


def c5_weights(dev, seed=4, H=5120, F=17408, heads=24, kv_heads=4, hd=256, NK=16, NV=48, gd=128, layers=16):
    """16 layers g g g a x 4, FP8 E4M3 weights with per-row fp32 scales drawn from N(0, 0.02), norms 1 + N(0, 0.02)"""
    g = torch.Generator(device=dev).manual_seed(seed)
    rn = lambda *s: torch.randn(s, generator=g, device=dev)  # noqa: E731
    kinds = ("ggga" * ((layers + 3) // 4))[:layers]
    out = []
    KD, VD = NK * gd, NV * gd
    for kind in kinds:
        w = {}
        if kind == "g":
            for n, shp in (("q", (KD, H)), ("k", (KD, H)), ("v", (VD, H)), ("z", (VD, H)), ("a", (NV, H)), ("b", (NV, H)),
                           ("o", (H, VD))):
                w["w_" + n], w["s_" + n] = _fp8_rows(g, dev, *shp)
            for n, width in (("q", KD), ("k", KD), ("v", VD)):
                w[f"w_{n}_conv"] = (rn(width, 4) * 0.1).to(torch.bfloat16)
            w["input_norm_w"] = (1 + 0.02 * rn(H)).to(torch.bfloat16)
            w["a_log"] = (torch.rand(NV, generator=g, device=dev) * 15 + 1).log()
            w["dt_bias"] = (rn(NV) * 0.02).to(torch.bfloat16)
            w["o_norm_w"] = (1 + 0.02 * rn(gd)).to(torch.bfloat16)
        else:
            for n, shp in (("q", (heads * hd * 2, H)), ("k", (kv_heads * hd, H)), ("v", (kv_heads * hd, H)),
                           ("o", (H, heads * hd))):
                w["w_" + n], w["s_" + n] = _fp8_rows(g, dev, *shp)
            w["ln1"] = 1 + 0.02 * rn(H)
            w["q_norm"] = 1 + 0.02 * rn(hd)
            w["k_norm"] = 1 + 0.02 * rn(hd)
        for n, shp in (("gate", (F, H)), ("up", (F, H)), ("down", (H, F))):
            w["w_" + n], w["s_" + n] = _fp8_rows(g, dev, *shp)
        w["ln2"] = 1 + 0.02 * rn(H)
        out.append(w)
    return out, kinds


def run_c5(args, fp8):
    import ax_dsl_kernels_b200 as q35
    from ax_dsl_kernels_b200 import layers as L, parallel
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import datetime
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=180))
    B, CTX, H, F, heads, kvh, hd, NK, NV, n_layers = 8, 131072, 5120, 17408, 24, 4, 256, 16, 48, args.layers
    ws, kinds = c5_weights(dev, layers=n_layers)  # the same full weights on every rank, then this rank's shard
    kw = dict(batch=B, heads=heads, kv_heads=kvh, head_dim=hd, rot=64, theta=1e7, max_tokens=CTX + PAGE, page_size=PAGE,
              kv_dtype=torch.float8_e4m3fn if fp8 else torch.bfloat16)
    tp_check = None
    if world > 1:
        # the first four layers (g g g a), short context, one step: this rank's tensor-parallel output against the whole
        # layers on this GPU alone (every rank holds the full weights at this point)
        small = dict(kw, max_tokens=256 + PAGE)
        xs = (torch.randn((B, H), generator=torch.Generator(device=dev).manual_seed(5), device=dev) * 0.5).to(torch.bfloat16)
        one = L.DecodeGroup(ws[:4], kinds[:4], **small)
        tp4 = parallel.tensor_parallel_decode_group(ws[:4], kinds[:4], reduce=args.ep_exchange, **small)
        outs = []
        for grp4 in (one, tp4):
            grp4.set_context([100] * B)
            outs.append(grp4.step(xs, advance=False).float())
        worst = ((outs[1] - outs[0]).abs().max() / outs[0].square().mean().sqrt()).reshape(1)
        dist.all_reduce(worst, op=dist.ReduceOp.MAX)
        tp_check = {"layers": 4, "max_err_over_rms_vs_one_gpu": float(worst.item()),
                    "all_reduce": "peer memory (ar.oneshot)" if getattr(tp4.reduce, "_px", None) else "nccl"}
        del one, tp4, outs
        grp = parallel.tensor_parallel_decode_group(ws, kinds, reduce=args.ep_exchange, **kw)
        del ws
        torch.cuda.empty_cache()
    else:
        grp = L.DecodeGroup(ws, kinds, **kw)
    g = torch.Generator(device=dev).manual_seed(40 + rank)
    for i, c in grp.cache.items():  # history: N(0, 1) keys and values (FP8: the constant-scale form stores 8 x)
        for p0 in range(0, c.shape[0], 1024):
            blk = torch.randn((min(1024, c.shape[0] - p0), *c.shape[1:]), generator=g, device=dev)
            c[p0:p0 + 1024] = (blk * 8).to(c.dtype) if fp8 else blk.to(c.dtype)
    for i, s in grp.state.items():
        s.copy_(torch.randn(s.shape, generator=g, device=dev) * 0.03)
    grp.set_context([CTX] * B)
    x = (torch.randn((B, H), generator=torch.Generator(device=dev).manual_seed(4), device=dev) * 0.5).to(torch.bfloat16)
    y = torch.empty_like(x)
    step = lambda: y.copy_(grp.step(x, advance=False))  # noqa: E731
    n_g, n_a = kinds.count("g"), kinds.count("a")
    wb = n_g * ((2 * NK * 128 + 2 * NV * 128 + 2 * NV) * H + H * NV * 128) + n_a * ((heads * hd * 2 + 2 * kvh * hd) * H + H * heads * hd) \
        + n_layers * 3 * F * H
    kvb = n_a * B * CTX * 2 * kvh * hd * (1 if fp8 else 2)
    stb = n_g * 2 * B * NV * 128 * 128 * 4
    nbytes = wb + kvb + stb
    _finish(args, "c5_fp8" if fp8 else "c5", "27B-class dense decode group tok/s (16 layers, batch 8 x 131072 context)",
            B, step, [x], [y], _hbm(nbytes, "whole decode group (weights + KV + GDN state)"),
            {"workload": f"{n_layers} layers ({n_g} GDN + {n_a} gated attention, each + dense SwiGLU FFN {F}), hidden {H}, "
             f"{heads} q / {kvh} kv heads of {hd}, GDN {NV} value / {NK} key heads, FP8 E4M3 per-row weights "
             f"({wb / 1e9:.2f} GB), batch {B}, context {CTX}, page {PAGE}, {'FP8 E4M3' if fp8 else 'bf16'} KV "
             f"({kvb / 1e9:.2f} GB read per step), fp32 GDN state ({stb / 1e9:.2f} GB read + written)",
             "parallelism": "1 GPU" if world == 1 else f"tensor parallel x{world}: heads, GDN value heads and FFN columns "
             "split, one all-reduce of the fp32 partial [8, 5120] per sublayer (this library's one-kernel all-reduce over "
             "peer memory, or NCCL with --ep-exchange nccl)"}, dist=dist, dev=dev, scaling="strong",
            extra=(lambda _ms: {"tp_check": tp_check}) if tp_check else None)


def run(args):
    name = args.config
    if name in ("c2", "c2_fp8"):
        run_c2(args, name.endswith("fp8"))
    elif name == "c3_decode":
        run_c3_decode(args)
    elif name == "c3_prefill":
        run_c3_prefill(args)
    elif name in ("c4_decode", "c4_prefill"):
        run_c4(args, name.endswith("prefill"))
    elif name in ("c5", "c5_fp8"):
        run_c5(args, name.endswith("fp8"))
    else:
        raise SystemExit(f"unknown --config {name}")
