"""Benchmark of the Qwen3.5 decoder hot path on B200: one decode step of the layer triple
GDN recurrent step + paged attention decode + MoE block at batch 64 x 16k context.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Prints ONE JSON line (rank 0).  `value` = tokens/s with every input resident in HBM; `e2e` = the same step driven
through the public Python API with the per-step activations starting in pinned host memory and the results copied
back; `roofline` = the dominant kernel (paged attention decode) against the measured HBM copy bandwidth;
`cpu_baseline` = the CPU oracle (a port of the reference's torch goldens) timed on a bounded sample.
Synthetic seeded inputs with the shapes and value distributions of the quoted configuration.
"""
import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

METRIC = "decode tok/s (MoE+attn+GDN layer)"
B, CTX, PAGE = 64, 16384, 64
HQ, HKV, D = 16, 2, 256
NK, NV, GD = 16, 32, 128
H, NE, FE, FS, TOPK = 2048, 256, 512, 512, 8


def measured_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        return float(json.load(open(p))["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def workload_name():
    return (f"decode layer triple, batch {B} x context {CTX}: gdn.step ({NV} value / {NK} key heads, d 128, fp32 state) "
            f"+ attn.paged_decode ({HQ} q / {HKV} kv heads, head_dim {D}, page {PAGE}, bf16 KV) "
            f"+ MoE block ({NE} experts top-{TOPK} MXFP4, shared expert, hidden {H})")


# ----------------------------------------------------------------------------------------------------------------
class Workload:
    """all tensors of one rank, generated on the device from a seed"""

    def __init__(self, dev, seed, n_experts_local=NE, attn=True):
        g = torch.Generator(device=dev).manual_seed(seed)
        bf = torch.bfloat16
        rn = lambda *s: torch.randn(s, generator=g, device=dev)  # noqa: E731
        # paged attention: every sequence at CTX, page table a random permutation of the physical pages
        n_pages = CTX // PAGE if attn else 1  # attn=False: profile cases of the other kernels keep the device small
        total = B * n_pages
        self.cache = torch.empty((total, 2, PAGE, HKV, D), dtype=bf, device=dev)
        for i in range(0, total, 2048):  # chunked: keeps the fp32 temporary small
            self.cache[i:i + 2048] = rn(min(2048, total - i), 2, PAGE, HKV, D).to(bf)
        self.indices = torch.randperm(total, generator=g, device=dev).to(torch.int32)
        self.indptr = (torch.arange(B + 1, device=dev) * n_pages).to(torch.int32)
        self.last = torch.full((B,), PAGE, dtype=torch.int32, device=dev)
        self.q = rn(B, HQ, D).to(bf)
        self.attn_out = torch.empty_like(self.q)
        self.sm_scale = torch.tensor([1.0 / 16], device=dev)
        # GDN recurrent step
        nrm = lambda t: (t / torch.sqrt(t.square().sum(-1, keepdim=True) + 1e-6))  # noqa: E731
        self.gq = (nrm(rn(B, NK, GD)) * GD ** -0.5).to(bf)
        self.gk = nrm(rn(B, NK, GD)).to(bf)
        self.gv = rn(B, NV, GD).to(bf)
        self.gg = -torch.nn.functional.softplus(rn(B, NV))
        self.gbeta = torch.sigmoid(rn(B, NV)).to(bf)
        self.state = rn(B, NV, GD, GD) * 0.03
        self.g_out = torch.empty_like(self.gv)
        # MoE block
        rb = lambda lo, hi, *s: torch.randint(lo, hi, s, generator=g, device=dev, dtype=torch.int32).to(torch.uint8)  # noqa: E731
        self.x1 = rn(B, H).to(bf)
        self.w = dict(
            ln2=torch.ones(H, device=dev), w_router=(rn(NE, H) / H ** 0.5).to(bf), w_shg=(rn(H) / H ** 0.5).to(bf),
            e_gw=rb(0, 256, n_experts_local, 2 * FE, H // 2), e_gs=rb(119, 128, n_experts_local, 2 * FE, H // 32),
            e_dw=rb(0, 256, n_experts_local, H, FE // 2), e_ds=rb(119, 128, n_experts_local, H, FE // 32),
            w_gate=rb(0, 256, FS, H // 2), s_gate=rb(119, 128, FS, H // 32), w_up=rb(0, 256, FS, H // 2),
            s_up=rb(119, 128, FS, H // 32), w_down=rb(0, 256, H, FS // 2), s_down=rb(119, 128, H, FS // 32))
        self.moe_out = torch.empty_like(self.x1)

    def attn_bytes(self):
        return B * CTX * 2 * HKV * D * 2


def run_ours(args):
    import ax_dsl_kernels_b200 as q35
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    wl = Workload(dev, seed=1000 + rank)
    moe_step = None
    if world > 1:
        from ax_dsl_kernels_b200 import parallel
        ep = parallel.ExpertParallelMoE(wl.w, TOPK, dist.group.WORLD)
        moe_step = lambda x: ep.forward(x, wl.moe_out)  # noqa: E731
    else:
        moe_step = lambda x: q35.moe_block(x, wl.w, TOPK, wl.moe_out)  # noqa: E731

    def step():
        q35.gdn_recurrent_step(wl.gq, wl.gk, wl.gv, wl.gg, wl.gbeta, wl.state, wl.g_out, wl.state)
        q35.paged_attention_decode(wl.q, wl.cache, wl.indptr, wl.indices, wl.last, wl.attn_out, sm_scale=wl.sm_scale)
        moe_step(wl.x1)

    def attn_only():
        q35.paged_attention_decode(wl.q, wl.cache, wl.indptr, wl.indices, wl.last, wl.attn_out, sm_scale=wl.sm_scale)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    clocks = ClockSampler(local) if rank == 0 else None
    if clocks:
        clocks.start()  # sampled from the warm-up to the end of the end-to-end loop (nvidia-smi, every 100 ms)
    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    # One GPU: the step is captured once into a CUDA graph through the public API and replayed (18 kernel launches
    # that together take ~0.55 ms would otherwise be paced by the Python launch path); both the device-resident loop
    # and the end-to-end loop replay it.  The NCCL variant runs eagerly.
    graph = None
    if world == 1 and not args.no_graph:
        graph = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            step()
            with torch.cuda.graph(graph, stream=side):
                step()
        torch.cuda.current_stream().wait_stream(side)
        for _ in range(3):
            graph.replay()
    run_step = graph.replay if graph is not None else step
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t0.record()
    for i in range(args.steps):
        run_step()
    t1.record()
    barrier()
    ms = t0.elapsed_time(t1)
    # the dominant kernel on its own, same process, right after the timed region (events cannot be placed inside a
    # replayed graph): K role calls = plan + decode + merge launches each
    a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    attn_only()
    a0.record()
    for i in range(args.steps):
        attn_only()
    a1.record()
    barrier()
    attn_ms = a0.elapsed_time(a1) / args.steps

    # end to end: per-step activations start in pinned host memory, results come back to the host
    host_in = {n: getattr(wl, n).cpu().pin_memory() for n in ("x1", "q", "gq", "gk", "gv", "gg", "gbeta")}
    host_out = {n: torch.empty_like(getattr(wl, n), device="cpu").pin_memory() for n in ("moe_out", "attn_out", "g_out")}
    h2d = sum(t.numel() * t.element_size() for t in host_in.values())
    d2h = sum(t.numel() * t.element_size() for t in host_out.values())

    def step_e2e():
        for n, t in host_in.items():
            getattr(wl, n).copy_(t, non_blocking=True)
        run_step()  # the captured step reads and writes the same device buffers the copies fill and drain
        for n, t in host_out.items():
            t.copy_(getattr(wl, n), non_blocking=True)
        torch.cuda.current_stream().synchronize()  # the caller reads the results

    for _ in range(3):
        step_e2e()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step_e2e()
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1)
    if clocks:
        clocks.stop()

    times = torch.tensor([ms, e2e_ms], device=dev)
    if dist is not None:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms, e2e_ms = times.tolist()
    status = q35.device_status()
    if rank == 0:
        peak, peak_src = measured_peak()
        achieved = wl.attn_bytes() / (attn_ms * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": world * B * args.steps / (ms * 1e-3), "unit": "tok/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic (seeded, on-device)",
            "config": {"workload": workload_name(), "batch_per_gpu": B, "context": CTX,
                       "arithmetic": "bf16 activations and KV, MXFP4 expert weights into the block-scaled MMA with the "
                       "activations as two E4M3 terms, fp32 accumulation and GDN state", "launch": "cuda graph replay" if graph is not None else "eager",
                       "parallelism": "1 GPU" if world == 1 else f"sequences data-parallel x{world}, experts sharded "
                       f"x{world} (NCCL all-gather of tokens + reduce-scatter of expert sums)", "l2": "inputs larger than L2 (2.1 GB KV + 0.43 GB experts + "
                       "0.27 GB state per step)"},
            "e2e": {"value": world * B * args.steps / (e2e_ms * 1e-3), "unit": "tok/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h},
            # kernels of this library per step (torch and NCCL kernels not counted): GDN 1, attention 3, MoE 14 with
            # the one-CTA routing plan (up to 4096 token-expert pairs per rank), 16 with the three-kernel plan
            "gpu_launches": args.steps * (18 if world * B * TOPK <= 4096 else 20),
            "roofline": {"bound": "hbm", "kernel": "attn_decode_kernel<256,bf16> (+ plan and merge launches)",
                         "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_source": peak_src, "traffic": attn_traffic(wl), "algorithmic_bytes": wl.attn_bytes(),
                         "ms_per_launch": attn_ms},
            "clocks": clocks.summary() if clocks else None,
            "device_status": status,
        }
        if world == 1 and not args.no_cpu:
            line["cpu_baseline"] = cpu_sample(1)
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


def attn_traffic(wl):
    """DRAM bytes of one attention decode launch, scaled from the ncu capture of the capture-sized case
    (profiles/attn_decode_bf16_b16_ctx8192.md: 268.70 MB read for 268.44 MB of K/V, i.e. every byte once; writes = the
    split-KV partials, one [m, l, O] per (segment or CTA, warp, query head of the group)).  Reads grow in proportion to
    the K/V bytes, the partials with the number of segments."""
    reads = wl.attn_bytes() * (268.70 / 268.44)
    partials = (B * HKV + 148) * 4 * (HQ // HKV) * (D + 2) * 4
    return int(reads + partials)


# ----------------------------------------------------------------------------------------------------------------
class ClockSampler:
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.f = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.p = None

    def start(self):
        try:
            self.p = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                       "--format=csv,noheader,nounits", "-lms", "100"], stdout=self.f,
                                      stderr=subprocess.DEVNULL)
        except OSError:
            self.p = None

    def stop(self):
        if self.p:
            self.p.terminate()
            self.p.wait()

    def summary(self):
        self.f.flush()
        self.f.seek(0)
        sm, mx, reasons = [], 0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.f.read().splitlines():
            c = [x.strip() for x in ln.split(",")]
            if len(c) < 7:
                continue
            try:
                sm.append(float(c[0]))
                mx = max(mx, float(c[1]))
            except ValueError:
                continue
            for n, v in zip(names, c[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx or None, "reasons": sorted(reasons),
                "samples": len(sm)}


# ----------------------------------------------------------------------------------------------------------------
def cpu_sample(reps, n_attn=2, n_moe=2, n_gdn=4):
    """the CPU oracle on a bounded sample of the same workload: n_attn sequences at the full context, n_moe tokens
    through the MoE block (dequantisation of the packed experts inside the timed region, as the accelerator also
    consumes packed weights), n_gdn sequences of the GDN step.  tokens/s = 1 / (per-token seconds of the three)."""
    from oracle import attention as oattn, codecs, gdn as ogdn, moe as omoe
    from _cases import dequant_shared, gdn_step_case, moe_case, paged_case
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    q, cache, indptr, indices, last, _ = paged_case([CTX] * n_attn, seed=1)
    x1, w = moe_case(n_moe, seed=3)
    gq, gk, gv, gg, gb, st = gdn_step_case(B=n_gdn, seed=2)
    best = None
    for _ in range(max(1, reps)):
        t0 = time.perf_counter()
        oattn.paged_decode(q, cache, indptr, indices, last, sm_scale=1.0 / 16)
        t1 = time.perf_counter()
        sg, su, sd = dequant_shared(w)
        omoe.moe_block(x1, w["ln2"], sg, su, sd, w["w_router"], w["w_shg"], w["e_gw"], w["e_gs"], w["e_dw"], w["e_ds"],
                       TOPK)
        t2 = time.perf_counter()
        ogdn.recurrent(gq, gk, gv, gg, gb, st)
        t3 = time.perf_counter()
        per_tok = (t1 - t0) / n_attn + (t2 - t1) / n_moe + (t3 - t2) / n_gdn
        best = per_tok if best is None else min(best, per_tok)
    return {"value": 1.0 / best, "unit": "tok/s", "cores": cores, "kind": "port",
            "sample": f"{n_attn} sequences of paged attention at context {CTX}, {n_moe} tokens of the MoE block (packed "
                      f"experts dequantised inside the timed region), {n_gdn} sequences of the GDN step; per-token "
                      "seconds of the three added", "seconds_per_token": best}


def run_reference(args):
    """the reference's own CPU implementation of the path = its torch goldens, restated in oracle/ (its kernels need
    the NPU DSL and cannot run); timed on the host cores, rank 0 only"""
    if int(os.environ.get("RANK", 0)) != 0:
        return
    for _ in range(min(args.warmup, 1)):
        cpu_sample(1)
    t0 = time.perf_counter()
    res = [cpu_sample(1) for _ in range(min(args.steps, 5))]
    wall = time.perf_counter() - t0
    best = max(r["value"] for r in res)
    cb = dict(res[0], value=best)
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": best, "unit": "tok/s", "n_gpus": int(os.environ.get("WORLD_SIZE", 1)),
        "steps": len(res), "warmup": min(args.warmup, 1), "ms_per_step": 1e3 * wall / len(res), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "fp32/bf16 torch on CPU", "data": "synthetic (seeded)",
        "config": {"workload": workload_name(), "note": "bounded sample per step, see cpu_baseline.sample"},
        "cpu_baseline": cb, "e2e": {"value": best, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }), flush=True)


def run_profile_case(name, reps):
    """one kernel on a case sized for a profiler capture (inputs larger than L2 where the kernel is memory-bound, well
    under a few GB); prints the device time per repetition, which is not a benchmark value of the decode workload"""
    import ax_dsl_kernels_b200 as q35
    global B, CTX
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    if name == "attn":
        B, CTX = 16, 8192  # 268 MB of bf16 KV
    g = torch.Generator(device=dev).manual_seed(1)
    rn = lambda *s: torch.randn(s, generator=g, device=dev)  # noqa: E731
    bf = torch.bfloat16
    if name == "gdn_prefill":  # chunked GDN prefill of one 16k-token sequence, 32 value / 16 key heads
        T = 16384
        nrm = lambda t: t / torch.sqrt(t.square().sum(-1, keepdim=True) + 1e-6)  # noqa: E731
        q = (nrm(rn(1, T, NK, GD)) * GD ** -0.5).to(bf)
        k = nrm(rn(1, T, NK, GD)).to(bf)
        v = rn(1, T, NV, GD).to(bf)
        gg = -torch.nn.functional.softplus(rn(1, T, NV))
        beta = torch.sigmoid(rn(1, T, NV)).to(bf)
        s0 = torch.zeros((1, NV, GD, GD), device=dev)
        o, s1 = torch.empty_like(v), torch.empty_like(s0)
        fn = lambda: q35.gdn_chunk_prefill(q, k, v, gg, beta, s0, o, s1)  # noqa: E731
        units = T
    elif name == "attn_prefill":  # causal prefill of one 8k-token sequence into an empty paged cache
        T = 8192
        npg = T // PAGE
        cache = rn(npg, 2, PAGE, HKV, D).to(bf)
        indptr = torch.tensor([0, npg], device=dev, dtype=torch.int32)
        indices = torch.randperm(npg, generator=g, device=dev).to(torch.int32)
        last = torch.tensor([PAGE], device=dev, dtype=torch.int32)
        qo = torch.tensor([0, T], device=dev, dtype=torch.int32)
        q = rn(T, HQ, D).to(bf)
        out = torch.empty_like(q)
        fn = lambda: q35.paged_attention_prefill(q, cache, qo, indptr, indices, last, out)  # noqa: E731
        units = T
    elif name == "moe_prefill":  # MoE block on 8192 tokens (prefill-sized groups on the tensor-core GEMM)
        wl = Workload(dev, seed=1, attn=False)
        T = 8192
        x1 = (rn(T, H) * 0.5).to(bf)
        out = torch.empty_like(x1)
        fn = lambda: q35.moe_block(x1, wl.w, TOPK, out)  # noqa: E731
        units = T
    elif name == "lm_head":  # MXFP4 output projection 248320 x 2048 (254 MB codes + 16 MB scales) on one token row
        from ax_dsl_kernels_b200.moe import lm_head
        N = 248320
        pk = torch.randint(0, 256, (N, H // 2), generator=g, device=dev, dtype=torch.uint8)
        sc = torch.randint(119, 128, (N, H // 32), generator=g, device=dev, dtype=torch.uint8)
        x = rn(1, H).to(bf)
        logits = torch.empty((1, N), dtype=torch.float32, device=dev)
        token = torch.empty((1,), dtype=torch.int32, device=dev)
        fn = lambda: lm_head(x, pk, sc, logits, token)  # noqa: E731
        units = 1
    else:
        wl = Workload(dev, seed=1, attn=(name == "attn"))
        units = B
        if name == "attn":
            fn = lambda: q35.paged_attention_decode(wl.q, wl.cache, wl.indptr, wl.indices, wl.last, wl.attn_out,  # noqa: E731
                                                    sm_scale=wl.sm_scale)
        elif name == "gdn":
            fn = lambda: q35.gdn_recurrent_step(wl.gq, wl.gk, wl.gv, wl.gg, wl.gbeta, wl.state, wl.g_out, wl.state)  # noqa: E731
        else:
            fn = lambda: q35.moe_block(wl.x1, wl.w, TOPK, wl.moe_out)  # noqa: E731
    fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / reps
    print(f"profile case {name}: {reps} repetitions, {ms * 1e3:.1f} us each ({units / ms * 1e3:.0f} tokens/s), "
          f"device status {q35.device_status()}")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline sample")
    ap.add_argument("--no-graph", action="store_true", help="launch the timed steps eagerly instead of replaying a CUDA graph")
    ap.add_argument("--profile-case", choices=["attn", "gdn", "moe", "gdn_prefill", "attn_prefill", "moe_prefill", "lm_head"], help="run one kernel on a capture-sized case")
    args = ap.parse_args()
    if args.profile_case:
        run_profile_case(args.profile_case, max(1, min(args.steps, 5)))
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
