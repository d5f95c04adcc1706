"""Benchmark of the Qwen3.5 decoder hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config NAME]

Default (`--config headline`): one decode step of the layer triple GDN recurrent step + paged attention decode + MoE
block at batch 64 x 16k context.  Prints ONE JSON line (rank 0).  `value` = tokens/s with every input resident in HBM;
`e2e` = the same step with the per-step activations starting in pinned host memory (one packed copy each way inside
the timed region); `roofline` = the dominant kernel (paged attention decode) against the measured HBM copy bandwidth,
`roofline_all` = every part and the whole step against the measured and the nominal (8 TB/s) bandwidth;
`full_layer` = the same step with the sublayer glue around the three kernels (projections, conv, norms, RoPE, KV
write, output projections); `cpu_baseline` = the CPU oracle (a port of the reference's torch goldens) on a bounded
sample.  A timed "round" is exactly K steps; rounds are repeated until half a second of device time has been measured
and the median round is reported.

Other configurations (one JSON line each, same schema): c2 / c2_fp8 (paged decode alone, mixed contexts), c3_decode,
c3_prefill, c4_decode, c4_prefill (with a block-scaled tensor-core peak measured in the same run), c5 (27B-class dense
decode group, batch 8 x 131072 context; tensor parallel over --gpus).  Synthetic seeded inputs with the shapes and
value distributions of the quoted configurations.
"""
import argparse
import json
import math
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
NOMINAL_GBS = 8000.0  # the HBM figure the target is quoted against
EXPERT_BYTES = 3 * H * FE // 2 + 3 * H * FE // 32  # one expert: gate, up, down codes + E8M0 scales = 1,671,168


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        j = json.load(open(p))
        return float(j["hbm_gbs"]), float(j.get("bf16_tflops", 1590.0)), "measured"
    return 6650.0, 1590.0, "fallback"


def workload_name():
    return (f"decode layer triple, batch {B} x context {CTX}: gdn.step ({NV} value / {NK} key heads, d 128, fp32 state) "
            f"+ attn.paged_decode ({HQ} q / {HKV} kv heads, head_dim {D}, page {PAGE}, bf16 KV) "
            f"+ MoE block ({NE} experts top-{TOPK} MXFP4, shared expert, hidden {H})")


def headline_config(world):
    """identical for both arms (ours and the CPU reference) at the same N"""
    return {"workload": workload_name(), "batch_per_gpu": B, "context": CTX,
            "arithmetic": "bf16 activations and KV, MXFP4 expert weights, fp32 accumulation and GDN state",
            "parallelism": "1 GPU" if world == 1 else f"sequences data-parallel x{world}, experts sharded x{world}",
            "l2": "inputs larger than L2 (2.1 GB KV + 0.43 GB experts + 0.27 GB state per step)"}


# ----------------------------------------------------------------------------------------------------------------
class Packed:
    """tensors carved out of ONE byte buffer (256-byte aligned pieces), so that a set of small per-step tensors moves
    between host and device as a single copy"""

    def __init__(self, specs, device, pin=False):
        self.offsets, off = {}, 0
        for name, shape, dtype in specs:
            n = math.prod(shape) * torch.empty((), dtype=dtype).element_size()
            self.offsets[name] = (off, n, shape, dtype)
            off = (off + n + 255) // 256 * 256
        self.buf = torch.empty(off, dtype=torch.uint8, device=device)
        if pin:
            self.buf = self.buf.pin_memory()
        self.nbytes = off

    def view(self, name):
        off, n, shape, dtype = self.offsets[name]
        return self.buf[off:off + n].view(dtype).reshape(shape)


class Workload:
    """all tensors of one rank, generated on the device from a seed; the per-step activations and results live in two
    packed buffers"""

    def __init__(self, dev, seed, n_experts_local=NE, attn=True, weight_seed=None):
        """weight_seed: the MoE weights from a seed of their own (several ranks: the same model on every rank, different
        tokens and caches per rank)"""
        g = torch.Generator(device=dev).manual_seed(seed)
        bf = torch.bfloat16
        rn = lambda *s: torch.randn(s, generator=g, device=dev)  # noqa: E731
        self.inputs = Packed([("x1", (B, H), bf), ("q", (B, HQ, D), bf), ("gq", (B, NK, GD), bf), ("gk", (B, NK, GD), bf),
                              ("gv", (B, NV, GD), bf), ("gg", (B, NV), torch.float32), ("gbeta", (B, NV), bf)], dev)
        self.outputs = Packed([("moe_out", (B, H), bf), ("attn_out", (B, HQ, D), bf), ("g_out", (B, NV, GD), bf)], dev)
        for n in self.inputs.offsets:
            setattr(self, n, self.inputs.view(n))
        for n in self.outputs.offsets:
            setattr(self, n, self.outputs.view(n))
        # paged attention: every sequence at CTX, page table a random permutation of the physical pages
        n_pages = CTX // PAGE if attn else 1  # attn=False: profile cases of the other kernels keep the device small
        total = B * n_pages
        self.cache = torch.empty((total, 2, PAGE, HKV, D), dtype=bf, device=dev)
        for i in range(0, total, 2048):  # chunked: keeps the fp32 temporary small
            self.cache[i:i + 2048] = rn(min(2048, total - i), 2, PAGE, HKV, D).to(bf)
        self.indices = torch.randperm(total, generator=g, device=dev).to(torch.int32)
        self.indptr = (torch.arange(B + 1, device=dev) * n_pages).to(torch.int32)
        self.last = torch.full((B,), PAGE, dtype=torch.int32, device=dev)
        self.q.copy_(rn(B, HQ, D).to(bf))
        self.sm_scale = torch.tensor([1.0 / 16], device=dev)
        # GDN recurrent step
        nrm = lambda t: (t / torch.sqrt(t.square().sum(-1, keepdim=True) + 1e-6))  # noqa: E731
        self.gq.copy_((nrm(rn(B, NK, GD)) * GD ** -0.5).to(bf))
        self.gk.copy_(nrm(rn(B, NK, GD)).to(bf))
        self.gv.copy_(rn(B, NV, GD).to(bf))
        self.gg.copy_(-torch.nn.functional.softplus(rn(B, NV)))
        self.gbeta.copy_(torch.sigmoid(rn(B, NV)).to(bf))
        self.state = rn(B, NV, GD, GD) * 0.03
        # MoE block
        rb = lambda lo, hi, *s: torch.randint(lo, hi, s, generator=g, device=dev, dtype=torch.int32).to(torch.uint8)  # noqa: E731
        self.x1.copy_(rn(B, H).to(bf))
        if weight_seed is not None:
            g = torch.Generator(device=dev).manual_seed(weight_seed)  # rn / rb below draw from this one
        self.w = dict(
            ln2=torch.ones(H, device=dev), w_router=(rn(NE, H) / H ** 0.5).to(bf), w_shg=(rn(H) / H ** 0.5).to(bf),
            e_gw=rb(0, 256, n_experts_local, 2 * FE, H // 2), e_gs=rb(119, 128, n_experts_local, 2 * FE, H // 32),
            e_dw=rb(0, 256, n_experts_local, H, FE // 2), e_ds=rb(119, 128, n_experts_local, H, FE // 32),
            w_gate=rb(0, 256, FS, H // 2), s_gate=rb(119, 128, FS, H // 32), w_up=rb(0, 256, FS, H // 2),
            s_up=rb(119, 128, FS, H // 32), w_down=rb(0, 256, H, FS // 2), s_down=rb(119, 128, H, FS // 32))

    def attn_bytes(self):
        return B * CTX * 2 * HKV * D * 2

    @staticmethod
    def gdn_bytes():
        return 2 * B * NV * GD * GD * 4

    @staticmethod
    def moe_bytes(distinct_experts):
        return distinct_experts * EXPERT_BYTES + EXPERT_BYTES + NE * H * 2 + 2 * B * H * 2


class FullLayer:
    """the sublayer glue of a 35B-A3B layer around the three kernels: MXFP8 projections (q/k/v/z/a/b/o of the GDN
    sublayer, q+gate/k/v/o of the attention sublayer: 34.7 + 28.1 MB), conv, norms, RoPE, KV write, output projections.
    Weights N(0, 0.02) quantised to MXFP8 on the device."""

    def __init__(self, dev, seed):
        g = torch.Generator(device=dev).manual_seed(seed)
        rn = lambda *s: torch.randn(s, generator=g, device=dev)  # noqa: E731

        def mx8(n, k):  # E8M0 per 32 inputs: e = ceil(log2(amax / 448)); payload e4m3
            w = rn(n, k) * 0.02
            blk = w.reshape(n, k // 32, 32)
            e = torch.ceil(torch.log2(blk.abs().amax(-1, keepdim=True).clamp_min(2.0 ** -126) / 448.0)).clamp(-127, 127)
            q8 = (blk / torch.exp2(e)).to(torch.float8_e4m3fn).reshape(n, k).contiguous()
            return q8, (e.squeeze(-1) + 127).to(torch.uint8).contiguous()

        KD, VD = NK * GD, NV * GD
        gw = {}
        for n, shp in (("q", (KD, H)), ("k", (KD, H)), ("v", (VD, H)), ("z", (VD, H)), ("a", (NV, H)), ("b", (NV, H)),
                       ("o", (H, VD))):
            gw["w_" + n], gw["s_" + n] = mx8(*shp)
        for n, width in (("q", KD), ("k", KD), ("v", VD)):
            gw[f"w_{n}_conv"] = (rn(width, 4) * 0.1).to(torch.bfloat16)
        gw["input_norm_w"] = (1 + 0.02 * rn(H)).to(torch.bfloat16)
        gw["a_log"] = (torch.rand(NV, generator=g, device=dev) * 15 + 1).log()
        gw["dt_bias"] = (rn(NV) * 0.02).to(torch.bfloat16)
        gw["o_norm_w"] = (1 + 0.02 * rn(GD)).to(torch.bfloat16)
        aw = {}
        for n, shp in (("q", (HQ * D * 2, H)), ("k", (HKV * D, H)), ("v", (HKV * D, H)), ("o", (H, HQ * D))):
            aw["w_" + n], aw["s_" + n] = mx8(*shp)
        aw["ln1"] = 1 + 0.02 * rn(H)
        aw["q_norm"] = 1 + 0.02 * rn(D)
        aw["k_norm"] = 1 + 0.02 * rn(D)
        self.gw, self.aw = gw, aw
        self.proj_bytes = sum(t.numel() * t.element_size() for w in (gw, aw) for k, t in w.items()
                              if k.startswith(("w_", "s_")) and "conv" not in k)
        self.conv = tuple(torch.zeros((B, 3, c), dtype=torch.bfloat16, device=dev) for c in (KD, KD, VD))
        self.x = (rn(B, H) * 0.5).to(torch.bfloat16)
        inv = 1.0 / (1e7 ** (torch.arange(0, 64, 2, device=dev).float() / 64))
        f = torch.full((B, 1), float(CTX), device=dev) * inv.reshape(1, -1)
        self.cos, self.sin = f.cos().contiguous(), f.sin().contiguous()

    def step(self, q35, wl, moe_step):
        """GDN sublayer -> attention sublayer (history of CTX - 1 tokens + the current one, whose row is written into
        the last slot of each sequence's last page) -> MoE block"""
        fused, _, _ = q35.layers.gdn(self.x.reshape(B, 1, H), torch.zeros_like(self.x).reshape(B, 1, H), self.gw,
                                     wl.state, self.conv)
        x1 = q35.layers.attention(fused.reshape(B, H), self.aw, self.cos, self.sin, wl.cache, wl.indptr, wl.indices,
                                  wl.last_hist, cache_location=wl.cache_loc, heads=HQ, kv_heads=HKV, head_dim=D,
                                  sm_scale=wl.sm_scale)
        return moe_step(x1)


# ----------------------------------------------------------------------------------------------------------------
def timed_rounds(run_step, steps, barrier, min_seconds=0.5, max_rounds=200, agree=None):
    """rounds of exactly `steps` steps, each bracketed by CUDA events on the launching stream.  The number of rounds is
    fixed after the first one so that about min_seconds of device time are measured (at least 3 rounds); with several
    ranks `agree` (a max-reduction over the ranks) makes every rank run the same number of rounds -- the rounds hold
    collectives.  Returns the per-round milliseconds."""
    rounds, n_rounds = [], 3
    while len(rounds) < n_rounds:
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        t0.record()
        for _ in range(steps):
            run_step()
        t1.record()
        barrier()
        rounds.append(t0.elapsed_time(t1))
        if len(rounds) == 1:
            first = agree(rounds[0]) if agree else rounds[0]
            n_rounds = max(3, min(max_rounds, int(math.ceil(min_seconds * 1e3 / max(first, 1e-3)))))
    return rounds


def median(xs):
    s = sorted(xs)
    return s[len(s) // 2]


def capture(fn, warm=2):
    """fn captured into a CUDA graph through the public API (kernel launches that together take a few hundred
    microseconds would otherwise be paced by the Python launch path)"""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        for _ in range(warm):
            fn()
        with torch.cuda.graph(graph, stream=side):
            fn()
    torch.cuda.current_stream().wait_stream(side)
    graph.replay()
    return graph


def part_entry(name, nbytes, ms, peak):
    gbs = nbytes / (ms * 1e-3) / 1e9
    return {"part": name, "algorithmic_bytes": int(nbytes), "ms": ms, "achieved": gbs, "unit": "GB/s",
            "frac": gbs / peak, "frac_of_nominal_8tbs": gbs / NOMINAL_GBS}


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
        import datetime
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=120))
    wl = Workload(dev, seed=1000 + rank, weight_seed=999 if world > 1 else None)
    L = q35._lib.lib()
    if world > 1:
        from ax_dsl_kernels_b200 import parallel
        ep = parallel.ExpertParallelMoE(wl.w, TOPK, dist.group.WORLD, exchange=args.ep_exchange)
        moe_step = lambda x: ep.forward(x, wl.moe_out)  # noqa: E731
    else:
        q35.prepare_moe_weights(wl.w)  # load-time re-layout of the E8M0 scales for the one-call decode block
        moe_step = lambda x: q35.moe_block(x, wl.w, TOPK, wl.moe_out)  # noqa: E731

    def gdn_only():
        q35.gdn_recurrent_step(wl.gq, wl.gk, wl.gv, wl.gg, wl.gbeta, wl.state, wl.g_out, wl.state)

    def attn_only():
        q35.paged_attention_decode(wl.q, wl.cache, wl.indptr, wl.indices, wl.last, wl.attn_out, sm_scale=wl.sm_scale)

    def step():
        gdn_only()
        attn_only()
        moe_step(wl.x1)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def agree(ms):  # the slowest rank's figure, the same on every rank
        if dist is None:
            return ms
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    clocks = ClockSampler(local) if rank == 0 else None
    if clocks:
        clocks.start()  # sampled from the warm-up to the end of the end-to-end loop (nvidia-smi, every 100 ms)
    warm = max(args.warmup, 3)
    for _ in range(warm):
        step()
    barrier()
    n0 = L.q35_launch_count()
    step()
    launches_per_step = L.q35_launch_count() - n0  # kernels of this library enqueued by one step (torch / NCCL not counted)
    # The step is captured once into a CUDA graph through the public API and replayed; with several ranks the graph
    # holds the NCCL collectives of the expert exchange as well.  --no-graph launches every step eagerly.
    graph, graph_note = None, ""
    if not args.no_graph:
        try:
            graph = capture(step)
        except RuntimeError as e:  # a communicator that cannot be captured: the step is launched eagerly instead
            if world == 1:
                raise
            graph_note = f" (graph capture of the step with its collectives failed: {str(e)[:80]})"
    run_step = graph.replay if graph is not None else step
    barrier()
    rounds = timed_rounds(run_step, args.steps, barrier, agree=agree)
    ms = median(rounds)

    # every part on its own, same process, right after the timed region (events cannot be placed inside a replayed
    # graph): each part's launches captured as a graph of their own and replayed `steps` times
    parts = {}
    if world == 1:
        for name, fn in (("attn.paged_decode (plan + decode + merge)", attn_only), ("gdn.step", gdn_only),
                         ("moe block (router, routed experts, shared expert, combine)", lambda: moe_step(wl.x1))):
            gph = capture(fn) if not args.no_graph else None
            parts[name] = median(timed_rounds(gph.replay if gph else fn, args.steps, barrier, min_seconds=0.2)) / args.steps
    else:
        gph = capture(attn_only) if not args.no_graph else None
        parts["attn.paged_decode (plan + decode + merge)"] = median(
            timed_rounds(gph.replay if gph else attn_only, args.steps, barrier, min_seconds=0.2, agree=agree)) / args.steps
    attn_ms = parts["attn.paged_decode (plan + decode + merge)"]
    ep_check = None
    if world > 1:  # the expert-parallel block against the one-GPU block on this rank's tokens (every rank holds all weights)
        ref = q35.moe_block(wl.x1, q35.prepare_moe_weights(wl.w), TOPK)[0].float()
        got = ep.forward(wl.x1, wl.moe_out).float()
        worst = ((got - ref).abs().max() / ref.square().mean().sqrt()).reshape(1)
        dist.all_reduce(worst, op=dist.ReduceOp.MAX)
        ep_check = {"max_err_over_rms_vs_one_gpu_block": float(worst.item()),
                    "exchange": "peer memory" if getattr(ep, "_peer", None) else "nccl"}
    ep_phases = None
    if world > 1:  # the expert-parallel MoE step piece by piece: each piece captured as a graph of its own and replayed
        ep_phases = {}
        for name, fn in ep.phases(wl.x1, wl.moe_out):
            gph = capture(fn) if not args.no_graph else None
            ep_phases[name] = round(median(timed_rounds(gph.replay if gph else fn, args.steps, barrier, min_seconds=0.1,
                                                        agree=agree)) / args.steps * 1e3, 1)
        gph = capture(lambda: ep.forward(wl.x1, wl.moe_out)) if not args.no_graph else None
        ep_phases["whole MoE step (shared expert overlapped)"] = round(median(timed_rounds(
            gph.replay if gph else (lambda: ep.forward(wl.x1, wl.moe_out)), args.steps, barrier, min_seconds=0.1,
            agree=agree)) / args.steps * 1e3, 1)

    # end to end: the per-step activations start in ONE pinned host block and the results come back into one
    host_in = torch.empty(wl.inputs.nbytes, dtype=torch.uint8).pin_memory()
    host_in.copy_(wl.inputs.buf)
    host_out = torch.empty(wl.outputs.nbytes, dtype=torch.uint8).pin_memory()

    def step_e2e():
        wl.inputs.buf.copy_(host_in, non_blocking=True)
        run_step()  # the captured step reads and writes the device buffers the copies fill and drain
        host_out.copy_(wl.outputs.buf, non_blocking=True)
        torch.cuda.current_stream().synchronize()  # the caller reads the results

    for _ in range(3):
        step_e2e()
    e2e_ms = median(timed_rounds(step_e2e, args.steps, barrier, agree=agree))

    # the same step with the sublayer glue (projections, conv, norms, RoPE, KV write, o-proj), one GPU only
    full = None
    if world == 1 and not args.no_full_layer:
        fl = FullLayer(dev, seed=7)
        # the attention sublayer appends the current token: history = CTX - 1 cached tokens, new row -> last slot
        wl.last_hist = torch.full((B,), PAGE - 1, dtype=torch.int32, device=dev)
        last_page = wl.indices[(wl.indptr[1:] - 1).long()]
        wl.cache_loc = torch.stack([last_page, torch.full_like(last_page, PAGE - 1)], 1).contiguous()
        full_step = lambda: fl.step(q35, wl, moe_step)  # noqa: E731
        full_step()
        n0 = L.q35_launch_count()
        full_step()
        full_launches = L.q35_launch_count() - n0
        fg = capture(full_step) if not args.no_graph else None
        full_ms = median(timed_rounds(fg.replay if fg else full_step, args.steps, barrier, min_seconds=0.3)) / args.steps
        full = {"workload": "the headline step inside its sublayers: GDN sublayer (folded RMSNorm, MXFP8 q/k/v/z/a/b "
                "projections, conv + SiLU, l2norm / gates, gdn.step, gated RMSNorm, o-proj + residual) -> attention "
                "sublayer (RMSNorm, MXFP8 q+gate/k/v projections, q/k norm, RoPE, paged decode with the current token, "
                "KV write, sigmoid gate, o-proj + residual) -> MoE block",
                "ms_per_step": full_ms, "value": B / (full_ms * 1e-3), "unit": "tok/s", "gpu_launches_per_step": int(full_launches),
                "projection_weight_bytes": int(fl.proj_bytes)}

    times = torch.tensor([ms, e2e_ms], device=dev)
    if dist is not None:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms, e2e_ms = times.tolist()
    status = q35.device_status()
    if rank == 0:
        peak, _, peak_src = measured_peaks()
        achieved = wl.attn_bytes() / (attn_ms * 1e-3) / 1e9
        sms = torch.cuda.get_device_properties(dev).multi_processor_count
        line = {
            "metric": METRIC, "value": world * B * args.steps / (ms * 1e-3), "unit": "tok/s", "n_gpus": world,
            "steps": args.steps, "warmup": warm, "ms_per_step": ms / args.steps, "rounds": len(rounds),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic (seeded, on-device)", "config": headline_config(world),
            "launch": ("cuda graph replay" if graph is not None else "eager") + graph_note,
            "timing": f"median of {len(rounds)} rounds of {args.steps} steps, CUDA events, max over ranks",
            "e2e": {"value": world * B * args.steps / (e2e_ms * 1e-3), "unit": "tok/s",
                    "h2d_bytes_per_step": wl.inputs.nbytes, "d2h_bytes_per_step": wl.outputs.nbytes},
            "gpu_launches": int(args.steps * launches_per_step), "gpu_launches_per_step": int(launches_per_step),
            "roofline": {"bound": "hbm", "kernel": "attn_decode_kernel<256,bf16> (+ plan and merge launches)",
                         "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_source": peak_src, "traffic": attn_traffic(wl, sms, args.attn_read_ratio),
                         "algorithmic_bytes": wl.attn_bytes(), "ms_per_launch": attn_ms},
            "clocks": clocks_summary(clocks),
            "device_status": status,
        }
        if ep_phases is not None:
            line["ep_phases_us_rank0"] = ep_phases
            line["ep_check"] = ep_check
        if world == 1:
            ids = q35.moe_block(wl.x1, wl.w, TOPK, wl.moe_out)[1]
            distinct = int(torch.unique(ids).numel())
            names = list(parts)
            all_parts = [part_entry(names[0], wl.attn_bytes(), parts[names[0]], peak),
                         part_entry(names[1], wl.gdn_bytes(), parts[names[1]], peak),
                         part_entry(names[2] + f", {distinct} distinct experts", wl.moe_bytes(distinct), parts[names[2]], peak)]
            total_bytes = wl.attn_bytes() + wl.gdn_bytes() + wl.moe_bytes(distinct)
            all_parts.append(part_entry("whole step", total_bytes, ms / args.steps, peak))
            line["roofline_all"] = all_parts
            if full is not None:
                full["roofline"] = part_entry("whole step with sublayer glue",
                                              total_bytes + full["projection_weight_bytes"], full["ms_per_step"], peak)
                line["full_layer"] = full
            if not args.no_cpu:
                line["cpu_baseline"] = cpu_sample(CpuCase(), 1)
        print(json.dumps(line), flush=True)
    if dist is not None:
        if graph is not None:  # captured collectives keep the communicator busy at teardown: leave without it
            barrier()
            sys.stdout.flush()
            os._exit(0)
        dist.destroy_process_group()


def attn_traffic(wl, sms, read_ratio):
    """DRAM bytes of one attention decode launch: reads = the K/V bytes times the read ratio an ncu capture of a
    capture-sized case of the same kernel measured (dram bytes read / K-V bytes: every byte once), writes = the
    split-KV partials, one [m, l, O] per (segment or CTA, warp, query head of the group)."""
    reads = wl.attn_bytes() * read_ratio
    partials = (B * HKV + sms) * 4 * (HQ // HKV) * (D + 2) * 4
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


def clocks_summary(clocks):
    if not clocks:
        return None
    clocks.stop()
    return clocks.summary()


# ----------------------------------------------------------------------------------------------------------------
class CpuCase:
    """bounded sample of the headline workload for the CPU oracle: n_attn sequences at the full context, n_moe tokens
    through the MoE block, n_gdn sequences of the GDN step (built once, outside the timed region)"""

    def __init__(self, n_attn=2, n_moe=16, n_gdn=4):
        from _cases import gdn_step_case, moe_case, paged_case
        self.n = (n_attn, n_moe, n_gdn)
        self.attn = paged_case([CTX] * n_attn, seed=1)
        self.moe = moe_case(n_moe, seed=3)
        self.gdn = gdn_step_case(B=n_gdn, seed=2)


def cpu_sample(case, reps):
    """the CPU oracle on the bounded sample: dequantisation of the packed experts happens inside the timed region (the
    accelerator also consumes packed weights).  tokens/s = 1 / (per-token seconds of the three parts added)."""
    from oracle import attention as oattn, gdn as ogdn, moe as omoe
    from _cases import dequant_shared
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    n_attn, n_moe, n_gdn = case.n
    q, cache, indptr, indices, last, _ = case.attn
    x1, w = case.moe
    gq, gk, gv, gg, gb, st = case.gdn
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
    the NPU DSL and cannot run); timed on the host cores, rank 0 only.  A step = the bounded sample; --steps and
    --warmup are honoured as long as the run stays within a few minutes (then fewer steps are run and reported)."""
    if int(os.environ.get("RANK", 0)) != 0:
        return
    world = int(os.environ.get("WORLD_SIZE", 1))
    case = CpuCase()
    budget_s = 200.0
    t_start = time.perf_counter()
    warm = 0
    for _ in range(max(0, args.warmup)):
        cpu_sample(case, 1)
        warm += 1
        if time.perf_counter() - t_start > 0.2 * budget_s:
            break
    res = []
    t0 = time.perf_counter()
    for _ in range(max(1, args.steps)):
        res.append(cpu_sample(case, 1))
        if time.perf_counter() - t_start > budget_s:
            break
    wall = time.perf_counter() - t0
    med = sorted(r["seconds_per_token"] for r in res)[len(res) // 2]
    value = 1.0 / med
    cb = dict(res[0], value=value, seconds_per_token=med)
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": "tok/s", "n_gpus": world,
        "steps": len(res), "warmup": warm, "ms_per_step": 1e3 * wall / len(res), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic (seeded)",
        "config": headline_config(world),
        "cpu_baseline": cb, "e2e": {"value": value, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
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
    if name == "attn_fp8":
        B, CTX = 32, 8192  # 268 MB of FP8 KV
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
    elif name == "moe_ep8":  # what one of 8 expert-parallel ranks runs per decode step: 512 gathered tokens, 32 local experts
        from ax_dsl_kernels_b200 import _lib, moe as qmoe
        wl = Workload(dev, seed=1, attn=False)
        T, lo, hi = 8 * B, 0, NE // 8
        h2 = (rn(T, H) * 0.5).to(bf)
        ids, rw = q35.route(rn(T, NE), TOPK)
        w = {k: wl.w[k][lo:hi].contiguous() for k in ("e_gw", "e_gs", "e_dw", "e_ds")}
        gs_t, ds_t = qmoe.tile_scales(w["e_gs"], True), qmoe.tile_scales(w["e_ds"], False)
        base = torch.tensor([lo], dtype=torch.int32, device=dev)
        partial = torch.empty((T, H), dtype=torch.float32, device=dev)
        fn = lambda: _lib.run("moe.experts", h2=h2, ids=ids, rw=rw, e_gw=qmoe._u8(w["e_gw"]), e_gs=qmoe._u8(w["e_gs"]),  # noqa: E731
                              e_dw=qmoe._u8(w["e_dw"]), e_ds=qmoe._u8(w["e_ds"]), expert_base=base, partial_out=partial,
                              e_gs_tiled=gs_t, e_ds_tiled=ds_t)
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
        wl = Workload(dev, seed=1, attn=name in ("attn", "attn_fp8"))
        units = B
        if name == "attn_fp8":  # the same launch over an FP8 E4M3 cache with per-head scales
            kvs = (wl.cache.float().abs().amax((0, 2, 4)) / 448.0).contiguous()
            c8 = (wl.cache.float() / kvs.reshape(1, 2, 1, HKV, 1)).to(torch.float8_e4m3fn)
            fn = lambda: q35.paged_attention_decode(wl.q, c8, wl.indptr, wl.indices, wl.last, wl.attn_out,  # noqa: E731
                                                    sm_scale=wl.sm_scale, kv_scale=kvs)
        elif name == "attn":
            fn = lambda: q35.paged_attention_decode(wl.q, wl.cache, wl.indptr, wl.indices, wl.last, wl.attn_out,  # noqa: E731
                                                    sm_scale=wl.sm_scale)
        elif name == "gdn":
            fn = lambda: q35.gdn_recurrent_step(wl.gq, wl.gk, wl.gv, wl.gg, wl.gbeta, wl.state, wl.g_out, wl.state)  # noqa: E731
        else:
            q35.prepare_moe_weights(wl.w)
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
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="headline")
    ap.add_argument("--layers", type=int, default=16, help="layers of the --config c5 decode group")
    ap.add_argument("--ep-exchange", default="auto", choices=["auto", "peer", "nccl"],
                    help="several GPUs: the expert-parallel exchange (headline) and the tensor-parallel all-reduce (c5) through this "
                    "library's peer-memory kernels or through NCCL")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline sample")
    ap.add_argument("--no-full-layer", action="store_true", help="skip the full-layer variant of the step")
    ap.add_argument("--no-graph", action="store_true", help="launch the timed steps eagerly instead of replaying a CUDA graph")
    ap.add_argument("--attn-read-ratio", type=float, default=268.70 / 268.44,
                    help="DRAM bytes read per K/V byte by the attention kernel, from an ncu capture (default: the capture "
                         "of the 16 x 8192 case, 268.70 MB read for 268.44 MB of K/V)")
    ap.add_argument("--profile-case", choices=["attn", "attn_fp8", "gdn", "moe", "moe_ep8", "gdn_prefill", "attn_prefill", "moe_prefill", "lm_head"], help="run one kernel on a capture-sized case")
    args = ap.parse_args()
    if args.profile_case:
        run_profile_case(args.profile_case, max(1, min(args.steps, 5)))
    elif args.config != "headline":
        import bench_configs
        bench_configs.run(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
