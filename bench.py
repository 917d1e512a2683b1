#!/usr/bin/env python
"""Benchmark of the MoE layer forward + backward on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One "step" is one forward + backward pass of the layer (router -> routing metadata -> expert
compute -> gradients of input, router weight and both expert weight tensors) over one batch of
seeded synthetic tokens.  N = 1 runs the Mixtral-8x7B-shaped layer; N > 1 runs the
DeepSeek-V3-shaped expert-parallel layer, experts sharded over the ranks (launch with torchrun).
Rank 0 prints ONE JSON line.

``--impl reference`` times the reference algorithm's CPU restatement (oracle/moe_oracle.py, fp32,
all host threads) on a bounded token sample of the same workload.  ``--impl reference_triton`` (used by the N = 1
run for its ``gpu_baseline`` entry when a checkout of the reference is found) times the reference's own Triton
grouped GEMMs on the GPU.

Every line of our arm carries ``parity``: after the timed region the device status word is read (a non-zero code
fails the run) and a fixed sample of tokens (every 257th) is recomputed by the fp32 oracle -- output and input
gradient -- at every N.
"""
from __future__ import annotations

import argparse
import datetime
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if "reference_triton" not in sys.argv:     # that mode imports the reference's package of the same name instead
    sys.path.insert(0, os.path.join(ROOT, "moe-explore_b200"))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

WORKLOADS = {
    # name: T (per GPU), d, E, k, I, router
    "mixtral_8x7b": dict(T=8192, d=4096, E=8, k=2, I=14336, router="linear"),
    "qwen15_moe_a27b": dict(T=16384, d=2048, E=60, k=4, I=1408, router="logits_bias"),
    "deepseek_v3_ep": dict(T=32768, d=7168, E=256, k=8, I=2048, router="zipf"),
    "olmoe_8192": dict(T=8192, d=2048, E=64, k=8, I=1024, router="logits"),
    # routing-stress sweep on the OLMoE shape: pick T with --tokens and the router with --router
    "olmoe_sweep": dict(T=8192, d=2048, E=64, k=8, I=1024, router="logits"),
}
METRIC = "moe_layer_fwd_bwd_tokens_per_s"


def algorithmic_flops(w, tokens, with_router):
    """18*R*d*I for the six expert contractions (+ 6*T*d*E when a router linear layer is timed)."""
    f = 18.0 * tokens * w["k"] * w["d"] * w["I"]
    if with_router:
        f += 6.0 * tokens * w["d"] * w["E"]
    return f


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            p = json.load(open(path))
            return dict(source="measured", burst=float(p["bf16_tflops"]), sustained=float(p["bf16_tflops_sustained"]),
                        hbm=float(p["hbm_gbs"]))
        except Exception:
            pass
    return dict(source="fallback", burst=1590.0, sustained=1400.0, hbm=6650.0)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-i", str(self.gpu_index), "-lms", "50"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, smax, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                smax = float(parts[2])
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return dict(sm_mhz=sm[len(sm) // 2] if sm else None, sm_max_mhz=smax, reasons=sorted(reasons), samples=len(sm))


# ----------------------------------------------------------------------------------------------
# synthetic inputs
# ----------------------------------------------------------------------------------------------
def make_logits(w, T, gen, device, rank=0):
    """Router logits for the workloads that supply them directly (no router GEMM in the step)."""
    E = w["E"]
    if w["router"] == "logits":
        return torch.randn(T, E, generator=gen, device=device)
    if w["router"] == "logits_bias":
        bias = torch.randn(E, generator=gen, device=device) * 0.5
        return torch.randn(T, E, generator=gen, device=device) + bias
    if w["router"] == "degenerate":
        # >= 90 % of the tokens send a slot to one expert; 8 experts never get a row
        logits = torch.randn(T, E, generator=gen, device=device)
        hot = torch.rand(T, generator=gen, device=device) < 0.95
        logits[hot, 5] += 20.0
        logits[:, E - 8:] = -1e4
        return logits
    if w["router"] in ("zipf", "zipf15"):
        # popularity ~ rank^-1.1 over a random expert permutation (same permutation on every rank);
        # log p + Gumbel noise, so the top-k is a sample without replacement proportional to p
        pg = torch.Generator(device=device).manual_seed(1234)
        p = torch.arange(1, E + 1, dtype=torch.float32, device=device) ** (-1.5 if w["router"] == "zipf15" else -1.1)
        p = (p / p.sum())[torch.randperm(E, generator=pg, device=device)]
        u = torch.rand(T, E, generator=gen, device=device).clamp_min(1e-20)
        return torch.log(p) - torch.log(-torch.log(u))
    raise ValueError(w["router"])


def make_inputs(w, device, rank=0, world=1, dtype=torch.bfloat16):
    """x ~ N(0,1); weights ~ N(0,0.02); gate/up drawn separately and interleaved (even = gate)."""
    from moe_explore.params import interleave_gate_up

    T, d, E, k, I = w["T"], w["d"], w["E"], w["k"], w["I"]
    gen = torch.Generator(device=device).manual_seed(rank)
    x = torch.randn(T, d, generator=gen, device=device).to(dtype)
    grad_out = torch.randn(T, d, generator=gen, device=device).to(dtype)
    e_local = E // world
    wgen = torch.Generator(device=device).manual_seed(1000 + rank)

    def normal(*shape):
        out = torch.empty(*shape, dtype=dtype, device=device)
        for e in range(shape[0]):  # per expert, to bound the fp32 temporary
            out[e] = (torch.randn(*shape[1:], generator=wgen, device=device) * 0.02).to(dtype)
        return out

    gate, up = normal(e_local, d, I), normal(e_local, d, I)
    w1 = interleave_gate_up(gate, up)
    del gate, up
    w2 = normal(e_local, I, d)
    router_weight, logits = None, None
    if w["router"] == "linear":
        rg = torch.Generator(device=device).manual_seed(77)
        router_weight = (torch.randn(d, E, generator=rg, device=device) * 0.02).to(dtype)
    else:
        logits = make_logits(w, T, gen, device, rank)
    return dict(x=x, grad_out=grad_out, w1=w1, w2=w2, router_weight=router_weight, logits=logits)


# ----------------------------------------------------------------------------------------------
# our arm
# ----------------------------------------------------------------------------------------------
def scores_from_logits(logits, k, dtype):
    top, idx = torch.topk(logits, k, dim=-1, sorted=False)
    return torch.softmax(top, dim=-1, dtype=torch.float32).to(dtype), idx


class Tracer:
    """Observer handed to the package (``_native.TRACER``): counts this library's launches and brackets each with
    CUDA events on the current stream, keyed by kernel variant."""

    def __init__(self, timing=True):
        self.launches = 0
        self.timing = timing
        self.sections = {}

    def count(self, n):
        self.launches += n

    class _Section:
        def __init__(self, owner, key, rows):
            self.owner, self.key, self.rows = owner, key, rows

        def __enter__(self):
            self.start = torch.cuda.Event(enable_timing=True)
            self.end = torch.cuda.Event(enable_timing=True)
            self.start.record()

        def __exit__(self, *exc):
            self.end.record()
            self.owner.sections.setdefault(self.key, []).append((self.start, self.end, self.rows))
            return False

    class _Off:
        def __enter__(self):
            return None

        def __exit__(self, *exc):
            return False

    def section(self, key, rows=None):
        return Tracer._Section(self, key, rows) if self.timing else Tracer._Off()

    def ms_per_step(self, steps):
        return {k_: round(sum(a.elapsed_time(b) for a, b, _ in v) / steps, 4) for k_, v in sorted(self.sections.items())}


def gate_up_key(sections):
    for key in ("mgrouped_gemm:glu+gather", "mgrouped_gemm:glu"):
        if key in sections:
            return key
    return None


def parity_record(x, out, dx, idx, scores, weights, grad_out, router_weight=None, topk=None):
    """Recompute a fixed sample of tokens (every 257th) with the fp32 oracle -- output and input gradient -- from the
    same bf16 inputs and routing decision; returns max |a-b| / max |b| for both.  ``weights`` = (w1, w2) holding ALL
    experts in the order ``idx`` refers to.  With ``router_weight`` the router is part of the step: the scores are
    re-derived from the sampled tokens in fp32 (softmax over the selected logits) so that the input gradient includes
    the path through the router, as the timed step's does."""
    from oracle import moe_oracle as O

    T = out.size(0)
    sample = torch.arange(0, T, 257, device=out.device)
    xs = x[sample].float().requires_grad_()
    if router_weight is not None:
        sc = torch.softmax(torch.gather(xs @ router_weight.detach().float(), -1, idx[sample]), -1)
    else:
        sc = scores[sample].float()
    ref = O.expert_compute(xs, sc, idx[sample], weights[0].detach(), weights[1].detach(), "swiglu")
    ref.backward(grad_out[sample].float())
    rel = lambda a, b: float((a.float() - b).abs().max() / b.abs().max().clamp_min(1e-30))
    return {"out": rel(out[sample], ref.detach()), "dx": rel(dx[sample], xs.grad), "tokens_checked": int(sample.numel())}


def bind_to_gpu_cpus(device_index: int):
    """Restrict this process to the CPU cores NVML reports as local to its GPU (reading NVML only; the affinity is a
    property of this process).  Page-locked buffers allocated afterwards are first touched, and so placed, on that
    socket's memory: with one rank per GPU on a two-socket host, buffers on the other socket send every host copy
    over the inter-socket link.  Returns the number of cores kept, or None when nothing was changed."""
    try:
        import pynvml

        pynvml.nvmlInit()
        uuid = str(torch.cuda.get_device_properties(device_index).uuid)
        handle = pynvml.nvmlDeviceGetHandleByUUID(uuid if uuid.startswith("GPU-") else "GPU-" + uuid)
        words = pynvml.nvmlDeviceGetCpuAffinity(handle, ((os.cpu_count() or 64) + 63) // 64)
        local = {64 * i + b for i, word in enumerate(words) for b in range(64) if (int(word) >> b) & 1}
        keep = os.sched_getaffinity(0) & local
        if keep and keep != os.sched_getaffinity(0):
            os.sched_setaffinity(0, keep)
            return len(keep)
    except Exception:
        pass
    return None


def run_ours(args):
    import torch.distributed as dist

    from moe_explore import _native
    from moe_explore.expert_compute import expert_compute
    from moe_explore.functional.topk_moe import topk_moe_forward
    from moe_explore.params import MLPParams, MOEParams, TopkRouterParams
    from moe_explore.router import router
    from moe_explore.routing_plan import build_routing_plan, device_status

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("--gpus N > 1 must be launched with torch.distributed.run (one rank per GPU)")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    cpu_binding = bind_to_gpu_cpus(local_rank) if world > 1 and not args.no_cpu_binding else None
    _native.load()
    _native.query_device(local_rank)
    if world > 1:
        # a collective that has not finished after five minutes never will: end the run instead of holding the GPUs
        dist.init_process_group("nccl", device_id=device, timeout=datetime.timedelta(minutes=5))

    name = args.workload or ("mixtral_8x7b" if world == 1 else "deepseek_v3_ep")
    w = dict(WORKLOADS[name])
    if args.tokens:
        w["T"] = args.tokens
    if args.router:
        w["router"] = args.router
    gather_in_gemm = {"auto": None, "on": True, "off": False}[args.gather_in_gemm]
    inp = make_inputs(w, device, rank, world)
    with_router = inp["router_weight"] is not None
    x, grad_out = inp["x"], inp["grad_out"]
    w1 = inp["w1"].requires_grad_()
    w2 = inp["w2"].requires_grad_()
    if with_router:
        inp["router_weight"].requires_grad_()

    ep_context = None
    remap = None
    if world > 1:
        from moe_explore.expert_parallel import EPContext, balanced_placement, ep_expert_compute

        if args.placement == "balanced":
            # static placement from the expert load of ANOTHER batch of the same router distribution (seeded apart
            # from the batch that is timed): what a deployment gets from load statistics of earlier steps
            with torch.no_grad():
                pgen = torch.Generator(device=device).manual_seed(10_000 + rank)
                other = make_logits(w, w["T"], pgen, device, rank)
                _, idx0 = scores_from_logits(other, w["k"], x.dtype)
                load = torch.bincount(idx0.reshape(-1), minlength=w["E"]).to(torch.int64)
                del other
            dist.all_reduce(load)
            remap = balanced_placement(load.cpu(), world).to(device)

        if args.ep_mode == "peer":
            ep_context = EPContext(dist.group.WORLD, w["T"], w["d"], w["k"], x.dtype, device,
                                   dispatch="dma" if args.ep_pull == "dma" else "pull")
            if args.ep_pull != "dma":
                ep_context.pull_mode = args.ep_pull
            if args.ep_reserved_sms is not None:
                ep_context.reserved_sms = args.ep_reserved_sms
            if args.ep_chunks:
                ep_context.chunks = args.ep_chunks
                ep_context.geometric = False
            if args.ep_slices != "auto":
                ep_context.slice_pairs = args.ep_slices == "pairs"

    def routing_of(x_in):
        """The routing decision of one step (same ops as inside the step): scores [T,k], positions in the weights."""
        with torch.no_grad():
            if with_router:
                scores, idx = router(x_in, TopkRouterParams(inp["router_weight"], w["k"], False, False))
            else:
                scores, idx = scores_from_logits(inp["logits"], w["k"], x_in.dtype)
            if remap is not None:
                idx = remap[idx]
        return scores, idx

    def step(x_in, g_in):
        """One forward + backward on device-resident inputs; returns (out, dx)."""
        x_in.requires_grad_(True)
        x_in.grad = None
        if world == 1:
            if with_router:
                params = MOEParams(TopkRouterParams(inp["router_weight"], w["k"], False, False),
                                   MLPParams(w1, w2, "swiglu"), w["E"], w["k"])
                out = topk_moe_forward(x_in, params, gather_in_gemm=gather_in_gemm)
            else:
                logits = inp["logits"].requires_grad_()
                scores, idx = scores_from_logits(logits, w["k"], x_in.dtype)
                plan = build_routing_plan(idx, w["E"], w["k"], want_perm=False)
                out = expert_compute(x_in, scores, w1, w2, plan, "swiglu", gather_in_gemm=gather_in_gemm)
        else:
            logits = inp["logits"].requires_grad_()
            scores, idx = scores_from_logits(logits, w["k"], x_in.dtype)
            if remap is not None:
                idx = remap[idx]   # logical expert id -> position in the sharded weights
            out = ep_expert_compute(x_in, scores, idx, w1, w2, w["E"], "swiglu", context=ep_context)
        out.backward(g_in)
        dx = x_in.grad
        x_in.requires_grad_(False)
        w1.grad = None
        w2.grad = None
        return out.detach(), dx

    def sync_all():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing ----
    for _ in range(max(args.warmup, 3)):
        step(x, grad_out)
    sync_all()
    tracer = Tracer(timing=not args.cuda_graph)
    _native.TRACER = tracer
    run_step = lambda: step(x, grad_out)
    launches_scale = 1
    if args.cuda_graph:
        # one captured forward+backward, replayed: removes the launch gaps that dominate small token counts
        if world != 1:
            raise SystemExit("--cuda-graph is a single-GPU option")
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            step(x, grad_out)
        launches_scale = args.steps      # the captured launches run once per replay
        run_step = graph.replay
        for _ in range(3):
            run_step()
        sync_all()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync_all()
    e0.record()
    for _ in range(args.steps):
        run_step()
    e1.record()
    sync_all()
    ms = e0.elapsed_time(e1) / args.steps
    launches = tracer.launches * launches_scale
    _native.TRACER = None
    clocks = sampler.stop() if rank == 0 else None

    # ---- correctness record of the timed configuration: status word + sampled tokens against the oracle ----
    out, dx = step(x, grad_out)
    torch.cuda.synchronize()
    status = torch.tensor([_native.read_status(device_status(device), reset=True)], device=device)
    weights = (w1, w2)
    if world > 1:
        dist.all_reduce(status, op=dist.ReduceOp.MAX)
        # every rank needs all experts for its own sampled tokens: gather the shards (position order = idx order)
        full = [torch.empty(w["E"], *t.shape[1:], dtype=t.dtype, device=device) for t in (w1, w2)]
        dist.all_gather_into_tensor(full[0], w1.detach())
        dist.all_gather_into_tensor(full[1], w2.detach())
        weights = full
    p_scores, p_idx = routing_of(x)
    parity = parity_record(x, out, dx, p_idx, p_scores, weights, grad_out, inp["router_weight"] if with_router else None)
    del weights
    if world > 1:
        full = None
        pt = torch.tensor([parity["out"], parity["dx"]], device=device)
        dist.all_reduce(pt, op=dist.ReduceOp.MAX)
        parity["out"], parity["dx"] = float(pt[0]), float(pt[1])
        parity["tokens_checked"] *= world
    parity["status"] = int(status.item())
    parity["tolerance"] = 2e-2
    torch.cuda.empty_cache()

    e2e = None
    if not args.device_only:
        e2e = run_e2e(args, step, x, grad_out, sync_all)
        e2e["cpu_binding"] = cpu_binding

    rows_per_rank = None
    if world > 1:
        t = torch.tensor([ms, e2e["ms"] if e2e is not None else 0.0], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t[0])
        if e2e is not None:
            e2e["ms"] = float(t[1])
        # routed rows each rank's experts received per step (same routing every step): sum over the chunk launches
        mine = [r for _, _, r in tracer.sections.get("mgrouped_gemm:glu", [])]
        rows = torch.tensor([float(sum(mine)) / args.steps], device=device)
        gathered = [torch.zeros_like(rows) for _ in range(world)]
        dist.all_gather(gathered, rows)
        rows_per_rank = [int(round(g.item())) for g in gathered]

    extras = {}
    if rank == 0 and world == 1 and not args.no_cpu_baseline and not args.device_only:
        extras["cpu_baseline"] = cpu_baseline(w, inp, budget_s=40.0)
    if world == 1 and not args.device_only and name == "mixtral_8x7b" and not args.tokens:
        del inp, w1, w2, x, grad_out, out, dx
        torch.cuda.empty_cache()
        if not args.no_scaling_base:
            # the expert-parallel workload on ONE GPU (all 256 experts local): the denominator for the N > 1 lines
            extras["ep_scaling_base"] = measure_single_gpu("deepseek_v3_ep", WORKLOADS["deepseek_v3_ep"], device, steps=20,
                                                           clocks=True, gather_in_gemm=gather_in_gemm)
        if not args.no_other_workloads:
            extras["other_workloads"] = other_workloads(device, gather_in_gemm)
            extras["forward_variants"] = [forward_variants(n, WORKLOADS[n], device)
                                          for n in ("qwen15_moe_a27b", "olmoe_8192")]
            extras["bmm_yardstick"] = [bmm_yardstick(n, WORKLOADS[n], device) for n in ("mixtral_8x7b", "olmoe_8192")]
            if args.csv:
                write_csv(args.csv, extras["other_workloads"])
        if not args.no_gpu_baseline:
            extras["gpu_baseline"] = gpu_baseline(name)
        inp = x = None

    if rank == 0:
        report(args, name, w, world, ms, e2e, launches, tracer, clocks, with_router, parity, rows_per_rank, extras)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if parity["status"] != 0 and parity["status"] != 4:
        raise SystemExit(f"device status word is {parity['status']} after the timed steps: results are not valid")
    if not (parity["out"] <= 2e-2 and parity["dx"] <= 2e-2):
        raise SystemExit(f"sampled tokens differ from the oracle beyond 2e-2: {parity}")


def run_e2e(args, step, x, grad_out, sync_all):
    """End to end: pinned host buffers in, results read back, every step; returns ms per step and, from CUDA events
    on the copy streams, the time the uploads and the read-backs took per step (they overlap the compute)."""
    hx = torch.empty(x.shape, dtype=x.dtype).pin_memory().copy_(x)
    hg = torch.empty(x.shape, dtype=x.dtype).pin_memory().copy_(grad_out)
    h_out = [torch.empty(x.shape, dtype=x.dtype).pin_memory() for _ in range(2)]
    h_dx = [torch.empty(x.shape, dtype=x.dtype).pin_memory() for _ in range(2)]
    dev_x = [torch.empty_like(x) for _ in range(2)]
    dev_g = [torch.empty_like(x) for _ in range(2)]
    copy_in, copy_out = torch.cuda.Stream(), torch.cuda.Stream()
    main = torch.cuda.current_stream()
    legs = {"h2d": [], "d2h": []}

    def timed_leg(kind, stream, fn):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        fn()
        b.record(stream)
        legs[kind].append((a, b))

    def upload(b):
        dev_x[b].copy_(hx, non_blocking=True)
        dev_g[b].copy_(hg, non_blocking=True)

    def e2e_loop(n):
        """Double-buffered: the upload of step i+1 and the read-back of step i-1 overlap step i's compute."""
        in_ready = [torch.cuda.Event(), torch.cuda.Event()]
        comp_done = [torch.cuda.Event(), torch.cuda.Event()]
        with torch.cuda.stream(copy_in):
            timed_leg("h2d", copy_in, lambda: upload(0))
            in_ready[0].record(copy_in)
        keep = []
        for i in range(n):
            b = i & 1
            if i + 1 < n:
                with torch.cuda.stream(copy_in):
                    if i >= 1:
                        copy_in.wait_event(comp_done[b ^ 1])  # buffer b^1 is free once step i-1 has computed
                    timed_leg("h2d", copy_in, lambda: upload(b ^ 1))
                    in_ready[b ^ 1].record(copy_in)
            main.wait_event(in_ready[b])
            out, dx = step(dev_x[b], dev_g[b])
            comp_done[b].record(main)
            keep.append((out, dx))
            with torch.cuda.stream(copy_out):
                copy_out.wait_event(comp_done[b])

                def download():
                    h_out[b].copy_(out, non_blocking=True)
                    h_dx[b].copy_(dx, non_blocking=True)

                timed_leg("d2h", copy_out, download)
            if len(keep) > 2:
                keep.pop(0)
        copy_out.synchronize()

    e2e_loop(3)
    sync_all()
    legs["h2d"].clear()
    legs["d2h"].clear()
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    e2e_loop(args.steps)
    t1.record()
    sync_all()
    leg_ms = {k_: sum(a.elapsed_time(b) for a, b in v) / max(len(v), 1) for k_, v in legs.items()}
    nbytes = 2 * x.numel() * x.element_size()
    return {"ms": t0.elapsed_time(t1) / args.steps, "h2d_ms": leg_ms["h2d"], "d2h_ms": leg_ms["d2h"],
            "h2d_gbs": nbytes / leg_ms["h2d"] / 1e6 if leg_ms["h2d"] > 0 else None,
            "d2h_gbs": nbytes / leg_ms["d2h"] / 1e6 if leg_ms["d2h"] > 0 else None}


def measure_single_gpu(name, w, device, steps, clocks=False, gather_in_gemm=None, cuda_graph=False):
    """Device-resident fwd+bwd of workload ``w`` on this GPU (logit-supplied routing): timed without any
    instrumentation, then a few more steps with per-kernel CUDA events for the dominant kernel's share."""
    from moe_explore import _native
    from moe_explore.expert_compute import expert_compute
    from moe_explore.routing_plan import build_routing_plan, check_device_status

    peaks = measured_peaks()
    inp = make_inputs(w, device)
    w1, w2 = inp["w1"].requires_grad_(), inp["w2"].requires_grad_()
    x, g, logits = inp["x"].requires_grad_(), inp["grad_out"], inp["logits"].requires_grad_()

    def one():
        scores, idx = scores_from_logits(logits, w["k"], x.dtype)
        plan = build_routing_plan(idx, w["E"], w["k"], want_perm=False)
        expert_compute(x, scores, w1, w2, plan, "swiglu", gather_in_gemm=gather_in_gemm).backward(g)
        x.grad = w1.grad = w2.grad = logits.grad = None

    for _ in range(3):
        one()
    torch.cuda.synchronize()
    run = one
    if cuda_graph:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            one()
        run = graph.replay
        run()
        torch.cuda.synchronize()
    sampler = ClockSampler(device.index)
    if clocks:
        sampler.start()
        time.sleep(0.2)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        run()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    rec = {"workload": name, "tokens": w["T"], "router": w["router"], "steps": steps, "ms_per_step": ms,
           "value": w["T"] / (ms * 1e-3), "unit": "tokens/s",
           "tflops": algorithmic_flops(w, w["T"], False) / (ms * 1e-3) / 1e12}
    rec["frac_bf16_peak"] = rec["tflops"] / peaks["burst"]
    if clocks:
        rec["clocks"] = sampler.stop()
    # dominant kernel (gate/up + SwiGLU) from CUDA-event brackets over a few extra steps
    tracer = Tracer()
    _native.TRACER = tracer
    extra = 5
    for _ in range(extra):
        one()
    torch.cuda.synchronize()
    _native.TRACER = None
    key = gate_up_key(tracer.sections)
    if key:
        durs = [a.elapsed_time(b) for a, b, _ in tracer.sections[key]]
        avg = sum(durs) / len(durs)
        ach = 4.0 * w["T"] * w["k"] * w["d"] * w["I"] / (avg * 1e-3) / 1e12
        rec["dominant_kernel"] = {"name": key, "avg_launch_ms": avg, "tflops": ach, "frac": ach / peaks["sustained"]}
    if clocks:
        rec["section_ms_per_step"] = tracer.ms_per_step(extra)
    rec["status"] = check_device_status(device)
    del inp, w1, w2, x, g, logits
    torch.cuda.empty_cache()
    return rec


def forward_variants(name, w, device, iters=10):
    """Inference forward (no gradient) of workload ``w`` three ways: the default (row copy, GEMMs, deterministic fold),
    with the fold fused into the down GEMM's epilogue (router weight x row added into the output by vector
    reductions), and with the row gather fused into the gate/up GEMM's operand loads; ms each and the largest
    deviation of the two fused forms from the default."""
    from moe_explore.expert_compute import expert_compute
    from moe_explore.routing_plan import build_routing_plan

    inp = make_inputs(w, device)
    x, w1, w2 = inp["x"], inp["w1"], inp["w2"]
    with torch.no_grad():
        scores, idx = scores_from_logits(inp["logits"], w["k"], x.dtype)
        plan = build_routing_plan(idx, w["E"], w["k"], want_perm=False)
        run = lambda **kw: expert_compute(x, scores, w1, w2, plan, "swiglu", **kw)
        base = run(gather_in_gemm=False)
        rec = {"workload": name, "tokens": w["T"], "forward_ms": event_ms(lambda: run(gather_in_gemm=False), iters)}
        fused = run(gather_in_gemm=False, fused_combine=True)
        rec["forward_fused_fold_ms"] = event_ms(lambda: run(gather_in_gemm=False, fused_combine=True), iters)
        rec["fused_fold_vs_default"] = float((fused.float() - base.float()).abs().max() / base.float().abs().max())
        gathered = run(gather_in_gemm=True)
        rec["forward_fused_gather_ms"] = event_ms(lambda: run(gather_in_gemm=True), iters)
        rec["fused_gather_equals_default"] = bool(torch.equal(gathered, base))
    del inp, x, w1, w2
    torch.cuda.empty_cache()
    return rec


def bmm_yardstick(name, w, device, iters=10):
    """The reference harness's yardstick (bench/bench_m_grouped_gemm.py:156-159): with perfectly balanced routing the
    ragged grouped GEMM is a batched GEMM, so ``torch.bmm`` (cuBLAS) on [E, R/E, K] x [E, K, N] bounds what a grouped
    kernel can reach.  Times the gate/up contraction (no activation) both ways on the same operands."""
    from moe_explore import _native
    from moe_explore.routing_plan import build_routing_plan
    from moe_explore.testing import perfect_routing

    T, d, E, k, I = w["T"], w["d"], w["E"], w["k"], w["I"]
    if (T * k) % (E * 128) != 0:
        return {"workload": name, "skipped": "rows per expert are not a multiple of the 128-row tile"}
    gen = torch.Generator(device=device).manual_seed(5)
    _, idx = perfect_routing(T, E, k, device, torch.bfloat16)
    plan = build_routing_plan(idx, E, k, want_perm=False)
    rows = T * k
    w1 = (torch.randn(E, d, 2 * I, generator=gen, device=device) * 0.02).bfloat16()
    xs = torch.zeros(plan.padded_rows, d, dtype=torch.bfloat16, device=device)
    xs[:rows] = torch.randn(rows, d, generator=gen, device=device).bfloat16()   # balanced: no padding inside experts
    out = torch.empty(plan.padded_rows, 2 * I, dtype=torch.bfloat16, device=device)
    ours = event_ms(lambda: _native.mgrouped_gemm(xs, w1, out, None, plan.mtile_expert, plan.tile_pairs, plan.num_mtiles,
                                                   False, None, plan.status), iters)
    a3 = xs[:rows].view(E, rows // E, d)
    ref = torch.bmm(a3, w1)
    same = bool(torch.equal(ref.view(rows, -1), out[:rows]))
    lib = event_ms(lambda: torch.bmm(a3, w1), iters)
    flops = 4.0 * rows * d * I
    rec = {"workload": name, "rows_per_expert": rows // E, "grouped_gemm_ms": ours, "grouped_gemm_tflops": flops / ours / 1e9,
           "torch_bmm_ms": lib, "torch_bmm_tflops": flops / lib / 1e9, "bit_identical": same}
    del w1, xs, out, ref
    torch.cuda.empty_cache()
    return rec


def other_workloads(device, gather_in_gemm):
    """The remaining single-GPU configurations, device-resident, 10 steps each: the Qwen1.5-MoE layer, the OLMoE layer
    at 8192 tokens and the routing-stress sweep (4 token counts x 3 router distributions; the two small token counts
    also as one captured CUDA graph, where launch gaps dominate)."""
    out = [measure_single_gpu("qwen15_moe_a27b", WORKLOADS["qwen15_moe_a27b"], device, 10, gather_in_gemm=gather_in_gemm)]
    for tokens in (128, 1024, 8192, 65536):
        for router_name in ("logits", "zipf15", "degenerate"):
            w = dict(WORKLOADS["olmoe_sweep"], T=tokens, router=router_name)
            rec = measure_single_gpu("olmoe_sweep", w, device, 10, gather_in_gemm=gather_in_gemm)
            if tokens <= 1024:
                graph = measure_single_gpu("olmoe_sweep", w, device, 10, gather_in_gemm=gather_in_gemm, cuda_graph=True)
                rec["ms_per_step_cuda_graph"] = graph["ms_per_step"]
            out.append(rec)
    return out


def write_csv(path, records):
    """The single-GPU workload table as CSV (one row per configuration), for plotting next to the reference's
    perf_report output."""
    import csv

    cols = ["workload", "tokens", "router", "ms_per_step", "ms_per_step_cuda_graph", "tflops", "frac_bf16_peak"]
    with open(path, "w", newline="") as f:
        out = csv.writer(f)
        out.writerow(cols)
        for r in records:
            out.writerow([r.get(c, "") for c in cols])


def gpu_baseline(name):
    """The reference's own Triton grouped GEMMs on this GPU (``--impl reference_triton`` in a child process, because
    its package has the same name as ours), when a checkout of the reference is present; else the reason."""
    ref = reference_checkout()
    if ref is None:
        return {"unavailable": "no checkout of arthurfeeney/moe-explore on this machine (MOE_EXPLORE_REFERENCE or "
                               "baseline/_ref): the reference's Triton kernels were not timed in this run"}
    cmd = [sys.executable, os.path.abspath(__file__), "--impl", "reference_triton", "--workload", name]
    try:
        r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=600,
                           env=dict(os.environ, MOE_EXPLORE_REFERENCE=ref))
        lines = [ln for ln in r.stdout.splitlines() if ln.startswith("{")]
        if r.returncode == 0 and lines:
            return json.loads(lines[-1])
        return {"unavailable": "the reference's Triton kernels did not run here: " + (r.stderr.strip().splitlines() or ["?"])[-1][:300]}
    except Exception as e:   # timeout and the like
        return {"unavailable": f"{type(e).__name__}: {e}"[:300]}


def reference_checkout():
    for cand in (os.environ.get("MOE_EXPLORE_REFERENCE"), os.path.join(ROOT, "baseline", "_ref")):
        if cand and os.path.isdir(os.path.join(cand, "src", "moe_explore")):
            return cand
    return None


def generic_gemm_case(args):
    """Seeded inputs of the stand-alone grouped-GEMM comparison: x, W1, W2, routing, and h (the down GEMM's input in
    (token, slot) order for the scatter call)."""
    name = args.workload or "mixtral_8x7b"
    w = dict(WORKLOADS[name])
    if args.tokens:
        w["T"] = args.tokens
    dev = torch.device("cuda", 0)
    T, d, E, k, I = w["T"], w["d"], w["E"], w["k"], w["I"]
    gen = torch.Generator(device=dev).manual_seed(0)
    x = torch.randn(T, d, generator=gen, device=dev).bfloat16()
    w1 = torch.empty(E, d, 2 * I, dtype=torch.bfloat16, device=dev)
    w2 = torch.empty(E, I, d, dtype=torch.bfloat16, device=dev)
    for e in range(E):
        w1[e] = (torch.randn(d, 2 * I, generator=gen, device=dev) * 0.02).bfloat16()
        w2[e] = (torch.randn(I, d, generator=gen, device=dev) * 0.02).bfloat16()
    if w["router"] == "linear":
        logits = (x @ (torch.randn(d, E, generator=gen, device=dev) * 0.02).bfloat16()).float()
    else:
        logits = make_logits(w, T, gen, dev)
    scores, idx = scores_from_logits(logits, k, x.dtype)
    h = torch.randn(T * k, I, generator=gen, device=dev).bfloat16()
    return name, w, x, w1, w2, scores, idx, h


def event_ms(fn, iters=10):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / iters


def run_generic_gemms(args):
    """The stand-alone ``m_grouped_gemm`` call with gather on W1 and with scatter on W2, without an activation, and
    ``get_token_indices``, at a benchmark shape -- on whichever package named ``moe_explore`` is first on sys.path:
    ``--impl reference_triton`` puts the reference's checkout there (the GPU baseline: its Triton kernels; with the
    Triton release installed here its activation epilogue does not compile -- epilogue_split.py assigns to a tuple
    item -- hence no activation), ``--impl ours_generic`` this repository's package."""
    impl = args.impl
    if impl == "reference_triton":
        ref = reference_checkout()
        if ref is None:
            print(json.dumps({"impl": impl, "unavailable": "no reference checkout"}))
            return
        sys.path.insert(0, os.path.join(ref, "src"))
    import moe_explore
    from moe_explore.expert_permute import get_token_indices
    from moe_explore.triton_kernels.m_grouped_gemm import MGroupedGEMMParams, m_grouped_gemm

    if impl == "reference_triton":
        assert os.path.abspath(ref) in os.path.abspath(moe_explore.__file__)
    name, w, x, w1, w2, scores, idx, h = generic_gemm_case(args)
    T, d, E, k, I = w["T"], w["d"], w["E"], w["k"], w["I"]
    rec = {"impl": impl, "workload": name, "tokens": T}
    with torch.no_grad():
        p = get_token_indices(idx, k, E, zero_prefix=True)
        gp = MGroupedGEMMParams(w1, p.group_indices, p.indices, gather=True, scatter=False, num_tokens=T, topk=k,
                                scales=None, activation=None)
        rec["gather_gemm_ms"] = event_ms(lambda: m_grouped_gemm(x, gp))
        rec["gather_gemm_tflops"] = 4.0 * T * k * d * I / rec["gather_gemm_ms"] / 1e9
        sp = MGroupedGEMMParams(w2, p.group_indices, p.indices, gather=False, scatter=True, num_tokens=T, topk=k,
                                scales=scores, activation=None)
        rec["scatter_gemm_ms"] = event_ms(lambda: m_grouped_gemm(h, sp))
        rec["scatter_gemm_tflops"] = 2.0 * T * k * d * I / rec["scatter_gemm_ms"] / 1e9
        rec["get_token_indices_ms"] = event_ms(lambda: get_token_indices(idx, k, E, zero_prefix=True))
    print(json.dumps(rec), flush=True)


def report(args, name, w, world, ms, e2e, launches, tracer, clocks, with_router, parity, rows_per_rank, extras):
    peaks = measured_peaks()
    tokens = w["T"] * world
    flops = algorithmic_flops(w, tokens, with_router)
    line = {
        "metric": METRIC, "value": tokens / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "tflops": flops / (ms * 1e-3) / 1e12,
        "frac_bf16_peak": flops / (ms * 1e-3) / 1e12 / world / peaks["burst"],
        "config": {"workload": name, "tokens_per_gpu": w["T"], "hidden": w["d"], "experts": w["E"], "topk": w["k"],
                   "intermediate": w["I"], "router": w["router"],
                   "parallelism": f"ep{world}-{args.ep_mode}" if world > 1 else "single",
                   "expert_placement": (args.placement + " (from the expert load of another seeded batch of the same "
                                        "router distribution)" if world > 1 and args.placement == "balanced"
                                        else (args.placement if world > 1 else None)),
                   "row_gather": "inside the gate/up and weight1-gradient GEMMs' operand loads (tile::gather4)"
                                 if args.gather_in_gemm == "on" and world == 1 else "separate copy kernel / peer pull",
                   "l2": "inputs larger than L2 (expert weights are re-read from HBM every step)",
                   "flops_per_step": flops},
        "clocks": clocks,
        "e2e": None if e2e is None else {
            "value": tokens / (e2e["ms"] * 1e-3), "unit": "tokens/s", "ms_per_step": e2e["ms"],
            "h2d_bytes_per_step": 2 * w["T"] * w["d"] * 2 * world,
            "d2h_bytes_per_step": 2 * w["T"] * w["d"] * 2 * world,
            "rank0_h2d_ms": e2e["h2d_ms"], "rank0_d2h_ms": e2e["d2h_ms"],
            "rank0_h2d_gbs": e2e["h2d_gbs"], "rank0_d2h_gbs": e2e["d2h_gbs"],
            "rank0_cpu_cores_bound_to_gpu": e2e.get("cpu_binding")},
        "gpu_launches": launches,
        "parity": parity,
    }
    if args.cuda_graph:
        line["config"]["cuda_graph"] = "one captured forward+backward step, replayed"
    if world > 1:
        line["config"]["ep_pull"] = args.ep_pull
        line["config"]["ep_slices"] = args.ep_slices + (" (pair ranges where one slice of whole experts would hold "
                                                        "more than 85 % of a rank's rows)" if args.ep_slices == "auto" else "")
    # roofline of the dominant kernel: the gate/up grouped GEMM (4*R*d*I FLOPs per launch)
    key = gate_up_key(tracer.sections)
    if key:
        torch.cuda.synchronize()
        dom = tracer.sections[key]
        durs = [a.elapsed_time(b) for a, b, _ in dom]
        avg = sum(durs) / len(durs)
        rows_local = sum(r for _, _, r in dom) / len(dom)  # routed rows one launch handled
        kflops = 4.0 * rows_local * w["d"] * w["I"]
        ach = kflops / (avg * 1e-3) / 1e12
        line["roofline"] = {"kernel": "grouped_gemm_kernel<gate/up, SwiGLU epilogue>" +
                                      (" with gathered A rows" if key.endswith("+gather") else ""),
                            "bound": "tensor",
                            "achieved": ach, "peak": peaks["sustained"], "unit": "TFLOP/s",
                            "frac": ach / peaks["sustained"], "peak_source": peaks["source"] + " (sustained)",
                            "frac_of_burst_peak": ach / peaks["burst"], "avg_launch_ms": avg,
                            "launches_timed": len(durs), "rows_per_launch": rows_local,
                            "traffic": TRAFFIC_BYTES.get(name) if not args.tokens else None}
    if rows_per_rank:
        mean = sum(rows_per_rank) / len(rows_per_rank)
        line["config"]["routed_rows_received_per_rank_per_step"] = rows_per_rank
        line["config"]["load_imbalance_max_over_mean"] = round(max(rows_per_rank) / mean, 4) if mean else None
    if tracer.sections:
        line["section_ms_per_step"] = tracer.ms_per_step(args.steps)
        for key in ("ep:wait_pull", "rows:gather_peer"):
            # per pipeline chunk (forward chunks, then backward chunks): where the GEMM stream waits for rows
            ev = tracer.sections.get(key)
            if ev and len(ev) % args.steps == 0:
                per = len(ev) // args.steps
                line.setdefault("per_chunk_ms", {})[key] = [
                    round(sum(ev[s_ * per + c][0].elapsed_time(ev[s_ * per + c][1]) for s_ in range(args.steps)) / args.steps, 3)
                    for c in range(per)]
    line.update(extras)
    print(json.dumps(line), flush=True)


# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) of one launch of the dominant kernel, from the
# ncu capture summarised under profiles/ (null where no capture has been taken for that workload).
TRAFFIC_BYTES = {"mixtral_8x7b": 3.6508e9 + 1.4292e9}


# ----------------------------------------------------------------------------------------------
# CPU baseline / reference arm: the oracle on the host cores
# ----------------------------------------------------------------------------------------------
def cpu_step(xs, scores, idx, w1, w2, grad):
    from oracle import moe_oracle as O

    for t in (xs, scores, w1, w2):
        t.grad = None
    out = O.expert_compute(xs, scores, idx, w1, w2, "swiglu")
    out.backward(grad)
    return out


def cpu_sample_inputs(w, inp, t_cpu):
    """First t_cpu tokens of the workload, same weights, upcast to fp32 on the host."""
    with torch.no_grad():
        x = inp["x"][:t_cpu].float().cpu()
        grad = inp["grad_out"][:t_cpu].float().cpu()
        if inp["router_weight"] is not None:
            logits = (inp["x"][:t_cpu] @ inp["router_weight"]).float().cpu()
        else:
            logits = inp["logits"][:t_cpu].float().cpu()
        top, idx = torch.topk(logits, w["k"], dim=-1, sorted=False)
        scores = torch.softmax(top, -1)
    return x.requires_grad_(), scores.requires_grad_(), idx, grad


def cpu_baseline(w, inp, budget_s):
    """Oracle forward+backward on the host, fp32, all threads, on a token sample grown to fill ~budget_s.

    The oracle's cost at few tokens is the per-expert weight-gradient products and their full-size outputs, which do
    not depend on the tokens; a sample of a few dozen tokens therefore understates the host's tokens/s many times
    over.  The sample is doubled, and timed again, while the measured passes predict that three more passes at twice
    the tokens still fit the budget."""
    torch.set_num_threads(os.cpu_count() or 1)
    w1 = inp["w1"].detach().float().cpu().requires_grad_()
    w2 = inp["w2"].detach().float().cpu().requires_grad_()
    started = time.perf_counter()
    t_cpu = min(64, w["T"])
    xs = cpu_sample_inputs(w, inp, t_cpu)
    cpu_step(xs[0], xs[1], xs[2], w1, w2, xs[3])      # first touch of the weight gradients
    growth = 1.5                                       # assumed cost ratio of a doubling until two sizes are measured
    last = None
    while True:
        t0 = time.perf_counter()
        cpu_step(xs[0], xs[1], xs[2], w1, w2, xs[3])
        probe = time.perf_counter() - t0
        if last is not None:
            growth = min(2.0, max(1.05, probe / last))
        last = probe
        spent = time.perf_counter() - started
        if t_cpu * 2 > min(w["T"], 4096) or spent + 3 * probe * growth > budget_s:
            break
        t_cpu *= 2
        xs = cpu_sample_inputs(w, inp, t_cpu)
    best = last
    t0 = time.perf_counter()
    cpu_step(xs[0], xs[1], xs[2], w1, w2, xs[3])
    best = min(best, time.perf_counter() - t0)
    return {"value": t_cpu / best, "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"first {t_cpu} of {w['T']} tokens, all {w['E']} experts' full-size weights, fp32, "
                      f"oracle forward+backward, best of 2 after warm-up ({best * 1e3:.0f} ms)"}


def run_reference(args):
    """The reference algorithm's CPU restatement, timed on the host cores (rank 0 only)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    world = args.gpus
    name = args.workload or ("mixtral_8x7b" if world == 1 else "deepseek_v3_ep")
    w = dict(WORKLOADS[name])
    torch.set_num_threads(os.cpu_count() or 1)
    torch.manual_seed(0)
    T, d, E, k, I = w["T"], w["d"], w["E"], w["k"], w["I"]
    # Per-step sample: a token subset against full-size fp32 weights of a subset of the experts.  The oracle's
    # cost is dominated by the per-expert weight-gradient products, so the number of experts is calibrated to
    # the time budget (and capped at 12 GB of weights); tokens are routed top-k among the sampled experts.
    e_full = E
    per_step_budget = 150.0 / (args.steps + args.warmup)
    e_cap = max(k, min(E, int(4e9 // (3 * d * I * 4))))   # at most ~4 GB of fp32 weights (and as much again of gradients)

    def make_weights(n):
        w1 = torch.empty(n, d, 2 * I)
        w2 = torch.empty(n, I, d)
        for e in range(n):
            w1[e].normal_(0, 0.02)
            w2[e].normal_(0, 0.02)
        return w1.requires_grad_(), w2.requires_grad_()

    def sample(t_cpu, n):
        x = torch.randn(t_cpu, d).requires_grad_()
        grad = torch.randn(t_cpu, d)
        top, idx = torch.topk(torch.randn(t_cpu, n), k, dim=-1, sorted=False)
        return x, torch.softmax(top, -1).requires_grad_(), idx, grad

    t_cpu = min(64, T)
    E = e_cap
    while True:
        w1, w2 = make_weights(E)
        xs = sample(t_cpu, E)
        cpu_step(xs[0], xs[1], xs[2], w1, w2, xs[3])          # first touch
        t0 = time.perf_counter()
        cpu_step(xs[0], xs[1], xs[2], w1, w2, xs[3])
        probe = time.perf_counter() - t0
        if probe <= per_step_budget or E <= k:
            break
        E = max(k, E // 2)                                    # too slow for the budget: fewer experts
    while t_cpu * 2 <= min(T, 4096) and probe * 2 < per_step_budget:
        t_cpu *= 2
        probe *= 1.3                                          # weight-gradient cost barely depends on the tokens
    xs = sample(t_cpu, E)
    for _ in range(args.warmup):
        cpu_step(xs[0], xs[1], xs[2], w1, w2, xs[3])
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_step(xs[0], xs[1], xs[2], w1, w2, xs[3])
    sec = (time.perf_counter() - t0) / args.steps
    value = t_cpu / sec
    sample_txt = (f"{t_cpu} of {T} tokens per step, full-size fp32 weights of {E} of the {e_full} experts "
                  f"(top-{k} routing among them), oracle forward+backward")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": name, "tokens_per_gpu": T, "hidden": d, "experts": e_full, "topk": k, "intermediate": I,
                   "router": w["router"], "sample_tokens_per_step": t_cpu, "sample_experts": E},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": "port",
                         "sample": sample_txt},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "reference_triton", "ours_generic"],
                    help="ours / reference: the two arms of the benchmark contract; reference_triton / ours_generic: the "
                         "stand-alone grouped-GEMM call on the reference's Triton kernels / on this library")
    ap.add_argument("--workload", default=None, choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-scaling-base", action="store_true",
                    help="N = 1: skip the extra measurement of the expert-parallel workload on one GPU")
    ap.add_argument("--no-other-workloads", action="store_true",
                    help="N = 1: skip the Qwen1.5-MoE / OLMoE / routing-stress-sweep measurements")
    ap.add_argument("--csv", default=None, help="N = 1: also write the other-workloads table to this CSV file")
    ap.add_argument("--no-gpu-baseline", action="store_true",
                    help="N = 1: skip timing the reference's Triton kernels (needs a checkout of the reference)")
    ap.add_argument("--gather-in-gemm", default="auto", choices=["auto", "on", "off"],
                    help="single GPU: token rows gathered by the GEMMs' operand loads (auto = the package default) or "
                         "copied into the expert-sorted layout first")
    ap.add_argument("--ep-pull", default="ldst", choices=["bulk", "ldst", "dedicated", "dma"],
                    help="N > 1, peer mode: pull rows with the copy-engine kernel on the reserved SMs or with the "
                         "load/store kernel on all SMs")
    ap.add_argument("--ep-reserved-sms", type=int, default=None,
                    help="N > 1, peer mode: SMs the GEMMs leave to the pull kernels (default 8)")
    ap.add_argument("--placement", default="balanced", choices=["balanced", "contiguous"],
                    help="N > 1: which experts each rank owns: evened out by measured load (default) or blocks of E/N")
    ap.add_argument("--ep-chunks", type=int, default=None,
                    help="N > 1, peer mode: slices of the local expert list the dispatch pull is pipelined in")
    ap.add_argument("--no-cpu-binding", action="store_true",
                    help="N > 1: do not restrict each rank to the CPU cores local to its GPU")
    ap.add_argument("--ep-slices", default="auto", choices=["auto", "pairs", "experts"],
                    help="N > 1, peer mode: pipeline slices cut in the list of row-tile pairs (a slice may end inside an "
                         "expert), made of whole experts, or (default) the former only where one expert holds most of a "
                         "rank's rows")
    ap.add_argument("--ep-mode", default="peer", choices=["peer", "collective"],
                    help="N > 1: rows over peer-mapped memory inside the kernels (default) or NCCL all-to-all")
    ap.add_argument("--router", default=None, choices=["logits", "logits_bias", "zipf", "zipf15", "degenerate"],
                    help="override the router distribution of a logit-supplied workload")
    ap.add_argument("--tokens", type=int, default=None, help="override tokens per GPU (profiling a smaller case)")
    ap.add_argument("--cuda-graph", action="store_true",
                    help="capture one forward+backward step in a CUDA graph and time replays (one GPU, device-resident)")
    ap.add_argument("--device-only", action="store_true",
                    help="skip the end-to-end and CPU-baseline legs (for short runs under a profiler)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.impl in ("reference_triton", "ours_generic"):
        run_generic_gemms(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
