"""Benchmark of the MoE data-parallel hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload moe|lans]

Workload "moe" (default, the configuration the headline metric is quoted on): per GPU S=16384
tokens, M=2048, fp16 tokens, fp32 gate probabilities, E=2*N experts, top-2, capacity factor 1.25,
dispatch in 4 chained chunks + exchange + combine.  A step is one pass over one batch of seeded
synthetic tokens.  One JSON line is printed by rank 0.
"""
import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402
import torch  # noqa: E402

S_TOKENS, M_DIM, TOP_K, CAP_FACTOR, N_CHUNKS = 16384, 2048, 2, 1.25, 4
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return d, "measured"
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the benchmark runs."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.tmp = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(gpu_index), "--query-gpu=" + self.FIELDS + ",timestamp",
                 "--format=csv,noheader,nounits", "-lms", "100"], stdout=self.tmp, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        self.tmp.flush()
        self.tmp.seek(0)
        rows = [r.strip().split(", ") for r in self.tmp.read().splitlines() if r.strip()]
        self.tmp.close()
        os.unlink(self.tmp.name)
        return rows

    @staticmethod
    def summarise(rows):
        sm, mx, reasons = [], [], set()
        for r in rows:
            try:
                clk, cmax = float(r[1]), float(r[2])
            except (ValueError, IndexError):
                continue
            sm.append(clk)
            mx.append(cmax)
            for name, col in (("hw_slowdown", 5), ("hw_thermal_slowdown", 6), ("sw_thermal_slowdown", 7),
                              ("sw_power_cap", 8)):
                if len(r) > col and r[col].strip().lower() == "active":
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        # under load = the upper half of the samples (idle samples before/after the region are low)
        hi = sorted(sm)[len(sm) // 2:]
        return {"sm_mhz": statistics.median(hi), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm)}


def synth_inputs(rank, world, S, M, dtype, device=None, sets=2):
    """Seeded synthetic tokens ~N(0,1) and softmax(N(0,1) logits) gate probabilities, seed 1000+rank."""
    E = 2 * world
    xs, gates = [], []
    for i in range(sets):
        g = torch.Generator().manual_seed(1000 + rank + 7919 * i)
        logits = torch.randn(S, E, generator=g)
        gates.append(torch.softmax(logits, dim=1))
        xs.append(torch.randn(S, M, generator=g).to(dtype))
    return xs, gates


def cpu_reference_sample(max_seconds, world=1, tokens=None):
    """Times the restatement of the reference's torch-CPU operators (per-token loops) on a sample
    of the workload; returns (tokens_per_s, cores, description, seconds)."""
    from oracle import moe_oracle as O
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    E = 2 * world
    # probe speed on 256 tokens, then size the sample
    def run(S):
        xs, gates = synth_inputs(0, world, S, M_DIM, torch.float16, sets=1)
        x, gate = xs[0].numpy(), gates[0].numpy()
        C = O.capacity(S, E, CAP_FACTOR, TOP_K)
        t0 = time.perf_counter()
        gs, il, cap, el, disp = O.loops_encode(x, gate, np.zeros(E, np.int32), C, TOP_K)
        out = O.loops_decode(disp, gs, il)
        dt = time.perf_counter() - t0
        return dt, float(np.abs(out.astype(np.float32)).sum())
    if tokens is None:
        dt, _ = run(256)
        tokens = int(min(S_TOKENS, max(256, 256 * (max_seconds / max(dt, 1e-6)))))
        tokens = max(256, tokens // 256 * 256)
    dt, _ = run(tokens)
    return tokens / dt, cores, "%d of %d tokens/GPU, M=%d, E=%d, top-%d, encode+decode with per-token loops" % (
        tokens, S_TOKENS, M_DIM, E, TOP_K) + " (torch CPU ops on %d threads, the loops are single-threaded Python)" % cores, dt, tokens


def run_reference_arm(args):
    """--impl reference: the reference's CPU implementation of the path (restated port; the reference
    itself has no CPU operator that builds without TVM) on the host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    world = args.gpus
    budget = 100.0 / max(1, args.steps + args.warmup)
    rate, cores, sample, dt, tokens = cpu_reference_sample(min(20.0, budget), world)
    for _ in range(max(0, args.warmup - 1)):
        cpu_reference_sample(0, world, tokens)
    times = []
    for _ in range(args.steps):
        r = cpu_reference_sample(0, world, tokens)
        times.append(r[3])
    ms = 1e3 * sum(times) / len(times)
    value = tokens / (ms / 1e3)
    line = {
        "impl": "reference", "metric": "moe_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": moe_config(world),
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit(line)


def moe_config(world):
    return {"workload": "moe_dispatch_a2a_combine: S=%d tokens/GPU, M=%d fp16, E=%d, top-%d, cf=%.2f, %d chunks" % (
        S_TOKENS, M_DIM, 2 * world, TOP_K, CAP_FACTOR, N_CHUNKS),
        "tokens_per_gpu": S_TOKENS, "model_dim": M_DIM, "experts": 2 * world, "top_k": TOP_K,
        "capacity_factor": CAP_FACTOR, "chunks": N_CHUNKS,
        "l2": "inputs rotate over 2 sets; 288 MiB touched per step exceeds the 126 MB L2"}


def run_moe(args):
    import lancet_b200 as LB
    from lancet_b200 import _capi
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit("bench.py: --gpus %d but WORLD_SIZE=%d (launch with torch.distributed.run for N>1)" % (
            args.gpus, world))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    L = _capi.lib()
    E = 2 * world
    xs_h, gates_h = synth_inputs(rank, world, S_TOKENS, M_DIM, torch.float16)
    xs = [x.to(dev) for x in xs_h]
    gates = [g.to(dev) for g in gates_h]
    if world == 1:
        plan = LB.ChunkedMoE(S_TOKENS, M_DIM, E, TOP_K, CAP_FACTOR, N_CHUNKS, torch.float16, device=dev)
    else:
        plan = LB.DistChunkedMoE(S_TOKENS, M_DIM, TOP_K, CAP_FACTOR, N_CHUNKS, torch.float16, device=dev)

    def step(i):
        # world > 1: the exchange is fused into both kernels (peer stores / peer loads) and the ranks
        # meet at a flag barrier between them; the experts are the identity for this metric
        plan.dispatch(xs[i % 2], gates[i % 2])
        return plan.combine()

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            import torch.distributed as dist
            dist.barrier()
            torch.cuda.synchronize()

    sampler = ClockSampler(local_rank) if rank == 0 else None
    for i in range(max(args.warmup, 3)):
        step(i)
    sync_all()
    kname = b"dispatch_rows_kernel" if world == 1 else b"dispatch_rows_peer_kernel"
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    use_graph = not args.no_graph
    if use_graph:
        # the step is a handful of short launches: replay it from a CUDA graph (one per input set; the receive
        # buffers of the multi-GPU plan alternate with the same period) to cut launch gaps
        graphs = []
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for i in range(2):
                gph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(gph, stream=side):
                    step(i)
                graphs.append(gph)
        torch.cuda.current_stream().wait_stream(side)
        launches_per_step = None
        for i in range(4):
            graphs[i % 2].replay()
        sync_all()
    # ---- timed region: K steps, device resident inputs ------------------------------------------
    launches0 = L.lancet_launch_count()
    if use_graph:
        ev0.record()
        for i in range(args.steps):
            graphs[i % 2].replay()
        ev1.record()
        sync_all()
        ms_total = ev0.elapsed_time(ev1)
        # per-kernel durations: the same steps launched eagerly right after, bracketed by events in the library
        L.lancet_profile_begin(kname)
        for i in range(min(args.steps, 200)):
            step(i)
        sync_all()
        launches = (L.lancet_launch_count() - launches0) // max(1, min(args.steps, 200)) * args.steps
    else:
        L.lancet_profile_begin(kname)
        ev0.record()
        for i in range(args.steps):
            step(i)
        ev1.record()
        sync_all()
        ms_total = ev0.elapsed_time(ev1)
        launches = L.lancet_launch_count() - launches0
    k_ms, k_n = ctypes.c_double(0), ctypes.c_longlong(0)
    _capi.check(L.lancet_profile_end(ctypes.byref(k_ms), ctypes.byref(k_n)))
    if world > 1:
        import torch.distributed as dist
        t = torch.tensor([ms_total], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total = float(t.item())
    ms_step = ms_total / args.steps
    value = S_TOKENS * world / (ms_step / 1e3)

    # ---- end to end: pinned host inputs in, combined output back, every step ---------------------
    # Three streams, double-buffered device tensors: the host->device copy of step i+1 and the device->host copy
    # of step i-1 run while step i computes (PCIe is full duplex), as a data loader with prefetch would do.
    e2e_steps = max(3, min(args.steps, 50))
    x_pin = [x.pin_memory() for x in xs_h]
    g_pin = [g.pin_memory() for g in gates_h]
    out_pin = [torch.empty((S_TOKENS, M_DIM), dtype=torch.float16).pin_memory() for _ in range(2)]
    x_dev = [torch.empty_like(xs[0]) for _ in range(2)]
    g_dev = [torch.empty_like(gates[0]) for _ in range(2)]
    out_dev = [torch.empty((S_TOKENS, M_DIM), dtype=torch.float16, device=dev) for _ in range(2)]
    s_comp = torch.cuda.current_stream()
    s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_comp = [torch.cuda.Event() for _ in range(2)]
    ev_outd = [torch.cuda.Event() for _ in range(2)]

    def e2e_step(i):
        b = i % 2
        with torch.cuda.stream(s_in):
            if i >= 2:
                s_in.wait_event(ev_comp[b])          # step i-2 has finished reading x_dev[b]
            x_dev[b].copy_(x_pin[b], non_blocking=True)
            g_dev[b].copy_(g_pin[b], non_blocking=True)
            ev_in[b].record(s_in)
        s_comp.wait_event(ev_in[b])
        if i >= 2:
            s_comp.wait_event(ev_outd[b])            # step i-2's result has left out_dev[b]
        plan.dispatch(x_dev[b], g_dev[b])
        plan.combine(out=out_dev[b])
        ev_comp[b].record(s_comp)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_comp[b])
            out_pin[b].copy_(out_dev[b], non_blocking=True)
            ev_outd[b].record(s_out)

    def e2e_join():
        s_comp.wait_stream(s_in)
        s_comp.wait_stream(s_out)

    for i in range(4):
        e2e_step(i)
    e2e_join()
    sync_all()
    ev0.record()
    for i in range(e2e_steps):
        e2e_step(i)
    e2e_join()
    ev1.record()
    sync_all()
    e2e_ms = ev0.elapsed_time(ev1)
    if world > 1:
        import torch.distributed as dist
        t = torch.tensor([e2e_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    e2e_value = S_TOKENS * world / (e2e_ms / e2e_steps / 1e3)
    clocks = ClockSampler.summarise(sampler.stop()) if sampler else None
    if world > 1:
        plan.check()
        cap_all = plan.capused.cpu().numpy()
        import torch.distributed as dist
        dist.barrier()
        plan.close()
        dist.destroy_process_group()
    if rank != 0:
        return
    # ---- roofline of the dominant kernel (dispatch scatter) ---------------------------------------
    peaks, peak_kind = load_peaks()
    hbm_peak = float(peaks.get("hbm_gbs", FALLBACK_PEAKS["hbm_gbs"]))
    cap = plan.capused.cpu().numpy() if world == 1 else cap_all
    kept_rows = int(cap[-1].sum())                      # rows written by the 4 dispatch launches of a step
    row_bytes = M_DIM * 2
    # algorithmic bytes of the dispatch launch (all chunks in one launch): token rows read once, the
    # whole padded [E,C,M] buffer written once (kept rows + zero rows)
    bytes_per_launch = S_TOKENS * row_bytes + E * plan.C * row_bytes
    roof = None
    if k_n.value > 0:
        avg_s = k_ms.value / k_n.value / 1e3
        achieved = bytes_per_launch / avg_s / 1e9
        roof = {"bound": "hbm", "kernel": kname.decode(), "achieved": achieved, "peak": hbm_peak, "unit": "GB/s",
                "frac": achieved / hbm_peak, "peak_kind": peak_kind, "traffic": None,
                "bytes_per_launch": bytes_per_launch, "avg_launch_us": avg_s * 1e6, "launches_timed": k_n.value}
        if world > 1:
            # the fused dispatch is bound by the bytes that leave this GPU over NVLink: (W-1)/W of the
            # padded expert buffer; peak = the pool's measured peer-copy bandwidth per direction
            remote_rows = int(cap[-1][plan.LE:].sum())          # rank 0 owns experts [0, LE): the rest crosses NVLink
            nv_bytes = remote_rows * row_bytes
            nv = nv_bytes / avg_s / 1e9
            roof.update({"bound": "nvlink", "achieved": nv, "peak": 770.0, "frac": nv / 770.0,
                         "peak_kind": "measured peer copy, per direction", "bytes_per_launch": nv_bytes,
                         "hbm_achieved": achieved})
        if world == 1:
            # dram read + write bytes per launch from the ncu capture of this workload
            # (profiles/moe_dispatch_combine_S16384_M2048_ncu_full.txt)
            roof["traffic"] = 177.2e6
    line = {
        "metric": "moe_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16", "data": "synthetic", "config": moe_config(world),
        "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": S_TOKENS * row_bytes + S_TOKENS * E * 4,
                "d2h_bytes_per_step": S_TOKENS * row_bytes, "steps": e2e_steps},
        "gpu_launches": int(launches), "clocks": clocks, "roofline": roof,
        "launch_mode": "cuda graph replay (kernel durations from an eager loop of the same steps)" if use_graph else "eager",
        "step_bytes": {"dispatch_read": S_TOKENS * row_bytes, "dispatch_write": E * plan.C * row_bytes,
                       "combine_read": kept_rows * row_bytes, "combine_write": S_TOKENS * row_bytes},
    }
    step_bytes = sum(line["step_bytes"].values())
    line["step_hbm_frac"] = step_bytes / (ms_step / 1e3) / 1e9 / hbm_peak
    if world == 1 and not args.no_cpu:
        rate, cores, sample, _, _ = cpu_reference_sample(15.0, 1)
        line["cpu_baseline"] = {"value": rate, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample}
    emit(line)


def lans_shapes(layers=24):
    """196 fp32 tensors, 354.6 M elements: GPT-2-medium-like (24 layers x 8 tensors + embeddings + final norm)."""
    shapes = [(50257, 1024), (1024, 1024)]
    for _ in range(layers):
        shapes += [(1024, 1024), (1024, 1024), (1024, 1024), (1024, 1024), (4096, 1024), (1024, 4096), (1024,), (1024,)]
    shapes += [(1024,), (1024,)]
    return shapes


def run_lans(args):
    import lancet_b200 as LB
    from lancet_b200 import _capi
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    L = _capi.lib()
    shapes = lans_shapes(args.lans_layers)
    g = torch.Generator(device=dev).manual_seed(0)
    P = [torch.randn(s, device=dev, generator=g) * 0.02 for s in shapes]
    G = [torch.randn(s, device=dev, generator=g) * 1e-3 for s in shapes]
    Mo = [torch.randn(s, device=dev, generator=g) * 1e-4 for s in shapes]
    V = [torch.rand(s, device=dev, generator=g) * 1e-6 for s in shapes]
    tl = G + P + Mo + V
    n_el = sum(p.numel() for p in P)
    state = LB.LansState(G, P, Mo, V)
    sampler = ClockSampler(dev.index)
    for i in range(max(args.warmup, 3)):
        LB.lans(tl, 10 + i, state=state)
    torch.cuda.synchronize()
    L.lancet_profile_begin(b"lans_phase2_kernel")
    l0 = L.lancet_launch_count()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for i in range(args.steps):
        LB.lans(tl, 20 + i, state=state)
    ev1.record()
    torch.cuda.synchronize()
    ms = ev0.elapsed_time(ev1) / args.steps
    launches = L.lancet_launch_count() - l0
    k_ms, k_n = ctypes.c_double(0), ctypes.c_longlong(0)
    _capi.check(L.lancet_profile_end(ctypes.byref(k_ms), ctypes.byref(k_n)))
    clocks = ClockSampler.summarise(sampler.stop())
    peaks, peak_kind = load_peaks()
    hbm_peak = float(peaks.get("hbm_gbs", FALLBACK_PEAKS["hbm_gbs"]))
    avg_s = k_ms.value / max(1, k_n.value) / 1e3
    achieved = 24.0 * n_el / avg_s / 1e9
    line = {
        "metric": "lans_elements_per_s", "value": n_el / (ms / 1e3), "unit": "elements/s", "n_gpus": 1,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "lans_step: %d fp32 tensors, %d elements" % (len(shapes), n_el),
                   "l2": "5.6 GB of state per step exceeds the 126 MB L2"},
        "gpu_launches": int(launches), "clocks": clocks,
        "roofline": {"bound": "hbm", "kernel": "lans_phase2_kernel", "achieved": achieved, "peak": hbm_peak,
                     "unit": "GB/s", "frac": achieved / hbm_peak, "peak_kind": peak_kind,
                     # 23.46 B/element measured by ncu on a 77.7 M-element list, scaled by the element count
                     # (profiles/lans_phase_kernels_77M_elements_ncu_full.txt)
                     "traffic": 23.46 * n_el,
                     "bytes_per_launch": 24.0 * n_el, "avg_launch_us": avg_s * 1e6},
        "step_hbm_frac": 52.0 * n_el / (ms / 1e3) / 1e9 / hbm_peak,
    }
    emit(line)


def run_ffn(args):
    """Expert FFN forward (config 'expert FFN grouped GEMM'): per GPU 2 local experts, rows from 8 source
    ranks x C=2560, M=2048, H=8192, bf16 with fp32 accumulation: GEMM1 + bias + GELU, GEMM2 + bias."""
    import lancet_b200 as LB
    from lancet_b200 import _capi
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    L = _capi.lib()
    G, LE, C, M, H = 8, 2, 2560, 2048, 8192
    g = torch.Generator(device=dev).manual_seed(0)
    x = torch.randn((G * LE, C, M), device=dev, generator=g).bfloat16()
    w1 = (torch.randn((LE, H, M), device=dev, generator=g) * 0.02).bfloat16()
    w2 = (torch.randn((LE, M, H), device=dev, generator=g) * 0.02).bfloat16()
    b1 = torch.zeros((LE, H), device=dev).bfloat16()
    b2 = torch.zeros((LE, M), device=dev).bfloat16()
    h = torch.empty((G * LE, C, H), device=dev, dtype=torch.bfloat16)
    y = torch.empty((G * LE, C, M), device=dev, dtype=torch.bfloat16)

    def step():
        LB.grouped_gemm_nt(x, w1, bias=b1, act="gelu", out=h)
        LB.grouped_gemm_nt(h, w2, bias=b2, out=y)

    sampler = ClockSampler(dev.index)
    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    L.lancet_profile_begin(b"grouped_gemm_nt_kernel")
    l0 = L.lancet_launch_count()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(args.steps):
        step()
    ev1.record()
    torch.cuda.synchronize()
    ms = ev0.elapsed_time(ev1) / args.steps
    launches = L.lancet_launch_count() - l0
    k_ms, k_n = ctypes.c_double(0), ctypes.c_longlong(0)
    _capi.check(L.lancet_profile_end(ctypes.byref(k_ms), ctypes.byref(k_n)))
    st = LB.gemm_status(dev)
    _capi.check(L.lancet_p2p_status(ctypes.c_void_p(st.data_ptr()), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)))
    # backward GEMMs of the same layer: dH = (dY W2) * gelu'(H_pre), dW2 = dY^T H, dX = dH W1, dW1 = dH^T X
    hpre = torch.empty_like(h)
    LB.grouped_gemm_nt(x, w1, bias=b1, act="gelu", out=h, preact=hpre)
    dy = torch.randn((G * LE, C, M), device=dev, generator=g).bfloat16()
    dh, dx = torch.empty_like(h), torch.empty_like(x)
    dw1, dw2 = torch.empty_like(w1), torch.empty_like(w2)

    def bwd_step():
        LB.grouped_gemm_nn(dy, w2, act="gelu", preact=hpre, out=dh)       # w2 is [LE, M, H]: contraction over M
        LB.grouped_gemm_tn(dy, h, LE, out=dw2)                            # [LE, M, H]
        LB.grouped_gemm_nn(dh, w1, out=dx)                                # w1 is [LE, H, M]: contraction over H
        LB.grouped_gemm_tn(dh, x, LE, out=dw1)                            # [LE, H, M]

    for _ in range(3):
        bwd_step()
    torch.cuda.synchronize()
    bsteps = max(3, min(args.steps, 20))
    ev0.record()
    for _ in range(bsteps):
        bwd_step()
    ev1.record()
    torch.cuda.synchronize()
    bwd_ms = ev0.elapsed_time(ev1) / bsteps
    _capi.check(L.lancet_p2p_status(ctypes.c_void_p(st.data_ptr()), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)))
    # same-box bar: the library GEMM the reference calls (cuBLAS through torch.matmul), same shapes
    xs = x.view(G, LE, C, M)
    def lib_step():
        for e in range(LE):
            a = xs[:, e].reshape(G * C, M)
            hh = torch.nn.functional.gelu(torch.addmm(b1[e], a, w1[e].t()))
            torch.addmm(b2[e], hh, w2[e].t())
    for _ in range(3):
        lib_step()
    torch.cuda.synchronize()
    ev0.record()
    lib_steps = max(3, min(args.steps, 20))
    for _ in range(lib_steps):
        lib_step()
    ev1.record()
    torch.cuda.synchronize()
    lib_ms = ev0.elapsed_time(ev1) / lib_steps
    clocks = ClockSampler.summarise(sampler.stop())
    peaks, peak_kind = load_peaks()
    flops = 2.0 * (G * LE * C) * M * H * 2
    sustained = float(peaks.get("bf16_tflops_sustained", peaks.get("bf16_tflops", FALLBACK_PEAKS["bf16_tflops"])))
    avg_s = k_ms.value / max(1, k_n.value) / 1e3
    ach = flops / 2 / avg_s / 1e12
    tokens = G * LE * C
    emit({
        "metric": "expert_ffn_rows_per_s", "value": tokens / (ms / 1e3), "unit": "rows/s", "n_gpus": 1, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "expert_ffn_forward: 16 groups x 2560 rows, M=2048, H=8192, 2 local experts, bias+GELU",
                   "l2": "1.2 GB touched per step exceeds the 126 MB L2"},
        "gpu_launches": int(launches), "clocks": clocks, "tflops": flops / (ms / 1e3) / 1e12,
        "backward": {"ms_per_step": bwd_ms, "tflops": 2.0 * flops / (bwd_ms / 1e3) / 1e12,
                     "what": "dH (NN, fused gelu'), dW2 (TN), dX (NN), dW1 (TN)"},
        "library_gemm": {"ms_per_step": lib_ms, "tflops": flops / (lib_ms / 1e3) / 1e12, "what": "torch.addmm + gelu (cuBLAS)"},
        "roofline": {"bound": "tensor", "kernel": "grouped_gemm_nt_kernel", "achieved": ach, "peak": sustained,
                     "unit": "TFLOP/s", "frac": ach / sustained, "peak_kind": peak_kind + " (sustained cuBLAS bf16)",
                     "traffic": None, "flops_per_launch": flops / 2, "avg_launch_us": avg_s * 1e6},
    })


def run_layer(args):
    """Whole MoE layer, forward + backward: gate probabilities in, dispatch (+exchange), expert FFN (M=2048,
    H=8192, GELU, 2 local experts), combine (+exchange); backward with the weight-gradient GEMMs on a side stream
    under the returning exchange.  S=16384 tokens per GPU, top-2, capacity factor 1.25, bf16."""
    import lancet_b200 as LB
    from lancet_b200 import _capi
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit("bench.py: --gpus %d but WORLD_SIZE=%d" % (args.gpus, world))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    fabric = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    else:
        fabric = LB.LocalFabric(1, 0, {})
    H = 8192
    xs_h, gates_h = synth_inputs(rank, world, S_TOKENS, M_DIM, torch.bfloat16)
    xs = [x.to(dev) for x in xs_h]
    gates = [g.to(dev) for g in gates_h]
    dout = torch.randn((S_TOKENS, M_DIM), device=dev).bfloat16()
    layer = LB.MoELayer(S_TOKENS, M_DIM, H, TOP_K, CAP_FACTOR, N_CHUNKS, torch.bfloat16, dev, 2, fabric=fabric, overlap_dw=True,
                        stages=args.stages)
    side = layer.side
    results = {}

    mode = {"v": "pipelined"}

    def step(i):
        if mode["v"] == "pipelined":
            layer.forward_pipelined(xs[i % 2], gates[i % 2])
            layer.backward_pipelined(dout)
        else:
            layer.forward(xs[i % 2], gates[i % 2])
            layer.backward(dout)

    # the three schedules take turns in short bursts, so that clock drift under the power cap hits them alike
    order = {"all": ("pipelined", True, False), "staged": ("pipelined",), "side": (True,), "single": (False,)}[args.schedule]
    rounds = 5 if args.steps >= 5 else 1
    per_round = max(args.steps // rounds, 1)
    results = {m: 0.0 for m in order}
    for i in range(max(args.warmup, 3)):
        for m in order:
            mode["v"] = m
            layer.side = side if m is True else None
            step(i)
    for rnd in range(rounds):
        for m in order:
            mode["v"] = m
            layer.side = side if m is True else None
            step(0)
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            ev0.record()
            for i in range(per_round):
                step(i)
            ev1.record()
            torch.cuda.synchronize()
            ms = ev0.elapsed_time(ev1) / per_round
            if world > 1:
                t = torch.tensor([ms], device=dev, dtype=torch.float64)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ms = float(t.item())
            results[m] += ms / rounds
    if world > 1:
        layer.moe.check()
    live = int(layer.moe.capused[-1].sum().item())
    st = LB.gemm_status(dev)
    _capi.check(_capi.lib().lancet_p2p_status(ctypes.c_void_p(st.data_ptr()),
                                              ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)))
    if world > 1:
        dist.barrier()
        layer.moe.close()
        dist.destroy_process_group()
    if rank != 0:
        return
    ms = min(results.values())
    flops = 6.0 * 2.0 * live * M_DIM * H            # per GPU: 2 GEMMs forward, 4 backward, live rows only
    peaks, peak_kind = load_peaks()
    sustained = float(peaks.get("bf16_tflops_sustained", FALLBACK_PEAKS["bf16_tflops"]))
    emit({
        "metric": "moe_layer_tokens_per_s", "value": S_TOKENS * world / (ms / 1e3), "unit": "tokens/s", "n_gpus": world,
        "steps": per_round * rounds, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "moe_layer_fwd_bwd: S=%d tokens/GPU, M=%d, H=%d, E=%d, top-%d, cf=%.2f, %d chunks" % (
            S_TOKENS, M_DIM, H, 2 * world, TOP_K, CAP_FACTOR, N_CHUNKS), "l2": "GBs touched per step exceed the 126 MB L2"},
        "tflops_per_gpu": flops / (ms / 1e3) / 1e12, "tensor_frac": flops / (ms / 1e3) / 1e12 / sustained,
        "peak_kind": peak_kind + " (sustained cuBLAS bf16)", "live_rows_rank0": live,
        "schedules": {"pipeline_stages": args.stages, "ms_pipelined_exchange": results.get("pipelined"),
                      "ms_dw_on_side_stream": results.get(True), "ms_single_stream": results.get(False)},
    })


def run_a2a(args):
    """Stand-alone `_all_to_all` of the [E,C,M] expert buffer of the MoE workload (160 MiB per GPU): NCCL grouped
    send/recv exactly as the reference issues it, and the peer-memory store kernel + flag barrier."""
    import lancet_b200 as LB
    import torch.distributed as dist
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus or world < 2:
        raise SystemExit("bench.py --workload a2a needs --gpus N >= 2 under torch.distributed.run")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist.init_process_group("nccl", device_id=dev)
    E = 2 * world
    C = LB.moe_capacity(S_TOKENS // N_CHUNKS, E, CAP_FACTOR * N_CHUNKS, TOP_K)
    x = torch.randn((E, C, M_DIM), device=dev).half()
    nbytes = x.numel() * 2
    comm = LB.Communicator(dev)
    sa = LB.SymmAllToAll(nbytes, dev)
    res = {}

    def timed(fn):
        for _ in range(max(args.warmup, 3)):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        for _ in range(args.steps):
            fn()
        ev1.record()
        torch.cuda.synchronize()
        t = torch.tensor([ev0.elapsed_time(ev1) / args.steps], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    out = torch.empty_like(x)
    res["nccl"] = timed(lambda: comm.all_to_all(x, out=out))
    res["peer"] = timed(lambda: sa.all_to_all(x))
    ok = bool(torch.equal(sa.recv_view(x), comm.all_to_all(x)))
    sa.check()
    comm.close()
    dist.barrier()
    sa.close()
    dist.destroy_process_group()
    if rank != 0:
        return
    link_bytes = nbytes * (world - 1) / world          # bytes that leave each GPU per call
    emit({
        "metric": "all_to_all_bus_gb_per_s", "value": link_bytes / (res["peer"] / 1e3) / 1e9, "unit": "GB/s per direction per GPU",
        "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": res["peer"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u8", "data": "synthetic",
        "config": {"workload": "all_to_all of the [E,C,M] fp16 expert buffer, %d bytes per GPU" % nbytes},
        "peer_memory": {"ms": res["peer"], "gb_per_s": link_bytes / (res["peer"] / 1e3) / 1e9},
        "nccl_grouped_send_recv": {"ms": res["nccl"], "gb_per_s": link_bytes / (res["nccl"] / 1e3) / 1e9},
        "results_identical": ok,
        "roofline": {"bound": "nvlink", "kernel": "a2a_store_kernel", "achieved": link_bytes / (res["peer"] / 1e3) / 1e9,
                     "peak": 770.0, "unit": "GB/s", "frac": link_bytes / (res["peer"] / 1e3) / 1e9 / 770.0,
                     "peak_kind": "measured peer copy, per direction", "traffic": None},
    })


def run_gpt(args):
    """Full GPT-MoE training step (nl=12, m=1024, nh=16, sl=512, b=16 per GPU, vocab 50257, every other layer MoE with
    2N experts of FFN 4096, top-2, capacity factor 1.25, bf16 autocast, LANS).  Token ids are uniform random from a seed."""
    import lancet_b200 as LB
    from lancet_b200.gpt_moe import GPTMoE, LansTrainer
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit("bench.py: --gpus %d but WORLD_SIZE=%d" % (args.gpus, world))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    fabric = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    else:
        fabric = LB.LocalFabric(1, 0, {})
    vocab, m, nh, nl, seq, batch, ffn = 50257, 1024, 16, 12, 512, 16, 4096
    model = GPTMoE(vocab, m, nh, nl, seq, batch, ffn, 2 * world, TOP_K, CAP_FACTOR, N_CHUNKS, dev, fabric=fabric, seed=0,
                   act="relu")     # the reference's GPT-2 blocks use ReLU
    trainer = LansTrainer(model, lr=1e-3)
    g = torch.Generator(device=dev).manual_seed(1000 + rank)
    ids = [torch.randint(0, vocab, (batch, seq), device=dev, generator=g) for _ in range(2)]
    losses = []
    for i in range(max(args.warmup, 3)):
        losses.append(float(trainer.step(ids[i % 2])))
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for i in range(args.steps):
        loss = trainer.step(ids[i % 2])
    ev1.record()
    torch.cuda.synchronize()
    losses.append(float(loss))
    ms = ev0.elapsed_time(ev1) / args.steps
    if world > 1:
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
        dist.barrier()
        model.close()
        dist.destroy_process_group()
    if rank != 0:
        return
    n_params = sum(p.numel() for p in model.parameters())
    emit({
        "metric": "gpt_moe_tokens_per_s", "value": batch * seq * world / (ms / 1e3), "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "gpt2_moe_nl12_m1024_nh16_sl512_b16 training step, %d experts, top-2, cf 1.25, LANS" % (2 * world),
                   "params_per_rank": n_params},
        "loss_first": losses[0], "loss_last": losses[-1],
    })


def main():
    # libraries (NCCL, torchrun) may write to stdout; keep it clean for the one JSON line
    saved_stdout = os.dup(1)
    os.dup2(2, 1)
    try:
        _main()
    finally:
        sys.stdout.flush()
        os.dup2(saved_stdout, 1)
        if _RESULT_LINES:
            os.write(1, ("\n".join(_RESULT_LINES) + "\n").encode())


_RESULT_LINES = []


def emit(line):
    _RESULT_LINES.append(json.dumps(line))


def _main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="moe", choices=["moe", "lans", "ffn", "layer", "a2a", "gpt"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-graph", action="store_true", help="launch every step eagerly instead of replaying a CUDA graph")
    ap.add_argument("--schedule", default="all", choices=["all", "staged", "side", "single"],
                    help="layer workload: which schedules to time (all: the three take turns)")
    ap.add_argument("--stages", type=int, default=4, help="layer workload: exchange stages of the pipelined schedule")
    ap.add_argument("--lans-layers", type=int, default=24, help="transformer layers in the LANS tensor list (24 = 196 tensors)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    if args.workload == "lans":
        run_lans(args)
    elif args.workload == "ffn":
        run_ffn(args)
    elif args.workload == "layer":
        run_layer(args)
    elif args.workload == "a2a":
        run_a2a(args)
    elif args.workload == "gpt":
        run_gpt(args)
    else:
        run_moe(args)


if __name__ == "__main__":
    main()
