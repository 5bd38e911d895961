"""Benchmark of the MoE data-parallel hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload moe|lans|ffn|layer|a2a|peerbw|gpt]

Workload "moe" (default, the configuration the headline metric is quoted on): per GPU S=16384
tokens, M=2048, fp16 tokens, fp32 gate probabilities, E=2*N experts, top-2, capacity factor 1.25,
dispatch in 4 chained chunks + exchange + combine.  A step is one pass over one batch of seeded
synthetic tokens.  One JSON line is printed by rank 0.

The default line also carries, under "workloads", short legs of the other parts of the path
(LANS step, expert FFN forward + backward, whole MoE layer; at N > 1 the layer and the NVLink
bandwidth yardstick), each with its own roofline, and "result_checked": after the timed region
one step is verified on every rank (combined output against sum_j gate_j * x, every row of the
receive buffer against a checksum of the source row it must hold, all other rows zero; at N > 1
also `_all_to_all` / `_all_to_allv` over NCCL and over peer memory against torch.distributed).
A failed check makes the run exit non-zero.

Timing: W >= 3 warm-up steps; the timed region is R bursts of K steps each (R chosen so that the
region lasts at least ~0.3 s), every burst bracketed by CUDA events on the launching stream;
ms_per_step = median burst / K, maximum over ranks.
"""
import argparse
import ctypes
import json
import math
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
NVLINK_NOMINAL_GBS = 900.0          # per direction per GPU
NVLINK_FALLBACK_GBS = 770.0         # an earlier peer-copy measurement on this pool, used only if the live leg fails
TARGET_REGION_S = 0.3


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return d, "measured"
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.tmp = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(gpu_index), "--query-gpu=" + self.FIELDS + ",timestamp",
                 "--format=csv,noheader,nounits", "-lms", "50"], stdout=self.tmp, stderr=subprocess.DEVNULL)
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
        sm, mx, power, reasons = [], [], [], set()
        for r in rows:
            try:
                clk, cmax = float(r[1]), float(r[2])
            except (ValueError, IndexError):
                continue
            sm.append(clk)
            mx.append(cmax)
            try:
                power.append(float(r[3]))
            except (ValueError, IndexError):
                pass
            for name, col in (("hw_slowdown", 5), ("hw_thermal_slowdown", 6), ("sw_thermal_slowdown", 7),
                              ("sw_power_cap", 8)):
                if len(r) > col and r[col].strip().lower() == "active":
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        # under load = the upper half of the samples (idle samples before/after the region are low)
        hi = sorted(sm)[len(sm) // 2:]
        return {"sm_mhz": statistics.median(hi), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm), "power_w_max": max(power) if power else None}


class Ctx:
    """Rank / device / process group of this run (one process per GPU)."""

    def __init__(self, args):
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        if self.world != args.gpus:
            raise SystemExit("bench.py: --gpus %d but WORLD_SIZE=%d (launch with torch.distributed.run for N>1)" % (
                args.gpus, self.world))
        torch.cuda.set_device(self.local_rank)
        self.dev = torch.device("cuda", self.local_rank)
        self.dist = None
        if self.world > 1:
            import torch.distributed as dist
            dist.init_process_group("nccl", device_id=self.dev)
            self.dist = dist

    def sync(self):
        torch.cuda.synchronize()
        if self.dist is not None:
            self.dist.barrier()
            torch.cuda.synchronize()

    def max_over_ranks(self, v):
        if self.dist is None:
            return float(v)
        t = torch.tensor([float(v)], device=self.dev, dtype=torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def all_true(self, ok):
        if self.dist is None:
            return bool(ok)
        t = torch.tensor([1 if ok else 0], device=self.dev, dtype=torch.int32)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MIN)
        return bool(t.item())

    def close(self):
        if self.dist is not None:
            self.dist.barrier()
            self.dist.destroy_process_group()
            self.dist = None


def timed_bursts(ctx, enqueue_burst, steps, target_s=TARGET_REGION_S, max_bursts=400, min_bursts=5):
    """Times R bursts of `steps` steps each, back to back, every burst bracketed by a CUDA event pair on the current
    stream; R is chosen from a pilot burst so that the region lasts >= target_s.  Returns (ms per step from the median
    burst, maximum over ranks; info dict)."""
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ctx.sync()
    e0.record()
    enqueue_burst()
    e1.record()
    torch.cuda.synchronize()
    pilot = ctx.max_over_ranks(e0.elapsed_time(e1))
    R = int(min(max_bursts, max(min_bursts, math.ceil(target_s * 1e3 / max(pilot, 1e-3)))))
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(R)]
    ctx.sync()
    t_host = time.perf_counter()
    for a, b in evs:
        a.record()
        enqueue_burst()
        b.record()
    ctx.sync()
    wall = time.perf_counter() - t_host
    times = [a.elapsed_time(b) for a, b in evs]
    med = ctx.max_over_ranks(statistics.median(times))
    info = {"bursts": R, "steps_per_burst": steps, "timed_steps": R * steps, "burst_ms_median": med,
            "burst_ms_min": min(times), "burst_ms_max": max(times),
            "burst_spread": (max(times) - min(times)) / med if med > 0 else None,
            "timed_region_s": sum(times) / 1e3, "timed_region_wall_s": wall}
    return med / steps, info


class NvlinkCounter:
    """NVLink data bytes sent / received by one GPU, summed over its links (NVML field values; read-only)."""
    TX, RX = 138, 139               # NVML_FI_DEV_NVLINK_THROUGHPUT_DATA_TX / _RX, in KiB

    def __init__(self, index):
        self.h = None
        self.why = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.read()
        except Exception as e:
            self.h = None
            self.why = "NVML unavailable: %s" % e

    def read(self):
        if self.h is None:
            return None
        try:
            vals = self.nv.nvmlDeviceGetFieldValues(self.h, [(self.TX, 0xFFFFFFFF), (self.RX, 0xFFFFFFFF)])
            out = []
            for v in vals:
                if v.nvmlReturn != 0:
                    self.why = "NVML field %d: return code %d" % (v.fieldId, v.nvmlReturn)
                    return None
                out.append(int(v.value.ullVal) * 1024)
            return tuple(out)
        except Exception as e:
            self.why = "NVML field query failed: %s" % e
            return None


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


# ---------------------------------------------------------------------------------------------------------------
# CPU arms (the only code in this file that executes oracle/)
# ---------------------------------------------------------------------------------------------------------------
def cpu_reference_sample(max_seconds, world=1, tokens=None):
    """Times the restatement of the reference's torch-CPU operators (per-token loops) on a sample
    of the workload; returns (tokens_per_s, cores, description, seconds, tokens)."""
    from oracle import moe_oracle as O
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    E = 2 * world

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
    what = "%d of %d tokens of ONE rank, M=%d, E=%d, top-%d, encode+decode with per-token loops" % (
        tokens, S_TOKENS, M_DIM, E, TOP_K) + " (torch CPU ops on %d threads, the loops are single-threaded Python)" % cores
    return tokens / dt, cores, what, dt, tokens


def cpu_vectorised_sample(world=1, repeats=3):
    """The same encode+decode with vectorised NumPy (argmax / cumulative counts / fancy indexing): the CPU number a
    NumPy user would get, next to the per-token loop port of the reference's torch-CPU operators."""
    from oracle import moe_oracle as O
    E = 2 * world
    xs, gates = synth_inputs(0, world, S_TOKENS, M_DIM, torch.float16, sets=1)
    x, gate = xs[0].numpy(), gates[0].numpy()
    C = O.capacity(S_TOKENS, E, CAP_FACTOR, TOP_K)
    times = []
    for _ in range(repeats):
        t0 = time.perf_counter()
        gs, il, cap, el = O.moe_gate(gate, np.zeros(E, np.int32), C, M_DIM, TOP_K)
        disp = O.moe_encode_fwd(il, x, E, C)
        out = O.moe_decode_fwd(disp, gs, il)
        times.append(time.perf_counter() - t0)
    dt = statistics.median(times)
    return {"value": S_TOKENS / dt, "unit": "tokens/s", "cores": 1, "kind": "port",
            "sample": "all %d tokens of one rank, vectorised NumPy encode+decode, median of %d" % (S_TOKENS, repeats)}


def cpu_lans_sample():
    """One LANS step of the NumPy float32 port on the eight tensors of one transformer layer of the bench's list
    (12.6 M elements, a few seconds): the CPU figure next to the LANS leg, a reported baseline."""
    from oracle import lans_oracle
    shapes = lans_shapes(1)[2:10]
    rng = np.random.default_rng(0)
    p = [rng.normal(0, 0.02, s).astype(np.float32) for s in shapes]
    g = [rng.normal(0, 1e-3, s).astype(np.float32) for s in shapes]
    m = [rng.normal(0, 1e-4, s).astype(np.float32) for s in shapes]
    v = [rng.uniform(0, 1e-6, s).astype(np.float32) for s in shapes]
    n_el = sum(a.size for a in p)
    t0 = time.perf_counter()
    lans_oracle.lans_step(g, p, m, v, step=10)
    dt = time.perf_counter() - t0
    return {"value": n_el / dt, "unit": "elements/s", "cores": 1, "kind": "port",
            "sample": "one step over the %d tensors of one transformer layer of the list, %.1f M elements, NumPy float32" % (
                len(shapes), n_el / 1e6)}


def run_reference_arm(args):
    """--impl reference: the reference's CPU implementation of the path (restated port; the reference
    itself has no CPU operator that builds without TVM) on the host cores.  One rank's work is timed, at any N."""
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
    if world > 1:
        sample += "; at N=%d this is ONE rank's throughput on the host, not %d ranks'" % (world, world)
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
        "tokens_per_gpu": S_TOKENS, "row_width": M_DIM, "experts": 2 * world, "top_k": TOP_K,
        "capacity_factor": CAP_FACTOR, "chunks": N_CHUNKS,
        "l2": "inputs rotate over 2 sets; 288 MiB touched per step exceeds the 126 MB L2"}


# ---------------------------------------------------------------------------------------------------------------
# result checks
# ---------------------------------------------------------------------------------------------------------------
def row_checksums(t, chunk_rows=8192):
    """Two int64 checksums per row of a 16-bit tensor [..., M]: a position-weighted sum of the raw bit patterns
    (detects wrong, shifted or permuted rows) and the sum of their absolute values (zero only for an all-zero row)."""
    M = t.shape[-1]
    flat = t.reshape(-1, M).view(torch.int16)
    w = (torch.arange(M, device=t.device) % 251 + 1).to(torch.int64)
    cs = torch.empty(flat.shape[0], dtype=torch.int64, device=t.device)
    ab = torch.empty_like(cs)
    for r0 in range(0, flat.shape[0], chunk_rows):
        blk = flat[r0:r0 + chunk_rows].to(torch.int64)
        cs[r0:r0 + chunk_rows] = (blk * w).sum(dim=1)
        ab[r0:r0 + chunk_rows] = blk.abs().sum(dim=1)
    return cs.view(t.shape[:-1]), ab.view(t.shape[:-1])


def verify_moe_step(ctx, plan, x, gate):
    """One dispatch + combine with identity experts, verified on this rank (see the module docstring)."""
    world, rank = ctx.world, ctx.rank
    recv = plan.dispatch(x, gate)
    out = plan.combine().clone()
    torch.cuda.synchronize()
    if world > 1:
        plan.check()
    k, S, M, C = plan.k, plan.S, plan.M, plan.C
    E = plan.E
    LE = plan.LE if world > 1 else E
    il = plan.idx_loc                               # [n, 2k, Sp]; locations are rows of the shared [E, C, M] buffer
    gs = plan.gates_s                               # [n, k, Sp]
    idx = [il[:, 2 * j, :].reshape(S).long() for j in range(k)]
    loc = [il[:, 2 * j + 1, :].reshape(S).long() for j in range(k)]
    kept = [(idx[j] >= 0) & (idx[j] < E) & (loc[j] >= 0) & (loc[j] < C) for j in range(k)]
    # (1) combined output = sum_j gate_j * x over the kept choices: fp32 products and sum, rounded once (the kernel's order)
    xf = x.float()
    acc = torch.zeros_like(xf)
    seen = torch.zeros(S, dtype=torch.bool, device=x.device)
    for j in range(k):
        prod = gs[:, j, :].reshape(S, 1) * xf
        acc = torch.where((kept[j] & seen)[:, None], acc + prod, torch.where(kept[j][:, None], prod, acc))
        seen |= kept[j]
    want = acc.to(x.dtype)
    exact = bool(torch.equal(out, want))
    err = float((out.float() - want.float()).abs().max())
    scale = float(want.float().abs().max())
    combine_ok = err <= 1e-2 * max(scale, 1e-6)      # fp16/bf16 tolerance of the path: rel 1e-2; normally bit-exact
    # (2) receive buffer: row (g, le, loc) must be the source row of the token of rank g routed there, all others zero
    tok_cs, _ = row_checksums(x)
    my_il = torch.stack(idx + loc + [kj.long() for kj in kept])           # [3k, S]
    if world > 1:
        all_il = [torch.empty_like(my_il) for _ in range(world)]
        all_cs = [torch.empty_like(tok_cs) for _ in range(world)]
        ctx.dist.all_gather(all_il, my_il)
        ctx.dist.all_gather(all_cs, tok_cs)
    else:
        all_il, all_cs = [my_il], [tok_cs]
    recv4 = recv.reshape(world, LE, C, M)
    got_cs, got_abs = row_checksums(recv4)
    want_cs = torch.zeros_like(got_cs)
    live = torch.zeros_like(got_cs, dtype=torch.bool)
    n_expected = 0
    for g in range(world):
        t = all_il[g]
        for j in range(k):
            e, l, kp = t[j], t[k + j], t[2 * k + j].bool()
            mine = kp & (torch.div(e, LE, rounding_mode="floor") == rank)
            le = e[mine] - rank * LE
            want_cs[g, le, l[mine]] = all_cs[g][mine]
            live[g, le, l[mine]] = True
            n_expected += int(mine.sum())
    rows_ok = bool(torch.equal(got_cs[live], want_cs[live])) and int(live.sum()) == n_expected
    zero_ok = bool((got_abs[~live] == 0).all())
    return {"ok": bool(combine_ok and rows_ok and zero_ok), "combine_bit_exact": exact, "combine_max_abs_err": err,
            "recv_rows_checked": n_expected, "recv_rows_ok": rows_ok, "recv_padding_zero": zero_ok}


def verify_collectives(ctx):
    """`_all_to_all` and `_all_to_allv`, over NCCL (what raf.op.nccl.* dispatches to) and over peer memory, against
    torch.distributed.all_to_all_single on the same data."""
    import lancet_b200 as LB
    dist, W, rank, dev = ctx.dist, ctx.world, ctx.rank, ctx.dev
    nch, chunk = 2, 4096
    g = torch.Generator(device=dev).manual_seed(77 + rank)
    x = torch.randn((W, nch, chunk), device=dev, generator=g)
    ref = torch.empty_like(x)
    dist.all_to_all_single(ref, x)
    comm = LB.Communicator(dev)
    sa = LB.SymmAllToAll(x.numel() * 4, dev, n_chunks=nch)
    ok_nccl = bool(torch.equal(comm.all_to_all(x), ref))
    ok_peer = bool(torch.equal(sa.all_to_all(x), ref))
    counts = torch.tensor([(i + j + rank) % 5 * 700 + 3 for i in range(W) for j in range(nch)], dtype=torch.int64, device=dev)
    ref_counts = torch.empty_like(counts)
    dist.all_to_all_single(ref_counts, counts)
    keep = torch.arange(chunk, device=dev)[None, None, :] < ref_counts.view(W, nch, 1)
    ref_v = torch.where(keep, ref, torch.zeros_like(ref))
    gn, rn = comm.all_to_allv(x, counts)
    ok_nccl_v = bool(torch.equal(gn, ref_v)) and bool(torch.equal(rn.view(torch.int64), ref_counts))
    gp, rp = sa.all_to_allv(x, counts)
    ok_peer_v = bool(torch.equal(gp.view_as(ref_v), ref_v)) and bool(torch.equal(rp.view(torch.int64), ref_counts))
    torch.cuda.synchronize()
    sa.check()
    comm.close()
    dist.barrier()
    sa.close()
    return {"ok": ok_nccl and ok_peer and ok_nccl_v and ok_peer_v, "all_to_all_nccl": ok_nccl, "all_to_all_peer": ok_peer,
            "all_to_allv_nccl": ok_nccl_v, "all_to_allv_peer": ok_peer_v}


# ---------------------------------------------------------------------------------------------------------------
# NVLink yardstick
# ---------------------------------------------------------------------------------------------------------------
def leg_peerbw(ctx, per_peer_mib=64, iters=10):
    """All N ranks send per_peer_mib MiB to every peer at the same time: (i) the copy engines, one cudaMemcpyAsync per
    peer on its own stream, (ii) the 16-byte peer-store kernel of the stand-alone all-to-all, at several grid sizes.
    GB/s are per direction per GPU (bytes that leave one GPU / time), maximum time over ranks."""
    import lancet_b200 as LB
    from lancet_b200 import _capi
    L = _capi.lib()
    W, rank, dev = ctx.world, ctx.rank, ctx.dev
    per = per_peer_mib << 20
    sa = LB.SymmAllToAll(per * W, dev)
    src = torch.empty(per * W, dtype=torch.uint8, device=dev).random_(0, 255)
    streams = [torch.cuda.Stream(device=dev) for _ in range(W)]
    out_bytes = per * (W - 1)
    res = {}

    def timed(fn):
        for _ in range(2):
            fn()
        ctx.sync()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = ctx.max_over_ranks(e0.elapsed_time(e1) / iters)
        ctx.sync()
        return out_bytes / (ms / 1e3) / 1e9

    def copy_engines():
        cur = torch.cuda.current_stream()
        for i in range(1, W):
            p = (rank + i) % W
            s = streams[p]
            s.wait_stream(cur)
            _capi.check(L.lancet_peer_copy(ctypes.c_void_p(sa.peer_recv[p] + rank * per), ctypes.c_void_p(src.data_ptr() + p * per),
                                           per, ctypes.c_void_p(s.cuda_stream)))
        for i in range(1, W):
            cur.wait_stream(streams[(rank + i) % W])

    res["copy_engine_gbs"] = timed(copy_engines)
    sweep = {}
    for ctas in (16, 32, 64, 148, 296, 0):
        _capi.check(L.lancet_set_cta_limits(ctas, 0))
        sweep[str(ctas) if ctas else "default"] = timed(lambda: sa.send(src))
    _capi.check(L.lancet_set_cta_limits(0, 0))
    res["store_kernel_gbs_by_ctas"] = sweep
    res["store_kernel_gbs"] = max(sweep.values())
    # the self block is a local copy inside the store kernel: (W-1)/W of the bytes cross NVLink, which is what is counted
    res["peak_gbs"] = max(res["copy_engine_gbs"], res["store_kernel_gbs"])
    res["nominal_gbs"] = NVLINK_NOMINAL_GBS
    res["bytes_out_per_gpu"] = out_bytes
    res["what"] = "all %d ranks send %d MiB to every peer at once; GB/s per direction per GPU, max time over ranks" % (W, per_peer_mib)
    sa.check()
    ctx.sync()
    sa.close()
    return res


# ---------------------------------------------------------------------------------------------------------------
# MoE dispatch + exchange + combine (the headline)
# ---------------------------------------------------------------------------------------------------------------
def run_moe(args):
    import lancet_b200 as LB
    from lancet_b200 import _capi
    ctx = Ctx(args)
    rank, world, dev = ctx.rank, ctx.world, ctx.dev
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

    K = args.steps
    warm = max(args.warmup, 3)
    for i in range(warm):
        step(i)
    ctx.sync()
    l0 = L.lancet_launch_count()
    step(0)
    launches_per_step = int(L.lancet_launch_count() - l0)
    kname = b"dispatch_rows_kernel" if world == 1 else b"dispatch_rows_peer_kernel"
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
        for i in range(4):
            graphs[i % 2].replay()
        ctx.sync()

        def burst():
            for i in range(K):
                graphs[i % 2].replay()
    else:
        def burst():
            for i in range(K):
                step(i)

    # ---- timed region: R bursts of K steps, device resident inputs ---------------------------------
    sampler = ClockSampler(ctx.local_rank) if rank == 0 else None
    ms_step, timing = timed_bursts(ctx, burst, K)
    value = S_TOKENS * world / (ms_step / 1e3)
    # per-kernel durations: the same steps launched eagerly right after, bracketed by events in the library
    n_prof = 100
    L.lancet_profile_begin(kname)
    for i in range(n_prof):
        step(i)
    ctx.sync()
    k_ms, k_n = ctypes.c_double(0), ctypes.c_longlong(0)
    _capi.check(L.lancet_profile_end(ctypes.byref(k_ms), ctypes.byref(k_n)))
    # the dominant kernel alone, launched back to back (no event pair around every launch): the duration without the
    # bracket's launch gap.  The routing table of the last step is reused; the two input sets alternate (128 MiB read and
    # 160 MiB written per pair of launches: more than the 126 MB L2)
    b2b_us = None
    if world == 1:
        def scatter_burst():
            for i in range(K):
                plan.scatter(xs[i % 2])
        scatter_burst()
        ms_b2b, _ = timed_bursts(ctx, scatter_burst, K, target_s=0.1)
        b2b_us = ms_b2b * 1e3

    # ---- end to end: pinned host inputs in, combined output back, every step ---------------------
    # Three streams, double-buffered device tensors: the host->device copy of step i+1 and the device->host copy
    # of step i-1 run while step i computes (PCIe is full duplex), as a data loader with prefetch would do.
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
    e2e_count = [0]

    def e2e_step():
        i = e2e_count[0]
        e2e_count[0] += 1
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

    def e2e_burst():
        for _ in range(K):
            e2e_step()
        s_comp.wait_stream(s_in)
        s_comp.wait_stream(s_out)

    e2e_burst()
    e2e_ms, e2e_timing = timed_bursts(ctx, e2e_burst, K, min_bursts=3)
    e2e_value = S_TOKENS * world / (e2e_ms / 1e3)
    clocks = ClockSampler.summarise(sampler.stop()) if sampler else None

    # ---- verification of one step on every rank ----------------------------------------------------
    chk = verify_moe_step(ctx, plan, xs[0], gates[0])
    coll = verify_collectives(ctx) if world > 1 else None
    checked = ctx.all_true(chk["ok"] and (coll is None or coll["ok"]))

    # ---- NVLink bytes per dispatch launch, read from the GPU's link counters (N > 1) --------------
    nv_traffic = None
    if world > 1:
        plan.check()
        nvc = NvlinkCounter(ctx.local_rank)
        ctx.sync()
        c0 = nvc.read()
        n_iter = 20
        for i in range(n_iter):
            plan.dispatch(xs[i % 2], gates[i % 2])
        ctx.sync()
        c1 = nvc.read()
        if c0 is None or c1 is None:
            nv_traffic = {"tx_bytes_per_launch": None, "rx_bytes_per_launch": None, "source": nvc.why}
        else:
            nv_traffic = {"tx_bytes_per_launch": (c1[0] - c0[0]) / n_iter, "rx_bytes_per_launch": (c1[1] - c0[1]) / n_iter,
                          "source": "NVML NVLink data throughput counters of GPU %d over %d dispatch launches" % (ctx.local_rank, n_iter)}
    cap_all = plan.capused.cpu().numpy()
    peer = leg_peerbw(ctx) if world > 1 else None
    workloads = {}
    if not args.no_legs:
        plan_C = plan.C
        if world > 1:
            ctx.dist.barrier()
            plan.close()
        plan = None
        torch.cuda.empty_cache()
        if world == 1:
            workloads["lans"] = leg_lans(args, ctx, steps=10)
            torch.cuda.empty_cache()
            workloads["ffn"] = leg_ffn(args, ctx, steps=10)
            torch.cuda.empty_cache()
        workloads["layer"] = leg_layer(args, ctx, steps=20)
        if peer is not None:
            workloads["peerbw"] = peer
    else:
        plan_C = plan.C
        if world > 1:
            ctx.dist.barrier()
            plan.close()
    ctx.close()
    if rank != 0:
        if not checked:
            sys.exit(3)
        return
    # ---- roofline of the dominant kernel (dispatch scatter) ---------------------------------------
    peaks, peak_kind = load_peaks()
    hbm_peak = float(peaks.get("hbm_gbs", FALLBACK_PEAKS["hbm_gbs"]))
    kept_rows = int(cap_all[-1].sum())                  # rows written by the dispatch launch of a step
    row_bytes = M_DIM * 2
    # algorithmic bytes of the dispatch launch (all chunks in one launch): token rows read once, the
    # whole padded [E,C,M] buffer written once (kept rows + zero rows)
    bytes_per_launch = S_TOKENS * row_bytes + E * plan_C * row_bytes
    roof = None
    if k_n.value > 0:
        avg_s = k_ms.value / k_n.value / 1e3
        achieved = bytes_per_launch / avg_s / 1e9
        roof = {"bound": "hbm", "kernel": kname.decode(), "achieved": achieved, "peak": hbm_peak, "unit": "GB/s",
                "frac": achieved / hbm_peak, "peak_kind": peak_kind, "traffic": None,
                "bytes_per_launch": bytes_per_launch, "avg_launch_us": avg_s * 1e6, "launches_timed": k_n.value}
        if world > 1:
            # the fused dispatch is bound by the bytes that leave this GPU over NVLink: the live rows whose expert
            # lives on another GPU; peak = the all-ranks-at-once peer bandwidth measured in this run (peerbw leg)
            LE = 2
            remote_rows = int(cap_all[-1][LE:].sum())           # rank 0 owns experts [0, LE): the rest crosses NVLink
            nv_bytes = remote_rows * row_bytes
            nv = nv_bytes / avg_s / 1e9
            peak = peer["peak_gbs"] if peer else NVLINK_FALLBACK_GBS
            roof.update({"bound": "nvlink", "achieved": nv, "peak": peak, "frac": nv / peak,
                         "peak_kind": ("measured in this run: all ranks to all peers, best of copy engines and store kernel"
                                       if peer else "earlier peer-copy measurement"),
                         "frac_of_nominal_900": nv / NVLINK_NOMINAL_GBS, "bytes_per_launch": nv_bytes, "hbm_achieved": achieved,
                         "traffic": nv_traffic["tx_bytes_per_launch"] if nv_traffic else None,   # NVLink bytes sent per launch (NVML)
                         "traffic_detail": nv_traffic})
        if world == 1:
            # dram read + write bytes per launch from the ncu capture of this workload
            # (profiles/moe_dispatch_combine_S16384_M2048_ncu_full.txt)
            roof["traffic"] = 177.2e6
            if b2b_us:
                # the kernel's average launch duration in a burst of launches of that kernel alone (one event pair around
                # the burst) is the figure the fraction is quoted on; the per-launch event bracket, which adds the gap of
                # two event records to every launch, is kept beside it
                roof.update({"bracketed_launch_us": roof["avg_launch_us"], "frac_bracketed": roof["frac"],
                             "achieved_bracketed": roof["achieved"], "avg_launch_us": b2b_us,
                             "achieved": bytes_per_launch / (b2b_us * 1e-6) / 1e9,
                             "frac": bytes_per_launch / (b2b_us * 1e-6) / 1e9 / hbm_peak,
                             "how": "burst of %d launches of the kernel between one CUDA event pair, median burst / %d" % (K, K)})
    line = {
        "metric": "moe_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": K,
        "warmup": warm, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16", "data": "synthetic", "config": moe_config(world),
        "timing": timing,
        "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": S_TOKENS * row_bytes + S_TOKENS * E * 4,
                "d2h_bytes_per_step": S_TOKENS * row_bytes, "steps": e2e_timing["timed_steps"], "ms_per_step": e2e_ms,
                "timed_region_s": e2e_timing["timed_region_s"]},
        "gpu_launches": launches_per_step * timing["timed_steps"], "gpu_launches_per_step": launches_per_step,
        "clocks": clocks, "roofline": roof,
        "result_checked": checked, "result_check": chk, "collectives_check": coll,
        "launch_mode": "cuda graph replay (kernel durations from an eager loop of the same steps)" if use_graph else "eager",
        "step_bytes": {"dispatch_read": S_TOKENS * row_bytes, "dispatch_write": E * plan_C * row_bytes,
                       "combine_read": kept_rows * row_bytes, "combine_write": S_TOKENS * row_bytes},
    }
    step_bytes = sum(line["step_bytes"].values())
    line["step_hbm_frac"] = step_bytes / (ms_step / 1e3) / 1e9 / hbm_peak
    if workloads:
        line["workloads"] = workloads
    if world == 1 and not args.no_cpu:
        rate, cores, sample, _, _ = cpu_reference_sample(15.0, 1)
        line["cpu_baseline"] = {"value": rate, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample}
        line["cpu_baseline_vectorised"] = cpu_vectorised_sample(1)
    emit(line)
    if not checked:
        sys.exit(3)


# ---------------------------------------------------------------------------------------------------------------
# LANS
# ---------------------------------------------------------------------------------------------------------------
def lans_shapes(layers=24):
    """196 fp32 tensors, 354.6 M elements: GPT-2-medium-like (24 layers x 8 tensors + embeddings + final norm)."""
    shapes = [(50257, 1024), (1024, 1024)]
    for _ in range(layers):
        shapes += [(1024, 1024), (1024, 1024), (1024, 1024), (1024, 1024), (4096, 1024), (1024, 4096), (1024,), (1024,)]
    shapes += [(1024,), (1024,)]
    return shapes


def leg_lans(args, ctx, steps):
    import lancet_b200 as LB
    from lancet_b200 import _capi
    dev = ctx.dev
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
    step_dev = torch.zeros((), dtype=torch.float32, device=dev)
    sampler = ClockSampler(dev.index)
    for i in range(max(args.warmup, 3)):
        LB.lans(tl, 10 + i, state=state)
    torch.cuda.synchronize()
    counter = [20]

    def burst():
        for _ in range(steps):
            LB.lans(tl, counter[0], state=state)
            counter[0] += 1

    l0 = L.lancet_launch_count()
    burst()
    launches = (L.lancet_launch_count() - l0) // steps
    ms, timing = timed_bursts(ctx, burst, steps)
    per_phase = {}
    for ph, bpe in (("lans_phase1_kernel", 4.0), ("lans_phase2_kernel", 24.0), ("lans_phase3_kernel", 20.0)):
        L.lancet_profile_begin(ph.encode())
        burst()
        torch.cuda.synchronize()
        k_ms, k_n = ctypes.c_double(0), ctypes.c_longlong(0)
        _capi.check(L.lancet_profile_end(ctypes.byref(k_ms), ctypes.byref(k_n)))
        avg_s = k_ms.value / max(1, k_n.value) / 1e3
        per_phase[ph] = {"avg_launch_us": avg_s * 1e6, "gbs": bpe * n_el / avg_s / 1e9, "bytes_per_element": bpe}
    # the same step with the step counter on the device (no host round trip): must cost the same
    def burst_dev():
        for _ in range(steps):
            step_dev.add_(1.0)
            LB.lans(tl, step_dev, state=state)
    step_dev.fill_(float(counter[0]))
    burst_dev()
    ms_dev, _ = timed_bursts(ctx, burst_dev, steps, target_s=0.1)
    clocks = ClockSampler.summarise(sampler.stop())
    peaks, peak_kind = load_peaks()
    hbm_peak = float(peaks.get("hbm_gbs", FALLBACK_PEAKS["hbm_gbs"]))
    p2 = per_phase["lans_phase2_kernel"]
    del P, G, Mo, V, tl, state
    cpu = None if getattr(args, "no_cpu", False) else cpu_lans_sample()
    return {
        "cpu_baseline": cpu,
        "metric": "lans_elements_per_s", "value": n_el / (ms / 1e3), "unit": "elements/s", "ms_per_step": ms,
        "dtype": "f32", "timing": timing,
        "config": {"workload": "lans_step: %d fp32 tensors, %d elements" % (len(shapes), n_el),
                   "l2": "5.6 GB of state per step exceeds the 126 MB L2"},
        "gpu_launches_per_step": int(launches), "clocks": clocks,
        "roofline": {"bound": "hbm", "kernel": "lans_phase2_kernel", "achieved": p2["gbs"], "peak": hbm_peak,
                     "unit": "GB/s", "frac": p2["gbs"] / hbm_peak, "peak_kind": peak_kind,
                     # 23.30 B/element measured by ncu on a 77.7 M-element list, scaled by the element count
                     # (profiles/lans_phase_kernels_77M_elements_ncu_full.txt)
                     "traffic": 23.30 * n_el,
                     "bytes_per_launch": 24.0 * n_el, "avg_launch_us": p2["avg_launch_us"]},
        "phases": per_phase,
        "step_hbm_frac": 48.0 * n_el / (ms / 1e3) / 1e9 / hbm_peak,
        "step_bytes_per_element": 48.0,
        "ms_per_step_device_step_counter": ms_dev,
    }


def as_line(leg, args, world=1):
    line = {"metric": leg["metric"], "value": leg["value"], "unit": leg["unit"], "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": leg["ms_per_step"], "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": leg.get("dtype", "bf16"), "data": "synthetic"}
    for k, v in leg.items():
        if k not in line:
            line[k] = v
    return line


# ---------------------------------------------------------------------------------------------------------------
# every form of the grouped GEMM alone (sustained, power-capped regime)
# ---------------------------------------------------------------------------------------------------------------
def leg_gemm_forms(args, ctx, steps):
    """Each form of the expert GEMM by itself in bursts of about 0.25 s (the regime of a training step: clocks under the
    power cap), on the shapes of the expert FFN configuration, paired and single-CTA form in turn, next to the library
    GEMM on the forward shape.  The value of the line is the plain forward form."""
    import lancet_b200 as LB
    from lancet_b200 import _capi
    dev = ctx.dev
    L = _capi.lib()
    G, LE, C, M, H = 8, 2, 2560, 2048, 8192
    g = torch.Generator(device=dev).manual_seed(0)
    x = torch.randn((G * LE, C, M), device=dev, generator=g).bfloat16()
    w1 = (torch.randn((LE, H, M), device=dev, generator=g) * 0.02).bfloat16()
    w2 = (torch.randn((LE, M, H), device=dev, generator=g) * 0.02).bfloat16()
    b1, b2 = torch.zeros((LE, H), device=dev).bfloat16(), torch.zeros((LE, M), device=dev).bfloat16()
    h = torch.empty((G * LE, C, H), device=dev, dtype=torch.bfloat16)
    hpre, dh = torch.empty_like(h), torch.empty_like(h)
    y = torch.empty((G * LE, C, M), device=dev, dtype=torch.bfloat16)
    dy = torch.randn((G * LE, C, M), device=dev, generator=g).bfloat16()
    dx, dw1, dw2 = torch.empty_like(x), torch.empty_like(w1), torch.empty_like(w2)
    flop = 2.0 * G * LE * C * M * H
    forms = {
        "nt_plain_K2048": lambda: LB.grouped_gemm_nt(x, w1, out=h),
        "nt_bias_gelu_pre_K2048": lambda: LB.grouped_gemm_nt(x, w1, bias=b1, act="gelu", out=h, preact=hpre),
        "nt_bias_gelu_K2048": lambda: LB.grouped_gemm_nt(x, w1, bias=b1, act="gelu", out=h),
        "nt_bias_gelu_tanh_pre_K2048": lambda: LB.grouped_gemm_nt(x, w1, bias=b1, act="gelu_tanh", out=h, preact=hpre),
        "nt_bias_relu_K2048": lambda: LB.grouped_gemm_nt(x, w1, bias=b1, act="relu", out=h),
        "nt_bias_K8192": lambda: LB.grouped_gemm_nt(h, w2, bias=b2, out=y),
        "nn_dgelu_K2048": lambda: LB.grouped_gemm_nn(dy, w2, act="gelu", preact=hpre, out=dh),
        "nn_dgelu_tanh_K2048": lambda: LB.grouped_gemm_nn(dy, w2, act="gelu_tanh", preact=hpre, out=dh),
        "nn_plain_K8192": lambda: LB.grouped_gemm_nn(dh, w1, out=dx),
        "tn_dw2": lambda: LB.grouped_gemm_tn(dy, h, LE, out=dw2),
        "tn_dw1": lambda: LB.grouped_gemm_tn(dh, x, LE, out=dw1),
    }
    xa = x.view(G, LE, C, M)[:, 0].reshape(G * C, M).contiguous()
    ha = torch.empty((G * C, H), device=dev, dtype=torch.bfloat16)

    def library():
        torch.matmul(xa, w1[0].t(), out=ha)
        torch.matmul(xa, w1[1].t(), out=ha)

    def timed(fn, target_s=0.25):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        n = max(5, int(target_s * 1e3 / max(e0.elapsed_time(e1), 1e-3)))
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n

    sampler = ClockSampler(dev.index)
    out = {}
    try:
        for name, fn in forms.items():
            row = {}
            for rep in range(2):                           # the two forms take turns twice: best of two per form
                for mode, flag in (("paired", 1), ("single_cta", 0)):
                    _capi.check(L.lancet_set_gemm_paired(flag))
                    ms = timed(fn)
                    row[mode] = min(ms, row.get(mode, ms))
            out[name] = {m: {"ms": v, "tflops": flop / v / 1e9} for m, v in row.items()}
    finally:
        _capi.check(L.lancet_set_gemm_paired(1))
    ms_lib = min(timed(library), timed(library))
    out["library_matmul_20480x8192x2048"] = {"ms": ms_lib, "tflops": flop / ms_lib / 1e9}
    clocks = ClockSampler.summarise(sampler.stop())
    st = LB.gemm_status(dev)
    _capi.check(L.lancet_p2p_status(ctypes.c_void_p(st.data_ptr()), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)))
    peaks, peak_kind = load_peaks()
    sustained = float(peaks.get("bf16_tflops_sustained", FALLBACK_PEAKS["bf16_tflops"]))
    best = out["nt_plain_K2048"]["paired"]
    return {"metric": "grouped_gemm_tflops", "value": best["tflops"], "unit": "TFLOP/s", "ms_per_step": best["ms"], "dtype": "bf16",
            "config": {"workload": "every form of the grouped GEMM alone: 16 groups x 2560 rows, M=2048, H=8192, bursts of 0.25 s",
                       "l2": "operands of 1.2 GB per launch exceed the 126 MB L2"},
            "clocks": clocks, "forms": out,
            "roofline": {"bound": "tensor", "kernel": "grouped_gemm_kernel (NT, plain, paired)", "achieved": best["tflops"],
                         "peak": sustained, "unit": "TFLOP/s", "frac": best["tflops"] / sustained,
                         "peak_kind": peak_kind + " (sustained cuBLAS bf16)", "traffic": None}}


# ---------------------------------------------------------------------------------------------------------------
# expert FFN
# ---------------------------------------------------------------------------------------------------------------
def leg_ffn(args, ctx, steps):
    """Expert FFN forward and backward (config 'expert FFN grouped GEMM'): per GPU 2 local experts, rows from 8 source
    ranks x C=2560, M=2048, H=8192, bf16 with fp32 accumulation: GEMM1 + bias + GELU, GEMM2 + bias; dH, dW2, dX, dW1."""
    import lancet_b200 as LB
    from lancet_b200 import _capi
    dev = ctx.dev
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
    hpre = torch.empty_like(h)
    st = LB.gemm_status(dev)

    def fwd_burst():
        for _ in range(steps):
            LB.grouped_gemm_nt(x, w1, bias=b1, act="gelu", out=h, preact=hpre)
            LB.grouped_gemm_nt(h, w2, bias=b2, out=y)

    sampler = ClockSampler(dev.index)
    for _ in range(max(args.warmup, 3) // steps + 1):
        fwd_burst()
    torch.cuda.synchronize()
    l0 = L.lancet_launch_count()
    fwd_burst()
    launches = (L.lancet_launch_count() - l0) // steps
    ms, timing = timed_bursts(ctx, fwd_burst, steps)
    L.lancet_profile_begin(b"grouped_gemm_nt_kernel")
    fwd_burst()
    torch.cuda.synchronize()
    k_ms, k_n = ctypes.c_double(0), ctypes.c_longlong(0)
    _capi.check(L.lancet_profile_end(ctypes.byref(k_ms), ctypes.byref(k_n)))
    _capi.check(L.lancet_p2p_status(ctypes.c_void_p(st.data_ptr()), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)))
    # backward GEMMs of the same layer: dH = (dY W2) * gelu'(H_pre), dW2 = dY^T H, dX = dH W1, dW1 = dH^T X, db2, db1
    dy = torch.randn((G * LE, C, M), device=dev, generator=g).bfloat16()
    dh, dx = torch.empty_like(h), torch.empty_like(x)
    dw1, dw2 = torch.empty_like(w1), torch.empty_like(w2)
    db1, db2 = torch.empty_like(b1), torch.empty_like(b2)

    def bwd_burst():
        for _ in range(steps):
            LB.grouped_gemm_nn(dy, w2, act="gelu", preact=hpre, out=dh)       # w2 is [LE, M, H]: contraction over M
            LB.grouped_gemm_tn(dy, h, LE, out=dw2)                            # [LE, M, H]
            LB.grouped_gemm_nn(dh, w1, out=dx)                                # w1 is [LE, H, M]: contraction over H
            LB.grouped_gemm_tn(dh, x, LE, out=dw1)                            # [LE, H, M]
            LB.grouped_bias_grad(dy, LE, out=db2)
            LB.grouped_bias_grad(dh, LE, out=db1)

    bwd_burst()
    bwd_ms, bwd_timing = timed_bursts(ctx, bwd_burst, steps)
    _capi.check(L.lancet_p2p_status(ctypes.c_void_p(st.data_ptr()), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)))
    # same-box bar: the library GEMM the reference calls (cuBLAS through torch), same shapes, forward
    xs = x.view(G, LE, C, M)

    def lib_burst():
        for _ in range(steps):
            for e in range(LE):
                a = xs[:, e].reshape(G * C, M)
                hh = torch.nn.functional.gelu(torch.addmm(b1[e], a, w1[e].t()))
                torch.addmm(b2[e], hh, w2[e].t())

    lib_burst()
    lib_ms, _ = timed_bursts(ctx, lib_burst, steps, target_s=0.15)
    clocks = ClockSampler.summarise(sampler.stop())
    peaks, peak_kind = load_peaks()
    flops = 2.0 * (G * LE * C) * M * H * 2
    sustained = float(peaks.get("bf16_tflops_sustained", peaks.get("bf16_tflops", FALLBACK_PEAKS["bf16_tflops"])))
    avg_s = k_ms.value / max(1, k_n.value) / 1e3
    ach = flops / 2 / avg_s / 1e12
    rows = G * LE * C
    return {
        "metric": "expert_ffn_rows_per_s", "value": rows / ((ms + bwd_ms) / 1e3), "unit": "rows/s", "ms_per_step": ms + bwd_ms,
        "dtype": "bf16", "timing": timing,
        "config": {"workload": "expert_ffn fwd+bwd: 16 groups x 2560 rows, M=2048, H=8192, 2 local experts, bias+GELU",
                   "l2": "1.2 GB touched per step exceeds the 126 MB L2"},
        "gpu_launches_per_step": int(launches), "clocks": clocks,
        "forward": {"ms_per_step": ms, "tflops": flops / (ms / 1e3) / 1e12, "frac_of_sustained": flops / (ms / 1e3) / 1e12 / sustained,
                    "what": "GEMM1 + bias + GELU (+ pre-activation copy), GEMM2 + bias"},
        "backward": {"ms_per_step": bwd_ms, "tflops": 2.0 * flops / (bwd_ms / 1e3) / 1e12,
                     "frac_of_sustained": 2.0 * flops / (bwd_ms / 1e3) / 1e12 / sustained, "timed_region_s": bwd_timing["timed_region_s"],
                     "what": "dH (NN, fused gelu'), dW2 (TN), dX (NN), dW1 (TN), db2, db1"},
        "library_gemm": {"ms_per_step": lib_ms, "tflops": flops / (lib_ms / 1e3) / 1e12, "what": "forward with torch.addmm + gelu (cuBLAS)"},
        # the two forward launches of the kernel in bursts (one event pair per burst) give its average launch duration; the
        # figure with an event pair around every launch, which adds the gap of two event records to each, is kept beside it
        "roofline": {"bound": "tensor", "kernel": "grouped_gemm_kernel (NT form: GEMM1 with bias + GELU + copy, GEMM2 with bias)",
                     "achieved": flops / (ms / 1e3) / 1e12, "peak": sustained, "unit": "TFLOP/s",
                     "frac": flops / (ms / 1e3) / 1e12 / sustained, "peak_kind": peak_kind + " (sustained cuBLAS bf16)",
                     "traffic": None, "flops_per_launch": flops / 2, "avg_launch_us": ms * 1e3 / 2,
                     "achieved_bracketed": ach, "frac_bracketed": ach / sustained, "bracketed_launch_us": avg_s * 1e6},
    }


# ---------------------------------------------------------------------------------------------------------------
# whole MoE layer
# ---------------------------------------------------------------------------------------------------------------
def leg_layer(args, ctx, steps):
    """Whole MoE layer, forward + backward: gate probabilities in, dispatch (+exchange), expert FFN (M=2048,
    H=8192, GELU, 2 local experts), combine (+exchange); backward with the weight-gradient GEMMs on a side stream
    under the returning exchange.  S=16384 tokens per GPU, top-2, capacity factor 1.25, bf16."""
    import lancet_b200 as LB
    from lancet_b200 import _capi
    rank, world, dev = ctx.rank, ctx.world, ctx.dev
    fabric = LB.LocalFabric(1, 0, {}) if world == 1 else None
    H = 8192
    xs_h, gates_h = synth_inputs(rank, world, S_TOKENS, M_DIM, torch.bfloat16)
    xs = [x.to(dev) for x in xs_h]
    gates = [g.to(dev) for g in gates_h]
    dout = torch.randn((S_TOKENS, M_DIM), device=dev).bfloat16()
    layer = LB.MoELayer(S_TOKENS, M_DIM, H, TOP_K, CAP_FACTOR, N_CHUNKS, torch.bfloat16, dev, 2, fabric=fabric, overlap_dw=True,
                        stages=args.stages, exchange_ctas=args.exchange_ctas, gemm_ctas=args.gemm_ctas)
    side = layer.side
    mode = {"v": "pipelined"}

    def step(i):
        if mode["v"] == "pipelined":
            layer.forward_pipelined(xs[i % 2], gates[i % 2])
            return layer.backward_pipelined(dout)
        layer.forward(xs[i % 2], gates[i % 2])
        return layer.backward(dout)

    def select(m):
        mode["v"] = m
        layer.side = side if m is True else None

    # the three schedules take turns in short bursts, so that clock drift under the power cap hits them alike
    order = {"all": ("pipelined", True, False), "staged": ("pipelined",), "side": (True,), "single": (False,)}[args.schedule]
    rounds = 5
    per_round = max(steps // rounds, 2)
    results = {m: [] for m in order}
    sampler = ClockSampler(ctx.local_rank) if rank == 0 else None
    for i in range(max(args.warmup, 3)):
        for m in order:
            select(m)
            step(i)
    region = 0.0
    for rnd in range(rounds):
        for m in order:
            select(m)
            step(0)
            ctx.sync()
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            ev0.record()
            for i in range(per_round):
                step(i)
            ev1.record()
            torch.cuda.synchronize()
            ms = ctx.max_over_ranks(ev0.elapsed_time(ev1) / per_round)
            results[m].append(ms)
            region += ms * per_round / 1e3
    clocks = ClockSampler.summarise(sampler.stop()) if sampler else None
    med = {m: statistics.median(v) for m, v in results.items()}
    # the schedules must agree bit for bit (same kernels on the same tiles, different order)
    identical = None
    if "pipelined" in order and len(order) > 1:
        select(order[1])
        o0 = layer.forward(xs[0], gates[0]).clone()
        dx0, dg0 = [t.clone() for t in layer.backward(dout)]
        w0 = [t.clone() for t in (layer.dw1, layer.dw2, layer.db1, layer.db2)]
        select("pipelined")
        o1 = layer.forward_pipelined(xs[0], gates[0])
        dx1, dg1 = layer.backward_pipelined(dout)
        torch.cuda.synchronize()
        identical = bool(torch.equal(o0, o1) and torch.equal(dx0, dx1) and torch.equal(dg0, dg1)
                         and all(torch.equal(a, b) for a, b in zip(w0, (layer.dw1, layer.dw2, layer.db1, layer.db2))))
        identical = ctx.all_true(identical)
    if world > 1:
        layer.moe.check()
    live = int(layer.moe.capused[-1].sum().item())
    st = LB.gemm_status(dev)
    _capi.check(_capi.lib().lancet_p2p_status(ctypes.c_void_p(st.data_ptr()),
                                              ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)))
    if world > 1:
        ctx.dist.barrier()
        layer.moe.close()
    ms = min(med.values())
    best = [m for m in order if med[m] == ms][0]
    flops = 6.0 * 2.0 * live * M_DIM * H            # per GPU: 2 GEMMs forward, 4 backward, live rows only
    peaks, peak_kind = load_peaks()
    sustained = float(peaks.get("bf16_tflops_sustained", FALLBACK_PEAKS["bf16_tflops"]))
    names = {"pipelined": "staged exchange (%d stages)" % args.stages, True: "dW on side stream", False: "single stream"}
    return {
        "metric": "moe_layer_tokens_per_s", "value": S_TOKENS * world / (ms / 1e3), "unit": "tokens/s", "ms_per_step": ms,
        "dtype": "bf16", "n_gpus": world,
        "config": {"workload": "moe_layer_fwd_bwd: S=%d tokens/GPU, M=%d, H=%d, E=%d, top-%d, cf=%.2f, %d chunks" % (
            S_TOKENS, M_DIM, H, 2 * world, TOP_K, CAP_FACTOR, N_CHUNKS), "l2": "GBs touched per step exceed the 126 MB L2"},
        "timing": {"rounds": rounds, "steps_per_round": per_round, "timed_region_s": region,
                   "what": "the schedules take turns in bursts; median burst per schedule, max over ranks"},
        "clocks": clocks, "tflops_per_gpu": flops / (ms / 1e3) / 1e12, "live_rows_rank0": live,
        "roofline": {"bound": "tensor", "kernel": "grouped_gemm_kernel (6 GEMMs of the layer; exchange hidden or exposed around them)",
                     "achieved": flops / (ms / 1e3) / 1e12, "peak": sustained, "unit": "TFLOP/s",
                     "frac": flops / (ms / 1e3) / 1e12 / sustained, "peak_kind": peak_kind + " (sustained cuBLAS bf16)",
                     "traffic": None, "flops_per_step": flops},
        "best_schedule": names[best],
        "schedules": {"pipeline_stages": args.stages, "exchange_ctas": args.exchange_ctas, "gemm_ctas": args.gemm_ctas,
                      "ms_pipelined_exchange": med.get("pipelined"),
                      "ms_dw_on_side_stream": med.get(True), "ms_single_stream": med.get(False),
                      "results_identical": identical},
    }


def run_single_leg(args, fn, needs_dist=False):
    ctx = Ctx(args)
    leg = fn(args, ctx, args.steps)
    world = ctx.world
    ctx.close()
    if ctx.rank == 0:
        emit(as_line(leg, args, world))


def run_peerbw(args):
    ctx = Ctx(args)
    if ctx.world < 2:
        raise SystemExit("bench.py --workload peerbw needs --gpus N >= 2 under torch.distributed.run")
    res = leg_peerbw(ctx)
    world = ctx.world
    ctx.close()
    if ctx.rank == 0:
        emit({"metric": "nvlink_peer_gb_per_s", "value": res["peak_gbs"], "unit": "GB/s per direction per GPU", "n_gpus": world,
              "steps": 10, "warmup": 2, "ms_per_step": res["bytes_out_per_gpu"] / res["peak_gbs"] / 1e6, "higher_is_better": True,
              "scaling": "weak", "vs_baseline": None, "dtype": "u8", "data": "synthetic",
              "config": {"workload": res["what"]}, "peerbw": res})


def run_a2a(args):
    """Stand-alone `_all_to_all` of the [E,C,M] expert buffer of the MoE workload (160 MiB per GPU): NCCL grouped
    send/recv exactly as the reference issues it, and the peer-memory store kernel + flag barrier."""
    import lancet_b200 as LB
    ctx = Ctx(args)
    rank, world, dev, dist = ctx.rank, ctx.world, ctx.dev, ctx.dist
    if world < 2:
        raise SystemExit("bench.py --workload a2a needs --gpus N >= 2 under torch.distributed.run")
    E = 2 * world
    C = LB.moe_capacity(S_TOKENS // N_CHUNKS, E, CAP_FACTOR * N_CHUNKS, TOP_K)
    x = torch.randn((E, C, M_DIM), device=dev).half()
    nbytes = x.numel() * 2
    comm = LB.Communicator(dev)
    sa = LB.SymmAllToAll(nbytes, dev)
    res = {}
    out = torch.empty_like(x)
    for name, fn in (("nccl", lambda: comm.all_to_all(x, out=out)), ("peer", lambda: sa.all_to_all(x))):
        for _ in range(max(args.warmup, 3)):
            fn()
        res[name], _ = timed_bursts(ctx, lambda: [fn() for _ in range(args.steps)], args.steps)
    ok = bool(torch.equal(sa.recv_view(x), comm.all_to_all(x)))
    sa.check()
    comm.close()
    dist.barrier()
    sa.close()
    peer = leg_peerbw(ctx)
    ctx.close()
    if rank != 0:
        return
    link_bytes = nbytes * (world - 1) / world          # bytes that leave each GPU per call
    ach = link_bytes / (res["peer"] / 1e3) / 1e9
    emit({
        "metric": "all_to_all_bus_gb_per_s", "value": ach, "unit": "GB/s per direction per GPU",
        "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": res["peer"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u8", "data": "synthetic",
        "config": {"workload": "all_to_all of the [E,C,M] fp16 expert buffer, %d bytes per GPU" % nbytes},
        "peer_memory": {"ms": res["peer"], "gb_per_s": ach},
        "nccl_grouped_send_recv": {"ms": res["nccl"], "gb_per_s": link_bytes / (res["nccl"] / 1e3) / 1e9},
        "results_identical": ok, "peerbw": peer,
        "roofline": {"bound": "nvlink", "kernel": "a2a_store_kernel", "achieved": ach,
                     "peak": peer["peak_gbs"], "unit": "GB/s", "frac": ach / peer["peak_gbs"],
                     "peak_kind": "measured in this run: all ranks to all peers, best of copy engines and store kernel",
                     "frac_of_nominal_900": ach / NVLINK_NOMINAL_GBS, "traffic": None},
    })


def run_gpt(args):
    """Full GPT-MoE training step (nl=12, m=1024, nh=16, sl=512, b=16 per GPU, vocab 50257, every other layer MoE with
    2N experts of FFN 4096, top-2, capacity factor 1.25, bf16 autocast, LANS).  Token ids are uniform random from a seed."""
    import lancet_b200 as LB
    from lancet_b200.gpt_moe import GPTMoE, LansTrainer
    ctx = Ctx(args)
    rank, world, dev = ctx.rank, ctx.world, ctx.dev
    fabric = LB.LocalFabric(1, 0, {}) if world == 1 else None
    vocab, m, nh, nl, seq, batch, ffn = 50257, 1024, 16, 12, 512, 16, 4096
    model = GPTMoE(vocab, m, nh, nl, seq, batch, ffn, 2 * world, TOP_K, CAP_FACTOR, N_CHUNKS, dev, fabric=fabric, seed=0,
                   act="relu", pipeline=not args.no_pipeline)     # the reference's GPT-2 blocks use ReLU
    trainer = LansTrainer(model, lr=1e-3, overlap_dw=not args.no_pipeline)
    g = torch.Generator(device=dev).manual_seed(1000 + rank)
    ids = [torch.randint(0, vocab, (batch, seq), device=dev, generator=g) for _ in range(2)]
    losses = []
    for i in range(max(args.warmup, 3)):
        losses.append(float(trainer.step(ids[i % 2])))
    ctx.sync()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for i in range(args.steps):
        loss = trainer.step(ids[i % 2])
    ev1.record()
    torch.cuda.synchronize()
    losses.append(float(loss))
    ms = ctx.max_over_ranks(ev0.elapsed_time(ev1) / args.steps)
    if world > 1:
        ctx.dist.barrier()
        model.close()
    ctx.close()
    if rank != 0:
        return
    n_params = sum(p.numel() for p in model.parameters())
    emit({
        "metric": "gpt_moe_tokens_per_s", "value": batch * seq * world / (ms / 1e3), "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "gpt2_moe_nl12_m1024_nh16_sl512_b16 training step, %d experts, top-2, cf 1.25, LANS" % (2 * world),
                   "params_per_rank": n_params, "pipelined_blocks": not args.no_pipeline},
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
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="moe", choices=["moe", "lans", "ffn", "gemm-forms", "layer", "a2a", "peerbw", "gpt"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-legs", action="store_true", help="moe workload: skip the lans / ffn / layer / peerbw legs")
    ap.add_argument("--no-graph", action="store_true", help="launch every step eagerly instead of replaying a CUDA graph")
    ap.add_argument("--schedule", default="all", choices=["all", "staged", "side", "single"],
                    help="layer workload: which schedules to time (all: the three take turns)")
    ap.add_argument("--stages", type=int, default=4, help="layer workload: exchange stages of the pipelined schedule")
    ap.add_argument("--exchange-ctas", type=int, default=0, help="layer workload, staged schedule: CTA cap of the exchange kernels")
    ap.add_argument("--gemm-ctas", type=int, default=0, help="layer workload, staged schedule: CTA cap of the expert GEMMs")
    ap.add_argument("--gemm-single", action="store_true", help="expert GEMMs: single-CTA 128x256 tiles instead of CTA pairs (A/B timing)")
    ap.add_argument("--plain-launches", action="store_true", help="dispatch path: plain kernel launches instead of programmatic stream serialization (A/B timing)")
    ap.add_argument("--no-pipeline", action="store_true", help="gpt workload: plain blocks (no chunked pipeline around the MoE layer)")
    ap.add_argument("--lans-layers", type=int, default=24, help="transformer layers in the LANS tensor list (24 = 196 tensors)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    if args.gemm_single:
        from lancet_b200 import _capi
        _capi.check(_capi.lib().lancet_set_gemm_paired(0))
    if args.plain_launches:
        from lancet_b200 import _capi
        _capi.check(_capi.lib().lancet_set_chained_launch(0))
    if args.workload == "lans":
        run_single_leg(args, leg_lans)
    elif args.workload == "ffn":
        run_single_leg(args, leg_ffn)
    elif args.workload == "gemm-forms":
        run_single_leg(args, leg_gemm_forms)
    elif args.workload == "layer":
        run_single_leg(args, leg_layer)
    elif args.workload == "a2a":
        run_a2a(args)
    elif args.workload == "peerbw":
        run_peerbw(args)
    elif args.workload == "gpt":
        run_gpt(args)
    else:
        run_moe(args)


if __name__ == "__main__":
    main()
