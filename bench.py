"""Benchmark of the packed decode-attention step (one layer, one query token per
sequence) on B200, with the roofline of its page-scan kernel and a CPU baseline.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload config2]
    python bench.py --impl reference ...      # CPU oracle port on the host cores

N > 1 is launched by torchrun, one rank per GPU; KV heads (and their query
heads) are sharded across ranks, each rank scans its own pages, and one
all-gather of the outputs closes the step.  Rank 0 prints one JSON line.

A step reads one layer's pages.  The pool holds several layers and consecutive
steps walk through them, so the bytes a step reads were last touched several
hundred MB ago: every step streams from HBM, not from L2.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

from winnow_b200 import workloads  # noqa: E402

METRIC = "packed_decode_attn_us_per_step"
NOMINAL_HBM_GBS = 8000.0
FALLBACK_HBM_GBS = 6650.0


def measured_peak():
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        try:
            return float(json.loads(f.read_text())["hbm_gbs"]), "measured"
        except Exception:                                   # noqa: BLE001
            pass
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while a region is being timed."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.path = index, None, None

    def __enter__(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-i", str(self.index), "-lms", "100"], stdout=fd, stderr=subprocess.DEVNULL)
            os.close(fd)
            # wait for the first sample: the tool's start-up (it attaches to every GPU
            # of the box) must be over before the timed region begins, or it can
            # stall launches inside a region that lasts only a few milliseconds
            deadline = time.time() + 5.0
            while time.time() < deadline and os.path.getsize(self.path) == 0:
                time.sleep(0.02)
            time.sleep(0.1)
        except Exception:                                   # noqa: BLE001
            self.proc = None
        return self

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:                               # noqa: BLE001
                self.proc.kill()

    def summary(self) -> dict:
        sm, mx, reasons = [], [], set()
        try:
            for line in Path(self.path).read_text().splitlines():
                f = [x.strip() for x in line.split(",")]
                if len(f) < 9:
                    continue
                sm.append(float(f[1]))
                mx.append(float(f[2]))
                for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown",
                                      "sw_power_cap"), f[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:                                   # noqa: BLE001
            pass
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        top = sorted(sm)[len(sm) // 2:]                      # the loaded half of the samples
        return {"sm_mhz": statistics.median(top), "sm_max_mhz": max(mx),
                "reasons": sorted(reasons), "samples": len(sm)}


# --------------------------------------------------------------------------
# distributed plumbing
# --------------------------------------------------------------------------
def init_ranks(gpus: int):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    elif gpus > 1:
        raise SystemExit("--gpus N > 1 must be launched with torch.distributed.run (one rank per GPU)")
    return rank, world, local


def barrier(world):
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
    torch.cuda.synchronize()


def max_over_ranks(x: float, world, dev) -> float:
    if world == 1:
        return x
    import torch.distributed as dist
    t = torch.tensor([x], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


# --------------------------------------------------------------------------
# workload construction (GPU arm)
# --------------------------------------------------------------------------
def build_gpu_cache(w, rank, world, layers, dev):
    """This rank's shard of the packed pool: kv heads [rank*Hkv/world, ...)."""
    from winnow_b200 import packed_attention as pa
    from winnow_b200.cache import _get_quantizer
    from winnow_b200.page_pool import PagePool

    if w.kv_heads % world:
        raise SystemExit(f"{w.kv_heads} kv heads do not shard over {world} ranks")
    hkv = w.kv_heads // world
    heads = slice(rank * hkv, (rank + 1) * hkv)
    kq = _get_quantizer(w.bits_k, w.head_dim, dev, 42)
    vq = _get_quantizer(w.bits_v, w.head_dim, dev, 43)
    table, total = workloads.page_assignment(w)
    S = w.page_size
    pool = PagePool(num_layers=layers, num_pages=total, num_kv_heads=hkv, page_size=S,
                    nb_k=w.head_dim * w.bits_k // 8, nb_v=w.head_dim * w.bits_v // 8, device=dev)
    lens = w.seq_lens()
    table_dev = table.to(dev)
    for b, L in enumerate(lens):
        k, v = workloads.dense_kv(w, b, heads)
        k, v = k.to(dev), v.to(dev)
        n_pg = -(-L // S)
        ids = table_dev[b, :n_pg].long()
        pad = n_pg * S - L
        for layer in range(layers):
            for dense, tq, pages, norms in ((k, kq, pool.k_pages, pool.k_norms),
                                            (v, vq, pool.v_pages, pool.v_norms)):
                # other layers hold the same vectors rotated along the token axis
                src = dense if layer == 0 else dense.roll(17 * layer, dims=1)
                codes, nrm = tq.quantize(src, packed=True)
                if pad:
                    codes = torch.nn.functional.pad(codes, (0, 0, 0, pad))
                    nrm = torch.nn.functional.pad(nrm, (0, pad))
                pages[layer][ids] = codes.view(hkv, n_pg, S, -1).permute(1, 0, 2, 3)
                norms[layer][ids] = nrm.to(torch.float16).view(hkv, n_pg, S).permute(1, 0, 2)
        del k, v
    seq = torch.tensor(lens, dtype=torch.int32, device=dev)
    handles = [pa.PackedKV(pool.k_pages[i], pool.k_norms[i], pool.v_pages[i], pool.v_norms[i],
                           table_dev, seq, pa.Quantizer.from_tq(kq), pa.Quantizer.from_tq(vq),
                           w.head_dim) for i in range(layers)]
    return pool, handles, (kq, vq)


def oracle_view(w, handle, seqs, kv_heads):
    """CPU oracle cache over the first `seqs` sequences of a GPU handle."""
    from oracle import tq_oracle as orc
    table = handle.page_table[:seqs].cpu()
    used = sorted({int(x) for x in table.flatten().tolist() if x >= 0})
    remap = {p: i for i, p in enumerate(used)}
    idx = torch.tensor(used, dtype=torch.long, device=handle.k_pages.device)
    small = table.clone()
    for r in range(small.shape[0]):
        for c in range(small.shape[1]):
            if small[r, c] >= 0:
                small[r, c] = remap[int(small[r, c])]
    return orc.OracleKV(handle.k_pages[idx][:, :kv_heads].cpu(), handle.k_norms[idx][:, :kv_heads].cpu(),
                        handle.v_pages[idx][:, :kv_heads].cpu(), handle.v_norms[idx][:, :kv_heads].cpu(),
                        small, handle.seq_lens[:seqs].cpu(),
                        handle.k_quant.Pi.cpu(), handle.k_quant.centroids.cpu(), handle.k_quant.bit_width,
                        handle.v_quant.Pi.cpu(), handle.v_quant.centroids.cpu(), handle.v_quant.bit_width,
                        handle.head_dim)


def time_cpu_port(q, okv, scale, reps):
    from oracle import tq_oracle as orc
    orc.tiled_attention(q, okv, scale)                       # warm-up
    t = []
    for _ in range(reps):
        t0 = time.perf_counter()
        orc.tiled_attention(q, okv, scale)
        t.append(time.perf_counter() - t0)
    return statistics.median(t)


# --------------------------------------------------------------------------
# arms
# --------------------------------------------------------------------------
def run_ours(args):
    """Main workload (the JSON line's top-level keys) and, unless `--extra none`,
    the other benchmark workloads measured the same way under `"workloads"`."""
    rank, world, local = init_ranks(args.gpus)
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    if args.only != "all":
        # one side measurement alone (what the ncu captures of those kernels run)
        if world != 1:
            raise SystemExit("--only dequant/prefill is a single-GPU measurement")
        if args.only == "dequant":
            print(json.dumps({"dequant": measure_dequant(dev)}))
        else:
            w = workloads.WORKLOADS[args.workload]
            pool, handles, _ = build_gpu_cache(w, 0, 1, 1, dev)
            us = time_prefill(w, handles[0], w.q_heads, w.head_dim ** -0.5, dev)
            print(json.dumps({"prefill_us": us, "query_tokens": PREFILL_Q, "workload": workload_label(w)}))
        return
    line = measure_workload(args.workload, args, rank, world, local, dev, main=True)
    extras = [] if args.extra in ("", "none") else [x for x in args.extra.split(",") if x]
    others = {}
    for name in extras:
        if name == args.workload or name not in workloads.WORKLOADS:
            continue
        w = workloads.WORKLOADS[name]
        if w.kv_heads % world:
            continue
        torch.cuda.empty_cache()
        r = measure_workload(name, args, rank, world, local, dev, main=False)
        if rank == 0:
            others[name] = r
    dequant = None
    if world == 1 and args.dequant:
        torch.cuda.empty_cache()
        dequant = measure_dequant(dev)
    if rank != 0:
        return
    if others:
        line["workloads"] = others
    if dequant is not None:
        line["dequant_gbs"] = dequant["gbs"]["tc"]
        line["dequant"] = dequant
    print(json.dumps(line))


def measure_workload(name, args, rank, world, local, dev, main):
    """One workload on this rank's shard: K timed steps (device resident, CUDA
    events, max over ranks), the scan kernel's own time, the end-to-end call
    with host buffers, parity against the CPU oracle.  Returns the JSON keys
    (rank 0; other ranks get None)."""
    from winnow_b200 import _lib
    from winnow_b200.packed_attention_cuda import (DecodePlan, decode_workspace,
                                                   packed_decode_attention)
    import ctypes

    w = workloads.WORKLOADS[name]
    lib = _lib.lib()
    hq = w.q_heads // world
    hkv = w.kv_heads // world
    per_layer = sum(w.seq_lens()) * hkv * w.bytes_per_token_head()
    layers = args.layers or max(2, min(16, -(-400_000_000 // max(per_layer, 1))))
    pool, handles, _ = build_gpu_cache(w, rank, world, layers, dev)
    scale = w.head_dim ** -0.5
    q_full = workloads.queries(w)
    q_host = q_full[:, rank * hq:(rank + 1) * hq].contiguous().pin_memory()
    q_dev = q_host.to(dev)
    B, D = w.batch, w.head_dim
    max_pages = handles[0].page_table.shape[1]
    ws = decode_workspace(B, hq, hkv, D, max_pages, w.page_size, args.splits, dev)
    gathered = torch.empty(world, B, hq, 1, D, dtype=w.dtype, device=dev)
    out_final = torch.empty(B, w.q_heads, 1, D, dtype=w.dtype, device=dev)
    out_host = torch.empty(B, w.q_heads, 1, D, dtype=w.dtype).pin_memory()
    if world > 1:
        import torch.distributed as dist

    target = out_final if world == 1 else gathered[rank]
    plans = [DecodePlan(q_dev, kv, scale, num_splits=args.splits, check_page_ids=False,
                        out=target, workspace=ws) for kv in handles]
    peer, exchange_note = None, "none"
    if world > 1:
        exchange_note = "nccl all_gather_into_tensor + permuting copy"
        if args.exchange == "peer":
            from winnow_b200 import tp
            why = ""
            try:
                peer = tp.PeerExchange(B, w.q_heads, D, w.dtype, dev)
                plans[0].run_exchange(peer.descriptor(), dry_run=True)
            except Exception as exc:                        # noqa: BLE001
                why = f"{type(exc).__name__}: {exc}"
            if tp._all_ranks_agree(why == "" and peer is not None, dev, None):
                exchange_note = "fused: merge kernel stores to every rank's buffer over NVLink + flag wait"
            else:
                peer = None
                exchange_note += f" (peer exchange unavailable on some rank{': ' + why if why else ''})"
    graphs = None
    if args.graph and peer is None:
        graphs = [pl.graph() for pl in plans]
    elif args.graph:
        # one graph per layer: fused decode + bounded wait; every capture and its
        # warm-up run is a real call of the exchange protocol on every rank
        graphs = []
        for pl in plans:
            pl.run_exchange(peer.descriptor()); peer.wait(); peer.step += 1
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                pl.run_exchange(peer.descriptor()); peer.wait()
            graphs.append(g)
        barrier(world)

    def gather():
        if world > 1:
            dist.all_gather_into_tensor(gathered.view(-1), gathered[rank].reshape(-1))
            out_final.view(B, world, hq, 1, D).copy_(gathered.permute(1, 0, 2, 3, 4))
        return out_final

    def direct_step(i):
        """Device-resident step issued call by call (pre-marshalled arguments)."""
        if peer is not None:
            peer.step += 1
            plans[i % layers].run_exchange(peer.descriptor())
            peer.wait()
            return peer.result(peer.step)
        plans[i % layers].run()
        return gather()

    def step(i):
        """Device-resident step: the CUDA graph of `direct_step` when enabled."""
        if graphs is None:
            return direct_step(i)
        graphs[i % layers].replay()
        if peer is not None:
            peer.step += 1
            return peer.result(peer.step)
        return gather()

    def api_step(i):
        """The call a user makes, arguments checked and marshalled every time."""
        if peer is not None:
            return step(i)
        packed_decode_attention(q_dev, handles[i % layers], scale, num_splits=args.splits,
                                check_page_ids=False, out=target, workspace=ws)
        return gather()

    # ---- parity against the oracle: the first sequence, every head of the FULL
    # (gathered) output of a step that used layer 0, checked on every rank
    parity = None
    if not args.no_check:
        from oracle import tq_oracle as orc
        got = step(0)                                       # layer 0
        torch.cuda.synchronize()
        full = got[:1].float().cpu().clone()
        okv = oracle_view(w, handles[0], 1, hkv)
        ref_local = orc.tiled_attention(q_full[:1, rank * hq:(rank + 1) * hq].float(), okv, scale)
        if world > 1:
            # every rank contributes the oracle rows of its own heads; the gathered
            # buffer of every rank must match the assembled reference
            parts = [torch.zeros_like(ref_local) for _ in range(world)]
            cpu_group = getattr(measure_workload, "_gloo", None)
            if cpu_group is None:
                cpu_group = dist.new_group(backend="gloo")
                measure_workload._gloo = cpu_group
            dist.all_gather(parts, ref_local.contiguous(), group=cpu_group)
            ref = torch.cat(parts, dim=1)
        else:
            ref = ref_local
        parity = max_over_ranks(float((full - ref).abs().max()), world, dev)

    steps = args.steps if main else max(args.steps, 100)
    for i in range(args.warmup):
        step(i)
    barrier(world)
    launches0 = lib.wtq_launch_count()
    plans[0].run()
    launches = (lib.wtq_launch_count() - launches0) * steps         # kernels of ours per step x K
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as clocks:
        barrier(world)                                       # every rank's sampler is up
        start.record()
        for i in range(steps):
            step(args.warmup + i)
        end.record()
        barrier(world)
        # the same K steps once more: a figure far from `value` means one of the two
        # regions was disturbed (they last only K x a few tens of microseconds)
        s1, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s1.record()
        for i in range(steps):
            step(args.warmup + i)
        e1.record()
        barrier(world)
        repeat_ms = max_over_ranks(s1.elapsed_time(e1) / steps, world, dev)
        steady_ms = None
        if main and steps < 200:
            # the same measurement over 200 steps (the K above may be a handful)
            s2, e2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s2.record()
            for i in range(200):
                step(args.warmup + i)
            e2.record()
            barrier(world)
            steady_ms = max_over_ranks(s2.elapsed_time(e2) / 200, world, dev)
        # second pass: same steps with events around the page-scan kernel only
        n_prof = max(steps, 100)
        lib.wtq_profile_enable(n_prof + 8)
        for i in range(n_prof):
            direct_step(args.warmup + i)
        torch.cuda.synchronize()
    k_ms, k_n = ctypes.c_double(0.0), ctypes.c_int(0)
    lib.wtq_profile_collect(ctypes.byref(k_ms), ctypes.byref(k_n))
    lib.wtq_profile_disable()
    ms = max_over_ranks(start.elapsed_time(end) / steps, world, dev)
    kernel_us = max_over_ranks(1e3 * k_ms.value / max(k_n.value, 1), world, dev)

    # ---- end to end through the public call with host buffers
    for i in range(min(args.warmup, 3)):
        api_step(i)
    barrier(world)
    e2e_steps = steps if main else min(steps, 50)
    t0 = time.perf_counter()
    for i in range(e2e_steps):
        q_dev.copy_(q_host, non_blocking=True)
        out_host.copy_(api_step(args.warmup + i), non_blocking=True)
        torch.cuda.synchronize()
    e2e_ms = max_over_ranks((time.perf_counter() - t0) * 1e3 / e2e_steps, world, dev)

    # ---- fused append of one token per sequence (reported beside the step)
    append_us = time_append(w, pool, handles, rank, world, dev, args)

    # ---- prefill chunk of 64 query tokens per sequence over this rank's pages
    prefill_us = time_prefill(w, handles[0], hq, scale, dev) if main else None
    if prefill_us is not None:
        prefill_us = max_over_ranks(prefill_us, world, dev)

    # ---- plain streaming read of this rank's pool: the read-only ceiling
    read_gbs = None
    if main:                                                 # slowest rank's figure
        read_gbs = -max_over_ranks(-time_stream_read(lib, pool.k_pages), world, dev)

    exchange_ok = True if peer is None else not peer.timed_out()
    exchange_ok = max_over_ranks(0.0 if exchange_ok else 1.0, world, dev) == 0.0
    cpu = None
    if main and rank == 0 and not args.no_cpu_baseline and world == 1:
        seqs = max(1, min(w.batch, args.cpu_seqs))
        okv = oracle_view(w, handles[0], seqs, hkv)
        t = time_cpu_port(q_full[:seqs, :hq].float(), okv, scale, reps=3)
        frac = (sum(w.seq_lens()[:seqs]) * hkv) / (sum(w.seq_lens()) * w.kv_heads)
        cpu = {"value": t * 1e6 / frac, "unit": "us", "cores": torch.get_num_threads(),
               "kind": "port",
               "sample": f"oracle tiled_attention, first {seqs} of {w.batch} sequences, "
                         f"{hkv} of {w.kv_heads} kv heads, median of 3, scaled by tokens"}
    del plans, graphs, pool, handles
    if rank != 0:
        return None
    peak, peak_kind = measured_peak()
    alg_total = w.algorithmic_bytes()
    alg_rank = w.algorithmic_bytes(kv_heads=hkv, q_heads=hq)
    achieved = alg_rank / (kernel_us * 1e-6) / 1e9
    ratio, ratio_source = dram_traffic_ratio(w.name, world)
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                "frac": achieved / peak, "frac_of_8tbs_nominal": achieved / NOMINAL_HBM_GBS,
                "traffic": alg_rank * ratio, "traffic_source": ratio_source, "peak_kind": peak_kind,
                "kernel": "page-scan kernel of wtq_decode", "kernel_us": kernel_us,
                "algorithmic_bytes_per_launch": alg_rank}
    if not main:
        return {"step_us": ms * 1e3, "repeat_us": repeat_ms * 1e3, "steps": steps, "e2e_us": e2e_ms * 1e3, "append_us": append_us,
                "hbm_gbs": alg_total / (ms * 1e-3) / 1e9, "roofline": roofline,
                "config": workload_label(w), "layers_rotated": layers,
                "parity_max_abs_err_vs_oracle": parity,
                "exchange_completed_without_timeout": exchange_ok}
    line = {
        "metric": METRIC, "value": ms * 1e3, "unit": "us", "n_gpus": world, "steps": steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": False, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_label(w),
                   "parallelism": f"kv-head tp{world}" if world > 1 else "single gpu",
                   "l2": f"steps rotate over {layers} layers of pages "
                         f"({layers * per_layer / 1e6:.0f} MB per GPU) so each step reads from HBM",
                   "num_splits": args.splits or "auto", "exchange": exchange_note,
                   "launch": "cuda graph replay" if args.graph else "pre-marshalled call"},
        "steady_us_over_200_steps": None if steady_ms is None else steady_ms * 1e3,
        "repeat_us": repeat_ms * 1e3,
        "hbm_gbs": alg_total / (ms * 1e-3) / 1e9,
        "hbm_frac_of_8tbs_nominal": alg_total / (ms * 1e-3) / 1e9 / (NOMINAL_HBM_GBS * world),
        "tokens_per_s": w.batch / (ms * 1e-3),
        "append_us": append_us,
        "prefill_us": prefill_us,
        "prefill": {"query_tokens": PREFILL_Q, "what": "packed_prefill_attention (wtq_prefill): the last "
                    f"{PREFILL_Q} tokens of every sequence attend causally over its packed history; "
                    "device time of the whole call (query permute, rotation, page scan, merge), "
                    "median of 5 after 2 warm-up calls"},
        "e2e": {"value": e2e_ms * 1e3, "unit": "us",
                "h2d_bytes_per_step": q_host.numel() * q_host.element_size(),
                "d2h_bytes_per_step": out_host.numel() * out_host.element_size()},
        "gpu_launches": int(launches),
        "roofline": roofline,
        "read_only_gbs": read_gbs,
        "cpu_baseline": cpu,
        "clocks": clocks.summary(),
        "parity_max_abs_err_vs_oracle": parity,
        "exchange_completed_without_timeout": exchange_ok,
    }
    return line


def workload_label(w) -> str:
    return (f"{w.name}: B{w.batch} Hq{w.q_heads} Hkv{w.kv_heads} D{w.head_dim} "
            f"ctx{w.context or 'ragged'} page{w.page_size} "
            f"{w.bits_k}-bit K/{w.bits_v}-bit V, q {str(w.dtype)[6:]}")


# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the scan kernel
# over its algorithmic bytes, from ncu captures of the named workloads (their
# summaries are kept under profiles/; the excess over 1 is the chunk states the
# kernel writes).  Other workloads and shards are scaled with the nearest entry.
DRAM_TRAFFIC_RATIO = {("config2", 1): (138.83 + 3.82) / 138.71,
                      ("config5", 1): (1114.06 + 23.03) / 1110.3,
                      ("headline32k", 1): (554.22 + 10.65) / 554.0}


def dram_traffic_ratio(name: str, world: int):
    if (name, world) in DRAM_TRAFFIC_RATIO:
        return DRAM_TRAFFIC_RATIO[(name, world)], f"ncu capture of the scan kernel on {name}, {world} GPU(s)"
    return DRAM_TRAFFIC_RATIO[("config2", 1)], ("scaled: ratio of an ncu capture on config2, 1 GPU "
                                               "(not captured for this workload/shard)")


def time_stream_read(lib, tensor) -> float:
    """GB/s of a plain streaming read (wtq_probe_read) over `tensor`'s storage."""
    flat = tensor.reshape(-1)
    nbytes = flat.numel() * flat.element_size() // 16 * 16
    sink = torch.zeros(1, dtype=torch.int32, device=tensor.device)
    stream = torch.cuda.current_stream(tensor.device).cuda_stream
    for _ in range(3):
        lib.wtq_probe_read(flat.data_ptr(), nbytes, sink.data_ptr(), stream)
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(10):
        lib.wtq_probe_read(flat.data_ptr(), nbytes, sink.data_ptr(), stream)
    e.record()
    torch.cuda.synchronize()
    return nbytes * 10 / (s.elapsed_time(e) * 1e-3) / 1e9


def measure_dequant(dev) -> dict:
    """Fused dequantisation (wtq_dequant_mode) of 2^20 packed 4-bit rows, the K
    side of 8 sequences x 4 kv heads x 32k tokens, to bf16: 64 B of codes and a
    2 B norm in, 256 B out per row, 338 MB per call (larger than L2, so every
    call streams from and to HBM).  Device time per call from CUDA events."""
    from winnow_b200.cache import _get_quantizer, dequantize_rows
    rows = 1 << 20
    tq = _get_quantizer(4, 128, dev, 42)
    g = torch.Generator(device=dev).manual_seed(5)
    packed = torch.randint(0, 256, (rows, 64), dtype=torch.uint8, device=dev, generator=g)
    norms = (torch.rand(rows, device=dev, generator=g) * 4 + 0.5).half()
    outs = {}
    nbytes = rows * (64 + 2 + 256)
    peak, kind = measured_peak()
    result = {"rows": rows, "bits": 4, "out_dtype": "bf16", "bytes_per_call": nbytes, "us": {}, "gbs": {},
              "modes": {"tc": "tcgen05 (accumulator in tensor memory), fp16 high/low split operands: what "
                              "bf16/fp16 outputs get by default",
                        "tc_fast": "tcgen05, single fp16 operands (the reference's allow_tf32 class)",
                        "tc_mma": "the split form on mma.sync (the fallback of tc)",
                        "tc_fast_mma": "the single form on mma.sync (the fallback of tc_fast)",
                        "exact": "fp32 on the CUDA cores"}}
    for mode, reps in (("tc", 20), ("tc_fast", 20), ("tc_mma", 20), ("tc_fast_mma", 20), ("exact", 3)):
        out = torch.empty(rows, 128, dtype=torch.bfloat16, device=dev)
        for _ in range(3):
            dequantize_rows(packed, norms, tq.centroids, tq.Pi, 4, 128, out=out, mode=mode)
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(reps):
            dequantize_rows(packed, norms, tq.centroids, tq.Pi, 4, 128, out=out, mode=mode)
        e.record()
        torch.cuda.synchronize()
        us = s.elapsed_time(e) * 1e3 / reps
        result["us"][mode] = us
        result["gbs"][mode] = nbytes / (us * 1e-6) / 1e9
        outs[mode] = out
    exact = outs["exact"].float()
    top = float(exact.abs().max())
    result["max_abs_diff_vs_exact_over_max"] = {m: float((outs[m].float() - exact).abs().max()) / top
                                                for m in ("tc", "tc_fast", "tc_mma", "tc_fast_mma")}
    result["frac_of_hbm_peak"] = result["gbs"]["tc"] / peak
    result["peak_kind"] = kind
    return result


PREFILL_Q = 64


def time_prefill(w, handle, hq, scale, dev):
    """Median device time (us) of one chunked-prefill call at PREFILL_Q query
    tokens per sequence over `handle`'s pages, or None if the chunk kernel does
    not serve this layout."""
    from winnow_b200.packed_attention_cuda import packed_prefill_attention, prefill_supported
    g = torch.Generator().manual_seed(w.seed + 64)
    # queries drawn like the decode step's (workloads.queries): N(0, 1) / sqrt(head_dim)
    q = (torch.randn(w.batch, hq, PREFILL_Q, w.head_dim, generator=g) * w.head_dim ** -0.5).to(dev, w.dtype)
    if not prefill_supported(q, handle):
        return None
    times = []
    for i in range(2 + 5):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        packed_prefill_attention(q, handle, scale, check_page_ids=False)
        e.record()
        torch.cuda.synchronize()
        if i >= 2:
            times.append(s.elapsed_time(e) * 1e3)
    return statistics.median(times)


def _first_seq(handle):
    from winnow_b200 import packed_attention as pa
    return pa.PackedKV(handle.k_pages, handle.k_norms, handle.v_pages, handle.v_norms,
                       handle.page_table[:1].contiguous(), handle.seq_lens[:1].contiguous(),
                       handle.k_quant, handle.v_quant, handle.head_dim)


def time_append(w, pool, handles, rank, world, dev, args):
    """Median time of the fused append of one new token per sequence.  The
    tokens overwrite the last stored position of every sequence with the vector
    already there, so the cache the decode step reads is unchanged."""
    from winnow_b200.cache import _get_quantizer
    hkv = w.kv_heads // world
    kq = _get_quantizer(w.bits_k, w.head_dim, dev, 42)
    vq = _get_quantizer(w.bits_v, w.head_dim, dev, 43)
    k, v = workloads.new_tokens(w)
    k = k[:, rank * hkv:(rank + 1) * hkv].to(dev)
    v = v[:, rank * hkv:(rank + 1) * hkv].to(dev)
    spare = pool.k_pages.shape[0] - 1                          # scratch layer: the last one
    kv = handles[spare]
    from winnow_b200.packed_backend import AppendPlan
    plan = AppendPlan(k, v, kv.k_pages, kv.k_norms, kv.v_pages, kv.v_norms, kv.page_table,
                      kv.seq_lens, kq, vq)
    times = []
    for i in range(3 + 7):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(20):                                    # back to back: device time per append
            plan.run()
        e.record()
        torch.cuda.synchronize()
        if i >= 3:
            times.append(s.elapsed_time(e) * 1e3 / 20)
    return statistics.median(times)


def run_reference(args):
    """The reference's CPU implementation of the step, as restated by the
    oracle, on the host cores.  Rank 0 only."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    from oracle import tq_oracle as orc
    # torchrun pins OMP_NUM_THREADS=1 for its children; the CPU arm is entitled to
    # every host core
    torch.set_num_threads(os.cpu_count() or 1)
    w = workloads.WORKLOADS[args.workload]
    seqs = max(1, min(w.batch, args.cpu_seqs))
    kq = orc.OracleQuantizer.get(w.bits_k, w.head_dim, 42)
    vq = orc.OracleQuantizer.get(w.bits_v, w.head_dim, 43)
    lens = w.seq_lens()[:seqs]
    ctx = min(max(lens), args.cpu_context)
    lens = [min(L, ctx) for L in lens]
    k = torch.zeros(seqs, w.kv_heads, ctx, w.head_dim)
    v = torch.zeros_like(k)
    for b in range(seqs):
        kb, vb = workloads.dense_kv(w, b)
        k[b, :, :lens[b]], v[b, :, :lens[b]] = kb[:, :lens[b]].float(), vb[:, :lens[b]].float()
    okv = orc.pages_from_dense(k, v, lens, kq, vq, w.page_size,
                               generator=torch.Generator().manual_seed(w.seed))
    q = workloads.queries(w)[:seqs].float()
    scale = w.head_dim ** -0.5
    for _ in range(min(args.warmup, 2)):
        orc.tiled_attention(q, okv, scale)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        orc.tiled_attention(q, okv, scale)
    per_step = (time.perf_counter() - t0) / args.steps
    frac = sum(lens) / sum(w.seq_lens())
    us = per_step * 1e6 / frac
    sample = (f"oracle port of tiled_compressed_attention on {seqs} of {w.batch} sequences at "
              f"context {ctx}, all {w.kv_heads} kv heads; time scaled by cached tokens to the full "
              "workload")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": us, "unit": "us",
        "n_gpus": int(os.environ.get("WORLD_SIZE", "1")), "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": us / 1e3, "higher_is_better": False, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"{w.name}: B{w.batch} Hq{w.q_heads} Hkv{w.kv_heads} D{w.head_dim} "
                               f"ctx{w.context or 'ragged'} page{w.page_size} "
                               f"{w.bits_k}-bit K/{w.bits_v}-bit V, q {str(w.dtype)[6:]}",
                   "parallelism": "host cpu"},
        "cpu_baseline": {"value": us, "unit": "us", "cores": torch.get_num_threads(), "kind": "port",
                         "sample": sample},
        "e2e": {"value": us, "unit": "us", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="config2", choices=sorted(workloads.WORKLOADS))
    ap.add_argument("--only", default="all", choices=["all", "dequant", "prefill"],
                    help="run just the dequantisation or the prefill measurement (single GPU)")
    ap.add_argument("--dequant", type=int, default=1,
                    help="1: also time the fused dequantisation kernels (single GPU only)")
    ap.add_argument("--extra", default="headline32k,config3,config4,config5",
                    help="comma list of further workloads reported under \"workloads\" (or none)")
    ap.add_argument("--layers", type=int, default=0, help="layers of pages to rotate over (0=auto)")
    ap.add_argument("--splits", type=int, default=0, help="split-K factor (0 = library's choice)")
    ap.add_argument("--cpu-seqs", type=int, default=2)
    ap.add_argument("--cpu-context", type=int, default=8192)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-check", action="store_true")
    ap.add_argument("--graph", action=argparse.BooleanOptionalAction, default=True,
                    help="replay each step as a CUDA graph (default) or issue the calls directly")
    ap.add_argument("--exchange", default="peer", choices=["peer", "nccl"],
                    help="multi-GPU output exchange: fused peer stores, or NCCL all-gather")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)
    if int(os.environ.get("WORLD_SIZE", "1")) > 1:
        import torch.distributed as dist
        if dist.is_initialized():
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
