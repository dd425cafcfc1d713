#!/usr/bin/env python
"""Benchmark of the sparse top-k global-attention path (indexer score + exact top-k + sparse attention).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload vggt32|pi3_64|ctx256|small] [--impl ours|reference]

One step = the path applied to every sparse global layer of the workload (VGGT 32 views: 11 layers of
N = 33312 tokens, k = 1024, 16x64 attention heads, 4x64 indexer heads, bf16), each layer with its own
synthetic ~N(0,1) inputs at the operator boundary.  With N > 1 GPUs the same global problem is split by
query rows (strong scaling); per layer every rank all-gathers K, V, K_idx and w and nothing else.

Prints ONE JSON line.  `value` = token-layer passes per second with inputs resident in HBM; `e2e` = the
same through the public Python API with pinned-host inputs copied in and outputs copied out every step.
`--impl reference` times the reference's CPU (`--backend torch`) op sequence on the host cores instead.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

WORKLOADS = {
    # name: (views, tokens/view, layers, description)
    "vggt32": (32, 1041, 11, "VGGT global layers 9-19, 32 views of 37x28 patches + 5 special tokens"),
    "pi3_64": (64, 782, 9, "Pi3 sparse global layers 9-17, 64 views of 37x21 patches + 5 register tokens"),
    "ctx256": (256, 1041, 1, "one VGGT-shaped layer over a 256-view context"),
    "small": (4, 1041, 2, "4 views (reference's CPU-runnable size), 2 layers"),
}
H, D, HI, DI, TOPK = 16, 64, 4, 64, 1024
METRIC = "global-attn tokens/s (indexer+top-k+sparse attn)"
UNIT = "tokens/s"


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default="vggt32", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--cpu-rows", type=int, default=1024, help="query rows per CPU-baseline sample")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--layers", type=int, default=0, help="override the number of layers per step (profiling)")
    ap.add_argument("--profile", action="store_true", help="profiling run: exact --warmup, no e2e pass, no CPU arm")
    ap.add_argument("--gather", choices=("group", "packed", "peer"), default="peer",
                    help="N > 1: how K_idx with w, and K with V, reach every rank: pulled from peer memory behind a flag barrier "
                         "(PeerExchange, default; NCCL packed where peer-mapped memory cannot be set up), one NCCL all-gather of the "
                         "pair packed side by side, or one coalesced NCCL group into separate tensors")
    ap.add_argument("--no-extra-legs", action="store_true",
                    help="skip the legs measured after the main region (attention in the HBM regime, the 256-view context, "
                         "operator inputs from the reference's projections)")
    ap.add_argument("--attn-bwd", action="store_true",
                    help="run only the attention backward on 8192 query rows of the main workload's shape (for profiler captures)")
    ap.add_argument("--attn-hbm", action="store_true",
                    help="run only the attention kernel in the regime where HBM binds (8192 queries, k = 1024, positions uniformly "
                         "random over 266496 keys: K + V = 1.09 GB) and print one JSON line; small enough for an ncu capture")
    ap.add_argument("--micro", action="store_true",
                    help="instead of the path, time the stand-alone operators (exact top-k of materialised scores, merge of "
                         "two lists, scalar attention kernels) and print one JSON line with their roofline fractions")
    return ap.parse_args()


def config_of(args, n_tokens, layers, desc, world):
    return {"workload": f"{args.workload}: {desc}", "tokens": n_tokens, "layers_per_step": layers, "topk": TOPK,
            "attn_heads": H, "head_dim": D, "indexer_heads": HI, "indexer_dim": DI,
            "partition": f"query rows over {world} GPU(s); all-gather of K,V,K_idx,w per layer" if world > 1 else "single GPU",
            "l2": "per-layer inputs (>= 230 MB for vggt32) exceed the 126 MB L2 and layers rotate; no explicit flush"}


# ---------------------------------------------------------------------------------------------------
# CPU arm: the reference's torch-backend op sequence on a bounded sample of query rows
# ---------------------------------------------------------------------------------------------------
def cpu_reference_tokens_per_s(n_tokens, rows, repeats, seed=7):
    """Time the reference's CPU (`--device cpu --backend torch`) arithmetic of the path on `rows` query rows of one
    layer with all keys resident.  With the staged copy of the reference present (baseline/_ref) its own functions
    run -- LightningIndexer.select_topk_projected and DSAAttention._sparse_attention, fp32 (kind "reference");
    otherwise the oracle's port of the same op sequence (kind "port")."""
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    g = torch.Generator().manual_seed(seed)
    q_idx = torch.randn(1, n_tokens, HI, DI, generator=g)
    k_idx = torch.randn(1, n_tokens, HI, DI, generator=g)
    w = torch.rand(1, n_tokens, HI, generator=g)
    q = torch.randn(1, H, n_tokens, D, generator=g)
    k = torch.randn(1, H, n_tokens, D, generator=g)
    v = torch.randn(1, H, n_tokens, D, generator=g)
    rows = min(rows, n_tokens)
    kind = "port"
    try:
        from baseline import ref_harness as rh

        if rh.available():
            rh.enable_import()
            from easyvolcap.official_vggt.layers.dsa_attention import DSAAttention

            attn = DSAAttention(H * D, num_heads=H, qk_norm=True, indexer_cfg=rh.indexer_cfg(TOPK, "torch")).eval()

            def one(sl):
                idx = attn.indexer.select_topk_projected(q_idx[:, sl], k_idx, w, topk=TOPK, return_scores=False)
                attn._sparse_attention(q[:, :, sl], k, v, idx, None)

            kind = "reference"
    except Exception as exc:  # a broken staging area must not take the GPU arm's line with it
        print(f"[bench] reference import failed, timing the port instead: {exc!r}", file=sys.stderr)
    if kind == "port":
        from oracle import gw_oracle as orc

        def one(sl):
            orc.reference_cpu_path(q_idx, k_idx, w, q, k, v, TOPK, DI ** -0.5, D ** -0.5, sl)

    times = []
    with torch.no_grad():
        for i in range(repeats + 1):
            lo = (i * rows) % max(1, n_tokens - rows + 1)
            t0 = time.perf_counter()
            one(slice(lo, lo + rows))
            times.append(time.perf_counter() - t0)
    times = times[1:] if len(times) > 1 else times  # first call warms the allocator
    per = statistics.median(times)
    sample = f"{rows} query rows of one layer with all {n_tokens} keys resident, fp32, median of {len(times)}"
    return rows / per, threads, per, sample, kind


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    views, tpv, layers, desc = WORKLOADS[args.workload]
    n_tokens = views * tpv
    t0 = time.perf_counter()
    tps, threads, per, sample, kind = cpu_reference_tokens_per_s(n_tokens, args.cpu_rows, max(1, args.steps))
    line = {"impl": "reference", "metric": METRIC, "value": tps, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": n_tokens * layers / tps * 1e3, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": config_of(args, n_tokens, layers, desc, 1),
            "cpu_baseline": {"value": tps, "unit": UNIT, "cores": threads, "kind": kind, "sample": sample},
            "e2e": {"value": tps, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "note": ("the reference's own LightningIndexer.select_topk_projected + DSAAttention._sparse_attention "
                     "(its `--device cpu --backend torch` arithmetic) from the staged copy under baseline/_ref"
                     if kind == "reference" else
                     "no staged copy of the reference here: a port of the op sequence its `--device cpu --backend torch` "
                     "path executes (same ATen ops)") + ", all host threads; ms_per_step is extrapolated linearly in rows x layers",
            "wall_s": time.perf_counter() - t0}
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------------
# clocks sampler
# ---------------------------------------------------------------------------------------------------
class Clocks:
    Q = "clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown," \
        "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index):
        self.samples = []
        self.proc = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) >= 7:
                self.samples.append((time.perf_counter(), parts))

    def stop(self, t_begin, t_end):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        rows = [p for (t, p) in self.samples if t_begin <= t <= t_end] or [p for (_, p) in self.samples]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        sm = [float(r[0]) for r in rows if r[0].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[3 + i].lower().startswith("active") for r in rows)]
        pw = [float(r[2]) for r in rows if r[2].replace(".", "").isdigit()]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": float(rows[0][1]) if rows[0][1].isdigit() else None,
                "power_w_max": max(pw) if pw else None, "samples": len(rows), "reasons": reasons}


# ---------------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------------
def bind_host_thread_near_gpu(dev) -> str:
    """Run this process (and place its pinned buffers) on the CPUs next to its GPU.  With one rank per GPU the
    host->device copies of all ranks run at once; a rank whose pinned pages sit on the other socket copies at a
    fraction of the link rate.  Only reads the topology (NVML) and sets this process's own CPU affinity."""
    try:
        import pynvml

        pynvml.nvmlInit()
        uuid = str(torch.cuda.get_device_properties(dev).uuid)
        handle = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid) if not uuid.startswith("GPU-") else uuid)
        n_cpu = os.cpu_count() or 1
        mask = pynvml.nvmlDeviceGetCpuAffinity(handle, (n_cpu + 63) // 64)
        near = {i for i in range(n_cpu) if (int(mask[i // 64]) >> (i % 64)) & 1}
        allowed = os.sched_getaffinity(0)
        pick = near & allowed
        if pick and pick != allowed:
            os.sched_setaffinity(0, pick)
            return f"{len(pick)} of {len(allowed)} CPUs"
        return "unchanged"
    except Exception as exc:  # no NVML, no permission: measure where we are
        return f"unavailable ({type(exc).__name__})"


def run_ours(args):
    import torch.distributed as dist

    import geoweave_b200
    from geoweave_b200 import _lib
    from geoweave_b200.custom_flash_attn import sparse_index_flash_attn_inference_func
    from geoweave_b200.custom_indexer import sparse_topk_indexer_inference_func
    from geoweave_b200.coarse_to_fine import select_topk_coarse_to_fine, source_layout
    from geoweave_b200.sharding import gather_rows_group, gather_rows_packed, row_partition

    _lib.load()  # fail loudly if the CUDA library is missing: there is no other path
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    host_binding = bind_host_thread_near_gpu(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    views, tpv, layers, desc = WORKLOADS[args.workload]
    if args.layers > 0:
        layers = args.layers
    n_tokens = views * tpv
    lo, hi = row_partition(n_tokens, world)[rank]
    rows = hi - lo
    bf = torch.bfloat16

    # per-layer inputs of this rank's token shard, on pinned host memory and resident on the device
    host, resident = [], []
    for layer in range(layers):
        g = torch.Generator().manual_seed(1234 + 1000 * layer + rank)
        t = {"q_idx": torch.randn(1, rows, HI, DI, generator=g).to(bf), "k_idx": torch.randn(1, rows, HI, DI, generator=g).to(bf),
             "w": torch.rand(1, rows, HI, generator=g).to(bf), "q": torch.randn(1, rows, H, D, generator=g).to(bf),
             "k": torch.randn(1, rows, H, D, generator=g).to(bf), "v": torch.randn(1, rows, H, D, generator=g).to(bf)}
        t = {n: x.pin_memory() for n, x in t.items()}
        host.append(t)
        resident.append({n: x.to(dev) for n, x in t.items()})
    out_host = [torch.empty((1, rows, H, D), dtype=bf).pin_memory() for _ in range(layers)]
    # end-to-end arm: two device staging sets so that the copy of layer i+1 overlaps the kernels of layer i
    staging = [{n: torch.empty_like(x, device=dev) for n, x in host[0].items()} for _ in range(2)]
    copy_in, copy_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    h2d = sum(x.numel() * x.element_size() for t in host for x in t.values())
    d2h = sum(x.numel() * x.element_size() for x in out_host)

    ev = lambda: torch.cuda.Event(enable_timing=True)
    stage_events = []  # (start, after indexer, after attention) per layer call, only while timing

    last = {}          # tensors of the most recent recorded layer call (for the bare-gather ceiling)

    use_peer, peer_error = False, None
    if args.gather == "peer" and world > 1:
        from geoweave_b200.sharding import PeerExchange

        # one object per exchange (each alternates its own buffer halves): K_idx, w by one pull kernel in front of the indexer;
        # K, V by copy engines beside it.  Where peer-mapped memory cannot be set up, every rank falls back to NCCL.
        try:
            ex_idx = PeerExchange(device=dev, pull="kernel")
            ex_kv = PeerExchange(device=dev, pull="copies", copy_streams=4)
            ok = torch.ones(1, device=dev)
        except Exception as exc:
            ok = torch.zeros(1, device=dev)
            peer_error = f"{type(exc).__name__}: {exc}"
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        use_peer = bool(ok.item())
        if not use_peer and peer_error is None:
            peer_error = "another rank could not set up peer-mapped memory"
    if use_peer:
        gather_idx, gather_kv = ex_idx.gather, ex_kv.gather
        # before anything is timed: three exchanges in a row (both halves of the buffers) must give what NCCL gives
        for layer in range(3):
            tt = resident[layer % layers]
            want = [x.contiguous() for x in gather_rows_packed([tt["k"], tt["v"]], n_tokens).result()]
            got = ex_kv.gather([tt["k"], tt["v"]], n_tokens, async_op=True).result()
            want_i = [x.contiguous() for x in gather_rows_packed([tt["k_idx"], tt["w"]], n_tokens).result()]
            got_i = ex_idx.gather([tt["k_idx"], tt["w"]], n_tokens).result()
            torch.cuda.synchronize()
            if not all(torch.equal(a, b) for a, b in zip(want + want_i, got + got_i)):
                raise RuntimeError("PeerExchange.gather disagrees with the NCCL all-gather")
        geoweave_b200.check_status()
    else:
        gather_idx = gather_kv = gather_rows_group if args.gather == "group" else gather_rows_packed

    def layer_op(t, record, n_tok=n_tokens, events=None, layout=None):
        if record:
            eg, e0, e1, ek, e2 = ev(), ev(), ev(), ev(), ev()
            eg.record()
        if world > 1:  # the indexer needs K_idx and w; K and V are gathered behind it
            k_idx, w = [x.contiguous() for x in gather_idx([t["k_idx"], t["w"]], n_tok).result()]
            kv_pend = gather_kv([t["k"], t["v"]], n_tok, async_op=True)
        else:
            k_idx, w, k, v = t["k_idx"], t["w"], t["k"], t["v"]
        if record:
            e0.record()
        if layout is not None:  # coarse-to-fine selection over 2x2-pooled sources instead of the full-resolution indexer
            idx = select_topk_coarse_to_fine(t["q_idx"], k_idx, w, layout, TOPK, DI ** -0.5)
        else:
            idx, _ = sparse_topk_indexer_inference_func(t["q_idx"], k_idx, w, None, TOPK, DI ** -0.5, 0, 0, return_scores=False)
        if record:
            e1.record()
        if world > 1:
            k, v = kv_pend.result()
        if record:
            ek.record()
        out, _ = sparse_index_flash_attn_inference_func(t["q"], k, v, idx, None, False, D ** -0.5, False)
        if record:
            e2.record()
            (stage_events if events is None else events).append((e0, e1, e2, eg, ek))
            last.update(idx=idx, k=k, v=v)
        return out

    def step_resident(record=False):
        for layer in range(layers):
            layer_op(resident[layer], record)

    enqueue_s = []  # host time spent enqueueing one end-to-end step (a step cannot be faster than this)
    timeline = {} if os.environ.get("GW_BENCH_TIMELINE") == "1" else None

    def step_e2e():
        """Every layer: pinned host inputs -> device (copy stream), the three stages (main stream), output ->
        pinned host (second copy stream).  The copy of layer i+1 is ENQUEUED before the kernels of layer i, so it
        overlaps them whether or not the host thread runs ahead of the device."""
        t_host = time.perf_counter()
        main = torch.cuda.current_stream(dev)
        used = [None, None]    # event: kernels that read staging set i have finished
        ready = [None, None]   # event: staging set i holds its layer's inputs

        def enqueue_copy_in(layer):
            st = staging[layer & 1]
            with torch.cuda.stream(copy_in):
                if used[layer & 1] is not None:
                    copy_in.wait_event(used[layer & 1])
                if timeline is not None:
                    timeline.setdefault(layer, {})["h2d0"] = ev()
                    timeline[layer]["h2d0"].record(copy_in)
                for n, x in host[layer].items():
                    st[n].copy_(x, non_blocking=True)
                ready[layer & 1] = ev() if timeline is not None else torch.cuda.Event()
                ready[layer & 1].record(copy_in)
                if timeline is not None:
                    timeline[layer]["h2d1"] = ready[layer & 1]

        enqueue_copy_in(0)
        for layer in range(layers):
            main.wait_event(ready[layer & 1])
            if layer + 1 < layers:
                enqueue_copy_in(layer + 1)  # the other staging set: free once layer - 1 has finished
            if timeline is not None:
                timeline[layer]["c0"] = ev()
                timeline[layer]["c0"].record(main)
            out = layer_op(staging[layer & 1], False)
            done = ev() if timeline is not None else torch.cuda.Event()
            done.record(main)
            if timeline is not None:
                timeline[layer]["c1"] = done
            used[layer & 1] = done
            with torch.cuda.stream(copy_out):
                copy_out.wait_event(done)
                out_host[layer].copy_(out, non_blocking=True)
                out.record_stream(copy_out)
        enqueue_s.append(time.perf_counter() - t_host)
        torch.cuda.synchronize()
        if timeline is not None and rank == 0:  # GW_BENCH_TIMELINE=1: device times of one step, ms from its first copy
            t0 = timeline[0]["h2d0"]
            for layer in range(layers):
                e = timeline[layer]
                print(f"[timeline] layer {layer}: copy-in {t0.elapsed_time(e['h2d0']):.2f}-{t0.elapsed_time(e['h2d1']):.2f}  "
                      f"kernels {t0.elapsed_time(e['c0']):.2f}-{t0.elapsed_time(e['c1']):.2f}", file=sys.stderr, flush=True)
            timeline.clear()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        barrier()
        a, b = ev(), ev()
        a.record()
        for _ in range(steps):
            fn()
        b.record()
        barrier()
        ms = torch.tensor([a.elapsed_time(b)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    n_warm = args.warmup if args.profile else max(3, args.warmup)
    for _ in range(n_warm):
        step_resident()
    geoweave_b200.check_status()
    clocks = Clocks(local) if rank == 0 else None
    t_begin = time.perf_counter()
    ms_total = timed(lambda: step_resident(True), args.steps)
    t_end = time.perf_counter()
    h2d_gbs = None
    if args.profile:
        ms_e2e = float("nan")
    else:
        step_e2e()
        ms_e2e = timed(step_e2e, args.steps)

        def copies_only():  # the same host->device copies with nothing else running: the link rate this rank gets
            with torch.cuda.stream(copy_in):
                for layer in range(layers):
                    for n, x in host[layer].items():
                        staging[layer & 1][n].copy_(x, non_blocking=True)
            torch.cuda.synchronize()

        ms_copy = timed(copies_only, 2) / 2
        h2d_gbs = h2d / ms_copy / 1e6
    geoweave_b200.check_status()
    clk = clocks.stop(t_begin, time.perf_counter()) if clocks else None

    idx_ms = statistics.mean(e[0].elapsed_time(e[1]) for e in stage_events)
    att_ms = statistics.mean(e[4].elapsed_time(e[2]) for e in stage_events)       # the attention launch alone
    kidx_gather_ms = statistics.mean(e[3].elapsed_time(e[0]) for e in stage_events)  # K_idx and w arriving, in front of the indexer
    kv_wait_ms = statistics.mean(e[1].elapsed_time(e[4]) for e in stage_events)      # what of the K, V gather the indexer did not cover
    lib = _lib.load()
    launches = layers * (lib.gw_indexer_topk_launch_count(1, rows, n_tokens, TOPK) + 1)
    if use_peer:
        launches += layers * 3  # per layer: the two exchanges' barrier kernels and the pull kernel of K_idx, w
    es = 2

    def attn_bytes_of(n_rows):
        """Algorithmic bytes of one attention launch: gathered K and V rows, the index list, q and the output."""
        return n_rows * (TOPK * 2 * H * D * es + TOPK * 4 + 2 * H * D * es)

    def time_ms(fn, warm, reps):
        for _ in range(warm):
            fn()
        torch.cuda.synchronize()
        a, b = ev(), ev()
        a.record()
        for _ in range(reps):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / reps

    def bare_gather_ms(kk, vv, pos):
        """The attention's bulk copies without its arithmetic, on the same index list (gw_debug_gather_rate)."""
        T_, K_ = pos.shape[1], pos.shape[2]

        def call():
            _lib.check(lib.gw_debug_gather_rate(kk.data_ptr(), vv.data_ptr(), pos.data_ptr(), T_, kk.shape[1], K_, H * D * es,
                                                kk.stride(1) * es, vv.stride(1) * es, _lib.status_word(dev).data_ptr(),
                                                _lib.stream_ptr(dev)), "gw_debug_gather_rate")

        return time_ms(call, 2, 3)

    extra = not (args.no_extra_legs or args.profile)
    # --- the ceiling of the gather method on the main workload's own index lists (L2-served at vggt32)
    gather_ms = bare_gather_ms(last["k"], last["v"], last["idx"]) if extra and last else None
    geoweave_b200.check_status()

    # --- attention where HBM is the bound: uniformly random positions over the 256-view key set (K + V = 1.09 GB)
    hbm_leg = None
    if extra:
        S_big, T_big = 256 * 1041, 8192
        gg = torch.Generator(device=dev).manual_seed(99)
        kb = torch.randn(1, S_big, H, D, device=dev, dtype=bf, generator=gg)
        vb = torch.randn(1, S_big, H, D, device=dev, dtype=bf, generator=gg)
        qb = torch.randn(1, T_big, H, D, device=dev, dtype=bf, generator=gg)
        pb = torch.randint(0, S_big, (1, T_big, TOPK), device=dev, dtype=torch.int32, generator=gg)
        ms_att = time_ms(lambda: sparse_index_flash_attn_inference_func(qb, kb, vb, pb, None, False, D ** -0.5, False), 3, 5)
        ms_gat = bare_gather_ms(kb, vb, pb)
        hbm_leg = {"ms": ms_att, "bytes": attn_bytes_of(T_big), "gather_ms": ms_gat, "queries": T_big, "keys": S_big}
        del kb, vb, qb, pb
        geoweave_b200.check_status()

    # --- the 256-view context (one layer, N = 266496), sharded like the main workload: the 1 -> N curve of the long context
    ctx = None
    if extra and args.workload == "vggt32":
        n_ctx = 256 * 1041
        clo, chi = row_partition(n_ctx, world)[rank]
        gg = torch.Generator(device=dev).manual_seed(4321 + rank)
        mk = lambda *shape: torch.randn(*shape, device=dev, dtype=bf, generator=gg)
        tc = {"q_idx": mk(1, chi - clo, HI, DI), "k_idx": mk(1, chi - clo, HI, DI),
              "w": torch.rand(1, chi - clo, HI, device=dev, generator=gg).to(bf), "q": mk(1, chi - clo, H, D),
              "k": mk(1, chi - clo, H, D), "v": mk(1, chi - clo, H, D)}
        ms_warm = timed(lambda: layer_op(tc, False, n_ctx), 1)
        geoweave_b200.check_status()
        # enough steps for the clock sampler (one sample per 200 ms) to see the region: at least 2, about 0.7 s, at most 32
        ctx_steps = int(min(32, max(2, -(-700.0 // max(ms_warm, 1.0)))))
        ctx_events = []
        ctx_clocks = Clocks(local) if rank == 0 else None
        t0c = time.perf_counter()
        ms_ctx = timed(lambda: layer_op(tc, True, n_ctx, ctx_events), ctx_steps) / ctx_steps
        ctx_clk = ctx_clocks.stop(t0c, time.perf_counter()) if ctx_clocks else None
        ctx = {"ms": ms_ctx, "idx_ms": statistics.mean(e[0].elapsed_time(e[1]) for e in ctx_events),
               "att_ms": statistics.mean(e[4].elapsed_time(e[2]) for e in ctx_events),
               "kidx_gather_ms": statistics.mean(e[3].elapsed_time(e[0]) for e in ctx_events),
               "kv_wait_ms": statistics.mean(e[1].elapsed_time(e[4]) for e in ctx_events), "rows": chi - clo, "tokens": n_ctx, "clocks": ctx_clk,
               "steps": ctx_steps}
        # the same layer with the coarse-to-fine selection (pooled sources, per-token queries) in place of the indexer call
        lay_ctx = source_layout(1041, 256, 5, 28, 37, dev)
        layer_op(tc, False, n_ctx, None, lay_ctx)
        c2f_events = []
        ms_c2f = timed(lambda: layer_op(tc, True, n_ctx, c2f_events, lay_ctx), 2) / 2
        ctx["c2f_layer_ms"] = ms_c2f
        ctx["c2f_select_ms"] = statistics.mean(e[0].elapsed_time(e[1]) for e in c2f_events)
        geoweave_b200.check_status()
        if world == 1:
            # the selection stage alone, coarse-to-fine (2x2-pooled sources, kept cells expanded) against the full-resolution
            # indexer call, on this context and on the main workload's 32 views
            from geoweave_b200.custom_indexer.sparse_topk_indexer import fused_score_topk

            c2f = {}
            for tag, n_views, src in (("ctx256", 256, tc), ("vggt32", views, resident[0])):
                lay = source_layout(1041, n_views, 5, 28, 37, dev)
                nn = 1041 * n_views
                f_c2f = lambda: select_topk_coarse_to_fine(src["q_idx"], src["k_idx"], src["w"], lay, TOPK, DI ** -0.5)
                f_full = lambda: fused_score_topk(src["q_idx"], src["k_idx"], src["w"], TOPK, DI ** -0.5, return_scores=False)
                f_c2f(), f_full()
                f_sym = lambda: select_topk_coarse_to_fine(src["q_idx"], src["k_idx"], src["w"], lay, TOPK, DI ** -0.5, pool_queries=True)
                f_sym()
                c2f[tag] = {"tokens": nn, "sources": lay.source_len, "kept_sources": lay.kept_sources(TOPK),
                            "coarse_to_fine_ms": timed(f_c2f, 3) / 3, "pooled_queries_too_ms": timed(f_sym, 3) / 3,
                            "full_indexer_ms": timed(f_full, 3) / 3}
            ctx["c2f"] = c2f
            geoweave_b200.check_status()
        del tc
        last.clear()
        torch.cuda.empty_cache()
        geoweave_b200.check_status()

    # --- one vggt32 layer whose operator inputs come out of the reference's own projection modules (seeded weights)
    proj = None
    if extra and args.workload == "vggt32":
        try:
            from baseline import ref_harness as rh

            if not rh.available():
                proj = {"unavailable": "no staged copy of the reference (baseline/_ref)"}
            else:
                rh.enable_import()
                blk = rh.build_block("vggt", TOPK, seed=0, device=dev, dtype=bf)
                xin, pin = rh.make_inputs("vggt", views, seed=0, device=dev, dtype=bf)
                with torch.no_grad():
                    full = rh.operator_inputs(blk, blk.norm1(xin), pin)
                tp = {n: x[:, lo:hi].contiguous() for n, x in zip(("q", "k", "v", "q_idx", "k_idx", "w"), full)}
                del blk, xin, full
                layer_op(tp, False)
                pev = []
                ms_p = timed(lambda: layer_op(tp, True, n_tokens, pev), 3) / 3
                g_ms = bare_gather_ms(last["k"], last["v"], last["idx"])
                proj = {"ms_per_layer": ms_p, "tokens_per_s": n_tokens / (ms_p * 1e-3),
                        "idx_ms": statistics.mean(e[0].elapsed_time(e[1]) for e in pev),
                        "att_ms": statistics.mean(e[4].elapsed_time(e[2]) for e in pev), "bare_gather_ms": g_ms,
                        "inputs": "q,k,v,q_idx,k_idx,w from the reference's DSABlock projections (qkv + q/k LayerNorm + rotary; "
                                  "LightningIndexer.project) of ~N(0,1) tokens, trunc-normal(0.02) weights, w_proj bias 1"}
                del tp
                last.clear()
                geoweave_b200.check_status()
        except Exception as exc:
            proj = {"unavailable": f"{type(exc).__name__}: {exc}"}

    if rank == 0:
        peaks = {}
        try:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        except Exception:
            pass
        hbm_peak = float(peaks.get("hbm_gbs", 6650.0))
        tc_peak = float(peaks.get("bf16_tflops", 1590.0))
        tc_sustained = float(peaks.get("bf16_tflops_sustained", 1400.0))
        peak_src = "measured (MEASURED_PEAKS.json)" if peaks else "fallback"
        attn_bytes = attn_bytes_of(rows)
        attn_gbs = attn_bytes / (att_ms * 1e-3) / 1e9
        traffic = recorded_dram_traffic("sparse_attn_mma_kernel", args.workload, rows)
        idx_flops = 2.0 * rows * n_tokens * HI * DI
        idx_tfs = idx_flops / (idx_ms * 1e-3) / 1e12
        ms_step = ms_total / args.steps
        value = n_tokens * layers / (ms_step * 1e-3)
        e2e_value = n_tokens * layers / (ms_e2e / args.steps * 1e-3)
        kv_mb = 2 * n_tokens * H * D * es / 1e6
        roof = {"kernel": "sparse_attn_mma_kernel (stage 3 gather)", "bound": "hbm",
                "regime": ("L2-served gather" if kv_mb < 400 else "HBM gather") + f": K+V of a layer = {kv_mb:.0f} MB against a 126 MB L2",
                "achieved": attn_gbs, "peak": hbm_peak, "unit": "GB/s", "frac": attn_gbs / hbm_peak, "traffic": traffic,
                "dram_frac": (traffic / (att_ms * 1e-3) / 1e9 / hbm_peak) if traffic else None,
                "peak_source": peak_src, "bytes_per_launch": attn_bytes, "ms_per_launch": att_ms,
                "note": "achieved = ALGORITHMIC gather bytes / time.  When K+V of a layer fit (most of) the L2, the gather is served "
                        "by the L2-to-SM path and this exceeds the HBM copy peak: frac is then not an HBM utilisation.  dram_frac = "
                        "DRAM bytes of the launch (ncu capture of this kernel source, null if none is on record) / time / peak; "
                        "gather_ceiling = the same bulk copies without any arithmetic on the same index lists, timed in this run; "
                        "roofline_hbm = the same kernel where HBM does bind"}
        if gather_ms:
            roof["gather_ceiling"] = {"achieved": attn_bytes / (gather_ms * 1e-3) / 1e9, "unit": "GB/s", "ms": gather_ms,
                                      "frac_of_ceiling": gather_ms / att_ms}
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": n_warm,
                "ms_per_step": ms_step, "ms_per_layer": ms_step / layers, "higher_is_better": True, "scaling": "strong",
                "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": config_of(args, n_tokens, layers, desc, world),
                "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                        "ms_per_step": ms_e2e / args.steps, "h2d_alone_gbs_rank0_clock": h2d_gbs, "host_binding": host_binding,
                        "host_enqueue_ms_per_step": (1e3 * statistics.median(enqueue_s)) if enqueue_s else None},
                "gpu_launches": launches * args.steps,
                "roofline": roof,
                "roofline_indexer": {"kernel": "indexer kernels (stage 1+2, all launches of one call)", "bound": "tensor",
                                     "achieved": idx_tfs, "peak": tc_peak, "unit": "TFLOP/s", "frac": idx_tfs / tc_peak,
                                     "frac_of_sustained": idx_tfs / tc_sustained, "flops_per_call": idx_flops,
                                     "ms_per_call": idx_ms, "peak_source": peak_src},
                "clocks": clk}
        if world > 1:
            line["exchange"] = {"gather": "peer" if use_peer else ("packed" if args.gather == "peer" else args.gather), "kidx_gather_ms": kidx_gather_ms, "indexer_ms": idx_ms, "kv_wait_ms": kv_wait_ms,
                                "attention_ms": att_ms, "fallback_reason": peer_error, "note": "mean per layer on rank 0's stream (CUDA events): K_idx and w arriving in "
                                "front of the indexer; the indexer call (the K, V gather runs beside it); what of the K, V gather is "
                                "left when the indexer ends; the attention launch"}
        if hbm_leg:
            gbs = hbm_leg["bytes"] / (hbm_leg["ms"] * 1e-3) / 1e9
            hbm_traffic = recorded_dram_traffic("sparse_attn_mma_kernel", "attn_hbm", hbm_leg["queries"])
            line["roofline_hbm"] = {
                "kernel": "sparse_attn_mma_kernel", "bound": "hbm", "achieved": gbs, "peak": hbm_peak, "unit": "GB/s",
                "frac": gbs / hbm_peak, "traffic": hbm_traffic,
                "dram_frac": (hbm_traffic / (hbm_leg["ms"] * 1e-3) / 1e9 / hbm_peak) if hbm_traffic else None,
                "peak_source": peak_src, "ms_per_launch": hbm_leg["ms"],
                "bytes_per_launch": hbm_leg["bytes"],
                "gather_ceiling": {"achieved": hbm_leg["bytes"] / (hbm_leg["gather_ms"] * 1e-3) / 1e9, "unit": "GB/s",
                                   "ms": hbm_leg["gather_ms"], "frac_of_ceiling": hbm_leg["gather_ms"] / hbm_leg["ms"]},
                "workload": f"{hbm_leg['queries']} queries, k = {TOPK}, positions uniformly random over {hbm_leg['keys']} keys "
                            "(K + V = 1.09 GB, nine times the L2): every gathered row comes from DRAM; measured after the timed region"}
        if ctx:
            cf = 2.0 * ctx["rows"] * ctx["tokens"] * HI * DI
            line["ctx256"] = {
                "workload": "one VGGT-shaped layer over 256 views (N = 266496, k = 1024), query rows sharded like the main workload",
                "ms_per_layer": ctx["ms"], "tokens_per_s": ctx["tokens"] / (ctx["ms"] * 1e-3), "indexer_ms": ctx["idx_ms"],
                "attention_ms": ctx["att_ms"], "indexer_tflops": cf / (ctx["idx_ms"] * 1e-3) / 1e12,
                "indexer_frac": cf / (ctx["idx_ms"] * 1e-3) / 1e12 / tc_peak,
                "attention_gbs": attn_bytes_of(ctx["rows"]) / (ctx["att_ms"] * 1e-3) / 1e9,
                "kidx_gather_ms": ctx["kidx_gather_ms"], "kv_wait_ms": ctx["kv_wait_ms"], "steps": ctx["steps"], "warmup": 1, "clocks": ctx["clocks"],
                "with_coarse_to_fine_selection": {"ms_per_layer": ctx["c2f_layer_ms"], "selection_ms": ctx["c2f_select_ms"],
                                                  "tokens_per_s": ctx["tokens"] / (ctx["c2f_layer_ms"] * 1e-3),
                                                  "note": "the same layer with the selection over 2x2-pooled sources (72 960 instead of "
                                                          "266 496 keys, 309 kept and expanded to 1024 tokens) -- the reference's reduction "
                                                          "for long contexts, an approximation of the exact selection"}}
        if ctx and "c2f" in ctx:
            line["coarse_to_fine_selection"] = dict(ctx["c2f"], note="selection stage alone (one call, CUDA events): pooled 2x2 "
                                                    "sources -> fused indexer over the sources -> expansion to 1024 tokens (and, second "
                                                    "figure, with the queries pooled too and each list broadcast to its cell's tokens), "
                                                    "against the full-resolution fused indexer on the same inputs; random inputs, so only the cost "
                                                    "is meaningful here, not which tokens are found")
        if proj is not None:
            if "ms_per_layer" in proj:
                proj["indexer_frac"] = idx_flops / (proj["idx_ms"] * 1e-3) / 1e12 / tc_peak
                proj["attention_gbs"] = attn_bytes / (proj["att_ms"] * 1e-3) / 1e9
                proj["bare_gather_gbs"] = attn_bytes / (proj["bare_gather_ms"] * 1e-3) / 1e9
            line["reference_projection_inputs"] = proj
        if world == 1 and not args.no_cpu_baseline and not args.profile:
            tps, threads, per, sample, kind = cpu_reference_tokens_per_s(n_tokens, args.cpu_rows, 2)
            line["cpu_baseline"] = {"value": tps, "unit": UNIT, "cores": threads, "kind": kind, "sample": sample}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def kernel_source_digest(files=("gw_attn_mma.cuh", "gw_attn.cu", "gw_common.cuh")):
    import hashlib

    hsh = hashlib.sha256()
    for name in files:
        with open(os.path.join(ROOT, "geoweave_b200", "csrc", name), "rb") as f:
            hsh.update(f.read())
    return hsh.hexdigest()


def recorded_dram_traffic(kernel, workload, rows):
    """DRAM bytes (read + write) of one launch of `kernel` on `workload`, from an ncu capture recorded in
    bench_traffic.json -- only if that capture was made of the kernel source as it is now (digest match);
    scaled by the rows of this launch for a sharded run.  None otherwise."""
    try:
        rec = json.load(open(os.path.join(ROOT, "bench_traffic.json")))[f"{kernel}/{workload}"]
    except Exception:
        return None
    if rec.get("source_sha256") != kernel_source_digest():
        return None
    return float(rec["dram_bytes_per_launch"]) * rows / float(rec["rows"])


def run_micro(args):
    """Stand-alone operators of the drop-in API that the fused path does not go through."""
    import geoweave_b200
    from geoweave_b200 import _lib
    from geoweave_b200.custom_flash_attn.sparse_index_flash_attn import sparse_attention_forward
    from geoweave_b200.custom_indexer.merge_two_topk_cuda import merge_two_topk_inplace
    from geoweave_b200.custom_indexer.topk_exact_cuda import topk_exact_select

    _lib.load()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    try:
        hbm_peak = float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["hbm_gbs"])
    except Exception:
        hbm_peak = 6650.0
    g = torch.Generator(device="cpu").manual_seed(3)

    def timed(fn, reps=5):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / reps

    out = []
    rows, cols, k = 8192, 33312, 1024  # 1.09 GB of fp32 scores: larger than L2
    sc = torch.randn(1, rows, cols, device=dev)
    o_s = torch.empty(1, rows, k, device=dev)
    o_p = torch.empty(1, rows, k, dtype=torch.int32, device=dev)
    ms = timed(lambda: topk_exact_select(sc, o_s, o_p))
    nbytes = 4 * rows * cols + 8 * rows * k
    out.append({"op": "topk_exact_select", "shape": [rows, cols, k], "ms": ms, "bound": "hbm", "achieved": nbytes / ms / 1e6,
                "peak": hbm_peak, "unit": "GB/s", "frac": nbytes / ms / 1e6 / hbm_peak})
    del sc
    rows = 33312
    a_s = torch.randn(1, rows, k, device=dev)
    b_s = torch.randn(1, rows, k, device=dev)
    a_i = torch.randint(0, 30000, (1, rows, k), device=dev, dtype=torch.int32)
    b_p = torch.randint(0, 3000, (1, rows, k), device=dev, dtype=torch.int64)
    m_s, m_i = torch.empty_like(a_s), torch.empty_like(a_i)
    ms = timed(lambda: merge_two_topk_inplace(a_s, a_i, b_s, b_p, 30000, m_s, m_i))
    nbytes = rows * k * (4 + 4 + 4 + 8 + 4 + 4)
    out.append({"op": "merge_two_topk_inplace", "shape": [rows, k], "ms": ms, "bound": "hbm", "achieved": nbytes / ms / 1e6,
                "peak": hbm_peak, "unit": "GB/s", "frac": nbytes / ms / 1e6 / hbm_peak})
    T, S = 4096, 33312
    for dtype, name in ((torch.float32, "sparse attention, scalar kernel, fp32"), (torch.bfloat16, "sparse attention, scalar kernel, bf16 head-major")):
        q = torch.randn(1, T, H, D, device=dev).to(dtype)
        kk = torch.randn(1, S, H, D, device=dev).to(dtype)
        vv = torch.randn(1, S, H, D, device=dev).to(dtype)
        pos = torch.randint(0, S, (1, T, TOPK), device=dev, dtype=torch.int32)
        if dtype == torch.bfloat16:  # [B,H,T,D] inputs are gathered head by head by the scalar kernel
            q, kk, vv = [x.transpose(1, 2).contiguous() for x in (q, kk, vv)]
            ms = timed(lambda: sparse_attention_forward(q, kk, vv, pos, None, False, False, "bhtd"))
        else:
            ms = timed(lambda: sparse_attention_forward(q, kk, vv, pos, None, False, False, "bthd"))
        es = q.element_size()
        nbytes = T * (TOPK * 2 * H * D * es + TOPK * 4 + 2 * H * D * es)
        out.append({"op": name, "shape": [T, S, TOPK], "ms": ms, "bound": "hbm", "achieved": nbytes / ms / 1e6, "peak": hbm_peak,
                    "unit": "GB/s", "frac": nbytes / ms / 1e6 / hbm_peak})
    # the forward with and without attn_sum on the benchmark's own shape (bf16, token-major, every row a query)
    T = S = 33312
    q = torch.randn(1, T, H, D, device=dev).bfloat16()
    kk = torch.randn(1, S, H, D, device=dev).bfloat16()
    vv = torch.randn(1, S, H, D, device=dev).bfloat16()
    pos = torch.randint(0, S, (1, T, TOPK), device=dev, dtype=torch.int32)
    nbytes = T * (TOPK * 2 * H * D * 2 + TOPK * 4 + 2 * H * D * 2)
    for with_sum, name in ((False, "sparse attention, tensor-core kernel, bf16"), (True, "sparse attention + attn_sum, tensor-core kernel, bf16")):
        ms = timed(lambda: sparse_attention_forward(q, kk, vv, pos, None, with_sum, with_sum, "bthd"), reps=3)
        out.append({"op": name, "shape": [T, S, TOPK], "ms": ms, "bound": "hbm", "achieved": nbytes / ms / 1e6, "peak": hbm_peak,
                    "unit": "GB/s", "frac": nbytes / ms / 1e6 / hbm_peak})
    # the bare gather of the same lists (bulk copies only) with fewer CTAs than SMs: is the rate a per-SM or a chip-wide limit?
    lib_ = _lib.load()
    stw = _lib.status_word(dev)
    for ctas in (148, 116, 74):
        fn_g = lambda: _lib.check(lib_.gw_debug_gather_rate_ctas(kk.data_ptr(), vv.data_ptr(), pos.data_ptr(), T, S, TOPK, H * D * 2, H * D * 2,
                                                                 H * D * 2, ctas, stw.data_ptr(), _lib.stream_ptr(dev)), "gather")
        ms = timed(fn_g, reps=3)
        out.append({"op": f"bare gather of K and V rows, {ctas} CTAs (one per SM)", "shape": [T, S, TOPK], "ms": ms, "bound": "hbm",
                    "achieved": nbytes / ms / 1e6, "peak": hbm_peak, "unit": "GB/s", "frac": nbytes / ms / 1e6 / hbm_peak,
                    "gbs_per_sm": nbytes / ms / 1e6 / ctas})
        fn_l = lambda: _lib.check(lib_.gw_debug_gather_rate_ldg(kk.data_ptr(), vv.data_ptr(), pos.data_ptr(), T, S, TOPK, ctas,
                                                                _lib.stream_ptr(dev)), "gather")
        ms = timed(fn_l, reps=3)
        out.append({"op": f"bare gather with plain 16-byte loads, {ctas} CTAs", "shape": [T, S, TOPK], "ms": ms, "bound": "hbm",
                    "achieved": nbytes / ms / 1e6, "peak": hbm_peak, "unit": "GB/s", "frac": nbytes / ms / 1e6 / hbm_peak,
                    "gbs_per_sm": nbytes / ms / 1e6 / ctas})
    # the backward of the same call (dQ, dK, dV; the index lists sorted by key inside the timed call)
    from geoweave_b200.custom_flash_attn.sparse_index_flash_attn import sparse_attention_backward
    o_f, _, lse_f = sparse_attention_forward(q, kk, vv, pos, None, False, True, "bthd")
    d_o = torch.randn_like(o_f)
    ms = timed(lambda: sparse_attention_backward(q, kk, vv, pos, o_f, lse_f, d_o, None, None), reps=3)
    # per (query, key) pair: the K and V rows, then from the key's side the q and dO rows; P and dP written and read once
    nbytes_bwd = T * TOPK * (4 * H * D * 2 + 4 * H * 4) + T * TOPK * 12
    out.append({"op": "sparse attention backward (query kernel + key kernel + sort of the lists), bf16", "shape": [T, S, TOPK],
                "ms": ms, "bound": "hbm", "achieved": nbytes_bwd / ms / 1e6, "peak": hbm_peak, "unit": "GB/s",
                "frac": nbytes_bwd / ms / 1e6 / hbm_peak})
    d_sum = torch.randn(1, T, TOPK, device=dev)
    ms = timed(lambda: sparse_attention_backward(q, kk, vv, pos, o_f, lse_f, d_o, d_sum, None), reps=3)
    out.append({"op": "sparse attention backward with a gradient through attn_sum (pre-pass over the K rows first), bf16",
                "shape": [T, S, TOPK], "ms": ms, "bound": "hbm", "achieved": (nbytes_bwd + T * TOPK * 2 * H * D) / ms / 1e6, "peak": hbm_peak,
                "unit": "GB/s", "frac": (nbytes_bwd + T * TOPK * 2 * H * D) / ms / 1e6 / hbm_peak})
    del o_f, lse_f, d_o, d_sum
    # the indexer's backward on the same lists: gradients of the selected scores for q_idx, k_idx and w
    from geoweave_b200.custom_indexer.sparse_topk_indexer import indexer_topk_backward
    qi_ = torch.randn(1, T, HI, DI, device=dev).bfloat16()
    ki_ = torch.randn(1, S, HI, DI, device=dev).bfloat16()
    wi_ = torch.rand(1, S, HI, device=dev).bfloat16()
    g_sc = torch.randn(1, T, TOPK, device=dev)
    ms = timed(lambda: indexer_topk_backward(qi_, ki_, wi_, pos, g_sc, None), reps=3)
    # per pair: the key's k_idx row and w, then from the key's side the q_idx row; the 32-byte scratch line written and read
    nbytes_ib = T * TOPK * (2 * HI * DI * 2 + 16 + 2 * 32 + 4 + 4) + T * TOPK * 12
    out.append({"op": "indexer backward (query kernel + key kernel + sort of the lists), bf16", "shape": [T, S, TOPK], "ms": ms,
                "bound": "hbm", "achieved": nbytes_ib / ms / 1e6, "peak": hbm_peak, "unit": "GB/s",
                "frac": nbytes_ib / ms / 1e6 / hbm_peak})
    del qi_, ki_, wi_, g_sc
    # projection front-end on the benchmark's shape: 33 312 tokens, 16 heads + 4 indexer heads (VGGT grid positions)
    from geoweave_b200.front_end import FrontEndParams, project_epilogue, rope_tables
    del q, kk, vv, pos
    N = 33312
    width = 3 * H * D + 2 * HI * DI + HI
    fused = torch.randn(1, N, width, device=dev).bfloat16()
    fpos = torch.randint(0, 38, (1, N, 2), device=dev)
    cos, sin = rope_tables(38, dev, torch.bfloat16)
    vec = lambda: (torch.rand(64, device=dev) + 0.5, torch.randn(64, device=dev) * 0.1, 1e-5)
    prm = FrontEndParams(torch.empty(0), None, H, HI, vec(), vec(), vec(), cos, sin)
    ms = timed(lambda: project_epilogue(fused, fpos, prm))
    nbytes = 2 * N * width * 2 + N * 16  # every value read once and written once, plus the positions
    out.append({"op": "projection front-end epilogue (LayerNorm, rotary, layout), bf16", "shape": [N, width], "ms": ms, "bound": "hbm",
                "achieved": nbytes / ms / 1e6, "peak": hbm_peak, "unit": "GB/s", "frac": nbytes / ms / 1e6 / hbm_peak})
    # the projection itself: library GEMM alone, library GEMM + epilogue kernel, and the fused tensor-core kernel
    import torch.nn.functional as Fnn
    from geoweave_b200.front_end import project_fused
    dimp = H * D
    prm_p = FrontEndParams((torch.randn(width, dimp, device=dev) * dimp ** -0.5).bfloat16(), torch.zeros(width, device=dev).bfloat16(),
                           H, HI, vec(), vec(), vec(), cos, sin)
    xp = torch.randn(1, N, dimp, device=dev).bfloat16()
    flops = 2.0 * N * width * dimp
    try:
        tc_peak = float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["bf16_tflops"])
    except Exception:
        tc_peak = 1590.0
    for name, fn in (("projection: library GEMM alone (cuBLAS, writes the raw product)", lambda: Fnn.linear(xp, prm_p.weight, prm_p.bias)),
                     ("projection: library GEMM + epilogue kernel", lambda: project_epilogue(Fnn.linear(xp, prm_p.weight, prm_p.bias), fpos, prm_p)),
                     ("projection: fused tcgen05 GEMM with LayerNorm / rotary / layout epilogue", lambda: project_fused(xp, fpos, prm_p))):
        ms = timed(fn)
        out.append({"op": name, "shape": [N, width, dimp], "ms": ms, "bound": "tensor", "achieved": flops / ms / 1e9, "peak": tc_peak,
                    "unit": "TFLOP/s", "frac": flops / ms / 1e9 / tc_peak})
    del xp
    # the whole layer as one call: projection front-end -> indexer -> attention
    from geoweave_b200.layer import SparseGlobalAttentionLayer
    dim = H * D
    prm = FrontEndParams((torch.randn(width, dim, device=dev) * dim ** -0.5).bfloat16(), torch.zeros(width, device=dev).bfloat16(),
                         H, HI, vec(), vec(), vec(), cos, sin)
    x = torch.randn(1, N, dim, device=dev).bfloat16()
    for graph in (False, True):
        layer = SparseGlobalAttentionLayer(prm, TOPK, use_cuda_graph=graph)
        ms = timed(lambda: layer(x, fpos), reps=3)
        out.append({"op": "whole layer: projection + front-end + indexer + attention" + (", CUDA graph" if graph else ", eager"),
                    "shape": [N, dim, TOPK], "ms": ms, "tokens_per_s": N / ms * 1e3})
    geoweave_b200.check_status()
    print(json.dumps({"micro": out}), flush=True)


def run_attn_hbm(args):
    """The sparse attention kernel alone on an index list that defeats the L2 (see --attn-hbm)."""
    import geoweave_b200
    from geoweave_b200 import _lib
    from geoweave_b200.custom_flash_attn import sparse_index_flash_attn_inference_func

    _lib.load()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    S_big, T_big, bf = 256 * 1041, 8192, torch.bfloat16
    gg = torch.Generator(device=dev).manual_seed(99)
    kb = torch.randn(1, S_big, H, D, device=dev, dtype=bf, generator=gg)
    vb = torch.randn(1, S_big, H, D, device=dev, dtype=bf, generator=gg)
    qb = torch.randn(1, T_big, H, D, device=dev, dtype=bf, generator=gg)
    pb = torch.randint(0, S_big, (1, T_big, TOPK), device=dev, dtype=torch.int32, generator=gg)
    fn = lambda: sparse_index_flash_attn_inference_func(qb, kb, vb, pb, None, False, D ** -0.5, False)
    for _ in range(max(1, args.warmup)):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(max(1, args.steps)):
        fn()
    b.record()
    torch.cuda.synchronize()
    geoweave_b200.check_status()
    ms = a.elapsed_time(b) / max(1, args.steps)
    nbytes = T_big * (TOPK * 2 * H * D * 2 + TOPK * 4 + 2 * H * D * 2)
    print(json.dumps({"leg": "attention, HBM regime", "queries": T_big, "keys": S_big, "topk": TOPK, "ms_per_launch": ms,
                      "bytes_per_launch": nbytes, "achieved_gbs": nbytes / ms / 1e6}), flush=True)


def run_attn_bwd(args):
    """The attention backward alone on a block of query rows of the main workload (see --attn-bwd): small enough for a
    multi-pass profiler capture (K + V = 136 MB, scratch 0.5 GB), large enough that DRAM figures mean something."""
    import geoweave_b200
    from geoweave_b200 import _lib
    from geoweave_b200.custom_flash_attn.sparse_index_flash_attn import sparse_attention_backward, sparse_attention_forward

    _lib.load()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    S, T, bf = 32 * 1041, 8192, torch.bfloat16
    gg = torch.Generator(device=dev).manual_seed(77)
    k = torch.randn(1, S, H, D, device=dev, dtype=bf, generator=gg)
    v = torch.randn(1, S, H, D, device=dev, dtype=bf, generator=gg)
    q = torch.randn(1, T, H, D, device=dev, dtype=bf, generator=gg)
    pos = torch.randint(0, S, (1, T, TOPK), device=dev, dtype=torch.int32, generator=gg)
    o, _, lse = sparse_attention_forward(q, k, v, pos, None, False, True, "bthd")
    d_o = torch.randn_like(o)
    fn = lambda: sparse_attention_backward(q, k, v, pos, o, lse, d_o, None, None)
    for _ in range(max(1, args.warmup)):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(max(1, args.steps)):
        fn()
    b.record()
    torch.cuda.synchronize()
    geoweave_b200.check_status()
    ms = a.elapsed_time(b) / max(1, args.steps)
    pairs = T * TOPK
    print(json.dumps({"leg": "attention backward", "queries": T, "keys": S, "topk": TOPK, "ms_per_call": ms,
                      "gather_bytes_per_kernel": pairs * 2 * H * D * 2, "scratch_bytes": pairs * H * 4}), flush=True)


def main():
    args = parse()
    if args.attn_hbm:
        run_attn_hbm(args)
        return
    if args.attn_bwd:
        run_attn_bwd(args)
        return
    if args.micro:
        run_micro(args)
        return
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
