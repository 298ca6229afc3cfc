#!/usr/bin/env python
"""Benchmark of the DFS sparse-attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload (N = 1 and the head-sharded N > 1 runs): the HunyuanVideo-13B 720p
joint self-attention shape -- latent grid 33x45x80 = 118 800 video tokens +
256 text tokens, 24 heads, head_dim 128, bf16, hilbert3d order, block 128,
tile 16, sparsity 0.3 -- on seeded synthetic structured Q/K/V.  One step = one
refresh call of the operator: Hilbert permute of Q/K/V, block scoring, top-k
selection, block-sparse attention with the inverse permute fused in its store.
The 24 heads are split across ranks (no collective on the data path); the
total work is fixed, so scaling is "strong".

metric: effective TFLOP/s = 4 * D * (selected token pairs, partial blocks
counted exactly) / step time; ms_per_step is the time per call.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

WORKLOADS = {
    "hunyuan_720p": dict(grid=(33, 45, 80), text=256, heads=24, dim=128, sparsity=0.3, flavor="hyvideo"),
    "wan_480p": dict(grid=(21, 30, 52), text=0, heads=40, dim=128, sparsity=0.3, flavor="wan"),
    "wan_720p": dict(grid=(21, 45, 80), text=0, heads=40, dim=128, sparsity=0.3, flavor="wan"),
    # small cases for ncu captures: inputs still larger than L2 (3 x 67 MB), kernels of a millisecond or two
    "wan_480p_h8": dict(grid=(21, 30, 52), text=0, heads=8, dim=128, sparsity=0.3, flavor="wan"),
    "hunyuan_480p_h4": dict(grid=(33, 30, 45), text=256, heads=4, dim=128, sparsity=0.3, flavor="hyvideo"),
    "tiny": dict(grid=(4, 16, 16), text=0, heads=2, dim=64, sparsity=0.3, flavor="hyvideo"),
    "tiny_wan": dict(grid=(4, 16, 16), text=0, heads=2, dim=128, sparsity=0.3, flavor="wan"),
    # the mask-caching trace: 50 denoising steps (12 dense, refreshes at 12 / 24 / 36 with sparsity
    # 0.3 / 0.2 / 0.1) over --trace-layers layers with drifting Q/K; one bench step = the whole trace
    "hunyuan_720p_trace": dict(grid=(33, 45, 80), text=256, heads=24, dim=128, sparsity=0.3, flavor="hyvideo",
                               trace=True),
    "tiny_trace": dict(grid=(5, 16, 32), text=64, heads=2, dim=128, sparsity=0.5, flavor="hyvideo", trace=True),
}
METRIC = "dfs_attn_effective_tflops"
UNIT = "TFLOP/s"


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return dict(hbm_gbs=p["hbm_gbs"], bf16_tflops=p["bf16_tflops"],
                    bf16_tflops_sustained=p.get("bf16_tflops_sustained", p["bf16_tflops"]), source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples taken while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.rows = []
        self.proc = None
        self.gpu_index = gpu_index
        self.nvml = None
        self._stop = threading.Event()

    # NVML read directly (a sample every ~10 ms: short timed regions are covered too); nvidia-smi as a
    # subprocess when the NVML binding is not importable.  Reading only: nothing is ever set.
    def _nvml_handle(self):
        import pynvml
        pynvml.nvmlInit()
        try:
            uuid = str(torch.cuda.get_device_properties(self.gpu_index).uuid)
            if not uuid.startswith("GPU-"):
                uuid = "GPU-" + uuid
            return pynvml, pynvml.nvmlDeviceGetHandleByUUID(uuid.encode())
        except Exception:
            return pynvml, pynvml.nvmlDeviceGetHandleByIndex(self.gpu_index)

    def _sample_nvml(self):
        nv, h = self.nvml
        bits = (nv.nvmlClocksEventReasonHwSlowdown, nv.nvmlClocksEventReasonHwThermalSlowdown,
                nv.nvmlClocksEventReasonSwThermalSlowdown, nv.nvmlClocksEventReasonSwPowerCap)
        try:
            sm = nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)
            mx = nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM)
            pw = nv.nvmlDeviceGetPowerUsage(h) / 1000.0
            mask = nv.nvmlDeviceGetCurrentClocksEventReasons(h)
            self.rows.append([str(sm), str(mx), str(pw)] + ["Active" if mask & bit else "Not Active" for bit in bits])
        except Exception:
            pass

    def _poll_nvml(self):
        while not self._stop.is_set():
            self._sample_nvml()
            self._stop.wait(0.01)

    def start(self):
        try:
            self.nvml = self._nvml_handle()
            self.thread = threading.Thread(target=self._poll_nvml, daemon=True)
            self.thread.start()
            return
        except Exception:
            self.nvml = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.nvml is not None:
            self._stop.set()
            self.thread.join(timeout=2)
            if not self.rows:   # a timed region shorter than the polling thread's start-up: one sample right after it
                self._sample_nvml()
        elif self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        else:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        sm, mx, reasons, power = [], [], set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
                power.append(float(r[2]))
            except (ValueError, IndexError):
                continue
            for n, val in zip(names, r[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons),
                "source": "nvml" if self.nvml is not None else "nvidia-smi"}


def dist_env():
    return (int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)),
            int(os.environ.get("WORLD_SIZE", 1)))


# --------------------------------------------------------------------------- #
# CPU reference arm / cpu_baseline: the reference's path on the host cores
# --------------------------------------------------------------------------- #
def load_by_path(name, path):
    """Import one source file without importing the package around it (the reference arm must
    not map libdfs_b200.so, which `import dfsattn_b200` does)."""
    import importlib.util
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def host_threads():
    """Use every core this process may run on (torch.distributed.run exports OMP_NUM_THREADS=1)."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    torch.set_num_threads(max(1, n))
    return torch.get_num_threads()


def reference_modules():
    """The reference's own attention modules when a checkout is reachable: the directory named by
    DFSATTN_REFERENCE_PATH, else baseline/_ref (not part of the source tree).  (None, reason) otherwise."""
    for cand in (os.environ.get("DFSATTN_REFERENCE_PATH"), os.path.join(ROOT, "baseline", "_ref")):
        if cand and os.path.exists(os.path.join(cand, "dfsattn", "attention_hyvideo.py")):
            try:
                if cand not in sys.path:
                    sys.path.insert(0, cand)
                import dfsattn.attention_hyvideo as ref_hy
                import dfsattn.attention_wan as ref_wan
                return (ref_hy, ref_wan), cand
            except Exception as exc:  # noqa: BLE001  (any import problem means: use the port)
                return None, f"reference at {cand} does not import: {type(exc).__name__}: {exc}"
    return None, "no reference checkout reachable"


def cpu_sample(spec, budget_blocks, ref=None):
    """One bounded sample of the workload on the CPU: ONE head, full scoring and selection,
    attention for the first `budget_blocks` query blocks.  With `ref` (the reference's own modules)
    the reference's `_compute_block_mask` and its packed CPU attention loop do the work, else the
    oracle restatement of the same two functions.  Returns (flops, seconds, note)."""
    import oracle
    structured_qkv = load_by_path("_dfs_synthetic", os.path.join(ROOT, "dfsattn_b200", "synthetic.py")).structured_qkv
    torch.manual_seed(0)
    f, h, w = spec["grid"]
    q, k, v = structured_qkv(spec["grid"], 1, spec["dim"], text_len=spec["text"], dtype=torch.float32,
                             device="cpu", seed=0, head_offset=0, total_heads=1)
    L = q.shape[2]
    video_len = L - spec["text"]
    vperm = torch.from_numpy(oracle.hilbert3d_perm(f, h, w)) if spec.get("order", "hilbert3d") == "hilbert3d" \
        else None
    hy = spec["flavor"] == "hyvideo"
    if ref is not None:
        ref_hy, ref_wan = ref
        attn = ref_hy.DFS_Attention(0, 0, spec["sparsity"], True, video_len, vperm, 128, 16, 16)
        scorer = attn if hy else ref_wan.DFS_Attention(0, 0, spec["sparsity"], True, vperm, 128, 16, 16)
        perm, inv = attn._compute_permutation(vperm, L, torch.device("cpu"))
        t0 = time.perf_counter()
        mask = scorer._compute_block_mask(q, k, perm, spec["sparsity"])
        t_mask = time.perf_counter() - t0
    else:
        perm, inv = oracle.build_permutation(vperm, L, video_len)
        t0 = time.perf_counter()
        mask = (oracle.block_mask_hyvideo(q, k, perm, video_len, spec["sparsity"]) if hy
                else oracle.block_mask_wan(q, k, perm, spec["sparsity"]))
        t_mask = time.perf_counter() - t0
    qb_total = mask.shape[1]
    nb = min(budget_blocks, qb_total)
    t0 = time.perf_counter()
    if ref is not None:
        # the reference's loop walks the rows of the mask it is given: the first nb query blocks
        sub_mask = mask[:, :nb].contiguous()
        attn._run_oracle_hybrid_attention(q, k, v, perm, inv, sub_mask, torch.zeros_like(sub_mask))
    else:
        oracle.block_sparse_attention(q, k, v, perm, inv, mask, q_block_range=(0, nb))
    t_attn = time.perf_counter() - t0
    sub = mask[:, :nb].clone()
    rows = min(nb * 128, L)
    k_last = L - 128 * (mask.shape[2] - 1)
    pairs = int(sub[:, :, :-1].sum()) * 128 * 128 + int(sub[:, :, -1].sum()) * 128 * k_last
    if nb == qb_total:
        pairs = oracle.block_interaction_count(mask, L)
    flops = 4.0 * spec["dim"] * pairs
    # scoring is per call for the whole head: charge the share of the sampled rows
    seconds = t_attn + t_mask * (nb / qb_total)
    who = "the reference's own _compute_block_mask + packed CPU attention loop" if ref is not None \
        else "oracle port of the reference's _compute_block_mask + packed CPU attention loop"
    note = (f"{who}, fp32; 1 of {spec['heads']} heads; scoring+selection of the whole head ({t_mask:.2f} s, "
            f"charged {nb}/{qb_total}) + attention of query blocks 0..{nb - 1} ({rows} rows, {t_attn:.2f} s)")
    return flops, seconds, note


def workload_config(args, spec, world):
    """The `config` object both arms print (same keys, same values)."""
    f, h, w = spec["grid"]
    L = f * h * w + spec["text"]
    return {"workload": args.workload, "grid": list(spec["grid"]), "text_tokens": spec["text"], "seq_len": L,
            "heads": spec["heads"], "heads_per_gpu": spec["heads"] // max(world, 1), "head_dim": spec["dim"],
            "sparsity": spec["sparsity"], "order": spec.get("order", "hilbert3d"), "block": 128, "tile": 16,
            "step": "refresh call: permute + score + select + attention (+fused unpermute)"}


def run_reference(args, spec, rank, world):
    """The reference arm: the reference's CPU implementation of the path on the host cores, rank 0
    only, with every core the process may use.  Nothing of the product is imported."""
    if rank != 0:
        return
    cores = host_threads()
    ref, where = reference_modules()
    times, flops_list, note = [], [], ""
    for i in range(args.warmup + args.steps):
        fl, s, note = cpu_sample(spec, args.cpu_blocks, ref)
        if i >= args.warmup:
            times.append(s)
            flops_list.append(fl)
    value = sum(flops_list) / sum(times) / 1e12
    kind = "reference" if ref is not None else "port"
    config = workload_config(args, spec, args.gpus)
    config["parallelism"] = f"host cores of rank 0 ({cores} threads); the GPU arm's heads are sharded x{args.gpus}"
    config["sample"] = note
    config["reference_source"] = where
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * sum(times) / len(times),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": config,
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": kind, "sample": note},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------- #
# GPU arm
# --------------------------------------------------------------------------- #
def timed(fn, steps, barrier, warm=0, per_step=None):
    """CUDA-event time of `steps` calls on the current stream, bracketed by barrier + synchronize;
    `warm` untimed calls first (they let torch's allocator settle).  With a list in `per_step`, an
    event after every call also gives each step's own time in ms (appended to the list)."""
    for _ in range(warm):
        fn()
    barrier()
    torch.cuda.synchronize()
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
    marks[0].record()
    for i in range(steps):
        fn()
        if per_step is not None or i == steps - 1:
            marks[i + 1].record()
    torch.cuda.synchronize()
    barrier()
    if per_step is not None:
        per_step.extend(marks[i].elapsed_time(marks[i + 1]) for i in range(steps))
    return marks[0].elapsed_time(marks[steps]) / 1e3  # seconds


def quartiles(xs):
    xs = sorted(xs)
    at = lambda f: xs[min(len(xs) - 1, max(0, round(f * (len(xs) - 1))))]  # noqa: E731
    return {"median": at(0.5), "p25": at(0.25), "p75": at(0.75)}


class Ranks:
    """The process group of a run (one process per GPU) and the two reductions the bench needs."""

    def __init__(self, rank, local_rank, world):
        import torch.distributed as dist
        self.dist, self.rank, self.world = dist, rank, world
        torch.cuda.set_device(local_rank)
        self.dev = torch.device("cuda", local_rank)
        if world > 1:
            dist.init_process_group("nccl", device_id=self.dev)

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()

    def _reduce(self, x, op):
        if self.world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=self.dev)
        self.dist.all_reduce(t, op=op)
        return float(t.item())

    def max(self, x):
        return self._reduce(x, self.dist.ReduceOp.MAX)

    def sum(self, x):
        return self._reduce(x, self.dist.ReduceOp.SUM)

    def min(self, x):
        return self._reduce(x, self.dist.ReduceOp.MIN)

    def close(self):
        if self.world > 1:
            self.dist.destroy_process_group()


def operator_call(spec, vperm, video_len, layer_idx=0):
    """The refresh call of the operator for a workload: step 12 (24 for Wan's doubled counter) is a
    refresh step, so scoring and selection run on every call."""
    from dfsattn_b200.attention_hyvideo import dfs_attention as hy_attention
    from dfsattn_b200.attention_wan import dfs_attention as wan_attention
    common = dict(skip_steps=12, cache_interval=12, layer_idx=layer_idx, sparsity=spec["sparsity"],
                  sparsity_dcrt=0.1, tile_size=16, block_size=128, video_perm=vperm)
    if spec["flavor"] == "hyvideo":
        return lambda qq, kk, vv, **extra: hy_attention(qq, kk, vv, step_idx=12, video_len=video_len, **common,
                                                        **extra)
    return lambda qq, kk, vv, **extra: wan_attention(qq, kk, vv, step_idx=24, **common, **extra)


def attention_class(spec):
    from dfsattn_b200.attention_hyvideo import DFS_Attention as HyAttn
    from dfsattn_b200.attention_wan import DFS_Attention as WanAttn
    return HyAttn if spec["flavor"] == "hyvideo" else WanAttn


def cached_pairs(spec, h_local, L):
    """Attended token pairs of this rank's heads, from the lists the last refresh call cached."""
    from dfsattn_b200 import ops
    lists = next(iter(attention_class(spec)._cached_metadata.values()))["block_lists"]
    return ops.interaction_count(lists.idx, lists.cnt, h_local, L), lists


# ---- the mask-caching trace --------------------------------------------------
def trace_pass(rk, spec, base, vperm, layout):
    """One 50-step trace over the layers in `base` (per layer q, k, v: head shards [1, H/P, L, D], or
    with layout "seq" sequence shards [1, H, L_r, D] swapped by NCCL all-to-alls around every call):
    per denoising step and layer either the dense call (warm-up steps), a refresh call (score +
    select + attention) or a call on cached lists, Q and K drifting from step to step
    (x <- 0.98 x + 0.2 N(0,1), outside the timed intervals).  Returns [(kind, sparsity, ms)]."""
    from dfsattn_b200 import parallel
    from dfsattn_b200.attention_hyvideo import (DFS_Attention, _compute_cache_schedule, _dfs_attention_instances,
                                                dfs_attention)
    from dfsattn_b200.fullattention import full_attention
    from dfsattn_b200.synthetic import drift
    n_steps, skip, interval, s0, dcrt = 50, 12, 12, spec["sparsity"], 0.1
    L = spec["grid"][0] * spec["grid"][1] * spec["grid"][2] + spec["text"]
    video_len = L - spec["text"]
    DFS_Attention.clear_cache()
    _dfs_attention_instances.clear()
    state = [list(t) for t in base]
    spans = []
    for step in range(n_steps):
        flag, cur = _compute_cache_schedule(step, skip, interval, s0, dcrt)
        for layer in range(len(base)):
            q, k, v = state[layer]
            if step > 0:
                q = drift(q, 1000 * layer + step)
                k = drift(k, 500000 + 1000 * layer + step)
                state[layer][0], state[layer][1] = q, k
            if step < skip:
                fn = lambda a, b, c: full_attention(a, b, c, mode="flash")  # noqa: E731
                kind = "dense"
            else:
                fn = lambda a, b, c: dfs_attention(  # noqa: E731
                    a, b, c, step_idx=step, skip_steps=skip, cache_interval=interval, layer_idx=layer,
                    sparsity=s0, sparsity_dcrt=dcrt, tile_size=16, block_size=128, video_len=video_len,
                    video_perm=vperm)
                kind = "refresh" if flag else "cached"
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            if layout == "seq":
                parallel.dfs_attention_sequence_parallel(q, k, v, L, fn)
            else:
                fn(q, k, v)
            e1.record()
            spans.append((kind, round(cur, 6), e0, e1))
    torch.cuda.synchronize()
    return [(kind, s, e0.elapsed_time(e1)) for kind, s, e0, e1 in spans]


def trace_inputs(rk, spec, layers, layout):
    from dfsattn_b200 import parallel
    from dfsattn_b200.synthetic import structured_qkv
    H, D = spec["heads"], spec["dim"]
    h_local = H // rk.world
    base = []
    for layer in range(layers):
        if layout == "seq":
            full = structured_qkv(spec["grid"], H, D, text_len=spec["text"], dtype=torch.bfloat16, device=rk.dev,
                                  seed=layer)
            t0, tn = parallel.seq_shard(full[0].shape[2], rk.rank, rk.world)
            base.append(tuple(t[:, :, t0:t0 + tn].contiguous() for t in full))
            del full
        else:
            base.append(structured_qkv(spec["grid"], h_local, D, text_len=spec["text"], dtype=torch.bfloat16,
                                       device=rk.dev, seed=layer, head_offset=rk.rank * h_local, total_heads=H))
    return base


def trace_flops(spec, layers, h_local, L):
    """Algorithmic FLOPs of one trace on this rank: dense calls 4*D*L^2 per head, sparse calls
    4*D*pairs of the lists they ran on (read back from the cache the trace left behind)."""
    from dfsattn_b200 import ops
    from dfsattn_b200.attention_hyvideo import DFS_Attention, _compute_cache_schedule
    pairs = {}
    for key, entry in DFS_Attention._cached_metadata.items():
        lists = entry["block_lists"]
        pairs[(key[0], round(key[4], 6))] = ops.interaction_count(lists.idx, lists.cnt, h_local, L)
    flops = 0.0
    for step in range(50):
        _, cur = _compute_cache_schedule(step, 12, 12, spec["sparsity"], 0.1)
        for layer in range(layers):
            flops += 4.0 * spec["dim"] * (h_local * L * L if step < 12 else pairs[(layer, round(cur, 6))])
    return flops


def summarize_trace(rk, spec, layers, runs, L):
    """(seconds per trace: max over ranks, FLOPs per trace: all ranks, per-kind table)."""
    h_local = spec["heads"] // rk.world
    totals, per_kind = [], {}
    for ms in runs:
        totals.append(sum(t for _, _, t in ms))
        for kind, s, t in ms:
            per_kind.setdefault(kind if kind == "dense" else f"{kind}@{s:g}", []).append(t)
    secs = rk.max(sum(totals) / len(totals) / 1e3)
    flops = rk.sum(trace_flops(spec, layers, h_local, L))
    table = {k: {"calls_per_trace": len(v) // len(runs), "mean_ms": rk.max(sum(v) / len(v))}
             for k, v in sorted(per_kind.items())}
    return secs, flops, table


def run_trace(args, spec, rank, local_rank, world):
    """Workloads *_trace: one bench step is the whole 50-step trace; the time is the sum of the
    CUDA-event intervals around the attention calls (max over ranks)."""
    from dfsattn_b200 import ops
    from dfsattn_b200.order import hilbert3d_perm
    rk = Ranks(rank, local_rank, world)
    H, D = spec["heads"], spec["dim"]
    if H % world != 0:
        raise SystemExit(f"{H} heads do not split over {world} ranks")
    layout = "seq" if args.layout == "seq" and world > 1 else "head"
    if args.layout == "seq-fused":
        raise SystemExit("the trace runs head-sharded (--layout head) or with NCCL all-to-alls (--layout seq)")
    layers = args.trace_layers
    vperm = hilbert3d_perm(*spec["grid"])
    base = trace_inputs(rk, spec, layers, layout)
    L = spec["grid"][0] * spec["grid"][1] * spec["grid"][2] + spec["text"]
    for _ in range(args.warmup):
        trace_pass(rk, spec, base, vperm, layout)
    sampler = ClockSampler(local_rank)
    sampler.start()
    rk.barrier()
    runs = [trace_pass(rk, spec, base, vperm, layout) for _ in range(args.steps)]
    rk.barrier()
    clocks = sampler.stop()
    ops.check_status(rk.dev)
    secs, flops, table = summarize_trace(rk, spec, layers, runs, L)
    cycles = rk.max(1e3 * secs * (clocks["sm_mhz"] or 0.0))
    if rank == 0:
        pk = peaks()
        value = flops / secs / 1e12
        config = workload_config(args, spec, world)
        config.update({"layers": layers, "denoising_steps": 50,
                       "schedule": {"skip_steps": 12, "cache_interval": 12, "sparsity": spec["sparsity"],
                                    "sparsity_dcrt": 0.1},
                       "step": "one 50-step trace: dense warm-up calls, refresh calls, calls on cached lists",
                       "parallelism": (f"sequence-sharded x{world}: NCCL all-to-all in and out around every call"
                                       if layout == "seq" else f"head-sharded x{world}, no collective"),
                       "l2": "inputs larger than L2 (no flush needed)", "flops_per_trace": flops})
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": 1e3 * secs, "ms_x_mhz": cycles, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": config,
            "clocks": clocks,
            # every call: status snapshot; dense call: + the attention kernel; cached: + permute + attention;
            # refresh: + pool, tile scores, block sums and selection
            "gpu_launches": args.steps * sum(v["calls_per_trace"] * (2 if k == "dense" else 7 if
                                             k.startswith("refresh") else 3) for k, v in table.items()),
            "calls_ms": table,
            "roofline": {"bound": "tensor", "kernel": "bsattn_fwd_kernel<128>", "achieved": value / world,
                         "peak": pk["bf16_tflops_sustained"], "unit": "TFLOP/s",
                         "frac": value / world / pk["bf16_tflops_sustained"],
                         "peak_source": f"{pk['source']} sustained cuBLAS bf16", "traffic": None},
            "e2e": None, "cpu_baseline": None,
        }
        print(json.dumps(line), flush=True)
    rk.close()


# ---- the other configurations, one timed call each ------------------------------
def other_configs(rk, args):
    """One timed refresh call each of the Wan shapes (480p; 720p at three sparsities and in raster
    order) and one 50-step, 1-layer mask-caching trace of the HunyuanVideo 720p shape, all sharded
    over the ranks of this run by head; at N > 1 the trace also with sequence-sharded inputs."""
    from dfsattn_b200.order import hilbert3d_perm
    from dfsattn_b200.synthetic import structured_qkv
    out = {}
    cases = [("wan_480p", 0.3, "hilbert3d"), ("wan_720p", 0.1, "hilbert3d"), ("wan_720p", 0.3, "hilbert3d"),
             ("wan_720p", 0.5, "hilbert3d"), ("wan_720p", 0.3, "org")]
    held = (None, None)
    for name, sparsity, order in cases:
        spec = dict(WORKLOADS[name], sparsity=sparsity, order=order)
        H, D = spec["heads"], spec["dim"]
        if H % rk.world:
            continue
        h_local = H // rk.world
        if held[0] != name:
            held = (None, None)
            held = (name, structured_qkv(spec["grid"], h_local, D, dtype=torch.bfloat16, device=rk.dev, seed=0,
                                         head_offset=rk.rank * h_local, total_heads=H))
        q, k, v = held[1]
        L = q.shape[2]
        vperm = hilbert3d_perm(*spec["grid"]) if order == "hilbert3d" else None
        call = operator_call(spec, vperm, L, layer_idx=("cfg", name, sparsity, order))
        attention_class(spec).clear_cache()
        secs = rk.max(timed(lambda: call(q, k, v), 3, rk.barrier, warm=2) / 3)
        pairs, _ = cached_pairs(spec, h_local, L)
        flops = rk.sum(4.0 * D * pairs)
        out[f"{name}_s{sparsity:g}_{'hilbert3d' if order == 'hilbert3d' else 'raster'}"] = {
            "ms_per_call": 1e3 * secs, "tflops": flops / secs / 1e12, "heads_per_gpu": h_local, "seq_len": L}
        attention_class(spec).clear_cache()
    del held
    spec = dict(WORKLOADS["hunyuan_720p_trace"], order="hilbert3d")
    if spec["heads"] % rk.world == 0:
        vperm = hilbert3d_perm(*spec["grid"])
        L = spec["grid"][0] * spec["grid"][1] * spec["grid"][2] + spec["text"]
        for layout in (["head", "seq"] if rk.world > 1 else ["head"]):
            base = trace_inputs(rk, spec, 1, layout)
            rk.barrier()
            run = trace_pass(rk, spec, base, vperm, layout)
            secs, flops, table = summarize_trace(rk, spec, 1, [run], L)
            out[f"hunyuan_720p_trace_1layer_{layout}"] = {
                "ms_per_trace": 1e3 * secs, "tflops": flops / secs / 1e12,
                "calls_ms": {k: round(v["mean_ms"], 3) for k, v in table.items()}}
            del base
        attention_class(spec).clear_cache()
    return out


# ---- sequence-sharded inputs (N > 1) ----------------------------------------------
def sequence_layouts(rk, spec, vperm, flops_total):
    """The step with inputs that arrive sequence-sharded, both forms: NCCL all-to-alls around the
    head-sharded call, and the fused exchange (peer loads in the gather, peer stores in the attention
    epilogue); the two all-to-alls alone; and on a small case whether both forms give the bits of
    the single-GPU call."""
    from dfsattn_b200 import engine, parallel
    from dfsattn_b200.attention_hyvideo import DFS_Attention, _dfs_attention_instances, dfs_attention
    from dfsattn_b200.order import hilbert3d_perm
    from dfsattn_b200.synthetic import structured_qkv
    H, D = spec["heads"], spec["dim"]
    full = structured_qkv(spec["grid"], H, D, text_len=spec["text"], dtype=torch.bfloat16, device=rk.dev, seed=0)
    L = full[0].shape[2]
    video_len = L - spec["text"]
    t0, tn = parallel.seq_shard(L, rk.rank, rk.world)
    shards = tuple(t[:, :, t0:t0 + tn].contiguous() for t in full)
    del full
    head_call = operator_call(spec, vperm, video_len, layer_idx=("seq",))
    out = {}
    secs = timed(lambda: parallel.dfs_attention_sequence_parallel(*shards, L, head_call), 3, rk.barrier, warm=2) / 3
    out["seq_ms"] = 1e3 * rk.max(secs)

    def swaps_only():
        heads = parallel.seq_to_head_shards([t[0] for t in shards], L)
        parallel.head_to_seq_shards(heads[0], H)
    out["all_to_all_ms"] = 1e3 * rk.max(timed(swaps_only, 3, rk.barrier, warm=1) / 3)
    exchange = parallel.SequenceShardExchange(H, L, D, rk.dev)
    for dst, src in zip(exchange.inputs(), shards):
        dst.copy_(src[0])
    perm_dev, _ = engine._perm_cache.get(vperm, L, video_len, rk.dev)
    secs = timed(lambda: exchange.run(head_call, perm_dev), 3, rk.barrier, warm=2) / 3
    out["seq_fused_ms"] = 1e3 * rk.max(secs)
    out["seq_tflops"] = flops_total / (out["seq_ms"] / 1e3) / 1e12
    out["seq_fused_tflops"] = flops_total / (out["seq_fused_ms"] / 1e3) / 1e12
    del exchange, shards

    # parity on a small case (L = 1360: neither a multiple of the world size nor of 128)
    grid, text, Hs = (5, 12, 21), 100, 8
    q, k, v = structured_qkv(grid, Hs, D, text_len=text, dtype=torch.bfloat16, device=rk.dev, seed=0)
    Ls = q.shape[2]
    sperm = hilbert3d_perm(*grid)
    kw = dict(step_idx=12, skip_steps=12, cache_interval=12, sparsity=0.5, sparsity_dcrt=0.1, tile_size=16,
              block_size=128, video_len=Ls - text, video_perm=sperm, layer_idx=("seq-parity",))

    def reset():
        DFS_Attention.clear_cache()
        _dfs_attention_instances.clear()
    s0, sn = parallel.seq_shard(Ls, rk.rank, rk.world)
    small = [t[:, :, s0:s0 + sn].contiguous() for t in (q, k, v)]
    reset()
    whole = dfs_attention(q, k, v, **kw)[0, :, s0:s0 + sn]
    reset()
    swapped = parallel.dfs_attention_sequence_parallel(*small, Ls, lambda a, b, c: dfs_attention(a, b, c, **kw))[0]
    reset()
    ex = parallel.SequenceShardExchange(Hs, Ls, D, rk.dev)
    for dst, src in zip(ex.inputs(), small):
        dst.copy_(src[0])
    sperm_dev, _ = engine._perm_cache.get(sperm, Ls, Ls - text, rk.dev)
    fused = ex.run(lambda a, b, c, **e: dfs_attention(a, b, c, **kw, **e), sperm_dev).clone()
    torch.cuda.synchronize()
    same = float(torch.equal(swapped, whole) and torch.equal(fused, whole))
    out["seq_parity"] = bool(rk.min(same) == 1.0)
    reset()
    return out


def copy_rates(rk, host_in, host_out, dev_in, dev_out):
    """Host<->device copy rates of this step's buffers with every rank copying at the same time:
    uploads alone, downloads alone, and both directions together on two streams (the floor of the
    host-buffer call: nothing of it can end before its bytes have crossed)."""
    up_s, down_s = torch.cuda.Stream(rk.dev), torch.cuda.Stream(rk.dev)
    cur = torch.cuda.current_stream(rk.dev)

    def up():
        up_s.wait_stream(cur)
        with torch.cuda.stream(up_s):
            for d, h in zip(dev_in, host_in):
                d.copy_(h, non_blocking=True)
        cur.wait_stream(up_s)

    def down():
        down_s.wait_stream(cur)
        with torch.cuda.stream(down_s):
            host_out.copy_(dev_out, non_blocking=True)
        cur.wait_stream(down_s)

    def both():
        up_s.wait_stream(cur)
        down_s.wait_stream(cur)
        with torch.cuda.stream(up_s):
            for d, h in zip(dev_in, host_in):
                d.copy_(h, non_blocking=True)
        with torch.cuda.stream(down_s):
            host_out.copy_(dev_out, non_blocking=True)
        cur.wait_stream(up_s)
        cur.wait_stream(down_s)
    up_bytes = sum(h.numel() * h.element_size() for h in host_in)
    down_bytes = host_out.numel() * host_out.element_size()
    t_up = rk.max(timed(up, 3, rk.barrier, warm=1) / 3)
    t_down = rk.max(timed(down, 3, rk.barrier, warm=1) / 3)
    t_both = rk.max(timed(both, 3, rk.barrier, warm=1) / 3)
    return {"h2d_gbs_per_gpu": up_bytes / t_up / 1e9, "d2h_gbs_per_gpu": down_bytes / t_down / 1e9,
            "copy_only_ms": 1e3 * t_both}


def run_gpu(args, spec, rank, local_rank, world):
    from dfsattn_b200 import engine, ops
    from dfsattn_b200.order import hilbert3d_perm
    from dfsattn_b200.synthetic import structured_qkv

    rk = Ranks(rank, local_rank, world)
    dev, barrier = rk.dev, rk.barrier
    H, D = spec["heads"], spec["dim"]
    if H % world != 0:
        raise SystemExit(f"{H} heads do not split over {world} ranks")
    h_local = H // world
    f, h, w = spec["grid"]
    seq_layout = args.layout in ("seq", "seq-fused") and world > 1
    fused_exchange = args.layout == "seq-fused" and world > 1
    if seq_layout:
        # sequence-sharded inputs: every rank holds all heads for its contiguous range of raster tokens
        from dfsattn_b200 import parallel
        qf, kf, vf = structured_qkv(spec["grid"], H, D, text_len=spec["text"], dtype=torch.bfloat16, device=dev,
                                    seed=0)
        L = qf.shape[2]
        t0, tn = parallel.seq_shard(L, rank, world)
        q_seq, k_seq, v_seq = (t[:, :, t0:t0 + tn].contiguous() for t in (qf, kf, vf))
        h0 = rank * h_local
        q, k, v = (t[:, h0:h0 + h_local].contiguous() for t in (qf, kf, vf))   # for the per-stage timings
        del qf, kf, vf
    else:
        q, k, v = structured_qkv(spec["grid"], h_local, D, text_len=spec["text"], dtype=torch.bfloat16,
                                 device=dev, seed=0, head_offset=rank * h_local, total_heads=H)
    L = q.shape[2]
    video_len = L - spec["text"]
    vperm = hilbert3d_perm(f, h, w) if spec.get("order", "hilbert3d") == "hilbert3d" else None
    hy = spec["flavor"] == "hyvideo"
    Attn = attention_class(spec)
    call = operator_call(spec, vperm, video_len)

    if fused_exchange:
        # shards in symmetric memory; the gather reads peers, the attention epilogue writes peers
        head_call = call
        exchange = parallel.SequenceShardExchange(H, L, D, dev)
        for dst, src in zip(exchange.inputs(), (q_seq, k_seq, v_seq)):
            dst.copy_(src[0])
        perm_dev, _ = engine._perm_cache.get(vperm, L, video_len, dev)

        def call(qq, kk, vv):  # noqa: F811  (inputs are the exchange's own shard buffers)
            return exchange.run(head_call, perm_dev)[None]
        step_inputs = (q_seq, k_seq, v_seq)
    elif seq_layout:
        head_call = call

        def call(qq, kk, vv):  # noqa: F811  one all-to-all in (Q,K,V together), one out
            return parallel.dfs_attention_sequence_parallel(qq, kk, vv, L, head_call)
        step_inputs = (q_seq, k_seq, v_seq)
    else:
        step_inputs = (q, k, v)

    Attn.clear_cache()
    for _ in range(max(args.warmup, 3)):
        out = call(*step_inputs)
    torch.cuda.synchronize()
    ops.check_status(dev)
    pairs_local, lists = cached_pairs(spec, h_local, L)
    flops_total = rk.sum(4.0 * D * pairs_local)

    sampler = ClockSampler(local_rank)   # every rank samples its own GPU
    sampler.start()
    step_ms = []
    secs_local = timed(lambda: call(*step_inputs), args.steps, barrier, per_step=step_ms)
    secs = rk.max(secs_local)
    clocks = sampler.stop()
    # step time in SM clock cycles (ms x median MHz under load of the rank's own GPU, max over ranks):
    # the 1 -> N curve with the power cap's clock differences taken out
    ms_x_mhz = rk.max(1e3 * secs_local / args.steps * (clocks["sm_mhz"] or 0.0))
    ops.check_status(dev)
    ms_step = 1e3 * secs / args.steps
    value = flops_total / (secs / args.steps) / 1e12

    # ---- per-stage device times (same inputs, same stream) -----------------
    perm, _ = engine._perm_cache.get(vperm, L, video_len, dev)
    qh, kh, vh = q[0], k[0], v[0]
    n_stage = max(3, min(args.steps, 10))
    if perm is not None:
        qp, kp, vp = ops.permute_qkv(qh, kh, vh, perm)
        t_perm = timed(lambda: ops.permute_qkv(qh, kh, vh, perm), n_stage, barrier, warm=2) / n_stage
    else:  # raster order: no gather at all
        qp, kp, vp = qh.contiguous(), kh.contiguous(), vh.contiguous()
        t_perm = float("nan")
    t_score = timed(lambda: engine.compute_block_lists(qp, kp, video_len, spec["sparsity"], spec["flavor"]),
                    n_stage, barrier, warm=1) / n_stage
    out_buf = torch.empty_like(qp)
    t_attn = timed(lambda: ops.block_sparse_fwd(qp, kp, vp, lists.idx, lists.cnt, out_row_map=perm, out=out_buf),
                   n_stage, barrier, warm=1) / n_stage
    t_attn = rk.max(t_attn)
    # the dense call of the warm-up steps (every key block, no lists): same kernel family
    n_dense = 3
    t_dense = rk.max(timed(lambda: ops.block_sparse_fwd(qp, kp, vp, None, None, out_row_map=perm, out=out_buf),
                           n_dense, barrier, warm=1) / n_dense)
    pk = peaks()
    attn_tflops = 4.0 * D * pairs_local / t_attn / 1e12          # this rank's kernel
    tensor_bytes = h_local * L * D * 2
    # how much the lists of neighbouring query blocks (in Hilbert order) have in common: |A & B| / |A | B|
    member = lists.to_bool_mask()
    ranked = (lists.cnt >= 0)
    a, b = member[:, 0:-1:2], member[:, 1::2]
    nn = min(a.shape[1], b.shape[1])
    both_ranked = (ranked[:, 0:-1:2][:, :nn] & ranked[:, 1::2][:, :nn])
    inter = (a[:, :nn] & b[:, :nn]).sum(-1).float()
    union = (a[:, :nn] | b[:, :nn]).sum(-1).float()
    jaccard = float((inter / union)[both_ranked].mean()) if bool(both_ranked.any()) else None
    del member, a, b
    stages = {
        "permute_ms": None if perm is None else 1e3 * t_perm,
        "permute_gbs": None if perm is None else 6 * tensor_bytes / t_perm / 1e9,
        "score_select_ms": 1e3 * t_score,
        "score_select_gbs_algorithmic": (2 * tensor_bytes + lists.idx.numel() * 4) / t_score / 1e9,
        "attention_ms": 1e3 * t_attn,
        "dense_attention_ms": 1e3 * t_dense,
        "dense_attention_tflops": 4.0 * D * h_local * L * L / t_dense / 1e12,
        "adjacent_list_jaccard": jaccard,
    }

    if hy:
        # The kp selector (fine top-p over the 16 x 16-token tiles inside the chosen blocks): what the tile
        # maps cost at a refresh call and what the attention kernel takes with them (not part of `value`).
        kp_lists = engine.compute_block_lists(qp, kp, video_len, spec["sparsity"], "hyvideo", fine_top_p=0.9)
        t_kp = timed(lambda: engine.compute_block_lists(qp, kp, video_len, spec["sparsity"], "hyvideo",
                                                        fine_top_p=0.9), n_stage, barrier, warm=1) / n_stage
        t_kp_attn = timed(lambda: ops.block_sparse_fwd(qp, kp, vp, kp_lists.idx, kp_lists.cnt, out_row_map=perm,
                                                       out=out_buf, fine=kp_lists.fine), n_stage, barrier,
                          warm=1) / n_stage
        stages["kp_score_select_refine_ms"] = 1e3 * t_kp
        stages["kp_attention_ms"] = 1e3 * rk.max(t_kp_attn)
        bytes8 = kp_lists.fine.view(torch.uint8)
        kept = sum(int(((bytes8 >> b) & 1).sum()) for b in range(8))
        stages["kp_tiles_kept_frac"] = kept / (64.0 * int(kp_lists.cnt.clamp(min=0).sum()))
        del kp_lists, bytes8

    # The processor-side fused step that makes the permute above unnecessary: projections
    # [L, H*D] -> normalised, rotated, permuted head-major Q/K/V in one pass (not part of `value`).
    src = [torch.randn(L, h_local * D, device=dev, dtype=torch.bfloat16) for _ in range(3)]
    gam = torch.ones(D if hy else h_local * D, device=dev, dtype=torch.bfloat16)
    ang = torch.rand(video_len, D // 2, device=dev) * 6.2831853
    tabs = (ang.cos().repeat_interleave(2, 1).contiguous(), ang.sin().repeat_interleave(2, 1).contiguous()) \
        if hy else (ang.cos(), ang.sin())
    prep = lambda: ops.qkv_prepare(*src, h_local, gamma_q=gam, gamma_k=gam, norm_across_heads=not hy,  # noqa: E731
                                   cos=tabs[0], sin=tabs[1], rope_rows=video_len, perm=perm, out=(qp, kp, vp))
    t_prep = timed(prep, n_stage, barrier, warm=2) / n_stage
    stages["fused_prepare_ms"] = 1e3 * t_prep
    stages["fused_prepare_gbs"] = 6 * tensor_bytes / t_prep / 1e9
    del src, ang, tabs

    if not hy and not seq_layout:
        # Both guidance passes of a Wan denoising step (a reuse step: lists cached): two operator calls
        # one after the other, as the reference runs them, against the one batched call.
        from dfsattn_b200.attention_wan import dfs_attention as wan_attention, dfs_attention_cfg_pair
        wkw = dict(skip_steps=12, cache_interval=12, layer_idx=0, sparsity=spec["sparsity"], sparsity_dcrt=0.1,
                   tile_size=16, block_size=128, video_perm=vperm)
        q2, k2, v2 = (torch.cat([t, t.flip(1)]) for t in (q, k, v))

        def two_calls():
            wan_attention(q2[0:1], k2[0:1], v2[0:1], step_idx=26, **wkw)
            wan_attention(q2[1:2], k2[1:2], v2[1:2], step_idx=27, **wkw)
        pair_call = lambda: dfs_attention_cfg_pair(q2, k2, v2, step_idx=26, **wkw)  # noqa: E731
        # alternate the two forms (the clocks settle during the first loops under the power cap); best of two
        t_two = t_pair = float("inf")
        for rnd in range(2):
            t_two = min(t_two, timed(two_calls, n_stage, barrier, warm=2 - rnd) / n_stage)
            t_pair = min(t_pair, timed(pair_call, n_stage, barrier, warm=2 - rnd) / n_stage)
        stages["cfg_two_calls_ms"] = 1e3 * rk.max(t_two)
        stages["cfg_pair_call_ms"] = 1e3 * rk.max(t_pair)
        del q2, k2, v2

    # ---- end to end through the public API with HOST buffers ----------------
    hq, hk, hv = (t.cpu().pin_memory() for t in step_inputs)
    hout = torch.empty(out.shape, dtype=out.dtype).pin_memory()
    dq, dk, dv = (torch.empty_like(t) for t in step_inputs)

    from dfsattn_b200.host_io import dfs_attention_host
    host_kw = dict(skip_steps=12, cache_interval=12, sparsity=spec["sparsity"], sparsity_dcrt=0.1,
                   tile_size=16, block_size=128, video_perm=vperm)
    if hy:
        host_kw.update(step_idx=12, video_len=video_len)
    else:
        host_kw.update(step_idx=24)

    def e2e_step():
        if fused_exchange:  # upload straight into the symmetric shard buffers, download the result shard
            for dst, src in zip(exchange.inputs(), (hq, hk, hv)):
                dst.copy_(src[0], non_blocking=True)
            hout.copy_(call(None, None, None), non_blocking=True)
        elif seq_layout:  # sequence shards: upload, swap, compute, swap back, download
            dq.copy_(hq, non_blocking=True)
            dk.copy_(hk, non_blocking=True)
            dv.copy_(hv, non_blocking=True)
            hout.copy_(call(dq, dk, dv), non_blocking=True)
        else:           # the host-buffer entry point: copies of head groups overlap the kernels
            dfs_attention_host(hq, hk, hv, out=hout, head_groups=args.e2e_head_groups, device=dev,
                               flavor="hyvideo" if hy else "wan", layer_idx=1000, **host_kw)

    n_e2e = max(2, min(args.steps, 5))
    e_secs = rk.max(timed(e2e_step, n_e2e, barrier, warm=2) / n_e2e)
    ops.check_status(dev)
    e2e = {"value": flops_total / e_secs / 1e12, "unit": UNIT, "ms_per_call": 1e3 * e_secs,
           "h2d_bytes_per_step": 3 * tensor_bytes * world, "d2h_bytes_per_step": tensor_bytes * world}
    e2e.update(copy_rates(rk, (hq, hk, hv), hout, (dq, dk, dv), torch.empty_like(dq)))
    # what bounds the call from below: its kernels, or its bytes crossing the host link
    e2e["floor_ms"] = max(ms_step, e2e["copy_only_ms"])
    del hq, hk, hv, hout, dq, dk, dv
    rk.barrier()

    extras = {}
    if not args.no_extras:
        del q, k, v, qp, kp, vp, out_buf, out, step_inputs
        if seq_layout:
            del q_seq, k_seq, v_seq
        torch.cuda.empty_cache()
        try:
            if world > 1 and args.layout == "head":
                extras["layouts"] = sequence_layouts(rk, spec, vperm, flops_total)
        except Exception as exc:  # noqa: BLE001  (the headline line must not die with an extra)
            extras["layouts"] = {"error": f"{type(exc).__name__}: {exc}"}
        try:
            extras["configs"] = other_configs(rk, args)
        except Exception as exc:  # noqa: BLE001
            extras["configs"] = {"error": f"{type(exc).__name__}: {exc}"}
        ops.check_status(dev)

    if rank == 0:
        cpu = None
        if world == 1 and not args.no_cpu_baseline:
            cores = host_threads()
            fl, s, note = cpu_sample(spec, args.cpu_blocks)
            cpu = {"value": fl / s / 1e12, "unit": UNIT, "cores": cores, "kind": "port", "sample": note}
        peak = pk["bf16_tflops_sustained"]
        config = workload_config(args, spec, world)
        config.update({
            "parallelism": (f"sequence-sharded x{world}: gather from and scatter to peer shards over "
                            f"NVLink inside the permute and attention kernels" if fused_exchange
                            else f"sequence-sharded x{world}: NCCL all-to-all in and out around "
                            f"head-sharded compute" if seq_layout
                            else f"head-sharded x{world}, no collective"),
            "l2": "inputs larger than L2 (no flush needed)", "flops_per_call": flops_total})
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "ms_per_step_stats": quartiles(step_ms),
            "ms_x_mhz": ms_x_mhz,
            "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": config,
            "clocks": clocks,
            "e2e": e2e,
            "gpu_launches": 7 * args.steps,   # status snapshot, permute, pool, tile scores, block sums, selection, attention
            "stages": stages,
            "roofline": {"bound": "tensor", "kernel": "bsattn_fwd_kernel<128>", "achieved": attn_tflops,
                         "peak": peak, "unit": "TFLOP/s", "frac": attn_tflops / peak,
                         "peak_source": f"{pk['source']} sustained cuBLAS bf16 (kernel runs tens of ms)",
                         # DRAM bytes per launch: ncu capture of a small case (dram read 3.008 x and
                         # write 0.796 x one tensor), scaled by the tensor size of this launch
                         "traffic": 3.804 * tensor_bytes, "traffic_unit": "bytes",
                         "algorithmic_flops": 4.0 * D * pairs_local},
            "cpu_baseline": cpu,
        }
        line.update(extras)
        print(json.dumps(line), flush=True)
    rk.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="hunyuan_720p", choices=list(WORKLOADS))
    ap.add_argument("--cpu-blocks", type=int, default=384, help="query blocks per CPU sample")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the other configurations and the sequence-sharded layouts after the headline step")
    ap.add_argument("--sparsity", type=float, default=None, help="override the workload's sparsity")
    ap.add_argument("--order", default="hilbert3d", choices=["hilbert3d", "org"],
                    help="token order: 3-D Hilbert curve or raster (no permutation)")
    ap.add_argument("--e2e-head-groups", type=int, default=12,
                    help="head groups the host-buffer entry point pipelines its copies over")
    ap.add_argument("--trace-layers", type=int, default=2, help="layers of the *_trace workloads")
    ap.add_argument("--layout", default="head", choices=["head", "seq", "seq-fused"],
                    help="how inputs arrive at N > 1: head shards (no collective), sequence shards swapped by "
                         "NCCL all-to-alls, or sequence shards in symmetric memory read and written in place "
                         "by the permute and attention kernels")
    args = ap.parse_args()
    rank, local_rank, world = dist_env()
    spec = dict(WORKLOADS[args.workload])
    if args.sparsity is not None:
        spec["sparsity"] = args.sparsity
    spec["order"] = args.order
    if args.impl == "reference":
        run_reference(args, spec, rank, world)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback for the product path)")
    if spec.get("trace"):
        run_trace(args, spec, rank, local_rank, world)
    else:
        run_gpu(args, spec, rank, local_rank, world)


if __name__ == "__main__":
    main()
