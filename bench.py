#!/usr/bin/env python
"""Benchmark of the paged NVFP4 decode path on B200.

    python bench.py --gpus N --steps K --warmup W            # this library
    python bench.py --impl reference --gpus N --steps K ...   # the CPU oracle path

One "step" is one decode step of one attention layer over the whole batch:
Q quantisation + split-KV paged decode, ONE launch (the decode kernel quantises the
BF16 query itself; the LSE merge is a second launch of the same call when it splits).  The workload is the uniform batch-decode configuration:
32 sequences x 4096 context, 32 query heads / 8 KV heads / head_dim 128,
128-token pages, key shift applied when the pages were written, no BF16 tail.

Prints ONE JSON line (rank 0).
"""

from __future__ import annotations

import argparse
import ctypes
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

ROWS, CTX, HQ, HKV, D, PAGE = 32, 4096, 32, 8, 128, 128
PAGES_PER_ROW = CTX // PAGE
POOL_PAGES = ROWS * PAGES_PER_ROW          # 1024 pages = 151 MB of NVFP4 K+V per pool
NUM_POOLS = 2                              # alternate so that L2 (126 MB) cannot hold a step's KV
KV_BYTES = ROWS * CTX * HKV * 144          # algorithmic bytes of one step (144 B per token-head)
# dram__bytes_read.sum + dram__bytes_write.sum of one decode launch of the default workload, from
# an ncu capture of that kernel (a constant: this program does not measure it)
NCU_TRAFFIC_BYTES = 151_752_448 + 5_598_592   # read + written, mean of the two captured launches
METRIC = "decode_attn_tokens_per_s"
UNIT = "tokens/s"
WORKLOAD = ("uniform batch decode: 32 seq x 4096 ctx, Hq32/Hkv8/D128, page 128, "
            "NVFP4 K/V (key shift applied at write), tail 0, bf16 out, 1 layer")


def set_context(ctx: int) -> None:
    """Re-derive the workload constants for a non-default context length (exploration only)."""
    global CTX, PAGES_PER_ROW, POOL_PAGES, KV_BYTES, WORKLOAD
    if ctx % PAGE:
        raise SystemExit("--ctx must be a multiple of 128")
    CTX = ctx
    PAGES_PER_ROW = CTX // PAGE
    POOL_PAGES = ROWS * PAGES_PER_ROW
    KV_BYTES = ROWS * CTX * HKV * 144
    WORKLOAD = WORKLOAD.replace("4096 ctx", f"{ctx} ctx")


# --------------------------------------------------------------------------- CPU arm
def _cpu_row(args):
    """One sequence of the workload through the CPU oracle (quantises Q/K/V itself)."""
    seed, ctx = args
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import numpy as np

    import nvfp4_oracle as O

    rng = np.random.default_rng(seed)
    pages = ctx // PAGE
    q = O.bf16_round(rng.standard_normal((1, HQ, D)).astype(np.float32))
    off = rng.standard_normal((HKV, D)).astype(np.float32) * 2.0
    k = O.bf16_round(rng.standard_normal((pages, PAGE, HKV, D)).astype(np.float32) + off)
    mu = O.bf16_round(k.reshape(-1, HKV, D).astype(np.float64).mean(0).astype(np.float32))
    k = O.bf16_round(k - mu)
    v = O.bf16_round(rng.standard_normal((pages, PAGE, HKV, D)).astype(np.float32))
    table = rng.permutation(pages).astype(np.int32).reshape(1, pages)
    t0 = time.perf_counter()
    out = O.reference_decode(q, k, v, table, np.array([ctx]), np.array([0]), np.array([0]),
                             D ** -0.5)
    return time.perf_counter() - t0, float(np.abs(out).sum())


def cpu_path(steps: int, warmup: int, rows_per_step: int | None = None):
    """Time the CPU oracle on a bounded sample of the workload, all host cores."""
    import multiprocessing as mp

    cores = os.cpu_count() or 1
    rows = rows_per_step or min(ROWS, cores)
    ctx = mp.get_context("spawn")
    os.environ.setdefault("OMP_NUM_THREADS", "1")
    workers = min(cores, rows)
    per_step = []
    with ctx.Pool(workers) as pool:
        for w in range(warmup):
            pool.map(_cpu_row, [(1000 + w * rows + r, CTX) for r in range(rows)])
        for s in range(steps):
            # input generation happens inside the workers but outside their timers; a step's time is
            # the oracle work with every worker busy
            per_step.append(sum(t for t, _ in pool.map(_cpu_row, [(s * rows + r, CTX) for r in range(rows)]))
                            / workers)
    dt = sorted(per_step)[len(per_step) // 2]
    return dict(
        value=rows / dt,
        ms_per_step=1e3 * dt,
        cores=min(cores, rows),
        rows=rows,
        sample=f"median of {steps} step(s) after {warmup} warm-up, each {rows} of the {ROWS} sequences "
               f"({CTX} ctx each, Q/K/V/P quantisation included), one process per sequence on "
               f"{min(cores, rows)} cores",
    )


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps = max(1, min(args.steps, 5))
    res = cpu_path(steps, min(args.warmup, 1))
    line = {
        "impl": "reference",
        "metric": METRIC, "value": res["value"], "unit": UNIT, "n_gpus": args.gpus,
        "steps": steps, "warmup": min(args.warmup, 1), "ms_per_step": res["ms_per_step"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "nvfp4", "data": "synthetic",
        "config": {"workload": WORKLOAD, "arm": "numpy restatement of the reference's torch oracle"},
        "cpu_baseline": {"value": res["value"], "unit": UNIT, "cores": res["cores"],
                         "kind": "port", "sample": res["sample"]},
        "e2e": {"value": res["value"], "unit": UNIT, "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------- GPU arm
class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.samples = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "20"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append([p.strip() for p in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        mhz, mx, reasons = [], None, set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for s in self.samples:
            if len(s) < 6:
                continue
            try:
                mhz.append(float(s[0]))
                mx = float(s[1])
            except ValueError:
                continue
            for name, flag in zip(names, s[2:6]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        mhz.sort()
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": mx,
                "reasons": sorted(reasons), "samples": len(mhz)}


REPEATS = 5   # timed regions per number; the number is their median


class StepState:
    """Device state that a serving step advances (the lengths and the slot table): kept after
    the warm-up and put back before every repeat, so that the repeats time the same steps."""

    def __init__(self, plane, seq_lens):
        self.tensors = [seq_lens, plane.slot_keys, plane.slot_last_seq, plane.slot_last_seen, plane.step]
        self.saved = [t.clone() for t in self.tensors]

    def restore(self):
        for t, s in zip(self.tensors, self.saved):
            t.copy_(s)


def build_pools(device, rows=None, pages_per_row=None, num_pools=None, hkv=None):
    """Disjoint page pools in the vLLM block layout, filled by the library's quantisers."""
    import torch

    from nvfp4_attn_kernel_b200.nvfp4_decode_kernel import quantize_kv_kernel as qkv

    ROWS_, PAGES_PER_ROW_ = rows or ROWS, pages_per_row or PAGES_PER_ROW
    POOL_PAGES_ = ROWS_ * PAGES_PER_ROW_
    NUM_POOLS_ = num_pools or NUM_POOLS
    HKV_ = hkv or HKV

    block = 2 * (PAGE * HKV_ * 64 + HKV_ * 1024)
    o1 = PAGE * HKV_ * 64
    o2 = o1 + HKV_ * 1024
    o3 = o2 + o1
    pools = []
    gen = torch.Generator(device=device)
    gen.manual_seed(1234)
    for _ in range(NUM_POOLS_):
        cache = torch.empty(POOL_PAGES_, block, dtype=torch.uint8, device=device)
        flat = cache.view(-1)
        kview = flat.as_strided((POOL_PAGES_, PAGE, HKV_, 64), (block, HKV_ * 64, 64, 1), 0)
        vview = flat.as_strided((POOL_PAGES_, HKV_, D, 64), (block, D * 64, 64, 1), o2)
        ksf = qkv.scale_view(flat, POOL_PAGES_, HKV_, block, o1)
        vsf = qkv.scale_view(flat, POOL_PAGES_, HKV_, block, o3)
        chunk = min(128, POOL_PAGES_)
        while POOL_PAGES_ % chunk:
            chunk -= 1
        offset = torch.randn(HKV_, D, device=device, generator=gen) * 2.0
        shift = None
        for lo in range(0, POOL_PAGES_, chunk):
            k = (torch.randn(chunk * PAGE, HKV_, D, device=device, generator=gen) + offset).to(torch.bfloat16)
            v = torch.randn(chunk * PAGE, HKV_, D, device=device, generator=gen).to(torch.bfloat16)
            if shift is None:
                shift = k.double().mean(0).to(torch.bfloat16).contiguous()  # per-channel K mean
            src = torch.arange(chunk, dtype=torch.int32, device=device) * PAGE
            dst = torch.arange(lo, lo + chunk, dtype=torch.int32, device=device)
            qkv.quantize_key_tokens_into(k, kview, ksf, src, dst, key_shift=shift)
            qkv.quantize_value_tokens_into(v, vview, vsf, src, dst)
        table = torch.randperm(POOL_PAGES_, device=device, generator=gen).to(torch.int32).reshape(
            ROWS_, PAGES_PER_ROW_)
        pools.append(dict(cache=cache, k=kview, ksf=ksf, v=vview, vsf=vsf, table=table, block=block))
    return pools


def load_peaks():
    try:
        return json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except (OSError, ValueError):
        return {}


def pin_rank_to_cores(local: int, world: int) -> str:
    """One process per GPU on one host: give every rank its own slice of the host's cores, so
    that eight Python interpreters do not migrate over each other's caches."""
    try:
        cores = sorted(os.sched_getaffinity(0))
        if world > 1 and len(cores) >= 2 * world:
            per = len(cores) // world
            mine = cores[local * per:(local + 1) * per]
            os.sched_setaffinity(0, mine)
            return f"{per} cores per rank"
    except (AttributeError, OSError):
        pass
    return "unpinned"


def _median(xs):
    xs = sorted(xs)
    return xs[len(xs) // 2]


def sampled_row_parity(pool, q, out_row, row, device):
    """max-abs of one output row against the CPU attention oracle fed the library's own
    dequantised bytes of that row's pages.  Test infrastructure used as a checker, outside every
    timed region."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import numpy as np
    import torch

    import nvfp4_oracle as O
    from nvfp4_attn_kernel_b200.nvfp4_decode_kernel import _quantize

    ids = pool["table"][row].long()
    k_dq = O.dequantize_key_pages(pool["k"][ids].contiguous().cpu().numpy(),
                                  _scale_rows(pool["ksf"], ids))
    v_dq = O.dequantize_value_pages(pool["v"][ids].contiguous().cpu().numpy(),
                                    _scale_rows(pool["vsf"], ids))
    q_fp4, q_sf = _quantize.quantize_query(q[row:row + 1].contiguous(), heads_kv=HKV)
    storage = q_sf.as_strided((1, HQ * 1024), (HQ * 1024, 1)).cpu().numpy().reshape(1, 1, HQ, 2, 32, 4, 4)
    q_dq = O.dequantize_query(q_fp4.view(torch.uint8).cpu().numpy(), storage, HKV)
    n = ids.numel()
    want = O.attention_from_dequantized(
        q[row:row + 1].float().cpu().numpy(), q_dq, k_dq, v_dq, np.arange(n, dtype=np.int32).reshape(1, n),
        np.array([n * PAGE], dtype=np.int32), softmax_scale=D ** -0.5)
    return float(np.abs(out_row.float().cpu().numpy() - want[0]).max())


def _scale_rows(view, ids):
    """[len(ids), Hkv * 1024] scale bytes of the given pages of a pitched scale view."""
    import torch

    heads = view.shape[-1]
    flat = view.view(torch.uint8).as_strided((view.shape[0], heads * 1024), (view.stride(0), 1),
                                             view.storage_offset())
    return flat[ids].contiguous().cpu().numpy()


def run_gpu(args) -> None:
    import torch
    import torch.distributed as dist

    import nvfp4_attn_kernel_b200._lib as L
    from nvfp4_attn_kernel_b200.nvfp4_decode_kernel import host_io_step

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU fallback for the kernels")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    pinning = pin_rank_to_cores(local, world)
    if world > 1:
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")   # the page-range exchange below uses plain peer stores
        dist.init_process_group("nccl", device_id=device)
    lib = L.load()
    impl = {"auto": L.IMPL_AUTO, "generic": L.IMPL_GENERIC, "sm100": L.IMPL_SM100}[args.decode_impl]

    pools = build_pools(device)
    gen = torch.Generator(device=device)
    gen.manual_seed(99 + rank)
    q = torch.randn(ROWS, HQ, D, device=device, generator=gen).to(torch.bfloat16)
    q_fp4 = torch.zeros(ROWS, 1, HQ, 64, dtype=torch.uint8, device=device)
    q_sf = torch.zeros(ROWS, HQ * 1024, dtype=torch.uint8, device=device)
    out = torch.zeros(ROWS, HQ, D, dtype=torch.bfloat16, device=device)
    seqused = torch.full((ROWS,), CTX, dtype=torch.int32, device=device)
    splits = args.num_splits
    ws_bytes = lib.nvfp4_decode_workspace_bytes(ROWS, HQ, splits)
    workspace = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=device)
    status = torch.zeros(1, dtype=torch.int32, device=device)

    def decode_args(pool):
        a = L.DecodeArgs()
        a.q_fp4, a.q_sf = q_fp4.data_ptr(), q_sf.data_ptr()
        a.k_packed, a.k_pitch = pool["k"].data_ptr(), pool["block"]
        a.k_sf, a.k_sf_pitch = pool["ksf"].data_ptr(), pool["block"]
        a.v_packed, a.v_pitch = pool["v"].data_ptr(), pool["block"]
        a.v_sf, a.v_sf_pitch = pool["vsf"].data_ptr(), pool["block"]
        a.num_pages = POOL_PAGES
        a.page_table, a.page_table_row_stride, a.max_pages = pool["table"].data_ptr(), PAGES_PER_ROW, PAGES_PER_ROW
        a.seqused_fp4 = seqused.data_ptr()
        a.out = out.data_ptr()
        a.rows, a.heads_q, a.heads_kv = ROWS, HQ, HKV
        a.softmax_scale = D ** -0.5
        a.num_splits, a.impl = splits, impl
        a.workspace, a.workspace_bytes = workspace.data_ptr(), ws_bytes
        a.status = status.data_ptr()
        return a

    dargs = [decode_args(p) for p in pools]
    # the step as a caller runs it: ONE launch that takes the BF16 query and quantises it inside
    fused = [decode_args(p) for p in pools]
    pdl = bool(args.pdl and splits == 1 and args.decode_impl != "generic")
    for a in fused:
        a.q_fp4, a.q_sf = None, None
        a.q_bf16, a.q_bf16_row_stride, a.q_bf16_head_stride = q.data_ptr(), q.stride(0), q.stride(1)
        # consecutive steps are chained with programmatic stream serialization: a launch's set-up
        # and first page loads overlap the previous launch's drain (the pages are not its output)
        a.flags = L.DECODE_PROGRAMMATIC_LAUNCH if pdl else 0
    L.check(lib.nvfp4_quantize_q(q.data_ptr(), q.stride(0), q.stride(1), None, q_fp4.data_ptr(),
                                 q_sf.data_ptr(), None, ROWS, HQ, HKV,
                                 torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()

    def step(i, stream, with_q=True):
        """with_q: BF16 query in, quantised inside the decode launch; else the query was
        quantised beforehand and the launch only streams the pages."""
        L.check(lib.nvfp4_decode(ctypes.byref((fused if with_q else dargs)[i % NUM_POOLS]), stream))

    def make_graph(with_q):
        """NUM_POOLS steps (one per page pool) in one CUDA graph on a side stream."""
        side = torch.cuda.Stream(device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for i in range(4):
                step(i, side.cuda_stream, with_q)
        side.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            for i in range(NUM_POOLS):
                step(i, torch.cuda.current_stream().cuda_stream, with_q)
        return graph

    def timed(graph, replays):
        """ms for `replays` replays: barrier + synchronize on both sides, CUDA events, max over ranks."""
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(replays):
            graph.replay()
        end.record()
        torch.cuda.synchronize()
        ms = start.elapsed_time(end)
        if world > 1:
            t = torch.tensor([ms], dtype=torch.float64, device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
            dist.barrier()
        return ms

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    g_step, g_kernel = make_graph(True), make_graph(False)
    for _ in range(max(2, args.warmup // NUM_POOLS)):
        g_step.replay()
        g_kernel.replay()
    # (1) the contract's region: exactly --steps steps, five times over; the line's value is the median
    k_replays = max(1, args.steps // NUM_POOLS)
    done = k_replays * NUM_POOLS
    k_ms = [timed(g_step, k_replays) / done for _ in range(REPEATS)]
    ms_step = _median(k_ms)
    # (2) long repeats (each at least 20 ms, so that the clock sampler sees the load): the step and
    #     the decode kernel alone (pre-quantised query, plain launches inside the graph)
    long_replays = max(k_replays, int(20.0 / (ms_step * NUM_POOLS)) + 1)
    long_step = [timed(g_step, long_replays) / (long_replays * NUM_POOLS) for _ in range(REPEATS)]
    long_kernel = [timed(g_kernel, long_replays) / (long_replays * NUM_POOLS) for _ in range(REPEATS)]
    clocks = sampler.stop() if rank == 0 else None
    kernel_s = _median(long_kernel) * 1e-3

    # the floor on this GPU: a launch that only reads the step's bytes, same pools, same timing
    def read_floor():
        import ctypes

        from nvfp4_attn_kernel_b200 import build as _build

        read_floor_lib = ctypes.CDLL(_build.BENCH_AID_PATH)   # a measurement aid, not the product library
        read_floor_lib.bench_read_floor.restype = ctypes.c_int
        read_floor_lib.bench_read_floor.argtypes = [ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p,
                                                    ctypes.c_void_p]
        sink = torch.zeros(1, dtype=torch.int32, device=device)
        side = torch.cuda.Stream(device)
        side.wait_stream(torch.cuda.current_stream())
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            for i in range(NUM_POOLS):
                cache = pools[i]["cache"]
                rc = read_floor_lib.bench_read_floor(cache.data_ptr(), cache.numel(), sink.data_ptr(),
                                                     torch.cuda.current_stream().cuda_stream)
                if rc:
                    raise RuntimeError(f"bench_read_floor: CUDA error {rc}")
        for _ in range(3):
            graph.replay()
        reps = max(50, long_replays // 2)
        return _median([timed(graph, reps) / (reps * NUM_POOLS) for _ in range(3)]) * 1e-3

    floor_s = read_floor()

    # end to end through the operator's host-buffer call: pinned query in, pinned rows out, the
    # copies and the wait inside the timed region, one call into the library per step
    q_host = q.cpu().pin_memory()
    out_host = torch.empty_like(out, device="cpu").pin_memory()
    q_dev = torch.empty_like(q)
    host_steps = [host_io_step(q_dev, p["k"], p["ksf"], p["v"], p["vsf"], p["table"], seqused, out=out)
                  for p in pools]
    # the same step without copy operations: the kernel reads and writes the pinned buffers itself
    direct_steps = [host_io_step(q_dev, p["k"], p["ksf"], p["v"], p["vsf"], p["table"], seqused, out=out,
                                 direct=True) for p in pools]
    out_host_direct = torch.empty_like(out, device="cpu").pin_memory()

    def e2e_region(n, steps=None, sink=None):
        steps = steps or host_steps
        sink = out_host if sink is None else sink
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        s2, e2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s2.record()
        for i in range(n):
            steps[i % NUM_POOLS](q_host, sink)
        e2.record()
        torch.cuda.synchronize()
        ms = s2.elapsed_time(e2)
        if world > 1:
            t = torch.tensor([ms], dtype=torch.float64, device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms / n

    e2e_steps = max(done, 200)
    e2e_region(max(3, min(args.warmup, 20)))
    e2e_ms = [e2e_region(e2e_steps) for _ in range(REPEATS)]
    e2e_step = _median(e2e_ms)
    e2e_region(max(3, min(args.warmup, 20)), direct_steps, out_host_direct)
    direct_ms = [e2e_region(e2e_steps, direct_steps, out_host_direct) for _ in range(REPEATS)]
    host_steps[0](q_host, out_host)
    direct_steps[0](q_host, out_host_direct)
    direct_same = bool(torch.equal(out_host, out_host_direct))
    if world > 1:
        dist.barrier()

    # parity of what was timed: one sampled row of the last step against the CPU oracle
    parity = None
    if rank == 0:
        L.check(lib.nvfp4_decode(ctypes.byref(fused[0]), torch.cuda.current_stream().cuda_stream))
        torch.cuda.synchronize()
        parity = {"row": 5, "max_abs_vs_oracle": sampled_row_parity(pools[0], q, out[5], 5, device),
                  "bound": 2e-2,
                  "oracle": "numpy attention oracle on the library's dequantised bytes of the row's 32 pages "
                            "(P quantised per 16 positions against the running maximum, as the reference's)"}
    bad = int(status.item())

    # the two partitioned workloads of the multi-GPU configurations, measured after the headline
    extras = {}
    if world > 1 and not args.no_multi_gpu_records:
        sub = argparse.Namespace(**vars(args))
        sub.steps, sub.warmup = 200, 20
        extras["long_context"] = run_long_context(sub, sub=True)
        # the same exchange at a size where streaming the pages outweighs the launch and the
        # exchange chain: 16 x 32768, four times the pages
        big = argparse.Namespace(**vars(sub))
        big.lc_rows, big.steps, big.warmup = 16, 96, 12
        extras["long_context_16_rows"] = run_long_context(big, sub=True, check=False)
        sub.steps, sub.warmup = 24, 4
        extras["tp_model_step"] = run_model_step(sub, sub=True)

    if rank == 0:
        peaks = load_peaks()
        peak = float(peaks.get("hbm_gbs", 6650.0))
        achieved = KV_BYTES / kernel_s / 1e9
        chained = KV_BYTES / (_median(long_step) * 1e-3) / 1e9
        cpu = None
        if world == 1 and not args.no_cpu_baseline:
            res = cpu_path(3, 1)
            cpu = {"value": res["value"], "unit": UNIT, "cores": res["cores"], "kind": "port",
                   "sample": res["sample"]}
        launches_per_step = 1 + (1 if splits > 1 else 0)   # decode (query quantised inside) [+ merge]
        launches = (REPEATS * done + REPEATS * 2 * long_replays * NUM_POOLS) * launches_per_step
        line = {
            "metric": METRIC, "value": world * ROWS / (ms_step * 1e-3), "unit": UNIT,
            "n_gpus": world, "steps": done, "warmup": args.warmup, "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "nvfp4", "data": "synthetic",
            "config": {
                "workload": WORKLOAD,
                "l2": f"{NUM_POOLS} rotating page pools of {KV_BYTES / 1e6:.0f} MB each (> 126 MB L2), "
                      "alternated every step",
                "timing": f"CUDA-graph replay, CUDA events on the replay stream, barrier + synchronize on "
                          f"both sides, max over ranks; value = median of {REPEATS} regions of exactly "
                          f"{done} steps",
                "step": "one decode launch (BF16 query quantised inside)"
                        + (", launches chained with programmatic stream serialization" if pdl else "")
                        + "; decode_kernel_us / roofline: the same kernel with a pre-quantised query, "
                          "plain launches",
                "decode_impl": args.decode_impl, "num_splits": splits,
                "sharding": "independent batch of 32 sequences per GPU, no collective"
                            + (f"; ranks pinned: {pinning}" if world > 1 else ""),
            },
            "repeats": {
                "n": REPEATS,
                "step_us": {"regions_of_steps": done, "median": ms_step * 1e3, "min": min(k_ms) * 1e3,
                            "max": max(k_ms) * 1e3},
                "step_us_long": {"steps_per_region": long_replays * NUM_POOLS, "median": _median(long_step) * 1e3,
                                 "min": min(long_step) * 1e3, "max": max(long_step) * 1e3},
                "decode_kernel_us_long": {"steps_per_region": long_replays * NUM_POOLS,
                                          "median": kernel_s * 1e6, "min": min(long_kernel) * 1e3,
                                          "max": max(long_kernel) * 1e3},
                "e2e_us": {"steps_per_region": e2e_steps, "median": e2e_step * 1e3, "min": min(e2e_ms) * 1e3,
                           "max": max(e2e_ms) * 1e3},
            },
            "hbm_gbs": achieved, "frac_of_8000": achieved / 8000.0,
            "decode_kernel_us": kernel_s * 1e6,
            "target": {"decode_kernel_us_for_75pct_of_8000_gbs": KV_BYTES / 6.0e12 * 1e6},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak,
                         "peak_source": "measured" if peaks else "fallback",
                         "basis": "decode kernel alone, pre-quantised query, plain launches (decode_kernel_us)",
                         "frac_of_chained_step": chained / peak,
                         "chained_step_note": "the step of identical launches chained with programmatic "
                                              "stream serialization hides a launch's set-up under its "
                                              "predecessor's drain; a best case, not the kernel",
                         "traffic": args.ncu_traffic if args.ncu_traffic is not None else (
                             NCU_TRAFFIC_BYTES if (CTX == 4096 and splits == 1 and args.decode_impl != "generic")
                             else None),
                         "traffic_source": "constant: dram__bytes_read.sum + dram__bytes_write.sum per launch of "
                                           "an ncu capture of this kernel and workload, not measured by this run",
                         "read_only_launch_us": floor_s * 1e6,
                         "kernel_over_read_only_launch": kernel_s / floor_s},
            "parity": parity,
            "cpu_baseline": cpu,
            "e2e": {"value": world * ROWS / (e2e_step * 1e-3), "unit": UNIT,
                    "h2d_bytes_per_step": q_host.numel() * 2, "d2h_bytes_per_step": out_host.numel() * 2,
                    "ms_per_step": e2e_step, "steps": e2e_steps,
                    "call": "host_io_step: nvfp4_decode_host_io (copy in, decode, copy out, wait) per step",
                    "without_copy_operations": {
                        "ms_per_step": _median(direct_ms), "min": min(direct_ms), "max": max(direct_ms),
                        "value": world * ROWS / (_median(direct_ms) * 1e-3),
                        "bitwise_equal_to_the_copy_form": direct_same,
                        "call": "host_io_step(direct=True): NVFP4_DECODE_HOST_IO_DIRECT, the kernel reads the "
                                "pinned query and writes the pinned rows over PCIe itself; one launch and the wait"}},
            "gpu_launches": launches,
            "clocks": clocks,
            "device_status_word": bad,
        }
        line.update(extras)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_long_context(args, sub: bool = False, check: bool = True):
    """Long-context workload: 4 sequences x 32768 context (``--lc-rows`` / ``--lc-ctx`` change the
    size), the KV pages of every sequence split by page range over the ranks (rank r holds only
    its pages), partial results merged over NVLink.  Strong scaling: the total work is fixed as
    the number of GPUs grows.
    ``sub``: called by the headline run on an initialised process group; returns the record
    (rank 0) instead of printing a line.  ``check``: also run the small correctness problem."""
    import torch
    import torch.distributed as dist

    import nvfp4_attn_kernel_b200._lib as L
    from nvfp4_attn_kernel_b200 import sharding
    from nvfp4_attn_kernel_b200.nvfp4_decode_kernel import _decode, _quantize
    from nvfp4_attn_kernel_b200.nvfp4_decode_kernel._decode import split_k_heuristic

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1 and not sub:
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=device)
    rows, ctx = args.lc_rows, args.lc_ctx
    pages = ctx // PAGE
    if pages % world:
        if sub:
            return {"skipped": f"{pages} pages do not divide over {world} ranks"} if rank == 0 else None
        raise SystemExit("the page count must divide over the ranks")
    local_pages = pages // world
    kv_bytes = rows * ctx * HKV * 144
    per_pool = rows * local_pages * 147456
    num_pools = max(2, -(-2 * 132 * 2 ** 20 // per_pool))   # together well past the 126 MB L2
    num_pools += num_pools & 1                               # the partial copies alternate in pairs
    pools = build_pools(device, rows, local_pages, num_pools)
    gen = torch.Generator(device=device)
    gen.manual_seed(7)                                       # the same query on every rank
    q = torch.randn(rows, HQ, D, device=device, generator=gen).to(torch.bfloat16)
    out = torch.zeros(rows, HQ, D, dtype=torch.bfloat16, device=device)
    seq = torch.full((rows,), local_pages * PAGE, dtype=torch.int32, device=device)
    q_fp4_s = torch.zeros(rows, 1, HQ, 64, dtype=torch.uint8, device=device)
    q_sf_s = torch.zeros(rows, 1, HQ, 2, 32, 4, 4, dtype=torch.uint8, device=device)
    # the kernel keeps two CTAs on an SM, so there are twice as many CTA slots as SMs
    slots = 2 * torch.cuda.get_device_properties(device).multi_processor_count
    splits = args.num_splits if args.num_splits > 1 else split_k_heuristic(rows, HKV, local_pages, sms=slots)
    grp = (sharding.PageRangeGroup(dist.group.WORLD, rows, HQ, device, args.exchange, heads_kv=HKV)
           if world > 1 else None)

    def step(i):
        pool = pools[i % num_pools]
        common = dict(query_fp4=None, query_scales=None, query_padded_bf16=None, query_bf16=q,
                      key_pages_fp4=pool["k"], key_scales=pool["ksf"], value_pages_fp4=pool["v"],
                      value_scales=pool["vsf"], fp4_page_table=pool["table"], seqused_fp4=seq,
                      softmax_scale=D ** -0.5, trusted_metadata=True)
        if grp is None:
            _decode.decode_fp4_split(**{k: v for k, v in common.items() if k != "query_padded_bf16"},
                                     num_splits=splits, out=out)
        elif args.exchange == "fused":
            # decode, fold of the local splits, push, wait and merge: ONE launch
            parts = grp.local_split_buffers(splits) if splits > 1 else grp.partial_buffers()
            _decode.decode_fp4(**common, num_splits=splits, _partials=parts, _exchange=grp.exchange_args(out))
        elif splits > 1:
            _decode.decode_fp4(**common, num_splits=splits, _partials=grp.local_split_buffers(splits))
            if args.exchange == "push":
                grp.merge(out, splits)          # folds the local splits in the same launch
            else:
                grp.fold_local_splits(splits)
                grp.merge(out)
        else:
            _decode.decode_fp4(**common, _partials=grp.partial_buffers())
            grp.merge(out)

    side = torch.cuda.Stream(device)
    side.wait_stream(torch.cuda.current_stream())
    workspace_warm = 2 * num_pools
    with torch.cuda.stream(side):
        for i in range(workspace_warm):
            step(i)
    side.synchronize()
    if world > 1:
        dist.barrier()
    # The NCCL exchange is timed with plain launches: a run that captured the all-gather into
    # the graph next to the hand-launched kernels did not finish on two GPUs.
    use_graph = grp is None or args.exchange != "nccl"
    if use_graph:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            for i in range(num_pools):
                step(i)
        one_round = graph.replay
    else:
        def one_round():
            for i in range(num_pools):
                step(i)
    reps = max(1, args.steps // num_pools)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    for _ in range(max(1, args.warmup // num_pools)):
        one_round()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(reps):
        one_round()
    end.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(end)
    if world > 1:
        t = torch.tensor([ms], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
        dist.barrier()
    clocks = sampler.stop() if rank == 0 else None
    done = reps * num_pools
    ms_step = ms / done
    status = int(grp.status.item()) if grp is not None else 0
    check = page_range_check(device, world, rank, args.exchange) if world > 1 and check else None
    line = None
    if rank == 0:
        peaks = load_peaks()
        peak = float(peaks.get("hbm_gbs", 6650.0))
        per_gpu = kv_bytes / world / (ms_step * 1e-3) / 1e9
        line = ({
            "metric": METRIC, "value": rows / (ms_step * 1e-3), "unit": UNIT, "n_gpus": world,
            "steps": done, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "nvfp4", "data": "synthetic",
            "config": {
                "workload": f"long-context split-KV: {rows} seq x {ctx} ctx, Hq32/Hkv8/D128, KV pages of every "
                            "sequence partitioned by page range over the GPUs, partial (O, LSE) merged over NVLink",
                "exchange": (f"{args.exchange}, {splits} local splits per GPU" if world > 1
                             else f"one GPU, num_splits={splits}"),
                "l2": f"{num_pools} rotating page pools per GPU, {per_pool / 1e6:.0f} MB each",
                "timing": ("CUDA-graph replay" if use_graph else "plain launches")
                          + " (decode with the query quantised inside + merge(s) per step), CUDA events, max over ranks",
            },
            "hbm_gbs_per_gpu": per_gpu,
            "roofline": {"bound": "hbm", "achieved": per_gpu, "peak": peak, "unit": "GB/s",
                         "frac": per_gpu / peak, "peak_source": "measured" if peaks else "fallback",
                         "traffic": None},
            "cpu_baseline": None, "e2e": None,
            "gpu_launches": done * (1 if world > 1 and args.exchange == "fused"
                                    else 2 if world == 1 or args.exchange == "push"
                                    else (2 if splits > 1 else 1) + (2 if args.exchange == "nccl" else 1)),
            "clocks": clocks, "device_status_word": status,
            "us_per_step": ms_step * 1e3, "frac_of_peak_per_gpu": per_gpu / peak,
        })
        if check:
            line.update(check)
        if not sub:
            print(json.dumps(line), flush=True)
    del pools
    torch.cuda.empty_cache()
    if world > 1 and not sub:
        dist.destroy_process_group()
    return line


def page_range_check(device, world, rank, exchange):
    """Correctness of the cross-GPU page-range exchange on a small problem every rank can hold:
    bit identity with the one-GPU split path (same partials, same merge order) and the distance to
    the CPU oracle run split by split.  Collective: every rank calls it.  Uses the parity tests'
    problem builder and the oracle as checkers, outside every timed region."""
    for extra in (os.path.join(ROOT, "oracle"), os.path.join(ROOT, "tests"), os.path.join(ROOT, "tests", "golden")):
        if extra not in sys.path:
            sys.path.insert(0, extra)
    import torch
    import torch.distributed as dist

    import inputs
    from helpers import Problem
    from nvfp4_attn_kernel_b200 import sharding

    lens = tuple(128 * (world * 3 + i) + (33, 0, 128, 77)[i % 4] for i in range(4))
    case = inputs.attention_case(71, 4, HQ, HKV, lens, 1.0, 0.0)
    prob = Problem(case, device)   # every rank holds the whole small cache; it only READS its range
    grp = sharding.PageRangeGroup(dist.group.WORLD, 4, HQ, device, exchange=exchange, heads_kv=HKV)
    table, lseq = sharding.local_page_table(prob.page_table, prob.seqused_fp4, rank, world)
    tail = {}
    if rank == 0:
        tail = dict(residual_key_pages_bf16=prob.k_pages, residual_value_pages_bf16=prob.v_pages,
                    residual_page_ids=prob.residual_page_ids, seqused_residual=prob.seqused_residual)
    out = torch.zeros(4, HQ, D, dtype=torch.bfloat16, device=device)
    same = True
    # The exchange's launch has 4 rows x 8 KV heads CTAs per rank: the kernel's wide form.  The two
    # forms add a row's pages in a different order, so the one-GPU comparison runs on the same form.
    from nvfp4_attn_kernel_b200.nvfp4_decode_kernel import _decode
    want = _decode.decode_fp4_split(
        query_fp4=None, query_scales=None, query_bf16=prob.q, key_pages_fp4=prob.k_fp4, key_scales=prob.k_sf,
        value_pages_fp4=prob.v_fp4, value_scales=prob.v_sf, fp4_page_table=prob.page_table,
        seqused_fp4=prob.seqused_fp4, softmax_scale=prob.softmax_scale, num_splits=world,
        residual_key_pages_bf16=prob.k_pages, residual_value_pages_bf16=prob.v_pages,
        residual_page_ids=prob.residual_page_ids, seqused_residual=prob.seqused_residual, wide_form=True)
    for _ in range(3):
        sharding.decode_page_range(grp, prob.q, prob.k_fp4, prob.k_sf, prob.v_fp4, prob.v_sf, table, lseq,
                                   out=out, softmax_scale=prob.softmax_scale, **tail)
        torch.cuda.synchronize()
        same = same and bool(torch.equal(out, want))
    gap = float((out.float() - want.float()).abs().max())
    err = None
    if rank == 0:
        oracle = torch.from_numpy(prob.oracle_from_bytes(splits=world)).to(device)
        err = float((out.float() - oracle).abs().max())
    flags = [None] * world
    dist.all_gather_object(flags, (same, int(grp.status.item()), gap))
    return {"check": {"problem": f"4 rows of {lens} tokens with tails, page ranges over {world} GPUs",
                      "bitwise_equal_to_one_gpu_split": all(f[0] for f in flags),
                      "max_abs_vs_one_gpu_split": max(f[2] for f in flags),
                      "one_gpu_split_kernel_form": "wide",
                      "device_status_words": [f[1] for f in flags],
                      "max_abs_vs_oracle_rows": err, "bound": 2e-2}}


def run_ragged(args) -> None:
    """Ragged serving step on one GPU: 32 sequences with lengths log-uniform in [128, 32768], every
    one with a BF16 tail, block tables drawn from a shuffled pool of 20000 pages.  A step is what a
    layer costs while serving: the slot control plane, ONE decode launch (query quantised inside,
    the step's K/V token appended to the tail inside, key shift on) and the tail flush; sequence
    lengths advance by one token per step on the device, so tails fill and get sealed as they would
    in an engine.  All launches of a step are inside the timed region."""
    import numpy as np
    import torch

    import nvfp4_attn_kernel_b200._lib as L
    from nvfp4_attn_kernel_b200.nvfp4_decode_kernel import _decode
    from nvfp4_attn_kernel_b200.nvfp4_vllm import layout
    from nvfp4_attn_kernel_b200.nvfp4_vllm.control import ControlPlane, WorkListPlan
    from nvfp4_attn_kernel_b200.nvfp4_decode_kernel import quantize_kv_kernel as qkv

    if int(os.environ.get("WORLD_SIZE", "1")) != 1:
        raise SystemExit("the ragged workload runs on one GPU")
    torch.cuda.set_device(0)
    device = torch.device("cuda", 0)
    lib = L.load()
    rows, pool_pages = ROWS, 20000
    rng = np.random.default_rng(3)
    lens = np.exp(rng.uniform(np.log(128), np.log(32768), rows)).astype(np.int64)
    per_graph = 8
    total_steps = (max(1, args.warmup // per_graph) + max(1, args.steps // per_graph) + 2) * per_graph
    columns = int((lens.max() + total_steps) // PAGE + 2)
    need = (lens + total_steps) // PAGE + 2                   # blocks a row may touch
    ids = rng.permutation(np.arange(1, pool_pages))           # block 0 is vLLM's null block
    table = np.zeros((rows, columns), dtype=np.int32)
    at = 0
    for r in range(rows):
        table[r, :need[r]] = ids[at:at + need[r]]
        at += int(need[r])
    # page data: quantised once into a dense pool, then placed at the rows' block ids
    full = (lens - 1) // PAGE
    used = int(full.sum())
    dense = build_pools(device, 1, -(-used // 128) * 128, 1)[0]
    block = layout.page_bytes(HKV)
    cache = torch.zeros(pool_pages, block, dtype=torch.uint8, device=device)
    live_ids = np.concatenate([table[r, :full[r]] for r in range(rows)]).astype(np.int64)
    cache[torch.from_numpy(live_ids).to(device)] = dense["cache"][:used]
    del dense
    k_fp4, k_sf, v_fp4, v_sf = layout.carve(cache, HKV, D)
    gen = torch.Generator(device=device)
    gen.manual_seed(4)
    tail_k = torch.randn(1, rows, PAGE, HKV, D, device=device, generator=gen).to(torch.bfloat16)
    tail_v = torch.randn(1, rows, PAGE, HKV, D, device=device, generator=gen).to(torch.bfloat16)
    q = torch.randn(rows, HQ, D, device=device, generator=gen).to(torch.bfloat16)
    k_new = (torch.randn(rows, HKV, D, device=device, generator=gen) + 1.0).to(torch.bfloat16)
    v_new = torch.randn(rows, HKV, D, device=device, generator=gen).to(torch.bfloat16)
    shift = torch.ones(HKV, D, device=device).to(torch.bfloat16)
    out = torch.zeros(rows, HQ, D, dtype=torch.bfloat16, device=device)
    block_table = torch.from_numpy(table).to(device)
    seq_lens = torch.from_numpy(lens.astype(np.int32)).to(device)
    starts = torch.arange(rows + 1, dtype=torch.int32, device=device)
    # the slot table as the prompts' prefill steps would have left it
    plane = ControlPlane(max_num_seqs=rows, max_num_batched_tokens=rows, device=device)
    plane.slot_keys.copy_(block_table[:, 0])
    plane.slot_last_seq.copy_(seq_lens)
    plane.slot_last_seen.zero_()
    bases = torch.tensor([[t.data_ptr()] for t in (k_fp4, k_sf, v_fp4, v_sf)], dtype=torch.int64, device=device)

    # One CTA walks a (row, KV head) serially, so the longest row sets the step time unless it is
    # split; every split of every row is a CTA with a fixed cost of its own, so not too finely:
    # as many splits as bring the longest piece to about 64 pages (measured here: 1 split 178 us,
    # 4 splits 112 us, 8 splits 131 us, 16 splits 163 us per step).  The lengths are host data in
    # a serving engine too (the scheduler's seq_lens).
    # --balance-pages T cuts every row by its own length instead (pieces of about T pages).
    splits = args.num_splits
    balance = args.balance_pages if args.balance_pages > 0 else None
    if args.balance_pages < 0:   # from what a scheduler knows on the host: the lengths
        sms = torch.cuda.get_device_properties(device).multi_processor_count
        balance = _decode.balance_pages_heuristic(int(full.sum()), HKV, sms=sms)
    if args.wide:
        balance = _decode.wide_piece_pages((lens + total_steps) // PAGE, HKV, tail_pieces=rows,
                                           sms=torch.cuda.get_device_properties(device).multi_processor_count)
    if balance:
        splits = 1
        space = torch.empty(_decode.balanced_workspace_bytes(rows, HQ, columns, balance),
                            dtype=torch.uint8, device=device)
    elif splits <= 1:
        splits = 1
        while int(lens.max() + total_steps) // PAGE > 64 * splits:
            splits *= 2
    how = dict(balance_pages=balance, workspace=space) if balance else dict(num_splits=splits)
    if args.wide:
        how["wide_form"] = True
    if args.persistent:
        balance, splits = None, 1
        how = dict(persistent_workspace=_decode.persistent_workspace(rows, HQ, HKV, device))

    # with the balanced split the control step lists the pieces in its own launch
    plan = WorkListPlan(rows, columns, balance, HQ, space) if balance else None
    if plan:
        how["reuse_work_list"] = True
        if args.merge_in_launch:
            how["merge_in_launch"] = True

    def step():
        seq_lens.add_(1)
        ctl = plane.prepare(block_table=block_table, seq_lens=seq_lens, query_start_loc=starts,
                            num_reqs=rows, num_actual_tokens=rows, work_list=plan)
        _decode.decode_fp4(
            query_fp4=None, query_scales=None, query_padded_bf16=None, query_bf16=q,
            key_pages_fp4=k_fp4, key_scales=k_sf, value_pages_fp4=v_fp4, value_scales=v_sf,
            fp4_page_table=block_table, seqused_fp4=ctl.seqused_fp4,
            residual_key_pages_bf16=tail_k[0], residual_value_pages_bf16=tail_v[0],
            residual_page_ids=ctl.row_to_slot, seqused_residual=ctl.seqused_residual,
            softmax_scale=D ** -0.5, trusted_metadata=True, out=out,
            append_key=k_new, append_value=v_new, key_shift=shift, **how)
        L.check(lib.nvfp4_tail_flush(
            tail_k.data_ptr(), tail_v.data_ptr(), rows * PAGE, ctl.promotion_source_tokens.data_ptr(),
            ctl.promotion_pages.data_ptr(), bases.data_ptr(), block, block, block, block, rows, 1, HKV,
            torch.cuda.current_stream(device).cuda_stream))

    side = torch.cuda.Stream(device)
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        step()
    side.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        for _ in range(per_graph):
            step()
    done_before = 1 + per_graph          # the capture itself does not run the kernels
    seq_lens.copy_(torch.from_numpy((lens + 1).astype(np.int32)).to(device))
    done_before = 1
    sampler = ClockSampler(0)
    sampler.start()
    warm = max(1, args.warmup // per_graph)
    for _ in range(warm):
        graph.replay()
    torch.cuda.synchronize()
    reps = max(1, args.steps // per_graph)
    state = StepState(plane, seq_lens)
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    repeat_ms = []
    for _ in range(REPEATS):       # the same steps each time: the state is put back in between
        state.restore()
        torch.cuda.synchronize()
        start.record()
        for _ in range(reps):
            graph.replay()
        end.record()
        torch.cuda.synchronize()
        repeat_ms.append(start.elapsed_time(end) / (reps * per_graph))
    clocks = sampler.stop()
    ms_step = _median(repeat_ms)
    errors = int(plane.error_code.item())
    # algorithmic bytes of the timed steps, from the lengths each of them saw
    first = done_before + warm * per_graph
    kv = 0.0
    for s_ in range(first, first + reps * per_graph):
        cur = lens + s_ + 1
        fp4 = ((cur - 1) // PAGE) * PAGE
        kv += HKV * float((fp4 * 144 + (cur - fp4) * 512).sum())
    kv /= reps * per_graph
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except (OSError, ValueError):
        pass
    peak = float(peaks.get("hbm_gbs", 6650.0))
    achieved = kv / (ms_step * 1e-3) / 1e9
    print(json.dumps({
        "metric": METRIC, "value": rows / (ms_step * 1e-3), "unit": UNIT, "n_gpus": 1,
        "steps": reps * per_graph, "warmup": warm * per_graph, "ms_per_step": ms_step,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "nvfp4",
        "data": "synthetic",
        "config": {
            "workload": "ragged serving step: 32 seq, lengths log-uniform in [128, 32768] growing one token "
                        "per step, BF16 tails, block tables from a shuffled pool of 20000 pages, key shift on",
            "step": "slot control plane (which also lists the decode pieces) + one decode launch (query "
                    "quantised and K/V token appended "
                    "inside, " + ("one persistent launch of two CTAs per SM" if args.persistent else
                                  f"pieces of {balance} pages per row and one piece per tail + merge launch"
                                  if balance else
                                  f"{splits} KV splits" + (" + merge launch" if splits > 1 else ""))
                    + ") + tail flush, all timed",
            "l2": f"{kv / 1e6:.0f} MB of pages and tails per step against a 126 MB L2 (one cache, so a "
                  "part of it may be served from L2)",
            "timing": f"CUDA-graph replay of {per_graph} steps, CUDA events",
        },
        "hbm_gbs": achieved, "kv_bytes_per_step": kv,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": achieved / peak, "peak_source": "measured" if peaks else "fallback",
                     "traffic": None},
        "cpu_baseline": None, "e2e": None, "gpu_launches": REPEATS * reps * per_graph * (3 if splits <= 1 and not balance else 4),
        "repeats": {"count": REPEATS, "ms_per_step": repeat_ms, "median": ms_step, "min": min(repeat_ms), "max": max(repeat_ms)},
        "clocks": clocks, "control_plane_error_word": errors,
    }), flush=True)


def run_model_step(args, sub: bool = False):
    """``sub``: called by the headline run on an initialised process group; returns the record
    (rank 0) instead of printing a line.

    One GPU's share of a full-model decode step under tensor parallelism by KV head: 32 layers,
    batch 32, contexts uniform in [1024, 16384] growing one token per step, 1 KV head and 4 query
    heads on this GPU (8 KV heads over 8 GPUs; the ranks share nothing, so every rank of a
    multi-GPU launch runs the same shape on its own heads).  A step = the slot control plane once,
    then per layer ONE decode call (query quantised and the step's K/V token appended inside, key
    shift on, rows cut into pieces by the step's shape: work list in the first layer, reused by
    the others), then one tail flush over all layers.  Every layer has its own block array (same
    block ids, as in vLLM) and its own tails."""
    import numpy as np
    import torch

    import nvfp4_attn_kernel_b200._lib as L
    from nvfp4_attn_kernel_b200.nvfp4_decode_kernel import _decode
    from nvfp4_attn_kernel_b200.nvfp4_vllm import layout
    from nvfp4_attn_kernel_b200.nvfp4_vllm.control import ControlPlane, WorkListPlan
    from nvfp4_attn_kernel_b200.nvfp4_vllm.runtime import piece_pages

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    import torch.distributed as dist
    if world > 1 and not sub:
        dist.init_process_group("nccl", device_id=device)
    lib = L.load()
    layers, rows, hkv, hq = 32, ROWS, 1, 4
    rng = np.random.default_rng(5)
    lens = rng.integers(1024, 16385, rows).astype(np.int64)
    total_steps = args.warmup + args.steps + 3
    columns = int((lens.max() + total_steps) // PAGE + 2)
    need = (lens + total_steps) // PAGE + 2
    pool_pages = int(need.sum()) + 1                          # block 0 is vLLM's null block
    ids = rng.permutation(np.arange(1, pool_pages))
    table = np.zeros((rows, columns), dtype=np.int32)
    at = 0
    for r in range(rows):
        table[r, :need[r]] = ids[at:at + need[r]]
        at += int(need[r])
    dense = build_pools(device, 1, 2048, 1, hkv=hkv)[0]["cache"]
    block = layout.page_bytes(hkv)
    index = torch.arange(pool_pages, device=device)
    caches = [dense[(index + 97 * layer) % dense.shape[0]].contiguous() for layer in range(layers)]
    del dense
    views = [layout.carve(cache, hkv, D) for cache in caches]
    gen = torch.Generator(device=device)
    gen.manual_seed(6)
    tail_k = torch.randn(layers, rows, PAGE, hkv, D, device=device, generator=gen).to(torch.bfloat16)
    tail_v = torch.randn(layers, rows, PAGE, hkv, D, device=device, generator=gen).to(torch.bfloat16)
    q = torch.randn(layers, rows, hq, D, device=device, generator=gen).to(torch.bfloat16)
    k_new = (torch.randn(layers, rows, hkv, D, device=device, generator=gen) + 1.0).to(torch.bfloat16)
    v_new = torch.randn(layers, rows, hkv, D, device=device, generator=gen).to(torch.bfloat16)
    shift = torch.ones(hkv, D, device=device).to(torch.bfloat16)
    out = torch.zeros(layers, rows, hq, D, dtype=torch.bfloat16, device=device)
    block_table = torch.from_numpy(table).to(device)
    seq_lens = torch.from_numpy(lens.astype(np.int32)).to(device)
    starts = torch.arange(rows + 1, dtype=torch.int32, device=device)
    plane = ControlPlane(max_num_seqs=rows, max_num_batched_tokens=rows, device=device)
    plane.slot_keys.copy_(block_table[:, 0])
    plane.slot_last_seq.copy_(seq_lens)
    plane.slot_last_seen.zero_()
    bases = torch.tensor([[v[i].data_ptr() for v in views] for i in range(4)], dtype=torch.int64,
                         device=device)
    sms = torch.cuda.get_device_properties(device).multi_processor_count
    piece = piece_pages(rows, hkv, columns, sms) if args.balance_pages < 0 else max(0, args.balance_pages)
    if args.wide:
        piece = _decode.wide_piece_pages((lens + total_steps) // PAGE, hkv, sms=sms, tail_pieces=rows)
    if piece >= columns:
        piece = 0
    # what a scheduler knows on the host, the lengths, says whether the step makes at most one CTA
    # per SM: then the decode runs on the kernel's wide form
    wide_form = args.wide or (piece > 0 and not args.persistent and _decode.wide_form_fits(
        (lens + total_steps) // PAGE, hkv, piece, sms=sms, tail_pieces=rows))
    pws = _decode.persistent_workspace(rows, hq, hkv, device) if args.persistent else None
    space = torch.empty(_decode.balanced_workspace_bytes(rows, hq, columns, piece) if piece else 16,
                        dtype=torch.uint8, device=device)

    # with the balanced split the control step lists the pieces in its own launch
    plan = WorkListPlan(rows, columns, piece, hq, space) if piece and not args.persistent else None

    def step():
        seq_lens.add_(1)
        ctl = plane.prepare(block_table=block_table, seq_lens=seq_lens, query_start_loc=starts,
                            num_reqs=rows, num_actual_tokens=rows, work_list=plan)
        for layer in range(layers):
            k_fp4, k_sf, v_fp4, v_sf = views[layer]
            how = dict(balance_pages=piece, workspace=space, reuse_work_list=True,
                       merge_in_launch=args.merge_in_launch) if piece else {}
            if wide_form:
                how["wide_form"] = True
            if args.persistent:
                how = dict(persistent_workspace=pws)
            _decode.decode_fp4(
                query_fp4=None, query_scales=None, query_padded_bf16=None, query_bf16=q[layer],
                key_pages_fp4=k_fp4, key_scales=k_sf, value_pages_fp4=v_fp4, value_scales=v_sf,
                fp4_page_table=block_table, seqused_fp4=ctl.seqused_fp4,
                residual_key_pages_bf16=tail_k[layer], residual_value_pages_bf16=tail_v[layer],
                residual_page_ids=ctl.row_to_slot, seqused_residual=ctl.seqused_residual,
                softmax_scale=D ** -0.5, trusted_metadata=True, out=out[layer],
                append_key=k_new[layer], append_value=v_new[layer], key_shift=shift, **how)
        L.check(lib.nvfp4_tail_flush(
            tail_k.data_ptr(), tail_v.data_ptr(), rows * PAGE, ctl.promotion_source_tokens.data_ptr(),
            ctl.promotion_pages.data_ptr(), bases.data_ptr(), block, block, block, block, rows, layers, hkv,
            torch.cuda.current_stream(device).cuda_stream))

    side = torch.cuda.Stream(device)
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        step()
    side.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        step()
    seq_lens.copy_(torch.from_numpy((lens + 1).astype(np.int32)).to(device))
    sampler = ClockSampler(local) if rank == 0 else None
    if sampler:
        sampler.start()
    for _ in range(max(3, args.warmup)):
        graph.replay()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    state = StepState(plane, seq_lens)
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    repeat_ms = []
    for _ in range(REPEATS):       # the same steps each time: the state is put back in between
        state.restore()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        start.record()
        for _ in range(args.steps):
            graph.replay()
        end.record()
        torch.cuda.synchronize()
        ms = start.elapsed_time(end)
        if world > 1:
            t = torch.tensor([ms], dtype=torch.float64, device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        repeat_ms.append(ms / args.steps)
    if world > 1:
        dist.barrier()
    clocks = sampler.stop() if sampler else None
    ms_step = _median(repeat_ms)
    errors = int(plane.error_code.item())
    # algorithmic bytes of the timed steps on this GPU, from the lengths each of them saw
    first = 1 + max(3, args.warmup)
    kv = 0.0
    for s_ in range(first, first + args.steps):
        cur = lens + s_ + 1
        fp4 = ((cur - 1) // PAGE) * PAGE
        kv += layers * hkv * float((fp4 * 144 + (cur - fp4) * 512).sum())
    kv /= args.steps
    peaks = load_peaks()
    peak = float(peaks.get("hbm_gbs", 6650.0))
    achieved = kv / (ms_step * 1e-3) / 1e9
    line = None
    if rank == 0:
        launches = layers * (2 if piece else 1) + 2   # control (lists the pieces too), decode (+ merge) per layer, flush
        line = ({
            "metric": METRIC, "value": rows / (ms_step * 1e-3), "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "nvfp4",
            "data": "synthetic",
            "config": {
                "workload": "full-model decode step, Llama-3.1-8B attention shapes: 32 layers, 32 seq, contexts "
                            "uniform in [1024, 16384] growing one token per step, BF16 tails, key shift on; tensor "
                            "parallel by KV head over 8 GPUs: 1 KV head and 4 query heads per GPU",
                "step": "slot control plane once + per layer one decode call (query quantised and K/V token "
                        "appended inside" + (f", rows cut into pieces of {piece} pages and one piece per tail: the list is "
                                              "built by the control step's launch and reused by every layer, "
                                              "+ merge launch" if piece else "")
                        + ") + one tail flush over all layers, all timed",
                "kernel_form": ("wide (the host-side lengths give at most one CTA per SM)" if wide_form
                                else "narrow (two CTAs per SM)"),
                "ranks": "every rank runs this shape on its own heads (no data-path collective); value is the "
                         "batch's tokens per second of attention time, ms_per_step the max over ranks",
                "l2": f"{kv / 1e6:.0f} MB of pages and tails per step and GPU against a 126 MB L2",
                "timing": "CUDA-graph replay of one step, CUDA events, max over ranks",
            },
            "attention_us_per_layer": ms_step * 1e3 / layers,
            "hbm_gbs_per_gpu": achieved, "kv_bytes_per_step_per_gpu": kv,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "peak_source": "measured" if peaks else "fallback",
                         "traffic": None},
            "cpu_baseline": None, "e2e": None, "gpu_launches": REPEATS * args.steps * launches,
            "repeats": {"count": REPEATS, "ms_per_step": repeat_ms, "median": ms_step, "min": min(repeat_ms), "max": max(repeat_ms)},
            "clocks": clocks, "control_plane_error_word": errors,
        })
        if not sub:
            print(json.dumps(line), flush=True)
    del caches, views, tail_k, tail_v
    torch.cuda.empty_cache()
    if world > 1 and not sub:
        dist.destroy_process_group()
    return line


# The reference project's published decode timings (its own kernel on an SM100 part it reports as
# a renamed B200; CUDA-graph replay, pre-quantised K/V/Q, page-aligned, no tail):
# docs/reports/data/llama31-8b-gqa-seqlen-sweep.json and docs/reports/1.decode-baseline-comparison.md:14-19.
PUBLISHED_SHAPES = [
    # (batch, context, Hkv, reference us, reference TB/s)
    (16, 4096, 8, 19.2, 3.93),
    (32, 4096, 8, None, None),
    (64, 4096, 8, 65.0, 4.65),
    (4, 32768, 8, 42.5, 3.55),
    (16, 32768, 8, 112.8, 5.35),
    (16, 131072, 8, 430.0, 5.62),
]
PUBLISHED_GROUP_PEAKS = {1: 6.58, 4: 5.55, 8: 4.36, 16: 2.83, 32: 1.52}   # TB/s, best shape per group size


def run_published(args) -> None:
    """The shapes the reference publishes numbers for, measured with its protocol: pre-quantised
    query, page-aligned contexts without a tail, CUDA-graph replay over rotating page pools, median
    of five repeats; and the sweep over query heads per KV head at 32 query heads.  For every shape
    the launch forms this library offers are timed and the best is reported with its name."""
    import torch

    import nvfp4_attn_kernel_b200._lib as L
    from nvfp4_attn_kernel_b200.nvfp4_decode_kernel import _decode
    from nvfp4_attn_kernel_b200.nvfp4_vllm.runtime import piece_pages

    if int(os.environ.get("WORLD_SIZE", "1")) != 1:
        raise SystemExit("the published-shape workload runs on one GPU")
    torch.cuda.set_device(0)
    device = torch.device("cuda", 0)
    lib = L.load()
    sms = torch.cuda.get_device_properties(device).multi_processor_count
    sampler = ClockSampler(0)
    sampler.start()

    def measure(batch, ctx, hkv):
        pages = ctx // PAGE
        pool_bytes = batch * ctx * hkv * 144
        num_pools = max(2, -(-2 * 132 * 2 ** 20 // pool_bytes))   # what lies between two uses of a pool exceeds L2
        pools = build_pools(device, batch, pages, num_pools, hkv=hkv)
        gen = torch.Generator(device=device)
        gen.manual_seed(11)
        q = torch.randn(batch, HQ, D, device=device, generator=gen).to(torch.bfloat16)
        q_fp4 = torch.zeros(batch, 1, HQ, 64, dtype=torch.uint8, device=device)
        q_sf = torch.zeros(batch, HQ * 1024, dtype=torch.uint8, device=device)
        L.check(lib.nvfp4_quantize_q(q.data_ptr(), q.stride(0), q.stride(1), None, q_fp4.data_ptr(),
                                     q_sf.data_ptr(), None, batch, HQ, hkv,
                                     torch.cuda.current_stream().cuda_stream))
        out = torch.zeros(batch, HQ, D, dtype=torch.bfloat16, device=device)
        seq = torch.full((batch,), ctx, dtype=torch.int32, device=device)
        status = torch.zeros(1, dtype=torch.int32, device=device)
        piece = piece_pages(batch, hkv, pages, sms)
        forms = {"whole rows": {}}
        if 0 < piece < pages:
            need = int(lib.nvfp4_decode_balanced_workspace_bytes(batch, HQ, pages, piece))
            forms[f"pieces of {piece} pages + merge launch"] = dict(
                target=piece, ws=torch.empty(need, dtype=torch.uint8, device=device))
        if lib.nvfp4_decode_persistent_supported(batch, HQ, hkv):
            need = int(lib.nvfp4_decode_persistent_workspace_bytes(batch, HQ, hkv))
            forms["one persistent launch"] = dict(persistent=True, ws=torch.zeros(need, dtype=torch.uint8, device=device))

        def args_for(pool, form):
            a = L.DecodeArgs()
            a.q_fp4, a.q_sf = q_fp4.data_ptr(), q_sf.data_ptr()
            a.k_packed, a.k_pitch = pool["k"].data_ptr(), pool["block"]
            a.k_sf, a.k_sf_pitch = pool["ksf"].data_ptr(), pool["block"]
            a.v_packed, a.v_pitch = pool["v"].data_ptr(), pool["block"]
            a.v_sf, a.v_sf_pitch = pool["vsf"].data_ptr(), pool["block"]
            a.num_pages = batch * pages
            a.page_table, a.page_table_row_stride, a.max_pages = pool["table"].data_ptr(), pages, pages
            a.seqused_fp4 = seq.data_ptr()
            a.out = out.data_ptr()
            a.rows, a.heads_q, a.heads_kv = batch, HQ, hkv
            a.softmax_scale = D ** -0.5
            a.num_splits, a.impl = 1, L.IMPL_AUTO
            a.status = status.data_ptr()
            if "ws" in form:
                a.workspace, a.workspace_bytes = form["ws"].data_ptr(), form["ws"].numel()
            if form.get("persistent"):
                a.flags = L.DECODE_PERSISTENT
            return a

        results = {}
        for name, form in forms.items():
            sets = [args_for(p, form) for p in pools]

            def launch(a, stream, form=form):
                if "target" in form:
                    L.check(lib.nvfp4_decode_balanced(ctypes.byref(a), form["target"], stream))
                else:
                    L.check(lib.nvfp4_decode(ctypes.byref(a), stream))

            side = torch.cuda.Stream(device)
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for a in sets:
                    launch(a, side.cuda_stream)
            side.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                for a in sets:
                    launch(a, torch.cuda.current_stream().cuda_stream)
            for _ in range(5):
                graph.replay()
            torch.cuda.synchronize()
            one = None
            times = []
            for _ in range(5):
                reps = 5 if one is None else max(5, int(10.0 / (one * len(sets))))   # ~10 ms per repeat
                start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                start.record()
                for _ in range(reps):
                    graph.replay()
                end.record()
                torch.cuda.synchronize()
                one = start.elapsed_time(end) / (reps * len(sets))
                times.append(one)
            results[name] = _median(times[1:]) * 1e3
        best = min(results, key=results.get)
        us = results[best]
        del pools
        torch.cuda.empty_cache()
        return {"us": us, "tb_per_s": pool_bytes / (us * 1e-6) / 1e12, "form": best,
                "all_forms_us": results, "pools": num_pools, "device_status_word": int(status.item())}

    rows = []
    for batch, ctx, hkv, ref_us, ref_tbs in PUBLISHED_SHAPES:
        r = measure(batch, ctx, hkv)
        r.update({"shape": f"b{batch} x s{ctx}, Hq32/Hkv{hkv}", "reference_us": ref_us, "reference_tb_per_s": ref_tbs,
                  "speedup_vs_reference": (ref_us / r["us"]) if ref_us else None})
        rows.append(r)
    sweep = []
    for group, ref_peak in PUBLISHED_GROUP_PEAKS.items():
        r = measure(32, 16384, HQ // group)
        r.update({"shape": f"b32 x s16384, Hq32/Hkv{HQ // group} (G = {group})",
                  "reference_peak_tb_per_s_best_shape": ref_peak})
        sweep.append(r)
    clocks = sampler.stop()
    # can the reference's own kernel be imported on this machine?  (its sources travel only as a
    # git-ignored copy for checker use; without them there is nothing to try)
    ref_src = os.path.join(ROOT, "oracle", "_ref", "src")
    if os.path.isdir(os.path.join(ref_src, "nvfp4_decode_kernel")):
        proc = subprocess.run(
            [sys.executable, "-c", "import sys; sys.path.insert(0, sys.argv[1]); import nvfp4_decode_kernel._decode",
             ref_src], capture_output=True, text=True, timeout=300)
        attempt = "imports" if proc.returncode == 0 else (proc.stderr.strip().splitlines() or ["failed"])[-1][:300]
    else:
        attempt = "the reference's sources are not on this machine"
    peaks = load_peaks()
    head = next(r for r in rows if r["shape"].startswith("b32 x s4096"))
    print(json.dumps({
        "metric": "decode_us_at_published_shapes", "value": head["us"], "unit": "us", "n_gpus": 1,
        "steps": 0, "warmup": 0, "ms_per_step": head["us"] * 1e-3, "higher_is_better": False,
        "scaling": "weak", "vs_baseline": None, "dtype": "nvfp4", "data": "synthetic",
        "config": {"workload": "the reference's published decode shapes with its protocol: pre-quantised query, "
                               "no tail, CUDA-graph replay over rotating pools, median of 4 repeats after one "
                               "discarded; value = b32 x s4096",
                   "reference_hardware": "an SM100 GPU with 148 SMs that nvidia-smi calls L20A, taken by the "
                                         "reference's authors for a renamed B200"},
        "published_shapes": rows, "group_sweep": sweep,
        "reference_kernel_on_this_machine": attempt,
        "hbm_peak_gbs_measured": peaks.get("hbm_gbs"),
        "cpu_baseline": None, "e2e": None, "gpu_launches": None, "clocks": clocks,
    }), flush=True)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--warmup", type=int, default=30)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--decode-impl", default="auto", choices=["auto", "generic", "sm100"])
    ap.add_argument("--num-splits", type=int, default=1)
    ap.add_argument("--balance-pages", type=int, default=-1,
                    help="ragged workload: pieces of about this many pages per row (0: one split "
                         "count for the batch; -1, the default: chosen from the lengths)")
    ap.add_argument("--wide", action="store_true",
                    help="ragged / model-step workloads: cut the rows, from their host-side lengths, into at "
                         "most one piece per SM and run the decode on the kernel's wide form")
    ap.add_argument("--merge-in-launch", action="store_true",
                    help="ragged / model-step workloads with the balanced split: the piece of a row that finishes "
                         "last merges the row's pieces inside the decode launch (no merge launch)")
    ap.add_argument("--persistent", action="store_true",
                    help="ragged / model-step workloads: run the decode as one persistent launch "
                         "(NVFP4_DECODE_PERSISTENT) instead of work list + pieces + merge")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-multi-gpu-records", action="store_true",
                    help="with more than one GPU: skip the long-context exchange and the tensor-parallel "
                         "model step that are measured after the headline")
    ap.add_argument("--ctx", type=int, default=CTX,
                    help="context length per sequence (default: the headline workload's 4096)")
    ap.add_argument("--workload", default="batch",
                    choices=["batch", "long-context", "ragged", "model-step", "published"],
                    help="batch: the headline uniform batch (default); long-context: 4 x 32768 split "
                         "by page range over the GPUs; ragged: 32 ragged sequences with tails, the "
                         "whole serving step (control plane, decode with fused append, flush); "
                         "model-step: 32 layers of one GPU's head shard (1 KV head, 4 query heads), "
                         "contexts uniform in [1024, 16384]")
    ap.add_argument("--exchange", default="fused", choices=["fused", "push", "peer", "nccl"])
    ap.add_argument("--lc-rows", type=int, default=4, help="sequences of the long-context workload")
    ap.add_argument("--lc-ctx", type=int, default=32768, help="context of the long-context workload")
    ap.add_argument("--pdl", action=argparse.BooleanOptionalAction, default=True,
                    help="launch the decode with programmatic stream serialization: a launch's set-up "
                         "and first page loads overlap the previous launch's drain")
    ap.add_argument("--ncu-traffic", type=float, default=None,
                    help="dram bytes per decode launch from an ncu capture (reported as roofline.traffic)")
    args = ap.parse_args()
    if args.ctx != CTX:
        set_context(args.ctx)
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "long-context":
        run_long_context(args)
    elif args.workload == "ragged":
        run_ragged(args)
    elif args.workload == "model-step":
        run_model_step(args)
    elif args.workload == "published":
        run_published(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
