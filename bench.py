"""Headline benchmark: decode tok/s of a Llama-3.2-1B-shaped fp32 model given as an exported (un-fused) op graph.

Workload (the full-model decode configuration of the benchmark plan): 16 layers, hidden 2048, 32 q / 8 kv heads,
head_dim 64, FFN 8192, vocab 128256, random-init weights; 64 independent requests per GPU decoded as one batch, 512-token uniform-random prompts,
then greedy-style decode steps of one token per request (context 512 + step).  A "step" is one decode
step over the 64 requests = one pass of the op graph through the host runtime and kernels of
librmlk_b200.so.  Requests are sharded across GPUs with no collective (one process per GPU, weights
replicated), so per-GPU work is fixed and scaling is "weak".

    python bench.py --gpus 1 --steps 32 --warmup 3
    python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference ...      # the CPU path (numpy oracle interpreter) on the host cores

Prints ONE JSON line (rank 0).  `value` is device-resident (inputs already in HBM); `e2e` feeds host
buffers and reads the logits back every step.  `roofline` is measured live (CUDA-graph replay between
events on the launching stream) for the kernel with the largest share of the step, the weight-streaming
tcgen05 MatMul, with the other heavy kernels of the step beside it; `cpu_baseline` times the CPU oracle on a bounded sample of the same step.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

REQUESTS_PER_GPU = 64
PROMPT = 512
METRIC = "decode_tokens_per_s"
UNIT = "tok/s"


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def workload_config(cfg, batch, prompt):
    return {
        "workload": f"llama-3.2-1b-shaped fp32 decode as un-fused ONNX ops; {batch} requests per GPU decoded as one batch, "
                    f"{prompt}-token uniform-random prompts, one token per request per step",
        "layers": cfg.n_layers, "hidden": cfg.hidden, "heads": cfg.n_heads, "kv_heads": cfg.n_kv_heads, "head_dim": cfg.head_dim,
        "ffn": cfg.ffn, "vocab": cfg.vocab, "requests_per_gpu": batch, "prompt_tokens": prompt,
        "l2": "weights (4.9 GB) and KV cache exceed L2 (126 MB): every step streams them from HBM, no flush needed",
        "sharding": "independent requests per GPU, weights replicated, no collective",
    }


# ---------------------------------------------------------------------------------------------------
# clocks
# ---------------------------------------------------------------------------------------------------
class ClockSampler:
    """nvidia-smi polled every 20 ms in the background; stop(windows) keeps the samples whose timestamp falls inside
    one of the (start, end) wall-clock windows, i.e. the samples taken under load during the timed regions."""
    FIELDS = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.path = os.path.join("/tmp", f"rmlk_clocks_{os.getpid()}.csv")

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "20",
                                          "-i", str(self.gpu)], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self, windows=None):
        import datetime
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if not self.proc:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons, total = [], [], set(), 0
        try:
            for line in open(self.path):
                f = [x.strip() for x in line.split(",")]
                if len(f) < 9:
                    continue
                try:
                    ts = datetime.datetime.strptime(f[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                    clk, cmax = float(f[1]), float(f[2])
                except ValueError:
                    continue
                total += 1
                if windows and not any(w0 <= ts <= w1 for w0, w1 in windows):
                    continue
                sm.append(clk)
                mx.append(cmax)
                for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
            os.remove(self.path)
        except Exception:
            pass
        if sm:
            out["sm_mhz"] = statistics.median(sm)
            out["sm_max_mhz"] = max(mx)
            out["samples"] = len(sm)
        out["samples_total"] = total
        out["reasons"] = sorted(reasons)
        return out


# ---------------------------------------------------------------------------------------------------
# CPU path (oracle): bounded sample of the same decode step
# ---------------------------------------------------------------------------------------------------
def cpu_decode_sample(cfg, batch, context, steps, seed=0):
    """Times `steps` decode steps of `batch` requests at context `context` through the numpy oracle
    interpreter with a synthetic KV cache.  Returns (tok/s, threads, description)."""
    import torch
    from oracle import graph_cpu
    from rmlk_b200 import llama
    threads = os.cpu_count() or 1
    # use every host core even when a launcher exported OMP_NUM_THREADS=1 (torchrun does)
    torch.set_num_threads(threads)
    try:
        from threadpoolctl import threadpool_limits
        threadpool_limits(limits=threads)
    except Exception:
        pass
    torch.manual_seed(seed)
    w = {}
    for name, shape in llama.weight_shapes(cfg).items():
        if name == "lm_head":
            continue
        w[name] = (torch.ones(shape) if name.endswith(("ln1", "ln2", "ln_f")) else torch.randn(shape) * 0.02).numpy()
    w["lm_head"] = np.ascontiguousarray(w["embed"].T)
    spec = llama.build_graph(cfg, w)
    rng = np.random.default_rng(seed)
    past = [(rng.standard_normal((batch, cfg.n_kv_heads, context, cfg.head_dim), dtype=np.float32),
             rng.standard_normal((batch, cfg.n_kv_heads, context, cfg.head_dim), dtype=np.float32)) for _ in range(cfg.n_layers)]
    times = []
    ctx = context
    for s in range(steps + 1):  # first step is a warm-up (BLAS thread pool, page faults)
        feeds = {"input_ids": rng.integers(0, cfg.vocab, size=(batch, 1)), "attention_mask": np.ones((batch, ctx + 1), np.int64),
                 "position_ids": np.full((batch, 1), ctx, np.int64)}
        for l in range(cfg.n_layers):
            feeds[f"past_key_values.{l}.key"], feeds[f"past_key_values.{l}.value"] = past[l]
        t0 = time.perf_counter()
        out = graph_cpu.run_graph(spec, feeds, fast=True)
        dt = time.perf_counter() - t0
        if s > 0:
            times.append(dt)
        past = [(out[f"present.{l}.key"], out[f"present.{l}.value"]) for l in range(cfg.n_layers)]
        ctx += 1
    total = sum(times)
    return batch * len(times) / total, threads, f"{batch} requests x {len(times)} decode steps at context {context}, synthetic KV cache, numpy oracle interpreter"


CPU_SAMPLE_STEPS = 2


def run_reference(args):
    """--impl reference: the reference has no CPU build of its own for this path (Rust + CUDA only), so
    the CPU arm is the numpy restatement of its op semantics (oracle/), on all host cores.  It runs the arm's own
    configuration - the same 64 requests as one batch at context 512 - for a bounded number of decode steps."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from rmlk_b200 import llama
    cfg = llama.LLAMA_1B
    batch = args.requests
    steps = max(1, min(args.steps, CPU_SAMPLE_STEPS))
    v, threads, sample = cpu_decode_sample(cfg, batch, args.prompt, steps)
    line = {
        "impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": args.gpus, "steps": steps, "warmup": 1,
        "ms_per_step": 1000.0 * batch / v, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": dict(workload_config(cfg, batch, args.prompt), requests_run=batch, steps_run=steps),
        "cpu_baseline": {"value": v, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ---------------------------------------------------------------------------------------------------
# GPU path
# ---------------------------------------------------------------------------------------------------
def time_graph(fn_of_i, n=16, replays=4):
    """Device time per launch: n launches captured into a CUDA graph on a side stream, the graph replayed
    between two events on that stream (no host launch overhead inside the timed region)."""
    import torch
    for i in range(3):
        fn_of_i(i)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        with torch.cuda.graph(g, stream=s):
            for i in range(n):
                fn_of_i(i)
        g.replay()
        s.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(s)
        for _ in range(replays):
            g.replay()
        e1.record(s)
        s.synchronize()
    return e0.elapsed_time(e1) / (n * replays)


# dram__bytes_read.sum + dram__bytes_write.sum per launch of the kernel named by DOMINANT, from one ncu capture of that
# kernel on this shape (a cross-check of the algorithmic bytes, not a live measurement: it goes stale when the kernel changes)
DOMINANT = "matmul_gate_up"
NCU_TRAFFIC_BYTES = {"matmul_gate_up": 134_809_600 + 3_740_416}
NCU_TRAFFIC_SOURCE = "ncu --set full capture of tc_gemm_kernel on [64,2048]x[2048,16384] (read 134.81 MB + write 3.74 MB per launch)"


def kernel_rooflines(batch, ctx, peak_gbs, peak_kind):
    """Live device timing of the decode step's heaviest kernels on the step's own shapes.  Every case rotates
    over a ring of operands larger than L2 (126 MB), so reads come from HBM.  Returns {name: entry}."""
    import torch
    from rmlk_b200 import kernels as K
    dev = "cuda"
    B, T = batch, ctx
    out = {}

    def ring(make, nbytes_each):
        return [make() for _ in range(max(2, min(6, (252 << 20) // max(nbytes_each, 1) + 1)))]

    def add(name, kernel, fn, algo_bytes, shape, flops=0):
        ms = time_graph(fn)
        ach = algo_bytes / (ms * 1e-3) / 1e9
        e = {"bound": "hbm", "achieved": ach, "peak": peak_gbs, "unit": "GB/s", "frac": ach / peak_gbs,
             "traffic": NCU_TRAFFIC_BYTES.get(name), "traffic_source": NCU_TRAFFIC_SOURCE if name in NCU_TRAFFIC_BYTES else None, "kernel": kernel, "shape": shape,
             "algorithmic_bytes_per_launch": algo_bytes, "us_per_launch": ms * 1e3, "peak_kind": f"of {peak_kind} copy bandwidth"}
        if flops:
            e["tflops"] = flops / (ms * 1e-3) / 1e12
        out[name] = e

    # decode attention as the step runs it: one launch per layer over the KV cache in place, B*8 problems of 4 query heads,
    # scores + additive mask + softmax + context; K and V are read once
    kc = ring(lambda: torch.randn(B, 8, T, 64, device=dev), 4 * B * 8 * T * 64)
    q = torch.randn(B, 8, 4, 64, device=dev)
    mask = torch.zeros(B, 1, 1, T, device=dev)
    cx = torch.empty(B, 8, 4, 64, device=dev)
    add("attention", "gqa_decode_flash_kernel<16>", lambda i: K.gqa_decode_attention(q, kc[i % len(kc)], kc[(i + 1) % len(kc)], 0.125, mask=mask, out=cx),
        4 * B * 8 * (2 * 64 * T + 2 * 4 * 64) + 4 * B * T, [B * 8, 4, 64, T], flops=4 * B * 32 * 64 * T)
    del kc, q, mask, cx
    # weight-streaming MatMul at the FFN gate/up shape and at the lm_head
    # gate | up projections as the runtime runs them (one MatMul on the concatenated weights), the down projection, the lm_head
    for name, (m, k, n) in (("matmul_gate_up", (B, 2048, 16384)), ("matmul_qkv", (B, 2048, 3072)), ("matmul_down", (B, 8192, 2048)),
                            ("matmul_lm_head", (B, 2048, 128256))):
        w = ring(lambda: torch.randn(k, n, device=dev) * 0.02, 4 * k * n)
        x = torch.randn(m, k, device=dev)
        y = torch.empty(m, n, device=dev)
        wsb = K.matmul_workspace_bytes(1, m, n, k)
        ws = torch.empty(max(wsb // 4, 1), device=dev) if wsb else None
        add(name, "tc_gemm_kernel (tcgen05 3xTF32)" if m > 16 else "skinny_kernel",
            lambda i: K.matmul(x, w[i % len(w)], out=y, workspace=ws), 4 * (m * k + k * n + m * n), [m, k, n], flops=2 * m * k * n)
        del w, x, y, ws
    torch.cuda.empty_cache()
    return out


def bind_to_gpu_numa_node(local):
    """Runs this process (and so its pinned host buffers, which are placed where the allocating thread runs) on the CPUs
    of the NUMA node the GPU hangs off: with several ranks per host, logits otherwise cross the socket link on their way
    to memory.  Returns the node, or None when the topology cannot be read (then nothing is changed)."""
    try:
        import torch
        bus = torch.cuda.get_device_properties(local).pci_bus_id
        dom = torch.cuda.get_device_properties(local).pci_domain_id
        dev = torch.cuda.get_device_properties(local).pci_device_id
        path = f"/sys/bus/pci/devices/{dom:04x}:{bus:02x}:{dev:02x}.0/numa_node"
        node = int(open(path).read().strip())
        if node < 0:
            return None
        cpus = set()
        for part in open(f"/sys/devices/system/node/node{node}/cpulist").read().strip().split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = cpus & os.sched_getaffinity(0)
        if not allowed:
            return None
        os.sched_setaffinity(0, allowed)
        return node
    except Exception:
        return None


def run_ours(args):
    import torch
    import torch.distributed as dist
    from rmlk_b200 import dtypes as dt
    from rmlk_b200 import llama

    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    numa_node = bind_to_gpu_numa_node(local) if world > 1 else None
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))

    cfg = llama.LLAMA_1B
    B, P = args.requests, args.prompt
    K_, W, R = args.steps, args.warmup, max(1, args.rounds)
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        weights = llama.make_weights_device(cfg, seed=0)
    stream.synchronize()
    spec = llama.build_graph(cfg, weights, device_weights=True)
    dec = llama.Decoder(cfg, spec, device=local, stream=stream.cuda_stream, arena_bytes=(2 << 30))
    inst = dec.inst
    rng = np.random.default_rng(1234 + rank)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        if world > 1:
            t = torch.tensor([ms], dtype=torch.float64, device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t.item())
        return ms

    class Workload:
        """`batch` requests with `P`-token prompts: prefill (untimed set-up), then decode steps fed from device-resident or
        pinned host inputs.  restore() brings the context back to the end of the prompt, so that every timed round covers
        the same context lengths."""

        def __init__(self, batch, n_steps):
            self.batch, self.n_steps = batch, n_steps
            self.prompt_ids = rng.integers(0, cfg.vocab, size=(batch, P))
            self.ids_host = torch.from_numpy(rng.integers(0, cfg.vocab, size=(n_steps, batch, 1))).pin_memory()
            self.ids_dev = self.ids_host.to("cuda", non_blocking=True)
            self.masks_dev = [torch.ones(batch, P + s + 1, dtype=torch.int64, device="cuda") for s in range(n_steps)]
            self.pos_dev = [torch.full((batch, 1), P + s, dtype=torch.int64, device="cuda") for s in range(n_steps)]
            self.mask_host = torch.ones(batch, P + n_steps + 1, dtype=torch.int64).pin_memory()
            self.pos_host = torch.empty(batch, 1, dtype=torch.int64).pin_memory()
            self.step_no = 0
            self.prefill_launches = 0
            self.saved = None
            torch.cuda.synchronize()

        def prefill(self):
            """The prompt through the graph (untimed set-up); the caches it leaves are kept on the host so that restore()
            can bring the context back without running the prefill again (a prefill is seconds of tensor-core work that
            would leave the GPU power-capped for the timed steps behind it)."""
            dec.reset(self.batch)
            dec.feed(self.prompt_ids)
            inst.launch()
            inst.synchronize()
            self.prefill_launches = inst.last_launches
            self.saved = [(inst.read(f"present.{l}.key"), inst.read(f"present.{l}.value")) for l in range(cfg.n_layers)]
            self.step_no = 0

        def restore(self):
            if self.saved is None:
                return self.prefill()
            for l, (k, v) in enumerate(self.saved):
                inst.set_input(f"past_key_values.{l}.key", k)
                inst.set_input(f"past_key_values.{l}.value", v)
            dec.context = P
            self.step_no = 0
            inst.synchronize()

        def device_step(self):
            s, b = self.step_no, self.batch
            t = dec.context + 1
            inst.set_input_ptr("input_ids", dt.I64, [b, 1], self.ids_dev[s].data_ptr(), True)
            inst.set_input_ptr("attention_mask", dt.I64, [b, t], self.masks_dev[s].data_ptr(), True)
            inst.set_input_ptr("position_ids", dt.I64, [b, 1], self.pos_dev[s].data_ptr(), True)
            inst.launch()
            dec.context = t
            self.step_no += 1

        def host_step(self):
            s, b = self.step_no, self.batch
            t = dec.context + 1
            self.pos_host.fill_(dec.context)
            mask_view = self.mask_host.view(-1)[: b * t].view(b, t)   # contiguous [b, t] of ones in pinned memory
            inst.set_input_ptr("input_ids", dt.I64, [b, 1], self.ids_host[s].data_ptr(), False)
            inst.set_input_ptr("attention_mask", dt.I64, [b, t], mask_view.data_ptr(), False)
            inst.set_input_ptr("position_ids", dt.I64, [b, 1], self.pos_host.data_ptr(), False)
            inst.launch()
            inst.wait_outputs()   # the logits were registered with stream_output: they arrive block by block behind the lm_head MatMul
            dec.context = t
            self.step_no += 1
            return b * 8 + b * t * 8 + b * 8

        def timed_rounds(self, step_fn, rounds, windows, after_restore=None, before_restore=None):
            """`rounds` times: restore the context, W warm-up steps, then EXACTLY K steps between two events on the launching
            stream, with a barrier + device synchronise on both sides; per round the maximum over ranks.  Returns the
            per-round milliseconds, per-round host enqueue milliseconds and the kernel launches of one round."""
            ms, host_ms, launches = [], [], 0
            for _ in range(rounds):
                if before_restore:
                    before_restore()
                self.restore()
                if after_restore:
                    after_restore()
                for _ in range(W):
                    step_fn()
                barrier()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                launches = 0
                win0 = time.time()
                e0.record(stream)
                h0 = time.perf_counter()
                for _ in range(K_):
                    step_fn()
                    launches += inst.last_launches
                h1 = time.perf_counter()
                e1.record(stream)
                barrier()
                wall = (time.perf_counter() - h0) * 1000.0
                windows.append((win0, time.time()))
                # a step that waits for its outputs on the host (end to end) is bounded by the wall clock as well
                dev = e0.elapsed_time(e1)
                ms.append(max_over_ranks(max(dev, wall) if step_fn == self.host_step else dev))
                host_ms.append((h1 - h0) * 1000.0)
            return ms, host_ms, launches

    wl = Workload(B, W + K_ + 6)
    with torch.cuda.stream(stream):
        sampler = ClockSampler(local)
        if rank == 0:
            sampler.start()
        windows = []

        # ---- device-resident timing ---------------------------------------------------------------
        dev_rounds, host_rounds, launches = wl.timed_rounds(wl.device_step, R, windows)
        decode_launches = inst.last_launches
        prefill_launches = wl.prefill_launches
        # host cost of enqueuing one step, measured from an empty stream (inside the rounds above the host runs ahead of the
        # GPU until the launch queue is full and then waits for it, so the loop's wall time only shows the device time)
        host_one = []
        for _ in range(5):
            inst.synchronize()
            h0 = time.perf_counter()
            wl.device_step()
            host_one.append((time.perf_counter() - h0) * 1000.0)
        inst.synchronize()

        # ---- end to end: host buffers in, logits out, every step --------------------------------
        logits_host = torch.empty(B, 1, cfg.vocab, dtype=torch.float32).pin_memory()
        h2d = B * 8 + B * (P + W + K_) * 8 + B * 8   # ids + attention mask at the longest context + positions
        # the logits of a decode step stream to pinned host memory; the registration is lifted around the prefill of restore(),
        # whose logits have another shape and are not read
        e2e_rounds, _, _ = wl.timed_rounds(wl.host_step, max(1, (R + 1) // 2), windows,
                                           after_restore=lambda: inst.stream_output("logits", logits_host.data_ptr(), logits_host.numel() * 4),
                                           before_restore=lambda: inst.stream_output("logits", 0, 0))
        inst.stream_output("logits", 0, 0)
        clocks = sampler.stop(windows) if rank == 0 else {}

        # ---- other operating points (same model, same code path), reported beside the headline -------------
        extra = {}
        if not args.no_extras:
            def side_run(batch):
                w2 = Workload(batch, W + K_)
                ms, _, _ = w2.timed_rounds(w2.device_step, 1, [])
                return ms[0]
            if world > 1 and B % world == 0:
                # the same 64 requests in total, split over the GPUs (per-GPU batch shrinks, the weight stream does not)
                ms = side_run(B // world)
                extra["strong_64_total"] = {"value": B * K_ / (ms * 1e-3), "unit": UNIT, "requests_per_gpu": B // world, "ms_per_step": ms / K_,
                                            "scaling": "strong"}
            if world > 1:
                # the one workload with a real exchange step: the 8B-shaped MatMuls split by columns over the GPUs, each rank's block of
                # columns stored into every rank's output over NVLink by the MatMul kernel itself, beside NCCL all-gather and one GPU
                try:
                    from rmlk_b200 import tpbench
                    torch.cuda.synchronize()
                    extra["tp_matmul"] = tpbench.sweep(world, rank, iters=10)
                except Exception as e:  # reported, not fatal: the headline does not depend on it
                    extra["tp_matmul_error"] = repr(e)[:300]
            if world == 1:
                ms = side_run(1)
                floor_ms = (cfg.params * 4 + cfg.kv_bytes_per_token() * (P + W + K_ // 2)) / (measured_peaks()[0] * 1e9) * 1e3
                extra["decode_batch1"] = {"value": K_ / (ms * 1e-3), "unit": UNIT, "ms_per_step": ms / K_, "hbm_floor_ms_per_step": floor_ms,
                                          "frac_of_hbm_floor": floor_ms / (ms / K_)}

    # ---- self-check (untimed; run after every timed region because the float64 decoder is seconds of heavy work): the logits
    # of the first decode step after the prompt, computed by the very path that was timed above, against a dense float64
    # restatement of the decoder in torch for the first requests of the batch
    selfcheck = None
    if rank == 0 and not args.no_selfcheck:
        wl.restore()
        wl.device_step()
        got = torch.from_numpy(inst.read("logits")).to("cuda")[:, 0]      # [B, vocab]
        nchk = min(2, B)
        seq = torch.from_numpy(np.concatenate([wl.prompt_ids[:nchk], wl.ids_host[0, :nchk].numpy()], axis=1)).to("cuda")
        want = llama.dense_decoder_f64(cfg, weights, seq)
        err = float((got[:nchk].double() - want).abs().max() / want.abs().max())
        same = bool(torch.equal(got[:nchk].argmax(-1), want.argmax(-1)))
        selfcheck = {"rel_err": err, "argmax_equal": same, "requests_checked": nchk, "against": "dense float64 decoder (torch) over the 513 tokens"}
        del got, want, seq
        torch.cuda.empty_cache()

    dev_ms = statistics.median(dev_rounds)
    e2e_ms = statistics.median(e2e_rounds)
    value = world * B * K_ / (dev_ms * 1e-3)
    e2e_value = world * B * K_ / (e2e_ms * 1e-3)
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peak, peak_kind = measured_peaks()
    roof = {}
    if not args.skip_kernel_roofline:
        with torch.cuda.stream(stream):
            per_kernel = kernel_rooflines(B, P + W + K_ // 2, peak, peak_kind)
        roof = dict(per_kernel[DOMINANT])
        roof["other_kernels"] = {k: {"kernel": v["kernel"], "achieved": v["achieved"], "frac": v["frac"], "us_per_launch": v["us_per_launch"]}
                                 for k, v in per_kernel.items() if k != DOMINANT}
    roof["peak_source"] = peak_kind
    # whole-step view: algorithmic bytes of one decode step = the weights once + the KV cache read once + the appended rows
    # (the runtime appends to the cache in place; nothing of the old cache is rewritten)
    ctx_mid = P + W + K_ // 2
    step_bytes = cfg.params * 4 + B * cfg.kv_bytes_per_token() * (ctx_mid + 1)
    roof["step_algorithmic_bytes"] = step_bytes
    roof["step_achieved_gbs"] = step_bytes / (dev_ms / K_ * 1e-3) / 1e9
    roof["step_frac"] = roof["step_achieved_gbs"] / peak

    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        v, threads, sample = cpu_decode_sample(cfg, B, P, CPU_SAMPLE_STEPS)
        cpu = {"value": v, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample}

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K_, "warmup": W, "ms_per_step": dev_ms / K_,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": dict(workload_config(cfg, B, P), **({"host_numa_node_of_rank0": numa_node} if numa_node is not None else {})),
        "roofline": roof, "cpu_baseline": cpu,
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": B * cfg.vocab * 4,
                "ms_per_step": e2e_ms / K_, "rounds_ms_per_step": [m / K_ for m in e2e_rounds]},
        "gpu_launches": launches, "launches_per_decode_step": decode_launches, "prefill_launches": prefill_launches,
        "timed_rounds": {"rounds": R, "each": f"{W} warm-up + {K_} timed steps from the end of the prompt", "reported": "median round",
                         "ms_per_step": [m / K_ for m in dev_rounds]},
        "host_enqueue_ms_per_step": statistics.median(host_one), "host_loop_ms_per_step": statistics.median(host_rounds) / K_, "selfcheck": selfcheck,
        "selfcheck_rel_err": selfcheck["rel_err"] if selfcheck else None, "extra": extra,
        "clocks": clocks, "context_range": [P + W, P + W + K_], "arena_peak_bytes": inst.arena_peak,
    }
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--requests", type=int, default=REQUESTS_PER_GPU)
    ap.add_argument("--prompt", type=int, default=PROMPT)
    ap.add_argument("--rounds", type=int, default=5, help="timed rounds of --steps steps each (the median round is reported)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-selfcheck", action="store_true")
    ap.add_argument("--no-extras", action="store_true")
    ap.add_argument("--skip-kernel-roofline", action="store_true", help="leave out the per-kernel timing (launch-list profiling runs)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
