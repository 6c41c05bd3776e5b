"""Benchmark of the hot path: a Llama-style decoder block executed as a TTNN flatbuffer through
tt::runtime::submit on 1..8 B200s (tensor parallel over a 1xN mesh, one process per GPU).

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference ...      # the CPU oracle on the host cores, same metric

Prints one JSON line (rank 0).  `value` is decoder-block tokens/s with all inputs resident in
HBM; `e2e` is the same through the public API with the step's activations coming from pinned
host memory and the result copied back.  `roofline` describes the dominant kernel (the tcgen05
GEMM) from per-launch CUDA events, against the burst bf16 peak when the timed region is shorter
than a second (`frac_of_sustained` beside it) and with the DRAM traffic read from the committed
ncu summary; `per_op` lists every kernel family the block launches; `clocks` are NVML samples taken
while the timed region runs.  After the timed loops the output of the program that was timed is
compared with the CPU oracle (`parity`; at N > 1 also a digest comparison across ranks) and the
process exits 3 if that fails.  At N = 1 `extra_workloads` adds one line per other benchmark
configuration (f32 MLP, quantization chain, weight-quantized linear, bottleneck block).
Inputs are synthetic (seeded), weights random-init, as the benchmark configuration states.

    --no-parity / --no-extra / --no-cpu-baseline   skip those parts
    --workload <name>                               time another configuration as the main line
    --profile                                       exactly --warmup + --steps passes, for runs under ncu
"""

from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
TRAFFIC_SUMMARY = os.path.join(ROOT, "profiles", "gemm_tcgen05_decoder_dram_traffic.md")
sys.path.insert(0, ROOT)

CONFIG = dict(seq=2048, hidden=4096, n_heads=32, n_kv_heads=8, head_dim=128, ffn=14336, batch=1)
METRIC = "decoder_block_tokens_per_s"
UNIT = "tokens/s"


def gemm_dram_bytes_per_launch():
    """DRAM bytes per launch of the block's GEMM kernel at N = 1, from the committed summary of the ncu
    capture (profiles/gemm_tcgen05_decoder_dram_traffic.md): the "sum" row of its table holds the bytes
    read and written over the launches listed above it.  None when the summary is missing or unreadable."""
    import re
    try:
        rows = [ln for ln in open(TRAFFIC_SUMMARY).read().splitlines() if ln.startswith("|")]
        launches = [ln for ln in rows[2:] if not ln.lower().startswith("| sum")]
        total = next(ln for ln in rows if ln.lower().startswith("| sum"))
        cells = [c.strip() for c in total.strip("|").split("|")]
        read_mb, written_mb = (float(re.match(r"([0-9.]+)\s*MB", cells[i]).group(1)) for i in (3, 4))
        return (read_mb + written_mb) * 1e6 / len(launches)
    except Exception:
        return None


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.samples = []
        self._stop = threading.Event()
        self._thread = None

    NAMES = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
    BITS = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20, "sw_power_cap": 0x4}

    def _nvml_setup(self):
        """NVML (read-only queries): initialised here, on the caller's thread and before the timed
        region, so that the sampling thread only reads."""
        import pynvml
        pynvml.nvmlInit()
        self._nvml = pynvml
        self._h = pynvml.nvmlDeviceGetHandleByIndex(self.gpu)
        self._mx = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        try:
            self._reasons_of = pynvml.nvmlDeviceGetCurrentClocksEventReasons
        except AttributeError:
            self._reasons_of = pynvml.nvmlDeviceGetCurrentClocksThrottleReasons

    def _sample_nvml(self):
        sm = self._nvml.nvmlDeviceGetClockInfo(self._h, self._nvml.NVML_CLOCK_SM)
        r = self._reasons_of(self._h)
        self.samples.append([str(sm), str(self._mx)] + ["Active" if r & self.BITS[n] else "Not Active" for n in self.NAMES])

    def _sample_smi(self):
        try:
            out = subprocess.run(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                  "-i", str(self.gpu)], capture_output=True, text=True, timeout=5).stdout.strip()
            if out:
                self.samples.append([x.strip() for x in out.split(",")])
        except Exception:
            pass

    def _run(self):
        # The timed region of the default run is tens of milliseconds long: NVML every 2 ms; a process
        # per sample (nvidia-smi) only where NVML is unavailable.
        while not self._stop.is_set():
            if self._nvml is not None:
                try:
                    self._sample_nvml()
                except Exception:
                    pass
                self._stop.wait(0.002)
            else:
                self._sample_smi()
                self._stop.wait(0.2)

    def start(self):
        """Sets NVML up, starts the sampling thread, and returns once it has taken a sample, so the
        caller may start its timed region right away."""
        self._nvml = None
        try:
            self._nvml_setup()
        except Exception:
            self._nvml = None
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()
        t0 = time.perf_counter()
        while not self.samples and time.perf_counter() - t0 < 2.0:
            time.sleep(0.0005)
        self._before = len(self.samples)

    def sample_now(self):
        """One more sample from the caller's thread (the bench takes one right after its last launch,
        while the GPU is still busy)."""
        try:
            if self._nvml is not None:
                self._sample_nvml()
        except Exception:
            pass

    def stop(self):
        self._stop.set()
        if self._thread:
            self._thread.join(timeout=10)
        sm, mx, reasons = [], 0, set()
        for s in self.samples:
            try:
                sm.append(float(s[0]))
                mx = max(mx, float(s[1]))
            except (ValueError, IndexError):
                continue
            for name, v in zip(["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"], s[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(sm)}


class Events:
    """CUDA events on the stream the runtime launches on (the library's own stream, not torch's)."""

    def __init__(self, lib, stream):
        self.lib, self.stream = lib, ctypes.c_void_p(stream)
        self.a, self.b = ctypes.c_void_p(), ctypes.c_void_p()
        assert lib.ttb_event_create(ctypes.byref(self.a)) == 0 and lib.ttb_event_create(ctypes.byref(self.b)) == 0

    def start(self):
        assert self.lib.ttb_event_record(self.a, self.stream) == 0

    def stop_ms(self) -> float:
        assert self.lib.ttb_event_record(self.b, self.stream) == 0
        assert self.lib.ttb_event_sync(self.b) == 0
        ms = ctypes.c_float()
        assert self.lib.ttb_event_elapsed_ms(self.a, self.b, ctypes.byref(ms)) == 0
        return float(ms.value)


def dist_env(args):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    if args.gpus > 1 and world == 1:
        raise SystemExit("for --gpus N > 1 launch with torch.distributed.run (one process per GPU)")
    return rank, world, local


def parity_metrics(got, want):
    """The figures the full-size parity tests use (tests/test_configs_gpu.py, tests/test_mesh_gpu.py):
    Pearson correlation, RMS error relative to the output's standard deviation, the share of elements
    within atol 1e-2 + one bf16 ulp of their own magnitude, and the largest error in ulps of the largest
    magnitude.  ok = PCC >= 0.999, RMS <= 1 % of sigma, >= 85 % within atol + 1 ulp, max error <= 2 ulps
    of the largest magnitude.  (Thirty chained bf16 ops: single-ulp disagreements of intermediate
    roundings reach the output through the residual adds; measured 93 % within one ulp on one GPU and
    90 % on two, where each all-reduce adds a rounding of the partial sums.)"""
    import math
    from oracle import metrics
    g, w = got.float(), want.float()
    err, mag = (g - w).abs(), w.abs()
    pcc = float(metrics.get_pcc(want, got))
    rms = err.pow(2).mean().sqrt().item() / max(w.std().item(), 1e-30)
    within = (err <= 1e-2 + 2.0 ** -7 * mag).float().mean().item()
    ulp_at_max = 2.0 ** (math.floor(math.log2(max(mag.max().item(), 1e-30))) - 7)
    max_ulps = err.max().item() / ulp_at_max
    ok = bool(pcc >= 0.999 and rms <= 0.01 and within >= 0.85 and max_ulps <= 2.0 and bool(g.isfinite().all()))
    return {"pcc": pcc, "rms_over_std": rms, "within_atol_1ulp": within, "max_err": err.max().item(),
            "max_err_in_ulps_of_max": max_ulps, "ok": ok}


def check_parity(rt, dist, rank, world, last, full_inputs):
    """Compares the output of the program that was just timed with the CPU oracle of the same graph
    (rank 0; full size, about a second of host time) and, at N > 1, the ranks' outputs with each
    other bit for bit (every rank holds the whole block output after the last all-reduce)."""
    import hashlib
    import torch
    from ttmlir_b200 import graphs
    from oracle.backend import OracleBuilder
    got = rt.to_torch(rt.to_host(last, untilize=True)[0])
    digest = torch.frombuffer(bytearray(hashlib.sha256(got.contiguous().view(torch.uint8).numpy().tobytes()).digest()),
                              dtype=torch.uint8)
    same = True
    if world > 1:
        mine = digest.cuda()
        every = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(every, mine)
        same = all(bool(torch.equal(e, every[0])) for e in every)
    if rank != 0:
        # Wait on the host until rank 0 has finished its oracle pass: a rank that went on alone would
        # sit in its next all-reduce longer than the kernel's one-second patience for a missing peer.
        dist.barrier()
        return None
    t0 = time.perf_counter()
    torch.set_num_threads(os.cpu_count() or 1)   # the launcher pins OMP_NUM_THREADS to 1; the other ranks are idle now
    ob = OracleBuilder(full_inputs, mesh_shape=(1, world))
    graphs.decoder_block_graph(ob, tp=world, **CONFIG)
    want = ob.results()[0]
    if world > 1:
        dist.barrier()
    p = parity_metrics(got, want)
    p.update(bitwise_equal_across_ranks=bool(same), oracle_s=time.perf_counter() - t0,
             against="CPU oracle of the same graph (mesh 1x%d), full size" % world)
    p["ok"] = bool(p["ok"] and same)
    return p


def run_b200(args):
    import torch
    import torch.distributed as dist
    from __graft_entry__ import load_package
    load_package()
    from ttmlir_b200 import graphs, runtime_api as rt

    rank, world, local = dist_env(args)
    torch.cuda.set_device(local)
    nccl_id = None
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        idt = torch.zeros(128, dtype=torch.uint8, device="cuda")
        if rank == 0:
            idt = torch.frombuffer(bytearray(rt.get_nccl_unique_id()), dtype=torch.uint8).cuda()
        dist.broadcast(idt, 0)
        nccl_id = bytes(idt.cpu().numpy().tobytes())

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    device = rt.open_mesh_device(rt.MeshDeviceOptions(mesh_shape=[1, world], device_ids=[local], process_rank=rank,
                                                      process_count=world, nccl_unique_id=nccl_id))
    stream, _ = device.stream(0)
    binary = rt.Binary.load_from_memory(graphs.build_binary(graphs.decoder_block_graph, mesh_shape=(1, world), tp=world,
                                                            presharded=world > 1, **CONFIG))
    rt.set_compatible_device_runtime(binary)
    full = graphs.decoder_block_inputs(**CONFIG)
    mine = graphs.shard_inputs(full, graphs.decoder_shard_dims(**CONFIG), world, rank)
    # weights and tables stay resident (retain); the activations are the per-step input
    dev_in = [rt.to_layout(rt.from_torch(t), device, rt.get_layout(binary, 0, i), retain=True) for i, t in enumerate(mine)]
    tokens = CONFIG["batch"] * CONFIG["seq"]

    def step_resident():
        return rt.submit(device, binary, 0, dev_in)[0]

    # End to end at N > 1 every rank feeds and receives its own 1/N of the sequence: the program
    # variant with sequence-sharded I/O gathers the activations over NVLink first and returns each
    # rank's rows, so host traffic per step is one copy of the activations each way in total.
    if world > 1:
        e2e_binary = rt.Binary.load_from_memory(graphs.build_binary(
            graphs.decoder_block_graph, mesh_shape=(1, world), tp=world, presharded=True, io_seq_sharded=True, **CONFIG))
        x_rows = torch.chunk(full[0], world, dim=1)[rank].contiguous()
    else:
        e2e_binary, x_rows = binary, mine[0]
    x_host = x_rows.clone().pin_memory()
    x_tensor = rt.from_torch(x_host)
    x_layout = rt.get_layout(e2e_binary, 0, 0)
    out_bytes = x_rows.numel() * x_rows.element_size()

    def read_result(h):
        """The step's result is in host memory once wait() returns; look at it in place."""
        rt.wait(h)
        view = (ctypes.c_uint16 * 2).from_address(h.host_ptr() + out_bytes - 4)
        return view[0] ^ view[1]

    def run_e2e(n):
        """n steps through the public API with host buffers on both sides.  A step uploads its
        activations from pinned memory (to_layout), runs (submit) and downloads its result
        (to_host, non-blocking); the three run on their own streams, so the upload of step
        i+1 and the download of step i-1 overlap the compute of step i.  The host reads the
        result of step i - depth while step i is in flight (depth = --e2e-depth); every step's
        result is read on the host before the loop ends."""
        pending, acc = [], 0
        clock = time.perf_counter
        for _ in range(n):
            t0 = clock()
            xd = rt.to_layout(x_tensor, device, x_layout)                     # H2D from pinned memory
            t1 = clock()
            out = rt.submit(device, e2e_binary, 0, [xd] + dev_in[1:])[0]
            t2 = clock()
            pending.append(rt.to_host(out, untilize=True, blocking=False)[0])  # D2H into pinned memory
            t3 = clock()
            if len(pending) > args.e2e_depth:
                acc ^= read_result(pending.pop(0))
            t4 = clock()
            for k, dt in zip(("to_layout", "submit", "to_host", "wait_and_read"), (t1 - t0, t2 - t1, t3 - t2, t4 - t3)):
                e2e_host[k] = e2e_host.get(k, 0.0) + dt
        while pending:
            acc ^= read_result(pending.pop(0))
        return acc

    e2e_host = {}  # where the host spends its time in the end-to-end loop (seconds, summed over the timed steps)

    for _ in range(args.warmup if args.profile else max(args.warmup, 3)):
        step_resident()
    rt.wait(step_resident())

    # ---- value: inputs resident in HBM ------------------------------------------------------
    sampler = ClockSampler(local)
    ev = Events(rt.lib, stream)
    sampler.start()          # NVML is set up and the first sample taken before the region starts
    barrier()
    launches0 = rt.launch_count()
    ev.start()
    last = None
    t_host = time.perf_counter()
    for _ in range(args.steps):
        last = step_resident()
    host_submit_us = (time.perf_counter() - t_host) / args.steps * 1e6   # CPU time to enqueue one step
    sampler.sample_now()     # everything is enqueued and the GPU still busy
    ms = ev.stop_ms()
    launches = rt.launch_count() - launches0
    barrier()
    clocks = sampler.stop()
    t = torch.tensor([ms], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_total = float(t.item())

    if args.profile:
        return dict(rank=rank, world=world, ms_total=ms_total, e2e_s=float("nan"), launches=launches, clocks=clocks,
                    prof=[], prof_steps=1, tokens=tokens, bytes_io=mine[0].numel() * 2, rt=rt, device=device,
                    host_submit_us=host_submit_us)

    # ---- e2e: host buffers in, host buffers out ---------------------------------------------
    # Like the resident loop, the end-to-end loop starts from an idle GPU: after --idle-s seconds
    # without work the clocks and the power budget are where they were before the first loop.
    if args.idle_s > 0:
        barrier()
        time.sleep(args.idle_s)
    run_e2e(3)
    barrier()
    e2e_host.clear()
    t0 = time.perf_counter()
    run_e2e(args.steps)
    barrier()
    e2e_s = time.perf_counter() - t0
    t = torch.tensor([e2e_s], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_s = float(t.item())

    # ---- parity of what was timed (outside every timed region) --------------------------------
    parity = check_parity(rt, dist if world > 1 else None, rank, world, last, full) if not args.no_parity else None

    # ---- per-kernel achieved rates from per-launch events (separate pass) ---------------------
    rt.lib.ttb_prof_enable(1)
    prof_steps = min(args.steps, 5)
    for _ in range(prof_steps):
        last = step_resident()
    rt.wait(last)
    buf = ctypes.create_string_buffer(1 << 16)
    assert rt.lib.ttb_prof_summary(buf, ctypes.c_size_t(len(buf))) == 0
    rt.lib.ttb_prof_enable(0)
    prof = json.loads(buf.value.decode())
    return dict(rank=rank, world=world, ms_total=ms_total, e2e_s=e2e_s, launches=launches, clocks=clocks, prof=prof,
                prof_steps=prof_steps, tokens=tokens, bytes_io=mine[0].numel() * 2, rt=rt, device=device,
                host_submit_us=host_submit_us, parity=parity,
                e2e_host_us={k: v / args.steps * 1e6 for k, v in e2e_host.items()})


# ---- the CPU oracle as baseline / reference arm -------------------------------------------------
def time_oracle(seq: int, iters: int, threads: int):
    """Seconds per pass of the decoder block through the CPU oracle (f32 math per op, bf16
    between ops), at `seq` tokens."""
    import torch
    from __graft_entry__ import load_package
    load_package()
    from ttmlir_b200 import graphs
    from oracle.backend import OracleBuilder
    torch.set_num_threads(threads)
    cfg = dict(CONFIG, seq=seq)
    ins = graphs.decoder_block_inputs(**cfg)

    def once():
        ob = OracleBuilder(ins)
        graphs.decoder_block_graph(ob, **cfg)
        return ob.results()[0]
    once()
    t0 = time.perf_counter()
    for _ in range(iters):
        once()
    return (time.perf_counter() - t0) / iters


def cpu_baseline(budget_s: float = 20.0):
    threads = os.cpu_count() or 1
    seq = CONFIG["seq"]
    probe = time_oracle(256, 1, threads)          # scale the sample to the time budget
    est_full = probe * (seq / 256) * 1.3
    if est_full * 2 > budget_s:
        seq = max(256, int(seq * budget_s / (est_full * 2)) // 256 * 256)
    sec = time_oracle(seq, 1, threads)
    return {"value": CONFIG["batch"] * seq / sec, "unit": UNIT, "cores": threads, "kind": "port",
            "sample": f"CPU oracle (torch f32 per op, bf16 between ops), one pass over {seq} of {CONFIG['seq']} tokens"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return None
    threads = os.cpu_count() or 1
    # Bound the run: each step is one pass over a sample of the sequence sized so that
    # warmup + steps stay within a few minutes.
    probe = time_oracle(256, 1, threads)
    seq = CONFIG["seq"]
    total = (args.steps + args.warmup) * probe * (seq / 256) * 1.3
    while total > 150.0 and seq > 256:
        seq //= 2
        total /= 2.2
    sec = time_oracle(seq, max(args.steps, 1), threads)
    value = CONFIG["batch"] * seq / sec
    sample = f"CPU oracle, {args.steps} passes over {seq} of {CONFIG['seq']} tokens, {threads} host threads"
    return {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "llama-style decoder block (BASELINE config 4), seq 2048, hidden 4096, 32q/8kv heads, ffn 14336",
                   "sample_tokens": seq},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }


# ---- the other benchmark configurations (single GPU), as extra report lines -----------------------
def side_workloads():
    """name -> (graph function, kwargs, input maker, algorithmic bytes, algorithmic flops, units per step, unit name)."""
    from ttmlir_b200 import graphs
    n2 = 4096 * 4096
    m3, k3, n3 = 2048, 4096, 11008
    px = 64 * 56 * 56
    return {
        "mlp": (graphs.mlp_graph, {}, graphs.mlp_inputs, 1220648.0, 52035584.0, 128, "rows"),
        # the same program hoisted into a trace (one CUDA graph replay per submit; the activation is
        # staged from host memory every step, as the trace contract has it)
        "mlp_traced": (graphs.mlp_traced_binary, {}, graphs.mlp_inputs, 1220648.0, 52035584.0, 128, "rows"),
        "quant": (graphs.quant_chain_graph, {}, graphs.quant_chain_inputs, 6.0 * n2, 0.0, n2, "elements"),
        "quant_int8": (graphs.quant_chain_graph, {"container": "Int8"}, graphs.quant_chain_inputs, 6.0 * n2, 0.0, n2, "elements"),
        "w8_linear": (graphs.w8_linear_graph, {}, graphs.w8_linear_inputs, 107020800.0, 2.0 * m3 * k3 * n3, m3, "rows"),
        # both operands quantized: activations per tensor (quantized on the fly), weights per channel; the contraction
        # runs on the 8-bit values (tcgen05.mma kind::i8) with the dequantize fused.  Algorithmic bytes: bf16
        # activations, int8 weights, f32 scales, bf16 bias and result once each.
        "w8a8_linear": (graphs.w8a8_linear_graph, {}, graphs.w8a8_linear_inputs, 107020800.0, 2.0 * m3 * k3 * n3, m3, "rows"),
        # the weight's dequantization hoisted into a const-eval function (evaluated once, then cached)
        "w8_linear_const_eval": (graphs.w8_linear_const_eval_binary, {}, graphs.w8_linear_inputs, 107020800.0,
                                 2.0 * m3 * k3 * n3, m3, "rows"),
        # serving: attention of one decode step, 32 users x 8192 cached tokens (1.07 GB of K and V read once)
        "decode_attention": (graphs.decode_attention_graph, {}, graphs.decode_attention_inputs,
                             2.0 * 32 * 8 * 8192 * 128 * 2 + 2.0 * 32 * 32 * 128 * 2, 4.0 * 32 * 32 * 8192 * 128, 32, "tokens"),
        # the N = 1 decoder block recorded as a trace (one CUDA graph replay per submit)
        "decoder_traced": (graphs.decoder_block_traced_binary, dict(CONFIG), lambda: graphs.decoder_block_inputs(**CONFIG),
                           0.0, graphs.decoder_block_flops(**CONFIG), CONFIG["batch"] * CONFIG["seq"], "tokens"),
        "bottleneck": (graphs.bottleneck_graph, {}, graphs.bottleneck_inputs, 128450560.0, 29.595e9, 64, "images"),
    }


def side_parity(workload, got, want):
    """Outputs of a side workload against the CPU oracle of the same graph at full size: integer
    tensors and the quantization chain bit for bit, f32 within 1e-4, bf16 with PCC >= 0.999 and
    |err| <= 3e-2 + 2^-6 |want| (two bf16 ulps; the tolerance of tests/test_configs_gpu.py)."""
    import torch
    from oracle import metrics
    res = {"ok": True, "outputs": []}
    for g, w in zip(got, want):
        if workload.startswith("quant") or not w.is_floating_point():
            bad = int((g != w).sum().item()) if g.shape == w.shape else -1
            res["outputs"].append({"bit_exact": bad == 0, "mismatches": bad})
            res["ok"] = res["ok"] and bad == 0
            continue
        tol = (0.999, 1e-4, 1e-4) if w.dtype == torch.float32 else (0.999, 3e-2, 2.0 ** -6)
        ok, report = metrics.check_close(w, g, *tol)
        res["outputs"].append({"ok": bool(ok), "report": report})
        res["ok"] = res["ok"] and bool(ok)
    return res


def measure_side(args, workload, steps=None, with_parity=True):
    """One of the single-GPU configurations through submit with resident inputs; returns its JSON line."""
    import torch  # noqa: F401
    from __graft_entry__ import load_package
    load_package()
    from ttmlir_b200 import graphs, runtime_api as rt
    graph, kw, make_inputs, abytes, aflops, units, unit_name = side_workloads()[workload]
    steps = steps or args.steps
    peaks = measured_peaks()
    device = rt.open_mesh_device(rt.MeshDeviceOptions(mesh_shape=[1, 1]))
    stream, _ = device.stream(0)
    whole_binary = graph.__name__.endswith("_binary")  # multi-program files come from their own factory
    binary = rt.Binary.load_from_memory(graph(**kw) if whole_binary else graphs.build_binary(graph, **kw))
    ins = make_inputs()
    dev_in = [rt.to_layout(rt.from_torch(t), device, rt.get_layout(binary, 0, i), retain=True) for i, t in enumerate(ins)]
    for _ in range(args.warmup if args.profile else max(args.warmup, 3)):
        out = rt.submit(device, binary, 0, dev_in)
    rt.wait(out[0])
    ev = Events(rt.lib, stream)
    launches0 = rt.launch_count()
    ev.start()
    t_host = time.perf_counter()
    for _ in range(steps):
        out = rt.submit(device, binary, 0, dev_in)
    host_us = (time.perf_counter() - t_host) / steps * 1e6
    ms = ev.stop_ms() / steps
    launches = rt.launch_count() - launches0
    parity = None
    if with_parity and not args.profile and not whole_binary:
        from oracle.backend import OracleBuilder
        got = [rt.to_torch(rt.to_host(o, untilize=True)[0]) for o in out]
        ob = OracleBuilder(ins)
        graph(ob, **kw)
        parity = side_parity(workload, got, ob.results())
    # The same pass with cold caches: several of these workloads are smaller than the 126 MB L2, so the
    # loop above re-reads inputs the previous pass left there.  Here a 256 MB buffer is overwritten
    # before every pass (outside the timed region) and every pass is timed on its own.
    flushed_ms = None
    if not args.profile:
        scratch = ctypes.c_void_p()
        flush_bytes = 256 << 20
        assert rt.lib.ttb_malloc(ctypes.byref(scratch), ctypes.c_size_t(flush_bytes), ctypes.c_void_p(stream)) == 0
        total = 0.0
        reps = min(steps, 30)
        for _ in range(reps):
            assert rt.lib.ttb_memset(scratch, 0, ctypes.c_size_t(flush_bytes), ctypes.c_void_p(stream)) == 0
            ev.start()
            out = rt.submit(device, binary, 0, dev_in)
            total += ev.stop_ms()
        flushed_ms = total / reps
        assert rt.lib.ttb_free(scratch, ctypes.c_void_p(stream)) == 0
    prof = []
    if not args.profile:
        rt.lib.ttb_prof_enable(1)
        for _ in range(min(steps, 5)):
            out = rt.submit(device, binary, 0, dev_in)
        rt.wait(out[0])
        buf = ctypes.create_string_buffer(1 << 16)
        assert rt.lib.ttb_prof_summary(buf, ctypes.c_size_t(len(buf))) == 0
        rt.lib.ttb_prof_enable(0)
        for k in json.loads(buf.value.decode()):
            e = {"kernel": k["tag"], "launches_per_step": k["launches"] / min(steps, 5), "avg_ms": k["ms"] / k["launches"]}
            if k["flops"] > 0:
                e.update(achieved=k["flops"] / (k["ms"] * 1e-3) / 1e12, unit="TFLOP/s")
                e["frac"] = e["achieved"] / peaks["bf16_tflops"]
            elif k["bytes"] > 0:
                e.update(achieved=k["bytes"] / (k["ms"] * 1e-3) / 1e9, unit="GB/s")
                e["frac"] = e["achieved"] / peaks["hbm_gbs"]
            prof.append(e)
    line = {"metric": f"{workload}_{unit_name}_per_s", "value": units / (ms * 1e-3), "unit": f"{unit_name}/s",
            "n_gpus": 1, "steps": steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
            "dtype": "f32" if workload.startswith("mlp") else "bf16", "data": "synthetic",
            "config": {"workload": workload, "host_enqueue_us_per_step": host_us}, "gpu_launches": launches,
            "ms_per_step_l2_flushed": flushed_ms,
            "graph_hbm_gbs": abytes / (ms * 1e-3) / 1e9, "graph_hbm_frac": abytes / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
            "graph_tflops": aflops / (ms * 1e-3) / 1e12, "graph_tensor_frac": aflops / (ms * 1e-3) / 1e12 / peaks["bf16_tflops"],
            "peak_source": f"{peaks['source']} (HBM copy; burst bf16)", "parity": parity, "per_op": prof}
    rt.close_mesh_device(device)
    return line


def run_side(args):
    print(json.dumps(measure_side(args, args.workload)))


def run_all_reduce(args):
    """The block's all-reduce (sum of [2048, 4096] bf16, 16.8 MB) on an in-process 1 x N mesh: the
    peer-memory kernel with its operand already staged (as after a GEMM), with a staging copy, with
    the fused residual add, and NCCL.  One process launches on all N devices in turn, so the
    figures include that launch skew."""
    from __graft_entry__ import load_package
    load_package()
    from ttmlir_b200 import runtime_api as rt
    lib, n = rt.lib, args.gpus
    count = 2048 * 4096
    devs = (ctypes.c_int * n)(*range(n))
    symms, comms = (ctypes.c_void_p * n)(), (ctypes.c_void_p * n)()

    def ck(rc):
        if rc != 0:
            raise RuntimeError(lib.ttb_last_error().decode())
    ck(lib.ttb_symm_create_all(symms, n, devs, ctypes.c_size_t(64 << 20)))
    ck(lib.ttb_comm_init_all(comms, n, devs))
    streams, ins, outs, ress = [], [], [], []
    for d in range(n):
        ck(lib.ttb_set_device(d))
        st = ctypes.c_void_p()
        ck(lib.ttb_stream_create(ctypes.byref(st)))
        streams.append(st)
        for lst in (ins, outs, ress):
            p = ctypes.c_void_p()
            ck(lib.ttb_malloc(ctypes.byref(p), ctypes.c_size_t(count * 2), st))
            ck(lib.ttb_memset(p, 0, ctypes.c_size_t(count * 2), st))
            lst.append(p)
        ck(lib.ttb_stream_sync(st))

    def symm(staged, residual):
        for d in range(n):
            ck(lib.ttb_set_device(d))
            src = ins[d]
            if staged:
                src = ctypes.c_void_p()
                ck(lib.ttb_symm_input_buffer(symms[d], ctypes.c_size_t(count * 2), ctypes.byref(src)))
            ck(lib.ttb_symm_all_reduce(symms[d], src, ress[d] if residual else None, outs[d], ctypes.c_size_t(count), 2, streams[d]))

    def nccl():
        ck(lib.ttb_group_start())
        for d in range(n):
            ck(lib.ttb_set_device(d))
            ck(lib.ttb_all_reduce(comms[d], ins[d], outs[d], ctypes.c_size_t(count), 2, 0, streams[d]))
        ck(lib.ttb_group_end())

    def timed(fn):
        for _ in range(max(args.warmup, 3)):
            fn()
        for d in range(n):
            ck(lib.ttb_set_device(d))
            ck(lib.ttb_stream_sync(streams[d]))
        ck(lib.ttb_set_device(0))
        ev = Events(lib, streams[0].value)
        ev.start()
        for _ in range(args.steps):
            fn()
        ck(lib.ttb_set_device(0))
        ms = ev.stop_ms()
        for d in range(n):
            ck(lib.ttb_set_device(d))
            ck(lib.ttb_stream_sync(streams[d]))
        return ms / args.steps * 1e3
    res = {"staged": timed(lambda: symm(True, False)), "staged_residual": timed(lambda: symm(True, True)),
           "copied": timed(lambda: symm(False, False)), "nccl": timed(nccl)}
    status = ctypes.c_int(-1)
    ck(lib.ttb_symm_status(symms[0], ctypes.byref(status)))
    peaks = measured_peaks()
    us = res["staged_residual"]
    # bytes crossing the links per rank and direction: one-shot (n = 2) pulls the whole operand,
    # two-shot pulls and pushes (n-1)/n of it
    link_bytes = count * 2 * (1.0 if n == 2 else 2.0 * (n - 1) / n)
    print(json.dumps({"metric": "all_reduce_us", "value": us, "unit": "us", "n_gpus": n, "steps": args.steps, "warmup": args.warmup,
                      "higher_is_better": False, "dtype": "bf16", "data": "synthetic",
                      "config": {"workload": "all_reduce(sum) of [2048, 4096] bf16 + residual add, in-process 1xN mesh"},
                      "us": res, "status": status.value,
                      "roofline": {"bound": "nvlink", "achieved": link_bytes / (us * 1e-6) / 1e9, "peak": 770.0, "unit": "GB/s",
                                   "frac": link_bytes / (us * 1e-6) / 1e9 / 770.0,
                                   "peak_source": "measured peer copy per direction on this pool"}}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-parity", action="store_true", help="skip the comparison of the timed program's output with the CPU oracle")
    ap.add_argument("--no-extra", action="store_true",
                    help="N = 1 only: skip the short passes over the other benchmark configurations (extra_workloads)")
    ap.add_argument("--e2e-depth", type=int, default=2,
                    help="steps in flight in the end-to-end loop before the host reads a result")
    ap.add_argument("--idle-s", type=float, default=1.0,
                    help="idle time before the end-to-end loop, so that it starts from the same GPU state as the resident loop")
    ap.add_argument("--profile", action="store_true",
                    help="for runs under a profiler: exactly --warmup warm-up steps, then --steps steps, nothing else")
    ap.add_argument("--workload", default="decoder",
                    choices=["decoder", "mlp", "mlp_traced", "quant", "quant_int8", "w8_linear", "w8a8_linear", "w8_linear_const_eval",
                             "bottleneck", "decode_attention", "decoder_traced", "all_reduce"],
                    help="decoder (default) is the benchmark; the others report the remaining configurations")
    args = ap.parse_args()

    if args.workload == "all_reduce":
        run_all_reduce(args)
        return
    if args.workload != "decoder":
        run_side(args)
        return
    if args.impl == "reference":
        line = run_reference(args)
        if line is not None:
            print(json.dumps(line))
        return

    r = run_b200(args)
    if r["rank"] != 0:
        r["rt"].close_mesh_device(r["device"])
        return
    from ttmlir_b200 import graphs
    peaks = measured_peaks()
    steps, tokens = args.steps, r["tokens"]
    ms_step = r["ms_total"] / steps
    value = tokens * steps / (r["ms_total"] * 1e-3)
    e2e_value = tokens * steps / r["e2e_s"]
    world = r["world"]

    # Tensor-core fractions: the burst cuBLAS figure when the timed region is shorter than a second
    # (clocks are still near their maximum), the sustained figure for longer loops; both are reported.
    region_s = r["ms_total"] * 1e-3
    burst = region_s < 1.0
    tensor_peak = peaks["bf16_tflops"] if burst else peaks["bf16_tflops_sustained"]
    per_op, dominant = [], None
    for k in r["prof"]:
        ms = k["ms"] / max(k["launches"], 1)
        entry = {"kernel": k["tag"], "launches_per_step": k["launches"] / r["prof_steps"], "avg_ms": ms}
        if k["flops"] > 0:
            tf = k["flops"] / (k["ms"] * 1e-3) / 1e12
            entry.update(bound="tensor", achieved=tf, unit="TFLOP/s", frac=tf / tensor_peak,
                         frac_of_sustained=tf / peaks["bf16_tflops_sustained"])
        elif k["bytes"] > 0:
            gbs = k["bytes"] / (k["ms"] * 1e-3) / 1e9
            entry.update(bound="hbm", achieved=gbs, unit="GB/s", frac=gbs / peaks["hbm_gbs"])
        entry["share_of_step"] = k["ms"] / r["prof_steps"] / ms_step
        per_op.append(entry)
        if dominant is None or k["ms"] > dominant[1]:
            dominant = (entry, k["ms"])
    per_op.sort(key=lambda e: -e["share_of_step"])
    dom = dominant[0] if dominant else {}
    traffic = gemm_dram_bytes_per_launch() if (world == 1 and dom.get("kernel") == "gemm_tcgen05") else None
    roofline = {"kernel": dom.get("kernel"), "bound": dom.get("bound"), "achieved": dom.get("achieved"),
                "peak": tensor_peak if dom.get("bound") == "tensor" else peaks["hbm_gbs"],
                "unit": dom.get("unit"), "frac": dom.get("frac"), "frac_of_sustained": dom.get("frac_of_sustained"),
                # DRAM bytes per launch of the dominant kernel, from the committed summary of an ncu capture of this workload
                "traffic": traffic,
                "traffic_unit": "bytes per launch (ncu dram__bytes_read.sum + dram__bytes_write.sum, N=1 capture, "
                                "profiles/gemm_tcgen05_decoder_dram_traffic.md)",
                "peak_source": f"{peaks['source']} ({'burst' if burst else 'sustained'} bf16 figure: the timed region is "
                               f"{region_s * 1e3:.1f} ms long)"}
    flops = graphs.decoder_block_flops(**CONFIG)
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": steps, "warmup": args.warmup,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": "llama-style decoder block (BASELINE config 4), seq 2048, hidden 4096, 32q/8kv heads, ffn 14336",
                   "parallelism": f"tp{world}", "l2": "inputs larger than L2 (436 MB of weights per step vs 126 MB)",
                   "block_tflops_per_s": flops * steps / (r["ms_total"] * 1e-3) / 1e12,
                   "host_enqueue_us_per_step": r["host_submit_us"],
                   "e2e_host_us_per_step": r.get("e2e_host_us", {}),
                   "e2e_idle_s_before": args.idle_s,
                   "e2e_io": ("pipelined loop, depth %d; " % args.e2e_depth) +
                             ("every rank uploads and downloads its 1/%d of the sequence (all_gather first, mesh_partition last)" % world
                              if world > 1 else "the activations are uploaded and the result downloaded every step")},
        "clocks": r["clocks"], "gpu_launches": r["launches"],
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": r["bytes_io"], "d2h_bytes_per_step": r["bytes_io"]},
        "roofline": roofline, "per_op": per_op,
    }
    if r.get("parity") is not None:
        line["parity"] = r["parity"]
    if world == 1 and not args.no_cpu_baseline and not args.profile:
        line["cpu_baseline"] = cpu_baseline()
    r["rt"].close_mesh_device(r["device"])
    if world == 1 and not args.no_extra and not args.profile:
        # The other benchmark configurations, a short pass each (resident inputs, back to back and with L2
        # flushed, per-kernel fractions, parity against the CPU oracle at full size).
        extra = []
        for name in ("mlp", "quant", "quant_int8", "w8_linear", "w8a8_linear", "bottleneck"):
            try:
                e = measure_side(args, name, steps=min(args.steps, 20))
                extra.append({k: e[k] for k in ("metric", "value", "unit", "ms_per_step", "ms_per_step_l2_flushed", "gpu_launches",
                                                "graph_hbm_frac", "graph_tensor_frac", "parity", "per_op")})
            except Exception as ex:  # a side line must not take the headline down with it
                extra.append({"metric": name, "error": str(ex)[:300]})
        line["extra_workloads"] = extra
    print(json.dumps(line))
    if line.get("parity") is not None and not line["parity"]["ok"]:
        sys.exit(3)


if __name__ == "__main__":
    main()
