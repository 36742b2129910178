#!/usr/bin/env python
"""Benchmark of the quantized-matmul hot path on B200, through the plugin's C ABI.

    python bench.py --gpus N --steps K --warmup W [--impl reference]

Workload at N = 1 (the decode configuration the metric is quoted on):
the decode GEMV sweep  x bf16 [M in {1,4,8,16}, K=4096] . W^T,  W [N=11008,
K=4096] 4-bit affine, group 64, bf16 scales/biases, fp32 accumulate, bf16 out.
A "step" is REPS passes over the sweep; every launch reads a different one of
R resident weight sets (R * 25.4 MB = 305 MB > 2 x L2), so each launch streams
its weights from HBM, never from L2.  value = algorithmic bytes of all
launches / device time (CUDA events on the launching stream), GB/s.

At N > 1 (torchrun, one process per GPU) the layer is column-sharded: every
rank holds its own 11008-column slice (weak scaling: the logical layer has
N * 11008 columns), and the decode kernel delivers its columns to every rank
over NVLink itself (qmatmul_sharded_push; --nccl-allgather: NCCL all-gather +
interleave instead).  Time = max over ranks.  After the sweep the two sharded
configurations proper run as strong-scaling legs (8-bit large GEMM, the
quantized-linear chain; --no-sharded-legs skips them).

`e2e` is the same metric through the reference-facing calls with HOST (page-
locked) buffers: buffer_copy_from_host_async(x) -> qmatmul ->
buffer_copy_to_host(y) per launch.
`--impl reference` times the CPU implementation of the path (the oracle, in
the reference CPU backend's loop style, all host threads) on a bounded sample.
"""
import argparse
import ctypes as C
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

# dram__bytes_read.sum + dram__bytes_write.sum of one qmv_mma launch (M=1) of this workload, from an ncu capture
# of `bench.py --kernel-only --no-graph` (counters cannot be read inside the timed run)
NCU_TRAFFIC_BYTES = 25461632.0
NCU_TRAFFIC_BYTES_BATCH = 919669248.0  # one qmv_batch<4,m8> launch of the sweep (ncu, dram read + write)
SWEEPS_PER_GRAPH = 5  # sweeps (of 4 x 12 launches) recorded in the CUDA graph the timed step replays

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "4-bit qmatmul: decode GEMV HBM GB/s; prefill GEMM TFLOPS; % of roofline"
K_DEC, N_DEC, BITS, GROUP = 4096, 11008, 4, 64
M_SWEEP = (1, 4, 8, 16)
R_SETS = 12
NOMINAL_HBM_GBS = 8000.0
FALLBACK_HBM_GBS = 6650.0


def e2e_driver_path():
    """The C host loop of the end-to-end leg (bench_e2e.c), built on demand with the host compiler."""
    here = os.path.dirname(os.path.abspath(__file__))
    src, lib = os.path.join(here, "bench_e2e.c"), os.path.join(here, "mlx_b200", "lib", "libbench_e2e.so")
    if not os.path.exists(lib) or os.path.getmtime(lib) < os.path.getmtime(src):
        cc = "/usr/bin/gcc" if os.path.exists("/usr/bin/gcc") else "gcc"
        subprocess.run([cc, "-O2", "-shared", "-fPIC", "-fvisibility=hidden", "-o", lib, src], check=True)
    return lib


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d, "measured"
    return {"hbm_gbs": FALLBACK_HBM_GBS, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


def shared_config():
    """The workload as both arms (GPU, CPU reference) name it."""
    return {"workload": "decode_gemv_sweep", "M": list(M_SWEEP), "K": K_DEC, "N": N_DEC, "bits": BITS, "group": GROUP,
            "l2": f"GPU arm: inputs larger than L2 ({R_SETS} rotating weight sets = {R_SETS * alg_bytes(1) / 1e6:.0f} MB, each launch "
                  "reads a set last touched 11 launches earlier); CPU arm: one layer, host caches as they fall"}


def alg_bytes(M, K=K_DEC, N=N_DEC):
    # every operand exactly once: packed weights + scales + biases + x + y  (bf16 = 2 B)
    return N * K * BITS // 8 + 2 * (N * K // GROUP) * 2 + M * K * 2 + M * N * 2


class ClockSampler:
    """nvidia-smi clocks and throttle reasons during the timed region."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.index)], stdout=subprocess.PIPE, text=True)
            self.thread = threading.Thread(target=lambda: self.lines.extend(self.proc.stdout), daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        self.thread.join(timeout=5)
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [t.strip() for t in ln.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0])); mx.append(float(f[1]))
            except ValueError:
                continue
            for nm, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# ---------------------------------------------------------------------------
# CPU baseline (the oracle; test infrastructure used here only as the baseline)
# ---------------------------------------------------------------------------
def cpu_baseline(limit_s=12.0):
    import oracle as O
    wq, s, b = O.make_layer(N_DEC, K_DEC, BITS, GROUP, O.BF16, config_id=2)
    xs = {M: O.make_x(M, K_DEC, O.BF16, config_id=2, tag=M) for M in M_SWEEP}
    O.qmatmul_ref_rowcache(xs[1], wq, s, b, BITS, GROUP)  # warm
    t0 = time.perf_counter()
    nbytes, sweeps = 0, 0
    while True:
        for M in M_SWEEP:
            O.qmatmul_ref_rowcache(xs[M], wq, s, b, BITS, GROUP)
            nbytes += alg_bytes(M)
        sweeps += 1
        dt = time.perf_counter() - t0
        if dt > limit_s or sweeps >= 50:
            break
    return {"value": nbytes / dt / 1e9, "unit": "GB/s", "cores": O.num_threads(), "kind": "port",
            "sample": f"{sweeps} sweep(s) of M in {list(M_SWEEP)} over one 11008x4096 4-bit layer, "
                      f"{dt:.1f} s, OpenMP over output rows, fp32 sequential k-sum (reference CPU backend style)"}, dt, sweeps


def run_reference(args, rank):
    if rank != 0:
        return
    import oracle as O
    O.build()
    wq, s, b = O.make_layer(N_DEC, K_DEC, BITS, GROUP, O.BF16, config_id=2)
    xs = {M: O.make_x(M, K_DEC, O.BF16, config_id=2, tag=M) for M in M_SWEEP}

    def step():
        for M in M_SWEEP:
            O.qmatmul_ref_rowcache(xs[M], wq, s, b, BITS, GROUP)

    for _ in range(max(1, min(args.warmup, 3))):
        step()
    steps = max(1, min(args.steps, 20))
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = time.perf_counter() - t0
    nbytes = steps * sum(alg_bytes(M) for M in M_SWEEP)
    val = nbytes / dt / 1e9
    sample = (f"{steps} step(s), each one sweep of M in {list(M_SWEEP)} over one 11008x4096 4-bit layer "
              f"(the GPU arm's step is {args.reps} such sweeps over {R_SETS} weight sets)")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": val, "unit": "GB/s", "n_gpus": args.gpus, "steps": steps,
        "warmup": args.warmup, "ms_per_step": dt / steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": shared_config(),
        "cpu_baseline": {"value": val, "unit": "GB/s", "cores": O.num_threads(), "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "the reference has no quantized matmul; this is its CPU backend's matmul loop "
                "(src/cpu_backend.cpp:243-266) with unpack+dequant fused, from oracle/qmm_oracle.c",
    }))


def cpu_reference_config_leg(ctx, O):
    """The CPU-backend reference configuration (x fp32 [1,4096]; W [4096,4096] 4-bit g64, fp32 scales, biases =
    -8*scale + N(0,1e-3); y fp32): the GPU fp32 path (qmv_simt) and the CPU restatement in the reference backend's
    loop style, on the same inputs, each checked against the fp64 truth before it is timed."""
    from mlx_b200 import F32
    M, K, N, bits, group = 1, 4096, 4096, 4, 64
    wq, s, b = O.make_layer(N, K, bits, group, O.F32, config_id=1, bias_noise=1e-3)
    x = O.make_x(M, K, O.F32, config_id=1)
    truth = O.qmatmul_truth(x, wq, s, b, bits, group)
    nbytes = N * K * bits // 8 + 2 * (N * K // group) * 4 + M * K * 4 + M * N * 4
    bx, bw, bs, bb = ctx.upload(x), ctx.upload(wq), ctx.upload(s), ctx.upload(b)
    by = ctx.empty((M, N), np.float32)
    ctx.qmatmul(bx, bw, bs, bb, by, M, K, N, bits, group, F32, F32, F32)
    err_gpu, _ = O.rel_err(by.to_host(), truth)
    for _ in range(5):
        ctx.qmatmul(bx, bw, bs, bb, by, M, K, N, bits, group, F32, F32, F32)
    ctx.sync()
    iters = 50
    ctx.timer_record(12)
    for _ in range(iters):
        ctx.qmatmul(bx, bw, bs, bb, by, M, K, N, bits, group, F32, F32, F32)
    ctx.timer_record(13)
    us_gpu = ctx.timer_elapsed_ms(12, 13) * 1e3 / iters
    kern = ctx.last_kernel()
    for h in (bx, bw, bs, bb, by):
        h.free()
    y_cpu = O.qmatmul_ref(x, wq, s, b, bits, group)
    err_cpu, _ = O.rel_err(y_cpu, truth)
    for _ in range(3):
        O.qmatmul_ref(x, wq, s, b, bits, group)
    ts = []
    for _ in range(10):
        t0 = time.perf_counter()
        O.qmatmul_ref(x, wq, s, b, bits, group)
        ts.append(time.perf_counter() - t0)
    us_cpu = statistics.median(ts) * 1e6
    return {"workload": "x fp32 [1,4096], W [4096,4096] 4-bit g64 fp32 scales/biases, y fp32", "algorithmic_bytes": nbytes,
            "gpu": {"kernel": kern, "us_per_call": us_gpu, "GBps": nbytes / us_gpu / 1e3, "max_rel_err": err_gpu,
                    "note": "weights L2-resident (8 MB): the same layer is launched back to back"},
            "cpu": {"us_per_call": us_cpu, "GBps": nbytes / us_cpu / 1e3, "cores": O.num_threads(), "max_rel_err": err_cpu,
                    "how": "oracle port in the reference CPU backend's loop style (src/cpu_backend.cpp:243-266), OpenMP over outputs, "
                           "median of 10 after 3 warm-up calls"},
            "tolerance": O.TOL[O.F32]}


def prefill_legs(ctx, O, BF16, peaks, only=None):
    """Tensor-bound legs (the prefill and the 8-bit large-GEMM configurations at one GPU): TFLOP/s = 2*M*N*K / device time.
    Rotating input sets keep every launch's operands colder than L2 capacity in total."""
    out = {}
    for name, (M, K, N, bits, group, R, iters) in {
        "prefill_4bit_M2048_K4096_N4096": (2048, 4096, 4096, 4, 64, 4, 10),
        "gemm_8bit_M512_K8192_N28672": (512, 8192, 28672, 8, 128, 2, 5),
        # the slice of the 8-bit configuration that one rank computes at 8 GPUs: 56 tiles on 148 SMs, the shape
        # the stream-K schedule is for
        "gemm_8bit_slice_M512_K8192_N3584": (512, 8192, 3584, 8, 128, 8, 5),
    }.items():
        if only and name != only:
            continue
        sets = []
        for r in range(R):
            wq, s, b = O.make_layer(N, K, bits, group, O.BF16, config_id=3 if bits == 4 else 4, layer=r)
            x = O.make_x(M, K, O.BF16, config_id=3 if bits == 4 else 4, layer=r)
            sets.append((ctx.upload(x), ctx.upload(wq), ctx.upload(s), ctx.upload(b), ctx.empty((M, N), np.uint16)))

        def go():
            for (bx, bw, bs, bb, by) in sets:
                ctx.qmatmul(bx, bw, bs, bb, by, M, K, N, bits, group, BF16, BF16, BF16)
        for _ in range(3):
            go()
        ctx.sync()
        ctx.timer_record(6)
        for _ in range(iters):
            go()
        ctx.timer_record(7)
        ms = ctx.timer_elapsed_ms(6, 7) / (iters * R)
        tf = 2.0 * M * N * K / ms / 1e9
        out[name] = {"us_per_launch": ms * 1e3, "TFLOPS": tf, "kernel": ctx.last_kernel(),
                     "roofline": {"bound": "tensor", "achieved": tf, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                                  "frac": tf / peaks["bf16_tflops"], "frac_of_sustained": tf / peaks["bf16_tflops_sustained"],
                                  "frac_of_nominal_2250": tf / 2250.0},
                     "input_bytes_rotated": R * (M * K * 2 + N * K * bits // 8 + 4 * N * K // group + M * N * 2)}
        for t in sets:
            for h in t:
                h.free()
    return out


def chain_leg(ctx, O, BF16, peaks):
    """The quantized-linear chain configuration at one GPU: one decode step (M = 8) through 32 layers of quantized
    projections (q,k,v,o 4096x4096; gate,up 11008x4096; down 4096x11008; 4-bit g64) with the full dataflow between them:
    a = bf16(q + k + v); o = Wo a; r = rms_norm(o); m = rms_norm(bf16(gate(r) * up(r))); d = Wd m; h' = rms_norm(d).
    q/k/v run as one N = 12288 launch and gate/up as one N = 22016 launch (the configuration allows it: same
    results), so a layer is 4 matmul launches + 4 small row kernels (sum3, rms-norm, mul+rms-norm, rms-norm), each
    ordered behind, and dependent on, the one before.  Four distinct layers' weights (455 MB, more than L2) are cycled
    eight times: a layer's weights were last read three layers earlier."""
    M, D, FF, L, DISTINCT = 8, 4096, 11008, 32, 4
    shapes = [("qkv", 3 * D, D), ("o", D, D), ("gateup", 2 * FF, D), ("down", D, FF)]
    layers = []
    for l in range(DISTINCT):
        ws = {}
        for pi, (name, N, K) in enumerate(shapes):
            wq, s, b = O.make_layer(N, K, BITS, GROUP, O.BF16, config_id=5, layer=l, proj=pi)
            ws[name] = (ctx.upload(wq), ctx.upload(s), ctx.upload(b), N, K)
        layers.append(ws)
    h = ctx.upload(O.make_x(M, D, O.BF16, config_id=5))
    t = {n: ctx.empty((M, N), np.uint16) for n, N in (("qkv", 3 * D), ("a", D), ("o", D), ("r", D), ("gateup", 2 * FF), ("m", FF), ("d", D))}

    def mm(ws, name, src, dst):
        bw, bs, bb, N, K = ws[name]
        ctx.qmatmul(src, bw, bs, bb, dst, M, K, N, BITS, GROUP, BF16, BF16, BF16)

    def step_separate():
        for l in range(L):
            ws = layers[l % DISTINCT]
            mm(ws, "qkv", h, t["qkv"])
            ctx.sum3(t["qkv"], t["a"], M, D, 3 * D)
            mm(ws, "o", t["a"], t["o"])
            ctx.rms_norm(t["o"], t["r"], M, D, 1e-6, BF16, BF16)
            mm(ws, "gateup", t["r"], t["gateup"])
            ctx.mul_rms_norm(t["gateup"], t["m"], M, FF, 2 * FF, 1e-6)
            mm(ws, "down", t["m"], t["d"])
            ctx.rms_norm(t["d"], h, M, D, 1e-6, BF16, BF16)

    from mlx_b200.plugin import PRO_RMS_NORM, PRO_SUM3

    def pro(ws, name, src, dst, which, ld):
        bw, bs, bb, N, K = ws[name]
        ctx.qmatmul_pro(src, bw, bs, bb, dst, M, K, N, BITS, GROUP, BF16, which, ld, 1e-6)

    def step_fused():
        # the same dataflow with sum3 and the two rms-norms whose row is 4096 long applied by the consuming decode
        # launch as it loads x: 5 launches per layer, and one rms-norm for the step's output
        for l in range(L):
            ws = layers[l % DISTINCT]
            if l == 0:
                mm(ws, "qkv", h, t["qkv"])
            else:
                pro(ws, "qkv", t["d"], t["qkv"], PRO_RMS_NORM, D)
            pro(ws, "o", t["qkv"], t["o"], PRO_SUM3, 3 * D)
            pro(ws, "gateup", t["o"], t["gateup"], PRO_RMS_NORM, D)
            ctx.mul_rms_norm(t["gateup"], t["m"], M, FF, 2 * FF, 1e-6)
            mm(ws, "down", t["m"], t["d"])
        ctx.rms_norm(t["d"], h, M, D, 1e-6, BF16, BF16)

    def timed(step):
        step()
        ctx.sync()
        ctx.graph_begin()
        step()
        g = ctx.graph_end()
        for _ in range(3):
            ctx.graph_launch(g)
        ctx.sync()
        iters = 10
        ctx.timer_record(8)
        for _ in range(iters):
            ctx.graph_launch(g)
        ctx.timer_record(9)
        ms = ctx.timer_elapsed_ms(8, 9) / iters
        ctx.graph_destroy(g)
        return ms

    # one step each way from the same input: the step's output must agree (the fused rms-norm sums a row's squares
    # in another order, so not bit for bit: the bar of the parity tests, 1e-2 of the largest output)
    h0 = h.to_host((M, D), np.uint16)
    step_separate()
    out_sep = O.from_bf16(h.to_host((M, D), np.uint16)).astype(np.float64)
    h.from_host(h0)
    step_fused()
    out_fus = O.from_bf16(h.to_host((M, D), np.uint16)).astype(np.float64)
    h.from_host(h0)
    dev = float(np.abs(out_fus - out_sep).max() / np.abs(out_sep).max())
    verified = (f"output of a 32-layer step, fused against separate launches: max deviation {dev:.2e} of the largest output"
                if np.isfinite(dev) and dev <= 1e-2 else f"FAILED: fused step deviates by {dev:.2e}")
    ms_sep = timed(step_separate)
    h.from_host(h0)
    ms = timed(step_fused)
    nbytes = L * sum(alg_bytes(M, K, N) for _, N, K in shapes)
    gbs = nbytes / ms / 1e6
    for ws in layers:
        for (bw, bs, bb, _, _) in ws.values():
            bw.free(); bs.free(); bb.free()
    for b in list(t.values()) + [h]:
        b.free()
    return {"workload": "32 layers x (qkv, o, gate/up, mul+rms-norm, down) + one rms-norm, M=8, one GPU: the dataflow "
                        "qkv, sum3, o, rms-norm, gate/up, mul+rms-norm, down, rms-norm with sum3 and the 4096-wide rms-norms "
                        "applied by the consuming decode launch as it loads x; every launch consumes the previous one's "
                        "output, one CUDA graph per step",
            "ms_per_step": ms, "launches_per_step": L * 5 + 1, "algorithmic_GB": nbytes / 1e9, "GBps": gbs,
            "separate_launches": {"ms_per_step": ms_sep, "launches_per_step": L * 8, "GBps": nbytes / ms_sep / 1e6},
            "verified": verified,
            "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": gbs / peaks["hbm_gbs"]}}


def gemm_sharded_leg(ctx, plugin, dist, rank, world, O, BF16, peaks, use_push):
    """The 8-bit large-GEMM configuration (M=512, K=8192, N=28672, g128) with N column-sharded over the ranks
    (strong scaling): every rank runs the tcgen05 GEMM on its 28672/world columns.  use_push: the GEMM's epilogue
    stores every tile into all ranks' copies of y (peer stores, two device-side rank barriers around the launch);
    else the slices are all-gathered with NCCL and interleaved.  Launched eagerly.  Rank 0 checks sampled
    outputs of the gathered y against the oracle."""
    import torch
    M, K, N, bits, group = 512, 8192, 28672, 8, 128
    nl = N // world
    q = plugin.quant
    comm, symm_y = None, None
    if use_push:
        from mlx_b200.plugin import SymmBuffer
        symm_y = SymmBuffer(ctx, rank, world, (M, N), np.uint16)
        mine = torch.tensor(list(symm_y.export()), dtype=torch.uint8, device="cuda")
        every = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(every, mine)
        symm_y.attach([bytes(t.cpu().tolist()) for t in every])
        dist.barrier()
    else:
        uid = (C.c_ubyte * 128)()
        if rank == 0:
            plugin.check(q.shard_unique_id(uid), "shard_unique_id")
        t = torch.tensor(list(uid), dtype=torch.uint8, device="cuda")
        dist.broadcast(t, 0)
        uid = (C.c_ubyte * 128)(*t.cpu().tolist())
        comm = C.c_void_p(None)
        plugin.check(q.shard_comm_create(ctx.handle, rank, world, uid, C.byref(comm)), "shard_comm_create")
    wq, s, b = O.make_layer(N, K, bits, group, O.BF16, config_id=4, layer=0)
    x = O.make_x(M, K, O.BF16, config_id=4, layer=0)
    sl = slice(rank * nl, (rank + 1) * nl)
    R = 2  # two copies of the slice, alternated: 2 x 235/world MB of weights
    sets = [(ctx.upload(wq[sl]), ctx.upload(s[sl]), ctx.upload(b[sl])) for _ in range(R)]
    bx = ctx.upload(x)
    y = symm_y.buffer if use_push else ctx.empty((M, N), np.uint16)
    staging = None if use_push else ctx.empty((world, M, nl), np.uint16)

    def go():
        for (bw, bs, bb) in sets:
            if use_push:
                symm_y.qmatmul(bx, bw, bs, bb, M, K, nl, bits, group, BF16)
            else:
                plugin.check(q.qmatmul_sharded(comm, bx.handle, bw.handle, bs.handle, bb.handle, y.handle, staging.handle,
                                               M, K, nl, bits, group, BF16, BF16, BF16), "qmatmul_sharded")
    go()
    ctx.sync()
    dist.barrier()
    verified = None
    if rank == 0:
        got = y.to_host()
        rows = [0, 257, 511]
        cols = np.arange(0, N, 97)
        truth = O.qmatmul_truth(x[rows], wq[cols], s[cols], b[cols], bits, group)
        err, _ = O.rel_err(got[np.ix_(rows, cols)], truth)
        verified = (f"sampled outputs of the gathered y within {O.TOL[O.BF16]} of the oracle (max rel err {err:.2e})"
                    if err <= O.TOL[O.BF16] else f"FAILED: sampled outputs off by {err:.3e}")
    dist.barrier()
    for _ in range(2):
        go()
    ctx.sync()
    dist.barrier()
    iters = 5
    ctx.timer_record(10)
    for _ in range(iters):
        go()
    ctx.timer_record(11)
    ms = ctx.timer_elapsed_ms(10, 11) / (iters * R)
    tt = torch.tensor([ms], dtype=torch.float64, device="cuda")
    dist.all_reduce(tt, op=dist.ReduceOp.MAX)
    ms = float(tt.item())
    ctx.sync()
    dist.barrier()
    if comm:
        q.shard_comm_destroy(comm)
    for tpl in sets:
        for h in tpl:
            h.free()
    bx.free()
    if use_push:
        symm_y.free()
    else:
        y.free()
        staging.free()
    tf = 2.0 * M * N * K / ms / 1e9
    how = "tiles stored into every rank's y from the GEMM epilogue" if use_push else "NCCL all-gather + interleave"
    # the same layer unsharded on one GPU (rank 0, the other ranks wait): T1 of the efficiency T1 / (G * T_G)
    t1 = None
    if rank == 0:
        t1 = prefill_legs(ctx, O, BF16, peaks, only="gemm_8bit_M512_K8192_N28672")["gemm_8bit_M512_K8192_N28672"]["us_per_launch"]
    dist.barrier()
    return {"workload": f"M=512 K=8192 N=28672 8-bit g128, N column-sharded over {world} GPUs, {how}",
            "scaling": "strong", "us_per_call": ms * 1e3, "TFLOPS_aggregate": tf, "us_per_call_one_gpu": t1,
            "efficiency": (t1 / (world * ms * 1e3)) if t1 else None,
            "allgather_bytes_per_rank": M * N * 2, "verified": verified}


def chain_sharded_leg(ctx, plugin, dist, rank, world, O, BF16, peaks):
    """The quantized-linear chain with every projection column-sharded over the ranks (strong scaling: the
    model is fixed, each rank keeps 1/world of every weight matrix) and the decode kernel delivering its
    columns to all ranks.  Same launches as chain_leg; x of every launch is the whole (gathered) activation.
    Before timing, rank 0 recomputes each of the four projections of one layer unsharded and compares the
    gathered outputs bit for bit."""
    import torch
    from mlx_b200.plugin import SymmBuffer
    M, D, FF, L, DISTINCT = 8, 4096, 11008, 32, 4
    shapes = [("qkv", 3 * D, D), ("o", D, D), ("gateup", 2 * FF, D), ("down", D, FF)]
    layers, full0 = [], {}
    for l in range(DISTINCT):
        ws = {}
        for pi, (name, N, K) in enumerate(shapes):
            wq, s, b = O.make_layer(N, K, BITS, GROUP, O.BF16, config_id=5, layer=l, proj=pi)
            nl = N // world
            sl = slice(rank * nl, (rank + 1) * nl)
            ws[name] = (ctx.upload(wq[sl]), ctx.upload(s[sl]), ctx.upload(b[sl]), nl, K)
            if l == 0 and rank == 0:
                full0[name] = (wq, s, b)
        layers.append(ws)
    symm = {}
    for name, N, _ in shapes:
        symm[name] = SymmBuffer(ctx, rank, world, (M, N), np.uint16)
        mine = torch.tensor(list(symm[name].export()), dtype=torch.uint8, device="cuda")
        every = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(every, mine)
        symm[name].attach([bytes(t.cpu().tolist()) for t in every])
    dist.barrier()
    h0 = O.make_x(M, D, O.BF16, config_id=5)
    h = ctx.upload(h0)
    a = ctx.empty((M, D), np.uint16)
    r_buf, m_buf = ctx.empty((M, D), np.uint16), ctx.empty((M, FF), np.uint16)

    def mm(ws, name, src):
        bw, bs, bb, nl, K = ws[name]
        symm[name].qmatmul(src, bw, bs, bb, M, K, nl, BITS, GROUP, BF16)

    from mlx_b200.plugin import PRO_RMS_NORM, PRO_SUM3

    def pro(ws, name, src, which, ld):
        bw, bs, bb, nl, K = ws[name]
        symm[name].qmatmul_pro(src, bw, bs, bb, M, K, nl, BITS, GROUP, BF16, which, ld, 1e-6)

    def layer_fused(ws, first):
        # chain_leg's fused dataflow: sum3 and the 4096-wide rms-norms applied by the consuming (sharded) decode launch
        # to the gathered activations as it loads them: 5 launches per layer
        if first:
            mm(ws, "qkv", h)
        else:
            pro(ws, "qkv", symm["down"].buffer, PRO_RMS_NORM, D)
        pro(ws, "o", symm["qkv"].buffer, PRO_SUM3, 3 * D)
        pro(ws, "gateup", symm["o"].buffer, PRO_RMS_NORM, D)
        ctx.mul_rms_norm(symm["gateup"].buffer, m_buf, M, FF, 2 * FF, 1e-6)
        mm(ws, "down", m_buf)

    def layer(ws):  # the dataflow of chain_leg; the elementwise steps run on every rank on the gathered rows
        mm(ws, "qkv", h)
        ctx.sum3(symm["qkv"].buffer, a, M, D, 3 * D)
        mm(ws, "o", a)
        ctx.rms_norm(symm["o"].buffer, r_buf, M, D, 1e-6, BF16, BF16)
        mm(ws, "gateup", r_buf)
        ctx.mul_rms_norm(symm["gateup"].buffer, m_buf, M, FF, 2 * FF, 1e-6)
        mm(ws, "down", m_buf)
        ctx.rms_norm(symm["down"].buffer, h, M, D, 1e-6, BF16, BF16)

    # check: one layer, gathered outputs against the unsharded matmuls on rank 0
    layer(layers[0])
    ctx.sync()
    dist.barrier()
    verified = None
    if rank == 0:
        inputs = {"qkv": h0, "o": a.to_host(), "gateup": r_buf.to_host(), "down": m_buf.to_host()}
        for name, N, K in shapes:
            wq, s, b = full0[name]
            bw, bs, bb, bx = ctx.upload(wq), ctx.upload(s), ctx.upload(b), ctx.upload(inputs[name])
            ref = ctx.empty((M, N), np.uint16)
            ctx.qmatmul(bx, bw, bs, bb, ref, M, K, N, BITS, GROUP, BF16, BF16, BF16)
            if not np.array_equal(symm[name].to_host(), ref.to_host()):
                verified = f"FAILED: sharded {name} differs from the unsharded matmul"
            for t in (bw, bs, bb, bx, ref):
                t.free()
        verified = verified or "gathered qkv / o / gate-up / down outputs of one layer bit-identical to the unsharded matmuls"
    dist.barrier()

    def step_separate():
        for l in range(L):
            layer(layers[l % DISTINCT])

    def step():
        for l in range(L):
            layer_fused(layers[l % DISTINCT], l == 0)
        ctx.rms_norm(symm["down"].buffer, h, M, D, 1e-6, BF16, BF16)

    # the two ways from the same input: the step's output must agree within the bar of the parity tests (the fused
    # rms-norm sums a row's squares in another order)
    h.from_host(h0)
    step_separate()
    out_sep = O.from_bf16(h.to_host((M, D), np.uint16)).astype(np.float64)
    h.from_host(h0)
    step()
    out_fus = O.from_bf16(h.to_host((M, D), np.uint16)).astype(np.float64)
    h.from_host(h0)
    dev = float(np.abs(out_fus - out_sep).max() / np.abs(out_sep).max())
    fused_ok = np.isfinite(dev) and dev <= 1e-2
    if rank == 0:
        verified += (f"; a 32-layer step with the prologues against separate launches: max deviation {dev:.2e} of the largest output"
                     if fused_ok else f"; FAILED: the step with prologues deviates by {dev:.2e}")
    dist.barrier()

    def timed_step(fn):
        fn()
        ctx.sync()
        dist.barrier()
        ctx.graph_begin()
        fn()
        g = ctx.graph_end()
        for _ in range(3):
            ctx.graph_launch(g)
        ctx.sync()
        dist.barrier()
        iters = 10
        ctx.timer_record(8)
        for _ in range(iters):
            ctx.graph_launch(g)
        ctx.timer_record(9)
        ms = ctx.timer_elapsed_ms(8, 9) / iters
        t = torch.tensor([ms], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ctx.sync()
        dist.barrier()
        ctx.graph_destroy(g)
        return float(t.item())

    ms_sep = timed_step(step_separate)
    h.from_host(h0)
    ms = timed_step(step)
    nbytes = L * sum(alg_bytes(M, K, N) for _, N, K in shapes)
    for sb in symm.values():
        sb.free()
    for ws in layers:
        for (bw, bs, bb, _, _) in ws.values():
            bw.free(); bs.free(); bb.free()
    for b in (h, a, r_buf, m_buf):
        b.free()
    # the same chain on one GPU (rank 0, the other ranks wait): T1 of the efficiency T1 / (G * T_G)
    t1 = None
    if rank == 0:
        t1 = chain_leg(ctx, O, BF16, peaks)["ms_per_step"]
    dist.barrier()
    return {"workload": f"32 layers x (qkv, sum3, o, rms-norm, gate/up, mul+rms-norm, down, rms-norm), M=8, every projection "
                        f"column-sharded over {world} GPUs, full dataflow; sum3 and the 4096-wide rms-norms applied by the consuming "
                        "sharded decode launch as it loads the gathered x (5 launches per layer, as on one GPU)",
            "scaling": "strong", "ms_per_step": ms, "launches_per_step": L * 5 + 1, "algorithmic_GB": nbytes / 1e9,
            "separate_launches": {"ms_per_step": ms_sep, "launches_per_step": L * 8},
            "GBps_aggregate": nbytes / ms / 1e6, "ms_per_step_one_gpu": t1,
            "efficiency": (t1 / (world * ms)) if t1 else None, "verified": verified}


# ---------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------
def run_ours(args, rank, world):
    import mlx_b200
    from mlx_b200 import BF16
    import oracle as O  # input generation + CPU baseline only

    local_rank = int(os.environ.get("LOCAL_RANK", rank))
    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    plugin = mlx_b200.Plugin(require_gpu=True)
    ctx = plugin.context(local_rank)
    q = plugin.quant
    if args.prefill_only:
        peaks, _ = measured_peaks()
        print(json.dumps({"prefill": prefill_legs(ctx, O, BF16, peaks)}))
        return
    if args.chain_only:
        peaks, _ = measured_peaks()
        print(json.dumps({"chain": chain_leg(ctx, O, BF16, peaks)}))
        return

    # resident inputs: R weight sets (each rank: its own column slice), x per M
    layers = []
    for r in range(R_SETS):
        wq, s, b = O.make_layer(N_DEC, K_DEC, BITS, GROUP, O.BF16, config_id=2, layer=r, proj=rank)
        layers.append((ctx.upload(wq), ctx.upload(s), ctx.upload(b)))
    x_host = {M: O.make_x(M, K_DEC, O.BF16, config_id=2, tag=M) for M in M_SWEEP}
    x_dev = {M: ctx.upload(x_host[M]) for M in M_SWEEP}
    n_total = N_DEC * world
    comm, staging, symm = None, {}, {}
    use_push = world > 1 and not args.nccl_allgather
    if use_push:
        # the all-gather is done by the decode kernel itself: every rank's y_full is a buffer its peers store into
        import torch
        for M in M_SWEEP:
            symm[M] = mlx_b200.plugin.SymmBuffer(ctx, rank, world, (M, n_total), np.uint16)
            mine = torch.tensor(list(symm[M].export()), dtype=torch.uint8, device="cuda")
            every = [torch.empty_like(mine) for _ in range(world)]
            dist.all_gather(every, mine)
            symm[M].attach([bytes(t.cpu().tolist()) for t in every])
        y_dev = {M: symm[M].buffer for M in M_SWEEP}
        dist.barrier()
    else:
        y_dev = {M: ctx.empty((M, n_total), np.uint16) for M in M_SWEEP}
    if world > 1 and not use_push:
        import torch
        uid = (C.c_ubyte * 128)()
        if rank == 0:
            plugin.check(q.shard_unique_id(uid), "shard_unique_id")
        t = torch.tensor(list(uid), dtype=torch.uint8, device="cuda")
        dist.broadcast(t, 0)
        uid = (C.c_ubyte * 128)(*t.cpu().tolist())
        comm = C.c_void_p(None)
        plugin.check(q.shard_comm_create(ctx.handle, rank, world, uid, C.byref(comm)), "shard_comm_create")
        staging = {M: ctx.empty((world, M, N_DEC), np.uint16) for M in M_SWEEP}

    def launch(M, r):
        w, s, b = layers[r]
        if world == 1:
            ctx.qmatmul(x_dev[M], w, s, b, y_dev[M], M, K_DEC, N_DEC, BITS, GROUP, BF16, BF16, BF16)
        elif use_push:
            symm[M].qmatmul(x_dev[M], w, s, b, M, K_DEC, N_DEC, BITS, GROUP, BF16)
        else:
            plugin.check(q.qmatmul_sharded(comm, x_dev[M].handle, w.handle, s.handle, b.handle, y_dev[M].handle,
                                           staging[M].handle, M, K_DEC, N_DEC, BITS, GROUP, BF16, BF16, BF16),
                         "qmatmul_sharded")

    # eager pass: creates workspaces, checks one result against the oracle
    for M in M_SWEEP:
        launch(M, 0)
    ctx.sync()
    if rank == 0:
        y = y_dev[4].to_host()[:, :N_DEC]
        wq0, s0, b0 = O.make_layer(N_DEC, K_DEC, BITS, GROUP, O.BF16, config_id=2, layer=0, proj=0)
        err, _ = O.rel_err(y, O.qmatmul_truth(x_host[4], wq0, s0, b0, BITS, GROUP))
        assert err <= O.TOL[O.BF16], f"parity check failed before timing: {err}"
    verified = None
    if world > 1:
        # every rank's columns, as they arrived on rank 0, against the same slice computed here on one GPU
        if dist is not None:
            ctx.sync()
            dist.barrier()
        if rank == 0:
            for M in (4, 16):
                got = y_dev[M].to_host((M, n_total), np.uint16)
                for r in range(world):
                    wq_r, s_r, b_r = O.make_layer(N_DEC, K_DEC, BITS, GROUP, O.BF16, config_id=2, layer=0, proj=r)
                    bw, bs, bb = ctx.upload(wq_r), ctx.upload(s_r), ctx.upload(b_r)
                    ref = ctx.empty((M, N_DEC), np.uint16)
                    ctx.qmatmul(x_dev[M], bw, bs, bb, ref, M, K_DEC, N_DEC, BITS, GROUP, BF16, BF16, BF16)
                    want = ref.to_host()
                    if not np.array_equal(got[:, r * N_DEC:(r + 1) * N_DEC], want):  # recorded, not raised: the
                        verified = f"FAILED: columns of rank {r} differ (M={M})"       # other ranks wait in a barrier
                        print(verified, file=sys.stderr, flush=True)
                    for h in (bw, bs, bb, ref):
                        h.free()
            verified = verified or "all ranks' columns on rank 0 bit-identical to the single-GPU kernel (M=4, 16)"
        dist.barrier()

    # one sweep = len(M_SWEEP) * R launches, recorded once as a CUDA graph per M
    l0 = ctx.launch_count()
    graphs = {}
    # one process per GPU: the NCCL all-gathers are launched eagerly (a capture of them hung a 2-rank run)
    use_graph = (world == 1 or use_push) and not args.no_graph
    if use_graph:
        for M in M_SWEEP:
            ctx.graph_begin()
            for r in range(R_SETS):
                launch(M, r)
            graphs[M] = ctx.graph_end()
        # the timed step replays whole sweeps: SWEEPS_PER_GRAPH of them per graph (graph boundaries serialise
        # fully, so longer graphs mean fewer of them per launch)
        ctx.graph_begin()
        for _ in range(SWEEPS_PER_GRAPH):
            for M in M_SWEEP:
                for r in range(R_SETS):
                    launch(M, r)
        graph_sweeps = ctx.graph_end()

    # The matmuls of a sweep are independent, so the timed step hands each sweep to the plugin as ONE call
    # (qmatmul_batch, on several GPUs qmatmul_sharded_push_batch: a persistent launch for the items with M <= 8, one
    # for those with M = 16) instead of 48 calls.  Every item has its own output (on several GPUs: its own place in
    # one symmetric buffer, whole on every rank when the call ends); three of them are checked against the single
    # calls, bit for bit (on several GPUs: all ranks' columns, on every rank).
    use_batch = (world == 1 or use_push) and not args.single_calls
    batch_graph, batch_verified, symm_all = None, None, None
    if use_batch:
        b_items = [(M, r) for M in M_SWEEP for r in range(R_SETS)]
        if world == 1:
            b_y = {it: ctx.empty((it[0], N_DEC), np.uint16) for it in b_items}

            def batch_call(items):
                ctx.qmatmul_batch([x_dev[M] for M, r in items], [layers[r][0] for M, r in items], [layers[r][1] for M, r in items],
                                  [layers[r][2] for M, r in items], [b_y[it] for it in items], [M for M, r in items],
                                  K_DEC, N_DEC, BITS, GROUP, BF16)

            def item_host(it):
                return b_y[it].to_host()
        else:
            import torch
            from mlx_b200.shard import batch_layout
            offs, total_bytes_y = batch_layout([M for M, r in b_items], n_total)
            b_off = dict(zip(b_items, offs))
            symm_all = mlx_b200.plugin.SymmBuffer(ctx, rank, world, (total_bytes_y // 2,), np.uint16)
            mine = torch.tensor(list(symm_all.export()), dtype=torch.uint8, device="cuda")
            every = [torch.empty_like(mine) for _ in range(world)]
            dist.all_gather(every, mine)
            symm_all.attach([bytes(t.cpu().tolist()) for t in every])
            dist.barrier()

            def batch_call(items):
                symm_all.qmatmul_batch([x_dev[M] for M, r in items], [layers[r][0] for M, r in items], [layers[r][1] for M, r in items],
                                       [layers[r][2] for M, r in items], [b_off[it] for it in items], [M for M, r in items],
                                       K_DEC, N_DEC, BITS, GROUP, BF16)

            def item_host(it):
                return symm_all.item_to_host(b_off[it], (it[0], n_total), np.uint16)
        batch_call(b_items)
        batch_kernel = ctx.last_kernel()
        ctx.sync()
        bad = []
        for it in ((1, 0), (8, R_SETS - 1), (16, R_SETS // 2)):
            launch(*it)
            if not np.array_equal(item_host(it), y_dev[it[0]].to_host((it[0], n_total), np.uint16)):
                bad.append(it)
        if dist is not None:
            import torch
            t = torch.tensor([len(bad)], dtype=torch.int64, device="cuda")
            dist.all_reduce(t)
            if int(t.item()) and not bad:
                bad = ["(on another rank)"]
        batch_verified = (f"FAILED: items {bad} differ from single calls" if bad else
                          "items (M=1, set 0), (M=8, last set), (M=16, middle set) of a batched sweep bit-identical to single "
                          + ("qmatmul calls" if world == 1 else "sharded calls: every rank's columns, compared on every rank"))
        if bad:
            print(batch_verified, file=sys.stderr, flush=True)
        if use_graph:
            ctx.graph_begin()
            for _ in range(SWEEPS_PER_GRAPH):
                batch_call(b_items)
            batch_graph = ctx.graph_end()

    def sweep():
        if use_batch:
            batch_call(b_items)
            return
        for M in M_SWEEP:
            if use_graph:
                ctx.graph_launch(graphs[M])
            else:
                for r in range(R_SETS):
                    launch(M, r)

    def barrier():
        ctx.sync()
        if dist is not None:
            dist.barrier()
        ctx.sync()

    def timed(fn, slot0=0, slot1=1):
        barrier()
        ctx.timer_record(slot0)
        fn()
        ctx.timer_record(slot1)
        ms = ctx.timer_elapsed_ms(slot0, slot1)
        barrier()
        if dist is not None:
            import torch
            t = torch.tensor([ms], dtype=torch.float64, device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    def step():
        done = 0
        while use_graph and done + SWEEPS_PER_GRAPH <= args.reps:
            ctx.graph_launch(batch_graph if use_batch else graph_sweeps)
            done += SWEEPS_PER_GRAPH
        for _ in range(args.reps - done):
            sweep()

    for _ in range(args.warmup):
        step()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    lc0 = ctx.launch_count()
    ms_total = timed(lambda: [step() for _ in range(args.steps)])
    launches = ctx.launch_count() - lc0
    clocks = sampler.stop() if rank == 0 else None

    # the same sweeps as single calls (one launch per matmul, 48 per sweep), for comparison
    single = None
    if use_batch:
        def step_single():
            done = 0
            while use_graph and done + SWEEPS_PER_GRAPH <= args.reps:
                ctx.graph_launch(graph_sweeps)
                done += SWEEPS_PER_GRAPH
            for _ in range(args.reps - done):
                for M in M_SWEEP:
                    for r in range(R_SETS):
                        launch(M, r)
        n_s = max(1, min(args.steps, 5))
        step_single()
        ms_s = timed(lambda: [step_single() for _ in range(n_s)], 10, 11)
        single = {"GBps": sum(alg_bytes(M) for M in M_SWEEP) * R_SETS * args.reps * n_s / ms_s / 1e6, "steps": n_s,
                  "us_per_matmul": ms_s * 1e3 / (len(M_SWEEP) * R_SETS * args.reps * n_s),
                  "how": "one qmatmul call (one launch) per matmul, the same sweeps replayed from CUDA graphs"}
        single["frac_of_peak"] = single["GBps"] / float(measured_peaks()[0]["hbm_gbs"])

    # per-M timing (same graphs, one M at a time) for the roofline of the dominant kernel
    per_m = {}
    reps_m = max(10, args.reps)
    for M in M_SWEEP:
        def run_m(M=M):
            for _ in range(reps_m):
                if use_graph:
                    ctx.graph_launch(graphs[M])
                else:
                    for r in range(R_SETS):
                        launch(M, r)
        launch(M, 0)  # (eagerly once: a graph replay does not update the context's "last kernel")
        kernel_name = ctx.last_kernel()
        run_m()
        ms = timed(run_m, 2, 3)
        n_launch = reps_m * R_SETS
        per_m[M] = {"us_per_launch": ms * 1e3 / n_launch, "GBps": alg_bytes(M) * world * n_launch / ms / 1e6,
                    "kernel": kernel_name}

    per_m_batched = None
    if use_batch:
        per_m_batched = {}
        for M in M_SWEEP:
            its = [it for it in b_items if it[0] == M]
            def run_b(its=its):
                for _ in range(reps_m):
                    batch_call(its)
            run_b()
            ms = timed(run_b, 2, 3)
            per_m_batched[str(M)] = {"us_per_matmul": ms * 1e3 / (reps_m * len(its)), "GBps": alg_bytes(M) * world * reps_m * len(its) / ms / 1e6,
                                     "kernel": batch_kernel if M > 8 else batch_kernel.replace("m16", "m8")}
    sweep_bytes = sum(alg_bytes(M) for M in M_SWEEP) * R_SETS * world
    total_bytes = sweep_bytes * args.reps * args.steps
    value = total_bytes / ms_total / 1e6  # GB/s
    n_launches_alg = len(M_SWEEP) * R_SETS * args.reps * args.steps

    # e2e: host buffers in, host buffers out, through the base vtable copies (blocking, reference semantics)
    e2e_calls = 0
    e2e_steps = max(1, min(args.steps, 5))
    e2e_reps = max(1, args.reps)  # an end-to-end step is a step of the timed region above: the same sweeps
    # page-locked host buffers on both sides, as a serving host keeps them
    x_pin, y_pin = {}, {}
    for M in M_SWEEP:
        x_pin[M] = ctx.pinned_array(x_host[M].shape, x_host[M].dtype)
        x_pin[M][...] = x_host[M]
        y_pin[M] = ctx.pinned_array((M, n_total), np.uint16)
    xp = {M: (C.c_void_p(x_pin[M].ctypes.data), x_pin[M].nbytes) for M in M_SWEEP}
    yp = {M: (C.c_void_p(y_pin[M].ctypes.data), y_pin[M].nbytes) for M in M_SWEEP}

    # The loop over the calls runs in C (bench_e2e.c), as a host of the plugin would run it: per call the plugin's
    # own buffer_copy_from_host_async, qmatmul (or qmatmul_sharded_push) and blocking buffer_copy_to_host, taken as
    # function pointers from the tables the plugin publishes.  (The same loop in Python, which --e2e-python runs
    # instead, costs about 2 us of interpreter and ctypes time per call on top.)
    e2e_native = None
    if not args.e2e_python and world > 1 and not use_push:
        args.e2e_python = True  # (the NCCL fallback takes a staging buffer and a communicator: not wired into the C loop)
    if not args.e2e_python:
        drv = C.CDLL(e2e_driver_path())

        class Call(C.Structure):
            _fields_ = [("x_dev", C.c_void_p), ("wq", C.c_void_p), ("scales", C.c_void_p), ("biases", C.c_void_p),
                        ("y_dev", C.c_void_p), ("y_symm", C.c_void_p), ("x_host", C.c_void_p), ("y_host", C.c_void_p),
                        ("x_bytes", C.c_size_t), ("y_bytes", C.c_size_t), ("M", C.c_int32), ("K", C.c_int32), ("N", C.c_int32),
                        ("bits", C.c_int32), ("group", C.c_int32), ("dtype", C.c_int32)]

        def _h(obj):  # a handle as an integer
            v = obj.handle if hasattr(obj, "handle") else obj
            return v.value if isinstance(v, C.c_void_p) else C.cast(v, C.c_void_p).value

        order = [(M, r) for M in M_SWEEP for r in range(R_SETS)]
        calls = (Call * len(order))()
        for i, (M, r) in enumerate(order):
            w, s_, b_ = layers[r]
            calls[i] = Call(_h(x_dev[M]), _h(w), _h(s_), _h(b_), _h(y_dev[M]), _h(symm[M]) if use_push else None,
                            xp[M][0].value, yp[M][0].value, xp[M][1], yp[M][1], M, K_DEC, N_DEC, BITS, GROUP, BF16)
        fn = lambda f: C.cast(f, C.c_void_p)
        drv.lux_bench_e2e.restype = C.c_int
        drv.lux_bench_e2e.argtypes = [C.c_void_p] * 5 + [C.POINTER(Call), C.c_int, C.c_int, C.POINTER(C.c_longlong)]
        e2e_native = (drv, calls, len(order), fn(q.buffer_copy_from_host_async), fn(q.qmatmul), fn(q.qmatmul_sharded_push),
                      fn(plugin.vtbl.buffer_copy_to_host))

    # The batched sweep end to end: every item's activations in one device buffer and one pinned host buffer (the
    # items' x are views into it), every item's output in one device buffer (several GPUs: the symmetric buffer), so
    # that a sweep is one host->device copy, one batched call and one blocking device->host copy of all outputs.
    e2e_batch = e2e_two = None
    if use_batch and e2e_native is not None:
        class Batch(C.Structure):
            _fields_ = [("x_all_dev", C.c_void_p), ("x_all_host", C.c_void_p), ("x_bytes", C.c_size_t),
                        ("y_all_dev", C.c_void_p), ("y_all_host", C.c_void_p), ("y_bytes", C.c_size_t), ("n", C.c_int32),
                        ("x", C.c_void_p), ("wq", C.c_void_p), ("scales", C.c_void_p), ("biases", C.c_void_p), ("y", C.c_void_p),
                        ("y_offset", C.c_void_p), ("M", C.c_void_p), ("y_symm", C.c_void_p),
                        ("K", C.c_int32), ("N", C.c_int32), ("bits", C.c_int32), ("group", C.c_int32), ("dtype", C.c_int32)]
        nb = len(b_items)
        from mlx_b200.shard import batch_layout, readback_share
        x_off, xo = batch_layout([M for M, r in b_items], K_DEC)
        y_off, yo = batch_layout([M for M, r in b_items], n_total)
        x_all = ctx.empty((xo // 2,), np.uint16)
        x_all_pin = ctx.pinned_array((xo // 2,), np.uint16)
        for (M, r), o in zip(b_items, x_off):
            x_all_pin[o // 2:o // 2 + M * K_DEC] = x_host[M].reshape(-1)
        y_all_pin = ctx.pinned_array((yo // 2,), np.uint16)
        x_base = x_all.device_ptr
        x_views = [ctx.wrap(x_base + o, M * K_DEC * 2) for (M, r), o in zip(b_items, x_off)]
        if world == 1:
            y_all = ctx.empty((yo // 2,), np.uint16)
            y_base = y_all.device_ptr
            y_views = [ctx.wrap(y_base + o, M * n_total * 2) for (M, r), o in zip(b_items, y_off)]
            y_all_handle, y_symm_handle = _h(y_all), None
        else:
            assert [b_off[it] for it in b_items] == y_off
            # every rank ends with all outputs whole; the hosts read them back ONCE between them: rank r its 1/world
            # share of the result buffer (a view into the symmetric buffer), not every rank everything
            y_all, y_views = None, []
            share_off, share_len = readback_share(rank, world, yo)
            share_view = ctx.wrap(symm_all.buffer.device_ptr + share_off, share_len)
            y_all_handle, y_symm_handle = _h(share_view), _h(symm_all)
        arr = lambda hs: (C.c_void_p * nb)(*hs)
        keep = {"x": arr([_h(v) for v in x_views]), "wq": arr([_h(layers[r][0]) for M, r in b_items]),
                "scales": arr([_h(layers[r][1]) for M, r in b_items]), "biases": arr([_h(layers[r][2]) for M, r in b_items]),
                "y": arr([_h(v) for v in y_views]) if y_views else None, "y_offset": (C.c_size_t * nb)(*y_off),
                "M": (C.c_int * nb)(*[M for M, r in b_items])}
        adr = lambda a: C.cast(a, C.c_void_p).value if a is not None else None
        bt = Batch(_h(x_all), x_all_pin.ctypes.data, xo, y_all_handle, y_all_pin.ctypes.data, yo if world == 1 else share_len, nb, adr(keep["x"]), adr(keep["wq"]),
                   adr(keep["scales"]), adr(keep["biases"]), adr(keep["y"]), adr(keep["y_offset"]), adr(keep["M"]), y_symm_handle,
                   K_DEC, N_DEC, BITS, GROUP, BF16)
        drv.lux_bench_e2e_batch.restype = C.c_int
        drv.lux_bench_e2e_batch.argtypes = [C.c_void_p] * 5 + [C.POINTER(Batch), C.c_int, C.POINTER(C.c_longlong)]
        e2e_batch = (bt, keep, x_views, y_views, x_all, y_all, x_all_pin, y_all_pin, fn(q.qmatmul_batch), fn(q.qmatmul_sharded_push_batch))
        if world == 1 and not args.e2e_one_context:
            # a second context (stream) with its own activations and outputs: sweep r computes while sweep r-1 is read back
            ctx2 = plugin.context(local_rank)
            x_all2, y_all2 = ctx2.empty((xo // 2,), np.uint16), ctx2.empty((yo // 2,), np.uint16)
            y_all_pin2 = ctx2.pinned_array((yo // 2,), np.uint16)
            x_views2 = [ctx2.wrap(x_all2.device_ptr + o, M * K_DEC * 2) for (M, r), o in zip(b_items, x_off)]
            y_views2 = [ctx2.wrap(y_all2.device_ptr + o, M * n_total * 2) for (M, r), o in zip(b_items, y_off)]
            keep2 = {"x": arr([_h(v) for v in x_views2]), "y": arr([_h(v) for v in y_views2])}
            bt2 = Batch(_h(x_all2), x_all_pin.ctypes.data, xo, _h(y_all2), y_all_pin2.ctypes.data, yo, nb, adr(keep2["x"]), adr(keep["wq"]),
                        adr(keep["scales"]), adr(keep["biases"]), adr(keep2["y"]), adr(keep["y_offset"]), adr(keep["M"]), None,
                        K_DEC, N_DEC, BITS, GROUP, BF16)
            drv.lux_bench_e2e_batch2.restype = C.c_int
            drv.lux_bench_e2e_batch2.argtypes = [C.c_void_p] * 3 + [C.POINTER(C.c_void_p), C.POINTER(C.POINTER(Batch)), C.c_int,
                                                                    C.POINTER(C.c_longlong)]
            e2e_two = (ctx2, bt2, keep2, x_views2, y_views2, x_all2, y_all2, y_all_pin2, (C.c_void_p * 2)(_h(ctx), _h(ctx2)),
                       (C.POINTER(Batch) * 2)(C.pointer(bt), C.pointer(bt2)))

    def e2e_batch_step(two=True):
        nonlocal e2e_calls
        bt = e2e_batch[0]
        done = C.c_longlong(0)
        if two and e2e_two is not None:
            rc = drv.lux_bench_e2e_batch2(e2e_native[3], e2e_batch[8], e2e_native[6], e2e_two[8], e2e_two[9], e2e_reps, C.byref(done))
            plugin.check(rc, "e2e batch loop (two contexts)")
            e2e_two[0].sync()
            e2e_calls += done.value
            return
        rc = drv.lux_bench_e2e_batch(e2e_native[3], e2e_batch[8], e2e_batch[9], e2e_native[6], ctx.handle, C.byref(bt), e2e_reps,
                                     C.byref(done))
        plugin.check(rc, "e2e batch loop")
        e2e_calls += done.value

    def e2e_step():
        nonlocal e2e_calls
        if e2e_native is not None:
            drv, calls, n, f_in, f_mm, f_push, f_out = e2e_native
            done = C.c_longlong(0)
            rc = drv.lux_bench_e2e(f_in, f_mm, f_push, f_out, ctx.handle, calls, n, e2e_reps, C.byref(done))
            plugin.check(rc, "e2e loop")
            e2e_calls += done.value
            return
        for _ in range(e2e_reps):
            for M in M_SWEEP:
                for r in range(R_SETS):
                    ctx.upload_async(x_dev[M], *xp[M])
                    launch(M, r)
                    y_dev[M].to_host_into(*yp[M])
                    e2e_calls += 1
    if args.kernel_only:
        e2e_steps = e2e_reps = 0
    e2e_step()
    e2e_calls = 0
    ms_e2e = timed(lambda: [e2e_step() for _ in range(e2e_steps)], 4, 5) if e2e_steps else float("nan")
    e2e_value = sweep_bytes * e2e_reps * e2e_steps / ms_e2e / 1e6
    e2e_single = None
    if e2e_batch is not None and e2e_steps:
        # the headline's own route end to end: keep the per-call figures beside it, then check what came back
        e2e_single = {"value": e2e_value, "unit": "GB/s", "calls": e2e_calls, "us_per_call": ms_e2e * 1e3 / max(1, e2e_calls),
                      "how": "one copy in, one qmatmul" + ("_sharded_push" if world > 1 else "") + ", one blocking copy out per matmul"}
        e2e_batch_step()
        bad = []
        if world == 1:
            for y_back in [e2e_batch[7]] + ([e2e_two[7]] if e2e_two is not None else []):
                for it in ((1, 0), (8, R_SETS - 1), (16, R_SETS // 2)):
                    i = b_items.index(it)
                    o, cnt = e2e_batch[1]["y_offset"][i] // 2, it[0] * n_total
                    if not np.array_equal(np.asarray(y_back[o:o + cnt]).reshape(it[0], n_total), item_host(it)):
                        bad.append(it)
            e2e_checked = f"FAILED: outputs {bad} read back differ" if bad else "three outputs as read back to the host bit-identical to the batched sweep's"
        else:
            # this rank's share as read back against the same bytes of its result buffer, and item (M=16, middle set) of that
            # buffer against the single sharded call (all ranks make the call)
            flat = symm_all.buffer.to_host((symm_all.buffer.nbytes,), np.uint8)
            if not np.array_equal(np.asarray(e2e_batch[7]).view(np.uint8)[:share_len], flat[share_off:share_off + share_len]):
                bad.append(f"share of rank {rank}")
            it = (16, R_SETS // 2)
            launch(*it)
            if not np.array_equal(item_host(it), y_dev[it[0]].to_host((it[0], n_total), np.uint16)):
                bad.append(it)
            import torch
            t = torch.tensor([len(bad)], dtype=torch.int64, device="cuda")
            dist.all_reduce(t)
            if int(t.item()) and not bad:
                bad = ["(on another rank)"]
            e2e_checked = (f"FAILED: {bad} read back differ" if bad else
                           "every rank's share as read back bit-identical to its result buffer, whose items are the single sharded calls'")
        if bad:
            print(e2e_checked, file=sys.stderr, flush=True)
        e2e_one = None
        if e2e_two is not None:
            e2e_batch_step(False)
            e2e_calls = 0
            ms_one = timed(lambda: [e2e_batch_step(False) for _ in range(e2e_steps)], 4, 5)
            e2e_one = {"value": sweep_bytes * e2e_reps * e2e_steps / ms_one / 1e6, "unit": "GB/s", "us_per_matmul": ms_one * 1e3 / max(1, e2e_calls),
                       "how": "the same with one context: copy in, batched call, blocking copy out, strictly one after the other"}
        e2e_calls = 0
        ms_e2e = timed(lambda: [e2e_batch_step() for _ in range(e2e_steps)], 4, 5)
        e2e_value = sweep_bytes * e2e_reps * e2e_steps / ms_e2e / 1e6
    h2d = sum(M * K_DEC * 2 for M in M_SWEEP) * R_SETS * e2e_reps * world  # summed over the ranks (x is replicated: every rank copies it in)
    d2h = sum(M * n_total * 2 for M in M_SWEEP) * R_SETS * e2e_reps

    peaks, which = measured_peaks()
    cpu_ref_config = cpu_reference_config_leg(ctx, O) if (world == 1 and not args.kernel_only) else None
    prefill = prefill_legs(ctx, O, BF16, peaks) if (world == 1 and not args.kernel_only) else None
    chain = chain_leg(ctx, O, BF16, peaks) if (world == 1 and not args.kernel_only) else None
    # the sharded configurations proper (strong scaling), after the sweep; a failure here must not lose the sweep
    gemm_sharded = chain_sharded = None
    if world > 1 and not args.kernel_only and not args.no_sharded_legs or world > 1 and args.gemm_sharded:
        try:
            gemm_sharded = gemm_sharded_leg(ctx, plugin, dist, rank, world, O, BF16, peaks, use_push)
        except Exception as e:  # the same on every rank (shapes, memory): nobody is left in a collective
            gemm_sharded = {"error": repr(e)[:300]}
    if world > 1 and use_push and (args.chain_sharded or (not args.kernel_only and not args.no_sharded_legs)):
        try:
            chain_sharded = chain_sharded_leg(ctx, plugin, dist, rank, world, O, BF16, peaks)
        except Exception as e:
            chain_sharded = {"error": repr(e)[:300]}
    if dist is not None:
        ctx.sync()
        dist.barrier()
        if comm:
            q.shard_comm_destroy(comm)
        for sb in symm.values():
            sb.free()
        if symm_all is not None:
            symm_all.free()
        dist.destroy_process_group()
    if rank != 0:
        return
    peak = float(peaks["hbm_gbs"])
    dom = max(M_SWEEP, key=lambda M: 1)  # all launches are the same kernel family; report the sweep average
    avg_us = ms_total * 1e3 / n_launches_alg
    achieved = value / world  # per-GPU GB/s of the kernel, averaged over the timed region
    cpu, _, _ = cpu_baseline() if (world == 1 and not args.kernel_only) else ({"value": None, "unit": "GB/s", "cores": None, "kind": "port",
                                                   "sample": "run at N=1 only"}, 0, 0)
    out = {
        "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_total / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": shared_config(),
        "run": {"layout": "one GPU" if world == 1 else f"weak scaling: each of {world} ranks holds its own {N_DEC}-column slice of a "
                          f"{n_total}-column layer and every rank ends with the whole y (all-gather of output slices)",
                   "N_total": n_total, "weight_sets": R_SETS, "sweeps_per_step": args.reps, "cuda_graph": use_graph,
                   "calls": (("one qmatmul_batch" if world == 1 else "one qmatmul_sharded_push_batch") + " call per sweep: its 48 independent matmuls run as two persistent launches (36 with M <= 8, "
                             "12 with M = 16)" if use_batch else "one call (one launch) per matmul"),
                   "batch_verified": batch_verified,
                   "launches_per_graph": (SWEEPS_PER_GRAPH * (2 if use_batch else len(M_SWEEP) * R_SETS)) if use_graph else None,
                   "allgather": None if world == 1 else (("peer stores from the batched decode kernel, the ranks meet once per launch" if use_batch else
                                                          "peer stores from the decode kernel (one launch per call)") if use_push
                                                         else "NCCL all-gather + interleave pass"),
                   "verified": verified,
                   "l2": f"inputs larger than L2: {R_SETS} rotating weight sets = {R_SETS * alg_bytes(1) / 1e6:.0f} MB, "
                         "each launch reads a set last touched 11 launches earlier"},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "peak_source": which, "frac_of_nominal_8TBps": achieved / NOMINAL_HBM_GBS,
                     "kernel": ("qmv_batch<4,m8|m16>" if world == 1 else "qmv_batch<4,m8|m16,push>") if use_batch else "qmv_mma<4,m8|m16>",
                     ("avg_us_per_matmul" if use_batch else "avg_us_per_launch"): avg_us,
                     "alg_bytes_per_launch": {str(M): alg_bytes(M) for M in M_SWEEP},
                     **({"traffic": NCU_TRAFFIC_BYTES_BATCH, "alg_bytes_of_that_launch": R_SETS * sum(alg_bytes(M) for M in M_SWEEP if M <= 8),
                         "traffic_unit": "bytes per launch (ncu dram read+write of one qmv_batch<4,m8> launch: the 36 matmuls with M <= 8)",
                         "traffic_over_algorithmic": NCU_TRAFFIC_BYTES_BATCH / (R_SETS * sum(alg_bytes(M) for M in M_SWEEP if M <= 8))}
                        if use_batch else
                        {"traffic": args.traffic_bytes, "traffic_unit": "bytes per launch (ncu dram read+write, M=1 launch)",
                         "traffic_over_algorithmic": args.traffic_bytes / alg_bytes(1) if args.traffic_bytes else None})},
        "per_M": {str(M): per_m[M] for M in M_SWEEP},
        "per_M_batched": per_m_batched,
        "single_calls": single,
        "cpu_reference_config": cpu_ref_config,
        "prefill": prefill,
        "chain": chain,
        "chain_sharded": chain_sharded,
        "gemm_sharded": gemm_sharded,
        "cpu_baseline": cpu,
        "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "steps": e2e_steps, "sweeps_per_step": e2e_reps,
                **({"matmuls": e2e_calls, "us_per_matmul": ms_e2e * 1e3 / max(1, e2e_calls)} if e2e_single else
                   {"calls": e2e_calls, "us_per_call": ms_e2e * 1e3 / max(1, e2e_calls)}),
                "driver": "python" if e2e_native is None else "C host loop (bench_e2e.c) over the plugin's entry points",
                "note": ("per sweep of 48 independent matmuls, pinned host buffers: ONE buffer_copy_from_host_async of every item's x, ONE "
                         + ("qmatmul_batch" if world == 1 else "qmatmul_sharded_push_batch") + " call, ONE blocking buffer_copy_to_host of "
                         + ("every item's y" if world == 1 else f"this rank's 1/{world} share of the result buffer (every rank ends with all outputs "
                            "whole; the hosts read them back once between them; both byte counts are summed over the ranks)")
                         + "; weights stay resident like the core's tensors (src/gpu_core.cpp:47-76)"
                         + ("; the host keeps two contexts (streams) and reads sweep r-1 back while sweep r computes" if e2e_two is not None else ""))
                        if e2e_single else
                        "per call, pinned host buffers: buffer_copy_from_host_async(x) + qmatmul + buffer_copy_to_host(y, blocking); weights stay resident "
                        "like the core's tensors (src/gpu_core.cpp:47-76)",
                **({"checked": e2e_checked, "one_context": e2e_one, "single_calls": e2e_single} if e2e_single else {})},
        "gpu_launches": int(launches),
        "clocks": clocks,
    }
    print(json.dumps(out))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--reps", type=int, default=50, help="sweeps per step")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--kernel-only", action="store_true",
                    help="skip the e2e and CPU-baseline legs (for short runs under a profiler)")
    ap.add_argument("--nccl-allgather", action="store_true",
                    help="N>1: gather the column slices with NCCL + an interleave pass instead of peer stores from the kernel")
    ap.add_argument("--e2e-one-context", action="store_true",
                    help="end-to-end leg: one context (copy in, batched call, blocking copy out, strictly one after the other)")
    ap.add_argument("--single-calls", action="store_true",
                    help="N=1: time the sweep as one call per matmul (the default hands each sweep to qmatmul_batch)")
    ap.add_argument("--e2e-python", action="store_true",
                    help="run the end-to-end leg's loop over the calls in Python instead of in C (bench_e2e.c)")
    ap.add_argument("--no-sharded-legs", action="store_true",
                    help="N>1: skip the column-sharded 8-bit GEMM and chain legs that follow the sweep by default")
    ap.add_argument("--gemm-sharded", action="store_true",
                    help="N>1: also run the column-sharded 8-bit large GEMM (strong scaling, NCCL all-gather) after the sweep")
    ap.add_argument("--chain-sharded", action="store_true",
                    help="N>1: also run the column-sharded quantized-linear chain (strong scaling) after the sweep")
    ap.add_argument("--chain-only", action="store_true", help="run only the quantized-linear chain leg")
    ap.add_argument("--prefill-only", action="store_true", help="run only the tensor-bound legs (short, for profiling)")
    ap.add_argument("--traffic-bytes", type=float, default=NCU_TRAFFIC_BYTES,
                    help="dram bytes per launch of the dominant kernel from an ncu capture, echoed into roofline.traffic")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            print(f"launch with torchrun --nproc-per-node {args.gpus} for --gpus {args.gpus}", file=sys.stderr)
            sys.exit(2)
    if args.impl == "reference":
        run_reference(args, rank)
    else:
        run_ours(args, rank, world)


if __name__ == "__main__":
    main()
