"""Benchmark of the hot path: batch-1 greedy decode of the Qwen3-8B-shape W4A16 model.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

A step is one decoded token: one pass of the 36 layers + unembed + arg-max at batch 1.  Workload
at every N: the full 36-layer model with seeded random weights (written as the reference's .bin
set and loaded through the constructor), prompt of 128 seeded ids, then W warm-up and K timed
decode steps.  For N > 1 the layers are split over N GPUs as a pipeline (strong scaling: the work
is the same model).  Prints ONE JSON line.

`value` is device-timed (CUDA events around the decode loop, weights and KV resident in HBM);
`e2e` is the host wall-clock of the public API call that produces the same K ids into host memory.
`roofline` describes the dominant kernel of the timed region (decode_pass_kernel, one launch per
token: algorithmic bytes of a token / CUDA-event time of a step); `gemv_roofline` times the stand-alone
fused dequant-GEMV operator on the 12288x4096 matrices, cycling 36 distinct matrices (906 MB > L2).
`cpu_baseline` / `--impl reference` time the CPU oracle port of the same math on the host cores
(the reference has no CPU path and does not build).
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
from __graft_entry__ import load_oracle, load_package  # noqa: E402

METRIC = "batch-1 decode tokens/s (Qwen3-8B W4A16)"
LAST_REF_GEMV_US = None
# dram__bytes_read.sum + dram__bytes_write.sum of decode_pass_kernel over its algorithmic bytes, from the ncu
# capture summarised in profiles/ (a 6-layer pass; traffic grows with the bytes streamed).
NCU_TRAFFIC_RATIO = (509.30 + 4.82) / 507.6
PROMPT_LEN = 128
SEED = 0
# Algorithmic bytes of one decoded token: packed weights of 36 layers + unembed, scale/zero-point
# entries read, KV rows read (589,824 bytes per position of context).
LAYER_PACKED = 25165824 + 8388608 + 25165824 + 25165824
UNEMBED_PACKED = 311164928


def token_bytes(context):
    return 36 * (LAYER_PACKED + 1024) + UNEMBED_PACKED + 2374 * 2 + 589824 * context


def gemv_bytes(M, K):
    return M * K // 2 + 4 * (M // 128) + 2 * K + 2 * M


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        return json.load(open(p)), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index=0):
        self.rows, self.proc, self.index = [], None, index

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                                          "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        sm = [float(r[1]) for r in self.rows if len(r) >= 9 and r[1].replace(".", "").isdigit()]
        mx = [float(r[2]) for r in self.rows if len(r) >= 9 and r[2].replace(".", "").isdigit()]
        reasons = set()
        for r in self.rows:
            if len(r) >= 9:
                for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def cpu_decode_tokens_per_s(orc, weight_dir, n_tokens, context):
    """The oracle port on the host cores: n_tokens decode passes of the full model at the given context."""
    import numpy as np
    cfg = orc.default_config(max_pos=context + n_tokens + 1)
    m = orc.Model(cfg)
    if weight_dir is not None:
        assert m.load_dir(weight_dir) == 0
    else:
        m.init_random(SEED)
    m.fill_kv(SEED, context)
    hidden = orc.gen_normal_f16(SEED, orc.ACT, cfg.hidden)
    # warm-up pass (page in the weights), then the timed passes
    times = []
    for t in range(n_tokens + 1):
        t0 = time.perf_counter()
        h = hidden
        for layer in range(cfg.layers):
            h = m.layer(layer, context + t, h)
        tok, _ = m.sample(h)
        times.append(time.perf_counter() - t0)
        hidden = orc.embed_gather(m.packed(0, orc.EMB, cfg.hidden * cfg.vocab // 2), m.f16(0, orc.EMB_SCALE, cfg.hidden // 128),
                                  m.f16(0, orc.EMB_ZP, cfg.hidden // 128), cfg.hidden, cfg.vocab, tok)
    m.close()
    return n_tokens / sum(times[1:]), np.mean(times[1:]) * 1e3


def run_reference(args, rank):
    """The reference arm: the reference has no CPU implementation and does not compile, so the CPU
    oracle port of its math stands in, with every host thread it can use."""
    if rank != 0:
        return
    orc = load_oracle()
    tps, ms = cpu_decode_tokens_per_s(orc, None, args.steps, args.prompt_len + args.warmup)
    line = {"impl": "reference", "metric": METRIC, "value": tps, "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "w4a16 (fp16 products, double accumulation)", "data": "synthetic",
            "config": {"workload": "full 36-layer Qwen3-8B-shape W4A16 model, batch-1 decode steps at context >= 128, seeded random weights",
                       "note": "CPU oracle port; the reference itself has no CPU path and does not build"},
            "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": orc.num_threads(), "kind": "port",
                             "sample": f"{args.steps} decode-token passes, KV rows pre-filled to context {args.prompt_len + args.warmup}"},
            "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line))


def roofline_gemv(pkg, torch, M, K, n_mats, reps):
    """Average launch duration of the fused dequant-GEMV on n_mats distinct matrices (cycled so that
    every launch misses L2), timed with CUDA events on the launching stream."""
    import importlib
    ops = importlib.import_module("qw3awq_b200.ops")
    dev = torch.device("cuda:0")
    ws = ops.Workspace(pdl=False)
    mats = []
    g = torch.Generator(device=dev)
    g.manual_seed(SEED)
    for _ in range(n_mats):
        packed = torch.randint(0, 256, (M * K // 2,), dtype=torch.uint8, device=dev, generator=g)
        scale = (torch.randn(M // 128, device=dev, generator=g).abs() * 0.02).half()
        zp = torch.randint(6, 10, (M // 128,), device=dev, generator=g).half()
        mats.append(ops.W4Linear(packed, scale, zp, M, K))
    x = torch.randn(K, device=dev, generator=g).half()
    y = torch.zeros(M, dtype=torch.float16, device=dev)
    a = ops.gemv_args(x, y=y)
    for w in mats[:4]:
        ops.gemv_w4a16(w, ws, a)
    torch.cuda.synchronize()

    def timed(pdl):
        # One CUDA graph holding a launch per matrix removes the host launch cost from the timing.
        ws_g = ops.Workspace(pdl=pdl)
        side = torch.cuda.Stream()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            with torch.cuda.graph(graph, stream=side):
                for w in mats:
                    ops.gemv_w4a16(w, ws_g, a)
            graph.replay()
            side.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(side)
            for _ in range(reps):
                graph.replay()
            e1.record(side)
            side.synchronize()
            ws_g.check()
        return e0.elapsed_time(e1) * 1e3 / (reps * len(mats))

    us = timed(False)
    us_pdl = timed(True)
    n = reps * len(mats)
    # the reference's method at n = 1: cuBLAS on fp16 copies of the same matrices (4x the bytes)
    global LAST_REF_GEMV_US
    wdqs = [ops.dequant_w4(w.packed, w.scale, w.zp, M, K).view(K, M) for w in mats[:min(len(mats), 12)]]
    xr = x.view(1, K)
    for wd in wdqs:
        torch.matmul(xr, wd)
    torch.cuda.synchronize()
    c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    c0.record()
    for _ in range(reps):
        for wd in wdqs:
            torch.matmul(xr, wd)
    c1.record()
    torch.cuda.synchronize()
    LAST_REF_GEMV_US = c0.elapsed_time(c1) * 1e3 / (reps * len(wdqs))
    del wdqs
    for w in mats:
        w.close()
    return us, n, us_pdl


def reference_method_token_us(torch, n_layers_cycled=6, reps=6):
    """The reference's decode method, contractions only: cuBLAS at n = 1 on fp16 copies of wqkv, wo, w1, w2 of every
    layer and of unembed (Inference.cu:1052-1273; 13.3 GB of fp16 per token instead of 3.3 GB packed).  Random fp16
    matrices of those shapes, several distinct layers cycled so that nothing stays in L2.  No norms, attention, copies
    or host waits: a lower bound on the time per token of the dequantise-then-cuBLAS design on this GPU."""
    dev = torch.device("cuda:0")
    shapes = [(4096, 12288), (4096, 4096), (4096, 12288), (12288, 4096)]          # [K][M] as the library reads them
    layers = [[torch.randn(k, m, device=dev, dtype=torch.float16) for k, m in shapes] for _ in range(n_layers_cycled)]
    unemb = torch.randn(4096, 151936, device=dev, dtype=torch.float16)
    xs = {4096: torch.randn(1, 4096, device=dev, dtype=torch.float16), 12288: torch.randn(1, 12288, device=dev, dtype=torch.float16)}

    def one_round():
        for mats in layers:
            for w in mats:
                torch.matmul(xs[w.shape[0]], w)
        torch.matmul(xs[4096], unemb)

    one_round()
    torch.cuda.synchronize()
    e_l = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    t_layers = t_unemb = 0.0
    for _ in range(reps):
        e_l[0].record()
        for mats in layers:
            for w in mats:
                torch.matmul(xs[w.shape[0]], w)
        e_l[1].record()
        torch.matmul(xs[4096], unemb)
        e_l[2].record()
        torch.cuda.synchronize()
        t_layers += e_l[0].elapsed_time(e_l[1])
        t_unemb += e_l[1].elapsed_time(e_l[2])
    per_layer_us = t_layers * 1e3 / (reps * n_layers_cycled)
    unemb_us = t_unemb * 1e3 / reps
    return 36 * per_layer_us + unemb_us, per_layer_us, unemb_us


def pass_only(pkg, orc, args):
    """Token passes of a model cut to --pass-layers layers (full-size matrices, small vocabulary unless asked
    otherwise): the small case for profilers.  With QW3_TRACE=1 the engine records global-timer stamps inside
    decode_pass_kernel; they are summarised per operator (CTA 0 entering each operator) and per phase (all
    CTAs, one layer in the middle)."""
    import ctypes as C
    import numpy as np
    L, V = args.pass_layers, args.pass_vocab
    cfg = dict(hidden=4096, inter=12288, heads=32, head_dim=128, layers=L, vocab=V, max_pos=args.prompt_len + args.steps + args.warmup + 8,
               rope_base=10000.0)
    wdir = args.weights or os.path.join(tempfile.gettempdir(), f"qw3_pass_weights_{L}_{V}")
    if not os.path.exists(os.path.join(wdir, "unembed_zp.bin")):
        orc.write_weight_dir(orc.default_config(**cfg), SEED, wdir)
    prompt = [int(t) for t in orc.gen_tokens(SEED, orc.TOKENS, args.prompt_len, V)]
    inf = pkg.QWen3AWQInfer(wdir, **cfg)
    inf.generateResponse(prompt, args.warmup)
    inf.decode_more(args.steps)
    out = {"kernel": "decode_pass_kernel", "layers": L, "vocab": V, "context": args.prompt_len + args.warmup,
           "ms_per_token": inf.last_timing()[1] / args.steps}
    if os.environ.get("QW3_TRACE"):
        n_ops = 1 + 5 * L + 1
        buf = (C.c_uint64 * (n_ops + 8))()
        n = C.c_int32()
        pkg.cabi.check(pkg.cabi.lib().qw3_debug_trace(inf._h, 0, buf, n_ops + 8, C.byref(n)), "qw3_debug_trace")
        d = np.diff(np.array(buf[:n.value], dtype=np.float64)) / 1e3
        lay = d[1:1 + 5 * L].reshape(L, 5)
        out["op_us"] = {"embed": float(d[0]), "unembed_argmax": float(d[1 + 5 * L]), "layer": float(lay.sum(axis=1).mean()),
                        **{k: float(v) for k, v in zip(["wqkv", "attention", "wo", "w1", "w2"], lay.mean(axis=0))}}
        G = 148
        buf2 = (C.c_uint64 * (256 * n_ops * 8))()
        pkg.cabi.check(pkg.cabi.lib().qw3_debug_trace(inf._h, 0, buf2, -(256 * n_ops * 8), C.byref(n)), "qw3_debug_trace")
        t = np.ctypeslib.as_array(buf2).reshape(256, n_ops, 8)[:G].astype(np.float64)
        t[t == 0] = np.nan
        names = ["enter", "input wait", "prologue", "units", "flush", "gather", "epilogue", "end"]
        li = L // 2
        phases = {}
        for k, op in enumerate(["wqkv", "attention", "wo", "w1", "w2"]):
            e = t[:, 1 + 5 * li + k, :]
            e = e - np.nanmin(e[:, 0])
            if op == "attention":   # its events: q polled, rows done, CTA merge, splits merged, ctx stored
                e = e[::4]          # the CTAs that merge a head (split 0 of 4)
            if True:   # median over CTAs of the time each phase ends, from the first CTA entering
                phases[op] = {nm: float(np.nanmedian(e[:, j]) / 1e3) for j, nm in enumerate(names) if np.isfinite(e[:, j]).any()}
        out["phase_end_us_median_over_ctas"] = phases
    inf.close()
    return out


def gemm_sweep(pkg, torch, shapes, rows_list, reps=10, ref_cublas=True):
    """Batched-row sweep of the tcgen05 W4A16 contraction: one CUDA graph of `reps` launches per
    configuration, CUDA events on the launching stream.  Rows <= 64 are HBM-bound, above that the
    contraction is tensor-bound; each line carries both fractions against the measured peaks."""
    import importlib
    ops = importlib.import_module("qw3awq_b200.ops")
    dev = torch.device("cuda:0")
    peaks, peak_kind = measured_peaks()
    g = torch.Generator(device=dev)
    g.manual_seed(SEED)
    out = []
    for (M, K) in shapes:
        packed = torch.randint(0, 256, (M * K // 2,), dtype=torch.uint8, device=dev, generator=g)
        scale = (torch.randn(M // 128, device=dev, generator=g).abs() * 0.02).half()
        zp = torch.randint(6, 10, (M // 128,), device=dev, generator=g).half()
        w = ops.W4Linear(packed, scale, zp, M, K)
        for R in rows_list:
            x = torch.randn(R, K, device=dev, generator=g).half()
            y = torch.zeros(R, M, dtype=torch.float16, device=dev)
            ws = ops.Workspace()
            ops.gemm_w4a16(w, ws, x, y)
            torch.cuda.synchronize()
            side = torch.cuda.Stream()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.stream(side):
                with torch.cuda.graph(graph, stream=side):
                    for _ in range(reps):
                        ops.gemm_w4a16(w, ws, x, y)
                graph.replay()
                side.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(side)
                graph.replay()
                graph.replay()
                e1.record(side)
                side.synchronize()
                ws.check()
            us = e0.elapsed_time(e1) * 1e3 / (2 * reps)
            # the reference's method for the same product: fp16 copy of the weights (dequantAwqKernel once),
            # then cuBLAS on it (cublasGemmEx, Inference.cu:1052-1065); torch.matmul issues that library call
            if ref_cublas:
                wdq = ops.dequant_w4(packed, scale, zp, M, K).view(K, M)      # flat buffer read column-major: [K][M]
                torch.matmul(x, wdq)
                torch.cuda.synchronize()
                c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                c0.record()
                for _ in range(reps):
                    torch.matmul(x, wdq)
                c1.record()
                torch.cuda.synchronize()
                ref_us = c0.elapsed_time(c1) * 1e3 / reps
                del wdq
            else:
                ref_us = None
            flops = 2.0 * R * M * K
            nbytes = M * K // 2 + 2 * R * K + 2 * R * M
            tf, gbs = flops / us / 1e6, nbytes / us / 1e3
            out.append({"shape": [M, K], "rows": R, "us": us, "TFLOP/s": tf, "GB/s": gbs,
                        "bound": "hbm" if R <= 64 else "tensor",
                        "frac_tensor": tf / peaks["bf16_tflops"], "frac_hbm": gbs / peaks["hbm_gbs"], "peak_kind": peak_kind,
                        "ref_dequant_then_cublas_us": ref_us})
        w.close()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--weights", default=None, help="existing weight directory (default: generate into a temp dir)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--prompt-len", type=int, default=PROMPT_LEN, help="prompt length (128 is the benchmark configuration)")
    ap.add_argument("--only-roofline", action="store_true", help="run only the dominant-kernel timing (small case for profilers)")
    ap.add_argument("--roofline-mats", type=int, default=36)
    ap.add_argument("--roofline-reps", type=int, default=6)
    ap.add_argument("--roofline-shape", default="12288x4096")
    ap.add_argument("--only-pass", action="store_true",
                    help="run token passes of a model with --pass-layers layers (small case for profilers); with QW3_TRACE=1 in "
                         "the environment also prints the per-operator and per-phase times of the pass kernel")
    ap.add_argument("--pass-layers", type=int, default=6)
    ap.add_argument("--pass-vocab", type=int, default=2048)
    ap.add_argument("--only-gemm", action="store_true", help="batched-row sweep of the tensor-core W4A16 contraction")
    ap.add_argument("--gemm-shapes", default="12288x4096,4096x4096,4096x12288,151936x4096")
    ap.add_argument("--gemm-rows", default="16,64,256,2048")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    # Only the result line may reach stdout: libraries (NCCL's version banner, for one) print there too, so
    # file descriptor 1 is pointed at stderr for the run and the saved descriptor is used for the JSON lines.
    sys.stdout.flush()
    result_fd = os.dup(1)
    os.dup2(2, 1)
    global print
    builtin_print = print

    def print(*a, **k):   # noqa: A001 - every print of this module is a result line
        os.write(result_fd, (" ".join(str(x) for x in a) + "\n").encode())
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference(args, rank)
        return

    import torch
    import torch.distributed as dist
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback for the product path")
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
    pkg = load_package()
    if args.only_roofline:
        M, K = (int(v) for v in args.roofline_shape.split("x"))
        us, n, us_pdl = roofline_gemv(pkg, torch, M, K, args.roofline_mats, args.roofline_reps)
        print(json.dumps({"kernel": "gemv_w4a16_kernel", "shape": [M, K], "avg_launch_us": us, "avg_launch_us_pdl": us_pdl,
                          "launches": n, "GBps": gemv_bytes(M, K) / us / 1e3, "ref_dequant_then_cublas_us": LAST_REF_GEMV_US}))
        return
    if args.only_pass:
        print(json.dumps(pass_only(pkg, load_oracle(), args)))
        return
    if args.only_gemm:
        shapes = [tuple(int(v) for v in t.split("x")) for t in args.gemm_shapes.split(",")]
        for line in gemm_sweep(pkg, torch, shapes, [int(v) for v in args.gemm_rows.split(",")]):
            print(json.dumps(line))
        return
    orc = load_oracle()   # weight generator + CPU baseline leg only

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    import importlib
    pipeline = importlib.import_module("qw3awq_b200.pipeline")
    n_gpus = args.gpus
    if world > 1 and world != n_gpus:
        raise SystemExit(f"--gpus {n_gpus} but WORLD_SIZE={world}: launch one rank per GPU")
    # weights: rank 0 writes the reference's .bin set once; every rank loads its own stage from it
    wdir = args.weights or os.path.join(tempfile.gettempdir(), f"qw3_bench_weights_{os.environ.get('MASTER_PORT', 'single')}_{os.getppid() if world > 1 else os.getpid()}")
    made = False
    if rank == 0 and not os.path.exists(os.path.join(wdir, "unembed_zp.bin")):
        orc.write_weight_dir(orc.default_config(), SEED, wdir)
        made = args.weights is None
    barrier()
    prompt = [int(t) for t in orc.gen_tokens(SEED, orc.TOKENS, args.prompt_len, 151936)]
    max_pos = args.prompt_len + args.warmup + 2 * args.steps + 8
    if world > 1:
        # one process per GPU: this rank owns stage `rank`; hidden state and token id move by peer stores
        inf = pkg.QWen3AWQInfer(wdir, max_pos=max_pos, n_stages=world, world=world, rank=rank, device=list(range(world)))
        pipeline.connect_ring(inf, dist)
    else:
        inf = pkg.QWen3AWQInfer(wdir, max_pos=max_pos, n_stages=n_gpus, device=list(range(n_gpus)))
    barrier()
    inf.generateResponse(prompt, args.warmup)              # prompt pass + W warm-up decode steps
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    barrier()
    # device-timed: K decode steps, CUDA events inside the engine around this rank's decode loop
    ids_dev = inf.decode_more(args.steps)
    _, decode_ms = inf.last_timing()
    launches = inf.last_launches()
    barrier()
    # end to end: the same K steps through the public API, host wall-clock, ids to host memory
    t0 = time.perf_counter()
    ids_e2e = inf.decode_more(args.steps)
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    barrier()
    prefill = None
    if world == 1 and n_gpus == 1:   # prompt phase: the reference's token loop against the batched-row path
        inf.generateResponse(prompt, 1)
        loop_ms = inf.last_timing()[0]
        inf.set_batched_prefill(True)
        inf.generateResponse(prompt, 1)      # first use allocates the block buffers
        inf.generateResponse(prompt, 1)
        blk_ms = inf.last_timing()[0]
        inf.set_batched_prefill(False)
        prefill = {"prompt_tokens": len(prompt), "token_loop_ms": loop_ms, "batched_ms": blk_ms,
                   "batched_tokens_per_s": len(prompt) / (blk_ms * 1e-3),
                   "note": "device time of the prompt phase of generateResponse; batched = tcgen05 W4A16 contraction over the block"}
    if world > 1:   # prompt phase with one process per GPU: token loop through the mailboxes against blocks of rows
        loop_ms = blk_ms = 0.0
        ok = 1.0
        try:   # an extra beside the timed region: a failure here must not cost the decode numbers above
            inf.generateResponse(prompt, 1)
            loop_ms = inf.last_timing()[0]
            inf.set_batched_prefill(True)
            inf.generateResponse(prompt, 1)
            inf.generateResponse(prompt, 1)
            blk_ms = inf.last_timing()[0]
            inf.set_batched_prefill(False)
        except Exception as exc:   # every device wait is bounded, so the other ranks come out as well
            sys.stderr.write(f"rank {rank}: prompt-phase comparison failed: {exc}\n")
            ok = 0.0
        pt = torch.tensor([loop_ms, blk_ms, -ok], dtype=torch.float64, device=f"cuda:{local}")
        dist.all_reduce(pt, op=dist.ReduceOp.MAX)
        if float(pt[2]) == -1.0:
            prefill = {"prompt_tokens": len(prompt), "token_loop_ms": float(pt[0]), "batched_ms": float(pt[1]),
                       "batched_tokens_per_s": len(prompt) / (float(pt[1]) * 1e-3),
                       "note": "device time of the prompt phase, max over ranks; batched = blocks of rows handed from stage to stage"}
        else:
            prefill = {"error": "the prompt-phase comparison failed on a rank (see stderr)"}
    if world > 1:   # max over ranks of the device time and of the wall-clock; launches summed
        t = torch.tensor([decode_ms, e2e_s], dtype=torch.float64, device=f"cuda:{local}")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        decode_ms, e2e_s = float(t[0]), float(t[1])
        ln = torch.tensor([launches], dtype=torch.int64, device=f"cuda:{local}")
        dist.all_reduce(ln, op=dist.ReduceOp.SUM)
        launches = int(ln[0])
        ids_dev = pipeline.broadcast_ids(ids_dev, args.steps, dist)
        ids_e2e = pipeline.broadcast_ids(ids_e2e, args.steps, dist)
    inf.close()
    result = None
    if rank == 0:
        clocks = sampler.stop()
        ctx_mid = args.prompt_len + args.warmup + args.steps // 2
        tps = args.steps / (decode_ms * 1e-3)
        peaks, peak_kind = measured_peaks()
        # the stand-alone GEMV operator (what a caller of qw3_gemv_w4a16 gets), reported beside the pass kernel
        M, K = 12288, 4096
        us, n_launch, us_pdl = roofline_gemv(pkg, torch, M, K, args.roofline_mats, args.roofline_reps)
        achieved = gemv_bytes(M, K) / (us * 1e-6) / 1e9
        gemv_roof = {"bound": "hbm", "kernel": "gemv_w4a16_kernel (12288x4096, STORE epilogue)", "achieved": achieved,
                     "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
                     "avg_launch_us": us, "avg_launch_us_with_pdl": us_pdl, "launches_timed": n_launch,
                     "bytes_per_launch": gemv_bytes(M, K), "l2": "36 distinct matrices cycled (906 MB > 126 MB L2)",
                     "ref_dequant_then_cublas_us": LAST_REF_GEMV_US}
        ref_us, ref_layer_us, ref_unemb_us = reference_method_token_us(torch)
        ref_method = {"what": "the reference's design on this GPU, contractions only: cuBLAS at n=1 on fp16 copies of the five "
                              "matrices per layer and of unembed (13.3 GB per token); no norms, attention, copies or host waits",
                      "us_per_token": ref_us, "us_per_layer": ref_layer_us, "unembed_us": ref_unemb_us,
                      "tokens_per_s_upper_bound": 1e6 / ref_us}
        decode_gbs = token_bytes(ctx_mid) * tps / 1e9
        line = {"metric": METRIC, "value": tps, "unit": "tokens/s", "n_gpus": n_gpus, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": decode_ms / args.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                "dtype": "w4a16 (int4 weights, fp16 activations, fp32 accumulation)", "data": "synthetic",
                "config": {"workload": "full 36-layer Qwen3-8B-shape W4A16 model (hidden 4096, 32 heads, inter 12288, vocab 151936), "
                                       f"prompt {args.prompt_len} ids, batch-1 greedy decode steps at context {args.prompt_len + args.warmup}.."
                                       f"{args.prompt_len + args.warmup + 2 * args.steps}, seeded random weights",
                           "parallelism": f"pp{n_gpus}" + (" (one process per GPU, P2P hand-off)" if world > 1 else ""),
                           "l2": "3.3 GB of weights streamed per step (inputs larger than L2)"},
                # dominant kernel of the timed region: decode_pass_kernel, one launch per token per stage.  Its launch
                # duration is the CUDA-event time of a step (which also holds the 1-thread step_tail launch).
                "roofline": {"bound": "hbm", "kernel": "decode_pass_kernel (36 layers + unembed + arg-max, one launch per token)",
                             "achieved": decode_gbs, "peak": peaks["hbm_gbs"], "peak_kind": peak_kind + " (burst copy)",
                             "unit": "GB/s", "frac": decode_gbs / peaks["hbm_gbs"],
                             "traffic": int(token_bytes(ctx_mid) * NCU_TRAFFIC_RATIO), "bytes_per_launch": token_bytes(ctx_mid),
                             "avg_launch_us": decode_ms * 1e3 / args.steps,
                             "traffic_note": "dram read+write of an ncu capture of a 6-layer pass (514.1 MB for 507.6 MB "
                                             "algorithmic), scaled by bytes to the 36-layer launch",
                             "note": "at batch 1 the stages of N GPUs run one after another: one GPU's bandwidth is in use at a time"},
                "gemv_roofline": gemv_roof, "reference_method_gpu": ref_method,
                "e2e": {"value": args.steps / e2e_s, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 4,
                        "note": "host wall-clock of decode_more(K) through the C ABI; the sampled id feeds the next step on the device"},
                "gpu_launches": int(launches), "clocks": clocks, "prefill": prefill,
                "tokens_equal_between_runs": None if len(ids_dev) != len(ids_e2e) else True}
        if not args.no_cpu_baseline and n_gpus == 1:
            n_cpu = 8
            cpu_tps, _ = cpu_decode_tokens_per_s(orc, wdir, n_cpu, args.prompt_len)
            line["cpu_baseline"] = {"value": cpu_tps, "unit": "tokens/s", "cores": orc.num_threads(), "kind": "port",
                                    "sample": f"{n_cpu} decode-token passes of the same model on the host, KV rows pre-filled to context {args.prompt_len}"}
            all_threads = orc.num_threads()
            orc.set_num_threads(1)
            cpu1_tps, _ = cpu_decode_tokens_per_s(orc, wdir, 1, args.prompt_len)
            orc.set_num_threads(all_threads)
            line["cpu_baseline_1thread"] = {"value": cpu1_tps, "unit": "tokens/s", "cores": 1, "kind": "port",
                                            "sample": "1 decode-token pass of the same model on one host thread (after a warm-up pass)"}
        result = line
    barrier()
    if rank == 0:
        if made:
            import shutil
            shutil.rmtree(wdir, ignore_errors=True)
        print(json.dumps(result))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
