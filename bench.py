"""Benchmark of the hot path: batch-1 greedy decode of the Qwen3-8B-shape W4A16 model.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

A step is one decoded token: one pass of the 36 layers + unembed + arg-max at batch 1.  Workload: the full
36-layer model with seeded random weights (written as the reference's .bin set and loaded through the
constructor); at N = 1 a prompt of 128 seeded ids, at N > 1 a prompt of 512 ids (the multi-GPU configuration of
the baseline), then W warm-up and K timed decode steps.  For N > 1 the same model is spread over N GPUs (strong
scaling), as a layer pipeline (--parallel pp, the reference's contract) or with every matrix row-split over the
GPUs (--parallel tp).  Prints ONE JSON line.

Every id the run produces (warm-up, timed and end-to-end steps) is compared with the golden ids the CPU oracle
produced for the same seed and prompt (tests/golden/golden.json): `ids_match_golden`; a mismatch makes the run fail.

`value` is device-timed: the timed region (K decode steps, CUDA events inside the engine around this rank's decode
loop, weights and KV resident in HBM) is repeated, the median of the repeats counts, all are listed.
`e2e` is the host wall-clock of the public API call that produces K more ids into host memory; `e2e_generate` the
wall-clock of generateResponse(prompt, K) with the prompt ids in host memory, prompt phase included.
`roofline` describes the dominant kernel of the timed region (one launch per token: algorithmic bytes of a token /
CUDA-event time of a step); `gemv_roofline` times the stand-alone fused dequant-GEMV operator on the 12288x4096
matrices, cycling 36 distinct matrices (906 MB > L2).  `cpu_baseline` / `--impl reference` time the CPU oracle port
of the same math on the host cores (the reference has no CPU path and does not build).
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
# dram__bytes_read.sum + dram__bytes_write.sum of fused_pass_kernel over its algorithmic bytes, from the ncu
# capture summarised in profiles/fused_pass_kernel_6layers_ncu.md (a 6-layer pass; traffic grows with the bytes streamed).
NCU_TRAFFIC_RATIO = (509.26 + 16.55) / 507.52
NCU_TRAFFIC_NOTE = ("dram read+write of an ncu capture of a 6-layer pass (525.8 MB for 507.5 MB algorithmic), scaled by bytes to the "
                    "36-layer launch")
PROMPT_LEN = 128          # one GPU: prompt 128 + 20 new ids is the baseline's single-GPU configuration
PROMPT_LEN_MULTI = 512    # several GPUs: prompt 512 + 128 new ids
SEED = 0
REPEATS = 7               # timed regions of K steps each; the median counts
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


def workload_string(args):
    return ("full 36-layer Qwen3-8B-shape W4A16 model (hidden 4096, 32 heads, inter 12288, vocab 151936), "
            f"prompt {args.prompt_len} ids, batch-1 greedy decode steps from context {args.prompt_len + args.warmup} on, "
            "seeded random weights")


def golden_ids(prompt_len):
    """Ids the CPU oracle produced for seed 0 and this prompt length (None when there is no such fixture)."""
    path = os.path.join(ROOT, "tests", "golden", "golden.json")
    if not os.path.exists(path):
        return None, None
    g = json.load(open(path))
    for name in ("full_model", "full_model_c4"):
        if name in g and g[name]["n_prompt"] == prompt_len and g[name]["seed"] == SEED and not g[name]["sample_first"]:
            return name, g[name]["ids"]
    return None, None


def run_reference(args, rank):
    """The reference arm: the reference has no CPU implementation and does not compile, so the CPU
    oracle port of its math stands in, with every host thread it can use."""
    if rank != 0:
        return
    orc = load_oracle()
    # every host core, whatever OMP_NUM_THREADS the launcher exported (torch.distributed.run sets it to 1)
    orc.set_num_threads(os.cpu_count() or 1)
    tps, ms = cpu_decode_tokens_per_s(orc, None, args.steps, args.prompt_len + args.warmup)
    line = {"impl": "reference", "metric": METRIC, "value": tps, "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "w4a16 (fp16 products, double accumulation)", "data": "synthetic",
            "config": {"workload": workload_string(args),
                       "note": "CPU oracle port on the host cores; the reference itself has no CPU path and does not build"},
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


def reference_method_token_us(torch, orc, weight_dir, n_layers_cycled=6, reps=6):
    """The reference's decode method on this GPU, contractions only (Inference.cu:1052-1273): its own dequantAwqKernel
    expands the packed matrices of several layers and of unembed to fp16 once (Inference.cu:908-1008), then its own
    cublasGemmEx call (m = out_dim, n = 1, k = in_dim on that buffer) runs per matrix, layers cycled so that nothing
    stays in L2 (13.3 GB of fp16 per token instead of 3.3 GB packed).  Both come from oracle/_ref (the reference's
    kernels compiled from its checkout); where that library is absent, torch.matmul on random fp16 matrices of the same
    shapes stands in and the result says so.  No norms, attention, copies or host waits: a lower bound on the time per
    token of the dequantise-then-cuBLAS design."""
    import ctypes as C
    import numpy as np
    dev = torch.device("cuda:0")
    shapes = [("wqkv", "bqkv", 12288, 4096), ("wo", "wo", 4096, 4096), ("w1", "w1", 12288, 4096), ("w2", "w2", 4096, 12288)]
    ref_so = os.path.join(ROOT, "oracle", "_ref", "libref_kernels.so")
    ref = None
    if os.path.exists(ref_so) and weight_dir is not None:
        ref = C.CDLL(ref_so)
        vp = C.c_void_p
        ref.ref_dequant.argtypes = [vp, vp, vp, vp, C.c_int, C.c_int, vp]
        ref.ref_gemv_cublas.argtypes = [vp, vp, vp, C.c_int, C.c_int, C.c_int, vp]

    def load(name, count, dtype):
        return torch.from_numpy(np.fromfile(os.path.join(weight_dir, name), dtype=dtype, count=count)).to(dev)

    def expand(stem, sz_stem, M, K, wrap):
        """fp16 buffer [M*K] as the reference's dequantAwqKernel writes it (rows = out_dim, cols = in_dim)."""
        packed = load(stem + ".bin", M * K // 2, np.uint8)
        n = M // 128
        sc, zp = load(sz_stem + "_scale.bin", n, np.float16), load(sz_stem + "_zp.bin", n, np.float16)
        if wrap and K // 128 > n:   # the reference indexes past its arrays here: wrap-extended copies, as the engine reads them
            idx = torch.arange(K // 128, device=dev) % n
            sc, zp = sc[idx].contiguous(), zp[idx].contiguous()
        out = torch.empty(M * K, dtype=torch.float16, device=dev)
        rc = ref.ref_dequant(packed.data_ptr(), sc.data_ptr(), zp.data_ptr(), out.data_ptr(), M, K, None)
        assert rc == 0, rc
        return out

    if ref is not None:
        layers = [[(expand(f"layer_{l}_{st}", f"layer_{l}_{sz}", M, K, True), M, K) for st, sz, M, K in shapes] for l in range(n_layers_cycled)]
        unemb = (expand("unembed", "unembed", 151936, 4096, False), 151936, 4096)
        how = "oracle/_ref: the reference's dequantAwqKernel once, then its cublasGemmEx call (CUBLAS_COMPUTE_16F) per matrix"
    else:
        layers = [[(torch.randn(M * K, device=dev, dtype=torch.float16), M, K) for _, _, M, K in shapes] for _ in range(n_layers_cycled)]
        unemb = (torch.randn(151936 * 4096, device=dev, dtype=torch.float16), 151936, 4096)
        how = "torch.matmul (cuBLAS) on random fp16 matrices of the reference's shapes (oracle/_ref not built)"
    xs = {4096: torch.randn(4096, device=dev, dtype=torch.float16), 12288: torch.randn(12288, device=dev, dtype=torch.float16)}
    ys = {4096: torch.empty(4096, device=dev, dtype=torch.float16), 12288: torch.empty(12288, device=dev, dtype=torch.float16),
          151936: torch.empty(151936, device=dev, dtype=torch.float16)}
    stream = torch.cuda.current_stream().cuda_stream

    def gemv(w, M, K):
        if ref is not None:
            rc = ref.ref_gemv_cublas(w.data_ptr(), xs[K].data_ptr(), ys[M].data_ptr(), M, K, 0, stream)
            assert rc == 0, rc
        else:
            torch.matmul(xs[K].view(1, K), w.view(K, M))

    def one_round():
        for mats in layers:
            for w, M, K in mats:
                gemv(w, M, K)
        gemv(*unemb)

    one_round()
    torch.cuda.synchronize()
    e_l = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    t_layers = t_unemb = 0.0
    for _ in range(reps):
        e_l[0].record()
        for mats in layers:
            for w, M, K in mats:
                gemv(w, M, K)
        e_l[1].record()
        gemv(*unemb)
        e_l[2].record()
        torch.cuda.synchronize()
        t_layers += e_l[0].elapsed_time(e_l[1])
        t_unemb += e_l[1].elapsed_time(e_l[2])
    per_layer_us = t_layers * 1e3 / (reps * n_layers_cycled)
    unemb_us = t_unemb * 1e3 / reps
    return 36 * per_layer_us + unemb_us, per_layer_us, unemb_us, how


def pass_only(pkg, orc, args):
    """Token passes of a model cut to --pass-layers layers (full-size matrices, small vocabulary unless asked
    otherwise): the small case for profilers (a 6-layer pass streams 503 MB per launch, four times the L2)."""
    L, V = args.pass_layers, args.pass_vocab
    cfg = dict(hidden=4096, inter=12288, heads=32, head_dim=128, layers=L, vocab=V, max_pos=args.prompt_len + args.steps + args.warmup + 8,
               rope_base=10000.0)
    wdir = args.weights or os.path.join(tempfile.gettempdir(), f"qw3_pass_weights_{L}_{V}")
    if not os.path.exists(os.path.join(wdir, "unembed_zp.bin")):
        orc.write_weight_dir(orc.default_config(**cfg), SEED, wdir)
    prompt = [int(t) for t in orc.gen_tokens(SEED, orc.TOKENS, args.prompt_len, V)]
    inf = pkg.QWen3AWQInfer(wdir, cluster=0 if args.no_cluster else 1, **cfg)
    inf.generateResponse(prompt, args.warmup)
    inf.decode_more(args.steps)
    layer_bytes = L * (LAYER_PACKED + 1024) + V * 4096 // 2
    ms = inf.last_timing()[1] / args.steps
    out = {"kernel": "fused_pass_kernel", "layers": L, "vocab": V, "context": args.prompt_len + args.warmup, "ms_per_token": ms,
           "packed_bytes_per_launch": layer_bytes, "GBps": layer_bytes / ms / 1e6, "cluster": not args.no_cluster}
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
    ap.add_argument("--prompt-len", type=int, default=None,
                    help="prompt length (default: 128 on one GPU, 512 on several: the baseline's two configurations)")
    ap.add_argument("--repeats", type=int, default=REPEATS, help="timed regions of --steps decode steps each (the median counts)")
    ap.add_argument("--parallel", default="tp", choices=["pp", "tp"],
                    help="several GPUs: row-split of every matrix over the GPUs (default: the only form in which a second GPU's "
                         "bandwidth works on the same token) or the reference's layer pipeline")
    ap.add_argument("--attn-split-min", type=int, default=0,
                    help="fused pass: contexts longer than this are split over the CTAs of a head group (0: the engine's default)")
    ap.add_argument("--no-cluster", action="store_true", help="fused pass: head groups exchange through global memory instead of a thread-block cluster (the library's default; "
                         "the bench turns clusters on unless this is given; needed under Nsight Compute, which terminates a process that "
                         "launches the cooperative cluster form)")
    ap.add_argument("--only-roofline", action="store_true", help="run only the dominant-kernel timing (small case for profilers)")
    ap.add_argument("--roofline-mats", type=int, default=36)
    ap.add_argument("--roofline-reps", type=int, default=6)
    ap.add_argument("--roofline-shape", default="12288x4096")
    ap.add_argument("--only-pass", action="store_true",
                    help="run token passes of a model with --pass-layers layers (small case for profilers)")
    ap.add_argument("--pass-layers", type=int, default=6)
    ap.add_argument("--pass-vocab", type=int, default=2048)
    ap.add_argument("--only-gemm", action="store_true", help="batched-row sweep of the tensor-core W4A16 contraction")
    ap.add_argument("--gemm-shapes", default="12288x4096,4096x4096,4096x12288,151936x4096")
    ap.add_argument("--gemm-rows", default="16,64,256,2048")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.prompt_len is None:
        args.prompt_len = PROMPT_LEN if args.gpus == 1 else PROMPT_LEN_MULTI
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
    tp = args.parallel == "tp" and n_gpus > 1
    # weights: rank 0 writes the reference's .bin set once; every rank loads its own part from it
    wdir = args.weights or os.path.join(tempfile.gettempdir(), f"qw3_bench_weights_{os.environ.get('MASTER_PORT', 'single')}_{os.getppid() if world > 1 else os.getpid()}")
    made = False
    if rank == 0 and not os.path.exists(os.path.join(wdir, "unembed_zp.bin")):
        orc.write_weight_dir(orc.default_config(), SEED, wdir)
        made = args.weights is None
    barrier()
    prompt = [int(t) for t in orc.gen_tokens(SEED, orc.TOKENS, args.prompt_len, 151936)]
    K, W, R = args.steps, args.warmup, args.repeats
    max_pos = args.prompt_len + W + (R + 2) * K + 8
    if world > 1 and tp:
        # one process per GPU, every matrix row-split over the GPUs; partial sums cross NVLink inside the pass kernel
        inf = pkg.QWen3AWQInfer(wdir, max_pos=max_pos, world=world, rank=rank, tensor_parallel=1, device=[local] * 8,
                                attn_split_min=args.attn_split_min)
        pipeline.connect_all(inf, dist)
    elif world > 1:
        # one process per GPU: this rank owns stage `rank`; hidden state and token id move by peer stores
        inf = pkg.QWen3AWQInfer(wdir, max_pos=max_pos, n_stages=world, world=world, rank=rank, device=list(range(world)))
        pipeline.connect_ring(inf, dist)
    else:
        inf = pkg.QWen3AWQInfer(wdir, max_pos=max_pos, n_stages=n_gpus, device=list(range(n_gpus)), attn_split_min=args.attn_split_min,
                                cluster=0 if args.no_cluster else 1)
    barrier()
    ids_all = inf.generateResponse(prompt, W)              # prompt pass + W warm-up decode steps
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    barrier()
    # device-timed: R regions of K decode steps, CUDA events inside the engine around this rank's decode loop
    region_ms, launches = [], 0
    for _ in range(R):
        ids_all += inf.decode_more(K)
        region_ms.append(inf.last_timing()[1])
        launches = inf.last_launches()
        barrier()
    # end to end: K more steps through the public API, host wall-clock, ids to host memory
    t0 = time.perf_counter()
    ids_all += inf.decode_more(K)
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    barrier()
    if rank == 0:
        clocks = sampler.stop()
    # end to end including the prompt: generateResponse(prompt, K) from host ids to host ids (prompt in blocks of rows
    # through the tensor-core contraction, as a serving caller would run it), and the reference's token loop beside it
    gen = {}
    try:
        inf.set_batched_prefill(True)
        inf.generateResponse(prompt, 1)                    # first use allocates the block buffers
        barrier()
        t0 = time.perf_counter()
        ids_gen = inf.generateResponse(prompt, K)
        torch.cuda.synchronize()
        gen["batched_s"] = time.perf_counter() - t0
        gen["batched_prompt_ms"] = inf.last_timing()[0]
        inf.set_batched_prefill(False)
        barrier()
        if not tp:
            t0 = time.perf_counter()
            ids_loop = inf.generateResponse(prompt, K)
            torch.cuda.synchronize()
            gen["loop_s"] = time.perf_counter() - t0
            gen["loop_prompt_ms"] = inf.last_timing()[0]
        else:
            ids_loop = ids_gen
        gen["ids_gen"], gen["ids_loop"] = ids_gen, ids_loop
    except Exception as exc:   # every device wait is bounded, so the other ranks come out as well
        sys.stderr.write(f"rank {rank}: generate timing failed: {exc}\n")
        gen = {"error": str(exc)}
    barrier()
    if world > 1:   # max over ranks of every time; launches summed; ids from the rank that samples
        t = torch.tensor(region_ms + [e2e_s, gen.get("batched_s", -1.0), gen.get("loop_s", -1.0), gen.get("batched_prompt_ms", -1.0),
                                      gen.get("loop_prompt_ms", -1.0), 1.0 if "error" in gen else 0.0], dtype=torch.float64, device=f"cuda:{local}")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        region_ms = [float(v) for v in t[:R]]
        e2e_s = float(t[R])
        if float(t[R + 5]) > 0:
            gen = {"error": gen.get("error", "failed on another rank")}
        else:
            gen.update(batched_s=float(t[R + 1]), loop_s=float(t[R + 2]), batched_prompt_ms=float(t[R + 3]), loop_prompt_ms=float(t[R + 4]))
        ln = torch.tensor([launches], dtype=torch.int64, device=f"cuda:{local}")
        dist.all_reduce(ln, op=dist.ReduceOp.SUM)
        launches = int(ln[0])
        n_ids = W + (R + 1) * K
        ids_all = pipeline.broadcast_ids(ids_all, n_ids, dist)
        if "error" not in gen:
            gen["ids_gen"] = pipeline.broadcast_ids(gen["ids_gen"], K, dist)
            gen["ids_loop"] = pipeline.broadcast_ids(gen["ids_loop"], K, dist)
    inf.close()
    result = None
    rc = 0
    if rank == 0:
        decode_ms = statistics.median(region_ms)
        ctx_mid = args.prompt_len + W + (R // 2) * K + K // 2
        tps = K / (decode_ms * 1e-3)
        peaks, peak_kind = measured_peaks()
        # parity of everything this run generated against the oracle's golden ids
        gname, gold = golden_ids(args.prompt_len)
        check = {"golden": gname, "ids_checked": 0, "ids_match_golden": None, "first_mismatch": None}
        if gold is not None:
            seqs = [("decode", ids_all)]
            if "error" not in gen:
                seqs += [("generate_batched_prompt", gen["ids_gen"]), ("generate_token_loop", gen["ids_loop"])]
            ok = True
            for name, ids in seqs:
                n = min(len(ids), len(gold))
                check["ids_checked"] += n
                for i in range(n):
                    if ids[i] != gold[i]:
                        ok = False
                        check["first_mismatch"] = check["first_mismatch"] or {"sequence": name, "step": i, "got": ids[i], "want": gold[i]}
                        break
            check["ids_match_golden"] = ok
            if not ok:
                rc = 3   # a run whose ids differ from the oracle's is not a measurement
        # the stand-alone GEMV operator (what a caller of qw3_gemv_w4a16 gets), reported beside the pass kernel
        M, Kd = 12288, 4096
        us, n_launch, us_pdl = roofline_gemv(pkg, torch, M, Kd, args.roofline_mats, args.roofline_reps)
        achieved = gemv_bytes(M, Kd) / (us * 1e-6) / 1e9
        gemv_roof = {"bound": "hbm", "kernel": "gemv_w4a16_kernel (12288x4096, STORE epilogue)", "achieved": achieved,
                     "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
                     "avg_launch_us": us, "avg_launch_us_with_pdl": us_pdl, "launches_timed": n_launch,
                     "bytes_per_launch": gemv_bytes(M, Kd), "l2": "36 distinct matrices cycled (906 MB > 126 MB L2)",
                     "ref_dequant_then_cublas_us": LAST_REF_GEMV_US}
        ref_us, ref_layer_us, ref_unemb_us, ref_how = reference_method_token_us(torch, orc, wdir)
        ref_method = {"what": "the reference's design on this GPU, contractions only: fp16 copies of the matrices of every layer and "
                              "of unembed, one cuBLAS call at n = 1 each (13.3 GB per token); no norms, attention, copies or host waits",
                      "how": ref_how, "us_per_token": ref_us, "us_per_layer": ref_layer_us, "unembed_us": ref_unemb_us,
                      "tokens_per_s_upper_bound": 1e6 / ref_us}
        decode_gbs = token_bytes(ctx_mid) * tps / 1e9
        par = "pp1" if n_gpus == 1 else (f"tp{n_gpus} (one process per GPU, matrices row-split, partial sums over NVLink)" if tp
                                         else f"pp{n_gpus}" + (" (one process per GPU, P2P hand-off)" if world > 1 else ""))
        e2e_gen = None
        if "error" not in gen:
            e2e_gen = {"value": K / gen["batched_s"], "unit": "tokens/s", "h2d_bytes_per_call": 4 * len(prompt), "d2h_bytes_per_call": 4 * K,
                       "wall_s": gen["batched_s"], "prompt_phase_ms": gen["batched_prompt_ms"],
                       "note": f"host wall-clock of generateResponse(prompt of {len(prompt)} ids in host memory, {K} new ids back in host memory); "
                               "prompt in blocks of rows through the tensor-core contraction",
                       "token_loop": None if tp else {"value": K / gen["loop_s"], "wall_s": gen["loop_s"], "prompt_phase_ms": gen["loop_prompt_ms"],
                                                      "note": "the same call with the reference's token-at-a-time prompt loop (set_batched_prefill(False))"}}
        line = {"metric": METRIC, "value": tps, "unit": "tokens/s", "n_gpus": n_gpus, "steps": K, "warmup": W,
                "ms_per_step": decode_ms / K, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                "dtype": "w4a16 (int4 weights, fp16 activations, fp32 accumulation)", "data": "synthetic",
                "config": {"workload": workload_string(args), "parallelism": par,
                           "l2": "3.3 GB of weights streamed per step (inputs larger than L2)",
                           "head_groups": ("global memory" if (n_gpus > 1 or args.no_cluster) else
                                           "thread-block clusters (Qw3Config.cluster = 1)")},
                "dtype_note": "the fused pass accumulates exactly in s32 on the integer tensor cores (fixed-point activations), fp32 in its epilogues",
                "timed_regions": {"repeats": R, "steps_each": K, "ms": region_ms, "median_ms": decode_ms,
                                  "spread": (max(region_ms) - min(region_ms)) / decode_ms},
                **check,
                # dominant kernel of the timed region: the token-pass kernel, one launch per token per GPU.  Its launch
                # duration is the CUDA-event time of a step (which also holds the 1-thread step_tail launch).
                "roofline": {"bound": "hbm", "kernel": "fused_pass_kernel (36 layers + unembed + arg-max, one launch per token)",
                             "achieved": decode_gbs, "peak": peaks["hbm_gbs"], "peak_kind": peak_kind + " (burst copy)",
                             "unit": "GB/s", "frac": decode_gbs / peaks["hbm_gbs"],
                             "traffic": int(token_bytes(ctx_mid) * NCU_TRAFFIC_RATIO), "bytes_per_launch": token_bytes(ctx_mid),
                             "avg_launch_us": decode_ms * 1e3 / K,
                             "traffic_note": NCU_TRAFFIC_NOTE,
                             "note": "N GPUs: value counts the whole job, achieved is the bytes of one token over the step time"},
                "gemv_roofline": gemv_roof, "reference_method_gpu": ref_method,
                "e2e": {"value": K / e2e_s, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 4,
                        "note": "host wall-clock of decode_more(K) through the C ABI; the sampled id feeds the next step on the device"},
                "e2e_generate": e2e_gen,
                "gpu_launches": int(launches), "clocks": clocks}
        if not args.no_cpu_baseline and n_gpus == 1:
            n_cpu = 8
            orc.set_num_threads(os.cpu_count() or 1)
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
        code = torch.tensor([rc], dtype=torch.int32, device=f"cuda:{local}")
        dist.all_reduce(code, op=dist.ReduceOp.MAX)
        rc = int(code[0])
        dist.destroy_process_group()
    if rc:
        raise SystemExit(rc)


if __name__ == "__main__":
    main()
