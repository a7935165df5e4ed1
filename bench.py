#!/usr/bin/env python
"""Benchmark of the DiT denoising step (Flux.1-dev architecture, 1024x1024, FP8 e4m3 per-tensor weights, bf16
activations, batch 1, random-init weights, synthetic inputs) on B200.

    python bench.py --gpus N --steps K --warmup W            # this library
    python bench.py --impl reference --steps K --warmup W     # the reference arithmetic on the host CPU cores

Prints ONE JSON line.  `value` = whole-job denoise steps/s with inputs resident in HBM (CUDA-graph replay of the
step, CUDA events, max over ranks); `e2e` = the same through `FluxDiTEngine.forward`-style host buffers (pinned
host -> device copies of every input and a device -> host read of the model output inside the timed region).
With N > 1 every rank denoises its own latent (independent replicas, weak scaling, no data-path collective).
By default the line also carries, under "wan", the Wan2.1-14B-architecture 480p step run sequence-parallel
(Ulysses) over the same N GPUs on ONE video (strong scaling); `--workload flux|wan` runs one of the two.
"""
import argparse
import importlib
import importlib.util
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
PKG_DIR = os.path.join(ROOT, "diffsynth-engine_b200")
sys.path.insert(0, ROOT)

FLUX = dict(d=3072, H=24, n_double=19, n_single=38, S_txt=512, height=128, width=128, txt_dim=4096, pooled_dim=768)
# Qwen-Image-architecture stand-in (the reference snapshot has no Qwen-Image code): 60 Flux-style double-stream
# blocks, 1328x1328 -> latent 166x166 -> 83*83 = 6889 image tokens + 256 text tokens of width 3584
QWEN = dict(d=3072, H=24, n_double=60, n_single=0, S_txt=256, height=166, width=166, txt_dim=3584, pooled_dim=768)
# Wan2.1-14B text-to-video at 81 frames x 480 x 832: latent 21 x 60 x 104, patch (1,2,2) -> 21*30*52 = 32760 tokens
WAN = dict(d=5120, ffn=13824, num_layers=40, H=40, frames=21, height=60, width=104, ctx=512, text_dim=4096)


def load_package():
    name = "diffsynth_engine_b200"
    if name not in sys.modules:
        spec = importlib.util.spec_from_file_location(name, os.path.join(PKG_DIR, "__init__.py"),
                                                      submodule_search_locations=[PKG_DIR])
        mod = importlib.util.module_from_spec(spec)
        sys.modules[name] = mod
        spec.loader.exec_module(mod)
    return sys.modules[name]


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm_gbs=p["hbm_gbs"], bf16=p["bf16_tflops"], bf16_sustained=p.get("bf16_tflops_sustained"),
                    source="measured")
    return dict(hbm_gbs=6650.0, bf16=1590.0, bf16_sustained=1400.0, source="fallback")


def flux_step_flops(c=FLUX):
    """Algorithmic work of one step: 2MKN per Linear on token rows, 4*S^2*H*D per attention."""
    d, St, Si = c["d"], c["S_txt"], (c["height"] // 2) * (c["width"] // 2)
    S = St + Si
    lin_double = 2 * S * d * (3 * d + d + 4 * d + 4 * d)
    lin_single = 2 * S * d * (7 * d + 5 * d)
    lin = c["n_double"] * lin_double + c["n_single"] * lin_single
    lin += 2 * St * c["txt_dim"] * d + 2 * Si * 64 * d * 2
    attn = (c["n_double"] + c["n_single"]) * 4 * S * S * d
    return lin, attn


# ------------------------------------------------------------------------------------ clocks
class ClockSampler:
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index=0):
        self.gpu_index, self.rows, self.proc, self.thread = gpu_index, [], None, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.gpu_index)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return self
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) < 9:
                continue
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
            except ValueError:
                continue
            for name, val in zip(names, r[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=[], samples=0)
        return dict(sm_mhz=statistics.median(sm), sm_max_mhz=max(mx), reasons=sorted(reasons), samples=len(sm))


# ------------------------------------------------------------------------- CPU arm (oracle port)
def cpu_reference_arm(steps=1, warmup=0, budget_s=150.0):
    """The reference's arithmetic on the host cores: the fp32 PyTorch restatement of one double-stream and one
    single-stream block (oracle/flux.py) at the full sequence length, extrapolated by the block counts."""
    import torch
    from oracle import flux as OF
    from oracle import ops as O
    from oracle.linear import LinearEval
    load_package()
    synth = importlib.import_module("diffsynth_engine_b200.synth")
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    c = FLUX
    d, H = c["d"], c["H"]
    St, side = c["S_txt"], c["height"] // 2
    wd = synth.make_state_dict(synth.flux_block_shapes("", d, H, "double"), seed=0)
    ws = synth.make_state_dict(synth.flux_block_shapes("", d, H, "single"), seed=1)
    xa, xb, temb = synth.randn((side * side, d), 2), synth.randn((St, d), 3), synth.randn((d,), 4)
    table = O.flux_rope_table(torch.cat([torch.zeros(St, 3), OF.image_ids(c["height"], c["width"])]))
    lin = LinearEval("fp32")
    times, t_start = [], time.time()
    with torch.no_grad():
        for i in range(warmup + steps):
            if times and time.time() - t_start > budget_s:
                break
            t0 = time.time()
            OF.double_block(xa, xb, temb, table, wd, "", H, lin)
            t1 = time.time()
            OF.single_block(torch.cat([xb, xa]), temb, table, ws, "", H, lin)
            t2 = time.time()
            if i >= warmup or (warmup + steps) == 1:
                times.append((t1 - t0, t2 - t1))
    td = statistics.mean(t[0] for t in times)
    tsg = statistics.mean(t[1] for t in times)
    step_s = c["n_double"] * td + c["n_single"] * tsg
    return dict(value=1.0 / step_s, unit="steps/s", cores=cores, kind="port",
                sample=(f"1 double-stream + 1 single-stream block at S=512+4096, fp32, {cores} threads "
                        f"({td:.2f}s + {tsg:.2f}s, mean of {len(times)}), extrapolated x19 / x38; embedders and "
                        f"final layer (<0.1% of the work) left out"),
                ms_per_step=step_s * 1e3, samples=len(times))


def wan_step_flops(c=WAN):
    S, d, L = c["frames"] * (c["height"] // 2) * (c["width"] // 2), c["d"], c["num_layers"]
    lin = L * (2 * S * d * (8 * d + 2 * c["ffn"]) + 2 * c["ctx"] * d * 2 * d)
    attn = L * (4 * S * S * d + 4 * S * c["ctx"] * d)
    return lin, attn


def run_wan(args, torch, pkg, synth, dev, dist, rank, world, steps, warmup):
    """Wan2.1-14B-architecture step, sequence-parallel (Ulysses) over all ranks: ONE video, strong scaling."""
    wan = importlib.import_module("diffsynth_engine_b200.wan")
    c = dict(WAN)
    if args.wan_layers:
        c["num_layers"] = args.wan_layers
    shapes = synth.wan_dit_shapes(d=c["d"], ffn=c["ffn"], num_layers=c["num_layers"], text_dim=c["text_dim"])
    sd = synth.make_state_dict(shapes, seed=1234, device=dev, dtype=torch.bfloat16)   # same weights on every rank
    eng = wan.WanDiTEngine(sd, fmt=args.wan_fmt, device=dev, num_layers=c["num_layers"], num_heads=c["H"],
                           group=(dist.group.WORLD if dist is not None else None), release_source=True)
    del sd
    torch.cuda.empty_cache()
    eng.prepare(c["frames"], c["height"], c["width"], c["ctx"], c["text_dim"])
    h_x = synth.randn((1, 16, c["frames"], c["height"], c["width"]), 7).bfloat16().pin_memory()
    h_ctx = synth.randn((1, c["ctx"], c["text_dim"]), 8).bfloat16().pin_memory()
    h_t = torch.tensor([500.0]).pin_memory()
    h_out = torch.empty((1, 16, c["frames"], c["height"], c["width"]), dtype=torch.bfloat16).pin_memory()

    def sync():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    eng.set_inputs(h_x, h_ctx, h_t)
    n0 = pkg._lib.launches
    for _ in range(max(1, warmup)):
        eng.step()
    launches = (pkg._lib.launches - n0) // max(1, warmup)
    sync()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        eng.step()
    e1.record()
    sync()
    ms = e0.elapsed_time(e1) / steps
    e0.record()
    for _ in range(steps):
        eng.set_inputs(h_x, h_ctx, h_t)
        out = eng.step()
        if rank == 0:
            h_out.copy_(out, non_blocking=True)
        torch.cuda.current_stream().synchronize()
    e1.record()
    sync()
    ms_e2e = e0.elapsed_time(e1) / steps
    if dist is not None:
        t = torch.tensor([ms, ms_e2e], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, ms_e2e = float(t[0]), float(t[1])
    pkg.ops.check_status(dev.index)
    lin_f, attn_f = wan_step_flops(c)
    peaks = measured_peaks()
    fp8 = args.wan_fmt != "bf16"
    roof_ms = (lin_f / (peaks["bf16"] * (2 if fp8 else 1) * 1e12) + attn_f / (peaks["bf16"] * 1e12)) * 1e3
    return {"workload": f"wan2.1-14B-arch t2v DiT step, 81x480x832 (32760 tokens, 512 context tokens), batch 1, "
                        f"{c['num_layers']} blocks, weights {args.wan_fmt}, Ulysses sequence parallel x{world}",
            "steps_per_s": 1e3 / ms, "ms_per_step": ms, "e2e_steps_per_s": 1e3 / ms_e2e, "e2e_ms_per_step": ms_e2e,
            "n_gpus": world, "scaling": "strong", "step_tflop": (lin_f + attn_f) / 1e12,
            "frac_of_roofline_all_gpus": roof_ms / (ms * world), "gpu_launches_per_step": launches,
            "h2d_bytes_per_step": sum(t.numel() * t.element_size() for t in (h_x, h_ctx, h_t)),
            "d2h_bytes_per_step": h_out.numel() * h_out.element_size()}


def run_sweeps(torch, pkg, dev):
    """Isolated kernel sweeps: FP8 e4m3 Linear (per-tensor and per-channel weight scale, bf16 out, fused
    bias + GELU-tanh) and joint attention (bf16, head_dim 128), N(0,1) values from a seed."""
    ops = pkg.ops
    peaks = measured_peaks()
    gen = torch.Generator(device=dev).manual_seed(0)

    def timeit(fn, n=10, warm=3):
        time.sleep(0.3)     # let the board leave its power cap: each case is timed as an isolated burst
        for _ in range(warm):
            fn()
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(n):
            fn()
        e.record()
        torch.cuda.synchronize()
        return s.elapsed_time(e) / n

    linear, attn = [], []
    for (K, N) in [(3072, 3072), (3072, 12288), (12288, 3072), (5120, 13824), (3072, 9216)]:
        w = torch.randn(N, K, generator=gen, device=dev) * 0.02
        bias = torch.randn(N, generator=gen, device=dev) * 0.02
        packs = {"per_tensor": ops.pack_quant_weight(w, ops.FMT_E4M3, False),
                 "per_channel": ops.pack_quant_weight(w, ops.FMT_E4M3, True)}
        for M in (1024, 4096, 8192, 32760):
            x = torch.randn(M, K, generator=gen, device=dev).to(torch.bfloat16)
            xq, rs = ops.quant_rows(x)
            out = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
            for mode, (wq, ws) in packs.items():
                ms = timeit(lambda: ops.gemm(xq, wq, row_scale=rs, col_scale=ws, bias=bias, act=ops.ACT_GELU_TANH,
                                             out=out))
                tf = 2.0 * M * N * K / ms / 1e9
                linear.append({"M": M, "K": K, "N": N, "scale": mode, "us": ms * 1e3, "tflops": tf,
                               "frac_of_2x_bf16_peak": tf / (2 * peaks["bf16"])})
    for H in (24, 40):
        for S in (1536, 4608, 7145, 32760):
            q, k, v = (torch.randn(1, S, H, 128, generator=gen, device=dev).to(torch.bfloat16) for _ in range(3))
            o = torch.empty_like(q)
            ms = timeit(lambda: ops.flash_attn(q, k, v, out=o), n=5 if S > 8192 else 10)
            tf = 4.0 * S * S * H * 128 / ms / 1e9
            attn.append({"H": H, "S": S, "us": ms * 1e3, "tflops": tf, "frac_of_bf16_peak": tf / peaks["bf16"]})
    ops.check_status(dev.index)
    return {"metric": "isolated kernel sweeps", "unit": "TFLOP/s", "data": "synthetic",
            "peak_source": f"MEASURED_PEAKS.json ({peaks['source']}): bf16 {peaks['bf16']} TFLOP/s; FP8 taken as 2x",
            "fp8_linear_bias_gelu": linear, "joint_attention": attn}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--fmt", default="fp8_tensor")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--blocks", default=None, help="n_double,n_single override (reduced-depth debugging; not a bench)")
    ap.add_argument("--workload", default="both", choices=["flux", "wan", "both", "qwen", "sweeps"],
                    help="flux: the headline line; wan: Wan-14B sequence-parallel step only; both: flux line with the "
                         "wan result attached under 'wan'")
    ap.add_argument("--wan-fmt", default="fp8_channel")
    ap.add_argument("--wan-layers", type=int, default=0, help="reduced depth (debugging; not a bench)")
    ap.add_argument("--wan-steps", type=int, default=2)
    ap.add_argument("--sp", action="store_true",
                    help="flux/qwen workloads under torchrun: ONE image, its token sequence split over all ranks (Ulysses, "
                         "strong scaling) instead of one replica per GPU")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    cfg = dict(QWEN if args.workload == "qwen" else FLUX)
    if args.blocks:
        cfg["n_double"], cfg["n_single"] = (int(v) for v in args.blocks.split(","))
    if args.workload == "qwen":
        wl = ("qwen-image-arch stand-in (Flux-style double-stream blocks), 1328x1328 (6889 image + 256 text tokens of "
              f"width 3584), batch 1, {cfg['n_double']} double blocks, weights {args.fmt}, bf16 activations")
    else:
        wl = ("flux1-dev-arch DiT step, 1024x1024 (4096 image + 512 text tokens), batch 1, "
              f"{cfg['n_double']} double + {cfg['n_single']} single blocks, weights {args.fmt}, bf16 activations")
    sp = args.sp and world > 1
    config = {"workload": wl,
              "parallelism": (f"sp{world} (Ulysses, one image)" if sp else f"replicas x{world}") if world > 1
              else "single GPU",
              "l2": "per-step working set (11.9 GB of weights) exceeds the 126 MB L2; no flush between steps"}

    if args.impl == "reference":
        if rank != 0:
            return
        r = cpu_reference_arm(steps=max(1, args.steps), warmup=args.warmup)
        line = {"impl": "reference", "metric": "DiT denoise steps/s", "value": r["value"], "unit": "steps/s",
                "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": r["ms_per_step"],
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp32", "data": "synthetic",
                "config": config, "cpu_baseline": {k: r[k] for k in ("value", "unit", "cores", "kind", "sample")},
                "e2e": {"value": r["value"], "unit": "steps/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(line), flush=True)
        return

    import torch
    pkg = load_package()
    ops = pkg.ops
    synth = importlib.import_module("diffsynth_engine_b200.synth")
    flux = importlib.import_module("diffsynth_engine_b200.flux")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device(f"cuda:{local_rank}")
    dist = None
    if world > 1:
        if os.environ.get("NCCL_DEBUG", "").upper() == "VERSION":
            os.environ["NCCL_DEBUG"] = "WARN"   # keep NCCL's version banner off stdout: one JSON line only
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    if args.workload == "sweeps":
        if rank == 0:
            print(json.dumps(run_sweeps(torch, pkg, dev)), flush=True)
        return
    if args.workload == "wan":
        r = run_wan(args, torch, pkg, synth, dev, dist, rank, world, max(1, args.steps), max(1, min(args.warmup, 3)))
        if rank == 0:
            line = {"metric": "DiT denoise steps/s", "value": r["steps_per_s"], "unit": "steps/s", "n_gpus": world,
                    "steps": args.steps, "warmup": max(1, min(args.warmup, 3)), "ms_per_step": r["ms_per_step"],
                    "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                    "dtype": "fp8_e4m3 linear, bf16 attention" if args.wan_fmt != "bf16" else "bf16",
                    "data": "synthetic", "config": {"workload": r["workload"], "parallelism": f"sp{world}"},
                    "e2e": {"value": r["e2e_steps_per_s"], "unit": "steps/s",
                            "h2d_bytes_per_step": r["h2d_bytes_per_step"], "d2h_bytes_per_step": r["d2h_bytes_per_step"]},
                    "gpu_launches": r["gpu_launches_per_step"] * args.steps, "wan": r}
            print(json.dumps(line), flush=True)
        if dist is not None:
            dist.barrier()
            dist.destroy_process_group()
        return

    # random-init weights of the architecture, drawn on the device, packed to FP8 layer by layer
    shapes = synth.flux_dit_shapes(d=cfg["d"], H=cfg["H"], n_double=cfg["n_double"], n_single=cfg["n_single"],
                                   txt_dim=cfg["txt_dim"], pooled_dim=cfg["pooled_dim"])
    seed = 0 if sp else rank            # sequence parallel: every rank holds the same model and the same inputs
    sd = synth.make_state_dict(shapes, seed=seed, device=dev, dtype=torch.bfloat16)
    eng = flux.FluxDiTEngine(sd, fmt=args.fmt, device=dev, n_double=cfg["n_double"], n_single=cfg["n_single"],
                             num_heads=cfg["H"], release_source=True, group=dist.group.WORLD if sp else None)
    del sd
    torch.cuda.empty_cache()
    eng.prepare(cfg["S_txt"], cfg["height"], cfg["width"], cfg["txt_dim"], cfg["pooled_dim"])
    # inputs on the host (pinned), as a pipeline would hold them between steps
    h_lat = synth.randn((1, 16, cfg["height"], cfg["width"]), 100 + seed).bfloat16().pin_memory()
    h_pe = synth.randn((1, cfg["S_txt"], cfg["txt_dim"]), 200 + seed).bfloat16().pin_memory()
    h_pool = synth.randn((1, cfg["pooled_dim"]), 300 + seed).pin_memory()
    h_t, h_g = torch.tensor([500.0]).pin_memory(), torch.tensor([3.5]).pin_memory()
    h_out = torch.empty((1, 16, cfg["height"], cfg["width"]), dtype=torch.bfloat16).pin_memory()
    h2d = sum(t.numel() * t.element_size() for t in (h_lat, h_pe, h_pool, h_t, h_g))
    d2h = h_out.numel() * h_out.element_size()
    eng.set_inputs(h_lat, h_t, h_pe, h_pool, h_g)
    n0 = pkg._lib.launches
    eng.step()
    launches_per_step = pkg._lib.launches - n0
    torch.cuda.synchronize()
    ops.check_status(local_rank)
    eng.capture()

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        if dist is None:
            return ms
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- device-resident throughput
    for _ in range(max(3, args.warmup)):
        eng.step()
    sampler = ClockSampler(local_rank).start() if rank == 0 else None
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.profiler.start()  # lets `ncu --profile-from-start off` see exactly the timed region
    e0.record()
    for _ in range(args.steps):
        eng.step()
    e1.record()
    barrier()
    torch.cuda.profiler.stop()
    ms_total = max_over_ranks(e0.elapsed_time(e1))
    clocks = sampler.stop() if sampler else None
    ms_per_step = ms_total / args.steps
    value = (1 if sp else world) * 1e3 / ms_per_step

    # ---- end to end: host buffers in, host buffer out, every step
    def e2e_step():
        eng.set_inputs(h_lat, h_t, h_pe, h_pool, h_g)
        out = eng.step()
        h_out.copy_(out, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    for _ in range(3):
        e2e_step()
    barrier()
    t0 = time.perf_counter()
    e0.record()
    for _ in range(args.steps):
        e2e_step()
    e1.record()
    barrier()
    e2e_ms = max_over_ranks(max(e0.elapsed_time(e1), 0.0)) / args.steps
    e2e_wall_ms = (time.perf_counter() - t0) * 1e3 / args.steps
    ops.check_status(local_rank)

    # ---- roofline of the dominant kernel (the FP8 GEMM): CUDA events around every launch of one eager step
    peaks = measured_peaks()
    recs = []
    real_gemm, real_gemm_qkv, real_group = ops.gemm, ops.gemm_qkv, ops.gemm_group

    def timed(fn, grouped=False):
        def wrapper(a, *rest, **kw):
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            r = fn(a, *rest, **kw)
            e.record()
            probs = a if grouped else [dict(a=a, w=rest[0])]
            recs.append((sum(2.0 * p["a"].shape[0] * p["a"].shape[1] * p["w"].shape[0] for p in probs), s, e))
            return r
        return wrapper

    eng._graph_saved, eng._graph = eng._graph, None
    # all three entry points launch gemm_kernel (a grouped launch runs two problems in one persistent grid)
    ops.gemm, ops.gemm_qkv, ops.gemm_group = timed(real_gemm), timed(real_gemm_qkv), timed(real_group, True)
    try:
        eng.step()
        torch.cuda.synchronize()
    finally:
        ops.gemm, ops.gemm_qkv, ops.gemm_group = real_gemm, real_gemm_qkv, real_group
        eng._graph = eng._graph_saved
    gemm_flops = sum(r[0] for r in recs)
    gemm_ms = sum(r[1].elapsed_time(r[2]) for r in recs)
    fp8 = args.fmt != "bf16"          # any 8-bit weight format: the tensor pipe runs at twice the bf16 rate
    int8 = args.fmt.startswith("int8")
    kind = "int8" if int8 else "fp8"
    peak_tf = peaks["bf16"] * (2.0 if fp8 else 1.0)
    ach_tf = gemm_flops / (gemm_ms * 1e-3) / 1e12
    lin_f, attn_f = flux_step_flops(cfg)
    roofline = {"kernel": f"gemm_kernel<{kind}> (256x256 CTA-pair tiles; 128x128 for the text stream)" if fp8
                else "gemm_kernel<bf16>", "bound": "tensor",
                "achieved": ach_tf, "peak": peak_tf, "unit": "TFLOP/s", "frac": ach_tf / peak_tf,
                # DRAM read+write bytes per GEMM launch: ncu capture of the 1+1-block case scaled by the block counts to the
                # step's 30.8 GB of GEMM traffic, over this step's GEMM launches
                # (the ncu summary of per-kernel DRAM traffic under profiles/); only meaningful for the full 19+38-block FP8 model
                "traffic": (30.8e9 / max(1, len(recs)) if (fp8 and not int8 and not args.blocks and args.workload != "qwen" and not sp) else None),
                "peak_source": (f"2 x bf16_tflops of MEASURED_PEAKS.json ({peaks['source']}); no 8-bit peak was measured"
                                if fp8 else f"bf16_tflops of MEASURED_PEAKS.json ({peaks['source']})"),
                "launches_per_step": len(recs), "gemm_ms_per_step": gemm_ms,
                "method": "CUDA events around each GEMM launch of one eager (un-graphed) step; 2MNK per launch",
                "step_tflop": (lin_f + attn_f) / 1e12,
                "step_frac_of_roofline": ((lin_f / (peak_tf * 1e12) + attn_f / (peaks["bf16"] * 1e12)) * 1e3) / (ms_per_step * (world if sp else 1))}

    line = {"metric": "DiT denoise steps/s", "value": value, "unit": "steps/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(3, args.warmup), "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong" if sp else "weak",
            "vs_baseline": None,
            "dtype": ("int8 x int8 -> int32 (linear), bf16 (attention)" if int8
                      else "fp8_e4m3 x fp8_e4m3 -> fp32 (linear), bf16 (attention)" if fp8 else "bf16"),
            "data": "synthetic", "config": config, "clocks": clocks,
            "e2e": {"value": (1 if sp else world) * 1e3 / e2e_ms, "unit": "steps/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms, "wall_ms_per_step": e2e_wall_ms},
            "gpu_launches": launches_per_step * args.steps, "gpu_launches_per_step": launches_per_step,
            "roofline": roofline}
    if args.workload == "both":
        del eng
        torch.cuda.empty_cache()
        line["wan"] = run_wan(args, torch, pkg, synth, dev, dist, rank, world, args.wan_steps, 1)
    if rank == 0:
        if not args.no_cpu_baseline and world == 1:
            r = cpu_reference_arm(steps=1, warmup=0)
            line["cpu_baseline"] = {k: r[k] for k in ("value", "unit", "cores", "kind", "sample")}
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
