#!/usr/bin/env python
"""Benchmark of the DiT denoising step on B200 (random-init weights of the architecture, synthetic inputs).

    python bench.py --gpus N --steps K --warmup W            # this library
    python bench.py --impl reference --steps K --warmup W     # the reference arithmetic on the host CPU cores

Prints ONE JSON line.  The headline (`value`) is the Wan2.1-14B-architecture 480p step (81 frames x 480 x 832 ->
32760 tokens, 40 blocks, FP8 e4m3 per-channel weights, bf16 activations, batch 1) run sequence-parallel (Ulysses)
over the N GPUs on ONE video: strong scaling, `value` = whole-job denoise steps/s with inputs resident in HBM (CUDA
events, max over ranks), `e2e` = the same through host buffers (pinned host -> device copies of every input and a
device -> host read of the model output inside the timed region).  At N = 1 the line also carries, under "flux", the
Flux.1-dev-architecture step at 1024 x 1024 (19 + 38 blocks, FP8 per-tensor weights) with its own roofline entry.
`parity` holds correctness checks made outside the timed region: finiteness of the timed output, a reduced-depth
model at full width against the CPU oracle, and (N > 1) the sequence-parallel output against a one-GPU run.
`--workload flux|wan|qwen|sweeps` runs one of the single workloads.
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
# the CPU arm's sample of the Wan step: one block on the first 1023 tokens as queries against all 32760 keys
WAN_CPU_ROWS = 1023   # about 1/32 of the sequence: the sample is 1023 / 32760 of one of the 40 blocks


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
        return dict(hbm_gbs=p["hbm_gbs"], bf16=p["bf16_tflops"],
                    bf16_sustained=p.get("bf16_tflops_sustained") or p["bf16_tflops"], source="measured")
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


def wan_step_flops(c=WAN):
    """Per block: six d x d Linears (self q, k, v, o; cross q, o) and the two FFN Linears on all S tokens, the
    cross-attention k and v Linears on the context tokens; self-attention 4*S^2*d, cross-attention 4*S*ctx*d."""
    S, d, L = c["frames"] * (c["height"] // 2) * (c["width"] // 2), c["d"], c["num_layers"]
    lin = L * (2 * S * d * (6 * d + 2 * c["ffn"]) + 2 * c["ctx"] * d * 2 * d)
    attn = L * (4 * S * S * d + 4 * S * c["ctx"] * d)
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
def cpu_wan_arm(steps=1, warmup=0, budget_s=900.0):
    """The reference's arithmetic on the host cores, as the fp32 PyTorch restatement of one Wan DiTBlock
    (oracle/wan.py) evaluated the way one member of a sequence-parallel group evaluates it: WAN_CPU_ROWS tokens as
    queries (all token-wise work on them) against the keys and values of all 32760 tokens.  One such evaluation is
    one "step" of this arm; it is rows / 32760 of one of the 40 blocks, and the denoise-step rate is extrapolated
    from it (the full step is 1678 TFLOP, about an hour of CPU time)."""
    import torch
    from oracle import ops as O
    from oracle import wan as OW
    from oracle.linear import LinearEval
    load_package()
    synth = importlib.import_module("diffsynth_engine_b200.synth")
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    c = WAN
    d, H, rows = c["d"], c["H"], WAN_CPU_ROWS
    S = c["frames"] * (c["height"] // 2) * (c["width"] // 2)
    w = synth.make_state_dict(synth.wan_block_shapes("", d, c["ffn"]), seed=0)
    x, ctx, tmod = synth.randn((rows, d), 1), synth.randn((c["ctx"], d), 2), synth.randn((6, d), 3) * 0.1
    other = (synth.randn((S - rows, d), 4), synth.randn((S - rows, d), 5))
    table = O.wan_rope_table(c["frames"], c["height"] // 2, c["width"] // 2)[:rows]
    lin = LinearEval("fp32")
    times, t_start = [], time.time()
    with torch.no_grad():
        for i in range(warmup + steps):
            if times and time.time() - t_start > budget_s:
                break
            t0 = time.time()
            OW.wan_block(x, ctx, tmod, table, w, "", H, lin, other_kv=other)
            if i >= warmup or (warmup + steps) == 1:
                times.append(time.time() - t0)
    t_sample = statistics.mean(times)
    fraction = rows / S / c["num_layers"]
    step_s = t_sample / fraction
    check = _reference_module_check(torch, synth, OW, O, lin, w, c, rows)
    return dict(value=1.0 / step_s, unit="steps/s", cores=cores, kind="port", reference_module_check=check,
                sample=(f"one Wan DiTBlock (oracle port, fp32, {cores} threads) on {rows} tokens as queries against all "
                        f"{S} keys = {fraction:.3e} of a step; {t_sample:.2f} s each (mean of {len(times)}), "
                        f"extrapolated to the 40-block, {S}-token step; embedders and head (<0.1% of the work) left out"),
                sample_ms=t_sample * 1e3, sample_fraction=fraction, samples=len(times))


def _reference_module_check(torch, synth, OW, O, lin, w, c, rows):
    """That the port is a fair stand-in for the reference on these cores: the reference's own ``DiTBlock``
    (models/wan/wan_dit.py:155-193, unmodified, from baseline/_ref, fp32) and the port on the same ``rows``-token
    problem - time of each and the rel-L2 between their outputs.  None when baseline/_ref is not installed."""
    try:
        sys.path.insert(0, os.path.join(ROOT, "baseline"))
        import install_reference
        ref = install_reference.import_reference()
        if ref is None:
            return None
        d, H = c["d"], c["H"]
        fr, hh, ww = 3, 11, rows // 33
        n = fr * hh * ww
        blk = ref.wan_dit.DiTBlock(False, d, H, c["ffn"], 1e-6, device="cpu", dtype=torch.float32)
        torch.nn.Module.load_state_dict(blk, w, strict=True)
        blk.eval()
        f_, h_, w_ = ref.wan_dit.precompute_freqs_cis_3d(d // H)
        freqs = torch.cat([f_[:fr].view(fr, 1, 1, -1).expand(fr, hh, ww, -1), h_[:hh].view(1, hh, 1, -1).expand(fr, hh, ww, -1),
                           w_[:ww].view(1, 1, ww, -1).expand(fr, hh, ww, -1)], dim=-1).reshape(n, 1, -1)
        x, ctx, tmod = synth.randn((1, n, d), 11), synth.randn((1, c["ctx"], d), 12), synth.randn((1, 6, d), 13) * 0.1
        with torch.no_grad():
            t0 = time.time()
            y_ref = blk(x, ctx, tmod, freqs)
            t_ref = time.time() - t0
            t0 = time.time()
            y_port = OW.wan_block(x[0], ctx[0], tmod[0], O.wan_rope_table(fr, hh, ww), w, "", H, lin)
            t_port = time.time() - t0
        return {"tokens": n, "reference_DiTBlock_s": t_ref, "port_s": t_port,
                "rel_l2_port_vs_reference": float((y_port - y_ref[0]).norm() / y_ref[0].norm())}
    except Exception as e:   # a baseline, not a gate: report instead of failing the arm
        return {"error": f"{type(e).__name__}: {str(e)[:160]}"}


def cpu_flux_arm(steps=1, warmup=0, budget_s=900.0):
    """Flux: the fp32 restatement of one double-stream and one single-stream block (oracle/flux.py) at the full
    sequence length, extrapolated by the block counts."""
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
                sample_ms=(td + tsg) * 1e3, sample_fraction=(td + tsg) / step_s, samples=len(times))


# --------------------------------------------------------------------------------------- helpers
class Ctx:
    """What every workload needs: torch, the package, the device, the process group and the timing helpers."""

    def __init__(self, torch, pkg, dev, dist, rank, world, local_rank):
        self.torch, self.pkg, self.dev, self.dist = torch, pkg, dev, dist
        self.rank, self.world, self.local_rank = rank, world, local_rank
        self.synth = importlib.import_module("diffsynth_engine_b200.synth")

    def barrier(self):
        self.torch.cuda.synchronize()
        if self.dist is not None:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, *vals):
        if self.dist is None:
            return vals if len(vals) > 1 else vals[0]
        t = self.torch.tensor(list(vals), device=self.dev, dtype=self.torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        out = [float(v) for v in t]
        return out if len(out) > 1 else out[0]

    def timed_steps(self, fn, steps):
        """`steps` calls of fn between two CUDA events on the current stream, barrier + synchronize on both sides;
        returns the mean milliseconds per call, max over ranks."""
        torch = self.torch
        self.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        self.barrier()
        return self.max_over_ranks(e0.elapsed_time(e1)) / steps


def timed_launches(ctx, module, names, run):
    """Runs `run()` once with the named functions of `module` wrapped in CUDA events; returns [(name, args, ms)]."""
    torch = ctx.torch
    recs, saved = [], {n: getattr(module, n) for n in names}

    def wrap(name, fn):
        def inner(*a, **kw):
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            r = fn(*a, **kw)
            e.record()
            recs.append((name, a, kw, s, e))
            return r
        return inner

    for n, fn in saved.items():
        setattr(module, n, wrap(n, fn))
    try:
        run()
        torch.cuda.synchronize()
    finally:
        for n, fn in saved.items():
            setattr(module, n, fn)
    return [(n, a, kw, s.elapsed_time(e)) for n, a, kw, s, e in recs]


def library_fp8_gemm_tflops(torch, dev):
    """cuBLASLt's FP8 GEMM (torch._scaled_mm, the kernel the reference's FP8 Linear calls, utils/fp8_linear.py:41)
    on 8192^3, best of 5: printed next to the assumed 8-bit peak so the assumption can be read against a
    measurement of this run.  None if the call is unavailable."""
    try:
        n = 8192
        a = torch.randn(n, n, device=dev).to(torch.float8_e4m3fn)
        b = torch.randn(n, n, device=dev).to(torch.float8_e4m3fn)
        one = torch.tensor(1.0, device=dev)
        best = None
        for _ in range(6):
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            torch._scaled_mm(a, b.t(), scale_a=one, scale_b=one, out_dtype=torch.bfloat16)
            e.record()
            torch.cuda.synchronize()
            ms = s.elapsed_time(e)
            best = ms if best is None else min(best, ms)
        return 2.0 * n ** 3 / best / 1e9
    except Exception:
        return None


# ------------------------------------------------------------------------------------------- Wan
def wan_parity(ctx, args):
    """Correctness evidence for the Wan path, outside any timed region.
    (1) N = 1 only: a 1-block model at full width on a 21 x 15 x 13 token grid (4095 tokens, the share of one
        of eight ranks) against the CPU oracle with the same quantisation: rel-L2 of the hidden state after the block
        and of the block's update;
    (2) N > 1: a 2-block model at full width on the FULL video, sequence-parallel over all ranks, against the same
        model run on rank 0 alone."""
    torch, synth, dev = ctx.torch, ctx.synth, ctx.dev
    wan = importlib.import_module("diffsynth_engine_b200.wan")
    c = WAN
    out = {}
    shapes = synth.wan_dit_shapes(d=c["d"], ffn=c["ffn"], num_layers=2, text_dim=c["text_dim"])
    sd = synth.make_state_dict(shapes, seed=77, device=dev, dtype=torch.bfloat16)
    x = synth.randn((1, 16, c["frames"], c["height"], c["width"]), 78).bfloat16()
    ctxt = synth.randn((1, c["ctx"], c["text_dim"]), 79).bfloat16()
    t = torch.tensor([417.0])
    if ctx.world > 1:
        # (a) the sequence-parallel dataflow with every attention row evaluated in one piece: the same arithmetic as
        # one GPU, so the comparison is exact; (b) the timed configuration, whose attention kernel may cut the items of
        # a partly filled last wave along the keys: those rows differ in fp32 summation order, and two blocks of FP8
        # arithmetic amplify that to the reproducibility floor of the arithmetic (see the one-GPU run's
        # oracle_vs_reordered_oracle figure: about 1.2e-2 per block)
        eng = wan.WanDiTEngine(dict(sd), fmt=args.wan_fmt, device=dev, num_layers=2, num_heads=c["H"],
                               group=ctx.dist.group.WORLD, exchange=args.wan_exchange, tail_split=False)
        y_sp = eng(x.to(dev), ctxt.to(dev), t.to(dev)).float()
        exch = eng.exchange
        del eng
        y_cut = None
        if exch == "peer" and args.wan_tail_split == "on":
            eng = wan.WanDiTEngine(dict(sd), fmt=args.wan_fmt, device=dev, num_layers=2, num_heads=c["H"],
                                   group=ctx.dist.group.WORLD, exchange=args.wan_exchange, tail_split=True)
            y_cut = eng(x.to(dev), ctxt.to(dev), t.to(dev)).float()
            del eng
        if ctx.rank == 0:
            one = wan.WanDiTEngine(dict(sd), fmt=args.wan_fmt, device=dev, num_layers=2, num_heads=c["H"])
            y_1 = one(x.to(dev), ctxt.to(dev), t.to(dev)).float()
            del one
            out["sp_vs_one_gpu_rel_l2"] = float((y_sp - y_1).norm() / y_1.norm())
            out["sp_vs_one_gpu_tolerance"] = 3e-3
            out["sp_check"] = (f"2-block model at full width, full 32760-token video, sp{ctx.world} "
                               f"(exchange: {exch}) vs rank 0 alone")
            if y_cut is not None:
                out["sp_with_cut_last_wave_vs_one_gpu_rel_l2"] = float((y_cut - y_1).norm() / y_1.norm())
                out["sp_with_cut_last_wave_note"] = (
                    "the timed configuration: attention rows of the last wave are summed in key ranges (fp32 order "
                    "differs); bounded by the reproducibility floor of two FP8 blocks, not by the 3e-3 of the exact "
                    "comparison above; the kernel-level bound (1e-3 on the attention output) is in the GPU tests")
        ctx.barrier()
    if ctx.rank == 0 and ctx.world == 1 and not args.no_oracle_parity:   # (N > 1: the other ranks would idle meanwhile)
        from oracle import flux as OF
        from oracle import ops as O
        from oracle import wan as OW
        from oracle.linear import LinearEval
        w1 = {k: v.float().cpu() for k, v in sd.items() if not k.startswith("blocks.1.")}
        xs = synth.randn((1, 16, 21, 30, 26), 80).bfloat16().float()
        cs = ctxt.float()
        mode = args.wan_fmt
        with torch.no_grad():
            _, h0_ref, h1_ref = OW.wan_dit_forward(w1, xs, cs, t, num_layers=1, H=c["H"], lin=LinearEval(mode),
                                                   rt=OF.round_bf16, return_hidden=True)
            # the same oracle with another fp32 summation order: the floor below which two evaluations of this
            # low-precision arithmetic do not agree with each other
            _, _, h1_alt = OW.wan_dit_forward(w1, xs, cs, t, num_layers=1, H=c["H"], lin=LinearEval(mode, shuffle_k=1),
                                              rt=OF.round_bf16, return_hidden=True)
        e1 = wan.WanDiTEngine(dict(w1), fmt=args.wan_fmt, device=dev, num_layers=1, num_heads=c["H"])
        e1(xs.to(dev), cs.to(dev), t.to(dev))
        h1 = e1.hidden().float().cpu()
        e0 = wan.WanDiTEngine(dict(w1), fmt=args.wan_fmt, device=dev, num_layers=0, num_heads=c["H"])
        e0(xs.to(dev), cs.to(dev), t.to(dev))
        h0 = e0.hidden().float().cpu()
        del e0, e1
        out["block_4095_tokens_rel_l2_vs_oracle"] = O.rel_l2(h1, h1_ref)
        out["block_update_rel_l2_vs_oracle"] = O.rel_l2(h1 - h0, h1_ref - h0_ref)
        out["oracle_vs_reordered_oracle_rel_l2"] = O.rel_l2(h1_alt, h1_ref)
        out["oracle_tolerance"] = 2e-3 if mode == "bf16" else 1e-2
        out["oracle_check"] = ("1-block model at width 5120 on a 21x15x13 token grid (4095 tokens) against the CPU oracle "
                               "with the same quantisation; passes when below max(tolerance, 1.5 x reordered-oracle figure)")
    del sd
    torch.cuda.empty_cache()
    if ctx.dist is not None:
        ctx.barrier()
    return out


def run_wan(ctx, args, steps, warmup):
    """Wan2.1-14B-architecture step, sequence-parallel (Ulysses) over all ranks: ONE video, strong scaling."""
    torch, pkg, synth, dev, dist = ctx.torch, ctx.pkg, ctx.synth, ctx.dev, ctx.dist
    wan = importlib.import_module("diffsynth_engine_b200.wan")
    c = dict(WAN)
    if args.wan_layers:
        c["num_layers"] = args.wan_layers
    parity = wan_parity(ctx, args) if not args.no_parity else {}
    shapes = synth.wan_dit_shapes(d=c["d"], ffn=c["ffn"], num_layers=c["num_layers"], text_dim=c["text_dim"])
    sd = synth.make_state_dict(shapes, seed=1234, device=dev, dtype=torch.bfloat16)   # same weights on every rank
    eng = wan.WanDiTEngine(sd, fmt=args.wan_fmt, device=dev, num_layers=c["num_layers"], num_heads=c["H"],
                           group=(dist.group.WORLD if dist is not None else None), release_source=True,
                           exchange=args.wan_exchange, tail_split=args.wan_tail_split == "on")
    del sd
    torch.cuda.empty_cache()
    eng.prepare(c["frames"], c["height"], c["width"], c["ctx"], c["text_dim"])
    h_x = synth.randn((1, 16, c["frames"], c["height"], c["width"]), 7).bfloat16().pin_memory()
    h_ctx = synth.randn((1, c["ctx"], c["text_dim"]), 8).bfloat16().pin_memory()
    h_t = torch.tensor([500.0]).pin_memory()
    h_out = torch.empty((1, 16, c["frames"], c["height"], c["width"]), dtype=torch.bfloat16).pin_memory()
    eng.set_inputs(h_x, h_ctx, h_t)
    eng.step()                      # first step of this prompt: also fills the cross-attention key / value cache
    n0 = pkg._lib.launches
    eng.step()
    launches = pkg._lib.launches - n0
    for _ in range(max(0, warmup - 2)):
        eng.step()
    # ---- device-resident throughput, clocks sampled during exactly this loop
    sampler = ClockSampler(ctx.local_rank).start() if ctx.rank == 0 else None
    torch.cuda.profiler.start()   # lets a profiler started with --profile-from-start off see exactly the timed region
    ms = ctx.timed_steps(eng.step, steps)
    torch.cuda.profiler.stop()
    clocks = sampler.stop() if sampler else None
    out_dev = eng.step()
    finite = bool(torch.isfinite(out_dev).all())
    checksum = float(out_dev.float().abs().mean())

    # ---- end to end: host buffers in, host buffer out, every step
    def e2e_step():
        eng.set_inputs(h_x, h_ctx, h_t)
        out = eng.step()
        if ctx.rank == 0:
            h_out.copy_(out, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    e2e_step()
    ms_e2e = ctx.timed_steps(e2e_step, steps)
    pkg.ops.check_status(dev.index)
    # ---- roofline of the dominant kernel (self-attention): CUDA events around every launch of one eager step
    recs = timed_launches(ctx, pkg.ops, ["flash_attn", "flash_attn_parts"], eng.step)
    S = c["frames"] * (c["height"] // 2) * (c["width"] // 2)

    def dims(r):   # (Sq, Sk, H) of a recorded attention launch
        a = r[1]
        if r[0] == "flash_attn_parts":   # (q_parts, q_rows, q_strides, k, v, o_parts, o_rows, o_strides, H, Sq)
            return a[9], a[3].shape[1], a[8]
        return a[0].shape[1], a[1].shape[1], a[0].shape[2]

    self_attn = [r for r in recs if dims(r)[1] > c["ctx"] + 257]              # keys = tokens, not the context
    attn_ms = sum(r[3] for r in self_attn)
    attn_flops = sum(4.0 * dims(r)[0] * dims(r)[1] * dims(r)[2] * 128 for r in self_attn)
    peaks = measured_peaks()
    lin_f, attn_f = wan_step_flops(c)
    fp8 = args.wan_fmt != "bf16"
    ach = attn_flops / (attn_ms * 1e-3) / 1e12 if attn_ms > 0 else 0.0
    roof_ms = (lin_f / (peaks["bf16"] * (2 if fp8 else 1) * 1e12) + attn_f / (peaks["bf16"] * 1e12)) * 1e3
    roofline = {
        "kernel": "flash_attn_kernel (bf16, head_dim 128; self-attention launches of one step)", "bound": "tensor",
        "achieved": ach, "peak": peaks["bf16_sustained"], "unit": "TFLOP/s", "frac": ach / peaks["bf16_sustained"],
        "peak_source": f"bf16_tflops_sustained of MEASURED_PEAKS.json ({peaks['source']}): the kernel is timed inside "
                       f"a seconds-long step under the power cap",
        "peak_burst": peaks["bf16"], "frac_of_burst_peak": ach / peaks["bf16"],
        "traffic": None, "traffic_source": "not measured in this run (needs an ncu capture)",
        "launches_per_step": len(self_attn), "kernel_ms_per_step": attn_ms,
        "share_of_step": attn_ms / ms if ms > 0 else None,
        "method": "CUDA events around each self-attention launch of one eager step; 4*Sq*Sk*H*128 flop per launch",
        "step_tflop": (lin_f + attn_f) / 1e12,
        "step_roofline_ms": roof_ms,
        "step_frac_of_roofline_all_gpus": roof_ms / (ms * ctx.world),
        "step_roofline_note": "linear flops at 2 x bf16 burst peak (no 8-bit peak in MEASURED_PEAKS.json) + attention "
                              "flops at the bf16 burst peak"}
    parity.update({"finite": finite, "mean_abs_output": checksum})
    return {"workload": f"wan2.1-14B-arch t2v DiT step, 81x480x832 (32760 tokens, 512 context tokens), batch 1, "
                        f"{c['num_layers']} blocks, weights {args.wan_fmt}, bf16 activations",
            "steps_per_s": 1e3 / ms, "ms_per_step": ms, "e2e_steps_per_s": 1e3 / ms_e2e, "e2e_ms_per_step": ms_e2e,
            "n_gpus": ctx.world, "gpu_launches_per_step": launches, "clocks": clocks, "roofline": roofline,
            "parity": parity,
            # how q and the attention output cross ranks ("peer": inside the attention kernel over mapped peer memory)
            "exchange": eng.exchange if ctx.world > 1 else None,
            # the prompt embedding is the same tensor at every step (as in the reference pipeline): it is copied, and the
            # cross-attention keys / values of all blocks are computed from it, once - during warm-up
            "cross_attention_kv_cache": "warm (context unchanged since warm-up; it is not copied or projected again)",
            "h2d_bytes_per_step": sum(t.numel() * t.element_size() for t in (h_x, h_t)),
            "d2h_bytes_per_step": h_out.numel() * h_out.element_size()}


# ------------------------------------------------------------------------------------------ Flux
def flux_parity(ctx, args, cfg):
    """A 1 + 1 block model at full width and the full 4096 + 512 token sequence against the CPU oracle with the same
    quantisation (rank 0 only; a few seconds of CPU)."""
    torch, synth, dev = ctx.torch, ctx.synth, ctx.dev
    if ctx.rank != 0 or args.no_parity or args.no_oracle_parity:
        return {}
    from oracle import flux as OF
    from oracle import ops as O
    from oracle.linear import LinearEval
    flux = importlib.import_module("diffsynth_engine_b200.flux")
    shapes = synth.flux_dit_shapes(d=cfg["d"], H=cfg["H"], n_double=1, n_single=1, txt_dim=cfg["txt_dim"],
                                   pooled_dim=cfg["pooled_dim"])
    w = {k: v.bfloat16().float().cpu() for k, v in synth.make_state_dict(shapes, seed=55, device=dev).items()}
    lat = synth.randn((1, 16, cfg["height"], cfg["width"]), 56).bfloat16().float()
    pe = synth.randn((1, cfg["S_txt"], cfg["txt_dim"]), 57).bfloat16().float()
    pooled = synth.randn((1, cfg["pooled_dim"]), 58)
    t, g = torch.tensor([500.0]), torch.tensor([3.5])
    with torch.no_grad():
        ref, hid_ref = OF.flux_dit_forward(w, lat, t, pe, pooled, g, n_double=1, n_single=1, H=cfg["H"],
                                           lin=LinearEval(args.fmt), rt=OF.round_bf16, return_hidden=True)
        alt, hid_alt = OF.flux_dit_forward(w, lat, t, pe, pooled, g, n_double=1, n_single=1, H=cfg["H"],
                                           lin=LinearEval(args.fmt, shuffle_k=1), rt=OF.round_bf16, return_hidden=True)
    eng = flux.FluxDiTEngine(dict(w), fmt=args.fmt, device=dev, n_double=1, n_single=1, num_heads=cfg["H"])
    out = eng(lat.to(dev), t.to(dev), pe.to(dev), pooled.to(dev), g.to(dev)).float().cpu()
    hid = eng._bufs["x"].float().cpu()
    del eng
    torch.cuda.empty_cache()
    return {"model_1p1_blocks_hidden_rel_l2_vs_oracle": O.rel_l2(hid, hid_ref),
            "model_1p1_blocks_output_rel_l2_vs_oracle": O.rel_l2(out, ref),
            "oracle_vs_reordered_oracle_hidden_rel_l2": O.rel_l2(hid_alt, hid_ref),
            "oracle_vs_reordered_oracle_output_rel_l2": O.rel_l2(alt, ref),
            "oracle_tolerance": 2e-3 if args.fmt == "bf16" else 1e-2,
            "oracle_check": "1 double + 1 single block at width 3072 on 4096 + 512 tokens against the CPU oracle with the "
                            "same quantisation; passes when below max(tolerance, 1.5 x reordered-oracle figure)"}


def run_flux(ctx, args, cfg, workload, steps, warmup):
    """Flux.1-dev-architecture (or the Qwen-arch stand-in) step on every rank: replicas, or with --sp ONE image whose
    token sequence is split over all ranks."""
    torch, pkg, synth, dev, dist = ctx.torch, ctx.pkg, ctx.synth, ctx.dev, ctx.dist
    ops = pkg.ops
    flux = importlib.import_module("diffsynth_engine_b200.flux")
    sp = args.sp and ctx.world > 1
    parity = flux_parity(ctx, args, cfg) if workload != "qwen" and not args.blocks else {}
    # random-init weights of the architecture, drawn on the device, packed to FP8 layer by layer
    shapes = synth.flux_dit_shapes(d=cfg["d"], H=cfg["H"], n_double=cfg["n_double"], n_single=cfg["n_single"],
                                   txt_dim=cfg["txt_dim"], pooled_dim=cfg["pooled_dim"])
    seed = 0 if sp else ctx.rank        # sequence parallel: every rank holds the same model and the same inputs
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
    ops.check_status(ctx.local_rank)
    eng.capture()
    for _ in range(max(3, warmup)):
        eng.step()
    sampler = ClockSampler(ctx.local_rank).start() if ctx.rank == 0 else None
    torch.cuda.profiler.start()
    ms_per_step = ctx.timed_steps(eng.step, steps)
    torch.cuda.profiler.stop()
    clocks = sampler.stop() if sampler else None
    out_dev = eng.step()
    parity.update({"finite": bool(torch.isfinite(out_dev).all()), "mean_abs_output": float(out_dev.float().abs().mean())})
    value = (1 if sp else ctx.world) * 1e3 / ms_per_step

    def e2e_step():
        eng.set_inputs(h_lat, h_t, h_pe, h_pool, h_g)
        out = eng.step()
        h_out.copy_(out, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    for _ in range(3):
        e2e_step()
    e2e_ms = ctx.timed_steps(e2e_step, steps)
    ops.check_status(ctx.local_rank)
    # ---- roofline of the dominant kernel (the FP8 GEMM): CUDA events around every launch of one eager step
    peaks = measured_peaks()
    eng._graph_saved, eng._graph = eng._graph, None
    try:
        recs = timed_launches(ctx, ops, ["gemm", "gemm_qkv", "gemm_group"], eng.step)
    finally:
        eng._graph = eng._graph_saved

    def flops_of(name, a):
        probs = a[0] if name == "gemm_group" else [dict(a=a[0], w=a[1])]
        return sum(2.0 * p["a"].shape[0] * p["a"].shape[1] * p["w"].shape[0] for p in probs)

    gemm_flops = sum(flops_of(n, a) for n, a, _, _ in recs)
    gemm_ms = sum(r[3] for r in recs)
    fp8 = args.fmt != "bf16"          # any 8-bit weight format: the tensor pipe runs at twice the bf16 rate
    int8 = args.fmt.startswith("int8")
    kind = "int8" if int8 else "fp8"
    mult = 2.0 if fp8 else 1.0
    ach_tf = gemm_flops / (gemm_ms * 1e-3) / 1e12
    lin_f, attn_f = flux_step_flops(cfg)
    lib_tf = library_fp8_gemm_tflops(torch, dev) if (fp8 and not int8 and ctx.rank == 0) else None
    roofline = {"kernel": f"gemm_kernel<{kind}> (256x256 CTA-pair tiles; 128x128 for the text stream)" if fp8
                else "gemm_kernel<bf16>", "bound": "tensor",
                "achieved": ach_tf, "peak": mult * peaks["bf16_sustained"], "unit": "TFLOP/s",
                "frac": ach_tf / (mult * peaks["bf16_sustained"]),
                "peak_source": (f"{'2 x ' if fp8 else ''}bf16_tflops_sustained of MEASURED_PEAKS.json ({peaks['source']}): "
                                f"the launches are timed inside a step under the power cap"
                                + ("; no 8-bit peak was measured by the driver, 2 x the bf16 figure is assumed" if fp8 else "")),
                "peak_burst": mult * peaks["bf16"], "frac_of_burst_peak": ach_tf / (mult * peaks["bf16"]),
                "library_fp8_gemm_tflops_8192": lib_tf,
                "traffic": None, "traffic_source": "not measured in this run (needs an ncu capture)",
                "launches_per_step": len(recs), "kernel_ms_per_step": gemm_ms,
                "method": "CUDA events around each GEMM launch of one eager (un-graphed) step; 2MNK per launch",
                "step_tflop": (lin_f + attn_f) / 1e12,
                "step_frac_of_roofline": ((lin_f / (mult * peaks["bf16"] * 1e12) + attn_f / (peaks["bf16"] * 1e12)) * 1e3)
                / (ms_per_step * (ctx.world if sp else 1)),
                "step_roofline_note": "linear flops at 2 x bf16 burst peak + attention flops at the bf16 burst peak"}
    del eng
    torch.cuda.empty_cache()
    return {"value": value, "ms_per_step": ms_per_step, "clocks": clocks, "parity": parity,
            "scaling": "strong" if sp else "weak",
            "dtype": ("int8 x int8 -> int32 (linear), bf16 (attention)" if int8
                      else "fp8_e4m3 x fp8_e4m3 -> fp32 (linear), bf16 (attention)" if fp8 else "bf16"),
            "e2e": {"value": (1 if sp else ctx.world) * 1e3 / e2e_ms, "unit": "steps/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms},
            "gpu_launches_per_step": launches_per_step, "roofline": roofline}


def run_reference_gpu(ctx, args):
    """The reference's own GPU path on this B200 next to the library: one Flux double-stream block, one Flux
    single-stream block (4096 + 512 tokens, width 3072) and one Wan DiTBlock (32760 tokens, width 5120), each as
    (a) the reference module as shipped in bf16 (cuBLAS + SDPA), (b) the reference module with its own FP8 path
    (``enable_fp8_linear`` + ``fp8_inference``: ``torch._scaled_mm`` with unit scales), (c) this library's step engine
    (time per block = difference between an n-block and a 1-block model).  Needs ``baseline/_ref``."""
    torch, pkg, synth, dev = ctx.torch, ctx.pkg, ctx.synth, ctx.dev
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    import install_reference
    ref = install_reference.import_reference()
    if ref is None:
        return {"workload": "reference-gpu", "unavailable": "baseline/_ref is not installed (python baseline/install_reference.py)"}
    flux = importlib.import_module("diffsynth_engine_b200.flux")
    wan = importlib.import_module("diffsynth_engine_b200.wan")

    def timeit(fn, n=8, warm=2):
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

    def load(module, sd):
        torch.nn.Module.load_state_dict(module, sd, strict=True)
        return module.to(dev, torch.bfloat16).eval()

    def both_paths(make, call):
        with torch.no_grad():
            blk = make()
            t_bf16 = timeit(lambda: call(blk))
            blk8 = make()
            ref.fp8_linear.enable_fp8_linear(blk8)
            origin = torch.nn.functional.linear
            try:
                with ref.fp8_linear.fp8_inference(True):
                    t_fp8 = timeit(lambda: call(blk8))
            except Exception as e:          # the reference's context manager does not restore F.linear on an error
                t_fp8 = f"failed: {type(e).__name__}: {str(e)[:120]}"
            finally:
                torch.nn.functional.linear = origin
        del blk, blk8
        torch.cuda.empty_cache()
        return t_bf16, t_fp8

    out = {"workload": "reference-gpu", "unit": "ms per block", "rows": []}
    # ---- Flux blocks
    d, H, St, side = FLUX["d"], FLUX["H"], FLUX["S_txt"], FLUX["height"] // 2
    ids = torch.zeros(St + side * side, 3)
    r = torch.arange(side, dtype=torch.float32)
    ids[St:, 1] = r[:, None].expand(side, side).reshape(-1)
    ids[St:, 2] = r[None, :].expand(side, side).reshape(-1)
    rope = ref.transformer_helper.RoPEEmbedding(d, 10000, [16, 56, 56])(ids[None]).to(dev)
    xa, xb = synth.randn((1, side * side, d), 1, dev).bfloat16(), synth.randn((1, St, d), 2, dev).bfloat16()
    temb = synth.randn((1, d), 3, dev).bfloat16()
    sd_d = synth.make_state_dict(synth.flux_block_shapes("", d, H, "double"), seed=0, device=dev)
    sd_s = synth.make_state_dict(synth.flux_block_shapes("", d, H, "single"), seed=1, device=dev)
    t_bf16, t_fp8 = both_paths(lambda: load(ref.flux_dit.FluxJointTransformerBlock(d, H, device="cpu", dtype=torch.float32), sd_d),
                               lambda b: b(xa, xb, temb, rope))
    out["rows"].append({"block": "Flux double-stream (4096 + 512 tokens, d 3072)", "reference_bf16_ms": t_bf16,
                        "reference_fp8_scaled_mm_ms": t_fp8})
    xs = torch.cat([xb, xa], dim=1)
    t_bf16, t_fp8 = both_paths(lambda: load(ref.flux_dit.FluxSingleTransformerBlock(d, H, device="cpu", dtype=torch.float32), sd_s),
                               lambda b: b(xs, None, temb, rope))
    out["rows"].append({"block": "Flux single-stream (4608 tokens, d 3072)", "reference_bf16_ms": t_bf16,
                        "reference_fp8_scaled_mm_ms": t_fp8})
    del sd_d, sd_s

    def engine_ms(fmt, nd, ns):
        shapes = synth.flux_dit_shapes(d=d, H=H, n_double=nd, n_single=ns)
        eng = flux.FluxDiTEngine(synth.make_state_dict(shapes, seed=0, device=dev, dtype=torch.bfloat16), fmt=fmt, device=dev,
                                 n_double=nd, n_single=ns, num_heads=H, release_source=True)
        eng.prepare(St, FLUX["height"], FLUX["width"])
        eng.step()
        eng.capture()
        t = timeit(eng.step)
        del eng
        torch.cuda.empty_cache()
        return t

    for fmt in ("bf16", "fp8_tensor"):
        base = engine_ms(fmt, 1, 1)
        out["rows"][0][f"library_{fmt}_ms"] = (engine_ms(fmt, 5, 1) - base) / 4
        out["rows"][1][f"library_{fmt}_ms"] = (engine_ms(fmt, 1, 5) - base) / 4
    # ---- Wan block
    c = WAN
    d, H = c["d"], c["H"]
    fr, hh, ww = c["frames"], c["height"] // 2, c["width"] // 2
    S = fr * hh * ww
    sd_w = synth.make_state_dict(synth.wan_block_shapes("", d, c["ffn"]), seed=2, device=dev)
    x, cx = synth.randn((1, S, d), 4, dev).bfloat16(), synth.randn((1, c["ctx"], d), 5, dev).bfloat16()
    tmod = (synth.randn((1, 6, d), 6, dev) * 0.1).bfloat16()
    f_, h_, w_ = ref.wan_dit.precompute_freqs_cis_3d(d // H)
    freqs = torch.cat([f_[:fr].view(fr, 1, 1, -1).expand(fr, hh, ww, -1), h_[:hh].view(1, hh, 1, -1).expand(fr, hh, ww, -1),
                       w_[:ww].view(1, 1, ww, -1).expand(fr, hh, ww, -1)], dim=-1).reshape(S, 1, -1).to(dev)
    t_bf16, t_fp8 = both_paths(lambda: load(ref.wan_dit.DiTBlock(False, d, H, c["ffn"], 1e-6, device="cpu", dtype=torch.float32), sd_w),
                               lambda b: b(x, cx, tmod, freqs))
    row = {"block": "Wan DiTBlock (32760 tokens, 512 context tokens, d 5120)", "reference_bf16_ms": t_bf16,
           "reference_fp8_scaled_mm_ms": t_fp8}
    del sd_w

    def wan_ms(fmt, layers):
        shapes = synth.wan_dit_shapes(d=d, ffn=c["ffn"], num_layers=layers, text_dim=c["text_dim"])
        eng = wan.WanDiTEngine(synth.make_state_dict(shapes, seed=3, device=dev, dtype=torch.bfloat16), fmt=fmt, device=dev,
                               num_layers=layers, num_heads=H, release_source=True)
        eng.prepare(c["frames"], c["height"], c["width"], c["ctx"], c["text_dim"])
        t = timeit(eng.step, n=4, warm=1)
        del eng
        torch.cuda.empty_cache()
        return t

    for fmt in ("bf16", "fp8_channel"):
        row[f"library_{fmt}_ms"] = (wan_ms(fmt, 3) - wan_ms(fmt, 1)) / 2
    out["rows"].append(row)
    pkg.ops.check_status(dev.index)
    return out


def run_kernels(torch, pkg, dev):
    """Per-kernel timings of the current build at the shapes of the two steps (CUDA events, each case 20-30
    back-to-back launches after warm-up): the GEMM with each of its epilogues, the bandwidth-bound row kernels on
    three rotating 335 MB inputs, attention at the sequence-parallel shards with and without the cut of the last wave.
    The figures the notes under ``profiles/`` quote for "the current build" come from this workload."""
    ops = pkg.ops

    def timeit(fn, n=20, warm=3):
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

    def q8(M, K):
        return torch.randn(M, K, device=dev).to(torch.float8_e4m3fn)

    out = {"metric": "per-kernel timings", "unit": "us", "data": "synthetic", "gemm_fp8": [], "row_kernels": [],
           "attention": []}
    d = 3072
    nq = torch.ones(128, device=dev)
    for (M, K, N, kind) in [(4096, d, 3 * d, "plain"), (4096, d, 3 * d, "norm_rope"), (4608, d, 7 * d, "norm_rope_gelu8_split"),
                            (4096, d, 4 * d, "gelu8"), (4096, 4 * d, d, "gate_resid"), (4096, d, d, "gate_resid"),
                            (4608, 5 * d, d, "gate_resid"), (32760, 5120, 5120, "gate_resid"),
                            (32760, 5120, 13824, "gelu8"), (32760, 13824, 5120, "gate_resid"), (8192, 8192, 8192, "plain")]:
        a, w = q8(M, K), q8(N, K)
        rs, cs, bias = torch.rand(M, device=dev) * 0.01, torch.rand(N, device=dev) * 0.01, torch.randn(N, device=dev)
        base = dict(a=a, w=w, row_scale=rs, col_scale=cs, bias=bias)
        if kind == "plain":
            o = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
            fn = lambda: ops.gemm_group([dict(base, out=o)])
        elif kind == "norm_rope":
            o = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
            rope = torch.randn(M, 64, 2, device=dev).half()
            fn = lambda: ops.gemm_group([dict(base, out=o, nq_w=nq, nk_w=nq, d_model=d, rope=rope)])
        elif kind == "norm_rope_gelu8_split":
            o = torch.empty(M, 3 * d, dtype=torch.bfloat16, device=dev)
            o1 = torch.empty(M, N - 3 * d, dtype=torch.float8_e4m3fn, device=dev)
            rope = torch.randn(M, 64, 2, device=dev).half()
            fn = lambda: ops.gemm_group([dict(base, out=o, out1=o1, split_col=3 * d, act=ops.ACT_GELU_TANH,
                                              act_col0=3 * d, nq_w=nq, nk_w=nq, d_model=d, rope=rope)])
        elif kind == "gelu8":
            o = torch.empty(M, N, dtype=torch.float8_e4m3fn, device=dev)
            fn = lambda: ops.gemm_group([dict(base, out=o, act=ops.ACT_GELU_TANH)])
        else:
            o = torch.randn(M, N, device=dev).bfloat16()
            gate = torch.randn(N, device=dev) * 0.01
            fn = lambda: ops.gemm_group([dict(base, out=o, gate=gate, resid=o)])
        t = timeit(fn, n=30 if M < 10000 else 10)
        out["gemm_fp8"].append({"M": M, "K": K, "N": N, "epilogue": kind, "us": t * 1e3, "tflops": 2.0 * M * N * K / t / 1e9})
        del a, w, o
    for (M, D) in [(32760, 5120), (4096, 5120), (4608, 3072)]:
        xs = [torch.randn(M, D, device=dev).bfloat16() for _ in range(3)]
        shift, scale, wn = torch.randn(D, device=dev) * 0.1, torch.randn(D, device=dev) * 0.1, torch.ones(D, device=dev)
        rope = torch.randn(M, 64, 2, device=dev)
        oq, rs = torch.empty(M, D, dtype=torch.float8_e4m3fn, device=dev), torch.empty(M, device=dev)
        i = [0]

        def nxt():
            i[0] = (i[0] + 1) % 3
            return xs[i[0]]

        for name, fn, nbytes in (
                ("ln_modulate_e4m3", lambda: ops.ln_modulate(nxt(), shift, scale, 1e-6, ops.FMT_E4M3, out=oq, row_scale=rs), 3),
                ("rmsnorm_full_rope", lambda: ops.rmsnorm_full(nxt(), wn, rope, 0, 1e-6), 4),
                ("quant_rows_e4m3", lambda: ops.quant_rows(nxt(), ops.FMT_E4M3, out=oq, row_scale=rs), 3)):
            t = timeit(fn)
            out["row_kernels"].append({"kernel": name, "M": M, "D": D, "us": t * 1e3, "gbs": nbytes * M * D / t / 1e6})
        del xs
    ws = ops.flash_attn_workspace(dev)
    for (H, Sq, Sk) in [(24, 4608, 4608), (40, 32760, 32760), (20, 32768, 32760), (10, 32768, 32760), (5, 32768, 32760)]:
        q, k, v = (torch.randn(1, s_, H, 128, device=dev).bfloat16() for s_ in (Sq, Sk, Sk))
        o = torch.empty_like(q)
        n = 10 if H * Sq < 400000 else 4
        t0 = timeit(lambda: ops.flash_attn(q, k, v, out=o), n=n)
        t1 = timeit(lambda: ops.flash_attn_parts([q[0]], Sq, (H * 128, 128), k, v, [o[0]], Sq, (H * 128, 128), H, Sq,
                                                 workspace=ws), n=n) if Sq % 128 == 0 else None
        fl = 4.0 * Sq * Sk * H * 128
        out["attention"].append({"H": H, "Sq": Sq, "Sk": Sk, "us": t0 * 1e3, "tflops": fl / t0 / 1e9,
                                 "us_last_wave_cut": None if t1 is None else t1 * 1e3})
        del q, k, v, o
    ops.check_status(dev.index)
    return out


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
    ap.add_argument("--fmt", default="fp8_tensor", help="weight format of the flux / qwen workloads")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-parity", action="store_true", help="skip the correctness checks made before timing")
    ap.add_argument("--no-oracle-parity", action="store_true", help="skip only the CPU-oracle part of them")
    ap.add_argument("--blocks", default=None, help="n_double,n_single override (reduced-depth debugging; not a bench)")
    ap.add_argument("--workload", default="both", choices=["flux", "wan", "both", "qwen", "sweeps", "kernels", "reference-gpu"],
                    help="both (default): the Wan sequence-parallel step as the line's value, the Flux step attached "
                         "under 'flux' at one GPU; wan / flux / qwen: that workload alone as the line's value")
    ap.add_argument("--wan-fmt", default="fp8_channel")
    ap.add_argument("--wan-layers", type=int, default=0, help="reduced depth (debugging; not a bench)")
    ap.add_argument("--wan-tail-split", default="on", choices=["on", "off"],
                    help="peer exchange only: cut the attention items of a partly filled last wave along the keys")
    ap.add_argument("--wan-exchange", default="auto", choices=["auto", "peer", "nccl"],
                    help="how q and the attention output cross ranks at N > 1 (see WanDiTEngine)")
    ap.add_argument("--sp", action="store_true",
                    help="flux/qwen workloads under torchrun: ONE image, its token sequence split over all ranks (Ulysses, "
                         "strong scaling) instead of one replica per GPU")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    warmup = max(3, args.warmup)
    steps = max(1, args.steps)
    wan_headline = args.workload in ("both", "wan")
    S_wan = WAN["frames"] * (WAN["height"] // 2) * (WAN["width"] // 2)
    wan_cfg = {"workload": (f"wan2.1-14B-arch t2v DiT step, 81x480x832 ({S_wan} tokens, 512 context tokens), batch 1, "
                            f"{args.wan_layers or WAN['num_layers']} blocks, weights {args.wan_fmt}, bf16 activations"),
               "parallelism": f"sp{world} (Ulysses sequence parallel, one video)" if world > 1 else "single GPU",
               "l2": "per-step working set (14 GB of weights, 335 MB activations per tensor) exceeds the 126 MB L2; no "
                     "flush between steps"}

    if args.impl == "reference":
        if rank != 0:
            return
        r = (cpu_wan_arm if wan_headline else cpu_flux_arm)(steps=steps, warmup=args.warmup)
        cfg = wan_cfg if wan_headline else {"workload": "flux1-dev-arch DiT step, 1024x1024 (4096 image + 512 text tokens), "
                                            "batch 1, 19 double + 38 single blocks", "parallelism": "single GPU"}
        line = {"impl": "reference", "metric": "DiT denoise steps/s", "value": r["value"], "unit": "steps/s",
                "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
                # one timed "step" of this arm is the bounded sample below; `value` extrapolates it to a whole step
                "ms_per_step": r["sample_ms"], "sample_fraction_of_a_step": r["sample_fraction"], "extrapolated": True,
                "higher_is_better": True, "scaling": "strong" if wan_headline else "weak", "vs_baseline": None,
                "dtype": "fp32", "data": "synthetic", "config": cfg,
                "cpu_baseline": {k: r[k] for k in ("value", "unit", "cores", "kind", "sample", "reference_module_check") if k in r},
                "e2e": {"value": r["value"], "unit": "steps/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(line), flush=True)
        return

    # Libraries underneath may write to the process's stdout (NCCL prints a version banner at the first communicator
    # under some NCCL_DEBUG settings): everything but the final JSON line goes to stderr.
    sys.stdout.flush()
    json_fd = os.dup(1)
    os.dup2(2, 1)

    def emit(obj):
        os.write(json_fd, (json.dumps(obj) + "\n").encode())

    import torch
    pkg = load_package()
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
    ctx = Ctx(torch, pkg, dev, dist, rank, world, local_rank)

    if args.workload == "sweeps":
        if rank == 0:
            emit(run_sweeps(torch, pkg, dev))
        return
    if args.workload == "kernels":
        if rank == 0:
            emit(run_kernels(torch, pkg, dev))
        return
    if args.workload == "reference-gpu":
        if rank == 0:
            emit(run_reference_gpu(ctx, args))
        return

    line = {"metric": "DiT denoise steps/s", "unit": "steps/s", "n_gpus": world, "steps": steps, "warmup": warmup,
            "higher_is_better": True, "vs_baseline": None, "data": "synthetic"}
    if wan_headline:
        r = run_wan(ctx, args, steps, warmup)
        line.update({"value": r["steps_per_s"], "ms_per_step": r["ms_per_step"], "scaling": "strong",
                     "dtype": "fp8_e4m3 x fp8_e4m3 -> fp32 (linear), bf16 (attention)" if args.wan_fmt != "bf16" else "bf16",
                     "config": wan_cfg, "clocks": r["clocks"],
                     "e2e": {"value": r["e2e_steps_per_s"], "unit": "steps/s", "ms_per_step": r["e2e_ms_per_step"],
                             "h2d_bytes_per_step": r["h2d_bytes_per_step"], "d2h_bytes_per_step": r["d2h_bytes_per_step"]},
                     "gpu_launches": r["gpu_launches_per_step"] * steps,
                     "gpu_launches_per_step": r["gpu_launches_per_step"],
                     "cross_attention_kv_cache": r["cross_attention_kv_cache"],
                     "sp_exchange": r["exchange"],
                     "roofline": r["roofline"], "parity": r["parity"]})
        if args.workload == "both" and world == 1:
            f = run_flux(ctx, args, dict(FLUX), "flux", steps, warmup)
            f["config"] = {"workload": "flux1-dev-arch DiT step, 1024x1024 (4096 image + 512 text tokens), batch 1, "
                                       f"19 double + 38 single blocks, weights {args.fmt}, bf16 activations",
                           "parallelism": "single GPU", "launch": "CUDA-graph replay of the step"}
            f["metric"], f["unit"] = "DiT denoise steps/s", "steps/s"
            line["flux"] = f
    else:
        cfg = dict(QWEN if args.workload == "qwen" else FLUX)
        if args.blocks:
            cfg["n_double"], cfg["n_single"] = (int(v) for v in args.blocks.split(","))
        sp = args.sp and world > 1
        if args.workload == "qwen":
            wl = ("qwen-image-arch stand-in (Flux-style double-stream blocks), 1328x1328 (6889 image + 256 text tokens of "
                  f"width 3584), batch 1, {cfg['n_double']} double blocks, weights {args.fmt}, bf16 activations")
        else:
            wl = ("flux1-dev-arch DiT step, 1024x1024 (4096 image + 512 text tokens), batch 1, "
                  f"{cfg['n_double']} double + {cfg['n_single']} single blocks, weights {args.fmt}, bf16 activations")
        f = run_flux(ctx, args, cfg, args.workload, steps, warmup)
        line.update({"value": f["value"], "ms_per_step": f["ms_per_step"], "scaling": f["scaling"], "dtype": f["dtype"],
                     "config": {"workload": wl,
                                "parallelism": (f"sp{world} (Ulysses, one image)" if sp else f"replicas x{world}")
                                if world > 1 else "single GPU",
                                "l2": "per-step working set (11.9 GB of weights) exceeds the 126 MB L2; no flush "
                                      "between steps"},
                     "clocks": f["clocks"], "e2e": f["e2e"], "gpu_launches": f["gpu_launches_per_step"] * steps,
                     "gpu_launches_per_step": f["gpu_launches_per_step"], "roofline": f["roofline"],
                     "parity": f["parity"]})
    if rank == 0:
        if not args.no_cpu_baseline and world == 1:
            r = (cpu_wan_arm if wan_headline else cpu_flux_arm)(steps=2, warmup=0, budget_s=40.0)
            line["cpu_baseline"] = {k: r[k] for k in ("value", "unit", "cores", "kind", "sample", "reference_module_check")
                                    if k in r}
        emit(line)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
