#!/usr/bin/env python
"""Headline benchmark: train tokens/s per optimiser step of the SeeML update-plan VM
on B200 (forward + autodiff backward + AdamW over a frozen base with LoRA adapters).

    python bench.py --gpus 1 --steps K --warmup W
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...
    python bench.py --impl reference ...      # the reference's CPU runtime, same metric

A "step" is one optimiser step over the global batch (config c4: 256 sequences x 512
tokens = 131072 tokens, executed as 8 chunks of the plan's compiled batch of 16384 rows,
chunks sharded across the ranks). Rank 0 prints ONE JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from see_ml_b200 import formats as F  # noqa: E402
from see_ml_b200 import plansynth as PS  # noqa: E402

# name -> model geometry + LoRA/optimiser request of the benchmark configurations
CONFIGS = {
    "c1": dict(kind="mlp", dims=[256, 512, 512, 10], acts=["relu", "gelu", None], rows=32, chunks=1,
               rank=8, alpha=16.0, targets=(), lr=1e-3),
    "c2": dict(kind="gpt", vocab=512, d=128, heads=4, ffn=512, layers=2, seq=64, seqs=16, chunks=1,
               rank=8, alpha=16.0, targets=("wq", "wv"), lr=1e-3),
    "c3": dict(kind="llama", vocab=4096, d=256, heads=4, ffn=768, layers=4, seq=128, seqs=64, chunks=1,
               rank=16, alpha=32.0, targets=("wq", "wk", "wv", "wo"), lr=5e-4),
    "c4": dict(kind="llama", vocab=32000, d=1024, heads=16, ffn=2816, layers=12, seq=512, seqs=32,
               chunks=8, rank=16, alpha=32.0, targets=("wq", "wk", "wv", "wo", "w_up", "w_down"), lr=3e-4),
    # two layers of c4 with a smaller vocabulary: the same per-layer kernel shapes in a few GB, sized for
    # profiler captures (not a bench line)
    "c4-slice": dict(kind="llama", vocab=8192, d=1024, heads=16, ffn=2816, layers=2, seq=512, seqs=32,
                     chunks=1, rank=16, alpha=32.0, targets=("wq", "wk", "wv", "wo", "w_up", "w_down"), lr=3e-4),
}


GEMM_KINDS = {"tf32x3": 0, "f16x2": 1, "simt": 2, "tf32": 3}


def build_model(cfg, seed=1):
    rng = np.random.default_rng(seed)
    if cfg["kind"] == "mlp":
        return PS.mlp_model(cfg["dims"], cfg["acts"], rng)
    fn = PS.llama_decoder if cfg["kind"] == "llama" else PS.gpt_decoder
    return fn(cfg["vocab"], cfg["d"], cfg["heads"], cfg["ffn"], cfg["layers"], cfg["seq"], rng)


def build_plan(cfg, model, rows, hasher):
    spec = PS.TrainSpec(batch=rows, lora_rank=cfg["rank"], lora_alpha=cfg["alpha"], targets=cfg["targets"],
                        lr=cfg["lr"], default_steps=1000)
    return PS.synthesize(model, spec, hasher=hasher)


def synth_batches(cfg, rows, n_chunks, seed):
    """Seeded synthetic corpus of the configuration's shape and value distribution:
    Zipf(1.1) token ids with next-token labels, or N(0,1) features with uniform labels."""
    rng = np.random.default_rng(seed)
    if cfg["kind"] == "mlp":
        x = rng.standard_normal((n_chunks, rows, cfg["dims"][0])).astype(np.float32)
        y = rng.integers(0, cfg["dims"][-1], (n_chunks, rows)).astype(np.int32)
        return x.reshape(n_chunks, -1), y
    S = cfg["seq"]
    if cfg["kind"] == "llama":
        recs = PS.zipf_tokens(rng, cfg["vocab"], (n_chunks, rows // S, S + 1))
    else:
        recs = rng.integers(0, cfg["vocab"], (n_chunks, rows // S, S + 1)).astype(np.int32)
    return (np.ascontiguousarray(recs[:, :, :-1]).reshape(n_chunks, -1),
            np.ascontiguousarray(recs[:, :, 1:]).reshape(n_chunks, -1))


def plan_work(plan_bytes):
    """Algorithmic GEMM FLOPs (2*M*N*K) of one execution of the train stream, and the
    dominant GEMM shape: the (M, N, K) whose launches carry the most FLOPs in total."""
    p = F.parse_plan(plan_bytes)
    total, by_shape = 0, {}
    for ins in p.train:
        if int(ins["opcode"]) in (1, 2, 3, 4):
            m, n, k = (int(v) for v in ins["out"])
            fl = 2 * m * n * k
            total += fl
            by_shape[(m, n, k)] = by_shape.get((m, n, k), 0) + fl
    top = None
    if by_shape:
        shape = max(sorted(by_shape), key=lambda sh: (by_shape[sh], sh[1]))   # ties: the wider output
        top = (2 * shape[0] * shape[1] * shape[2], shape)
    return total, top


def profiled_traffic(m, n, k):
    """DRAM bytes per launch (read + write) of the tensor-core GEMM at this shape, from the
    committed profiler summary; None when that shape was not captured."""
    path = os.path.join(ROOT, "profiles", "dram_traffic.txt")
    if not os.path.exists(path):
        return None
    for line in open(path):
        f = line.split()
        if len(f) == 3 and f[0] == "gemm_tc_kernel" and f[1] == f"{m}x{n}x{k}":
            return int(f[2])
    return None


class ClockSampler:
    """nvidia-smi clocks and throttle reasons during the timed region."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.rows, self.proc, self.idx = [], None, gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-i", str(self.idx), "-lms", "200"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                pass
        sm = [float(r[1]) for r in self.rows if len(r) >= 9 and r[1].replace(".", "").isdigit()]
        mx = [float(r[2]) for r in self.rows if len(r) >= 9 and r[2].replace(".", "").isdigit()]
        reasons = set()
        for r in self.rows:
            if len(r) >= 9:
                for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"),
                                   r[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d.get("hbm_gbs", 6650.0), d.get("bf16_tflops", 1590.0), d.get("bf16_tflops_sustained", 1400.0), "measured"
    return 6650.0, 1590.0, 1400.0, "fallback"


# ------------------------------------------------------------------------------- reference arm
def cpu_reference_sample(cfg, model, steps, warmup, threads):
    """Times the reference's own CPU runtime (oracle/_ref: UpdateEngine::ExecuteTrainOnce, its stock
    path, built with its phase timers) - or the C restatement when the reference build is absent -
    on a bounded sample of the workload: a plan compiled for one sequence (token configs) or one
    compiled batch (MLP) of the same model. The reference pays forward + backward per row and the
    optimiser once per global step, so the rate for the workload's global step is
    global_rows / (fwd_bwd_seconds_per_row * global_rows + optimiser_seconds)."""
    from oracle import pyoracle as O
    rows = cfg["seq"] if cfg["kind"] != "mlp" else cfg["rows"]
    global_rows = (cfg["rows"] if cfg["kind"] == "mlp" else cfg["seqs"] * cfg["seq"]) * cfg["chunks"]
    hasher = lambda b, o: int(O.port().orc_plan_self_hash(np.frombuffer(b, np.uint8).ctypes.data, len(b), o))
    blob, _ = build_plan(cfg, model, rows, hasher)
    inp, lab = synth_batches(cfg, rows, 1, seed=5)
    h = F.PlanHeader.unpack(blob)
    if O.have_ref():
        kind = "reference"
        O.ref().ref_set_threads(threads)
        e = O.RefEngine(blob)
        arena = e.arena()
        arena[h.input_ref:h.input_ref + inp[0].nbytes] = inp[0].view(np.uint8)
        arena[h.label_ref:h.label_ref + lab[0].nbytes] = lab[0].view(np.uint8)
        for _ in range(warmup):
            e.execute_train_once()
        s0 = e.step_timings()
        for _ in range(steps):
            e.execute_train_once()
        s1 = e.step_timings()
        n = max(s1[0] - s0[0], 1)
        t_fb = ((s1[1] - s0[1]) + (s1[2] - s0[2])) / n
        t_opt = (s1[3] - s0[3]) / n
    else:
        kind, threads = "port", 1
        plan = F.parse_plan(blob)
        opt_begin = int(np.nonzero(np.isin(plan.train["opcode"], (17, 18, 28)))[0][0])
        arena = np.zeros(F.align_up(h.arena_size), np.uint8)
        arena[:h.persist_init_size] = plan.persist_init
        arena[h.input_ref:h.input_ref + inp[0].nbytes] = inp[0].view(np.uint8)
        arena[h.label_ref:h.label_ref + lab[0].nbytes] = lab[0].view(np.uint8)
        t_fb = t_opt = 0.0
        for i in range(warmup + steps):
            t0 = time.perf_counter()
            O.execute("port", plan.train[:opt_begin], arena, np.asarray(plan.rodata), lr=h.lr, step=i + 1)
            t1 = time.perf_counter()
            O.execute("port", plan.train[opt_begin:], arena, np.asarray(plan.rodata), lr=h.lr, step=i + 1)
            t2 = time.perf_counter()
            if i >= warmup:
                t_fb += (t1 - t0) / max(steps, 1)
                t_opt += (t2 - t1) / max(steps, 1)
    t_global = t_fb * (global_rows / rows) + t_opt
    return dict(value=global_rows / t_global, unit="tokens/s", cores=threads, kind=kind,
                sample=f"{steps} timed execution(s) of a {rows}-row plan of the workload's model after {warmup} warm-up: "
                       f"forward+backward {t_fb * 1e3:.1f} ms per {rows} rows, optimiser {t_opt * 1e3:.2f} ms; rate for the "
                       f"{global_rows}-row global step = rows / (fwd_bwd per row * rows + optimiser)",
                rows_timed=rows, fwd_bwd_ms=t_fb * 1e3, opt_ms=t_opt * 1e3), t_global * 1e3


def run_reference(args, cfg):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    model = build_model(cfg)
    threads = args.ref_threads or os.cpu_count() or 1
    base, ms = cpu_reference_sample(cfg, model, args.steps, args.warmup, threads)
    config = workload_config(args, cfg)
    config["reference_rows_timed_per_execution"] = base["rows_timed"]
    config["sampled_rate"] = True
    line = {"metric": "train tokens/sec per update step", "value": base["value"], "unit": "tokens/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic", "impl": "reference", "config": config,
            "cpu_baseline": base,
            "e2e": {"value": base["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0,
                    "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def workload_config(args, cfg):
    rows = cfg["rows"] if cfg["kind"] == "mlp" else cfg["seqs"] * cfg["seq"]
    d = {"workload": args.config, "rows_per_chunk": rows, "chunks_per_step": cfg["chunks"],
         "global_rows_per_step": rows * cfg["chunks"], "lora_rank": cfg["rank"],
         "lora_targets": list(cfg["targets"]) or "all", "optimizer": "adamw",
         "l2": "inputs and activations exceed L2 (arena >> 126 MB)" if args.config in ("c3", "c4")
               else "L2 flushed between timed steps"}
    for k in ("vocab", "d", "heads", "ffn", "layers", "seq", "dims"):
        if k in cfg:
            d[k] = cfg[k]
    return d



# ------------------------------------------------------------------------ HBM-bound kernel rooflines
def hbm_rooflines(lib, dev, rows, d, ffn, vocab, rank, hbm_peak, src):
    """Achieved bandwidth of the memory-bound kernels at the workload's shapes: algorithmic bytes
    (each operand read once, each output written once) over the CUDA-event time of one launch on the
    stream it runs on, L2 flushed (a 256 MB write) between launches."""
    import torch
    from see_ml_b200.engine import Context
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import opcases
    Op = F.Op
    rng = np.random.default_rng(3)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    out = []

    def timed(name, build, bytes_):
        Lo = opcases.Layout()
        prog = build(Lo)
        arena, ro = Lo.done()
        ctx = Context(arena.size, ro, device=dev.index)
        ctx.write(0, arena)
        pid = ctx.build(prog, mode=1)
        st = torch.cuda.ExternalStream(lib.seeml_b200_ctx_stream(ctx.h), device=dev)
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ts = []
        for it in range(6):
            with torch.cuda.stream(st):
                flush.fill_(it & 1)
                ev0.record()
                ctx.run(pid, 0, len(prog), sync=False)
                ev1.record()
            torch.cuda.synchronize()
            if it:
                ts.append(ev0.elapsed_time(ev1))
        ctx.close()
        ms = float(np.median(ts))
        gbs = bytes_ / (ms * 1e-3) / 1e9
        out.append({"kernel": name, "bound": "hbm", "algorithmic_bytes": int(bytes_), "ms_per_launch": ms, "achieved": gbs,
                    "peak": hbm_peak, "unit": "GB/s", "frac": gbs / hbm_peak, "peak_source": f"copy bandwidth, {src}"})

    I = opcases._ins
    rn = lambda *sh: rng.standard_normal(sh, dtype=np.float32)
    n = rows * ffn
    timed(f"swiglu forward (silu + mul) [{rows}x{ffn}]",
          lambda L: np.concatenate([I(Op.SILU_FWD, [L.put(rn(n)), (s_ := L.out(n))], [n]), I(Op.MUL, [s_, L.put(rn(n)), L.out(n)], [n])]),
          4 * 4 * n)
    n2 = rows * d
    timed(f"add [{rows}x{d}]", lambda L: I(Op.ADD, [L.put(rn(n2)), L.put(rn(n2)), L.out(n2)], [n2]), 12 * n2)

    def rms(L):
        dy, x, g, rs = L.put(rn(n2)), L.put(rn(n2)), L.put(rn(d), ro=True), L.put(np.abs(rn(rows)) + 0.5)
        return I(Op.RMSNORM_BWD, [dy, x, g, L.out(n2)], [rs, F.pack32(rows, d)])
    timed(f"rmsnorm backward [{rows}x{d}]", rms, 12 * n2)
    xr = min(rows, 4096)

    def xent(L):
        z, lab = L.put(rn(xr, vocab)), L.put(rng.integers(0, vocab, xr).astype(np.int32))
        loss, probs, seed = L.out(1), L.out(xr * vocab), L.out(1)
        return np.concatenate([I(Op.XENT_FWD, [z, lab, loss, probs], [xr, vocab]), I(Op.FILL, [seed, F.f32_bits(1.0)], [1]),
                               I(Op.XENT_BWD, [probs, lab, seed, z], [xr, vocab]), I(Op.FILL, [probs, 0], [4])])
    timed(f"softmax-xent forward + backward [{xr}x{vocab}]", xent, 8 * xr * vocab)

    def adam(L):
        sizes = [d * rank, rank * d, d * rank, rank * ffn, ffn * rank, rank * d] * 24
        return np.concatenate([I(Op.ADAMW, [L.put(rn(k)), L.put(rn(k)), L.put(np.zeros(k, np.float32)), L.put(np.zeros(k, np.float32))], [k])
                               for k in sizes])
    nparam = sum([d * rank, rank * d, d * rank, rank * ffn, ffn * rank, rank * d]) * 24
    timed(f"adamw, 144 adapter tensors in one launch ({nparam} parameters)", adam, 28 * nparam)
    return out


# ------------------------------------------------------------------------------- C5: MatMul / LoRA sweep
def run_sweep(args):
    """BASELINE configs[4]: Y = X.W + (alpha/r)(X.A).B with its backward (dX, dA, dB), fp32 in / out,
    M in {2048, 16384, 131072}, (K, N) in {(1024,1024), (1024,2816), (2816,1024), (4096,4096)}, r in {8,16,64},
    entries ~N(0,1). Each shape runs as the instruction sequences the compiler emits, in fused mode; the
    forward group and the backward group (dgrad + both weight gradients) are timed separately."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    import torch
    from see_ml_b200 import _lib as L
    from see_ml_b200.engine import Context, MODE_FUSED
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import opcases
    lib = L.lib()
    Op = F.Op
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    hbm, tf_burst, tf_sust, src = measured_peaks()
    gemm = GEMM_KINDS[args.gemm]
    I = opcases._ins
    rows_out, tot_fl, tot_ms = [], 0.0, 0.0
    Ms = [int(m) for m in args.sweep_m.split(",")]
    gen = torch.Generator(device=dev)
    for M in Ms:
        for (K, N) in [(1024, 1024), (1024, 2816), (2816, 1024), (4096, 4096)]:
            for r in (8, 16, 64):
                alpha = 2.0 * r
                Lo, cur = {}, 0
                def slot(name, count):
                    nonlocal cur
                    Lo[name] = cur
                    cur = F.align_up(cur + 4 * count, 256)
                for nm, cnt in (("x", M * K), ("a", K * r), ("b", r * N), ("g", M * N), ("c", M * N), ("t", M * r), ("u", M * N),
                                ("s", M * N), ("y", M * N), ("ds", M * N), ("dt", M * r), ("dB", r * N), ("dx1", M * K),
                                ("dA", K * r), ("dx2", M * K), ("dX", M * K)):
                    slot(nm, cnt)
                gen.manual_seed(M * 31 + K * 7 + N + r)
                W = torch.randn(K * N, generator=gen, device=dev, dtype=torch.float32)
                ctx = Context(cur + 4096, W.cpu().numpy().view(np.uint8), device=dev.index, gemm=gemm)
                del W
                base = lib.seeml_b200_ctx_arena(ctx.h)
                for nm, cnt in (("x", M * K), ("a", K * r), ("b", r * N), ("g", M * N)):
                    v = torch.randn(cnt, generator=gen, device=dev, dtype=torch.float32)
                    L.check(lib.seeml_b200_d2d(ctx.h, Lo[nm], v.data_ptr(), 4 * cnt))
                    L.check(lib.seeml_b200_sync(ctx.h))
                    del v
                w = F.RODATA_BIT | 0
                sc = F.f32_bits(alpha / r)
                o = Lo
                fwd = np.concatenate([I(Op.GEMM_NN, [o["x"], w, o["c"]], [M, N, K]), I(Op.GEMM_NN, [o["x"], o["a"], o["t"]], [M, r, K]),
                                      I(Op.GEMM_NN, [o["t"], o["b"], o["u"]], [M, N, r]), I(Op.SCALE, [o["u"], o["s"], sc], [M * N]),
                                      I(Op.ADD, [o["c"], o["s"], o["y"]], [M * N])])
                bwd = np.concatenate([I(Op.SCALE, [o["g"], o["ds"], sc], [M * N]), I(Op.GEMM_NT, [o["ds"], o["b"], o["dt"]], [M, r, N]),
                                      I(Op.GEMM_TN, [o["t"], o["ds"], o["dB"]], [r, N, M]), I(Op.GEMM_NT, [o["dt"], o["a"], o["dx1"]], [M, K, r]),
                                      I(Op.GEMM_TN, [o["x"], o["dt"], o["dA"]], [K, r, M]), I(Op.GEMM_NT, [o["g"], w, o["dx2"]], [M, K, N]),
                                      I(Op.ADD, [o["dx1"], o["dx2"], o["dX"]], [M * K])])
                prog = np.concatenate([fwd, bwd])
                pid = ctx.build(prog, mode=MODE_FUSED)
                st = torch.cuda.ExternalStream(lib.seeml_b200_ctx_stream(ctx.h), device=dev)
                ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
                tf_, tb_ = [], []
                for it in range(4):
                    with torch.cuda.stream(st):
                        ev[0].record()
                        ctx.run(pid, 0, len(fwd), sync=False)
                        ev[1].record()
                        ctx.run(pid, len(fwd), len(prog), sync=False)
                        ev[2].record()
                    torch.cuda.synchronize()
                    if it:
                        tf_.append(ev[0].elapsed_time(ev[1]))
                        tb_.append(ev[1].elapsed_time(ev[2]))
                ctx.close()
                f_ms, b_ms = float(np.median(tf_)), float(np.median(tb_))
                f_fl = 2.0 * M * K * N + 2.0 * M * K * r + 2.0 * M * r * N
                b_fl = 2.0 * M * K * N + 2.0 * (2.0 * M * N * r + 2.0 * M * K * r)
                rows_out.append({"M": M, "K": K, "N": N, "r": r, "forward_ms": f_ms, "backward_ms": b_ms,
                                 "forward_tflops": f_fl / (f_ms * 1e-3) / 1e12, "backward_tflops": b_fl / (b_ms * 1e-3) / 1e12,
                                 "forward_frac": f_fl / (f_ms * 1e-3) / 1e12 / tf_burst,
                                 "backward_frac": b_fl / (b_ms * 1e-3) / 1e12 / tf_burst})
                tot_fl += f_fl + b_fl
                tot_ms += f_ms + b_ms
    cpu = None
    if not args.no_cpu_baseline:
        from oracle import pyoracle as O
        kind = "reference" if O.have_ref() else "port"
        if kind == "reference":
            O.ref().ref_set_threads(os.cpu_count() or 1)
        rng = np.random.default_rng(0)
        cl = []
        Mc = 2048
        for (K, N) in [(1024, 1024), (1024, 2816), (2816, 1024), (4096, 4096)]:
            Lo = opcases.Layout()
            x, g_ = Lo.put(rng.standard_normal((Mc, K), dtype=np.float32)), Lo.put(rng.standard_normal((Mc, N), dtype=np.float32))
            wv = Lo.put(rng.standard_normal((K, N), dtype=np.float32), ro=True)
            y, dx = Lo.out(Mc * N), Lo.out(Mc * K)
            arena, ro = Lo.done()
            res = {}
            for nm, ins in (("GemmNN", I(Op.GEMM_NN, [x, wv, y], [Mc, N, K])), ("GemmNT", I(Op.GEMM_NT, [g_, wv, dx], [Mc, K, N]))):
                t0 = time.perf_counter()
                O.execute("ref" if kind == "reference" else "port", ins, arena, ro)
                res[nm] = 2.0 * Mc * K * N / (time.perf_counter() - t0) / 1e9
            cl.append({"M": Mc, "K": K, "N": N, **{k + "_gflops": v for k, v in res.items()}})
        cpu = {"value": float(np.mean([c["GemmNN_gflops"] for c in cl])) / 1e3, "unit": "TFLOP/s", "cores": os.cpu_count() if kind == "reference" else 1,
               "kind": kind, "sample": "kernels::GemmNN / GemmNT, one call per (K, N) at M = 2048 (the rate does not depend on M)", "shapes": cl}
    value = tot_fl / (tot_ms * 1e-3) / 1e12
    best = max(rows_out, key=lambda r_: r_["forward_tflops"])
    line = {"metric": "MatMul/LoRA sweep: algorithmic TFLOP/s, forward + backward over all shapes", "value": value, "unit": "TFLOP/s",
            "n_gpus": 1, "steps": 3, "warmup": 1, "ms_per_step": tot_ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": args.gemm, "data": "synthetic", "config": {"workload": "c5", "M": Ms, "mode": "fused", "l2": "operands exceed L2 except at M = 2048"},
            "roofline": {"bound": "tensor", "kernel": f"best forward shape M={best['M']} K={best['K']} N={best['N']} r={best['r']}",
                         "achieved": best["forward_tflops"], "peak": tf_burst, "unit": "TFLOP/s", "frac": best["forward_frac"],
                         "peak_source": f"bf16 dense burst, {src}", "traffic": None},
            "sweep": rows_out, "cpu_baseline": cpu, "gpu_launches": None, "e2e": None}
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------- seeml-bench shaped report (C1-C3)
def run_seeml_bench(args):
    """The reference's benchmark report (tool/seeml_bench.cc:289-334) for this backend: per fixture the plan
    statistics, load time, and - by steps regression between two run lengths, medians over repeats - the
    per-step time, rows/s, GEMM GFLOP/s and the forward / backward / optimiser split of StepTimings."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    from see_ml_b200 import _lib as L
    from see_ml_b200.engine import Dataset, UpdateEngine
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import cfgcases
    lib = L.lib()
    hasher = lambda b, o: int(lib.seeml_b200_plan_self_hash(np.frombuffer(b, np.uint8).ctypes.data, len(b), o))
    lo, hi, repeats = args.steps_lo, args.steps_hi, 3
    fixtures = {}
    for name in args.seeml_bench.split(","):
        cfg, model, spec = cfgcases.model_and_spec(name)
        t0 = time.perf_counter()
        blob, _ = PS.synthesize(model, spec, hasher=hasher)
        compile_ms = (time.perf_counter() - t0) * 1e3
        plan = F.parse_plan(blob)
        h = plan.header
        flops, _ = plan_work(blob)
        e = UpdateEngine(int(os.environ.get("LOCAL_RANK", "0")), 1, GEMM_KINDS[args.gemm])
        t0 = time.perf_counter()
        e.load_from_memory(blob)
        load_ms = (time.perf_counter() - t0) * 1e3
        x, y = cfgcases.corpus(name)
        ds = Dataset.from_memory(x, y) if y is not None else Dataset.from_tokens(x)
        e.train(ds, 4)
        e.enable_step_timing(True)
        e.reset_step_timings()
        slopes, life = [], []
        for _ in range(repeats):
            t0 = time.perf_counter(); e.train(ds, lo); w_lo = (time.perf_counter() - t0) * 1e3
            t0 = time.perf_counter(); e.train(ds, hi); w_hi = (time.perf_counter() - t0) * 1e3
            slopes.append((w_hi - w_lo) / (hi - lo))
            life.append(w_lo - slopes[-1] * lo)
        steps, fwd, bwd, opt = e.step_timings()
        step_ms = float(np.median(slopes))
        t0 = time.perf_counter(); e.run_merge(); merge_ms = (time.perf_counter() - t0) * 1e3
        fixtures[name] = {"kind": cfg["kind"], "batch_rows": int(h.batch), "seq": int(h.seq_len), "plan_bytes": len(blob),
                          "arena_bytes": int(h.arena_size), "persistent_bytes": int(h.persistent_size), "rodata_bytes": int(h.rodata_size),
                          "train_instructions": int(h.train_instr_count), "gemm_flops_per_step": int(flops),
                          "compile_ms": round(compile_ms, 2), "load_ms": round(load_ms, 3),
                          "threads": {"gpu": {"step_ms": round(step_ms, 3), "lifecycle_ms": round(float(np.median(life)), 2),
                                              "rows_per_s": round(1000.0 * h.batch / step_ms), "gemm_gflops": round(flops / (step_ms * 1e6), 1),
                                              "fwd_ms": round(1e3 * fwd / max(steps, 1), 3), "bwd_ms": round(1e3 * bwd / max(steps, 1), 3),
                                              "opt_ms": round(1e3 * opt / max(steps, 1), 3)}},
                          "merge_ms": round(merge_ms, 3)}
        e.close()
    print(json.dumps({"seeml_version": "seeml_b200", "schema": 1,
                      "config": {"steps_lo": lo, "steps_hi": hi, "repeats": repeats, "threads": "gpu"}, "fixtures": fixtures}), flush=True)


# ------------------------------------------------------------------------------------ our arm
def run_ours(args, cfg):
    import torch
    import torch.distributed as dist
    from see_ml_b200 import _lib as L
    from see_ml_b200.dp import DataParallelTrainer
    from see_ml_b200.engine import Context

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the backend has no CPU fallback")
    torch.cuda.set_device(local_rank)
    group = None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", local_rank))
        group = dist.group.WORLD
    lib = L.lib()
    hasher = lambda b, o: int(lib.seeml_b200_plan_self_hash(np.frombuffer(b, np.uint8).ctypes.data, len(b), o))
    model = build_model(cfg)
    rows = cfg["rows"] if cfg["kind"] == "mlp" else cfg["seqs"] * cfg["seq"]
    K = max(cfg["chunks"], world)
    blob, _ = build_plan(cfg, model, rows, hasher)
    gemm = GEMM_KINDS[args.gemm]
    tr = DataParallelTrainer(blob, K, rank, world, local_rank, mode=1 if args.fused else 0, gemm=gemm,
                             group=group)
    local = tr.local
    n_steps = args.warmup + args.steps
    dev = torch.device("cuda", local_rank)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)   # > 126 MB L2

    def batches_for(step):   # this rank's chunks of the global step (seeded per step)
        tok, lab = synth_batches(cfg, rows, K, seed=1000 + step)
        return tok[rank * local:(rank + 1) * local], lab[rank * local:(rank + 1) * local]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        if world == 1:
            return ms
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- arm A: inputs resident in HBM ----------------------------------------------------
    host = [batches_for(s) for s in range(min(n_steps, 4))]
    resident = [(torch.from_numpy(np.ascontiguousarray(t)).to(dev), torch.from_numpy(np.ascontiguousarray(l)).to(dev))
                for t, l in host]
    for s in range(args.warmup):
        tr.step_resident(*resident[s % len(resident)])
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches = 0
    with torch.cuda.stream(tr.stream):
        ev0.record()
        for s in range(args.steps):
            if args.config in ("c1", "c2"):
                flush.fill_(s & 1)
            tr.step_resident(*resident[(args.warmup + s) % len(resident)])
            launches += tr.launches
        ev1.record()
    barrier()
    ms_total = max_over_ranks(ev0.elapsed_time(ev1))
    clocks = sampler.stop() if rank == 0 else None
    loss_a = tr.engine.loss_value()
    # digest of the persistent segment (adapters + optimiser state) after warm-up + timed steps:
    # equal across GPU counts for equal --steps/--warmup, since the gradient tree is fixed
    import hashlib
    params_digest = hashlib.sha256(tr.persistent().tobytes()).hexdigest()[:16]
    ms_step = ms_total / args.steps
    tokens = rows * K
    value = tokens / (ms_step * 1e-3)

    # ---- arm B: end to end through the public API from host buffers --------------------------
    e2e = None
    if not args.no_e2e:
        e2e_steps = max(1, args.steps)
        hb = [batches_for(100 + s) for s in range(e2e_steps + 1)]
        for _ in range(min(args.warmup, 2)):
            tr.step(*hb[0])
        barrier()
        with torch.cuda.stream(tr.stream):
            ev0.record()
            for s in range(e2e_steps):
                tr.step(*hb[1 + s])
            ev1.record()
        barrier()
        e2e_ms = max_over_ranks(ev0.elapsed_time(ev1)) / e2e_steps
        e2e = {"value": tokens / (e2e_ms * 1e-3), "unit": "tokens/s",
               "h2d_bytes_per_step": int(tr.h2d_bytes * world), "d2h_bytes_per_step": int(tr.d2h_bytes * world),
               "ms_per_step": e2e_ms, "steps": e2e_steps}

    if rank == 0:
        hbm, tf_burst, tf_sust, src = measured_peaks()
        flops, top = plan_work(blob)
        # roofline of the dominant kernel: the GEMM shape that carries the most FLOPs of the
        # stream, against a frozen weight as in the stream, timed alone with CUDA events on the
        # stream it is launched on
        roof = None
        if top is not None and not args.no_e2e:
            fl, (m, n, k) = top
            rng = np.random.default_rng(0)
            w = (rng.standard_normal(k * n, dtype=np.float32) * 0.02).view(np.uint8)
            ctx = Context((m * k + m * n) * 4 + 4096, w, device=local_rank, gemm=gemm)
            gi = np.zeros(1, dtype=F.INSTR_DTYPE)
            gi["in"] = F.NULL_REF
            gi["opcode"] = 2    # A[M,K] @ B[N,K]^T: both operands K-major, the tensor-core form
            a_off, c_off = 0, F.align_up(m * k * 4)
            gi["in"][0, :3] = (a_off, F.RODATA_BIT | 0, c_off)
            gi["out"][0] = (m, n, k)
            ctx.write(a_off, rng.standard_normal(m * k, dtype=np.float32))
            pid = ctx.build(gi)
            st = torch.cuda.ExternalStream(lib.seeml_b200_ctx_stream(ctx.h), device=dev)
            for _ in range(3):
                ctx.run(pid, 0, 1)
            reps = 10
            with torch.cuda.stream(st):
                ev0.record()
                for _ in range(reps):
                    ctx.run(pid, 0, 1, sync=False)
                ev1.record()
            torch.cuda.synchronize()
            t_ms = ev0.elapsed_time(ev1) / reps
            ach = fl / (t_ms * 1e-3) / 1e12
            issue = {"tf32x3": 3, "f16x2": 3, "tf32": 1}.get(args.gemm)
            roof = {"bound": "tensor", "kernel": f"gemm_tc_kernel M={m} N={n} K={k} ({args.gemm})",
                    "achieved": ach, "peak": tf_burst, "unit": "TFLOP/s", "frac": ach / tf_burst,
                    "peak_source": f"bf16 dense burst, {src}", "traffic": profiled_traffic(m, n, k),
                    "ms_per_launch": t_ms, "algorithmic_bytes": 4 * (m * k + n * k + m * n),
                    "mma_products_per_flop": issue,
                    "note": "achieved counts 2*M*N*K once; the f32-parity path issues three kind::tf32 "
                            "products per step (tf32 runs at half the bf16 rate), so 1/6 of the bf16 "
                            "peak is the ceiling of this column for tf32x3"}
            ctx.close()
        hbm_lines = None
        if not args.no_e2e and cfg["kind"] == "llama":
            hbm_lines = hbm_rooflines(lib, dev, min(rows, 16384), cfg["d"], cfg["ffn"], cfg["vocab"], cfg["rank"], hbm, src)
        cpu = None
        if world == 1 and not args.no_cpu_baseline:
            cpu, _ = cpu_reference_sample(cfg, model, 1, 0, os.cpu_count() or 1)
        line = {"metric": "train tokens/sec per update step", "value": value, "unit": "tokens/s",
                "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                "dtype": {"tf32x3": "f32 (3xTF32 tensor-core split, f32 accumulate)",
                          "f16x2": "f32 (two-term fp16 split of scaled operands, three products, f32 accumulate)",
                          "simt": "f32", "tf32": "tf32"}[args.gemm],
                "data": "synthetic", "config": workload_config(args, cfg),
                "mode": "fused" if args.fused else "contract",
                "gemm_tflops_algorithmic": flops * K / (ms_step * 1e-3) / 1e12,
                "loss": loss_a, "params_sha256_16": params_digest, "e2e": e2e, "gpu_launches": int(launches),
                "clocks": clocks, "roofline": roof, "rooflines_hbm": hbm_lines, "cpu_baseline": cpu}
        print(json.dumps(line), flush=True)
    tr.close()
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="c4", choices=sorted(CONFIGS) + ["c5"])
    ap.add_argument("--sweep-m", default="2048,16384,131072", help="row counts of the c5 sweep")
    ap.add_argument("--seeml-bench", default="", help="comma-separated fixtures (c1,c2,c3): print the seeml-bench shaped report")
    ap.add_argument("--ref-threads", type=int, default=0, help="host threads of the reference arm (0 = all cores)")
    ap.add_argument("--steps-lo", type=int, default=20)
    ap.add_argument("--steps-hi", type=int, default=80)
    ap.add_argument("--gemm", default="f16x2", choices=sorted(GEMM_KINDS))
    ap.add_argument("--fused", type=int, default=1)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--chunks", type=int, default=0, help="override chunks per step (profiling aid)")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer arm (profiling aid)")
    args = ap.parse_args()
    if args.seeml_bench:
        return run_seeml_bench(args)
    if args.config == "c5":
        return run_sweep(args)
    cfg = dict(CONFIGS[args.config])
    if args.chunks:
        cfg["chunks"] = args.chunks
    if args.impl == "reference":
        run_reference(args, cfg)
    else:
        run_ours(args, cfg)


if __name__ == "__main__":
    main()
