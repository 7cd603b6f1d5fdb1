#!/usr/bin/env python
"""Benchmark of the compiled training step (fwd + bwd + clip + AdamW).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--config c3]

One JSON line on stdout (rank 0).  `value` is tokens/s of the whole job with the
batch already on the device (CUDA-graph replays between two CUDA events, max
over ranks); `e2e` is the same metric through the public API with host arrays
(`ct.replay_step(x, y)`: pinned H2D of ids/targets and the D2H loss read every
step; `e2e.pipelined_value` is the same loop with `ct.replay_step_async`, which
reads step i's loss after step i+1 is queued).  N > 1 (launched by torchrun): data parallel + ZeRO-1, one process per
GPU, weak scaling (fixed per-GPU batch).  `--impl reference` times the numpy
restatement of the reference's step on the host cores (the only place besides
`cpu_baseline` where this file runs anything from oracle/).

Other keys of the line: `roofline` (all GEMM launches of one eager step, per-op CUDA events, against the
sustained cuBLAS figure), `kernels` (every op kind's time and share), `attn_bwd` (the isolated causal
flash-attention backward at Q/dO [4,24,2048,64], K/V [4,8,2048,64]: ms, TFLOP/s, fraction of the measured
burst and sustained bf16 rates), `cpu_baseline` (bounded sample of the workload, extrapolated; numpy version,
BLAS threads and cores stated) and `c1_measured` (the reference's own CPU-runnable case run in full on the
host cores, with the same case on the GPU in fp32 beside it).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

RANK = int(os.environ.get("RANK", "0"))
WORLD = int(os.environ.get("WORLD_SIZE", "1"))
LOCAL_RANK = int(os.environ.get("LOCAL_RANK", "0"))
if WORLD > 1 and "AXIS_KEEP_VISIBLE" not in os.environ:
    # one GPU per process, as the engine expects (axis/_csrc/runtime.cu:57-65 is process-global)
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    devs = vis.split(",") if vis else [str(i) for i in range(64)]
    os.environ["CUDA_VISIBLE_DEVICES"] = devs[LOCAL_RANK % len(devs)]

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CONFIGS = {
    # BASELINE configs[2]: the 1B-class step the headline metric is quoted on
    "c3": dict(cfg=dict(vocab_size=32000, dim=1536, n_layers=48, n_heads=24, n_kv_heads=8, mlp_hidden=4096,
                        tie_embeddings=True), B=4, T=2048, dtype="bf16", ignore=0.05, lora=0, lr=3e-4,
               name="1B-class V32000 D1536 L48 H24/KV8 MLP4096 B4 T2048 bf16+fp32 masters, graph replay"),
    # BASELINE configs[0]: the reference's CPU-runnable plumbing case
    "c1": dict(cfg=dict(vocab_size=1024, dim=256, n_layers=4, n_heads=8, n_kv_heads=4, mlp_hidden=688,
                        tie_embeddings=True), B=2, T=256, dtype="fp32", ignore=0.10, lora=0, lr=3e-4,
               name="V1024 D256 L4 H8/KV4 MLP688 B2 T256 fp32"),
    # BASELINE configs[4]: LoRA fine-tune on a long sequence
    "c5": dict(cfg=dict(vocab_size=32000, dim=1536, n_layers=48, n_heads=24, n_kv_heads=8, mlp_hidden=4096,
                        tie_embeddings=True), B=1, T=8192, dtype="bf16", ignore=0.0, lora=16, lr=1e-4,
               name="1B-class LoRA r16 a32 B1 T8192 bf16, 40% prompt masked"),
    # BASELINE configs[3]: 7B data parallel + ZeRO-1 (needs >= 2 GPUs for the optimizer state)
    "c4": dict(cfg=dict(vocab_size=32000, dim=4096, n_layers=32, n_heads=32, n_kv_heads=32, mlp_hidden=11008,
                        tie_embeddings=True), B=2, T=4096, dtype="bf16", ignore=0.0, lora=0, lr=3e-4,
               name="7B-class V32000 D4096 L32 H32/KV32 MLP11008 B2/GPU T4096 bf16 ZeRO-1"),
    # small stand-in used by smoke runs
    "tiny": dict(cfg=dict(vocab_size=512, dim=256, n_layers=2, n_heads=4, n_kv_heads=2, mlp_hidden=384,
                          tie_embeddings=True), B=2, T=256, dtype="bf16", ignore=0.05, lora=0, lr=3e-4,
                 name="tiny"),
}
METRIC = "train tok/s (fwd+bwd+AdamW)"
# tok/s the reference publishes for the same model/config on ONE A100-80GB (its README.md:148-163): the only published
# numbers for this metric; `vs_baseline` = per-GPU tok/s here / that figure (other hardware, see `baseline_note`)
PUBLISHED_TOK_S = {"c3": 10279.0}
# DRAM bytes per GEMM launch (dram__bytes_read.sum + dram__bytes_write.sum, mean over the GEMM launches of one step)
# from an ncu capture of `bench.py --layers 2` of the same workload, and where its summary is committed
GEMM_TRAFFIC = {"c3": (148.1e6, "ncu dram__bytes_read.sum + dram__bytes_write.sum of the GEMM launches of 2- and 3-layer variants, "
                               "scaled to 48 layers: profiles/gemm_step_dram_traffic_1b.md")}


def step_flops(c) -> float:
    """6 * dense params * tokens + 7 * B*H*T^2*DH*L (causal attention, fwd+bwd)."""
    cfg, B, T = c["cfg"], c["B"], c["T"]
    D, L, H, V, MLP = cfg["dim"], cfg["n_layers"], cfg["n_heads"], cfg["vocab_size"], cfg["mlp_hidden"]
    KV = cfg["n_kv_heads"]
    DH = D // H
    per_layer = D * H * DH + 2 * D * KV * DH + H * DH * D + 3 * D * MLP
    dense = L * per_layer + V * D
    mult = 4 if c["lora"] else 6
    return mult * dense * B * T + 7.0 * B * H * T * T * DH * L


def make_weights(cfg, seed):
    from axis_b200.model import Transformer
    return Transformer(cfg["vocab_size"], cfg["dim"], cfg["n_layers"], cfg["n_heads"], cfg["n_kv_heads"],
                       cfg["mlp_hidden"], cfg["tie_embeddings"], seed=seed, std=0.02)


def make_batch(c, rng):
    V, B, T = c["cfg"]["vocab_size"], c["B"], c["T"]
    x = rng.integers(0, V, size=(B, T)).astype(np.int64)
    y = rng.integers(0, V, size=(B, T)).astype(np.int64)
    if c["lora"]:
        y[:, :int(0.4 * T)] = -1
    elif c["ignore"] > 0:
        y = np.where(rng.random((B, T)) < c["ignore"], -1, y)
    return x, y


class ClockSampler:
    """nvidia-smi samples every 200 ms while the timed region runs (read-only queries)."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc = [], None

    def start(self):
        try:
            dev = os.environ.get("CUDA_VISIBLE_DEVICES", "0").split(",")[0] or "0"
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", dev], stdout=subprocess.PIPE, text=True)
            self.th = threading.Thread(target=self._read, daemon=True)
            self.th.start()
        except (OSError, ValueError):
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([f.strip() for f in line.split(",")])

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], None, set()
        for r in self.rows:
            try:
                sm.append(float(r[0])); mx = float(r[1])
            except (ValueError, IndexError):
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


def blas_threads():
    """Threads the BLAS behind numpy will use, as reported by threadpoolctl (else from the environment)."""
    try:
        from threadpoolctl import threadpool_info
        n = [int(p.get("num_threads", 0)) for p in threadpool_info() if p.get("user_api") == "blas"]
        if n:
            return max(n)
    except Exception:
        pass
    for k in ("OPENBLAS_NUM_THREADS", "OMP_NUM_THREADS", "MKL_NUM_THREADS"):
        if os.environ.get(k, "").isdigit():
            return int(os.environ[k])
    return None


def host_cores():
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def _oracle_steps(cfg, c, B, T, timed):
    """One warm-up step, then `timed` steps of the numpy restatement of the reference's training step; their times."""
    from oracle import step_numpy as O
    w = O.init_weights(cfg, seed=1)
    kw = {}
    if c["lora"]:
        tg = ("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj")
        w.update(O.init_lora(cfg, c["lora"], tg))
        kw = dict(lora_rank=c["lora"], lora_alpha=2.0 * c["lora"], lora_targets=tg)
    model = O.OracleTransformer(cfg, w, **kw)
    opt = O.OracleAdamW(model, lr=c["lr"])
    rng = np.random.default_rng(0)
    x, y = O.make_batch(rng, cfg["vocab_size"], B, T, c["ignore"])
    O.train_step(model, opt, x, y, max_grad_norm=1.0)             # warm: BLAS threads up, pages touched
    out = []
    for _ in range(timed):
        t0 = time.perf_counter()
        O.train_step(model, opt, x, y, max_grad_norm=1.0)
        out.append(time.perf_counter() - t0)
    return out


def cpu_reference(c, timed=3):
    """The numpy restatement of the reference's step on the host cores.  A workload that fits the time budget
    (dim <= 512) runs in full: 1 warm-up + `timed` steps, median.  A larger one runs a bounded sample — the same
    widths and vocabulary at batch 1, a shorter sequence and 1 and 2 layers, each 1 warm-up + `timed` steps,
    medians — and is extrapolated linearly in layers and tokens (attention by its flops at the full length)."""
    cfg = dict(c["cfg"])
    L_full, B_full, T_full = cfg["n_layers"], c["B"], c["T"]
    small = cfg["dim"] <= 512
    T = T_full if small else min(T_full, 512)
    B = B_full if small else 1
    med = {}
    for L in ((L_full,) if small else (1, 2)):
        cfg["n_layers"] = L
        med[L] = float(np.median(_oracle_steps(cfg, c, B, T, timed)))
    if small:
        step_s = med[L_full]
        sample = f"full workload, median of {timed} timed steps after 1 warm-up"
    else:
        per_layer = max(med[2] - med[1], 1e-9)
        # attention is quadratic in T: scale the per-layer time by the flop ratio at the full T
        H, DH, D, MLP, KV = cfg["n_heads"], cfg["dim"] // cfg["n_heads"], cfg["dim"], cfg["mlp_hidden"], cfg["n_kv_heads"]
        lin = 6.0 * (D * H * DH + 2 * D * KV * DH + H * DH * D + 3 * D * MLP)
        att = lambda t: 7.0 * H * t * DH
        scale_T = (lin + att(T_full)) / (lin + att(T))
        head = max(med[1] - per_layer, 0.0)
        step_s = (head + L_full * per_layer * scale_T) * (B_full * T_full) / (B * T)
        sample = (f"B={B} T={T} with 1 and 2 layers (same widths/vocab), median of {timed} timed steps after 1 warm-up "
                  f"each; extrapolated to L={L_full} B={B_full} T={T_full} (linear in layers and tokens, attention by flops)")
    return {"value": c["B"] * c["T"] / step_s, "unit": "tok/s", "cores": host_cores(), "kind": "port",
            "sample": sample, "step_s_est": step_s, "numpy": np.__version__, "blas_threads": blas_threads()}


def cpu_c1_measured(timed=3):
    """The reference's own CPU-runnable case (vocab 1024, dim 256, 4 layers, batch 2 x seq 256, fp32) run in full on
    the host cores: 1 warm-up + 3 timed steps, tok/s = 512 / median step time."""
    c = CONFIGS["c1"]
    ts = _oracle_steps(dict(c["cfg"]), c, c["B"], c["T"], timed)
    med = float(np.median(ts))
    return {"workload": c["name"], "value": c["B"] * c["T"] / med, "unit": "tok/s", "step_s": med, "steps_timed": timed,
            "cores": host_cores(), "numpy": np.__version__, "blas_threads": blas_threads(), "kind": "port"}


def run_config(c, args, zero):
    """`config` of the JSON line: the same keys from both arms."""
    return {"workload": c["name"], "parallelism": f"dp{WORLD}" + ("+zero1" if zero else ""),
            "l2": "working set per step far exceeds the 126 MB L2 (no flush needed)",
            "global_batch": c["B"] * WORLD, "seq_len": c["T"],
            "recompute_blocks": bool(args.recompute), "overlap_dw": not args.no_overlap_dw and not c["lora"] and not args.recompute}


def reduce_max(val: float) -> float:
    if WORLD == 1:
        return val
    import torch
    import torch.distributed as dist
    t = torch.tensor([val], dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t[0])


def barrier():
    if WORLD > 1:
        import torch.distributed as dist
        dist.barrier()


_RESULT_FD = None


def _guard_stdout():
    """Libraries loaded below (NCCL with NCCL_DEBUG set in the environment, for one) may write to
    file descriptor 1.  The contract is ONE JSON line on stdout, so everything else is sent to stderr
    and the result line is written to a private copy of the original descriptor."""
    global _RESULT_FD
    sys.stdout.flush()
    _RESULT_FD = os.dup(1)
    os.dup2(2, 1)


def emit(line):
    data = (json.dumps(line) + "\n").encode()
    if _RESULT_FD is None:
        sys.stdout.write(data.decode()); sys.stdout.flush()
    else:
        os.write(_RESULT_FD, data)


def main():
    _guard_stdout()
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="axis_b200")
    ap.add_argument("--config", default="c3")
    ap.add_argument("--zero", type=int, default=1)
    ap.add_argument("--recompute", action="store_true",
                    help="keep one set of activations and re-run each block's forward inside the backward")
    ap.add_argument("--no-overlap-dw", action="store_true",
                    help="run the weight-gradient GEMMs inline instead of on the side stream")
    ap.add_argument("--batch", type=int, default=0, help="sequences per GPU (default: the configuration's)")
    ap.add_argument("--layers", type=int, default=0,
                    help="run a variant of the workload with this many layers (profiling captures; not the benchmark)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-kernel-table", action="store_true")
    args = ap.parse_args()
    c = dict(CONFIGS[args.config])
    c["key"] = args.config
    if args.layers:
        c["cfg"] = dict(c["cfg"], n_layers=args.layers)
        c["name"] = c["name"].replace(f"L{CONFIGS[args.config]['cfg']['n_layers']}", f"L{args.layers}") + f" ({args.layers}-layer variant)"
        c["key"] = None
    if args.batch:
        c["name"] = c["name"].replace(f"B{c['B']}", f"B{args.batch}")
        c["B"] = args.batch
    W = max(args.warmup, 3)
    K = max(args.steps, 1)

    zero = args.zero if WORLD > 1 else 0
    if args.impl == "reference":
        if RANK != 0:
            return
        cb = cpu_reference(c)
        line = {"metric": METRIC, "value": cb["value"], "unit": "tok/s", "n_gpus": args.gpus, "steps": K, "warmup": W,
                "ms_per_step": cb["step_s_est"] * 1e3, "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "f32", "data": "synthetic", "impl": "reference",
                "config": run_config(c, args, zero), "cpu_baseline": cb,
                "e2e": {"value": cb["value"], "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                "gpu_launches": 0}
        if args.config == "c3":
            line["c1_measured"] = cpu_c1_measured()
        emit(line)
        return

    if WORLD > 1:
        import torch.distributed as dist
        dist.init_process_group("gloo", init_method=f"tcp://{os.environ.get('MASTER_ADDR', '127.0.0.1')}:"
                                f"{os.environ.get('MASTER_PORT', '29500')}", rank=RANK, world_size=WORLD)

    from axis_b200.compile import CompiledTransformer, compile_model
    if c["cfg"]["dim"] >= 4096 and not c["lora"]:
        # 7B-class: weights are drawn tensor by tensor while they are uploaded (every rank would otherwise hold
        # 26 GB of fp32 host arrays at once)
        from axis_b200.model import lazy_weights
        ct = CompiledTransformer(None, c["cfg"], lazy_weights(c["cfg"], seed=42), c["B"], c["T"], dtype=c["dtype"], lr=c["lr"],
                                 max_grad_norm=1.0, grad_sync=WORLD > 1, zero_stage=zero, rank=RANK, world=WORLD,
                                 recompute_blocks=args.recompute, overlap_dw=not args.no_overlap_dw)
    else:
        model = make_weights(c["cfg"], seed=42)
        if c["lora"]:
            model.apply_lora(rank=c["lora"], alpha=2.0 * c["lora"])
        ct = compile_model(model, batch=c["B"], seq=c["T"], dtype=c["dtype"], lr=c["lr"], max_grad_norm=1.0,
                           grad_sync=WORLD > 1, zero_stage=zero, rank=RANK, world=WORLD,
                           recompute_blocks=args.recompute, overlap_dw=not args.no_overlap_dw)
        del model
    eng = ct.eng
    if WORLD > 1:
        import torch
        import torch.distributed as dist
        uid = torch.zeros(128, dtype=torch.uint8)
        if RANK == 0:
            uid = torch.frombuffer(bytearray(eng.nccl_id()), dtype=torch.uint8).clone()
        dist.broadcast(uid, src=0)
        eng.nccl_init(RANK, WORLD, bytes(uid.numpy().tobytes()), timeout_ms=120000)

    rng = np.random.default_rng(100 + RANK)
    batches = [make_batch(c, rng) for _ in range(4)]
    ct.capture()
    losses = []
    for i in range(W):
        losses.append(ct.replay_step(*batches[i % 4]))

    # ── device-resident throughput: K replays between two events ──
    clocks = ClockSampler()
    clocks.start()
    eng.sync(); barrier()
    eng.launch_count(reset=True)
    # graph replays timed by events inside the engine
    ms_dev = time_replays(eng, K)
    launches = eng.launch_count()
    ms_dev = reduce_max(ms_dev)
    barrier()
    # ── end to end through the public API: host arrays in, loss out, every step ──
    eng.sync(); barrier()
    t0 = time.perf_counter()
    for i in range(K):
        losses.append(ct.replay_step(*batches[i % 4]))
    eng.sync()
    e2e_s = reduce_max(time.perf_counter() - t0)
    # the same with the loss of step i read after step i+1 is queued (pinned read-back ring)
    eng.sync(); barrier()
    t0 = time.perf_counter()
    for i in range(K):
        ct.replay_step_async(*batches[i % 4])
    losses.append(ct.flush())
    e2e_async_s = reduce_max(time.perf_counter() - t0)
    clk = clocks.stop()

    tokens = c["B"] * c["T"] * WORLD
    value = tokens * K / (ms_dev / 1e3)
    e2e = tokens * K / e2e_s

    line = {"metric": METRIC, "value": value, "unit": "tok/s", "n_gpus": WORLD, "steps": K, "warmup": W,
            "ms_per_step": ms_dev / K, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": (value / PUBLISHED_TOK_S[args.config] / WORLD) if c["key"] in PUBLISHED_TOK_S and not args.batch else None,
            "dtype": c["dtype"], "data": "synthetic",
            "config": run_config(c, args, zero),
            "e2e": {"value": e2e, "unit": "tok/s", "h2d_bytes_per_step": 2 * 4 * c["B"] * c["T"],
                    "d2h_bytes_per_step": 4, "pipelined_value": tokens * K / e2e_async_s},
            "gpu_launches": int(launches), "clocks": clk, "loss_first": losses[0], "loss_last": losses[-1],
            "step_tflops": step_flops(c) * K / (ms_dev / 1e3) / 1e12 / 1.0,
            "device_status": eng.device_status()}
    if line["vs_baseline"] is not None:
        line["baseline_note"] = "reference's published 10,279 tok/s for this config was measured on 1x A100-80GB (its README.md:148-156)"

    if not args.no_kernel_table:
        # every rank runs the profiled step (it contains the collectives); rank 0 reports
        table = kernel_table(ct, c, batches[0])
        if RANK == 0:
            line.update(table)
    if RANK == 0 and not args.no_cpu_baseline and WORLD == 1:
        line["cpu_baseline"] = cpu_reference(c)
    if RANK == 0 and WORLD == 1 and c["key"] == "c3" and not args.no_kernel_table:
        # the second half of the metric: the isolated flash-attention backward (the engine is rebuilt for it, so last)
        ct.eng.shutdown()
        line["attn_bwd"] = attn_bwd_isolated()
        if not args.no_cpu_baseline:
            line["c1_measured"] = {"cpu": cpu_c1_measured(), "gpu_fp32": gpu_c1()}
        line["other_configs"] = {"c5": other_config("c5")}
    barrier()
    if RANK == 0:
        emit(line)
    if WORLD > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


def time_replays(eng, K):
    """K graph launches between two CUDA events on the engine stream (milliseconds)."""
    import ctypes
    lib = eng.lib
    if not hasattr(lib, "eng_time_replay"):
        raise RuntimeError("libaxeng.so lacks eng_time_replay")
    lib.eng_time_replay.argtypes = [ctypes.c_int, ctypes.POINTER(ctypes.c_float)]
    ms = ctypes.c_float(0)
    rc = lib.eng_time_replay(K, ctypes.byref(ms))
    if rc:
        raise RuntimeError(f"eng_time_replay rc={rc}: {eng.last_error()}")
    return float(ms.value)


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return d.get("hbm_gbs", 6650.0), d.get("bf16_tflops", 1590.0), d.get("bf16_tflops_sustained", 1400.0), "measured"
    return 6650.0, 1590.0, 1400.0, "fallback"


def attn_bwd_isolated(reps=20):
    """Causal flash-attention backward alone at the isolated-backward benchmark shape: Q/dO [4,24,2048,64],
    K/V [4,8,2048,64] bf16 ~N(0,1), scale 1/8, LSE from the forward on the same inputs; dQ/dK/dV out (dK/dV summed
    over each kv group).  L2 flushed between repetitions; flops = 5 * B*H*T^2*DH (causal half of 5 matmuls)."""
    from axis_b200 import engine as E
    from axis_b200.engine import Engine, op
    Bq, H, KV, T, DH = 4, 24, 8, 2048, 64
    eng = Engine()
    eng.alloc(4)
    rng = np.random.default_rng(2)

    def buf(n):
        i = eng.alloc(n, 2)
        eng.upload_raw(i, E.f32_to_bf16_bits(rng.standard_normal(n, dtype=np.float32)))
        return i
    nq, nk = Bq * T * H * DH, Bq * T * KV * DH
    q, k, v, do = buf(nq), buf(nk), buf(nk), buf(nq)
    o, lse, scr = eng.alloc(nq, 2), eng.alloc(Bq * H * T), eng.alloc(Bq * H * T + nq)
    dq, dk, dv = eng.alloc(nq, 2), eng.alloc(nk, 2), eng.alloc(nk, 2)
    eng.run([op(E.ATTN_FWD, a=q, b=k, d=v, c=o, sa=lse, m=T, n=DH, k=KV, batch=Bq, tb=H, dt=1, alpha=0.125)])
    plan = [op(E.ATTN_BWD, a=q, b=k, d=v, c=do, sa=lse, sb=o, tb=dq, sc=dk, oa=dv, ob=H, oc=scr,
               m=T, n=DH, k=KV, batch=Bq, dt=1, alpha=0.125)]
    for _ in range(3):
        eng.run(plan)
    ms = eng.time_plan(plan, reps=reps, flush_l2=True)
    st = eng.device_status()
    eng.shutdown()
    flops = 5.0 * Bq * H * T * T * DH
    hbm, tf_burst, tf_sus, src = peaks()
    tf = flops / (ms * 1e-3) / 1e12
    return {"shape": "Q/dO [4,24,2048,64] K/V [4,8,2048,64] bf16 causal GQA 3:1", "ms": ms, "tflops": tf, "flops": flops,
            "frac_burst": tf / tf_burst, "frac_sustained": tf / tf_sus, "peak_source": src, "reps": reps,
            "l2": "flushed between repetitions", "launches_per_call": 4, "device_status": st}


def other_config(key, steps=5, warmup=3):
    """A second configuration measured by this script itself in a child process (`bench.py --config <key>`), reduced
    to the figures that matter: the long-sequence adapter fine-tune (BASELINE configs[4]) next to the headline line."""
    import subprocess
    cmd = [sys.executable, os.path.abspath(__file__), "--config", key, "--steps", str(steps), "--warmup", str(warmup),
           "--no-cpu-baseline"]
    try:
        r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
        d = json.loads(r.stdout.strip().splitlines()[-1])
    except (subprocess.SubprocessError, ValueError, IndexError) as e:
        return {"error": f"{type(e).__name__}: {e}"[:200], "command": " ".join(cmd[1:])}
    gemm = sum(v["calls"] for k_, v in d.get("kernels", {}).items() if k_.startswith("GEMM") and k_ != "GEMM_XSEG")
    return {"workload": d["config"]["workload"], "metric": d["metric"], "value": d["value"], "unit": d["unit"],
            "ms_per_step": d["ms_per_step"], "steps": d["steps"], "warmup": d["warmup"], "gemm_launches_per_step": gemm,
            "gpu_launches": d["gpu_launches"], "loss_first": d["loss_first"], "loss_last": d["loss_last"],
            "clocks": d["clocks"], "device_status": d["device_status"], "command": "python bench.py " + " ".join(cmd[2:])}


def gpu_c1(steps=30):
    """The reference's CPU-runnable case on the GPU in fp32 (graph replay, host tokens in, loss out every step)."""
    from axis_b200.compile import compile_model
    c = CONFIGS["c1"]
    ct = compile_model(make_weights(c["cfg"], seed=42), batch=c["B"], seq=c["T"], dtype="fp32", lr=c["lr"], max_grad_norm=1.0)
    rng = np.random.default_rng(42)
    batches = [make_batch(c, rng) for _ in range(4)]
    ct.capture()
    for i in range(5):
        ct.replay_step(*batches[i % 4])
    ct.eng.sync()
    t0 = time.perf_counter()
    for i in range(steps):
        ct.replay_step(*batches[i % 4])
    ct.eng.sync()
    dt_ = time.perf_counter() - t0
    ct.eng.shutdown()
    return {"workload": c["name"], "value": c["B"] * c["T"] * steps / dt_, "unit": "tok/s", "ms_per_step": dt_ / steps * 1e3,
            "steps": steps, "how": "ct.replay_step with host arrays, wall clock"}


def kernel_table(ct, c, batch):
    """Per-op-kind device time of one eager step (CUDA events around every op), the GEMM
    roofline entry, and the isolated flash-attention backward at the benchmark shape."""
    from axis_b200 import engine as E
    eng = ct.eng
    hbm, tf_burst, tf_sus, src = peaks()
    ct._feed(*batch)
    eng.profile(True)
    eng.run(ct.plan_step, sync=True)
    prof = eng.profile_read()
    eng.profile(False)
    total = sum(v[0] for v in prof.values()) or 1.0
    gemm_kinds = ("GEMM", "GEMM_SB", "GEMM_EX", "GEMM_GROUP")
    gemm_ms = sum(prof.get(k, (0, 0))[0] for k in gemm_kinds)
    gemm_calls = sum(prof.get(k, (0, 0))[1] for k in gemm_kinds)
    gemm_flops, gemm_bytes = 0.0, 0.0       # algorithmic: 2 m n k; operands and results touched once
    for o in ct.plan_step:
        eo = 2 if o[13] == 1 else 4             # output element size (dt 1: bf16, dt 2: bf16 in / fp32 out)
        ei = 2 if o[13] >= 1 else 4
        if o[0] in (E.GEMM, E.GEMM_SB, E.GEMM_EX):
            m_, n_, k_, bt = o[5], o[6], o[7], max(o[8], 1)
            gemm_flops += 2.0 * m_ * n_ * k_ * bt
            gemm_bytes += bt * ((m_ * k_ + k_ * n_) * ei + m_ * n_ * eo * (2 if o[0] == E.GEMM_EX else 1))
        elif o[0] == E.GEMM_GROUP:
            # o = (kind, a, b, c, d, m, n, k, batch=count, tb, sa, sb, sc, dt, oa, ob, oc=mode, ...)
            m_, n_, k_, cnt, mode = o[5], o[6], o[7], o[8], o[16]
            if mode == 3:      # two independent problems: m = o[5], o[14]; n = o[6], o[15]; k = o[7]
                gemm_flops += 2.0 * k_ * (m_ * n_ + o[14] * o[15])
                gemm_bytes += ((m_ + o[14]) * k_ + k_ * (n_ + o[15])) * ei + (m_ * n_ + o[14] * o[15]) * eo
            elif mode == 4:    # gate and up projections of width n each; outputs g, u and h
                gemm_flops += 2.0 * m_ * 2 * n_ * k_
                gemm_bytes += (m_ * k_ + 2 * k_ * n_) * ei + 3 * m_ * n_ * eo
            else:
                extra = sum((o[14], o[15])[:cnt - 1])
                if mode == 1:  # one input, several outputs
                    gemm_flops += 2.0 * m_ * (n_ + extra) * k_
                    gemm_bytes += (m_ * k_ + k_ * (n_ + extra)) * ei + m_ * (n_ + extra) * eo
                else:          # one output summed over K-segments
                    gemm_flops += 2.0 * m_ * n_ * (k_ + extra)
                    gemm_bytes += (m_ * (k_ + extra) + (k_ + extra) * n_) * ei + m_ * n_ * eo
    achieved = gemm_flops / (gemm_ms / 1e3) / 1e12 if gemm_ms > 0 else 0.0
    # DRAM bytes per GEMM launch: not measurable from inside the process; the figure comes from an ncu capture of
    # the GEMM launches of a two-layer variant of this workload (summary and command: profiles/, named below)
    traffic, traffic_source = GEMM_TRAFFIC.get(c.get("key"), (None, None))
    out = {"roofline": {"bound": "tensor", "kernel": "k_gemm_tc2 / k_gemm_tc (tcgen05 bf16 GEMM, all GEMM ops of the step)",
                        "achieved": achieved, "peak": tf_sus, "unit": "TFLOP/s", "frac": achieved / tf_sus,
                        "peak_source": f"{src} (sustained cuBLAS bf16)", "launches": gemm_calls,
                        "avg_launch_ms": gemm_ms / max(gemm_calls, 1), "traffic": traffic, "traffic_source": traffic_source,
                        "algorithmic_bytes_per_launch": gemm_bytes / max(gemm_calls, 1)},
           "kernels": {k: {"ms": round(v[0], 3), "calls": v[1], "share": round(v[0] / total, 4)}
                       for k, v in sorted(prof.items(), key=lambda kv: -kv[1][0])}}
    return out


if __name__ == "__main__":
    main()
