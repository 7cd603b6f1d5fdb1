"""Per-kernel micro-benchmark through the C ABI.

    python opbench.py gemm --m 8192 --n 1536 --k 1536 --tb 0 --dt 1
    python opbench.py attn_bwd --B 4 --H 24 --KV 8 --T 2048 --DH 64
    python opbench.py rmsnorm_bwd --rows 8192 --dim 1536
    python opbench.py all            # the step's kernels at the 1B-class shapes
    python opbench.py rmsnorm --chain 8   # eight instances back to back in one timed plan

Each run prints one JSON line: mean milliseconds over `--reps` launches (CUDA
events on the engine stream, L2 flushed between launches unless --no-flush),
the algorithmic bytes or flops of the op, the achieved GB/s or TFLOP/s and
its fraction of the measured peak (MEASURED_PEAKS.json beside this file when
present, else 6650 GB/s / 1590 TFLOP/s).  `--check` also verifies the result
against a numpy evaluation on a sample of the output.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import numpy as np

from axis_b200 import engine as E
from axis_b200.engine import Engine, op

ROOT = os.path.dirname(os.path.abspath(__file__))


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return float(d.get("hbm_gbs", 6650.0)), float(d.get("bf16_tflops", 1590.0)), "measured"
    return 6650.0, 1590.0, "fallback"


class Bench:
    def __init__(self, reps, flush):
        self.eng = Engine()
        self.eng.alloc(4)
        self.reps, self.flush = reps, flush
        self.rng = np.random.default_rng(0)
        self.hbm, self.tf, self.src = peaks()

    def buf(self, n, dt, fill="randn", scale=1.0):
        """n elements of storage type dt (0 fp32, 1 bf16), filled on the host in pieces."""
        i = self.eng.alloc(n, 2 if dt else 4)
        step = 1 << 24
        for o in range(0, n, step):
            m = min(step, n - o)
            a = np.zeros(m, np.float32) if fill == "zero" else (self.rng.standard_normal(m, dtype=np.float32) * scale)
            if dt:
                self.eng.upload_raw(i, E.f32_to_bf16_bits(a), o * 2)
            else:
                self.eng.upload_raw(i, a, o * 4)
        return i

    def time(self, plan):
        for _ in range(3):
            self.eng.run(plan)
        return self.eng.time_plan(plan, reps=self.reps, flush_l2=self.flush)

    def report(self, name, ms, bytes_=None, flops=None, **extra):
        out = {"op": name, "ms": round(ms, 5), "reps": self.reps, "l2_flush": self.flush, "peak_source": self.src}
        if flops is not None:
            tf = flops / (ms * 1e-3) / 1e12
            out.update(bound="tensor", flops=flops, achieved_tflops=round(tf, 2), peak_tflops=self.tf, frac=round(tf / self.tf, 4))
        if bytes_ is not None:
            gb = bytes_ / (ms * 1e-3) / 1e9
            out.update(algorithmic_bytes=bytes_, achieved_gbs=round(gb, 1))
            if flops is None:
                out.update(bound="hbm", peak_gbs=self.hbm, frac=round(gb / self.hbm, 4))
        out.update(extra)
        out["device_status"] = self.eng.device_status()
        print(json.dumps(out), flush=True)
        return out


def run_gemm(b, m, n, k, tb, dt, fallback=0):
    ia = b.buf(m * k, 1 if dt else 0)
    ib = b.buf(k * n, 1 if dt else 0)
    ic = b.eng.alloc(m * n, 2 if dt == 1 else 4)
    b.eng.set_fallback(fallback)
    ms = b.time([op(E.GEMM_SB, a=ia, b=ib, c=ic, m=m, n=n, k=k, batch=1, tb=tb, dt=dt)])
    b.eng.set_fallback(0)
    return b.report(f"gemm tb={tb} dt={dt} {m}x{n}x{k}" + (" (general path)" if fallback else ""), ms,
                    bytes_=(m * k + k * n) * (2 if dt else 4) + m * n * (2 if dt == 1 else 4), flops=2.0 * m * n * k)


def run_attn(b, which, B, H, KV, T, DH, dt=1, fallback=0, check=False):
    es = 2 if dt else 4
    q, kk, v, do = (b.buf(B * T * H * DH, dt), b.buf(B * T * KV * DH, dt), b.buf(B * T * KV * DH, dt), b.buf(B * T * H * DH, dt))
    o, lse = b.eng.alloc(B * T * H * DH, es), b.eng.alloc(B * H * T)
    scr = b.eng.alloc(B * H * T + B * T * H * DH)
    dq, dk, dv = b.eng.alloc(B * T * H * DH, es), b.eng.alloc(B * T * KV * DH, es), b.eng.alloc(B * T * KV * DH, es)
    sc = 1.0 / np.sqrt(DH)
    fwd = [op(E.ATTN_FWD, a=q, b=kk, d=v, c=o, sa=lse, m=T, n=DH, k=KV, batch=B, tb=H, dt=dt, alpha=sc)]
    bwd = [op(E.ATTN_BWD, a=q, b=kk, d=v, c=do, sa=lse, sb=o, tb=dq, sc=dk, oa=dv, ob=H, oc=scr,
              m=T, n=DH, k=KV, batch=B, dt=dt, alpha=sc)]
    b.eng.set_fallback(fallback)
    b.eng.run(fwd)
    ms = b.time(fwd if which == "attn_fwd" else bwd)
    b.eng.set_fallback(0)
    mm = 2 if which == "attn_fwd" else 5
    flops = mm * 2.0 * T * T * DH * B * H * 0.5
    byts = (2 * B * T * H * DH + 2 * B * T * KV * DH) * es * (1 if which == "attn_fwd" else 2) + B * H * T * 4
    extra = {}
    if check:
        extra["check"] = check_attn(b, q, kk, v, do, o, lse, dq, dk, dv, B, H, KV, T, DH, dt)
    return b.report(f"{which} B{B} H{H} KV{KV} T{T} DH{DH}" + (" (general path)" if fallback else ""), ms,
                    bytes_=byts, flops=flops, **extra)


def check_attn(b, q, kk, v, do, o, lse, dq, dk, dv, B, H, KV, T, DH, dt):
    """Worst relative error over one (batch, kv group) slice against numpy in fp32."""
    e = b.eng
    get = (lambda i, sh: e.download_bf16(i, sh)) if dt else (lambda i, sh: e.download(i, sh))
    Q, Kk, V, DO = get(q, (B, T, H, DH)), get(kk, (B, T, KV, DH)), get(v, (B, T, KV, DH)), get(do, (B, T, H, DH))
    O_, DQ, DK, DV = get(o, (B, T, H, DH)), get(dq, (B, T, H, DH)), get(dk, (B, T, KV, DH)), get(dv, (B, T, KV, DH))
    LSE = e.download(lse, (B, H, T))
    rep, sc = H // KV, 1.0 / np.sqrt(DH)
    bb, g = B - 1, KV - 1
    mask = np.triu(np.full((T, T), -1e30, np.float32), 1)
    dk_ref = np.zeros((T, DH), np.float32); dv_ref = np.zeros((T, DH), np.float32)
    worst = {}
    rel = lambda a, r: float(np.abs(a - r).max() / (np.abs(r).max() + 1e-9))
    for hh in range(rep):
        h = g * rep + hh
        s = Q[bb, :, h] @ Kk[bb, :, g].T * np.float32(sc) + mask
        m = s.max(-1, keepdims=True); p = np.exp(s - m); l = p.sum(-1, keepdims=True); p /= l
        o_ref = p @ V[bb, :, g]
        dp = DO[bb, :, h] @ V[bb, :, g].T
        ds = p * (dp - (dp * p).sum(-1, keepdims=True))
        dv_ref += p.T @ DO[bb, :, h]; dk_ref += ds.T @ Q[bb, :, h] * np.float32(sc)
        worst["o"] = max(worst.get("o", 0), rel(O_[bb, :, h], o_ref))
        worst["lse"] = max(worst.get("lse", 0), float(np.abs(LSE[bb, h] - (m + np.log(l))[:, 0]).max()))
        worst["dq"] = max(worst.get("dq", 0), rel(DQ[bb, :, h], ds @ Kk[bb, :, g] * np.float32(sc)))
    worst["dk"] = rel(DK[bb, :, g], dk_ref); worst["dv"] = rel(DV[bb, :, g], dv_ref)
    return {k: round(v, 5) for k, v in worst.items()}


def run_rows(b, which, rows, dim, dt, chain=1):
    """chain > 1: that many instances on separate buffers in one timed plan (together far larger than L2),
    the figure is per instance — how the kernel runs inside a captured step, without the per-launch floor."""
    es = 2 if dt else 4
    plan = []
    for _ in range(chain):
        x, w, g, res = b.buf(rows * dim, dt), b.buf(dim, dt), b.buf(rows * dim, dt), b.buf(rows * dim, dt)
        y, dw, scr = b.eng.alloc(rows * dim, es), b.eng.alloc(dim), b.eng.alloc(296 * dim)
        if which == "rmsnorm":
            plan.append(op(E.RMSNORM, a=x, b=w, c=y, m=rows, n=dim, dt=dt, alpha=1e-5))
        else:
            plan.append(op(E.RMSNORM_BWD_ACC, a=x, b=w, d=g, c=y, tb=res, sa=dw, sb=scr, m=rows, n=dim, dt=dt, alpha=1e-5))
    ms = b.time(plan) / chain
    tag = f" (chain of {chain})" if chain > 1 else ""
    if which == "rmsnorm":
        return b.report(f"rmsnorm {rows}x{dim} dt={dt}{tag}", ms, bytes_=2 * rows * dim * es)
    return b.report(f"rmsnorm_bwd (dx + residual + dw) {rows}x{dim} dt={dt}{tag}", ms, bytes_=4 * rows * dim * es)


def run_elem(b, which, n, dt, B=4, T=2048, H=24, DH=64, chain=1):
    es = 2 if dt else 4
    tag = f" (chain of {chain})" if chain > 1 else ""
    if which == "rope":
        n = B * T * H * DH
        from axis_b200.compile import np as _np
        half = DH // 2
        ang = _np.outer(_np.arange(T, dtype=_np.float32), 1.0 / (10000.0 ** (_np.arange(half, dtype=_np.float32) / half)))
        cs, sn = b.eng.new_tensor(_np.cos(ang).astype(_np.float32)), b.eng.new_tensor(_np.sin(ang).astype(_np.float32))
        plan = []
        for _ in range(chain):
            x = b.buf(n, dt)
            plan.append(op(E.ROPE_BTHD, a=x, b=cs, d=sn, c=x, batch=B, m=T, k=H, n=DH, dt=dt))
        ms = b.time(plan) / chain
        return b.report(f"rope in place B{B} T{T} H{H} DH{DH} dt={dt}{tag}", ms, bytes_=2 * n * es)
    plan = []
    for _ in range(chain):
        a, c_, d = b.buf(n, dt), b.buf(n, dt), b.buf(n, dt)
        o1, o2 = b.eng.alloc(n, es), b.eng.alloc(n, es)
        if which == "silu":
            plan.append(op(E.SILU_MUL, a=a, b=c_, c=o1, n=n, dt=dt))
        else:
            plan.append(op(E.SILU_BWD, a=a, b=c_, d=d, c=o1, tb=o2, n=n, dt=dt))
    ms = b.time(plan) / chain
    if which == "silu":
        return b.report(f"silu_mul n={n} dt={dt}{tag}", ms, bytes_=3 * n * es)
    return b.report(f"silu_bwd n={n} dt={dt}{tag}", ms, bytes_=5 * n * es)


def run_ce(b, N, V, dt):
    es = 2 if dt else 4
    lg = b.buf(N * V, dt)
    tg = b.eng.alloc(N)
    b.eng.upload_tokens(tg, b.rng.integers(0, V, N), V)
    loss, den, scr = b.eng.alloc(1), b.eng.alloc(1), b.eng.alloc(N + 8)
    ms = b.time([op(E.CE_FUSED, a=lg, b=tg, c=lg, d=loss, sa=den, sb=scr, m=N, n=V, dt=dt)])
    return b.report(f"cross-entropy fwd+bwd in place {N}x{V} dt={dt}", ms, bytes_=2 * N * V * es)


def run_adamw(b, n):
    n = n // 1024 * 1024
    p, g = b.buf(n, 0, scale=0.02), b.buf(n, 0, scale=1e-3)
    m, v = b.eng.alloc_zero(n * 4), b.eng.alloc_zero(n * 4)
    mir = b.eng.alloc(n, 2)
    fl = b.eng.alloc(n // 1024, 1)
    b.eng.upload_raw(fl, np.ones(n // 1024, np.uint8))
    t, lr = b.eng.new_tensor(np.zeros(1, np.float32)), b.eng.new_tensor(np.array([3e-4], np.float32))
    part, ss, gn = b.eng.alloc(n // 8192 + 1), b.eng.alloc(1), b.eng.alloc(1)
    plan = [op(E.GNORM_FLAT, a=g, c=part, d=ss, ob=0, m=n // 1024, oa=0, tb=t),
            op(E.ADAMW_FLAT, a=p, b=g, c=m, d=v, m=n // 1024, k=0, sa=mir, sb=lr, tb=t, sc=fl, oa=ss, ob=1, oc=gn,
               alpha=1.0, beta=0.1, gamma=1e-8)]
    ms = b.time(plan)
    return b.report(f"clip + AdamW over a flat arena of {n} params", ms, bytes_=34 * n)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("what")
    for a, d in (("m", 8192), ("n", 1536), ("k", 1536), ("tb", 0), ("dt", 1), ("B", 4), ("H", 24), ("KV", 8), ("T", 2048),
                 ("DH", 64), ("rows", 8192), ("dim", 1536), ("V", 32000), ("count", 8192 * 4096), ("reps", 20), ("fallback", 0),
                 ("chain", 1)):
        ap.add_argument("--" + a, type=int, default=d)
    ap.add_argument("--no-flush", action="store_true")
    ap.add_argument("--check", action="store_true")
    a = ap.parse_args()
    b = Bench(a.reps, not a.no_flush)
    w = a.what
    if w == "gemm":
        run_gemm(b, a.m, a.n, a.k, a.tb, a.dt, a.fallback)
    elif w in ("attn_fwd", "attn_bwd"):
        run_attn(b, w, a.B, a.H, a.KV, a.T, a.DH, a.dt, a.fallback, a.check)
    elif w in ("rmsnorm", "rmsnorm_bwd"):
        run_rows(b, w, a.rows, a.dim, a.dt, a.chain)
    elif w in ("rope", "silu", "silu_bwd"):
        run_elem(b, w, a.count, a.dt, a.B, a.T, a.H, a.DH, a.chain)
    elif w == "ce":
        run_ce(b, a.rows, a.V, a.dt)
    elif w == "adamw":
        run_adamw(b, a.count)
    elif w == "all":
        N, D, MLP, V = 8192, 1536, 4096, 32000
        for (m, n, k, tb, dt) in [(N, D, D, 0, 1), (N, 512, D, 0, 1), (N, MLP, D, 0, 1), (N, D, MLP, 0, 1), (N, V, D, 1, 1),
                                  (N, D, D, 1, 1), (N, D, MLP, 1, 1), (N, MLP, D, 1, 1), (N, D, V, 0, 1),
                                  (D, D, N, 2, 2), (D, 512, N, 2, 2), (D, MLP, N, 2, 2), (MLP, D, N, 2, 2), (V, D, N, 2, 2)]:
            run_gemm(b, m, n, k, tb, dt)
        run_attn(b, "attn_fwd", 4, 24, 8, 2048, 64)
        run_attn(b, "attn_bwd", 4, 24, 8, 2048, 64, check=a.check)
        run_rows(b, "rmsnorm", N, D, 1); run_rows(b, "rmsnorm_bwd", N, D, 1)
        run_elem(b, "rope", 0, 1); run_elem(b, "silu", N * MLP, 1); run_elem(b, "silu_bwd", N * MLP, 1)
        run_ce(b, N, V, 1)
        run_adamw(b, 256 * 1024 * 1024)
    else:
        sys.exit(f"unknown op {w}")
    b.eng.shutdown()


if __name__ == "__main__":
    main()
