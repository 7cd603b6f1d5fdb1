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

    python opbench.py refcmp [--lib oracle/_ref/libaxeng_ref.so]

times, at the 1B-class shapes, the plan fragments that the reference's own lowering emits for the hot ops
(reference op kinds only: its flash backward with row dots, zero fills and casts; RMSNorm backward + column sum;
count + cross-entropy; per-tensor L2 / clip / AdamW; rotary + permutes; SwiGLU; cuBLAS GEMMs) on the library
given by --lib (the reference's engine, built by oracle/build_ref.py: the kernels to beat), and beside each the
fused op of this library that replaces the fragment.  Both run as captured graphs replayed back to back on
buffer sets larger than L2; one JSON line per case.
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


def run_embed_bwd(b, N, D, V, dt):
    """Deterministic embedding gradient: N token rows of width D summed into the fp32 table rows of their ids."""
    es = 2 if dt else 4
    g = b.buf(N * D, dt)
    ids = b.eng.alloc(N)
    b.eng.upload_tokens(ids, b.rng.integers(0, V, N), V)
    table = b.eng.alloc(V * D)
    ms = b.time([op(E.EMBED_BWD_DET, a=g, b=ids, c=table, m=N, n=D, dt=dt)])
    # read the gradient rows once, read-modify-write one table row per token at most
    return b.report(f"embed_bwd_det {N} tokens x {D} into {V} rows dt={dt}", ms, bytes_=N * D * es + 2 * min(N, V) * D * 4)


def run_lora(b, which, N, Fs, R, chain=1):
    """LORA_PROJ (skinny products x A / g B^T) or LORA_GRAD (adapter weight gradients) on 1-3 widths; chain > 1: that many
    instances back to back on separate buffers, figure per instance."""
    plan, nbytes = [], 0
    pad = lambda v: list(v) + [0] * (3 - len(v))
    for _ in range(chain):
        xs = pad([b.buf(N * F, 1) for F in Fs])
        f_ = pad(Fs)
        if which == "lora_proj":
            ws = pad([b.buf(F * R, 1, scale=0.05) for F in Fs])
            outs = pad([b.eng.alloc(N * R, 2) for _ in Fs])
            plan.append(op(E.LORA_PROJ, a=xs[0], sa=xs[1], sb=xs[2], b=ws[0], d=ws[1], sc=ws[2], c=outs[0], oa=outs[1], ob=outs[2],
                           n=f_[0], k=f_[1], oc=f_[2], m=N, batch=len(Fs), tb=1, gamma=float(R), dt=1))
        else:
            ss = pad([b.buf(N * R, 1) for _ in Fs])
            out = b.eng.alloc(sum(Fs) * R)
            offs = pad(list(np.cumsum([0] + [F * R for F in Fs[:-1]])))
            plan.append(op(E.LORA_GRAD, a=xs[0], sa=xs[1], sb=xs[2], b=ss[0], d=ss[1], sc=ss[2], c=out, oa=int(offs[0]),
                           ob=int(offs[1]), oc=int(offs[2]), n=f_[0], k=f_[1], tb=f_[2], m=N, batch=len(Fs), gamma=float(R), dt=1))
        nbytes = sum(N * F * 2 for F in Fs)
    ms = b.time(plan) / chain
    tag = f" (chain of {chain})" if chain > 1 else ""
    return b.report(f"{which} N={N} F={list(Fs)} R={R}{tag}", ms, bytes_=nbytes)


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


class RawEngine:
    """The reference's twelve exports only (axis/engine.py:78-174): what any libaxeng-compatible library offers."""

    def __init__(self, lib_path):
        import ctypes
        self.ct = ctypes
        self.lib = L = ctypes.CDLL(lib_path)
        L.eng_init.restype = ctypes.c_int
        L.eng_alloc.argtypes = [ctypes.c_int, ctypes.c_longlong, ctypes.c_int]
        L.eng_upload.argtypes = [ctypes.c_int, ctypes.POINTER(ctypes.c_float), ctypes.c_longlong]
        L.eng_run_plan.argtypes = [ctypes.POINTER(E._EngOp), ctypes.c_int, ctypes.c_int]
        L.eng_capture_plan.argtypes = [ctypes.POINTER(E._EngOp), ctypes.c_int]
        L.eng_replay.argtypes = [ctypes.c_int, ctypes.c_int]
        rc = L.eng_init()
        if rc:
            raise RuntimeError(f"eng_init rc={rc}")
        self.next = 0

    def alloc(self, n, itemsize=4):
        i = self.next
        self.next += 1
        rc = self.lib.eng_alloc(i, int(n), int(itemsize))
        if rc:
            raise RuntimeError(f"eng_alloc rc={rc}")
        return i

    def fill(self, i, nbytes, rng, scale=1.0):
        """Random fp32 words (a bf16 buffer gets random bf16 pairs of modest size: zero the low mantissa noise)"""
        n = nbytes // 4
        step = 1 << 24
        for o in range(0, n, step):
            m = min(step, n - o)
            a = (rng.standard_normal(m, dtype=np.float32) * scale)
            # upload goes to the start of the buffer only; larger buffers are filled in one call
            if o == 0 and m == n:
                self.lib.eng_upload(i, a.ctypes.data_as(self.ct.POINTER(self.ct.c_float)), m)
                return
        a = rng.standard_normal(n, dtype=np.float32) * scale
        self.lib.eng_upload(i, a.ctypes.data_as(self.ct.POINTER(self.ct.c_float)), n)

    def time_graph(self, plan, reps):
        pp = E.PackedPlan(plan)
        rc = self.lib.eng_run_plan(pp.ptr, pp.n, 1)
        if rc:
            raise RuntimeError(f"run_plan rc={rc}")
        rc = self.lib.eng_capture_plan(pp.ptr, pp.n)
        if rc:
            raise RuntimeError(f"capture rc={rc}")
        self.lib.eng_replay(2, 1)
        import time
        t0 = time.perf_counter()
        rc = self.lib.eng_replay(reps, 1)
        dt = time.perf_counter() - t0
        if rc:
            raise RuntimeError(f"replay rc={rc}")
        return dt / reps * 1e3


def bf16_buf(e, rng, n, scale=1.0):
    """n bf16 elements holding N(0, scale) values (uploaded as fp32 words whose halves are valid bf16 numbers)"""
    i = e.alloc(n, 2)
    a = rng.standard_normal(n, dtype=np.float32) * scale
    bits = E.f32_to_bf16_bits(a)
    words = bits.view(np.uint32) if n % 2 == 0 else np.concatenate([bits, np.zeros(1, np.uint16)]).view(np.uint32)
    f = words.view(np.float32)
    e.lib.eng_upload(i, f.ctypes.data_as(e.ct.POINTER(e.ct.c_float)), f.size)
    return i


def refcmp(lib_path, reps):
    """Reference fragments on `lib_path` vs this library's fused ops; shapes of the 1B-class step."""
    from axis_b200._build import engine_lib
    N, D, MLP, V = 8192, 1536, 4096, 32000
    B, H, KV, T, DH = 4, 24, 8, 2048, 64
    rng = np.random.default_rng(0)
    out = []

    def run(which, name, build, chain, algo_bytes=None, flops=None):
        e = RawEngine(lib_path if which == "reference" else engine_lib())
        e.alloc(4)
        plan = []
        for _ in range(chain):
            plan += build(e)
        ms = e.time_graph(plan, reps) / chain
        rec = {"case": name, "library": which, "ms": round(ms, 5), "instances_per_replay": chain, "reps": reps}
        if algo_bytes:
            rec["gbs_algorithmic"] = round(algo_bytes / (ms * 1e-3) / 1e9, 1)
        if flops:
            rec["tflops"] = round(flops / (ms * 1e-3) / 1e12, 1)
        print(json.dumps(rec), flush=True)
        out.append(rec)
        e.lib.eng_shutdown() if hasattr(e.lib, "eng_shutdown") else None
        return ms

    nq, nk = B * T * H * DH, B * T * KV * DH

    # flash-attention backward: reference fragment (axis/compile.py:406-421) on [B,H,T,DH] vs ATTN_BWD on [B,T,H,DH]
    def ref_flash_bwd(e):
        q, k, v, do, o = (bf16_buf(e, rng, nq), bf16_buf(e, rng, nk), bf16_buf(e, rng, nk), bf16_buf(e, rng, nq), e.alloc(nq, 2))
        lse, bD = e.alloc(B * H * T), e.alloc(B * H * T)
        dqf, dkf, dvf = e.alloc(nq), e.alloc(nk), e.alloc(nk)
        dq, dk, dv = e.alloc(nq, 2), e.alloc(nk, 2), e.alloc(nk, 2)
        pre = [op(E.FLASH, a=q, b=k, d=v, c=o, m=T, n=DH, k=KV, batch=B, tb=H, sa=lse, dt=1, alpha=0.125)]
        pp = E.PackedPlan(pre)
        e.lib.eng_run_plan(pp.ptr, pp.n, 1)
        return [op(E.ROWDOT, a=do, b=o, c=bD, m=B * T * H, n=DH, dt=1),
                op(E.SCALE, a=dqf, c=dqf, n=nq, alpha=0.0), op(E.SCALE, a=dkf, c=dkf, n=nk, alpha=0.0),
                op(E.SCALE, a=dvf, c=dvf, n=nk, alpha=0.0),
                op(E.FLASH_BWD, a=q, b=k, d=v, c=do, sa=lse, sb=bD, tb=dqf, sc=dkf, oa=dvf, ob=H, m=T, n=DH, k=KV, batch=B,
                   dt=1, alpha=0.125),
                op(E.CAST, a=dqf, c=dq, m=nq, tb=0), op(E.CAST, a=dkf, c=dk, m=nk, tb=0), op(E.CAST, a=dvf, c=dv, m=nk, tb=0)]

    def our_attn_bwd(e):
        q, k, v, do, o = (bf16_buf(e, rng, nq), bf16_buf(e, rng, nk), bf16_buf(e, rng, nk), bf16_buf(e, rng, nq), e.alloc(nq, 2))
        lse, scr = e.alloc(B * H * T), e.alloc(B * H * T + nq)
        dq, dk, dv = e.alloc(nq, 2), e.alloc(nk, 2), e.alloc(nk, 2)
        pre = [op(E.ATTN_FWD, a=q, b=k, d=v, c=o, sa=lse, m=T, n=DH, k=KV, batch=B, tb=H, dt=1, alpha=0.125)]
        pp = E.PackedPlan(pre)
        e.lib.eng_run_plan(pp.ptr, pp.n, 1)
        return [op(E.ATTN_BWD, a=q, b=k, d=v, c=do, sa=lse, sb=o, tb=dq, sc=dk, oa=dv, ob=H, oc=scr, m=T, n=DH, k=KV,
                   batch=B, dt=1, alpha=0.125)]
    fl = 5.0 * B * H * T * T * DH
    run("reference", "flash-attention backward (row dots, zero fills, kernel, casts)", ref_flash_bwd, 3, flops=fl)
    run("this", "flash-attention backward (ATTN_BWD)", our_attn_bwd, 3, flops=fl)

    def ref_flash_fwd(e):
        q, k, v, o = bf16_buf(e, rng, nq), bf16_buf(e, rng, nk), bf16_buf(e, rng, nk), e.alloc(nq, 2)
        return [op(E.FLASH, a=q, b=k, d=v, c=o, m=T, n=DH, k=KV, batch=B, tb=H, sa=e.alloc(B * H * T), dt=1, alpha=0.125)]

    def our_attn_fwd(e):
        q, k, v, o = bf16_buf(e, rng, nq), bf16_buf(e, rng, nk), bf16_buf(e, rng, nk), e.alloc(nq, 2)
        return [op(E.ATTN_FWD, a=q, b=k, d=v, c=o, sa=e.alloc(B * H * T), m=T, n=DH, k=KV, batch=B, tb=H, dt=1, alpha=0.125)]
    run("reference", "flash-attention forward (FLASH)", ref_flash_fwd, 3, flops=2.0 * B * H * T * T * DH)
    run("this", "flash-attention forward (ATTN_FWD)", our_attn_fwd, 3, flops=2.0 * B * H * T * T * DH)

    # RMSNorm backward + weight gradient (axis/compile.py:397-400) vs the fused pass with residual
    def ref_norm_bwd(e):
        x, w, g = bf16_buf(e, rng, N * D), bf16_buf(e, rng, D), bf16_buf(e, rng, N * D)
        dx, tmp, dw = e.alloc(N * D, 2), e.alloc(N * D, 2), e.alloc(D)
        res, out_ = bf16_buf(e, rng, N * D), e.alloc(N * D, 2)
        return [op(E.RMSNORM_BWD, a=x, b=w, d=g, c=dx, tb=tmp, m=N, n=D, dt=1, alpha=1e-5),
                op(E.COLSUM, a=tmp, c=dw, m=N, n=D, dt=2),
                op(E.ADD, a=res, b=dx, c=out_, n=N * D, dt=1)]

    def our_norm_bwd(e):
        x, w, g, res = bf16_buf(e, rng, N * D), bf16_buf(e, rng, D), bf16_buf(e, rng, N * D), bf16_buf(e, rng, N * D)
        dx, dw, scr = e.alloc(N * D, 2), e.alloc(D), e.alloc(296 * D)
        return [op(E.RMSNORM_BWD_ACC, a=x, b=w, d=g, c=dx, tb=res, sa=dw, sb=scr, m=N, n=D, dt=1, alpha=1e-5)]
    nb = 4 * N * D * 2
    run("reference", "RMSNorm backward + column sum + residual add", ref_norm_bwd, 8, algo_bytes=nb)
    run("this", "RMSNorm backward (RMSNORM_BWD_ACC: dx + residual + dw)", our_norm_bwd, 8, algo_bytes=nb)

    def ref_norm(e):
        x, w, y = bf16_buf(e, rng, N * D), bf16_buf(e, rng, D), e.alloc(N * D, 2)
        return [op(E.RMSNORM, a=x, b=w, c=y, m=N, n=D, dt=1, alpha=1e-5)]
    run("reference", "RMSNorm forward", ref_norm, 8, algo_bytes=2 * N * D * 2)
    run("this", "RMSNorm forward", ref_norm, 8, algo_bytes=2 * N * D * 2)

    # count + cross-entropy (axis/compile.py:369-372) vs CE_FUSED
    tg_f = rng.integers(0, V, N).astype(np.float32)

    def ref_ce(e):
        lg, dl = bf16_buf(e, rng, N * V), e.alloc(N * V, 2)
        tg = e.alloc(N)
        e.lib.eng_upload(tg, tg_f.ctypes.data_as(e.ct.POINTER(e.ct.c_float)), N)
        loss, den = e.alloc(1), e.alloc(1)
        return [op(E.SCALE, a=loss, c=loss, n=1, alpha=0.0), op(E.SCALE, a=den, c=den, n=1, alpha=0.0),
                op(E.COUNTVALID, a=tg, c=den, m=N), op(E.CE, a=lg, b=tg, c=dl, d=loss, sa=den, m=N, n=V, dt=1)]

    def our_ce(e):
        lg = bf16_buf(e, rng, N * V)
        tg = e.alloc(N)
        ti = rng.integers(0, V, N).astype(np.int32).view(np.float32)
        e.lib.eng_upload(tg, ti.ctypes.data_as(e.ct.POINTER(e.ct.c_float)), N)
        loss, den, scr = e.alloc(1), e.alloc(1), e.alloc(N + 8)
        return [op(E.CE_FUSED, a=lg, b=tg, c=lg, d=loss, sa=den, sb=scr, m=N, n=V, dt=1)]
    run("reference", "count + cross-entropy forward/backward", ref_ce, 1, algo_bytes=2 * N * V * 2)
    run("this", "cross-entropy (CE_FUSED, in place)", our_ce, 1, algo_bytes=2 * N * V * 2)

    # clip + AdamW over 16 tensors of 1536 x 4096 (axis/compile.py:497-532) vs the flat pass
    nt, el = 16, D * MLP

    def ref_adamw(e):
        ps = [(e.alloc(el), e.alloc(el), e.alloc(el), e.alloc(el), e.alloc(el, 2)) for _ in range(nt)]
        for (p_, g_, m_, v_, _) in ps:
            e.fill(p_, el * 4, rng, 0.02); e.fill(g_, el * 4, rng, 1e-3); e.fill(m_, el * 4, rng, 0.0); e.fill(v_, el * 4, rng, 0.0)
        gn, gs, t_, lr = e.alloc(1), e.alloc(1), e.alloc(1), e.alloc(1)
        one = np.array([3e-4], np.float32)
        e.lib.eng_upload(lr, one.ctypes.data_as(e.ct.POINTER(e.ct.c_float)), 1)
        z = np.zeros(1, np.float32)
        e.lib.eng_upload(t_, z.ctypes.data_as(e.ct.POINTER(e.ct.c_float)), 1)
        return ([op(E.SCALE, a=gn, c=gn, n=1, alpha=0.0)] + [op(E.L2ACC, a=g_, c=gn, n=el) for (_, g_, _, _, _) in ps] +
                [op(E.CLIPSCALE, a=gn, c=gs, alpha=1.0), op(E.TICK, a=t_)] +
                [op(E.ADAMW, a=p_, b=g_, c=m_, d=v_, tb=t_, sa=mir, sb=lr, oa=gs, n=el, alpha=3e-4, beta=0.1, gamma=1e-8)
                 for (p_, g_, m_, v_, mir) in ps])

    def our_adamw(e):
        n = nt * el
        p_, g_, m_, v_, mir = e.alloc(n), e.alloc(n), e.alloc(n), e.alloc(n), e.alloc(n, 2)
        e.fill(p_, n * 4, rng, 0.02); e.fill(g_, n * 4, rng, 1e-3); e.fill(m_, n * 4, rng, 0.0); e.fill(v_, n * 4, rng, 0.0)
        fl_ = e.alloc(n // 1024, 1)
        ones = np.ones(n // 1024, np.uint8).view(np.float32)
        e.lib.eng_upload(fl_, ones.ctypes.data_as(e.ct.POINTER(e.ct.c_float)), ones.size)
        t_, lr, part, ss, gn = e.alloc(1), e.alloc(1), e.alloc(n // 8192 + 1), e.alloc(1), e.alloc(1)
        one = np.array([3e-4], np.float32)
        e.lib.eng_upload(lr, one.ctypes.data_as(e.ct.POINTER(e.ct.c_float)), 1)
        z = np.zeros(1, np.float32)
        e.lib.eng_upload(t_, z.ctypes.data_as(e.ct.POINTER(e.ct.c_float)), 1)
        return [op(E.GNORM_FLAT, a=g_, c=part, d=ss, ob=0, m=n // 1024, oa=0, tb=t_),
                op(E.ADAMW_FLAT, a=p_, b=g_, c=m_, d=v_, m=n // 1024, k=0, sa=mir, sb=lr, tb=t_, sc=fl_, oa=ss, ob=1, oc=gn,
                   alpha=1.0, beta=0.1, gamma=1e-8)]
    run("reference", "L2 norm + clip + per-tensor AdamW (16 tensors, 100.7 M params)", ref_adamw, 1, algo_bytes=34 * nt * el)
    run("this", "clip + AdamW over the flat arena (100.7 M params)", our_adamw, 1, algo_bytes=34 * nt * el)

    # rotary on q: reference permutes to [B,H,T,DH] and rotates there (axis/compile.py:319-323); here in place on [B,T,H,DH]
    half = DH // 2
    ang = np.outer(np.arange(T, dtype=np.float32), 1.0 / (10000.0 ** (np.arange(half, dtype=np.float32) / half)))
    cosv, sinv = np.cos(ang).astype(np.float32).reshape(-1), np.sin(ang).astype(np.float32).reshape(-1)

    def tables(e):
        cs, sn = e.alloc(T * half), e.alloc(T * half)
        e.lib.eng_upload(cs, cosv.ctypes.data_as(e.ct.POINTER(e.ct.c_float)), cosv.size)
        e.lib.eng_upload(sn, sinv.ctypes.data_as(e.ct.POINTER(e.ct.c_float)), sinv.size)
        return cs, sn

    def ref_rope(e):
        cs, sn = tables(e)
        x, xp, xr = bf16_buf(e, rng, nq), e.alloc(nq, 2), e.alloc(nq, 2)
        return [op(E.PERM_0213, a=x, c=xp, m=B, n=T, k=H, batch=DH, dt=1),
                op(E.ROPE, a=xp, b=cs, d=sn, c=xr, batch=B * H, m=T, n=DH, dt=1)]

    def our_rope(e):
        cs, sn = tables(e)
        x = bf16_buf(e, rng, nq)
        return [op(E.ROPE_BTHD, a=x, b=cs, d=sn, c=x, batch=B, m=T, k=H, n=DH, dt=1)]
    run("reference", "head permute + rotary on q", ref_rope, 6, algo_bytes=2 * nq * 2)
    run("this", "rotary in place on [B,T,H,DH] (ROPE_BTHD)", our_rope, 6, algo_bytes=2 * nq * 2)

    def silu_bwd(e):
        g, u, gr = bf16_buf(e, rng, N * MLP), bf16_buf(e, rng, N * MLP), bf16_buf(e, rng, N * MLP)
        return [op(E.SILU_BWD, a=g, b=u, d=gr, c=e.alloc(N * MLP, 2), tb=e.alloc(N * MLP, 2), n=N * MLP, dt=1)]
    run("reference", "SwiGLU backward (SILU_BWD)", silu_bwd, 2, algo_bytes=5 * N * MLP * 2)
    run("this", "SwiGLU backward (SILU_BWD)", silu_bwd, 2, algo_bytes=5 * N * MLP * 2)

    # GEMMs: the reference calls cuBLAS (runtime.cu:878-917)
    for (m, n, k, tb, dt) in [(N, MLP, D, 0, 1), (N, D, MLP, 0, 1), (N, D, D, 1, 1), (D, MLP, N, 2, 2), (N, V, D, 1, 1)]:
        def gemm(e, m=m, n=n, k=k, tb=tb, dt=dt):
            a, b_ = bf16_buf(e, rng, m * k), bf16_buf(e, rng, k * n)
            return [op(E.GEMM_SB, a=a, b=b_, c=e.alloc(m * n, 2 if dt == 1 else 4), m=m, n=n, k=k, batch=1, tb=tb, dt=dt)]
        nm = f"GEMM tb={tb} dt={dt} {m}x{n}x{k}"
        ch = 1 if m * n > (1 << 27) else 4
        run("reference", nm + " (cuBLAS)", gemm, ch, flops=2.0 * m * n * k)
        run("this", nm, gemm, ch, flops=2.0 * m * n * k)
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("what")
    for a, d in (("m", 8192), ("n", 1536), ("k", 1536), ("tb", 0), ("dt", 1), ("B", 4), ("H", 24), ("KV", 8), ("T", 2048),
                 ("DH", 64), ("rows", 8192), ("dim", 1536), ("V", 32000), ("count", 8192 * 4096), ("reps", 20), ("fallback", 0),
                 ("chain", 1)):
        ap.add_argument("--" + a, type=int, default=d)
    ap.add_argument("--lib", default=os.path.join(ROOT, "oracle", "_ref", "libaxeng_ref.so"))
    ap.add_argument("--no-flush", action="store_true")
    ap.add_argument("--check", action="store_true")
    a = ap.parse_args()
    if a.what == "refcmp":
        refcmp(a.lib, a.reps)
        return
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
    elif w in ("lora_proj", "lora_grad"):
        for Fs in ((a.dim,), (4096,), (a.dim, 512, 512), (4096, 4096)):
            run_lora(b, w, a.rows, Fs, 16, a.chain)
    elif w == "embed_bwd":
        run_embed_bwd(b, a.rows, a.dim, a.V, a.dt)
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
        run_embed_bwd(b, N, D, V, 1)
        run_adamw(b, 256 * 1024 * 1024)
    else:
        sys.exit(f"unknown op {w}")
    b.eng.shutdown()


if __name__ == "__main__":
    main()
