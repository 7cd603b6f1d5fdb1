"""Test helper: a training step written ONLY with the reference's 32 op kinds, one
buffer per tensor and one op per primitive — the kind of plan the reference's
own lowering sends through the C ABI (per-tensor AdamW, separate adds, head
permutes, ROWDOT + FLASH_BWD into pre-zeroed fp32 buffers + CAST, or the tiled
GEMM / SOFTMAX_CAUSAL attention in fp32).  It exists so that the drop-in claim
(an unmodified caller of the reference ABI gets correct results from this
library) is tested end to end on the GPU without the reference tree.
"""
from __future__ import annotations

import numpy as np

from axis_b200 import engine as E
from axis_b200.engine import Engine, op


class LegacyStep:
    def __init__(self, cfg, weights, B, T, dtype="fp32", lr=3e-4, wd=0.1, max_norm=1.0, eps=1e-5, tile=16):
        self.eng = eng = Engine()
        hf = dtype == "bf16"
        dt, dtw, es = (1, 2, 2) if hf else (0, 0, 4)
        V, D, L, H = cfg["vocab_size"], cfg["dim"], cfg["n_layers"], cfg["n_heads"]
        KV = cfg.get("n_kv_heads") or H
        DH, MLP, N, rep = D // H, cfg["mlp_hidden"], B * T, H // (cfg.get("n_kv_heads") or H)
        tied = cfg.get("tie_embeddings", True)
        sc = 1.0 / np.sqrt(DH)
        half = DH // 2
        ang = np.outer(np.arange(T, dtype=np.float32), 1.0 / (10000.0 ** (np.arange(half, dtype=np.float32) / half)))
        cos, sin = eng.new_tensor(np.cos(ang).astype(np.float32)), eng.new_tensor(np.sin(ang).astype(np.float32))
        new = lambda n, size=es: eng.alloc(n, size)
        self.names = list(weights)
        self.shapes = {k: v.shape for k, v in weights.items()}
        self.master = {k: eng.new_tensor(np.ascontiguousarray(v, np.float32)) for k, v in weights.items()}
        self.grad = {k: new(v.size, 4) for k, v in weights.items()}
        self.m = {k: eng.new_tensor(np.zeros(v.size, np.float32)) for k, v in weights.items()}
        self.v = {k: eng.new_tensor(np.zeros(v.size, np.float32)) for k, v in weights.items()}
        W = dict(self.master)
        if hf:
            W = {k: new(v.size) for k, v in weights.items()}
            eng.run([op(E.CAST, a=self.master[k], c=W[k], m=weights[k].size, tb=0) for k in weights])
        self.ids, self.tgt = new(N, 4), new(N, 4)
        self.loss, self.den, self.t = new(1, 4), new(1, 4), eng.new_tensor(np.zeros(1, np.float32))
        self.lr, self.acc, self.gsc = eng.new_tensor(np.array([lr], np.float32)), new(1, 4), new(1, 4)
        G = self.grad
        plan = []
        add = plan.append

        def gemm(a, b, c, m, n, k, tb=0, d=dt, **kw):
            add(op(E.GEMM_SB, a=a, b=b, c=c, m=m, n=n, k=k, batch=1, tb=tb, dt=d, **kw))

        x = [new(N * D) for _ in range(L + 1)]
        add(op(E.EMBED, a=W["embed.weight"], b=self.ids, c=x[0], m=N, n=D, dt=dt))
        saved = []
        for i in range(L):
            p = f"blocks.{i}."
            y, q0, k0, v0 = new(N * D), new(N * D), new(N * KV * DH), new(N * KV * DH)
            q1, k1, v1, q2, k2 = new(N * D), new(N * KV * DH), new(N * KV * DH), new(N * D), new(N * KV * DH)
            at, at2, o_, r1, z = new(N * D), new(N * D), new(N * D), new(N * D), new(N * D)
            g_, u_, h_, mo = new(N * MLP), new(N * MLP), new(N * MLP), new(N * D)
            lse = new(B * H * T, 4)
            add(op(E.RMSNORM, a=x[i], b=W[p + "attn_norm.weight"], c=y, m=N, n=D, dt=dt, alpha=eps))
            gemm(y, W[p + "attn.q_proj.weight"], q0, N, H * DH, D)
            gemm(y, W[p + "attn.k_proj.weight"], k0, N, KV * DH, D)
            gemm(y, W[p + "attn.v_proj.weight"], v0, N, KV * DH, D)
            add(op(E.PERM_0213, a=q0, c=q1, m=B, n=T, k=H, batch=DH, dt=dt))
            add(op(E.PERM_0213, a=k0, c=k1, m=B, n=T, k=KV, batch=DH, dt=dt))
            add(op(E.PERM_0213, a=v0, c=v1, m=B, n=T, k=KV, batch=DH, dt=dt))
            add(op(E.ROPE, a=q1, b=cos, d=sin, c=q2, batch=B * H, m=T, n=DH, dt=dt))
            add(op(E.ROPE, a=k1, b=cos, d=sin, c=k2, batch=B * KV, m=T, n=DH, dt=dt))
            if hf:
                add(op(E.FLASH, a=q2, b=k2, d=v1, c=at, m=T, n=DH, k=KV, batch=B, tb=H, sa=lse, dt=dt, alpha=sc))
            else:
                self._tiled_fwd(plan, q2, k2, v1, at, B, H, KV, T, DH, tile, sc, dt)
            add(op(E.PERM_0213, a=at, c=at2, m=B, n=H, k=T, batch=DH, dt=dt))
            gemm(at2, W[p + "attn.o_proj.weight"], o_, N, D, H * DH)
            add(op(E.ADD, a=x[i], b=o_, c=r1, n=N * D, dt=dt))
            add(op(E.RMSNORM, a=r1, b=W[p + "mlp_norm.weight"], c=z, m=N, n=D, dt=dt, alpha=eps))
            gemm(z, W[p + "mlp.gate_proj.weight"], g_, N, MLP, D)
            gemm(z, W[p + "mlp.up_proj.weight"], u_, N, MLP, D)
            add(op(E.SILU_MUL, a=g_, b=u_, c=h_, n=N * MLP, dt=dt))
            gemm(h_, W[p + "mlp.down_proj.weight"], mo, N, D, MLP)
            add(op(E.ADD, a=r1, b=mo, c=x[i + 1], n=N * D, dt=dt))
            saved.append(dict(y=y, q2=q2, k2=k2, v1=v1, at2=at2, r1=r1, z=z, g=g_, u=u_, h=h_, lse=lse))
        xf, logits, dlog = new(N * D), new(N * V), new(N * V)
        head = W["embed.weight"] if tied else W["lm_head.weight"]
        add(op(E.RMSNORM, a=x[L], b=W["norm.weight"], c=xf, m=N, n=D, dt=dt, alpha=eps))
        gemm(xf, head, logits, N, V, D, tb=1 if tied else 0)
        add(op(E.SCALE, a=self.loss, c=self.loss, n=1, alpha=0.0))
        add(op(E.SCALE, a=self.den, c=self.den, n=1, alpha=0.0))
        add(op(E.COUNTVALID, a=self.tgt, c=self.den, m=N))
        add(op(E.CE, a=logits, b=self.tgt, c=dlog, d=self.loss, sa=self.den, m=N, n=V, dt=dt))
        # backward
        dxf, dcur, tmp = new(N * D), new(N * D), new(N * D)
        if tied:
            gemm(dlog, head, dxf, N, D, V, tb=0)
            gemm(dlog, xf, G["embed.weight"], V, D, N, tb=2, d=dtw)
        else:
            gemm(dlog, head, dxf, N, D, V, tb=1)
            gemm(xf, dlog, G["lm_head.weight"], D, V, N, tb=2, d=dtw)
        add(op(E.RMSNORM_BWD, a=x[L], b=W["norm.weight"], d=dxf, c=dcur, tb=tmp, m=N, n=D, dt=dt, alpha=eps))
        add(op(E.COLSUM, a=tmp, c=G["norm.weight"], m=N, n=D, dt=dtw))
        for i in reversed(range(L)):
            p, s = f"blocks.{i}.", saved[i]
            dh, dg, du, dz1, dz2, dz = new(N * MLP), new(N * MLP), new(N * MLP), new(N * D), new(N * D), new(N * D)
            dr1b, dr1, dat2, dat = new(N * D), new(N * D), new(N * D), new(N * D)
            dq2, dk2, dv1 = new(N * D), new(N * KV * DH), new(N * KV * DH)
            dq1, dk1, dq0, dk0, dv0 = new(N * D), new(N * KV * DH), new(N * D), new(N * KV * DH), new(N * KV * DH)
            dy1, dy2, dy3, dy, dx1, dxin = (new(N * D) for _ in range(6))

            def lin_b(g, xin, wname, dx, fin, fout):
                gemm(g, W[wname], dx, N, fin, fout, tb=1)
                gemm(xin, g, G[wname], fin, fout, N, tb=2, d=dtw)
            lin_b(dcur, s["h"], p + "mlp.down_proj.weight", dh, MLP, D)
            add(op(E.SILU_BWD, a=s["g"], b=s["u"], d=dh, c=dg, tb=du, n=N * MLP, dt=dt))
            lin_b(dg, s["z"], p + "mlp.gate_proj.weight", dz1, D, MLP)
            lin_b(du, s["z"], p + "mlp.up_proj.weight", dz2, D, MLP)
            add(op(E.ADD, a=dz1, b=dz2, c=dz, n=N * D, dt=dt))
            add(op(E.RMSNORM_BWD, a=s["r1"], b=W[p + "mlp_norm.weight"], d=dz, c=dr1b, tb=tmp, m=N, n=D, dt=dt, alpha=eps))
            add(op(E.COLSUM, a=tmp, c=G[p + "mlp_norm.weight"], m=N, n=D, dt=dtw))
            add(op(E.ADD, a=dcur, b=dr1b, c=dr1, n=N * D, dt=dt))
            lin_b(dr1, s["at2"], p + "attn.o_proj.weight", dat2, H * DH, D)
            add(op(E.PERM_0213, a=dat2, c=dat, m=B, n=T, k=H, batch=DH, dt=dt))
            if hf:
                bD, dqf, dkf, dvf = new(N * H, 4), new(N * D, 4), new(N * KV * DH, 4), new(N * KV * DH, 4)
                add(op(E.ROWDOT, a=dat2, b=s["at2"], c=bD, m=N * H, n=DH, dt=dt))
                for buf, cnt in ((dqf, N * D), (dkf, N * KV * DH), (dvf, N * KV * DH)):
                    add(op(E.SCALE, a=buf, c=buf, n=cnt, alpha=0.0))
                add(op(E.FLASH_BWD, a=s["q2"], b=s["k2"], d=s["v1"], c=dat, sa=s["lse"], sb=bD, tb=dqf, sc=dkf, oa=dvf,
                       ob=H, m=T, n=DH, k=KV, batch=B, dt=dt, alpha=sc))
                for src, dst, cnt in ((dqf, dq2, N * D), (dkf, dk2, N * KV * DH), (dvf, dv1, N * KV * DH)):
                    add(op(E.CAST, a=src, c=dst, m=cnt, tb=0))
            else:
                self._tiled_bwd(plan, s["q2"], s["k2"], s["v1"], dat, dq2, dk2, dv1, B, H, KV, T, DH, tile, sc, dt)
            add(op(E.ROPE, a=dq2, b=cos, d=sin, c=dq1, batch=B * H, m=T, n=DH, tb=1, dt=dt))
            add(op(E.ROPE, a=dk2, b=cos, d=sin, c=dk1, batch=B * KV, m=T, n=DH, tb=1, dt=dt))
            add(op(E.PERM_0213, a=dq1, c=dq0, m=B, n=H, k=T, batch=DH, dt=dt))
            add(op(E.PERM_0213, a=dk1, c=dk0, m=B, n=KV, k=T, batch=DH, dt=dt))
            add(op(E.PERM_0213, a=dv1, c=dv0, m=B, n=KV, k=T, batch=DH, dt=dt))
            lin_b(dq0, s["y"], p + "attn.q_proj.weight", dy1, D, H * DH)
            lin_b(dk0, s["y"], p + "attn.k_proj.weight", dy2, D, KV * DH)
            lin_b(dv0, s["y"], p + "attn.v_proj.weight", dy3, D, KV * DH)
            add(op(E.ADD, a=dy1, b=dy2, c=dy, n=N * D, dt=dt))
            add(op(E.ADD, a=dy, b=dy3, c=dy, n=N * D, dt=dt))
            add(op(E.RMSNORM_BWD, a=x[i], b=W[p + "attn_norm.weight"], d=dy, c=dx1, tb=tmp, m=N, n=D, dt=dt, alpha=eps))
            add(op(E.COLSUM, a=tmp, c=G[p + "attn_norm.weight"], m=N, n=D, dt=dtw))
            add(op(E.ADD, a=dr1, b=dx1, c=dxin, n=N * D, dt=dt))
            add(op(E.COPY, a=dxin, c=dcur, n=N * D, dt=dt))
        if not tied:
            add(op(E.SCALE, a=G["embed.weight"], c=G["embed.weight"], n=V * D, alpha=0.0))
        add(op(E.EMBED_BWD, a=dcur, b=self.ids, c=G["embed.weight"], m=N, n=D, dt=dtw))
        self.plan_fb = list(plan)
        add(op(E.SCALE, a=self.acc, c=self.acc, n=1, alpha=0.0))
        for k in self.names:
            add(op(E.L2ACC, a=G[k], c=self.acc, n=weights[k].size))
        add(op(E.CLIPSCALE, a=self.acc, c=self.gsc, alpha=max_norm))
        add(op(E.TICK, a=self.t))
        for k in self.names:
            add(op(E.ADAMW, a=self.master[k], b=G[k], c=self.m[k], d=self.v[k], tb=self.t, sa=(W[k] if hf else 0),
                   sb=self.lr, oa=self.gsc, n=weights[k].size, alpha=lr, beta=(wd if weights[k].ndim >= 2 else 0.0), gamma=1e-8))
        self.plan_step = plan
        self.N = N

    def _tiles(self, T, tile):
        return [(qs, min(tile, T - qs)) for qs in range(0, T, tile)]

    def _scratch(self, B, KV, T, tile, n):
        key = ("attn_scratch", n)
        if not hasattr(self, "_scr"):
            self._scr = {}
        if key not in self._scr:
            self._scr[key] = [self.eng.alloc(B * KV * tile * T, 4) for _ in range(n)]
        return self._scr[key]

    def _tiled_fwd(self, plan, q, k, v, out, B, H, KV, T, DH, tile, sc, dt):
        """Query-tiled causal attention batched over (batch, kv head): for group member j and
        query tile [qs, qs+qt) only the keys [0, qs+qt) are scored; q/out are addressed with
        element offsets inside the [B,H,T,DH] buffers."""
        rep, BKV = H // KV, B * KV
        s_, p_ = self._scratch(B, KV, T, tile, 4)[:2]
        for j in range(rep):
            for qs, qt in self._tiles(T, tile):
                kl, off = qs + qt, (j * T + qs) * DH
                plan.append(op(E.GEMM_SB, a=q, b=k, c=s_, m=qt, k=DH, n=kl, batch=BKV, tb=1, sa=rep * T * DH,
                               sb=T * DH, sc=qt * kl, oa=off, dt=dt, alpha=sc))
                plan.append(op(E.SOFTMAX_CAUSAL, a=s_, c=p_, batch=BKV, m=qt, n=kl, k=qs, dt=dt))
                plan.append(op(E.GEMM_SB, a=p_, b=v, c=out, m=qt, k=kl, n=DH, batch=BKV, sa=qt * kl, sb=T * DH,
                               sc=rep * T * DH, oc=off, dt=dt))

    def _tiled_bwd(self, plan, q, k, v, dat, dq, dk, dv, B, H, KV, T, DH, tile, sc, dt):
        rep, BKV = H // KV, B * KV
        s_, p_, dp_, ds_ = self._scratch(B, KV, T, tile, 4)
        plan.append(op(E.SCALE, a=dk, c=dk, n=B * KV * T * DH, dt=dt, alpha=0.0))
        plan.append(op(E.SCALE, a=dv, c=dv, n=B * KV * T * DH, dt=dt, alpha=0.0))
        for j in range(rep):
            for qs, qt in self._tiles(T, tile):
                kl, off = qs + qt, (j * T + qs) * DH
                g = dict(batch=BKV, dt=dt)
                plan.append(op(E.GEMM_SB, a=q, b=k, c=s_, m=qt, k=DH, n=kl, tb=1, sa=rep * T * DH, sb=T * DH,
                               sc=qt * kl, oa=off, alpha=sc, **g))
                plan.append(op(E.SOFTMAX_CAUSAL, a=s_, c=p_, batch=BKV, m=qt, n=kl, k=qs, dt=dt))
                plan.append(op(E.GEMM_SB, a=dat, b=v, c=dp_, m=qt, k=DH, n=kl, tb=1, sa=rep * T * DH, sb=T * DH,
                               sc=qt * kl, oa=off, **g))
                plan.append(op(E.GEMM_SB, a=p_, b=dat, c=dv, m=kl, n=DH, k=qt, tb=2, sa=qt * kl, sb=rep * T * DH,
                               sc=T * DH, ob=off, beta=1.0, **g))
                plan.append(op(E.SOFTMAX_BWD, a=p_, b=dp_, c=ds_, batch=BKV, m=qt, n=kl, dt=dt))
                plan.append(op(E.GEMM_SB, a=ds_, b=k, c=dq, m=qt, k=kl, n=DH, sa=qt * kl, sb=T * DH,
                               sc=rep * T * DH, oc=off, alpha=sc, **g))
                plan.append(op(E.GEMM_SB, a=ds_, b=q, c=dk, m=kl, n=DH, k=qt, tb=2, sa=qt * kl, sb=rep * T * DH,
                               sc=T * DH, ob=off, alpha=sc, beta=1.0, **g))

    def upload(self, x, y):
        self.eng.upload(self.ids, x.reshape(-1).astype(np.float32))
        self.eng.upload(self.tgt, y.reshape(-1).astype(np.float32))

    def grads(self):
        return {k: self.eng.download(self.grad[k], self.shapes[k]) for k in self.names}

    def weights(self):
        return {k: self.eng.download(self.master[k], self.shapes[k]) for k in self.names}
