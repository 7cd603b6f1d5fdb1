"""Test-only plan interpreter: executes the engine's op tuples with numpy.

It stands in for `axis_b200.engine.Engine` in the CPU tests so that the host
lowering (buffer plan, op plan, arena layout, bucketed reduction schedule,
ownership) can be checked against the oracle without a GPU.  It is test
infrastructure: nothing in the package imports it, and the GPU tests never use
it.  bf16 storage is emulated with round-to-nearest-even on uint16 bit
patterns; collectives run over a `torch.distributed` gloo group when given.
"""
from __future__ import annotations

import numpy as np

from axis_b200 import engine as E
from oracle import step_numpy as O


class InterpEngine:
    has_flash = True

    def __init__(self, dist=None):
        self.bufs = []          # numpy uint8 arrays (views share memory)
        self.dist = dist        # torch.distributed module with an initialised gloo group, or None
        self.rank = dist.get_rank() if dist else 0
        self.world = dist.get_world_size() if dist else 1
        self.launches = 0
        self.captured = None
        self.trace = []

    # ── buffers ──
    def alloc(self, nelems, itemsize=4):
        self.bufs.append(np.full(int(nelems) * itemsize, 0xFF, dtype=np.uint8))   # garbage, not zeros
        return len(self.bufs) - 1

    def alloc_zero(self, nbytes):
        self.bufs.append(np.zeros(int(nbytes), dtype=np.uint8))
        return len(self.bufs) - 1

    def view(self, parent, byte_offset, nbytes):
        assert byte_offset + nbytes <= self.bufs[parent].size
        self.bufs.append(self.bufs[parent][byte_offset:byte_offset + nbytes])
        return len(self.bufs) - 1

    def bytes_allocated(self):
        """bytes of the allocations (views of an allocation are not counted)"""
        return sum(b.size for b in self.bufs if b.base is None)

    def new_tensor(self, arr):
        i = self.alloc(arr.size)
        self.upload(i, arr)
        return i

    def _f32(self, i, n=None, off=0):
        v = self.bufs[i].view(np.float32)
        return v[off:] if n is None else v[off:off + n]

    def _get(self, i, n, dt, off=0):
        """Read n elements as float32 from storage type dt (0 fp32, 1 bf16)."""
        if dt == 1:
            return E.bf16_bits_to_f32(self.bufs[i].view(np.uint16)[off:off + n])
        return self.bufs[i].view(np.float32)[off:off + n].copy()

    def _put(self, i, arr, dt, off=0):
        a = np.asarray(arr, dtype=np.float32).reshape(-1)
        if dt == 1:
            self.bufs[i].view(np.uint16)[off:off + a.size] = E.f32_to_bf16_bits(a)
        else:
            self.bufs[i].view(np.float32)[off:off + a.size] = a

    def upload(self, i, arr):
        a = np.ascontiguousarray(arr, dtype=np.float32).reshape(-1)
        self.bufs[i].view(np.float32)[:a.size] = a

    def download(self, i, shape):
        n = int(np.prod(shape))
        return self.bufs[i].view(np.float32)[:n].reshape(shape).copy()

    def upload_raw(self, i, arr, byte_offset=0):
        b = np.ascontiguousarray(arr).view(np.uint8).reshape(-1)
        self.bufs[i][byte_offset:byte_offset + b.size] = b

    def download_raw(self, i, shape, dtype, byte_offset=0):
        n = int(np.prod(shape)) * np.dtype(dtype).itemsize
        return self.bufs[i][byte_offset:byte_offset + n].view(dtype).reshape(shape).copy()

    def download_async(self, i, nfloats=1):
        if not hasattr(self, "_tickets"):
            self._tickets, self._tk = {}, 0
        self._tk += 1
        self._tickets[self._tk] = self.bufs[i].view(np.float32)[:nfloats].copy()
        for old in [t for t in self._tickets if t <= self._tk - 8]:
            del self._tickets[old]
        return self._tk

    def download_wait(self, ticket, nfloats=1):
        if ticket not in getattr(self, "_tickets", {}):
            raise RuntimeError("download_wait failed rc=4")
        return self._tickets.pop(ticket)[:nfloats]

    def upload_tokens(self, i, tokens, limit):
        t = np.asarray(tokens, dtype=np.int64).reshape(-1)
        if (t >= limit).any() or (t < -1).any():
            raise RuntimeError("upload_tokens failed rc=3")
        self.bufs[i].view(np.int32)[:t.size] = t.astype(np.int32)

    def set_tf32(self, on): pass
    def sync(self): pass
    def nccl_id(self): return bytes(128)
    def nccl_init(self, *a, **k): pass
    def launch_count(self, reset=False): return self.launches

    # ── plans ──
    def run(self, plan, sync=True):
        for i, o in enumerate(plan):
            try:
                self._exec(o)
            except Exception as e:      # pragma: no cover - debugging aid
                raise RuntimeError(f"op {i} kind {E.KIND_NAMES[o[0]]} failed: {e}") from e

    def capture(self, plan):
        self.captured = list(plan)

    def replay(self, times=1, sync=True):
        if self.captured is None:
            raise RuntimeError("replay failed rc=1")
        for _ in range(times):
            self.run(self.captured)

    # ── ops ──
    def _gemm(self, o, ex):
        (kind, a, b, c, d, m, n, k, batch, tb, sa, sb, sc, dt, oa, ob, oc, alpha, beta, _) = o
        in_dt = 1 if dt >= 1 else 0
        out_dt = 1 if dt == 1 else 0
        alpha = 1.0 if alpha == 0.0 else alpha
        batch = max(batch, 1)
        for z in range(batch):
            A = self._get(a, m * k, in_dt, oa + z * sa)
            B = self._get(b, k * n, in_dt, ob + z * sb)
            if tb == 0:
                r = A.reshape(m, k) @ B.reshape(k, n)
            elif tb == 1:
                r = A.reshape(m, k) @ B.reshape(n, k).T
            else:
                r = A.reshape(k, m).T @ B.reshape(k, n)
            r = np.float32(alpha) * r
            if beta != 0.0:
                src = d if (ex and d >= 0) else c
                r = r + np.float32(beta) * self._get(src, m * n, out_dt, oc + z * sc).reshape(m, n)
            self._put(c, r, out_dt, oc + z * sc)

    def _lora_grad(self, o):
        (kind, a, b, c, d, m, n, k, batch, tb, sa, sb, sc, dt, oa, ob, oc, alpha, beta, gamma) = o
        R, lay = int(gamma), beta != 0.0
        xs_, ss_, fs_, offs_ = (a, sa if sa > 0 else a, sb if sb > 0 else a), (b, d, sc), (n, k, tb), (oa, ob, oc)
        in_dt = 1 if dt >= 1 else 0
        for g_ in range(abs(batch)):
            X = self._get(xs_[g_], m * fs_[g_], in_dt).reshape(m, fs_[g_])
            S = self._get(ss_[g_], m * R, in_dt).reshape(m, R)
            r = np.float32(1.0 if alpha == 0.0 else alpha) * (X.T @ S)
            self._put(c, r.T if lay else r, 0, offs_[g_])

    def _exec(self, o):
        (kind, a, b, c, d, m, n, k, batch, tb, sa, sb, sc, dt, oa, ob, oc, alpha, beta, gamma) = o
        self.trace.append(kind)
        if kind not in (E.GROUP, E.FORK, E.JOIN, E.STREAM, E.EVENT):
            self.launches += 1
        if kind in (E.GEMM, E.GEMM_SB):
            return self._gemm(o, False)
        if kind == E.GEMM_EX:
            return self._gemm(o, True)
        if kind == E.GEMM_XSEG:
            # no launch: extra operands of the next GEMM_GROUP
            self.launches -= 1
            self._xseg = dict(n=batch, a=(a, b, d), b=(sa, sb, sc), k=k, addend=c if c > 0 else 0, beta=beta)
            return None
        if kind == E.LORA_PROJ:
            R = int(gamma)
            xs_, ws_, os_, fs_ = (a, sa if sa > 0 else a, sb if sb > 0 else a), (b, d, sc), (c, oa, ob), (n, k, oc)
            sdt = 1 if dt >= 1 else 0
            for g_ in range(batch):
                X = self._get(xs_[g_], m * fs_[g_], sdt).reshape(m, fs_[g_])
                W = self._get(ws_[g_], fs_[g_] * R, sdt)
                W = W.reshape(R, fs_[g_]).T if tb else W.reshape(fs_[g_], R)
                self._put(os_[g_], np.float32(1.0 if alpha == 0.0 else alpha) * (X @ W), sdt)
            return None
        if kind == E.LORA_GRAD:
            # batch < 0: noted only; batch == 0: everything noted runs now (as one launch pair in the library)
            pend = getattr(self, "_lgrad", [])
            if batch == 0:
                self._lgrad = []
                self.launches += 1 if pend else -1
                for o2 in pend:
                    self._lora_grad(o2)
                return None
            if batch < 0:
                self.launches -= 1
                self._lgrad = pend + [o]
                return None
            self.launches += 1
            return self._lora_grad(o)
        if kind == E.GEMM_GROUP:
            # expanded into the plain GEMMs it stands for (same semantics as the library's fallback)
            self.launches -= 1
            xs = getattr(self, "_xseg", None)
            self._xseg = None
            if xs is not None:
                assert oc in (1, 2) and (oc == 2 or (xs["n"] == batch and not xs["addend"]))
            ia, ic, dims = (a, sa, sb), (c, d, sc), (n if oc == 1 else k, oa, ob)
            ib = (b, sa, sb) if oc == 1 else (b, d, sc)
            if oc == 4:
                for (w_, out_) in ((b, c), (sa, d)):
                    self.launches += 1
                    self._gemm(E.op(E.GEMM_SB, a=a, b=w_, c=out_, m=m, n=n, k=k, batch=1, tb=tb, dt=dt, alpha=alpha), False)
                self.launches += 1
                g_, u_ = self._get(c, m * n, dt), self._get(d, m * n, dt)
                return self._put(sc, O.silu_mul_fwd(g_, u_)[0], dt)
            for g_ in range(batch):
                if oc == 3:
                    sub = E.op(E.GEMM_SB, a=(a, sa)[g_], b=(b, sb)[g_], c=(c, d)[g_], m=(m, oa)[g_], n=(n, ob)[g_], k=k,
                               batch=1, tb=tb, dt=dt, alpha=alpha)
                elif oc == 1:
                    sub = E.op(E.GEMM_SB, a=a, b=ib[g_], c=ic[g_], m=m, n=dims[g_], k=k, batch=1, tb=tb, dt=dt, alpha=alpha)
                elif g_ == 0 and xs is not None and xs["addend"]:
                    sub = E.op(E.GEMM_EX, a=ia[0], b=ib[0], c=c, d=xs["addend"], m=m, n=n, k=dims[0], batch=1, tb=tb, dt=dt,
                               alpha=alpha, beta=xs["beta"])
                else:
                    sub = E.op(E.GEMM_SB, a=ia[g_], b=ib[g_], c=c, m=m, n=n, k=dims[g_], batch=1, tb=tb, dt=dt, alpha=alpha,
                               beta=1.0 if g_ else 0.0)
                self.launches += 1
                self._gemm(sub, sub[0] == E.GEMM_EX)
                if oc == 1 and xs is not None:      # the output's own low-rank term
                    self._gemm(E.op(E.GEMM_SB, a=xs["a"][g_], b=xs["b"][g_], c=ic[g_], m=m, n=dims[g_], k=xs["k"], batch=1,
                                    tb=tb, dt=dt, alpha=alpha, beta=1.0), False)
            if oc == 2 and xs is not None:          # further K-segments
                for g_ in range(xs["n"]):
                    self._gemm(E.op(E.GEMM_SB, a=xs["a"][g_], b=xs["b"][g_], c=c, m=m, n=n, k=xs["k"], batch=1, tb=tb, dt=dt,
                                    alpha=alpha, beta=1.0), False)
            if oc == 1 and gamma > 0:       # rotary on the first two outputs ([m, heads*64], row = batch*T + token)
                T_ = self.bufs[int(beta)].size // (32 * 4)
                cos = self._f32(int(beta), T_ * 32).reshape(T_, 32)
                sin = self._f32(int(gamma), T_ * 32).reshape(T_, 32)
                for buf_, width in ((c, n), (d, oa)):
                    x = self._get(buf_, m * width, dt).reshape(m // T_, T_, width // 64, 64).transpose(0, 2, 1, 3)
                    self._put(buf_, O.rope_fwd(x, cos, sin).transpose(0, 2, 1, 3), dt)
            return None
        if kind == E.EMBED_I32:
            ids = self.bufs[b].view(np.int32)[:m]
            tab = self._get(a, self.bufs[a].size // (2 if dt == 1 else 4), dt).reshape(-1, n)
            return self._put(c, tab[ids], dt)
        if kind == E.RMSNORM:
            x = self._get(a, m * n, dt).reshape(m, n)
            y, _ = O.rmsnorm_fwd(x, self._get(b, n, dt), alpha)
            return self._put(c, y, dt)
        if kind == E.ROPE_BTHD:
            B_, T, H, DH = batch, m, k, n
            cos = self._f32(b, T * (DH // 2)).reshape(T, DH // 2)
            sin = self._f32(d, T * (DH // 2)).reshape(T, DH // 2)
            for (src, dst, heads) in ((a, c, H),) + (((sa, sb, sc),) if sc > 0 else ()):
                x = self._get(src, B_ * T * heads * DH, dt).reshape(B_, T, heads, DH).transpose(0, 2, 1, 3)
                y = O.rope_bwd(x, cos, sin) if tb else O.rope_fwd(x, cos, sin)
                self._put(dst, y.transpose(0, 2, 1, 3), dt)
            return None
        if kind == E.ATTN_FWD:
            B_, T, DH, KV, H = batch, m, n, k, tb
            q = self._get(a, B_ * T * H * DH, dt).reshape(B_, T, H, DH).transpose(0, 2, 1, 3)
            kk = self._get(b, B_ * T * KV * DH, dt).reshape(B_, T, KV, DH).transpose(0, 2, 1, 3)
            v = self._get(d, B_ * T * KV * DH, dt).reshape(B_, T, KV, DH).transpose(0, 2, 1, 3)
            out, lse = O.attention_fwd(q, kk, v, alpha)
            self._put(c, out.transpose(0, 2, 1, 3), dt)
            return self._put(sa, lse, 0)
        if kind == E.ATTN_BWD:
            B_, T, DH, KV, H = batch, m, n, k, ob
            q = self._get(a, B_ * T * H * DH, dt).reshape(B_, T, H, DH).transpose(0, 2, 1, 3)
            kk = self._get(b, B_ * T * KV * DH, dt).reshape(B_, T, KV, DH).transpose(0, 2, 1, 3)
            v = self._get(d, B_ * T * KV * DH, dt).reshape(B_, T, KV, DH).transpose(0, 2, 1, 3)
            do = self._get(c, B_ * T * H * DH, dt).reshape(B_, T, H, DH).transpose(0, 2, 1, 3)
            dq, dk, dv = O.attention_bwd(q, kk, v, do, alpha)
            if gamma > 0:       # inverse rotary of dq and dk inside the op; beta / gamma name the cos / sin tables
                cos = self._f32(int(beta), T * (DH // 2)).reshape(T, DH // 2)
                sin = self._f32(int(gamma), T * (DH // 2)).reshape(T, DH // 2)
                dq, dk = O.rope_bwd(dq, cos, sin), O.rope_bwd(dk, cos, sin)
            self._put(tb, dq.transpose(0, 2, 1, 3), dt)
            self._put(sc, dk.transpose(0, 2, 1, 3), dt)
            return self._put(oa, dv.transpose(0, 2, 1, 3), dt)
        if kind == E.SILU_MUL:
            g, u = self._get(a, n, dt), self._get(b, n, dt)
            return self._put(c, O.silu_mul_fwd(g, u)[0], dt)
        if kind == E.SILU_BWD:
            g, u, gr = self._get(a, n, dt), self._get(b, n, dt), self._get(d, n, dt)
            sig = 1.0 / (1.0 + np.exp(-g))
            dg, du = O.silu_mul_bwd(g, u, sig, gr)
            self._put(c, dg, dt)
            return self._put(tb, du, dt)
        if kind == E.CE_FUSED:
            lg = self._get(a, m * n, dt).reshape(m, n)
            tg = self.bufs[b].view(np.int32)[:m].astype(np.int64)
            tg = np.where(tg < 0, -1, tg)
            cnt = O.count_valid(tg)
            self._f32(sa)[0] = cnt
            if cnt == 0:
                self._put(c, np.zeros_like(lg), dt)
                self._f32(d)[0] = np.nan
                return
            loss, dl, _ = O.cross_entropy_fwd_bwd(lg, tg, -1)
            self._f32(d)[0] = loss
            return self._put(c, dl, dt)
        if kind == E.RMSNORM_BWD_ACC:
            x = self._get(a, m * n, dt).reshape(m, n)
            w = self._get(b, n, dt)
            g = self._get(d, m * n, dt).reshape(m, n)
            _, inv = O.rmsnorm_fwd(x, w, alpha)
            dx, dw = O.rmsnorm_bwd(x, w, inv, g)
            if tb > 0:
                dx = dx + self._get(tb, m * n, dt).reshape(m, n)
            self._put(c, dx, dt)
            if sa > 0 and oa > 0:       # deferred: the partial sums stay in scratch area oa-1 (row 0 here)
                area = 296 * n
                self._f32(sb)[(oa - 1) * area:(oa - 1) * area + n] = dw
            elif sa > 0:
                self._put(sa, dw, 0)
            return
        if kind == E.COLSUM_BATCH:
            area = 296 * n
            tab = self.bufs[b].view(np.int32)
            for i in range(oa, oa + m):
                part = self._f32(a)[i * area:(i + 1) * area].reshape(296, n)
                off = int(tab[i]) * k
                self._f32(c)[off:off + n] = part.sum(axis=0, dtype=np.float32)
            return
        if kind == E.EMBED_BWD_DET:
            ids = self.bufs[b].view(np.int32)[:m]
            g = self._get(a, m * n, 1 if dt >= 1 else 0).reshape(m, n)
            tab = self._f32(c).reshape(-1, n)
            np.add.at(tab, ids, g)
            return
        if kind == E.ADD:
            return self._put(c, self._get(a, n, dt) + self._get(b, n, dt), dt)
        if kind == E.COPY:
            return self._put(c, self._get(a, n, dt), dt)
        if kind == E.SCALE:
            if alpha == 0.0:
                return self._put(c, np.zeros(n, np.float32), dt)
            return self._put(c, self._get(a, n, dt) * np.float32(alpha), dt)
        if kind == E.CAST:
            cnt = m * max(n, 1)
            if tb == 0:
                return self._put(c, self._get(a, cnt, 0), 1)
            return self._put(c, self._get(a, cnt, 1), 0)
        if kind == E.TRANSPOSE_BF16:
            src = self.bufs[a].view(np.uint16)[:m * n].reshape(m, n).T
            if dt == 1:
                self.bufs[c].view(np.uint16)[:m * n] = src.reshape(-1)
            else:
                self.bufs[c].view(np.float32)[:m * n] = E.bf16_bits_to_f32(np.ascontiguousarray(src).reshape(-1))
            return
        if kind == E.GNORM_FLAT:
            g = self._f32(a, m * E.CHUNK, oa * E.CHUNK)
            if tb > 0:
                self._f32(tb)[0] += 1.0
            self._f32(d)[ob] = np.float32((g.astype(np.float64) ** 2).sum())
            return
        if kind == E.ADAMW_FLAT:
            cnt, off = m * E.CHUNK, k * E.CHUNK
            p = self._f32(a, cnt); mm = self._f32(c, cnt); vv = self._f32(d, cnt)
            g = self._f32(b, cnt, off)
            flags = np.repeat(self.bufs[sc][k:k + m], E.CHUNK).astype(bool)
            tot = float(np.sqrt(np.float32(self._f32(oa, ob).astype(np.float64).sum())))
            if oc > 0:
                self._f32(oc)[0] = tot
            gs = alpha / tot if (alpha > 0 and tot > alpha) else 1.0
            t = float(self._f32(tb)[0]); lr = float(self._f32(sb)[0])
            bc1, bc2 = 1 - 0.9 ** t, 1 - 0.95 ** t
            gi = g * np.float32(gs)
            mm[:] = 0.9 * mm + np.float32(0.1) * gi
            vv[:] = 0.95 * vv + np.float32(0.05) * gi * gi
            decay = np.where(flags, np.float32(1 - lr * beta), np.float32(1.0))
            p[:] = p * decay - np.float32(lr * np.sqrt(bc2) / bc1) * mm / (np.sqrt(vv) + np.float32(gamma * np.sqrt(bc2)))
            if sa > 0:
                self._put(sa, p, 1, off)
            return
        if kind in (E.GROUP, E.FORK, E.JOIN, E.STREAM, E.EVENT):
            return
        if kind in (E.REDUCE, E.BROADCAST, E.ALLREDUCE):
            import torch
            half = kind == E.BROADCAST and dt == 1
            cnt = m * E.CHUNK if m > 0 else n
            off = oa * E.CHUNK if m > 0 else 0
            if half:        # gloo moves bytes; a broadcast does not care about the element type
                view = self.bufs[a][off * 2:(off + cnt) * 2]
            else:
                view = self.bufs[a].view(np.float32)[off:off + cnt]
            tns = torch.from_numpy(view)
            if kind == E.BROADCAST:
                self.dist.broadcast(tns, src=tb)
            elif kind == E.REDUCE:
                self.dist.reduce(tns, dst=tb, op=self.dist.ReduceOp.SUM)
                if self.rank == tb:
                    view /= np.float32(self.world)
            else:
                self.dist.all_reduce(tns, op=self.dist.ReduceOp.SUM)
                view /= np.float32(self.world)
            return
        if kind == E.ALLGATHER_F32:
            import torch
            send = torch.from_numpy(self._f32(a, n, oa).copy())
            outs = [torch.empty(n) for _ in range(self.world)]
            self.dist.all_gather(outs, send)
            self._f32(c)[:n * self.world] = torch.cat(outs).numpy()
            return
        raise NotImplementedError(E.KIND_NAMES[kind])
