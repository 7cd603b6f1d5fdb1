"""ctypes binding to libaxeng.so — the host side of the C ABI.

Mirrors the reference binding (axis/engine.py:17-174): the same 32 op-kind
constants, the same 80-byte op descriptor, the same `op()` builder and the same
`Engine` methods (`alloc / upload / download / new_tensor / run / capture /
replay / sync / set_tf32 / nccl_id / nccl_init`), with integer return codes
turned into `RuntimeError`.  Added on top: fused op kinds (>= 32), buffer
views, raw/typed transfers, packed-plan caching (a plan is packed once, not on
every step) and device-side timing.

There is no CPU path: constructing an `Engine` without the built library or
without a CUDA device raises.
"""
from __future__ import annotations

import ctypes
from typing import Dict, Sequence, Tuple

import numpy as np

# op kinds 0..31 — identical to the reference (axis/engine.py:17-21)
(GEMM, ADD, MUL, SILU_MUL, RMSNORM, ADAMW, SCALE, COPY,
 GEMM_SB, PERM_0213, ROPE, SOFTMAX_CAUSAL, REPEAT_KV,
 RMSNORM_BWD, COLSUM, REPEAT_KV_BWD, SOFTMAX_BWD, SILU_BWD,
 EMBED, EMBED_BWD, CE, TICK, CAST, FLASH, ROWDOT, FLASH_BWD,
 ALLREDUCE, GROUP, L2ACC, CLIPSCALE, COUNTVALID, BROADCAST) = range(32)
# fused kinds of this engine (include/axeng.h)
(GEMM_EX, ROPE_BTHD, ATTN_FWD, ATTN_BWD, RMSNORM_BWD_ACC, CE_FUSED, EMBED_BWD_DET,
 GNORM_FLAT, ADAMW_FLAT, EMBED_I32, REDUCE, ALLGATHER_F32, FORK, JOIN, STREAM,
 SILU_MUL_BWD_RC, GEMM_GROUP, TRANSPOSE_BF16, COLSUM_BATCH, EVENT, GEMM_XSEG, LORA_GRAD, LORA_PROJ) = range(32, 55)
KIND_COUNT = 55
KIND_NAMES = ["GEMM", "ADD", "MUL", "SILU_MUL", "RMSNORM", "ADAMW", "SCALE", "COPY", "GEMM_SB",
              "PERM_0213", "ROPE", "SOFTMAX_CAUSAL", "REPEAT_KV", "RMSNORM_BWD", "COLSUM",
              "REPEAT_KV_BWD", "SOFTMAX_BWD", "SILU_BWD", "EMBED", "EMBED_BWD", "CE", "TICK", "CAST",
              "FLASH", "ROWDOT", "FLASH_BWD", "ALLREDUCE", "GROUP", "L2ACC", "CLIPSCALE",
              "COUNTVALID", "BROADCAST", "GEMM_EX", "ROPE_BTHD", "ATTN_FWD", "ATTN_BWD",
              "RMSNORM_BWD_ACC", "CE_FUSED", "EMBED_BWD_DET", "GNORM_FLAT", "ADAMW_FLAT",
              "EMBED_I32", "REDUCE", "ALLGATHER_F32", "FORK", "JOIN", "STREAM", "SILU_MUL_BWD_RC",
              "GEMM_GROUP", "TRANSPOSE_BF16", "COLSUM_BATCH", "EVENT", "GEMM_XSEG", "LORA_GRAD", "LORA_PROJ"]

_I32_MAX = 2 ** 31 - 1
CHUNK = 1024          # arena granularity of the flat optimizer / collective ops
GNORM_CHUNK = 8192    # elements per grad-norm partial


class _EngOp(ctypes.Structure):
    _fields_ = [
        ("kind", ctypes.c_int),
        ("a", ctypes.c_int), ("b", ctypes.c_int),
        ("c", ctypes.c_int), ("d", ctypes.c_int),
        ("m", ctypes.c_int), ("n", ctypes.c_int), ("k", ctypes.c_int),
        ("batch", ctypes.c_int), ("tb", ctypes.c_int),
        ("sa", ctypes.c_int), ("sb", ctypes.c_int), ("sc", ctypes.c_int),
        ("dt", ctypes.c_int),
        ("oa", ctypes.c_int), ("ob", ctypes.c_int), ("oc", ctypes.c_int),
        ("alpha", ctypes.c_float), ("beta", ctypes.c_float), ("gamma", ctypes.c_float),
    ]


_OP_DTYPE = np.dtype([(n, "<i4") for n in
                      ("kind", "a", "b", "c", "d", "m", "n", "k", "batch", "tb", "sa", "sb", "sc",
                       "dt", "oa", "ob", "oc")] + [(n, "<f4") for n in ("alpha", "beta", "gamma")])
assert _OP_DTYPE.itemsize == ctypes.sizeof(_EngOp) == 80


def op(kind: int, a: int = -1, b: int = -1, c: int = -1, d: int = -1,
       m: int = 0, n: int = 0, k: int = 0,
       batch: int = 0, tb: int = 0, sa: int = 0, sb: int = 0, sc: int = 0,
       dt: int = 0, oa: int = 0, ob: int = 0, oc: int = 0,
       alpha: float = 0.0, beta: float = 0.0, gamma: float = 0.0) -> Tuple:
    """Op descriptor tuple, field for field the reference's (axis/engine.py:38-75).
    dt: 0 = fp32, 1 = bf16 storage, 2 = bf16 inputs / fp32 output.

    Role maps of the reference kinds are unchanged.  Fused kinds (extra buffer
    references in tb/sa/sb/sc/oa/ob/oc follow the reference's "0 = none"
    convention — slot 0 is always the rotary cos table):

    GEMM_EX:   as GEMM_SB, plus d = addend with c's shape: c = alpha*a@b + beta*d
    ROPE_BTHD: a=x b=cos d=sin c=out on [batch=B, m=T, k=heads, n=DH]; tb=1 inverse; optional second
               tensor in the same launch: sa=x2 sb=out2 sc=its heads (0 = none)
    ATTN_FWD:  a=q [B,T,H,DH] b=k d=v [B,T,KV,DH] c=o; sa=lse [B,H,T];
               m=T n=DH k=KV batch=B tb=H; alpha=scale
    ATTN_BWD:  a=q b=k d=v c=dO; sa=lse sb=o tb=dq sc=dk oa=dv ob=H oc=scratch (B*H*T
               floats, plus B*T*H*DH floats to enable the tensor-core path);
               m=T n=DH k=KV batch=B; alpha=scale; outputs in storage dtype;
               gamma > 0: dq and dk leave the op with the inverse rotary applied, beta / gamma
               being the buffer indices of the cos / sin tables (float-encoded, sin never slot 0)
    RMSNORM_BWD_ACC: a=x b=w d=g c=dx; tb=residual added to dx; sa=dw (fp32);
               sb=scratch; m=N n=D; alpha=eps
    CE_FUSED:  a=logits b=targets(int32) c=dlogits (may alias a) d=loss; sa=count
               out; sb=scratch (N+8 floats); m=N n=V
    EMBED_BWD_DET: a=g b=ids(int32) c=table grad (fp32, accumulated); m=N n=D
    EMBED_I32: a=table b=ids(int32) c=out; m=N n=D
    GNORM_FLAT: a=grad arena c=partials scratch; m=chunks oa=chunk offset;
               d=scalar out buffer, ob=index in it; tb=step counter to tick
    ADAMW_FLAT: a=master b=grad arena c=m d=v; m=chunks; k=chunk offset applied to
               b / mirror / flags; sa=bf16 mirror arena; sb=lr; tb=t; sc=decay
               flags; oa=sumsq scalars, ob=their count; oc=norm out;
               alpha=max_norm beta=wd gamma=eps
    REDUCE / BROADCAST / ALLREDUCE with m>0: m chunks at chunk offset oa of a
    ALLGATHER_F32: a=send (offset oa) c=recv; n=count per rank
    FORK / JOIN / STREAM(tb): side-stream control for overlapped collectives (tb: 0 main, 1 collectives,
               2 side stream of the overlapped weight-gradient GEMMs)
    EVENT: tb=1 record event oa on stream sa / tb=2 stream sa waits for event oa (sa as STREAM's tb)
    GEMM_GROUP: batch = 2 or 3 GEMMs of one layer as one launch; m, tb, dt, alpha as GEMM_SB.
               oc=1 (one input, several outputs): a=A; b,sa,sb = B_g; c,d,sc = C_g; n,oa,ob = n_g; k;
                    gamma > 0: outputs 0 and 1 are [m, heads*64] query / key projections (row = batch*T + token)
                    and leave the op with the rotary embedding applied; beta / gamma = buffer indices of the
                    cos / sin tables ([T, 32] fp32)
               oc=2 (one output summed over K-segments): c=C; a,sa,sb = A_s; b,d,sc = B_s;
               k,oa,ob = k_s; n
               oc=3 (two independent problems of one depth k): a,sa = A_g; b,sb = B_g; c,d = C_g;
               m,oa = m_g; n,ob = n_g
               oc=4 (SwiGLU pair, batch=2): a=A; b=gate weights, sa=up weights (n wide each);
               c=g, d=u, sc=h=silu(g)*u
    GEMM_XSEG: no launch — extra operands of the NEXT GEMM_GROUP: a,b,d = A'_g; sa,sb,sc = B'_g (batch of them, depth k
               each); before oc=1: output g gets + A'_g B'_g (an adapter's low-rank term inside the projection's launch);
               before oc=2 (batch may then be 1): they are further K-segments of the sum (six at most in all), and
               c > 0 = addend D with factor beta: C = alpha * sum + beta * D
    LORA_GRAD: adapter weight gradients alpha * X_g^T S_g of batch <= 3 projections: X_g = a,sa,sb (0 = same as a) [m, F_g];
               S_g = b,d,sc [m, R]; F_g = n,k,tb; R = gamma; out = fp32 buffer c at element offsets oa,ob,oc, laid out
               [F_g, R], or [R, F_g] with beta = 1; dt 1/2 = bf16 inputs; batch < 0: the |batch| products are only noted (at most
               16), batch = 0: everything noted runs as one launch pair (a whole layer's adapters)
    LORA_PROJ: out_g [m, R] = alpha * X_g W_g for batch <= 3 adapters: X_g = a,sa,sb (0 = same as a) [m, F_g]; W_g = b,d,sc,
               [F_g, R] with tb=0 (u = x A) or [R, F_g] with tb=1 (t = g B^T); out_g = buffers c,oa,ob; F_g = n,k,oc; R = gamma
    RMSNORM_BWD_ACC with oa=j>0: dw is deferred, the per-block partial sums stay in area j-1 of the scratch sb
               (areas of 296*n floats, allocated zeroed)
    COLSUM_BATCH: a=scratch areas, b=int32 table, c=fp32 arena; areas oa..oa+m-1 are summed into
               c[table[i]*k : +n]
    TRANSPOSE_BF16: a = bf16 [m,n]; c = [n,m], bf16 (dt=1) or widened to fp32 (dt=0); not in place
    """
    return (kind, a, b, c, d, m, n, k, batch, tb, sa, sb, sc, dt, oa, ob, oc,
            alpha, beta, gamma)


class PackedPlan:
    """A plan packed into the C array once; reusable across steps."""

    def __init__(self, plan: Sequence[Tuple]):
        arr = np.zeros(len(plan), dtype=_OP_DTYPE)
        if len(plan):
            cols = list(zip(*plan))
            for j, name in enumerate(_OP_DTYPE.names):
                if j >= 17:
                    arr[name] = np.asarray(cols[j], dtype=np.float32)
                    continue
                col = np.asarray(cols[j], dtype=np.int64)
                bad = np.nonzero((col > _I32_MAX) | (col < -_I32_MAX - 1))[0]
                if bad.size:        # the descriptor's integer fields are 32 bits wide: refuse, never wrap
                    i = int(bad[0])
                    raise OverflowError(f"op {i} (kind {plan[i][0]}): field '{name}' = {int(col[i])} does not fit "
                                        f"the 32-bit op descriptor")
                arr[name] = col
        self.arr = arr
        self.n = len(plan)
        self.ptr = arr.ctypes.data_as(ctypes.POINTER(_EngOp))


class Engine:
    """Owns the runtime: buffers, plans, graphs (axis/engine.py:78-174)."""

    def __init__(self, lib_path: str = None):
        if lib_path is None:
            from axis_b200._build import engine_lib
            lib_path = engine_lib()
        self.lib_path = lib_path
        self.lib = L = ctypes.CDLL(lib_path)
        c_i, c_ll, c_p = ctypes.c_int, ctypes.c_longlong, ctypes.c_void_p
        L.eng_init.restype = c_i
        L.eng_alloc.argtypes = [c_i, c_ll, c_i]
        L.eng_upload.argtypes = [c_i, ctypes.POINTER(ctypes.c_float), c_ll]
        L.eng_download.argtypes = [c_i, ctypes.POINTER(ctypes.c_float), c_ll]
        L.eng_run_plan.argtypes = [ctypes.POINTER(_EngOp), c_i, c_i]
        L.eng_capture_plan.argtypes = [ctypes.POINTER(_EngOp), c_i]
        L.eng_replay.argtypes = [c_i, c_i]
        L.eng_nccl_id.argtypes = [c_p]
        L.eng_nccl_init.argtypes = [c_i, c_i, c_p]
        L.eng_nccl_init_timeout.argtypes = [c_i, c_i, c_p, c_i]
        L.eng_alloc_view.argtypes = [c_i, c_i, c_ll, c_ll]
        L.eng_alloc_zero.argtypes = [c_i, c_ll]
        L.eng_upload_raw.argtypes = [c_i, c_ll, c_p, c_ll]
        L.eng_download_raw.argtypes = [c_i, c_ll, c_p, c_ll]
        L.eng_upload_tokens.argtypes = [c_i, c_p, c_ll, c_ll]
        L.eng_download_async.argtypes = [c_i, c_ll]
        L.eng_download_wait.argtypes = [c_i, c_p, c_ll]
        L.eng_last_error.restype = ctypes.c_char_p
        L.eng_time_plan.argtypes = [ctypes.POINTER(_EngOp), c_i, c_i, c_i, ctypes.POINTER(ctypes.c_float)]
        L.eng_profile_read.argtypes = [ctypes.POINTER(ctypes.c_float), ctypes.POINTER(c_i), c_i]
        L.eng_launch_count.restype = c_ll
        L.eng_launch_count.argtypes = [c_i]
        L.eng_bytes_allocated.restype = c_ll
        rc = L.eng_init()
        if rc:
            raise RuntimeError(f"engine init failed rc={rc}: {self.last_error()}")
        self._next = 0
        self.has_flash = bool(L.eng_has_flash())
        self._packed: Dict[int, PackedPlan] = {}

    def last_error(self) -> str:
        return (self.lib.eng_last_error() or b"").decode(errors="replace")

    def _check(self, rc: int, what: str) -> None:
        if rc:
            raise RuntimeError(f"{what} failed rc={rc}: {self.last_error()}")

    # ── buffers ──
    def _slot(self) -> int:
        idx = self._next
        self._next += 1
        return idx

    def alloc(self, nelems: int, itemsize: int = 4) -> int:
        idx = self._slot()
        self._check(self.lib.eng_alloc(idx, int(nelems), int(itemsize)), f"alloc({nelems}x{itemsize})")
        return idx

    def alloc_zero(self, nbytes: int) -> int:
        idx = self._slot()
        self._check(self.lib.eng_alloc_zero(idx, int(nbytes)), f"alloc_zero({nbytes})")
        return idx

    def view(self, parent: int, byte_offset: int, nbytes: int) -> int:
        idx = self._slot()
        self._check(self.lib.eng_alloc_view(idx, parent, int(byte_offset), int(nbytes)), "alloc_view")
        return idx

    def upload(self, idx: int, arr: np.ndarray) -> None:
        a = np.ascontiguousarray(arr, dtype=np.float32)
        self._check(self.lib.eng_upload(idx, a.ctypes.data_as(ctypes.POINTER(ctypes.c_float)), a.size), "upload")

    def download(self, idx: int, shape) -> np.ndarray:
        out = np.empty(shape, dtype=np.float32)
        self._check(self.lib.eng_download(idx, out.ctypes.data_as(ctypes.POINTER(ctypes.c_float)), out.size), "download")
        return out

    def upload_raw(self, idx: int, arr: np.ndarray, byte_offset: int = 0) -> None:
        a = np.ascontiguousarray(arr)
        self._check(self.lib.eng_upload_raw(idx, int(byte_offset), a.ctypes.data, a.nbytes), "upload_raw")

    def download_raw(self, idx: int, shape, dtype, byte_offset: int = 0) -> np.ndarray:
        out = np.empty(shape, dtype=dtype)
        self._check(self.lib.eng_download_raw(idx, int(byte_offset), out.ctypes.data, out.nbytes), "download_raw")
        return out

    def download_async(self, idx: int, nfloats: int = 1) -> int:
        """Queue a read-back of `nfloats` floats behind the queued work; returns a ticket for download_wait."""
        tk = self.lib.eng_download_async(idx, int(nfloats))
        if tk < 0:
            raise RuntimeError(f"download_async failed rc={tk}: {self.last_error()}")
        return tk

    def download_wait(self, ticket: int, nfloats: int = 1) -> np.ndarray:
        out = np.empty(int(nfloats), dtype=np.float32)
        self._check(self.lib.eng_download_wait(int(ticket), out.ctypes.data, int(nfloats)), "download_wait")
        return out

    def upload_bf16(self, idx: int, arr: np.ndarray) -> None:
        self.upload_raw(idx, f32_to_bf16_bits(arr))

    def download_bf16(self, idx: int, shape) -> np.ndarray:
        return bf16_bits_to_f32(self.download_raw(idx, shape, np.uint16))

    def upload_tokens(self, idx: int, tokens: np.ndarray, limit: int) -> None:
        t = np.ascontiguousarray(tokens, dtype=np.int64).reshape(-1)
        self._check(self.lib.eng_upload_tokens(idx, t.ctypes.data, t.size, int(limit)), "upload_tokens")

    def new_tensor(self, arr: np.ndarray) -> int:
        idx = self.alloc(arr.size)
        self.upload(idx, arr)
        return idx

    # ── NCCL ──
    def nccl_id(self) -> bytes:
        buf = (ctypes.c_char * 128)()
        self._check(self.lib.eng_nccl_id(buf), "nccl_id")
        return bytes(buf)

    def nccl_init(self, rank: int, world: int, uid: bytes, timeout_ms: int = 0) -> None:
        if len(uid) != 128:
            raise ValueError("NCCL unique id must be 128 bytes")
        rc = self.lib.eng_nccl_init_timeout(rank, world, uid, int(timeout_ms))
        self._check(rc, f"nccl_init(rank={rank}/{world})")

    # ── plans ──
    def pack(self, plan) -> PackedPlan:
        if isinstance(plan, PackedPlan):
            return plan
        key = id(plan)
        pp = self._packed.get(key)
        if pp is None or pp.n != len(plan):
            pp = PackedPlan(plan)
            if isinstance(plan, list) and len(plan) > 64:      # long-lived step plans
                self._packed[key] = pp
                pp._keep = plan
        return pp

    def zero(self, idx: int, nfloats: int) -> Tuple:
        return op(SCALE, a=idx, c=idx, n=nfloats, alpha=0.0)

    def run(self, plan, sync: bool = True) -> None:
        pp = self.pack(plan)
        rc = self.lib.eng_run_plan(pp.ptr, pp.n, 1 if sync else 0)
        if rc:
            where = "?"
            if rc >= 1000:
                kind = int(pp.arr["kind"][rc - 1000])
                where = f"op {rc - 1000} kind {KIND_NAMES[kind] if 0 <= kind < KIND_COUNT else kind}"
            raise RuntimeError(f"run_plan failed rc={rc} ({where}): {self.last_error()}")

    def capture(self, plan) -> None:
        pp = self.pack(plan)
        rc = self.lib.eng_capture_plan(pp.ptr, pp.n)
        if rc:
            raise RuntimeError(f"capture failed rc={rc}: {self.last_error()}")

    def replay(self, times: int = 1, sync: bool = True) -> None:
        self._check(self.lib.eng_replay(times, 1 if sync else 0), "replay")

    def sync(self) -> None:
        self._check(self.lib.eng_sync(), "sync")

    def set_tf32(self, on: bool) -> None:
        self.lib.eng_set_tf32(1 if on else 0)

    def set_fallback(self, mask: int) -> None:
        self.lib.eng_set_fallback(int(mask))

    # ── measurement ──
    def time_plan(self, plan, reps: int = 10, flush_l2: bool = True) -> float:
        """Mean milliseconds per execution (CUDA events on the engine stream)."""
        pp = self.pack(plan)
        ms = ctypes.c_float(0)
        rc = self.lib.eng_time_plan(pp.ptr, pp.n, reps, 1 if flush_l2 else 0, ctypes.byref(ms))
        if rc:
            raise RuntimeError(f"time_plan failed rc={rc}: {self.last_error()}")
        return float(ms.value)

    def profile(self, on: bool) -> None:
        self.lib.eng_profile(1 if on else 0)

    def profile_read(self) -> Dict[str, Tuple[float, int]]:
        ms = (ctypes.c_float * KIND_COUNT)()
        calls = (ctypes.c_int * KIND_COUNT)()
        self.lib.eng_profile_read(ms, calls, KIND_COUNT)
        return {KIND_NAMES[i]: (float(ms[i]), int(calls[i])) for i in range(KIND_COUNT) if calls[i]}

    def launch_count(self, reset: bool = False) -> int:
        return int(self.lib.eng_launch_count(1 if reset else 0))

    def device_status(self, clear: bool = True) -> int:
        return int(self.lib.eng_device_status(1 if clear else 0))

    def last_variant(self) -> int:
        """Code of the kernel variant the last GEMM / cross-entropy op ran on (include/axeng.h)."""
        return int(self.lib.eng_last_variant())

    def bytes_allocated(self) -> int:
        return int(self.lib.eng_bytes_allocated())

    def shutdown(self) -> None:
        self.lib.eng_shutdown()


def f32_to_bf16_bits(a: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even fp32 -> bf16, as uint16 bit patterns."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    r = ((u >> 16) & 1) + np.uint32(0x7FFF)
    return ((u + r) >> 16).astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (b.astype(np.uint32) << 16).view(np.float32)
