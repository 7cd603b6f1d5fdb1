"""Lowering of a Llama-class training step to one fused execution plan.

Host-side mirror of the reference's `axis.compile` (axis/compile.py:27-664):
same constructor arguments, same public attributes (`eng, pnames, shapes,
owner, owned, rank, world, zero, attn_impl, lr, dtype, B, T, N, V, lora_r`) and
same methods (`step / capture / replay_step / set_lr / grads / get_weights /
state_dict / load_state_dict`).  What differs is the plan it emits:

* parameters, gradients and AdamW moments live in flat arenas (per-tensor
  buffers are windows into them), so clipping + AdamW is two launches over the
  arena instead of two per tensor;
* q/k/v stay in the [B,T,H,DH] layout the projections produce — rotary is
  applied in place and the attention kernels read that layout directly, so no
  head permutes exist;
* residual adds ride in GEMM epilogues and in the RMSNorm backward; gradient
  joins use accumulate-in-epilogue GEMMs; RMSNorm backward produces dx and dw
  in one pass; cross-entropy writes dlogits over the logits; the embedding
  scatter-add is ordered (no atomics);
* data parallel: gradients are reduced to their owner rank in buckets on a
  side stream while backward continues (axis/compile.py:490-496 all-reduces
  per tensor after backward); ZeRO-1 keeps the reference's per-tensor greedy
  owner map (axis/compile.py:128-139) bit for bit.

Additions to the reference's surface: `recompute_blocks` (per-block activation recompute),
`step_accumulate` (gradient accumulation), `replay_step_async` / `flush` (the host reads step i's loss after
step i+1 is queued), and weights given as checkpoint tensors still in their file layout (see pretrained.py).
"""
from __future__ import annotations

from typing import Dict, List, Sequence

import numpy as np

from axis_b200.engine import (
    ADAMW_FLAT, ADD, ALLGATHER_F32, ATTN_BWD, ATTN_FWD, BROADCAST, CAST, CE_FUSED, CHUNK, COLSUM_BATCH, COPY, EMBED_BWD_DET,
    EMBED_I32, FORK, GEMM_EX, GEMM_GROUP, GEMM_SB, GEMM_XSEG, GNORM_FLAT, GROUP, JOIN, LORA_GRAD, LORA_PROJ, REDUCE, RMSNORM, RMSNORM_BWD_ACC,
    ROPE_BTHD, SCALE, SILU_BWD, SILU_MUL, STREAM, EVENT, Engine, f32_to_bf16_bits, op)

LIN_ORDER = ("attn.q_proj", "attn.k_proj", "attn.v_proj", "attn.o_proj",
             "mlp.gate_proj", "mlp.up_proj", "mlp.down_proj")
RB_BLOCKS = 148 * 2          # blocks of the fused RMSNorm backward (scratch rows)


def _numel(shape) -> int:
    return int(np.prod(shape))


def _pad(n: int, q: int = CHUNK) -> int:
    return (n + q - 1) // q * q


def greedy_owner(pnames: Sequence[str], shapes: Dict[str, tuple], world: int, sharded: bool):
    """Per-tensor owner map, identical to axis/compile.py:132-137: visit tensors
    by decreasing size (stable), give each to the first least-loaded rank."""
    load = [0] * world
    owner = {}
    for nm in sorted(pnames, key=lambda n: -_numel(shapes[n])):
        r = int(np.argmin(load)) if sharded else 0
        owner[nm] = r
        load[r] += _numel(shapes[nm])
    return owner, load


class CompiledTransformer:
    def __init__(self, lib_path: str, cfg: dict, weights: Dict[str, np.ndarray],
                 batch: int, seq: int, lr: float = 3e-4, wd: float = 0.1,
                 eps: float = 1e-5, tf32: bool = True, recompute_attn: bool = True,
                 dtype: str = "fp32", attn_tile: int = 256, attn_impl: str = "auto",
                 lora_r: int = 0, lora_alpha: float = 16.0,
                 lora_targets=("q_proj", "k_proj", "v_proj", "o_proj",
                               "gate_proj", "up_proj", "down_proj"),
                 grad_sync: bool = False, max_grad_norm: float = 0.0,
                 zero_stage: int = 0, rank: int = 0, world: int = 1,
                 bucket_layers: int = 4, adam_eps: float = 1e-8, recompute_blocks: bool = False,
                 overlap_dw: bool = True):
        assert dtype in ("fp32", "bf16")
        assert attn_impl in ("auto", "flash", "tiled")
        self.cfg = cfg
        self.B, self.T = batch, seq
        self.lr, self.wd = lr, wd
        self.max_grad_norm = max_grad_norm
        self.dtype = dtype
        hf = dtype == "bf16"
        DT = 1 if hf else 0
        DTW = 2 if hf else 0
        isz = 2 if hf else 4
        V, D = cfg["vocab_size"], cfg["dim"]
        L, H = cfg["n_layers"], cfg["n_heads"]
        KV = cfg.get("n_kv_heads") or H
        DH = D // H
        MLP = cfg["mlp_hidden"]
        tied = cfg.get("tie_embeddings", True)
        theta = cfg.get("rope_theta", 10000.0)
        B, T = batch, seq
        N = B * T
        scale = 1.0 / float(np.sqrt(DH))
        self.N, self.V = N, V
        self._L = L
        lora = lora_r > 0
        sc_l = float(lora_alpha) / lora_r if lora else 0.0
        self.lora_r = lora_r
        lin_geom = {"attn.q_proj": (D, H * DH), "attn.k_proj": (D, KV * DH),
                    "attn.v_proj": (D, KV * DH), "attn.o_proj": (H * DH, D),
                    "mlp.gate_proj": (D, MLP), "mlp.up_proj": (D, MLP),
                    "mlp.down_proj": (MLP, D)}
        lset = set(lora_targets) if lora else set()
        if H % KV or DH % 2:
            raise ValueError("n_heads must be a multiple of n_kv_heads and head_dim even")

        # lib_path is the library path (None = the in-tree build); an object with the
        # Engine interface is used as is (the CPU tests pass a plan interpreter)
        eng = lib_path if hasattr(lib_path, "alloc") else Engine(lib_path)
        eng.set_tf32(tf32)
        self.eng = eng
        A = eng.alloc
        # the fused attention ops serve fp32 and bf16 alike; "tiled" is accepted for API
        # compatibility and runs the same kernels
        self.attn_impl = "flash" if (hf and attn_impl != "tiled") else "tiled"
        self.attn_tile = max(1, min(attn_tile, T))

        # slot 0 / 1: rotary tables (fp32) — slot 0 doubles as the "none" sentinel
        half = DH // 2
        freqs = 1.0 / (theta ** (np.arange(half, dtype=np.float32) / half))
        ang = np.outer(np.arange(T, dtype=np.float32), freqs)
        b_cos = eng.new_tensor(np.cos(ang).astype(np.float32))
        b_sin = eng.new_tensor(np.sin(ang).astype(np.float32))
        assert b_cos == 0

        # ── parameter names / shapes (axis/compile.py:95-122) ──
        base_names = ["embed.weight"]
        for i in range(L):
            p = f"blocks.{i}."
            base_names += [p + "attn_norm.weight", p + "attn.q_proj.weight",
                           p + "attn.k_proj.weight", p + "attn.v_proj.weight",
                           p + "attn.o_proj.weight", p + "mlp_norm.weight",
                           p + "mlp.gate_proj.weight", p + "mlp.up_proj.weight",
                           p + "mlp.down_proj.weight"]
        base_names.append("norm.weight")
        if not tied:
            base_names.append("lm_head.weight")
        if lora:
            self.pnames, self.shapes = [], {}
            for i in range(L):
                for pref, (fin, fout) in lin_geom.items():
                    if pref.split(".")[-1] in lset:
                        self.pnames += [f"blocks.{i}.{pref}.lora_a", f"blocks.{i}.{pref}.lora_b"]
                        self.shapes[f"blocks.{i}.{pref}.lora_a"] = (fin, lora_r)
                        self.shapes[f"blocks.{i}.{pref}.lora_b"] = (lora_r, fout)
        else:
            self.pnames = base_names
            self.shapes = {nm: tuple(weights[nm].shape) for nm in self.pnames}

        # ── ownership (ZeRO-1) ──
        zero = zero_stage >= 1 and world > 1
        if zero:
            assert hf, "ZeRO sharding requires dtype='bf16'"
            assert grad_sync, "ZeRO sharding requires grad_sync=True (multi-GPU)"
        self.owner, _ = greedy_owner(self.pnames, self.shapes, world, zero)
        self.rank, self.world, self.zero = rank, world, zero
        self.owned = [nm for nm in self.pnames if not zero or self.owner[nm] == rank]
        self.grad_sync = bool(grad_sync) and world > 1
        # reduction owner: the same greedy map over `world` ranks in both modes, so that
        # replicated DP and ZeRO-1 sum every gradient in the same order
        cw = world if self.grad_sync else 1
        self._cown, _ = greedy_owner(self.pnames, self.shapes, cw, cw > 1)

        # ── arena layout: by reduction owner, then by bucket (order of completion in backward) ──
        # Layers complete in reverse order; `bucket_layers` of them form a bucket, except that the layers finished
        # last (the first of the model) form buckets of half, a quarter ... one layer: the reduction of the final
        # bucket has nothing left to hide behind, and under ZeRO-1 the first forward ops of the next step wait for
        # exactly these weights, so both should be small.
        sizes, rem = [], L
        while rem > bucket_layers:
            sizes.append(bucket_layers); rem -= bucket_layers
        while rem > 1:
            sizes.append(rem - rem // 2); rem //= 2
        sizes.append(1)
        pos_bucket, bucket_end = [], set()      # backward position (L-1-layer) -> bucket; positions that end a bucket
        for b_, sz in enumerate(sizes):
            pos_bucket += [1 + b_] * sz
            bucket_end.add(len(pos_bucket) - 1)

        def bucket_of(nm: str) -> int:
            if nm in ("norm.weight", "lm_head.weight"):
                return 0
            if nm == "embed.weight":         # its scatter-add ends the backward: a bucket of its own, reduced last
                return 1 + len(sizes)
            return pos_bucket[L - 1 - int(nm.split(".")[1])]
        nb = 2 + len(sizes)
        self._nbuckets = nb
        off = 0
        self._off: Dict[str, int] = {}
        self._seg = []                     # (start, length) per reduction owner, in elements
        self._groups = [[None] * nb for _ in range(cw)]     # (start, length) of (owner, bucket)
        for r in range(cw):
            s0 = off
            for b in range(nb):
                g0 = off
                for nm in self.pnames:
                    if self._cown[nm] == r and bucket_of(nm) == b:
                        self._off[nm] = off
                        off += _pad(_numel(self.shapes[nm]))
                self._groups[r][b] = (g0, off - g0)
            self._seg.append((s0, off - s0))
        P_total = off
        self._P_total = P_total
        my_seg = self._seg[rank] if zero else (0, P_total)
        self._my_seg = my_seg

        # arenas: grads (all), mirror (all, bf16 mode), master/m/v (own segment under ZeRO)
        self.a_grad = eng.alloc_zero(P_total * 4)
        self.a_master = eng.alloc_zero(max(my_seg[1], 1) * 4)
        self.a_m = eng.alloc_zero(max(my_seg[1], 1) * 4)
        self.a_v = eng.alloc_zero(max(my_seg[1], 1) * 4)
        self.a_mirror = eng.alloc_zero(P_total * 2) if hf else -1
        flags = np.zeros(max(P_total // CHUNK, 1), dtype=np.uint8)
        for nm in self.pnames:
            if len(self.shapes[nm]) >= 2:
                o = self._off[nm] // CHUNK
                flags[o:o + _pad(_numel(self.shapes[nm])) // CHUNK] = 1
        self.b_wdflag = eng.alloc(max(flags.size, 4), 1)
        eng.upload_raw(self.b_wdflag, flags)

        self.master, self.gbuf, self._mb, self._vb = {}, {}, {}, {}
        P: Dict[str, int] = {}               # compute view of every weight the plan reads
        src = dict(weights)
        # A weight is an fp32 array, or a checkpoint tensor still in its file layout (an object with
        # `shape` in this engine's layout and `load_into`, see pretrained.HfTensor) that is converted on the
        # device through one staging buffer.
        lazy = [w for w in src.values() if hasattr(w, "load_into")]
        stage = A(max(_numel(w.shape) for w in lazy), 2) if lazy else -1

        def put(dst: int, w, fp32_out: bool) -> None:
            if hasattr(w, "load_into"):
                w.load_into(eng, dst, fp32_out, stage)
            elif fp32_out:
                eng.upload(dst, np.ascontiguousarray(w, dtype=np.float32).reshape(-1))
            else:
                eng.upload_raw(dst, f32_to_bf16_bits(np.ascontiguousarray(w, dtype=np.float32)))
        if lora:
            rng_l = np.random.default_rng(0)
            for i in range(L):
                for pref, (fin, fout) in lin_geom.items():
                    if pref.split(".")[-1] in lset:
                        ka, kb = f"blocks.{i}.{pref}.lora_a", f"blocks.{i}.{pref}.lora_b"
                        if ka not in src:
                            src[ka] = (rng_l.standard_normal((fin, lora_r)) / np.sqrt(lora_r)).astype(np.float32)
                        if kb not in src:
                            src[kb] = np.zeros((lora_r, fout), dtype=np.float32)
            # frozen base: compute copies only (bf16 bits converted on the host, or fp32)
            tot = sum(_pad(_numel(weights[nm].shape)) for nm in base_names)
            self.a_base = eng.alloc_zero(tot * isz)
            o = 0
            for nm in base_names:
                n_el = _numel(weights[nm].shape)
                P[nm] = eng.view(self.a_base, o * isz, n_el * isz)
                put(P[nm], weights[nm], not hf)
                o += _pad(n_el)
        for nm in self.pnames:
            n_el = _numel(self.shapes[nm])
            o = self._off[nm]
            self.gbuf[nm] = eng.view(self.a_grad, o * 4, n_el * 4)
            w = src[nm]
            if tuple(w.shape) != tuple(self.shapes[nm]):
                raise ValueError(f"{nm}: shape {w.shape} != {self.shapes[nm]}")
            if hf:
                P[nm] = eng.view(self.a_mirror, o * 2, n_el * 2)
            if not zero or self._cown[nm] == rank:
                lo = o - my_seg[0]
                self.master[nm] = eng.view(self.a_master, lo * 4, n_el * 4)
                self._mb[nm] = eng.view(self.a_m, lo * 4, n_el * 4)
                self._vb[nm] = eng.view(self.a_v, lo * 4, n_el * 4)
                put(self.master[nm], w, True)
                if not hf:
                    P[nm] = self.master[nm]
            if hf and zero and self._cown[nm] != rank:
                put(P[nm], w, False)
        if hf and my_seg[1] > 0:
            eng.run(self._cast_segment())
        self.pb = P

        # ── io + scalars ──
        self.b_ids = A(N)            # int32 token ids
        self.b_tgt = A(N)            # int32 targets (< 0 ignored)
        self.b_loss = A(1)
        self.b_denom = A(1)          # valid-target count
        self.b_lr = eng.new_tensor(np.array([lr], dtype=np.float32))
        self.b_t = eng.new_tensor(np.zeros(1, dtype=np.float32))
        self.b_gnorm = A(1)          # global gradient norm of the last step
        self.b_sumsq = eng.alloc_zero(4 * 64)             # per-owner (or, on one GPU, per-bucket) sums of squares
        self.b_sumsq_local = eng.alloc_zero(4)
        npart = max(1, (max(s[1] for s in self._seg) + 8191) // 8192)
        self.b_partials = A(npart)
        self.b_ce_scratch = A(N + 8)
        # RMSNorm backward leaves its per-block dw partials in one zeroed scratch area per norm; a batched column
        # sum per reduction bucket turns them into the weight gradients (one launch instead of one per norm)
        n_norms = 0 if lora else 2 * L + 1
        self.b_rb_scratch = eng.alloc_zero(max(n_norms, 1) * RB_BLOCKS * D * 4)
        self.b_rb_table = A(max(n_norms, 1))
        rb_names: List[str] = []             # norm weights in the order of their backward launches
        rb_pending: List[int] = []

        # ── saved activations ──
        # With recompute_blocks only the input of every block is kept (N*D per layer); the other
        # activations live in ONE set of buffers that every block overwrites, and the backward re-runs a
        # block's forward from its saved input before it differentiates it (the eager engine's
        # ops.checkpoint, axis/ops.py:440-475, per transformer block).  Every forward kernel is
        # deterministic, so the recomputed activations are the bits of the first pass: the backward sees
        # the same inputs as without recompute.
        self.recompute_blocks = rc = bool(recompute_blocks)

        def per_layer(n_el, esz=isz):
            if rc:
                return [A(n_el, esz)] * L
            return [A(n_el, esz) for _ in range(L)]
        xs = [A(N * D, isz) for _ in range(L + 1)]
        ys = per_layer(N * D)
        q2s = per_layer(N * H * DH)
        k2s = per_layer(N * KV * DH)
        vs = per_layer(N * KV * DH)
        at2s = per_layer(N * H * DH)
        r1s = per_layer(N * D)
        zs = per_layer(N * D)
        gs = per_layer(N * MLP)
        us = per_layer(N * MLP)
        hs = per_layer(N * MLP)
        lses = per_layer(B * H * T, 4)
        # ── scratch ──
        xf = A(N * D, isz)
        logits = A(N * V, isz)               # dlogits overwrite the logits
        dxf = A(N * D, isz)
        dcur = A(N * D, isz); dr1 = A(N * D, isz); dz = A(N * D, isz); dy = A(N * D, isz)
        dh_ = A(N * MLP, isz); dg_ = A(N * MLP, isz); du_ = A(N * MLP, isz)
        dat2 = A(N * H * DH, isz); dq = A(N * H * DH, isz)
        dk = A(N * KV * DH, isz); dv = A(N * KV * DH, isz)
        bD = A(N * H + (N * H * DH if hf else 0))     # row dots, then the fp32 dQ accumulator of the bf16 path
        if lora:
            # u = s * x@A of every adapted projection is kept for the backward; t = s * g@B^T lives until the
            # projection's gradient ops have run (one buffer per projection kind, reused by every layer)
            u_l = {(i, pref): A(N * lora_r, isz) for i in range(L) for pref in lin_geom
                   if pref.split(".")[-1] in lset}
            t_l = {pref: A(N * lora_r, isz) for pref in lin_geom if pref.split(".")[-1] in lset}
        G = self.gbuf

        def adapted(pref):
            return lora and pref.split(".")[-1] in lset

        def lora_proj(xs_, ws_, outs_, fs_, tb):
            """outs_[g] [N, r] = s * xs_[g] @ W_g (W_g [F, r], tb=0) or @ W_g^T (W_g [r, F], tb=1): the skinny products of up
            to three adapters as one streaming launch"""
            pad = lambda v: list(v) + [0] * (3 - len(v))
            x_, w_, o_, f_ = pad(xs_), pad(ws_), pad(outs_), pad(fs_)
            same = all(v == x_[0] for v in xs_)
            return [op(LORA_PROJ, a=x_[0], sa=0 if same else x_[1], sb=0 if same else x_[2], b=w_[0], d=w_[1], sc=w_[2],
                       c=o_[0], oa=o_[1], ob=o_[2], n=f_[0], k=f_[1], oc=f_[2], m=N, batch=len(xs_), tb=tb,
                       gamma=float(lora_r), alpha=sc_l, dt=DT)]

        def lora_grads(i, prefs, x, gs_):
            """dA_p = x^T t_p and dB_p = u_p^T g_p of the adapted projections among prefs (x shared): streams over the
            wide operands with a fixed summation order"""
            pp = [(p_, g_) for p_, g_ in zip(prefs, gs_) if adapted(p_)]
            if not pp:
                return []
            pad = lambda v: list(v) + [0] * (3 - len(v))
            ts, us_ = pad([t_l[p_] for p_, _ in pp]), pad([u_l[(i, p_)] for p_, _ in pp])
            gg = pad([g_ for _, g_ in pp])
            offa = pad([self._off[f"blocks.{i}.{p_}.lora_a"] for p_, _ in pp])
            offb = pad([self._off[f"blocks.{i}.{p_}.lora_b"] for p_, _ in pp])
            fin = lin_geom[pp[0][0]][0]
            fo = pad([lin_geom[p_][1] for p_, _ in pp])
            # batch < 0: only noted here; one launch at the end of the layer's backward runs the layer's whole set
            return [op(LORA_GRAD, a=x, b=ts[0], d=ts[1], sc=ts[2], c=self.a_grad, oa=offa[0], ob=offa[1], oc=offa[2],
                       n=fin, k=fin, tb=fin, m=N, batch=-len(pp), gamma=float(lora_r), dt=DT),
                    op(LORA_GRAD, a=gg[0], sa=gg[1], sb=gg[2], b=us_[0], d=us_[1], sc=us_[2], c=self.a_grad,
                       oa=offb[0], ob=offb[1], oc=offb[2], n=fo[0], k=fo[1], tb=fo[2], m=N, batch=-len(pp),
                       gamma=float(lora_r), beta=1.0, dt=DT)]

        def lin_f(x, i, pref, y, res=-1):
            """y = x@W (+ res) (+ u@B with u = s * x@A saved: the adapter's term is a K-segment of the same launch)"""
            fin, fout = lin_geom[pref]
            key = f"blocks.{i}.{pref}"
            if adapted(pref):
                u = u_l[(i, pref)]
                return lora_proj([x], [P[key + ".lora_a"]], [u], [fin], 0) + [
                        op(GEMM_XSEG, a=u, sa=P[key + ".lora_b"], k=lora_r, batch=1, c=(res if res >= 0 else 0), beta=1.0),
                        op(GEMM_GROUP, a=x, b=P[key + ".weight"], c=y, m=N, k=fin, n=fout, batch=1, oc=2, dt=DT)]
            if res >= 0:
                return [op(GEMM_EX, a=x, b=P[key + ".weight"], c=y, d=res, m=N, k=fin, n=fout, batch=1, dt=DT, beta=1.0)]
            return [op(GEMM_SB, a=x, b=P[key + ".weight"], c=y, m=N, k=fin, n=fout, batch=1, dt=DT)]

        # ── weight-gradient GEMMs on a side stream ──
        # The dW GEMMs of a block feed nothing until the optimizer (or the bucket's reduction), so they are
        # queued on a side stream and fill the SMs that the main chain's kernels leave idle (partial last
        # waves of the dX GEMMs and of the attention backward).  Dependencies are explicit events: the side
        # stream waits for the main chain before each group (its inputs were just produced there), and the main
        # chain waits for the side stream's last reader of a gradient buffer before it overwrites that buffer.
        # Not used with adapters (their gradients chain through shared scratch) nor with per-block recompute
        # (the shared activation set is rewritten while a side GEMM could still read it).
        side_dw = bool(overlap_dw) and not lora and not rc
        self.overlap_dw = side_dw
        ev = [0]                              # last event id handed out
        side_reads: Dict[int, int] = {}       # gradient buffer -> event after its last side-stream reader

        def on_side(ops_, reads):
            if not side_dw or not ops_:
                return ops_
            e_in, e_out = ev[0] + 1, ev[0] + 2
            ev[0] = e_out
            for b_ in reads:
                side_reads[b_] = e_out
            return [op(EVENT, tb=1, sa=0, oa=e_in), op(EVENT, tb=2, sa=2, oa=e_in), op(STREAM, tb=2)] + ops_ + \
                   [op(EVENT, tb=1, sa=2, oa=e_out), op(STREAM, tb=0)]

        def before_write(*bufs):
            """main chain: wait until the side stream has finished reading the buffers about to be rewritten"""
            es = [side_reads.pop(b_) for b_ in bufs if b_ in side_reads]
            if not es:
                return []
            e = max(es)                        # the side stream runs in order: later events imply earlier ones
            for b_ in [b_ for b_, v in side_reads.items() if v <= e]:
                del side_reads[b_]
            return [op(EVENT, tb=2, sa=0, oa=e)]

        def lin_b(g, x, i, pref, dx, dw=True):
            """dx = g@W^T (+ t@A^T with t = s * g@B^T); weight grads: dW (dw=False leaves it to a later grouped launch),
            or the adapter's dA / dB"""
            fin, fout = lin_geom[pref]
            key = f"blocks.{i}.{pref}"
            if adapted(pref):
                t = t_l[pref]
                return lora_proj([g], [P[key + ".lora_b"]], [t], [fout], 1) + [
                        op(GEMM_XSEG, a=t, sa=P[key + ".lora_a"], k=lora_r, batch=1),
                        op(GEMM_GROUP, a=g, b=P[key + ".weight"], c=dx, m=N, k=fout, n=fin, batch=1, oc=2, tb=1, dt=DT)] + \
                    lora_grads(i, (pref,), x, (g,))
            o_ = [op(GEMM_SB, a=g, b=P[key + ".weight"], c=dx, m=N, k=fout, n=fin, batch=1, tb=1, dt=DT)]
            if not lora and dw:
                o_ += on_side([op(GEMM_SB, a=x, b=g, c=G[key + ".weight"], m=fin, n=fout, k=N, batch=1, tb=2, dt=DTW)], [g])
            return o_

        def lin_f_group(x, i, prefs, ys_, rope=False, adapters=True):
            """ys_[g] = x@W_g for projections that share their input: one grouped launch.  With adapters on all of
            them a second grouped launch computes the u_g = s * x@A_g first and every output takes its u_g@B_g as a
            K-segment of its own.  rope: the first two outputs (query and key projections) leave the launch with the
            rotary embedding applied"""
            fin = lin_geom[prefs[0]][0]
            fo = [lin_geom[p][1] for p in prefs] + [0]
            w = [P[f"blocks.{i}.{p}.weight"] for p in prefs] + [0]
            yy = list(ys_) + [0]
            o_ = []
            if adapters and adapted(prefs[0]):  # the caller passes projections that are all adapted or all plain
                la = [P[f"blocks.{i}.{p}.lora_a"] for p in prefs] + [0]
                lb = [P[f"blocks.{i}.{p}.lora_b"] for p in prefs] + [0]
                uu = [u_l[(i, p)] for p in prefs] + [0]
                o_ += lora_proj([x] * len(prefs), la[:len(prefs)], uu[:len(prefs)], [fin] * len(prefs), 0)
                o_ += [op(GEMM_XSEG, a=uu[0], b=uu[1], d=uu[2], sa=lb[0], sb=lb[1], sc=lb[2], k=lora_r, batch=len(prefs))]
            o_ += [op(GEMM_GROUP, a=x, b=w[0], sa=w[1], sb=w[2], c=yy[0], d=yy[1], sc=yy[2], m=N, k=fin,
                      n=fo[0], oa=fo[1], ob=fo[2], batch=len(prefs), oc=1, dt=DT,
                      beta=float(b_cos) if rope else 0.0, gamma=float(b_sin) if rope else 0.0)]
            return o_

        def lin_b_group(gs_, x, i, prefs, dx):
            """dx = sum_g gs_[g]@W_g^T in one launch (with adapters: + sum_g t_g@A_g^T as further K-segments of it, the
            t_g = s * gs_[g]@B_g^T computed first); weight grads of all g in one launch, or the adapters' dA / dB"""
            fin = lin_geom[prefs[0]][0]
            fo = [lin_geom[p][1] for p in prefs] + [0]
            keys = [f"blocks.{i}.{p}" for p in prefs]
            w = [P[k_ + ".weight"] for k_ in keys] + [0]
            gg = list(gs_) + [0]
            o_ = []
            ad = [q for q, p in enumerate(prefs) if adapted(p)]
            if ad:
                pad = lambda v: list(v) + [0] * (3 - len(v))
                tt = [t_l[p] if adapted(p) else 0 for p in prefs]
                lb = [P[k_ + ".lora_b"] if adapted(p) else 0 for p, k_ in zip(prefs, keys)]
                o_ += lora_proj([gg[q] for q in ad], [lb[q] for q in ad], [tt[q] for q in ad], [fo[q] for q in ad], 1)
                xa, xb = pad([tt[q] for q in ad]), pad([P[keys[q] + ".lora_a"] for q in ad])
                o_ += [op(GEMM_XSEG, a=xa[0], b=xa[1], d=xa[2], sa=xb[0], sb=xb[1], sc=xb[2], k=lora_r, batch=len(ad))]
            o_ += [op(GEMM_GROUP, c=dx, a=gg[0], sa=gg[1], sb=gg[2], b=w[0], d=w[1], sc=w[2], m=N, n=fin,
                      k=fo[0], oa=fo[1], ob=fo[2], batch=len(prefs), oc=2, tb=1, dt=DT)]
            if not lora:
                gw = [G[k_ + ".weight"] for k_ in keys] + [0]
                o_ += on_side([op(GEMM_GROUP, a=x, b=gg[0], sa=gg[1], sb=gg[2], c=gw[0], d=gw[1], sc=gw[2], m=fin, k=N,
                                  n=fo[0], oa=fo[1], ob=fo[2], batch=len(prefs), oc=1, tb=2, dt=DTW)], list(gs_))
            else:
                o_ += lora_grads(i, prefs, x, gs_)
            return o_

        def lin_f_mixed(x, i, prefs, ys_):
            """projections of one input of which only some carry an adapter: the grouped base launch, then every
            adapter's two products one by one"""
            o_ = lin_f_group(x, i, prefs, ys_, adapters=False)
            for p_, y_ in zip(prefs, ys_):
                if adapted(p_):
                    fin, fout = lin_geom[p_]
                    key, u = f"blocks.{i}.{p_}", u_l[(i, p_)]
                    o_ += lora_proj([x], [P[key + ".lora_a"]], [u], [fin], 0)
                    o_ += [op(GEMM_SB, a=u, b=P[key + ".lora_b"], c=y_, m=N, k=lora_r, n=fout, batch=1, dt=DT, beta=1.0)]
            return o_

        def lin_group_ok(prefs):
            """projections that share an input run as one group when all of them, or none, carry an adapter"""
            return len({adapted(p) for p in prefs}) == 1

        def norm_b(x, wname, g, res, out):
            """out = res + rmsnorm_bwd(x, w, g); dw -> G[wname] unless frozen"""
            if lora:
                return [op(RMSNORM_BWD_ACC, a=x, b=P[wname], d=g, c=out, tb=(res if res >= 0 else 0), sa=0,
                           sb=self.b_rb_scratch, m=N, n=D, dt=DT, alpha=eps)]
            rb_pending.append(len(rb_names))
            rb_names.append(wname)
            return [op(RMSNORM_BWD_ACC, a=x, b=P[wname], d=g, c=out, tb=(res if res >= 0 else 0),
                       sa=G[wname], sb=self.b_rb_scratch, oa=len(rb_names), m=N, n=D, dt=DT, alpha=eps)]

        def flush_dw():
            """weight gradients of the norms whose backward ran since the last flush"""
            if not rb_pending:
                return []
            o_ = [op(COLSUM_BATCH, a=self.b_rb_scratch, b=self.b_rb_table, c=self.a_grad, m=len(rb_pending), n=D,
                     oa=rb_pending[0], k=CHUNK)]
            rb_pending.clear()
            return o_

        # ── forward ──
        def block_f(i, down=True):
            """forward of block i from xs[i]; down=False stops before the down projection (all that the
            backward of the block reads is then in place)"""
            plan = []
            p = f"blocks.{i}."
            plan += [op(RMSNORM, a=xs[i], b=P[p + "attn_norm.weight"], c=ys[i], m=N, n=D, dt=DT, alpha=eps)]
            # rotary of q and k: in the epilogue of the projection launch (head_dim 64; an adapter's term is part of
            # the same accumulator, so it is rotated with it), else one launch over both, in place
            qkv = ("attn.q_proj", "attn.k_proj", "attn.v_proj")
            fuse_rope = DH == 64 and lin_group_ok(qkv)
            if lin_group_ok(qkv):
                plan += lin_f_group(ys[i], i, qkv, (q2s[i], k2s[i], vs[i]), rope=fuse_rope)
            else:
                plan += lin_f_mixed(ys[i], i, qkv, (q2s[i], k2s[i], vs[i]))
            if not fuse_rope:
                plan += [op(ROPE_BTHD, a=q2s[i], b=b_cos, d=b_sin, c=q2s[i], batch=B, m=T, k=H, n=DH, dt=DT,
                            sa=k2s[i], sb=k2s[i], sc=KV)]
            plan += [op(ATTN_FWD, a=q2s[i], b=k2s[i], d=vs[i], c=at2s[i], sa=lses[i],
                        m=T, n=DH, k=KV, batch=B, tb=H, dt=DT, alpha=scale)]
            plan += lin_f(at2s[i], i, "attn.o_proj", r1s[i], res=xs[i])
            plan += [op(RMSNORM, a=r1s[i], b=P[p + "mlp_norm.weight"], c=zs[i], m=N, n=D, dt=DT, alpha=eps)]
            gu = ("mlp.gate_proj", "mlp.up_proj")
            if adapted(gu[0]) or adapted(gu[1]):
                plan += lin_f_group(zs[i], i, gu, (gs[i], us[i])) if lin_group_ok(gu) else lin_f_mixed(zs[i], i, gu, (gs[i], us[i]))
                plan += [op(SILU_MUL, a=gs[i], b=us[i], c=hs[i], n=N * MLP, dt=DT)]
            else:   # gate and up projections with the activation in the epilogue: g, u and h = silu(g)*u in one launch
                plan += [op(GEMM_GROUP, a=zs[i], b=P[p + "mlp.gate_proj.weight"], sa=P[p + "mlp.up_proj.weight"],
                            c=gs[i], d=us[i], sc=hs[i], m=N, n=MLP, k=D, batch=2, oc=4, dt=DT)]
            if down:
                plan += lin_f(hs[i], i, "mlp.down_proj", xs[i + 1], res=r1s[i])
            return plan

        # ZeRO-1: the owners' bf16 segments are broadcast at the START of the step, bucket by bucket in forward
        # order on the collectives stream, and the forward waits for a bucket's event just before its first use —
        # the gather of the weights that the previous step's AdamW wrote overlaps the forward instead of ending
        # that step on the main stream.  (The first step broadcasts the initial weights: a no-op in value.)
        EV_W = 1 << 14                         # event ids of the weight buckets (the side-stream ids stay below)
        self._w_events = zero and not lora

        def wait_weights(b):
            return [op(EVENT, tb=2, sa=0, oa=EV_W + b)] if self._w_events else []
        plan = wait_weights(nb - 1) + [op(EMBED_I32, a=P["embed.weight"], b=self.b_ids, c=xs[0], m=N, n=D, dt=DT)]
        for i in range(L):
            if i == 0 or bucket_of(f"blocks.{i}.x") != bucket_of(f"blocks.{i - 1}.x"):
                plan += wait_weights(bucket_of(f"blocks.{i}.x"))
            plan += block_f(i)

        # ── head + loss ──
        lm_w = P["embed.weight"] if tied else P["lm_head.weight"]
        plan += wait_weights(0)
        plan += [
            op(RMSNORM, a=xs[L], b=P["norm.weight"], c=xf, m=N, n=D, dt=DT, alpha=eps),
            op(GEMM_SB, a=xf, b=lm_w, c=logits, m=N, k=D, n=V, batch=1, tb=(1 if tied else 0), dt=DT),
            op(CE_FUSED, a=logits, b=self.b_tgt, c=logits, d=self.b_loss, sa=self.b_denom,
               sb=self.b_ce_scratch, m=N, n=V, dt=DT),
        ]
        dlogits = logits
        self._b_logits = logits

        # ── backward ──
        bucket_done: List[int] = []          # plan index after which bucket b is complete
        if tied:
            plan += [op(GEMM_SB, a=dlogits, b=lm_w, c=dxf, m=N, k=V, n=D, batch=1, tb=0, dt=DT)]
            if not lora:
                plan += [op(GEMM_SB, a=dlogits, b=xf, c=G["embed.weight"], m=V, n=D, k=N, batch=1, tb=2, dt=DTW)]
        else:
            plan += [op(GEMM_SB, a=dlogits, b=lm_w, c=dxf, m=N, k=V, n=D, batch=1, tb=1, dt=DT)]
            if not lora:
                plan += [op(GEMM_SB, a=xf, b=dlogits, c=G["lm_head.weight"], m=D, n=V, k=N, batch=1, tb=2, dt=DTW)]
        plan += norm_b(xs[L], "norm.weight", dxf, -1, dcur)
        plan += flush_dw()
        marks = {0: len(plan)}
        mark_ev = {0: 0}                      # last side-stream event a bucket's gradients depend on
        for i in reversed(range(L)):
            p = f"blocks.{i}."
            if rc and i < L - 1:      # the last block's activations are still in place after the forward
                plan += block_f(i, down=False)
            plan += lin_b(dcur, hs[i], i, "mlp.down_proj", dh_)
            plan += before_write(dg_, du_)
            plan += [op(SILU_BWD, a=gs[i], b=us[i], d=dh_, c=dg_, tb=du_, n=N * MLP, dt=DT)]
            plan += lin_b_group((dg_, du_), zs[i], i, ("mlp.gate_proj", "mlp.up_proj"), dz)
            plan += before_write(dr1)
            plan += norm_b(r1s[i], p + "mlp_norm.weight", dz, dcur, dr1)
            plan += lin_b(dr1, at2s[i], i, "attn.o_proj", dat2)
            plan += before_write(dq, dk, dv)
            # the inverse rotary of dq and dk is part of the op (beta / gamma name the cos / sin tables): the
            # tensor-core backward applies it before it rounds to bf16, other paths run the rotary kernel behind it
            plan += [
                op(ATTN_BWD, a=q2s[i], b=k2s[i], d=vs[i], c=dat2, sa=lses[i], sb=at2s[i],
                   tb=dq, sc=dk, oa=dv, ob=H, oc=bD, m=T, n=DH, k=KV, batch=B, dt=DT, alpha=scale,
                   beta=float(b_cos), gamma=float(b_sin)),
            ]
            plan += lin_b_group((dq, dk, dv), ys[i], i, ("attn.q_proj", "attn.k_proj", "attn.v_proj"), dy)
            if lora:
                # every operand of the layer's adapter gradients is still in place (the incoming gradient dcur is
                # overwritten by the next op): all of them as one launch
                plan += [op(LORA_GRAD, batch=0)]
            plan += before_write(dcur)
            plan += norm_b(xs[i], p + "attn_norm.weight", dy, dr1, dcur)
            if (L - 1 - i) in bucket_end:
                plan += flush_dw()
                marks[pos_bucket[L - 1 - i]] = len(plan)
                mark_ev[pos_bucket[L - 1 - i]] = ev[0]
        if not lora:
            if not tied:
                plan += [op(SCALE, a=G["embed.weight"], c=G["embed.weight"], n=V * D, alpha=0.0)]
            plan += [op(EMBED_BWD_DET, a=dcur, b=self.b_ids, c=G["embed.weight"], m=N, n=D, dt=DT)]
        plan += flush_dw()
        marks[nb - 1] = len(plan)
        mark_ev[nb - 1] = ev[0]
        if ev[0]:                             # the main chain ends after the last side-stream GEMM
            plan += [op(EVENT, tb=2, sa=0, oa=ev[0])]
        self.plan_fb = plan
        if rb_names:
            eng.upload_raw(self.b_rb_table, np.array([self._off[nm] // CHUNK for nm in rb_names], dtype=np.int32))

        # ── gradient reduction: bucketed, on the side stream, overlapped with backward ──
        def comm_ops(b):
            red = [op(REDUCE, a=self.a_grad, m=ln // CHUNK, oa=st // CHUNK, tb=r)
                   for r in range(cw) for (st, ln) in [self._groups[r][b]] if ln > 0]
            if not red:
                return []
            dep = mark_ev.get(b, 0)          # the bucket's weight gradients come from the side stream
            out = [op(FORK)] + ([op(EVENT, tb=2, sa=1, oa=dep)] if dep else []) + \
                  [op(STREAM, tb=1), op(GROUP, tb=0)] + red + [op(GROUP, tb=1)]
            if not zero:     # replicated: everyone gets the reduced gradients back
                out += [op(GROUP, tb=0)] + [op(BROADCAST, a=self.a_grad, m=o[5], oa=o[14], tb=o[9]) for o in red] \
                    + [op(GROUP, tb=1)]
            return out + [op(STREAM, tb=0)]
        self.plan_ar = []
        if self.grad_sync:
            merged, last = [], 0
            for b in range(nb):
                cut = marks.get(b, last)
                merged += plan[last:cut] + comm_ops(b)
                last = cut
            merged += plan[last:] + [op(JOIN)]
            self._plan_fb_sync = merged
            self.plan_ar = [o for b in range(nb) for o in comm_ops(b)] + [op(JOIN)]
        else:
            self._plan_fb_sync = plan

        # ── clip + AdamW over the arena ──
        def opt_ops(max_norm):
            ops_ = []
            if zero:
                s0, sl = my_seg
                ops_ += [op(GNORM_FLAT, a=self.a_grad, c=self.b_partials, d=self.b_sumsq_local, ob=0,
                            m=sl // CHUNK, oa=s0 // CHUNK, tb=self.b_t),
                         op(ALLGATHER_F32, a=self.b_sumsq_local, c=self.b_sumsq, n=1)]
            else:
                for r in range(cw):
                    s0, sl = self._seg[r]
                    ops_ += [op(GNORM_FLAT, a=self.a_grad, c=self.b_partials, d=self.b_sumsq, ob=r,
                                m=sl // CHUNK, oa=s0 // CHUNK, tb=(self.b_t if r == 0 else 0))]
            s0, sl = my_seg
            ops_ += [op(ADAMW_FLAT, a=self.a_master, b=self.a_grad, c=self.a_m, d=self.a_v,
                        m=sl // CHUNK, k=s0 // CHUNK, sa=(self.a_mirror if hf else 0), sb=self.b_lr,
                        tb=self.b_t, sc=self.b_wdflag, oa=self.b_sumsq, ob=cw, oc=self.b_gnorm,
                        alpha=float(max_norm or 0.0), beta=self.wd, gamma=adam_eps)]
            if zero and not self._w_events:
                ops_ += self._mirror_bcast_ops()
            return ops_
        self._opt_ops = opt_ops

        def gather_ops():
            """mirror broadcasts of every bucket in forward order on the collectives stream, one event each"""
            if not self._w_events:
                return []
            out = [op(FORK), op(STREAM, tb=1)]
            for b in reversed(range(nb)):
                segs = [(r, self._groups[r][b]) for r in range(cw) if self._groups[r][b][1] > 0]
                if segs:
                    out += [op(GROUP, tb=0)] + [op(BROADCAST, a=self.a_mirror, m=ln // CHUNK, oa=st // CHUNK, tb=r, dt=1)
                                                for r, (st, ln) in segs] + [op(GROUP, tb=1)]
                out += [op(EVENT, tb=1, sa=1, oa=EV_W + b)]
            return out + [op(STREAM, tb=0)]
        self._gather_ops = gather_ops

        # One GPU: the squared norm of a bucket's gradients is taken as soon as the bucket is complete and AdamW sums
        # the per-bucket figures in bucket order.  With the weight gradients on the side stream the norms run there too
        # (behind the bucket's dW GEMMs, which that stream runs in order, and behind an event for what the main chain
        # contributes: norm weight gradients, the embedding scatter), so the pass over the gradient arena that the clip
        # needs runs under the backward instead of between it and AdamW.  The inline plan takes the same per-bucket
        # sums on the main chain, so both plans add the same numbers in the same order.
        def plan_with_bucket_norms():
            merged, last, e = [], 0, ev[0]
            for b in range(nb):
                cut = marks.get(b, last)
                merged += plan[last:cut]
                last = cut
                st, ln = self._groups[0][b]
                gn = op(GNORM_FLAT, a=self.a_grad, c=self.b_partials, d=self.b_sumsq, ob=b, m=ln // CHUNK,
                        oa=st // CHUNK, tb=(self.b_t if b == 0 else 0))
                if side_dw:
                    e += 2
                    merged += [op(EVENT, tb=1, sa=0, oa=e - 1), op(EVENT, tb=2, sa=2, oa=e - 1), op(STREAM, tb=2), gn,
                               op(EVENT, tb=1, sa=2, oa=e), op(STREAM, tb=0)]
                else:
                    merged += [gn]
            merged += plan[last:] + ([op(EVENT, tb=2, sa=0, oa=e)] if side_dw else [])
            s0, sl = my_seg
            return merged + [op(ADAMW_FLAT, a=self.a_master, b=self.a_grad, c=self.a_m, d=self.a_v,
                                m=sl // CHUNK, k=s0 // CHUNK, sa=(self.a_mirror if hf else 0), sb=self.b_lr,
                                tb=self.b_t, sc=self.b_wdflag, oa=self.b_sumsq, ob=nb, oc=self.b_gnorm,
                                alpha=float(max_grad_norm or 0.0), beta=self.wd, gamma=adam_eps)]
        self.bucket_norms = bool(cw == 1 and not zero and nb <= 64 and all(self._groups[0][b][1] > 0 for b in range(nb)))
        if self.bucket_norms:
            self.plan_step = plan_with_bucket_norms()
        else:
            self.plan_step = gather_ops() + self._plan_fb_sync + opt_ops(max_grad_norm)
        self._plan_noclip = None
        self._captured = False
        self._pending_loss = None            # read-back ticket of the last replay_step_async

    def _mirror_bcast_ops(self):
        """ZeRO-1: every owner broadcasts its segment of the bf16 mirror (one grouped launch)."""
        return [op(GROUP, tb=0)] + \
            [op(BROADCAST, a=self.a_mirror, m=ln // CHUNK, oa=st // CHUNK, tb=r, dt=1)
             for r, (st, ln) in enumerate(self._seg) if ln > 0] + [op(GROUP, tb=1)]

    def _cast_segment(self):
        """fp32 masters of this rank's segment -> its bf16 mirror segment (padding is zero on both sides).
        The count goes in as chunks x CHUNK (CAST converts m*n elements): a 7B-class segment has more
        elements than a 32-bit field holds.  The reference casts tensor by tensor (axis/compile.py:192-200)."""
        s0, sl = self._my_seg
        if not hasattr(self, "_mirror_seg"):
            self._mirror_seg = self.eng.view(self.a_mirror, s0 * 2, sl * 2)
        return [op(CAST, a=self.a_master, c=self._mirror_seg, m=sl // CHUNK, n=CHUNK, tb=0)]

    # ── API (axis/compile.py:547-615) ──
    def set_lr(self, lr: float) -> None:
        """Learning rate for subsequent steps; lives in a device buffer, so it
        also takes effect under CUDA-graph replay."""
        self.lr = float(lr)
        self.eng.upload(self.b_lr, np.array([lr], dtype=np.float32))

    def _feed(self, tokens: np.ndarray, targets: np.ndarray) -> None:
        if tokens.size != self.N or targets.size != self.N:
            raise ValueError(f"expected {self.B}x{self.T} tokens and targets")
        self.eng.upload_tokens(self.b_ids, np.where(np.asarray(tokens) < 0, self.V, tokens), self.V)
        self.eng.upload_tokens(self.b_tgt, np.maximum(np.asarray(targets), -1), self.V)

    def step(self, tokens: np.ndarray, targets: np.ndarray, t: int = None) -> float:
        self._feed(tokens, targets)
        if t is None:
            self.eng.run(self.plan_step, sync=False)
        else:
            # parity path: bias correction for step t, no clipping
            if self._plan_noclip is None:
                self._plan_noclip = self._gather_ops() + self._plan_fb_sync + self._opt_ops(0.0)
            self.eng.upload(self.b_t, np.array([t - 1], dtype=np.float32))
            self.eng.run(self._plan_noclip, sync=False)
        return float(self.eng.download(self.b_loss, (1,))[0])

    def capture(self, t: int = None) -> None:
        if t is None:
            self.eng.capture(self.plan_step)
        else:
            if self._plan_noclip is None:
                self._plan_noclip = self._gather_ops() + self._plan_fb_sync + self._opt_ops(0.0)
            self.eng.upload(self.b_t, np.array([t - 1], dtype=np.float32))
            self.eng.capture(self._plan_noclip)
        self._captured = True

    def replay_step(self, tokens: np.ndarray, targets: np.ndarray) -> float:
        self._feed(tokens, targets)
        self.eng.replay(1, sync=False)
        return float(self.eng.download(self.b_loss, (1,))[0])

    def replay_step_async(self, tokens: np.ndarray, targets: np.ndarray):
        """Launch one captured step and return the loss of the step launched BEFORE it (None on the first
        call): the host never waits for the step it has just queued, so batch preparation for step i+1
        overlaps step i on the GPU.  Token conversion goes through the engine's pinned ring and the loss
        comes back through a pinned read-back ring.  `flush()` collects the last loss."""
        self._feed(tokens, targets)
        self.eng.replay(1, sync=False)
        tk = self.eng.download_async(self.b_loss, 1)
        prev, self._pending_loss = self._pending_loss, tk
        return None if prev is None else float(self.eng.download_wait(prev, 1)[0])

    def flush(self):
        """Loss of the last step queued with replay_step_async (None if there is none); waits for it."""
        prev, self._pending_loss = self._pending_loss, None
        return None if prev is None else float(self.eng.download_wait(prev, 1)[0])

    def step_accumulate(self, batches) -> float:
        """One optimizer step over several micro-batches of the compiled shape (gradient accumulation).

        The gradient applied is the mean of the micro-batch gradients, each normalised by its own count of
        valid targets — with micro-batches of equal valid counts this is the gradient of the concatenated
        batch (the equivalence the reference checks in tests/test_generate_accum.py:51); the returned loss is
        the mean of the micro-batch losses.  Under data parallelism the averaged gradient is reduced once, after
        the last micro-batch.  Costs one extra fp32 arena of the gradients' size."""
        batches = list(batches)
        n = len(batches)
        if n < 1:
            raise ValueError("no micro-batches")
        if not hasattr(self, "_acc_plans"):
            self.a_gacc = self.eng.alloc_zero(self._P_total * 4)
            lim = 1 << 30                     # element counts of flat ops stay inside int32

            def flat(kind, **kw):
                out = []
                for o in range(0, self._P_total, lim):
                    ln = min(lim, self._P_total - o)
                    v = {k_: (self.eng.view(b_, o * 4, ln * 4) if o or ln < self._P_total else b_) for k_, b_ in kw["bufs"].items()}
                    out.append(op(kind, n=ln, dt=0, alpha=kw.get("alpha", 0.0), **v))
                return out
            self._acc_flat = flat
            self._acc_plans = {}
        if n not in self._acc_plans:
            inv = 1.0 / n
            first = self._gather_ops() + self.plan_fb + self._acc_flat(SCALE, bufs=dict(a=self.a_grad, c=self.a_gacc), alpha=inv)
            nxt = self.plan_fb + self._acc_flat(SCALE, bufs=dict(a=self.a_grad, c=self.a_grad), alpha=inv) \
                + self._acc_flat(ADD, bufs=dict(a=self.a_gacc, b=self.a_grad, c=self.a_gacc))
            last = self._acc_flat(COPY, bufs=dict(a=self.a_gacc, c=self.a_grad)) + self.plan_ar \
                + self._opt_ops(self.max_grad_norm)
            self._acc_plans[n] = (first, nxt, last)
        first, nxt, last = self._acc_plans[n]
        total = 0.0
        for i, (x, y) in enumerate(batches):
            self._feed(x, y)
            self.eng.run(first if i == 0 else nxt, sync=False)
            total += float(self.eng.download(self.b_loss, (1,))[0])
        self.eng.run(last, sync=False)
        return total / n

    def forward_backward(self, tokens: np.ndarray, targets: np.ndarray) -> float:
        """Forward + backward only (no reduction, no update); for gradient checks."""
        self._feed(tokens, targets)
        if self._w_events and not hasattr(self, "_plan_fb_gather"):
            self._plan_fb_gather = self._gather_ops() + self.plan_fb + [op(JOIN)]
        self.eng.run(self._plan_fb_gather if self._w_events else self.plan_fb, sync=False)
        return float(self.eng.download(self.b_loss, (1,))[0])

    def gather_weights(self) -> None:
        """ZeRO-1: bring every rank's bf16 compute copy up to date with the owners' last update now.  A step does
        this by itself at its start (overlapped with its forward); call it before reading the compute weights of
        tensors this rank does not own outside a step.  Collective: every rank calls it.  No-op otherwise."""
        if self._w_events:
            self.eng.run(self._gather_ops() + [op(JOIN)], sync=True)

    def grad_norm(self) -> float:
        """Global gradient norm seen by the last optimizer step (before clipping)."""
        return float(self.eng.download(self.b_gnorm, (1,))[0])

    def valid_count(self) -> int:
        """Number of non-ignored targets in the last batch (exact integer)."""
        return int(self.eng.download(self.b_denom, (1,))[0])

    def grads(self) -> Dict[str, np.ndarray]:
        return {nm: self.eng.download(self.gbuf[nm], self.shapes[nm]) for nm in self.pnames}

    def get_weights(self) -> Dict[str, np.ndarray]:
        """Current fp32 master weights; under ZeRO only this rank's owned shard."""
        return {nm: self.eng.download(self.master[nm], self.shapes[nm]) for nm in self.owned}

    def state_dict(self) -> Dict[str, np.ndarray]:
        st = {}
        for nm in self.owned:
            sh = self.shapes[nm]
            st[f"w/{nm}"] = self.eng.download(self.master[nm], sh)
            st[f"m/{nm}"] = self.eng.download(self._mb[nm], sh)
            st[f"v/{nm}"] = self.eng.download(self._vb[nm], sh)
        st["_t"] = self.eng.download(self.b_t, (1,))
        st["_lr"] = np.array([self.lr], dtype=np.float32)
        return st

    def load_state_dict(self, st: Dict[str, np.ndarray]) -> None:
        for nm in self.owned:
            self.eng.upload(self.master[nm], np.asarray(st[f"w/{nm}"]).reshape(-1))
            self.eng.upload(self._mb[nm], np.asarray(st[f"m/{nm}"]).reshape(-1))
            self.eng.upload(self._vb[nm], np.asarray(st[f"v/{nm}"]).reshape(-1))
        if self.dtype == "bf16" and self._my_seg[1] > 0:
            self.eng.run(self._cast_segment())
        if self.zero:
            # the other ranks' segments of the bf16 mirror still hold the weights this object was built with:
            # every owner publishes its freshly cast segment, so the first step after a resume computes from the
            # restored weights everywhere (collective: every rank calls load_state_dict)
            self.eng.run(self._mirror_bcast_ops())
        self.eng.upload(self.b_t, np.asarray(st["_t"], dtype=np.float32).reshape(-1))
        self.set_lr(float(np.asarray(st["_lr"]).reshape(-1)[0]))


def compile_model(model, batch: int, seq: int, lib_path: str = None,
                  lr: float = 3e-4, wd: float = 0.1, tf32: bool = True,
                  recompute_attn: bool = True, dtype: str = "fp32",
                  attn_tile: int = 256, attn_impl: str = "auto",
                  grad_sync: bool = False, max_grad_norm: float = 0.0,
                  zero_stage: int = 0, rank: int = 0, world: int = 1,
                  recompute_blocks: bool = False, overlap_dw: bool = True) -> CompiledTransformer:
    """Compile a Transformer into a native training step (axis/compile.py:618-664).

    `model` is anything shaped like the reference's `axis.nn.Transformer`:
    `named_parameters()` yielding (name, obj-with-.data), `blocks` (with
    `.attn.n_heads / .attn.n_kv_heads`), `tie_embeddings`.  LoRA-wrapped models
    are detected from parameter names (`...lora_a` / `...lora_b`,
    `...base.weight`), the rank from the adapter shape and alpha from the
    wrapper's `scaling` attribute; base weights are then frozen.

    `recompute_blocks` (not in the reference's compiled engine, whose signature ends at `world`) trades a
    second forward of every block for activation memory: see CompiledTransformer.  `overlap_dw=False` keeps the
    weight-gradient GEMMs on the main stream.
    """
    weights = {n.replace(".base.weight", ".weight"): np.asarray(p.data)
               for n, p in model.named_parameters()}
    lora_r, lora_alpha = 0, 16.0
    a_keys = [k for k in weights if k.endswith(".lora_a")]
    if a_keys:
        lora_r = int(weights[a_keys[0]].shape[1])
        lora_alpha = float(_find_lora_scaling(model)) * lora_r
    targets = tuple(sorted({k.split(".")[-2] for k in a_keys})) if lora_r else ()
    blk = model.blocks[0]
    cfg = dict(vocab_size=weights["embed.weight"].shape[0],
               dim=weights["embed.weight"].shape[1],
               n_layers=len(model.blocks),
               n_heads=blk.attn.n_heads,
               n_kv_heads=blk.attn.n_kv_heads,
               mlp_hidden=weights["blocks.0.mlp.gate_proj.weight"].shape[1],
               tie_embeddings=model.tie_embeddings)
    return CompiledTransformer(lib_path, cfg, weights, batch, seq, lr=lr, wd=wd, tf32=tf32,
                               recompute_attn=recompute_attn, dtype=dtype, attn_tile=attn_tile,
                               attn_impl=attn_impl, lora_r=lora_r, lora_alpha=lora_alpha,
                               lora_targets=targets or ("q_proj", "k_proj", "v_proj", "o_proj"),
                               grad_sync=grad_sync, max_grad_norm=max_grad_norm,
                               zero_stage=zero_stage, rank=rank, world=world,
                               recompute_blocks=recompute_blocks, overlap_dw=overlap_dw)


def _find_lora_scaling(model) -> float:
    """alpha / rank of the first adapter module found (attribute `scaling`)."""
    stack, seen = [model], set()
    while stack:
        m = stack.pop()
        if id(m) in seen:
            continue
        seen.add(id(m))
        if hasattr(m, "lora_a") and hasattr(m, "scaling"):
            return float(m.scaling)
        for child in getattr(m, "_modules", {}).values():
            if hasattr(child, "_modules") or hasattr(child, "lora_a"):
                stack.append(child)
            else:
                try:
                    stack.extend(list(child))
                except TypeError:
                    pass
    return 1.0
