"""CPU oracle for the compiled training step (test infrastructure, NOT product code).

A plain-numpy restatement of the reference's training-step arithmetic: a
Llama-class decoder (RMSNorm, half-split RoPE, grouped-query causal attention,
SwiGLU, tied or untied head), token-mean cross-entropy with ignored targets,
global-norm clipping and decoupled AdamW, plus the LoRA adapter path.  It is
written as explicit forward/backward passes (no tape), layer by layer, so that
every intermediate the GPU engine produces has a named counterpart here.

Only tests, the smoke check and the benchmark's CPU-baseline leg may import
this module; the engine never does.

Parity status: PINNED.  `tests/golden/make_golden.py` runs the reference's own
numpy autograd (axis.nn.Transformer / axis.optim) on seeded inputs and stores
its losses, gradients and updated weights; `tests/test_oracle.py` checks this
file against those vectors (and against the live reference when its tree is
present).

Reference semantics followed (paths inside the reference project):
  embedding gather / scatter-add ........ axis/ops.py:322-333
  cross_entropy (mean over valid) ....... axis/ops.py:336-372
  silu_mul .............................. axis/ops.py:378-393
  rmsnorm ............................... axis/ops.py:396-420
  rope (half split) ..................... axis/ops.py:423-447, axis/nn.py:230-236
  fused_causal_attention ................ axis/ops.py:478-524
  attention block, grouped GQA repeat ... axis/nn.py:265-298
  SwiGLU / block / Transformer .......... axis/nn.py:301-387
  LoRA linear ........................... axis/lora.py:29-54
  AdamW, clip_grad_norm ................. axis/optim.py:19-66, 110-118
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

F32 = np.float32

LORA_GEOM = ("attn.q_proj", "attn.k_proj", "attn.v_proj", "attn.o_proj",
             "mlp.gate_proj", "mlp.up_proj", "mlp.down_proj")


# ───────────────────────── elementary pieces ──────────────────────────────

def rope_tables(T: int, head_dim: int, theta: float = 10000.0):
    """cos/sin [T, head_dim/2] in fp32 (axis/nn.py:230-236)."""
    half = head_dim // 2
    freqs = 1.0 / (theta ** (np.arange(half, dtype=F32) / half))
    ang = np.outer(np.arange(T, dtype=F32), freqs)
    return np.cos(ang).astype(F32), np.sin(ang).astype(F32)


def rmsnorm_fwd(x: np.ndarray, w: np.ndarray, eps: float):
    ms = (x * x).mean(axis=-1, keepdims=True, dtype=F32)
    inv = (ms + F32(eps)) ** F32(-0.5)
    return x * inv * w, inv


def rmsnorm_bwd(x, w, inv, g):
    """Returns dx, dw (axis/ops.py:412-416)."""
    D = x.shape[-1]
    gwx = (g * w * x).sum(axis=-1, keepdims=True, dtype=F32)
    dx = g * w * inv - x * ((inv ** 3) * (gwx / D))
    dw = (g * x * inv).reshape(-1, D).sum(axis=0, dtype=F32)
    return dx.astype(F32), dw.astype(F32)


def rope_fwd(x: np.ndarray, cos: np.ndarray, sin: np.ndarray):
    """x [B, H, T, DH]; rotates (x[..., :DH/2], x[..., DH/2:])."""
    h = x.shape[-1] // 2
    x1, x2 = x[..., :h], x[..., h:]
    c, s = cos[None, None], sin[None, None]
    return np.concatenate([x1 * c - x2 * s, x1 * s + x2 * c], axis=-1).astype(F32)


def rope_bwd(g: np.ndarray, cos: np.ndarray, sin: np.ndarray):
    h = g.shape[-1] // 2
    g1, g2 = g[..., :h], g[..., h:]
    c, s = cos[None, None], sin[None, None]
    return np.concatenate([g1 * c + g2 * s, -g1 * s + g2 * c], axis=-1).astype(F32)


def silu_mul_fwd(g, u):
    sig = 1.0 / (1.0 + np.exp(-g))
    return ((g * sig) * u).astype(F32), sig


def silu_mul_bwd(g, u, sig, grad):
    dg = grad * u * (sig * (1.0 + g * (1.0 - sig)))
    du = grad * (g * sig)
    return dg.astype(F32), du.astype(F32)


def causal_probs(q, k, scale):
    """softmax(mask(q k^T * scale)) with the additive -1e30 mask; q,k [..., T, DH]."""
    T = q.shape[-2]
    s = (q @ np.swapaxes(k, -1, -2)) * F32(scale)
    s = s + np.triu(np.full((T, T), -1e30, dtype=F32), k=1)
    s = s - s.max(axis=-1, keepdims=True)
    e = np.exp(s)
    return (e / e.sum(axis=-1, keepdims=True, dtype=F32)).astype(F32)


def attention_fwd(q, k, v, scale):
    """q [B,H,T,DH]; k,v [B,KV,T,DH] (grouped GQA: head j uses kv j // rep).
    Returns o [B,H,T,DH] and the natural-log LSE [B,H,T] of the scaled scores."""
    B, H, T, DH = q.shape
    KV = k.shape[1]
    rep = H // KV
    o = np.empty_like(q)
    lse = np.empty((B, H, T), dtype=F32)
    mask = np.triu(np.full((T, T), -1e30, dtype=F32), k=1)
    for b in range(B):
        for h in range(H):
            g = h // rep
            s = (q[b, h] @ k[b, g].T) * F32(scale) + mask
            m = s.max(axis=-1, keepdims=True)
            e = np.exp(s - m)
            l = e.sum(axis=-1, keepdims=True, dtype=F32)
            o[b, h] = (e / l) @ v[b, g]
            lse[b, h] = (m + np.log(l))[:, 0]
    return o.astype(F32), lse


def attention_bwd(q, k, v, do, scale):
    """Gradients of causal GQA attention (axis/ops.py:507-521 applied per
    query head, with dK/dV summed over each kv group as the grouped repeat's
    backward does, axis/nn.py:280-292).  Shapes as attention_fwd."""
    B, H, T, DH = q.shape
    KV = k.shape[1]
    rep = H // KV
    dq = np.zeros_like(q)
    dk = np.zeros_like(k)
    dv = np.zeros_like(v)
    for b in range(B):
        for h in range(H):
            g = h // rep
            p = causal_probs(q[b, h], k[b, g], scale)
            dv[b, g] += p.T @ do[b, h]
            dp = do[b, h] @ v[b, g].T
            ds = p * (dp - (dp * p).sum(axis=-1, keepdims=True))
            dq[b, h] = (ds @ k[b, g]) * F32(scale)
            dk[b, g] += (ds.T @ q[b, h]) * F32(scale)
    return dq.astype(F32), dk.astype(F32), dv.astype(F32)


def cross_entropy_fwd_bwd(logits: np.ndarray, targets: np.ndarray, ignore_index: int = -1):
    """Mean NLL over targets != ignore_index and d(loss)/d(logits).
    Raises ValueError when nothing is valid (axis/ops.py:345-348)."""
    t = np.asarray(targets).astype(np.int64).reshape(-1)
    x = logits.reshape(-1, logits.shape[-1]).astype(F32)
    valid = t != ignore_index
    n_valid = int(valid.sum())
    if n_valid == 0:
        raise ValueError("cross_entropy: no valid targets")
    sh = x - x.max(axis=-1, keepdims=True)
    lse = np.log(np.exp(sh).sum(axis=-1, keepdims=True))
    logp = sh - lse
    rows = np.arange(x.shape[0])
    safe = np.where(valid, t, 0)
    nll = np.where(valid, -logp[rows, safe], 0.0)
    loss = F32(float(nll.sum()) / n_valid)
    p = np.exp(logp)
    p[rows, safe] -= 1.0
    p *= (valid[:, None] / n_valid)
    return loss, p.astype(F32), n_valid


def count_valid(targets: np.ndarray, ignore_below: int = 0) -> int:
    """Integer count of positions the engine treats as valid (target >= 0)."""
    return int((np.asarray(targets).reshape(-1) >= ignore_below).sum())


def embedding_bwd(ids: np.ndarray, g: np.ndarray, V: int):
    """Scatter-add of row gradients in row order (axis/ops.py:327-331)."""
    out = np.zeros((V, g.shape[-1]), dtype=F32)
    np.add.at(out, np.asarray(ids).reshape(-1).astype(np.int64), g.reshape(-1, g.shape[-1]))
    return out


# ───────────────────────── parameter bookkeeping ──────────────────────────

def base_param_names(n_layers: int, tied: bool) -> List[str]:
    """Parameter order of the compiled engine (axis/compile.py:95-105)."""
    names = ["embed.weight"]
    for i in range(n_layers):
        p = f"blocks.{i}."
        names += [p + "attn_norm.weight", p + "attn.q_proj.weight",
                  p + "attn.k_proj.weight", p + "attn.v_proj.weight",
                  p + "attn.o_proj.weight", p + "mlp_norm.weight",
                  p + "mlp.gate_proj.weight", p + "mlp.up_proj.weight",
                  p + "mlp.down_proj.weight"]
    names.append("norm.weight")
    if not tied:
        names.append("lm_head.weight")
    return names


def init_weights(cfg: dict, seed: int = 42, std: float = 0.02) -> Dict[str, np.ndarray]:
    """Benchmark-style initialisation: every 2-D tensor ~ N(0, std) drawn in
    parameter order from default_rng(seed); 1-D norm weights = 1."""
    V, D, L = cfg["vocab_size"], cfg["dim"], cfg["n_layers"]
    H = cfg["n_heads"]
    KV = cfg.get("n_kv_heads") or H
    DH = D // H
    MLP = cfg["mlp_hidden"]
    tied = cfg.get("tie_embeddings", True)
    shapes = {"embed.weight": (V, D), "norm.weight": (D,), "lm_head.weight": (D, V)}
    for i in range(L):
        p = f"blocks.{i}."
        shapes.update({p + "attn_norm.weight": (D,), p + "mlp_norm.weight": (D,),
                       p + "attn.q_proj.weight": (D, H * DH),
                       p + "attn.k_proj.weight": (D, KV * DH),
                       p + "attn.v_proj.weight": (D, KV * DH),
                       p + "attn.o_proj.weight": (H * DH, D),
                       p + "mlp.gate_proj.weight": (D, MLP),
                       p + "mlp.up_proj.weight": (D, MLP),
                       p + "mlp.down_proj.weight": (MLP, D)})
    rng = np.random.default_rng(seed)
    out = {}
    for nm in base_param_names(L, tied):
        sh = shapes[nm]
        out[nm] = (np.ones(sh, dtype=F32) if len(sh) == 1
                   else (rng.standard_normal(sh) * std).astype(F32))
    return out


def init_lora(cfg: dict, rank: int, targets: Sequence[str], seed: int = 7,
              std: float = 0.02) -> Dict[str, np.ndarray]:
    """A ~ N(0, std), B = 0 for every targeted projection, in layer order."""
    D, L, H = cfg["dim"], cfg["n_layers"], cfg["n_heads"]
    KV = cfg.get("n_kv_heads") or H
    DH = D // H
    MLP = cfg["mlp_hidden"]
    geom = {"attn.q_proj": (D, H * DH), "attn.k_proj": (D, KV * DH),
            "attn.v_proj": (D, KV * DH), "attn.o_proj": (H * DH, D),
            "mlp.gate_proj": (D, MLP), "mlp.up_proj": (D, MLP), "mlp.down_proj": (MLP, D)}
    rng = np.random.default_rng(seed)
    out = {}
    for i in range(L):
        for pref in LORA_GEOM:
            if pref.split(".")[-1] in targets:
                fin, fout = geom[pref]
                out[f"blocks.{i}.{pref}.lora_a"] = (rng.standard_normal((fin, rank)) * std).astype(F32)
                out[f"blocks.{i}.{pref}.lora_b"] = np.zeros((rank, fout), dtype=F32)
    return out


def zero_ownership(pnames: Sequence[str], shapes: Dict[str, tuple], world: int,
                   sharded: bool = True) -> Tuple[Dict[str, int], List[int]]:
    """Greedy per-tensor owner map of ZeRO-1 (axis/compile.py:132-137): visit
    tensors by decreasing element count (stable), give each to the least
    loaded rank (first minimum).  Integer work: must be reproduced exactly."""
    load = [0] * world
    owner = {}
    for nm in sorted(pnames, key=lambda n: -int(np.prod(shapes[n]))):
        r = int(np.argmin(load)) if sharded else 0
        owner[nm] = r
        load[r] += int(np.prod(shapes[nm]))
    return owner, load


# ───────────────────────── the model step ─────────────────────────────────

class OracleTransformer:
    """Forward + hand-derived backward of the decoder.  `weights` maps the
    engine's parameter names to fp32 arrays (Linear weights are [in, out]).
    With `lora_rank > 0` the base weights are frozen and only adapters named
    `blocks.{i}.{proj}.lora_a/.lora_b` receive gradients."""

    def __init__(self, cfg: dict, weights: Dict[str, np.ndarray], eps: float = 1e-5,
                 lora_rank: int = 0, lora_alpha: float = 16.0,
                 lora_targets: Sequence[str] = ()):
        self.cfg = cfg
        self.V, self.D, self.L = cfg["vocab_size"], cfg["dim"], cfg["n_layers"]
        self.H = cfg["n_heads"]
        self.KV = cfg.get("n_kv_heads") or self.H
        self.DH = self.D // self.H
        self.MLP = cfg["mlp_hidden"]
        self.tied = cfg.get("tie_embeddings", True)
        self.theta = cfg.get("rope_theta", 10000.0)
        self.eps = eps
        self.w = {k: np.ascontiguousarray(v, dtype=F32).copy() for k, v in weights.items()}
        self.lora_rank = lora_rank
        self.lora_scale = float(lora_alpha) / lora_rank if lora_rank else 0.0
        self.lora_targets = set(lora_targets) if lora_rank else set()
        if lora_rank:
            self.trainable = [k for i in range(self.L) for pref in LORA_GEOM
                              if pref.split(".")[-1] in self.lora_targets
                              for k in (f"blocks.{i}.{pref}.lora_a", f"blocks.{i}.{pref}.lora_b")]
        else:
            self.trainable = base_param_names(self.L, self.tied)

    # linear with optional adapter
    def _lin_f(self, x, key, cache):
        y = x @ self.w[key + ".weight"]
        if key.split(".")[-1] in self.lora_targets:
            u = x @ self.w[key + ".lora_a"]
            cache[key + "/u"] = u
            y = y + (u @ self.w[key + ".lora_b"]) * F32(self.lora_scale)
        return y.astype(F32)

    def _lin_b(self, g, x, key, cache, grads):
        dx = g @ self.w[key + ".weight"].T
        if not self.lora_rank:
            grads[key + ".weight"] = (x.reshape(-1, x.shape[-1]).T
                                      @ g.reshape(-1, g.shape[-1])).astype(F32)
        elif key.split(".")[-1] in self.lora_targets:
            s = F32(self.lora_scale)
            t1 = (g @ self.w[key + ".lora_b"].T) * s
            dx = dx + t1 @ self.w[key + ".lora_a"].T
            grads[key + ".lora_a"] = (x.reshape(-1, x.shape[-1]).T
                                      @ t1.reshape(-1, t1.shape[-1])).astype(F32)
            u = cache[key + "/u"]
            grads[key + ".lora_b"] = ((u.reshape(-1, u.shape[-1]).T
                                       @ g.reshape(-1, g.shape[-1])) * s).astype(F32)
        return dx.astype(F32)

    def loss_and_grads(self, tokens: np.ndarray, targets: np.ndarray,
                       ignore_index: int = -1, return_logits: bool = False):
        B, T = tokens.shape
        H, KV, DH, D = self.H, self.KV, self.DH, self.D
        w = self.w
        cos, sin = rope_tables(T, DH, self.theta)
        scale = 1.0 / math.sqrt(DH)
        ids = np.asarray(tokens).astype(np.int64)
        x = w["embed.weight"][ids]                      # [B,T,D]
        saved = []
        for i in range(self.L):
            p = f"blocks.{i}."
            c = {}
            y, inv1 = rmsnorm_fwd(x, w[p + "attn_norm.weight"], self.eps)
            q = self._lin_f(y, p + "attn.q_proj", c).reshape(B, T, H, DH).transpose(0, 2, 1, 3)
            k = self._lin_f(y, p + "attn.k_proj", c).reshape(B, T, KV, DH).transpose(0, 2, 1, 3)
            v = self._lin_f(y, p + "attn.v_proj", c).reshape(B, T, KV, DH).transpose(0, 2, 1, 3)
            q = rope_fwd(q, cos, sin)
            k = rope_fwd(k, cos, sin)
            o, _ = attention_fwd(q, k, v, scale)
            at = o.transpose(0, 2, 1, 3).reshape(B, T, H * DH)
            r1 = x + self._lin_f(at, p + "attn.o_proj", c)
            z, inv2 = rmsnorm_fwd(r1, w[p + "mlp_norm.weight"], self.eps)
            gte = self._lin_f(z, p + "mlp.gate_proj", c)
            up = self._lin_f(z, p + "mlp.up_proj", c)
            hmid, sig = silu_mul_fwd(gte, up)
            xn = r1 + self._lin_f(hmid, p + "mlp.down_proj", c)
            saved.append((x, y, inv1, q, k, v, at, r1, z, inv2, gte, up, sig, hmid, c))
            x = xn
        xf, invf = rmsnorm_fwd(x, w["norm.weight"], self.eps)
        head = w["embed.weight"].T if self.tied else w["lm_head.weight"]
        logits = (xf @ head).astype(F32)
        loss, dlogits, _ = cross_entropy_fwd_bwd(logits.reshape(B * T, self.V),
                                                 targets.reshape(-1), ignore_index)
        grads: Dict[str, np.ndarray] = {}
        dlog = dlogits.reshape(B, T, self.V)
        dxf = dlog @ head.T
        if not self.lora_rank:
            if self.tied:
                head_grad = (dlog.reshape(-1, self.V).T @ xf.reshape(-1, D)).astype(F32)
            else:
                grads["lm_head.weight"] = (xf.reshape(-1, D).T @ dlog.reshape(-1, self.V)).astype(F32)
        dcur, dwn = rmsnorm_bwd(x, w["norm.weight"], invf, dxf)
        if not self.lora_rank:
            grads["norm.weight"] = dwn
        for i in reversed(range(self.L)):
            p = f"blocks.{i}."
            (x0, y, inv1, q, k, v, at, r1, z, inv2, gte, up, sig, hmid, c) = saved[i]
            dh = self._lin_b(dcur, hmid, p + "mlp.down_proj", c, grads)
            dg, du = silu_mul_bwd(gte, up, sig, dh)
            dz = self._lin_b(dg, z, p + "mlp.gate_proj", c, grads) \
                + self._lin_b(du, z, p + "mlp.up_proj", c, grads)
            dr1b, dw2 = rmsnorm_bwd(r1, w[p + "mlp_norm.weight"], inv2, dz)
            if not self.lora_rank:
                grads[p + "mlp_norm.weight"] = dw2
            dr1 = dcur + dr1b
            dat = self._lin_b(dr1, at, p + "attn.o_proj", c, grads)
            do = dat.reshape(B, T, H, DH).transpose(0, 2, 1, 3)
            dq, dk, dv = attention_bwd(q, k, v, do, scale)
            dq = rope_bwd(dq, cos, sin)
            dk = rope_bwd(dk, cos, sin)
            dq0 = dq.transpose(0, 2, 1, 3).reshape(B, T, H * DH)
            dk0 = dk.transpose(0, 2, 1, 3).reshape(B, T, KV * DH)
            dv0 = dv.transpose(0, 2, 1, 3).reshape(B, T, KV * DH)
            dy = self._lin_b(dq0, y, p + "attn.q_proj", c, grads) \
                + self._lin_b(dk0, y, p + "attn.k_proj", c, grads) \
                + self._lin_b(dv0, y, p + "attn.v_proj", c, grads)
            dx1, dw1 = rmsnorm_bwd(x0, w[p + "attn_norm.weight"], inv1, dy)
            if not self.lora_rank:
                grads[p + "attn_norm.weight"] = dw1
            dcur = dr1 + dx1
        if not self.lora_rank:
            eg = embedding_bwd(ids, dcur, self.V)
            grads["embed.weight"] = (head_grad + eg) if self.tied else eg
        if return_logits:
            return loss, grads, logits
        return loss, grads


def clip_scale(grads: Dict[str, np.ndarray], names: Sequence[str], max_norm: float):
    """Global-norm clip factor (axis/optim.py:110-118): returns (norm, scale)."""
    total = math.sqrt(sum(float((grads[n] * grads[n]).sum()) for n in names))
    if max_norm and max_norm > 0 and total > max_norm and total > 0.0:
        return total, max_norm / total
    return total, 1.0


class OracleAdamW:
    """Decoupled AdamW with bias correction; tensors with fewer than two
    dimensions are exempt from weight decay (axis/optim.py:42-63)."""

    def __init__(self, model: OracleTransformer, lr=3e-4, betas=(0.9, 0.95), eps=1e-8, wd=0.1):
        self.model = model
        self.lr, self.b1, self.b2, self.eps, self.wd = lr, betas[0], betas[1], eps, wd
        self.t = 0
        self.m = {n: np.zeros_like(model.w[n]) for n in model.trainable}
        self.v = {n: np.zeros_like(model.w[n]) for n in model.trainable}

    def step(self, grads: Dict[str, np.ndarray], scale: float = 1.0):
        self.t += 1
        bc1 = 1.0 - self.b1 ** self.t
        bc2 = 1.0 - self.b2 ** self.t
        for n in self.model.trainable:
            g = grads[n] * F32(scale) if scale != 1.0 else grads[n]
            self.m[n] = (self.b1 * self.m[n] + (1.0 - self.b1) * g).astype(F32)
            self.v[n] = (self.b2 * self.v[n] + (1.0 - self.b2) * (g * g)).astype(F32)
            p = self.model.w[n]
            if self.wd > 0.0 and p.ndim >= 2:
                p *= F32(1.0 - self.lr * self.wd)
            p -= (self.lr * (self.m[n] / bc1) / (np.sqrt(self.v[n] / bc2) + self.eps)).astype(F32)


def train_step(model: OracleTransformer, opt: OracleAdamW, tokens, targets,
               max_grad_norm: float = 0.0, ignore_index: int = -1):
    """One fwd + bwd + clip + AdamW step; returns (loss, grads_before_clip, grad_norm)."""
    loss, grads = model.loss_and_grads(tokens, targets, ignore_index)
    norm, sc = clip_scale(grads, model.trainable, max_grad_norm)
    opt.step(grads, sc)
    return float(loss), grads, norm


def make_batch(rng: np.random.Generator, V: int, B: int, T: int, ignore_frac: float = 0.0,
               shifted: bool = True):
    """Synthetic batch in the benchmark's style: x uniform in [0, V); y = x
    shifted left by one; a fraction of targets set to -1."""
    x = rng.integers(0, V, size=(B, T)).astype(np.int64)
    y = np.roll(x, -1, axis=1) if shifted else rng.integers(0, V, size=(B, T)).astype(np.int64)
    if ignore_frac > 0:
        y = np.where(rng.random((B, T)) < ignore_frac, -1, y)
    return x, y.astype(np.int64)
