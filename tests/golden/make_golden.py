"""Generate the golden vectors under tests/golden/ from the reference itself.

Run where the reference tree is importable:

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py /path/to/reference

It drives the reference's own numpy autograd (axis.nn.Transformer.loss ->
backward -> optim.clip_grad_norm -> optim.AdamW.step, and axis.lora) on small
seeded cases and stores losses, gradients and updated weights.  The ZeRO-1
owner map is taken from the reference's CompiledTransformer built on a stub
engine (no GPU involved).  The outputs are committed; the GPU box never runs
this script.
"""
from __future__ import annotations

import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def _weights(model, rng, std=0.02):
    for _, p in model.named_parameters():
        if p.data.ndim >= 2:
            p.data[...] = (rng.standard_normal(p.data.shape) * std).astype(np.float32)
        else:
            p.data[...] = 1.0


def step_case(name, V, D, L, H, KV, MLP, B, T, tied, steps, seed, ignore_frac,
              max_norm=1.0, lora=None):
    import axis
    from axis import nn, optim
    from axis.tensor import Tensor
    axis.manual_seed(seed)
    model = nn.Transformer(vocab_size=V, dim=D, n_layers=L, n_heads=H, n_kv_heads=KV,
                           mlp_hidden=MLP, max_seq_len=T, tie_embeddings=tied)
    rng = np.random.default_rng(seed)
    _weights(model, rng)
    out = {}
    if lora:
        from axis.lora import apply_lora, trainable_parameters
        apply_lora(model, rank=lora["rank"], alpha=lora["alpha"], target_modules=lora["targets"])
        for n, p in model.named_parameters():
            if n.endswith("lora_a"):
                p.data[...] = (rng.standard_normal(p.data.shape) * 0.02).astype(np.float32)
            if n.endswith("lora_b"):       # non-zero B so that dA is exercised
                p.data[...] = (rng.standard_normal(p.data.shape) * 0.02).astype(np.float32)
        params = trainable_parameters(model)
    else:
        params = list(model.parameters())
    norm = lambda n: n.replace(".base.weight", ".weight")
    for n, p in model.named_parameters():
        out["w0/" + norm(n)] = p.data.copy()
    opt = optim.AdamW(params, lr=3e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    losses, norms = [], []
    for s in range(steps):
        x = rng.integers(0, V, size=(B, T)).astype(np.int64)
        y = np.roll(x, -1, axis=1)
        y = np.where(rng.random((B, T)) < ignore_frac, -1, y).astype(np.int64)
        out[f"x/{s}"] = x
        out[f"y/{s}"] = y
        for p in model.parameters():
            p.grad = None
        loss = model.loss(Tensor(x), Tensor(y), ignore_index=-1)
        loss.backward()
        losses.append(float(loss.data))
        if s == 0:
            for n, p in model.named_parameters():
                if p.grad is not None and p.requires_grad:
                    out["g0/" + norm(n)] = p.grad.copy()
        norms.append(optim.clip_grad_norm(params, max_norm))
        opt.step()
    for n, p in model.named_parameters():
        if p.requires_grad:
            out["w1/" + norm(n)] = p.data.copy()
    out["losses"] = np.array(losses, dtype=np.float64)
    out["norms"] = np.array(norms, dtype=np.float64)
    out["cfg"] = np.array(json.dumps(dict(
        vocab_size=V, dim=D, n_layers=L, n_heads=H, n_kv_heads=KV, mlp_hidden=MLP,
        tie_embeddings=tied, B=B, T=T, steps=steps, max_norm=max_norm, lora=lora)))
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **out)
    print(name, "losses", losses, "norms", norms)


def attention_case():
    from axis import ops
    from axis.tensor import Tensor
    rng = np.random.default_rng(11)
    B, H, KV, T, DH = 2, 6, 2, 24, 16
    rep = H // KV
    q = rng.standard_normal((B, H, T, DH)).astype(np.float32)
    k = rng.standard_normal((B, KV, T, DH)).astype(np.float32)
    v = rng.standard_normal((B, KV, T, DH)).astype(np.float32)
    do = rng.standard_normal((B, H, T, DH)).astype(np.float32)
    scale = 1.0 / np.sqrt(DH)
    qt = Tensor(q, requires_grad=True)
    kr = Tensor(np.repeat(k, rep, axis=1), requires_grad=True)   # grouped repeat
    vr = Tensor(np.repeat(v, rep, axis=1), requires_grad=True)
    o = ops.fused_causal_attention(qt, kr, vr, scale)
    o.backward(do)
    dk = kr.grad.reshape(B, KV, rep, T, DH).sum(axis=2)
    dv = vr.grad.reshape(B, KV, rep, T, DH).sum(axis=2)
    np.savez_compressed(os.path.join(HERE, "attention_gqa.npz"), q=q, k=k, v=v, do=do,
                        o=o.data, dq=qt.grad, dk=dk, dv=dv, scale=np.float32(scale))
    print("attention_gqa done")


class _StubEngine:
    """Stands in for axis.engine.Engine so that the reference's plan builder
    runs without a GPU; it only hands out buffer indices."""
    has_flash = True

    def __init__(self, *_a, **_k):
        self.n = 0
        self.bytes = 0

    def alloc(self, nelems, itemsize=4):
        self.n += 1
        self.bytes += int(nelems) * itemsize
        return self.n - 1

    def new_tensor(self, arr):
        return self.alloc(arr.size)

    def upload(self, *_a): pass
    def run(self, *_a, **_k): pass
    def set_tf32(self, *_a): pass


def ownership_case():
    """ZeRO-1 owner map of the 7B-class shape at world 2/4/8, from the
    reference plan builder with shape-only (zero-strided) weights."""
    import axis.compile as rc
    rc.Engine = _StubEngine
    V, D, L, H, KV, MLP = 32000, 4096, 32, 32, 32, 11008
    cfg = dict(vocab_size=V, dim=D, n_layers=L, n_heads=H, n_kv_heads=KV,
               mlp_hidden=MLP, tie_embeddings=True)
    def fake(shape):
        return np.lib.stride_tricks.as_strided(np.zeros(1, np.float32), shape=shape,
                                               strides=(0,) * len(shape))
    shapes = {"embed.weight": (V, D), "norm.weight": (D,)}
    for i in range(L):
        p = f"blocks.{i}."
        shapes.update({p + "attn_norm.weight": (D,), p + "mlp_norm.weight": (D,),
                       p + "attn.q_proj.weight": (D, D), p + "attn.k_proj.weight": (D, D),
                       p + "attn.v_proj.weight": (D, D), p + "attn.o_proj.weight": (D, D),
                       p + "mlp.gate_proj.weight": (D, MLP), p + "mlp.up_proj.weight": (D, MLP),
                       p + "mlp.down_proj.weight": (MLP, D)})

    class W(dict):
        def __getitem__(self, k):
            return fake(shapes[k])
    res = {}
    orig_asc = np.ascontiguousarray
    rc.np.ascontiguousarray = lambda a, dtype=None: a       # keep shape-only arrays
    orig_zl = np.zeros_like
    rc.np.zeros_like = lambda a: a
    try:
        for world in (2, 4, 8):
            ct = rc.CompiledTransformer("stub", cfg, W(shapes), 2, 64, dtype="bf16",
                                        grad_sync=True, zero_stage=1, rank=0, world=world,
                                        max_grad_norm=1.0)
            load = [0] * world
            for nm, r in ct.owner.items():
                load[r] += int(np.prod(shapes[nm]))
            res[str(world)] = dict(owner=ct.owner, load=load, owned_rank0=len(ct.owned))
    finally:
        rc.np.ascontiguousarray = orig_asc
        rc.np.zeros_like = orig_zl
    with open(os.path.join(HERE, "zero_ownership_7b.json"), "w") as f:
        json.dump(res, f)
    print("ownership", {w: (r["load"], r["owned_rank0"]) for w, r in res.items()})


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit("usage: python make_golden.py <path to a checkout of the reference repository>")
    ref = sys.argv[1]
    sys.path.insert(0, ref)
    sys.dont_write_bytecode = True
    step_case("step_tied_gqa", V=96, D=64, L=2, H=4, KV=2, MLP=80, B=2, T=12, tied=True,
              steps=3, seed=42, ignore_frac=0.10)
    step_case("step_untied_mha", V=50, D=32, L=1, H=2, KV=2, MLP=40, B=1, T=9, tied=False,
              steps=2, seed=5, ignore_frac=0.0)
    step_case("step_lora", V=64, D=64, L=2, H=4, KV=2, MLP=96, B=2, T=10, tied=True,
              steps=2, seed=9, ignore_frac=0.4,
              lora=dict(rank=4, alpha=8.0, targets=["q_proj", "k_proj", "v_proj", "o_proj",
                                                    "gate_proj", "up_proj", "down_proj"]))
    attention_case()
    ownership_case()
