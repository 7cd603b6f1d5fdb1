"""The CPU oracle against the golden vectors produced by the reference's own
numpy autograd (tests/golden/make_golden.py) — pins the oracle."""
import json
import os

import numpy as np
import pytest

from oracle import step_numpy as O

G = os.path.join(os.path.dirname(__file__), "golden")


def rel(got, ref):
    return float(np.abs(got - ref).max() / (np.abs(ref).max() + 1e-9))


def _load(name):
    z = np.load(os.path.join(G, name + ".npz"))
    cfg = json.loads(str(z["cfg"]))
    return z, cfg


@pytest.mark.parametrize("name", ["step_tied_gqa", "step_untied_mha", "step_lora"])
def test_step_matches_reference(name):
    z, cfg = _load(name)
    w0 = {k[3:]: z[k] for k in z.files if k.startswith("w0/")}
    lora = cfg["lora"]
    kw = {}
    if lora:
        kw = dict(lora_rank=lora["rank"], lora_alpha=lora["alpha"], lora_targets=lora["targets"])
    model = O.OracleTransformer(cfg, w0, **kw)
    opt = O.OracleAdamW(model, lr=3e-4, betas=(0.9, 0.95), eps=1e-8, wd=0.1)
    for s in range(cfg["steps"]):
        loss, grads, norm = O.train_step(model, opt, z[f"x/{s}"], z[f"y/{s}"],
                                         max_grad_norm=cfg["max_norm"])
        assert abs(loss - z["losses"][s]) <= 1e-6 * max(1.0, abs(z["losses"][s]))
        assert abs(norm - z["norms"][s]) <= 1e-5 * z["norms"][s]
        if s == 0:
            g0 = {k[3:]: z[k] for k in z.files if k.startswith("g0/")}
            assert set(g0) == set(model.trainable)
            for nm, ref in g0.items():
                assert rel(grads[nm], ref) <= 1e-5, nm
    for k in z.files:
        if k.startswith("w1/"):
            # AdamW normalises by sqrt(v): entries whose gradient is ~0 amplify
            # fp32 rounding, so allow a few percent of one lr-sized update
            assert np.abs(model.w[k[3:]] - z[k]).max() <= 0.05 * 3e-4, k


def test_attention_bwd_matches_reference():
    z = np.load(os.path.join(G, "attention_gqa.npz"))
    o, lse = O.attention_fwd(z["q"], z["k"], z["v"], float(z["scale"]))
    assert rel(o, z["o"]) <= 1e-6
    dq, dk, dv = O.attention_bwd(z["q"], z["k"], z["v"], z["do"], float(z["scale"]))
    assert rel(dq, z["dq"]) <= 1e-5
    assert rel(dk, z["dk"]) <= 1e-5
    assert rel(dv, z["dv"]) <= 1e-5
    # the saved LSE reproduces the probabilities
    B, H, T, DH = z["q"].shape
    rep = H // z["k"].shape[1]
    s = (z["q"][0, 3] @ z["k"][0, 3 // rep].T) * float(z["scale"])
    p = np.where(np.tril(np.ones((T, T), bool)), np.exp(s - lse[0, 3][:, None]), 0)
    np.testing.assert_allclose(p.sum(-1), 1.0, rtol=1e-5)


def test_zero_ownership_is_bit_exact():
    with open(os.path.join(G, "zero_ownership_7b.json")) as f:
        ref = json.load(f)
    V, D, L, MLP = 32000, 4096, 32, 11008
    shapes = {"embed.weight": (V, D), "norm.weight": (D,)}
    for i in range(L):
        p = f"blocks.{i}."
        shapes.update({p + "attn_norm.weight": (D,), p + "mlp_norm.weight": (D,),
                       p + "attn.q_proj.weight": (D, D), p + "attn.k_proj.weight": (D, D),
                       p + "attn.v_proj.weight": (D, D), p + "attn.o_proj.weight": (D, D),
                       p + "mlp.gate_proj.weight": (D, MLP), p + "mlp.up_proj.weight": (D, MLP),
                       p + "mlp.down_proj.weight": (MLP, D)})
    names = O.base_param_names(L, True)
    for world in (2, 4, 8):
        owner, load = O.zero_ownership(names, shapes, world)
        assert owner == ref[str(world)]["owner"]
        assert load == ref[str(world)]["load"]
        assert sum(1 for n in names if owner[n] == 0) == ref[str(world)]["owned_rank0"]


def test_ce_ignore_and_count():
    rng = np.random.default_rng(0)
    logits = rng.standard_normal((7, 11)).astype(np.float32)
    t = np.array([3, -1, 0, 10, -1, 5, 2])
    loss, dl, n = O.cross_entropy_fwd_bwd(logits, t)
    assert n == 5 == O.count_valid(t)
    assert np.all(dl[[1, 4]] == 0)
    lp = logits - np.log(np.exp(logits).sum(-1, keepdims=True))
    manual = -np.mean([lp[i, t[i]] for i in range(7) if t[i] >= 0])
    assert abs(loss - manual) < 1e-6
    with pytest.raises(ValueError):
        O.cross_entropy_fwd_bwd(logits, np.full(7, -1))


def test_gradcheck_small():
    """Finite differences on the oracle itself (same eps/tolerances the
    reference's gradcheck uses: eps 1e-3, rtol 1e-2, atol 1e-3)."""
    cfg = dict(vocab_size=17, dim=16, n_layers=1, n_heads=2, n_kv_heads=1, mlp_hidden=24,
               tie_embeddings=True)
    w = O.init_weights(cfg, seed=3, std=0.3)
    w = {k: v.astype(np.float64) for k, v in w.items()}
    rng = np.random.default_rng(1)
    x, y = O.make_batch(rng, 17, 2, 5, 0.2)

    def f(ww):
        m = O.OracleTransformer(cfg, ww)
        m.w = {k: v.astype(np.float64) for k, v in ww.items()}
        return m
    m = f(w)
    O_F32 = O.F32
    O.F32 = np.float64
    try:
        loss, grads = m.loss_and_grads(x, y)
        for nm in ("blocks.0.attn.k_proj.weight", "blocks.0.mlp_norm.weight", "embed.weight"):
            idx = tuple(rng.integers(0, s) for s in w[nm].shape)
            wp = {k: v.copy() for k, v in w.items()}
            wp[nm][idx] += 1e-3
            lp, _ = f(wp).loss_and_grads(x, y)
            wp[nm][idx] -= 2e-3
            lm, _ = f(wp).loss_and_grads(x, y)
            fd = (float(lp) - float(lm)) / 2e-3
            assert abs(fd - grads[nm][idx]) <= 1e-3 + 1e-2 * abs(fd), nm
    finally:
        O.F32 = O_F32
