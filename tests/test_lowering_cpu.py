"""Host lowering checked on CPU: the plan emitted by CompiledTransformer is run
by the numpy plan interpreter (tests/plan_interp.py) and compared with the
golden vectors from the reference autograd.  Covers buffer/arena layout, op
arguments, fused-op semantics, the optimizer path, state_dict and capture."""
import json
import os

import numpy as np
import pytest

from axis_b200.compile import CompiledTransformer, compile_model, greedy_owner
from axis_b200.model import Transformer
from oracle import step_numpy as O
from tests.plan_interp import InterpEngine

G = os.path.join(os.path.dirname(__file__), "golden")


def rel(got, ref):
    return float(np.abs(got - ref).max() / (np.abs(ref).max() + 1e-9))


def load(name):
    z = np.load(os.path.join(G, name + ".npz"))
    cfg = json.loads(str(z["cfg"]))
    w0 = {k[3:]: z[k] for k in z.files if k.startswith("w0/")}
    return z, cfg, w0


def build(cfg, w0, dtype="fp32", **kw):
    lora = cfg.get("lora")
    if lora:
        kw.update(lora_r=lora["rank"], lora_alpha=lora["alpha"], lora_targets=tuple(lora["targets"]))
    return CompiledTransformer(InterpEngine(), cfg, w0, cfg["B"], cfg["T"], dtype=dtype,
                               max_grad_norm=cfg["max_norm"], **kw)


@pytest.mark.parametrize("name", ["step_tied_gqa", "step_untied_mha", "step_lora"])
def test_fp32_plan_matches_reference(name):
    z, cfg, w0 = load(name)
    ct = build(cfg, w0)
    for s in range(cfg["steps"]):
        loss = ct.step(z[f"x/{s}"], z[f"y/{s}"])
        assert abs(loss - z["losses"][s]) <= 2e-6 * max(1, abs(z["losses"][s]))
        assert abs(ct.grad_norm() - z["norms"][s]) <= 1e-5 * z["norms"][s]
        assert ct.valid_count() == int((z[f"y/{s}"] >= 0).sum())
        if s == 0:
            g = ct.grads()
            g0 = {k[3:]: z[k] for k in z.files if k.startswith("g0/")}
            assert set(g) == set(g0)
            for nm in g0:
                assert rel(g[nm], g0[nm]) <= 1e-5, nm
    w = ct.get_weights()
    for k in z.files:
        if k.startswith("w1/"):
            assert np.abs(w[k[3:]] - z[k]).max() <= 0.05 * 3e-4, k


def test_bf16_plan_tracks_fp32():
    z, cfg, w0 = load("step_tied_gqa")
    ct = build(cfg, w0, dtype="bf16")
    loss = ct.step(z["x/0"], z["y/0"])
    assert abs(loss - z["losses"][0]) <= 1e-3 * abs(z["losses"][0]) + 1e-3
    g = ct.grads()
    for k in z.files:
        if k.startswith("g0/"):
            assert rel(g[k[3:]], z[k]) <= 2e-2, k


def test_capture_replay_and_set_lr():
    z, cfg, w0 = load("step_tied_gqa")
    a, b = build(cfg, w0), build(cfg, w0)
    b.capture()
    for s in range(2):
        if s == 1:
            a.set_lr(1e-3); b.set_lr(1e-3)
        la = a.step(z[f"x/{s}"], z[f"y/{s}"])
        lb = b.replay_step(z[f"x/{s}"], z[f"y/{s}"])
        assert la == lb
    wa, wb = a.get_weights(), b.get_weights()
    for nm in wa:
        assert np.array_equal(wa[nm], wb[nm])


def test_state_dict_roundtrip_resume():
    z, cfg, w0 = load("step_tied_gqa")
    a = build(cfg, w0)
    a.step(z["x/0"], z["y/0"])
    st = a.state_dict()
    assert set(st) == {f"{p}/{n}" for p in "wmv" for n in a.pnames} | {"_t", "_lr"}
    assert float(st["_t"][0]) == 1.0
    b = build(cfg, w0)
    b.load_state_dict(st)
    la = a.step(z["x/1"], z["y/1"])
    lb = b.step(z["x/1"], z["y/1"])
    assert la == lb
    for nm, w in a.get_weights().items():
        assert np.array_equal(w, b.get_weights()[nm])


def test_parity_step_argument_t():
    """step(x, y, t=k): bias correction of step k, no clipping (reference parity path)."""
    z, cfg, w0 = load("step_tied_gqa")
    ct = build(cfg, w0)
    ct.step(z["x/0"], z["y/0"], t=1)
    m = O.OracleTransformer(cfg, w0)
    opt = O.OracleAdamW(m)
    O.train_step(m, opt, z["x/0"], z["y/0"], max_grad_norm=0.0)
    for nm, w in ct.get_weights().items():
        assert np.abs(w - m.w[nm]).max() <= 0.05 * 3e-4, nm


def test_compile_model_detects_config_and_lora():
    m = Transformer(vocab_size=40, dim=32, n_layers=2, n_heads=4, n_kv_heads=2, mlp_hidden=48)
    ct = compile_model(m, batch=1, seq=6, lib_path=InterpEngine())
    assert ct.cfg["n_kv_heads"] == 2 and ct.cfg["mlp_hidden"] == 48 and ct.lora_r == 0
    assert ct.pnames[0] == "embed.weight" and ct.pnames[-1] == "norm.weight"
    m.apply_lora(rank=4, alpha=8.0, targets=("q_proj", "v_proj"))
    ct = compile_model(m, batch=1, seq=6, lib_path=InterpEngine())
    assert ct.lora_r == 4 and len(ct.pnames) == 2 * 2 * 2
    assert all(n.endswith(("lora_a", "lora_b")) for n in ct.pnames)
    rng = np.random.default_rng(0)
    x, y = O.make_batch(rng, 40, 1, 6)
    l0 = ct.step(x, y)
    assert np.isfinite(l0)
    g = ct.grads()
    # B = 0 at start: dA vanishes, dB does not
    assert all(np.abs(g[n]).max() == 0 for n in g if n.endswith("lora_a"))
    assert any(np.abs(g[n]).max() > 0 for n in g if n.endswith("lora_b"))


def test_owner_map_and_arena_are_consistent():
    shapes = {"a": (5, 7), "b": (100,), "c": (64, 64), "d": (3,), "e": (64, 64)}
    names = list(shapes)
    owner, load_ = greedy_owner(names, shapes, 3, True)
    assert owner == O.zero_ownership(names, shapes, 3)[0]
    assert sum(load_) == sum(int(np.prod(s)) for s in shapes.values())
    z, cfg, w0 = load("step_tied_gqa")
    ct = build(cfg, w0)
    offs = sorted((ct._off[n], int(np.prod(ct.shapes[n]))) for n in ct.pnames)
    for (o1, n1), (o2, _) in zip(offs, offs[1:]):
        assert o1 % 1024 == 0 and o1 + n1 <= o2
    assert ct._P_total % 1024 == 0


def test_invalid_inputs_are_rejected():
    z, cfg, w0 = load("step_tied_gqa")
    ct = build(cfg, w0)
    x = z["x/0"].copy()
    x[0, 0] = cfg["vocab_size"]
    with pytest.raises(RuntimeError):
        ct.step(x, z["y/0"])
    with pytest.raises(ValueError):
        ct.step(z["x/0"][:, :-1], z["y/0"])


def test_gradient_accumulation_equals_the_concatenated_batch():
    """Two micro-batches with the same number of valid targets, accumulated, give the step of the
    concatenated batch (the reference's accumulation equivalence, tests/test_generate_accum.py:51)."""
    cfg = dict(vocab_size=61, dim=32, n_layers=2, n_heads=4, n_kv_heads=2, mlp_hidden=48, tie_embeddings=True)
    B, T = 2, 12
    w0 = O.init_weights(cfg, seed=4)
    rng = np.random.default_rng(4)
    xs = [rng.integers(0, cfg["vocab_size"], (B, T)) for _ in range(2)]
    ys = [np.roll(x, -1, axis=1) for x in xs]              # no ignored targets: equal counts
    ct = CompiledTransformer(InterpEngine(), cfg, w0, B, T, dtype="fp32", max_grad_norm=1.0)
    loss = ct.step_accumulate(list(zip(xs, ys)))
    model = O.OracleTransformer(cfg, w0)
    opt = O.OracleAdamW(model)
    l_ref = O.train_step(model, opt, np.concatenate(xs), np.concatenate(ys), max_grad_norm=1.0)[0]
    assert abs(loss - l_ref) <= 2e-6 * abs(l_ref)
    w = ct.get_weights()
    for nm in w:
        assert np.abs(w[nm] - model.w[nm]).max() <= 0.02 * 3e-4, nm
    # a second accumulated step reuses the cached plans and keeps tracking the oracle
    loss2 = ct.step_accumulate(list(zip(xs[::-1], ys[::-1])))
    l2 = O.train_step(model, opt, np.concatenate(xs[::-1]), np.concatenate(ys[::-1]), max_grad_norm=1.0)[0]
    assert abs(loss2 - l2) <= 5e-6 * abs(l2)


@pytest.mark.parametrize("name,dtype", [("step_tied_gqa", "fp32"), ("step_lora", "fp32"), ("step_untied_mha", "bf16")])
def test_block_recompute_reproduces_the_plain_plan_bit_for_bit(name, dtype):
    """Keeping only each block's input and re-running the block's forward inside the backward (the eager
    engine's ops.checkpoint, axis/ops.py:440-475) gives the same losses, gradients and weights, bit for
    bit, and still matches the reference's golden step."""
    z, cfg, w0 = load(name)
    a = build(cfg, w0, dtype=dtype)
    b = build(cfg, w0, dtype=dtype, recompute_blocks=True)
    assert b.recompute_blocks and not a.recompute_blocks
    L = cfg["n_layers"]
    from axis_b200.engine import ATTN_FWD, ATTN_BWD
    kinds = lambda ct: [int(o[0]) for o in ct.plan_fb]
    assert kinds(a).count(ATTN_FWD) == L and kinds(b).count(ATTN_FWD) == 2 * L - 1
    assert kinds(a).count(ATTN_BWD) == kinds(b).count(ATTN_BWD) == L
    for s in range(2):
        la = a.step(z[f"x/{s}"], z[f"y/{s}"])
        lb = b.step(z[f"x/{s}"], z[f"y/{s}"])
        assert la == lb
        if dtype == "fp32":
            assert abs(lb - z["losses"][s]) <= 2e-6 * max(1, abs(z["losses"][s]))
        ga, gb = a.grads(), b.grads()
        for nm in ga:
            assert np.array_equal(ga[nm], gb[nm]), nm
    wa, wb = a.get_weights(), b.get_weights()
    for nm in wa:
        assert np.array_equal(wa[nm], wb[nm]), nm


def test_block_recompute_keeps_one_set_of_activations():
    """Device bytes of the activations: L sets without recompute, one set (plus a block input per layer) with."""
    cfg = dict(vocab_size=61, dim=32, n_layers=6, n_heads=4, n_kv_heads=2, mlp_hidden=48, tie_embeddings=True)
    w0 = O.init_weights(cfg, seed=1)
    e0, e1 = InterpEngine(), InterpEngine()
    CompiledTransformer(e0, cfg, w0, 2, 16, dtype="bf16")
    CompiledTransformer(e1, cfg, w0, 2, 16, dtype="bf16", recompute_blocks=True)
    N, D, MLP, H, KV, DH, L = 32, 32, 48, 4, 2, 8, 6
    per_block = 2 * (N * D * 5 + N * KV * DH * 2 + N * MLP * 3) + 4 * 2 * H * 16      # all but the block input
    assert e0.bytes_allocated() - e1.bytes_allocated() == (L - 1) * per_block


def test_async_replay_returns_the_previous_loss():
    """replay_step_async hands out step i's loss when step i+1 is queued; the sequence equals replay_step's."""
    z, cfg, w0 = load("step_tied_gqa")
    a, b = build(cfg, w0), build(cfg, w0)
    a.capture(); b.capture()
    xs = [(z[f"x/{s % cfg['steps']}"], z[f"y/{s % cfg['steps']}"]) for s in range(4)]
    want = [a.replay_step(x, y) for x, y in xs]
    got = [b.replay_step_async(x, y) for x, y in xs]
    assert got[0] is None and got[1:] == want[:-1]
    assert b.flush() == want[-1] and b.flush() is None
    assert b.replay_step_async(*xs[0]) is None          # after a flush the pipeline starts empty again
    with pytest.raises(RuntimeError):
        b.eng.download_wait(12345)
