"""Host lowering checked on CPU: the plan emitted by CompiledTransformer is run
by the numpy plan interpreter (tests/plan_interp.py) and compared with the
golden vectors from the reference autograd.  Covers buffer/arena layout, op
arguments, fused-op semantics, the optimizer path, state_dict and capture."""
import json
import os

import numpy as np
import pytest

from axis_b200 import engine as E
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


def _side_stream_hazards(plan):
    """Static check of a plan that queues weight-gradient GEMMs on the side stream (STREAM tb=2): every such GEMM
    must start after an event recorded on the main chain directly before it, and until the main chain (or the
    collectives stream, for REDUCE / BROADCAST) has waited for the event recorded after it, no op there may write
    a buffer the GEMM reads or touch a buffer it writes.  Returns a list of violations."""
    from axis_b200 import engine as E
    F = dict(kind=0, a=1, b=2, c=3, d=4, m=5, n=6, k=7, batch=8, tb=9, sa=10, sb=11, sc=12, dt=13, oa=14, ob=15, oc=16)
    writes = {E.GEMM_SB: ["c"], E.GEMM_EX: ["c"], E.GEMM_GROUP: ["c", "d", "sc"], E.SILU_BWD: ["c", "tb"],
              E.RMSNORM_BWD_ACC: ["c", "sb"], E.RMSNORM: ["c"], E.ATTN_FWD: ["c", "sa"],
              E.ATTN_BWD: ["tb", "sc", "oa", "oc"], E.ROPE_BTHD: ["c", "sb"], E.CE_FUSED: ["c", "d", "sa", "sb"],
              E.EMBED_I32: ["c"], E.EMBED_BWD_DET: ["c"], E.SILU_MUL: ["c"], E.SCALE: ["c"]}
    bad, stream = [], 0
    n_norms = [0]
    side = []                                   # (index, reads, writes, e_out or None)
    for i, o in enumerate(plan):
        k = o[0]
        if k == E.STREAM:
            stream = o[F["tb"]]
            continue
        if k == E.EVENT:
            if o[F["tb"]] == 1 and o[F["sa"]] == 2 and side and side[-1][3] is None:
                side[-1][3] = o[F["oa"]]        # the event recorded after the last side GEMM
            if o[F["tb"]] == 2 and o[F["sa"]] in (0, 1):      # main / collectives caught up with the side stream
                for s_ in side:
                    if s_[3] is not None and s_[3] <= o[F["oa"]]:
                        s_[4].add(o[F["sa"]])
            continue
        if stream == 2:
            if k == E.GNORM_FLAT:
                # a bucket's squared norm, in order behind the bucket's dW GEMMs on this stream: it must also wait for
                # the main chain (norm weight gradients, embedding scatter) and be awaited before AdamW
                prev = plan[i - 1], plan[i - 2], plan[i - 3]
                if not (prev[0][0] == E.STREAM and prev[1][0] == E.EVENT and prev[1][F["tb"]] == 2 and prev[1][F["sa"]] == 2
                        and prev[2][0] == E.EVENT and prev[2][F["tb"]] == 1 and prev[2][F["sa"]] == 0
                        and prev[1][F["oa"]] == prev[2][F["oa"]]):
                    bad.append((i, "side-stream norm does not wait for the main chain"))
                side.append([i, set(), {o[F["c"]], o[F["d"]]}, None, set()])
                n_norms[0] += 1
                continue
            if k not in (E.GEMM_SB, E.GEMM_GROUP):
                bad.append((i, "non-GEMM op on the side stream"))
            prev = plan[i - 1], plan[i - 2], plan[i - 3]
            if not (prev[0][0] == E.STREAM and prev[1][0] == E.EVENT and prev[1][F["tb"]] == 2 and prev[1][F["sa"]] == 2
                    and prev[2][0] == E.EVENT and prev[2][F["tb"]] == 1 and prev[2][F["sa"]] == 0
                    and prev[1][F["oa"]] == prev[2][F["oa"]]):
                bad.append((i, "side GEMM does not wait for the main chain"))
            grp = k == E.GEMM_GROUP
            rd = {o[F[f]] for f in (("a", "b", "sa", "sb") if grp else ("a", "b"))} - {0, -1}
            wr = {o[F[f]] for f in (("c", "d", "sc") if grp else ("c",))} - {0, -1}
            side.append([i, rd, wr, None, set()])
            continue
        if k in (E.GROUP, E.FORK, E.JOIN):
            continue
        who = 1 if stream == 1 else 0
        touched = {o[F[f]] for f in ("a", "b", "c", "d", "sa", "sb", "sc", "tb", "oa", "oc") if isinstance(o[F[f]], int)}
        written = {o[F[f]] for f in writes.get(k, [])}
        for s_ in side:
            if who in s_[4]:
                continue                        # this stream has waited for that GEMM
            if written & s_[1]:
                bad.append((i, f"op {E.KIND_NAMES[k]} rewrites an input of the side GEMM at {s_[0]}"))
            if k not in (E.COLSUM_BATCH, E.GNORM_FLAT, E.ADAMW_FLAT, E.REDUCE, E.BROADCAST) and touched & s_[2]:
                bad.append((i, f"op {E.KIND_NAMES[k]} touches an output of the side GEMM at {s_[0]}"))
            if k in (E.GNORM_FLAT, E.ADAMW_FLAT, E.REDUCE, E.BROADCAST):
                bad.append((i, f"{E.KIND_NAMES[k]} over the gradient arena before the side GEMM at {s_[0]} is awaited"))
    if any(0 not in s_[4] for s_ in side):
        bad.append((len(plan), "the main chain ends before the side stream"))
    return bad, len(side) - n_norms[0]


@pytest.mark.parametrize("world", [1, 2])
def test_side_stream_weight_gradients_are_ordered_by_events(world):
    """The dW GEMMs run on a side stream; the plan orders them against the main chain and the collectives with
    events only.  The checker finds no hazard in the emitted plans and does find one when a wait is removed."""
    from axis_b200 import engine as E
    cfg = dict(vocab_size=61, dim=32, n_layers=5, n_heads=4, n_kv_heads=2, mlp_hidden=48, tie_embeddings=True)
    w0 = O.init_weights(cfg, seed=1)
    kw = dict(grad_sync=True, zero_stage=1, rank=0, world=2, bucket_layers=2) if world == 2 else {}
    ct = CompiledTransformer(InterpEngine(), cfg, w0, 2, 8, dtype="bf16", max_grad_norm=1.0, **kw)
    assert ct.overlap_dw
    bad, n_side = _side_stream_hazards(ct.plan_step)
    assert not bad, bad[:5]
    assert n_side == 4 * cfg["n_layers"]
    # drop the wait in front of one SiLU backward: the rewrite of dg/du races with the previous block's dW
    plan = list(ct.plan_step)
    idx = [i for i, o in enumerate(plan) if o[0] == E.SILU_BWD][2]
    assert plan[idx - 1][0] == E.EVENT and plan[idx - 1][9] == 2
    del plan[idx - 1]
    bad2, _ = _side_stream_hazards(plan)
    assert any("rewrites an input" in msg for _, msg in bad2)
    # adapters and per-block recompute keep everything on the main chain
    for kw2 in (dict(lora_r=4), dict(recompute_blocks=True), dict(overlap_dw=False)):
        c2 = CompiledTransformer(InterpEngine(), cfg, w0, 2, 8, dtype="bf16", **kw2)
        assert not c2.overlap_dw and not any(o[0] == E.EVENT for o in c2.plan_step)


class _ShapeOnlyEngine:
    """Engine stand-in that holds no data: it hands out slots, tracks sizes and packs every plan it is given, so
    a 7B-class buffer plan and op plan can be built and checked on a small host."""
    has_flash = True

    def __init__(self):
        self.sizes, self.ran = [], []

    def alloc(self, nelems, itemsize=4):
        self.sizes.append(int(nelems) * itemsize)
        return len(self.sizes) - 1

    def alloc_zero(self, nbytes):
        self.sizes.append(int(nbytes))
        return len(self.sizes) - 1

    def view(self, parent, byte_offset, nbytes):
        assert 0 <= byte_offset and byte_offset + nbytes <= self.sizes[parent]
        self.sizes.append(int(nbytes))
        return len(self.sizes) - 1

    def new_tensor(self, arr):
        return self.alloc(arr.size)

    def run(self, plan, sync=True):
        from axis_b200.engine import PackedPlan
        self.ran.append((list(plan), PackedPlan(plan)))

    def upload(self, *a): pass
    def upload_raw(self, *a, **k): pass
    def set_tf32(self, *a): pass


class _ShapeOnlyWeight:
    def __init__(self, shape):
        self.shape = tuple(shape)

    def load_into(self, eng, dst, fp32_out, stage):
        pass


@pytest.mark.parametrize("world", [1, 2, 8])
def test_7b_plan_fits_the_32bit_op_descriptor(world):
    """The 7B-class arenas hold more elements than an int32: every integer field of every op of the plan, and of
    the set-up ops the constructor runs (master -> bf16 mirror cast), must survive packing unchanged."""
    from axis_b200 import engine as E
    V, D, L, H, MLP = 32000, 4096, 32, 32, 11008
    cfg = dict(vocab_size=V, dim=D, n_layers=L, n_heads=H, n_kv_heads=H, mlp_hidden=MLP, tie_embeddings=True)
    shapes = {"embed.weight": (V, D), "norm.weight": (D,)}
    for i in range(L):
        p = f"blocks.{i}."
        shapes.update({p + "attn_norm.weight": (D,), p + "mlp_norm.weight": (D,),
                       p + "attn.q_proj.weight": (D, D), p + "attn.k_proj.weight": (D, D),
                       p + "attn.v_proj.weight": (D, D), p + "attn.o_proj.weight": (D, D),
                       p + "mlp.gate_proj.weight": (D, MLP), p + "mlp.up_proj.weight": (D, MLP),
                       p + "mlp.down_proj.weight": (MLP, D)})
    eng = _ShapeOnlyEngine()
    ct = CompiledTransformer(eng, cfg, {n: _ShapeOnlyWeight(s) for n, s in shapes.items()}, 2, 4096, dtype="bf16",
                             max_grad_norm=1.0, grad_sync=world > 1, zero_stage=1 if world > 1 else 0, rank=0, world=world)
    assert ct._P_total > 2 ** 31 or world > 1
    # the constructor's cast of the owned segment: element count carried as chunks x CHUNK
    casts = [o for plan, _ in eng.ran for o in plan if o[0] == E.CAST]
    assert sum(o[5] * max(o[6], 1) for o in casts) == ct._my_seg[1]
    for plan in (ct.plan_step, ct.plan_fb, ct.plan_ar):
        pp = E.PackedPlan(plan)
        for j, name in enumerate(E._OP_DTYPE.names[:17]):
            assert [int(v) for v in pp.arr[name]] == [int(o[j]) for o in plan], name
    # and the packer refuses what it cannot represent instead of wrapping
    with pytest.raises(OverflowError):
        E.PackedPlan([E.op(E.CAST, a=0, c=1, m=ct._P_total if ct._P_total > 2 ** 31 else 2 ** 31 + 5)])


@pytest.mark.parametrize("dtype,lim_l,lim_g", [("fp32", 2e-6, 1e-5), ("bf16", 2e-3, 3e-2)])
def test_head_dim_64_plan_with_rotary_inside_the_projection_and_the_attention_backward(dtype, lim_l, lim_g):
    """At head_dim 64 the plan has no rotary op of its own: the forward rotation rides in the q/k/v projection launch
    (GEMM_GROUP with gamma > 0) and the inverse one in ATTN_BWD.  Against the oracle."""
    from axis_b200 import engine as E
    cfg = dict(vocab_size=70, dim=128, n_layers=2, n_heads=2, n_kv_heads=1, mlp_hidden=96, tie_embeddings=True)
    w0 = O.init_weights(cfg, seed=11)
    rng = np.random.default_rng(11)
    x, y = O.make_batch(rng, 70, 2, 24, 0.1)
    l_ref, g_ref = O.OracleTransformer(cfg, w0).loss_and_grads(x, y)
    ct = CompiledTransformer(InterpEngine(), cfg, w0, 2, 24, dtype=dtype, max_grad_norm=1.0)
    assert not any(o[0] in (E.ROPE, E.ROPE_BTHD) for o in ct.plan_step)
    loss = ct.forward_backward(x, y)
    assert abs(loss - l_ref) <= lim_l * abs(l_ref)
    g = ct.grads()
    for nm in g_ref:
        assert rel(g[nm], g_ref[nm]) <= lim_g, nm


def test_adapter_plan_is_a_few_fat_launches_per_layer():
    """With adapters on all seven projections a layer lowers to 8 tensor-core GEMM launches (the four projection groups
    each way, adapter terms riding as K-segments), 8 streaming launches for the skinny products and one for all adapter
    gradients — not to four extra GEMMs per projection as in axis/compile.py:270-305."""
    cfg = dict(vocab_size=64, dim=64, n_layers=2, n_heads=4, n_kv_heads=2, mlp_hidden=96, tie_embeddings=True)
    w = O.init_weights(cfg, seed=3)
    w.update(O.init_lora(cfg, 8, ["q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj"], seed=4))
    ct = CompiledTransformer(InterpEngine(), cfg, w, 2, 16, dtype="bf16", lora_r=8, lora_alpha=16.0,
                             lora_targets=("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj"))
    kinds = [o[0] for o in ct.plan_step]
    L = cfg["n_layers"]
    gemms = sum(kinds.count(k) for k in (E.GEMM, E.GEMM_SB, E.GEMM_EX, E.GEMM_GROUP))
    assert gemms == 8 * L + 2                       # + logits and their input gradient
    assert kinds.count(E.LORA_PROJ) == 8 * L
    assert sum(1 for o in ct.plan_step if o[0] == E.LORA_GRAD and o[8] == 0) == L        # one run per layer ...
    assert sum(-o[8] for o in ct.plan_step if o[0] == E.LORA_GRAD and o[8] < 0) == 14 * L   # ... of its 14 noted products
    assert kinds.count(E.GEMM_XSEG) == 8 * L
    assert kinds.count(E.ROPE_BTHD) == L            # head_dim 16 here: the rotary epilogue serves head_dim 64


def test_bucket_norms_on_the_side_stream_match_the_single_pass():
    """One GPU: the clip's gradient norm is assembled from per-bucket sums taken as the buckets complete — on the side
    stream when the weight gradients run there, on the main chain otherwise; both plans give the same bits, the norm is
    the norm of all gradients, and the step counter ticks once per step."""
    cfg = dict(vocab_size=61, dim=32, n_layers=5, n_heads=4, n_kv_heads=2, mlp_hidden=48, tie_embeddings=True)
    w0 = O.init_weights(cfg, seed=2)
    rng = np.random.default_rng(2)
    a = CompiledTransformer(InterpEngine(), cfg, w0, 2, 8, dtype="fp32", max_grad_norm=0.5)
    b = CompiledTransformer(InterpEngine(), cfg, w0, 2, 8, dtype="fp32", max_grad_norm=0.5, overlap_dw=False)
    assert a.bucket_norms and b.bucket_norms and a.overlap_dw and not b.overlap_dw
    assert sum(1 for o in a.plan_step if o[0] == E.GNORM_FLAT) == a._nbuckets
    assert any(o[0] == E.STREAM and o[9] == 2 for o in a.plan_step) and not any(o[0] == E.EVENT for o in b.plan_step)
    for _ in range(3):
        x, y = O.make_batch(rng, cfg["vocab_size"], 2, 8, 0.1)
        la, lb = a.step(x, y), b.step(x, y)
        assert la == lb and a.grad_norm() == b.grad_norm()       # the same sums in the same order
        # the model's own reference: one pass over all gradients
        g = a.grads()
        total = np.sqrt(sum(float((v.astype(np.float64) ** 2).sum()) for v in g.values()))
        assert abs(a.grad_norm() - total) <= 1e-5 * total
    wa, wb = a.get_weights(), b.get_weights()
    assert all(np.array_equal(wa[n], wb[n]) for n in wa)
    assert a.state_dict()["_t"][0] == b.state_dict()["_t"][0] == 3.0
