"""Data-parallel / ZeRO-1 lowering on CPU: two gloo ranks run the plan
interpreter with real collectives.  Mirrors the reference's distributed gates
(engine/modal_ddp_test.py:130-188, engine/modal_zero_test.py:96-142): different
data per rank vs one process on the concatenated batch, and replicated DP vs
ZeRO-1 equality (bit-exact here)."""
import json
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
G = os.path.join(os.path.dirname(__file__), "golden")

CFG = dict(vocab_size=61, dim=32, n_layers=3, n_heads=4, n_kv_heads=2, mlp_hidden=40, tie_embeddings=True)
B, T, STEPS = 2, 8, 3


def _data(rank, step):
    rng = np.random.default_rng(100 + rank + 10 * step)
    x = rng.integers(0, CFG["vocab_size"], size=(B, T)).astype(np.int64)
    return x, np.roll(x, -1, axis=1)


def _worker(rank, world, port, zero, dtype, recompute, out, resume_at=0):
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    from axis_b200.compile import CompiledTransformer
    from oracle import step_numpy as O
    from tests.plan_interp import InterpEngine
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    w0 = O.init_weights(CFG, seed=3)
    ct = CompiledTransformer(InterpEngine(dist), CFG, w0, B, T, dtype=dtype, grad_sync=True,
                             zero_stage=1 if zero else 0, rank=rank, world=world, max_grad_norm=1.0,
                             bucket_layers=2, recompute_blocks=recompute)
    losses = []
    for s in range(STEPS):
        if resume_at and s == resume_at:
            # save, rebuild from OTHER initial weights, load: the next step must continue the uninterrupted run
            st = ct.state_dict()
            ct = CompiledTransformer(InterpEngine(dist), CFG, O.init_weights(CFG, seed=4), B, T, dtype=dtype,
                                     grad_sync=True, zero_stage=1 if zero else 0, rank=rank, world=world,
                                     max_grad_norm=1.0, bucket_layers=2, recompute_blocks=recompute)
            ct.load_state_dict(st)
        losses.append(ct.step(*_data(rank, s)))
    ct.gather_weights()          # ZeRO-1 gathers the updated compute weights at the start of the NEXT step
    res = {"losses": losses, "owned": ct.owned, "norm": ct.grad_norm(),
           "w": ct.get_weights(), "g": ct.grads() if not zero else {},
           "mirror": ct.eng.bufs[ct.a_mirror].copy() if dtype == "bf16" else None,
           "trace": ct.eng.trace[:]}
    out[rank] = res
    dist.barrier()
    dist.destroy_process_group()


def _run(world, zero, dtype, recompute=False, resume_at=0):
    import torch.multiprocessing as mp
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(world, port, zero, dtype, recompute, out, resume_at), nprocs=world, join=True)
    return [out[r] for r in range(world)]


@pytest.fixture(scope="module")
def runs():
    return {"dp32": _run(2, False, "fp32"), "dp16": _run(2, False, "bf16"), "z16": _run(2, True, "bf16"),
            "z16rc": _run(2, True, "bf16", recompute=True), "z16resume": _run(2, True, "bf16", resume_at=2)}


def test_dp_matches_single_process_on_concatenated_batch(runs):
    from axis_b200.compile import CompiledTransformer
    from oracle import step_numpy as O
    from tests.plan_interp import InterpEngine
    w0 = O.init_weights(CFG, seed=3)
    ct = CompiledTransformer(InterpEngine(), CFG, w0, 2 * B, T, dtype="fp32", max_grad_norm=1.0)
    for s in range(STEPS):
        xs, ys = zip(*[_data(r, s) for r in range(2)])
        loss = ct.step(np.concatenate(xs), np.concatenate(ys))
        mean = np.mean([runs["dp32"][r]["losses"][s] for r in range(2)])
        assert abs(loss - mean) < 1e-5
    ref_w = ct.get_weights()
    for r in range(2):
        for nm, w in runs["dp32"][r]["w"].items():
            assert np.abs(w - ref_w[nm]).max() < 1e-5, nm
    ref_g = ct.grads()
    for nm, g in runs["dp32"][0]["g"].items():
        assert np.abs(g - ref_g[nm]).max() / (np.abs(ref_g[nm]).max() + 1e-9) < 1e-4, nm


def test_replicas_stay_identical(runs):
    a, b = runs["dp32"]
    for nm in a["w"]:
        assert np.array_equal(a["w"][nm], b["w"][nm])
    assert a["norm"] == b["norm"]


def test_zero1_equals_replicated_dp_bit_for_bit(runs):
    dp, z = runs["dp16"], runs["z16"]
    owned = [set(z[r]["owned"]) for r in range(2)]
    assert owned[0].isdisjoint(owned[1]) and len(owned[0] | owned[1]) == len(dp[0]["w"])
    for r in range(2):
        assert z[r]["losses"] == dp[r]["losses"]
        for nm, w in z[r]["w"].items():
            assert np.array_equal(w, dp[0]["w"][nm]), nm
    # every rank holds the full bf16 model after the owners' broadcast
    assert np.array_equal(z[0]["mirror"], z[1]["mirror"])
    assert np.array_equal(z[0]["mirror"], dp[0]["mirror"])


def test_zero_owner_map_follows_reference_greedy(runs):
    from oracle import step_numpy as O
    w0 = O.init_weights(CFG, seed=3)
    names = O.base_param_names(CFG["n_layers"], True)
    owner, _ = O.zero_ownership(names, {k: v.shape for k, v in w0.items()}, 2)
    for r in range(2):
        assert runs["z16"][r]["owned"] == [n for n in names if owner[n] == r]


def test_reduction_is_bucketed_inside_backward(runs):
    from axis_b200 import engine as E
    tr = runs["dp32"][0]["trace"]
    n = tr.index(E.GNORM_FLAT)
    first = tr[:n]
    red = [i for i, k in enumerate(first) if k == E.REDUCE]
    gemm_after_first_reduce = [i for i, k in enumerate(first) if k == E.GEMM_SB and i > red[0]]
    assert len(red) >= 3 and gemm_after_first_reduce, "reductions must be interleaved with backward GEMMs"
    # every reduction group forks the collectives stream off the main chain; stream switches come in pairs
    # (collectives and the side stream of the weight-gradient GEMMs); the main chain joins at the end
    assert first.count(E.FORK) >= 3 and first.count(E.STREAM) % 2 == 0 and first[-1] == E.JOIN
    assert first.count(E.EVENT) > 0


def test_zero1_with_block_recompute_equals_zero1_bit_for_bit(runs):
    """Per-block recompute re-runs forward ops inside the backward; the bucket boundaries of the overlapped
    reduction move with them and the result does not change."""
    from axis_b200 import engine as E
    z, rc = runs["z16"], runs["z16rc"]
    for r in range(2):
        assert rc[r]["losses"] == z[r]["losses"] and rc[r]["owned"] == z[r]["owned"]
        for nm, w in z[r]["w"].items():
            assert np.array_equal(w, rc[r]["w"][nm]), nm
        assert np.array_equal(z[r]["mirror"], rc[r]["mirror"])
        step0 = lambda tr: tr[:tr.index(E.GNORM_FLAT)]
        assert step0(rc[r]["trace"]).count(E.REDUCE) == step0(z[r]["trace"]).count(E.REDUCE)
        assert step0(rc[r]["trace"]).count(E.ATTN_FWD) == 2 * CFG["n_layers"] - 1


def test_zero1_resume_continues_the_run_bit_for_bit(runs):
    """state_dict -> a freshly built step (other initial weights) -> load_state_dict under ZeRO-1: the owners
    re-publish their bf16 segments, so the step after the resume equals the uninterrupted run's on every rank
    (engine/modal_zero_test.py:124-131 checks the saved shards; the reference's load leaves the non-owned
    mirrors stale)."""
    z, rs = runs["z16"], runs["z16resume"]
    for r in range(2):
        assert rs[r]["losses"] == z[r]["losses"]
        for nm, w in z[r]["w"].items():
            assert np.array_equal(w, rs[r]["w"][nm]), nm
        assert np.array_equal(z[r]["mirror"], rs[r]["mirror"])


def test_zero1_gathers_the_weights_at_the_start_of_the_step(runs):
    """ZeRO-1: the owners' bf16 segments are broadcast before the first forward kernel of a step (one event per
    bucket, waited for just before the bucket's first use) and nothing follows the optimizer on the main chain."""
    from axis_b200 import engine as E
    tr = runs["z16"][0]["trace"]
    end = tr.index(E.ADAMW_FLAT)
    step0 = tr[:end + 1]
    assert step0.index(E.BROADCAST) < step0.index(E.EMBED_I32)
    first_gemm = min(step0.index(k) for k in (E.GEMM_GROUP, E.GEMM_SB) if k in step0)
    assert step0[:first_gemm].count(E.BROADCAST) == step0.count(E.BROADCAST) > 0
    nxt = tr[end + 1:]
    assert nxt[0] == E.FORK and E.BROADCAST in nxt[:8]          # the next step opens with the gather, not this one's tail
