"""Data parallel and ZeRO-1 on real GPUs (needs >= 2): one process per GPU, NCCL
bootstrap through the C ABI with the unique id ferried over a multiprocessing
queue, as the reference's harnesses do (engine/modal_ddp_test.py:54-107,
engine/modal_zero_test.py:96-142).  Gates: per-rank different data vs one GPU
on the concatenated batch (loss mean, gradients, weights after 3 steps);
replicated DP == ZeRO-1 bit for bit; graph replay with the side-stream
reductions captured; rendezvous timeout and bad arguments reported as codes."""
import ctypes
import multiprocessing as mp
import os
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CFG = dict(vocab_size=512, dim=256, n_layers=4, n_heads=4, n_kv_heads=2, mlp_hidden=384, tie_embeddings=True)
B, T, STEPS = 2, 128, 3


def _ngpu():
    if os.environ.get("AXIS_DP_CHILD"):      # spawned ranks must not touch CUDA before choosing their GPU
        return 0
    try:
        cu = ctypes.CDLL("libcuda.so.1")
        n = ctypes.c_int(0)
        return n.value if (cu.cuInit(0) == 0 and cu.cuDeviceGetCount(ctypes.byref(n)) == 0) else 0
    except OSError:
        return 0


def _data(rank, step):
    rng = np.random.default_rng(100 + rank + 10 * step)
    x = rng.integers(0, CFG["vocab_size"], size=(B, T)).astype(np.int64)
    return x, np.roll(x, -1, axis=1)


def _worker(rank, world, zero, dtype, graph, q_uid, q_out):
    os.environ["CUDA_VISIBLE_DEVICES"] = str(rank)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    sys.path.insert(0, ROOT)
    try:
        from axis_b200.compile import CompiledTransformer
        from oracle import step_numpy as O
        w0 = O.init_weights(CFG, seed=3)
        ct = CompiledTransformer(None, CFG, w0, B, T, dtype=dtype, grad_sync=True, zero_stage=1 if zero else 0,
                                 rank=rank, world=world, max_grad_norm=1.0, bucket_layers=2)
        if rank == 0:
            uid = ct.eng.nccl_id()
            for _ in range(world - 1):
                q_uid.put(uid)
        else:
            uid = q_uid.get(timeout=120)
        ct.eng.nccl_init(rank, world, uid, timeout_ms=120000)
        if graph:
            ct.capture()
        losses = []
        for s in range(STEPS):
            x, y = _data(rank, s)
            losses.append(ct.replay_step(x, y) if graph else ct.step(x, y))
        ct.gather_weights()      # ZeRO-1 gathers the updated compute weights at the start of the next step
        mirror = ct.eng.download_raw(ct.a_mirror, ct._P_total, np.uint16) if dtype == "bf16" else None
        q_out.put((rank, dict(losses=losses, owned=ct.owned, norm=ct.grad_norm(), w=ct.get_weights(),
                              g=ct.grads() if not zero else {}, mirror=mirror, status=ct.eng.device_status())))
        ct.eng.shutdown()
    except Exception as e:      # surface the failure to the parent instead of hanging it
        q_out.put((rank, dict(error=repr(e))))


def _run(world, zero, dtype, graph=False):
    ctx = mp.get_context("spawn")
    q_uid, q_out = ctx.Queue(), ctx.Queue()
    ps = [ctx.Process(target=_worker, args=(r, world, zero, dtype, graph, q_uid, q_out)) for r in range(world)]
    os.environ["AXIS_DP_CHILD"] = "1"
    try:
        for p in ps:
            p.start()
    finally:
        del os.environ["AXIS_DP_CHILD"]
    out = {}
    for _ in range(world):
        r, res = q_out.get(timeout=240)
        out[r] = res
    for p in ps:
        p.join(timeout=60)
    for r in range(world):
        assert "error" not in out[r], out[r]
    return [out[r] for r in range(world)]


needs2 = pytest.mark.skipif(_ngpu() < 2, reason="needs two GPUs")


@needs2
def test_dp_fp32_matches_single_gpu_on_concatenated_batch():
    from axis_b200.compile import CompiledTransformer
    from oracle import step_numpy as O
    dp = _run(2, False, "fp32")
    w0 = O.init_weights(CFG, seed=3)
    ct = CompiledTransformer(None, CFG, w0, 2 * B, T, dtype="fp32", max_grad_norm=1.0)
    for s in range(STEPS):
        xs, ys = zip(*[_data(r, s) for r in range(2)])
        loss = ct.step(np.concatenate(xs), np.concatenate(ys))
        assert abs(loss - np.mean([dp[r]["losses"][s] for r in range(2)])) < 1e-4
    ref_w, ref_g = ct.get_weights(), ct.grads()
    for r in range(2):
        assert dp[r]["status"] == 0
        for nm, w in dp[r]["w"].items():
            assert np.abs(w - ref_w[nm]).max() < 1e-4, nm
    for nm, g in dp[0]["g"].items():
        assert np.abs(g - ref_g[nm]).max() / (np.abs(ref_g[nm]).max() + 1e-9) < 1e-3, nm
    for nm in dp[0]["w"]:
        assert np.array_equal(dp[0]["w"][nm], dp[1]["w"][nm])            # replicas identical


@needs2
def test_zero1_equals_replicated_dp_bit_for_bit_and_under_graph_replay():
    dp = _run(2, False, "bf16")
    z = _run(2, True, "bf16")
    zg = _run(2, True, "bf16", graph=True)
    owned = [set(z[r]["owned"]) for r in range(2)]
    assert owned[0].isdisjoint(owned[1]) and len(owned[0] | owned[1]) == len(dp[0]["w"])
    for r in range(2):
        assert z[r]["losses"] == dp[r]["losses"] == zg[r]["losses"]
        for nm, w in z[r]["w"].items():
            assert np.array_equal(w, dp[0]["w"][nm]), nm
            assert np.array_equal(w, zg[r]["w"][nm]), nm
    assert np.array_equal(z[0]["mirror"], z[1]["mirror"])
    assert np.array_equal(z[0]["mirror"], dp[0]["mirror"])


def _timeout_worker(q):
    os.environ["CUDA_VISIBLE_DEVICES"] = "0"
    sys.path.insert(0, ROOT)
    from axis_b200.engine import Engine
    e = Engine()
    uid = e.nccl_id()
    res = {}
    for name, args in (("alone_in_world_2", (0, 2, uid, 1500)), ("bad_rank", (5, 2, uid, 1500))):
        try:
            e.nccl_init(*args)
            res[name] = "ok"
        except RuntimeError as ex:
            res[name] = str(ex)
    try:
        e.nccl_init(0, 1, b"short")
    except ValueError as ex:
        res["short_uid"] = str(ex)
    q.put(res)


def test_rendezvous_failures_are_reported_not_hung():
    """A rank whose peer never joins gets code 7 after the deadline; bad arguments are refused."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    p = ctx.Process(target=_timeout_worker, args=(q,))
    os.environ["AXIS_DP_CHILD"] = "1"
    try:
        p.start()
    finally:
        del os.environ["AXIS_DP_CHILD"]
    res = q.get(timeout=120)
    p.join(timeout=30)
    assert "rc=7" in res["alone_in_world_2"] and "timed out" in res["alone_in_world_2"]
    assert "rc=8" in res["bad_rank"]
    assert "128 bytes" in res["short_uid"]
