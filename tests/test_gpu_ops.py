"""Every op kind of the C ABI against numpy, through ctypes on a real GPU.

Reference kinds 0..31 are exercised with the argument roles the reference's
plan uses (axis/engine.py:43-73), including its quirks (alpha == 0 -> 1 in
GEMM, SCALE alpha == 0 = zero fill that never reads the source, fp32-encoded
ids/targets, 0 as the "none" sentinel).  Fused kinds (>= 32) are checked
against the oracle's pieces.  Sizes include ragged / unaligned cases."""
import numpy as np
import pytest

from axis_b200 import engine as E
from axis_b200.engine import Engine, op
from oracle import step_numpy as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def eng():
    e = Engine()
    e.alloc(4)          # slot 0 is reserved (the plan's cos table / "none" sentinel)
    yield e
    e.shutdown()


def put(eng, arr, dt=0):
    arr = np.ascontiguousarray(arr, dtype=np.float32)
    i = eng.alloc(max(arr.size, 1), 2 if dt == 1 else 4)
    if dt == 1:
        eng.upload_bf16(i, arr)
    else:
        eng.upload(i, arr)
    return i


def get(eng, i, shape, dt=0):
    return eng.download_bf16(i, shape) if dt == 1 else eng.download(i, shape)


def rnd(rng, shape, dt):
    a = rng.standard_normal(shape).astype(np.float32)
    return E.bf16_bits_to_f32(E.f32_to_bf16_bits(a)) if dt == 1 else a


def tol(dt):
    return 1.2e-2 if dt == 1 else 2e-5


def close(got, ref, dt, scale=None):
    s = np.abs(ref).max() + 1e-6 if scale is None else scale
    err = np.abs(got - ref).max() / s
    assert err <= tol(dt), err


@pytest.mark.parametrize("dt", [0, 1])
@pytest.mark.parametrize("n", [1, 7, 1024, 4099])
def test_binary_scale_copy_cast(eng, dt, n):
    rng = np.random.default_rng(n)
    a, b = rnd(rng, n, dt), rnd(rng, n, dt)
    ia, ib, ic = put(eng, a, dt), put(eng, b, dt), eng.alloc(n, 4)
    for kind, ref in ((E.ADD, a + b), (E.MUL, a * b), (E.SILU_MUL, a / (1 + np.exp(-a)) * b)):
        eng.run([op(kind, a=ia, b=ib, c=ic, n=n, dt=dt)])
        close(get(eng, ic, n, dt), ref, dt)
    eng.run([op(E.SCALE, a=ia, c=ic, n=n, dt=dt, alpha=0.5)])
    close(get(eng, ic, n, dt), a * 0.5, dt)
    # alpha == 0: explicit zero even when the source holds NaN
    inan = put(eng, np.full(n, np.nan), dt)
    eng.run([op(E.SCALE, a=inan, c=inan, n=n, dt=dt, alpha=0.0)])
    assert np.all(get(eng, inan, n, dt) == 0)
    eng.run([op(E.COPY, a=ia, c=ic, n=n, dt=dt)])
    assert np.array_equal(get(eng, ic, n, dt), a)
    if dt == 0:
        ih = eng.alloc(n, 2)
        eng.run([op(E.CAST, a=ia, c=ih, m=n, tb=0), op(E.CAST, a=ih, c=ic, m=n, tb=1)])
        assert np.array_equal(get(eng, ic, n), E.bf16_bits_to_f32(E.f32_to_bf16_bits(a)))


@pytest.mark.parametrize("dt", [0, 1])
@pytest.mark.parametrize("rows,dim", [(5, 48), (33, 256), (8, 1536), (3, 100),
                                      # wide rows (several warps per row); row counts that leave ragged last
                                      # groups and make blocks loop (more rows than one wave holds)
                                      (37, 2048), (9, 3072), (700, 4096), (2500, 4096), (11, 5120)])
def test_rmsnorm_fwd_bwd(eng, dt, rows, dim):
    rng = np.random.default_rng(rows * dim)
    x, w, g, res = rnd(rng, (rows, dim), dt), rnd(rng, dim, dt), rnd(rng, (rows, dim), dt), rnd(rng, (rows, dim), dt)
    ix, iw, ig, ir = put(eng, x, dt), put(eng, w, dt), put(eng, g, dt), put(eng, res, dt)
    iy, idx, itmp = eng.alloc(rows * dim), eng.alloc(rows * dim), eng.alloc(rows * dim)
    idw, iscr = eng.alloc(dim), eng.alloc(296 * dim)
    y, inv = O.rmsnorm_fwd(x, w, 1e-5)
    dx, dw = O.rmsnorm_bwd(x, w, inv, g)
    eng.run([op(E.RMSNORM, a=ix, b=iw, c=iy, m=rows, n=dim, dt=dt, alpha=1e-5)])
    close(get(eng, iy, (rows, dim), dt), y, dt)
    # reference two-op form
    eng.run([op(E.RMSNORM_BWD, a=ix, b=iw, d=ig, c=idx, tb=itmp, m=rows, n=dim, dt=dt, alpha=1e-5),
             op(E.COLSUM, a=itmp, c=idw, m=rows, n=dim, dt=2 if dt else 0)])
    close(get(eng, idx, (rows, dim), dt), dx, dt)
    close(eng.download(idw, dim), dw, dt, scale=np.abs(dw).max() + np.sqrt(rows) * 0.05 * dt)
    # fused form, with and without the residual, dw optional
    eng.run([op(E.RMSNORM_BWD_ACC, a=ix, b=iw, d=ig, c=idx, tb=ir, sa=idw, sb=iscr, m=rows, n=dim, dt=dt, alpha=1e-5)])
    close(get(eng, idx, (rows, dim), dt), dx + res, dt)
    close(eng.download(idw, dim), dw, 0 if dt == 0 else 1, scale=np.abs(dw).max())
    eng.run([op(E.RMSNORM_BWD_ACC, a=ix, b=iw, d=ig, c=idx, tb=0, sa=0, m=rows, n=dim, dt=dt, alpha=1e-5)])
    close(get(eng, idx, (rows, dim), dt), dx, dt)


@pytest.mark.parametrize("dt", [0, 1])
def test_perm_rope_repeat(eng, dt):
    rng = np.random.default_rng(1)
    B, T, H, KV, DH = 2, 17, 6, 2, 16
    x = rnd(rng, (B, T, H, DH), dt)
    ix, io = put(eng, x, dt), eng.alloc(x.size)
    eng.run([op(E.PERM_0213, a=ix, c=io, m=B, n=T, k=H, batch=DH, dt=dt)])
    assert np.array_equal(get(eng, io, (B, H, T, DH), dt), x.transpose(0, 2, 1, 3))
    x3 = rnd(rng, (B, T, H, 3), dt)          # odd inner size -> scalar path
    i3, o3 = put(eng, x3, dt), eng.alloc(x3.size)
    eng.run([op(E.PERM_0213, a=i3, c=o3, m=B, n=T, k=H, batch=3, dt=dt)])
    assert np.array_equal(get(eng, o3, (B, H, T, 3), dt), x3.transpose(0, 2, 1, 3))
    cos, sin = O.rope_tables(T, DH)
    ic, isn = put(eng, cos), put(eng, sin)
    xb = x.transpose(0, 2, 1, 3).copy()          # [B,H,T,DH]
    ib = put(eng, xb, dt)
    eng.run([op(E.ROPE, a=ib, b=ic, d=isn, c=io, batch=B * H, m=T, n=DH, dt=dt)])
    close(get(eng, io, xb.shape, dt), O.rope_fwd(xb, cos, sin), dt)
    eng.run([op(E.ROPE, a=ib, b=ic, d=isn, c=io, batch=B * H, m=T, n=DH, tb=1, dt=dt)])
    close(get(eng, io, xb.shape, dt), O.rope_bwd(xb, cos, sin), dt)
    # [B,T,H,DH] layout, in place, forward then inverse restores the input
    eng.run([op(E.ROPE_BTHD, a=ix, b=ic, d=isn, c=ix, batch=B, m=T, k=H, n=DH, dt=dt)])
    close(get(eng, ix, x.shape, dt), O.rope_fwd(xb, cos, sin).transpose(0, 2, 1, 3), dt)
    eng.run([op(E.ROPE_BTHD, a=ix, b=ic, d=isn, c=ix, batch=B, m=T, k=H, n=DH, tb=1, dt=dt)])
    close(get(eng, ix, x.shape, dt), x, dt)
    # a second tensor with its own head count in the same launch (query and key projections)
    xk = rnd(rng, (B, T, KV, DH), dt)
    ik = put(eng, xk, dt)
    eng.run([op(E.ROPE_BTHD, a=ix, b=ic, d=isn, c=ix, batch=B, m=T, k=H, n=DH, dt=dt, sa=ik, sb=ik, sc=KV)])
    close(get(eng, ix, x.shape, dt), O.rope_fwd(xb, cos, sin).transpose(0, 2, 1, 3), dt)
    close(get(eng, ik, xk.shape, dt), O.rope_fwd(xk.transpose(0, 2, 1, 3), cos, sin).transpose(0, 2, 1, 3), dt)
    eng.run([op(E.ROPE_BTHD, a=ix, b=ic, d=isn, c=ix, batch=B, m=T, k=H, n=DH, tb=1, dt=dt, sa=ik, sb=ik, sc=KV)])
    close(get(eng, ix, x.shape, dt), x, dt)
    close(get(eng, ik, xk.shape, dt), xk, dt)
    # head_dim 6: scalar rotary path
    x6 = rnd(rng, (B, 2, T, 6), dt)
    c6, s6 = O.rope_tables(T, 6)
    i6, o6 = put(eng, x6, dt), eng.alloc(x6.size)
    eng.run([op(E.ROPE, a=i6, b=put(eng, c6), d=put(eng, s6), c=o6, batch=B * 2, m=T, n=6, dt=dt)])
    close(get(eng, o6, x6.shape, dt), O.rope_fwd(x6, c6, s6), dt)
    # grouped repeat and its group-sum backward
    kv = rnd(rng, (B, KV, T, DH), dt)
    ikv, ibig = put(eng, kv, dt), eng.alloc(B * H * T * DH)
    eng.run([op(E.REPEAT_KV, a=ikv, c=ibig, batch=B, tb=KV, n=H, m=T, k=DH, dt=dt)])
    assert np.array_equal(get(eng, ibig, (B, H, T, DH), dt), np.repeat(kv, H // KV, axis=1))
    eng.run([op(E.REPEAT_KV_BWD, a=ib, c=ikv, batch=B, tb=KV, n=H, m=T, k=DH, dt=dt)])
    close(get(eng, ikv, kv.shape, dt), xb.reshape(B, KV, H // KV, T, DH).sum(2), dt)


@pytest.mark.parametrize("dt", [0, 1])
def test_softmax_pair_silu_bwd_rowdot(eng, dt):
    rng = np.random.default_rng(2)
    batch, qt, kl, qoff = 3, 8, 24, 16
    s = rnd(rng, (batch, qt, kl), dt)
    i_s, i_p = put(eng, s, dt), eng.alloc(s.size)
    eng.run([op(E.SOFTMAX_CAUSAL, a=i_s, c=i_p, batch=batch, m=qt, n=kl, k=qoff, dt=dt)])
    ref = np.zeros_like(s)
    for r in range(qt):
        t = min(qoff + r, kl - 1)
        e = np.exp(s[:, r, :t + 1] - s[:, r, :t + 1].max(-1, keepdims=True))
        ref[:, r, :t + 1] = e / e.sum(-1, keepdims=True)
    close(get(eng, i_p, s.shape, dt), ref, dt)
    dp = rnd(rng, s.shape, dt)
    p = E.bf16_bits_to_f32(E.f32_to_bf16_bits(ref)) if dt else ref
    i_pp, i_dp, i_ds = put(eng, p, dt), put(eng, dp, dt), eng.alloc(s.size)
    eng.run([op(E.SOFTMAX_BWD, a=i_pp, b=i_dp, c=i_ds, batch=batch, m=qt, n=kl, dt=dt)])
    close(get(eng, i_ds, s.shape, dt), p * (dp - (dp * p).sum(-1, keepdims=True)), dt)
    n = 1000
    g, u, gr = rnd(rng, n, dt), rnd(rng, n, dt), rnd(rng, n, dt)
    ig, iu, igr, idg, idu = put(eng, g, dt), put(eng, u, dt), put(eng, gr, dt), eng.alloc(n), eng.alloc(n)
    eng.run([op(E.SILU_BWD, a=ig, b=iu, d=igr, c=idg, tb=idu, n=n, dt=dt)])
    dg, du = O.silu_mul_bwd(g, u, 1 / (1 + np.exp(-g)), gr)
    close(get(eng, idg, n, dt), dg, dt)
    close(get(eng, idu, n, dt), du, dt)
    a, b = rnd(rng, (37, 48), dt), rnd(rng, (37, 48), dt)
    ic = eng.alloc(37)
    eng.run([op(E.ROWDOT, a=put(eng, a, dt), b=put(eng, b, dt), c=ic, m=37, n=48, dt=dt)])
    close(eng.download(ic, 37), (a * b).sum(-1), 0)


@pytest.mark.parametrize("dt", [0, 1])
def test_embedding_and_cross_entropy(eng, dt):
    rng = np.random.default_rng(3)
    N, V, D = 50, 97, 24
    table = rnd(rng, (V, D), dt)
    ids = rng.integers(0, V, N)
    ids[7] = ids[3]; ids[40] = ids[3]                     # repeated tokens
    tgt = rng.integers(0, V, N)
    tgt[[1, 5, 6]] = -1
    it, iidf, io = put(eng, table, dt), put(eng, ids.astype(np.float32)), eng.alloc(N * D)
    eng.run([op(E.EMBED, a=it, b=iidf, c=io, m=N, n=D, dt=dt)])
    assert np.array_equal(get(eng, io, (N, D), dt), table[ids])
    iid = eng.alloc(N); eng.upload_tokens(iid, ids, V)
    eng.run([op(E.EMBED_I32, a=it, b=iid, c=io, m=N, n=D, dt=dt)])
    assert np.array_equal(get(eng, io, (N, D), dt), table[ids])
    g = rnd(rng, (N, D), dt)
    ig = put(eng, g, dt)
    ref = O.embedding_bwd(ids, g, V)
    base = rng.standard_normal((V, D)).astype(np.float32)
    idT = put(eng, base)
    eng.run([op(E.EMBED_BWD, a=ig, b=iidf, c=idT, m=N, n=D, dt=2 if dt else 0)])
    close(eng.download(idT, (V, D)), base + ref, 0)
    eng.upload(idT, base)
    eng.run([op(E.EMBED_BWD_DET, a=ig, b=iid, c=idT, m=N, n=D, dt=dt)])
    got1 = eng.download(idT, (V, D))
    close(got1, base + ref, 0)
    eng.upload(idT, base)
    eng.run([op(E.EMBED_BWD_DET, a=ig, b=iid, c=idT, m=N, n=D, dt=dt)])
    assert np.array_equal(got1, eng.download(idT, (V, D)))          # run-to-run identical
    # cross-entropy, reference form: zero loss/denom, count, CE
    logits = rnd(rng, (N, V), dt) * 4          # a power of two keeps bf16 values exact
    il, itf, idl = put(eng, logits, dt), put(eng, tgt.astype(np.float32)), eng.alloc(N * V)
    iloss, iden = eng.alloc(1), eng.alloc(1)
    loss, dl, cnt = O.cross_entropy_fwd_bwd(logits, tgt, -1)
    eng.run([op(E.SCALE, a=iloss, c=iloss, n=1, alpha=0.0), op(E.SCALE, a=iden, c=iden, n=1, alpha=0.0),
             op(E.COUNTVALID, a=itf, c=iden, m=N),
             op(E.CE, a=il, b=itf, c=idl, d=iloss, sa=iden, m=N, n=V, dt=dt)])
    assert eng.download(iden, 1)[0] == cnt == 47
    assert abs(eng.download(iloss, 1)[0] - loss) <= 1e-5 * abs(loss)
    close(get(eng, idl, (N, V), dt), dl, dt)
    # sa = 0: mean over all N rows
    eng.run([op(E.SCALE, a=iloss, c=iloss, n=1, alpha=0.0),
             op(E.CE, a=il, b=itf, c=idl, d=iloss, sa=0, m=N, n=V, dt=dt)])
    assert abs(eng.download(iloss, 1)[0] - loss * cnt / N) <= 1e-5 * abs(loss)
    # fused form: int32 targets, in place, count + loss produced by the op
    itg = eng.alloc(N); eng.upload_tokens(itg, tgt, V)
    iscr = eng.alloc(N + 8)
    eng.run([op(E.CE_FUSED, a=il, b=itg, c=il, d=iloss, sa=iden, sb=iscr, m=N, n=V, dt=dt)])
    assert eng.download(iden, 1)[0] == cnt
    assert abs(eng.download(iloss, 1)[0] - loss) <= 1e-5 * abs(loss)
    close(get(eng, il, (N, V), dt), dl, dt)
    assert np.all(get(eng, il, (N, V), dt)[[1, 5, 6]] == 0)


def test_adamw_clip_tick_per_tensor_and_flat(eng):
    rng = np.random.default_rng(4)
    n = 3 * 1024
    p0, g = rng.standard_normal(n).astype(np.float32), (rng.standard_normal(n) * 3).astype(np.float32)
    lr, wd, eps, mx = 1e-3, 0.1, 1e-8, 1.0
    # numpy reference of two steps with clipping
    def ref_steps(decay_mask):
        p, m, v = p0.copy(), np.zeros(n, np.float32), np.zeros(n, np.float32)
        tot = np.sqrt(float((g.astype(np.float64) ** 2).sum()))
        sc = mx / tot if tot > mx else 1.0
        for t in (1, 2):
            gi = g * np.float32(sc)
            m = 0.9 * m + np.float32(0.1) * gi
            v = 0.95 * v + np.float32(0.05) * gi * gi
            p = p * np.where(decay_mask, np.float32(1 - lr * wd), np.float32(1)) \
                - np.float32(lr) * (m / (1 - 0.9 ** t)) / (np.sqrt(v / (1 - 0.95 ** t)) + eps)
        return p.astype(np.float32), tot
    ip, ig, im, iv = put(eng, p0), put(eng, g), put(eng, np.zeros(n)), put(eng, np.zeros(n))
    it, ilr, iacc, isc, ibf = put(eng, np.zeros(1)), put(eng, np.array([lr])), eng.alloc(1), eng.alloc(1), eng.alloc(n, 2)
    plan = [op(E.SCALE, a=iacc, c=iacc, n=1, alpha=0.0), op(E.L2ACC, a=ig, c=iacc, n=n),
            op(E.CLIPSCALE, a=iacc, c=isc, alpha=mx), op(E.TICK, a=it),
            op(E.ADAMW, a=ip, b=ig, c=im, d=iv, tb=it, sa=ibf, sb=ilr, oa=isc, n=n, alpha=lr, beta=wd, gamma=eps)]
    eng.run(plan); eng.run(plan)
    ref, tot = ref_steps(np.ones(n, bool))
    assert np.abs(eng.download(ip, n) - ref).max() <= 2e-6
    assert abs(np.sqrt(eng.download(iacc, 1)[0]) - tot) <= 1e-4 * tot
    assert eng.download(it, 1)[0] == 2.0
    assert np.array_equal(eng.download_bf16(ibf, n), E.bf16_bits_to_f32(E.f32_to_bf16_bits(eng.download(ip, n))))
    # host-folded form (tb = -1, no lr buffer, no scale buffer)
    ip2, im2, iv2 = put(eng, p0), put(eng, np.zeros(n)), put(eng, np.zeros(n))
    a_lr = lr * np.sqrt(1 - 0.95) / (1 - 0.9)
    eng.run([op(E.ADAMW, a=ip2, b=ig, c=im2, d=iv2, tb=-1, n=n, alpha=a_lr, beta=0.0, gamma=eps * np.sqrt(0.05))])
    m1 = 0.1 * g; v1 = 0.05 * g * g
    assert np.abs(eng.download(ip2, n) - (p0 - lr * (m1 / 0.1) / (np.sqrt(v1 / 0.05) + eps))).max() <= 2e-6
    # flat arena: decay flags per 1024-chunk (middle chunk exempt), segment offset
    flags = np.array([1, 0, 1], np.uint8)
    ifl = eng.alloc(4, 1); eng.upload_raw(ifl, flags)
    ip3, im3, iv3 = put(eng, p0), eng.alloc_zero(n * 4), eng.alloc_zero(n * 4)
    it3, ipart, iss, ign, ibf3 = put(eng, np.zeros(1)), eng.alloc(8), eng.alloc(2), eng.alloc(1), eng.alloc(n, 2)
    plan = [op(E.GNORM_FLAT, a=ig, c=ipart, d=iss, ob=0, m=3, oa=0, tb=it3),
            op(E.ADAMW_FLAT, a=ip3, b=ig, c=im3, d=iv3, m=3, k=0, sa=ibf3, sb=ilr, tb=it3, sc=ifl, oa=iss, ob=1,
               oc=ign, alpha=mx, beta=wd, gamma=eps)]
    eng.run(plan); eng.run(plan)
    ref3, tot = ref_steps(np.repeat(flags, 1024).astype(bool))
    assert np.abs(eng.download(ip3, n) - ref3).max() <= 2e-6
    assert abs(eng.download(ign, 1)[0] - tot) <= 1e-5 * tot
    assert np.array_equal(eng.download_bf16(ibf3, n), E.bf16_bits_to_f32(E.f32_to_bf16_bits(eng.download(ip3, n))))


def test_error_codes_and_validation(eng):
    with pytest.raises(RuntimeError, match="rc=1000"):
        eng.run([op(99)])
    a = eng.alloc(16)
    with pytest.raises(RuntimeError, match="rc=1001"):
        eng.run([op(E.SCALE, a=a, c=a, n=16, alpha=0.0), op(E.ADD, a=a, b=a, c=a, n=17)])   # past the end
    with pytest.raises(RuntimeError, match="rc=1000"):
        eng.run([op(E.ADD, a=a, b=60000, c=a, n=4)])                                       # missing buffer
    with pytest.raises(RuntimeError):
        eng.run([op(E.ALLREDUCE, a=a, n=16)])                                              # no communicator
    with pytest.raises(RuntimeError, match="rc=1000"):
        eng.run([op(E.FLASH, a=a, b=a, d=a, c=a, m=4, n=24, k=1, batch=1, tb=1, dt=1, alpha=1.0)])  # head_dim % 16
    with pytest.raises(RuntimeError):
        eng.replay(1)                                                                      # nothing captured yet
    assert eng.device_status() == 0


def test_graph_capture_replay_counts(eng):
    n = 4096
    a = put(eng, np.ones(n))
    eng.capture([op(E.ADD, a=a, b=a, c=a, n=n)])
    eng.replay(3)
    assert np.all(eng.download(a, n) == 8.0)
    before = eng.launch_count(reset=True)
    eng.replay(2)
    assert eng.launch_count() == 2 and before >= 3


@pytest.mark.parametrize("dt", [0, 1])
@pytest.mark.parametrize("dim", [256, 1536, 4096])
def test_rmsnorm_deferred_dw_and_batched_column_sum(eng, dt, dim):
    """Three RMSNorm backward launches leave their per-block partial sums in consecutive zeroed scratch areas
    (oa = 1, 2, 3); one COLSUM_BATCH over areas 1..2 and one over area 0 give the same dw, bit for bit, as the
    immediate form, at offsets of an fp32 arena taken from a device table."""
    rng = np.random.default_rng(dim + dt)
    unit = 1024
    rows = [40, 700, 9]
    arena = eng.alloc_zero(4 * 8 * 4096)
    offs = np.array([4, 0, 8], dtype=np.int32)                 # in units of `unit` elements; disjoint for dim <= 4096
    table = eng.alloc(4)
    eng.upload_raw(table, offs)
    scratch = eng.alloc_zero(3 * 296 * dim * 4)
    one = eng.alloc(296 * dim)
    want, plan = [], []
    for j, r in enumerate(rows):
        x, w, g = rnd(rng, (r, dim), dt), rnd(rng, dim, dt), rnd(rng, (r, dim), dt)
        ix, iw, ig = put(eng, x, dt), put(eng, w, dt), put(eng, g, dt)
        idx, idw = eng.alloc(r * dim), eng.alloc(dim)
        eng.run([op(E.RMSNORM_BWD_ACC, a=ix, b=iw, d=ig, c=idx, tb=0, sa=idw, sb=one, m=r, n=dim, dt=dt, alpha=1e-5)])
        want.append((eng.download(idw, dim), get(eng, idx, (r, dim), dt)))
        plan.append(op(E.RMSNORM_BWD_ACC, a=ix, b=iw, d=ig, c=idx, tb=0, sa=idw, sb=scratch, oa=j + 1, m=r, n=dim,
                       dt=dt, alpha=1e-5))
        eng.run([op(E.SCALE, a=idw, c=idw, n=dim, alpha=0.0)])
    plan += [op(E.COLSUM_BATCH, a=scratch, b=table, c=arena, m=2, n=dim, oa=1, k=unit),
             op(E.COLSUM_BATCH, a=scratch, b=table, c=arena, m=1, n=dim, oa=0, k=unit)]
    for _ in range(2):                                          # a second pass over the same areas
        eng.run(plan)
        got = eng.download(arena, 8 * 4096)
        for j in range(3):
            o = int(offs[j]) * unit
            assert np.array_equal(got[o:o + dim], want[j][0]), j
    assert eng.device_status() == 0
    # a destination outside the arena is skipped and reported
    eng.upload_raw(table, np.array([10 ** 6, 0, 0], dtype=np.int32))
    eng.run([op(E.COLSUM_BATCH, a=scratch, b=table, c=arena, m=1, n=dim, oa=0, k=unit)])
    assert eng.device_status(clear=True) == 130
    assert eng.device_status() == 0


@pytest.mark.parametrize("dt", [0, 1])
def test_out_of_range_ids_and_targets_are_skipped_with_a_status(eng, dt):
    """An id or target that lies inside its int/float buffer but outside the table / vocabulary never reaches
    memory: the row is skipped (gather: zero-filled) and the device status word carries a code."""
    rng = np.random.default_rng(7)
    N, V, D = 12, 20, 16
    table = rnd(rng, (V, D), dt)
    ids = rng.integers(0, V, N)
    bad = ids.copy(); bad[5] = V + 3
    it, io = put(eng, table, dt), eng.alloc(N * D, 2 if dt else 4)
    assert eng.device_status() == 0
    # gather through the reference ABI's fp32-encoded ids
    eng.run([op(E.EMBED, a=it, b=put(eng, bad.astype(np.float32)), c=io, m=N, n=D, dt=dt)])
    out = get(eng, io, (N, D), dt)
    assert eng.device_status() == 0x401
    ok = np.arange(N) != 5
    assert np.array_equal(out[ok], table[ids][ok]) and np.all(out[5] == 0)
    # scatter-add, both forms: the bad row adds nothing anywhere
    g = rnd(rng, (N, D), dt)
    ref = O.embedding_bwd(ids[ok], g[ok], V)
    # the table gradient is a window of V rows at the front of a larger buffer: a wild write would land behind it
    ig, ipar = put(eng, g, dt), eng.alloc(V * D + 64)
    idT = eng.view(ipar, 0, V * D * 4)
    iid = eng.alloc(N); eng.upload_raw(iid, bad.astype(np.int32))
    for form in ("det", "atomic"):
        eng.run([op(E.SCALE, a=ipar, c=ipar, n=V * D + 64, alpha=0.0)])
        if form == "det":
            eng.run([op(E.EMBED_BWD_DET, a=ig, b=iid, c=idT, m=N, n=D, dt=dt)])
        else:
            eng.run([op(E.EMBED_BWD, a=ig, b=put(eng, bad.astype(np.float32)), c=idT, m=N, n=D, dt=2 if dt else 0)])
        full = eng.download(ipar, V * D + 64)
        assert eng.device_status() == 0x402
        assert np.all(full[V * D:] == 0)
        close(full[:V * D].reshape(V, D), ref, 0)
    # cross-entropy: a target >= V counts as ignored and is reported
    logits = rnd(rng, (N, V), dt)
    tgt = rng.integers(0, V, N); tgt[3] = -1
    tbad = tgt.copy(); tbad[8] = V + 1
    tref = tgt.copy(); tref[8] = -1
    loss, dl, cnt = O.cross_entropy_fwd_bwd(logits, tref, -1)
    il, itg = put(eng, logits, dt), eng.alloc(N)
    eng.upload_raw(itg, tbad.astype(np.int32))
    iloss, iden, iscr = eng.alloc(1), eng.alloc(1), eng.alloc(N + 8)
    eng.run([op(E.CE_FUSED, a=il, b=itg, c=il, d=iloss, sa=iden, sb=iscr, m=N, n=V, dt=dt)])
    assert eng.device_status() == 0x403
    assert eng.download(iden, 1)[0] == cnt
    assert abs(eng.download(iloss, 1)[0] - loss) <= 1e-5 * abs(loss)
    close(get(eng, il, (N, V), dt), dl, dt)


def test_gemm_rejects_negative_offsets_and_strides(eng):
    a, b, c = eng.alloc(64), eng.alloc(64), eng.alloc(64)
    for bad in (dict(oa=-8), dict(ob=-1), dict(oc=-4), dict(batch=2, sa=-16, sb=0, sc=0)):
        kw = dict(a=a, b=b, c=c, m=4, n=4, k=4, batch=1)
        kw.update(bad)
        with pytest.raises(RuntimeError, match="rc=1000"):
            eng.run([op(E.GEMM_SB, **kw)])
