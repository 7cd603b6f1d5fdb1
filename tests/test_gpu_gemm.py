"""GEMM op (kinds GEMM / GEMM_SB / GEMM_EX) on the GPU against numpy: the three
operand layouts the plan uses (tb 0/1/2, axis/engine.py:47), fp32 and bf16
storage, bf16-in/fp32-out weight gradients, alpha/beta epilogues, offsets and
strided batches, tile tails, and tensor-core path vs general path agreement."""
import numpy as np
import pytest

from axis_b200 import engine as E
from axis_b200.engine import Engine, op
from oracle import step_numpy as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def eng():
    e = Engine()
    e.alloc(4)
    yield e
    e.shutdown()


def bf(a):
    return E.bf16_bits_to_f32(E.f32_to_bf16_bits(a))


def put(eng, arr, dt):
    i = eng.alloc(arr.size, 2 if dt else 4)
    eng.upload_bf16(i, arr) if dt else eng.upload(i, arr)
    return i


def run_gemm(eng, rng, m, n, k, tb, dt, alpha=0.0, beta=0.0, addend=False, fallback=0):
    in_bf, out_bf = dt >= 1, dt == 1
    sha = (k, m) if tb == 2 else (m, k)
    shb = (n, k) if tb == 1 else (k, n)
    A = rng.standard_normal(sha).astype(np.float32)
    B = rng.standard_normal(shb).astype(np.float32)
    C0 = rng.standard_normal((m, n)).astype(np.float32)
    if in_bf:
        A, B = bf(A), bf(B)
    if out_bf:
        C0 = bf(C0)
    ia, ib = put(eng, A, in_bf), put(eng, B, in_bf)
    ic = put(eng, C0, out_bf)
    idd = put(eng, C0, out_bf) if addend else -1
    if addend:
        eng.upload_bf16(ic, np.zeros((m, n), np.float32)) if out_bf else eng.upload(ic, np.zeros((m, n), np.float32))
    eng.set_fallback(fallback)
    kind = E.GEMM_EX if addend else E.GEMM_SB
    eng.run([op(kind, a=ia, b=ib, c=ic, d=idd, m=m, n=n, k=k, batch=1, tb=tb, dt=dt, alpha=alpha, beta=beta)])
    eng.set_fallback(0)
    got = eng.download_bf16(ic, (m, n)) if out_bf else eng.download(ic, (m, n))
    Aop = A.T if tb == 2 else A
    Bop = B.T if tb == 1 else B
    ref = (alpha if alpha != 0.0 else 1.0) * (Aop.astype(np.float64) @ Bop.astype(np.float64)) + beta * C0
    return got, ref.astype(np.float32)


def check(got, ref, out_bf, k):
    scale = np.abs(ref).max() + 1e-6
    err = np.abs(got - ref).max() / scale
    lim = 6e-3 if out_bf else 3e-6 * max(1.0, np.sqrt(k) / 4)
    assert err <= lim, (err, lim)


@pytest.mark.parametrize("tb", [0, 1, 2])
@pytest.mark.parametrize("m,n,k", [(1, 1, 1), (5, 7, 3), (64, 64, 16), (100, 130, 70), (257, 96, 33)])
def test_fp32_gemm_is_true_fp32(eng, tb, m, n, k):
    rng = np.random.default_rng(m * n + k)
    got, ref = run_gemm(eng, rng, m, n, k, tb, 0)
    check(got, ref, False, k)
    got, ref = run_gemm(eng, rng, m, n, k, tb, 0, alpha=0.5, beta=1.0)
    check(got, ref, False, k)


@pytest.mark.parametrize("tb", [0, 1, 2])
@pytest.mark.parametrize("dt", [1, 2])
@pytest.mark.parametrize("m,n,k", [(128, 128, 64), (256, 256, 128), (384, 512, 192), (200, 136, 72),
                                   (128, 264, 1000), (1000, 128, 64)])
def test_bf16_tensor_core_gemm(eng, tb, dt, m, n, k):
    if tb == 2 and m % 8:
        pytest.skip("M-major operand needs m % 8 == 0 for the TMA path")
    rng = np.random.default_rng(m + n + k + tb)
    got, ref = run_gemm(eng, rng, m, n, k, tb, dt)
    check(got, ref, dt == 1, k)
    assert eng.device_status() == 0


@pytest.mark.parametrize("tb", [0, 1, 2])
def test_bf16_epilogues_and_addend(eng, tb):
    rng = np.random.default_rng(tb)
    for dt in (1, 2):
        got, ref = run_gemm(eng, rng, 256, 384, 128, tb, dt, alpha=2.0, beta=1.0)
        check(got, ref, dt == 1, 128)
        got, ref = run_gemm(eng, rng, 256, 384, 128, tb, dt, beta=1.0, addend=True)
        check(got, ref, dt == 1, 128)


@pytest.mark.parametrize("tb", [0, 1, 2])
@pytest.mark.parametrize("dt", [1, 2])
@pytest.mark.parametrize("m,n,k", [(520, 776, 320), (256, 264, 64), (1032, 256, 2112)])
def test_paired_kernel_staged_output(eng, tb, dt, m, n, k):
    """Paired-CTA kernel forced (mask 8): output pieces staged in shared memory and written by TMA
    stores clipped at ragged edges; in-place accumulation and a separate addend arrive by TMA loads;
    the long-k shape also runs the split-K workspace through the same stores."""
    rng = np.random.default_rng(m + n + k + tb + dt)
    got, ref = run_gemm(eng, rng, m, n, k, tb, dt, fallback=8)
    check(got, ref, dt == 1, k)
    got, ref = run_gemm(eng, rng, m, n, k, tb, dt, alpha=0.5, beta=1.0, fallback=8)
    check(got, ref, dt == 1, k)
    got, ref = run_gemm(eng, rng, m, n, k, tb, dt, beta=-2.0, addend=True, fallback=8)
    check(got, ref, dt == 1, k)
    assert eng.device_status() == 0


@pytest.mark.parametrize("tb", [0, 1, 2])
def test_tensor_core_and_general_path_agree(eng, tb):
    for dt in (1, 2):
        a = run_gemm(eng, np.random.default_rng(9), 256, 256, 256, tb, dt)[0]
        b = run_gemm(eng, np.random.default_rng(9), 256, 256, 256, tb, dt, fallback=1)[0]
        assert np.abs(a - b).max() <= (2e-2 if dt == 1 else 1e-3) * np.abs(b).max()


@pytest.mark.parametrize("dt", [0, 1])
def test_small_and_unaligned_bf16_and_batched_offsets(eng, dt):
    rng = np.random.default_rng(5)
    for (m, n, k, tb) in [(3, 5, 7, 0), (130, 16, 136, 0), (16, 130, 130, 2), (130, 136, 16, 1), (129, 131, 67, 1)]:
        got, ref = run_gemm(eng, rng, m, n, k, tb, dt)
        check(got, ref, dt == 1, k)
    # strided batch with element offsets, as the tiled attention plan issues them
    batch, qt, kl, DH, T, rep = 4, 8, 24, 16, 32, 2
    q = rng.standard_normal((batch, rep, T, DH)).astype(np.float32)
    kk = rng.standard_normal((batch, T, DH)).astype(np.float32)
    if dt:
        q, kk = bf(q), bf(kk)
    iq, ik, ic = put(eng, q, dt), put(eng, kk, dt), eng.alloc(batch * qt * kl)
    j, qs = 1, 16
    eng.run([op(E.GEMM_SB, a=iq, b=ik, c=ic, m=qt, k=DH, n=kl, batch=batch, tb=1, sa=rep * T * DH, sb=T * DH,
                sc=qt * kl, oa=(j * T + qs) * DH, dt=dt, alpha=0.25)])
    ref = 0.25 * np.einsum("bqd,bkd->bqk", q[:, j, qs:qs + qt], kk[:, :kl])
    got = eng.download_bf16(ic, ref.shape) if dt else eng.download(ic, ref.shape)
    check(got, ref, dt == 1, DH)


@pytest.mark.parametrize("dt", [0, 1, 2])
@pytest.mark.parametrize("tb", [0, 1, 2])
@pytest.mark.parametrize("count", [2, 3])
def test_grouped_gemm_shared_input(eng, dt, tb, count):
    """GEMM_GROUP mode 1: one input, several outputs with their own widths (ragged ones included)."""
    rng = np.random.default_rng(10 * tb + count + dt)
    m, k, ns = 520, 320, (520, 264, 136)[:count]
    in_bf, out_bf = dt >= 1, dt == 1
    A = rng.standard_normal((k, m) if tb == 2 else (m, k)).astype(np.float32)
    Bs = [rng.standard_normal((n, k) if tb == 1 else (k, n)).astype(np.float32) for n in ns]
    if in_bf:
        A, Bs = bf(A), [bf(b) for b in Bs]
    ia = put(eng, A, in_bf)
    ib = [put(eng, b, in_bf) for b in Bs] + [0]
    ic = [eng.alloc(m * n, 2 if out_bf else 4) for n in ns] + [0]
    nn = list(ns) + [0]
    eng.run([op(E.GEMM_GROUP, a=ia, b=ib[0], sa=ib[1], sb=ib[2], c=ic[0], d=ic[1], sc=ic[2], m=m, k=k,
                n=nn[0], oa=nn[1], ob=nn[2], batch=count, oc=1, tb=tb, dt=dt, alpha=0.5)])
    Aop = A.T if tb == 2 else A
    for g, n in enumerate(ns):
        got = eng.download_bf16(ic[g], (m, n)) if out_bf else eng.download(ic[g], (m, n))
        Bop = Bs[g].T if tb == 1 else Bs[g]
        check(got, (0.5 * (Aop.astype(np.float64) @ Bop.astype(np.float64))).astype(np.float32), out_bf, k)
    assert eng.device_status() == 0


@pytest.mark.parametrize("dt", [0, 1, 2])
@pytest.mark.parametrize("tb", [0, 1, 2])
@pytest.mark.parametrize("count", [2, 3])
def test_grouped_gemm_summed_segments(eng, dt, tb, count):
    """GEMM_GROUP mode 2: one output accumulated over K-segments of different depths (one not a multiple
    of the 64-wide k-block)."""
    rng = np.random.default_rng(100 + 10 * tb + count + dt)
    m, n, ks = 520, 392, (320, 136, 200)[:count]
    in_bf, out_bf = dt >= 1, dt == 1
    As = [rng.standard_normal((k, m) if tb == 2 else (m, k)).astype(np.float32) for k in ks]
    Bs = [rng.standard_normal((n, k) if tb == 1 else (k, n)).astype(np.float32) for k in ks]
    if in_bf:
        As, Bs = [bf(a) for a in As], [bf(b) for b in Bs]
    ia = [put(eng, a, in_bf) for a in As] + [0]
    ib = [put(eng, b, in_bf) for b in Bs] + [0]
    ic = eng.alloc(m * n, 2 if out_bf else 4)
    kk = list(ks) + [0]
    eng.run([op(E.GEMM_GROUP, c=ic, a=ia[0], sa=ia[1], sb=ia[2], b=ib[0], d=ib[1], sc=ib[2], m=m, n=n,
                k=kk[0], oa=kk[1], ob=kk[2], batch=count, oc=2, tb=tb, dt=dt)])
    ref = np.zeros((m, n), np.float64)
    for a, b_ in zip(As, Bs):
        ref += (a.T if tb == 2 else a).astype(np.float64) @ (b_.T if tb == 1 else b_).astype(np.float64)
    got = eng.download_bf16(ic, (m, n)) if out_bf else eng.download(ic, (m, n))
    check(got, ref.astype(np.float32), out_bf, sum(ks))
    assert eng.device_status() == 0


@pytest.mark.parametrize("dt", [0, 1, 2])
@pytest.mark.parametrize("tb", [0, 1, 2])
def test_grouped_gemm_independent_problems(eng, dt, tb):
    """GEMM_GROUP mode 3: two problems with their own operands, heights and widths, one depth."""
    rng = np.random.default_rng(300 + 10 * tb + dt)
    k, ms, ns = 328, (776, 264), (392, 520)
    in_bf, out_bf = dt >= 1, dt == 1
    As = [rng.standard_normal((k, m) if tb == 2 else (m, k)).astype(np.float32) for m in ms]
    Bs = [rng.standard_normal((n, k) if tb == 1 else (k, n)).astype(np.float32) for n in ns]
    if in_bf:
        As, Bs = [bf(a) for a in As], [bf(b) for b in Bs]
    ia = [put(eng, a, in_bf) for a in As]
    ib = [put(eng, b, in_bf) for b in Bs]
    ic = [eng.alloc(m * n, 2 if out_bf else 4) for m, n in zip(ms, ns)]
    eng.run([op(E.GEMM_GROUP, a=ia[0], sa=ia[1], b=ib[0], sb=ib[1], c=ic[0], d=ic[1], m=ms[0], oa=ms[1],
                n=ns[0], ob=ns[1], k=k, batch=2, oc=3, tb=tb, dt=dt)])
    for g in range(2):
        got = eng.download_bf16(ic[g], (ms[g], ns[g])) if out_bf else eng.download(ic[g], (ms[g], ns[g]))
        ref = (As[g].T if tb == 2 else As[g]).astype(np.float64) @ (Bs[g].T if tb == 1 else Bs[g]).astype(np.float64)
        check(got, ref.astype(np.float32), out_bf, k)
    assert eng.device_status() == 0


@pytest.mark.parametrize("dt", [0, 1])
@pytest.mark.parametrize("m,n,k", [(520, 392, 320), (256, 128, 64), (1032, 1000, 136)])
def test_grouped_gemm_swiglu_pair(eng, dt, m, n, k):
    """GEMM_GROUP mode 4: gate and up projections with h = silu(g) * u written by the same launch (bf16);
    the fp32 plan runs the unfused sequence behind the same op."""
    rng = np.random.default_rng(m + n + k + dt)
    A = rng.standard_normal((m, k)).astype(np.float32) * 0.5
    Wg = rng.standard_normal((k, n)).astype(np.float32) * 0.2
    Wu = rng.standard_normal((k, n)).astype(np.float32) * 0.2
    if dt:
        A, Wg, Wu = bf(A), bf(Wg), bf(Wu)
    ia, ig, iu = put(eng, A, dt), put(eng, Wg, dt), put(eng, Wu, dt)
    og, ou, oh = (eng.alloc(m * n, 2 if dt else 4) for _ in range(3))
    eng.run([op(E.GEMM_GROUP, a=ia, b=ig, sa=iu, c=og, d=ou, sc=oh, m=m, n=n, k=k, batch=2, oc=4, dt=dt)])
    g = A.astype(np.float64) @ Wg.astype(np.float64)
    u = A.astype(np.float64) @ Wu.astype(np.float64)
    h = g / (1.0 + np.exp(-g)) * u
    get_ = (lambda i: eng.download_bf16(i, (m, n))) if dt else (lambda i: eng.download(i, (m, n)))
    check(get_(og), g.astype(np.float32), dt == 1, k)
    check(get_(ou), u.astype(np.float32), dt == 1, k)
    check(get_(oh), h.astype(np.float32), dt == 1, k)
    assert eng.device_status() == 0


@pytest.mark.parametrize("fallback", [0, 1])
def test_grouped_projection_with_rotary_in_the_epilogue(eng, fallback):
    """GEMM_GROUP mode 1 with gamma > 0: q and k leave the launch rotated, v does not.  fallback 0: the paired-CTA
    kernel rotates in its epilogue (fp32 accumulators, one rounding); fallback 1: general GEMMs, then the rotary kernel."""
    rng = np.random.default_rng(5)
    B_, T, D, H, KV = 2, 256, 192, 6, 2
    N = B_ * T
    bf = lambda a: E.bf16_bits_to_f32(E.f32_to_bf16_bits(a))
    x = bf(rng.standard_normal((N, D)).astype(np.float32))
    wq, wk, wv = (bf(rng.standard_normal((D, w)).astype(np.float32) * 0.1) for w in (H * 64, KV * 64, KV * 64))
    cos, sin = O.rope_tables(T, 64)

    def put(a, bf16=True):
        i = eng.alloc(a.size, 2 if bf16 else 4)
        eng.upload_bf16(i, a) if bf16 else eng.upload(i, a)
        return i
    ix, iq, ik, iv = put(x), put(wq), put(wk), put(wv)
    ic, isn = put(cos, False), put(sin, False)
    oq, ok_, ov = eng.alloc(N * H * 64, 2), eng.alloc(N * KV * 64, 2), eng.alloc(N * KV * 64, 2)
    eng.set_fallback(fallback)
    eng.launch_count(reset=True)
    eng.run([op(E.GEMM_GROUP, a=ix, b=iq, sa=ik, sb=iv, c=oq, d=ok_, sc=ov, m=N, k=D, n=H * 64, oa=KV * 64, ob=KV * 64,
                batch=3, oc=1, dt=1, beta=float(ic), gamma=float(isn))])
    launches = eng.launch_count()
    eng.set_fallback(0)
    assert launches == (1 if fallback == 0 else 4)
    rot = lambda y, heads: O.rope_fwd(y.reshape(B_, T, heads, 64).transpose(0, 2, 1, 3), cos, sin).transpose(0, 2, 1, 3).reshape(N, heads * 64)
    q_ref, k_ref, v_ref = rot(x @ wq, H), rot(x @ wk, KV), x @ wv
    for got, ref in ((eng.download_bf16(oq, (N, H * 64)), q_ref), (eng.download_bf16(ok_, (N, KV * 64)), k_ref),
                     (eng.download_bf16(ov, (N, KV * 64)), v_ref)):
        assert np.abs(got - ref).max() <= 1.2e-2 * np.abs(ref).max()
    assert eng.device_status() == 0


@pytest.mark.parametrize("dt", [0, 1])
@pytest.mark.parametrize("tb", [0, 1])
@pytest.mark.parametrize("count", [2, 3])
def test_grouped_gemm_shared_input_with_a_low_rank_term_per_output(eng, dt, tb, count):
    """GEMM_XSEG before GEMM_GROUP mode 1: C_g = alpha * (A B_g + A'_g B'_g) — an adapter's rank-16 product as a
    K-segment of its projection's launch; the variant number tells that the grouped kernel served it in bf16."""
    rng = np.random.default_rng(500 + 10 * tb + count + dt)
    m, k, r, ns = 520, 320, 16, (520, 264, 136)[:count]
    mk = lambda sh: bf(rng.standard_normal(sh).astype(np.float32)) if dt else rng.standard_normal(sh).astype(np.float32)
    A = mk((m, k))
    Bs = [mk((n, k) if tb == 1 else (k, n)) for n in ns]
    XAs = [mk((m, r)) for _ in ns]
    XBs = [mk((n, r) if tb == 1 else (r, n)) for n in ns]
    ia = put(eng, A, dt)
    ib = [put(eng, b, dt) for b in Bs] + [0]
    xa = [put(eng, a, dt) for a in XAs] + [0]
    xb = [put(eng, b, dt) for b in XBs] + [0]
    ic = [eng.alloc(m * n, 2 if dt else 4) for n in ns] + [0]
    nn = list(ns) + [0]
    eng.launch_count(reset=True)
    eng.run([op(E.GEMM_XSEG, a=xa[0], b=xa[1], d=xa[2], sa=xb[0], sb=xb[1], sc=xb[2], k=r, batch=count),
             op(E.GEMM_GROUP, a=ia, b=ib[0], sa=ib[1], sb=ib[2], c=ic[0], d=ic[1], sc=ic[2], m=m, k=k,
                n=nn[0], oa=nn[1], ob=nn[2], batch=count, oc=1, tb=tb, dt=dt, alpha=0.5)])
    if dt:
        assert eng.launch_count() == 1                       # one grouped launch, nothing run one by one
    for g, n in enumerate(ns):
        got = eng.download_bf16(ic[g], (m, n)) if dt else eng.download(ic[g], (m, n))
        Bop = Bs[g].T if tb == 1 else Bs[g]
        XBop = XBs[g].T if tb == 1 else XBs[g]
        ref = 0.5 * (A.astype(np.float64) @ Bop.astype(np.float64) + XAs[g].astype(np.float64) @ XBop.astype(np.float64))
        check(got, ref.astype(np.float32), dt == 1, k + r)
    assert eng.device_status() == 0


@pytest.mark.parametrize("dt", [0, 1])
@pytest.mark.parametrize("tb", [0, 1])
@pytest.mark.parametrize("count,extra,addend", [(3, 3, False), (1, 1, True), (2, 2, True), (3, 1, False)])
def test_grouped_gemm_up_to_six_segments_and_an_addend(eng, dt, tb, count, extra, addend):
    """GEMM_XSEG before GEMM_GROUP mode 2: further K-segments (depth 16) behind the op's own, and a residual addend:
    C = sum_s A_s B_s + D."""
    rng = np.random.default_rng(600 + 10 * tb + 3 * count + extra + dt)
    m, n, r, ks = 520, 392, 16, (320, 136, 200)[:count]
    mk = lambda sh: bf(rng.standard_normal(sh).astype(np.float32)) if dt else rng.standard_normal(sh).astype(np.float32)
    As = [mk((m, k)) for k in ks] + [mk((m, r)) for _ in range(extra)]
    Bs = [mk((n, k) if tb == 1 else (k, n)) for k in ks] + [mk((n, r) if tb == 1 else (r, n)) for _ in range(extra)]
    D = mk((m, n))
    ia = [put(eng, a, dt) for a in As[:count]] + [0, 0]
    ib = [put(eng, b, dt) for b in Bs[:count]] + [0, 0]
    xa = [put(eng, a, dt) for a in As[count:]] + [0, 0]
    xb = [put(eng, b, dt) for b in Bs[count:]] + [0, 0]
    idd = put(eng, D, dt) if addend else 0
    ic = eng.alloc(m * n, 2 if dt else 4)
    kk = list(ks) + [0, 0]
    eng.launch_count(reset=True)
    eng.run([op(E.GEMM_XSEG, a=xa[0], b=xa[1], d=xa[2], sa=xb[0], sb=xb[1], sc=xb[2], k=r, batch=extra, c=idd, beta=1.0),
             op(E.GEMM_GROUP, c=ic, a=ia[0], sa=ia[1], sb=ia[2], b=ib[0], d=ib[1], sc=ib[2], m=m, n=n,
                k=kk[0], oa=kk[1], ob=kk[2], batch=count, oc=2, tb=tb, dt=dt)])
    if dt:
        assert eng.launch_count() == 1
    ref = D.astype(np.float64) if addend else np.zeros((m, n), np.float64)
    for a, b_ in zip(As, Bs):
        ref = ref + a.astype(np.float64) @ (b_.T if tb == 1 else b_).astype(np.float64)
    got = eng.download_bf16(ic, (m, n)) if dt else eng.download(ic, (m, n))
    check(got, ref.astype(np.float32), dt == 1, sum(ks) + r * extra)
    assert eng.device_status() == 0


def test_extra_operands_are_refused_where_they_have_no_meaning(eng):
    """A GEMM_XSEG whose count differs from the mode-1 group's, or before a mode-3 group, is an error, and the pending
    operands do not leak into a later group."""
    rng = np.random.default_rng(7)
    m, k, n, r = 256, 64, 64, 16
    A, B = bf(rng.standard_normal((m, k)).astype(np.float32)), bf(rng.standard_normal((k, n)).astype(np.float32))
    ia, ib, ic, id_ = put(eng, A, 1), put(eng, B, 1), eng.alloc(m * n, 2), eng.alloc(m * n, 2)
    xa, xb = put(eng, bf(rng.standard_normal((m, r)).astype(np.float32)), 1), put(eng, bf(rng.standard_normal((r, n)).astype(np.float32)), 1)
    grp = op(E.GEMM_GROUP, a=ia, b=ib, sa=ib, c=ic, d=id_, m=m, k=k, n=n, oa=n, batch=2, oc=1, dt=1)
    with pytest.raises(RuntimeError):
        eng.run([op(E.GEMM_XSEG, a=xa, sa=xb, k=r, batch=1), grp])
    eng.run([grp])                                   # the refused operands are gone
    got = eng.download_bf16(ic, (m, n))
    check(got, (A.astype(np.float64) @ B.astype(np.float64)).astype(np.float32), True, k)


@pytest.mark.parametrize("layout", [0, 1])
@pytest.mark.parametrize("R", [8, 16, 32])
def test_adapter_gradients_stream_kernel(eng, layout, R):
    """LORA_GRAD: alpha * X_g^T S_g for three products (ragged widths and token count), written at offsets of one fp32
    buffer as [F, R] or [R, F]; bit-identical on a second run (fixed summation order)."""
    rng = np.random.default_rng(800 + layout + R)
    N, Fs = 1000, (520, 264, 1536)
    Xs = [bf(rng.standard_normal((N, F)).astype(np.float32)) for F in Fs]
    Ss = [bf(rng.standard_normal((N, R)).astype(np.float32)) for _ in Fs]
    ix = [put(eng, x, 1) for x in Xs]
    is_ = [put(eng, s_, 1) for s_ in Ss]
    offs = [64, 64 + Fs[0] * R + 8, 64 + Fs[0] * R + 8 + Fs[1] * R + 8]
    total = offs[2] + Fs[2] * R + 64
    out = eng.alloc(total)
    eng.upload(out, np.full(total, 7.0, np.float32))
    plan = [op(E.LORA_GRAD, a=ix[0], sa=ix[1], sb=ix[2], b=is_[0], d=is_[1], sc=is_[2], c=out, oa=offs[0], ob=offs[1],
               oc=offs[2], n=Fs[0], k=Fs[1], tb=Fs[2], m=N, batch=3, gamma=float(R), beta=float(layout), alpha=0.5, dt=1)]
    eng.run(plan)
    assert eng.last_variant() == 0x60                         # the streaming kernel, not the GEMM path
    got = eng.download(out, total)
    eng.run(plan)
    assert np.array_equal(got, eng.download(out, total))
    touched = np.zeros(total, bool)
    for g, F in enumerate(Fs):
        ref = 0.5 * (Xs[g].astype(np.float64).T @ Ss[g].astype(np.float64))
        ref = ref.T if layout else ref
        seg = got[offs[g]:offs[g] + F * R].reshape(ref.shape)
        assert np.abs(seg - ref).max() <= 2e-5 * np.abs(ref).max() + 1e-4
        touched[offs[g]:offs[g] + F * R] = True
    assert np.all(got[~touched] == 7.0)                       # nothing outside the three outputs is written
    # the GEMM path (library fallback switch) gives the same numbers within fp32 summation order
    eng.set_fallback(1)
    eng.run(plan)
    eng.set_fallback(0)
    assert np.abs(eng.download(out, total) - got)[touched].max() <= 1e-3 * np.abs(got[touched]).max()
    assert eng.device_status() == 0


@pytest.mark.parametrize("tb", [0, 1])
@pytest.mark.parametrize("R", [8, 16, 32])
def test_adapter_skinny_products_stream_kernel(eng, tb, R):
    """LORA_PROJ: out_g [N, R] = alpha * X_g W_g (W [F, R]) or X_g W_g^T (W [R, F]) for three adapters at once, ragged token
    count and widths (one narrower than a 256-column piece, one of several pieces)."""
    rng = np.random.default_rng(900 + tb + R)
    N, Fs = 1000, (520, 136, 1536)
    Xs = [bf(rng.standard_normal((N, F)).astype(np.float32)) for F in Fs]
    Ws = [bf(rng.standard_normal((R, F) if tb else (F, R)).astype(np.float32) * 0.1) for F in Fs]
    ix, iw = [put(eng, x, 1) for x in Xs], [put(eng, w, 1) for w in Ws]
    io = [eng.alloc(N * R + 64, 2) for _ in Fs]
    for o_ in io:
        eng.upload_bf16(o_, np.full(N * R + 64, 3.0, np.float32))
    plan = [op(E.LORA_PROJ, a=ix[0], sa=ix[1], sb=ix[2], b=iw[0], d=iw[1], sc=iw[2], c=io[0], oa=io[1], ob=io[2],
               n=Fs[0], k=Fs[1], oc=Fs[2], m=N, batch=3, tb=tb, gamma=float(R), alpha=2.0, dt=1)]
    eng.launch_count(reset=True)
    eng.run(plan)
    assert eng.last_variant() == 0x62 and eng.launch_count() == 1
    for g, F in enumerate(Fs):
        got = eng.download_bf16(io[g], (N * R + 64,))
        ref = 2.0 * (Xs[g].astype(np.float64) @ (Ws[g].T if tb else Ws[g]).astype(np.float64))
        check(got[:N * R].reshape(N, R), ref.astype(np.float32), True, F)
        assert np.all(got[N * R:] == 3.0)
    # one shared input (the u_g = x A_g of projections of one input), against the GEMM path
    plan2 = [op(E.LORA_PROJ, a=ix[2], b=iw[2], d=iw[2], c=io[0], oa=io[1], n=Fs[2], k=Fs[2], m=N, batch=2, tb=tb,
                gamma=float(R), dt=1)]
    eng.run(plan2)
    a0, a1 = eng.download_bf16(io[0], (N, R)), eng.download_bf16(io[1], (N, R))
    assert np.array_equal(a0, a1)
    eng.set_fallback(1)
    eng.run(plan2)
    eng.set_fallback(0)
    check(eng.download_bf16(io[0], (N, R)), a0, True, Fs[2])
    assert eng.device_status() == 0


def test_adapter_gradients_noted_and_run_as_one_launch(eng):
    """LORA_GRAD with batch < 0 only notes its products; batch = 0 runs all of them (both layouts mixed) as one launch pair."""
    rng = np.random.default_rng(77)
    N, R, Fs = 777, 16, (264, 520, 136, 1032)
    Xs = [bf(rng.standard_normal((N, F)).astype(np.float32)) for F in Fs]
    Ss = [bf(rng.standard_normal((N, R)).astype(np.float32)) for _ in Fs]
    ix, is_ = [put(eng, x, 1) for x in Xs], [put(eng, s_, 1) for s_ in Ss]
    offs = list(np.cumsum([0] + [F * R for F in Fs]))
    out = eng.alloc(int(offs[-1]))
    eng.upload(out, np.zeros(int(offs[-1]), np.float32))
    eng.launch_count(reset=True)
    eng.run([op(E.LORA_GRAD, a=ix[0], sa=ix[1], b=is_[0], d=is_[1], c=out, oa=int(offs[0]), ob=int(offs[1]), n=Fs[0], k=Fs[1],
                m=N, batch=-2, gamma=float(R), dt=1),
             op(E.LORA_GRAD, a=ix[2], sa=ix[3], b=is_[2], d=is_[3], c=out, oa=int(offs[2]), ob=int(offs[3]), n=Fs[2], k=Fs[3],
                m=N, batch=-2, gamma=float(R), beta=1.0, dt=1)])
    assert eng.launch_count() == 0 and np.all(eng.download(out, int(offs[-1])) == 0)      # nothing has run yet
    eng.run([op(E.LORA_GRAD, batch=0)])
    assert eng.launch_count() == 2 and eng.last_variant() == 0x60
    got = eng.download(out, int(offs[-1]))
    for g, F in enumerate(Fs):
        ref = Xs[g].astype(np.float64).T @ Ss[g].astype(np.float64)
        ref = ref.T if g >= 2 else ref
        seg = got[offs[g]:offs[g + 1]].reshape(ref.shape)
        assert np.abs(seg - ref).max() <= 2e-5 * np.abs(ref).max() + 1e-4
    eng.run([op(E.LORA_GRAD, batch=0)])              # an empty set is a no-op
    assert eng.launch_count() == 2 and eng.device_status() == 0
