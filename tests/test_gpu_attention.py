"""Causal GQA attention forward/backward on the GPU against the oracle: the
reference layout ops (FLASH / ROWDOT / FLASH_BWD on [B,H,T,DH], fp32 outputs)
and the fused ops on [B,T,H,DH]; fp32 and bf16; head_dim 16..128; ragged T;
MHA / GQA / MQA; determinism."""
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


def get(eng, i, shape, dt):
    return eng.download_bf16(i, shape) if dt else eng.download(i, shape)


def rel(got, ref):
    return float(np.abs(got - ref).max() / (np.abs(ref).max() + 1e-9))


def make(rng, B, H, KV, T, DH, dt):
    q = rng.standard_normal((B, H, T, DH)).astype(np.float32)
    k = rng.standard_normal((B, KV, T, DH)).astype(np.float32)
    v = rng.standard_normal((B, KV, T, DH)).astype(np.float32)
    do = rng.standard_normal((B, H, T, DH)).astype(np.float32)
    if dt:
        q, k, v, do = bf(q), bf(k), bf(v), bf(do)
    return q, k, v, do


CASES = [(2, 4, 2, 32, 32), (1, 6, 2, 17, 16), (2, 2, 2, 64, 64), (1, 4, 1, 40, 128), (1, 3, 3, 130, 64),
         # head_dim 64 with whole 128-token tiles: the tcgen05 kernels when fallback == 0
         (1, 4, 4, 128, 64), (2, 6, 2, 256, 64), (2, 3, 1, 384, 64), (1, 4, 2, 1024, 64),
         # head_dim 128 with whole tiles: the head_dim-128 tcgen05 kernels when fallback == 0
         (1, 2, 2, 128, 128), (2, 4, 2, 256, 128), (1, 3, 1, 640, 128)]


@pytest.mark.parametrize("dt", [0, 1])
@pytest.mark.parametrize("B,H,KV,T,DH", CASES)
@pytest.mark.parametrize("fallback", [0, 2])
def test_fused_attention_bthd(eng, dt, B, H, KV, T, DH, fallback):
    rng = np.random.default_rng(T * DH + H)
    q, k, v, do = make(rng, B, H, KV, T, DH, dt)
    scale = 1.0 / np.sqrt(DH)
    o_ref, lse_ref = O.attention_fwd(q, k, v, scale)
    t = lambda x: np.ascontiguousarray(x.transpose(0, 2, 1, 3))
    iq, ik, iv, ido = put(eng, t(q), dt), put(eng, t(k), dt), put(eng, t(v), dt), put(eng, t(do), dt)
    # scratch of the backward: D = rowsum(dO*O) followed by the fp32 dQ accumulator of the tensor-core path
    io, ilse, iD = eng.alloc(q.size), eng.alloc(B * H * T), eng.alloc(B * H * T + q.size)
    idq, idk, idv = eng.alloc(q.size), eng.alloc(k.size), eng.alloc(k.size)
    eng.set_fallback(fallback)
    eng.run([op(E.ATTN_FWD, a=iq, b=ik, d=iv, c=io, sa=ilse, m=T, n=DH, k=KV, batch=B, tb=H, dt=dt, alpha=scale)])
    o = get(eng, io, (B, T, H, DH), dt).transpose(0, 2, 1, 3)
    lse = eng.download(ilse, (B, H, T))
    lim = 1.5e-2 if dt else 2e-5
    assert rel(o, o_ref) <= lim
    assert np.abs(lse - lse_ref).max() <= (2e-2 if dt else 2e-5)
    o_in = bf(o) if dt else o
    dq_ref, dk_ref, dv_ref = O.attention_bwd(q, k, v, do, scale)
    eng.launch_count(reset=True)
    eng.run([op(E.ATTN_BWD, a=iq, b=ik, d=iv, c=ido, sa=ilse, sb=io, tb=idq, sc=idk, oa=idv, ob=H, oc=iD,
                m=T, n=DH, k=KV, batch=B, dt=dt, alpha=scale)])
    eng.set_fallback(0)
    # the tensor-core backward is four launches (memset, prep, main, convert), the general one three
    tc_expected = dt == 1 and fallback == 0 and DH in (64, 128) and T % 128 == 0
    assert eng.launch_count() == (4 if tc_expected else 3)
    dq = get(eng, idq, (B, T, H, DH), dt).transpose(0, 2, 1, 3)
    dk = get(eng, idk, (B, T, KV, DH), dt).transpose(0, 2, 1, 3)
    dv = get(eng, idv, (B, T, KV, DH), dt).transpose(0, 2, 1, 3)
    lim = 2e-2 if dt else 3e-5
    assert rel(dq, dq_ref) <= lim and rel(dk, dk_ref) <= lim and rel(dv, dv_ref) <= lim
    assert eng.device_status() == 0


def test_reference_layout_flash_ops(eng):
    """FLASH -> (permute) -> ROWDOT on [B,T,H,DH] -> FLASH_BWD into fp32 buffers, as the
    reference plan chains them (axis/compile.py:329-331, 406-421)."""
    rng = np.random.default_rng(0)
    B, H, KV, T, DH = 2, 4, 2, 48, 32
    q, k, v, do = make(rng, B, H, KV, T, DH, 1)
    scale = 1.0 / np.sqrt(DH)
    iq, ik, iv, ido = put(eng, q, 1), put(eng, k, 1), put(eng, v, 1), put(eng, do, 1)
    io, ilse = eng.alloc(q.size, 2), eng.alloc(B * H * T)
    eng.run([op(E.FLASH, a=iq, b=ik, d=iv, c=io, m=T, n=DH, k=KV, batch=B, tb=H, sa=ilse, dt=1, alpha=scale)])
    o_ref, lse_ref = O.attention_fwd(q, k, v, scale)
    o = eng.download_bf16(io, q.shape)
    assert rel(o, o_ref) <= 1.5e-2
    assert np.abs(eng.download(ilse, (B, H, T)) - lse_ref).max() <= 2e-2
    io2, ido2, iD = eng.alloc(q.size, 2), eng.alloc(q.size, 2), eng.alloc(B * T * H)
    idq, idk, idv = eng.alloc(q.size), eng.alloc(k.size), eng.alloc(k.size)
    eng.run([op(E.PERM_0213, a=io, c=io2, m=B, n=H, k=T, batch=DH, dt=1),
             op(E.PERM_0213, a=ido, c=ido2, m=B, n=H, k=T, batch=DH, dt=1),
             op(E.ROWDOT, a=ido2, b=io2, c=iD, m=B * T * H, n=DH, dt=1),
             op(E.SCALE, a=idq, c=idq, n=q.size, alpha=0.0), op(E.SCALE, a=idk, c=idk, n=k.size, alpha=0.0),
             op(E.SCALE, a=idv, c=idv, n=k.size, alpha=0.0),
             op(E.FLASH_BWD, a=iq, b=ik, d=iv, c=ido, sa=ilse, sb=iD, tb=idq, sc=idk, oa=idv, ob=H,
                m=T, n=DH, k=KV, batch=B, dt=1, alpha=scale)])
    dq_ref, dk_ref, dv_ref = O.attention_bwd(q, k, v, do, scale)
    assert rel(eng.download(idq, q.shape), dq_ref) <= 2e-2
    assert rel(eng.download(idk, k.shape), dk_ref) <= 2e-2
    assert rel(eng.download(idv, k.shape), dv_ref) <= 2e-2


@pytest.mark.parametrize("T", [256, 1024])
@pytest.mark.parametrize("DH", [64, 128])
@pytest.mark.parametrize("fallback", [0, 2])
def test_attention_backward_is_deterministic(eng, fallback, DH, T):
    """dK/dV are summed on chip in a fixed order in both paths.  dQ is bit-stable in the
    general path; the tensor-core path adds its per-key-tile dQ pieces with an unordered
    fp32 reduce-add (as the reference's atomics do), so dQ is only checked there for
    closeness."""
    rng = np.random.default_rng(1)
    B, H, KV = 1, 6, 2         # T = 1024: eight key tiles, deep pipelines (ring slots and TMEM buffers reused many times)
    q, k, v, do = make(rng, B, H, KV, T, DH, 1)
    t = lambda x: np.ascontiguousarray(x.transpose(0, 2, 1, 3))
    iq, ik, iv, ido = put(eng, t(q), 1), put(eng, t(k), 1), put(eng, t(v), 1), put(eng, t(do), 1)
    io, ilse, iD = eng.alloc(q.size, 2), eng.alloc(B * H * T), eng.alloc(B * H * T + q.size)
    idq, idk, idv = eng.alloc(q.size, 2), eng.alloc(k.size, 2), eng.alloc(k.size, 2)
    plan = [op(E.ATTN_FWD, a=iq, b=ik, d=iv, c=io, sa=ilse, m=T, n=DH, k=KV, batch=B, tb=H, dt=1, alpha=0.125),
            op(E.ATTN_BWD, a=iq, b=ik, d=iv, c=ido, sa=ilse, sb=io, tb=idq, sc=idk, oa=idv, ob=H, oc=iD,
               m=T, n=DH, k=KV, batch=B, dt=1, alpha=0.125)]
    eng.set_fallback(fallback)
    eng.run(plan)
    first = [eng.download_raw(i, n, np.uint16) for i, n in ((idq, q.size), (idk, k.size), (idv, k.size))]
    for _ in range(3):
        eng.run(plan)
        for which, (f, (i, n)) in enumerate(zip(first, ((idq, q.size), (idk, k.size), (idv, k.size)))):
            again = eng.download_raw(i, n, np.uint16)
            if which == 0 and fallback == 0:
                a, b2 = E.bf16_bits_to_f32(f), E.bf16_bits_to_f32(again)
                assert np.abs(a - b2).max() <= 1e-2 * np.abs(a).max()
            else:
                assert np.array_equal(f, again)
    eng.set_fallback(0)
    assert eng.device_status() == 0


@pytest.mark.parametrize("dt,B,H,KV,T,DH", [(1, 2, 6, 2, 256, 64), (1, 1, 4, 2, 256, 128), (0, 1, 4, 2, 40, 32), (1, 1, 3, 1, 130, 64)])
def test_attention_backward_with_the_inverse_rotary_inside(eng, dt, B, H, KV, T, DH):
    """ATTN_BWD with gamma > 0 returns dq and dk already rotated back (the compiled step's form): the head_dim-64
    tensor-core kernel applies the rotation before rounding, every other path runs the rotary kernel behind the
    attention kernels.  Reference: attention_bwd followed by rope_bwd of the oracle."""
    rng = np.random.default_rng(7 * T + DH)
    q, k, v, do = make(rng, B, H, KV, T, DH, dt)
    scale = 1.0 / np.sqrt(DH)
    cos, sin = O.rope_tables(T, DH)
    t = lambda x: np.ascontiguousarray(x.transpose(0, 2, 1, 3))
    iq, ik, iv, ido = put(eng, t(q), dt), put(eng, t(k), dt), put(eng, t(v), dt), put(eng, t(do), dt)
    ic, isn = put(eng, cos, 0), put(eng, sin, 0)
    io, ilse, iD = eng.alloc(q.size), eng.alloc(B * H * T), eng.alloc(B * H * T + q.size)
    idq, idk, idv = eng.alloc(q.size), eng.alloc(k.size), eng.alloc(k.size)
    eng.run([op(E.ATTN_FWD, a=iq, b=ik, d=iv, c=io, sa=ilse, m=T, n=DH, k=KV, batch=B, tb=H, dt=dt, alpha=scale),
             op(E.ATTN_BWD, a=iq, b=ik, d=iv, c=ido, sa=ilse, sb=io, tb=idq, sc=idk, oa=idv, ob=H, oc=iD,
                m=T, n=DH, k=KV, batch=B, dt=dt, alpha=scale, beta=float(ic), gamma=float(isn))])
    dq_ref, dk_ref, dv_ref = O.attention_bwd(q, k, v, do, scale)
    dq_ref, dk_ref = O.rope_bwd(dq_ref, cos, sin), O.rope_bwd(dk_ref, cos, sin)
    dq = get(eng, idq, (B, T, H, DH), dt).transpose(0, 2, 1, 3)
    dk = get(eng, idk, (B, T, KV, DH), dt).transpose(0, 2, 1, 3)
    dv = get(eng, idv, (B, T, KV, DH), dt).transpose(0, 2, 1, 3)
    lim = 2e-2 if dt else 3e-5
    assert rel(dq, dq_ref) <= lim and rel(dk, dk_ref) <= lim and rel(dv, dv_ref) <= lim
    assert eng.device_status() == 0
