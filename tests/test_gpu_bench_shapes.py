"""Parity at the shapes the benchmark runs, against the CPU oracle.

The small-shape tests elsewhere cover every op; these cover the kernels and code paths that only the
benchmarked sizes reach: the register-resident cross-entropy rows (bf16, vocabulary 32000), attention at
T = 2048 with 24/8 heads (16 key tiles, 96 sub-tile iterations per CTA) and at head_dim 128 / T = 4096, the
8192-row grouped GEMMs, split-K weight gradients and the tied-head 32000-wide GEMMs inside one-layer steps of
the 1B-class and 7B-class widths, and the LoRA step on a long masked sequence.  Tolerances are the
north-star's bf16 bars: gradients <= 2e-2 per-tensor max-relative, loss <= 1e-3 relative (the gates of
engine/modal_bf16_test.py:59-136, modal_harden_test.py:51-115 and modal_longseq_test.py:42-74 at these
sizes).  The oracle is evaluated on slices where the full problem would not fit a host's memory."""
import numpy as np
import pytest

from axis_b200 import engine as E
from axis_b200.compile import CompiledTransformer
from axis_b200.engine import Engine, op
from oracle import step_numpy as O

pytestmark = pytest.mark.gpu


def bf(a):
    return E.bf16_bits_to_f32(E.f32_to_bf16_bits(a))


def rel(got, ref):
    return float(np.abs(got - ref).max() / (np.abs(ref).max() + 1e-9))


@pytest.fixture()
def eng():
    e = Engine()
    e.alloc(4)
    yield e
    e.shutdown()


def test_cross_entropy_register_rows_at_vocab_32000(eng):
    """CE_FUSED in bf16 at V = 32000 runs on the kernel that keeps a row in registers (one read, one write,
    exponentials held as packed fp16); 5 % of the targets are ignored."""
    N, V = 256, 32000
    rng = np.random.default_rng(11)
    logits = bf(rng.standard_normal((N, V)).astype(np.float32) * 2.0)
    tgt = rng.integers(0, V, N)
    tgt[rng.random(N) < 0.05] = -1
    tgt[0] = V - 1; tgt[1] = 0
    loss, dl, cnt = O.cross_entropy_fwd_bwd(logits, tgt, -1)
    il = eng.alloc(N * V, 2); eng.upload_bf16(il, logits)
    it = eng.alloc(N); eng.upload_tokens(it, tgt, V)
    iloss, iden, iscr = eng.alloc(1), eng.alloc(1), eng.alloc(N + 8)
    eng.run([op(E.CE_FUSED, a=il, b=it, c=il, d=iloss, sa=iden, sb=iscr, m=N, n=V, dt=1)])
    assert eng.last_variant() == 0x11                                # the register-resident kernel
    assert eng.download(iden, 1)[0] == cnt == int((tgt >= 0).sum())  # integer work: exact
    assert abs(eng.download(iloss, 1)[0] - loss) <= 1e-5 * abs(loss)
    got = eng.download_bf16(il, (N, V))
    assert rel(got, dl) <= 1.2e-2
    assert np.all(got[tgt < 0] == 0)
    eng.upload_bf16(il, logits)
    eng.run([op(E.CE_FUSED, a=il, b=it, c=il, d=iloss, sa=iden, sb=iscr, m=N, n=V, dt=1)])
    again = eng.download_bf16(il, (N, V))
    assert np.array_equal(got, again)                                # run-to-run identical
    assert eng.device_status() == 0


def _attention_case(eng, B, H, KV, T, DH, slices, seed):
    """Forward + backward on the GPU at the full shape; oracle on the (batch, kv group) slices given."""
    rng = np.random.default_rng(seed)
    rep = H // KV
    q = bf(rng.standard_normal((B, T, H, DH), dtype=np.float32))
    k = bf(rng.standard_normal((B, T, KV, DH), dtype=np.float32))
    v = bf(rng.standard_normal((B, T, KV, DH), dtype=np.float32))
    do = bf(rng.standard_normal((B, T, H, DH), dtype=np.float32))
    scale = 1.0 / np.sqrt(DH)

    def put(a):
        i = eng.alloc(a.size, 2); eng.upload_bf16(i, a); return i
    iq, ik, iv, ido = put(q), put(k), put(v), put(do)
    io, ilse, iD = eng.alloc(q.size, 2), eng.alloc(B * H * T), eng.alloc(B * H * T + q.size)
    idq, idk, idv = eng.alloc(q.size, 2), eng.alloc(k.size, 2), eng.alloc(k.size, 2)
    eng.run([op(E.ATTN_FWD, a=iq, b=ik, d=iv, c=io, sa=ilse, m=T, n=DH, k=KV, batch=B, tb=H, dt=1, alpha=scale)])
    eng.launch_count(reset=True)
    eng.run([op(E.ATTN_BWD, a=iq, b=ik, d=iv, c=ido, sa=ilse, sb=io, tb=idq, sc=idk, oa=idv, ob=H, oc=iD,
                m=T, n=DH, k=KV, batch=B, dt=1, alpha=scale)])
    assert eng.launch_count() == 4                                   # memset, prep, tensor-core kernel, convert
    o = eng.download_bf16(io, (B, T, H, DH)); lse = eng.download(ilse, (B, H, T))
    dq = eng.download_bf16(idq, (B, T, H, DH))
    dk = eng.download_bf16(idk, (B, T, KV, DH)); dv = eng.download_bf16(idv, (B, T, KV, DH))
    worst = {}
    for (b, g) in slices:
        hs = slice(g * rep, (g + 1) * rep)
        t = lambda x: np.ascontiguousarray(x.transpose(0, 2, 1, 3))         # [1,T,h,DH] -> [1,h,T,DH]
        qs, ks, vs, dos = t(q[b:b + 1, :, hs]), t(k[b:b + 1, :, g:g + 1]), t(v[b:b + 1, :, g:g + 1]), t(do[b:b + 1, :, hs])
        o_ref, lse_ref = O.attention_fwd(qs, ks, vs, scale)
        dq_ref, dk_ref, dv_ref = O.attention_bwd(qs, ks, vs, dos, scale)    # dk/dv summed over the group's heads
        for nm, got, ref in (("o", t(o[b:b + 1, :, hs]), o_ref), ("dq", t(dq[b:b + 1, :, hs]), dq_ref),
                             ("dk", t(dk[b:b + 1, :, g:g + 1]), dk_ref), ("dv", t(dv[b:b + 1, :, g:g + 1]), dv_ref)):
            worst[nm] = max(worst.get(nm, 0.0), rel(got, ref))
        worst["lse"] = max(worst.get("lse", 0.0), float(np.abs(lse[b, hs] - lse_ref[0]).max()))
    assert worst["o"] <= 1.5e-2 and worst["lse"] <= 2e-2, worst
    assert worst["dq"] <= 2e-2 and worst["dk"] <= 2e-2 and worst["dv"] <= 2e-2, worst
    assert eng.device_status() == 0


def test_attention_at_the_isolated_backward_benchmark_shape(eng):
    """Q/dO [4,24,2048,64], K/V [4,8,2048,64] (GQA 3:1), scale 1/8; first, middle and last (batch, kv group)."""
    _attention_case(eng, 4, 24, 8, 2048, 64, [(0, 0), (1, 4), (3, 7)], seed=21)


def test_attention_head_dim_128_at_the_7b_shape(eng):
    """B2 H32 KV32 T4096 DH128: two heads against the oracle."""
    _attention_case(eng, 2, 32, 32, 4096, 128, [(0, 0), (1, 31)], seed=22)


def _one_layer_step(cfg, B, T, ignore_frac, seed, lora=None, prompt_frac=0.0):
    w0 = O.init_weights(cfg, seed=seed)
    rng = np.random.default_rng(seed)
    V = cfg["vocab_size"]
    x, y = O.make_batch(rng, V, B, T, ignore_frac)
    if prompt_frac:
        y = y.copy(); y[:, :int(prompt_frac * T)] = -1
    kw = {}
    if lora:
        w0.update(O.init_lora(cfg, lora["rank"], lora["targets"], seed=seed + 1))
        for k_ in list(w0):
            if k_.endswith(".lora_b"):        # non-zero B, or the A gradients are identically zero
                w0[k_] = (np.random.default_rng(seed + 2).standard_normal(w0[k_].shape) * 0.02).astype(np.float32)
        kw = dict(lora_r=lora["rank"], lora_alpha=lora["alpha"], lora_targets=tuple(lora["targets"]))
        model = O.OracleTransformer(cfg, w0, lora_rank=lora["rank"], lora_alpha=lora["alpha"], lora_targets=lora["targets"])
    else:
        model = O.OracleTransformer(cfg, w0)
    l_ref, g_ref = model.loss_and_grads(x, y)
    ct = CompiledTransformer(None, cfg, w0, B, T, dtype="bf16", max_grad_norm=1.0, **kw)
    loss = ct.forward_backward(x, y)
    g = ct.grads()
    assert ct.valid_count() == int((y >= 0).sum())
    assert abs(loss - l_ref) <= 1e-3 * abs(l_ref), (loss, l_ref)
    worst = max((rel(g[nm], g_ref[nm]), nm) for nm in g)
    assert worst[0] <= 2e-2, worst
    assert ct.eng.device_status() == 0
    ct.eng.shutdown()


def test_one_layer_step_at_the_1b_widths():
    """V32000 D1536 H24/KV8 MLP4096, B1 T2048, bf16, 5 % ignored: the 2048-row grouped GEMMs, split-K weight
    gradients, the tied-head 32000 x 1536 GEMMs and the register-resident cross-entropy meet the oracle."""
    cfg = dict(vocab_size=32000, dim=1536, n_layers=1, n_heads=24, n_kv_heads=8, mlp_hidden=4096, tie_embeddings=True)
    _one_layer_step(cfg, 1, 2048, 0.05, seed=31)


def test_one_layer_step_at_the_7b_widths():
    """V32000 D4096 H32/KV32 (head_dim 128) MLP11008, B1 T512: the wide-row RMSNorm kernels and head_dim-128
    attention inside a step."""
    cfg = dict(vocab_size=32000, dim=4096, n_layers=1, n_heads=32, n_kv_heads=32, mlp_hidden=11008, tie_embeddings=True)
    _one_layer_step(cfg, 1, 512, 0.0, seed=32)


def test_one_layer_lora_step_at_the_1b_widths():
    """LoRA r16 alpha 32 on all seven projections, frozen base, T = 1024, first 40 % of the targets masked."""
    cfg = dict(vocab_size=32000, dim=1536, n_layers=1, n_heads=24, n_kv_heads=8, mlp_hidden=4096, tie_embeddings=True)
    lora = dict(rank=16, alpha=32.0, targets=["q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj"])
    _one_layer_step(cfg, 1, 1024, 0.0, seed=33, lora=lora, prompt_frac=0.4)
