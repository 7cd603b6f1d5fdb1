"""Drop-in check: a step expressed only in the reference's 32 op kinds (one op per
primitive, per-tensor buffers, per-tensor AdamW — tests/legacy_plan.py) gives the
oracle's loss, gradients and updated weights; fp32 with the tiled attention ops,
bf16 with FLASH / ROWDOT / FLASH_BWD; eager and captured."""
import numpy as np
import pytest

from oracle import step_numpy as O
from tests.legacy_plan import LegacyStep

pytestmark = pytest.mark.gpu
CFGS = [dict(vocab_size=120, dim=64, n_layers=2, n_heads=4, n_kv_heads=2, mlp_hidden=96, tie_embeddings=True),
        dict(vocab_size=80, dim=64, n_layers=1, n_heads=2, n_kv_heads=2, mlp_hidden=72, tie_embeddings=False)]


def rel(a, b):
    return float(np.abs(a - b).max() / (np.abs(b).max() + 1e-9))


@pytest.mark.parametrize("cfg", CFGS)
@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
def test_reference_style_plan_matches_oracle(cfg, dtype):
    B, T = 2, 40
    w0 = O.init_weights(cfg, seed=5)
    rng = np.random.default_rng(5)
    x, y = O.make_batch(rng, cfg["vocab_size"], B, T, 0.1)
    ls = LegacyStep(cfg, w0, B, T, dtype=dtype)
    model = O.OracleTransformer(cfg, w0)
    opt = O.OracleAdamW(model)
    l_ref, g_ref = model.loss_and_grads(x, y)
    ls.upload(x, y)
    ls.eng.run(ls.plan_fb)
    loss = float(ls.eng.download(ls.loss, (1,))[0])
    lim_l, lim_g = (2e-6, 1e-5) if dtype == "fp32" else (1e-3, 2e-2)
    assert abs(loss - l_ref) <= lim_l * abs(l_ref) + 1e-6
    g = ls.grads()
    worst = max((rel(g[n], g_ref[n]), n) for n in g_ref)
    assert worst[0] <= lim_g, worst
    # two full steps (clip + tick + per-tensor AdamW), the second one from a captured graph
    ls.eng.run(ls.plan_step)
    ls.eng.capture(ls.plan_step)
    x2, y2 = O.make_batch(rng, cfg["vocab_size"], B, T, 0.1)
    ls.upload(x2, y2)
    ls.eng.replay(1)
    O.train_step(model, opt, x, y, max_grad_norm=1.0)
    O.train_step(model, opt, x2, y2, max_grad_norm=1.0)
    w = ls.weights()
    # Adam moves a weight by about lr per step whatever the gradient's size, so a bf16 gradient whose
    # rounding flips the sign of a near-zero element shifts that weight by up to 2 lr per step
    tol = 0.05 * 3e-4 if dtype == "fp32" else 4.5 * 3e-4
    for n in w:
        assert np.abs(w[n] - model.w[n]).max() <= tol, n
    assert ls.eng.device_status() == 0
    ls.eng.shutdown()
