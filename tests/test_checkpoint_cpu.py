"""Checkpoint files of the compiled step: layout (the reference's eager format), atomic write,
round trip, ZeRO-1 shard merge and its consistency checks — with a stand-in for the compiled step."""
import json
import os

import numpy as np
import pytest

from axis_b200 import checkpoint as C


class FakeStep:
    def __init__(self, shapes, owned=None, rank=0, world=1, seed=0):
        self.pnames = list(shapes)
        self.shapes = dict(shapes)
        self.owned = list(owned) if owned is not None else list(shapes)
        self.rank, self.world = rank, world
        rng = np.random.default_rng(seed)
        self.st = {}
        for nm in self.owned:
            for pre in ("w/", "m/", "v/"):
                self.st[pre + nm] = rng.standard_normal(shapes[nm]).astype(np.float32)
        self.st["_t"] = np.array([7.0], np.float32)
        self.st["_lr"] = np.array([2.5e-4], np.float32)

    def state_dict(self):
        return dict(self.st)

    def load_state_dict(self, st):
        self.st = {k: np.array(v) for k, v in st.items() if k[:2] in ("w/", "m/", "v/") and k[2:] in self.owned}
        self.st["_t"], self.st["_lr"] = np.array(st["_t"]), np.array(st["_lr"])


SHAPES = {"embed.weight": (16, 8), "blocks.0.attn.q_proj.weight": (8, 8), "blocks.0.attn_norm.weight": (8,),
          "norm.weight": (8,)}


def test_layout_matches_the_eager_checkpoint_format(tmp_path):
    ct = FakeStep(SHAPES)
    p = str(tmp_path / "a.npz")
    C.save(p, ct, step=12, meta={"run": "x"})
    assert not [f for f in os.listdir(tmp_path) if f.endswith(".tmp")]
    with np.load(p, allow_pickle=False) as z:
        hdr = json.loads(bytes(z["__header__"]).decode())
        assert hdr["step"] == 12 and hdr["meta"] == {"run": "x"} and hdr["optimizer"] == {"t": 7, "lr": pytest.approx(2.5e-4)}
        for i, nm in enumerate(ct.pnames):
            assert np.array_equal(z[f"model/{nm}"], ct.st[f"w/{nm}"])
            assert np.array_equal(z[f"opt/m/{i}"], ct.st[f"m/{nm}"])
            assert np.array_equal(z[f"opt/v/{i}"], ct.st[f"v/{nm}"])


def test_round_trip_and_shape_check(tmp_path):
    a, b = FakeStep(SHAPES, seed=1), FakeStep(SHAPES, seed=2)
    p = str(tmp_path / "a.npz")
    C.save(p, a, step=3)
    hdr = C.load(p, b)
    assert hdr["step"] == 3
    for k in a.st:
        assert np.array_equal(a.st[k], b.st[k]), k
    wrong = FakeStep({**SHAPES, "norm.weight": (9,)})
    with pytest.raises(ValueError):
        C.load(p, wrong)


def test_zero_shards_merge_into_the_full_state(tmp_path):
    names = list(SHAPES)
    full = FakeStep(SHAPES, seed=5)
    shards = []
    for rk, own in enumerate((names[:1] + names[3:], names[1:3])):
        s = FakeStep(SHAPES, owned=own, rank=rk, world=2)
        s.st = {k: v for k, v in full.st.items() if k[:2] in ("w/", "m/", "v/") and k[2:] in own}
        s.st["_t"], s.st["_lr"] = full.st["_t"], full.st["_lr"]
        p = str(tmp_path / f"shard{rk}.npz")
        C.save(p, s, step=9)
        shards.append(p)
    out = str(tmp_path / "full.npz")
    C.merge_shards(shards, out)
    hdr, st = C.read(out)
    assert hdr["owned"] == names and hdr["world"] == 1 and hdr["step"] == 9
    for k in full.st:
        assert np.array_equal(st[k], full.st[k]), k
    # a rank of a differently sharded run restores what it owns from the merged file
    other = FakeStep(SHAPES, owned=names[2:], rank=1, world=2, seed=8)
    C.load(out, other)
    assert all(np.array_equal(other.st[f"w/{nm}"], full.st[f"w/{nm}"]) for nm in names[2:])
    # one shard alone is not a full checkpoint; the same shard twice is rejected
    with pytest.raises(ValueError):
        C.merge_shards(shards[:1], str(tmp_path / "bad.npz"))
    with pytest.raises(ValueError):
        C.merge_shards([shards[0], shards[0]], str(tmp_path / "bad.npz"))
    with pytest.raises(KeyError):
        C.load(shards[0], FakeStep(SHAPES))


def _reference_style_file(path, weights, moment_names, scheduler_step=None):
    """A file as the reference's eager `checkpoint.save` writes it (axis/checkpoint.py:19-35): no parameter names for
    the moments, which follow the optimizer's parameter list."""
    rng = np.random.default_rng(4)
    payload = {f"model/{nm}": w for nm, w in weights.items()}
    moments = {}
    for i, nm in enumerate(moment_names):
        moments[nm] = (rng.standard_normal(weights[nm].shape).astype(np.float32), rng.standard_normal(weights[nm].shape).astype(np.float32))
        payload[f"opt/m/{i}"], payload[f"opt/v/{i}"] = moments[nm]
    hdr = {"step": 4, "meta": {}, "optimizer": {"t": 4, "lr": 1e-3}}
    if scheduler_step is not None:
        hdr["scheduler_step"] = scheduler_step
    payload["__header__"] = np.frombuffer(json.dumps(hdr).encode(), dtype=np.uint8)
    np.savez(path, **payload)
    return moments


def test_reference_file_with_an_optimizer_over_the_adapters_only(tmp_path):
    """An eager adapter run saves every model tensor but moments only for the trainable ones: they are matched to the
    adapter parameters in model order with a shape check; a count that fits neither reading is refused."""
    rng = np.random.default_rng(3)
    shapes = {"embed.weight": (16, 8), "blocks.0.attn.q_proj.weight": (8, 8), "blocks.0.attn.q_proj.lora_a": (8, 4),
              "blocks.0.attn.q_proj.lora_b": (4, 8), "norm.weight": (8,)}
    weights = {nm: rng.standard_normal(sh).astype(np.float32) for nm, sh in shapes.items()}
    adapters = [nm for nm in shapes if "lora_" in nm]
    p = str(tmp_path / "ref.npz")
    moments = _reference_style_file(p, weights, adapters, scheduler_step=11)
    hdr, st = C.read(p)
    assert hdr["scheduler_step"] == 11
    for nm in adapters:
        assert np.array_equal(st[f"m/{nm}"], moments[nm][0]) and np.array_equal(st[f"v/{nm}"], moments[nm][1])
    assert "m/embed.weight" not in st
    ct = FakeStep({nm: shapes[nm] for nm in adapters})           # the compiled adapter step owns the adapters only
    C.load(p, ct)
    assert all(np.array_equal(ct.st[f"m/{nm}"], moments[nm][0]) for nm in adapters)
    _reference_style_file(p, weights, list(shapes)[:3])          # three moments: neither all five nor the two adapters
    with pytest.raises(ValueError):
        C.read(p)
    _reference_style_file(p, weights, list(shapes))              # a moment per parameter: the plain case
    _, st = C.read(p)
    assert all(f"m/{nm}" in st for nm in shapes)


def test_moment_shapes_are_checked_and_the_schedule_position_travels(tmp_path):
    a = FakeStep(SHAPES, seed=1)
    p = str(tmp_path / "a.npz")
    C.save(p, a, step=3, scheduler_step=42)
    hdr = C.load(p, FakeStep(SHAPES, seed=2))
    assert hdr["scheduler_step"] == 42
    a.st["m/norm.weight"] = np.zeros((9,), np.float32)            # a moment of the wrong shape
    C.save(p, a, step=3)
    with pytest.raises(ValueError):
        C.load(p, FakeStep(SHAPES, seed=2))
    # the schedule position survives a shard merge
    names = list(SHAPES)
    full, shards = FakeStep(SHAPES, seed=5), []
    for rk, own in enumerate((names[:2], names[2:])):
        s = FakeStep(SHAPES, owned=own, rank=rk, world=2)
        s.st = {k: v for k, v in full.st.items() if k[:2] in ("w/", "m/", "v/") and k[2:] in own}
        s.st["_t"], s.st["_lr"] = full.st["_t"], full.st["_lr"]
        shards.append(str(tmp_path / f"s{rk}.npz"))
        C.save(shards[-1], s, step=9, scheduler_step=17)
    assert C.merge_shards(shards, str(tmp_path / "f.npz")).get("scheduler_step") == 17
    assert C.read(str(tmp_path / "f.npz"))[0]["scheduler_step"] == 17
