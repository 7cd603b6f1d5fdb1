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
