"""Checkpoint files for the compiled training step.

File layout: the one the reference's eager checkpoints use (axis/checkpoint.py:19-53), so a file
written here loads there and the other way round — one numpy `.npz` with

    model/<param name>      fp32 master weights
    opt/m/<i>, opt/v/<i>    AdamW moments, i = position of the parameter in `ct.pnames`
    __header__              UTF-8 JSON as uint8: {"step", "meta", "optimizer": {"t", "lr"}, ...}

written atomically (temporary file in the same directory, fsync, rename).  Additions in the header,
ignored by the reference's loader: "pnames" (the parameter order the moment indices refer to) and, for a
ZeRO-1 rank, "owned" (the names this shard holds) with "rank" / "world".

Under ZeRO-1 every rank saves the shard it owns (`save(path_for_rank, ct)`); `merge_shards` joins the
shards into one full checkpoint, as the reference's ZeRO harness merges the owned dictionaries
(engine/modal_zero_test.py:124-131).  `load` accepts a full file on any rank (each rank takes what it owns).
"""
from __future__ import annotations

import json
import os
import tempfile
from typing import Dict, Iterable, List, Optional

import numpy as np


def _write_npz_atomic(path: str, payload: Dict[str, np.ndarray]) -> None:
    d = os.path.dirname(os.path.abspath(path)) or "."
    os.makedirs(d, exist_ok=True)
    fd, tmp = tempfile.mkstemp(dir=d, suffix=".tmp")
    try:
        with os.fdopen(fd, "wb") as f:
            np.savez(f, **payload)
            f.flush()
            os.fsync(f.fileno())
        os.replace(tmp, path)
    except BaseException:
        if os.path.exists(tmp):
            os.unlink(tmp)
        raise


def _pack(state: Dict[str, np.ndarray], pnames: List[str], owned: Iterable[str], step: int, meta: Optional[dict],
          rank: int, world: int, scheduler_step: Optional[int] = None) -> Dict[str, np.ndarray]:
    owned = list(owned)
    index = {nm: i for i, nm in enumerate(pnames)}
    payload: Dict[str, np.ndarray] = {}
    for nm in owned:
        payload[f"model/{nm}"] = np.asarray(state[f"w/{nm}"], dtype=np.float32)
        payload[f"opt/m/{index[nm]}"] = np.asarray(state[f"m/{nm}"], dtype=np.float32)
        payload[f"opt/v/{index[nm]}"] = np.asarray(state[f"v/{nm}"], dtype=np.float32)
    header = {"step": int(step), "meta": meta or {},
              "optimizer": {"t": int(round(float(np.asarray(state["_t"]).reshape(-1)[0]))),
                            "lr": float(np.asarray(state["_lr"]).reshape(-1)[0])},
              "pnames": list(pnames), "owned": owned, "rank": int(rank), "world": int(world)}
    if scheduler_step is not None:      # the reference's key (axis/checkpoint.py:34-35)
        header["scheduler_step"] = int(scheduler_step)
    payload["__header__"] = np.frombuffer(json.dumps(header).encode("utf-8"), dtype=np.uint8)
    return payload


def save(path: str, ct, step: int = 0, meta: Optional[dict] = None, scheduler_step: Optional[int] = None) -> None:
    """Write the state this rank holds (everything, or its ZeRO-1 shard) to `path`.  scheduler_step: the position of
    the caller's learning-rate schedule, stored under the reference's header key."""
    _write_npz_atomic(path, _pack(ct.state_dict(), list(ct.pnames), list(ct.owned), step, meta,
                                  getattr(ct, "rank", 0), getattr(ct, "world", 1), scheduler_step))


def _moment_owners(names: List[str], shapes: Dict[str, tuple], moments: Dict[int, tuple]) -> Dict[str, int]:
    """Which parameter each `opt/m/<i>` of a reference-written file belongs to (such a file names no parameters for its
    moments: they follow the optimizer's parameter list, axis/checkpoint.py:27-33).  With a moment per model entry the
    lists coincide.  With fewer — an optimizer over the trainable subset, e.g. adapters on a frozen base — the
    moments are matched, in order, to the adapter parameters if their count fits, and every pairing must agree in
    shape; anything else is refused rather than guessed."""
    idx = sorted(moments)
    if idx != list(range(len(idx))):
        raise ValueError("optimizer moments are not numbered 0..n-1")
    if len(idx) == len(names):
        cand = names
    else:
        cand = [nm for nm in names if nm.endswith((".lora_a", ".lora_b"))]
        if len(cand) != len(idx):
            raise ValueError(f"{len(idx)} optimizer moments for {len(names)} parameters ({len(cand)} of them adapters): "
                             "the file does not say which parameters the optimizer covered")
    for i, nm in zip(idx, cand):
        if tuple(moments[i]) != tuple(shapes[nm]):
            raise ValueError(f"opt/m/{i} has shape {tuple(moments[i])}, parameter {nm} has {tuple(shapes[nm])}")
    return {nm: i for i, nm in zip(idx, cand)}


def read(path: str):
    """(header, {"w/<name>", "m/<name>", "v/<name>", "_t", "_lr"}) of a checkpoint file."""
    with np.load(path, allow_pickle=False) as z:
        header = json.loads(bytes(z["__header__"]).decode("utf-8"))
        names = [k[len("model/"):] for k in z.files if k.startswith("model/")]
        pnames = header.get("pnames")
        if pnames is not None:
            index = {nm: i for i, nm in enumerate(pnames)}
        else:
            # a file written by the reference
            moments = {int(k.rsplit("/", 1)[1]): z[k].shape for k in z.files if k.startswith("opt/m/")}
            index = _moment_owners(names, {nm: z[f"model/{nm}"].shape for nm in names}, moments) if moments else {}
        state: Dict[str, np.ndarray] = {}
        for nm in names:
            state[f"w/{nm}"] = z[f"model/{nm}"]
            if nm in index:
                mk, vk = f"opt/m/{index[nm]}", f"opt/v/{index[nm]}"
                if mk in z.files:
                    state[f"m/{nm}"] = z[mk]
                    state[f"v/{nm}"] = z[vk]
        opt = header.get("optimizer", {"t": 0, "lr": 0.0})
        state["_t"] = np.array([opt["t"]], dtype=np.float32)
        state["_lr"] = np.array([opt["lr"]], dtype=np.float32)
    return header, state


def load(path: str, ct) -> dict:
    """Restore `ct` from a checkpoint holding at least what this rank owns; returns the header."""
    header, state = read(path)
    missing = [nm for nm in ct.owned if f"w/{nm}" not in state]
    if missing:
        raise KeyError(f"checkpoint {path} lacks {len(missing)} tensors this rank owns, e.g. {missing[0]}")
    for nm in ct.owned:
        if tuple(state[f"w/{nm}"].shape) != tuple(ct.shapes[nm]):
            raise ValueError(f"{nm}: checkpoint shape {state[f'w/{nm}'].shape} != model shape {ct.shapes[nm]}")
        if f"m/{nm}" not in state:      # weights-only file: fresh optimizer state
            state[f"m/{nm}"] = np.zeros(ct.shapes[nm], np.float32)
            state[f"v/{nm}"] = np.zeros(ct.shapes[nm], np.float32)
        for pre in ("m/", "v/"):
            if tuple(state[pre + nm].shape) != tuple(ct.shapes[nm]):
                raise ValueError(f"{nm}: checkpoint moment {pre[0]} has shape {state[pre + nm].shape}, model has {ct.shapes[nm]}")
    ct.load_state_dict(state)
    return header               # "scheduler_step", when the writer had a schedule, is in the header for the caller's schedule


def merge_shards(paths: Iterable[str], out_path: str) -> dict:
    """Join per-rank ZeRO-1 shard files into one full checkpoint; checks that the shards agree on the step
    counters and that together they hold every parameter exactly once."""
    paths = list(paths)
    if not paths:
        raise ValueError("no shard files")
    merged: Dict[str, np.ndarray] = {}
    first = None
    seen: Dict[str, str] = {}
    for p in paths:
        header, state = read(p)
        if first is None:
            first = header
        else:
            for k in ("step", "pnames", "scheduler_step"):
                if header.get(k) != first.get(k):
                    raise ValueError(f"shard {p} disagrees with {paths[0]} on {k}")
            if header["optimizer"] != first["optimizer"]:
                raise ValueError(f"shard {p} disagrees with {paths[0]} on the optimizer counters")
        for nm in header.get("owned", [k[2:] for k in state if k.startswith("w/")]):
            if nm in seen:
                raise ValueError(f"{nm} is in both {seen[nm]} and {p}")
            seen[nm] = p
            for pre in ("w/", "m/", "v/"):
                merged[pre + nm] = state[pre + nm]
    pnames = first["pnames"]
    lacking = [nm for nm in pnames if nm not in seen]
    if lacking:
        raise ValueError(f"shards lack {len(lacking)} parameters, e.g. {lacking[0]}")
    merged["_t"] = np.array([first["optimizer"]["t"]], np.float32)
    merged["_lr"] = np.array([first["optimizer"]["lr"]], np.float32)
    _write_npz_atomic(out_path, _pack(merged, pnames, pnames, first["step"], first.get("meta"), 0, 1,
                                      first.get("scheduler_step")))
    return first
