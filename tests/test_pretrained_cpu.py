"""Checkpoint directory (config.json + safetensors shards, HuggingFace Llama names, [out,in] projections,
bf16) -> compiled step without an fp32 host copy: names, layouts and values as the reference's loader
produces them (axis/pretrained.py:88-153), on the plan interpreter."""
import json
import os
import struct

import numpy as np
import pytest

from axis_b200 import engine as E
from axis_b200.compile import CompiledTransformer
from axis_b200.pretrained import HfTensor, compile_pretrained, open_checkpoint, open_safetensors
from oracle import step_numpy as O
from tests.plan_interp import InterpEngine

CFG = dict(vocab_size=67, dim=32, n_layers=2, n_heads=4, n_kv_heads=2, mlp_hidden=40, tie_embeddings=False)


def write_safetensors(path, tensors):
    """tensors: {name: (tag, ndarray of the stored dtype)}"""
    header, blobs, off = {}, [], 0
    for name, (tag, arr) in tensors.items():
        raw = np.ascontiguousarray(arr).tobytes()
        header[name] = {"dtype": tag, "shape": list(arr.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    header["__metadata__"] = {"format": "pt"}
    hj = json.dumps(header).encode("utf-8")
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)


def make_checkpoint(tmp, cfg, tag="BF16", shards=2, seed=0):
    """A checkpoint directory in HuggingFace layout from the oracle's weights; returns the weights a correct
    loader must produce (engine layout, fp32, rounded to the stored type)."""
    w = O.init_weights(cfg, seed=seed)
    rng = np.random.default_rng(seed)
    for k in w:                                   # norm weights away from 1 so a mix-up shows
        if k.endswith("norm.weight"):
            w[k] = (1.0 + 0.1 * rng.standard_normal(w[k].shape)).astype(np.float32)
    enc = (lambda a: E.f32_to_bf16_bits(a).reshape(a.shape)) if tag == "BF16" else \
          (lambda a: a.astype(np.float16 if tag == "F16" else np.float32))
    dec = (lambda a: E.bf16_bits_to_f32(a).reshape(a.shape)) if tag == "BF16" else (lambda a: a.astype(np.float32))
    hf, expect = {}, {}

    def add(hf_name, name, transposed):
        stored = enc(np.ascontiguousarray(w[name].T) if transposed else w[name])
        hf[hf_name] = (tag, stored)
        expect[name] = np.ascontiguousarray(dec(stored).T) if transposed else dec(stored)
    add("model.embed_tokens.weight", "embed.weight", False)
    add("model.norm.weight", "norm.weight", False)
    if not cfg["tie_embeddings"]:
        add("lm_head.weight", "lm_head.weight", True)
    for i in range(cfg["n_layers"]):
        h, a = f"model.layers.{i}.", f"blocks.{i}."
        add(h + "input_layernorm.weight", a + "attn_norm.weight", False)
        add(h + "post_attention_layernorm.weight", a + "mlp_norm.weight", False)
        for p in ("q_proj", "k_proj", "v_proj", "o_proj"):
            add(h + f"self_attn.{p}.weight", a + f"attn.{p}.weight", True)
        for p in ("gate_proj", "up_proj", "down_proj"):
            add(h + f"mlp.{p}.weight", a + f"mlp.{p}.weight", True)
    hf["model.layers.0.self_attn.rotary_emb.inv_freq"] = ("F32", np.ones(4, np.float32))    # ignored extra
    hf["some.int.table"] = ("I64", np.arange(3, dtype=np.int64))
    names = list(hf)
    per = (len(names) + shards - 1) // shards
    wmap = {}
    for s in range(shards):
        fn = "model.safetensors" if shards == 1 else f"model-{s + 1:05d}-of-{shards:05d}.safetensors"
        part = {n: hf[n] for n in names[s * per:(s + 1) * per]}
        write_safetensors(os.path.join(tmp, fn), part)
        wmap.update({n: fn for n in part})
    if shards > 1:
        with open(os.path.join(tmp, "model.safetensors.index.json"), "w") as f:
            json.dump({"weight_map": wmap}, f)
    with open(os.path.join(tmp, "config.json"), "w") as f:
        json.dump(dict(vocab_size=cfg["vocab_size"], hidden_size=cfg["dim"], num_hidden_layers=cfg["n_layers"],
                       num_attention_heads=cfg["n_heads"], num_key_value_heads=cfg["n_kv_heads"],
                       intermediate_size=cfg["mlp_hidden"], rms_norm_eps=1e-6, rope_theta=50000.0,
                       tie_word_embeddings=cfg["tie_embeddings"]), f)
    return expect


@pytest.mark.parametrize("tag,shards,tied", [("BF16", 2, False), ("BF16", 1, True), ("F32", 1, False), ("F16", 3, True)])
@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
def test_checkpoint_weights_arrive_in_engine_layout(tmp_path, tag, shards, tied, dtype):
    cfg = dict(CFG, tie_embeddings=tied)
    expect = make_checkpoint(str(tmp_path), cfg, tag, shards)
    ct = compile_pretrained(str(tmp_path), 2, 8, lib_path=InterpEngine(), dtype=dtype)
    assert ct.cfg["rope_theta"] == 50000.0 and ct.cfg["norm_eps"] == 1e-6
    got = ct.get_weights()
    assert set(got) == set(expect)
    for nm in expect:
        assert got[nm].shape == expect[nm].shape and np.array_equal(got[nm], expect[nm]), nm
    # and the step is the step of the same weights handed over as fp32 arrays
    ref = CompiledTransformer(InterpEngine(), dict(cfg, rope_theta=50000.0), expect, 2, 8, dtype=dtype, eps=1e-6)
    rng = np.random.default_rng(3)
    x, y = O.make_batch(rng, cfg["vocab_size"], 2, 8, 0.1)
    assert ct.step(x, y) == ref.step(x, y)
    wa, wb = ct.get_weights(), ref.get_weights()
    for nm in wa:
        assert np.array_equal(wa[nm], wb[nm]), nm


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
def test_lora_base_goes_to_the_device_without_an_fp32_copy(tmp_path, dtype):
    expect = make_checkpoint(str(tmp_path), CFG, "BF16", 2)
    eng = InterpEngine()
    ct = compile_pretrained(str(tmp_path), 2, 8, lib_path=eng, dtype=dtype, lora_r=4, lora_alpha=8.0,
                            lora_targets=("q_proj", "v_proj", "down_proj"))
    assert ct.lora_r == 4 and all(nm.endswith(("lora_a", "lora_b")) for nm in ct.pnames)
    for nm, w in expect.items():                  # the frozen compute copies
        if dtype == "bf16":
            got = E.bf16_bits_to_f32(eng.download_raw(ct.pb[nm], w.size, np.uint16)).reshape(w.shape)
        else:
            got = eng.download(ct.pb[nm], w.shape)
        assert np.array_equal(got, w), nm
    ref = CompiledTransformer(InterpEngine(), dict(CFG, rope_theta=50000.0), expect, 2, 8, dtype=dtype, eps=1e-6,
                              lora_r=4, lora_alpha=8.0, lora_targets=("q_proj", "v_proj", "down_proj"))
    rng = np.random.default_rng(5)
    x, y = O.make_batch(rng, CFG["vocab_size"], 2, 8, 0.1)
    for _ in range(2):                            # second step: adapters have moved, the base has not
        assert ct.step(x, y) == ref.step(x, y)


def test_reader_and_mapping_reject_bad_input(tmp_path):
    expect = make_checkpoint(str(tmp_path), CFG, "BF16", 1)
    cfg, tensors = open_checkpoint(str(tmp_path))
    assert cfg["n_kv_heads"] == 2 and set(tensors) == set(expect)
    t = tensors["blocks.1.mlp.down_proj.weight"]
    assert isinstance(t, HfTensor) and t.transposed and t.shape == (CFG["mlp_hidden"], CFG["dim"])
    assert t.data.shape == (CFG["dim"], CFG["mlp_hidden"]) and t.data.dtype == np.uint16
    assert np.array_equal(t.to_f32(), expect["blocks.1.mlp.down_proj.weight"])
    assert not tensors["embed.weight"].transposed
    raw = open_safetensors(os.path.join(str(tmp_path), "model.safetensors"))
    assert "some.int.table" not in raw and raw["model.norm.weight"][0] == "BF16"
    # a parameter without a tensor
    part = {k: v for k, v in raw.items() if k != "model.layers.1.mlp.up_proj.weight"}
    d2 = tmp_path / "lacking"
    d2.mkdir()
    write_safetensors(str(d2 / "model.safetensors"), part)
    (d2 / "config.json").write_text((tmp_path / "config.json").read_text())
    with pytest.raises(KeyError, match="up_proj"):
        open_checkpoint(str(d2))
    # offsets that do not match the shape
    d3 = tmp_path / "broken"
    d3.mkdir()
    hj = json.dumps({"x": {"dtype": "BF16", "shape": [4, 4], "data_offsets": [0, 30]}}).encode()
    (d3 / "model.safetensors").write_bytes(struct.pack("<Q", len(hj)) + hj + bytes(32))
    with pytest.raises(ValueError, match="bytes for shape"):
        open_safetensors(str(d3 / "model.safetensors"))
    with pytest.raises(FileNotFoundError):
        open_checkpoint_dir = tmp_path / "empty"
        open_checkpoint_dir.mkdir()
        (open_checkpoint_dir / "config.json").write_text((tmp_path / "config.json").read_text())
        open_checkpoint(str(open_checkpoint_dir))
