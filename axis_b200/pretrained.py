"""Fast load of a HuggingFace Llama-family checkpoint into the compiled training step.

The reference reaches the compiled engine through `from_pretrained` (axis/pretrained.py:131-153): every
safetensors shard is read whole, each bf16 tensor is widened to fp32 on the host, every projection is
transposed on the host ([out,in] -> the engine's [in,out], axis/pretrained.py:88-110), the fp32 model is handed
to `compile_model`, and the frozen base of a LoRA run then goes through one fp32 staging buffer on the device to
become bf16 again (axis/compile.py:144-153).

Here the shards are memory-mapped and the bf16 bits go to the device as they lie in the file; the layout change
and, for trainable weights, the widening to the fp32 master happen on the device (TRANSPOSE_BF16 / CAST through
one staging buffer the size of the largest tensor).  No fp32 copy of the model exists on the host, and for a LoRA
run none exists anywhere.  fp32 / fp16 checkpoints take the host path (widen, transpose, upload).

    ct = compile_pretrained(model_dir, batch=1, seq=8192, dtype="bf16", lora_r=16, lora_alpha=32.0)

Name and layout mapping (axis/pretrained.py:88-110): embedding and norm weights map directly; the seven
projections of a block are transposed; q/k need no permutation (both sides use the half-split rotary
convention); `lm_head.weight` is used only when the embeddings are not tied.
"""
from __future__ import annotations

import json
import os
import struct
from typing import Dict, Tuple

import numpy as np

from .compile import CompiledTransformer
from .engine import CAST, TRANSPOSE_BF16, bf16_bits_to_f32, f32_to_bf16_bits, op

# safetensors dtype tag -> numpy dtype of the stored bytes (bf16 is kept as its 16-bit pattern)
_ST_DTYPES = {"F64": np.float64, "F32": np.float32, "F16": np.float16, "BF16": np.uint16}


class HfTensor:
    """One checkpoint tensor, still in its file layout (normally a view of a memory-mapped shard).

    `shape` is the shape in the engine's layout: reversed for a transposed projection."""

    def __init__(self, data: np.ndarray, st_dtype: str, transposed: bool):
        if transposed and data.ndim != 2:
            raise ValueError("only matrices are transposed")
        self.data, self.st_dtype, self.transposed = data, st_dtype, bool(transposed)

    @property
    def shape(self) -> Tuple[int, ...]:
        return tuple(reversed(self.data.shape)) if self.transposed else tuple(self.data.shape)

    def to_f32(self) -> np.ndarray:
        """Host copy in the engine's layout, fp32 (the slow path; also what the tests compare with)."""
        a = bf16_bits_to_f32(np.asarray(self.data)).reshape(self.data.shape) if self.st_dtype == "BF16" \
            else np.asarray(self.data, dtype=np.float32)
        return np.ascontiguousarray(a.T if self.transposed else a)

    def load_into(self, eng, dst: int, fp32_out: bool, stage: int) -> None:
        """Fill device buffer `dst` (engine layout; fp32 or bf16) from the file bytes."""
        if self.st_dtype != "BF16":
            a = self.to_f32()
            if fp32_out:
                eng.upload(dst, a.reshape(-1))
            else:
                eng.upload_raw(dst, f32_to_bf16_bits(a))
            return
        if not self.transposed and not fp32_out:
            eng.upload_raw(dst, self.data)
            return
        eng.upload_raw(stage, self.data)
        if self.transposed:
            rows, cols = self.data.shape
            eng.run([op(TRANSPOSE_BF16, a=stage, c=dst, m=rows, n=cols, dt=0 if fp32_out else 1)], sync=False)
        else:
            eng.run([op(CAST, a=stage, c=dst, m=int(self.data.size), tb=1)], sync=False)


def open_safetensors(path: str) -> Dict[str, Tuple[str, np.ndarray]]:
    """{name: (dtype tag, array)} of one .safetensors file: an 8-byte little-endian header length, a JSON header
    with dtype / shape / data_offsets per tensor, then the tensor bytes.  Arrays are views of one read-only
    memory map; nothing is read until it is used."""
    with open(path, "rb") as f:
        (hlen,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(hlen).decode("utf-8"))
    size = os.path.getsize(path)
    blob = np.memmap(path, dtype=np.uint8, mode="r", offset=8 + hlen) if size > 8 + hlen else np.zeros(0, np.uint8)
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        tag = meta["dtype"]
        if tag not in _ST_DTYPES:
            continue                         # integer / bool side tensors are of no use to the training step
        b, e = meta["data_offsets"]
        shape = tuple(meta["shape"])
        dt = np.dtype(_ST_DTYPES[tag])
        n = int(np.prod(shape)) if shape else 1
        if e - b != n * dt.itemsize or e > blob.size:
            raise ValueError(f"{path}: {name} has {e - b} bytes for shape {shape} of {tag}")
        out[name] = (tag, blob[b:e].view(dt).reshape(shape))
    return out


def _open_all_shards(model_dir: str) -> Dict[str, Tuple[str, np.ndarray]]:
    index = os.path.join(model_dir, "model.safetensors.index.json")
    single = os.path.join(model_dir, "model.safetensors")
    if os.path.exists(index):
        with open(index) as f:
            files = sorted(set(json.load(f)["weight_map"].values()))
    elif os.path.exists(single):
        files = ["model.safetensors"]
    else:
        files = sorted(fn for fn in os.listdir(model_dir) if fn.endswith(".safetensors"))
        if not files:
            raise FileNotFoundError(f"no .safetensors found in {model_dir}")
    state = {}
    for fn in files:
        state.update(open_safetensors(os.path.join(model_dir, fn)))
    return state


def config_from_hf(cfg: dict) -> dict:
    """HF Llama config.json -> the configuration dictionary of CompiledTransformer (axis/pretrained.py:114-128)."""
    return dict(vocab_size=cfg["vocab_size"], dim=cfg["hidden_size"], n_layers=cfg["num_hidden_layers"],
                n_heads=cfg["num_attention_heads"],
                n_kv_heads=cfg.get("num_key_value_heads", cfg["num_attention_heads"]),
                mlp_hidden=cfg["intermediate_size"], rope_theta=cfg.get("rope_theta", 10000.0),
                norm_eps=cfg.get("rms_norm_eps", 1e-5), tie_embeddings=cfg.get("tie_word_embeddings", False))


def open_checkpoint(model_dir: str):
    """(configuration, {engine parameter name: HfTensor}) of a checkpoint directory (config.json + safetensors).
    Raises KeyError when a parameter of the architecture has no tensor (axis/pretrained.py:145-151)."""
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = config_from_hf(json.load(f))
    hf = _open_all_shards(model_dir)
    want = [("embed.weight", "model.embed_tokens.weight", False), ("norm.weight", "model.norm.weight", False)]
    if not cfg["tie_embeddings"]:
        want.append(("lm_head.weight", "lm_head.weight", True))
    for i in range(cfg["n_layers"]):
        h, a = f"model.layers.{i}.", f"blocks.{i}."
        want += [(a + "attn_norm.weight", h + "input_layernorm.weight", False),
                 (a + "mlp_norm.weight", h + "post_attention_layernorm.weight", False)]
        want += [(a + f"attn.{p}.weight", h + f"self_attn.{p}.weight", True) for p in ("q_proj", "k_proj", "v_proj", "o_proj")]
        want += [(a + f"mlp.{p}.weight", h + f"mlp.{p}.weight", True) for p in ("gate_proj", "up_proj", "down_proj")]
    missing = [src for _, src, _ in want if src not in hf]
    if missing:
        raise KeyError(f"checkpoint lacks {len(missing)} tensors, e.g. {missing[:5]}")
    return cfg, {dst: HfTensor(hf[src][1], hf[src][0], tr) for dst, src, tr in want}


def compile_pretrained(model_dir: str, batch: int, seq: int, lib_path: str = None, dtype: str = "bf16",
                       **kw) -> CompiledTransformer:
    """The compiled training step of a checkpoint directory.  `kw` goes to CompiledTransformer (lr, wd,
    lora_r / lora_alpha / lora_targets, max_grad_norm, grad_sync, zero_stage, rank, world, recompute_blocks ...).
    The norm epsilon comes from the checkpoint's configuration unless given."""
    cfg, weights = open_checkpoint(model_dir)
    kw.setdefault("eps", cfg["norm_eps"])
    return CompiledTransformer(lib_path, cfg, weights, batch, seq, dtype=dtype, **kw)
