"""Weight containers shaped like the reference's `axis.nn.Transformer`, enough
for `compile_model` (which only reads names, arrays and a few attributes).
They hold parameters; all arithmetic happens in the engine."""
from __future__ import annotations

from types import SimpleNamespace
from typing import Dict, Iterator, Sequence, Tuple

import numpy as np


class Param:
    def __init__(self, data: np.ndarray):
        self.data = np.ascontiguousarray(data, dtype=np.float32)


class Transformer:
    """Parameter set of a Llama-class decoder (names as in axis/nn.py:331-364).
    2-D tensors ~ N(0, std) drawn in `named_parameters()` order from
    `default_rng(seed)`; norm weights are ones."""

    def __init__(self, vocab_size: int, dim: int, n_layers: int, n_heads: int,
                 n_kv_heads: int = None, mlp_hidden: int = None, tie_embeddings: bool = True,
                 seed: int = 42, std: float = 0.02):
        n_kv_heads = n_kv_heads or n_heads
        mlp_hidden = mlp_hidden or int(dim * 8 / 3)
        dh = dim // n_heads
        self.tie_embeddings = tie_embeddings
        self.blocks = [SimpleNamespace(attn=SimpleNamespace(n_heads=n_heads, n_kv_heads=n_kv_heads))
                       for _ in range(n_layers)]
        rng = np.random.default_rng(seed)
        self._params: Dict[str, Param] = {}
        self.lora_scaling = None

        def mat(name, shape):
            self._params[name] = Param((rng.standard_normal(shape) * std).astype(np.float32))

        def ones(name, n):
            self._params[name] = Param(np.ones(n, dtype=np.float32))
        mat("embed.weight", (vocab_size, dim))
        for i in range(n_layers):
            p = f"blocks.{i}."
            ones(p + "attn_norm.weight", dim)
            mat(p + "attn.q_proj.weight", (dim, n_heads * dh))
            mat(p + "attn.k_proj.weight", (dim, n_kv_heads * dh))
            mat(p + "attn.v_proj.weight", (dim, n_kv_heads * dh))
            mat(p + "attn.o_proj.weight", (n_heads * dh, dim))
            ones(p + "mlp_norm.weight", dim)
            mat(p + "mlp.gate_proj.weight", (dim, mlp_hidden))
            mat(p + "mlp.up_proj.weight", (dim, mlp_hidden))
            mat(p + "mlp.down_proj.weight", (mlp_hidden, dim))
        ones("norm.weight", dim)
        if not tie_embeddings:
            mat("lm_head.weight", (dim, vocab_size))

    def named_parameters(self) -> Iterator[Tuple[str, Param]]:
        return iter(self._params.items())

    def apply_lora(self, rank: int, alpha: float,
                   targets: Sequence[str] = ("q_proj", "k_proj", "v_proj", "o_proj",
                                             "gate_proj", "up_proj", "down_proj"),
                   seed: int = 7, std: float = 0.02) -> "Transformer":
        """Add adapters A ~ N(0, std) [in, r], B = 0 [r, out] on the named
        projections (W_eff = W + alpha/r * A B, axis/lora.py:29-54); the base
        weights become frozen when the model is compiled."""
        rng = np.random.default_rng(seed)
        new: Dict[str, Param] = {}
        for name, p in self._params.items():
            parts = name.split(".")
            if len(parts) == 5 and parts[3] in targets and parts[4] == "weight":
                stem = ".".join(parts[:4])
                fin, fout = p.data.shape
                new[stem + ".base.weight"] = p
                new[stem + ".lora_a"] = Param((rng.standard_normal((fin, rank)) * std).astype(np.float32))
                new[stem + ".lora_b"] = Param(np.zeros((rank, fout), dtype=np.float32))
            else:
                new[name] = p
        self._params = new
        self.lora_a = True               # marks the container as adapter-carrying
        self.scaling = float(alpha) / rank
        return self


class LazyNormal:
    """A weight that exists only as (shape, seed): drawn from N(0, std) (ones for 1-D tensors) at the moment it is
    uploaded, so a model too large to hold on the host in fp32 — every rank of a multi-GPU job builds its own —
    costs one tensor of host memory at a time.  `CompiledTransformer` accepts it wherever it accepts an array
    (the `shape` / `load_into` protocol of pretrained.HfTensor)."""

    def __init__(self, shape, seed, std: float = 0.02):
        self.shape = tuple(int(v) for v in shape)
        self.seed, self.std = seed, std

    def to_f32(self) -> np.ndarray:
        if len(self.shape) == 1:
            return np.ones(self.shape, dtype=np.float32)
        rng = np.random.default_rng(self.seed)
        return rng.standard_normal(self.shape, dtype=np.float32) * np.float32(self.std)

    def load_into(self, eng, dst: int, fp32_out: bool, stage: int) -> None:
        from axis_b200.engine import f32_to_bf16_bits
        a = self.to_f32()
        if fp32_out:
            eng.upload(dst, a.reshape(-1))
        else:
            eng.upload_raw(dst, f32_to_bf16_bits(a))
        eng.sync()                       # the host array is dropped on return


def lazy_weights(cfg: dict, seed: int = 42, std: float = 0.02) -> Dict[str, LazyNormal]:
    """{name: LazyNormal} for a Llama-class decoder configuration (names and shapes as `Transformer`)."""
    V, D, L, H = cfg["vocab_size"], cfg["dim"], cfg["n_layers"], cfg["n_heads"]
    KV = cfg.get("n_kv_heads") or H
    MLP, dh = cfg["mlp_hidden"], D // H
    shapes = {"embed.weight": (V, D)}
    for i in range(L):
        p = f"blocks.{i}."
        shapes.update({p + "attn_norm.weight": (D,), p + "attn.q_proj.weight": (D, H * dh), p + "attn.k_proj.weight": (D, KV * dh),
                       p + "attn.v_proj.weight": (D, KV * dh), p + "attn.o_proj.weight": (H * dh, D), p + "mlp_norm.weight": (D,),
                       p + "mlp.gate_proj.weight": (D, MLP), p + "mlp.up_proj.weight": (D, MLP), p + "mlp.down_proj.weight": (MLP, D)})
    shapes["norm.weight"] = (D,)
    if not cfg.get("tie_embeddings", True):
        shapes["lm_head.weight"] = (D, V)
    return {nm: LazyNormal(sh, [seed, idx], std) for idx, (nm, sh) in enumerate(shapes.items())}
