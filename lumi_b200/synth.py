"""Seeded synthetic `config.json` + weight sets in the reference's safetensors schema.

Tensor names, shapes and the `item.` prefix follow the loader of the reference
(inference/src/main.rs:83-86, inference/src/model.rs:185-231, 469-489, 643-728) and its
export script (scripts/export_native_safetensors.py:103-143).

Initialisation (the benchmark configurations name the distributions; the trainer's own
init is training/src/native_trainer.rs:1871-1994):
  * `embedding.weight`, `in_proj.weight`, attention/MLP matrices ~ N(0, 0.02)
  * `out_proj.weight`, `attn_out_proj.weight`, `mlp_down.weight` ~ N(0, 0.02) / sqrt(2 * n_layers)
  * `ssm.dt_bias` ~ U(-4, -1)   (the only bias in the dt / A chain; in_proj has no bias)
  * `b_norm.gamma`, `c_norm.gamma`, `b_bias`, `c_bias`, `norm.gamma`, `final_norm.gamma`, `ssm.d` = 1
  * `ssm.h_init` ~ N(0, 0.01), stored 2-D `[n_heads, d_state]` (the shape the loader asks for,
    inference/src/model.rs:214)
Every tensor draws from its own Philox stream keyed by (seed, crc32(name)), so a tensor's values
do not depend on which other tensors exist or on generation order.

`weights_dtype="bf16"` rounds rank-2 tensors to bfloat16 (round to nearest even); rank-1 tensors
and `h_init` stay fp32.
"""
from __future__ import annotations

import json
import zlib
from dataclasses import dataclass, field, asdict
from typing import Dict, Iterator, List, Tuple

import numpy as np

F32 = 0
BF16 = 1


@dataclass
class ModelConfig:
    """Mirror of `ModelConfig` (inference/src/model.rs:20-86) plus three optional extensions
    (`attn_mlp_dim`, `attn_rope_base`, `norm_eps`) that default to the reference behaviour."""
    d_model: int = 1024
    n_layers: int = 48
    d_state: int = 64
    expand: int = 2
    n_heads: int = 64
    n_groups: int = 8
    vocab_size: int = 32000
    max_seq_len: int = 2048
    attention_interval: int = 0
    attn_n_heads: int = 16
    attn_kv_heads: int = 4
    attn_mlp_expand: int = 4
    attn_window_sizes: List[int] = field(default_factory=list)
    attention_layers: List[int] = field(default_factory=list)
    byte_level: bool = False
    attn_mlp_dim: int = 0          # 0 = attn_mlp_expand * d_model (reference)
    attn_rope_base: float = 0.0    # 0 = no rotary embedding in attention (reference)

    def __post_init__(self):
        if self.byte_level:
            self.vocab_size = 259      # inference/src/main.rs:75-77

    # helper dims, inference/src/model.rs:50-86
    @property
    def d_inner(self): return self.expand * self.d_model
    @property
    def head_dim(self): return self.d_inner // self.n_heads
    @property
    def attn_head_dim(self): return self.d_model // self.attn_n_heads
    @property
    def attn_kv_dim(self): return self.attn_kv_heads * self.attn_head_dim
    @property
    def mlp_dim(self): return self.attn_mlp_dim if self.attn_mlp_dim > 0 else self.attn_mlp_expand * self.d_model
    @property
    def bc_size(self): return self.n_groups * self.d_state
    @property
    def in_proj_out(self):
        return 2 * self.d_inner + 2 * self.bc_size + 3 * self.n_heads + self.n_heads * self.d_state // 2

    def is_attention_layer(self, i: int) -> bool:
        if self.attention_layers:
            return i in self.attention_layers
        return self.attention_interval > 0 and (i + 1) % self.attention_interval == 0

    def n_attn_layers(self) -> int:
        return sum(1 for i in range(self.n_layers) if self.is_attention_layer(i))

    def attn_window_size(self, attn_idx: int) -> int:
        return self.attn_window_sizes[attn_idx] if attn_idx < len(self.attn_window_sizes) else 0

    def to_json(self) -> str:
        d = asdict(self)
        if d["attn_mlp_dim"] == 0:
            del d["attn_mlp_dim"]
        if d["attn_rope_base"] == 0.0:
            del d["attn_rope_base"]
        return json.dumps(d)

    @staticmethod
    def from_json(text: str) -> "ModelConfig":
        raw = json.loads(text)
        known = {k: raw[k] for k in ModelConfig.__dataclass_fields__ if k in raw}
        return ModelConfig(**known)


def base_config(**kw) -> ModelConfig:
    """The 48-layer base model of the benchmark configurations."""
    return ModelConfig(**kw)


def tiny_config(**kw) -> ModelConfig:
    """d_model 128, 8 heads of 32, d_state 16 — the shape family of the reference's own smoke
    configurations (training/src/native_trainer.rs:1689-1708)."""
    base = dict(d_model=128, n_layers=4, d_state=16, expand=2, n_heads=8, n_groups=2,
                vocab_size=512, max_seq_len=64, attn_n_heads=4, attn_kv_heads=2, attn_mlp_expand=2)
    base.update(kw)
    return ModelConfig(**base)


def f32_to_bf16_bits(a: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even fp32 -> bf16 bit patterns (uint16)."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    rounded = u + (np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1)))
    return (rounded >> np.uint32(16)).astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (b.astype(np.uint32) << np.uint32(16)).view(np.float32)


def _rng(seed: int, name: str) -> np.random.Generator:
    return np.random.Generator(np.random.Philox(key=[seed & 0xFFFFFFFFFFFFFFFF, zlib.crc32(name.encode())]))


def tensor_specs(cfg: ModelConfig) -> List[Tuple[str, Tuple[int, ...], str, float]]:
    """(name without the `item.` prefix, shape, kind, scale) for every tensor of the model."""
    out_scale = 0.02 / float(np.sqrt(2.0 * cfg.n_layers))
    specs: List[Tuple[str, Tuple[int, ...], str, float]] = [
        ("embedding.weight", (cfg.vocab_size, cfg.d_model), "normal", 0.02)]
    for i in range(cfg.n_layers):
        p = f"blocks.{i}."
        if cfg.is_attention_layer(i):
            specs += [
                (p + "attn_norm.gamma", (cfg.d_model,), "ones", 0.0),
                (p + "q_proj.weight", (cfg.d_model, cfg.d_model), "normal", 0.02),
                (p + "k_proj.weight", (cfg.attn_kv_dim, cfg.d_model), "normal", 0.02),
                (p + "v_proj.weight", (cfg.attn_kv_dim, cfg.d_model), "normal", 0.02),
                (p + "attn_out_proj.weight", (cfg.d_model, cfg.d_model), "normal", out_scale),
                (p + "mlp_norm.gamma", (cfg.d_model,), "ones", 0.0),
                (p + "mlp_gate.weight", (cfg.mlp_dim, cfg.d_model), "normal", 0.02),
                (p + "mlp_up.weight", (cfg.mlp_dim, cfg.d_model), "normal", 0.02),
                (p + "mlp_down.weight", (cfg.d_model, cfg.mlp_dim), "normal", out_scale),
            ]
        else:
            specs += [
                (p + "norm.gamma", (cfg.d_model,), "ones", 0.0),
                (p + "in_proj.weight", (cfg.in_proj_out, cfg.d_model), "normal", 0.02),
                (p + "b_norm.gamma", (cfg.bc_size,), "ones", 0.0),
                (p + "c_norm.gamma", (cfg.bc_size,), "ones", 0.0),
                (p + "b_bias", (cfg.bc_size,), "ones", 0.0),
                (p + "c_bias", (cfg.bc_size,), "ones", 0.0),
                (p + "ssm.d", (cfg.n_heads,), "ones", 0.0),
                (p + "ssm.dt_bias", (cfg.n_heads,), "dt_bias", 0.0),
                (p + "ssm.h_init", (cfg.n_heads, cfg.d_state), "h_init", 0.01),
                (p + "out_proj.weight", (cfg.d_model, cfg.d_inner), "normal", out_scale),
            ]
    specs.append(("final_norm.gamma", (cfg.d_model,), "ones", 0.0))
    return specs


def iter_tensors(cfg: ModelConfig, seed: int = 0, weights_dtype: str = "f32",
                 perturb_ones: float = 0.0) -> Iterator[Tuple[str, int, np.ndarray]]:
    """Yield (name with `item.` prefix, dtype code, array). bf16 tensors come as uint16 bit patterns.

    `perturb_ones` > 0 adds N(0, perturb_ones) noise to the all-ones tensors (tests use it so that
    gamma / bias / D indexing mistakes cannot hide behind constant values)."""
    for name, shape, kind, scale in tensor_specs(cfg):
        g = _rng(seed, name)
        if kind == "normal" or kind == "h_init":
            a = g.standard_normal(shape, dtype=np.float32) * np.float32(scale)
        elif kind == "dt_bias":
            a = g.uniform(-4.0, -1.0, shape).astype(np.float32)
        else:
            a = np.ones(shape, dtype=np.float32)
            if perturb_ones > 0.0:
                a = a + g.standard_normal(shape, dtype=np.float32) * np.float32(perturb_ones)
        if weights_dtype == "bf16" and len(shape) == 2 and kind == "normal":
            yield "item." + name, BF16, f32_to_bf16_bits(a)
        else:
            yield "item." + name, F32, np.ascontiguousarray(a, dtype=np.float32)


def as_f32(dtype: int, arr: np.ndarray) -> np.ndarray:
    """What the reference loader sees: every tensor converted to fp32 (inference/src/main.rs:83-85)."""
    return bf16_bits_to_f32(arr) if dtype == BF16 else arr


def write_safetensors(path: str, tensors: Dict[str, Tuple[int, np.ndarray]]) -> None:
    """Minimal safetensors writer (8-byte LE header length, JSON header, raw little-endian data)."""
    header = {}
    off = 0
    blobs = []
    for name, (dt, arr) in tensors.items():
        raw = np.ascontiguousarray(arr).tobytes()
        header[name] = {"dtype": "BF16" if dt == BF16 else "F32", "shape": list(arr.shape),
                        "data_offsets": [off, off + len(raw)]}
        off += len(raw)
        blobs.append(raw)
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * ((8 - len(hj) % 8) % 8)
    with open(path, "wb") as f:
        f.write(len(hj).to_bytes(8, "little"))
        f.write(hj)
        for b in blobs:
            f.write(b)


def write_model_dir(dirpath: str, cfg: ModelConfig, seed: int = 0, weights_dtype: str = "f32",
                    perturb_ones: float = 0.0) -> Tuple[str, str]:
    """Write `config.json` and `model.safetensors`; returns their paths."""
    import os
    os.makedirs(dirpath, exist_ok=True)
    cpath = os.path.join(dirpath, "config.json")
    mpath = os.path.join(dirpath, "model.safetensors")
    with open(cpath, "w") as f:
        f.write(cfg.to_json())
    write_safetensors(mpath, {n: (dt, a) for n, dt, a in iter_tensors(cfg, seed, weights_dtype, perturb_ones)})
    return cpath, mpath


def random_prompt_row(b: int, length: int, vocab: int, seed: int = 0) -> np.ndarray:
    """Row `b` of random_prompts(): uniform ids in [3, vocab) from the Philox stream keyed by (seed, b)."""
    g = np.random.Generator(np.random.Philox(key=[seed, 0x70726F6D + b]))
    return g.integers(3, vocab, size=length, dtype=np.uint32)


def random_prompts(batch: int, length: int, vocab: int, seed: int = 0) -> np.ndarray:
    """Uniform ids in [3, vocab): one Philox stream keyed by (seed, sequence index)."""
    out = np.empty((batch, length), dtype=np.uint32)
    for b in range(batch):
        out[b] = random_prompt_row(b, length, vocab, seed)
    return out


# The benchmark configurations 1-5: (config kwargs, weights dtype, batch per GPU, prompt length, decode tokens,
# sampling, prompt seed).  Weights always come from seed 0.  Configuration 5 is the throughput sweep; its batch
# here is one resident wave of a GPU (the first 2048 of the 4096 sequences, whose prompts use seed 1000).
BENCH_CONFIGS = {
    "config1": (dict(), "f32", 1, 32, 256, dict(), 0),
    "config2": (dict(), "bf16", 64, 128, 512, dict(), 0),
    "config3": (dict(n_layers=96), "bf16", 256, 2048, 256, dict(), 0),
    "config4": (dict(attention_interval=6, attn_mlp_dim=2816, attn_rope_base=10000.0), "bf16", 128, 1024, 1024,
                dict(temperature=0.8, top_k=50, seed=1234), 0),
    "config5": (dict(n_layers=96, byte_level=True), "bf16", 2048, 512, 256, dict(), 1000),
}
