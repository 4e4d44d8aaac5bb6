"""ctypes wrapper around oracle/liblumi_oracle.so (TEST INFRASTRUCTURE, NOT PRODUCT).

Only tests, the smoke check and the benchmark's CPU-baseline legs import this module.
Parity unpinned: see the header of lumi_oracle.cpp.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from typing import Optional

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liblumi_oracle.so")
_lib = None


def build(force: bool = False) -> str:
    src = os.path.join(_HERE, "lumi_oracle.cpp")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-B", "liblumi_oracle.so"], check=True,
                       stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
    return _LIB_PATH


def lib():
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(_LIB_PATH)
        L.oracle_set_threads.restype = C.c_int32
        L.oracle_set_threads.argtypes = [C.c_int32]
        L.oracle_model_new.restype = C.c_void_p
        L.oracle_model_new.argtypes = [C.c_void_p, C.c_float, C.c_void_p, C.c_void_p]
        L.oracle_model_free.argtypes = [C.c_void_p]
        L.oracle_set_tensor.argtypes = [C.c_void_p, C.c_char_p, C.c_void_p, C.c_int64]
        L.oracle_state_new.restype = C.c_void_p
        L.oracle_state_new.argtypes = [C.c_void_p]
        L.oracle_state_free.argtypes = [C.c_void_p]
        L.oracle_forward_step.argtypes = [C.c_void_p, C.c_void_p, C.c_uint32, C.c_void_p, C.c_void_p]
        L.oracle_mamba_block.argtypes = [C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p]
        L.oracle_attention_block.argtypes = [C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p]
        L.oracle_read_state.argtypes = [C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p]
        L.oracle_argmax.restype = C.c_uint32
        L.oracle_argmax.argtypes = [C.c_void_p, C.c_int32]
        L.oracle_sample.restype = C.c_uint32
        L.oracle_sample.argtypes = [C.c_void_p, C.c_int32, C.c_double, C.c_int32, C.c_float]
        L.oracle_generate.restype = C.c_int32
        L.oracle_generate.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_double,
                                      C.c_int32, C.c_void_p, C.c_uint32, C.c_int32, C.c_void_p, C.c_void_p]
        _lib = L
    return _lib


def _p(a: Optional[np.ndarray]):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


class OracleModel:
    """The reference's `NmModel` restated on the CPU: load / init_states / forward_step."""

    def __init__(self, cfg, tensors):
        """cfg: lumi_b200.synth.ModelConfig; tensors: iterable of (name with `item.` prefix, dtype, array)."""
        from lumi_b200 import synth
        self.cfg = cfg
        ints = np.array([cfg.d_model, cfg.n_layers, cfg.d_state, cfg.expand, cfg.n_heads, cfg.n_groups,
                         cfg.vocab_size, cfg.attn_n_heads, cfg.attn_kv_heads, cfg.mlp_dim], dtype=np.int32)
        is_attn = np.array([1 if cfg.is_attention_layer(i) else 0 for i in range(cfg.n_layers)], dtype=np.uint8)
        window = np.zeros(cfg.n_layers, dtype=np.int32)
        ai = 0
        for i in range(cfg.n_layers):
            if is_attn[i]:
                window[i] = cfg.attn_window_size(ai)
                ai += 1
        self._m = lib().oracle_model_new(_p(ints), float(cfg.attn_rope_base), _p(is_attn), _p(window))
        for name, dt, arr in tensors:
            assert name.startswith("item.")
            a = np.ascontiguousarray(synth.as_f32(dt, arr), dtype=np.float32)
            lib().oracle_set_tensor(self._m, name[5:].encode(), _p(a), a.size)

    def __del__(self):
        if getattr(self, "_m", None):
            lib().oracle_model_free(self._m)
            self._m = None

    def init_states(self) -> "OracleState":
        return OracleState(self)


class OracleState:
    def __init__(self, model: OracleModel):
        self.model = model
        self._s = lib().oracle_state_new(model._m)

    def __del__(self):
        if getattr(self, "_s", None):
            lib().oracle_state_free(self._s)
            self._s = None

    def forward_step(self, token: int, want_hidden: bool = False):
        cfg = self.model.cfg
        logits = np.empty(cfg.vocab_size, dtype=np.float32)
        hidden = np.empty(cfg.d_model, dtype=np.float32) if want_hidden else None
        lib().oracle_forward_step(self.model._m, self._s, int(token), _p(logits), _p(hidden))
        return (logits, hidden) if want_hidden else logits

    def mamba_block(self, layer: int, x: np.ndarray) -> np.ndarray:
        x = np.array(x, dtype=np.float32, copy=True)
        lib().oracle_mamba_block(self.model._m, self._s, layer, _p(x))
        return x

    def attention_block(self, layer: int, x: np.ndarray) -> np.ndarray:
        x = np.array(x, dtype=np.float32, copy=True)
        lib().oracle_attention_block(self.model._m, self._s, layer, _p(x))
        return x

    def read_state(self, layer: int):
        cfg = self.model.cfg
        h = np.empty((cfg.n_heads, cfg.head_dim, cfg.d_state), dtype=np.float32)
        pbx = np.empty_like(h)
        cum = np.empty((cfg.n_heads, cfg.d_state // 2), dtype=np.float32)
        lib().oracle_read_state(self._s, layer, _p(h), _p(pbx), _p(cum))
        return h, pbx, cum

    def generate(self, prompt, n_new: int, temperature: float = 0.0, top_k: int = 0, uniforms=None,
                 eos: int = 2, ignore_eos: bool = False, dump_logits: bool = False):
        cfg = self.model.cfg
        prompt = np.ascontiguousarray(prompt, dtype=np.uint32)
        out = np.zeros(n_new, dtype=np.uint32)
        dump = np.zeros((n_new, cfg.vocab_size), dtype=np.float32) if dump_logits else None
        u = None if uniforms is None else np.ascontiguousarray(uniforms, dtype=np.float32)
        n = lib().oracle_generate(self.model._m, self._s, _p(prompt), len(prompt), n_new, float(temperature),
                                  int(top_k), _p(u), int(eos), int(bool(ignore_eos)), _p(out), _p(dump))
        return (out[:n], dump[:n]) if dump_logits else out[:n]


def set_threads(n: int) -> int:
    """Sets the OpenMP thread count of the oracle's matvecs; returns the count in effect."""
    return int(lib().oracle_set_threads(int(n)))


def argmax(logits: np.ndarray) -> int:
    a = np.ascontiguousarray(logits, dtype=np.float32)
    return int(lib().oracle_argmax(_p(a), a.size))


def sample(logits: np.ndarray, temperature: float, top_k: int, r: float) -> int:
    a = np.ascontiguousarray(logits, dtype=np.float32)
    return int(lib().oracle_sample(_p(a), a.size, float(temperature), int(top_k), float(r)))
