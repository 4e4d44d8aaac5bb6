"""Host-side mirror of the reference's inference API over the C ABI (include/lumi_b200.h).

`NmModel.load / init_states / forward_step` and `generate` keep the names and argument meaning of
inference/src/model.rs:643-801 and inference/src/main.rs:96-177; everything runs in
liblumi_b200.so on the GPU.  There is no CPU fallback: importing works anywhere, but the first
call that needs the library raises if it is not built or no CUDA device is present.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Iterable, Optional, Sequence, Tuple

import numpy as np

from . import synth

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "liblumi_b200.so")
_lib = None

# every symbol include/lumi_b200.h declares
EXPORTS = [
    "lumi_last_error", "lumi_model_create", "lumi_model_load_tensor", "lumi_model_load_safetensors",
    "lumi_model_finalize", "lumi_model_free", "lumi_model_info", "lumi_session_create", "lumi_session_reset",
    "lumi_session_free", "lumi_session_set_option", "lumi_prefill", "lumi_prefill_ragged", "lumi_decode_step", "lumi_generate",
    "lumi_decode_loop_device", "lumi_profile_step", "lumi_score", "lumi_session_read_state", "lumi_session_state_bytes", "lumi_session_save_state", "lumi_session_load_state", "lumi_debug_run_block", "lumi_k_gemm_bf16_tcgen05",
    "lumi_k_gemv", "lumi_debug_gemm_wait_timeout", "lumi_debug_gemm_plan", "lumi_k_ssm_step", "lumi_k_ssd_prefill", "lumi_mamba_block_static",
]


class LumiError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"lumi_b200 error {code}: {message}")
        self.code = code
        self.message = message


class Sampling(C.Structure):
    _fields_ = [("temperature", C.c_float), ("top_k", C.c_int32), ("seed", C.c_uint64),
                ("eos_id", C.c_uint32), ("ignore_eos", C.c_int32)]


class Stats(C.Structure):
    _fields_ = [("prompt_tokens", C.c_int64), ("decode_tokens", C.c_int64), ("ms_prefill", C.c_float),
                ("ms_decode", C.c_float), ("bytes_per_step", C.c_int64), ("kernel_launches", C.c_int64),
                ("achieved_gbps", C.c_float), ("waves", C.c_int32)]


def lib():
    """Loads liblumi_b200.so; raises (never falls back) when it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: run `python -m lumi_b200.build` (nvcc, sm_100a)")
        L = C.CDLL(LIB_PATH)
        vp, i32, i64, u64 = C.c_void_p, C.c_int32, C.c_int64, C.c_uint64
        L.lumi_last_error.restype = C.c_char_p
        L.lumi_model_create.argtypes = [C.c_char_p, i32, C.POINTER(vp)]
        L.lumi_model_load_tensor.argtypes = [vp, C.c_char_p, i32, C.POINTER(i64), i32, vp, u64]
        L.lumi_model_load_safetensors.argtypes = [vp, C.c_char_p]
        L.lumi_model_finalize.argtypes = [vp]
        L.lumi_model_free.argtypes = [vp]
        L.lumi_model_free.restype = None
        L.lumi_model_info.argtypes = [vp, C.POINTER(i64)]
        L.lumi_session_create.argtypes = [vp, i32, i32, C.POINTER(vp)]
        L.lumi_session_reset.argtypes = [vp, vp, i32]
        L.lumi_session_free.argtypes = [vp]
        L.lumi_session_free.restype = None
        L.lumi_session_set_option.argtypes = [vp, C.c_char_p, i64]
        L.lumi_prefill.argtypes = [vp, vp, i32, i32, vp]
        L.lumi_prefill_ragged.argtypes = [vp, vp, vp, i32, i32, vp]
        L.lumi_decode_step.argtypes = [vp, vp, i32, C.POINTER(Sampling), i32, vp, vp]
        L.lumi_generate.argtypes = [vp, vp, i32, i32, i32, C.POINTER(Sampling), vp, vp, vp, C.POINTER(Stats)]
        L.lumi_decode_loop_device.argtypes = [vp, i32, i32, C.POINTER(C.c_float), C.POINTER(i64)]
        L.lumi_profile_step.argtypes = [vp, i32, C.POINTER(C.c_float), C.POINTER(i64)]
        L.lumi_session_read_state.argtypes = [vp, i32, i32, vp, vp, vp, vp]
        L.lumi_score.argtypes = [vp, vp, i32, i32, vp]
        L.lumi_session_state_bytes.argtypes = [vp, vp]
        L.lumi_session_save_state.argtypes = [vp, i32, vp, C.c_int64]
        L.lumi_session_load_state.argtypes = [vp, i32, vp, C.c_int64]
        L.lumi_debug_run_block.argtypes = [vp, i32, vp, i32]
        L.lumi_k_gemm_bf16_tcgen05.argtypes = [u64, u64, u64, u64, i32, i32, i32, i32, i32, u64]
        L.lumi_k_gemv.argtypes = [u64, u64, i32, u64, u64, u64, i32, i32, i32, u64]
        L.lumi_k_ssm_step.argtypes = [u64, i32] + [u64] * 11 + [i32] * 5 + [u64]
        L.lumi_debug_gemm_wait_timeout.argtypes = [u64, u64, u64, i32, i32, i32, u64, i32, u64]
        L.lumi_debug_gemm_plan.argtypes = [i32, i32, i32, i32, i32, C.POINTER(C.c_int32), C.POINTER(C.c_int32)]
        L.lumi_k_ssd_prefill.argtypes = [u64, i32] + [u64] * 13 + [i32] * 4 + [u64]
        L.lumi_mamba_block_static.argtypes = [vp, i32, u64, u64, u64, u64, u64, i32, u64]
        _lib = L
    return _lib


def check(status: int) -> None:
    if status != 0:
        raise LumiError(status, lib().lumi_last_error().decode(errors="replace"))


def _ptr(a: Optional[np.ndarray]):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


class NmModel:
    """The reference's `NmModel` (inference/src/model.rs:632-827) on one GPU."""

    def __init__(self, handle, cfg: synth.ModelConfig):
        self._h = handle
        self.config = cfg

    @staticmethod
    def _create(config_json: str, device: int):
        h = C.c_void_p()
        check(lib().lumi_model_create(config_json.encode(), device, C.byref(h)))
        return h

    @classmethod
    def load(cls, model_path: str, config_path: str, device: int = 0) -> "NmModel":
        """`load_model` of inference/src/main.rs:72-89: config.json + one safetensors file."""
        with open(config_path) as f:
            text = f.read()
        h = cls._create(text, device)
        m = cls(h, synth.ModelConfig.from_json(text))
        check(lib().lumi_model_load_safetensors(h, model_path.encode()))
        check(lib().lumi_model_finalize(h))
        return m

    @classmethod
    def from_tensors(cls, cfg: synth.ModelConfig, tensors: Iterable[Tuple[str, int, np.ndarray]], device: int = 0) -> "NmModel":
        """Loads from in-memory (name, dtype code, array) entries — the per-tensor entry point a host
        that does its own safetensors parsing would call."""
        h = cls._create(cfg.to_json(), device)
        m = cls(h, cfg)
        for name, dt, arr in tensors:
            m.load_tensor(name, dt, arr)
        check(lib().lumi_model_finalize(h))
        return m

    def load_tensor(self, name: str, dtype: int, arr: np.ndarray) -> None:
        arr = np.ascontiguousarray(arr)
        shape = (C.c_int64 * arr.ndim)(*arr.shape)
        check(lib().lumi_model_load_tensor(self._h, name.encode(), dtype, shape, arr.ndim, _ptr(arr), arr.nbytes))

    def info(self) -> dict:
        o = (C.c_int64 * 12)()
        check(lib().lumi_model_info(self._h, o))
        keys = ["d_model", "n_layers", "d_state", "n_heads", "head_dim", "n_groups", "vocab_size", "n_mamba",
                "n_attention", "in_proj_out", "weights_dtype", "weight_bytes"]
        return dict(zip(keys, list(o)))

    def init_states(self, max_batch: int = 1, max_tokens_kv: int = 0) -> "Session":
        """`NmModel::init_states` (inference/src/model.rs:731-763) for `max_batch` sequences."""
        if max_tokens_kv <= 0:
            max_tokens_kv = self.config.max_seq_len
        return Session(self, max_batch, max_tokens_kv)

    def close(self):
        if self._h:
            lib().lumi_model_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Session:
    """Per-layer state for a batch of independent sequences (`Vec<LayerState>` of the reference)."""

    def __init__(self, model: NmModel, max_batch: int, max_tokens_kv: int):
        self.model = model
        self.max_batch = max_batch
        h = C.c_void_p()
        check(lib().lumi_session_create(model._h, max_batch, max_tokens_kv, C.byref(h)))
        self._h = h

    def close(self):
        if getattr(self, "_h", None):
            lib().lumi_session_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def set_option(self, name: str, value: int) -> None:
        check(lib().lumi_session_set_option(self._h, name.encode(), int(value)))

    def reset(self, slots: Optional[Sequence[int]] = None) -> None:
        if slots is None:
            check(lib().lumi_session_reset(self._h, None, 0))
        else:
            a = np.ascontiguousarray(slots, dtype=np.int32)
            check(lib().lumi_session_reset(self._h, _ptr(a), len(a)))

    def forward_step(self, tokens, sampling: Optional[Sampling] = None, step: int = 0,
                     want_logits: bool = True):
        """`NmModel::forward_step` (inference/src/model.rs:766-801) for one token per sequence.
        Returns (logits [batch, vocab] or None, next tokens [batch])."""
        tokens = np.ascontiguousarray(np.atleast_1d(tokens), dtype=np.uint32)
        B = len(tokens)
        V = self.model.config.vocab_size
        logits = np.empty((B, V), dtype=np.float32) if want_logits else None
        out = np.empty(B, dtype=np.uint32)
        sp = sampling if sampling is not None else Sampling(0.0, 0, 0, 2, 1)
        check(lib().lumi_decode_step(self._h, _ptr(tokens), B, C.byref(sp), step, _ptr(out), _ptr(logits)))
        return logits, out

    def prefill(self, prompts, want_logits: bool = True):
        prompts = np.ascontiguousarray(np.atleast_2d(prompts), dtype=np.uint32)
        B, T = prompts.shape
        logits = np.empty((B, self.model.config.vocab_size), dtype=np.float32) if want_logits else None
        check(lib().lumi_prefill(self._h, _ptr(prompts), B, T, _ptr(logits)))
        return logits

    def prefill_ragged(self, prompts, lengths, want_logits: bool = True):
        """Prompts of different lengths: prompts [batch, T_max] of which row b uses the first lengths[b] tokens."""
        prompts = np.ascontiguousarray(np.atleast_2d(prompts), dtype=np.uint32)
        lengths = np.ascontiguousarray(lengths, dtype=np.int32)
        B, T = prompts.shape
        logits = np.empty((B, self.model.config.vocab_size), dtype=np.float32) if want_logits else None
        check(lib().lumi_prefill_ragged(self._h, _ptr(prompts), _ptr(lengths), B, T, _ptr(logits)))
        return logits

    def score(self, tokens) -> np.ndarray:
        """log p(tokens[b][t+1] | tokens[b][:t+1]) for every position (inference/src/eval.rs:39-139); [batch, T-1]."""
        tokens = np.ascontiguousarray(np.atleast_2d(tokens), dtype=np.uint32)
        B, T = tokens.shape
        out = np.empty((B, T - 1), dtype=np.float32)
        check(lib().lumi_score(self._h, _ptr(tokens), B, T, _ptr(out)))
        return out

    def generate(self, prompts, n_new: int, temperature: float = 0.0, top_k: int = 0, seed: int = 0, eos_id: int = 2,
                 ignore_eos: bool = False, dump_logits: bool = False):
        """The `generate` loop of inference/src/main.rs:118-170 for a batch of equally long prompts.
        Returns (tokens [batch, n_new], lengths [batch], logits [n_new, batch, vocab] or None, Stats)."""
        prompts = np.ascontiguousarray(np.atleast_2d(prompts), dtype=np.uint32)
        B, T = prompts.shape
        out = np.zeros((B, max(n_new, 1)), dtype=np.uint32)[:, :n_new].copy()
        lens = np.zeros(B, dtype=np.int32)
        dump = np.empty((n_new, B, self.model.config.vocab_size), dtype=np.float32) if dump_logits else None
        sp = Sampling(float(temperature), int(top_k), int(seed), int(eos_id), int(bool(ignore_eos)))
        st = Stats()
        check(lib().lumi_generate(self._h, _ptr(prompts), B, T, n_new, C.byref(sp), _ptr(out), _ptr(lens), _ptr(dump), C.byref(st)))
        return out, lens, dump, st

    def decode_loop_device(self, batch: int, n_steps: int):
        ms = C.c_float()
        n = C.c_int64()
        check(lib().lumi_decode_loop_device(self._h, batch, n_steps, C.byref(ms), C.byref(n)))
        return float(ms.value), int(n.value)

    FAMILIES = ["embedding", "norm_split", "in_proj", "ssm_step", "out_proj", "attention_block", "lm_head", "sample"]

    def profile_step(self, batch: int) -> dict:
        """One decode step with a CUDA event before every launch: {family: (ms, launches)}."""
        ms = (C.c_float * 8)()
        n = (C.c_int64 * 8)()
        check(lib().lumi_profile_step(self._h, batch, ms, n))
        return {f: (float(ms[i]), int(n[i])) for i, f in enumerate(self.FAMILIES)}

    def read_state(self, slot: int, layer: int):
        c = self.model.config
        h = np.empty((c.n_heads, c.head_dim, c.d_state), dtype=np.float32)
        xp = np.empty((c.n_heads, c.head_dim), dtype=np.float32)
        bp = np.empty((c.n_heads, c.d_state), dtype=np.float32)
        cum = np.empty((c.n_heads, c.d_state // 2), dtype=np.float32)
        check(lib().lumi_session_read_state(self._h, slot, layer, _ptr(h), _ptr(xp), _ptr(bp), _ptr(cum)))
        return h, xp, bp, cum

    def save_state(self, slot: int) -> np.ndarray:
        """Snapshot of one sequence (SSM state, K/V pages, position) as bytes on the host."""
        n = C.c_int64()
        check(lib().lumi_session_state_bytes(self._h, C.byref(n)))
        buf = np.empty(n.value, dtype=np.uint8)
        check(lib().lumi_session_save_state(self._h, slot, _ptr(buf), n.value))
        return buf

    def load_state(self, slot: int, snapshot: np.ndarray) -> None:
        snapshot = np.ascontiguousarray(snapshot, dtype=np.uint8)
        check(lib().lumi_session_load_state(self._h, slot, _ptr(snapshot), snapshot.nbytes))

    def run_block(self, layer: int, x: np.ndarray) -> np.ndarray:
        x = np.array(np.atleast_2d(x), dtype=np.float32, copy=True)
        check(lib().lumi_debug_run_block(self._h, layer, _ptr(x), x.shape[0]))
        return x


class TextCodec:
    """The text boundary of `lumi-infer generate` (inference/src/main.rs:100-113, 154-165): byte-level models map
    byte b to id b + 3 with eos 2 and print single bytes that are valid UTF-8 on their own; other models use a
    HuggingFace `tokenizer.json` (byte-level BPE as the trainer builds it, training/src/tokenizer.rs:19-76) through
    the `tokenizers` package, eos = id of "<eos>" or 2, pieces decoded token by token with special tokens skipped."""

    def __init__(self, byte_level: bool, tokenizer_path: Optional[str] = None):
        self.byte_level = byte_level
        self._tok = None
        if not byte_level:
            if tokenizer_path is None:
                raise ValueError("a model that is not byte-level needs a tokenizer.json (main.rs:105-107 loads one)")
            try:
                from tokenizers import Tokenizer
            except ImportError as e:      # the package is the same library the reference links as a crate
                raise RuntimeError("the `tokenizers` package is needed for tokenizer.json models") from e
            self._tok = Tokenizer.from_file(tokenizer_path)

    @property
    def eos_id(self) -> int:
        if self.byte_level:
            return 2
        eos = self._tok.token_to_id("<eos>")
        return 2 if eos is None else int(eos)

    def encode(self, text: str) -> np.ndarray:
        if self.byte_level:
            return np.frombuffer(text.encode(), dtype=np.uint8).astype(np.uint32) + 3
        return np.asarray(self._tok.encode(text, add_special_tokens=False).ids, dtype=np.uint32)

    def piece(self, token: int) -> str:
        """What the loop prints for one generated token (main.rs:154-165)."""
        if self.byte_level:
            return chr(token - 3) if 3 <= token < 131 else ""
        return self._tok.decode([int(token)], skip_special_tokens=True)

    def decode(self, tokens) -> str:
        return "".join(self.piece(int(t)) for t in tokens)


def generate(model_path: str, config_path: str, prompt: str, max_tokens: int = 200, temperature: float = 0.8,
             top_k: int = 0, seed: int = 0, device: int = 0, tokenizer_path: Optional[str] = None) -> Tuple[str, np.ndarray]:
    """`lumi-infer generate` (inference/src/main.rs:96-177): encode the prompt, run the token loop on the GPU until
    eos or `max_tokens`, return prompt + generated text and the generated ids."""
    model = NmModel.load(model_path, config_path, device)
    codec = TextCodec(bool(model.config.byte_level), tokenizer_path)
    ids = codec.encode(prompt)
    if len(ids) == 0:
        raise ValueError("empty prompt")
    sess = model.init_states(1, len(ids) + max_tokens + 1)
    out, lens, _, _ = sess.generate(ids[None, :], max_tokens, temperature=temperature, top_k=top_k, seed=seed, eos_id=codec.eos_id)
    toks = out[0, :lens[0]]
    return prompt + codec.decode(toks), toks
