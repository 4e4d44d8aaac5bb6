"""CPU: the C-ABI library loads, exports every symbol the header declares, and its host-side logic
(config parsing, argument checks) answers with the documented status codes.  No compute calls."""
import ctypes as C
import os
import re

import numpy as np
import pytest

import lumi_b200
from lumi_b200 import synth

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_functions():
    text = open(os.path.join(ROOT, "include", "lumi_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(lumi_[a-z0-9_]+)\s*\(", text)))


def test_exports_match_header():
    names = header_functions()
    assert names == sorted(lumi_b200.EXPORTS)
    L = lumi_b200.lib()
    for n in names:
        assert hasattr(L, n), n


def _create(cfg_text):
    h = C.c_void_p()
    st = lumi_b200.lib().lumi_model_create(cfg_text.encode(), 0, C.byref(h))
    msg = lumi_b200.lib().lumi_last_error().decode()
    if st == 0:
        lumi_b200.lib().lumi_model_free(h)
    return st, msg


@pytest.mark.parametrize("text,frag", [
    ("{", "config.json"),
    ('{"d_model": 128}', "missing key 'n_layers'"),
    (synth.tiny_config().to_json().replace('"n_heads": 8', '"n_heads": 7'), "not divisible by n_heads"),
    (synth.tiny_config().to_json().replace('"n_groups": 2', '"n_groups": 3'), "not divisible by n_groups"),
    (synth.tiny_config().to_json().replace('"d_state": 16', '"d_state": 15'), "must be even"),
    (synth.tiny_config().to_json().replace('"byte_level": false', '"byte_level": 1'), "must be a boolean"),
    (synth.tiny_config().to_json().replace('"d_model": 128', '"d_model": "x"'), "non-negative integer"),
])
def test_bad_config_is_rejected(text, frag):
    st, msg = _create(text)
    assert st == -2 and frag in msg          # LUMI_E_CONFIG, before any device is touched


def test_good_config_passes_parsing():
    # unknown keys are ignored, as the reference's serde struct does (inference/README.md:44-62)
    text = synth.tiny_config().to_json()[:-1] + ', "d_conv": 4, "chunk_size": 64}'
    st, msg = _create(text)
    assert st in (0, -6), msg                # OK on a GPU box, LUMI_E_CUDA where no device exists


def test_null_arguments():
    L = lumi_b200.lib()
    assert L.lumi_model_finalize(None) == -1
    assert L.lumi_session_reset(None, None, 0) == -1
    assert L.lumi_prefill(None, None, 1, 1, None) == -1
    assert L.lumi_session_create(None, 1, 0, C.byref(C.c_void_p())) == -1
    assert L.lumi_model_load_safetensors(None, b"x") == -1


def test_safetensors_writer_roundtrip(tmp_path):
    st = pytest.importorskip("safetensors.numpy")
    cfg = synth.tiny_config(n_layers=1)
    _, mpath = synth.write_model_dir(str(tmp_path), cfg, seed=2)
    got = st.load_file(mpath)
    want = {n: a for n, dt, a in synth.iter_tensors(cfg, seed=2)}
    assert set(got) == set(want)
    for k in want:
        assert np.array_equal(got[k], want[k])


def test_bf16_rounding_is_nearest_even():
    x = np.array([1.0, 1.00390625, 1.01171875, -2.5, 3.14159265], dtype=np.float32)
    # 1 + 2^-8 is a tie between 1.0 and 1 + 2^-7 -> even (1.0); 1 + 3*2^-8 ties up to 1 + 2^-6
    got = synth.bf16_bits_to_f32(synth.f32_to_bf16_bits(x))
    assert got[0] == 1.0 and got[1] == 1.0 and got[2] == 1.015625 and got[3] == -2.5
    assert abs(got[4] - 3.14159265) < 2 ** -7


@pytest.mark.parametrize("shape,two,producer,want", [
    ((2048, 7360, 1024), 1, 0, (208, 1)),      # in_proj of a 2048-sequence wave: 576 tiles = 4 rounds of 148 SMs
    ((2048, 1024, 2048), 1, 1, (128, 1)),      # out_proj: one round of 128 tiles; widths are multiples of 32 for the folded norm
    ((64, 7360, 1024), 1, 0, (64, 1)),         # 115 tiles already fill the SMs: no split
    ((64, 1024, 2048), 1, 1, (32, 4)),         # 32 narrow tiles and a long K: K split over 4 CTAs
    ((128, 1024, 2816), 1, 1, (32, 4)),        # the MLP's second product at 128 rows
    ((128, 1024, 1024), 1, 1, (32, 1)),        # K too short for a split to pay
    ((256, 1024, 2048), 1, 1, (32, 1)),        # two row tiles: measured slower split, stays whole
    ((512, 259, 1024), 1, 0, (32, 1)),
])
def test_gemm_tile_and_split_choice(shape, two, producer, want):
    """Host logic of the tensor-core GEMM: which tile width and K split a shape gets (no device needed; 148 SMs assumed
    where none is present)."""
    w, sp = C.c_int32(), C.c_int32()
    st = lumi_b200.lib().lumi_debug_gemm_plan(*shape, two, producer, C.byref(w), C.byref(sp))
    assert st == 0 and (w.value, sp.value) == want, (shape, w.value, sp.value)
    assert lumi_b200.lib().lumi_debug_gemm_plan(64, 64, 100, 1, 0, C.byref(w), C.byref(sp)) == -1      # K % 64

