"""CPU: the C++ oracle against the committed golden vectors, the independent numpy restatement, and
the structural pins the reference's own tests hold for this path."""
import numpy as np
import pytest

from lumi_b200 import synth
from oracle import cpu_oracle, numpy_restatement as nr
from tests.helpers import GOLDEN_CASES, load_golden, rel_err


@pytest.mark.parametrize("name", GOLDEN_CASES)
def test_oracle_matches_golden(name):
    z, cfg, tens = load_golden(name)
    st = cpu_oracle.OracleModel(cfg, tens).init_states()
    toks, dump = st.generate(z["prompt"], len(z["tokens"]), ignore_eos=True, dump_logits=True)
    assert np.array_equal(toks, z["tokens"])
    for i in range(len(toks)):
        assert rel_err(dump[i], z["logits"][i]) < 2e-5
    h, pbx, cum = st.read_state(int(z["first_mamba"]))
    assert np.abs(h - z["h"]).max() < 1e-4 * max(1.0, np.abs(z["h"]).max())
    assert np.abs(cum - z["cum"]).max() < 1e-4


@pytest.mark.parametrize("name", GOLDEN_CASES)
def test_oracle_sampling_matches_golden(name):
    z, cfg, tens = load_golden(name)
    st = cpu_oracle.OracleModel(cfg, tens).init_states()
    toks = st.generate(z["prompt"], len(z["sampled_tokens"]), temperature=0.8, top_k=5, uniforms=z["uniforms"], ignore_eos=True)
    assert np.array_equal(toks, z["sampled_tokens"])


def test_oracle_vs_numpy_fresh_seed():
    cfg = synth.tiny_config(attention_interval=3, n_layers=6)
    tens = list(synth.iter_tensors(cfg, seed=99, perturb_ones=0.2))
    om, nm = cpu_oracle.OracleModel(cfg, tens), nr.NumpyModel(cfg, tens)
    prompt = synth.random_prompts(1, 9, cfg.vocab_size, seed=1)[0]
    t1, d1 = om.init_states().generate(prompt, 16, ignore_eos=True, dump_logits=True)
    t2, d2, _ = nm.generate(prompt, 16, ignore_eos=True)
    assert np.array_equal(t1, t2)
    assert max(rel_err(a, b) for a, b in zip(d1, d2)) < 2e-5


def test_eos_stops_generation():
    z, cfg, tens = load_golden("tiny_mamba")
    st = cpu_oracle.OracleModel(cfg, tens).init_states()
    eos = int(z["tokens"][3])
    first = int(np.argmax(z["tokens"] == eos))
    toks = st.generate(z["prompt"], 24, eos=eos)                     # inference/src/main.rs:150
    assert len(toks) == first and np.array_equal(toks, z["tokens"][:first])


def test_h_init_missing_means_zero_state():
    cfg = synth.tiny_config(n_layers=1)
    tens = [t for t in synth.iter_tensors(cfg, seed=3) if not t[0].endswith("ssm.h_init")]
    st = cpu_oracle.OracleModel(cfg, tens).init_states()              # inference/src/model.rs:746-748
    h, pbx, cum = st.read_state(0)
    assert not h.any() and not pbx.any() and not cum.any()


# ---- structural pins from the reference's tests ------------------------------------------------------
def test_in_proj_out_is_7360():                                        # training/tests/training_init_tests.rs:24-31
    assert synth.base_config().in_proj_out == 7360


def test_helper_dims():                                                # training/tests/config_tests.rs:108-123
    c = synth.base_config()
    assert (c.d_inner, c.head_dim, c.attn_head_dim, c.attn_kv_dim, c.mlp_dim) == (2048, 32, 64, 256, 4096)


def test_attention_placement():                                        # training/tests/config_tests.rs:125-140, 199-220
    c = synth.base_config(attention_interval=8)
    assert [i for i in range(48) if c.is_attention_layer(i)] == [7, 15, 23, 31, 39, 47]
    c = synth.base_config(attention_interval=8, attention_layers=[1, 5])
    assert [i for i in range(48) if c.is_attention_layer(i)] == [1, 5] and c.n_attn_layers() == 2


def test_window_lookup():                                              # training/tests/config_tests.rs:161-179
    c = synth.base_config(attention_interval=8, attn_window_sizes=[128, 0, 256])
    assert [c.attn_window_size(i) for i in range(5)] == [128, 0, 256, 0, 0]


def test_byte_level_forces_vocab_259():                                # training/tests/config_tests.rs:275-297
    assert synth.base_config(byte_level=True, vocab_size=32000).vocab_size == 259


def test_byte_level_ids():                                             # training/tests/data_tests.rs:88-117
    ids = np.frombuffer(b"Hello\nWorld\n", dtype=np.uint8).astype(np.uint32) + 3
    assert len(ids) + 2 == 14 and ids[0] == ord("H") + 3 and ids.min() >= 3


def test_param_count_base_model():                                     # training/tests/config_tests.rs:142-148 (450-550 M)
    n = sum(int(np.prod(s)) for _, s, _, _ in synth.tensor_specs(synth.base_config()))
    assert n == 495_541_248
    n96 = sum(int(np.prod(s)) for _, s, _, _ in synth.tensor_specs(synth.base_config(n_layers=96)))
    assert n96 == 958_313_472


# ---- Philox4x32-10 known answers (Random123 kat_vectors) ---------------------------------------------
def test_philox_known_answers():
    assert nr.philox4x32_10([0, 0, 0, 0], [0, 0]) == [0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8]
    assert nr.philox4x32_10([0xffffffff] * 4, [0xffffffff] * 2) == [0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd]
    assert nr.philox4x32_10([0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344], [0xa4093822, 0x299f31d0]) == \
        [0xd16cfe09, 0x94fdcceb, 0x5001e420, 0x24126ea1]


def test_sampling_cdf_walk():
    logits = np.log(np.array([0.1, 0.2, 0.3, 0.4], dtype=np.float32))
    assert cpu_oracle.sample(logits, 1.0, 0, 0.05) == 0                # inference/src/main.rs:197-209
    assert cpu_oracle.sample(logits, 1.0, 0, 0.25) == 1
    assert cpu_oracle.sample(logits, 1.0, 0, 0.95) == 3
    assert cpu_oracle.sample(logits, 1.0, 2, 0.05) == 2                # top-2 keeps {2, 3}: p = 3/7, 4/7
    assert cpu_oracle.sample(logits, 1.0, 2, 0.50) == 3
    for r in (0.0, 0.3, 0.77):
        assert cpu_oracle.sample(logits, 0.7, 3, r) == nr.sample_from_logits(logits, 0.7, 3, np.float32(r))
