"""The text boundary of the generate command: byte-level ids and tokenizer.json models (CPU part; the GPU part runs
the loop through it)."""
import numpy as np
import pytest

import lumi_b200
from lumi_b200 import synth


def _train_tokenizer(path):
    """A byte-level BPE with the special tokens and components the reference's trainer sets up
    (training/src/tokenizer.rs:25-52), on a few synthetic sentences."""
    tk = pytest.importorskip("tokenizers")
    tok = tk.Tokenizer(tk.models.BPE())
    tok.pre_tokenizer = tk.pre_tokenizers.ByteLevel()
    tok.decoder = tk.decoders.ByteLevel()
    tok.post_processor = tk.processors.ByteLevel()
    trainer = tk.trainers.BpeTrainer(vocab_size=320, special_tokens=["<pad>", "<bos>", "<eos>", "<unk>"], show_progress=False)
    corpus = ["state space models keep a state per head", "the state is updated once per token", "tensor cores multiply tiles"] * 30
    tok.train_from_iterator(corpus, trainer)
    tok.save(str(path))
    return tok


def test_byte_level_codec_matches_the_reference_rules():
    c = lumi_b200.TextCodec(True)
    ids = c.encode("Hi\n")
    assert ids.tolist() == [ord("H") + 3, ord("i") + 3, 13] and c.eos_id == 2      # training/tests/data_tests.rs:88-117
    assert c.decode([ord("o") + 3, ord("k") + 3, 2, 200, 258]) == "ok"              # eos, pad-range and non-ASCII bytes print nothing


def test_tokenizer_json_codec_round_trip(tmp_path):
    tok = _train_tokenizer(tmp_path / "tokenizer.json")
    c = lumi_b200.TextCodec(False, str(tmp_path / "tokenizer.json"))
    text = "the state per token"
    ids = c.encode(text)
    assert ids.dtype == np.uint32 and ids.tolist() == tok.encode(text, add_special_tokens=False).ids
    assert c.eos_id == tok.token_to_id("<eos>") == 2
    assert c.decode(ids).strip() == text
    assert c.piece(c.eos_id) == ""                                                  # special tokens are skipped (main.rs:162)
    with pytest.raises(ValueError):
        lumi_b200.TextCodec(False, None)


@pytest.mark.gpu
def test_generate_with_tokenizer_json(tmp_path):
    from oracle import cpu_oracle
    tok = _train_tokenizer(tmp_path / "tokenizer.json")
    cfg = synth.tiny_config(n_layers=2, vocab_size=tok.get_vocab_size())
    cpath, mpath = synth.write_model_dir(str(tmp_path), cfg, seed=3, perturb_ones=0.1)
    prompt = "the state"
    text, toks = lumi_b200.generate(mpath, cpath, prompt, max_tokens=12, temperature=0.0, tokenizer_path=str(tmp_path / "tokenizer.json"))
    ids = np.asarray(tok.encode(prompt, add_special_tokens=False).ids, dtype=np.uint32)
    ref = cpu_oracle.OracleModel(cfg, list(synth.iter_tensors(cfg, seed=3, perturb_ones=0.1))).init_states().generate(ids, 12, eos=2)
    assert np.array_equal(toks, ref)
    assert text == prompt + "".join(tok.decode([int(t)], skip_special_tokens=True) for t in ref)
