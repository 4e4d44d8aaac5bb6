"""Generates the committed fixtures in this directory from oracle/numpy_restatement.py.

    python tests/golden/make_golden.py

The reference itself cannot run where this was written (Rust on Candle, no toolchain), and its
inference crate ships no golden vectors, so these are outputs of the numpy restatement of
inference/src/model.rs / main.rs on seeded synthetic weights — "parity unpinned" fixtures that pin
the C++ oracle and the CUDA path to one another and to this file's history.
Each .npz holds: cfg (JSON), seed, perturb, prompt, tokens (greedy), logits [n_new, vocab],
h / cum of the first Mamba layer after the run, and for the sampled case the uniforms and tokens.
"""
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from lumi_b200 import synth  # noqa: E402
from oracle import numpy_restatement as nr  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))

CASES = {
    "tiny_mamba": dict(),
    "tiny_hybrid": dict(attention_interval=2),
    "tiny_hybrid_ext": dict(attention_interval=2, attn_rope_base=10000.0, attn_window_sizes=[5], attn_mlp_dim=320),
    "tiny_bytelevel": dict(byte_level=True, n_layers=2),
}


def main():
    for name, kw in CASES.items():
        cfg = synth.tiny_config(**kw)
        seed, perturb = 11, 0.1
        tens = list(synth.iter_tensors(cfg, seed=seed, perturb_ones=perturb))
        model = nr.NumpyModel(cfg, tens)
        prompt = synth.random_prompts(1, 12, cfg.vocab_size, seed=5)[0]
        n_new = 24
        toks, dumps, states = model.generate(prompt, n_new, ignore_eos=True)
        first = next(i for i in range(cfg.n_layers) if not cfg.is_attention_layer(i))
        uniforms = np.array([nr.sampler_uniform(7, 0, i) for i in range(n_new)], dtype=np.float32)
        stoks, _, _ = model.generate(prompt, n_new, temperature=0.8, top_k=5, uniforms=uniforms, ignore_eos=True)
        np.savez_compressed(
            os.path.join(HERE, name + ".npz"), cfg=json.dumps(kw), seed=seed, perturb=perturb, prompt=prompt,
            tokens=toks, logits=np.stack(dumps).astype(np.float32), h=states[first]["h"], cum=states[first]["cum"],
            first_mamba=first, uniforms=uniforms, sampled_tokens=stoks)
        print(name, toks[:8], stoks[:8])


if __name__ == "__main__":
    main()
