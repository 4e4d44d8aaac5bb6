"""Generates the fixtures for the parity tests at the benchmark configurations' own shapes.

    python tests/golden/make_config_fixtures.py [config2 config3 config4 config5]

For each configuration (lumi_b200.synth.BENCH_CONFIGS: layers, vocabulary, bf16 weights, batch, prompt
length, sampling) the CPU oracle (oracle/lumi_oracle.cpp, the restatement of inference/src/model.rs and
main.rs) runs a few sequences of the batch — the first, the last and two in between — through the whole
prompt token by token and then 64 generated tokens.  The oracle needs minutes to hours for this at 48 / 96
layers, so its outputs are committed as tests/golden/configN.npz and the GPU tests compare with them:

    rows        [R]            indices of the sequences inside the batch
    tokens      [R][64]        generated ids (greedy, or sampled with the Philox uniforms of the configuration)
    steps       [S]            generated positions whose logits are kept
    logits      [R][S][vocab]  the oracle's logits at those positions
    margin      [R][64]        top-1 minus top-2 logit over max|logit| at every generated position
    layers      [2]            first and last Mamba layer
    heads       [2]            first and last head
    h, pbx      [R][2][2][P][N]   state of those layers / heads after the prompt (before any generated token)
    cum         [R][2][2][N/2]

Prompts and weights are not stored: both sides regenerate them from the seeds (lumi_b200.synth).
"Parity unpinned" applies to these as to the other fixtures: they are outputs of the restatement.
"""
import os
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from lumi_b200 import synth  # noqa: E402
from oracle import cpu_oracle, numpy_restatement as nr  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))
N_NEW = 64
KEEP_STEPS = [0, 31, 63]


def rows_of(batch):
    return sorted({0, batch // 3, (2 * batch) // 3, batch - 1})


def run_config(name):
    kw, wdt, batch, T, _, samp, pseed = synth.BENCH_CONFIGS[name]
    cfg = synth.base_config(**kw)
    t0 = time.time()
    tens = list(synth.iter_tensors(cfg, seed=0, weights_dtype=wdt))
    om = cpu_oracle.OracleModel(cfg, tens)
    del tens
    print(f"{name}: model ready in {time.time() - t0:.0f} s", flush=True)
    mamba = [i for i in range(cfg.n_layers) if not cfg.is_attention_layer(i)]
    layers = [mamba[0], mamba[-1]]
    heads = [0, cfg.n_heads - 1]
    rows = rows_of(batch)
    temperature = float(samp.get("temperature", 0.0))
    top_k = int(samp.get("top_k", 0))
    seed = int(samp.get("seed", 0))
    P, N = cfg.head_dim, cfg.d_state
    out = dict(
        rows=np.array(rows, dtype=np.int32), tokens=np.zeros((len(rows), N_NEW), dtype=np.uint32),
        steps=np.array(KEEP_STEPS, dtype=np.int32), logits=np.zeros((len(rows), len(KEEP_STEPS), cfg.vocab_size), dtype=np.float32),
        margin=np.zeros((len(rows), N_NEW), dtype=np.float32), layers=np.array(layers, dtype=np.int32), heads=np.array(heads, dtype=np.int32),
        h=np.zeros((len(rows), 2, 2, P, N), dtype=np.float32), pbx=np.zeros((len(rows), 2, 2, P, N), dtype=np.float32),
        cum=np.zeros((len(rows), 2, 2, N // 2), dtype=np.float32))
    for ri, b in enumerate(rows):
        t0 = time.time()
        prompt = synth.random_prompt_row(b, T, cfg.vocab_size, seed=pseed)
        st = om.init_states()
        for t in prompt:
            lg = st.forward_step(int(t))
        for li, layer in enumerate(layers):
            h, pbx, cum = st.read_state(layer)
            out["h"][ri, li] = h[heads]
            out["pbx"][ri, li] = pbx[heads]
            out["cum"][ri, li] = cum[heads]
        for i in range(N_NEW):
            if i in KEEP_STEPS:
                out["logits"][ri, KEEP_STEPS.index(i)] = lg
            s = np.sort(lg.astype(np.float64))
            out["margin"][ri, i] = (s[-1] - s[-2]) / max(np.abs(s).max(), 1e-30)
            if temperature <= 0.0:
                tok = cpu_oracle.argmax(lg)
            else:
                # the sampler's uniform for (seed, sequence index in the batch, generated position)
                tok = cpu_oracle.sample(lg, temperature, top_k, float(nr.sampler_uniform(seed, b, i)))
            out["tokens"][ri, i] = tok
            if i + 1 < N_NEW:
                lg = st.forward_step(tok)
        print(f"{name}: row {b} done in {time.time() - t0:.0f} s; tokens {out['tokens'][ri, :6]} min margin {out['margin'][ri].min():.2e}", flush=True)
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **out)       # partial results survive an interruption


def main():
    cpu_oracle.set_threads(os.cpu_count() or 1)
    for name in (sys.argv[1:] or ["config2", "config4", "config5", "config3"]):
        run_config(name)


if __name__ == "__main__":
    main()
