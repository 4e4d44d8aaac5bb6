"""GPU: the CUDA token loop through the C ABI against the CPU oracle and the committed fixtures.

Tolerances (the ones the benchmark definition states): identical greedy token ids, and at every
generated position max|g - r| / max|r| <= 1e-3 over the logits for fp32 weights, 2e-2 for bf16
weights.  The oracle's top-1/top-2 margin is printed when a token differs, so a flip at a
sub-tolerance margin can be told from a bug.
"""
import numpy as np
import pytest

import lumi_b200
from lumi_b200 import synth
from oracle import cpu_oracle, numpy_restatement as nr
from tests.helpers import GOLDEN_CASES, load_golden, rel_err, top2_margin

pytestmark = pytest.mark.gpu

TOL_F32 = 1e-3
TOL_BF16 = 2e-2


def _compare_tokens(got, ref, ref_logits, label):
    if np.array_equal(got, ref):
        return
    i = int(np.argmax(got != ref))
    raise AssertionError(f"{label}: token {i} differs (got {got[i]}, oracle {ref[i]}); oracle top-2 margin "
                         f"{top2_margin(ref_logits[i]):.3e}, |logit| max {np.abs(ref_logits[i]).max():.3e}")


@pytest.mark.parametrize("name", GOLDEN_CASES)
@pytest.mark.parametrize("graph", [1, 0])
def test_golden_fixture_parity(name, graph):
    z, cfg, tens = load_golden(name)
    model = lumi_b200.NmModel.from_tensors(cfg, tens)
    sess = model.init_states(2, 64)
    sess.set_option("graph", graph)
    prompts = np.stack([z["prompt"], z["prompt"]])
    toks, lens, dump, st = sess.generate(prompts, len(z["tokens"]), ignore_eos=True, dump_logits=True)
    for b in range(2):
        for i in range(len(z["tokens"])):
            assert rel_err(dump[i, b], z["logits"][i]) < TOL_F32
        _compare_tokens(toks[b], z["tokens"], z["logits"], f"{name} slot {b}")
    assert st.kernel_launches > 0


@pytest.mark.parametrize("name", ["tiny_mamba", "tiny_hybrid_ext"])
def test_golden_sampled_tokens(name):
    z, cfg, tens = load_golden(name)
    model = lumi_b200.NmModel.from_tensors(cfg, tens)
    sess = model.init_states(1, 64)
    toks, lens, _, _ = sess.generate(z["prompt"][None, :], len(z["sampled_tokens"]), temperature=0.8, top_k=5, seed=7, ignore_eos=True)
    assert np.array_equal(toks[0], z["sampled_tokens"])


def test_state_parity_after_prefill():
    cfg = synth.tiny_config(n_layers=3)
    tens = list(synth.iter_tensors(cfg, seed=21, perturb_ones=0.1))
    om = cpu_oracle.OracleModel(cfg, tens)
    st = om.init_states()
    prompt = synth.random_prompts(1, 20, cfg.vocab_size, seed=2)[0]
    for t in prompt:
        ref_logits = st.forward_step(int(t))
    model = lumi_b200.NmModel.from_tensors(cfg, tens)
    sess = model.init_states(1)
    logits = sess.prefill(prompt[None, :])
    assert rel_err(logits[0], ref_logits) < TOL_F32
    for layer in range(cfg.n_layers):
        h, xp, bp, cum = sess.read_state(0, layer)
        rh, rpbx, rcum = st.read_state(layer)
        assert np.abs(h - rh).max() <= 1e-4 * max(1.0, np.abs(rh).max())
        assert np.abs(xp[:, :, None] * bp[:, None, :] - rpbx).max() <= 1e-4 * max(1.0, np.abs(rpbx).max())
        assert np.abs(cum - rcum).max() < 1e-4


def test_mamba_block_alone_base_dims():
    """One block at the benchmark's dimensions (d_model 1024, 64 heads of 32, d_state 64, 8 groups)."""
    cfg = synth.base_config(n_layers=1, vocab_size=512)
    tens = list(synth.iter_tensors(cfg, seed=4, perturb_ones=0.1))
    om = cpu_oracle.OracleModel(cfg, tens)
    st = om.init_states()
    model = lumi_b200.NmModel.from_tensors(cfg, tens)
    sess = model.init_states(3)
    g = np.random.default_rng(0)
    for step in range(4):
        x = g.standard_normal((3, cfg.d_model)).astype(np.float32)
        x[1] = x[0]
        got = sess.run_block(0, x)
        ref = st.mamba_block(0, x[0])
        assert rel_err(got[0], ref) < 1e-5
        assert np.array_equal(got[0], got[1])          # identical sequences give identical bits
    h, xp, bp, cum = sess.read_state(0, 0)
    rh, rpbx, rcum = st.read_state(0)
    assert np.abs(h - rh).max() <= 1e-5 * max(1.0, np.abs(rh).max())
    assert np.abs(cum - rcum).max() < 1e-5


@pytest.mark.parametrize("wdt", ["f32", "bf16"])
def test_batch1_persistent_kernel_and_chain_agree_with_oracle(wdt):
    """Base dimensions, 3 layers, batch 1: the one-kernel-per-call path and the kernel-chain path
    both against the oracle — tokens, logits, final state — greedy and sampled."""
    cfg = synth.base_config(n_layers=3, vocab_size=1000)
    tens = list(synth.iter_tensors(cfg, seed=5, weights_dtype=wdt, perturb_ones=0.05))
    prompt = synth.random_prompts(1, 9, cfg.vocab_size, seed=2)[0]
    n_new = 20
    om = cpu_oracle.OracleModel(cfg, tens)
    ost = om.init_states()
    ref_toks, ref_logits = ost.generate(prompt, n_new, ignore_eos=True, dump_logits=True)
    uniforms = np.array([nr.sampler_uniform(99, 0, i) for i in range(n_new)], dtype=np.float32)
    ref_sampled = om.init_states().generate(prompt, n_new, temperature=0.7, top_k=8, uniforms=uniforms, ignore_eos=True)
    model = lumi_b200.NmModel.from_tensors(cfg, tens)
    for mega in (1, 0):
        sess = model.init_states(1)
        sess.set_option("megakernel", mega)
        toks, lens, dump, st = sess.generate(prompt[None, :], n_new, ignore_eos=True, dump_logits=True)
        worst = max(rel_err(dump[i, 0], ref_logits[i]) for i in range(n_new))
        assert worst < TOL_F32, (mega, worst)
        _compare_tokens(toks[0], ref_toks, ref_logits, f"megakernel={mega}")
        assert lens[0] == n_new
        # the device loop stops one forward_step before the oracle's loop: catch up, then compare state
        sess.forward_step([int(toks[0, -1])])
        for layer in range(cfg.n_layers):
            h, xp, bp, cum = sess.read_state(0, layer)
            rh, rpbx, rcum = ost.read_state(layer)
            assert np.abs(h - rh).max() <= 1e-4 * max(1.0, np.abs(rh).max()), (mega, layer)
            assert np.abs(cum - rcum).max() < 1e-4
        sess.reset()
        stoks, _, _, _ = sess.generate(prompt[None, :], n_new, temperature=0.7, top_k=8, seed=99, ignore_eos=True)
        assert np.array_equal(stoks[0], ref_sampled), (mega, stoks[0], ref_sampled)
        # eos handling on this path
        sess.reset()
        eos = int(ref_toks[5])
        first = int(np.argmax(ref_toks == eos))
        etoks, elens, _, _ = sess.generate(prompt[None, :], n_new, eos_id=eos)
        assert elens[0] == first
        # bad token id is reported, not followed
        with pytest.raises(lumi_b200.LumiError) as e:
            sess.forward_step([cfg.vocab_size + 1])
        assert e.value.code == -8
        sess.close()


@pytest.mark.parametrize("mega", [1, 0])
def test_config1_shape_fp32_greedy_parity(mega):
    """The base 48-layer fp32 model, batch 1, 32-token prompt: identical greedy ids for the first 64
    generated tokens and logits within 1e-3."""
    cfg = synth.base_config()
    tens = list(synth.iter_tensors(cfg, seed=0))
    prompt = synth.random_prompts(1, 32, cfg.vocab_size, seed=0)[0]
    n_new = 64
    ref_toks, ref_logits = cpu_oracle.OracleModel(cfg, tens).init_states().generate(prompt, n_new, ignore_eos=True, dump_logits=True)
    model = lumi_b200.NmModel.from_tensors(cfg, tens)
    del tens
    sess = model.init_states(1)
    sess.set_option("megakernel", mega)
    toks, lens, dump, st = sess.generate(prompt[None, :], n_new, ignore_eos=True, dump_logits=True)
    worst = max(rel_err(dump[i, 0], ref_logits[i]) for i in range(n_new))
    print(f"config-1 parity (persistent kernel {mega}): worst logits rel err {worst:.3e}; min oracle top-2 margin "
          f"{min(top2_margin(l) for l in ref_logits):.3e}; decode {st.decode_tokens / st.ms_decode * 1e3:.0f} tok/s")
    assert worst < TOL_F32
    _compare_tokens(toks[0], ref_toks, ref_logits, "config 1")


@pytest.mark.parametrize("gemm,split,tol", [(0, 1, TOL_F32), (0, 0, TOL_BF16), (1, 1, TOL_F32)])
def test_bf16_batched_parity(gemm, split, tol):
    """bf16 weights, batch 64, base dimensions with 6 layers: sampled sequences against the oracle
    run on the same bf16-rounded weights.  gemm 0 = tensor-core GEMMs (batch > 8), 1 = CUDA cores.
    With split activations the tensor-core path must meet the fp32 tolerance."""
    cfg = synth.base_config(n_layers=6, vocab_size=4096)
    tens = list(synth.iter_tensors(cfg, seed=0, weights_dtype="bf16"))
    B, T, n_new = 64, 16, 24
    prompts = synth.random_prompts(B, T, cfg.vocab_size, seed=0)
    model = lumi_b200.NmModel.from_tensors(cfg, tens)
    sess = model.init_states(B)
    sess.set_option("gemm", gemm)
    sess.set_option("split_activations", split)
    toks, lens, dump, st = sess.generate(prompts, n_new, ignore_eos=True, dump_logits=True)
    om = cpu_oracle.OracleModel(cfg, tens)
    for b in (0, 17, 63):
        ref_toks, ref_logits = om.init_states().generate(prompts[b], n_new, ignore_eos=True, dump_logits=True)
        # compare logits while the token histories agree
        n_same = n_new if np.array_equal(toks[b], ref_toks) else int(np.argmax(toks[b] != ref_toks)) + 1
        worst = max(rel_err(dump[i, b], ref_logits[i]) for i in range(n_same))
        assert worst < tol, (b, worst)
        if split:
            _compare_tokens(toks[b], ref_toks, ref_logits, f"bf16 batch slot {b}")


@pytest.mark.parametrize("rows", [32768, 192])
def test_chunked_ssd_prefill_matches_stepwise_and_oracle(rows):
    """bf16 Mamba-only model, 200-token prompts (three full chunks of 64 and a ragged one): the
    chunked scan against the token-by-token prefill on the GPU and against the oracle's sequential
    prefill — last-position logits, every layer's state, and the greedy continuation.  rows = 192
    forces several passes (64 tokens each), so the state hand-over between launches is covered."""
    cfg = synth.base_config(n_layers=3, vocab_size=1000)
    tens = list(synth.iter_tensors(cfg, seed=6, weights_dtype="bf16", perturb_ones=0.05))
    B, T, n_new = 3, 200, 8
    prompts = synth.random_prompts(B, T, cfg.vocab_size, seed=9)
    model = lumi_b200.NmModel.from_tensors(cfg, tens)
    step = model.init_states(B)
    step.set_option("chunked_prefill", 0)
    lg_step = step.prefill(prompts)
    chk = model.init_states(B)
    chk.set_option("chunked_prefill", 64)
    chk.set_option("prefill_rows", rows)
    lg_chk = chk.prefill(prompts)
    two_pi = 2 * np.pi
    for b in range(B):
        assert rel_err(lg_chk[b], lg_step[b]) < 1e-4
        for layer in range(cfg.n_layers):
            h1, xp1, bp1, cu1 = chk.read_state(b, layer)
            h0, xp0, bp0, cu0 = step.read_state(b, layer)
            assert np.abs(h1 - h0).max() <= 2e-4 * max(1.0, np.abs(h0).max()), (b, layer)
            assert np.abs(xp1 - xp0).max() <= 1e-4 * max(1.0, np.abs(xp0).max())
            assert np.abs(bp1 - bp0).max() <= 1e-3 * max(1.0, np.abs(bp0).max())     # follows the accumulated angle
            d = np.abs(np.mod(cu1 - cu0 + np.pi, two_pi) - np.pi)          # equal modulo 2 pi
            assert d.max() < 1e-3, (b, layer, d.max())   # 200 accumulated increments from two differently rounded GEMM paths
    # against the oracle, including what decode makes of the handed-over state
    ost = cpu_oracle.OracleModel(cfg, tens).init_states()
    ref_toks, ref_logits = ost.generate(prompts[1], n_new, ignore_eos=True, dump_logits=True)
    chk.reset()
    toks, lens, dump, st = chk.generate(prompts, n_new, ignore_eos=True, dump_logits=True)
    assert max(rel_err(dump[i, 1], ref_logits[i]) for i in range(n_new)) < TOL_F32
    _compare_tokens(toks[1], ref_toks, ref_logits, "chunked prefill, sequence 1")
    assert st.ms_prefill > 0


def test_two_lane_execution_matches_single_lane():
    """Large tensor-core batches run as two lanes of sequences on separate streams; rows are
    independent, so tokens and logits must not change at all."""
    cfg = synth.base_config(n_layers=4, vocab_size=2048)
    tens = list(synth.iter_tensors(cfg, seed=2, weights_dtype="bf16"))
    B, T, n_new = 96, 6, 10
    prompts = synth.random_prompts(B, T, cfg.vocab_size, seed=4)
    model = lumi_b200.NmModel.from_tensors(cfg, tens)
    outs = []
    for overlap in (0, 32):
        sess = model.init_states(B)
        sess.set_option("overlap", overlap)
        toks, lens, dump, st = sess.generate(prompts, n_new, ignore_eos=True, dump_logits=True)
        outs.append((toks.copy(), dump.copy()))
        sess.close()
    assert np.array_equal(outs[0][0], outs[1][0])
    assert np.array_equal(outs[0][1], outs[1][1])
    ref_toks, ref_logits = cpu_oracle.OracleModel(cfg, tens).init_states().generate(prompts[95], n_new, ignore_eos=True, dump_logits=True)
    assert max(rel_err(outs[1][1][i, 95], ref_logits[i]) for i in range(n_new)) < TOL_F32
    _compare_tokens(outs[1][0][95], ref_toks, ref_logits, "two lanes, last sequence")


def test_hybrid_bf16_tensor_core_path():
    cfg = synth.tiny_config(attention_interval=2, attn_rope_base=10000.0, attn_mlp_dim=320)
    tens = list(synth.iter_tensors(cfg, seed=8, weights_dtype="bf16", perturb_ones=0.1))
    B, T, n_new = 12, 10, 12
    prompts = synth.random_prompts(B, T, cfg.vocab_size, seed=3)
    model = lumi_b200.NmModel.from_tensors(cfg, tens)
    sess = model.init_states(B, 64)
    toks, lens, dump, st = sess.generate(prompts, n_new, ignore_eos=True, dump_logits=True)
    om = cpu_oracle.OracleModel(cfg, tens)
    for b in (0, 11):
        ref_toks, ref_logits = om.init_states().generate(prompts[b], n_new, ignore_eos=True, dump_logits=True)
        n_same = n_new if np.array_equal(toks[b], ref_toks) else int(np.argmax(toks[b] != ref_toks)) + 1
        assert max(rel_err(dump[i, b], ref_logits[i]) for i in range(n_same)) < TOL_BF16   # bf16 KV cache


def test_forward_step_api_and_sampling_with_philox():
    z, cfg, tens = load_golden("tiny_mamba")
    model = lumi_b200.NmModel.from_tensors(cfg, tens)
    sess = model.init_states(1)
    om = cpu_oracle.OracleModel(cfg, tens).init_states()
    tok = int(z["prompt"][0])
    sp = lumi_b200.Sampling(0.9, 0, 1234, 2, 1)
    for step in range(12):
        logits, nxt = sess.forward_step([tok], sampling=sp, step=step)
        ref = om.forward_step(tok)
        assert rel_err(logits[0], ref) < TOL_F32
        r = nr.sampler_uniform(1234, 0, step)
        want = cpu_oracle.sample(logits[0], 0.9, 0, float(r))
        # whole-vocabulary sampling sums in chunk order: allow a different pick only at a CDF boundary
        if int(nxt[0]) != want:
            p = np.exp((logits[0] * np.float32(1 / 0.9)).astype(np.float64))
            cdf = np.cumsum(p / p.sum())
            assert np.abs(cdf - float(r)).min() < 1e-5
        tok = want


def test_eos_and_lengths():
    z, cfg, tens = load_golden("tiny_mamba")
    model = lumi_b200.NmModel.from_tensors(cfg, tens)
    sess = model.init_states(1)
    eos = int(z["tokens"][3])
    first = int(np.argmax(z["tokens"] == eos))
    toks, lens, _, _ = sess.generate(z["prompt"][None, :], 24, eos_id=eos)
    assert lens[0] == first and np.array_equal(toks[0, :first], z["tokens"][:first])


def test_session_reset_restores_initial_state():
    z, cfg, tens = load_golden("tiny_hybrid")
    model = lumi_b200.NmModel.from_tensors(cfg, tens)
    sess = model.init_states(2, 64)
    a, _, _, _ = sess.generate(np.stack([z["prompt"]] * 2), 8, ignore_eos=True)
    sess.reset([1])
    sess.reset([0])
    b, _, _, _ = sess.generate(np.stack([z["prompt"]] * 2), 8, ignore_eos=True)
    assert np.array_equal(a, b)


@pytest.mark.parametrize("kind", ["tiny_mamba", "tiny_hybrid"])
def test_sequence_snapshot_resumes_in_another_slot(kind):
    """Park a sequence on the host after a few tokens and resume it in another slot of another session:
    the continuation is the one the uninterrupted run (and the oracle) produces."""
    cfg = synth.tiny_config(n_layers=4, attention_layers=[1, 3] if kind == "tiny_hybrid" else [])
    tens = list(synth.iter_tensors(cfg, seed=8, perturb_ones=0.1))
    prompt = synth.random_prompts(1, 7, cfg.vocab_size, seed=4)[0]
    ref = cpu_oracle.OracleModel(cfg, tens).init_states().generate(prompt, 12, ignore_eos=True)
    model = lumi_b200.NmModel.from_tensors(cfg, tens)
    s1 = model.init_states(1, 32)
    s1.prefill(prompt[None, :-1], want_logits=False)
    cur, got = prompt[-1:], []
    for i in range(5):
        _, cur = s1.forward_step(cur, want_logits=False)
        got.append(int(cur[0]))
    snap = s1.save_state(0)
    s2 = model.init_states(3, 32)
    other = synth.random_prompts(3, 4, cfg.vocab_size, seed=9)
    s2.prefill(other, want_logits=False)              # the other slots hold unrelated sequences
    s2.load_state(2, snap)
    toks = np.array([other[0, -1], other[1, -1], cur[0]], dtype=np.uint32)
    for i in range(7):
        _, toks = s2.forward_step(toks, want_logits=False)
        got.append(int(toks[2]))
    assert got == [int(t) for t in ref]
    # a snapshot of another model is refused
    cfg2 = synth.tiny_config(n_layers=2)
    m2 = lumi_b200.NmModel.from_tensors(cfg2, list(synth.iter_tensors(cfg2, seed=1)))
    with pytest.raises(lumi_b200.LumiError):
        m2.init_states(1, 32).load_state(0, snap)


@pytest.mark.parametrize("case", ["tiny_hybrid_f32", "base_bf16_batch12", "base_bf16_long", "hybrid_bf16_long"])
def test_score_matches_oracle_log_softmax(case):
    """Teacher-forced log-probabilities at every position (what `evaluate` sums, inference/src/eval.rs:39-139)
    against log-softmax of the oracle's per-position logits; the state afterwards continues like a prefill."""
    if case == "tiny_hybrid_f32":
        cfg = synth.tiny_config(n_layers=4, attention_layers=[2])
        tens = list(synth.iter_tensors(cfg, seed=6, perturb_ones=0.1))
        B, T, tol = 3, 11, 2e-4
    elif case == "base_bf16_batch12":
        cfg = synth.base_config(n_layers=2, vocab_size=777)
        tens = list(synth.iter_tensors(cfg, seed=6, weights_dtype="bf16"))
        B, T, tol = 12, 6, 2e-3
    else:
        # long windows go through the batched prefill (chunked scan, head as one GEMM over all rows)
        kw = dict(attention_layers=[1], attn_mlp_dim=512) if case == "hybrid_bf16_long" else {}
        cfg = synth.base_config(n_layers=2, vocab_size=777, **kw)
        tens = list(synth.iter_tensors(cfg, seed=6, weights_dtype="bf16"))
        B, T, tol = 3, 140, 2e-3
    toks = synth.random_prompts(B, T, cfg.vocab_size, seed=12)
    model = lumi_b200.NmModel.from_tensors(cfg, tens)
    sess = model.init_states(B, 256)
    got = sess.score(toks)
    assert got.shape == (B, T - 1)
    om = cpu_oracle.OracleModel(cfg, tens)
    for b in (0, B - 1):
        st = om.init_states()
        for t in range(T - 1):
            lg = st.forward_step(int(toks[b, t])).astype(np.float64)
            ref = lg[toks[b, t + 1]] - (np.log(np.exp(lg - lg.max()).sum()) + lg.max())
            assert abs(got[b, t] - ref) < tol * max(1.0, abs(ref)), (b, t, got[b, t], ref)
    # the state is that of a prefill of all T tokens: the same next tokens as prefill + decode
    _, nxt = sess.forward_step(toks[:, -1] * 0 + 5, want_logits=False)
    s2 = model.init_states(B, 256)
    s2.prefill(toks, want_logits=False)
    _, nxt2 = s2.forward_step(toks[:, -1] * 0 + 5, want_logits=False)
    assert np.array_equal(nxt, nxt2)


@pytest.mark.parametrize("rows", [32768, 256])
def test_chunked_prefill_with_attention_layers(rows):
    """bf16 hybrid model (Mamba, attention, Mamba, attention), 150-token prompts: the batched prefill — chunked
    scan for the Mamba layers, all rows of a slice through the attention layers at once — against the
    token-by-token prefill and the oracle: last-position logits, Mamba state, and the greedy continuation
    (which reads the K/V cache the prefill left behind).  rows = 256 forces slices of 64 tokens."""
    cfg = synth.base_config(n_layers=4, vocab_size=1000, attention_layers=[1, 3], attn_mlp_dim=512, attn_rope_base=10000.0)
    tens = list(synth.iter_tensors(cfg, seed=16, weights_dtype="bf16", perturb_ones=0.05))
    B, T, n_new = 4, 150, 8
    prompts = synth.random_prompts(B, T, cfg.vocab_size, seed=19)
    model = lumi_b200.NmModel.from_tensors(cfg, tens)
    step = model.init_states(B, 256)
    step.set_option("chunked_prefill", 0)
    lg_step = step.prefill(prompts)
    chk = model.init_states(B, 256)
    chk.set_option("chunked_prefill", 64)
    chk.set_option("prefill_rows", rows)
    lg_chk = chk.prefill(prompts)
    for b in range(B):
        assert rel_err(lg_chk[b], lg_step[b]) < 2e-4, (b, rel_err(lg_chk[b], lg_step[b]))
        for layer in (0, 2):
            h1, xp1, bp1, cu1 = chk.read_state(b, layer)
            h0, xp0, bp0, cu0 = step.read_state(b, layer)
            assert np.abs(h1 - h0).max() <= 2e-4 * max(1.0, np.abs(h0).max()), (b, layer)
    # continuation: both sessions decode the same tokens from their caches
    nxt = prompts[:, -1] * 0 + 7
    for i in range(4):
        _, a = step.forward_step(nxt, want_logits=False)
        _, c = chk.forward_step(nxt, want_logits=False)
        assert np.array_equal(a, c), (i, a, c)
        nxt = a
    ost = cpu_oracle.OracleModel(cfg, tens).init_states()
    ref_toks, ref_logits = ost.generate(prompts[2], n_new, ignore_eos=True, dump_logits=True)
    chk.reset()
    toks, lens, dump, st = chk.generate(prompts, n_new, ignore_eos=True, dump_logits=True)
    assert max(rel_err(dump[i, 2], ref_logits[i]) for i in range(n_new)) < TOL_BF16
    _compare_tokens(toks[2], ref_toks, ref_logits, "hybrid chunked prefill, sequence 2")


@pytest.mark.parametrize("case", ["hpk1", "hpk2", "hpk8", "window", "slices", "many_pages"])
def test_tensor_core_attention_shapes(case):
    """The attention kernel for a bf16 cache with 64-wide heads (tensor cores, pages staged by tensor-map copies) against
    the oracle, over what its index arithmetic depends on: 1 / 2 / 8 query heads per KV head (16, 8, 2 token rows per
    CTA in the batched prefill; 4 is what the other hybrid tests run, with a ragged last group: 150 is not a multiple of 16), a sliding window whose ring wraps
    (decode form only: such a prompt goes token by token), and a context long enough to be split over several CTAs at a
    batch of two (partial pages at the slice ends), or over more slices than it has pages (empty slices; a capacity of more
    than 64 pages).  The batched prefill is also held against the token-by-token one."""
    kv = {"hpk1": 16, "hpk2": 8, "hpk8": 2}.get(case, 4)
    kw = dict(n_layers=2, vocab_size=500, attention_layers=[1], attn_mlp_dim=256, attn_rope_base=10000.0, attn_kv_heads=kv)
    B, T, n_new, cap = 3, 150, 6, 256
    if case == "window":
        kw["attn_window_sizes"] = [40]
        T = 70
    if case == "slices":
        B, T, cap = 2, 600, 1024
    if case == "many_pages":
        B, T, cap = 1, 150, 4200     # a page table too long for the kernel's shared-memory copy, and 16 slices of which 13 are empty
    cfg = synth.base_config(**kw)
    assert cfg.attn_head_dim == 64
    tens = list(synth.iter_tensors(cfg, seed=21, weights_dtype="bf16", perturb_ones=0.05))
    prompts = synth.random_prompts(B, T, cfg.vocab_size, seed=5)
    model = lumi_b200.NmModel.from_tensors(cfg, tens)
    sess = model.init_states(B, cap)
    toks, lens, dump, st = sess.generate(prompts, n_new, ignore_eos=True, dump_logits=True)
    om = cpu_oracle.OracleModel(cfg, tens)
    worst = 0.0
    for b in (0, B - 1):
        ref_toks, ref_logits = om.init_states().generate(prompts[b], n_new, ignore_eos=True, dump_logits=True)
        n_same = n_new if np.array_equal(toks[b], ref_toks) else int(np.argmax(toks[b] != ref_toks)) + 1
        worst = max(worst, max(rel_err(dump[i, b], ref_logits[i]) for i in range(n_same)))
        _compare_tokens(toks[b], ref_toks, ref_logits, f"{case}, sequence {b}")
    print(f"{case}: worst logit error against the oracle {worst:.2e}")
    assert worst < 2e-4            # measured 4e-6 .. 8e-6 (the cache holds bf16 K / V, the oracle fp32)
    if case != "window":
        step = model.init_states(B, cap)
        step.set_option("chunked_prefill", 0)
        lg_step = step.prefill(prompts)
        sess.reset()
        lg = sess.prefill(prompts)
        for b in range(B):
            assert rel_err(lg[b], lg_step[b]) < 2e-4, (b, rel_err(lg[b], lg_step[b]))
        step.close()
    sess.close()
    model.close()


@pytest.mark.parametrize("case", ["mamba", "hybrid", "hybrid_hd32"])
def test_ragged_prefill_of_long_prompts_takes_the_batched_path(case):
    """Prompts of different lengths, the longest long enough for the batched prefill (chunked scan, tensor-core GEMMs, every row
    of a slice through the attention layers at once): each sequence must end in the state, with the last-position logits
    and the K/V cache, of a prefill of its own tokens alone; the logits are also held against the oracle, and decoding
    continues for all sequences together.  Lengths cover: the longest, one token, exactly one chunk, one past a chunk, a
    slice boundary (prefill_rows forces 64-token slices in the hybrid cases) and a ragged group of attention rows."""
    kw = dict(n_layers=3, vocab_size=700)
    if case == "hybrid":
        kw.update(attention_layers=[1], attn_mlp_dim=256, attn_rope_base=10000.0)                 # 64-wide heads: tensor-core attention
    if case == "hybrid_hd32":
        kw.update(attention_layers=[1], attn_mlp_dim=256, attn_n_heads=32, attn_kv_heads=8)        # 32-wide heads: CUDA-core attention
    cfg = synth.base_config(**kw)
    tens = list(synth.iter_tensors(cfg, seed=29, weights_dtype="bf16", perturb_ones=0.05))
    lengths = np.array([200, 1, 64, 65, 128, 137, 199, 3], dtype=np.int32)
    B, T_max, cap = len(lengths), 200, 256
    prompts = synth.random_prompts(B, T_max, cfg.vocab_size, seed=31)
    padded = prompts.copy()
    for b in range(B):
        padded[b, lengths[b]:] = 0xFFFFFFF0                  # padding is never looked at, not even range-checked
    model = lumi_b200.NmModel.from_tensors(cfg, tens)
    sess = model.init_states(B, cap)
    if case != "mamba":
        sess.set_option("prefill_rows", 512)                 # 8 sequences x 64 tokens per slice
    logits = sess.prefill_ragged(padded, lengths)
    mamba_layers = [i for i in range(cfg.n_layers) if not cfg.is_attention_layer(i)]
    om = cpu_oracle.OracleModel(cfg, tens)
    alone = model.init_states(1, cap)
    alone.set_option("chunked_prefill", 1)                  # the batched path whatever the length: the same arithmetic as above
    nxt = np.zeros(B, dtype=np.uint32)
    refs = []
    for b in range(B):
        alone.reset()
        lg1 = alone.prefill(prompts[b:b + 1, :lengths[b]])
        assert rel_err(logits[b], lg1[0]) < 2e-4, (case, b, int(lengths[b]), rel_err(logits[b], lg1[0]))
        for layer in mamba_layers:
            h, xp, bp, cum = sess.read_state(b, layer)
            h1, xp1, bp1, cum1 = alone.read_state(0, layer)
            assert np.abs(h - h1).max() <= 2e-4 * max(1.0, np.abs(h1).max()), (case, b, layer)
            assert np.abs(xp - xp1).max() <= 2e-4 * max(1.0, np.abs(xp1).max()) and np.abs(bp - bp1).max() <= 2e-4 * max(1.0, np.abs(bp1).max())
            assert np.abs(cum - cum1).max() < 2e-4
        st = om.init_states()
        for t in prompts[b, :lengths[b]]:
            ref = st.forward_step(int(t))
        refs.append(st)
        assert rel_err(logits[b], ref) < TOL_F32, (case, b, int(lengths[b]), rel_err(logits[b], ref))
        nxt[b] = cpu_oracle.argmax(ref)
    # decoding continues for all sequences together: reads every sequence's K/V cache at its own position
    for i in range(4):
        lg, out = sess.forward_step(nxt, step=i)
        for b in range(B):
            ref = refs[b].forward_step(int(nxt[b]))
            assert rel_err(lg[b], ref) < TOL_F32, (case, "decode", i, b, rel_err(lg[b], ref))
            nxt[b] = cpu_oracle.argmax(ref)
    alone.close()
    sess.close()
    model.close()


def test_slot_reuse_by_transplanting_a_prefilled_sequence():
    """Continuous batching with the snapshot calls: while a batch of three sequences decodes, sequence 1 ends; a new
    prompt is prefilled in a one-slot side session, its snapshot is loaded into slot 1, and decoding goes on.
    The newcomer's tokens are the oracle's for its prompt; the neighbours never notice."""
    cfg = synth.tiny_config(n_layers=4, attention_layers=[2])
    tens = list(synth.iter_tensors(cfg, seed=21, perturb_ones=0.1))
    om = cpu_oracle.OracleModel(cfg, tens)
    prompts = synth.random_prompts(3, 6, cfg.vocab_size, seed=22)
    newcomer = synth.random_prompts(1, 9, cfg.vocab_size, seed=23)[0]
    refs = [om.init_states().generate(prompts[b], 10, ignore_eos=True) for b in range(3)]
    ref_new = om.init_states().generate(newcomer, 6, ignore_eos=True)
    model = lumi_b200.NmModel.from_tensors(cfg, tens)
    main = model.init_states(3, 64)
    main.prefill(prompts[:, :-1], want_logits=False)
    cur = prompts[:, -1].copy()
    got = [[], [], []]
    for i in range(4):
        _, cur = main.forward_step(cur, want_logits=False)
        for b in range(3): got[b].append(int(cur[b]))
    # sequence 1 is done: bring the newcomer in
    side = model.init_states(1, 64)
    side.prefill(newcomer[None, :-1], want_logits=False)
    main.load_state(1, side.save_state(0))
    cur = cur.copy(); cur[1] = newcomer[-1]
    new_tokens = []
    for i in range(6):
        _, cur = main.forward_step(cur, want_logits=False)
        got[0].append(int(cur[0])); got[2].append(int(cur[2])); new_tokens.append(int(cur[1]))
    assert got[0] == [int(t) for t in refs[0]] and got[2] == [int(t) for t in refs[2]]
    assert got[1] == [int(t) for t in refs[1][:4]]
    assert new_tokens == [int(t) for t in ref_new]


@pytest.mark.parametrize("wdt,B", [("f32", 1), ("bf16", 3), ("f32", 8)])
def test_greedy_head_with_fused_argmax_matches_logits_path_and_oracle(wdt, B):
    """Batch <= 8, greedy, no logits asked for: the argmax rides behind the lm_head GEMV (per-CTA partials, one
    finishing kernel) and no logits are written.  Tokens, lengths and eos handling must equal the path that writes the
    logits and samples from them, and the oracle's greedy tokens; lumi_decode_step without a logits buffer takes the
    same path."""
    cfg = synth.base_config(n_layers=2, vocab_size=8192)
    tens = list(synth.iter_tensors(cfg, seed=17, weights_dtype=wdt, perturb_ones=0.05))
    T, n_new = 7, 24
    prompts = synth.random_prompts(B, T, cfg.vocab_size, seed=6)
    model = lumi_b200.NmModel.from_tensors(cfg, tens)
    sess = model.init_states(B)
    toks_fused, lens_fused, _, st = sess.generate(prompts, n_new, ignore_eos=True)                    # fused head
    sess.reset()
    toks_plain, lens_plain, dump, _ = sess.generate(prompts, n_new, ignore_eos=True, dump_logits=True)  # logits + sample_kernel
    assert np.array_equal(toks_fused, toks_plain) and np.array_equal(lens_fused, lens_plain)
    om = cpu_oracle.OracleModel(cfg, tens)
    for b in (0, B - 1):
        ref_toks, ref_logits = om.init_states().generate(prompts[b], n_new, ignore_eos=True, dump_logits=True)
        _compare_tokens(toks_fused[b], ref_toks, ref_logits, f"fused greedy head, sequence {b}")
    # eos: stop where the plain path stops
    eos = int(toks_plain[0, 5])
    sess.reset()
    a, la, _, _ = sess.generate(prompts, n_new, eos_id=eos)
    sess.reset()
    b_, lb, _, _ = sess.generate(prompts, n_new, eos_id=eos, dump_logits=True)
    assert np.array_equal(la, lb)
    for i in range(B):
        assert np.array_equal(a[i, :la[i]], b_[i, :lb[i]])
    # token by token through lumi_decode_step without a logits buffer
    sess.reset()
    sess.prefill(prompts[:, :-1], want_logits=False)
    tok = prompts[:, -1].copy()
    for i in range(6):
        _, tok = sess.forward_step(tok, want_logits=False, step=i)
        assert np.array_equal(tok, toks_plain[:, i]), i


@pytest.mark.parametrize("case", ["mamba_f32", "hybrid_f32", "mamba_bf16_tc"])
def test_ragged_prefill_equals_each_prompt_alone(case):
    """Prompts of different lengths in one call: every sequence must end in the state, and give the last-position
    logits, of a prefill of its own tokens alone — and decoding continues from there like the oracle."""
    if case == "hybrid_f32":
        cfg = synth.tiny_config(attention_interval=2, attn_rope_base=10000.0, attn_window_sizes=[5])
        wdt, B = "f32", 4
    elif case == "mamba_bf16_tc":
        cfg = synth.base_config(n_layers=2, vocab_size=1000)
        wdt, B = "bf16", 12                                  # batch > 8: tensor-core GEMMs with the folded norm
    else:
        cfg = synth.base_config(n_layers=2, vocab_size=1000)
        wdt, B = "f32", 3
    tens = list(synth.iter_tensors(cfg, seed=23, weights_dtype=wdt, perturb_ones=0.05))
    g = np.random.default_rng(5)
    T_max = 11
    lengths = g.integers(1, T_max + 1, size=B).astype(np.int32)
    lengths[0], lengths[-1] = T_max, 1
    prompts = synth.random_prompts(B, T_max, cfg.vocab_size, seed=8)
    padded = prompts.copy()
    for b in range(B):
        padded[b, lengths[b]:] = 0xFFFFFFF0                  # padding is never looked at, not even range-checked
    model = lumi_b200.NmModel.from_tensors(cfg, tens)
    sess = model.init_states(B, 64)
    logits = sess.prefill_ragged(padded, lengths)
    om = cpu_oracle.OracleModel(cfg, tens)
    mamba_layers = [i for i in range(cfg.n_layers) if not cfg.is_attention_layer(i)]
    tol = TOL_F32
    nxt = np.zeros(B, dtype=np.uint32)
    refs = []
    for b in range(B):
        st = om.init_states()
        for t in prompts[b, :lengths[b]]:
            ref = st.forward_step(int(t))
        refs.append(st)
        assert rel_err(logits[b], ref) < tol, (case, b, int(lengths[b]))
        nxt[b] = cpu_oracle.argmax(ref)
        for layer in mamba_layers:
            h, xp, bp, cum = sess.read_state(b, layer)
            rh, rpbx, rcum = st.read_state(layer)
            assert np.abs(h - rh).max() <= 1e-4 * max(1.0, np.abs(rh).max()), (case, b, layer)
            assert np.abs(xp[:, :, None] * bp[:, None, :] - rpbx).max() <= 1e-4 * max(1.0, np.abs(rpbx).max())
            assert np.abs(cum - rcum).max() < 1e-4
    # decoding continues for all sequences together (this also checks the attention positions of the hybrid case)
    for i in range(4):
        lg, out = sess.forward_step(nxt, step=i)
        for b in range(B):
            ref = refs[b].forward_step(int(nxt[b]))
            assert rel_err(lg[b], ref) < tol, (case, "decode", i, b)
            nxt[b] = cpu_oracle.argmax(ref)
