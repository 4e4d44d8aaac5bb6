"""GPU: the CPU oracle's block functions against whole-block outputs computed by the reference's OWN CUDA
forward kernels, chained as the reference's trainer chains them (tests/ref_chain.py:
`mamba_block_forward`, training/src/native_trainer.rs:198-266, and `attention_block_forward`, :110-194).

This pins `oracle_mamba_block` and `oracle_attention_block` (no rotary embedding — the reference has none) to
code written by the reference's authors beyond the recurrence alone: RMSNorm, the in_proj column layout and
its 5-way split, sigmoid / negative softplus with clamp / SiLU, BCNorm over all n_groups * d_state with bias,
the scan with h_init, D skip and z gate, out_proj and the residual; and for attention q/k/v, the GQA head
mapping, 1/sqrt(head_dim), the causal (and sliding-window) softmax, the output projection and the
sigmoid-gated MLP.  The CUDA path of this library is compared with the same outputs in the same test.

Tolerance: the reference kernels use exp2f / rsqrtf forms, sin/cos.approx and atomics (fast-math build,
training/build.rs:38-41), so agreement is to ~1e-4 of the largest output, not to the last bit; TF32 is
switched off for the child process (NVIDIA_TF32_OVERRIDE=0) so cuBLAS does not dominate the difference.
"""
import os
import subprocess
import sys

import numpy as np
import pytest

import lumi_b200
from lumi_b200 import synth
from oracle import cpu_oracle
from tests.helpers import rel_err

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "oracle", "_ref", "libref_fwd.so")
TOL_REF = 5e-4


def _run_chain(tmp_path, **arrays):
    if not os.path.exists(REF):
        pytest.skip("oracle/_ref/libref_fwd.so not built (needs the reference checkout)")
    fin, fout = str(tmp_path / "in.npz"), str(tmp_path / "out.npz")
    np.savez(fin, **arrays)
    env = dict(os.environ, NVIDIA_TF32_OVERRIDE="0")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "ref_chain.py"), fin, fout], env=env,
                       stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:]
    return np.load(fout)["y"]


def _w(tens, name):
    for n, dt, a in tens:
        if n == "item." + name:
            return synth.as_f32(dt, a)
    raise KeyError(name)


@pytest.mark.parametrize("shape", ["base", "tiny"])
def test_mamba_block_against_reference_kernel_chain(tmp_path, shape):
    cfg = synth.base_config(n_layers=1, vocab_size=512) if shape == "base" else synth.tiny_config(n_layers=1)
    tens = list(synth.iter_tensors(cfg, seed=12, perturb_ones=0.1))
    B, T = 2, 40
    g = np.random.default_rng(3)
    x = g.standard_normal((B, T, cfg.d_model)).astype(np.float32)
    pre = "blocks.0."
    want = _run_chain(
        tmp_path, kind="mamba", batch=B, seq=T, d_model=cfg.d_model, eps=1e-5, x=x, n_heads=cfg.n_heads, head_dim=cfg.head_dim,
        d_state=cfg.d_state, n_groups=cfg.n_groups, in_proj=_w(tens, pre + "in_proj.weight"), out_proj=_w(tens, pre + "out_proj.weight"),
        norm_g=_w(tens, pre + "norm.gamma"), b_gamma=_w(tens, pre + "b_norm.gamma"), c_gamma=_w(tens, pre + "c_norm.gamma"),
        b_bias=_w(tens, pre + "b_bias"), c_bias=_w(tens, pre + "c_bias"), d_skip=_w(tens, pre + "ssm.d"), dt_bias=_w(tens, pre + "ssm.dt_bias"),
        h_init=_w(tens, pre + "ssm.h_init"))
    # the oracle, one sequence at a time, token by token (inference/src/model.rs:296-375)
    om = cpu_oracle.OracleModel(cfg, tens)
    got_oracle = np.zeros_like(want)
    for b in range(B):
        st = om.init_states()
        for t in range(T):
            got_oracle[b, t] = st.mamba_block(0, x[b, t])
    # residual stream in, residual stream out: compare what the block ADDED, so the identity part cannot mask an error
    e_oracle = rel_err(got_oracle - x, want - x)
    # this library's CUDA block on the same inputs
    model = lumi_b200.NmModel.from_tensors(cfg, tens)
    sess = model.init_states(B)
    got_cuda = np.zeros_like(want)
    for t in range(T):
        got_cuda[:, t] = sess.run_block(0, np.ascontiguousarray(x[:, t]))
    e_cuda = rel_err(got_cuda - x, want - x)
    print(f"mamba block ({shape}) vs the reference's kernel chain over {T} tokens: oracle {e_oracle:.2e}, CUDA path {e_cuda:.2e}")
    assert e_oracle < TOL_REF
    assert e_cuda < TOL_REF


@pytest.mark.parametrize("window", [0, 7])
def test_attention_block_against_reference_kernel_chain(tmp_path, window):
    # base attention dimensions: 16 query heads / 4 kv heads of 64, sigmoid-gated MLP of 4 * d_model
    cfg = synth.base_config(n_layers=1, vocab_size=512, attention_layers=[0], attn_window_sizes=[window] if window else [])
    tens = list(synth.iter_tensors(cfg, seed=13, perturb_ones=0.1))
    # the reference's softmax kernel reduces over min(seq, 256) threads with a halving loop
    # (training/csrc/elementwise_ops.cu:1021-1024, 1043-1046), which is only complete for a power-of-two count
    B, T = 2, 32
    g = np.random.default_rng(4)
    x = g.standard_normal((B, T, cfg.d_model)).astype(np.float32)
    pre = "blocks.0."
    want = _run_chain(
        tmp_path, kind="attention", batch=B, seq=T, d_model=cfg.d_model, eps=1e-5, x=x, attn_n_heads=cfg.attn_n_heads,
        attn_kv_heads=cfg.attn_kv_heads, attn_head_dim=cfg.attn_head_dim, mlp_dim=cfg.mlp_dim, window=window,
        q_proj=_w(tens, pre + "q_proj.weight"), k_proj=_w(tens, pre + "k_proj.weight"), v_proj=_w(tens, pre + "v_proj.weight"),
        attn_out_proj=_w(tens, pre + "attn_out_proj.weight"), mlp_gate=_w(tens, pre + "mlp_gate.weight"),
        mlp_up=_w(tens, pre + "mlp_up.weight"), mlp_down=_w(tens, pre + "mlp_down.weight"),
        attn_norm_g=_w(tens, pre + "attn_norm.gamma"), mlp_norm_g=_w(tens, pre + "mlp_norm.gamma"))
    om = cpu_oracle.OracleModel(cfg, tens)
    got_oracle = np.zeros_like(want)
    for b in range(B):
        st = om.init_states()
        for t in range(T):
            got_oracle[b, t] = st.attention_block(0, x[b, t])
    e_oracle = rel_err(got_oracle - x, want - x)
    model = lumi_b200.NmModel.from_tensors(cfg, tens)
    sess = model.init_states(B, 64)
    got_cuda = np.zeros_like(want)
    for t in range(T):
        got_cuda[:, t] = sess.run_block(0, np.ascontiguousarray(x[:, t]))
    e_cuda = rel_err(got_cuda - x, want - x)
    print(f"attention block (window {window}) vs the reference's kernel chain over {T} tokens: oracle {e_oracle:.2e}, CUDA path {e_cuda:.2e}")
    assert e_oracle < TOL_REF
    assert e_cuda < TOL_REF
