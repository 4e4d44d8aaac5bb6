"""GPU: the allocation-free Mamba block (lumi_mamba_block_static), through the C ABI.

Collected last on purpose.  Some hosts cannot allocate at the point where they need a block — their
own pool owns the device, or they are inside a stream capture, or they may not take the
synchronisation an allocation implies — so this entry point keeps its intermediates in a fixed
device array inside the library and takes everything else as device pointers.  The checks: calls in a
row (consecutive tokens, sharing the array) give the residual stream and the state of the existing
session entry point AND of the CPU oracle's block, within the tolerance the block tests use, for batch
sizes that take each of the GEMV kernels (3, 5, 8); the free device memory does not move across the
calls after the first; and requests beyond the fixed array are refused."""
import numpy as np
import pytest

import lumi_b200
from lumi_b200 import synth
from oracle import cpu_oracle

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("wdt,B", [("f32", 3), ("bf16", 3), ("f32", 5), ("bf16", 8)])
def test_static_block_matches_session_block_and_oracle(wdt, B):
    import torch
    cfg = synth.base_config(n_layers=2, vocab_size=512)
    tens = list(synth.iter_tensors(cfg, seed=13, weights_dtype=wdt, perturb_ones=0.1))
    model = lumi_b200.NmModel.from_tensors(cfg, tens)
    layer, n_calls = 1, 3
    H, P, N, D = cfg.n_heads, cfg.head_dim, cfg.d_state, cfg.d_model
    g = np.random.default_rng(3)
    xs = [g.standard_normal((B, D)).astype(np.float32) for _ in range(n_calls)]

    # existing entry point: session scratch
    sess = model.init_states(B)
    want = [sess.run_block(layer, x) for x in xs]
    want_state = [sess.read_state(b, layer) for b in range(B)]
    # the CPU oracle's block (inference/src/model.rs:296-375), first and last sequence
    om = cpu_oracle.OracleModel(cfg, tens)
    oracle_rows = {}
    for b in (0, B - 1):
        st = om.init_states()
        oracle_rows[b] = [st.mamba_block(layer, x[b]) for x in xs]

    # new entry point: caller-owned device buffers, library-owned fixed scratch
    h_init = synth.as_f32(*[(dt, a) for n, dt, a in tens if n == f"item.blocks.{layer}.ssm.h_init"][0])
    h = torch.from_numpy(np.broadcast_to(h_init[None, :, None, :], (B, H, P, N)).copy()).cuda()
    xp = torch.zeros((B, H, P), dtype=torch.float32, device="cuda")
    bp = torch.zeros((B, H, N), dtype=torch.float32, device="cuda")
    cum = torch.zeros((B, H, N // 2), dtype=torch.float32, device="cuda")
    xds = [torch.from_numpy(x).cuda() for x in xs]       # every buffer exists before the calls: nothing below allocates
    torch.cuda.synchronize()
    free_after_first = None
    for i, xd in enumerate(xds):                         # calls in a row share the scratch
        lumi_b200.api.check(lumi_b200.lib().lumi_mamba_block_static(model._h, layer, xd.data_ptr(), h.data_ptr(), xp.data_ptr(),
                                                                bp.data_ptr(), cum.data_ptr(), B, 0))
        torch.cuda.synchronize()
        free_now = torch.cuda.mem_get_info()[0]
        if i == 0:
            free_after_first = free_now                  # the first launch of a kernel may load its code
        else:
            assert free_now == free_after_first, "device memory moved across an allocation-free call"
    got = [xd.cpu().numpy() for xd in xds]
    for a, b in zip(got, want):
        assert np.abs(a - b).max() <= 1e-5 * np.abs(b).max()
    for b, rows in oracle_rows.items():
        for i in range(n_calls):
            added, ref = got[i][b] - xs[i][b], rows[i] - xs[i][b]          # what the block added to the residual stream
            assert np.abs(added - ref).max() <= 1e-5 * np.abs(ref).max(), (b, i)
    for b in range(B):
        wh, wxp, wbp, wcum = want_state[b]
        assert np.abs(h[b].cpu().numpy() - wh).max() <= 1e-5 * max(1.0, np.abs(wh).max())
        assert np.abs(xp[b].cpu().numpy() - wxp).max() <= 1e-6 and np.abs(bp[b].cpu().numpy() - wbp).max() <= 1e-5
        assert np.abs(cum[b].cpu().numpy() - wcum).max() <= 1e-5


def test_static_block_refuses_oversize():
    import torch
    cfg = synth.tiny_config(n_layers=1)
    model = lumi_b200.NmModel.from_tensors(cfg, synth.iter_tensors(cfg, seed=1))
    buf = torch.zeros(1 << 20, dtype=torch.float32, device="cuda")
    p = buf.data_ptr()
    st = lumi_b200.lib().lumi_mamba_block_static(model._h, 0, p, p, p, p, p, 9, 0)
    assert st == -10 and "batch 9" in lumi_b200.lib().lumi_last_error().decode()
    st = lumi_b200.lib().lumi_mamba_block_static(model._h, 5, p, p, p, p, p, 1, 0)
    assert st == -1
    # a block whose two intermediates need more than the fixed 16384 floats per sequence
    wide = synth.base_config(n_layers=1, vocab_size=64, d_model=2048, n_heads=128)
    assert wide.in_proj_out + wide.d_inner > 16384
    big = lumi_b200.NmModel.from_tensors(wide, synth.iter_tensors(wide, seed=1))
    st = lumi_b200.lib().lumi_mamba_block_static(big._h, 0, p, p, p, p, p, 1, 0)
    assert st == -10 and "exceeds the fixed scratch" in lumi_b200.lib().lumi_last_error().decode()
