"""GPU: the allocation-free Mamba block (lumi_mamba_block_static) against the session-based block.

Collected last on purpose.  Some hosts cannot allocate at the point where they need a block — their
own pool owns the device, or they are inside a stream capture, or they may not take the
synchronisation an allocation implies — so this entry point keeps its intermediates in a fixed
device array inside the library and takes everything else as device pointers.  The check: two calls
in a row (two consecutive tokens) give the same residual stream and the same state as two calls of
the existing session entry point, within the tolerance the block tests use; and oversize requests
are refused."""
import numpy as np
import pytest

import lumi_b200
from lumi_b200 import synth

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("wdt", ["f32", "bf16"])
def test_static_block_matches_session_block_twice(wdt):
    import torch
    cfg = synth.base_config(n_layers=2, vocab_size=512)
    tens = list(synth.iter_tensors(cfg, seed=13, weights_dtype=wdt, perturb_ones=0.1))
    model = lumi_b200.NmModel.from_tensors(cfg, tens)
    B, layer = 3, 1
    H, P, N, D = cfg.n_heads, cfg.head_dim, cfg.d_state, cfg.d_model
    g = np.random.default_rng(3)
    xs = [g.standard_normal((B, D)).astype(np.float32) for _ in range(2)]

    # existing entry point: session scratch
    sess = model.init_states(B)
    want = [sess.run_block(layer, x) for x in xs]
    want_state = [sess.read_state(b, layer) for b in range(B)]

    # new entry point: caller-owned device buffers, library-owned fixed scratch
    h_init = dict((n, a) for n, _, a in tens)[f"item.blocks.{layer}.ssm.h_init"]
    h = torch.from_numpy(np.broadcast_to(h_init[None, :, None, :], (B, H, P, N)).copy()).cuda()
    xp = torch.zeros((B, H, P), dtype=torch.float32, device="cuda")
    bp = torch.zeros((B, H, N), dtype=torch.float32, device="cuda")
    cum = torch.zeros((B, H, N // 2), dtype=torch.float32, device="cuda")
    got = []
    for x in xs:                                   # two calls in a row share the scratch
        xd = torch.from_numpy(x).cuda()
        torch.cuda.synchronize()
        lumi_b200.api.check(lumi_b200.lib().lumi_mamba_block_static(model._h, layer, xd.data_ptr(), h.data_ptr(), xp.data_ptr(),
                                                                bp.data_ptr(), cum.data_ptr(), B, 0))
        torch.cuda.synchronize()
        got.append(xd.cpu().numpy())
    for a, b in zip(got, want):
        assert np.abs(a - b).max() <= 1e-5 * np.abs(b).max()
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
