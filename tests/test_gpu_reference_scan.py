"""GPU: the fused state step against the reference's OWN CUDA forward scan
(training/csrc/ssm_scan.cu, `ssm_scan_fwd_gpu`), compiled from the reference's sources into
oracle/_ref/ by `make -C oracle ref`.  The reference kernel uses sin/cos.approx, exp2-based
softplus/sigmoid and shared-memory atomics for y, so the comparison is loose (2e-3 of the
largest |y|); what it pins is the recurrence itself — trapezoid coefficients, the DD-RoPE pair
convention and angle accumulation, group-to-head mapping, the D skip and the z gate — against
code the reference's authors wrote."""
import ctypes as C
import os

import numpy as np
import pytest

import lumi_b200

pytestmark = pytest.mark.gpu

REF = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref", "libref_ssm_scan.so")


def _silu(x):
    return x / (1 + np.exp(-x))


@pytest.mark.parametrize("H,P,N,G", [(64, 32, 64, 8), (8, 32, 16, 2)])
def test_state_step_matches_reference_cuda_scan(H, P, N, G):
    if not os.path.exists(REF):
        pytest.skip("oracle/_ref/libref_ssm_scan.so not built (needs the reference checkout)")
    import torch
    ref = C.CDLL(REF)
    ref.ssm_scan_fwd_gpu.argtypes = [C.c_void_p] * 13 + [C.c_int] * 6
    B, T = 2, 24
    DI, BC = H * P, G * N
    R = 2 * DI + 2 * BC + 3 * H + H * N // 2
    g = np.random.default_rng(7)
    proj = g.standard_normal((T, B, R)).astype(np.float32)
    bg = (1 + 0.1 * g.standard_normal(BC)).astype(np.float32)
    cg = (1 + 0.1 * g.standard_normal(BC)).astype(np.float32)
    bb = (1 + 0.1 * g.standard_normal(BC)).astype(np.float32)
    cb = (1 + 0.1 * g.standard_normal(BC)).astype(np.float32)
    dsk = (1 + 0.1 * g.standard_normal(H)).astype(np.float32)
    dtb = g.uniform(-4, -1, H).astype(np.float32)
    h_init = (0.01 * g.standard_normal((H, N))).astype(np.float32)

    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    # ---- this library: T calls of the fused step
    h = dev(np.broadcast_to(h_init[None, :, None, :], (B, H, P, N)).copy())
    xp, bp, cum = dev(np.zeros((B, H, P), np.float32)), dev(np.zeros((B, H, N), np.float32)), dev(np.zeros((B, H, N // 2), np.float32))
    params = [dev(a) for a in (bg, cg, bb, cb, dsk, dtb)]
    projd = dev(proj)
    y = torch.empty((T, B, DI), dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    for t in range(T):
        lumi_b200.api.check(lumi_b200.lib().lumi_k_ssm_step(
            projd[t].data_ptr(), R, *[p.data_ptr() for p in params], h.data_ptr(), xp.data_ptr(), bp.data_ptr(), cum.data_ptr(),
            y[t].data_ptr(), B, H, P, N, G, 0))
    torch.cuda.synchronize()
    got = y.cpu().numpy().transpose(1, 0, 2)                                   # [B, T, DI]

    # ---- the reference kernel's inputs, prepared as mamba_block_forward does (native_trainer.rs:222-259)
    pr = proj.transpose(1, 0, 2).astype(np.float64)                            # [B, T, R]
    x_in = _silu(pr[..., :DI])
    z_in = pr[..., DI:2 * DI]
    bproj, cproj = pr[..., 2 * DI:2 * DI + BC], pr[..., 2 * DI + BC:2 * DI + 2 * BC]
    bn = bproj / np.sqrt((bproj ** 2).mean(-1, keepdims=True) + 1e-5) * bg + bb
    cn = cproj / np.sqrt((cproj ** 2).mean(-1, keepdims=True) + 1e-5) * cg + cb
    o = 2 * DI + 2 * BC
    dt_raw, lam = pr[..., o:o + H], 1 / (1 + np.exp(-pr[..., o + H:o + 2 * H]))
    a_vals = np.clip(-np.log1p(np.exp(pr[..., o + 2 * H:o + 3 * H])), -1e6, -1e-4)
    theta = pr[..., o + 3 * H:]
    f = lambda a: dev(a.astype(np.float32))
    d_x, d_dt, d_b, d_c = f(x_in), f(dt_raw), f(bn), f(cn)
    d_D, d_dtb, d_hi, d_lam, d_th, d_A, d_z = f(dsk), f(dtb), f(h_init), f(lam), f(theta), f(a_vals), f(z_in)
    d_y = torch.zeros((B, T, DI), dtype=torch.float32, device="cuda")
    d_yg = torch.zeros_like(d_y)
    torch.cuda.synchronize()
    ref.ssm_scan_fwd_gpu(*[t.data_ptr() for t in (d_x, d_dt, d_b, d_c, d_D, d_dtb, d_hi, d_lam, d_th, d_A, d_z, d_y, d_yg)],
                         B, T, H, P, N, G)
    torch.cuda.synchronize()
    want = d_yg.cpu().numpy()
    err = np.abs(got - want).max() / np.abs(want).max()
    print(f"state step vs reference CUDA scan: max rel err {err:.3e} over {T} steps")
    assert err < 2e-3


def _prepare_reference_inputs(proj, H, P, N, G, bg, cg, bb, cb):
    """in_proj output rows [B, T, R] -> the reference scan's inputs, as mamba_block_forward does (native_trainer.rs:222-259)."""
    DI, BC = H * P, G * N
    pr = proj.astype(np.float64)
    x_in = _silu(pr[..., :DI])
    z_in = pr[..., DI:2 * DI]
    bproj, cproj = pr[..., 2 * DI:2 * DI + BC], pr[..., 2 * DI + BC:2 * DI + 2 * BC]
    bn = bproj / np.sqrt((bproj ** 2).mean(-1, keepdims=True) + 1e-5) * bg + bb
    cn = cproj / np.sqrt((cproj ** 2).mean(-1, keepdims=True) + 1e-5) * cg + cb
    o = 2 * DI + 2 * BC
    dt_raw, lam = pr[..., o:o + H], 1 / (1 + np.exp(-pr[..., o + H:o + 2 * H]))
    a_vals = np.clip(-np.log1p(np.exp(pr[..., o + 2 * H:o + 3 * H])), -1e6, -1e-4)
    theta = pr[..., o + 3 * H:]
    return x_in, dt_raw, bn, cn, lam, theta, a_vals, z_in


@pytest.mark.parametrize("T", [200, 64])
def test_chunked_prefill_scan_matches_reference_cuda_scan(T):
    """The chunked tensor-core scan (lumi_k_ssd_prefill) over T tokens at once against the reference's sequential
    CUDA scan on the same in_proj rows, from h_init: gated outputs of every token (bf16 hi + lo summed)."""
    if not os.path.exists(REF):
        pytest.skip("oracle/_ref/libref_ssm_scan.so not built (needs the reference checkout)")
    import torch
    ref = C.CDLL(REF)
    ref.ssm_scan_fwd_gpu.argtypes = [C.c_void_p] * 13 + [C.c_int] * 6
    H, P, N, G = 64, 32, 64, 8
    B = 3
    DI, BC = H * P, G * N
    R = 2 * DI + 2 * BC + 3 * H + H * N // 2
    g = np.random.default_rng(11)
    proj = g.standard_normal((B, T, R)).astype(np.float32)
    bg = (1 + 0.1 * g.standard_normal(BC)).astype(np.float32)
    cg = (1 + 0.1 * g.standard_normal(BC)).astype(np.float32)
    bb = (1 + 0.1 * g.standard_normal(BC)).astype(np.float32)
    cb = (1 + 0.1 * g.standard_normal(BC)).astype(np.float32)
    dsk = (1 + 0.1 * g.standard_normal(H)).astype(np.float32)
    dtb = g.uniform(-4, -1, H).astype(np.float32)
    h_init = (0.01 * g.standard_normal((H, N))).astype(np.float32)
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    f = lambda a: dev(a.astype(np.float32))

    h = dev(np.broadcast_to(h_init[None, :, None, :], (B, H, P, N)).copy())
    xp, bp, cum = dev(np.zeros((B, H, P), np.float32)), dev(np.zeros((B, H, N), np.float32)), dev(np.zeros((B, H, N // 2), np.float32))
    params = [dev(a) for a in (bg, cg, bb, cb, dsk, dtb)]
    projd = dev(proj.reshape(B * T, R))
    yhi = torch.zeros((B * T, DI), dtype=torch.bfloat16, device="cuda")
    ylo = torch.zeros_like(yhi)
    scratch = torch.zeros(2 * B * T, dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    lumi_b200.api.check(lumi_b200.lib().lumi_k_ssd_prefill(
        projd.data_ptr(), R, *[p.data_ptr() for p in params], h.data_ptr(), xp.data_ptr(), bp.data_ptr(), cum.data_ptr(),
        yhi.data_ptr(), ylo.data_ptr(), scratch.data_ptr(), B, T, H, G, 0))
    torch.cuda.synchronize()
    got = (yhi.float() + ylo.float()).cpu().numpy().reshape(B, T, DI)

    x_in, dt_raw, bn, cn, lam, theta, a_vals, z_in = _prepare_reference_inputs(proj, H, P, N, G, bg, cg, bb, cb)
    d_x, d_dt, d_b, d_c = f(x_in), f(dt_raw), f(bn), f(cn)
    d_D, d_dtb, d_hi, d_lam, d_th, d_A, d_z = f(dsk), f(dtb), f(h_init), f(lam), f(theta), f(a_vals), f(z_in)
    d_y = torch.zeros((B, T, DI), dtype=torch.float32, device="cuda")
    d_yg = torch.zeros_like(d_y)
    torch.cuda.synchronize()
    ref.ssm_scan_fwd_gpu(*[t.data_ptr() for t in (d_x, d_dt, d_b, d_c, d_D, d_dtb, d_hi, d_lam, d_th, d_A, d_z, d_y, d_yg)],
                         B, T, H, P, N, G)
    torch.cuda.synchronize()
    want = d_yg.cpu().numpy()
    err = np.abs(got - want).max() / np.abs(want).max()
    print(f"chunked prefill scan vs reference CUDA scan over {T} tokens: max rel err {err:.3e}")
    assert err < 2e-3
