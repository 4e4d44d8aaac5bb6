"""GPU: single kernels through the C ABI against plain references (numpy fp64 / torch fp32)."""
import numpy as np
import pytest

import lumi_b200
from lumi_b200 import synth

pytestmark = pytest.mark.gpu


def _torch():
    import torch
    return torch


@pytest.mark.parametrize("wdt", ["f32", "bf16"])
@pytest.mark.parametrize("M,N,K", [(1, 7360, 1024), (3, 1000, 2048), (8, 259, 1024), (20, 512, 128),
                                   (1, 1024, 2048), (2, 7360, 1024), (4, 3000, 512), (1, 100, 128), (1, 9000, 1024), (2, 2960, 4096)])
def test_gemv_matches_fp64(wdt, M, N, K):
    torch = _torch()
    g = np.random.default_rng(M * 1000 + N)
    a = g.standard_normal((M, K)).astype(np.float32)
    w = (g.standard_normal((N, K)) * 0.05).astype(np.float32)
    gamma = (1 + 0.1 * g.standard_normal(K)).astype(np.float32)
    res = g.standard_normal((M, N)).astype(np.float32)
    if wdt == "bf16":
        wbits = synth.f32_to_bf16_bits(w)
        w = synth.bf16_bits_to_f32(wbits)
        wd = torch.from_numpy(wbits.view(np.int16)).cuda()
    else:
        wd = torch.from_numpy(w).cuda()
    ad, gd, rd = torch.from_numpy(a).cuda(), torch.from_numpy(gamma).cuda(), torch.from_numpy(res).cuda()
    out = torch.empty((M, N), dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    lumi_b200.api.check(lumi_b200.lib().lumi_k_gemv(ad.data_ptr(), wd.data_ptr(), 1 if wdt == "bf16" else 0, out.data_ptr(),
                                                rd.data_ptr(), gd.data_ptr(), M, N, K, 0))
    torch.cuda.synchronize()
    a64 = a.astype(np.float64)
    xn = a64 / np.sqrt((a64 ** 2).mean(axis=1, keepdims=True) + 1e-5) * gamma
    ref = xn @ w.astype(np.float64).T + res
    got = out.cpu().numpy()
    assert np.abs(got - ref).max() / np.abs(ref).max() < 2e-6
    # run-to-run bit stability (fixed summation order)
    out2 = torch.empty_like(out)
    lumi_b200.api.check(lumi_b200.lib().lumi_k_gemv(ad.data_ptr(), wd.data_ptr(), 1 if wdt == "bf16" else 0, out2.data_ptr(),
                                                rd.data_ptr(), gd.data_ptr(), M, N, K, 0))
    torch.cuda.synchronize()
    assert torch.equal(out, out2)


@pytest.mark.parametrize("split", [True, False])
@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (64, 7360, 1024), (200, 259, 1024), (300, 1024, 2048), (2048, 512, 128),
                                   (2048, 7360, 1024), (1000, 5000, 512), (2300, 4100, 64),    # more tiles than SMs: persistent CTAs
                                   (64, 1024, 2048), (512, 1024, 2048), (100, 1024, 2816), (300, 512, 4096),    # few tiles: K split over CTAs
                                   (64, 1000, 2048), (128, 264, 4096), (17, 36, 1024)])                    # ... with ragged last tiles
def test_tcgen05_gemm_matches_torch(split, M, N, K):
    torch = _torch()
    g = torch.Generator(device="cpu").manual_seed(M + N + K)
    a = torch.randn((M, K), generator=g, dtype=torch.float32)
    w = (torch.randn((N, K), generator=g, dtype=torch.float32) * 0.05).to(torch.bfloat16)
    hi = a.to(torch.bfloat16)
    lo = (a - hi.float()).to(torch.bfloat16)
    prev = torch.randn((M, N), generator=g, dtype=torch.float32)
    a_eff = (hi.double() + lo.double()) if split else hi.double()
    ref = a_eff @ w.double().T
    hid, lod, wd = hi.cuda(), lo.cuda(), w.cuda()
    for acc in (0, 1):
        d = prev.clone().cuda()
        torch.cuda.synchronize()
        lumi_b200.api.check(lumi_b200.lib().lumi_k_gemm_bf16_tcgen05(hid.data_ptr(), lod.data_ptr() if split else 0, wd.data_ptr(),
                                                                 d.data_ptr(), M, N, K, N, acc, 0))
        torch.cuda.synchronize()
        want = ref + (prev.double() if acc else 0)
        err = (d.cpu().double() - want).abs().max().item() / want.abs().max().item()
        # tensor-core fp32 accumulation is not round-to-nearest at every add: allow 2e-5 of the largest output
        assert err < 2e-5, (M, N, K, split, acc, err)
        # the same call again gives the same bits (K split over CTAs adds its partial tiles in a fixed order)
        d2 = prev.clone().cuda()
        lumi_b200.api.check(lumi_b200.lib().lumi_k_gemm_bf16_tcgen05(hid.data_ptr(), lod.data_ptr() if split else 0, wd.data_ptr(),
                                                                 d2.data_ptr(), M, N, K, N, acc, 0))
        torch.cuda.synchronize()
        assert torch.equal(d, d2)


def test_tcgen05_gemm_rejects_bad_k():
    torch = _torch()
    a = torch.zeros((8, 100), dtype=torch.bfloat16, device="cuda")
    w = torch.zeros((8, 100), dtype=torch.bfloat16, device="cuda")
    d = torch.zeros((8, 8), dtype=torch.float32, device="cuda")
    st = lumi_b200.lib().lumi_k_gemm_bf16_tcgen05(a.data_ptr(), 0, w.data_ptr(), d.data_ptr(), 8, 8, 100, 8, 0, 0)
    assert st == -10


def test_tcgen05_gemm_without_k_split_in_child_process():
    """K is split over CTAs by default where the tiles alone leave SMs idle (the few-tile shapes of the test above).
    LUMI_GEMM_SPLITK=1 turns that off and is latched at first use: run those shapes unsplit in a child process, and
    check run-to-run bit stability there too."""
    import os, subprocess, sys
    code = (
        "import torch, lumi_b200\n"
        "L = lumi_b200.lib()\n"
        "for (M, N, K) in [(64, 1024, 2048), (512, 1024, 2048), (100, 1024, 2816)]:\n"
        "    g = torch.Generator().manual_seed(M + N + K)\n"
        "    a = torch.randn((M, K), generator=g); w = (torch.randn((N, K), generator=g) * 0.05).to(torch.bfloat16)\n"
        "    hi = a.to(torch.bfloat16); lo = (a - hi.float()).to(torch.bfloat16); prev = torch.randn((M, N), generator=g)\n"
        "    ref = (hi.double() + lo.double()) @ w.double().T + prev.double()\n"
        "    outs = []\n"
        "    for rep in range(2):\n"
        "        d = prev.clone().cuda(); hid, lod, wd = hi.cuda(), lo.cuda(), w.cuda(); torch.cuda.synchronize()\n"
        "        assert L.lumi_k_gemm_bf16_tcgen05(hid.data_ptr(), lod.data_ptr(), wd.data_ptr(), d.data_ptr(), M, N, K, N, 1, 0) == 0\n"
        "        torch.cuda.synchronize(); outs.append(d.cpu())\n"
        "    err = (outs[0].double() - ref).abs().max().item() / ref.abs().max().item()\n"
        "    assert err < 2e-5, (M, N, K, err)\n"
        "    assert torch.equal(outs[0], outs[1])\n"
        "print('ok')\n")
    env = dict(os.environ, LUMI_GEMM_SPLITK="1", PYTHONPATH=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    out = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0 and "ok" in out.stdout, out.stderr[-2000:]
