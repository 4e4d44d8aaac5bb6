"""GPU: failures injected on the host (never on the device) come back as status codes and leave
the handles usable."""
import numpy as np
import pytest

import lumi_b200
from lumi_b200 import synth
from tests.helpers import load_golden

pytestmark = pytest.mark.gpu


def test_missing_tensor_and_wrong_shape():
    cfg = synth.tiny_config(n_layers=1)
    tens = list(synth.iter_tensors(cfg, seed=1))
    with pytest.raises(lumi_b200.LumiError) as e:
        lumi_b200.NmModel.from_tensors(cfg, [t for t in tens if "out_proj" not in t[0]])
    assert e.value.code == -3 and "out_proj.weight" in e.value.message
    bad = [(n, dt, a[:-1] if n.endswith("in_proj.weight") else a) for n, dt, a in tens]
    with pytest.raises(lumi_b200.LumiError) as e:
        lumi_b200.NmModel.from_tensors(cfg, bad)
    assert e.value.code == -3 and "expected [" in e.value.message


def test_optional_tensors_default():
    # b_bias / c_bias default to ones, h_init to zeros (inference/src/model.rs:209-214)
    cfg = synth.tiny_config(n_layers=1)
    tens = list(synth.iter_tensors(cfg, seed=1))
    full = lumi_b200.NmModel.from_tensors(cfg, tens)
    part = lumi_b200.NmModel.from_tensors(cfg, [t for t in tens if not t[0].endswith(("b_bias", "c_bias"))])
    prompt = synth.random_prompts(1, 6, cfg.vocab_size, seed=0)
    a = full.init_states(1).prefill(prompt)
    b = part.init_states(1).prefill(prompt)
    assert np.array_equal(a, b)
    noh = lumi_b200.NmModel.from_tensors(cfg, [t for t in tens if not t[0].endswith("h_init")])
    h, _, _, _ = noh.init_states(1).read_state(0, 0)
    assert not h.any()
    flat = [(n, dt, a.reshape(-1) if n.endswith("h_init") else a) for n, dt, a in tens]     # 1-D h_init accepted
    h2, _, _, _ = lumi_b200.NmModel.from_tensors(cfg, flat).init_states(1).read_state(0, 0)
    want = dict((n, a) for n, _, a in tens)["item.blocks.0.ssm.h_init"]
    assert np.array_equal(h2[:, 0, :], want) and np.array_equal(h2[:, 5, :], want)


def test_corrupt_safetensors(tmp_path):
    cfg = synth.tiny_config(n_layers=1)
    cpath, mpath = synth.write_model_dir(str(tmp_path), cfg, seed=1)
    ok = lumi_b200.NmModel.load(mpath, cpath)
    assert ok.info()["n_mamba"] == 1
    raw = open(mpath, "rb").read()
    trunc = tmp_path / "trunc.safetensors"
    trunc.write_bytes(raw[: len(raw) // 2])
    with pytest.raises(lumi_b200.LumiError) as e:
        lumi_b200.NmModel.load(str(trunc), cpath)
    assert e.value.code == -4
    garbage = tmp_path / "garbage.safetensors"
    garbage.write_bytes((1 << 40).to_bytes(8, "little") + b"{}")
    with pytest.raises(lumi_b200.LumiError) as e:
        lumi_b200.NmModel.load(str(garbage), cpath)
    assert e.value.code == -4
    with pytest.raises(lumi_b200.LumiError) as e:
        lumi_b200.NmModel.load(str(tmp_path / "nope.safetensors"), cpath)
    assert e.value.code == -4


def test_bad_token_and_batch_and_kv_capacity():
    z, cfg, tens = load_golden("tiny_hybrid")
    model = lumi_b200.NmModel.from_tensors(cfg, tens)
    sess = model.init_states(2, 8)
    with pytest.raises(lumi_b200.LumiError) as e:
        sess.forward_step([cfg.vocab_size + 5, 3])
    assert e.value.code == -8
    with pytest.raises(lumi_b200.LumiError) as e:
        sess.forward_step([1, 2, 3])
    assert e.value.code == -1
    sess.reset()
    with pytest.raises(lumi_b200.LumiError) as e:
        sess.prefill(np.full((1, 12), 5, dtype=np.uint32))          # 12 tokens into an 8-token cache
    assert e.value.code == -9
    sess.reset()                                                    # the session stays usable
    logits = sess.prefill(np.full((1, 4), 5, dtype=np.uint32))
    assert np.isfinite(logits).all()


def test_score_and_snapshot_argument_errors():
    """Bad arguments to the scoring and snapshot calls come back as status codes, never as aborts."""
    import ctypes as C
    cfg = synth.tiny_config(n_layers=2)
    model = lumi_b200.NmModel.from_tensors(cfg, list(synth.iter_tensors(cfg, seed=1)))
    sess = model.init_states(2, 32)
    with pytest.raises(lumi_b200.LumiError):
        sess.score(np.array([[5], [6]], dtype=np.uint32))                 # a window of one token has nothing to score
    with pytest.raises(lumi_b200.LumiError):
        sess.score(np.array([[5, cfg.vocab_size + 7, 3]], dtype=np.uint32))   # token id out of range
    with pytest.raises(lumi_b200.LumiError):
        sess.save_state(2)                                                # slot out of range
    snap = sess.save_state(1)
    with pytest.raises(lumi_b200.LumiError):
        sess.load_state(0, snap[: len(snap) // 2])                        # truncated
    bad = snap.copy()
    bad[0] ^= 0xFF
    with pytest.raises(lumi_b200.LumiError):
        sess.load_state(0, bad)                                           # not a snapshot
    sess.load_state(0, snap)                                              # the intact one still loads
    n = C.c_int64()
    assert lumi_b200.lib().lumi_session_state_bytes(sess._h, C.byref(n)) == 0 and n.value == len(snap)


def test_bounded_device_wait_runs_out_and_the_library_recovers():
    """A device-side wait that can never be satisfied: the producer warp of the persistent tensor-core GEMM is told
    to stop before one output tile, every wait is limited to 2 ms, and the consumers' waits run out.  The kernel must
    return by itself (no trap, no unbounded spin), report STATUS_TIMEOUT -> LUMI_E_TIMEOUT, free its tensor memory,
    and the same GEMM must work right afterwards."""
    import torch
    L = lumi_b200.lib()
    M, N, K = 256, 512, 256
    g = torch.Generator(device="cuda").manual_seed(1)
    a = torch.randn((M, K), generator=g, device="cuda").to(torch.bfloat16).contiguous()
    w = torch.randn((N, K), generator=g, device="cuda").to(torch.bfloat16).contiguous()
    d = torch.zeros((M, N), dtype=torch.float32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    rc = L.lumi_debug_gemm_wait_timeout(a.data_ptr(), w.data_ptr(), d.data_ptr(), M, N, K, 2_000_000, 1, status.data_ptr())
    assert rc == -7, L.lumi_last_error().decode()                  # LUMI_E_TIMEOUT
    assert "wait expired" in L.lumi_last_error().decode()
    assert int(status.item()) & 4                                  # STATUS_TIMEOUT
    # nothing was skipped: the same entry point, then the ordinary one, give the product
    status.zero_()
    torch.cuda.synchronize()
    rc = L.lumi_debug_gemm_wait_timeout(a.data_ptr(), w.data_ptr(), d.data_ptr(), M, N, K, 2_000_000, -1, status.data_ptr())
    assert rc == 0, L.lumi_last_error().decode()
    ref = a.float() @ w.float().t()
    assert float((d - ref).abs().max() / ref.abs().max()) < 1e-5
    d.zero_()
    lumi_b200.api.check(L.lumi_k_gemm_bf16_tcgen05(a.data_ptr(), 0, w.data_ptr(), d.data_ptr(), M, N, K, N, 0, 0))
    torch.cuda.synchronize()
    assert float((d - ref).abs().max() / ref.abs().max()) < 1e-5
