#!/usr/bin/env python
"""Decode throughput of the lumi token loop on B200, against the HBM roofline.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Workload (the benchmark definition's throughput sweep): the 96-layer Mamba-3 LM in byte-level
mode (vocab 259), bf16 weights, fp32 state; 4096 independent sequences sharded contiguously over
the N ranks with no collective; seeded uniform-random prompts prefilled (untimed) by the batched path
(chunked SSD scan); then greedy decode.  One "step" is one decode step of every resident sequence.
Per-rank state for more than `--capacity` sequences does not fit one GPU (fp32 state is
53.5 MB per sequence), so a rank runs its shard in waves; a step of the job is then one step of
each wave and the times add.

Prints ONE JSON line on rank 0.  `value` times the steps with tokens resident on the device
(CUDA events on the session stream); `e2e` times the same steps through lumi_decode_step with
host token buffers copied in and out every step.  `--impl reference` times the CPU restatement of
the reference's own CPU path on the host cores instead.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from lumi_b200 import shard, synth  # noqa: E402

METRIC = "decode_tokens_per_second"
UNIT = "tok/s"


def measured_peak_gbs():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json, stream copy)"
    except Exception:
        return 6650.0, "fallback (6.65 TB/s, earlier measurement on this pool)"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons, sampled while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx = gpu_index
        self.lines = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.idx), f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is not None:
            self.proc.terminate()          # the exact process started above
            try:
                self.proc.wait(timeout=5)
            except Exception:
                pass
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def workload_config(args) -> synth.ModelConfig:
    return synth.base_config(n_layers=args.layers, byte_level=True, max_seq_len=4096)


def state_bytes_per_seq_step(cfg) -> int:
    """Read + write of h, the rank-1 factors of prev_bx and cum_angle, per Mamba layer."""
    per = cfg.n_heads * cfg.head_dim * cfg.d_state + cfg.d_inner + cfg.n_heads * cfg.d_state + cfg.n_heads * cfg.d_state // 2
    return 2 * 4 * per


# --------------------------------------------------------------------------------------------------
def run_reference(args, rank, world):
    """The reference arm: the CPU restatement of lumi-infer's CPU path (the Rust/Candle binary cannot
    be built on this image) on the host cores, all OpenMP threads.  A step = one decode token for each
    of `--ref-seqs` sequences, run one after another (the reference has no batching)."""
    if rank != 0:
        return
    from oracle import cpu_oracle
    cores = cpu_oracle.set_threads(os.cpu_count() or 1)          # torchrun exports OMP_NUM_THREADS=1
    cfg = workload_config(args)
    tens = list(synth.iter_tensors(cfg, seed=0, weights_dtype="bf16"))
    om = cpu_oracle.OracleModel(cfg, tens)
    del tens
    nseq = args.ref_seqs
    prompts = synth.random_prompts(nseq, 4, cfg.vocab_size, seed=0)
    states, toks = [], []
    for b in range(nseq):
        st = om.init_states()
        for t in prompts[b]:
            lg = st.forward_step(int(t))
        states.append(st)
        toks.append(cpu_oracle.argmax(lg))

    def step():
        for b in range(nseq):
            toks[b] = cpu_oracle.argmax(states[b].forward_step(toks[b]))
    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = time.perf_counter() - t0
    value = nseq * args.steps / dt
    sample = f"{nseq} sequence(s) x {args.steps} decode tokens of the same 96-layer model, after a 4-token prompt"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD_NAME(args), "reference": "CPU restatement (oracle/lumi_oracle.cpp) of inference/src/model.rs CPU branch; "
                   "the Rust/Candle reference cannot be built here (no cargo/rustc, crates not vendored)"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }), flush=True)


def WORKLOAD_NAME(args):
    return (f"throughput sweep: {args.layers}-layer Mamba-3 LM, byte-level vocab 259, bf16 weights, fp32 state; "
            f"{args.sequences} sequences x {args.prompt_len}-token uniform-random prompts, greedy decode")


def cpu_baseline(args, cfg):
    """Rank 0, N = 1: the oracle timed on the host cores on a bounded sample of the same workload."""
    from oracle import cpu_oracle
    cores = cpu_oracle.set_threads(os.cpu_count() or 1)
    tens = list(synth.iter_tensors(cfg, seed=0, weights_dtype="bf16"))
    om = cpu_oracle.OracleModel(cfg, tens)
    del tens
    st = om.init_states()
    prompt = synth.random_prompts(1, 4, cfg.vocab_size, seed=0)[0]
    for t in prompt:
        lg = st.forward_step(int(t))
    tok = cpu_oracle.argmax(lg)
    n = args.cpu_tokens
    t0 = time.perf_counter()
    for _ in range(n):
        tok = cpu_oracle.argmax(st.forward_step(tok))
    dt = time.perf_counter() - t0
    return {"value": n / dt, "unit": UNIT, "cores": cores, "kind": "port",
            "sample": f"1 sequence x {n} decode tokens of the same {cfg.n_layers}-layer model after a 4-token prompt "
                      f"(the reference runs sequences one at a time: per-sequence tok/s)"}


def batch1_line(args, peak_gbs):
    """Secondary figure: the base 48-layer fp32 model at batch 1 (weights-bound decode)."""
    import lumi_b200
    cfg = synth.base_config(n_layers=args.b1_layers)
    model = lumi_b200.NmModel.from_tensors(cfg, synth.iter_tensors(cfg, seed=0))
    sess = model.init_states(1)
    prompt = synth.random_prompts(1, 32, cfg.vocab_size, seed=0)
    sess.prefill(prompt, want_logits=True)
    sess.decode_loop_device(1, 8)
    best = None
    for _ in range(3):
        ms, _ = sess.decode_loop_device(1, 64)
        best = ms if best is None else min(best, ms)
    per_step = model.info()["weight_bytes"] + model.info()["n_mamba"] * state_bytes_per_seq_step(cfg)
    toks = 64 / (best * 1e-3)
    ach = per_step * toks / 1e9
    sess.close(); model.close()
    return {"workload": f"base {cfg.n_layers}-layer Mamba-3 LM, fp32 weights, batch 1, 32-token prompt, greedy decode (64 timed steps, best of 3)",
            "value": toks, "unit": UNIT, "bytes_per_step": per_step, "achieved_gbs": ach, "peak_gbs": peak_gbs, "frac": ach / peak_gbs}


# name: (config kwargs, weights dtype, batch, prompt length, decode tokens, sampling, prompt seed)
CONFIGS = {k: v for k, v in synth.BENCH_CONFIGS.items() if k != "config5"}      # config 5 is the default sweep


def scan_compare(nb=64, T=2048, reps=3):
    """The chunked prefill scan of this library (lumi_k_ssd_prefill) and the reference's own sequential CUDA scan
    (training/csrc/ssm_scan.cu, built into oracle/_ref/ from the reference's sources) on the same random in_proj
    rows: nb sequences x T tokens at the base dimensions, CUDA events, best of `reps`.  Returns microseconds per
    (sequence, head, 64-token chunk) for both and their ratio; the reference entry is None when its library was
    not built (no reference checkout at build time)."""
    import ctypes as C
    import torch
    import lumi_b200
    H, P, N, G = 64, 32, 64, 8
    DI, BC = H * P, G * N
    R = 2 * DI + 2 * BC + 3 * H + H * N // 2
    gen = torch.Generator(device="cuda").manual_seed(0)
    proj = torch.randn((nb * T, R), generator=gen, device="cuda", dtype=torch.float32)
    one = lambda n: 1 + 0.1 * torch.randn(n, generator=gen, device="cuda")
    bg, cg, bb, cb, dsk = one(BC), one(BC), one(BC), one(BC), one(H)
    dtb = -4 + 3 * torch.rand(H, generator=gen, device="cuda")
    h_init = 0.01 * torch.randn((H, N), generator=gen, device="cuda")
    units = nb * H * ((T + 63) // 64)

    def fresh_state():
        return (h_init[None, :, None, :].expand(nb, H, P, N).contiguous(), torch.zeros((nb, H, P), device="cuda"),
                torch.zeros((nb, H, N), device="cuda"), torch.zeros((nb, H, N // 2), device="cuda"))
    yhi = torch.empty((nb * T, DI), dtype=torch.bfloat16, device="cuda")
    ylo = torch.empty_like(yhi)
    scratch = torch.empty(2 * nb * T, dtype=torch.float32, device="cuda")
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ours = None
    for _ in range(reps + 1):
        h, xp, bp, cum = fresh_state()
        torch.cuda.synchronize()
        ev0.record()
        lumi_b200.api.check(lumi_b200.lib().lumi_k_ssd_prefill(
            proj.data_ptr(), R, bg.data_ptr(), cg.data_ptr(), bb.data_ptr(), cb.data_ptr(), dsk.data_ptr(), dtb.data_ptr(),
            h.data_ptr(), xp.data_ptr(), bp.data_ptr(), cum.data_ptr(), yhi.data_ptr(), ylo.data_ptr(), scratch.data_ptr(),
            nb, T, H, G, torch.cuda.current_stream().cuda_stream))
        ev1.record()
        torch.cuda.synchronize()
        ms = ev0.elapsed_time(ev1)
        ours = ms if ours is None else min(ours, ms)
    out = {"sequences": nb, "tokens": T, "units": units, "ours_ms": ours, "ours_us_per_unit": ours * 1e3 / units}
    ref_path = os.path.join(ROOT, "oracle", "_ref", "libref_ssm_scan.so")
    if not os.path.exists(ref_path):
        out["reference_us_per_unit"] = None
        return out
    ref = C.CDLL(ref_path)
    ref.ssm_scan_fwd_gpu.argtypes = [C.c_void_p] * 13 + [C.c_int] * 6
    # the reference kernel's inputs, prepared as its trainer does before the scan (native_trainer.rs:222-259); untimed
    pr = proj.view(nb, T, R)
    x_in = torch.nn.functional.silu(pr[..., :DI]).contiguous()
    z_in = pr[..., DI:2 * DI].contiguous()
    bproj, cproj = pr[..., 2 * DI:2 * DI + BC], pr[..., 2 * DI + BC:2 * DI + 2 * BC]
    bn = (bproj * torch.rsqrt((bproj ** 2).mean(-1, keepdim=True) + 1e-5) * bg + bb).contiguous()
    cn = (cproj * torch.rsqrt((cproj ** 2).mean(-1, keepdim=True) + 1e-5) * cg + cb).contiguous()
    o = 2 * DI + 2 * BC
    dt_raw = pr[..., o:o + H].contiguous()
    lam = torch.sigmoid(pr[..., o + H:o + 2 * H]).contiguous()
    a_vals = torch.clamp(-torch.nn.functional.softplus(pr[..., o + 2 * H:o + 3 * H]), -1e6, -1e-4).contiguous()
    theta = pr[..., o + 3 * H:].contiguous()
    y = torch.empty((nb, T, DI), device="cuda")
    yg = torch.empty_like(y)
    theirs = None
    for _ in range(2):
        torch.cuda.synchronize()
        ev0.record()
        ref.ssm_scan_fwd_gpu(x_in.data_ptr(), dt_raw.data_ptr(), bn.data_ptr(), cn.data_ptr(), dsk.data_ptr(), dtb.data_ptr(),
                             h_init.data_ptr(), lam.data_ptr(), theta.data_ptr(), a_vals.data_ptr(), z_in.data_ptr(), y.data_ptr(),
                             yg.data_ptr(), nb, T, H, P, N, G)       # launches on the legacy default stream, as the reference does
        ev1.record()
        torch.cuda.synchronize()
        ms = ev0.elapsed_time(ev1)
        theirs = ms if theirs is None else min(theirs, ms)
    # agreement of the two kernels on the first 256 tokens (tests/test_gpu_reference_scan.py holds the bound; over thousands
    # of tokens of unit-variance random rows the reference's sin/cos.approx angles drift away from any exact evaluation)
    n_cmp = min(T, 256)
    got = (yhi.float() + ylo.float()).view(nb, T, DI)[:, :n_cmp]
    out.update({"reference_ms": theirs, "reference_us_per_unit": theirs * 1e3 / units, "speedup": theirs / ours,
                "max_rel_diff_first_256_tokens": float((got - yg[:, :n_cmp]).abs().max() / yg[:, :n_cmp].abs().max())})
    return out


def run_named_config(args, rank, local_rank, world):
    """The other benchmark configurations, one GPU, through Session.generate (prefill + decode timed
    by CUDA events inside the library).  Sequences would shard over ranks exactly as in the sweep."""
    if rank != 0:
        return
    import lumi_b200
    kw, wdt, batch, T, n_new, samp, pseed = CONFIGS[args.workload]
    if args.steps_override:
        n_new = args.steps_override
    cfg = synth.base_config(max_seq_len=4096, **kw)
    peak_gbs, peak_src = measured_peak_gbs()
    model = lumi_b200.NmModel.from_tensors(cfg, synth.iter_tensors(cfg, seed=0, weights_dtype=wdt), device=local_rank)
    info = model.info()
    sess = model.init_states(batch, T + n_new + 1)
    prompts = synth.random_prompts(batch, T, cfg.vocab_size, seed=pseed)
    sess.generate(prompts[:, :min(T, 128)], 4, ignore_eos=True, **samp)        # warm-up (graphs, attributes)
    sess.reset()
    sampler = ClockSampler(local_rank)
    sampler.start()
    t0 = time.perf_counter()
    toks, lens, _, st = sess.generate(prompts, n_new + 1, ignore_eos=True, **samp)
    wall = time.perf_counter() - t0
    clocks = sampler.stop()
    sess.close(); model.close()
    scan = None
    if args.workload == "config3":           # the chunked scan alone, beside the reference's sequential CUDA scan
        import torch
        torch.cuda.set_device(local_rank)
        scan = scan_compare()
    S = state_bytes_per_seq_step(cfg)
    kv = 0
    if info["n_attention"]:
        t_mean = T + n_new / 2.0
        kv = int(info["n_attention"] * (2 * t_mean * cfg.attn_kv_dim * 2 + 2 * cfg.attn_kv_dim * 2))
    step_bytes = info["weight_bytes"] + batch * (info["n_mamba"] * S + kv)
    dec_tps = st.decode_tokens / (st.ms_decode * 1e-3)
    gbs = step_bytes * (st.decode_tokens / batch) / (st.ms_decode * 1e-3) / 1e9
    print(json.dumps({
        "metric": METRIC, "value": dec_tps, "unit": UNIT, "n_gpus": 1, "steps": int(st.decode_tokens // batch), "warmup": 4,
        "ms_per_step": st.ms_decode / (st.decode_tokens / batch), "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"{args.workload}: {cfg.n_layers} layers ({info['n_attention']} attention), {wdt} weights, batch {batch}, "
                               f"{T}-token prompts, {n_new} decode tokens, sampling {samp or 'greedy'}"},
        "gpu_launches": int(st.kernel_launches),
        "prefill": {"tokens_per_second": st.prompt_tokens / (st.ms_prefill * 1e-3), "ms": st.ms_prefill},
        "e2e": {"value": (st.decode_tokens + batch) / wall, "unit": UNIT, "note": "whole generate call incl. prefill, wall clock",
                "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "roofline": {"bound": "hbm", "kernel": "whole decode step", "achieved": gbs, "peak": peak_gbs, "unit": "GB/s", "frac": gbs / peak_gbs,
                     "traffic": None, "peak_source": peak_src, "bytes_per_step": step_bytes},
        "clocks": clocks,
        "prefill_scan": scan if scan is not None else None,
    }), flush=True)


def run_ours(args, rank, local_rank, world):
    import torch
    import torch.distributed as dist
    import lumi_b200

    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    dev = torch.device("cuda", local_rank)
    cfg = workload_config(args)
    peak_gbs, peak_src = measured_peak_gbs()

    lo, hi = shard.shard_range(args.sequences, rank, world)
    my_waves = shard.waves(hi - lo, args.capacity)
    cap = max(b - a for a, b in my_waves)
    model = lumi_b200.NmModel.from_tensors(cfg, synth.iter_tensors(cfg, seed=0, weights_dtype="bf16"), device=local_rank)
    info = model.info()
    sess = model.init_states(cap)
    sess.set_option("split_activations", args.split)
    prompts = synth.random_prompts(hi - lo, args.prompt_len, cfg.vocab_size, seed=1000 + lo) if hi > lo else None

    S = state_bytes_per_seq_step(cfg)
    t_dev_ms, t_e2e_ms, launches = 0.0, 0.0, 0
    fam_ms, fam_n, ssm_batch = {}, {}, 0
    single_ms, single_nb = None, 0
    sampler = ClockSampler(local_rank)
    h2d = d2h = 0
    for wi, (a, b) in enumerate(my_waves):
        nb = b - a
        sess.reset()
        sess.prefill(prompts[a:b], want_logits=True)                 # untimed: prompt, then first token
        sess.decode_loop_device(nb, max(args.warmup, 3))              # warm-up steps (>= 3)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        if wi == 0:
            sampler.start()
        ms, n = sess.decode_loop_device(nb, args.steps)               # timed: EXACTLY K steps, CUDA events
        torch.cuda.synchronize()
        t_dev_ms += ms
        launches += n
        # end to end through the C ABI with host buffers: tokens in and out every step
        toks = np.full(nb, 5, dtype=np.uint32)
        _, toks = sess.forward_step(toks, want_logits=False)
        if world > 1:
            dist.barrier()
        t0 = time.perf_counter()
        for i in range(args.steps):
            _, toks = sess.forward_step(toks, want_logits=False, step=i)
        t_e2e_ms += (time.perf_counter() - t0) * 1e3
        h2d += nb * 4 + 80
        d2h += nb * 4 + 80
        # secondary figure: activations rounded to bf16 once instead of the hi + lo split (half the MMAs)
        if wi == len(my_waves) - 1 and args.split:
            sess.set_option("split_activations", 0)
            sess.decode_loop_device(nb, 3)
            ms1, _ = sess.decode_loop_device(nb, args.steps)
            single_ms = ms1 / args.steps
            single_nb = nb
            sess.set_option("split_activations", 1)
        # live per-kernel times (an event in front of every launch), second of two profiled steps
        sess.profile_step(nb)
        prof = sess.profile_step(nb)
        if nb >= ssm_batch:
            ssm_batch = nb
            fam_ms = {k: v[0] for k, v in prof.items()}
            fam_n = {k: v[1] for k, v in prof.items()}
    clocks = sampler.stop()

    units = float((hi - lo) * args.steps)
    if world > 1:
        dist.barrier()
        tmax, total_units = shard.reduce_max_sum(dist, t_dev_ms, units, device=dev)
        emax, _ = shard.reduce_max_sum(dist, t_e2e_ms, 0.0, device=dev)
        lsum = shard.reduce_max_sum(dist, 0.0, float(launches), device=dev)[1]
    else:
        tmax, total_units, emax, lsum = t_dev_ms, units, t_e2e_ms, float(launches)

    if rank == 0:
        value = total_units / (tmax * 1e-3)
        e2e = total_units / (emax * 1e-3)
        # whole-step roofline on this rank: algorithmic bytes of its waves' steps over its device time
        step_bytes = sum(info["weight_bytes"] + (b - a) * info["n_mamba"] * S for a, b in my_waves)
        step_gbs = step_bytes * args.steps / (t_dev_ms * 1e-3) / 1e9
        # dominant kernel: the fused Mamba state step; algorithmic bytes per launch = batch * S
        ssm_launch_ms = fam_ms.get("ssm_step", 0.0) / max(1, fam_n.get("ssm_step", 1))
        ssm_bytes = ssm_batch * S
        ssm_gbs = ssm_bytes / (ssm_launch_ms * 1e-3) / 1e9 if ssm_launch_ms > 0 else 0.0
        traffic = None
        tpath = os.path.join(ROOT, "profiles", "ssm_step_traffic.json")
        if os.path.exists(tpath):
            try:
                with open(tpath) as f:
                    traffic = float(json.load(f)["dram_bytes_per_sequence_layer"]) * ssm_batch
            except Exception:
                traffic = None
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": tmax / args.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD_NAME(args), "sequences_per_gpu": hi - lo, "waves_per_gpu": len(my_waves),
                       "resident_sequences": cap, "weights": "bf16", "state": "fp32",
                       "activations_into_gemm": "bf16 hi+lo split" if args.split else "bf16",
                       "l2": "inputs larger than L2: each step streams %.1f GB of state" % (cap * info["n_mamba"] * S / 1e9),
                       "prefill": "untimed; 512-token bf16 prompts take the batched path (chunked SSD scan + tensor-core GEMMs over all prompt tokens)"},
            "gpu_launches": int(lsum),
            "e2e": {"value": e2e, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "roofline": {"bound": "hbm", "kernel": "ssm_step_kernel<32,64>", "achieved": ssm_gbs, "peak": peak_gbs, "unit": "GB/s",
                         "frac": ssm_gbs / peak_gbs, "traffic": traffic, "peak_source": peak_src,
                         "algorithmic_bytes_per_launch": ssm_bytes, "launch_ms": ssm_launch_ms,
                         "whole_step": {"bytes_per_step": step_bytes, "achieved": step_gbs, "frac": step_gbs / peak_gbs,
                                        "frac_of_8TBs_nominal": step_gbs / 8000.0}},
            "kernel_ms_per_step": fam_ms, "kernel_launches_per_step": fam_n,
            "single_rounded_activations": None if single_ms is None else {
                "note": "same step with activations rounded to bf16 once (logit tolerance 2e-2 instead of 1e-3); last wave only",
                "ms_per_wave_step": single_ms, "tok_per_s_this_wave": single_nb / (single_ms * 1e-3),
                "whole_step_frac": (info["weight_bytes"] + single_nb * info["n_mamba"] * S) / (single_ms * 1e-3) / 1e9 / peak_gbs},
            "clocks": clocks,
        }
        if world == 1 and not args.no_cpu:
            line["cpu_baseline"] = cpu_baseline(args, cfg)
        sess.close(); model.close()
        if not args.no_batch1:
            try:
                line["batch1"] = batch1_line(args, peak_gbs)
            except Exception as e:        # the secondary figure must not take the headline down
                line["batch1"] = {"error": str(e)}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=16)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--sequences", type=int, default=4096)
    ap.add_argument("--capacity", type=int, default=2048, help="resident sequences per GPU (fp32 state: 53.5 MB each at 96 layers)")
    ap.add_argument("--prompt-len", type=int, default=512)
    ap.add_argument("--layers", type=int, default=96)
    ap.add_argument("--split", type=int, default=1)
    ap.add_argument("--ref-seqs", type=int, default=1)
    ap.add_argument("--cpu-tokens", type=int, default=24)
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-batch1", action="store_true")
    ap.add_argument("--only-batch1", action="store_true", help="run just the batch-1 figure (profiling)")
    ap.add_argument("--b1-layers", type=int, default=48)
    ap.add_argument("--workload", default="sweep", choices=["sweep", "scan"] + sorted(CONFIGS))
    ap.add_argument("--scan-seqs", type=int, default=64, help="--workload scan: sequences")
    ap.add_argument("--scan-tokens", type=int, default=2048, help="--workload scan: tokens per sequence")
    ap.add_argument("--steps-override", type=int, default=0, help="decode tokens for --workload configN (0 = the configuration's own)")
    args = ap.parse_args()
    rank, local_rank, world = shard.env_rank_world()
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE {world}")
    if args.workload == "scan":       # the chunked prefill scan alone beside the reference's CUDA scan (profiling, small cases)
        if rank == 0:
            import torch
            torch.cuda.set_device(local_rank)
            print(json.dumps({"prefill_scan": scan_compare(args.scan_seqs, args.scan_tokens)}), flush=True)
    elif args.workload != "sweep":
        run_named_config(args, rank, local_rank, world)
    elif args.only_batch1:
        print(json.dumps({"batch1": batch1_line(args, measured_peak_gbs()[0])}), flush=True)
    elif args.impl == "reference":
        run_reference(args, rank, world)
    else:
        run_ours(args, rank, local_rank, world)


if __name__ == "__main__":
    main()
