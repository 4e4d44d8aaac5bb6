"""Runs the reference's OWN CUDA forward kernels (oracle/_ref/libref_fwd.so, built from
training/csrc/{elementwise_ops,cublas_ops,ssm_scan}.cu where they lie) chained exactly as the reference's
trainer chains them — `mamba_block_forward` (training/src/native_trainer.rs:198-266) and
`attention_block_forward` (:110-194) — over a window of tokens, and writes the block output.

    python tests/ref_chain.py in.npz out.npz

Test infrastructure: started as a child process by tests/test_gpu_reference_blocks.py so that
NVIDIA_TF32_OVERRIDE=0 (set by the parent) is in the environment before cuBLAS is loaded — the reference's
cublas_init asks for TF32 (training/csrc/cublas_ops.cu:65), which would cost three digits of the comparison.
Weights arrive in the inference layout [out, in] and are transposed to the trainer's [in, out]
(scripts/export_native_safetensors.py:78-82 does the opposite on export).
"""
import ctypes as C
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(os.path.dirname(HERE), "oracle", "_ref", "libref_fwd.so")


def main():
    import torch
    z = np.load(sys.argv[1])
    ref = C.CDLL(LIB)
    P, I, F = C.c_void_p, C.c_int, C.c_float
    ref.cublas_init.argtypes = []
    ref.rmsnorm_fwd.argtypes = [P, P, P, F, I, I]
    ref.rmsnorm_bias_fwd.argtypes = [P, P, P, P, F, I, I]
    ref.matmul_f32.argtypes = [P, P, P, I, I, I]
    ref.matmul_f32_batched.argtypes = [P, P, P, I, I, I, I]
    ref.matmul_f32_bt_batched.argtypes = [P, P, P, I, I, I, I]
    ref.fused_split_5.argtypes = [P] * 6 + [I] * 12
    ref.strided_split.argtypes = [P, P, I, I, I, I]
    ref.sigmoid_fwd.argtypes = [P, P, I]
    ref.silu_fwd.argtypes = [P, P, I]
    ref.neg_softplus_clamp.argtypes = [P, P, F, F, I]
    ref.elemwise_add.argtypes = [P, P, P, I]
    ref.elemwise_mul.argtypes = [P, P, P, I]
    ref.scale_tensor.argtypes = [P, P, F, I]
    ref.transpose_0213.argtypes = [P, P, I, I, I, I]
    ref.gqa_expand.argtypes = [P, P, I, I, I, I, I]
    ref.causal_softmax_fwd.argtypes = [P, P, I, I, I]
    ref.ssm_scan_fwd_gpu.argtypes = [P] * 13 + [I] * 6
    ref.cublas_init()

    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).cuda()
    buf = lambda *shape: torch.zeros(shape, dtype=torch.float32, device="cuda")
    p = lambda t: t.data_ptr()
    wt = lambda name: dev(z[name].T)                       # [out, in] -> [in, out]
    kind = str(z["kind"])
    batch, seq, D = int(z["batch"]), int(z["seq"]), int(z["d_model"])
    bs = batch * seq
    eps = float(z["eps"])
    x = dev(z["x"]).reshape(bs, D).contiguous()
    torch.cuda.synchronize()

    if kind == "mamba":
        H, Pd, N, G = int(z["n_heads"]), int(z["head_dim"]), int(z["d_state"]), int(z["n_groups"])
        DI, BC = H * Pd, G * N
        R = 2 * DI + 2 * BC + 3 * H + H * N // 2
        w_in, w_out = wt("in_proj"), wt("out_proj")
        gam, bg, cg, bb, cb = dev(z["norm_g"]), dev(z["b_gamma"]), dev(z["c_gamma"]), dev(z["b_bias"]), dev(z["c_bias"])
        dsk, dtb, hin = dev(z["d_skip"]), dev(z["dt_bias"]), dev(z["h_init"])
        residual, xn, proj = buf(bs, D), buf(bs, D), buf(bs, R)
        xs, zb, braw, craw, dtv = buf(bs, DI), buf(bs, DI), buf(bs, BC), buf(bs, BC), buf(bs, H)
        lam_raw, lam, a_raw, a_vals, theta = buf(bs, H), buf(bs, H), buf(bs, H), buf(bs, H), buf(bs, H * N // 2)
        xact, bn, cn, y, yg, out = buf(bs, DI), buf(bs, BC), buf(bs, BC), buf(bs, DI), buf(bs, DI), buf(bs, D)
        residual.copy_(x)                                                          # native_trainer.rs:212-213
        torch.cuda.synchronize()
        ref.rmsnorm_fwd(p(x), p(xn), p(gam), eps, bs, D)                           # :216
        ref.matmul_f32(p(xn), p(w_in), p(proj), bs, R, D)                          # :219
        ref.fused_split_5(p(proj), p(xs), p(zb), p(braw), p(craw), p(dtv), bs, R,  # :222-227
                          0, DI, DI, DI, 2 * DI, BC, 2 * DI + BC, BC, 2 * DI + 2 * BC, H)
        lo = 2 * DI + 2 * BC + H
        ref.strided_split(p(proj), p(lam_raw), bs, R, lo, H)                       # :230-232
        ref.sigmoid_fwd(p(lam_raw), p(lam), bs * H)
        ref.strided_split(p(proj), p(a_raw), bs, R, lo + H, H)                     # :235-237
        ref.neg_softplus_clamp(p(a_raw), p(a_vals), -1e6, -1e-4, bs * H)
        ref.strided_split(p(proj), p(theta), bs, R, lo + 2 * H, H * N // 2)        # :240-242
        ref.silu_fwd(p(xs), p(xact), bs * DI)                                      # :245
        ref.rmsnorm_bias_fwd(p(braw), p(bn), p(bg), p(bb), eps, bs, BC)            # :248-249
        ref.rmsnorm_bias_fwd(p(craw), p(cn), p(cg), p(cb), eps, bs, BC)
        ref.ssm_scan_fwd_gpu(p(xact), p(dtv), p(bn), p(cn), p(dsk), p(dtb), p(hin), p(lam), p(theta), p(a_vals), p(zb),
                             p(y), p(yg), batch, seq, H, Pd, N, G)                 # :252-258
        ref.matmul_f32(p(yg), p(w_out), p(out), bs, D, DI)                         # :261
        ref.elemwise_add(p(out), p(residual), p(x), bs * D)                        # :264
    else:
        NH, KVH, HD, MLP, window = int(z["attn_n_heads"]), int(z["attn_kv_heads"]), int(z["attn_head_dim"]), int(z["mlp_dim"]), int(z["window"])
        KV = KVH * HD
        bnh = batch * NH
        wq, wk, wv, wo = wt("q_proj"), wt("k_proj"), wt("v_proj"), wt("attn_out_proj")
        wg, wu, wd = wt("mlp_gate"), wt("mlp_up"), wt("mlp_down")
        g1, g2 = dev(z["attn_norm_g"]), dev(z["mlp_norm_g"])
        residual, xn, q, k, v = buf(bs, D), buf(bs, D), buf(bs, D), buf(bs, KV), buf(bs, KV)
        qt, tmp, kt, vt = buf(bs * D), buf(bs * KV), buf(bs * D), buf(bs * D)
        scores, weights = buf(bnh * seq * seq), buf(bnh * seq * seq)
        ctxt, ctx, out = buf(bs * D), buf(bs, D), buf(bs, D)
        hid, gated = buf(bs, MLP), buf(bs, MLP)
        residual.copy_(x)                                                          # native_trainer.rs:125-126
        torch.cuda.synchronize()
        ref.rmsnorm_fwd(p(x), p(xn), p(g1), eps, bs, D)                            # :129
        ref.matmul_f32(p(xn), p(wq), p(q), bs, D, D)                               # :133-135
        ref.matmul_f32(p(xn), p(wk), p(k), bs, KV, D)
        ref.matmul_f32(p(xn), p(wv), p(v), bs, KV, D)
        ref.transpose_0213(p(q), p(qt), batch, seq, NH, HD)                        # :144-148
        ref.transpose_0213(p(k), p(tmp), batch, seq, KVH, HD)
        ref.gqa_expand(p(tmp), p(kt), batch, KVH, NH, seq, HD)
        ref.transpose_0213(p(v), p(tmp), batch, seq, KVH, HD)
        ref.gqa_expand(p(tmp), p(vt), batch, KVH, NH, seq, HD)
        ref.matmul_f32_bt_batched(p(qt), p(kt), p(scores), seq, seq, HD, bnh)      # :151-152
        ref.scale_tensor(p(scores), p(scores), 1.0 / float(np.sqrt(np.float32(HD))), bnh * seq * seq)   # :153-154
        ref.causal_softmax_fwd(p(scores), p(weights), bnh, seq, window)            # :155
        ref.matmul_f32_batched(p(weights), p(vt), p(ctxt), seq, HD, seq, bnh)      # :156-157
        ref.transpose_0213(p(ctxt), p(ctx), batch, NH, seq, HD)                    # :158
        ref.matmul_f32(p(ctx), p(wo), p(out), bs, D, D)                            # :161
        ref.elemwise_add(p(out), p(residual), p(x), bs * D)                        # :162
        torch.cuda.synchronize()
        residual.copy_(x)                                                          # :170-171
        torch.cuda.synchronize()
        ref.rmsnorm_fwd(p(x), p(xn), p(g2), eps, bs, D)                            # :174
        ref.matmul_f32(p(xn), p(wg), p(hid), bs, MLP, D)                           # :178-179
        ref.matmul_f32(p(xn), p(wu), p(gated), bs, MLP, D)
        ref.sigmoid_fwd(p(hid), p(hid), bs * MLP)                                  # :187
        ref.elemwise_mul(p(hid), p(gated), p(gated), bs * MLP)                     # :189
        ref.matmul_f32(p(gated), p(wd), p(out), bs, D, MLP)                        # :193
        ref.elemwise_add(p(out), p(residual), p(x), bs * D)                        # :194
    torch.cuda.synchronize()
    np.savez(sys.argv[2], y=x.cpu().numpy().reshape(batch, seq, D))


if __name__ == "__main__":
    main()
