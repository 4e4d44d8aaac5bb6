"""Second, independently written restatement of the lumi-infer CPU path, in numpy tensor ops.

TEST INFRASTRUCTURE, NOT PRODUCT.  Parity unpinned (the reference cannot run where this was
written and its inference crate has no golden vectors): this file exists so that two
restatements written separately from the same source lines — this one in whole-tensor numpy
operations shaped like the reference's Candle calls, oracle/lumi_oracle.cpp in scalar loops —
can catch each other's slips.  It also makes the committed fixtures under tests/golden/.

Follows inference/src/model.rs:100-106 (RmsNorm), :296-375 (Mamba step, CPU branch),
:492-556 + :133-152 (attention step + cache), :731-763 (state init), :766-801 (forward_step),
inference/src/main.rs:118-170 and :197-209 (token loop, sampling).
All arithmetic is float32; matmuls are numpy's (summation order differs from the C++ oracle,
so the two agree to rounding, not bit for bit).
"""
from __future__ import annotations

import numpy as np

f32 = np.float32


def _sigmoid(x):
    one = np.ones_like(x)
    return one / (one + np.exp(-x))


def _softplus(x):
    return np.log(np.exp(x) + f32(1.0))


def _silu(x):
    return x / (f32(1.0) + np.exp(-x))


def _rms_norm(x, gamma):
    mean_sq = np.mean(np.square(x), axis=-1, keepdims=True, dtype=f32)
    norm = f32(1.0) / np.sqrt(mean_sq + f32(1e-5))
    return (x * norm) * gamma


class NumpyModel:
    def __init__(self, cfg, tensors):
        from lumi_b200 import synth
        self.cfg = cfg
        self.t = {n[5:]: np.asarray(synth.as_f32(dt, a), dtype=f32) for n, dt, a in tensors}

    def init_states(self):
        c = self.cfg
        states = []
        ai = 0
        for i in range(c.n_layers):
            if c.is_attention_layer(i):
                states.append({"k": None, "v": None, "window": c.attn_window_size(ai), "pos": 0})
                ai += 1
            else:
                hi = self.t.get(f"blocks.{i}.ssm.h_init")
                if hi is not None:
                    h = np.broadcast_to(hi.reshape(c.n_heads, 1, c.d_state),
                                        (c.n_heads, c.head_dim, c.d_state)).astype(f32).copy()
                else:
                    h = np.zeros((c.n_heads, c.head_dim, c.d_state), f32)
                states.append({"h": h, "prev_bx": np.zeros_like(h),
                               "cum": np.zeros((c.n_heads, c.d_state // 2), f32)})
        return states

    def mamba_step(self, i, x, st):
        c, t = self.cfg, self.t
        p = f"blocks.{i}."
        di, bc, H, P, N, G = c.d_inner, c.bc_size, c.n_heads, c.head_dim, c.d_state, c.n_groups
        residual = x
        xn = _rms_norm(x, t[p + "norm.gamma"])
        proj = t[p + "in_proj.weight"] @ xn
        o = 0
        x_ssm = proj[o:o + di]; o += di
        z = proj[o:o + di]; o += di
        b_proj = proj[o:o + bc]; o += bc
        c_proj = proj[o:o + bc]; o += bc
        dt = proj[o:o + H]; o += H
        lam = _sigmoid(proj[o:o + H]); o += H
        dda = proj[o:o + H]; o += H
        theta = proj[o:o + H * N // 2].reshape(H, N // 2)
        x_act = _silu(x_ssm)
        ones = np.ones(bc, f32)
        b_n = _rms_norm(b_proj, t[p + "b_norm.gamma"]) + t.get(p + "b_bias", ones)
        c_n = _rms_norm(c_proj, t[p + "c_norm.gamma"]) + t.get(p + "c_bias", ones)
        dt_pos = _softplus(dt + t[p + "ssm.dt_bias"])
        a_vals = np.clip(-_softplus(dda), f32(-1e6), f32(-1e-4))
        a_bar = np.exp(a_vals * dt_pos)
        x_heads = x_act.reshape(H, P)
        b_e = np.repeat(b_n.reshape(G, N), H // G, axis=0)
        c_e = np.repeat(c_n.reshape(G, N), H // G, axis=0)
        pi = f32(np.pi)
        angle = np.tanh(theta) * pi
        st["cum"] = np.fmod(st["cum"] + dt_pos[:, None] * angle, f32(2.0) * pi).astype(f32)
        ca, sa = np.cos(st["cum"]), np.sin(st["cum"])

        def rot(v):
            e, od = v[:, 0::2], v[:, 1::2]
            out = np.empty_like(v)
            out[:, 0::2] = ca * e - sa * od
            out[:, 1::2] = sa * e + ca * od
            return out
        b_r, c_r = rot(b_e), rot(c_e)
        bx = x_heads[:, :, None] * b_r[:, None, :]
        lam3 = lam[:, None, None]
        oml = lam3 * f32(-1.0) + f32(1.0)
        ab3 = a_bar[:, None, None]
        new_h = (ab3 * st["h"] + (ab3 * oml) * st["prev_bx"]) + lam3 * bx
        st["h"] = new_h.astype(f32)
        st["prev_bx"] = bx.astype(f32)
        y = (c_r[:, None, :] * st["h"]).sum(axis=2, dtype=f32) + t[p + "ssm.d"][:, None] * x_heads
        y = y.reshape(di) * _silu(z)
        return t[p + "out_proj.weight"] @ y + residual

    def attention_step(self, i, x, st):
        c, t = self.cfg, self.t
        p = f"blocks.{i}."
        nh, kh, hd = c.attn_n_heads, c.attn_kv_heads, c.attn_head_dim
        residual = x
        xn = _rms_norm(x, t[p + "attn_norm.gamma"])
        q = (t[p + "q_proj.weight"] @ xn).reshape(nh, hd)
        k = (t[p + "k_proj.weight"] @ xn).reshape(kh, 1, hd)
        v = (t[p + "v_proj.weight"] @ xn).reshape(kh, 1, hd)
        if c.attn_rope_base > 0:
            idx = np.arange(hd // 2, dtype=f32)
            inv = np.power(f32(c.attn_rope_base), -(f32(2.0) * idx) / f32(hd)).astype(f32)
            ang = (f32(st["pos"]) * inv).astype(f32)
            ca, sa = np.cos(ang), np.sin(ang)

            def rot(a):
                e, od = a[..., 0::2].copy(), a[..., 1::2].copy()
                a = a.copy()
                a[..., 0::2] = ca * e - sa * od
                a[..., 1::2] = sa * e + ca * od
                return a
            q, k = rot(q), rot(k)
        st["pos"] += 1
        if st["k"] is None:
            st["k"], st["v"] = k, v
        else:
            st["k"] = np.concatenate([st["k"], k], axis=1)
            st["v"] = np.concatenate([st["v"], v], axis=1)
        w = st["window"]
        if w > 0 and st["k"].shape[1] > w:
            st["k"], st["v"] = st["k"][:, -w:], st["v"][:, -w:]
        ke = np.repeat(st["k"], nh // kh, axis=0)
        ve = np.repeat(st["v"], nh // kh, axis=0)
        scale = f32(1.0 / np.sqrt(float(hd)))
        scores = np.einsum("hd,htd->ht", q, ke).astype(f32) * scale
        scores = scores - scores.max(axis=1, keepdims=True)
        e = np.exp(scores)
        wts = e / e.sum(axis=1, keepdims=True, dtype=f32)
        ctx = np.einsum("ht,htd->hd", wts, ve).astype(f32).reshape(c.d_model)
        x = t[p + "attn_out_proj.weight"] @ ctx + residual
        residual = x
        xn = _rms_norm(x, t[p + "mlp_norm.gamma"])
        hidden = _sigmoid(t[p + "mlp_gate.weight"] @ xn) * (t[p + "mlp_up.weight"] @ xn)
        return t[p + "mlp_down.weight"] @ hidden + residual

    def forward_step(self, token, states):
        c, t = self.cfg, self.t
        x = t["embedding.weight"][int(token)].copy()
        for i in range(c.n_layers):
            if c.is_attention_layer(i):
                x = self.attention_step(i, x, states[i])
            else:
                x = self.mamba_step(i, x, states[i])
        self.last_hidden = x
        xn = _rms_norm(x, t["final_norm.gamma"])
        return (t["embedding.weight"] @ xn).astype(f32)

    def generate(self, prompt, n_new, temperature=0.0, top_k=0, uniforms=None, eos=2, ignore_eos=False):
        states = self.init_states()
        logits = None
        for tok in prompt:
            logits = self.forward_step(tok, states)
        out, dumps = [], []
        for i in range(n_new):
            if logits is None:
                break
            dumps.append(logits)
            if temperature <= 0:
                nxt = int(np.argmax(logits))
            else:
                nxt = sample_from_logits(logits, temperature, top_k, uniforms[i])
            if nxt == eos and not ignore_eos:
                break
            out.append(nxt)
            logits = self.forward_step(nxt, states)
        return np.array(out, dtype=np.uint32), dumps, states


def sample_from_logits(logits, temperature, top_k, r):
    """softmax(logits / temperature) then the CDF walk of main.rs:197-209; `top_k` > 0 keeps the k
    largest logits (ties towards the lower index) and renormalises (an extension)."""
    n = logits.shape[0]
    sc = logits * f32(1.0 / temperature)
    keep = np.ones(n, bool)
    if 0 < top_k < n:
        order = np.argsort(-logits, kind="stable")
        keep[:] = False
        keep[order[:top_k]] = True
    mx = sc[keep].max()
    e = np.where(keep, np.exp(sc - mx), f32(0)).astype(f32)
    s = f32(0)
    for v in e[keep]:
        s = f32(s + v)
    cum = f32(0)
    last = n - 1
    for i in np.nonzero(keep)[0]:
        last = int(i)
        cum = f32(cum + f32(e[i] / s))
        if cum >= r:
            return int(i)
    return last


# ---- Philox4x32-10 (Salmon et al., SC'11), restated for the sampler's uniforms -----------------
_M0, _M1 = 0xD2511F53, 0xCD9E8D57
_W0, _W1 = 0x9E3779B9, 0xBB67AE85


def philox4x32_10(counter, key):
    """counter: 4 uint32, key: 2 uint32 -> 4 uint32."""
    c = [int(v) & 0xFFFFFFFF for v in counter]
    k = [int(v) & 0xFFFFFFFF for v in key]
    for _ in range(10):
        p0 = _M0 * c[0]
        p1 = _M1 * c[2]
        c = [((p1 >> 32) ^ c[1] ^ k[0]) & 0xFFFFFFFF, p1 & 0xFFFFFFFF,
             ((p0 >> 32) ^ c[3] ^ k[1]) & 0xFFFFFFFF, p0 & 0xFFFFFFFF]
        k = [(k[0] + _W0) & 0xFFFFFFFF, (k[1] + _W1) & 0xFFFFFFFF]
    return c


def sampler_uniform(seed: int, sequence: int, step: int) -> np.float32:
    """The uniform in [0,1) the sampler draws for (seed, sequence, step):
    key = (seed low 32 bits, seed high 32 bits), counter = (step, sequence, 0, 0), first output word,
    top 24 bits scaled by 2^-24."""
    w = philox4x32_10([step, sequence, 0, 0], [seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF])[0]
    return f32((w >> 8) * (1.0 / 16777216.0))
