// TEST INFRASTRUCTURE, NOT PRODUCT.  CPU restatement of the lumi-infer CPU path.
//
// Only the test-suite, the smoke check and the benchmark's CPU-baseline legs may load this
// library; the CUDA product never links, imports or calls it.
//
// PARITY UNPINNED: the reference's inference crate has no tests, golden vectors or fixtures,
// and the reference (Rust on Candle 0.9.2; crates not vendored, no Rust toolchain) cannot be
// built where this was written.  The arithmetic below follows the reference source line by
// line; what lives inside candle-core / candle-nn 0.9.2 (matmul summation order, argmax tie
// rule, softmax / silu / mean implementations) is fixed here BY DECLARATION:
//   * dot products: 16 interleaved partial sums (element k goes to partial k % 16, fused
//     multiply-add), combined by a fixed pairwise tree — see dot16();
//   * small reductions (mean of squares, C.h over d_state, softmax sums): ascending-index
//     sequential fp32 sums;
//   * argmax: lowest index among equal maxima;
//   * silu(x) = x / (1 + exp(-x)); softmax = exp(x - max) / sum; mean = sum * (1/n).
// It is cross-checked against an independently written numpy restatement
// (oracle/numpy_restatement.py) and, structurally, against the reference's own pins
// (in_proj_out == 7360, layer placement, byte-level ids).
//
// PINNED BY REFERENCE-AUTHORED CODE (on a GPU, by the tests): mamba_step and attention_step (without the rotary
// extension) — whole-block outputs over a window of tokens equal those of the reference's own CUDA forward kernels
// (training/csrc/elementwise_ops.cu, cublas_ops.cu, ssm_scan.cu, built from where they lie) chained as the
// reference's trainer chains them (training/src/native_trainer.rs:198-266 and :110-194).  Everything else in this
// file — embedding, final norm + head, argmax, the sampler, the extensions, the loaders — stays unpinned.
//
// What each function follows (paths inside the reference project):
//   rms_norm            inference/src/model.rs:100-106
//   sigmoid / softplus  inference/src/model.rs:12-17, 830-832
//   mamba_step          inference/src/model.rs:296-375   (CPU branch of MambaBlock::forward_step)
//   attention_step      inference/src/model.rs:492-556, KvCache::append 133-152
//   state init          inference/src/model.rs:731-763
//   forward_step        inference/src/model.rs:766-801
//   generate / sampling inference/src/main.rs:118-170, 197-209
// Extensions that the reference does not have, all off by default: rotary embedding in the
// attention block (rope_base > 0), an explicit MLP width, top-k filtering before sampling.

#include <cmath>
#include <cstdint>
#include <cstring>
#include <map>
#include <string>
#include <vector>
#include <algorithm>
#ifdef _OPENMP
#include <omp.h>
#endif

namespace {

struct Cfg {
    int d_model, n_layers, d_state, expand, n_heads, n_groups, vocab;
    int attn_n_heads, attn_kv_heads, mlp_dim;
    float rope_base;
    int d_inner() const { return expand * d_model; }
    int head_dim() const { return d_inner() / n_heads; }
    int bc() const { return n_groups * d_state; }
    int in_proj_out() const { return 2 * d_inner() + 2 * bc() + 3 * n_heads + n_heads * d_state / 2; }
    int attn_head_dim() const { return d_model / attn_n_heads; }
    int kv_dim() const { return attn_kv_heads * attn_head_dim(); }
};

struct Model {
    Cfg c;
    std::vector<uint8_t> is_attn;     // [n_layers]
    std::vector<int> window;          // [n_layers] (0 for Mamba layers / unbounded)
    std::map<std::string, std::vector<float>> t;
    const float* get(const std::string& n) const {
        auto it = t.find(n);
        return it == t.end() ? nullptr : it->second.data();
    }
};

struct LayerState {
    std::vector<float> h, prev_bx, cum;   // Mamba
    std::vector<float> k, v;              // attention: [kv_heads][len][head_dim] kept as [len][kv_dim]
    int len = 0;                          // cached tokens
    int64_t pos = 0;                      // absolute position of the next token (rotary extension)
};

struct State {
    std::vector<LayerState> L;
};

// 16 interleaved partial sums with fused multiply-add, then a fixed pairwise tree.
inline float dot16(const float* w, const float* x, int n) {
    float acc[16];
    for (int j = 0; j < 16; ++j) acc[j] = 0.0f;
    int k = 0;
    for (; k + 16 <= n; k += 16)
        for (int j = 0; j < 16; ++j) acc[j] = __builtin_fmaf(w[k + j], x[k + j], acc[j]);
    for (int j = 0; k < n; ++k, ++j) acc[j] = __builtin_fmaf(w[k], x[k], acc[j]);
    for (int s = 8; s > 0; s >>= 1)
        for (int j = 0; j < s; ++j) acc[j] = acc[j] + acc[j + s];
    return acc[0];
}

// y[r] = W[r,:] . x  for W [rows, cols] row-major (Linear without bias, model.rs:203,215,299,373)
void matvec(const float* W, const float* x, float* y, int rows, int cols) {
#pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; ++r) y[r] = dot16(W + (size_t)r * cols, x, cols);
}

// model.rs:100-106 : sqr -> mean -> +eps -> sqrt -> recip -> mul -> mul gamma
void rms_norm(const float* x, const float* gamma, float* out, int n) {
    float s = 0.0f;
    for (int i = 0; i < n; ++i) s += x[i] * x[i];
    float mean = s * (float)(1.0 / (double)n);
    float r = 1.0f / sqrtf(mean + 1e-5f);
    for (int i = 0; i < n; ++i) out[i] = (x[i] * r) * gamma[i];
}

inline float sigmoidf_ref(float x) { return 1.0f / (1.0f + expf(-x)); }   // model.rs:12-17
inline float softplusf_ref(float x) { return logf(expf(x) + 1.0f); }      // model.rs:830-832
inline float siluf_ref(float x) { return x / (1.0f + expf(-x)); }

void mamba_step(const Model& m, int layer, LayerState& st, float* x /* [d_model], in/out */) {
    const Cfg& c = m.c;
    const int D = c.d_model, DI = c.d_inner(), H = c.n_heads, P = c.head_dim(), N = c.d_state;
    const int G = c.n_groups, BC = c.bc(), HPG = H / G, HN = N / 2, R = c.in_proj_out();
    const std::string p = "blocks." + std::to_string(layer) + ".";
    const float* gamma = m.get(p + "norm.gamma");
    const float* Win = m.get(p + "in_proj.weight");
    const float* Wout = m.get(p + "out_proj.weight");
    const float* bg = m.get(p + "b_norm.gamma");
    const float* cg = m.get(p + "c_norm.gamma");
    const float* bb = m.get(p + "b_bias");
    const float* cb = m.get(p + "c_bias");
    const float* dskip = m.get(p + "ssm.d");
    const float* dtb = m.get(p + "ssm.dt_bias");

    std::vector<float> xn(D), proj(R);
    rms_norm(x, gamma, xn.data(), D);                       // :297
    matvec(Win, xn.data(), proj.data(), R, D);              // :298-299

    const float* x_ssm = proj.data();                       // :301-308
    const float* z = proj.data() + DI;
    const float* b_proj = proj.data() + 2 * DI;
    const float* c_proj = proj.data() + 2 * DI + BC;
    const float* dt = proj.data() + 2 * DI + 2 * BC;
    const float* lam_raw = dt + H;
    const float* dda = dt + 2 * H;
    const float* theta = dt + 3 * H;                        // :330-331

    std::vector<float> xa(DI), bn(BC), cn(BC);
    for (int i = 0; i < DI; ++i) xa[i] = siluf_ref(x_ssm[i]);            // :310
    rms_norm(b_proj, bg, bn.data(), BC);                                  // :311-312 (norm over all bc)
    rms_norm(c_proj, cg, cn.data(), BC);
    for (int i = 0; i < BC; ++i) { bn[i] = bn[i] + (bb ? bb[i] : 1.0f); cn[i] = cn[i] + (cb ? cb[i] : 1.0f); }

    std::vector<float> brot(N), crot(N);
    std::vector<float> y(DI);
    const float PI = 3.14159265358979323846f;
    const float two_pi = 2.0f * PI;
    for (int h = 0; h < H; ++h) {
        float dtp = softplusf_ref(dt[h] + dtb[h]);                        // :314-315
        float a = -softplusf_ref(dda[h]);                                 // :316
        a = std::min(std::max(a, -1e6f), -1e-4f);
        float abar = expf(a * dtp);                                       // :317
        float lam = sigmoidf_ref(lam_raw[h]);                             // :307
        float oml = lam * -1.0f + 1.0f;                                   // :356 affine(-1, 1)
        float c2 = abar * oml;                                            // :359
        const float* bgp = bn.data() + (h / HPG) * N;                     // :319-327
        const float* cgp = cn.data() + (h / HPG) * N;
        for (int k = 0; k < HN; ++k) {                                    // :338-350
            float angle = tanhf(theta[h * HN + k]) * PI;
            float& cu = st.cum[h * HN + k];
            cu = fmodf(cu + dtp * angle, two_pi);
            float ca = cosf(cu), sa = sinf(cu);
            brot[2 * k] = ca * bgp[2 * k] - sa * bgp[2 * k + 1];
            brot[2 * k + 1] = sa * bgp[2 * k] + ca * bgp[2 * k + 1];
            crot[2 * k] = ca * cgp[2 * k] - sa * cgp[2 * k + 1];
            crot[2 * k + 1] = sa * cgp[2 * k] + ca * cgp[2 * k + 1];
        }
        for (int pp = 0; pp < P; ++pp) {                                  // :354-368
            float xv = xa[h * P + pp];
            float* hh = st.h.data() + ((size_t)h * P + pp) * N;
            float* pb = st.prev_bx.data() + ((size_t)h * P + pp) * N;
            float acc = 0.0f;
            for (int s = 0; s < N; ++s) {
                float bx = xv * brot[s];
                float t1 = abar * hh[s];
                float t2 = c2 * pb[s];
                float t3 = lam * bx;
                float nh = (t1 + t2) + t3;
                hh[s] = nh;
                pb[s] = bx;
                acc += crot[s] * nh;
            }
            float yv = acc + dskip[h] * xv;                               // :367-368
            y[h * P + pp] = yv * siluf_ref(z[h * P + pp]);                // :370
        }
    }
    std::vector<float> out(D);
    matvec(Wout, y.data(), out.data(), D, DI);                            // :372-373
    for (int i = 0; i < D; ++i) x[i] = out[i] + x[i];                     // :374
}

void attention_step(const Model& m, int layer, LayerState& st, float* x) {
    const Cfg& c = m.c;
    const int D = c.d_model, NH = c.attn_n_heads, KH = c.attn_kv_heads, HD = c.attn_head_dim();
    const int KV = c.kv_dim(), HPK = NH / KH, MLP = c.mlp_dim;
    const std::string p = "blocks." + std::to_string(layer) + ".";
    std::vector<float> xn(D), q(D), k(KV), v(KV);
    rms_norm(x, m.get(p + "attn_norm.gamma"), xn.data(), D);              // :500
    matvec(m.get(p + "q_proj.weight"), xn.data(), q.data(), D, D);        // :504-506
    matvec(m.get(p + "k_proj.weight"), xn.data(), k.data(), KV, D);
    matvec(m.get(p + "v_proj.weight"), xn.data(), v.data(), KV, D);
    if (c.rope_base > 0.0f) {   // extension: interleaved-pair rotary embedding at the absolute position
        for (int i = 0; i < HD / 2; ++i) {
            float inv = powf(c.rope_base, -(float)(2 * i) / (float)HD);
            float ang = (float)st.pos * inv;
            float ca = cosf(ang), sa = sinf(ang);
            for (int hq = 0; hq < NH; ++hq) {
                float a0 = q[hq * HD + 2 * i], a1 = q[hq * HD + 2 * i + 1];
                q[hq * HD + 2 * i] = ca * a0 - sa * a1;
                q[hq * HD + 2 * i + 1] = sa * a0 + ca * a1;
            }
            for (int hk = 0; hk < KH; ++hk) {
                float a0 = k[hk * HD + 2 * i], a1 = k[hk * HD + 2 * i + 1];
                k[hk * HD + 2 * i] = ca * a0 - sa * a1;
                k[hk * HD + 2 * i + 1] = sa * a0 + ca * a1;
            }
        }
    }
    st.pos += 1;
    // KvCache::append, :133-152 — concatenate, then keep the last `window` entries
    st.k.insert(st.k.end(), k.begin(), k.end());
    st.v.insert(st.v.end(), v.begin(), v.end());
    st.len += 1;
    int win = m.window[layer];
    if (win > 0 && st.len > win) {
        int drop = st.len - win;
        st.k.erase(st.k.begin(), st.k.begin() + (size_t)drop * KV);
        st.v.erase(st.v.begin(), st.v.begin() + (size_t)drop * KV);
        st.len = win;
    }
    const int T = st.len;
    const float scale = (float)(1.0 / sqrt((double)HD));                  // :530
    std::vector<float> ctx(D), sc(T);
    for (int hq = 0; hq < NH; ++hq) {
        int hk = hq / HPK;                                                // :520-525
        float mx = -INFINITY;
        for (int t = 0; t < T; ++t) {
            const float* kr = st.k.data() + (size_t)t * KV + hk * HD;
            float s = 0.0f;
            for (int d = 0; d < HD; ++d) s += q[hq * HD + d] * kr[d];
            s = s * scale;                                                // :532 affine(scale, 0)
            sc[t] = s;
            mx = std::max(mx, s);
        }
        float sum = 0.0f;                                                 // :535
        for (int t = 0; t < T; ++t) { sc[t] = expf(sc[t] - mx); sum += sc[t]; }
        for (int t = 0; t < T; ++t) sc[t] = sc[t] / sum;
        for (int d = 0; d < HD; ++d) {                                    // :538
            float a = 0.0f;
            for (int t = 0; t < T; ++t) a += sc[t] * st.v[(size_t)t * KV + hk * HD + d];
            ctx[hq * HD + d] = a;
        }
    }
    std::vector<float> o(D);
    matvec(m.get(p + "attn_out_proj.weight"), ctx.data(), o.data(), D, D);   // :542
    for (int i = 0; i < D; ++i) x[i] = o[i] + x[i];                           // :543
    // sigmoid-gated MLP, :546-555
    rms_norm(x, m.get(p + "mlp_norm.gamma"), xn.data(), D);
    std::vector<float> g(MLP), u(MLP), hid(MLP);
    matvec(m.get(p + "mlp_gate.weight"), xn.data(), g.data(), MLP, D);
    matvec(m.get(p + "mlp_up.weight"), xn.data(), u.data(), MLP, D);
    for (int i = 0; i < MLP; ++i) hid[i] = sigmoidf_ref(g[i]) * u[i];
    matvec(m.get(p + "mlp_down.weight"), hid.data(), o.data(), D, MLP);
    for (int i = 0; i < D; ++i) x[i] = o[i] + x[i];
}

void init_state(const Model& m, State& s) {                               // model.rs:731-763
    const Cfg& c = m.c;
    const int H = c.n_heads, P = c.head_dim(), N = c.d_state;
    s.L.assign(c.n_layers, LayerState());
    for (int l = 0; l < c.n_layers; ++l) {
        LayerState& st = s.L[l];
        if (m.is_attn[l]) continue;
        st.h.assign((size_t)H * P * N, 0.0f);
        st.prev_bx.assign((size_t)H * P * N, 0.0f);
        st.cum.assign((size_t)H * N / 2, 0.0f);
        const float* hi = m.get("blocks." + std::to_string(l) + ".ssm.h_init");
        if (hi)
            for (int h = 0; h < H; ++h)
                for (int p = 0; p < P; ++p)
                    for (int n = 0; n < N; ++n) st.h[((size_t)h * P + p) * N + n] = hi[h * N + n];
    }
}

void forward_step(const Model& m, State& s, uint32_t tok, float* logits, float* hidden_out) {  // :766-801
    const Cfg& c = m.c;
    const float* E = m.get("embedding.weight");
    std::vector<float> x(E + (size_t)tok * c.d_model, E + (size_t)(tok + 1) * c.d_model);
    for (int l = 0; l < c.n_layers; ++l) {
        if (m.is_attn[l]) attention_step(m, l, s.L[l], x.data());
        else mamba_step(m, l, s.L[l], x.data());
    }
    if (hidden_out) memcpy(hidden_out, x.data(), sizeof(float) * c.d_model);
    if (!logits) return;
    std::vector<float> xn(c.d_model);
    rms_norm(x.data(), m.get("final_norm.gamma"), xn.data(), c.d_model);
    matvec(E, xn.data(), logits, c.vocab, c.d_model);
}

// greedy: main.rs:142-143 (lowest index wins ties by declaration)
uint32_t argmax(const float* l, int n) {
    int best = 0;
    for (int i = 1; i < n; ++i) if (l[i] > l[best]) best = i;
    return (uint32_t)best;
}

// main.rs:145-147 + 197-209, with optional top-k filtering (extension) before the softmax.
// Survivors: the k largest logits, ties broken towards the lower index.
uint32_t sample(const float* logits, int n, double temperature, int top_k, float r) {
    std::vector<float> sc(n);
    const float inv_t = (float)(1.0 / temperature);         // Tensor / f64 == affine(1/t, 0)
    for (int i = 0; i < n; ++i) sc[i] = logits[i] * inv_t;
    std::vector<uint8_t> keep(n, 1);
    if (top_k > 0 && top_k < n) {
        std::vector<int> idx(n);
        for (int i = 0; i < n; ++i) idx[i] = i;
        std::stable_sort(idx.begin(), idx.end(), [&](int a, int b) { return logits[a] > logits[b]; });
        std::fill(keep.begin(), keep.end(), 0);
        for (int i = 0; i < top_k; ++i) keep[idx[i]] = 1;
    }
    float mx = -INFINITY;
    for (int i = 0; i < n; ++i) if (keep[i]) mx = std::max(mx, sc[i]);
    float sum = 0.0f;
    for (int i = 0; i < n; ++i) if (keep[i]) { sc[i] = expf(sc[i] - mx); sum += sc[i]; }
    float cum = 0.0f;
    int last = n - 1;
    for (int i = 0; i < n; ++i) {
        if (!keep[i]) continue;
        last = i;
        cum += sc[i] / sum;
        if (cum >= r) return (uint32_t)i;
    }
    return (uint32_t)last;      // main.rs:208 (last index; last survivor when filtering)
}

}  // namespace

extern "C" {

// Launchers such as torchrun export OMP_NUM_THREADS=1; a timed CPU baseline sets its thread count itself.
int32_t oracle_set_threads(int32_t n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
    return omp_get_max_threads();
#else
    (void)n;
    return 1;
#endif
}

// cfg: d_model, n_layers, d_state, expand, n_heads, n_groups, vocab, attn_n_heads, attn_kv_heads, mlp_dim
void* oracle_model_new(const int32_t* cfg, float rope_base, const uint8_t* is_attn, const int32_t* window) {
    Model* m = new Model();
    m->c = Cfg{cfg[0], cfg[1], cfg[2], cfg[3], cfg[4], cfg[5], cfg[6], cfg[7], cfg[8], cfg[9], rope_base};
    m->is_attn.assign(is_attn, is_attn + cfg[1]);
    m->window.assign(window, window + cfg[1]);
    return m;
}
void oracle_model_free(void* m) { delete (Model*)m; }

// name without the "item." prefix; data is copied
void oracle_set_tensor(void* mp, const char* name, const float* data, int64_t n) {
    ((Model*)mp)->t[name].assign(data, data + n);
}

void* oracle_state_new(void* mp) {
    State* s = new State();
    init_state(*(Model*)mp, *s);
    return s;
}
void oracle_state_free(void* s) { delete (State*)s; }

void oracle_forward_step(void* mp, void* sp, uint32_t tok, float* logits, float* hidden_out) {
    forward_step(*(Model*)mp, *(State*)sp, tok, logits, hidden_out);
}

// one Mamba block on a caller-supplied residual stream (kernel-level parity tests)
void oracle_mamba_block(void* mp, void* sp, int32_t layer, float* x) {
    mamba_step(*(Model*)mp, layer, ((State*)sp)->L[layer], x);
}
void oracle_attention_block(void* mp, void* sp, int32_t layer, float* x) {
    attention_step(*(Model*)mp, layer, ((State*)sp)->L[layer], x);
}

// Copies the Mamba state of one layer (any pointer may be null).
void oracle_read_state(void* sp, int32_t layer, float* h, float* prev_bx, float* cum) {
    LayerState& st = ((State*)sp)->L[layer];
    if (h) memcpy(h, st.h.data(), st.h.size() * sizeof(float));
    if (prev_bx) memcpy(prev_bx, st.prev_bx.data(), st.prev_bx.size() * sizeof(float));
    if (cum) memcpy(cum, st.cum.data(), st.cum.size() * sizeof(float));
}

uint32_t oracle_argmax(const float* l, int32_t n) { return argmax(l, n); }
uint32_t oracle_sample(const float* l, int32_t n, double temperature, int32_t top_k, float r) {
    return sample(l, n, temperature, top_k, r);
}

// The generate loop (main.rs:118-170).  `uniforms` holds one r in [0,1) per generated token and
// is read only when temperature > 0.  `logits_dump` (may be null) receives the logits each
// generated token was chosen from: [n_new, vocab].  Returns the number of tokens generated.
int32_t oracle_generate(void* mp, void* sp, const uint32_t* prompt, int32_t T, int32_t n_new,
                        double temperature, int32_t top_k, const float* uniforms, uint32_t eos,
                        int32_t ignore_eos, uint32_t* out, float* logits_dump) {
    Model& m = *(Model*)mp;
    State& s = *(State*)sp;
    const int V = m.c.vocab;
    std::vector<float> logits(V);
    if (T <= 0) return 0;                                    // main.rs:137-140 (no logits: stop)
    for (int t = 0; t < T; ++t) forward_step(m, s, prompt[t], logits.data(), nullptr);   // :121-125
    int n = 0;
    for (int i = 0; i < n_new; ++i) {
        if (logits_dump) memcpy(logits_dump + (size_t)i * V, logits.data(), sizeof(float) * V);
        uint32_t next = (temperature <= 0.0) ? argmax(logits.data(), V)
                                             : sample(logits.data(), V, temperature, top_k, uniforms[i]);
        if (next == eos && !ignore_eos) break;               // :150
        out[n++] = next;
        forward_step(m, s, next, logits.data(), nullptr);    // :169
    }
    return n;
}

}  // extern "C"
