// Chunked (SSD-style) prefill of the Mamba-3 trapezoidal recurrence, chunk length 64.
//
// The reference prefills token by token (inference/src/main.rs:121-125) and its only NVIDIA scan
// is sequential in time (training/csrc/ssm_scan.cu:137-227; SSD_FWD_CHUNK there is dead code).
// This kernel evaluates the same recurrence (inference/src/model.rs:354-368)
//     S_t = a_t S_{t-1} + (1 - lam_t) a_t U_{t-1} + lam_t U_t ,   U_t = x_t (x) B~_t ,   y_t = S_t C~_t + D x_t
// a chunk at a time.  With the augmented state  S^_t = S_t + (1 - lam_{t+1}) U_t  it becomes
//     S^_t = a_t S^_{t-1} + kap_t U_t ,   kap_t = lam_t + 1 - lam_{t+1} ,   S_t = a_t S^_{t-1} + lam_t U_t ,
// an ordinary decayed linear recurrence, so inside a chunk starting at t0 (l_i = sum of log a up to i)
//     y_i = e^{l_i} (S^_in C~_i) + sum_{j<i} e^{l_i - l_j} kap_j (C~_i . B~_j) x_j + lam_i (C~_i . B~_i) x_i + D x_i
//     S^_out = e^{l_last} S^_in + sum_j e^{l_last - l_j} kap_j x_j (x) B~_j
// — three small matrix products per (sequence, head, chunk).  The last token of a launch uses
// kap = lam, which makes S^ equal the true S: every launch ends with exactly the state the decode
// kernel expects (h, x_prev, B~_prev, cum_angle), and the next launch rebuilds S^ from it.
// DD-RoPE angles are a prefix sum over the chunk taken mod 2 pi at the end (the reference reduces
// mod 2 pi every step: same angle, rounding-level differences; the stored angle may differ from the
// sequential one by a multiple of 2 pi).
//
// One CTA per (head, sequence); fp32 arithmetic on CUDA cores with shared-memory tiles.
#include "internal.h"

namespace lumi {

namespace {

constexpr int LCH = 64;          // chunk length
constexpr int LDS_ = 68;         // row stride of the shared tiles (floats): 16-byte aligned, conflict-free row walks

__device__ __forceinline__ float sigmoid_ref(float x) { return __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-x))); }
__device__ __forceinline__ float softplus_ref(float x) { return logf(__fadd_rn(expf(x), 1.0f)); }
__device__ __forceinline__ float silu_ref(float x) { return __fdiv_rn(x, __fadd_rn(1.0f, expf(-x))); }
__device__ __forceinline__ float dot4(const float4& a, const float4& b) { return fmaf(a.x, b.x, fmaf(a.y, b.y, fmaf(a.z, b.z, a.w * b.w))); }
__device__ __forceinline__ void split_bf16(float v, __nv_bfloat16& hi, __nv_bfloat16& lo) {
    hi = __float2bfloat16_rn(v);
    lo = __float2bfloat16_rn(v - __bfloat162float(hi));
}

struct PfSmem {
    float Bt[LCH][LDS_];       // rotated B~ of the chunk              [token][n]
    float Ct[LCH][LDS_];       // rotated C~                           [token][n]
    float Wm[LCH][LDS_];       // masked, decayed (C~ B~^T)            [i][j]
    float Xt[32][LDS_];        // silu(x) transposed                   [p][token]
    float Sh[32][LDS_];        // augmented state S^                   [p][n]
    float Gt[LCH][33];         // silu(z) gate                         [token][p]
    float seg[9][32];          // angle prefix sums of the 8 token segments
    float ell[LCH], lam[LCH + 1], kap[LCH], dtp[LCH], wj[LCH];
    float cum[32];
};

// row r = b * ts + t  of the super-chunk; token ids come from prompt[(t_abs) * batch_total + b_abs]
template <typename WT>
__global__ void embed_rows_kernel(const WT* __restrict__ emb, const uint32_t* __restrict__ prompt, float* __restrict__ x, int D,
                                  int vocab, int ts, int t_abs0, int b_abs0, int batch_total, StepCtl* ctl) {
    const int r = blockIdx.x, b = r / ts, t = r - b * ts;
    uint32_t tok = prompt[(size_t)(t_abs0 + t) * batch_total + b_abs0 + b];
    if (tok >= (uint32_t)vocab) { if (threadIdx.x == 0) atomicOr(&ctl->status, STATUS_BAD_TOKEN); tok = 0; }
    const WT* row = emb + (size_t)tok * D;
    for (int k = threadIdx.x; k < D; k += blockDim.x) {
        float v;
        if (sizeof(WT) == 4) v = reinterpret_cast<const float*>(row)[k];
        else v = __uint_as_float((uint32_t)reinterpret_cast<const uint16_t*>(row)[k] << 16);
        x[(size_t)r * D + k] = v;
    }
}

// BCNorm scales of every token row: r_b, r_c = 1 / sqrt(mean(B^2) + eps) over all n_groups * d_state (model.rs:311-312)
__global__ void bc_stats_kernel(const float* __restrict__ proj, int ldp, int off_b, int BC, float eps, float* __restrict__ rb,
                                float* __restrict__ rc, int rows) {
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= rows) return;
    const float* Bp = proj + (size_t)warp * ldp + off_b;
    const float* Cp = Bp + BC;
    float sb = 0.f, sc = 0.f;
    for (int i = lane; i < BC; i += 32) { sb = fmaf(Bp[i], Bp[i], sb); sc = fmaf(Cp[i], Cp[i], sc); }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) { sb += __shfl_xor_sync(0xffffffffu, sb, o); sc += __shfl_xor_sync(0xffffffffu, sc, o); }
    if (lane == 0) {
        rb[warp] = __frcp_rn(__fsqrt_rn(__fadd_rn(__fmul_rn(sb, (float)(1.0 / (double)BC)), eps)));
        rc[warp] = __frcp_rn(__fsqrt_rn(__fadd_rn(__fmul_rn(sc, (float)(1.0 / (double)BC)), eps)));
    }
}

// last token's residual row of every sequence -> x[b][D] (for the lm_head after the prompt)
__global__ void gather_last_kernel(const float* __restrict__ xr, float* __restrict__ x, int D, int ts, int b0) {
    const int b = blockIdx.x;
    for (int k = threadIdx.x; k < D; k += blockDim.x) x[(size_t)(b0 + b) * D + k] = xr[((size_t)b * ts + ts - 1) * D + k];
}

__global__ void __launch_bounds__(256, 2) ssd_prefill_kernel(PrefillArgs a) {
    constexpr int P = 32, N = 64, HN = 32;
    extern __shared__ uint8_t pf_raw[];
    PfSmem& sm = *reinterpret_cast<PfSmem*>((reinterpret_cast<uintptr_t>(pf_raw) + 15) & ~(uintptr_t)15);
    const int h = blockIdx.x, b = blockIdx.y, tid = threadIdx.x, lane = tid & 31;
    const int H = a.H, DI = H * P, BC = a.G * N, ts = a.ts, R = a.ldp;
    const int g = h / (H / a.G);
    const size_t bh = (size_t)(a.b0 + b) * H + h;
    const float* prow0 = a.proj + (size_t)b * ts * R;      // first token row of this sequence
    const int off_b = 2 * DI, off_c = off_b + BC, off_dt = off_c + BC;
    const float PI_F = 3.14159265358979323846f;
    const float TWO_PI = __fmul_rn(2.0f, PI_F);
    const float dskip = a.dskip[h], dtb = a.dtb[h];

    // incoming state: S (true state of the decode representation); S^ is formed once lam of the first token is known
    for (int i = tid; i < P * N; i += 256) sm.Sh[i / N][i % N] = a.h[bh * (size_t)(P * N) + i];
    if (tid < HN) sm.cum[tid] = a.cum[bh * HN + tid];
    __syncthreads();

    // BCNorm weights of this thread's angle pair (the same for every token)
    const int kk0 = g * N + 2 * (tid & 31);
    const float kbg0 = a.bg[kk0], kbg1 = a.bg[kk0 + 1], kbb0 = a.bb[kk0], kbb1 = a.bb[kk0 + 1];
    const float kcg0 = a.cg[kk0], kcg1 = a.cg[kk0 + 1], kcb0 = a.cb[kk0], kcb1 = a.cb[kk0 + 1];

    int last_valid = 0;
    for (int t0 = 0; t0 < ts; t0 += LCH) {
        const int nv = min(LCH, ts - t0);                  // valid tokens in this chunk
        last_valid = nv - 1;
        // ---- 1. per-token scalars (model.rs:307, 314-317)
        if (tid < LCH) {
            float dtpv = 0.f, gl = 0.f, lm = 0.f;
            if (tid < nv) {
                const float* pr = prow0 + (size_t)(t0 + tid) * R;
                dtpv = softplus_ref(__fadd_rn(pr[off_dt + h], dtb));
                float av = -softplus_ref(pr[off_dt + 2 * H + h]);
                av = fminf(fmaxf(av, -1e6f), -1e-4f);
                gl = __fmul_rn(av, dtpv);                 // log a_t
                lm = sigmoid_ref(pr[off_dt + H + h]);
            }
            sm.dtp[tid] = dtpv; sm.ell[tid] = gl; sm.lam[tid] = lm;
        }
        if (tid == LCH) {
            // lam of the token after this chunk; < 0 marks "none in this launch"
            sm.lam[LCH] = (t0 + LCH < ts) ? sigmoid_ref(prow0[(size_t)(t0 + LCH) * R + off_dt + H + h]) : -1.0f;
        }
        __syncthreads();
        if (tid < 32) {                                    // inclusive prefix of log a over the chunk
            float v0 = sm.ell[2 * lane], v1 = sm.ell[2 * lane + 1];
            float s = v0 + v1, incl = s;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) { float n = __shfl_up_sync(0xffffffffu, incl, o); if (lane >= o) incl += n; }
            const float excl = incl - s;
            sm.ell[2 * lane] = excl + v0;
            sm.ell[2 * lane + 1] = excl + s;
        }
        __syncthreads();
        if (tid < LCH) {
            const int i = tid;
            float k = 0.f;
            if (i < nv) {
                const float ln = (i + 1 < nv) ? sm.lam[i + 1] : ((nv == LCH) ? sm.lam[LCH] : -1.0f);
                k = (ln < 0.f) ? sm.lam[i] : __fadd_rn(sm.lam[i], __fsub_rn(1.0f, ln));
            }
            sm.kap[i] = k;
            sm.wj[i] = expf(sm.ell[LCH - 1] - sm.ell[i]) * k;
        }
        if (t0 == 0) {
            // S^_in = S + (1 - lam_first) x_prev (x) B~_prev   (prev_bx of the decode state, model.rs:359)
            const float oml = __fadd_rn(__fmul_rn(sm.lam[0], -1.0f), 1.0f);
            for (int i = tid; i < P * N; i += 256) {
                const int p = i / N, n = i % N;
                sm.Sh[p][n] += oml * (a.xprev[bh * P + p] * a.bprev[bh * N + n]);
            }
        }
        // ---- 2. x, gate, normalised B / C, angles, rotation
        {
            // all loads of the chunk's x and z first (8 tokens per thread), then the activations: the projection rows
            // come from DRAM and a load-use-load chain per token was the largest stall of this kernel
            constexpr int NE = LCH * P / 256;
            float xr[NE], zr[NE];
#pragma unroll
            for (int q = 0; q < NE; ++q) {
                const int e = tid + 256 * q, i = e / P, p = e % P;
                xr[q] = 0.f; zr[q] = 0.f;
                if (i < nv) {
                    const float* pr = prow0 + (size_t)(t0 + i) * R;
                    xr[q] = pr[h * P + p];
                    zr[q] = pr[DI + h * P + p];
                }
            }
#pragma unroll
            for (int q = 0; q < NE; ++q) {
                const int e = tid + 256 * q, i = e / P, p = e % P;
                sm.Xt[p][i] = i < nv ? silu_ref(xr[q]) : 0.f;      // model.rs:310
                sm.Gt[i][p] = i < nv ? silu_ref(zr[q]) : 0.f;      // model.rs:370
            }
        }
        {
            const int k = tid & 31, sg = tid >> 5;         // angle pair k, token segment sg (8 tokens)
            float loc[8], run = 0.f;
            // this thread's 8 tokens: theta and the raw B / C pairs are requested together, ahead of any arithmetic
            float thv[8], rb8[8], rc8[8], pb0[8], pb1[8], pc0[8], pc1[8];
            const int i0k = g * N + 2 * k;
#pragma unroll
            for (int ii = 0; ii < 8; ++ii) {
                const int i = sg * 8 + ii;
                thv[ii] = 0.f; rb8[ii] = rc8[ii] = 0.f; pb0[ii] = pb1[ii] = pc0[ii] = pc1[ii] = 0.f;
                if (i < nv) {
                    const float* pr = prow0 + (size_t)(t0 + i) * R;
                    const size_t row = (size_t)b * ts + t0 + i;
                    thv[ii] = pr[off_dt + 3 * H + h * HN + k];
                    rb8[ii] = a.rb[row]; rc8[ii] = a.rc[row];
                    pb0[ii] = pr[off_b + i0k]; pb1[ii] = pr[off_b + i0k + 1];
                    pc0[ii] = pr[off_c + i0k]; pc1[ii] = pr[off_c + i0k + 1];
                }
            }
#pragma unroll
            for (int ii = 0; ii < 8; ++ii) {
                const int i = sg * 8 + ii;
                float d = 0.f;
                if (i < nv) d = __fmul_rn(sm.dtp[i], __fmul_rn(tanhf(thv[ii]), PI_F));     // model.rs:341-342
                run += d;
                loc[ii] = run;
            }
            sm.seg[sg + 1][k] = run;
            __syncthreads();
            if (tid < 32) {
                float off = sm.cum[tid];
                sm.seg[0][tid] = off;
                // reduced mod 2 pi at every segment boundary, so sums stay small and keep their low bits
                for (int s2 = 1; s2 <= 8; ++s2) { off = fmodf(off + sm.seg[s2][tid], TWO_PI); sm.seg[s2][tid] = off; }
                sm.cum[tid] = off;                         // angle after the chunk's last valid token
            }
            __syncthreads();
            const float base = sm.seg[sg][k];
#pragma unroll
            for (int ii = 0; ii < 8; ++ii) {
                const int i = sg * 8 + ii;
                float b0 = 0.f, b1 = 0.f, c0 = 0.f, c1 = 0.f;
                if (i < nv) {
                    const float rb = rb8[ii], rc = rc8[ii];
                    const float nb0 = __fadd_rn(__fmul_rn(__fmul_rn(pb0[ii], rb), kbg0), kbb0);
                    const float nb1 = __fadd_rn(__fmul_rn(__fmul_rn(pb1[ii], rb), kbg1), kbb1);
                    const float nc0 = __fadd_rn(__fmul_rn(__fmul_rn(pc0[ii], rc), kcg0), kcb0);
                    const float nc1 = __fadd_rn(__fmul_rn(__fmul_rn(pc1[ii], rc), kcg1), kcb1);
                    float sa, ca;
                    sincosf(fmodf(base + loc[ii], TWO_PI), &sa, &ca);
                    b0 = __fsub_rn(__fmul_rn(ca, nb0), __fmul_rn(sa, nb1));   // model.rs:345-348
                    b1 = __fadd_rn(__fmul_rn(sa, nb0), __fmul_rn(ca, nb1));
                    c0 = __fsub_rn(__fmul_rn(ca, nc0), __fmul_rn(sa, nc1));
                    c1 = __fadd_rn(__fmul_rn(sa, nc0), __fmul_rn(ca, nc1));
                }
                sm.Bt[i][2 * k] = b0; sm.Bt[i][2 * k + 1] = b1;
                sm.Ct[i][2 * k] = c0; sm.Ct[i][2 * k + 1] = c1;
            }
        }
        __syncthreads();
        // ---- 3. W[i][j] = (C~_i . B~_j) * decay * weight, lower triangle
        {
            const int ti = tid >> 4, tj = tid & 15;        // rows ti + 16a, cols tj + 16b
            float acc[4][4];
#pragma unroll
            for (int x = 0; x < 4; ++x)
#pragma unroll
                for (int y = 0; y < 4; ++y) acc[x][y] = 0.f;
#pragma unroll 4
            for (int n4 = 0; n4 < N / 4; ++n4) {
                float4 c4[4], b4[4];
#pragma unroll
                for (int x = 0; x < 4; ++x) c4[x] = *reinterpret_cast<const float4*>(&sm.Ct[ti + 16 * x][4 * n4]);
#pragma unroll
                for (int y = 0; y < 4; ++y) b4[y] = *reinterpret_cast<const float4*>(&sm.Bt[tj + 16 * y][4 * n4]);
#pragma unroll
                for (int x = 0; x < 4; ++x)
#pragma unroll
                    for (int y = 0; y < 4; ++y) acc[x][y] += dot4(c4[x], b4[y]);
            }
#pragma unroll
            for (int x = 0; x < 4; ++x)
#pragma unroll
                for (int y = 0; y < 4; ++y) {
                    const int i = ti + 16 * x, j = tj + 16 * y;
                    float w = 0.f;
                    if (j < i) w = acc[x][y] * expf(sm.ell[i] - sm.ell[j]) * sm.kap[j];
                    else if (j == i) w = acc[x][y] * sm.lam[i];
                    sm.Wm[i][j] = w;
                }
        }
        __syncthreads();
        // ---- 4. y = W X + e^{l_i} (C~ S^_in^T) + D x, gated                     (model.rs:365-370)
        {
            const int r = tid >> 3, c = tid & 7;           // rows r + 32a, cols c + 8b
            float yi[2][4], ys[2][4];
#pragma unroll
            for (int x = 0; x < 2; ++x)
#pragma unroll
                for (int y = 0; y < 4; ++y) { yi[x][y] = 0.f; ys[x][y] = 0.f; }
#pragma unroll 4
            for (int q = 0; q < LCH / 4; ++q) {
                float4 w4[2], x4[4], c4[2], s4[4];
#pragma unroll
                for (int x = 0; x < 2; ++x) { w4[x] = *reinterpret_cast<const float4*>(&sm.Wm[r + 32 * x][4 * q]); c4[x] = *reinterpret_cast<const float4*>(&sm.Ct[r + 32 * x][4 * q]); }
#pragma unroll
                for (int y = 0; y < 4; ++y) { x4[y] = *reinterpret_cast<const float4*>(&sm.Xt[c + 8 * y][4 * q]); s4[y] = *reinterpret_cast<const float4*>(&sm.Sh[c + 8 * y][4 * q]); }
#pragma unroll
                for (int x = 0; x < 2; ++x)
#pragma unroll
                    for (int y = 0; y < 4; ++y) { yi[x][y] += dot4(w4[x], x4[y]); ys[x][y] += dot4(c4[x], s4[y]); }
            }
#pragma unroll
            for (int x = 0; x < 2; ++x) {
                const int i = r + 32 * x;
                if (i < nv) {
                    const float el = expf(sm.ell[i]);
                    const size_t row = (size_t)b * ts + t0 + i;
#pragma unroll
                    for (int y = 0; y < 4; ++y) {
                        const int p = c + 8 * y;
                        float yv = yi[x][y] + el * ys[x][y] + dskip * sm.Xt[p][i];
                        yv *= sm.Gt[i][p];
                        const size_t o = row * DI + h * P + p;
                        __nv_bfloat16 hh, ll;
                        split_bf16(yv, hh, ll);
                        a.yhi[o] = hh;
                        if (a.ylo) a.ylo[o] = ll;
                    }
                }
            }
        }
        __syncthreads();
        // ---- 5. S^_out = e^{l_last} S^_in + sum_j wj[j] x_j (x) B~_j
        {
            const int pr = tid >> 4, n4 = tid & 15;        // rows pr + 16a, columns 4 n4 .. 4 n4 + 3
            const float el = expf(sm.ell[LCH - 1]);
            float4 acc[2];
#pragma unroll
            for (int x = 0; x < 2; ++x) {
                const float4 s = *reinterpret_cast<const float4*>(&sm.Sh[pr + 16 * x][4 * n4]);
                acc[x] = make_float4(el * s.x, el * s.y, el * s.z, el * s.w);
            }
#pragma unroll 4
            for (int j = 0; j < LCH; ++j) {
                const float4 b4 = *reinterpret_cast<const float4*>(&sm.Bt[j][4 * n4]);
                const float w = sm.wj[j];
#pragma unroll
                for (int x = 0; x < 2; ++x) {
                    const float xw = sm.Xt[pr + 16 * x][j] * w;
                    acc[x].x = fmaf(xw, b4.x, acc[x].x); acc[x].y = fmaf(xw, b4.y, acc[x].y);
                    acc[x].z = fmaf(xw, b4.z, acc[x].z); acc[x].w = fmaf(xw, b4.w, acc[x].w);
                }
            }
#pragma unroll
            for (int x = 0; x < 2; ++x) *reinterpret_cast<float4*>(&sm.Sh[pr + 16 * x][4 * n4]) = acc[x];
        }
        __syncthreads();
    }
    // ---- hand-over: the exact decode state after the last token of this launch
    for (int i = tid; i < P * N; i += 256) a.h[bh * (size_t)(P * N) + i] = sm.Sh[i / N][i % N];
    if (tid < P) a.xprev[bh * P + tid] = sm.Xt[tid][last_valid];
    if (tid < N) a.bprev[bh * N + tid] = sm.Bt[last_valid][tid];
    if (tid < HN) a.cum[bh * HN + tid] = sm.cum[tid];
}

}  // namespace

bool prefill_ssd_supported(const Config& c) { return c.head_dim() == 32 && c.d_state == 64; }

cudaError_t launch_prefill_embed(const void* emb, int dtype, const uint32_t* prompt, float* x, int D, int vocab, int rows, int ts,
                                 int t_abs0, int b_abs0, int batch_total, StepCtl* ctl, cudaStream_t st) {
    if (dtype == LUMI_DTYPE_BF16)
        embed_rows_kernel<__nv_bfloat16><<<rows, 128, 0, st>>>((const __nv_bfloat16*)emb, prompt, x, D, vocab, ts, t_abs0, b_abs0, batch_total, ctl);
    else
        embed_rows_kernel<float><<<rows, 128, 0, st>>>((const float*)emb, prompt, x, D, vocab, ts, t_abs0, b_abs0, batch_total, ctl);
    return cudaGetLastError();
}

cudaError_t launch_prefill_scan(const PrefillArgs& a, cudaStream_t st) {
    const size_t smem = sizeof(PfSmem) + 16;
    static bool set = false;
    if (!set) {
        cudaError_t e = cudaFuncSetAttribute(ssd_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        set = true;
    }
    const int rows = a.nb * a.ts;
    bc_stats_kernel<<<(rows * 32 + 255) / 256, 256, 0, st>>>(a.proj, a.ldp, 2 * a.H * 32, a.G * 64, a.eps, a.rb, a.rc, rows);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    ssd_prefill_kernel<<<dim3(a.H, a.nb), 256, smem, st>>>(a);
    return cudaGetLastError();
}

cudaError_t launch_gather_last(const float* xr, float* x, int D, int ts, int nb, int b0, cudaStream_t st) {
    gather_last_kernel<<<nb, 256, 0, st>>>(xr, x, D, ts, b0);
    return cudaGetLastError();
}

}  // namespace lumi
