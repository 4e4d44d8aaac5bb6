// Bandwidth-bound kernels of the decode step: embedding gather, RMSNorm, weight-streaming GEMV,
// the fused Mamba-3 state update, and sampling.
//
// Arithmetic follows the reference's CPU branch (inference/src/model.rs:296-375) operation by
// operation; where the reference rounds after every multiply and add (Rust never contracts to FMA),
// the round-to-nearest intrinsics below are used so the compiler cannot contract either.  Dot
// products use FMA with a fixed summation order (per-lane strided partials, xor-shuffle tree), so
// results are bit-stable from run to run.
#include "internal.h"

#include <cfloat>
#include <cmath>
#include <cstdlib>

namespace lumi {

namespace {

// Programmatic dependent launch: a kernel launched with the attribute may start while its
// predecessor still runs; everything that touches the predecessor's results comes after pdl_wait().
// Without the attribute both instructions are no-ops.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// model.rs:12-17, :830-832 and candle's silu, in the reference's operation order
__device__ __forceinline__ float sigmoid_ref(float x) { return __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-x))); }
__device__ __forceinline__ float softplus_ref(float x) { return logf(__fadd_rn(expf(x), 1.0f)); }
__device__ __forceinline__ float silu_ref(float x) { return __fdiv_rn(x, __fadd_rn(1.0f, expf(-x))); }
__device__ __forceinline__ float rms_scale(float sumsq, int n, float eps) {
    float mean = __fmul_rn(sumsq, (float)(1.0 / (double)n));
    return __frcp_rn(__fsqrt_rn(__fadd_rn(mean, eps)));
}

__device__ __forceinline__ void split_bf16(float v, __nv_bfloat16& hi, __nv_bfloat16& lo) {
    hi = __float2bfloat16_rn(v);
    lo = __float2bfloat16_rn(v - __bfloat162float(hi));
}

// ---- 16-byte weight loads ------------------------------------------------------------------------
template <typename WT> struct WLoad;
template <> struct WLoad<float> {
    static constexpr int E = 4;
    __device__ static __forceinline__ void load(const float* p, float (&w)[4]) {
        float4 v = __ldg(reinterpret_cast<const float4*>(p));
        w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w;
    }
};
template <> struct WLoad<__nv_bfloat16> {
    static constexpr int E = 8;
    __device__ static __forceinline__ void load(const __nv_bfloat16* p, float (&w)[8]) {
        uint4 v = __ldg(reinterpret_cast<const uint4*>(p));
        const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            w[2 * i] = __uint_as_float(u[i] << 16);
            w[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u);
        }
    }
};

// ---- embedding gather (model.rs:772-773) -----------------------------------------------------------
template <typename WT>
__global__ void embed_kernel(const WT* __restrict__ emb, const uint32_t* __restrict__ tok_cur, float* __restrict__ x,
                             int D, int vocab, StepCtl* ctl) {
    const int b = blockIdx.x;
    pdl_launch_dependents();
    pdl_wait();
    // during prefill the token comes from the uploaded prompt, afterwards from the last sampled one
    const int pp = ctl->prompt_pos;
    uint32_t t = (pp < ctl->prompt_len) ? ctl->prompt[(size_t)pp * ctl->batch + b] : tok_cur[b];
    if (t >= (uint32_t)vocab) {          // reported to the host; the row read stays in bounds
        if (threadIdx.x == 0) atomicOr(&ctl->status, STATUS_BAD_TOKEN);
        t = 0;
    }
    constexpr int E = WLoad<WT>::E;
    const WT* row = emb + (size_t)t * D;
    for (int c = threadIdx.x; c < D / E; c += blockDim.x) {
        float w[E];
        WLoad<WT>::load(row + c * E, w);
#pragma unroll
        for (int e = 0; e < E; ++e) x[(size_t)b * D + c * E + e] = w[e];
    }
}

// ---- RMSNorm to bf16 halves for the tensor-core GEMMs (model.rs:100-106) ---------------------------
__global__ void __launch_bounds__(256) norm_split_kernel(const float* __restrict__ x, const float* __restrict__ gamma,
                                                         __nv_bfloat16* __restrict__ hi, __nv_bfloat16* __restrict__ lo,
                                                         int D, float eps) {
    __shared__ float red[8];
    const int b = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    pdl_launch_dependents();
    pdl_wait();
    const float* xr = x + (size_t)b * D;
    float r = 1.0f;
    if (gamma) {
        float s = 0.f;
        for (int i = threadIdx.x; i < D; i += 256) s = fmaf(xr[i], xr[i], s);
        s = warp_sum(s);
        if (lane == 0) red[warp] = s;
        __syncthreads();
        float t = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) t += red[w];
        r = rms_scale(t, D, eps);
    }
    for (int i = threadIdx.x; i < D; i += 256) {
        float v = xr[i];
        if (gamma) v = __fmul_rn(__fmul_rn(v, r), gamma[i]);
        __nv_bfloat16 h, l;
        split_bf16(v, h, l);
        hi[(size_t)b * D + i] = h;
        if (lo) lo[(size_t)b * D + i] = l;
    }
}

// ---- weight-streaming GEMV for small batches ---------------------------------------------------------
// D[m][n] = sum_k A'[m][k] W[n][k] (+ R[m][n]),  A' = RMSNorm(A; gamma) when gamma != null.
//
// A warp owns RPW output rows and one K segment of them (KSEG = 32 lanes x U chunks of 16 bytes).
// It loads its whole share of the weights into registers FIRST — before the dependent-launch wait
// and before the activation prologue — so the HBM stream of this kernel overlaps its predecessor
// and its own prologue.  Rows longer than one segment are split over KS warps of the same CTA and
// combined through shared memory in segment order (fixed summation order: per-lane partials in
// ascending k, 5-step xor tree, then segments 0..KS-1).
constexpr int kGemvU = 8;

template <typename WT> struct WRaw;      // 16 raw bytes -> floats
template <> struct WRaw<float> {
    __device__ static __forceinline__ void cvt(const uint4& v, float (&w)[4]) {
        w[0] = __uint_as_float(v.x); w[1] = __uint_as_float(v.y); w[2] = __uint_as_float(v.z); w[3] = __uint_as_float(v.w);
    }
};
template <> struct WRaw<__nv_bfloat16> {
    __device__ static __forceinline__ void cvt(const uint4& v, float (&w)[8]) {
        const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) { w[2 * i] = __uint_as_float(u[i] << 16); w[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u); }
    }
};

template <typename WT, int NB, int RPW, int ACT>
__global__ void __launch_bounds__(256) gemv_kernel(const float* __restrict__ A, int lda, const WT* __restrict__ W,
                                                   float* __restrict__ D, int ldd, const float* __restrict__ R,
                                                   const float* __restrict__ gamma, int M, int N, int K, float eps, int KS) {
    extern __shared__ float4 gemv_smem4[];
    float* xs = reinterpret_cast<float*>(gemv_smem4);
    constexpr int E = WLoad<WT>::E;
    constexpr int U = kGemvU;
    constexpr int NR = (ACT == 1) ? 2 * RPW : RPW;     // ACT == 1 pairs weight rows n (gate) and n + N (up)
    __shared__ float part[8][NR][NB];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m0 = blockIdx.y * NB;
    const int nb = min(NB, M - m0);
    const int K4 = K >> 2, KC = K / E;
    const int gpc = 8 / KS;                             // row groups per CTA
    const int g = warp / KS, seg = warp - g * KS;
    const int row0 = (blockIdx.x * gpc + g) * RPW;
    const int c0 = seg * 32 * U + lane;                 // this lane's first 16-byte chunk

    pdl_launch_dependents();
    // the weights do not depend on the previous kernel: all loads go out before waiting for it
    uint4 wreg[NR][U];
#pragma unroll
    for (int r = 0; r < NR; ++r) {
        const int row = min(row0 + (r % RPW), N - 1) + ((ACT == 1 && r >= RPW) ? N : 0);
        const WT* wp = W + (size_t)row * K;
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int c = c0 + 32 * u;
            wreg[r][u] = (c < KC && row0 < N) ? __ldg(reinterpret_cast<const uint4*>(wp + (size_t)c * E)) : make_uint4(0u, 0u, 0u, 0u);
        }
    }
    pdl_wait();

    for (int i = threadIdx.x; i < NB * K4; i += 256) {
        int b = i / K4, k4 = i - b * K4;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (b < nb) v = *reinterpret_cast<const float4*>(A + (size_t)(m0 + b) * lda + 4 * k4);
        reinterpret_cast<float4*>(xs)[i] = v;
    }
    __syncthreads();
    if (gamma != nullptr) {
        // RMSNorm of the NB staged rows by the whole CTA: per-thread partials in ascending k, xor tree,
        // then the 8 warp sums in warp order
        __shared__ float nred[NB][8];
#pragma unroll
        for (int b = 0; b < NB; ++b) {
            float s = 0.f;
            if (b < nb) for (int k = threadIdx.x; k < K; k += 256) s = fmaf(xs[b * K + k], xs[b * K + k], s);
            s = warp_sum(s);
            if (lane == 0) nred[b][warp] = s;
        }
        __syncthreads();
#pragma unroll
        for (int b = 0; b < NB; ++b) {
            if (b < nb) {
                float t = 0.f;
#pragma unroll
                for (int w = 0; w < 8; ++w) t += nred[b][w];
                const float r = rms_scale(t, K, eps);
                for (int k = threadIdx.x; k < K; k += 256) xs[b * K + k] = __fmul_rn(__fmul_rn(xs[b * K + k], r), gamma[k]);
            }
        }
        __syncthreads();
    }
    float acc[NR][NB];
#pragma unroll
    for (int r = 0; r < NR; ++r)
#pragma unroll
        for (int b = 0; b < NB; ++b) acc[r][b] = 0.f;
#pragma unroll
    for (int u = 0; u < U; ++u) {
        const int c = c0 + 32 * u;
        if (c < KC) {
            float w[NR][E];
#pragma unroll
            for (int r = 0; r < NR; ++r) WRaw<WT>::cvt(wreg[r][u], w[r]);
#pragma unroll
            for (int b = 0; b < NB; ++b) {
                float xv[E];
#pragma unroll
                for (int q = 0; q < E / 4; ++q) {
                    float4 v = *reinterpret_cast<const float4*>(xs + b * K + c * E + 4 * q);
                    xv[4 * q] = v.x; xv[4 * q + 1] = v.y; xv[4 * q + 2] = v.z; xv[4 * q + 3] = v.w;
                }
#pragma unroll
                for (int r = 0; r < NR; ++r)
#pragma unroll
                    for (int e = 0; e < E; ++e) acc[r][b] = fmaf(w[r][e], xv[e], acc[r][b]);
            }
        }
    }
#pragma unroll
    for (int r = 0; r < NR; ++r)
#pragma unroll
        for (int b = 0; b < NB; ++b) acc[r][b] = warp_sum(acc[r][b]);
    if (KS > 1) {
        if (lane == 0) {
#pragma unroll
            for (int r = 0; r < NR; ++r)
#pragma unroll
                for (int b = 0; b < NB; ++b) part[warp][r][b] = acc[r][b];
        }
        __syncthreads();
        if (seg != 0) return;
#pragma unroll
        for (int r = 0; r < NR; ++r)
#pragma unroll
            for (int b = 0; b < NB; ++b) {
                float t = part[warp][r][b];
                for (int sg = 1; sg < KS; ++sg) t += part[warp + sg][r][b];
                acc[r][b] = t;
            }
    }
    if (lane == 0 && row0 < N) {
#pragma unroll
        for (int r = 0; r < RPW; ++r) {
            int row = row0 + r;
            if (row >= N) break;
#pragma unroll
            for (int b = 0; b < NB; ++b) {
                if (b >= nb) break;
                float v = acc[r][b];
                if constexpr (ACT == 1) v = __fmul_rn(sigmoid_ref(v), acc[RPW + r][b]);     // model.rs:550-552
                size_t o = (size_t)(m0 + b) * ldd + row;
                if (R != nullptr) v = __fadd_rn(v, R[o]);
                D[o] = v;
            }
        }
    }
}

// ---- fused Mamba-3 decode step ---------------------------------------------------------------------
// One warp per (sequence, head).  Prologue: BCNorm statistics over all n_groups*d_state elements
// (block-wide), per-head scalars, DD-RoPE with one rotation pair per lane, staged in shared memory.
// Main loop: the head's [P][N] fp32 state tile as consecutive float4 (lane-contiguous, coalesced);
// prev_bx is rebuilt from its rank-1 factors x_prev (x) B_prev, which are what is kept in HBM.
template <int P, int N>
struct SsmSmem {
    float bt[N], ct[N], xa[P], xp[P], gate[P], yout[P];
};

// WPH warps share one head: each owns P / WPH consecutive state rows.  WPH = 1 at large batch (a
// warp streams a whole 8 KiB tile); WPH = 4 at small batch, where the tile compute of one warp
// would otherwise sit on the critical path of the token.
template <int P, int N, int WPH, int MINB>
__global__ void __launch_bounds__(256, MINB) ssm_step_kernel(SsmArgs a) {
    __shared__ SsmSmem<P, N> sm_all[8];
    __shared__ float red[2][8];
    constexpr int CG = N / 4;              // lanes sharing one state row
    constexpr int RS = 32 / CG;            // state rows covered by one warp-wide float4 access
    constexpr int IT = P / RS;             // accesses per tile
    constexpr int ITW = IT / WPH;          // accesses per warp
    constexpr int CH = ITW < 16 ? ITW : 16;
    constexpr int ROWS = P / WPH;          // rows per warp
    static_assert(IT % WPH == 0 && ITW >= 1, "rows must split evenly over the warps of a head");
    const int b = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nwarp = blockDim.x >> 5;
    const int hpb = nwarp / WPH;
    const int hl = warp / WPH, sub = warp - hl * WPH;
    const int h = blockIdx.x * hpb + hl;
    const int H = a.H, DI = H * P, BC = a.G * N, HN = N / 2;
    const bool active = h < H;
    const size_t bh = (size_t)b * H + (active ? h : H - 1);
    const int c = lane % CG, r0 = lane / CG;

    pdl_launch_dependents();
    // State is only ever written by this same kernel one token earlier, and every step starts with a
    // kernel that is not launched early, so the whole previous step has finished before this line:
    // the state can be requested ahead of the dependency wait and its HBM latency runs under the
    // predecessor's tail and the prologue below.
    float4* h4 = reinterpret_cast<float4*>(a.h + bh * (size_t)(P * N)) + (size_t)sub * ITW * 32;
    float4 t[CH];
    float4 bpq = make_float4(0.f, 0.f, 0.f, 0.f);
    float cu_old[(HN + 31) / 32];
    if (active) {
#pragma unroll
        for (int i = 0; i < CH; ++i) t[i] = h4[i * 32 + lane];
        bpq = reinterpret_cast<const float4*>(a.bprev + bh * N)[c];
#pragma unroll
        for (int j = 0; j < (HN + 31) / 32; ++j) cu_old[j] = (lane + 32 * j < HN) ? a.cum[bh * HN + lane + 32 * j] : 0.f;
    }
    pdl_wait();

    const float* pr = a.proj + (size_t)b * a.ldp;
    const float* Bp = pr + 2 * DI;
    const float* Cp = Bp + BC;
    const float* dt = Cp + BC;
    const float* lam_raw = dt + H;
    const float* dda = dt + 2 * H;
    const float* theta = dt + 3 * H;
    const int hh = active ? h : H - 1;
    const int g = hh / (H / a.G);

    // every global value the prologue needs is requested here, ahead of the block barrier, so the
    // loads overlap instead of forming a chain of round trips
    const float v_dt = dt[hh], v_dtb = a.dtb[hh], v_dda = dda[hh], v_lam = lam_raw[hh], v_dskip = a.dskip[hh];
    constexpr int NJ = (N / 2 + 31) / 32;
    float v_th[NJ], v_b0[NJ], v_b1[NJ], v_c0[NJ], v_c1[NJ], g_b0[NJ], g_b1[NJ], g_c0[NJ], g_c1[NJ], o_b0[NJ], o_b1[NJ], o_c0[NJ], o_c1[NJ];
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
        const int k = min(lane + 32 * j, HN - 1);
        const int i0 = g * N + 2 * k;
        v_th[j] = theta[hh * HN + k];
        v_b0[j] = Bp[i0]; v_b1[j] = Bp[i0 + 1]; v_c0[j] = Cp[i0]; v_c1[j] = Cp[i0 + 1];
        g_b0[j] = a.bg[i0]; g_b1[j] = a.bg[i0 + 1]; g_c0[j] = a.cg[i0]; g_c1[j] = a.cg[i0 + 1];
        o_b0[j] = a.bb[i0]; o_b1[j] = a.bb[i0 + 1]; o_c0[j] = a.cb[i0]; o_c1[j] = a.cb[i0 + 1];
    }
    constexpr int ROWS_PL = (P / WPH + 31) / 32;
    float v_x[ROWS_PL], v_z[ROWS_PL], v_xp[ROWS_PL];
#pragma unroll
    for (int j = 0; j < ROWS_PL; ++j) {
        const int row = min(sub * ROWS + lane + 32 * j, P - 1);
        v_x[j] = pr[hh * P + row];
        v_z[j] = pr[DI + hh * P + row];
        v_xp[j] = a.xprev[bh * P + row];
    }

    // BCNorm statistics (model.rs:311-312: the norm runs over the whole bc vector)
    float sb = 0.f, sc = 0.f;
    for (int i = threadIdx.x; i < BC; i += blockDim.x) {
        float v = Bp[i];
        sb = fmaf(v, v, sb);
        v = Cp[i];
        sc = fmaf(v, v, sc);
    }
    sb = warp_sum(sb);
    sc = warp_sum(sc);
    if (lane == 0) { red[0][warp] = sb; red[1][warp] = sc; }
    __syncthreads();       // also orders every warp's reads of bprev / cum / xprev above before the writes below
    if (!active) return;
    float tb = 0.f, tc = 0.f;
    for (int w = 0; w < nwarp; ++w) { tb += red[0][w]; tc += red[1][w]; }
    const float rb = rms_scale(tb, BC, a.eps), rc = rms_scale(tc, BC, a.eps);

    SsmSmem<P, N>& sm = sm_all[warp];

    // per-head scalars (model.rs:307, 314-317, 355-359)
    const float dtp = softplus_ref(__fadd_rn(v_dt, v_dtb));
    float av = -softplus_ref(v_dda);
    av = fminf(fmaxf(av, -1e6f), -1e-4f);
    const float abar = expf(__fmul_rn(av, dtp));
    const float lam = sigmoid_ref(v_lam);
    const float oml = __fadd_rn(__fmul_rn(lam, -1.0f), 1.0f);
    const float c2 = __fmul_rn(abar, oml);

    // DD-RoPE (model.rs:338-350): lane k rotates pair (2k, 2k+1) of the normalised B and C
    const float PI_F = 3.14159265358979323846f;
    const float TWO_PI = __fmul_rn(2.0f, PI_F);
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
        const int k = lane + 32 * j;
        if (k < HN) {
            float angle = __fmul_rn(tanhf(v_th[j]), PI_F);
            float cu = fmodf(__fadd_rn(cu_old[j], __fmul_rn(dtp, angle)), TWO_PI);
            if (sub == 0) a.cum[bh * HN + k] = cu;
            float sa, ca;
            sincosf(cu, &sa, &ca);
            float b0 = __fadd_rn(__fmul_rn(__fmul_rn(v_b0[j], rb), g_b0[j]), o_b0[j]);
            float b1 = __fadd_rn(__fmul_rn(__fmul_rn(v_b1[j], rb), g_b1[j]), o_b1[j]);
            float c0 = __fadd_rn(__fmul_rn(__fmul_rn(v_c0[j], rc), g_c0[j]), o_c0[j]);
            float c1 = __fadd_rn(__fmul_rn(__fmul_rn(v_c1[j], rc), g_c1[j]), o_c1[j]);
            sm.bt[2 * k] = __fsub_rn(__fmul_rn(ca, b0), __fmul_rn(sa, b1));
            sm.bt[2 * k + 1] = __fadd_rn(__fmul_rn(sa, b0), __fmul_rn(ca, b1));
            sm.ct[2 * k] = __fsub_rn(__fmul_rn(ca, c0), __fmul_rn(sa, c1));
            sm.ct[2 * k + 1] = __fadd_rn(__fmul_rn(sa, c0), __fmul_rn(ca, c1));
        }
    }
    const int prow0 = sub * ROWS;          // first state row of this warp
#pragma unroll
    for (int j = 0; j < ROWS_PL; ++j) {
        const int p = lane + 32 * j;
        if (p < ROWS) {
            const int row = prow0 + p;
            sm.xa[row] = silu_ref(v_x[j]);                  // model.rs:310
            sm.xp[row] = v_xp[j];
            sm.gate[row] = silu_ref(v_z[j]);                // model.rs:370
        }
    }
    __syncwarp();

    const float4 bq = reinterpret_cast<const float4*>(sm.bt)[c];
    const float4 cq = reinterpret_cast<const float4*>(sm.ct)[c];
#pragma unroll 1
    for (int i0 = 0; i0 < ITW; i0 += CH) {
        if (i0 > 0) {
#pragma unroll
            for (int i = 0; i < CH; ++i) t[i] = h4[(i0 + i) * 32 + lane];
        }
#pragma unroll
        for (int i = 0; i < CH; ++i) {
            const int row = r0 + (sub * ITW + i0 + i) * RS;
            const float xv = sm.xa[row], xpv = sm.xp[row];
            float part;
            {   // model.rs:354-366 : h = (abar*h + (abar*(1-lam))*prev_bx) + lam*bx ; y = sum_s C~[s] h[s]
                float nh;
                nh = __fadd_rn(__fadd_rn(__fmul_rn(abar, t[i].x), __fmul_rn(c2, __fmul_rn(xpv, bpq.x))), __fmul_rn(lam, __fmul_rn(xv, bq.x)));
                t[i].x = nh; part = __fmul_rn(cq.x, nh);
                nh = __fadd_rn(__fadd_rn(__fmul_rn(abar, t[i].y), __fmul_rn(c2, __fmul_rn(xpv, bpq.y))), __fmul_rn(lam, __fmul_rn(xv, bq.y)));
                t[i].y = nh; part = fmaf(cq.y, nh, part);
                nh = __fadd_rn(__fadd_rn(__fmul_rn(abar, t[i].z), __fmul_rn(c2, __fmul_rn(xpv, bpq.z))), __fmul_rn(lam, __fmul_rn(xv, bq.z)));
                t[i].z = nh; part = fmaf(cq.z, nh, part);
                nh = __fadd_rn(__fadd_rn(__fmul_rn(abar, t[i].w), __fmul_rn(c2, __fmul_rn(xpv, bpq.w))), __fmul_rn(lam, __fmul_rn(xv, bq.w)));
                t[i].w = nh; part = fmaf(cq.w, nh, part);
            }
            h4[(i0 + i) * 32 + lane] = t[i];
#pragma unroll
            for (int o = CG / 2; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
            if (c == 0) sm.yout[row] = part;
        }
    }
    __syncwarp();
    for (int p = lane; p < ROWS; p += 32) {
        const int row = prow0 + p;
        float xv = sm.xa[row];
        float yv = __fadd_rn(sm.yout[row], __fmul_rn(v_dskip, xv));   // model.rs:367-368
        yv = __fmul_rn(yv, sm.gate[row]);                                // model.rs:370
        const size_t o = (size_t)b * DI + h * P + row;
        if (a.y32) a.y32[o] = yv;
        if (a.yhi) {
            __nv_bfloat16 hh, ll;
            split_bf16(yv, hh, ll);
            a.yhi[o] = hh;
            if (a.ylo) a.ylo[o] = ll;
        }
        a.xprev[bh * P + row] = xv;
    }
    if (sub == 0)
        for (int s2 = lane; s2 < N; s2 += 32) a.bprev[bh * N + s2] = sm.bt[s2];
}

// h <- h_init broadcast over head_dim (model.rs:744-748); factors and angles <- 0 (:751-752)
__global__ void state_reset_kernel(float* h, float* xprev, float* bprev, float* cum, const float* __restrict__ h_init,
                                   const int32_t* __restrict__ slots, int H, int P, int N) {
    const int slot = slots ? slots[blockIdx.x] : blockIdx.x;
    const size_t per = (size_t)H * P * N;
    for (size_t i = threadIdx.x; i < per; i += blockDim.x) {
        int n = i % N;
        int hh = i / ((size_t)P * N);
        h[(size_t)slot * per + i] = h_init ? h_init[hh * N + n] : 0.f;
    }
    for (int i = threadIdx.x; i < H * P; i += blockDim.x) xprev[(size_t)slot * H * P + i] = 0.f;
    for (int i = threadIdx.x; i < H * N; i += blockDim.x) bprev[(size_t)slot * H * N + i] = 0.f;
    for (int i = threadIdx.x; i < H * N / 2; i += blockDim.x) cum[(size_t)slot * H * (N / 2) + i] = 0.f;
}

// ---- sampling (main.rs:142-148, 197-209) -----------------------------------------------------------
__device__ __forceinline__ void philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint32_t k0, uint32_t k1,
                                              uint32_t& o0) {
#pragma unroll
    for (int i = 0; i < 10; ++i) {
        uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
        uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
        uint32_t n0 = hi1 ^ c1 ^ k0, n1 = lo1, n2 = hi0 ^ c3 ^ k1, n3 = lo0;
        c0 = n0; c1 = n1; c2 = n2; c3 = n3;
        k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
    }
    o0 = c0;
}

struct BestPair { float v; int i; };
__device__ __forceinline__ bool better(float v, int i, float bv, int bi) { return v > bv || (v == bv && i < bi); }

__device__ BestPair block_argmax(float v, int i, BestPair* red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, v, o);
        int oi = __shfl_xor_sync(0xffffffffu, i, o);
        if (better(ov, oi, v, i)) { v = ov; i = oi; }
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    __syncthreads();                       // red may still be read from a previous round
    if (lane == 0) { red[warp].v = v; red[warp].i = i; }
    __syncthreads();
    BestPair r = red[0];
    for (int w = 1; w < nw; ++w) if (better(red[w].v, red[w].i, r.v, r.i)) r = red[w];
    return r;
}

constexpr int kMaxTopK = 256;

// One block per sequence.  Greedy: argmax with the lowest index on ties.  Otherwise temperature
// softmax over the top-k survivors (or the whole vocabulary) and the walk over the cumulative
// distribution in vocabulary order.
__global__ void __launch_bounds__(1024) sample_kernel(const float* __restrict__ logits, int V, StepCtl* ctl,
                                                      uint32_t* tok_cur, int32_t* finished, int32_t* out_len) {
    __shared__ BestPair red[32];
    __shared__ float top_v[kMaxTopK];
    __shared__ int top_i[kMaxTopK];
    __shared__ float chunk_sum[1024];
    __shared__ int result;
    const int b = blockIdx.x, tid = threadIdx.x, nt = blockDim.x;
    pdl_launch_dependents();
    pdl_wait();
    const float* lg = logits + (size_t)b * V;
    const int step = ctl->step;
    if (ctl->want_dump) {
        float* d = ctl->dump + ((size_t)step * ctl->batch + b) * V;
        for (int i = tid; i < V; i += nt) d[i] = lg[i];
    }
    const float temperature = ctl->temperature;
    int chosen;
    if (temperature <= 0.f) {
        float bv = -INFINITY; int bi = 0x7fffffff;
        for (int i = tid; i < V; i += nt) { float v = lg[i]; if (better(v, i, bv, bi)) { bv = v; bi = i; } }
        BestPair r = block_argmax(bv, bi, red);
        chosen = r.i;
    } else {
        const float inv_t = (float)(1.0 / (double)temperature);
        uint32_t rw;
        philox4x32_10((uint32_t)step, (uint32_t)b, 0u, 0u, ctl->seed_lo, ctl->seed_hi, rw);
        const float r = (float)(rw >> 8) * (1.0f / 16777216.0f);
        int k = ctl->top_k;
        if (k > kMaxTopK) k = kMaxTopK;
        if (k > 0 && k < V) {
            // k rounds of block-wide argmax over the not-yet-taken entries
            for (int round = 0; round < k; ++round) {
                float bv = -INFINITY; int bi = 0x7fffffff;
                for (int i = tid; i < V; i += nt) {
                    float v = lg[i];
                    bool taken = false;
                    if (round > 0) {
                        // an entry is taken iff it is at least as good as the last survivor
                        float lv = top_v[round - 1]; int li = top_i[round - 1];
                        taken = !better(lv, li, v, i);
                    }
                    if (!taken && better(v, i, bv, bi)) { bv = v; bi = i; }
                }
                BestPair rr = block_argmax(bv, bi, red);
                if (tid == 0) { top_v[round] = rr.v; top_i[round] = rr.i; }
                __syncthreads();
            }
            if (tid == 0) {
                // survivors into vocabulary order (insertion sort, k <= 256)
                for (int a1 = 1; a1 < k; ++a1) {
                    float v = top_v[a1]; int i = top_i[a1]; int j = a1 - 1;
                    while (j >= 0 && top_i[j] > i) { top_v[j + 1] = top_v[j]; top_i[j + 1] = top_i[j]; --j; }
                    top_v[j + 1] = v; top_i[j + 1] = i;
                }
                float mx = -INFINITY;
                for (int j = 0; j < k; ++j) { top_v[j] = __fmul_rn(top_v[j], inv_t); mx = fmaxf(mx, top_v[j]); }
                float sum = 0.f;
                for (int j = 0; j < k; ++j) { top_v[j] = expf(__fsub_rn(top_v[j], mx)); sum = __fadd_rn(sum, top_v[j]); }
                float cum = 0.f; int pick = top_i[k - 1];
                for (int j = 0; j < k; ++j) {
                    cum = __fadd_rn(cum, __fdiv_rn(top_v[j], sum));
                    if (cum >= r) { pick = top_i[j]; break; }
                }
                result = pick;
            }
            __syncthreads();
            chosen = result;
        } else {
            // whole vocabulary: each thread owns a contiguous chunk; chunk sums are combined in
            // chunk order, so the cumulative sums differ from a single sequential pass only by rounding
            float bv = -INFINITY; int bi = 0x7fffffff;
            for (int i = tid; i < V; i += nt) { float v = __fmul_rn(lg[i], inv_t); if (better(v, i, bv, bi)) { bv = v; bi = i; } }
            const float mx = block_argmax(bv, bi, red).v;
            const int per = (V + nt - 1) / nt;
            const int lo = tid * per, hi = min(V, lo + per);
            float s = 0.f;
            for (int i = lo; i < hi; ++i) s = __fadd_rn(s, expf(__fsub_rn(__fmul_rn(lg[i], inv_t), mx)));
            chunk_sum[tid] = s;
            if (tid == 0) result = V - 1;
            __syncthreads();
            float total = 0.f, before = 0.f;
            for (int t = 0; t < nt; ++t) { if (t == tid) before = total; total = __fadd_rn(total, chunk_sum[t]); }
            float cum = __fdiv_rn(before, total);
            for (int i = lo; i < hi; ++i) {
                cum = __fadd_rn(cum, __fdiv_rn(expf(__fsub_rn(__fmul_rn(lg[i], inv_t), mx)), total));
                if (cum >= r) { atomicMin(&result, i); break; }
            }
            __syncthreads();
            chosen = result;
        }
    }
    if (tid == 0) {
        tok_cur[b] = (uint32_t)chosen;
        if (ctl->record) {
            ctl->out_tokens[(size_t)step * ctl->batch + b] = (uint32_t)chosen;
            if (!finished[b]) {
                if ((uint32_t)chosen == ctl->eos_id && !ctl->ignore_eos) finished[b] = 1;   // main.rs:150
                else out_len[b] += 1;
            }
        }
    }
}

// End of a step: next prompt position / next output row, and one more cached token per sequence.
__global__ void advance_step_kernel(StepCtl* ctl, int32_t* kv_pos, int B, int sampled) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    pdl_launch_dependents();
    pdl_wait();
    if (kv_pos != nullptr && i < B) kv_pos[i] += 1;
    if (i == 0) {
        if (ctl->prompt_pos < ctl->prompt_len) ctl->prompt_pos += 1;
        if (sampled) ctl->step += 1;
    }
}

// D = sigmoid(gate) * up for the attention block's MLP (model.rs:550-552); gu = [gate | up] per row
__global__ void gate_mul_kernel(const float* __restrict__ gu, int ld, float* out32, __nv_bfloat16* hi, __nv_bfloat16* lo,
                                int mlp) {
    const int b = blockIdx.y;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    pdl_launch_dependents();
    pdl_wait();
    if (i >= mlp) return;
    float v = __fmul_rn(sigmoid_ref(gu[(size_t)b * ld + i]), gu[(size_t)b * ld + mlp + i]);
    if (out32) out32[(size_t)b * mlp + i] = v;
    if (hi) {
        __nv_bfloat16 hh, ll;
        split_bf16(v, hh, ll);
        hi[(size_t)b * mlp + i] = hh;
        if (lo) lo[(size_t)b * mlp + i] = ll;
    }
}

}  // namespace

// ---- launchers -------------------------------------------------------------------------------------
static thread_local bool g_pdl = false;
void set_launch_pdl(bool on) { g_pdl = on; }

// Launch with (optionally) the programmatic-stream-serialization attribute.
template <typename... KArgs, typename... Args>
static cudaError_t launch_k(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
}

cudaError_t launch_embed(const void* emb, int dtype, const uint32_t* tok_cur, float* x, int B, int D, int vocab,
                         StepCtl* ctl, cudaStream_t st) {
    // The first kernel of a step is never launched early: it starts only when the previous step has
    // completely finished, which is what lets later kernels of this step read state ahead of their
    // own dependency wait.
    const bool keep = g_pdl;
    g_pdl = false;
    cudaError_t e;
    if (dtype == LUMI_DTYPE_BF16)
        e = launch_k(embed_kernel<__nv_bfloat16>, dim3(B), dim3(128), 0, st, (const __nv_bfloat16*)emb, tok_cur, x, D, vocab, ctl);
    else
        e = launch_k(embed_kernel<float>, dim3(B), dim3(128), 0, st, (const float*)emb, tok_cur, x, D, vocab, ctl);
    g_pdl = keep;
    return e;
}

cudaError_t launch_norm_split(const float* x, const float* gamma, __nv_bfloat16* hi, __nv_bfloat16* lo, int B, int D,
                              float eps, cudaStream_t st) {
    return launch_k(norm_split_kernel, dim3(B), dim3(256), 0, st, x, gamma, hi, lo, D, eps);
}

template <typename WT, int NB, int RPW, int ACT>
static cudaError_t gemv_launch(const GemvArgs& a, int KS, cudaStream_t st) {
    auto kern = gemv_kernel<WT, NB, RPW, ACT>;
    size_t smem = (size_t)NB * a.K * sizeof(float);
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
    }
    const int rows_per_cta = (8 / KS) * RPW;
    dim3 grid((a.N + rows_per_cta - 1) / rows_per_cta, (a.M + NB - 1) / NB);
    return launch_k(kern, grid, dim3(256), smem, st, a.A, a.lda, (const WT*)a.W, a.D, a.ldd, a.R, a.gamma, a.M, a.N, a.K, a.eps, KS);
}

template <typename WT, int NB, int ACT>
static cudaError_t gemv_dispatch(const GemvArgs& a, cudaStream_t st) {
    constexpr int E = WLoad<WT>::E;
    const int kseg = 32 * kGemvU * E;
    int KS = 1;
    while (KS < 8 && KS * kseg < a.K) KS *= 2;
    if (KS * kseg < a.K) return cudaErrorInvalidValue;          // K beyond 8 segments per row
    // two rows per warp only when that still leaves at least two CTAs per SM
    if (ACT == 0 && NB <= 4 && (long)a.N / ((8 / KS) * 2) >= 296) return gemv_launch<WT, NB, 2, ACT>(a, KS, st);
    return gemv_launch<WT, NB, 1, ACT>(a, KS, st);
}

template <typename WT>
static cudaError_t gemv_by_batch(const GemvArgs& a, cudaStream_t st) {
    if (a.act == 1) {
        if (a.M <= 1) return gemv_dispatch<WT, 1, 1>(a, st);
        if (a.M <= 2) return gemv_dispatch<WT, 2, 1>(a, st);
        return gemv_dispatch<WT, 4, 1>(a, st);
    }
    if (a.M <= 1) return gemv_dispatch<WT, 1, 0>(a, st);
    if (a.M <= 2) return gemv_dispatch<WT, 2, 0>(a, st);
    if (a.M <= 4) return gemv_dispatch<WT, 4, 0>(a, st);
    return gemv_dispatch<WT, 8, 0>(a, st);
}

cudaError_t launch_gemv(const GemvArgs& a, cudaStream_t st) {
    if (a.w_dtype == LUMI_DTYPE_BF16) return gemv_by_batch<__nv_bfloat16>(a, st);
    return gemv_by_batch<float>(a, st);
}

bool ssm_shape_supported(int P, int N) {
    return (P == 16 || P == 32 || P == 64) && (N == 16 || N == 32 || N == 64 || N == 128);
}

template <int P, int N, int WPH, int MINB>
static cudaError_t ssm_variant(const SsmArgs& a, cudaStream_t st) {
    int hpb = 8 / WPH;
    if (hpb > a.H) hpb = a.H;
    dim3 grid((a.H + hpb - 1) / hpb, a.B);
    return launch_k(ssm_step_kernel<P, N, WPH, MINB>, grid, dim3(hpb * WPH * 32), 0, st, a);
}

// LUMI_SSM_VARIANT (tuning aid): warps per head x minimum resident blocks per SM for the
// large-batch launch of the 32 x 64 tile; 0 / unset = the default choice.
static int ssm_variant_env() {
    static int v = -1;
    if (v < 0) { const char* e = getenv("LUMI_SSM_VARIANT"); v = e ? atoi(e) : 0; }
    return v;
}

template <int P, int N>
static cudaError_t ssm_launch(const SsmArgs& a, cudaStream_t st) {
    constexpr int IT = P / (128 / N);
    if constexpr (IT % 4 == 0) {
        if (a.B <= 8) {        // small batch: four warps per head, two heads per CTA
            int hpb = a.H < 2 ? a.H : 2;
            dim3 grid((a.H + hpb - 1) / hpb, a.B);
            return launch_k(ssm_step_kernel<P, N, 4, 3>, grid, dim3(hpb * 4 * 32), 0, st, a);
        }
    }
    if constexpr (P == 32 && N == 64) {
        switch (ssm_variant_env()) {
            case 1: return ssm_variant<P, N, 1, 2>(a, st);
            case 2: return ssm_variant<P, N, 2, 3>(a, st);
            case 3: return ssm_variant<P, N, 2, 4>(a, st);
            case 4: return ssm_variant<P, N, 4, 4>(a, st);
            case 5: return ssm_variant<P, N, 4, 3>(a, st);
            case 6: return ssm_variant<P, N, 1, 3>(a, st);
            default: break;
        }
    }
    return ssm_variant<P, N, 1, 2>(a, st);
}

cudaError_t launch_ssm_step(const SsmArgs& a, cudaStream_t st) {
#define LUMI_SSM_CASE(PP, NN) if (a.P == PP && a.N == NN) return ssm_launch<PP, NN>(a, st);
    LUMI_SSM_CASE(32, 64) LUMI_SSM_CASE(32, 16) LUMI_SSM_CASE(32, 32) LUMI_SSM_CASE(32, 128)
    LUMI_SSM_CASE(16, 16) LUMI_SSM_CASE(16, 32) LUMI_SSM_CASE(16, 64) LUMI_SSM_CASE(16, 128)
    LUMI_SSM_CASE(64, 16) LUMI_SSM_CASE(64, 32) LUMI_SSM_CASE(64, 64) LUMI_SSM_CASE(64, 128)
#undef LUMI_SSM_CASE
    return cudaErrorInvalidValue;
}

cudaError_t launch_state_reset(float* h, float* xprev, float* bprev, float* cum, const float* h_init, const int32_t* slots,
                               int n_slots, int H, int P, int N, cudaStream_t st) {
    state_reset_kernel<<<n_slots, 256, 0, st>>>(h, xprev, bprev, cum, h_init, slots, H, P, N);
    return cudaGetLastError();
}

cudaError_t launch_sample(const float* logits, int B, int V, StepCtl* ctl, uint32_t* tok_cur, int32_t* finished,
                          int32_t* out_len, cudaStream_t st) {
    return launch_k(sample_kernel, dim3(B), dim3(1024), 0, st, logits, V, ctl, tok_cur, finished, out_len);
}

cudaError_t launch_advance_step(StepCtl* ctl, int32_t* kv_pos, int B, int sampled, cudaStream_t st) {
    return launch_k(advance_step_kernel, dim3((B + 127) / 128), dim3(128), 0, st, ctl, kv_pos, B, sampled);
}

cudaError_t launch_gate_mul(const float* gu, int ld, float* out32, __nv_bfloat16* hi, __nv_bfloat16* lo, int B, int mlp,
                            cudaStream_t st) {
    dim3 grid((mlp + 255) / 256, B);
    return launch_k(gate_mul_kernel, grid, dim3(256), 0, st, gu, ld, out32, hi, lo, mlp);
}

}  // namespace lumi
