// Bandwidth-bound kernels of the decode step: embedding gather, RMSNorm, weight-streaming GEMV,
// the fused Mamba-3 state update, and sampling.
//
// Arithmetic follows the reference's CPU branch (inference/src/model.rs:296-375) operation by
// operation; where the reference rounds after every multiply and add (Rust never contracts to FMA),
// the round-to-nearest intrinsics below are used so the compiler cannot contract either.  Dot
// products use FMA with a fixed summation order (per-lane strided partials, xor-shuffle tree), so
// results are bit-stable from run to run.
#include "internal.h"
#include <type_traits>

#include <cfloat>
#include <cmath>
#include <cstdlib>

namespace lumi {

namespace {

// Programmatic dependent launch: a kernel launched with the attribute may start while its
// predecessor still runs; everything that touches the predecessor's results comes after pdl_wait().
// Pointers to data that an earlier kernel of the chain produced (activations, residuals, logits) are NOT
// declared `const __restrict__`: that qualifier lets the compiler treat their loads as invariant and move
// them above the wait, where they would read the values of the previous layer.  Only weights carry it.
// Without the attribute both instructions are no-ops.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

#ifdef LUMI_TIMELINE
// debugging aid (not compiled by default): per-kernel time stamps of a few CTAs
__device__ unsigned long long g_tl[65536 * 10];
__device__ unsigned g_tl_n;
__device__ __forceinline__ unsigned long long tl_now() { unsigned long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t; }
__device__ __forceinline__ bool tl_on() { return threadIdx.x == 0 && (blockIdx.x == 0 || blockIdx.x == gridDim.x / 2 || blockIdx.x == gridDim.x - 1) && blockIdx.y == 0; }
__device__ __forceinline__ void tl_rec(int kind, const unsigned long long (&m)[6], unsigned long long cend) {
    unsigned i = atomicAdd(&g_tl_n, 1u);
    if (i < 65536u) {
        unsigned smid; asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
        g_tl[i * 10] = kind; g_tl[i * 10 + 1] = blockIdx.x; g_tl[i * 10 + 2] = smid;
        for (int j = 0; j < 6; ++j) g_tl[i * 10 + 3 + j] = m[j];
        g_tl[i * 10 + 9] = cend;
    }
}
// slot 0: start (global ns); slots 1..4: SM cycle counter at the marks; slot 5: global ns at the wait's end
#define TL_T0 unsigned long long tlm[6] = {tl_now(), 0, 0, 0, 0, 0};
#define TL_T1 tlm[5] = tl_now(); tlm[1] = clock64();
#define TL_MARK(i) tlm[i] = clock64();
#define TL_END(kind) if (tl_on()) { tl_rec(kind, tlm, clock64()); }
#else
#define TL_T0
#define TL_T1
#define TL_MARK(i)
#define TL_END(kind)
#endif
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
__global__ void embed_kernel(const WT* __restrict__ emb, const uint32_t* tok_cur, float* x,
                             int D, int vocab, StepCtl* ctl, const int32_t* row_len) {
    const int b = blockIdx.x;
    pdl_launch_dependents();
    pdl_wait();
    // during prefill the token comes from the uploaded prompt, afterwards from the last sampled one
    const int pp = ctl->prompt_pos;
    uint32_t t = (pp < ctl->prompt_len) ? ctl->prompt[(size_t)pp * ctl->batch + b] : tok_cur[b];
    // prompts of different lengths: a sequence whose prompt has ended idles (its state is left alone by the kernels
    // that own state); what is stored beyond its length is padding and is not looked at
    if (row_len != nullptr && pp < ctl->prompt_len && pp >= row_len[b]) t = 0;
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
// ssq == null: hi (+ lo) = x * r * gamma.  ssq != null (the form the GEMM with a folded norm consumes): hi (+ lo) =
// x * gamma and ssq[b * ssq_stride] = sum of x^2 — the per-row scale r is applied by the GEMM's epilogue.
__global__ void __launch_bounds__(256) norm_split_kernel(const float* x, const float* __restrict__ gamma,
                                                         __nv_bfloat16* hi, __nv_bfloat16* lo,
                                                         int D, float eps, float* ssq, int ssq_stride) {
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
        if (ssq != nullptr) { if (threadIdx.x == 0) ssq[(size_t)b * ssq_stride] = t; }
        else r = rms_scale(t, D, eps);
    }
    for (int i = threadIdx.x; i < D; i += 256) {
        float v = xr[i];
        if (gamma) v = ssq != nullptr ? __fmul_rn(v, gamma[i]) : __fmul_rn(__fmul_rn(v, r), gamma[i]);
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
__global__ void __launch_bounds__(256) gemv_kernel(const float* A, int lda, const WT* __restrict__ W,
                                                   float* D, int ldd, const float* R,
                                                   const float* __restrict__ gamma, int M, int N, int K, float eps, int KS,
                                                   float* amax_val, int* amax_idx, int amax_stride) {
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
        if (seg == 0) {
#pragma unroll
            for (int r = 0; r < NR; ++r)
#pragma unroll
                for (int b = 0; b < NB; ++b) {
                    float t = part[warp][r][b];
                    for (int sg = 1; sg < KS; ++sg) t += part[warp + sg][r][b];
                    acc[r][b] = t;
                }
        }
    }
    // greedy head: this warp's best (value, lowest row on ties) per batch row, for the per-CTA partial below
    float bestv[NB];
    int besti[NB];
#pragma unroll
    for (int b = 0; b < NB; ++b) { bestv[b] = -INFINITY; besti[b] = 0x7fffffff; }
    if (seg == 0 && lane == 0 && row0 < N) {
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
                if (D != nullptr) D[o] = v;
                if (v > bestv[b] || (v == bestv[b] && row < besti[b])) { bestv[b] = v; besti[b] = row; }
            }
        }
    }
    if (amax_val != nullptr) {
        // argmax fused behind the product (replaces the host-side argmax of inference/src/main.rs:142-143): one
        // (value, row) partial per CTA and batch row; a small second stage picks among the partials
        __shared__ float sbv[8][NB];
        __shared__ int sbi[8][NB];
        if (lane == 0) {
#pragma unroll
            for (int b = 0; b < NB; ++b) { sbv[warp][b] = bestv[b]; sbi[warp][b] = besti[b]; }
        }
        __syncthreads();
        if ((int)threadIdx.x < nb) {
            const int b = threadIdx.x;
            float bv = sbv[0][b];
            int bi = sbi[0][b];
            for (int w = 1; w < 8; ++w)
                if (sbv[w][b] > bv || (sbv[w][b] == bv && sbi[w][b] < bi)) { bv = sbv[w][b]; bi = sbi[w][b]; }
            amax_val[(size_t)(m0 + b) * amax_stride + blockIdx.x] = bv;
            amax_idx[(size_t)(m0 + b) * amax_stride + blockIdx.x] = bi;
        }
    }
}

// ---- single-wave GEMV whose whole weight share is requested before the dependency wait ---------------
// For the smallest batches the chain of a token is latency-bound: each kernel waits for its predecessor,
// then for HBM.  Here a CTA owns N / gridDim.x consecutive output rows and asks for ALL of their weights
// the moment it becomes resident — the first 8 * RPW rows straight into registers (RPW rows per warp), the
// rest by bulk copies into shared memory (one mbarrier per warp, armed with the bytes of that warp's rows) —
// and only then executes the dependency wait.  Launched with programmatic dependent launch, the CTAs become resident while the predecessors
// still run, so the HBM stream of this kernel overlaps them; after the wait only the activation staging,
// the RMSNorm and the dot products from on-chip memory remain.  One wave, at most one CTA per SM; the
// register / shared-memory split is chosen so that the three kernels of a block fit on an SM together.
// Summation order of a row: lane l owns chunks l, l + 32, ...; two per-lane partial sums (even and odd
// chunks, each in ascending k) are added, then the 5-step xor tree.
constexpr int kPreMaxSmemRows = 64;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint64_t globaltimer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

template <typename WT, int NB, int U, int RPW>
__global__ void __launch_bounds__(256, 2) gemv_pre_kernel(const float* A, int lda, const WT* __restrict__ W,
                                                          float* D, int ldd, const float* R,
                                                          const float* __restrict__ gamma, int M, int N, int K, float eps,
                                                          int rows_per_cta, int pace_ns, int pre_delay_ns, int32_t* status) {
    extern __shared__ float4 gemv_smem4[];
    constexpr int E = WLoad<WT>::E;
    constexpr int GN = (U * E + 7) / 8;                 // gamma values per thread: K / 256 rounded up
    constexpr int RR = 8 * RPW;                         // rows held in registers
    constexpr int GR = U >= 16 ? 2 : (RPW <= 1 ? 6 : 4);   // shared-memory rows of a warp evaluated together
    // One sequence and a short row: every warp keeps the whole activation row in registers (lane l owns the
    // 16-byte chunks l, l + 32, ... — exactly the ones it multiplies), computes the RMSNorm scale itself and
    // never touches shared memory or a block barrier for the activations.
    constexpr bool XREG = (NB == 1) && (U * E <= 32);
    __shared__ __align__(8) uint64_t bars[8];           // one per warp: completes when all of that warp's rows have landed
    __shared__ float nred[NB][8];
    float* xs = reinterpret_cast<float*>(gemv_smem4);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int K4 = K >> 2, KC = K / E;
    const int nb = min(NB, M);
    const int row_base = blockIdx.x * rows_per_cta;
    const int nrows = min(rows_per_cta, N - row_base);
    const int ns = max(0, nrows - RR);                  // rows that go through shared memory
    const uint32_t row_bytes = (uint32_t)K * (uint32_t)sizeof(WT);
    unsigned char* wrows = reinterpret_cast<unsigned char*>(xs + (size_t)NB * K);

    TL_T0
    pdl_launch_dependents();
    if (threadIdx.x == 0) {
        for (int j = 0; j < 8; ++j) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&bars[j])));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (threadIdx.x < 8 && (int)threadIdx.x < ns) {     // rows threadIdx.x, threadIdx.x + 8, ... belong to that warp
        const uint32_t bytes = (uint32_t)((ns - (int)threadIdx.x + 7) / 8) * row_bytes;
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(&bars[threadIdx.x])), "r"(bytes) : "memory");
    }
    if (pre_delay_ns > 0) __nanosleep(pre_delay_ns);
    uint4 wreg[RPW > 0 ? RPW : 1][U];
#pragma unroll
    for (int r = 0; r < RPW; ++r) {
        const int lr = warp + 8 * r;                    // this warp's r-th register row
        const WT* wp = W + (size_t)(row_base + min(lr, max(nrows - 1, 0))) * K;
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int c = lane + 32 * u;
            wreg[r][u] = lr < nrows ? __ldg(reinterpret_cast<const uint4*>(wp + (size_t)c * E)) : make_uint4(0u, 0u, 0u, 0u);
        }
    }
    // bulk copies of the other rows: all at once, or one every pace_ns so that the stream does not
    // swamp the memory system while the kernels ahead in the chain wait for their few dependent loads
    if (pace_ns <= 0) {
        if ((int)threadIdx.x < ns) {
            const int j = threadIdx.x;
            const uint32_t bar = smem_u32(&bars[j & 7]);
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                         ::"r"(smem_u32(wrows + (size_t)j * row_bytes)), "l"(W + (size_t)(row_base + RR + j) * K), "r"(row_bytes), "r"(bar) : "memory");
        }
    } else if (threadIdx.x == 224) {
        for (int j = 0; j < ns; ++j) {
            const uint32_t bar = smem_u32(&bars[j & 7]);
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                         ::"r"(smem_u32(wrows + (size_t)j * row_bytes)), "l"(W + (size_t)(row_base + RR + j) * K), "r"(row_bytes), "r"(bar) : "memory");
            __nanosleep(pace_ns);
        }
    }
    float gam[XREG ? 1 : GN];
    if constexpr (XREG) {
        // the norm weights wait in the staging area (the activations themselves never go there)
        if (gamma != nullptr) {
            for (int i = threadIdx.x; i < K4; i += 256) reinterpret_cast<float4*>(xs)[i] = reinterpret_cast<const float4*>(gamma)[i];
        }
        gam[0] = 0.f;
        __syncthreads();
    } else {
#pragma unroll
        for (int i = 0; i < GN; ++i) {
            const int k = threadIdx.x + 256 * i;
            gam[i] = (gamma != nullptr && k < K) ? gamma[k] : 0.f;
        }
    }
    pdl_wait();
    TL_T1

    // residuals of the rows whose stores this lane owns (register rows, first shared-memory group)
    float rres_r[NB], rres_s[NB];
#pragma unroll
    for (int b = 0; b < NB; ++b) rres_r[b] = rres_s[b] = 0.f;
    if (R != nullptr) {
        if (lane < RPW && warp + 8 * lane < nrows) {
#pragma unroll
            for (int b = 0; b < NB; ++b)
                if (b < nb) rres_r[b] = R[(size_t)b * ldd + row_base + warp + 8 * lane];
        }
        if (lane < GR && warp + 8 * lane < ns) {
#pragma unroll
            for (int b = 0; b < NB; ++b)
                if (b < nb) rres_s[b] = R[(size_t)b * ldd + row_base + RR + warp + 8 * lane];
        }
    }

    float xr[XREG ? U * E : 1];
    if constexpr (XREG) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int c = lane + 32 * u;
#pragma unroll
            for (int q = 0; q < E / 4; ++q) {
                const float4 v = *reinterpret_cast<const float4*>(A + c * E + 4 * q);
                xr[u * E + 4 * q] = v.x; xr[u * E + 4 * q + 1] = v.y; xr[u * E + 4 * q + 2] = v.z; xr[u * E + 4 * q + 3] = v.w;
            }
        }
        if (gamma != nullptr) {
            // sum of squares: four running sums per lane (elements 0, 1, 2, 3 of its quads in ascending k),
            // (s0 + s1) + (s2 + s3), then the xor tree
            float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll
            for (int i = 0; i < U * E; i += 4) {
                s0 = fmaf(xr[i], xr[i], s0); s1 = fmaf(xr[i + 1], xr[i + 1], s1);
                s2 = fmaf(xr[i + 2], xr[i + 2], s2); s3 = fmaf(xr[i + 3], xr[i + 3], s3);
            }
            const float tot = warp_sum(__fadd_rn(__fadd_rn(s0, s1), __fadd_rn(s2, s3)));
            const float rs = rms_scale(tot, K, eps);
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int c = lane + 32 * u;
#pragma unroll
                for (int q = 0; q < E / 4; ++q) {
                    const float4 gq = *reinterpret_cast<const float4*>(xs + c * E + 4 * q);
                    const int i = u * E + 4 * q;
                    xr[i] = __fmul_rn(__fmul_rn(xr[i], rs), gq.x); xr[i + 1] = __fmul_rn(__fmul_rn(xr[i + 1], rs), gq.y);
                    xr[i + 2] = __fmul_rn(__fmul_rn(xr[i + 2], rs), gq.z); xr[i + 3] = __fmul_rn(__fmul_rn(xr[i + 3], rs), gq.w);
                }
            }
        }
        TL_MARK(2)
    } else {
        for (int i = threadIdx.x; i < NB * K4; i += 256) {
            int b = i / K4, k4 = i - b * K4;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (b < nb) v = *reinterpret_cast<const float4*>(A + (size_t)b * lda + 4 * k4);
            reinterpret_cast<float4*>(xs)[i] = v;
        }
        __syncthreads();
        TL_MARK(2)
        if (gamma != nullptr) {
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
#pragma unroll
                    for (int i = 0; i < GN; ++i) {
                        const int k = threadIdx.x + 256 * i;
                        if (k < K) xs[b * K + k] = __fmul_rn(__fmul_rn(xs[b * K + k], r), gam[i]);
                    }
                }
            }
            __syncthreads();
        }
    }

    // Rows are evaluated several at a time so that their multiply-add chains overlap; each row keeps two
    // accumulators (even and odd chunks) that are added at the end.  Lane s of a warp owns the residual
    // and the store of the warp's s-th row of a pass.
    auto accum = [&](const uint4& wv, int u, int c, float (&acc)[NB]) {
        float w[E];
        WRaw<WT>::cvt(wv, w);
        if constexpr (XREG) {
#pragma unroll
            for (int e = 0; e < E; ++e) acc[0] = fmaf(w[e], xr[u * E + e], acc[0]);
        } else {
#pragma unroll
            for (int b = 0; b < NB; ++b) {
#pragma unroll
                for (int q = 0; q < E / 4; ++q) {
                    const float4 v = *reinterpret_cast<const float4*>(xs + b * K + c * E + 4 * q);
                    acc[b] = fmaf(w[4 * q], v.x, acc[b]);
                    acc[b] = fmaf(w[4 * q + 1], v.y, acc[b]);
                    acc[b] = fmaf(w[4 * q + 2], v.z, acc[b]);
                    acc[b] = fmaf(w[4 * q + 3], v.w, acc[b]);
                }
            }
        }
    };

    if constexpr (RPW > 0) {
        float acc[RPW][2][NB];
#pragma unroll
        for (int r = 0; r < RPW; ++r)
#pragma unroll
            for (int b = 0; b < NB; ++b) acc[r][0][b] = acc[r][1][b] = 0.f;
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int c = lane + 32 * u;
#pragma unroll
            for (int r = 0; r < RPW; ++r) accum(wreg[r][u], u, c, acc[r][u & 1]);
        }
#pragma unroll
        for (int r = 0; r < RPW; ++r)
#pragma unroll
            for (int b = 0; b < NB; ++b) acc[r][0][b] = warp_sum(__fadd_rn(acc[r][0][b], acc[r][1][b]));
#pragma unroll
        for (int r = 0; r < RPW; ++r) {
            if (lane == r && warp + 8 * r < nrows) {
#pragma unroll
                for (int b = 0; b < NB; ++b)
                    if (b < nb) {
                        float v = acc[r][0][b];
                        if (R != nullptr) v = __fadd_rn(v, rres_r[b]);
                        D[(size_t)b * ldd + row_base + warp + 8 * r] = v;
                    }
            }
        }
    }
    TL_MARK(3)
    bool timed_out = false;
    for (int j0 = warp; j0 < ns && !timed_out; j0 += 8 * GR) {
        if (j0 != warp) {            // later groups (rare): their residuals are fetched here
#pragma unroll
            for (int b = 0; b < NB; ++b) rres_s[b] = 0.f;
            if (R != nullptr && lane < GR && j0 + 8 * lane < ns) {
#pragma unroll
                for (int b = 0; b < NB; ++b)
                    if (b < nb) rres_s[b] = R[(size_t)b * ldd + row_base + RR + j0 + 8 * lane];
            }
        }
        if (j0 == warp) {
            const uint32_t bar = smem_u32(&bars[warp]);
            uint32_t done = 0, polls = 0;
            uint64_t t0 = 0;
            while (true) {
                asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], 0;\nselp.u32 %0, 1, 0, p;\n}"
                             : "=r"(done) : "r"(bar) : "memory");
                if (done) break;
                if ((++polls & 255u) == 0u) {           // the clock is read rarely: it is slow to read
                    const uint64_t now = globaltimer_ns();
                    if (t0 == 0) t0 = now;
                    else if (now - t0 > 500000000ull) { timed_out = true; break; }
                }
            }
            if (timed_out) break;
        }
        if (timed_out) break;
        if (j0 == warp) { TL_MARK(4) }
        const int ng = min(GR, (ns - j0 + 7) / 8);      // valid rows of this group
        // one straight-line body per row count, so that no branch sits between the loads and their use
        auto body = [&](auto ngc) {
            constexpr int NG = decltype(ngc)::value;
            float acc[NG][2][NB];
#pragma unroll
            for (int g = 0; g < NG; ++g)
#pragma unroll
                for (int b = 0; b < NB; ++b) acc[g][0][b] = acc[g][1][b] = 0.f;
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int c = lane + 32 * u;
                uint4 wv[NG];
#pragma unroll
                for (int g = 0; g < NG; ++g) wv[g] = reinterpret_cast<const uint4*>(wrows + (size_t)(j0 + 8 * g) * row_bytes)[c];
#pragma unroll
                for (int g = 0; g < NG; ++g) accum(wv[g], u, c, acc[g][u & 1]);
            }
#pragma unroll
            for (int g = 0; g < NG; ++g)
#pragma unroll
                for (int b = 0; b < NB; ++b) acc[g][0][b] = warp_sum(__fadd_rn(acc[g][0][b], acc[g][1][b]));
#pragma unroll
            for (int g = 0; g < NG; ++g) {
                if (lane == g) {
#pragma unroll
                    for (int b = 0; b < NB; ++b)
                        if (b < nb) {
                            float v = acc[g][0][b];
                            if (R != nullptr) v = __fadd_rn(v, rres_s[b]);
                            D[(size_t)b * ldd + row_base + RR + j0 + 8 * g] = v;
                        }
                }
            }
        };
        switch (ng) {
            case 1: body(std::integral_constant<int, 1>{}); break;
            case 2: body(std::integral_constant<int, 2>{}); break;
            case 3: body(std::integral_constant<int, 3>{}); break;
            case 4: body(std::integral_constant<int, 4>{}); break;
            case 5: if constexpr (GR >= 5) body(std::integral_constant<int, 5>{}); break;
            case 6: if constexpr (GR >= 6) body(std::integral_constant<int, 6>{}); break;
            default: break;
        }
    }
    if (timed_out) {
        // report, then give this warp's copies a second, equally bounded chance to land before the CTA's shared memory goes away
        if (lane == 0 && status != nullptr) atomicOr(status, STATUS_TIMEOUT);
        const uint32_t bar = smem_u32(&bars[warp]);
        uint32_t done = 0, polls = 0;
        uint64_t t0 = 0;
        while (!done) {
            asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], 0;\nselp.u32 %0, 1, 0, p;\n}"
                         : "=r"(done) : "r"(bar) : "memory");
            if (!done && (++polls & 255u) == 0u) {
                const uint64_t now = globaltimer_ns();
                if (t0 == 0) t0 = now;
                else if (now - t0 > 500000000ull) break;
            }
        }
    }
    TL_END(K == 1024 ? 1 : 3)
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

    TL_T0
    pdl_launch_dependents();
    // prompts of different lengths: a sequence whose prompt has ended keeps its state until the others are done
    // (prompt_pos was advanced by the previous step, which has finished: see below)
    if (a.row_len != nullptr) {
        const int pp = a.ctl->prompt_pos;
        if (pp < a.ctl->prompt_len && pp >= a.row_len[b]) return;
    }
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
    // parameters of the layer and the factor of the previous token: not produced by the predecessor either
    const int hh = active ? h : H - 1;
    const int g = hh / (H / a.G);
    const float v_dtb = a.dtb[hh], v_dskip = a.dskip[hh];
    constexpr int NJ = (N / 2 + 31) / 32;
    float g_b0[NJ], g_b1[NJ], g_c0[NJ], g_c1[NJ], o_b0[NJ], o_b1[NJ], o_c0[NJ], o_c1[NJ];
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
        const int k = min(lane + 32 * j, HN - 1);
        const int i0 = g * N + 2 * k;
        g_b0[j] = a.bg[i0]; g_b1[j] = a.bg[i0 + 1]; g_c0[j] = a.cg[i0]; g_c1[j] = a.cg[i0 + 1];
        o_b0[j] = a.bb[i0]; o_b1[j] = a.bb[i0 + 1]; o_c0[j] = a.cb[i0]; o_c1[j] = a.cb[i0 + 1];
    }
    constexpr int ROWS_PL = (P / WPH + 31) / 32;
    float v_xp[ROWS_PL];
#pragma unroll
    for (int j = 0; j < ROWS_PL; ++j) v_xp[j] = a.xprev[bh * P + min(sub * ROWS + lane + 32 * j, P - 1)];
    pdl_wait();
    TL_T1

    const float* pr = a.proj + (size_t)b * a.ldp;
    const float* Bp = pr + 2 * DI;
    const float* Cp = Bp + BC;
    const float* dt = Cp + BC;
    const float* lam_raw = dt + H;
    const float* dda = dt + 2 * H;
    const float* theta = dt + 3 * H;

    // every value of the predecessor that the prologue needs is requested here, ahead of any use, so the
    // loads overlap instead of forming a chain of round trips
    const float v_dt = dt[hh], v_dda = dda[hh], v_lam = lam_raw[hh];
    float v_th[NJ], v_b0[NJ], v_b1[NJ], v_c0[NJ], v_c1[NJ];
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
        const int k = min(lane + 32 * j, HN - 1);
        const int i0 = g * N + 2 * k;
        v_th[j] = theta[hh * HN + k];
        v_b0[j] = Bp[i0]; v_b1[j] = Bp[i0 + 1]; v_c0[j] = Cp[i0]; v_c1[j] = Cp[i0 + 1];
    }
    float v_x[ROWS_PL], v_z[ROWS_PL];
#pragma unroll
    for (int j = 0; j < ROWS_PL; ++j) {
        const int row = min(sub * ROWS + lane + 32 * j, P - 1);
        v_x[j] = pr[hh * P + row];
        v_z[j] = pr[DI + hh * P + row];
    }
    // BCNorm statistics (model.rs:311-312: the norm runs over the whole bc vector): the first NQ rounds of
    // 16-byte loads go out together; what is left (large BC, small CTAs, odd layouts) runs as a plain loop.
    // Order of the sum: per thread its quads in ascending position (x, y, z, w within a quad), then the rest
    // loop, the xor tree, and the warps in order.
    constexpr int NQ = WPH == 1 ? 1 : 2;
    const bool vec_ok = ((a.ldp | (2 * DI) | BC) & 3) == 0 && (reinterpret_cast<uintptr_t>(a.proj) & 15) == 0;
    const int BC4 = vec_ok ? (BC >> 2) : 0;
    float4 qb[NQ], qc[NQ];
#pragma unroll
    for (int j = 0; j < NQ; ++j) {
        const int i = threadIdx.x + j * blockDim.x;
        qb[j] = i < BC4 ? reinterpret_cast<const float4*>(Bp)[i] : make_float4(0.f, 0.f, 0.f, 0.f);
        qc[j] = i < BC4 ? reinterpret_cast<const float4*>(Cp)[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    }

    // per-head scalars (model.rs:307, 314-317, 355-359) and the rotation angles (model.rs:338-345): they do not
    // need the statistics, so their arithmetic runs while the loads above are still in flight
    const float dtp = softplus_ref(__fadd_rn(v_dt, v_dtb));
    float av = -softplus_ref(v_dda);
    av = fminf(fmaxf(av, -1e6f), -1e-4f);
    const float abar = expf(__fmul_rn(av, dtp));
    const float lam = sigmoid_ref(v_lam);
    const float oml = __fadd_rn(__fmul_rn(lam, -1.0f), 1.0f);
    const float c2 = __fmul_rn(abar, oml);
    const float PI_F = 3.14159265358979323846f;
    const float TWO_PI = __fmul_rn(2.0f, PI_F);
    float cu_new[NJ], sa[NJ], ca[NJ];
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
        const float angle = __fmul_rn(tanhf(v_th[j]), PI_F);
        cu_new[j] = fmodf(__fadd_rn(cu_old[j], __fmul_rn(dtp, angle)), TWO_PI);
        sincosf(cu_new[j], &sa[j], &ca[j]);
    }
    float xa_v[ROWS_PL], gate_v[ROWS_PL];
#pragma unroll
    for (int j = 0; j < ROWS_PL; ++j) {
        xa_v[j] = silu_ref(v_x[j]);                          // model.rs:310
        gate_v[j] = silu_ref(v_z[j]);                        // model.rs:370
    }

    float sb = 0.f, sc = 0.f;
#pragma unroll
    for (int j = 0; j < NQ; ++j) {
        sb = fmaf(qb[j].x, qb[j].x, sb); sb = fmaf(qb[j].y, qb[j].y, sb); sb = fmaf(qb[j].z, qb[j].z, sb); sb = fmaf(qb[j].w, qb[j].w, sb);
        sc = fmaf(qc[j].x, qc[j].x, sc); sc = fmaf(qc[j].y, qc[j].y, sc); sc = fmaf(qc[j].z, qc[j].z, sc); sc = fmaf(qc[j].w, qc[j].w, sc);
    }
    for (int i = (vec_ok ? 4 * NQ * (int)blockDim.x : 0) + threadIdx.x; i < BC; i += blockDim.x) {
        float v = Bp[i];
        sb = fmaf(v, v, sb);
        v = Cp[i];
        sc = fmaf(v, v, sc);
    }
    sb = warp_sum(sb);
    sc = warp_sum(sc);
    if (lane == 0) { red[0][warp] = sb; red[1][warp] = sc; }
    __syncthreads();       // also orders every warp's reads of bprev / cum / xprev above before the writes below
    TL_MARK(2)
    if (!active) return;
    float tb = 0.f, tc = 0.f;
    for (int w = 0; w < nwarp; ++w) { tb += red[0][w]; tc += red[1][w]; }
    const float rb = rms_scale(tb, BC, a.eps), rc = rms_scale(tc, BC, a.eps);

    SsmSmem<P, N>& sm = sm_all[warp];

    // DD-RoPE (model.rs:346-350): lane k rotates pair (2k, 2k+1) of the normalised B and C
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
        const int k = lane + 32 * j;
        if (k < HN) {
            if (sub == 0) a.cum[bh * HN + k] = cu_new[j];
            float b0 = __fadd_rn(__fmul_rn(__fmul_rn(v_b0[j], rb), g_b0[j]), o_b0[j]);
            float b1 = __fadd_rn(__fmul_rn(__fmul_rn(v_b1[j], rb), g_b1[j]), o_b1[j]);
            float c0 = __fadd_rn(__fmul_rn(__fmul_rn(v_c0[j], rc), g_c0[j]), o_c0[j]);
            float c1 = __fadd_rn(__fmul_rn(__fmul_rn(v_c1[j], rc), g_c1[j]), o_c1[j]);
            sm.bt[2 * k] = __fsub_rn(__fmul_rn(ca[j], b0), __fmul_rn(sa[j], b1));
            sm.bt[2 * k + 1] = __fadd_rn(__fmul_rn(sa[j], b0), __fmul_rn(ca[j], b1));
            sm.ct[2 * k] = __fsub_rn(__fmul_rn(ca[j], c0), __fmul_rn(sa[j], c1));
            sm.ct[2 * k + 1] = __fadd_rn(__fmul_rn(sa[j], c0), __fmul_rn(ca[j], c1));
        }
    }
    const int prow0 = sub * ROWS;          // first state row of this warp
#pragma unroll
    for (int j = 0; j < ROWS_PL; ++j) {
        const int p = lane + 32 * j;
        if (p < ROWS) {
            const int row = prow0 + p;
            sm.xa[row] = xa_v[j];
            sm.xp[row] = v_xp[j];
            sm.gate[row] = gate_v[j];
        }
    }
    __syncwarp();

    TL_MARK(3)
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
    TL_MARK(4)
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
    TL_END(2)
}

// h <- h_init broadcast over head_dim (model.rs:744-748); factors and angles <- 0 (:751-752)
__global__ void state_reset_kernel(float* h, float* xprev, float* bprev, float* cum, const float* __restrict__ h_init,
                                   const int32_t* __restrict__ slots, int H, int P, int N) {
    // one block per (sequence, head): the head's P x N tile, its P + N factors and its N / 2 angles
    const int slot = slots ? slots[blockIdx.x] : blockIdx.x;
    const int hh = blockIdx.y;
    float* ht = h + ((size_t)slot * H + hh) * P * N;
    for (int i = threadIdx.x; i < P * N; i += blockDim.x) ht[i] = h_init ? h_init[hh * N + i % N] : 0.f;
    for (int i = threadIdx.x; i < P; i += blockDim.x) xprev[((size_t)slot * H + hh) * P + i] = 0.f;
    for (int i = threadIdx.x; i < N; i += blockDim.x) bprev[((size_t)slot * H + hh) * N + i] = 0.f;
    for (int i = threadIdx.x; i < N / 2; i += blockDim.x) cum[((size_t)slot * H + hh) * (N / 2) + i] = 0.f;
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
    if (warp == 0) {                       // the per-warp winners (at most 32) by one more xor tree
        float wv = lane < nw ? red[lane].v : -INFINITY;
        int wi = lane < nw ? red[lane].i : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            float ov = __shfl_xor_sync(0xffffffffu, wv, o);
            int oi = __shfl_xor_sync(0xffffffffu, wi, o);
            if (better(ov, oi, wv, wi)) { wv = ov; wi = oi; }
        }
        if (lane == 0) { red[32].v = wv; red[32].i = wi; }
    }
    __syncthreads();
    return red[32];
}

constexpr int kMaxTopK = 256;
constexpr int kSelEqMax = 1024;       // tied entries at the k-th value handled by the fast selection (more: the round-by-round path)

// One block per sequence.  Greedy: argmax with the lowest index on ties.  Otherwise temperature
// softmax over the top-k survivors (or the whole vocabulary) and the walk over the cumulative
// distribution in vocabulary order.
__global__ void __launch_bounds__(1024) sample_kernel(const float* logits, int V, StepCtl* ctl,
                                                      uint32_t* tok_cur, int32_t* finished, int32_t* out_len) {
    __shared__ BestPair red[33];           // 32 warp winners + the block winner
    __shared__ float top_v[kMaxTopK];
    __shared__ int top_i[kMaxTopK];
    __shared__ float chunk_sum[1024];
    __shared__ int result;
    __shared__ int sel_hist[256], sel_eq[kSelEqMax];
    __shared__ int sel_digit, sel_above, sel_n, sel_neq;
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
            // k rounds of block-wide argmax over the not-yet-taken entries.  When the row fits (up to 32 entries
            // per thread) each thread keeps its entries in registers with a taken-mask and a cached local best,
            // so a round costs one block reduction and a rescan by the single thread that owned the winner.
            constexpr int kRegVals = 32;
            bool selected = false;
            if (V <= nt * kRegVals) {
                // The row fits in registers (up to 32 entries per thread).  The k-th largest value is found by a radix
                // select over an order-preserving integer image of the floats (four passes of 256-bin histograms in
                // shared memory); then everything above it survives, and of the entries equal to it the ones with the
                // lowest ids — the same set k rounds of "largest remaining, lowest id on ties" would pick.
                uint32_t keys[kRegVals];                              // the float is recovered from its key where needed
                auto key_to_float = [](uint32_t key) { return __uint_as_float((key & 0x80000000u) ? (key & 0x7fffffffu) : ~key); };
#pragma unroll
                for (int j = 0; j < kRegVals; ++j) {
                    const int i = tid + j * nt;
                    float v = i < V ? lg[i] : -INFINITY;
                    if (v != v) v = -INFINITY;                       // a NaN is never chosen
                    const uint32_t u = __float_as_uint(v);
                    keys[j] = i < V ? ((u & 0x80000000u) ? ~u : (u | 0x80000000u)) : 0u;    // padding sorts below every real entry
                }
                uint32_t prefix = 0u;
                int want = k;                                          // rank (from the top) still to be located inside the prefix
                for (int shift = 24; shift >= 0; shift -= 8) {
                    for (int i = tid; i < 256; i += nt) sel_hist[i] = 0;
                    __syncthreads();
                    const uint32_t hi_mask = shift == 24 ? 0u : (0xffffffffu << (shift + 8));
#pragma unroll
                    for (int j = 0; j < kRegVals; ++j)
                        if (tid + j * nt < V && (keys[j] & hi_mask) == prefix) atomicAdd(&sel_hist[(keys[j] >> shift) & 255u], 1);
                    __syncthreads();
                    if (tid < 32) {
                        // bins 8 * lane .. 8 * lane + 7; suffix counts from the top bin down
                        int c[8], tot = 0;
#pragma unroll
                        for (int q = 0; q < 8; ++q) { c[q] = sel_hist[8 * tid + q]; tot += c[q]; }
                        int above = 0;                                  // entries in the bins of higher lanes
                        for (int l2 = 31; l2 > 0; --l2) { const int t2 = __shfl_sync(0xffffffffu, tot, l2); if (l2 > tid) above += t2; }
                        int acc = above;
#pragma unroll
                        for (int q = 7; q >= 0; --q) {
                            if (acc < want && want <= acc + c[q]) { sel_digit = 8 * tid + q; sel_above = acc; }
                            acc += c[q];
                        }
                    }
                    __syncthreads();
                    prefix |= (uint32_t)sel_digit << shift;
                    want -= sel_above;
                    __syncthreads();
                }
                // prefix is the key of the k-th largest entry; `want` of the entries equal to it survive (lowest ids)
                if (tid == 0) { sel_n = 0; sel_neq = 0; }
                __syncthreads();
#pragma unroll
                for (int j = 0; j < kRegVals; ++j) {
                    const int i = tid + j * nt;
                    if (i < V) {
                        if (keys[j] > prefix) { const int o = atomicAdd(&sel_n, 1); top_v[o] = key_to_float(keys[j]); top_i[o] = i; }
                        else if (keys[j] == prefix) { const int o = atomicAdd(&sel_neq, 1); if (o < kSelEqMax) sel_eq[o] = i; }
                    }
                }
                __syncthreads();
                const int n_gt = sel_n, n_eq = sel_neq;
                if (n_eq <= kSelEqMax) {
                    // rank of every tied entry among the tied ids; the `want` lowest go in
                    for (int e = tid; e < n_eq; e += nt) {
                        const int me = sel_eq[e];
                        int rank = 0;
                        for (int f = 0; f < n_eq; ++f) rank += sel_eq[f] < me ? 1 : 0;
                        if (rank < want) {
                            top_v[n_gt + rank] = key_to_float(prefix);
                            top_i[n_gt + rank] = me;
                        }
                    }
                    selected = true;
                }
                __syncthreads();
            }
            if (!selected)
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
            // survivors into vocabulary order: entry j goes to the position given by the number of smaller ids
            {
                float sv = 0.f; int si = 0, rank = 0;
                if (tid < k) {
                    sv = top_v[tid]; si = top_i[tid];
                    for (int j = 0; j < k; ++j) rank += top_i[j] < si ? 1 : 0;
                }
                __syncthreads();
                if (tid < k) { top_v[rank] = sv; top_i[rank] = si; }
                __syncthreads();
            }
            if (tid == 0) {
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

// Greedy head, second stage (batch <= 8): one warp per sequence picks the best of the per-CTA partials the head's GEMV
// left behind (value, lowest id on ties — the rule of the single-stage argmax), records the token exactly as
// sample_kernel does, and the block then does the end-of-step bookkeeping of advance_step_kernel.  One launch
// instead of two, and nothing re-reads the logits.
__global__ void __launch_bounds__(256) head_finish_kernel(const float* amax_val, const int* amax_idx, int nparts, int stride, int B,
                                                         StepCtl* ctl, uint32_t* tok_cur, int32_t* finished, int32_t* out_len,
                                                         int32_t* kv_pos) {
    const int b = threadIdx.x >> 5, lane = threadIdx.x & 31;
    pdl_launch_dependents();
    pdl_wait();
    const int step = ctl->step;
    if (b < B) {
        float bv = -INFINITY;
        int bi = 0x7fffffff;
        for (int i = lane; i < nparts; i += 32) {
            const float v = amax_val[(size_t)b * stride + i];
            const int id = amax_idx[(size_t)b * stride + i];
            if (better(v, id, bv, bi)) { bv = v; bi = id; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
        }
        if (lane == 0) {
            tok_cur[b] = (uint32_t)bi;
            if (ctl->record) {
                ctl->out_tokens[(size_t)step * ctl->batch + b] = (uint32_t)bi;
                if (!finished[b]) {
                    if ((uint32_t)bi == ctl->eos_id && !ctl->ignore_eos) finished[b] = 1;   // main.rs:150
                    else out_len[b] += 1;
                }
            }
            if (kv_pos != nullptr) kv_pos[b] += 1;
        }
    }
    __syncthreads();                       // every warp has read ctl->step
    if (threadIdx.x == 0) {
        if (ctl->prompt_pos < ctl->prompt_len) ctl->prompt_pos += 1;
        ctl->step += 1;
    }
}

// End of a step: next prompt position / next output row, and one more cached token per sequence.
__global__ void advance_step_kernel(StepCtl* ctl, int32_t* kv_pos, int B, int sampled, const int32_t* row_len) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    pdl_launch_dependents();
    pdl_wait();
    const int pp0 = ctl->prompt_pos;
    const bool idle = row_len != nullptr && i < B && pp0 < ctl->prompt_len && pp0 >= row_len[i];
    __syncthreads();                       // block 0 changes prompt_pos below; B <= blockDim.x * gridDim.x rows read it above
    if (kv_pos != nullptr && i < B && !idle) kv_pos[i] += 1;
    if (i == 0) {
        if (ctl->prompt_pos < ctl->prompt_len) ctl->prompt_pos += 1;
        if (sampled) ctl->step += 1;
    }
}

// D = sigmoid(gate) * up for the attention block's MLP (model.rs:550-552); gu = [gate | up] per row
__global__ void gate_mul_kernel(const float* gu, int ld, float* out32, __nv_bfloat16* hi, __nv_bfloat16* lo,
                                int mlp) {
    const int b = blockIdx.x;                        // rows on x: a prefill slice has more than 65535
    const int i = blockIdx.y * blockDim.x + threadIdx.x;
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
bool launch_pdl_on() { return g_pdl; }
static thread_local bool g_pdl_gemm = false;
void set_launch_pdl_gemm(bool on) { g_pdl_gemm = on; }
bool launch_pdl_gemm_on() { return g_pdl_gemm; }

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
                         StepCtl* ctl, cudaStream_t st, const int32_t* row_len) {
    // The first kernel of a step is never launched early: it starts only when the previous step has
    // completely finished, which is what lets later kernels of this step read state ahead of their
    // own dependency wait.
    const bool keep = g_pdl;
    g_pdl = false;
    cudaError_t e;
    if (dtype == LUMI_DTYPE_BF16)
        e = launch_k(embed_kernel<__nv_bfloat16>, dim3(B), dim3(128), 0, st, (const __nv_bfloat16*)emb, tok_cur, x, D, vocab, ctl, row_len);
    else
        e = launch_k(embed_kernel<float>, dim3(B), dim3(128), 0, st, (const float*)emb, tok_cur, x, D, vocab, ctl, row_len);
    g_pdl = keep;
    return e;
}

cudaError_t launch_norm_split(const float* x, const float* gamma, __nv_bfloat16* hi, __nv_bfloat16* lo, int B, int D,
                              float eps, cudaStream_t st, float* ssq, int ssq_stride) {
    return launch_k(norm_split_kernel, dim3(B), dim3(256), 0, st, x, gamma, hi, lo, D, eps, ssq, ssq_stride);
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
    if (a.amax_val != nullptr) {
        if ((int)grid.x > a.amax_stride) return cudaErrorInvalidValue;
        if (a.amax_parts != nullptr) *a.amax_parts = (int)grid.x;
    }
    return launch_k(kern, grid, dim3(256), smem, st, a.A, a.lda, (const WT*)a.W, a.D, a.ldd, a.R, a.gamma, a.M, a.N, a.K, a.eps, KS,
                    a.amax_val, a.amax_idx, a.amax_stride);
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

// ---- the preloading single-wave variant: when it applies and how it is launched ----
static int sm_count() {
    static int n = 0;
    if (n == 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
            n = 148;
    }
    return n;
}

// LUMI_GEMV_PRE=0 keeps every small-batch product on the multi-wave kernel (tuning aid).
static bool gemv_pre_enabled() {
    static int v = -1;
    if (v < 0) { const char* e = getenv("LUMI_GEMV_PRE"); v = e ? atoi(e) : 1; }
    return v != 0;
}

// LUMI_GEMV_PACE_NS: pause between the bulk copies of a CTA's shared-memory rows (0 = all at once).
static int gemv_pre_pace_ns() {
    static int v = -1;
    if (v < 0) { const char* e = getenv("LUMI_GEMV_PACE_NS"); v = e ? atoi(e) : 0; }
    return v;
}

static int gemv_pre_policy() {
    static int v = -1;
    if (v < 0) { const char* e = getenv("LUMI_GEMV_PRE_POLICY"); v = e ? atoi(e) : 0; }
    return v;
}

// LUMI_GEMV_PRE_DELAY_NS: a CTA with a large share waits this long before it requests its weights, so that
// the few dependent loads of the kernel that has just been released go ahead of the burst.
static int gemv_pre_delay_ns() {
    static int v = -1;
    if (v < 0) { const char* e = getenv("LUMI_GEMV_PRE_DELAY_NS"); v = e ? atoi(e) : 0; }
    return v;
}

constexpr size_t kPreSmemBudget = 176 * 1024;      // leaves room on the SM for the neighbouring kernels of the chain
constexpr size_t kPreAllSmemBytes = 64 * 1024;     // a CTA share up to this size goes through shared memory only

template <typename WT, int NB, int U, int RPW>
static cudaError_t gemv_pre_launch(const GemvArgs& a, int rows_per_cta, size_t smem, cudaStream_t st) {
    auto kern = gemv_pre_kernel<WT, NB, U, RPW>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
    }
    dim3 grid((a.N + rows_per_cta - 1) / rows_per_cta);
    return launch_k(kern, grid, dim3(256), smem, st, a.A, a.lda, (const WT*)a.W, a.D, a.ldd, a.R, a.gamma, a.M, a.N, a.K, a.eps,
                    rows_per_cta, gemv_pre_pace_ns(), smem > 64 * 1024 ? gemv_pre_delay_ns() : 0, a.status);
}

// Returns true (and the launch result in *err) when the product was given to the preloading kernel.
template <typename WT>
static bool gemv_pre_try(const GemvArgs& a, cudaStream_t st, cudaError_t* err) {
    constexpr int E = WLoad<WT>::E;
    if (!gemv_pre_enabled() || !a.allow_preload || a.amax_val != nullptr || a.act != 0 || a.M > 4 || a.M < 1 || (a.K % E) != 0 || a.K < E) return false;
    const int KC = a.K / E;
    const int U = (KC + 31) / 32;
    if (U > 16 || KC != 32 * U || (U & (U - 1)) != 0) return false;     // rows of exactly 32 * U chunks, U a power of two
    const int NB = a.M <= 1 ? 1 : (a.M <= 2 ? 2 : 4);
    const int rows_per_cta = (a.N + sm_count() - 1) / sm_count();
    const size_t row_bytes = (size_t)a.K * sizeof(WT);
    // small shares: shared memory only (few registers); larger ones: two rows per warp in registers
    // (one when a row is long), the rest in shared memory
    // one register row per warp plus shared-memory rows measured best for the chain of a block at batch 1;
    // LUMI_GEMV_PRE_POLICY=1 (tuning aid): small shares through shared memory only, large ones with two
    // register rows per warp
    int RPW = 1;
    if (gemv_pre_policy() == 1) {
        RPW = 0;
        if (rows_per_cta * row_bytes > kPreAllSmemBytes) RPW = U <= 8 ? 2 : 1;
    }
    const int smem_rows = rows_per_cta > 8 * RPW ? rows_per_cta - 8 * RPW : 0;
    const size_t smem = (size_t)NB * a.K * sizeof(float) + smem_rows * row_bytes;
    if (smem_rows > kPreMaxSmemRows || smem > kPreSmemBudget) return false;
#define LUMI_PRE_CASE(NBV, UV)                                                                                    \
    if (NB == NBV && U <= UV) {                                                                                  \
        if (RPW == 0) *err = gemv_pre_launch<WT, NBV, UV, 0>(a, rows_per_cta, smem, st);                         \
        else if (RPW == 1) *err = gemv_pre_launch<WT, NBV, UV, 1>(a, rows_per_cta, smem, st);                    \
        else *err = gemv_pre_launch<WT, NBV, UV, (UV <= 8 ? 2 : 1)>(a, rows_per_cta, smem, st);                  \
        return true;                                                                                             \
    }
    LUMI_PRE_CASE(1, 1) LUMI_PRE_CASE(1, 2) LUMI_PRE_CASE(1, 4) LUMI_PRE_CASE(1, 8) LUMI_PRE_CASE(1, 16)
    LUMI_PRE_CASE(2, 1) LUMI_PRE_CASE(2, 2) LUMI_PRE_CASE(2, 4) LUMI_PRE_CASE(2, 8) LUMI_PRE_CASE(2, 16)
    LUMI_PRE_CASE(4, 1) LUMI_PRE_CASE(4, 2) LUMI_PRE_CASE(4, 4) LUMI_PRE_CASE(4, 8) LUMI_PRE_CASE(4, 16)
#undef LUMI_PRE_CASE
    return false;
}

cudaError_t launch_gemv(const GemvArgs& a, cudaStream_t st) {
    cudaError_t e = cudaSuccess;
    if (a.w_dtype == LUMI_DTYPE_BF16) {
        if (gemv_pre_try<__nv_bfloat16>(a, st, &e)) return e;
        return gemv_by_batch<__nv_bfloat16>(a, st);
    }
    if (gemv_pre_try<float>(a, st, &e)) return e;
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
            static int hpb_env = -1;
            if (hpb_env < 0) { const char* e = getenv("LUMI_SSM_HPB"); hpb_env = e ? atoi(e) : 1; }
            int hpb = a.H < hpb_env ? a.H : hpb_env;
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
    state_reset_kernel<<<dim3(n_slots, H), 256, 0, st>>>(h, xprev, bprev, cum, h_init, slots, H, P, N);
    return cudaGetLastError();
}

cudaError_t launch_sample(const float* logits, int B, int V, StepCtl* ctl, uint32_t* tok_cur, int32_t* finished,
                          int32_t* out_len, cudaStream_t st) {
    return launch_k(sample_kernel, dim3(B), dim3(1024), 0, st, logits, V, ctl, tok_cur, finished, out_len);
}

// log-probability of a given next token from a row of logits (inference/src/eval.rs:39-139 scores with
// log-softmax over the window's logits): m = max, s = sum exp(l - m), out = l[target] - m - log(s).
// Per-thread partials in ascending index, xor tree, the 8 warps in order.
__global__ void __launch_bounds__(256) logprob_kernel(const float* logits, int V, const uint32_t* targets, int batch, float* out,
                                                      int out_stride, int out_col) {
    __shared__ float red[8];
    const int b = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const float* l = logits + (size_t)b * V;
    float m = -FLT_MAX;
    for (int i = threadIdx.x; i < V; i += 256) m = fmaxf(m, l[i]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (lane == 0) red[warp] = m;
    __syncthreads();
    m = red[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) m = fmaxf(m, red[w]);
    __syncthreads();
    float sum = 0.f;
    for (int i = threadIdx.x; i < V; i += 256) sum += expf(l[i] - m);
    sum = warp_sum(sum);
    if (lane == 0) red[warp] = sum;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) t += red[w];
        const uint32_t tg = targets[b];
        out[(size_t)b * out_stride + out_col] = tg < (uint32_t)V ? (l[tg] - m) - logf(t) : -INFINITY;
    }
}

// The same for the token rows of a prefill slice: logits row i belongs to workspace row r = row0 + i = (sequence b0 + r / ts,
// position t0 + r % ts); the target is the prompt's next token, rows at the last position have none.
__global__ void __launch_bounds__(256) logprob_rows_kernel(const float* logits, int V, const uint32_t* prompt, int batch_total,
                                                           int T, int ts, int t0, int b0, int row0, float* out) {
    __shared__ float red[8];
    const int r = row0 + blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int b = b0 + r / ts, t = t0 + r % ts;
    if (t >= T - 1) return;
    const float* l = logits + (size_t)blockIdx.x * V;
    float m = -FLT_MAX;
    for (int i = threadIdx.x; i < V; i += 256) m = fmaxf(m, l[i]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (lane == 0) red[warp] = m;
    __syncthreads();
    m = red[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) m = fmaxf(m, red[w]);
    __syncthreads();
    float sum = 0.f;
    for (int i = threadIdx.x; i < V; i += 256) sum += expf(l[i] - m);
    sum = warp_sum(sum);
    if (lane == 0) red[warp] = sum;
    __syncthreads();
    if (threadIdx.x == 0) {
        float tot = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) tot += red[w];
        const uint32_t tg = prompt[(size_t)(t + 1) * batch_total + b];
        out[(size_t)b * (T - 1) + t] = tg < (uint32_t)V ? (l[tg] - m) - logf(tot) : -INFINITY;
    }
}

cudaError_t launch_logprob_rows(const float* logits, int rows, int V, const uint32_t* prompt, int batch_total, int T, int ts, int t0,
                                int b0, int row0, float* out, cudaStream_t st) {
    logprob_rows_kernel<<<rows, 256, 0, st>>>(logits, V, prompt, batch_total, T, ts, t0, b0, row0, out);
    return cudaGetLastError();
}

cudaError_t launch_logprob(const float* logits, int B, int V, const uint32_t* targets, float* out, int out_stride, int out_col,
                           cudaStream_t st) {
    logprob_kernel<<<B, 256, 0, st>>>(logits, V, targets, B, out, out_stride, out_col);
    return cudaGetLastError();
}

cudaError_t launch_head_finish(const float* amax_val, const int* amax_idx, int nparts, int stride, int B, StepCtl* ctl, uint32_t* tok_cur,
                               int32_t* finished, int32_t* out_len, int32_t* kv_pos, cudaStream_t st) {
    if (B < 1 || B > 8) return cudaErrorInvalidValue;
    return launch_k(head_finish_kernel, dim3(1), dim3(256), 0, st, amax_val, amax_idx, nparts, stride, B, ctl, tok_cur, finished, out_len, kv_pos);
}

cudaError_t launch_advance_step(StepCtl* ctl, int32_t* kv_pos, int B, int sampled, cudaStream_t st, const int32_t* row_len) {
    if (row_len != nullptr && B > 1024) return cudaErrorInvalidValue;       // one block, so every row sees prompt_pos before it moves
    const int threads = row_len != nullptr ? ((B + 31) / 32) * 32 : 128;
    return launch_k(advance_step_kernel, dim3((B + threads - 1) / threads), dim3(threads), 0, st, ctl, kv_pos, B, sampled, row_len);
}

// Prompts of different lengths: the residual row of every sequence that is at its last prompt token goes to xlast.
__global__ void capture_last_kernel(const float* x, float* xlast, const int32_t* row_len, const StepCtl* ctl, int D) {
    const int b = blockIdx.x;
    if (ctl->prompt_pos != row_len[b] - 1) return;
    for (int k = threadIdx.x; k < D; k += blockDim.x) xlast[(size_t)b * D + k] = x[(size_t)b * D + k];
}
cudaError_t launch_capture_last(const float* x, float* xlast, const int32_t* row_len, const StepCtl* ctl, int B, int D, cudaStream_t st) {
    capture_last_kernel<<<B, 256, 0, st>>>(x, xlast, row_len, ctl, D);
    return cudaGetLastError();
}

cudaError_t launch_gate_mul(const float* gu, int ld, float* out32, __nv_bfloat16* hi, __nv_bfloat16* lo, int B, int mlp,
                            cudaStream_t st) {
    dim3 grid(B, (mlp + 255) / 256);
    return launch_k(gate_mul_kernel, grid, dim3(256), 0, st, gu, ld, out32, hi, lo, mlp);
}

}  // namespace lumi

#ifdef LUMI_TIMELINE
extern "C" int lumi_debug_timeline(unsigned long long* out, int max_records, int reset) {
    unsigned n = 0;
    cudaDeviceSynchronize();
    cudaMemcpyFromSymbol(&n, lumi::g_tl_n, sizeof(n));
    if (n > 65536u) n = 65536u;
    if ((int)n > max_records) n = max_records;
    if (out && n) cudaMemcpyFromSymbol(out, lumi::g_tl, (size_t)n * 10 * sizeof(unsigned long long));
    if (reset) { unsigned z = 0; cudaMemcpyToSymbol(lumi::g_tl_n, &z, sizeof(z)); }
    return (int)n;
}
#endif
