// Chunked (SSD-style) prefill of the Mamba-3 trapezoidal recurrence, chunk length 64, with the chunk's
// projection rows staged by TMA and the chunk products on tensor cores.
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
// — four small matrix products per (sequence, head, chunk):
//     G = C~ B~^T (64x64x64),  Y1 = W X with W = mask/decay(G) (64x64x32),  Y2 = C~ S^_in^T (64x64x32),
//     S^_out += (w x)^T B~ (32x64x64).
// The last token of a launch uses kap = lam, which makes S^ equal the true S: every launch ends with exactly
// the state the decode kernel expects (h, x_prev, B~_prev, cum_angle), and the next launch rebuilds S^ from it.
// DD-RoPE angles are a prefix sum over the chunk taken mod 2 pi (the reference reduces mod 2 pi every step:
// same angle, rounding-level differences; the stored angle may differ from the sequential one by a multiple
// of 2 pi).
//
// One CTA of four warps per (head, sequence), three CTAs per SM (69 KiB of shared memory, 168 registers).
//   * Staging: the chunk's x, z, theta (64 x 32 fp32 each) and the group's raw B, C (64 x 64 fp32 each) arrive by
//     five cp.async.bulk.tensor copies on one mbarrier (bounded wait).  The operand tiles are built IN PLACE over the
//     raw rows, so the copies for chunk c+1 are issued when chunk c's products are done; their flight time is covered
//     by the two other CTAs of the SM (and the per-token scalars dt, lambda, A, BCNorm scales of chunk c+1 are
//     requested into registers at the start of chunk c).
//   * Arithmetic: every operand is an fp32 value split into bf16 hi + lo; a product is three
//     mma.sync.m16n8k16 (hi*hi + hi*lo + lo*hi, fp32 accumulate), which keeps ~16 mantissa bits per factor.
//     Warp w owns tokens 16w..16w+15: its C~ rows stay in registers as A fragments, G's accumulators are masked,
//     decayed and re-used in place as the A fragments of W X (no trip through shared memory), and the state S^
//     lives in accumulator registers across the chunks of a launch (warp w: 16 rows of P x 32 columns of N).
//     Independent accumulators are interleaved so that no multiply-add waits for the one issued just before it.
//   * The pointwise part (softplus / sigmoid / tanh / SiLU / sin / cos) uses the fast hardware forms here: their
//     error (~1e-6) is far below the operand split's (1.5e-5) — the decode step keeps the exact forms.
#include "internal.h"

#include <cuda.h>

#include <type_traits>

namespace lumi {

// defined in gemm_tcgen05.cu: cuTensorMapEncodeTiled for a row-major fp32 matrix [rows][cols], no swizzle
int32_t make_f32_map_2d(CUtensorMap* map, const void* ptr, uint64_t rows, uint64_t cols, uint64_t pitch_bytes, uint32_t box_cols,
                        uint32_t box_rows);

namespace {

constexpr int LCH = 64;          // chunk length
constexpr int TSB = 72;          // row stride (bf16 elements) of the operand tiles: 144 bytes, conflict-free fragment loads
constexpr uint64_t kScanWaitLimitNs = 500ull * 1000 * 1000;

__device__ __forceinline__ float sigmoid_ref(float x) { return __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-x))); }
__device__ __forceinline__ float softplus_ref(float x) { return logf(__fadd_rn(expf(x), 1.0f)); }
__device__ __forceinline__ float silu_fast(float x) { return __fdividef(x, 1.0f + __expf(-x)); }
__device__ __forceinline__ float tanh_fast(float x) {
    // 1 - 2 / (e^{2x} + 1): absolute error ~1e-7; the argument is clamped so e^{2x} stays finite
    const float xc = fminf(fmaxf(x, -15.f), 15.f);
    return 1.0f - __fdividef(2.0f, __expf(2.0f * xc) + 1.0f);
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint64_t globaltimer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: false when the limit expired.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, uint64_t limit_ns) {
    if (mbar_try_wait(bar, parity)) return true;
    const uint64_t t0 = globaltimer_ns();
    for (;;) {
        if (mbar_try_wait(bar, parity)) return true;
        if (globaltimer_ns() - t0 > limit_ns) return false;
    }
}
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
        : "memory");
}

// D (16x8, fp32) += A (16x16, bf16, row) * B (16x8, bf16, col)
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// (a_hi + a_lo)(b_hi + b_lo) without the lo*lo term, for the two 8-column tiles whose B fragments one ldmatrix.x4
// delivers (bh / bl: {b0, b1} of the first tile, {b0, b1} of the second).  The six multiply-adds alternate between
// the two accumulators so that no instruction waits for the one just before it.
__device__ __forceinline__ void mma3x2(float (&d0)[4], float (&d1)[4], const uint32_t (&ah)[4], const uint32_t (&al)[4],
                                       const uint32_t (&bh)[4], const uint32_t (&bl)[4]) {
    mma_bf16(d0, ah, bh[0], bh[1]);
    mma_bf16(d1, ah, bh[2], bh[3]);
    mma_bf16(d0, ah, bl[0], bl[1]);
    mma_bf16(d1, ah, bl[2], bl[3]);
    mma_bf16(d0, al, bh[0], bh[1]);
    mma_bf16(d1, al, bh[2], bh[3]);
}
// the same for four tiles (two ldmatrix.x4 per plane): twelve multiply-adds round-robin over four accumulators
__device__ __forceinline__ void mma3x4(float (&d0)[4], float (&d1)[4], float (&d2)[4], float (&d3)[4], const uint32_t (&ah)[4],
                                       const uint32_t (&al)[4], const uint32_t (&bh0)[4], const uint32_t (&bl0)[4],
                                       const uint32_t (&bh1)[4], const uint32_t (&bl1)[4]) {
    mma_bf16(d0, ah, bh0[0], bh0[1]); mma_bf16(d1, ah, bh0[2], bh0[3]); mma_bf16(d2, ah, bh1[0], bh1[1]); mma_bf16(d3, ah, bh1[2], bh1[3]);
    mma_bf16(d0, ah, bl0[0], bl0[1]); mma_bf16(d1, ah, bl0[2], bl0[3]); mma_bf16(d2, ah, bl1[0], bl1[1]); mma_bf16(d3, ah, bl1[2], bl1[3]);
    mma_bf16(d0, al, bh0[0], bh0[1]); mma_bf16(d1, al, bh0[2], bh0[3]); mma_bf16(d2, al, bh1[0], bh1[1]); mma_bf16(d3, al, bh1[2], bh1[3]);
}
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
// two fp32 values -> bf16x2 hi word and bf16x2 lo word (first value in the low half)
__device__ __forceinline__ void split2(float v0, float v1, uint32_t& hi, uint32_t& lo) {
    __nv_bfloat162 h = __floats2bfloat162_rn(v0, v1);
    const float2 hf = __bfloat1622float2(h);
    __nv_bfloat162 l = __floats2bfloat162_rn(v0 - hf.x, v1 - hf.y);
    hi = *reinterpret_cast<uint32_t*>(&h);
    lo = *reinterpret_cast<uint32_t*>(&l);
}
__device__ __forceinline__ float2 unpack2(uint32_t w) {
    return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
}
__device__ __forceinline__ void split_bf16(float v, __nv_bfloat16& hi, __nv_bfloat16& lo) {
    hi = __float2bfloat16_rn(v);
    lo = __float2bfloat16_rn(v - __bfloat162float(hi));
}

// Shared memory of a CTA (69 KiB: three CTAs per SM).  The five bulk tensor copies of a chunk land in rx, rth, rB, rC, rz
// (dense boxes).  The operand tiles of the tensor-core products are then written IN PLACE over the raw rows they were
// computed from — token i's raw B row (256 bytes) becomes B~ hi (first 128 bytes) and B~ lo (last 128 bytes) of token i,
// the same for C, silu(x) transposed replaces the raw x rows, the gate replaces z — so no operand tile needs memory of
// its own.  Inside a 128-byte row the eight 16-byte chunks are XOR-ed with (row % 8) so that ldmatrix and the fragment
// stores stay free of bank conflicts without padding.
struct PfSmem {
    float rx[LCH][32];                 // raw x            -> X^T: [plane hi | lo][p = 32 rows][token, 128 bytes]
    float rth[LCH][32];                // raw theta
    float rB[LCH][64];                 // raw B (group)    -> B~: row = token, [hi 128 bytes | lo 128 bytes]
    float rC[LCH][64];                 // raw C (group)    -> C~: same layout
    float rz[LCH][32];                 // raw z            -> gate silu(z)
    uint8_t St[2 * 32 * 128];          // augmented state S^: [plane hi | lo][p = 32 rows][n, 128 bytes]
    float ell[LCH], eli[LCH], lam[LCH + 4], kap[LCH], wj[LCH], dtp[LCH], rbs[LCH], rcs[LCH];
    float seg[5][32];                  // angle prefix sums at the boundaries of the four 16-token segments
    float cum[32];
    float gam[4][64];                  // this group's BCNorm weights: b gamma, b bias, c gamma, c bias
    unsigned long long bar;
    int ok;
};

// byte offset of bf16 element (row, col) inside a tile whose rows are `pitch` bytes apart and hold 64 bf16 (128 bytes)
// with the 16-byte chunks XOR-ed by row % 8
__device__ __forceinline__ int swz(int row, int col, int pitch) {
    return row * pitch + ((((col >> 3) ^ (row & 7)) << 4) | ((col & 7) << 1));
}

constexpr uint32_t kChunkTxBytes = 3 * LCH * 32 * 4 + 2 * LCH * 64 * 4;

// row r = b * ts + t  of the super-chunk; token ids come from prompt[(t_abs) * batch_total + b_abs]
template <typename WT>
__global__ void embed_rows_kernel(const WT* __restrict__ emb, const uint32_t* __restrict__ prompt, float* __restrict__ x, int D,
                                  int vocab, int ts, int t_abs0, int b_abs0, int batch_total, StepCtl* ctl, const int32_t* __restrict__ lens) {
    const int r = blockIdx.x, b = r / ts, t = r - b * ts;
    if (lens != nullptr && t_abs0 + t >= lens[b_abs0 + b]) {      // padding behind a shorter prompt: never looked at, the row is zero
        for (int k = threadIdx.x; k < D; k += blockDim.x) x[(size_t)r * D + k] = 0.f;
        return;
    }
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
__global__ void gather_last_kernel(const float* __restrict__ xr, float* __restrict__ x, int D, int ts, int b0, const int32_t* __restrict__ lens,
                                   int t_abs0) {
    const int b = blockIdx.x;
    const int idx = lens != nullptr ? lens[b0 + b] - 1 - t_abs0 : ts - 1;      // the sequence's last prompt token, if this slice holds it
    if (idx < 0 || idx >= ts) return;
    for (int k = threadIdx.x; k < D; k += blockDim.x) x[(size_t)(b0 + b) * D + k] = xr[((size_t)b * ts + idx) * D + k];
}

__global__ void __launch_bounds__(128, 3)
ssd_prefill_kernel(const __grid_constant__ CUtensorMap map32, const __grid_constant__ CUtensorMap map64, PrefillArgs a) {
    constexpr int P = 32, N = 64, HN = 32;
    extern __shared__ uint8_t pf_raw[];
    PfSmem& sm = *reinterpret_cast<PfSmem*>((reinterpret_cast<uintptr_t>(pf_raw) + 1023) & ~(uintptr_t)1023);
    const int h = blockIdx.x, b = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g4 = lane >> 2, t4 = lane & 3;               // mma fragment coordinates: row group, column pair
    const int H = a.H, DI = H * P, BC = a.G * N, R = a.ldp;
    const int tsl = a.ts;                                   // rows per sequence in the projection / output arrays
    // tokens this sequence takes from the launch (prompts of different lengths end early; none: the state stays as it is)
    const int ts = a.lens != nullptr ? max(0, min(tsl, a.lens[a.b0 + b] - a.t_abs0)) : tsl;
    if (ts == 0) return;
    const int grp = h / (H / a.G);
    const size_t bh = (size_t)(a.b0 + b) * H + h;
    const float* prow0 = a.proj + (size_t)b * tsl * R;     // first token row of this sequence
    const int off_b = 2 * DI, off_c = off_b + BC, off_dt = off_c + BC;
    const float PI_F = 3.14159265358979323846f;
    const float TWO_PI = 6.28318530717958647692f;
    const float INV_TWO_PI = 0.15915494309189533577f;
    const float dskip = a.dskip[h], dtb = a.dtb[h];
    uint64_t* bar = reinterpret_cast<uint64_t*>(&sm.bar);

    // a wait that expired in an earlier CTA of this launch: do not start new work
    if (a.status != nullptr && (*reinterpret_cast<volatile int32_t*>(a.status) & STATUS_TIMEOUT)) return;

    if (tid == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(bar)));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (tid < HN) sm.cum[tid] = a.cum[bh * HN + tid];
    if (tid < 64) {
        const int c = grp * N + tid;
        sm.gam[0][tid] = a.bg[c]; sm.gam[1][tid] = a.bb[c]; sm.gam[2][tid] = a.cg[c]; sm.gam[3][tid] = a.cb[c];
    }
    __syncthreads();

    auto issue_chunk = [&](int t0) {               // one thread: the five box copies of the chunk starting at token t0
        const int row0 = b * tsl + t0;
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(kChunkTxBytes) : "memory");
        tma_load_2d(&sm.rx[0][0], &map32, bar, h * P, row0);
        tma_load_2d(&sm.rz[0][0], &map32, bar, DI + h * P, row0);
        tma_load_2d(&sm.rth[0][0], &map32, bar, off_dt + 3 * H + h * HN, row0);
        tma_load_2d(&sm.rB[0][0], &map64, bar, off_b + grp * N, row0);
        tma_load_2d(&sm.rC[0][0], &map64, bar, off_c + grp * N, row0);
    };
    uint8_t* const tB = reinterpret_cast<uint8_t*>(&sm.rB[0][0]);     // B~ tile (in place): pitch 256, lo plane at +128
    uint8_t* const tC = reinterpret_cast<uint8_t*>(&sm.rC[0][0]);     // C~ tile (in place)
    uint8_t* const tX = reinterpret_cast<uint8_t*>(&sm.rx[0][0]);     // X^T tile (in place): pitch 128, lo plane at +4096
    uint8_t* const tS = sm.St;                                        // S^ tile: pitch 128, lo plane at +4096
    // per-token scalars of a chunk, requested into registers one chunk ahead (threads 0..63: own token; thread 64:
    // lambda of the token after the chunk)
    float n_dt = 0.f, n_lam = 0.f, n_a = 0.f, n_rb = 0.f, n_rc = 0.f;
    auto request_scalars = [&](int t0) {
        if (tid < LCH && t0 + tid < ts) {
            const float* pr = prow0 + (size_t)(t0 + tid) * R;
            const size_t row = (size_t)b * tsl + t0 + tid;
            n_dt = pr[off_dt + h]; n_lam = pr[off_dt + H + h]; n_a = pr[off_dt + 2 * H + h];
            n_rb = a.rb[row]; n_rc = a.rc[row];
        } else if (tid == LCH && t0 + LCH < ts) {
            n_lam = prow0[(size_t)(t0 + LCH) * R + off_dt + H + h];
        }
    };
    if (tid == 0) issue_chunk(0);
    request_scalars(0);

    // state S^ of this warp: rows p0 + {g4, g4 + 8}, columns n0 + 8 nt + 2 t4 + {0, 1}
    const int p0 = 16 * (warp & 1), n0 = 32 * (warp >> 1);
    float S[4][4];
    {
        const float* hp = a.h + bh * (size_t)(P * N);
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
            const float2 v0 = *reinterpret_cast<const float2*>(hp + (p0 + g4) * N + n0 + 8 * nt + 2 * t4);
            const float2 v1 = *reinterpret_cast<const float2*>(hp + (p0 + g4 + 8) * N + n0 + 8 * nt + 2 * t4);
            S[nt][0] = v0.x; S[nt][1] = v0.y; S[nt][2] = v1.x; S[nt][3] = v1.y;
        }
    }

    // this warp's block of S^ as bf16 hi + lo into the shared tile (B operand of C~ S^T in the next chunk)
    auto store_state_tile = [&]() {
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
            uint32_t hi, lo;
            const int col = n0 + 8 * nt + 2 * t4;
            split2(S[nt][0], S[nt][1], hi, lo);
            *reinterpret_cast<uint32_t*>(tS + swz(p0 + g4, col, 128)) = hi;
            *reinterpret_cast<uint32_t*>(tS + 4096 + swz(p0 + g4, col, 128)) = lo;
            split2(S[nt][2], S[nt][3], hi, lo);
            *reinterpret_cast<uint32_t*>(tS + swz(p0 + g4 + 8, col, 128)) = hi;
            *reinterpret_cast<uint32_t*>(tS + 4096 + swz(p0 + g4 + 8, col, 128)) = lo;
        }
    };

    uint32_t phase = 0;
    // One chunk.  FULL: all 64 tokens are valid, so every "past the end of the sequence" test folds away.
    auto do_chunk = [&](auto full_c, const int t0, const int chunk) -> bool {
        constexpr bool FULL = decltype(full_c)::value;
        const int nv = FULL ? LCH : min(LCH, ts - t0);     // valid tokens in this chunk
        auto valid = [&](int i) { return FULL || i < nv; };
        const bool last_chunk = t0 + LCH >= ts;
        // ---- 0. the chunk's raw rows have landed (one thread waits, bounded; everyone follows its verdict)
        if (tid == 0) sm.ok = mbar_wait(bar, phase, kScanWaitLimitNs) ? 1 : 0;
        // ---- 1. per-token scalars (model.rs:307, 314-317) from the registers requested a chunk earlier
        if (tid < LCH) {
            float dtpv = 0.f, gl = 0.f, lm = 0.f;
            if (valid(tid)) {
                dtpv = softplus_ref(__fadd_rn(n_dt, dtb));
                float av = -softplus_ref(n_a);
                av = fminf(fmaxf(av, -1e6f), -1e-4f);
                gl = __fmul_rn(av, dtpv);                 // log a_t
                lm = sigmoid_ref(n_lam);
            }
            sm.dtp[tid] = dtpv; sm.ell[tid] = gl; sm.lam[tid] = lm;
            sm.rbs[tid] = n_rb; sm.rcs[tid] = n_rc;
        }
        if (tid == LCH) sm.lam[LCH] = (t0 + LCH < ts) ? sigmoid_ref(n_lam) : -1.0f;      // < 0: no next token in this launch
        __syncthreads();
        if (!sm.ok) return false;
        phase ^= 1;
        if (!last_chunk) request_scalars(t0 + LCH);        // the next chunk's scalars travel while this chunk is computed
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
            if (valid(i)) {
                const float ln = valid(i + 1) && i + 1 < LCH ? sm.lam[i + 1] : ((nv == LCH) ? sm.lam[LCH] : -1.0f);
                k = (ln < 0.f) ? sm.lam[i] : __fadd_rn(sm.lam[i], __fsub_rn(1.0f, ln));
            }
            sm.kap[i] = k;
            sm.wj[i] = __expf(sm.ell[LCH - 1] - sm.ell[i]) * k;
            sm.eli[i] = __expf(sm.ell[i]);
        }
        if (chunk == 0) {
            // S^_in = S + (1 - lam_first) x_prev (x) B~_prev   (prev_bx of the decode state, model.rs:359)
            const float oml = __fadd_rn(__fmul_rn(sm.lam[0], -1.0f), 1.0f);
            const float xp0 = a.xprev[bh * P + p0 + g4] * oml, xp1 = a.xprev[bh * P + p0 + g4 + 8] * oml;
#pragma unroll
            for (int nt = 0; nt < 4; ++nt) {
                const float2 bp = *reinterpret_cast<const float2*>(a.bprev + bh * N + n0 + 8 * nt + 2 * t4);
                S[nt][0] = fmaf(xp0, bp.x, S[nt][0]); S[nt][1] = fmaf(xp0, bp.y, S[nt][1]);
                S[nt][2] = fmaf(xp1, bp.x, S[nt][2]); S[nt][3] = fmaf(xp1, bp.y, S[nt][3]);
            }
            store_state_tile();
        }
        // ---- 2. thread (lane, warp) takes column `lane` (angle pair k, head dim p) of the warp's 16 tokens: angles, rotated
        //         B~ and C~ (one sin / cos for both), silu(x) transposed, gate.  Every raw row is read only by the warp that owns
        //         its token, so a row can be overwritten by its operand tile after a warp-level barrier.
        {
            const int k = lane, i0 = 16 * warp;
            float loc[16], run = 0.f;
#pragma unroll
            for (int ii = 0; ii < 16; ++ii) {
                const float d = sm.dtp[i0 + ii] * (tanh_fast(sm.rth[i0 + ii][k]) * PI_F);      // model.rs:341-342; dtp = 0 past the end
                run += d;
                loc[ii] = run;
            }
            sm.seg[warp + 1][k] = run;
            // x -> silu (registers; the tile is written after every warp has read its raw x) ; z -> gate in place
            const int p = lane;
            float xs[16];
#pragma unroll
            for (int ii = 0; ii < 16; ++ii) {
                const int i = i0 + ii;
                xs[ii] = valid(i) ? silu_fast(sm.rx[i][p]) : 0.f;                              // model.rs:310
                sm.rz[i][p] = valid(i) ? silu_fast(sm.rz[i][p]) : 0.f;                         // model.rs:370
                if (last_chunk && i == nv - 1) a.xprev[bh * P + p] = xs[ii];                   // hand-over: x of the launch's last token
            }
            __syncthreads();
            if (tid < 32) {
                float off = sm.cum[tid];
                sm.seg[0][tid] = off;
                // reduced mod 2 pi at every segment boundary, so sums stay small and keep their low bits
                for (int s2 = 1; s2 <= 4; ++s2) { off = fmodf(off + sm.seg[s2][tid], TWO_PI); sm.seg[s2][tid] = off; }
                sm.cum[tid] = off;                         // angle after the chunk's last valid token
            }
            // X^T tile over the raw x rows: row p, tokens i0 .. i0 + 15 (two per 32-bit word)
#pragma unroll
            for (int ii = 0; ii < 16; ii += 2) {
                uint32_t hi, lo;
                split2(xs[ii], xs[ii + 1], hi, lo);
                *reinterpret_cast<uint32_t*>(tX + swz(p, i0 + ii, 128)) = hi;
                *reinterpret_cast<uint32_t*>(tX + 4096 + swz(p, i0 + ii, 128)) = lo;
            }
            __syncthreads();
            const float base = sm.seg[warp][k];
            const float bgm0 = sm.gam[0][2 * k], bgm1 = sm.gam[0][2 * k + 1], bbs0 = sm.gam[1][2 * k], bbs1 = sm.gam[1][2 * k + 1];
            const float cgm0 = sm.gam[2][2 * k], cgm1 = sm.gam[2][2 * k + 1], cbs0 = sm.gam[3][2 * k], cbs1 = sm.gam[3][2 * k + 1];
#pragma unroll
            for (int i4 = 0; i4 < 16; i4 += 4) {           // four tokens at a time: all lanes read the raw rows, then overwrite them
                float2 rawb[4], rawc[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    rawb[q] = *reinterpret_cast<const float2*>(&sm.rB[i0 + i4 + q][2 * k]);
                    rawc[q] = *reinterpret_cast<const float2*>(&sm.rC[i0 + i4 + q][2 * k]);
                }
                __syncwarp();
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const int i = i0 + i4 + q;
                    float ang = base + loc[i4 + q];
                    ang -= TWO_PI * rintf(ang * INV_TWO_PI);                 // into [-pi, pi] for the fast sin / cos
                    float b0 = 0.f, b1 = 0.f, c0 = 0.f, c1 = 0.f;
                    if (valid(i)) {
                        const float rb = sm.rbs[i], rc = sm.rcs[i];
                        const float nb0 = fmaf(rawb[q].x * rb, bgm0, bbs0), nb1 = fmaf(rawb[q].y * rb, bgm1, bbs1);      // model.rs:311-313
                        const float nc0 = fmaf(rawc[q].x * rc, cgm0, cbs0), nc1 = fmaf(rawc[q].y * rc, cgm1, cbs1);
                        float sa, ca;
                        __sincosf(ang, &sa, &ca);
                        b0 = ca * nb0 - sa * nb1;                            // model.rs:345-348
                        b1 = sa * nb0 + ca * nb1;
                        c0 = ca * nc0 - sa * nc1;
                        c1 = sa * nc0 + ca * nc1;
                        if (last_chunk && i == nv - 1) {                     // hand-over: B~ of the launch's last token, in fp32
                            a.bprev[bh * N + 2 * k] = b0;
                            a.bprev[bh * N + 2 * k + 1] = b1;
                        }
                    }
                    uint32_t hi, lo;
                    split2(b0, b1, hi, lo);
                    *reinterpret_cast<uint32_t*>(tB + swz(i, 2 * k, 256)) = hi;
                    *reinterpret_cast<uint32_t*>(tB + 128 + swz(i, 2 * k, 256)) = lo;
                    split2(c0, c1, hi, lo);
                    *reinterpret_cast<uint32_t*>(tC + swz(i, 2 * k, 256)) = hi;
                    *reinterpret_cast<uint32_t*>(tC + 128 + swz(i, 2 * k, 256)) = lo;
                }
                __syncwarp();
            }
        }
        __syncthreads();
        // ---- 2b. this warp's C~ rows as A fragments (hi, lo) from its own rows of the tile
        uint32_t Ch[4][4], Cl[4][4];
        {
            const int lm = lane >> 3, lr = lane & 7;
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
                const int row = 16 * warp + 8 * (lm & 1) + lr, col = 16 * ks + 8 * (lm >> 1);
                ldsm_x4(Ch[ks], tC + swz(row, col, 256));
                ldsm_x4(Cl[ks], tC + 128 + swz(row, col, 256));
            }
        }
        // ---- 3. Y2 = C~ S^_in^T, G = C~ B~^T (causal part), W = mask / decay (G) (+ D on the diagonal), Y1 = W X
        float y1[4][4], y2[4][4];
#pragma unroll
        for (int nt = 0; nt < 4; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) { y1[nt][e] = 0.f; y2[nt][e] = 0.f; }
        {
            // ldmatrix row address of this lane inside a [rows][TSB] tile: matrix m = lane / 8, row r = lane % 8
            const int lm = lane >> 3, lr = lane & 7;
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
                uint32_t sh0[4], sl0[4], sh1[4], sl1[4];   // p tiles 0, 1 and 2, 3
                const int row = 8 * (lm >> 1) + lr, col = 16 * ks + 8 * (lm & 1);
                ldsm_x4(sh0, tS + swz(row, col, 128));
                ldsm_x4(sl0, tS + 4096 + swz(row, col, 128));
                ldsm_x4(sh1, tS + swz(row + 16, col, 128));
                ldsm_x4(sl1, tS + 4096 + swz(row + 16, col, 128));
                mma3x4(y2[0], y2[1], y2[2], y2[3], Ch[ks], Cl[ks], sh0, sl0, sh1, sl1);
            }
            const int ia = 16 * warp + g4, ib = ia + 8;
            const float ella = sm.ell[ia], ellb = sm.ell[ib];
            for (int jp = 0; jp <= warp; ++jp) {           // token columns 16 jp .. 16 jp + 15
                // six independent accumulation chains (hi*hi, hi*lo, lo*hi of the two 8-column tiles), added at the end
                float g0[4] = {0.f, 0.f, 0.f, 0.f}, g1[4] = {0.f, 0.f, 0.f, 0.f};
                float g0b[4] = {0.f, 0.f, 0.f, 0.f}, g1b[4] = {0.f, 0.f, 0.f, 0.f}, g0c[4] = {0.f, 0.f, 0.f, 0.f}, g1c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int ks = 0; ks < 4; ++ks) {
                    uint32_t bh4[4], bl4[4];
                    const int row = 16 * jp + 8 * (lm >> 1) + lr, col = 16 * ks + 8 * (lm & 1);
                    ldsm_x4(bh4, tB + swz(row, col, 256));
                    ldsm_x4(bl4, tB + 128 + swz(row, col, 256));
                    mma_bf16(g0, Ch[ks], bh4[0], bh4[1]);
                    mma_bf16(g1, Ch[ks], bh4[2], bh4[3]);
                    mma_bf16(g0b, Ch[ks], bl4[0], bl4[1]);
                    mma_bf16(g1b, Ch[ks], bl4[2], bl4[3]);
                    mma_bf16(g0c, Cl[ks], bh4[0], bh4[1]);
                    mma_bf16(g1c, Cl[ks], bh4[2], bh4[3]);
                }
#pragma unroll
                for (int e = 0; e < 4; ++e) { g0[e] += g0b[e] + g0c[e]; g1[e] += g1b[e] + g1c[e]; }
                // element e of tile q: row (e < 2 ? ia : ib), column 16 jp + 8 q + 2 t4 + (e & 1)
                float wv[2][4];
#pragma unroll
                for (int q = 0; q < 2; ++q)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int i = (e < 2) ? ia : ib, j = 16 * jp + 8 * q + 2 * t4 + (e & 1);
                        const float gv = q == 0 ? g0[e] : g1[e];
                        float w = 0.f;
                        if (j < i) w = gv * __expf(((e < 2) ? ella : ellb) - sm.ell[j]) * sm.kap[j];
                        else if (j == i) w = fmaf(gv, sm.lam[i], dskip);          // lam_i (C~_i . B~_i) x_i + D x_i
                        wv[q][e] = w;
                    }
                uint32_t wh[4], wl[4];
                split2(wv[0][0], wv[0][1], wh[0], wl[0]);
                split2(wv[0][2], wv[0][3], wh[1], wl[1]);
                split2(wv[1][0], wv[1][1], wh[2], wl[2]);
                split2(wv[1][2], wv[1][3], wh[3], wl[3]);
                {
                    uint32_t xh0[4], xl0[4], xh1[4], xl1[4];
                    const int row = 8 * (lm >> 1) + lr, col = 16 * jp + 8 * (lm & 1);
                    ldsm_x4(xh0, tX + swz(row, col, 128));
                    ldsm_x4(xl0, tX + 4096 + swz(row, col, 128));
                    ldsm_x4(xh1, tX + swz(row + 16, col, 128));
                    ldsm_x4(xl1, tX + 4096 + swz(row + 16, col, 128));
                    mma3x4(y1[0], y1[1], y1[2], y1[3], wh, wl, xh0, xl0, xh1, xl1);
                }
            }
            // y = Y1 + e^{l_i} Y2, gated; four lanes of a quad exchange words so that each stores 16 bytes of a row
            const float ela = sm.eli[ia], elb = sm.eli[ib];
            uint32_t oh[2][4], ol[2][4];                   // [row a / b][p tile]
#pragma unroll
            for (int nt = 0; nt < 4; ++nt) {
                const float2 ga = *reinterpret_cast<const float2*>(&sm.rz[ia][8 * nt + 2 * t4]);
                const float2 gb = *reinterpret_cast<const float2*>(&sm.rz[ib][8 * nt + 2 * t4]);
                split2(fmaf(ela, y2[nt][0], y1[nt][0]) * ga.x, fmaf(ela, y2[nt][1], y1[nt][1]) * ga.y, oh[0][nt], ol[0][nt]);
                split2(fmaf(elb, y2[nt][2], y1[nt][2]) * gb.x, fmaf(elb, y2[nt][3], y1[nt][3]) * gb.y, oh[1][nt], ol[1][nt]);
            }
#pragma unroll
            for (int rr = 0; rr < 2; ++rr) {
                const int i = rr == 0 ? ia : ib;
                uint32_t vh[4], vl[4];
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    // step r: this lane hands over its word for p tile (t4 - r) & 3 and receives, from lane (t4 + r) & 3
                    // of its quad, that lane's word for p tile t4
                    const int give = (t4 - r) & 3, from = (lane & ~3) | ((t4 + r) & 3);
                    const uint32_t sh_ = give == 0 ? oh[rr][0] : give == 1 ? oh[rr][1] : give == 2 ? oh[rr][2] : oh[rr][3];
                    const uint32_t sl_ = give == 0 ? ol[rr][0] : give == 1 ? ol[rr][1] : give == 2 ? ol[rr][2] : ol[rr][3];
                    const uint32_t rh = __shfl_sync(0xffffffffu, sh_, from);
                    const uint32_t rl = __shfl_sync(0xffffffffu, sl_, from);
                    const int slot = (t4 + r) & 3;
                    if (slot == 0) { vh[0] = rh; vl[0] = rl; } else if (slot == 1) { vh[1] = rh; vl[1] = rl; }
                    else if (slot == 2) { vh[2] = rh; vl[2] = rl; } else { vh[3] = rh; vl[3] = rl; }
                }
                if (valid(i)) {
                    const size_t o = ((size_t)b * tsl + t0 + i) * DI + h * P + 8 * t4;
                    *reinterpret_cast<uint4*>(a.yhi + o) = make_uint4(vh[0], vh[1], vh[2], vh[3]);
                    if (a.ylo) *reinterpret_cast<uint4*>(a.ylo + o) = make_uint4(vl[0], vl[1], vl[2], vl[3]);
                }
            }
        }
        __syncthreads();                                   // every warp has read S^_in's tile
        // ---- 4. S^_out = e^{l_last} S^_in + (w x)^T B~  for this warp's 16 x 32 block; new S^ tile for the next chunk
        {
            const float el = __expf(sm.ell[LCH - 1]);
#pragma unroll
            for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) S[nt][e] *= el;
            const int lm = lane >> 3, lr = lane & 7;
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {               // tokens 16 ks .. 16 ks + 15
                uint32_t ah[4], al[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int p = p0 + g4 + 8 * (e & 1), j = 16 * ks + 2 * t4 + 8 * (e >> 1);
                    const float2 xh = unpack2(*reinterpret_cast<const uint32_t*>(tX + swz(p, j, 128)));
                    const float2 xl = unpack2(*reinterpret_cast<const uint32_t*>(tX + 4096 + swz(p, j, 128)));
                    split2((xh.x + xl.x) * sm.wj[j], (xh.y + xl.y) * sm.wj[j + 1], ah[e], al[e]);
                }
                {
                    uint32_t bh0[4], bl0[4], bh1[4], bl1[4];   // state columns n0 .. n0 + 15 and n0 + 16 .. n0 + 31
                    const int row = 16 * ks + 8 * (lm & 1) + lr, col = n0 + 8 * (lm >> 1);
                    ldsm_x4_trans(bh0, tB + swz(row, col, 256));
                    ldsm_x4_trans(bl0, tB + 128 + swz(row, col, 256));
                    ldsm_x4_trans(bh1, tB + swz(row, col + 16, 256));
                    ldsm_x4_trans(bl1, tB + 128 + swz(row, col + 16, 256));
                    mma3x4(S[0], S[1], S[2], S[3], ah, al, bh0, bl0, bh1, bl1);
                }
            }
            if (!last_chunk) store_state_tile();
        }
        // every operand tile and raw row of this chunk has been consumed: order these generic-proxy accesses before the copies
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncthreads();
        if (!last_chunk && tid == 0) issue_chunk(t0 + LCH);
        return true;
    };
    bool failed = false;
    {
        int chunk = 0;
        for (int t0 = 0; t0 < ts && !failed; t0 += LCH, ++chunk) {
            const bool okc = (t0 + LCH <= ts) ? do_chunk(std::true_type{}, t0, chunk) : do_chunk(std::false_type{}, t0, chunk);
            failed = !okc;
        }
    }
    if (failed) {
        // the wait gave up: report, let this CTA's copies land (bounded) so nothing writes into shared memory after exit
        if (tid == 0) {
            if (a.status != nullptr) atomicOr(a.status, STATUS_TIMEOUT);
            mbar_wait(bar, phase, kScanWaitLimitNs);
        }
        __syncthreads();
        return;
    }
    // ---- hand-over: the exact decode state after the last token of this launch (kap = lam on it, so S^ = S)
    {
        float* hp = a.h + bh * (size_t)(P * N);
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
            *reinterpret_cast<float2*>(hp + (p0 + g4) * N + n0 + 8 * nt + 2 * t4) = make_float2(S[nt][0], S[nt][1]);
            *reinterpret_cast<float2*>(hp + (p0 + g4 + 8) * N + n0 + 8 * nt + 2 * t4) = make_float2(S[nt][2], S[nt][3]);
        }
    }
    if (tid < HN) a.cum[bh * HN + tid] = sm.cum[tid];
}

}  // namespace

// head_dim 32 and d_state 64 are what the fragments are laid out for; n_heads % 4 keeps every box of the staged
// projection rows on a 16-byte boundary (row pitch and the offsets of the theta columns)
bool prefill_ssd_supported(const Config& c) {
    return c.head_dim() == 32 && c.d_state == 64 && c.n_groups > 0 && c.n_heads % c.n_groups == 0 && c.n_heads % 4 == 0;
}

cudaError_t launch_prefill_embed(const void* emb, int dtype, const uint32_t* prompt, float* x, int D, int vocab, int rows, int ts,
                                 int t_abs0, int b_abs0, int batch_total, StepCtl* ctl, cudaStream_t st, const int32_t* lens) {
    if (dtype == LUMI_DTYPE_BF16)
        embed_rows_kernel<__nv_bfloat16><<<rows, 128, 0, st>>>((const __nv_bfloat16*)emb, prompt, x, D, vocab, ts, t_abs0, b_abs0, batch_total, ctl, lens);
    else
        embed_rows_kernel<float><<<rows, 128, 0, st>>>((const float*)emb, prompt, x, D, vocab, ts, t_abs0, b_abs0, batch_total, ctl, lens);
    return cudaGetLastError();
}

cudaError_t launch_prefill_scan(const PrefillArgs& a, cudaStream_t st) {
    const size_t smem = sizeof(PfSmem) + 1024;
    static bool set = false;
    if (!set) {
        cudaError_t e = cudaFuncSetAttribute(ssd_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        set = true;
    }
    const int rows = a.nb * a.ts;
    // the projection rows as a 2-D fp32 tensor [rows][ldp]; boxes of 64 tokens x 32 columns (x, z, theta) and x 64 (B, C)
    CUtensorMap m32, m64;
    if (make_f32_map_2d(&m32, a.proj, (uint64_t)rows, (uint64_t)a.ldp, (uint64_t)a.ldp * 4, 32, LCH) != LUMI_OK ||
        make_f32_map_2d(&m64, a.proj, (uint64_t)rows, (uint64_t)a.ldp, (uint64_t)a.ldp * 4, 64, LCH) != LUMI_OK)
        return cudaErrorInvalidValue;
    bc_stats_kernel<<<(rows * 32 + 255) / 256, 256, 0, st>>>(a.proj, a.ldp, 2 * a.H * 32, a.G * 64, a.eps, a.rb, a.rc, rows);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    ssd_prefill_kernel<<<dim3(a.H, a.nb), 128, smem, st>>>(m32, m64, a);
    return cudaGetLastError();
}

cudaError_t launch_gather_last(const float* xr, float* x, int D, int ts, int nb, int b0, cudaStream_t st, const int32_t* lens, int t_abs0) {
    gather_last_kernel<<<nb, 256, 0, st>>>(xr, x, D, ts, b0, lens, t_abs0);
    return cudaGetLastError();
}

}  // namespace lumi
