// bf16 x bf16 -> fp32 GEMM on the 5th-generation tensor cores (tcgen05.mma, accumulators in TMEM),
// operands staged by TMA (cp.async.bulk.tensor, 128-byte swizzle, no multicast).
//
//   D[M][N] (+)= A[M][K] * W[N][K]^T        A = activations (batch rows), W = weights as stored
//
// replacing the Linear layers of the reference at batch >= 9 with bf16 weights
// (inference/src/model.rs:299,373,504-506,542,550-553,800; the trainer's cuBLAS call sites
// training/src/native_trainer.rs:220,262,545-548).  Each fp32 activation can be fed as the sum of
// two bf16 values (hi + lo): two MMAs per weight tile into the same accumulator, which keeps ~16
// mantissa bits of the activation while the weight tile is loaded once.
//
// One CTA computes one 128 x BN tile.  Warp 0: TMA producer.  Warp 1: TMEM allocation + MMA issue
// (one elected lane).  Warps 2-5: epilogue (tcgen05.ld -> registers -> global).
// Every wait on an mbarrier is bounded by a wall-clock limit; on expiry the kernel records
// STATUS_TIMEOUT, drains its own copies, frees its TMEM and returns.
#include "internal.h"

#include <cuda.h>
#include <cstdlib>

namespace lumi {

int32_t gemm_tcgen05_init();

namespace {

constexpr int BM = 128;
constexpr int BK = 64;                       // 64 bf16 = 128 bytes = one swizzle atom row
constexpr int kSmemBudget = 196608;          // bytes of pipeline stages
constexpr int kMaxSplits = 4;                // K split over at most this many CTAs
constexpr uint64_t kWaitLimitNs = 500ull * 1000 * 1000;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ uint64_t globaltimer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
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
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, uint64_t limit_ns = kWaitLimitNs) {
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

// K-major operand tile, 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);        // start address, bits [0,14)
    d |= (uint64_t)1 << 16;                             // leading byte offset (unused with swizzle), bits [16,30)
    d |= (uint64_t)(1024 >> 4) << 32;                   // stride byte offset, bits [32,46)
    d |= (uint64_t)1 << 46;                             // descriptor version (Blackwell)
    d |= (uint64_t)2 << 61;                             // layout: SWIZZLE_128B
    return d;
}

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// OCC = CTAs meant to share an SM: with 2, each gets half the stage budget and the epilogue of one
// tile runs under the main loop of the other.
template <int BN, bool SPLIT, int OCC>
struct Tile {
    static constexpr int A_BYTES = BM * BK * 2;                 // 16 KiB
    static constexpr int B_BYTES = BN * BK * 2;
    static constexpr int STAGE = A_BYTES * (SPLIT ? 2 : 1) + B_BYTES;
    static constexpr int STAGES = (kSmemBudget / OCC) / STAGE;
    static constexpr int SMEM = STAGES * STAGE + 1024 /* alignment slack */ + 256 /* barriers */;
    static_assert(STAGES >= 2, "pipeline needs at least two stages");
};

template <int BN, bool SPLIT, int OCC>
__global__ void __launch_bounds__(192, OCC)
gemm_kernel(const __grid_constant__ CUtensorMap map_ahi, const __grid_constant__ CUtensorMap map_alo,
            const __grid_constant__ CUtensorMap map_w, float* __restrict__ D, int ldd, int M, int N, int K,
            int accumulate, int32_t* status) {
    using T = Tile<BN, SPLIT, OCC>;
    constexpr int S = T::STAGES;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(base + S * T::STAGE);
    uint64_t* empty_bar = full_bar + S;
    uint64_t* tmem_full = empty_bar + S;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_full + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * BN, m0 = blockIdx.y * BM;
    const int num_kb = K / BK;

    // a wait that expired in an earlier CTA of this launch: do not start new work
    if (status != nullptr && (*reinterpret_cast<volatile int32_t*>(status) & STATUS_TIMEOUT)) return;

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        mbar_init(tmem_full, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)BN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);

    bool timed_out = false;
    if (warp == 0) {
        if (lane == 0) {
            int issued = 0;
            for (int kb = 0; kb < num_kb; ++kb) {
                const int s = kb % S;
                const uint32_t ph = (uint32_t)(kb / S) & 1u;
                if (!mbar_wait(&empty_bar[s], ph ^ 1u)) { timed_out = true; break; }
                uint8_t* st = base + s * T::STAGE;
                mbar_expect_tx(&full_bar[s], (uint32_t)T::STAGE);
                tma_load_2d(st, &map_ahi, &full_bar[s], kb * BK, m0);
                if (SPLIT) tma_load_2d(st + T::A_BYTES, &map_alo, &full_bar[s], kb * BK, m0);
                tma_load_2d(st + T::A_BYTES * (SPLIT ? 2 : 1), &map_w, &full_bar[s], kb * BK, n0);
                issued = kb + 1;
            }
            if (timed_out) {
                // drain: wait (bounded) for the copies this thread issued and nobody may consume
                for (int kb = max(0, issued - S); kb < issued; ++kb)
                    mbar_wait(&full_bar[kb % S], (uint32_t)(kb / S) & 1u);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
            for (int kb = 0; kb < num_kb; ++kb) {
                const int s = kb % S;
                const uint32_t ph = (uint32_t)(kb / S) & 1u;
                if (!mbar_wait(&full_bar[s], ph)) { timed_out = true; break; }
                tc_fence_after();
                const uint32_t a_hi = smem_u32(base + s * T::STAGE);
                const uint32_t b_addr = a_hi + T::A_BYTES * (SPLIT ? 2 : 1);
#pragma unroll
                for (int k = 0; k < BK / 16; ++k) {
                    // 16 bf16 = 32 bytes along K inside the 128-byte swizzled row
                    umma_bf16(tmem_base, make_smem_desc(a_hi + k * 32), make_smem_desc(b_addr + k * 32), idesc,
                              (kb > 0 || k > 0) ? 1u : 0u);
                }
                if (SPLIT) {
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k)
                        umma_bf16(tmem_base, make_smem_desc(a_hi + T::A_BYTES + k * 32), make_smem_desc(b_addr + k * 32), idesc, 1u);
                }
                umma_commit(&empty_bar[s]);      // arrives when these MMAs have finished reading the stage
            }
            umma_commit(tmem_full);              // arrives when every MMA issued so far has completed
            if (timed_out) mbar_wait(tmem_full, 0);
        }
    } else {
        const int q = warp & 3;                  // TMEM lane quarter this warp may read
        if (!mbar_wait(tmem_full, 0)) timed_out = true;
        timed_out = __any_sync(0xffffffffu, timed_out);     // tcgen05.ld below is warp-collective
        tc_fence_after();
        if (!timed_out) {
            const int row = m0 + q * 32 + lane;
            const bool vec_ok = (ldd & 3) == 0;
#pragma unroll 1
            for (int cb = 0; cb < BN / 32; ++cb) {
                uint32_t r[32];
                tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(cb * 32), r);
                const int col0 = n0 + cb * 32;
                if (row < M && col0 < N) {
                    float* dp = D + (size_t)row * ldd + col0;
                    if (vec_ok && col0 + 32 <= N) {
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            float4 v = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                                   __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
                            if (accumulate) {
                                float4 o = *reinterpret_cast<const float4*>(dp + 4 * j);
                                v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
                            }
                            *reinterpret_cast<float4*>(dp + 4 * j) = v;
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            if (col0 + j < N) {
                                float v = __uint_as_float(r[j]);
                                if (accumulate) v += dp[j];
                                dp[j] = v;
                            }
                        }
                    }
                }
            }
        }
    }
    if (timed_out && status != nullptr) atomicOr(status, STATUS_TIMEOUT);
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)BN) : "memory");
    }
}

// ---- persistent form: one CTA per SM walks over tiles, two accumulators in TMEM ---------------------
// Used when a problem has more tiles than SMs.  The epilogue of tile i (TMEM -> registers -> global)
// runs while the tensor core already works on tile i + 1 in the other accumulator, and TMEM allocation,
// barrier set-up and pipeline fill are paid once per CTA instead of once per tile.  Tiles are numbered
// with the row-tile index fastest, so the CTAs running at the same time share weight tiles in L2.
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

template <int BN, bool SPLIT>
__global__ void __launch_bounds__(192, 1)
gemm_persistent_kernel(const __grid_constant__ CUtensorMap map_ahi, const __grid_constant__ CUtensorMap map_alo,
                       const __grid_constant__ CUtensorMap map_w, float* D, int ldd, int M, int N, int K,
                       int accumulate, int tiles_m, int ntiles, int splits, int32_t* tile_counters, float* scratch, int32_t* status,
                       uint64_t wait_ns, int skip_unit, NormFuse nf) {
    using T = Tile<BN, SPLIT, 1>;
    constexpr int S = T::STAGES;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(base + S * T::STAGE);
    uint64_t* empty_bar = full_bar + S;
    uint64_t* tmem_full = empty_bar + S;          // [2]
    uint64_t* tmem_empty = tmem_full + 2;         // [2]
    uint64_t* drain_bar = tmem_empty + 2;         // failure path only
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(drain_bar + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_kb = K / BK;

    // A successor launched with programmatic dependent launch may become resident now and run the part of its
    // prologue that does not depend on this kernel (the state step requests its state tiles there).
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (status != nullptr && (*reinterpret_cast<volatile int32_t*>(status) & STATUS_TIMEOUT)) return;

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(&tmem_full[i], 1); mbar_init(&tmem_empty[i], 4); }
        mbar_init(drain_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    constexpr uint32_t ACC_COLS = BN > 128 ? 256u : (BN > 64 ? 128u : 64u);      // TMEM columns per accumulator (allocation is a power of two)
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(2u * ACC_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);
    // Launched with programmatic dependent launch (small batches), this CTA may have become resident and done all of the
    // above — barrier set-up, TMEM allocation — while its predecessor (the state step) still ran; everything below reads
    // what predecessors produced.  Without the launch attribute this is a no-op.
    // The weights do not depend on any predecessor: the producer requests the weight tiles of its first stages before the
    // wait, so that they stream from HBM under the predecessor's tail (at 64-128 rows the weights are most of the bytes).
    uint32_t pre = 0;                            // stages whose weight tile is already on its way (and whose bytes are expected)
    if (warp == 0 && lane == 0 && (int)blockIdx.x < ntiles * splits && (int)blockIdx.x != skip_unit) {
        const int t = blockIdx.x / splits, sp = blockIdx.x - t * splits;
        const int n0 = (t / tiles_m) * BN;
        const int kb0 = sp * num_kb / splits, kb1 = (sp + 1) * num_kb / splits;
        pre = (uint32_t)min(S, kb1 - kb0);
        for (uint32_t i = 0; i < pre; ++i) {
            mbar_expect_tx(&full_bar[i], (uint32_t)T::STAGE);
            tma_load_2d(base + i * T::STAGE + T::A_BYTES * (SPLIT ? 2 : 1), &map_w, &full_bar[i], (kb0 + (int)i) * BK, n0);
        }
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");

    bool timed_out = false;
    if (warp == 0) {
        if (lane == 0) {
            uint32_t kbg = 0;                    // k-blocks issued so far, over all tiles of this CTA
            for (int u = blockIdx.x; u < ntiles * splits && !timed_out; u += gridDim.x) {
                if (u == skip_unit) break;       // test hook: this unit's operands never arrive, so the waits below it run out
                const int t = u / splits, sp = u - t * splits;
                const int m0 = (t % tiles_m) * BM, n0 = (t / tiles_m) * BN;
                const int kb0 = sp * num_kb / splits, kb1 = (sp + 1) * num_kb / splits;
                for (int kb = kb0; kb < kb1; ++kb, ++kbg) {
                    const int s = kbg % S;
                    const uint32_t ph = (kbg / S) & 1u;
                    if (!mbar_wait(&empty_bar[s], ph ^ 1u, wait_ns)) { timed_out = true; break; }
                    uint8_t* st = base + s * T::STAGE;
                    if (kbg >= pre) mbar_expect_tx(&full_bar[s], (uint32_t)T::STAGE);
                    tma_load_2d(st, &map_ahi, &full_bar[s], kb * BK, m0);
                    if (SPLIT) tma_load_2d(st + T::A_BYTES, &map_alo, &full_bar[s], kb * BK, m0);
                    if (kbg >= pre) tma_load_2d(st + T::A_BYTES * (SPLIT ? 2 : 1), &map_w, &full_bar[s], kb * BK, n0);
                }
            }
            if (timed_out) {
                // drain: wait (bounded) for the copies this thread issued and nobody may consume
                for (uint32_t k = kbg > (uint32_t)S ? kbg - S : 0; k < kbg; ++k) mbar_wait(&full_bar[k % S], (k / S) & 1u, wait_ns);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
            uint32_t kbg = 0, it = 0;
            for (int u = blockIdx.x; u < ntiles * splits && !timed_out; u += gridDim.x, ++it) {
                const uint32_t as = it & 1u, aph = (it >> 1) & 1u;
                if (!mbar_wait(&tmem_empty[as], aph ^ 1u, wait_ns)) { timed_out = true; break; }     // the epilogue has drained this accumulator
                tc_fence_after();
                const uint32_t acc = tmem_base + as * ACC_COLS;
                const int sp = u % splits;
                const int kb0 = sp * num_kb / splits, kb1 = (sp + 1) * num_kb / splits;
                for (int kb = kb0; kb < kb1; ++kb, ++kbg) {
                    const int s = kbg % S;
                    const uint32_t ph = (kbg / S) & 1u;
                    if (!mbar_wait(&full_bar[s], ph, wait_ns)) { timed_out = true; break; }
                    tc_fence_after();
                    const uint32_t a_hi = smem_u32(base + s * T::STAGE);
                    const uint32_t b_addr = a_hi + T::A_BYTES * (SPLIT ? 2 : 1);
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k)
                        umma_bf16(acc, make_smem_desc(a_hi + k * 32), make_smem_desc(b_addr + k * 32), idesc, (kb > kb0 || k > 0) ? 1u : 0u);
                    if (SPLIT) {
#pragma unroll
                        for (int k = 0; k < BK / 16; ++k)
                            umma_bf16(acc, make_smem_desc(a_hi + T::A_BYTES + k * 32), make_smem_desc(b_addr + k * 32), idesc, 1u);
                    }
                    umma_commit(&empty_bar[s]);
                }
                if (timed_out) break;
                umma_commit(&tmem_full[as]);
            }
            if (timed_out) {                     // let every MMA issued so far finish before TMEM is freed
                umma_commit(drain_bar);
                mbar_wait(drain_bar, 0, wait_ns);         // bounded
            }
        }
    } else {
        const int q = warp & 3;                  // TMEM lane quarter this warp may read
        const bool vec_ok = (ldd & 3) == 0;
        uint32_t it = 0;
        for (int u = blockIdx.x; u < ntiles * splits; u += gridDim.x, ++it) {
            const uint32_t as = it & 1u, aph = (it >> 1) & 1u;
            const int t = u / splits, sp = u - t * splits;
            const int m0 = (t % tiles_m) * BM, n0 = (t / tiles_m) * BN;
            // RMSNorm folded around the product (inference/src/model.rs:100-106 with the per-row scale moved behind the
            // contraction): the rows of A were written as x * gamma WITHOUT the scale 1 / sqrt(mean(x^2) + eps); the
            // sums of squares arrive as `ssq_parts` partial sums per row (one per 32 columns of x, added in column order,
            // so the result does not depend on any tile shape) and the scale multiplies the accumulator below.
            // Read while the tensor core still works on this tile.
            float rs = 1.0f;
            if (nf.ssq_in != nullptr && m0 + q * 32 + lane < M) {
                const float* pp = nf.ssq_in + (size_t)(m0 + q * 32 + lane) * nf.ssq_stride;
                float t = 0.f;
                int pz = 0;
                if ((nf.ssq_stride & 3) == 0) {
                    for (; pz + 16 <= nf.ssq_parts; pz += 16) {          // four 16-byte loads in flight, added in column order
                        const float4 a0 = *reinterpret_cast<const float4*>(pp + pz), a1 = *reinterpret_cast<const float4*>(pp + pz + 4);
                        const float4 a2 = *reinterpret_cast<const float4*>(pp + pz + 8), a3 = *reinterpret_cast<const float4*>(pp + pz + 12);
                        t += a0.x; t += a0.y; t += a0.z; t += a0.w; t += a1.x; t += a1.y; t += a1.z; t += a1.w;
                        t += a2.x; t += a2.y; t += a2.z; t += a2.w; t += a3.x; t += a3.y; t += a3.z; t += a3.w;
                    }
                }
                for (; pz < nf.ssq_parts; ++pz) t += pp[pz];
                rs = __frcp_rn(__fsqrt_rn(__fadd_rn(__fmul_rn(t, nf.inv_k), nf.eps)));
            }
            if (!mbar_wait(&tmem_full[as], aph, wait_ns)) timed_out = true;
            timed_out = __any_sync(0xffffffffu, timed_out);     // tcgen05.ld below is warp-collective
            if (timed_out) break;
            tc_fence_after();
            const int acc_in = accumulate;
            if (splits > 1) {
                // K split over several CTAs: every split parks its partial tile in scratch memory; the warp that
                // arrives last at the counter of its row quarter adds the partials in split order (a fixed order,
                // so the result does not depend on timing) and writes D.  Nobody waits for anybody.
                const int row_l = q * 32 + lane;
                float* part = scratch + ((size_t)(sp * ntiles + t) * BM + row_l) * BN;
#pragma unroll 1
                for (int cb = 0; cb < (BN + 31) / 32; ++cb) {
                    uint32_t r[32];
                    tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + as * ACC_COLS + (uint32_t)(cb * 32), r);
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        if (cb * 32 + 4 * j < BN && m0 + row_l < M)
                            *reinterpret_cast<float4*>(part + cb * 32 + 4 * j) = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                                                                           __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&tmem_empty[as]);
                __threadfence();
                __syncwarp();
                int last = 0;
                if (lane == 0) {
                    const int32_t old = atomicAdd(tile_counters + t * 4 + q, 1);
                    last = old == splits - 1;
                    if (last) atomicExch(tile_counters + t * 4 + q, 0);          // ready for the next launch
                }
                last = __shfl_sync(0xffffffffu, last, 0);
                if (last) {
                    __threadfence();
                    const int row = m0 + row_l;
                    const int nlim = min(N, n0 + BN);
                    if (row < M) {
                        // 16 columns at a time: the residual and every split's partial are requested together, added in
                        // split order, and only then stored (a load behind a store would wait out an L2 round trip)
                        float ssq = 0.f;
                        for (int c16 = 0; c16 < BN; c16 += 16) {
                            const int col = n0 + c16;
                            if (col >= nlim) break;
                            float* dp = D + (size_t)row * ldd + col;
                            const bool vec = (ldd & 3) == 0 && col + 16 <= nlim;
                            float v[16];
                            if (vec) {
                                float4 o[4], pv[kMaxSplits][4];
#pragma unroll
                                for (int j = 0; j < 4; ++j) o[j] = acc_in ? __ldcg(reinterpret_cast<const float4*>(dp + 4 * j)) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                                for (int s2 = 0; s2 < kMaxSplits; ++s2)
#pragma unroll
                                    for (int j = 0; j < 4; ++j)
                                        pv[s2][j] = s2 < splits ? __ldcg(reinterpret_cast<const float4*>(scratch + ((size_t)(s2 * ntiles + t) * BM + row_l) * BN + c16 + 4 * j))
                                                                : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                                for (int j = 0; j < 4; ++j) {
                                    float4 sum = pv[0][j];
#pragma unroll
                                    for (int s2 = 1; s2 < kMaxSplits; ++s2)
                                        if (s2 < splits) { sum.x += pv[s2][j].x; sum.y += pv[s2][j].y; sum.z += pv[s2][j].z; sum.w += pv[s2][j].w; }
                                    v[4 * j] = fmaf(sum.x, rs, o[j].x); v[4 * j + 1] = fmaf(sum.y, rs, o[j].y);
                                    v[4 * j + 2] = fmaf(sum.z, rs, o[j].z); v[4 * j + 3] = fmaf(sum.w, rs, o[j].w);
                                }
#pragma unroll
                                for (int j = 0; j < 4; ++j) *reinterpret_cast<float4*>(dp + 4 * j) = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                            } else {
                                for (int e = 0; e < 16; ++e) {
                                    v[e] = 0.f;
                                    if (col + e < nlim) {
                                        float sum = 0.f;
                                        for (int s2 = 0; s2 < splits; ++s2) sum += __ldcg(scratch + ((size_t)(s2 * ntiles + t) * BM + row_l) * BN + c16 + e);
                                        v[e] = fmaf(sum, rs, acc_in ? __ldcg(dp + e) : 0.f);
                                        dp[e] = v[e];
                                    }
                                }
                            }
                            if (nf.out_hi != nullptr) {
                                // the folded norm's producer side, as in the unsplit epilogue: x * gamma as bf16 hi + lo, x^2 per 32-column strip
                                // N is a multiple of 8 here and tiles start on multiples of 32: groups of 8 columns are whole
#pragma unroll
                                for (int g8 = 0; g8 < 16; g8 += 8) {
                                    if (col + g8 < nlim) {
                                        const float4 ga = __ldg(reinterpret_cast<const float4*>(nf.gamma_next + col + g8));
                                        const float4 gb = __ldg(reinterpret_cast<const float4*>(nf.gamma_next + col + g8 + 4));
                                        const float gg[8] = {ga.x, ga.y, ga.z, ga.w, gb.x, gb.y, gb.z, gb.w};
                                        uint32_t hw[4], lw[4];
#pragma unroll
                                        for (int e = 0; e < 8; e += 2) {
                                            const float x0 = v[g8 + e], x1 = v[g8 + e + 1];
                                            ssq = fmaf(x0, x0, fmaf(x1, x1, ssq));
                                            const float w0 = x0 * gg[e], w1 = x1 * gg[e + 1];
                                            const __nv_bfloat162 h01 = __floats2bfloat162_rn(w0, w1);
                                            const float2 f01 = __bfloat1622float2(h01);
                                            const __nv_bfloat162 l01 = __floats2bfloat162_rn(w0 - f01.x, w1 - f01.y);
                                            hw[e >> 1] = *reinterpret_cast<const uint32_t*>(&h01);
                                            lw[e >> 1] = *reinterpret_cast<const uint32_t*>(&l01);
                                        }
                                        const size_t oo = (size_t)row * N + col + g8;
                                        *reinterpret_cast<uint4*>(nf.out_hi + oo) = make_uint4(hw[0], hw[1], hw[2], hw[3]);
                                        if (nf.out_lo != nullptr) *reinterpret_cast<uint4*>(nf.out_lo + oo) = make_uint4(lw[0], lw[1], lw[2], lw[3]);
                                    }
                                }
                                if (((col + 16) & 31) == 0 || col + 16 >= nlim) { nf.ssq_out[(size_t)row * nf.ssq_stride + (col >> 5)] = ssq; ssq = 0.f; }
                            }
                        }
                    }
                }
                continue;
            }
            const int row = m0 + q * 32 + lane;
#pragma unroll 1
            for (int cb = 0; cb < (BN + 31) / 32; ++cb) {
                uint32_t r[32];
                tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + as * ACC_COLS + (uint32_t)(cb * 32), r);
                const int col0 = n0 + cb * 32;
                const int nlim = min(N, n0 + BN);            // columns of this tile that exist
                float ssq = 0.f;                             // producer side: this row's sum of squares over this 32-column strip
                if (row < M && col0 < nlim) {
                    float* dp = D + (size_t)row * ldd + col0;
                    if (vec_ok && col0 + 32 <= nlim) {
                        // every load of this 32-column strip goes out before the first store: the output pointers may alias
                        // as far as the compiler can tell, and a load behind a store would wait a whole L2 round trip
                        float4 o[8];
#pragma unroll
                        for (int j = 0; j < 8; ++j) o[j] = acc_in ? __ldcg(reinterpret_cast<const float4*>(dp + 4 * j)) : make_float4(0.f, 0.f, 0.f, 0.f);
                        float4 v[8];
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            v[j] = make_float4(fmaf(__uint_as_float(r[4 * j]), rs, o[j].x), fmaf(__uint_as_float(r[4 * j + 1]), rs, o[j].y),
                                               fmaf(__uint_as_float(r[4 * j + 2]), rs, o[j].z), fmaf(__uint_as_float(r[4 * j + 3]), rs, o[j].w));
                        if (nf.out_hi != nullptr) {
                            // the next RMSNorm's input for the next product: x * gamma as bf16 hi + lo (16-byte stores), and x^2 summed
                            float4 gm[8];
#pragma unroll
                            for (int j = 0; j < 8; ++j) gm[j] = __ldg(reinterpret_cast<const float4*>(nf.gamma_next + col0 + 4 * j));
#pragma unroll
                            for (int j = 0; j < 8; ++j) *reinterpret_cast<float4*>(dp + 4 * j) = v[j];
#pragma unroll
                            for (int jj = 0; jj < 4; ++jj) {
                                uint32_t hw[4], lw[4];
#pragma unroll
                                for (int e = 0; e < 2; ++e) {
                                    const float4 vv = v[2 * jj + e], gg = gm[2 * jj + e];
                                    ssq = fmaf(vv.x, vv.x, fmaf(vv.y, vv.y, fmaf(vv.z, vv.z, fmaf(vv.w, vv.w, ssq))));
                                    const float w0 = vv.x * gg.x, w1 = vv.y * gg.y, w2 = vv.z * gg.z, w3 = vv.w * gg.w;
                                    const __nv_bfloat162 h01 = __floats2bfloat162_rn(w0, w1), h23 = __floats2bfloat162_rn(w2, w3);
                                    const float2 f01 = __bfloat1622float2(h01), f23 = __bfloat1622float2(h23);
                                    const __nv_bfloat162 l01 = __floats2bfloat162_rn(w0 - f01.x, w1 - f01.y), l23 = __floats2bfloat162_rn(w2 - f23.x, w3 - f23.y);
                                    hw[2 * e] = *reinterpret_cast<const uint32_t*>(&h01); hw[2 * e + 1] = *reinterpret_cast<const uint32_t*>(&h23);
                                    lw[2 * e] = *reinterpret_cast<const uint32_t*>(&l01); lw[2 * e + 1] = *reinterpret_cast<const uint32_t*>(&l23);
                                }
                                const size_t oo = (size_t)row * N + col0 + 8 * jj;
                                *reinterpret_cast<uint4*>(nf.out_hi + oo) = make_uint4(hw[0], hw[1], hw[2], hw[3]);
                                if (nf.out_lo != nullptr) *reinterpret_cast<uint4*>(nf.out_lo + oo) = make_uint4(lw[0], lw[1], lw[2], lw[3]);
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 8; ++j) *reinterpret_cast<float4*>(dp + 4 * j) = v[j];
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            if (col0 + j < nlim) {
                                float v = __uint_as_float(r[j]) * rs;
                                if (acc_in) v += __ldcg(dp + j);
                                dp[j] = v;
                                if (nf.out_hi != nullptr) {
                                    ssq = fmaf(v, v, ssq);
                                    const float w0 = v * nf.gamma_next[col0 + j];
                                    const __nv_bfloat16 hh = __float2bfloat16_rn(w0);
                                    nf.out_hi[(size_t)row * N + col0 + j] = hh;
                                    if (nf.out_lo != nullptr) nf.out_lo[(size_t)row * N + col0 + j] = __float2bfloat16_rn(w0 - __bfloat162float(hh));
                                }
                            }
                        }
                    }
                    if (nf.out_hi != nullptr) nf.ssq_out[(size_t)row * nf.ssq_stride + (col0 >> 5)] = ssq;
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&tmem_empty[as]);          // this warp has read its quarter of the accumulator

        }
    }
    if (timed_out && status != nullptr) atomicOr(status, STATUS_TIMEOUT);
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(2u * ACC_COLS) : "memory");
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;

// [rows][K] bf16 row-major, box = 64 (K) x box_rows, 128-byte swizzle, out-of-range reads give zeros
int32_t make_map(CUtensorMap* map, const void* ptr, int rows, int K, int box_rows) {
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(LUMI_E_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d (rows %d, K %d)", (int)r, rows, K);
    return LUMI_OK;
}

template <int BN, bool SPLIT, int OCC>
int32_t launch_t(const GemmArgs& a, cudaStream_t st) {
    using T = Tile<BN, SPLIT, OCC>;
    CUtensorMap mh, ml, mw;
    LUMI_TRY(make_map(&mh, a.a_hi, a.M, a.K, BM));
    LUMI_TRY(make_map(&ml, SPLIT ? a.a_lo : a.a_hi, a.M, a.K, BM));
    LUMI_TRY(make_map(&mw, a.w, a.N, a.K, BN));
    auto kern = gemm_kernel<BN, SPLIT, OCC>;
    LUMI_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, T::SMEM));
    dim3 grid((a.N + BN - 1) / BN, (a.M + BM - 1) / BM);
    kern<<<grid, 192, T::SMEM, st>>>(mh, ml, mw, a.d, a.ldd, a.M, a.N, a.K, a.accumulate, a.status_word);
    LUMI_CUDA(cudaGetLastError());
    return LUMI_OK;
}

int sm_count_gemm() {
    static int n = 0;
    if (n == 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
            n = 148;
    }
    return n;
}

template <int BN, bool SPLIT>
int32_t launch_persistent(const GemmArgs& a, int splits, cudaStream_t st) {
    using T = Tile<BN, SPLIT, 1>;
    CUtensorMap mh, ml, mw;
    LUMI_TRY(make_map(&mh, a.a_hi, a.M, a.K, BM));
    LUMI_TRY(make_map(&ml, SPLIT ? a.a_lo : a.a_hi, a.M, a.K, BM));
    LUMI_TRY(make_map(&mw, a.w, a.N, a.K, BN));
    auto kern = gemm_persistent_kernel<BN, SPLIT>;
    LUMI_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, T::SMEM));
    const int tiles_m = (a.M + BM - 1) / BM, tiles_n = (a.N + BN - 1) / BN;
    const int ntiles = tiles_m * tiles_n;
    const int units = ntiles * splits;
    const int grid = units < sm_count_gemm() ? units : sm_count_gemm();
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(192);
    cfg.dynamicSmemBytes = T::SMEM;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = launch_pdl_gemm_on() ? 1 : 0;   // the set-up overlaps the predecessor's tail
    LUMI_CUDA(cudaLaunchKernelEx(&cfg, kern, mh, ml, mw, a.d, a.ldd, a.M, a.N, a.K, a.accumulate, tiles_m, ntiles, splits, a.tile_counters,
                                 a.scratch, a.status_word, a.wait_limit_ns ? a.wait_limit_ns : kWaitLimitNs, a.debug_skip_unit, a.nf));
    return LUMI_OK;
}

}  // namespace

// Row-major fp32 matrix [rows][cols] (row pitch in bytes) as a 2-D tensor map with a dense box_rows x box_cols box,
// no swizzle, zeros for out-of-range elements.  Used by the chunked prefill scan to stage projection rows.
int32_t make_f32_map_2d(CUtensorMap* map, const void* ptr, uint64_t rows, uint64_t cols, uint64_t pitch_bytes, uint32_t box_cols,
                        uint32_t box_rows) {
    LUMI_TRY(gemm_tcgen05_init());
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)pitch_bytes};
    cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(LUMI_E_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d (fp32 %llu x %llu)", (int)r, (unsigned long long)rows, (unsigned long long)cols);
    return LUMI_OK;
}

// bf16 matrix [rows][64] (128-byte rows, dense) as a 2-D tensor map with a box of box_rows whole rows and the 128-byte swizzle
// (the 16-byte chunks of row r land XOR-ed with r % 8).  Used by the attention kernel to stage KV pages.
int32_t make_bf16_map_rows64(CUtensorMap* map, const void* ptr, uint64_t rows, uint32_t box_rows) {
    LUMI_TRY(gemm_tcgen05_init());
    cuuint64_t dims[2] = {64, (cuuint64_t)rows};
    cuuint64_t strides[1] = {128};
    cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(LUMI_E_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d (bf16 rows %llu)", (int)r, (unsigned long long)rows);
    return LUMI_OK;
}

int32_t gemm_tcgen05_init() {
    if (g_encode != nullptr) return LUMI_OK;
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    LUMI_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q));
    if (fn == nullptr || q != cudaDriverEntryPointSuccess)
        return fail(LUMI_E_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    g_encode = reinterpret_cast<EncodeTiledFn>(fn);
    return LUMI_OK;
}

// Tile width of the persistent kernel: the GPU works in rounds of one tile per SM, a round costs about its tile's
// width, so take the width with the least rounds x width (7360 columns x 16 row tiles: 208 -> 4 rounds of 576 tiles,
// against 4 rounds of 464 tiles at 256).  Ties go to the wider tile (less operand traffic per flop).
//
// K is split over 2 or 4 CTAs as well where even the narrowest tiles leave most SMs idle and K is long (out_proj and the
// FFN's second product at 64-128 rows: 32 tiles of 32 columns); the last warp to arrive at a tile adds the parked partial
// tiles in split order.  The estimate behind the choice counts operand bytes per CTA (a k-block is the 128-row activation
// tile, hi and lo, plus the weight rows) and charges the fix-up a round trip through L2 per 16 columns, which is what it
// measures (about 1 us, as much as three k-blocks); a split is taken only where that comes out at least 1.3 times faster
// (measured at 64 x 1024 x 2048: 19.1 us against 23.2 us, +12.6 % tokens per second on the 64-sequence decode; wide split
// tiles lost more in the fix-up than they gained).
// LUMI_GEMM_SPLITK=1 turns splitting off.
static void pick_tile(const GemmArgs& a, int* width, int* splits) {
    static const int widths[] = {256, 224, 208, 192, 160, 128, 96, 64, 32};
    static const int env_splits = getenv("LUMI_GEMM_SPLITK") ? atoi(getenv("LUMI_GEMM_SPLITK")) : kMaxSplits;
    const int max_splits = env_splits < 1 ? 1 : (env_splits > kMaxSplits ? kMaxSplits : env_splits);
    const long tiles_m = (a.M + BM - 1) / BM;
    const int num_kb = a.K / BK;
    const long sms = sm_count_gemm();
    int best = 256;
    long best_cost = -1, best_rounds = 1;
    for (int w : widths) {
        if (a.nf.out_hi != nullptr && (w % 32) != 0) continue;       // the folded norm's partial sums are per 32 aligned columns
        const long tiles = tiles_m * ((a.N + w - 1) / w);
        const long rounds = (tiles + sms - 1) / sms;
        const long cost = rounds * (w + 32);                         // + 32: the part of a tile's time that does not shrink
        if (best_cost < 0 || cost < best_cost) { best = w; best_cost = cost; best_rounds = rounds; }
    }
    *width = best;
    *splits = 1;
    if (max_splits < 2 || tiles_m > 1 || a.tile_counters == nullptr || a.scratch == nullptr) return;   // one row tile only: 256 rows measured 3 % slower split
    const long a_kb = a.a_lo != nullptr ? 32 : 16;                   // KiB of activations per k-block of a 128-row tile
    const long unsplit = best_rounds * num_kb * (a_kb + best / 8);   // KiB through one CTA
    long best_split = -1;
    for (int w : {64, 32}) {
        const long tiles = tiles_m * ((a.N + w - 1) / w);
        for (int sp = 2; sp <= max_splits; sp *= 2) {
            if (tiles * sp > sms || num_kb / sp < 8 || 4 * tiles > a.n_counters || (size_t)sp * tiles * BM * w > a.scratch_floats) break;
            const long est = (num_kb + sp - 1) / sp * (a_kb + w / 8) + 110 * (w / 16) + 110;
            if (13 * est <= 10 * unsplit && (best_split < 0 || est < best_split)) { best_split = est; *width = w; *splits = sp; }
        }
    }
}

// The tile width and K split launch_gemm_tcgen05 would take for these arguments (host-side choice only; nothing is launched).
void gemm_tcgen05_plan(const GemmArgs& a, int* width, int* splits) { pick_tile(a, width, splits); }

int32_t launch_gemm_tcgen05(const GemmArgs& a, cudaStream_t st) {
    if (a.M <= 0 || a.N <= 0 || a.K <= 0 || (a.K % BK) != 0)
        return fail(LUMI_E_UNSUPPORTED, "tcgen05 GEMM needs K %% 64 == 0 (M %d N %d K %d)", a.M, a.N, a.K);
    if ((reinterpret_cast<uintptr_t>(a.a_hi) | reinterpret_cast<uintptr_t>(a.w) | reinterpret_cast<uintptr_t>(a.a_lo)) & 15)
        return fail(LUMI_E_INVALID, "tcgen05 GEMM operands must be 16-byte aligned");
    LUMI_TRY(gemm_tcgen05_init());
    const bool split = a.a_lo != nullptr;
    const bool fused = a.nf.ssq_in != nullptr || a.nf.out_hi != nullptr;
    if (a.nf.out_hi != nullptr && ((a.N & 7) != 0 || a.nf.gamma_next == nullptr || a.nf.ssq_out == nullptr || a.nf.ssq_stride * 32 < a.N))
        return fail(LUMI_E_INVALID, "folded RMSNorm output needs N %% 8 == 0, the next norm's weights and room for N / 32 partial sums per row");
    // LUMI_GEMM_MODE (tuning aid): 0 = default choice, 1 = 128-wide tiles two CTAs per SM, 2 = 128-wide one CTA per SM,
    // 3 = 256-wide one CTA per SM
    static const int mode = getenv("LUMI_GEMM_MODE") ? atoi(getenv("LUMI_GEMM_MODE")) : 0;
    if (!fused) {
        if (mode == 1) return split ? launch_t<128, true, 2>(a, st) : launch_t<128, false, 2>(a, st);
        if (mode == 2) return split ? launch_t<128, true, 1>(a, st) : launch_t<128, false, 1>(a, st);
        if (mode == 3) return split ? launch_t<256, true, 1>(a, st) : launch_t<256, false, 1>(a, st);
    }
    // wide tiles when the problem has enough of them to fill the GPU; more than one tile per SM: persistent CTAs
    const long tiles256 = (long)((a.N + 255) / 256) * ((a.M + BM - 1) / BM);
    static const int persist = getenv("LUMI_GEMM_PERSIST") ? atoi(getenv("LUMI_GEMM_PERSIST")) : 1;     // 0: tuning aid
    if (persist || fused) {
        int best = 256, best_splits = 1;
        pick_tile(a, &best, &best_splits);
#define LUMI_PERSIST_CASE(W) if (best == W) return split ? launch_persistent<W, true>(a, best_splits, st) : launch_persistent<W, false>(a, best_splits, st);
        LUMI_PERSIST_CASE(256) LUMI_PERSIST_CASE(224) LUMI_PERSIST_CASE(208) LUMI_PERSIST_CASE(192) LUMI_PERSIST_CASE(160) LUMI_PERSIST_CASE(128)
        LUMI_PERSIST_CASE(96) LUMI_PERSIST_CASE(64) LUMI_PERSIST_CASE(32)
#undef LUMI_PERSIST_CASE
    }
    if (tiles256 >= 148) return split ? launch_t<256, true, 1>(a, st) : launch_t<256, false, 1>(a, st);
    return split ? launch_t<128, true, 1>(a, st) : launch_t<128, false, 1>(a, st);
}

}  // namespace lumi
