// Batch-1 decode as ONE persistent kernel per call (Mamba-only models, head_dim 32, d_state 64).
//
// At batch 1 a decode step is 2 GB of weights behind ~150 tiny dependent kernels: launch gaps and
// the cold start of every kernel leave HBM idle most of the time.  Here one CTA per SM lives for the
// whole call.  Warp 0 of each CTA streams that CTA's slice of every weight matrix — in_proj rows,
// out_proj rows, lm_head rows, layer after layer, token after token — through a shared-memory ring
// with bulk asynchronous copies (cp.async.bulk + mbarrier), running ahead of the arithmetic by the
// depth of the ring, so the HBM stream never waits for a dependency.  Warps 1-12 consume the ring
// (one fixed warp per ring slot), warps 1-15 share the rest of the work:
//   phase A  in_proj rows of this CTA  x  RMSNorm(x)            -> proj (global)
//   phase B  CTAs 0..H-1: the Mamba-3 state step of one head    -> y (global)     [model.rs:301-370]
//   phase C  out_proj rows of this CTA x y + residual           -> x (global)
//   head     final norm, lm_head rows, per-CTA argmax partials; CTA 0 picks the token
// Phases hand their results to each other as epoch-tagged 64-bit words that the consumers poll (no
// grid barrier per phase); only the token pick uses counter barriers.  Every wait — ring mbarriers,
// tagged polls and counter barriers — is bounded by wall-clock time; on expiry the CTA raises a global
// abort flag that all other waits poll, copies in flight are drained, and the kernel returns with
// STATUS_TIMEOUT in the control block.  The kernel is launched cooperatively, so all CTAs are
// co-resident and the barriers cannot starve.
//
// Arithmetic and operation order inside a phase are those of the kernel-chain path (kernels.cu);
// dot products sum per lane in ascending k, then a 5-step xor tree.
#include "internal.h"

#include <cooperative_groups.h>

namespace lumi {

namespace {

constexpr int kStageBytes = 16384;
constexpr int kSlots = 13;
constexpr int kThreads = 512;
constexpr int kConsumerWarps = kThreads / 32 - 1;      // warps 1..15
constexpr int kConsumers = kConsumerWarps * 32;
constexpr uint64_t kWaitNs = 200ull * 1000 * 1000;     // per-wait wall-clock limit

struct Smem {
    alignas(128) uint8_t ring[kSlots][kStageBytes];
    alignas(16) float xs[2048];                         // activation vector of phases A / C; raw B | C rows in phase B
    alignas(16) float bt[64], ct[64], xa[32], xp[32], gate[32];
    float red[2][16];
    float amax_v[16];
    int amax_i[16];
    uint64_t full[kSlots], empty[kSlots];
    int token;
    float xown[64];             // this CTA's rows of the residual stream (also kept in global x)
    volatile int wtok[2];       // verdicts of grid waits, alternating
    volatile int fail;          // a consumer warp gave up on a ring wait
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint64_t now_ns() { uint64_t t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t; }
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float sigmoid_ref(float x) { return __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-x))); }
__device__ __forceinline__ float softplus_ref(float x) { return logf(__fadd_rn(expf(x), 1.0f)); }
__device__ __forceinline__ float silu_ref(float x) { return __fdiv_rn(x, __fadd_rn(1.0f, expf(-x))); }
__device__ __forceinline__ float rms_scale(float sumsq, int n, float eps) {
    return __frcp_rn(__fsqrt_rn(__fadd_rn(__fmul_rn(sumsq, (float)(1.0 / (double)n)), eps)));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kConsumers) : "memory"); }

// Grid-wide control words (global memory, zeroed by the host before every launch).
struct GridCtl {
    unsigned cnt_start, cnt_a, cnt_b, cnt_c, cnt_d, cnt_e;
    unsigned abort;
    unsigned diag;        // first self-check that failed: (code << 24) | detail
};

// Bounded wait on a ring barrier; polls the global abort flag.  false = give up.
__device__ __forceinline__ bool ring_wait(uint64_t* bar, uint32_t parity, GridCtl* gc) {
    if (mbar_try(bar, parity)) return true;
    const uint64_t t0 = now_ns();
    for (;;) {
        if (mbar_try(bar, parity)) return true;
        if (*reinterpret_cast<volatile unsigned*>(&gc->abort)) return false;
        if (now_ns() - t0 > kWaitNs) { atomicExch(&gc->abort, 1u); return false; }
    }
}
// Bounded wait until *cnt >= target (one lane polls).  false = give up.
__device__ __forceinline__ bool grid_wait(const unsigned* cnt, unsigned target, GridCtl* gc) {
    if (ld_acquire(cnt) >= target) return true;
    const uint64_t t0 = now_ns();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 32; ++i)            // the clock and the abort word are looked at every 32 polls
            if (ld_acquire(cnt) >= target) return true;
        if (*reinterpret_cast<volatile unsigned*>(&gc->abort)) return false;
        if (now_ns() - t0 > kWaitNs) { atomicExch(&gc->abort, 1u); return false; }
    }
}
// All consumer threads have finished their global writes of this phase -> one arrival.  The release
// of the reduction orders the writes of every consumer thread (seen through the CTA barrier) before it.
__device__ __forceinline__ void grid_arrive(unsigned* cnt, int ctid) {
    consumer_sync();
    if (ctid == 0) asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(cnt) : "memory");
}

// Self-check: records the first violated condition and tells the caller to skip the access.
__device__ __forceinline__ bool guard(bool cond, GridCtl* gc, unsigned code, unsigned detail) {
    if (!cond) {
        atomicCAS(&gc->diag, 0u, (code << 24) | (detail & 0xffffffu));
        atomicExch(&gc->abort, 1u);
    }
    return cond;
}

template <typename WT> struct Elt;
template <> struct Elt<float> {
    static constexpr int PER16 = 4;
    __device__ static __forceinline__ void cvt(const uint4& v, float (&w)[4]) {
        w[0] = __uint_as_float(v.x); w[1] = __uint_as_float(v.y); w[2] = __uint_as_float(v.z); w[3] = __uint_as_float(v.w);
    }
};
template <> struct Elt<__nv_bfloat16> {
    static constexpr int PER16 = 8;
    __device__ static __forceinline__ void cvt(const uint4& v, float (&w)[8]) {
        const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) { w[2 * i] = __uint_as_float(u[i] << 16); w[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u); }
    }
};

__device__ __forceinline__ void rows_of(int c, int G, int total, int& lo, int& hi) {
    lo = (int)((long long)c * total / G);
    hi = (int)((long long)(c + 1) * total / G);
}
__device__ __forceinline__ int items_of(int nrows, int rps) { return (nrows + rps - 1) / rps; }

// One warp: dot products of `nr` staged rows (K elements each) with xs, four rows at a time so that
// four independent accumulation chains hide the shared-memory and FMA latencies.  out(r, value) stores.
template <typename WT, typename F>
__device__ __forceinline__ void warp_rows(const uint8_t* stage, int nr, int K, const float* xs, int lane, F&& out) {
    constexpr int E = Elt<WT>::PER16;
    const int KC = K / E;
    const size_t rowbytes = (size_t)K * sizeof(WT);
    for (int r = 0; r < nr; r += 4) {
        const uint4* w[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) w[q] = reinterpret_cast<const uint4*>(stage + (size_t)min(r + q, nr - 1) * rowbytes);
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 2
        for (int c = lane; c < KC; c += 32) {
            float xv[E];
#pragma unroll
            for (int q = 0; q < E / 4; ++q) {
                const float4 v = *reinterpret_cast<const float4*>(xs + c * E + 4 * q);
                xv[4 * q] = v.x; xv[4 * q + 1] = v.y; xv[4 * q + 2] = v.z; xv[4 * q + 3] = v.w;
            }
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                float f[E];
                Elt<WT>::cvt(w[q][c], f);
#pragma unroll
                for (int e = 0; e < E; ++e) acc[q] = fmaf(f[e], xv[e], acc[q]);
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
            for (int q = 0; q < 4; ++q) acc[q] += __shfl_xor_sync(0xffffffffu, acc[q], o);
        }
        if (lane == 0) {
#pragma unroll
            for (int q = 0; q < 4; ++q) if (r + q < nr) out(r + q, acc[q]);
        }
    }
}

// ---- tagged dataflow ----------------------------------------------------------------------------
// Activations that cross CTAs (x, proj, y) live in global memory as 64-bit words: fp32 value in the
// low half, an epoch number in the high half, written with ONE 64-bit store (single-copy atomic).
// A consumer polls exactly the words it needs until their epoch is the one it expects: readiness
// and data arrive in the same L2 round trip, with no atomics, fences or grid barriers.  Epochs grow
// monotonically across layers, tokens and launches (the host advances the base), so stale words can
// never match.  A word is only overwritten after every reader has finished with it: the next write
// of x / proj / y depends, through the data itself, on all CTAs having consumed the previous one.
__device__ __forceinline__ void put_tagged(unsigned long long* p, float v, uint32_t epoch) {
    const unsigned long long w = ((unsigned long long)epoch << 32) | (unsigned long long)__float_as_uint(v);
    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}
__device__ __forceinline__ unsigned long long ld_tagged(const unsigned long long* p) {
    unsigned long long w;
    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(w) : "l"(p) : "memory");
    return w;
}
// Polls up to NV words (indices idx[i], valid when i < n) until all carry `epoch`; values to val[].
// Bounded: gives up (false) when the abort flag is up or the wall-clock limit passes.
template <int NV>
__device__ __forceinline__ bool poll_tagged(const unsigned long long* base, const int (&idx)[NV], int n, uint32_t epoch,
                                            float (&val)[NV], GridCtl* gc) {
    unsigned pending = (n >= 32) ? 0xffffffffu : ((1u << n) - 1u);
    uint64_t t0 = 0;
    for (int spin = 0;; ++spin) {
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            if (pending & (1u << i)) {
                const unsigned long long w = ld_tagged(base + idx[i]);
                if ((uint32_t)(w >> 32) == epoch) { val[i] = __uint_as_float((uint32_t)w); pending &= ~(1u << i); }
            }
        }
        if (pending == 0) return true;
        if ((spin & 63) == 63) {
            if (*reinterpret_cast<volatile unsigned*>(&gc->abort)) return false;
            if (t0 == 0) t0 = now_ns();
            else if (now_ns() - t0 > kWaitNs) { atomicExch(&gc->abort, 1u); return false; }
        }
    }
}

template <typename WT>
__global__ void __launch_bounds__(kThreads, 1) decode_b1_kernel(B1Args a) {
    extern __shared__ uint8_t smem_raw[];
    Smem& sm = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~(uintptr_t)127);
    GridCtl* gc = reinterpret_cast<GridCtl*>(a.grid_ctl);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int c = blockIdx.x, G = gridDim.x;
    const int D = a.D, DI = a.DI, R = a.R, H = a.H, BC = a.BC, V = a.vocab, L = a.n_layers;
    constexpr int P = 32, N = 64, HN = 32;
    const int rps_in = kStageBytes / (D * (int)sizeof(WT));        // staged rows per ring slot
    const int rps_out = kStageBytes / (DI * (int)sizeof(WT));
    int in_lo, in_hi, out_lo, out_hi, v_lo, v_hi;
    rows_of(c, G, R, in_lo, in_hi);
    rows_of(c, G, D, out_lo, out_hi);
    rows_of(c, G, V, v_lo, v_hi);
    const int items_in = items_of(in_hi - in_lo, rps_in), items_out = items_of(out_hi - out_lo, rps_out);
    const int items_v = items_of(v_hi - v_lo, rps_in);
    unsigned long long* xt = a.xt;       // [D]  residual stream, tagged
    unsigned long long* pt = a.pt;       // [R]  in_proj output, tagged
    unsigned long long* yt = a.yt;       // [DI] gated state-step output, tagged

    if (tid == 0) {
        sm.fail = 0;
        for (int s = 0; s < kSlots; ++s) { mbar_init(&sm.full[s], 1); mbar_init(&sm.empty[s], 1); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();

    // which tokens end with the lm_head: the last prompt position and every decode position
    const int prompt_len = a.ctl->prompt_len, prompt_pos0 = a.ctl->prompt_pos;
    auto need_head = [&](int t) { return a.head_mode != 0 && (prompt_pos0 + t >= prompt_len - 1); };

    if (warp == 0) {
        // ---------------- producer: the whole call's weight stream of this CTA, in consumption order
        if (lane == 0) {
            long long it = 0;
            bool ok = true;
            auto push = [&](const uint8_t* base, int row_lo, int nrows, int rps, size_t rowbytes) {
                for (int r = 0; r < nrows && ok; r += rps) {
                    const int slot = (int)(it % kSlots);
                    const uint32_t ph = (uint32_t)((it / kSlots) & 1);
                    if (!ring_wait(&sm.empty[slot], ph ^ 1u, gc)) { ok = false; break; }
                    const int nr = min(rps, nrows - r);
                    const uint32_t bytes = (uint32_t)(nr * rowbytes);
                    const uint8_t* src = base + (size_t)(row_lo + r) * rowbytes;
                    if (!guard(nr > 0 && bytes <= (uint32_t)kStageBytes && (bytes & 15u) == 0 && (reinterpret_cast<uintptr_t>(src) & 15) == 0 &&
                                   (smem_u32(sm.ring[slot]) & 15u) == 0 && base != nullptr, gc, 1u, (unsigned)(it & 0xffffff))) { ok = false; break; }
                    mbar_expect_tx(&sm.full[slot], bytes);
                    bulk_load(sm.ring[slot], src, bytes, &sm.full[slot]);
                    ++it;
                }
            };
            for (int t = 0; t < a.n_tokens && ok; ++t) {
                for (int l = 0; l < L && ok; ++l) {
                    push(reinterpret_cast<const uint8_t*>(a.layers[l].in_proj), in_lo, in_hi - in_lo, rps_in, (size_t)D * sizeof(WT));
                    push(reinterpret_cast<const uint8_t*>(a.layers[l].out_proj), out_lo, out_hi - out_lo, rps_out, (size_t)DI * sizeof(WT));
                }
                if (need_head(t)) push(reinterpret_cast<const uint8_t*>(a.emb), v_lo, v_hi - v_lo, rps_in, (size_t)D * sizeof(WT));
            }
            // drain: every copy issued must have landed before the CTA may exit
            const long long first = it > kSlots ? it - kSlots : 0;
            for (long long j = first; j < it; ++j) {
                const uint64_t t0 = now_ns();
                while (!mbar_try(&sm.full[j % kSlots], (uint32_t)((j / kSlots) & 1))) {
                    if (now_ns() - t0 > kWaitNs) break;
                }
            }
        }
    } else {
        // ---------------- consumers
        const int cw = warp - 1;                       // 0..14
        const int ctid = tid - 32;                     // 0..479
        long long it_base = 0;                         // ring index of the first item of the current phase
        bool ok = true;
        unsigned ep_head = 0;                          // completed head phases (counter barriers, once per token)

        // Consumes the `nitems` ring items of a phase.  Ring slot s is always consumed by consumer warp s
        // (item index mod kSlots), in order: mbarrier parity waits can only tell adjacent phases apart,
        // so no barrier may ever be waited on by a warp that is a whole round ahead of it.
        auto consume = [&](int nitems, int nrows, int rps, int K, auto&& out) {
            const int first = (int)(((cw - it_base) % kSlots + kSlots) % kSlots);
            for (int j = (cw < kSlots ? first : nitems); j < nitems; j += kSlots) {
                const long long it = it_base + j;
                const int slot = (int)(it % kSlots);
                bool got = true;
                if (lane == 0) got = ring_wait(&sm.full[slot], (uint32_t)((it / kSlots) & 1), gc);
                got = __shfl_sync(0xffffffffu, got ? 1 : 0, 0) != 0;
                if (!got) { sm.fail = 1; break; }
                const int r0 = j * rps, nr = min(rps, nrows - r0);
                if (!guard(nr > 0 && nr <= rps && (size_t)nr * K * sizeof(WT) <= (size_t)kStageBytes && K <= 2048, gc, 2u, (unsigned)j)) { sm.fail = 1; break; }
                warp_rows<WT>(sm.ring[slot], nr, K, sm.xs, lane, [&](int r, float v) { out(r0 + r, v); });
                __syncwarp();
                if (lane == 0) mbar_arrive(&sm.empty[slot]);
            }
            it_base += nitems;
        };
        // CTA-uniform verdict after a step in which some thread may have given up
        auto synced_ok = [&]() {
            consumer_sync();
            if (sm.fail) ok = false;
            return ok;
        };
        int widx = 0;
        auto wait_all = [&](const unsigned* cnt, unsigned target) {       // counter barriers (head phase only)
            const int w = widx & 1;
            ++widx;
            if (ctid == 0) sm.wtok[w] = grid_wait(cnt, target, gc) ? 1 : 0;
            consumer_sync();
            if (sm.wtok[w] == 0) ok = false;
            return ok;
        };
        // Gathers the tagged vector src[0..n) of `epoch` into xs (each thread polls its own words) and,
        // when gamma != null, turns it into RMSNorm(x; gamma) (model.rs:100-106).
        auto gather = [&](const unsigned long long* src, int n, uint32_t epoch, const float* gamma) {
            constexpr int NV = 5;                       // 5 * 480 >= 2048
            int idx[NV];
            float val[NV];
            int cnt = 0;
#pragma unroll
            for (int i = 0; i < NV; ++i) { idx[i] = ctid + i * kConsumers; if (idx[i] < n) cnt = i + 1; else idx[i] = 0; }
            if (!poll_tagged<NV>(src, idx, cnt, epoch, val, gc)) sm.fail = 1;
            float s = 0.f;
#pragma unroll
            for (int i = 0; i < NV; ++i) if (i < cnt) { sm.xs[idx[i]] = val[i]; s = fmaf(val[i], val[i], s); }
            if (gamma != nullptr) {
                s = warp_sum(s);
                if (lane == 0) sm.red[0][cw] = s;
                consumer_sync();
                float tot = 0.f;
#pragma unroll
                for (int w = 0; w < kConsumerWarps; ++w) tot += sm.red[0][w];
                const float r = rms_scale(tot, n, a.eps);
#pragma unroll
                for (int i = 0; i < NV; ++i) if (i < cnt) sm.xs[idx[i]] = __fmul_rn(__fmul_rn(val[i], r), gamma[idx[i]]);
            }
            return synced_ok();
        };

        // optional timestamps: CTA 0 (a head CTA) and CTA 100 (no head), last token only
        const int tsel = (c == 0) ? 0 : (c == 100 ? 1 : -1);
        auto stamp = [&](int t, int l, int i) {
            if (a.timing != nullptr && tsel >= 0 && t == a.n_tokens - 1 && ctid == 0) a.timing[((size_t)tsel * L + l) * 10 + i] = now_ns();
        };

        for (int t = 0; t < a.n_tokens && ok; ++t) {
            const uint32_t ep0 = a.epoch_base + (uint32_t)t * (uint32_t)(L + 1);     // epoch of the embedded token; layer l writes ep0 + l + 1
            // ---- embedding: this CTA publishes its own rows of the residual stream (model.rs:772-773)
            {
                const int pp = prompt_pos0 + t;
                uint32_t tok = (pp < prompt_len) ? a.ctl->prompt[(size_t)pp * a.ctl->batch] : __ldcg(a.tok_cur);
                if (tok >= (uint32_t)V) { if (c == 0 && ctid == 0) atomicOr(&a.ctl->status, STATUS_BAD_TOKEN); tok = 0; }
                const WT* erow = reinterpret_cast<const WT*>(a.emb) + (size_t)tok * D;
                for (int k = out_lo + ctid; k < out_hi; k += kConsumers) {
                    float v;
                    if (sizeof(WT) == 4) v = reinterpret_cast<const float*>(erow)[k];
                    else v = __uint_as_float((uint32_t)reinterpret_cast<const uint16_t*>(erow)[k] << 16);
                    sm.xown[k - out_lo] = v;
                    put_tagged(xt + k, v, ep0);
                }
            }
            for (int l = 0; l < L && ok; ++l) {
                const B1Layer& Ly = a.layers[l];
                const uint32_t ep_in = ep0 + (uint32_t)l, ep_out = ep_in + 1;
                // state of this CTA's head: requested now, long before it is needed
                float4 st[2];
                float4 bpq = make_float4(0.f, 0.f, 0.f, 0.f);
                float cu_old = 0.f;
                const bool head_cta = c < H;
                const int rgrp = cw;                   // consumer warps 0..7 own 4 state rows each
                if (head_cta && rgrp < 8) {
                    const float4* h4 = reinterpret_cast<const float4*>(Ly.h + (size_t)c * P * N) + rgrp * 64;
                    st[0] = __ldcg(h4 + lane);
                    st[1] = __ldcg(h4 + 32 + lane);
                    bpq = __ldcg(reinterpret_cast<const float4*>(Ly.bprev + (size_t)c * N) + (lane & 15));
                }
                if (head_cta && cw == 8) cu_old = __ldcg(Ly.cum + (size_t)c * HN + lane);

                // ---- phase A: proj[rows of this CTA] = in_proj . RMSNorm(x)      (model.rs:297-299)
                stamp(t, l, 0);
                if (!gather(xt, D, ep_in, Ly.norm_g)) break;
                stamp(t, l, 1);
                consume(items_in, in_hi - in_lo, rps_in, D, [&](int r, float v) { put_tagged(pt + in_lo + r, v, ep_out); });
                stamp(t, l, 2);

                // ---- phase B: the state step of head c                             (model.rs:301-370)
                if (head_cta) {
                    consumer_sync();                   // every warp is done with xs (it is reused for B | C below)
                    const unsigned long long* Bt = pt + 2 * DI;
                    const unsigned long long* Ct = Bt + BC;
                    const unsigned long long* dtt = Ct + BC;
                    // raw B and C (BCNorm runs over all of them), and this head's scalars
                    int idx[5];
                    float val[5];
                    int cnt = 0;
#pragma unroll
                    for (int i = 0; i < 5; ++i) { idx[i] = ctid + i * kConsumers; if (idx[i] < 2 * BC) cnt = i + 1; else idx[i] = 0; }
                    if (!poll_tagged<5>(Bt, idx, cnt, ep_out, val, gc)) sm.fail = 1;
                    float sb = 0.f, sc = 0.f;
#pragma unroll
                    for (int i = 0; i < 5; ++i) if (i < cnt) {
                        const bool isb = idx[i] < BC;
                        sm.xs[isb ? idx[i] : 1024 + idx[i] - BC] = val[i];
                        if (isb) sb = fmaf(val[i], val[i], sb); else sc = fmaf(val[i], val[i], sc);
                    }
                    sb = warp_sum(sb); sc = warp_sum(sc);
                    if (lane == 0) { sm.red[0][cw] = sb; sm.red[1][cw] = sc; }
                    int sidx[3] = {c, H + c, 2 * H + c};
                    float sval[3] = {0.f, 0.f, 0.f};
                    if (!poll_tagged<3>(dtt, sidx, 3, ep_out, sval, gc)) sm.fail = 1;
                    // per-head scalars, every thread (model.rs:307, 314-317, 355-359)
                    const float dtp = softplus_ref(__fadd_rn(sval[0], Ly.dtb[c]));
                    float av = -softplus_ref(sval[2]);
                    av = fminf(fmaxf(av, -1e6f), -1e-4f);
                    const float abar = expf(__fmul_rn(av, dtp));
                    const float lam = sigmoid_ref(sval[1]);
                    const float oml = __fadd_rn(__fmul_rn(lam, -1.0f), 1.0f);
                    const float c2 = __fmul_rn(abar, oml);
                    float th = 0.f, xraw = 0.f, zraw = 0.f, xpv = 0.f;
                    float sa = 0.f, ca = 1.f;
                    if (cw == 8) {                     // DD-RoPE angles, one pair per lane (model.rs:338-344); needs only theta and dt
                        int i1[1] = {3 * H + c * HN + lane};
                        float v1[1] = {0.f};
                        if (!poll_tagged<1>(dtt, i1, 1, ep_out, v1, gc)) sm.fail = 1;
                        th = v1[0];
                        const float PI_F = 3.14159265358979323846f;
                        const float TWO_PI = __fmul_rn(2.0f, PI_F);
                        const float angle = __fmul_rn(tanhf(th), PI_F);
                        const float cu = fmodf(__fadd_rn(cu_old, __fmul_rn(dtp, angle)), TWO_PI);
                        Ly.cum[(size_t)c * HN + lane] = cu;
                        sincosf(cu, &sa, &ca);
                    }
                    if (cw == 9) {
                        int i2[2] = {c * P + lane, DI + c * P + lane};
                        float v2[2] = {0.f, 0.f};
                        if (!poll_tagged<2>(pt, i2, 2, ep_out, v2, gc)) sm.fail = 1;
                        xraw = v2[0]; zraw = v2[1];
                        xpv = __ldcg(Ly.xprev + c * P + lane);
                        sm.xa[lane] = silu_ref(xraw); sm.xp[lane] = xpv; sm.gate[lane] = silu_ref(zraw);
                    }
                    if (!synced_ok()) break;
                    stamp(t, l, 4);
                    if (cw == 8) {                     // BCNorm + rotation of this head's group (model.rs:311-312, 345-348)
                        float tb = 0.f, tc = 0.f;
#pragma unroll
                        for (int w = 0; w < kConsumerWarps; ++w) { tb += sm.red[0][w]; tc += sm.red[1][w]; }
                        const float rb = rms_scale(tb, BC, a.eps), rc = rms_scale(tc, BC, a.eps);
                        const int g = c / (H / a.G), k = lane, i0 = g * N + 2 * k;
                        const float b0 = __fadd_rn(__fmul_rn(__fmul_rn(sm.xs[i0], rb), Ly.bg[i0]), Ly.bb[i0]);
                        const float b1 = __fadd_rn(__fmul_rn(__fmul_rn(sm.xs[i0 + 1], rb), Ly.bg[i0 + 1]), Ly.bb[i0 + 1]);
                        const float c0 = __fadd_rn(__fmul_rn(__fmul_rn(sm.xs[1024 + i0], rc), Ly.cg[i0]), Ly.cb[i0]);
                        const float c1 = __fadd_rn(__fmul_rn(__fmul_rn(sm.xs[1024 + i0 + 1], rc), Ly.cg[i0 + 1]), Ly.cb[i0 + 1]);
                        sm.bt[2 * k] = __fsub_rn(__fmul_rn(ca, b0), __fmul_rn(sa, b1));
                        sm.bt[2 * k + 1] = __fadd_rn(__fmul_rn(sa, b0), __fmul_rn(ca, b1));
                        sm.ct[2 * k] = __fsub_rn(__fmul_rn(ca, c0), __fmul_rn(sa, c1));
                        sm.ct[2 * k + 1] = __fadd_rn(__fmul_rn(sa, c0), __fmul_rn(ca, c1));
                    }
                    consumer_sync();
                    if (rgrp < 8) {                    // 4 state rows per warp, 16 lanes per row
                        const int cc = lane & 15, r0 = lane >> 4;
                        const float4 bq = reinterpret_cast<const float4*>(sm.bt)[cc];
                        const float4 cq = reinterpret_cast<const float4*>(sm.ct)[cc];
                        float4* h4 = reinterpret_cast<float4*>(Ly.h + (size_t)c * P * N) + rgrp * 64;
                        const float dsk = Ly.dskip[c];
#pragma unroll
                        for (int i = 0; i < 2; ++i) {
                            const int row = rgrp * 4 + r0 + 2 * i;
                            const float xv = sm.xa[row], xpp = sm.xp[row];
                            float nh, part;
                            nh = __fadd_rn(__fadd_rn(__fmul_rn(abar, st[i].x), __fmul_rn(c2, __fmul_rn(xpp, bpq.x))), __fmul_rn(lam, __fmul_rn(xv, bq.x)));
                            st[i].x = nh; part = __fmul_rn(cq.x, nh);
                            nh = __fadd_rn(__fadd_rn(__fmul_rn(abar, st[i].y), __fmul_rn(c2, __fmul_rn(xpp, bpq.y))), __fmul_rn(lam, __fmul_rn(xv, bq.y)));
                            st[i].y = nh; part = fmaf(cq.y, nh, part);
                            nh = __fadd_rn(__fadd_rn(__fmul_rn(abar, st[i].z), __fmul_rn(c2, __fmul_rn(xpp, bpq.z))), __fmul_rn(lam, __fmul_rn(xv, bq.z)));
                            st[i].z = nh; part = fmaf(cq.z, nh, part);
                            nh = __fadd_rn(__fadd_rn(__fmul_rn(abar, st[i].w), __fmul_rn(c2, __fmul_rn(xpp, bpq.w))), __fmul_rn(lam, __fmul_rn(xv, bq.w)));
                            st[i].w = nh; part = fmaf(cq.w, nh, part);
                            h4[i * 32 + lane] = st[i];
#pragma unroll
                            for (int o = 8; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
                            if (cc == 0) {
                                float yv = __fadd_rn(part, __fmul_rn(dsk, xv));          // model.rs:367-368
                                yv = __fmul_rn(yv, sm.gate[row]);                        // model.rs:370
                                put_tagged(yt + c * P + row, yv, ep_out);
                                Ly.xprev[c * P + row] = xv;
                            }
                        }
                    }
                    // the old B~ was taken into registers by every row warp at the top of the layer
                    if (cw == 10) { Ly.bprev[(size_t)c * N + lane] = sm.bt[lane]; Ly.bprev[(size_t)c * N + 32 + lane] = sm.bt[32 + lane]; }
                    stamp(t, l, 5);
                }

                // ---- phase C: x[rows of this CTA] += out_proj . y                   (model.rs:372-374)
                consumer_sync();                       // xs (and bt / ct readers) are done before y overwrites xs
                if (!gather(yt, DI, ep_out, nullptr)) break;
                stamp(t, l, 7);
                consume(items_out, out_hi - out_lo, rps_out, DI, [&](int r, float v) {
                    const float nx = __fadd_rn(v, sm.xown[r]);        // residual kept on chip: no global round trip
                    sm.xown[r] = nx;
                    put_tagged(xt + out_lo + r, nx, ep_out);
                });
                stamp(t, l, 8);
                consumer_sync();                       // xs is free again for the next gather
                stamp(t, l, 9);
            }
            if (!ok) break;

            // ---- head: final norm, tied lm_head, greedy pick                         (model.rs:783-800, main.rs:142-143)
            const bool head = need_head(t);
            if (head) {
                if (!gather(xt, D, ep0 + (uint32_t)L, a.final_g)) break;
                const int step_now = *reinterpret_cast<volatile int*>(&a.ctl->step);
                float* dump = a.ctl->want_dump ? a.ctl->dump + (size_t)step_now * a.ctl->batch * V : nullptr;
                float bv = -INFINITY;
                int bi = 0x7fffffff;
                consume(items_v, v_hi - v_lo, rps_in, D, [&](int r, float v) {
                    const int idx = v_lo + r;
                    a.logits[idx] = v;
                    if (dump) dump[idx] = v;
                    if (v > bv || (v == bv && idx < bi)) { bv = v; bi = idx; }
                });
                if (lane == 0) { sm.amax_v[cw] = bv; sm.amax_i[cw] = bi; }
                consumer_sync();
                if (sm.fail) { ok = false; break; }
                if (ctid == 0) {
                    for (int w = 1; w < kConsumerWarps; ++w)
                        if (sm.amax_v[w] > bv || (sm.amax_v[w] == bv && sm.amax_i[w] < bi)) { bv = sm.amax_v[w]; bi = sm.amax_i[w]; }
                    a.amax_val[c] = bv;
                    a.amax_idx[c] = bi;
                    // same thread: its partial and (through the barrier above) every logit of this CTA precede the release
                    asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(&gc->cnt_d) : "memory");
                }
                ++ep_head;
                if (c == 0) {
                    if (!wait_all(&gc->cnt_d, ep_head * G)) break;
                    if (cw == 0) {
                        float v = -INFINITY;
                        int i = 0x7fffffff;
                        for (int k = lane; k < G; k += 32) {
                            const float ov = __ldcg(a.amax_val + k);
                            const int oi = __ldcg(a.amax_idx + k);
                            if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
                        }
#pragma unroll
                        for (int o = 16; o > 0; o >>= 1) {
                            const float ov = __shfl_xor_sync(0xffffffffu, v, o);
                            const int oi = __shfl_xor_sync(0xffffffffu, i, o);
                            if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
                        }
                        if (lane == 0 && a.do_argmax) {
                            StepCtl* ctl = a.ctl;
                            const int step = ctl->step;
                            a.tok_cur[0] = (uint32_t)i;
                            if (ctl->record) {
                                ctl->out_tokens[(size_t)step * ctl->batch] = (uint32_t)i;
                                if (!a.finished[0]) {
                                    if ((uint32_t)i == ctl->eos_id && !ctl->ignore_eos) a.finished[0] = 1;   // main.rs:150
                                    else a.out_len[0] += 1;
                                }
                            }
                            ctl->step = step + 1;
                        }
                    }
                    grid_arrive(&gc->cnt_e, ctid);
                }
                if (!wait_all(&gc->cnt_e, ep_head)) break;
            }
        }
        if (c == 0 && ctid == 0) {
            // bookkeeping the chain path does in advance_step_kernel
            int pp = a.ctl->prompt_pos + a.n_tokens;
            a.ctl->prompt_pos = pp < a.ctl->prompt_len ? pp : a.ctl->prompt_len;
        }
    }
    __syncthreads();
    if (tid == 0 && *reinterpret_cast<volatile unsigned*>(&gc->abort)) atomicOr(&a.ctl->status, STATUS_TIMEOUT);
}

}  // namespace

size_t decode_b1_smem_bytes() { return sizeof(Smem) + 128; }

bool decode_b1_supported(const Config& c, int n_attn, int device) {
    if (n_attn > 0 || c.head_dim() != 32 || c.d_state != 64) return false;
    if (c.d_model > 2048 || c.d_inner() > 2048 || c.bc() > 1024 || (c.d_model % 32) || (c.d_inner() % 32)) return false;
    if (c.d_model * 4 > kStageBytes || c.d_inner() * 4 > kStageBytes) return false;
    int coop = 0, sms = 0;
    if (cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, device) != cudaSuccess || !coop) return false;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) return false;
    return c.n_heads <= sms && (c.d_model + sms - 1) / sms + 1 <= 64;
}

cudaError_t launch_decode_b1(const B1Args& a, int w_dtype, int device, cudaStream_t st) {
    int sms = 0;
    cudaError_t e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    if (e != cudaSuccess) return e;
    const size_t smem = decode_b1_smem_bytes();
    void* fn = w_dtype == LUMI_DTYPE_BF16 ? (void*)decode_b1_kernel<__nv_bfloat16> : (void*)decode_b1_kernel<float>;
    e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    int per_sm = 0;
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, fn, kThreads, smem);
    if (e != cudaSuccess) return e;
    if (per_sm < 1) return cudaErrorLaunchOutOfResources;
    e = cudaMemsetAsync(a.grid_ctl, 0, sizeof(GridCtl), st);
    if (e != cudaSuccess) return e;
    B1Args args = a;
    void* params[] = {&args};
    return cudaLaunchCooperativeKernel(fn, dim3(sms), dim3(kThreads), params, smem, st);
}

}  // namespace lumi
