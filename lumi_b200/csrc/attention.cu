// Single-token GQA attention over a paged KV cache, replacing AttentionBlock::forward_step's
// cache append + softmax(q K^T / sqrt(d)) V (inference/src/model.rs:508-538, KvCache::append
// :133-152).  A CTA serves all query heads of a KV head's group, so K and V are read once; the cached
// tokens are walked in tiles with a running softmax, and split over several CTAs when the batch alone
// would not fill the GPU.  The sliding window of the reference (keep the last `window` tokens) is a ring:
// token t lives in slot t % window.  Optional rotary embedding (extension, off by default).
//
// Three kernels: attn_mma_kernel (bf16 cache, 64-wide heads: scores and context on the tensor cores, also the attend pass
// of a prompt slice with several token rows per CTA), attn_decode_kernel (fp32 cache or other head widths: the same walk
// on the CUDA cores), kv_append_kernel (the append pass of a prompt slice).  All stage whole pages in shared memory.
#include "internal.h"

#include <cuda.h>

#include <cmath>

namespace lumi {

int32_t make_bf16_map_rows64(CUtensorMap* map, const void* ptr, uint64_t rows, uint32_t box_rows);     // gemm_tcgen05.cu

namespace {

template <typename T> struct KvIo;
template <> struct KvIo<float> {
    __device__ static float ld(const float* p) { return *p; }
    __device__ static void st(float* p, float v) { *p = v; }
};
template <> struct KvIo<__nv_bfloat16> {
    __device__ static float ld(const __nv_bfloat16* p) { return __bfloat162float(*p); }
    __device__ static void st(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
};

__device__ __forceinline__ void split_bf16(float v, __nv_bfloat16& hi, __nv_bfloat16& lo) {
    hi = __float2bfloat16_rn(v);
    lo = __float2bfloat16_rn(v - __bfloat162float(hi));
}

// Page layout: [page][K|V][kv_head][kPageTokens][head_dim] — the rows one CTA reads (one KV head) are contiguous inside a
// page (64 tokens x head_dim), so its loads walk whole DRAM bursts instead of one quarter of every token row.
template <typename KT>
__device__ __forceinline__ KT* kv_ptr(KT* pool, const int32_t* pt, int slot, int sel, int kv_heads, int kvh, int hd) {
    const int page = pt[slot / kPageTokens];
    return pool + ((((size_t)page * 2 + sel) * kv_heads + kvh) * kPageTokens + (slot % kPageTokens)) * hd;
}

constexpr int kAttnTile = kPageTokens;    // cached tokens scored per pass = one page: the shared-memory footprint does not depend on the context
constexpr int kAttnSliceMin = 256;        // a slice of the context is worth a CTA from this many tokens on
constexpr int kAttnMaxSplits = 16;
constexpr uint64_t kAttnWaitNs = 500000000ull;   // limit of the wait for one staged page

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint64_t timer_ns() { uint64_t t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t; }
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_addr(dst)), "l"(src), "r"(bytes), "r"(smem_addr(bar)) : "memory");
}
// false if the phase did not complete within the limit
__device__ __forceinline__ bool page_wait(uint64_t* bar, uint32_t parity) {
    const uint32_t addr = smem_addr(bar);
    uint32_t done = 0, polls = 0;
    uint64_t t0 = 0;
    while (true) {
        asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
                     : "=r"(done) : "r"(addr), "r"(parity) : "memory");
        if (done) return true;
        if ((++polls & 255u) == 0u) {                   // the clock is read rarely: it is slow to read
            const uint64_t now = timer_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > kAttnWaitNs) return false;
        }
    }
}

// Work is split three ways: token row (x), KV head (y) and, when rows x KV heads would not fill the GPU, a
// contiguous slice of the cached tokens (z).  A KV head's 64 rows of a page are one contiguous block, so thread 0
// brings the K and the V block of each page into a ring of shared-memory stages with one bulk copy each (an mbarrier
// per stage counts the bytes; every wait on it is bounded and reports STATUS_TIMEOUT) while the CTA works on the
// pages that have landed: the copies of the next NST - 1 pages are always in flight.  Every CTA walks its slice in tiles
// of kAttnTile tokens (one page) with a running maximum / sum / context (the usual rescaling when the maximum grows), so the softmax of inference/src/model.rs:535
// is evaluated without ever holding more than one tile of scores.  With one slice the CTA normalises and writes the
// context itself.  With several, each parks (max, sum, unnormalised context) per query head in `part`, and the CTA
// that arrives last at the (row, KV head) counter merges the slices in slice order — a fixed order, so the result
// does not depend on timing; nobody waits for anybody.
// The new token's K / V row is appended to the cache by slice 0; every slice reads that row from its own
// shared-memory copy (rounded through the cache's element type, i.e. the value the cache will hold) instead of from
// the cache, so no CTA depends on another CTA's store.
template <typename KT, int HD, int HPK, int NST>
__global__ void __launch_bounds__(128) attn_decode_kernel(AttnArgs a, KT* pool) {
    __shared__ float qs[HD * HPK];                       // rotated q, head-interleaved [HD][HPK]
    __shared__ float red[4 * HPK * HD];                  // cross-warp reductions
    __shared__ float sc[HPK * kAttnTile];                // scores / weights of the current tile
    __shared__ __align__(16) KT knew[HD], vnew[HD];      // the new token's rows as the cache will hold them
    __shared__ float hsum[HPK];
    __shared__ __align__(8) uint64_t full[NST];          // one per stage: the K and the V block of a page have landed
    __shared__ int32_t pages[64];                        // this sequence's page table (when it fits), so that later requests need no global load
    __shared__ int is_last;
    extern __shared__ __align__(128) unsigned char stage_mem[];      // NST x (K block, V block) of one page of this KV head
    constexpr int BLOCK_ELEMS = kPageTokens * HD;        // elements of one K (or V) block

    const int r = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z, nsplit = gridDim.z;
    const int b = a.b0 + r / a.rows_per_seq;             // sequence slot
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int D = a.n_heads * HD, KV = a.kv_heads * HD;
    const float* q = a.qkv + (size_t)r * a.ldq + (size_t)kvh * HPK * HD;
    const float* kn = a.qkv + (size_t)r * a.ldq + D + kvh * HD;
    const float* vn = kn + KV;
    if (a.row_len != nullptr) {                          // prompts of different lengths: this sequence's prompt has ended
        if (a.phase == 0) {
            const int pp = a.ctl->prompt_pos;
            if (pp < a.ctl->prompt_len && pp >= a.row_len[b]) return;
        } else if (a.pos[b] + r % a.rows_per_seq >= a.row_len[b]) {
            // a row of a prompt slice behind a shorter prompt: nothing to attend to; its output row is zero, so that
            // whatever follows it through the layers stays finite
            for (int i = tid; i < HPK * HD; i += 128) {
                const size_t o = (size_t)r * D + (size_t)kvh * HPK * HD + i;
                if (a.ctx32) a.ctx32[o] = 0.f;
                if (a.chi) { a.chi[o] = __float2bfloat16_rn(0.f); if (a.clo) a.clo[o] = __float2bfloat16_rn(0.f); }
            }
            return;
        }
    }
    const int pos = a.pos[b] + r % a.rows_per_seq;
    const int32_t* pt = a.page_table + (size_t)b * a.pages_per_seq;
    const int cap = a.window > 0 ? min(a.window, a.max_tokens) : a.max_tokens;
    int T, slot_new;
    if (a.window > 0 && a.window <= a.max_tokens) { slot_new = pos % a.window; T = min(pos + 1, a.window); }
    else { slot_new = pos; T = pos + 1; }
    if (pos < 0 || slot_new >= cap || T > cap) {      // position outside the cache (full, or a corrupt position): report, write nothing
        if (tid == 0) atomicOr(&a.ctl->status, STATUS_KV_FULL);
        return;
    }

    // this CTA's slice of the cached tokens, in whole pages; its first pages are requested before anything else is done
    const int per = ((T + nsplit - 1) / nsplit + kPageTokens - 1) / kPageTokens * kPageTokens;
    const int tb = split * per, te = min(T, tb + per);
    const int ntiles = te <= tb ? 0 : (te - tb + kPageTokens - 1) / kPageTokens;
    const bool pages_ok = a.pages_per_seq <= 64;
    auto issue = [&](int i, bool staged) {               // thread 0: page i of the slice into stage i % NST
        const int t00 = tb + i * kPageTokens;
        const uint32_t bytes = (uint32_t)min(kPageTokens, te - t00) * HD * (uint32_t)sizeof(KT);
        const int page = staged ? pages[t00 / kPageTokens] : pt[t00 / kPageTokens];
        const size_t blk = ((size_t)page * 2 * a.kv_heads + kvh) * BLOCK_ELEMS;
        KT* dst = reinterpret_cast<KT*>(stage_mem) + (size_t)(i % NST) * 2 * BLOCK_ELEMS;
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(&full[i % NST])), "r"(2u * bytes) : "memory");
        bulk_g2s(dst, pool + blk, bytes, &full[i % NST]);
        bulk_g2s(dst + BLOCK_ELEMS, pool + blk + (size_t)a.kv_heads * BLOCK_ELEMS, bytes, &full[i % NST]);
    };
    if (tid == 0) {
        for (int j = 0; j < NST; ++j) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_addr(&full[j])));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        for (int i = 0; i < NST && i < ntiles; ++i) issue(i, false);
    }

    // rotary embedding on interleaved pairs at the absolute position (extension), then stage q and the new K / V row
    for (int i = tid; i < HPK * HD / 2; i += 128) {
        const int hq = i / (HD / 2), pr = i % (HD / 2);
        float q0 = q[hq * HD + 2 * pr], q1 = q[hq * HD + 2 * pr + 1];
        if (a.rope_base > 0.f) {
            float inv = powf(a.rope_base, -(float)(2 * pr) / (float)HD);
            float ang = __fmul_rn((float)pos, inv);
            float sa, ca;
            sincosf(ang, &sa, &ca);
            float r0 = __fsub_rn(__fmul_rn(ca, q0), __fmul_rn(sa, q1));
            float r1 = __fadd_rn(__fmul_rn(sa, q0), __fmul_rn(ca, q1));
            q0 = r0; q1 = r1;
        }
        qs[(2 * pr) * HPK + hq] = q0;
        qs[(2 * pr + 1) * HPK + hq] = q1;
    }
    for (int pr = tid; pr < HD / 2 && a.phase != 2; pr += 128) {
        float k0 = kn[2 * pr], k1 = kn[2 * pr + 1];
        if (a.rope_base > 0.f) {
            float inv = powf(a.rope_base, -(float)(2 * pr) / (float)HD);
            float ang = __fmul_rn((float)pos, inv);
            float sa, ca;
            sincosf(ang, &sa, &ca);
            float r0 = __fsub_rn(__fmul_rn(ca, k0), __fmul_rn(sa, k1));
            float r1 = __fadd_rn(__fmul_rn(sa, k0), __fmul_rn(ca, k1));
            k0 = r0; k1 = r1;
        }
        KvIo<KT>::st(&knew[2 * pr], k0);
        KvIo<KT>::st(&knew[2 * pr + 1], k1);
        KvIo<KT>::st(&vnew[2 * pr], vn[2 * pr]);
        KvIo<KT>::st(&vnew[2 * pr + 1], vn[2 * pr + 1]);
        if (split == 0) {                                // KvCache::append (model.rs:133-152)
            KT* kd = kv_ptr(pool, pt, slot_new, 0, a.kv_heads, kvh, HD);
            KT* vd = kv_ptr(pool, pt, slot_new, 1, a.kv_heads, kvh, HD);
            kd[2 * pr] = knew[2 * pr]; kd[2 * pr + 1] = knew[2 * pr + 1];
            vd[2 * pr] = vnew[2 * pr]; vd[2 * pr + 1] = vnew[2 * pr + 1];
        }
    }
    const int local_slot = a.phase == 2 ? -1 : slot_new; // attend only: every row is already in the cache
    if (pages_ok) for (int i = tid; i < a.pages_per_seq; i += 128) pages[i] = pt[i];
    __syncthreads();

    // A cached K row is HD * sizeof(KT) bytes = LPR lanes x 16 bytes, so one warp-wide 16-byte load covers RPI rows;
    // UNR such loads are in flight per lane.  Lane (rg, sub) multiplies its EPL elements of row rg with the same
    // elements of the HPK query heads (kept in registers) and the LPR partial sums of a row are added by a xor tree.
    constexpr int EPL = 16 / (int)sizeof(KT);          // elements per lane per row
    constexpr int LPR = HD / EPL;                      // lanes per row
    constexpr int RPI = 32 / LPR;                      // rows per warp-wide load
    constexpr int UNR = 4;
    static_assert(LPR >= 1 && LPR <= 32 && (32 % LPR) == 0, "a row must be 16 to 512 bytes");
    const int rg = lane / LPR, sub = lane % LPR;
    auto unpack = [](const uint4& raw, float (&f)[EPL]) {
        if constexpr (sizeof(KT) == 4) {
            f[0] = __uint_as_float(raw.x); f[1] = __uint_as_float(raw.y); f[2] = __uint_as_float(raw.z); f[3] = __uint_as_float(raw.w);
        } else {
            const uint32_t u[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) { f[2 * i] = __uint_as_float(u[i] << 16); f[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u); }
        }
    };
    float qr[HPK][EPL];
#pragma unroll
    for (int hq = 0; hq < HPK; ++hq)
#pragma unroll
        for (int e = 0; e < EPL; ++e) qr[hq][e] = qs[(sub * EPL + e) * HPK + hq];
    const float scale = (float)(1.0 / sqrt((double)HD));            // model.rs:530

    float m_run[HPK], lsum[HPK], ctx[HPK][EPL];        // running maximum (uniform), this thread's share of the sum and the context
#pragma unroll
    for (int hq = 0; hq < HPK; ++hq) {
        m_run[hq] = -INFINITY; lsum[hq] = 0.f;
#pragma unroll
        for (int e = 0; e < EPL; ++e) ctx[hq][e] = 0.f;
    }
    bool dead = false;                                   // a staged page did not arrive in time
    int dead_it = 0;
    for (int it = 0; it < ntiles; ++it) {
        const int t00 = tb + it * kAttnTile;
        const int tn = min(kAttnTile, te - t00);        // tokens of this tile
        const KT* kst = reinterpret_cast<const KT*>(stage_mem) + (size_t)(it % NST) * 2 * BLOCK_ELEMS;
        const KT* vst = kst + BLOCK_ELEMS;
        bool ok = page_wait(&full[it % NST], (uint32_t)(it / NST) & 1u);
        if (ok && local_slot >= t00 && local_slot < t00 + tn && tid < 2 * LPR) {
            // the new token's row: the value the cache will hold, from this CTA's own copy (slice 0 is still storing it)
            KT* row = const_cast<KT*>(tid < LPR ? kst : vst) + (size_t)(local_slot - t00) * HD;
            reinterpret_cast<uint4*>(row)[tid % LPR] = reinterpret_cast<const uint4*>(tid < LPR ? knew : vnew)[tid % LPR];
        }
        if (__syncthreads_or(!ok)) { dead = true; dead_it = it; break; }
        auto load_row = [&](int t, int sel) -> uint4 {   // row t of the staged page
            return *reinterpret_cast<const uint4*>((sel == 0 ? kst : vst) + (size_t)t * HD + sub * EPL);
        };
        float lmax[HPK];
#pragma unroll
        for (int hq = 0; hq < HPK; ++hq) lmax[hq] = -INFINITY;
        for (int t0 = warp * RPI; t0 < tn; t0 += 4 * RPI * UNR) {
            uint4 raw[UNR];
#pragma unroll
            for (int u = 0; u < UNR; ++u) {
                const int t = t0 + u * 4 * RPI + rg;
                raw[u] = t < tn ? load_row(t, 0) : make_uint4(0u, 0u, 0u, 0u);
            }
#pragma unroll
            for (int u = 0; u < UNR; ++u) {
                const int t = t0 + u * 4 * RPI + rg;
                float kf[EPL];
                unpack(raw[u], kf);
                float acc[HPK];
#pragma unroll
                for (int hq = 0; hq < HPK; ++hq) {
                    acc[hq] = 0.f;
#pragma unroll
                    for (int e = 0; e < EPL; ++e) acc[hq] = fmaf(qr[hq][e], kf[e], acc[hq]);
#pragma unroll
                    for (int o = LPR / 2; o > 0; o >>= 1) acc[hq] += __shfl_xor_sync(0xffffffffu, acc[hq], o);
                }
                if (sub == 0 && t < tn) {
#pragma unroll
                    for (int hq = 0; hq < HPK; ++hq) {
                        const float sv = __fmul_rn(acc[hq], scale);     // model.rs:532
                        sc[hq * kAttnTile + t] = sv;
                        lmax[hq] = fmaxf(lmax[hq], sv);
                    }
                }
            }
        }
        // tile maximum per head, then the new running maximum and the factor that brings the old sums to it
#pragma unroll
        for (int hq = 0; hq < HPK; ++hq) {
            float v = lmax[hq];
            for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
            if (lane == 0) red[warp * HPK + hq] = v;
        }
        __syncthreads();
#pragma unroll
        for (int hq = 0; hq < HPK; ++hq) {
            const float hmax = fmaxf(fmaxf(red[hq], red[HPK + hq]), fmaxf(red[2 * HPK + hq], red[3 * HPK + hq]));
            const float mn = fmaxf(m_run[hq], hmax);
            const float f = m_run[hq] == -INFINITY ? 0.f : expf(__fsub_rn(m_run[hq], mn));
            m_run[hq] = mn;
            lsum[hq] *= f;
#pragma unroll
            for (int e = 0; e < EPL; ++e) ctx[hq][e] *= f;
        }
        for (int t = tid; t < tn; t += 128) {
#pragma unroll
            for (int hq = 0; hq < HPK; ++hq) {
                const float e = expf(__fsub_rn(sc[hq * kAttnTile + t], m_run[hq]));    // model.rs:535
                sc[hq * kAttnTile + t] = e;
                lsum[hq] += e;
            }
        }
        __syncthreads();
        // context: same lane mapping over the V rows; a lane accumulates its EPL dims over the rows of its row group
        for (int t0 = warp * RPI; t0 < tn; t0 += 4 * RPI * UNR) {
            uint4 raw[UNR];
#pragma unroll
            for (int u = 0; u < UNR; ++u) {
                const int t = t0 + u * 4 * RPI + rg;
                raw[u] = t < tn ? load_row(t, 1) : make_uint4(0u, 0u, 0u, 0u);
            }
#pragma unroll
            for (int u = 0; u < UNR; ++u) {
                const int t = t0 + u * 4 * RPI + rg;
                if (t < tn) {
                    float vf[EPL];
                    unpack(raw[u], vf);
#pragma unroll
                    for (int hq = 0; hq < HPK; ++hq) {
                        const float p = sc[hq * kAttnTile + t];
#pragma unroll
                        for (int e = 0; e < EPL; ++e) ctx[hq][e] = fmaf(p, vf[e], ctx[hq][e]);
                    }
                }
            }
        }
        __syncthreads();                                 // sc, red and this stage are reused from here on
        if (tid == 0 && it + NST < ntiles) {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // the CTA's reads of the stage come before the copy's writes
            issue(it + NST, pages_ok);
        }
    }
    if (dead && tid == 0) {
        // report, and let the copies that are still on their way land (again with a limit) before the shared memory goes away;
        // the CTA then finishes as usual, so that the slice counters stay consistent
        atomicOr(&a.ctl->status, STATUS_TIMEOUT);
        for (int j = dead_it; j < ntiles && j < dead_it + NST; ++j) page_wait(&full[j % NST], (uint32_t)(j / NST) & 1u);
    }
    // block totals: the sums by a xor tree and the four warps in order; the context likewise
#pragma unroll
    for (int hq = 0; hq < HPK; ++hq) {
        float v = lsum[hq];
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if (lane == 0) red[warp * HPK + hq] = v;
    }
    __syncthreads();
    if (tid < HPK) hsum[tid] = (red[tid] + red[HPK + tid]) + (red[2 * HPK + tid] + red[3 * HPK + tid]);
    __syncthreads();
#pragma unroll
    for (int hq = 0; hq < HPK; ++hq)
#pragma unroll
        for (int e = 0; e < EPL; ++e)
#pragma unroll
            for (int o = LPR; o < 32; o <<= 1) ctx[hq][e] += __shfl_xor_sync(0xffffffffu, ctx[hq][e], o);
    if (rg == 0) {
#pragma unroll
        for (int hq = 0; hq < HPK; ++hq)
#pragma unroll
            for (int e = 0; e < EPL; ++e) red[warp * HPK * HD + hq * HD + sub * EPL + e] = ctx[hq][e];
    }
    __syncthreads();
    auto emit = [&](int i, float v) {
        const size_t o = (size_t)r * D + (size_t)kvh * HPK * HD + i;
        if (a.ctx32) a.ctx32[o] = v;
        if (a.chi) {
            __nv_bfloat16 hh, ll;
            split_bf16(v, hh, ll);
            a.chi[o] = hh;
            if (a.clo) a.clo[o] = ll;
        }
    };
    if (nsplit == 1) {
        for (int i = tid; i < HPK * HD; i += 128) {
            const float v = (red[i] + red[HPK * HD + i]) + (red[2 * HPK * HD + i] + red[3 * HPK * HD + i]);
            emit(i, __fdiv_rn(v, hsum[i / HD]));
        }
        return;
    }
    // several slices: park this slice's (max, sum, context) and let the last arriver merge them in slice order
    constexpr int PW = HPK * (HD + 2);                   // floats per slice
    float* mine = a.part + ((size_t)(r * a.kv_heads + kvh) * kAttnMaxSplits + split) * PW;
    for (int i = tid; i < HPK * HD; i += 128)
        mine[2 * HPK + i] = (red[i] + red[HPK * HD + i]) + (red[2 * HPK * HD + i] + red[3 * HPK * HD + i]);
    if (tid < HPK) { mine[tid] = m_run[tid]; mine[HPK + tid] = hsum[tid]; }
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const int old = atomicAdd(a.part_count + r * a.kv_heads + kvh, 1);
        is_last = old == nsplit - 1;
        if (is_last) a.part_count[r * a.kv_heads + kvh] = 0;             // ready for the next launch
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    const float* all = a.part + (size_t)(r * a.kv_heads + kvh) * kAttnMaxSplits * PW;
    for (int i = tid; i < HPK * HD; i += 128) {
        const int hq = i / HD;
        float m = -INFINITY;
        for (int sp = 0; sp < nsplit; ++sp) m = fmaxf(m, __ldcg(all + (size_t)sp * PW + hq));
        float den = 0.f, num = 0.f;
        for (int sp = 0; sp < nsplit; ++sp) {
            const float ms = __ldcg(all + (size_t)sp * PW + hq);
            const float f = ms == -INFINITY ? 0.f : expf(__fsub_rn(ms, m));
            den = fmaf(f, __ldcg(all + (size_t)sp * PW + HPK + hq), den);
            num = fmaf(f, __ldcg(all + (size_t)sp * PW + 2 * HPK + i), num);
        }
        emit(i, __fdiv_rn(num, den));
    }
}

// The append-only pass of a prompt slice (phase 1): one thread per (token row, KV head, pair of dims) rotates the K pair at the
// row's position (extension) and stores the K and the V pair as the cache holds them (KvCache::append, model.rs:133-152).
template <typename KT>
__global__ void __launch_bounds__(256) kv_append_kernel(AttnArgs a, KT* pool, long total) {
    const long i = (long)blockIdx.x * 256 + threadIdx.x;
    if (i >= total) return;
    const int HD = a.head_dim, half = HD / 2;
    const int pr = (int)(i % half), kvh = (int)((i / half) % a.kv_heads), r = (int)(i / ((long)half * a.kv_heads));
    const int b = a.b0 + r / a.rows_per_seq;
    const int pos = a.pos[b] + r % a.rows_per_seq;
    if (a.row_len != nullptr && pos >= a.row_len[b]) return;          // padding behind a shorter prompt
    const int cap = a.window > 0 ? min(a.window, a.max_tokens) : a.max_tokens;
    const int slot = (a.window > 0 && a.window <= a.max_tokens) ? pos % a.window : pos;
    if (pos < 0 || slot >= cap) {
        atomicOr(&a.ctl->status, STATUS_KV_FULL);
        return;
    }
    const float* kn = a.qkv + (size_t)r * a.ldq + (size_t)a.n_heads * HD + (size_t)kvh * HD;
    const float* vn = kn + (size_t)a.kv_heads * HD;
    float k0 = kn[2 * pr], k1 = kn[2 * pr + 1];
    if (a.rope_base > 0.f) {
        float inv = powf(a.rope_base, -(float)(2 * pr) / (float)HD);
        float ang = __fmul_rn((float)pos, inv);
        float sa, ca;
        sincosf(ang, &sa, &ca);
        float x0 = __fsub_rn(__fmul_rn(ca, k0), __fmul_rn(sa, k1));
        float x1 = __fadd_rn(__fmul_rn(sa, k0), __fmul_rn(ca, k1));
        k0 = x0; k1 = x1;
    }
    const int32_t* pt = a.page_table + (size_t)b * a.pages_per_seq;
    KT* kd = kv_ptr(pool, pt, slot, 0, a.kv_heads, kvh, HD);
    KT* vd = kv_ptr(pool, pt, slot, 1, a.kv_heads, kvh, HD);
    KvIo<KT>::st(&kd[2 * pr], k0); KvIo<KT>::st(&kd[2 * pr + 1], k1);
    KvIo<KT>::st(&vd[2 * pr], vn[2 * pr]); KvIo<KT>::st(&vd[2 * pr + 1], vn[2 * pr + 1]);
}

// ---- bf16 cache, head_dim 64: the same walk on the tensor cores ---------------------------------------------
// D (16x8, fp32) += A (16x16, bf16, row) * B (16x8, bf16, col)
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldsm4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm4t(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
// two fp32 values -> bf16x2 hi word and bf16x2 lo word (first value in the low half)
__device__ __forceinline__ void split_pair(float v0, float v1, uint32_t& hi, uint32_t& lo) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(v0, v1);
    const float2 hf = __bfloat1622float2(h);
    const __nv_bfloat162 l = __floats2bfloat162_rn(v0 - hf.x, v1 - hf.y);
    hi = *reinterpret_cast<const uint32_t*>(&h);
    lo = *reinterpret_cast<const uint32_t*>(&l);
}
// byte offset of the 16-byte chunk `chunk` of row `row` in a tile of 128-byte rows stored with the 128-byte swizzle
__device__ __forceinline__ uint32_t swz128(int row, int chunk) { return (uint32_t)(row * 128 + ((chunk ^ (row & 7)) << 4)); }

constexpr int kMmaStages = 3;
constexpr int kMmaStageBytes = 2 * kPageTokens * 128;      // K block + V block of one page of one KV head (head_dim 64, bf16)
constexpr float kMaskedScore = -1.0e30f;                   // finite, so that a fully masked row never produces inf - inf

// One CTA = up to 16 / HPK consecutive token rows of one sequence (one in decode) x the HPK query heads of one KV head:
// 16 "query columns" m = row * HPK + head, the M side of mma.m16n8k16.  Scores S = Q K^T with A = Q (bf16 hi + lo, so
// that fp32 queries lose nothing that matters) and B = the staged K page as it lies ([token][dim] is the col-major B
// operand); the softmax weights of a 16-token strip are already laid out as the A operand of P V (again hi + lo), with
// B = the staged V page through ldmatrix.trans.  The pages arrive by one tensor-map copy each for K and V (128-byte
// swizzle, so ldmatrix meets no bank conflict) into a ring of kMmaStages stages; waits are bounded.  The four warps take
// 16 tokens each of a page and keep their own running maximum / sum / context; they are merged at the end in warp order.
// Rows of a CTA differ in how many cached tokens they may see (row j of a prompt slice sees one token more than row
// j - 1); scores beyond a row's limit are replaced by a large negative constant before the maximum is taken.
template <int HPK>
__global__ void __launch_bounds__(128) attn_mma_kernel(AttnArgs a, const __grid_constant__ CUtensorMap kvmap, int q_rows, int groups_per_seq) {
    constexpr int HD = 64;
    __shared__ __align__(16) __nv_bfloat16 knew[HD], vnew[HD];
    __shared__ __align__(8) uint64_t full[kMmaStages];
    __shared__ int32_t pages[64];
    __shared__ int is_last;
    extern __shared__ unsigned char dyn_raw[];
    // the swizzle pattern repeats every 1024 bytes: stages start on that boundary
    unsigned char* dyn = dyn_raw + ((1024u - (smem_addr(dyn_raw) & 1023u)) & 1023u);
    unsigned char* qtile = dyn + kMmaStages * kMmaStageBytes;       // Q hi [16][64] then Q lo [16][64], swizzled like the pages

    const int grp = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z, nsplit = gridDim.z;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, tq = lane & 3;
    const int ts = a.rows_per_seq;
    const int sidx = grp / groups_per_seq, i0 = (grp % groups_per_seq) * q_rows;
    const int nrow = min(q_rows, ts - i0);                // token rows of this CTA
    const int r0 = sidx * ts + i0;                        // first of them in the projection / output arrays
    const int b = a.b0 + sidx;
    const int D = a.n_heads * HD, KV = a.kv_heads * HD;
    const int pos0 = a.pos[b] + i0;
    int nvalid = nrow;                                   // rows of this CTA that belong to their sequence's prompt
    if (a.row_len != nullptr) {                          // prompts of different lengths
        if (a.phase == 0) {                              // decode form: this sequence's prompt has ended
            const int pp = a.ctl->prompt_pos;
            if (pp < a.ctl->prompt_len && pp >= a.row_len[b]) return;
        } else {
            nvalid = max(0, min(nrow, a.row_len[b] - pos0));
        }
    }
    if (nvalid < nrow) {
        // rows of a prompt slice behind a shorter prompt: nothing to attend to; their output rows are zero, so that
        // whatever follows them through the layers stays finite
        for (int i = tid + nvalid * HPK * HD; i < nrow * HPK * HD; i += 128) {
            const int m = i / HD;
            const size_t oo = (size_t)(r0 + m / HPK) * D + (size_t)(kvh * HPK + m % HPK) * HD + i % HD;
            if (a.ctx32) a.ctx32[oo] = 0.f;
            if (a.chi) { a.chi[oo] = __float2bfloat16_rn(0.f); if (a.clo) a.clo[oo] = __float2bfloat16_rn(0.f); }
        }
        if (nvalid == 0) return;
    }
    const int32_t* pt = a.page_table + (size_t)b * a.pages_per_seq;
    const int cap = a.window > 0 ? min(a.window, a.max_tokens) : a.max_tokens;
    // cached tokens the first row sees; row j sees j more (several rows only without a window: the host takes care of that)
    int T0, slot_new;
    if (a.window > 0 && a.window <= a.max_tokens) { slot_new = pos0 % a.window; T0 = min(pos0 + 1, a.window); }
    else { slot_new = pos0; T0 = pos0 + 1; }
    const int T = T0 + nvalid - 1;                        // ... and the last row that counts
    if (pos0 < 0 || slot_new >= cap || T > cap) {
        if (tid == 0) atomicOr(&a.ctl->status, STATUS_KV_FULL);
        return;
    }
    const int per = ((T + nsplit - 1) / nsplit + kPageTokens - 1) / kPageTokens * kPageTokens;
    const int tb = split * per, te = min(T, tb + per);
    const int ntiles = te <= tb ? 0 : (te - tb + kPageTokens - 1) / kPageTokens;
    const bool pages_ok = a.pages_per_seq <= 64;
    auto issue = [&](int i, bool staged) {               // thread 0: page i of the slice into stage i % kMmaStages
        const int t00 = tb + i * kPageTokens;
        const int page = staged ? pages[t00 / kPageTokens] : pt[t00 / kPageTokens];
        const int row = (page * 2 * a.kv_heads + kvh) * kPageTokens;          // first row of the K block in the layer's pool
        unsigned char* dst = dyn + (i % kMmaStages) * kMmaStageBytes;
        uint64_t* bar = &full[i % kMmaStages];
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"((uint32_t)kMmaStageBytes) : "memory");
        asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                     ::"r"(smem_addr(dst)), "l"(&kvmap), "r"(smem_addr(bar)), "r"(0), "r"(row) : "memory");
        asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                     ::"r"(smem_addr(dst + kMmaStageBytes / 2)), "l"(&kvmap), "r"(smem_addr(bar)), "r"(0), "r"(row + a.kv_heads * kPageTokens) : "memory");
    };
    if (tid == 0) {
        for (int j = 0; j < kMmaStages; ++j) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_addr(&full[j])));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        for (int i = 0; i < kMmaStages && i < ntiles; ++i) issue(i, false);
    }

    // Q: rotary embedding at each row's own position (extension), then bf16 hi / lo into the swizzled 16 x 64 tiles;
    // query columns beyond the CTA's rows are zero
    for (int i = tid; i < 16 * HD / 2; i += 128) {
        const int m = i / (HD / 2), pr = i % (HD / 2);
        const int j = m / HPK, hq = m % HPK;
        float q0 = 0.f, q1 = 0.f;
        if (j < nvalid) {
            const float* q = a.qkv + (size_t)(r0 + j) * a.ldq + (size_t)(kvh * HPK + hq) * HD;
            q0 = q[2 * pr]; q1 = q[2 * pr + 1];
            if (a.rope_base > 0.f) {
                float inv = powf(a.rope_base, -(float)(2 * pr) / (float)HD);
                float ang = __fmul_rn((float)(pos0 + j), inv);
                float sa, ca;
                sincosf(ang, &sa, &ca);
                float x0 = __fsub_rn(__fmul_rn(ca, q0), __fmul_rn(sa, q1));
                float x1 = __fadd_rn(__fmul_rn(sa, q0), __fmul_rn(ca, q1));
                q0 = x0; q1 = x1;
            }
        }
        uint32_t hi, lo;
        split_pair(q0, q1, hi, lo);
        const uint32_t off = swz128(m, pr >> 2) + (uint32_t)(pr & 3) * 4u;
        *reinterpret_cast<uint32_t*>(qtile + off) = hi;
        *reinterpret_cast<uint32_t*>(qtile + 16 * 128 + off) = lo;
    }
    // decode (phase 0): the new token's K / V row as the cache will hold it; slice 0 appends it (KvCache::append, model.rs:133-152)
    if (a.phase == 0) {
        const float* kn = a.qkv + (size_t)r0 * a.ldq + D + kvh * HD;
        const float* vn = kn + KV;
        for (int pr = tid; pr < HD / 2; pr += 128) {
            float k0 = kn[2 * pr], k1 = kn[2 * pr + 1];
            if (a.rope_base > 0.f) {
                float inv = powf(a.rope_base, -(float)(2 * pr) / (float)HD);
                float ang = __fmul_rn((float)pos0, inv);
                float sa, ca;
                sincosf(ang, &sa, &ca);
                float x0 = __fsub_rn(__fmul_rn(ca, k0), __fmul_rn(sa, k1));
                float x1 = __fadd_rn(__fmul_rn(sa, k0), __fmul_rn(ca, k1));
                k0 = x0; k1 = x1;
            }
            knew[2 * pr] = __float2bfloat16_rn(k0); knew[2 * pr + 1] = __float2bfloat16_rn(k1);
            vnew[2 * pr] = __float2bfloat16_rn(vn[2 * pr]); vnew[2 * pr + 1] = __float2bfloat16_rn(vn[2 * pr + 1]);
            if (split == 0) {
                __nv_bfloat16* pool = reinterpret_cast<__nv_bfloat16*>(a.pool);
                __nv_bfloat16* kd = kv_ptr(pool, pt, slot_new, 0, a.kv_heads, kvh, HD);
                __nv_bfloat16* vd = kv_ptr(pool, pt, slot_new, 1, a.kv_heads, kvh, HD);
                kd[2 * pr] = knew[2 * pr]; kd[2 * pr + 1] = knew[2 * pr + 1];
                vd[2 * pr] = vnew[2 * pr]; vd[2 * pr + 1] = vnew[2 * pr + 1];
            }
        }
    }
    const int local_slot = a.phase == 0 ? slot_new : -1; // attend only (phase 2): every row is already in the cache
    if (pages_ok) for (int i = tid; i < a.pages_per_seq; i += 128) pages[i] = pt[i];
    __syncthreads();

    // A fragments of Q for the four 16-dim steps: matrices (rows 0-7 | 8-15) x (dims +0..7 | +8..15)
    uint32_t qh[4][4], ql[4][4];
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
        const uint32_t off = swz128(lane & 15, 2 * ks + (lane >> 4));
        ldsm4(qh[ks], smem_addr(qtile) + off);
        ldsm4(ql[ks], smem_addr(qtile + 16 * 128) + off);
    }
    // per-row limits of the two query columns this thread sees in the accumulators (g and g + 8): 0 for unused columns
    const int lim0 = (g / HPK) < nvalid ? T0 + g / HPK : 0;
    const int lim1 = ((g + 8) / HPK) < nvalid ? T0 + (g + 8) / HPK : 0;
    const float scale = 0.125f;                          // 1 / sqrt(64), model.rs:530

    float m0 = kMaskedScore, m1 = kMaskedScore, l0 = 0.f, l1 = 0.f;    // running maximum and this thread's share of the sum, rows g and g + 8
    float o[8][4];                                       // context: 8 tiles of 8 dims; [0..1] row g, [2..3] row g + 8
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) { o[nt][0] = 0.f; o[nt][1] = 0.f; o[nt][2] = 0.f; o[nt][3] = 0.f; }
    bool dead = false;
    int dead_it = 0;
    for (int it = 0; it < ntiles; ++it) {
        const int t00 = tb + it * kPageTokens;
        const int tn = min(kPageTokens, te - t00);
        unsigned char* kst = dyn + (it % kMmaStages) * kMmaStageBytes;
        unsigned char* vst = kst + kMmaStageBytes / 2;
        const bool ok = page_wait(&full[it % kMmaStages], (uint32_t)(it / kMmaStages) & 1u);
        if (ok) {
            if (local_slot >= t00 && local_slot < t00 + tn && tid < 16) {
                // the new token's row from this CTA's own copy (slice 0 is still storing it)
                const int row = local_slot - t00, c = tid & 7;
                *reinterpret_cast<uint4*>((tid < 8 ? kst : vst) + swz128(row, c)) = reinterpret_cast<const uint4*>(tid < 8 ? knew : vnew)[c];
            }
            // rows of the page that hold no token yet: their weights are zero, and zero times whatever the memory holds must stay zero
            for (int i = tid; i < (kPageTokens - tn) * 8; i += 128)
                *reinterpret_cast<uint4*>(vst + (tn + i / 8) * 128 + (i & 7) * 16) = make_uint4(0u, 0u, 0u, 0u);
        }
        if (__syncthreads_or(!ok)) { dead = true; dead_it = it; break; }
        const int tw = 16 * warp;                        // this warp's 16 tokens of the page
        if (tw < tn) {
            float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};     // tokens tw .. tw + 7 and tw + 8 .. tw + 15
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
                uint32_t kb[4];
                const int tok = tw + ((lane >> 4) << 3) + (lane & 7);
                ldsm4(kb, smem_addr(kst) + swz128(tok, 2 * ks + ((lane >> 3) & 1)));
                mma16816(s0, qh[ks], kb[0], kb[1]);
                mma16816(s1, qh[ks], kb[2], kb[3]);
                mma16816(s0, ql[ks], kb[0], kb[1]);
                mma16816(s1, ql[ks], kb[2], kb[3]);
            }
            // scale (model.rs:532), mask, running maximum per query column (a quad holds one row of a tile)
            const int tc = t00 + tw + 2 * tq;            // token of element [0] of the first tile
            s0[0] = tc < lim0 ? __fmul_rn(s0[0], scale) : kMaskedScore;
            s0[1] = tc + 1 < lim0 ? __fmul_rn(s0[1], scale) : kMaskedScore;
            s0[2] = tc < lim1 ? __fmul_rn(s0[2], scale) : kMaskedScore;
            s0[3] = tc + 1 < lim1 ? __fmul_rn(s0[3], scale) : kMaskedScore;
            s1[0] = tc + 8 < lim0 ? __fmul_rn(s1[0], scale) : kMaskedScore;
            s1[1] = tc + 9 < lim0 ? __fmul_rn(s1[1], scale) : kMaskedScore;
            s1[2] = tc + 8 < lim1 ? __fmul_rn(s1[2], scale) : kMaskedScore;
            s1[3] = tc + 9 < lim1 ? __fmul_rn(s1[3], scale) : kMaskedScore;
            float x0 = fmaxf(fmaxf(s0[0], s0[1]), fmaxf(s1[0], s1[1]));
            float x1 = fmaxf(fmaxf(s0[2], s0[3]), fmaxf(s1[2], s1[3]));
            x0 = fmaxf(x0, __shfl_xor_sync(0xffffffffu, x0, 1)); x0 = fmaxf(x0, __shfl_xor_sync(0xffffffffu, x0, 2));
            x1 = fmaxf(x1, __shfl_xor_sync(0xffffffffu, x1, 1)); x1 = fmaxf(x1, __shfl_xor_sync(0xffffffffu, x1, 2));
            const float n0 = fmaxf(m0, x0), n1 = fmaxf(m1, x1);
            const float f0 = expf(__fsub_rn(m0, n0)), f1 = expf(__fsub_rn(m1, n1));
            m0 = n0; m1 = n1;
            float p0[4], p1[4];
            p0[0] = tc < lim0 ? expf(__fsub_rn(s0[0], n0)) : 0.f;
            p0[1] = tc + 1 < lim0 ? expf(__fsub_rn(s0[1], n0)) : 0.f;
            p0[2] = tc < lim1 ? expf(__fsub_rn(s0[2], n1)) : 0.f;
            p0[3] = tc + 1 < lim1 ? expf(__fsub_rn(s0[3], n1)) : 0.f;
            p1[0] = tc + 8 < lim0 ? expf(__fsub_rn(s1[0], n0)) : 0.f;
            p1[1] = tc + 9 < lim0 ? expf(__fsub_rn(s1[1], n0)) : 0.f;
            p1[2] = tc + 8 < lim1 ? expf(__fsub_rn(s1[2], n1)) : 0.f;
            p1[3] = tc + 9 < lim1 ? expf(__fsub_rn(s1[3], n1)) : 0.f;
            l0 = fmaf(l0, f0, (p0[0] + p0[1]) + (p1[0] + p1[1]));
            l1 = fmaf(l1, f1, (p0[2] + p0[3]) + (p1[2] + p1[3]));
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) { o[nt][0] *= f0; o[nt][1] *= f0; o[nt][2] *= f1; o[nt][3] *= f1; }
            // the weights as the A operand of P V: (row g | g + 8) x (tokens 2tq.. | 8 + 2tq..)
            uint32_t ph[4], pl[4];
            split_pair(p0[0], p0[1], ph[0], pl[0]);
            split_pair(p0[2], p0[3], ph[1], pl[1]);
            split_pair(p1[0], p1[1], ph[2], pl[2]);
            split_pair(p1[2], p1[3], ph[3], pl[3]);
#pragma unroll
            for (int dn = 0; dn < 4; ++dn) {             // 16 dims per step: tiles 2 dn and 2 dn + 1
                uint32_t vb[4];
                const int tok = tw + (((lane >> 3) & 1) << 3) + (lane & 7);
                ldsm4t(vb, smem_addr(vst) + swz128(tok, 2 * dn + (lane >> 4)));
                mma16816(o[2 * dn], ph, vb[0], vb[1]);
                mma16816(o[2 * dn + 1], ph, vb[2], vb[3]);
                mma16816(o[2 * dn], pl, vb[0], vb[1]);
                mma16816(o[2 * dn + 1], pl, vb[2], vb[3]);
            }
        }
        __syncthreads();                                 // this stage is free again
        if (tid == 0 && it + kMmaStages < ntiles) {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // the CTA's accesses to the stage come before the copy's writes
            issue(it + kMmaStages, pages_ok);
        }
    }
    if (dead && tid == 0) {
        // report, and let the copies still on their way land (again with a limit) before the shared memory goes away; the CTA
        // then finishes as usual, so that the slice counters stay consistent
        atomicOr(&a.ctl->status, STATUS_TIMEOUT);
        for (int j = dead_it; j < ntiles && j < dead_it + kMmaStages; ++j) page_wait(&full[j % kMmaStages], (uint32_t)(j / kMmaStages) & 1u);
    }
    if (dead) __syncthreads();

    // merge the four warps (the stages are free: every requested page has landed and been used)
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    constexpr int CW = HD + 2;                           // per query column: maximum, sum, context
    float* comb = reinterpret_cast<float*>(dyn);         // [4 warps][16][CW]
    {
        float* mine = comb + (size_t)warp * 16 * CW;
        if (tq == 0) { mine[g * CW] = m0; mine[g * CW + 1] = l0; mine[(g + 8) * CW] = m1; mine[(g + 8) * CW + 1] = l1; }
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
            mine[g * CW + 2 + nt * 8 + 2 * tq] = o[nt][0]; mine[g * CW + 2 + nt * 8 + 2 * tq + 1] = o[nt][1];
            mine[(g + 8) * CW + 2 + nt * 8 + 2 * tq] = o[nt][2]; mine[(g + 8) * CW + 2 + nt * 8 + 2 * tq + 1] = o[nt][3];
        }
    }
    __syncthreads();
    auto emit = [&](int m, int d, float v) {
        const size_t oo = (size_t)(r0 + m / HPK) * D + (size_t)(kvh * HPK + m % HPK) * HD + d;
        if (a.ctx32) a.ctx32[oo] = v;
        if (a.chi) {
            __nv_bfloat16 hh, ll;
            split_bf16(v, hh, ll);
            a.chi[oo] = hh;
            if (a.clo) a.clo[oo] = ll;
        }
    };
    constexpr int PW = HPK * (HD + 2);                   // floats per slice in `part`: [HPK] maxima, [HPK] sums, [HPK][HD] context
    float* mine = nsplit > 1 ? a.part + ((size_t)(grp * a.kv_heads + kvh) * kAttnMaxSplits + split) * PW : nullptr;
    for (int i = tid; i < nvalid * HPK * HD; i += 128) {
        const int m = i / HD, d = i % HD;
        float mx = comb[m * CW];
#pragma unroll
        for (int w = 1; w < 4; ++w) mx = fmaxf(mx, comb[(w * 16 + m) * CW]);
        float den = 0.f, num = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float f = expf(__fsub_rn(comb[(w * 16 + m) * CW], mx));
            den = fmaf(f, comb[(w * 16 + m) * CW + 1], den);
            num = fmaf(f, comb[(w * 16 + m) * CW + 2 + d], num);
        }
        if (nsplit == 1) emit(m, d, __fdiv_rn(num, den));
        else {
            mine[2 * HPK + i] = num;                     // one row per CTA here: m is the head
            if (d == 0) { mine[m] = mx; mine[HPK + m] = den; }
        }
    }
    if (nsplit == 1) return;
    // several slices: the last arriver merges them in slice order (nobody waits for anybody)
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const int old = atomicAdd(a.part_count + grp * a.kv_heads + kvh, 1);
        is_last = old == nsplit - 1;
        if (is_last) a.part_count[grp * a.kv_heads + kvh] = 0;           // ready for the next launch
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    const float* all = a.part + (size_t)(grp * a.kv_heads + kvh) * kAttnMaxSplits * PW;
    for (int i = tid; i < HPK * HD; i += 128) {
        const int hq = i / HD;
        float m = kMaskedScore;
        for (int sp = 0; sp < nsplit; ++sp) m = fmaxf(m, __ldcg(all + (size_t)sp * PW + hq));
        float den = 0.f, num = 0.f;
        for (int sp = 0; sp < nsplit; ++sp) {
            const float f = expf(__fsub_rn(__ldcg(all + (size_t)sp * PW + hq), m));
            den = fmaf(f, __ldcg(all + (size_t)sp * PW + HPK + hq), den);
            num = fmaf(f, __ldcg(all + (size_t)sp * PW + 2 * HPK + i), num);
        }
        emit(hq, i % HD, __fdiv_rn(num, den));
    }
}


static int attn_sm_count() {
    static int n = 0;
    if (n == 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    }
    return n;
}

// number of context slices: enough CTAs to give every SM two, at least kAttnSliceMin tokens each, and only where the caller
// gave room for the partial results (decode); the batched prefill has rows to spare
static int pick_slices(const AttnArgs& a) {
    if (a.part == nullptr || a.part_count == nullptr || a.phase != 0) return 1;
    // two CTAs per SM; splitting further was measured slower at 128 sequences x 4 KV heads (3.56 against 3.39 ms per
    // decode step of the hybrid model: the partial results and their merge cost more than the extra overlap brings)
    const long units = (long)a.B * a.kv_heads;
    int nsplit = (int)((2L * attn_sm_count() + units - 1) / units);
    const int by_len = (a.max_ctx_hint + kAttnSliceMin - 1) / kAttnSliceMin;
    if (nsplit > by_len) nsplit = by_len;
    if (nsplit > kAttnMaxSplits) nsplit = kAttnMaxSplits;
    return nsplit < 1 ? 1 : nsplit;
}

template <typename KT, int HD, int HPK>
cudaError_t launch_t(const AttnArgs& a, cudaStream_t st) {
    const int nsplit = pick_slices(a);
    dim3 grid(a.B, a.kv_heads, nsplit);
    // stages of one page (K block + V block of this KV head): three of 16 KiB leave room for four CTAs per SM
    constexpr int STAGE_BYTES = 2 * kPageTokens * HD * (int)sizeof(KT);
    constexpr int NST = STAGE_BYTES <= 16384 ? 3 : 2;
    static bool attr_set = false;                        // per instantiation
    if (!attr_set) {
        const cudaError_t e = cudaFuncSetAttribute(attn_decode_kernel<KT, HD, HPK, NST>, cudaFuncAttributeMaxDynamicSharedMemorySize, NST * STAGE_BYTES);
        if (e != cudaSuccess) return e;
        attr_set = true;
    }
    attn_decode_kernel<KT, HD, HPK, NST><<<grid, 128, NST * STAGE_BYTES, st>>>(a, reinterpret_cast<KT*>(a.pool));
    return cudaGetLastError();
}

template <int HPK>
cudaError_t launch_mma(const AttnArgs& a, cudaStream_t st) {
    CUtensorMap map;
    if (make_bf16_map_rows64(&map, a.pool, a.pool_bytes / 128, kPageTokens) != LUMI_OK) return cudaErrorUnknown;
    const int ts = a.rows_per_seq;
    const int q_rows = a.phase == 2 ? 16 / HPK : 1;
    const int gps = (ts + q_rows - 1) / q_rows;
    constexpr int kDyn = kMmaStages * kMmaStageBytes + 2 * 16 * 128 + 1024;
    static bool attr_set = false;
    if (!attr_set) {
        const cudaError_t e = cudaFuncSetAttribute(attn_mma_kernel<HPK>, cudaFuncAttributeMaxDynamicSharedMemorySize, kDyn);
        if (e != cudaSuccess) return e;
        attr_set = true;
    }
    dim3 grid((a.B / ts) * gps, a.kv_heads, pick_slices(a));
    attn_mma_kernel<HPK><<<grid, 128, kDyn, st>>>(a, map, q_rows, gps);
    return cudaGetLastError();
}

template <typename KT>
cudaError_t launch_kt(const AttnArgs& a, cudaStream_t st) {
    const int hpk = a.n_heads / a.kv_heads;
    if (a.phase == 1) {
        const long total = (long)a.B * a.kv_heads * (a.head_dim / 2);
        kv_append_kernel<KT><<<(unsigned)((total + 255) / 256), 256, 0, st>>>(a, reinterpret_cast<KT*>(a.pool), total);
        return cudaGetLastError();
    }
    if constexpr (sizeof(KT) == 2) {
        // bf16 cache with 64-wide heads: the tensor-core kernel (attend; the append-only pass of a prompt slice stays below)
        if (a.head_dim == 64 && a.phase != 1 && a.pool_bytes > 0 && a.pool_bytes / 128 < (size_t)1 << 31 && (a.B % a.rows_per_seq) == 0 &&
            (a.phase == 0 ? (a.rows_per_seq == 1) : (a.window == 0))) {
            if (hpk == 1) return launch_mma<1>(a, st);
            if (hpk == 2) return launch_mma<2>(a, st);
            if (hpk == 4) return launch_mma<4>(a, st);
            if (hpk == 8) return launch_mma<8>(a, st);
        }
    }
#define LUMI_ATT(HD_, HPK_) if (a.head_dim == HD_ && hpk == HPK_) return launch_t<KT, HD_, HPK_>(a, st);
    LUMI_ATT(64, 4) LUMI_ATT(64, 1) LUMI_ATT(64, 2) LUMI_ATT(64, 8)
    LUMI_ATT(32, 1) LUMI_ATT(32, 2) LUMI_ATT(32, 4) LUMI_ATT(32, 8)
    LUMI_ATT(128, 1) LUMI_ATT(128, 2) LUMI_ATT(128, 4) LUMI_ATT(128, 8)
#undef LUMI_ATT
    return cudaErrorInvalidValue;
}

__global__ void kv_advance_kernel(int32_t* kv_pos, int b0, int nb, int by, const int32_t* lens, int t_abs0) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= nb) return;
    // prompts of different lengths: a sequence advances by the tokens of the slice that belong to its prompt
    kv_pos[b0 + i] += lens != nullptr ? max(0, min(by, lens[b0 + i] - t_abs0)) : by;
}

}  // namespace

cudaError_t launch_kv_advance(int32_t* kv_pos, int b0, int nb, int by, cudaStream_t st, const int32_t* lens, int t_abs0) {
    kv_advance_kernel<<<(nb + 127) / 128, 128, 0, st>>>(kv_pos, b0, nb, by, lens, t_abs0);
    return cudaGetLastError();
}

// The cache element type follows the weights: fp32 weights keep an fp32 cache (so fp32 parity is
// not limited by cache rounding), bf16 weights a bf16 cache.  `pool` carries the type by flag.
cudaError_t launch_attention_decode(const AttnArgs& a, cudaStream_t st) {
    if (a.kv_is_f32) return launch_kt<float>(a, st);
    return launch_kt<__nv_bfloat16>(a, st);
}

}  // namespace lumi
