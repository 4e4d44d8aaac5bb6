// lumi_mamba_block_static: one Mamba block for callers that must not allocate.
//
// Everything else in this library gets its scratch from a session, and creating a session calls
// cudaMalloc.  Some hosts cannot do that at the point where they need a block evaluated: a serving
// process whose own pool already owns the whole device (a further cudaMalloc simply fails), code
// running between cudaStreamBeginCapture and EndCapture, or a latency-critical loop that may not
// take the device-wide synchronisation an allocation implies.  For them the two intermediate
// arrays of the block — in_proj's output and the gated state-step output — live in a fixed array
// in the library's own device image.  The price: a hard upper size, and one array shared by every
// call on a device.
#include "internal.h"

#include <mutex>

namespace lumi {
namespace {

constexpr int kStaticMaxBatch = 8;
constexpr int kStaticMaxPerSeq = 16384;      // floats per sequence: in_proj_out + d_inner must fit
constexpr int kStaticMaxDevices = 64;

// Scratch of the block: [batch][in_proj_out] followed by [batch][d_inner].  512 KiB, present on every
// GPU that loads this library, until the process exits.
static __device__ __align__(256) float g_block_scratch[kStaticMaxBatch * kStaticMaxPerSeq];

// In host code `g_block_scratch` is only a handle for the runtime, not an address a kernel may use:
// the device address is asked for once per device and kept here.
float* g_scratch_addr[kStaticMaxDevices] = {nullptr};
std::mutex g_scratch_mutex;

int32_t scratch_for_device(int device, float** out) {
    if (device < 0 || device >= kStaticMaxDevices) return fail(LUMI_E_INVALID, "device %d outside the table of %d devices", device, kStaticMaxDevices);
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    if (g_scratch_addr[device] == nullptr) {
        int current = -1;
        LUMI_CUDA(cudaGetDevice(&current));
        if (current != device) return fail(LUMI_E_INVALID, "device %d must be current for the first call (current is %d)", device, current);
        float* p = nullptr;
        LUMI_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_block_scratch));
        if (p == nullptr) return fail(LUMI_E_CUDA, "cudaGetSymbolAddress returned a null address for the block scratch");
        g_scratch_addr[device] = p;
    }
    *out = g_scratch_addr[device];
    return LUMI_OK;
}

}  // namespace
}  // namespace lumi

using namespace lumi;

extern "C" int32_t lumi_mamba_block_static(lumi_model* m, int32_t layer, uint64_t x, uint64_t h, uint64_t x_prev, uint64_t b_prev,
                                           uint64_t cum_angle, int32_t batch, uint64_t stream) {
    if (!m || !x || !h || !x_prev || !b_prev || !cum_angle) return fail(LUMI_E_INVALID, "null argument to lumi_mamba_block_static");
    if (!m->finalized) return fail(LUMI_E_INVALID, "lumi_model_finalize must succeed first");
    const Config& c = m->cfg;
    if (layer < 0 || layer >= c.n_layers || m->layers[layer].is_attn) return fail(LUMI_E_INVALID, "layer %d is not a Mamba layer", layer);
    const int R = c.in_proj_out(), DI = c.d_inner(), D = c.d_model;
    if (batch < 1 || batch > kStaticMaxBatch)
        return fail(LUMI_E_UNSUPPORTED, "lumi_mamba_block_static: batch %d outside [1, %d] (fixed scratch; use a session for larger batches)", batch, kStaticMaxBatch);
    if (R + DI > kStaticMaxPerSeq)
        return fail(LUMI_E_UNSUPPORTED, "lumi_mamba_block_static: in_proj_out + d_inner = %d floats per sequence exceeds the fixed scratch of %d", R + DI, kStaticMaxPerSeq);
    if (!ssm_shape_supported(c.head_dim(), c.d_state)) return fail(LUMI_E_UNSUPPORTED, "head_dim %d / d_state %d not built", c.head_dim(), c.d_state);
    LUMI_CUDA(cudaSetDevice(m->device));                    // stays current after the call (documented in the header)
    float* scratch = nullptr;
    LUMI_TRY(scratch_for_device(m->device, &scratch));      // first call per device: cudaGetSymbolAddress
    float* proj = scratch;                                   // [batch][R]
    float* y = scratch + (size_t)kStaticMaxBatch * R;        // [batch][DI]; R + DI <= kStaticMaxPerSeq keeps it inside
    const Layer& L = m->layers[layer];
    cudaStream_t st = (cudaStream_t)stream;
    float* xd = reinterpret_cast<float*>(x);
    // Nothing in the scratch has to start at zero: in_proj writes every element of proj[0..batch) and the
    // state step every element of y[0..batch) before anything reads them.
    // The two projections run on the multi-wave GEMV, which waits on nothing on the device: this call enqueues and
    // returns without synchronising, so it could not report a device-side wait that gave up — it launches no kernel
    // that has one.
    GemvArgs g1{xd, D, L.m.in_proj.p, L.m.in_proj.dtype, proj, R, nullptr, L.m.norm_g, batch, R, D, c.eps, 0};
    g1.allow_preload = false;
    LUMI_CUDA(launch_gemv(g1, st));
    SsmArgs a{};
    a.proj = proj; a.ldp = R;
    a.bg = L.m.b_gamma; a.cg = L.m.c_gamma; a.bb = L.m.b_bias; a.cb = L.m.c_bias; a.dskip = L.m.d_skip; a.dtb = L.m.dt_bias;
    a.h = reinterpret_cast<float*>(h); a.xprev = reinterpret_cast<float*>(x_prev);
    a.bprev = reinterpret_cast<float*>(b_prev); a.cum = reinterpret_cast<float*>(cum_angle);
    a.y32 = y;
    a.B = batch; a.H = c.n_heads; a.P = c.head_dim(); a.N = c.d_state; a.G = c.n_groups; a.eps = c.eps;
    LUMI_CUDA(launch_ssm_step(a, st));
    GemvArgs g2{y, DI, L.m.out_proj.p, L.m.out_proj.dtype, xd, D, xd, nullptr, batch, D, DI, c.eps, 0};
    g2.allow_preload = false;
    LUMI_CUDA(launch_gemv(g2, st));
    return LUMI_OK;
}
