// C ABI of liblumi_b200.so: config / weight loading, sessions, the decode step and the generate
// loop.  Replaces load_model + NmModel::{load, init_states, forward_step} and the token loop of
// the reference (inference/src/main.rs:72-89, 118-170; inference/src/model.rs:643-801).
#include "internal.h"
#include "json_min.h"

#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <algorithm>

using namespace lumi;

// ---- errors -----------------------------------------------------------------------------------------
namespace lumi {
static thread_local char g_err[1024] = "";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}
int32_t fail(int32_t code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

bool Config::is_attention_layer(int i) const {          // model.rs:66-71
    if (!attention_layers.empty())
        return std::find(attention_layers.begin(), attention_layers.end(), i) != attention_layers.end();
    return attention_interval > 0 && (i + 1) % attention_interval == 0;
}
int Config::n_attn_layers() const {
    int n = 0;
    for (int i = 0; i < n_layers; ++i) n += is_attention_layer(i) ? 1 : 0;
    return n;
}

static bool get_int(const JsonValue& root, const char* key, bool required, int& out, std::string& err) {
    const JsonValue* v = root.find(key);
    if (!v) {
        if (required) { err = std::string("config.json: missing key '") + key + "'"; return false; }
        return true;
    }
    if (v->kind != JsonValue::Number || v->num < 0 || v->num != (double)(long long)v->num) {
        err = std::string("config.json: key '") + key + "' must be a non-negative integer";
        return false;
    }
    out = (int)v->num;
    return true;
}
static bool get_int_list(const JsonValue& root, const char* key, std::vector<int>& out, std::string& err) {
    const JsonValue* v = root.find(key);
    if (!v) return true;
    if (v->kind != JsonValue::Array) { err = std::string("config.json: key '") + key + "' must be an array"; return false; }
    for (auto& e : v->arr) {
        if (e.kind != JsonValue::Number || e.num < 0) { err = std::string("config.json: '") + key + "' holds a non-integer"; return false; }
        out.push_back((int)e.num);
    }
    return true;
}

int32_t parse_config(const char* json, Config& c) {
    if (!json) return fail(LUMI_E_INVALID, "config text is null");
    JsonValue root;
    std::string err;
    JsonParser p(json, strlen(json));
    if (!p.parse(root, err) || root.kind != JsonValue::Object) return fail(LUMI_E_CONFIG, "config.json: %s", err.empty() ? "not a JSON object" : err.c_str());
    bool ok = get_int(root, "d_model", true, c.d_model, err) && get_int(root, "n_layers", true, c.n_layers, err) &&
              get_int(root, "d_state", true, c.d_state, err) && get_int(root, "expand", true, c.expand, err) &&
              get_int(root, "n_heads", true, c.n_heads, err) && get_int(root, "n_groups", true, c.n_groups, err) &&
              get_int(root, "vocab_size", true, c.vocab, err) && get_int(root, "max_seq_len", true, c.max_seq_len, err) &&
              get_int(root, "attention_interval", false, c.attention_interval, err) &&
              get_int(root, "attn_n_heads", false, c.attn_n_heads, err) && get_int(root, "attn_kv_heads", false, c.attn_kv_heads, err) &&
              get_int(root, "attn_mlp_expand", false, c.attn_mlp_expand, err) && get_int(root, "attn_mlp_dim", false, c.attn_mlp_dim, err) &&
              get_int_list(root, "attn_window_sizes", c.attn_window_sizes, err) &&
              get_int_list(root, "attention_layers", c.attention_layers, err);
    if (!ok) return fail(LUMI_E_CONFIG, "%s", err.c_str());
    if (const JsonValue* v = root.find("byte_level")) {
        if (v->kind != JsonValue::Bool) return fail(LUMI_E_CONFIG, "config.json: key 'byte_level' must be a boolean");
        c.byte_level = v->b;
    }
    if (const JsonValue* v = root.find("attn_rope_base")) {
        if (v->kind != JsonValue::Number || v->num < 0) return fail(LUMI_E_CONFIG, "config.json: key 'attn_rope_base' must be a number >= 0");
        c.attn_rope_base = (float)v->num;
    }
    if (c.byte_level) c.vocab = 259;                                    // main.rs:75-77
    // the reference's divisibility invariants (training/tests/training_init_tests.rs:70-112) plus vector widths
    if (c.d_model <= 0 || c.n_layers <= 0 || c.d_state <= 0 || c.expand <= 0 || c.n_heads <= 0 || c.n_groups <= 0 || c.vocab <= 0)
        return fail(LUMI_E_CONFIG, "config.json: dimensions must be positive");
    if (c.d_inner() % c.n_heads) return fail(LUMI_E_CONFIG, "config.json: expand*d_model (%d) not divisible by n_heads (%d)", c.d_inner(), c.n_heads);
    if (c.n_heads % c.n_groups) return fail(LUMI_E_CONFIG, "config.json: n_heads (%d) not divisible by n_groups (%d)", c.n_heads, c.n_groups);
    if (c.d_state % 2) return fail(LUMI_E_CONFIG, "config.json: d_state (%d) must be even", c.d_state);
    if (c.d_model % 8) return fail(LUMI_E_CONFIG, "config.json: d_model (%d) must be a multiple of 8", c.d_model);
    if (c.n_attn_layers() > 0) {
        if (c.attn_n_heads <= 0 || c.attn_kv_heads <= 0 || c.d_model % c.attn_n_heads || c.attn_n_heads % c.attn_kv_heads)
            return fail(LUMI_E_CONFIG, "config.json: attention heads (%d query / %d kv) do not divide d_model", c.attn_n_heads, c.attn_kv_heads);
        if (c.mlp_dim() % 8) return fail(LUMI_E_CONFIG, "config.json: attention MLP width (%d) must be a multiple of 8", c.mlp_dim());
        for (int l : c.attention_layers) if (l >= c.n_layers) return fail(LUMI_E_CONFIG, "config.json: attention_layers entry %d >= n_layers", l);
    }
    return LUMI_OK;
}
}  // namespace lumi

extern "C" const char* lumi_last_error(void) { return lumi::g_err; }

// ---- model ------------------------------------------------------------------------------------------
static float bf16_to_f32(uint16_t b) {
    uint32_t u = (uint32_t)b << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

extern "C" int32_t lumi_model_create(const char* config_json, int32_t device_id, lumi_model** out) {
    if (!out) return fail(LUMI_E_INVALID, "out pointer is null");
    *out = nullptr;
    Config c;
    LUMI_TRY(parse_config(config_json, c));
    int ndev = 0;
    LUMI_CUDA(cudaGetDeviceCount(&ndev));
    if (device_id < 0 || device_id >= ndev) return fail(LUMI_E_INVALID, "device %d not available (%d CUDA devices)", device_id, ndev);
    if (!ssm_shape_supported(c.head_dim(), c.d_state) && c.n_attn_layers() < c.n_layers)
        return fail(LUMI_E_UNSUPPORTED, "head_dim %d / d_state %d: kernels exist for head_dim in {16,32,64} and d_state in {16,32,64,128}", c.head_dim(), c.d_state);
    lumi_model* m = new lumi_model();
    m->cfg = c;
    m->device = device_id;
    *out = m;
    return LUMI_OK;
}

// Expected shape of a tensor by its name (without the "item." prefix); rank 0 = not a tensor of this model.
static int expected_shape(const lumi_model* m, const std::string& name, int64_t shp[2]) {
    const Config& c = m->cfg;
    if (name == "embedding.weight") { shp[0] = c.vocab; shp[1] = c.d_model; return 2; }
    if (name == "final_norm.gamma") { shp[0] = c.d_model; return 1; }
    if (name.rfind("blocks.", 0) != 0) return 0;
    size_t dot = name.find('.', 7);
    if (dot == std::string::npos) return 0;
    int layer = -1;
    try { layer = std::stoi(name.substr(7, dot - 7)); } catch (...) { return 0; }
    if (layer < 0 || layer >= c.n_layers) return 0;
    const std::string k = name.substr(dot + 1);
    const bool attn = c.is_attention_layer(layer);
    if (!attn) {
        if (k == "norm.gamma") { shp[0] = c.d_model; return 1; }
        if (k == "in_proj.weight") { shp[0] = c.in_proj_out(); shp[1] = c.d_model; return 2; }
        if (k == "out_proj.weight") { shp[0] = c.d_model; shp[1] = c.d_inner(); return 2; }
        if (k == "b_norm.gamma" || k == "c_norm.gamma" || k == "b_bias" || k == "c_bias") { shp[0] = c.bc(); return 1; }
        if (k == "ssm.d" || k == "ssm.dt_bias") { shp[0] = c.n_heads; return 1; }
        if (k == "ssm.h_init") { shp[0] = c.n_heads; shp[1] = c.d_state; return 2; }
        return 0;
    }
    if (k == "attn_norm.gamma" || k == "mlp_norm.gamma") { shp[0] = c.d_model; return 1; }
    if (k == "q_proj.weight" || k == "attn_out_proj.weight") { shp[0] = c.d_model; shp[1] = c.d_model; return 2; }
    if (k == "k_proj.weight" || k == "v_proj.weight") { shp[0] = c.kv_dim(); shp[1] = c.d_model; return 2; }
    if (k == "mlp_gate.weight" || k == "mlp_up.weight") { shp[0] = c.mlp_dim(); shp[1] = c.d_model; return 2; }
    if (k == "mlp_down.weight") { shp[0] = c.d_model; shp[1] = c.mlp_dim(); return 2; }
    return 0;
}

extern "C" int32_t lumi_model_load_tensor(lumi_model* m, const char* name, int32_t dtype, const int64_t* shape, int32_t rank,
                                          const void* host_data, uint64_t nbytes) {
    if (!m || !name || !host_data || (!shape && rank > 0)) return fail(LUMI_E_INVALID, "null argument to lumi_model_load_tensor");
    if (m->finalized) return fail(LUMI_E_INVALID, "model already finalized");
    if (dtype != LUMI_DTYPE_F32 && dtype != LUMI_DTYPE_BF16) return fail(LUMI_E_TENSOR, "tensor '%s': dtype code %d not supported (F32, BF16)", name, dtype);
    std::string n(name);
    if (n.rfind("item.", 0) != 0) return LUMI_OK;         // the reference only reads names under "item." (main.rs:86)
    n = n.substr(5);
    int64_t exp[2] = {0, 0};
    const int erank = expected_shape(m, n, exp);
    if (erank == 0) return LUMI_OK;                       // tensors the model never asks for are ignored, as VarBuilder does
    if (m->tensors.count(n)) return fail(LUMI_E_TENSOR, "tensor '%s' loaded twice", name);
    int64_t count = 1;
    for (int i = 0; i < rank; ++i) count *= shape[i];
    const bool is_hinit = n.size() > 10 && n.compare(n.size() - 10, 10, "ssm.h_init") == 0;
    bool shape_ok = (rank == erank);
    for (int i = 0; shape_ok && i < rank; ++i) shape_ok = (shape[i] == exp[i]);
    if (is_hinit && rank == 1 && shape[0] == exp[0] * exp[1]) shape_ok = true;   // the trainer writes it flat (native_checkpoint.rs:55)
    if (!shape_ok) {
        char got[128] = "", want[128] = "";
        for (int i = 0; i < rank && i < 4; ++i) snprintf(got + strlen(got), sizeof(got) - strlen(got), "%s%lld", i ? "," : "", (long long)shape[i]);
        for (int i = 0; i < erank; ++i) snprintf(want + strlen(want), sizeof(want) - strlen(want), "%s%lld", i ? "," : "", (long long)exp[i]);
        return fail(LUMI_E_TENSOR, "tensor '%s': shape [%s], expected [%s]", name, got, want);
    }
    const size_t esz = dtype == LUMI_DTYPE_BF16 ? 2 : 4;
    if ((uint64_t)count * esz != nbytes) return fail(LUMI_E_TENSOR, "tensor '%s': %llu bytes given, shape needs %llu", name, (unsigned long long)nbytes, (unsigned long long)(count * esz));
    LUMI_CUDA(cudaSetDevice(m->device));
    DevTensor t;
    const bool keep_width = (erank == 2) && !is_hinit;
    if (keep_width) {
        if (m->wdtype >= 0 && m->wdtype != dtype) return fail(LUMI_E_TENSOR, "tensor '%s': rank-2 tensors mix F32 and BF16", name);
        m->wdtype = dtype;
        t.dtype = dtype;
        t.rows = exp[0]; t.cols = exp[1];
        t.bytes = nbytes;
        LUMI_CUDA(cudaMalloc(&t.p, t.bytes));
        LUMI_CUDA(cudaMemcpy(t.p, host_data, t.bytes, cudaMemcpyHostToDevice));
    } else {
        std::vector<float> tmp;
        const float* src = (const float*)host_data;
        if (dtype == LUMI_DTYPE_BF16) {
            tmp.resize(count);
            const uint16_t* b = (const uint16_t*)host_data;
            for (int64_t i = 0; i < count; ++i) tmp[i] = bf16_to_f32(b[i]);
            src = tmp.data();
        }
        t.dtype = LUMI_DTYPE_F32;
        t.rows = 1; t.cols = count;
        t.bytes = (size_t)count * 4;
        LUMI_CUDA(cudaMalloc(&t.p, t.bytes));
        LUMI_CUDA(cudaMemcpy(t.p, src, t.bytes, cudaMemcpyHostToDevice));
    }
    m->tensors[n] = t;
    return LUMI_OK;
}

static int32_t need(lumi_model* m, const std::string& n, DevTensor& out) {
    auto it = m->tensors.find(n);
    if (it == m->tensors.end()) return fail(LUMI_E_TENSOR, "tensor 'item.%s' is missing", n.c_str());
    out = it->second;
    return LUMI_OK;
}
static int32_t need_f(lumi_model* m, const std::string& n, const float*& out) {
    DevTensor t;
    LUMI_TRY(need(m, n, t));
    out = (const float*)t.p;
    return LUMI_OK;
}
static int32_t ones_default(lumi_model* m, const std::string& n, int count, const float*& out) {   // model.rs:209-212
    auto it = m->tensors.find(n);
    if (it != m->tensors.end()) { out = (const float*)it->second.p; return LUMI_OK; }
    std::vector<float> ones(count, 1.0f);
    void* p = nullptr;
    LUMI_CUDA(cudaMalloc(&p, (size_t)count * 4));
    LUMI_CUDA(cudaMemcpy(p, ones.data(), (size_t)count * 4, cudaMemcpyHostToDevice));
    m->owned.push_back(p);
    out = (const float*)p;
    return LUMI_OK;
}
// rows of several [r_i][cols] matrices stacked into one allocation; the parts are released
static int32_t concat_rows(lumi_model* m, const std::vector<std::string>& names, DevTensor& out) {
    std::vector<DevTensor> parts(names.size());
    size_t total = 0;
    int64_t rows = 0;
    for (size_t i = 0; i < names.size(); ++i) { LUMI_TRY(need(m, names[i], parts[i])); total += parts[i].bytes; rows += parts[i].rows; }
    void* p = nullptr;
    LUMI_CUDA(cudaMalloc(&p, total));
    size_t off = 0;
    for (size_t i = 0; i < names.size(); ++i) {
        LUMI_CUDA(cudaMemcpy((char*)p + off, parts[i].p, parts[i].bytes, cudaMemcpyDeviceToDevice));
        off += parts[i].bytes;
        LUMI_CUDA(cudaFree(parts[i].p));
        m->tensors[names[i]].p = nullptr;
    }
    m->owned.push_back(p);
    out = parts[0];
    out.p = p; out.rows = rows; out.bytes = total;
    return LUMI_OK;
}

extern "C" int32_t lumi_model_finalize(lumi_model* m) {
    if (!m) return fail(LUMI_E_INVALID, "model is null");
    if (m->finalized) return LUMI_OK;
    LUMI_CUDA(cudaSetDevice(m->device));
    const Config& c = m->cfg;
    LUMI_TRY(need(m, "embedding.weight", m->embedding));
    LUMI_TRY(need_f(m, "final_norm.gamma", m->final_norm_g));
    m->weight_bytes = 0;
    for (auto& kv : m->tensors) m->weight_bytes += (int64_t)kv.second.bytes;
    m->layers.assign(c.n_layers, Layer());
    int im = 0, ia = 0;
    for (int i = 0; i < c.n_layers; ++i) {
        Layer& L = m->layers[i];
        const std::string p = "blocks." + std::to_string(i) + ".";
        L.is_attn = c.is_attention_layer(i);
        if (!L.is_attn) {
            L.kind_idx = im++;
            LUMI_TRY(need_f(m, p + "norm.gamma", L.m.norm_g));
            LUMI_TRY(need(m, p + "in_proj.weight", L.m.in_proj));
            LUMI_TRY(need(m, p + "out_proj.weight", L.m.out_proj));
            LUMI_TRY(need_f(m, p + "b_norm.gamma", L.m.b_gamma));
            LUMI_TRY(need_f(m, p + "c_norm.gamma", L.m.c_gamma));
            LUMI_TRY(ones_default(m, p + "b_bias", c.bc(), L.m.b_bias));
            LUMI_TRY(ones_default(m, p + "c_bias", c.bc(), L.m.c_bias));
            LUMI_TRY(need_f(m, p + "ssm.d", L.m.d_skip));
            LUMI_TRY(need_f(m, p + "ssm.dt_bias", L.m.dt_bias));
            auto it = m->tensors.find(p + "ssm.h_init");                 // optional: zeros (model.rs:214, 744-748)
            L.m.h_init = it == m->tensors.end() ? nullptr : (const float*)it->second.p;
        } else {
            L.kind_idx = ia;
            L.window = c.attn_window_size(ia);
            ++ia;
            LUMI_TRY(need_f(m, p + "attn_norm.gamma", L.a.attn_norm_g));
            LUMI_TRY(need_f(m, p + "mlp_norm.gamma", L.a.mlp_norm_g));
            LUMI_TRY(concat_rows(m, {p + "q_proj.weight", p + "k_proj.weight", p + "v_proj.weight"}, L.a.qkv));
            LUMI_TRY(need(m, p + "attn_out_proj.weight", L.a.o));
            LUMI_TRY(concat_rows(m, {p + "mlp_gate.weight", p + "mlp_up.weight"}, L.a.gate_up));
            LUMI_TRY(need(m, p + "mlp_down.weight", L.a.down));
        }
    }
    m->n_mamba = im;
    m->n_attn = ia;
    if (m->wdtype < 0) m->wdtype = LUMI_DTYPE_F32;
    m->finalized = true;
    return LUMI_OK;
}

extern "C" void lumi_model_free(lumi_model* m) {
    if (!m) return;
    cudaSetDevice(m->device);
    for (auto& kv : m->tensors) if (kv.second.p) cudaFree(kv.second.p);
    for (void* p : m->owned) cudaFree(p);
    delete m;
}

extern "C" int32_t lumi_model_info(const lumi_model* m, int64_t* o) {
    if (!m || !o) return fail(LUMI_E_INVALID, "null argument to lumi_model_info");
    const Config& c = m->cfg;
    o[0] = c.d_model; o[1] = c.n_layers; o[2] = c.d_state; o[3] = c.n_heads; o[4] = c.head_dim(); o[5] = c.n_groups;
    o[6] = c.vocab; o[7] = m->n_mamba; o[8] = m->n_attn; o[9] = c.in_proj_out(); o[10] = m->wdtype; o[11] = m->weight_bytes;
    return LUMI_OK;
}

// ---- sessions ---------------------------------------------------------------------------------------
static size_t state_h_per_seq(const Config& c) { return (size_t)c.n_heads * c.head_dim() * c.d_state; }

extern "C" void lumi_session_free(lumi_session* s) {
    if (!s) return;
    cudaSetDevice(s->m->device);
    if (s->stream) cudaStreamSynchronize(s->stream);
    for (auto& g : s->graphs) if (g.second.exec) cudaGraphExecDestroy(g.second.exec);
    void* dev[] = {s->score_logits, s->gemm_counters, s->gemm_scratch, s->h, s->xprev, s->bprev, s->cum, s->kv_pool, s->page_table, s->kv_pos, s->x, s->proj, s->y32, s->logits,
                   s->act_hi, s->act_lo, s->tok_cur, s->finished, s->out_len, s->ctl, s->gen_out, s->prompt_dev, s->gen_dump,
                   s->pf_x, s->pf_proj, s->pf_rb, s->pf_rc, s->pf_hi, s->pf_lo, s->slot_buf, s->xn_hi, s->xn_lo, s->ssq, s->attn_part, s->attn_part_count, s->amax_val, s->amax_idx, s->row_len, s->xlast,
                   s->b1_layers, s->b1_grid_ctl, s->b1_amax_val, s->b1_amax_idx, s->b1_timing, s->b1_tagged};
    for (void* p : dev) if (p) cudaFree(p);
    if (s->ctl_host) cudaFreeHost(s->ctl_host);
    if (s->pin_tokens) cudaFreeHost(s->pin_tokens);
    if (s->ev0) cudaEventDestroy(s->ev0);
    if (s->ev1) cudaEventDestroy(s->ev1);
    if (s->ev2) cudaEventDestroy(s->ev2);
    for (int i = 0; i < 2; ++i) {
        if (s->lane_hi[i]) cudaStreamDestroy(s->lane_hi[i]);
        if (s->lane_lo[i]) cudaStreamDestroy(s->lane_lo[i]);
        for (int j = 0; j < 2; ++j) if (s->lane_ev[i][j]) cudaEventDestroy(s->lane_ev[i][j]);
        if (s->ev_join[i]) cudaEventDestroy(s->ev_join[i]);
    }
    if (s->ev_fork) cudaEventDestroy(s->ev_fork);
    if (s->ev_stagger) cudaEventDestroy(s->ev_stagger);
    if (s->stream) cudaStreamDestroy(s->stream);
    delete s;
}

static int32_t session_alloc(lumi_session* s) {
    const Config& c = s->m->cfg;
    const size_t B = s->max_batch;
    const int nm = s->m->n_mamba, na = s->m->n_attn;
    LUMI_CUDA(cudaStreamCreateWithFlags(&s->stream, cudaStreamNonBlocking));
    LUMI_CUDA(cudaEventCreate(&s->ev0));
    LUMI_CUDA(cudaEventCreate(&s->ev1));
    LUMI_CUDA(cudaEventCreate(&s->ev2));
    {
        int lo_prio = 0, hi_prio = 0;                     // numerically lower = higher priority
        LUMI_CUDA(cudaDeviceGetStreamPriorityRange(&lo_prio, &hi_prio));
        for (int i = 0; i < 2; ++i) {
            LUMI_CUDA(cudaStreamCreateWithPriority(&s->lane_hi[i], cudaStreamNonBlocking, hi_prio));
            LUMI_CUDA(cudaStreamCreateWithPriority(&s->lane_lo[i], cudaStreamNonBlocking, lo_prio));
            for (int j = 0; j < 2; ++j) LUMI_CUDA(cudaEventCreateWithFlags(&s->lane_ev[i][j], cudaEventDisableTiming));
            LUMI_CUDA(cudaEventCreateWithFlags(&s->ev_join[i], cudaEventDisableTiming));
        }
        LUMI_CUDA(cudaEventCreateWithFlags(&s->ev_fork, cudaEventDisableTiming));
        LUMI_CUDA(cudaEventCreateWithFlags(&s->ev_stagger, cudaEventDisableTiming));
    }
    if (nm > 0) {
        LUMI_CUDA(cudaMalloc(&s->h, sizeof(float) * nm * B * state_h_per_seq(c)));
        LUMI_CUDA(cudaMalloc(&s->xprev, sizeof(float) * nm * B * c.d_inner()));
        LUMI_CUDA(cudaMalloc(&s->bprev, sizeof(float) * nm * B * c.n_heads * c.d_state));
        LUMI_CUDA(cudaMalloc(&s->cum, sizeof(float) * nm * B * c.n_heads * (c.d_state / 2)));
    }
    if (na > 0) {
        if (s->max_tokens_kv <= 0) return fail(LUMI_E_INVALID, "max_tokens_kv must be > 0 for a model with attention layers");
        s->pages_per_seq = (s->max_tokens_kv + kPageTokens - 1) / kPageTokens;
        const size_t esz = s->m->wdtype == LUMI_DTYPE_BF16 ? 2 : 4;
        s->kv_layer_bytes = B * s->pages_per_seq * 2 * kPageTokens * (size_t)c.kv_dim() * esz;
        LUMI_CUDA(cudaMalloc(&s->kv_pool, s->kv_layer_bytes * na));
        LUMI_CUDA(cudaMalloc(&s->page_table, sizeof(int32_t) * B * s->pages_per_seq));
        // partial results of an attention context split over several CTAs: used only while batch x KV heads is small
        // enough for a split to pay, so a fixed number of (row, KV head) units is enough
        {
            const size_t pw = (size_t)(c.attn_n_heads / std::max(1, c.attn_kv_heads)) * (c.attn_head_dim() + 2);
            LUMI_CUDA(cudaMalloc(&s->attn_part, sizeof(float) * kAttnPartUnits * kAttnPartSlices * pw));
            LUMI_CUDA(cudaMalloc(&s->attn_part_count, sizeof(int32_t) * kAttnPartUnits));
            LUMI_CUDA(cudaMemset(s->attn_part_count, 0, sizeof(int32_t) * kAttnPartUnits));
        }
        std::vector<int32_t> pt(B * s->pages_per_seq);
        for (size_t i = 0; i < pt.size(); ++i) pt[i] = (int32_t)i;       // slot b owns pages [b*pps, (b+1)*pps)
        LUMI_CUDA(cudaMemcpy(s->page_table, pt.data(), pt.size() * sizeof(int32_t), cudaMemcpyHostToDevice));
    }
    LUMI_CUDA(cudaMalloc(&s->kv_pos, sizeof(int32_t) * B));
    LUMI_CUDA(cudaMalloc(&s->slot_buf, sizeof(int32_t) * B));
    LUMI_CUDA(cudaMalloc(&s->row_len, sizeof(int32_t) * B));
    LUMI_CUDA(cudaMalloc(&s->xlast, sizeof(float) * B * c.d_model));
    LUMI_CUDA(cudaMalloc(&s->gemm_counters, sizeof(int32_t) * 2 * kGemmCounters));
    LUMI_CUDA(cudaMemset(s->gemm_counters, 0, sizeof(int32_t) * 2 * kGemmCounters));
    LUMI_CUDA(cudaMalloc(&s->gemm_scratch, sizeof(float) * 2 * kGemmScratchFloats));
    const size_t kmax = std::max<size_t>({(size_t)c.d_model, (size_t)c.d_inner(), na > 0 ? (size_t)c.mlp_dim() : 0});
    const size_t pmax = std::max<size_t>({nm > 0 ? (size_t)c.in_proj_out() : 0, na > 0 ? (size_t)(c.d_model + 2 * c.kv_dim()) : 0,
                                          na > 0 ? (size_t)(2 * c.mlp_dim()) : 0});
    LUMI_CUDA(cudaMalloc(&s->x, sizeof(float) * B * c.d_model));
    LUMI_CUDA(cudaMalloc(&s->proj, sizeof(float) * B * pmax));
    LUMI_CUDA(cudaMalloc(&s->y32, sizeof(float) * B * kmax));
    LUMI_CUDA(cudaMalloc(&s->logits, sizeof(float) * B * c.vocab));
    // per-CTA argmax partials of the greedy head at batch <= 8 (at most one CTA per vocabulary row)
    s->amax_stride = c.vocab;
    LUMI_CUDA(cudaMalloc(&s->amax_val, sizeof(float) * 8 * (size_t)c.vocab));
    LUMI_CUDA(cudaMalloc(&s->amax_idx, sizeof(int) * 8 * (size_t)c.vocab));
    if (s->m->wdtype == LUMI_DTYPE_BF16) {
        // rows padded to a whole 128-row tile so TMA boxes never start outside the allocation
        const size_t rows = (B + 127) / 128 * 128;
        s->act_ld = kmax;
        LUMI_CUDA(cudaMalloc(&s->act_hi, sizeof(__nv_bfloat16) * rows * kmax));
        LUMI_CUDA(cudaMalloc(&s->act_lo, sizeof(__nv_bfloat16) * rows * kmax));
        LUMI_CUDA(cudaMemset(s->act_hi, 0, sizeof(__nv_bfloat16) * rows * kmax));
        LUMI_CUDA(cudaMemset(s->act_lo, 0, sizeof(__nv_bfloat16) * rows * kmax));
        // the residual stream times the next norm's weights (bf16 halves) and its per-row partial sums of squares:
        // written by the epilogue of the product that updates the residual, read by the next product
        s->ssq_stride = (c.d_model + 31) / 32;
        LUMI_CUDA(cudaMalloc(&s->xn_hi, sizeof(__nv_bfloat16) * rows * c.d_model));
        LUMI_CUDA(cudaMalloc(&s->xn_lo, sizeof(__nv_bfloat16) * rows * c.d_model));
        LUMI_CUDA(cudaMemset(s->xn_hi, 0, sizeof(__nv_bfloat16) * rows * c.d_model));
        LUMI_CUDA(cudaMemset(s->xn_lo, 0, sizeof(__nv_bfloat16) * rows * c.d_model));
        LUMI_CUDA(cudaMalloc(&s->ssq, sizeof(float) * rows * s->ssq_stride));
        LUMI_CUDA(cudaMemset(s->ssq, 0, sizeof(float) * rows * s->ssq_stride));
    }
    LUMI_CUDA(cudaMalloc(&s->tok_cur, sizeof(uint32_t) * B));
    LUMI_CUDA(cudaMalloc(&s->finished, sizeof(int32_t) * B));
    LUMI_CUDA(cudaMalloc(&s->out_len, sizeof(int32_t) * B));
    LUMI_CUDA(cudaMalloc(&s->ctl, sizeof(StepCtl)));
    LUMI_CUDA(cudaMallocHost(&s->ctl_host, sizeof(StepCtl)));
    LUMI_CUDA(cudaMallocHost(&s->pin_tokens, sizeof(uint32_t) * B));
    memset(s->ctl_host, 0, sizeof(StepCtl));
    LUMI_CUDA(cudaMemset(s->tok_cur, 0, sizeof(uint32_t) * B));
    // batch-1 persistent kernel: per-layer pointer table, barrier words, argmax partials
    s->b1_ok = decode_b1_supported(c, na, s->m->device);
    if (s->b1_ok) {
        std::vector<B1Layer> tab;
        for (const Layer& L : s->m->layers) {
            const size_t l = L.kind_idx;
            B1Layer t{L.m.in_proj.p, L.m.out_proj.p, L.m.norm_g, L.m.b_gamma, L.m.c_gamma, L.m.b_bias, L.m.c_bias, L.m.d_skip, L.m.dt_bias,
                      s->h + l * B * state_h_per_seq(c), s->xprev + l * B * c.d_inner(), s->bprev + l * B * c.n_heads * c.d_state,
                      s->cum + l * B * c.n_heads * (c.d_state / 2)};
            tab.push_back(t);
        }
        LUMI_CUDA(cudaMalloc(&s->b1_layers, sizeof(B1Layer) * tab.size()));
        LUMI_CUDA(cudaMemcpy(s->b1_layers, tab.data(), sizeof(B1Layer) * tab.size(), cudaMemcpyHostToDevice));
        LUMI_CUDA(cudaMalloc(&s->b1_grid_ctl, 64));
        LUMI_CUDA(cudaMalloc(&s->b1_amax_val, sizeof(float) * 1024));
        LUMI_CUDA(cudaMalloc(&s->b1_amax_idx, sizeof(int) * 1024));
        const size_t ntag = (size_t)c.d_model + c.in_proj_out() + c.d_inner();
        LUMI_CUDA(cudaMalloc(&s->b1_tagged, ntag * 8));
        LUMI_CUDA(cudaMemset(s->b1_tagged, 0, ntag * 8));          // epoch 0 is never used
    }
    return LUMI_OK;
}

extern "C" int32_t lumi_session_create(lumi_model* m, int32_t max_batch, int32_t max_tokens_kv, lumi_session** out) {
    if (!m || !out) return fail(LUMI_E_INVALID, "null argument to lumi_session_create");
    *out = nullptr;
    if (!m->finalized) return fail(LUMI_E_INVALID, "lumi_model_finalize must succeed before a session is created");
    if (max_batch <= 0) return fail(LUMI_E_INVALID, "max_batch must be > 0");
    LUMI_CUDA(cudaSetDevice(m->device));
    lumi_session* s = new lumi_session();
    s->m = m;
    s->max_batch = max_batch;
    s->max_tokens_kv = max_tokens_kv;
    if (const char* e = getenv("LUMI_PDL")) s->opt_pdl = atoi(e) ? 1 : 0;       // default for new sessions
    if (const char* e = getenv("LUMI_GRAPH")) s->opt_graph = atoi(e) ? 1 : 0;
    if (const char* e = getenv("LUMI_MEGAKERNEL")) s->opt_mega = atoi(e) ? 1 : 0;
    if (const char* e = getenv("LUMI_CHUNKED_PREFILL")) s->opt_chunked_prefill = atoi(e) < 0 ? 0 : atoi(e);
    if (const char* e = getenv("LUMI_OVERLAP")) s->opt_overlap = atoi(e) < 0 ? 0 : atoi(e);
    int32_t st = session_alloc(s);
    if (st == LUMI_OK) st = lumi_session_reset(s, nullptr, 0);
    if (st != LUMI_OK) {
        char keep[sizeof(lumi::g_err)];
        memcpy(keep, lumi::g_err, sizeof(keep));
        cudaGetLastError();
        lumi_session_free(s);
        memcpy(lumi::g_err, keep, sizeof(keep));
        return st;
    }
    *out = s;
    return LUMI_OK;
}

extern "C" int32_t lumi_session_reset(lumi_session* s, const int32_t* slots, int32_t n_slots) {
    if (!s) return fail(LUMI_E_INVALID, "session is null");
    const Config& c = s->m->cfg;
    LUMI_CUDA(cudaSetDevice(s->m->device));
    const size_t B = s->max_batch;
    int32_t* dslots = nullptr;
    int n = (int)B;
    if (slots) {
        if (n_slots <= 0) return LUMI_OK;
        for (int i = 0; i < n_slots; ++i)
            if (slots[i] < 0 || slots[i] >= s->max_batch) return fail(LUMI_E_INVALID, "slot %d out of range [0,%d)", slots[i], s->max_batch);
        if (n_slots > s->max_batch) return fail(LUMI_E_INVALID, "%d slots given, the session has %d", n_slots, s->max_batch);
        dslots = s->slot_buf;                        // allocated with the session: a reset allocates nothing
        LUMI_CUDA(cudaMemcpyAsync(dslots, slots, sizeof(int32_t) * n_slots, cudaMemcpyHostToDevice, s->stream));
        n = n_slots;
    }
    for (auto& L : s->m->layers) {
        if (L.is_attn) continue;
        const size_t l = L.kind_idx;
        LUMI_CUDA(launch_state_reset(s->h + l * B * state_h_per_seq(c), s->xprev + l * B * c.d_inner(),
                                     s->bprev + l * B * c.n_heads * c.d_state, s->cum + l * B * c.n_heads * (c.d_state / 2),
                                     L.m.h_init, dslots, n, c.n_heads, c.head_dim(), c.d_state, s->stream));
    }
    if (!slots) {
        LUMI_CUDA(cudaMemsetAsync(s->kv_pos, 0, sizeof(int32_t) * B, s->stream));
    } else {
        for (int i = 0; i < n_slots; ++i) LUMI_CUDA(cudaMemsetAsync(s->kv_pos + slots[i], 0, sizeof(int32_t), s->stream));
    }
    LUMI_CUDA(cudaStreamSynchronize(s->stream));
    return LUMI_OK;
}

extern "C" int32_t lumi_session_set_option(lumi_session* s, const char* name, int64_t value) {
    if (!s || !name) return fail(LUMI_E_INVALID, "null argument to lumi_session_set_option");
    const std::string n(name);
    if (n == "gemm") { if (value < 0 || value > 2) return fail(LUMI_E_INVALID, "option gemm: 0, 1 or 2"); s->opt_gemm = (int)value; }
    else if (n == "split_activations") s->opt_split = value ? 1 : 0;
    else if (n == "graph") s->opt_graph = value ? 1 : 0;
    else if (n == "pdl") s->opt_pdl = value ? 1 : 0;
    else if (n == "megakernel") s->opt_mega = value ? 1 : 0;
    else if (n == "overlap") s->opt_overlap = value < 0 ? 0 : (int)value;
    else if (n == "chunked_prefill") s->opt_chunked_prefill = value < 0 ? 0 : (int)value;
    else if (n == "prefill_rows") s->opt_prefill_rows = value < 64 ? 64 : (int)value;
    else return fail(LUMI_E_INVALID, "unknown option '%s'", name);
    for (auto& g : s->graphs) if (g.second.exec) cudaGraphExecDestroy(g.second.exec);   // captured choices are stale
    s->graphs.clear();
    return LUMI_OK;
}

// ---- one step ---------------------------------------------------------------------------------------
namespace {

enum Family { FAM_EMBED = 0, FAM_NORM, FAM_IN_PROJ, FAM_SSM, FAM_OUT_PROJ, FAM_ATTN, FAM_HEAD, FAM_SAMPLE, FAM_COUNT };

struct StepPlan {
    lumi_session* s;
    int B;
    bool tc;         // tensor-core GEMMs (bf16 weights, batch > 8) or the weight-streaming GEMV
    int64_t n = 0;   // launches enqueued
    int row0 = 0;                                                 // first sequence of this plan's rows (B of them)
    cudaStream_t st_hi = nullptr, st_lo = nullptr;               // GEMM / norm stream and state-step stream (both = session stream unless two lanes run)
    int fam = FAM_EMBED;                                          // family of the launches that follow
    // tensor-core path: the residual rows times the next norm's weights (bf16 halves) and their partial sums of squares are
    // already in xn_hi / xn_lo / ssq — left there by the epilogue of the product that last updated the residual
    bool xn_ready = false;
    int ssq_parts = 0;
    const int32_t* row_len = nullptr;                             // prompts of different lengths (ragged prefill), else null
    std::vector<std::pair<int, cudaEvent_t>>* prof = nullptr;     // profiling: an event before every launch
};

// Counts a launch and, when profiling, drops an event in front of it.
void mark(StepPlan& p) {
    p.n += 1;
    if (p.prof) {
        cudaEvent_t e = nullptr;
        if (cudaEventCreate(&e) == cudaSuccess) {
            cudaEventRecord(e, p.s->stream);
            p.prof->push_back({p.fam, e});
        }
    }
}

bool use_tc(const lumi_session* s, int B) {
    const Config& c = s->m->cfg;
    if (s->m->wdtype != LUMI_DTYPE_BF16 || s->opt_gemm == 1) return false;
    if ((c.d_model % 64) || (c.d_inner() % 64) || (s->m->n_attn > 0 && (c.mlp_dim() % 64))) return false;
    return s->opt_gemm == 2 || B > 8;
}

// norm_in: the input is RMSNorm(residual; gamma) and the tensor-core path takes it in the folded form (rows of x * gamma
// in xn_hi / xn_lo, scale applied in the product's epilogue).  gamma_next != null: the output IS the residual stream;
// the tensor-core product also leaves residual * gamma_next and its sums of squares for the next product.
int32_t linear(StepPlan& p, const DevTensor& W, const float* in32, int K, float* out, int ldd, const float* residual,
               const float* gamma, int act, int N, bool norm_in = false, const float* gamma_next = nullptr) {
    lumi_session* s = p.s;
    const Config& c = s->m->cfg;
    if (!p.tc) {
        GemvArgs g{in32, K, W.p, W.dtype, out, ldd, residual, gamma, p.B, N, K, c.eps, act, &s->ctl->status};
        mark(p);
        LUMI_CUDA(launch_gemv(g, p.st_hi));
        return LUMI_OK;
    }
    // tensor-core path: the caller has already put the bf16 halves of the input into this plan's
    // region of act_hi / act_lo (rows packed with leading dimension K from the region's start)
    const size_t aoff = (size_t)p.row0 * s->act_ld, xoff = (size_t)p.row0 * c.d_model, soff = (size_t)p.row0 * s->ssq_stride;
    const __nv_bfloat16* ahi = norm_in ? s->xn_hi + xoff : s->act_hi + aoff;
    const __nv_bfloat16* alo = norm_in ? s->xn_lo + xoff : s->act_lo + aoff;
    GemmArgs g{ahi, s->opt_split ? alo : nullptr, (const __nv_bfloat16*)W.p, out, ldd, p.B, N, K,
               residual != nullptr ? 1 : 0, &s->ctl->status, s->gemm_counters + (p.row0 > 0 ? kGemmCounters : 0), kGemmCounters,
               s->gemm_scratch + (p.row0 > 0 ? kGemmScratchFloats : 0), kGemmScratchFloats};
    if (norm_in) {
        g.nf.ssq_in = s->ssq + soff; g.nf.ssq_parts = p.ssq_parts; g.nf.ssq_stride = s->ssq_stride;
        g.nf.inv_k = (float)(1.0 / (double)K); g.nf.eps = c.eps;
    }
    if (gamma_next != nullptr) {
        g.nf.gamma_next = gamma_next; g.nf.out_hi = s->xn_hi + xoff; g.nf.out_lo = s->opt_split ? s->xn_lo + xoff : nullptr;
        g.nf.ssq_out = s->ssq + soff; g.nf.ssq_stride = s->ssq_stride;
    }
    mark(p);
    LUMI_TRY(launch_gemm_tcgen05(g, p.st_hi));
    if (gamma_next != nullptr) { p.xn_ready = true; p.ssq_parts = (N + 31) / 32; }      // one partial sum per 32 columns, whatever the tile width
    return LUMI_OK;
}

// Tensor-core path: makes sure xn_hi / xn_lo / ssq hold residual * gamma for the norm that comes next (only the first
// norm of a step needs a kernel of its own; afterwards the products' epilogues keep them current).
int32_t ensure_norm_input(StepPlan& p, const float* x, const float* gamma) {
    lumi_session* s = p.s;
    const Config& c = s->m->cfg;
    if (p.xn_ready) return LUMI_OK;
    const size_t xoff = (size_t)p.row0 * c.d_model, soff = (size_t)p.row0 * s->ssq_stride;
    const int fam = p.fam;
    p.fam = FAM_NORM;
    mark(p);
    LUMI_CUDA(launch_norm_split(x, gamma, s->xn_hi + xoff, s->opt_split ? s->xn_lo + xoff : nullptr, p.B, c.d_model, c.eps, p.st_hi,
                                s->ssq + soff, s->ssq_stride));
    p.fam = fam;
    p.xn_ready = true;
    p.ssq_parts = 1;
    return LUMI_OK;
}

// The weights of the norm that reads the residual stream after layer `li`: the next layer's first norm, or the final norm.
const float* next_norm_gamma(const lumi_session* s, size_t li) {
    if (li + 1 < s->m->layers.size()) {
        const Layer& nx = s->m->layers[li + 1];
        return nx.is_attn ? nx.a.attn_norm_g : nx.m.norm_g;
    }
    return s->m->final_norm_g;
}

// One Mamba block for rows [p.row0, p.row0 + p.B).  With two lanes running, `between` (if given) is
// recorded/awaited around the state step so that it runs on the lane's low-priority stream.
int32_t mamba_block(StepPlan& p, const Layer& L, cudaEvent_t ev_gemm_done = nullptr, cudaEvent_t ev_ssm_done = nullptr) {
    lumi_session* s = p.s;
    const Config& c = s->m->cfg;
    const size_t B = s->max_batch, l = L.kind_idx, r0 = p.row0;
    const int D = c.d_model, DI = c.d_inner(), R = c.in_proj_out();
    const size_t aoff = r0 * s->act_ld;
    float* x = s->x + r0 * D;
    float* proj = s->proj + r0 * R;
    float* y32 = s->y32 ? s->y32 + r0 * DI : nullptr;
    const size_t li = (size_t)(&L - s->m->layers.data());
    if (p.tc) LUMI_TRY(ensure_norm_input(p, x, L.m.norm_g));
    p.fam = FAM_IN_PROJ;
    LUMI_TRY(linear(p, L.m.in_proj, x, D, proj, R, nullptr, L.m.norm_g, 0, R, true));
    p.xn_ready = false;                                   // consumed; the out_proj below renews it
    if (ev_gemm_done) {
        LUMI_CUDA(cudaEventRecord(ev_gemm_done, p.st_hi));
        LUMI_CUDA(cudaStreamWaitEvent(p.st_lo, ev_gemm_done, 0));
    }
    SsmArgs a{};
    a.proj = proj; a.ldp = R;
    a.bg = L.m.b_gamma; a.cg = L.m.c_gamma; a.bb = L.m.b_bias; a.cb = L.m.c_bias; a.dskip = L.m.d_skip; a.dtb = L.m.dt_bias;
    a.h = s->h + (l * B + r0) * state_h_per_seq(c);
    a.xprev = s->xprev + (l * B + r0) * DI;
    a.bprev = s->bprev + (l * B + r0) * c.n_heads * c.d_state;
    a.cum = s->cum + (l * B + r0) * c.n_heads * (c.d_state / 2);
    a.y32 = p.tc ? nullptr : y32;
    a.yhi = p.tc ? s->act_hi + aoff : nullptr;
    a.ylo = (p.tc && s->opt_split) ? s->act_lo + aoff : nullptr;
    a.B = p.B; a.H = c.n_heads; a.P = c.head_dim(); a.N = c.d_state; a.G = c.n_groups; a.eps = c.eps;
    a.row_len = p.row_len; a.ctl = s->ctl;
    p.fam = FAM_SSM;
    mark(p);
    LUMI_CUDA(launch_ssm_step(a, p.st_lo));
    if (ev_ssm_done) {
        LUMI_CUDA(cudaEventRecord(ev_ssm_done, p.st_lo));
        LUMI_CUDA(cudaStreamWaitEvent(p.st_hi, ev_ssm_done, 0));
    }
    p.fam = FAM_OUT_PROJ;
    LUMI_TRY(linear(p, L.m.out_proj, y32, DI, x, D, x, nullptr, 0, D, false, next_norm_gamma(s, li)));
    return LUMI_OK;
}

int32_t attention_block(StepPlan& p, const Layer& L) {
    lumi_session* s = p.s;
    const Config& c = s->m->cfg;
    const int D = c.d_model, KV = c.kv_dim(), Q = D + 2 * KV, MLP = c.mlp_dim();
    const size_t li = (size_t)(&L - s->m->layers.data());
    p.fam = FAM_ATTN;
    if (p.tc) LUMI_TRY(ensure_norm_input(p, s->x, L.a.attn_norm_g));
    p.fam = FAM_ATTN;
    LUMI_TRY(linear(p, L.a.qkv, s->x, D, s->proj, Q, nullptr, L.a.attn_norm_g, 0, Q, true));
    p.xn_ready = false;
    AttnArgs a{};
    a.qkv = s->proj; a.ldq = Q;
    a.pool = (char*)s->kv_pool + (size_t)L.kind_idx * s->kv_layer_bytes;
    a.pool_bytes = s->kv_layer_bytes;
    a.kv_is_f32 = s->m->wdtype == LUMI_DTYPE_BF16 ? 0 : 1;
    a.page_table = s->page_table; a.pages_per_seq = s->pages_per_seq;
    a.pos = s->kv_pos;
    a.ctx32 = p.tc ? nullptr : s->y32;
    a.chi = p.tc ? s->act_hi : nullptr;
    a.clo = (p.tc && s->opt_split) ? s->act_lo : nullptr;
    a.B = p.B; a.n_heads = c.attn_n_heads; a.kv_heads = c.attn_kv_heads; a.head_dim = c.attn_head_dim();
    a.window = L.window; a.max_tokens = s->pages_per_seq * kPageTokens;
    if (a.max_tokens > s->max_tokens_kv) a.max_tokens = s->max_tokens_kv;
    a.rope_base = c.attn_rope_base;
    a.ctl = s->ctl;
    a.row_len = p.row_len;
    if ((long)p.B * c.attn_kv_heads <= kAttnPartUnits) {      // few rows: the context may be split over CTAs
        a.part = s->attn_part; a.part_count = s->attn_part_count;
        a.max_ctx_hint = L.window > 0 ? std::min(L.window, a.max_tokens) : a.max_tokens;
    }
    mark(p);
    cudaError_t e = launch_attention_decode(a, p.st_hi);
    if (e == cudaErrorInvalidValue) return fail(LUMI_E_UNSUPPORTED, "attention head_dim %d with %d query heads per kv head is not built", a.head_dim, a.n_heads / a.kv_heads);
    LUMI_CUDA(e);
    LUMI_TRY(linear(p, L.a.o, s->y32, D, s->x, D, s->x, nullptr, 0, D, false, L.a.mlp_norm_g));
    // sigmoid-gated MLP (model.rs:546-555)
    if (p.tc) {
        LUMI_TRY(linear(p, L.a.gate_up, nullptr, D, s->proj, 2 * MLP, nullptr, nullptr, 0, 2 * MLP, true));
        p.xn_ready = false;
        mark(p);
        LUMI_CUDA(launch_gate_mul(s->proj, 2 * MLP, nullptr, s->act_hi, s->opt_split ? s->act_lo : nullptr, p.B, MLP, p.st_hi));
    } else {
        LUMI_TRY(linear(p, L.a.gate_up, s->x, D, s->y32, MLP, nullptr, L.a.mlp_norm_g, 1, MLP));
    }
    LUMI_TRY(linear(p, L.a.down, s->y32, MLP, s->x, D, s->x, nullptr, 0, D, false, next_norm_gamma(s, li)));
    return LUMI_OK;
}

// embedding -> blocks -> (final norm -> logits -> sample) -> advance
// Largest batch of the tensor-core path whose CUDA-core kernels are launched with programmatic dependent launch
// (LUMI_PDL_TC; 0 = never): the state step then becomes resident under the in_proj GEMM and requests its tiles early.
static int pdl_tc_max() {
    static int v = -1;
    if (v < 0) { const char* e = getenv("LUMI_PDL_TC"); v = e ? atoi(e) : 128; }     // measured: +6 % at 64 rows, -3..5 % at 512-2048
    return v;
}

static int pdl_gemm_max() {
    static int v = -1;
    if (v < 0) { const char* e = getenv("LUMI_PDL_GEMM"); v = e ? atoi(e) : 1024; }     // measured: +2 % at 64-128 rows, +1.2 % at 512, neutral at 2048
    return v;
}

int32_t enqueue_step(lumi_session* s, int B, bool with_head, int64_t* launches,
                     std::vector<std::pair<int, cudaEvent_t>>* prof = nullptr, const int32_t* row_len = nullptr) {
    const Config& c = s->m->cfg;
    StepPlan p{s, B, use_tc(s, B)};
    p.prof = prof;
    p.row_len = row_len;
    // dependent launch overlaps each kernel's prologue (weight prefetch) with its predecessor; it is
    // used on the weight-streaming path, where launch gaps are the same order as the kernels
    struct PdlScope { PdlScope(bool on) { set_launch_pdl(on); } ~PdlScope() { set_launch_pdl(false); } } pdl_scope(s->opt_pdl && prof == nullptr && (!p.tc || (pdl_tc_max() > 0 && B <= pdl_tc_max())));
    // the tensor-core GEMMs themselves: dependent launch up to LUMI_PDL_GEMM rows (their barrier / TMEM set-up then runs under the
    // tail of the state step; unlike an early state step this takes nothing from a running GEMM)
    struct PdlGemmScope { PdlGemmScope(bool on) { set_launch_pdl_gemm(on); } ~PdlGemmScope() { set_launch_pdl_gemm(false); } } pdl_gemm_scope(s->opt_pdl && prof == nullptr && p.tc && B <= pdl_gemm_max());
    p.st_hi = p.st_lo = s->stream;
    mark(p);
    LUMI_CUDA(launch_embed(s->m->embedding.p, s->m->embedding.dtype, s->tok_cur, s->x, B, c.d_model, c.vocab, s->ctl, s->stream, row_len));
    const bool two_lanes = p.tc && prof == nullptr && row_len == nullptr && s->opt_overlap > 0 && B >= s->opt_overlap && s->m->n_attn == 0 && B >= 2;
    if (!two_lanes) {
        for (const Layer& L : s->m->layers) {
            if (L.is_attn) LUMI_TRY(attention_block(p, L));
            else LUMI_TRY(mamba_block(p, L));
        }
    } else {
        // Two lanes of sequences run the whole layer chain independently.  The GEMMs (tensor pipe,
        // shared memory) of one lane are meant to run under the state step (HBM) of the other, so
        // GEMM kernels go to high-priority streams — pending high-priority CTAs are placed before
        // the thousands of pending state-step CTAs — and lane 1 starts one GEMM ahead of lane 0.
        const int half = (B / 2 + 127) / 128 * 128 < B ? (B / 2 + 127) / 128 * 128 : B / 2;
        StepPlan lane[2] = {p, p};
        lane[0].row0 = 0; lane[0].B = half;
        lane[1].row0 = half; lane[1].B = B - half;
        LUMI_CUDA(cudaEventRecord(s->ev_fork, s->stream));
        for (int i = 0; i < 2; ++i) {
            lane[i].n = 0;
            lane[i].st_hi = s->lane_hi[i];
            lane[i].st_lo = s->lane_lo[i];
            LUMI_CUDA(cudaStreamWaitEvent(s->lane_hi[i], s->ev_fork, 0));
        }
        bool first = true;
        for (const Layer& L : s->m->layers) {
            LUMI_TRY(mamba_block(lane[1], L, s->lane_ev[1][0], s->lane_ev[1][1]));
            if (first) {        // lane 0 begins once lane 1's first in_proj is done
                LUMI_CUDA(cudaStreamWaitEvent(s->lane_hi[0], s->lane_ev[1][0], 0));
                first = false;
            }
            LUMI_TRY(mamba_block(lane[0], L, s->lane_ev[0][0], s->lane_ev[0][1]));
        }
        for (int i = 0; i < 2; ++i) {
            LUMI_CUDA(cudaEventRecord(s->ev_join[i], s->lane_hi[i]));
            LUMI_CUDA(cudaStreamWaitEvent(s->stream, s->ev_join[i], 0));
            p.n += lane[i].n;
        }
        // both lanes left their rows of the folded-norm input behind, in the same per-strip form
        p.xn_ready = lane[0].xn_ready && lane[1].xn_ready && lane[0].ssq_parts == lane[1].ssq_parts;
        p.ssq_parts = lane[0].ssq_parts;
    }
    // greedy head at small batch: the argmax rides behind the lm_head GEMV (per-CTA partials) and one small kernel
    // finishes the token and the step — no logits are written and nothing re-reads them
    const bool fused = with_head && s->fused_head && !p.tc && B <= 8 && c.vocab >= 4096 && prof == nullptr;
    if (fused) {
        p.fam = FAM_HEAD;
        int nparts = 0;
        GemvArgs g{s->x, c.d_model, s->m->embedding.p, s->m->embedding.dtype, nullptr, c.vocab, nullptr, s->m->final_norm_g, B, c.vocab,
                   c.d_model, c.eps, 0, &s->ctl->status};
        g.amax_val = s->amax_val; g.amax_idx = s->amax_idx; g.amax_stride = s->amax_stride; g.amax_parts = &nparts;
        mark(p);
        LUMI_CUDA(launch_gemv(g, s->stream));
        p.fam = FAM_SAMPLE;
        mark(p);
        LUMI_CUDA(launch_head_finish(s->amax_val, s->amax_idx, nparts, s->amax_stride, B, s->ctl, s->tok_cur, s->finished, s->out_len,
                                     s->m->n_attn > 0 ? s->kv_pos : nullptr, s->stream));
        *launches = p.n;
        return LUMI_OK;
    }
    if (with_head) {
        p.fam = FAM_HEAD;
        if (p.tc) LUMI_TRY(ensure_norm_input(p, s->x, s->m->final_norm_g));
        p.fam = FAM_HEAD;
        LUMI_TRY(linear(p, s->m->embedding, s->x, c.d_model, s->logits, c.vocab, nullptr, s->m->final_norm_g, 0, c.vocab, true));
        p.fam = FAM_SAMPLE;
        mark(p);
        LUMI_CUDA(launch_sample(s->logits, B, c.vocab, s->ctl, s->tok_cur, s->finished, s->out_len, s->stream));
    }
    if (row_len != nullptr) {                      // ragged prefill: keep the residual of every sequence that is at its last prompt token
        mark(p);
        LUMI_CUDA(launch_capture_last(s->x, s->xlast, row_len, s->ctl, B, c.d_model, s->stream));
    }
    p.fam = FAM_SAMPLE;
    mark(p);
    LUMI_CUDA(launch_advance_step(s->ctl, s->m->n_attn > 0 ? s->kv_pos : nullptr, B, with_head ? 1 : 0, s->stream, row_len));
    if (prof) {   // closing event
        p.fam = FAM_COUNT;
        mark(p);
        p.n -= 1;
    }
    *launches = p.n;
    return LUMI_OK;
}

// Runs one step, through a captured graph when enabled.
// `reps` consecutive identical steps as one graph launch (reps > 1 only for small batches, where the gap
// between two graph launches is a visible part of a step).
int32_t run_step(lumi_session* s, int B, bool with_head, int reps = 1) {
    if (!s->opt_graph) {
        for (int r = 0; r < reps; ++r) {
            int64_t n = 0;
            LUMI_TRY(enqueue_step(s, B, with_head, &n));
            s->launches += n;
        }
        return LUMI_OK;
    }
    const int64_t key = (((((int64_t)B * 2 + (with_head ? 1 : 0)) << 1) | (s->fused_head ? 1 : 0)) << 8) | (int64_t)reps;
    auto it = s->graphs.find(key);
    if (it == s->graphs.end()) {
        GraphEntry ge;
        for (int attempt = 0; attempt < 2; ++attempt) {
            cudaGraph_t graph = nullptr;
            LUMI_CUDA(cudaStreamBeginCapture(s->stream, cudaStreamCaptureModeThreadLocal));
            int32_t st = LUMI_OK;
            ge.launches = 0;
            for (int r = 0; r < reps && st == LUMI_OK; ++r) {
                int64_t n = 0;
                st = enqueue_step(s, B, with_head, &n);
                ge.launches += n;
            }
            cudaError_t e = cudaStreamEndCapture(s->stream, &graph);
            if (st == LUMI_OK && e == cudaSuccess) {
                e = cudaGraphInstantiate(&ge.exec, graph, 0);
                cudaGraphDestroy(graph);
                if (e == cudaSuccess) break;
            } else if (graph) {
                cudaGraphDestroy(graph);
            }
            // a driver that cannot capture programmatic edges: once more with plain edges
            if (attempt == 0 && s->opt_pdl) { s->opt_pdl = 0; cudaGetLastError(); ge = GraphEntry(); continue; }
            if (st != LUMI_OK) return st;
            LUMI_CUDA(e);
        }
        it = s->graphs.emplace(key, ge).first;
    }
    LUMI_CUDA(cudaGraphLaunch(it->second.exec, s->stream));
    s->launches += it->second.launches;
    return LUMI_OK;
}

// n identical steps: at small batch in graphs of kStepsPerGraph steps, the rest one by one
constexpr int kStepsPerGraph = 8;
int32_t run_steps(lumi_session* s, int B, bool with_head, int n) {
    if (s->opt_graph && B <= 16)
        for (; n >= kStepsPerGraph; n -= kStepsPerGraph) LUMI_TRY(run_step(s, B, with_head, kStepsPerGraph));
    for (; n > 0; --n) LUMI_TRY(run_step(s, B, with_head));
    return LUMI_OK;
}

bool use_b1(const lumi_session* s, int batch) { return batch == 1 && s->b1_ok && s->opt_mega; }

// n_tokens forward steps of sequence 0 in one persistent kernel (decode_b1.cu)
int32_t run_b1(lumi_session* s, int n_tokens, int head_mode, int do_argmax) {
    if (n_tokens <= 0) return LUMI_OK;
    const Config& c = s->m->cfg;
    B1Args a{};
    a.layers = s->b1_layers; a.n_layers = c.n_layers;
    a.emb = s->m->embedding.p; a.final_g = s->m->final_norm_g;
    a.vocab = c.vocab; a.D = c.d_model; a.DI = c.d_inner(); a.R = c.in_proj_out(); a.H = c.n_heads; a.G = c.n_groups; a.BC = c.bc();
    a.eps = c.eps;
    a.xt = s->b1_tagged; a.pt = a.xt + c.d_model; a.yt = a.pt + c.in_proj_out();
    a.logits = s->logits;
    // epochs never repeat within a session: (layers + 1) per token, and a margin per launch
    const uint64_t need = (uint64_t)n_tokens * (c.n_layers + 1) + 2;
    if ((uint64_t)s->b1_epoch + need >= 0xffffff00ull) {
        LUMI_CUDA(cudaMemsetAsync(s->b1_tagged, 0, ((size_t)c.d_model + c.in_proj_out() + c.d_inner()) * 8, s->stream));
        s->b1_epoch = 1;
    }
    a.epoch_base = s->b1_epoch;
    s->b1_epoch += (uint32_t)need;
    a.tok_cur = s->tok_cur; a.finished = s->finished; a.out_len = s->out_len;
    a.ctl = s->ctl;
    a.grid_ctl = s->b1_grid_ctl; a.amax_val = s->b1_amax_val; a.amax_idx = s->b1_amax_idx;
    a.n_tokens = n_tokens; a.head_mode = head_mode; a.do_argmax = do_argmax;
    // LUMI_B1_TIMING=1 (tuning aid): per-phase timestamps of the last token, printed to stderr
    static const bool want_timing = getenv("LUMI_B1_TIMING") && atoi(getenv("LUMI_B1_TIMING"));
    if (want_timing && !s->b1_timing) {
        LUMI_CUDA(cudaMalloc(&s->b1_timing, sizeof(unsigned long long) * 2 * c.n_layers * 10));
    }
    a.timing = want_timing ? s->b1_timing : nullptr;
    if (want_timing) LUMI_CUDA(cudaMemsetAsync(s->b1_timing, 0, sizeof(unsigned long long) * 2 * c.n_layers * 10, s->stream));
    LUMI_CUDA(launch_decode_b1(a, s->m->wdtype, s->m->device, s->stream));
    s->launches += 1;
    if (want_timing && n_tokens > 1) {
        std::vector<unsigned long long> tm((size_t)2 * c.n_layers * 10);
        LUMI_CUDA(cudaMemcpyAsync(tm.data(), s->b1_timing, tm.size() * 8, cudaMemcpyDeviceToHost, s->stream));
        LUMI_CUDA(cudaStreamSynchronize(s->stream));
        static const char* names[9] = {"gatherX", "rowsA", "-", "pollB", "stepB", "-", "gatherY", "rowsC", "sync"};
        for (int sel = 0; sel < 2; ++sel) {
            double acc[9] = {0};
            int n = 0;
            for (int l = 1; l < c.n_layers; ++l) {
                const unsigned long long* r = &tm[((size_t)sel * c.n_layers + l) * 10];
                if (!r[0] || !r[9]) continue;
                unsigned long long prev = r[0];
                for (int i = 1; i < 10; ++i) {
                    if (!r[i]) continue;           // stamps a CTA without a head never writes
                    acc[i - 1] += (double)(r[i] - prev);
                    prev = r[i];
                }
                ++n;
            }
            fprintf(stderr, "[b1 timing] CTA %d, mean ns per layer over %d layers:", sel == 0 ? 0 : 100, n);
            double tot = 0;
            for (int i = 0; i < 9; ++i) { fprintf(stderr, " %s %.0f", names[i], n ? acc[i] / n : 0.0); tot += n ? acc[i] / n : 0.0; }
            fprintf(stderr, " | layer %.0f\n", tot);
        }
    }
    return LUMI_OK;
}

// after run_b1(..., do_argmax = 0): temperature / top-k sampling of the logits it left behind
int32_t sample_after_b1(lumi_session* s) {
    const Config& c = s->m->cfg;
    LUMI_CUDA(launch_sample(s->logits, 1, c.vocab, s->ctl, s->tok_cur, s->finished, s->out_len, s->stream));
    LUMI_CUDA(launch_advance_step(s->ctl, nullptr, 1, 1, s->stream));
    s->launches += 2;
    return LUMI_OK;
}

template <typename T>
int32_t grow(T*& p, size_t& cap, size_t need_elems) {
    if (need_elems <= cap) return LUMI_OK;
    if (p) LUMI_CUDA(cudaFree(p));
    p = nullptr; cap = 0;
    LUMI_CUDA(cudaMalloc(&p, need_elems * sizeof(T)));
    cap = need_elems;
    return LUMI_OK;
}

bool use_chunked_prefill(const lumi_session* s, int batch, int T) {
    if (!(s->opt_chunked_prefill > 0 && T >= s->opt_chunked_prefill && s->m->wdtype == LUMI_DTYPE_BF16 && s->opt_gemm != 1 &&
          prefill_ssd_supported(s->m->cfg) && (s->m->cfg.d_model % 64) == 0 && (s->m->cfg.d_inner() % 64) == 0))
        return false;
    if (s->m->n_attn > 0) {
        // attention layers: every row of a slice is appended before any row attends, which a sliding-window ring
        // cannot take (later rows of the slice would overwrite slots that earlier rows still need)
        if ((s->m->cfg.mlp_dim() % 64) != 0) return false;
        for (const Layer& L : s->m->layers) if (L.is_attn && L.window > 0) return false;
    }
    return true;
}

// Prompt of T tokens for sequences 0..batch-1 through the chunked SSD scan; tokens come from
// prompt_dev[T][batch].  Leaves the decode state of every layer as the step-by-step path would, the
// last position's residual in x, and (with_head) its logits plus the sampled first token.
// score_out (device, [batch][T-1]) != null: log p(next prompt token) at every position, from the head over all rows.
// lens (device, [batch]) != null: prompts of different lengths inside the [T][batch] rectangle (T = the longest): every sequence
// ends in the state after its own last token, x holds the residual at that token, and padding is never looked at.
int32_t prefill_chunked(lumi_session* s, int batch, int T, bool with_head, float* score_out = nullptr, const int32_t* lens = nullptr) {
    const Config& c = s->m->cfg;
    const int D = c.d_model, DI = c.d_inner(), R = c.in_proj_out();
    const bool hybrid = s->m->n_attn > 0;
    const int KVD = hybrid ? c.kv_dim() : 0, Q = D + 2 * KVD, MLP = hybrid ? c.mlp_dim() : 0;
    const size_t wproj = std::max<size_t>({(size_t)R, (size_t)Q, (size_t)2 * MLP});       // widest fp32 row of a projection
    const size_t wact = std::max<size_t>({(size_t)DI, (size_t)D, (size_t)MLP});           // widest bf16 operand row
    const int nb_max = std::min(batch, 2048);
    int TS = std::max(64, (std::max(64, s->opt_prefill_rows) / nb_max) / 64 * 64);
    if (TS > T) TS = T;
    const size_t rows_max = (size_t)nb_max * TS;
    if (rows_max > s->pf_rows) {
        void* olds[] = {s->pf_x, s->pf_proj, s->pf_rb, s->pf_rc, s->pf_hi, s->pf_lo};
        for (void* q : olds) if (q) LUMI_CUDA(cudaFree(q));
        s->pf_x = s->pf_proj = s->pf_rb = s->pf_rc = nullptr; s->pf_hi = s->pf_lo = nullptr; s->pf_rows = 0;
        const size_t rp = (rows_max + 127) / 128 * 128;
        LUMI_CUDA(cudaMalloc(&s->pf_x, sizeof(float) * rp * D));
        LUMI_CUDA(cudaMalloc(&s->pf_proj, sizeof(float) * rp * wproj));
        LUMI_CUDA(cudaMalloc(&s->pf_rb, sizeof(float) * rp));
        LUMI_CUDA(cudaMalloc(&s->pf_rc, sizeof(float) * rp));
        LUMI_CUDA(cudaMalloc(&s->pf_hi, sizeof(__nv_bfloat16) * rp * wact));
        LUMI_CUDA(cudaMalloc(&s->pf_lo, sizeof(__nv_bfloat16) * rp * wact));
        // rows that a launch skips (padding behind a shorter prompt) keep what they held: make that finite from the start
        LUMI_CUDA(cudaMemsetAsync(s->pf_x, 0, sizeof(float) * rp * D, s->stream));
        LUMI_CUDA(cudaMemsetAsync(s->pf_proj, 0, sizeof(float) * rp * wproj, s->stream));
        LUMI_CUDA(cudaMemsetAsync(s->pf_hi, 0, sizeof(__nv_bfloat16) * rp * wact, s->stream));
        LUMI_CUDA(cudaMemsetAsync(s->pf_lo, 0, sizeof(__nv_bfloat16) * rp * wact, s->stream));
        s->pf_rows = rows_max;
    }
    const size_t B = s->max_batch;
    __nv_bfloat16* lo = s->opt_split ? s->pf_lo : nullptr;
    for (int b0 = 0; b0 < batch; b0 += nb_max) {
        const int nb = std::min(nb_max, batch - b0);
        for (int t0 = 0; t0 < T; t0 += TS) {
            const int ts = std::min(TS, T - t0);
            const int M = nb * ts;
            LUMI_CUDA(launch_prefill_embed(s->m->embedding.p, s->m->embedding.dtype, s->prompt_dev, s->pf_x, D, c.vocab, M, ts, t0, b0,
                                           batch, s->ctl, s->stream, lens));
            s->launches += 1;
            for (const Layer& L : s->m->layers) {
                const size_t l = L.kind_idx;
                if (L.is_attn) {
                    // AttentionBlock over all rows of the slice (model.rs:562-611 in forward_window's terms): q|k|v for every
                    // row, the slice's K/V appended to the cache, then every row attends to the cache up to its own position
                    LUMI_CUDA(launch_norm_split(s->pf_x, L.a.attn_norm_g, s->pf_hi, lo, M, D, c.eps, s->stream));
                    GemmArgs gq{s->pf_hi, lo, (const __nv_bfloat16*)L.a.qkv.p, s->pf_proj, Q, M, Q, D, 0, &s->ctl->status};
                    LUMI_TRY(launch_gemm_tcgen05(gq, s->stream));
                    AttnArgs a{};
                    a.qkv = s->pf_proj; a.ldq = Q;
                    a.pool = (char*)s->kv_pool + l * s->kv_layer_bytes;
                    a.pool_bytes = s->kv_layer_bytes;
                    a.kv_is_f32 = 0;
                    a.page_table = s->page_table; a.pages_per_seq = s->pages_per_seq;
                    a.pos = s->kv_pos;
                    a.ctx32 = nullptr; a.chi = s->pf_hi; a.clo = lo;
                    a.B = M; a.n_heads = c.attn_n_heads; a.kv_heads = c.attn_kv_heads; a.head_dim = c.attn_head_dim();
                    a.window = 0; a.max_tokens = std::min(s->pages_per_seq * kPageTokens, s->max_tokens_kv);
                    a.rope_base = c.attn_rope_base;
                    a.ctl = s->ctl;
                    a.rows_per_seq = ts; a.b0 = b0;
                    a.row_len = lens;
                    for (int phase = 1; phase <= 2; ++phase) {
                        a.phase = phase;
                        cudaError_t e = launch_attention_decode(a, s->stream);
                        if (e == cudaErrorInvalidValue) return fail(LUMI_E_UNSUPPORTED, "attention head_dim %d with %d query heads per kv head is not built", a.head_dim, a.n_heads / a.kv_heads);
                        LUMI_CUDA(e);
                    }
                    GemmArgs go{s->pf_hi, lo, (const __nv_bfloat16*)L.a.o.p, s->pf_x, D, M, D, D, 1, &s->ctl->status};
                    LUMI_TRY(launch_gemm_tcgen05(go, s->stream));
                    // sigmoid-gated MLP (model.rs:546-555)
                    LUMI_CUDA(launch_norm_split(s->pf_x, L.a.mlp_norm_g, s->pf_hi, lo, M, D, c.eps, s->stream));
                    GemmArgs gu{s->pf_hi, lo, (const __nv_bfloat16*)L.a.gate_up.p, s->pf_proj, 2 * MLP, M, 2 * MLP, D, 0, &s->ctl->status};
                    LUMI_TRY(launch_gemm_tcgen05(gu, s->stream));
                    LUMI_CUDA(launch_gate_mul(s->pf_proj, 2 * MLP, nullptr, s->pf_hi, lo, M, MLP, s->stream));
                    GemmArgs gd{s->pf_hi, lo, (const __nv_bfloat16*)L.a.down.p, s->pf_x, D, M, D, MLP, 1, &s->ctl->status};
                    LUMI_TRY(launch_gemm_tcgen05(gd, s->stream));
                    s->launches += 10;
                    continue;
                }
                LUMI_CUDA(launch_norm_split(s->pf_x, L.m.norm_g, s->pf_hi, lo, M, D, c.eps, s->stream));
                GemmArgs g1{s->pf_hi, lo, (const __nv_bfloat16*)L.m.in_proj.p, s->pf_proj, R, M, R, D, 0, &s->ctl->status};
                LUMI_TRY(launch_gemm_tcgen05(g1, s->stream));
                PrefillArgs a{};
                a.proj = s->pf_proj; a.ldp = R;
                a.bg = L.m.b_gamma; a.cg = L.m.c_gamma; a.bb = L.m.b_bias; a.cb = L.m.c_bias; a.dskip = L.m.d_skip; a.dtb = L.m.dt_bias;
                a.h = s->h + l * B * state_h_per_seq(c);
                a.xprev = s->xprev + l * B * DI;
                a.bprev = s->bprev + l * B * c.n_heads * c.d_state;
                a.cum = s->cum + l * B * c.n_heads * (c.d_state / 2);
                a.rb = s->pf_rb; a.rc = s->pf_rc;
                a.yhi = s->pf_hi; a.ylo = lo;
                a.H = c.n_heads; a.G = c.n_groups; a.ts = ts; a.nb = nb; a.b0 = b0; a.eps = c.eps;
                a.status = &s->ctl->status;
                a.lens = lens; a.t_abs0 = t0;
                LUMI_CUDA(launch_prefill_scan(a, s->stream));
                GemmArgs g2{s->pf_hi, lo, (const __nv_bfloat16*)L.m.out_proj.p, s->pf_x, D, M, D, DI, 1, &s->ctl->status};
                LUMI_TRY(launch_gemm_tcgen05(g2, s->stream));
                s->launches += 5;
            }
            if (hybrid) {
                LUMI_CUDA(launch_kv_advance(s->kv_pos, b0, nb, ts, s->stream, lens, t0));
                s->launches += 1;
            }
            if (score_out != nullptr) {
                // final norm + tied head over the rows of the slice, a block of rows at a time, then log-softmax at the target
                const int V = c.vocab;
                const int SR = (int)std::min<size_t>(4096, std::max<size_t>(128, ((size_t)256 << 20) / ((size_t)V * sizeof(float)) / 128 * 128));
                LUMI_TRY(grow(s->score_logits, s->score_logits_cap, (size_t)SR * V));
                LUMI_CUDA(launch_norm_split(s->pf_x, s->m->final_norm_g, s->pf_hi, lo, M, D, c.eps, s->stream));
                for (int r0 = 0; r0 < M; r0 += SR) {
                    const int nr = std::min(SR, M - r0);
                    GemmArgs gh{s->pf_hi + (size_t)r0 * D, lo ? lo + (size_t)r0 * D : nullptr, (const __nv_bfloat16*)s->m->embedding.p,
                                s->score_logits, V, nr, V, D, 0, &s->ctl->status};
                    LUMI_TRY(launch_gemm_tcgen05(gh, s->stream));
                    LUMI_CUDA(launch_logprob_rows(s->score_logits, nr, V, s->prompt_dev, batch, T, ts, t0, b0, r0, score_out, s->stream));
                    s->launches += 2;
                }
                s->launches += 1;
            }
            if (t0 + ts >= T || lens != nullptr) {      // different lengths: every slice may hold some sequence's last token
                LUMI_CUDA(launch_gather_last(s->pf_x, s->x, D, ts, nb, b0, s->stream, lens, t0));
                s->launches += 1;
            }
        }
    }
    if (with_head) {
        StepPlan p{s, batch, true};
        p.st_hi = p.st_lo = s->stream;
        LUMI_CUDA(launch_norm_split(s->x, s->m->final_norm_g, s->act_hi, s->opt_split ? s->act_lo : nullptr, batch, D, c.eps, s->stream));
        p.fam = FAM_HEAD;
        LUMI_TRY(linear(p, s->m->embedding, s->x, D, s->logits, c.vocab, nullptr, s->m->final_norm_g, 0, c.vocab));
        LUMI_CUDA(launch_sample(s->logits, batch, c.vocab, s->ctl, s->tok_cur, s->finished, s->out_len, s->stream));
        LUMI_CUDA(launch_advance_step(s->ctl, nullptr, batch, 1, s->stream));      // positions were advanced slice by slice
        s->launches += 3 + p.n;
    }
    return LUMI_OK;
}

int32_t check_status(lumi_session* s) {
    const int st = s->ctl_host->status;
    if (st & STATUS_TIMEOUT) {
        unsigned words[8] = {0};
        if (s->b1_grid_ctl) cudaMemcpy(words, s->b1_grid_ctl, sizeof(words), cudaMemcpyDeviceToHost);
        return fail(LUMI_E_TIMEOUT, "a bounded device-side wait expired (tensor-core GEMM or persistent decode kernel; barrier words %u %u %u %u %u %u abort %u diag 0x%x)",
                    words[0], words[1], words[2], words[3], words[4], words[5], words[6], words[7]);
    }
    if (st & STATUS_BAD_TOKEN) return fail(LUMI_E_TOKEN, "a token id was >= vocab_size (%d)", s->m->cfg.vocab);
    if (st & STATUS_KV_FULL) return fail(LUMI_E_KV_FULL, "attention cache capacity (%d tokens per sequence) exceeded", s->max_tokens_kv);
    return LUMI_OK;
}

int32_t check_batch(lumi_session* s, int batch) {
    if (!s) return fail(LUMI_E_INVALID, "session is null");
    if (batch <= 0 || batch > s->max_batch) return fail(LUMI_E_INVALID, "batch %d outside [1, %d]", batch, s->max_batch);
    return LUMI_OK;
}

void fill_ctl(lumi_session* s, int batch, const lumi_sampling* sp) {
    StepCtl& c = *s->ctl_host;
    memset(&c, 0, sizeof(c));
    c.batch = batch;
    if (sp) {
        c.temperature = sp->temperature;
        c.top_k = sp->top_k;
        c.seed_lo = (uint32_t)(sp->seed & 0xffffffffu);
        c.seed_hi = (uint32_t)(sp->seed >> 32);
        c.eos_id = sp->eos_id;
        c.ignore_eos = sp->ignore_eos;
    }
}

int32_t push_ctl(lumi_session* s) {
    LUMI_CUDA(cudaMemcpyAsync(s->ctl, s->ctl_host, sizeof(StepCtl), cudaMemcpyHostToDevice, s->stream));
    return LUMI_OK;
}
int32_t pull_ctl(lumi_session* s) {
    LUMI_CUDA(cudaMemcpyAsync(s->ctl_host, s->ctl, sizeof(StepCtl), cudaMemcpyDeviceToHost, s->stream));
    return LUMI_OK;
}

// prompt[batch][T] (host) -> prompt_dev[T][batch]
int32_t upload_prompt(lumi_session* s, const uint32_t* tokens, int batch, int T) {
    LUMI_TRY(grow(s->prompt_dev, s->prompt_cap, (size_t)batch * T));
    std::vector<uint32_t> tr((size_t)batch * T);
    for (int b = 0; b < batch; ++b)
        for (int t = 0; t < T; ++t) tr[(size_t)t * batch + b] = tokens[(size_t)b * T + t];
    LUMI_CUDA(cudaMemcpyAsync(s->prompt_dev, tr.data(), tr.size() * sizeof(uint32_t), cudaMemcpyHostToDevice, s->stream));
    LUMI_CUDA(cudaStreamSynchronize(s->stream));     // tr goes out of scope
    return LUMI_OK;
}

}  // namespace

extern "C" int32_t lumi_prefill(lumi_session* s, const uint32_t* tokens, int32_t batch, int32_t T, float* last_logits) {
    LUMI_TRY(check_batch(s, batch));
    if (!tokens || T <= 0) return fail(LUMI_E_INVALID, "prefill needs tokens and T > 0");
    LUMI_CUDA(cudaSetDevice(s->m->device));
    s->fused_head = false;
    LUMI_TRY(upload_prompt(s, tokens, batch, T));
    fill_ctl(s, batch, nullptr);
    s->ctl_host->prompt = s->prompt_dev;
    s->ctl_host->prompt_len = T;
    const bool chunked = !use_b1(s, batch) && use_chunked_prefill(s, batch, T);
    if (chunked) s->ctl_host->prompt_pos = T;          // the scan consumes the whole prompt itself
    LUMI_TRY(push_ctl(s));
    if (use_b1(s, batch)) LUMI_TRY(run_b1(s, T, last_logits != nullptr ? 1 : 0, 1));
    else if (chunked) LUMI_TRY(prefill_chunked(s, batch, T, last_logits != nullptr));
    else
        {
            LUMI_TRY(run_steps(s, batch, false, T - 1));
            LUMI_TRY(run_step(s, batch, last_logits != nullptr));
        }
    if (last_logits)
        LUMI_CUDA(cudaMemcpyAsync(last_logits, s->logits, sizeof(float) * batch * s->m->cfg.vocab, cudaMemcpyDeviceToHost, s->stream));
    LUMI_TRY(pull_ctl(s));
    LUMI_CUDA(cudaStreamSynchronize(s->stream));
    return check_status(s);
}

// Prompts of different lengths in one call.  Every sequence goes through its own tokens position by position, as
// lumi_prefill's token-by-token form does; once a sequence's prompt has ended, the kernels that own per-sequence state
// (state step, cache append, position) skip it, so it simply waits for the longest one.
extern "C" int32_t lumi_prefill_ragged(lumi_session* s, const uint32_t* tokens, const int32_t* lengths, int32_t batch, int32_t T_max,
                                       float* last_logits) {
    LUMI_TRY(check_batch(s, batch));
    if (!tokens || !lengths || T_max <= 0) return fail(LUMI_E_INVALID, "ragged prefill needs tokens, lengths and T_max > 0");
    if (batch > 1024) return fail(LUMI_E_UNSUPPORTED, "ragged prefill takes at most 1024 sequences per call");
    int longest = 0;
    for (int b = 0; b < batch; ++b) {
        if (lengths[b] < 1 || lengths[b] > T_max) return fail(LUMI_E_INVALID, "length %d of sequence %d outside [1, %d]", lengths[b], b, T_max);
        longest = std::max(longest, lengths[b]);
    }
    LUMI_CUDA(cudaSetDevice(s->m->device));
    s->fused_head = false;
    LUMI_TRY(upload_prompt(s, tokens, batch, T_max));
    LUMI_CUDA(cudaMemcpyAsync(s->row_len, lengths, sizeof(int32_t) * batch, cudaMemcpyHostToDevice, s->stream));
    fill_ctl(s, batch, nullptr);
    s->ctl_host->prompt = s->prompt_dev;
    s->ctl_host->prompt_len = longest;
    // long prompts: the batched path over the rectangle of the longest one (each sequence stops at its own length)
    const bool chunked = use_chunked_prefill(s, batch, longest);
    if (chunked) s->ctl_host->prompt_pos = longest;
    LUMI_TRY(push_ctl(s));
    if (chunked) {
        LUMI_TRY(prefill_chunked(s, batch, longest, false, nullptr, s->row_len));
    } else {
        const bool mega = s->opt_mega;
        s->opt_mega = 0;
        int32_t rc = LUMI_OK;
        for (int t = 0; t < longest && rc == LUMI_OK; ++t) {       // launched directly: the captured graphs of the step do not carry the length table
            int64_t n = 0;
            rc = enqueue_step(s, batch, false, &n, nullptr, s->row_len);
            s->launches += n;
        }
        s->opt_mega = mega;
        LUMI_TRY(rc);
    }
    if (last_logits) {
        // final norm + tied head on each sequence's residual at its own last token
        if (!chunked) LUMI_CUDA(cudaMemcpyAsync(s->x, s->xlast, sizeof(float) * batch * s->m->cfg.d_model, cudaMemcpyDeviceToDevice, s->stream));
        StepPlan p{s, batch, use_tc(s, batch)};
        p.st_hi = p.st_lo = s->stream;
        const Config& c = s->m->cfg;
        if (p.tc) LUMI_TRY(ensure_norm_input(p, s->x, s->m->final_norm_g));
        p.fam = FAM_HEAD;
        LUMI_TRY(linear(p, s->m->embedding, s->x, c.d_model, s->logits, c.vocab, nullptr, s->m->final_norm_g, 0, c.vocab, true));
        s->launches += p.n;
        LUMI_CUDA(cudaMemcpyAsync(last_logits, s->logits, sizeof(float) * batch * c.vocab, cudaMemcpyDeviceToHost, s->stream));
    }
    LUMI_TRY(pull_ctl(s));
    LUMI_CUDA(cudaStreamSynchronize(s->stream));
    return check_status(s);
}

// Teacher-forced scoring: log p(tokens[b][t+1] | tokens[b][0..t]) for t = 0 .. T-2, the quantity the reference's
// `evaluate` command sums into perplexities and continuation scores (inference/src/eval.rs:39-139, over
// forward_window's logits, model.rs:806-826).  The session's state ends up as after a prefill of all T tokens.
extern "C" int32_t lumi_score(lumi_session* s, const uint32_t* tokens, int32_t batch, int32_t T, float* logprobs_out) {
    LUMI_TRY(check_batch(s, batch));
    if (!tokens || !logprobs_out || T < 2) return fail(LUMI_E_INVALID, "score needs tokens, an output buffer and T >= 2");
    LUMI_CUDA(cudaSetDevice(s->m->device));
    s->fused_head = false;
    LUMI_TRY(upload_prompt(s, tokens, batch, T));
    LUMI_TRY(grow(s->gen_dump, s->gen_dump_cap, (size_t)batch * (T - 1)));
    fill_ctl(s, batch, nullptr);
    s->ctl_host->prompt = s->prompt_dev;
    s->ctl_host->prompt_len = T;
    s->ctl_host->ignore_eos = 1;
    const bool chunked = use_chunked_prefill(s, batch, T);
    if (chunked) s->ctl_host->prompt_pos = T;          // the batched path consumes the whole prompt itself
    LUMI_TRY(push_ctl(s));
    if (chunked) {
        LUMI_TRY(prefill_chunked(s, batch, T, false, s->gen_dump));
        LUMI_CUDA(cudaMemcpyAsync(logprobs_out, s->gen_dump, sizeof(float) * (size_t)batch * (T - 1), cudaMemcpyDeviceToHost, s->stream));
        LUMI_TRY(pull_ctl(s));
        LUMI_CUDA(cudaStreamSynchronize(s->stream));
        return check_status(s);
    }
    const bool mega = s->opt_mega;
    s->opt_mega = 0;                                    // the persistent kernel has no per-position head
    int32_t rc = LUMI_OK;
    for (int t = 0; t < T && rc == LUMI_OK; ++t) {
        rc = run_step(s, batch, t < T - 1);
        if (rc == LUMI_OK && t < T - 1) {
            cudaError_t e = launch_logprob(s->logits, batch, s->m->cfg.vocab, s->prompt_dev + (size_t)(t + 1) * batch, s->gen_dump, T - 1, t, s->stream);
            if (e != cudaSuccess) rc = fail(LUMI_E_CUDA, "logprob kernel: %s", cudaGetErrorString(e));
        }
    }
    s->opt_mega = mega;
    LUMI_TRY(rc);
    LUMI_CUDA(cudaMemcpyAsync(logprobs_out, s->gen_dump, sizeof(float) * (size_t)batch * (T - 1), cudaMemcpyDeviceToHost, s->stream));
    LUMI_TRY(pull_ctl(s));
    LUMI_CUDA(cudaStreamSynchronize(s->stream));
    return check_status(s);
}

extern "C" int32_t lumi_decode_step(lumi_session* s, const uint32_t* in_tokens, int32_t batch, const lumi_sampling* sp,
                                    int32_t step, uint32_t* out_tokens, float* logits_out) {
    LUMI_TRY(check_batch(s, batch));
    if (!in_tokens) return fail(LUMI_E_INVALID, "in_tokens is null");
    LUMI_CUDA(cudaSetDevice(s->m->device));
    s->fused_head = (!sp || sp->temperature <= 0.f) && logits_out == nullptr;
    fill_ctl(s, batch, sp);
    s->ctl_host->step = step;
    LUMI_TRY(push_ctl(s));
    memcpy(s->pin_tokens, in_tokens, sizeof(uint32_t) * batch);
    LUMI_CUDA(cudaMemcpyAsync(s->tok_cur, s->pin_tokens, sizeof(uint32_t) * batch, cudaMemcpyHostToDevice, s->stream));
    if (use_b1(s, batch)) {
        const bool greedy = !sp || sp->temperature <= 0.f;
        LUMI_TRY(run_b1(s, 1, 1, greedy ? 1 : 0));
        if (!greedy) LUMI_TRY(sample_after_b1(s));
    } else {
        LUMI_TRY(run_step(s, batch, true));
    }
    LUMI_CUDA(cudaMemcpyAsync(s->pin_tokens, s->tok_cur, sizeof(uint32_t) * batch, cudaMemcpyDeviceToHost, s->stream));
    if (logits_out)
        LUMI_CUDA(cudaMemcpyAsync(logits_out, s->logits, sizeof(float) * batch * s->m->cfg.vocab, cudaMemcpyDeviceToHost, s->stream));
    LUMI_TRY(pull_ctl(s));
    LUMI_CUDA(cudaStreamSynchronize(s->stream));
    if (out_tokens) memcpy(out_tokens, s->pin_tokens, sizeof(uint32_t) * batch);
    return check_status(s);
}

extern "C" int32_t lumi_generate(lumi_session* s, const uint32_t* prompts, int32_t batch, int32_t T, int32_t n_new,
                                 const lumi_sampling* sp, uint32_t* out_tokens, int32_t* out_lens, float* logits_dump,
                                 lumi_stats* stats) {
    LUMI_TRY(check_batch(s, batch));
    if (!prompts || T <= 0 || n_new < 0 || !sp) return fail(LUMI_E_INVALID, "generate needs prompts, T > 0, n_new >= 0 and sampling parameters");
    LUMI_CUDA(cudaSetDevice(s->m->device));
    const int V = s->m->cfg.vocab;
    s->fused_head = sp->temperature <= 0.f && logits_dump == nullptr;
    LUMI_TRY(upload_prompt(s, prompts, batch, T));
    LUMI_TRY(grow(s->gen_out, s->gen_out_cap, (size_t)std::max(1, n_new) * batch));
    if (logits_dump) LUMI_TRY(grow(s->gen_dump, s->gen_dump_cap, (size_t)std::max(1, n_new) * batch * V));
    fill_ctl(s, batch, sp);
    StepCtl& c = *s->ctl_host;
    c.prompt = s->prompt_dev;
    c.prompt_len = T;
    c.record = 1;
    c.want_dump = logits_dump ? 1 : 0;
    c.out_tokens = s->gen_out;
    c.dump = s->gen_dump;
    const bool chunked = !use_b1(s, batch) && use_chunked_prefill(s, batch, T);
    if (chunked) c.prompt_pos = T;
    LUMI_TRY(push_ctl(s));
    LUMI_CUDA(cudaMemsetAsync(s->finished, 0, sizeof(int32_t) * batch, s->stream));
    LUMI_CUDA(cudaMemsetAsync(s->out_len, 0, sizeof(int32_t) * batch, s->stream));
    const int64_t l0 = s->launches;
    LUMI_CUDA(cudaEventRecord(s->ev0, s->stream));
    // main.rs:121-125: the prompt goes through forward_step token by token; the last position's
    // logits give generated token 0
    const bool b1 = use_b1(s, batch);
    const bool greedy = sp->temperature <= 0.f;
    if (b1) {
        LUMI_TRY(run_b1(s, T, n_new > 0 ? 1 : 0, greedy ? 1 : 0));
        if (n_new > 0 && !greedy) LUMI_TRY(sample_after_b1(s));
    } else if (chunked) {
        LUMI_TRY(prefill_chunked(s, batch, T, n_new > 0));
    } else {
        LUMI_TRY(run_steps(s, batch, false, T - 1));
        LUMI_TRY(run_step(s, batch, n_new > 0));
    }
    LUMI_CUDA(cudaEventRecord(s->ev1, s->stream));
    if (b1 && greedy) {
        LUMI_TRY(run_b1(s, n_new - 1, 1, 1));                                // main.rs:136-170, all tokens in one launch
    } else if (b1) {
        for (int i = 1; i < n_new; ++i) { LUMI_TRY(run_b1(s, 1, 1, 0)); LUMI_TRY(sample_after_b1(s)); }
    } else {
        LUMI_TRY(run_steps(s, batch, true, n_new - 1));                          // main.rs:136-170
    }
    LUMI_CUDA(cudaEventRecord(s->ev2, s->stream));
    std::vector<uint32_t> tmp((size_t)n_new * batch);
    if (n_new > 0) LUMI_CUDA(cudaMemcpyAsync(tmp.data(), s->gen_out, tmp.size() * sizeof(uint32_t), cudaMemcpyDeviceToHost, s->stream));
    if (logits_dump && n_new > 0)
        LUMI_CUDA(cudaMemcpyAsync(logits_dump, s->gen_dump, sizeof(float) * (size_t)n_new * batch * V, cudaMemcpyDeviceToHost, s->stream));
    if (out_lens) LUMI_CUDA(cudaMemcpyAsync(out_lens, s->out_len, sizeof(int32_t) * batch, cudaMemcpyDeviceToHost, s->stream));
    LUMI_TRY(pull_ctl(s));
    LUMI_CUDA(cudaStreamSynchronize(s->stream));
    if (out_tokens)
        for (int i = 0; i < n_new; ++i)
            for (int b = 0; b < batch; ++b) out_tokens[(size_t)b * n_new + i] = tmp[(size_t)i * batch + b];
    if (stats) {
        memset(stats, 0, sizeof(*stats));
        stats->prompt_tokens = (int64_t)batch * T;
        stats->decode_tokens = (int64_t)batch * std::max(0, n_new - 1);
        LUMI_CUDA(cudaEventElapsedTime(&stats->ms_prefill, s->ev0, s->ev1));
        LUMI_CUDA(cudaEventElapsedTime(&stats->ms_decode, s->ev1, s->ev2));
        stats->kernel_launches = s->launches - l0;
        const Config& cf = s->m->cfg;
        const int64_t per_seq = (int64_t)s->m->n_mamba * 2 * 4 *
                                ((int64_t)state_h_per_seq(cf) + cf.d_inner() + cf.n_heads * cf.d_state + cf.n_heads * (cf.d_state / 2));
        stats->bytes_per_step = s->m->weight_bytes + (int64_t)batch * per_seq;
        const int64_t steps = std::max(0, n_new - 1);
        stats->achieved_gbps = (steps > 0 && stats->ms_decode > 0.f) ? (float)((double)stats->bytes_per_step * (double)steps / ((double)stats->ms_decode * 1e-3) / 1e9) : 0.f;
        stats->waves = 1;
    }
    return check_status(s);
}

extern "C" int32_t lumi_decode_loop_device(lumi_session* s, int32_t batch, int32_t n_steps, float* ms_out, int64_t* launches_out) {
    LUMI_TRY(check_batch(s, batch));
    if (n_steps <= 0) return fail(LUMI_E_INVALID, "n_steps must be > 0");
    LUMI_CUDA(cudaSetDevice(s->m->device));
    lumi_sampling sp{};
    sp.ignore_eos = 1;
    s->fused_head = true;
    fill_ctl(s, batch, &sp);
    LUMI_TRY(push_ctl(s));
    const int64_t l0 = s->launches;
    LUMI_CUDA(cudaEventRecord(s->ev0, s->stream));
    if (use_b1(s, batch)) LUMI_TRY(run_b1(s, n_steps, 1, 1));
    else
        LUMI_TRY(run_steps(s, batch, true, n_steps));
    LUMI_CUDA(cudaEventRecord(s->ev1, s->stream));
    LUMI_TRY(pull_ctl(s));
    LUMI_CUDA(cudaStreamSynchronize(s->stream));
    float ms = 0.f;
    LUMI_CUDA(cudaEventElapsedTime(&ms, s->ev0, s->ev1));
    if (ms_out) *ms_out = ms;
    if (launches_out) *launches_out = s->launches - l0;
    return check_status(s);
}

extern "C" int32_t lumi_profile_step(lumi_session* s, int32_t batch, float* ms_by_family, int64_t* launches_by_family) {
    LUMI_TRY(check_batch(s, batch));
    if (!ms_by_family || !launches_by_family) return fail(LUMI_E_INVALID, "null output to lumi_profile_step");
    LUMI_CUDA(cudaSetDevice(s->m->device));
    lumi_sampling sp{};
    sp.ignore_eos = 1;
    fill_ctl(s, batch, &sp);
    LUMI_TRY(push_ctl(s));
    std::vector<std::pair<int, cudaEvent_t>> ev;
    int64_t n = 0;
    int32_t st = enqueue_step(s, batch, true, &n, &ev);
    cudaError_t e = cudaStreamSynchronize(s->stream);
    for (int f = 0; f < 8; ++f) { ms_by_family[f] = 0.f; launches_by_family[f] = 0; }
    if (st == LUMI_OK && e == cudaSuccess) {
        for (size_t i = 0; i + 1 < ev.size(); ++i) {
            float ms = 0.f;
            cudaEventElapsedTime(&ms, ev[i].second, ev[i + 1].second);
            if (ev[i].first < 8) { ms_by_family[ev[i].first] += ms; launches_by_family[ev[i].first] += 1; }
        }
    }
    for (auto& pe : ev) cudaEventDestroy(pe.second);
    if (st != LUMI_OK) return st;
    LUMI_CUDA(e);
    s->launches += n;
    LUMI_TRY(pull_ctl(s));
    LUMI_CUDA(cudaStreamSynchronize(s->stream));
    return check_status(s);
}

extern "C" int32_t lumi_session_read_state(lumi_session* s, int32_t slot, int32_t layer, float* h, float* x_prev, float* b_prev,
                                           float* cum_angle) {
    if (!s) return fail(LUMI_E_INVALID, "session is null");
    const Config& c = s->m->cfg;
    if (slot < 0 || slot >= s->max_batch) return fail(LUMI_E_INVALID, "slot %d out of range", slot);
    if (layer < 0 || layer >= c.n_layers || s->m->layers[layer].is_attn) return fail(LUMI_E_INVALID, "layer %d is not a Mamba layer", layer);
    LUMI_CUDA(cudaSetDevice(s->m->device));
    const size_t B = s->max_batch, l = s->m->layers[layer].kind_idx;
    const size_t nh = state_h_per_seq(c), nx = c.d_inner(), nb = (size_t)c.n_heads * c.d_state, nc = (size_t)c.n_heads * (c.d_state / 2);
    LUMI_CUDA(cudaStreamSynchronize(s->stream));
    if (h) LUMI_CUDA(cudaMemcpy(h, s->h + (l * B + slot) * nh, nh * 4, cudaMemcpyDeviceToHost));
    if (x_prev) LUMI_CUDA(cudaMemcpy(x_prev, s->xprev + (l * B + slot) * nx, nx * 4, cudaMemcpyDeviceToHost));
    if (b_prev) LUMI_CUDA(cudaMemcpy(b_prev, s->bprev + (l * B + slot) * nb, nb * 4, cudaMemcpyDeviceToHost));
    if (cum_angle) LUMI_CUDA(cudaMemcpy(cum_angle, s->cum + (l * B + slot) * nc, nc * 4, cudaMemcpyDeviceToHost));
    return LUMI_OK;
}

// ---- sequence snapshots ---------------------------------------------------------------------------
namespace {
struct SnapHeader {
    uint32_t magic, version, n_mamba, n_attn;
    uint64_t payload_bytes;
    int32_t kv_pos;
    uint32_t reserved;
};
constexpr uint32_t kSnapMagic = 0x4c4d5353u;     // "LMSS"

struct SnapLayout {
    size_t nh, nx, nb, nc;      // floats per sequence per Mamba layer: h, x_prev, B_prev, angles
    size_t kv_seq_bytes;        // bytes per sequence per attention layer (its pages_per_seq pages)
    size_t payload;
};
SnapLayout snap_layout(const lumi_session* s) {
    const Config& c = s->m->cfg;
    SnapLayout L{};
    L.nh = state_h_per_seq(c); L.nx = c.d_inner(); L.nb = (size_t)c.n_heads * c.d_state; L.nc = (size_t)c.n_heads * (c.d_state / 2);
    L.kv_seq_bytes = s->m->n_attn > 0 ? s->kv_layer_bytes / (size_t)s->max_batch : 0;
    L.payload = (size_t)s->m->n_mamba * (L.nh + L.nx + L.nb + L.nc) * sizeof(float) + (size_t)s->m->n_attn * L.kv_seq_bytes;
    return L;
}
}  // namespace

extern "C" int32_t lumi_session_state_bytes(const lumi_session* s, int64_t* bytes) {
    if (!s || !bytes) return fail(LUMI_E_INVALID, "null argument");
    *bytes = (int64_t)(sizeof(SnapHeader) + snap_layout(s).payload);
    return LUMI_OK;
}

static int32_t snap_copy(lumi_session* s, int32_t slot, char* buf, bool save) {
    const SnapLayout L = snap_layout(s);
    const size_t B = s->max_batch;
    const cudaMemcpyKind kind = save ? cudaMemcpyDeviceToHost : cudaMemcpyHostToDevice;
    auto xfer = [&](void* dev, size_t bytes) -> cudaError_t {
        cudaError_t e = save ? cudaMemcpyAsync(buf, dev, bytes, kind, s->stream) : cudaMemcpyAsync(dev, buf, bytes, kind, s->stream);
        buf += bytes;
        return e;
    };
    for (size_t l = 0; l < (size_t)s->m->n_mamba; ++l) {
        LUMI_CUDA(xfer(s->h + (l * B + slot) * L.nh, L.nh * sizeof(float)));
        LUMI_CUDA(xfer(s->xprev + (l * B + slot) * L.nx, L.nx * sizeof(float)));
        LUMI_CUDA(xfer(s->bprev + (l * B + slot) * L.nb, L.nb * sizeof(float)));
        LUMI_CUDA(xfer(s->cum + (l * B + slot) * L.nc, L.nc * sizeof(float)));
    }
    for (size_t a = 0; a < (size_t)s->m->n_attn; ++a)      // slot b owns pages [b * pages_per_seq, (b + 1) * pages_per_seq)
        LUMI_CUDA(xfer((char*)s->kv_pool + a * s->kv_layer_bytes + (size_t)slot * L.kv_seq_bytes, L.kv_seq_bytes));
    return LUMI_OK;
}

extern "C" int32_t lumi_session_save_state(lumi_session* s, int32_t slot, void* host_buf, int64_t nbytes) {
    if (!s || !host_buf) return fail(LUMI_E_INVALID, "null argument");
    if (slot < 0 || slot >= s->max_batch) return fail(LUMI_E_INVALID, "slot %d out of range", slot);
    const SnapLayout L = snap_layout(s);
    if (nbytes < (int64_t)(sizeof(SnapHeader) + L.payload))
        return fail(LUMI_E_INVALID, "snapshot buffer of %lld bytes, %zu needed", (long long)nbytes, sizeof(SnapHeader) + L.payload);
    LUMI_CUDA(cudaSetDevice(s->m->device));
    SnapHeader hd{kSnapMagic, 1u, (uint32_t)s->m->n_mamba, (uint32_t)s->m->n_attn, (uint64_t)L.payload, 0, 0u};
    LUMI_CUDA(cudaMemcpyAsync(&hd.kv_pos, s->kv_pos + slot, sizeof(int32_t), cudaMemcpyDeviceToHost, s->stream));
    LUMI_TRY(snap_copy(s, slot, (char*)host_buf + sizeof(SnapHeader), true));
    LUMI_CUDA(cudaStreamSynchronize(s->stream));
    memcpy(host_buf, &hd, sizeof(hd));
    return LUMI_OK;
}

extern "C" int32_t lumi_session_load_state(lumi_session* s, int32_t slot, const void* host_buf, int64_t nbytes) {
    if (!s || !host_buf) return fail(LUMI_E_INVALID, "null argument");
    if (slot < 0 || slot >= s->max_batch) return fail(LUMI_E_INVALID, "slot %d out of range", slot);
    const SnapLayout L = snap_layout(s);
    SnapHeader hd;
    if (nbytes < (int64_t)sizeof(hd)) return fail(LUMI_E_INVALID, "snapshot shorter than its header");
    memcpy(&hd, host_buf, sizeof(hd));
    if (hd.magic != kSnapMagic || hd.version != 1u) return fail(LUMI_E_INVALID, "not a sequence snapshot");
    if (hd.n_mamba != (uint32_t)s->m->n_mamba || hd.n_attn != (uint32_t)s->m->n_attn || hd.payload_bytes != (uint64_t)L.payload)
        return fail(LUMI_E_TENSOR, "snapshot of another model or cache size (%u Mamba + %u attention layers, %llu bytes; this session: %d + %d, %zu)",
                    hd.n_mamba, hd.n_attn, (unsigned long long)hd.payload_bytes, s->m->n_mamba, s->m->n_attn, L.payload);
    if (nbytes < (int64_t)(sizeof(hd) + L.payload)) return fail(LUMI_E_INVALID, "snapshot truncated");
    // the position indexes the page table and the cache: a value outside what this session can hold is refused here
    // (with a sliding window on every attention layer positions may run past the capacity: the ring wraps)
    if (hd.kv_pos < 0) return fail(LUMI_E_INVALID, "snapshot with a negative position (%d)", hd.kv_pos);
    if (s->m->n_attn > 0) {
        bool all_windowed = true;
        for (const Layer& Ly : s->m->layers) if (Ly.is_attn && !(Ly.window > 0 && Ly.window <= s->max_tokens_kv)) all_windowed = false;
        if (!all_windowed && hd.kv_pos > s->max_tokens_kv)
            return fail(LUMI_E_INVALID, "snapshot at position %d, this session's cache holds %d tokens", hd.kv_pos, s->max_tokens_kv);
    }
    LUMI_CUDA(cudaSetDevice(s->m->device));
    LUMI_CUDA(cudaMemcpyAsync(s->kv_pos + slot, &hd.kv_pos, sizeof(int32_t), cudaMemcpyHostToDevice, s->stream));
    LUMI_TRY(snap_copy(s, slot, (char*)const_cast<void*>(host_buf) + sizeof(SnapHeader), false));
    LUMI_CUDA(cudaStreamSynchronize(s->stream));
    return LUMI_OK;
}

extern "C" int32_t lumi_debug_run_block(lumi_session* s, int32_t layer, float* x, int32_t batch) {
    LUMI_TRY(check_batch(s, batch));
    const Config& c = s->m->cfg;
    if (!x || layer < 0 || layer >= c.n_layers) return fail(LUMI_E_INVALID, "bad layer or null x");
    LUMI_CUDA(cudaSetDevice(s->m->device));
    fill_ctl(s, batch, nullptr);
    LUMI_TRY(push_ctl(s));
    LUMI_CUDA(cudaMemcpyAsync(s->x, x, sizeof(float) * batch * c.d_model, cudaMemcpyHostToDevice, s->stream));
    StepPlan p{s, batch, use_tc(s, batch)};
    p.st_hi = p.st_lo = s->stream;
    const Layer& L = s->m->layers[layer];
    if (L.is_attn) {
        LUMI_TRY(attention_block(p, L));
        LUMI_CUDA(launch_advance_step(s->ctl, s->kv_pos, batch, 0, s->stream));
    } else {
        LUMI_TRY(mamba_block(p, L));
    }
    LUMI_CUDA(cudaMemcpyAsync(x, s->x, sizeof(float) * batch * c.d_model, cudaMemcpyDeviceToHost, s->stream));
    LUMI_TRY(pull_ctl(s));
    LUMI_CUDA(cudaStreamSynchronize(s->stream));
    return check_status(s);
}

// ---- single kernels over caller-owned device pointers ---------------------------------------------------
extern "C" int32_t lumi_k_gemm_bf16_tcgen05(uint64_t a_hi, uint64_t a_lo, uint64_t w, uint64_t d, int32_t M, int32_t N, int32_t K,
                                            int32_t ldd, int32_t accumulate, uint64_t stream) {
    if (!a_hi || !w || !d) return fail(LUMI_E_INVALID, "null device pointer");
    // split-K needs zeroed counters: one small buffer per device for this test entry, made on first use
    static std::mutex mu;
    static int32_t* counters[64] = {nullptr};
    static float* scratch[64] = {nullptr};
    int dev = 0;
    LUMI_CUDA(cudaGetDevice(&dev));
    int32_t* cnt = nullptr;
    if (dev >= 0 && dev < 64) {
        std::lock_guard<std::mutex> lock(mu);
        if (counters[dev] == nullptr) {
            LUMI_CUDA(cudaMalloc(&counters[dev], sizeof(int32_t) * kGemmCounters));
            LUMI_CUDA(cudaMemset(counters[dev], 0, sizeof(int32_t) * kGemmCounters));
            LUMI_CUDA(cudaMalloc(&scratch[dev], sizeof(float) * kGemmScratchFloats));
        }
        cnt = counters[dev];
    }
    GemmArgs g{(const __nv_bfloat16*)a_hi, (const __nv_bfloat16*)a_lo, (const __nv_bfloat16*)w, (float*)d, ldd, M, N, K, accumulate, nullptr,
               cnt, cnt ? kGemmCounters : 0, cnt ? scratch[dev] : nullptr, cnt ? kGemmScratchFloats : 0};
    return launch_gemm_tcgen05(g, (cudaStream_t)stream);
}

// Failure-path test hook: the persistent tcgen05 GEMM with a caller-chosen wait limit and a work unit whose operands
// the producer never requests.  The consumers' bounded waits run out, the kernel records STATUS_TIMEOUT in
// *status_word (device int32, zeroed by the caller), drains what it issued, frees its TMEM and returns; the call
// then answers LUMI_E_TIMEOUT.  Nothing faults and the context stays usable.
// Host-side only: which tile width and K split the tensor-core GEMM takes for a shape (two_planes: activations as bf16
// hi + lo; producer: the epilogue also leaves the next norm's input, which restricts the widths to multiples of 32).
extern "C" int32_t lumi_debug_gemm_plan(int32_t M, int32_t N, int32_t K, int32_t two_planes, int32_t producer, int32_t* width,
                                        int32_t* splits) {
    if (M <= 0 || N <= 0 || K <= 0 || (K % 64) != 0 || !width || !splits) return fail(LUMI_E_INVALID, "gemm plan needs M, N > 0, K %% 64 == 0 and two outputs");
    static int32_t dummy_counter = 0;
    static float dummy_f = 0.f;
    static __nv_bfloat16 dummy_h;
    GemmArgs g{};
    g.M = M; g.N = N; g.K = K;
    g.a_hi = &dummy_h; g.a_lo = two_planes ? &dummy_h : nullptr;
    g.tile_counters = &dummy_counter; g.n_counters = kGemmCounters;          // never dereferenced by the choice
    g.scratch = &dummy_f; g.scratch_floats = kGemmScratchFloats;
    if (producer) g.nf.out_hi = &dummy_h;
    int w = 0, sp = 0;
    gemm_tcgen05_plan(g, &w, &sp);
    *width = w; *splits = sp;
    return LUMI_OK;
}

extern "C" int32_t lumi_debug_gemm_wait_timeout(uint64_t a_hi, uint64_t w, uint64_t d, int32_t M, int32_t N, int32_t K, uint64_t wait_limit_ns,
                                                int32_t skip_unit, uint64_t status_word) {
    if (!a_hi || !w || !d || !status_word) return fail(LUMI_E_INVALID, "null device pointer");
    GemmArgs g{(const __nv_bfloat16*)a_hi, nullptr, (const __nv_bfloat16*)w, (float*)d, N, M, N, K, 0, (int32_t*)status_word};
    g.wait_limit_ns = wait_limit_ns;
    g.debug_skip_unit = skip_unit;
    LUMI_TRY(launch_gemm_tcgen05(g, nullptr));
    LUMI_CUDA(cudaStreamSynchronize(nullptr));
    int32_t st = 0;
    LUMI_CUDA(cudaMemcpy(&st, (const void*)status_word, sizeof(st), cudaMemcpyDeviceToHost));
    if (st & STATUS_TIMEOUT) return fail(LUMI_E_TIMEOUT, "a bounded device-side wait expired in the tensor-core GEMM (limit %llu ns)", (unsigned long long)wait_limit_ns);
    return LUMI_OK;
}

extern "C" int32_t lumi_k_gemv(uint64_t a_f32, uint64_t w, int32_t w_dtype, uint64_t d, uint64_t residual, uint64_t norm_gamma,
                               int32_t M, int32_t N, int32_t K, uint64_t stream) {
    if (!a_f32 || !w || !d || M <= 0 || N <= 0 || K <= 0) return fail(LUMI_E_INVALID, "bad argument to lumi_k_gemv");
    if (K % 8) return fail(LUMI_E_UNSUPPORTED, "K must be a multiple of 8");
    GemvArgs g{(const float*)a_f32, K, (const void*)w, w_dtype, (float*)d, N, (const float*)residual, (const float*)norm_gamma, M, N, K, 1e-5f, 0};
    LUMI_CUDA(launch_gemv(g, (cudaStream_t)stream));
    return LUMI_OK;
}

extern "C" int32_t lumi_k_ssm_step(uint64_t proj, int32_t ldp, uint64_t b_gamma, uint64_t c_gamma, uint64_t b_bias, uint64_t c_bias,
                                   uint64_t d_skip, uint64_t dt_bias, uint64_t h, uint64_t x_prev, uint64_t b_prev, uint64_t cum_angle,
                                   uint64_t y, int32_t B, int32_t H, int32_t P, int32_t N, int32_t G, uint64_t stream) {
    if (!proj || !b_gamma || !c_gamma || !b_bias || !c_bias || !d_skip || !dt_bias || !h || !x_prev || !b_prev || !cum_angle || !y)
        return fail(LUMI_E_INVALID, "null device pointer to lumi_k_ssm_step");
    if (B <= 0 || H <= 0 || G <= 0 || (H % G) || !ssm_shape_supported(P, N)) return fail(LUMI_E_UNSUPPORTED, "unsupported shape for lumi_k_ssm_step");
    SsmArgs a{};
    a.proj = (const float*)proj; a.ldp = ldp;
    a.bg = (const float*)b_gamma; a.cg = (const float*)c_gamma; a.bb = (const float*)b_bias; a.cb = (const float*)c_bias;
    a.dskip = (const float*)d_skip; a.dtb = (const float*)dt_bias;
    a.h = (float*)h; a.xprev = (float*)x_prev; a.bprev = (float*)b_prev; a.cum = (float*)cum_angle;
    a.y32 = (float*)y;
    a.B = B; a.H = H; a.P = P; a.N = N; a.G = G; a.eps = 1e-5f;
    LUMI_CUDA(launch_ssm_step(a, (cudaStream_t)stream));
    return LUMI_OK;
}

extern "C" int32_t lumi_k_ssd_prefill(uint64_t proj, int32_t ldp, uint64_t b_gamma, uint64_t c_gamma, uint64_t b_bias, uint64_t c_bias,
                                      uint64_t d_skip, uint64_t dt_bias, uint64_t h, uint64_t x_prev, uint64_t b_prev, uint64_t cum_angle,
                                      uint64_t y_hi, uint64_t y_lo, uint64_t scratch, int32_t nb, int32_t ts, int32_t H, int32_t G,
                                      uint64_t stream) {
    if (!proj || !b_gamma || !c_gamma || !b_bias || !c_bias || !d_skip || !dt_bias || !h || !x_prev || !b_prev || !cum_angle || !y_hi || !scratch)
        return fail(LUMI_E_INVALID, "null device pointer to lumi_k_ssd_prefill");
    if (nb <= 0 || ts <= 0 || H <= 0 || G <= 0 || (H % G) || (H % 4) || (ldp % 4) || ldp < 2 * H * 32 + 2 * G * 64 + 3 * H + H * 32)
        return fail(LUMI_E_UNSUPPORTED, "unsupported shape for lumi_k_ssd_prefill (head_dim 32, d_state 64, n_heads %% 4 == 0)");
    PrefillArgs a{};
    a.proj = (const float*)proj; a.ldp = ldp;
    a.bg = (const float*)b_gamma; a.cg = (const float*)c_gamma; a.bb = (const float*)b_bias; a.cb = (const float*)c_bias;
    a.dskip = (const float*)d_skip; a.dtb = (const float*)dt_bias;
    a.h = (float*)h; a.xprev = (float*)x_prev; a.bprev = (float*)b_prev; a.cum = (float*)cum_angle;
    a.rb = (float*)scratch; a.rc = (float*)scratch + (size_t)nb * ts;
    a.yhi = (__nv_bfloat16*)y_hi; a.ylo = (__nv_bfloat16*)y_lo;
    a.H = H; a.G = G; a.ts = ts; a.nb = nb; a.b0 = 0; a.eps = 1e-5f;
    LUMI_CUDA(launch_prefill_scan(a, (cudaStream_t)stream));
    return LUMI_OK;
}
