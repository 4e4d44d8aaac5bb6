//! `extern "C"` declarations for include/lumi_b200.h (token-loop subset).
use std::os::raw::{c_char, c_void};

#[repr(C)]
pub struct LumiSampling {
    pub temperature: f32,
    pub top_k: i32,
    pub seed: u64,
    pub eos_id: u32,
    pub ignore_eos: i32,
}

#[repr(C)]
#[derive(Default)]
pub struct LumiStats {
    pub prompt_tokens: i64,
    pub decode_tokens: i64,
    pub ms_prefill: f32,
    pub ms_decode: f32,
    pub bytes_per_step: i64,
    pub kernel_launches: i64,
    pub achieved_gbps: f32,
    pub waves: i32,
}

pub enum LumiModel {}
pub enum LumiSession {}

extern "C" {
    pub fn lumi_last_error() -> *const c_char;
    pub fn lumi_model_create(config_json: *const c_char, device_id: i32, out: *mut *mut LumiModel) -> i32;
    pub fn lumi_model_load_tensor(m: *mut LumiModel, name: *const c_char, dtype: i32, shape: *const i64, rank: i32,
                                  host_data: *const c_void, nbytes: u64) -> i32;
    pub fn lumi_model_load_safetensors(m: *mut LumiModel, path: *const c_char) -> i32;
    pub fn lumi_model_finalize(m: *mut LumiModel) -> i32;
    pub fn lumi_model_free(m: *mut LumiModel);
    pub fn lumi_model_info(m: *const LumiModel, out12: *mut i64) -> i32;
    pub fn lumi_session_create(m: *mut LumiModel, max_batch: i32, max_tokens_kv: i32, out: *mut *mut LumiSession) -> i32;
    pub fn lumi_session_reset(s: *mut LumiSession, slots: *const i32, n_slots: i32) -> i32;
    pub fn lumi_session_free(s: *mut LumiSession);
    pub fn lumi_session_state_bytes(s: *const LumiSession, bytes: *mut i64) -> i32;
    pub fn lumi_session_save_state(s: *mut LumiSession, slot: i32, host_buf: *mut c_void, nbytes: i64) -> i32;
    pub fn lumi_session_load_state(s: *mut LumiSession, slot: i32, host_buf: *const c_void, nbytes: i64) -> i32;
    pub fn lumi_score(s: *mut LumiSession, tokens: *const u32, batch: i32, t: i32, logprobs_out: *mut f32) -> i32;
    pub fn lumi_prefill(s: *mut LumiSession, tokens: *const u32, batch: i32, t: i32, last_logits: *mut f32) -> i32;
    pub fn lumi_decode_step(s: *mut LumiSession, in_tokens: *const u32, batch: i32, sp: *const LumiSampling, step: i32,
                            out_tokens: *mut u32, logits_out: *mut f32) -> i32;
    pub fn lumi_generate(s: *mut LumiSession, prompts: *const u32, batch: i32, t: i32, n_new: i32, sp: *const LumiSampling,
                         out_tokens: *mut u32, out_lens: *mut i32, logits_dump: *mut f32, stats: *mut LumiStats) -> i32;
}

pub fn check(status: i32) -> anyhow::Result<()> {
    if status == 0 {
        return Ok(());
    }
    let msg = unsafe { std::ffi::CStr::from_ptr(lumi_last_error()) }.to_string_lossy().into_owned();
    Err(anyhow::anyhow!("lumi_b200 error {status}: {msg}"))
}
