//! `lumi-infer-b200 generate` — the reference's generate command (inference/src/main.rs:96-177) with the
//! model behind the C ABI.  Streaming variant: one lumi_decode_step per token, printing each piece as the
//! reference does (main.rs:154-167).
mod ffi;

use clap::{Parser, Subcommand};
use ffi::*;
use std::ffi::CString;
use std::io::Write;

#[derive(Parser)]
#[command(name = "lumi-infer-b200", about = "Lumi inference on B200")]
struct Cli {
    #[command(subcommand)]
    command: Command,
}

#[derive(Subcommand)]
enum Command {
    Generate {
        #[arg(short, long)]
        model: String,
        #[arg(short, long)]
        config: String,
        #[arg(short, long)]
        tokenizer: Option<String>,
        #[arg(short, long)]
        prompt: String,
        #[arg(long, default_value = "200")]
        max_tokens: usize,
        #[arg(long, default_value = "0.8")]
        temperature: f64,
        #[arg(long, default_value = "0")]
        top_k: i32,
    },
}

fn main() -> anyhow::Result<()> {
    let Command::Generate { model, config, tokenizer, prompt, max_tokens, temperature, top_k } = Cli::parse().command;
    let cfg_text = std::fs::read_to_string(&config)?;
    let byte_level = cfg_text.contains("\"byte_level\": true") || cfg_text.contains("\"byte_level\":true");
    let (mut m, mut s) = (std::ptr::null_mut(), std::ptr::null_mut());
    unsafe {
        check(lumi_model_create(CString::new(cfg_text)?.as_ptr(), 0, &mut m))?;
        check(lumi_model_load_safetensors(m, CString::new(model)?.as_ptr()))?;
        check(lumi_model_finalize(m))?;
    }
    // prompt ids and eos exactly as main.rs:100-113
    let (ids, eos, tok): (Vec<u32>, u32, Option<tokenizers::Tokenizer>) = if byte_level {
        (prompt.as_bytes().iter().map(|&b| b as u32 + 3).collect(), 2, None)
    } else {
        let path = tokenizer.as_deref().unwrap_or("tokenizer.json");
        let t = tokenizers::Tokenizer::from_file(path).map_err(|e| anyhow::anyhow!("Failed to load tokenizer: {e}"))?;
        let enc = t.encode(prompt.as_str(), false).map_err(|e| anyhow::anyhow!("Failed to encode: {e}"))?;
        let eos = t.token_to_id("<eos>").unwrap_or(2);
        (enc.get_ids().to_vec(), eos, Some(t))
    };
    eprintln!("Prompt: {} tokens", ids.len());
    unsafe { check(lumi_session_create(m, 1, (ids.len() + max_tokens + 1) as i32, &mut s))? };
    let sp = LumiSampling { temperature: temperature as f32, top_k, seed: rand::random(), eos_id: eos, ignore_eos: 0 };
    let start = std::time::Instant::now();
    // the last prompt position's logits give token 0: prefill all but the last token, then step
    let (head, last) = ids.split_at(ids.len() - 1);
    if !head.is_empty() {
        unsafe { check(lumi_prefill(s, head.as_ptr(), 1, head.len() as i32, std::ptr::null_mut()))? };
    }
    let mut cur = last[0];
    eprintln!("Prompt processed in {:.1}ms", start.elapsed().as_millis());
    print!("{prompt}");
    let gen_start = std::time::Instant::now();
    let mut n = 0usize;
    for step in 0..max_tokens {
        let mut next = 0u32;
        unsafe { check(lumi_decode_step(s, &cur, 1, &sp, step as i32, &mut next, std::ptr::null_mut()))? };
        if next == eos {
            break; // main.rs:150
        }
        n += 1;
        if byte_level {
            if (3..131).contains(&next) {
                print!("{}", (next - 3) as u8 as char);
            }
        } else if let Some(t) = &tok {
            if let Ok(text) = t.decode(&[next], true) {
                print!("{text}");
            }
        }
        std::io::stdout().flush()?;
        cur = next;
    }
    println!();
    eprintln!("\nGenerated {} tokens in {:.1}ms ({:.1} tok/s)", n, gen_start.elapsed().as_millis(), n as f64 / gen_start.elapsed().as_secs_f64());
    unsafe {
        lumi_session_free(s);
        lumi_model_free(m);
    }
    Ok(())
}
