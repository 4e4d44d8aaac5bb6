// lumi-infer-b200 — the `generate` subcommand of lumi-infer (inference/src/main.rs:16-58, 96-177)
// over the C ABI.  Byte-level models encode the prompt as byte + 3 with eos = 2 (main.rs:100-103);
// BPE models need token ids (--prompt-ids), the tokenizer.json boundary lies outside this library.
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <sstream>
#include <string>
#include <vector>

#include "../../include/lumi_b200.h"

static int die(const char* what, int32_t st) {
    fprintf(stderr, "%s failed (%d): %s\n", what, st, lumi_last_error());
    return 1;
}

static void usage() {
    fprintf(stderr,
            "usage: lumi-infer-b200 generate -m <model.safetensors> -c <config.json> (-p <prompt> | --prompt-ids a,b,c)\n"
            "           [--max-tokens 200] [--temperature 0.8] [--top-k 0] [--seed 0] [--batch 1] [--ignore-eos] [--device 0]\n");
}

int main(int argc, char** argv) {
    if (argc < 2 || strcmp(argv[1], "generate") != 0) { usage(); return 2; }
    std::string model_path, config_path, prompt, ids_text;
    int max_tokens = 200, top_k = 0, batch = 1, device = 0, ignore_eos = 0;
    double temperature = 0.8;
    unsigned long long seed = 0;
    for (int i = 2; i < argc; ++i) {
        std::string a = argv[i];
        auto next = [&](const char* name) -> const char* {
            if (i + 1 >= argc) { fprintf(stderr, "%s needs a value\n", name); exit(2); }
            return argv[++i];
        };
        if (a == "-m" || a == "--model") model_path = next("--model");
        else if (a == "-c" || a == "--config") config_path = next("--config");
        else if (a == "-p" || a == "--prompt") prompt = next("--prompt");
        else if (a == "--prompt-ids") ids_text = next("--prompt-ids");
        else if (a == "--max-tokens") max_tokens = atoi(next("--max-tokens"));
        else if (a == "--temperature") temperature = atof(next("--temperature"));
        else if (a == "--top-k") top_k = atoi(next("--top-k"));
        else if (a == "--seed") seed = strtoull(next("--seed"), nullptr, 10);
        else if (a == "--batch") batch = atoi(next("--batch"));
        else if (a == "--device") device = atoi(next("--device"));
        else if (a == "--ignore-eos") ignore_eos = 1;
        else { usage(); return 2; }
    }
    if (model_path.empty() || config_path.empty() || (prompt.empty() && ids_text.empty()) || batch < 1) { usage(); return 2; }

    std::ifstream cf(config_path);
    if (!cf) { fprintf(stderr, "cannot read %s\n", config_path.c_str()); return 1; }
    std::stringstream ss;
    ss << cf.rdbuf();
    const std::string cfg = ss.str();
    fprintf(stderr, "Loading config: %s\n", config_path.c_str());
    lumi_model* model = nullptr;
    int32_t st = lumi_model_create(cfg.c_str(), device, &model);
    if (st) return die("lumi_model_create", st);
    fprintf(stderr, "Loading model: %s\n", model_path.c_str());
    if ((st = lumi_model_load_safetensors(model, model_path.c_str()))) return die("lumi_model_load_safetensors", st);
    if ((st = lumi_model_finalize(model))) return die("lumi_model_finalize", st);
    int64_t info[12];
    lumi_model_info(model, info);
    fprintf(stderr, "Model: d_model=%lld, layers=%lld (%lld Mamba + %lld Attention), heads=%lld, vocab=%lld\n", (long long)info[0],
            (long long)info[1], (long long)info[7], (long long)info[8], (long long)info[3], (long long)info[6]);
    const bool byte_level = info[6] == 259;

    std::vector<uint32_t> ids;
    if (!ids_text.empty()) {
        std::stringstream is(ids_text);
        std::string tok;
        while (std::getline(is, tok, ',')) ids.push_back((uint32_t)strtoul(tok.c_str(), nullptr, 10));
    } else if (byte_level) {
        for (unsigned char ch : prompt) ids.push_back((uint32_t)ch + 3);          // main.rs:102
    } else {
        fprintf(stderr, "this model is not byte-level: pass --prompt-ids (tokenizer.json is not handled here)\n");
        return 2;
    }
    if (ids.empty()) { fprintf(stderr, "empty prompt\n"); return 2; }
    fprintf(stderr, "Prompt: %zu tokens%s\n", ids.size(), byte_level ? " (byte-level)" : "");

    lumi_session* sess = nullptr;
    if ((st = lumi_session_create(model, batch, (int32_t)(ids.size() + max_tokens + 1), &sess))) return die("lumi_session_create", st);
    std::vector<uint32_t> prompts;
    for (int b = 0; b < batch; ++b) prompts.insert(prompts.end(), ids.begin(), ids.end());
    std::vector<uint32_t> out((size_t)batch * max_tokens);
    std::vector<int32_t> lens(batch);
    lumi_sampling sp{(float)temperature, top_k, seed, 2u, ignore_eos};
    lumi_stats stats{};
    if ((st = lumi_generate(sess, prompts.data(), batch, (int32_t)ids.size(), max_tokens, &sp, out.data(), lens.data(), nullptr, &stats)))
        return die("lumi_generate", st);
    fprintf(stderr, "Prompt processed in %.1fms (%.0f tok/s)\n", stats.ms_prefill, stats.prompt_tokens / (stats.ms_prefill * 1e-3));
    if (!prompt.empty()) fputs(prompt.c_str(), stdout);
    for (int i = 0; i < lens[0]; ++i) {
        const uint32_t t = out[i];
        if (byte_level) { if (t >= 3 && t < 131) fputc((int)(t - 3), stdout); }     // main.rs:154-160: single bytes that are valid UTF-8
        else printf(" %u", t);
    }
    printf("\n");
    long long produced = 0;
    for (int b = 0; b < batch; ++b) produced += lens[b];
    fprintf(stderr, "\nGenerated %lld tokens in %.1fms (%.1f tok/s)\n", produced, stats.ms_decode,
            stats.decode_tokens / (stats.ms_decode > 0 ? stats.ms_decode * 1e-3 : 1.0));
    lumi_session_free(sess);
    lumi_model_free(model);
    return 0;
}
