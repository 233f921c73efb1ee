// vlrf_b200_cli: the command line over the C interface, with the commands and option names of the reference's
// tools/vlrf_cli.cpp (:93-121, usage :123-170).  It includes vlrf_b200.h and nothing else of the library.
//
//   vlrf_b200_cli run  --model DIR (--prompt "text" | --prompt-ids 1,2,3 | --prompts-file F) [--tokens N] [--ctx N]
//                      [--temp F] [--top-k N] [--top-p F] [--seed N] [--greedy] [--repeat-penalty F] [--freq-penalty F]
//                      [--presence-penalty F] [--no-repeat-ngram N] [--stop-id N]... [--dtype bfloat16|float32]
//   vlrf_b200_cli info --model DIR
//   vlrf_b200_cli init --config PRESET|config.json --out DIR [--seed N]
//
// Without a tokenizer, --prompt "text" is encoded as the reference does without one (byte + 4, capped at the
// vocabulary: src/api/vlrf_api.cpp:373-381) and token ids are printed.  A prompts file holds one id list a line.
#include "vlrf_b200.h"

#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <sstream>
#include <string>
#include <vector>

namespace {

struct Args {
    std::string command, model, prompt, prompt_ids, prompts_file, config, out, dtype = "bfloat16";
    bool has_prompt = false;
    int tokens = 128, ctx = 0, top_k = 50, no_repeat_ngram = 0;
    float temp = 0.8f, top_p = 0.9f, repeat_penalty = 1.0f, freq_penalty = 0.0f, presence_penalty = 0.0f;
    unsigned seed = 42, init_seed = 1234;
    bool greedy = false, seed_given = false;
    std::vector<int> stop_ids;
};

int usage(const char* why) {
    if (why) fprintf(stderr, "vlrf_b200_cli: %s\n", why);
    fprintf(stderr,
            "usage: vlrf_b200_cli run  --model DIR (--prompt TEXT | --prompt-ids 1,2,3 | --prompts-file F) [--tokens N] [--ctx N]\n"
            "                          [--temp F] [--top-k N] [--top-p F] [--seed N] [--greedy] [--repeat-penalty F] [--freq-penalty F]\n"
            "                          [--presence-penalty F] [--no-repeat-ngram N] [--stop-id N]... [--dtype bfloat16|float32]\n"
            "       vlrf_b200_cli info --model DIR\n"
            "       vlrf_b200_cli init --config PRESET|config.json --out DIR [--seed N]\n");
    return 2;
}

std::vector<int32_t> parse_ids(const std::string& text) {
    std::vector<int32_t> ids;
    std::string token;
    std::istringstream in(text);
    char c;
    while (in.get(c)) {
        if (c == ',' || c == ' ' || c == '\t') {
            if (!token.empty()) { ids.push_back(atoi(token.c_str())); token.clear(); }
        } else {
            token.push_back(c);
        }
    }
    if (!token.empty()) ids.push_back(atoi(token.c_str()));
    return ids;
}

int fail(const char* what, VlrfB200Status st) {
    fprintf(stderr, "vlrf_b200_cli %s: %s (%s)\n", what, vlrf_b200_last_error(), vlrf_b200_status_str(st));
    return 1;
}

int cmd_info(const Args& a) {
    if (a.model.empty()) return usage("info needs --model");
    std::vector<char> text(1 << 16);
    VlrfB200Status st = vlrf_b200_describe_dir(a.model.c_str(), text.data(), (int32_t)text.size());
    if (st != VLRF_B200_OK) return fail("info", st);
    fputs(text.data(), stdout);
    return 0;
}

int cmd_init(const Args& a) {
    if (a.config.empty() || a.out.empty()) return usage("init needs --config and --out");
    VlrfB200Status st = vlrf_b200_write_random_model(a.config.c_str(), a.seed_given ? a.seed : a.init_seed, a.out.c_str());
    if (st != VLRF_B200_OK) return fail("init", st);
    printf("wrote %s/config.json and %s/model.safetensors (seed %u)\n", a.out.c_str(), a.out.c_str(), a.seed_given ? a.seed : a.init_seed);
    return 0;
}

int cmd_run(const Args& a) {
    if (a.model.empty()) return usage("run needs --model");
    std::vector<std::vector<int32_t>> prompts;
    bool from_text = false;
    if (!a.prompts_file.empty()) {
        std::ifstream f(a.prompts_file);
        if (!f.good()) { fprintf(stderr, "vlrf_b200_cli run: cannot read %s\n", a.prompts_file.c_str()); return 1; }
        std::string line;
        while (std::getline(f, line))
            if (line.find_first_not_of(" \t\r") != std::string::npos) prompts.push_back(parse_ids(line));
    } else if (!a.prompt_ids.empty()) {
        prompts.push_back(parse_ids(a.prompt_ids));
    } else if (a.has_prompt) {
        std::vector<int32_t> ids;
        for (unsigned char c : a.prompt) ids.push_back((int32_t)c + 4);
        prompts.push_back(ids);
        from_text = true;
    } else {
        return usage("run: give --prompt, --prompt-ids or --prompts-file");
    }
    int need = 0;
    for (auto& p : prompts) need += ((int)p.size() + a.tokens + 63) / 64 * 64;
    printf("Loading model from %s ...\n", a.model.c_str());
    VlrfB200Model model = vlrf_b200_create_model();
    if (model == nullptr) return fail("run", VLRF_B200_ERR_DEVICE);
    VlrfB200Status st = vlrf_b200_load_dir(model, a.model.c_str(), a.dtype.c_str(), a.ctx > 0 ? a.ctx : need, 0);
    if (st != VLRF_B200_OK) { int rc = fail("run", st); vlrf_b200_free_model(model); return rc; }
    std::vector<char> text(1 << 16);
    if (vlrf_b200_model_summary(model, text.data(), (int32_t)text.size()) == VLRF_B200_OK) printf("%s\n", text.data());
    VlrfB200ModelInfo info;
    st = vlrf_b200_get_info(model, &info);
    if (st != VLRF_B200_OK) { int rc = fail("run", st); vlrf_b200_free_model(model); return rc; }
    if (from_text)
        for (auto& t : prompts[0]) if (t >= info.vocab_size) t = info.vocab_size - 1;
    VlrfB200Sampling p;
    vlrf_b200_default_sampling(&p);
    p.max_new_tokens = a.tokens; p.temperature = a.temp; p.top_k = a.top_k; p.top_p = a.top_p; p.use_sampling = a.greedy ? 0 : 1;
    p.repetition_penalty = a.repeat_penalty; p.frequency_penalty = a.freq_penalty; p.presence_penalty = a.presence_penalty;
    p.no_repeat_ngram_size = a.no_repeat_ngram; p.seed = a.seed;
    if (!a.stop_ids.empty()) {
        if (a.stop_ids.size() > 8) { vlrf_b200_free_model(model); return usage("at most 8 --stop-id"); }
        p.n_stop_ids = (int32_t)a.stop_ids.size();
        for (size_t i = 0; i < a.stop_ids.size(); ++i) p.stop_ids[i] = a.stop_ids[i];
    }
    std::vector<int32_t> flat, lens, out((size_t)prompts.size() * (size_t)(a.tokens > 0 ? a.tokens : 1)), out_lens(prompts.size()),
        reasons(prompts.size());
    for (auto& q : prompts) { lens.push_back((int32_t)q.size()); flat.insert(flat.end(), q.begin(), q.end()); }
    auto t0 = std::chrono::steady_clock::now();
    st = vlrf_b200_generate_ids(model, flat.data(), lens.data(), (int32_t)prompts.size(), &p, 1, out.data(), a.tokens, out_lens.data(),
                                reasons.data());
    double dt = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
    if (st != VLRF_B200_OK) { int rc = fail("run", st); vlrf_b200_free_model(model); return rc; }
    const char* reason_text[3] = {"stop", "length", "context"};
    long total = 0, ctx = 0;
    for (size_t i = 0; i < prompts.size(); ++i) {
        printf("--- Prompt %zu ---\n", i);
        for (size_t j = 0; j < prompts[i].size(); ++j) printf("%s%d", j ? " " : "", prompts[i][j]);
        printf("\n--- Output (%s) ---\n", reason_text[reasons[i] >= 0 && reasons[i] < 3 ? reasons[i] : 1]);
        for (int j = 0; j < out_lens[i]; ++j) printf("%s%d", j ? " " : "", out[i * (size_t)a.tokens + j]);
        printf("\n");
        total += out_lens[i];
        ctx += (long)prompts[i].size() + out_lens[i];
    }
    printf("\n[%ld tokens in context, %ld generated, %.2f s, %.1f tok/s]\n", ctx, total, dt, total / (dt > 1e-9 ? dt : 1e-9));
    vlrf_b200_free_model(model);
    return 0;
}

}  // namespace

int main(int argc, char** argv) {
    if (argc < 2) return usage(nullptr);
    Args a;
    a.command = argv[1];
    for (int i = 2; i < argc; ++i) {
        std::string k = argv[i];
        auto value = [&](const char* name) -> const char* {
            if (i + 1 >= argc) { fprintf(stderr, "vlrf_b200_cli: %s needs a value\n", name); exit(2); }
            return argv[++i];
        };
        if (k == "--model") a.model = value("--model");
        else if (k == "--prompt") { a.prompt = value("--prompt"); a.has_prompt = true; }
        else if (k == "--prompt-ids") a.prompt_ids = value("--prompt-ids");
        else if (k == "--prompts-file") a.prompts_file = value("--prompts-file");
        else if (k == "--tokens") a.tokens = atoi(value("--tokens"));
        else if (k == "--ctx") a.ctx = atoi(value("--ctx"));
        else if (k == "--temp") a.temp = (float)atof(value("--temp"));
        else if (k == "--top-k") a.top_k = atoi(value("--top-k"));
        else if (k == "--top-p") a.top_p = (float)atof(value("--top-p"));
        else if (k == "--seed") { a.seed = (unsigned)strtoul(value("--seed"), nullptr, 10); a.seed_given = true; }
        else if (k == "--greedy") a.greedy = true;
        else if (k == "--repeat-penalty") a.repeat_penalty = (float)atof(value("--repeat-penalty"));
        else if (k == "--freq-penalty") a.freq_penalty = (float)atof(value("--freq-penalty"));
        else if (k == "--presence-penalty") a.presence_penalty = (float)atof(value("--presence-penalty"));
        else if (k == "--no-repeat-ngram") a.no_repeat_ngram = atoi(value("--no-repeat-ngram"));
        else if (k == "--stop-id") a.stop_ids.push_back(atoi(value("--stop-id")));
        else if (k == "--dtype") a.dtype = value("--dtype");
        else if (k == "--config") a.config = value("--config");
        else if (k == "--out") a.out = value("--out");
        else return usage(("unknown option " + k).c_str());
    }
    if (a.tokens < 0) return usage("--tokens must not be negative");
    if (a.command == "run") return cmd_run(a);
    if (a.command == "info") return cmd_info(a);
    if (a.command == "init") return cmd_init(a);
    return usage(("unknown command " + a.command).c_str());
}
