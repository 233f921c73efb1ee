// A C++ program over vlrf_b200.h alone, driven by tests/test_capi.py: loads a model folder, generates greedily for a
// batch of unequal prompts, reads logits, and runs single steps.  It prints what it got, one item a line:
//   sizes <sizeof(VlrfB200Sampling)> <sizeof(VlrfB200ModelInfo)>
//   info <vocab> <max_seq_len> <width> <layers> <cache_tokens> <cache_slots> <bos> <eos>
//   gen <i> <reason> <ids…>                   new tokens of prompt i
//   logits <checksum> <argmax>                of get_logits on the first prompt
//   step <max abs difference>                 prompt-then-one-token steps against get_logits on the same tokens
//   status <name> <code>                      what refused calls return
// usage: capi_program MODEL_DIR DTYPE N_SLOTS MAX_NEW  len,len,…  SEED
#include "vlrf_b200.h"

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

static int die(const char* what, VlrfB200Status st) {
    fprintf(stderr, "%s: %s (%s)\n", what, vlrf_b200_last_error(), vlrf_b200_status_str(st));
    return 1;
}

int main(int argc, char** argv) {
    if (argc < 7) return 2;
    const char* dir = argv[1];
    const char* dtype = argv[2];
    const int n_slots = atoi(argv[3]), max_new = atoi(argv[4]);
    std::vector<int> lens;
    for (char* tok = strtok(argv[5], ","); tok; tok = strtok(nullptr, ",")) lens.push_back(atoi(tok));
    unsigned seed = (unsigned)atoi(argv[6]);
    printf("sizes %zu %zu\n", sizeof(VlrfB200Sampling), sizeof(VlrfB200ModelInfo));

    VlrfB200Model m = vlrf_b200_create_model();
    if (!m) return die("create", VLRF_B200_ERR_DEVICE);
    VlrfB200ModelInfo info;
    printf("status info_before_load %d\n", (int)vlrf_b200_get_info(m, &info));
    printf("status load_missing %d\n", (int)vlrf_b200_load_dir(m, "/nonexistent/model", dtype, 0, 0));
    VlrfB200Status st = vlrf_b200_load_dir(m, dir, dtype, 64 * 8, n_slots);
    if (st != VLRF_B200_OK) return die("load_dir", st);
    st = vlrf_b200_get_info(m, &info);
    if (st != VLRF_B200_OK) return die("get_info", st);
    printf("info %d %d %d %d %d %d %d %d\n", info.vocab_size, info.max_seq_len, info.width, info.n_layers, info.cache_tokens,
           info.cache_slots, info.bos_token_id, info.eos_token_id);

    // the prompts: a fixed pseudo-random stream of ids, the same as the test draws
    std::vector<int32_t> flat, plens;
    unsigned long long x = seed;
    for (int n : lens) {
        plens.push_back(n);
        for (int i = 0; i < n; ++i) {
            x = x * 6364136223846793005ULL + 1442695040888963407ULL;
            flat.push_back((int32_t)((x >> 33) % (unsigned)info.vocab_size));
        }
    }
    VlrfB200Sampling p;
    vlrf_b200_default_sampling(&p);
    p.max_new_tokens = max_new; p.use_sampling = 0; p.n_stop_ids = 0;
    std::vector<int32_t> out(lens.size() * (size_t)max_new), out_lens(lens.size()), reasons(lens.size());
    st = vlrf_b200_generate_ids(m, flat.data(), plens.data(), (int32_t)lens.size(), &p, 1, out.data(), max_new, out_lens.data(), reasons.data());
    if (st != VLRF_B200_OK) return die("generate_ids", st);
    for (size_t i = 0; i < lens.size(); ++i) {
        printf("gen %zu %d", i, reasons[i]);
        for (int j = 0; j < out_lens[i]; ++j) printf(" %d", out[i * max_new + j]);
        printf("\n");
    }
    // logits of the first prompt, and the same through single steps: the prompt without its last token, then that token
    std::vector<float> logits(info.vocab_size), stepped(2 * (size_t)info.vocab_size);
    st = vlrf_b200_get_logits(m, flat.data(), plens[0], logits.data());
    if (st != VLRF_B200_OK) return die("get_logits", st);
    double sum = 0; int best = 0;
    for (int v = 0; v < info.vocab_size; ++v) { sum += logits[v]; if (logits[v] > logits[best]) best = v; }
    printf("logits %.6f %d\n", sum, best);
    if (plens[0] >= 2) {
        int32_t slot = -1;
        st = vlrf_b200_start_sequence(m, &slot);
        if (st != VLRF_B200_OK) return die("start_sequence", st);
        int32_t count = plens[0] - 1, want_count = 0;
        st = vlrf_b200_step(m, 1, &slot, &count, flat.data(), &want_count, nullptr, stepped.data(), 2);
        if (st != VLRF_B200_OK) return die("step (prompt)", st);
        if (vlrf_b200_context_length(m, slot) != plens[0] - 1) return die("context_length", VLRF_B200_ERR_UNKNOWN);
        count = 1; want_count = 1;
        int32_t want = 0;
        st = vlrf_b200_step(m, 1, &slot, &count, flat.data() + plens[0] - 1, &want_count, &want, stepped.data(), 2);
        if (st != VLRF_B200_OK) return die("step (token)", st);
        double worst = 0;
        for (int v = 0; v < info.vocab_size; ++v) worst = fmax(worst, fabs((double)stepped[v] - logits[v]));
        printf("step %.3e\n", worst);
        int32_t bad = info.vocab_size + 5;
        printf("status step_bad_token %d\n", (int)vlrf_b200_step(m, 1, &slot, &count, &bad, &want_count, &want, stepped.data(), 2));
        st = vlrf_b200_reset_slot(m, slot);
        if (st != VLRF_B200_OK) return die("reset_slot", st);
        printf("status step_freed_slot %d\n", (int)vlrf_b200_step(m, 1, &slot, &count, flat.data(), &want_count, &want, stepped.data(), 2));
    }
    printf("status too_long %d\n", (int)vlrf_b200_get_logits(m, std::vector<int32_t>(info.max_seq_len + 1, 1).data(), info.max_seq_len + 1, logits.data()));
    printf("cache_bytes %lld\n", (long long)vlrf_b200_kv_cache_bytes(m));
    vlrf_b200_free_model(m);
    return 0;
}
