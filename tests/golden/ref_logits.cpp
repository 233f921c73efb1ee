// Test-only driver: runs VLRF-org/VLRF's own CPU model code (headers under include/) on weights that
// make_golden.py wrote, and prints last-position logits for given prefixes of a token sequence.
// It is compiled by make_golden.py against the reference's include folders and is not part of the
// library.  Input file: int32 count; per tensor: int32 name length, name, int32 ndim, int32 dims[],
// float32 data.
#include "transformer.hpp"
#include <cstdio>
#include <cstdlib>
#include <fstream>
#include <iostream>
#include <string>
#include <vector>

using namespace vlrf;

static int32_t read_i32(std::ifstream& f) { int32_t v; f.read((char*)&v, 4); return v; }

int main(int argc, char** argv) {
    // argv: weights.bin vocab d_model d_ff n_heads n_layers max_seq eps per_layer_scale(0/1) out.bin n_ids ids... n_prefix prefix_lens...
    if (argc < 12) { std::cerr << "usage\n"; return 2; }
    int a = 1;
    std::string wpath = argv[a++];
    ModelConfig cfg;
    cfg.vocab_size = atoi(argv[a++]);
    cfg.d_model = atoi(argv[a++]);
    cfg.d_ff = atoi(argv[a++]);
    cfg.n_heads = atoi(argv[a++]);
    cfg.n_kv_heads = cfg.n_heads;
    cfg.n_layers = atoi(argv[a++]);
    cfg.max_seq_len = atoi(argv[a++]);
    cfg.layer_norm_eps = (float)atof(argv[a++]);
    int per_layer_scale = atoi(argv[a++]);
    std::string opath = argv[a++];
    cfg.pos_embedding = PosEmbedding::LEARNED;
    cfg.activation = Activation::GELU;
    cfg.pre_norm = true;
    cfg.tie_embeddings = true;
    int n_ids = atoi(argv[a++]);
    std::vector<int> ids(n_ids);
    for (int i = 0; i < n_ids; ++i) ids[i] = atoi(argv[a++]);
    int n_prefix = atoi(argv[a++]);
    std::vector<int> prefixes(n_prefix);
    for (int i = 0; i < n_prefix; ++i) prefixes[i] = atoi(argv[a++]);

    TransformerModel m;
    m.init(cfg);
    std::ifstream f(wpath, std::ios::binary);
    int32_t count = read_i32(f);
    for (int t = 0; t < count; ++t) {
        int32_t nl = read_i32(f);
        std::string name(nl, ' ');
        f.read(&name[0], nl);
        int32_t nd = read_i32(f);
        std::vector<int32_t> dims(nd);
        for (auto& d : dims) d = read_i32(f);
        Shape s;
        if (nd == 1) s = Shape({dims[0]});
        else s = Shape({dims[0], dims[1]});
        Tensor tt(s);
        f.read((char*)tt.data_ptr(), (std::streamsize)tt.numel() * 4);
        m.wm.tensors[name] = std::move(tt);
    }
    m.bind_weights();
    if (per_layer_scale) {
        // 1/sqrt(d_head)/(layer+1): the reference has no such option; its public per-layer
        // attention_multiplier replaces the scale (include/model/attention.hpp:53,373-374)
        for (int l = 0; l < cfg.n_layers; ++l)
            m.layers[l].attn.attention_multiplier = 1.f / std::sqrt((float)cfg.d_head()) / (float)(l + 1);
    }
    std::ofstream o(opath, std::ios::binary);
    for (int p : prefixes) {
        std::vector<int> pre(ids.begin(), ids.begin() + p);
        m.reset_kv_cache();
        Tensor lg = m.forward(pre, /*use_cache=*/false);
        o.write((char const*)lg.data_ptr(), (std::streamsize)cfg.vocab_size * 4);
    }
    // incremental: prefix of half, then one token at a time with the cache; last logits
    {
        m.reset_kv_cache();
        int half = n_ids / 2;
        std::vector<int> pre(ids.begin(), ids.begin() + half);
        Tensor lg = m.forward(pre, true);
        for (int i = half; i < n_ids; ++i) lg = m.forward({ids[i]}, true);
        o.write((char const*)lg.data_ptr(), (std::streamsize)cfg.vocab_size * 4);
    }
    return 0;
}
