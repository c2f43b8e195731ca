// Runs the reference's own model code (tattooinmtl/Ultima.cpp, compiled unchanged) on a tiny
// Qwen3 model held in memory, and writes its logits.  The reference's file loader is for
// Windows only, so the model reaches it through its abstract LoadedModel interface, as its own
// configuration tests do (tests/unit/test_qwen_config.cpp:18-38).
//
// input file: int32 {layers, hidden, ffn, heads, kv_heads, head_dim, vocab, ctx, tied, n_tokens, window},
//             int32 pattern[layers] (1: the layer attends to the last ``window`` positions only; all 0
//             and window 0 for a model without a window), float32 {eps, theta}, int32 tokens[n_tokens],
//             then every tensor as float32 in the order of golden_weights.tensor_list.
// output file: float32 logits [n_tokens, vocab] from token-by-token decode, then float32
//              logits [vocab] of a whole-prompt prefill (its last position).
#include "ultima/kv_cache/kv_cache.hpp"
#include "ultima/model/imodel.hpp"
#include "ultima/model/loaded_model.hpp"
#include "ultima/runtime/thread_pool.hpp"

#include <cstdint>
#include <cstdio>
#include <map>
#include <span>
#include <string>
#include <vector>

using namespace ultima::model;

struct Mem : LoadedModel {
    std::string arch = "qwen3";
    MetadataStore md;
    std::vector<TensorInfo> infos;
    std::map<std::string, std::vector<float>, std::less<>> data;
    std::vector<std::uint8_t> blob;        // what stands in for the file: the per-layer window pattern

    void add(const std::string& name, std::vector<std::uint64_t> dims_inner_first, std::vector<float> v) {
        TensorInfo ti;
        ti.name = name; ti.dims = dims_inner_first; ti.dtype = DataType::F32; ti.offset = 0;
        ti.size_bytes = v.size() * 4;
        infos.push_back(ti);
        data[name] = std::move(v);
    }
    const std::string& architecture() const override { return arch; }
    const MetadataStore& metadata() const override { return md; }
    const std::vector<TensorInfo>& tensor_infos() const override { return infos; }
    std::optional<TensorView> tensor(std::string_view name) const override {
        for (const auto& ti : infos)
            if (ti.name == name) return TensorView{ti, data.find(name)->second.data()};
        return std::nullopt;
    }
    std::uint64_t file_size_bytes() const override { return blob.size(); }
    std::uint64_t alignment() const override { return 32; }
    std::uint32_t gguf_version() const override { return 3; }
    const std::uint8_t* file_data() const override { return blob.empty() ? nullptr : blob.data(); }
};

static std::vector<float> rd(FILE* f, std::size_t n) {
    std::vector<float> v(n);
    if (std::fread(v.data(), 4, n, f) != n) { std::fprintf(stderr, "short read\n"); std::exit(3); }
    return v;
}

int main(int argc, char** argv) {
    if (argc != 3) { std::fprintf(stderr, "usage: harness IN OUT\n"); return 2; }
    FILE* f = std::fopen(argv[1], "rb");
    if (!f) return 2;
    std::int32_t h[11];
    if (std::fread(h, 4, 11, f) != 11) return 3;
    const std::uint64_t L = h[0], H = h[1], F = h[2], nh = h[3], nkv = h[4], hd = h[5], V = h[6], ctx = h[7];
    const bool tied = h[8] != 0;
    const int n_tok = h[9];
    const std::uint64_t window = h[10];
    std::vector<std::int32_t> pattern(L);
    if (std::fread(pattern.data(), 4, L, f) != L) return 3;
    float fl[2];
    if (std::fread(fl, 4, 2, f) != 2) return 3;
    std::vector<std::int32_t> toks(n_tok);
    if (std::fread(toks.data(), 4, n_tok, f) != (std::size_t)n_tok) return 3;

    Mem m;
    m.md.insert("general.architecture", MetadataValue{std::string("qwen3")});
    m.md.insert("qwen3.context_length", MetadataValue{std::uint64_t{ctx}});
    m.md.insert("qwen3.embedding_length", MetadataValue{std::uint64_t{H}});
    m.md.insert("qwen3.block_count", MetadataValue{std::uint64_t{L}});
    m.md.insert("qwen3.feed_forward_length", MetadataValue{std::uint64_t{F}});
    m.md.insert("qwen3.attention.head_count", MetadataValue{std::uint64_t{nh}});
    m.md.insert("qwen3.attention.head_count_kv", MetadataValue{std::uint64_t{nkv}});
    m.md.insert("qwen3.attention.key_length", MetadataValue{std::uint64_t{hd}});
    m.md.insert("qwen3.attention.layer_norm_rms_epsilon", MetadataValue{fl[0]});
    m.md.insert("qwen3.rope.freq_base", MetadataValue{fl[1]});
    m.md.insert("tokenizer.ggml.tokens", MetadataValue{std::vector<std::string>(V, "x")});
    if (window > 0) {
        // the window engages only with both keys (src/model/qwen_config.cpp:229-253); the pattern is an
        // array that the reference reads from the file's bytes (src/model/loaded_model.cpp:50-61)
        for (auto v : pattern) m.blob.push_back(v ? 1 : 0);
        m.md.insert("qwen3.attention.sliding_window", MetadataValue{std::uint64_t{window}});
        m.md.insert("qwen3.attention.sliding_window_pattern", MetadataValue{MetadataArrayView{0, L, 0}});
    }

    m.add("token_embd.weight", {H, V}, rd(f, V * H));
    for (std::uint64_t i = 0; i < L; ++i) {
        const std::string p = "blk." + std::to_string(i) + ".";
        m.add(p + "attn_norm.weight", {H}, rd(f, H));
        m.add(p + "attn_q.weight", {H, nh * hd}, rd(f, nh * hd * H));
        m.add(p + "attn_k.weight", {H, nkv * hd}, rd(f, nkv * hd * H));
        m.add(p + "attn_v.weight", {H, nkv * hd}, rd(f, nkv * hd * H));
        m.add(p + "attn_q_norm.weight", {hd}, rd(f, hd));
        m.add(p + "attn_k_norm.weight", {hd}, rd(f, hd));
        m.add(p + "attn_output.weight", {nh * hd, H}, rd(f, H * nh * hd));
        m.add(p + "ffn_norm.weight", {H}, rd(f, H));
        m.add(p + "ffn_gate.weight", {H, F}, rd(f, F * H));
        m.add(p + "ffn_up.weight", {H, F}, rd(f, F * H));
        m.add(p + "ffn_down.weight", {F, H}, rd(f, H * F));
    }
    m.add("output_norm.weight", {H}, rd(f, H));
    if (!tied) m.add("output.weight", {H, V}, rd(f, V * H));
    std::fclose(f);

    ultima::runtime::ThreadPool pool{2};
    auto mr = load_model(m, pool);
    if (!mr) { std::fprintf(stderr, "load_model failed: %s\n", mr.error().message.c_str()); return 4; }
    auto& model = **mr;
    const auto& d = model.dims();
    std::fprintf(stderr, "arch=qwen3 layers=%zu hidden=%zu heads=%zu/%zu head_dim=%zu q_dim=%zu vocab=%zu eps=%g\n",
                 d.n_layers, d.hidden, d.n_heads, d.n_kv_heads, d.head_dim, d.q_dim, d.vocab, (double)d.rms_eps);
    ultima::kv_cache::KVCache::Config kc;
    kc.n_slots = 2; kc.n_ctx = ctx; kc.n_layers = d.n_layers; kc.n_kv_heads = d.n_kv_heads;
    kc.head_dim = d.head_dim; kc.dtype = DataType::F32;
    ultima::kv_cache::KVCache kv{kc};

    FILE* o = std::fopen(argv[2], "wb");
    if (!o) return 2;
    std::vector<float> logits(V);
    auto s1 = kv.acquire(1);
    for (int t = 0; t < n_tok; ++t) {
        auto r = model.decode(kv, s1, toks[t], logits.data());
        if (!r) { std::fprintf(stderr, "decode failed\n"); return 5; }
        std::fwrite(logits.data(), 4, V, o);
    }
    auto s2 = kv.acquire(2);
    auto r = model.prefill(kv, s2, std::span<const std::int32_t>(toks), logits.data());
    if (!r) { std::fprintf(stderr, "prefill failed\n"); return 5; }
    std::fwrite(logits.data(), 4, V, o);
    std::fclose(o);
    return 0;
}
